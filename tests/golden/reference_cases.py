"""Known-answer vectors for the tensor hot path, transcribed from the reference's own tests.

Every case cites the test it was read from (paths relative to libs/rtensors/src/ of
aheschl1/rtensors).  The reference is Rust and cannot be built or imported where these tests run,
so the vectors were transcribed by reading its test sources as text; nothing here was computed
by this repository's code.  They pin the CPU oracle (tests/test_oracle_golden.py) and are
replayed against the CUDA library (tests/test_gpu_golden.py).

Tensor spec:  {"buf": [...], "shape": [...]}  or  {"ones": shape} / {"zeros": shape},
optional "set": [(coord, value), ...] applied to the fresh tensor, optional "view": list of
  ("slice", dim, start, end, step)   -- Slice{start,end,step}; None = unbounded
  ("index", dim, i)                  -- `slice(dim, i..i)`: removes the dim
  ("permute", dims)
Expectations: "values" (row-major list), "all" (every element equals it), "spots" [(coord, v)],
"shape".
"""

S = "slice"
I = "index"

CASES = [
    # ---------------------------------------------------------------- scalar ops, in place
    dict(name="add_after_slice", cite="ops/mod.rs:127-142", kind="scalar_assign", dtype="i32",
         a=dict(buf=[1, 2, 3, 4, 5, 6], shape=[2, 3], view=[(I, 0, 1)]), ops=[("add", 100)],
         buf=[1, 2, 3, 104, 105, 106]),
    dict(name="mul_after_slice", cite="ops/mod.rs:170-185", kind="scalar_assign", dtype="i32",
         a=dict(buf=[1, 2, 3, 4, 5, 6, 7, 8], shape=[2, 2, 2], view=[(I, 0, 0)]), ops=[("mul", 10)],
         buf=[10, 20, 30, 40, 5, 6, 7, 8]),
    dict(name="mul_after_column_slice", cite="ops/mod.rs:200-215", kind="scalar_assign", dtype="i32",
         a=dict(buf=[1, 2, 3, 4, 5, 6], shape=[2, 3], view=[(I, 1, 1)]), ops=[("mul", 3)],
         buf=[1, 6, 3, 4, 15, 6]),
    dict(name="add_ref_after_slice_chain", cite="ops/mod.rs:230-252", kind="scalar_assign", dtype="i32",
         a=dict(buf=[1, 2, 3, 4, 5, 6, 7, 8], shape=[2, 2, 2], view=[(I, 0, 1), (I, 0, 0)]),
         ops=[("add", 1000)], buf=[1, 2, 3, 4, 1005, 1006, 7, 8]),
    dict(name="non_square_slice_operations", cite="ops/mod.rs:741-756", kind="scalar_assign", dtype="i32",
         a=dict(buf=list(range(1, 13)), shape=[3, 4], view=[(I, 0, 1)]), ops=[("mul", 10)],
         buf=[1, 2, 3, 4, 50, 60, 70, 80, 9, 10, 11, 12]),
    dict(name="large_values", cite="ops/mod.rs:793-805", kind="scalar_assign", dtype="i32",
         a=dict(buf=[1_000_000, 2_000_000, 3_000_000], shape=[3]), ops=[("add", 500_000)],
         buf=[1_500_000, 2_500_000, 3_500_000]),
    dict(name="f32_operations", cite="ops/mod.rs:810-823", kind="scalar_assign", dtype="f32",
         a=dict(buf=[1.5, 2.5, 3.5, 4.5], shape=[4]), ops=[("mul", 2.0), ("add", 1.0)],
         buf=[4.0, 6.0, 8.0, 10.0]),
    dict(name="f64_operations", cite="ops/mod.rs:826-839", kind="scalar_assign", dtype="f64",
         a=dict(buf=[1.0, 2.0, 3.0, 4.0], shape=[4]), ops=[("add", 0.5), ("mul", 2.0)],
         buf=[3.0, 5.0, 7.0, 9.0]),
    dict(name="i64_operations", cite="ops/mod.rs:842-852", kind="scalar_assign", dtype="i64",
         a=dict(buf=[100, 200, 300, 400], shape=[4]), ops=[("sub", 50), ("mul", 3)],
         buf=[150, 450, 750, 1050]),
    dict(name="u32_operations", cite="ops/mod.rs:855-865", kind="scalar_assign", dtype="u32",
         a=dict(buf=[10, 20, 30, 40], shape=[4]), ops=[("add", 5), ("mul", 2)], buf=[30, 50, 70, 90]),
    dict(name="i16_operations", cite="ops/mod.rs:868-878", kind="scalar_assign", dtype="i16",
         a=dict(buf=[1, 2, 3, 4, 5, 6], shape=[2, 3]), ops=[("mul", 10), ("add", 5)],
         buf=[15, 25, 35, 45, 55, 65]),
    dict(name="multiple_noncontiguous_operations", cite="ops/mod.rs:883-900", kind="scalar_assign", dtype="i32",
         a=dict(buf=list(range(1, 13)), shape=[4, 3], view=[(I, 1, 1)]), ops=[("add", 100), ("mul", 2)],
         buf=[1, 204, 3, 4, 210, 6, 7, 216, 9, 10, 222, 12]),
    dict(name="3d_noncontiguous_slice", cite="ops/mod.rs:922-951", kind="scalar_assign", dtype="i32",
         a=dict(buf=list(range(1, 25)), shape=[2, 3, 4], view=[(I, 1, 1)]), ops=[("add", 100)],
         expect_meta=dict(shape=[2, 4], strides=[12, 1], offset=4, contiguous=False),
         buf=[v + 100 if v in (5, 6, 7, 8, 17, 18, 19, 20) else v for v in range(1, 25)]),
    dict(name="4d_tensor_operations", cite="ops/mod.rs:978-986", kind="scalar_assign", dtype="i32",
         a=dict(buf=list(range(1, 17)), shape=[2, 2, 2, 2]), ops=[("add", 10)], buf=list(range(11, 27))),
    dict(name="4d_slice_operation", cite="ops/mod.rs:989-1003", kind="scalar_assign", dtype="i32",
         a=dict(buf=list(range(1, 25)), shape=[2, 3, 2, 2], view=[(I, 0, 1)]), ops=[("mul", 10)],
         buf=[v * 10 if v > 12 else v for v in range(1, 25)]),
    dict(name="5d_tensor_operations", cite="ops/mod.rs:1006-1016", kind="scalar_assign", dtype="i32",
         a=dict(buf=list(range(1, 33)), shape=[2, 2, 2, 2, 2]), ops=[("mul", 2), ("add", 5)],
         buf=[v * 2 + 5 for v in range(1, 33)]),
    # ---------------------------------------------------------------- scalar ops, out of place
    dict(name="add_not_inplace_with_slice", cite="ops/mod.rs:324-337", kind="scalar", dtype="i32",
         a=dict(buf=[1, 2, 3, 4, 5, 6], shape=[2, 3], view=[(I, 0, 1)]), op="add", value=100,
         shape=[3], values=[104, 105, 106]),
    dict(name="mul_not_inplace_with_noncontiguous_slice", cite="ops/mod.rs:340-357", kind="scalar", dtype="i32",
         a=dict(buf=[1, 2, 3, 4, 5, 6], shape=[2, 3], view=[(I, 1, 1)]), op="mul", value=3,
         shape=[2], values=[6, 15]),
    dict(name="add_not_inplace_chained_slices", cite="ops/mod.rs:395-410", kind="scalar", dtype="i32",
         a=dict(buf=[1, 2, 3, 4, 5, 6, 7, 8], shape=[2, 2, 2], view=[(I, 0, 1), (I, 0, 0)]), op="add",
         value=1000, shape=[2], values=[1005, 1006]),
    dict(name="broadcast_with_negative_step_2_slice", cite="ops/mod.rs:2529-2547", kind="scalar", dtype="f32",
         a=dict(buf=[1, 2, 3, 4, 5, 6, 7, 8], shape=[8], view=[(S, 0, None, None, -2)]), op="add", value=100.0,
         shape=[4], values=[108.0, 106.0, 104.0, 102.0]),
    dict(name="broadcast_scalar_with_complex_negative_slice", cite="ops/mod.rs:2638-2656", kind="scalar",
         dtype="i32", a=dict(buf=list(range(1, 11)), shape=[10], view=[(S, 0, 8, 2, -2)]), op="add", value=100,
         shape=[3], values=[109, 107, 105]),
    # ---------------------------------------------------------------- broadcast binary ops
    dict(name="broadcast_flipped", cite="ops/mod.rs:1154-1171", kind="binary", dtype="f32", op="add",
         a=dict(ones=[1, 3], set=[((0, 0), 22.0)]), b=dict(ones=[3, 1]), shape=[3, 3],
         values=[23.0, 2.0, 2.0] * 3),
    dict(name="broadcast_same", cite="ops/mod.rs:1174-1191", kind="binary", dtype="f32", op="add",
         a=dict(ones=[3, 1], set=[((0, 0), 22.0)]), b=dict(ones=[3, 1]), shape=[3, 1], values=[23.0, 2.0, 2.0]),
    dict(name="broadcast_3d_scalar_to_tensor", cite="ops/mod.rs:1200-1214", kind="binary", dtype="f32", op="add",
         a=dict(buf=[5.0], shape=[]), b=dict(ones=[2, 3, 4]), shape=[2, 3, 4], all=6.0),
    dict(name="broadcast_3d_vector_along_last_dim", cite="ops/mod.rs:1217-1232", kind="binary", dtype="f32",
         op="add", a=dict(buf=[1.0, 2.0, 3.0], shape=[3]), b=dict(ones=[2, 4, 3]), shape=[2, 4, 3],
         values=[2.0, 3.0, 4.0] * 8),
    dict(name="broadcast_3d_matrix_to_tensor", cite="ops/mod.rs:1235-1249", kind="binary", dtype="f32", op="add",
         a=dict(ones=[3, 4]), b=dict(ones=[2, 3, 4]), shape=[2, 3, 4], all=2.0),
    dict(name="broadcast_3d_singleton_dims", cite="ops/mod.rs:1252-1266", kind="binary", dtype="f32", op="add",
         a=dict(ones=[1, 3, 1]), b=dict(ones=[2, 3, 4]), shape=[2, 3, 4], all=2.0),
    dict(name="broadcast_3d_prepend_dims", cite="ops/mod.rs:1269-1283", kind="binary", dtype="f32", op="add",
         a=dict(ones=[3, 4]), b=dict(ones=[5, 3, 4]), shape=[5, 3, 4], all=2.0),
    dict(name="broadcast_4d_vector_to_tensor", cite="ops/mod.rs:1288-1304", kind="binary", dtype="f32", op="add",
         a=dict(buf=[10.0, 20.0], shape=[2]), b=dict(ones=[3, 4, 5, 2]), shape=[3, 4, 5, 2],
         values=[11.0, 21.0] * 60),
    dict(name="broadcast_4d_complex_singletons", cite="ops/mod.rs:1307-1323", kind="binary", dtype="f32",
         op="add", a=dict(ones=[1, 1, 5, 1]), b=dict(ones=[2, 3, 5, 4]), shape=[2, 3, 5, 4], all=2.0),
    dict(name="broadcast_4d_3d_to_4d", cite="ops/mod.rs:1326-1342", kind="binary", dtype="f32", op="add",
         a=dict(ones=[3, 5, 4]), b=dict(ones=[2, 3, 5, 4]), shape=[2, 3, 5, 4], all=2.0),
    dict(name="broadcast_5d_scalar_to_tensor", cite="ops/mod.rs:1347-1365", kind="binary", dtype="f32", op="add",
         a=dict(buf=[100.0], shape=[]), b=dict(ones=[2, 2, 2, 2, 2]), shape=[2, 2, 2, 2, 2], all=101.0),
    dict(name="broadcast_5d_multiple_singletons", cite="ops/mod.rs:1368-1379", kind="binary", dtype="f32",
         op="add", a=dict(ones=[1, 2, 1, 3, 1]), b=dict(ones=[4, 2, 5, 3, 6]), shape=[4, 2, 5, 3, 6],
         spots=[((0, 0, 0, 0, 0), 2.0), ((3, 1, 4, 2, 5), 2.0)]),
    dict(name="broadcast_2d_to_4d", cite="ops/mod.rs:1383-1399", kind="binary", dtype="f32", op="add",
         a=dict(ones=[3, 4]), b=dict(ones=[2, 5, 3, 4]), shape=[2, 5, 3, 4], all=2.0),
    dict(name="broadcast_1d_to_5d", cite="ops/mod.rs:1402-1422", kind="binary", dtype="f32", op="add",
         a=dict(buf=[1.0, 2.0, 3.0], shape=[3]), b=dict(ones=[2, 4, 5, 6, 3]), shape=[2, 4, 5, 6, 3],
         values=[2.0, 3.0, 4.0] * 240),
    dict(name="broadcast_div_scalar_to_tensor", cite="ops/mod.rs:1428-1440", kind="binary", dtype="f32", op="div",
         a=dict(buf=[10.0], shape=[]), b=dict(buf=[2.0] * 6, shape=[2, 3]), shape=[2, 3], all=5.0),
    dict(name="broadcast_div_3d_vector_along_last_dim", cite="ops/mod.rs:1443-1458", kind="binary", dtype="f32",
         op="div", a=dict(ones=[2, 3, 4]), b=dict(buf=[1.0, 2.0, 4.0, 8.0], shape=[4]), shape=[2, 3, 4],
         values=[1.0, 0.5, 0.25, 0.125] * 6),
    dict(name="broadcast_div_2d_matrices", cite="ops/mod.rs:1474-1487", kind="binary", dtype="f32", op="div",
         a=dict(buf=[100.0, 200.0, 300.0, 400.0], shape=[2, 2]), b=dict(buf=[10.0, 20.0], shape=[1, 2]),
         shape=[2, 2], values=[10.0, 10.0, 30.0, 20.0]),
    dict(name="broadcast_both_singletons_2d_pattern1", cite="ops/mod.rs:1710-1727", kind="binary", dtype="f32",
         op="add", a=dict(ones=[1, 4], set=[((0, 0), 5.0), ((0, 1), 6.0)]), b=dict(ones=[3, 1]), shape=[3, 4],
         values=[6.0, 7.0, 2.0, 2.0] * 3),
    dict(name="broadcast_both_singletons_2d_pattern2", cite="ops/mod.rs:1730-1747", kind="binary", dtype="f32",
         op="add", a=dict(ones=[4, 1], set=[((0, 0), 10.0), ((1, 0), 20.0)]), b=dict(ones=[1, 5]), shape=[4, 5],
         values=[11.0] * 5 + [21.0] * 5 + [2.0] * 10),
    dict(name="broadcast_both_singletons_3d_complementary", cite="ops/mod.rs:1750-1765", kind="binary",
         dtype="f32", op="add", a=dict(ones=[1, 3, 1]), b=dict(ones=[2, 1, 4]), shape=[2, 3, 4], all=2.0),
    dict(name="broadcast_both_singletons_3d_alternating", cite="ops/mod.rs:1768-1787", kind="binary",
         dtype="f32", op="add", a=dict(ones=[1, 4, 5], set=[((0, 0, 0), 100.0)]),
         b=dict(ones=[3, 1, 5], set=[((0, 0, 0), 200.0)]), shape=[3, 4, 5],
         spots=[((0, 0, 0), 300.0), ((1, 0, 0), 101.0), ((2, 0, 0), 101.0), ((0, 1, 0), 201.0),
                ((0, 2, 0), 201.0)]),
    dict(name="broadcast_both_singletons_3d_partial_overlap", cite="ops/mod.rs:1790-1806", kind="binary",
         dtype="f32", op="add", a=dict(ones=[5, 1, 3]), b=dict(ones=[1, 4, 3]), shape=[5, 4, 3], all=2.0),
    dict(name="broadcast_both_singletons_4d_zigzag", cite="ops/mod.rs:1809-1820", kind="binary", dtype="f32",
         op="add", a=dict(ones=[1, 3, 1, 5]), b=dict(ones=[2, 1, 4, 1]), shape=[2, 3, 4, 5], all=2.0),
    dict(name="broadcast_both_singletons_4d_complex", cite="ops/mod.rs:1823-1834", kind="binary", dtype="f32",
         op="add", a=dict(ones=[1, 1, 6, 7]), b=dict(ones=[5, 4, 1, 1]), shape=[5, 4, 6, 7], all=2.0),
    dict(name="broadcast_both_singletons_5d_checkerboard", cite="ops/mod.rs:1837-1848", kind="binary",
         dtype="f32", op="add", a=dict(ones=[1, 2, 1, 3, 1]), b=dict(ones=[4, 1, 5, 1, 6]),
         shape=[4, 2, 5, 3, 6], all=2.0),
    dict(name="broadcast_both_singletons_5d_all_different", cite="ops/mod.rs:1851-1863", kind="binary",
         dtype="f32", op="add", a=dict(ones=[1, 3, 1, 1, 7]), b=dict(ones=[2, 1, 4, 5, 1]),
         shape=[2, 3, 4, 5, 7], all=2.0),
    dict(name="broadcast_both_singletons_mixed_ranks", cite="ops/mod.rs:1866-1881", kind="binary", dtype="f32",
         op="add", a=dict(ones=[1, 5]), b=dict(ones=[3, 1, 1]), shape=[3, 1, 5], all=2.0),
    dict(name="sub_broadcast_basic", cite="ops/mod.rs:1951-1965", kind="binary", dtype="f32", op="sub",
         a=dict(ones=[3, 3], set=[((0, 0), 5.0)]), b=dict(ones=[3, 1]), shape=[3, 3],
         values=[4.0, 0.0, 0.0] + [0.0] * 6),
    dict(name="sub_3d_broadcast", cite="ops/mod.rs:1968-1982", kind="binary", dtype="f32", op="sub",
         a=dict(buf=[10.0, 20.0, 30.0], shape=[3]), b=dict(ones=[2, 4, 3]), shape=[2, 4, 3],
         values=[9.0, 19.0, 29.0] * 8),
    dict(name="mul_broadcast_basic", cite="ops/mod.rs:2006-2018", kind="binary", dtype="f32", op="mul",
         a=dict(ones=[3, 3], set=[((0, 0), 5.0)]), b=dict(ones=[3, 1], set=[((1, 0), 2.0)]), shape=[3, 3],
         values=[5.0, 1.0, 1.0, 2.0, 2.0, 2.0, 1.0, 1.0, 1.0]),
    dict(name="mul_3d_broadcast", cite="ops/mod.rs:2021-2035", kind="binary", dtype="f32", op="mul",
         a=dict(buf=[2.0, 3.0, 4.0], shape=[3]), b=dict(ones=[2, 4, 3]), shape=[2, 4, 3],
         values=[2.0, 3.0, 4.0] * 8),
    dict(name="mul_scalar_broadcast", cite="ops/mod.rs:2038-2049", kind="binary", dtype="f32", op="mul",
         a=dict(buf=[5.0], shape=[]), b=dict(buf=[1.0, 2.0, 3.0, 4.0], shape=[2, 2]), shape=[2, 2],
         values=[5.0, 10.0, 15.0, 20.0]),
    # ---------------------------------------------------------------- broadcast on strided / reversed views
    dict(name="broadcast_post_slice", cite="ops/mod.rs:2435-2452", kind="binary", dtype="f32", op="add",
         a=dict(ones=[4, 3], view=[(S, 0, 0, 3, 2)]), b=dict(ones=[2, 1], set=[((0, 0), 2.0)]), shape=[2, 3],
         values=[3.0, 3.0, 3.0, 2.0, 2.0, 2.0]),
    dict(name="broadcast_with_negative_step_slice", cite="ops/mod.rs:2455-2479", kind="binary", dtype="f32",
         op="add", a=dict(buf=list(range(1, 13)), shape=[4, 3], view=[(S, 0, None, None, -1)]),
         b=dict(buf=[10.0, 20.0, 30.0], shape=[3]), shape=[4, 3],
         values=[20.0, 31.0, 42.0, 17.0, 28.0, 39.0, 14.0, 25.0, 36.0, 11.0, 22.0, 33.0]),
    dict(name="broadcast_with_column_slice_negative_step", cite="ops/mod.rs:2482-2504", kind="binary",
         dtype="f32", op="add", a=dict(buf=[1, 2, 3, 4, 5, 6], shape=[2, 3], view=[(S, 1, None, None, -1)]),
         b=dict(buf=[100.0, 200.0], shape=[2, 1]), shape=[2, 3],
         values=[103.0, 102.0, 101.0, 206.0, 205.0, 204.0]),
    dict(name="broadcast_with_step_2_slice", cite="ops/mod.rs:2507-2526", kind="binary", dtype="f32", op="add",
         a=dict(buf=[1, 2, 3, 4, 5, 6, 7, 8], shape=[8], view=[(S, 0, None, None, 2)]),
         b=dict(buf=[10.0], shape=[]), shape=[4], values=[11.0, 13.0, 15.0, 17.0]),
    dict(name="broadcast_with_3d_negative_step", cite="ops/mod.rs:2550-2577", kind="binary", dtype="f32",
         op="add", a=dict(buf=list(range(1, 13)), shape=[3, 2, 2], view=[(S, 0, None, None, -1)]),
         b=dict(buf=[10.0, 20.0, 30.0, 40.0], shape=[2, 2]), shape=[3, 2, 2],
         values=[19.0, 30.0, 41.0, 52.0, 15.0, 26.0, 37.0, 48.0, 11.0, 22.0, 33.0, 44.0]),
    dict(name="broadcast_chained_slices_with_negative_steps", cite="ops/mod.rs:2604-2635", kind="binary",
         dtype="f32", op="add",
         a=dict(buf=list(range(1, 17)), shape=[4, 4], view=[(S, 0, None, None, -1), (S, 1, None, None, 2)]),
         b=dict(buf=[100.0, 200.0], shape=[1, 2]), shape=[4, 2],
         values=[113.0, 215.0, 109.0, 211.0, 105.0, 207.0, 101.0, 203.0]),
    dict(name="broadcast_vector_to_negative_step_matrix_slice", cite="ops/mod.rs:2659-2681", kind="binary",
         dtype="f32", op="add", a=dict(buf=list(range(1, 13)), shape=[4, 3], view=[(S, 0, 3, None, -2)]),
         b=dict(buf=[5.0, 10.0], shape=[2, 1]), shape=[2, 3], values=[15.0, 16.0, 17.0, 14.0, 15.0, 16.0]),
    dict(name="broadcast_both_tensors_sliced_negative_steps", cite="ops/mod.rs:2684-2710", kind="binary",
         dtype="f32", op="add", a=dict(buf=[1, 2, 3, 4, 5, 6], shape=[2, 3], view=[(S, 1, None, None, -1)]),
         b=dict(buf=[10.0, 20.0, 30.0], shape=[1, 3], view=[(S, 1, None, None, -1)]), shape=[2, 3],
         values=[33.0, 22.0, 11.0, 36.0, 25.0, 14.0]),
    dict(name="broadcast_4d_with_negative_step_multiple_dims", cite="ops/mod.rs:2713-2737", kind="binary",
         dtype="f32", op="add",
         a=dict(buf=list(range(1, 17)), shape=[2, 2, 2, 2], view=[(S, 0, None, None, -1), (S, 2, None, None, -1)]),
         b=dict(buf=[100.0, 200.0], shape=[2]), shape=[2, 2, 2, 2],
         spots=[((0, 0, 0, 0), 111.0), ((0, 0, 0, 1), 212.0)]),
    # ---------------------------------------------------------------- broadcast, in place
    dict(name="broadcast_div_in_place", cite="ops/mod.rs:1461-1471", kind="binary_assign", dtype="f32", op="div",
         a=dict(buf=[10.0, 20.0, 30.0, 40.0], shape=[4]), b=dict(buf=[2.0], shape=[]),
         buf=[5.0, 10.0, 15.0, 20.0]),
    dict(name="add_assign_broadcast", cite="ops/mod.rs:1930-1936", kind="binary_assign", dtype="i32", op="add",
         a=dict(zeros=[3, 3]), b=dict(ones=[3]), buf=[1] * 9),
    dict(name="sub_assign_broadcast", cite="ops/mod.rs:1985-1991", kind="binary_assign", dtype="i32", op="sub",
         a=dict(buf=[5, 10, 15], shape=[3]), b=dict(ones=[3]), buf=[4, 9, 14]),
    dict(name="mul_assign_broadcast", cite="ops/mod.rs:2052-2058", kind="binary_assign", dtype="i32", op="mul",
         a=dict(buf=[2, 4, 6], shape=[3]), b=dict(buf=[3, 3, 3], shape=[3]), buf=[6, 12, 18]),
    dict(name="broadcast_inplace_with_negative_step", cite="ops/mod.rs:2580-2601", kind="binary_assign",
         dtype="f32", op="add", a=dict(buf=[1, 2, 3, 4, 5, 6], shape=[2, 3], view=[(S, 1, None, None, -1)]),
         b=dict(buf=[10.0], shape=[1, 1]), buf=[11.0, 12.0, 13.0, 14.0, 15.0, 16.0]),
    # ---------------------------------------------------------------- shape errors
    dict(name="broadcast_incompatible_dimensions_3d", cite="ops/mod.rs:1491-1498", kind="broadcast_error",
         a_shape=[3, 4], b_shape=[2, 5, 6]),
    dict(name="broadcast_both_singletons_incompatible_2d", cite="ops/mod.rs:1886-1894", kind="broadcast_error",
         a_shape=[3, 4], b_shape=[5, 1]),
    dict(name="add_assign_broadcast_incompatible", cite="ops/mod.rs:1940-1945", kind="assign_shape_error",
         a_shape=[1, 3], b_shape=[4, 3]),
    # ---------------------------------------------------------------- reductions (f64, (4,2) matrix)
    dict(name="reduce_total_sum_case1", cite="backend/cpu.rs:1166-1171", kind="reduce_total", dtype="f64", op="sum",
         a=dict(buf=[0.2, 0.3, 0.1, 0.3, 0.3, -0.1, -0.3, 0.3], shape=[4, 2]), value=1.0999999999999999,
         # the reference's own CUDA test of the same tensor expects the tree-ordered sum
         # (backend/cuda.rs:2304-2309): a GPU engine is checked against this value instead
         cuda_value=1.1),
    dict(name="reduce_total_max_case1", cite="backend/cpu.rs:1174-1179", kind="reduce_total", dtype="f64", op="max",
         a=dict(buf=[0.2, 0.3, 0.1, 0.3, 0.3, -0.1, -0.3, 0.3], shape=[4, 2]), value=0.3),
    dict(name="reduce_total_min_case1", cite="backend/cpu.rs:1182-1187", kind="reduce_total", dtype="f64", op="min",
         a=dict(buf=[0.2, 0.3, 0.1, -0.9, 0.3, -0.1, -0.3, 0.3], shape=[4, 2]), value=-0.9),
    dict(name="reduce_total_prod_case1", cite="backend/cpu.rs:1191-1196", kind="reduce_total", dtype="f64",
         op="prod", a=dict(buf=[1., 2., 3., 4., 5., 6., 7., 8.], shape=[4, 2]), value=40320.0),
    dict(name="reduce_sum_case1", cite="backend/cpu.rs:1199-1210", kind="reduce_axis", dtype="f64", op="sum", axis=0,
         a=dict(buf=[1., 0., 1., 0., 1., 1., 1., 0.], shape=[4, 2]), shape=[1, 2], values=[4., 1.]),
    dict(name="reduce_max_case1", cite="backend/cpu.rs:1213-1223", kind="reduce_axis", dtype="f64", op="max", axis=0,
         a=dict(buf=[3., 5., 6., 8., 1., 2., -1., 4.], shape=[4, 2]), shape=[1, 2], values=[6., 8.]),
    dict(name="reduce_min_case1", cite="backend/cpu.rs:1226-1237", kind="reduce_axis", dtype="f64", op="min", axis=0,
         a=dict(buf=[3., 5., 6., 8., 1., 2., -1., 4.], shape=[4, 2]), shape=[1, 2], values=[-1., 2.]),
    dict(name="reduce_prod_case1", cite="backend/cpu.rs:1240-1249", kind="reduce_axis", dtype="f64", op="prod",
         axis=0, a=dict(buf=[3., 5., 6., 8., 1., 2., -1., 4.], shape=[4, 2]), shape=[1, 2], values=[-18., 320.]),
    dict(name="reduce_mean_case1", cite="backend/cpu.rs:1252-1263", kind="reduce_axis", dtype="f64", op="mean",
         axis=0, a=dict(buf=[1., 2., 3., 4., 5., 6., 7., 8.], shape=[4, 2]), shape=[1, 2], values=[4.0, 5.0]),
    dict(name="reduce_mean_case2", cite="backend/cpu.rs:1267-1278", kind="reduce_axis", dtype="f64", op="mean",
         axis=1, a=dict(buf=[1., 2., 3., 4., 5., 6., 7., 8.], shape=[4, 2]), shape=[4, 1],
         values=[1.5, 3.5, 5.5, 7.5]),
    # ---------------------------------------------------------------- reductions only the reference's CUDA backend has
    # (its CPU backend panics for them); values are the ones its CUDA tests expect
    dict(name="reduce_total_argmax_case1", cite="backend/cuda.rs:2320-2331", kind="reduce_ext", dtype="f64", op="argmax",
         axis=None, a=dict(buf=[0.2, 0.3, 0.1, 0.7, 0.3, -0.1, -0.3, 0.3], shape=[4, 2]), shape=[], values=[3]),
    dict(name="reduce_total_argmin_case1", cite="backend/cuda.rs:2333-2344", kind="reduce_ext", dtype="f64", op="argmin",
         axis=None, a=dict(buf=[0.2, 0.3, 0.1, 0.7, 0.3, -0.1, -0.3, 0.3], shape=[4, 2]), shape=[], values=[6]),
    dict(name="reduce_total_variance_unbiased", cite="backend/cuda.rs:2376-2382", kind="reduce_ext", dtype="f64", op="var",
         axis=None, a=dict(buf=[1., 2., 3., 4., 5., 6., 7., 8.], shape=[4, 2]), shape=[], values=[6.0]),
    dict(name="reduce_total_variance_biased", cite="backend/cuda.rs:2384-2390", kind="reduce_ext", dtype="f64", op="pop_var",
         axis=None, a=dict(buf=[1., 2., 3., 4., 5., 6., 7., 8.], shape=[4, 2]), shape=[], values=[5.25]),
    dict(name="reduce_total_stdev_unbiased", cite="backend/cuda.rs:2392-2398", kind="reduce_ext", dtype="f64", op="std",
         axis=None, a=dict(buf=[1., 2., 3., 4., 5., 6., 7., 8.], shape=[4, 2]), shape=[], values=[2.449489742783178]),
    dict(name="reduce_total_stdev_biased", cite="backend/cuda.rs:2400-2406", kind="reduce_ext", dtype="f64", op="pop_std",
         axis=None, a=dict(buf=[1., 2., 3., 4., 5., 6., 7., 8.], shape=[4, 2]), shape=[], values=[2.29128784747792]),
    dict(name="reduce_total_norm_l1", cite="backend/cuda.rs:2408-2414", kind="reduce_ext", dtype="f64", op="l1",
         axis=None, a=dict(buf=[1., 2., 3., 4., 5., 6., 7., 8.], shape=[4, 2]), shape=[], values=[36.]),
    dict(name="reduce_total_norm_l2", cite="backend/cuda.rs:2416-2422", kind="reduce_ext", dtype="f64", op="l2",
         axis=None, a=dict(buf=[1., 2., 3., 4., 5., 6., 7., 8.], shape=[4, 2]), shape=[], values=[14.2828568570857]),
    dict(name="reduce_argmax_case1", cite="backend/cuda.rs:2474-2485", kind="reduce_ext", dtype="f64", op="argmax", axis=0,
         a=dict(buf=[1., 4., 3., 2., 9., 6., 7., 1.], shape=[4, 2]), shape=[1, 2], values=[2, 2]),
    dict(name="reduce_argmin_case1", cite="backend/cuda.rs:2489-2500", kind="reduce_ext", dtype="f64", op="argmin", axis=0,
         a=dict(buf=[1., -4., 3., 2., 9., 6., -7., 1.], shape=[4, 2]), shape=[1, 2], values=[3, 0]),
    dict(name="reduce_variance_case1", cite="backend/cuda.rs:2514-2526", kind="reduce_ext", dtype="f64", op="var", axis=0,
         a=dict(buf=[1., 2., 3., 4., 5., 6., 7., 8.], shape=[4, 2]), shape=[1, 2], values=[6.666666666666667, 6.666666666666667]),
    dict(name="reduce_pop_var_case1", cite="backend/cuda.rs:2528-2535", kind="reduce_ext", dtype="f64", op="pop_var", axis=0,
         a=dict(buf=[1., 2., 3., 4., 5., 6., 7., 8.], shape=[4, 2]), shape=[1, 2], values=[5., 5.]),
    dict(name="reduce_stdev_unbiased", cite="backend/cuda.rs:2537-2544", kind="reduce_ext", dtype="f64", op="std", axis=0,
         a=dict(buf=[1., 2., 3., 4., 5., 6., 7., 8.], shape=[4, 2]), shape=[1, 2], values=[2.581988897471611, 2.581988897471611]),
    dict(name="reduce_stdev_biased", cite="backend/cuda.rs:2546-2553", kind="reduce_ext", dtype="f64", op="pop_std", axis=0,
         a=dict(buf=[1., 2., 3., 4., 5., 6., 7., 8.], shape=[4, 2]), shape=[1, 2], values=[2.23606797749979, 2.23606797749979]),
    dict(name="reduce_logsumexp", cite="backend/cuda.rs:2555-2562", kind="reduce_ext", dtype="f64", op="logsumexp", axis=0,
         a=dict(buf=[1., 2., 3., 4., 5., 6., 7., 8.], shape=[4, 2]), shape=[1, 2], values=[7.145077938960783, 8.145077938960782]),
    dict(name="reduce_norm_l1", cite="backend/cuda.rs:2564-2571", kind="reduce_ext", dtype="f64", op="l1", axis=0,
         a=dict(buf=[1., 2., 3., 4., 5., 6., 7., 8.], shape=[4, 2]), shape=[1, 2], values=[16., 20.]),
    dict(name="reduce_norm_l2", cite="backend/cuda.rs:2573-2580", kind="reduce_ext", dtype="f64", op="l2", axis=0,
         a=dict(buf=[1., 2., 3., 4., 5., 6., 7., 8.], shape=[4, 2]), shape=[1, 2], values=[9.16515138991168, 10.954451150103322]),
    dict(name="reduce_norm_l2_f32", cite="backend/cuda.rs:2582-2589", kind="reduce_ext", dtype="f32", op="l2", axis=0,
         a=dict(buf=[1., 2., 3., 4., 5., 6., 7., 8.], shape=[4, 2]), shape=[1, 2], values=[9.165152, 10.954452]),
    # ---------------------------------------------------------------- unary fixtures (three layouts)
    # testing/mod.rs:97-195: contiguous (2,1); 1-D strided = (3,1) sliced step 2 on dim 0;
    # N-d strided = (4,4,1) sliced step 2 on dims 0 and 1.  truth applied to viewed elements.
    dict(name="unary_negate_contiguous", cite="ops/unary/mod.rs:407-411", kind="unary_fixture", dtype="f64",
         layout="contiguous", definition=[1.0, 1.0], op="neg", truth="neg"),
    dict(name="unary_negate_1d_strided", cite="ops/unary/mod.rs:414-418", kind="unary_fixture", dtype="f64",
         layout="1d", definition=[1.0, 1.0, 1.0], op="neg", truth="neg"),
    dict(name="unary_negate_nd_strided", cite="ops/unary/mod.rs:421-425", kind="unary_fixture", dtype="f64",
         layout="nd", definition=[1.0] * 16, op="neg", truth="neg"),
    dict(name="unary_relu_contiguous", cite="ops/unary/mod.rs:428-430", kind="unary_fixture", dtype="f64",
         layout="contiguous", definition=[-1.0, 1.0], op="relu", truth="max0"),
    dict(name="unary_relu_1d_strided", cite="ops/unary/mod.rs:433-439", kind="unary_fixture", dtype="f64",
         layout="1d", definition=[-1.0, 1.0, -1.0], op="relu", truth="max0"),
    dict(name="unary_relu_nd_strided", cite="ops/unary/mod.rs:442-451", kind="unary_fixture", dtype="f64",
         layout="nd",
         definition=[-1.0, 1.0, 0.0, 2.0, 1.0, 2.3, -0.3, 0.4, 0.0, -0.3, 0.4, 0.5, -0.2, 0.1, 0.2, -0.5],
         op="relu", truth="max0"),
    dict(name="unary_sign_contiguous", cite="ops/unary/mod.rs:950-952", kind="unary_fixture", dtype="f64",
         layout="contiguous", definition=[0.5, -0.25], op="sign", truth="signum"),
    dict(name="unary_sign_1d_strided", cite="ops/unary/mod.rs:955-957", kind="unary_fixture", dtype="f64",
         layout="1d", definition=[-0.125, 0.5, -0.25], op="sign", truth="signum"),
    dict(name="unary_sign_nd_strided", cite="ops/unary/mod.rs:960-962", kind="unary_fixture", dtype="f64",
         layout="nd", definition=[0.5] * 16, op="sign", truth="signum"),
    # ---------------------------------------------------------------- remaining float unary families
    # Same three-layout fixtures; the reference compares with eps_eq at TEST_TOLERANCE = 1e-5
    # (testing/mod.rs:97-195, core/value.rs:496-497), the truth being a Rust std function.
]


def _ext(name, op, truth, c2, c3, c16, lines, dtype="f64"):
    out = []
    sfx = "" if dtype == "f64" else "_" + dtype
    for layout, d, ln in (("contiguous", c2, lines[0]), ("1d", c3, lines[1]), ("nd", c16, lines[2])):
        out.append(dict(name=f"unary_{name}_{layout}{sfx}", cite=f"ops/unary/mod.rs:{ln}", kind="unary_fixture", dtype=dtype,
                        layout=layout, definition=list(d), op=op, truth=truth, tol=1e-5))
    return out


CASES += _ext("sigmoid", "sigmoid", "sigmoid", [1.0, 1.0], [1.0] * 3, [1.0] * 16, ("453-459", "462-468", "471-477"))
CASES += _ext("silu", "silu", "silu", [1.0, 1.0], [1.0] * 3, [1.0] * 16, ("480-486", "489-495", "498-504"))
CASES += _ext("tanh", "tanh", "tanh", [1.0, 1.0], [1.0] * 3, [1.0] * 16, ("507-513", "516-522", "525-531"))
CASES += _ext("sqrt", "sqrt", "sqrt", [1.0, 1.0], [1.0] * 3, [1.0] * 16, ("534-536", "539-545", "534-536"))
CASES += _ext("ln", "ln", "ln", [1.0, 1.0], [1.0] * 3, [1.0] * 16, ("553-555", "558-564", "553-555"))
CASES += _ext("sin", "sin", "sin", [1.0, 1.0], [1.0] * 3, [1.0] * 16, ("705-707", "710-714", "716-718"))
CASES += _ext("cos", "cos", "cos", [1.0, 1.0], [1.0] * 3, [1.0] * 16, ("721-723", "726-729", "731-733"))
CASES += _ext("tan", "tan", "tan", [1.0, 1.0], [1.0] * 3, [1.0] * 16, ("736-738", "741-744", "746-748"))
CASES += _ext("asin", "asin", "asin", [0.5, 0.5], [0.5] * 3, [0.5] * 16, ("752-754", "757-760", "762-764"))
CASES += _ext("acos", "acos", "acos", [0.5, 0.5], [0.5] * 3, [0.5] * 16, ("767-769", "772-775", "777-779"))
CASES += _ext("atan", "atan", "atan", [1.0, 1.0], [1.0] * 3, [1.0] * 16, ("782-784", "787-790", "792-794"))
CASES += _ext("sinh", "sinh", "sinh", [1.0, 1.0], [1.0] * 3, [1.0] * 16, ("798-800", "803-806", "808-810"))
CASES += _ext("cosh", "cosh", "cosh", [1.0, 1.0], [1.0] * 3, [1.0] * 16, ("813-815", "818-821", "823-825"))
CASES += _ext("asinh", "asinh", "asinh", [1.0, 1.0], [0.5] * 3, [0.5] * 16, ("829-831", "834-837", "839-841"))
CASES += _ext("acosh", "acosh", "acosh", [1.0, 1.0], [1.0] * 3, [1.0] * 16, ("844-846", "849-852", "854-856"))
CASES += _ext("atanh", "atanh", "atanh", [0.5, 0.25], [0.5] * 3, [0.5] * 16, ("859-861", "864-867", "869-871"))
CASES += _ext("rsqrt", "rsqrt", "rsqrt", [0.5, 0.25], [0.5] * 3, [0.5] * 16, ("875-877", "880-883", "885-887"))
CASES += _ext("reciprocal", "reciprocal", "reciprocal", [0.5, 0.25], [0.5] * 3, [0.5] * 16, ("890-892", "895-898", "900-902"))
CASES += _ext("square", "square", "square", [0.5, 0.25], [0.5] * 3, [0.5] * 16, ("905-907", "910-913", "915-917"))
CASES += _ext("cube", "cube", "cube", [0.5, 0.25], [0.5] * 3, [0.5] * 16, ("920-922", "925-928", "930-932"))
CASES += _ext("exp", "exp", "exp", [0.5, 0.25], [0.125, 0.5, 0.25], [0.5] * 16, ("935-937", "940-942", "945-947"))


# ---------------------------------------------------------------------------------------------
# The remaining CPU-side tests of ops/mod.rs (the `_cuda` / `_remote` twins of every test in that
# file repeat the same tensors and expectations on the other backends).
# Extra expectation keys: "buf_close" (values, eps) for the tests that assert |x - e| < eps;
# "buf_at" [(flat index, value)] for the tests that look at single buffer elements.
# kind "program": steps on ONE tensor, in order --
#   ("assign", view ops, op, value)            view op= value
#   ("out", view ops, op, value, values)       (view op value) == values, tensor untouched
# kind "view_values": the elements of a view, read one by one with get().
# ---------------------------------------------------------------------------------------------
def _sa(name, cite, dtype, buf, shape, ops, out, **kw):
    return dict(name=name, cite=f"ops/mod.rs:{cite}", kind="scalar_assign", dtype=dtype, a=dict(buf=buf, shape=shape),
                ops=ops, buf=out, **kw)


def _so(name, cite, dtype, buf, shape, op, value, oshape, values, view=None):
    a = dict(buf=buf, shape=shape)
    if view:
        a["view"] = view
    return dict(name=name, cite=f"ops/mod.rs:{cite}", kind="scalar", dtype=dtype, a=a, op=op, value=value, shape=oshape,
                values=values)


def _bb(name, cite, op, a, b, oshape, **expect):
    return dict(name=name, cite=f"ops/mod.rs:{cite}", kind="binary", dtype="f32", op=op, a=a, b=b, shape=oshape, **expect)


def _v2(x, y):
    return dict(buf=[x, y], shape=[2])


_ONES23 = dict(ones=[2, 3])

CASES += [
    _sa("add", "16-25", "i32", [1, 2, 3], [3], [("add", 5)], [6, 7, 8]),
    _sa("add_ref", "26-35", "i32", [1, 2, 3], [3], [("add", 10)], [11, 12, 13]),
    _sa("add_negative", "36-45", "i32", [10, 20, 30], [3], [("add", -5)], [5, 15, 25]),
    _sa("sub", "46-54", "i32", [10, 20, 30], [3], [("sub", 5)], [5, 15, 25]),
    _sa("sub_ref", "55-64", "i32", [10, 20, 30], [3], [("sub", 10)], [0, 10, 20]),
    _sa("sub_negative", "65-75", "i32", [1, 2, 3], [3], [("sub", -5)], [6, 7, 8]),
    _sa("mul", "76-84", "i32", [1, 2, 3], [3], [("mul", 5)], [5, 10, 15]),
    _sa("div", "85-93", "f32", [1., 2., 3.], [3], [("div", 5.)], [0.2, 0.4, 0.6]),
    _sa("mul_ref", "94-103", "i32", [1, 2, 3], [3], [("mul", 10)], [10, 20, 30]),
    _sa("mul_negative", "104-113", "i32", [1, 2, 3], [3], [("mul", -5)], [-5, -10, -15]),
    _so("add_not_inplace", "257-270", "i32", [1, 2, 3], [3], "add", 5, [3], [6, 7, 8]),
    _so("add_ref_not_inplace", "271-281", "i32", [1, 2, 3], [3], "add", 10, [3], [11, 12, 13]),
    _so("sub_not_inplace", "282-291", "i32", [10, 20, 30], [3], "sub", 5, [3], [5, 15, 25]),
    _so("sub_ref_not_inplace", "292-302", "i32", [10, 20, 30], [3], "sub", 10, [3], [0, 10, 20]),
    _so("mul_not_inplace", "303-312", "i32", [1, 2, 3], [3], "mul", 5, [3], [5, 10, 15]),
    _so("mul_ref_not_inplace", "313-323", "i32", [1, 2, 3], [3], "mul", 10, [3], [10, 20, 30]),
    _so("add_not_inplace_negative_values", "375-384", "i32", [10, 20, 30], [3], "add", -5, [3], [5, 15, 25]),
    _so("mul_not_inplace_negative_values", "385-394", "i32", [1, 2, 3], [3], "mul", -5, [3], [-5, -10, -15]),
    _so("mul_not_inplace_matrix", "413-426", "i32", [1, 2, 3, 4], [2, 2], "mul", 10, [2, 2], [10, 20, 30, 40]),
    _so("sub_not_inplace_scalar", "427-442", "i32", [100], [], "sub", 50, [], [50]),
    _so("add_immutable_view_inline", "443-455", "i32", [1, 2, 3, 4], [4], "add", 10, [4], [11, 12, 13, 14]),
    _so("add_immutable_view_ref", "456-467", "i32", [5, 10, 15], [3], "add", 100, [3], [105, 110, 115]),
    _so("sub_immutable_view_inline", "468-479", "i32", [100, 200, 300], [3], "sub", 50, [3], [50, 150, 250]),
    _so("sub_immutable_view_with_slice", "480-493", "i32", [10, 20, 30, 40, 50, 60], [2, 3], "sub", 5, [3], [5, 15, 25],
        view=[(I, 0, 0)]),
    _so("mul_immutable_view_inline", "494-505", "i32", [2, 4, 6, 8], [4], "mul", 3, [4], [6, 12, 18, 24]),
    _so("mul_immutable_view_matrix", "506-530", "i32", [1, 2, 3, 4, 5, 6], [2, 3], "mul", 10, [2, 3],
        [10, 20, 30, 40, 50, 60]),
    _so("sub_immutable_view_scalar", "531-543", "i32", [999], [], "sub", 99, [], [900]),
    _so("mul_immutable_view_noncontiguous_slice", "544-573", "i32", [1, 2, 3, 4, 5, 6], [2, 3], "mul", 5, [2], [10, 25],
        view=[(I, 1, 1)]),
    _so("sub_immutable_view_negative_values", "574-584", "i32", [-10, -20, -30], [3], "sub", 5, [3], [-15, -25, -35]),
    _so("mul_immutable_view_with_ref", "585-602", "i32", [7, 14, 21], [3], "mul", 2, [3], [14, 28, 42]),
    _sa("scalar_add_operation", "603-611", "i32", [42], [], [("add", 10)], [52]),
    _sa("scalar_mul_operation", "612-619", "i32", [7], [], [("mul", 6)], [42]),
    _sa("scalar_sub_operation", "620-627", "i32", [100], [], [("sub", 58)], [42]),
    _sa("scalar_negative_value", "628-636", "i32", [-10], [], [("mul", -3), ("add", 5)], [35]),
    _sa("scalar_zero_operations", "637-646", "i32", [0], [], [("add", 42), ("mul", 0), ("add", 10)], [10]),
    _so("scalar_non_inplace", "647-657", "i32", [100], [], "add", 50, [], [150]),
    _sa("single_element_1d", "658-666", "i32", [5], [1], [("add", 10), ("mul", 2)], [30]),
    _sa("single_element_2d", "667-674", "i32", [8], [1, 1], [("mul", 5)], [40]),
    _sa("single_element_3d", "675-685", "i32", [3], [1, 1, 1], [("add", 7), ("mul", 3)], [30]),
    _sa("tall_matrix_operations", "686-693", "i32", list(range(1, 10)), [9, 1], [("mul", 2)], list(range(2, 19, 2))),
    _sa("wide_matrix_operations", "694-701", "i32", list(range(1, 10)), [1, 9], [("add", 10)], list(range(11, 20))),
    _sa("rectangular_matrix_2x5", "702-715", "i32", list(range(1, 11)), [2, 5], [("mul", 3)], list(range(3, 31, 3))),
    _sa("rectangular_matrix_5x2", "716-729", "i32", list(range(1, 11)), [5, 2], [("sub", 1)], list(range(0, 10))),
    _sa("rectangular_3d_tensor", "730-740", "i32", list(range(1, 25)), [2, 3, 4], [("add", 100)], list(range(101, 125))),
    _sa("zero_tensor_operations", "760-768", "i32", [0, 0, 0, 0], [4], [("add", 10), ("mul", 2)], [20, 20, 20, 20]),
    _sa("operations_resulting_in_zero", "769-776", "i32", [5, 10, 15, 20], [4], [("mul", 0)], [0, 0, 0, 0]),
    _sa("mixed_positive_negative_values", "777-792", "i32", [-5, 10, -15, 20, -25, 30], [6], [("mul", 2), ("add", 10)],
        [0, 30, -20, 50, -40, 70]),
    dict(name="3d_noncontiguous_slice_view", cite="ops/mod.rs:954-977", kind="view_values", dtype="i32",
         a=dict(buf=list(range(1, 25)), shape=[2, 3, 4], view=[(I, 1, 1)]), shape=[2, 4],
         values=[5, 6, 7, 8, 17, 18, 19, 20]),
    _sa("long_operation_chain", "1020-1038", "i32", [1, 2, 3, 4], [4],
        [("add", 1), ("mul", 2), ("sub", 1), ("mul", 3), ("add", 10), ("sub", 5), ("mul", 2), ("add", 2), ("sub", 10),
         ("mul", 1)], [20, 32, 44, 56]),
    dict(name="alternating_inplace_noninplace", cite="ops/mod.rs:1039-1062", kind="program", dtype="i32",
         a=dict(buf=[5, 10, 15], shape=[3]),
         steps=[("assign", [], "add", 5), ("out", [], "mul", 2, [20, 30, 40]), ("assign", [], "mul", 3),
                ("out", [], "add", 10, [40, 55, 70])], buf=[30, 45, 60]),
    dict(name="multiple_views_different_ops", cite="ops/mod.rs:1063-1092", kind="program", dtype="i32",
         a=dict(buf=[1, 2, 3, 4, 5, 6], shape=[2, 3]),
         steps=[("assign", [(I, 0, 0)], "add", 10), ("assign", [(I, 0, 1)], "mul", 5)], buf=[11, 12, 13, 20, 25, 30]),
    dict(name="f32_small_values", cite="ops/mod.rs:1093-1107", kind="scalar_assign", dtype="f32",
         a=dict(buf=[0.0001, 0.0002, 0.0003], shape=[3]), ops=[("mul", 1000.0)], buf_close=([0.1, 0.2, 0.3], 1e-6)),
    dict(name="f64_precision", cite="ops/mod.rs:1108-1124", kind="scalar_assign", dtype="f64",
         a=dict(buf=[1.0 / 3.0, 2.0 / 3.0, 1.0], shape=[3]), ops=[("mul", 3.0)], buf_close=([1.0, 2.0, 3.0], 1e-10)),
    dict(name="very_imbalanced_shape_1000x2", cite="ops/mod.rs:1125-1138", kind="scalar_assign", dtype="i32",
         a=dict(buf=list(range(1, 2001)), shape=[1000, 2]), ops=[("add", 5)],
         buf_at=[(0, 6), (1, 7), (1998, 2004), (1999, 2005)]),
    dict(name="very_imbalanced_shape_2x1000", cite="ops/mod.rs:1139-1153", kind="scalar_assign", dtype="i32",
         a=dict(buf=list(range(1, 2001)), shape=[2, 1000]), ops=[("mul", 2)],
         buf_at=[(0, 2), (999, 2000), (1000, 2002), (1999, 4000)]),
    # ---- broadcast shape errors (#[should_panic]) and broadcast shapes / spot values
    dict(name="broadcast_incompatible_inner_dim", cite="ops/mod.rs:1501-1510", kind="broadcast_error", a_shape=[5], b_shape=[2, 3, 7]),
    dict(name="broadcast_incompatible_middle_dim", cite="ops/mod.rs:1511-1520", kind="broadcast_error", a_shape=[2, 3, 4], b_shape=[2, 5, 4]),
    dict(name="broadcast_incompatible_4d", cite="ops/mod.rs:1521-1530", kind="broadcast_error", a_shape=[2, 3, 4, 5], b_shape=[2, 7, 4, 5]),
    dict(name="broadcast_incompatible_5d_multiple", cite="ops/mod.rs:1531-1540", kind="broadcast_error", a_shape=[1, 2, 3, 4, 5],
         b_shape=[6, 2, 7, 4, 5]),
    dict(name="broadcast_both_non_singleton_mismatch", cite="ops/mod.rs:1541-1551", kind="broadcast_error", a_shape=[4, 5, 6],
         b_shape=[4, 3, 6]),
    _bb("broadcast_all_singletons", "1552-1563", "add", dict(ones=[1, 1, 1]), dict(ones=[5, 6, 7]), [5, 6, 7],
        spots=[((0, 0, 0), 2.0), ((4, 5, 6), 2.0)]),
    _bb("broadcast_identity", "1564-1580", "add", dict(ones=[3, 4, 5]), dict(ones=[3, 4, 5]), [3, 4, 5], all=2.0),
    _bb("broadcast_alternating_singletons", "1581-1592", "add", dict(ones=[1, 4, 1, 6]), dict(ones=[3, 1, 5, 1]), [3, 4, 5, 6],
        spots=[((0, 0, 0, 0), 2.0), ((2, 3, 4, 5), 2.0)]),
    _bb("broadcast_trailing_singleton", "1593-1609", "add", dict(ones=[3, 4, 1]), dict(ones=[3, 4, 5]), [3, 4, 5], all=2.0),
    _bb("broadcast_leading_singleton", "1610-1628", "add", dict(ones=[1, 4, 5]), dict(ones=[3, 4, 5]), [3, 4, 5], all=2.0),
    _bb("broadcast_shape_2d_plus_3d", "1629-1639", "add", dict(ones=[4, 5]), dict(ones=[3, 4, 5]), [3, 4, 5]),
    _bb("broadcast_shape_1d_plus_4d", "1640-1650", "add", dict(ones=[7]), dict(ones=[2, 3, 4, 7]), [2, 3, 4, 7]),
    _bb("broadcast_shape_singleton_expansion", "1651-1661", "add", dict(ones=[1, 5, 1]), dict(ones=[4, 5, 6]), [4, 5, 6]),
    _bb("broadcast_shape_prepending", "1662-1672", "add", dict(ones=[5, 6]), dict(ones=[2, 3, 4, 5, 6]), [2, 3, 4, 5, 6]),
    _bb("broadcast_shape_both_expand", "1673-1683", "add", dict(ones=[1, 4, 1, 6]), dict(ones=[3, 1, 5, 6]), [3, 4, 5, 6]),
    _bb("broadcast_shape_scalar_expansion", "1684-1694", "add", dict(buf=[42.0], shape=[]), dict(ones=[2, 3, 4, 5, 6]),
        [2, 3, 4, 5, 6]),
    _bb("broadcast_shape_complex_5d", "1695-1709", "add", dict(ones=[1, 1, 3, 1, 5]), dict(ones=[2, 4, 3, 6, 5]), [2, 4, 3, 6, 5]),
    dict(name="broadcast_both_singletons_incompatible_3d", cite="ops/mod.rs:1897-1907", kind="broadcast_error", a_shape=[2, 1, 4],
         b_shape=[1, 3, 5]),
    dict(name="broadcast_both_singletons_incompatible_4d", cite="ops/mod.rs:1908-1918", kind="broadcast_error", a_shape=[1, 3, 1, 6],
         b_shape=[2, 1, 4, 7]),
    dict(name="broadcast_both_singletons_incompatible_middle", cite="ops/mod.rs:1919-1929", kind="broadcast_error", a_shape=[2, 4, 1],
         b_shape=[3, 1, 5]),
    dict(name="sub_assign_broadcast_incompatible", cite="ops/mod.rs:1995-2005", kind="assign_shape_error", a_shape=[1, 3], b_shape=[4, 3]),
    dict(name="mul_assign_broadcast_incompatible", cite="ops/mod.rs:2062-2073", kind="assign_shape_error", a_shape=[1, 3], b_shape=[4, 3]),
    # ---- every owner / view / reference combination of the operands reaches the same backend call
    _bb("tensorbase_add_tensorbase", "2074-2082", "add", _ONES23, _ONES23, [2, 3], spots=[((0, 0), 2.0)]),
    _bb("tensorbase_sub_tensorbase", "2083-2091", "sub", _v2(5.0, 3.0), dict(ones=[2]), [2], values=[4.0, 2.0]),
    _bb("tensorbase_mul_tensorbase", "2092-2101", "mul", _v2(2.0, 3.0), _v2(4.0, 5.0), [2], values=[8.0, 15.0]),
    _bb("tensorbase_add_tensorview", "2102-2109", "add", _ONES23, _ONES23, [2, 3], spots=[((0, 0), 2.0)]),
    _bb("tensorbase_sub_tensorview", "2110-2118", "sub", _v2(10.0, 20.0), _v2(3.0, 7.0), [2], values=[7.0, 13.0]),
    _bb("tensorbase_mul_tensorview", "2119-2128", "mul", _v2(6.0, 7.0), _v2(2.0, 3.0), [2], values=[12.0, 21.0]),
    _bb("tensorbase_add_tensorviewmut", "2129-2136", "add", _ONES23, _ONES23, [2, 3], spots=[((1, 2), 2.0)]),
    _bb("tensorbase_sub_tensorviewmut", "2137-2145", "sub", _v2(8.0, 9.0), _v2(3.0, 4.0), [2], values=[5.0, 5.0]),
    _bb("tensorbase_mul_tensorviewmut", "2146-2155", "mul", _v2(5.0, 6.0), _v2(2.0, 2.0), [2], values=[10.0, 12.0]),
    _bb("tensorbase_add_ref_tensorbase", "2156-2163", "add", _ONES23, _ONES23, [2, 3], spots=[((0, 0), 2.0)]),
    _bb("tensorbase_sub_ref_tensorbase", "2164-2172", "sub", _v2(15.0, 25.0), _v2(5.0, 10.0), [2], values=[10.0, 15.0]),
    _bb("tensorbase_mul_ref_tensorbase", "2173-2182", "mul", _v2(3.0, 4.0), _v2(5.0, 6.0), [2], values=[15.0, 24.0]),
    _bb("ref_tensorbase_add_tensorbase", "2183-2190", "add", _ONES23, _ONES23, [2, 3], spots=[((0, 0), 2.0)]),
    _bb("ref_tensorbase_sub_tensorbase", "2191-2199", "sub", _v2(20.0, 30.0), _v2(8.0, 12.0), [2], values=[12.0, 18.0]),
    _bb("ref_tensorbase_mul_tensorbase", "2200-2209", "mul", _v2(7.0, 8.0), _v2(2.0, 3.0), [2], values=[14.0, 24.0]),
    _bb("ref_tensorbase_add_ref_tensorbase", "2210-2217", "add", _ONES23, _ONES23, [2, 3], spots=[((0, 0), 2.0)]),
    _bb("ref_tensorbase_sub_ref_tensorbase", "2218-2226", "sub", _v2(100.0, 200.0), _v2(30.0, 70.0), [2], values=[70.0, 130.0]),
    _bb("ref_tensorbase_mul_ref_tensorbase", "2227-2236", "mul", _v2(9.0, 10.0), _v2(2.0, 4.0), [2], values=[18.0, 40.0]),
    _bb("tensorview_add_tensorbase", "2237-2244", "add", _ONES23, _ONES23, [2, 3], spots=[((0, 0), 2.0)]),
    _bb("tensorview_sub_tensorbase", "2245-2253", "sub", _v2(50.0, 60.0), _v2(20.0, 25.0), [2], values=[30.0, 35.0]),
    _bb("tensorview_mul_tensorbase", "2254-2263", "mul", _v2(11.0, 12.0), _v2(3.0, 4.0), [2], values=[33.0, 48.0]),
    _bb("tensorview_add_tensorview", "2264-2271", "add", _ONES23, _ONES23, [2, 3], spots=[((0, 0), 2.0)]),
    _bb("tensorview_sub_tensorview", "2272-2280", "sub", _v2(70.0, 80.0), _v2(30.0, 35.0), [2], values=[40.0, 45.0]),
    _bb("tensorview_mul_tensorview", "2281-2290", "mul", _v2(13.0, 14.0), _v2(2.0, 5.0), [2], values=[26.0, 70.0]),
    _bb("tensorviewmut_add_tensorbase", "2291-2298", "add", _ONES23, _ONES23, [2, 3], spots=[((0, 0), 2.0)]),
    _bb("tensorviewmut_sub_tensorbase", "2299-2307", "sub", _v2(90.0, 100.0), _v2(40.0, 45.0), [2], values=[50.0, 55.0]),
    _bb("tensorviewmut_mul_tensorbase", "2308-2317", "mul", _v2(15.0, 16.0), _v2(2.0, 3.0), [2], values=[30.0, 48.0]),
    _bb("tensorviewmut_add_tensorviewmut", "2318-2325", "add", _ONES23, _ONES23, [2, 3], spots=[((0, 0), 2.0)]),
    _bb("tensorviewmut_sub_tensorviewmut", "2326-2334", "sub", _v2(110.0, 120.0), _v2(50.0, 60.0), [2], values=[60.0, 60.0]),
    _bb("tensorviewmut_mul_tensorviewmut", "2335-2344", "mul", _v2(17.0, 18.0), _v2(3.0, 4.0), [2], values=[51.0, 72.0]),
    _bb("ref_tensorview_add_ref_tensorview", "2345-2352", "add", _ONES23, _ONES23, [2, 3], spots=[((0, 0), 2.0)]),
    _bb("ref_tensorview_sub_ref_tensorview", "2353-2361", "sub", _v2(150.0, 200.0), _v2(50.0, 100.0), [2], values=[100.0, 100.0]),
    _bb("ref_tensorview_mul_ref_tensorview", "2362-2371", "mul", _v2(19.0, 20.0), _v2(2.0, 5.0), [2], values=[38.0, 100.0]),
    _bb("ref_tensorviewmut_add_ref_tensorviewmut", "2372-2379", "add", _ONES23, _ONES23, [2, 3], spots=[((0, 0), 2.0)]),
    _bb("ref_tensorviewmut_sub_ref_tensorviewmut", "2380-2388", "sub", _v2(250.0, 300.0), _v2(100.0, 150.0), [2],
        values=[150.0, 150.0]),
    _bb("ref_tensorviewmut_mul_ref_tensorviewmut", "2389-2398", "mul", _v2(21.0, 22.0), _v2(3.0, 4.0), [2], values=[63.0, 88.0]),
    dict(name="tensorviewmut_add_assign_tensorbase", cite="ops/mod.rs:2399-2409", kind="binary_assign", dtype="f32", op="add",
         a=dict(ones=[2, 3]), b=dict(ones=[2, 3]), buf=[2.0] * 6),
    dict(name="tensorviewmut_sub_assign_tensorview", cite="ops/mod.rs:2410-2421", kind="binary_assign", dtype="f32", op="sub",
         a=_v2(10.0, 20.0), b=_v2(3.0, 7.0), buf=[7.0, 13.0]),
    dict(name="tensorviewmut_mul_assign_tensorviewmut", cite="ops/mod.rs:2422-2434", kind="binary_assign", dtype="f32", op="mul",
         a=_v2(5.0, 6.0), b=_v2(2.0, 3.0), buf=[10.0, 18.0]),
]


# ---------------------------------------------------------------------------------------------
# ops/scalar/mod.rs: log / log1p / leaky_relu / elu with a scalar operand, on the three fixture
# layouts of testing/mod.rs, each compared element by element (eps_eq, 1e-5) with the closure the
# test passes as its truth.  f32 / i32 cases from the CPU module (:176-295), f64 cases from the
# CUDA module of the same file (:323-470), which runs the same helper.
# kind "scalar_fixture": op = scalar op code name, value = the operand, truth = formula name.
# ---------------------------------------------------------------------------------------------
_ALT16 = [(-1) ** (k + 1) * (k + 1) for k in range(16)]   # -1, 2, -3, 4, ... 16


def _sfx(fam, dtype, value, truth, c2, c3, c16, lines, v16=None):
    out = []
    for layout, d, ln in (("contiguous", c2, lines[0]), ("1d", c3, lines[1]), ("nd", c16, lines[2])):
        out.append(dict(name=f"scalar_{fam}_{layout}_{dtype}", cite=f"ops/scalar/mod.rs:{ln}", kind="scalar_fixture", dtype=dtype,
                        layout=layout, definition=list(d), op=fam, value=(v16 if (layout == "nd" and v16 is not None) else value),
                        truth=truth, tol=1e-5))
    return out


CASES += _sfx("log", "f32", 10.0, "log_base", [1.4, 2.6], [1.4, 2.6, 3.5], [1.4] * 16, ("185-188", "176-183", "191-194"))
CASES += _sfx("log1p", "f32", 10.0, "log1p_base", [1.4, 2.6], [1.4, 2.6, 3.5], [1.4] * 16, ("205-208", "196-203", "211-214"))
CASES += _sfx("leaky_relu", "f32", 0.1, "leaky", [2.0, -1.5], [1.0, -2.0, 3.0], [float(v) for v in _ALT16],
              ("225-232", "216-223", "234-241"), v16=0.2)
CASES += _sfx("elu", "f32", 0.1, "elu", [2.0, -1.5], [1.0, -2.0, 3.0], [float(v) for v in _ALT16],
              ("252-259", "243-250", "261-268"), v16=0.2)
CASES += _sfx("leaky_relu", "i32", 1, "leaky", [2, -1], [1, -2, 3], _ALT16, ("279-286", "270-277", "288-295"), v16=2)
CASES += _sfx("log", "f64", 10.0, "log_base", [1.4, 2.6], [1.4, 2.6, 3.5], [1.4] * 16, ("333-336", "323-331", "338-341"))
CASES += _sfx("log1p", "f64", 10.0, "log1p_base", [1.4, 2.6], [1.4, 2.6, 3.5], [1.4] * 16, ("373-376", "363-371", "378-381"))
CASES += _sfx("elu", "f64", 0.1, "elu", [2.0, -1.5], [1.0, -2.0, 3.0], [float(v) for v in _ALT16],
              ("455-462", "446-453", "464-471"), v16=0.2)


# ops/unary/mod.rs, the f32 fixtures of the CPU module (:572-702) and the f64 fixtures that only the
# CUDA module of the same file holds (:1565-1802, same helper, same eps)
CASES += _ext("ln", "ln", "ln", [1.5] * 2, [1.5] * 3, [1.5] * 16, ("586-588", "577-583", "572-574"), "f32")
CASES += _ext("expm1", "expm1", "expm1", [1.5] * 2, [1.5] * 3, [1.5] * 16, ("605-607", "596-602", "591-593"), "f32")
CASES += _ext("ln1p", "ln1p", "ln1p", [0.5] * 2, [0.5] * 3, [0.5] * 16, ("624-626", "615-621", "610-612"), "f32")
CASES += _ext("floor", "floor", "floor", [1.7, 2.3], [1.7, 2.3, 3.9], [1.7] * 16, ("643-645", "634-640", "629-631"), "f32")
CASES += _ext("ceil", "ceil", "ceil", [1.3, 2.7], [1.3, 2.7, 3.1], [1.3] * 16, ("662-664", "653-659", "648-650"), "f32")
CASES += _ext("round", "round", "round", [1.4, 2.6], [1.4, 2.6, 3.5], [1.4] * 16, ("681-683", "672-678", "667-669"), "f32")
CASES += _ext("trunc", "trunc", "trunc", [-1.4, 2.6], [-1.4, 2.6, 3.5], [-1.4] * 16, ("700-702", "691-697", "686-688"), "f32")
CASES += [dict(name="unary_sqrt_contiguous_again", cite="ops/unary/mod.rs:548-550", kind="unary_fixture", dtype="f64",
               layout="contiguous", definition=[1.0, 1.0], op="sqrt", truth="sqrt", tol=1e-5),
          dict(name="unary_ln_contiguous_again", cite="ops/unary/mod.rs:567-569", kind="unary_fixture", dtype="f64",
               layout="contiguous", definition=[1.0, 1.0], op="ln", truth="ln", tol=1e-5)]
CASES += _ext("ln_b", "ln", "ln", [1.5] * 2, [1.5, 1.1, 1.5], [1.5] * 16, ("1579-1581", "1570-1576", "1565-1567"))
CASES += _ext("expm1", "expm1", "expm1", [1.5] * 2, [1.5, 1.1, 1.5], [1.5] * 16, ("1598-1600", "1589-1595", "1584-1586"))
CASES += _ext("ln1p", "ln1p", "ln1p", [0.5] * 2, [0.5, 0.1, 0.5], [0.5] * 16, ("1636-1638", "1627-1633", "1622-1624"))
CASES += _ext("floor", "floor", "floor", [1.7, 2.3], [1.7, 2.3, 3.9], [1.7] * 16, ("1674-1676", "1665-1671", "1660-1662"))
CASES += _ext("ceil", "ceil", "ceil", [1.3, 2.7], [1.3, 2.7, 3.1], [1.3] * 16, ("1712-1714", "1703-1709", "1698-1700"))
CASES += _ext("round", "round", "round", [1.3, 2.7], [1.3, 2.7, 3.1], [1.3] * 16, ("1752-1756", "1743-1749", "1736-1740"))
CASES += _ext("trunc", "trunc", "trunc", [-1.3, 2.7], [-1.3, 2.7, 3.1], [-1.3] * 16, ("1798-1802", "1789-1795", "1782-1786"))


# ---------------------------------------------------------------------------------------------
# core/mod.rs: view arithmetic of slicing (ranges, negative and custom steps, errors).  Rust range
# syntax is written out as the Slice it converts to (core/slice.rs:35-103): a..b -> (a, b, +-1),
# a..=b -> end made exclusive (None when a reversed range ends at 0), Slice::from(r).step(k) -> r's
# bounds with step k.
# kind "view_check": shape (and strides, when the test asserts them) of the view, and single elements
# read through it.  kind "slice_error": the slice must be refused; "bounds" = IdxOutOfBounds,
# "shape" = InvalidShape.  kind "view_set": writes through a view, read back through the base tensor.
# ---------------------------------------------------------------------------------------------
def _vc(name, cite, buf, shape, view, oshape, spots, strides=None):
    c = dict(name=name, cite=f"core/mod.rs:{cite}", kind="view_check", dtype="i32", a=dict(buf=buf, shape=shape, view=view),
             shape=oshape, spots=spots)
    if strides is not None:
        c["strides"] = strides
    return c


_R8, _R10, _R16 = list(range(1, 9)), list(range(1, 11)), list(range(16))

CASES += [
    _vc("range_slice_matrix_rows", "115-139", list(range(1, 13)), [4, 3], [(S, 0, 1, 3, 1)], [2, 3],
        [((0, 0), 4), ((0, 1), 5), ((0, 2), 6), ((1, 0), 7), ((1, 1), 8), ((1, 2), 9)], strides=[3, 1]),
    _vc("range_slice_matrix_columns", "142-165", list(range(1, 13)), [3, 4], [(S, 1, 1, 3, 1)], [3, 2],
        [((0, 0), 2), ((0, 1), 3), ((1, 0), 6), ((1, 1), 7), ((2, 0), 10), ((2, 1), 11)], strides=[4, 1]),
    _vc("range_slice_cube_depth", "168-202", list(range(1, 17)), [4, 2, 2], [(S, 0, 1, 3, 1)], [2, 2, 2],
        [((0, 0, 0), 5), ((0, 0, 1), 6), ((0, 1, 0), 7), ((0, 1, 1), 8), ((1, 0, 0), 9), ((1, 0, 1), 10), ((1, 1, 0), 11),
         ((1, 1, 1), 12)], strides=[4, 2, 1]),
    _vc("range_slice_first_n_elements", "205-218", _R8, [8], [(S, 0, 0, 5, 1)], [5], [((0,), 1), ((1,), 2), ((4,), 5)], strides=[1]),
    _vc("range_slice_last_n_elements", "221-234", _R8, [8], [(S, 0, 5, 8, 1)], [3], [((0,), 6), ((1,), 7), ((2,), 8)], strides=[1]),
    _vc("range_slice_of_range_slice_1", "237-248", _R10, [10], [(S, 0, 2, 8, 1)], [6], [((0,), 3), ((5,), 8)]),
    _vc("range_slice_of_range_slice_2", "251-256", _R10, [10], [(S, 0, 2, 8, 1), (S, 0, 1, 4, 1)], [3],
        [((0,), 4), ((1,), 5), ((2,), 6)]),
    dict(name="range_slice_mut", cite="core/mod.rs:259-275", kind="view_set", dtype="i32", a=dict(buf=_R8, shape=[4, 2]),
         view=[(S, 0, 1, 3, 1)], shape=[2, 2], sets=[((0, 0), 30), ((1, 1), 80)], base_spots=[((1, 0), 30), ((2, 1), 80)]),
    _vc("range_slice_full_dimension", "278-292", [1, 2, 3, 4, 5, 6], [2, 3], [(S, 0, 0, 2, 1)], [2, 3], [((0, 0), 1), ((1, 2), 6)],
        strides=[3, 1]),
    _vc("range_slice_single_element", "295-306", [1, 2, 3, 4, 5, 6], [6], [(S, 0, 2, 3, 1)], [1], [((0,), 3)], strides=[1]),
    dict(name="range_slice_errors_1", cite="core/mod.rs:313-316", kind="slice_error", a_shape=[2, 2], slice=(0, 0, 3, 1), error="bounds"),
    dict(name="range_slice_errors_2", cite="core/mod.rs:319-322", kind="slice_error", a_shape=[2, 2], slice=(0, 3, 4, 1), error="bounds"),
    dict(name="range_slice_errors_3", cite="core/mod.rs:325-328", kind="slice_error", a_shape=[2, 2], slice=(0, 2, 1, -1), error="bounds"),
    _vc("negative_step_basic", "332-345", _R8, [8], [(S, 0, None, None, -1)], [8], [((0,), 8), ((1,), 7), ((7,), 1)]),
    _vc("negative_step_with_range", "348-362", _R8, [8], [(S, 0, 6, 2, -1)], [4], [((0,), 7), ((1,), 6), ((2,), 5), ((3,), 4)]),
    _vc("negative_step_skip_elements", "365-378", _R8, [8], [(S, 0, None, None, -2)], [4], [((0,), 8), ((1,), 6), ((2,), 4), ((3,), 2)]),
    _vc("negative_step_matrix_rows", "381-406", list(range(1, 13)), [4, 3], [(S, 0, None, None, -1)], [4, 3],
        [((0, 0), 10), ((0, 1), 11), ((0, 2), 12), ((3, 0), 1), ((3, 1), 2), ((3, 2), 3)]),
    _vc("negative_step_with_start_less_than_end", "409-418", [1, 2, 3, 4, 5, 6], [6], [(S, 0, 2, 5, -1)], [], []),
    _vc("positive_step_with_start_greater_than_end", "421-430", [1, 2, 3, 4, 5, 6], [6], [(S, 0, 5, 2, 1)], [], []),
    _vc("negative_step_partial_range", "433-445", _R8, [8], [(S, 0, 5, None, -1)], [6], [((0,), 6), ((5,), 1)]),
    _vc("negative_step_partial_end", "448-460", _R8, [8], [(S, 0, None, 3, -1)], [4], [((0,), 8), ((3,), 5)]),
    _vc("negative_step_3d_tensor", "463-486", list(range(1, 17)), [4, 2, 2], [(S, 0, None, None, -1)], [4, 2, 2],
        [((0, 0, 0), 13), ((0, 1, 1), 16), ((3, 0, 0), 1), ((3, 1, 1), 4)]),
    _vc("negative_step_chained_1", "489-498", _R10, [10], [(S, 0, None, None, -1)], [10], [((0,), 10)]),
    _vc("negative_step_chained_2", "501-506", _R10, [10], [(S, 0, None, None, -1), (S, 0, None, None, 2)], [5],
        [((0,), 10), ((1,), 8), ((4,), 2)]),
    _vc("negative_step_funtax", "509-522", _R10, [10], [(S, 0, 9, None, -1)], [10], [((0,), 10), ((1,), 9), ((2,), 8)]),
    dict(name="negative_step_mut", cite="core/mod.rs:525-541", kind="view_set", dtype="i32", a=dict(buf=[1, 2, 3, 4, 5, 6], shape=[6]),
         view=[(S, 0, None, None, -1)], shape=[6], sets=[((0,), 60), ((5,), 10)], base_spots=[((0,), 10), ((5,), 60)]),
    dict(name="negative_step_mut_funtax", cite="core/mod.rs:544-560", kind="view_set", dtype="i32",
         a=dict(buf=[1, 2, 3, 4, 5, 6], shape=[6]), view=[(S, 0, None, None, -1)], shape=[6], sets=[((0,), 60), ((5,), 10)],
         base_spots=[((0,), 10), ((5,), 60)]),
    dict(name="negative_step_errors_1", cite="core/mod.rs:567-570", kind="slice_error", a_shape=[6], slice=(0, 10, 2, -1), error="bounds"),
    dict(name="negative_step_errors_2", cite="core/mod.rs:573-576", kind="slice_error", a_shape=[6], slice=(0, 5, 10, -1), error="bounds"),
    dict(name="negative_step_errors_3", cite="core/mod.rs:579-582", kind="slice_error", a_shape=[6], slice=(0, 2, 5, 0), error="shape"),
    _vc("reverse_range_auto_negative_step_1", "586-598", _R10, [10], [(S, 0, 9, 0, -1)], [9], [((0,), 10), ((1,), 9), ((8,), 2)]),
    _vc("reverse_range_auto_negative_step_2", "601-606", _R10, [10], [(S, 0, 9, None, -1)], [10], [((0,), 10), ((9,), 1)]),
    _vc("custom_positive_step_1", "609-622", _R16, [16], [(S, 0, None, None, 2)], [8], [((0,), 0), ((1,), 2), ((2,), 4), ((7,), 14)]),
    _vc("custom_positive_step_2", "624-628", _R16, [16], [(S, 0, 1, 8, 3)], [3], [((0,), 1), ((1,), 4), ((2,), 7)]),
    _vc("custom_positive_step_3", "630-634", _R16, [16], [(S, 0, None, 12, 4)], [3], [((0,), 0), ((1,), 4), ((2,), 8)]),
    _vc("custom_positive_step_4", "636-640", _R16, [16], [(S, 0, 3, None, 5)], [3], [((0,), 3), ((1,), 8), ((2,), 13)]),
    _vc("custom_positive_step_5", "642-645", _R16, [16], [(S, 0, 2, None, 10)], [2], [((0,), 2), ((1,), 12)]),
    _vc("custom_negative_step_1", "648-660", _R16, [16], [(S, 0, None, None, -2)], [8], [((0,), 15), ((1,), 13), ((2,), 11), ((7,), 1)]),
    _vc("custom_negative_step_2", "662-666", _R16, [16], [(S, 0, 10, 1, -3)], [3], [((0,), 10), ((1,), 7), ((2,), 4)]),
    _vc("custom_negative_step_3", "668-673", _R16, [16], [(S, 0, None, 2, -4)], [4], [((0,), 15), ((1,), 11), ((2,), 7), ((3,), 3)]),
    _vc("custom_negative_step_4", "675-679", _R16, [16], [(S, 0, 14, None, -5)], [3], [((0,), 14), ((1,), 9), ((2,), 4)]),
]


# core/mod.rs: fill through a view (Backend::fill_*), and owned() = the row-major copy of a view
# (view_to_contiguous).  kind "fill": value written through the view, then single elements of the
# BASE tensor; kind "owned": shape and buffer of the copy.
_R12 = list(range(12))
CASES += [
    dict(name="fill_contiguous", cite="core/mod.rs:1176-1186", kind="fill", dtype="i32", a=dict(buf=_R12, shape=[3, 4]), value=42,
         buf=[42] * 12),
    dict(name="fill_contiguous_slice", cite="core/mod.rs:1189-1207", kind="fill", dtype="i32",
         a=dict(buf=_R12, shape=[3, 4], view=[(I, 0, 1)]), value=99, buf=[0, 1, 2, 3, 99, 99, 99, 99, 8, 9, 10, 11]),
    dict(name="fill_strided_column", cite="core/mod.rs:1210-1222", kind="fill", dtype="i32",
         a=dict(buf=_R12, shape=[3, 4], view=[(I, 1, 2)]), value=7,
         base_spots=[((0, 2), 7), ((1, 2), 7), ((2, 2), 7), ((0, 0), 0), ((0, 1), 1), ((0, 3), 3)]),
    dict(name="fill_2d_slice", cite="core/mod.rs:1225-1254", kind="fill", dtype="i32",
         a=dict(buf=list(range(24)), shape=[4, 6], view=[(S, 0, 1, 3, 1), (S, 1, 2, 5, 1)]), value=5,
         base_spots=[((1, 2), 5), ((1, 3), 5), ((1, 4), 5), ((2, 2), 5), ((2, 3), 5), ((2, 4), 5), ((0, 2), 2), ((1, 1), 7),
                     ((1, 5), 11), ((3, 2), 20)]),
    dict(name="view_to_owned_contiguous", cite="core/mod.rs:1486-1495", kind="owned", dtype="i32",
         a=dict(buf=[1, 2, 3, 4, 5, 6], shape=[2, 3]), shape=[2, 3], values=[1, 2, 3, 4, 5, 6]),
    dict(name="view_to_owned_noncontiguous_column", cite="core/mod.rs:1498-1515", kind="owned", dtype="i32",
         a=dict(buf=[1, 2, 3, 4, 5, 6], shape=[2, 3], view=[(I, 1, 1)]), shape=[2], values=[2, 5], view_contiguous=False),
    dict(name="view_to_owned_row_slice", cite="core/mod.rs:1518-1528", kind="owned", dtype="i32",
         a=dict(buf=[1, 2, 3, 4, 5, 6], shape=[2, 3], view=[(I, 0, 1)]), shape=[3], values=[4, 5, 6], view_contiguous=True),
    dict(name="view_to_owned_3d_slice", cite="core/mod.rs:1543-1553", kind="owned", dtype="i32",
         a=dict(buf=[1, 2, 3, 4, 5, 6, 7, 8], shape=[2, 2, 2], view=[(I, 0, 1)]), shape=[2, 2], values=[5, 6, 7, 8]),
    dict(name="viewmut_to_owned", cite="core/mod.rs:1556-1563", kind="owned", dtype="i32",
         a=dict(buf=[1, 2, 3, 4, 5, 6], shape=[2, 3]), shape=[2, 3], values=[1, 2, 3, 4, 5, 6]),
]


# core/mod.rs: transpose (= all dims reversed) and permute, on tensors and on slices, read and
# written through.  kind "permute_error": WrongDims / InvalidDim, both reported as a dimension error.
P = "permute"
_M23 = [1, 2, 3, 4, 5, 6]
CASES += [
    _vc("transpose_2d", "2056-2076", _M23, [2, 3], [(P, [1, 0])], [3, 2],
        [((0, 0), 1), ((0, 1), 4), ((1, 0), 2), ((1, 1), 5), ((2, 0), 3), ((2, 1), 6)], strides=[1, 3]),
    _vc("transpose_3d", "2079-2098", list(range(1, 9)), [2, 2, 2], [(P, [2, 1, 0])], [2, 2, 2],
        [((0, 0, 0), 1), ((1, 0, 0), 2), ((0, 1, 0), 3), ((0, 0, 1), 5), ((1, 1, 1), 8)], strides=[1, 2, 4]),
    dict(name="transpose_mut_2d", cite="core/mod.rs:2101-2121", kind="view_set", dtype="i32", a=dict(buf=_M23, shape=[2, 3]),
         view=[(P, [1, 0])], shape=[3, 2], sets=[((0, 0), 10), ((1, 1), 50), ((2, 1), 60)],
         base_spots=[((0, 0), 10), ((1, 1), 50), ((1, 2), 60)]),
    dict(name="transpose_mut_3d", cite="core/mod.rs:2124-2141", kind="view_set", dtype="i32",
         a=dict(buf=list(range(1, 9)), shape=[2, 2, 2]), view=[(P, [2, 1, 0])], shape=[2, 2, 2],
         sets=[((0, 0, 0), 100), ((1, 0, 0), 200), ((0, 0, 1), 500)],
         base_spots=[((0, 0, 0), 100), ((0, 0, 1), 200), ((1, 0, 0), 500)]),
    _vc("permute_2d_swap", "2144-2158", _M23, [2, 3], [(P, [1, 0])], [3, 2], [((0, 0), 1), ((1, 0), 2), ((2, 1), 6)],
        strides=[1, 3]),
    _vc("permute_3d_rotate", "2161-2179", list(range(1, 13)), [2, 2, 3], [(P, [2, 0, 1])], [3, 2, 2],
        [((0, 0, 0), 1), ((1, 0, 0), 2), ((0, 0, 1), 4), ((2, 1, 1), 12)], strides=[1, 6, 3]),
    _vc("permute_3d_partial_swap", "2182-2194", list(range(1, 9)), [2, 2, 2], [(P, [1, 0, 2])], [2, 2, 2],
        [((0, 0, 0), 1), ((1, 0, 0), 3), ((0, 1, 1), 6)], strides=[2, 4, 1]),
    dict(name="permute_mut_with_write", cite="core/mod.rs:2197-2218", kind="view_set", dtype="i32",
         a=dict(buf=list(range(1, 13)), shape=[2, 2, 3]), view=[(P, [2, 0, 1])], shape=[3, 2, 2],
         sets=[((0, 0, 0), 100), ((1, 0, 0), 200), ((2, 1, 1), 1200)],
         base_spots=[((0, 0, 0), 100), ((0, 0, 1), 200), ((1, 1, 2), 1200)]),
    _vc("permute_identity", "2221-2232", _M23, [2, 3], [(P, [0, 1])], [2, 3], [((0, 0), 1), ((1, 2), 6)], strides=[3, 1]),
    _vc("permute_4d", "2235-2247", list(range(1, 17)), [2, 2, 2, 2], [(P, [3, 2, 1, 0])], [2, 2, 2, 2],
        [((0, 0, 0, 0), 1), ((1, 0, 0, 0), 2), ((1, 1, 1, 1), 16)], strides=[1, 2, 4, 8]),
    _vc("permute_on_slice", "2250-2267", list(range(1, 13)), [3, 4], [(S, 0, 1, 3, 1), (P, [1, 0])], [4, 2],
        [((0, 0), 5), ((3, 1), 12)]),
    _vc("transpose_on_slice", "2270-2288", list(range(1, 13)), [4, 3], [(S, 0, 1, 3, 1), (P, [1, 0])], [3, 2],
        [((0, 0), 4), ((2, 1), 9)]),
    _vc("chained_permutations", "2291-2308", list(range(1, 9)), [2, 2, 2], [(P, [2, 0, 1]), (P, [1, 2, 0])], [2, 2, 2],
        [((0, 0, 0), 1), ((1, 0, 0), 5), ((0, 1, 0), 3), ((1, 1, 1), 8)]),
    dict(name="permute_mut_chained", cite="core/mod.rs:2311-2324", kind="view_set", dtype="i32",
         a=dict(buf=list(range(1, 9)), shape=[2, 2, 2]), view=[(P, [1, 0, 2]), (P, [2, 0, 1])], shape=[2, 2, 2],
         sets=[((0, 0, 0), 111)], base_spots=[((0, 0, 0), 111)]),
    dict(name="permute_wrong_dims_error_1", cite="core/mod.rs:2327-2333", kind="permute_error", a_shape=[2, 3], dims=[0]),
    dict(name="permute_wrong_dims_error_2", cite="core/mod.rs:2334-2338", kind="permute_error", a_shape=[2, 3], dims=[0, 1, 2]),
    dict(name="permute_invalid_dim_error_1", cite="core/mod.rs:2341-2347", kind="permute_error", a_shape=[2, 3], dims=[0, 3]),
    dict(name="permute_invalid_dim_error_2", cite="core/mod.rs:2348-2352", kind="permute_error", a_shape=[2, 3], dims=[2, 1]),
    _vc("transpose_then_slice", "2355-2372", _M23, [2, 3], [(P, [1, 0]), (I, 0, 0)], [2], [((0,), 1), ((1,), 4)]),
    dict(name="slice_then_transpose_mut", cite="core/mod.rs:2375-2397", kind="view_set", dtype="i32",
         a=dict(buf=list(range(1, 13)), shape=[3, 4]), view=[(S, 0, 0, 2, 1), (P, [1, 0])], shape=[4, 2],
         sets=[((0, 0), 100), ((3, 1), 800)], base_spots=[((0, 0), 100), ((1, 3), 800), ((2, 0), 9)]),
    dict(name="permute_write_compatibility_complex", cite="core/mod.rs:2400-2422", kind="view_set", dtype="i32",
         a=dict(buf=list(range(1, 25)), shape=[2, 3, 4]), view=[(S, 0, 1, 2, 1), (P, [2, 0, 1])], shape=[4, 1, 3],
         sets=[((0, 0, 0), 1300), ((3, 0, 2), 2400)], base_spots=[((1, 0, 0), 1300), ((1, 2, 3), 2400), ((0, 0, 0), 1)]),
]


# core/mod.rs: unsqueeze / unsqueeze_at / squeeze / squeeze_at (a sample: plain tensors, after slices,
# over negative strides).  View ops ("unsqueeze", dim) and ("squeeze", dim | None).
U, Q = "unsqueeze", "squeeze"
CASES += [
    _vc("unsqueeze_scalar", "2492-2503", [42], [], [(U, 0)], [1], [((0,), 42)], strides=[1]),
    _vc("unsqueeze_1d", "2506-2523", [1, 2, 3, 4, 5], [5], [(U, 0)], [1, 5], [((0, k), k + 1) for k in range(5)], strides=[5, 1]),
    _vc("unsqueeze_2d", "2526-2544", _M23, [2, 3], [(U, 0)], [1, 2, 3],
        [((0, 0, 0), 1), ((0, 0, 1), 2), ((0, 0, 2), 3), ((0, 1, 0), 4), ((0, 1, 1), 5), ((0, 1, 2), 6)], strides=[6, 3, 1]),
    _vc("double_unsqueeze", "2547-2564", [1, 2, 3], [3], [(U, 0), (U, 0)], [1, 1, 3], [((0, 0, 0), 1), ((0, 0, 1), 2), ((0, 0, 2), 3)],
        strides=[3, 3, 1]),
    _vc("unsqueeze_after_slice", "2567-2585", _M23, [2, 3], [(I, 0, 0), (U, 0)], [1, 3], [((0, 0), 1), ((0, 1), 2), ((0, 2), 3)],
        strides=[3, 1]),
    _vc("unsqueeze_after_column_slice", "2588-2606", _M23, [2, 3], [(I, 1, 0), (U, 0)], [1, 2], [((0, 0), 1), ((0, 1), 4)],
        strides=[6, 3]),
    _vc("unsqueeze_at_beginning", "2794-2805", _M23, [2, 3], [(U, 0)], [1, 2, 3],
        [((0, 0, 0), 1), ((0, 0, 2), 3), ((0, 1, 0), 4), ((0, 1, 2), 6)], strides=[6, 3, 1]),
    _vc("unsqueeze_at_middle", "2808-2819", _M23, [2, 3], [(U, 1)], [2, 1, 3],
        [((0, 0, 0), 1), ((0, 0, 2), 3), ((1, 0, 0), 4), ((1, 0, 2), 6)], strides=[3, 3, 1]),
    _vc("unsqueeze_at_end", "2822-2833", _M23, [2, 3], [(U, 2)], [2, 3, 1],
        [((0, 0, 0), 1), ((0, 2, 0), 3), ((1, 0, 0), 4), ((1, 2, 0), 6)], strides=[3, 1, 1]),
    _vc("unsqueeze_at_with_negative_stride", "3199-3214", _R8, [8], [(S, 0, None, None, -1), (U, 0)], [1, 8],
        [((0, 0), 8), ((0, 7), 1)], strides=[-8, -1]),
    _vc("unsqueeze_at_negative_stride_2d", "3217-3236", list(range(1, 13)), [3, 4], [(S, 0, None, None, -1), (U, 1)], [3, 1, 4],
        [((0, 0, 0), 9), ((0, 0, 3), 12), ((2, 0, 0), 1)], strides=[-4, 4, 1]),
    _vc("squeeze_basic_2d", "3501-3513", [1, 2, 3], [1, 3], [(Q, None)], [3], [((0,), 1), ((1,), 2), ((2,), 3)], strides=[1]),
    _vc("squeeze_basic_3d", "3516-3527", _M23, [1, 2, 1, 3], [(Q, None)], [2, 3], [((0, 0), 1), ((0, 2), 3), ((1, 0), 4), ((1, 2), 6)],
        strides=[3, 1]),
    _vc("squeeze_all_dimensions", "3530-3538", [42], [1, 1, 1], [(Q, None)], [], [((), 42)], strides=[]),
    _vc("squeeze_no_size_one_dims", "3541-3550", _M23, [2, 3], [(Q, None)], [2, 3], [((0, 0), 1), ((1, 2), 6)], strides=[3, 1]),
    _vc("squeeze_at_specific_dim", "3553-3562", _M23, [1, 2, 3], [(Q, 0)], [2, 3], [((0, 0), 1), ((1, 2), 6)], strides=[3, 1]),
    _vc("squeeze_at_middle_dim", "3565-3574", _M23, [2, 1, 3], [(Q, 1)], [2, 3], [((0, 0), 1), ((1, 2), 6)], strides=[3, 1]),
    _vc("squeeze_at_end_dim", "3577-3586", _M23, [2, 3, 1], [(Q, 2)], [2, 3], [((0, 0), 1), ((1, 2), 6)], strides=[3, 1]),
    _vc("squeeze_after_slice", "3589-3603", _M23, [2, 3], [(I, 0, 0), (U, 0), (Q, None)], [3], [((0,), 1), ((2,), 3)]),
    _vc("squeeze_after_column_slice", "3606-3624", _M23, [2, 3], [(I, 1, 1), (U, 1), (Q, None)], [2], [((0,), 2), ((1,), 5)]),
]


# core/mod.rs: view_as (relabel a contiguous view, offset kept) and shape_to_stride.
# View op ("view_as", shape); kind "strides_of": row-major strides of a shape.
V = "view_as"
CASES += [
    _vc("view_as_owned_success", "927-943", _M23, [2, 3], [(V, [3, 2])], [3, 2],
        [((0, 0), 1), ((0, 1), 2), ((1, 0), 3), ((1, 1), 4), ((2, 0), 5), ((2, 1), 6)], strides=[2, 1]),
    dict(name="view_as_owned_error", cite="core/mod.rs:945-951", kind="view_as_error", a_shape=[2, 3], new_shape=[4, 2]),
    _vc("view_as_slice_success", "954-973", _M23, [2, 3], [(I, 0, 1), (V, [1, 3])], [1, 3], [((0, 0), 4), ((0, 1), 5), ((0, 2), 6)],
        strides=[3, 1]),
    _vc("view_as_mut_view_modify", "975-988", [1, 2, 40, 4], [2, 2], [(V, [4])], [4], [((2,), 40)], strides=[1]),
    _vc("view_as_scalar_1", "990-1000", [99], [], [(V, [1])], [1], [((0,), 99)], strides=[1]),
    _vc("view_as_scalar_2", "1002-1003", [99], [], [(V, [1]), (V, [1, 1, 1])], [1, 1, 1], [((0, 0, 0), 99)]),
    dict(name="shape_to_stride", cite="core/mod.rs:1023-1028", kind="strides_of", shape=[2, 2, 3], strides=[6, 3, 1]),
    dict(name="shape_to_stride_single_dim", cite="core/mod.rs:1031-1036", kind="strides_of", shape=[4], strides=[1]),
    dict(name="shape_to_stride_empty", cite="core/mod.rs:1039-1044", kind="strides_of", shape=[], strides=[]),
    dict(name="shape_to_stride_ones", cite="core/mod.rs:1047-1052", kind="strides_of", shape=[1, 1, 1], strides=[1, 1, 1]),
    dict(name="shape_to_stride_mixed", cite="core/mod.rs:1055-1060", kind="strides_of", shape=[5, 1, 2], strides=[2, 2, 1]),
    dict(name="shape_to_stride_larger", cite="core/mod.rs:1063-1068", kind="strides_of", shape=[3, 4, 5], strides=[20, 5, 1]),
]


# core/mod.rs: index slices (`slice(dim, i..i)` removes the dim) of matrices and cubes.
_CUBE = [1, 2, 4, 5, 6, 7, 8, 9]
CASES += [
    _vc("slice_matrix_row", "26-41", _M23, [2, 3], [(I, 0, 0)], [3], [((0,), 1), ((1,), 2), ((2,), 3)], strides=[1]),
    _vc("slice_matrix_column", "43-49", _M23, [2, 3], [(I, 1, 0)], [2], [((0,), 1), ((1,), 4)], strides=[3]),
    _vc("slice_cube_depth0", "52-64", _CUBE, [2, 2, 2], [(I, 0, 0)], [2, 2], [((0, 0), 1), ((0, 1), 2), ((1, 0), 4), ((1, 1), 5)],
        strides=[2, 1]),
    _vc("slice_cube_depth1", "66-74", _CUBE, [2, 2, 2], [(I, 0, 1)], [2, 2], [((0, 0), 6), ((0, 1), 7), ((1, 0), 8), ((1, 1), 9)],
        strides=[2, 1]),
    _vc("slice_cube_row", "76-84", _CUBE, [2, 2, 2], [(I, 1, 0)], [2, 2], [((0, 0), 1), ((0, 1), 2), ((1, 0), 6), ((1, 1), 7)],
        strides=[4, 1]),
    _vc("slice_cube_column", "86-94", _CUBE, [2, 2, 2], [(I, 2, 0)], [2, 2], [((0, 0), 1), ((0, 1), 4), ((1, 0), 6), ((1, 1), 8)],
        strides=[4, 2]),
    _vc("slice_of_slice_1", "96-106", _M23, [2, 3], [(I, 0, 1)], [3], [((0,), 4), ((1,), 5), ((2,), 6)]),
    _vc("slice_of_slice_2", "108-111", _M23, [2, 3], [(I, 0, 1), (I, 0, 2)], [], [((), 6)]),
]


# core/mod.rs: offsets, sizes and contiguity of views.  kind "meta_check": offset / size / contiguous
# of the view (keys present are checked); "a_meta" builds a MetaTensor directly from (shape, strides).
CASES += [
    dict(name="meta_size_scalar", cite="core/mod.rs:1370-1373", kind="meta_check", a=dict(buf=[42], shape=[]), size=1),
    dict(name="meta_size_vector", cite="core/mod.rs:1375-1376", kind="meta_check", a=dict(buf=[1, 2, 3, 4], shape=[4]), size=4),
    dict(name="meta_size_matrix", cite="core/mod.rs:1378-1379", kind="meta_check", a=dict(buf=_M23, shape=[2, 3]), size=6),
    dict(name="meta_offsets_on_slices_1", cite="core/mod.rs:1382-1388", kind="meta_check",
         a=dict(buf=[1, 2, 3, 4], shape=[2, 2], view=[(I, 0, 1)]), offset=2),
    dict(name="meta_offsets_on_slices_2", cite="core/mod.rs:1390-1394", kind="meta_check",
         a=dict(buf=list(range(1, 9)), shape=[2, 2, 2], view=[(I, 0, 1)]), offset=4),
    dict(name="meta_offsets_on_slices_3", cite="core/mod.rs:1396-1397", kind="meta_check",
         a=dict(buf=list(range(1, 9)), shape=[2, 2, 2], view=[(I, 0, 1), (I, 1, 1)]), offset=5),
    dict(name="is_contiguous_owned", cite="core/mod.rs:1401-1404", kind="meta_check", a=dict(buf=_M23, shape=[2, 3]), contiguous=True),
    dict(name="is_contiguous_row_slice", cite="core/mod.rs:1406-1408", kind="meta_check",
         a=dict(buf=_M23, shape=[2, 3], view=[(I, 0, 1)]), contiguous=True),
    dict(name="is_contiguous_column_slice", cite="core/mod.rs:1410-1412", kind="meta_check",
         a=dict(buf=_M23, shape=[2, 3], view=[(I, 1, 0)]), contiguous=False),
    dict(name="tensor_meta_direct_contiguous", cite="core/mod.rs:1437-1454", kind="meta_check", a_meta=([2, 3], [3, 1], 0), size=6,
         offset=0, contiguous=True),
    dict(name="tensor_meta_direct_noncontiguous", cite="core/mod.rs:1456-1460", kind="meta_check", a_meta=([2], [3], 0), size=2,
         contiguous=False),
]


# core/mod.rs: writes through custom-step slices, read back through the base tensor
def _vs(name, cite, buf, shape, view, vshape, sets, base_spots):
    return dict(name=name, cite=f"core/mod.rs:{cite}", kind="view_set", dtype="i32", a=dict(buf=buf, shape=shape), view=view,
                shape=vshape, sets=sets, base_spots=base_spots)


CASES += [
    _vs("custom_positive_step_mut", "692-716", _R16, [16], [(S, 0, None, None, 2)], [8], [((0,), 100), ((1,), 102), ((7,), 114)],
        [((0,), 100), ((1,), 1), ((2,), 102), ((3,), 3), ((14,), 114), ((15,), 15)]),
    _vs("custom_positive_step_mut_with_range", "719-741", _R16, [16], [(S, 0, 1, 10, 3)], [3], [((0,), 101), ((1,), 104), ((2,), 107)],
        [((0,), 0), ((1,), 101), ((4,), 104), ((7,), 107), ((8,), 8)]),
    _vs("custom_negative_step_mut", "744-766", _R16, [16], [(S, 0, None, None, -2)], [8], [((0,), 115), ((1,), 113), ((7,), 101)],
        [((1,), 101), ((2,), 2), ((13,), 113), ((14,), 14), ((15,), 115)]),
    _vs("custom_negative_step_mut_with_range", "769-791", _R16, [16], [(S, 0, 12, 3, -3)], [3], [((0,), 212), ((1,), 209), ((2,), 206)],
        [((6,), 206), ((7,), 7), ((9,), 209), ((10,), 10), ((12,), 212)]),
]


# core/mod.rs: the range syntaxes (written out as the Slice each converts to), read and written through
_T8 = [10, 20, 30, 40, 50, 60, 70, 80]
_T10 = _T8 + [90, 100]


def _rw(name, cite, buf, shape, view, vshape, reads, sets, base_spots):
    return [_vc(name + "_read", cite, buf, shape, view, vshape, reads),
            _vs(name + "_write", cite, buf, shape, view, vshape, sets, base_spots)]


CASES += _rw("range_to_syntax", "1585-1614", _T8, [8], [(S, 0, None, 5, 1)], [5], [((k,), 10 * (k + 1)) for k in range(5)],
             [((0,), 11), ((2,), 33), ((4,), 55)], [((0,), 11), ((2,), 33), ((4,), 55), ((5,), 60)])
CASES += _rw("range_from_syntax", "1617-1643", _T8, [8], [(S, 0, 2, None, 1)], [6], [((0,), 30), ((1,), 40), ((5,), 80)],
             [((0,), 333), ((5,), 888)], [((2,), 333), ((7,), 888), ((0,), 10), ((1,), 20)])
CASES += _rw("range_full_syntax", "1646-1671", [10, 20, 30, 40], [4], [(S, 0, None, None, 1)], [4],
             [((0,), 10), ((1,), 20), ((2,), 30), ((3,), 40)], [((0,), 100), ((3,), 400)], [((0,), 100), ((3,), 400)])
CASES += _rw("inclusive_range_syntax", "1674-1701", _T8, [8], [(S, 0, 2, 6, 1)], [4], [((0,), 30), ((1,), 40), ((2,), 50), ((3,), 60)],
             [((0,), 333), ((3,), 666)], [((2,), 333), ((5,), 666), ((1,), 20), ((6,), 70)])
CASES += _rw("inclusive_range_zero_end", "1704-1726", [10, 20, 30, 40, 50], [5], [(S, 0, 0, 3, 1)], [3],
             [((0,), 10), ((1,), 20), ((2,), 30)], [((1,), 222)], [((1,), 222)])
CASES += _rw("single_index_syntax", "1729-1754", [10, 20, 30, 40, 50, 60], [2, 3], [(I, 1, 1)], [2], [((0,), 20), ((1,), 50)],
             [((0,), 222), ((1,), 555)], [((0, 1), 222), ((1, 1), 555), ((0, 0), 10), ((0, 2), 30)])
CASES += _rw("reverse_range_exclusive_with_values", "1757-1783", _T8, [8], [(S, 0, 5, 2, -1)], [3],
             [((0,), 60), ((1,), 50), ((2,), 40)], [((0,), 666), ((2,), 444)], [((5,), 666), ((3,), 444), ((2,), 30), ((6,), 70)])
CASES += _rw("slice_from_with_step", "1786-1811", _T10, [10], [(S, 0, 8, None, -1)], [9], [((0,), 90), ((1,), 80), ((8,), 10)],
             [((0,), 999), ((8,), 111)], [((8,), 999), ((0,), 111), ((9,), 100)])
CASES += _rw("slice_to_with_step", "1814-1841", _T8, [8], [(S, 0, None, 5, -1)], [2], [((0,), 80), ((1,), 70)],
             [((0,), 888), ((1,), 777)], [((7,), 888), ((6,), 777), ((5,), 60), ((4,), 50)])
CASES += _rw("reverse_first_n_elements", "1844-1871", _T8, [8], [(S, 0, 4, None, -1)], [5],
             [((0,), 50), ((1,), 40), ((2,), 30), ((3,), 20), ((4,), 10)], [((0,), 555), ((4,), 111)], [((4,), 555), ((0,), 111)])
CASES += _rw("manual_slice_construction_values", "1874-1899", _T10, [10], [(S, 0, 8, 2, -2)], [3],
             [((0,), 90), ((1,), 70), ((2,), 50)], [((0,), 999), ((2,), 555)], [((8,), 999), ((4,), 555), ((6,), 70)])
CASES += [_vc("empty_slice_same_indices", "1902-1911", [10, 20, 30, 40, 50, 60], [6], [(S, 0, 5, 5, 1)], [], [])]
CASES += _rw("matrix_column_slice_with_mutation", "1914-1943", list(range(1, 13)), [3, 4], [(S, 1, 2, 3, 1)], [3, 1],
             [((0, 0), 3), ((1, 0), 7), ((2, 0), 11)], [((0, 0), 33), ((2, 0), 111)], [((0, 2), 33), ((2, 2), 111), ((1, 2), 7)])


# backend/cuda_tests.rs repeats the slicing / fill tests of core/mod.rs on the CUDA backend with the
# same tensors; the two it adds: a float fill, and a 10-million-element upload read at both ends.
CASES += [
    dict(name="cuda_fill_f32", cite="backend/cuda_tests.rs:602-614", kind="fill", dtype="f32",
         a=dict(buf=[0., 1., 2., 3., 4., 5.], shape=[2, 3]), value=3.14, buf=[3.14] * 6),
    dict(name="rediculously_large_cuda_tensor", cite="backend/cuda_tests.rs:363-370", kind="owned", dtype="u8",
         a=dict(ones=[10_000_000]), shape=[10_000_000], ends=(1, 1)),
]


# core/mod.rs: more unsqueeze / unsqueeze_at (writes through, indexing, 1-D / 3-D / sequential)
_T12 = [10 * k for k in range(1, 13)]
_R24 = list(range(1, 25))
CASES += [
    _vc("unsqueeze_mut_basic", "2620-2638", [1, 2, 3, 4], [2, 2], [(U, 0)], [1, 2, 2], [((0, 0, 0), 1), ((0, 1, 1), 4)], strides=[4, 2, 1]),
    _vs("unsqueeze_mut_with_write", "2641-2665", _M23, [2, 3], [(U, 0)], [1, 2, 3], [((0, 0, 0), 100), ((0, 1, 2), 600)],
        [((0, 0), 100), ((1, 2), 600), ((0, 1), 2), ((1, 0), 4)]),
    _vs("unsqueeze_mut_after_slice", "2668-2694", _R8, [2, 4], [(I, 0, 1), (U, 0)], [1, 4], [((0, 0), 500), ((0, 3), 800)],
        [((1, 0), 500), ((1, 3), 800), ((0, 0), 1), ((0, 3), 4)]),
    _vs("unsqueeze_scalar_mut", "2697-2717", [99], [], [(U, 0)], [1], [((0,), 77)], [((), 77)]),
    _vc("unsqueeze_indexing_comprehensive", "2720-2756", _T12, [3, 4], [(U, 0)], [1, 3, 4],
        [((0, r, c), _T12[4 * r + c]) for r in range(3) for c in range(4)], strides=[12, 4, 1]),
    _vc("unsqueeze_3d_indexing", "2759-2791", _R24, [2, 3, 4], [(U, 0)], [1, 2, 3, 4],
        [((0, 0, 0, 0), 1), ((0, 0, 0, 3), 4), ((0, 0, 2, 3), 12), ((0, 1, 0, 0), 13), ((0, 1, 2, 3), 24)], strides=[24, 12, 4, 1]),
    _vc("unsqueeze_at_1d_tensor_front", "2848-2853", [1, 2, 3, 4], [4], [(U, 0)], [1, 4], [], strides=[4, 1]),
    _vc("unsqueeze_at_1d_tensor_back", "2855-2861", [1, 2, 3, 4], [4], [(U, 1)], [4, 1], [], strides=[1, 1]),
    _vc("unsqueeze_at_3d_tensor_0", "2864-2873", _R24, [2, 3, 4], [(U, 0)], [1, 2, 3, 4], [], strides=[24, 12, 4, 1]),
    _vc("unsqueeze_at_3d_tensor_1", "2875-2878", _R24, [2, 3, 4], [(U, 1)], [2, 1, 3, 4], [], strides=[12, 12, 4, 1]),
    _vc("unsqueeze_at_3d_tensor_2", "2880-2883", _R24, [2, 3, 4], [(U, 2)], [2, 3, 1, 4], [], strides=[12, 4, 4, 1]),
    _vc("unsqueeze_at_3d_tensor_3", "2885-2890", _R24, [2, 3, 4], [(U, 3)], [2, 3, 4, 1], [], strides=[12, 4, 1, 1]),
    _vc("unsqueeze_at_multiple_sequential", "2893-2912", [1, 2, 3, 4], [2, 2], [(U, 0), (U, 1), (U, 2)], [1, 1, 1, 2, 2],
        [((0, 0, 0, 0, 0), 1), ((0, 0, 0, 1, 1), 4)]),
    _vc("unsqueeze_at_multiple_different_positions", "2915-2940", _M23, [2, 3], [(U, 2), (U, 0), (U, 2)], [1, 2, 1, 3, 1],
        [((0, 0, 0, 0, 0), 1), ((0, 0, 0, 2, 0), 3), ((0, 1, 0, 0, 0), 4), ((0, 1, 0, 2, 0), 6)]),
]


# core/mod.rs: more squeeze cases (after 3-D slices, writes through, chained with slices, over a
# negative stride, several size-1 dims)
CASES += [
    _vc("squeeze_after_3d_slice", "3628-3648", _R24, [2, 3, 4], [(I, 0, 1), (U, 0), (Q, None)], [3, 4], [((0, 0), 13), ((2, 3), 24)]),
    _vs("squeeze_mut_basic", "3651-3664", [1, 2, 3], [1, 3], [(Q, None)], [3], [((1,), 20)], [((0, 1), 20)]),
    _vs("squeeze_mut_after_modifications", "3667-3687", _M23, [1, 2, 3], [(Q, None)], [2, 3],
        [((0, 0), 10), ((0, 2), 30), ((1, 1), 50)], [((0, 0, 0), 10), ((0, 0, 2), 30), ((0, 1, 1), 50), ((0, 0, 1), 2), ((0, 1, 0), 4)]),
    _vs("squeeze_at_mut_basic", "3690-3703", _M23, [2, 1, 3], [(Q, 1)], [2, 3], [((0, 0), 10), ((1, 2), 60)],
        [((0, 0, 0), 10), ((1, 0, 2), 60)]),
    _vs("squeeze_mut_after_slice", "3706-3731", list(range(1, 13)), [3, 4], [(I, 0, 1), (U, 0), (Q, None)], [4],
        [((0,), 50), ((3,), 80)], [((1, 0), 50), ((1, 3), 80)]),
    _vs("squeeze_mut_after_column_slice", "3734-3763", list(range(1, 10)), [3, 3], [(I, 1, 1), (U, 1), (Q, None)], [3],
        [((0,), 20), ((2,), 80)], [((0, 1), 20), ((1, 1), 5), ((2, 1), 80)]),
    _vc("squeeze_chained_with_slices", "3766-3795", _R24, [2, 3, 4], [(I, 0, 0), (U, 1), (I, 2, 2), (U, 0), (Q, None)], [3],
        [((0,), 3), ((1,), 7), ((2,), 11)]),
    _vc("squeeze_preserves_data_after_negative_stride", "3798-3814", _M23, [6], [(S, 0, None, None, -1), (U, 0), (Q, None)], [6],
        [((0,), 6), ((5,), 1)]),
    _vc("squeeze_multiple_dims_2d", "3817-3828", _M23, [1, 6, 1], [(Q, None)], [6], [((k,), k + 1) for k in range(6)], strides=[1]),
]
