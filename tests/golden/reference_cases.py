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


def _ext(name, op, truth, c2, c3, c16, lines):
    out = []
    for layout, d, ln in (("contiguous", c2, lines[0]), ("1d", c3, lines[1]), ("nd", c16, lines[2])):
        out.append(dict(name=f"unary_{name}_{layout}", cite=f"ops/unary/mod.rs:{ln}", kind="unary_fixture", dtype="f64",
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
