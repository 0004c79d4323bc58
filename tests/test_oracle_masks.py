"""The oracle's relu / abs gradient maps (ops/unary/mod.rs:213-252) on hand-checked values: the map
is 1 where the input is > 0, else 0 (relu) or -1 (abs) -- zero and NaN fall on the `else` side."""
import numpy as np
import pytest

import oracle as O


@pytest.mark.parametrize("fast", [False, True])
def test_maps_on_a_small_matrix_and_its_views(fast):
    b = np.array([-1.0, 0.0, 2.0, 3.0, -0.5, np.nan], np.float32)
    m = O.Meta.contiguous((2, 3))
    assert O.grad_mask(b, O.MASK_RELU, m, fast=fast).tolist() == [0, 0, 1, 1, 0, 0]
    assert O.grad_mask(b, O.MASK_ABS, m, fast=fast).tolist() == [-1, -1, 1, 1, -1, -1]
    assert O.grad_mask(b, O.MASK_RELU, m.permute((1, 0)), fast=fast).tolist() == [0, 1, 0, 0, 1, 0]
    assert O.grad_mask(b, O.MASK_ABS, m.slice(1, None, None, -1), fast=fast).tolist() == [1, -1, -1, -1, -1, 1]
    assert O.grad_mask(b, O.MASK_LEAKY_RELU, m, 0.125, fast=fast).tolist() == [0.125, 0.125, 1, 1, 0.125, 0.125]
    r = O.grad_mask(b, O.MASK_RECIPROCAL, m, fast=fast)
    assert r[:5].tolist() == [-1.0, np.inf, 0.5, np.float32(1) / np.float32(3), -2.0] and np.isnan(r[5])


def test_integer_types_and_refusals():
    i = np.array([-3, 0, 7], np.int16)
    m = O.Meta.contiguous((3,))
    assert O.grad_mask(i, O.MASK_RELU, m).tolist() == [0, 0, 1]
    assert O.grad_mask(i, O.MASK_ABS, m).tolist() == [-1, -1, 1]
    assert O.grad_mask(i, O.MASK_LEAKY_RELU, m, 9).tolist() == [9, 9, 1]
    assert O.grad_mask(i, O.MASK_RECIPROCAL, m).tolist() == [0, 0, 0]   # 1 / -3 truncates to 0; 1 / 0 -> 0 by convention
    assert O.grad_mask(np.array([1, -1, 2], np.int16), O.MASK_RECIPROCAL, m).tolist() == [1, -1, 0]
    with pytest.raises(O.OracleError):
        O.grad_mask(np.array([1, 0], np.bool_), O.MASK_RECIPROCAL, O.Meta.contiguous((2,)))
    u = np.array([0, 5], np.uint8)
    assert O.grad_mask(u, O.MASK_RELU, O.Meta.contiguous((2,))).tolist() == [0, 1]
    with pytest.raises(O.OracleError):
        O.grad_mask(u, O.MASK_ABS, O.Meta.contiguous((2,)))
    assert O.grad_mask(np.zeros(1, np.float32), O.MASK_RELU, O.Meta.contiguous((0, 4))).size == 0
