"""Pins the CPU oracle: every known-answer case transcribed from the reference's own tests must
reproduce, on both oracle builds (-O2 parity build and -O3 timed-baseline build)."""
import numpy as np
import pytest

from golden.reference_cases import CASES
from golden_runner import OracleEngine, run_case


@pytest.mark.parametrize("fast", [False, True], ids=["O2", "O3"])
@pytest.mark.parametrize("case", CASES, ids=[c["name"] for c in CASES])
def test_reference_case(case, fast):
    run_case(case, OracleEngine(fast=fast))


def test_builds_agree_bitwise():
    import oracle as O
    rng = np.random.default_rng(7)
    x = rng.standard_normal(100003).astype(np.float32)
    for op in (O.SUM, O.MAX, O.MIN, O.MEAN):
        a = O.reduce_flat(x, 0, x.size, op, fast=False)
        b = O.reduce_flat(x, 0, x.size, op, fast=True)
        assert a.tobytes() == b.tobytes()
    y = x.copy(); z = x.copy()
    m = O.Meta.contiguous((x.size,))
    for op, v in ((O.MUL, 3.0), (O.ADD, 2.0), (O.SUB, 1.0), (O.DIV, 7.0)):
        O.scalar_op(y, op, v, m, fast=False)
        O.scalar_op(z, op, v, m, fast=True)
    assert y.tobytes() == z.tobytes()
    # the elementwise chain is the IEEE single-op sequence numpy computes too
    ref = ((x * np.float32(3.0) + np.float32(2.0)) - np.float32(1.0)) / np.float32(7.0)
    assert ref.tobytes() == y.tobytes()
