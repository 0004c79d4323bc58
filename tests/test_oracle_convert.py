"""The C oracle's dtype conversion against an exact-arithmetic model of the reference's rules
(Backend::convert, backend/cpu.rs:221-233; DTypeConversion, core/value.rs:270-290), and against the
one literal case the reference's tests carry (backend/remote/remote_tests.rs:816-825)."""
import numpy as np
import pytest

import oracle as O
from convert_cases import ALL_CODES, NAMES, decode, encode, model_convert, same, samples


@pytest.mark.parametrize("fast", [False, True], ids=["parity", "fast"])
@pytest.mark.parametrize("src", ALL_CODES, ids=lambda c: NAMES[c])
def test_oracle_convert_matches_exact_model(src, fast):
    rng = np.random.default_rng(1000 + src)
    vals = samples(src, rng)
    raw = encode(src, vals)
    vals = decode(src, raw)  # what the buffer really holds (f32 rounding of the edge list)
    for dst in ALL_CODES:
        got = decode(dst, O.convert(raw, src, dst, fast))
        want = model_convert(src, dst, vals)
        assert same(dst, got, want), (NAMES[src], NAMES[dst],
                                      [(v, g, w) for v, g, w in zip(vals, got, want) if not same(dst, [g], [w])][:5])


def test_reference_literal_case():
    raw = encode(O.F32, [1.7, -2.2, 3.0])
    assert decode(O.I64, O.convert(raw, O.F32, O.I64)) == [2, -2, 3]
    assert decode(O.BOOL, O.convert(raw, O.F32, O.BOOL)) == [True, True, True]


def test_empty_and_bad_dtype():
    assert O.convert(b"", O.F32, O.I8) == b""
    with pytest.raises(O.OracleError):
        O.convert(b"\0" * 4, O.F32, 13)
