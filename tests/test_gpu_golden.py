"""Replays the reference's known-answer cases against the CUDA library through the C ABI."""
import pytest

from golden.reference_cases import CASES
from golden_runner import run_case

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("case", CASES, ids=[c["name"] for c in CASES])
def test_reference_case_cuda(case):
    from cuda_engine import CudaEngine
    run_case(case, CudaEngine())
