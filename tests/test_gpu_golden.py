"""The CUDA back end, called through the C ABI with host buffers, must reproduce every golden
vector of the reference's own unit tests (the same driver that pins the oracle)."""
import pytest

import golden_cases as gc

pytestmark = pytest.mark.gpu
CASES = gc.load("reference_goldens.json")


@pytest.mark.parametrize("case", CASES, ids=[gc.case_id(c) for c in CASES])
def test_cuda_matches_reference_golden(zb, ctx, case):
    gc.run_case(ctx, case, zb.ZantError)
