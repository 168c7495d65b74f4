"""The oracle must reproduce every golden vector of the reference's own unit tests."""
import pytest

import golden_cases as gc

CASES = gc.load("reference_goldens.json")


@pytest.mark.parametrize("case", CASES, ids=[gc.case_id(c) for c in CASES])
def test_oracle_matches_reference_golden(oracle, case):
    gc.run_case(oracle, case, oracle.OracleError)
