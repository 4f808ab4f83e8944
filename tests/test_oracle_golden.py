"""The CPU oracle against the reference's own golden vectors (no GPU needed).

This is the pin of the oracle: every function of tests/verify_tensor.py carries
literal expected values transcribed from src/cortex/verify/tensor.clj.
"""
import pytest

import verify_tensor as vt


@pytest.mark.parametrize("fn,datatype", vt.case_params(), ids=vt.case_id)
def test_oracle_matches_reference_literals(oracle_driver, fn, datatype):
    fn(oracle_driver, datatype)
