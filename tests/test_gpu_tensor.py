"""The B200 backend against the reference's golden vectors, through the C ABI."""
import pytest

import verify_tensor as vt

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("fn,datatype", vt.case_params(), ids=vt.case_id)
def test_b200_matches_reference_literals(b200_driver, fn, datatype):
    fn(b200_driver, datatype)
