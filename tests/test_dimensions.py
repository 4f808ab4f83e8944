"""Descriptor algebra of the host mirror against the reference's own cases
(test/clj/cortex/tensor_dimensions_test.clj:7-51, dimensions-in-place-reshape-test)."""
import pytest

from cortex_b200 import dimensions as ct_dims

CASES = [
    # (shape, strides) -> new shape -> expected {shape, strides}
    (([3, 2, 2], [4, 2, 1]), [6, 2], ([6, 2], [2, 1])),
    (([3, 2, 2], [4, 2, 1]), [3, 4], ([3, 4], [4, 1])),
    (([3, 2, 2], [5, 2, 1]), [3, 4], ([3, 4], [5, 1])),
    (([4, 5, 8], [50, 10, 1]), [20, 8], ([20, 8], [10, 1])),
    (([4, 5, 8], [50, 10, 1]), [20, 8, 1, 1], ([20, 8, 1, 1], [10, 1, 1, 1])),
    (([4, 5, 8], [50, 10, 1]), [1, 1, 20, 8], ([1, 1, 20, 8], [200, 200, 10, 1])),
    (([845], [1]), [169, 5], ([169, 5], [5, 1])),
    # dense dimensions: any reshape that preserves the element count is an arbitrary reinterpretation
    (([10, 1, 18, 2], [36, 36, 2, 1]), [10, 4, 9], ([10, 4, 9], [36, 9, 1])),
    (([13, 13, 5, 1], [1625, 125, 25, 1]), [845, 1], ([845, 1], [25, 1])),
    (([1], [1]), [1, 1], ([1, 1], [1, 1])),
]


@pytest.mark.parametrize("source,new_shape,expected", CASES, ids=lambda c: str(c))
def test_dimensions_in_place_reshape(source, new_shape, expected):
    shape, strides = source
    got = ct_dims.in_place_reshape(ct_dims.dimensions(shape, strides=strides), new_shape)
    assert list(got["shape"]) == expected[0] and list(got["strides"]) == expected[1]
