"""The oracle on the seeded configuration-shaped cases against plain numpy fp64 math
(CPU only): guards the oracle beyond the reference's small literals."""
import numpy as np
import pytest

import parity_cases as pc
from cortex_b200 import tensor as ct


def _run(oracle_driver, datatype, fn):
    stream = oracle_driver.default_device().create_stream()
    with ct.with_stream(stream), ct.with_datatype(datatype):
        return fn()


@pytest.mark.parametrize("datatype", ["float", "double"])
@pytest.mark.parametrize("ta,tb", [(False, False), (False, True), (True, False), (True, True)])
def test_gemm_views(oracle_driver, datatype, ta, tb):
    for (m, n, k, pad, off) in [(5, 7, 9, 0, 0), (64, 48, 80, 12, 3), (130, 70, 96, 128, 64)]:
        run, ref = pc.gemm_case(datatype, m, n, k, ta, tb, 1.5, 0.5, pad, off)
        assert pc.rel_err(_run(oracle_driver, datatype, run), ref()) <= pc.TOL[datatype] * (10 if datatype == "float" else 1)


@pytest.mark.parametrize("datatype", ["float", "double"])
def test_eltwise_reduce_softmax(oracle_driver, datatype):
    rows, cols = 64, 96
    out = _run(oracle_driver, datatype, pc.eltwise_case(datatype, rows, cols))
    X = np.random.default_rng(301).standard_normal((rows, cols)).astype(pc.NP[datatype]).astype(np.float64)
    b = (np.random.default_rng(302).standard_normal((1, cols)) * 0.1).astype(pc.NP[datatype]).astype(np.float64)
    y = (X + b).astype(pc.NP[datatype]).astype(np.float64)
    tol = pc.TOL[datatype]
    assert np.array_equal(out["biased"].reshape(rows, cols), (X + b).astype(pc.NP[datatype]))
    assert np.array_equal(out["biased_inplace"], out["biased"])
    assert np.array_equal(out["relu"].reshape(rows, cols), np.maximum(y, 0).astype(pc.NP[datatype]))
    assert np.array_equal(out["rowmax"].reshape(-1), np.maximum(y, 0).max(axis=1).astype(pc.NP[datatype]))
    assert pc.rel_err(out["rowsum"].reshape(-1), np.maximum(y, 0).sum(axis=1)) <= tol
    e = np.exp(y - y.max(axis=1, keepdims=True))
    assert pc.rel_err(out["softmax"], e / e.sum(axis=1, keepdims=True)) <= tol
    assert pc.rel_err(out["softmax_decomposed"], e / e.sum(axis=1, keepdims=True)) <= tol


@pytest.mark.parametrize("datatype", ["int", "long", "float"])
def test_gather_bit_exact(oracle_driver, datatype):
    run, ref = pc.gather_case(datatype, 100, 57, 24)
    assert np.array_equal(_run(oracle_driver, datatype, run).reshape(57, 24), ref())


@pytest.mark.parametrize("datatype", ["float", "double"])
def test_mlp(oracle_driver, datatype):
    run, ref = pc.mlp_case(datatype, 16, [784, 500, 10], bias_scale=0.1)
    assert pc.rel_err(_run(oracle_driver, datatype, run), ref()) <= pc.TOL[datatype]


@pytest.mark.parametrize("datatype", ["float", "double"])
def test_conv(oracle_driver, datatype):
    run, ref = pc.conv_case(datatype, 2, 4, 9, 5, bias_scale=0.1)
    assert pc.rel_err(_run(oracle_driver, datatype, run), ref()) <= pc.TOL[datatype]
    run, ref = pc.conv_case(datatype, 2, 3, 8, 4, k=2, pad=0, stride=2, bias_scale=0.1)
    assert pc.rel_err(_run(oracle_driver, datatype, run), ref()) <= pc.TOL[datatype]


def test_philox_known_answers():
    """The generator behind rand! against the known-answer vectors published with the algorithm
    (Random123's Philox-4x32-10: zero counter and key, all-ones, and the digits-of-pi vector)."""
    import ctypes

    import numpy as np

    from oracle import cpu_backend
    lib = cpu_backend.load()
    vectors = [
        ([0, 0, 0, 0], [0, 0], [0x6627e8d5, 0xe169c58d, 0xbc57ac4c, 0x9b00dbd8]),
        ([0xffffffff] * 4, [0xffffffff] * 2, [0x408f276d, 0x41c83b0e, 0xa20bc7c6, 0x6d5451fd]),
        ([0x243f6a88, 0x85a308d3, 0x13198a2e, 0x03707344], [0xa4093822, 0x299f31d0],
         [0xd16cfe09, 0x94fdcceb, 0x5001e420, 0x24126ea1]),
    ]
    for ctr, key, want in vectors:
        c, k, out = np.asarray(ctr, np.uint32), np.asarray(key, np.uint32), np.zeros(4, np.uint32)
        lib.orc_philox4x32_10(c.ctypes.data_as(ctypes.c_void_p), k.ctypes.data_as(ctypes.c_void_p),
                              out.ctypes.data_as(ctypes.c_void_p))
        assert [int(v) for v in out] == want
