"""The allocation-free convolution entry point (cb200_convolution_forward_static).

It exists for embedders that must not call cudaMalloc on the inference path (their own pool owns
the device memory, or an allocation's implicit device-wide synchronisation is unacceptable there):
the unrolled input lives in a fixed 64 MiB device array inside the library instead of a scratch
buffer grown on demand.  Checked here, through the C ABI: calls in a row give the same result
as the allocating entry point AND as the CPU oracle within the fp32 / fp64 parity bounds, the
array's previous contents do not leak into the next (differently shaped) call, a filter whose
row length is not a multiple of 4 takes the per-image kernel, and oversized problems are refused.
This file sorts last on purpose: a `pytest -x` run has then already run every other test.
"""
import ctypes as C

import numpy as np
import pytest

from cortex_b200 import _lib
from cortex_b200 import tensor as ct
from cortex_b200.tensor_math import conv_desc_struct, wire

pytestmark = pytest.mark.gpu
TOL = {"float": 1e-4, "double": 1e-12}
NP = {"float": np.float32, "double": np.float64}


def _rel_err(got, ref):
    got, ref = np.asarray(got, np.float64), np.asarray(ref, np.float64)
    rms = float(np.sqrt(np.mean(ref ** 2))) or 1.0
    return float(np.max(np.abs(got - ref) / np.maximum(np.abs(ref), rms)))


def _oracle_conv(oracle_driver, datatype, x, w, desc_args, out_shape):
    """The same call on the CPU oracle (per-image im2col + gemm, as the reference's CPU backend)."""
    stream = oracle_driver.default_device().create_stream()
    with ct.with_stream(stream), ct.with_datatype(datatype):
        desc = ct.convolution_descriptor(datatype, *desc_args)
        out = ct.new_tensor(out_shape, datatype)
        ct.assign(out, 3.0)
        ct.convolution_forward(out, 0.5, ct.to_tensor(x, datatype), ct.to_tensor(w, datatype), None, desc, None)
        res = ct.to_array(out)
    stream.sync()
    return res


def _conv_both_ways(stream, datatype, batch, cin, hw, cout, k, pad, stride, seed, oracle_driver=None):
    rng = np.random.default_rng(seed)
    x = rng.standard_normal((batch, cin, hw, hw)).astype(NP[datatype])
    w = (rng.standard_normal((cout, cin * k * k)) * np.sqrt(2.0 / (cin * k * k))).astype(NP[datatype])
    out_hw = (hw + 2 * pad - k) // stride + 1
    if oracle_driver is not None:
        oracle = _oracle_conv(oracle_driver, datatype, x, w, (cout, cin, k, k, pad, pad, stride, stride),
                              [batch, cout, out_hw, out_hw])
    desc = ct.convolution_descriptor(datatype, cout, cin, k, k, pad, pad, stride, stride)
    xt, wt = ct.to_tensor(x, datatype), ct.to_tensor(w, datatype)
    ref = ct.new_tensor([batch, cout, out_hw, out_hw], datatype)
    ct.assign(ref, 3.0)
    got = ct.new_tensor([batch, cout, out_hw, out_hw], datatype)
    ct.assign(got, 3.0)
    # existing entry point (allocating scratch), out = conv + 0.5 * out
    ct.convolution_forward(ref, 0.5, xt, wt, None, desc, None)
    # new entry point, straight through the C ABI
    _lib.call("cb200_convolution_forward_static", stream.handle, _lib.DTYPE_CODE[datatype], got.buffer.ptr,
              C.byref(wire(got.dimensions)), 0.5, xt.buffer.ptr, C.byref(wire(xt.dimensions)), wt.buffer.ptr,
              C.byref(wire(wt.dimensions)), C.byref(conv_desc_struct(desc)))
    if oracle_driver is not None:
        assert _rel_err(ct.to_array(got), oracle) <= TOL[datatype]
    return ct.to_array(got), ct.to_array(ref)


@pytest.mark.parametrize("datatype", ["float", "double"])
def test_static_scratch_conv_matches_allocating_conv_twice(b200_driver, oracle_driver, datatype):
    stream = b200_driver.default_device().create_stream()
    with ct.with_stream(stream), ct.with_datatype(datatype):
        # first call: fills a large part of the array
        got, ref = _conv_both_ways(stream, datatype, 16, 32, 28, 24, 3, 1, 1, seed=11)
        assert _rel_err(got, ref) <= TOL[datatype]
        # second call, right after, smaller and differently shaped: stale contents must not matter
        got, ref = _conv_both_ways(stream, datatype, 2, 4, 9, 5, 3, 0, 2, seed=12, oracle_driver=oracle_driver)
        assert _rel_err(got, ref) <= TOL[datatype]
        # third: 3 input channels, 3x3 filter -> rows of 27 weights, not a multiple of 4: for fp32 the
        # unrolled matrix is multiplied image by image on the plain-FMA kernel instead of the tensor cores
        got, ref = _conv_both_ways(stream, datatype, 3, 3, 12, 7, 3, 1, 1, seed=13, oracle_driver=oracle_driver)
        assert _rel_err(got, ref) <= TOL[datatype]
    stream.sync()


def test_static_scratch_conv_rejects_oversized_problem(b200_driver):
    stream = b200_driver.default_device().create_stream()
    with ct.with_stream(stream), ct.with_datatype("float"):
        # 64 x 64 x 56 x 56 with a 3x3 kernel unrolls to 462 MB > 64 MiB
        desc = ct.convolution_descriptor("float", 64, 64, 3, 3, 1, 1, 1, 1)
        x = ct.new_tensor([64, 64, 56, 56], "float")
        w = ct.new_tensor([64, 576], "float")
        out = ct.new_tensor([64, 64, 56, 56], "float")
        with pytest.raises(_lib.B200Error) as err:
            _lib.call("cb200_convolution_forward_static", stream.handle, _lib.DTYPE_CODE["float"], out.buffer.ptr,
                      C.byref(wire(out.dimensions)), 0.0, x.buffer.ptr, C.byref(wire(x.dimensions)), w.buffer.ptr,
                      C.byref(wire(w.dimensions)), C.byref(conv_desc_struct(desc)))
        assert err.value.code == 1 and "static scratch" in str(err.value)
    stream.sync()
