"""CPU oracle backend -- TEST INFRASTRUCTURE, not product code.

Plays the role the reference's own CPU backend plays in its test-suite
(src/cortex/compute/cpu/{driver,tensor_math}.clj): the same tensor API
(``cortex_b200.tensor``) runs against it, so every verification function is
instantiated once per backend, exactly as the reference instantiates
``cortex.verify.tensor`` for CPUStream and CudaStream.

Elementwise / reduce / softmax / small gemm / conv go through ``oracle.c``
(a restatement of the reference CPU arithmetic); large GEMMs go through
numpy's bundled OpenBLAS ``sgemm`` / ``dgemm``, which stands in for the
reference's netlib-java BLAS (com.github.fommil.netlib/all 1.1.2, not vendored).

Only tests/, the smoke check and bench.py's cpu_baseline / reference arms may
import this module.
"""
import ctypes as C
import os
import subprocess

import numpy as np

from cortex_b200._lib import DTYPE_CODE, DTYPE_SIZE, NUMPY_NAME, ConvDesc, Dims
from cortex_b200.driver import Buffer
from cortex_b200.tensor_math import CTensorMath

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "_build", "liboracle.so")
_lib = None

_vp, _i, _i64, _d = C.c_void_p, C.c_int, C.c_int64, C.c_double
_pd = C.POINTER(Dims)
_SIGS = {
    "orc_memset": [_i, _vp, _i64, _d, _i64],
    "orc_assign_constant": [_i, _vp, _pd, _d, _i64],
    "orc_assign": [_i, _vp, _pd, _i, _vp, _pd, _i64],
    "orc_unary_accum": [_i, _vp, _pd, _d, _i, _i64],
    "orc_unary_op": [_i, _vp, _pd, _vp, _pd, _d, _i, _i64],
    "orc_binary_accum_constant": [_i, _vp, _pd, _d, _d, _i64, _i, _i],
    "orc_binary_op_constant": [_i, _vp, _pd, _vp, _pd, _d, _d, _i64, _i, _i],
    "orc_binary_accum": [_i, _vp, _pd, _d, _vp, _pd, _d, _i64, _i, _i, _i],
    "orc_binary_op": [_i, _vp, _pd, _vp, _pd, _d, _vp, _pd, _d, _i64, _i],
    "orc_unary_reduce": [_i, _vp, _pd, _d, _vp, _pd, _i],
    "orc_gemm": [_i, _vp, _i64, _i, _i, _d, _vp, _i64, _i64, _i64, _vp, _i64, _i64, _d],
    "orc_batch_normalize": [_i, _vp, _vp, _vp, _vp, _vp, _vp, _d, _i64, _i64, _i64],
    "orc_pooling_forward": [_i, _vp, _vp] + [_i64] * 11 + [_i],
    "orc_pooling_backward": [_i, _vp, _vp, _vp, _vp] + [_i64] * 11 + [_i],
    "orc_lrn": [_i, _i, _vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _i64, _d, _d, _d],
    "orc_batch_normalize_update": [_i, _vp, _vp, _vp, _vp, _vp, _d, _i64, _i64, _i64],
    "orc_batch_normalize_gradients": [_i] + [_vp] * 8 + [_d, _i64, _i64, _i64],
    "orc_gemv": [_i, _vp, _i64, _i, _d, _vp, _i64, _i64, _i64, _vp, _i64, _d],
    "orc_ternary_op": [_i, _vp, _pd, _vp, _pd, _d, _vp, _pd, _d, _vp, _pd, _d, _i64, _i],
    "orc_activation_gradient": [_i, _vp, _pd, _vp, _pd, _vp, _pd, _i, _i64],
    "orc_softmax_eltwise": [_i, _vp, _pd, _vp, _pd],
    "orc_softmax_spatial": [_i, _vp, _pd, _vp, _pd],
    "orc_convolution_forward": [_i, _vp, _pd, _d, _vp, _pd, _vp, _pd, _vp, _i64, C.POINTER(ConvDesc)],
    "orc_convolution_backward_weights": [_i, _vp, _pd, _d, _vp, _pd, _vp, _pd, _vp, _i64, C.POINTER(ConvDesc)],
    "orc_convolution_backward_data": [_i, _vp, _pd, _d, _vp, _pd, _vp, _pd, _vp, _i64, C.POINTER(ConvDesc)],
    "orc_bias_relu_rowstats": [_i, _vp, _i64, _vp, _i64, _vp, _i64, _i64, _vp, _vp],
    "orc_adam_step": [_i, _d, _d, _d, _d, _d, _d, _d, _vp, _vp, _vp, _vp, _i64],
    "orc_adadelta_step": [_i, _d, _d, _vp, _vp, _d, _vp, _vp, _i64],
    "orc_rand": [_vp, _pd, _i, _d, _d, C.c_uint64, C.c_uint64],
    "orc_philox4x32_10": [_vp, _vp, _vp],
}


def build():
    subprocess.run(["make", "-C", _HERE], check=True, capture_output=True)
    return LIB_PATH


def load():
    global _lib
    if _lib is None:
        try:
            build()          # make: rebuilds only when oracle.c is newer than the library
        except Exception:
            if not os.path.exists(LIB_PATH):
                raise
        lib = C.CDLL(LIB_PATH)
        for name, argtypes in _SIGS.items():
            fn = getattr(lib, name)
            fn.argtypes, fn.restype = argtypes, _i
        _lib = lib
    return _lib


class OracleError(RuntimeError):
    pass


def _call(name, *args):
    rc = getattr(load(), "orc_" + name)(*args)
    if rc != 0:
        raise OracleError("oracle %s failed (unsupported dtype or shape)" % name)


class _MemBuffer(Buffer):
    """Host memory owned by a numpy array; used both as 'device' and as host buffer."""

    def __init__(self, n, dtype, device):
        arr = np.zeros(max(int(n), 1), dtype=NUMPY_NAME[dtype])
        super().__init__(arr.ctypes.data, dtype, n, device, host=True)
        self._array = arr

    def release(self):
        self._released = True


class OracleEvent:
    def wait_for_event(self):
        pass


class OracleStream(CTensorMath):
    """The oracle's CPUStream: every call runs synchronously on the caller's thread."""

    is_oracle = True

    # GEMMs above this many multiply-adds go to OpenBLAS instead of the C loop nest
    BLAS_THRESHOLD = 1 << 18

    def __init__(self, device):
        self.device = device

    def _tm(self, name, *args):
        return _call(name, *args)

    def _tm_nostream(self, name, *args):
        raise NotImplementedError

    def get_device(self):
        return self.device

    def get_driver(self):
        return self.device.driver

    @staticmethod
    def _move(dst_ptr, src_ptr, nbytes):
        C.memmove(dst_ptr, src_ptr, nbytes)

    def copy_host_to_device(self, host_buffer, host_offset, device_buffer, device_offset, elem_count):
        es = DTYPE_SIZE[device_buffer.dtype]
        self._move(device_buffer.ptr + device_offset * es, host_buffer.ptr + host_offset * es, elem_count * es)

    def copy_device_to_host(self, device_buffer, device_offset, host_buffer, host_offset, elem_count):
        es = DTYPE_SIZE[device_buffer.dtype]
        self._move(host_buffer.ptr + host_offset * es, device_buffer.ptr + device_offset * es, elem_count * es)

    def copy_device_to_device(self, src, src_offset, dst, dst_offset, elem_count):
        es = DTYPE_SIZE[src.dtype]
        self._move(dst.ptr + dst_offset * es, src.ptr + src_offset * es, elem_count * es)

    def memset(self, device_buffer, device_offset, elem_val, elem_count):
        _call("memset", DTYPE_CODE[device_buffer.dtype], device_buffer.ptr, int(device_offset), float(elem_val),
              int(elem_count))

    def create_event(self, timing=False):
        return OracleEvent()

    def sync_event(self, event):
        pass

    def sync(self):
        pass

    def batch_normalize_eltwise(self, output, input, means, variances, scale, bias, epsilon, batch_count, element_count):
        _call("batch_normalize", DTYPE_CODE[output.dtype], output.ptr, input.ptr, means.ptr, variances.ptr, scale.ptr,
              bias.ptr, float(epsilon), int(batch_count), int(element_count), 1)

    def batch_normalize_spatial(self, output, input, means, variances, scale, bias, epsilon, batch_count, channel_count,
                                element_count):
        _call("batch_normalize", DTYPE_CODE[output.dtype], output.ptr, input.ptr, means.ptr, variances.ptr, scale.ptr,
              bias.ptr, float(epsilon), int(batch_count), int(channel_count), int(element_count))

    def pooling_forward(self, output, output_dims, output_alpha, input, input_dims, pool_descriptor):
        from cortex_b200._lib import POOL_OPS
        batch, channels, in_h, in_w = input_dims["shape"]
        _b, _c, out_h, out_w = output_dims["shape"]
        d = pool_descriptor
        _call("pooling_forward", DTYPE_CODE[output.dtype], output.ptr, input.ptr, batch * channels, in_h, in_w, out_h,
              out_w, d["kernel-width"], d["kernel-height"], d["pad-x"], d["pad-y"], d["stride-x"], d["stride-y"],
              POOL_OPS[d["pool-op"]])

    def pooling_backward(self, input_grad, input_grad_dims, input_grad_alpha, input, input_dims, output, output_dims,
                         output_grad, output_grad_dims, pool_descriptor):
        """cpu/tensor_math.clj:1829-1866: input-grad-alpha is not read; the loops add onto input-grad."""
        from cortex_b200._lib import POOL_OPS
        batch, channels, in_h, in_w = input_dims["shape"]
        _b, _c, out_h, out_w = output_dims["shape"]
        d = pool_descriptor
        _call("pooling_backward", DTYPE_CODE[output.dtype], input_grad.ptr, input.ptr, output.ptr, output_grad.ptr,
              batch * channels, in_h, in_w, out_h, out_w, d["kernel-width"], d["kernel-height"], d["pad-x"], d["pad-y"],
              d["stride-x"], d["stride-y"], POOL_OPS[d["pool-op"]])

    # -- lrn: not in the reference's CPU backend; restated from the operation its CUDA backend calls ----
    def lrn_descriptor(self, n, k, alpha, beta):
        return {"n": int(n), "k": float(k), "alpha": float(alpha), "beta": float(beta)}

    @staticmethod
    def _lrn_extents(dims):
        shape = list(dims["shape"])
        batch = 1
        for v in shape[:-3]:
            batch *= v
        return batch, shape[-3], shape[-2] * shape[-1]

    def lrn_forward(self, output, output_dims, input, input_dims, d):
        _call("lrn", DTYPE_CODE[output.dtype], 0, output.ptr, None, None, input.ptr, None, *self._lrn_extents(input_dims),
              d["n"], d["k"], d["alpha"], d["beta"])

    def lrn_backward(self, input_gradient, input_grad_dims, output, output_dims, input, input_dims, output_gradient,
                     output_grad_dims, d):
        _call("lrn", DTYPE_CODE[output.dtype], 1, None, input_gradient.ptr, output.ptr, input.ptr, output_gradient.ptr,
              *self._lrn_extents(input_dims), d["n"], d["k"], d["alpha"], d["beta"])

    # -- batch-normalize training half (cpu/tensor_math.clj:1574-1640) ------------------------
    def batch_normalize_update_and_apply_eltwise(self, output, input, batch_means, batch_variances, running_means,
                                                 running_variances, average_factor, scale, bias, epsilon, batch_count,
                                                 element_count):
        self.batch_normalize_update_and_apply_spatial(output, input, batch_means, batch_variances, running_means,
                                                      running_variances, average_factor, scale, bias, epsilon,
                                                      batch_count, element_count, 1)

    def batch_normalize_update_and_apply_spatial(self, output, input, batch_means, batch_variances, running_means,
                                                 running_variances, average_factor, scale, bias, epsilon, batch_count,
                                                 channel_count, element_count):
        _call("batch_normalize_update", DTYPE_CODE[output.dtype], input.ptr, batch_means.ptr, batch_variances.ptr,
              running_means.ptr, running_variances.ptr, float(average_factor), int(batch_count), int(channel_count),
              int(element_count))
        _call("batch_normalize", DTYPE_CODE[output.dtype], output.ptr, input.ptr, batch_means.ptr, batch_variances.ptr,
              scale.ptr, bias.ptr, float(epsilon), int(batch_count), int(channel_count), int(element_count))

    def batch_normalize_gradients_eltwise(self, input_gradient, scale_gradient, bias_gradient, output_gradient, output,
                                          input, batch_means, batch_variances, scale, bias, epsilon, batch_count,
                                          element_count):
        self.batch_normalize_gradients_spatial(input_gradient, scale_gradient, bias_gradient, output_gradient, output,
                                               input, batch_means, batch_variances, scale, bias, epsilon, batch_count,
                                               element_count, 1)

    def batch_normalize_gradients_spatial(self, input_gradient, scale_gradient, bias_gradient, output_gradient, output,
                                          input, batch_means, batch_variances, scale, bias, epsilon, batch_count,
                                          channel_count, element_count):
        _call("batch_normalize_gradients", DTYPE_CODE[output.dtype], input_gradient.ptr, scale_gradient.ptr,
              bias_gradient.ptr, output_gradient.ptr, input.ptr, batch_means.ptr, batch_variances.ptr, scale.ptr,
              float(epsilon), int(batch_count), int(channel_count), int(element_count))

    # -- gemm: BLAS semantics (src/cortex/compute/cpu/tensor_math.clj:672-699) ---------------
    @staticmethod
    def _matrix(buf, rows, cols, ld):
        raw = (C.c_char * (((rows - 1) * ld + cols) * DTYPE_SIZE[buf.dtype])).from_address(buf.ptr)
        flat = np.frombuffer(raw, dtype=NUMPY_NAME[buf.dtype])
        return np.lib.stride_tricks.as_strided(flat, shape=(rows, cols), strides=(ld * flat.itemsize, flat.itemsize))

    def gemm(self, c, c_colstride, trans_a, trans_b, alpha, a, a_row_count, a_col_count, a_colstride, b, b_col_count,
             b_colstride, beta):
        M, K, N = int(a_row_count), int(a_col_count), int(b_col_count)
        if M * N * K <= self.BLAS_THRESHOLD or min(M, N, K) == 0:
            return super().gemm(c, c_colstride, trans_a, trans_b, alpha, a, M, K, a_colstride, b, N, b_colstride, beta)
        A = self._matrix(a, K, M, a_colstride).T if trans_a else self._matrix(a, M, K, a_colstride)
        B = self._matrix(b, N, K, b_colstride).T if trans_b else self._matrix(b, K, N, b_colstride)
        Cm = self._matrix(c, M, N, c_colstride)
        dt = Cm.dtype.type
        prod = A @ B                      # OpenBLAS sgemm / dgemm in the element type
        if dt(beta) == 0:
            Cm[...] = dt(alpha) * prod
        else:
            Cm[...] = dt(alpha) * prod + dt(beta) * Cm

    def choose_convolution_algorithms(self, conv_descriptor, input_width, input_height, output_width, output_height,
                                      batch_size, max_ideal_workspace_size, use_defaults):
        # cpu/tensor_math.clj:1670-1680: the CPU path unrolls the whole batch
        k = conv_descriptor["kernel-width"] * conv_descriptor["kernel-height"] * conv_descriptor["in-channels"]
        return {"workspace-size": k * output_width * output_height * batch_size}

    def convolution_forward(self, output, output_dims, output_alpha, input, input_dims, weights, weight_dims,
                            workspace, workspace_ecount, conv_descriptor, algorithms):
        batch, cin, in_h, in_w = [int(x) for x in input_dims["shape"]]
        _, cout, out_h, out_w = [int(x) for x in output_dims["shape"]]
        kh, kw = conv_descriptor["kernel-height"], conv_descriptor["kernel-width"]
        flops = batch * cout * out_h * out_w * cin * kh * kw
        if flops <= (1 << 24):
            return super().convolution_forward(output, output_dims, output_alpha, input, input_dims, weights,
                                               weight_dims, workspace, workspace_ecount, conv_descriptor, algorithms)
        # big cases: same im2col + per-image BLAS gemm decomposition, vectorised with numpy
        npdt = NUMPY_NAME[output.dtype]
        x = self._matrix(input, batch, cin * in_h * in_w, cin * in_h * in_w).reshape(batch, cin, in_h, in_w)
        w = self._matrix(weights, cout, cin * kh * kw, cin * kh * kw)
        out = self._matrix(output, batch, cout * out_h * out_w, cout * out_h * out_w).reshape(batch, cout, out_h * out_w)
        px, py = conv_descriptor["pad-x"], conv_descriptor["pad-y"]
        sx, sy = conv_descriptor["stride-x"], conv_descriptor["stride-y"]
        for n in range(batch):
            xp = np.zeros((cin, in_h + 2 * py, in_w + 2 * px), dtype=npdt)
            xp[:, py:py + in_h, px:px + in_w] = x[n]
            cols = np.empty((out_h * out_w, cin, kh, kw), dtype=npdt)
            for ky in range(kh):
                for kx in range(kw):
                    patch = xp[:, ky:ky + sy * out_h:sy, kx:kx + sx * out_w:sx]
                    cols[:, :, ky, kx] = patch.reshape(cin, -1).T
            prod = w @ cols.reshape(out_h * out_w, -1).T
            if float(output_alpha) == 0.0:
                out[n] = prod
            else:
                out[n] = prod + np.dtype(npdt).type(output_alpha) * out[n]


class OracleDevice:
    def __init__(self, driver):
        self.driver, self.index, self.name = driver, 0, "cpu-oracle"

    def memory_info(self):
        return {"free": 0, "total": 0}

    def create_stream(self):
        return OracleStream(self)

    def allocate_device_buffer(self, elem_count, elem_type):
        return _MemBuffer(elem_count, elem_type, self)

    def get_device(self):
        return self

    def get_driver(self):
        return self.driver


class OracleDriver:
    def __init__(self):
        load()
        self._device = OracleDevice(self)

    def get_devices(self):
        return [self._device]

    def default_device(self):
        return self._device

    def allocate_host_buffer(self, elem_count, elem_type, usage_type="one-time"):
        return _MemBuffer(elem_count, elem_type, None)
