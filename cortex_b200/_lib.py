"""ctypes binding of libcortex_b200.so (the C ABI declared in include/cortex_b200.h).

This is the stand-in, in this repository, for the JNA/JavaCPP stub a cortex
maintainer would write.  There is no fallback: if the shared library is missing
the import raises, and if it was built without a usable GPU the first call fails
with the CUDA error text.
"""
import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "lib", "libcortex_b200.so")

DTYPES = ("byte", "short", "int", "long", "float", "double")
DTYPE_CODE = {n: i for i, n in enumerate(DTYPES)}
DTYPE_SIZE = {"byte": 1, "short": 2, "int": 4, "long": 8, "float": 4, "double": 8}
NUMPY_NAME = {"byte": "int8", "short": "int16", "int": "int32", "long": "int64", "float": "float32",
              "double": "float64"}

BINARY_OPS = {"+": 0, "-": 1, "*": 2, "/": 3, "min": 4, "max": 5, "bit-and": 6, "bit-xor": 7, "eq": 8,
              ">": 9, ">=": 10, "<": 11, "<=": 12}
UNARY_OPS = {"floor": 0, "ceil": 1, "round": 2, "-": 3, "tanh": 4, "logistic": 5, "exp": 6, "sqrt": 7, "noop": 8}
TERNARY_OPS = {"select": 0}
REDUCE_OPS = {"max": 0, "min": 1, "sum": 2, "mean": 3, "magnitude": 4, "magnitude-squared": 5}
ACTIVATIONS = {None: 0, "none": 0, "relu": 1, "tanh": 2, "logistic": 3, "softmax": 4}    # softmax: gemm_bias_act only
DISTRIBUTIONS = {"flat": 0, "gaussian": 1}
STREAM_OPTIONS = {"gemm-auto-presplit": 0, "presplit-variant": 1, "f64-simple-kernel": 2, "wait-limit-cycles": 3,
                  "inject-fault": 4, "conv-route": 5, "gemm-k-slices": 6, "gemm-tile-n": 7, "gemm-slice-handover": 8}


class Dims(C.Structure):
    _fields_ = [("rev_shape", C.c_int32 * 5), ("rev_strides", C.c_int32 * 5), ("index", C.c_void_p * 5)]


class ConvDesc(C.Structure):
    _fields_ = [(n, C.c_int32) for n in ("out_channels", "in_channels", "kernel_width", "kernel_height",
                                         "pad_x", "pad_y", "stride_x", "stride_y")]


class PoolDesc(C.Structure):
    _fields_ = [(n, C.c_int32) for n in ("kernel_width", "kernel_height", "pad_x", "pad_y", "stride_x", "stride_y",
                                         "pool_op")]


POOL_OPS = {"max": 0, "avg": 1, "avg-exc-pad": 2}


class LrnDesc(C.Structure):
    _fields_ = [("n", C.c_int32), ("k", C.c_double), ("alpha", C.c_double), ("beta", C.c_double)]


class B200Error(RuntimeError):
    def __init__(self, code, message):
        super().__init__("cortex_b200 error %d: %s" % (code, message))
        self.code = code


_vp, _i, _i64, _d, _sz = C.c_void_p, C.c_int, C.c_int64, C.c_double, C.c_size_t
_pd = C.POINTER(Dims)

# name -> argtypes; every function returns int unless listed in _RESTYPE
SIGNATURES = {
    "cb200_device_count": [C.POINTER(_i)],
    "cb200_device_info": [_i, C.c_char_p, _i, C.POINTER(_i), C.POINTER(_i), C.POINTER(_i)],
    "cb200_mem_info": [_i, C.POINTER(_sz), C.POINTER(_sz)],
    "cb200_stream_create": [_i, C.POINTER(_vp)],
    "cb200_stream_destroy": [_vp],
    "cb200_stream_native": [_vp],
    "cb200_stream_device": [_vp],
    "cb200_malloc": [_i, _sz, C.POINTER(_vp)],
    "cb200_free": [_i, _vp],
    "cb200_host_alloc": [_sz, C.POINTER(_vp)],
    "cb200_host_free": [_vp],
    "cb200_host_alloc_near": [_i, _sz, C.POINTER(_vp), C.POINTER(_i)],
    "cb200_device_numa_node": [_i, C.POINTER(_i)],
    "cb200_memcpy_h2d": [_vp, _vp, _vp, _sz],
    "cb200_memcpy_d2h": [_vp, _vp, _vp, _sz],
    "cb200_memcpy_d2d": [_vp, _vp, _vp, _sz],
    "cb200_memset": [_vp, _i, _vp, _i64, _d, _i64],
    "cb200_event_record": [_vp, _i, C.POINTER(_vp)],
    "cb200_stream_wait_event": [_vp, _vp],
    "cb200_event_wait": [_vp],
    "cb200_event_elapsed_ms": [_vp, _vp, C.POINTER(C.c_float)],
    "cb200_event_destroy": [_vp],
    "cb200_stream_sync": [_vp],
    "cb200_assign_constant": [_vp, _i, _vp, _pd, _d, _i64],
    "cb200_assign": [_vp, _i, _vp, _pd, _i, _vp, _pd, _i64],
    "cb200_unary_accum": [_vp, _i, _vp, _pd, _d, _i, _i64],
    "cb200_unary_op": [_vp, _i, _vp, _pd, _vp, _pd, _d, _i, _i64],
    "cb200_binary_accum_constant": [_vp, _i, _vp, _pd, _d, _d, _i64, _i, _i],
    "cb200_binary_op_constant": [_vp, _i, _vp, _pd, _vp, _pd, _d, _d, _i64, _i, _i],
    "cb200_binary_accum": [_vp, _i, _vp, _pd, _d, _vp, _pd, _d, _i64, _i, _i, _i],
    "cb200_binary_op": [_vp, _i, _vp, _pd, _vp, _pd, _d, _vp, _pd, _d, _i64, _i],
    "cb200_unary_reduce": [_vp, _i, _vp, _pd, _d, _vp, _pd, _i],
    "cb200_gemm": [_vp, _i, _vp, _i64, _i, _i, _d, _vp, _i64, _i64, _i64, _vp, _i64, _i64, _d],
    "cb200_softmax_eltwise": [_vp, _i, _vp, _pd, _vp, _pd],
    "cb200_softmax_spatial": [_vp, _i, _vp, _pd, _vp, _pd],
    "cb200_convolution_workspace_size": [C.POINTER(ConvDesc), _i, _i, _i, _i, _i, C.POINTER(_i64)],
    "cb200_convolution_forward": [_vp, _i, _vp, _pd, _d, _vp, _pd, _vp, _pd, _vp, _i64, C.POINTER(ConvDesc)],
    "cb200_convolution_backward_weights": [_vp, _i, _vp, _pd, _d, _vp, _pd, _vp, _pd, _vp, _i64, C.POINTER(ConvDesc)],
    "cb200_convolution_backward_data": [_vp, _i, _vp, _pd, _d, _vp, _pd, _vp, _pd, _vp, _i64, C.POINTER(ConvDesc)],
    "cb200_convolution_forward_static": [_vp, _i, _vp, _pd, _d, _vp, _pd, _vp, _pd, C.POINTER(ConvDesc)],
    "cb200_convolution_forward_bias_act": [_vp, _i, _vp, _pd, _d, _vp, _pd, _vp, _pd, C.POINTER(ConvDesc), _vp, _i],
    "cb200_ternary_op": [_vp, _i, _vp, _pd, _vp, _pd, _d, _vp, _pd, _d, _vp, _pd, _d, _i64, _i],
    "cb200_gemv": [_vp, _i, _vp, _i64, _i, _d, _vp, _i64, _i64, _i64, _vp, _i64, _d],
    "cb200_batch_normalize_eltwise": [_vp, _i, _vp, _vp, _vp, _vp, _vp, _vp, _d, _i64, _i64],
    "cb200_batch_normalize_spatial": [_vp, _i, _vp, _vp, _vp, _vp, _vp, _vp, _d, _i64, _i64, _i64],
    "cb200_pooling_forward": [_vp, _i, _vp, _pd, _d, _vp, _pd, C.POINTER(PoolDesc)],
    "cb200_pooling_backward": [_vp, _i, _vp, _pd, _d, _vp, _pd, _vp, _pd, _vp, _pd, C.POINTER(PoolDesc)],
    "cb200_lrn_forward": [_vp, _i, _vp, _pd, _vp, _pd, C.POINTER(LrnDesc)],
    "cb200_lrn_backward": [_vp, _i, _vp, _pd, _vp, _pd, _vp, _pd, _vp, _pd, C.POINTER(LrnDesc)],
    "cb200_batch_normalize_update_and_apply_eltwise": [_vp, _i] + [_vp] * 6 + [_d, _vp, _vp, _d, _i64, _i64],
    "cb200_batch_normalize_update_and_apply_spatial": [_vp, _i] + [_vp] * 6 + [_d, _vp, _vp, _d, _i64, _i64, _i64],
    "cb200_batch_normalize_gradients_eltwise": [_vp, _i] + [_vp] * 10 + [_d, _i64, _i64],
    "cb200_batch_normalize_gradients_spatial": [_vp, _i] + [_vp] * 10 + [_d, _i64, _i64, _i64],
    "cb200_adam_step": [_vp, _i, _d, _d, _d, _d, _d, _d, _d, _vp, _vp, _vp, _vp, _i64],
    "cb200_adadelta_step": [_vp, _i, _d, _d, _vp, _vp, _d, _vp, _vp, _i64],
    "cb200_rand": [_vp, _vp, _pd, _i, _d, _d, C.c_uint64, C.c_uint64],
    "cb200_unsupported": [C.c_char_p],
    "cb200_gemm_bias_act": [_vp, _i, _vp, _i64, _i, _i, _d, _vp, _i64, _i64, _i64, _vp, _i64, _i64, _d, _vp, _i],
    "cb200_gemm_bias_act_peers": [_vp, _i, _vp, _i64, _i, _i, _d, _vp, _i64, _i64, _i64, _vp, _i64, _i64, _d, _vp, _i,
                                  _i, C.POINTER(_vp)],
    "cb200_graph_capture_begin": [_vp],
    "cb200_graph_capture_end": [_vp, C.POINTER(_vp)],
    "cb200_graph_launch": [_vp, _vp],
    "cb200_graph_destroy": [_vp],
    "cb200_peer_enable": [_i, _i],
    "cb200_ipc_export": [_i, _vp, C.c_char_p],
    "cb200_ipc_import": [_i, C.c_char_p, C.POINTER(_vp)],
    "cb200_ipc_close": [_i, _vp],
    "cb200_activation_gradient": [_vp, _i, _vp, _pd, _vp, _pd, _vp, _pd, _i, _i64],
    "cb200_split_lo": [_vp, _vp, _vp, _i64],
    "cb200_gemm_bias_act_presplit": [_vp, _vp, _vp, _i64, _d, _vp, _vp, _i64, _i64, _i64, _vp, _vp, _i64, _i64, _d, _vp, _i],
    "cb200_bias_relu_rowstats": [_vp, _i, _vp, _i64, _vp, _i64, _vp, _i64, _i64, _vp, _vp],
    "cb200_stream_set_option": [_vp, _i, _i64],
    "cb200_stream_workspace_info": [_vp, C.POINTER(_sz), C.POINTER(_i), C.POINTER(_i)],
    "cb200_gemm_f32_variant": [_vp, _i, _i, _vp, _i64, _i, _i, _d, _vp, _i64, _i64, _i64, _vp, _i64, _i64, _d],
    "cb200_launch_count": [_vp],
    "cb200_stream_status": [_vp, C.POINTER(_i), C.POINTER(_i)],
    "cb200_last_error": [],
}
_RESTYPE = {"cb200_last_error": C.c_char_p, "cb200_stream_native": _vp, "cb200_launch_count": _i64}
# entry points that do not follow "return status code"
_NO_CHECK = set(_RESTYPE) | {"cb200_stream_device"}

_lib = None


def load():
    """Load the shared library once; raises if it has not been built."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise ImportError("%s is missing: build it with `python -m cortex_b200.build` "
                          "(there is no CPU fallback)" % LIB_PATH)
    lib = C.CDLL(LIB_PATH)
    for name, argtypes in SIGNATURES.items():
        fn = getattr(lib, name)
        fn.argtypes = argtypes
        fn.restype = _RESTYPE.get(name, _i)
    _lib = lib
    return lib


def last_error():
    msg = load().cb200_last_error()
    return msg.decode("utf-8", "replace") if msg else ""


def call(name, *args):
    """Call a status-returning entry point; a non-zero status becomes B200Error
    (as check-cuda-error turns CUDA statuses into exceptions,
    src/cortex/compute/cuda/driver.clj:40-49)."""
    rc = getattr(load(), name)(*args)
    if name not in _NO_CHECK and rc != 0:
        raise B200Error(rc, last_error())
    return rc
