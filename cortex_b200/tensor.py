"""The tensor API of the hot path: a host-side mirror of ``cortex.tensor``
(src/cortex/tensor.clj).

All argument checking, broadcast rules, alias detection and the dispatch between
the op / accum / constant forms of the backend protocol happen here, exactly
where the reference does them, so that a backend only ever sees
``(stream, buffer, dimensions, scalars, op, n-elems)``.  The backend is whatever
stream object is bound with :func:`with_stream` (the B200 stream in production).
"""
import contextlib
import math
import threading

import numpy as np

from . import dimensions as dims
from .dimensions import ALL, DimensionError  # noqa: F401  (re-exported)
from ._lib import NUMPY_NAME

class _Bindings(threading.local):
    """ct/*stream* and ct/*datatype* are Clojure dynamic vars: bindings are per thread, which is what lets
    N host threads drive N streams of one device at once (src/cortex/verify/nn/train.clj:211-236)."""
    stream = None
    datatype = "double"       # ct/*datatype* defaults to :double (tensor.clj:106)


_bound = _Bindings()

UNARY_OPERATIONS = ["floor", "ceil", "round", "-", "tanh", "logistic", "exp", "sqrt", "noop"]
BINARY_OPERATIONS = ["+", "-", "*", "/", "max", "min", "bit-and", "bit-xor", "eq", ">", ">=", "<", "<="]
UNARY_REDUCTION_OPERATIONS = ["max", "min", "sum", "mean", "magnitude-squared", "magnitude"]


class TensorError(ValueError):
    pass


def _require(cond, msg, data=None):
    if not cond:
        raise TensorError("%s %s" % (msg, data if data is not None else ""))


@contextlib.contextmanager
def with_stream(stream):
    """ct/with-stream (tensor.clj:91-100)."""
    prev, _bound.stream = _bound.stream, stream
    try:
        yield stream
    finally:
        _bound.stream = prev


@contextlib.contextmanager
def with_datatype(datatype):
    prev, _bound.datatype = _bound.datatype, datatype
    try:
        yield
    finally:
        _bound.datatype = prev


def check_stream():
    _require(_bound.stream is not None, "Stream is nil. Use with_stream to bind a stream.")
    return _bound.stream


def dtype_cast(value, datatype):
    """drv/dtype-cast (src/cortex/compute/driver.clj:20-43)."""
    if datatype == "double":
        return float(value)
    if datatype == "float":
        return float(np.float32(value))
    bits = {"byte": 8, "short": 16, "int": 32, "long": 64}[datatype]
    v = int(value)
    _require(-(1 << (bits - 1)) <= v < (1 << (bits - 1)), "Value out of range for %s" % datatype, value)
    return v


class Tensor:
    """defrecord Tensor [device dimensions buffer] (tensor.clj:174-196)."""

    def __init__(self, device, dimensions, buffer):
        self.device, self.dimensions, self.buffer = device, dimensions, buffer

    def get_datatype(self):
        return self.buffer.dtype

    def shape(self):
        return dims.shape(self.dimensions)

    def ecount(self):
        return dims.ecount(self.dimensions)

    def _with(self, dimensions=None, buffer=None):
        return Tensor(self.device, dimensions if dimensions is not None else self.dimensions,
                      buffer if buffer is not None else self.buffer)

    def __repr__(self):
        return "Tensor<%s %r strides %r>" % (self.get_datatype(), self.dimensions["shape"], self.dimensions["strides"])


def scalar(item):
    return isinstance(item, (int, float, np.integer, np.floating)) and not isinstance(item, bool)


def get_datatype(tensor):
    return tensor.get_datatype()


def shape(tensor):
    return tensor.shape()


def ecount(tensor):
    return tensor.ecount()


def _kind(item):
    if isinstance(item, Tensor):
        return "tensor"
    if scalar(item):
        return "number"
    raise TensorError("argument is neither a tensor nor a number: %r" % (item,))


def _column_stride(d):
    """dimensions->column-stride (tensor.clj:198-204): the row pitch of the 2-d view."""
    st = d["strides"]
    if len(st) > 1:
        return st[-2]
    shp = d["shape"]
    return shp[0] if shp else 1


def _num_columns(d):
    shp = d["shape"]
    return shp[1] if len(shp) > 1 else 1


def tensor_to_2d_shape(t):
    return dims.to_2d_shape(t.dimensions)


def tensor_to_batch_shape(t):
    return dims.to_batch_shape(t.dimensions)


def in_place_reshape(tensor, new_shape):
    return tensor._with(dimensions=dims.in_place_reshape(tensor.dimensions, list(new_shape)))


def dense(tensor):
    return dims.dense(tensor.dimensions)


def strided(tensor):
    return not dense(tensor)


def as_batch_matrix(tensor):
    shp = tensor.dimensions["shape"]
    if len(shp) == 2 and type(shp[0]) is int and type(shp[1]) is int:
        return tensor                 # already [batch, rest]: the reshape is the identity (and costs ~10 us of host time)
    return in_place_reshape(tensor, tensor_to_batch_shape(tensor))


def as_2d_matrix(tensor):
    return in_place_reshape(tensor, tensor_to_2d_shape(tensor))


def as_vector(tensor):
    """m/as-vector on a tensor: a dense tensor viewed as [ecount]."""
    _require(dense(tensor) or tensor.ecount() == 1 or len(tensor.shape()) == 1,
             "as-vector needs a dense tensor", tensor)
    if len(tensor.shape()) == 1:
        return tensor
    return in_place_reshape(tensor, [tensor.ecount()])


def as_column_vector(tensor):
    _require(_num_columns(tensor.dimensions) == 1 or dense(tensor),
             "Column vectors must either be dense or have num-columns = 1")
    return tensor._with(dimensions=dims.dimensions([tensor.ecount(), 1]))


def as_row_vector(tensor):
    _require(_num_columns(tensor.dimensions) == 1 or dense(tensor),
             "Row vectors must either be dense or have num-columns = 1")
    return tensor._with(dimensions=dims.dimensions([tensor.ecount()]))


def as_dense(tensor):
    if dense(tensor) and dims.access_increasing(tensor.dimensions):
        return tensor
    return None


def _ensure_datatypes(datatype, *args):
    _require(all(a.get_datatype() == datatype for a in args), "Not all arguments match required datatype",
             {"datatype": datatype, "argument-datatypes": [a.get_datatype() for a in args]})


def _ensure_same_device(*args):
    first = args[0].device
    _require(all(a.device is first for a in args), "Tensor arguments are not all on same device")


def _check_partial_alias(*args):
    bufs = [a.buffer for a in args]
    for i in range(len(bufs)):
        for j in range(i + 1, len(bufs)):
            _require(not bufs[i].partially_alias(bufs[j]), "Partially overlapping arguments detected.")


def _commensurate(lhs, rhs):
    return rhs == 0 or lhs % rhs == 0


# ------------------------------ construction ---------------------------------

def _index_value(tensor, i):
    """dtype/get-value on an index tensor's buffer: one element read back from the device."""
    return int(to_array(tensor)[i])


def to_tensor(data, datatype=None):
    """->tensor (tensor.clj:415-435): upload nested sequence / array data."""
    datatype = datatype or _bound.datatype
    stream = check_stream()
    arr = np.ascontiguousarray(np.asarray(data), dtype=NUMPY_NAME[datatype])
    n = int(arr.size)
    device = stream.get_device()
    drv = stream.get_driver()
    host = drv.allocate_host_buffer(n, datatype)
    host.as_numpy()[:] = arr.reshape(-1)
    dev = device.allocate_device_buffer(n, datatype)
    stream.copy_host_to_device(host, 0, dev, 0, n)
    stream.sync()
    host.release()
    return Tensor(device, dims.dimensions(list(arr.shape)), dev)


def new_tensor(shp, datatype=None, init_value=0):
    """new-tensor (tensor.clj:438-450)."""
    datatype = datatype or _bound.datatype
    shp = [int(s) for s in shp]
    stream = check_stream()
    device = stream.get_device()
    n = 1
    for s in shp:
        n *= s
    dev = device.allocate_device_buffer(n, datatype)
    if init_value is not None:
        stream.memset(dev, 0, 0, n)
    return Tensor(device, dims.dimensions(shp), dev)


def make_dense(tensor):
    d = as_dense(tensor)
    if d is not None:
        return d
    out = new_tensor(tensor.shape(), datatype=tensor.get_datatype(), init_value=None)
    assign(out, tensor)
    return out


def to_array(tensor):
    """copy-to-java-type (tensor.clj:376-391): dense copy, download, host sync."""
    stream = check_stream()
    t = make_dense(tensor)
    n = t.ecount()
    host = stream.get_driver().allocate_host_buffer(n, t.get_datatype())
    stream.copy_device_to_host(t.buffer, 0, host, 0, n)
    stream.create_event().wait_for_event()
    out = np.array(host.as_numpy(), copy=True)
    host.release()
    return out


def to_double_array(tensor):
    return to_array(tensor).astype(np.float64)


# ------------------------------ views ----------------------------------------

def transpose(tensor, reorder):
    return tensor._with(dimensions=dims.transpose(tensor.dimensions, list(reorder)))


def select(tensor, *args):
    """select (tensor.clj:462-477)."""
    r = dims.select(tensor.dimensions, *args, index_value=_index_value)
    off = r["elem-offset"]
    buf = tensor.buffer
    return tensor._with(dimensions=r["dimensions"], buffer=buf.sub_buffer(off, buf.ecount() - off))


def subvector(tensor, offset, length=None):
    _require(offset >= 0, "Offset must be >= 0")
    v = as_vector(tensor)
    stop = offset + length if length is not None else v.ecount()
    return select(v, list(range(offset, stop)))


def submatrix(tensor, row_start, row_length, col_start, col_length):
    """submatrix (tensor.clj:490-513): window of the 2-d view, parent strides kept."""
    t = as_2d_matrix(tensor)
    n_rows, n_cols = t.shape()
    d = t.dimensions
    rev_shape, rev_strides = list(reversed(d["shape"])), list(reversed(d["strides"]))
    addr = dims.elem_idx_to_addr(rev_shape, rev_strides, rev_shape, row_start * n_cols + col_start)
    buf = t.buffer.sub_buffer(addr, t.buffer.ecount() - addr)
    return t._with(dimensions={"shape": [row_length, col_length], "strides": list(d["strides"])}, buffer=buf)


def rows(tensor):
    n_rows, n_cols = tensor_to_2d_shape(tensor)
    return [select(tensor, r, list(range(n_cols))) for r in range(n_rows)]


def columns(tensor):
    n_rows, n_cols = tensor_to_2d_shape(tensor)
    return [select(tensor, list(range(n_rows)), c) for c in range(n_cols)]


# ------------------------------ assign! ---------------------------------------

def _memcpy_semantics(dest, src):
    return (dest.ecount() == src.ecount() and dense(dest) and dense(src)
            and dims.access_increasing(dest.dimensions) and dims.access_increasing(src.dimensions)
            and dest.get_datatype() == src.get_datatype())


def assign(dest, src):
    """assign! / typed-assign! (tensor.clj:83-86, 535-589)."""
    stream = check_stream()
    if _kind(src) == "number":
        if dense(dest):
            stream.memset(dest.buffer, 0, src, dest.ecount())
        else:
            stream.assign_constant(dest.buffer, dest.dimensions, src, dest.ecount())
        return dest
    de, se = dest.ecount(), src.ecount()
    _require(de >= se, "destination element count must be >= src element count", (de, se))
    _require(_commensurate(de, se), "Src element count must evenly divide dest ecount.", (de, se))
    _ensure_same_device(dest, src)
    _check_partial_alias(dest, src)
    if _memcpy_semantics(dest, src):
        stream.copy_device_to_device(src.buffer, 0, dest.buffer, 0, se)
    else:
        stream.assign(dest.buffer, dest.dimensions, src.buffer, src.dimensions, max(se, de))
    return dest


def _ensure_broadcast_rules(*args):
    """tensor.clj:592-604: every extent divides the op-wide maximum."""
    r = dims.dimension_seq_to_max_shape(*[a.dimensions for a in args])
    mx = r["max-shape"]
    for d in r["dimensions"]:
        shp = dims.shape(d)
        _require(all(m % s == 0 for m, s in zip(mx, shp)),
                 "Shapes are not broadcast-compatible (dimension counts must be commensurate)",
                 {"shapes": [dims.shape(x) for x in r["dimensions"]], "max-shapes": mx})


# ------------------------------ unary-op! --------------------------------------

def _jvm_round(v):
    if v != v:
        return 0
    return int(math.floor(v + 0.5)) if abs(v) < 2 ** 52 else int(v)


def _perform_unary_op(value, op):
    return {
        "ceil": lambda v: float(math.ceil(v)), "round": lambda v: float(_jvm_round(v)),
        "floor": lambda v: float(math.floor(v)), "-": lambda v: -v, "tanh": math.tanh,
        "logistic": lambda v: 1.0 / (1.0 + math.exp(-v)), "exp": math.exp, "sqrt": math.sqrt, "noop": lambda v: v,
    }[op](value)


def unary_op(dest, alpha, x, op):
    """dest[idx] = op(alpha * x)   (tensor.clj:627-651)."""
    _require(op in UNARY_OPERATIONS, "unknown unary operation", op)
    stream = check_stream()
    if _kind(x) == "number":
        dt = dest.get_datatype()
        assign(dest, _perform_unary_op(float(dtype_cast(alpha, dt)) * float(dtype_cast(x, dt)), op))
        return dest
    if dest.buffer.alias(x.buffer):
        stream.unary_accum(dest.buffer, dest.dimensions, alpha, op, dest.ecount())
    else:
        _ensure_datatypes(dest.get_datatype(), x)
        _ensure_same_device(dest, x)
        _ensure_broadcast_rules(dest, x)
        _check_partial_alias(dest, x)
        stream.unary_op(dest.buffer, dest.dimensions, x.buffer, x.dimensions, alpha, op,
                        max(dest.ecount(), x.ecount()))
    return dest


# ------------------------------ binary-op! --------------------------------------

def _binary_op_constant(dest, alpha, x, beta, y, op, reverse_operands):
    """tensor.clj:676-708."""
    stream = check_stream()
    _ensure_broadcast_rules(dest, x)
    _ensure_datatypes(dest.get_datatype(), x)
    y = float(beta) * float(y)
    if op == "*":
        return unary_op(dest, float(alpha) * y, x, "noop")
    if dest.buffer.alias(x.buffer):
        stream.binary_accum_constant(dest.buffer, dest.dimensions, alpha, y, dest.ecount(), op, reverse_operands)
    else:
        _check_partial_alias(dest, x)
        stream.binary_op_constant(dest.buffer, dest.dimensions, x.buffer, x.dimensions, alpha, y,
                                  max(x.ecount(), dest.ecount()), op, reverse_operands)
    return dest


def _typed_binary_op(dest, alpha, x, beta, y, op):
    kx, ky = _kind(x), _kind(y)
    stream = check_stream()
    if kx == "number" and ky == "number":
        a, b = float(alpha) * float(x), float(beta) * float(y)
        table = {"+": a + b, "-": a - b, "*": a * b, "max": max(a, b), "min": min(a, b)}
        if op == "/":
            return assign(dest, a / b)
        _require(op in table, "operation is not defined for two scalars", op)
        return assign(dest, table[op])
    if kx == "tensor" and ky == "number":
        return _binary_op_constant(dest, alpha, x, beta, y, op, False)
    if kx == "number" and ky == "tensor":
        return _binary_op_constant(dest, beta, y, alpha, x, op, True)
    # tensor, tensor (tensor.clj:716-761)
    r = dims.dimension_seq_to_max_shape(dest.dimensions, x.dimensions, y.dimensions)
    max_shape = r["max-shape"]
    dest_dims, x_dims, y_dims = r["dimensions"]
    x_alias = dest.buffer.alias(x.buffer)
    arg_alias = x_alias or dest.buffer.alias(y.buffer)
    dest_is_max_shape = dims.shape(dest_dims) == max_shape
    if not dest_is_max_shape and not arg_alias:
        raise TensorError("If destination is a broadcast target then it must be one of the operands")
    if arg_alias:
        if x_alias:
            a, b, other, rev = alpha, beta, y, False
        else:
            a, b, other, rev = beta, alpha, x, True
        _ensure_broadcast_rules(dest, other)
        _ensure_datatypes(dest.get_datatype(), other)
        stream.binary_accum(dest.buffer, dest.dimensions, a, other.buffer, other.dimensions, b,
                            max(dest.ecount(), other.ecount()), op, rev, not dest_is_max_shape)
    else:
        _ensure_broadcast_rules(dest, x, y)
        _ensure_datatypes(x.get_datatype(), y, dest)
        stream.binary_op(dest.buffer, dest_dims, x.buffer, x_dims, alpha, y.buffer, y_dims, beta,
                         max(dest.ecount(), x.ecount(), y.ecount()), op)
    return dest


def binary_op(dest, alpha, x, beta, y, op):
    """dest = alpha * x op beta * y   (tensor.clj:768-779)."""
    _require(op in BINARY_OPERATIONS, "unknown binary operation", op)
    if op == "-":
        _typed_binary_op(dest, alpha, x, -float(beta), y, "+")
    else:
        _typed_binary_op(dest, alpha, x, beta, y, op)
    return dest


# ------------------------------ ternary-op! ---------------------------------------

def activation_gradient(input_gradient, output_gradient, output, op):
    """input-gradient from the output of an activation (tensor.clj:1256-1283):
    logistic: out * (1 - out) * out-grad;  tanh: (1 - out * out) * out-grad;  relu: (out > 0) ? out-grad : 0."""
    _ensure_datatypes(input_gradient.get_datatype(), output, output_gradient)
    _ensure_same_device(input_gradient, output, output_gradient)
    _require(input_gradient.get_datatype() in ("float", "double"),
             "activation-gradient! is only defined for float and double tensors", input_gradient.get_datatype())
    _require(op in ("logistic", "tanh", "relu"), "Only :logistic :tanh and :relu are supported", op)
    out_ecount = output.ecount()
    _require(out_ecount == input_gradient.ecount() and out_ecount == output_gradient.ecount(),
             "All element ecounts must match",
             {"out-ecount": out_ecount, "in-grad-ecount": input_gradient.ecount(),
              "out-grad-ecount": output_gradient.ecount()})
    check_stream().activation_gradient(input_gradient.buffer, input_gradient.dimensions, output_gradient.buffer,
                                       output_gradient.dimensions, output.buffer, output.dimensions, op, out_ecount)
    return input_gradient


TERNARY_OPERATIONS = ("select",)


def ternary_op(dest, alpha, x, beta, y, gamma, z, op):
    """dest = op(alpha * x, beta * y, gamma * z); x, y, z tensors or numbers (tensor.clj:808-854).
    select: the reference's backends (and its own tests) give  alpha*x >= 0 ? gamma*z : beta*y."""
    _require(op in TERNARY_OPERATIONS, "unknown ternary operation", op)
    args = [(x, alpha, "x"), (y, beta, "y"), (z, gamma, "z")]
    tensors = [(a, f, nm) for a, f, nm in args if _kind(a) == "tensor"]
    constants = [(a, f, nm) for a, f, nm in args if _kind(a) != "tensor"]
    if not tensors:
        a, b, c = (float(f) * float(v) for v, f, _ in args)
        return assign(dest, c if a >= 0 else b)          # inline-ternary-op (tensor.clj:782-789)
    _ensure_datatypes(dest.get_datatype(), *[t for t, _, _ in tensors])
    _ensure_same_device(dest, *[t for t, _, _ in tensors])
    for t, _, _ in tensors:
        _ensure_broadcast_rules(dest, t)
    n_elems = max(t.ecount() for t, _, _ in tensors)
    stream = check_stream()
    # order-ternary-args (tensor.clj:792-805): tensors first, then constants already multiplied
    arg_order = [nm for _, _, nm in tensors] + [nm for _, _, nm in constants]
    consts = [float(v) * float(f) for v, f, _ in constants]
    if len(tensors) == 3:
        stream.ternary_op(dest.buffer, dest.dimensions, x.buffer, x.dimensions, alpha, y.buffer, y.dimensions, beta,
                          z.buffer, z.dimensions, gamma, n_elems, op)
    elif len(tensors) == 2:
        (a, af, _), (b, bf, _) = tensors
        stream.ternary_op_constant(dest.buffer, dest.dimensions, a.buffer, a.dimensions, af, b.buffer, b.dimensions, bf,
                                   consts[0], n_elems, op, arg_order)
    else:
        (a, af, _), = tensors
        stream.ternary_op_constant_constant(dest.buffer, dest.dimensions, a.buffer, a.dimensions, af, consts[0],
                                            consts[1], n_elems, op, arg_order)
    return dest


# ------------------------------ unary-reduce! ------------------------------------

def unary_reduce(output, alpha, input, op):
    """tensor.clj:861-884: reduce the last axis of input into output[..., 1]."""
    _require(op in UNARY_REDUCTION_OPERATIONS, "unknown reduction", op)
    oshape, ishape = output.shape(), input.shape()
    _require(oshape[:-1] == ishape[:-1], "Output leading dimensions must match input leading dimensions",
             (oshape, ishape))
    _require(oshape[-1] == 1, "Last dimension of output must be 1", oshape)
    _ensure_same_device(output, input)
    _ensure_datatypes(output.get_datatype(), input)
    check_stream().unary_reduce(output.buffer, output.dimensions, alpha, input.buffer, input.dimensions, op)
    return output


# ------------------------------ gemm! ---------------------------------------------

def _external_library_check(name, *tensors):
    """tensor.clj:895-917."""
    _ensure_datatypes(tensors[0].get_datatype(), *tensors[1:])
    _ensure_same_device(*tensors)
    _require(tensors[0].get_datatype() in ("float", "double"),
             "%s is only defined for float and double tensors" % name)
    _require(all(dims.access_increasing(t.dimensions) for t in tensors),
             "External libraries (blas (gemm gemv) and cudnn require dimensions access to be increasing")


def _trans_2d_shape(trans, t):
    r, c = tensor_to_2d_shape(t)
    return (c, r) if trans else (r, c)


def gemm(C, trans_a, trans_b, alpha, A, B, beta):
    """C = alpha * (trans-a? A) * (trans-b? B) + beta * C   (tensor.clj:920-951)."""
    _external_library_check("gemm!", C, A, B)
    a_rows, a_cols = _trans_2d_shape(trans_a, A)
    b_rows, b_cols = _trans_2d_shape(trans_b, B)
    c_rows, c_cols = tensor_to_2d_shape(C)
    _require(a_cols == b_rows, "A col count doesn't match B row count", ((a_rows, a_cols), (b_rows, b_cols)))
    _require(a_rows == c_rows, "C row count doesn't match A row count", ((c_rows, c_cols), (a_rows, a_cols)))
    _require(b_cols == c_cols, "C col count doesn't match B col count", ((c_rows, c_cols), (b_rows, b_cols)))
    check_stream().gemm(C.buffer, _column_stride(C.dimensions), trans_a, trans_b, alpha, A.buffer, a_rows, a_cols,
                        _column_stride(A.dimensions), B.buffer, b_cols, _column_stride(B.dimensions), beta)
    return C


def _ensure_vector_indexable(*tensors):
    """tensor.clj:954-962."""
    for t in tensors:
        _require(dense(t) or _num_columns(t.dimensions) == 1, "Argument is not vector-indexable", t)


def _blas_vector_increment(t):
    """tensor.clj:965-971."""
    return 1 if dense(t) else (t.dimensions["strides"][-1] or 1)


def gemv(c, trans_a, alpha, A, x, beta):
    """c = alpha * (trans-a? A) * x + beta * c   (tensor.clj:974-989)."""
    _external_library_check("gemv!", c, A, x)
    _ensure_vector_indexable(x, c)
    a_rows, a_cols = tensor_to_2d_shape(A)
    check_stream().gemv(c.buffer, _blas_vector_increment(c), trans_a, alpha, A.buffer, a_rows, a_cols,
                        _column_stride(A.dimensions), x.buffer, _blas_vector_increment(x), beta)
    return c


def _batch_normalize_setup(io_args, stat_args, epsilon):
    """The shared precondition checks of the batch-normalize calls (tensor.clj:1047-1102): returns
    (kind, stat tensors as row vectors, input shape with a leading 1 for vectors)."""
    input = io_args[0]
    input_shape = input.shape()
    if len(input_shape) == 1:
        input_shape = [1, input_shape[0]]
    _external_library_check("batch-normalize", *io_args, *stat_args)
    _require(float(epsilon) > 1e-5, "Epsilon cannot be smaller than 1e-5 (cudnn limitation", epsilon)
    _require(input.get_datatype() in ("float", "double"),
             "batch-normalization is only defined for float and double tensors", input.get_datatype())
    _ensure_vector_indexable(*stat_args)
    stats = [as_row_vector(t) for t in stat_args]
    _require(len(input_shape) > 1, "Input shape needs at least 2 dimensions", input.shape())
    _require(len({tuple(t.shape()) for t in io_args}) == 1, "Tensor input and output shapes do not match",
             [t.shape() for t in io_args])
    _require(len({tuple(t.shape()) for t in stats}) == 1, "means, variances, scale, bias must have same shape",
             [t.shape() for t in stats])
    n_stats = stats[0].shape()[0]
    if len(input_shape) == 2:
        _require(input_shape[1] == n_stats, "Means, variances, scale, bias must match input element count.",
                 (input_shape, n_stats))
        return "eltwise", stats, input_shape
    _require(input_shape[-2] == n_stats, "means, variances, scale bias size must match input channel count",
             (input_shape, n_stats))
    return "spatial", stats, input_shape


def _spatial_extents(input_shape):
    batch_count = 1
    for v in input_shape[:-2]:
        batch_count *= v
    return batch_count, input_shape[-2], input_shape[-1]


def batch_normalize(output, input, means, variances, scale, bias, epsilon):
    """output = (input - mean) / sqrt(variance + epsilon) * scale + bias   (tensor.clj:1105-1145).
    2 dimensions: elementwise, statistics per column; more: 'spatial', statistics per entry of the
    second-to-last dimension, everything before it is batch."""
    kind, stats, input_shape = _batch_normalize_setup([output, input], [means, variances, scale, bias], epsilon)
    stream = check_stream()
    bufs = [t.buffer for t in stats]
    if kind == "eltwise":
        stream.batch_normalize_eltwise(output.buffer, input.buffer, *bufs, epsilon, input_shape[0], input_shape[1])
    else:
        stream.batch_normalize_spatial(output.buffer, input.buffer, *bufs, epsilon, *_spatial_extents(input_shape))
    return output


def batch_normalize_update_and_apply(output, input, batch_means, batch_variances, running_means, running_variances,
                                     ave_factor, scale, bias, epsilon):
    """Per-batch statistics, running statistics (running * (1 - ave-factor) + batch * ave-factor) and the
    normalised output in one call (tensor.clj:1147-1199).  Returns
    [output, batch_means, batch_variances, running_means, running_variances]."""
    kind, stats, input_shape = _batch_normalize_setup(
        [output, input], [batch_means, batch_variances, running_means, running_variances, scale, bias], epsilon)
    bm, bv, rm, rv, sc, bi = [t.buffer for t in stats]
    stream = check_stream()
    if kind == "eltwise":
        stream.batch_normalize_update_and_apply_eltwise(output.buffer, input.buffer, bm, bv, rm, rv, ave_factor, sc, bi,
                                                        epsilon, input_shape[0], input_shape[1])
    else:
        stream.batch_normalize_update_and_apply_spatial(output.buffer, input.buffer, bm, bv, rm, rv, ave_factor, sc, bi,
                                                        epsilon, *_spatial_extents(input_shape))
    return [output, batch_means, batch_variances, running_means, running_variances]


def batch_normalize_gradients(input_gradient, scale_gradient, bias_gradient, output_gradient, output, input,
                              batch_means, batch_variances, scale, bias, epsilon):
    """Gradients of the training form; batch_means / batch_variances must be what update-and-apply wrote
    (tensor.clj:1202-1250).  Returns [input_gradient, scale_gradient, bias_gradient]."""
    kind, stats, input_shape = _batch_normalize_setup(
        [output, input, output_gradient, input_gradient],
        [batch_means, batch_variances, scale, bias, scale_gradient, bias_gradient], epsilon)
    bm, bv, sc, bi, sg, bg = [t.buffer for t in stats]
    stream = check_stream()
    args = (input_gradient.buffer, sg, bg, output_gradient.buffer, output.buffer, input.buffer, bm, bv, sc, bi, epsilon)
    if kind == "eltwise":
        stream.batch_normalize_gradients_eltwise(*args, input_shape[0], input_shape[1])
    else:
        stream.batch_normalize_gradients_spatial(*args, *_spatial_extents(input_shape))
    return [input_gradient, scale_gradient, bias_gradient]


# ------------------------------ softmax! -------------------------------------------

def gaussian_distribution(mean=0, variance=1):
    """ct/gaussian-distribution (tensor.clj:990-998)."""
    return {"type": "gaussian", "mean": float(mean), "variance": float(variance)}


def flat_distribution(minimum=0, maximum=1):
    """ct/flat-distribution (tensor.clj:1001-1014): [minimum, maximum)."""
    _require(float(minimum) < float(maximum), "Minimum must be less than maximum",
             {"minimum": minimum, "maximum": maximum})
    return {"type": "flat", "minimum": float(minimum), "maximum": float(maximum)}


_rand_state = {"seed": 0x5EEDC0DE, "sequence": 0}
_rand_lock = threading.Lock()


def seed_rand(seed):
    """Restart the generator behind rand!: the same seed replays the same sequence of rand! results.
    (The reference draws from SecureRandom / cuRAND's default generator and cannot be replayed.)"""
    with _rand_lock:
        _rand_state["seed"], _rand_state["sequence"] = int(seed), 0


def rand(dest, distribution):
    """ct/rand! (tensor.clj:1028-1044): float tensors only, dense, access-increasing."""
    _require(dest.get_datatype() == "float", "Can only generate rands into floating point buffers",
             {"expected-datatype": "float", "received-datatype": dest.get_datatype()})
    _require(dims.dense(dest.dimensions) and dims.access_increasing(dest.dimensions),
             "Rand generation must have simple dense buffers")
    _require(distribution.get("type") in ("gaussian", "flat"), "Invalid distibution type",
             {"valid-types": ["flat", "gaussian"], "type": distribution.get("type")})
    with _rand_lock:
        seed, sequence = _rand_state["seed"], _rand_state["sequence"]
        _rand_state["sequence"] += 1
    check_stream().rand(dest.buffer, dest.dimensions, distribution, seed, sequence)
    return dest


def softmax(output, input):
    """tensor.clj:1286-1312."""
    _external_library_check("softmax!", output, input)
    _require(output.shape() == input.shape(), "Input, output shapes do not match", (input.shape(), output.shape()))
    stream = check_stream()
    if len(input.shape()) == 3:
        stream.softmax_spatial(output.buffer, output.dimensions, input.buffer, input.dimensions)
    else:
        i2, o2 = as_batch_matrix(input), as_batch_matrix(output)
        stream.softmax_eltwise(o2.buffer, o2.dimensions, i2.buffer, i2.dimensions)
    return output


# ------------------------------ convolution ------------------------------------------

def convolution_descriptor(datatype, out_channels, in_channels, kern_width, kern_height, pad_x, pad_y, stride_x,
                           stride_y):
    """tensor.clj:1322-1348."""
    args = dict(out_channels=out_channels, in_channels=in_channels, kern_width=kern_width, kern_height=kern_height,
                pad_x=pad_x, pad_y=pad_y, stride_x=stride_x, stride_y=stride_y)
    _require(all(v is not None for v in args.values()), "Arguments were nil:", args)
    return {"datatype": datatype, "out-channels": out_channels, "in-channels": in_channels,
            "kernel-width": kern_width, "kernel-height": kern_height, "pad-x": pad_x, "pad-y": pad_y,
            "stride-x": stride_x, "stride-y": stride_y,
            "descriptor": check_stream().convolution_descriptor(datatype, out_channels, in_channels, kern_width,
                                                                kern_height, pad_x, pad_y, stride_x, stride_y)}


def _padded_strided_dimension(input_dim, pad, kernel_size, stride, dimension_op):
    partial = (float(input_dim) + 2 * float(pad) - float(kernel_size)) / float(stride)
    partial = math.floor(partial) if dimension_op == "floor" else math.ceil(partial)
    return int(partial + 1)


def get_convolution_output_dimensions(conv_descriptor, input_width, input_height):
    """tensor.clj:1351-1382."""
    op = conv_descriptor.get("dimension-op", "floor")
    return {"output-width": _padded_strided_dimension(input_width, conv_descriptor["pad-x"],
                                                      conv_descriptor["kernel-width"], conv_descriptor["stride-x"], op),
            "output-height": _padded_strided_dimension(input_height, conv_descriptor["pad-y"],
                                                       conv_descriptor["kernel-height"], conv_descriptor["stride-y"],
                                                       op)}


def choose_convolution_algorithms(descriptor, input_width, input_height, batch_size, max_ideal_workspace_size,
                                  use_defaults=False):
    out = get_convolution_output_dimensions(descriptor, input_width, input_height)
    return check_stream().choose_convolution_algorithms(descriptor, input_width, input_height, out["output-width"],
                                                        out["output-height"], batch_size, max_ideal_workspace_size,
                                                        use_defaults)


def _ensure_conv_io(conv_descriptor, input, output):
    batch, _in_c, in_h, in_w = input.shape()
    # the reference passes (in-height in-width) into (input-width input-height) here (tensor.clj:1424)
    out = get_convolution_output_dimensions(conv_descriptor, in_h, in_w)
    expected_in = [batch, conv_descriptor["in-channels"], in_h, in_w]
    expected_out = [batch, conv_descriptor["out-channels"], out["output-width"], out["output-height"]]
    _require(dense(input) and dense(output), "Convolution arguments must be dense tensors")
    _require(input.shape() == expected_in, "Input dimensions do not match expected dimensions",
             (expected_in, input.shape()))
    _require(output.shape() == expected_out, "Output dimensions do not match expected dimensions",
             (expected_out, output.shape()))


POOL_OPERATIONS = ("max", "avg", "avg-exc-pad")


def pooling_descriptor(datatype, channels, kern_width, kern_height, pad_x, pad_y, stride_x, stride_y,
                       dimension_op="ceil", pool_op="max"):
    """tensor.clj:1499-1524."""
    _require(pool_op in POOL_OPERATIONS, "Max pooling layers have three possible pool operations:", pool_op)
    _require(dimension_op in ("floor", "ceil"), "dimension-op must be :floor or :ceil", dimension_op)
    desc = {"in-channels": channels, "out-channels": channels, "datatype": datatype, "kernel-width": kern_width,
            "kernel-height": kern_height, "pad-x": pad_x, "pad-y": pad_y, "stride-x": stride_x, "stride-y": stride_y,
            "pool-op": pool_op, "dimension-op": dimension_op}
    _require(all(v is not None for v in desc.values()), "Arguments were nil:", desc)
    desc["descriptor"] = check_stream().pooling_descriptor(datatype, kern_width, kern_height, pad_x, pad_y, stride_x,
                                                           stride_y, pool_op, dimension_op)
    return desc


def pooling_forward(output, output_alpha, input, pool_descriptor):
    """tensor.clj:1527-1538."""
    _external_library_check("pooling-forward!", output, input)
    _require(len(input.shape()) == 4 and len(output.shape()) == 4, "Input, output must be 4d tensors")
    _ensure_conv_io(pool_descriptor, input, output)
    check_stream().pooling_forward(output.buffer, output.dimensions, output_alpha, input.buffer, input.dimensions,
                                   pool_descriptor)
    return output


def pooling_backward(input_gradient, input_grad_alpha, input, output, output_gradient, pool_descriptor):
    """tensor.clj:1541-1551."""
    _external_library_check("pooling-backward!", input_gradient, input, output, output_gradient)
    for t in (input_gradient, input, output, output_gradient):
        _require(len(t.shape()) == 4, "Input, output must be 4d tensors")
    _ensure_conv_io(pool_descriptor, input_gradient, output)
    _ensure_conv_io(pool_descriptor, input, output_gradient)
    check_stream().pooling_backward(input_gradient.buffer, input_gradient.dimensions, input_grad_alpha, input.buffer,
                                    input.dimensions, output.buffer, output.dimensions, output_gradient.buffer,
                                    output_gradient.dimensions, pool_descriptor)
    return input_gradient


def lrn_descriptor(n=5, k=2, alpha=1e-4, beta=0.75):
    """Local response normalisation across channels (tensor.clj:1553-1560)."""
    return check_stream().lrn_descriptor(n, k, alpha, beta)


def _lrn_checks(name, output, *others):
    shapes = [t.shape() for t in (output,) + others]
    _require(all(sh == shapes[0] for sh in shapes), "Input and output shapes must match", shapes)
    _require(len(shapes[0]) >= 3, "tensor must be of at least rank 3", shapes[0])
    _ensure_datatypes(output.get_datatype(), *others)
    _require(output.get_datatype() in ("float", "double"), name + " is only defined for float and double tensors",
             output.get_datatype())


def lrn_forward(output, input, lrn_descriptor):
    """a[i] = a[i] / (k + alpha/n * sum of a[j]^2 over the window around i)^beta   (tensor.clj:1563-1585)."""
    _lrn_checks("lrn-forward", output, input)
    check_stream().lrn_forward(output.buffer, output.dimensions, input.buffer, input.dimensions, lrn_descriptor)
    return output


def lrn_backward(input_gradient, output, input, output_gradient, lrn_descriptor):
    """tensor.clj:1588-1617."""
    _lrn_checks("lrn-backward", output, input, input_gradient, output_gradient)
    check_stream().lrn_backward(input_gradient.buffer, input_gradient.dimensions, output.buffer, output.dimensions,
                                input.buffer, input.dimensions, output_gradient.buffer, output_gradient.dimensions,
                                lrn_descriptor)
    return input_gradient


def convolution_forward(output, output_alpha, input, weights, workspace, conv_descriptor, algorithms):
    """tensor.clj:1454-1466."""
    _external_library_check("convolution-forward!", output, input, weights)
    _require(len(input.shape()) == 4 and len(output.shape()) == 4, "Input, output must be 4d tensors")
    _ensure_conv_io(conv_descriptor, input, output)
    check_stream().convolution_forward(output.buffer, output.dimensions, output_alpha, input.buffer, input.dimensions,
                                       weights.buffer, weights.dimensions,
                                       workspace.buffer if workspace is not None else None,
                                       workspace.ecount() if workspace is not None else 0, conv_descriptor, algorithms)
    return output


def convolution_forward_bias_act(output, output_alpha, input, weights, conv_descriptor, bias=None, act=None):
    """Fused extra of this backend (no protocol counterpart): convolution-forward!, the layer's bias add and the
    following activation as one call.  bias: a dense tensor of out-channels elements or None; act: None, "relu",
    "tanh" or "logistic"."""
    _external_library_check("convolution-forward!", output, input, weights)
    _require(len(input.shape()) == 4 and len(output.shape()) == 4, "Input, output must be 4d tensors")
    _require(act in (None, "none", "relu", "tanh", "logistic"), "convolution epilogue activation must be relu, tanh or logistic")
    _ensure_conv_io(conv_descriptor, input, output)
    if bias is not None:
        _require(bias.ecount() == conv_descriptor["out-channels"] and dense(bias), "bias must be a dense tensor of out-channels elements")
        _require(bias.get_datatype() == output.get_datatype(), "bias datatype differs from the output's")
    check_stream().convolution_forward_bias_act(output.buffer, output.dimensions, output_alpha, input.buffer,
                                                input.dimensions, weights.buffer, weights.dimensions, conv_descriptor,
                                                bias.buffer if bias is not None else None, act)
    return output


def convolution_backward_weights(weight_gradient, weight_gradient_alpha, output_gradient, input, workspace,
                                 conv_descriptor, algorithms):
    """tensor.clj:1469-1479."""
    _external_library_check("convolution-backward-weights!", weight_gradient, output_gradient, input)
    check_stream().convolution_backward_weights(
        weight_gradient.buffer, weight_gradient.dimensions, weight_gradient_alpha, output_gradient.buffer,
        output_gradient.dimensions, input.buffer, input.dimensions,
        workspace.buffer if workspace is not None else None, workspace.ecount() if workspace is not None else 0,
        conv_descriptor, algorithms)
    return weight_gradient


def convolution_backward_data(input_gradient, input_gradient_alpha, output_gradient, weights, workspace,
                              conv_descriptor, algorithms):
    """tensor.clj:1482-1493."""
    _external_library_check("convolution-backward-data!", input_gradient, output_gradient, weights)
    _ensure_conv_io(conv_descriptor, input_gradient, output_gradient)
    check_stream().convolution_backward_data(
        input_gradient.buffer, input_gradient.dimensions, input_gradient_alpha, output_gradient.buffer,
        output_gradient.dimensions, weights.buffer, weights.dimensions,
        workspace.buffer if workspace is not None else None, workspace.ecount() if workspace is not None else 0,
        conv_descriptor, algorithms)
    return input_gradient
