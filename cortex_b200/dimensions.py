"""Shape / stride / index-tensor descriptor algebra.

Host-side mirror of ``cortex.tensor.dimensions`` (src/cortex/tensor/dimensions.clj):
a *dimensions* value is a dict ``{"shape": [...], "strides": [...]}`` whose shape
entries are ints or 1-d int32 index tensors (indirect addressing of that
dimension).  First entry = slowest changing, last = fastest changing.  Nothing
here touches a device; the C ABI receives the reversed, 5-padded wire form built
by :func:`to_wire`.
"""
from functools import reduce
import operator


class DimensionError(ValueError):
    """Raised where the reference throws ex-info from when-not-error (dimensions.clj:14-17)."""


def _is_number(x):
    return type(x) is int or (isinstance(x, int) and not isinstance(x, bool))


def _prod(seq):
    return reduce(operator.mul, seq, 1)


def disambiguate_shape_entry(entry):
    """dimensions.clj:46-52 -- an index tensor counts as its element count."""
    if type(entry) is int:
        return entry
    if _is_number(entry):
        return int(entry)
    return int(entry.ecount())


def disambiguate_shape(shape):
    # the common case (every entry a plain int) without a call per entry: this runs on every tensor operation
    return [e if type(e) is int else disambiguate_shape_entry(e) for e in shape]


def direct_shape(shape):
    for e in shape:                      # a plain loop: this runs several times per tensor operation
        if type(e) is not int and not _is_number(e):
            return False
    return True


def extend_strides(shape, strides=None):
    """dimensions.clj:75-92 -- fill missing (outer) strides densely, innermost first."""
    strides = list(strides or [])
    rev_strides = list(reversed(strides))
    rev_shape = list(reversed(disambiguate_shape(shape)))
    new = []
    for d in range(len(shape)):
        cur = rev_strides[d] if d < len(rev_strides) else None
        if d == 0:
            new.append(cur if cur is not None else 1)
        else:
            new.append(cur if cur is not None else new[d - 1] * rev_shape[d - 1])
    return list(reversed(new))


def dimensions(shape, strides=None, names=None):
    """dimensions.clj:95-118."""
    shape = list(shape)
    strides = extend_strides(shape, strides)
    pairs = sorted(zip(disambiguate_shape(shape), strides), key=lambda p: -p[1])
    max_stride = max([0] + [p[1] for p in pairs])
    elem_count = _prod([p[0] for p in pairs[1:]])
    if not elem_count <= max_stride:
        raise DimensionError("Stride appears to be too small for element count: %r %r" % (shape, strides))
    return {"shape": shape, "strides": strides, "names": names}


def ecount(dims):
    return _prod(disambiguate_shape(dims["shape"]))


def shape(dims):
    return disambiguate_shape(dims["shape"])


def strides(dims):
    return list(dims["strides"])


def _ensure_direct(seq):
    if not direct_shape(seq):
        raise DimensionError("Index buffers not supported for this operation.")
    return seq


def to_2d_shape(dims):
    """dimensions.clj:144-153 -- [prod(leading), last]."""
    shp = dims["shape"]
    if not shp:
        raise DimensionError("Invalid shape in dimension map")
    if len(shp) == 1:
        return [1, disambiguate_shape_entry(shp[0])]
    return [_prod(_ensure_direct(shp[:-1])), disambiguate_shape_entry(shp[-1])]


def to_batch_shape(dims):
    """dimensions.clj:156-165 -- [first, prod(rest)]."""
    shp = dims["shape"]
    if not shp:
        raise DimensionError("Invalid shape in dimension map")
    if len(shp) == 1:
        return [1, disambiguate_shape_entry(shp[0])]
    return [disambiguate_shape_entry(shp[0]), _prod(_ensure_direct(shp[1:]))]


def dense(dims):
    """dimensions.clj:178-191."""
    shp, st = dims["shape"], dims["strides"]
    if not direct_shape(shp):
        return False
    if len(shp) == 1:
        return st[0] == 1
    pairs = sorted([(s, t) for s, t in zip(shp, st) if s != 1], key=lambda p: -p[1])
    if not pairs:
        # every extent is 1: the reference compares nil with 1 here and answers false
        return False
    return pairs[0][1] == _prod([p[0] for p in pairs[1:]])


def direct(dims):
    return direct_shape(dims["shape"])


def access_increasing(dims):
    """dimensions.clj:204-211 -- strides non-increasing and no index tensors."""
    st = dims["strides"]
    if not direct_shape(dims["shape"]):
        return False
    for i in range(len(st) - 1):
        if st[i] < st[i + 1]:
            return False
    return True


def elem_idx_to_addr(rev_shape, rev_strides, rev_max_shape, arg, index_value=None):
    """dimensions.clj:226-252.  ``index_value(entry, i)`` reads entry i of an index tensor."""
    offset = 0
    for d in range(len(rev_shape)):
        entry = rev_shape[d]
        nxt_max = int(rev_max_shape[d])
        dim = disambiguate_shape_entry(entry)
        idx = arg % dim
        if not _is_number(entry):
            idx = int(index_value(entry, idx))
        offset += int(rev_strides[d]) * idx
        arg //= nxt_max
    return offset


def _max_extend_strides(shp, st, max_count):
    """dimensions.clj:279-299 -- left-pad strides with stride*extent of the largest-stride dim."""
    shp = disambiguate_shape(shp)
    max_idx = 0
    for i in range(1, len(shp)):
        if st[i] > st[max_idx]:
            max_idx = i
    stride_val = st[max_idx] * shp[max_idx] if shp else 1
    return [stride_val] * (max_count - len(st)) + list(st)


def dimension_seq_to_max_shape(*dims_seq):
    """dimensions.clj:326-353."""
    for d in dims_seq:
        if len(d["shape"]) != len(d["strides"]):
            raise DimensionError("Some dimensions have different shape and stride counts")
    max_count = max([0] + [len(d["shape"]) for d in dims_seq])
    new_strides = [_max_extend_strides(d["shape"], d["strides"], max_count) for d in dims_seq]
    new_shapes = [[1] * (max_count - len(d["shape"])) + list(d["shape"]) for d in dims_seq]
    max_shape = [max([0] + [disambiguate_shape_entry(s[i]) for s in new_shapes]) for i in range(max_count)]
    return {"max-shape": max_shape,
            "dimensions": [{"shape": s, "strides": t} for s, t in zip(new_shapes, new_strides)]}


def minimize(dims):
    """dimensions.clj:356-383 -- drop unit dims, merge densely packed neighbours."""
    stripped = [(s, t) for s, t in zip(dims["shape"], dims["strides"]) if not (_is_number(s) and s == 1)]
    if not stripped:
        return {"shape": [1], "strides": [1]}
    rev = list(reversed(stripped))
    out = [rev[0]]
    for (cur_shp, cur_str), (last_shp, last_str) in zip(rev[1:], rev[:-1]):
        if _is_number(last_shp) and cur_str == last_shp * last_str:
            s_shp, s_str = out[-1]
            out[-1] = (s_shp * cur_shp, s_str)
        else:
            out.append((cur_shp, cur_str))
    out = list(reversed(out))
    return {"shape": [p[0] for p in out], "strides": [p[1] for p in out]}


def in_place_reshape(existing, new_shape):
    """dimensions.clj:386-470."""
    new_shape = list(new_shape)
    new_dims = dimensions(new_shape)
    if not ecount(new_dims) <= ecount(existing):
        raise DimensionError("Reshaped dimensions are larger than tensor")
    if access_increasing(existing) and dense(existing):
        return {"shape": new_shape, "strides": extend_strides(new_shape, [])}
    if access_increasing(existing):
        ex = minimize(existing)
        info = [list(p) for p in zip(reversed(ex["shape"]), reversed(ex["strides"]))]
        old_count = len(info)
        rev_shape = list(reversed(new_shape))
        rev_new_strides = []
        new_idx = old_idx = 0
        while new_idx < len(new_shape):
            old_dim, old_stride = info[min(old_idx, old_count - 1)]
            new_dim = rev_shape[new_idx]
            if not (old_idx < old_count or new_dim == 1):
                raise DimensionError("Ran out of old shape dimensions")
            if new_dim == 1:
                prev_stride = rev_new_strides[-1] if rev_new_strides else 1
                prev_dim = rev_shape[new_idx - 1] if new_idx >= 1 else 1
                rev_new_strides.append(prev_stride * prev_dim)
                new_idx += 1
            elif old_dim == new_dim:
                rev_new_strides.append(old_stride)
                new_idx += 1
                old_idx += 1
            elif old_dim < new_dim:
                raise DimensionError("Cannot combine dimensions across padded boundaries")
            else:
                if old_dim % new_dim != 0:
                    raise DimensionError("New dimension not commensurate with old dimension")
                info[old_idx] = [old_dim // new_dim, old_stride * new_dim]
                rev_new_strides.append(old_stride)
                new_idx += 1
        return {"shape": new_shape, "strides": extend_strides(new_shape, list(reversed(rev_new_strides)))}
    raise DimensionError("Cannot (at this point) in-place-reshape transposed or indirect dimensions")


def transpose(dims, reorder):
    """dimensions.clj:473-484."""
    if len(set(reorder)) != len(dims["shape"]):
        raise DimensionError("Every dimension must be represented in the reorder vector")
    return {"shape": [dims["shape"][i] for i in reorder], "strides": [dims["strides"][i] for i in reorder]}


ALL = "all"


def select(dims, *args, index_value=None):
    """dimensions.clj:487-569.  Each arg: ALL, an int, a contiguous increasing
    list of ints, or a 1-d index tensor.  Returns {"dimensions", "elem-offset"}."""
    data_shp = shape(dims)
    if len(data_shp) != len(args):
        raise DimensionError("arg count must match shape count")
    norm = []
    for dim, arg in zip(dims["shape"], args):
        if isinstance(arg, str) and arg == ALL:
            norm.append(list(range(disambiguate_shape_entry(dim))))
        elif isinstance(arg, (list, tuple, range)):
            arg = list(arg)
            if not all(arg[i] < arg[i + 1] for i in range(len(arg) - 1)):
                raise DimensionError("Argument is not monotonicly increasing")
            if not disambiguate_shape_entry(dim) > max([0] + arg):
                raise DimensionError("Argument out of range of dimension")
            norm.append(arg)
        elif _is_number(arg):
            norm.append(arg)
        elif hasattr(arg, "ecount") and hasattr(arg, "shape"):
            if len(arg.shape()) != 1:
                raise DimensionError("Index arguments must be vectors")
            norm.append(arg)
        else:
            raise DimensionError("argument to select of incorrect type")
    rev_args = list(reversed(norm))
    rev_shape = list(reversed(dims["shape"]))
    rev_strides = list(reversed(dims["strides"]))
    products = []
    for item in rev_shape:
        products.append(disambiguate_shape_entry(item) * (products[-1] if products else 1))
    first_idx = 0
    for arg, prev in zip(rev_args, [None] + products):
        first = arg if _is_number(arg) else (arg[0] if isinstance(arg, list) else 0)
        first_idx += (prev or 1) * first
    elem_addr = elem_idx_to_addr(rev_shape, rev_strides, rev_shape, first_idx, index_value)
    kept = [(a, s) for a, s in zip(rev_args, rev_strides) if not _is_number(a)]
    new_strides = list(reversed([s for _, s in kept]))
    new_shape = list(reversed([len(a) if isinstance(a, list) else a for a, _ in kept]))
    return {"dimensions": {"shape": new_shape, "strides": new_strides}, "elem-offset": elem_addr}


def to_wire(dims, index_pointer=None):
    """The 5-padded reversed form the device consumes (dimensions->cuda,
    src/cortex/compute/cuda/tensor_math.clj:34-51): shape padded with 1,
    strides padded with the outermost stride, one index pointer (or 0) per dim.
    ``index_pointer(tensor)`` returns the device address of an int32 index tensor."""
    shp, st = list(dims["shape"]), list(dims["strides"])
    if len(shp) > 5:
        raise DimensionError("at most 5 dimensions are supported")
    rev_complex = list(reversed(shp)) + [1] * (5 - len(shp))
    rev_shape = disambiguate_shape(rev_complex)
    rev_strides = list(reversed(st)) + [st[0] if st else 1] * (5 - len(st))
    ptrs = [0 if _is_number(e) else int(index_pointer(e)) for e in rev_complex]
    return rev_shape, rev_strides, ptrs
