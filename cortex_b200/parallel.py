"""Multi-GPU partitioning of the dense-inference path (one process per GPU).

The reference has no multi-device code (README.md:48 lists it as future work);
this module adds exactly what the path needs:

* batch sharding -- every op on the path is independent across rows, so rank r
  takes rows [r*B/g, (r+1)*B/g) with weights replicated and NO collective;
* a column-sharded last layer for outputs too wide for one device: rank r owns
  W_r = W[r*n/g:(r+1)*n/g, :], computes logits_r = h . W_r^T, and the shards are
  exchanged with ONE all-gather (NCCL over NVLink on GPUs, gloo on CPU tests).
  The gathered buffer [g, B, n/g] is read through the rank-3 descriptor
  {shape [B, g, n/g], strides [n/g, B*n/g, 1]} -- the kind of view cortex's
  dimension/stride descriptors express -- and made dense with one assign!
  before softmax!, which (like the reference's, src/cortex/tensor.clj:903-917)
  wants non-increasing strides.

``torch.distributed`` is plumbing only: rendezvous, barrier, the all-gather.
"""
import numpy as np

from . import dimensions as dims
from . import tensor as ct
from ._lib import NUMPY_NAME


def shard_bounds(total, world_size, rank):
    """Rows (or columns) [lo, hi) of rank `rank`; the remainder goes to the first ranks."""
    if not (0 <= rank < world_size):
        raise ValueError("rank %d outside world of %d" % (rank, world_size))
    base, rem = divmod(int(total), int(world_size))
    lo = rank * base + min(rank, rem)
    return lo, lo + base + (1 if rank < rem else 0)


def weighted_shard_bounds(total, rates, quantum=1, keep_equal_within=0.0):
    """[lo, hi) for every rank with row counts proportional to `rates` (each rank's measured throughput), in
    multiples of `quantum` rows (the last rank takes the remainder), every rank keeping at least one quantum.
    Batch sharding is embarrassingly parallel, so ranks may own different amounts: on a box whose GPUs do not
    all get the same host-link bandwidth the host-fed pass ends when the slowest link ends, and rows in
    proportion to the rates make the links end together.  When the rates are within `keep_equal_within`
    (relative, max over min minus 1) of each other the even split of shard_bounds() is returned."""
    world = len(rates)
    total, quantum = int(total), max(1, int(quantum))
    if world < 1 or any(not (r > 0) for r in rates):
        raise ValueError("rates must be positive, one per rank")
    if max(rates) / min(rates) - 1.0 <= keep_equal_within or total < world * quantum:
        return [shard_bounds(total, world, r) for r in range(world)]
    units = total // quantum                                   # whole quanta to hand out
    share = [units * r / float(sum(rates)) for r in rates]
    counts = [max(1, int(sh)) for sh in share]
    # largest remainders first until the quanta are used up (or taken back where the floor of 1 overshot)
    order = sorted(range(world), key=lambda i: share[i] - int(share[i]), reverse=True)
    i = 0
    while sum(counts) < units:
        counts[order[i % world]] += 1
        i += 1
    while sum(counts) > units:
        j = max(range(world), key=lambda k: counts[k])
        counts[j] -= 1
    bounds, lo = [], 0
    for r in range(world):
        hi = total if r == world - 1 else lo + counts[r] * quantum
        bounds.append((lo, hi))
        lo = hi
    return bounds


def shard_rows(array, world_size, rank):
    lo, hi = shard_bounds(array.shape[0], world_size, rank)
    return array[lo:hi]


def _as_torch(buffer, shape):
    """A torch tensor aliasing a backend buffer (device memory through
    __cuda_array_interface__, oracle/host memory through numpy)."""
    import torch
    if buffer.host:
        return torch.from_numpy(buffer.as_numpy()).view(*shape)

    class _Cai:
        pass

    holder = _Cai()
    typestr = np.dtype(NUMPY_NAME[buffer.dtype]).str
    holder.__cuda_array_interface__ = {"data": (buffer.ptr, False), "shape": tuple(int(s) for s in shape),
                                       "typestr": typestr, "version": 2}
    return torch.as_tensor(holder, device="cuda:%d" % buffer.device.index)


_external_streams = {}


def _external(stream):
    """The backend stream as a torch stream (cached per stream handle), so that a torch.distributed
    collective can be enqueued ON it: ordered after the kernels already there, before the ones that
    follow, with no host synchronisation on either side."""
    import torch
    key = (stream.device.index, stream.native_handle())
    ext = _external_streams.get(key)
    if ext is None:
        ext = torch.cuda.ExternalStream(key[1], device=torch.device("cuda", key[0]))
        _external_streams[key] = ext
    return ext


def all_gather_buffers(local, gathered, world_size, group=None):
    """gathered[r] = rank r's `local` (both backend tensors, dense).  One collective, enqueued on the
    backend's own stream (NCCL), or run on the host after a stream sync (gloo, CPU tests)."""
    import torch.distributed as dist
    stream = ct.check_stream()
    n = local.ecount()
    src = _as_torch(local.buffer, [n])
    dst = _as_torch(gathered.buffer, [world_size * n])
    if dst.is_cuda:
        import torch
        with torch.cuda.stream(_external(stream)):
            dist.all_gather_into_tensor(dst, src, group=group)
    else:
        stream.sync()                  # host collective: the producers must have finished
        parts = [dst[r * n:(r + 1) * n] for r in range(world_size)]
        dist.all_gather(parts, src, group=group)
    return gathered


def column_sharded_head(h, w_shard, b_shard, n_total, world_size, rank, group=None, workspace=None):
    """softmax(h . W^T + b) where W[n_total, k] is split by output column across ranks.

    h        [B, k]            this rank's (replicated or gathered) activations
    w_shard  [n_total/g, k]    this rank's rows of W
    b_shard  [n_total/g]
    workspace  a dict the caller keeps between calls: the three intermediate tensors are then allocated
               once per shape instead of per call (allocation synchronises the device)
    returns  [B, n_total]      dense probabilities, identical on every rank
    """
    if n_total % world_size:
        raise ValueError("column sharding needs n_total divisible by the world size")
    B = h.shape()[0]
    per = n_total // world_size
    dt = h.get_datatype()
    bufs = workspace if workspace is not None else {}
    key = (B, per, world_size, dt)
    if bufs.get("key") != key:
        bufs.clear()
        bufs["key"] = key
        bufs["local"] = ct.new_tensor([B, per], datatype=dt, init_value=None)
        bufs["gathered"] = ct.new_tensor([world_size, B, per], datatype=dt, init_value=None)
        bufs["logits"] = ct.new_tensor([B, world_size, per], datatype=dt, init_value=None)
    local, gathered, logits = bufs["local"], bufs["gathered"], bufs["logits"]
    ct.assign(local, b_shard)
    ct.gemm(local, False, True, 1.0, h, w_shard, 1.0)
    all_gather_buffers(local, gathered, world_size, group)
    view = ct.Tensor(gathered.device, {"shape": [B, world_size, per], "strides": [per, B * per, 1]}, gathered.buffer)
    ct.assign(logits, view)                                   # strided gather through the index system
    logits2d = ct.in_place_reshape(logits, [B, n_total])
    return ct.softmax(logits2d, logits2d)


class PeerLogits:
    """The full [B, n_total] logits buffer of every rank, mapped into this rank's address space
    (CUDA IPC, one process per GPU), so that a column-sharded layer's GEMM can store its
    [B, n_total/g] window straight into all of them: no separate all-gather, the NVLink transfer
    overlaps the math tile by tile.  `torch.distributed` carries the 64-byte handles only."""

    def __init__(self, device, B, n_total, world_size, rank, datatype="float", group=None):
        import torch.distributed as dist
        if n_total % world_size:
            raise ValueError("column sharding needs n_total divisible by the world size")
        self.device, self.B, self.n_total, self.world, self.rank = device, B, n_total, world_size, rank
        self.per, self.datatype, self.group = n_total // world_size, datatype, group
        self.local = device.allocate_device_buffer(B * n_total, datatype)
        handles = [None] * world_size
        dist.all_gather_object(handles, self.local.ipc_export(), group=group)
        self.remote = {r: device.ipc_import(handles[r], B * n_total, datatype) for r in range(world_size) if r != rank}
        self.tensor = ct.Tensor(device, dims.dimensions([B, n_total]), self.local)

    def window_ptrs(self):
        """Address of this rank's column window inside every OTHER rank's logits buffer."""
        from ._lib import DTYPE_SIZE
        off = self.rank * self.per * DTYPE_SIZE[self.datatype]
        return [self.remote[r].ptr + off for r in sorted(self.remote)]

    def close(self):
        for buf in self.remote.values():
            self.device.ipc_close(buf)
        self.remote = {}


def column_sharded_head_fused(h, w_shard, b_shard, exchange, fence):
    """column_sharded_head without the all-gather and the re-layout: ONE fused kernel computes this
    rank's logits window (bias added in the epilogue) and stores it into every rank's full logits
    buffer over NVLink; `fence()` must then order all ranks (every rank's kernel finished) before
    softmax! runs on the local full buffer.  Returns the [B, n_total] probabilities tensor.

    softmax! runs IN PLACE on the buffer the peers store into.  Before this function is called again
    with the same `exchange`, the caller must issue one more `fence()` after it has consumed the
    probabilities: otherwise a faster rank's next GEMM overwrites this rank's logits while its softmax
    (or its reader) is still on them."""
    stream = ct.check_stream()
    B, k = h.shape()
    per, n_total = exchange.per, exchange.n_total
    window = exchange.local.sub_buffer(exchange.rank * per, B * n_total - exchange.rank * per)
    stream.gemm_bias_act_peers(window, n_total, False, True, 1.0, h.buffer, B, k, h.dimensions["strides"][0],
                               w_shard.buffer, per, w_shard.dimensions["strides"][0], 0.0, b_shard.buffer, None,
                               exchange.window_ptrs())
    fence()
    return ct.softmax(exchange.tensor, exchange.tensor)


def stream_fence(stream, group=None):
    """A cross-rank fence enqueued on the backend's own stream: a one-element all-reduce issued
    with that stream current, so later kernels on it start only after every rank's earlier kernels
    (and their peer stores) are complete.  No host synchronisation."""
    import torch
    import torch.distributed as dist
    ext = _external(stream)
    token = torch.zeros(1, device=ext.device, dtype=torch.float32)

    def fence():
        with torch.cuda.stream(ext):
            dist.all_reduce(token, group=group)

    return fence
