"""Multi-GPU data path on real devices: fused GEMM -> peer stores.

The one-device tests run wherever a GPU is present; the rest need at least two GPUs on the box
and skip otherwise (the world-size-2 host logic is also covered on CPU in test_parallel_gloo.py).
"""
import os
import subprocess
import sys

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _devices():
    from cortex_b200.driver import driver
    return driver().get_devices()


def _rel_err(got, want):
    want = np.asarray(want, np.float64)
    return float(np.abs(np.asarray(got, np.float64) - want).max() / max(np.abs(want).max(), np.sqrt((want ** 2).mean())))


@pytest.mark.parametrize("datatype,tol", [("float", 1e-4), ("double", 1e-12)])
@pytest.mark.parametrize("M,K,N,ld,col0,n_peers", [(300, 256, 200, 1000, 400, 2), (128, 64, 125, 1000, 125, 3),
                                                   (512, 512, 256, 1024, 512, 7), (100, 30, 17, 53, 5, 1),
                                                   # few tiles, long reductions: the K slices of a tile (one
                                                   # cluster, or through L2) finish the peer stores as well
                                                   (1024, 4096, 125, 1000, 125, 3), (1024, 4096, 248, 1000, 248, 2),
                                                   (256, 2048, 64, 256, 64, 2)])
def test_gemm_epilogue_stores_to_every_destination(datatype, tol, M, K, N, ld, col0, n_peers):
    """All destinations on ONE device: the epilogue writes the same window of each, and nothing else."""
    from cortex_b200 import tensor as ct
    dev = _devices()[0]
    stream = dev.create_stream()
    npdt = np.float32 if datatype == "float" else np.float64
    rng = np.random.default_rng(77)
    a = rng.standard_normal((M, K)).astype(npdt)
    w = rng.standard_normal((N, K)).astype(npdt)
    bias = rng.standard_normal(N).astype(npdt)
    want = np.maximum(a.astype(np.float64) @ w.astype(np.float64).T + bias, 0.0)
    with ct.with_stream(stream), ct.with_datatype(datatype):
        at, wt, bt = ct.to_tensor(a), ct.to_tensor(w), ct.to_tensor(bias)
        frames = [ct.to_tensor(np.full((M, ld), -7.0, npdt)) for _ in range(n_peers + 1)]
        windows = [f.buffer.sub_buffer(col0, M * ld - col0) for f in frames]
        stream.gemm_bias_act_peers(windows[0], ld, False, True, 1.0, at.buffer, M, K, K, wt.buffer, N, K, 0.0,
                                   bt.buffer, "relu", [wd.ptr for wd in windows[1:]])
        for f in frames:
            got = ct.to_array(f).reshape(M, ld)
            assert _rel_err(got[:, col0:col0 + N], want) <= tol
            frame = got.copy()
            frame[:, col0:col0 + N] = -7.0
            assert np.all(frame == -7.0)           # outside the window: untouched


def test_peer_list_validation():
    from cortex_b200 import _lib
    from cortex_b200 import tensor as ct
    dev = _devices()[0]
    stream = dev.create_stream()
    with ct.with_stream(stream), ct.with_datatype("float"):
        t = ct.new_tensor([4, 4])
        with pytest.raises(_lib.B200Error):
            stream.gemm_bias_act_peers(t.buffer, 4, False, True, 1.0, t.buffer, 4, 4, 4, t.buffer, 4, 4, 0.0, None,
                                       None, [t.buffer.ptr] * 8)
        with pytest.raises(_lib.B200Error):
            dev.enable_peer(dev)


def test_two_devices_one_process_peer_stores():
    """One process, two GPUs (the JVM deployment): each device's GEMM stores its column window into
    both devices' full buffers; both end up with the whole matrix."""
    devs = _devices()
    if len(devs) < 2:
        pytest.skip("needs two GPUs")
    from cortex_b200 import tensor as ct
    d0, d1 = devs[0], devs[1]
    d0.enable_peer(d1)
    d1.enable_peer(d0)
    s0, s1 = d0.create_stream(), d1.create_stream()
    B, k, n = 512, 1024, 512
    rng = np.random.default_rng(5)
    h = rng.standard_normal((B, k)).astype(np.float32)
    w = (rng.standard_normal((n, k)) * 0.05).astype(np.float32)
    want = h.astype(np.float64) @ w.astype(np.float64).T
    full, parts = {}, {}
    for dev, stream in ((d0, s0), (d1, s1)):
        with ct.with_stream(stream), ct.with_datatype("float"):
            full[dev.index] = ct.to_tensor(np.zeros((B, n), np.float32))
            parts[dev.index] = (ct.to_tensor(h), ct.to_tensor(w[:n // 2] if dev is d0 else w[n // 2:]))
    s0.sync()
    s1.sync()
    for r, (dev, stream, other) in enumerate(((d0, s0, d1), (d1, s1, d0))):
        ht, wt = parts[dev.index]
        off = r * (n // 2)
        mine = full[dev.index].buffer.sub_buffer(off, B * n - off)
        theirs = full[other.index].buffer.sub_buffer(off, B * n - off)
        stream.gemm_bias_act_peers(mine, n, False, True, 1.0, ht.buffer, B, k, k, wt.buffer, n // 2, k, 0.0, None, None,
                                   [theirs.ptr])
    s0.sync()
    s1.sync()
    for dev, stream in ((d0, s0), (d1, s1)):
        with ct.with_stream(stream):
            assert _rel_err(ct.to_array(full[dev.index]).reshape(B, n), want) <= 1e-4


def test_column_sharded_head_two_processes():
    """One process per GPU: NCCL all-gather path and fused peer-store path against numpy."""
    if len(_devices()) < 2:
        pytest.skip("needs two GPUs")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr",
           "127.0.0.1", "--master-port", "29541", os.path.join(ROOT, "tests", "mp_column_head.py")]
    res = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)
    assert res.returncode == 0, res.stdout[-3000:] + res.stderr[-3000:]
