"""Multi-rank host logic on CPU: world_size-2 gloo ranks running the oracle backend.

Covers what bench.py --gpus N relies on: shard bounds, batch-sharded inference being a
row-wise concatenation of the single-rank result, and the column-sharded last layer
(one all-gather + strided descriptor view) matching the unsharded head."""
import os
import socket
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _inputs():
    rng = np.random.default_rng(77)
    X = rng.standard_normal((12, 32)).astype(np.float32)
    W1 = (rng.standard_normal((32, 32)) * 0.25).astype(np.float32)
    b1 = (rng.standard_normal(32) * 0.1).astype(np.float32)
    W2 = (rng.standard_normal((20, 32)) * 0.25).astype(np.float32)
    b2 = (rng.standard_normal(20) * 0.1).astype(np.float32)
    return X, W1, b1, W2, b2


def _reference():
    X, W1, b1, W2, b2 = _inputs()
    h = np.maximum(X.astype(np.float64) @ W1.astype(np.float64).T + b1, 0)
    z = h @ W2.astype(np.float64).T + b2
    e = np.exp(z - z.max(axis=1, keepdims=True))
    return e / e.sum(axis=1, keepdims=True)


def _worker(rank, world, port, out_dir):
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from cortex_b200 import nn, parallel
    from cortex_b200 import tensor as ct
    from oracle.cpu_backend import OracleDriver
    X, W1, b1, W2, b2 = _inputs()
    stream = OracleDriver().default_device().create_stream()
    with ct.with_stream(stream), ct.with_datatype("float"):
        # 1. batch sharding: this rank's rows through the replicated network
        net = nn.MLP([(ct.to_tensor(W1), ct.to_tensor(b1), "relu"), (ct.to_tensor(W2), ct.to_tensor(b2), "softmax")])
        lo, hi = parallel.shard_bounds(X.shape[0], world, rank)
        local = ct.to_array(net.infer(ct.to_tensor(X[lo:hi]))).reshape(hi - lo, 20)
        # 2. column-sharded head on replicated activations
        h = ct.new_tensor([X.shape[0], 32])
        nn.Linear(ct.to_tensor(W1), ct.to_tensor(b1)).forward(ct.to_tensor(X), h)
        nn.relu(h, h)
        clo, chi = parallel.shard_bounds(20, world, rank)
        probs = parallel.column_sharded_head(h, ct.to_tensor(W2[clo:chi]), ct.to_tensor(b2[clo:chi]), 20, world, rank)
        full = ct.to_array(probs).reshape(X.shape[0], 20)
    np.save(os.path.join(out_dir, "local_%d.npy" % rank), local)
    np.save(os.path.join(out_dir, "full_%d.npy" % rank), full)
    dist.barrier()
    dist.destroy_process_group()


def test_shard_bounds_cover_everything():
    from cortex_b200.parallel import shard_bounds
    for total in (0, 1, 7, 65536, 1000):
        for world in (1, 2, 3, 8):
            spans = [shard_bounds(total, world, r) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == total
            assert all(spans[i][1] == spans[i + 1][0] for i in range(world - 1))
            sizes = [b - a for a, b in spans]
            assert max(sizes) - min(sizes) <= 1
    with pytest.raises(ValueError):
        shard_bounds(10, 2, 2)


def test_two_gloo_ranks_match_single_rank(tmp_path):
    world = 2
    port = _free_port()
    mp.spawn(_worker, args=(world, port, str(tmp_path)), nprocs=world, join=True)
    ref = _reference()
    locals_ = [np.load(tmp_path / ("local_%d.npy" % r)) for r in range(world)]
    assert np.max(np.abs(np.concatenate(locals_, axis=0) - ref)) <= 1e-5
    for r in range(world):
        full = np.load(tmp_path / ("full_%d.npy" % r))
        assert np.max(np.abs(full - ref)) <= 1e-5          # identical probabilities on every rank
    assert np.array_equal(np.load(tmp_path / "full_0.npy"), np.load(tmp_path / "full_1.npy"))


def test_weighted_shard_bounds():
    from cortex_b200.parallel import shard_bounds, weighted_shard_bounds
    # the host-link rates seen on an 8-GPU box: GPUs 0-3 at ~20 GB/s, 4-7 at ~29 GB/s
    rates = [20.0] * 4 + [29.0] * 4
    spans = weighted_shard_bounds(65536, rates, quantum=512)
    assert spans[0][0] == 0 and spans[-1][1] == 65536
    assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
    sizes = [hi - lo for lo, hi in spans]
    assert all(sz % 512 == 0 and sz > 0 for sz in sizes)
    assert abs(sizes[0] / 65536 - 20.0 / 196.0) < 0.01 and abs(sizes[7] / 65536 - 29.0 / 196.0) < 0.01
    # rates within the tolerance: the even split
    assert weighted_shard_bounds(1000, [1.0, 1.04, 0.99], 8, keep_equal_within=0.08) == [shard_bounds(1000, 3, r) for r in range(3)]
    # a rank that is almost idle keeps one quantum; the remainder (total not a multiple of the quantum) goes last
    spans = weighted_shard_bounds(1003, [1e-3, 1.0, 1.0], 8)
    assert spans[0] == (0, 8) and spans[-1][1] == 1003 and all(hi > lo for lo, hi in spans)
    for total, rates, q in ((7, [1.0, 2.0], 1), (4096, [3.0, 1.0, 1.0, 1.0], 256), (100, [5.0, 1.0], 64)):
        spans = weighted_shard_bounds(total, rates, q)
        assert spans[0][0] == 0 and spans[-1][1] == total and all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
        assert all(hi > lo for lo, hi in spans)
    with pytest.raises(ValueError):
        weighted_shard_bounds(10, [1.0, 0.0])
