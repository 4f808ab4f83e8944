"""Worker of tests/test_gpu_multi.py: one process per GPU (launched by torch.distributed.run).

Checks on every rank that the column-sharded last layer gives the same probabilities through
(a) the NCCL all-gather path and (b) the fused GEMM -> peer-store path, and that both match a
float64 numpy evaluation of softmax(h . W^T + b).  Exits non-zero on any mismatch.
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def main():
    import torch
    import torch.distributed as dist
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", local))
    from cortex_b200 import tensor as ct
    from cortex_b200.driver import driver
    from cortex_b200.parallel import (PeerLogits, column_sharded_head, column_sharded_head_fused, shard_bounds,
                                      stream_fence)
    dev = driver().get_devices()[local]
    stream = dev.create_stream()
    failures = []
    for datatype, tol in (("float", 1e-4), ("double", 1e-12)):
        npdt = np.float32 if datatype == "float" else np.float64
        for B, k, n_total in ((300, 512, 40 * world), (1024, 1024, 1000 if 1000 % world == 0 else 96 * world)):
            rng = np.random.default_rng(900 + B)
            h = rng.standard_normal((B, k)).astype(npdt)
            w = (rng.standard_normal((n_total, k)) * np.sqrt(2.0 / k)).astype(npdt)
            b = (rng.standard_normal(n_total) * 0.1).astype(npdt)
            logits = h.astype(np.float64) @ w.astype(np.float64).T + b
            e = np.exp(logits - logits.max(axis=1, keepdims=True))
            want = e / e.sum(axis=1, keepdims=True)
            lo, hi = shard_bounds(n_total, world, rank)
            with ct.with_stream(stream), ct.with_datatype(datatype):
                ht, ws, bs = ct.to_tensor(h), ct.to_tensor(w[lo:hi]), ct.to_tensor(b[lo:hi])
                got_nccl = ct.to_array(column_sharded_head(ht, ws, bs, n_total, world, rank)).reshape(B, n_total)
                exchange = PeerLogits(dev, B, n_total, world, rank, datatype)
                fence = stream_fence(stream)
                fence()                                   # nobody writes before every rank has mapped the buffers
                for _ in range(2):                        # twice: the buffers are reused
                    probs = column_sharded_head_fused(ht, ws, bs, exchange, fence)
                    got_fused = ct.to_array(probs).reshape(B, n_total)
                    fence()                               # peers may overwrite the logits only after everyone has read
                    stream.sync()
                stream.sync()
                dist.barrier()
                exchange.close()
            for name, got in (("nccl", got_nccl), ("fused", got_fused)):
                err = float(np.abs(got - want).max() / max(np.abs(want).max(), np.sqrt((want ** 2).mean())))
                if not err <= tol:
                    failures.append("%s %s B=%d n=%d: err %.3e > %.1e" % (datatype, name, B, n_total, err, tol))
    dist.barrier()
    dist.destroy_process_group()
    if failures:
        print("rank %d FAILED:\n  %s" % (rank, "\n  ".join(failures)), flush=True)
        sys.exit(1)
    print("rank %d ok" % rank, flush=True)


if __name__ == "__main__":
    main()
