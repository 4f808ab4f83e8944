"""bench.py's host-side logic that needs no GPU: rank -> GPU placement and the workload description the two arms
share."""
import importlib.util
import os

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _bench():
    spec = importlib.util.spec_from_file_location("bench_module", os.path.join(ROOT, "bench.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def test_ranks_are_spread_over_the_visible_gpus():
    b = _bench()
    assert [b.rank_device(r, 1, 8) for r in range(1)] == [0]
    assert [b.rank_device(r, 2, 8) for r in range(2)] == [0, 4]
    assert [b.rank_device(r, 4, 8) for r in range(4)] == [0, 2, 4, 6]
    assert [b.rank_device(r, 8, 8) for r in range(8)] == list(range(8))
    assert [b.rank_device(r, 2, 2) for r in range(2)] == [0, 1]          # exactly `world` GPUs visible: identity
    assert [b.rank_device(r, 4, 6) for r in range(4)] == [0, 1, 2, 3]    # stride 1 when they do not divide
    assert [b.rank_device(r, 4, 2) for r in range(4)] == [0, 1, 2, 3]    # more ranks than GPUs: left to the launcher


def test_both_arms_describe_the_same_workload():
    b = _bench()
    for world in (1, 2, 8):
        cfg = b.workload_config(world)
        assert cfg["global_batch"] == b.BATCH and "wide_mlp" in cfg["workload"]
        assert cfg["parallelism"] == "batch-shard x%d" % world
