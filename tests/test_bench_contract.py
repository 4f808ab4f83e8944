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


def test_clock_sampler_keeps_the_samples_of_the_marked_region():
    """The sampler starts before the warm-up (nvidia-smi needs a moment to deliver); only lines that arrived inside
    the marked region count, the nearest one when the region was shorter than a sampling period."""
    b = _bench()

    class _Done:
        def terminate(self):
            pass

        def wait(self, timeout=None):
            return 0

    def line(mhz, cap):
        return "0, %d, 1965, 700.0, 0x4, Not Active, Not Active, Not Active, %s" % (mhz, cap)

    s = b.ClockSampler(0)
    s.proc = _Done()
    s.lines = [(10.00, line(345, "Not Active")), (10.02, line(1965, "Not Active")), (10.04, line(1440, "Active")),
               (10.06, line(1460, "Active")), (10.30, line(345, "Not Active"))]
    s.t_begin, s.t_end = 10.03, 10.07
    got = s.stop()
    assert got["samples"] == 2 and got["sm_mhz"] == 1450.0 and got["reasons"] == ["sw_power_cap"]
    s = b.ClockSampler(0)
    s.proc = _Done()
    s.lines = [(10.00, line(345, "Not Active")), (10.20, line(1965, "Not Active"))]
    s.t_begin, s.t_end = 10.17, 10.171            # nothing arrived inside: the nearest sample
    got = s.stop()
    assert got["samples"] == 1 and got["sm_mhz"] == 1965.0
    s = b.ClockSampler(0)
    s.proc = _Done()
    s.lines = [(1.0, line(1500, "Active")), (2.0, line(1700, "Active"))]       # unmarked: everything counts
    assert s.stop()["samples"] == 2
