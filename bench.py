#!/usr/bin/env python
"""bench.py -- headline benchmark of the B200 backend.

Workload (the configuration the multi-GPU half of the headline metric is quoted
on): wide MLP batch inference, fp32, batch 65536 x 4096 -> 4 x (linear
4096->4096 + ReLU) -> linear 4096->1000 + softmax, He-normal weights from fixed
seeds, zero biases, batch-sharded over the GPUs with replicated weights (strong
scaling on the same 65536 rows).  One step = one forward pass over this rank's
shard.  `value` = samples/s with the shard resident in HBM; `e2e` = the same
pass through the host-buffer pipeline (pinned host input -> H2D -> layers ->
D2H of the probabilities, every step).  The other half of the headline metric,
the standalone 4096^3 fp32 gemm!, and the HBM-bound elementwise / reduce kernels
are reported in the `gemm_4096` / `eltwise` objects of the same line (N=1 only).

  python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time


def _host_cores():
    try:
        return len(os.sched_getaffinity(0))
    except (AttributeError, OSError):
        return os.cpu_count() or 1


if "--impl" in sys.argv and "reference" in sys.argv:
    # The CPU arm uses every host core it may run on.  torch.distributed.run exports OMP_NUM_THREADS=1 to
    # its workers; OpenBLAS and the OpenMP runtime read these variables when they are loaded, so they are
    # set here, before numpy is imported.
    for _var in ("OMP_NUM_THREADS", "OPENBLAS_NUM_THREADS"):
        os.environ[_var] = str(_host_cores())

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

BATCH, WIDTH, CLASSES, HIDDEN_LAYERS = 65536, 4096, 1000, 4
SEED_X, SEED_W = 501, 502
FLOPS_PER_SAMPLE = 2.0 * (HIDDEN_LAYERS * WIDTH * WIDTH + WIDTH * CLASSES)
CPU_SAMPLE_ROWS = 8192        # rows of the batch the CPU arm runs per step (one 8-GPU shard)


def workload_config(world, dt="float"):
    """The `config` object: the same for the B200 arm and for the CPU reference arm."""
    prec = "fp32" if dt == "float" else "fp64"
    return {"workload": "wide_mlp: batch 65536 x 4096 -> 4 x (linear 4096 + ReLU) -> linear 1000 + softmax, %s, "
                        "He-normal weights (seeds 502-506), zero biases, batch-sharded, weights replicated" % prec,
            "global_batch": BATCH, "parallelism": "batch-shard x%d" % world,
            "l2": "inputs larger than L2 (every layer streams >= %d MiB of activations per GPU)"
                  % ((BATCH // max(world, 1)) * WIDTH * 4 >> 20)}


def rank_device(local_rank, world, visible):
    """GPU index a local rank uses: ranks spread evenly over the visible GPUs (stride = visible // world)."""
    if 1 < world <= visible:
        return local_rank * (visible // world)
    return local_rank


def threads_in_use():
    """Thread counts the loaded BLAS / OpenMP runtimes report (what the CPU arm really ran on)."""
    try:
        import threadpoolctl
        info = threadpoolctl.threadpool_info()
        return {"%s:%s" % (i.get("user_api"), i.get("internal_api")): i.get("num_threads") for i in info}
    except Exception as exc:      # reporting only
        return {"error": repr(exc)}


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        p = json.load(open(path))
        return {"hbm_gbs": p["hbm_gbs"], "bf16_burst": p["bf16_tflops"], "bf16_sustained": p["bf16_tflops_sustained"],
                "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_burst": 1590.0, "bf16_sustained": 1400.0, "source": "fallback"}


def measure_library_peaks(device_index, sustained_s=4.0):
    """MEASUREMENT ONLY -- never on the product path.  The library matmul (torch.matmul -> cuBLAS) timed the way
    MEASURED_PEAKS.json was (best of 10 = burst; back to back for `sustained_s` seconds = sustained, CUDA
    events on torch's stream): fp32 with TF32 tensor cores (the 3xTF32 roofline is this / 3), fp32 without
    (the CUDA-core SGEMM the reference's cuBLAS 8 would run), and fp64.  8192^3, 2*N^3 flop."""
    import torch
    dev = torch.device("cuda", device_index)
    n = 8192
    flop = 2.0 * n ** 3

    def set_tf32(on):
        try:
            torch.backends.cuda.matmul.fp32_precision = "tf32" if on else "ieee"
        except Exception:
            torch.backends.cuda.matmul.allow_tf32 = bool(on)

    def run(dtype, tf32, sustained):
        set_tf32(tf32)
        with torch.cuda.device(dev):
            a = torch.randn(n, n, device=dev, dtype=dtype)
            b = torch.randn(n, n, device=dev, dtype=dtype)
            c = torch.empty_like(a)
            for _ in range(3):
                torch.matmul(a, b, out=c)
            torch.cuda.synchronize(dev)
            best = None
            for _ in range(10):
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                torch.matmul(a, b, out=c)
                e1.record()
                e1.synchronize()
                ms = e0.elapsed_time(e1)
                best = ms if best is None else min(best, ms)
            out = {"burst_tflops": round(flop / best / 1e9, 1)}
            if sustained:
                per = max(1, int(0.25 * 1000.0 / best))       # launches per quarter second
                total_ms, count = 0.0, 0
                while total_ms < sustained * 1000.0:
                    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                    e0.record()
                    for _ in range(per):
                        torch.matmul(a, b, out=c)
                    e1.record()
                    e1.synchronize()
                    total_ms += e0.elapsed_time(e1)
                    count += per
                out["sustained_tflops"] = round(flop * count / total_ms / 1e9, 1)
            del a, b, c
        return out

    res = {"how": "torch.matmul 8192^3 (cuBLAS), best of 10 and back to back for %.0f s, CUDA events; "
                  "measurement only" % sustained_s}
    try:
        res["fp32_tf32"] = run(torch.float32, True, sustained_s)
        res["fp32_no_tf32"] = run(torch.float32, False, 0)
        res["fp64"] = run(torch.float64, False, sustained_s)
    except Exception as exc:
        res["error"] = repr(exc)
    finally:
        set_tf32(False)
        torch.cuda.empty_cache()
    return res


def rooflines(peaks, lib):
    """Denominators: 3xTF32 = measured library TF32 rate / 3 (three MMAs per product); fp64 = measured library
    dgemm rate.  Falls back to the bf16-derived proxy / the nominal fp64 figure when the measurement is missing."""
    out = {"source": {}}
    tf = (lib or {}).get("fp32_tf32")
    if tf and "sustained_tflops" in tf:
        out["tf32x3_burst"], out["tf32x3_sustained"] = tf["burst_tflops"] / 3.0, tf["sustained_tflops"] / 3.0
        out["source"]["tf32x3"] = "measured in this run: library fp32 matmul with TF32 on, / 3"
    else:
        out["tf32x3_burst"], out["tf32x3_sustained"] = peaks["bf16_burst"] / 6.0, peaks["bf16_sustained"] / 6.0
        out["source"]["tf32x3"] = "%s bf16 / 2 (tf32 rate) / 3 (proxy: no TF32 measurement in this run)" % peaks["source"]
    f64 = (lib or {}).get("fp64")
    if f64 and "sustained_tflops" in f64:
        out["fp64_burst"], out["fp64_sustained"] = f64["burst_tflops"], f64["sustained_tflops"]
        out["source"]["fp64"] = "measured in this run: library fp64 matmul"
    else:
        out["fp64_burst"] = out["fp64_sustained"] = 37.0
        out["source"]["fp64"] = "nominal B200 fp64 dense rate (no measurement in this run)"
    return out


def fp64_forward(x, weights):
    """float64 numpy forward of the benchmark network on a few rows: the arbiter of the parity figures."""
    h = x.astype(np.float64)
    for i, w in enumerate(weights):
        h = h @ w.astype(np.float64).T
        if i + 1 < len(weights):
            h = np.maximum(h, 0.0)
    e = np.exp(h - h.max(axis=1, keepdims=True))
    return e / e.sum(axis=1, keepdims=True)


def rel_err(got, ref):
    """max abs(got - ref) / max(abs(ref), rms(ref)) -- the measure the parity tests use."""
    ref = np.asarray(ref, np.float64)
    got = np.asarray(got, np.float64).reshape(ref.shape)
    rms = float(np.sqrt(np.mean(ref ** 2))) or 1.0
    return float(np.max(np.abs(got - ref) / np.maximum(np.abs(ref), rms)))


def make_weights():
    ws = []
    for i in range(HIDDEN_LAYERS + 1):
        out = WIDTH if i < HIDDEN_LAYERS else CLASSES
        w = np.random.default_rng(SEED_W + i).standard_normal((out, WIDTH), dtype=np.float32)
        w *= np.float32(np.sqrt(2.0 / WIDTH))
        ws.append(w)
    return ws


def make_input(lo, hi):
    """Rows [lo, hi) of the seeded N(0,1) batch, generated in 4096-row blocks so that any
    sharding sees the same global matrix."""
    out = np.empty((hi - lo, WIDTH), np.float32)
    blk = 4096
    for b0 in range(lo // blk * blk, hi, blk):
        rows = np.random.default_rng([SEED_X, b0 // blk]).standard_normal((blk, WIDTH), dtype=np.float32)
        s, e = max(lo, b0), min(hi, b0 + blk)
        out[s - lo:e - lo] = rows[s - b0:e - b0]
    return out


class ClockSampler:
    """nvidia-smi clocks / throttle reasons sampled every 20 ms while the timed regions run."""
    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.gpu_index, self.proc, self.lines = gpu_index, None, []
        self.t_begin = self.t_end = None

    def mark_begin(self):
        """The timed region starts now (the sampler was started earlier: nvidia-smi needs ~0.1-0.3 s to deliver its
        first line, longer than a short timed region lasts)."""
        self.t_begin = time.monotonic()

    def mark_end(self):
        self.t_end = time.monotonic()

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.gpu_index), "--query-gpu=" + self.FIELDS,
                                          "--format=csv,noheader,nounits", "-lms", "20"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append((time.monotonic(), line.strip()))

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            pass
        sm, mx, reasons = [], [], set()
        lines = self.lines
        if self.t_begin is not None and self.t_end is not None:
            # samples that arrived inside the marked region (a line describes the ~20 ms before it arrived)
            inside = [ln for ln in lines if self.t_begin <= ln[0] <= self.t_end + 0.025]
            if not inside and lines:
                # region shorter than the sampling period: the sample nearest to it
                mid = 0.5 * (self.t_begin + self.t_end)
                inside = [min(lines, key=lambda ln: abs(ln[0] - mid))]
            lines = inside
        for _t, line in lines:
            f = [x.strip() for x in line.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                mx.append(float(f[2]))
            except ValueError:
                continue
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        # under load = the upper half of the samples (the sampler also sees the idle edges)
        sm_sorted = sorted(sm)
        return {"sm_mhz": float(np.median(sm_sorted)) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "samples": len(sm), "reasons": sorted(reasons)}


# --------------------------------------------------------------------------------------
# reference arm: the CPU oracle (restatement of the reference's CPU backend) on host cores
# --------------------------------------------------------------------------------------

def cpu_arm(sample_rows, weights):
    """The oracle MLP forward (bias assign!, gemm! NT beta=1, ReLU binary-op!, softmax!: the reference's call
    sequence) on `sample_rows` rows of the workload.  Returns step() -> (samples/s, seconds) for one pass."""
    from cortex_b200 import nn
    from cortex_b200 import tensor as ct
    from oracle.cpu_backend import OracleDriver
    drv = OracleDriver()
    stream = drv.default_device().create_stream()
    x = make_input(0, sample_rows)
    with ct.with_stream(stream), ct.with_datatype("float"):
        layers = []
        for i, w in enumerate(weights):
            act = "softmax" if i == len(weights) - 1 else "relu"
            layers.append((ct.to_tensor(w), ct.to_tensor(np.zeros(w.shape[0], np.float32)), act))
        net = nn.MLP(layers, fused=False)
        xt = ct.to_tensor(x)
        net.infer(xt)   # touch buffers once

    def step():
        with ct.with_stream(stream), ct.with_datatype("float"):
            t0 = time.perf_counter()
            net.infer(xt)
            dt = time.perf_counter() - t0
        return sample_rows / dt, dt

    return step


def cpu_baseline_object(value, secs, sample):
    pools = threads_in_use()
    counts = [v for v in pools.values() if isinstance(v, int)]
    return {"value": value, "unit": "samples/s", "cores": max(counts) if counts else 1, "kind": "port",
            "host_cores_available": _host_cores(), "thread_pools": pools, "sample_rows": sample,
            "sample": "%d rows of the 65536-row batch per step (%.2f s per step), samples/s = rows / time; oracle "
                      "elementwise / softmax in C with OpenMP, gemm! through OpenBLAS sgemm; the reference itself is "
                      "Clojure on the JVM and cannot run here" % (sample, secs)}


def run_reference(args, rank, world):
    if rank != 0:
        return
    sample = CPU_SAMPLE_ROWS
    step = cpu_arm(sample, make_weights())
    for _ in range(args.warmup):
        step()
    t0 = time.perf_counter()
    rates = [step()[0] for _ in range(args.steps)]
    total = time.perf_counter() - t0
    value = float(np.mean(rates))
    line = {
        "impl": "reference", "metric": "wide_mlp_inference_samples_per_s", "value": value, "unit": "samples/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1000.0 * sample / value,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": workload_config(world),
        "cpu_baseline": cpu_baseline_object(value, sample / value, sample),
        "e2e": {"value": value, "unit": "samples/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0, "wall_s": total,
    }
    print(json.dumps(line), flush=True)


# --------------------------------------------------------------------------------------
# B200 arm
# --------------------------------------------------------------------------------------

def time_region(stream, fn, iters, prime=None):
    """Mean device time of `fn` over `iters` back-to-back calls, CUDA events on the launching stream.
    `prime` enqueues a few milliseconds of unrelated work first, so that the host runs ahead of the
    device and the timed launches are not spaced by host-side call overhead (short kernels only)."""
    if prime is not None:
        prime()
    e0 = stream.create_event(timing=True)
    for _ in range(iters):
        fn()
    e1 = stream.create_event(timing=True)
    e1.wait_for_event()
    stream.sync()
    return e1.elapsed_ms_since(e0) / iters


def bench_gemm_4096(drv, dev, roofs):
    """Config 2 in brief: C = 1.5*op(A)*op(B) + 0.5*C, 4096^3 fp32, all four transposes, on dense operands
    and on [4096, 4096] windows at (64, 64) of [4224, 4224] backing buffers (row pitch 4224)."""
    from cortex_b200 import tensor as ct
    stream = dev.create_stream()
    rng = np.random.default_rng(201)
    out, pitched = {}, {}
    combos = (("NT", False, True), ("NN", False, False), ("TN", True, False), ("TT", True, True))
    with ct.with_stream(stream), ct.with_datatype("float"):
        A = ct.to_tensor(rng.standard_normal((4096, 4096), dtype=np.float32))
        B = ct.to_tensor(rng.standard_normal((4096, 4096), dtype=np.float32))
        Cm = ct.to_tensor(rng.standard_normal((4096, 4096), dtype=np.float32))
        for name, ta, tb in combos:
            for _ in range(3):
                ct.gemm(Cm, ta, tb, 1.5, A, B, 0.5)
            ms = time_region(stream, lambda: ct.gemm(Cm, ta, tb, 1.5, A, B, 0.5), 10)
            out[name] = round(2.0 * 4096 ** 3 / ms / 1e9, 1)
        big = [ct.to_tensor(rng.standard_normal((4224, 4224), dtype=np.float32)) for _ in range(3)]
        Av, Bv, Cv = (ct.submatrix(t, 64, 4096, 64, 4096) for t in big)
        for name, ta, tb in combos:
            for _ in range(3):
                ct.gemm(Cv, ta, tb, 1.5, Av, Bv, 0.5)
            ms = time_region(stream, lambda: ct.gemm(Cv, ta, tb, 1.5, Av, Bv, 0.5), 10)
            pitched[name] = round(2.0 * 4096 ** 3 / ms / 1e9, 1)
    peak = roofs["tf32x3_burst"]
    return {"tflops": out, "tflops_pitch_4224_views": pitched, "roofline_peak_tflops": round(peak, 1),
            "frac": {k: round(v / peak, 3) for k, v in out.items()},
            "note": "peak (burst, kernel timed alone): %s; work counted as 2*M*N*K" % roofs["source"]["tf32x3"],
            "best": max(out.values())}


def bench_eltwise(drv, dev, peaks):
    """Config 3 in brief: GB/s of the HBM-bound kernels on [8192, 4096] fp32, rotating 4 buffer sets."""
    from cortex_b200 import tensor as ct
    from cortex_b200.dimensions import ALL
    stream = dev.create_stream()
    rows, cols, sets = 8192, 4096, 4
    rng = np.random.default_rng(301)
    res = {}
    with ct.with_stream(stream), ct.with_datatype("float"):
        xs = [ct.to_tensor(rng.standard_normal((rows, cols), dtype=np.float32)) for _ in range(sets)]
        ys = [ct.new_tensor([rows, cols]) for _ in range(sets)]
        bias = ct.to_tensor((rng.standard_normal((1, cols)) * 0.1).astype(np.float32))
        stat = [ct.new_tensor([rows, 1]) for _ in range(sets)]
        idx = ct.to_tensor(rng.integers(0, rows, size=rows, dtype=np.int32), datatype="int")
        gathered = [ct.select(x, idx, ALL) for x in xs]      # descriptor views, built once
        ga = ct.to_tensor(rng.standard_normal((4096, 4096), dtype=np.float32))
        gb = ct.to_tensor(rng.standard_normal((4096, 4096), dtype=np.float32))
        gc = ct.new_tensor([4096, 4096])

        def prime():
            for _ in range(4):
                ct.gemm(gc, False, True, 1.0, ga, gb, 0.0)

        state = {"i": 0}

        def rot():
            state["i"] = (state["i"] + 1) % sets
            return state["i"]

        cases = {
            "bias_add": (lambda i: ct.binary_op(ys[i], 1.0, xs[i], 1.0, bias, "+"), 2 * rows * cols * 4 + cols * 4),
            "relu": (lambda i: ct.binary_op(ys[i], 1.0, xs[i], 1.0, 0, "max"), 2 * rows * cols * 4),
            "reduce_max": (lambda i: ct.unary_reduce(stat[i], 1.0, xs[i], "max"), rows * cols * 4 + rows * 4),
            "reduce_sum": (lambda i: ct.unary_reduce(stat[i], 1.0, xs[i], "sum"), rows * cols * 4 + rows * 4),
            "softmax": (lambda i: ct.softmax(ys[i], xs[i]), 2 * rows * cols * 4),
            "gather_rows": (lambda i: ct.assign(ys[i], gathered[i]), 2 * rows * cols * 4 + rows * 4),
            "fused_bias_relu_rowstats": (lambda i: stream.bias_relu_rowstats(ys[i].buffer, cols, xs[i].buffer, cols,
                                                                            bias.buffer, rows, cols, stat[i].buffer,
                                                                            stat[(i + 1) % sets].buffer),
                                         2 * rows * cols * 4 + cols * 4 + 2 * rows * 4),
        }
        # next to the path: ternary select (PReLU-shaped: x >= 0 ? x : 0.25 * x) and gemv! (A [8192, 4096])
        vec = ct.to_tensor(rng.standard_normal(cols).astype(np.float32))
        outv = ct.new_tensor([rows])
        cases["ternary_select_prelu"] = (lambda i: ct.ternary_op(ys[i], 1.0, xs[i], 0.25, xs[i], 1.0, xs[i], "select"),
                                         2 * rows * cols * 4)
        cases["gemv_8192x4096"] = (lambda i: ct.gemv(outv, False, 1.0, xs[i], vec, 0.0), rows * cols * 4 + cols * 4 + rows * 4)
        # backward ring: activation-gradient! (reads output and output-gradient, writes input-gradient)
        grads = [ct.to_tensor(rng.standard_normal((rows, cols), dtype=np.float32)) for _ in range(sets)]
        for op_name in ("relu", "tanh"):
            cases["activation_gradient_" + op_name] = (
                lambda i, op_name=op_name: ct.activation_gradient(ys[i], grads[i], xs[i], op_name), 3 * rows * cols * 4)
        # batch-normalize! (inference, spatial form) on the config-4 activation shape viewed as [128, 64, 4096]
        bn_stats = [ct.to_tensor(np.abs(rng.standard_normal(64)).astype(np.float32) + 0.5) for _ in range(4)]
        bn_in = [ct.in_place_reshape(x, [128, 64, 4096]) for x in xs]
        bn_out = [ct.in_place_reshape(y, [128, 64, 4096]) for y in ys]
        cases["batch_normalize_spatial"] = (lambda i: ct.batch_normalize(bn_out[i], bn_in[i], *bn_stats, 1e-3),
                                            2 * rows * cols * 4)
        # pooling-forward!: 3x3 max, stride 2, pad 1 on [128, 64, 64, 64]
        pool_desc = ct.pooling_descriptor("float", 64, 3, 3, 1, 1, 2, 2, dimension_op="floor", pool_op="max")
        pool_in = [ct.in_place_reshape(x, [128, 64, 64, 64]) for x in xs]      # [8192, 4096] = 128 x 64 x 64 x 64
        pool_out = [ct.new_tensor([128, 64, 32, 32]) for _ in range(sets)]
        cases["pooling_max_3x3s2"] = (lambda i: stream.pooling_forward(pool_out[i].buffer, pool_out[i].dimensions, 0.0,
                                                                       pool_in[i].buffer, pool_in[i].dimensions, pool_desc),
                                      rows * cols * 4 + rows * cols)
        # pooling-backward! of that layer (reads input, output, output gradient; writes the input gradient)
        pool_og = [ct.to_tensor(rng.standard_normal((128, 64, 32, 32), dtype=np.float32)) for _ in range(2)]
        for i in range(sets):
            stream.pooling_forward(pool_out[i].buffer, pool_out[i].dimensions, 0.0, pool_in[i].buffer, pool_in[i].dimensions,
                                   pool_desc)
        pool_ig = [ct.in_place_reshape(y, [128, 64, 64, 64]) for y in ys]
        cases["pooling_backward_max_3x3s2"] = (lambda i: ct.pooling_backward(pool_ig[i], 0.0, pool_in[i], pool_out[i],
                                                                              pool_og[i % 2], pool_desc),
                                               2 * rows * cols * 4 + 2 * rows * cols)
        # batch-normalize training half, spatial form [128, 64, 4096].  Bytes counted as the algorithm's passes: mean,
        # variance about the rounded mean, apply = input read three times + output written; gradients = input and
        # output gradient read by the sums pass and again by the input-gradient pass + its write
        bn_batch = [ct.new_tensor([64]) for _ in range(2)]
        bn_run = [ct.to_tensor(np.ones(64, np.float32)) for _ in range(2)]
        bn_grads = [ct.new_tensor([64]) for _ in range(2)]
        cases["batch_normalize_update_and_apply_spatial"] = (
            lambda i: ct.batch_normalize_update_and_apply(bn_out[i], bn_in[i], bn_batch[0], bn_batch[1], bn_run[0], bn_run[1],
                                                          0.1, bn_stats[2], bn_stats[3], 1e-3), 4 * rows * cols * 4)
        bn_og = [ct.in_place_reshape(g_, [128, 64, 4096]) for g_ in grads]
        cases["batch_normalize_gradients_spatial"] = (
            lambda i: ct.batch_normalize_gradients(bn_out[i], bn_grads[0], bn_grads[1], bn_og[i], bn_out[i], bn_in[i],
                                                   bn_batch[0], bn_batch[1], bn_stats[2], bn_stats[3], 1e-3),
            5 * rows * cols * 4)
        # lrn across channels, n = 5, on [128, 64, 64, 64]
        lrn_desc = ct.lrn_descriptor(n=5, k=2, alpha=1e-4, beta=0.75)
        cases["lrn_forward_n5"] = (lambda i: ct.lrn_forward(pool_ig[i], pool_in[i], lrn_desc), 2 * rows * cols * 4)
        # optimiser steps over a flat 64 Mi-parameter buffer (two buffer sets of 4 x 256 MiB: far beyond L2) and rand!
        n_par = 64 << 20
        from cortex_b200 import optimize
        opt_sets = [[ct.new_tensor([n_par]) for _ in range(4)] for _ in range(2)]       # gradient, parameters, 2 x state
        for st_ in opt_sets:
            ct.rand(st_[0], ct.gaussian_distribution())
            ct.rand(st_[2], ct.flat_distribution(minimum=0.0, maximum=0.01))
            ct.rand(st_[3], ct.flat_distribution(minimum=0.0, maximum=0.01))
        adam, adadelta = optimize.Adam().batch_update(), optimize.Adadelta()
        cases["adam_step_64Mi"] = (lambda i: adam.compute_parameters(
            {"m": opt_sets[i % 2][2], "v": opt_sets[i % 2][3]}, 1.0, 0, opt_sets[i % 2][0], opt_sets[i % 2][1]), 7 * n_par * 4)
        # adadelta's accumulators are running averages of squares: non-negative (adam's m above is not)
        acc_sets = [[ct.new_tensor([n_par]) for _ in range(2)] for _ in range(2)]
        for st_ in acc_sets:
            for t_ in st_:
                ct.rand(t_, ct.flat_distribution(minimum=0.0, maximum=0.01))
        cases["adadelta_step_64Mi"] = (lambda i: adadelta.compute_parameters(
            {"grad-accum": acc_sets[i % 2][0], "dx-accum": acc_sets[i % 2][1]}, 1.0, 0, opt_sets[i % 2][0],
            opt_sets[i % 2][1]), 7 * n_par * 4)
        cases["rand_gaussian_64Mi"] = (lambda i: ct.rand(opt_sets[i % 2][0], ct.gaussian_distribution()), n_par * 4)
        cases["rand_flat_64Mi"] = (lambda i: ct.rand(opt_sets[i % 2][0], ct.flat_distribution()), n_par * 4)
        for name, (fn, nbytes) in cases.items():
            for _ in range(3):
                fn(rot())
            ms = time_region(stream, lambda: fn(rot()), 20, prime)
            gbs = nbytes / ms / 1e6
            res[name] = {"gbs": round(gbs, 0), "frac_of_%s_hbm" % peaks["source"]: round(gbs / peaks["hbm_gbs"], 3)}
    return res


def bench_conv(drv, dev, roofs):
    """Config 4 in brief: NCHW conv 64x64x56x56, 3x3 s1 p1, 64 output channels, + bias + ReLU, fp32."""
    from cortex_b200 import nn
    from cortex_b200 import tensor as ct
    stream = dev.create_stream()
    rng = np.random.default_rng(401)
    with ct.with_stream(stream), ct.with_datatype("float"):
        x = ct.to_tensor(rng.standard_normal((64, 64, 56, 56), dtype=np.float32))
        w = ct.to_tensor((rng.standard_normal((64, 576), dtype=np.float32) * np.float32(np.sqrt(2.0 / 576))))
        b = ct.new_tensor([64])
        out = ct.new_tensor([64, 64, 56, 56])
        layer = nn.Convolution(w, b, (3, 3), (1, 1), (1, 1), 64, 64, "float")

        def fwd():
            layer.forward(x, out)
            nn.relu(out, out)

        for _ in range(3):
            fwd()
        ms = time_region(stream, fwd, 10)
        conv_only = lambda: ct.convolution_forward(out, 0.0, x, w, layer.workspace, layer.desc, layer.algorithms)
        ms_conv = time_region(stream, conv_only, 10)
        fused = lambda: layer.forward_fused(x, out, "relu")      # bias + ReLU in the convolution's epilogue
        for _ in range(3):
            fused()
        ms_fused = time_region(stream, fused, 10)
    flops = 2.0 * 64 * 64 * 3136 * 576
    hbm_bytes = 2 * 64 * 64 * 56 * 56 * 4 + 64 * 576 * 4
    return {"ms": round(ms, 4), "tflops": round(flops / ms / 1e9, 1), "images_per_s": round(64 / ms * 1000.0, 0),
            "conv_kernel_ms": round(ms_conv, 4), "conv_kernel_tflops": round(flops / ms_conv / 1e9, 1),
            "conv_kernel_frac_of_tf32x3_burst": round(flops / ms_conv / 1e9 / roofs["tf32x3_burst"], 3),
            "conv_kernel_gbs_compulsory": round(hbm_bytes / ms_conv / 1e6, 0),
            "fused_ms": round(ms_fused, 4), "fused_tflops": round(flops / ms_fused / 1e9, 1),
            "fused_frac_of_tf32x3_burst": round(flops / ms_fused / 1e9 / roofs["tf32x3_burst"], 3),
            "note": "ms = conv + bias + ReLU as the reference's 3 protocol calls; fused_ms = the same layer as one call "
                    "(convolution_forward_bias_act: bias and ReLU in the kernel's epilogue, same bits); work = "
                    "2*64*64*3136*576; compulsory bytes = input + output + weights once"}


def bench_backward(drv, dev, peaks):
    """The backward ring at the benchmark's layer shapes (fp32, CUDA events): one hidden layer of the wide MLP
    on an 8192-row shard (bias gradient = a slab sum over the batch, input gradient = gemm! NN, weight
    gradient = gemm! TN, ReLU gradient) and the config-4 convolution layer's backward."""
    from cortex_b200 import nn
    from cortex_b200 import tensor as ct
    stream = dev.create_stream()
    rows = 8192
    rng = np.random.default_rng(701)
    res = {}
    with ct.with_stream(stream), ct.with_datatype("float"):
        lin = nn.Linear(ct.to_tensor(make_weights()[0]), ct.new_tensor([WIDTH]))
        x = ct.to_tensor(make_input(0, rows))
        out = ct.new_tensor([rows, WIDTH])
        lin.forward_fused(x, out, "relu")
        og = ct.to_tensor(rng.standard_normal((rows, WIDTH), dtype=np.float32))
        g_act, g_in = ct.new_tensor([rows, WIDTH]), ct.new_tensor([rows, WIDTH])
        g_w, g_b = ct.new_tensor([WIDTH, WIDTH]), ct.new_tensor([WIDTH])
        act = nn.Activation("relu")

        def layer_bwd():
            act.backward(out, g_act, og)
            lin.backward(x, out, g_in, g_act, g_w, g_b)

        for _ in range(2):
            layer_bwd()
        ms = time_region(stream, layer_bwd, 5)
        ms_bias = time_region(stream, lambda: ct.binary_op(g_b, 1.0, g_act, 1.0, g_b, "+"), 5)
        ms_in = time_region(stream, lambda: ct.gemm(g_in, False, False, 1.0, g_act, lin.weights, 0.0), 5)
        ms_w = time_region(stream, lambda: ct.gemm(g_w, True, False, 1.0, g_act, x, 1.0), 5)
        flops = 2.0 * rows * WIDTH * WIDTH
        res["mlp_layer_8192x4096x4096"] = {
            "ms": round(ms, 4), "input_gradient_ms": round(ms_in, 4), "input_gradient_tflops": round(flops / ms_in / 1e9, 1),
            "weight_gradient_ms": round(ms_w, 4), "weight_gradient_tflops": round(flops / ms_w / 1e9, 1),
            "bias_gradient_ms": round(ms_bias, 4)}
        cx = ct.to_tensor(rng.standard_normal((64, 64, 56, 56), dtype=np.float32))
        cw = ct.to_tensor((rng.standard_normal((64, 576), dtype=np.float32) * np.float32(np.sqrt(2.0 / 576))))
        cout = ct.new_tensor([64, 64, 56, 56])
        conv = nn.Convolution(cw, ct.new_tensor([64]), (3, 3), (1, 1), (1, 1), 64, 64, "float")
        conv.forward(cx, cout)
        cog = ct.to_tensor(rng.standard_normal((64, 64, 56, 56), dtype=np.float32))
        c_gin, c_gw, c_gb = ct.new_tensor([64, 64, 56, 56]), ct.new_tensor([64, 576]), ct.new_tensor([64])
        for _ in range(2):
            conv.backward(cx, c_gin, cog, c_gw, c_gb)
        ms_c = time_region(stream, lambda: conv.backward(cx, c_gin, cog, c_gw, c_gb), 3)
        ms_cw = time_region(stream, lambda: ct.convolution_backward_weights(c_gw, 0.0, cog, cx, None, conv.desc, None), 3)
        ms_cd = time_region(stream, lambda: ct.convolution_backward_data(c_gin, 0.0, cog, cw, None, conv.desc, None), 3)
        res["conv_64x64x56x56"] = {"ms": round(ms_c, 3), "backward_weights_ms": round(ms_cw, 3),
                                   "backward_data_ms": round(ms_cd, 3),
                                   "note": "weights: channel-major gradient + transposed unroll + one tensor-core gemm! NT over all pixels (K-sliced) + transpose-add; data: forward patch convolution of the output gradient with the mirrored filter; work 2 x 1.48e10 flop"}
    return res


def bench_gemm_f64(drv, dev, roofs=None):
    """Config 2, fp64: 4096^3 DMMA gemm!, alpha 1.5 beta 0.5."""
    from cortex_b200 import tensor as ct
    stream = dev.create_stream()
    rng = np.random.default_rng(201)
    out = {}
    with ct.with_stream(stream), ct.with_datatype("double"):
        A = ct.to_tensor(rng.standard_normal((4096, 4096)))
        B = ct.to_tensor(rng.standard_normal((4096, 4096)))
        Cm = ct.to_tensor(rng.standard_normal((4096, 4096)))
        for name, ta, tb in (("NT", False, True), ("NN", False, False)):
            ct.gemm(Cm, ta, tb, 1.5, A, B, 0.5)
            ms = time_region(stream, lambda: ct.gemm(Cm, ta, tb, 1.5, A, B, 0.5), 3)
            out[name] = round(2.0 * 4096 ** 3 / ms / 1e9, 2)
    res = {"tflops": out}
    if roofs:
        res["roofline_peak_tflops"] = round(roofs["fp64_burst"], 2)
        res["frac"] = {k: round(v / roofs["fp64_burst"], 3) for k, v in out.items()}
        res["note"] = "peak (burst): %s" % roofs["source"]["fp64"]
    return res


def bench_mlp_128(drv, dev):
    """Config 1: MNIST-shaped MLP, batch 128 (launch-latency-bound; roofline fractions are not meaningful here)."""
    from cortex_b200 import nn
    from cortex_b200 import tensor as ct
    stream = dev.create_stream()
    res = {}
    with ct.with_stream(stream), ct.with_datatype("float"):
        x = ct.to_tensor(np.random.default_rng(101).random((128, 784), dtype=np.float32))
        w1 = ct.to_tensor((np.random.default_rng(102).standard_normal((500, 784)) * np.sqrt(2.0 / 784)).astype(np.float32))
        w2 = ct.to_tensor((np.random.default_rng(103).standard_normal((10, 500)) * np.sqrt(2.0 / 500)).astype(np.float32))
        b1, b2 = ct.new_tensor([500]), ct.new_tensor([10])
        for label, fused in (("reference_call_sequence", False), ("fused", True)):
            net = nn.MLP([(w1, b1, "relu"), (w2, b2, "softmax")], fused=fused)
            for _ in range(5):
                net.infer(x)
            ms = time_region(stream, lambda: net.infer(x), 200)
            res[label] = {"us_per_forward": round(ms * 1000.0, 1), "samples_per_s": round(128 / ms * 1000.0, 0)}
        for _ in range(5):
            net.infer_replayed(x)          # run, capture, replay
        ms = time_region(stream, lambda: net.infer_replayed(x), 500)
        res["fused_graph_replay"] = {"us_per_forward": round(ms * 1000.0, 1), "samples_per_s": round(128 / ms * 1000.0, 0)}
    return res


def bench_mnist_convnet(drv, dev):
    """The reference's MNIST-NETWORK shape (conv 5x5 -> max-pool -> batch-norm -> ReLU -> conv 5x5 -> max-pool ->
    batch-norm -> linear 500 + ReLU -> linear 10 -> softmax), batch 128, inference."""
    from cortex_b200 import nn
    from cortex_b200 import tensor as ct
    stream = dev.create_stream()
    with ct.with_stream(stream), ct.with_datatype("float"):
        rng = np.random.default_rng(601)
        t = lambda a: ct.to_tensor(np.asarray(a, np.float32))
        he = lambda shape, fan: rng.standard_normal(shape) * np.sqrt(2.0 / fan)
        bn = lambda n: [t(rng.standard_normal(n) * 0.1), t(np.abs(rng.standard_normal(n)) + 0.5),
                        t(1 + 0.1 * rng.standard_normal(n)), t(rng.standard_normal(n) * 0.1)]
        net = nn.ConvNet([
            ("conv", nn.Convolution(t(he((20, 25), 25)), t(np.zeros(20)), (5, 5), (0, 0), (1, 1), 1, 20, "float")),
            ("pool", nn.Pooling(20, (2, 2), (0, 0), (2, 2), "float")), ("bn", nn.BatchNormalization(*bn(20))), ("relu",),
            ("conv", nn.Convolution(t(he((50, 500), 500)), t(np.zeros(50)), (5, 5), (0, 0), (1, 1), 20, 50, "float")),
            ("pool", nn.Pooling(50, (2, 2), (0, 0), (2, 2), "float")), ("flatten",), ("bn", nn.BatchNormalization(*bn(800))),
            ("linear", nn.Linear(t(he((500, 800), 800)), t(np.zeros(500))), "relu"),
            ("linear", nn.Linear(t(he((10, 500), 500)), t(np.zeros(10))), None), ("softmax",)])
        x = t(rng.random((128, 1, 28, 28)))
        for _ in range(3):
            net.infer(x)
        l0 = stream.launch_count()
        ms = time_region(stream, lambda: net.infer(x), 50)
        launches = (stream.launch_count() - l0) // 50
        for _ in range(3):
            net.infer_replayed(x)
        ms_g = time_region(stream, lambda: net.infer_replayed(x), 200)
    return {"us_per_forward": round(ms * 1000.0, 1), "samples_per_s": round(128 / ms * 1000.0, 0),
            "launches_per_forward": launches, "graph_replay_us_per_forward": round(ms_g * 1000.0, 1),
            "graph_replay_samples_per_s": round(128 / ms_g * 1000.0, 0)}


def bench_mlp_layer(drv, dev, peaks):
    """One hidden layer of the wide MLP on an 8192-row shard (the N=8 shard): the fused
    gemm_bias_act launch the benchmark's roofline is quoted on, small enough for an ncu capture."""
    from cortex_b200 import nn
    from cortex_b200 import tensor as ct
    stream = dev.create_stream()
    rows = 8192
    with ct.with_stream(stream), ct.with_datatype("float"):
        w = ct.to_tensor(make_weights()[0])
        b = ct.new_tensor([WIDTH])
        x = ct.to_tensor(make_input(0, rows))
        out = ct.new_tensor([rows, WIDTH])
        lin = nn.Linear(w, b)
        for _ in range(3):
            lin.forward_fused(x, out, "relu")
        ms = time_region(stream, lambda: lin.forward_fused(x, out, "relu"), 10)
        x_lo, out_lo = ct.new_tensor([rows, WIDTH]), ct.new_tensor([rows, WIDTH])
        stream.split_lo(x_lo.buffer, x.buffer, rows * WIDTH)
        for _ in range(3):
            lin.forward_presplit(x, x_lo, out, out_lo, "relu")
        ms_p = time_region(stream, lambda: lin.forward_presplit(x, x_lo, out, out_lo, "relu"), 10)
    tf = 2.0 * rows * WIDTH * WIDTH / ms / 1e9
    return {"rows": rows, "ms": round(ms, 4), "tflops": round(tf, 1), "presplit_ms": round(ms_p, 4),
            "presplit_tflops": round(2.0 * rows * WIDTH * WIDTH / ms_p / 1e9, 1),
            "algorithmic_bytes": rows * WIDTH * 4 * 2 + WIDTH * WIDTH * 4 + WIDTH * 4}


def bench_mlp_f64(drv, dev):
    """The fp64 variant of the wide MLP on a 16384-row slice of the batch (DMMA gemm + fused epilogue)."""
    from cortex_b200 import nn
    from cortex_b200 import tensor as ct
    stream = dev.create_stream()
    rows = 16384
    with ct.with_stream(stream), ct.with_datatype("double"):
        layers = []
        for i, w in enumerate(make_weights()):
            layers.append((ct.to_tensor(w.astype(np.float64)), ct.new_tensor([w.shape[0]]),
                           "softmax" if i == HIDDEN_LAYERS else "relu"))
        net = nn.MLP(layers, fused=True)
        x = ct.to_tensor(make_input(0, rows).astype(np.float64))
        net.infer(x)
        ms = time_region(stream, lambda: net.infer(x), 2)
    return {"rows": rows, "samples_per_s": round(rows / ms * 1000.0, 0),
            "tflops": round(rows * FLOPS_PER_SAMPLE / ms / 1e9, 2), "ms": round(ms, 2),
            "note": "full fp64 run of the benchmark: --dtype double"}


def bench_column_head(dev, stream, world, rank, dt, dist):
    """The column-sharded last layer (4096 -> 1000 split by output column over the ranks) on an
    8192-row replicated activation block: (a) GEMM, NCCL all-gather enqueued on the backend's stream,
    re-layout assign!, softmax!; (b) ONE fused GEMM whose epilogue stores its window into every rank's
    logits over NVLink, a stream-ordered fence, softmax!.  Device time, max over ranks.  Outside the
    timed regions both results are compared with a float64 softmax(h . W^T) on sampled rows, over all
    1000 columns (every rank's window), max over ranks."""
    import torch
    from cortex_b200 import tensor as ct
    from cortex_b200.parallel import (PeerLogits, column_sharded_head, column_sharded_head_fused, shard_bounds,
                                      stream_fence)
    B = 8192
    npdt = np.float32 if dt == "float" else np.float64
    lo, hi = shard_bounds(CLASSES, world, rank)
    w = make_weights()[-1].astype(npdt)
    h_host = np.maximum(make_input(0, B), 0).astype(npdt)
    res = {"rows": B, "columns_per_rank": hi - lo}
    with ct.with_stream(stream), ct.with_datatype(dt):
        h = ct.to_tensor(h_host)
        ws, bs = ct.to_tensor(w[lo:hi]), ct.new_tensor([hi - lo])
        exchange = PeerLogits(dev, B, CLASSES, world, rank, dt)
        fence = stream_fence(stream)
        fence()
        nccl_ws = {}
        out = {}

        def fused():
            out["fused"] = column_sharded_head_fused(h, ws, bs, exchange, fence)
            fence()       # the logits buffers are reused by the next call

        def nccl():
            out["nccl"] = column_sharded_head(h, ws, bs, CLASSES, world, rank, workspace=nccl_ws)

        for name, fn, iters in (("nccl_allgather_ms", nccl, 10), ("fused_peer_store_ms", fused, 10)):
            for _ in range(3):
                fn()
            stream.sync()
            dist.barrier()
            ms = time_region(stream, fn, iters)
            t = torch.tensor([ms], device="cuda", dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            res[name] = round(float(t[0]), 4)
        # parity, outside the timed regions: 48 sampled rows x all columns against float64
        rows_s = np.random.default_rng(77).choice(B, size=48, replace=False)
        z = h_host[rows_s].astype(np.float64) @ w.astype(np.float64).T
        e = np.exp(z - z.max(axis=1, keepdims=True))
        want = e / e.sum(axis=1, keepdims=True)
        errs = []
        for name in ("nccl", "fused"):
            got = ct.to_array(out[name]).reshape(B, CLASSES)
            errs.append(rel_err(got[rows_s], want))
            if name == "fused":
                res["max_abs_rowsum_minus_1"] = float(np.abs(got.sum(axis=1) - 1.0).max())
        t = torch.tensor(errs, device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        res["parity"] = {"nccl_allgather_rel_err_vs_fp64": float(t[0]), "fused_peer_store_rel_err_vs_fp64": float(t[1]),
                         "sample": "48 rows x all 1000 columns (every rank's window), max over ranks; "
                                   "abs(got-ref)/max(abs(ref), rms(ref))"}
        stream.sync()
        dist.barrier()
        exchange.close()
    return res


def with_clocks(local_rank, fn):
    """Runs fn() with nvidia-smi clock sampling around it; the clocks object is attached to fn's dict."""
    sampler = ClockSampler(local_rank)
    sampler.start()
    try:
        res = fn()
    finally:
        clocks = sampler.stop()
    if isinstance(res, dict):
        res["clocks"] = clocks
    return res


def run_b200(args, rank, world, local_rank):
    import torch  # plumbing only: rendezvous, barrier, max-over-ranks (and the measurement-only library peaks)
    dist = None
    # Ranks are spread evenly over the GPUs this process can see (stride = visible / world): on an 8-GPU board
    # consecutive GPUs share a PCIe switch / host bridge, and the host-fed path is bound by those links (measured:
    # four ranks on GPUs 0-3 upload at 26 GB/s each, two at 54 GB/s each).  With exactly `world` GPUs visible this
    # is the identity.
    visible = torch.cuda.device_count()
    local_rank = rank_device(local_rank, world, visible)
    if world > 1:
        import torch.distributed as dist
        torch.cuda.set_device(local_rank)
        dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", local_rank))
    from cortex_b200 import dimensions as dims
    from cortex_b200 import nn
    from cortex_b200 import tensor as ct
    from cortex_b200.driver import driver
    from cortex_b200.parallel import shard_bounds
    from cortex_b200.pipeline import BatchPipeline

    peaks = measured_peaks()
    drv = driver()
    dev = drv.get_devices()[local_rank]
    stream = dev.create_stream()
    lo, hi = shard_bounds(BATCH, world, rank)
    rows = hi - lo
    dt = args.dtype                                    # "float" (the headline) or "double" (the fp64 variant)
    npdt = np.float32 if dt == "float" else np.float64
    weights = [w.astype(npdt) for w in make_weights()]
    # page-locked staging buffers on the NUMA node of this GPU's PCIe slot
    x_host = drv.allocate_host_buffer(rows * WIDTH, dt, near=dev)
    x_host.as_numpy()[:] = make_input(lo, hi).reshape(-1)
    y_host = drv.allocate_host_buffer(rows * CLASSES, dt, near=dev)

    def barrier():
        stream.sync()
        if dist is not None:
            torch.cuda.synchronize()
            dist.barrier()
            torch.cuda.synchronize()

    lib_peaks = None
    if rank == 0 and not args.no_peaks:
        lib_peaks = measure_library_peaks(local_rank)
    roofs = rooflines(peaks, lib_peaks)

    with ct.with_stream(stream), ct.with_datatype(dt):
        layers = []
        for i, w in enumerate(weights):
            act = "softmax" if i == len(weights) - 1 else "relu"
            layers.append((ct.to_tensor(w), ct.new_tensor([w.shape[0]]), act))
        presplit = dt == "float"      # fp32: pre-split layer GEMMs (weights split once, activations by the epilogues)
        net = nn.MLP(layers, fused=True, presplit=presplit)
        x_dev = dev.allocate_device_buffer(rows * WIDTH, dt)
        stream.copy_host_to_device(x_host, 0, x_dev, 0, rows * WIDTH)
        x = ct.Tensor(dev, dims.dimensions([rows, WIDTH]), x_dev)

        # ---- resident: inputs already in HBM ------------------------------------------------
        gemm_events = []

        # resident arm: depth-first over 16384-row blocks when the shard is larger (measured at N = 1: 1.69 M
        # samples/s against 1.61 M layer by layer over all 65536 rows; the activations between layers then fit
        # partly in L2, DRAM traffic and power drop, and the power-capped clock settles ~10 % higher)
        if args.row_block < 0:
            row_block = 16384 if (dt == "float" and rows > 16384) else None
        else:
            row_block = args.row_block if args.row_block > 0 else None
        open_event = {}

        def trace(idx, when):
            # timing events around the hidden-layer GEMM launches
            if idx >= HIDDEN_LAYERS:
                return
            if when == "begin":
                open_event[idx] = stream.create_event(timing=True)
            else:
                gemm_events.append((open_event.pop(idx), stream.create_event(timing=True)))

        def step(record=False):
            return net.infer(x, row_block=row_block, trace=trace if record else None)

        sampler = ClockSampler(local_rank)      # started before the warm-up so that it is delivering by the timed region
        if rank == 0:
            sampler.start()
        for _ in range(args.warmup):
            resident_out = step()
        barrier()
        sampler.mark_begin()
        launches0 = stream.launch_count()
        e0 = stream.create_event(timing=True)
        for _ in range(args.steps):
            step(record=True)
        e1 = stream.create_event(timing=True)
        e1.wait_for_event()
        sampler.mark_end()
        barrier()
        clocks = sampler.stop() if rank == 0 else None
        launches = stream.launch_count() - launches0
        ms_step = e1.elapsed_ms_since(e0) / args.steps
        gemm_ms = float(np.mean([b.elapsed_ms_since(a) for a, b in gemm_events]))
        # rows of the resident result kept for the parity object below
        resident_all = ct.to_array(resident_out).reshape(rows, CLASSES).copy()     # this rank's rows [lo, hi)

        # ---- end to end: pinned host in -> H2D -> layers -> D2H, every step --------------------
        # chunks of 4096-8192 rows (>= 256 pair tiles each, two waves of the 74 clusters or more), three
        # rotating input slots so that two uploads can be in flight under one chunk's compute
        def chunk_for(n):
            return min(8192, max(4096, n // 2))

        # Host-fed sharding.  The GPUs of one box do not all get the same host-link bandwidth (measured on an
        # 8-GPU box of this pool: GPUs 0-3 ~20 GB/s each, GPUs 4-7 ~29 GB/s with all eight uploading), and with
        # even shards the pass ends when the slowest link ends.  Two calibration steps with even shards, every
        # rank at once, give each rank's rate (rows / its own device time); the rows are then re-dealt in
        # proportion, in multiples of 512, unless the rates are within 8 % of each other.  No data moves between
        # ranks: every rank regenerates the rows of its new range from the seeds.
        e2e_lo, e2e_hi = lo, hi
        rates = None
        if dist is not None and not args.even_shards:
            cal = BatchPipeline(dev, net, WIDTH, CLASSES, chunk_for(rows), dt, slots=3)
            cal.run(x_host, y_host, rows)
            my_rate = 0.0
            for _ in range(2):                  # two measurements of two steps each, the better one counts
                barrier()
                c0 = cal.compute.create_event(timing=True)
                for _ in range(2):
                    cal.run(x_host, y_host, rows, wait=False)
                cal.drain()
                cal.download.sync()
                c1 = cal.compute.create_event(timing=True)
                c1.wait_for_event()
                my_rate = max(my_rate, 2.0 * rows / max(c1.elapsed_ms_since(c0), 1e-6))
            cal.release()
            gathered = [torch.zeros(1, device="cuda", dtype=torch.float64) for _ in range(world)]
            dist.all_gather(gathered, torch.tensor([my_rate], device="cuda", dtype=torch.float64))
            rates = [float(g_[0]) for g_ in gathered]
            if args.shard_rates:                       # testing aid: pretend these were the measured rates
                rates = [float(v) for v in args.shard_rates.split(",")]
                assert len(rates) == world, "--shard-rates wants one value per rank"
            from cortex_b200.parallel import weighted_shard_bounds
            mean_rate = sum(rates) / world      # one bad measurement must not starve or flood a rank
            dealt = [min(max(r_, 0.6 * mean_rate), 1.6 * mean_rate) for r_ in rates]
            e2e_lo, e2e_hi = weighted_shard_bounds(BATCH, dealt, quantum=512, keep_equal_within=0.08)[rank]
        e2e_rows = e2e_hi - e2e_lo
        if (e2e_lo, e2e_hi) != (lo, hi):
            x_host = drv.allocate_host_buffer(e2e_rows * WIDTH, dt, near=dev)
            x_host.as_numpy()[:] = make_input(e2e_lo, e2e_hi).astype(npdt).reshape(-1)
            y_host = drv.allocate_host_buffer(e2e_rows * CLASSES, dt, near=dev)
        chunk = chunk_for(e2e_rows)
        pipe = BatchPipeline(dev, net, WIDTH, CLASSES, chunk, dt, slots=3)
        resident_rows, rows = rows, e2e_rows          # from here on `rows` is this rank's host-fed row count
        h2d = d2h = 0
        sampler = ClockSampler(local_rank)
        if rank == 0:
            sampler.start()
        for _ in range(min(args.warmup, 3)):
            pipe.run(x_host, y_host, rows)
        barrier()
        sampler.mark_begin()
        t0 = pipe.compute.create_event(timing=True)
        for _ in range(args.steps):
            h2d, d2h = pipe.run(x_host, y_host, rows, wait=False)    # steps stream back to back, drained once
        pipe.drain()
        pipe.download.sync()
        t1 = pipe.compute.create_event(timing=True)
        t1.wait_for_event()
        sampler.mark_end()
        barrier()
        e2e_ms = t1.elapsed_ms_since(t0) / args.steps
        e2e_clocks = sampler.stop() if rank == 0 else None
        # two more steps with timing events around every copy and every chunk's forward pass (not timed above)
        for _ in range(2):
            pipe.run(x_host, y_host, rows, wait=False, profile=True)
        pipe.drain()
        pipe.download.sync()
        pstats = pipe.stats()
        barrier()
        probs = y_host.as_numpy().reshape(rows, CLASSES)
        checksum = float(np.abs(probs.sum(axis=1) - 1.0).max())
        # parity of what came back through the pipeline: sampled rows of this rank's shard against float64
        parity_rows = np.random.default_rng(1000 + rank).choice(rows, size=min(16, rows), replace=False)
        want = fp64_forward(x_host.as_numpy().reshape(rows, WIDTH)[parity_rows], weights)
        parity_err = rel_err(probs[parity_rows], want)
        # host-fed chunks and the resident shard differ in row count, so the GEMM may share the K range of some
        # tiles differently (same products, another summation order): compared at rounding level, not bit for bit,
        # on rows this rank holds in both arms (global rows [lo, hi) resident, [e2e_lo, e2e_hi) host-fed)
        both_lo, both_hi = max(lo, e2e_lo), min(hi, e2e_hi)
        if both_hi > both_lo:
            common = both_lo + np.random.default_rng(2000 + rank).choice(both_hi - both_lo, size=min(16, both_hi - both_lo), replace=False)
            e2e_vs_resident = rel_err(probs[common - e2e_lo], resident_all[common - lo].astype(np.float64))
        else:
            e2e_vs_resident = 0.0
        column_head = bench_column_head(dev, stream, world, rank, dt, dist) if world > 1 else None

    # max over ranks
    rank_stats = [pstats.get("h2d", {}).get("gbs") or 0.0, pstats.get("d2h", {}).get("gbs") or 0.0,
                  pstats.get("compute", {}).get("ms_per_chunk") or 0.0, pstats.get("compute", {}).get("ms") or 0.0]
    if dist is not None:
        t = torch.tensor([ms_step, e2e_ms, parity_err, e2e_vs_resident], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms_step, e2e_ms, parity_err, e2e_vs_resident = float(t[0]), float(t[1]), float(t[2]), float(t[3])
        lt = torch.tensor([launches, h2d, d2h], device="cuda", dtype=torch.int64)
        dist.all_reduce(lt, op=dist.ReduceOp.SUM)
        launches, h2d_all, d2h_all = int(lt[0]), int(lt[1]), int(lt[2])
        rows_t = [torch.zeros(1, device="cuda", dtype=torch.int64) for _ in range(world)]
        dist.all_gather(rows_t, torch.tensor([rows], device="cuda", dtype=torch.int64))
        e2e_rows_per_rank = [int(r_[0]) for r_ in rows_t]
        gathered = [torch.zeros(4, device="cuda", dtype=torch.float64) for _ in range(world)]
        dist.all_gather(gathered, torch.tensor(rank_stats, device="cuda", dtype=torch.float64))
        all_stats = [[float(v) for v in g] for g in gathered]
    else:
        all_stats = [rank_stats]
        h2d_all, d2h_all, e2e_rows_per_rank = h2d, d2h, [rows]
    if rank != 0:
        if dist is not None:
            dist.destroy_process_group()
        return

    value = BATCH / (ms_step / 1000.0)
    e2e_value = BATCH / (e2e_ms / 1000.0)
    gemm_rows = min(resident_rows, row_block) if row_block else resident_rows
    gemm_flops = 2.0 * gemm_rows * WIDTH * WIDTH
    timed_s = ms_step * args.steps / 1000.0
    regime = "sustained" if timed_s >= 1.0 else "burst"
    if dt == "float":
        peak = roofs["tf32x3_" + regime]
        peak_note = ("3xTF32 roofline = TF32 rate / 3 (three tf32 MMAs per fp32 product; work counted as 2*M*N*K); %s; "
                     "%s figure because the timed region lasted %.2f s" % (roofs["source"]["tf32x3"], regime, timed_s))
        kernel_name = "gemm_presplit_pair_kernel"
        kernel_path = "split_lo + gemm_bias_act_presplit (tcgen05 cta_group::2 3xTF32 on pre-split operands, CTA pairs, bias+ReLU fused) x5 + softmax"
    else:
        peak = roofs["fp64_" + regime]
        peak_note = "fp64 roofline: %s; %s figure (timed region %.2f s); work 2*M*N*K" % (roofs["source"]["fp64"], regime, timed_s)
        kernel_name, kernel_path = "gemm_f64_kernel (DMMA)", "gemm_bias_act (DMMA fp64, bias+ReLU fused) x5 + softmax"
    achieved = gemm_flops / gemm_ms / 1e9
    # fp32: the pre-split kernel reads hi + lo of both operands and writes C + C_lo
    gemm_bytes = ((4 * gemm_rows * WIDTH + 2 * WIDTH * WIDTH + WIDTH) * 4 if dt == "float"
                  else (2 * gemm_rows * WIDTH + WIDTH * WIDTH + WIDTH) * 8)
    if dt == "float":
        # dram__bytes_read + dram__bytes_write of the same kernel on an 8192-row shard (ncu, one launch),
        # scaled by the number of row tiles
        traffic = (1221.3e6 + 243.7e6) * gemm_rows / 8192.0
        traffic_note = ("ncu capture of the 8192-row launch of gemm_presplit_pair_kernel (1.22 GB read + 0.24 GB "
                        "written) x rows/8192; not memory-bound (~18 % of HBM rate)")
    else:
        traffic, traffic_note = None, "no capture of the fp64 kernel's DRAM counters"
    config = workload_config(world, dt)
    line = {
        "metric": "wide_mlp_inference_samples_per_s" + ("" if dt == "float" else "_fp64"), "value": value, "unit": "samples/s", "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_step, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "f32" if dt == "float" else "f64", "data": "synthetic",
        "config": config, "rows_per_gpu": resident_rows, "row_block": row_block, "kernel_path": kernel_path,
        "gpu_indices": [rank_device(r, world, visible) for r in range(world)],
        "tflops": value * FLOPS_PER_SAMPLE / 1e12,
        "e2e": {"value": e2e_value, "unit": "samples/s", "h2d_bytes_per_step": h2d_all, "d2h_bytes_per_step": d2h_all,
                "ms_per_step": e2e_ms, "chunk_rows": chunk, "input_slots": pipe.slots,
                "rows_per_rank": e2e_rows_per_rank,
                "sharding": ("even" if len(set(e2e_rows_per_rank)) <= 1 else
                             "rows in proportion to each rank's host-fed rate in two calibration steps with even "
                             "shards (multiples of 512; even when the rates are within 8 %)"),
                "calibration_rows_per_ms": [round(r_, 1) for r_ in rates] if rates else None,
                "host_buffer_numa_node": getattr(x_host, "numa_node", -1),
                "max_abs_rowsum_minus_1": checksum, "clocks": e2e_clocks,
                "per_rank": [{"h2d_gbs": round(s_[0], 2), "d2h_gbs": round(s_[1], 2), "forward_ms_per_chunk": round(s_[2], 3),
                              "compute_busy_frac": round(s_[3] / 2.0 / e2e_ms, 3) if e2e_ms > 0 else None} for s_ in all_stats],
                "per_rank_note": "two extra profiled steps after the timed region: achieved copy rates (copy time "
                                 "includes waiting for the link), device time of one chunk's forward pass, and that "
                                 "time x chunks / the timed ms_per_step"},
        "gpu_launches": launches,
        "roofline": {"bound": "tensor", "kernel": "%s (M=%d, N=4096, K=4096)" % (kernel_name, gemm_rows),
                     "achieved": achieved, "peak": peak, "unit": "TFLOP/s", "frac": achieved / peak,
                     "traffic": traffic, "traffic_note": traffic_note, "algorithmic_bytes": gemm_bytes, "ms_per_launch": gemm_ms,
                     "peak_note": peak_note, "frac_of_burst": achieved / (roofs["tf32x3_burst"] if dt == "float" else roofs["fp64_burst"])},
        "parity": {"batch_sharded_rel_err_vs_fp64": parity_err, "tolerance": 1e-4 if dt == "float" else 1e-12,
                   "e2e_rows_vs_resident_rel_err": e2e_vs_resident,
                   "sample": "16 random rows of every rank's shard, as returned through the host pipeline, against a "
                             "float64 numpy forward; abs(got-ref)/max(abs(ref), rms(ref)), max over ranks"},
        "clocks": clocks,
        "library_peaks": lib_peaks,
    }
    if column_head is not None:
        line["column_sharded_head"] = column_head
    if world == 1 and dt == "float":
        step_cpu = cpu_arm(CPU_SAMPLE_ROWS, weights)
        rate, secs = step_cpu()
        line["cpu_baseline"] = cpu_baseline_object(rate, secs, CPU_SAMPLE_ROWS)
        extra = lambda fn: with_clocks(local_rank, fn)
        line["gemm_4096"] = extra(lambda: bench_gemm_4096(drv, dev, roofs))
        line["gemm_4096_f64"] = extra(lambda: bench_gemm_f64(drv, dev, roofs))
        line["eltwise"] = extra(lambda: bench_eltwise(drv, dev, peaks))
        line["conv_64x64x56x56"] = extra(lambda: bench_conv(drv, dev, roofs))
        line["mlp_128x784_500_10"] = extra(lambda: bench_mlp_128(drv, dev))
        line["wide_mlp_fp64"] = extra(lambda: bench_mlp_f64(drv, dev))
        line["mnist_convnet_128"] = extra(lambda: bench_mnist_convnet(drv, dev))
        line["backward"] = extra(lambda: bench_backward(drv, dev, peaks))
    print(json.dumps(line), flush=True)
    if dist is not None:
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--dtype", default="float", choices=["float", "double"],
                    help="float = the headline workload; double = its fp64 variant (DMMA gemm)")
    ap.add_argument("--row-block", type=int, default=-1,
                    help="resident arm: run the layer stack depth-first over blocks of this many rows "
                         "(0 = whole shard per layer, -1 = automatic)")
    ap.add_argument("--even-shards", action="store_true",
                    help="N > 1: keep the even row split for the host-fed arm (no calibration / re-dealing)")
    ap.add_argument("--shard-rates", default="",
                    help="N > 1, testing aid: comma-separated rates to re-deal the host-fed rows by, instead of the "
                         "calibrated ones (e.g. 1,1.5 on two GPUs exercises the uneven path)")
    ap.add_argument("--no-peaks", action="store_true",
                    help="skip the measurement-only library matmul peaks (rooflines then use the bf16-derived proxy)")
    ap.add_argument("--case", default="mlp", choices=["mlp", "gemm4096", "eltwise", "conv", "gemm4096f64", "mlp128", "mlplayer", "mnistcnn", "backward"],
                    help="mlp = the benchmark; gemm4096 / eltwise = the small single-purpose runs used for ncu captures")
    args = ap.parse_args()
    if args.case != "mlp":
        from cortex_b200.driver import driver
        drv = driver()
        dev = drv.default_device()
        peaks = measured_peaks()
        roofs = rooflines(peaks, None)
        fns = {"gemm4096": lambda: bench_gemm_4096(drv, dev, roofs), "eltwise": lambda: bench_eltwise(drv, dev, peaks),
               "conv": lambda: bench_conv(drv, dev, roofs), "gemm4096f64": lambda: bench_gemm_f64(drv, dev, roofs),
               "mlp128": lambda: bench_mlp_128(drv, dev), "mlplayer": lambda: bench_mlp_layer(drv, dev, peaks), "mnistcnn": lambda: bench_mnist_convnet(drv, dev),
               "backward": lambda: bench_backward(drv, dev, peaks)}
        print(json.dumps({args.case: fns[args.case]()}), flush=True)
        return
    args.warmup = max(args.warmup, 3) if args.impl == "b200" else args.warmup
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference(args, rank, world)
    else:
        run_b200(args, rank, world, local_rank)


if __name__ == "__main__":
    main()
