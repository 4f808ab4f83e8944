"""B200 kernels against the CPU oracle on seeded, configuration-shaped inputs,
through the C ABI.  Tolerances are the ones the backend is specified to:
bit-exact for integer / copy work, max rel err <= 1e-4 (fp32) and <= 1e-12
(fp64), error measured as abs(gpu - ref) / max(abs(ref), rms(ref))."""
import ctypes

import numpy as np
import pytest

import parity_cases as pc
from cortex_b200 import tensor as ct

pytestmark = pytest.mark.gpu


def _on(driver, datatype, fn, options=None):
    stream = driver.default_device().create_stream()
    for name, value in (options or {}).items():
        stream.set_option(name, value)
    with ct.with_stream(stream), ct.with_datatype(datatype):
        out = fn()
    stream.sync()
    return out


GEMM_SHAPES = [
    # m, n, k, pitch_pad, offset
    (3, 3, 3, 0, 0),          # the reference's own literal size
    (128, 256, 32, 0, 0),     # exactly one tile, one k-block
    (128, 256, 96, 0, 0),
    (200, 136, 100, 0, 0),    # ragged in every dimension
    (130, 10, 500, 2, 0),     # MLP tail; pitch not a multiple of 4 -> SIMT kernel for fp32
    (257, 300, 129, 4, 4),    # pitched window at (4,4): pitch multiple of 4, 16-byte aligned origin
    (64, 64, 64, 8, 3),       # window origin not 16-byte aligned
    (512, 384, 1024, 128, 64),
]


@pytest.mark.parametrize("datatype", ["float", "double"])
@pytest.mark.parametrize("ta,tb", [(False, False), (False, True), (True, False), (True, True)],
                         ids=["NN", "NT", "TN", "TT"])
@pytest.mark.parametrize("shape", GEMM_SHAPES, ids=lambda s: "x".join(map(str, s)))
def test_gemm_matches_oracle(b200_driver, oracle_driver, datatype, ta, tb, shape):
    m, n, k, pad, off = shape
    for alpha, beta in ((1.5, 0.5), (1.0, 0.0), (1.0, 1.0)):
        run, ref64 = pc.gemm_case(datatype, m, n, k, ta, tb, alpha, beta, pad, off)
        gpu = _on(b200_driver, datatype, run)
        cpu = _on(oracle_driver, datatype, run)
        assert pc.rel_err(gpu, cpu) <= pc.TOL[datatype], (alpha, beta)
        assert pc.rel_err(gpu, ref64()) <= pc.TOL[datatype], (alpha, beta)


@pytest.mark.parametrize("ta,tb", [(False, False), (False, True), (True, False), (True, True)],
                         ids=["NN", "NT", "TN", "TT"])
@pytest.mark.parametrize("shape", GEMM_SHAPES + [(700, 520, 4200, 8, 4)], ids=lambda s: "x".join(map(str, s)))
def test_gemm_through_presplit_pair_path(b200_driver, oracle_driver, ta, tb, shape):
    """gemm! forced onto the path large problems take: operands split (MN-major ones also transposed) into
    the stream's workspace, then the CTA-pair kernel.  Same cases and bounds as test_gemm_matches_oracle,
    whole backing buffer compared (the frame around a pitched window stays untouched).  The routing is a
    per-stream option: 2 = take that path whenever TMA can address the operands."""
    m, n, k, pad, off = shape
    for alpha, beta in ((1.5, 0.5), (1.0, 0.0), (1.0, 1.0)):
        run, ref64 = pc.gemm_case("float", m, n, k, ta, tb, alpha, beta, pad, off)
        gpu = _on(b200_driver, "float", run, {"gemm-auto-presplit": 2})
        cpu = _on(oracle_driver, "float", run)
        assert pc.rel_err(gpu, cpu) <= pc.TOL["float"], (alpha, beta)
        assert pc.rel_err(gpu, ref64()) <= pc.TOL["float"], (alpha, beta)


@pytest.mark.parametrize("ta,tb", [(False, True), (True, False)], ids=["NT", "TN"])
def test_gemm_pair_path_shared_tail_tiles(b200_driver, ta, tb):
    """84 pair tiles on 74 clusters: the 10 tiles of the last round are each reduced by two clusters (one per
    K half) and combined by whichever finishes second; with beta != 0 and twice in a row (the flags that
    order the two halves must be left clear)."""
    m, n, k = 3072, 1792, 320
    run, ref64 = pc.gemm_case("float", m, n, k, ta, tb, 1.5, 0.5, 0, 0)
    for _ in range(2):
        gpu = _on(b200_driver, "float", run, {"gemm-auto-presplit": 2})
        assert pc.rel_err(gpu, ref64()) <= pc.TOL["float"]


def test_gemm_beta_zero_ignores_nan_in_c(b200_driver):
    """BLAS semantics: with beta = 0, C is overwritten without being read."""
    rng = np.random.default_rng(5)
    A = rng.standard_normal((128, 64)).astype(np.float32)
    B = rng.standard_normal((64, 64)).astype(np.float32)

    def run():
        c = ct.to_tensor(np.full((128, 64), np.nan, np.float32), "float")
        ct.gemm(c, False, True, 1.0, ct.to_tensor(A, "float"), ct.to_tensor(B, "float"), 0.0)
        return ct.to_array(c)

    out = _on(b200_driver, "float", run).reshape(128, 64)
    assert np.isfinite(out).all()
    assert pc.rel_err(out, A.astype(np.float64) @ B.astype(np.float64).T) <= 1e-4


@pytest.mark.parametrize("datatype", ["float", "double"])
@pytest.mark.parametrize("rows,cols", [(64, 96), (257, 1000), (512, 4096), (33, 10), (16, 9000)])
def test_eltwise_reduce_softmax(b200_driver, oracle_driver, datatype, rows, cols):
    case = pc.eltwise_case(datatype, rows, cols)
    gpu, cpu = _on(b200_driver, datatype, case), _on(oracle_driver, datatype, case)
    for key in ("biased", "biased_inplace", "relu", "rowmax"):
        assert np.array_equal(gpu[key], cpu[key]), key          # one rounding of an exact double result: bit-exact
    for key in ("rowsum", "softmax", "softmax_decomposed"):
        assert pc.rel_err(gpu[key], cpu[key]) <= pc.TOL[datatype], key


@pytest.mark.parametrize("datatype", ["int", "long", "float", "double"])
def test_gather_bit_exact(b200_driver, oracle_driver, datatype):
    for (src_rows, n_idx, cols) in ((100, 57, 24), (1024, 512, 4096), (50, 31, 7)):
        run, ref = pc.gather_case(datatype, src_rows, n_idx, cols)
        gpu = _on(b200_driver, datatype, run)
        assert np.array_equal(gpu.reshape(n_idx, cols), ref())
        assert np.array_equal(gpu, _on(oracle_driver, datatype, run))


@pytest.mark.parametrize("datatype", ["float", "double"])
@pytest.mark.parametrize("fused", [False, True], ids=["unfused", "fused"])
def test_mlp_matches_oracle(b200_driver, oracle_driver, datatype, fused):
    for batch, widths in ((128, [784, 500, 10]), (256, [1024, 1024, 1024, 1000])):
        run_gpu, ref = pc.mlp_case(datatype, batch, widths, fused=fused, bias_scale=0.1)
        run_cpu, _ = pc.mlp_case(datatype, batch, widths, fused=False, bias_scale=0.1)
        gpu, cpu = _on(b200_driver, datatype, run_gpu), _on(oracle_driver, datatype, run_cpu)
        assert pc.rel_err(gpu, cpu) <= pc.TOL[datatype]
        assert pc.rel_err(gpu, ref()) <= pc.TOL[datatype]


@pytest.mark.parametrize("datatype", ["float", "double"])
@pytest.mark.parametrize("op", ["relu", "tanh", "logistic"])
def test_activation_gradient_bit_exact(b200_driver, oracle_driver, datatype, op):
    """activation-gradient!: float views computed in double and rounded once on both sides -> identical bits;
    dense operands (16-byte path) and windows of wider buffers (index-system path, frame untouched)."""
    for rows, cols, pitched in ((257, 1000, False), (512, 4096, False), (33, 10, False), (130, 75, True), (64, 1024, True)):
        run = pc.activation_gradient_case(datatype, rows, cols, op, pitched=pitched)
        assert np.array_equal(_on(b200_driver, datatype, run), _on(oracle_driver, datatype, run)), (rows, cols, pitched)


@pytest.mark.parametrize("datatype", ["float", "double"])
@pytest.mark.parametrize("act", ["relu", "tanh"])
def test_mlp_backward_matches_oracle(b200_driver, oracle_driver, datatype, act):
    """Forward + backward of config 1's network (128 x 784 -> 500 -> 10) and of a 3-layer 256-wide one: input
    gradient and every weight / bias gradient against the oracle's identical call sequence and float64 numpy."""
    for batch, widths in ((128, [784, 500, 10]), (64, [256, 256, 256, 100])):
        run, ref = pc.mlp_backward_case(datatype, batch, widths, act=act)
        gpu, cpu = _on(b200_driver, datatype, run), _on(oracle_driver, datatype, run)
        assert pc.rel_err(gpu, cpu) <= pc.TOL[datatype]
        assert pc.rel_err(gpu, ref()) <= pc.TOL[datatype]


@pytest.mark.parametrize("datatype", ["float", "double"])
def test_conv_backward_matches_oracle(b200_driver, oracle_driver, datatype):
    """ConvolutionLayer backward (bias gradient = a slab sum over batch and pixels, weight gradient, input gradient)
    against the oracle's restatement of the CPU backend and a float64 numpy convolution transpose."""
    for args in (dict(batch=2, cin=4, hw=9, cout=5), dict(batch=2, cin=3, hw=8, cout=4, k=2, pad=0, stride=2),
                 dict(batch=3, cin=16, hw=13, cout=40, k=5, pad=2), dict(batch=2, cin=32, hw=17, cout=36, k=3, pad=1, stride=2),
                 dict(batch=4, cin=64, hw=28, cout=64),
                 # stride 1 and a multiple of 16 output channels: the fp32 data gradient runs as a forward
                 # convolution of the output gradient (mirrored filter, padding k - 1 - pad) on the TMA-fed kernels
                 dict(batch=2, cin=24, hw=16, cout=32, k=3, pad=1), dict(batch=3, cin=8, hw=20, cout=16, k=5, pad=2),
                 dict(batch=2, cin=16, hw=12, cout=16, k=3, pad=0), dict(batch=2, cin=40, hw=32, cout=48, k=1, pad=0),
                 # 4096 and more pixels in the batch: the fp32 weight gradient is one tensor-core gemm! over all
                 # pixels (gradient made channel-major, input unrolled transposed), its reduction sliced over the SMs
                 dict(batch=8, cin=16, hw=32, cout=24, k=3, pad=1), dict(batch=5, cin=6, hw=31, cout=70, k=5, pad=2, stride=1),
                 dict(batch=16, cin=8, hw=36, cout=12, k=3, pad=1, stride=2)):
        run, ref = pc.conv_backward_case(datatype, **args)
        gpu, cpu = _on(b200_driver, datatype, run), _on(oracle_driver, datatype, run)
        assert pc.rel_err(gpu, cpu) <= pc.TOL[datatype], args
        assert pc.rel_err(gpu, ref()) <= pc.TOL[datatype], args


@pytest.mark.parametrize("datatype", ["float", "double"])
def test_conv_matches_oracle(b200_driver, oracle_driver, datatype):
    for args in (dict(batch=2, cin=4, hw=9, cout=5), dict(batch=2, cin=3, hw=8, cout=4, k=2, pad=0, stride=2),
                 dict(batch=4, cin=64, hw=28, cout=64),
                 # channel counts that are multiples of 16 take the tap-major gather
                 dict(batch=3, cin=16, hw=13, cout=40, k=5, pad=2),
                 dict(batch=2, cin=32, hw=17, cout=130, k=3, pad=1, stride=2),
                 dict(batch=1, cin=48, hw=10, cout=100, k=1, pad=0)):
        run, ref = pc.conv_case(datatype, bias_scale=0.1, **args)
        gpu, cpu = _on(b200_driver, datatype, run), _on(oracle_driver, datatype, run)
        assert pc.rel_err(gpu, cpu) <= pc.TOL[datatype]
        assert pc.rel_err(gpu, ref()) <= pc.TOL[datatype]


@pytest.mark.parametrize("args", [
    dict(batch=3, cin=16, hw=16, cout=24),                       # 16 x 8 boxes, one per tile
    dict(batch=5, cin=32, hw=24, cout=72),                       # 8 x 8 boxes, two per tile, the last tile half empty
    dict(batch=2, cin=16, hw=56, cout=64),                       # config 4's geometry
    dict(batch=1, cin=64, hw=32, cout=200, k=5, pad=2),          # 256-wide channel tile
    dict(batch=2, cin=16, hw=20, cout=8, k=1, pad=0),            # 1 x 1 filter
    dict(batch=2, cin=16, hw=18, cout=16, k=3, pad=0),           # no padding
    dict(batch=1, cin=16, hw=14, cout=16, k=3, pad=2),           # padding wider than the filter's reach
    dict(batch=3, cin=16, hw=13, cout=40, k=5, pad=2),           # 16 x 2 boxes, four per tile, overhang in x and y
    dict(batch=2, cin=32, hw=32, cout=100, k=3, pad=1),          # 8 x 16 patch tiles exactly, two channel blocks
    dict(batch=1, cin=16, hw=40, cout=64, k=7, pad=3),           # 7 x 7 filter: 14 x 22 patch
    dict(batch=2, cin=48, hw=24, cout=20, k=2, pad=0),           # even filter, output 23 x 23 (overhang)
    dict(batch=40, cin=32, hw=32, cout=48),                      # 320 tiles on 296 slots: the 24 tiles of the last round are shared over the channel blocks
    # stride 2: the per-tap kernel's boxes walk the input with the tensor map's traversal stride
    # (layers with at least ~400 products per input element; the others stay on the gather kernel)
    dict(batch=3, cin=32, hw=32, cout=200, k=3, pad=1, stride=2),
    dict(batch=2, cin=16, hw=56, cout=72, k=5, pad=2, stride=2),
    dict(batch=2, cin=16, hw=56, cout=64, k=1, pad=0, stride=2),      # too little work per element: gather kernel
], ids=lambda a: "x".join(str(v) for v in a.values()))
def test_conv_tma_fed_kernels(b200_driver, oracle_driver, args):
    """Stride-1 fp32 convolutions with a multiple of 16 input channels run kernels whose operand tiles all arrive
    by TMA: by geometry (route 0) the one that keeps the input patch in shared memory across the filter taps, or
    the one that loads a shifted tile per tap (route 2: forced here so that both run on every geometry they
    accept).  Against the oracle, float64, and the thread-gathered kernel (route 1), which sums in the same
    k order."""
    run, ref = pc.conv_case("float", bias_scale=0.1, **args)
    by_geometry = _on(b200_driver, "float", run)                       # reads the NCHW input itself where it can
    behind_prepass = _on(b200_driver, "float", run, {"conv-route": 3}) # the patch kernel behind its layout pre-pass
    per_tap = _on(b200_driver, "float", run, {"conv-route": 2})
    gathered = _on(b200_driver, "float", run, {"conv-route": 1})
    cpu = _on(oracle_driver, "float", run)
    want = ref()
    for got in (by_geometry, behind_prepass, per_tap):
        assert pc.rel_err(got, cpu) <= pc.TOL["float"]
        assert pc.rel_err(got, want) <= pc.TOL["float"]
        assert pc.rel_err(got, gathered) <= 2e-5


def test_fused_bias_relu_rowstats(b200_driver, oracle_driver):
    rng = np.random.default_rng(9)
    for dt, npdt in (("float", np.float32), ("double", np.float64)):
        X = rng.standard_normal((300, 4096)).astype(npdt)
        b = (rng.standard_normal(4096) * 0.1).astype(npdt)

        def run():
            stream = ct.check_stream()
            x, bias = ct.to_tensor(X, dt), ct.to_tensor(b, dt)
            y, mx, sm = ct.new_tensor([300, 4096], dt), ct.new_tensor([300], dt), ct.new_tensor([300], dt)
            stream.bias_relu_rowstats(y.buffer, 4096, x.buffer, 4096, bias.buffer, 300, 4096, mx.buffer, sm.buffer)
            return ct.to_array(y), ct.to_array(mx), ct.to_array(sm)

        g, c = _on(b200_driver, dt, run), _on(oracle_driver, dt, run)
        assert np.array_equal(g[0], c[0]) and np.array_equal(g[1], c[1])
        assert pc.rel_err(g[2], c[2]) <= pc.TOL[dt]


def test_batch_pipeline_matches_resident_inference(b200_driver):
    """Host-buffer pipeline (pinned in -> H2D -> layers -> D2H, ragged last chunk) gives exactly the
    resident result: same kernels on the same rows."""
    from cortex_b200 import nn
    from cortex_b200.pipeline import BatchPipeline
    rng = np.random.default_rng(21)
    rows, width, classes, chunk = 1000, 256, 24, 384
    X = rng.standard_normal((rows, width)).astype(np.float32)
    W1 = (rng.standard_normal((width, width)) * np.sqrt(2.0 / width)).astype(np.float32)
    W2 = (rng.standard_normal((classes, width)) * np.sqrt(2.0 / width)).astype(np.float32)
    b1 = (rng.standard_normal(width) * 0.1).astype(np.float32)
    b2 = (rng.standard_normal(classes) * 0.1).astype(np.float32)
    dev = b200_driver.default_device()
    stream = dev.create_stream()
    with ct.with_stream(stream), ct.with_datatype("float"):
        net = nn.MLP([(ct.to_tensor(W1), ct.to_tensor(b1), "relu"), (ct.to_tensor(W2), ct.to_tensor(b2), "softmax")],
                     fused=True)
        resident = ct.to_array(net.infer(ct.to_tensor(X))).reshape(rows, classes)
        stream.sync()
        host_in = b200_driver.allocate_host_buffer(rows * width, "float")
        host_in.as_numpy()[:] = X.reshape(-1)
        host_out = b200_driver.allocate_host_buffer(rows * classes, "float")
        pipe = BatchPipeline(dev, net, width, classes, chunk, "float")
        for _ in range(2):                      # second pass reuses the slots
            h2d, d2h = pipe.run(host_in, host_out, rows)
        pipe.release()
    assert (h2d, d2h) == (rows * width * 4, rows * classes * 4)
    got = host_out.as_numpy().reshape(rows, classes)
    assert np.array_equal(got, resident)
    assert np.abs(got.sum(axis=1) - 1.0).max() < 1e-5


@pytest.mark.gpu
@pytest.mark.parametrize("fused", [False, True])
def test_graph_replay_matches_direct_inference(fused):
    """The captured launch sequence replays to the same bits as the direct calls, also after the
    input buffer's contents change."""
    import numpy as np
    from cortex_b200 import nn
    from cortex_b200 import tensor as ct
    from cortex_b200.driver import driver
    dev = driver().default_device()
    stream = dev.create_stream()
    rng = np.random.default_rng(31)
    with ct.with_stream(stream), ct.with_datatype("float"):
        w1 = ct.to_tensor((rng.standard_normal((500, 784)) * 0.05).astype(np.float32))
        w2 = ct.to_tensor((rng.standard_normal((10, 500)) * 0.06).astype(np.float32))
        b1 = ct.to_tensor((rng.standard_normal(500) * 0.1).astype(np.float32))
        b2 = ct.to_tensor((rng.standard_normal(10) * 0.1).astype(np.float32))
        net = nn.MLP([(w1, b1, "relu"), (w2, b2, "softmax")], fused=fused)
        x = ct.to_tensor(rng.random((128, 784), dtype=np.float32))
        launches_per_forward = None
        for trial in range(4):
            if trial:
                ct.assign(x, ct.to_tensor(rng.random((128, 784), dtype=np.float32)))
            before = stream.launch_count()
            direct = ct.to_array(net.infer(x)).copy()
            per = stream.launch_count() - before
            before = stream.launch_count()
            replayed = ct.to_array(net.infer_replayed(x)).copy()
            if trial >= 2:      # trial 0 runs directly, trial 1 captures and replays once
                assert stream.launch_count() - before == per
            assert np.array_equal(direct, replayed)
            launches_per_forward = per
        # fused: the hidden layer's kernel and the head's (bias + softmax in its epilogue); unfused: the call sequence
        assert launches_per_forward >= (2 if fused else 3)


@pytest.mark.gpu
@pytest.mark.parametrize("datatype", ["float", "double"])
def test_gemv_matches_oracle(b200_driver, oracle_driver, datatype):
    """gemv! on configuration-like shapes: both transposes, beta 0 and non-zero, a pitched matrix view and a
    strided (column) vector."""
    npdt = np.float32 if datatype == "float" else np.float64
    rng = np.random.default_rng(71)
    for rows, cols in ((128, 784), (500, 37), (1000, 4096), (33, 2050)):
        A = rng.standard_normal((rows, cols + 8)).astype(npdt)
        xn = rng.standard_normal(cols).astype(npdt)
        xt = rng.standard_normal((rows, 3)).astype(npdt)          # a column of this is a strided vector
        c0n = rng.standard_normal(rows).astype(npdt)
        c0t = rng.standard_normal(cols).astype(npdt)

        def run():
            a = ct.submatrix(ct.to_tensor(A, datatype), 0, rows, 0, cols)        # row pitch cols + 8
            cn, ctt = ct.to_tensor(c0n, datatype), ct.to_tensor(c0t, datatype)
            ct.gemv(cn, False, 1.5, a, ct.to_tensor(xn, datatype), 0.5)
            ct.gemv(ctt, True, 0.75, a, ct.columns(ct.to_tensor(xt, datatype))[1], 0.0)
            return ct.to_array(cn), ct.to_array(ctt)

        g, c = _on(b200_driver, datatype, run), _on(oracle_driver, datatype, run)
        for gv, cv in zip(g, c):
            assert pc.rel_err(gv, cv) <= pc.TOL[datatype]
        A64 = A[:, :cols].astype(np.float64)
        assert pc.rel_err(g[0], 1.5 * A64 @ xn + 0.5 * c0n) <= pc.TOL[datatype]
        assert pc.rel_err(g[1], 0.75 * A64.T @ xt[:, 1]) <= pc.TOL[datatype]


@pytest.mark.gpu
@pytest.mark.parametrize("datatype", ["float", "double", "int", "long", "short", "byte"])
def test_ternary_select_matches_oracle(b200_driver, oracle_driver, datatype):
    """ternary-op! select: three tensors (dense, and with a broadcast row), tensor + constants in every
    position: bit-exact against the oracle."""
    npdt = np.dtype(pc.NP[datatype])
    rng = np.random.default_rng(72)
    if npdt.kind == "f":
        X, Y, Z = (rng.standard_normal((257, 1000)).astype(npdt) for _ in range(3))
    else:
        hi = min(np.iinfo(npdt).max, 1000)
        X, Y, Z = (rng.integers(-hi, hi, size=(257, 1000)).astype(npdt) for _ in range(3))
    row = Y[:1].copy()

    def run():
        x, y, z, r = (ct.to_tensor(v, datatype) for v in (X, Y, Z, row))
        outs = []
        for args in ((1.0, x, 2.0, y, 3.0, z), (1.0, x, 2.0, r, 1.0, z), (-1.0, x, 1.0, 0.0, 1.0, z),
                     (1.0, x, 1.0, y, 0.25, -3.0), (1.0, x, 2.0, 5.0, 1.0, -1.0)):
            d = ct.new_tensor([257, 1000], datatype)
            ct.ternary_op(d, *args, "select")
            outs.append(ct.to_array(d))
        return outs

    g, c = _on(b200_driver, datatype, run), _on(oracle_driver, datatype, run)
    for gv, cv in zip(g, c):
        assert np.array_equal(gv, cv)
    ref = np.where(X.astype(np.float64) >= 0, 3.0 * Z.astype(np.float64), 2.0 * Y.astype(np.float64))
    if npdt.kind == "f":
        assert pc.rel_err(g[0], ref.astype(npdt)) == 0.0


@pytest.mark.gpu
@pytest.mark.parametrize("datatype", ["float", "double"])
def test_batch_normalize_matches_oracle(b200_driver, oracle_driver, datatype):
    """batch-normalize! inference form, eltwise and spatial, incl. a zero variance and ragged sizes.  double:
    bit-exact against the oracle (same arithmetic).  float: the oracle (as the reference CPU backend) evaluates
    in double and rounds once, the B200 in single precision with three roundings: compared at 1e-5 (bound 1e-4)."""
    npdt = np.float32 if datatype == "float" else np.float64
    rng = np.random.default_rng(73)
    for shape in ((128, 500), (33, 7), (64, 64, 56 * 56), (3, 5, 9), (2, 3, 16, 10)):
        ch = shape[-1] if len(shape) == 2 else shape[-2]
        X = rng.standard_normal(shape).astype(npdt)
        mean = rng.standard_normal(ch).astype(npdt)
        var = np.abs(rng.standard_normal(ch)).astype(npdt)
        var[0] = 0
        gamma, beta = rng.standard_normal(ch).astype(npdt), rng.standard_normal(ch).astype(npdt)

        def run():
            out = ct.new_tensor(list(shape), datatype)
            ct.batch_normalize(out, ct.to_tensor(X, datatype), ct.to_tensor(mean, datatype), ct.to_tensor(var, datatype),
                               ct.to_tensor(gamma, datatype), ct.to_tensor(beta, datatype), 1e-3)
            return ct.to_array(out)

        g, c = _on(b200_driver, datatype, run), _on(oracle_driver, datatype, run)
        if datatype == "double":
            assert np.array_equal(g, c)
        else:
            assert pc.rel_err(g, c) <= 1e-5
        bshape = (1, ch) if len(shape) == 2 else (1,) * (len(shape) - 2) + (ch, 1)
        eps = np.float64(npdt(1e-3))
        ref = (X.astype(np.float64) - mean.reshape(bshape)) / np.sqrt(var.reshape(bshape).astype(np.float64) + eps) * \
            gamma.reshape(bshape) + beta.reshape(bshape)
        assert pc.rel_err(g.reshape(shape), ref) <= (1e-5 if datatype == "float" else 1e-12)


@pytest.mark.gpu
@pytest.mark.parametrize("datatype", ["float", "double"])
@pytest.mark.parametrize("pool_op", ["max", "avg", "avg-exc-pad"])
def test_pooling_forward_matches_oracle(b200_driver, oracle_driver, datatype, pool_op):
    """pooling-forward!: several geometries incl. ceil-mode output sizes, non-square windows and strides;
    bit-exact against the oracle (same position-by-position arithmetic)."""
    npdt = np.float32 if datatype == "float" else np.float64
    rng = np.random.default_rng(74)
    for (batch, ch, h, w, kw, kh, px, py, sx, sy, dim_op) in (
            (2, 4, 4, 4, 3, 3, 1, 1, 2, 2, "floor"), (3, 5, 13, 17, 3, 2, 1, 0, 2, 3, "ceil"),
            (2, 16, 56, 56, 3, 3, 1, 1, 2, 2, "ceil"), (1, 3, 9, 9, 2, 2, 0, 0, 2, 2, "floor"),
            (2, 2, 7, 7, 7, 7, 0, 0, 1, 1, "floor"), (2, 8, 20, 23, 3, 3, 1, 1, 1, 1, "floor"),
            (1, 4, 9, 10, 2, 2, 1, 1, 1, 1, "floor"), (3, 2, 11, 13, 3, 3, 1, 1, 2, 1, "ceil"),
            # rows that are multiples of 4 floats wide: the 16-byte-vector kernel (strides 1 / 2, pad 0 / 1)
            (2, 3, 12, 16, 2, 2, 0, 0, 2, 2, "floor"), (1, 2, 8, 8, 3, 3, 0, 0, 1, 1, "floor"),
            (2, 2, 10, 12, 3, 3, 1, 1, 1, 1, "floor"), (1, 3, 9, 20, 2, 2, 1, 1, 2, 2, "ceil"),
            (2, 3, 16, 64, 3, 3, 0, 0, 2, 2, "ceil"), (1, 2, 6, 8, 2, 2, 1, 0, 1, 2, "ceil")):
        X = rng.standard_normal((batch, ch, h, w)).astype(npdt)

        def run():
            desc = ct.pooling_descriptor(datatype, ch, kw, kh, px, py, sx, sy, dimension_op=dim_op, pool_op=pool_op)
            od = ct.get_convolution_output_dimensions(desc, h, w)
            out = ct.new_tensor([batch, ch, od["output-width"], od["output-height"]], datatype)
            ct.pooling_forward(out, 0.0, ct.to_tensor(X, datatype), desc)
            return ct.to_array(out)

        g, c = _on(b200_driver, datatype, run), _on(oracle_driver, datatype, run)
        # (a ceil-mode window that lies wholly in the padding averages 0 / 0 = NaN in the reference too)
        assert np.array_equal(g, c, equal_nan=True)


@pytest.mark.gpu
@pytest.mark.parametrize("datatype", ["float", "double"])
def test_mnist_convnet_matches_oracle(b200_driver, oracle_driver, datatype):
    """The reference's MNIST network shape end to end (conv, max-pool, batch-norm, ReLU, linear, softmax)."""
    run = pc.mnist_convnet_case(datatype)
    gpu = _on(b200_driver, datatype, run)
    cpu = _on(oracle_driver, datatype, lambda: run(fused=False))
    assert pc.rel_err(gpu.reshape(32, 10), cpu.reshape(32, 10)) <= pc.TOL[datatype]
    assert np.abs(gpu.reshape(32, 10).astype(np.float64).sum(axis=1) - 1.0).max() <= (1e-5 if datatype == "float" else 1e-12)


@pytest.mark.gpu
@pytest.mark.parametrize("M,N,K", [(300, 384, 256), (130, 1000, 500), (128, 256, 16), (513, 260, 4112), (1024, 4096, 4096),
                                   (1300, 520, 48),
                                   # 84 / 91 / 80 pair tiles on 74 clusters: each tile of the last round is reduced
                                   # by two clusters, one per K half (the third also drains mid-tile in both halves)
                                   (3072, 1792, 320), (3300, 1700, 272), (2560, 2048, 4160)])
@pytest.mark.parametrize("act", [None, "relu"])
@pytest.mark.parametrize("variant", [1, 2])
def test_presplit_layer_gemm(b200_driver, M, N, K, act, variant):
    """The pre-split layer GEMM (operands given as hi / lo matrices, result written as hi / lo) against the
    general fused kernel (same arithmetic: equal up to summation order) and against float64, on both of its
    kernels: 128-row tiles per CTA, and 256-row tiles on CTA pairs (ragged last pair: M = 130, 300, 513, 1300
    leave the second CTA of the last pair partly or wholly outside the matrix)."""
    rng = np.random.default_rng(M * 7 + N)
    A = rng.standard_normal((M, K)).astype(np.float32)
    W = (rng.standard_normal((N, K)) / np.sqrt(K)).astype(np.float32)
    bias = rng.standard_normal(N).astype(np.float32)
    stream = b200_driver.default_device().create_stream()
    stream.set_option("presplit-variant", variant)      # 1 = single-CTA tiles, 2 = CTA pairs
    with ct.with_stream(stream), ct.with_datatype("float"):
        a, w, b = ct.to_tensor(A), ct.to_tensor(W), ct.to_tensor(bias)
        a_lo, w_lo = ct.new_tensor([M, K]), ct.new_tensor([N, K])
        stream.split_lo(a_lo.buffer, a.buffer, M * K)
        stream.split_lo(w_lo.buffer, w.buffer, N * K)
        lo_host = ct.to_array(a_lo).reshape(M, K)
        hi_trunc = (A.view(np.uint32) & np.uint32(0xffffe000)).view(np.float32)
        assert np.array_equal(lo_host, A - hi_trunc)                      # lo = x - trunc_tf32(x), exact
        c, c_lo, ref = ct.new_tensor([M, N]), ct.new_tensor([M, N]), ct.new_tensor([M, N])
        for _ in range(2):
            stream.gemm_bias_act_presplit(c.buffer, c_lo.buffer, N, 1.0, a.buffer, a_lo.buffer, M, K, K, w.buffer,
                                          w_lo.buffer, N, K, 0.0, b.buffer, act)
        stream.gemm_bias_act(ref.buffer, N, False, True, 1.0, a.buffer, M, K, K, w.buffer, N, K, 0.0, b.buffer, act)
        got, got_lo, want = (ct.to_array(t).reshape(M, N) for t in (c, c_lo, ref))
    exact = A.astype(np.float64) @ W.astype(np.float64).T + bias
    if act == "relu":
        exact = np.maximum(exact, 0.0)
    assert pc.rel_err(got, exact) <= 1e-4
    assert pc.rel_err(got, want) <= 2e-5
    got_trunc = (got.view(np.uint32) & np.uint32(0xffffe000)).view(np.float32)
    assert np.array_equal(got_lo, got - got_trunc)


@pytest.mark.gpu
def test_presplit_mlp_matches_oracle(b200_driver, oracle_driver):
    """A 4-layer MLP through the pre-split layer GEMMs (weights split once, every layer writes its output
    split) against the oracle's unfused call sequence."""
    widths = [784, 1024, 1024, 1024, 1000]
    run_gpu, ref = pc.mlp_case("float", 300, widths, seed=77, bias_scale=0.1, presplit=True)
    run_cpu, _ = pc.mlp_case("float", 300, widths, seed=77, bias_scale=0.1, fused=False)
    gpu = _on(b200_driver, "float", run_gpu).reshape(300, 1000)
    cpu = _on(oracle_driver, "float", run_cpu).reshape(300, 1000)
    assert pc.rel_err(gpu, cpu) <= pc.TOL["float"]
    assert pc.rel_err(gpu, ref()) <= pc.TOL["float"]


@pytest.mark.parametrize("ta,tb", [(False, True), (True, False)], ids=["NT", "TN"])
def test_tensor_core_reads_fp32_words_truncated(b200_driver, ta, tb):
    """The fact the hi / lo split rests on: fed an fp32 word as tf32, the tensor core drops the low 13 mantissa
    bits (truncation, not rounding).  One-term run (no split) of the tcgen05 kernel against float64 products of
    (a) truncated and (b) round-to-nearest-tf32 inputs: it must agree with (a) to accumulation error and be far
    from (b); and hi + lo must rebuild every input exactly, so the three-term product loses nothing."""
    from cortex_b200._lib import call
    m, n, k = 256, 256, 512
    rng = np.random.default_rng(11)
    a_shape, b_shape = ((k, m) if ta else (m, k)), ((n, k) if tb else (k, n))
    A = rng.standard_normal(a_shape).astype(np.float32)
    B = rng.standard_normal(b_shape).astype(np.float32)
    stream = b200_driver.default_device().create_stream()
    with ct.with_stream(stream), ct.with_datatype("float"):
        a, b, c = ct.to_tensor(A), ct.to_tensor(B), ct.new_tensor([m, n])
        # extents are those of op(A) (m x k) and op(B) (.. x n); pitches those of the stored matrices
        call("cb200_gemm_f32_variant", stream.handle, 1, 1, c.buffer.ptr, n, int(ta), int(tb), 1.0, a.buffer.ptr,
             m, k, a_shape[1], b.buffer.ptr, n, b_shape[1], 0.0)
        got = ct.to_array(c).reshape(m, n).astype(np.float64)
    stream.sync()

    def trunc(x):
        return (x.view(np.uint32) & np.uint32(0xffffe000)).view(np.float32)

    def rna(x):   # round to nearest, ties away: add half an ulp of the 10-bit mantissa, then truncate
        return ((x.view(np.uint32) + np.uint32(0x1000)) & np.uint32(0xffffe000)).view(np.float32)

    def product(f):
        a64, b64 = f(A).astype(np.float64), f(B).astype(np.float64)
        return (a64.T if ta else a64) @ (b64.T if tb else b64)

    err_trunc, err_rna = pc.rel_err(got, product(trunc)), pc.rel_err(got, product(rna))
    assert err_trunc <= 2e-5, err_trunc
    assert err_rna >= 20 * err_trunc, (err_trunc, err_rna)
    for x in (A, B):
        hi = trunc(x)
        assert np.array_equal(hi.astype(np.float64) + (x - hi).astype(np.float64), x.astype(np.float64))


@pytest.mark.parametrize("M,N,K,act", [(128, 500, 784, "relu"), (128, 24, 500, None), (64, 1000, 2048, "tanh"),
                                       (300, 72, 1040, None), (8192, 125, 4096, None)])
@pytest.mark.parametrize("handover", [0, 1])
def test_small_gemm_is_sliced_over_k(b200_driver, M, N, K, act, handover):
    """Problems with fewer tiles than half the SMs are reduced by several CTAs per tile, each over a slice of K,
    combined by whichever finishes last (in slice order: the result does not depend on who that is).  Config 1's
    first layer, a 24-column head, a wide-K case, a ragged one and the 8-way column-sharded head; twice in a row (the per-tile
    counters must be left clear), fused bias + activation, against float64."""
    rng = np.random.default_rng(M + N + K)
    A = rng.standard_normal((M, K)).astype(np.float32)
    W = (rng.standard_normal((N, K)) / np.sqrt(K)).astype(np.float32)
    bias = rng.standard_normal(N).astype(np.float32)
    stream = b200_driver.default_device().create_stream()
    # 0: up to 8 slices meet in distributed shared memory (the slices of a tile launched as one cluster); 1: through L2
    stream.set_option("gemm-slice-handover", handover)
    outs = []
    with ct.with_stream(stream), ct.with_datatype("float"):
        a, w, b = ct.to_tensor(A), ct.to_tensor(W), ct.to_tensor(bias)
        for _ in range(2):
            c = ct.to_tensor(np.full((M, N), np.nan, np.float32))
            stream.gemm_bias_act(c.buffer, N, False, True, 1.0, a.buffer, M, K, K, w.buffer, N, K, 0.0, b.buffer, act)
            outs.append(ct.to_array(c).reshape(M, N))
    exact = A.astype(np.float64) @ W.astype(np.float64).T + bias
    if act == "relu":
        exact = np.maximum(exact, 0.0)
    elif act == "tanh":
        exact = np.tanh(exact)
    assert pc.rel_err(outs[0], exact) <= pc.TOL["float"]
    assert np.array_equal(outs[0], outs[1])
    stream.sync()       # raises if a launch reported a status


@pytest.mark.parametrize("datatype", ["float", "double"])
@pytest.mark.parametrize("M,N,K", [(128, 10, 500), (1, 1, 1), (37, 16, 333), (4096, 3, 64), (200, 16, 16384),
                                   (128, 40, 500), (64, 1000, 256)])
@pytest.mark.parametrize("act", [None, "relu", "logistic", "softmax"])
def test_classifier_head_with_fused_softmax(b200_driver, datatype, M, N, K, act):
    """gemm_bias_act on heads of up to 16 columns runs on the one-CTA-per-row kernel, which also normalises the
    row when the activation is softmax; wider heads take the layer kernel and a softmax! launch behind the same
    call.  alpha, beta and a pitched output included; against float64; twice for run-to-run equality."""
    rng = np.random.default_rng(7 * M + N + K)
    npdt = pc.NP[datatype]
    A = rng.standard_normal((M, K)).astype(npdt)
    W = (rng.standard_normal((N, K)) / np.sqrt(K)).astype(npdt)
    bias = rng.standard_normal(N).astype(npdt)
    ldc = N + 3
    C0 = rng.standard_normal((M, ldc)).astype(npdt)
    alpha, beta = 1.25, 0.5
    stream = b200_driver.default_device().create_stream()
    outs = []
    with ct.with_stream(stream), ct.with_datatype(datatype):
        a, w, b = ct.to_tensor(A, datatype), ct.to_tensor(W, datatype), ct.to_tensor(bias, datatype)
        for _ in range(2):
            c = ct.to_tensor(C0, datatype)
            stream.gemm_bias_act(c.buffer, ldc, False, True, alpha, a.buffer, M, K, K, w.buffer, N, K, beta, b.buffer, act)
            outs.append(ct.to_array(c).reshape(M, ldc))
    z = alpha * (A.astype(np.float64) @ W.astype(np.float64).T) + beta * C0[:, :N].astype(np.float64) + bias
    if act == "relu":
        z = np.maximum(z, 0.0)
    elif act == "logistic":
        z = 1.0 / (1.0 + np.exp(-z))
    elif act == "softmax":
        e = np.exp(z - z.max(axis=1, keepdims=True))
        z = e / e.sum(axis=1, keepdims=True)
    assert pc.rel_err(outs[0][:, :N], z) <= pc.TOL[datatype]
    assert np.array_equal(outs[0][:, N:], C0[:, N:])          # the pitch padding is not touched
    assert np.array_equal(outs[0], outs[1])
    stream.sync()


@pytest.mark.parametrize("M,N,K,ta,tb", [(256, 256, 8192, False, True), (300, 72, 50000, False, True),
                                         (500, 784, 20000, True, False), (64, 24, 140000, False, True),
                                         (1024, 1024, 8192, False, True)])
def test_long_reduction_is_cut_inside_one_launch(b200_driver, M, N, K, ta, tb):
    """gemm! with K above 4096: tcgen05 accumulates with truncation, so the reduction is cut into pieces of at
    most 4096 joined by round-to-nearest adds.  Problems with few output tiles get the pieces as K slices of one
    launch (a weight gradient summed over a whole batch), the others as chained launches; all-positive operands
    are the worst case for the drift.  Against float64, twice for run-to-run equality."""
    rng = np.random.default_rng(M + N + K)
    A = (rng.random((K, M) if ta else (M, K)) + 0.5).astype(np.float32)
    B = (rng.random((N, K) if tb else (K, N)) + 0.5).astype(np.float32)
    C0 = rng.standard_normal((M, N)).astype(np.float32)
    stream = b200_driver.default_device().create_stream()
    outs = []
    with ct.with_stream(stream), ct.with_datatype("float"):
        a, b = ct.to_tensor(A), ct.to_tensor(B)
        for _ in range(2):
            c = ct.to_tensor(C0)
            before = stream.launch_count()
            ct.gemm(c, ta, tb, 0.75, a, b, 0.5)
            launches = stream.launch_count() - before
            outs.append(ct.to_array(c).reshape(M, N))
    opA = A.T.astype(np.float64) if ta else A.astype(np.float64)
    opB = B.T.astype(np.float64) if tb else B.astype(np.float64)
    exact = 0.75 * (opA @ opB) + 0.5 * C0
    assert pc.rel_err(outs[0], exact) <= pc.TOL["float"]
    assert np.array_equal(outs[0], outs[1])
    if M * N <= 256 * 256:
        assert launches <= 2, launches          # slices inside the launch, not one launch per 4096 of K
    stream.sync()


def test_gemm_tile_width_and_slices_are_interchangeable(b200_driver):
    """The launch picks the tile width and the number of K slices from a timing model; every pair it could pick
    (forced here through the stream options) computes the same product within the fp32 bound, ragged edges and
    alpha / beta included.  Values outside the option's domain are rejected."""
    M, N, K = 300, 328, 1040
    rng = np.random.default_rng(77)
    A = rng.standard_normal((M, K)).astype(np.float32)
    B = rng.standard_normal((N, K)).astype(np.float32)
    C0 = rng.standard_normal((M, N)).astype(np.float32)
    exact = 1.5 * (A.astype(np.float64) @ B.astype(np.float64).T) + 0.5 * C0
    stream = b200_driver.default_device().create_stream()
    with ct.with_stream(stream), ct.with_datatype("float"):
        a, b = ct.to_tensor(A), ct.to_tensor(B)
        for tile_n in (0, 64, 128, 256):
            for slices in (0, 1, 2, 4):
                outs = []
                for handover in (0, 1):      # slices meeting in distributed shared memory (one cluster per tile) / through L2
                    stream.set_option("gemm-tile-n", tile_n)
                    stream.set_option("gemm-k-slices", slices)
                    stream.set_option("gemm-slice-handover", handover)
                    c = ct.to_tensor(C0)
                    ct.gemm(c, False, True, 1.5, a, b, 0.5)
                    outs.append(ct.to_array(c).reshape(M, N))
                    assert pc.rel_err(outs[-1], exact) <= pc.TOL["float"], (tile_n, slices, handover)
                assert np.array_equal(outs[0], outs[1]), (tile_n, slices)     # both sum the slices in slice order
        stream.set_option("gemm-tile-n", 0)
        stream.set_option("gemm-k-slices", 0)
        stream.set_option("gemm-slice-handover", 0)
        with pytest.raises(Exception):
            stream.set_option("gemm-tile-n", 96)
    stream.sync()


@pytest.mark.parametrize("datatype", ["float", "double"])
@pytest.mark.parametrize("args", [
    dict(batch=2, cin=16, hw=56, cout=64),                       # config 4's geometry: the patch kernel on the NCHW input
    dict(batch=3, cin=16, hw=13, cout=40, k=5, pad=2),           # patch kernel with overhang
    dict(batch=2, cin=32, hw=17, cout=130, k=3, pad=1, stride=2),  # strided: the thread-gathered kernel
    dict(batch=2, cin=3, hw=8, cout=4, k=2, pad=0, stride=2),    # three input channels
    dict(batch=2, cin=16, hw=30, cout=24, k=3, pad=1),           # rows not a multiple of 4: behind the layout pre-pass
], ids=lambda a: "x".join(str(v) for v in a.values()))
def test_conv_bias_relu_in_the_epilogue(b200_driver, oracle_driver, datatype, args):
    """convolution_forward_bias_act: the layer's bias add and ReLU inside the convolution's epilogue give the bits
    of the three-call sequence (conv, binary-op! +, ReLU) on every kernel route, and match the oracle's sequence."""
    fused_run, ref = pc.conv_case(datatype, bias_scale=0.3, fused=True, **args)
    plain_run, _ = pc.conv_case(datatype, bias_scale=0.3, **args)
    cpu = _on(oracle_driver, datatype, plain_run)
    for options in (None, {"conv-route": 1}, {"conv-route": 2}, {"conv-route": 3}):
        fused = _on(b200_driver, datatype, fused_run, options)
        plain = _on(b200_driver, datatype, plain_run, options)
        assert np.array_equal(fused, plain), options
        assert pc.rel_err(fused, cpu) <= pc.TOL[datatype]
        assert pc.rel_err(fused, ref()) <= pc.TOL[datatype]


def test_conv_epilogue_activations_and_accumulate(b200_driver):
    """The other epilogue activations and out_alpha: act(conv + out_alpha * out + bias) against float64."""
    rng = np.random.default_rng(9)
    batch, cin, hw, cout = 2, 16, 12, 20
    X = rng.standard_normal((batch, cin, hw, hw)).astype(np.float32)
    W = (rng.standard_normal((cout, cin * 9)) * 0.1).astype(np.float32)
    b = rng.standard_normal(cout).astype(np.float32)
    O0 = rng.standard_normal((batch, cout, hw, hw)).astype(np.float32)
    xp = np.zeros((batch, cin, hw + 2, hw + 2)); xp[:, :, 1:-1, 1:-1] = X
    conv = np.zeros((batch, cout, hw, hw))
    W4 = W.reshape(cout, cin, 3, 3).astype(np.float64)
    for ky in range(3):
        for kx in range(3):
            conv += np.einsum("bchw,oc->bohw", xp[:, :, ky:ky + hw, kx:kx + hw], W4[:, :, ky, kx])
    z = conv + 0.5 * O0 + b[None, :, None, None]
    want = {None: z, "relu": np.maximum(z, 0), "tanh": np.tanh(z), "logistic": 1 / (1 + np.exp(-z))}
    stream = b200_driver.default_device().create_stream()
    with ct.with_stream(stream), ct.with_datatype("float"):
        desc = ct.convolution_descriptor("float", cout, cin, 3, 3, 1, 1, 1, 1)
        x, w, bias = ct.to_tensor(X), ct.to_tensor(W), ct.to_tensor(b)
        for act, exact in want.items():
            out = ct.to_tensor(O0)
            ct.convolution_forward_bias_act(out, 0.5, x, w, desc, bias, act)
            assert pc.rel_err(ct.to_array(out).reshape(exact.shape), exact) <= pc.TOL["float"], act
        with pytest.raises(Exception):
            ct.convolution_forward_bias_act(out, 0.0, x, w, desc, bias, "softmax")
    stream.sync()
