"""pooling-backward! and the training half of batch normalisation on the B200 against the CPU oracle,
through the C ABI.

Pooling backward is a gather over the reference's scatter loop in the same visiting order: bit for bit,
also when it accumulates (input-grad-alpha = 1) onto a non-zero gradient, which is what the CPU backend
always does.  Batch-normalisation statistics: the elementwise form sums in the reference's order (bit for
bit up to the power function in the gradient); the spatial form uses a tree reduction in double, so the
comparison is at 1e-12 relative (double) / 1e-5 (float, bound 1e-4).  lrn against the oracle's restatement of the
published definition.  Then the layers together: one training pass of the reference's MNIST network against the
oracle's pass, and forty Adam steps on a fixed batch (the loss must fall)."""
import numpy as np
import pytest

import parity_cases as pc
from cortex_b200 import tensor as ct

pytestmark = pytest.mark.gpu
NP = {"float": np.float32, "double": np.float64}
TOL = {"float": 1e-5, "double": 1e-12}


def _run(driver, datatype, fn):
    stream = driver.default_device().create_stream()
    with ct.with_stream(stream), ct.with_datatype(datatype):
        out = fn()
    stream.sync()
    return out


def _rel(a, b):
    a, b = np.asarray(a, np.float64).reshape(-1), np.asarray(b, np.float64).reshape(-1)
    scale = np.maximum(np.abs(b), np.sqrt(np.mean(b * b)) + 1e-300)
    return float(np.max(np.abs(a - b) / scale)) if a.size else 0.0


POOL_GEOMETRIES = (
    # batch, channels, h, w, kw, kh, pad_x, pad_y, stride_x, stride_y, dimension-op
    (2, 4, 4, 4, 3, 3, 1, 1, 2, 2, "floor"), (3, 5, 13, 17, 3, 2, 1, 0, 2, 3, "ceil"),
    (2, 16, 56, 56, 3, 3, 1, 1, 2, 2, "ceil"), (1, 3, 9, 9, 2, 2, 0, 0, 2, 2, "floor"),
    (2, 2, 7, 7, 7, 7, 0, 0, 1, 1, "floor"), (2, 8, 20, 23, 3, 3, 1, 1, 1, 1, "floor"),
    (1, 4, 9, 10, 2, 2, 1, 1, 1, 1, "floor"), (3, 2, 11, 13, 3, 3, 1, 1, 2, 1, "ceil"),
    (1, 2, 10, 10, 2, 2, 0, 0, 3, 3, "floor"),       # stride > window: some inputs belong to no window
    (2, 3, 24, 24, 2, 2, 0, 0, 2, 2, "floor"),       # the reference MNIST network's pooling layers
    # vector-width rows with the window / stride pairs that have their own kernels, every padding remainder
    (2, 4, 16, 16, 3, 3, 0, 0, 2, 2, "ceil"), (1, 3, 12, 12, 3, 3, 2, 2, 2, 2, "floor"),
    (2, 3, 8, 8, 3, 3, 1, 1, 1, 1, "floor"), (1, 4, 8, 8, 2, 2, 1, 1, 2, 2, "floor"), (1, 2, 8, 12, 3, 3, 1, 0, 2, 2, "ceil"),
)


@pytest.mark.parametrize("datatype", ["float", "double"])
@pytest.mark.parametrize("pool_op", ["max", "avg", "avg-exc-pad"])
@pytest.mark.parametrize("alpha", [0.0, 1.0])
def test_pooling_backward_matches_oracle(b200_driver, oracle_driver, datatype, pool_op, alpha):
    rng = np.random.default_rng(91)
    for (batch, ch, h, w, kw, kh, px, py, sx, sy, dim_op) in POOL_GEOMETRIES:
        # quantised inputs so that the maximum is shared by several positions of a window now and then
        X = np.round(rng.standard_normal((batch, ch, h, w)) * 4).astype(NP[datatype]) / 4
        G0 = rng.standard_normal((batch, ch, h, w)).astype(NP[datatype]) if alpha else np.zeros((batch, ch, h, w), NP[datatype])
        seed = int(rng.integers(1 << 30))

        def run():
            desc = ct.pooling_descriptor(datatype, ch, kw, kh, px, py, sx, sy, dimension_op=dim_op, pool_op=pool_op)
            od = ct.get_convolution_output_dimensions(desc, h, w)
            shape = [batch, ch, od["output-width"], od["output-height"]]
            inp = ct.to_tensor(X, datatype)
            out = ct.new_tensor(shape, datatype)
            ct.pooling_forward(out, 0.0, inp, desc)
            og = ct.to_tensor(np.random.default_rng(seed).standard_normal(shape).astype(NP[datatype]), datatype)
            in_grad = ct.to_tensor(G0, datatype)
            ct.pooling_backward(in_grad, alpha, inp, out, og, desc)
            return ct.to_array(in_grad)

        g, c = _run(b200_driver, datatype, run), _run(oracle_driver, datatype, run)
        assert np.array_equal(g, c, equal_nan=True), (pool_op, (batch, ch, h, w, kw, kh, px, py, sx, sy, dim_op))


def test_pooling_backward_rejects_mismatched_shapes(b200_driver):
    def run():
        desc = ct.pooling_descriptor("float", 2, 2, 2, 0, 0, 2, 2, dimension_op="floor", pool_op="max")
        inp, out = ct.new_tensor([1, 2, 8, 8], "float"), ct.new_tensor([1, 2, 4, 4], "float")
        with pytest.raises(Exception):
            ct.pooling_backward(ct.new_tensor([1, 2, 8, 6], "float"), 0.0, inp, out, out, desc)
    _run(b200_driver, "float", run)


BN_SHAPES = ([4, 3], [128, 800], [1, 7], [33, 130], [2, 3, 4], [8, 20, 576], [4, 16, 56 * 56], [3, 5, 1], [1, 64, 4097],
             [2, 3, 4, 5])


def _bn_case(datatype, shape, seed):
    rng = np.random.default_rng(seed)
    channels = shape[1] if len(shape) == 2 else shape[-2]
    X = (rng.standard_normal(shape) * 2 + 0.5).astype(NP[datatype])
    OG = rng.standard_normal(shape).astype(NP[datatype])
    vec = lambda lo, hi: rng.uniform(lo, hi, channels).astype(NP[datatype])
    stats = {"rm": vec(-1, 1), "rv": vec(0.5, 2), "scale": vec(0.5, 1.5), "bias": vec(-1, 1)}

    def run():
        inp, og = ct.to_tensor(X, datatype), ct.to_tensor(OG, datatype)
        out, in_grad = ct.new_tensor(shape, datatype), ct.new_tensor(shape, datatype)
        bm, bv = ct.new_tensor([channels], datatype), ct.new_tensor([channels], datatype)
        rm, rv = ct.to_tensor(stats["rm"], datatype), ct.to_tensor(stats["rv"], datatype)
        scale, bias = ct.to_tensor(stats["scale"], datatype), ct.to_tensor(stats["bias"], datatype)
        sg, bg = ct.new_tensor([channels], datatype), ct.new_tensor([channels], datatype)
        ct.batch_normalize_update_and_apply(out, inp, bm, bv, rm, rv, 0.3, scale, bias, 1e-3)
        ct.batch_normalize_gradients(in_grad, sg, bg, og, out, inp, bm, bv, scale, bias, 1e-3)
        return {k: ct.to_array(t) for k, t in (("out", out), ("batch-means", bm), ("batch-variances", bv),
                                               ("running-means", rm), ("running-variances", rv), ("in-grad", in_grad),
                                               ("scale-grad", sg), ("bias-grad", bg))}
    return run


@pytest.mark.parametrize("datatype", ["float", "double"])
@pytest.mark.parametrize("shape", BN_SHAPES, ids=lambda s: "x".join(map(str, s)))
def test_batch_normalize_training_matches_oracle(b200_driver, oracle_driver, datatype, shape):
    run = _bn_case(datatype, shape, 17 + len(shape) + shape[0])
    g, c = _run(b200_driver, datatype, run), _run(oracle_driver, datatype, run)
    eltwise = len(shape) == 2
    for key in ("batch-means", "batch-variances", "running-means", "running-variances"):
        if eltwise:       # same summation order: identical statistics
            assert np.array_equal(g[key], c[key]), key
        else:
            assert _rel(g[key], c[key]) <= TOL[datatype], (key, _rel(g[key], c[key]))
    for key in ("out", "scale-grad", "bias-grad"):
        assert _rel(g[key], c[key]) <= TOL[datatype], (key, _rel(g[key], c[key]))
    # the input gradient is a difference of nearly equal terms: measured against the size of those terms
    terms = np.abs(np.asarray(c["in-grad"], np.float64)).max() + 1.0
    assert np.abs(np.asarray(g["in-grad"], np.float64) - np.asarray(c["in-grad"], np.float64)).max() / terms <= TOL[datatype]


@pytest.mark.parametrize("datatype", ["float", "double"])
def test_batch_normalize_update_normalises(b200_driver, datatype):
    """Size-independent property at a large size: the output of update-and-apply with scale 1 / bias 0 has
    per-channel mean 0 and variance N / (N + eps-ish) ~ 1; average factor 1 makes the running statistics the
    batch statistics (unbiased variance)."""
    shape = [16, 32, 64 * 64]
    rng = np.random.default_rng(5)
    X = (rng.standard_normal(shape) * 3 + 2).astype(NP[datatype])

    def run():
        inp, out = ct.to_tensor(X, datatype), ct.new_tensor(shape, datatype)
        bm, bv, rm, rv = (ct.new_tensor([32], datatype) for _ in range(4))
        scale, bias = ct.to_tensor(np.ones(32), datatype), ct.to_tensor(np.zeros(32), datatype)
        ct.batch_normalize_update_and_apply(out, inp, bm, bv, rm, rv, 1.0, scale, bias, 1e-4)
        return ct.to_array(out), ct.to_array(bm), ct.to_array(bv), ct.to_array(rm), ct.to_array(rv)

    out, bm, bv, rm, rv = _run(b200_driver, datatype, run)
    x64 = X.astype(np.float64)
    n = shape[0] * shape[2]
    tol = 1e-4 if datatype == "float" else 1e-10
    assert np.allclose(bm, x64.mean(axis=(0, 2)), rtol=tol, atol=tol)
    assert np.allclose(bv, x64.var(axis=(0, 2)), rtol=tol, atol=tol)
    assert np.array_equal(rm, bm)
    assert np.allclose(rv, x64.var(axis=(0, 2)) * n / (n - 1), rtol=tol, atol=tol)
    o = np.asarray(out, np.float64).reshape(shape)
    assert np.abs(o.mean(axis=(0, 2))).max() <= 10 * tol
    assert np.abs(o.var(axis=(0, 2)) - 1.0).max() <= 1e-3


@pytest.mark.parametrize("datatype", ["float", "double"])
@pytest.mark.parametrize("shape,n", [([2, 3, 2, 2], 1), ([2, 3, 2, 2], 2), ([2, 7, 5, 3], 5), ([3, 16, 9, 9], 4),
                                     ([5, 6, 7], 3), ([2, 2, 4, 3, 3], 9), ([1, 96, 27, 27], 5),
                                     # 4096 and more (batch entry, pixel) columns: the forward walks each column with the
                                     # window in registers
                                     ([16, 24, 20, 20], 5), ([16, 24, 20, 20], 2), ([4, 8, 40, 40], 8), ([8, 3, 32, 32], 1)],
                         ids=lambda v: "x".join(map(str, v)) if isinstance(v, list) else "n%d" % v)
def test_lrn_matches_oracle(b200_driver, oracle_driver, datatype, shape, n):
    """lrn-forward! / lrn-backward!: both sides evaluate in double and round once; compared at the backend's
    bounds (the power function differs in the last bits between the two maths libraries)."""
    rng = np.random.default_rng(3 + n)
    X = rng.standard_normal(shape).astype(NP[datatype])
    DY = rng.standard_normal(shape).astype(NP[datatype])

    def run():
        inp, dy = ct.to_tensor(X, datatype), ct.to_tensor(DY, datatype)
        out, dx = ct.new_tensor(shape, datatype), ct.new_tensor(shape, datatype)
        desc = ct.lrn_descriptor(n=n, k=2, alpha=0.3, beta=0.75)
        ct.lrn_forward(out, inp, desc)
        ct.lrn_backward(dx, out, inp, dy, desc)
        return ct.to_array(out), ct.to_array(dx)

    (g_out, g_dx), (c_out, c_dx) = _run(b200_driver, datatype, run), _run(oracle_driver, datatype, run)
    assert _rel(g_out, c_out) <= TOL[datatype]
    assert _rel(g_dx, c_dx) <= TOL[datatype]


@pytest.mark.parametrize("datatype", ["float", "double"])
def test_mnist_convnet_training_pass_matches_oracle(b200_driver, oracle_driver, datatype):
    """The reference's MNIST network (conv, max-pool, batch-norm, ReLU, conv, max-pool, batch-norm, linear + ReLU,
    linear, softmax) through one training pass on both backends: output with batch statistics, updated running
    statistics, and the gradient of every parameter.  The loss gradient fed to the B200 pass is the one the oracle
    pass built, so both differentiate the same function at the same point."""
    run = pc.mnist_convnet_training_case(datatype)
    cpu, _ = _run(oracle_driver, datatype, run)
    gpu, _ = _run(b200_driver, datatype, run)
    assert set(cpu) == set(gpu) and len(cpu) >= 15
    for key in sorted(cpu):
        if key in ("layer0-bias-gradient", "layer4-bias-gradient"):
            # a bias in front of a batch-norm layer has gradient zero (the layer removes the mean): both sides hold
            # rounding noise only
            assert np.abs(gpu[key]).max() <= (1e-5 if datatype == "float" else 1e-12), key
            continue
        err = pc.rel_err(gpu[key], cpu[key])
        assert err <= (2e-4 if datatype == "float" else 1e-10), (key, err)


def test_mnist_convnet_learns_a_batch(b200_driver):
    """End to end on the B200: forward with batch statistics, backward through every layer, Adam steps on every
    parameter (one optimiser state buffer for the whole network, stepped per layer at its offset, as the reference's
    compute binding does).  Forty steps on one fixed batch must cut the cross-entropy loss by more than half."""
    from cortex_b200 import nn, optimize
    dt, batch = "float", 32
    rng = np.random.default_rng(77)
    X = rng.random((batch, 1, 28, 28)).astype(np.float32)
    labels = rng.integers(0, 10, size=batch)
    onehot = np.zeros((batch, 10), np.float32)
    onehot[np.arange(batch), labels] = 1
    he = lambda shape, fan_in: (rng.standard_normal(shape) * np.sqrt(2.0 / fan_in)).astype(np.float32)

    def run():
        t = lambda a: ct.to_tensor(a, dt)
        bn = lambda n: nn.BatchNormalization(t(np.zeros(n)), t(np.ones(n)), t(np.ones(n)), t(np.zeros(n)), epsilon=1e-3)
        layers = [("conv", nn.Convolution(t(he((20, 25), 25)), t(np.zeros(20)), (5, 5), (0, 0), (1, 1), 1, 20, dt)),
                  ("pool", nn.Pooling(20, (2, 2), (0, 0), (2, 2), dt)), ("bn", bn(20)), ("relu",),
                  ("conv", nn.Convolution(t(he((50, 500), 500)), t(np.zeros(50)), (5, 5), (0, 0), (1, 1), 20, 50, dt)),
                  ("pool", nn.Pooling(50, (2, 2), (0, 0), (2, 2), dt)), ("flatten",), ("bn", bn(800)),
                  ("linear", nn.Linear(t(he((500, 800), 800)), t(np.zeros(500))), "relu"),
                  ("linear", nn.Linear(t(he((10, 500), 500)), t(np.zeros(10))), None), ("softmax",)]
        net = nn.ConvNet(layers, fused=False)
        params = []                                    # (parameter tensor, key of its gradient, layer index)
        for idx, spec in enumerate(layers):
            if spec[0] in ("conv", "linear"):
                params += [(spec[1].weights, "weights", idx), (spec[1].bias, "bias", idx)]
            elif spec[0] == "bn":
                params += [(spec[1].scale, "scale", idx), (spec[1].bias, "bias", idx)]
        total = sum(p.ecount() for p, _k, _i in params)
        state = {"m": ct.new_tensor([total], datatype=dt), "v": ct.new_tensor([total], datatype=dt)}
        adam = optimize.Adam(alpha=0.003)
        x = t(X)
        losses = []

        def loss_gradient(out):        # cross-entropy on the softmax output: (p - onehot) / batch at the softmax INPUT
            probs = ct.to_array(out).reshape(batch, 10)
            losses.append(float(-np.log(np.maximum(probs[np.arange(batch), labels], 1e-30)).mean()))
            return t((probs - onehot) / batch)

        for _ in range(40):
            _out, _g, grads = net.train_forward_backward(x, loss_gradient)
            adam.batch_update()
            offset = 0
            for p, key, idx in params:
                adam.compute_parameters(state, 1.0, offset, grads[idx][key], p)
                offset += p.ecount()
        return losses

    losses = _run(b200_driver, dt, run)
    assert np.isfinite(losses).all()
    assert losses[-1] < 0.5 * losses[0], (losses[0], losses[-1])
