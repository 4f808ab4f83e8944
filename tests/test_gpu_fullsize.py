"""The benchmark configurations at their FULL sizes, checked through properties that do not need a
full-size CPU run: sampled entries against float64 dot products, exact scaling by powers of two,
bit-exact single-rounding elementwise results against numpy, row sums of softmax.
Tolerances as everywhere: bit-exact for copies / single-rounding ops, |gpu - ref| / max(|ref|, rms(ref))
<= 1e-4 for fp32 and <= 1e-12 for fp64."""
import numpy as np
import pytest

from cortex_b200 import nn
from cortex_b200 import tensor as ct
from cortex_b200.dimensions import ALL

pytestmark = pytest.mark.gpu

TOL = {"float": 1e-4, "double": 1e-12}
NP = {"float": np.float32, "double": np.float64}


def _stream(b200_driver):
    return b200_driver.default_device().create_stream()


def _sample_err(got, ref_fn, idx, scale):
    ref = np.array([ref_fn(i, j) for i, j in idx])
    g = np.array([got[i, j] for i, j in idx], np.float64)
    return float(np.abs(g - ref).max() / scale)


@pytest.mark.parametrize("datatype", ["float", "double"])
@pytest.mark.parametrize("ta,tb", [(False, False), (False, True), (True, False), (True, True)],
                         ids=["NN", "NT", "TN", "TT"])
def test_gemm_4096_cubed_sampled_and_exact_scaling(b200_driver, datatype, ta, tb):
    """Config 2: C = 1.5 op(A) op(B) + 0.5 C at M = N = K = 4096, dense and on 4224-pitch sub-views."""
    n = 4096
    dt = NP[datatype]
    rng = np.random.default_rng(2024)
    A = rng.standard_normal((n, n)).astype(dt)
    B = rng.standard_normal((n, n)).astype(dt)
    C0 = rng.standard_normal((n, n)).astype(dt)
    opA = A.T if ta else A
    opB = B.T if tb else B
    idx = [(int(i), int(j)) for i, j in rng.integers(0, n, size=(1500, 2))]

    def ref(i, j):
        return 1.5 * np.dot(opA[i, :].astype(np.float64), opB[:, j].astype(np.float64)) + 0.5 * float(C0[i, j])

    scale = float(np.sqrt(1.5 ** 2 * n + 0.25))           # rms of the result for N(0,1) inputs
    stream = _stream(b200_driver)
    with ct.with_stream(stream), ct.with_datatype(datatype):
        a, b = ct.to_tensor(A), ct.to_tensor(B)
        c = ct.to_tensor(C0)
        ct.gemm(c, ta, tb, 1.5, a, b, 0.5)
        got = ct.to_array(c).reshape(n, n)
        assert _sample_err(got, ref, idx, scale) <= TOL[datatype]
        # scaling an operand by a power of two scales every product exactly: bit-exact property
        c2 = ct.new_tensor([n, n])
        ct.gemm(c2, ta, tb, 1.0, a, b, 0.0)
        a4 = ct.to_tensor(A * dt(4.0))
        c3 = ct.new_tensor([n, n])
        ct.gemm(c3, ta, tb, 1.0, a4, b, 0.0)
        assert np.array_equal(ct.to_array(c3), ct.to_array(c2) * dt(4.0))
        # the same product on pitched windows (row stride 4224) of larger backing buffers
        pitch = 4224
        big = [ct.to_tensor(np.pad(M_, ((0, 0), (0, pitch - n)))) for M_ in (A, B, C0)]
        va, vb, vc = (ct.submatrix(t, 0, n, 0, n) for t in big)
        ct.gemm(vc, ta, tb, 1.5, va, vb, 0.5)
        backing = ct.to_array(big[2]).reshape(n, pitch)
        assert np.array_equal(backing[:, :n], got)         # same kernel, same tiles: identical bits
        assert not backing[:, n:].any()                    # the frame beyond the window is untouched


def test_broadcast_eltwise_reduce_gather_full_size(b200_driver):
    """Config 3: [8192, 4096] + bias row, ReLU, row max / sum, int32 gather of 8192 random rows."""
    rows, cols = 8192, 4096
    rng = np.random.default_rng(303)
    X = rng.standard_normal((rows, cols), dtype=np.float32)
    bias = (rng.standard_normal((1, cols)) * 0.1).astype(np.float32)
    ids = rng.integers(0, rows, size=rows, dtype=np.int32)
    stream = _stream(b200_driver)
    with ct.with_stream(stream), ct.with_datatype("float"):
        x, b = ct.to_tensor(X), ct.to_tensor(bias)
        y = ct.new_tensor([rows, cols])
        ct.binary_op(y, 1.0, x, 1.0, b, "+")
        want = X + bias                                    # one fp32 rounding per element, as on the device
        assert np.array_equal(ct.to_array(y).reshape(rows, cols), want)
        ct.binary_op(y, 1.0, y, 1.0, 0, "max")
        want = np.maximum(want, np.float32(0))
        assert np.array_equal(ct.to_array(y).reshape(rows, cols), want)
        mx, sm = ct.new_tensor([rows, 1]), ct.new_tensor([rows, 1])
        ct.unary_reduce(mx, 1.0, y, "max")
        ct.unary_reduce(sm, 1.0, y, "sum")
        assert np.array_equal(ct.to_array(mx).reshape(rows), want.max(axis=1))
        ref_sum = want.astype(np.float64).sum(axis=1)
        assert np.abs(ct.to_array(sm).reshape(rows) - ref_sum).max() / np.abs(ref_sum).max() <= 1e-6
        p = ct.new_tensor([rows, cols])
        ct.softmax(p, y)
        probs = ct.to_array(p).reshape(rows, cols)
        assert np.abs(probs.astype(np.float64).sum(axis=1) - 1.0).max() <= 1e-5
        e = np.exp(want[:64].astype(np.float64) - want[:64].max(axis=1, keepdims=True))
        assert np.abs(probs[:64] - e / e.sum(axis=1, keepdims=True)).max() <= 1e-4 * (e / e.sum(axis=1, keepdims=True)).max()
        idx = ct.to_tensor(ids, datatype="int")
        g = ct.new_tensor([rows, cols])
        ct.assign(g, ct.select(x, idx, ALL))
        assert np.array_equal(ct.to_array(g).reshape(rows, cols), X[ids])
    with ct.with_stream(stream), ct.with_datatype("int"):
        xi = ct.to_tensor(rng.integers(-2 ** 31, 2 ** 31 - 1, size=(rows, 64), dtype=np.int32))
        gi = ct.new_tensor([rows, 64])
        ct.assign(gi, ct.select(xi, ct.to_tensor(ids), ALL))
        assert np.array_equal(ct.to_array(gi).reshape(rows, 64), ct.to_array(xi).reshape(rows, 64)[ids])


def test_convolution_config_full_size_sampled(b200_driver):
    """Config 4: [64, 64, 56, 56] NCHW, 3x3 stride 1 pad 1, 64 output channels, bias + ReLU."""
    batch, cin, hw, cout, k = 64, 64, 56, 64, 3
    rng = np.random.default_rng(404)
    X = rng.standard_normal((batch, cin, hw, hw), dtype=np.float32)
    W = (rng.standard_normal((cout, cin * k * k)) * np.sqrt(2.0 / (cin * k * k))).astype(np.float32)
    bvec = (rng.standard_normal(cout) * 0.1).astype(np.float32)
    Xp = np.pad(X, ((0, 0), (0, 0), (1, 1), (1, 1))).astype(np.float64)
    W4 = W.reshape(cout, cin, k, k).astype(np.float64)
    stream = _stream(b200_driver)
    with ct.with_stream(stream), ct.with_datatype("float"):
        layer = nn.Convolution(ct.to_tensor(W), ct.to_tensor(bvec), (k, k), (1, 1), (1, 1), cin, cout, "float")
        out = ct.new_tensor([batch, cout, hw, hw])
        layer.forward(ct.to_tensor(X), out)
        nn.relu(out, out)
        got = ct.to_array(out).reshape(batch, cout, hw, hw)
    # corners, edges and interior pixels of every image border case plus random positions
    pos = [(0, 0, 0, 0), (63, 63, 55, 55), (5, 7, 0, 55), (9, 1, 55, 0), (31, 40, 0, 17), (2, 3, 28, 55)]
    pos += [tuple(int(v) for v in rng.integers(0, (batch, cout, hw, hw))) for _ in range(3000)]
    ref = np.array([max(0.0, float((Xp[n, :, y:y + k, x:x + k] * W4[co]).sum() + bvec[co])) for n, co, y, x in pos])
    g = np.array([got[p_] for p_ in pos], np.float64)
    rms = float(np.sqrt((ref ** 2).mean()))
    assert np.abs(g - ref).max() / max(np.abs(ref).max(), rms) <= 1e-4


@pytest.mark.parametrize("datatype,rows,presplit", [("float", 8192, False), ("float", 8192, True), ("double", 2048, False)])
def test_wide_mlp_full_width_sampled_rows(b200_driver, datatype, rows, presplit):
    """Config 5 at full width (4096 -> 4 x 4096 + ReLU -> 1000 + softmax) on a slice of the batch:
    every row sums to 1; sampled rows against a float64 forward."""
    dt = NP[datatype]
    rng = np.random.default_rng(505)
    Ws = [(rng.standard_normal((4096 if i < 4 else 1000, 4096)) * np.sqrt(2.0 / 4096)).astype(dt) for i in range(5)]
    X = rng.standard_normal((rows, 4096)).astype(dt)
    stream = _stream(b200_driver)
    with ct.with_stream(stream), ct.with_datatype(datatype):
        layers = [(ct.to_tensor(w), ct.new_tensor([w.shape[0]]), "softmax" if i == 4 else "relu")
                  for i, w in enumerate(Ws)]
        net = nn.MLP(layers, fused=True, presplit=presplit)
        probs = ct.to_array(net.infer(ct.to_tensor(X))).reshape(rows, 1000)
    assert np.abs(probs.astype(np.float64).sum(axis=1) - 1.0).max() <= (1e-5 if datatype == "float" else 1e-13)
    pick = rng.integers(0, rows, size=48)
    h = X[pick].astype(np.float64)
    for i, w in enumerate(Ws):
        h = h @ w.astype(np.float64).T
        if i < 4:
            h = np.maximum(h, 0.0)
    e = np.exp(h - h.max(axis=1, keepdims=True))
    want = e / e.sum(axis=1, keepdims=True)
    err = np.abs(probs[pick] - want).max() / max(want.max(), float(np.sqrt((want ** 2).mean())))
    assert err <= TOL[datatype]


@pytest.mark.parametrize("M,N,K", [(300, 200, 4096), (128, 1000, 4112), (513, 260, 8200), (4096, 4096, 4096)])
@pytest.mark.parametrize("beta", [0.0, 0.75])
@pytest.mark.parametrize("never_slice", [False, True])
def test_fused_layer_long_reduction(b200_driver, M, N, K, beta, never_slice):
    """gemm_bias_act with K >= 4096: the reduction of every output tile is cut at least in two -- K slices
    where the tiles leave SMs free (the small shapes here), otherwise, or with slicing switched off, two K
    halves by two CTAs of one launch (and host-chained launches past 4096); alpha, beta, bias and ReLU must
    come out as for one reduction.  Sampled entries against float64."""
    rng = np.random.default_rng(K + M)
    A = rng.standard_normal((M, K)).astype(np.float32)
    W = (rng.standard_normal((N, K)) / np.sqrt(K)).astype(np.float32)
    C0 = rng.standard_normal((M, N)).astype(np.float32)
    bias = rng.standard_normal(N).astype(np.float32)
    stream = _stream(b200_driver)
    stream.set_option("gemm-k-slices", 1 if never_slice else 0)
    with ct.with_stream(stream), ct.with_datatype("float"):
        a, w, c, b = ct.to_tensor(A), ct.to_tensor(W), ct.to_tensor(C0), ct.to_tensor(bias)
        for _ in range(2):      # twice: the per-tile flags must be left clean by the first launch
            ct.assign(c, ct.to_tensor(C0))
            stream.gemm_bias_act(c.buffer, N, False, True, 1.25, a.buffer, M, K, K, w.buffer, N, K, beta, b.buffer, "relu")
        got = ct.to_array(c).reshape(M, N)
    idx = rng.integers(0, (M, N), size=(800, 2))
    ref = np.array([max(0.0, 1.25 * float(A[i].astype(np.float64) @ W[j].astype(np.float64)) + beta * float(C0[i, j]) + float(bias[j]))
                    for i, j in idx])
    g = np.array([got[i, j] for i, j in idx], np.float64)
    scale = max(float(np.abs(ref).max()), float(np.sqrt((ref ** 2).mean())))
    assert np.abs(g - ref).max() / scale <= 1e-4
