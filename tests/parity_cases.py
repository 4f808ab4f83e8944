"""Seeded parity cases shared by the CPU suite (oracle vs plain numpy) and the GPU
suite (B200 vs oracle).  Inputs follow the benchmark configurations: same
distributions and seeds, sizes scaled down where noted so that the oracle
finishes in seconds.  Each case builds its inputs with numpy, runs the SAME
tensor-API calls on whatever backend is bound, and returns host arrays."""
import numpy as np

from cortex_b200 import nn
from cortex_b200 import tensor as ct
from cortex_b200.dimensions import ALL

NP = {"float": np.float32, "double": np.float64, "int": np.int32, "long": np.int64, "short": np.int16,
      "byte": np.int8}
TOL = {"float": 1e-4, "double": 1e-12}


def rel_err(got, ref):
    """abs(got - ref) / max(abs(ref), rms(ref)), the parity measure used for fp results."""
    ref = np.asarray(ref, np.float64)
    got = np.asarray(got, np.float64).reshape(ref.shape)
    rms = float(np.sqrt(np.mean(ref ** 2))) or 1.0
    return float(np.max(np.abs(got - ref) / np.maximum(np.abs(ref), rms))) if ref.size else 0.0


def gemm_case(datatype, m, n, k, trans_a, trans_b, alpha, beta, pitch_pad=0, offset=0, seed=201):
    """C = alpha*op(A)*op(B) + beta*C on [rows, cols] windows of larger backing buffers
    (row pitch = cols + pitch_pad, window origin (offset, offset)): config 2's shape at any size."""
    rng = np.random.default_rng(seed)
    dt = NP[datatype]

    def backing(rows, cols):
        full = rng.standard_normal((rows + offset, cols + pitch_pad + offset)).astype(dt)
        return full

    a_shape = (k, m) if trans_a else (m, k)
    b_shape = (n, k) if trans_b else (k, n)
    A_full, B_full, C_full = backing(*a_shape), backing(*b_shape), backing(m, n)

    def run():
        ta, tb, tc = ct.to_tensor(A_full, datatype), ct.to_tensor(B_full, datatype), ct.to_tensor(C_full, datatype)
        va = ct.submatrix(ta, offset, a_shape[0], offset, a_shape[1])
        vb = ct.submatrix(tb, offset, b_shape[0], offset, b_shape[1])
        vc = ct.submatrix(tc, offset, m, offset, n)
        ct.gemm(vc, trans_a, trans_b, alpha, va, vb, beta)
        return ct.to_array(tc)      # whole backing buffer: the frame around the window must be untouched

    def reference():
        A = A_full[offset:offset + a_shape[0], offset:offset + a_shape[1]].astype(np.float64)
        B = B_full[offset:offset + b_shape[0], offset:offset + b_shape[1]].astype(np.float64)
        opa, opb = (A.T if trans_a else A), (B.T if trans_b else B)
        out = C_full.astype(np.float64).copy()
        out[offset:offset + m, offset:offset + n] = alpha * (opa @ opb) + beta * out[offset:offset + m, offset:offset + n]
        return out

    return run, reference


def eltwise_case(datatype, rows, cols, seed=301):
    """Config 3: X + bias (out of place and in place), ReLU, row max / sum, softmax and its decomposition."""
    rng = np.random.default_rng(seed)
    dt = NP[datatype]
    X = rng.standard_normal((rows, cols)).astype(dt)
    bias = (np.random.default_rng(seed + 1).standard_normal((1, cols)) * 0.1).astype(dt)

    def run():
        x, b = ct.to_tensor(X, datatype), ct.to_tensor(bias, datatype)
        y = ct.new_tensor([rows, cols], datatype)
        ct.binary_op(y, 1.0, x, 1.0, b, "+")                      # out of place, row broadcast
        biased = ct.to_array(y)
        x2 = ct.to_tensor(X, datatype)
        ct.binary_op(x2, 1.0, x2, 1.0, ct.in_place_reshape(b, [cols]), "+")   # in place, bias as [cols]
        biased_inplace = ct.to_array(x2)
        r = ct.new_tensor([rows, cols], datatype)
        ct.binary_op(r, 1.0, y, 1.0, 0, "max")                    # ReLU
        relu = ct.to_array(r)
        mx, sm = ct.new_tensor([rows, 1], datatype), ct.new_tensor([rows, 1], datatype)
        ct.unary_reduce(mx, 1.0, r, "max")
        ct.unary_reduce(sm, 1.0, r, "sum")
        s = ct.new_tensor([rows, cols], datatype)
        ct.softmax(s, y)
        # decomposed softmax: max -> subtract (column broadcast) -> exp -> sum -> divide
        m2 = ct.new_tensor([rows, 1], datatype)
        ct.unary_reduce(m2, 1.0, y, "max")
        d = ct.new_tensor([rows, cols], datatype)
        ct.binary_op(d, 1.0, y, 1.0, m2, "-")
        ct.unary_op(d, 1.0, d, "exp")
        s2 = ct.new_tensor([rows, 1], datatype)
        ct.unary_reduce(s2, 1.0, d, "sum")
        ct.binary_op(d, 1.0, d, 1.0, s2, "/")
        return {"biased": biased, "biased_inplace": biased_inplace, "relu": relu, "rowmax": ct.to_array(mx),
                "rowsum": ct.to_array(sm), "softmax": ct.to_array(s), "softmax_decomposed": ct.to_array(d)}

    return run


def gather_case(datatype, src_rows, n_idx, cols, seed=303):
    """Config 3's index gather: dest[i, :] = M[idx[i], :] through select + assign!; bit-exact."""
    rng = np.random.default_rng(seed)
    idx = rng.integers(0, src_rows, size=n_idx, dtype=np.int32)
    if datatype in ("int", "long"):
        info = np.iinfo(NP[datatype])
        M = np.random.default_rng(seed + 1).integers(info.min, info.max, size=(src_rows, cols), dtype=NP[datatype],
                                                      endpoint=True)
    else:
        M = np.random.default_rng(seed + 1).standard_normal((src_rows, cols)).astype(NP[datatype])

    def run():
        m = ct.to_tensor(M, datatype)
        it = ct.to_tensor(idx, "int")
        dest = ct.new_tensor([n_idx, cols], datatype)
        ct.assign(dest, ct.select(m, it, ALL))
        return ct.to_array(dest)

    return run, lambda: M[idx]


def mlp_case(datatype, batch, widths, seed=101, fused=False, bias_scale=0.0, presplit=False):
    """Configs 1 and 5: dense layers with ReLU, softmax head.  widths = [in, h1, ..., out]."""
    dt = NP[datatype]
    X = np.random.default_rng(seed).random((batch, widths[0])).astype(dt)
    Ws, bs = [], []
    for i in range(len(widths) - 1):
        fan_in = widths[i]
        Ws.append((np.random.default_rng(seed + 1 + i).standard_normal((widths[i + 1], fan_in))
                   * np.sqrt(2.0 / fan_in)).astype(dt))
        bs.append((np.random.default_rng(seed + 50 + i).standard_normal(widths[i + 1]) * bias_scale).astype(dt))

    def run():
        layers = []
        for i, (w, b) in enumerate(zip(Ws, bs)):
            act = "softmax" if i == len(Ws) - 1 else "relu"
            layers.append((ct.to_tensor(w, datatype), ct.to_tensor(b, datatype), act))
        net = nn.MLP(layers, fused=fused, presplit=presplit)
        return ct.to_array(net.infer(ct.to_tensor(X, datatype)))

    def reference():
        h = X.astype(np.float64)
        for i, (w, b) in enumerate(zip(Ws, bs)):
            h = h @ w.astype(np.float64).T + b.astype(np.float64)
            if i < len(Ws) - 1:
                h = np.maximum(h, 0.0)
        e = np.exp(h - h.max(axis=1, keepdims=True))
        return e / e.sum(axis=1, keepdims=True)

    return run, reference


def mlp_backward_case(datatype, batch, widths, seed=131, act="relu"):
    """One training step's forward + backward through dense layers with an activation between them and a
    softmax head: d(loss)/d(logits) = probs - onehot (softmax + cross-entropy), then the reference's backward
    calls per layer (assign! for softmax, activation-gradient!, biased-multiply-backward!).
    Returns the concatenation [input-gradient, weight and bias gradients of every layer]."""
    dt = NP[datatype]
    rng = np.random.default_rng(seed)
    X = rng.random((batch, widths[0])).astype(dt)
    labels = rng.integers(0, widths[-1], size=batch)
    Ws = [(rng.standard_normal((widths[i + 1], widths[i])) * np.sqrt(2.0 / widths[i])).astype(dt)
          for i in range(len(widths) - 1)]
    bs = [(rng.standard_normal(widths[i + 1]) * 0.1).astype(dt) for i in range(len(widths) - 1)]
    onehot = np.zeros((batch, widths[-1]), dt)
    onehot[np.arange(batch), labels] = 1

    def run():
        n = len(Ws)
        lins = [nn.Linear(ct.to_tensor(w, datatype), ct.to_tensor(b, datatype)) for w, b in zip(Ws, bs)]
        acts = [nn.Activation(act) for _ in range(n - 1)]
        x = ct.to_tensor(X, datatype)
        pre, post, cur = [], [], x
        for i, lin in enumerate(lins):
            z = ct.new_tensor([batch, widths[i + 1]], datatype)
            lin.forward(cur, z)
            pre.append(z)
            if i < n - 1:
                a = ct.new_tensor([batch, widths[i + 1]], datatype)
                acts[i].forward(z, a)
            else:
                a = ct.new_tensor([batch, widths[i + 1]], datatype)
                nn.Softmax().forward(z, a)
            post.append(a)
            cur = a
        # loss gradient with respect to the softmax layer's output buffer, as the reference's softmax-loss gives it
        grad = ct.new_tensor([batch, widths[-1]], datatype)
        nn.softmax_loss_gradient(post[-1], ct.to_tensor(onehot, datatype), grad)
        outs = []
        g_in = ct.new_tensor([batch, widths[-1]], datatype)
        nn.Softmax().backward(g_in, grad)
        grad = g_in
        for i in range(n - 1, -1, -1):
            inp = x if i == 0 else post[i - 1]
            w_grad = ct.new_tensor([widths[i + 1], widths[i]], datatype)
            b_grad = ct.new_tensor([widths[i + 1]], datatype)
            in_grad = ct.new_tensor([batch, widths[i]], datatype)
            lins[i].backward(inp, pre[i], in_grad, grad, w_grad, b_grad)
            outs = [ct.to_array(w_grad).ravel(), ct.to_array(b_grad).ravel()] + outs
            grad = in_grad
            if i > 0:
                g2 = ct.new_tensor([batch, widths[i]], datatype)
                acts[i - 1].backward(post[i - 1], g2, grad)
                grad = g2
        return np.concatenate([ct.to_array(grad).ravel()] + outs)

    def reference():
        h = X.astype(np.float64)
        hs, zs = [h], []
        for i, (w, b) in enumerate(zip(Ws, bs)):
            z = h @ w.astype(np.float64).T + b.astype(np.float64)
            zs.append(z)
            if i < len(Ws) - 1:
                h = {"relu": lambda v: np.maximum(v, 0.0), "tanh": np.tanh,
                     "logistic": lambda v: 1.0 / (1.0 + np.exp(-v))}[act](z)
                hs.append(h)
        e = np.exp(z - z.max(axis=1, keepdims=True))
        g = e / e.sum(axis=1, keepdims=True) - onehot
        outs = []
        for i in range(len(Ws) - 1, -1, -1):
            outs = [(g.T @ hs[i]).ravel(), g.sum(axis=0)] + outs
            g = g @ Ws[i].astype(np.float64)
            if i > 0:
                a = hs[i]
                g = g * {"relu": (a > 0).astype(np.float64), "tanh": 1.0 - a * a, "logistic": a * (1.0 - a)}[act]
        return np.concatenate([g.ravel()] + outs)

    return run, reference


def activation_gradient_case(datatype, rows, cols, op, seed=141, pitched=False):
    """activation-gradient! on dense [rows, cols] operands, or on windows of wider buffers (index-system path)."""
    dt = NP[datatype]
    rng = np.random.default_rng(seed + rows)
    pad = 5 if pitched else 0
    OUT = rng.standard_normal((rows, cols + pad)).astype(dt)
    if op == "logistic":
        OUT = (1.0 / (1.0 + np.exp(-OUT))).astype(dt)
    elif op == "tanh":
        OUT = np.tanh(OUT).astype(dt)
    GRAD = rng.standard_normal((rows, cols + pad)).astype(dt)

    def run():
        out, grad = ct.to_tensor(OUT, datatype), ct.to_tensor(GRAD, datatype)
        dest = ct.new_tensor([rows, cols + pad], datatype)
        if pitched:
            out, grad, d = (ct.submatrix(t, 0, rows, 2, cols) for t in (out, grad, dest))
            ct.activation_gradient(d, grad, out, op)
        else:
            ct.activation_gradient(dest, grad, out, op)
        return ct.to_array(dest)

    return run


def conv_backward_case(datatype, batch, cin, hw, cout, k=3, pad=1, stride=1, seed=451):
    """ConvolutionLayer forward + backward: returns [input-gradient, weight-gradient, bias-gradient]."""
    dt = NP[datatype]
    rng = np.random.default_rng(seed)
    X = rng.standard_normal((batch, cin, hw, hw)).astype(dt)
    W = (rng.standard_normal((cout, cin * k * k)) * np.sqrt(2.0 / (cin * k * k))).astype(dt)
    b = (rng.standard_normal(cout) * 0.1).astype(dt)
    out_hw = (hw + 2 * pad - k) // stride + 1
    OG = rng.standard_normal((batch, cout, out_hw, out_hw)).astype(dt)

    def run():
        layer = nn.Convolution(ct.to_tensor(W, datatype), ct.to_tensor(b, datatype), (k, k), (pad, pad),
                               (stride, stride), cin, cout, datatype)
        x = ct.to_tensor(X, datatype)
        out = ct.new_tensor([batch, cout, out_hw, out_hw], datatype)
        layer.forward(x, out)
        in_grad = ct.new_tensor([batch, cin, hw, hw], datatype)
        w_grad, b_grad = ct.new_tensor([cout, cin * k * k], datatype), ct.new_tensor([cout], datatype)
        ct.assign(in_grad, 3)       # must be overwritten (alpha = 0)
        ct.assign(w_grad, 3)
        layer.backward(x, in_grad, ct.to_tensor(OG, datatype), w_grad, b_grad)
        return np.concatenate([ct.to_array(t).ravel() for t in (in_grad, w_grad, b_grad)])

    def reference():
        Xp = np.zeros((batch, cin, hw + 2 * pad, hw + 2 * pad), np.float64)
        Xp[:, :, pad:pad + hw, pad:pad + hw] = X
        W4 = W.astype(np.float64).reshape(cout, cin, k, k)
        og = OG.astype(np.float64)
        gw = np.zeros_like(W4)
        gx = np.zeros_like(Xp)
        for ky in range(k):
            for kx in range(k):
                patch = Xp[:, :, ky:ky + stride * out_hw:stride, kx:kx + stride * out_hw:stride]   # [B, cin, oh, ow]
                gw[:, :, ky, kx] = np.einsum("bohw,bchw->oc", og, patch)
                gx[:, :, ky:ky + stride * out_hw:stride, kx:kx + stride * out_hw:stride] += np.einsum(
                    "bohw,oc->bchw", og, W4[:, :, ky, kx])
        gx = gx[:, :, pad:pad + hw, pad:pad + hw]
        return np.concatenate([gx.ravel(), gw.ravel(), og.sum(axis=(0, 2, 3))])

    return run, reference


def conv_case(datatype, batch, cin, hw, cout, k=3, pad=1, stride=1, seed=401, bias_scale=0.0, fused=False):
    """Config 4: NCHW conv + bias + ReLU, as the reference's three calls or (fused) as one call whose epilogue adds
    the bias and applies the activation."""
    dt = NP[datatype]
    X = np.random.default_rng(seed).standard_normal((batch, cin, hw, hw)).astype(dt)
    W = (np.random.default_rng(seed + 1).standard_normal((cout, cin * k * k)) * np.sqrt(2.0 / (cin * k * k))).astype(dt)
    b = (np.random.default_rng(seed + 2).standard_normal(cout) * bias_scale).astype(dt)
    out_hw = (hw + 2 * pad - k) // stride + 1

    def run():
        layer = nn.Convolution(ct.to_tensor(W, datatype), ct.to_tensor(b, datatype), (k, k), (pad, pad),
                               (stride, stride), cin, cout, datatype)
        out = ct.new_tensor([batch, cout, out_hw, out_hw], datatype)
        if fused:
            layer.forward_fused(ct.to_tensor(X, datatype), out, "relu")
        else:
            layer.forward(ct.to_tensor(X, datatype), out)
            nn.relu(out, out)
        return ct.to_array(out)

    def reference():
        xp = np.zeros((batch, cin, hw + 2 * pad, hw + 2 * pad), np.float64)
        xp[:, :, pad:pad + hw, pad:pad + hw] = X
        cols = np.empty((batch, out_hw * out_hw, cin, k, k), np.float64)
        for ky in range(k):
            for kx in range(k):
                patch = xp[:, :, ky:ky + stride * out_hw:stride, kx:kx + stride * out_hw:stride]
                cols[:, :, :, ky, kx] = patch.reshape(batch, cin, -1).transpose(0, 2, 1)
        out = np.einsum("ok,npk->nop", W.astype(np.float64), cols.reshape(batch, out_hw * out_hw, -1))
        out = out + b.astype(np.float64)[None, :, None]
        return np.maximum(out, 0.0).reshape(batch, cout, out_hw, out_hw)

    return run, reference


def mnist_convnet_case(datatype, batch=32, seed=601):
    """The reference's MNIST-NETWORK (src/cortex/verify/nn/train.clj:24-41) as an inference pass on seeded data:
    conv 5x5 (1->20) -> max-pool 2 -> batch-norm (spatial) -> ReLU -> conv 5x5 (20->50) -> max-pool 2 ->
    batch-norm -> linear 500 + ReLU -> linear 10 -> softmax   (dropout is the identity at inference)."""
    dt = NP[datatype]
    rng = np.random.default_rng(seed)
    X = rng.random((batch, 1, 28, 28)).astype(dt)

    def he(shape, fan_in):
        return (rng.standard_normal(shape) * np.sqrt(2.0 / fan_in)).astype(dt)

    W1, b1 = he((20, 25), 25), (rng.standard_normal(20) * 0.1).astype(dt)
    W2, b2 = he((50, 500), 500), (rng.standard_normal(50) * 0.1).astype(dt)
    W3, b3 = he((500, 800), 800), (rng.standard_normal(500) * 0.1).astype(dt)
    W4, b4 = he((10, 500), 500), (rng.standard_normal(10) * 0.1).astype(dt)
    bn1 = [(rng.standard_normal(20) * 0.1).astype(dt), (np.abs(rng.standard_normal(20)) + 0.5).astype(dt),
           (1 + 0.1 * rng.standard_normal(20)).astype(dt), (rng.standard_normal(20) * 0.1).astype(dt)]
    bn2 = [(rng.standard_normal(800) * 0.1).astype(dt), (np.abs(rng.standard_normal(800)) + 0.5).astype(dt),
           (1 + 0.1 * rng.standard_normal(800)).astype(dt), (rng.standard_normal(800) * 0.1).astype(dt)]

    def run(fused=True):
        t = lambda a: ct.to_tensor(a, datatype)
        net = nn.ConvNet([
            ("conv", nn.Convolution(t(W1), t(b1), (5, 5), (0, 0), (1, 1), 1, 20, datatype)),
            ("pool", nn.Pooling(20, (2, 2), (0, 0), (2, 2), datatype)),
            ("bn", nn.BatchNormalization(*[t(a) for a in bn1])),
            ("relu",),
            ("conv", nn.Convolution(t(W2), t(b2), (5, 5), (0, 0), (1, 1), 20, 50, datatype)),
            ("pool", nn.Pooling(50, (2, 2), (0, 0), (2, 2), datatype)),
            ("flatten",),
            ("bn", nn.BatchNormalization(*[t(a) for a in bn2])),
            ("linear", nn.Linear(t(W3), t(b3)), "relu"),
            ("linear", nn.Linear(t(W4), t(b4)), None),
            ("softmax",),
        ], fused=fused)
        return ct.to_array(net.infer(t(X)))

    return run


def mnist_convnet_training_case(datatype, batch=16, seed=611):
    """One training pass (forward with batch statistics, backward through every layer) of the same network, with
    the cross-entropy gradient (softmax output - one-hot labels) / batch at its output.  Returns the output, the
    updated running statistics of both batch-norm layers and every parameter gradient."""
    dt = NP[datatype]
    rng = np.random.default_rng(seed)
    X = rng.random((batch, 1, 28, 28)).astype(dt)
    labels = rng.integers(0, 10, size=batch)

    def he(shape, fan_in):
        return (rng.standard_normal(shape) * np.sqrt(2.0 / fan_in)).astype(dt)

    W1, b1 = he((20, 25), 25), (rng.standard_normal(20) * 0.1).astype(dt)
    W2, b2 = he((50, 500), 500), (rng.standard_normal(50) * 0.1).astype(dt)
    W3, b3 = he((500, 800), 800), (rng.standard_normal(500) * 0.1).astype(dt)
    W4, b4 = he((10, 500), 500), (rng.standard_normal(10) * 0.1).astype(dt)
    bn_params = lambda n: [np.zeros(n, dt), np.ones(n, dt), (1 + 0.1 * rng.standard_normal(n)).astype(dt),
                           (rng.standard_normal(n) * 0.1).astype(dt)]
    bn1, bn2 = bn_params(20), bn_params(800)

    def run():
        t = lambda a: ct.to_tensor(a, datatype)
        bns = [nn.BatchNormalization(*[t(a) for a in bn1], epsilon=1e-3), nn.BatchNormalization(*[t(a) for a in bn2], epsilon=1e-3)]
        net = nn.ConvNet([
            ("conv", nn.Convolution(t(W1), t(b1), (5, 5), (0, 0), (1, 1), 1, 20, datatype)),
            ("pool", nn.Pooling(20, (2, 2), (0, 0), (2, 2), datatype)),
            ("bn", bns[0]),
            ("relu",),
            ("conv", nn.Convolution(t(W2), t(b2), (5, 5), (0, 0), (1, 1), 20, 50, datatype)),
            ("pool", nn.Pooling(50, (2, 2), (0, 0), (2, 2), datatype)),
            ("flatten",),
            ("bn", bns[1]),
            ("linear", nn.Linear(t(W3), t(b3)), "relu"),
            ("linear", nn.Linear(t(W4), t(b4)), None),
            ("softmax",),
        ], fused=False)
        x = t(X)
        probs = ct.to_array(net.infer(x)).reshape(batch, 10)          # only to build a loss gradient of the right size
        onehot = np.zeros((batch, 10), dt)
        onehot[np.arange(batch), labels] = 1
        out_grad = t(((probs - onehot) / batch).astype(dt))
        out, _g, grads = net.train_forward_backward(x, out_grad)
        res = {"output": ct.to_array(out)}
        for i, bn in enumerate(bns):
            res["bn%d-running-means" % i] = ct.to_array(bn.means)
            res["bn%d-running-variances" % i] = ct.to_array(bn.variances)
        for idx, g in enumerate(grads):
            if g:
                for name, tensor in g.items():
                    res["layer%d-%s-gradient" % (idx, name)] = ct.to_array(tensor)
        return res, out_grad

    return run
