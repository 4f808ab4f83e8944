"""Layer glue of the dense-inference path, written purely in terms of the tensor API.

Mirrors the reference's compute layers:
  biased_multiply   nn-backend/biased-multiply!   src/cortex/compute/nn/backend.clj:98-112
  Linear            (defrecord Linear)            src/cortex/compute/nn/layers.clj:66-88
  relu / Activation activations/relu, ActivationLayer   compute/nn/activations.clj:15-16, layers.clj:91-116
  Softmax           SoftmaxLayer                  compute/nn/layers.clj:141-168
  Convolution       ConvolutionLayer              compute/nn/layers.clj:306-360
  Pooling           PoolingLayer                  compute/nn/layers.clj:391-409
  BatchNormalization  (inference branch)          compute/nn/layers.clj:228-285
  ConvNet           a layer list run in order, the shape of verify/nn/train.clj:24-41 (MNIST-NETWORK)
Backward passes of the dense layers (the next ring around the inference path):
  biased_multiply_backward   nn-backend/biased-multiply-backward!   compute/nn/backend.clj:115-139
  Linear.backward / Activation.backward / Softmax.backward          compute/nn/layers.clj:78-88, 104-116, 164-168
  Convolution.backward                                              compute/nn/layers.clj:320-340
  softmax_loss_gradient      calculate-cross-entropy-gradient       src/cortex/loss/softmax.clj:13-20

``fused=True`` replaces the reference's three calls per dense layer
(assign! bias, gemm! NT beta=1, binary-op! max 0) with the backend's single
gemm_bias_act entry point; results are the same up to fp32 summation order
(the bias joins after the product instead of before it).
"""
from . import tensor as ct


def biased_multiply(input, weights, bias, output):
    """output[batch, out] = bias (broadcast) ; output += input[batch, in] . weights[out, in]^T"""
    input = ct.as_batch_matrix(input)
    output = ct.as_batch_matrix(output)
    ct.assign(output, bias)
    ct.gemm(output, False, True, 1.0, input, weights, 1.0)
    return output


def biased_multiply_backward(input, weights, bias, output, input_gradient, weight_gradient, bias_gradient,
                             output_gradient):
    """bias-gradient += sum over the batch of output-gradient (binary-op! with a destination smaller than the
    operation: the reference accumulates with compare-and-swap, this backend with a slab sum); input-gradient = output-gradient . weights (gemm! NN, beta 0);
    weight-gradient += output-gradient^T . input (gemm! TN, beta 1).  Any of the three gradients may be None."""
    if bias_gradient is not None:
        ct.binary_op(bias_gradient, 1.0, output_gradient, 1.0, bias_gradient, "+")
    if input_gradient is not None:
        ct.gemm(ct.as_batch_matrix(input_gradient), False, False, 1.0, ct.as_batch_matrix(output_gradient), weights, 0.0)
    if weight_gradient is not None:
        ct.gemm(weight_gradient, True, False, 1.0, ct.as_batch_matrix(output_gradient), ct.as_batch_matrix(input), 1.0)


def softmax_loss_gradient(output, target, gradient):
    """d(cross-entropy)/d(softmax input) = output - target, written into the output's gradient buffer
    (calculate-cross-entropy-gradient, src/cortex/loss/softmax.clj:13-20)."""
    return ct.binary_op(gradient, 1.0, output, 1.0, target, "-")


def relu(input, output):
    """tops/max output input 0  ->  binary-op! output 1.0 input 1.0 0 :max"""
    return ct.binary_op(output, 1.0, input, 1.0, 0, "max")


def logistic(input, output):
    return ct.unary_op(output, 1.0, input, "logistic")


def tanh(input, output):
    return ct.unary_op(output, 1.0, input, "tanh")


_ACTIVATIONS = {"relu": relu, "logistic": logistic, "tanh": tanh}


class Linear:
    def __init__(self, weights, bias):
        self.weights, self.bias = weights, bias

    def forward(self, input, output):
        return biased_multiply(input, self.weights, self.bias, output)

    def backward(self, input, output, input_gradient, output_gradient, weight_gradient, bias_gradient):
        """Gradients ACCUMULATE into weight_gradient / bias_gradient, as in the reference (the optimiser clears them)."""
        return biased_multiply_backward(input, self.weights, self.bias, output, input_gradient, weight_gradient,
                                        bias_gradient, output_gradient)

    def prepare_presplit(self):
        """Compute the weights' lo matrix (x - trunc_tf32(x)) once; needed by forward_presplit."""
        if getattr(self, "weights_lo", None) is None:
            self.weights_lo = ct.new_tensor(self.weights.shape(), datatype="float", init_value=None)
            ct.check_stream().split_lo(self.weights_lo.buffer, self.weights.buffer, self.weights.ecount())
        return self.weights_lo

    def forward_presplit(self, input, input_lo, output, output_lo, act=None):
        """One kernel: output = act(input . W^T + bias) from operands that are already split into hi / lo,
        and (if output_lo is given) the output's lo matrix for the next layer."""
        input, output = ct.as_batch_matrix(input), ct.as_batch_matrix(output)
        m, k = input.shape()
        n = self.weights.shape()[0]
        w_lo = self.prepare_presplit()
        ct.check_stream().gemm_bias_act_presplit(
            output.buffer, output_lo.buffer if output_lo is not None else None, output.dimensions["strides"][0], 1.0,
            input.buffer, input_lo.buffer, m, k, input.dimensions["strides"][0], self.weights.buffer, w_lo.buffer, n,
            self.weights.dimensions["strides"][0], 0.0, self.bias.buffer, act)
        return output

    def forward_fused(self, input, output, act=None):
        """One kernel: output = act(input . W^T + bias)."""
        input, output = ct.as_batch_matrix(input), ct.as_batch_matrix(output)
        m, k = input.shape()
        n = self.weights.shape()[0]
        stream = ct.check_stream()
        stream.gemm_bias_act(output.buffer, output.dimensions["strides"][0], False, True, 1.0, input.buffer, m, k,
                             input.dimensions["strides"][0], self.weights.buffer, n,
                             self.weights.dimensions["strides"][0], 0.0, self.bias.buffer, act)
        return output


def _presplit_ok(linear, input):
    """The pre-split kernel wants fp32, dense row-major operands with 16-byte aligned rows and a wide output."""
    k = linear.weights.shape()[1]
    return (input.get_datatype() == "float" and k % 4 == 0 and linear.weights.shape()[0] > 128 and
            hasattr(ct.check_stream(), "gemm_bias_act_presplit") and not getattr(ct.check_stream(), "is_oracle", False))


class Activation:
    def __init__(self, act_type):
        self.act_type = act_type

    def forward(self, input, output):
        return _ACTIVATIONS[self.act_type](input, output)

    def backward(self, output, input_gradient, output_gradient):
        return ct.activation_gradient(input_gradient, output_gradient, output, self.act_type)


class Softmax:
    """SoftmaxLayer (compute/nn/layers.clj:141-168).  `output_channels` > 1: the buffer is read as
    [ecount / channels, channels] rows (softmax over runs of `channels` values); `output_channels` == 1 with
    an image-shaped input (`input_dimension` = (channels, height, width), channels != 1): spatial softmax over
    the channel axis of [batch, channels, height*width]; otherwise one softmax per batch row."""

    def __init__(self, output_channels=1, input_dimension=None):
        self.output_channels, self.input_dimension = int(output_channels), input_dimension

    def _tensor(self, t):
        """softmax-tensor (layers.clj:141-152)."""
        if self.output_channels > 1:
            return ct.in_place_reshape(t, [t.ecount() // self.output_channels, self.output_channels])
        if self.input_dimension is not None and self.input_dimension[0] != 1:
            channels, height, width = self.input_dimension
            return ct.in_place_reshape(t, [t.shape()[0], channels, height * width])
        return ct.as_batch_matrix(t)

    def forward(self, input, output):
        return ct.softmax(self._tensor(output), self._tensor(input))

    def backward(self, input_gradient, output_gradient):
        """The reference pairs softmax with the cross-entropy loss: the layer passes the gradient through."""
        return ct.assign(self._tensor(input_gradient), self._tensor(output_gradient))


class Convolution:
    """conv (+ bias reshaped [C_out 1 1] added with binary-op! :+), as ConvolutionLayer.forward."""

    def __init__(self, weights, bias, kernel, pad, stride, in_channels, out_channels, datatype):
        self.weights, self.bias = weights, bias
        self.desc = ct.convolution_descriptor(datatype, out_channels, in_channels, kernel[0], kernel[1], pad[0], pad[1],
                                              stride[0], stride[1])
        self.workspace = None
        self.algorithms = None

    def forward(self, input, output):
        batch, _c, in_h, in_w = input.shape()
        if self.algorithms is None:
            self.algorithms = ct.choose_convolution_algorithms(self.desc, in_w, in_h, batch, 100000)
            self.workspace = ct.new_tensor([int(self.algorithms["workspace-size"])], datatype=input.get_datatype())
        bias = ct.in_place_reshape(self.bias, [self.desc["out-channels"], 1, 1])
        ct.convolution_forward(output, 0.0, input, self.weights, self.workspace, self.desc, self.algorithms)
        ct.binary_op(output, 1.0, output, 1.0, bias, "+")
        return output

    def forward_fused(self, input, output, act=None):
        """One call: output = act(conv + bias) in the convolution kernel's epilogue (this backend's fused extra)."""
        return ct.convolution_forward_bias_act(output, 0.0, input, self.weights, self.desc, self.bias, act)

    def backward(self, input, input_gradient, output_gradient, weight_gradient, bias_gradient):
        """ConvolutionLayer.backward (compute/nn/layers.clj:320-340): the bias gradient accumulates over batch and
        pixels (destination [C_out 1 1] smaller than the operation), weight and input gradients are overwritten."""
        bias_gradient = ct.in_place_reshape(bias_gradient, [self.desc["out-channels"], 1, 1])
        ct.binary_op(bias_gradient, 1.0, output_gradient, 1.0, bias_gradient, "+")
        ct.convolution_backward_weights(weight_gradient, 0.0, output_gradient, input, self.workspace, self.desc,
                                        self.algorithms)
        if input_gradient is not None:
            ct.convolution_backward_data(input_gradient, 0.0, output_gradient, self.weights, self.workspace, self.desc,
                                         self.algorithms)
        return input_gradient


class _Replayable:
    """Launch-sequence capture for networks whose forward pass is launch-bound (small batches)."""

    def infer_replayed(self, x):
        """infer() for launch-bound batch sizes: the first call for a given input buffer runs the
        layers normally, the second records them into a graph, later calls replay it with one host
        call.  The result tensor is the same network-owned buffer every time; x's CONTENTS may
        change between calls, its buffer and shape may not."""
        stream = ct.check_stream()
        key = (x.buffer.ptr, tuple(x.shape()), x.get_datatype(), id(stream))
        entry = self._graphs.get(key)
        if entry is None:
            out = self.infer(x)
            self._graphs[key] = [None, out]
            return out
        if entry[0] is None:
            stream.begin_capture()
            try:
                self.infer(x)
            finally:
                entry[0] = stream.end_capture()
        entry[0].launch(stream)
        return entry[1]


class Pooling:
    """PoolingLayer.forward: pooling-forward! output 0.0 input pool-desc."""

    def __init__(self, channels, kernel, pad, stride, datatype, pool_op="max", dimension_op="ceil"):
        self.desc = ct.pooling_descriptor(datatype, channels, kernel[0], kernel[1], pad[0], pad[1], stride[0], stride[1],
                                          dimension_op=dimension_op, pool_op=pool_op)

    def output_shape(self, input_shape):
        batch, ch, h, w = input_shape
        od = ct.get_convolution_output_dimensions(self.desc, h, w)
        return [batch, ch, od["output-width"], od["output-height"]]

    def forward(self, input, output):
        return ct.pooling_forward(output, 0.0, input, self.desc)

    def backward(self, input, output, input_gradient, output_gradient):
        """PoolingLayer.backward (compute/nn/layers.clj:400-409): pooling-backward! input-gradient 0.0 ..."""
        return ct.pooling_backward(input_gradient, 0.0, input, output, output_gradient, self.desc)


class BatchNormalization:
    """Inference branch of the BatchNormalization layer: batch-normalize! with the running statistics.
    A 4-d input [batch, channels, h, w] is normalised per channel (spatial mode) through the view
    [batch, channels, h*w]; a 2-d input per column."""

    def __init__(self, means, variances, scale, bias, epsilon=1e-4):
        self.means, self.variances, self.scale, self.bias, self.epsilon = means, variances, scale, bias, epsilon

    def forward(self, input, output):
        shp = input.shape()
        if len(shp) == 4:
            view = [shp[0], shp[1], shp[2] * shp[3]]
            ct.batch_normalize(ct.in_place_reshape(output, view), ct.in_place_reshape(input, view), self.means,
                               self.variances, self.scale, self.bias, self.epsilon)
        else:
            ct.batch_normalize(output, input, self.means, self.variances, self.scale, self.bias, self.epsilon)
        return output

    # --- training branch (compute/nn/layers.clj:228-262) ----------------------------------------
    @staticmethod
    def _view(t):
        shp = t.shape()
        return ct.in_place_reshape(t, [shp[0], shp[1], shp[2] * shp[3]]) if len(shp) == 4 else t

    def train_forward(self, input, output, average_factor=0.01):
        """batch-normalize-update-and-apply!: this batch's statistics normalise the output and are folded into the
        running means / variances.  The very first batch sets the running statistics to the batch's (factor 1.0), as
        the reference's local-average-factor atom does; later ones interpolate with `average_factor`."""
        n = self.means.shape()[0]
        if getattr(self, "batch_means", None) is None:
            dt = input.get_datatype()
            self.batch_means, self.batch_variances = ct.new_tensor([n], datatype=dt), ct.new_tensor([n], datatype=dt)
            self._factor = 1.0
        ct.batch_normalize_update_and_apply(self._view(output), self._view(input), self.batch_means, self.batch_variances,
                                            self.means, self.variances, self._factor, self.scale, self.bias, self.epsilon)
        self._factor = average_factor
        return output

    def backward(self, input, output, input_gradient, output_gradient, scale_gradient, bias_gradient):
        """batch-normalize-gradients! with the statistics train_forward left behind."""
        ct.batch_normalize_gradients(self._view(input_gradient), scale_gradient, bias_gradient, self._view(output_gradient),
                                     self._view(output), self._view(input), self.batch_means, self.batch_variances,
                                     self.scale, self.bias, self.epsilon)
        return input_gradient


class ConvNet(_Replayable):
    """Runs a list of layer specs in order (inference; dropout layers are the identity and are left out):
      ("conv", Convolution)  ("pool", Pooling)  ("bn", BatchNormalization)  ("relu",)  ("flatten",)
      ("linear", Linear, act-or-None)  ("softmax",)
    Activation buffers are allocated on first use per (layer, batch) and reused."""

    def __init__(self, layers, fused=True):
        self.layers, self.fused, self._buffers, self._graphs = layers, fused, {}, {}

    def _buffer(self, idx, shape, datatype):
        key = (idx, tuple(shape), datatype)
        if key not in self._buffers:
            self._buffers[key] = ct.new_tensor(list(shape), datatype=datatype, init_value=None)
        return self._buffers[key]

    def infer(self, x):
        dt = x.get_datatype()
        cur = x
        # fused: a layer's bias and the activation layer right behind it join the producing kernel's epilogue
        # (convolution + bias [+ ReLU], linear + bias + activation, linear + softmax head)
        fuse_conv = self.fused and hasattr(ct.check_stream(), "convolution_forward_bias_act")
        skip = -1
        for idx, spec in enumerate(self.layers):
            kind = spec[0]
            if idx == skip:
                continue
            nxt = self.layers[idx + 1][0] if idx + 1 < len(self.layers) else None
            if kind == "conv":
                conv = spec[1]
                batch, _c, h, w = cur.shape()
                od = ct.get_convolution_output_dimensions(conv.desc, h, w)
                out = self._buffer(idx, [batch, conv.desc["out-channels"], od["output-width"], od["output-height"]], dt)
                if fuse_conv:
                    cur = conv.forward_fused(cur, out, "relu" if nxt == "relu" else None)
                    if nxt == "relu":
                        skip = idx + 1
                else:
                    cur = conv.forward(cur, out)
            elif kind == "pool":
                out = self._buffer(idx, spec[1].output_shape(cur.shape()), dt)
                cur = spec[1].forward(cur, out)
            elif kind == "bn":
                cur = spec[1].forward(cur, self._buffer(idx, cur.shape(), dt))
            elif kind == "relu":
                cur = relu(cur, cur)
            elif kind == "flatten":
                cur = ct.as_batch_matrix(cur)
            elif kind == "linear":
                lin, act = spec[1], spec[2]
                out = self._buffer(idx, [cur.shape()[0], lin.weights.shape()[0]], dt)
                if self.fused:
                    if act is None and nxt == "softmax":
                        act, skip = "softmax", idx + 1
                    cur = lin.forward_fused(cur, out, act)
                else:
                    cur = lin.forward(cur, out)
                    if act is not None:
                        _ACTIVATIONS[act](cur, cur)
            elif kind == "softmax":
                cur = ct.softmax(cur, cur)
            else:
                raise ValueError("unknown layer kind %r" % (kind,))
        return cur

    def train_forward_backward(self, x, output_gradient):
        """One training pass of the layer list (what cortex.nn.execute drives through ComputeLayer.forward /
        .backward): batch-norm layers use and update batch statistics, every layer keeps its input and output, and the
        backward sweep returns the loss gradient with respect to x and a list of per-layer parameter gradients
        ({"weights": .., "bias": ..} for conv / linear, {"scale": .., "bias": ..} for batch-norm, None otherwise).
        `output_gradient` is the gradient at the network's output, or a function of the output tensor returning it; a
        trailing softmax passes it through (the layer is paired with the cross-entropy loss, whose gradient is already
        with respect to the softmax input)."""
        dt = x.get_datatype()
        new = lambda shape: ct.new_tensor(list(shape), datatype=dt)
        acts = [x]                      # acts[i] = input of layer i, acts[i + 1] = its output
        cur = x
        for spec in self.layers:
            kind = spec[0]
            if kind == "conv":
                conv = spec[1]
                batch, _c, h, w = cur.shape()
                od = ct.get_convolution_output_dimensions(conv.desc, h, w)
                cur = conv.forward(cur, new([batch, conv.desc["out-channels"], od["output-width"], od["output-height"]]))
            elif kind == "pool":
                cur = spec[1].forward(cur, new(spec[1].output_shape(cur.shape())))
            elif kind == "bn":
                cur = spec[1].train_forward(cur, new(cur.shape()))
            elif kind == "relu":
                cur = relu(cur, new(cur.shape()))
            elif kind == "flatten":
                cur = ct.as_batch_matrix(cur)
            elif kind == "linear":
                lin, act = spec[1], spec[2]
                cur = lin.forward(cur, new([cur.shape()[0], lin.weights.shape()[0]]))
                if act is not None:
                    _ACTIVATIONS[act](cur, cur)
            elif kind == "softmax":
                cur = ct.softmax(new(cur.shape()), cur)
            else:
                raise ValueError("unknown layer kind %r" % (kind,))
            acts.append(cur)
        grads = [None] * len(self.layers)
        # a callable gets the network's output (a loss whose gradient depends on this very forward pass)
        g_out = output_gradient(cur) if callable(output_gradient) else output_gradient
        for idx in range(len(self.layers) - 1, -1, -1):
            spec, inp, out = self.layers[idx], acts[idx], acts[idx + 1]
            kind = spec[0]
            if kind == "softmax":
                g_in = g_out
            elif kind == "linear":
                lin, act = spec[1], spec[2]
                if act is not None:
                    g_act = new(out.shape())
                    ct.activation_gradient(g_act, g_out, out, act)
                    g_out = g_act
                g_in = new(inp.shape())
                wg, bg = new(lin.weights.shape()), new(lin.bias.shape())
                lin.backward(inp, out, g_in, g_out, wg, bg)
                grads[idx] = {"weights": wg, "bias": bg}
            elif kind == "flatten":
                g_in = ct.in_place_reshape(g_out, inp.shape())
            elif kind == "relu":
                g_in = new(inp.shape())
                ct.activation_gradient(g_in, g_out, out, "relu")
            elif kind == "bn":
                bn = spec[1]
                g_in = new(inp.shape())
                sg, bg = new(bn.scale.shape()), new(bn.bias.shape())
                bn.backward(inp, out, g_in, g_out, sg, bg)
                grads[idx] = {"scale": sg, "bias": bg}
            elif kind == "pool":
                g_in = new(inp.shape())
                spec[1].backward(inp, out, g_in, g_out)
            elif kind == "conv":
                conv = spec[1]
                g_in = new(inp.shape()) if idx > 0 else None
                wg, bg = new(conv.weights.shape()), new(conv.bias.shape())
                conv.backward(inp, g_in, g_out, wg, bg)
                grads[idx] = {"weights": wg, "bias": bg}
            g_out = g_in
        return acts[-1], g_out, grads


class MLP(_Replayable):
    """A stack of dense layers: [(weights[out,in], bias[out], act)], act in
    {None, "relu", "tanh", "logistic", "softmax"}.  Activation buffers are
    allocated once per batch size and reused (the reference pools them in
    nn/compute_binding.clj:208-259)."""

    def __init__(self, layers, fused=False, presplit=False):
        """presplit (implies fused; fp32 on the B200 backend only): layers whose operands qualify run the
        pre-split GEMM: weights are split into hi / lo once, every layer writes its output already split."""
        self.layers = [(Linear(w, b), act) for (w, b, act) in layers]
        self.fused = fused or presplit
        self.presplit = presplit
        self._buffers = {}
        self._graphs = {}

    def _buffer(self, idx, batch, width, datatype):
        key = (idx, batch, width, datatype)
        if key not in self._buffers:
            self._buffers[key] = ct.new_tensor([batch, width], datatype=datatype, init_value=None)
        return self._buffers[key]

    def infer(self, x, row_block=None, trace=None):
        """Forward pass.  `row_block`: run the stack depth-first over blocks of that many rows (every layer of
        block 0, then block 1, ...): the activations between layers are then block-sized buffers that are reused
        for every block, so they stay (partly) in L2 from one layer to the next instead of streaming through
        HBM; the result is the same, bit for bit (rows are independent).  `trace(idx, when)` is called around
        every layer's GEMM launch with when = "begin" / "end" (measurement hooks)."""
        batch = x.shape()[0]
        if not row_block or batch <= row_block:
            return self._infer_rows(x, trace)
        dt = x.get_datatype()
        in_width = x.shape()[1]
        out_width = self.layers[-1][0].weights.shape()[0]
        full = self._buffer(("row-blocked-out",), batch, out_width, dt)
        stream = ct.check_stream()
        xm = ct.as_batch_matrix(x)
        ct._require(ct.dense(xm), "row-blocked inference wants a dense input")
        from . import dimensions as dims
        for r0 in range(0, batch, row_block):
            nr = min(row_block, batch - r0)
            xb = ct.Tensor(x.device, dims.dimensions([nr, in_width]), xm.buffer.sub_buffer(r0 * in_width, nr * in_width))
            yb = self._infer_rows(xb, trace)
            stream.copy_device_to_device(yb.buffer, 0, full.buffer, r0 * out_width, nr * out_width)
        return full

    def _infer_rows(self, x, trace=None):
        batch = x.shape()[0]
        dt = x.get_datatype()
        cur = x
        cur_lo = None          # lo matrix of `cur`, when the previous layer produced it
        for idx, (lin, act) in enumerate(self.layers):
            width = lin.weights.shape()[0]
            out = self._buffer(idx, batch, width, dt)
            if self.presplit and _presplit_ok(lin, cur):
                if cur_lo is None:
                    cur_lo = self._buffer(("lo-in", idx), batch, cur.shape()[1], dt)
                    ct.check_stream().split_lo(cur_lo.buffer, cur.buffer, cur.ecount())
                nxt = self.layers[idx + 1][0] if idx + 1 < len(self.layers) else None
                out_lo = self._buffer(("lo", idx), batch, width, dt) if nxt is not None and self.presplit else None
                if trace:
                    trace(idx, "begin")
                lin.forward_presplit(cur, cur_lo, out, out_lo, act if act != "softmax" else None)
                if trace:
                    trace(idx, "end")
                if act == "softmax":
                    ct.softmax(out, out)
                cur, cur_lo = out, out_lo
                continue
            cur_lo = None
            if trace:
                trace(idx, "begin")
            if self.fused and act in (None, "relu", "tanh", "logistic"):
                lin.forward_fused(cur, out, act)
                if trace:
                    trace(idx, "end")
            elif self.fused and act == "softmax":
                # one call: heads of up to 16 classes are normalised by the kernel that computes them
                lin.forward_fused(cur, out, "softmax")
                if trace:
                    trace(idx, "end")
            else:
                lin.forward(cur, out)
                if trace:
                    trace(idx, "end")
                if act == "softmax":
                    ct.softmax(out, out)
                elif act is not None:
                    _ACTIVATIONS[act](out, out)   # in place: binary-accum-constant! on the backend
            cur = out
        return cur
