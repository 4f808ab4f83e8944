"""Layer glue of the dense-inference path, written purely in terms of the tensor API.

Mirrors the reference's compute layers:
  biased_multiply   nn-backend/biased-multiply!   src/cortex/compute/nn/backend.clj:98-112
  Linear            (defrecord Linear)            src/cortex/compute/nn/layers.clj:66-88
  relu / Activation activations/relu, ActivationLayer   compute/nn/activations.clj:15-16, layers.clj:91-116
  Softmax           SoftmaxLayer                  compute/nn/layers.clj:141-168
  Convolution       ConvolutionLayer              compute/nn/layers.clj:306-360

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


class Activation:
    def __init__(self, act_type):
        self.act_type = act_type

    def forward(self, input, output):
        return _ACTIVATIONS[self.act_type](input, output)


class Softmax:
    def forward(self, input, output):
        return ct.softmax(output, input)


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


class MLP:
    """A stack of dense layers: [(weights[out,in], bias[out], act)], act in
    {None, "relu", "tanh", "logistic", "softmax"}.  Activation buffers are
    allocated once per batch size and reused (the reference pools them in
    nn/compute_binding.clj:208-259)."""

    def __init__(self, layers, fused=False):
        self.layers = [(Linear(w, b), act) for (w, b, act) in layers]
        self.fused = fused
        self._buffers = {}
        self._graphs = {}

    def _buffer(self, idx, batch, width, datatype):
        key = (idx, batch, width, datatype)
        if key not in self._buffers:
            self._buffers[key] = ct.new_tensor([batch, width], datatype=datatype, init_value=None)
        return self._buffers[key]

    def infer(self, x):
        batch = x.shape()[0]
        dt = x.get_datatype()
        cur = x
        for idx, (lin, act) in enumerate(self.layers):
            width = lin.weights.shape()[0]
            out = self._buffer(idx, batch, width, dt)
            if self.fused and act in (None, "relu", "tanh", "logistic"):
                lin.forward_fused(cur, out, act)
            elif self.fused and act == "softmax":
                lin.forward_fused(cur, out, None)
                ct.softmax(out, out)
            else:
                lin.forward(cur, out)
                if act == "softmax":
                    ct.softmax(out, out)
                elif act is not None:
                    _ACTIVATIONS[act](out, out)   # in place: binary-accum-constant! on the backend
            cur = out
        return cur

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
