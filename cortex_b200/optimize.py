"""Gradient optimisers over flat parameter buffers: host-side mirror of ``cortex.optimize``.

  PGradientOptimizer   batch-update / compute-parameters!      src/cortex/optimize.clj
  Adam                 src/cortex/optimize/adam.clj:144-160      (kernel: resources/adam.cu)
  Adadelta             src/cortex/optimize/adadelta.clj:21-30    (kernel: resources/adadelta.cu)
  SGD                  src/cortex/optimize/sgd.clj:16-53         (four tensor calls, no kernel of its own)

As in the reference, ``compute_parameters`` takes the optimiser's own state buffers sized for ALL
parameters of a network plus the offset of the buffer being stepped, so one state allocation serves
every layer (src/cortex/nn/compute_binding.clj:817-854).  Adam and Adadelta are one fused pass over
HBM each (cb200_adam_step / cb200_adadelta_step); SGD with momentum is issued as the reference issues
it: unary-op! :noop, binary-op! :+, binary-op! :-, binary-op! :+.
"""
from . import tensor as ct


def _flat(t):
    return ct.as_vector(t)


class Adam:
    """defrecord Adam + (adam) defaults: alpha 0.001, beta1 0.9, beta2 0.999, epsilon 1e-8."""

    def __init__(self, alpha=0.001, beta1=0.9, beta2=0.999, epsilon=1e-8):
        self.alpha, self.beta1, self.beta2, self.epsilon = alpha, beta1, beta2, epsilon
        self.pow_beta1_t = 1.0
        self.pow_beta2_t = 1.0

    def batch_update(self):
        """Once per mini-batch, before the per-buffer steps (adam.clj:146-150)."""
        self.pow_beta1_t *= float(self.beta1)
        self.pow_beta2_t *= float(self.beta2)
        return self

    def compute_parameters(self, state, gradient_alpha, offset, gradient, parameters):
        """state: {"m": tensor, "v": tensor} over all parameters; `gradient` / `parameters` are the
        buffers of one layer, `offset` their position inside m and v."""
        n = gradient.ecount()
        ct._require(parameters.ecount() == n, "gradient and parameter element counts differ")
        ct._ensure_datatypes(parameters.get_datatype(), gradient, state["m"], state["v"])
        m = _flat(state["m"]).buffer.sub_buffer(offset, state["m"].ecount() - offset)
        v = _flat(state["v"]).buffer.sub_buffer(offset, state["v"].ecount() - offset)
        ct.check_stream().adam_step(self.alpha, self.beta1, self.beta2, self.epsilon, self.pow_beta1_t,
                                    self.pow_beta2_t, gradient_alpha, gradient.buffer, parameters.buffer, m, v, n)


class Adadelta:
    """defrecord Adadelta + (adadelta) defaults: decay 0.05, epsilon 1e-6."""

    def __init__(self, decay=0.05, epsilon=1e-6):
        self.decay, self.epsilon = decay, epsilon

    def batch_update(self):
        return self

    def compute_parameters(self, state, gradient_alpha, offset, gradient, parameters):
        """state: {"grad-accum": tensor, "dx-accum": tensor} over all parameters."""
        n = gradient.ecount()
        ct._require(parameters.ecount() == n, "gradient and parameter element counts differ")
        ct._ensure_datatypes(parameters.get_datatype(), gradient, state["grad-accum"], state["dx-accum"])
        ga = _flat(state["grad-accum"]).buffer.sub_buffer(offset, state["grad-accum"].ecount() - offset)
        dxa = _flat(state["dx-accum"]).buffer.sub_buffer(offset, state["dx-accum"].ecount() - offset)
        ct.check_stream().adadelta_step(self.decay, self.epsilon, ga, dxa, gradient_alpha, gradient.buffer,
                                        parameters.buffer, n)


class SGD:
    """defrecord SGD + (sgd) defaults: learning-rate 0.001, momentum 0.9 (tensor-sgd, sgd.clj:16-40)."""

    def __init__(self, learning_rate=0.001, momentum=0.9):
        self.learning_rate, self.momentum = learning_rate, momentum
        self._temp = None

    def batch_update(self):
        return self

    def compute_parameters(self, state, gradient_alpha, offset, gradient, parameters):
        """state: {"momentum-vals": tensor} over all parameters."""
        momentum = float(self.momentum)
        gradient, parameters = _flat(gradient), _flat(parameters)
        n = gradient.ecount()
        momentum_vals = ct.subvector(_flat(state["momentum-vals"]), offset, length=n)
        dt = gradient.get_datatype()
        if self._temp is None or self._temp.ecount() < n or self._temp.get_datatype() != dt:
            self._temp = ct.new_tensor([n], datatype=dt, init_value=None)      # :sgd-temp, resizeable
        gradient_temp = ct.subvector(self._temp, 0, length=n)
        dxm = ct.unary_op(gradient_temp, momentum, momentum_vals, "noop")
        ct.binary_op(momentum_vals, 1.0, dxm, float(self.learning_rate) * float(gradient_alpha), gradient, "+")
        dx = ct.binary_op(gradient_temp, 1.0, dxm, 1 + momentum, momentum_vals, "-")
        ct.binary_op(parameters, 1.0, parameters, 1.0, dx, "+")
