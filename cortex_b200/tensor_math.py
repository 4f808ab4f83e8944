"""TensorMath protocol methods (src/cortex/tensor/math.clj:11-252) marshalled onto
a C ABI.

``CTensorMath`` is a mixin for a stream class that provides
``_tm(name, *c_args)`` -- "call entry point <prefix><name> for this stream".
Method names, argument order and meaning are the protocol's; buffers are
objects with ``.ptr`` / ``.dtype`` and dimensions are the dicts of
``cortex_b200.dimensions``.
"""
import ctypes as C

from . import dimensions as dims_mod
from ._lib import ACTIVATIONS, BINARY_OPS, DTYPE_CODE, REDUCE_OPS, TERNARY_OPS, UNARY_OPS, ConvDesc, Dims


def _index_pointer(tensor):
    if tensor.get_datatype() != "int":
        raise TypeError("Index buffers must be integer tensors")
    return tensor.buffer.ptr


def wire(dimensions):
    """dimensions->cuda (src/cortex/compute/cuda/tensor_math.clj:34-51) as a C struct."""
    rev_shape, rev_strides, ptrs = dims_mod.to_wire(dimensions, _index_pointer)
    d = Dims()
    for i in range(5):
        d.rev_shape[i] = rev_shape[i]
        d.rev_strides[i] = rev_strides[i]
        d.index[i] = ptrs[i] or None
    return d


def conv_desc_struct(desc):
    return ConvDesc(desc["out-channels"], desc["in-channels"], desc["kernel-width"], desc["kernel-height"],
                    desc["pad-x"], desc["pad-y"], desc["stride-x"], desc["stride-y"])


class CTensorMath:
    def assign_constant(self, buffer, dimensions, value, n_elems):
        self._tm("assign_constant", DTYPE_CODE[buffer.dtype], buffer.ptr, C.byref(wire(dimensions)), float(value),
                 int(n_elems))

    def assign(self, dest, dest_dims, src, src_dims, n_elems):
        self._tm("assign", DTYPE_CODE[dest.dtype], dest.ptr, C.byref(wire(dest_dims)), DTYPE_CODE[src.dtype], src.ptr,
                 C.byref(wire(src_dims)), int(n_elems))

    def unary_accum(self, dest, dest_dims, alpha, op, n_elems):
        self._tm("unary_accum", DTYPE_CODE[dest.dtype], dest.ptr, C.byref(wire(dest_dims)), float(alpha),
                 UNARY_OPS[op], int(n_elems))

    def unary_op(self, dest, dest_dims, x, x_dims, alpha, op, n_elems):
        self._tm("unary_op", DTYPE_CODE[dest.dtype], dest.ptr, C.byref(wire(dest_dims)), x.ptr, C.byref(wire(x_dims)),
                 float(alpha), UNARY_OPS[op], int(n_elems))

    def binary_accum_constant(self, dest, dest_dims, dest_alpha, scalar, n_elems, op, reverse_operands):
        self._tm("binary_accum_constant", DTYPE_CODE[dest.dtype], dest.ptr, C.byref(wire(dest_dims)),
                 float(dest_alpha), float(scalar), int(n_elems), BINARY_OPS[op], 1 if reverse_operands else 0)

    def binary_op_constant(self, dest, dest_dims, x, x_dims, x_alpha, scalar, n_elems, op, reverse_operands):
        self._tm("binary_op_constant", DTYPE_CODE[dest.dtype], dest.ptr, C.byref(wire(dest_dims)), x.ptr,
                 C.byref(wire(x_dims)), float(x_alpha), float(scalar), int(n_elems), BINARY_OPS[op],
                 1 if reverse_operands else 0)

    def binary_accum(self, dest, dest_dims, dest_alpha, y, y_dims, y_alpha, n_elems, op, reverse_operands,
                     dest_requires_cas):
        self._tm("binary_accum", DTYPE_CODE[dest.dtype], dest.ptr, C.byref(wire(dest_dims)), float(dest_alpha),
                 y.ptr, C.byref(wire(y_dims)), float(y_alpha), int(n_elems), BINARY_OPS[op],
                 1 if reverse_operands else 0, 1 if dest_requires_cas else 0)

    def binary_op(self, dest, dest_dims, x, x_dims, x_alpha, y, y_dims, y_alpha, n_elems, op):
        self._tm("binary_op", DTYPE_CODE[dest.dtype], dest.ptr, C.byref(wire(dest_dims)), x.ptr,
                 C.byref(wire(x_dims)), float(x_alpha), y.ptr, C.byref(wire(y_dims)), float(y_alpha), int(n_elems),
                 BINARY_OPS[op])

    def unary_reduce(self, output, output_dims, input_alpha, input, input_dims, op):
        self._tm("unary_reduce", DTYPE_CODE[output.dtype], output.ptr, C.byref(wire(output_dims)), float(input_alpha),
                 input.ptr, C.byref(wire(input_dims)), REDUCE_OPS[op])

    def gemm(self, c, c_colstride, trans_a, trans_b, alpha, a, a_row_count, a_col_count, a_colstride, b, b_col_count,
             b_colstride, beta):
        self._tm("gemm", DTYPE_CODE[c.dtype], c.ptr, int(c_colstride), 1 if trans_a else 0, 1 if trans_b else 0,
                 float(alpha), a.ptr, int(a_row_count), int(a_col_count), int(a_colstride), b.ptr, int(b_col_count),
                 int(b_colstride), float(beta))

    def softmax_eltwise(self, output, output_dims, input, input_dims):
        self._tm("softmax_eltwise", DTYPE_CODE[output.dtype], output.ptr, C.byref(wire(output_dims)), input.ptr,
                 C.byref(wire(input_dims)))

    def softmax_spatial(self, output, output_dims, input, input_dims):
        self._tm("softmax_spatial", DTYPE_CODE[output.dtype], output.ptr, C.byref(wire(output_dims)), input.ptr,
                 C.byref(wire(input_dims)))

    def convolution_descriptor(self, datatype, out_channels, in_channels, kern_width, kern_height, pad_x, pad_y,
                               stride_x, stride_y):
        return None   # nothing to create on the device

    def choose_convolution_algorithms(self, conv_descriptor, input_width, input_height, output_width, output_height,
                                      batch_size, max_ideal_workspace_size, use_defaults):
        n = C.c_int64()
        self._tm_nostream("convolution_workspace_size", C.byref(conv_desc_struct(conv_descriptor)), int(input_width),
                          int(input_height), int(output_width), int(output_height), int(batch_size), C.byref(n))
        return {"workspace-size": n.value}

    def convolution_forward(self, output, output_dims, output_alpha, input, input_dims, weights, weight_dims,
                            workspace, workspace_ecount, conv_descriptor, algorithms):
        self._tm("convolution_forward", DTYPE_CODE[output.dtype], output.ptr, C.byref(wire(output_dims)),
                 float(output_alpha), input.ptr, C.byref(wire(input_dims)), weights.ptr, C.byref(wire(weight_dims)),
                 workspace.ptr if workspace is not None else None, int(workspace_ecount),
                 C.byref(conv_desc_struct(conv_descriptor)))

    def convolution_forward_bias_act(self, output, output_dims, output_alpha, input, input_dims, weights, weight_dims,
                                     conv_descriptor, bias, act):
        """Fused extra: act(conv + output_alpha * output + bias[channel]) in the convolution's epilogue."""
        self._tm("convolution_forward_bias_act", DTYPE_CODE[output.dtype], output.ptr, C.byref(wire(output_dims)),
                 float(output_alpha), input.ptr, C.byref(wire(input_dims)), weights.ptr, C.byref(wire(weight_dims)),
                 C.byref(conv_desc_struct(conv_descriptor)), bias.ptr if bias is not None else None, ACTIVATIONS[act])

    def convolution_backward_weights(self, weight_gradient, weight_gradient_dims, weight_gradient_alpha,
                                     output_gradient, output_gradient_dims, input, input_dims, workspace,
                                     workspace_ecount, conv_descriptor, algorithms):
        self._tm("convolution_backward_weights", DTYPE_CODE[weight_gradient.dtype], weight_gradient.ptr,
                 C.byref(wire(weight_gradient_dims)), float(weight_gradient_alpha), output_gradient.ptr,
                 C.byref(wire(output_gradient_dims)), input.ptr, C.byref(wire(input_dims)),
                 workspace.ptr if workspace is not None else None, int(workspace_ecount),
                 C.byref(conv_desc_struct(conv_descriptor)))

    def convolution_backward_data(self, input_gradient, input_gradient_dims, input_gradient_alpha, output_gradient,
                                  output_gradient_dims, weights, weight_dims, workspace, workspace_ecount,
                                  conv_descriptor, algorithms):
        self._tm("convolution_backward_data", DTYPE_CODE[input_gradient.dtype], input_gradient.ptr,
                 C.byref(wire(input_gradient_dims)), float(input_gradient_alpha), output_gradient.ptr,
                 C.byref(wire(output_gradient_dims)), weights.ptr, C.byref(wire(weight_dims)),
                 workspace.ptr if workspace is not None else None, int(workspace_ecount),
                 C.byref(conv_desc_struct(conv_descriptor)))

    # --- fused extras (no protocol counterpart) ----------------------------------
    def gemm_bias_act(self, c, c_colstride, trans_a, trans_b, alpha, a, a_row_count, a_col_count, a_colstride, b,
                      b_col_count, b_colstride, beta, bias, act):
        self._tm("gemm_bias_act", DTYPE_CODE[c.dtype], c.ptr, int(c_colstride), 1 if trans_a else 0,
                 1 if trans_b else 0, float(alpha), a.ptr, int(a_row_count), int(a_col_count), int(a_colstride),
                 b.ptr, int(b_col_count), int(b_colstride), float(beta), bias.ptr if bias is not None else None,
                 ACTIVATIONS[act])

    def gemm_bias_act_peers(self, c, c_colstride, trans_a, trans_b, alpha, a, a_row_count, a_col_count, a_colstride, b,
                            b_col_count, b_colstride, beta, bias, act, peer_ptrs):
        """gemm_bias_act whose epilogue also stores the C window at the same position of every
        address in `peer_ptrs` (other GPUs' memory)."""
        import ctypes as C
        arr = (C.c_void_p * max(1, len(peer_ptrs)))(*[int(p) for p in peer_ptrs])
        self._tm("gemm_bias_act_peers", DTYPE_CODE[c.dtype], c.ptr, int(c_colstride), 1 if trans_a else 0,
                 1 if trans_b else 0, float(alpha), a.ptr, int(a_row_count), int(a_col_count), int(a_colstride),
                 b.ptr, int(b_col_count), int(b_colstride), float(beta), bias.ptr if bias is not None else None,
                 ACTIVATIONS[act], len(peer_ptrs), arr)

    def split_lo(self, lo, x, n_elems):
        """lo = x - trunc_tf32(x) over a dense span (fp32)."""
        self._tm("split_lo", lo.ptr, x.ptr, int(n_elems))

    def gemm_bias_act_presplit(self, c, c_lo, ldc, alpha, a_hi, a_lo, a_rows, a_cols, lda, b_hi, b_lo, b_rows, ldb, beta,
                               bias, act):
        self._tm("gemm_bias_act_presplit", c.ptr, c_lo.ptr if c_lo is not None else None, int(ldc), float(alpha),
                 a_hi.ptr, a_lo.ptr, int(a_rows), int(a_cols), int(lda), b_hi.ptr, b_lo.ptr, int(b_rows), int(ldb),
                 float(beta), bias.ptr if bias is not None else None, ACTIVATIONS[act])

    def bias_relu_rowstats(self, y, ldy, x, ldx, bias, rows, cols, rowmax, rowsum):
        self._tm("bias_relu_rowstats", DTYPE_CODE[y.dtype], y.ptr, int(ldy), x.ptr, int(ldx), bias.ptr, int(rows),
                 int(cols), rowmax.ptr if rowmax is not None else None, rowsum.ptr if rowsum is not None else None)

    def _tm_nostream(self, name, *args):
        from ._lib import call
        return call("cb200_" + name, *args)

    # --- protocol methods outside the dense-inference path -----------------------
    def _unsupported(self, name):
        from ._lib import call
        call("cb200_unsupported", name.encode())

    def activation_gradient(self, input_gradient, input_grad_dims, output_gradient, output_grad_dims, output,
                            output_dims, op, element_count):
        """tm/activation-gradient! (tensor/math.clj; CPU cpu/tensor_math.clj:1638-1650)."""
        self._tm("activation_gradient", DTYPE_CODE[input_gradient.dtype], input_gradient.ptr,
                 C.byref(wire(input_grad_dims)), output_gradient.ptr, C.byref(wire(output_grad_dims)), output.ptr,
                 C.byref(wire(output_dims)), ACTIVATIONS[op], int(element_count))

    # --- ternary-op! family: one C entry point, constants travel as (NULL pointer, value * factor) ------
    def _ternary(self, dest, dest_dims, args, n_elems, op):
        """args: three (buffer-or-None, dims-or-None, scalar) in x, y, z order."""
        c_args = []
        for buf, dms, scalar in args:
            c_args += [buf.ptr if buf is not None else None, C.byref(wire(dms)) if buf is not None else None,
                       float(scalar)]
        self._tm("ternary_op", DTYPE_CODE[dest.dtype], dest.ptr, C.byref(wire(dest_dims)), *c_args, int(n_elems),
                 TERNARY_OPS[op])

    def ternary_op(self, dest, dest_dims, x, x_dims, alpha, y, y_dims, beta, z, z_dims, gamma, n_elems, op):
        self._ternary(dest, dest_dims, [(x, x_dims, alpha), (y, y_dims, beta), (z, z_dims, gamma)], n_elems, op)

    @staticmethod
    def _expand_arg_order(arg_order, entries):
        """entries are in arg-order (tensors first, then constants); returns them as x, y, z."""
        by_name = dict(zip(arg_order, entries))
        return [by_name["x"], by_name["y"], by_name["z"]]

    def ternary_op_constant(self, dest, dest_dims, a, a_dims, a_alpha, b, b_dims, b_alpha, constant, n_elems, op,
                            arg_order):
        self._ternary(dest, dest_dims, self._expand_arg_order(
            arg_order, [(a, a_dims, a_alpha), (b, b_dims, b_alpha), (None, None, constant)]), n_elems, op)

    def ternary_op_constant_constant(self, dest, dest_dims, a, a_dims, a_alpha, const_1, const_2, n_elems, op, arg_order):
        self._ternary(dest, dest_dims, self._expand_arg_order(
            arg_order, [(a, a_dims, a_alpha), (None, None, const_1), (None, None, const_2)]), n_elems, op)

    def gemv(self, c, inc_c, trans_a, alpha, a, a_row_count, a_col_count, a_colstride, x, inc_x, beta):
        self._tm("gemv", DTYPE_CODE[c.dtype], c.ptr, int(inc_c), 1 if trans_a else 0, float(alpha), a.ptr,
                 int(a_row_count), int(a_col_count), int(a_colstride), x.ptr, int(inc_x), float(beta))

    def batch_normalize_eltwise(self, output, input, means, variances, scale, bias, epsilon, batch_count, element_count):
        self._tm("batch_normalize_eltwise", DTYPE_CODE[output.dtype], output.ptr, input.ptr, means.ptr, variances.ptr,
                 scale.ptr, bias.ptr, float(epsilon), int(batch_count), int(element_count))

    def batch_normalize_spatial(self, output, input, means, variances, scale, bias, epsilon, batch_count, channel_count,
                                element_count):
        self._tm("batch_normalize_spatial", DTYPE_CODE[output.dtype], output.ptr, input.ptr, means.ptr, variances.ptr,
                 scale.ptr, bias.ptr, float(epsilon), int(batch_count), int(channel_count), int(element_count))

    def batch_normalize_update_and_apply_eltwise(self, output, input, batch_means, batch_variances, running_means,
                                                 running_variances, average_factor, scale, bias, epsilon, batch_count,
                                                 element_count):
        """tm/batch-normalize-update-and-apply-eltwise! (tensor/math.clj:137-148)."""
        self._tm("batch_normalize_update_and_apply_eltwise", DTYPE_CODE[output.dtype], output.ptr, input.ptr,
                 batch_means.ptr, batch_variances.ptr, running_means.ptr, running_variances.ptr, float(average_factor),
                 scale.ptr, bias.ptr, float(epsilon), int(batch_count), int(element_count))

    def batch_normalize_update_and_apply_spatial(self, output, input, batch_means, batch_variances, running_means,
                                                 running_variances, average_factor, scale, bias, epsilon, batch_count,
                                                 channel_count, element_count):
        """tm/batch-normalize-update-and-apply-spatial! (tensor/math.clj:149-158)."""
        self._tm("batch_normalize_update_and_apply_spatial", DTYPE_CODE[output.dtype], output.ptr, input.ptr,
                 batch_means.ptr, batch_variances.ptr, running_means.ptr, running_variances.ptr, float(average_factor),
                 scale.ptr, bias.ptr, float(epsilon), int(batch_count), int(channel_count), int(element_count))

    def batch_normalize_gradients_eltwise(self, input_gradient, scale_gradient, bias_gradient, output_gradient, output,
                                          input, batch_means, batch_variances, scale, bias, epsilon, batch_count,
                                          element_count):
        """tm/batch-normalize-gradients-eltwise! (tensor/math.clj:159-166)."""
        self._tm("batch_normalize_gradients_eltwise", DTYPE_CODE[output.dtype], input_gradient.ptr, scale_gradient.ptr,
                 bias_gradient.ptr, output_gradient.ptr, output.ptr, input.ptr, batch_means.ptr, batch_variances.ptr,
                 scale.ptr, bias.ptr, float(epsilon), int(batch_count), int(element_count))

    def batch_normalize_gradients_spatial(self, input_gradient, scale_gradient, bias_gradient, output_gradient, output,
                                          input, batch_means, batch_variances, scale, bias, epsilon, batch_count,
                                          channel_count, element_count):
        """tm/batch-normalize-gradients-spatial! (tensor/math.clj:167-174)."""
        self._tm("batch_normalize_gradients_spatial", DTYPE_CODE[output.dtype], input_gradient.ptr, scale_gradient.ptr,
                 bias_gradient.ptr, output_gradient.ptr, output.ptr, input.ptr, batch_means.ptr, batch_variances.ptr,
                 scale.ptr, bias.ptr, float(epsilon), int(batch_count), int(channel_count), int(element_count))

    def pooling_descriptor(self, datatype, kern_width, kern_height, pad_x, pad_y, stride_x, stride_y, pool_op,
                           dimension_op):
        """The reference builds a cudnn descriptor here; this backend needs none."""
        return None

    def pooling_forward(self, output, output_dims, output_alpha, input, input_dims, pool_descriptor):
        from ._lib import POOL_OPS, PoolDesc
        d = pool_descriptor
        desc = PoolDesc(d["kernel-width"], d["kernel-height"], d["pad-x"], d["pad-y"], d["stride-x"], d["stride-y"],
                        POOL_OPS[d["pool-op"]])
        self._tm("pooling_forward", DTYPE_CODE[output.dtype], output.ptr, C.byref(wire(output_dims)), float(output_alpha),
                 input.ptr, C.byref(wire(input_dims)), C.byref(desc))

    def pooling_backward(self, input_grad, input_grad_dims, input_grad_alpha, input, input_dims, output, output_dims,
                         output_grad, output_grad_dims, pool_descriptor):
        """tm/pooling-backward! (tensor/math.clj:223-236)."""
        from ._lib import POOL_OPS, PoolDesc
        d = pool_descriptor
        desc = PoolDesc(d["kernel-width"], d["kernel-height"], d["pad-x"], d["pad-y"], d["stride-x"], d["stride-y"],
                        POOL_OPS[d["pool-op"]])
        self._tm("pooling_backward", DTYPE_CODE[output.dtype], input_grad.ptr, C.byref(wire(input_grad_dims)),
                 float(input_grad_alpha), input.ptr, C.byref(wire(input_dims)), output.ptr, C.byref(wire(output_dims)),
                 output_grad.ptr, C.byref(wire(output_grad_dims)), C.byref(desc))

    def lrn_descriptor(self, n, k, alpha, beta):
        """tm/lrn-descriptor (tensor/math.clj:240): the reference builds a cudnn descriptor; here a plain record."""
        return {"n": int(n), "k": float(k), "alpha": float(alpha), "beta": float(beta)}

    @staticmethod
    def _lrn_desc(d):
        from ._lib import LrnDesc
        return LrnDesc(d["n"], d["k"], d["alpha"], d["beta"])

    def lrn_forward(self, output, output_dims, input, input_dims, lrn_descriptor):
        """tm/lrn-forward! (tensor/math.clj:242-245)."""
        desc = self._lrn_desc(lrn_descriptor)
        self._tm("lrn_forward", DTYPE_CODE[output.dtype], output.ptr, C.byref(wire(output_dims)), input.ptr,
                 C.byref(wire(input_dims)), C.byref(desc))

    def lrn_backward(self, input_gradient, input_grad_dims, output, output_dims, input, input_dims, output_gradient,
                     output_grad_dims, lrn_descriptor):
        """tm/lrn-backward! (tensor/math.clj:247-252)."""
        desc = self._lrn_desc(lrn_descriptor)
        self._tm("lrn_backward", DTYPE_CODE[output.dtype], input_gradient.ptr, C.byref(wire(input_grad_dims)),
                 output.ptr, C.byref(wire(output_dims)), input.ptr, C.byref(wire(input_dims)), output_gradient.ptr,
                 C.byref(wire(output_grad_dims)), C.byref(desc))

    def rand(self, dest, dest_dims, distribution, seed=0, sequence=0):
        """tm/rand! (tensor/math.clj:237) + the (seed, sequence) pair of the counter-based generator."""
        from ._lib import DISTRIBUTIONS
        kind = distribution["type"]
        p0, p1 = ((distribution["minimum"], distribution["maximum"]) if kind == "flat"
                  else (distribution["mean"], distribution["variance"]))
        self._tm("rand", dest.ptr, C.byref(wire(dest_dims)), DISTRIBUTIONS[kind], float(p0), float(p1),
                 int(seed) & 0xFFFFFFFFFFFFFFFF, int(sequence) & 0xFFFFFFFFFFFFFFFF)

    # --- optimiser steps (cortex.optimize.adam / adadelta): buffers are flat, already offset by the caller ---
    def adam_step(self, alpha, beta1, beta2, epsilon, pow_beta1_t, pow_beta2_t, gradient_alpha, gradient, parameters,
                  m, v, n_elems):
        self._tm("adam_step", DTYPE_CODE[parameters.dtype], float(alpha), float(beta1), float(beta2), float(epsilon),
                 float(pow_beta1_t), float(pow_beta2_t), float(gradient_alpha), gradient.ptr, parameters.ptr, m.ptr,
                 v.ptr, int(n_elems))

    def adadelta_step(self, decay, epsilon, grad_accum, dx_accum, gradient_beta, gradient, parameters, n_elems):
        self._tm("adadelta_step", DTYPE_CODE[parameters.dtype], float(decay), float(epsilon), grad_accum.ptr,
                 dx_accum.ptr, float(gradient_beta), gradient.ptr, parameters.ptr, int(n_elems))
