"""Backend-agnostic verification functions of the tensor API.

Transcribed from the reference's own verification namespace
(src/cortex/verify/tensor.clj): same inputs, same literal expected vectors.
Each function takes ``(driver, datatype)`` and is instantiated once per backend
(CPU oracle in the CPU suite, B200 in the ``gpu`` suite), which is how the
reference stamps out its CPU and CUDA tests
(test/clj/cortex/compute/{cpu,cuda}/tensor_test.clj).
"""
import contextlib
import math

import numpy as np

from cortex_b200 import dimensions as ct_dims
from cortex_b200 import tensor as ct
from cortex_b200.dimensions import ALL

ALL_DTYPES = ["byte", "short", "int", "long", "float", "double"]
CAS_DTYPES = ["int", "long", "float", "double"]
FLOAT_DTYPES = ["float", "double"]
INT_LONG = ["int", "long"]


@contextlib.contextmanager
def tensor_context(driver, datatype):
    stream = driver.default_device().create_stream()
    with ct.with_stream(stream), ct.with_datatype(datatype):
        yield stream
    stream.sync()


def _eq(expected, actual, tol=0.0):
    expected = np.asarray(expected, dtype=np.float64).reshape(-1)
    actual = np.asarray(actual, dtype=np.float64).reshape(-1)
    assert expected.shape == actual.shape, (expected.shape, actual.shape)
    if tol == 0.0:
        assert np.array_equal(expected, actual), (expected, actual)
    else:
        assert np.allclose(expected, actual, rtol=0, atol=tol), (expected, actual)


def _part(seq, n):
    seq = list(seq)
    return [seq[i:i + n] for i in range(0, len(seq), n)]


def assign_constant(driver, datatype):
    """verify/tensor.clj:20-42"""
    with tensor_context(driver, datatype):
        tensor = ct.to_tensor(_part(range(9), 3))
        assert tensor.ecount() == 9
        _eq(range(9), ct.to_double_array(tensor))
        ct.assign(tensor, 1)
        _eq([1] * 9, ct.to_double_array(tensor))
        rows, columns = ct.rows(tensor), ct.columns(tensor)
        for row in rows:
            ct.assign(row, 2)
        _eq([2] * 9, ct.to_double_array(tensor))
        c1, c2, c3 = columns
        ct.assign(c1, 1)
        ct.assign(c2, 2)
        ct.assign(c3, 3)
        _eq([1, 2, 3] * 3, ct.to_double_array(tensor))


def assign_marshal(driver, datatype):
    """verify/tensor.clj:45-57"""
    with tensor_context(driver, datatype):
        tensor = ct.to_tensor(_part(range(9), 3))
        intermediate = ct.new_tensor([3, 3], datatype="int")
        final = ct.new_tensor([3, 3], datatype="double")
        ct.assign(intermediate, tensor)
        ct.assign(final, intermediate)
        _eq(range(9), ct.to_double_array(final))


def unary_op(driver, datatype):
    """verify/tensor.clj:60-80"""
    with tensor_context(driver, datatype):
        tens_a = ct.to_tensor(_part(range(9), 3))
        tens_b = ct.to_tensor(_part([1] * 9, 3))
        a = float(ct.dtype_cast(2.5, datatype))
        ct.unary_op(tens_b, 2.5, tens_a, "ceil")
        _eq([math.ceil(v * a) for v in range(9)], ct.to_double_array(tens_b))
        ct.unary_op(tens_b, 1.0, tens_b, "-")
        _eq([-math.ceil(v * a) for v in range(9)], ct.to_double_array(tens_b))
        src = [0, 1, 2, 3, 4]
        tens_src, tens_b = ct.to_tensor(src), ct.to_tensor(src)
        tol = 1e-6 if datatype == "float" else 0.0   # fp32 views evaluate exp in single precision on the device
        ct.unary_op(tens_b, 1.0, tens_src, "exp")
        _eq([_cast(math.exp(v), datatype) for v in src], ct.to_double_array(tens_b), tol * math.exp(4))
        ct.unary_op(tens_b, 1.0, tens_src, "sqrt")
        _eq([_cast(math.sqrt(v), datatype) for v in src], ct.to_double_array(tens_b))


def _cast(v, datatype):
    if datatype == "double":
        return float(v)
    if datatype == "float":
        return float(np.float32(v))
    return int(v)


def channel_op(driver, datatype):
    """verify/tensor.clj:83-94"""
    with tensor_context(driver, datatype):
        tens_a = ct.to_tensor(np.arange(18).reshape(2, 3, 3))
        tens_chan = ct.in_place_reshape(ct.to_tensor(range(3)), [3, 1])
        tens_result = ct.new_tensor([2, 3, 3])
        ct.binary_op(tens_result, 1.0, tens_a, 1.0, tens_chan, "*")
        _eq([0.0, 0.0, 0.0, 3.0, 4.0, 5.0, 12.0, 14.0, 16.0, 0.0, 0.0, 0.0, 12.0, 13.0, 14.0, 30.0, 32.0, 34.0],
            ct.to_double_array(tens_result))


def binary_constant_op(driver, datatype):
    """verify/tensor.clj:97-126"""
    with tensor_context(driver, datatype):
        tens_a = ct.to_tensor(_part(range(9), 3))
        tens_b = ct.to_tensor(_part([1] * 9, 3))
        if datatype != "byte":
            ct.binary_op(tens_b, 2.0, tens_a, 3.0, 4.0, "*")
            _eq([24 * v for v in range(9)], ct.to_double_array(tens_b))
        ct.binary_op(tens_b, 2.0, tens_a, 3.0, 4.0, "+")
        _eq([12 + 2 * v for v in range(9)], ct.to_double_array(tens_b))
        # reversed operands
        ct.binary_op(tens_b, 3.0, 4.0, 2.0, tens_a, "-")
        _eq([12 - 2 * v for v in range(9)], ct.to_double_array(tens_b))
        ct.assign(tens_b, 1.0)
        _eq([1] * 9, ct.to_double_array(tens_b))
        # accumulation
        ct.binary_op(tens_b, 1.0, tens_b, 1.0, 1.0, "+")
        _eq([2] * 9, ct.to_double_array(tens_b))


def binary_op(driver, datatype):
    """verify/tensor.clj:129-249"""
    with tensor_context(driver, datatype):
        tens_a = ct.to_tensor(_part(range(9), 3))
        tens_b = ct.to_tensor(_part([2] * 9, 3))
        tens_c = ct.to_tensor(_part([10] * 9, 3))
        ct.binary_op(tens_c, 2.0, tens_a, 2.0, tens_b, "*")
        _eq([2 * 2 * 2 * v for v in range(9)], ct.to_double_array(tens_c))
        ct.binary_op(tens_b, 1.0, tens_c, 2.0, tens_a, "-")
        _eq([0.0, 6.0, 12.0, 18.0, 24.0, 30.0, 36.0, 42.0, 48.0], ct.to_double_array(tens_b))
        # destination is one of the operands
        ct.binary_op(tens_c, 1.0, tens_c, 2.0, tens_a, "-")
        _eq([0.0, 6.0, 12.0, 18.0, 24.0, 30.0, 36.0, 42.0, 48.0], ct.to_double_array(tens_c))
        if datatype in CAS_DTYPES:
            # destination smaller than the operation: broadcast-accumulate (needs the CAS form)
            tens_c_small = ct.subvector(tens_c, 0, length=3)
            sub = lambda nth: [row[nth] for row in _part(range(9), 3)]
            c_data = list(ct.to_double_array(tens_c))
            ct.binary_op(tens_c_small, 1.0, tens_c_small, 2.0, tens_a, "-")
            _eq([c_data[i] - sum(2.0 * v for v in sub(i)) for i in range(3)], ct.to_double_array(tens_c_small))
            c_data = list(ct.to_double_array(tens_c_small))
            ct.binary_op(tens_c_small, 2.0, tens_a, 1.0, tens_c_small, "+")
            _eq([c_data[i] + sum(2.0 * v for v in sub(i)) for i in range(3)], ct.to_double_array(tens_c_small))
        if datatype in FLOAT_DTYPES:
            n_batches, n_channels, img_dim = 3, 5, 4
            rng = np.random.default_rng(7)
            big = rng.random((n_batches, n_channels, img_dim, img_dim))
            sums = big.sum(axis=(0, 2, 3))
            big_m = ct.to_tensor(big)
            test_vec = ct.in_place_reshape(ct.new_tensor([n_channels]), [n_channels, 1, 1])
            ct.binary_op(test_vec, 1.0, test_vec, 1.0, big_m, "+")
            _eq(sums, ct.to_double_array(test_vec), 1e-4)
        tens_a4 = ct.to_tensor([_part(range(9), 3)] * 4)
        result = ct.new_tensor(tens_a4.shape())
        ct.binary_op(result, 1.0, tens_a4, 1.0, 5, "eq")
        _eq([1 if int(v) == 5 else 0 for v in ct.to_double_array(tens_a4)], ct.to_double_array(result))
        # bias add over [4 3 3]
        tens_z = ct.new_tensor([4, 3, 3])
        bias = ct.in_place_reshape(ct.to_tensor([1, 2, 3, 4]), [4, 1, 1])
        ct.binary_op(tens_z, 1.0, tens_z, 1.0, bias, "+")
        _eq([v for b in [1, 2, 3, 4] for v in [b] * 9], ct.to_double_array(tens_z))
        if datatype in CAS_DTYPES:
            # bias gradient: sum over everything but the channel
            tens_g = ct.to_tensor([np.full((3, 3), v) for v in [1, 2, 3, 4]])
            bias_g = ct.in_place_reshape(ct.new_tensor([4]), [4, 1, 1])
            ct.binary_op(bias_g, 1.0, tens_g, 1.0, bias_g, "+")
            _eq([9, 18, 27, 36], ct.to_double_array(bias_g))
        tens_1, tens_2 = ct.to_tensor([1, 1, 0, 0]), ct.to_tensor([-1, 1, 2, -2])
        result = ct.new_tensor(tens_2.shape())
        for op, expected in ((">", [1, 0, 0, 1]), (">=", [1, 1, 0, 1]), ("<", [0, 0, 1, 0]), ("<=", [0, 1, 1, 0])):
            ct.binary_op(result, 1.0, tens_1, 1.0, tens_2, op)
            _eq(expected, ct.to_double_array(result))
        tens_1, tens_2 = ct.to_tensor([1, 1, 0, 0]), ct.to_tensor([1, 1, 1, 1])
        result = ct.new_tensor(tens_2.shape())
        ct.binary_op(result, 1.0, tens_1, 1.0, tens_2, "bit-xor")
        _eq([0, 0, 1, 1], ct.to_double_array(result))


def gemm(driver, datatype):
    """verify/tensor.clj:252-284 -- also checks sub-matrix views"""
    with tensor_context(driver, datatype):
        tens_a = ct.to_tensor(_part(range(9), 3))
        tens_b = ct.to_tensor(_part([2] * 9, 3))
        tens_c = ct.to_tensor(_part([10] * 9, 3))
        ct.gemm(tens_c, False, False, 1, tens_a, tens_b, 1)
        _eq([16.0, 16.0, 16.0, 34.0, 34.0, 34.0, 52.0, 52.0, 52.0], ct.to_double_array(tens_c))
        ct.gemm(tens_c, False, False, 1, tens_a, tens_b, 0)
        _eq([6.0, 6.0, 6.0, 24.0, 24.0, 24.0, 42.0, 42.0, 42.0], ct.to_double_array(tens_c))
        ct.gemm(tens_c, True, False, 1, tens_a, tens_b, 0)
        _eq([18.0, 18.0, 18.0, 24.0, 24.0, 24.0, 30.0, 30.0, 30.0], ct.to_double_array(tens_c))
        sa, sb = ct.submatrix(tens_a, 0, 2, 0, 2), ct.submatrix(tens_b, 0, 2, 0, 2)
        sc = ct.submatrix(tens_c, 0, 2, 0, 2)
        ct.gemm(sc, False, False, 1, sa, sb, 0)
        _eq([2, 2, 14, 14], ct.to_double_array(sc))
        _eq([2.0, 2.0, 18.0, 14.0, 14.0, 24.0, 30.0, 30.0, 30.0], ct.to_double_array(tens_c))
        sa, sb = ct.submatrix(tens_a, 1, 2, 1, 2), ct.submatrix(tens_b, 0, 2, 0, 2)
        sc = ct.submatrix(tens_c, 1, 2, 1, 2)
        ct.gemm(sc, False, False, 1, sa, sb, 1)
        _eq([32, 42, 60, 60], ct.to_double_array(sc))
        _eq([2.0, 2.0, 18.0, 14.0, 32.0, 42.0, 30.0, 60.0, 60.0], ct.to_double_array(tens_c))


def activation_forward(driver, datatype):
    """verify/tensor.clj:532-554"""
    with tensor_context(driver, datatype):
        inp = ct.to_tensor(range(-4, 8))
        out = ct.new_tensor([12])
        ct.unary_op(out, 1.0, inp, "logistic")
        _eq([0.01798620996209156, 0.04742587317756678, 0.11920292202211755, 0.2689414213699951, 0.5,
             0.7310585786300049, 0.8807970779778823, 0.9525741268224334, 0.9820137900379085, 0.9933071490757153,
             0.9975273768433653, 0.9990889488055994], ct.to_double_array(out), 1e-4)
        ct.unary_op(out, 1.0, inp, "tanh")
        _eq([-0.999329299739067, -0.9950547536867305, -0.9640275800758169, -0.7615941559557649, 0.0,
             0.7615941559557649, 0.9640275800758169, 0.9950547536867305, 0.999329299739067, 0.9999092042625951,
             0.9999877116507956, 0.9999983369439447], ct.to_double_array(out), 1e-4)
        ct.binary_op(out, 1.0, inp, 0, 0, "max")
        _eq([0.0, 0.0, 0.0, 0.0, 0.0, 1.0, 2.0, 3.0, 4.0, 5.0, 6.0, 7.0], ct.to_double_array(out))


SOFTMAX_1234 = [0.03205860328008499, 0.08714431874203256, 0.2368828180899101, 0.6439142598879722]


def softmax(driver, datatype):
    """verify/tensor.clj:577-620"""
    with tensor_context(driver, datatype):
        inp = ct.to_tensor([[1, 2, 3, 4]] * 10)
        out = ct.new_tensor([10, 4])
        ct.softmax(out, inp)
        _eq(SOFTMAX_1234 * 10, ct.to_double_array(out), 1e-4)
        img_dim = 4
        inp = ct.to_tensor([[[v] * (img_dim * img_dim) for v in [1, 2, 3, 4]]])
        out = ct.new_tensor([1, 4, img_dim * img_dim])
        ct.softmax(out, inp)
        _eq([v for s in SOFTMAX_1234 for v in [s] * (img_dim * img_dim)], ct.to_double_array(out), 1e-4)
        # strided (non-contiguous) columns, in place
        pred = ct.to_tensor([list(range(10))] * 5)
        sel = ct.select(pred, ALL, list(range(2, 10)))
        test_tensor = ct.to_tensor(range(2, 10))
        answer = ct.softmax(test_tensor, test_tensor)
        ct.softmax(sel, sel)
        _eq(([0, 1] + list(ct.to_double_array(answer))) * 5, ct.to_double_array(pred))


def gemv(driver, datatype):
    """verify/tensor.clj:287-306"""
    with tensor_context(driver, datatype):
        tens_a = ct.to_tensor(np.arange(12).reshape(4, 3))
        tens_b = ct.to_tensor([2] * 4)
        tens_c = ct.to_tensor(list(range(4)))
        ct.subvector(tens_b, 0, length=3)     # built but unused in the reference test as well
        ct.gemv(tens_c, False, 1, tens_a, tens_b, 1)
        _eq([6.0, 25.0, 44.0, 63.0], ct.to_double_array(tens_c))
        ct.gemv(tens_c, False, 1, tens_a, tens_b, 0)
        _eq([6, 24, 42, 60], ct.to_double_array(tens_c))
        tens_c_sub = ct.subvector(tens_c, 0, length=3)
        tens_a_col = ct.columns(tens_a)[1]          # [1 4 7 10]
        ct.gemv(tens_c_sub, True, 1, tens_a, tens_a_col, 0)
        _eq([144.0, 166.0, 188.0], ct.to_double_array(tens_c_sub))


def batch_normalize(driver, datatype):
    """verify/tensor.clj:309-347 (inference form; a variance of 0 is included on purpose)"""
    with tensor_context(driver, datatype):
        inp = ct.to_tensor(np.arange(12).reshape(4, 3))
        out = ct.new_tensor([4, 3])
        means, variances = ct.to_tensor([1] * 3), ct.to_tensor(list(range(3)))
        scale, bias = ct.to_tensor([3] * 3), ct.to_tensor([4] * 3)
        ct.batch_normalize(out, inp, means, variances, scale, bias, 1e-2)
        _eq([-26.0, 4.0, 6.116036847575795, 64.0, 12.955334711889902, 12.46414739030318, 154.0, 21.910669423779805,
             18.812257933030565, 244.0, 30.86600413566971, 25.16036847575795], ct.to_double_array(out), 1e-4)
        inp = ct.to_tensor(np.arange(24).reshape(2, 3, 4))
        out = ct.new_tensor([2, 3, 4])
        ct.batch_normalize(out, inp, means, variances, scale, bias, 1e-2)
        _eq([-26.0, 4.0, 34.0, 64.0, 12.955334711889902, 15.94044628251987, 18.925557853149837, 21.910669423779805,
             18.812257933030565, 20.92829478060636, 23.044331628182157, 25.16036847575795, 334.0, 364.0, 394.0, 424.0,
             48.77667355944951, 51.76178513007948, 54.74689670070945, 57.73200827133942, 44.204700103940105,
             46.3207369515159, 48.436773799091696, 50.55281064666749], ct.to_double_array(out), 1e-4)


_BN_TRAIN_ELTWISE_OUT = [-0.023134696804511745, -0.023134696804511745, -0.023134696804511745, 2.6589551010651626,
                         2.6589551010651626, 2.6589551010651626, 5.341044898934837, 5.341044898934837,
                         5.341044898934837, 8.023134696804512, 8.023134696804512, 8.023134696804512]
_BN_TRAIN_SPATIAL_OUT = [0.3139510961275713, 0.8054242833105618, 1.2968974704935523, 1.7883706576765428,
                         0.3139510961275713, 0.8054242833105618, 1.2968974704935523, 1.7883706576765428,
                         0.3139510961275713, 0.8054242833105618, 1.2968974704935523, 1.7883706576765428,
                         6.211629342323457, 6.703102529506448, 7.194575716689438, 7.686048903872429,
                         6.211629342323457, 6.703102529506448, 7.194575716689438, 7.686048903872429,
                         6.211629342323457, 6.703102529506448, 7.194575716689438, 7.686048903872429]


def _bn_train_stats():
    return {"means": ct.to_tensor([1] * 3), "variances": ct.to_tensor(list(range(3))),       # a variance of 0 included
            "running-means": ct.to_tensor([2] * 3), "running-variances": ct.to_tensor([4] * 3),
            "scale": ct.to_tensor([3] * 3), "bias": ct.to_tensor([4] * 3)}


def batch_normalize_update_and_apply(driver, datatype):
    """verify/tensor.clj:349-428"""
    with tensor_context(driver, datatype):
        for shape, exp_out, exp_means, exp_rm, exp_rv in (
                ([4, 3], _BN_TRAIN_ELTWISE_OUT, [4.5, 5.5, 6.5], [4.0, 4.8, 5.6000000000000005], [12.8] * 3),
                ([2, 3, 4], _BN_TRAIN_SPATIAL_OUT, [7.5, 11.5, 15.5], [6.4, 9.6, 12.8], [34.857142857142854] * 3)):
            inp = ct.to_tensor(np.arange(int(np.prod(shape))).reshape(shape))
            out = ct.new_tensor(shape)
            st = _bn_train_stats()
            ct.batch_normalize_update_and_apply(out, inp, st["means"], st["variances"], st["running-means"],
                                                st["running-variances"], 0.8, st["scale"], st["bias"], 1e-2)
            _eq(exp_out, ct.to_double_array(out), 1e-4)
            _eq(exp_means, ct.to_double_array(st["means"]), 1e-4)
            _eq(exp_rm, ct.to_double_array(st["running-means"]), 1e-4)
            _eq(exp_rv, ct.to_double_array(st["running-variances"]), 1e-4)


def batch_normalize_gradients(driver, datatype):
    """verify/tensor.clj:431-530"""
    with tensor_context(driver, datatype):
        cases = (
            ([4, 3], _BN_TRAIN_ELTWISE_OUT,
             [-0.003572943780465465, -0.003572943780465465, -0.003572943780465465, -0.001190981260155155,
              -0.001190981260154711, -0.001190981260154489, 0.001190981260154933, 0.001190981260155155,
              0.0011909812601555991, 0.0035729437804663533, 0.0035729437804663533, 0.0035729437804663533], 1e-4,
             [13.410448989348373] * 3, [18, 22, 26]),
            ([2, 3, 4], _BN_TRAIN_SPATIAL_OUT,
             [-9.892777519776665E-4, -8.57374051714065E-4, -7.254703514504634E-4, -5.935666511868618E-4,
              -9.89277751978103E-4, -8.57374051714065E-4, -7.254703514500268E-4, -5.935666511868618E-4,
              -9.89277751978103E-4, -8.57374051714065E-4, -7.254703514500268E-4, -5.935666511868618E-4,
              5.935666511868618E-4, 7.254703514504634E-4, 8.57374051714065E-4, 9.892777519776665E-4,
              5.935666511868618E-4, 7.254703514500268E-4, 8.57374051714065E-4, 9.89277751978103E-4,
              5.935666511868618E-4, 7.254703514500268E-4, 8.57374051714065E-4, 9.89277751978103E-4], 1e-6,
             [48.81966992684372] * 3, [60.0, 92.0, 124.0]))
        for shape, exp_out, exp_in_grad, grad_tol, exp_scale_grad, exp_bias_grad in cases:
            n = int(np.prod(shape))
            inp = ct.to_tensor(np.arange(n).reshape(shape))
            out = ct.new_tensor(shape)
            in_grad = ct.new_tensor(shape)
            out_grad = ct.to_tensor(np.arange(n).reshape(shape))
            st = _bn_train_stats()
            scale_grad, bias_grad = ct.new_tensor([3]), ct.new_tensor([3])
            ct.batch_normalize_update_and_apply(out, inp, st["means"], st["variances"], st["running-means"],
                                                st["running-variances"], 0.8, st["scale"], st["bias"], 1e-2)
            ct.batch_normalize_gradients(in_grad, scale_grad, bias_grad, out_grad, out, inp, st["means"],
                                         st["variances"], st["scale"], st["bias"], 1e-2)
            _eq(exp_out, ct.to_double_array(out), 1e-4)
            _eq(exp_in_grad, ct.to_double_array(in_grad), grad_tol)
            _eq(exp_scale_grad, ct.to_double_array(scale_grad), 1e-4)
            _eq(exp_bias_grad, ct.to_double_array(bias_grad), 1e-4)


_POOL_MAX_BACKWARD = [
    0.0, 0.0, 0.0, 0.0, 0.0, 1.0, 0.0, 1.0, 0.0, 0.0, 0.0, 0.0, 0.0, 1.0, 0.0, 1.0, 0.0, 1.0, 0.0, 1.0, 0.0, 0.0,
    0.0, 0.0, 0.0, 0.0, 0.0, 0.0, 0.0, 1.0, 0.0, 1.0, 0.0, 0.0, 0.0, 0.0, 0.0, 2.0, 0.0, 2.0, 0.0, 0.0, 0.0, 0.0,
    0.0, 0.0, 0.0, 0.0, 0.0, 0.0, 0.0, 0.0, 0.0, 1.0, 0.0, 1.0, 0.0, 1.0, 0.0, 1.0, 0.0, 0.0, 0.0, 0.0, 0.0, 0.0,
    0.0, 0.0, 0.0, 1.0, 0.0, 1.0, 0.0, 0.0, 0.0, 0.0, 0.0, 1.0, 0.0, 1.0, 0.0, 0.0, 0.0, 0.0, 0.0, 1.0, 0.0, 1.0,
    0.0, 0.0, 0.0, 0.0, 0.0, 1.0, 0.0, 1.0, 0.0, 1.0, 0.0, 1.0, 0.0, 0.0, 0.0, 0.0, 0.0, 0.0, 0.0, 0.0, 0.0, 1.0,
    0.0, 1.0, 0.0, 0.0, 0.0, 0.0, 0.0, 2.0, 0.0, 2.0, 0.0, 0.0, 0.0, 0.0, 0.0, 0.0, 0.0, 0.0]


def pooling_operator(driver, datatype):
    """verify/tensor.clj:893-1033: the three pool operations forward, then backward with an output gradient of
    ones into zeroed input gradients."""
    with tensor_context(driver, datatype):
        channels, dimension, batch = 4, 4, 2
        n = batch * channels * dimension * dimension
        data = np.resize(np.arange(-5, 15), n).reshape(batch, channels, dimension, dimension)
        inp = ct.to_tensor(data)
        outs, grads = {}, {}
        for op in ("max", "avg", "avg-exc-pad"):
            desc = ct.pooling_descriptor(datatype, channels, 3, 3, 1, 1, 2, 2, pool_op=op, dimension_op="floor")
            od = ct.get_convolution_output_dimensions(desc, dimension, dimension)
            out_shape = [batch, channels, od["output-width"], od["output-height"]]
            out = ct.new_tensor(out_shape)
            ct.pooling_forward(out, 0.0, inp, desc)
            outs[op] = ct.to_double_array(out)
            out_grad = ct.to_tensor(np.ones(out_shape))
            in_grad = ct.new_tensor([batch, channels, dimension, dimension])
            ct.pooling_backward(in_grad, 0.0, inp, out, out_grad, desc)
            grads[op] = ct.to_double_array(in_grad)
        _eq([0.0, 2.0, 8.0, 10.0, 12.0, 14.0, 4.0, 6.0, 12.0, 14.0, 12.0, 14.0, 8.0, 10.0, 12.0, 14.0, 4.0, 6.0, 12.0,
             14.0, 0.0, 2.0, 8.0, 10.0, 12.0, 14.0, 4.0, 6.0, 12.0, 14.0, 12.0, 14.0], outs["max"])
        _eq([-1.1111111111111112, -0.6666666666666666, 2.3333333333333335, 5.0, 1.5555555555555556,
             3.3333333333333335, -0.3333333333333333, 1.0, 4.222222222222222, 7.333333333333333, 1.4444444444444444,
             3.6666666666666665, 2.4444444444444446, 4.666666666666667, 3.2222222222222223, 6.333333333333333,
             0.6666666666666666, 2.0, 5.0, 9.0, -1.1111111111111112, -0.6666666666666666, 2.3333333333333335, 5.0,
             1.5555555555555556, 3.3333333333333335, -0.3333333333333333, 1.0, 4.222222222222222, 7.333333333333333,
             1.4444444444444444, 3.6666666666666665], outs["avg"], 1e-4)
        _eq([-2.5, -1.0, 3.5, 5.0, 3.5, 5.0, -0.5, 1.0, 9.5, 11.0, 2.1666666666666665, 3.6666666666666665, 5.5, 7.0,
             4.833333333333333, 6.333333333333333, 1.5, 3.0, 7.5, 9.0, -2.5, -1.0, 3.5, 5.0, 3.5, 5.0, -0.5, 1.0, 9.5,
             11.0, 2.1666666666666665, 3.6666666666666665], outs["avg-exc-pad"], 1e-4)
        _eq(_POOL_MAX_BACKWARD, grads["max"], 1e-4)
        # the averaged forms give every plane the same pattern (the reference spells the 128 values out)
        ninth = 0.1111111111111111
        avg_plane = [ninth, 2 * ninth, ninth, ninth, 2 * ninth, 4 * ninth, 2 * ninth, 2 * ninth,
                     ninth, 2 * ninth, ninth, ninth, ninth, 2 * ninth, ninth, ninth]
        _eq(avg_plane * (batch * channels), grads["avg"], 1e-4)
        exc_plane = [0.25, 0.41666666666666663, 0.16666666666666666, 0.16666666666666666, 0.41666666666666663,
                     0.6944444444444444, 0.2777777777777778, 0.2777777777777778, 0.16666666666666666,
                     0.2777777777777778, ninth, ninth, 0.16666666666666666, 0.2777777777777778, ninth, ninth]
        _eq(exc_plane * (batch * channels), grads["avg-exc-pad"], 1e-4)


def _lrn_forward_backward(num_input_channels, lrn_n):
    """verify/tensor.clj:1068-1085"""
    batch_size, input_dim = 2, 2
    n_input = num_input_channels * input_dim * input_dim
    shape = [batch_size, num_input_channels, input_dim, input_dim]
    inp = ct.in_place_reshape(ct.to_tensor(list(range(n_input)) * batch_size), shape)
    out_grad = ct.in_place_reshape(ct.to_tensor([1.0] * (batch_size * n_input)), shape)
    out, in_grad = ct.new_tensor(shape), ct.new_tensor(shape)
    desc = ct.lrn_descriptor(n=lrn_n, k=1, alpha=1, beta=1)
    ct.lrn_forward(out, inp, desc)
    ct.lrn_backward(in_grad, out, inp, out_grad, desc)
    return ct.to_double_array(out), ct.to_double_array(in_grad), ct.to_double_array(inp)


def lrn_operator(driver, datatype):
    """verify/tensor.clj:1088-1136 (the reference runs it on its CUDA backend only)"""
    with tensor_context(driver, datatype):
        out, in_grad, data = _lrn_forward_backward(3, 1)
        _eq([v / (1 + v * v) for v in data], out, 1e-4)
        _eq([1.0, 0.0, -0.12000000000000002, -0.07999999999999999, -0.0519031141868512, -0.03550295857988165,
             -0.02556610664718773, -0.019200000000000002, -0.0149112426035503, -0.01189767995240928,
             -0.009704930889128518, -0.008062348830959416] * 2, in_grad, 1e-4)
        out, in_grad, _ = _lrn_forward_backward(3, 2)
        _eq([0.0, 0.07142857142857142, 0.09523809523809523, 0.1, 0.0975609756097561, 0.09259259259259259,
             0.08695652173913043, 0.08139534883720931, 0.24242424242424243, 0.21686746987951808, 0.19607843137254902,
             0.17886178861788618] * 2, out, 1e-4)
        _eq([0.1111111111111111, 0.06461185297164132, 0.03602827394347783, 0.020493960699477193,
             -0.014512656716972328, -0.016183480513356906, -0.016136733799491102, -0.015355548198598244,
             -0.02846648301193755, -0.022935113949774988, -0.0188389081122645, -0.015731376825963386] * 2, in_grad, 1e-4)
        out, in_grad, _ = _lrn_forward_backward(3, 3)
        _eq([0.0, 0.10344827586206898, 0.13953488372093023, 0.14754098360655737, 0.14457831325301207,
             0.13636363636363638, 0.1258741258741259, 0.11538461538461539, 0.28915662650602414, 0.24770642201834867,
             0.21582733812949642, 0.19075144508670522] * 2, out, 1e-4)
        _eq([0.15789473684210528, 0.09383457316653729, 0.05326649810721716, 0.030864211553852466,
             -0.005661199012919144, -0.04352114602312829, -0.04715638623434852, -0.04169062137988738,
             -0.047466976339091305, -0.03569676147971518, -0.027076332292621106, -0.020863959610017586] * 2, in_grad, 1e-4)


def ternary_op_select(driver, datatype):
    """verify/tensor.clj:623-645"""
    with tensor_context(driver, datatype):
        dest = ct.to_tensor([0] * 10)
        x_arg = ct.to_tensor(list(range(-5, 5)))
        y_arg = ct.to_tensor(list(range(10)))
        z_arg = ct.to_tensor([2] * 10)
        ct.ternary_op(dest, 1, x_arg, 2.0, y_arg, 3.0, z_arg, "select")
        _eq([0, 2, 4, 6, 8, 6, 6, 6, 6, 6], ct.to_double_array(dest))
        ct.ternary_op(dest, 1, x_arg, 1.0, -1, 3.0, z_arg, "select")
        _eq([-1, -1, -1, -1, -1, 6, 6, 6, 6, 6], ct.to_double_array(dest))
        ct.ternary_op(dest, 1, x_arg, 3.0, z_arg, 1.0, -1, "select")
        _eq([6, 6, 6, 6, 6, -1, -1, -1, -1, -1], ct.to_double_array(dest))
        ct.ternary_op(dest, 1, x_arg, 3.0, 2.0, 1.0, -1, "select")
        _eq([6, 6, 6, 6, 6, -1, -1, -1, -1, -1], ct.to_double_array(dest))
        ct.ternary_op(dest, 1, x_arg, 1.0, -1, 3.0, 2.0, "select")
        _eq([-1, -1, -1, -1, -1, 6, 6, 6, 6, 6], ct.to_double_array(dest))


def activation_gradient(driver, datatype):
    """verify/tensor.clj:557-574"""
    with tensor_context(driver, datatype):
        output = ct.to_tensor(list(range(12)))
        output_gradient = ct.to_tensor(list(range(-4, 8)))
        input_gradient = ct.new_tensor([12])
        ct.activation_gradient(input_gradient, output_gradient, output, "logistic")
        _eq([-0.0, -0.0, 4.0, 6.0, -0.0, -20.0, -60.0, -126.0, -224.0, -360.0, -540.0, -770.0],
            ct.to_double_array(input_gradient))
        ct.activation_gradient(input_gradient, output_gradient, output, "tanh")
        _eq([-4.0, -0.0, 6.0, 8.0, -0.0, -24.0, -70.0, -144.0, -252.0, -400.0, -594.0, -840.0],
            ct.to_double_array(input_gradient))
        ct.activation_gradient(input_gradient, output_gradient, output, "relu")
        _eq([0.0, -3.0, -2.0, -1.0, 0.0, 1.0, 2.0, 3.0, 4.0, 5.0, 6.0, 7.0], ct.to_double_array(input_gradient))


def linear_layer_backward(driver, datatype):
    """verify/nn/layers.clj:193-235 (linear, linear-batch): forward, then biased-multiply-backward! into
    zeroed gradient buffers."""
    from cortex_b200 import nn
    with tensor_context(driver, datatype):
        for batch in (1, 10):
            lin = nn.Linear(ct.to_tensor([[1, 2], [3, 4]]), ct.to_tensor([0, 10]))
            x = ct.to_tensor([[1, 2]] * batch)
            out_grad = ct.to_tensor([[1, 2]] * batch)
            out, in_grad = ct.new_tensor([batch, 2]), ct.new_tensor([batch, 2])
            w_grad, b_grad = ct.new_tensor([2, 2]), ct.new_tensor([2])
            lin.forward(x, out)
            lin.backward(x, out, in_grad, out_grad, w_grad, b_grad)
            _eq([5, 21] * batch, ct.to_double_array(out))
            _eq([v * batch for v in (1, 2, 2, 4)], ct.to_double_array(w_grad))
            _eq([v * batch for v in (1, 2)], ct.to_double_array(b_grad))
            _eq([7, 10] * batch, ct.to_double_array(in_grad))


def relu_layer_backward(driver, datatype):
    """verify/nn/layers.clj:155-191 (relu-activation, relu-activation-batch)"""
    from cortex_b200 import nn
    with tensor_context(driver, datatype):
        for batch, items in ((1, 10), (5, 10000)):
            act = nn.Activation("relu")
            x = ct.to_tensor(np.tile([-1, 1], batch * items // 2).reshape(batch, items))
            out_grad = ct.to_tensor(np.ones((batch, items)))
            out, in_grad = ct.new_tensor([batch, items]), ct.new_tensor([batch, items])
            act.forward(x, out)
            act.backward(out, in_grad, out_grad)
            assert float(np.sum(ct.to_double_array(out))) == batch * items / 2
            assert float(np.sum(ct.to_double_array(in_grad))) == batch * items / 2


def softmax_layer(driver, datatype):
    """verify/nn/layers.clj:399-499: softmax, softmax-batch, softmax-image (spatial: one softmax per pixel over
    4 channels), softmax-batch-channels (:output-channels 4), forward and backward through the layer."""
    from cortex_b200 import nn
    row = [0.015127670383492609, 0.041121271510366035, 0.11177920510975863, 0.30384738204945333,
           0.015127670383492609, 0.041121271510366035, 0.11177920510975863, 0.30384738204945333,
           0.015127670383492609, 0.041121271510366035]
    chan = [0.03205860328008499, 0.08714431874203257, 0.23688281808991013, 0.6439142598879724]
    tol = 1e-6 / 10 if datatype == "double" else 1e-6       # about-there?: summed abs difference < 1e-6
    with tensor_context(driver, datatype):
        for batch in (1, 10):                                 # softmax, softmax-batch
            layer = nn.Softmax()
            x = ct.to_tensor([([1, 2, 3, 4] * 3)[:10]] * batch)
            out, in_grad = ct.new_tensor([batch, 10]), ct.new_tensor([batch, 10])
            out_grad = ct.to_tensor(np.ones((batch, 10)))
            layer.forward(x, out)
            layer.backward(in_grad, out_grad)
            _eq(row * batch, ct.to_double_array(out), tol)
            _eq([1.0] * (10 * batch), ct.to_double_array(in_grad))
        # softmax-image: input 5x5 image, 4 channels, channel c filled with c + 1
        img = 5
        layer = nn.Softmax(output_channels=1, input_dimension=(4, img, img))
        data = [[float(c)] * (img * img) for c in range(1, 5)]
        x = ct.to_tensor([np.asarray(data).reshape(-1)])
        out, in_grad = ct.new_tensor([1, 4 * img * img]), ct.new_tensor([1, 4 * img * img])
        out_grad = ct.to_tensor([np.asarray(data).reshape(-1)])
        layer.forward(x, out)
        layer.backward(in_grad, out_grad)
        _eq([v for c in chan for v in [c] * (img * img)], ct.to_double_array(out), 1e-4)
        _eq(np.asarray(data).reshape(-1), ct.to_double_array(in_grad), 1e-6)
        # softmax-batch-channels: 10 pixels of [1 2 3 4], :output-channels 4
        batch, pixels = 10, 10
        layer = nn.Softmax(output_channels=4)
        x = ct.to_tensor([[1, 2, 3, 4] * pixels] * batch)
        out, in_grad = ct.new_tensor([batch, 4 * pixels]), ct.new_tensor([batch, 4 * pixels])
        out_grad = ct.to_tensor(np.ones((batch, 4 * pixels)))
        layer.forward(x, out)
        layer.backward(in_grad, out_grad)
        assert float(np.abs(np.asarray(chan * (pixels * batch)) - ct.to_double_array(out).reshape(-1)).sum()) < 1e-4
        _eq([1.0] * (4 * pixels * batch), ct.to_double_array(in_grad))


def basic_conv_layer(driver, datatype):
    """verify/nn/layers.clj:502-556: 2x2 kernels (kernel k filled with k, bias 1) over a 3x3 and a 3-wide x
    4-high single-channel input, batch 10: output, weight / bias gradients and input gradient."""
    from cortex_b200 import nn
    cases = [
        # (in_w, in_h, out_grad per image, output, weight grad per kernel, bias grad, input grad)
        (3, 3, [13.0, 17.0, 25.0, 29.0, 25.0, 33.0, 49.0, 57.0, 37.0, 49.0, 73.0, 85.0, 49.0, 65.0, 97.0, 113.0],
         [120.0, 160.0, 240.0, 280.0], 4, [1, 2, 1, 2, 4, 2, 1, 2, 1]),
        (3, 4, [13.0, 17.0, 25.0, 29.0, 37.0, 41.0, 25.0, 33.0, 49.0, 57.0, 73.0, 81.0, 37.0, 49.0, 73.0, 85.0, 109.0,
                121.0, 49.0, 65.0, 97.0, 113.0, 145.0, 161.0],
         [270.0, 330.0, 450.0, 510.0], 6, [1, 2, 1, 2, 4, 2, 2, 4, 2, 1, 2, 1]),
    ]
    batch, kernels, k = 10, 4, 2
    with tensor_context(driver, datatype):
        for in_w, in_h, output, w_grad_k, bias_per_image, in_grad_unit in cases:
            out_w, out_h = in_w - k + 1, in_h - k + 1
            weights = ct.to_tensor([[float(i)] * (k * k) for i in range(1, kernels + 1)])
            bias = ct.to_tensor([1.0] * kernels)
            layer = nn.Convolution(weights, bias, (k, k), (0, 0), (1, 1), 1, kernels, datatype)
            x = ct.to_tensor(np.tile(np.arange(1, in_w * in_h + 1), batch).reshape(batch, 1, in_h, in_w))
            out = ct.new_tensor([batch, kernels, out_h, out_w])
            out_grad = ct.to_tensor(np.ones((batch, kernels, out_h, out_w)))
            in_grad = ct.new_tensor([batch, 1, in_h, in_w])
            w_grad, b_grad = ct.new_tensor([kernels, k * k]), ct.new_tensor([kernels])
            layer.forward(x, out)
            layer.backward(x, in_grad, out_grad, w_grad, b_grad)
            _eq(output * batch, ct.to_double_array(out))
            _eq(w_grad_k * kernels, ct.to_double_array(w_grad))
            _eq([float(bias_per_image * batch)] * kernels, ct.to_double_array(b_grad))
            _eq([10.0 * v for v in in_grad_unit] * batch, ct.to_double_array(in_grad))


ADAM_ANSWERS = [
    [0.999000000005, 1.9990000000025, 2.9990000000016668, 3.99900000000125],
    [0.9980000262138343, 1.9980000130723587, 2.998000008707231, 3.998000006527546],
    [0.9970000960651408, 1.9970000478972731, 2.9970000319014805, 3.9970000239148513],
    [0.9960002269257634, 1.9960001131228113, 2.9960000753397424, 3.9960000564765217],
    [0.995000436052392, 1.9950002173334274, 2.995000144735273, 3.995000108493863],
    [0.9940007405541528, 1.9940003690339771, 2.994000245746984, 3.9940001842069432],
    [0.9930011573564278, 1.9930005766318695, 2.9930003839675967, 3.993000287805732],
    [0.9920017031661642, 1.9920008484199827, 2.992000564912314, 3.992000423421624],
    [0.9910023944389119, 1.991001192560463, 2.9910007940080785, 3.9910005951194076],
    [0.9900032473478027, 1.9900016170695067, 2.9900010765834972, 3.990000806889731],
    [0.9890042777546556, 1.9890021298032192, 2.9890014178594777, 3.9890010626421075],
    [0.9880055011833645, 1.9880027384446224, 2.9880018229406398, 3.988001366198499],
    [0.9870069327956914, 1.987003450491873, 2.98700229680753, 3.9870017212875037],
    [0.9860085873695607, 1.986004273247733, 2.9860028443096756, 3.9860021315391725],
    [0.9850104792799151, 1.9850052138103236, 2.9850034701594894, 3.9850026004804673],
    [0.9840126224821667, 1.984006279065173, 2.984004178927043, 3.984003131531364],
    [0.9830150304982433, 1.9830074756785594, 2.9830049750356973, 3.9830037280016044],
    [0.9820177164052082, 1.9820088100921336, 2.982005862758586, 3.9820043930880837],
    [0.9810206928263993, 1.9810102885187928, 2.981006846215933, 3.9810051298728633],
]


def adam_optimizer(driver, datatype):
    """compute/verify/optimize.clj:11-61 (test-adam): 19 steps on parameters [1 2 3 4] with gradient
    2 * parameters; a second buffer at offset 4 of m / v stepped with gradient-alpha 0 must not move.
    about-there? = summed abs difference < 1e-6; a float buffer cannot hold the literals closer than its
    own spacing (2.4e-7 at 4.0), so floats are compared at 2e-6."""
    from cortex_b200 import optimize
    tol = 1e-6 if datatype == "double" else 2e-6
    with tensor_context(driver, datatype):
        parameters_1, parameters_2 = ct.to_tensor([1, 2, 3, 4]), ct.to_tensor([1, 2, 3, 4])
        state = {"m": ct.new_tensor([8]), "v": ct.new_tensor([8])}
        optimizer = optimize.Adam()
        for item in ADAM_ANSWERS:
            gradient_1 = ct.to_tensor(2.0 * ct.to_double_array(parameters_1))
            gradient_2 = ct.to_tensor(2.0 * ct.to_double_array(parameters_2))
            optimizer = optimizer.batch_update()
            optimizer.compute_parameters(state, 1.0, 0, gradient_1, parameters_1)
            optimizer.compute_parameters(state, 0.0, 4, gradient_2, parameters_2)
            assert float(np.abs(ct.to_double_array(parameters_1) - np.asarray(item)).sum()) < tol
            assert float(np.abs(ct.to_double_array(parameters_2) - np.asarray([1.0, 2.0, 3.0, 4.0])).sum()) < 1e-6


def rand_operator(driver, datatype):
    """verify/tensor.clj:1036-1066: mean and variance of 10,000 draws within 1 of the request, for means /
    variances 1..10 (gaussian) and centres 1..10 with half-width 2 (flat)."""
    with tensor_context(driver, datatype):
        test_vec = []
        for idx in range(1, 11):
            tens = ct.rand(ct.new_tensor([10000]), ct.gaussian_distribution(mean=idx, variance=idx))
            values = ct.to_double_array(tens)
            test_vec += [float(np.mean(values)), float(np.var(values, ddof=1))]
        expected = [v for idx in range(1, 11) for v in (idx, idx)]
        assert np.all(np.abs(np.asarray(test_vec) - np.asarray(expected)) <= 1.0), test_vec
        test_vec = []
        for idx in range(1, 11):
            tens = ct.rand(ct.new_tensor([10000]), ct.flat_distribution(minimum=idx - 2, maximum=idx + 2))
            values = ct.to_double_array(tens)
            assert values.min() >= idx - 2 and values.max() <= idx + 2
            test_vec.append(float(np.mean(values)))
        assert np.all(np.abs(np.asarray(test_vec) - np.arange(1, 11)) <= 1.0), test_vec


def unary_reduce(driver, datatype):
    """verify/tensor.clj:648-665"""
    with tensor_context(driver, datatype):
        dest = ct.new_tensor([10, 1])
        src_data = [0, 3, 5, 2, 1, 9, 5, 7, 7, 2]
        src = ct.to_tensor([src_data] * 10)
        ct.unary_reduce(dest, 2.0, src, "max")
        _eq([18] * 10, ct.to_double_array(dest))
        ct.unary_reduce(dest, 1.0, src, "sum")
        _eq([sum(src_data)] * 10, ct.to_double_array(dest))
        ct.unary_reduce(dest, 1.0, src, "mean")
        _eq([_cast(sum(src_data) / len(src_data), datatype)] * 10, ct.to_double_array(dest))


def transpose(driver, datatype):
    """verify/tensor.clj:668-684"""
    with tensor_context(driver, datatype):
        img_dim = 4
        img = ct.to_tensor(np.tile(np.array([1, 2, 3]), (img_dim, img_dim, 1)))
        planar = ct.transpose(img, [2, 0, 1])
        rgb = ct.transpose(planar, [1, 2, 0])
        n = img_dim * img_dim
        _eq([1] * n + [2] * n + [3] * n, ct.to_double_array(planar))
        _eq([1, 2, 3] * n, ct.to_double_array(rgb))


def mask(driver, datatype):
    """verify/tensor.clj:687-717 (int and long only)"""
    with tensor_context(driver, datatype):
        rgba = 1 + (2 << 8) + (3 << 16) + (255 << 24)
        if datatype == "int":
            rgba -= 1 << 32   # the reference builds it from (int ...) values: wraps to a negative int
        img_dim = 4
        img = ct.to_tensor(np.full((img_dim, img_dim), rgba, dtype=np.int64))
        mask_t = ct.in_place_reshape(ct.to_tensor([0xFF, 0xFF << 8, 0xFF << 16]), [3, 1, 1])
        div_t = ct.in_place_reshape(ct.to_tensor([1, 1 << 8, 1 << 16]), [3, 1, 1])
        result = ct.new_tensor([3, img_dim, img_dim])
        ct.binary_op(result, 1.0, img, 1.0, mask_t, "bit-and")
        ct.binary_op(result, 1.0, result, 1.0, div_t, "/")
        n = img_dim * img_dim
        _eq([1] * n + [2] * n + [3] * n, ct.to_double_array(result))


def select(driver, datatype):
    """verify/tensor.clj:720-782"""
    with tensor_context(driver, datatype):
        mat = ct.to_tensor([_part(range(9), 3)] * 2)
        s = ct.select(mat, ALL, ALL, [1, 2])
        _eq([1, 2, 4, 5, 7, 8] * 2, ct.to_double_array(s))
        assert s.shape() == [2, 3, 2]
        s = ct.select(mat, ALL, ALL, [2])
        _eq([2, 5, 8] * 2, ct.to_double_array(s))
        assert s.shape() == [2, 3, 1]
        s = ct.select(mat, ALL, ALL, 2)
        _eq([2, 5, 8] * 2, ct.to_double_array(s))
        assert s.shape() == [2, 3] and not ct.dense(s)
        s = ct.select(mat, ALL, [1, 2], ALL)
        _eq([3, 4, 5, 6, 7, 8] * 2, ct.to_double_array(s))
        assert s.shape() == [2, 2, 3] and not ct.dense(s)
        s = ct.select(mat, ALL, [2], ALL)
        _eq([6, 7, 8] * 2, ct.to_double_array(s))
        assert s.shape() == [2, 1, 3] and not ct.dense(s)
        s = ct.select(mat, ALL, 0, ALL)
        _eq([0, 1, 2] * 2, ct.to_double_array(s))
        assert s.shape() == [2, 3] and not ct.dense(s)
        s = ct.select(mat, [1], [1], ALL)
        _eq([3, 4, 5], ct.to_double_array(s))
        assert s.shape() == [1, 1, 3] and ct.dense(s)
        s = ct.select(mat, 1, 1, ALL)
        _eq([3, 4, 5], ct.to_double_array(s))
        assert s.shape() == [3] and ct.dense(s)
        s = ct.select(mat, 1, ALL, 2)
        _eq([2, 5, 8], ct.to_double_array(s))
        assert s.shape() == [3] and not ct.dense(s)


def select_transpose_interaction(driver, datatype):
    """verify/tensor.clj:785-805"""
    with tensor_context(driver, datatype):
        img_dim = 4
        mat = ct.to_tensor(np.tile(np.array([1, 2, 3]), (img_dim, img_dim, 1)))
        planar = ct.transpose(mat, [2, 0, 1])
        n = img_dim * img_dim
        r, g, b = (ct.select(planar, c, ALL, ALL) for c in range(3))
        _eq([1] * n, ct.to_double_array(r))
        _eq([2] * n, ct.to_double_array(g))
        _eq([3] * n, ct.to_double_array(b))
        bgr = ct.new_tensor([img_dim, img_dim, 3])
        planes = ct.transpose(bgr, [2, 0, 1])
        ct.assign(ct.select(planes, 0, ALL, ALL), b)
        ct.assign(ct.select(planes, 1, ALL, ALL), g)
        ct.assign(ct.select(planes, 2, ALL, ALL), r)
        _eq([3, 2, 1] * n, ct.to_double_array(bgr))


CONV_EXPECTED = [25062.0, 25692.0, 27582.0, 28212.0, 62646.0, 64572.0, 70350.0, 72276.0, 100230.0, 103452.0, 113118.0,
                 116340.0, 65382.0, 66012.0, 67902.0, 68532.0, 185910.0, 187836.0, 193614.0, 195540.0, 306438.0,
                 309660.0, 319326.0, 322548.0, 105702.0, 106332.0, 108222.0, 108852.0, 309174.0, 311100.0, 316878.0,
                 318804.0, 512646.0, 515868.0, 525534.0, 528756.0]


CONV_WEIGHT_GRADIENT = [798, 810, 822, 846, 858, 870, 894, 906, 918, 990, 1002, 1014, 1038, 1050, 1062, 1086,
        1098, 1110, 1182, 1194, 1206, 1230, 1242, 1254, 1278, 1290, 1302, 1374, 1386, 1398, 1422, 1434, 1446, 1470,
        1482, 1494, 798, 810, 822, 846, 858, 870, 894, 906, 918, 990, 1002, 1014, 1038, 1050, 1062, 1086, 1098,
        1110, 1182, 1194, 1206, 1230, 1242, 1254, 1278, 1290, 1302, 1374, 1386, 1398, 1422, 1434, 1446, 1470, 1482,
        1494, 798, 810, 822, 846, 858, 870, 894, 906, 918, 990, 1002, 1014, 1038, 1050, 1062, 1086, 1098, 1110,
        1182, 1194, 1206, 1230, 1242, 1254, 1278, 1290, 1302, 1374, 1386, 1398, 1422, 1434, 1446, 1470, 1482, 1494]

CONV_INPUT_GRADIENT = [108, 219, 225, 114, 225, 456, 468, 237, 243, 492, 504, 255, 126, 255, 261, 132, 135,
        273, 279, 141, 279, 564, 576, 291, 297, 600, 612, 309, 153, 309, 315, 159, 162, 327, 333, 168, 333, 672,
        684, 345, 351, 708, 720, 363, 180, 363, 369, 186, 189, 381, 387, 195, 387, 780, 792, 399, 405, 816, 828,
        417, 207, 417, 423, 213, 108, 219, 225, 114, 225, 456, 468, 237, 243, 492, 504, 255, 126, 255, 261, 132,
        135, 273, 279, 141, 279, 564, 576, 291, 297, 600, 612, 309, 153, 309, 315, 159, 162, 327, 333, 168, 333,
        672, 684, 345, 351, 708, 720, 363, 180, 363, 369, 186, 189, 381, 387, 195, 387, 780, 792, 399, 405, 816,
        828, 417, 207, 417, 423, 213, 108, 219, 225, 114, 225, 456, 468, 237, 243, 492, 504, 255, 126, 255, 261,
        132, 135, 273, 279, 141, 279, 564, 576, 291, 297, 600, 612, 309, 153, 309, 315, 159, 162, 327, 333, 168,
        333, 672, 684, 345, 351, 708, 720, 363, 180, 363, 369, 186, 189, 381, 387, 195, 387, 780, 792, 399, 405,
        816, 828, 417, 207, 417, 423, 213]


def convolution_operator(driver, datatype):
    """verify/tensor.clj:808-890 (forward, backward-weights, backward-data)"""
    with tensor_context(driver, datatype):
        batch, cin, cout, dim = 3, 4, 3, 4
        inp = ct.to_tensor(np.arange(dim * dim * batch * cin).reshape(batch, cin, dim, dim))
        desc = ct.convolution_descriptor(datatype, cout, cin, 3, 3, 0, 0, 1, 1)
        od = ct.get_convolution_output_dimensions(desc, dim, dim)
        out = ct.new_tensor([batch, cout, od["output-height"], od["output-width"]])
        algorithms = ct.choose_convolution_algorithms(desc, dim, dim, batch, 1000)
        workspace = ct.new_tensor([int(algorithms["workspace-size"])])
        weights = ct.to_tensor(np.arange(cout * 3 * 3 * cin).reshape(cout, 3 * 3 * cin))
        ct.assign(out, 1)   # pre-existing contents must not leak through out_alpha = 0
        ct.convolution_forward(out, 0.0, inp, weights, workspace, desc, algorithms)
        tol = 0.0 if datatype == "double" else 0.5   # exact in fp64; fp32 results reach 5e5 (ulp 0.03)
        _eq(CONV_EXPECTED, ct.to_double_array(out), tol)
        out_grad = ct.in_place_reshape(ct.to_tensor([1] * (batch * cout * od["output-height"] * od["output-width"])),
                                       [batch, cout, od["output-height"], od["output-width"]])
        weight_gradient, input_gradient = ct.new_tensor(weights.shape()), ct.new_tensor(inp.shape())
        ct.assign(weight_gradient, 1)   # pre-existing contents must not leak through alpha = 0
        ct.assign(input_gradient, 1)
        ct.convolution_backward_weights(weight_gradient, 0.0, out_grad, inp, workspace, desc, algorithms)
        _eq(CONV_WEIGHT_GRADIENT, ct.to_double_array(weight_gradient))
        ct.convolution_backward_data(input_gradient, 0.0, out_grad, weights, workspace, desc, algorithms)
        _eq(CONV_INPUT_GRADIENT, ct.to_double_array(input_gradient))


def indexed_tensor(driver, datatype):
    """verify/tensor.clj:1147-1199"""
    with tensor_context(driver, datatype):
        mat = ct.to_tensor([_part(range(9), 3)] * 2)
        index = ct.to_tensor([1, 2, 1, 2, 1, 2], datatype="int")
        sel = ct.select(mat, ALL, ALL, index)
        assert not ct_dims.access_increasing(sel.dimensions)
        assert sel.shape() == [2, 3, 6]
        _eq([1, 2, 1, 2, 1, 2, 4, 5, 4, 5, 4, 5, 7, 8, 7, 8, 7, 8] * 2, ct.to_double_array(sel))
        # the center-loss pattern: gather rows, then scatter-accumulate through the same index
        centers = ct.select(mat, 0, ct.to_tensor([0, 1, 0, 2, 1], datatype="int"), ALL)
        batch_data = ct.new_tensor([5, 3])
        ct.assign(batch_data, centers)
        _eq([0, 1, 2, 3, 4, 5, 0, 1, 2, 6, 7, 8, 3, 4, 5], ct.to_double_array(batch_data))
        if datatype in CAS_DTYPES:
            ct.binary_op(centers, 1.0, batch_data, 1.0, centers, "+")
            _eq([0, 3, 6, 9, 12, 15, 0, 3, 6, 12, 14, 16, 9, 12, 15], ct.to_double_array(centers))
        # broadcasting with several indexes in one tensor
        mat2 = ct.to_tensor(_part(range(9), 3))
        sel2 = ct.select(mat2, ct.to_tensor([0, 1, 1, 2], datatype="int"), ct.to_tensor([2, 1, 0], datatype="int"))
        dest = ct.new_tensor([8, 6])
        ct.assign(dest, sel2)
        rows = [[2, 1, 0], [2, 1, 0], [5, 4, 3], [5, 4, 3], [5, 4, 3], [5, 4, 3], [8, 7, 6], [8, 7, 6]] * 2
        _eq([v for r in rows for v in r], ct.to_double_array(dest))


def magnitude_and_mag_squared(driver, datatype):
    """verify/tensor.clj:1202-1228"""
    with tensor_context(driver, datatype):
        n = 10
        src_data = np.arange(n * n).reshape(n, n)
        src = ct.to_tensor(src_data)
        dst = ct.new_tensor([n, 1])
        ct.unary_reduce(dst, 1.0, src, "magnitude-squared")
        _eq((src_data.astype(np.float64) ** 2).sum(axis=1), ct.to_double_array(dst), 1e-4)
        ct.unary_reduce(dst, 1.0, src, "magnitude")
        expected = np.sqrt((src_data.astype(np.float64) ** 2).sum(axis=1))
        tol = 1e-4 if datatype in FLOAT_DTYPES else 1.0   # integer views store the truncated square root
        _eq(expected if datatype in FLOAT_DTYPES else np.floor(expected), ct.to_double_array(dst), tol)


# how the reference instantiates them (test/clj/cortex/compute/cpu/tensor_test.clj:17-119)
CASES = [
    (assign_constant, ALL_DTYPES), (assign_marshal, ALL_DTYPES), (unary_op, ALL_DTYPES), (channel_op, ALL_DTYPES),
    (binary_constant_op, ALL_DTYPES), (binary_op, ALL_DTYPES), (gemm, FLOAT_DTYPES), (gemv, FLOAT_DTYPES),
    (ternary_op_select, ALL_DTYPES), (batch_normalize, FLOAT_DTYPES), (pooling_operator, FLOAT_DTYPES),
    (batch_normalize_update_and_apply, FLOAT_DTYPES), (batch_normalize_gradients, FLOAT_DTYPES),
    (lrn_operator, FLOAT_DTYPES),
    (activation_gradient, FLOAT_DTYPES), (linear_layer_backward, FLOAT_DTYPES), (relu_layer_backward, FLOAT_DTYPES),
    (activation_forward, FLOAT_DTYPES), (softmax, FLOAT_DTYPES), (unary_reduce, ALL_DTYPES), (transpose, ALL_DTYPES),
    (mask, INT_LONG), (select, ALL_DTYPES), (select_transpose_interaction, ALL_DTYPES),
    (convolution_operator, FLOAT_DTYPES), (indexed_tensor, ALL_DTYPES), (magnitude_and_mag_squared, FLOAT_DTYPES),
    (softmax_layer, FLOAT_DTYPES), (basic_conv_layer, FLOAT_DTYPES), (adam_optimizer, FLOAT_DTYPES),
    (rand_operator, ["float"]),
]


def case_params():
    return [(fn, dt) for fn, dts in CASES for dt in dts]


def case_id(param):
    return param.__name__ if callable(param) else str(param)
