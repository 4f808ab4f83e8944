"""Optimiser steps and rand! on the B200 against the CPU oracle, through the C ABI.

Adam and Adadelta on double buffers follow the reference CPU backend's arithmetic operation for
operation, so the comparison is bit for bit; on float buffers the B200 evaluates in single precision
(as the reference's CUDA kernels do) where the CPU backend evaluates in double and rounds on store:
compared at 1e-5 relative after three steps (bound for fp32: 1e-4).  Aligned and unaligned parameter
offsets, ragged lengths.  SGD with momentum is the reference's four tensor calls (single-rounding
operations: bit for bit).  rand! is a counter-based generator: the uniform draws are bit-identical to
the oracle's restatement, the gaussian ones agree to a few ulp of the single-precision log / sin / cos."""
import numpy as np
import pytest

from cortex_b200 import optimize
from cortex_b200 import tensor as ct

pytestmark = pytest.mark.gpu
NP = {"float": np.float32, "double": np.float64}


def _run(driver, datatype, fn):
    stream = driver.default_device().create_stream()
    with ct.with_stream(stream), ct.with_datatype(datatype):
        out = fn()
    stream.sync()
    return out


def _steps(kind, datatype, n, offset, steps, seed):
    rng = np.random.default_rng(seed)
    p0 = rng.standard_normal(n).astype(NP[datatype])
    grads = [rng.standard_normal(n).astype(NP[datatype]) for _ in range(steps)]
    state0 = {"a": np.abs(rng.standard_normal(n + offset + 5)).astype(NP[datatype]) * 0.01,
              "b": np.abs(rng.standard_normal(n + offset + 5)).astype(NP[datatype]) * 0.01}

    def run():
        params = ct.to_tensor(p0)
        if kind == "adam":
            opt, state = optimize.Adam(), {"m": ct.to_tensor(state0["a"]), "v": ct.to_tensor(state0["b"])}
        elif kind == "adadelta":
            opt = optimize.Adadelta()
            state = {"grad-accum": ct.to_tensor(state0["a"]), "dx-accum": ct.to_tensor(state0["b"])}
        else:
            opt, state = optimize.SGD(learning_rate=0.01, momentum=0.9), {"momentum-vals": ct.to_tensor(state0["a"])}
        for g in grads:
            opt = opt.batch_update()
            opt.compute_parameters(state, 0.5, offset, ct.to_tensor(g), params)
        return [ct.to_array(params)] + [ct.to_array(t) for t in state.values()]

    return run


@pytest.mark.parametrize("datatype", ["float", "double"])
@pytest.mark.parametrize("kind", ["adam", "adadelta", "sgd"])
@pytest.mark.parametrize("n,offset", [(4, 0), (1000, 4), (100003, 3), (1 << 20, 0)])
def test_optimizer_steps_match_oracle(b200_driver, oracle_driver, datatype, kind, n, offset):
    run = _steps(kind, datatype, n, offset, 3, seed=n + offset)
    gpu = _run(b200_driver, datatype, run)
    cpu = _run(oracle_driver, datatype, run)
    for g, c in zip(gpu, cpu):
        if datatype == "double" or kind == "sgd":
            assert np.array_equal(g, c), (kind, datatype, n, offset, float(np.abs(g.astype(np.float64) - c).max()))
        else:
            c64 = c.astype(np.float64)
            err = np.abs(g.astype(np.float64) - c64) / np.maximum(np.abs(c64), np.sqrt(np.mean(c64 ** 2)))
            assert float(err.max()) <= 1e-5, (kind, n, offset, float(err.max()))


@pytest.mark.parametrize("n", [1, 7, 4096, 100001])
def test_rand_matches_oracle_and_replays(b200_driver, oracle_driver, n):
    def run():
        ct.seed_rand(1234)
        flat = ct.to_array(ct.rand(ct.new_tensor([n]), ct.flat_distribution(minimum=-3, maximum=5)))
        gauss = ct.to_array(ct.rand(ct.new_tensor([n]), ct.gaussian_distribution(mean=2, variance=9)))
        ct.seed_rand(1234)
        again = ct.to_array(ct.rand(ct.new_tensor([n]), ct.flat_distribution(minimum=-3, maximum=5)))
        other = ct.to_array(ct.rand(ct.new_tensor([n]), ct.flat_distribution(minimum=-3, maximum=5)))
        return flat, gauss, again, other

    g_flat, g_gauss, g_again, g_other = _run(b200_driver, "float", run)
    c_flat, c_gauss, _, _ = _run(oracle_driver, "float", run)
    assert np.array_equal(g_flat, c_flat)                       # same generator, same shaping: same bits
    assert np.array_equal(g_flat, g_again)                      # (seed, sequence) replays
    assert n < 4 or not np.array_equal(g_flat, g_other)         # the next call is a different stream
    assert g_flat.min() >= -3 and g_flat.max() <= 5
    assert np.abs(g_gauss.astype(np.float64) - c_gauss).max() <= 1e-4 * 3.0     # 3 = sqrt(variance)


def test_rand_rejects_non_float_and_bad_ranges(b200_driver):
    stream = b200_driver.default_device().create_stream()
    with ct.with_stream(stream), ct.with_datatype("double"):
        with pytest.raises(ct.TensorError):
            ct.rand(ct.new_tensor([8]), ct.gaussian_distribution())
        with pytest.raises(ct.TensorError):
            ct.flat_distribution(minimum=2, maximum=1)
    stream.sync()
