"""Driver-level behaviour of the B200 backend through the C ABI: the reference's own driver
golden, its many-threads x many-streams usage model, a bounded device-side wait that is made
to run out, and replay of a captured launch sequence after the stream's workspace has grown."""
import threading

import numpy as np
import pytest

import parity_cases as pc
from cortex_b200 import _lib
from cortex_b200 import nn
from cortex_b200 import tensor as ct

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("datatype", ["byte", "short", "int", "long", "float", "double"])
def test_simple_stream(b200_driver, datatype):
    """src/cortex/compute/verify/driver.clj:11-30 -- host buffer -> device, offset memset of 5 elements
    at offset 5, device -> host, per datatype (the reference stamps it out with def-all-dtype-test)."""
    stream = b200_driver.default_device().create_stream()
    buf_a = b200_driver.allocate_host_buffer(10, datatype)
    output_buf_a = b200_driver.allocate_host_buffer(10, datatype)
    buf_b = b200_driver.default_device().allocate_device_buffer(10, datatype)
    buf_a.as_numpy()[:] = np.arange(10)
    buf_a.as_numpy()[0] = 100
    stream.copy_host_to_device(buf_a, 0, buf_b, 0, 10)
    stream.memset(buf_b, 5, 20.0, 5)
    stream.copy_device_to_host(buf_b, 0, output_buf_a, 0, 10)
    stream.sync()
    assert [100.0, 1.0, 2.0, 3.0, 4.0, 20.0, 20.0, 20.0, 20.0, 20.0] == [float(v) for v in output_buf_a.as_numpy()]


def test_eight_threads_eight_streams_one_result(b200_driver):
    """The reference's usage model (src/cortex/verify/nn/train.clj:156-167, 211-236): several host threads,
    each with its own stream on the one device, run the same network on the same data at once and must all
    get the same answer.  Config 1's MLP, 8 threads x 8 streams, 20 forward passes each, both as the
    reference's call sequence and fused; weights are shared, every thread owns its activations."""
    dev = b200_driver.default_device()
    rng = np.random.default_rng(101)
    x = rng.random((128, 784)).astype(np.float32)
    w1 = (rng.standard_normal((500, 784)) * np.sqrt(2.0 / 784)).astype(np.float32)
    w2 = (rng.standard_normal((10, 500)) * np.sqrt(2.0 / 500)).astype(np.float32)
    b1 = (rng.standard_normal(500) * 0.1).astype(np.float32)
    b2 = (rng.standard_normal(10) * 0.1).astype(np.float32)
    setup = dev.create_stream()
    with ct.with_stream(setup), ct.with_datatype("float"):
        shared = [ct.to_tensor(a) for a in (w1, b1, w2, b2)]
    setup.sync()
    results, errors = {}, []
    start = threading.Barrier(8)

    def worker(i):
        try:
            stream = dev.create_stream()
            with ct.with_stream(stream), ct.with_datatype("float"):
                assert ct.check_stream() is stream
                tw1, tb1, tw2, tb2 = shared
                net = nn.MLP([(tw1, tb1, "relu"), (tw2, tb2, "softmax")], fused=(i % 2 == 1))
                xt = ct.to_tensor(x)
                start.wait()
                outs = [ct.to_array(net.infer(xt)).reshape(128, 10).copy() for _ in range(20)]
            stream.sync()
            results[i] = outs
        except Exception as exc:      # surfaced below, in the main thread
            errors.append((i, repr(exc)))
            try:
                start.abort()
            except Exception:
                pass

    threads = [threading.Thread(target=worker, args=(i,)) for i in range(8)]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    assert not errors, errors
    assert len(results) == 8
    for family in (0, 1):     # unfused threads agree bit for bit with each other, fused ones likewise
        outs = [o for i in range(family, 8, 2) for o in results[i]]
        assert all(np.array_equal(outs[0], o) for o in outs[1:])
    exact = np.maximum(x.astype(np.float64) @ w1.T.astype(np.float64) + b1, 0) @ w2.T.astype(np.float64) + b2
    exact = np.exp(exact - exact.max(axis=1, keepdims=True))
    exact /= exact.sum(axis=1, keepdims=True)
    assert pc.rel_err(results[0][0], exact) <= 1e-4 and pc.rel_err(results[1][0], exact) <= 1e-4


@pytest.mark.parametrize("route", ["general", "presplit-single", "presplit-pair"])
def test_bounded_wait_runs_out_and_the_stream_recovers(b200_driver, route):
    """Every device-side wait of the tensor-core GEMMs is bounded.  Here the host withholds the producers'
    loads (a per-stream option: the full barriers are never armed) and shortens the limit to ~1e6 cycles,
    so the consumers' waits run out: the kernel must unwind through its abort path (TMEM freed, no trap),
    cb200_stream_sync must report CB200_ERR_TIMEOUT, and the next launch on the same stream must be clean."""
    M, N, K = 512, 512, 256
    rng = np.random.default_rng(9)
    A = rng.standard_normal((M, K)).astype(np.float32)
    W = rng.standard_normal((N, K)).astype(np.float32)
    stream = b200_driver.default_device().create_stream()
    if route != "general":
        stream.set_option("presplit-variant", 1 if route == "presplit-single" else 2)
    with ct.with_stream(stream), ct.with_datatype("float"):
        a, w, c = ct.to_tensor(A), ct.to_tensor(W), ct.new_tensor([M, N])
        a_lo, w_lo = ct.new_tensor([M, K]), ct.new_tensor([N, K])
        stream.split_lo(a_lo.buffer, a.buffer, M * K)
        stream.split_lo(w_lo.buffer, w.buffer, N * K)

        def launch():
            if route == "general":
                ct.gemm(c, False, True, 1.0, a, w, 0.0)
            else:
                stream.gemm_bias_act_presplit(c.buffer, None, N, 1.0, a.buffer, a_lo.buffer, M, K, K, w.buffer,
                                              w_lo.buffer, N, K, 0.0, None, None)

        launch()
        stream.sync()                                   # the healthy path first
        good = ct.to_array(c).reshape(M, N).copy()
        stream.set_option("wait-limit-cycles", 1000000)
        stream.set_option("inject-fault", 1)
        launch()
        with pytest.raises(_lib.B200Error) as err:
            stream.sync()
        assert err.value.code == 4, str(err.value)      # CB200_ERR_TIMEOUT
        stream.set_option("inject-fault", 0)
        stream.set_option("wait-limit-cycles", 0)
        stream.sync()                                   # status word was cleared by the failing sync
        ct.assign(c, 0.0)
        launch()
        stream.sync()
        again = ct.to_array(c).reshape(M, N)
    assert np.array_equal(good, again)
    assert pc.rel_err(good, A.astype(np.float64) @ W.astype(np.float64).T) <= 1e-4


def test_graph_replay_survives_workspace_growth(b200_driver):
    """A captured forward pass holds the stream's workspace address as a kernel argument.  When a later
    call needs a larger workspace the old block must stay alive while the graph does: the replay after
    the growth reads and writes valid memory and gives the same bits as before.  Growing DURING a
    capture is refused."""
    stream = b200_driver.default_device().create_stream()
    rng = np.random.default_rng(3)
    with ct.with_stream(stream), ct.with_datatype("double"):
        # a convolution in fp64 unrolls its input into the stream's workspace
        desc = ct.convolution_descriptor("double", 6, 3, 3, 3, 1, 1, 1, 1)
        x = ct.to_tensor(rng.standard_normal((2, 3, 8, 8)))
        w = ct.to_tensor(rng.standard_normal((6, 27)))
        out = ct.new_tensor([2, 6, 8, 8])
        ct.convolution_forward(out, 0.0, x, w, None, desc, None)          # first use sizes the workspace
        direct = ct.to_array(out).copy()
        stream.begin_capture()
        ct.convolution_forward(out, 0.0, x, w, None, desc, None)
        graph = stream.end_capture()
        before = stream.workspace_info()
        assert before["live-graphs"] == 1 and before["retired-blocks"] == 0
        # a much larger problem on the same stream: the workspace has to grow
        xb = ct.to_tensor(rng.standard_normal((8, 16, 32, 32)))
        wb = ct.to_tensor(rng.standard_normal((8, 144)))
        outb = ct.new_tensor([8, 8, 32, 32])
        descb = ct.convolution_descriptor("double", 8, 16, 3, 3, 1, 1, 1, 1)
        ct.convolution_forward(outb, 0.0, xb, wb, None, descb, None)
        after = stream.workspace_info()
        assert after["bytes"] > before["bytes"] and after["retired-blocks"] == 1
        ct.assign(out, 0.0)
        graph.launch(stream)
        stream.sync()
        assert np.array_equal(ct.to_array(out), direct)
        # growth while capturing is refused (nothing may be allocated inside a capture)
        xc = ct.to_tensor(rng.standard_normal((16, 16, 48, 48)))
        outc = ct.new_tensor([16, 8, 48, 48])
        stream.begin_capture()
        try:
            with pytest.raises(_lib.B200Error) as err:
                ct.convolution_forward(outc, 0.0, xc, wb, None, descb, None)
            assert err.value.code == 1 and "capturing" in str(err.value)
        finally:
            stream.end_capture().release()
        graph.release()
        assert stream.workspace_info()["live-graphs"] == 0
    stream.sync()
