"""Host <-> device batch pipeline around the dense-inference path.

Counterpart of the reference's `dataset->uploading-batches` / `run` loop
(src/cortex/nn/execute.clj:387-434, 475-518) and of its output download
(src/cortex/nn/compute_binding.clj:514-554): batches are staged in page-locked
host memory, uploaded on dedicated streams while the previous batch computes,
and results come back on a download stream; streams are ordered with events
only (drv/sync-streams), never with a device-wide barrier.
"""
from . import dimensions as dims
from . import tensor as ct


class BatchPipeline:
    """Runs ``net.infer`` over a host array in chunks of ``chunk_rows`` rows.

    host_in  : pinned Buffer [rows, in_width]   (driver.allocate_host_buffer, ideally near=device)
    host_out : pinned Buffer [rows, out_width]
    ``slots`` device input buffers (default 3) rotate, each with its own upload stream, so that two
    uploads can be in flight while a third chunk computes; two output buffers ping-pong between the
    compute stream and the download stream.
    """

    def __init__(self, device, net, in_width, out_width, chunk_rows, datatype="float", slots=3):
        self.device, self.net = device, net
        self.in_width, self.out_width, self.chunk_rows, self.datatype = in_width, out_width, chunk_rows, datatype
        self.slots = max(2, int(slots))
        self.compute = device.create_stream()
        self.upload = [device.create_stream() for _ in range(self.slots)]
        self.download = device.create_stream()
        self.in_slots = [device.allocate_device_buffer(chunk_rows * in_width, datatype) for _ in range(self.slots)]
        self.out_slots = [device.allocate_device_buffer(chunk_rows * out_width, datatype) for _ in range(2)]
        self._slot_free = [None] * self.slots    # event: compute finished reading in_slot[i]
        self._out_free = [None, None]            # event: download finished reading out_slot[i]
        self._next_in = 0                        # slots keep rotating across run() calls
        self._next_out = 0
        self._marks = []                         # (kind, start event, stop event, bytes) when profiling

    def run(self, host_in, host_out, rows, wait=True, profile=False):
        """Returns (h2d_bytes, d2h_bytes).  With wait=True blocks until every result is in host_out;
        with wait=False returns once everything is enqueued (call drain() before reading host_out), so
        that consecutive batches overlap: the first upload of the next batch runs under this one's tail.
        profile=True brackets every upload, chunk forward pass and download with timing events
        (read them with stats() after drain())."""
        es = {"float": 4, "double": 8}[self.datatype]
        h2d = d2h = 0
        n_chunks = (rows + self.chunk_rows - 1) // self.chunk_rows
        last_download = None
        with ct.with_stream(self.compute), ct.with_datatype(self.datatype):
            for i in range(n_chunks):
                slot, oslot = self._next_in, self._next_out
                self._next_in = (slot + 1) % self.slots
                self._next_out = 1 - oslot
                r0 = i * self.chunk_rows
                nr = min(self.chunk_rows, rows - r0)
                up = self.upload[slot]
                if self._slot_free[slot] is not None:
                    up.sync_event(self._slot_free[slot])
                m0 = up.create_event(timing=True) if profile else None
                up.copy_host_to_device(host_in, r0 * self.in_width, self.in_slots[slot], 0, nr * self.in_width)
                uploaded = up.create_event(timing=profile)
                if profile:
                    self._marks.append(("h2d", m0, uploaded, nr * self.in_width * es))
                h2d += nr * self.in_width * es
                self.compute.sync_event(uploaded)
                if self._out_free[oslot] is not None:
                    self.compute.sync_event(self._out_free[oslot])
                x = ct.Tensor(self.device, dims.dimensions([nr, self.in_width]), self.in_slots[slot])
                m0 = self.compute.create_event(timing=True) if profile else None
                y = self.net.infer(x)
                # the network owns y; copy it into the download slot so the next chunk may overwrite it
                self.compute.copy_device_to_device(y.buffer, 0, self.out_slots[oslot], 0, nr * self.out_width)
                computed = self.compute.create_event(timing=profile)
                if profile:
                    self._marks.append(("compute", m0, computed, nr))
                self._slot_free[slot] = computed
                self.download.sync_event(computed)
                m0 = self.download.create_event(timing=True) if profile else None
                self.download.copy_device_to_host(self.out_slots[oslot], 0, host_out, r0 * self.out_width,
                                                  nr * self.out_width)
                self._out_free[oslot] = self.download.create_event(timing=profile)
                if profile:
                    self._marks.append(("d2h", m0, self._out_free[oslot], nr * self.out_width * es))
                last_download = self._out_free[oslot]
                d2h += nr * self.out_width * es
        self._last_download = last_download
        if wait:
            self.drain()
        return h2d, d2h

    def drain(self):
        """Block until the results of every run() issued so far are in host memory."""
        last = getattr(self, "_last_download", None)
        if last is not None:
            last.wait_for_event()

    def stats(self):
        """Per-kind totals of the profiled copies / forward passes since the last call:
        {"h2d": {"ms": busy time, "bytes": n, "gbs": achieved rate, "count": copies}, "compute": ..., "d2h": ...}.
        A copy's time includes any wait for the PCIe link behind another copy, so `gbs` is the rate this
        stream actually got."""
        out = {}
        for kind, e0, e1, amount in self._marks:
            d = out.setdefault(kind, {"ms": 0.0, "amount": 0, "count": 0})
            d["ms"] += e1.elapsed_ms_since(e0)
            d["amount"] += amount
            d["count"] += 1
        self._marks = []
        for kind, d in out.items():
            if kind == "compute":
                d["rows"] = d.pop("amount")
                d["ms_per_chunk"] = d["ms"] / max(d["count"], 1)
            else:
                d["bytes"] = d.pop("amount")
                d["gbs"] = d["bytes"] / d["ms"] / 1e6 if d["ms"] > 0 else None
        return out

    def release(self):
        for s in [self.compute, self.download] + self.upload:
            s.sync()
