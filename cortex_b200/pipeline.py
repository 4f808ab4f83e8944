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

    host_in  : pinned Buffer [rows, in_width]   (allocate with driver.allocate_host_buffer)
    host_out : pinned Buffer [rows, out_width]
    Two device input slots and two output slots ping-pong so that the upload of
    chunk i+1 and the download of chunk i-1 overlap the compute of chunk i.
    """

    def __init__(self, device, net, in_width, out_width, chunk_rows, datatype="float"):
        self.device, self.net = device, net
        self.in_width, self.out_width, self.chunk_rows, self.datatype = in_width, out_width, chunk_rows, datatype
        self.compute = device.create_stream()
        self.upload = [device.create_stream(), device.create_stream()]
        self.download = device.create_stream()
        self.in_slots = [device.allocate_device_buffer(chunk_rows * in_width, datatype) for _ in range(2)]
        self.out_slots = [device.allocate_device_buffer(chunk_rows * out_width, datatype) for _ in range(2)]
        self._slot_free = [None, None]     # event: compute finished reading in_slot[i]
        self._out_free = [None, None]      # event: download finished reading out_slot[i]

    def run(self, host_in, host_out, rows, wait=True):
        """Returns (h2d_bytes, d2h_bytes).  With wait=True blocks until every result is in host_out;
        with wait=False returns once everything is enqueued (call drain() before reading host_out), so
        that consecutive batches overlap: the first upload of the next batch runs under this one's tail."""
        es = {"float": 4, "double": 8}[self.datatype]
        h2d = d2h = 0
        n_chunks = (rows + self.chunk_rows - 1) // self.chunk_rows
        last_download = None
        with ct.with_stream(self.compute), ct.with_datatype(self.datatype):
            for i in range(n_chunks):
                slot = i % 2
                r0 = i * self.chunk_rows
                nr = min(self.chunk_rows, rows - r0)
                up = self.upload[slot]
                if self._slot_free[slot] is not None:
                    up.sync_event(self._slot_free[slot])
                up.copy_host_to_device(host_in, r0 * self.in_width, self.in_slots[slot], 0, nr * self.in_width)
                uploaded = up.create_event()
                h2d += nr * self.in_width * es
                self.compute.sync_event(uploaded)
                if self._out_free[slot] is not None:
                    self.compute.sync_event(self._out_free[slot])
                x = ct.Tensor(self.device, dims.dimensions([nr, self.in_width]), self.in_slots[slot])
                y = self.net.infer(x)
                # the network owns y; copy it into the download slot so the next chunk may overwrite it
                self.compute.copy_device_to_device(y.buffer, 0, self.out_slots[slot], 0, nr * self.out_width)
                computed = self.compute.create_event()
                self._slot_free[slot] = computed
                self.download.sync_event(computed)
                self.download.copy_device_to_host(self.out_slots[slot], 0, host_out, r0 * self.out_width,
                                                  nr * self.out_width)
                self._out_free[slot] = self.download.create_event()
                last_download = self._out_free[slot]
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

    def release(self):
        for s in [self.compute, self.download] + self.upload:
            s.sync()
