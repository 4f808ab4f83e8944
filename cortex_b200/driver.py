"""Driver / device / stream / buffer / event objects of the B200 backend.

Host-side mirror of the reference's compute-driver protocols
(src/cortex/compute/driver.clj:46-61 PDriver, :74-84 PDevice, :87-96 PBuffer,
:180-194 PStream, :201-203 PEvent) as implemented by its CUDA backend
(src/cortex/compute/cuda/driver.clj:725-733, 849-1045).  Offsets and counts are
in ELEMENTS, as in the reference.  Every method forwards to one C-ABI call.
"""
import ctypes as C

import numpy as np

from . import _lib
from ._lib import DTYPE_CODE, DTYPE_SIZE, NUMPY_NAME, call
from .tensor_math import CTensorMath


class Buffer:
    """A typed span of device (or pinned host) memory: DevicePointer /
    PageLockedPointer of src/cortex/compute/cuda/driver.clj:489-542."""

    def __init__(self, ptr, dtype, n, device, owner=None, host=False):
        self.ptr, self.dtype, self.n, self.device = int(ptr), dtype, int(n), device
        self._owner, self.host = owner, host
        self._released = False

    def ecount(self):
        return self.n

    def get_datatype(self):
        return self.dtype

    def nbytes(self):
        return self.n * DTYPE_SIZE[self.dtype]

    # PBuffer
    def sub_buffer(self, offset, length):
        """drv/sub-buffer (driver.clj:206-214): a view that shares the backing store."""
        offset, length = int(offset), int(length)
        if offset < 0 or length > self.n - offset:
            raise ValueError("Sub buffer out of range.")
        return Buffer(self.ptr + offset * DTYPE_SIZE[self.dtype], self.dtype, length, self.device,
                      owner=self._owner or self, host=self.host)

    def alias(self, other):
        return self.ptr == other.ptr

    def partially_alias(self, other):
        a0, a1 = self.ptr, self.ptr + self.nbytes()
        b0, b1 = other.ptr, other.ptr + other.nbytes()
        return (b0 <= a0 < b1) or (a0 <= b0 < a1)

    def as_numpy(self):
        """Host buffers only: a numpy view of the pinned memory."""
        if not self.host:
            raise TypeError("device memory cannot be viewed from the host; copy it first")
        raw = (C.c_char * self.nbytes()).from_address(self.ptr)
        return np.frombuffer(raw, dtype=NUMPY_NAME[self.dtype], count=self.n)

    def ipc_export(self):
        """64-byte CUDA IPC handle of this device allocation (whole cb200_malloc'ed buffers only)."""
        if self.host or self._owner is not None:
            raise TypeError("only whole device allocations can be exported")
        raw = C.create_string_buffer(64)
        call("cb200_ipc_export", self.device.index, self.ptr, raw)
        return raw.raw

    def release(self):
        if self._owner is not None or self._released:
            return
        self._released = True
        if self.host:
            call("cb200_host_free", self.ptr)
        else:
            call("cb200_free", self.device.index, self.ptr)

    def __del__(self):
        try:
            self.release()
        except Exception:
            pass


class B200Event:
    def __init__(self, handle):
        self.handle = handle

    def wait_for_event(self):
        call("cb200_event_wait", self.handle)

    def elapsed_ms_since(self, start):
        ms = C.c_float()
        call("cb200_event_elapsed_ms", start.handle, self.handle, C.byref(ms))
        return ms.value

    def release(self):
        if self.handle:
            call("cb200_event_destroy", self.handle)
            self.handle = None

    def __del__(self):
        try:
            self.release()
        except Exception:
            pass


class B200Graph:
    """A captured launch sequence (B200Stream.begin_capture / end_capture), replayed with launch()."""

    def __init__(self, handle):
        self.handle = handle

    def launch(self, stream):
        call("cb200_graph_launch", self.handle, stream.handle)

    def release(self):
        if self.handle:
            call("cb200_graph_destroy", self.handle)
            self.handle = None

    def __del__(self):
        try:
            self.release()
        except Exception:
            pass


class B200Stream(CTensorMath):
    """CudaStream of the reference + its TensorMath implementation
    (extend-type CudaStream, src/cortex/compute/cuda/tensor_math.clj:289)."""

    def __init__(self, device):
        self.device = device
        h = C.c_void_p()
        call("cb200_stream_create", device.index, C.byref(h))
        self.handle = h.value

    # --- TensorMath plumbing ---------------------------------------------------
    def _tm(self, name, *args):
        return call("cb200_" + name, self.handle, *args)

    def get_device(self):
        return self.device

    def get_driver(self):
        return self.device.driver

    # --- launch-sequence capture -----------------------------------------------
    def begin_capture(self):
        call("cb200_graph_capture_begin", self.handle)

    def end_capture(self):
        h = C.c_void_p()
        call("cb200_graph_capture_end", self.handle, C.byref(h))
        return B200Graph(h.value)

    # --- PStream ------------------------------------------------------------------
    def copy_host_to_device(self, host_buffer, host_offset, device_buffer, device_offset, elem_count):
        es = DTYPE_SIZE[device_buffer.dtype]
        if host_buffer.dtype != device_buffer.dtype:
            raise TypeError("host and device buffer datatypes differ")
        call("cb200_memcpy_h2d", self.handle, device_buffer.ptr + device_offset * es,
             host_buffer.ptr + host_offset * es, elem_count * es)

    def copy_device_to_host(self, device_buffer, device_offset, host_buffer, host_offset, elem_count):
        es = DTYPE_SIZE[device_buffer.dtype]
        if host_buffer.dtype != device_buffer.dtype:
            raise TypeError("host and device buffer datatypes differ")
        call("cb200_memcpy_d2h", self.handle, host_buffer.ptr + host_offset * es,
             device_buffer.ptr + device_offset * es, elem_count * es)

    def copy_device_to_device(self, src, src_offset, dst, dst_offset, elem_count):
        es = DTYPE_SIZE[src.dtype]
        if src.dtype != dst.dtype:
            raise TypeError("device->device copies do not marshal datatypes")
        call("cb200_memcpy_d2d", self.handle, dst.ptr + dst_offset * es, src.ptr + src_offset * es, elem_count * es)

    def memset(self, device_buffer, device_offset, elem_val, elem_count):
        call("cb200_memset", self.handle, DTYPE_CODE[device_buffer.dtype], device_buffer.ptr, int(device_offset),
             float(elem_val), int(elem_count))

    def create_event(self, timing=False):
        h = C.c_void_p()
        call("cb200_event_record", self.handle, 1 if timing else 0, C.byref(h))
        return B200Event(h.value)

    def sync_event(self, event):
        call("cb200_stream_wait_event", self.handle, event.handle)

    def sync(self):
        """drv/sync-stream (driver.clj:217-221); also raises on a device-side status."""
        call("cb200_stream_sync", self.handle)

    def native_handle(self):
        return _lib.load().cb200_stream_native(self.handle)

    def set_option(self, name, value):
        """A per-stream routing / diagnostic option (cb200_stream_set_option): see _lib.STREAM_OPTIONS."""
        call("cb200_stream_set_option", self.handle, _lib.STREAM_OPTIONS[name], int(value))

    def workspace_info(self):
        b, r, g = C.c_size_t(), C.c_int(), C.c_int()
        call("cb200_stream_workspace_info", self.handle, C.byref(b), C.byref(r), C.byref(g))
        return {"bytes": b.value, "retired-blocks": r.value, "live-graphs": g.value}

    def launch_count(self):
        return int(_lib.load().cb200_launch_count(self.handle))

    def release(self):
        if self.handle:
            call("cb200_stream_destroy", self.handle)
            self.handle = None

    def __del__(self):
        try:
            self.release()
        except Exception:
            pass


class B200Device:
    def __init__(self, driver, index):
        self.driver, self.index = driver, index
        name = C.create_string_buffer(256)
        sm, major, minor = C.c_int(), C.c_int(), C.c_int()
        call("cb200_device_info", index, name, 256, C.byref(sm), C.byref(major), C.byref(minor))
        self.name, self.sm_count = name.value.decode(), sm.value
        self.compute_capability = (major.value, minor.value)

    def memory_info(self):
        f, t = C.c_size_t(), C.c_size_t()
        call("cb200_mem_info", self.index, C.byref(f), C.byref(t))
        return {"free": f.value, "total": t.value}

    def create_stream(self):
        return B200Stream(self)

    def allocate_device_buffer(self, elem_count, elem_type):
        p = C.c_void_p()
        call("cb200_malloc", self.index, int(elem_count) * DTYPE_SIZE[elem_type], C.byref(p))
        return Buffer(p.value, elem_type, elem_count, self)

    def enable_peer(self, peer):
        """Let kernels on this device address `peer`'s memory (one process, several GPUs)."""
        call("cb200_peer_enable", self.index, peer.index)

    def ipc_import(self, handle, elem_count, elem_type):
        """Map another process's exported allocation into this device's address space.  The
        returned buffer is a borrowed view: close it with ipc_close(), never release()."""
        p = C.c_void_p()
        call("cb200_ipc_import", self.index, bytes(handle), C.byref(p))
        buf = Buffer(p.value, elem_type, elem_count, self, owner=self)
        return buf

    def ipc_close(self, buffer):
        call("cb200_ipc_close", self.index, buffer.ptr)

    def get_device(self):
        return self

    def get_driver(self):
        return self.driver


class B200Driver:
    """`(driver)` of the reference CUDA backend (cuda/driver.clj:1157-1163)."""

    def __init__(self):
        _lib.load()
        self._devices = None

    def get_devices(self):
        if self._devices is None:
            n = C.c_int()
            call("cb200_device_count", C.byref(n))
            self._devices = [B200Device(self, i) for i in range(n.value)]
        return self._devices

    def default_device(self):
        devs = self.get_devices()
        if not devs:
            raise _lib.B200Error(3, "no CUDA device is visible")
        return devs[0]

    def allocate_host_buffer(self, elem_count, elem_type, usage_type="one-time", near=None):
        """Page-locked host memory.  `near` (a device) places it on the NUMA node of that GPU's PCIe slot;
        the buffer's `numa_node` attribute then says which (-1: unknown / not bound)."""
        if usage_type not in ("one-time", "reusable"):
            raise ValueError("Usage type is not in expected set")
        p = C.c_void_p()
        node = C.c_int(-1)
        if near is not None:
            call("cb200_host_alloc_near", near.index, int(elem_count) * DTYPE_SIZE[elem_type], C.byref(p), C.byref(node))
        else:
            call("cb200_host_alloc", int(elem_count) * DTYPE_SIZE[elem_type], C.byref(p))
        buf = Buffer(p.value, elem_type, elem_count, None, host=True)
        buf.numa_node = node.value
        return buf


_driver = None


def driver():
    global _driver
    if _driver is None:
        _driver = B200Driver()
    return _driver
