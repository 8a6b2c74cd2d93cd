"""Host-side mirror of `tenferro-device` (tenferro-device/src/lib.rs): memory spaces,
compute devices, op kinds, device preference and the error enum, plus the per-device
context that owns the stream and the stream-ordered pool."""
from __future__ import annotations

import ctypes as C
import enum
import threading
from dataclasses import dataclass
from typing import List, Optional

from . import _lib
from ._lib import lib


# ---------------------------------------------------------------- errors
class Error(Exception):
    """tenferro_device::Error (tenferro-device/src/lib.rs:109-159)."""


class ShapeMismatch(Error):
    pass


class RankMismatch(Error):
    pass


class DeviceError(Error):
    pass


class NoCompatibleComputeDevice(Error):
    pass


class CrossMemorySpaceOperation(Error):
    pass


class InvalidArgument(Error):
    pass


class Strided(Error):
    pass


_STATUS = {
    1: ShapeMismatch,
    2: RankMismatch,
    3: DeviceError,
    4: NoCompatibleComputeDevice,
    5: CrossMemorySpaceOperation,
    6: InvalidArgument,
    7: Strided,
}


def check(status: int) -> None:
    """Turn a tfb_status into the matching Error variant."""
    if status != 0:
        raise _STATUS.get(status, Error)(_lib.last_error())


# ---------------------------------------------------------------- enums
@dataclass(frozen=True)
class LogicalMemorySpace:
    """tenferro-device/src/lib.rs:30-38.  `space_id is None` means MainMemory."""

    space_id: Optional[int] = None

    @staticmethod
    def MainMemory() -> "LogicalMemorySpace":
        return LogicalMemorySpace(None)

    @staticmethod
    def GpuMemory(space_id: int) -> "LogicalMemorySpace":
        return LogicalMemorySpace(int(space_id))

    @property
    def is_gpu(self) -> bool:
        return self.space_id is not None

    def __repr__(self) -> str:
        return "MainMemory" if self.space_id is None else f"GpuMemory {{ space_id: {self.space_id} }}"


@dataclass(frozen=True)
class ComputeDevice:
    """tenferro-device/src/lib.rs:46-72; `str()` gives "cpu:0" / "cuda:1" / "hip:2"."""

    kind: str
    device_id: int

    @staticmethod
    def Cpu(device_id: int = 0) -> "ComputeDevice":
        return ComputeDevice("cpu", device_id)

    @staticmethod
    def Cuda(device_id: int) -> "ComputeDevice":
        return ComputeDevice("cuda", device_id)

    @staticmethod
    def Hip(device_id: int) -> "ComputeDevice":
        return ComputeDevice("hip", device_id)

    def __str__(self) -> str:
        kind = {"cpu": 0, "cuda": 1, "hip": 2}[self.kind]
        buf = C.create_string_buffer(64)
        lib.tfb_compute_device_format(_lib.TfbComputeDevice(kind, self.device_id), buf, 64)
        return buf.value.decode()


class OpKind(enum.IntEnum):
    """tenferro-device/src/lib.rs:77-90."""

    Contract = 0
    BatchedGemm = 1
    Reduce = 2
    Trace = 3
    Permute = 4
    ElementwiseMul = 5


def preferred_compute_devices(space: LogicalMemorySpace, op_kind: OpKind) -> List[ComputeDevice]:
    """tenferro-device/src/lib.rs:92-105."""
    out = (_lib.TfbComputeDevice * 16)()
    n = C.c_size_t(0)
    kind = 1 if space.is_gpu else 0
    check(lib.tfb_preferred_compute_devices(kind, space.space_id or 0, int(op_kind), out, 16, C.byref(n)))
    names = {0: "cpu", 1: "cuda", 2: "hip"}
    return [ComputeDevice(names[out[i].kind], out[i].device_id) for i in range(min(n.value, 16))]


# ---------------------------------------------------------------- context
class Context:
    """One per CUDA device: stream + stream-ordered pool (tfb_ctx)."""

    _lock = threading.Lock()
    _by_device = {}

    def __init__(self, device_id: int):
        h = C.c_void_p()
        check(lib.tfb_ctx_create(device_id, C.byref(h)))
        self.handle = h
        self.device_id = device_id

    @classmethod
    def get(cls, device_id: int = 0) -> "Context":
        with cls._lock:
            ctx = cls._by_device.get(device_id)
            if ctx is None:
                ctx = cls(device_id)
                cls._by_device[device_id] = ctx
            return ctx

    # -- memory
    def alloc(self, nbytes: int) -> int:
        p = C.c_void_p()
        check(lib.tfb_alloc(self.handle, nbytes, C.byref(p)))
        return p.value or 0

    def free(self, ptr: int) -> None:
        if ptr:
            check(lib.tfb_free(self.handle, C.c_void_p(ptr)))

    def h2d(self, dst: int, src, nbytes: int) -> None:
        check(lib.tfb_memcpy_h2d_async(self.handle, C.c_void_p(dst), src, nbytes))

    def d2h(self, dst, src: int, nbytes: int) -> None:
        check(lib.tfb_memcpy_d2h_async(self.handle, dst, C.c_void_p(src), nbytes))

    def h2d_2d(self, dst: int, dst_pitch: int, src, src_pitch: int, width: int, height: int) -> None:
        """`height` rows of `width` bytes from (pinned) host memory, rows `*_pitch` bytes apart."""
        check(lib.tfb_memcpy_h2d_2d_async(self.handle, C.c_void_p(dst), dst_pitch, src, src_pitch, width, height))

    def d2h_2d(self, dst, dst_pitch: int, src: int, src_pitch: int, width: int, height: int) -> None:
        check(lib.tfb_memcpy_d2h_2d_async(self.handle, dst, dst_pitch, C.c_void_p(src), src_pitch, width, height))

    def d2d(self, dst: int, src: int, nbytes: int) -> None:
        check(lib.tfb_memcpy_d2d_async(self.handle, C.c_void_p(dst), C.c_void_p(src), nbytes))

    def memset(self, dst: int, value: int, nbytes: int) -> None:
        check(lib.tfb_memset_async(self.handle, C.c_void_p(dst), value, nbytes))

    @staticmethod
    def host_alloc(nbytes: int) -> int:
        """Page-locked host memory (for asynchronous transfers)."""
        p = C.c_void_p()
        check(lib.tfb_host_alloc(nbytes, C.byref(p)))
        return p.value or 0

    @staticmethod
    def host_free(ptr: int) -> None:
        check(lib.tfb_host_free(C.c_void_p(ptr)))

    def pool_stats(self):
        r, u = C.c_size_t(), C.c_size_t()
        check(lib.tfb_pool_stats(self.handle, C.byref(r), C.byref(u)))
        return r.value, u.value

    # -- stream
    def synchronize(self) -> None:
        check(lib.tfb_ctx_synchronize(self.handle))

    @property
    def stream(self) -> int:
        s = C.c_void_p()
        check(lib.tfb_ctx_stream(self.handle, C.byref(s)))
        return s.value or 0

    def set_stream(self, stream: Optional[int]) -> None:
        """Enqueue on a caller-owned stream from now on.  The new stream first waits for what is
        already enqueued: a context is one in-order queue.  Overlap needs a second `Context`."""
        check(lib.tfb_ctx_set_stream(self.handle, C.c_void_p(stream or 0)))

    def properties(self):
        sm, mem, major, minor = C.c_int(), C.c_size_t(), C.c_int(), C.c_int()
        check(lib.tfb_ctx_properties(self.handle, C.byref(sm), C.byref(mem), C.byref(major), C.byref(minor)))
        return {"sm_count": sm.value, "total_mem": mem.value, "cc": (major.value, minor.value)}

    # -- measurement
    def profile_begin(self) -> None:
        check(lib.tfb_ctx_profile_begin(self.handle))

    def profile_read(self, kernel: str):
        """(launches, total device ms) of one kernel family since profile_begin()."""
        n, ms = C.c_size_t(), C.c_double()
        check(lib.tfb_ctx_profile_read(self.handle, kernel.encode(), C.byref(n), C.byref(ms)))
        return n.value, ms.value

    def profile_end(self) -> None:
        check(lib.tfb_ctx_profile_end(self.handle))

    def probe_fp64_tflops(self) -> float:
        v = C.c_double()
        check(lib.tfb_probe_fp64_tflops(self.handle, C.byref(v)))
        return v.value

    def probe_tf32_tflops(self) -> float:
        v = C.c_double()
        check(lib.tfb_probe_tf32_tflops(self.handle, C.byref(v)))
        return v.value

    def probe_tf32_tflops_sustained(self, seconds: float = 4.0) -> float:
        v = C.c_double()
        check(lib.tfb_probe_tf32_tflops_sustained(self.handle, float(seconds), C.byref(v)))
        return v.value

    def selftest_wait_expiry(self, polls: int = 4096) -> None:
        """Launch the kernel whose bounded wait must run out; the next synchronize() raises DeviceError."""
        check(lib.tfb_selftest_wait_expiry(self.handle, polls))

    def probe_mma_issue_cycles(self, m: int, n: int, issuers: int = 1):
        """(clocks per tcgen05.mma m x n x 8 for the issuing thread, clocks per MMA until all completed)."""
        a, b = C.c_double(), C.c_double()
        check(lib.tfb_probe_mma_issue_cycles(self.handle, m, n, issuers, C.byref(a), C.byref(b)))
        return a.value, b.value

    def probe_hbm_gbs(self) -> float:
        v = C.c_double()
        check(lib.tfb_probe_hbm_gbs(self.handle, C.byref(v)))
        return v.value

    @staticmethod
    def kernel_launch_count() -> int:
        return int(lib.tfb_kernel_launch_count())

    def capture_begin(self) -> None:
        """Calls on this context (from this thread) are recorded into a graph from here on instead of
        being enqueued; the sequence must have run once before (see tfb_ctx_capture_begin)."""
        check(lib.tfb_ctx_capture_begin(self.handle))

    def capture_end(self) -> "CapturedGraph":
        h = C.c_void_p()
        check(lib.tfb_ctx_capture_end(self.handle, C.byref(h)))
        return CapturedGraph(h, self)

    def record_event(self) -> "CompletionEvent":
        h = C.c_void_p()
        check(lib.tfb_event_record(self.handle, C.byref(h)))
        return CompletionEvent(h)

    def wait_event(self, ev: "CompletionEvent") -> None:
        check(lib.tfb_event_wait(self.handle, ev.handle))


class CapturedGraph:
    """A captured sequence of calls, replayed with `launch()` on the context's stream
    (tfb_graph_*).  The buffers the captured calls named must stay alive and in place."""

    def __init__(self, handle, ctx):
        self.handle, self.ctx = handle, ctx

    def launch(self) -> None:
        check(lib.tfb_graph_launch(self.handle))

    def __del__(self):
        try:
            if self.handle:
                lib.tfb_graph_destroy(self.handle)
                self.handle = None
        except Exception:
            pass


class CompletionEvent:
    """tenferro-tensor/src/lib.rs:301-309: tracks pending accelerator work."""

    def __init__(self, handle):
        self.handle = handle

    def synchronize(self) -> None:
        check(lib.tfb_event_synchronize(self.handle))

    def is_ready(self) -> bool:
        r = C.c_int(0)
        check(lib.tfb_event_query(self.handle, C.byref(r)))
        return bool(r.value)

    def elapsed_ms(self, later: "CompletionEvent") -> float:
        ms = C.c_float(0)
        check(lib.tfb_event_elapsed_ms(self.handle, later.handle, C.byref(ms)))
        return ms.value

    def __del__(self):
        try:
            if self.handle:
                lib.tfb_event_destroy(self.handle)
                self.handle = None
        except Exception:
            pass
