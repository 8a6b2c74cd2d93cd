"""Host-side mirror of `tenferro-tensor` with device-resident storage
(`DataBuffer::Cuda`, the variant tenferro-tensor/src/lib.rs:133-137 leaves for later).

A `Tensor` is a ref-counted device block plus dims, signed element strides and an offset
(tenferro-tensor/src/lib.rs:167-181).  View operations only rewrite that metadata
(:502-542); data operations enqueue kernels on the context's stream and hand back a tensor
that carries a `CompletionEvent` (:301-309, 677-713).
"""
from __future__ import annotations

import ctypes as C
import enum
from typing import List, Optional, Sequence, Tuple

import numpy as np

from . import _lib
from ._lib import lib
from .device import (
    ComputeDevice,
    CompletionEvent,
    Context,
    CrossMemorySpaceOperation,
    InvalidArgument,
    LogicalMemorySpace,
    NoCompatibleComputeDevice,
    OpKind,
    RankMismatch,
    ShapeMismatch,
    check,
    preferred_compute_devices,
)

DTYPES = {np.dtype("float32"): 0, np.dtype("float64"): 1, np.dtype("complex64"): 2, np.dtype("complex128"): 3}


def dtype_code(dt) -> int:
    dt = np.dtype(dt)
    if dt not in DTYPES:
        raise InvalidArgument(f"unsupported scalar type {dt}; Standard algebra covers f32, f64, Complex32, Complex64")
    return DTYPES[dt]


class MemoryOrder(enum.Enum):
    """tenferro-tensor/src/lib.rs:110-127."""

    ColumnMajor = 0
    RowMajor = 1


def contiguous_strides(dims: Sequence[int], order: MemoryOrder) -> Tuple[int, ...]:
    strides = [0] * len(dims)
    acc = 1
    idx = range(len(dims)) if order == MemoryOrder.ColumnMajor else range(len(dims) - 1, -1, -1)
    for i in idx:
        strides[i] = acc
        acc *= dims[i]
    return tuple(strides)


class _Block:
    """A device allocation shared by every view of it; returns to the pool when the last goes."""

    def __init__(self, ctx: Context, nbytes: int):
        self.ctx = ctx
        self.nbytes = nbytes
        self.ptr = ctx.alloc(nbytes)
        self.event: Optional[CompletionEvent] = None  # latest write; shared by every view of the block

    def __del__(self):
        try:
            if self.ptr:
                self.ctx.free(self.ptr)
                self.ptr = 0
        except Exception:
            pass


class _HostBlock:
    """Page-locked main memory (`LogicalMemorySpace::MainMemory`): the staging end of
    `to_memory_space_async`.  No kernel of this backend computes on it."""

    def __init__(self, nbytes: int):
        self.ctx = None
        self.nbytes = nbytes
        self.ptr = Context.host_alloc(max(nbytes, 16))
        self.event: Optional[CompletionEvent] = None

    def array(self, dtype) -> np.ndarray:
        n = self.nbytes // np.dtype(dtype).itemsize
        return np.ctypeslib.as_array((C.c_char * self.nbytes).from_address(self.ptr)).view(dtype)[:n]

    def __del__(self):
        try:
            if self.ptr:
                if self.event is not None:
                    self.event.synchronize()  # a copy may still be reading or writing the buffer
                Context.host_free(self.ptr)
                self.ptr = 0
        except Exception:
            pass


class _Borrowed:
    """Device memory owned by someone else (for example a torch tensor handed to NCCL):
    `owner` is kept alive for as long as any view of the block exists."""

    def __init__(self, ctx: Context, ptr: int, nbytes: int, owner):
        self.ctx, self.ptr, self.nbytes, self.owner = ctx, ptr, nbytes, owner
        self.event: Optional[CompletionEvent] = None


def make_view(ptr: int, dims, strides, offset: int, conj: bool, keep: list) -> _lib.TfbView:
    """Build a tfb_view; the ctypes arrays are appended to `keep` so they outlive the call."""
    n = len(dims)
    d = (C.c_size_t * max(n, 1))(*dims)
    s = (C.c_ssize_t * max(n, 1))(*strides)
    keep += [d, s]
    return _lib.TfbView(C.c_void_p(ptr), n, d, s, offset, 1 if conj else 0)


class Tensor:
    """Device tensor.  Construct with `zeros`, `ones`, `from_slice` or `from_numpy`."""

    def __init__(self, block, dims, strides, offset, dtype, space, preferred=None, event=None, conj=False):
        self._block = block
        self._dims = tuple(int(d) for d in dims)
        self._strides = tuple(int(s) for s in strides)
        self._offset = int(offset)
        self.dtype = np.dtype(dtype)
        self._space = space
        self._preferred = preferred
        self._event: Optional[CompletionEvent] = None  # used only by storage-less (metadata) tensors
        if event is not None:
            self.event = event
        self._conj = bool(conj) and self.dtype.kind == "c"

    @property
    def event(self) -> Optional[CompletionEvent]:
        """Completion of the latest write to the buffer (tenferro-tensor/src/lib.rs:301-309).  It
        lives on the storage block, so a view taken before a later write still sees that write."""
        return self._block.event if self._block is not None else self._event

    @event.setter
    def event(self, ev: Optional[CompletionEvent]) -> None:
        if self._block is not None:
            self._block.event = ev
        else:
            self._event = ev

    # ------------------------------------------------------------ constructors
    @staticmethod
    def _ctx_of(space: LogicalMemorySpace) -> Context:
        if not space.is_gpu:
            raise NoCompatibleComputeDevice(
                "no compatible compute device on MainMemory: this backend computes on GPU memory only")
        return Context.get(space.space_id)

    @classmethod
    def empty(cls, dims, dtype=np.float64, memory_space=LogicalMemorySpace.GpuMemory(0),
              order=MemoryOrder.ColumnMajor) -> "Tensor":
        n = int(np.prod(dims, dtype=np.int64)) if len(dims) else 1
        if not memory_space.is_gpu:
            block = _HostBlock(max(n, 1) * np.dtype(dtype).itemsize)
        else:
            block = _Block(cls._ctx_of(memory_space), max(n, 1) * np.dtype(dtype).itemsize)
        return cls(block, dims, contiguous_strides(dims, order), 0, dtype, memory_space)

    @classmethod
    def zeros(cls, dims, memory_space=LogicalMemorySpace.GpuMemory(0), order=MemoryOrder.ColumnMajor,
              dtype=np.float64) -> "Tensor":
        """tenferro-tensor/src/lib.rs:336."""
        t = cls.empty(dims, dtype, memory_space, order)
        if not memory_space.is_gpu:
            t._block.array(np.uint8)[:] = 0
            return t
        t._block.ctx.memset(t._block.ptr, 0, t._block.nbytes)
        t.event = t._block.ctx.record_event()
        return t

    @classmethod
    def ones(cls, dims, memory_space=LogicalMemorySpace.GpuMemory(0), order=MemoryOrder.ColumnMajor,
             dtype=np.float64) -> "Tensor":
        """tenferro-tensor/src/lib.rs:347."""
        n = int(np.prod(dims, dtype=np.int64)) if len(dims) else 1
        return cls.from_slice(np.ones(n, dtype=dtype), dims, order, memory_space)

    @classmethod
    def from_slice(cls, data, dims, order=MemoryOrder.ColumnMajor,
                   memory_space=LogicalMemorySpace.GpuMemory(0)) -> "Tensor":
        """tenferro-tensor/src/lib.rs:360: `data` is the flat buffer in `order`."""
        data = np.ascontiguousarray(data).reshape(-1)
        n = int(np.prod(dims, dtype=np.int64)) if len(dims) else 1
        if data.size != n:
            raise ShapeMismatch(f"shape mismatch: expected {list(dims)} ({n} elements), got {data.size} elements")
        if not memory_space.is_gpu:
            # MainMemory: a page-locked staging buffer; compute needs to_memory_space_async first
            block = _HostBlock(max(n, 1) * data.dtype.itemsize)
            block.array(data.dtype)[:n] = data
            return cls(block, dims, contiguous_strides(dims, order), 0, data.dtype, memory_space)
        t = cls.empty(dims, data.dtype, memory_space, order)
        ctx = t._block.ctx
        if n:
            ctx.h2d(t._block.ptr, data.ctypes.data_as(C.c_void_p), data.nbytes)
            ctx.synchronize()  # `data` may be a temporary
        return t

    @classmethod
    def from_numpy(cls, array: np.ndarray, order=MemoryOrder.ColumnMajor,
                   memory_space=LogicalMemorySpace.GpuMemory(0)) -> "Tensor":
        """Logical copy of a NumPy array (any layout) into a contiguous device tensor."""
        array = np.asarray(array)
        flat = array.reshape(-1, order="F" if order == MemoryOrder.ColumnMajor else "C")
        return cls.from_slice(flat, array.shape, order, memory_space)

    @classmethod
    def from_device_pointer(cls, ptr: int, nbytes: int, dims, dtype, memory_space, owner=None,
                            order=MemoryOrder.ColumnMajor, strides=None, offset=0) -> "Tensor":
        """View device memory allocated elsewhere (it must live in `memory_space`)."""
        block = _Borrowed(cls._ctx_of(memory_space), int(ptr), int(nbytes), owner)
        strides = contiguous_strides(dims, order) if strides is None else strides
        return cls(block, dims, strides, offset, dtype, memory_space)

    @classmethod
    def _meta(cls, dims, strides=None, offset=0, dtype=np.float64, order=MemoryOrder.ColumnMajor) -> "Tensor":
        """Metadata-only tensor (no storage): lets the view rules be exercised without a GPU."""
        strides = contiguous_strides(dims, order) if strides is None else strides
        return cls(None, dims, strides, offset, dtype, LogicalMemorySpace.GpuMemory(0))

    # ------------------------------------------------------------ metadata
    def dims(self) -> Tuple[int, ...]:
        return self._dims

    def strides(self) -> Tuple[int, ...]:
        return self._strides

    def offset(self) -> int:
        return self._offset

    def ndim(self) -> int:
        return len(self._dims)

    def len(self) -> int:
        return int(np.prod(self._dims, dtype=np.int64)) if self._dims else 1

    def __len__(self) -> int:
        return self.len()

    def is_empty(self) -> bool:
        return self.len() == 0

    def logical_memory_space(self) -> LogicalMemorySpace:
        return self._space

    def preferred_compute_device(self) -> Optional[ComputeDevice]:
        return self._preferred

    def set_preferred_compute_device(self, device: Optional[ComputeDevice]) -> None:
        self._preferred = device

    def effective_compute_devices(self, op_kind: OpKind) -> List[ComputeDevice]:
        """tenferro-tensor/src/lib.rs:420-436: the override if set, else the defaults."""
        if self._preferred is not None:
            return [self._preferred]
        return preferred_compute_devices(self._space, op_kind)

    @property
    def ctx(self) -> Context:
        return self._ctx_of(self._space)

    @property
    def is_conj(self) -> bool:
        return self._conj

    def _derive(self, dims, strides, offset=None, conj=None) -> "Tensor":
        return Tensor(self._block, dims, strides, self._offset if offset is None else offset, self.dtype,
                      self._space, self._preferred, None, self._conj if conj is None else conj)

    def as_operand_view(self, keep: list) -> _lib.TfbView:
        """Non-blocking operand view (tenferro-tensor/src/lib.rs:473-488): pending work is
        ordered by the stream, the host does not wait."""
        ptr = self._block.ptr if self._block is not None else 0
        return make_view(ptr, self._dims, self._strides, self._offset, self._conj, keep)

    # ------------------------------------------------------------ view operations (zero-copy)
    def permute(self, perm: Sequence[int]) -> "Tensor":
        """tenferro-tensor/src/lib.rs:490-504."""
        perm = [int(p) for p in perm]
        if sorted(perm) != list(range(self.ndim())):
            raise InvalidArgument(f"{perm} is not a permutation of 0..{self.ndim()}")
        return self._derive([self._dims[p] for p in perm], [self._strides[p] for p in perm])

    def broadcast(self, target_dims: Sequence[int]) -> "Tensor":
        """tenferro-tensor/src/lib.rs:506-516: size-1 axes expand with stride 0."""
        target_dims = [int(d) for d in target_dims]
        if len(target_dims) != self.ndim():
            raise RankMismatch(f"rank mismatch: expected {self.ndim()}, got {len(target_dims)}")
        strides = []
        for have, want, s in zip(self._dims, target_dims, self._strides):
            if have == want:
                strides.append(s)
            elif have == 1:
                strides.append(0)
            else:
                raise ShapeMismatch(f"shape mismatch: expected {list(self._dims)}, got {target_dims}")
        return self._derive(target_dims, strides)

    def diagonal(self, axes: Sequence[Tuple[int, int]]) -> "Tensor":
        """tenferro-tensor/src/lib.rs:518-529: each (i, j) pair collapses into one axis (at the
        position of i) whose stride is the sum of the two."""
        dims, strides = list(self._dims), list(self._strides)
        drop = set()
        for i, j in axes:
            if not (0 <= i < self.ndim() and 0 <= j < self.ndim()) or i == j or i in drop or j in drop:
                raise InvalidArgument(f"invalid axis pair ({i}, {j}) for rank {self.ndim()}")
            if dims[i] != dims[j]:
                raise ShapeMismatch(f"shape mismatch: expected [{dims[i]}], got [{dims[j]}] (diagonal axes)")
            strides[i] += strides[j]
            drop.add(j)
        keep = [a for a in range(self.ndim()) if a not in drop]
        return self._derive([dims[a] for a in keep], [strides[a] for a in keep])

    def is_contiguous(self) -> bool:
        """tenferro-tensor/src/lib.rs:598-604: dense in column- or row-major order."""
        return self._strides in (contiguous_strides(self._dims, MemoryOrder.ColumnMajor),
                                 contiguous_strides(self._dims, MemoryOrder.RowMajor)) or self.len() <= 1

    def _order(self) -> Optional[MemoryOrder]:
        if self._strides == contiguous_strides(self._dims, MemoryOrder.ColumnMajor):
            return MemoryOrder.ColumnMajor
        if self._strides == contiguous_strides(self._dims, MemoryOrder.RowMajor):
            return MemoryOrder.RowMajor
        return None

    def reshape(self, new_dims: Sequence[int]) -> "Tensor":
        """tenferro-tensor/src/lib.rs:531-542: contiguous data only, same element count."""
        new_dims = [int(d) for d in new_dims]
        n = int(np.prod(new_dims, dtype=np.int64)) if new_dims else 1
        if n != self.len():
            raise ShapeMismatch(f"shape mismatch: expected {self.len()} elements, got {new_dims}")
        order = self._order()
        if order is None:
            if self.len() <= 1:
                order = MemoryOrder.ColumnMajor
            else:
                raise InvalidArgument("reshape needs a contiguous tensor; call contiguous() first")
        return self._derive(new_dims, contiguous_strides(new_dims, order))

    # ------------------------------------------------------------ data operations
    def _copy_into_new(self, order: MemoryOrder, conj: bool) -> "Tensor":
        from .prims import CudaBackend, PrimDescriptor  # circular at import time

        out = Tensor.empty(self._dims, self.dtype, self._space, order)
        out._preferred = self._preferred
        modes = list(range(self.ndim()))
        plan = CudaBackend.plan(PrimDescriptor.Permute(modes, modes), [self._dims, self._dims], self.dtype,
                                ctx=self.ctx)
        src = self if not conj else self._derive(self._dims, self._strides, conj=not self._conj)
        CudaBackend.execute(plan, 1.0, [src], 0.0, out)
        return out

    def contiguous(self, order: MemoryOrder = MemoryOrder.ColumnMajor) -> "Tensor":
        """tenferro-tensor/src/lib.rs:544-554: a copy in `order` (a Permute plan underneath)."""
        return self._copy_into_new(order, conj=False)

    def into_contiguous(self, order: MemoryOrder = MemoryOrder.ColumnMajor) -> "Tensor":
        """tenferro-tensor/src/lib.rs:556-596: no copy when already contiguous in `order`."""
        if self._order() == order and not self._conj:
            return self
        return self._copy_into_new(order, conj=False)

    def conj(self) -> "Tensor":
        """tenferro-tensor/src/lib.rs:606-647: element-wise conjugate, layout preserved.  Real
        types come back as a plain copy."""
        if self.dtype.kind != "c":
            return self._copy_layout()
        out = self._copy_layout(conj_flip=True)
        return out

    def _copy_layout(self, conj_flip: bool = False) -> "Tensor":
        # Keep dims/strides when they are contiguous in some order; otherwise densify.
        order = self._order() or MemoryOrder.ColumnMajor
        return self._copy_into_new(order, conj=conj_flip)

    def into_conj(self) -> "Tensor":
        """tenferro-tensor/src/lib.rs:649-658: consumes self and may reuse the buffer.  Here the
        buffer is always reused: the result reads the same block through a conjugating view,
        and contraction kernels fold the sign flip into their operand loads."""
        return self._derive(self._dims, self._strides, conj=not self._conj)

    def to_memory_space_async(self, target: LogicalMemorySpace) -> "Tensor":
        """tenferro-tensor/src/lib.rs:660-671.  Same space: zero-copy (self comes back).  Main ->
        GPU and GPU -> Main copy through page-locked memory; GPU -> GPU goes over NVLink.  The
        call only enqueues; the result's event completes when the copy has landed."""
        if target == self._space:
            return self
        if not self._space.is_gpu:
            # MainMemory -> GpuMemory: host tensors are always dense (from_slice made them)
            order = self._order() or MemoryOrder.ColumnMajor
            dst = Tensor.empty(self._dims, self.dtype, target, order)
            dctx = dst.ctx
            if self.len():
                dctx.h2d(dst._block.ptr, C.c_void_p(self._block.ptr), self.len() * self.dtype.itemsize)
            dst.event = dctx.record_event()
            self._block.event = dst.event  # the staging buffer is busy until the copy has read it
            dst._conj = self._conj
            dst._keepalive = self
            return dst
        src = self if self._order() is not None else self.into_contiguous(MemoryOrder.ColumnMajor)
        order = src._order() or MemoryOrder.ColumnMajor
        nbytes = src.len() * src.dtype.itemsize
        src_ptr = src._block.ptr + src._offset * src.dtype.itemsize
        if not target.is_gpu:
            # GpuMemory -> MainMemory, on the source's stream (ordered behind its producer)
            block = _HostBlock(max(nbytes, 1))
            sctx = src.ctx
            if nbytes:
                sctx.d2h(C.c_void_p(block.ptr), src_ptr, nbytes)
            dst = Tensor(block, src._dims, contiguous_strides(src._dims, order), 0, src.dtype, target, conj=src._conj)
            dst.event = sctx.record_event()
            dst._keepalive = src
            return dst
        dst = Tensor.empty(src._dims, src.dtype, target, order)
        dctx = dst.ctx
        # the copy runs on the destination's stream: it must come after the latest write to the
        # source buffer, whichever view of it that write went through
        ev = src.event if src.event is not None else src.ctx.record_event()
        dctx.wait_event(ev)
        check(lib.tfb_memcpy_p2p_async(dctx.handle, C.c_void_p(dst._block.ptr), target.space_id,
                                       C.c_void_p(src_ptr), src._space.space_id, nbytes))
        dst.event = dctx.record_event()
        dst._conj = src._conj
        dst._keepalive = src  # the source block must outlive the copy
        return dst

    def wait(self) -> None:
        """tenferro-tensor/src/lib.rs:677-704."""
        if self.event is not None:
            self.event.synchronize()

    def is_ready(self) -> bool:
        """tenferro-tensor/src/lib.rs:706-713."""
        return self.event is None or self.event.is_ready()

    def to_numpy(self) -> np.ndarray:
        """Host copy of the logical contents (waits for pending work)."""
        if self.len() == 0:
            return np.zeros(self._dims, dtype=self.dtype)
        if not self._space.is_gpu:
            self.wait()
            raw = self._block.array(self.dtype).copy()
        else:
            ctx = self.ctx
            ctx.synchronize()
            raw = np.empty(self._block.nbytes // self.dtype.itemsize, dtype=self.dtype)
            ctx.d2h(raw.ctypes.data_as(C.c_void_p), self._block.ptr, raw.nbytes)
            ctx.synchronize()
        v = np.lib.stride_tricks.as_strided(raw[self._offset:] if self._offset >= 0 else raw, shape=self._dims,
                                            strides=[s * self.dtype.itemsize for s in self._strides])
        if self._offset < 0:
            raise InvalidArgument("negative offset")
        out = np.array(v, order="F")
        return np.conj(out) if self._conj else out

    def __repr__(self) -> str:
        return (f"Tensor(dims={list(self._dims)}, strides={list(self._strides)}, offset={self._offset}, "
                f"dtype={self.dtype}, space={self._space!r}{', conj' if self._conj else ''})")


def check_same_space(tensors: Sequence[Tensor]) -> LogicalMemorySpace:
    """Mixed spaces are an error (tenferro-device/src/lib.rs:144-150)."""
    space = tensors[0].logical_memory_space()
    for t in tensors[1:]:
        if t.logical_memory_space() != space:
            raise CrossMemorySpaceOperation(
                f"cross-memory-space operation between {space!r} and {t.logical_memory_space()!r}")
    return space
