"""Host-side mirror of `tenferro-prims`: `PrimDescriptor`, `ReduceOp`, `Extension` and the
CUDA implementation of `TensorPrims<Standard>` (tenferro-prims/src/lib.rs:100-128, 152-245,
278-340).  Same names, same argument order, same error variants; the work happens in
libtenferro_b200.so."""
from __future__ import annotations

import ctypes as C
import enum
from dataclasses import dataclass, field
from typing import List, Optional, Sequence, Tuple

import numpy as np

from . import _lib
from ._lib import lib
from .device import Context, InvalidArgument, NoCompatibleComputeDevice, check
from .tensor import Tensor, check_same_space, dtype_code


class ReduceOp(enum.IntEnum):
    """tenferro-prims/src/lib.rs:100-107."""

    Sum = 0
    Max = 1
    Min = 2


class Extension(enum.IntEnum):
    """tenferro-prims/src/lib.rs:123-128."""

    Contract = 0
    ElementwiseMul = 1


class ContractKernel(enum.IntEnum):
    Auto = 0
    Simt = 1
    Dmma = 2
    Tcgen05 = 3
    Dmma4 = 4  # Complex64 with four real products per complex one: Re and Im each to their own accuracy


class Algebra(enum.IntEnum):
    """The algebra parameter A of `TensorPrims<A>` (tenferro-algebra/src/lib.rs:56, 74-106).
    Standard: (+, *).  MaxPlus: add = max, mul = +, zero = -inf, one = 0.  MinPlus: its mirror."""

    Standard = 0
    MaxPlus = 1
    MinPlus = 2


_OPS = {"BatchedGemm": 0, "Reduce": 1, "Trace": 2, "Permute": 3, "AntiTrace": 4, "AntiDiag": 5, "Contract": 6,
        "ElementwiseMul": 7}


@dataclass
class PrimDescriptor:
    """One variant of tenferro-prims' `PrimDescriptor` (src/lib.rs:152-245).  Build with the
    class methods named after the variants."""

    variant: str
    modes_a: List[int] = field(default_factory=list)
    modes_b: List[int] = field(default_factory=list)
    modes_c: List[int] = field(default_factory=list)
    paired: List[Tuple[int, int]] = field(default_factory=list)
    op: ReduceOp = ReduceOp.Sum
    batch_dims: List[int] = field(default_factory=list)
    m: int = 0
    n: int = 0
    k: int = 0

    @classmethod
    def BatchedGemm(cls, batch_dims, m, n, k):
        return cls("BatchedGemm", batch_dims=list(batch_dims), m=m, n=n, k=k)

    @classmethod
    def Reduce(cls, modes_a, modes_c, op):
        return cls("Reduce", modes_a=list(modes_a), modes_c=list(modes_c), op=ReduceOp(op))

    @classmethod
    def Trace(cls, modes_a, modes_c, paired):
        return cls("Trace", modes_a=list(modes_a), modes_c=list(modes_c), paired=[tuple(p) for p in paired])

    @classmethod
    def Permute(cls, modes_a, modes_b):
        return cls("Permute", modes_a=list(modes_a), modes_b=list(modes_b))

    @classmethod
    def AntiTrace(cls, modes_a, modes_c, paired):
        return cls("AntiTrace", modes_a=list(modes_a), modes_c=list(modes_c), paired=[tuple(p) for p in paired])

    @classmethod
    def AntiDiag(cls, modes_a, modes_c, paired):
        return cls("AntiDiag", modes_a=list(modes_a), modes_c=list(modes_c), paired=[tuple(p) for p in paired])

    @classmethod
    def Contract(cls, modes_a, modes_b, modes_c):
        return cls("Contract", modes_a=list(modes_a), modes_b=list(modes_b), modes_c=list(modes_c))

    @classmethod
    def ElementwiseMul(cls):
        return cls("ElementwiseMul")

    @property
    def n_inputs(self) -> int:
        return 2 if self.variant in ("BatchedGemm", "Contract", "ElementwiseMul") else 1

    def _to_c(self, keep: list) -> _lib.TfbDesc:
        def u32(v):
            arr = (C.c_uint32 * max(len(v), 1))(*v)
            keep.append(arr)
            return arr

        flat_pairs = [x for p in self.paired for x in p]
        bd = (C.c_size_t * max(len(self.batch_dims), 1))(*self.batch_dims)
        keep.append(bd)
        return _lib.TfbDesc(
            _OPS[self.variant], int(self.op),
            u32(self.modes_a), len(self.modes_a),
            u32(self.modes_b), len(self.modes_b),
            u32(self.modes_c), len(self.modes_c),
            u32(flat_pairs), len(self.paired),
            bd, len(self.batch_dims), self.m, self.n, self.k)


class CudaPlan:
    """`TensorPrims::Plan<T>` of the CUDA backend: an owned tfb_plan handle."""

    def __init__(self, handle, dtype, desc: PrimDescriptor, ctx: Context):
        self.handle = handle
        self.dtype = np.dtype(dtype)
        self.desc = desc
        self.ctx = ctx

    def set_algebra(self, algebra: Algebra) -> "CudaPlan":
        """Compute over another semiring: output = alpha (x) op(inputs) (+) beta (x) output."""
        check(lib.tfb_plan_set_algebra(self.handle, int(algebra)))
        return self

    def force_kernel(self, kernel: ContractKernel) -> "CudaPlan":
        check(lib.tfb_plan_force_kernel(self.handle, int(kernel)))
        return self

    @property
    def kernel_name(self) -> str:
        return lib.tfb_plan_kernel_name(self.handle).decode()

    def __del__(self):
        try:
            if self.handle:
                lib.tfb_plan_destroy(self.handle)
                self.handle = None
        except Exception:
            pass


def scalar_arg(value, dtype) -> C.Array:
    """One host scalar of `dtype` as a ctypes buffer."""
    arr = np.array([value], dtype=dtype)
    buf = (C.c_char * arr.nbytes).from_buffer_copy(arr.tobytes())
    return buf


class CudaBackend:
    """`impl TensorPrims<Standard> for CudaBackend`: associated functions only, like the
    reference's `CpuBackend` (tenferro-prims/src/lib.rs:259-262, 417-439)."""

    @staticmethod
    def plan(desc: PrimDescriptor, shapes: Sequence[Sequence[int]], dtype=np.float64,
             ctx: Optional[Context] = None, algebra: Algebra = Algebra.Standard) -> CudaPlan:
        """`plan::<T>(desc, shapes)`; shapes are inputs first, then the output.  `algebra` is the A of
        `impl TensorPrims<A> for CudaBackend`."""
        ctx = ctx or Context.get(0)
        keep: list = []
        cdesc = desc._to_c(keep)
        n = len(shapes)
        ranks = (C.c_size_t * max(n, 1))(*[len(s) for s in shapes])
        rows = [(C.c_size_t * max(len(s), 1))(*[int(x) for x in s]) for s in shapes]
        dims = (_lib.c_size_p * max(n, 1))(*[C.cast(r, _lib.c_size_p) for r in rows])
        h = C.c_void_p()
        check(lib.tfb_plan_create(ctx.handle, C.byref(cdesc), dtype_code(dtype), n, ranks, dims, C.byref(h)))
        plan = CudaPlan(h, dtype, desc, ctx)
        if algebra != Algebra.Standard:
            plan.set_algebra(algebra)
        return plan

    @staticmethod
    def execute(plan: CudaPlan, alpha, inputs: Sequence[Tensor], beta, output: Tensor) -> None:
        """`execute(plan, alpha, inputs, beta, output)`: output = alpha * op(inputs) + beta * output.
        Returns once the work is enqueued; `output.event` marks its completion."""
        tensors = list(inputs) + [output]
        for t in tensors:
            if t.dtype != plan.dtype:
                raise InvalidArgument(f"plan was made for {plan.dtype}, got a {t.dtype} tensor")
        space = check_same_space(tensors)
        if not space.is_gpu:
            raise NoCompatibleComputeDevice(
                "no compatible compute device on MainMemory: move the tensors with to_memory_space_async first")
        ctx = plan.ctx
        for t in inputs:
            if t.event is not None and t.ctx is not ctx:
                ctx.wait_event(t.event)
        keep: list = []
        views = (_lib.TfbView * max(len(inputs), 1))(*[t.as_operand_view(keep) for t in inputs])
        out_view = output.as_operand_view(keep)
        a = scalar_arg(alpha, plan.dtype)
        b = scalar_arg(beta, plan.dtype)
        check(lib.tfb_execute(plan.handle, a, len(inputs), views, b, C.byref(out_view)))
        output.event = ctx.record_event()

    @staticmethod
    def has_extension_for(dtype, ext: Extension, algebra: Algebra = Algebra.Standard) -> bool:
        """`has_extension_for::<T>(ext)` of the backend for `algebra`."""
        try:
            code = dtype_code(dtype)
        except InvalidArgument:
            return False
        return bool(lib.tfb_has_extension_for_algebra(int(algebra), code, int(ext)))


class PreparedGroupedGemm:
    """A problem table prepared once (tfb_grouped_plan_*): validated, cut into tiles and copied
    to the device at construction; `run` is then one launch.  The operand buffers the table
    points to must stay alive and in place while the object is used."""

    def __init__(self, problems, dtype, alpha=1.0, beta=0.0, ctx: Optional[Context] = None):
        self.ctx = ctx or Context.get(0)
        problems = list(problems)
        self.n = len(problems)
        arr = (_lib.TfbGemmProblem * max(self.n, 1))()
        for i, p in enumerate(problems):
            arr[i] = _lib.TfbGemmProblem(*p)
        self.alpha, self.beta = scalar_arg(alpha, dtype), scalar_arg(beta, dtype)
        self.handle = C.c_void_p()
        check(lib.tfb_grouped_plan_create(self.ctx.handle, dtype_code(dtype), self.n, arr, C.byref(self.handle)))

    def run(self) -> None:
        check(lib.tfb_grouped_plan_execute(self.handle, self.alpha, self.beta))

    def __del__(self):
        try:
            if self.handle:
                lib.tfb_grouped_plan_destroy(self.handle)
                self.handle = None
        except Exception:
            pass


def grouped_gemm(problems, dtype, alpha=1.0, beta=0.0, ctx: Optional[Context] = None) -> None:
    """Ragged batch of C_p = alpha * A_p @ B_p + beta * C_p in one persistent launch.
    `problems`: iterable of (m, n, k, a_ptr, a_rs, a_cs, b_ptr, b_rs, b_cs, c_ptr, c_rs, c_cs)."""
    ctx = ctx or Context.get(0)
    problems = list(problems)
    arr = (_lib.TfbGemmProblem * max(len(problems), 1))()
    for i, p in enumerate(problems):
        arr[i] = _lib.TfbGemmProblem(*p)
    check(lib.tfb_grouped_gemm(ctx.handle, dtype_code(dtype), len(problems), arr, scalar_arg(alpha, dtype),
                               scalar_arg(beta, dtype)))


def reduce_static(modes_a, a: Tensor, modes_c, c: Tensor, op: ReduceOp = ReduceOp.Sum, alpha=1.0, beta=0.0,
                  ctx: Optional[Context] = None) -> None:
    """`c[modes_c] = alpha * op(a[modes_a]) + beta * c` through the entry point that allocates
    nothing on the device (tfb_reduce_static): for callers that may not allocate when they call.
    Outputs above 2 MiB are rejected; calls that overlap on the GPU race on the shared scratch."""
    ctx = ctx or a.ctx
    keep: list = []
    va, vc = a.as_operand_view(keep), c.as_operand_view(keep)
    ma = (C.c_uint32 * max(len(modes_a), 1))(*[int(m) for m in modes_a])
    mc = (C.c_uint32 * max(len(modes_c), 1))(*[int(m) for m in modes_c])
    check(lib.tfb_reduce_static(ctx.handle, dtype_code(c.dtype), int(op), ma, len(modes_a), C.byref(va), mc,
                                len(modes_c), C.byref(vc), scalar_arg(alpha, c.dtype), scalar_arg(beta, c.dtype)))
    c.event = ctx.record_event()
