"""Host-side mirror of `tenferro-einsum` (tenferro-einsum/src/lib.rs): `Subscripts`,
`ContractionTree` and the nine `einsum*` entry points.  Parsing, tree optimisation and the
tree walk all run in libtenferro_b200.so; intermediates never leave the device."""
from __future__ import annotations

import ctypes as C
from typing import List, Optional, Sequence, Tuple

import numpy as np

from . import _lib
from ._lib import lib
from .device import Context, InvalidArgument, NoCompatibleComputeDevice, OpKind, check
from .prims import scalar_arg
from .tensor import MemoryOrder, Tensor, check_same_space, dtype_code


def _shape_args(shapes: Sequence[Sequence[int]]):
    n = len(shapes)
    ranks = (C.c_size_t * max(n, 1))(*[len(s) for s in shapes])
    rows = [(C.c_size_t * max(len(s), 1))(*[int(x) for x in s]) for s in shapes]
    dims = (_lib.c_size_p * max(n, 1))(*[C.cast(r, _lib.c_size_p) for r in rows])
    return ranks, dims, rows


class Subscripts:
    """tenferro-einsum/src/lib.rs:239-284."""

    def __init__(self, inputs: Sequence[Sequence[int]], output: Sequence[int], _handle=None):
        """`Subscripts::new(inputs, output)` with integer labels."""
        if _handle is None:
            n = len(inputs)
            ranks = (C.c_size_t * max(n, 1))(*[len(i) for i in inputs])
            rows = [(C.c_uint32 * max(len(i), 1))(*[int(x) for x in i]) for i in inputs]
            ptrs = (_lib.c_u32_p * max(n, 1))(*[C.cast(r, _lib.c_u32_p) for r in rows])
            out = (C.c_uint32 * max(len(output), 1))(*[int(x) for x in output])
            h = C.c_void_p()
            check(lib.tfb_subscripts_new(n, ranks, ptrs, len(output), out, C.byref(h)))
            _handle = h
        self.handle = _handle
        self.inputs: List[List[int]] = []
        for i in range(lib.tfb_subscripts_n_inputs(self.handle)):
            n = lib.tfb_subscripts_input(self.handle, i, None, 0)
            buf = (C.c_uint32 * max(n, 1))()
            lib.tfb_subscripts_input(self.handle, i, buf, n)
            self.inputs.append([buf[j] for j in range(n)])
        n = lib.tfb_subscripts_output(self.handle, None, 0)
        buf = (C.c_uint32 * max(n, 1))()
        lib.tfb_subscripts_output(self.handle, buf, n)
        self.output: List[int] = [buf[j] for j in range(n)]

    @classmethod
    def new(cls, inputs, output) -> "Subscripts":
        return cls(inputs, output)

    @classmethod
    def parse(cls, notation: str) -> "Subscripts":
        """`Subscripts::parse("ij,jk->ik")`; parentheses fix the pairwise order."""
        h = C.c_void_p()
        check(lib.tfb_subscripts_parse(notation.encode(), C.byref(h)))
        return cls(None, None, _handle=h)

    @property
    def has_order(self) -> bool:
        return bool(lib.tfb_subscripts_has_order(self.handle))

    def __del__(self):
        try:
            if self.handle:
                lib.tfb_subscripts_destroy(self.handle)
                self.handle = None
        except Exception:
            pass


class ContractionTree:
    """tenferro-einsum/src/lib.rs:297-356."""

    def __init__(self, handle, subscripts: Subscripts):
        self.handle = handle
        self.subscripts = subscripts

    @classmethod
    def optimize(cls, subscripts: Subscripts, shapes: Sequence[Sequence[int]]) -> "ContractionTree":
        ranks, dims, _rows = _shape_args(shapes)
        if len(shapes) != len(subscripts.inputs):
            raise InvalidArgument(f"{len(subscripts.inputs)} operands in the subscripts, {len(shapes)} shapes")
        h = C.c_void_p()
        check(lib.tfb_tree_optimize(subscripts.handle, ranks, dims, C.byref(h)))
        return cls(h, subscripts)

    @classmethod
    def from_pairs(cls, subscripts: Subscripts, shapes, pairs: Sequence[Tuple[int, int]]) -> "ContractionTree":
        ranks, dims, _rows = _shape_args(shapes)
        if len(shapes) != len(subscripts.inputs):
            raise InvalidArgument(f"{len(subscripts.inputs)} operands in the subscripts, {len(shapes)} shapes")
        flat = (C.c_size_t * max(2 * len(pairs), 1))(*[int(x) for p in pairs for x in p])
        h = C.c_void_p()
        check(lib.tfb_tree_from_pairs(subscripts.handle, ranks, dims, len(pairs), flat, C.byref(h)))
        return cls(h, subscripts)

    @property
    def pairs(self) -> List[Tuple[int, int]]:
        n = lib.tfb_tree_n_steps(self.handle)
        buf = (C.c_size_t * max(2 * n, 1))()
        lib.tfb_tree_pairs(self.handle, buf, n)
        return [(buf[2 * i], buf[2 * i + 1]) for i in range(n)]

    @property
    def macs(self) -> float:
        return lib.tfb_tree_macs(self.handle)

    @property
    def output_dims(self) -> List[int]:
        n = lib.tfb_tree_output_dims(self.handle, None, 0)
        buf = (C.c_size_t * max(n, 1))()
        lib.tfb_tree_output_dims(self.handle, buf, n)
        return [buf[i] for i in range(n)]

    def __del__(self):
        try:
            if self.handle:
                lib.tfb_tree_destroy(self.handle)
                self.handle = None
        except Exception:
            pass


def _select_context(operands: Sequence[Tensor], output: Optional[Tensor] = None) -> Context:
    """Backend selection from the tensors' memory space and device pins
    (tenferro-einsum/src/lib.rs:16-20, 179-207)."""
    tensors = list(operands) + ([output] if output is not None else [])
    space = check_same_space(tensors)
    choice = None
    for t in tensors:
        devs = t.effective_compute_devices(OpKind.Contract)
        if choice is None:
            choice = devs
        else:
            choice = [d for d in choice if d in devs]
    cuda = [d for d in (choice or []) if d.kind == "cuda"]
    if not cuda:
        raise NoCompatibleComputeDevice(f"no compatible compute device for Contract on {space!r}")
    if cuda[0].device_id != space.space_id:
        raise NoCompatibleComputeDevice(
            f"no compatible compute device for Contract on {space!r}: {cuda[0]} was pinned, but this backend computes "
            "on the GPU that owns the memory; move the tensors with to_memory_space_async")
    return Context.get(cuda[0].device_id)


def einsum_with_plan_into(tree: ContractionTree, operands: Sequence[Tensor], alpha, beta, output: Tensor) -> None:
    """tenferro-einsum/src/lib.rs:584-621: output = alpha * einsum(operands) + beta * output."""
    ctx = _select_context(operands, output)
    dtype = output.dtype
    for t in operands:
        if t.dtype != dtype:
            raise InvalidArgument(f"operand dtype {t.dtype} differs from the output's {dtype}")
    keep: list = []
    views = (_lib.TfbView * max(len(operands), 1))(*[t.as_operand_view(keep) for t in operands])
    out_view = output.as_operand_view(keep)
    check(lib.tfb_einsum_with_plan_into(ctx.handle, tree.handle, dtype_code(dtype), len(operands), views,
                                        scalar_arg(alpha, dtype), scalar_arg(beta, dtype), C.byref(out_view)))
    output.event = ctx.record_event()


class PreparedEinsum:
    """`einsum_with_plan_into` with the argument marshalling done once: for hot loops that
    repeat one contraction on the same buffers (tenferro-einsum/src/lib.rs:124-144).  `run`
    only enqueues; it records no event (use `ctx.record_event()` when one is needed)."""

    def __init__(self, tree: ContractionTree, operands: Sequence[Tensor], output: Tensor, alpha=1.0, beta=0.0):
        self.ctx = _select_context(operands, output)
        self.tree, self.operands, self.output = tree, list(operands), output
        dtype = output.dtype
        for t in operands:
            if t.dtype != dtype:
                raise InvalidArgument(f"operand dtype {t.dtype} differs from the output's {dtype}")
        self._keep: list = []
        self._views = (_lib.TfbView * max(len(operands), 1))(*[t.as_operand_view(self._keep) for t in operands])
        self._out = output.as_operand_view(self._keep)
        self._alpha, self._beta = scalar_arg(alpha, dtype), scalar_arg(beta, dtype)
        self._code = dtype_code(dtype)

    def run(self) -> None:
        check(lib.tfb_einsum_with_plan_into(self.ctx.handle, self.tree.handle, self._code, len(self.operands),
                                            self._views, self._alpha, self._beta, C.byref(self._out)))


def einsum_with_plan(tree: ContractionTree, operands: Sequence[Tensor]) -> Tensor:
    """tenferro-einsum/src/lib.rs:415-430."""
    if not operands:
        raise InvalidArgument("einsum needs at least one operand")
    out = Tensor.empty(tree.output_dims, operands[0].dtype, operands[0].logical_memory_space(),
                       MemoryOrder.ColumnMajor)
    einsum_with_plan_into(tree, operands, 1.0, 0.0, out)
    return out


def einsum_with_subscripts(subscripts: Subscripts, operands: Sequence[Tensor]) -> Tensor:
    """tenferro-einsum/src/lib.rs:400-413."""
    tree = ContractionTree.optimize(subscripts, [t.dims() for t in operands])
    return einsum_with_plan(tree, operands)


def einsum(subscripts: str, operands: Sequence[Tensor]) -> Tensor:
    """tenferro-einsum/src/lib.rs:358-398."""
    return einsum_with_subscripts(Subscripts.parse(subscripts), operands)


def einsum_with_subscripts_into(subscripts: Subscripts, operands, alpha, beta, output: Tensor) -> None:
    """tenferro-einsum/src/lib.rs:552-582."""
    tree = ContractionTree.optimize(subscripts, [t.dims() for t in operands])
    einsum_with_plan_into(tree, operands, alpha, beta, output)


def einsum_into(subscripts: str, operands, alpha, beta, output: Tensor) -> None:
    """tenferro-einsum/src/lib.rs:500-550."""
    einsum_with_subscripts_into(Subscripts.parse(subscripts), operands, alpha, beta, output)


# Consuming variants (tenferro-einsum/src/lib.rs:432-498).  Ownership passes to the call:
# the operand list is emptied so the blocks return to the pool as soon as the enqueued work
# has used them, where the next intermediate of the same size picks them up.
def einsum_with_plan_owned(tree: ContractionTree, operands: List[Tensor]) -> Tensor:
    out = einsum_with_plan(tree, operands)
    operands.clear()
    return out


def einsum_with_subscripts_owned(subscripts: Subscripts, operands: List[Tensor]) -> Tensor:
    out = einsum_with_subscripts(subscripts, operands)
    operands.clear()
    return out


def einsum_owned(subscripts: str, operands: List[Tensor]) -> Tensor:
    out = einsum(subscripts, operands)
    operands.clear()
    return out
