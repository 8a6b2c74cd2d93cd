"""CPU oracle for the tenferro contraction hot path.  TEST INFRASTRUCTURE: imported only by
tests/, by `__graft_entry__.smoke()` and by the CPU-baseline leg of bench.py - never by the
product package.

PARITY UNPINNED.  The reference ships no executable arithmetic for this path (all bodies are
`todo!()`: tenferro-prims/src/lib.rs:422-438, tenferro-einsum/src/lib.rs:393-621), its CPU
kernels are an un-vendored, un-pinned git dependency (strided-rs, tenferro-prims/Cargo.toml:12-13;
a GEMM from faer or cblas per AGENTS.md:25,102), no Rust toolchain exists on these machines and
its five runnable doctests assert no numbers.  The oracle therefore restates the DOCUMENTED
semantics twice, independently:

  * `Np*` functions below: one NumPy function per `PrimDescriptor` variant
    (tenferro-prims/src/lib.rs:152-245), written against the variant's own formula, in
    float64 / complex128;
  * `oracle.c`: plain nested loops over signed element strides with the label rules
    (batch / free / summed, repeated label = diagonal), reached through `c_execute`.

and the tests hold the two against each other, against the known answers of the reference's
doc examples (tests/golden/), and the CUDA path against both.

`ttgt_contract` is the timed CPU baseline: permute -> GEMM -> permute on OpenBLAS, the
"strided kernel + GEMM" structure AGENTS.md:102 names for the reference's CPU backend.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess
from pathlib import Path
from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np

HERE = Path(__file__).resolve().parent
SO_PATH = HERE / "build" / "liboracle.so"

DTYPE_CODE = {np.dtype("float32"): 0, np.dtype("float64"): 1, np.dtype("complex64"): 2, np.dtype("complex128"): 3}


def wide(dtype) -> np.dtype:
    """The accumulation type: float64 for real, complex128 for complex."""
    return np.dtype("complex128") if np.dtype(dtype).kind == "c" else np.dtype("float64")


# ---------------------------------------------------------------------------------------
# C oracle
# ---------------------------------------------------------------------------------------
def build_c_oracle(force: bool = False) -> Path:
    """Compile oracle.c with gcc into oracle/build/liboracle.so."""
    src = HERE / "oracle.c"
    if SO_PATH.exists() and not force and SO_PATH.stat().st_mtime >= src.stat().st_mtime:
        return SO_PATH
    SO_PATH.parent.mkdir(exist_ok=True)
    subprocess.run(["gcc", "-O2", "-std=c11", "-shared", "-fPIC", "-o", str(SO_PATH), str(src), "-lm"], check=True)
    return SO_PATH


_clib = None


def _c():
    global _clib
    if _clib is None:
        if not SO_PATH.exists():
            build_c_oracle()
        _clib = C.CDLL(str(SO_PATH))
        i64p, u32p = C.POINTER(C.c_int64), C.POINTER(C.c_uint32)
        _clib.oracle_execute.restype = C.c_int
        _clib.oracle_execute.argtypes = [
            C.c_int, C.c_int,
            C.c_int, i64p, i64p, u32p, C.c_void_p, C.c_int,
            C.c_int, i64p, i64p, u32p, C.c_void_p, C.c_int,
            C.c_int, i64p, i64p, u32p, C.c_void_p,
            C.POINTER(C.c_double), C.POINTER(C.c_double), C.c_int]
    return _clib


class StridedBuf:
    """A flat host buffer seen through dims / element strides / offset - the fields of
    `Tensor<T>` (tenferro-tensor/src/lib.rs:167-171)."""

    def __init__(self, buf: np.ndarray, dims, strides, offset=0, conj=False):
        self.buf = buf
        self.dims = tuple(int(d) for d in dims)
        self.strides = tuple(int(s) for s in strides)
        self.offset = int(offset)
        self.conj = conj

    @classmethod
    def col_major(cls, array: np.ndarray) -> "StridedBuf":
        a = np.asarray(array)
        buf = np.array(a.reshape(-1, order="F"))
        strides, acc = [], 1
        for d in a.shape:
            strides.append(acc)
            acc *= d
        return cls(buf, a.shape, strides)

    def view(self) -> np.ndarray:
        """Logical array (a NumPy view of buf; conj applied as a copy)."""
        it = self.buf.dtype.itemsize
        v = np.lib.stride_tricks.as_strided(self.buf[self.offset:], shape=self.dims,
                                            strides=[s * it for s in self.strides], writeable=True)
        return np.conj(v) if self.conj else v


def c_execute(labels_in: Sequence[Sequence[int]], inputs: Sequence[StridedBuf], labels_out: Sequence[int],
              out: StridedBuf, alpha=1.0, beta=0.0, reduce_op: int = 0) -> None:
    """Run oracle.c on host buffers; `out.buf` is updated in place."""
    lib = _c()
    dtype = out.buf.dtype
    i64 = lambda v: (C.c_int64 * max(len(v), 1))(*v)
    u32 = lambda v: (C.c_uint32 * max(len(v), 1))(*v)

    def parts(sb: Optional[StridedBuf], labels):
        if sb is None:
            return [0, i64([]), i64([]), u32([]), None, 0]
        ptr = sb.buf.ctypes.data + sb.offset * sb.buf.dtype.itemsize
        return [len(sb.dims), i64(sb.dims), i64(sb.strides), u32(list(labels)), C.c_void_p(ptr), int(sb.conj)]

    a = parts(inputs[0], labels_in[0])
    b = parts(inputs[1], labels_in[1]) if len(inputs) == 2 else parts(None, [])
    c = parts(out, labels_out)[:5]
    al = (C.c_double * 2)(complex(alpha).real, complex(alpha).imag)
    be = (C.c_double * 2)(complex(beta).real, complex(beta).imag)
    rc = lib.oracle_execute(DTYPE_CODE[np.dtype(dtype)], len(inputs), *a, *b, *c, al, be, reduce_op)
    if rc != 0:
        raise ValueError(f"oracle_execute failed with code {rc}")


# ---------------------------------------------------------------------------------------
# NumPy oracle: one function per PrimDescriptor variant.  Inputs are logical arrays; the
# result is `alpha * op(inputs) + beta * out_old`, computed in float64/complex128 and
# returned in the element type.
# ---------------------------------------------------------------------------------------
def _finish(value, alpha, beta, out_old, dtype):
    w = wide(dtype)
    res = np.asarray(alpha, dtype=w) * np.asarray(value, dtype=w)
    if beta != 0:
        res = res + np.asarray(beta, dtype=w) * np.asarray(out_old, dtype=w)
    return res.astype(dtype)


def np_contract(modes_a, a, modes_b, b, modes_c, alpha=1.0, beta=0.0, out_old=None):
    """PrimDescriptor::Contract (tenferro-prims/src/lib.rs:227-239)."""
    w = wide(a.dtype)
    val = np.einsum(a.astype(w), list(modes_a), b.astype(w), list(modes_b), list(modes_c))
    return _finish(val, alpha, beta, out_old, a.dtype)


def np_batched_gemm(a, b, alpha=1.0, beta=0.0, out_old=None):
    """PrimDescriptor::BatchedGemm (tenferro-prims/src/lib.rs:156-168): shapes
    A[batch..., m, k], B[batch..., k, n] -> C[batch..., m, n]."""
    w = wide(a.dtype)
    return _finish(np.matmul(a.astype(w), b.astype(w)), alpha, beta, out_old, a.dtype)


def np_reduce(modes_a, a, modes_c, op: int, alpha=1.0, beta=0.0, out_old=None):
    """PrimDescriptor::Reduce (tenferro-prims/src/lib.rs:170-180); op 0 sum, 1 max, 2 min."""
    w = wide(a.dtype)
    axes = tuple(i for i, m in enumerate(modes_a) if m not in modes_c)
    fn = (np.sum, np.max, np.min)[op]
    val = fn(a.astype(w), axis=axes) if axes else a.astype(w)
    left = [m for m in modes_a if m in modes_c]
    val = np.transpose(val, [left.index(m) for m in modes_c]) if left else val
    return _finish(val, alpha, beta, out_old, a.dtype)


def np_trace(modes_a, a, modes_c, paired, alpha=1.0, beta=0.0, out_old=None):
    """PrimDescriptor::Trace (tenferro-prims/src/lib.rs:182-192): for each pair (i, j) sum the
    diagonal where mode i == mode j."""
    w = wide(a.dtype)
    val = a.astype(w)
    modes = list(modes_a)
    for i, j in paired:
        ai, aj = modes.index(i), modes.index(j)
        val = np.trace(val, axis1=ai, axis2=aj)
        modes = [m for m in modes if m not in (i, j)]
    val = np.transpose(val, [modes.index(m) for m in modes_c]) if modes else val
    return _finish(val, alpha, beta, out_old, a.dtype)


def np_permute(modes_a, a, modes_b, alpha=1.0, beta=0.0, out_old=None):
    """PrimDescriptor::Permute (tenferro-prims/src/lib.rs:194-202).  alpha = 1, beta = 0 moves
    bits: the result is the transposed copy itself, no arithmetic."""
    t = np.transpose(a, [list(modes_a).index(m) for m in modes_b])
    if alpha == 1 and beta == 0:
        return np.array(t)
    return _finish(t, alpha, beta, out_old, a.dtype)


def _embed_diagonal(modes_a, a, modes_c, dims_c, paired):
    """Value tensor of shape dims_c holding `a` where every pair (i, j) has equal indices and
    zero elsewhere.  `a` may or may not carry the first label of a pair (AntiDiag / AntiTrace)."""
    w = wide(a.dtype)
    full = np.zeros(dims_c, dtype=w)
    modes_c = list(modes_c)
    it = np.ndindex(*dims_c)
    pair_pos = [(modes_c.index(i), modes_c.index(j)) for i, j in paired]
    alias = {j: i for i, j in paired}
    src_pos = []
    for m in modes_a:
        m = alias.get(m, m)
        src_pos.append(modes_c.index(m))
    aw = a.astype(w)
    for idx in it:
        if all(idx[p] == idx[q] for p, q in pair_pos):
            full[idx] = aw[tuple(idx[p] for p in src_pos)]
    return full


def np_anti_trace(modes_a, a, modes_c, dims_c, paired, alpha=1.0, beta=0.0, out_old=None):
    """PrimDescriptor::AntiTrace (tenferro-prims/src/lib.rs:204-212): the adjoint of Trace -
    the input is spread along the diagonals of the paired output modes."""
    return _finish(_embed_diagonal(modes_a, a, modes_c, dims_c, paired), alpha, beta, out_old, a.dtype)


def np_anti_diag(modes_a, a, modes_c, dims_c, paired, alpha=1.0, beta=0.0, out_old=None):
    """PrimDescriptor::AntiDiag (tenferro-prims/src/lib.rs:214-222): the adjoint of diagonal
    extraction - input element i lands at output position (i, i)."""
    return _finish(_embed_diagonal(modes_a, a, modes_c, dims_c, paired), alpha, beta, out_old, a.dtype)


def np_elementwise_mul(a, b, alpha=1.0, beta=0.0, out_old=None):
    """PrimDescriptor::ElementwiseMul (tenferro-prims/src/lib.rs:241-244)."""
    w = wide(a.dtype)
    return _finish(a.astype(w) * b.astype(w), alpha, beta, out_old, a.dtype)


# ---------------------------------------------------------------------------------------
# einsum
# ---------------------------------------------------------------------------------------
def np_semiring_contract(labels_in, operands, labels_out, algebra: int, alpha=None, beta=None, out_old=None):
    """Contraction over a tropical semiring (tenferro-algebra/src/lib.rs:74-106: zero, one, add, mul;
    MaxPlus at :81-90).  algebra 1 = MaxPlus (add = max, mul = +, zero = -inf, one = 0), 2 = MinPlus.
        out = alpha (x) (+)_{labels not in the output} (x)_t operands[t]   (+)   beta (x) out_old
    evaluated by broadcasting every operand to the full index space (small cases only)."""
    red = np.max if algebra == 1 else np.min
    pick = np.maximum if algebra == 1 else np.minimum
    zero = -np.inf if algebra == 1 else np.inf
    all_labels = list(labels_out) + sorted({l for ls in labels_in for l in ls} - set(labels_out))
    ext = {}
    for ls, op in zip(labels_in, operands):
        for l, e in zip(ls, op.shape):
            ext[l] = e
    total = np.zeros([ext[l] for l in all_labels], dtype=np.float64)
    for ls, op in zip(labels_in, operands):
        # diagonal of repeated labels first, then broadcast into the full space
        uniq = []
        for l in ls:
            if l not in uniq:
                uniq.append(l)
        sub = np.einsum(op.astype(np.float64), list(ls), uniq)
        shape = [ext[l] if l in uniq else 1 for l in all_labels]
        total = total + np.transpose(sub, [uniq.index(l) for l in all_labels if l in uniq]).reshape(shape)
    n_out = len(labels_out)
    value = red(total.reshape(total.shape[:n_out] + (-1,)), axis=-1) if total.ndim > n_out else total
    if alpha is not None:
        value = value + alpha
    if beta is not None and beta != zero and out_old is not None:
        value = pick(value, out_old.astype(np.float64) + beta)
    return value


def parse_notation(notation: str) -> Tuple[List[List[int]], List[int]]:
    """Labels of "ij,(jk,kl)->il" with a-z -> 0..25, A-Z -> 26..51
    (tenferro-einsum/src/lib.rs:260-283).  Parentheses only order the work, so they drop out."""
    s = notation.replace(" ", "").replace("(", "").replace(")", "")
    lhs, rhs = s.split("->")
    code = lambda ch: ord(ch) - ord("a") if ch.islower() else 26 + ord(ch) - ord("A")
    return [[code(ch) for ch in term] for term in lhs.split(",")], [code(ch) for ch in rhs]


def np_einsum(notation_or_labels, operands: Sequence[np.ndarray], alpha=1.0, beta=0.0, out_old=None,
              dtype=None):
    """Whole einsum in float64/complex128 (the truth for tolerance checks).  Repeated output
    labels ("i->ii") are embedded on the diagonal (tenferro-einsum/src/lib.rs:52-63)."""
    if isinstance(notation_or_labels, str):
        ins, out = parse_notation(notation_or_labels)
    else:
        ins, out = notation_or_labels
    dtype = np.dtype(dtype or operands[0].dtype)
    w = wide(dtype)
    uniq = list(dict.fromkeys(out))
    args = []
    for op, labels in zip(operands, ins):
        args += [np.asarray(op).astype(w), list(labels)]
    simple = len(operands) >= 3 and len(uniq) == len(out) and all(len(set(l)) == len(l) for l in ins)
    if simple:
        val = _pairwise(ins, [np.asarray(op).astype(w) for op in operands], uniq)
    else:
        val = np.einsum(*args, uniq, optimize=True)
    if len(uniq) != len(out):
        ext = {l: val.shape[i] for i, l in enumerate(uniq)}
        full = np.zeros([ext[l] for l in out], dtype=w)
        for idx in np.ndindex(*val.shape):
            full[tuple(idx[uniq.index(l)] for l in out)] = val[idx]
        val = full
    return _finish(val, alpha, beta, out_old, dtype)


def _pairwise(ins, ops, out):
    """N-ary contraction as a greedy sequence of pairwise permute + GEMM steps (smallest
    intermediate first).  numpy's own einsum leaves BLAS for some complex networks and then
    needs minutes where this needs milliseconds; same sums, different order."""
    ins, ops = [list(l) for l in ins], list(ops)
    while len(ops) > 1:
        best = None
        for x in range(len(ops)):
            for y in range(x + 1, len(ops)):
                others = set(out)
                for z in range(len(ops)):
                    if z != x and z != y:
                        others |= set(ins[z])
                keep = [l for l in dict.fromkeys(ins[x] + ins[y]) if l in others]
                ext = {l: ops[x].shape[i] for i, l in enumerate(ins[x])}
                ext.update({l: ops[y].shape[i] for i, l in enumerate(ins[y])})
                size = int(np.prod([ext[l] for l in keep], dtype=np.int64)) if keep else 1
                shared = bool(set(ins[x]) & set(ins[y]))
                key = (not shared, size)
                if best is None or key < best[0]:
                    best = (key, x, y, keep)
        _, x, y, keep = best
        only_x = [l for l in ins[x] if l not in keep and l not in ins[y]]
        only_y = [l for l in ins[y] if l not in keep and l not in ins[x]]
        a, la = ops[x], ins[x]
        b, lb = ops[y], ins[y]
        if only_x:
            a = a.sum(axis=tuple(la.index(l) for l in only_x))
            la = [l for l in la if l not in only_x]
        if only_y:
            b = b.sum(axis=tuple(lb.index(l) for l in only_y))
            lb = [l for l in lb if l not in only_y]
        val = ttgt_contract(la, a, lb, b, keep)
        for z in sorted((x, y), reverse=True):
            del ops[z], ins[z]
        ops.append(val)
        ins.append(keep)
    return np.transpose(ops[0], [ins[0].index(l) for l in out])


def tree_macs(inputs: Sequence[Sequence[int]], output: Sequence[int], extents: Dict[int, int],
              pairs: Sequence[Tuple[int, int]]) -> float:
    """Multiply-adds of a pairwise order, intermediates numbered from len(inputs)
    (tenferro-einsum/src/lib.rs:320-344)."""
    live = {i: list(dict.fromkeys(l)) for i, l in enumerate(inputs)}
    nxt, total = len(inputs), 0.0
    for x, y in pairs:
        lx, ly = live.pop(x), live.pop(y)
        union = list(dict.fromkeys(lx + ly))
        total += float(np.prod([extents[l] for l in union], dtype=np.float64))
        needed = set(output)
        for labels in live.values():
            needed |= set(labels)
        live[nxt] = [l for l in union if l in needed]
        nxt += 1
    return total


def best_macs(inputs, output, extents) -> float:
    """Exhaustive minimum of tree_macs over all pairwise orders (small operand counts only)."""
    n = len(inputs)

    def rec(live: Dict[int, List[int]], nxt: int) -> float:
        if len(live) == 1:
            return 0.0
        best = float("inf")
        ids = sorted(live)
        for i in range(len(ids)):
            for j in range(i + 1, len(ids)):
                x, y = ids[i], ids[j]
                rest = {k: v for k, v in live.items() if k not in (x, y)}
                union = list(dict.fromkeys(live[x] + live[y]))
                cost = float(np.prod([extents[l] for l in union], dtype=np.float64))
                needed = set(output)
                for labels in rest.values():
                    needed |= set(labels)
                rest[nxt] = [l for l in union if l in needed]
                best = min(best, cost + rec(rest, nxt + 1))
        return best

    return rec({i: list(dict.fromkeys(l)) for i, l in enumerate(inputs)}, n)


# ---------------------------------------------------------------------------------------
# Timed CPU baseline: TTGT on OpenBLAS
# ---------------------------------------------------------------------------------------
def ttgt_contract(modes_a, a, modes_b, b, modes_c):
    """Transpose-Transpose-GEMM-Transpose in the operands' own precision: the structure of a
    'strided kernel + GEMM' CPU backend (AGENTS.md:102)."""
    la, lb, lc = list(modes_a), list(modes_b), list(modes_c)
    batch = [l for l in lc if l in la and l in lb]
    m = [l for l in la if l in lc and l not in lb]
    n = [l for l in lb if l in lc and l not in la]
    k = [l for l in la if l in lb and l not in lc]
    ext = {l: a.shape[i] for i, l in enumerate(la)}
    ext.update({l: b.shape[i] for i, l in enumerate(lb)})
    size = lambda ls: int(np.prod([ext[l] for l in ls], dtype=np.int64)) if ls else 1
    a2 = np.transpose(a, [la.index(l) for l in batch + m + k]).reshape(size(batch), size(m), size(k))
    b2 = np.transpose(b, [lb.index(l) for l in batch + k + n]).reshape(size(batch), size(k), size(n))
    c2 = np.matmul(a2, b2).reshape([ext[l] for l in batch + m + n])
    order = batch + m + n
    return np.transpose(c2, [order.index(l) for l in lc])


def rel_frobenius(got: np.ndarray, want: np.ndarray) -> float:
    """|got - want|_F / |want|_F in float64/complex128."""
    w = wide(want.dtype)
    d = np.linalg.norm((np.asarray(got).astype(w) - np.asarray(want).astype(w)).reshape(-1))
    n = np.linalg.norm(np.asarray(want).astype(w).reshape(-1))
    return float(d / n) if n > 0 else float(d)


# ---------------------------------------------------------------------------------------
# Seeded inputs of the five benchmark configurations (seed = 1000 * config + tensor index)
# ---------------------------------------------------------------------------------------
def normal(seed: int, shape, dtype, scale: float = 1.0) -> np.ndarray:
    rng = np.random.default_rng(seed)
    dtype = np.dtype(dtype)
    if dtype.kind == "c":
        real = np.float32 if dtype == np.complex64 else np.float64
        out = np.empty(shape, dtype=dtype, order="F")
        out.real = rng.standard_normal(shape).astype(real) * scale
        out.imag = rng.standard_normal(shape).astype(real) * scale
        return out
    return np.asfortranarray((rng.standard_normal(shape) * scale).astype(dtype))


def uniform(seed: int, shape, dtype) -> np.ndarray:
    rng = np.random.default_rng(seed)
    return np.asfortranarray(rng.uniform(-1.0, 1.0, shape).astype(dtype))


def grouped_table(seed: int, n_problems: int) -> np.ndarray:
    """(n, 3) table of (i, j, k) drawn uniformly from {16, 32, 64, 128}."""
    rng = np.random.default_rng(seed)
    return rng.choice(np.array([16, 32, 64, 128]), size=(n_problems, 3))
