"""Shared test plumbing: import paths, the `gpu` marker, and helpers that place the same
strided host buffer on the device and in front of the CPU oracle."""
from __future__ import annotations

import sys
from pathlib import Path

import numpy as np
import pytest

ROOT = Path(__file__).resolve().parents[1]
sys.path.insert(0, str(ROOT / "tenferro-rs_b200"))
sys.path.insert(0, str(ROOT))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


@pytest.fixture(scope="session")
def tb():
    import tenferro_b200

    return tenferro_b200


@pytest.fixture(scope="session")
def ctx(tb):
    """The context of cuda:0.  GPU tests must fail - not skip - when it cannot be made."""
    return tb.Context.get(0)


@pytest.fixture(scope="session")
def oracle():
    from oracle import oracle as o

    o.build_c_oracle()
    return o


class Strided:
    """A random strided layout of a logical array: the same flat buffer is uploaded to the
    device (as a tenferro_b200.Tensor) and handed to the oracle (as an oracle.StridedBuf)."""

    def __init__(self, logical: np.ndarray, rng: np.random.Generator, layout: str = "random", conj: bool = False):
        self.logical = np.asarray(logical)
        dims = self.logical.shape
        nd = len(dims)
        if layout == "col":
            order, pad, flips, offset = list(range(nd)), [0] * nd, [False] * nd, 0
        elif layout == "row":
            order, pad, flips, offset = list(range(nd - 1, -1, -1)), [0] * nd, [False] * nd, 0
        else:
            order = list(rng.permutation(nd))
            pad = [int(rng.integers(0, 3)) for _ in range(nd)]
            flips = [bool(rng.integers(0, 2)) and layout == "random" for _ in range(nd)]
            offset = int(rng.integers(0, 5))
        strides = [0] * nd
        acc = 1
        for ax in order:
            strides[ax] = acc
            acc *= dims[ax] + pad[ax]
        total = acc + offset + 4
        for ax in range(nd):
            if flips[ax] and dims[ax] > 0:
                offset += (dims[ax] - 1) * strides[ax]
                strides[ax] = -strides[ax]
        # Fill the gaps with a sentinel so that stray reads and writes show up.
        if self.logical.dtype.kind == "c":
            self.buf = np.full(total, 777.0 + 555.0j, dtype=self.logical.dtype)
        else:
            self.buf = np.full(total, 777.0, dtype=self.logical.dtype)
        self.dims, self.strides, self.offset, self.conj = tuple(dims), tuple(strides), offset, conj
        stored = np.conj(self.logical) if conj else self.logical
        self.host_view()[...] = stored

    def host_view(self) -> np.ndarray:
        it = self.buf.dtype.itemsize
        return np.lib.stride_tricks.as_strided(self.buf[self.offset:], shape=self.dims,
                                               strides=[s * it for s in self.strides])

    def to_device(self, tb):
        from tenferro_b200.tensor import _Block
        import ctypes as C

        ctx = tb.Context.get(0)
        block = _Block(ctx, self.buf.nbytes)
        ctx.h2d(block.ptr, self.buf.ctypes.data_as(C.c_void_p), self.buf.nbytes)
        ctx.synchronize()
        return tb.Tensor(block, self.dims, self.strides, self.offset, self.buf.dtype,
                         tb.LogicalMemorySpace.GpuMemory(0), conj=self.conj)

    def to_oracle(self, oracle):
        return oracle.StridedBuf(self.buf.copy(), self.dims, self.strides, self.offset, self.conj)

    def read_back(self, tensor) -> np.ndarray:
        """Whole device buffer (gaps included) as a flat host array."""
        import ctypes as C

        ctx = tensor.ctx
        ctx.synchronize()
        raw = np.empty_like(self.buf)
        ctx.d2h(raw.ctypes.data_as(C.c_void_p), tensor._block.ptr, raw.nbytes)
        ctx.synchronize()
        return raw


def random_array(rng: np.random.Generator, shape, dtype) -> np.ndarray:
    dtype = np.dtype(dtype)
    if dtype.kind == "c":
        real = np.float32 if dtype == np.complex64 else np.float64
        return (rng.standard_normal(shape).astype(real) + 1j * rng.standard_normal(shape).astype(real)).astype(dtype)
    return rng.standard_normal(shape).astype(dtype)


TOL = {np.dtype("float32"): 1e-5, np.dtype("complex64"): 1e-5, np.dtype("float64"): 1e-12,
       np.dtype("complex128"): 1e-12}
ALL_DTYPES = [np.float32, np.float64, np.complex64, np.complex128]
