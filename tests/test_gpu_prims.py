"""Parity of every PrimDescriptor variant on the GPU, through the C ABI, against the CPU
oracle on the same seeded strided buffers.  Bit-exact for Permute and the diagonal
embeddings; relative Frobenius error <= 1e-5 (f32, Complex32) / 1e-12 (f64, Complex64) for
everything that sums."""
from pathlib import Path

import numpy as np
import pytest

from conftest import ALL_DTYPES, TOL, Strided, random_array
from lowering import lower

pytestmark = pytest.mark.gpu
GOLDEN = Path(__file__).resolve().parent / "golden"


def run_desc(tb, oracle, desc, ins, out, alpha, beta, dtype, force=None):
    """Execute on the device and in the C oracle; return (device logical result, device raw
    buffer, oracle StridedBuf)."""
    shapes = [s.dims for s in ins] + [out.dims]
    plan = tb.CudaBackend.plan(desc, shapes, dtype)
    if force is not None:
        plan.force_kernel(force)
    d_ins = [s.to_device(tb) for s in ins]
    d_out = out.to_device(tb)
    tb.CudaBackend.execute(plan, alpha, d_ins, beta, d_out)
    raw = out.read_back(d_out)
    low = lower(desc)
    if low is None:
        r = len(out.dims)
        low = ([list(range(r)), list(range(r))], list(range(r)))
    o_out = out.to_oracle(oracle)
    oracle.c_execute(low[0], [s.to_oracle(oracle) for s in ins], low[1], o_out, alpha, beta, int(desc.op))
    return d_out.to_numpy(), raw, o_out, plan


def assert_gaps_untouched(raw, o_out):
    """Device and oracle buffers agree outside the view too (nothing strays)."""
    idx = np.lib.stride_tricks.as_strided(np.arange(o_out.buf.size)[o_out.offset:], shape=o_out.dims,
                                          strides=[s * 8 for s in o_out.strides])
    mask = np.ones(o_out.buf.shape, dtype=bool)
    mask[idx.reshape(-1)] = False
    assert np.array_equal(raw[mask], o_out.buf[mask])


@pytest.mark.parametrize("dtype", ALL_DTYPES)
def test_contract_random_layouts(tb, oracle, dtype):
    rng = np.random.default_rng(101)
    P = tb.PrimDescriptor
    for trial in range(12):
        m, n, k, b = (int(x) for x in rng.integers(1, 40, size=4))
        b = b % 4 + 1
        a = Strided(random_array(rng, (b, m, k), dtype), rng, conj=bool(trial % 2))
        bb = Strided(random_array(rng, (k, b, n), dtype), rng, conj=bool(trial % 3 == 0))
        c = Strided(random_array(rng, (n, m, b), dtype), rng)
        alpha, beta = [(1.0, 0.0), (0.5, -1.0), (-1.0, 1.0), (2.0, 0.5)][trial % 4]
        if np.dtype(dtype).kind == "c" and trial % 4 == 1:
            alpha, beta = 0.5 - 0.25j, 1.5j
        desc = P.Contract([0, 1, 2], [2, 0, 3], [3, 1, 0])
        got, raw, o_out, plan = run_desc(tb, oracle, desc, [a, bb], c, alpha, beta, dtype)
        want = oracle.np_contract([0, 1, 2], a.logical, [2, 0, 3], bb.logical, [3, 1, 0], alpha, beta, c.logical)
        assert oracle.rel_frobenius(got, want) <= TOL[np.dtype(dtype)], (trial, plan.kernel_name)
        assert oracle.rel_frobenius(got, o_out.view()) <= TOL[np.dtype(dtype)]
        assert_gaps_untouched(raw, o_out)


@pytest.mark.parametrize("dtype", [np.float64, np.complex128])
@pytest.mark.parametrize("shape", [(64, 64, 4096), (130, 70, 33), (512, 512, 1024), (1, 1, 5000), (257, 3, 64),
                                   (8, 300, 17)])
def test_contract_fp64_pipe_vs_simt(tb, oracle, dtype, shape):
    """The DMMA kernel (with its split ranges and fix-up pass) against the SIMT kernel and the
    NumPy truth, on shapes that cut tiles in every way."""
    m, n, k = shape
    rng = np.random.default_rng(m * 7 + n * 3 + k)
    a = random_array(rng, (m, k), dtype)
    b = random_array(rng, (k, n), dtype)
    want = oracle.np_contract([0, 1], a, [1, 2], b, [0, 2])
    P = tb.PrimDescriptor
    res = {}
    for layout in ("col", "row"):
        sa, sb = Strided(a, rng, layout), Strided(b, rng, layout)
        for kern in (tb.ContractKernel.Dmma, tb.ContractKernel.Simt):
            plan = tb.CudaBackend.plan(P.Contract([0, 1], [1, 2], [0, 2]), [a.shape, b.shape, (m, n)], dtype)
            plan.force_kernel(kern)
            out = tb.Tensor.zeros((m, n), dtype=dtype)
            tb.CudaBackend.execute(plan, 1.0, [sa.to_device(tb), sb.to_device(tb)], 0.0, out)
            got = out.to_numpy()
            assert plan.kernel_name == ("dmma_f64" if kern == tb.ContractKernel.Dmma else "simt")
            assert oracle.rel_frobenius(got, want) <= 1e-12, (layout, kern)
            res[(layout, kern)] = got
    # Same kernel, same inputs, twice: bitwise reproducible.
    plan = tb.CudaBackend.plan(P.Contract([0, 1], [1, 2], [0, 2]), [a.shape, b.shape, (m, n)], dtype)
    ta, tb_ = tb.Tensor.from_numpy(a), tb.Tensor.from_numpy(b)
    outs = []
    for _ in range(2):
        out = tb.Tensor.zeros((m, n), dtype=dtype)
        tb.CudaBackend.execute(plan, 1.0, [ta, tb_], 0.0, out)
        outs.append(out.to_numpy())
    assert np.array_equal(outs[0], outs[1])


@pytest.mark.parametrize("dtype", ALL_DTYPES)
def test_batched_gemm(tb, oracle, dtype):
    rng = np.random.default_rng(5)
    P = tb.PrimDescriptor
    for batch in ([], [3], [2, 3]):
        m, n, k = 17, 9, 23
        a = Strided(random_array(rng, (*batch, m, k), dtype), rng)
        b = Strided(random_array(rng, (*batch, k, n), dtype), rng)
        c = Strided(random_array(rng, (*batch, m, n), dtype), rng)
        got, raw, o_out, _ = run_desc(tb, oracle, P.BatchedGemm(batch, m, n, k), [a, b], c, 1.0, 1.0, dtype)
        want = oracle.np_batched_gemm(a.logical, b.logical, 1.0, 1.0, c.logical)
        assert oracle.rel_frobenius(got, want) <= TOL[np.dtype(dtype)]
        assert oracle.rel_frobenius(got, o_out.view()) <= TOL[np.dtype(dtype)]


@pytest.mark.parametrize("dtype", ALL_DTYPES)
def test_permute_bit_exact(tb, oracle, dtype):
    rng = np.random.default_rng(9)
    P = tb.PrimDescriptor
    cases = [((5, 7), [1, 0]), ((70, 130), [1, 0]), ((33, 5, 65), [2, 0, 1]), ((4, 5, 6, 7), [3, 2, 1, 0]),
             ((16, 3, 64), [0, 2, 1]), ((1, 9), [1, 0]), ((0, 4), [1, 0]), ((128, 2, 96), [2, 1, 0])]
    for shape, perm in cases:
        for layout in ("col", "row", "random"):
            a = Strided(random_array(rng, shape, dtype), rng, layout)
            out_shape = tuple(shape[p] for p in perm)
            c = Strided(random_array(rng, out_shape, dtype), rng, layout)
            modes = list(range(len(shape)))
            desc = P.Permute(modes, [modes[p] for p in perm])
            got, raw, o_out, _ = run_desc(tb, oracle, desc, [a], c, 1.0, 0.0, dtype)
            want = np.transpose(a.logical, perm)
            assert got.tobytes() == np.asfortranarray(want).tobytes(order="F") or np.array_equal(got, want)
            assert np.array_equal(raw.view(np.uint8), o_out.buf.view(np.uint8))  # every byte, gaps included


@pytest.mark.parametrize("dtype", ALL_DTYPES)
def test_permute_alpha_beta_conj(tb, oracle, dtype):
    rng = np.random.default_rng(10)
    P = tb.PrimDescriptor
    a = Strided(random_array(rng, (12, 40, 3), dtype), rng, conj=True)
    c = Strided(random_array(rng, (3, 12, 40), dtype), rng)
    got, raw, o_out, _ = run_desc(tb, oracle, P.Permute([0, 1, 2], [2, 0, 1]), [a], c, 0.5, 2.0, dtype)
    want = oracle.np_permute([0, 1, 2], a.logical, [2, 0, 1], 0.5, 2.0, c.logical)
    assert oracle.rel_frobenius(got, want) <= TOL[np.dtype(dtype)]
    assert oracle.rel_frobenius(got, o_out.view()) <= TOL[np.dtype(dtype)]


@pytest.mark.parametrize("dtype", ALL_DTYPES)
def test_reduce(tb, oracle, dtype):
    rng = np.random.default_rng(12)
    P = tb.PrimDescriptor
    ops = [tb.ReduceOp.Sum] if np.dtype(dtype).kind == "c" else [tb.ReduceOp.Sum, tb.ReduceOp.Max, tb.ReduceOp.Min]
    cases = [((6, 5, 4), [2, 0]), ((300, 40), [1]), ((300, 40), [0]), ((7, 9, 11), []), ((2000,), []),
             ((3, 1, 5), [0, 2]), ((64, 3000), [0])]
    for shape, kept in cases:
        for op in ops:
            for layout in ("col", "random"):
                a = Strided(random_array(rng, shape, dtype), rng, layout)
                out_shape = tuple(shape[m] for m in kept)
                c = Strided(random_array(rng, out_shape, dtype), rng, layout)
                modes = list(range(len(shape)))
                alpha, beta = (1.0, 0.0) if op != tb.ReduceOp.Sum else (0.5, 1.0)
                got, raw, o_out, _ = run_desc(tb, oracle, P.Reduce(modes, kept, op), [a], c, alpha, beta, dtype)
                want = oracle.np_reduce(modes, a.logical, kept, int(op), alpha, beta, c.logical)
                if op == tb.ReduceOp.Sum:
                    assert oracle.rel_frobenius(got, want) <= TOL[np.dtype(dtype)] * 2, (shape, kept, layout)
                else:
                    assert np.array_equal(got, want), (shape, kept, op, layout)
                    assert np.array_equal(got, np.array(o_out.view()))


@pytest.mark.parametrize("dtype", ALL_DTYPES)
def test_trace_antitrace_antidiag(tb, oracle, dtype):
    rng = np.random.default_rng(13)
    P = tb.PrimDescriptor
    tol = TOL[np.dtype(dtype)]
    a = Strided(random_array(rng, (6, 5, 6), dtype), rng)
    c = Strided(random_array(rng, (5,), dtype), rng)
    got, _, o_out, _ = run_desc(tb, oracle, P.Trace([0, 1, 2], [1], [(0, 2)]), [a], c, 1.0, 0.0, dtype)
    assert oracle.rel_frobenius(got, oracle.np_trace([0, 1, 2], a.logical, [1], [(0, 2)])) <= tol
    assert oracle.rel_frobenius(got, o_out.view()) <= tol
    # two pairs at once, full trace to a scalar
    a = Strided(random_array(rng, (4, 3, 4, 3), dtype), rng)
    c = Strided(random_array(rng, (), dtype), rng)
    got, _, _, _ = run_desc(tb, oracle, P.Trace([0, 1, 2, 3], [], [(0, 2), (1, 3)]), [a], c, 2.0, 0.5, dtype)
    want = oracle.np_trace([0, 1, 2, 3], a.logical, [], [(0, 2), (1, 3)], 2.0, 0.5, c.logical)
    assert oracle.rel_frobenius(got, want) <= tol
    # AntiTrace: gradient of the trace spread on the diagonal, off-diagonal = beta * old
    for beta in (0.0, 1.0, -0.5):
        g = Strided(random_array(rng, (5,), dtype), rng)
        c = Strided(random_array(rng, (6, 5, 6), dtype), rng)
        got, raw, o_out, _ = run_desc(tb, oracle, P.AntiTrace([1], [0, 1, 2], [(0, 2)]), [g], c, 1.0, beta, dtype)
        want = oracle.np_anti_trace([1], g.logical, [0, 1, 2], (6, 5, 6), [(0, 2)], 1.0, beta, c.logical)
        assert oracle.rel_frobenius(got, want) <= tol
        assert np.array_equal(raw, o_out.buf) or oracle.rel_frobenius(got, o_out.view()) <= tol
        d = Strided(random_array(rng, (6, 5), dtype), rng)
        c = Strided(random_array(rng, (6, 5, 6), dtype), rng)
        got, raw, o_out, _ = run_desc(tb, oracle, P.AntiDiag([0, 1], [0, 1, 2], [(0, 2)]), [d], c, 1.0, beta, dtype)
        want = oracle.np_anti_diag([0, 1], d.logical, [0, 1, 2], (6, 5, 6), [(0, 2)], 1.0, beta, c.logical)
        assert oracle.rel_frobenius(got, want) <= tol
        if beta == 0.0:
            assert np.array_equal(got, want)  # pure placement: exact


@pytest.mark.parametrize("dtype", ALL_DTYPES)
def test_elementwise_mul(tb, oracle, dtype):
    rng = np.random.default_rng(14)
    P = tb.PrimDescriptor
    a = Strided(random_array(rng, (9, 31, 4), dtype), rng)
    b = Strided(random_array(rng, (9, 31, 4), dtype), rng, conj=True)
    c = Strided(random_array(rng, (9, 31, 4), dtype), rng)
    got, raw, o_out, _ = run_desc(tb, oracle, P.ElementwiseMul(), [a, b], c, 1.0, -1.0, dtype)
    want = oracle.np_elementwise_mul(a.logical, b.logical, 1.0, -1.0, c.logical)
    assert oracle.rel_frobenius(got, want) <= TOL[np.dtype(dtype)]
    assert oracle.rel_frobenius(got, o_out.view()) <= TOL[np.dtype(dtype)]
    # broadcast operand through a stride-0 view (tenferro-tensor/src/lib.rs:506-516)
    col = tb.Tensor.from_numpy(random_array(rng, (9, 1, 4), dtype))
    full = tb.Tensor.from_numpy(a.logical)
    out = tb.Tensor.zeros((9, 31, 4), dtype=dtype)
    plan = tb.CudaBackend.plan(P.ElementwiseMul(), [(9, 31, 4)] * 3, dtype)
    tb.CudaBackend.execute(plan, 1.0, [full, col.broadcast([9, 31, 4])], 0.0, out)
    assert oracle.rel_frobenius(out.to_numpy(), a.logical * col.to_numpy()) <= TOL[np.dtype(dtype)]


@pytest.mark.parametrize("name,dtype", [("f32", np.float32), ("f64", np.float64), ("c32", np.complex64),
                                        ("c64", np.complex128)])
def test_golden_fixtures_on_gpu(tb, oracle, name, dtype):
    g = np.load(GOLDEN / "golden.npz")
    P = tb.PrimDescriptor
    tol = TOL[np.dtype(dtype)]
    T = tb.Tensor.from_numpy

    def run(desc, ins, out0, alpha=1.0, beta=0.0):
        out = T(out0)
        plan = tb.CudaBackend.plan(desc, [i.shape for i in ins] + [out0.shape], dtype)
        tb.CudaBackend.execute(plan, alpha, [T(i) for i in ins], beta, out)
        return out.to_numpy()

    got = run(P.Contract([0, 1, 2], [2, 1, 3], [3, 0]), [g[f"contract_{name}_a"], g[f"contract_{name}_b"]],
              g[f"contract_{name}_c0"], 0.5, -2.0)
    assert oracle.rel_frobenius(got, g[f"contract_{name}_out"]) <= tol
    got = run(P.BatchedGemm([4], 3, 2, 5), [g[f"bgemm_{name}_a"], g[f"bgemm_{name}_b"]], np.zeros((4, 3, 2), dtype))
    assert oracle.rel_frobenius(got, g[f"bgemm_{name}_out"]) <= tol
    got = run(P.Reduce([0, 1, 2], [2, 0], tb.ReduceOp.Sum), [g[f"reduce_{name}_a"]], np.zeros((5, 4), dtype))
    assert oracle.rel_frobenius(got, g[f"reduce_{name}_sum"]) <= tol
    got = run(P.Trace([0, 1, 2], [1], [(0, 2)]), [g[f"trace_{name}_a"]], np.zeros((3,), dtype))
    assert oracle.rel_frobenius(got, g[f"trace_{name}_out"]) <= tol
    got = run(P.Permute([0, 1, 2], [2, 0, 1]), [g[f"permute_{name}_a"]], np.zeros((5, 3, 4), dtype))
    assert np.array_equal(got, g[f"permute_{name}_out"])
    got = run(P.AntiTrace([1], [0, 1, 2], [(0, 2)]), [g[f"antitrace_{name}_a"]], np.zeros((4, 3, 4), dtype))
    assert np.array_equal(got, g[f"antitrace_{name}_out"])
    got = run(P.AntiDiag([0, 1], [0, 1, 2], [(0, 2)]), [g[f"antidiag_{name}_a"]], np.zeros((4, 3, 4), dtype))
    assert np.array_equal(got, g[f"antidiag_{name}_out"])
    got = run(P.ElementwiseMul(), [g[f"ewmul_{name}_a"], g[f"ewmul_{name}_b"]], np.zeros((3, 4), dtype))
    assert oracle.rel_frobenius(got, g[f"ewmul_{name}_out"]) <= tol


def test_execute_errors(tb):
    P = tb.PrimDescriptor
    plan = tb.CudaBackend.plan(P.Contract([0, 1], [1, 2], [0, 2]), [[3, 4], [4, 5], [3, 5]], np.float64)
    a, b = tb.Tensor.zeros([3, 4]), tb.Tensor.zeros([4, 5])
    with pytest.raises(tb.ShapeMismatch):
        tb.CudaBackend.execute(plan, 1.0, [a, b], 0.0, tb.Tensor.zeros([3, 6]))
    with pytest.raises(tb.RankMismatch):
        tb.CudaBackend.execute(plan, 1.0, [a, b], 0.0, tb.Tensor.zeros([3, 5, 1]))
    with pytest.raises(tb.InvalidArgument):
        tb.CudaBackend.execute(plan, 1.0, [a], 0.0, tb.Tensor.zeros([3, 5]))
    with pytest.raises(tb.InvalidArgument):
        tb.CudaBackend.execute(plan, 1.0, [a, b], 0.0, tb.Tensor.zeros([3, 5], dtype=np.float32))


def test_preferred_devices_and_pool(tb, ctx):
    devs = tb.preferred_compute_devices(tb.LogicalMemorySpace.GpuMemory(0), tb.OpKind.Contract)
    assert devs[0] == tb.ComputeDevice.Cuda(0)
    with pytest.raises(tb.NoCompatibleComputeDevice):
        tb.preferred_compute_devices(tb.LogicalMemorySpace.MainMemory(), tb.OpKind.Permute)
    p = ctx.alloc(1 << 20)
    reserved, used = ctx.pool_stats()
    assert used >= 1 << 20 and reserved >= used
    ctx.free(p)
    ctx.synchronize()
    assert ctx.properties()["cc"][0] >= 10
