"""Edge cases of the descriptor semantics (tenferro-prims/src/lib.rs:130-245): empty extents,
rank-0 outputs, broadcast (stride 0) and reversed operands, scalars alpha = 0 / beta != 0."""
import numpy as np
import pytest

from conftest import ALL_DTYPES, TOL, Strided, random_array

pytestmark = pytest.mark.gpu


def _contract(tb, la, a, lb, b, lc, c0, alpha, beta, dtype):
    plan = tb.CudaBackend.plan(tb.PrimDescriptor.Contract(la, lb, lc), [a.dims, b.dims, c0.shape], dtype)
    out = tb.Tensor.from_numpy(c0)
    tb.CudaBackend.execute(plan, alpha, [a.to_device(tb), b.to_device(tb)], beta, out)
    return out.to_numpy()


@pytest.mark.parametrize("dtype", ALL_DTYPES)
def test_empty_contracted_mode_leaves_beta_c(tb, oracle, dtype):
    """A contracted mode of extent 0 sums nothing: C = beta * C (tenferro-prims/src/lib.rs:229)."""
    rng = np.random.default_rng(1)
    a = Strided(random_array(rng, (5, 0), dtype), rng, "col")
    b = Strided(random_array(rng, (0, 7), dtype), rng, "col")
    c0 = random_array(rng, (5, 7), dtype)
    got = _contract(tb, [0, 1], a, [1, 2], b, [0, 2], c0, 2.0, -0.5, dtype)
    assert oracle.rel_frobenius(got, -0.5 * c0) <= TOL[np.dtype(dtype)]
    got = _contract(tb, [0, 1], a, [1, 2], b, [0, 2], c0, 2.0, 0.0, dtype)
    assert np.array_equal(got, np.zeros_like(c0))


@pytest.mark.parametrize("dtype", [np.float32, np.complex128])
def test_empty_free_mode_is_a_no_op(tb, dtype):
    rng = np.random.default_rng(2)
    a = Strided(random_array(rng, (0, 6), dtype), rng, "col")
    b = Strided(random_array(rng, (6, 4), dtype), rng, "col")
    got = _contract(tb, [0, 1], a, [1, 2], b, [0, 2], np.zeros((0, 4), dtype), 1.0, 0.0, dtype)
    assert got.shape == (0, 4)
    x = tb.Tensor.from_numpy(np.zeros((3, 0, 2), dtype))
    assert x.permute([2, 0, 1]).contiguous().to_numpy().shape == (2, 3, 0)


@pytest.mark.parametrize("dtype", ALL_DTYPES)
def test_rank0_outputs(tb, oracle, dtype):
    """Full contractions and full reductions produce rank-0 tensors ('ij,ij->', 'ijk->')."""
    rng = np.random.default_rng(3)
    a, b = random_array(rng, (33, 17), dtype), random_array(rng, (33, 17), dtype)
    got = tb.einsum("ij,ij->", [tb.Tensor.from_numpy(a), tb.Tensor.from_numpy(b)]).to_numpy()
    assert got.shape == ()
    assert oracle.rel_frobenius(got, oracle.np_einsum("ij,ij->", [a, b])) <= 10 * TOL[np.dtype(dtype)]
    t = random_array(rng, (9, 10, 11), dtype)
    got = tb.einsum("ijk->", [tb.Tensor.from_numpy(t)]).to_numpy()
    assert oracle.rel_frobenius(got, oracle.np_einsum("ijk->", [t])) <= 10 * TOL[np.dtype(dtype)]


@pytest.mark.parametrize("dtype", [np.float32, np.float64, np.complex64])
@pytest.mark.parametrize("shape", [(40, 24, 48), (300, 260, 320)])
def test_broadcast_and_reversed_operands(tb, oracle, dtype, shape):
    """A stride-0 (broadcast, tenferro-tensor/src/lib.rs:508-509) operand and a reversed one go
    through the same contraction; whichever kernel takes them, the numbers are the oracle's."""
    m, n, k = shape
    rng = np.random.default_rng(m + n)
    row = random_array(rng, (1, k), dtype)
    a_dev = tb.Tensor.from_numpy(row).broadcast([m, k])          # every row the same, stride 0
    b = random_array(rng, (k, n), dtype)
    b_rev = Strided(b, rng, "random")                              # random order, pads, flips, offset
    plan = tb.CudaBackend.plan(tb.PrimDescriptor.Contract([0, 1], [1, 2], [0, 2]), [(m, k), (k, n), (m, n)], dtype)
    out = tb.Tensor.zeros((m, n), dtype=dtype)
    tb.CudaBackend.execute(plan, 1.0, [a_dev, b_rev.to_device(tb)], 0.0, out)
    want = oracle.np_contract([0, 1], np.broadcast_to(row, (m, k)), [1, 2], b, [0, 2])
    assert oracle.rel_frobenius(out.to_numpy(), want) <= TOL[np.dtype(dtype)]


@pytest.mark.parametrize("dtype", ALL_DTYPES)
def test_alpha_zero_keeps_only_beta_c(tb, oracle, dtype):
    rng = np.random.default_rng(5)
    a = Strided(random_array(rng, (64, 48), dtype), rng, "col")
    b = Strided(random_array(rng, (48, 72), dtype), rng, "col")
    c0 = random_array(rng, (64, 72), dtype)
    got = _contract(tb, [0, 1], a, [1, 2], b, [0, 2], c0, 0.0, 3.0, dtype)
    assert oracle.rel_frobenius(got, 3.0 * c0) <= TOL[np.dtype(dtype)]


def test_writes_stay_inside_the_output_view(tb, oracle):
    """A padded, offset output view: the tensor-core epilogues touch exactly the view's elements."""
    rng = np.random.default_rng(6)
    for dtype, shape in ((np.float32, (300, 280, 96)), (np.complex64, (150, 140, 64)), (np.complex128, (70, 90, 40))):
        m, n, k = shape
        a, b = random_array(rng, (m, k), dtype), random_array(rng, (k, n), dtype)
        c = Strided(np.zeros((m, n), dtype), rng, "random")
        plan = tb.CudaBackend.plan(tb.PrimDescriptor.Contract([0, 1], [1, 2], [0, 2]), [(m, k), (k, n), (m, n)], dtype)
        out = c.to_device(tb)
        tb.CudaBackend.execute(plan, 1.0, [tb.Tensor.from_numpy(a), tb.Tensor.from_numpy(b)], 0.0, out)
        raw = c.read_back(out)
        want = oracle.np_contract([0, 1], a, [1, 2], b, [0, 2])
        it = raw.dtype.itemsize
        view = np.lib.stride_tricks.as_strided(raw[c.offset:], shape=c.dims, strides=[s * it for s in c.strides])
        assert oracle.rel_frobenius(view, want) <= TOL[np.dtype(dtype)]
        mask = np.ones(raw.shape, dtype=bool)
        idx = c.offset + sum(np.arange(d).reshape([-1 if i == ax else 1 for i in range(2)]) * s
                             for ax, (d, s) in enumerate(zip(c.dims, c.strides)))
        mask[idx.reshape(-1)] = False
        sentinel = c.buf[mask]
        assert np.array_equal(raw[mask], sentinel), dtype
