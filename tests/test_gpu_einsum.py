"""The einsum front end and tree executor on the GPU: the reference's doc-example forms
(known answers in tests/golden/kat.json), the five benchmark einsums, asynchronous chaining
and the device-resident Tensor operations."""
import json
from pathlib import Path

import numpy as np
import pytest

from conftest import ALL_DTYPES, TOL, random_array

pytestmark = pytest.mark.gpu
GOLDEN = Path(__file__).resolve().parent / "golden"


@pytest.fixture(scope="module")
def kat():
    return json.loads((GOLDEN / "kat.json").read_text())


@pytest.fixture(scope="module")
def golden():
    return np.load(GOLDEN / "golden.npz")


@pytest.mark.parametrize("notation", ["ij,jk->ik", "ii->", "i,j->ij", "i,i->", "ij,j->i", "i->ii", "ii->i", "i->iii",
                                      "ij->ji", "ijk->"])
@pytest.mark.parametrize("dtype", [np.float64, np.float32])
def test_doc_example_forms(tb, kat, notation, dtype):
    # tenferro-einsum/src/lib.rs:24-70
    case = kat[notation]
    ops = [tb.Tensor.from_numpy(np.array(x, dtype=dtype)) for x in case["operands"]]
    got = tb.einsum(notation, ops)
    want = np.array(case["result"], dtype=dtype)
    assert got.dims() == want.shape
    assert np.array_equal(got.to_numpy(), want)


def test_from_slice_and_views_on_device(tb, kat):
    c = kat["from_slice_2x3"]
    a = tb.Tensor.from_slice(np.array(c["data"], dtype=np.float64), c["dims"], tb.MemoryOrder.ColumnMajor)
    assert a.to_numpy().tolist() == c["logical"]
    at = a.permute([1, 0])
    assert at.to_numpy().tolist() == np.array(c["logical"]).T.tolist()
    assert not at.is_contiguous() or at.dims() == (3, 2)
    dense = at.contiguous(tb.MemoryOrder.ColumnMajor)
    assert dense.strides() == (1, 3) and np.array_equal(dense.to_numpy(), at.to_numpy())
    assert at.into_contiguous(tb.MemoryOrder.RowMajor) is at  # already row-major: no copy
    r = tb.Tensor.from_slice(np.arange(6.0), [2, 3], tb.MemoryOrder.RowMajor)
    assert r.to_numpy().tolist() == [[0, 1, 2], [3, 4, 5]]
    d = tb.Tensor.from_numpy(np.arange(16.0).reshape(4, 4)).diagonal([(0, 1)])
    assert d.to_numpy().tolist() == [0, 5, 10, 15]
    ones = tb.Tensor.ones([2, 2])
    assert ones.to_numpy().tolist() == [[1, 1], [1, 1]] and tb.Tensor.zeros([3]).to_numpy().tolist() == [0, 0, 0]


def test_conj_doc_example(tb, kat):
    c = kat["conj"]
    z = np.array([complex(*p) for p in c["operand"]])
    want = np.array([complex(*p) for p in c["result"]])
    a = tb.Tensor.from_numpy(z)
    assert np.array_equal(a.conj().to_numpy(), want)
    lazy = a.into_conj()
    assert lazy.is_conj and np.array_equal(lazy.to_numpy(), want)
    # the lazy flag is honoured by kernels: sum_i conj(z_i) * z_i = |z|^2
    dot = tb.einsum("i,i->", [lazy, a]).to_numpy()
    assert abs(dot - np.vdot(z, z)) < 1e-12
    r = tb.Tensor.from_numpy(np.array([1.0, -2.0]))
    assert np.array_equal(r.conj().to_numpy(), [1.0, -2.0])


def test_accumulate_doc_example(tb, kat):
    # tenferro-einsum/src/lib.rs:526-537
    c = kat["accumulate"]
    ops = [tb.Tensor.from_numpy(np.array(x, dtype=np.float64)) for x in c["operands"]]
    out = tb.Tensor.zeros([2, 2])
    tb.einsum_into(c["notation"], ops, 1.0, 0.0, out)
    tb.einsum_into(c["notation"], ops, c["alpha"], c["beta"], out)
    assert out.to_numpy().tolist() == c["result_after_two_calls"]


def test_batch_shape_rules(tb):
    # tenferro-einsum/src/lib.rs:75-93
    z = lambda *d: tb.Tensor.zeros(list(d))
    assert tb.einsum("bij,bjk->bik", [z(10, 3, 4), z(10, 4, 5)]).dims() == (10, 3, 5)
    assert tb.einsum("abij,abjk->abik", [z(2, 3, 4, 5), z(2, 3, 5, 6)]).dims() == (2, 3, 4, 6)
    assert tb.einsum("bij,jk->bik", [z(10, 3, 4), z(4, 5)]).dims() == (10, 3, 5)


@pytest.mark.parametrize("dtype", ALL_DTYPES)
def test_random_einsums(tb, oracle, dtype):
    rng = np.random.default_rng(21)
    cases = [
        ("bij,bjk->bik", [(5, 7, 9), (5, 9, 4)]),
        ("bij,jk->bik", [(5, 7, 9), (9, 4)]),
        ("ij,(jk,kl)->il", [(6, 7), (7, 30), (30, 5)]),
        ("ijk,jlm,kmn,lnp->ip", [(5, 6, 7), (6, 4, 3), (7, 3, 5), (4, 5, 8)]),
        ("abc,bcd->ad", [(9, 8, 7), (8, 7, 6)]),
        ("ijkl,klmn->ijmn", [(3, 4, 5, 6), (5, 6, 2, 3)]),
        ("ab,asc,bsd->cd", [(8, 8), (8, 2, 8), (8, 2, 8)]),
        ("iij,jk->ik", [(5, 5, 6), (6, 4)]),
        ("ij,kl->ijkl", [(3, 4), (5, 2)]),
        ("ijk,k->ij", [(4, 5, 6), (6,)]),
        ("ij,ij->ij", [(7, 8), (7, 8)]),
        ("ij,ij->", [(7, 8), (7, 8)]),
        ("ijx,jk->ik", [(4, 5, 3), (5, 6)]),
        ("i,j,k->kji", [(3,), (4,), (5,)]),
        ("ij,jk->kii", [(3, 4), (4, 5)]),
    ]
    for notation, shapes in cases:
        arrays = [random_array(rng, s, dtype) for s in shapes]
        got = tb.einsum(notation, [tb.Tensor.from_numpy(a) for a in arrays]).to_numpy()
        want = oracle.np_einsum(notation, arrays)
        assert got.shape == want.shape, notation
        assert oracle.rel_frobenius(got, want) <= TOL[np.dtype(dtype)], notation


def test_with_plan_and_owned_variants(tb, oracle):
    rng = np.random.default_rng(22)
    a, b, c = (random_array(rng, s, np.float64) for s in ((3, 4), (4, 100), (100, 5)))
    subs = tb.Subscripts.new([[0, 1], [1, 2], [2, 3]], [0, 3])
    tree = tb.ContractionTree.from_pairs(subs, [a.shape, b.shape, c.shape], [(1, 2), (0, 3)])
    T = tb.Tensor.from_numpy
    want = a @ b @ c
    assert oracle.rel_frobenius(tb.einsum_with_plan(tree, [T(a), T(b), T(c)]).to_numpy(), want) <= 1e-12
    assert oracle.rel_frobenius(tb.einsum_with_subscripts(subs, [T(a), T(b), T(c)]).to_numpy(), want) <= 1e-12
    ops = [T(a), T(b), T(c)]
    got = tb.einsum_with_plan_owned(tree, ops)
    assert ops == [] and oracle.rel_frobenius(got.to_numpy(), want) <= 1e-12
    out = T(np.ones((3, 5)))
    for _ in range(3):  # hot loop on a pre-allocated output (tenferro-einsum/src/lib.rs:124-144)
        tb.einsum_with_plan_into(tree, [T(a), T(b), T(c)], 1.0, 0.0, out)
    assert oracle.rel_frobenius(out.to_numpy(), want) <= 1e-12
    tb.einsum_with_subscripts_into(subs, [T(a), T(b), T(c)], 2.0, -1.0, out)
    assert oracle.rel_frobenius(out.to_numpy(), want) <= 1e-12
    with pytest.raises(tb.ShapeMismatch):
        tb.einsum_with_plan(tree, [T(a), T(b), T(np.zeros((100, 6)))])
    with pytest.raises(tb.ShapeMismatch):
        tb.einsum_with_plan_into(tree, [T(a), T(b), T(c)], 1.0, 0.0, tb.Tensor.zeros([3, 6]))


def test_async_chaining(tb, oracle):
    # tenferro-einsum/src/lib.rs:146-177: results chain on the stream without host waits
    rng = np.random.default_rng(23)
    a, b = random_array(rng, (300, 300), np.float64), random_array(rng, (300, 300), np.float64)
    ta, tb_ = tb.Tensor.from_numpy(a), tb.Tensor.from_numpy(b)
    c = tb.einsum("ij,jk->ik", [ta, tb_])
    d = tb.einsum("ij,jk->ik", [c, tb_])
    assert d.event is not None
    d.wait()
    assert d.is_ready() and c.is_ready()
    assert oracle.rel_frobenius(d.to_numpy(), a @ b @ b) <= 1e-12


def test_device_pinning_errors(tb):
    a, b = tb.Tensor.zeros([3, 4]), tb.Tensor.zeros([4, 5])
    a.set_preferred_compute_device(tb.ComputeDevice.Cuda(1))
    b.set_preferred_compute_device(tb.ComputeDevice.Cuda(1))
    with pytest.raises(tb.NoCompatibleComputeDevice):
        tb.einsum("ij,jk->ik", [a, b])
    a.set_preferred_compute_device(None)
    with pytest.raises(tb.NoCompatibleComputeDevice):
        tb.einsum("ij,jk->ik", [a, b])
    b.set_preferred_compute_device(None)
    assert tb.einsum("ij,jk->ik", [a, b]).dims() == (3, 5)


# ---------------------------------------------------------------- the benchmark einsums
def test_golden_benchmark_einsums_scaled_down(tb, oracle, golden):
    g = golden
    T = tb.Tensor.from_numpy
    got = tb.einsum("abc,bcd->ad", [T(g["cfg1_a"]), T(g["cfg1_b"])]).to_numpy()
    assert oracle.rel_frobenius(got, g["cfg1_out"]) <= 1e-12
    site = T(g["cfg2_a"])
    got = tb.einsum("ab,asc,bsd->cd", [T(g["cfg2_e"]), site, site.into_conj()]).to_numpy()
    assert oracle.rel_frobenius(got, g["cfg2_out"]) <= 1e-12
    got = tb.einsum("ijk,jlm,kmn,lnp->ip", [T(g[f"cfg4_op{i}"]) for i in range(4)]).to_numpy()
    assert oracle.rel_frobenius(got, g["cfg4_out"]) <= 1e-5
    got = tb.einsum("ijkl,klmn->ijmn", [T(g["cfg5_a"]), T(g["cfg5_b"])]).to_numpy()
    assert oracle.rel_frobenius(got, g["cfg5_out"]) <= 1e-5


def test_config1_full_size(tb, oracle):
    """'abc,bcd->ad', f64, all dims 64, N(0,1): the parity anchor, tolerance 1e-12."""
    a, b = oracle.normal(1000, (64, 64, 64), np.float64), oracle.normal(1001, (64, 64, 64), np.float64)
    got = tb.einsum("abc,bcd->ad", [tb.Tensor.from_numpy(a), tb.Tensor.from_numpy(b)]).to_numpy()
    want = oracle.np_einsum("abc,bcd->ad", [a, b])
    assert got.shape == (64, 64)
    assert oracle.rel_frobenius(got, want) <= 1e-12
    assert oracle.rel_frobenius(oracle.ttgt_contract([0, 1, 2], a, [1, 2, 3], b, [0, 3]), want) <= 1e-12


def test_config2_chain_full_bond_dimension(tb, oracle):
    """MPS transfer-matrix chain at chi = 512, d = 2, complex128, 4 of the 32 sites: every
    environment is compared with NumPy at 1e-12."""
    chi, d, sites = 512, 2, 4
    tree = tb.ContractionTree.optimize(tb.Subscripts.parse("ab,asc,bsd->cd"), [[chi, chi], [chi, d, chi], [chi, d, chi]])
    env = np.eye(chi, dtype=np.complex128)
    e_dev = tb.Tensor.from_numpy(env)
    for s in range(sites):
        a = oracle.normal(2000 + s, (chi, d, chi), np.complex128, scale=(1.0 / chi) ** 0.5)
        a_dev = tb.Tensor.from_numpy(a)
        nxt = tb.Tensor.empty([chi, chi], np.complex128)
        tb.einsum_with_plan_into(tree, [e_dev, a_dev, a_dev.into_conj()], 1.0, 0.0, nxt)
        e_dev = nxt
        env = np.einsum("ab,asc,bsd->cd", env, a, np.conj(a), optimize=True)
        assert oracle.rel_frobenius(e_dev.to_numpy(), env) <= 1e-12, s


def test_config3_grouped_sample(tb, oracle, golden):
    """Ragged 'ij,jk->ik' problems with dims from {16,32,64,128}, f32, U(-1,1), in one launch."""
    table = oracle.grouped_table(3000, 64)
    ctx = tb.Context.get(0)
    held, probs, wants = [], [], []
    for p, (i, j, k) in enumerate(table):
        a, b = oracle.uniform(3001 + 2 * p, (i, j), np.float32), oracle.uniform(3002 + 2 * p, (j, k), np.float32)
        ta, tb_, tc = tb.Tensor.from_numpy(a), tb.Tensor.from_numpy(b), tb.Tensor.zeros((i, k), dtype=np.float32)
        held += [ta, tb_, tc]
        probs.append((i, k, j, ta._block.ptr, 1, i, tb_._block.ptr, 1, j, tc._block.ptr, 1, i))
        wants.append(oracle.np_batched_gemm(a, b))
    tb.grouped_gemm(probs, np.float32, 1.0, 0.0, ctx)
    num = den = 0.0
    for p, want in enumerate(wants):
        got = held[3 * p + 2].to_numpy()
        assert oracle.rel_frobenius(got, want) <= 1e-5, p
        num += np.linalg.norm(got.astype(np.float64) - want) ** 2
        den += np.linalg.norm(want.astype(np.float64)) ** 2
    assert (num / den) ** 0.5 <= 1e-5
    for p in range(6):  # committed fixtures
        got = held[3 * p + 2].to_numpy()
        assert oracle.rel_frobenius(got, golden[f"cfg3_out{p}"]) <= 1e-5


@pytest.mark.parametrize("odd", [False, True])
def test_grouped_plan_runs_twice_with_accumulate(tb, oracle, odd):
    """The prepared form of the grouped product: C_p = alpha A_p B_p + beta C_p, executed twice on
    the same table (the second run accumulates onto the first).  `odd` adds a problem whose
    dims are not multiples of 16, which sends the whole table to the SIMT kernel."""
    table = [tuple(r) for r in oracle.grouped_table(3100, 40)]
    if odd:
        table.append((7, 13, 5))
    held, probs, ab = [], [], []
    for p, (i, j, k) in enumerate(table):
        a, b = oracle.uniform(3101 + 2 * p, (i, j), np.float32), oracle.uniform(3102 + 2 * p, (j, k), np.float32)
        c0 = oracle.uniform(3900 + p, (i, k), np.float32)
        ta, tb_, tc = tb.Tensor.from_numpy(a), tb.Tensor.from_numpy(b), tb.Tensor.from_numpy(c0)
        held += [ta, tb_, tc]
        probs.append((i, k, j, ta._block.ptr, 1, i, tb_._block.ptr, 1, j, tc._block.ptr, 1, i))
        ab.append((oracle.np_batched_gemm(a, b), c0.astype(np.float64)))
    plan = tb.PreparedGroupedGemm(probs, np.float32, alpha=0.5, beta=-2.0)
    plan.run()
    plan.run()
    tb.Context.get(0).synchronize()
    for p, (prod, c0) in enumerate(ab):
        want = 0.5 * prod - 2.0 * (0.5 * prod - 2.0 * c0)
        assert oracle.rel_frobenius(held[3 * p + 2].to_numpy(), want) <= 1e-5, p


def test_config4_network_dim24(tb, oracle):
    """'ijk,jlm,kmn,lnp->ip', complex64, N(0,1) parts, every index 24 (96 in the benchmark)."""
    ops = [oracle.normal(4000 + i, (24, 24, 24), np.complex64) for i in range(4)]
    got = tb.einsum("ijk,jlm,kmn,lnp->ip", [tb.Tensor.from_numpy(o) for o in ops]).to_numpy()
    assert oracle.rel_frobenius(got, oracle.np_einsum("ijk,jlm,kmn,lnp->ip", ops)) <= 1e-5


def test_config5_scaled(tb, oracle):
    """'ijkl,klmn->ijmn', f32, i=j=m=n=32, k=l=64 (128 / 256 in the benchmark), N(0,1)."""
    a, b = oracle.normal(5000, (32, 32, 64, 64), np.float32), oracle.normal(5001, (64, 64, 32, 32), np.float32)
    got = tb.einsum("ijkl,klmn->ijmn", [tb.Tensor.from_numpy(a), tb.Tensor.from_numpy(b)]).to_numpy()
    want = oracle.np_einsum("ijkl,klmn->ijmn", [a, b])
    assert oracle.rel_frobenius(got, want) <= 1e-5
    # shard over i (a strided sub-view, no communication) and over k (partial sums): both
    # reassemble to the single-device answer
    ta, tb_ = tb.Tensor.from_numpy(a), tb.Tensor.from_numpy(b)
    parts = []
    for r in range(2):
        sub = tb.Tensor(ta._block, (16, 32, 64, 64), ta.strides(), r * 16, np.float32, ta.logical_memory_space())
        parts.append(tb.einsum("ijkl,klmn->ijmn", [sub, tb_]).to_numpy())
    assert oracle.rel_frobenius(np.concatenate(parts, axis=0), want) <= 1e-5
    acc = tb.Tensor.zeros((32, 32, 32, 32), dtype=np.float32)
    for r in range(2):
        sa = tb.Tensor(ta._block, (32, 32, 32, 64), ta.strides(), r * 32 * ta.strides()[2], np.float32,
                       ta.logical_memory_space())
        sb = tb.Tensor(tb_._block, (32, 64, 32, 32), tb_.strides(), r * 32, np.float32, tb_.logical_memory_space())
        tb.einsum_into("ijkl,klmn->ijmn", [sa, sb], 1.0, 1.0, acc)
    assert oracle.rel_frobenius(acc.to_numpy(), want) <= 1e-5


@pytest.mark.parametrize("dtype,shape,perm", [
    (np.float32, (2048, 1024), (1, 0)),
    (np.float32, (32, 32, 32, 32), (3, 2, 1, 0)),
    (np.float32, (32, 32, 32, 32), (1, 0, 3, 2)),
    (np.float64, (96, 96, 96), (2, 0, 1)),
    (np.complex128, (512, 2, 512), (1, 2, 0)),
])
def test_permute_set_bit_exact(tb, dtype, shape, perm):
    """The permute benchmark set at reduced extents: bit-exact against numpy transpose().copy()."""
    rng = np.random.default_rng(31)
    a = random_array(rng, shape, dtype)
    t = tb.Tensor.from_numpy(a)
    got = t.permute(perm).contiguous(tb.MemoryOrder.ColumnMajor)
    want = np.transpose(a, perm).copy()
    assert got.strides()[0] == 1
    assert got.to_numpy().tobytes(order="F") == want.tobytes(order="F")
    # permuting back restores every bit (a size-independent property used at full size too)
    inv = np.argsort(perm)
    back = got.permute(list(inv)).contiguous(tb.MemoryOrder.ColumnMajor)
    assert back.to_numpy().tobytes(order="F") == a.tobytes(order="F")


def test_reduce_set(tb, oracle):
    rng = np.random.default_rng(32)
    a = random_array(rng, (2048, 1024), np.float32)
    t = tb.Tensor.from_numpy(a)
    for notation in ("ij->j", "ij->i", "ij->"):
        got = tb.einsum(notation, [t]).to_numpy()
        assert oracle.rel_frobenius(got, oracle.np_einsum(notation, [a])) <= 1e-5
    b = random_array(rng, (64, 96, 64), np.float64)
    got = tb.einsum("ijk->ik", [tb.Tensor.from_numpy(b)]).to_numpy()
    assert oracle.rel_frobenius(got, b.sum(axis=1)) <= 1e-12
    P = tb.PrimDescriptor
    for op, fn in ((tb.ReduceOp.Max, np.max), (tb.ReduceOp.Min, np.min)):
        out = tb.Tensor.zeros((1024,), dtype=np.float32)
        plan = tb.CudaBackend.plan(P.Reduce([0, 1], [1], op), [a.shape, (1024,)], np.float32)
        tb.CudaBackend.execute(plan, 1.0, [t], 0.0, out)
        assert np.array_equal(out.to_numpy(), fn(a, axis=0))
