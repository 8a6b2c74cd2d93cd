"""The tcgen05 3xTF32 contraction kernel (f32): every operand-major combination, ragged tile
edges, batches, alpha/beta, against the float64 oracle at relative Frobenius 1e-5, and against
the exact-FMA SIMT kernel.  Layouts TMA cannot describe must fall back, not fail."""
import numpy as np
import pytest

from conftest import Strided, random_array

pytestmark = pytest.mark.gpu


def run(tb, a_arr, b_arr, la, lb, kernel, alpha=1.0, beta=0.0, c0=None):
    m, k = a_arr.shape[-2:]
    n = b_arr.shape[-1]
    batch = list(a_arr.shape[:-2])
    rng = np.random.default_rng(0)
    sa, sb = Strided(a_arr, rng, la), Strided(b_arr, rng, lb)
    plan = tb.CudaBackend.plan(tb.PrimDescriptor.BatchedGemm(batch, m, n, k),
                               [a_arr.shape, b_arr.shape, (*batch, m, n)], np.float32)
    plan.force_kernel(kernel)
    out = tb.Tensor.from_numpy(c0) if c0 is not None else tb.Tensor.zeros((*batch, m, n), dtype=np.float32)
    tb.CudaBackend.execute(plan, alpha, [sa.to_device(tb), sb.to_device(tb)], beta, out)
    return out.to_numpy(), plan.kernel_name


@pytest.mark.parametrize("shape", [(128, 256, 64), (256, 128, 32), (132, 300, 100), (512, 512, 512), (64, 64, 8),
                                   (1024, 768, 2048), (36, 44, 1000)])
@pytest.mark.parametrize("la", ["col", "row"])
@pytest.mark.parametrize("lb", ["col", "row"])
def test_tf32x3_all_majors(tb, oracle, shape, la, lb):
    m, n, k = shape
    rng = np.random.default_rng(m + 3 * n + 7 * k)
    a, b = random_array(rng, (m, k), np.float32), random_array(rng, (k, n), np.float32)
    want = oracle.np_batched_gemm(a, b)
    got, name = run(tb, a, b, la, lb, tb.ContractKernel.Auto)
    assert name == "tcgen05_tf32x3", (name, shape, la, lb)
    err = oracle.rel_frobenius(got, want)
    assert err <= 1e-5, (err, shape, la, lb)
    simt, name2 = run(tb, a, b, la, lb, tb.ContractKernel.Simt)
    assert name2 == "simt"
    assert oracle.rel_frobenius(got, simt) <= 1e-5


def test_tf32x3_is_far_better_than_plain_tf32(tb, oracle):
    """N(0,1) inputs at K = 4096: single-pass TF32 would sit near 1e-3; the split holds 1e-5."""
    rng = np.random.default_rng(3)
    a, b = random_array(rng, (256, 4096), np.float32), random_array(rng, (4096, 256), np.float32)
    got, name = run(tb, a, b, "row", "col", tb.ContractKernel.Tcgen05)
    assert name == "tcgen05_tf32x3"
    err = oracle.rel_frobenius(got, oracle.np_batched_gemm(a, b))
    assert err <= 3e-6, err


def test_tf32x3_alpha_beta_and_batch(tb, oracle):
    rng = np.random.default_rng(4)
    a, b = random_array(rng, (3, 160, 96), np.float32), random_array(rng, (3, 96, 272), np.float32)
    c0 = random_array(rng, (3, 160, 272), np.float32)
    got, name = run(tb, a, b, "row", "row", tb.ContractKernel.Auto, 0.5, -2.0, c0)
    assert name == "tcgen05_tf32x3"
    assert oracle.rel_frobenius(got, oracle.np_batched_gemm(a, b, 0.5, -2.0, c0)) <= 1e-5


@pytest.mark.parametrize("shape", [(384, 640, 96), (300, 700, 200), (256, 256, 8), (1280, 260, 520)])
@pytest.mark.parametrize("la,lb", [("col", "col"), ("row", "col"), ("col", "row")])
def test_cta_pair_tiles_odd_counts_and_ragged_edges(tb, oracle, shape, la, lb):
    """Outputs of 256 x 256 and more run on CTA pairs (two 128-row tiles x two 128-column tiles
    per pair): odd tile counts leave one CTA of the last pair without a tile, ragged extents
    leave partial tiles; alpha and beta apply once."""
    m, n, k = shape
    rng = np.random.default_rng(11 * m + 5 * n + k)
    a, b = random_array(rng, (m, k), np.float32), random_array(rng, (k, n), np.float32)
    c0 = random_array(rng, (m, n), np.float32)
    got, name = run(tb, a, b, la, lb, tb.ContractKernel.Auto, -1.5, 0.25, c0)
    assert name == "tcgen05_tf32x3"
    assert oracle.rel_frobenius(got, oracle.np_batched_gemm(a, b, -1.5, 0.25, c0)) <= 1e-5


@pytest.mark.parametrize("shape,beta,la,lb", [((4096, 4096, 72), 0.0, "col", "row"), ((2100, 4200, 250), 0.75, "col", "col"),
                                              ((3, 600, 1100, 256), 0.0, "row", "row")])
def test_short_k_products_drain_through_dedicated_warps(tb, oracle, shape, beta, la, lb, monkeypatch):
    """K of at most 256: the sums in tensor memory are final, half of the converter warps only
    drain them to the output while the other half keeps converting.  Several tiles per CTA pair, so
    both accumulators are reused many times; ragged edges; beta; the same result, to rounding, as
    the kernel that promotes and stores from the converter warps."""
    *batch, m, n, k = shape
    rng = np.random.default_rng(m + n + k)
    a, b = random_array(rng, (*batch, m, k), np.float32), random_array(rng, (*batch, k, n), np.float32)
    c0 = random_array(rng, (*batch, m, n), np.float32)
    got, name = run(tb, a, b, la, lb, tb.ContractKernel.Auto, 1.25, beta, c0.copy())
    assert name == "tcgen05_tf32x3"
    want = oracle.np_batched_gemm(a, b, 1.25, beta, c0)
    assert oracle.rel_frobenius(got, want) <= 1e-5
    monkeypatch.setenv("TFB_TC_SHORTK", "0")
    other, _ = run(tb, a, b, la, lb, tb.ContractKernel.Auto, 1.25, beta, c0.copy())
    assert oracle.rel_frobenius(got, other) <= 2e-6


@pytest.mark.parametrize("shape,beta", [((2048, 2304, 256), 0.0), ((1100, 900, 248), 0.5), ((2, 640, 768, 192), 0.0),
                                        ((512, 512, 200), -1.0), ((768, 1024, 1024), 0.0), ((640, 520, 2100), 0.25),
                                        ((200, 300, 9216), 0.0)])
@pytest.mark.parametrize("la,lb", [("row", "col"), ("col", "col"), ("row", "row"), ("col", "row")])
@pytest.mark.parametrize("spread", [0, 12], ids=["N(0,1)", "magnitudes over 2^24"])
def test_corrections_as_one_bf16_product(tb, oracle, shape, beta, la, lb, spread, monkeypatch):
    """The CTA-pair kernel runs the two correction terms of 3xTF32 as one bf16 product of the
    remainders and the values: short K (one accumulation chunk, 192 to 256), long K (promotions,
    ragged last k-block) and split K, every operand-major combination, a batch.  Same bar against
    float64 as the three-TF32 form, which TFB_TC_BF16_CORRECTIONS=0 brings back, and the two agree
    to rounding - also when the operands' magnitudes spread over 2^24, where a correction term
    rounded too early would show."""
    *batch, m, n, k = shape
    if batch and (la, lb) != ("row", "col"):
        pytest.skip("the batched case is built with both operands K-major")
    rng = np.random.default_rng(m + 2 * n + 3 * k + spread)
    a, b = random_array(rng, (*batch, m, k), np.float32), random_array(rng, (*batch, k, n), np.float32)
    if spread:
        a = (a * np.exp2(rng.integers(-spread, spread + 1, a.shape))).astype(np.float32)
        b = (b * np.exp2(rng.integers(-spread, spread + 1, b.shape))).astype(np.float32)
    c0 = random_array(rng, (*batch, m, n), np.float32)

    def product():
        if not batch:
            return run(tb, a, b, la, lb, tb.ContractKernel.Auto, 1.0, beta, c0.copy())
        # [batch, i, k] and [batch, j, k], both with k next to each other in memory and the batch outermost
        bt = np.ascontiguousarray(np.swapaxes(b, -1, -2))
        plan = tb.CudaBackend.plan(tb.PrimDescriptor.Contract([0, 1, 2], [0, 3, 2], [0, 1, 3]), [a.shape, bt.shape, c0.shape],
                                   np.float32)
        out = tb.Tensor.from_numpy(c0.copy())
        tb.CudaBackend.execute(plan, 1.0, [Strided(a, rng, "row").to_device(tb), Strided(bt, rng, "row").to_device(tb)], beta, out)
        return out.to_numpy(), plan.kernel_name

    got, name = product()
    assert name == "tcgen05_tf32x3"
    want = oracle.np_batched_gemm(a, b, 1.0, beta, c0)
    err = oracle.rel_frobenius(got, want)
    assert err <= 1e-5, err
    monkeypatch.setenv("TFB_TC_BF16_CORRECTIONS", "0")
    other, _ = product()
    err3 = oracle.rel_frobenius(other, want)
    assert err3 <= 1e-5, err3
    assert err <= 2 * err3 + 1e-6, (err, err3)
    assert oracle.rel_frobenius(got, other) <= 3e-6
    assert not np.array_equal(got, other)  # the switch does select another form of the corrections


@pytest.mark.parametrize("shape,la,lb,copies", [((384, 8192, 640), "col", "col", 1), ((8192, 300, 520), "row", "row", 1),
                                                ((8192, 8192, 512), "col", "row", 2), ((384, 4096, 640), "col", "col", 0),
                                                ((384, 8192, 640), "row", "col", 0)])
def test_large_products_copy_mn_major_operands_k_major(tb, oracle, shape, la, lb, copies, monkeypatch):
    """An operand whose free index is the contiguous one is copied K-major first when the other
    operand has 8192 rows or more (the copy costs less than the faster conversion of K-major tiles
    saves); smaller products and K-major operands run as they lie.  Same result either way."""
    m, n, k = shape
    rng = np.random.default_rng(m + n + k)
    a, b = random_array(rng, (m, k), np.float32), random_array(rng, (k, n), np.float32)
    ctx = tb.Context.get(0)
    ctx.profile_begin()
    got, name = run(tb, a, b, la, lb, tb.ContractKernel.Auto)
    ctx.synchronize()
    launched = ctx.profile_read("repack_operand")[0]
    ctx.profile_end()
    assert name == "tcgen05_tf32x3"
    assert launched == copies, (launched, copies)
    assert oracle.rel_frobenius(got, oracle.np_batched_gemm(a, b)) <= 1e-5
    monkeypatch.setenv("TFB_TC_REPACK_MN", "0")
    ctx.profile_begin()
    other, _ = run(tb, a, b, la, lb, tb.ContractKernel.Auto)
    ctx.synchronize()
    assert ctx.profile_read("repack_operand")[0] == 0
    ctx.profile_end()
    assert oracle.rel_frobenius(got, other) <= 1e-6


@pytest.mark.parametrize("k", [256, 4096])
def test_bf16_corrections_keep_exact_products_exact(tb, oracle, k):
    """Operands that TF32 holds exactly (small integers) have zero remainders: the correction
    product adds nothing and the sums come out exact."""
    rng = np.random.default_rng(5)
    a = rng.integers(-8, 9, (768, k)).astype(np.float32)
    b = rng.integers(-8, 9, (k, 1024)).astype(np.float32)
    for la, lb in (("row", "col"), ("col", "row")):
        got, name = run(tb, a, b, la, lb, tb.ContractKernel.Auto)
        assert name == "tcgen05_tf32x3"
        assert np.array_equal(got, (a.astype(np.float64) @ b.astype(np.float64)).astype(np.float32))


def test_short_k_product_into_an_output_without_common_column_stride(tb, oracle):
    """Three free modes on the N side: the drain warps take the column offsets from the table."""
    rng = np.random.default_rng(77)
    a = random_array(rng, (320, 64), np.float32)                    # [i, k]
    b = random_array(rng, (64, 6, 10, 7), np.float32)               # [k, p, q, r]
    plan = tb.CudaBackend.plan(tb.PrimDescriptor.Contract([0, 1], [1, 2, 3, 4], [3, 0, 4, 2]),
                               [a.shape, b.shape, (10, 320, 7, 6)], np.float32)
    out = tb.Tensor.zeros((10, 320, 7, 6), dtype=np.float32)
    tb.CudaBackend.execute(plan, 1.0, [tb.Tensor.from_numpy(a), tb.Tensor.from_numpy(b)], 0.0, out)
    assert oracle.rel_frobenius(out.to_numpy(), oracle.np_einsum("ik,kpqr->qirp", [a, b])) <= 1e-5


@pytest.mark.parametrize("shape", [(96, 96, 9216), (96, 1000, 4096), (200, 120, 2052), (2, 130, 300, 1536)])
def test_split_k_for_small_outputs_with_long_k(tb, oracle, shape):
    """Few output tiles and a long K: the k-blocks of a tile are shared out among several CTAs
    and a finishing kernel adds their partial tiles in a fixed order (so reruns agree bit for
    bit) and applies alpha and beta."""
    *batch, m, n, k = shape
    rng = np.random.default_rng(m + n + k)
    a, b = random_array(rng, (*batch, m, k), np.float32), random_array(rng, (*batch, k, n), np.float32)
    c0 = random_array(rng, (*batch, m, n), np.float32)
    want = oracle.np_batched_gemm(a, b, 2.0, -0.5, c0)
    lb = "row" if batch else "col"  # column-major with a batch puts the unit stride on the batch mode
    got, name = run(tb, a, b, "row", lb, tb.ContractKernel.Auto, 2.0, -0.5, c0)
    assert name == "tcgen05_tf32x3"
    assert oracle.rel_frobenius(got, want) <= 1e-5
    again, _ = run(tb, a, b, "row", lb, tb.ContractKernel.Auto, 2.0, -0.5, c0)
    assert np.array_equal(got, again)


def test_layouts_tma_cannot_describe_fall_back(tb, oracle):
    rng = np.random.default_rng(5)
    a, b = random_array(rng, (130, 67), np.float32), random_array(rng, (67, 150), np.float32)
    want = oracle.np_batched_gemm(a, b)
    for la, lb in (("col", "col"), ("random", "random")):
        got, name = run(tb, a, b, la, lb, tb.ContractKernel.Auto)
        assert oracle.rel_frobenius(got, want) <= 1e-5, (la, lb, name)
    sa, sb = Strided(a, rng, "random"), Strided(b, rng, "random")
    plan = tb.CudaBackend.plan(tb.PrimDescriptor.BatchedGemm([], 130, 150, 67), [(130, 67), (67, 150), (130, 150)],
                               np.float32)
    plan.force_kernel(tb.ContractKernel.Tcgen05)
    with pytest.raises(tb.InvalidArgument):
        tb.CudaBackend.execute(plan, 1.0, [sa.to_device(tb), sb.to_device(tb)], 0.0,
                               tb.Tensor.zeros((130, 150), dtype=np.float32))


def test_einsum_ijkl_klmn_uses_tensor_cores(tb, oracle):
    """'ijkl,klmn->ijmn' (config 5 at i=j=m=n=16, k=l=32): M = (i,j) fused and unit stride (MN-major
    A), K = (k,l) fused and unit stride in B (K-major B)."""
    a, b = oracle.normal(5000, (16, 16, 32, 32), np.float32), oracle.normal(5001, (32, 32, 16, 16), np.float32)
    plan = tb.CudaBackend.plan(tb.PrimDescriptor.Contract([0, 1, 2, 3], [2, 3, 4, 5], [0, 1, 4, 5]),
                               [a.shape, b.shape, (16, 16, 16, 16)], np.float32)
    out = tb.Tensor.zeros((16, 16, 16, 16), dtype=np.float32)
    tb.CudaBackend.execute(plan, 1.0, [tb.Tensor.from_numpy(a), tb.Tensor.from_numpy(b)], 0.0, out)
    assert plan.kernel_name == "tcgen05_tf32x3"
    assert oracle.rel_frobenius(out.to_numpy(), oracle.np_einsum("ijkl,klmn->ijmn", [a, b])) <= 1e-5


@pytest.mark.parametrize("case", [
    # (labels_a, shape_a, labels_b, shape_b, labels_c): groups with two non-fusable modes each way
    ("free pair, MN-major, packed", [0, 1, 2], (64, 6, 40), [2, 3], (40, 72), [0, 1, 3], "sub_i"),
    ("free pair, MN-major, inner extent 16 (what sharding a mode eight ways leaves): tiles mostly padding",
     [0, 1, 2], (32, 40, 48), [2, 3], (48, 264), [0, 1, 3], "sub_i"),
    ("the same at a size where the operand is repacked K-major first", [0, 1, 2], (32, 256, 512), [2, 3], (512, 512),
     [0, 1, 3], "sub_i"),
    ("free pair, K-major, inner extent 96 padded to the tile", [2, 0, 1], (64, 96, 5), [2, 3], (64, 160), [0, 1, 3], None),
    ("free pair, K-major, packed small inner extent", [2, 0, 1], (48, 32, 9), [2, 3], (48, 96), [0, 1, 3], None),
    ("contracted pair not fusable in B", [0, 1, 2], (96, 96, 40), [3, 2, 1, 4], (24, 40, 96, 3), [0, 3, 4], None),
    ("dim-96 network step", [0, 1, 2], (96, 96, 96), [3, 2, 1, 4], (96, 96, 96, 8), [0, 3, 4], None),
])
def test_tf32x3_two_modes_per_group(tb, oracle, case):
    name, la, sa, lb, sb, lc, special = case
    rng = np.random.default_rng(sum(sa) + sum(sb))
    a, b = random_array(rng, sa, np.float32), random_array(rng, sb, np.float32)
    ext = dict(zip(la, sa))
    ext.update(dict(zip(lb, sb)))
    sc = tuple(ext[l] for l in lc)
    ta, tbt = tb.Tensor.from_numpy(a), tb.Tensor.from_numpy(b)
    if special == "sub_i":
        # a strided sub-view: the first half of mode 0 (what sharding a free index produces)
        half = sa[0] // 2
        ta = tb.Tensor(ta._block, (half,) + tuple(sa[1:]), ta.strides(), 0, np.float32, ta.logical_memory_space())
        a = a[:half]
        sc = (half,) + sc[1:]
    plan = tb.CudaBackend.plan(tb.PrimDescriptor.Contract(la, lb, lc), [a.shape, b.shape, sc], np.float32)
    out = tb.Tensor.zeros(sc, dtype=np.float32)
    tb.CudaBackend.execute(plan, 1.0, [ta, tbt], 0.0, out)
    assert plan.kernel_name == "tcgen05_tf32x3", (name, plan.kernel_name)
    want = oracle.np_contract(la, a, lb, b, lc)
    assert oracle.rel_frobenius(out.to_numpy(), want) <= 1e-5, name


@pytest.mark.parametrize("shape", [(64, 96, 40), (130, 70, 33), (256, 256, 512), (96, 1152, 96)])
def test_complex64_on_tensor_cores(tb, oracle, shape):
    """Complex32 contractions as one real product of doubled extents: the 2 x 2 real embedding of
    A gathered from any layout (conj and alpha folded in), B copied K-major or used in place,
    the result written straight into the complex output; complex beta applied beforehand."""
    m, n, k = shape
    rng = np.random.default_rng(m + n + k)
    for trial, layout in enumerate(("col", "row", "random")):
        a = Strided(random_array(rng, (m, k), np.complex64), rng, layout, conj=bool(trial % 2))
        b = Strided(random_array(rng, (k, n), np.complex64), rng, layout, conj=bool(trial == 2))
        c = Strided(random_array(rng, (m, n), np.complex64), rng, layout if layout != "random" else "col")
        alpha, beta = [(1.0, 0.0), (0.5 - 0.25j, 1.5j), (-1.0, 1.0)][trial]
        plan = tb.CudaBackend.plan(tb.PrimDescriptor.Contract([0, 1], [1, 2], [0, 2]), [(m, k), (k, n), (m, n)], np.complex64)
        out = c.to_device(tb)
        tb.CudaBackend.execute(plan, alpha, [a.to_device(tb), b.to_device(tb)], beta, out)
        assert plan.kernel_name == "tcgen05_tf32x3", (layout, plan.kernel_name)
        want = oracle.np_contract([0, 1], a.logical, [1, 2], b.logical, [0, 2], alpha, beta, c.logical)
        err = oracle.rel_frobenius(out.to_numpy(), want)
        assert err <= 1e-5, (err, layout, shape)


def test_network_einsum_complex64_dim32(tb, oracle):
    ops = [oracle.normal(4000 + i, (32, 32, 32), np.complex64) for i in range(4)]
    got = tb.einsum("ijk,jlm,kmn,lnp->ip", [tb.Tensor.from_numpy(o) for o in ops]).to_numpy()
    assert oracle.rel_frobenius(got, oracle.np_einsum("ijk,jlm,kmn,lnp->ip", ops)) <= 1e-5


def _einsum_both_store_paths(tb, monkeypatch, notation, ops, alpha=1.0):
    """Run one einsum with the TMA-store epilogue on and off; returns the two results."""
    outs = []
    tree = tb.ContractionTree.optimize(tb.Subscripts.parse(notation), [o.dims() for o in ops])
    for flag in ("1", "0"):
        monkeypatch.setenv("TFB_TC_TMA_STORE", flag)
        out = tb.Tensor.empty(tree.output_dims, ops[0].dtype)
        tb.einsum_with_plan_into(tree, ops, alpha, 0.0, out)
        outs.append(out.to_numpy())
    return outs


@pytest.mark.parametrize("k", [64, 1000], ids=["short-K drain warps", "general kernel"])
def test_tma_store_epilogue_matches_per_element_stores(tb, oracle, monkeypatch, k):
    """Outputs the CTA-pair kernel can describe as a tensor map leave through TMA tensor stores
    (32 x 32 boxes staged in shared memory).  Same arithmetic, another way out: the results must be
    bit-identical to the per-element store path, for ragged edges, two-mode row and column groups,
    the float view of a complex output, and alpha != 1."""
    rng = np.random.default_rng(500 + k)
    T = tb.Tensor.from_numpy
    space = tb.LogicalMemorySpace.GpuMemory(0)
    # ragged single-mode rows and columns
    a, b = random_array(rng, (300, k), np.float32), random_array(rng, (k, 520), np.float32)
    on, off = _einsum_both_store_paths(tb, monkeypatch, "ij,jk->ik", [T(a), T(b)], alpha=0.5)
    assert np.array_equal(on, off)
    assert oracle.rel_frobenius(on, 0.5 * (a.astype(np.float64) @ b.astype(np.float64))) <= 1e-5
    # two-mode rows (i = 64 of a pitch of 96, then j) and two-mode columns (m = 96 of a pitch of 128, then n)
    kk = k // 4 * 4
    a_full, b_full = random_array(rng, (96, 5, kk), np.float32), random_array(rng, (kk, 128, 7), np.float32)
    ta, tb_ = T(a_full), T(b_full)
    a_view = tb.Tensor(ta._block, (64, 5, kk), ta.strides(), 0, np.float32, space)
    b_view = tb.Tensor(tb_._block, (kk, 96, 7), tb_.strides(), 0, np.float32, space)
    on, off = _einsum_both_store_paths(tb, monkeypatch, "ijk,kmn->ijmn", [a_view, b_view])
    want = np.einsum("ijk,kmn->ijmn", a_full[:64].astype(np.float64), b_full[:, :96].astype(np.float64))
    assert np.array_equal(on, off)
    assert oracle.rel_frobenius(on, want) <= 1e-5
    # complex64: the output is written through its float view (interleaved real and imaginary rows)
    ca, cb = random_array(rng, (200, k), np.complex64), random_array(rng, (k, 300), np.complex64)
    on, off = _einsum_both_store_paths(tb, monkeypatch, "ij,jk->ik", [T(ca), T(cb)])
    assert np.array_equal(on, off)
    assert oracle.rel_frobenius(on, ca.astype(np.complex128) @ cb.astype(np.complex128)) <= 1e-5
    # an output whose unit-stride mode belongs to neither group's first mode: falls back, same result
    on, off = _einsum_both_store_paths(tb, monkeypatch, "ijk,kmn->jinm", [a_view, b_view])
    assert np.array_equal(on, off)
    assert oracle.rel_frobenius(on, np.transpose(want, (1, 0, 3, 2))) <= 1e-5


@pytest.mark.parametrize("shape", [(4096, 192, 512), (192, 4096, 512), (2048, 100, 300), (1000, 64, 64), (300, 256, 96),
                                   (700, 40, 1000), (5000, 32, 2048), (96 * 2, 9216, 640), (256, 300, 128), (260, 250, 8200)])
@pytest.mark.parametrize("la,lb", [("col", "col"), ("row", "col"), ("col", "row"), ("row", "row")])
def test_narrow_outputs_are_one_pair_tile_of_their_own_width(tb, oracle, shape, la, lb, monkeypatch):
    """An output with at most 256 columns (or, with the operands' roles exchanged, at most 256
    rows) is one CTA-pair tile whose MMAs are exactly as wide as it needs: half-tiles of 32, 64,
    96 or 128 columns.  Same answers as the full-width tiling and as float64, with alpha, beta
    and an old output, short and long K (one accumulation chunk, several, split-K)."""
    m, n, k = shape
    rng = np.random.default_rng(13 * m + 7 * n + k)
    a, b = random_array(rng, (m, k), np.float32), random_array(rng, (k, n), np.float32)
    c0 = random_array(rng, (m, n), np.float32)
    want = oracle.np_batched_gemm(a, b, 0.75, -0.5, c0)
    got, name = run(tb, a, b, la, lb, tb.ContractKernel.Auto, 0.75, -0.5, c0)
    assert name == "tcgen05_tf32x3"
    assert oracle.rel_frobenius(got, want) <= 1e-5, (shape, la, lb)
    got0, _ = run(tb, a, b, la, lb, tb.ContractKernel.Auto)  # beta = 0: the tensor-store epilogue where it applies
    assert oracle.rel_frobenius(got0, oracle.np_batched_gemm(a, b)) <= 1e-5, (shape, la, lb)
    monkeypatch.setenv("TFB_TC_NARROW", "0")
    wide, _ = run(tb, a, b, la, lb, tb.ContractKernel.Auto, 0.75, -0.5, c0)
    assert oracle.rel_frobenius(got, wide.astype(np.float64)) <= 2e-6, (shape, la, lb)


@pytest.mark.parametrize("shape", [(96, 4096, 512), (48, 2048, 100), (128, 1024, 4100), (160, 1000, 64), (4096, 96, 512),
                                   (2048, 48, 100), (3000, 130, 260)])
def test_complex64_narrow_rows_exchange_roles(tb, oracle, shape):
    """Complex64 with few rows: the embedded operand (2 M real rows) becomes the column side of the
    real product; M' = 96, 192, 256 take the narrow tile, 320 does not."""
    m, n, k = shape
    rng = np.random.default_rng(17 * m + n + 3 * k)
    a, b = random_array(rng, (m, k), np.complex64), random_array(rng, (k, n), np.complex64)
    c0 = random_array(rng, (m, n), np.complex64)
    ta, tb_, tc = tb.Tensor.from_numpy(a), tb.Tensor.from_numpy(b), tb.Tensor.from_numpy(c0)
    tb.einsum_into("ik,kj->ij", [ta, tb_], 0.5 - 0.25j, 2.0, tc)
    want = (0.5 - 0.25j) * (a.astype(np.complex128) @ b.astype(np.complex128)) + 2.0 * c0.astype(np.complex128)
    assert oracle.rel_frobenius(tc.to_numpy(), want) <= 1e-5, shape
