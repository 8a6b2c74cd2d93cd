"""The benchmark configurations at their full sizes, checked through properties that do not
need a CPU run of the same size: rank-structured operands whose product is known in closed
form, checksums that are linear in the inputs, and - where the CPU oracle still finishes in
seconds - a direct comparison."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def test_config5_full_size_rank_structured(tb, oracle):
    """'ijkl,klmn->ijmn', f32, i=j=m=n=128, k=l=256 (M = N = 16384, K = 65536, 2^45 flop).
    With A = u[i,j] v[k,l] and B = w[k,l] z[m,n] the result is (sum_kl v w) u[i,j] z[m,n]: every
    tile of the output and every k-block of the sum has a known value.  The deviation is measured
    on the device: C -= s u z, then |C|^2, all through the library's own einsum."""
    rng = np.random.default_rng(50)
    u, z = (rng.standard_normal((128, 128)).astype(np.float32) for _ in range(2))
    v, w = (rng.standard_normal((256, 256)).astype(np.float32) for _ in range(2))
    tu, tv, tw, tz = (tb.Tensor.from_numpy(x) for x in (u, v, w, z))
    A = tb.einsum("ij,kl->ijkl", [tu, tv])
    B = tb.einsum("kl,mn->klmn", [tw, tz])
    C = tb.einsum("ijkl,klmn->ijmn", [A, B])
    del A, B
    s = float(np.sum(v.astype(np.float64) * w.astype(np.float64)))
    ref_norm = abs(s) * np.linalg.norm(u.astype(np.float64)) * np.linalg.norm(z.astype(np.float64))
    tb.einsum_into("ij,mn->ijmn", [tu, tz], -s, 1.0, C)          # C <- C - s u z
    sq = tb.einsum("ijmn,ijmn->ijmn", [C, C])                    # element-wise square, then a plain reduction
    dev = float(tb.einsum("ijmn->", [sq]).to_numpy()) ** 0.5
    # the f32 rounding of s u z in the subtraction contributes ~6e-8 on top of the 3xTF32 error
    assert dev / ref_norm <= 1e-5, dev / ref_norm


def test_config3_full_table_checksums(tb, oracle):
    """All 4096 ragged problems: per problem, 1^T C 1 = (1^T A)(B 1), evaluated in float64 from
    the inputs - a checksum per problem that is linear in A and in B."""
    table = oracle.grouped_table(3000, 4096)
    rng = np.random.default_rng(30)
    held, probs, sums = [], [], []
    for (i, j, k) in table:
        a = rng.uniform(-1, 1, (i, j)).astype(np.float32)
        b = rng.uniform(-1, 1, (j, k)).astype(np.float32)
        ta, tb_, tc = tb.Tensor.from_numpy(a), tb.Tensor.from_numpy(b), tb.Tensor.zeros((i, k), dtype=np.float32)
        held.append((ta, tb_, tc))
        probs.append((i, k, j, ta._block.ptr, 1, i, tb_._block.ptr, 1, j, tc._block.ptr, 1, i))
        ra, cb = a.astype(np.float64).sum(axis=0), b.astype(np.float64).sum(axis=1)
        # scale of the checksum's rounding: sum_j |1^T A|_j |B 1|_j
        sums.append((float(ra @ cb), float(np.abs(ra) @ np.abs(cb)) + 1e-30))
    tb.grouped_gemm(probs, np.float32, 1.0, 0.0)
    worst = 0.0
    for (want, scale), (_, _, tc) in zip(sums, held):
        got = float(tc.to_numpy().astype(np.float64).sum())
        worst = max(worst, abs(got - want) / scale)
    assert worst <= 1e-5, worst


def test_config4_full_size_against_the_oracle(tb, oracle):
    """'ijk,jlm,kmn,lnp->ip', complex64, every index 96 (131 GFLOP, two 679 MB intermediates)."""
    ops = [oracle.normal(4000 + i, (96, 96, 96), np.complex64) for i in range(4)]
    got = tb.einsum("ijk,jlm,kmn,lnp->ip", [tb.Tensor.from_numpy(o) for o in ops]).to_numpy()
    want = oracle.np_einsum("ijk,jlm,kmn,lnp->ip", ops)
    assert oracle.rel_frobenius(got, want) <= 1e-5


def test_config2_full_chain_against_the_oracle(tb, oracle):
    """The whole benchmark chain: 32 sites, chi = 512, d = 2, complex128, site tensors from the
    benchmark's seeds 2000 + s, E_0 = identity.  Every one of the 32 environments is compared with
    the oracle's TTGT contraction (137 GFLOP of ZGEMM on the host) at 1e-12."""
    chi, d, sites = 512, 2, 32
    tree = tb.ContractionTree.optimize(tb.Subscripts.parse("ab,asc,bsd->cd"), [[chi, chi], [chi, d, chi], [chi, d, chi]])
    env = np.eye(chi, dtype=np.complex128)
    e_dev = tb.Tensor.from_numpy(env)
    worst = 0.0
    for s in range(sites):
        a = oracle.normal(2000 + s, (chi, d, chi), np.complex128, scale=(1.0 / chi) ** 0.5)
        a_dev = tb.Tensor.from_numpy(a)
        nxt = tb.Tensor.empty([chi, chi], np.complex128)
        tb.einsum_with_plan_into(tree, [e_dev, a_dev, a_dev.into_conj()], 1.0, 0.0, nxt)
        e_dev = nxt
        t = oracle.ttgt_contract([0, 1], env, [0, 2, 3], a, [1, 2, 3])            # ab,asc->bsc
        env = oracle.ttgt_contract([1, 2, 3], t, [1, 2, 4], np.conj(a), [3, 4])   # bsc,bsd->cd
        err = oracle.rel_frobenius(e_dev.to_numpy(), env)
        worst = max(worst, err)
        assert err <= 1e-12, (s, err)
    assert worst <= 1e-12


def test_config5_full_size_sampled_rows(tb, oracle):
    """'ijkl,klmn->ijmn' at full size with N(0,1) operands (seeds 5000, 5001 on the device's own
    generator): 8 random (i,j) rows x 2048 random (m,n) columns of C against a float64 sum over all
    65536 (k,l) on the host, relative Frobenius error <= 1e-5.  Generic data, so a fault in part
    of a k range or in one tile shows up, which rank-structured operands cannot guarantee."""
    import torch

    i = j = m = n = 128
    k = l = 256
    dev = torch.device("cuda", 0)
    gen = torch.Generator(device=dev)
    gen.manual_seed(5000)
    a_t = torch.randn((l, k, j, i), generator=gen, device=dev, dtype=torch.float32)  # column-major [i,j,k,l]
    gen.manual_seed(5001)
    b_t = torch.randn((n, m, l, k), generator=gen, device=dev, dtype=torch.float32)  # column-major [k,l,m,n]
    c_t = torch.empty((n, m, j, i), device=dev, dtype=torch.float32)
    space = tb.LogicalMemorySpace.GpuMemory(0)
    wrap = lambda t, dims: tb.Tensor.from_device_pointer(t.data_ptr(), t.numel() * 4, dims, np.float32, space, t)
    torch.cuda.synchronize()
    tb.einsum_into("ijkl,klmn->ijmn", [wrap(a_t, [i, j, k, l]), wrap(b_t, [k, l, m, n])], 1.0, 0.0, wrap(c_t, [i, j, m, n]))
    tb.Context.get(0).synchronize()
    rng = np.random.default_rng(55)
    rows = [(int(rng.integers(i)), int(rng.integers(j))) for _ in range(8)]
    cols = [(int(rng.integers(m)), int(rng.integers(n))) for _ in range(2048)]
    ci, cj = torch.tensor([r[0] for r in rows], device=dev), torch.tensor([r[1] for r in rows], device=dev)
    cm, cn = torch.tensor([c[0] for c in cols], device=dev), torch.tensor([c[1] for c in cols], device=dev)
    a_rows = a_t[:, :, cj, ci].reshape(l * k, len(rows)).cpu().numpy().astype(np.float64)   # [(l,k), row]
    b_cols = b_t[cn, cm].reshape(len(cols), l * k).cpu().numpy().astype(np.float64)         # [col, (l,k)]
    want = (b_cols @ a_rows).T                                                              # [row, col]
    got = c_t[cn[None, :], cm[None, :], cj[:, None], ci[:, None]].cpu().numpy().astype(np.float64)
    err = oracle.rel_frobenius(got, want)
    assert err <= 1e-5, err
    # and the same bound row by row: no single row hides behind the others
    for r in range(len(rows)):
        assert oracle.rel_frobenius(got[r], want[r]) <= 1e-5, (rows[r],)
