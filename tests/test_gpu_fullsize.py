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


def test_config2_full_chain_norm_is_preserved(tb, oracle):
    """32 sites, chi = 512, d = 2, complex128.  With isometric site tensors
    (sum_{a,s} conj(A[a,s,c]) A[a,s,d] = delta_cd) the identity environment is a fixed point of
    'ab,asc,bsd->cd': after any number of sites E stays the identity to 1e-12."""
    chi, d, sites = 512, 2, 32
    rng = np.random.default_rng(20)
    tree = tb.ContractionTree.optimize(tb.Subscripts.parse("ab,asc,bsd->cd"), [[chi, chi], [chi, d, chi], [chi, d, chi]])
    env = tb.Tensor.from_numpy(np.eye(chi, dtype=np.complex128))
    for s in range(sites):
        if s % 8 == 0:  # four distinct isometries, reused: QR of a (chi d) x chi Gaussian matrix
            g = rng.standard_normal((chi * d, chi)) + 1j * rng.standard_normal((chi * d, chi))
            q, _ = np.linalg.qr(g)
            a_dev = tb.Tensor.from_numpy(np.asfortranarray(q.reshape(chi, d, chi, order="F")))
        nxt = tb.Tensor.empty([chi, chi], np.complex128)
        tb.einsum_with_plan_into(tree, [env, a_dev, a_dev.into_conj()], 1.0, 0.0, nxt)
        env = nxt
    assert oracle.rel_frobenius(env.to_numpy(), np.eye(chi, dtype=np.complex128)) <= 1e-12
