"""`TensorPrims<A>` for an algebra other than Standard: the tropical semirings MaxPlus and MinPlus
(tenferro-algebra/src/lib.rs:74-106) on the GPU, through the C ABI, against the oracle's
broadcast-and-reduce restatement.  max and + of floats are exact operations up to the rounding
of each single addition, so the comparison is to 1e-6 (f32) / 1e-14 (f64) of the result's norm."""
import numpy as np
import pytest

from conftest import Strided, random_array

pytestmark = pytest.mark.gpu
TOL = {np.dtype("float32"): 1e-6, np.dtype("float64"): 1e-14}


def run(tb, desc, ins, out, dtype, algebra, alpha, beta):
    shapes = [s.dims for s in ins] + [out.dims]
    plan = tb.CudaBackend.plan(desc, shapes, dtype, algebra=algebra)
    d_out = out.to_device(tb)
    tb.CudaBackend.execute(plan, alpha, [s.to_device(tb) for s in ins], beta, d_out)
    return d_out.to_numpy(), plan


@pytest.mark.parametrize("dtype", [np.float32, np.float64])
@pytest.mark.parametrize("algebra", [1, 2], ids=["MaxPlus", "MinPlus"])
def test_tropical_contract_random_layouts(tb, oracle, dtype, algebra):
    rng = np.random.default_rng(400 + algebra)
    P, A = tb.PrimDescriptor, tb.Algebra(algebra)
    zero = -np.inf if algebra == 1 else np.inf
    for trial in range(8):
        b, m, n, k = (int(x) for x in rng.integers(1, 70, size=4))
        b = b % 3 + 1
        a = Strided(random_array(rng, (b, m, k), dtype), rng)
        bb = Strided(random_array(rng, (k, b, n), dtype), rng)
        c = Strided(random_array(rng, (n, m, b), dtype), rng)
        alpha, beta = [(0.0, zero), (0.5, -1.0), (-2.0, 0.0), (1.25, zero)][trial % 4]
        got, plan = run(tb, P.Contract([0, 1, 2], [2, 0, 3], [3, 1, 0]), [a, bb], c, dtype, A, alpha, beta)
        want = oracle.np_semiring_contract([[0, 1, 2], [2, 0, 3]], [a.logical, bb.logical], [3, 1, 0], algebra,
                                           alpha, beta, c.logical)
        assert plan.kernel_name == "simt_semiring"
        assert oracle.rel_frobenius(got, want) <= TOL[np.dtype(dtype)], (trial, b, m, n, k)


def test_tropical_shortest_path_squaring(tb, oracle):
    """MinPlus matrix 'multiplication' of a distance matrix with itself relaxes every path by one
    more edge: repeated squaring reaches all-pairs shortest paths (checked against Floyd-Warshall)."""
    rng = np.random.default_rng(410)
    n = 96
    w = rng.uniform(1.0, 10.0, (n, n))
    w[rng.uniform(size=(n, n)) < 0.7] = np.inf
    np.fill_diagonal(w, 0.0)
    fw = w.copy()
    for k in range(n):
        fw = np.minimum(fw, fw[:, k:k + 1] + fw[k:k + 1, :])
    plan = tb.CudaBackend.plan(tb.PrimDescriptor.BatchedGemm([], n, n, n), [(n, n)] * 3, np.float64,
                               algebra=tb.Algebra.MinPlus)
    d = tb.Tensor.from_numpy(w)
    for _ in range(7):  # 2^7 >= n - 1 edges
        nxt = tb.Tensor.empty((n, n), np.float64)
        tb.CudaBackend.execute(plan, 0.0, [d, d], np.inf, nxt)
        d = nxt
    got = d.to_numpy()
    finite = np.isfinite(fw)
    assert np.array_equal(np.isfinite(got), finite)
    assert np.allclose(got[finite], fw[finite], rtol=1e-13, atol=0)


@pytest.mark.parametrize("algebra", [1, 2], ids=["MaxPlus", "MinPlus"])
def test_tropical_reduce_elementwise_permute_trace(tb, oracle, algebra):
    rng = np.random.default_rng(420 + algebra)
    P, A = tb.PrimDescriptor, tb.Algebra(algebra)
    zero = -np.inf if algebra == 1 else np.inf
    dtype = np.float64
    # Reduce(Sum) adds with the algebra's (+): a maximum / minimum over the reduced modes
    a = Strided(random_array(rng, (9, 40, 17), dtype), rng)
    c = Strided(random_array(rng, (17, 9), dtype), rng)
    got, _ = run(tb, P.Reduce([0, 1, 2], [2, 0], tb.ReduceOp.Sum), [a], c, dtype, A, 0.25, 0.5)
    want = oracle.np_semiring_contract([[0, 1, 2]], [a.logical], [2, 0], algebra, 0.25, 0.5, c.logical)
    assert oracle.rel_frobenius(got, want) <= 1e-14
    # ElementwiseMul multiplies with (x) = +
    x, y = Strided(random_array(rng, (12, 31), dtype), rng), Strided(random_array(rng, (12, 31), dtype), rng)
    o = Strided(random_array(rng, (12, 31), dtype), rng)
    got, _ = run(tb, P.ElementwiseMul(), [x, y], o, dtype, A, 0.0, zero)
    assert oracle.rel_frobenius(got, x.logical + y.logical) <= 1e-14
    # Permute: alpha (x) A (+) beta (x) B
    p_in, p_out = Strided(random_array(rng, (5, 6, 7), dtype), rng), Strided(random_array(rng, (7, 5, 6), dtype), rng)
    got, _ = run(tb, P.Permute([0, 1, 2], [2, 0, 1]), [p_in], p_out, dtype, A, 1.0, -1.0)
    pick = np.maximum if algebra == 1 else np.minimum
    assert oracle.rel_frobenius(got, pick(np.transpose(p_in.logical, (2, 0, 1)) + 1.0, p_out.logical - 1.0)) <= 1e-14
    # Trace: the tropical sum over a diagonal
    t_in, t_out = Strided(random_array(rng, (11, 11, 4), dtype), rng), Strided(random_array(rng, (4,), dtype), rng)
    got, _ = run(tb, P.Trace([0, 1, 2], [2], [(0, 1)]), [t_in], t_out, dtype, A, 0.0, zero)
    want = oracle.np_semiring_contract([[0, 0, 2]], [t_in.logical], [2], algebra)
    assert oracle.rel_frobenius(got, want) <= 1e-14


def test_tropical_capabilities_and_rejections(tb):
    B, E, A = tb.CudaBackend, tb.Extension, tb.Algebra
    assert B.has_extension_for(np.float64, E.Contract, A.MaxPlus) and B.has_extension_for(np.float32, E.Contract, A.MinPlus)
    assert not B.has_extension_for(np.complex128, E.Contract, A.MaxPlus)
    assert B.has_extension_for(np.complex64, E.Contract, A.Standard)
    P = tb.PrimDescriptor
    with pytest.raises(tb.InvalidArgument, match="f32 and f64"):
        B.plan(P.Contract([0, 1], [1, 2], [0, 2]), [(3, 4), (4, 5), (3, 5)], np.complex128, algebra=A.MaxPlus)
    with pytest.raises(tb.InvalidArgument, match="Standard"):
        B.plan(P.AntiDiag([0], [0, 1], [(0, 1)]), [(3,), (3, 3)], np.float64, algebra=A.MaxPlus)
    plan = B.plan(P.Reduce([0, 1], [0], tb.ReduceOp.Max), [(3, 4), (3,)], np.float64, algebra=A.MaxPlus)
    with pytest.raises(tb.InvalidArgument, match="ReduceOp::Sum"):
        B.execute(plan, 0.0, [tb.Tensor.zeros((3, 4))], -np.inf, tb.Tensor.zeros((3,)))
