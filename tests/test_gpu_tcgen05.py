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
    assert err <= 2e-6, err


def test_tf32x3_alpha_beta_and_batch(tb, oracle):
    rng = np.random.default_rng(4)
    a, b = random_array(rng, (3, 160, 96), np.float32), random_array(rng, (3, 96, 272), np.float32)
    c0 = random_array(rng, (3, 160, 272), np.float32)
    got, name = run(tb, a, b, "row", "row", tb.ContractKernel.Auto, 0.5, -2.0, c0)
    assert name == "tcgen05_tf32x3"
    assert oracle.rel_frobenius(got, oracle.np_batched_gemm(a, b, 0.5, -2.0, c0)) <= 1e-5


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
