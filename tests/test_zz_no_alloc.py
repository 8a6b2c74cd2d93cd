"""The allocation-free reduce entry point (tfb_reduce_static), called through the C ABI.

It serves callers that may not allocate device memory at the time of the call (their own
allocator owns the device, a latency-critical loop, a framework callback): the partial sums of
a split reduction sit in a fixed array inside the library.  The check is that it returns what
the ordinary Reduce plan returns - twice in a row on different data, because the array keeps
whatever the previous call left in it.  This file sorts last so that a run stopping at the
first failure has already executed every other test."""
import numpy as np
import pytest

from conftest import random_array

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("dtype,tol", [(np.float32, 1e-5), (np.float64, 1e-12), (np.complex128, 1e-12)])
def test_static_reduce_matches_plan_twice(tb, oracle, dtype, tol):
    from tenferro_b200.prims import reduce_static

    rng = np.random.default_rng(77)
    P = tb.PrimDescriptor
    shape, kept = (48, 200000), [0]  # few outputs, long rows: the reduction is split and uses the scratch
    plan = tb.CudaBackend.plan(P.Reduce([0, 1], kept, tb.ReduceOp.Sum), [shape, (48,)], dtype)
    for call in range(2):
        a = random_array(rng, shape, dtype) * (call + 1)
        c0 = random_array(rng, (48,), dtype)
        ta = tb.Tensor.from_numpy(a)
        ref, got = tb.Tensor.from_numpy(c0), tb.Tensor.from_numpy(c0)
        tb.CudaBackend.execute(plan, 0.5, [ta], -1.0, ref)
        reduce_static([0, 1], ta, kept, got, tb.ReduceOp.Sum, 0.5, -1.0)
        want = oracle.np_reduce([0, 1], a, kept, 0, 0.5, -1.0, c0)
        assert oracle.rel_frobenius(got.to_numpy(), ref.to_numpy()) <= tol, call
        assert oracle.rel_frobenius(got.to_numpy(), want) <= tol * 2, call


def test_static_reduce_max_and_layouts(tb):
    from tenferro_b200.prims import reduce_static

    rng = np.random.default_rng(78)
    a = random_array(rng, (300, 70, 9), np.float32)
    ta = tb.Tensor.from_numpy(a).permute([2, 0, 1])  # a strided view: modes (2, 0, 1)
    for op, fn in ((tb.ReduceOp.Max, np.max), (tb.ReduceOp.Min, np.min)):
        out = tb.Tensor.zeros((70,), dtype=np.float32)
        reduce_static([2, 0, 1], ta, [1], out, op)
        assert np.array_equal(out.to_numpy(), fn(a, axis=(0, 2)))
    # kept mode contiguous in the input, reduced mode strided (the other thread layout)
    out = tb.Tensor.zeros((300,), dtype=np.float32)
    reduce_static([2, 0, 1], ta, [0], out, tb.ReduceOp.Sum)
    assert np.allclose(out.to_numpy(), a.sum(axis=(1, 2)), rtol=1e-5, atol=1e-4)


def test_static_reduce_rejects_large_outputs(tb):
    from tenferro_b200.prims import reduce_static

    a = tb.Tensor.zeros((600000, 2), dtype=np.float32)  # output of 2.4 MB > 2 MiB
    out = tb.Tensor.zeros((600000,), dtype=np.float32)
    with pytest.raises(tb.InvalidArgument, match="allocation-free"):
        reduce_static([0, 1], a, [0], out)
    with pytest.raises(tb.InvalidArgument):
        reduce_static([0, 0], tb.Tensor.zeros((4, 4)), [0], tb.Tensor.zeros((4,)))


def test_static_reduce_empty_range_matches_the_plan(tb):
    """A reduced mode of extent 0: the sum over nothing is 0, so both entry points leave beta * C."""
    from tenferro_b200.prims import reduce_static

    c0 = np.arange(6, dtype=np.float64)
    a = tb.Tensor.zeros((6, 0), dtype=np.float64)
    ref, got = tb.Tensor.from_numpy(c0), tb.Tensor.from_numpy(c0)
    plan = tb.CudaBackend.plan(tb.PrimDescriptor.Reduce([0, 1], [0], tb.ReduceOp.Sum), [(6, 0), (6,)], np.float64)
    tb.CudaBackend.execute(plan, 2.0, [a], -0.5, ref)
    reduce_static([0, 1], a, [0], got, tb.ReduceOp.Sum, 2.0, -0.5)
    assert np.array_equal(ref.to_numpy(), -0.5 * c0) and np.array_equal(got.to_numpy(), ref.to_numpy())
    with pytest.raises(tb.InvalidArgument):
        reduce_static([0, 1], a, [0], got, tb.ReduceOp.Max)
