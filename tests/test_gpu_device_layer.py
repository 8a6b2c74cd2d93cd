"""The device layer either side of the contraction path: moving tensors between memory spaces
(tenferro-tensor/src/lib.rs:660-713), completion events shared by the views of one buffer, the
capped pool, streams and contexts, pitched copies, and the kernels' bounded waits running out
without harming the context (Error::DeviceError, tenferro-device/src/lib.rs:128-130)."""
import ctypes as C
import os

import numpy as np
import pytest

from conftest import random_array

pytestmark = pytest.mark.gpu


# ---------------------------------------------------------------- to_memory_space_async
def test_main_to_gpu_and_back(tb, oracle):
    rng = np.random.default_rng(300)
    a = random_array(rng, (37, 5, 11), np.complex128)
    main, gpu = tb.LogicalMemorySpace.MainMemory(), tb.LogicalMemorySpace.GpuMemory(0)
    host = tb.Tensor.from_numpy(a, memory_space=main)
    assert host.logical_memory_space() == main and host.dims() == (37, 5, 11)
    assert np.array_equal(host.to_numpy(), a)
    dev = host.to_memory_space_async(gpu)
    assert dev.logical_memory_space() == gpu and dev.event is not None
    dev.wait()
    assert dev.is_ready()
    assert np.array_equal(dev.to_numpy(), a)
    # compute on the moved tensor, then bring the result back: the D2H copy is ordered behind the kernel
    out = tb.einsum("asc,asd->cd", [dev, dev.into_conj()])
    back = out.to_memory_space_async(main)
    assert back.logical_memory_space() == main
    back.wait()
    want = np.einsum("asc,asd->cd", a, np.conj(a))
    assert oracle.rel_frobenius(back.to_numpy(), want) <= 1e-12


def test_same_space_is_zero_copy(tb):
    gpu = tb.LogicalMemorySpace.GpuMemory(0)
    t = tb.Tensor.from_numpy(np.arange(12.0).reshape(3, 4))
    assert t.to_memory_space_async(gpu) is t
    h = tb.Tensor.from_numpy(np.arange(6.0), memory_space=tb.LogicalMemorySpace.MainMemory())
    assert h.to_memory_space_async(tb.LogicalMemorySpace.MainMemory()) is h


def test_strided_view_moves_as_its_logical_contents(tb):
    rng = np.random.default_rng(301)
    a = random_array(rng, (20, 30), np.float32)
    t = tb.Tensor.from_numpy(a).permute([1, 0])  # a non-contiguous view
    back = t.to_memory_space_async(tb.LogicalMemorySpace.MainMemory())
    assert np.array_equal(back.to_numpy(), a.T)


def test_main_memory_tensors_do_not_compute(tb):
    main = tb.LogicalMemorySpace.MainMemory()
    a = tb.Tensor.from_numpy(np.ones((3, 4)), memory_space=main)
    b = tb.Tensor.from_numpy(np.ones((4, 5)), memory_space=main)
    with pytest.raises(tb.NoCompatibleComputeDevice):
        tb.einsum("ij,jk->ik", [a, b])
    with pytest.raises(tb.CrossMemorySpaceOperation):
        tb.einsum("ij,jk->ik", [a, tb.Tensor.from_numpy(np.ones((4, 5)))])
    plan = tb.CudaBackend.plan(tb.PrimDescriptor.Permute([0, 1], [1, 0]), [(3, 4), (4, 3)], np.float64)
    with pytest.raises(tb.NoCompatibleComputeDevice):
        tb.CudaBackend.execute(plan, 1.0, [a], 0.0, tb.Tensor.zeros((4, 3), memory_space=main))


def test_views_share_the_completion_event_of_their_buffer(tb):
    """A view taken BEFORE a write to its parent must see that write's event: the event belongs to
    the storage, not to the view object."""
    out = tb.Tensor.zeros((64, 64), dtype=np.float64)
    view = out.permute([1, 0])
    first = view.event
    a = tb.Tensor.from_numpy(np.eye(64))
    tb.einsum_into("ij,jk->ik", [a, a], 1.0, 0.0, out)
    assert out.event is not None and view.event is out.event and view.event is not first
    moved = view.to_memory_space_async(tb.LogicalMemorySpace.MainMemory())
    assert np.array_equal(moved.to_numpy(), np.eye(64))


def test_gpu_to_gpu_over_nvlink(tb, oracle):
    """GpuMemory{0} -> GpuMemory{1}: a plain peer copy on the destination's stream, ordered behind
    the producer on the source's stream by its completion event."""
    import torch

    if torch.cuda.device_count() < 2:
        pytest.skip("needs two visible GPUs")
    rng = np.random.default_rng(302)
    a, b = random_array(rng, (300, 200), np.float64), random_array(rng, (200, 260), np.float64)
    g0, g1 = tb.LogicalMemorySpace.GpuMemory(0), tb.LogicalMemorySpace.GpuMemory(1)
    prod = tb.einsum("ij,jk->ik", [tb.Tensor.from_numpy(a, memory_space=g0), tb.Tensor.from_numpy(b, memory_space=g0)])
    there = prod.to_memory_space_async(g1)  # enqueued right behind the product, no host wait
    assert there.logical_memory_space() == g1
    twice = tb.einsum("ik,ik->ik", [there, there])  # computed on GPU 1
    assert oracle.rel_frobenius(there.to_numpy(), a @ b) <= 1e-12
    assert oracle.rel_frobenius(twice.to_numpy(), (a @ b) ** 2) <= 1e-12
    with pytest.raises(tb.CrossMemorySpaceOperation):
        tb.einsum("ik,ik->ik", [there, prod])


# ---------------------------------------------------------------- pool, contexts, streams
def test_capped_pool_reports_device_error_and_recovers(tb):
    """TFB_POOL_BYTES caps the pool of contexts created while it is set: an allocation past the cap
    fails with DeviceError, and the very next call on the same context works."""
    os.environ["TFB_POOL_BYTES"] = str(64 << 20)
    try:
        ctx = tb.Context(0)  # a context of its own, with its own pool
    finally:
        os.environ.pop("TFB_POOL_BYTES", None)
    small = ctx.alloc(16 << 20)
    with pytest.raises(tb.DeviceError, match="pool allocation"):
        ctx.alloc(256 << 20)
    again = ctx.alloc(16 << 20)
    ctx.memset(again, 0, 16 << 20)
    ctx.synchronize()
    ctx.free(small)
    ctx.free(again)
    ctx.synchronize()
    reserved, used = ctx.pool_stats()
    assert used == 0 and reserved <= 64 << 20


def test_first_use_of_a_layout_on_one_stream_then_another(tb, oracle):
    """The offset tables of a layout are built by kernels on the stream that first needs them.  A
    second context (another stream) that hits the cache right afterwards must wait for that build."""
    rng = np.random.default_rng(303)
    # a layout no other test uses: odd extents and strides, so the tables are certainly new
    a, b = random_array(rng, (7, 131, 59), np.float64), random_array(rng, (59, 7, 113), np.float64)
    want = np.einsum("bmk,kbn->nmb", a, b)
    other = tb.Context(0)
    plan_x = tb.CudaBackend.plan(tb.PrimDescriptor.Contract([0, 1, 2], [2, 0, 3], [3, 1, 0]),
                                 [a.shape, b.shape, want.shape], np.float64)
    plan_y = tb.CudaBackend.plan(tb.PrimDescriptor.Contract([0, 1, 2], [2, 0, 3], [3, 1, 0]),
                                 [a.shape, b.shape, want.shape], np.float64, ctx=other)
    ta, tb_ = tb.Tensor.from_numpy(a), tb.Tensor.from_numpy(b)
    cx, cy = tb.Tensor.zeros(want.shape), tb.Tensor.zeros(want.shape)
    tb.Context.get(0).synchronize()
    tb.CudaBackend.execute(plan_x, 1.0, [ta, tb_], 0.0, cx)   # misses the cache: builds on stream X
    tb.CudaBackend.execute(plan_y, 1.0, [ta, tb_], 0.0, cy)   # hits it at once, on stream Y
    other.synchronize()
    assert oracle.rel_frobenius(cx.to_numpy(), want) <= 1e-12
    assert oracle.rel_frobenius(cy.to_numpy(), want) <= 1e-12


def test_set_stream_orders_the_new_stream_behind_the_old(tb, oracle):
    import torch

    ctx = tb.Context(0)
    rng = np.random.default_rng(304)
    a = random_array(rng, (512, 512), np.float64)
    ta = tb.Tensor.from_numpy(a)
    out1, out2 = tb.Tensor.zeros((512, 512)), tb.Tensor.zeros((512, 512))
    plan = tb.CudaBackend.plan(tb.PrimDescriptor.Contract([0, 1], [1, 2], [0, 2]), [(512, 512)] * 3, np.float64, ctx=ctx)
    s2 = torch.cuda.Stream(device=0)
    tb.Context.get(0).synchronize()
    tb.CudaBackend.execute(plan, 1.0, [ta, ta], 0.0, out1)        # on the context's own stream
    ctx.set_stream(s2.cuda_stream)
    tb.CudaBackend.execute(plan, 1.0, [out1, ta], 0.0, out2)      # reads out1 from the other stream
    ctx.synchronize()
    ctx.set_stream(None)
    assert oracle.rel_frobenius(out2.to_numpy(), a @ a @ a) <= 1e-12


def test_pitched_copies(tb):
    ctx = tb.Context.get(0)
    rng = np.random.default_rng(305)
    host = rng.integers(0, 255, size=(40, 96), dtype=np.uint8)      # 40 rows, pitch 96
    dev = ctx.alloc(40 * 64)
    ctx.h2d_2d(dev, 64, host.ctypes.data_as(C.c_void_p), 96, 48, 40)  # 48 bytes of every row, device pitch 64
    back = np.zeros((40, 80), dtype=np.uint8)
    ctx.d2h_2d(back.ctypes.data_as(C.c_void_p), 80, dev, 64, 48, 40)
    ctx.synchronize()
    ctx.free(dev)
    assert np.array_equal(back[:, :48], host[:, :48]) and not back[:, 48:].any()
    with pytest.raises(tb.InvalidArgument):
        ctx.h2d_2d(dev, 16, host.ctypes.data_as(C.c_void_p), 96, 48, 40)


# ---------------------------------------------------------------- bounded waits
def test_a_bounded_wait_runs_out_and_the_context_survives(tb, oracle):
    """One CTA waits, for at most 4096 polls, on an mbarrier nothing arrives on.  The wait gives up,
    the kernel records its code and returns; synchronize() reports DeviceError with that code,
    clears it, and an ordinary contraction on the same context then succeeds."""
    ctx = tb.Context.get(0)
    ctx.synchronize()
    ctx.selftest_wait_expiry(4096)
    with pytest.raises(tb.DeviceError, match="0x7e57"):
        ctx.synchronize()
    ctx.synchronize()  # the status word was cleared
    rng = np.random.default_rng(306)
    a, b = random_array(rng, (300, 280), np.float32), random_array(rng, (280, 290), np.float32)
    got = tb.einsum("ij,jk->ik", [tb.Tensor.from_numpy(a), tb.Tensor.from_numpy(b)]).to_numpy()
    assert oracle.rel_frobenius(got, a.astype(np.float64) @ b.astype(np.float64)) <= 1e-5
    with pytest.raises(tb.InvalidArgument):
        ctx.selftest_wait_expiry(0)


# ---------------------------------------------------------------- complex products with badly scaled parts
def test_complex128_imaginary_part_alone(tb, oracle):
    """Re ~ N(0,1), Im ~ 1e-8 N(0,1).  The default Complex64 kernel forms a complex product from
    three real ones: the result is exact to 1e-12 of its norm, but its imaginary part alone keeps
    only about half its digits.  Kernel 4 (four real products) keeps the imaginary part to
    1e-12 of ITS norm.  Both facts are asserted, so the documented trade-off stays true."""
    rng = np.random.default_rng(307)
    m = n = 256
    k = 1024
    a = (rng.standard_normal((m, k)) + 1e-8j * rng.standard_normal((m, k))).astype(np.complex128)
    b = (rng.standard_normal((k, n)) + 1e-8j * rng.standard_normal((k, n))).astype(np.complex128)
    # reference in extended precision: the four real products in longdouble
    L = np.longdouble
    ar, ai, br, bi = a.real.astype(L), a.imag.astype(L), b.real.astype(L), b.imag.astype(L)
    want_re = (ar @ br - ai @ bi).astype(np.float64)
    want_im = (ar @ bi + ai @ br).astype(np.float64)
    ta, tb_ = tb.Tensor.from_numpy(a), tb.Tensor.from_numpy(b)
    desc = tb.PrimDescriptor.Contract([0, 1], [1, 2], [0, 2])
    errs = {}
    for name, kernel in (("three", tb.ContractKernel.Dmma), ("four", tb.ContractKernel.Dmma4)):
        plan = tb.CudaBackend.plan(desc, [(m, k), (k, n), (m, n)], np.complex128)
        plan.force_kernel(kernel)
        out = tb.Tensor.zeros((m, n), dtype=np.complex128)
        tb.CudaBackend.execute(plan, 1.0, [ta, tb_], 0.0, out)
        got = out.to_numpy()
        errs[name] = (oracle.rel_frobenius(got, want_re + 1j * want_im),
                      oracle.rel_frobenius(got.imag, want_im))
    print("complex128 badly scaled parts: (norm-wise, imaginary part alone)", errs)
    assert errs["three"][0] <= 1e-12 and errs["four"][0] <= 1e-12   # the contract's tolerance, both
    assert errs["four"][1] <= 1e-12                                  # four products: Im to its own size
    assert errs["three"][1] <= 1e-6                                  # three products: Im keeps ~half its digits


def test_mma_issue_probe_reports_plausible_clocks(tb):
    """tfb_probe_mma_issue_cycles: a small tcgen05.mma costs its issuing thread tens of clocks, more
    issuers shorten the time per MMA of the CTA, and shapes the probe does not take are refused."""
    ctx = tb.Context.get(0)
    issue1, done1 = ctx.probe_mma_issue_cycles(128, 16, 1)
    issue2, done2 = ctx.probe_mma_issue_cycles(128, 16, 2)
    assert 20.0 <= issue1 <= 400.0 and 20.0 <= done1 <= 400.0, (issue1, done1)
    assert done2 < done1, (done1, done2)
    big, _ = ctx.probe_mma_issue_cycles(128, 256, 1)
    assert big >= 100.0, big  # 128 x 256 x 8 is 128 clocks of tensor-pipe work
    for bad in ((96, 16, 1), (128, 24, 1), (128, 256, 2), (128, 16, 5)):
        with pytest.raises(tb.InvalidArgument):
            ctx.probe_mma_issue_cycles(*bad)
    ctx.synchronize()


def test_capture_and_replay_of_a_contraction_sequence(tb, oracle):
    """tfb_ctx_capture_begin / _end / tfb_graph_launch: a sequence that ran once is captured (nothing runs
    while capturing), the graph's replays redo it on the buffers' current contents, and calls that
    make no sense while capturing are refused.  The f64 product is one whose K is split over the
    CTAs (two launches), the chain step one that uses the in-kernel stream-K reduction."""
    ctx = tb.Context.get(0)
    a, b = oracle.normal(9100, (64, 64, 64), np.float64), oracle.normal(9101, (64, 64, 64), np.float64)
    A, B = tb.Tensor.from_numpy(a), tb.Tensor.from_numpy(b)
    out = tb.Tensor.zeros([64, 64], dtype=np.float64)
    tree = tb.ContractionTree.optimize(tb.Subscripts.parse("abc,bcd->ad"), [a.shape, b.shape])
    chi = 256
    e0 = oracle.normal(9102, (chi, chi), np.complex128)
    s0 = oracle.normal(9103, (chi, 2, chi), np.complex128, scale=(1.0 / chi) ** 0.5)
    E, S = tb.Tensor.from_numpy(e0), tb.Tensor.from_numpy(s0)
    Sc = S.conj()
    nxt = tb.Tensor.zeros([chi, chi], dtype=np.complex128)
    tree3 = tb.ContractionTree.optimize(tb.Subscripts.parse("ab,asc,bsd->cd"), [e0.shape, s0.shape, s0.shape])

    def sequence():
        tb.einsum_with_plan_into(tree, [A, B], 1.0, 0.0, out)
        tb.einsum_with_plan_into(tree3, [E, S, Sc], 1.0, 0.0, nxt)

    sequence()  # first use: plans, tables, kernel attributes
    ctx.synchronize()
    want_out, want_nxt = out.to_numpy(), nxt.to_numpy()
    assert oracle.rel_frobenius(want_out, np.einsum("abc,bcd->ad", a, b)) <= 1e-12
    ctx.memset(out._block.ptr, 0, out._block.nbytes)
    ctx.memset(nxt._block.ptr, 0, nxt._block.nbytes)
    ctx.synchronize()

    ctx.capture_begin()
    with pytest.raises(tb.InvalidArgument):
        ctx.synchronize()
    with pytest.raises(tb.InvalidArgument):
        ctx.capture_begin()
    sequence()
    graph = ctx.capture_end()
    ctx.synchronize()
    assert not out.to_numpy().any() and not nxt.to_numpy().any()  # capturing ran nothing

    for _ in range(3):  # replays, the stream-K flags of the last run still raised
        graph.launch()
    ctx.synchronize()
    assert np.array_equal(out.to_numpy(), want_out)
    assert np.array_equal(nxt.to_numpy(), want_nxt)

    # a replay reads the operands as they are now
    a2 = oracle.normal(9104, (64, 64, 64), np.float64)
    a2_col = np.ascontiguousarray(a2.ravel(order="F"))  # tensors are stored column-major
    ctx.h2d(A._block.ptr, a2_col.ctypes.data_as(C.c_void_p), a2_col.nbytes)
    graph.launch()
    ctx.synchronize()
    assert oracle.rel_frobenius(out.to_numpy(), np.einsum("abc,bcd->ad", a2, b)) <= 1e-12
    with pytest.raises(tb.InvalidArgument):
        ctx.capture_end()  # not capturing
