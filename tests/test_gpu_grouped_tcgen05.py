"""The tcgen05 form of the grouped product (tfb_grouped_gemm / tfb_grouped_plan_*): ragged tables
of column-major f32 problems against the float64 oracle at relative Frobenius 1e-5, with the
kernel that ran read back from the launch profile.  It is the kernel for tables the mma.sync kernel
declines (dims that are not multiples of 16, K above 128) and can be asked for first with
TFB_GROUPED_PREFER_TCGEN05=1.  Covers what its planner branches on: dims that are not multiples of
the 32-wide boxes, pitched columns, problems of several 128 x 128 units, K from 1 to the longest
chain the path takes, alpha / beta, a table longer than the barrier ring, and tables the path
must decline (the SIMT kernel then takes them)."""
import os

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def kernel_that_ran(ctx, fn, prefer_tcgen05=False):
    """Runs fn (which builds the plan: the preference is read then) and names the grouped kernels launched."""
    if prefer_tcgen05:
        os.environ["TFB_GROUPED_PREFER_TCGEN05"] = "1"
    try:
        ctx.profile_begin()
        fn()
        ctx.synchronize()
        names = [nm for nm in ("grouped_tcgen05", "grouped_tf32x3", "grouped_simt") if ctx.profile_read(nm)[0] > 0]
        ctx.profile_end()
    finally:
        os.environ.pop("TFB_GROUPED_PREFER_TCGEN05", None)
    return names


def build(tb, oracle, table, seed, pitched=False, c_init=False):
    """table: (m, n, k) per problem.  Returns (held tensors, problem tuples, float64 products, C before)."""
    held, probs, wants, before = [], [], [], []
    for p, (m, n, k) in enumerate(table):
        a = oracle.uniform(seed + 3 * p, (m, k), np.float32)
        b = oracle.uniform(seed + 3 * p + 1, (k, n), np.float32)
        a_cs = (m + 3) // 4 * 4 + (8 if pitched else 0) if (pitched or m % 4) else m
        b_cs = (k + 3) // 4 * 4 + (4 if pitched else 0) if (pitched or k % 4) else k
        c_cs = m + (5 if pitched else 0)
        # tensors are stored column-major: element (i, j) of a (cs, cols) array sits at i + j * cs, so
        # the rows beyond the problem's are the pitch between columns
        a_buf = np.full((a_cs, k), np.nan, np.float32)
        a_buf[:m] = a
        b_buf = np.full((b_cs, n), np.nan, np.float32)
        b_buf[:k] = b
        c0 = oracle.uniform(seed + 3 * p + 2, (c_cs, n), np.float32) if c_init else np.full((c_cs, n), 7.0, np.float32)
        ta, tb_, tc = tb.Tensor.from_numpy(a_buf), tb.Tensor.from_numpy(b_buf), tb.Tensor.from_numpy(c0)
        held += [ta, tb_, tc]
        probs.append((m, n, k, ta._block.ptr, 1, a_cs, tb_._block.ptr, 1, b_cs, tc._block.ptr, 1, c_cs))
        wants.append(oracle.np_batched_gemm(a, b))
        before.append(c0)
    return held, probs, wants, before


def check(oracle, held, table, wants, before, alpha, beta):
    num = den = 0.0
    for p, (m, n, k) in enumerate(table):
        got = held[3 * p + 2].to_numpy()  # (c_cs, n)
        want = alpha * wants[p] + beta * before[p][:m].astype(np.float64)
        err = oracle.rel_frobenius(got[:m], want)
        assert err <= 1e-5, (p, (m, n, k), err)
        # the padding between columns is not the kernel's to write
        assert np.array_equal(got[m:], before[p][m:]), (p, (m, n, k))
        num += np.linalg.norm(got[:m].astype(np.float64) - want) ** 2
        den += np.linalg.norm(want) ** 2
    assert (num / den) ** 0.5 <= 1e-5


def test_ragged_table_runs_on_tcgen05(tb, oracle):
    table = [tuple(int(x) for x in (r[0], r[2], r[1])) for r in oracle.grouped_table(3300, 600)]  # (i, j, k) -> (m, n, k)
    held, probs, wants, before = build(tb, oracle, table, 33000)
    ctx = tb.Context.get(0)
    names = kernel_that_ran(ctx, lambda: tb.grouped_gemm(probs, np.float32, 1.0, 0.0, ctx), prefer_tcgen05=True)
    assert names == ["grouped_tcgen05"], names
    check(oracle, held, table, wants, before, 1.0, 0.0)


@pytest.mark.parametrize("pitched", [False, True])
def test_edges_tiles_and_depths(tb, oracle, pitched):
    table = [(1, 1, 1), (4, 4, 4), (16, 16, 16), (50, 70, 33), (128, 128, 128), (129, 127, 31), (300, 200, 100),
             (20, 260, 512), (260, 20, 257), (96, 48, 8), (33, 16, 40), (12, 130, 96), (128, 16, 512), (8, 8, 300)]
    held, probs, wants, before = build(tb, oracle, table, 34000, pitched=pitched)
    ctx = tb.Context.get(0)
    names = kernel_that_ran(ctx, lambda: tb.grouped_gemm(probs, np.float32, 1.0, 0.0, ctx))
    assert names == ["grouped_tcgen05"], names
    check(oracle, held, table, wants, before, 1.0, 0.0)


def test_alpha_beta_and_second_run(tb, oracle):
    table = [(64, 32, 48), (16, 128, 128), (100, 36, 64), (128, 128, 16), (40, 40, 200)] * 5
    held, probs, wants, before = build(tb, oracle, table, 35000, pitched=True, c_init=True)
    os.environ["TFB_GROUPED_PREFER_TCGEN05"] = "1"
    try:
        plan = tb.PreparedGroupedGemm(probs, np.float32, alpha=0.5, beta=-2.0)
    finally:
        del os.environ["TFB_GROUPED_PREFER_TCGEN05"]
    ctx = tb.Context.get(0)
    names = kernel_that_ran(ctx, plan.run)
    assert names == ["grouped_tcgen05"], names
    check(oracle, held, table, wants, before, 0.5, -2.0)
    mid = [held[3 * p + 2].to_numpy() for p in range(len(table))]
    plan.run()
    ctx.synchronize()
    check(oracle, held, table, wants, mid, 0.5, -2.0)


def test_many_small_stages_wrap_the_barrier_ring(tb, oracle):
    """More stages per CTA than barrier sets, all of them small: on a table of 148 x 40 tiny
    problems every CTA laps its ring of barrier sets and of bytes."""
    rng = np.random.default_rng(36)
    sm = tb.Context.get(0).sm_count if hasattr(tb.Context.get(0), "sm_count") else 148
    table = [(int(rng.choice([8, 16, 24])), int(rng.choice([8, 16, 40])), int(rng.choice([8, 16, 64]))) for _ in range(sm * 40)]
    held, probs, wants, before = build(tb, oracle, table, 36000)
    ctx = tb.Context.get(0)
    names = kernel_that_ran(ctx, lambda: tb.grouped_gemm(probs, np.float32, 1.0, 0.0, ctx), prefer_tcgen05=True)
    assert names == ["grouped_tcgen05"], names
    check(oracle, held, table, wants, before, 1.0, 0.0)


def test_agrees_with_the_mma_sync_kernel(tb, oracle):
    table = [tuple(int(x) for x in (r[0], r[2], r[1])) for r in oracle.grouped_table(3700, 200)]
    held, probs, wants, before = build(tb, oracle, table, 37000)
    ctx = tb.Context.get(0)
    names = kernel_that_ran(ctx, lambda: tb.grouped_gemm(probs, np.float32, 1.0, 0.0, ctx), prefer_tcgen05=True)
    assert names == ["grouped_tcgen05"], names
    first = [held[3 * p + 2].to_numpy() for p in range(len(table))]
    names = kernel_that_ran(ctx, lambda: tb.grouped_gemm(probs, np.float32, 1.0, 0.0, ctx))
    assert names == ["grouped_tf32x3"], names  # the default for a table of multiples of 16
    for p in range(len(table)):
        assert oracle.rel_frobenius(held[3 * p + 2].to_numpy(), first[p].astype(np.float64)) <= 1e-5, p


def test_declines_what_tma_cannot_describe(tb, oracle):
    """A column pitch that is not a multiple of 16 bytes, or K beyond the chain the path
    accumulates in tensor memory: the table goes to another kernel, with the same answer."""
    ctx = tb.Context.get(0)
    for table, other in (([(16, 16, 16), (7, 13, 5)], "grouped_simt"), ([(32, 32, 1024), (64, 64, 64)], "grouped_simt")):
        held, probs, wants, before = build(tb, oracle, table, 38000)
        if table[1] == (7, 13, 5):
            # rebuild the odd problem with unpadded columns (pitch 7 floats)
            m, n, k = table[1]
            a, b = oracle.uniform(1, (m, k), np.float32), oracle.uniform(2, (k, n), np.float32)
            ta, tb_ = tb.Tensor.from_numpy(a), tb.Tensor.from_numpy(b)
            held[3], held[4] = ta, tb_
            probs[1] = (m, n, k, ta._block.ptr, 1, m, tb_._block.ptr, 1, k, held[5]._block.ptr, 1, m)
            wants[1] = oracle.np_batched_gemm(a, b)
        names = kernel_that_ran(ctx, lambda: tb.grouped_gemm(probs, np.float32, 1.0, 0.0, ctx))
        assert names == [other], (names, table)
        check(oracle, held, table, wants, before, 1.0, 0.0)
