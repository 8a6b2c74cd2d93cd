"""A trailing element-wise multiplication fused into the product that feeds it.

A tree node without summed labels whose one operand is the product of the node before it (for
example the last step of 'ij,jk,ik->ik' ordered as [(0,1),(2,3)]) runs inside that product's
epilogue: C = alpha * (A B) . D + beta * C in one kernel, no intermediate tensor.  Checked
against the oracle for every dtype and kernel family, against the unfused execution of the
same tree, and by the kernel-launch counter (the fused tree launches fewer kernels)."""
import os

import numpy as np
import pytest

from conftest import ALL_DTYPES, TOL, random_array

pytestmark = pytest.mark.gpu


def _run(tb, notation, arrays, pairs, alpha=1.0, beta=0.0, out=None, conj=()):
    subs = tb.Subscripts.parse(notation)
    tree = tb.ContractionTree.from_pairs(subs, [a.shape for a in arrays], pairs)
    ops = [tb.Tensor.from_numpy(a) for a in arrays]
    for i in conj:
        ops[i] = ops[i].into_conj()
    if out is None:
        return tb.einsum_with_plan(tree, ops).to_numpy()
    o = tb.Tensor.from_numpy(out)
    tb.einsum_with_plan_into(tree, ops, alpha, beta, o)
    return o.to_numpy()


def _launches(tb, fn):
    tb.Context.get(0).synchronize()
    before = tb.Context.kernel_launch_count()
    r = fn()
    return r, tb.Context.kernel_launch_count() - before


@pytest.fixture
def unfused():
    """Runs the body of a `with` block with the fusion switched off."""
    class Off:
        def __enter__(self):
            os.environ["TFB_EINSUM_FUSE_MUL"] = "0"

        def __exit__(self, *exc):
            os.environ.pop("TFB_EINSUM_FUSE_MUL", None)
    return Off()


# (notation, shapes, pairs): the last pair multiplies the product by an operand over (a subset of) its labels
CASES = [
    ("ij,jk,ik->ik", [(70, 50), (50, 90), (70, 90)], [(0, 1), (2, 3)]),          # small: exact kernels
    ("ij,jk,ik->ki", [(300, 200), (200, 260), (300, 260)], [(0, 1), (2, 3)]),    # tensor cores, transposed output
    ("ij,jk,k->ik", [(256, 512), (512, 384), (384,)], [(0, 1), (2, 3)]),         # multiplier broadcast along i
    ("ij,jk,i->ik", [(256, 512), (512, 384), (256,)], [(0, 1), (3, 2)]),         # ... along k, product on the right
    ("bij,bjk,bik->bik", [(3, 130, 64), (3, 64, 140), (3, 130, 140)], [(0, 1), (2, 3)]),
    ("ijl,jlk,ik->ik", [(257, 8, 33), (8, 33, 300), (257, 300)], [(0, 1), (2, 3)]),
    ("ij,jk,ki->ik", [(700, 96), (96, 900), (900, 700)], [(0, 1), (2, 3)]),      # short K: the drain warps multiply
]


@pytest.mark.parametrize("dtype", ALL_DTYPES)
@pytest.mark.parametrize("case", CASES, ids=[c[0] for c in CASES])
def test_fused_multiplier_matches_oracle_and_unfused(tb, oracle, unfused, dtype, case):
    notation, shapes, pairs = case
    rng = np.random.default_rng(91)
    arrays = [random_array(rng, s, dtype) for s in shapes]
    want = oracle.np_einsum(notation, arrays)
    got, n_fused = _launches(tb, lambda: _run(tb, notation, arrays, pairs))
    assert got.shape == want.shape
    assert oracle.rel_frobenius(got, want) <= TOL[np.dtype(dtype)]
    with unfused:
        ref, n_plain = _launches(tb, lambda: _run(tb, notation, arrays, pairs))
    assert oracle.rel_frobenius(ref, want) <= TOL[np.dtype(dtype)]
    # second runs: offset tables are cached, so the counts compare the kernels proper
    _, n_fused = _launches(tb, lambda: _run(tb, notation, arrays, pairs))
    with unfused:
        _, n_plain = _launches(tb, lambda: _run(tb, notation, arrays, pairs))
    if np.dtype(dtype) != np.complex64:  # complex64 multiplies in place after the product: no launch saved
        assert n_fused < n_plain, (n_fused, n_plain)


@pytest.mark.parametrize("dtype", ALL_DTYPES)
def test_fused_multiplier_with_accumulate_and_conj(tb, oracle, dtype):
    # output = alpha * einsum + beta * output with the fused node last; the multiplier conjugated lazily
    rng = np.random.default_rng(92)
    a, b, d = (random_array(rng, s, dtype) for s in ((192, 300), (300, 200), (192, 200)))
    old = random_array(rng, (192, 200), dtype)
    cplx = np.issubdtype(np.dtype(dtype), np.complexfloating)
    alpha, beta = (0.5 - 0.25j, -1.5 + 2j) if cplx else (0.5, -1.5)
    dd = np.conj(d) if cplx else d
    want = alpha * oracle.np_einsum("ij,jk,ik->ik", [a, b, dd]) + beta * old.astype(np.complex128 if cplx else np.float64)
    got = _run(tb, "ij,jk,ik->ik", [a, b, d], [(0, 1), (2, 3)], alpha, beta, old.copy(), conj=(2,) if cplx else ())
    assert oracle.rel_frobenius(got, want) <= 2 * TOL[np.dtype(dtype)]


def test_fused_multiplier_in_the_middle_of_a_tree(tb, oracle, unfused):
    # (A B) . D feeds a further product: the fused result is an intermediate
    rng = np.random.default_rng(93)
    shapes = [(140, 96), (96, 150), (140, 150), (150, 40)]
    arrays = [random_array(rng, s, np.float64) for s in shapes]
    notation, pairs = "ij,jk,ik,kl->il", [(0, 1), (2, 4), (5, 3)]
    want = oracle.np_einsum(notation, arrays)
    got, n_fused = _launches(tb, lambda: _run(tb, notation, arrays, pairs))
    with unfused:
        ref, n_plain = _launches(tb, lambda: _run(tb, notation, arrays, pairs))
    assert oracle.rel_frobenius(got, want) <= 1e-12 and oracle.rel_frobenius(ref, want) <= 1e-12
    _, n_fused = _launches(tb, lambda: _run(tb, notation, arrays, pairs))  # offset tables cached by now
    with unfused:
        _, n_plain = _launches(tb, lambda: _run(tb, notation, arrays, pairs))
    assert n_fused < n_plain


def test_not_fused_when_the_consumer_sums_or_the_multiplier_comes_later(tb, oracle):
    rng = np.random.default_rng(94)
    # the consumer sums k away: a contraction, not an element-wise node
    arrays = [random_array(rng, s, np.float64) for s in ((40, 30), (30, 50), (40, 50))]
    got = _run(tb, "ij,jk,ik->i", arrays, [(0, 1), (2, 3)])
    assert oracle.rel_frobenius(got, oracle.np_einsum("ij,jk,ik->i", arrays)) <= 1e-12
    # the other operand of the element-wise node is itself computed after the product
    arrays = [random_array(rng, s, np.float64) for s in ((40, 30), (30, 50), (40, 20), (20, 50))]
    got = _run(tb, "ij,jk,il,lk->ik", arrays, [(0, 1), (2, 3), (4, 5)])
    assert oracle.rel_frobenius(got, oracle.np_einsum("ij,jk,il,lk->ik", arrays)) <= 1e-12
    # ... and computed before it: fused
    got = _run(tb, "ij,jk,il,lk->ik", arrays, [(2, 3), (0, 1), (5, 4)])
    assert oracle.rel_frobenius(got, oracle.np_einsum("ij,jk,il,lk->ik", arrays)) <= 1e-12


@pytest.mark.parametrize("dtype", ALL_DTYPES)
def test_summed_labels_of_extent_one_take_the_unfused_path(tb, oracle, dtype):
    """A summed label of extent 1 vanishes when the modes are fused, so the product has nothing to
    sum and cannot carry a multiplier: such a tree must run (unfused) and give the same result."""
    rng = np.random.default_rng(95)
    # j = 1: 'ij,jk' is an outer product
    arrays = [random_array(rng, s, dtype) for s in ((60, 1), (1, 70), (60, 70))]
    got = _run(tb, "ij,jk,ik->ik", arrays, [(0, 1), (2, 3)])
    assert oracle.rel_frobenius(got, oracle.np_einsum("ij,jk,ik->ik", arrays)) <= TOL[np.dtype(dtype)]
    # batched product whose every summed label has extent 1
    arrays = [random_array(rng, s, dtype) for s in ((3, 40, 1, 1), (3, 1, 1, 50), (3, 40, 50))]
    got = _run(tb, "bijl,bjlk,bik->bik", arrays, [(0, 1), (2, 3)])
    assert oracle.rel_frobenius(got, oracle.np_einsum("bijl,bjlk,bik->bik", arrays)) <= TOL[np.dtype(dtype)]
    # one summed label of extent 1 beside a real one: still fused, still right
    arrays = [random_array(rng, s, dtype) for s in ((40, 1, 30), (1, 30, 50), (40, 50))]
    got = _run(tb, "ijl,jlk,ik->ik", arrays, [(0, 1), (2, 3)])
    assert oracle.rel_frobenius(got, oracle.np_einsum("ijl,jlk,ik->ik", arrays)) <= TOL[np.dtype(dtype)]
