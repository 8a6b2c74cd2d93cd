"""Host-side logic that needs no GPU: notation parsing, contraction trees, descriptor
validation and the zero-copy view rules.  Known answers are the ones the reference's doc
examples state (file:line in each test)."""
import numpy as np
import pytest


# ---------------------------------------------------------------- Subscripts
def test_subscripts_new(tb):
    # tenferro-einsum/src/lib.rs:222-229
    subs = tb.Subscripts.new([[0, 1], [1, 2]], [0, 2])
    assert len(subs.inputs) == 2
    assert subs.output == [0, 2]


def test_subscripts_parse_matmul(tb):
    # tenferro-einsum/src/lib.rs:231-236
    subs = tb.Subscripts.parse("ij,jk->ik")
    assert len(subs.inputs) == 2
    i, j, k = 8, 9, 10
    assert subs.inputs == [[i, j], [j, k]] and subs.output == [i, k]
    assert not subs.has_order


@pytest.mark.parametrize("notation,n_in,out_len", [("ii->i", 1, 1), ("ijk->", 1, 0), ("ij,(jk,kl)->il", 3, 2),
                                                   ("i->iii", 1, 3), ("bij,jk->bik", 2, 3), ("aB,Bc->ac", 2, 2)])
def test_subscripts_parse_forms(tb, notation, n_in, out_len):
    # tenferro-einsum/src/lib.rs:266-276
    subs = tb.Subscripts.parse(notation)
    assert len(subs.inputs) == n_in and len(subs.output) == out_len


def test_subscripts_upper_case_distinct(tb):
    subs = tb.Subscripts.parse("aA->Aa")
    assert subs.inputs == [[0, 26]] and subs.output == [26, 0]


@pytest.mark.parametrize("bad", ["ij,(jk->ik", "ij,jk)->ik", "ij,jk-ik", "ij,j1->i", "ij->ik", "ij,jk->i k!"])
def test_subscripts_parse_errors(tb, bad):
    with pytest.raises(tb.InvalidArgument):
        tb.Subscripts.parse(bad)


# ---------------------------------------------------------------- ContractionTree
def test_from_pairs_doc_example(tb):
    # tenferro-einsum/src/lib.rs:330-343: B*C -> T(index 3), then A*T
    subs = tb.Subscripts.new([[0, 1], [1, 2], [2, 3]], [0, 3])
    tree = tb.ContractionTree.from_pairs(subs, [[3, 4], [4, 5], [5, 6]], [(1, 2), (0, 3)])
    assert tree.pairs == [(1, 2), (0, 3)]
    assert tree.output_dims == [3, 6]
    assert tree.macs == 4 * 5 * 6 + 3 * 4 * 6


def test_from_pairs_rejects_bad_sequences(tb):
    subs = tb.Subscripts.new([[0, 1], [1, 2], [2, 3]], [0, 3])
    shapes = [[3, 4], [4, 5], [5, 6]]
    for pairs in ([(1, 2)], [(1, 2), (1, 3)], [(0, 0), (1, 2)], [(1, 2), (0, 4)]):
        with pytest.raises(tb.InvalidArgument):
            tb.ContractionTree.from_pairs(subs, shapes, pairs)


def test_optimize_avoids_large_intermediate(tb):
    # tenferro-einsum/src/lib.rs:108-121: with shapes 3x4, 4x100, 100x5 contract B*C first.
    subs = tb.Subscripts.parse("ij,jk,kl->il")
    tree = tb.ContractionTree.optimize(subs, [[3, 4], [4, 100], [100, 5]])
    assert tree.pairs[0] == (1, 2)


def test_parentheses_fix_the_order(tb):
    subs = tb.Subscripts.parse("(ij,jk),kl->il")
    tree = tb.ContractionTree.optimize(subs, [[3, 4], [4, 100], [100, 5]])
    assert tree.pairs == [(0, 1), (3, 2)]


def test_optimize_shape_errors(tb):
    subs = tb.Subscripts.parse("ij,jk->ik")
    with pytest.raises(tb.ShapeMismatch):
        tb.ContractionTree.optimize(subs, [[3, 4], [5, 6]])
    with pytest.raises(tb.RankMismatch):
        tb.ContractionTree.optimize(subs, [[3, 4, 2], [4, 6]])


def test_optimize_matches_exhaustive_search(tb, oracle):
    rng = np.random.default_rng(7)
    letters = list(range(8))
    for trial in range(30):
        n = int(rng.integers(2, 6))
        inputs = [list(rng.choice(letters, size=int(rng.integers(1, 4)), replace=False)) for _ in range(n)]
        seen = sorted({l for t in inputs for l in t})
        output = [l for l in seen if rng.random() < 0.35]
        ext = {l: int(rng.integers(2, 9)) for l in seen}
        shapes = [[ext[l] for l in t] for t in inputs]
        tree = tb.ContractionTree.optimize(tb.Subscripts.new(inputs, output), shapes)
        assert tree.macs == oracle.tree_macs(inputs, output, ext, tree.pairs)
        assert tree.macs == oracle.best_macs(inputs, output, ext), (inputs, output, ext)


def test_benchmark_trees(tb):
    # MPS transfer-matrix step: never contract A with conj(A) first.
    chi, d = 512, 2
    tree = tb.ContractionTree.optimize(tb.Subscripts.parse("ab,asc,bsd->cd"), [[chi, chi], [chi, d, chi], [chi, d, chi]])
    assert tree.macs == 2 * chi**3 * d
    assert 0 in tree.pairs[0]
    # 4-tensor network of dim 96: 2 * 96^5 + 96^4 multiply-adds.
    tree = tb.ContractionTree.optimize(tb.Subscripts.parse("ijk,jlm,kmn,lnp->ip"), [[96] * 3] * 4)
    assert tree.macs == 2 * 96**5 + 96**4


# ---------------------------------------------------------------- plan validation
def test_plan_doc_examples_validate(tb):
    P = tb.PrimDescriptor
    plan = lambda d, s, dt=np.float64: tb.CudaBackend.plan(d, s, dt, ctx=_NoCtx)
    # tenferro-prims/src/lib.rs:46-49, 59-62, 72-75, 408-412
    plan(P.BatchedGemm([], 3, 5, 4), [[3, 4], [4, 5], [3, 5]])
    plan(P.Reduce([0, 1], [0], tb.ReduceOp.Sum), [[3, 4], [3]])
    plan(P.Contract([0, 1], [1, 2], [0, 2]), [[3, 4], [4, 5], [3, 5]])
    plan(P.Permute([0, 1], [1, 0]), [[3, 4], [4, 3]])
    plan(P.Trace([0, 1, 2], [2], [(0, 1)]), [[4, 4, 3], [3]])
    plan(P.AntiTrace([2], [0, 1, 2], [(0, 1)]), [[3], [4, 4, 3]])
    plan(P.AntiDiag([0], [0, 1], [(0, 1)]), [[4], [4, 4]])
    plan(P.ElementwiseMul(), [[2, 3], [2, 3], [2, 3]])


class _NoCtxType:
    handle = None


_NoCtx = _NoCtxType()


def test_plan_errors(tb):
    P = tb.PrimDescriptor
    plan = lambda d, s, dt=np.float64: tb.CudaBackend.plan(d, s, dt, ctx=_NoCtx)
    with pytest.raises(tb.ShapeMismatch):
        plan(P.Contract([0, 1], [1, 2], [0, 2]), [[3, 4], [5, 6], [3, 6]])
    with pytest.raises(tb.RankMismatch):
        plan(P.Contract([0, 1], [1, 2], [0, 2]), [[3, 4, 1], [4, 6], [3, 6]])
    with pytest.raises(tb.InvalidArgument):
        plan(P.Contract([0, 1], [1, 2], [0, 7]), [[3, 4], [4, 6], [3, 6]])
    with pytest.raises(tb.ShapeMismatch):
        plan(P.BatchedGemm([2], 3, 5, 4), [[2, 3, 4], [2, 4, 5], [2, 3, 6]])
    with pytest.raises(tb.InvalidArgument):
        plan(P.Permute([0, 1], [1, 2]), [[3, 4], [4, 3]])
    with pytest.raises(tb.InvalidArgument):
        plan(P.Reduce([0, 1], [2], tb.ReduceOp.Sum), [[3, 4], [3]])
    with pytest.raises(tb.InvalidArgument):  # Max/Min undefined for complex
        plan(P.Reduce([0, 1], [0], tb.ReduceOp.Max), [[3, 4], [3]], np.complex128)
    with pytest.raises(tb.ShapeMismatch):
        plan(P.Trace([0, 1], [], [(0, 1)]), [[3, 4], []])
    with pytest.raises(tb.InvalidArgument):
        plan(P.Contract([0, 1], [1, 2], [0, 2]), [[3, 4], [4, 5]])
    with pytest.raises(tb.ShapeMismatch):
        plan(P.ElementwiseMul(), [[2, 3], [2, 3], [3, 2]])


def test_has_extension_for(tb):
    # tenferro-prims/src/lib.rs:322-339
    for dt in (np.float32, np.float64, np.complex64, np.complex128):
        assert tb.CudaBackend.has_extension_for(dt, tb.Extension.Contract)
        assert tb.CudaBackend.has_extension_for(dt, tb.Extension.ElementwiseMul)
    assert not tb.CudaBackend.has_extension_for(np.int32, tb.Extension.Contract)


def test_reduce_op_equality(tb):
    # tenferro-prims/src/lib.rs:93-98
    assert tb.ReduceOp.Sum == tb.ReduceOp.Sum and tb.ReduceOp.Sum != tb.ReduceOp.Max


# ---------------------------------------------------------------- view rules (metadata only)
def test_permute_and_reshape_doc_example(tb):
    # tenferro-tensor/src/lib.rs:45-51
    a = tb.Tensor._meta([2, 3])
    at = a.permute([1, 0])
    assert at.dims() == (3, 2) and at.strides() == (2, 1)
    assert a.reshape([6]).dims() == (6,)
    with pytest.raises(tb.InvalidArgument):
        a.permute([0, 0])
    with pytest.raises(tb.ShapeMismatch):
        a.reshape([5])


def test_broadcast_doc_example(tb):
    # tenferro-tensor/src/lib.rs:57-61
    col = tb.Tensor._meta([3, 1])
    exp = col.broadcast([3, 4])
    assert exp.dims() == (3, 4) and exp.strides()[1] == 0
    with pytest.raises(tb.ShapeMismatch):
        col.broadcast([4, 4])


def test_diagonal_doc_example(tb):
    # tenferro-tensor/src/lib.rs:87-91
    a = tb.Tensor._meta([4, 4])
    d = a.diagonal([(0, 1)])
    assert d.dims() == (4,) and d.strides() == (5,)
    with pytest.raises(tb.ShapeMismatch):
        tb.Tensor._meta([4, 3]).diagonal([(0, 1)])


def test_contiguity_doc_example(tb):
    # tenferro-tensor/src/lib.rs:578-592
    a = tb.Tensor._meta([3, 4])
    assert a.is_contiguous()
    assert tb.Tensor._meta([3, 4], order=tb.MemoryOrder.RowMajor).is_contiguous()
    sub = tb.Tensor._meta([3, 4], strides=[2, 8])
    assert not sub.is_contiguous()
    with pytest.raises(tb.InvalidArgument):
        sub.reshape([12])


def test_column_major_strides(tb):
    # tenferro-tensor/src/lib.rs:110-127: column-major = first dim has stride 1
    assert tb.Tensor._meta([2, 3, 4]).strides() == (1, 2, 6)
    assert tb.Tensor._meta([2, 3, 4], order=tb.MemoryOrder.RowMajor).strides() == (12, 4, 1)


def test_device_preference(tb):
    t = tb.Tensor._meta([2, 2])
    t.set_preferred_compute_device(tb.ComputeDevice.Cuda(1))
    assert t.effective_compute_devices(tb.OpKind.Contract) == [tb.ComputeDevice.Cuda(1)]
    assert t.preferred_compute_device() == tb.ComputeDevice.Cuda(1)
