"""The N > 1 host logic on two CPU ranks (gloo): shard views of a free index, of a contracted
index (partial sums + sum-reduction) and of a problem table.  NumPy stands in for the device
kernels - what is checked is the view arithmetic and the exchange step the GPU ranks run."""
import os
import socket
import sys
from pathlib import Path

import numpy as np
import pytest

ROOT = Path(__file__).resolve().parents[1]


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _strided(buf, dims, strides, offset):
    it = buf.dtype.itemsize
    return np.lib.stride_tricks.as_strided(buf[offset:], shape=dims, strides=[s * it for s in strides])


def _worker(rank, world, port, out_dir):
    sys.path.insert(0, str(ROOT / "tenferro-rs_b200"))
    import torch
    import torch.distributed as dist
    from tenferro_b200 import sharding

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    rng = np.random.default_rng(123)  # every rank draws the same full tensors
    i, j, k, l, m, n = 6, 3, 4, 5, 2, 7
    a = np.asfortranarray(rng.standard_normal((i, j, k, l)))
    b = np.asfortranarray(rng.standard_normal((k, l, m, n)))
    want = np.einsum("ijkl,klmn->ijmn", a, b)
    abuf, bbuf = a.reshape(-1, order="F"), b.reshape(-1, order="F")
    col = lambda d: [int(np.prod(d[:x])) for x in range(len(d))]
    views = [((i, j, k, l), col((i, j, k, l)), 0), ((k, l, m, n), col((k, l, m, n)), 0)]
    labels = [[0, 1, 2, 3], [2, 3, 4, 5]]

    # free index i: each rank computes its slice of C, no exchange needed to be correct
    (da, sa, oa), (db, sb, ob) = sharding.shard_operands(labels, views, 0, world, rank)
    part = np.einsum("ijkl,klmn->ijmn", _strided(abuf, da, sa, oa), _strided(bbuf, db, sb, ob))
    lo, hi = sharding.split_range(i, world, rank)
    assert np.allclose(part, want[lo:hi])
    gathered = [torch.zeros(1) for _ in range(world)]
    dist.all_gather(gathered, torch.tensor([float(hi - lo)]))
    assert sum(int(g.item()) for g in gathered) == i

    # contracted index l: partial sums of the whole output, summed across the ranks
    (da, sa, oa), (db, sb, ob) = sharding.shard_operands(labels, views, 3, world, rank)
    partial = np.einsum("ijkl,klmn->ijmn", _strided(abuf, da, sa, oa), _strided(bbuf, db, sb, ob))
    t = torch.from_numpy(np.ascontiguousarray(partial))
    dist.all_reduce(t, op=dist.ReduceOp.SUM)  # gloo has no reduce_scatter; every rank keeps its slice
    flat = t.numpy().reshape(-1)
    s0, s1 = sharding.split_range(flat.size, world, rank)
    assert np.allclose(flat[s0:s1], np.ascontiguousarray(want).reshape(-1)[s0:s1])

    # problem table: contiguous ranges, every problem exactly once, byte totals balanced
    table = rng.choice(np.array([16, 32, 64, 128]), size=(257, 3))
    nbytes = 4 * (table[:, 0] * table[:, 1] + table[:, 1] * table[:, 2] + table[:, 0] * table[:, 2])
    cuts = sharding.split_table_by_bytes(nbytes, world)
    mine = nbytes[cuts[rank]:cuts[rank + 1]].sum()
    tot = torch.tensor([float(mine), float(cuts[rank + 1] - cuts[rank])])
    dist.all_reduce(tot)
    assert int(tot[1].item()) == 257 and abs(tot[0].item() - nbytes.sum()) < 1
    assert abs(mine - nbytes.sum() / world) <= nbytes.max()
    dist.barrier()
    dist.destroy_process_group()
    (Path(out_dir) / f"ok{rank}").write_text("ok")


def test_two_rank_sharding(tmp_path):
    import torch.multiprocessing as mp

    port = _free_port()
    mp.spawn(_worker, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    assert (tmp_path / "ok0").exists() and (tmp_path / "ok1").exists()


def test_split_range_and_views():
    sys.path.insert(0, str(ROOT / "tenferro-rs_b200"))
    from tenferro_b200 import sharding

    assert [sharding.split_range(10, 3, r) for r in range(3)] == [(0, 4), (4, 7), (7, 10)]
    assert sharding.split_range(2, 4, 3) == (2, 2)  # empty share
    dims, strides, off = sharding.shard_view([8, 5], [1, 8], 3, 0, 2, 1)
    assert (dims, strides, off) == ([4, 5], [1, 8], 7)
    dims, strides, off = sharding.shard_view([8, 5], [1, 8], 0, 1, 5, 4)
    assert (dims, off) == ([8, 1], 32)
    with pytest.raises(ValueError):
        sharding.split_range(4, 2, 2)
    assert sharding.split_table_by_bytes([1, 1, 1, 1], 2) == [0, 2, 4]
