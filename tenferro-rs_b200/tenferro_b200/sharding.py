"""Host-side shard arithmetic for running one contraction on several GPUs (one process per
GPU).  Nothing here touches a device: a shard is a strided sub-view - same buffer, same
strides, new extent and offset - so the kernels see it like any other view
(tenferro-tensor/src/lib.rs:167-171 describes the fields).

  * a FREE index (one that survives into the output) splits with no communication: every rank
    contracts its slice of the operand that carries the index and writes its slice of C;
  * a CONTRACTED index splits into partial sums of the whole output, which a reduce-scatter
    (sum) then leaves distributed;
  * a table of independent problems splits into contiguous ranges of equal byte counts.
"""
from __future__ import annotations

from typing import List, Sequence, Tuple

import numpy as np


def split_range(extent: int, world: int, rank: int) -> Tuple[int, int]:
    """[start, stop) of `rank`'s contiguous share of range(extent); shares differ by at most one."""
    if world < 1 or not 0 <= rank < world:
        raise ValueError(f"rank {rank} out of range for {world} ranks")
    base, extra = divmod(extent, world)
    start = rank * base + min(rank, extra)
    return start, start + base + (1 if rank < extra else 0)


def shard_view(dims: Sequence[int], strides: Sequence[int], offset: int, axis: int, world: int, rank: int):
    """(dims, strides, offset) of `rank`'s slice along `axis` of a strided view."""
    start, stop = split_range(dims[axis], world, rank)
    new_dims = list(dims)
    new_dims[axis] = stop - start
    return new_dims, list(strides), offset + start * strides[axis]


def shard_operands(labels: Sequence[Sequence[int]], views: Sequence[Tuple[Sequence[int], Sequence[int], int]],
                   label: int, world: int, rank: int):
    """Slice every view that carries `label` (a free or a contracted index) for `rank`.
    `views` are (dims, strides, offset) triples; views without the label are returned as they are."""
    out = []
    for labs, (dims, strides, offset) in zip(labels, views):
        if label in labs:
            out.append(shard_view(dims, strides, offset, list(labs).index(label), world, rank))
        else:
            out.append((list(dims), list(strides), offset))
    return out


def split_table_by_bytes(bytes_per_problem: Sequence[float], world: int) -> List[int]:
    """Cut points (world + 1 of them) of contiguous problem ranges with near-equal byte totals."""
    cum = np.concatenate([[0.0], np.cumsum(np.asarray(bytes_per_problem, dtype=np.float64))])
    cuts = [int(np.searchsorted(cum, cum[-1] * q / world)) for q in range(world + 1)]
    cuts[0], cuts[-1] = 0, len(bytes_per_problem)
    for i in range(1, world + 1):
        cuts[i] = max(cuts[i], cuts[i - 1])
    return cuts
