"""Multi-GPU host logic: how each workload shards over ranks, and the one exchange the path has.

The reference is single-GPU (1-D grids only, emmy_ptx/frontend.py:83); sharding is this backend's
addition. Every workload partitions without a data-path exchange - softmax by rows, matmul and the MLP
by output rows, attention by (batch, head) pairs - except the array sum, whose per-GPU partial results
are combined by ONE collective: an all-reduce (default), or, for ``strict``, an all-gather followed by
a fold in rank order on every rank, because an all-reduce's order of additions is the library's own
and would break bit-exactness across runs and world sizes.
"""

from __future__ import annotations


def shard(units: int, rank: int, world: int) -> range:
    """The contiguous share of ``units`` (rows, elements, (batch, head) pairs) that ``rank`` owns:
    sizes differ by at most one, every unit belongs to exactly one rank."""
    if not 0 <= rank < world:
        raise ValueError(f"rank {rank} outside 0..{world - 1}")
    base, extra = divmod(units, world)
    lo = rank * base + min(rank, extra)
    return range(lo, lo + base + (1 if rank < extra else 0))


SHARDED_AXIS = {"sum": "elements", "softmax": "rows", "matmul": "rows of A and C (B replicated)",
                "attention": "(batch, head) pairs", "mlp": "token rows (weights replicated)",
                "fragments": "rows of A and C (B replicated)"}


def combine_sum(partial, strict: bool = False, group=None):
    """Combine the per-rank scalar results of the array sum, in place, and return the tensor."""
    import torch
    import torch.distributed as dist
    if not dist.is_initialized() or dist.get_world_size(group) == 1:
        return partial
    if not strict:
        dist.all_reduce(partial, op=dist.ReduceOp.SUM, group=group)
        return partial
    parts = [torch.empty_like(partial) for _ in range(dist.get_world_size(group))]
    dist.all_gather(parts, partial, group=group)
    total = parts[0].clone()
    for p in parts[1:]:  # rank order, the same on every rank
        total += p
    partial.copy_(total)
    return partial
