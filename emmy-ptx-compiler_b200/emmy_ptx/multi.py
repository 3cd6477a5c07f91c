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


MAX_PEERS = 8  # EMB_MAX_PEERS of csrc/templates/emb_peer.cuh
RECORD_BYTES = 8 * MAX_PEERS + 24  # slot pointers, rank, world, step, status, wait limit (us), reserved
WAIT_LIMIT_US = 2_000_000
SLOT_BYTES = 2 * MAX_PEERS * 8  # per rank: u64 slot[2][MAX_PEERS]


def exchange_record(slot_ptrs: list, rank: int, world: int, wait_limit_us: int = WAIT_LIMIT_US) -> bytes:
    """The bytes of ``emb::PeerExchange`` (csrc/templates/emb_peer.cuh) for this rank. ``slot_ptrs[r]`` is the
    address, as THIS rank sees it, of rank r's slot memory (``u64 slot[2][MAX_PEERS]``, zeroed)."""
    import struct
    if not 1 <= world <= MAX_PEERS or not 0 <= rank < world or len(slot_ptrs) != world:
        raise ValueError(f"an exchange of {world} ranks (at most {MAX_PEERS}), rank {rank}, {len(slot_ptrs)} pointers")
    return struct.pack(f"<{MAX_PEERS}Q6I", *slot_ptrs, *([0] * (MAX_PEERS - world)), rank, world, 0, 0, int(wait_limit_us), 0)


class PeerExchange:
    """Symmetric slot memory of all ranks mapped into every rank, and the device record the sum's last kernel
    takes (``emb::peer_all_sum``): the sharded array sum's one exchange step then happens inside that kernel,
    by peer stores over NVLink and a bounded wait, instead of an all-reduce launched after it.

    ``PeerExchange.create(group)`` allocates the slots through torch's symmetric memory and meets the other
    ranks; ``PeerExchange.alone(device)`` is the one-rank form on ordinary device memory (the kernel then
    exchanges with itself: the same code path, nothing to wait for)."""

    def __init__(self, slots, slot_ptrs: list, rank: int, world: int, keep=None, wait_limit_us: int = WAIT_LIMIT_US):
        import torch
        self.slots, self.rank, self.world, self.keep = slots, rank, world, keep
        raw = exchange_record(slot_ptrs, rank, world, wait_limit_us)
        self.record = torch.frombuffer(bytearray(raw), dtype=torch.uint8).to(slots.device)

    @classmethod
    def alone(cls, device):
        import torch
        slots = torch.zeros(SLOT_BYTES // 4, dtype=torch.float32, device=device)
        return cls(slots, [slots.data_ptr()], 0, 1)

    @classmethod
    def create(cls, group=None):
        import torch
        import torch.distributed as dist
        import torch.distributed._symmetric_memory as symm
        group = group or dist.group.WORLD
        world, rank = dist.get_world_size(group), dist.get_rank(group)
        device = torch.device("cuda", torch.cuda.current_device())
        slots = symm.empty(SLOT_BYTES // 4, dtype=torch.float32, device=device)
        slots.zero_()
        handle = symm.rendezvous(slots, group.group_name)
        torch.cuda.synchronize(device)
        dist.barrier(group)  # every rank's slots are zero before any kernel stores into them
        return cls(slots, [int(p) for p in handle.buffer_ptrs], rank, world, keep=handle)

    def words(self) -> list:
        """rank, world, steps completed, status (0, or 1 + the rank that was waited for in vain)."""
        import torch
        return self.record[8 * MAX_PEERS:8 * MAX_PEERS + 16].cpu().view(dtype=torch.int32).tolist()

    def check(self) -> None:
        """Raise if a kernel's wait for a peer gave up."""
        from . import driver
        words = self.words()
        if words[3]:
            raise driver.EmbError(-3, f"exchange: rank {words[0]} waited in vain for rank {words[3] - 1} at step {words[2] + 1}")

    @property
    def steps(self) -> int:
        return int(self.words()[2])
