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


SHARDED_AXIS = {"sum": "element range", "softmax": "rows", "matmul": "rows of A and C (B replicated)",
                "attention": "(batch, head) pairs", "mlp": "token rows (weights and scales replicated)",
                "fragments": "rows of A and C (B replicated)", "elementwise": "rows (the bias row replicated)",
                "elementwise_add": "rows (the bias row replicated)"}

# The full-size workloads: what is sharded, in which units (a unit is the smallest piece a rank may own, so
# that every shard keeps the alignment its template wants), and which operands are sliced along it.
#   units(sizes) -> count; build(sizes, count) -> keyword arguments of the problems.* builder for `count` units;
#   sliced: operand -> how many leading elements one unit is (None: the operand is replicated on every rank)
FULL_SIZES = {
    "sum": dict(n=1 << 24), "softmax": dict(rows=8192, cols=4096), "matmul": dict(m=8192, n=8192, k=8192),
    "attention": dict(batch=8, heads=32, seq=4096, dim=128), "mlp": dict(tokens=16384, d_model=4096, hidden=16384),
    "fragments": dict(m=8192, n=8192, k=8192), "elementwise": dict(rows=8192, cols=4096),
    "elementwise_add": dict(rows=8192, cols=4096),
}
SUM_RUN = 1024   # elements per unit of the array sum: one trip of a 256-thread block on 16-byte runs
ROW_BLOCK = 128  # rows per unit of the tensor-core workloads: one row of output tiles


def sum_grid(n: int, block: int = 256, vec: int = 4) -> int:
    """Blocks of the sum's first kernel: whole waves of 148 SMs, at least two trips per block, at most eight
    blocks per SM (1184 for 2^24 elements, the geometry the one-GPU measurement was tuned on)."""
    trips = max(1, n // (block * vec))
    return 148 * max(1, min(8, trips // (148 * 2))) if trips >= 148 else trips


def plan(workload: str, rank: int, world: int, sizes: dict | None = None) -> dict:
    """How ``rank`` of ``world`` takes part in one workload: ``units`` (what is divided), ``share`` (the
    contiguous range this rank owns), ``kwargs`` (arguments of the ``problems`` builder for a problem of the
    share's size), ``slices`` (operand -> (first element, elements) along its leading axis; operands that are
    not listed are replicated) and ``reshape`` (operand -> the shape the slice takes in the shard's problem).
    No workload needs data from another rank, except the sum's scalar (``combine_sum`` / ``PeerExchange``)."""
    z = dict(FULL_SIZES[workload], **(sizes or {}))
    slices, reshape = {}, {}
    if workload == "sum":
        if z["n"] % SUM_RUN:
            raise ValueError(f"the sum's length {z['n']} is not a multiple of {SUM_RUN}")
        units = z["n"] // SUM_RUN
        share = shard(units, rank, world)
        n = len(share) * SUM_RUN
        kwargs = dict(n=n, grid=sum_grid(n))
        slices["x"] = (share.start * SUM_RUN, n)
    elif workload in ("softmax", "elementwise", "elementwise_add"):
        units = z["rows"]
        share = shard(units, rank, world)
        kwargs = dict(rows=len(share), cols=z["cols"])
        for name in ("x", "res") if workload == "elementwise_add" else ("x",):
            slices[name] = (share.start, len(share))  # (the pointwise workloads' bias row is replicated)
    elif workload in ("matmul", "fragments"):
        if z["m"] % ROW_BLOCK:
            raise ValueError(f"M = {z['m']} is not a multiple of {ROW_BLOCK}")
        units = z["m"] // ROW_BLOCK
        share = shard(units, rank, world)
        kwargs = dict(m=len(share) * ROW_BLOCK, n=z["n"], k=z["k"])
        slices["a" if workload == "matmul" else "x0"] = (share.start * ROW_BLOCK, len(share) * ROW_BLOCK)
    elif workload == "attention":
        units = z["batch"] * z["heads"]
        share = shard(units, rank, world)
        kwargs = dict(batch=1, heads=len(share), seq=z["seq"], dim=z["dim"])
        for name in "qkv":
            slices[name] = (share.start, len(share))
            reshape[name] = (units, z["seq"], z["dim"])
    elif workload == "mlp":
        if z["tokens"] % ROW_BLOCK:
            raise ValueError(f"{z['tokens']} tokens are not a multiple of {ROW_BLOCK}")
        units = z["tokens"] // ROW_BLOCK
        share = shard(units, rank, world)
        kwargs = dict(tokens=len(share) * ROW_BLOCK, d_model=z["d_model"], hidden=z["hidden"])
        slices["x"] = (share.start * ROW_BLOCK, len(share) * ROW_BLOCK)
    else:
        raise KeyError(workload)
    if len(share) == 0:
        raise ValueError(f"{workload}: rank {rank} of {world} gets none of the {units} units")
    return dict(workload=workload, units=units, share=share, kwargs=kwargs, slices=slices, reshape=reshape,
                axis=SHARDED_AXIS[workload])


def shard_inputs(pl: dict, full: dict, shard_args: list) -> dict:
    """The shard's host inputs cut out of the full problem's (``full``: name -> numpy array as
    ``runner.host_inputs`` makes them): sliced operands along their leading axis, everything else whole.
    ``shard_args`` are the shard problem's meta.json arguments (for the shapes the slices take)."""
    shapes = {a["name"]: a["shape"] for a in shard_args}
    out = {}
    for name, array in full.items():
        if name in pl["slices"]:
            lo, count = pl["slices"][name]
            lead = pl["reshape"].get(name)
            piece = (array.reshape(lead) if lead else array)[lo:lo + count]
            out[name] = piece.reshape(shapes[name]).copy()
        else:
            out[name] = array
    return out


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
