"""The multi-rank host logic on CPU: two gloo ranks on 127.0.0.1."""

import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from emmy_ptx import multi


def test_shards_cover_every_unit_exactly_once():
    for units, world in [(8192, 8), (256, 3), (5, 8), (1 << 24, 7)]:
        seen = np.zeros(units, int)
        for r in range(world):
            s = multi.shard(units, r, world)
            seen[s.start:s.stop] += 1
        assert (seen == 1).all()
        sizes = [len(multi.shard(units, r, world)) for r in range(world)]
        assert max(sizes) - min(sizes) <= 1
    with pytest.raises(ValueError):
        multi.shard(10, 2, 2)


def _rank(rank, world, port, strict, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    x = np.random.default_rng(0).uniform(-1, 1, 1 << 16).astype(np.float32)
    mine = multi.shard(x.size, rank, world)
    partial = torch.tensor([x[mine.start:mine.stop].sum(dtype=np.float32)])
    total = multi.combine_sum(partial, strict=strict)
    out.put((rank, float(total.item())))
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("strict", [False, True])
def test_two_ranks_combine_their_partial_sums(strict):
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    procs = [ctx.Process(target=_rank, args=(r, 2, port, strict, out)) for r in range(2)]
    for p in procs:
        p.start()
    results = dict(out.get(timeout=120) for _ in procs)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    x = np.random.default_rng(0).uniform(-1, 1, 1 << 16).astype(np.float32)
    a, b = x[:1 << 15].sum(dtype=np.float32), x[1 << 15:].sum(dtype=np.float32)
    assert results[0] == results[1] == float(np.float32(a + b))


def test_exchange_record_layout():
    """The bytes handed to the kernel as emb::PeerExchange: eight slot pointers, rank, world, step, status, the wait limit."""
    import struct

    import pytest

    from emmy_ptx import multi
    raw = multi.exchange_record([0x10000, 0x20000, 0x30000], rank=2, world=3)
    assert len(raw) == multi.RECORD_BYTES == 88
    words = struct.unpack("<8Q6I", raw)
    assert words[:3] == (0x10000, 0x20000, 0x30000) and words[3:8] == (0,) * 5
    assert words[8:] == (2, 3, 0, 0, multi.WAIT_LIMIT_US, 0)
    assert multi.SLOT_BYTES == 128
    with pytest.raises(ValueError):
        multi.exchange_record([1] * 9, 0, 9)
    with pytest.raises(ValueError):
        multi.exchange_record([1, 2], 2, 2)


def test_exchange_protocol_with_ranks_as_threads():
    """The slot protocol of csrc/templates/emb_peer.cuh restated on host memory, ranks as threads that run at random
    speeds: one (step, value) word per (parity, sender) slot in every rank's memory; a rank stores its word into all
    ranks' slots of parity step & 1, waits for every sender's word of that step in its own slots, and adds in rank order.
    Every rank must see the same sums for many steps, although a fast rank may already be writing the next step (other
    parity) while a slow one still reads: it can never be two steps ahead, because its wait of the step between needs
    the slow rank's word, which is stored only after the slow rank has read the older values."""
    import random
    import threading
    import time

    world, steps = 4, 300
    slots = [[[(0, 0.0)] * world for _ in range(2)] for _ in range(world)]  # slots[owner][parity][sender] = (step, value)
    results = [[] for _ in range(world)]
    failed = []

    def rank_main(rank: int) -> None:
        rng = random.Random(rank)
        for q in range(1, steps + 1):
            mine = float(np.float32(rank + 1) * np.float32(q))
            if rng.random() < 0.2:
                time.sleep(rng.random() * 0.002)
            for owner in range(world):
                slots[owner][q & 1][rank] = (q, mine)
            got = []
            for sender in range(world):
                deadline = time.time() + 5.0
                while slots[rank][q & 1][sender][0] != q:
                    if time.time() > deadline:
                        failed.append((rank, q, sender))
                        return
                    time.sleep(0)
                got.append(slots[rank][q & 1][sender][1])
            total = np.float32(got[0])
            for v in got[1:]:
                total = np.float32(total + np.float32(v))
            results[rank].append(float(total))

    threads = [threading.Thread(target=rank_main, args=(r,)) for r in range(world)]
    for t in threads:
        t.start()
    for t in threads:
        t.join(60)
    assert not failed, failed
    want = [float(np.float32(sum(range(1, world + 1))) * np.float32(q)) for q in range(1, steps + 1)]
    for r in range(world):
        assert results[r] == want
