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


# ---------------------------------------------------------------- sharding plans: N ranks solve the one-GPU problem

SMALL = {"sum": dict(n=1 << 14), "softmax": dict(rows=24, cols=256), "matmul": dict(m=384, n=64, k=64),
         "attention": dict(batch=2, heads=3, seq=32, dim=16), "mlp": dict(tokens=384, d_model=64, hidden=64),
         "fragments": dict(m=384, n=64, k=64), "elementwise": dict(rows=24, cols=256), "elementwise_add": dict(rows=24, cols=256)}


def _full_inputs(workload, sizes):
    from emmy_ptx import problems, runner
    full = problems.WORKLOADS[workload](ident="full", **multi.plan(workload, 0, 1, sizes)["kwargs"])
    meta = problems._meta(full)
    host = {}
    for km in meta["kernels"]:
        host.update(runner.host_inputs(km["args"]))
    return full, host


@pytest.mark.parametrize("workload", sorted(SMALL))
def test_plans_partition_every_workload(workload):
    """Every unit belongs to one rank; the sliced operands of all ranks put together are the full operands, everything
    else is replicated; the shard problems have the shapes their slices need."""
    from emmy_ptx import problems
    sizes = SMALL[workload]
    _, host = _full_inputs(workload, sizes)
    for world in (1, 2, 3):
        plans = [multi.plan(workload, r, world, sizes) for r in range(world)]
        assert sum(len(p["share"]) for p in plans) == plans[0]["units"]
        assert all(a["share"].stop == b["share"].start for a, b in zip(plans, plans[1:]))
        pieces = {}
        for r, pl in enumerate(plans):
            shard = problems.WORKLOADS[workload](ident=f"s{r}", **pl["kwargs"])
            args = [a for km in problems._meta(shard)["kernels"] for a in km["args"]]
            ins = multi.shard_inputs(pl, host, args)
            shapes = {a["name"]: tuple(a["shape"]) for a in args if not a.get("output") and not a.get("intermediate")}
            for name, array in ins.items():
                assert tuple(array.shape) == shapes[name], (name, array.shape, shapes[name])
                if name in pl["slices"]:
                    pieces.setdefault(name, []).append(array.reshape(-1))
                else:
                    assert array is host[name]
        for name, parts in pieces.items():
            assert np.array_equal(np.concatenate(parts).view(np.uint8), host[name].reshape(-1).view(np.uint8)), name
    with pytest.raises(ValueError):
        multi.plan(workload, 10 ** 6 - 1, 10 ** 6, sizes)  # more ranks than units: the last ranks would get nothing


def test_the_sums_grid_keeps_whole_waves():
    assert multi.sum_grid(1 << 24) == 1184 and multi.sum_grid(1 << 21) == 888 and multi.sum_grid(1 << 14) == 16
    for world in (2, 4, 8):
        pl = multi.plan("sum", world - 1, world)
        assert pl["kwargs"]["n"] * world == 1 << 24 and pl["kwargs"]["grid"] % 148 == 0


def _sharded_rank(rank, world, port, workload, out):
    """One rank of a CPU run: its shard of the workload through the oracle (standing in for the GPU kernels), the sum's
    scalars combined as the bench does without peer memory."""
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from emmy_ptx import problems, runner
    from oracle import ir_oracle
    sizes = SMALL[workload]
    _, host = _full_inputs(workload, sizes)
    pl = multi.plan(workload, rank, world, sizes)
    shard = problems.WORKLOADS[workload](ident="s", **pl["kwargs"])
    args = [a for km in problems._meta(shard)["kernels"] for a in km["args"]]
    bufs = dict(multi.shard_inputs(pl, host, args))
    for kern in shard["kernels"]:
        name, shape, dt = kern["output"]
        bufs[name] = np.zeros(shape, runner.numpy_dtype(dt))
        ir_oracle.run(kern["body"], bufs, kern["grid"], kern["block"])
    final = shard["kernels"][-1]["output"][0]
    result = np.asarray(bufs[final], np.float32).reshape(-1)
    if workload == "sum":
        result = multi.combine_sum(torch.from_numpy(result.copy()), strict=True).numpy()
    out.put((rank, result))
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("workload", ["sum", "softmax", "attention", "elementwise_add"])
def test_two_ranks_solve_the_one_rank_problem(workload):
    """Strong scaling on the host: two gloo ranks each run their shard; put together (rows, pairs) or combined in rank
    order (the sum) the results are the one-rank problem's - bit for bit where rows are independent."""
    from emmy_ptx import problems, runner
    from oracle import ir_oracle
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    procs = [ctx.Process(target=_sharded_rank, args=(r, 2, port, workload, out)) for r in range(2)]
    for p in procs:
        p.start()
    results = dict(out.get(timeout=180) for _ in procs)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    full, host = _full_inputs(workload, SMALL[workload])
    bufs = dict(host)
    for kern in full["kernels"]:
        name, shape, dt = kern["output"]
        bufs[name] = np.zeros(shape, runner.numpy_dtype(dt))
        ir_oracle.run(kern["body"], bufs, kern["grid"], kern["block"])
    want = np.asarray(bufs[full["kernels"][-1]["output"][0]], np.float32).reshape(-1)
    if workload == "sum":
        assert np.array_equal(results[0], results[1])  # every rank holds the same bits
        assert abs(float(results[0][0]) - float(want[0])) <= 1e-5 * np.sqrt(SMALL["sum"]["n"])
    else:
        assert np.array_equal(np.concatenate([results[0], results[1]]).view(np.uint32), want.view(np.uint32))
