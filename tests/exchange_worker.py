"""One rank of the two-or-more-GPU test of the in-kernel exchange (launched by test_gpu_exchange.py through
torch.distributed.run): every rank sums its own copy of the array scaled by (rank + 1); the last kernel of each must
return the f32 sum of all ranks' scalars in rank order, the same bits everywhere, step after step."""

import os
import sys
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT / "emmy-ptx-compiler_b200"))


def main(folder: str, steps: int) -> None:
    import torch
    import torch.distributed as dist

    from emmy_ptx import multi, runner
    rank, local = int(os.environ["RANK"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    world = dist.get_world_size()
    plain = runner.Problem(folder, "optimized", device=local)
    x = plain.host["x"] * np.float32(rank + 1)
    alone = runner.Problem(folder, "optimized", device=local, inputs={"x": x}).run()["sum_1"].copy()
    mine = torch.from_numpy(alone).cuda()
    parts = [torch.empty_like(mine) for _ in range(world)]
    dist.all_gather(parts, mine)
    want = parts[0].clone()
    for p in parts[1:]:
        want += p  # rank order in f32, as the kernel adds
    ex = multi.PeerExchange.create()
    prob = runner.Problem(folder, "optimized", device=local, inputs={"x": x}, exchange=ex)
    for step in range(steps):
        got = prob.run()["sum_1"]
        assert got.tobytes() == want.cpu().numpy().tobytes(), (rank, step, got, want)
    assert ex.steps == steps
    dist.barrier()
    if rank == 0:
        print(f"exchange ok: {world} ranks, {steps} steps, total {float(want[0])!r}")
    dist.destroy_process_group()


if __name__ == "__main__":
    main(sys.argv[1], int(sys.argv[2]))
