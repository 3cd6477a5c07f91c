"""The exchange step of the sharded array sum inside its last kernel (csrc/templates/emb_peer.cuh)."""

import os
import subprocess
import sys
from pathlib import Path

import pytest

from emmy_ptx import multi, problems, runner

pytestmark = pytest.mark.gpu
HERE = Path(__file__).resolve().parent


def small_sum(tmp_path):
    return problems.write(problems.array_sum(n=1 << 16, grid=16, block=256, ident="t_sum"), tmp_path)


def test_one_rank_exchanges_with_itself(tmp_path):
    """World of one: the kernel stores into its own slot, finds its own flag and returns its own value - the same
    code path as with peers, with nothing to wait for; the step counter and both parities are walked."""
    import torch
    folder = small_sum(tmp_path)
    want = runner.Problem(folder, "strict").run()["sum_1"]
    ex = multi.PeerExchange.alone(torch.device("cuda", 0))
    prob = runner.Problem(folder, "strict", exchange=ex)
    assert any(p["kind"] == "exchange" for p in prob.kernels[-1].launch_info["params"])
    for step in range(1, 4):
        got = prob.run()["sum_1"]
        assert got.tobytes() == want.tobytes()
        assert ex.steps == step
    prob.check_status()


def test_a_wait_for_a_peer_that_never_stores_runs_out(tmp_path):
    """Failure detection without a fault: a record that names a second rank whose slots nobody writes (ordinary memory
    of this GPU). The kernel's wait for that rank gives up after the record's limit (20 ms here), the kernel ends
    normally, the host reads which rank was missing; later steps return at once instead of waiting again."""
    import time

    import torch

    from emmy_ptx import driver
    folder = small_sum(tmp_path)
    dev = torch.device("cuda", 0)
    mine = torch.zeros(multi.SLOT_BYTES // 4, dtype=torch.float32, device=dev)
    silent = torch.zeros(multi.SLOT_BYTES // 4, dtype=torch.float32, device=dev)
    ex = multi.PeerExchange(mine, [mine.data_ptr(), silent.data_ptr()], rank=0, world=2, keep=silent, wait_limit_us=20_000)
    prob = runner.Problem(folder, "optimized", exchange=ex)
    t0 = time.perf_counter()
    with pytest.raises(driver.EmbError, match="waited in vain for rank 1"):
        prob.run()
    assert time.perf_counter() - t0 < 5.0
    assert ex.words() == [0, 2, 1, 2]  # the step is counted, rank 1 was waited for in vain
    t0 = time.perf_counter()
    for _ in range(50):
        driver.launch(prob.launches, prob.stream)
    torch.cuda.synchronize()
    assert time.perf_counter() - t0 < 0.5 and ex.steps == 1  # no more exchanges, no more waiting
    assert torch.zeros(1, device=dev).item() == 0  # the context is alive


def test_ranks_on_several_gpus_agree_bit_for_bit(tmp_path):
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    n = 2
    folder = small_sum(tmp_path)
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={n}", "--master-addr", "127.0.0.1",
                        "--master-port", "29517", str(HERE / "exchange_worker.py"), str(folder), "6"],
                       capture_output=True, text=True, timeout=600, env=env)
    assert r.returncode == 0 and "exchange ok" in r.stdout, (r.stdout[-2000:], r.stderr[-4000:])
