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


def test_a_tensor_core_templates_wait_gives_up_and_reports():
    """The bounded mbarrier wait every tensor-core template uses (csrc/templates/emb_tc.cuh: mbar_wait), made to run
    out on purpose and harmlessly: a barrier nobody arrives on, a limit of 20 ms instead of 2 s. The waiting thread
    must come back with `false`, the status word must carry (code, CTA, step), the CTA's abort flag must make a later
    wait return at once, the host must turn the word into EmbError(-3), and the context must be alive afterwards."""
    import time

    import torch
    from emmy_ptx import driver, runner, toolchain
    source = r'''
#include "emb_tc.cuh"
extern "C" __global__ void __launch_bounds__(64) k_wait_runs_out(unsigned* status) {
    __shared__ uint64_t bar;
    __shared__ int abort_flag;
    if (threadIdx.x == 0) {
        emb::tc::mbar_init(&bar, 1);
        abort_flag = 0;
        emb::tc::mbar_init_fence();
    }
    __syncthreads();
    const emb::tc::Guard guard{status, &abort_flag};
    if (threadIdx.x == 32) status[3] = emb::tc::mbar_wait(&bar, 0, guard, emb::tc::WAIT_TMEM_FULL, 77) ? 1u : 2u;
    __syncthreads();
    if (threadIdx.x == 0) {
        const unsigned long long t0 = emb::tc::global_ns();
        status[6] = emb::tc::mbar_wait(&bar, 0, guard, emb::tc::WAIT_SMEM_FULL, 5) ? 1u : 2u;  // gives up at once: the CTA is aborting
        status[7] = static_cast<unsigned>((emb::tc::global_ns() - t0) / 1000);
    }
}
'''
    ptx = toolchain.cuda_to_ptx(source, ("-DEMB_WAIT_LIMIT_NS=20000000ull",))
    cubin, _ = toolchain.assemble(ptx)
    driver.init(0)
    fn = driver.Module(cubin).function("k_wait_runs_out")
    status = torch.zeros(8, dtype=torch.int32, device="cuda")
    t0 = time.time()
    driver.launch([driver.Launch(fn, [3, 1, 1], [64, 1, 1], 1, 0, [status.data_ptr()])], torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    assert time.time() - t0 < 1.5
    word = status.cpu().tolist()
    assert word[0] == 3 and word[1] in (0, 1, 2) and word[2] == 77  # the first CTA to give up: accumulator never completed, step 77
    assert word[3] == 2 and word[6] == 2 and word[7] < 5000          # both waits returned false, the second within microseconds
    with pytest.raises(driver.EmbError) as err:
        runner.raise_on_status("k_wait_runs_out", word)
    assert err.value.code == -3 and "code 3" in str(err.value) and "step 77" in str(err.value)
    assert float((torch.ones(4, device="cuda") * 2).sum()) == 8.0  # the context is alive
