#!/usr/bin/env python3
"""Benchmark of the hot path: one pass of a workload's kernel chain per step, on 1..8 GPUs.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload mlp|softmax|...] [--mode optimized|strict]
    python bench.py --impl reference ...      # the CPU interpreter of the same IR on the host cores

One JSON line on stdout (rank 0). ``value`` is microseconds per pass of the workload's kernel
chain with the inputs resident in HBM: K passes back to back between one CUDA event pair on the
launching stream, the passes rotating through enough copies of every buffer that none finds its
data in L2, max over ranks; ``e2e`` is the same pass through the public API from HOST buffers
(pinned host -> device copy of the step's inputs, the launches, device -> host copy of the result,
all inside the event pair; operands the sharding replicates - the MLP's weights and scales, the
matmul's B - are the job's parameters and stay resident, as they do at every world size);
``roofline`` is the dominant kernel's algorithmic bytes or flops per launch over its measured
duration against the measured peak; ``cpu_baseline`` is the oracle (a port of the reference's numpy
interpreter) timed on a bounded sample of the same workload, ``cpu_baseline_f64`` the float64 torch
expression of the problem on all host cores (how the reference makes its expected values). The
``families`` entries carry the same keys for the other workloads.

Multi-GPU (torchrun, one rank per GPU): STRONG scaling. The N ranks solve the one-GPU problem
together: rank r owns ``multi.shard(units, r, N)`` of it - an element range of the sum, rows of the
softmax and the pointwise workloads, rows of A and C of the matmul (B copied once into each GPU's own
memory before the timed region), (batch, head) pairs of the attention, token rows of the MLP (weights
and scales replicated) - compiled for the shard's size, on the shard of the same seeded inputs. No
data-path collective, except the sum: its per-GPU scalars are combined inside the sum's last kernel
(peer stores into symmetric memory, bounded wait; ``--exchange nccl``: an NCCL all-reduce after it),
and the bench checks the exchanged result bit for bit against the rank-order f32 sum of the
all-gathered per-rank scalars.
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import sys
import tempfile
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
PKG = ROOT / "emmy-ptx-compiler_b200"
for p in (PKG, ROOT):
    if str(p) not in sys.path:
        sys.path.insert(0, str(p))


def _sum_work(k):
    return dict(bytes=k["n"] * 4)


def _rows_work(k):
    return dict(bytes=2 * k["rows"] * k["cols"] * 4)


def _matmul_work(k):
    return dict(flops=2 * k["m"] * k["n"] * k["k"])


def _attention_work(k):
    return dict(flops=4 * k["batch"] * k["heads"] * k["dim"] * k["seq"] * (k["seq"] + 1) // 2)


def _mlp_work(k):
    one = 2 * k["tokens"] * k["d_model"] * k["hidden"]
    return dict(flops=one, chain_flops=2 * one)


WORKLOADS = {
    # name: problem folder of the one-GPU size, what bounds the dominant kernel, that kernel (its index among the pass's
    # launches, or its entry), and the algorithmic work of one launch as a function of the (shard's) sizes
    "mlp": dict(folder="k_mlp_gelu_tanh_16384x4096x16384", bound="tensor", dominant="k_mlp_gelu__h", dtype="bf16", work=_mlp_work,
                describe="GELU MLP 16384x4096x16384, bf16 x, e4m3 weights decoded to bf16, bf16 tcgen05 MMA (BASELINE configs[4])"),
    "softmax": dict(folder="f_softmax_8192x4096", bound="hbm", dominant=0, dtype="f32", work=_rows_work,
                    describe="row softmax [8192,4096] f32 (BASELINE configs[1])"),
    "sum": dict(folder="r_sum_16m", bound="hbm", dominant=0, dtype="f32", work=_sum_work,
                describe="f32 array sum of 2^24 (BASELINE configs[0]): block partials + final fold"),
    "matmul": dict(folder="m_f16_8192", bound="tensor", dominant=0, dtype="f16", work=_matmul_work,
                   describe="f16 GEMM 8192^3, f32 accumulate (BASELINE configs[2])"),
    "attention": dict(folder="a_f16_causal_8x32x4096x128", bound="tensor", dominant=0, dtype="f16", work=_attention_work,
                      describe="causal attention 8x32x4096x128 f16 (BASELINE configs[3])"),
    # pointwise work on the streaming template: y = gelu_tanh(x + bias) (compute-heavy per byte) and
    # y = relu(x + bias) + res (two additions per 16 bytes)
    "elementwise": dict(folder="e_bias_gelu_8192x4096", bound="hbm", dominant=0, dtype="f32", work=_rows_work,
                        describe="pointwise bias + tanh-GELU over [8192,4096] f32 (8 B per element)"),
    "elementwise_add": dict(folder="e_bias_relu_res_8192x4096", bound="hbm", dominant=0, dtype="f32",
                            work=lambda k: dict(bytes=3 * k["rows"] * k["cols"] * 4),
                            describe="pointwise relu(x + bias) + res over [8192,4096] f32 (12 B per element)"),
    # the array sum in emmy's own scalar spelling (one-name loads strided over the block, two unrolled copies): the
    # regroup rewrite deals 16-byte chunks to the threads
    "sum_scalar": dict(folder="r_sum_16m_scalar", bound="hbm", dominant=0, dtype="f32", work=_sum_work, sizes=dict(n=1 << 24),
                       describe="f32 array sum of 2^24 in emmy's scalar spelling, regrouped into 16-byte chunks"),
    # a mid-size MLP whose d_model fits the cluster-fused template (EMMY_PTX_PREFER=dsmem), as the default two-matmul
    # chain and fused: the measured reason why the chain is the default
    "mlp_2048": dict(folder="k_mlp_gelu_tanh_16384x2048x8192", bound="tensor", dominant="k_mlp_gelu__h", dtype="bf16", work=_mlp_work,
                     sizes=dict(tokens=16384, d_model=2048, hidden=8192),
                     describe="GELU MLP 16384x2048x8192 as decode + two tcgen05 matmuls (the default)"),
    "mlp_2048_fused": dict(folder="k_mlp_gelu_tanh_16384x2048x8192", bound="tensor", dominant="k_mlp_gelu", dtype="bf16", prefer="dsmem",
                           work=lambda k: dict(flops=2 * _mlp_work(k)["flops"]), sizes=dict(tokens=16384, d_model=2048, hidden=8192),
                           describe="GELU MLP 16384x2048x8192 fused in clusters of 8 (hidden chunks through distributed shared memory)"),
    # the matmul handed over as a warp-level mma.sync schedule (fragment form) plus its fold kernel: optimized mode proves
    # it a matmul and runs the tcgen05 template, --mode plain runs the schedule as written
    "fragments": dict(folder="m_f16_8192_fragments", bound="tensor", dominant=0, dtype="f16", work=_matmul_work, oracle="fragment",
                      describe="f16 GEMM 8192^3 given in fragment form (mma.sync schedule, B stored N x K) + fold kernel"),
}
CHUNKED = ("mlp", "matmul", "attention", "fragments")  # e2e in slices of the units (pipeline.ChunkedProblem)
DEFAULT_FAMILIES = "sum,softmax,matmul,attention,elementwise,elementwise_add,sum_scalar,fragments,mlp_2048,mlp_2048_fused"
# dram__bytes_read.sum + dram__bytes_write.sum per launch of the dominant kernel at the one-GPU size, from the ncu
# captures summarised under profiles/ (None until captured)
NCU_TRAFFIC = {"softmax": 212.3e6, "sum": 67.5e6, "matmul": 1253.1e6, "attention": 1057.0e6, "mlp": 1380.1e6, "fragments": 1326.0e6,
               "elementwise": 219.5e6, "elementwise_add": 359.3e6, "sum_scalar": 67.5e6, "mlp_2048_fused": 775.1e6}
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}


def peaks() -> tuple:
    f = ROOT / "MEASURED_PEAKS.json"
    if f.exists():
        d = json.loads(f.read_text())
        return d, "measured"
    return FALLBACK_PEAKS, "fallback"


class ClockSampler(threading.Thread):
    """Samples SM clock and clock-event reasons through NVML while the timed region runs (read only)."""

    REASONS = {0x4: "sw_power_cap", 0x8: "hw_slowdown", 0x20: "sw_thermal_slowdown", 0x40: "hw_thermal_slowdown",
               0x80: "hw_power_brake_slowdown", 0x2: "applications_clocks_setting"}

    def __init__(self, device: int):
        super().__init__(daemon=True)
        self.samples, self.reasons, self.max_mhz, self.ok = [], set(), None, False
        self.stop_flag = threading.Event()
        try:
            import pynvml
            import torch
            pynvml.nvmlInit()
            self.nv = pynvml
            try:
                uuid = str(torch.cuda.get_device_properties(device).uuid)
                self.h = pynvml.nvmlDeviceGetHandleByUUID(("GPU-" + uuid).encode() if not uuid.startswith("GPU-") else uuid.encode())
            except Exception:
                self.h = pynvml.nvmlDeviceGetHandleByIndex(device)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
            self.ok = True
        except Exception:
            self.ok = False

    def run(self):
        if not self.ok:
            return
        while not self.stop_flag.is_set():
            try:
                self.samples.append(self.nv.nvmlDeviceGetClockInfo(self.h, self.nv.NVML_CLOCK_SM))
                get = getattr(self.nv, "nvmlDeviceGetCurrentClocksEventReasons", None) or \
                    self.nv.nvmlDeviceGetCurrentClocksThrottleReasons
                bits = get(self.h)
                for bit, name in self.REASONS.items():
                    if bits & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            time.sleep(0.002)

    def result(self) -> dict:
        self.stop_flag.set()
        if self.is_alive():
            self.join(timeout=1)
        if not self.samples:
            return dict(sm_mhz=None, sm_max_mhz=self.max_mhz, reasons=sorted(self.reasons), samples=0)
        return dict(sm_mhz=statistics.median(self.samples), sm_max_mhz=self.max_mhz, reasons=sorted(self.reasons),
                    samples=len(self.samples))


# ---------------------------------------------------------------- CPU baselines (rank 0, bounded samples)

_JOB = None  # (body, buffers, grid, block) of the oracle run the forked workers share


def _oracle_share(blocks):
    from oracle import fragment_oracle  # runs plain bodies as ir_oracle does, and the tensor-core statements
    body, bufs, grid, block = _JOB
    fragment_oracle.run(body, bufs, grid, block, blocks=blocks)
    return len(blocks)


def full_problem(workload: str) -> tuple:
    """(the authored problem at the one-GPU size, the arguments of its kernels from meta.json)."""
    from emmy_ptx import problems
    p = problems.WORKLOADS[workload.replace("_fused", "")]()
    meta = json.loads((PKG / "problems" / WORKLOADS[workload]["folder"] / "meta.json").read_text())
    return p, meta["kernels"]


def oracle_sample(workload: str, budget_s: float, workers: int, host: dict | None = None) -> dict:
    """Time the oracle on a bounded sample of the workload's blocks and extrapolate to the grid.
    The sample is a seeded random choice of blocks (so a workload whose blocks differ in cost - causal attention:
    the keys grow with the query - is sampled at its mean), taken in growing batches until the budget is used.
    ``workers`` > 1 interprets disjoint shares of a batch in that many forked processes (blocks are independent
    in the interpreter)."""
    global _JOB
    import multiprocessing as mp

    import numpy as np
    from emmy_ptx import runner
    from oracle import ir_oracle
    if WORKLOADS[workload].get("oracle") == "fragment":  # the interpreter's extension to the tensor-core statements
        from oracle import fragment_oracle as ir_oracle
    p, meta_args = full_problem(workload)
    total_us, notes, cores = 0.0, [], 1
    scale, reduced = 1.0, ""
    if host is None:  # the interpreter indexes the real buffers: generate the real inputs once
        host = {}
        for km in meta_args:
            host.update(runner.host_inputs(km["args"]))
    if workload.startswith("mlp"):
        # one CTA of the full problem walks 2048 hidden units of 4096-long dot products per thread: minutes in the
        # interpreter. Its cost is linear in the hidden units (every trip runs the same statements), so the sample is a
        # CTA of the same IR on the first 256 hidden units of the same weights, scaled by hidden / 256.
        from emmy_ptx import problems
        full_hidden, cut = host["w1"].shape[1], 256
        p = problems.gelu_mlp(tokens=host["x"].shape[0], d_model=host["x"].shape[1], hidden=cut)
        host = dict(host, w1=np.ascontiguousarray(host["w1"][:, :cut]), w2=np.ascontiguousarray(host["w2"][:cut]))
        scale, reduced = full_hidden / cut, f"on the first {cut} of {full_hidden} hidden units, times {full_hidden // cut}; "
    for kern in p["kernels"]:
        grid, block = kern["grid"], kern["block"]
        bufs = dict(host)
        for k2 in p["kernels"]:
            n2, s2, d2 = k2["output"]
            bufs.setdefault(n2, np.zeros(s2, runner.numpy_dtype(d2)))
        order = np.random.default_rng(12345).permutation(grid)
        share = budget_s / len(p["kernels"])
        done, spent, used = 0, 0.0, 1
        while done < grid and (done == 0 or spent < share):
            if done < 2:
                take = 1  # two single blocks first: their cost sizes the batches
            else:
                take = int(max(1, min(grid - done, (share - spent) / (spent / done) * (workers if done >= 4 else 1) * 0.8)))
            blocks = [int(b) for b in order[done:done + take]]
            t0 = time.perf_counter()
            if workers > 1 and len(blocks) >= 2 * workers:
                used = workers
                _JOB = (kern["body"], bufs, grid, block)
                with mp.get_context("fork").Pool(workers) as pool:
                    pool.map(_oracle_share, [blocks[i::workers] for i in range(workers)])
                # what one core would have needed for these blocks is not measured: the batch counts at its wall time
            else:
                ir_oracle.run(kern["body"], bufs, grid, block, blocks=blocks)
            spent += time.perf_counter() - t0
            done += len(blocks)
        total_us += spent / done * grid * 1e6 * scale
        cores = max(cores, used)
        notes.append(f"{kern['entry']}: {reduced}{done} of {grid} CTAs (seeded random choice) interpreted in {spent:.1f} s on up to {used} "
                     "core(s), scaled to the grid")
    return dict(value=total_us, unit="us", cores=cores, kind="port", sample="; ".join(notes) +
                " (oracle/ir_oracle.py: numpy restatement of the reference's interpreter; extrapolated)")


def f64_sample(workload: str, host: dict, budget_s: float = 3.0) -> dict | None:
    """The problem's expression in float64 torch on all host cores (how the reference makes its expected values,
    and what its tools time as the CPU figure): a slice of the sharded axis, timed and scaled to the whole."""
    import numpy as np
    import torch
    threads = torch.get_num_threads()

    def t64(a):
        if a.dtype == np.uint8:
            import ml_dtypes
            return torch.from_numpy(a.view(ml_dtypes.float8_e4m3fn).astype(np.float64))
        return torch.from_numpy(np.asarray(a, dtype=np.float64))

    def timed(fn, part: int, whole: int, what: str):
        fn()  # warm-up: threads, allocations
        reps, t0 = 0, time.perf_counter()
        while reps < 1 or (time.perf_counter() - t0 < budget_s / 3 and reps < 20):
            fn()
            reps += 1
        dt = (time.perf_counter() - t0) / reps
        return dict(value=dt * whole / part * 1e6, unit="us", cores=threads, kind="f64 expression (torch, float64)",
                    sample=f"{what}: {part} of {whole} in {dt * 1e3:.1f} ms, scaled")

    if workload in ("sum", "sum_scalar"):
        x = t64(host["x"].reshape(-1))
        return timed(lambda: x.sum(), x.numel(), x.numel(), "elements")
    if workload == "softmax":
        rows = 1024
        x = t64(host["x"][:rows])
        return timed(lambda: torch.softmax(x, dim=-1), rows, host["x"].shape[0], "rows")
    if workload == "elementwise":
        rows = 1024
        x, b = t64(host["x"][:rows]), t64(host["bias"])
        return timed(lambda: torch.nn.functional.gelu(x + b, approximate="tanh"), rows, host["x"].shape[0], "rows")
    if workload == "elementwise_add":
        rows = 1024
        x, b, r = t64(host["x"][:rows]), t64(host["bias"]), t64(host["res"][:rows])
        return timed(lambda: torch.relu(x + b) + r, rows, host["x"].shape[0], "rows")
    if workload in ("matmul", "fragments"):
        an, bn = ("a", "b") if workload == "matmul" else ("x0", "x1")
        rows = 256
        a, b = t64(host[an][:rows]), t64(host[bn])
        return timed(lambda: a @ b.T, rows, host[an].shape[0], "rows of A")
    if workload == "attention":
        q, k, v = (host[n].reshape(-1, *host[n].shape[-2:]) for n in "qkv")
        pairs = 1
        qq, kk, vv = t64(q[:pairs]), t64(k[:pairs]), t64(v[:pairs])
        return timed(lambda: torch.nn.functional.scaled_dot_product_attention(qq, kk, vv, is_causal=True), pairs, q.shape[0],
                     "(batch, head) pairs")
    if workload.startswith("mlp"):
        rows = 128
        x = t64(host["x"][:rows])
        w1, w2 = t64(host["w1"]) * float(host["w1_scale"][0]), t64(host["w2"]) * float(host["w2_scale"][0])
        return timed(lambda: torch.nn.functional.gelu(x @ w1, approximate="tanh") @ w2, rows, host["x"].shape[0], "token rows")
    return None


def reference_arm(args) -> None:
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    w = WORKLOADS[args.workload]
    steps = max(1, args.steps)
    vals = []
    base = None
    for _ in range(min(steps, 3)):  # each step is a bounded sample; more than a few repeats adds nothing
        base = oracle_sample(args.workload, budget_s=8.0, workers=os.cpu_count() or 1)
        vals.append(base["value"])
    value = statistics.median(vals)
    base["value"] = value
    line = dict(impl="reference", metric="us_per_kernel", value=value, unit="us", n_gpus=args.gpus, steps=len(vals),
                warmup=0, ms_per_step=value / 1000.0, higher_is_better=False, scaling="strong", vs_baseline=None,
                dtype=w["dtype"], data="synthetic", config=dict(workload=w["describe"], l2="n/a (CPU)"),
                cpu_baseline=base, e2e=dict(value=value, unit="us", h2d_bytes_per_step=0, d2h_bytes_per_step=0))
    print(json.dumps(line))


# ---------------------------------------------------------------- the GPU arm


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--workload", default="mlp", choices=sorted(WORKLOADS))
    ap.add_argument("--mode", default="optimized", choices=("optimized", "strict", "plain"))
    ap.add_argument("--exchange", default="fused", choices=("fused", "nccl"),
                    help="several GPUs, the array sum: combine the per-GPU scalars inside the last kernel, or by NCCL after it")
    ap.add_argument("--impl", default="ours", choices=("ours", "reference"))
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--buffer-sets", type=int, default=0, help="copies of every buffer the passes rotate through (0: enough "
                    "to exceed L2; 1 keeps device memory small for a profiler capture)")
    ap.add_argument("--families", default=None, help="comma-separated extra workloads measured after the headline one "
                    "(default: all of them; 'none' for the headline alone)")
    args = ap.parse_args()
    if args.impl == "reference":
        return reference_arm(args)

    import numpy as np
    import torch
    import torch.distributed as dist
    from emmy_ptx import driver, multi, pipeline, problems, runner

    rank, world = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if args.families is None:
        args.families = DEFAULT_FAMILIES
    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no CUDA device; the kernels run on the GPU only")
    torch.cuda.set_device(local)
    if world > 1:
        import datetime
        # a rank that dies must end the others' next collective within minutes, not NCCL's default ten
        dist.init_process_group("nccl", device_id=torch.device("cuda", local), timeout=datetime.timedelta(minutes=4))
    warmup = max(args.warmup, 3)
    pk, pk_kind = peaks()
    scratch_root = Path(tempfile.mkdtemp(prefix=f"emb_bench_r{rank}_"))

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def all_max(x: float) -> float:
        t = torch.tensor([x], dtype=torch.float64, device="cuda")
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    def agreed(ok: bool) -> bool:
        """Do ALL ranks say ok? (a rank that failed to build a workload must not leave the others in its collectives)"""
        t = torch.tensor([1 if ok else 0], device="cuda")
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MIN)
        return bool(int(t.item()))

    def build(workload: str, exchange):
        """The rank's share of the workload as a compiled problem bound to its shard of the seeded inputs:
        (problem, its sizes, the sharding plan or None when the workload is not sharded, the FULL problem's host inputs)."""
        w = WORKLOADS[workload]
        p_full, meta_full = full_problem(workload)
        if "sizes" in w:  # measured on one GPU only
            prefer = os.environ.get("EMMY_PTX_PREFER")
            if w.get("prefer"):
                os.environ["EMMY_PTX_PREFER"] = w["prefer"]
            try:
                prob = runner.Problem(PKG / "problems" / w["folder"], args.mode, device=local)
            finally:
                if w.get("prefer"):
                    os.environ.pop("EMMY_PTX_PREFER") if prefer is None else os.environ.update(EMMY_PTX_PREFER=prefer)
            return prob, dict(w["sizes"]), None, prob.host
        pl = multi.plan(workload, rank, world)
        kw = dict(multi.FULL_SIZES[workload], **pl["kwargs"])
        if world == 1:  # the whole problem: the folder written (and compiled) at build time
            prob = runner.Problem(PKG / "problems" / w["folder"], args.mode, device=local, exchange=exchange)
            return prob, kw, pl, prob.host
        shard = problems.WORKLOADS[workload](ident=f"{p_full['id']}_w{world}", **pl["kwargs"])
        folder = problems.write(shard, scratch_root)
        full_host = {}
        for km in meta_full:
            full_host.update(runner.host_inputs(km["args"]))
        shard_meta = json.loads((folder / "meta.json").read_text())["kernels"]
        inputs = multi.shard_inputs(pl, full_host, [a for km in shard_meta for a in km["args"]])
        prob = runner.Problem(folder, args.mode, device=local, inputs=inputs, exchange=exchange)
        return prob, kw, pl, full_host

    def check_exchange(prob, pl, full_host) -> dict:
        """The sum's exchanged result against the rank-order f32 sum of the per-rank scalars, bit for bit, on every
        buffer set (each holds what its last timed pass wrote), and against the f64 sum of the whole array."""
        finals = [prob.tensors["sum_1"]] + [c["sum_1"] for c in getattr(prob, "copies", [])]
        got = torch.stack([f.reshape(-1)[0] for f in finals])
        # this rank's own scalar: the same kernels on the same data with no exchange record
        alone = runner.Problem(prob.folder, args.mode, device=local, inputs=prob.host)
        mine = torch.from_numpy(alone.run()["sum_1"].reshape(-1)[:1].copy()).cuda()
        parts = [torch.empty_like(mine) for _ in range(world)]
        dist.all_gather(parts, mine)
        total = np.float32(parts[0].item())
        for q in parts[1:]:
            total = np.float32(total + np.float32(q.item()))
        want = np.float32(total).view(np.uint32)
        same = bool((got.cpu().numpy().view(np.uint32) == want).all())
        flag = torch.tensor([1 if same else 0], device="cuda")
        dist.all_reduce(flag, op=dist.ReduceOp.MIN)
        exact = float(np.sum(full_host["x"].astype(np.float64)))
        return dict(exchange_checked=bool(int(flag.item())), checked_buffer_sets=len(finals), exchanged_sum=float(total),
                    f64_sum=exact, within_1e5_sqrt_n=bool(abs(float(total) - exact) <= 1e-5 * (full_host["x"].size ** 0.5)))

    def measure(workload: str, steps: int):
        w = WORKLOADS[workload]
        exchange, how = None, None
        sharded_sum = workload == "sum" and world > 1
        if sharded_sum:
            # the one real exchange of the path: the per-GPU scalars are combined inside the sum's last kernel (peer stores
            # into symmetric memory, bounded wait); an NCCL all-reduce after the kernel only if that memory cannot be had
            if args.exchange == "fused":
                how, why = "in-kernel (peer stores + bounded wait, emb_peer.cuh)", ""
                try:
                    exchange = multi.PeerExchange.create()
                except Exception as e:  # every rank fails alike (no fabric / IPC handles on this box)
                    why = f": {type(e).__name__}: {e}"
                if not agreed(exchange is not None):  # all ranks take the same route
                    exchange, how = None, f"NCCL all-reduce after the kernel (symmetric memory unavailable{why})"[:240]
            else:
                how = "NCCL all-reduce after the kernel (--exchange nccl)"
        prob = kw = pl = full_host = None
        failure = None
        try:
            prob, kw, pl, full_host = build(workload, exchange)
        except Exception as e:  # noqa: BLE001 - reported in the family's entry; the other ranks skip it too
            failure = f"{type(e).__name__}: {e}"[:300]
        if not agreed(failure is None):
            raise RuntimeError(failure or "another rank could not build this workload")
        work = w["work"](kw)
        stream = prob.stream
        if args.buffer_sets == 1:
            nsets = 1
        else:  # the buffer sets together exceed the 126 MB L2: every pass is cold
            nsets = prob.rotate(min_bytes=512 << 20, max_sets=args.buffer_sets or 8)
        set_bytes = sum(t.numel() * t.element_size() for n, t in prob.tensors.items() if n != runner.EXCHANGE)
        nccl = sharded_sum and exchange is None
        barrier()
        if not nccl:
            total_us = prob.time_rotating_us(warmup=warmup, iters=1, batch=steps)[0] * steps
        else:
            finals = [prob.tensors["sum_1"]] + [c["sum_1"] for c in getattr(prob, "copies", [])]
            for i in range(warmup):
                driver.launch(prob.sets[i % nsets], stream)
                multi.combine_sum(finals[i % nsets], strict=args.mode == "strict")
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            for i in range(warmup, warmup + steps):
                driver.launch(prob.sets[i % nsets], stream)
                multi.combine_sum(finals[i % nsets], strict=args.mode == "strict")
            b.record()
            b.synchronize()
            total_us = a.elapsed_time(b) * 1000.0
        barrier()
        mean_us = all_max(total_us) / steps
        checked = check_exchange(prob, pl, full_host) if sharded_sum and not nccl else None
        per_launch = prob.time_rotating_us(warmup=3, iters=max(10, min(steps, 50)), batch=1)  # one event pair per pass
        # the dominant kernel alone over the same kind of timed region, for the roofline (the pass itself when it is one launch)
        entries = [(e, k) for k in prob.kernels for e in [p_["entry"] for p_ in k.launch_info.get("pre", ())] + [k.meta["entry"]]]
        dominant = w["dominant"] if isinstance(w["dominant"], int) else [e for e, _ in entries].index(w["dominant"])
        if len(prob.launches) == 1 and not nccl:
            dom_us = mean_us
        else:
            dom_us = all_max(prob.time_rotating_us(warmup=warmup, iters=1, batch=steps, only=dominant)[0])
        if w["bound"] == "hbm":
            achieved = work["bytes"] / dom_us / 1e3  # GB/s
            peak, unit = float(pk["hbm_gbs"]), "GB/s"
            whole = work["bytes"] * 1.0
        else:
            achieved = work["flops"] / dom_us / 1e6  # TFLOP/s
            # a timed region of seconds runs under the power cap: the sustained cuBLAS figure is the denominator then
            long_run = steps * mean_us > 1e6 and "bf16_tflops_sustained" in pk
            peak, unit = float(pk["bf16_tflops_sustained" if long_run else "bf16_tflops"]), "TFLOP/s"
            whole = work.get("chain_flops", work["flops"]) * 1.0
        dom_entry, dom_kernel = entries[dominant]
        traffic = NCU_TRAFFIC.get(workload)
        roof = dict(bound=w["bound"], achieved=achieved, peak=peak, unit=unit, frac=achieved / peak,
                    traffic=traffic if world == 1 else None, kernel=dom_entry, kernel_us=dom_us,
                    peak_source=f"of {pk_kind}", family=dom_kernel.launch_info.get("family"),
                    work_per_launch=work.get("bytes", work.get("flops")))
        timing = dict(buffer_sets=nsets, bytes_per_set=set_bytes, us_per_pass_with_an_event_pair_each=statistics.median(per_launch))
        if how:
            timing["exchange"] = how
        if checked:
            timing.update(checked)
        # whole-job rate: every rank's share of the work over the slowest rank's time
        total_work = torch.tensor([whole], dtype=torch.float64, device="cuda")
        if world > 1:
            dist.all_reduce(total_work, op=dist.ReduceOp.SUM)
        rate = float(total_work.item()) / mean_us / (1e3 if w["bound"] == "hbm" else 1e6)
        aggregate = dict(value=rate, unit="GB/s" if w["bound"] == "hbm" else "TFLOP/s")

        # ---- end to end: the step's inputs from pinned host memory, the launches, the result back to the host
        # operands the sharding replicates are the job's parameters, resident on every GPU at every world size
        resident = sorted(n for n in prob.host if pl is not None and n not in pl["slices"])
        moving = [n for n in prob.host if n not in resident]
        ins = {n: prob.tensors[n] for n in moving}
        pinned = {n: torch.empty(t.shape, dtype=t.dtype, device="cpu", pin_memory=True).copy_(t.cpu()) for n, t in ins.items()}
        outs = [a["name"] for a in prob.meta["kernels"][-1]["args"] if a.get("output")]
        out_host = {n: torch.empty(prob.tensors[n].shape, dtype=prob.tensors[n].dtype, device="cpu", pin_memory=True) for n in outs}
        h2d = sum(t.numel() * t.element_size() for t in pinned.values())
        d2h = sum(t.numel() * t.element_size() for t in out_host.values())
        reps = max(3, min(steps, 10))
        times = []
        # rows are independent in a row-wise kernel: the public API pipelines slices of rows (copy in, launch, copy out on a
        # few streams) so that both directions of the host link and the GPU work at once
        pipelined = prob.rows_pipeline(chunks=8, streams=4)
        chunked = None
        if pipelined is None and pl is not None and workload in CHUNKED and exchange is None:
            # several launches, tensor maps: the same overlap by compiling the rank's share in slices of its units
            try:
                chunked = pipeline.ChunkedProblem(workload, kw, prob.host, args.mode, local, chunks=pipeline.slice_count(len(pl["share"])),
                                                  streams=4, root=scratch_root)
            except Exception as e:  # noqa: BLE001 - the plain sequence below still measures the call
                chunked = None
                timing["chunked_e2e_unavailable"] = f"{type(e).__name__}: {e}"[:200]
        barrier()
        for i in range(2 + reps):
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            if pipelined is not None:
                pipelined(pinned, out_host)
            elif chunked is not None:
                chunked.run(pinned, out_host)
            else:
                for n, t in pinned.items():
                    ins[n].copy_(t, non_blocking=True)
                driver.launch(prob.launches, stream)
                for n in outs:
                    out_host[n].copy_(prob.tensors[n], non_blocking=True)
            b.record()
            b.synchronize()
            if i >= 2:
                times.append(a.elapsed_time(b) * 1000.0)
        barrier()
        e2e = dict(value=all_max(statistics.mean(times)), unit="us", h2d_bytes_per_step=int(all_sum(h2d)), d2h_bytes_per_step=int(all_sum(d2h)),
                   resident=resident,
                   how=("8 row slices on 4 streams: copy in, launch, copy out overlap" if pipelined is not None else
                        f"{len(chunked.parts)} slices of the units, each compiled for its size, on 4 streams: copy in, launches, copy out overlap; "
                        "preparation of resident operands (weight decode) once per step" if chunked is not None else
                        "copy in, launches, copy out on one stream") + "; bytes are the sum over ranks")
        if chunked is not None:
            chunked.check_status()
        del pinned, out_host, chunked
        return dict(prob=prob, kw=kw, pl=pl, host=full_host, mean_us=mean_us, timing=timing, roofline=roof, e2e=e2e,
                    aggregate=aggregate)

    def all_sum(x: float) -> float:
        t = torch.tensor([float(x)], dtype=torch.float64, device="cuda")
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.SUM)
        return float(t.item())

    def cpu_legs(workload: str, host: dict, budget_s: float) -> tuple:
        """(oracle port on one core, f64 expression on all cores), on rank 0 of a one-GPU run only."""
        if rank != 0 or world != 1 or args.no_cpu_baseline:
            return None, None
        try:
            port = oracle_sample(workload, budget_s=budget_s, workers=1, host=host)
        except Exception as e:  # noqa: BLE001
            port = dict(error=f"{type(e).__name__}: {e}"[:200])
        try:
            f64 = f64_sample(workload, host)
        except Exception as e:  # noqa: BLE001
            f64 = dict(error=f"{type(e).__name__}: {e}"[:200])
        return port, f64

    def sharding_note(workload: str, m: dict) -> str:
        if world == 1:
            return "one GPU: the whole problem"
        if m["pl"] is None:
            return "not sharded: every rank runs the whole problem"
        pl = m["pl"]
        return (f"strong: rank r of {world} owns multi.shard({pl['units']} units, r, {world}) of the {pl['axis']} "
                f"(rank 0: {len(pl['share'])} units = {m['kw']}); compiled for the shard's size")

    sampler = ClockSampler(local)
    sampler.start()
    head = measure(args.workload, args.steps)
    clocks = sampler.result()
    w = WORKLOADS[args.workload]
    launches = args.steps * head["prob"].launch_count()
    cpu, cpu64 = cpu_legs(args.workload, head["host"], 10.0)
    head_note = sharding_note(args.workload, head)
    head_bytes = head["timing"]["bytes_per_set"]
    head.pop("prob")
    head.pop("host")
    torch.cuda.empty_cache()

    families = []
    names = [f for f in args.families.split(",") if f and f != "none" and f != args.workload and f in WORKLOADS]
    for name in names:
        fw = WORKLOADS[name]
        if world > 1 and "sizes" in fw:
            continue
        try:
            m = measure(name, min(args.steps, 30))
            port, f64 = cpu_legs(name, m["host"], 3.0)
            families.append(dict(workload=fw["describe"], name=name, us_per_pass=m["mean_us"], whole_chain=m["aggregate"],
                                 timing=m["timing"], roofline=m["roofline"], e2e=m["e2e"], cpu_baseline=port, cpu_baseline_f64=f64,
                                 launches_per_pass=m["prob"].launch_count(), sharding=sharding_note(name, m)))
            del m
        except Exception as e:  # an extra line must not cost the headline one
            families.append(dict(workload=fw["describe"], name=name, error=f"{type(e).__name__}: {e}"[:300]))
        torch.cuda.empty_cache()

    if rank == 0:
        line = dict(metric="us_per_kernel", value=head["mean_us"], unit="us", n_gpus=world, steps=args.steps, warmup=warmup,
                    ms_per_step=head["mean_us"] / 1000.0, higher_is_better=False, scaling="strong", vs_baseline=None, dtype=w["dtype"],
                    data="synthetic", timing=head["timing"],
                    config=dict(workload=w["describe"], mode=args.mode,
                                l2=f"inputs larger than L2: passes rotate through {head['timing']['buffer_sets']} buffer sets of "
                                   f"{head_bytes >> 20} MiB, no flush",
                                sharding=head_note),
                    roofline=head["roofline"], cpu_baseline=cpu, cpu_baseline_f64=cpu64, e2e=head["e2e"], gpu_launches=launches,
                    clocks=clocks, families=families, aggregate=head["aggregate"])
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
