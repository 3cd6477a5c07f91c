#!/usr/bin/env python3
"""Benchmark of the hot path: one pass of a workload's kernel chain per step, on 1..8 GPUs.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload softmax|sum|...] [--mode optimized|strict]
    python bench.py --impl reference ...      # the CPU interpreter of the same IR on the host cores

One JSON line on stdout (rank 0). ``value`` is microseconds per pass of the workload's kernel
chain with the inputs resident in HBM: K passes back to back between one CUDA event pair on the
launching stream, the passes rotating through enough copies of every buffer that none finds its
data in L2, max over ranks; ``e2e`` is the same pass through the public API from HOST buffers
(pinned host -> device copy of the inputs, the launches, device -> host copy of the result, all
inside the event pair); ``roofline`` is the dominant kernel's algorithmic bytes per launch over
its measured duration against the measured HBM peak; ``cpu_baseline`` is the oracle (a port of the
reference's numpy interpreter) timed on a bounded sample of the same workload.

Multi-GPU: launched by torchrun with one rank per GPU. The workloads shard without any data-path
exchange (rows, batch*heads, element ranges), every rank runs the full single-GPU workload on its
own shard of an N-times larger job (weak scaling); the array sum adds its one exchange: the per-GPU
scalars are combined inside the sum's last kernel by peer stores into symmetric memory and a bounded
wait (``--exchange nccl``, or a box without such memory: an NCCL all-reduce after the kernel).
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
PKG = ROOT / "emmy-ptx-compiler_b200"
for p in (PKG, ROOT):
    if str(p) not in sys.path:
        sys.path.insert(0, str(p))

WORKLOADS = {
    # name: (problem folder, algorithmic bytes of the dominant kernel per launch, unit work for the tensor ones)
    "softmax": dict(folder="f_softmax_8192x4096", bound="hbm", bytes=2 * 8192 * 4096 * 4, dominant=0, dtype="f32",
                    describe="row softmax [8192,4096] f32 (BASELINE configs[1])"),
    "sum": dict(folder="r_sum_16m", bound="hbm", bytes=(1 << 24) * 4, dominant=0, dtype="f32",
                describe="f32 array sum of 2^24 (BASELINE configs[0]): block partials + final fold"),
    "matmul": dict(folder="m_f16_8192", bound="tensor", flops=2 * 8192 ** 3, dominant=0, dtype="f16",
                   describe="f16 GEMM 8192^3, f32 accumulate (BASELINE configs[2])"),
    "attention": dict(folder="a_f16_causal_8x32x4096x128", bound="tensor", flops=4 * 8 * 32 * 128 * 4096 * 4097 // 2,
                      dominant=0, dtype="f16", describe="causal attention 8x32x4096x128 f16 (BASELINE configs[3])"),
    # the chain is decode w1, decode w2, h = gelu(x w1), y = h w2: the two matmuls weigh the same; the roofline kernel is the first
    "mlp": dict(folder="k_mlp_gelu_tanh_16384x4096x16384", bound="tensor", flops=2 * 16384 * 4096 * 16384, dominant=2,
                chain_flops=2 * 2 * 16384 * 4096 * 16384, dtype="bf16",
                describe="GELU MLP 16384x4096x16384, bf16 x, e4m3 weights decoded to bf16, bf16 tcgen05 MMA (BASELINE configs[4])"),
    # the same product handed over as a warp-level mma.sync schedule (fragment form) plus its fold kernel: optimized mode proves
    # it a matmul and runs the tcgen05 template, --mode plain runs the schedule as written (what the reference's lowering emits)
    "fragments": dict(folder="m_f16_8192_fragments", bound="tensor", flops=2 * 8192 ** 3, dominant=0, dtype="f16", oracle="fragment",
                      describe="f16 GEMM 8192^3 given in fragment form (mma.sync schedule, B stored N x K) + fold kernel"),
}
# dram__bytes_read.sum + dram__bytes_write.sum per launch of the dominant kernel, from the ncu
# captures summarised under profiles/ (None until captured)
NCU_TRAFFIC = {"softmax": 212.3e6, "sum": 67.5e6, "matmul": 1253.1e6, "attention": 1056.2e6, "mlp": 1723.4e6, "fragments": 1326.0e6}
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


_JOB = None  # (body, buffers, grid, block) of the oracle run the forked workers share


def _oracle_share(blocks):
    from oracle import fragment_oracle  # runs plain bodies as ir_oracle does, and the tensor-core statements
    body, bufs, grid, block = _JOB
    fragment_oracle.run(body, bufs, grid, block, blocks=blocks)
    return len(blocks)


def oracle_sample(workload: str, budget_s: float, workers: int) -> dict:
    """Time the oracle on a bounded sample of the workload's blocks and extrapolate to the grid.
    ``workers`` > 1 interprets disjoint shares of the sample in that many forked processes (blocks are
    independent in the interpreter)."""
    global _JOB
    import multiprocessing as mp

    import numpy as np
    from emmy_ptx import problems, runner
    from oracle import ir_oracle
    if WORKLOADS[workload].get("oracle") == "fragment":  # the interpreter's extension to the tensor-core statements
        from oracle import fragment_oracle as ir_oracle
    make = problems.WORKLOADS[workload]
    p = make()
    meta_args = json.loads((PKG / "problems" / WORKLOADS[workload]["folder"] / "meta.json").read_text())["kernels"]
    total_us, notes = 0.0, []
    host = None
    for kern, km in zip(p["kernels"], meta_args):
        grid, block = kern["grid"], kern["block"]
        if host is None:  # the interpreter indexes the real buffers: generate the real inputs once
            host = runner.host_inputs(km["args"])
        bufs = dict(host)
        for k2 in p["kernels"]:
            n2, s2, d2 = k2["output"]
            bufs.setdefault(n2, np.zeros(s2, runner.numpy_dtype(d2)))
        probe = max(1, min(grid, 2))
        t0 = time.perf_counter()
        ir_oracle.run(kern["body"], bufs, grid, block, blocks=range(probe))
        per_block = (time.perf_counter() - t0) / probe
        sample = int(max(probe, min(grid, workers * budget_s / max(per_block, 1e-9) / len(p["kernels"]))))
        step = max(1, grid // sample)
        blocks = list(range(0, grid, step))[:sample]
        used = max(1, min(workers, len(blocks)))
        t0 = time.perf_counter()
        if used == 1:
            ir_oracle.run(kern["body"], bufs, grid, block, blocks=blocks)
        else:
            _JOB = (kern["body"], bufs, grid, block)
            with mp.get_context("fork").Pool(used) as pool:
                pool.map(_oracle_share, [blocks[i::used] for i in range(used)])
        dt_s = time.perf_counter() - t0
        total_us += dt_s / len(blocks) * grid * 1e6
        notes.append(f"{kern['entry']}: {len(blocks)} of {grid} CTAs interpreted in {dt_s:.1f} s on {used} core(s), scaled to the grid")
    return dict(value=total_us, unit="us", cores=max(1, workers), kind="port", sample="; ".join(notes) +
                " (oracle/ir_oracle.py: numpy restatement of the reference's interpreter; extrapolated)")


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
                warmup=0, ms_per_step=value / 1000.0, higher_is_better=False, scaling="weak", vs_baseline=None,
                dtype=w["dtype"], data="synthetic", config=dict(workload=w["describe"], l2="n/a (CPU)"),
                cpu_baseline=base, e2e=dict(value=value, unit="us", h2d_bytes_per_step=0, d2h_bytes_per_step=0))
    print(json.dumps(line))


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--workload", default="softmax", choices=sorted(WORKLOADS))
    ap.add_argument("--mode", default="optimized", choices=("optimized", "strict", "plain"))
    ap.add_argument("--exchange", default="fused", choices=("fused", "nccl"),
                    help="several GPUs, the array sum: combine the per-GPU scalars inside the last kernel, or by NCCL after it")
    ap.add_argument("--impl", default="ours", choices=("ours", "reference"))
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--buffer-sets", type=int, default=0, help="copies of every buffer the passes rotate through (0: enough "
                    "to exceed L2; 1 keeps device memory small for a profiler capture)")
    ap.add_argument("--families", default=None, help="comma-separated extra workloads measured after the headline one "
                    "(default: all of them on one GPU, the array sum with its exchange on several)")
    args = ap.parse_args()
    if args.impl == "reference":
        return reference_arm(args)

    import torch
    import torch.distributed as dist
    from emmy_ptx import driver, multi, runner

    rank, world = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if args.families is None:
        args.families = "sum,matmul,fragments,attention,mlp" if world == 1 else "sum"
    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no CUDA device; the kernels run on the GPU only")
    torch.cuda.set_device(local)
    if world > 1:
        import datetime
        # a rank that dies must end the others' next collective within minutes, not NCCL's default ten
        dist.init_process_group("nccl", device_id=torch.device("cuda", local), timeout=datetime.timedelta(minutes=4))
    warmup = max(args.warmup, 3)
    pk, pk_kind = peaks()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def measure(workload: str, steps: int, with_e2e: bool):
        w = WORKLOADS[workload]
        exchange, how = None, None
        if workload == "sum" and world > 1:
            # the one real exchange of the path: the per-GPU scalars are combined inside the sum's last kernel (peer stores
            # into symmetric memory, bounded wait); an NCCL all-reduce after the kernel only if that memory cannot be had
            how = "in-kernel (peer stores + bounded wait, emb_peer.cuh)"
            if args.exchange == "fused":
                try:
                    exchange = multi.PeerExchange.create()
                except Exception as e:  # every rank fails alike (no fabric / IPC handles on this box)
                    how = f"NCCL all-reduce after the kernel (symmetric memory unavailable: {type(e).__name__}: {e})"[:240]
            else:
                how = "NCCL all-reduce after the kernel (--exchange nccl)"
            agreed = torch.tensor([0 if exchange is None else 1], device="cuda")
            dist.all_reduce(agreed, op=dist.ReduceOp.MIN)  # all ranks take the same route
            if exchange is not None and int(agreed.item()) == 0:
                exchange, how = None, "NCCL all-reduce after the kernel (symmetric memory unavailable on another rank)"
        prob = runner.Problem(PKG / "problems" / w["folder"], args.mode, device=local, exchange=exchange)
        stream = prob.stream
        if args.buffer_sets == 1:
            nsets = 1
        else:  # the buffer sets together exceed the 126 MB L2: every pass is cold
            nsets = prob.rotate(min_bytes=512 << 20, max_sets=args.buffer_sets or 8)
        set_bytes = sum(t.numel() * t.element_size() for n, t in prob.tensors.items() if n != runner.EXCHANGE)
        nccl = workload == "sum" and world > 1 and exchange is None
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
        total = torch.tensor([total_us], dtype=torch.float64, device="cuda")
        if world > 1:
            dist.all_reduce(total, op=dist.ReduceOp.MAX)
        mean_us = float(total.item()) / steps
        per_launch = prob.time_rotating_us(warmup=3, iters=max(10, min(steps, 50)), batch=1)  # one event pair per pass
        # the dominant kernel alone over the same kind of timed region, for the roofline (the pass itself when it is one launch)
        entries = [e for k in prob.kernels for e in [p_["entry"] for p_ in k.launch_info.get("pre", ())] + [k.meta["entry"]]]
        if len(prob.launches) == 1 and not nccl:
            dom_us = mean_us
        else:
            dom_us = prob.time_rotating_us(warmup=warmup, iters=1, batch=steps, only=w["dominant"])[0]
        if w["bound"] == "hbm":
            achieved = w["bytes"] / dom_us / 1e3  # GB/s
            peak, unit = float(pk["hbm_gbs"]), "GB/s"
        else:
            achieved = w["flops"] / dom_us / 1e6  # TFLOP/s
            # a timed region of seconds runs under the power cap: the sustained cuBLAS figure is the denominator then
            long_run = steps * mean_us > 1e6 and "bf16_tflops_sustained" in pk
            peak, unit = float(pk["bf16_tflops_sustained" if long_run else "bf16_tflops"]), "TFLOP/s"
        roof = dict(bound=w["bound"], achieved=achieved, peak=peak, unit=unit, frac=achieved / peak,
                    traffic=NCU_TRAFFIC.get(workload), kernel=entries[w["dominant"]], kernel_us=dom_us,
                    peak_source=f"of {pk_kind}", family=prob.kernels[-1 if w["dominant"] else 0].launch_info.get("family"))
        timing = dict(buffer_sets=nsets, bytes_per_set=set_bytes, us_per_pass_with_an_event_pair_each=statistics.median(per_launch))
        if how:
            timing["exchange"] = how
        e2e = None
        if with_e2e:
            ins = {n: prob.tensors[n] for n in prob.host}
            pinned = {n: torch.empty(t.shape, dtype=t.dtype, device="cpu", pin_memory=True).copy_(t.cpu()) for n, t in ins.items()}
            outs = [a["name"] for a in prob.meta["kernels"][-1]["args"] if a.get("output")]
            out_host = {n: torch.empty(prob.tensors[n].shape, dtype=prob.tensors[n].dtype, device="cpu", pin_memory=True) for n in outs}
            h2d = sum(t.numel() * t.element_size() for t in pinned.values())
            d2h = sum(t.numel() * t.element_size() for t in out_host.values())
            reps = max(3, min(steps, 10))
            times = []
            # rows are independent in this workload's kernel: the public API pipelines slices of rows (copy in, launch,
            # copy out on a few streams) so that both directions of the host link and the GPU work at once
            pipelined = prob.rows_pipeline(chunks=8, streams=4)
            barrier()
            for i in range(2 + reps):
                a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                a.record()
                if pipelined is not None:
                    pipelined(pinned, out_host)
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
            t_e2e = torch.tensor([statistics.mean(times)], dtype=torch.float64, device="cuda")
            if world > 1:
                dist.all_reduce(t_e2e, op=dist.ReduceOp.MAX)
            e2e = dict(value=float(t_e2e.item()), unit="us", h2d_bytes_per_step=h2d, d2h_bytes_per_step=d2h,
                       how="8 row slices on 4 streams: copy in, launch, copy out overlap" if pipelined is not None else
                           "copy in, launches, copy out on one stream")
        return prob, mean_us, timing, roof, e2e

    sampler = ClockSampler(local)
    sampler.start()
    prob, mean_us, timing, roof, e2e = measure(args.workload, args.steps, True)
    clocks = sampler.result()
    w = WORKLOADS[args.workload]
    launches = args.steps * prob.launch_count()

    families = []
    for name in [f for f in args.families.split(",") if f and f != "none" and f != args.workload and f in WORKLOADS]:
        try:
            fp, f_mean, f_med, f_roof, _ = measure(name, min(args.steps, 30), False)
            fw = WORKLOADS[name]
            whole = (fw.get("bytes", 0) / f_mean / 1e3) if fw["bound"] == "hbm" else fw.get("chain_flops", fw["flops"]) / f_mean / 1e6
            families.append(dict(workload=fw["describe"], us_per_pass=f_mean, whole_chain=dict(
                                 value=whole, unit="GB/s" if fw["bound"] == "hbm" else "TFLOP/s"), timing=f_med, roofline=f_roof,
                                 launches_per_pass=fp.launch_count()))
        except Exception as e:  # an extra line must not cost the headline one
            families.append(dict(workload=name, error=f"{type(e).__name__}: {e}"[:300]))

    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        cpu = oracle_sample(args.workload, budget_s=12.0, workers=1)
    if rank == 0:
        line = dict(metric="us_per_kernel", value=mean_us, unit="us", n_gpus=world, steps=args.steps, warmup=warmup,
                    ms_per_step=mean_us / 1000.0, higher_is_better=False, scaling="weak", vs_baseline=None, dtype=w["dtype"],
                    data="synthetic", timing=timing,
                    config=dict(workload=w["describe"], mode=args.mode,
                                l2=f"inputs larger than L2: passes rotate through {timing['buffer_sets']} buffer sets of "
                                   f"{timing['bytes_per_set'] >> 20} MiB, no flush",
                                sharding=f"weak: each rank runs the full workload on its own {multi.SHARDED_AXIS[args.workload]}"),
                    roofline=roof, cpu_baseline=cpu, e2e=e2e, gpu_launches=launches, clocks=clocks, families=families,
                    aggregate=dict(value=(w.get("bytes", 0) * world / mean_us / 1e3) if w["bound"] == "hbm" else
                                   (w.get("chain_flops", w["flops"]) * world / mean_us / 1e6),
                                   unit="GB/s" if w["bound"] == "hbm" else "TFLOP/s"))
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
