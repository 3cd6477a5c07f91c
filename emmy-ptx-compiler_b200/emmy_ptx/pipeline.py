"""A problem run in slices so that host copies and kernels overlap.

The reference's runner receives a problem's inputs with the request and returns its outputs with the answer
(tools/run_suite.py:77-111); a local host that holds its data in host memory pays the copies itself. For a workload
whose units are independent (the rows, pairs or token rows ``multi.plan`` shards over GPUs) the same cut works
inside one GPU: ``ChunkedProblem`` compiles the workload for a slice of the units, once per slice, and ``run``
walks the slices on a few streams - copy in, launch, copy out - so a slice's copies overlap its neighbours'
kernels and the copies of the opposite direction. Operands every slice needs whole (weights, scales, a bias
row: what a sharded run replicates) are uploaded once and shared, and launches that only prepare such operands
(the MLP's weight decode) run once per ``run``, not once per slice.
"""

from __future__ import annotations

import json
import tempfile
from pathlib import Path

from . import driver, multi, problems, runner


def slice_count(units: int) -> int:
    """How many slices a share of ``units`` is cut into for the end-to-end pipeline: eight where a slice still holds at
    least eight units (1024 rows of a matmul: enough tiles for every SM), else four. Measured on the GELU MLP
    (16384 x 4096 x 16384, host to host): 4 slices on 3 streams 5167 us, 6 on 3: 4020, 8 on 3: 4204, 8 on 4: 3767,
    16 on 4: 3667 us - the first slice's copy in and the last one's copy out are what is not overlapped."""
    return 8 if units >= 64 else 4


class ChunkedProblem:
    def __init__(self, workload: str, sizes: dict, host: dict, mode: str = "optimized", device: int = 0, chunks: int = 4,
                 streams: int = 3, root=None):
        """``sizes``: the builder's size arguments of the whole problem (``multi.FULL_SIZES`` keys); ``host``: its inputs
        as numpy arrays (``runner.host_inputs``)."""
        import torch
        self.device = torch.device("cuda", device)
        self.root = Path(root) if root else Path(tempfile.mkdtemp(prefix="emb_chunks_"))
        units = multi.plan(workload, 0, 1, sizes)["units"]
        chunks = max(1, min(chunks, units))
        self.plans = [multi.plan(workload, c, chunks, sizes) for c in range(chunks)]
        self.resident = sorted(n for n in host if n not in self.plans[0]["slices"])
        self.parts, shared = [], {}
        for c, pl in enumerate(self.plans):
            sub = problems.WORKLOADS[workload](ident=f"{workload}_{c}of{chunks}", **pl["kwargs"])
            folder = problems.write(sub, self.root)
            args = [a for km in json.loads((folder / "meta.json").read_text())["kernels"] for a in km["args"]]
            prob = runner.Problem(folder, mode, device, inputs=multi.shard_inputs(pl, host, args), share=shared)
            launches = list(prob.launches)
            prepare = [l for l in launches if l.scratch and set(l.buffers) <= set(self.resident) | set(l.scratch_names())]
            if c == 0:
                for n in self.resident:
                    shared[n] = prob.tensors[n]
                for l in prepare:
                    for key in l.scratch:
                        shared[key] = prob.tensors[key]
                self.prepare = prepare
            work = [l for l in launches if l not in prepare]
            self.parts.append((pl, prob, work))
        self.outputs = [a["name"] for a in self.parts[0][1].meta["kernels"][-1]["args"] if a.get("output")]
        self.pool = [torch.cuda.Stream(self.device) for _ in range(max(1, min(streams, chunks)))]

    def run(self, host_in: dict, host_out: dict) -> None:
        """``host_in`` / ``host_out``: name -> pinned host tensor of the WHOLE problem's shape (only the sliced operands
        are read; the resident ones were uploaded at construction). Enqueues everything and makes the current stream
        wait for it; the caller synchronizes."""
        import torch
        main = torch.cuda.current_stream(self.device)
        start = torch.cuda.Event()
        start.record(main)
        ready = None
        if self.prepare:  # once per run, ahead of every slice's kernels
            first = self.pool[0]
            first.wait_event(start)
            driver.launch(self.prepare, first.cuda_stream)
            ready = torch.cuda.Event()
            ready.record(first)
        for idx, (pl, prob, work) in enumerate(self.parts):
            s = self.pool[idx % len(self.pool)]
            s.wait_event(start)
            with torch.cuda.stream(s):
                for name, (lo, count) in pl["slices"].items():
                    lead = pl["reshape"].get(name)
                    src = (host_in[name].reshape(lead) if lead else host_in[name])[lo:lo + count]
                    prob.tensors[name].view(src.shape).copy_(src, non_blocking=True)
                if ready is not None:
                    s.wait_event(ready)
                driver.launch(work, s.cuda_stream)
                for name in self.outputs:
                    lo, count = self.out_slice(pl, host_out[name], prob.tensors[name])
                    host_out[name].reshape(-1)[lo:lo + count].copy_(prob.tensors[name].reshape(-1), non_blocking=True)
        for s in self.pool:
            main.wait_stream(s)

    @staticmethod
    def out_slice(pl: dict, whole, part) -> tuple:
        """Where a slice's output lies in the whole output, in elements: outputs are cut along the sharded units in
        order, so a slice's elements are a contiguous run proportional to its units."""
        per_unit = whole.numel() // pl["units"]
        return pl["share"].start * per_unit, part.numel()

    def check_status(self) -> None:
        for _, prob, _ in self.parts:
            prob.check_status()
