"""The local runner: what the reference's remote service did, on this machine's GPU.

The reference posts PTX to an HTTP service that assembles it (``/compile``) and
launches it (``/run``) with inputs made from the ``seed`` of each argument in
``meta.json`` (tools/run_suite.py:66-111; inputs are
``np.random.default_rng(seed).standard_normal(shape).astype(dtype)``, checked
against the shipped ``expected.npz`` files). ``Problem`` does the same locally:
compile every kernel of the folder (compile.py's ``compile_file``), assemble
with ptxas, load through libemmyb200.so, allocate torch tensors for the
arguments, chain ``intermediate`` arguments from the kernel that produced them
(:81-85), zero the ``zero_outputs``, launch in order, and time with CUDA events
(median of 20 after 3 warm-ups is the reference's protocol, :91).

Additions to ``meta.json`` arguments understood here (all optional): ``dist``
("normal" default, "uniform_pm1"), ``scale`` (multiplies the draw), ``quant``
(per-tensor e4m3 quantisation; names the argument that receives the scale) and
``scale_of``. The launch itself comes from the module's ``// launch:`` header
when it has one (a template may need its own geometry, a cluster size, dynamic
shared memory or tensor maps), else from ``meta.json`` as in the reference.
"""

from __future__ import annotations

import json
import re
from pathlib import Path

import numpy as np

from . import compile_file, driver, toolchain

TORCH_DTYPE = {"f32": "float32", "f64": "float64", "f16": "float16", "bf16": "bfloat16", "i32": "int32", "i64": "int64",
               "u8": "uint8", "i8": "int8", "i16": "int16", "bool": "uint8", "f8e4m3": "uint8", "f8e5m2": "uint8"}
NUMPY_DTYPE = {"f32": np.float32, "f64": np.float64, "f16": np.float16, "i32": np.int32, "i64": np.int64, "u8": np.uint8,
               "i8": np.int8, "i16": np.int16, "u32": np.uint32, "bool": np.uint8}


def numpy_dtype(name: str):
    if name == "bf16":
        import ml_dtypes
        return ml_dtypes.bfloat16
    if name in ("f8e4m3", "f8e5m2"):
        return np.uint8
    return NUMPY_DTYPE[name]


def quantize_e4m3(w: np.ndarray) -> tuple:
    """Per-tensor e4m3 codes and f32 scale: s = max|w| / 448, code = e4m3(w / s), round to nearest
    even, saturating at +-448 (the encode of emmy_ptx/elementwise.py:113-123; ml_dtypes would give
    NaN past 464, so the quotient is clamped first)."""
    import ml_dtypes
    s = np.float32(np.max(np.abs(w)) / 448.0)
    q = np.clip(w.astype(np.float32) / s, -448.0, 448.0)
    return q.astype(ml_dtypes.float8_e4m3fn).view(np.uint8), s


def host_inputs(args: list) -> dict:
    """name -> numpy array for every argument that is neither an output nor an intermediate."""
    out, scales = {}, {}
    for a in args:
        if a.get("output") or a.get("intermediate") or "scale_of" in a or "scale_product" in a:
            continue
        if "data" in a:
            out[a["name"]] = np.array(a["data"], numpy_dtype(a["dtype"])).reshape(a["shape"])
            continue
        rng = np.random.default_rng(a.get("seed", 0))
        if a.get("dist", "normal") == "uniform_pm1":
            draw = rng.uniform(-1.0, 1.0, a["shape"])
        else:
            draw = rng.standard_normal(a["shape"])
        if "scale" in a:
            draw = draw * a["scale"]
        if "quant" in a:
            codes, s = quantize_e4m3(draw.astype(np.float32))
            out[a["name"]] = codes
            scales[a["name"]] = s
        else:
            out[a["name"]] = draw.astype(numpy_dtype(a["dtype"]))
    for a in args:
        if "scale_of" in a:
            out[a["name"]] = np.array([scales[a["scale_of"]]], np.float32)
        elif "scale_product" in a:
            out[a["name"]] = np.array([np.prod([np.float32(scales[n]) for n in a["scale_product"]], dtype=np.float32)], np.float32)
    return out


def to_torch(array: np.ndarray, dtype: str, device):
    import torch
    if dtype == "bf16":
        return torch.from_numpy(array.view(np.int16).copy()).view(torch.bfloat16).to(device)
    return torch.from_numpy(np.ascontiguousarray(array)).to(device)


def to_numpy(tensor, dtype: str) -> np.ndarray:
    import torch
    t = tensor.detach().cpu()
    if dtype == "bf16":
        import ml_dtypes
        return t.view(torch.int16).numpy().view(ml_dtypes.bfloat16)
    return t.numpy()


def parse_launch(ptx: str):
    m = re.search(r"^// launch: (\{.*\})$", ptx, re.M)
    return json.loads(m.group(1)) if m else None


class CompiledKernel:
    """One kernel of a problem: PTX, cubin, ptxas resources, loaded function."""

    def __init__(self, ir_path: Path, meta: dict, mode: dict):
        self.meta, self.ir_path = meta, ir_path
        self.ptx = compile_file(str(ir_path), **mode)
        self.launch_info = parse_launch(self.ptx) or dict(
            grid=meta["grid"], block=meta["block"], cluster=1, smem_bytes=meta.get("smem_bytes", 0),
            params=[dict(kind="buffer", name=n) for n in meta["arg_order"]], family="foreign")
        cubin, info = toolchain.assemble(self.ptx)
        self.resources = info.get(meta["entry"], {})
        self.module = driver.Module(cubin)
        self.function = self.module.function(meta["entry"])

    def bind(self, tensors: dict) -> list:
        """The launches of this kernel on ``tensors`` (name -> torch tensor), in order: the auxiliary
        entries its launch header lists under ``pre``, then the kernel itself. Parameters that are not
        arguments of meta.json get their own tensors, kept in ``tensors`` under ``"<entry>.<name>"``: a
        zeroed ``status`` word (what the kernel's bounded waits report into, read by ``check_status``)
        and ``scratch`` buffers (device memory between the kernels of one module)."""
        import torch
        entry = self.meta["entry"]
        anchor = next(iter(tensors.values()))

        def own(name, make):
            key = f"{entry}.{name}"
            if key not in tensors:
                tensors[key] = make()
            return tensors[key]

        def resolve(name):
            return tensors[name] if name in tensors else tensors[f"{entry}.{name}"]

        def one(fn, li):
            params = []
            for p in li["params"]:
                if p["kind"] == "buffer":
                    params.append(resolve(p["name"]).data_ptr())
                elif p["kind"] == "status":
                    params.append(own("status", lambda: torch.zeros(8, dtype=torch.int32, device=anchor.device)).data_ptr())
                elif p["kind"] == "scratch":
                    params.append(own(p["name"], lambda: torch.empty(p["bytes"], dtype=torch.uint8, device=anchor.device)).data_ptr())
                elif p["kind"] == "tmap":
                    t = resolve(p["buffer"])
                    params.append(driver.TensorMap(t.data_ptr() + p.get("offset_bytes", 0), p["dtype"], p["dims"],
                                                   p["strides_bytes"], p["box"], p.get("swizzle", "128B")))
                elif p["kind"] == "exchange":  # the device record of multi.PeerExchange, or null: no exchange
                    params.append(tensors[EXCHANGE].data_ptr() if EXCHANGE in tensors else 0)
                else:
                    raise ValueError(f"unknown parameter kind {p['kind']!r}")
            flags = driver.LAUNCH_PDL if li.get("pdl") else 0
            launch = driver.Launch(fn, li["grid"], li["block"], li.get("cluster", 1), li.get("smem_bytes", 0), params, flags)
            # what the launch touches, by name: lets a host tell parameter preparation (reads only the job's resident
            # operands, writes scratch) from the launches that depend on a step's inputs
            launch.buffers = [p["name"] for p in li["params"] if p["kind"] == "buffer"] + [p["buffer"] for p in li["params"] if p["kind"] == "tmap"]
            launch.scratch = [f"{entry}.{p['name']}" for p in li["params"] if p["kind"] == "scratch"]
            return launch

        li = self.launch_info
        # scratch must exist before a tensor map over it is built: make them in the order the header lists them
        out = [one(self.module.function(pre["entry"]), pre) for pre in li.get("pre", ())]
        out.append(one(self.function, li))
        return out


WAIT_CODES = {1: "shared-memory stage never filled", 2: "shared-memory stage never released",
              3: "accumulator never completed", 4: "accumulator never drained"}  # emb::tc::WAIT_* of csrc/templates/emb_tc.cuh


def raise_on_status(entry: str, word: list) -> None:
    """The status word a tensor-core template's bounded waits report into: [0] the first failure's code (0: none),
    [1] the CTA, [2] the step it was waiting at. A non-zero code becomes ``EmbError(-3)``."""
    if word and word[0]:
        where = WAIT_CODES.get(word[0], "wait")
        raise driver.EmbError(-3, f"{entry}: a bounded wait ran out ({where}; code {word[0]}, CTA {word[1]}, step {word[2]})")


EXCHANGE = "__exchange__"  # key of the exchange record among a problem's tensors (shared by all buffer sets)


class Problem:
    """A problem folder compiled in one mode and bound to tensors on one device. ``exchange`` (a multi.PeerExchange)
    makes the last kernel of a sharded sum combine its scalar with the other ranks' inside the kernel. ``canary``
    puts every output and intermediate buffer between two guard zones and fills all of it with a poison pattern (NaN
    for floats): ``check_canaries`` then shows a kernel that wrote outside its buffer, a NaN left in an output one that
    did not write all of it (the stand-in for a memory checker on small shapes)."""

    GUARD_BYTES = 4096

    def __init__(self, folder, mode: str = "optimized", device: int = 0, inputs: dict | None = None, share: dict | None = None,
                 exchange=None, canary: bool = False):
        """``inputs``: name -> numpy array instead of the seeded draws of meta.json. ``share``: name -> device tensor to bind
        instead of making one (an operand or a scratch buffer, ``"<entry>.<name>"``, that several problems use)."""
        import torch
        self.folder = Path(folder)
        self.meta = json.loads((self.folder / "meta.json").read_text())
        self.mode = mode
        flags = {"optimized": {}, "strict": {"strict": True}, "plain": {"plain": True}}[mode]
        if not torch.cuda.is_available():
            raise driver.EmbError(-101, "no CUDA device: the kernels run on the GPU only")
        self.device = torch.device("cuda", device)
        torch.cuda.set_device(self.device)
        driver.init(device)
        self.kernels = [CompiledKernel(self.folder / f"{k['entry']}.ir.json", k, flags) for k in self.meta["kernels"]]
        self.tensors: dict = {}
        self.dtypes: dict = {}
        self.host: dict = {}
        for k in self.meta["kernels"]:
            given = inputs if inputs is not None else host_inputs(k["args"])
            for a in k["args"]:
                name = a["name"]
                self.dtypes.setdefault(name, a["dtype"])
                if name in self.tensors:
                    continue
                if share and name in share:
                    self.tensors[name] = share[name]
                    if not (a.get("output") or a.get("intermediate")):
                        self.host[name] = given[name]
                    continue
                if a.get("output") or a.get("intermediate"):
                    shape = a["shape"] or [1]
                    dtype = getattr(torch, TORCH_DTYPE[a["dtype"]])
                    if canary:
                        self.tensors[name] = self._guarded(name, shape, dtype)
                    else:
                        self.tensors[name] = torch.zeros(shape, dtype=dtype, device=self.device)
                else:
                    self.host[name] = given[name]
                    self.tensors[name] = to_torch(given[name], a["dtype"], self.device)
        for name, t in (share or {}).items():  # shared scratch: found by bind() under its "<entry>.<name>" key
            self.tensors.setdefault(name, t)
        self.exchange = exchange
        if exchange is not None:
            self.tensors[EXCHANGE] = exchange.record
        self.launches = [l for k in self.kernels for l in k.bind(self.tensors)]
        self.sets = [self.launches]  # further copies of every buffer, for cold-cache timing (rotate())
        self.zero = [n for k in self.meta["kernels"] for n in k.get("zero_outputs", ())]

    @property
    def stream(self) -> int:
        import torch
        return torch.cuda.current_stream(self.device).cuda_stream

    def _guarded(self, name: str, shape, dtype):
        import math

        import torch
        numel = math.prod(shape)
        size = torch.empty(0, dtype=dtype).element_size()
        pad = self.GUARD_BYTES // size
        whole = torch.empty(numel + 2 * pad, dtype=dtype, device=self.device)
        whole.view(torch.uint8).fill_(0xFF)  # NaN in every float format, -1 in the integer ones
        self.guards = getattr(self, "guards", {})
        self.guards[name] = (whole, pad, numel)
        return whole[pad:pad + numel].view(shape)

    def check_canaries(self) -> None:
        """Raise if a guard zone around an output or intermediate buffer no longer holds the poison pattern."""
        import torch
        for name, (whole, pad, numel) in getattr(self, "guards", {}).items():
            raw = whole.view(torch.uint8)
            size = whole.element_size()
            for zone, part in (("before", raw[:pad * size]), ("after", raw[(pad + numel) * size:])):
                bad = (part != 0xFF).nonzero()
                if bad.numel():
                    raise driver.EmbError(-4, f"{name}: {bad.numel()} byte(s) written {zone} the buffer (first at byte {int(bad[0])} of the zone)")

    def run(self) -> dict:
        """Launch the chain once and return the final kernels' outputs as numpy arrays."""
        import torch
        for n in self.zero:
            self.tensors[n].zero_()
        driver.launch(self.launches, self.stream)
        torch.cuda.synchronize(self.device)
        self.check_status()
        return self.outputs()

    def check_status(self) -> None:
        """Raise if a kernel's bounded wait gave up (its status word is non-zero)."""
        import torch
        if self.exchange is not None:
            self.exchange.check()
        for tensors in [self.tensors] + list(getattr(self, "copies", [])):
            for name, t in tensors.items():
                if name.endswith(".status") and t.dtype == torch.int32:
                    raise_on_status(name[:-7], t.cpu().tolist())

    def outputs(self) -> dict:
        names = [a["name"] for k in self.meta["kernels"] for a in k["args"] if a.get("output")]
        return {n: to_numpy(self.tensors[n], self.dtypes[n]) for n in names}

    def time_us(self, warmup: int = 3, iters: int = 20, flush=None) -> list:
        out = driver.time_chain(self.launches, self.stream, warmup, iters, flush)
        self.check_status()
        return out

    def rotate(self, min_bytes: int = 512 << 20, max_sets: int = 16) -> int:
        """Bind further copies of every tensor until the sets together hold ``min_bytes``:
        timing then walks the sets, so a run never finds its data in the 126 MB L2."""
        if getattr(self, "guards", None):
            raise driver.EmbError(-2, "rotate() on a canary problem: the copies would have no guard zones (check one set, time another problem)")
        per_set = sum(t.numel() * t.element_size() for n, t in self.tensors.items() if n != EXCHANGE)
        want = max(2, min(max_sets, -(-min_bytes // max(per_set, 1))))
        self.copies = getattr(self, "copies", [])
        while len(self.sets) < want:
            clone = {n: (t if n == EXCHANGE else t.clone()) for n, t in self.tensors.items()}
            self.copies.append(clone)
            self.sets.append([l for k in self.kernels for l in k.bind(clone)])
        return len(self.sets)

    def time_rotating_us(self, warmup: int = 3, iters: int = 20, only=None, batch: int = 1) -> list:
        sets = self.sets if only is None else [[s[only]] for s in self.sets]
        out = driver.time_rotating(sets, self.stream, warmup, iters, batch)
        self.check_status()
        return out

    def rows_pipeline(self, chunks: int = 4, streams: int = 3):
        """For a one-kernel problem whose launch header declares its rows independent (a fixed number of CTAs per row of
        the listed buffers, one unless the header says otherwise): a callable ``run(host_in, host_out)`` that processes
        the rows in ``chunks`` slices, each slice's host-to-device copy, launch and device-to-host copy on one of ``streams`` CUDA streams, so that the copies of
        one slice overlap the compute and the opposite-direction copies of its neighbours. ``host_in`` / ``host_out``
        map buffer names to pinned host tensors of the full shapes. Returns None when the kernel declares no such rows."""
        import torch
        if len(self.kernels) != 1 or len(self.launches) != 1:
            return None
        k = self.kernels[0]
        info = k.launch_info.get("rows")
        if not info or any(p["kind"] != "buffer" for p in k.launch_info["params"]):
            return None
        total, per_row = info["count"], info.get("ctas_per_row", 1)
        bounds = [total * c // chunks for c in range(chunks + 1)]
        pool = [torch.cuda.Stream(self.device) for _ in range(streams)]
        li = k.launch_info
        pieces = []
        for c in range(chunks):
            lo, hi = bounds[c], bounds[c + 1]
            if hi == lo:
                continue
            params = [self.tensors[p["name"]].data_ptr() + lo * info["buffers"].get(p["name"], 0) for p in li["params"]]
            pieces.append((lo, hi, driver.Launch(k.function, [(hi - lo) * per_row, 1, 1], li["block"], li.get("cluster", 1),
                                                 li.get("smem_bytes", 0), params)))
        # buffers every row shares (0 bytes per row: a bias row, a scalar) stay where they are
        ins = [n for n, row_bytes in info["buffers"].items() if n in self.host and row_bytes]
        outs = [n for n, row_bytes in info["buffers"].items() if n not in self.host and row_bytes]

        def run(host_in: dict, host_out: dict) -> None:
            main = torch.cuda.current_stream(self.device)
            start = torch.cuda.Event()
            start.record(main)
            for idx, (lo, hi, launch) in enumerate(pieces):
                s = pool[idx % len(pool)]
                s.wait_event(start)
                with torch.cuda.stream(s):
                    for n in ins:
                        if n in host_in:
                            self.tensors[n][lo:hi].copy_(host_in[n][lo:hi], non_blocking=True)
                    driver.launch([launch], s.cuda_stream)
                    for n in outs:
                        host_out[n][lo:hi].copy_(self.tensors[n][lo:hi], non_blocking=True)
            for s in pool:
                main.wait_stream(s)
        return run

    def launch_count(self) -> int:
        return len(self.launches)


def run_source(src, arrays: dict, mode: str = "optimized", device: int = 0) -> dict:
    """Lower a ``KernelSource`` built in memory (as the reference's tests do,
    tests/test_gpu_lowering.py:63-80), run it once on ``arrays`` (name -> numpy array, outputs
    included) and return every buffer the kernel writes."""
    import torch

    from . import PTX_VERSION, TARGET
    from .lower import Lowerer
    flags = {"optimized": {}, "strict": {"strict": True}, "plain": {"plain": True}}[mode]
    kernel = Lowerer(src, **flags).run()
    ptx = kernel.render(PTX_VERSION, TARGET)
    cubin, _ = toolchain.assemble(ptx)
    if not torch.cuda.is_available():
        raise driver.EmbError(-101, "no CUDA device: the kernels run on the GPU only")
    dev = torch.device("cuda", device)
    torch.cuda.set_device(dev)
    driver.init(device)
    fn = driver.Module(cubin).function(src.name)
    tensors = {n: to_torch(a, src.buffers[n].dtype, dev) for n, a in arrays.items()}
    li = kernel.launch
    params, status = [], None
    for p in li["params"]:
        if p["kind"] == "buffer":
            params.append(tensors[p["name"]].data_ptr())
        elif p["kind"] == "status":
            status = torch.zeros(8, dtype=torch.int32, device=dev)
            params.append(status.data_ptr())
        else:
            t = tensors[p["buffer"]]
            params.append(driver.TensorMap(t.data_ptr() + p.get("offset_bytes", 0), p["dtype"], p["dims"], p["strides_bytes"],
                                           p["box"], p.get("swizzle", "128B")))
    launch = driver.Launch(fn, li["grid"], li["block"], li["cluster"], li["smem_bytes"], params)
    driver.launch([launch], torch.cuda.current_stream(dev).cuda_stream)
    torch.cuda.synchronize(dev)
    if status is not None and int(status[0]):
        raise driver.EmbError(-3, f"{src.name}: a bounded wait ran out (status {status.cpu().tolist()})")
    return {n: to_numpy(tensors[n], src.buffers[n].dtype) for n in src.written}
