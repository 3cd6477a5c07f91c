"""Front end: one ``<kernel>.ir.json`` file plus the ``meta.json`` beside it -> ``KernelSource``.

Same contract as the reference's front end (emmy_ptx/frontend.py:52-92): the
IR file holds exactly one ``KernelOp`` node whose ``op_fields.body`` is the list
of serialized statements; every node output is a buffer (name, shape, dtype);
a scalar ``ConstantOp`` whose output has one element is a compile-time constant
(:70-75); ``meta.json`` gives the parameter order and the launch geometry and
wins over the IR (:80-86, looked up by ``entry``, then ``node``, else the only
kernel, :115-124); without it both are derived from the IR with a warning
(:87-91, :127-148). The reference deserializes with the emmy package; here the
statements are read by ``ir.parse``.
"""

from __future__ import annotations

import json
import math
import sys
from dataclasses import dataclass, field
from pathlib import Path

from . import ir

DEFAULT_BLOCK = 256  # threads of a Tile that names no cooperative block (emmy_ptx/frontend.py:20)


@dataclass(frozen=True)
class Buffer:
    name: str
    shape: tuple
    dtype: str  # emmy dtype name: f32, f16, bf16, f64, i32, u8, f8e4m3, ...


@dataclass(frozen=True)
class Launch:
    grid: int
    block: int
    smem_bytes: int


@dataclass(frozen=True)
class KernelSource:
    name: str
    body: tuple
    params: tuple  # buffer names in launch-argument order
    buffers: dict
    launch: Launch
    written: frozenset
    constants: dict = field(default_factory=dict)
    meta: dict | None = None  # this kernel's meta.json entry, if there was one
    path: str | None = None


def load(ir_path) -> KernelSource:
    ir_path = Path(ir_path)
    graph = json.loads(ir_path.read_text())
    kernels = [(nid, n) for nid, n in graph["nodes"].items() if n.get("op") == "KernelOp"]
    if len(kernels) != 1:
        raise ValueError(f"{ir_path.name}: expected exactly one KernelOp, found {len(kernels)}")
    node_id, node = kernels[0]
    fields = node["op_fields"]
    body = tuple(ir.parse(text) for text in fields["body"])
    name = fields.get("name") or node_id

    buffers, constants = {}, {}
    for n in graph["nodes"].values():
        for t in n.get("outputs", ()):
            buffers[t["name"]] = Buffer(t["name"], tuple(int(d) for d in t["shape"]), t["dtype"])
        if n.get("op") == "ConstantOp":
            value = n.get("op_fields", {}).get("value")
            outs = n.get("outputs", ())
            if (isinstance(value, (int, float)) and not isinstance(value, bool)
                    and n["op_fields"].get("source_path") is None and len(outs) == 1
                    and math.prod(int(d) for d in outs[0]["shape"]) == 1):
                constants[outs[0]["name"]] = value

    shared = {s.name for s in ir.walk(body) if ir.kind(s) == "Smem"}
    written = frozenset(_written(body) - shared)

    meta = find_meta(ir_path, name, node_id)
    if meta is not None:
        params = tuple(meta["arg_order"])
        launch = Launch(int(meta["grid"][0]), int(meta["block"][0]), int(meta.get("smem_bytes", 0)))
        for arg in meta.get("args", ()):
            if arg["name"] not in buffers:
                buffers[arg["name"]] = Buffer(arg["name"], tuple(arg["shape"]), arg["dtype"])
    else:
        print(f"warning: no meta.json entry for {name}; deriving parameters and launch from the IR", file=sys.stderr)
        params = _signature_order(body, shared)
        launch = _derived_launch(body)
    return KernelSource(name, body, params, buffers, launch, written, constants, meta, str(ir_path))


def _written(body) -> set:
    out = set()
    for s in ir.walk(body):
        k = ir.kind(s)
        if k == "Write":
            out.add(s.output)
        elif k == "RegStore":
            out.add(s.dst_buffer)
        elif k == "ZeroPrologue":
            out.add(s.dst)
    return out


def find_meta(ir_path: Path, entry: str, node_id: str):
    meta_path = Path(ir_path).with_name("meta.json")
    if not meta_path.exists():
        return None
    kernels = json.loads(meta_path.read_text()).get("kernels", [])
    for key, want in (("entry", entry), ("node", node_id)):
        for k in kernels:
            if k.get(key) == want:
                return k
    return kernels[0] if len(kernels) == 1 else None


def _signature_order(body, shared) -> tuple:
    """Inputs by first read, then outputs by first write (emmy_ptx/frontend.py:127-139)."""
    reads, writes = {}, {}
    for s in ir.walk(body):
        k = ir.kind(s)
        if k == "Load" and s.input not in shared:
            reads.setdefault(s.input)
        elif k == "CpAsyncCopy":
            reads.setdefault(s.src)
        elif k == "Write" and s.output not in shared:
            writes.setdefault(s.output)
    return tuple(reads) + tuple(w for w in writes if w not in reads)


def _derived_launch(body) -> Launch:
    tiles = [s for s in ir.walk(body) if ir.kind(s) == "Tile"]
    if not tiles:
        return Launch(1, DEFAULT_BLOCK, 0)
    tile = tiles[0]
    cells = tile.block_threads or DEFAULT_BLOCK
    n = math.prod(a.extent.as_static() for a in tile.axes)
    return Launch(max(1, -(-n // cells)), cells + (tile.aux_threads or 0), 0)
