"""Front end: a ``<kernel>.ir.json`` file and the ``meta.json`` beside it become a ``KernelSource``.

The contract is the reference front end's (its emmy_ptx/frontend.py:52-92):

  * the graph holds exactly one ``KernelOp`` node; its ``op_fields.body`` lists the serialized statements and
    ``op_fields.name`` is the entry point;
  * every output of every node is a buffer (name, shape, dtype);
  * a ``ConstantOp`` with a plain number as value, no ``source_path`` and a one-element output is a compile-time
    constant as well as a buffer (:70-75);
  * ``meta.json`` decides the parameter order and the launch (``arg_order``, ``grid[0]``, ``block[0]``,
    ``smem_bytes``) and may add buffers the graph does not mention (:80-86); its entry for the kernel is found by
    ``entry``, else by ``node``, else it is the only one (:115-124);
  * without ``meta.json`` a warning goes to stderr and both are derived from the IR: inputs in order of first
    read, then outputs in order of first write; one thread per Tile cell in blocks of the Tile's ``block_threads``
    (256 if it names none) plus its auxiliary threads (:87-91, :127-148).

The reference hands the statements to the emmy package; here ``ir.parse`` reads them.
"""

from __future__ import annotations

import json
import math
import sys
from dataclasses import dataclass, field
from pathlib import Path

from . import ir

DEFAULT_BLOCK = 256


@dataclass(frozen=True)
class Buffer:
    name: str
    shape: tuple
    dtype: str  # f32, f16, bf16, f64, i32, u8, f8e4m3, ...


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
    meta: dict | None = None  # the kernel's entry of meta.json, when there is one
    path: str | None = None


def load(ir_path) -> KernelSource:
    ir_path = Path(ir_path)
    nodes = json.loads(ir_path.read_text())["nodes"]
    node_id, fields = _the_kernel(nodes, ir_path.name)
    name = fields.get("name") or node_id
    body = tuple(ir.parse(text) for text in fields["body"])
    buffers = {b.name: b for b in _outputs(nodes)}
    scratch = {s.name for s in ir.walk(body) if ir.kind(s) == "Smem"}

    meta = find_meta(ir_path, name, node_id)
    if meta is None:
        print(f"warning: no meta.json entry for {name}; deriving parameters and launch from the IR", file=sys.stderr)
        params, launch = _order_from_ir(body, scratch), _launch_from_ir(body)
    else:
        params = tuple(meta["arg_order"])
        launch = Launch(int(meta["grid"][0]), int(meta["block"][0]), int(meta.get("smem_bytes", 0)))
        for arg in meta.get("args", ()):
            buffers.setdefault(arg["name"], Buffer(arg["name"], tuple(arg["shape"]), arg["dtype"]))
    return KernelSource(name=name, body=body, params=params, buffers=buffers, launch=launch,
                        written=frozenset(_stored(body) - scratch), constants=_constants(nodes), meta=meta, path=str(ir_path))


def _the_kernel(nodes: dict, file_name: str) -> tuple:
    found = [(key, node["op_fields"]) for key, node in nodes.items() if node.get("op") == "KernelOp"]
    if len(found) != 1:
        raise ValueError(f"{file_name}: expected exactly one KernelOp, found {len(found)}")
    return found[0]


def _outputs(nodes: dict):
    for node in nodes.values():
        for out in node.get("outputs", ()):
            yield Buffer(out["name"], tuple(int(d) for d in out["shape"]), out["dtype"])


def _constants(nodes: dict) -> dict:
    values = {}
    for node in nodes.values():
        if node.get("op") != "ConstantOp":
            continue
        fields, outs = node.get("op_fields", {}), node.get("outputs", ())
        value = fields.get("value")
        is_number = isinstance(value, (int, float)) and not isinstance(value, bool)
        if is_number and fields.get("source_path") is None and len(outs) == 1 and math.prod(outs[0]["shape"]) == 1:
            values[outs[0]["name"]] = value
    return values


def _stored(body) -> set:
    """Names of everything the kernel stores to (shared arrays included)."""
    target = {"Write": "output", "RegStore": "dst_buffer", "ZeroPrologue": "dst"}
    return {getattr(s, target[ir.kind(s)]) for s in ir.walk(body) if ir.kind(s) in target}


def find_meta(ir_path, entry: str, node_id: str):
    meta_file = Path(ir_path).with_name("meta.json")
    if not meta_file.exists():
        return None
    kernels = json.loads(meta_file.read_text()).get("kernels", [])
    by_entry = [k for k in kernels if k.get("entry") == entry]
    by_node = [k for k in kernels if k.get("node") == node_id]
    if by_entry or by_node:
        return (by_entry or by_node)[0]
    return kernels[0] if len(kernels) == 1 else None


def _order_from_ir(body, scratch: set) -> tuple:
    read, stored = [], []
    for s in ir.walk(body):
        k = ir.kind(s)
        name = s.input if k == "Load" else s.src if k == "CpAsyncCopy" else None
        if name is not None and name not in scratch and name not in read:
            read.append(name)
        if k == "Write" and s.output not in scratch and s.output not in stored:
            stored.append(s.output)
    return tuple(read) + tuple(n for n in stored if n not in read)


def _launch_from_ir(body) -> Launch:
    tile = next((s for s in ir.walk(body) if ir.kind(s) == "Tile"), None)
    if tile is None:
        return Launch(1, DEFAULT_BLOCK, 0)
    per_block = tile.block_threads or DEFAULT_BLOCK
    cells = math.prod(a.extent.as_static() for a in tile.axes)
    return Launch(max(1, math.ceil(cells / per_block)), per_block + (tile.aux_threads or 0), 0)
