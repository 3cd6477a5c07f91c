"""Sharing a loop's column-free work across a thread-block cluster through distributed shared memory.

The rewrite of the reference's emmy_ptx/cluster.py (plan :88-117, _split :120-164) for the
statement-by-statement lowering: when consecutive blocks differ only in one Tile coordinate (the
"column") and a loop's body splits into a part that does not depend on that coordinate (the same in
all blocks of a cluster: emmy's column-recomputing MLP recomputes the hidden activations for every
output column, examples/k_gelu_mlp/k_matmul_reduce_6918c9.ir.txt) and a part that does, the blocks of a
cluster of 8 each compute one eighth of the loop's iterations of the shared part, stash the values it
hands over (at most four f32) in their own shared memory, meet at a cluster barrier, and then every block
runs all iterations of its own part reading the values from the owner's shared memory (DSMEM). The
additions of the own part happen in the original order, so results are bit for bit those of the plain
loop, and the rewrite is allowed under ``--strict`` (docs/DESIGN.md:483-485 of the reference).

Conditions, the reference's: no rasterisation or auxiliary threads, cells == grid * block,
grid % 8 == 0, every other coordinate either inside a block or across whole blocks, a pure loop whose
trip count is a multiple of 8 and the same for all threads (a Loop, or a StridedLoop that starts at a
thread coordinate equal to its step), no fold carried in the shared part, 1..4 f32 values handed over,
at least 2048 shared inner iterations.
"""

from __future__ import annotations

import math
from dataclasses import dataclass

from . import ir
from .ir import kind

CLUSTER = 8
MAX_VALUES = 4
MIN_SHARED_WORK = 2048
PURE = ("Load", "Assign", "Accum", "Let", "Loop", "StridedLoop", "Select", "Init")


@dataclass
class ClusterPlan:
    before: tuple
    loop: object
    shared: tuple
    own: tuple
    after: tuple
    values: tuple
    trips: int
    slots: int
    start: object  # expression of a thread's first iteration
    step: int


def reads(s) -> set:
    k = kind(s)
    out = set()
    if k == "Load":
        for e in s.index:
            out |= ir.expr_vars(e)
    elif k == "Write":
        out |= set(s.values)
        for e in s.index:
            out |= ir.expr_vars(e)
    elif k == "Assign":
        out |= set(s.args)
    elif k == "Accum":
        out |= {s.name, s.value} | ({s.base} if s.base else set())
    elif k == "Let":
        out |= ir.expr_vars(s.value)
    elif k == "Cond":
        out |= ir.expr_vars(s.cond)
    elif k == "StridedLoop":
        out |= ir.expr_vars(s.start) | ir.expr_vars(s.step) | (ir.expr_vars(s.end) if s.end is not None else set())
    elif k == "Select":
        for b in s.branches:
            out.add(b.value)
            if b.select is not None:
                out |= ir.expr_vars(b.select)
    return out


def writes(s) -> set:
    k = kind(s)
    if k == "Load":
        return set(s.names)
    if k in ("Assign", "Accum", "Let", "Init", "Select"):
        return {s.name}
    if k in ("Loop", "StridedLoop"):
        out = {s.axis.name}
        for t in ir.walk(s.body):
            out |= writes(t)
        return out
    if k == "Cond":
        out = set()
        for t in ir.walk(s.body + s.else_body):
            out |= writes(t)
        return out
    return set()


def all_reads(s) -> set:
    out = reads(s)
    for child in s.nested():
        for t in ir.walk(child):
            out |= reads(t)
    return out


def dependents(stmts, roots: set) -> set:
    """``roots`` and every name bound (transitively) from a value that may depend on one of them."""
    dep = set(roots)
    while True:
        size = len(dep)
        for s in ir.walk(stmts):
            if reads(s) & dep:
                dep |= writes(s)
        if len(dep) == size:
            return dep


def inner_trips(stmts) -> int:
    total = 0
    for s in stmts:
        if kind(s) == "Loop":
            total += s.axis.extent.as_static() * max(1, inner_trips(s.body))
        elif kind(s) == "StridedLoop" and kind(s.step) == "Literal" and s.end is None:
            total += -(-s.axis.extent.as_static() // max(1, int(s.step.value))) * max(1, inner_trips(s.body))
    return total


def plan(tile, grid: int, block: int):
    """A ClusterPlan, or the reason (a string) why the Tile's work is not shared across a cluster."""
    extents = [a.extent.as_static() for a in tile.axes]
    n = math.prod(extents)
    if tile.aux_threads or (tile.raster_axes and tile.raster_group is not None) or n != grid * block:
        return "rasterized, banded, or threads outside the Tile"
    if grid % CLUSTER:
        return f"the grid is not a multiple of {CLUSTER}"
    stride, column, threads = n, None, {}
    for axis, extent in zip(tile.axes, extents):
        stride //= extent
        if stride < block:
            if block % (stride * extent):
                return "a coordinate straddles block boundaries"
            threads[axis.name] = extent
        elif stride % block:
            return "a coordinate straddles block boundaries"
        elif stride == block and extent % CLUSTER == 0:
            column = axis.name
    if column is None:
        return "no coordinate steps from one block to the next with an extent that is a multiple of 8"
    body = list(tile.body)
    reason = "no loop with work to share"
    for i, s in enumerate(body):
        if kind(s) not in ("Loop", "StridedLoop"):
            continue
        found = split(s, column, threads)
        if isinstance(found, str):
            reason = found
            continue
        shared, own, values, trips, start, step = found
        return ClusterPlan(tuple(body[:i]), s, shared, own, tuple(body[i + 1:]), values, trips, trips // CLUSTER, start, step)
    return reason


def split(loop, column: str, threads: dict):
    if loop.unroll or any(kind(t) not in PURE for t in ir.walk(loop.body)):
        return "the loop is not pure"
    extent = loop.axis.extent.as_static()
    if kind(loop) == "Loop":
        start, step, trips = ir.Literal(value=0, dtype="int"), 1, extent
    else:
        if loop.end is not None or kind(loop.step) != "Literal":
            return "the loop's bounds differ between threads"
        step = int(loop.step.value)
        start = loop.start
        if kind(start) != "Var" or threads.get(start.name) != step or extent % step:
            return "the loop does not start at a thread coordinate equal to its step"
        trips = extent // step
    if trips % CLUSTER:
        return f"the trip count is not a multiple of {CLUSTER}"
    dep = dependents(loop.body, {column})
    own = tuple(s for s in loop.body if writes(s) & dep)
    shared = tuple(s for s in loop.body if s not in own)
    if not own or not shared:
        return "nothing to share, or nothing that depends on the column"
    if any(kind(s) == "Accum" for s in shared):
        return "the shared part carries a fold across iterations"
    made = set().union(*(writes(s) for s in shared))
    needed = set().union(*(all_reads(s) for s in own))
    values = tuple(sorted(made & needed))
    if not values or len(values) > MAX_VALUES:
        return f"{len(values)} values would pass from the shared part to the column's part (1..{MAX_VALUES} allowed)"
    for v in values:
        defs = [t for t in ir.walk(shared) if kind(t) in ("Assign", "Accum") and t.name == v]
        if not defs or any(ir.dtype_name(t.dtype) not in (None, "f32") for t in defs):
            return f"{v} is not an f32 value the shared part computes"
    work = trips * max(1, inner_trips(shared))
    if work < MIN_SHARED_WORK:
        return f"only {work} shared inner iterations (fewer than {MIN_SHARED_WORK})"
    return shared, own, values, trips, start, step
