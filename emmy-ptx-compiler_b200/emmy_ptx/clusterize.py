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


class Placement:
    """Where the Tile's coordinates fall on the launch. Cells are numbered row-major over the axes and dealt to
    threads in order, ``block`` per CTA, so an axis whose period (its stride times its extent) divides the block
    varies only with the thread inside a CTA, and an axis whose stride is a multiple of the block varies only with
    the CTA; anything else straddles CTA boundaries."""

    def __init__(self, tile, block: int):
        self.block = block
        self.extent = {a.name: a.extent.as_static() for a in tile.axes}
        names = [a.name for a in tile.axes]
        self.stride = {name: math.prod(self.extent[m] for m in names[i + 1:]) for i, name in enumerate(names)}
        self.cells = math.prod(self.extent.values())

    def within_cta(self, name: str) -> bool:
        period = self.stride[name] * self.extent[name]
        return self.stride[name] < self.block and self.block % period == 0

    def across_ctas(self, name: str) -> bool:
        return self.stride[name] >= self.block and self.stride[name] % self.block == 0

    def straddlers(self) -> list:
        return [n for n in self.extent if not (self.within_cta(n) or self.across_ctas(n))]

    def thread_extents(self) -> dict:
        """coordinate -> extent, for the coordinates that enumerate threads of one CTA"""
        return {n: self.extent[n] for n in self.extent if self.within_cta(n)}

    def neighbour_axis(self):
        """The coordinate that steps from one CTA to the next (stride exactly one block) if a cluster's worth of its
        values is a whole number of clusters, else None: the CTAs of a cluster then differ in it alone."""
        for n in self.extent:
            if self.stride[n] == self.block and self.extent[n] % CLUSTER == 0:
                return n
        return None


def plan(tile, grid: int, block: int):
    """A ClusterPlan, or the reason (a string) why the Tile's work is not shared across a cluster."""
    where = Placement(tile, block)
    rasterized = bool(tile.raster_axes) and tile.raster_group is not None
    if tile.aux_threads or rasterized or where.cells != grid * block:
        return "rasterized, banded, or threads outside the Tile"
    if grid % CLUSTER:
        return f"the grid is not a multiple of {CLUSTER}"
    if where.straddlers():
        return "a coordinate straddles block boundaries"
    column = where.neighbour_axis()
    if column is None:
        return "no coordinate steps from one block to the next with an extent that is a multiple of 8"
    body = tuple(tile.body)
    reason = "no loop with work to share"
    for at, stmt in enumerate(body):
        if kind(stmt) not in ("Loop", "StridedLoop"):
            continue
        cut = LoopCut(stmt, column, where.thread_extents())
        refusal = cut.refusal()
        if refusal is None:
            return ClusterPlan(body[:at], stmt, cut.shared, cut.own, body[at + 1:], cut.values, cut.trips, cut.trips // CLUSTER,
                               cut.start, cut.step)
        reason = refusal
    return reason


class LoopCut:
    """One loop of the Tile cut into the part every CTA of a cluster computes alike (it never reads the column) and the
    part that is the CTA's own; ``refusal()`` runs the legality checks in order and leaves the cut in the attributes."""

    def __init__(self, loop, column: str, thread_extents: dict):
        self.loop, self.column, self.thread_extents = loop, column, thread_extents
        self.start, self.step, self.trips = ir.Literal(value=0, dtype="int"), 1, 0
        self.shared = self.own = self.values = ()

    def refusal(self):
        for check in (self.purity, self.iteration_space, self.partition, self.handover, self.worth):
            why = check()
            if why is not None:
                return why
        return None

    def purity(self):
        impure = any(kind(t) not in PURE for t in ir.walk(self.loop.body))
        return "the loop is not pure" if impure or self.loop.unroll else None

    def iteration_space(self):
        """Every thread must make the same trips, numbered alike in all CTAs of the cluster: a counted Loop, or a
        StridedLoop whose start is a thread coordinate that runs over exactly one step."""
        loop, extent = self.loop, self.loop.axis.extent.as_static()
        if kind(loop) == "Loop":
            self.trips = extent
        else:
            if loop.end is not None or kind(loop.step) != "Literal":
                return "the loop's bounds differ between threads"
            self.step, self.start = int(loop.step.value), loop.start
            lanes = self.thread_extents.get(self.start.name) if kind(self.start) == "Var" else None
            if lanes != self.step or extent % self.step:
                return "the loop does not start at a thread coordinate equal to its step"
            self.trips = extent // self.step
        return None if self.trips % CLUSTER == 0 else f"the trip count is not a multiple of {CLUSTER}"

    def partition(self):
        tainted = dependents(self.loop.body, {self.column})
        self.own = tuple(s for s in self.loop.body if writes(s) & tainted)
        self.shared = tuple(s for s in self.loop.body if not (writes(s) & tainted))
        if not (self.own and self.shared):
            return "nothing to share, or nothing that depends on the column"
        if any(kind(s) == "Accum" for s in self.shared):
            return "the shared part carries a fold across iterations"
        return None

    def handover(self):
        produced = {name for s in self.shared for name in writes(s)}
        consumed = {name for s in self.own for name in all_reads(s)}
        self.values = tuple(sorted(produced & consumed))
        if not 1 <= len(self.values) <= MAX_VALUES:
            return f"{len(self.values)} values would pass from the shared part to the column's part (1..{MAX_VALUES} allowed)"
        for v in self.values:
            makers = [t for t in ir.walk(self.shared) if kind(t) in ("Assign", "Accum") and t.name == v]
            if not makers or any(ir.dtype_name(t.dtype) not in (None, "f32") for t in makers):
                return f"{v} is not an f32 value the shared part computes"
        return None

    def worth(self):
        work = self.trips * max(1, inner_trips(self.shared))
        return None if work >= MIN_SHARED_WORK else f"only {work} shared inner iterations (fewer than {MIN_SHARED_WORK})"
