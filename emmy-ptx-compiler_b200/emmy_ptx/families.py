"""Pattern matching of the bandwidth-bound kernel families and instantiation of their templates.

Each ``match_*`` function takes a ``KernelSource`` and either returns a
``Plan`` (the CUDA source that instantiates a template of ``csrc/templates``,
the launch it needs and the remarks for ``--report``) or raises ``Refusal``
with the reason; the caller then falls back to the statement-by-statement
lowering (codegen.py). A template is instantiated only when the IR has exactly
the shape matched here AND the legality conditions hold; they are the
reference's, restated for these templates:

  * block reduction (emmy_ptx/regroup.py:75-147 ``combine_refusal``,
    emmy_ptx/lower.py:250-272 ``_ownership_refusal``, :1385-1402
    ``_tree_refusal``): the per-thread partial flows only into the combines of
    its own state, every warp's partial reaches the tree exactly once, a barrier
    separates the slab's writes from the tree, ``lane`` and ``warp`` are not
    redefined, the loads are from a buffer the kernel does not write, nothing
    reads the slab after the tree, and the tree is not inside a loop;
  * the 16-byte accesses need the run's first element index, the step and the
    row length to be multiples of the run (emmy_ptx/regroup.py:192-233 asks
    ``extent % (4*B) == 0`` for its regrouping; here the IR already spells the
    run as a multi-name Load, so only alignment is left to prove).
"""

from __future__ import annotations

import math
from dataclasses import dataclass, field

from . import codegen, ir
from .codegen import CANON, CTYPE, Emitter, divisible
from .ir import dtype_name, kind

# Tunables of the reduction template (None: chosen from the kernel's shape).
REDUCE_UNROLL = None      # trips of the strided fold in flight per round
REDUCE_MIN_BLOCKS = None  # second argument of __launch_bounds__: caps registers so that many CTAs fit an SM
MAX_FULL_UNROLL = 16      # a fold of at most this many trips is one fully unrolled, predicated round

OP_TYPE = {"add": "emb::OpAdd", "multiply": "emb::OpMul", "maximum": "emb::OpMax", "minimum": "emb::OpMin"}


class Refusal(Exception):
    """The kernel is not of this family, or a legality condition fails (the text says which)."""


@dataclass
class Plan:
    family: str
    source: str  # CUDA C++ translation unit
    remarks: list = field(default_factory=list)
    grid: int | None = None  # None: the launch of meta.json stands
    block: int | None = None
    cluster: int = 1
    smem_bytes: int | None = None
    extra_params: list = field(default_factory=list)  # tensor maps and scratch the launch header lists
    nvcc_flags: tuple = ()
    pre: list = field(default_factory=list)  # launches of auxiliary entries of the same module, run before the main one
    rows: dict | None = None  # row independence: {"count": R, "buffers": {name: bytes per row}}, one CTA per row


def need(cond, why: str) -> None:
    if not cond:
        raise Refusal(why)


def is_var(e, name=None) -> bool:
    return kind(e) == "Var" and (name is None or e.name == name)


def is_int(e, value=None) -> bool:
    return kind(e) == "Literal" and isinstance(e.value, int) and (value is None or e.value == value)


def eq_zero(cond, name: str) -> bool:
    return (kind(cond) == "BinaryExpr" and cond.op == "==" and
            ((is_var(cond.left, name) and is_int(cond.right, 0)) or (is_var(cond.right, name) and is_int(cond.left, 0))))


def same_expr(a, b, rename: dict) -> bool:
    """Structural equality of two expressions, names of ``a`` mapped through ``rename``."""
    if kind(a) != kind(b):
        return False
    k = kind(a)
    if k == "Var":
        return rename.get(a.name, a.name) == b.name
    if k == "Literal":
        return a.value == b.value and type(a.value) is type(b.value)
    if k == "BinaryExpr":
        return a.op == b.op and same_expr(a.left, b.left, rename) and same_expr(a.right, b.right, rename)
    return repr(a) == repr(b)


def single_tile(src):
    need(len(src.body) == 1 and kind(src.body[0]) == "Tile", "the body is not a single Tile")
    tile = src.body[0]
    need(not (tile.raster_axes and tile.raster_group is not None) and not tile.aux_threads, "rasterized or banded Tile")
    need(tile.block_threads in (None, src.launch.block), "the Tile's block is not the launch's")
    cells = math.prod(a.extent.as_static() for a in tile.axes)
    need(cells == src.launch.grid * src.launch.block, "the launch has threads outside the Tile")
    for s in ir.walk(tile.body):
        if kind(s) == "Let":
            need(s.name not in ("lane", "warp"), "lane or warp is redefined")
    need(all(a.name not in ("lane", "warp") for a in tile.axes), "lane or warp is redefined")
    return tile


def thread_axis(tile, block: int):
    """The innermost axis must be exactly the block's threads (so it equals threadIdx.x)."""
    t = tile.axes[-1]
    need(t.extent.as_static() == block, "the innermost Tile axis is not the block's threads")
    return t.name


@dataclass
class Combine:
    """A matched butterfly (+ slab + barrier + tree) over one state."""
    state: str
    shuffle_op: str
    shuffle_len: int
    tree_op: str | None
    tree_len: int
    consumed: int  # statements taken


def match_combine(stmts, pos: int, state: str, block: int) -> Combine:
    need(pos < len(stmts) and kind(stmts[pos]) == "WarpShuffle", f"no butterfly after the fold of {state}")
    ws = stmts[pos]
    need(tuple(ws.state) == (state,) and len(ws.state_b) == 1 and len(ws.combine_states) == 1,
         "the butterfly carries other states")
    c = ws.combine_states[0]
    need(c.name == state and tuple(c.args) == (state, ws.state_b[0]) and c.dtype is None
         and CANON.get(c.op.name) in OP_TYPE, "the butterfly's combine is not state = op(state, partner)")
    length = int(ws.length)
    need(length & (length - 1) == 0 and 1 <= length <= 32 and length == min(block, 32),
         "the butterfly does not span the warp")
    shuffle_op = CANON[c.op.name]
    rest = stmts[pos + 1:pos + 5]
    if block <= 32 or not rest or kind(rest[0]) != "Smem":
        need(block <= 32, "more than one warp but no tree over the warps")
        return Combine(state, shuffle_op, length, None, 0, 1)
    need(len(rest) == 4 and [kind(s) for s in rest] == ["Smem", "Cond", "Sync", "TreeHalve"],
         "the warps' partials are not combined by slab, barrier and tree")
    smem, cond, sync, tree = rest
    warps = block // 32
    need(tuple(int(e) for e in smem.extents) == (warps,) and (smem.dtype or "float") == "float",
         "the slab is not one float per warp")
    need(eq_zero(cond.cond, "lane") and not cond.else_body and len(cond.body) == 1 and kind(cond.body[0]) == "Write",
         "the slab is not written by lane 0 of each warp")
    w = cond.body[0]
    need(w.output == smem.name and len(w.index) == 1 and is_var(w.index[0], "warp") and tuple(w.values) == (state,)
         and not w.atomic, "each warp's partial does not reach its own slab entry exactly once")
    need(not sync.warp, "the barrier before the tree is only a warp's")
    need(tuple(tree.bufs) == (smem.name,) and tuple(tree.state) == (state,) and tree.inner is None
         and tree.tid_var == "warp" and int(tree.length) == warps and len(tree.combine_states) == 1,
         "the tree is not over the warps' slab")
    tc = tree.combine_states[0]
    need(tc.name == state and tuple(tc.args) == (state, tree.state_b[0]) and tc.dtype is None
         and CANON.get(tc.op.name) in OP_TYPE, "the tree's combine is not state = op(state, partner)")
    return Combine(state, shuffle_op, length, CANON[tc.op.name], warps, 5)


def slab_read_later(stmts, names: set) -> bool:
    return any(kind(s) == "Load" and s.input in names for s in ir.walk(stmts))


def row_pointer(em: Emitter, src, load, loop_var: str) -> tuple:
    """(pointer expression of the row the loop walks, row length): every index but the last must
    not move with the loop, the last must be the loop variable itself."""
    buf = src.buffers.get(load.input)
    need(buf is not None and buf.dtype == "f32" and dtype_name(load.dtype) in (None, "f32"), "the fold does not load f32")
    need(load.input not in src.written, "the kernel writes the buffer it folds")
    need(len(load.index) == len(buf.shape) >= 1 and is_var(load.index[-1], loop_var),
         "the load is not indexed by the loop variable itself")
    for e in load.index[:-1]:
        need(loop_var not in ir.expr_vars(e), "an outer index moves with the loop")
    if len(buf.shape) == 1:
        return f"p_{load.input}", int(buf.shape[0])
    lead = em.flat(buf.shape[:-1], load.index[:-1])
    return f"(p_{load.input} + ({lead}) * {int(buf.shape[-1])}LL)", int(buf.shape[-1])


def tile_decode(em: Emitter, tile, block: int) -> None:
    em.emit(f"const long long gid = (long long)blockIdx.x * {block} + threadIdx.x;")
    stride = 1
    for axis in reversed(tile.axes):
        n = axis.extent.as_static()
        term = "gid" if stride == 1 else f"(gid / {stride}LL)"
        em.emit(f"{em.var(axis.name, 'i64')} = {term} % {n}LL;")
        em.facts[axis.name] = None
        stride *= n


def finish(em: Emitter, src, includes: str, strict: bool, shared: list, min_blocks=None, extra_sig=()) -> str:
    decls = [f"    {CTYPE[dt]} v_{n} = emb::zero<{CTYPE[dt]}>();" for n, dt in em.vars.items() if n not in ("lane", "warp")]
    head = [f"#define EMB_STRICT {int(strict)}", includes, codegen.PRELUDE.split("\n", 1)[1],
            f'extern "C" __global__ void __launch_bounds__({src.launch.block}{f", {min_blocks}" if min_blocks else ""}) '
            f'{src.name}({", ".join([codegen.signature(src), *extra_sig])}) {{',
            "    int v_lane = threadIdx.x & 31, v_warp = threadIdx.x >> 5;", "    (void)v_lane; (void)v_warp;",
            "    const unsigned emb_warp = 0xffffffffu; (void)emb_warp;"] + codegen.pdl_prologue(src, True)
    return "\n".join(head + shared + decls + em.lines + ["}"]) + "\n"


# ---------------------------------------------------------------- block reduction


def match_reduce(src, strict: bool) -> Plan:
    tile = single_tile(src)
    block = src.launch.block
    t_axis = thread_axis(tile, block)
    body = list(tile.body)
    need(body and kind(body[0]) == "StridedLoop", "the Tile does not start with a strided fold")
    loop = body[0]
    need(loop.seed and not has_cross(loop.body), "the fold is not seeded or holds cross-thread statements")
    need(loop.body and kind(loop.body[0]) == "Load", "the fold's first statement is not a Load")
    load = loop.body[0]
    vec = len(load.names)
    need(vec in (1, 2, 4), "a load of 3 or more than 4 names")
    accs = loop.body[1:]
    need(len(accs) == vec and all(kind(a) == "Accum" for a in accs), "the fold is not one Accum per loaded value")
    state = accs[0].name
    op = CANON.get(accs[0].op.name)
    need(op in OP_TYPE, f"no template for a fold with {accs[0].op.name}")
    for a, name in zip(accs, load.names):
        need(a.name == state and a.value == name and a.base is None and CANON.get(a.op.name) == op
             and dtype_name(a.dtype) in (None, "f32"), "the Accums do not fold the loaded values, in order, into one f32 state")
    need(state not in load.names, "the state is overwritten by the load")

    em = Emitter(src, plain=False, strict=strict)
    em.depth = 1
    tile_decode(em, tile, block)
    var = loop.axis.name
    pointer, row = row_pointer(em, src, load, var)
    extent = loop.axis.extent.as_static()
    need(extent <= row, "the loop runs past the buffer's row")
    em.facts[var] = (loop.start, loop.step)
    if vec > 1:
        need(divisible(loop.start, vec, em.facts) and divisible(loop.step, vec, em.facts) and extent % vec == 0
             and row % vec == 0 and (loop.end is None or divisible(loop.end, vec, em.facts)),
             f"the {vec * 4}-byte runs are not provably aligned")
    (start, ks), (step, kt) = em.expr(loop.start), em.expr(loop.step)
    need(ks == "int" and kt == "int", "a float loop bound")
    end = f"{extent}LL"
    if loop.end is not None:
        end_code, ke = em.expr(loop.end)
        need(ke == "int", "a float loop bound")
        end = end_code

    comb = match_combine(body, 1, state, block)
    tail = body[1 + comb.consumed:]
    need(not has_cross(tail), "cross-thread statements after the tree")
    slabs = {s.name for s in body if kind(s) == "Smem"}
    need(not slab_read_later(tail, slabs), "the slab is read after the tree")
    for s in ir.walk(tail):
        need(kind(s) in ("Cond", "Write", "Assign", "Let", "Load"), f"a {kind(s)} after the tree")

    trips = None
    if is_int(loop.step) and loop.end is None and loop.step.value > 0:
        trips = -(-extent // loop.step.value)  # the most trips any thread takes
    if REDUCE_UNROLL is not None:
        unroll = REDUCE_UNROLL
    elif trips is not None and trips <= MAX_FULL_UNROLL:
        unroll = trips
    else:
        unroll = 8
    min_blocks = REDUCE_MIN_BLOCKS
    if min_blocks is None and src.launch.grid > TARGET_SMS:
        # enough CTAs per SM for the whole grid to be resident at once, when the registers allow
        per_sm = -(-src.launch.grid // TARGET_SMS)
        if per_sm * block <= 2048 and 65536 // (per_sm * block) >= 24 + (1 if strict else unroll) * vec:
            min_blocks = per_sm
    tree_op = OP_TYPE[comb.tree_op] if comb.tree_op else OP_TYPE[op]
    em.emit(f"float acc_ = emb::strided_fold<{vec}, {OP_TYPE[op]}, {unroll}, {str(bool(strict)).lower()}>("
            f"{pointer}, {start}, {step}, {end});")
    em.emit(f"acc_ = emb::block_combine<{OP_TYPE[comb.shuffle_op]}, {comb.shuffle_len}, {tree_op}, {comb.tree_len}>"
            f"(acc_, emb_slab);")
    exchange = final_sum(src, op, comb, tail, state)
    if exchange:  # the last kernel of a sum: its scalar may be one GPU's share (emb_peer.cuh)
        em.emit("acc_ = emb::peer_all_sum(acc_, px, &emb_bcast);")
    em.emit(f"{em.var(state, 'f32')} = acc_;")
    em.block(tail, None)
    shared = [f"    __shared__ float emb_slab[{max(comb.tree_len, 1)}];"] + (["    __shared__ float emb_bcast;"] if exchange else [])
    source = finish(em, src, '#include "emb_reduce.cuh"' + ('\n#include "emb_peer.cuh"' if exchange else ""), strict, shared, min_blocks,
                    ["emb::PeerExchange* px"] if exchange else [])
    how = "in the IR's own order" if strict else f"on {unroll * vec} independent accumulators per thread"
    how += f", {unroll} trips in flight per round"
    remarks = [f"block reduction template: {op} fold of {load.input} in {vec * 4}-byte ld.global.nc runs, {how}",
               f"butterfly over {comb.shuffle_len} lanes" +
               (f", then the {comb.tree_len} warps' partials folded in the tree's order by every thread behind one barrier"
                if comb.tree_len else "")]
    remarks += em.remarks
    if exchange:
        remarks.append("the result is a sum that ends the problem: given an exchange (the element range sharded over GPUs), the "
                       "kernel itself stores its share into every peer's memory, waits (bounded) for theirs and adds them in rank order")
    return Plan("reduce", source, remarks, extra_params=[dict(kind="exchange", name="px")] if exchange else [])


def final_sum(src, op: str, comb, tail, state: str) -> bool:
    """Is this the one-block kernel that ends a sum (meta.json: ``final``), storing the combined f32 state as the
    problem's scalar result? Then its value may be one GPU's share of a sharded range, to be exchanged in place."""
    meta = getattr(src, "meta", None) or {}
    if not meta.get("final") or src.launch.grid != 1 or op != "add" or (comb.tree_op or "add") != "add" or comb.shuffle_op != "add":
        return False
    writes = [s for s in ir.walk(tail) if kind(s) == "Write"]
    if len(writes) != 1 or tuple(writes[0].values) != (state,) or writes[0].atomic:
        return False
    out = src.buffers.get(writes[0].output)
    return out is not None and out.dtype == "f32" and math.prod(out.shape or (1,)) == 1 and len(list(ir.walk(tail))) <= 2


def has_cross(stmts) -> bool:
    return codegen.has_cross_thread(stmts)


# ---------------------------------------------------------------- row softmax

TARGET_SMS = 148
MAX_ROW_VALUES = 64  # floats of the row one thread keeps in registers


def match_softmax(src, strict: bool) -> Plan:
    tile = single_tile(src)
    block = src.launch.block
    t_axis = thread_axis(tile, block)
    need(block >= 32, "a block smaller than a warp")
    body = list(tile.body)
    need(len(body) >= 3 and kind(body[0]) == "StridedLoop", "the Tile does not start with a strided fold")

    # phase 1: m = max over the row
    l1 = body[0]
    need(l1.seed and l1.end is None and l1.body and kind(l1.body[0]) == "Load", "phase 1 is not a seeded fold of a load")
    ld1 = l1.body[0]
    vec = len(ld1.names)
    need(vec in (1, 2, 4) and len(l1.body) == 1 + vec, "phase 1 is not one Accum per loaded value")
    m = l1.body[1].name
    for a, name in zip(l1.body[1:], ld1.names):
        need(kind(a) == "Accum" and a.name == m and a.value == name and a.base is None
             and CANON.get(a.op.name) == "maximum" and dtype_name(a.dtype) in (None, "f32"), "phase 1 does not fold a maximum")
    c1 = match_combine(body, 1, m, block)
    need(c1.shuffle_op == "maximum" and c1.tree_op in (None, "maximum"), "the row maximum is not combined with maximum")
    pos = 1 + c1.consumed

    # phase 2: l = sum of exp(x - m)
    need(pos < len(body) and kind(body[pos]) == "StridedLoop", "no second phase")
    l2 = body[pos]
    rename2 = {l1.axis.name: l2.axis.name}
    need(l2.seed and l2.end is None and same_expr(l1.start, l2.start, rename2) and same_expr(l1.step, l2.step, rename2)
         and l2.axis.extent.as_static() == l1.axis.extent.as_static(), "phase 2 walks the row differently")
    ld2 = l2.body[0] if l2.body else None
    need(ld2 is not None and kind(ld2) == "Load" and ld2.input == ld1.input and len(ld2.names) == vec
         and len(ld2.index) == len(ld1.index) and all(same_expr(a, b, rename2) for a, b in zip(ld1.index, ld2.index)),
         "phase 2 does not reload the row")
    need(len(l2.body) == 1 + 3 * vec, "phase 2 is not subtract, exp, Accum per value")
    lsum = l2.body[3].name if len(l2.body) > 3 else None
    for j, name in enumerate(ld2.names):
        d, e, a = l2.body[1 + 3 * j:4 + 3 * j]
        need(kind(d) == "Assign" and d.op.name == "subtract" and tuple(d.args) == (name, m), "phase 2: no x - m")
        need(kind(e) == "Assign" and e.op.name == "exp" and tuple(e.args) == (d.name,), "phase 2: no exp(x - m)")
        need(kind(a) == "Accum" and a.name == lsum and a.value == e.name and a.base is None and CANON.get(a.op.name) == "add",
             "phase 2: no sum of the exponentials")
        need(all(dtype_name(s.dtype) in (None, "f32") for s in (d, e, a)), "phase 2 is not f32")
    c2 = match_combine(body, pos + 1, lsum, block)
    need(c2.shuffle_op == "add" and c2.tree_op in (None, "add"), "the row sum is not combined with add")
    pos += 1 + c2.consumed

    # inv = 1 / l, then phase 3
    need(pos + 2 == len(body), "statements besides the three phases")
    inv, l3 = body[pos], body[pos + 1]
    need(kind(inv) == "Assign" and inv.op.name == "reciprocal" and tuple(inv.args) == (lsum,)
         and dtype_name(inv.dtype) in (None, "f32"), "no reciprocal of the row sum")
    need(kind(l3) == "StridedLoop" and l3.end is None, "no third phase")
    rename3 = {l1.axis.name: l3.axis.name}
    need(same_expr(l1.start, l3.start, rename3) and same_expr(l1.step, l3.step, rename3)
         and l3.axis.extent.as_static() == l1.axis.extent.as_static(), "phase 3 walks the row differently")
    ld3 = l3.body[0] if l3.body else None
    need(ld3 is not None and kind(ld3) == "Load" and ld3.input == ld1.input and len(ld3.names) == vec
         and all(same_expr(a, b, rename3) for a, b in zip(ld1.index, ld3.index)), "phase 3 does not reload the row")
    need(len(l3.body) == 2 + 3 * vec and kind(l3.body[-1]) == "Write", "phase 3 is not subtract, exp, multiply, Write")
    outs = []
    for j, name in enumerate(ld3.names):
        d, e, o = l3.body[1 + 3 * j:4 + 3 * j]
        need(kind(d) == "Assign" and d.op.name == "subtract" and tuple(d.args) == (name, m), "phase 3: no x - m")
        need(kind(e) == "Assign" and e.op.name == "exp" and tuple(e.args) == (d.name,), "phase 3: no exp(x - m)")
        need(kind(o) == "Assign" and o.op.name == "multiply" and set(o.args) == {e.name, inv.name}, "phase 3: no e * inv")
        need(all(dtype_name(s.dtype) in (None, "f32") for s in (d, e, o)), "phase 3 is not f32")
        outs.append(o.name)
    w = l3.body[-1]
    out_buf = src.buffers.get(w.output)
    need(tuple(w.values) == tuple(outs) and not w.atomic and out_buf is not None and out_buf.dtype == "f32"
         and w.output != ld1.input and len(w.index) == len(ld3.index)
         and all(same_expr(a, b, {}) for a, b in zip(ld3.index, w.index)), "phase 3 does not write the row's cells")
    need(out_buf.shape == src.buffers[ld1.input].shape, "input and output shapes differ")

    em = Emitter(src, plain=False, strict=strict)
    tile_decode(em, tile, block)
    var = l1.axis.name
    pointer, row = row_pointer(em, src, ld1, var)
    cols = l1.axis.extent.as_static()
    need(cols == row, "the loops do not cover the whole row")
    # thread t must own elements t*vec + k*block*vec + j: that is what the template keeps in registers
    want_start = ir.BinaryExpr(op="*", left=ir.Var(name=t_axis), right=ir.Literal(value=vec, dtype="int"))
    need(same_expr(l1.start, want_start, {}) or (vec == 1 and is_var(l1.start, t_axis)),
         "a thread's first element is not thread * run")
    need(is_int(l1.step, block * vec), "the step is not block * run")
    need(cols % vec == 0, "the row length is not a multiple of the run")
    trips = -(-cols // (block * vec))
    need(trips * vec <= MAX_ROW_VALUES, f"a thread would hold {trips * vec} values of the row (more than {MAX_ROW_VALUES})")
    out_pointer = pointer.replace(f"p_{ld1.input}", f"p_{w.output}")
    # softmax_row indexes the row itself: pass the buffers and the row number
    lead = "0LL" if len(ld1.index) == 1 else em.flat(src.buffers[ld1.input].shape[:-1], ld1.index[:-1])
    em.emit(f"emb::softmax_row<{block}, {vec}, {cols}, {str(bool(strict)).lower()}>(p_{ld1.input}, p_{w.output}, {lead});")
    source = finish(em, src, '#include "emb_softmax.cuh"', strict, [])
    remarks = [f"row softmax template: one CTA per row of {cols}, the row held in registers ({trips * vec} values per thread), "
               f"read once and written once in {vec * 4}-byte runs; the IR's three loads of the row become one",
               "exp(x - max) computed once for the sum and the quotient",
               "row maximum: " + ("butterfly and tree in the IR's order" if strict else "redux.sync.max per warp, then the tree"),
               "row sum: butterfly over 32 lanes, then the tree's order behind one barrier"]
    del out_pointer
    lead_rows = math.prod(src.buffers[ld1.input].shape[:-1])
    independent = dict(count=lead_rows, buffers={ld1.input: cols * 4, w.output: cols * 4}) if lead_rows == src.launch.grid else None
    return Plan("softmax", source, remarks, rows=independent)


MATCHERS = (("softmax", match_softmax), ("reduce", match_reduce))
