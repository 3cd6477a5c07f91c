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


def finish(em: Emitter, src, includes: str, strict: bool, shared: list, min_blocks=None, extra_sig=(), block=None) -> str:
    decls = [f"    {CTYPE[dt]} v_{n} = emb::zero<{CTYPE[dt]}>();" for n, dt in em.vars.items() if n not in ("lane", "warp")]
    head = [f"#define EMB_STRICT {int(strict)}", includes, codegen.PRELUDE.split("\n", 1)[1],
            f'extern "C" __global__ void __launch_bounds__({block or src.launch.block}{f", {min_blocks}" if min_blocks else ""}) '
            f'{src.name}({", ".join([codegen.signature(src), *extra_sig])}) {{',
            "    int v_lane = threadIdx.x & 31, v_warp = threadIdx.x >> 5;", "    (void)v_lane; (void)v_warp;",
            "    const unsigned emb_warp = 0xffffffffu; (void)emb_warp;"] + codegen.pdl_prologue(src, True)
    return "\n".join(head + shared + decls + em.lines + ["}"]) + "\n"


# ---------------------------------------------------------------- block reduction


@dataclass
class FoldCopy:
    """One copy of a fold's body: Load x[.., loop variable + offset]; Assign*; Accum(state, value)."""
    load: object
    offset: int
    chain: list
    accum: object


def index_offset(e, var: str):
    """k when the expression is ``var`` or ``var + k`` / ``k + var`` for an integer literal k, else None."""
    if is_var(e, var):
        return 0
    if kind(e) == "BinaryExpr" and e.op == "+":
        if is_var(e.left, var) and is_int(e.right):
            return e.right.value
        if is_var(e.right, var) and is_int(e.left):
            return e.left.value
    return None


def fold_copies(loop) -> list:
    """The loop body as copies of Load (one name), Assigns, Accum; raises Refusal when it is anything else."""
    copies, cur = [], None
    var = loop.axis.name
    for st in loop.body:
        k = kind(st)
        if k == "Load":
            need(cur is None, "a Load before the previous value was folded")
            need(len(st.names) == 1 and st.index, "the fold's Load is not of one value")
            off = index_offset(st.index[-1], var)
            need(off is not None, "the load is not indexed by the loop variable (plus a constant)")
            cur = FoldCopy(st, off, [], None)
        elif k == "Assign":
            need(cur is not None, "arithmetic before the fold's Load")
            cur.chain.append(st)
        elif k == "Accum":
            need(cur is not None, "an Accum without a loaded value")
            cur.accum = st
            copies.append(cur)
            cur = None
        else:
            raise Refusal(f"a {k} inside the fold")
    need(cur is None and copies, "the fold does not end with an Accum")
    return copies


def thread_varying(pre, t_axis: str, src) -> set:
    """Names bound before the fold whose value may differ between the threads of a block: whatever reads the thread
    axis, lane or warp, a buffer the kernel writes, or another such name. (The other Tile axes are the same in all
    threads of a block, the thread axis being the innermost; a name never bound reads as zero everywhere.)"""
    varying = {t_axis, "lane", "warp"}
    for st in pre:
        k = kind(st)
        if k == "Let":
            reads, names = ir.expr_vars(st.value), (st.name,)
        elif k == "Assign":
            reads, names = set(st.args), (st.name,)
        elif k == "Load":
            reads = set().union(*[ir.expr_vars(e) for e in st.index]) if st.index else set()
            names = tuple(st.names)
            if st.input in src.written or st.input not in src.buffers:
                reads = reads | {t_axis}
        else:
            continue
        if reads & varying:
            varying.update(names)
        else:
            varying.difference_update(names)
    return varying


def regroup_refusal(src, tile, pre, loop, copies, merges, comb, tail, t_axis: str, block: int, op: str):
    """Why the cooperating threads of the block may NOT take 16-byte chunks ``4 t + 4 B k + j`` instead of their
    stride ``t + B k`` (None: they may). The reference's conditions, over this module's own analysis:
    shape (emmy_ptx/regroup.py:187-233): the loop starts at the thread's rank, steps by copies * B, has no end
    expression, 4 B divides its extent, copy j reads the loop variable plus j B, every copy computes alike;
    combine (emmy_ptx/regroup.py:75-147): the partials flow only into combines with the loop's own fold - the
    copies' merges, the butterfly over the block's lanes, the tree over its warps - and are not read otherwise;
    ownership (emmy_ptx/lower.py:250-272): nothing the body reads from outside differs between the threads, no
    outer index moves with the thread, the loads read memory the kernel does not write."""
    B, R, var = block, len(copies), loop.axis.name
    extent = loop.axis.extent.as_static()
    if not is_var(loop.start, t_axis):
        return "the loop does not start at each thread's own rank among the block's threads"
    if not is_int(loop.step, R * B):
        return f"the step is not {R} cop{'y' if R == 1 else 'ies'} x {B} threads"
    if loop.end is not None:
        return "the loop has an end expression"
    if extent % (4 * B) or extent < 4 * B:
        return f"{4 * B} (four elements for each of the {B} threads) does not divide the extent {extent}"
    if sorted(c.offset for c in copies) != [j * B for j in range(R)]:
        return "the copies do not read the loop variable plus 0, B, 2 B, ..."
    first = min(copies, key=lambda c: c.offset)
    varying = thread_varying(pre, t_axis, src)
    bound_anywhere = {c.load.names[0] for c in copies} | {a.name for c in copies for a in c.chain}
    states = {c.accum.name for c in copies}
    for c in copies:
        ld = c.load
        buf = src.buffers.get(ld.input)
        if buf is None or ld.input in src.written:
            return f"it reads {ld.input}, which the kernel also writes"
        if ld.input != first.load.input or len(ld.index) != len(first.load.index) or any(
                not same_expr(a, b, {}) for a, b in zip(ld.index[:-1], first.load.index[:-1])):
            return "the copies read different rows"
        for e in ld.index[:-1]:
            if {var, t_axis, "lane", "warp"} & ir.expr_vars(e):
                return "an outer index moves with the loop or with the thread (an element would take its new thread's row)"
        rename = {ld.names[0]: first.load.names[0]}
        if len(c.chain) != len(first.chain):
            return "the copies do not compute alike"
        for a, b in zip(c.chain, first.chain):
            if a.op.name != b.op.name or dtype_name(a.dtype) != dtype_name(b.dtype) or len(a.args) != len(b.args):
                return "the copies do not compute alike"
            for x, y in zip(a.args, b.args):
                if x in states or x == var:
                    return "the body reads an accumulator or the loop variable's value"
                if x in bound_anywhere:
                    if rename.get(x) != y:
                        return "the copies do not compute alike"
                elif x != y:
                    return "the copies do not compute alike"
                elif x in varying:
                    return f"{x} may differ between the cooperating threads (an element would take its new thread's)"
            rename[a.name] = b.name
        acc = c.accum
        if CANON.get(acc.op.name) != op or acc.base is not None or dtype_name(acc.dtype) not in (None, "f32"):
            return "a copy folds with another operation or type"
        if rename.get(acc.value) != (first.accum.value if first.accum.value in bound_anywhere else None):
            return "the copies do not fold the value they computed alike"
    if len(states) != R and len(states) != 1:
        return "the copies share some accumulators and not others"
    live = first.accum.name if len(states) == 1 else None
    merged = set()
    for m in merges:
        if CANON.get(m.op.name) != op:
            return f"{m.value} is folded into {m.name} with {m.op.name}, but the loop folds it with {op}"
        merged.add(m.value)
        live = m.name
    if len(states) > 1 and (live is None or merged | {live} != states or live in merged):
        return "the copies' partials are not all folded into one before the butterfly"
    if comb.state != (live or first.accum.name):
        return "the butterfly does not combine the loop's partial"
    if comb.shuffle_op != op:
        return f"the butterfly combines with {comb.shuffle_op}, but the loop folds with {op}"
    if comb.tree_op is not None and comb.tree_op != op:
        return f"the tree combines with {comb.tree_op}, but the loop folds with {op}"
    for st in ir.walk(tail):
        reads = set(getattr(st, "args", ()) or ()) | set(getattr(st, "values", ()) or ())
        if reads & merged:
            return "a partial folded away is still read"
    return None


def match_reduce(src, strict: bool, disable=frozenset()) -> Plan:
    tile = single_tile(src)
    block = src.launch.block
    t_axis = thread_axis(tile, block)
    body = list(tile.body)
    at = 0
    while at < len(body) and kind(body[at]) in ("Let", "Load", "Assign"):
        at += 1
    pre = body[:at]
    need(at < len(body) and kind(body[at]) == "StridedLoop", "the Tile does not start with a strided fold")
    need(all(kind(s) != "Load" or (len(s.names) == 1 and s.input not in src.written) for s in pre),
         "a Load before the fold that is not one read-only value")
    loop = body[at]
    need(loop.seed and not has_cross(loop.body), "the fold is not seeded or holds cross-thread statements")
    need(loop.body and kind(loop.body[0]) == "Load", "the fold's first statement is not a Load")
    vec = len(loop.body[0].names)
    need(vec in (1, 2, 4), "a load of 3 or more than 4 names")
    var = loop.axis.name
    extent = loop.axis.extent.as_static()
    regrouped, merges, copies = False, [], None
    if vec > 1:
        # the run is spelled in the IR: Load of `vec` names, one Accum per name into one state, in order
        load = loop.body[0]
        accs = loop.body[1:]
        need(len(accs) == vec and all(kind(a) == "Accum" for a in accs), "the fold is not one Accum per loaded value")
        state = accs[0].name
        op = CANON.get(accs[0].op.name)
        need(op in OP_TYPE, f"no template for a fold with {accs[0].op.name}")
        for a, name in zip(accs, load.names):
            need(a.name == state and a.value == name and a.base is None and CANON.get(a.op.name) == op
                 and dtype_name(a.dtype) in (None, "f32"), "the Accums do not fold the loaded values, in order, into one f32 state")
        need(state not in load.names, "the state is overwritten by the load")
        need(not pre, "statements before a fold of multi-name loads")
        chain, value = [], None
    else:
        copies = fold_copies(loop)
        op = CANON.get(copies[0].accum.op.name)
        need(op in OP_TYPE, f"no template for a fold with {copies[0].accum.op.name}")
        load = min(copies, key=lambda c: c.offset).load
    pos = at + 1
    if copies is not None:
        states = {c.accum.name for c in copies}
        while pos < len(body) and kind(body[pos]) == "Accum" and body[pos].base is None and body[pos].name in states \
                and body[pos].value in states and body[pos].name != body[pos].value:
            merges.append(body[pos])
            pos += 1
        state = merges[-1].name if merges else copies[0].accum.name
    comb = match_combine(body, pos, state, block)
    tail = body[pos + comb.consumed:]
    need(not has_cross(tail), "cross-thread statements after the tree")
    slabs = {s.name for s in body if kind(s) == "Smem"}
    need(not slab_read_later(tail, slabs), "the slab is read after the tree")
    for s in ir.walk(tail):
        need(kind(s) in ("Cond", "Write", "Assign", "Let", "Load"), f"a {kind(s)} after the tree")

    remarks = []
    if copies is not None:
        why = None
        if strict:
            why = "--strict keeps the IR's order of additions"
        elif "regroup" in disable:
            why = "disabled"
        else:
            why = regroup_refusal(src, tile, pre, loop, copies, merges, comb, tail, t_axis, block, op)
        if why is None:
            regrouped = True
        else:
            if not strict:
                remarks.append(f"loop {var}: kept strided, not regrouped: {why}")
            c0 = copies[0]
            need(len(copies) == 1 and not merges and c0.offset == 0,
                 f"an unrolled fold that is not regrouped: {why} (the statement lowering keeps its copies)")
            need(c0.accum.base is None and dtype_name(c0.accum.dtype) in (None, "f32"), "the Accum is not a plain f32 fold")
            need(c0.accum.name not in {a for st in c0.chain for a in st.args} and var not in {a for st in c0.chain for a in st.args},
                 "the body reads its accumulator or the loop variable's value")
        first = min(copies, key=lambda c: c.offset)
        chain, value = first.chain, first.accum.value
        need(all(dtype_name(a.dtype) in (None, "f32") for a in chain), "arithmetic in the fold that is not f32")
        need(value == first.load.names[0] or value in {a.name for a in chain}, "the Accum does not fold a value of the body")

    em = Emitter(src, plain=False, strict=strict)
    em.depth = 1
    tile_decode(em, tile, block)
    em.block(pre, None)
    pointer, row = row_pointer(em, src, load, var)
    need(extent <= row, "the loop runs past the buffer's row")
    if regrouped:
        B4 = 4 * block
        need(row % 4 == 0, "the row length is not a multiple of the 16-byte run")
        run, start, step, end = 4, f"(long long)v_{t_axis} * 4LL", f"{B4}LL", f"{extent}LL"
        trips = extent // B4
        if trips > 8 and REDUCE_UNROLL is None:  # two rounds of eight 16-byte loads in flight rather than sixteen at once
            trips = None
    else:
        run = vec
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
        if per_sm * block <= 2048 and 65536 // (per_sm * block) >= 24 + (1 if strict else unroll) * run:
            min_blocks = per_sm
    tree_op = OP_TYPE[comb.tree_op] if comb.tree_op else OP_TYPE[op]
    mapped = ""
    if chain:  # what the body computes from a loaded value before folding it: the statement lowering's expressions
        keep, em.lines = em.lines, []
        em.depth += 1
        em.emit(f"{em.var(load.names[0], 'f32')} = in_;")
        for a in chain:
            em.s_Assign(a)
        code, dt = em.use(value)
        em.emit(f"return {em.convert(code, dt, 'f32')};")
        em.depth -= 1
        inner, em.lines = em.lines, keep
        em.emit("auto map_ = [&](float in_) -> float {")
        em.lines += inner
        em.emit("};")
        mapped = ", map_"
    em.emit(f"float acc_ = emb::strided_fold<{run}, {OP_TYPE[op]}, {unroll}, {str(bool(strict)).lower()}>("
            f"{pointer}, {start}, {step}, {end}{mapped});")
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
    how = "in the IR's own order" if strict else f"on {unroll * run} independent accumulators per thread"
    how += f", {unroll} trips in flight per round"
    if regrouped:
        folds = ", ".join(sorted({f"{c.accum.name} by {c.accum.op.name}" for c in copies}))
        remarks.append(f"loop {var}: the {block} cooperating threads take contiguous 16-byte chunks (4 t + {4 * block} k + j) instead of "
                       f"a stride (checked: the partials ({folds}) flow only into combines with the same fold, and no element's "
                       "value depends on the thread that folds it; the sum is reassociated, so --strict keeps the stride)")
    remarks += [f"block reduction template: {op} fold of {load.input} in {run * 4}-byte ld.global.nc runs, {how}",
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


# ---------------------------------------------------------------- pointwise (elementwise streaming)

POINTWISE_BLOCK = 256   # threads of a CTA of the pointwise template
POINTWISE_RUN = 4       # consecutive cells a thread owns per run (16 bytes of f32)
POINTWISE_RUNS = 4      # runs per thread, BLOCK * RUN cells apart, all of their loads in flight before the arithmetic
STREAM_BYTES = {"f32": 4, "i32": 4, "u32": 4, "f64": 8, "i64": 8, "u64": 8, "f16": 2, "bf16": 2, "i16": 2, "u16": 2,
                "u8": 1, "i8": 1, "bool": 1, "f8e4m3": 1, "f8e5m2": 1}


class PointwiseEmitter(Emitter):
    """The statement lowering with the streaming accesses of a pointwise body rerouted: a Load or Write that
    ``stream`` lists (by identity) takes or leaves lane ``j_`` of a register run instead of touching memory."""

    def __init__(self, src, strict: bool):
        super().__init__(src, plain=False, strict=strict)
        self.stream: dict = {}  # id(statement) -> (register array, element dtype)

    def s_Load(self, s) -> None:
        hit = self.stream.get(id(s))
        if hit is None:
            return super().s_Load(s)
        run, dt = hit
        vdt = self.value_dtype(dt)
        out = dtype_name(s.dtype) or vdt
        self.const_from.pop(s.names[0], None)
        self.reciprocal_of.pop(s.names[0], None)
        self.emit(f"{self.var(s.names[0], out)} = {self.convert(f'{run}.v[j_]', vdt, out)};")

    def s_Write(self, s) -> None:
        hit = self.stream.get(id(s))
        if hit is None:
            return super().s_Write(s)
        run, dt = hit
        code, d = self.use(s.values[0])
        self.emit(f"{run}.v[j_] = {self.convert(code, d, self.value_dtype(dt))};")


def match_pointwise(src, strict: bool) -> Plan:
    """A Tile whose every thread computes its own cell from Loads, Lets and Assigns and writes it: emmy's
    pointwise kernels (the statement kinds of emmy_ptx/elementwise.py; one thread per element, scalar accesses).
    Cells are independent, so which thread owns which cell is free: here a thread owns runs of four cells that are
    consecutive along the innermost axis and moves each run with one access. The arithmetic stays the statement
    lowering's, so every mode keeps its results bit for bit (also --strict: no operation is reordered).
    Conditions: no loop, branch or cross-thread statement; no name read before it is defined (a thread starts a
    cell with zeros in the IR, here with the previous cell's values) and no use of lane or warp (the template
    moves the cells between threads); every streamed buffer is indexed [.., innermost axis] with the outer indices
    free of that axis, row lengths and the axis extent multiples of four, loads from buffers the kernel does not write."""
    tile = single_tile(src)
    body = list(tile.body)
    allowed = ("Load", "Let", "Assign", "Write", "Init", "Select")
    need(body and all(kind(s) in allowed for s in body), "statements other than Load, Let, Assign, Select, Write")
    inner = tile.axes[-1]
    E = inner.extent.as_static()
    axes = [a.name for a in tile.axes]
    need(E % POINTWISE_RUN == 0, f"the innermost axis ({E}) is not a multiple of {POINTWISE_RUN}")
    cells = math.prod(a.extent.as_static() for a in tile.axes)

    defined = set(axes)

    def uses(names):
        for n in names:
            need(n not in ("lane", "warp"), "lane or warp is used (the template moves the cells between threads)")
            need(n in defined, f"{n} is read before it is defined")

    streams = []  # (statement, buffer name, dtype, is_write)
    for st in body:
        k = kind(st)
        if k == "Load":
            for e in st.index:
                uses(ir.expr_vars(e))
            if stream_access(src, st.input, st.index, inner.name) and len(st.names) == 1 and st.input not in src.written:
                streams.append((st, st.input, src.buffers[st.input].dtype, False))
            defined.update(st.names)
        elif k == "Write":
            for e in st.index:
                uses(ir.expr_vars(e))
            uses(st.values)
            need(not st.atomic, "an atomic Write")
            need(st.output in src.buffers, "a Write to shared memory")
            need(stream_access(src, st.output, st.index, inner.name) and len(st.values) == 1,
                 "a Write that is not one value at [.., innermost axis]")
            streams.append((st, st.output, src.buffers[st.output].dtype, True))
        elif k == "Let":
            uses(ir.expr_vars(st.value))
            defined.add(st.name)
        elif k == "Assign":
            uses(st.args)
            defined.add(st.name)
        elif k == "Select":
            for br in st.branches:
                uses([br.value])
                if getattr(br, "select", None) is not None:
                    uses(ir.expr_vars(br.select))
            defined.add(st.name)
        else:  # Init
            defined.add(st.name)
    writes = [x for x in streams if x[3]]
    need(writes, "nothing is written")
    read_names = {x[1] for x in streams if not x[3]}
    need(not ({x[1] for x in writes} & read_names), "a buffer is both streamed in and written")
    need(not any(kind(st) == "Load" and st.input in src.written for st in body), "a Load from a buffer the kernel writes")

    block, run = POINTWISE_BLOCK, POINTWISE_RUN
    runs = POINTWISE_RUNS if cells >= 2 * TARGET_SMS * block * run * POINTWISE_RUNS else 1
    per_cta = block * run * runs
    grid = -(-cells // per_cta)
    em = PointwiseEmitter(src, strict)
    em.depth = 1
    for a in tile.axes:
        em.var(a.name, "i64")
        em.facts[a.name] = None

    def decode(cell: str, with_inner: bool) -> None:
        stride = 1
        for axis in reversed(tile.axes):
            n = axis.extent.as_static()
            if axis is not inner or with_inner:
                term = cell if stride == 1 else f"({cell} / {stride}LL)"
                em.emit(f"v_{axis.name} = {term} % {n}LL;")
            stride *= n

    em.emit(f"const long long first_ = ((long long)blockIdx.x * {runs * block} + threadIdx.x) * {run};")
    em.emit(f"bool ok_[{runs}];")
    for i, (st, buf, dt, is_write) in enumerate(streams):
        em.emit(f"long long at{i}_[{runs}];")
        if not is_write:
            em.emit(f"emb::Run4<{CTYPE[dt]}> in{i}_[{runs}];")
    em.emit("#pragma unroll")
    em.emit(f"for (int u_ = 0; u_ < {runs}; ++u_) {{")
    em.depth += 1
    em.emit(f"long long c_ = first_ + (long long)u_ * {block * run};")
    em.emit(f"ok_[u_] = c_ < {cells}LL;")
    em.emit("if (!ok_[u_]) c_ = 0;")
    decode("c_", True)
    for i, (st, buf, dt, is_write) in enumerate(streams):
        index = st.index
        em.emit(f"at{i}_[u_] = {em.flat(src.buffers[buf].shape, index)};")
    em.depth -= 1
    em.emit("}")
    em.emit("#pragma unroll")
    em.emit(f"for (int u_ = 0; u_ < {runs}; ++u_) {{")
    em.depth += 1
    for i, (st, buf, dt, is_write) in enumerate(streams):
        if not is_write:
            em.emit(f"if (ok_[u_]) in{i}_[u_] = emb::load_run(p_{buf} + at{i}_[u_]);")
    em.depth -= 1
    em.emit("}")
    em.emit("#pragma unroll")
    em.emit(f"for (int u_ = 0; u_ < {runs}; ++u_) {{")
    em.depth += 1
    em.emit("if (!ok_[u_]) continue;")
    em.emit(f"const long long c_ = first_ + (long long)u_ * {block * run};")
    decode("c_", True)
    em.emit(f"const long long inner_ = v_{inner.name};")
    for i, (st, buf, dt, is_write) in enumerate(streams):
        if is_write:
            em.emit(f"emb::Run4<{CTYPE[dt]}> out{i}_;")
            em.stream[id(st)] = (f"out{i}_", dt)
        else:
            em.stream[id(st)] = (f"in{i}_[u_]", dt)
    em.emit("#pragma unroll")
    em.emit(f"for (int j_ = 0; j_ < {run}; ++j_) {{")
    em.depth += 1
    em.emit(f"v_{inner.name} = inner_ + j_;")
    em.block(body, None)
    em.depth -= 1
    em.emit("}")
    for i, (st, buf, dt, is_write) in enumerate(streams):
        if is_write:
            em.emit(f"emb::store_run(p_{buf} + at{i}_[u_], out{i}_);")
    em.depth -= 1
    em.emit("}")
    source = finish(em, src, '#include "emb_pointwise.cuh"', strict, [], None, (), block)
    ins = [x for x in streams if not x[3]]
    moved = sum(STREAM_BYTES[dt] for _, _, dt, _ in streams)
    remarks = [f"pointwise template: {cells} independent cells, {grid} CTAs of {block} threads, {runs} run(s) of {run} consecutive "
               f"cells per thread; {len(ins)} buffer(s) streamed in with one ld.global.nc.L1::no_allocate per run, {len(writes)} out "
               f"with one st.global.cs per run ({moved} B per cell), every load of a thread issued before its arithmetic",
               "the arithmetic is the statement lowering's, statement by statement: the same bits in every mode"]
    remarks += em.remarks
    rows = pointwise_rows(src, tile, streams, body, per_cta)
    return Plan("pointwise", source, remarks, grid=grid, block=block, rows=rows)


def stream_access(src, name: str, index, inner: str) -> bool:
    """Is buffer[index] one element per cell, consecutive in memory for consecutive values of the innermost axis,
    and 4-element aligned whenever that axis is at a multiple of four?"""
    buf = src.buffers.get(name)
    if buf is None or buf.dtype not in STREAM_BYTES or not index or len(index) != len(buf.shape):
        return False
    if not is_var(index[-1], inner) or any(inner in ir.expr_vars(e) for e in index[:-1]):
        return False
    return len(buf.shape) == 1 or int(buf.shape[-1]) % POINTWISE_RUN == 0


def pointwise_rows(src, tile, streams, body, per_cta: int):
    """Row independence for the host (see Plan.rows): the leading Tile axis is used only as the leading index of
    full-rank streamed buffers, and a row is a whole number of CTAs."""
    if len(tile.axes) < 2:
        return None
    lead = tile.axes[0].name
    row_cells = math.prod(a.extent.as_static() for a in tile.axes[1:])
    if row_cells % per_cta:
        return None
    buffers = {}
    streamed = {id(st) for st, _, _, _ in streams}
    for st in body:
        k = kind(st)
        if id(st) in streamed:
            buf = src.buffers[st.input if k == "Load" else st.output]
            if any(lead in ir.expr_vars(e) for e in st.index[1:]):
                return None
            if is_var(st.index[0], lead) and int(buf.shape[0]) == tile.axes[0].extent.as_static():
                buffers[st.input if k == "Load" else st.output] = math.prod(buf.shape[1:]) * STREAM_BYTES[buf.dtype]
            elif lead in ir.expr_vars(st.index[0]):
                return None
            else:
                buffers[st.input if k == "Load" else st.output] = 0
        else:
            used = set()
            if k == "Load":
                for e in st.index:
                    used |= set(ir.expr_vars(e))
            elif k == "Let":
                used = set(ir.expr_vars(st.value))
            elif k == "Assign":
                used = set(st.args)
            elif k == "Select":
                return None
            if lead in used:
                return None
    return dict(count=tile.axes[0].extent.as_static(), ctas_per_row=row_cells // per_cta, buffers=buffers)


MATCHERS = (("softmax", match_softmax), ("reduce", match_reduce), ("pointwise", match_pointwise))
