"""Tensor-core families: matmul, attention and the fused MLP matched in their SIMT IR form and
instantiated as tcgen05 / TMA / TMEM templates.

The reference reaches its tensor-core code from emmy's *fragment* statements
(emmy_ptx/tensorcore.py:147-420), which its interpreter cannot run
(tests/oracle.py:21-23, 120-125). The workloads here are written in the
interpreter's SIMT subset instead (one thread per output cell, a serial loop
over the contraction), so the same file is both the oracle's program and the
pattern these matchers recognise. What is recognised, and the conditions that
must hold (the reference's, where it has the same notion):

  matmul     Tile[m, n]{ Loop k { Load A[m,k]; Load B[n,k]; multiply -> f32; Accum add f32 }; Write C[m,n] }
             accumulators f32 (emmy_ptx/lanes.py:162,250), a pure loop (emmy_ptx/mapping.py:225-227),
             operands read-only, output cast on the Write (tests/oracle.py:225)

Under ``--strict`` these templates refuse: the tensor cores add the products of
a K-slice in an order of their own, so only the statement lowering keeps the
IR's order bit for bit (the reference keeps its mma.sync path under --strict only
because emmy's fragment IR already fixes that order).
"""

from __future__ import annotations

import math

from . import codegen
from .families import Plan, Refusal, is_var, need, single_tile
from .ir import dtype_name, kind

TARGET_SMS = 148
GEMM_STAGES = 4
GEMM_GROUP_M = 16
GEMM_GROUP_M_H = 32       # row-blocks per group of the MLP's first matmul (K = d_model): its B (w1, 128 MiB) is re-read from HBM once per group; measured 16: 3388, 32: 3309, 64: 3515, 8: 3419 us per pass
GEMM_PAIR_STAGES = 6      # CTA pairs: a stage is 32 KB per CTA
GEMM_PAIR_GROUP_M = 8     # in 256-row tiles: the same L2 footprint as 16 row-blocks of 128
GEMM_PAIR_MIN_TILES = 74  # CTA pairs (256 x 256 tiles) only when they give every TPC of the GPU a tile; 0 switches them off
ATTN_POLY_PERIOD = 4  # 128-key template: every n-th pair of softmax weights gets its 2^x from an FMA polynomial instead of the SFU (0: none)
# From a work item's second key tile on, no pass of its own for the row maximum (emb_attention.cuh: OPTIMISTIC). Measured SLOWER on B200
# (1142 against 1070 us on the causal 8 x 32 x 4096 x 128 workload), so it is off unless EMMY_PTX_PREFER=onepass asks for it.
ATTN_OPTIMISTIC = False
# Key tile of the attention template: 64 (two score buffers per query tile and one MMA issuer per query tile, so the next scores are
# ready before the softmax of the current ones ends, emb_attention64.cuh) or 128 (one score buffer per query tile,
# emb_attention.cuh). Measured on the causal 8 x 32 x 4096 x 128 workload: 64: 995-1010 us, 128: 1065 us per pass.
# EMMY_PTX_PREFER=keys64 / keys128 overrides.
ATTN_KEY_TILE = 64
# The 64-key template's share of polynomial exponentials: none. Its softmax warps are bound by issue slots about as much as by
# the SFU (measured 0: 1006, 8: 1011, 4: 1011, 2: 1096 us), so trading one for the other gains nothing.
ATTN_POLY_PERIOD_64 = 0
# Threads per query row of the 64-key template: 1 keeps one softmax warp group per query tile; 2 puts two on it (32 scores of a
# row each, maxima exchanged through shared memory). Measured SLOWER (1090 against 998 us): the exchange costs more than the
# shorter per-tile chain saves, so 2 is only taken when EMMY_PTX_PREFER=split2 asks for it.
ATTN_ROW_SPLIT = 1
GEMM_PAIR_GROUP_M_H = 16  # 256-row tiles per group of a chain matmul with a short contraction (K <= 4096), as GEMM_GROUP_M_H
MLP_GEMM_PAIRS = True  # the MLP chain's matmuls on CTA pairs where the matmul template would take them
# K and V of all heads up to this size: work items longest first over all heads instead of head by head. Measured on causal
# 4096 x 128 f16, one B200: 32 heads (64 MiB) 147.7 -> 129.4 us, 64 heads (128 MiB) 264.1 -> 261.8 us, 128 heads 503.9 -> 543.6 us.
ATTN_L2_RESIDENT_BYTES = 128 << 20


def wrapper(src, includes: str, body: list, extra_sig: list, threads: int, min_blocks: int = 1, cluster: int = 1) -> str:
    sig = codegen.signature(src)
    sig = ", ".join([sig] + extra_sig) if extra_sig else sig
    attrs = f"__cluster_dims__({cluster}, 1, 1) " if cluster > 1 else ""  # the module itself asks for the cluster (.reqnctapercluster)
    head = [includes,
            f'extern "C" __global__ void {attrs}__launch_bounds__({threads}, {min_blocks}) {src.name}({sig}) {{']
    return "\n".join(head + codegen.pdl_prologue(src, True) + body + ["}"]) + "\n"


def prefers(name: str) -> bool:
    """Is the optional, not-by-default rewrite ``name`` asked for (EMMY_PTX_PREFER, a comma-separated list)?"""
    import os
    return name in {n.strip() for n in os.environ.get("EMMY_PTX_PREFER", "").split(",")}


ELEMENT_BYTES = {"u8": 1, "f8e4m3": 1, "f16": 2, "bf16": 2, "f32": 4}
SWIZZLE_SPAN = {"none": None, "32B": 32, "64B": 64, "128B": 128}


def tmap(name: str, buffer: str, dtype: str, dims, strides_bytes, box, swizzle: str = "128B", step=None) -> dict:
    """A tensor-map parameter for the launch header, proved usable on the host before any kernel runs: the
    role the reference's bulk-copy planner has for its copy-engine fills (emmy_ptx/bulk.py:34-57,138-148: it
    evaluates every address and only hands over runs that are contiguous and 16-byte aligned). What a TMA tile
    copy needs: row strides that are multiples of 16 bytes, a box of at most 256 per dimension whose inner extent
    is the swizzle span, and - the one rule nothing checks at run time - inner coordinates that are multiples of
    16 bytes; the templates only ever ask for coordinates that are multiples of ``step`` (default: the box)."""
    size = ELEMENT_BYTES[dtype]
    step = list(step) if step is not None else list(box)
    need(all(int(s) % 16 == 0 for s in strides_bytes), f"tensor map {name}: a row stride is not a multiple of 16 bytes")
    need(all(1 <= int(b) <= 256 for b in box), f"tensor map {name}: a box extent is outside 1..256")
    need((int(box[0]) * size) % 16 == 0, f"tensor map {name}: the inner box extent is not a multiple of 16 bytes")
    span = SWIZZLE_SPAN[swizzle]
    need(span is None or int(box[0]) * size == span, f"tensor map {name}: the inner box extent is not the {swizzle} swizzle span")
    need((int(step[0]) * size) % 16 == 0, f"tensor map {name}: the template's inner coordinates are not multiples of 16 bytes")
    need(all(int(d) >= 1 for d in dims) and len(dims) == len(box) == len(strides_bytes) + 1, f"tensor map {name}: rank mismatch")
    return dict(kind="tmap", name=name, buffer=buffer, dtype=dtype, dims=[int(d) for d in dims],
                strides_bytes=[int(s) for s in strides_bytes], box=[int(b) for b in box], swizzle=swizzle)


# ---------------------------------------------------------------- matmul


def gemm_geometry(M: int, N: int, elem_bytes: int = 2) -> dict:
    """How the matmul template walks an M x N result: lone CTAs on 128 x 256 tiles, or - when there are enough
    256 x 256 tiles to give every pair of SMs one - clusters of two CTAs that run each tile as one
    tcgen05.mma.cta_group::2 (half the operand bytes per CTA for the same tensor work, a deeper ring)."""
    pair_tiles = math.ceil(M / 256) * math.ceil(N / 256)
    if GEMM_PAIR_MIN_TILES and pair_tiles >= GEMM_PAIR_MIN_TILES:
        stage = (128 + 128) * 128
        return dict(kernel="gemm_tn_pair_kernel", stages=GEMM_PAIR_STAGES, group=GEMM_PAIR_GROUP_M, b_rows=128, tiles=pair_tiles,
                    tile="256 x 256", grid=2 * min(TARGET_SMS // 2, pair_tiles), cluster=2, stage=stage,
                    smem=GEMM_PAIR_STAGES * stage + 1024 + 256,
                    how="clusters of two CTAs (one tcgen05.mma.cta_group::2 of 256 x 256 x 16 per step; each CTA loads and "
                        "drains its 128 rows)")
    tiles = math.ceil(M / 128) * math.ceil(N / 256)
    stage = (128 + 256) * 128
    return dict(kernel="gemm_tn_kernel", stages=GEMM_STAGES, group=GEMM_GROUP_M, b_rows=256, tiles=tiles, tile="128 x 256",
                grid=min(TARGET_SMS, tiles), cluster=1, stage=stage, smem=GEMM_STAGES * stage + 1024 + 256,
                how="persistent CTAs")


def match_matmul(src, strict: bool) -> Plan:
    """C = epilogue(A B^T): one thread per cell, a serial contraction loop of f32 products, then optionally Loads
    and Assigns that make the written value from the sum (a bias row, an activation, a scale: what emmy fuses behind
    a matmul), then one Write. B may be stored [N, K] (column-major B) or [K, N] (row-major B: read through an
    MN-major descriptor). The epilogue statements are lowered one by one, with the statement lowering's own rules,
    into a per-cell function the template calls between tensor memory and the store."""
    tile = single_tile(src)
    need(len(tile.axes) == 2, "the Tile is not over (row, column) cells")
    m_axis, n_axis = tile.axes[0].name, tile.axes[1].name
    M, N = tile.axes[0].extent.as_static(), tile.axes[1].extent.as_static()
    body = list(tile.body)
    need(len(body) >= 2 and kind(body[0]) == "Loop" and kind(body[-1]) == "Write", "the cell is not a loop, ..., one Write")
    loop, epilogue, write = body[0], body[1:-1], body[-1]
    k_axis, K = loop.axis.name, loop.axis.extent.as_static()
    need(loop.seed and len(loop.body) == 4 and [kind(s) for s in loop.body] == ["Load", "Load", "Assign", "Accum"],
         "the loop is not Load, Load, multiply, Accum")
    la, lb, mul, acc = loop.body
    need(len(la.names) == 1 and len(lb.names) == 1 and la.dtype is None and lb.dtype is None, "the operand loads are not plain")
    need(mul.op.name == "multiply" and set(mul.args) == {la.names[0], lb.names[0]} and dtype_name(mul.dtype) == "f32",
         "the product is not an f32 multiply of the two loads")
    need(acc.value == mul.name and acc.base is None and codegen.CANON.get(acc.op.name) == "add"
         and dtype_name(acc.dtype) in (None, "f32"), "the accumulator is not an f32 sum of the products")

    def indexed(load, first, second):
        return len(load.index) == 2 and is_var(load.index[0], first) and is_var(load.index[1], second)
    a = next((ld for ld in (la, lb) if indexed(ld, m_axis, k_axis)), None)
    need(a is not None, "no operand is read as A[row, k]")
    b = lb if a is la else la
    if indexed(b, n_axis, k_axis):
        b_kn = False
    elif indexed(b, k_axis, n_axis):
        b_kn = True
    else:
        raise Refusal("the other operand is neither B[column, k] nor B[k, column]")
    A, B, C = src.buffers.get(a.input), src.buffers.get(b.input), src.buffers.get(write.output)
    need(A is not None and B is not None and C is not None, "unknown buffers")
    need(A.dtype == B.dtype and A.dtype in ("f16", "bf16"), "the operands are not both f16 or both bf16")
    need(C.dtype == A.dtype, "the output type differs from the operands'")
    need(tuple(A.shape) == (M, K) and tuple(B.shape) == ((K, N) if b_kn else (N, K)) and tuple(C.shape) == (M, N),
         "buffer shapes do not fit the cells")
    need(a.input not in src.written and b.input not in src.written, "the kernel writes an operand")
    need(not write.atomic and len(write.values) == 1 and len(write.index) == 2
         and is_var(write.index[0], m_axis) and is_var(write.index[1], n_axis), "the Write is not C[row, column] = one value")
    # the epilogue: per-cell statements that may read the sum, the cell's coordinates and read-only buffers
    inner = {la.names[0], lb.names[0], mul.name, k_axis}
    made = {acc.name}
    for st in epilogue:
        k = kind(st)
        need(k in ("Load", "Assign", "Let"), f"a {k} between the loop and the Write")
        if k == "Load":
            need(st.input in src.buffers and st.input not in src.written, "the epilogue loads from a buffer the kernel writes")
            used = set().union(*[ir_vars(e) for e in st.index]) if st.index else set()
            made.update(st.names)
        elif k == "Assign":
            used = set(st.args)
            made.add(st.name)
        else:
            used = ir_vars(st.value)
            made.add(st.name)
        need(not (used & inner), "the epilogue reads a value of the loop's last trip")
        need(not (used & {"lane", "warp"}), "the epilogue reads lane or warp (the template re-deals the cells)")
    need(write.values[0] in made, "the written value is made neither by the loop nor by the epilogue")
    need(epilogue or write.values[0] == acc.name, "the Write is not C[row, column] = acc")
    need(not strict, "the tensor cores sum a K-slice in their own order (--strict keeps the IR's)")
    need(K % 8 == 0 and (not b_kn or N % 8 == 0), "a row stride of an operand is not a multiple of 16 bytes")
    need(M * N >= 128 * 256 // 4, "too small for a 128 x 256 tensor-core tile")

    bf16 = A.dtype == "bf16"
    g = gemm_geometry(M, N)
    if b_kn:  # the MN-major read exists on lone CTAs only
        tiles = math.ceil(M / 128) * math.ceil(N / 256)
        stage = (128 + 256) * 128
        g = dict(kernel="gemm_tn_kernel", stages=GEMM_STAGES, group=GEMM_GROUP_M, b_rows=256, tiles=tiles, tile="128 x 256",
                 grid=min(TARGET_SMS, tiles), cluster=1, stage=stage, smem=GEMM_STAGES * stage + 1024 + 256, how="persistent CTAs")
    pre_lines, cell = [], ""
    if epilogue or write.values[0] != acc.name:
        em = codegen.Emitter(src, plain=False, strict=False)
        em.depth = 2
        em.emit(f"{em.var(m_axis, 'i64')} = row_; {em.var(n_axis, 'i64')} = col_; {em.var(acc.name, 'f32')} = acc_;")
        em.facts[m_axis] = em.facts[n_axis] = None
        for st in epilogue:
            getattr(em, "s_" + kind(st))(st)
        code, dt = em.use(write.values[0])
        em.emit(f"return {em.convert(code, dt, 'f32')};")
        decls = [f"    {codegen.CTYPE[d]} v_{n} = emb::zero<{codegen.CTYPE[d]}>();" for n, d in em.vars.items() if n not in ("lane", "warp")]
        pre_lines = decls + ["    auto cell_ = [&](float acc_, int row_, int col_) -> float {"] + em.lines + ["    };"]
        cell = ", nullptr, cell_"
    lone = g["kernel"] == "gemm_tn_kernel"
    flags = f"{str(bf16).lower()}, emb::EPI_NONE, false" + (f", {str(b_kn).lower()}, false" if lone else "") + (", decltype(cell_)" if cell else "")
    call = pre_lines + [f"    emb::{g['kernel']}<{g['stages']}, {g['group']}, {flags}>(&tmap_a, &tmap_b, p_{write.output}, "
                        f"emb::GemmShape{{{M}, {N}, {K}}}, status{cell});"]
    extra_sig = ["const __grid_constant__ CUtensorMap tmap_a", "const __grid_constant__ CUtensorMap tmap_b",
                 "unsigned* __restrict__ status"]
    includes = '#include "emb_gemm.cuh"' + ("\n" + codegen.PRELUDE.split("\n", 1)[1] if cell else "")
    source = wrapper(src, includes, call, extra_sig, 192, cluster=g["cluster"])
    b_map = tmap("b", b.input, B.dtype, (N, K), (N * 2,), (64, 64)) if b_kn else tmap("b", b.input, B.dtype, (K, N), (K * 2,), (64, g["b_rows"]))
    extra = [tmap("a", a.input, A.dtype, (K, M), (K * 2,), (64, 128)), b_map, dict(kind="status", name="status")]
    remarks = [f"tensor-core matmul template: {M} x {N} x {K} {A.dtype}, f32 accumulation in tensor memory; {g['tiles']} tiles of "
               f"{g['tile']} walked by {g['grid']} CTAs of 192 threads (TMA producer, tcgen05.mma issuer, 4 epilogue warps): {g['how']}",
               f"TMA tensor-map loads (128-byte swizzle, no multicast) into {g['stages']} stages of {g['stage']} B on mbarriers; "
               "two 256-column TMEM accumulators so that a tile's epilogue overlaps the next tile's MMAs",
               f"tile order: {g['group']} row-blocks share each B panel in L2"]
    if b_kn:
        remarks.append("B is stored [K, N]: its tiles are read through an MN-major shared-memory descriptor (four 64-column boxes per stage)")
    if cell:
        remarks.append(f"{len(epilogue)} statement(s) between the loop and the Write run per cell on the accumulator as it leaves tensor "
                       "memory (lowered one by one, as the statement lowering would)")
    return Plan("tensorcore", source, remarks, grid=g["grid"], block=192, cluster=g["cluster"], smem_bytes=g["smem"], extra_params=extra)


def ir_vars(e) -> set:
    from . import ir
    return ir.expr_vars(e)


def match_matmul_e4m3(src, strict: bool) -> Plan:
    """C = scale * A B^T with both operands e4m3 codes decoded by from_f8e4m3 (exact), f32 products and sum:
    tcgen05 kind::f8f6f4 on the codes themselves, the scalar in the epilogue."""
    tile = single_tile(src)
    need(len(tile.axes) == 2, "the Tile is not over (row, column) cells")
    m_axis, n_axis = tile.axes[0].name, tile.axes[1].name
    M, N = tile.axes[0].extent.as_static(), tile.axes[1].extent.as_static()
    body = list(tile.body)
    need(len(body) == 4 and [kind(s) for s in body] == ["Load", "Loop", "Assign", "Write"], "the cell is not scale load, loop, scale, Write")
    sl, loop, scale, write = body
    sbuf = src.buffers.get(sl.input)
    need(sbuf is not None and math.prod(sbuf.shape) == 1 and sbuf.dtype == "f32" and len(sl.names) == 1, "the leading Load is not an f32 scalar")
    k_axis, K = loop.axis.name, loop.axis.extent.as_static()
    need(loop.seed and [kind(s) for s in loop.body] == ["Load", "Load", "Assign", "Assign", "Assign", "Accum"],
         "the loop is not Load, Load, decode, decode, multiply, Accum")
    la, lb, da, db, mul, acc = loop.body
    need({da.op.name, db.op.name} == {"from_f8e4m3"} and {da.args[0], db.args[0]} == {la.names[0], lb.names[0]}
         and mul.op.name == "multiply" and set(mul.args) == {da.name, db.name} and dtype_name(mul.dtype) == "f32"
         and acc.value == mul.name and acc.base is None and codegen.CANON.get(acc.op.name) == "add",
         "the loop does not sum the f32 products of the two decoded codes")
    def operand(load, axis):
        return len(load.index) == 2 and is_var(load.index[0], axis) and is_var(load.index[1], k_axis)
    if operand(la, m_axis) and operand(lb, n_axis):
        a, b = la, lb
    elif operand(lb, m_axis) and operand(la, n_axis):
        a, b = lb, la
    else:
        raise Refusal("the operands are not A[row, k] and B[column, k]")
    A, B, C = src.buffers.get(a.input), src.buffers.get(b.input), src.buffers.get(write.output)
    need(A is not None and B is not None and C is not None and A.dtype == B.dtype == "f8e4m3" and C.dtype in ("bf16", "f16"),
         "not e4m3 operands with a 16-bit result")
    need(tuple(A.shape) == (M, K) and tuple(B.shape) == (N, K) and tuple(C.shape) == (M, N), "buffer shapes do not fit the cells")
    need(scale.op.name == "multiply" and set(scale.args) == {acc.name, sl.names[0]} and tuple(write.values) == (scale.name,)
         and len(write.index) == 2 and is_var(write.index[0], m_axis) and is_var(write.index[1], n_axis) and not write.atomic,
         "the result is not the sum times the scalar, written at C[row, column]")
    need(a.input not in src.written and b.input not in src.written, "the kernel writes an operand")
    need(not strict, "the tensor cores sum a K-slice in their own order (--strict keeps the IR's)")
    need(K % 16 == 0, "the row stride of the operands is not a multiple of 16 bytes (K % 16)")
    tiles = math.ceil(M / 128) * math.ceil(N / 256)
    grid = min(TARGET_SMS, tiles)
    stage = (128 + 256) * 128
    smem = GEMM_STAGES * stage + 1024 + 256
    call = [f"    emb::gemm_tn_kernel<{GEMM_STAGES}, {GEMM_GROUP_M}, {str(C.dtype == 'bf16').lower()}, emb::EPI_SCALE, true>(&tmap_a, &tmap_b, "
            f"p_{write.output}, emb::GemmShape{{{M}, {N}, {K}}}, status, p_{sl.input});"]
    extra_sig = ["const __grid_constant__ CUtensorMap tmap_a", "const __grid_constant__ CUtensorMap tmap_b",
                 "unsigned* __restrict__ status"]
    source = wrapper(src, '#include "emb_gemm.cuh"', call, extra_sig, 192)
    extra = [tmap("a", a.input, "u8", (K, M), (K,), (128, 128)), tmap("b", b.input, "u8", (K, N), (K,), (128, 256)),
             dict(kind="status", name="status")]
    remarks = [f"tensor-core matmul template, e4m3 operands: {M} x {N} x {K}, tcgen05 kind::f8f6f4 on the byte codes, f32 accumulation "
               f"in tensor memory, the scalar in the epilogue; {tiles} tiles of 128 x 256 walked by {grid} persistent CTAs"]
    return Plan("tensorcore", source, remarks, grid=grid, block=192, smem_bytes=smem, extra_params=extra)


# ---------------------------------------------------------------- attention


def _assign(stmts: dict, name, op=None):
    st = stmts.get(name)
    need(st is not None and kind(st) == "Assign" and (op is None or st.op.name == op), f"{name} is not an Assign of {op}")
    return st


def match_attention(src, strict: bool, disable=frozenset()) -> Plan:
    """emmy's fused attention (examples/a01_attention/k_matmul_softmax_reduce_b55365.ir.txt,
    tests/test_oracle.py:204-231): per (row, output column) thread a key loop that recomputes the row's
    score, then the online update gn = max(m, s), alpha = exp(m - gn), beta = exp(s - gn),
    l = alpha l + beta, o = alpha o + beta v, m = max(m, s); legality as emmy_ptx/mapping.py:413-467
    (the update reads m before m moves, no two sums share an addend, the scores read no carried state).
    Spellings taken: the scale as a literal Let or as the reciprocal of a constant (emmy's split of a source
    division, ``reciprocal(div_c1)``); an additive per-key mask loaded between the scaling and the update
    (tests/test_gpu_lowering.py:256-306); the key loop ending at ``query + 1`` (causal) or at the key count; any
    key count (a partial last key tile scores -inf past the end, emmy_ptx/mapping.py:743-754)."""
    tile = single_tile(src)
    need(len(tile.axes) >= 2, "the Tile is not over (..., query, column) cells")
    lead = tile.axes[:-2]
    q_axis, c_axis = tile.axes[-2].name, tile.axes[-1].name
    S, D = tile.axes[-2].extent.as_static(), tile.axes[-1].extent.as_static()
    need(D in (64, 128) and src.launch.block == D, "the head dimension (= block) is neither 64 nor 128")
    body = list(tile.body)
    # constants named before the key loop: literal Lets, scalars loaded from ConstantOp buffers, reciprocals of those
    consts, at = {}, 0
    while at < len(body) and kind(body[at]) != "StridedLoop":
        st = body[at]
        k = kind(st)
        if k == "Let" and kind(st.value) == "Literal":
            consts[st.name] = float(st.value.value)
        elif k == "Load" and len(st.names) == 1 and src.constants.get(st.input) is not None:
            consts[st.names[0]] = float(src.constants[st.input])
        elif k == "Assign" and st.op.name == "reciprocal" and len(st.args) == 1 and consts.get(st.args[0]):
            import numpy as np
            consts[st.name] = float(np.float32(1.0) / np.float32(consts[st.args[0]]))
        else:
            raise Refusal(f"a {k} before the key loop that does not name a constant")
        at += 1
    rest = body[at:]
    need(len(rest) == 4 and [kind(s) for s in rest] == ["StridedLoop", "Assign", "Assign", "Write"],
         "the cell is not key loop, reciprocal, multiply, Write")
    loop, inv, res, write = rest
    key_axis = loop.axis.name
    need(loop.seed and kind(loop.start) == "Literal" and loop.start.value == 0 and kind(loop.step) == "Literal"
         and loop.step.value == 1 and loop.axis.extent.as_static() == S, "the key loop is not 0 .. S step 1")
    if loop.end is None:
        causal = False
    else:
        e = loop.end
        need(kind(e) == "BinaryExpr" and e.op == "+" and is_var(e.left, q_axis) and kind(e.right) == "Literal"
             and e.right.value == 1, "the key loop's end is neither S nor query + 1")
        causal = True
    lb_ = list(loop.body)
    need(lb_ and kind(lb_[0]) == "Loop", "the key loop does not start with the score's dot product")
    dot_loop = lb_[0]
    need(dot_loop.seed and dot_loop.axis.extent.as_static() == D and len(dot_loop.body) == 4
         and [kind(s) for s in dot_loop.body] == ["Load", "Load", "Assign", "Accum"], "the dot product is not Load, Load, multiply, Accum")
    d_axis = dot_loop.axis.name
    l1, l2, prod, dot = dot_loop.body
    need(prod.op.name == "multiply" and set(prod.args) == {l1.names[0], l2.names[0]} and dtype_name(prod.dtype) == "f32"
         and dot.value == prod.name and dot.base is None and codegen.CANON.get(dot.op.name) == "add", "the score is not an f32 dot product")
    lead_names = [a.name for a in lead]

    def indexed(load, row_axis, col_axis):
        idx = load.index
        return (len(idx) == len(lead) + 2 and all(is_var(e, n) for e, n in zip(idx, lead_names))
                and is_var(idx[-2], row_axis) and is_var(idx[-1], col_axis))
    if indexed(l1, q_axis, d_axis) and indexed(l2, key_axis, d_axis):
        ql, kl = l1, l2
    elif indexed(l2, q_axis, d_axis) and indexed(l1, key_axis, d_axis):
        ql, kl = l2, l1
    else:
        raise Refusal("the score does not read Q[.., query, d] and K[.., key, d]")
    tail = lb_[1:]
    for st in tail:  # constants may also be named inside the loop (the reference's test spells its scale there)
        if kind(st) == "Let" and kind(st.value) == "Literal":
            consts[st.name] = float(st.value.value)
    tail = [st for st in tail if not (kind(st) == "Let" and kind(st.value) == "Literal")]
    stmts = {getattr(s, "name", None): s for s in tail if kind(s) == "Assign"}
    accums = [s for s in tail if kind(s) == "Accum"]
    loads = [s for s in tail if kind(s) == "Load"]
    need(len(accums) == 3 and len(loads) in (1, 2) and len(tail) == len(stmts) + 3 + len(loads), "the update is not three Accums around the Load of V")
    m_acc = tail[-1]
    need(kind(m_acc) == "Accum" and codegen.CANON.get(m_acc.op.name) == "maximum" and m_acc.base is None,
         "the maximum does not move last (the update must read m before it moves)")
    m, s_name = m_acc.name, m_acc.value
    sums = [a for a in accums if a is not m_acc]
    need(all(codegen.CANON.get(a.op.name) == "add" and a.base is not None for a in sums), "the sums are not rescaled sums")
    # the score: dot * scale, optionally + mask[key]
    s_st = _assign(stmts, s_name)
    mask_load = None
    if s_st.op.name == "add":
        need(len(loads) == 2, "a score with an addend that is not a loaded mask")
        mask_load = next((ld for ld in loads if ld.names[0] in s_st.args), None)
        need(mask_load is not None and len(s_st.args) == 2, "a score with an addend that is not a loaded mask")
        scaled = [a for a in s_st.args if a != mask_load.names[0]][0]
        s_st = _assign(stmts, scaled, "multiply")
        mbuf = src.buffers.get(mask_load.input)
        need(mbuf is not None and mbuf.dtype == "f32" and tuple(mbuf.shape) == (S,) and len(mask_load.index) == 1
             and is_var(mask_load.index[0], key_axis) and mask_load.input not in src.written, "the mask is not one f32 per key")
    else:
        need(s_st.op.name == "multiply" and len(loads) == 1, "the score is not the scaled dot product")
    need(dot.name in s_st.args, "the score is not the scaled dot product")
    scale_name = [a for a in s_st.args if a != dot.name]
    need(len(scale_name) == 1 and consts.get(scale_name[0], 0.0) > 0, "the scale is not a positive constant")
    scale = consts[scale_name[0]]
    # the two rescaling factors
    exps = [a for a in stmts.values() if a.op.name == "exp"]
    need(len(exps) == 2, "the update does not have exactly two exponentials")

    def factor(e):
        d = _assign(stmts, e.args[0], "subtract")
        g = _assign(stmts, d.args[1], "maximum")
        need(set(g.args) == {m, s_name}, "the new maximum is not max(m, s)")
        return d.args[0]
    alpha = next((e for e in exps if factor(e) == m), None)
    beta = next((e for e in exps if factor(e) == s_name), None)
    need(alpha is not None and beta is not None, "the factors are not exp(m - max) and exp(s - max)")
    vload = next(ld for ld in loads if ld is not mask_load)
    need(indexed(vload, key_axis, c_axis), "V is not read at [.., key, column]")
    l_acc = o_acc = None
    for a in sums:
        base = _assign(stmts, a.base, "multiply")
        need(set(base.args) == {a.name, alpha.name}, "a sum is not rescaled by alpha")
        val = _assign(stmts, a.value, "multiply")
        need(beta.name in val.args, "an addend is not weighted by beta")
        other = [x for x in val.args if x != beta.name][0]
        if other == vload.names[0]:
            o_acc = a
        else:
            need(consts.get(other) == 1.0, "the running sum's addend is not beta * 1")
            l_acc = a
    need(l_acc is not None and o_acc is not None and l_acc.value != o_acc.value, "no running sum and output pair (or a shared addend)")
    need(inv.op.name == "reciprocal" and tuple(inv.args) == (l_acc.name,) and res.op.name == "multiply"
         and set(res.args) == {o_acc.name, inv.name}, "the epilogue is not o / l")
    need(tuple(write.values) == (res.name,) and not write.atomic and len(write.index) == len(lead) + 2
         and all(is_var(e, n) for e, n in zip(write.index, lead_names + [q_axis, c_axis])), "the Write is not O[.., query, column]")
    bufs = [src.buffers.get(n) for n in (ql.input, kl.input, vload.input, write.output)]
    need(all(b is not None for b in bufs), "unknown buffers")
    shape = tuple(a.extent.as_static() for a in lead) + (S, D)
    need(all(tuple(b.shape) == shape for b in bufs), "Q, K, V, O do not share the shape [.., S, D]")
    dt = bufs[0].dtype
    need(dt in ("f16", "bf16") and all(b.dtype == dt for b in bufs), "Q, K, V, O are not all f16 or all bf16")
    need(not ({ql.input, kl.input, vload.input} & set(src.written)), "the kernel writes an operand")
    need(not strict, "the tensor cores and the per-tile softmax sum in their own order (--strict keeps the IR's)")
    need(S >= 1, "no keys")

    nq = 2 if S % 256 == 0 else 1
    bh = math.prod(a.extent.as_static() for a in lead) if lead else 1
    items = bh * math.ceil(S / (nq * 128))
    grid = min(TARGET_SMS, items)
    threads = 64 + 128 * nq
    scale_log2 = scale * math.log2(math.e)
    masked = mask_load is not None
    onepass = (ATTN_OPTIMISTIC or prefers("onepass")) and "onepass" not in disable
    key_tile = 64 if prefers("keys64") else 128 if prefers("keys128") or onepass else ATTN_KEY_TILE  # (one-pass exists on 128-key tiles only)
    # head by head keeps a head's K and V in L2 while its query blocks run; when ALL heads' K and V fit L2 together (a shard of
    # the workload on one of several GPUs) the longest blocks of every head go first, which evens out the end of the launch
    longest_first = causal and 2 * bh * S * D * 2 <= ATTN_L2_RESIDENT_BYTES
    shape_arg = f"emb::AttnShape{{{bh}, {S}, {codegen.c_float(scale_log2)}, {codegen.c_float(1.0 / scale)}, {int(longest_first)}}}"
    mask_arg = ", p_" + mask_load.input if masked else ""
    poly = ATTN_POLY_PERIOD_64 if key_tile == 64 else ATTN_POLY_PERIOD
    flags = f"{nq}, {str(causal).lower()}, {str(dt == 'bf16').lower()}, {poly}, {str(masked).lower()}"
    split = 1
    if key_tile == 64:
        split = 1 if prefers("split1") else 2 if prefers("split2") else ATTN_ROW_SPLIT
        threads = 32 * (1 + nq) + 128 * nq * split  # producer, one issuer per query tile, the softmax warp groups
        smem = nq * (D // 64) * 16384 + 2 * 4 * (D // 64) * 8192 + 1024 + 512 + (4096 if split == 2 else 0)
        include = '#include "emb_attention64.cuh"'
        call = [f"    emb::attention_fwd_kernel64<{flags}, {D}, {split}>(&tmap_q, &tmap_k, &tmap_v, p_{write.output}, {shape_arg}, status{mask_arg});"]
    else:
        smem = (nq + 4) * (D // 64) * 16384 + 1024 + 256
        include = '#include "emb_attention.cuh"'
        call = [f"    emb::attention_fwd_kernel<{flags}, {str(onepass).lower()}, {D}>(&tmap_q, &tmap_k, &tmap_v, p_{write.output}, {shape_arg}, "
                f"status{mask_arg});"]
    extra_sig = ["const __grid_constant__ CUtensorMap tmap_q", "const __grid_constant__ CUtensorMap tmap_k",
                 "const __grid_constant__ CUtensorMap tmap_v", "unsigned* __restrict__ status"]
    source = wrapper(src, include, call, extra_sig, threads)

    def head_map(name, buffer, rows):  # (d, row of the head, head): rows past the end of a head read as zeros
        return tmap(name, buffer, dt, (D, S, bh), (D * 2, S * D * 2), (64, rows, 1))
    extra = [head_map("q", ql.input, 128), head_map("k", kl.input, key_tile), head_map("v", vload.input, key_tile),
             dict(kind="status", name="status")]
    remarks = [f"attention template: {bh} (batch, head) pairs x {S} queries, head dimension {D}, {dt}, "
               f"{'causal' if causal else 'full'}{', additive per-key mask' if masked else ''}; {grid} persistent CTAs of {threads} threads claim "
               f"{items} work items of {nq} query tile(s) of 128 rows against {key_tile}-key tiles (scheduler + TMA producer, "
               f"{'one tcgen05.mma issuer per query tile' if key_tile == 64 else 'tcgen05.mma issuer'}, "
               f"{'two softmax warp groups' if split == 2 else 'one softmax warp group'} per query tile); the next item's loads and first scores overlap the previous item's epilogue",
               f"online softmax recognised (m, l, o with alpha = exp(m - max), beta = exp(s - max)); applied once per {key_tile}-key "
               "tile in base 2, O rescaled in tensor memory only when the maximum moves by more than 2^8" +
               ("; from an item's second key tile on the tile's maximum is tracked during the weights' pass (no pass of its own), a "
                "score more than 2^15 above the reference moves it at once" if onepass else ""),
               "S = Q K^T and O += P V on tcgen05.mma with S, P and O in tensor memory; K, V in " +
               ("four TMA stages each, the scores double-buffered so that the next tile's are ready before the current softmax ends; "
                if key_tile == 64 else "two TMA stages each; ") +
               ("K and V of all heads fit L2 together: work items longest first over all heads" if longest_first else
                "the CTAs of one (batch, head) are neighbours so that K and V are shared in L2")]
    if S % 128:
        remarks.append(f"{S} keys are not a multiple of the 128-key tile: the last tile's slots past the end score -inf, its rows "
                       "past the end are zeros (three-dimensional tensor maps) and are not stored")
    return Plan("blocking", source, remarks, grid=grid, block=threads, smem_bytes=smem, extra_params=extra)


# ---------------------------------------------------------------- fused GELU MLP

GELU_OPS = ["multiply", "multiply", "multiply", "multiply", "add", "multiply", "tanh", "add", "multiply", "multiply"]


MLP_CLUSTER = 8            # CTAs per cluster of the fused MLP template
MLP_FUSED_MAX_COLS = 256   # columns of y one CTA can hold in tensor memory beside two accumulators of a hidden chunk
MLP_FUSED_CLUSTERS = 16    # clusters launched (128 of the 148 SMs: a cluster of 8 must sit inside one GPC)


def mlp_fused_refusal(T: int, D: int, Hd: int):
    """Why the cluster-fused MLP template does not fit these sizes (None: it fits)."""
    C = MLP_CLUSTER
    if D % (16 * C) or D // C > MLP_FUSED_MAX_COLS:
        return (f"d_model {D} over a cluster of {C}: {D / C:g} columns of y per CTA (a multiple of 16, at most {MLP_FUSED_MAX_COLS}: "
                "y's f32 accumulators must fit the tensor memory of the cluster beside the hidden chunk's)")
    if D % 64:
        return f"d_model {D} is not a multiple of the 64-element K-slice"
    if Hd % (128 * C):
        return f"hidden {Hd} is not a multiple of {128 * C} (a chunk of 128 units per CTA and round)"
    return None


def match_mlp(src, strict: bool, disable=frozenset()) -> Plan:
    """y = (gelu_tanh((x . w1) s1) . w2) s2 in emmy's column-recomputing form (examples/k_gelu_mlp/
    k_matmul_reduce_6918c9.ir.txt, tests/kernels.py:99-122): thread (row, column, lane) walks the hidden
    units lane, lane + L, ..., recomputes h = x[row, :] . w1[:, unit] for each (the work the reference's cluster
    rewrite shares, emmy_ptx/cluster.py:120-164), applies GELU, folds g * w2[unit, column]; the L lanes combine
    by butterfly. Weights are e4m3 codes decoded by from_f8e4m3 with per-tensor f32 scales."""
    tile = single_tile(src)
    need(len(tile.axes) == 3, "the Tile is not over (row, column, lane) cells")
    row, col, lane = (a.name for a in tile.axes)
    T, D, L = (a.extent.as_static() for a in tile.axes)
    body = list(tile.body)
    scalars = {}
    while body and kind(body[0]) == "Load":
        ld = body.pop(0)
        buf = src.buffers.get(ld.input)
        need(buf is not None and math.prod(buf.shape) == 1 and len(ld.names) == 1, "a leading Load is not of a scalar")
        scalars[ld.names[0]] = ld.input
    need(len(body) == 4 and [kind(s) for s in body] == ["StridedLoop", "WarpShuffle", "Assign", "Cond"],
         "the cell is not hidden loop, butterfly, scale, guarded Write")
    outer, shuffle, scale_y, cond = body
    need(outer.seed and outer.end is None and is_var(outer.start, lane) and kind(outer.step) == "Literal"
         and outer.step.value == L, "the hidden loop is not lane, lane + L, ...")
    Hd = outer.axis.extent.as_static()
    h_axis = outer.axis.name
    ob = list(outer.body)
    need(len(ob) == 1 + len(GELU_OPS) + 4 and kind(ob[0]) == "Loop", "the hidden loop's body is not dot product, GELU, fold")
    inner = ob[0]
    k_axis = inner.axis.name
    need(inner.seed and inner.axis.extent.as_static() == D and [kind(s) for s in inner.body] == ["Load", "Load", "Assign", "Assign", "Accum"],
         "the dot product is not Load x, Load w1, decode, multiply, Accum")
    lx, lw, dec, mul, acc0 = inner.body
    need(len(lx.index) == 2 and is_var(lx.index[0], row) and is_var(lx.index[1], k_axis) and dtype_name(lx.dtype) == "f32",
         "x is not read as f32 at [row, k]")
    need(len(lw.index) == 2 and is_var(lw.index[0], k_axis) and is_var(lw.index[1], h_axis), "w1 is not read at [k, unit]")
    need(dec.op.name == "from_f8e4m3" and tuple(dec.args) == (lw.names[0],) and mul.op.name == "multiply"
         and set(mul.args) == {dec.name, lx.names[0]} and acc0.value == mul.name and acc0.base is None
         and codegen.CANON.get(acc0.op.name) == "add", "the dot product does not decode w1 and sum x * w1 in f32")
    gelu = ob[1:1 + len(GELU_OPS)]
    need(all(kind(s) == "Assign" for s in gelu) and [s.op.name for s in gelu] == GELU_OPS, "the activation is not the tanh-form GELU")
    hp, h2, h3, t0, t1, t2, th, t3, t4, g = gelu
    consts = {n: src.constants.get(b) for n, b in scalars.items()}

    def const(name, value):
        return name in consts and consts[name] is not None and abs(consts[name] - value) <= 1e-6 * abs(value)
    s1 = [a for a in hp.args if a != acc0.name]
    need(acc0.name in hp.args and len(s1) == 1 and s1[0] in scalars, "h is not the dot product times a scalar scale")
    need(set(h2.args) == {hp.name} and set(h3.args) == {h2.name, hp.name} and h3.name in t0.args
         and any(const(a, 0.044715) for a in t0.args) and set(t1.args) == {hp.name, t0.name} and t1.name in t2.args
         and any(const(a, math.sqrt(2 / math.pi)) for a in t2.args) and tuple(th.args) == (t2.name,)
         and th.name in t3.args and any(const(a, 1.0) for a in t3.args) and hp.name in t4.args
         and any(const(a, 0.5) for a in t4.args) and set(g.args) == {t3.name, t4.name},
         "the activation's constants or wiring are not 0.5 h (1 + tanh(sqrt(2/pi) (h + 0.044715 h^3)))")
    lw2, dec2, mul2, acc1 = ob[1 + len(GELU_OPS):]
    need(kind(lw2) == "Load" and len(lw2.index) == 2 and is_var(lw2.index[0], h_axis) and is_var(lw2.index[1], col)
         and kind(dec2) == "Assign" and dec2.op.name == "from_f8e4m3" and tuple(dec2.args) == (lw2.names[0],)
         and kind(mul2) == "Assign" and mul2.op.name == "multiply" and set(mul2.args) == {dec2.name, g.name}
         and kind(acc1) == "Accum" and acc1.value == mul2.name and acc1.base is None and codegen.CANON.get(acc1.op.name) == "add",
         "the second fold is not sum over units of g * decode(w2[unit, column])")
    need(tuple(shuffle.state) == (acc1.name,) and int(shuffle.length) == L and len(shuffle.combine_states) == 1
         and codegen.CANON.get(shuffle.combine_states[0].op.name) == "add", "the lanes do not add their partial sums")
    s2 = [a for a in scale_y.args if a != acc1.name]
    need(scale_y.op.name == "multiply" and acc1.name in scale_y.args and len(s2) == 1 and s2[0] in scalars, "y is not the sum times a scalar scale")
    from .families import eq_zero
    need(eq_zero(cond.cond, lane) and len(cond.body) == 1 and kind(cond.body[0]) == "Write" and not cond.else_body,
         "the result is not written by lane 0")
    w = cond.body[0]
    need(tuple(w.values) == (scale_y.name,) and len(w.index) == 2 and is_var(w.index[0], row) and is_var(w.index[1], col)
         and not w.atomic, "the Write is not y[row, column]")
    X, W1, W2, Y = (src.buffers.get(n) for n in (lx.input, lw.input, lw2.input, w.output))
    need(all(b is not None for b in (X, W1, W2, Y)), "unknown buffers")
    need(X.dtype == "bf16" and Y.dtype == "bf16" and W1.dtype == "f8e4m3" and W2.dtype == "f8e4m3",
         "not bf16 activations with e4m3 weights")
    need(tuple(X.shape) == (T, D) and tuple(W1.shape) == (D, Hd) and tuple(W2.shape) == (Hd, D) and tuple(Y.shape) == (T, D),
         "buffer shapes do not fit the cells")
    need(Hd % L == 0, "the hidden units do not divide among the lanes")
    need(not ({lx.input, lw.input, lw2.input} & set(src.written)), "the kernel writes an operand")
    need(not strict, "the tensor cores sum in their own order and h is rounded to bf16 between the products (--strict keeps the IR's)")
    need(D % 8 == 0 and Hd % 8 == 0, "row strides are not multiples of 16 bytes")

    e = src.name
    s1_buf, s2_buf = scalars[s1[0]], scalars[s2[0]]
    sig = codegen.signature(src)
    def decode_grid(rows, cols, stream):  # CTAs of the decode: 64 x 128 tiles on the streaming path, else 64 x 64
        return (rows // 64) * (cols // 128) if stream else math.ceil(rows / 64) * math.ceil(cols / 64)
    stream1, stream2 = D % 64 == 0 and Hd % 128 == 0, Hd % 64 == 0 and D % 128 == 0
    decode = ['#include "emb_dequant.cuh"',
              f'extern "C" __global__ void __launch_bounds__(256) {e}__w1(const unsigned char* __restrict__ codes, __nv_bfloat16* __restrict__ out) {{',
              f"    emb::dequant_transpose_e4m3<false, {str(stream1).lower()}>(codes, out, {D}, {Hd});", "}",
              f'extern "C" __global__ void __launch_bounds__(256) {e}__w2(const unsigned char* __restrict__ codes, __nv_bfloat16* __restrict__ out) {{',
              f"    emb::dequant_transpose_e4m3<false, {str(stream2).lower()}>(codes, out, {Hd}, {D});", "}"]
    pre = [
        dict(entry=f"{e}__w1", grid=[decode_grid(D, Hd, stream1), 1, 1], block=[256, 1, 1], cluster=1, smem_bytes=0,
             params=[dict(kind="buffer", name=lw.input), dict(kind="scratch", name="w1t", bytes=Hd * D * 2)]),
        dict(entry=f"{e}__w2", grid=[decode_grid(Hd, D, stream2), 1, 1], block=[256, 1, 1], cluster=1, smem_bytes=0,
             params=[dict(kind="buffer", name=lw2.input), dict(kind="scratch", name="w2t", bytes=D * Hd * 2)]),
    ]
    if "dsmem" in disable:
        fused_why = "disabled"
    elif not prefers("dsmem"):
        fused_why = ("it fits these sizes but is not the default: measured on B200 it is several times slower than the two-matmul "
                     "chain (its operand rings, the chunk and the staging slots share 224 KB of shared memory, too little in flight "
                     "for the TMA latency); EMMY_PTX_PREFER=dsmem selects it") if mlp_fused_refusal(T, D, Hd) is None else \
            mlp_fused_refusal(T, D, Hd)
    else:
        fused_why = mlp_fused_refusal(T, D, Hd)
    if fused_why is None:
        C, ncols = MLP_CLUSTER, D // MLP_CLUSTER
        tiles = math.ceil(T / 128)
        clusters = min(tiles, MLP_FUSED_CLUSTERS)
        smem = 7 * 32768 + 1024 + 256
        lines = ['#include "emb_mlp_fused.cuh"', *decode,
                 f'extern "C" __global__ void __cluster_dims__({C}, 1, 1) __launch_bounds__(256, 1) {e}({sig}, '
                 "const __grid_constant__ CUtensorMap tmap_x, const __grid_constant__ CUtensorMap tmap_w1t, "
                 "const __grid_constant__ CUtensorMap tmap_w2t, unsigned* __restrict__ status) {",
                 f"    emb::mlp_fused_kernel<{C}, {ncols}>(&tmap_x, &tmap_w1t, &tmap_w2t, p_{w.output}, emb::MlpShape{{{T}, {D}, {Hd}}}, "
                 f"p_{s1_buf}, p_{s2_buf}, status);", "}"]
        extra = [tmap("x", lx.input, "bf16", (D, T), (D * 2,), (64, 128)), tmap("w1t", "w1t", "bf16", (D, Hd), (D * 2,), (64, 128)),
                 tmap("w2t", "w2t", "bf16", (Hd, D), (Hd * 2,), (64, ncols)), dict(kind="status", name="status")]
        remarks = [f"MLP template, fused in clusters of {C}: {T} tokens, d_model {D}, hidden {Hd}; a cluster owns 128 token rows, every CTA "
                   f"the f32 accumulators of {ncols} columns of y in tensor memory; per round each CTA computes one chunk of 128 hidden "
                   "units (tcgen05, tanh-GELU on the way out of tensor memory, bf16 into its own shared memory) and gathers the other "
                   f"{C - 1} chunks from its peers' shared memory (mapa + ld.shared::cluster) for y += h_j w2_j: the hidden activations "
                   "never leave the cluster",
                   f"three launches from one module: {e}__w1, {e}__w2 (e4m3 -> bf16 decode, K-major), {e} ({clusters} clusters x {C} CTAs "
                   f"of 256 threads, {smem} B of shared memory each); scratch: {(2 * Hd * D * 2) >> 20} MiB (the decoded weights; no h)",
                   "cluster-wide hand-offs on mbarriers with remote arrivals and bounded waits (no barrier.cluster inside the loop)"]
        return Plan("clusters", "\n".join(lines) + "\n", remarks, grid=clusters * C, block=256, cluster=C, smem_bytes=smem,
                    extra_params=extra, pre=pre)

    # each matmul of the chain on the geometry the matmul template would take for its shape: CTA pairs (cta_group::2,
    # 256 x 256 tiles) when there are enough tiles for every pair of SMs, else lone CTAs
    def chain_gemm(M, N, K, lone_group, epi):
        g = gemm_geometry(M, N) if MLP_GEMM_PAIRS else dict(gemm_geometry(M, N), kernel="")
        if g["kernel"] != "gemm_tn_pair_kernel":
            tiles = math.ceil(M / 128) * math.ceil(N / 256)
            stage = (128 + 256) * 128
            g = dict(kernel="gemm_tn_kernel", stages=GEMM_STAGES, group=lone_group, b_rows=256, tiles=tiles, tile="128 x 256",
                     grid=min(TARGET_SMS, tiles), cluster=1, smem=GEMM_STAGES * stage + 1024 + 256)
        if g["cluster"] == 2 and K <= 4096:
            g["group"] = GEMM_PAIR_GROUP_M_H
        g["call"] = f"emb::{g['kernel']}<{g['stages']}, {g['group']}, true, emb::{epi}>"
        g["attrs"] = "__cluster_dims__(2, 1, 1) " if g["cluster"] == 2 else ""
        return g
    g1 = chain_gemm(T, Hd, D, GEMM_GROUP_M_H, "EPI_SCALE_GELU")
    g2 = chain_gemm(T, D, Hd, GEMM_GROUP_M, "EPI_SCALE")
    tiles1, tiles2 = g1["tiles"], g2["tiles"]
    # launch order: decode w1, h = gelu(x w1), decode w2, y = h w2. The second decode does not need h: it is launched
    # programmatically dependent on the first matmul (which lets its dependents go at once), runs beside it on the SMs'
    # spare shared memory and threads, and one of its threads waits for the matmul at the very end, so the second matmul,
    # an ordinary launch behind it, still starts only when both are complete.
    lines = ['#include "emb_gemm.cuh"', decode[0], *decode[1:4],
             f'extern "C" __global__ void __launch_bounds__(256) {e}__w2(const unsigned char* __restrict__ codes, __nv_bfloat16* __restrict__ out) {{',
             f"    emb::dequant_transpose_e4m3<true, false>(codes, out, {Hd}, {D});", "}",
             f'extern "C" __global__ void {g1["attrs"]}__launch_bounds__(192, 1) {e}__h(const __grid_constant__ CUtensorMap tmap_x, '
             "const __grid_constant__ CUtensorMap tmap_w1t, __nv_bfloat16* __restrict__ h, const float* __restrict__ scale, "
             "unsigned* __restrict__ status) {",
             '    asm volatile("griddepcontrol.launch_dependents;");',
             f"    {g1['call']}(&tmap_x, &tmap_w1t, h, emb::GemmShape{{{T}, {Hd}, {D}}}, status, scale);", "}",
             f'extern "C" __global__ void {g2["attrs"]}__launch_bounds__(192, 1) {e}({sig}, const __grid_constant__ CUtensorMap tmap_h, '
             "const __grid_constant__ CUtensorMap tmap_w2t, unsigned* __restrict__ status) {",
             f"    {g2['call']}(&tmap_h, &tmap_w2t, p_{w.output}, emb::GemmShape{{{T}, {D}, {Hd}}}, status, p_{s2_buf});", "}"]
    w2_decode = dict(pre[1], pdl=True, grid=[decode_grid(Hd, D, False), 1, 1])  # (beside the matmul: the general path, see emb_dequant.cuh)
    pre = [pre[0],
           dict(entry=f"{e}__h", grid=[g1["grid"], 1, 1], block=[192, 1, 1], cluster=g1["cluster"], smem_bytes=g1["smem"],
                params=[tmap("x", lx.input, "bf16", (D, T), (D * 2,), (64, 128)),
                        tmap("w1t", "w1t", "bf16", (D, Hd), (D * 2,), (64, g1["b_rows"])),
                        dict(kind="scratch", name="h", bytes=T * Hd * 2), dict(kind="buffer", name=s1_buf), dict(kind="status", name="status")]),
           w2_decode]
    extra = [tmap("h", "h", "bf16", (Hd, T), (Hd * 2,), (64, 128)), tmap("w2t", "w2t", "bf16", (Hd, D), (Hd * 2,), (64, g2["b_rows"])),
             dict(kind="status", name="status")]
    remarks = [f"MLP template: {T} tokens, d_model {D}, hidden {Hd}; the e4m3 weights are decoded once to bf16 (exactly) and "
               "transposed to K-major, then two tcgen05 matmuls: h = gelu_tanh(s1 x w1) with the activation in the first one's "
               "epilogue (h kept in bf16), y = s2 h w2",
               f"four launches from one module: {e}__w1 (decode), {e}__h ({tiles1} tiles), {e}__w2 (decode, beside {e}__h: launched "
               f"programmatically dependent on it, waits for it only at its end), {e} ({tiles2} tiles); "
               f"scratch: {(2 * Hd * D * 2 + T * Hd * 2) >> 20} MiB",
               f"not fused in a cluster: {fused_why}; h makes one bf16 round trip through L2 / HBM between the two matmuls"]
    return Plan("clusters", "\n".join(lines) + "\n", remarks, grid=g2["grid"], block=192, cluster=g2["cluster"], smem_bytes=g2["smem"],
                extra_params=extra, pre=pre)
