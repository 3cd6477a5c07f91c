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
from .codegen import CTYPE
from .families import Plan, Refusal, is_var, need, single_tile
from .ir import dtype_name, kind

TARGET_SMS = 148
GEMM_STAGES = 4
GEMM_GROUP_M = 16
ATTN_POLY_PERIOD = 0  # every n-th pair of softmax weights gets its 2^x from an FMA polynomial instead of the SFU (0: none)


def wrapper(src, includes: str, body: list, extra_sig: list, threads: int, min_blocks: int = 1) -> str:
    sig = codegen.signature(src)
    sig = ", ".join([sig] + extra_sig) if extra_sig else sig
    head = [includes,
            f'extern "C" __global__ void __launch_bounds__({threads}, {min_blocks}) {src.name}({sig}) {{']
    return "\n".join(head + codegen.pdl_prologue(src, True) + body + ["}"]) + "\n"


def tmap(name: str, buffer: str, dtype: str, dims, strides_bytes, box, swizzle: str = "128B") -> dict:
    return dict(kind="tmap", name=name, buffer=buffer, dtype=dtype, dims=[int(d) for d in dims],
                strides_bytes=[int(s) for s in strides_bytes], box=[int(b) for b in box], swizzle=swizzle)


# ---------------------------------------------------------------- matmul


def match_matmul(src, strict: bool) -> Plan:
    tile = single_tile(src)
    need(len(tile.axes) == 2, "the Tile is not over (row, column) cells")
    m_axis, n_axis = tile.axes[0].name, tile.axes[1].name
    M, N = tile.axes[0].extent.as_static(), tile.axes[1].extent.as_static()
    body = list(tile.body)
    need(len(body) == 2 and kind(body[0]) == "Loop" and kind(body[1]) == "Write", "the cell is not one loop and one Write")
    loop, write = body
    k_axis, K = loop.axis.name, loop.axis.extent.as_static()
    need(loop.seed and len(loop.body) == 4 and [kind(s) for s in loop.body] == ["Load", "Load", "Assign", "Accum"],
         "the loop is not Load, Load, multiply, Accum")
    la, lb, mul, acc = loop.body
    need(len(la.names) == 1 and len(lb.names) == 1 and la.dtype is None and lb.dtype is None, "the operand loads are not plain")
    need(mul.op.name == "multiply" and set(mul.args) == {la.names[0], lb.names[0]} and dtype_name(mul.dtype) == "f32",
         "the product is not an f32 multiply of the two loads")
    need(acc.value == mul.name and acc.base is None and codegen.CANON.get(acc.op.name) == "add"
         and dtype_name(acc.dtype) in (None, "f32"), "the accumulator is not an f32 sum of the products")
    # which load is the row operand?
    def operand(load, axis):
        return len(load.index) == 2 and is_var(load.index[0], axis) and is_var(load.index[1], k_axis)
    if operand(la, m_axis) and operand(lb, n_axis):
        a, b = la, lb
    elif operand(lb, m_axis) and operand(la, n_axis):
        a, b = lb, la
    else:
        raise Refusal("the operands are not A[row, k] and B[column, k] (row-major A, column-major B)")
    A, B, C = src.buffers.get(a.input), src.buffers.get(b.input), src.buffers.get(write.output)
    need(A is not None and B is not None and C is not None, "unknown buffers")
    need(A.dtype == B.dtype and A.dtype in ("f16", "bf16"), "the operands are not both f16 or both bf16")
    need(C.dtype == A.dtype, "the output type differs from the operands'")
    need(tuple(A.shape) == (M, K) and tuple(B.shape) == (N, K) and tuple(C.shape) == (M, N), "buffer shapes do not fit the cells")
    need(a.input not in src.written and b.input not in src.written, "the kernel writes an operand")
    need(tuple(write.values) == (acc.name,) and not write.atomic and len(write.index) == 2
         and is_var(write.index[0], m_axis) and is_var(write.index[1], n_axis), "the Write is not C[row, column] = acc")
    need(not strict, "the tensor cores sum a K-slice in their own order (--strict keeps the IR's)")
    need(K % 8 == 0, "the row stride of the operands is not a multiple of 16 bytes (K % 8)")
    need(M * N >= 128 * 256 // 4, "too small for a 128 x 256 tensor-core tile")

    bf16 = A.dtype == "bf16"
    tiles = math.ceil(M / 128) * math.ceil(N / 256)
    grid = min(TARGET_SMS, tiles)
    stage = (128 + 256) * 64 * 2
    smem = GEMM_STAGES * stage + 1024 + 256
    call = [f"    emb::gemm_tn_kernel<{GEMM_STAGES}, {GEMM_GROUP_M}, {str(bf16).lower()}>(&tmap_a, &tmap_b, p_{write.output}, "
            f"emb::GemmShape{{{M}, {N}, {K}}}, status);"]
    extra_sig = ["const __grid_constant__ CUtensorMap tmap_a", "const __grid_constant__ CUtensorMap tmap_b",
                 "unsigned* __restrict__ status"]
    source = wrapper(src, '#include "emb_gemm.cuh"', call, extra_sig, 192)
    extra = [tmap("a", a.input, A.dtype, (K, M), (K * 2,), (64, 128)),
             tmap("b", b.input, B.dtype, (K, N), (K * 2,), (64, 256)),
             dict(kind="status", name="status")]
    remarks = [f"tensor-core matmul template: {M} x {N} x {K} {A.dtype}, f32 accumulation in tensor memory; {tiles} tiles of "
               f"128 x 256 walked by {grid} persistent CTAs of 192 threads (TMA producer, tcgen05.mma issuer, 4 epilogue warps)",
               f"TMA tensor-map loads (128-byte swizzle, no multicast) into {GEMM_STAGES} stages of {stage} B on mbarriers; "
               "two 256-column TMEM accumulators so that a tile's epilogue overlaps the next tile's MMAs",
               f"tile order: {GEMM_GROUP_M} row-blocks share each B panel in L2"]
    return Plan("tensorcore", source, remarks, grid=grid, block=192, smem_bytes=smem, extra_params=extra)


# ---------------------------------------------------------------- attention


def _assign(stmts: dict, name, op=None):
    st = stmts.get(name)
    need(st is not None and kind(st) == "Assign" and (op is None or st.op.name == op), f"{name} is not an Assign of {op}")
    return st


def match_attention(src, strict: bool) -> Plan:
    """emmy's fused attention (examples/a01_attention/k_matmul_softmax_reduce_b55365.ir.txt,
    tests/test_oracle.py:204-231): per (row, output column) thread a key loop that recomputes the row's
    score, then the online update gn = max(m, s), alpha = exp(m - gn), beta = exp(s - gn),
    l = alpha l + beta, o = alpha o + beta v, m = max(m, s); legality as emmy_ptx/mapping.py:413-467
    (the update reads m before m moves, no two sums share an addend, the scores read no carried state)."""
    tile = single_tile(src)
    need(len(tile.axes) >= 2, "the Tile is not over (..., query, column) cells")
    lead = tile.axes[:-2]
    q_axis, c_axis = tile.axes[-2].name, tile.axes[-1].name
    S, D = tile.axes[-2].extent.as_static(), tile.axes[-1].extent.as_static()
    need(D == 128 and src.launch.block == D, "the head dimension (= block) is not 128")
    body = list(tile.body)
    lets = {s.name: s for s in body if kind(s) == "Let"}
    rest = [s for s in body if kind(s) != "Let"]
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
    stmts = {getattr(s, "name", None): s for s in tail if kind(s) == "Assign"}
    accums = [s for s in tail if kind(s) == "Accum"]
    loads = [s for s in tail if kind(s) == "Load"]
    need(len(accums) == 3 and len(loads) == 1 and len(tail) == len(stmts) + 4, "the update is not three Accums around one Load of V")
    m_acc = tail[-1]
    need(kind(m_acc) == "Accum" and codegen.CANON.get(m_acc.op.name) == "maximum" and m_acc.base is None,
         "the maximum does not move last (the update must read m before it moves)")
    m, s_name = m_acc.name, m_acc.value
    sums = [a for a in accums if a is not m_acc]
    need(all(codegen.CANON.get(a.op.name) == "add" and a.base is not None for a in sums), "the sums are not rescaled sums")
    s_st = _assign(stmts, s_name, "multiply")
    need(dot.name in s_st.args, "the score is not the scaled dot product")
    scale_name = [a for a in s_st.args if a != dot.name]
    need(len(scale_name) == 1 and scale_name[0] in lets and kind(lets[scale_name[0]].value) == "Literal"
         and float(lets[scale_name[0]].value.value) > 0, "the scale is not a positive constant")
    scale = float(lets[scale_name[0]].value.value)
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
    vload = loads[0]
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
            need(other in lets and kind(lets[other].value) == "Literal" and float(lets[other].value.value) == 1.0,
                 "the running sum's addend is not beta * 1")
            l_acc = a
    need(l_acc is not None and o_acc is not None and l_acc.value != o_acc.value, "no running sum and output pair (or a shared addend)")
    need(inv.op.name == "reciprocal" and tuple(inv.args) == (l_acc.name,) and res.op.name == "multiply"
         and set(res.args) == {o_acc.name, inv.name}, "the epilogue is not o / l")
    need(tuple(write.values) == (res.name,) and not write.atomic and len(write.index) == len(lead) + 2
         and all(is_var(e, n) for e, n in zip(write.index, lead_names + [q_axis, c_axis])), "the Write is not O[.., query, column]")
    bufs = [src.buffers.get(n) for n in (ql.input, kl.input, vload.input, write.output)]
    need(all(b is not None for b in bufs), "unknown buffers")
    shape = tuple(a.extent.as_static() for a in lead) + (S, D)
    need(all(tuple(b.shape) == shape for b in bufs), "Q, K, V, O do not share the shape [.., S, 128]")
    dt = bufs[0].dtype
    need(dt in ("f16", "bf16") and all(b.dtype == dt for b in bufs), "Q, K, V, O are not all f16 or all bf16")
    need(not ({ql.input, kl.input, vload.input} & set(src.written)), "the kernel writes an operand")
    need(not strict, "the tensor cores and the per-tile softmax sum in their own order (--strict keeps the IR's)")
    need(S % 128 == 0, "the sequence length is not a multiple of the 128-row tile")

    nq = 2 if S % 256 == 0 else 1
    bh = math.prod(a.extent.as_static() for a in lead) if lead else 1
    grid = bh * (S // (nq * 128))
    threads = 64 + 128 * nq
    smem = (nq + 4) * 32768 + 1024 + 256
    scale_log2 = scale * math.log2(math.e)
    call = [f"    emb::attention_fwd_kernel<{nq}, {str(causal).lower()}, {str(dt == 'bf16').lower()}, {ATTN_POLY_PERIOD}>(&tmap_q, &tmap_k, &tmap_v, "
            f"p_{write.output}, emb::AttnShape{{{bh}, {S}, {codegen.c_float(scale_log2)}}}, status);"]
    extra_sig = ["const __grid_constant__ CUtensorMap tmap_q", "const __grid_constant__ CUtensorMap tmap_k",
                 "const __grid_constant__ CUtensorMap tmap_v", "unsigned* __restrict__ status"]
    source = wrapper(src, '#include "emb_attention.cuh"', call, extra_sig, threads)
    rows = bh * S
    extra = [tmap("q", ql.input, dt, (D, rows), (D * 2,), (64, 128)), tmap("k", kl.input, dt, (D, rows), (D * 2,), (64, 128)),
             tmap("v", vload.input, dt, (D, rows), (D * 2,), (64, 128)), dict(kind="status", name="status")]
    remarks = [f"attention template: {bh} (batch, head) pairs x {S} queries, head dimension 128, {dt}, "
               f"{'causal' if causal else 'full'}; {grid} CTAs of {threads} threads, each {nq} query tile(s) of 128 rows "
               "against 128-key tiles (TMA producer, tcgen05.mma issuer, one softmax warp group per query tile)",
               "online softmax recognised (m, l, o with alpha = exp(m - max), beta = exp(s - max)); applied once per 128-key "
               "tile in base 2, O rescaled in tensor memory only when the maximum moves by more than 2^8",
               "S = Q K^T and O += P V on tcgen05.mma with S, P and O in tensor memory; K, V in two TMA stages each; "
               "the CTAs of one (batch, head) are neighbours so that K and V are shared in L2"]
    return Plan("blocking", source, remarks, grid=grid, block=threads, smem_bytes=smem, extra_params=extra)


def match_mlp(src, strict: bool):
    raise Refusal("not built yet")
