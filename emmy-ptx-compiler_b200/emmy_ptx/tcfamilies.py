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


def match_attention(src, strict: bool):
    raise Refusal("not built yet")


def match_mlp(src, strict: bool):
    raise Refusal("not built yet")
