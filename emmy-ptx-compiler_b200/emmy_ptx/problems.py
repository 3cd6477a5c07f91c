"""Authoring of problem folders (``<kernel>.ir.json`` files plus ``meta.json``) for the five workloads.

The reference ships four small example problems (examples/README.md) and gets
the rest from a generator that is not part of it (tools/make_corpus.py:41).
The five benchmark workloads therefore have their Kernel IR written here, in
the file format the examples pin (examples/r01_array_sum/k_sum_1_reduce.ir.json,
examples/m_f16_128/meta.json for a chain of two kernels) and inside the
statement subset the reference's interpreter runs (tests/oracle.py:21-23), so
that the same file drives the compiler and the oracle. Every builder takes the
sizes as arguments: the tests instantiate small ones, ``write_all`` the
full-size ones.

Spelling rules followed (they decide what the oracle computes):
  * an ``Assign`` over f16/bf16/f8 operands carries ``dtype=f32`` (otherwise the
    all-f16 promotion rule keeps the product in f16, emmy_ptx/elementwise.py:62-63);
  * a ``Load`` of several names reads consecutive elements (tests/oracle.py:214-219):
    that is how a thread's 16-byte run is written, so the IR's own order of
    operations is already the vector order and ``--strict`` keeps full bandwidth;
  * scalar constants are ``ConstantOp`` nodes with a one-element argument carrying
    ``data`` (examples/k_gelu_mlp/meta.json).
"""

from __future__ import annotations

import json
import math
from pathlib import Path

from .ir import (Accum, Assign, Axis, BinaryExpr, Cond, Let, Literal, Load, Loop, Smem, StridedLoop, Sync, Tile,
                 TreeHalve, Var, WarpShuffle, Write, datatype)

F32 = datatype("f32")


def I(v):  # noqa: E743
    return Literal(value=int(v), dtype="int")


def B(op, a, b):
    return BinaryExpr(op=op, left=a, right=b)


def V(name):
    return Var(name=name)


def _block_combine(state: str, op: str, block: int, tag: str = "") -> list:
    """The cooperative finish of a per-thread fold: butterfly over the lanes, one slab entry
    per warp, a tree over the warps (the idiom of examples/r01_array_sum/k_sum_1_reduce.ir.txt:5-10)."""
    other = f"{state}__o"
    combine = (Assign(name=state, op=op, args=(state, other), dtype=None),)
    out = [WarpShuffle(state=(state,), state_b=(other,), combine_states=combine, length=min(block, 32), dtype=F32)]
    if block > 32:
        warps = block // 32
        slab = f"{state}_smem{tag}"
        out += [Smem(name=slab, extents=(warps,), dtype="float", align=0),
                Cond(cond=B("==", V("lane"), I(0)),
                     body=(Write(output=slab, index=(V("warp"),), values=(state,), value_dtype=F32),), else_body=()),
                Sync(barrier_id=0, count=None, warp=False),
                TreeHalve(bufs=(slab,), state=(state,), state_b=(other,), combine_states=combine, length=warps,
                          tid_var="warp", dtype=F32, barrier_id=0, barrier_count=None, inner=None)]
    return out


# ---------------------------------------------------------------- cfg 1: array sum (block partials, then their fold)


def sum_partial_body(n: int, grid: int, block: int, vec: int = 4):
    """Kernel 1: block g, thread t folds x[(g*block + t)*vec + k*grid*block*vec + j], j < vec, in that order."""
    loads = tuple(f"in{j}" for j in range(vec))
    body = [Load(names=loads, input="x", index=(V("a0"),), dtype=F32)]
    body += [Accum(name="acc0", value=v, op="add", dtype=F32, axes=("a0",), base=None) for v in loads]
    start = B("*", B("+", B("*", V("a0_b"), I(block)), V("a0_t")), I(vec))
    loop = StridedLoop(axis=Axis(name="a0", extent=n), start=start, step=I(grid * block * vec), body=tuple(body),
                       unroll=False, end=None, seed=True)
    tail = Cond(cond=B("==", V("a0_t"), I(0)),
                body=(Write(output="sum__partial", index=(V("a0_b"),), values=("acc0",), value_dtype=F32),), else_body=())
    return (Tile(axes=(Axis(name="a0_b", extent=grid), Axis(name="a0_t", extent=block)),
                 body=(loop, *_block_combine("acc0", "add", block), tail), block_threads=block, aux_threads=0,
                 raster_axes=None, raster_group=None, raster_orient="m"),)


def sum_final_body(parts: int, block: int):
    """Kernel 2: one block folds the partials the same cooperative way and writes the scalar."""
    loop = StridedLoop(axis=Axis(name="p", extent=parts), start=V("p_t"), step=I(block), body=(
        Load(names=("part",), input="sum__partial", index=(V("p"),), dtype=F32),
        Accum(name="acc0", value="part", op="add", dtype=F32, axes=("p",), base=None)), unroll=False, end=None, seed=True)
    tail = Cond(cond=B("==", V("p_t"), I(0)),
                body=(Write(output="sum_1", index=(), values=("acc0",), value_dtype=F32),), else_body=())
    return (Tile(axes=(Axis(name="p_t", extent=block),), body=(loop, *_block_combine("acc0", "add", block), tail),
                 block_threads=block, aux_threads=0, raster_axes=None, raster_group=None, raster_orient="m"),)


def array_sum(n: int = 1 << 24, grid: int = 1184, block: int = 256, final_block: int = 256, vec: int = 4,
              ident: str = "r_sum_16m") -> dict:
    assert n % vec == 0 and block % 32 == 0 and final_block % 32 == 0
    k1 = dict(node="sum__partial", entry="k_sum__partial", body=sum_partial_body(n, grid, block, vec),
              grid=grid, block=block, inputs=["x"], output=("sum__partial", [grid], "f32"), final=False)
    k2 = dict(node="sum_1", entry="k_sum_1_reduce", body=sum_final_body(grid, final_block), grid=1, block=final_block,
              inputs=["sum__partial"], output=("sum_1", [], "f32"), final=True)
    return dict(id=ident, code=f"(torch.rand({n}) * 2 - 1).sum()", rtol=1e-5, atol=1e-5, graph_inputs=["x"],
                graph_outputs=["sum_1"], kernels=[k1, k2],
                tensors={"x": dict(dtype="f32", shape=[n], seed=0, dist="uniform_pm1")})


def scalar_fold_body(rows: int, cols: int, block: int, src: str, dst: str, copies: int = 1):
    """emmy's own spelling of a cooperative sum (examples/r01_array_sum/k_sum_1_reduce.ir.txt:1-12): block r, thread t
    folds x[r, t], x[r, t + B], ... one scalar at a time; with ``copies`` > 1 the loop is unrolled as emmy does it
    (step copies * B, copy j reads a + j B into an accumulator of its own, the accumulators merged before the butterfly)."""
    row = (V("a0"),) if rows > 1 else ()
    stmts, merges = [], []
    for j in range(copies):
        idx = V("a1") if j == 0 else B("+", V("a1"), I(j * block))
        stmts += [Load(names=(f"in{j}",), input=src, index=(*row, idx), dtype=F32),
                  Accum(name=f"acc{j}", value=f"in{j}", op="add", dtype=F32, axes=("a1",), base=None)]
        if j:
            merges.append(Accum(name="acc0", value=f"acc{j}", op="add", dtype=F32, axes=(), base=None))
    loop = StridedLoop(axis=Axis(name="a1", extent=cols), start=V("a1_co"), step=I(copies * block), body=tuple(stmts),
                       unroll=False, end=None, seed=True)
    tail = Cond(cond=B("==", V("a1_co"), I(0)),
                body=(Write(output=dst, index=row, values=("acc0",), value_dtype=F32),), else_body=())
    axes = ((Axis(name="a0", extent=rows),) if rows > 1 else ()) + (Axis(name="a1_co", extent=block),)
    return (Tile(axes=axes, body=(loop, *merges, *_block_combine("acc0", "add", block), tail), block_threads=block,
                 aux_threads=0, raster_axes=None, raster_group=None, raster_orient="m"),)


def array_sum_scalar(n: int = 1 << 24, grid: int = 2048, block: int = 256, copies: int = 2, ident: str = "r_sum_16m_scalar") -> dict:
    """The array sum as emmy writes it, before any regrouping: scalar loads strided over the block's threads, x seen as
    [grid, n / grid] (one row per block), then the same form over the partials."""
    assert n % grid == 0 and (n // grid) % (copies * block) == 0
    k1 = dict(node="sum__partial", entry="k_sum__partial", body=scalar_fold_body(grid, n // grid, block, "x", "sum__partial", copies),
              grid=grid, block=block, inputs=["x"], output=("sum__partial", [grid], "f32"), final=False)
    k2 = dict(node="sum_1", entry="k_sum_1_reduce", body=scalar_fold_body(1, grid, block, "sum__partial", "sum_1"), grid=1,
              block=block, inputs=["sum__partial"], output=("sum_1", [], "f32"), final=True)
    return dict(id=ident, code=f"(torch.rand({n}) * 2 - 1).sum()", rtol=1e-5, atol=1e-5, graph_inputs=["x"],
                graph_outputs=["sum_1"], kernels=[k1, k2],
                tensors={"x": dict(dtype="f32", shape=[grid, n // grid] if grid > 1 else [n], seed=0, dist="uniform_pm1")})


# ---------------------------------------------------------------- cfg 2: row softmax


def softmax_body(rows: int, cols: int, block: int, vec: int = 4):
    start, step = B("*", V("a1_t"), I(vec)), I(block * vec)

    def loop(axis, body):
        return StridedLoop(axis=Axis(name=axis, extent=cols), start=start, step=step, body=tuple(body), unroll=False,
                           end=None, seed=True)

    def load(prefix, axis):
        names = tuple(f"{prefix}{j}" for j in range(vec))
        return names, Load(names=names, input="x", index=(V("a0"), V(axis)), dtype=F32)

    xs, ld1 = load("xa", "a1")
    phase1 = loop("a1", [ld1] + [Accum(name="m", value=v, op="maximum", dtype=F32, axes=("a1",), base=None) for v in xs])
    ys, ld2 = load("xb", "a2")
    body2 = [ld2]
    for j, v in enumerate(ys):
        body2 += [Assign(name=f"d{j}", op="subtract", args=(v, "m"), dtype=F32),
                  Assign(name=f"e{j}", op="exp", args=(f"d{j}",), dtype=F32),
                  Accum(name="l", value=f"e{j}", op="add", dtype=F32, axes=("a2",), base=None)]
    phase2 = loop("a2", body2)
    zs, ld3 = load("xc", "a3")
    body3 = [ld3]
    for j, v in enumerate(zs):
        body3 += [Assign(name=f"g{j}", op="subtract", args=(v, "m"), dtype=F32),
                  Assign(name=f"h{j}", op="exp", args=(f"g{j}",), dtype=F32),
                  Assign(name=f"o{j}", op="multiply", args=(f"h{j}", "inv"), dtype=F32)]
    body3.append(Write(output="softmax", index=(V("a0"), V("a3")), values=tuple(f"o{j}" for j in range(vec)),
                       value_dtype=F32))
    phase3 = loop("a3", body3)
    stmts = [phase1, *_block_combine("m", "maximum", block, "_m"), phase2, *_block_combine("l", "add", block, "_l"),
             Assign(name="inv", op="reciprocal", args=("l",), dtype=F32), phase3]
    return (Tile(axes=(Axis(name="a0", extent=rows), Axis(name="a1_t", extent=block)), body=tuple(stmts),
                 block_threads=block, aux_threads=0, raster_axes=None, raster_group=None, raster_orient="m"),)


def row_softmax(rows: int = 8192, cols: int = 4096, block: int = 256, vec: int = 4, ident: str = "f_softmax_8192x4096"):
    assert cols % vec == 0 and block % 32 == 0
    k = dict(node="softmax", entry="k_softmax_reduce", body=softmax_body(rows, cols, block, vec), grid=rows, block=block,
             inputs=["x"], output=("softmax", [rows, cols], "f32"), final=True)
    return dict(id=ident, code=f"torch.softmax(torch.randn({rows}, {cols}), dim=-1)", rtol=1e-5, atol=1e-5,
                graph_inputs=["x"], graph_outputs=["softmax"], kernels=[k],
                tensors={"x": dict(dtype="f32", shape=[rows, cols], seed=0, dist="normal")})


# ---------------------------------------------------------------- cfg 3: f16 matmul, A row-major, B column-major


def matmul_body(m: int, n: int, k: int, block: int):
    loop = Loop(axis=Axis(name="a2", extent=k), body=(
        Load(names=("in0",), input="a", index=(V("a0"), V("a2")), dtype=None),
        Load(names=("in1",), input="b", index=(V("a1"), V("a2")), dtype=None),
        Assign(name="v0", op="multiply", args=("in0", "in1"), dtype=F32),
        Accum(name="acc0", value="v0", op="add", dtype=F32, axes=("a2",), base=None)), unroll=False, seed=True)
    store = Write(output="matmul", index=(V("a0"), V("a1")), values=("acc0",), value_dtype=F32)
    return (Tile(axes=(Axis(name="a0", extent=m), Axis(name="a1", extent=n)), body=(loop, store), block_threads=block,
                 aux_threads=0, raster_axes=None, raster_group=None, raster_orient="m"),)


def matmul_f16(m: int = 8192, n: int = 8192, k: int = 8192, block: int = 256, dtype: str = "f16",
               ident: str = "m_f16_8192"):
    assert (m * n) % block == 0
    kern = dict(node="matmul", entry="k_matmul", body=matmul_body(m, n, k, block), grid=m * n // block, block=block,
                inputs=["a", "b"], output=("matmul", [m, n], dtype), final=True)
    scale = 1.0 / math.sqrt(k)
    return dict(id=ident, code=f"a = torch.randn({m}, {k}, dtype=torch.float16) / {k}**0.5; "
                               f"b = torch.randn({n}, {k}, dtype=torch.float16) / {k}**0.5; a @ b.T",
                rtol=2e-3, atol=2e-3, graph_inputs=["a", "b"], graph_outputs=["matmul"], kernels=[kern],
                tensors={"a": dict(dtype=dtype, shape=[m, k], seed=0, dist="normal", scale=scale),
                         "b": dict(dtype=dtype, shape=[n, k], seed=1, dist="normal", scale=scale)})


def matmul_bias_relu(m: int = 512, n: int = 512, k: int = 256, block: int = 256, dtype: str = "f16", b_layout: str = "nk",
                     ident: str = "m_bias_relu"):
    """C = relu(A B^T + bias) * gain: the matmul with statements between its loop and its Write (a bias row, an activation,
    a scalar), and with B stored [N, K] (``b_layout="nk"``) or [K, N] (``"kn"``)."""
    assert (m * n) % block == 0 and b_layout in ("nk", "kn")
    b_index = (V("a1"), V("a2")) if b_layout == "nk" else (V("a2"), V("a1"))
    loop = Loop(axis=Axis(name="a2", extent=k), body=(
        Load(names=("in0",), input="a", index=(V("a0"), V("a2")), dtype=None),
        Load(names=("in1",), input="b", index=b_index, dtype=None),
        Assign(name="v0", op="multiply", args=("in0", "in1"), dtype=F32),
        Accum(name="acc0", value="v0", op="add", dtype=F32, axes=("a2",), base=None)), unroll=False, seed=True)
    epilogue = (Load(names=("bv",), input="bias", index=(V("a1"),), dtype=F32),
                Load(names=("gn",), input="gain", index=(I(0),), dtype=F32),
                Assign(name="z", op="add", args=("acc0", "bv"), dtype=F32),
                Assign(name="r", op="relu", args=("z",), dtype=F32),
                Assign(name="y", op="multiply", args=("r", "gn"), dtype=F32))
    store = Write(output="matmul", index=(V("a0"), V("a1")), values=("y",), value_dtype=F32)
    body = (Tile(axes=(Axis(name="a0", extent=m), Axis(name="a1", extent=n)), body=(loop, *epilogue, store), block_threads=block,
                 aux_threads=0, raster_axes=None, raster_group=None, raster_orient="m"),)
    kern = dict(node="matmul", entry="k_matmul_bias_relu", body=body, grid=m * n // block, block=block,
                inputs=["gain", "a", "b", "bias"], output=("matmul", [m, n], dtype), final=True)
    scale = 1.0 / math.sqrt(k)
    return dict(id=ident, code="torch.relu(a @ b.T + bias) * 1.5", rtol=2e-3, atol=2e-3, graph_inputs=["a", "b", "bias"],
                graph_outputs=["matmul"], kernels=[kern],
                tensors={"a": dict(dtype=dtype, shape=[m, k], seed=0, dist="normal", scale=scale),
                         "b": dict(dtype=dtype, shape=[n, k] if b_layout == "nk" else [k, n], seed=1, dist="normal", scale=scale),
                         "bias": dict(dtype="f32", shape=[n], seed=2, dist="normal", scale=0.5),
                         "gain": dict(dtype="f32", shape=[1], data=[1.5], constant=1.5)})


def matmul_fp8_body(m: int, n: int, k: int, block: int):
    """C = (A . B^T) * scale with A [m, k] and B [n, k] e4m3 codes: decode, f32 products, f32 sum, one scale."""
    loop = Loop(axis=Axis(name="a2", extent=k), body=(
        Load(names=("c0",), input="a", index=(V("a0"), V("a2")), dtype=None),
        Load(names=("c1",), input="b", index=(V("a1"), V("a2")), dtype=None),
        Assign(name="w0", op="from_f8e4m3", args=("c0",), dtype=F32),
        Assign(name="w1", op="from_f8e4m3", args=("c1",), dtype=F32),
        Assign(name="v0", op="multiply", args=("w0", "w1"), dtype=F32),
        Accum(name="acc0", value="v0", op="add", dtype=F32, axes=("a2",), base=None)), unroll=False, seed=True)
    return (Tile(axes=(Axis(name="a0", extent=m), Axis(name="a1", extent=n)), body=(
        Load(names=("s",), input="ab_scale", index=(I(0),), dtype=F32), loop,
        Assign(name="y", op="multiply", args=("acc0", "s"), dtype=F32),
        Write(output="matmul", index=(V("a0"), V("a1")), values=("y",), value_dtype=F32)), block_threads=block,
        aux_threads=0, raster_axes=None, raster_group=None, raster_orient="m"),)


def matmul_fp8(m: int = 8192, n: int = 8192, k: int = 8192, block: int = 256, ident: str = "m_e4m3_8192"):
    """Both operands e4m3 (drawn from N(0, 1), per-tensor scaled), f32 accumulation, bf16 result."""
    assert (m * n) % block == 0
    kern = dict(node="matmul", entry="k_matmul_e4m3", body=matmul_fp8_body(m, n, k, block), grid=m * n // block, block=block,
                inputs=["ab_scale", "a", "b"], output=("matmul", [m, n], "bf16"), final=True)
    return dict(id=ident, code="(deq(a) @ deq(b).T) with e4m3 a, b", rtol=3e-2, atol=3e-2, graph_inputs=["a", "b"],
                graph_outputs=["matmul"], kernels=[kern],
                tensors={"a": dict(dtype="f8e4m3", shape=[m, k], seed=0, dist="normal", quant="a_scale"),
                         "b": dict(dtype="f8e4m3", shape=[n, k], seed=1, dist="normal", quant="b_scale"),
                         "ab_scale": dict(dtype="f32", shape=[1], scale_product=["a", "b"])})


# ---------------------------------------------------------------- cfg 4: causal attention, online softmax


def attention_body(batch: int, heads: int, seq: int, dim: int, scale: float, causal: bool = True, mask: bool = False,
                   scale_as: str = "let"):
    """One block per (batch, head, query): thread c holds output column c; every thread of the block
    computes the row's scores (the work a template shares), emmy's fused form
    (examples/a01_attention/k_matmul_softmax_reduce_b55365.ir.txt, tests/test_oracle.py:214-231). ``mask`` adds a
    per-key f32 value to the scaled score (tests/test_gpu_lowering.py:256-306); ``scale_as="reciprocal"`` spells
    the scale as emmy does after splitting a source division: the reciprocal of the constant ``div_c1``."""
    bhq = (V("a0"), V("a1"), V("a2"))
    dot = Loop(axis=Axis(name="a5", extent=dim), body=(
        Load(names=("qv",), input="q", index=(*bhq, V("a5")), dtype=None),
        Load(names=("kv",), input="k", index=(V("a0"), V("a1"), V("a4"), V("a5")), dtype=None),
        Assign(name="p", op="multiply", args=("qv", "kv"), dtype=F32),
        Accum(name="dot", value="p", op="add", dtype=F32, axes=("a5",), base=None)), unroll=False, seed=True)
    score = ((Assign(name="s", op="multiply", args=("dot", "scale"), dtype=F32),) if not mask else
             (Assign(name="s0", op="multiply", args=("dot", "scale"), dtype=F32),
              Load(names=("mk",), input="mask", index=(V("a4"),), dtype=F32),
              Assign(name="s", op="add", args=("s0", "mk"), dtype=F32)))
    update = (
        dot,
        *score,
        Assign(name="gn", op="maximum", args=("m", "s"), dtype=F32),
        Assign(name="dg", op="subtract", args=("m", "gn"), dtype=F32),
        Assign(name="alpha", op="exp", args=("dg",), dtype=F32),
        Assign(name="dgo", op="subtract", args=("s", "gn"), dtype=F32),
        Assign(name="beta", op="exp", args=("dgo",), dtype=F32),
        Assign(name="la", op="multiply", args=("l", "alpha"), dtype=F32),
        Assign(name="lb", op="multiply", args=("one", "beta"), dtype=F32),
        Accum(name="l", value="lb", op="add", dtype=F32, axes=("a4",), base="la"),
        Assign(name="oa", op="multiply", args=("o", "alpha"), dtype=F32),
        Load(names=("vv",), input="v", index=(V("a0"), V("a1"), V("a4"), V("a3")), dtype=None),
        Assign(name="ob", op="multiply", args=("vv", "beta"), dtype=F32),
        Accum(name="o", value="ob", op="add", dtype=F32, axes=("a4",), base="oa"),
        Accum(name="m", value="s", op="maximum", dtype=F32, axes=("a4",), base=None),
    )
    keys = StridedLoop(axis=Axis(name="a4", extent=seq), start=I(0), step=I(1), body=update, unroll=False,
                       end=B("+", V("a2"), I(1)) if causal else None, seed=True)
    if scale_as == "let":
        named = (Let(name="scale", value=Literal(value=float(scale), dtype="float"), dtype=F32),)
    else:
        named = (Load(names=("dc",), input="div_c1", index=(I(0),), dtype=F32),
                 Assign(name="scale", op="reciprocal", args=("dc",), dtype=F32))
    stmts = (*named,
             Let(name="one", value=Literal(value=1.0, dtype="float"), dtype=F32),
             keys,
             Assign(name="inv", op="reciprocal", args=("l",), dtype=F32),
             Assign(name="res", op="multiply", args=("o", "inv"), dtype=F32),
             Write(output="attn", index=(*bhq, V("a3")), values=("res",), value_dtype=F32))
    axes = (Axis(name="a0", extent=batch), Axis(name="a1", extent=heads), Axis(name="a2", extent=seq),
            Axis(name="a3", extent=dim))
    return (Tile(axes=axes, body=stmts, block_threads=dim, aux_threads=0, raster_axes=None, raster_group=None,
                 raster_orient="m"),)


def attention(batch: int = 8, heads: int = 32, seq: int = 4096, dim: int = 128, causal: bool = True,
              dtype: str = "f16", mask: bool = False, scale_as: str = "let", ident: str = "a_f16_causal_8x32x4096x128"):
    import numpy as np
    scale = float(np.float32(1.0 / math.sqrt(dim)))
    shape = [batch, heads, seq, dim]
    extra = (["mask"] if mask else []) + (["div_c1"] if scale_as == "reciprocal" else [])
    kern = dict(node="attn", entry="k_attention", body=attention_body(batch, heads, seq, dim, scale, causal, mask, scale_as),
                grid=batch * heads * seq, block=dim, inputs=[*extra, "q", "k", "v"], output=("attn", shape, dtype), final=True)
    tensors = {n: dict(dtype=dtype, shape=shape, seed=i, dist="normal") for i, n in enumerate("qkv")}
    if mask:  # a tenth of the keys far below every score; the tests overwrite it to mask whole tiles
        tensors["mask"] = dict(dtype="f32", shape=[seq], seed=7, dist="normal", scale=1.0)
    if scale_as == "reciprocal":
        tensors["div_c1"] = dict(dtype="f32", shape=[1], data=[math.sqrt(dim)], constant=math.sqrt(dim))
    return dict(id=ident, code="torch.nn.functional.scaled_dot_product_attention(q, k, v, is_causal=%s)" % causal,
                rtol=2e-3, atol=2e-3, graph_inputs=["q", "k", "v"], graph_outputs=["attn"], kernels=[kern], tensors=tensors)


# ---------------------------------------------------------------- cfg 5: fused tanh-GELU MLP, bf16 x, e4m3 weights

GELU_C = math.sqrt(2.0 / math.pi)
GELU_K = 0.044715


def mlp_body(tokens: int, d_model: int, hidden: int, lanes: int):
    """Thread (row, col, lane): lane-strided hidden units, each recomputing h = x[row,:] . w1[:,unit]
    (the work the cluster template shares), the shape of examples/k_gelu_mlp/k_matmul_reduce_6918c9.ir.txt."""
    inner = Loop(axis=Axis(name="a3", extent=d_model), body=(
        Load(names=("xv",), input="x", index=(V("a0"), V("a3")), dtype=F32),
        Load(names=("c1",), input="w1", index=(V("a3"), V("a2")), dtype=None),
        Assign(name="wa", op="from_f8e4m3", args=("c1",), dtype=F32),
        Assign(name="v0", op="multiply", args=("wa", "xv"), dtype=F32),
        Accum(name="acc0", value="v0", op="add", dtype=F32, axes=("a3",), base=None)), unroll=False, seed=True)
    gelu = (
        Assign(name="hp", op="multiply", args=("acc0", "s1"), dtype=F32),
        Assign(name="h2", op="multiply", args=("hp", "hp"), dtype=F32),
        Assign(name="h3", op="multiply", args=("h2", "hp"), dtype=F32),
        Assign(name="t0", op="multiply", args=("h3", "gk"), dtype=F32),
        Assign(name="t1", op="add", args=("hp", "t0"), dtype=F32),
        Assign(name="t2", op="multiply", args=("t1", "gc"), dtype=F32),
        Assign(name="th", op="tanh", args=("t2",), dtype=F32),
        Assign(name="t3", op="add", args=("one", "th"), dtype=F32),
        Assign(name="t4", op="multiply", args=("hp", "half"), dtype=F32),
        Assign(name="g", op="multiply", args=("t3", "t4"), dtype=F32),
    )
    outer = StridedLoop(axis=Axis(name="a2", extent=hidden), start=V("a2_co"), step=I(lanes), body=(
        inner, *gelu,
        Load(names=("c2",), input="w2", index=(V("a2"), V("a1")), dtype=None),
        Assign(name="wb", op="from_f8e4m3", args=("c2",), dtype=F32),
        Assign(name="v6", op="multiply", args=("wb", "g"), dtype=F32),
        Accum(name="acc1", value="v6", op="add", dtype=F32, axes=("a2",), base=None)), unroll=False, end=None, seed=True)
    pre = (Load(names=("s1",), input="w1_scale", index=(I(0),), dtype=F32),
           Load(names=("s2",), input="w2_scale", index=(I(0),), dtype=F32),
           Load(names=("half",), input="gelu_half", index=(I(0),), dtype=F32),
           Load(names=("gc",), input="gelu_c", index=(I(0),), dtype=F32),
           Load(names=("gk",), input="gelu_k", index=(I(0),), dtype=F32),
           Load(names=("one",), input="gelu_one", index=(I(0),), dtype=F32))
    shuffle = WarpShuffle(state=("acc1",), state_b=("acc1__o",),
                          combine_states=(Assign(name="acc1", op="add", args=("acc1", "acc1__o"), dtype=None),),
                          length=lanes, dtype=F32)
    post = (Assign(name="yv", op="multiply", args=("acc1", "s2"), dtype=F32),
            Cond(cond=B("==", V("a2_co"), I(0)),
                 body=(Write(output="mlp", index=(V("a0"), V("a1")), values=("yv",), value_dtype=F32),), else_body=()))
    axes = (Axis(name="a0", extent=tokens), Axis(name="a1", extent=d_model), Axis(name="a2_co", extent=lanes))
    return (Tile(axes=axes, body=(*pre, outer, shuffle, *post), block_threads=None, aux_threads=0, raster_axes=None,
                 raster_group=None, raster_orient="m"),)


def gelu_mlp(tokens: int = 16384, d_model: int = 4096, hidden: int = 16384, lanes: int = 8, block: int = 256,
             ident: str = "k_mlp_gelu_tanh_16384x4096x16384"):
    cells = tokens * d_model * lanes
    assert cells % block == 0 and hidden % lanes == 0 and block % lanes == 0
    consts = {"gelu_half": 0.5, "gelu_c": GELU_C, "gelu_k": GELU_K, "gelu_one": 1.0}
    kern = dict(node="mlp", entry="k_mlp_gelu", body=mlp_body(tokens, d_model, hidden, lanes), grid=cells // block,
                block=block, inputs=["w1_scale", "w2_scale", *consts, "x", "w1", "w2"],
                output=("mlp", [tokens, d_model], "bf16"), final=True)
    tensors = {"x": dict(dtype="bf16", shape=[tokens, d_model], seed=0, dist="normal"),
               "w1": dict(dtype="f8e4m3", shape=[d_model, hidden], seed=1, dist="normal", scale=0.02, quant="w1_scale"),
               "w2": dict(dtype="f8e4m3", shape=[hidden, d_model], seed=2, dist="normal", scale=0.02, quant="w2_scale"),
               "w1_scale": dict(dtype="f32", shape=[1], scale_of="w1"),
               "w2_scale": dict(dtype="f32", shape=[1], scale_of="w2")}
    for name, value in consts.items():
        tensors[name] = dict(dtype="f32", shape=[1], data=[value], constant=value)
    return dict(id=ident, code="torch.nn.functional.gelu(x @ deq(w1), approximate='tanh') @ deq(w2)", rtol=3e-2,
                atol=3e-2, graph_inputs=["x", "w1", "w2"], graph_outputs=["mlp"], kernels=[kern], tensors=tensors)


# ---------------------------------------------------------------- pointwise: bias + tanh-GELU, and bias + ReLU + residual


def _gelu_tanh(x: str, out: str, tag: str = "") -> list:
    """out = 0.5 x (1 + tanh(c (x + k x^3))), one Assign per operation (the spelling of tools/corpus_specs.py:104-105
    after emmy splits it; constants as loaded one-element arguments like examples/k_gelu_mlp/meta.json)."""
    t = lambda n: f"{n}{tag}"  # noqa: E731
    return [Assign(name=t("x2"), op="multiply", args=(x, x), dtype=F32),
            Assign(name=t("x3"), op="multiply", args=(t("x2"), x), dtype=F32),
            Assign(name=t("u0"), op="multiply", args=(t("x3"), "gk"), dtype=F32),
            Assign(name=t("u1"), op="add", args=(x, t("u0")), dtype=F32),
            Assign(name=t("u2"), op="multiply", args=(t("u1"), "gc"), dtype=F32),
            Assign(name=t("th"), op="tanh", args=(t("u2"),), dtype=F32),
            Assign(name=t("u3"), op="add", args=("one", t("th")), dtype=F32),
            Assign(name=t("u4"), op="multiply", args=(x, "half"), dtype=F32),
            Assign(name=out, op="multiply", args=(t("u3"), t("u4")), dtype=F32)]


def bias_gelu_body(rows: int, cols: int, block: int):
    """One thread per element (emmy's pointwise form): y[r, c] = gelu_tanh(x[r, c] + bias[c])."""
    consts = (Load(names=("half",), input="gelu_half", index=(I(0),), dtype=F32),
              Load(names=("gc",), input="gelu_c", index=(I(0),), dtype=F32),
              Load(names=("gk",), input="gelu_k", index=(I(0),), dtype=F32),
              Load(names=("one",), input="gelu_one", index=(I(0),), dtype=F32))
    stmts = (*consts,
             Load(names=("xv",), input="x", index=(V("a0"), V("a1")), dtype=F32),
             Load(names=("bv",), input="bias", index=(V("a1"),), dtype=F32),
             Assign(name="z", op="add", args=("xv", "bv"), dtype=F32),
             *_gelu_tanh("z", "g"),
             Write(output="y", index=(V("a0"), V("a1")), values=("g",), value_dtype=F32))
    return (Tile(axes=(Axis(name="a0", extent=rows), Axis(name="a1", extent=cols)), body=stmts, block_threads=block,
                 aux_threads=0, raster_axes=None, raster_group=None, raster_orient="m"),)


def bias_gelu(rows: int = 8192, cols: int = 4096, block: int = 256, ident: str = "e_bias_gelu_8192x4096"):
    assert (rows * cols) % block == 0
    consts = {"gelu_half": 0.5, "gelu_c": GELU_C, "gelu_k": GELU_K, "gelu_one": 1.0}
    kern = dict(node="y", entry="k_bias_gelu", body=bias_gelu_body(rows, cols, block), grid=rows * cols // block, block=block,
                inputs=[*consts, "x", "bias"], output=("y", [rows, cols], "f32"), final=True)
    tensors = {"x": dict(dtype="f32", shape=[rows, cols], seed=0, dist="normal"),
               "bias": dict(dtype="f32", shape=[cols], seed=1, dist="normal")}
    for name, value in consts.items():
        tensors[name] = dict(dtype="f32", shape=[1], data=[value], constant=value)
    return dict(id=ident, code=f"torch.nn.functional.gelu(torch.randn({rows}, {cols}) + torch.randn({cols}), approximate='tanh')",
                rtol=1e-5, atol=1e-6, graph_inputs=["x", "bias"], graph_outputs=["y"], kernels=[kern], tensors=tensors)


def bias_relu_residual_body(rows: int, cols: int, block: int):
    """y[r, c] = max(x[r, c] + bias[c], 0) + res[r, c]: three streams of 4 bytes per element, two IEEE additions."""
    stmts = (Load(names=("xv",), input="x", index=(V("a0"), V("a1")), dtype=F32),
             Load(names=("bv",), input="bias", index=(V("a1"),), dtype=F32),
             Load(names=("rv",), input="res", index=(V("a0"), V("a1")), dtype=F32),
             Assign(name="z", op="add", args=("xv", "bv"), dtype=F32),
             Assign(name="a", op="relu", args=("z",), dtype=F32),
             Assign(name="o", op="add", args=("a", "rv"), dtype=F32),
             Write(output="y", index=(V("a0"), V("a1")), values=("o",), value_dtype=F32))
    return (Tile(axes=(Axis(name="a0", extent=rows), Axis(name="a1", extent=cols)), body=stmts, block_threads=block,
                 aux_threads=0, raster_axes=None, raster_group=None, raster_orient="m"),)


def bias_relu_residual(rows: int = 8192, cols: int = 4096, block: int = 256, ident: str = "e_bias_relu_res_8192x4096"):
    assert (rows * cols) % block == 0
    kern = dict(node="y", entry="k_bias_relu_res", body=bias_relu_residual_body(rows, cols, block), grid=rows * cols // block,
                block=block, inputs=["x", "bias", "res"], output=("y", [rows, cols], "f32"), final=True)
    tensors = {"x": dict(dtype="f32", shape=[rows, cols], seed=0, dist="normal"),
               "bias": dict(dtype="f32", shape=[cols], seed=1, dist="normal"),
               "res": dict(dtype="f32", shape=[rows, cols], seed=2, dist="normal")}
    return dict(id=ident, code=f"torch.relu(torch.randn({rows}, {cols}) + torch.randn({cols})) + torch.randn({rows}, {cols})",
                rtol=0.0, atol=0.0, graph_inputs=["x", "bias", "res"], graph_outputs=["y"], kernels=[kern], tensors=tensors)


# ---------------------------------------------------------------- files


def _graph(problem: dict, kern: dict) -> dict:
    nodes = {}
    for name in kern["inputs"]:
        t = problem["tensors"].get(name)
        if t is None:  # the output of an earlier kernel of the chain
            prev = next(k for k in problem["kernels"] if k["output"][0] == name)
            t = dict(dtype=prev["output"][2], shape=prev["output"][1])
        out = [dict(name=name, shape=list(t["shape"]), dtype=t["dtype"])]
        if "constant" in t:
            nodes[name] = dict(op="ConstantOp", op_fields=dict(
                name=name, value=t["constant"], context_value=None, load_ops=[], source_path=None, source_parts=[],
                source_shape=None, source_dtype=None, source_graph=None), inputs=[], outputs=out)
        else:
            nodes[name] = dict(op="InputOp", op_fields={}, inputs=[], outputs=out)
    oname, oshape, odtype = kern["output"]
    nodes[kern["node"]] = dict(op="KernelOp", op_fields=dict(body=[repr(s) for s in kern["body"]], name=kern["entry"],
                                                             zero_delegated=[], serial=[]),
                               inputs=list(kern["inputs"]), outputs=[dict(name=oname, shape=list(oshape), dtype=odtype)])
    return dict(inputs=list(kern["inputs"]), outputs=[oname], nodes=nodes)


def _meta(problem: dict) -> dict:
    kernels = []
    produced = set()
    for kern in problem["kernels"]:
        args = []
        for name in kern["inputs"]:
            t = problem["tensors"].get(name)
            if name in produced:
                prev = next(k for k in problem["kernels"] if k["output"][0] == name)
                args.append(dict(name=name, dtype=prev["output"][2], shape=list(prev["output"][1]), intermediate=True))
            elif "data" in t:
                args.append(dict(name=name, dtype=t["dtype"], shape=list(t["shape"]), data=list(t["data"])))
            else:  # ``seed`` as in the reference; dist/scale/quant/scale_of are this build's additions
                extra = {k: t[k] for k in ("seed", "dist", "scale", "quant", "scale_of", "scale_product") if k in t}
                args.append(dict(name=name, dtype=t["dtype"], shape=list(t["shape"]), **extra))
        oname, oshape, odtype = kern["output"]
        args.append(dict(name=oname, dtype=odtype, shape=list(oshape) or [1], output=True))
        produced.add(oname)
        kernels.append(dict(node=kern["node"], entry=kern["entry"], arg_order=[a["name"] for a in args],
                            grid=[kern["grid"], 1, 1], block=[kern["block"], 1, 1], smem_bytes=0, zero_outputs=[],
                            args=args, final=bool(kern["final"])))
    return dict(id=problem["id"], code=problem["code"], rtol=problem["rtol"], atol=problem["atol"],
                graph_inputs=problem["graph_inputs"], graph_outputs=problem["graph_outputs"], kernels=kernels)


def write(problem: dict, root) -> Path:
    """Write ``<root>/<id>/{<entry>.ir.json..., meta.json}`` and return the folder."""
    folder = Path(root) / problem["id"]
    folder.mkdir(parents=True, exist_ok=True)
    for kern in problem["kernels"]:
        (folder / f"{kern['entry']}.ir.json").write_text(json.dumps(_graph(problem, kern), indent=1))
    (folder / "meta.json").write_text(json.dumps(_meta(problem), indent=1))
    return folder


def matmul_fragments(m: int = 8192, n: int = 8192, k: int = 8192, ident: str = "m_f16_8192_fragments"):
    """The matmul workload as emmy hands tensor-core kernels over: a warp-level mma.sync schedule (B stored N x K,
    one K-slab) and the fold kernel behind it, in the form of examples/m_f16_128 of the reference."""
    from . import fragproblems
    return fragproblems.fragment_matmul(m=m, n=n, k=k, splits=1, dtype="f16", b_layout="nk", ident=ident)


WORKLOADS = {"sum": array_sum, "softmax": row_softmax, "matmul": matmul_f16, "attention": attention, "mlp": gelu_mlp,
             "fragments": matmul_fragments, "elementwise": bias_gelu, "elementwise_add": bias_relu_residual,
             "sum_scalar": array_sum_scalar,
             "mlp_2048": lambda **kw: gelu_mlp(**{**dict(tokens=16384, d_model=2048, hidden=8192, ident="k_mlp_gelu_tanh_16384x2048x8192"), **kw})}


def write_all(root) -> list:
    """The five full-size workloads, the matmul once more in fragment form, and the two pointwise workloads."""
    return [write(make(), root) for make in WORKLOADS.values()]
