"""Authoring of split-K matmul problems in emmy's tensor-core (fragment) form, at any size.

The reference ships one such problem (examples/m_f16_128: 128 x 128 x 128 in two K-slabs, then the fold of the
slabs). ``fragment_matmul`` writes the same kind of schedule for other sizes, operand types and B layouts, in the
statement vocabulary of that example (k_matmul__partial.ir.txt): a block of two warps owns a 16 x 32 tile of one
K-slab; 64 threads fill a 16 x 32 A slab and a 32 x 32 B slab per K-step of 32 with 16-byte cp.async into
64-byte-swizzled shared memory, double-buffered; each warp reads its operands with ldmatrix and issues two
mma.sync m16n8k16 per 16 k; RegStore writes the f32 partial. ``staged=False`` is the schedule without shared
memory: every lane reads its fragment elements from global memory, with the row / column clamps and the zero
fill past K that let M, N and the slab length be ragged.
"""

from __future__ import annotations

import math

from .ir import (Accum, Axis, CpAsyncCommit, CpAsyncCopy, CpAsyncWait, LdmatrixLoad, Load, Loop, MmaSyncPtx, RegFragment,
                 RegStore, Smem, StridedLoop, Sync, TernaryExpr, Tile, Write, datatype)
from .problems import B, I, V

F32 = datatype("f32")
SHAPE = (16, 8, 16)


def _sum(*terms):
    out = terms[0]
    for t in terms[1:]:
        out = B("+", out, t)
    return out


def partial_body(m: int, n: int, k: int, splits: int, dtype: str, b_layout: str, staged: bool, guarded: bool = True):
    ks = k // splits
    el = datatype(dtype)
    axes = (Axis(name="_a2_ks", extent=splits), Axis(name="a0_b", extent=math.ceil(m / 16)),
            Axis(name="a1_b", extent=math.ceil(n / 32)), Axis(name="a0_u", extent=1), Axis(name="a1_u", extent=2),
            Axis(name="_lane", extent=32))
    frags = [RegFragment(name="_a0", role="a", shape=SHAPE, dtype=el, count=1, nregs=None),
             RegFragment(name="_b", role="b", shape=SHAPE, dtype=el, count=2, nregs=None),
             RegFragment(name="_c0_", role="c", shape=SHAPE, dtype=F32, count=2, nregs=None)]
    row0, col0 = B("*", V("a0_b"), I(16)), _sum(B("*", V("a1_b"), I(32)), B("*", V("a1_u"), I(16)))
    k_base = B("*", V("_a2_ks"), I(ks))
    mma = StridedLoop(axis=Axis(name="_r0", extent=2), start=I(0), step=I(1), body=(
        MmaSyncPtx(c_frag="_c0_[_r0]", a_frag="_a0", b_frag="_b[_r0]", shape=SHAPE, ab_dtype=dtype, c_dtype="f32",
                   b_row_major=False, sfa_frag=None, sfb_frag=None),), unroll=True, end=None, seed=True)
    if staged:
        assert m % 16 == 0 and n % 32 == 0 and ks % 32 == 0
        t8 = B("*", _sum(B("*", _sum(B("*", V("a0_u"), I(2)), V("a1_u")), I(32)), V("_lane")), I(8))
        row, col = B("/", t8, I(32)), B("%", t8, I(32))  # the thread's 16-byte chunk of a 32-wide slab

        def fills(k_off, stage):
            """cp.async of one K-step into buffer ``stage`` (an expression): A 16 x 32, B 32 x 32 (two per thread)."""
            a = CpAsyncCopy(smem="_a_smem", smem_index=(_sum(B("*", stage, I(16)), I(0)), I(0)), src="x0",
                            src_index=(_sum(row0, row), _sum(k_base, k_off, col)), nbytes=16, swizzle="B64",
                            lane_index=(row, col), lane_rows=16)
            bs = []
            for half in (0, 16):
                if b_layout == "kn":  # slab rows are k
                    src = (_sum(k_base, k_off, row, I(half)), _sum(B("*", V("a1_b"), I(32)), col))
                else:  # slab rows are n
                    src = (_sum(B("*", V("a1_b"), I(32)), row, I(half)), _sum(k_base, k_off, col))
                bs.append(CpAsyncCopy(smem="_b_smem", smem_index=(_sum(B("*", stage, I(32)), I(half)), I(0)), src="x1",
                                      src_index=src, nbytes=16, swizzle="B64", lane_index=(row, col), lane_rows=16))
            return [a, *bs]

        this = B("%", B("/", V("_ks"), I(32)), I(2))
        nxt = B("%", B("+", B("/", V("_ks"), I(32)), I(1)), I(2))
        ahead = TernaryExpr(cond=B("<", B("+", V("_ks"), I(32)), I(ks)), if_true=B("+", V("_ks"), I(32)), if_false=I(max(ks - 32, 0)))
        if b_layout == "kn":
            b_index, b_trans = (_sum(B("*", this, I(32)), V("_ki")), B("*", V("a1_u"), I(16))), False
        else:
            b_index, b_trans = (_sum(B("*", this, I(32)), B("*", V("a1_u"), I(16))), V("_ki")), True
        inner = StridedLoop(axis=Axis(name="_ki", extent=32), start=I(0), step=I(16), body=(
            LdmatrixLoad(frag="_a0", src_buffer="_a_smem", src_index=(_sum(B("*", this, I(16)), B("*", V("a0_u"), I(16))), V("_ki")),
                         role="a", ldm=32, swizzle="B64", staged=True),
            LdmatrixLoad(frag="_b[0]", src_buffer="_b_smem", src_index=b_index, role="b", ldm=32, swizzle="B64", staged=True,
                         b_trans=b_trans, pair_frag="_b[1]"),
            mma), unroll=True, end=None, seed=True)
        outer = StridedLoop(axis=Axis(name="_ks", extent=ks), start=I(0), step=I(32), body=(
            *fills(ahead, nxt), CpAsyncCommit(), CpAsyncWait(group=1), Sync(barrier_id=0, count=None, warp=False), inner,
            Sync(barrier_id=0, count=None, warp=False)), unroll=False, end=None, seed=True)
        work = [Smem(name="_a_smem", extents=(32, 32), dtype="__half" if dtype == "f16" else "__nv_bfloat16", align=512),
                Smem(name="_b_smem", extents=(64, 32), dtype="__half" if dtype == "f16" else "__nv_bfloat16", align=512),
                *fills(I(0), I(0)), CpAsyncCommit(), outer]
        guards = dict(m_guard=None, n_guard=None)
    else:
        k_here = _sum(k_base, V("_ks"))
        k_zero = (k_here, B("*", B("+", V("_a2_ks"), I(1)), I(ks))) if guarded else None
        assert guarded or (m % 16 == 0 and n % 32 == 0 and ks % 16 == 0)
        loads = [LdmatrixLoad(frag="_a0", src_buffer="x0", src_index=(row0, k_here), role="a", ldm=0, staged=False,
                              gmem_guard=(row0, I(m)) if guarded else None, k_zero=k_zero)]
        for r in (0, 1):
            col = _sum(col0, I(8 * r))
            index = (k_here, col) if b_layout == "kn" else (col, k_here)
            loads.append(LdmatrixLoad(frag=f"_b[{r}]", src_buffer="x1", src_index=index, role="b", ldm=0, staged=False,
                                      gmem_guard=(col, I(n)) if guarded else None, k_zero=k_zero, b_trans=b_layout == "nk"))
        work = [StridedLoop(axis=Axis(name="_ks", extent=ks), start=I(0), step=I(16), body=(*loads, mma), unroll=False,
                            end=None, seed=True)]
        guards = dict(m_guard=(row0, I(m)) if guarded else None, n_guard=None)
    stores = []
    for r in (0, 1):
        col = _sum(col0, I(8 * r))
        g = dict(guards)
        if not staged and guarded:
            g["n_guard"] = (col, I(n))
        stores.append(RegStore(dst_buffer="matmul__partial", dst_index=(V("_a2_ks"), row0, col), frag=f"_c0_[{r}]", shape=SHAPE,
                               ldm=0, epilogue=None, extra_frags=(), atomic=False, fragment_index=(0, r), swizzle="NONE",
                               row_dim=1, col_dim=2, **g))
    return (Tile(axes=axes, body=(*frags, *work, *stores), block_threads=64, aux_threads=0, raster_axes=None,
                 raster_group=None, raster_orient="m"),)


def fold_body(m: int, n: int, splits: int, block: int):
    """The second kernel: the slabs summed in index order and rounded once (examples/m_f16_128/k_matmul.ir.txt)."""
    loop = Loop(axis=Axis(name="_a2_ks", extent=splits), body=(
        Load(names=("acc0__p",), input="matmul__partial", index=(V("_a2_ks"), V("a0"), V("a1")), dtype=None),
        Accum(name="acc0", value="acc0__p", op="add", dtype=F32, axes=("_a2_ks",), base=None)), unroll=False, seed=True)
    store = Write(output="matmul", index=(V("a0"), V("a1")), values=("acc0",), value_dtype=F32)
    return (Tile(axes=(Axis(name="a0", extent=m), Axis(name="a1", extent=n)), body=(loop, store), block_threads=block,
                 aux_threads=0, raster_axes=None, raster_group=None, raster_orient="m"),)


def fragment_matmul(m: int = 128, n: int = 128, k: int = 128, splits: int = 2, dtype: str = "f16", b_layout: str = "kn",
                    staged: bool = True, guarded: bool = True, ident: str = "m_fragments"):
    assert k % splits == 0 and b_layout in ("kn", "nk")
    # every 8-column fragment must start inside the matrix (its clamp keeps the lanes in range, not the tile)
    assert staged or n % 32 == 0 or n % 32 > 24
    grid = splits * math.ceil(m / 16) * math.ceil(n / 32)
    fold_block = 256  # a ragged last block is masked by the Tile
    k1 = dict(node="matmul__partial", entry="k_matmul__partial", body=partial_body(m, n, k, splits, dtype, b_layout, staged, guarded),
              grid=grid, block=64, inputs=["x1", "x0"], output=("matmul__partial", [splits, m, n], "f32"), final=False)
    k2 = dict(node="matmul", entry="k_matmul", body=fold_body(m, n, splits, fold_block), grid=math.ceil(m * n / fold_block),
              block=fold_block, inputs=["matmul__partial"], output=("matmul", [m, n], "f16"), final=True)
    scale = 1.0 / math.sqrt(k)
    b_shape = [k, n] if b_layout == "kn" else [n, k]
    return dict(id=ident, code=f"x0 [{m}, {k}] @ x1 [{'K, N' if b_layout == 'kn' else 'N, K'}], {dtype}, {splits} K-slabs",
                rtol=2e-3, atol=2e-3, graph_inputs=["x0", "x1"], graph_outputs=["matmul"], kernels=[k1, k2],
                tensors={"x0": dict(dtype=dtype, shape=[m, k], seed=0, dist="normal", scale=scale),
                         "x1": dict(dtype=dtype, shape=b_shape, seed=1, dist="normal", scale=scale)})
