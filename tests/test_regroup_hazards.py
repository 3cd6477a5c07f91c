"""The reference's six known-answer kernels for cooperative sums that must NOT be regrouped (tests/kernels.py:187-246,
checked there on the GPU by tests/test_gpu_lowering.py): in each, handing an element to another thread, or a warp's
partial to a total it stays out of, changes the answer, and the inputs are small integers in f32, so any wrong grouping
shows exactly. Rebuilt here with this repository's node classes; the answers are the reference's, stated inline.

On the CPU the oracle must give them; on the GPU every lowering mode must (whatever template or statement path
takes the kernel)."""

import numpy as np
import pytest

from emmy_ptx import runner
from emmy_ptx.ir import (Accum, Assign, Axis, BinaryExpr, Cond, Let, Literal, Load, Smem, StridedLoop, Sync, Tile, TreeHalve, Var,
                         WarpShuffle, Write, datatype)
from helpers import same_bits, source
from oracle import ir_oracle

F32 = datatype("f32")


def lit(v):
    return Literal(value=v, dtype="int" if isinstance(v, int) else "float")


def op(o, a, b):
    return BinaryExpr(op=o, left=a, right=b)


T, IDX = Var(name="t"), Var(name="i")
PLUS = (Assign(name="s", op="add", args=("s", "sb"), dtype=None),)
LANES = WarpShuffle(state=("s",), state_b=("sb",), combine_states=PLUS, length=32, dtype=F32)


def fold(extent, step, body, start=T, axis="i"):
    return StridedLoop(axis=Axis(name=axis, extent=extent), start=start, step=lit(step), body=tuple(body), unroll=False, end=None, seed=True)


def kernel(threads, body, axes=None):
    axes = axes or (Axis(name="t", extent=threads),)
    return (Tile(axes=axes, body=tuple(body), block_threads=threads, aux_threads=0, raster_axes=None, raster_group=None,
                 raster_orient="m"),)


def load(name, buf, *index):
    return Load(names=(name,), input=buf, index=tuple(index), dtype=None)


def acc(name, value):
    return Accum(name=name, value=value, op="add", dtype=F32, axes=(), base=None)


def store(buf, index, value):
    return Write(output=buf, index=(index,), values=(value,), value_dtype=None)


def unit(at, n):
    x = np.zeros(n, np.float32)
    x[at] = 1
    return x


def hazards() -> dict:
    """name -> (body, inputs, threads, answer)"""
    four_ones = np.zeros(128, np.float32)
    four_ones[:4] = 1
    corner = np.zeros((32, 128), np.float32)
    corner[0, 1] = 1
    out = {}
    # every thread weights its own elements by its index: the ones at 0..3 add up to 0 + 1 + 2 + 3
    out["weight"] = (kernel(32, [Let(name="w", value=T, dtype=F32),
                                 fold(128, 32, [load("v", "x", IDX), Assign(name="vw", op="multiply", args=("v", "w"), dtype=None), acc("s", "vw")]),
                                 LANES, store("out", T, "s")]), {"x": four_ones}, 32, np.full(32, 6, np.float32))
    # thread t walks row t: the one at (0, 1) belongs to no thread's elements
    out["row_of_thread"] = (kernel(32, [fold(128, 32, [load("v", "x", T, IDX), acc("s", "v")]), LANES, store("out", T, "s")]),
                            {"x": corner}, 32, np.zeros(32, np.float32))
    # two unrolled copies that scale differently: element 1 is the first copy's, times 2
    out["copies"] = (kernel(32, [Let(name="two", value=lit(2.0), dtype=F32), Let(name="three", value=lit(3.0), dtype=F32),
                                 fold(256, 64, [load("v0", "x", IDX), Assign(name="w0", op="multiply", args=("v0", "two"), dtype=None), acc("s", "w0"),
                                                load("v1", "x", op("+", IDX, lit(32))), Assign(name="w1", op="multiply", args=("v1", "three"), dtype=None),
                                                acc("s1", "w1")]),
                                 acc("s", "s1"), LANES, store("out", T, "s")]), {"x": unit(1, 256)}, 32, np.full(32, 2, np.float32))
    # 4 x 8 cells whose fold starts at the cell's row: the lanes of a row repeat its rank; row 1 owns element 1
    out["start"] = (kernel(32, [fold(64, 4, [load("v", "x", IDX), acc("s", "v")], start=Var(name="r")),
                                WarpShuffle(state=("s",), state_b=("sb",), combine_states=PLUS, length=4, dtype=F32),
                                store("out", op("+", op("*", Var(name="r"), lit(8)), Var(name="c")), "s")],
                           axes=(Axis(name="r", extent=4), Axis(name="c", extent=8))),
                    {"x": unit(1, 64)}, 32, np.repeat(np.array([0, 4, 0, 0], np.float32), 8))
    # only thread 0 hands a partial to the tree (slot 0, warp 0's): element 63 is warp 1's and stays out
    out["one_warp_handed"] = (kernel(64, [Smem(name="slab", extents=(2,), dtype="float", align=0), Let(name="zero", value=lit(0.0), dtype=F32),
                                          Cond(cond=op("<", T, lit(2)), body=(store("slab", T, "zero"),), else_body=()),
                                          Sync(barrier_id=0, count=None, warp=False),
                                          fold(256, 64, [load("v", "x", IDX), acc("s", "v")]), LANES,
                                          Cond(cond=op("==", T, lit(0)), body=(store("slab", lit(0), "s"),), else_body=()),
                                          Sync(barrier_id=0, count=None, warp=False),
                                          TreeHalve(bufs=("slab",), state=("s",), state_b=("sb",), combine_states=PLUS, length=2, tid_var="warp",
                                                    dtype=F32, barrier_id=0, barrier_count=None, inner=None),
                                          store("out", T, "s")]), {"x": unit(63, 256)}, 64, np.zeros(64, np.float32))
    # every thread folds back what it wrote itself (no barrier needed): moved elsewhere, it would read others' writes
    j = Var(name="j")
    out["own_writes"] = (kernel(32, [Smem(name="buf", extents=(128,), dtype="float", align=0),
                                     fold(128, 32, [load("u", "x", j), Let(name="tf", value=T, dtype=F32),
                                                    Assign(name="ut", op="multiply", args=("u", "tf"), dtype=None), store("buf", j, "ut")], axis="j"),
                                     fold(128, 32, [load("v", "buf", IDX), acc("s", "v")]), LANES, store("out", T, "s")]),
                         {"x": np.ones(128, np.float32)}, 32, np.full(32, 4 * sum(range(32)), np.float32))
    return out


@pytest.mark.parametrize("name", sorted(hazards()))
def test_the_oracle_gives_the_known_answers(name):
    body, inputs, threads, answer = hazards()[name]
    bufs = {**{k: v.copy() for k, v in inputs.items()}, "out": np.zeros(answer.shape, np.float32)}
    ir_oracle.run(body, bufs, 1, threads)
    assert same_bits(bufs["out"], answer)


@pytest.mark.gpu
@pytest.mark.parametrize("mode", ["optimized", "strict", "plain"])
@pytest.mark.parametrize("name", sorted(hazards()))
def test_every_lowering_gives_the_known_answers(name, mode):
    body, inputs, threads, answer = hazards()[name]
    out = {"out": np.zeros(answer.shape, np.float32)}
    got = runner.run_source(source("k_hazard", body, inputs, out, 1, threads), {**inputs, **out}, mode)["out"]
    assert same_bits(got, answer), (name, mode, got)
