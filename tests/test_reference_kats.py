"""Known-answer kernels of the reference's GPU tests (tests/test_gpu_lowering.py) that are not random: the segmented
tree with an inner slot and the segmented butterfly (:141-177), the one-cell maximum over 70000 values on a whole block
(:335-345), the division recovered from x * reciprocal(c) by the constant's name (:498-551), the tree that leaves its
levels in shared memory (:853-871) and the cross-lane maximum of per-lane sums (:874-890). Rebuilt with this
repository's node classes; the oracle must give the stated answers on the CPU, every lowering mode on the GPU."""

import numpy as np
import pytest

from emmy_ptx import runner
from emmy_ptx.ir import (Accum, Assign, Axis, BinaryExpr, Cond, Init, Let, Literal, Load, Loop, Smem, StridedLoop, Sync, Tile, TreeHalve, Var,
                         WarpShuffle, Write, datatype)
from helpers import same_bits, source
from oracle import ir_oracle

F32 = datatype("f32")
T = Var(name="t")


def num(v):
    return Literal(value=v, dtype="int" if isinstance(v, int) else "float")


def bop(o, a, b):
    return BinaryExpr(op=o, left=a, right=b)


def tile(threads, body, axes=None):
    axes = (Axis(name="t", extent=threads),) if axes is None else axes
    return (Tile(axes=axes, body=tuple(body), block_threads=threads if axes else None, aux_threads=0, raster_axes=None, raster_group=None,
                 raster_orient="m"),)


def plus(state, other):
    return (Assign(name=state, op="add", args=(state, other), dtype=None),)


def ld(name, buf, *index):
    return Load(names=(name,), input=buf, index=tuple(index), dtype=None)


def st(buf, index, value):
    return Write(output=buf, index=tuple(index), values=(value,), value_dtype=None)


def rng():
    return np.random.default_rng(42)


def segmented_tree(named: bool):
    """slot = segment * 4 + inner: every thread ends with the sum over the 32 segments of its inner slot"""
    x = rng().standard_normal(128).astype(np.float32)
    barrier = Sync(barrier_id=1, count=128, warp=False) if named else Sync(barrier_id=0, count=None, warp=False)
    body = tile(128, [ld("x0", "x", T), Smem(name="buf", extents=(128,), dtype="float", align=0), st("buf", (T,), "x0"), barrier,
                      Let(name="seg", value=bop("/", T, num(4)), dtype=None), Let(name="inn", value=bop("%", T, num(4)), dtype=None),
                      Init(name="acc", identity=0.0, dtype=F32),
                      TreeHalve(bufs=("buf",), state=("acc",), state_b=("acc__o",), combine_states=plus("acc", "acc__o"), length=32,
                                tid_var="seg", dtype=F32, barrier_id=1 if named else 0, barrier_count=128 if named else None, inner=("inn", 4)),
                      st("out", (T,), "acc")])
    want = x.reshape(32, 4).astype(np.float64).sum(0)[np.arange(128) % 4]
    return body, {"x": x}, (128,), 1, 128, ("close", want)


def segmented_butterfly():
    x = rng().standard_normal(64).astype(np.float32)
    body = tile(64, [ld("x0", "x", T), Init(name="acc", identity=0.0, dtype=F32), Accum(name="acc", value="x0", op="add", dtype=F32),
                     WarpShuffle(state=("acc",), state_b=("acc__o",), combine_states=plus("acc", "acc__o"), length=8, dtype=F32),
                     st("out", (T,), "acc")])
    return body, {"x": x}, (64,), 1, 64, ("close", np.repeat(x.reshape(8, 8).astype(np.float64).sum(1), 8))


def one_cell_maximum():
    x = rng().standard_normal(70000).astype(np.float32)
    body = tile(256, [Loop(axis=Axis(name="k", extent=70000), body=(ld("xv", "x", Var(name="k")), Accum(name="top", value="xv", op="maximum", dtype=F32)),
                           unroll=False, seed=True), st("out", (), "top")], axes=())
    return body, {"x": x}, (1,), 1, 256, ("exact", np.array([x.max()], np.float32))


def tree_left_in_shared_memory():
    """after the tree, slot 0 holds the root and the other slots what the tree left there: 1+2+3+4 -> [10, 6, 3, 4]"""
    warp = bop(">>", T, num(5))
    body = tile(128, [Smem(name="partials", extents=(4,), dtype="float", align=0), Init(name="s", identity=0.0, dtype=F32),
                      Let(name="v", value=bop("+", warp, num(1)), dtype=None),
                      Cond(cond=bop("==", bop("&", T, num(31)), num(0)), body=(st("partials", (warp,), "v"),), else_body=()),
                      Sync(barrier_id=0, count=None, warp=False),
                      TreeHalve(bufs=("partials",), state=("s",), state_b=("sb",), combine_states=plus("s", "sb"), length=4, tid_var="t",
                                dtype=F32, barrier_id=0, barrier_count=None, inner=None),
                      ld("slot", "partials", bop("&", T, num(3))), st("out", (num(0), T), "s"), st("out", (num(1), T), "slot")])
    want = np.stack([np.full(128, 10.0, np.float32), np.tile(np.array([10, 6, 3, 4], np.float32), 32)])
    return body, {}, (2, 128), 1, 128, ("exact", want)


def cross_lane(op: str, answer: float):
    """each lane sums four strided elements, then the lanes combine: with a maximum the elements must stay with their lanes
    (ones at 0..3 give 1, not 4)"""
    x = np.zeros(128, np.float32)
    x[:4] = 1
    i = Var(name="i")
    body = tile(32, [StridedLoop(axis=Axis(name="i", extent=128), start=T, step=num(32), body=(ld("v", "x", i), Accum(name="s", value="v", op="add", dtype=F32)),
                                 unroll=False, end=None, seed=True),
                     WarpShuffle(state=("s",), state_b=("sb",), combine_states=(Assign(name="s", op=op, args=("s", "sb"), dtype=None),), length=32, dtype=F32),
                     st("out", (T,), "s")])
    return body, {"x": x}, (32,), 1, 32, ("exact", np.full(32, answer, np.float32))


CASES = {"segmented tree": lambda: segmented_tree(False), "segmented tree, named barrier": lambda: segmented_tree(True),
         "segmented butterfly": segmented_butterfly, "one-cell maximum": one_cell_maximum, "tree left in shared memory": tree_left_in_shared_memory,
         "maximum of lane sums": lambda: cross_lane("maximum", 1.0), "sum of lane sums": lambda: cross_lane("add", 4.0)}


def verdict(got, kind_, want):
    if kind_ == "exact":
        return same_bits(np.asarray(got).reshape(want.shape), want)
    return np.allclose(got, want, rtol=1e-5, atol=1e-5)


@pytest.mark.parametrize("name", sorted(CASES))
def test_the_oracle_gives_the_answers(name):
    body, inputs, shape, grid, block, (kind_, want) = CASES[name]()
    bufs = {**inputs, "out": np.zeros(shape, np.float32)}
    ir_oracle.run(body, bufs, grid, block)
    assert verdict(bufs["out"], kind_, want)


@pytest.mark.gpu
@pytest.mark.parametrize("mode", ["optimized", "strict", "plain"])
@pytest.mark.parametrize("name", sorted(CASES))
def test_every_lowering_gives_the_answers(name, mode):
    body, inputs, shape, grid, block, (kind_, want) = CASES[name]()
    out = {"out": np.zeros(shape, np.float32)}
    got = runner.run_source(source("k_kat", body, inputs, out, grid, block), {**inputs, **out}, mode)["out"]
    assert verdict(got, kind_, want), (name, mode)


# ---------------------------------------------------------------- the division emmy split


DIVISORS = {"div_c1": 3.0, "div_2_c1": 7.0, "div_3_c1": -0.1, "x_mean_count": 300.0, "div_4_c1": 0.5}


def division_kernel(n: int):
    i = Var(name="i")
    stmts = [ld("x", "xs", i)]
    for k, name in enumerate(DIVISORS):
        stmts += [ld(f"c{k}", name, num(0)), Assign(name=f"r{k}", op="reciprocal", args=(f"c{k}",), dtype=None),
                  Assign(name=f"q{k}", op="multiply", args=("x", f"r{k}"), dtype=None), st("out", (num(k), i), f"q{k}")]
    return tile(256, stmts, axes=(Axis(name="i", extent=n),))


def division_inputs(n: int):
    x = np.concatenate([rng().standard_normal(n - 6), [0.0, -0.0, 1e-40, -3e37, 3e37, 1e30]]).astype(np.float32)
    return {"xs": x, **{name: np.array([c], np.float32) for name, c in DIVISORS.items()}}


def test_quotient_rewrite_is_in_the_report_only_when_optimizing():
    from emmy_ptx.lower import Lowerer
    n = 1024
    inputs = division_inputs(n)
    src = source("k_div", division_kernel(n), inputs, {"out": np.zeros((len(DIVISORS), n), np.float32)}, n // 256, 256, constants=DIVISORS)
    assert any("correctly rounded x / c" in r for r in Lowerer(src).run().remarks)
    for flags in ({"strict": True}, {"plain": True}):
        assert not any("correctly rounded" in r for r in Lowerer(src, **flags).run().remarks)


@pytest.mark.gpu
@pytest.mark.parametrize("mode", ["optimized", "strict", "plain"])
def test_division_by_a_named_constant_is_correctly_rounded(mode):
    """Optimized: the quotient numpy's x / c gives, bit for bit (a power-of-two divisor stays a multiply, which is exact).
    Strict and plain: the IR's own x * RN(1 / c)."""
    n = 4096
    inputs = division_inputs(n)
    out = {"out": np.zeros((len(DIVISORS), n), np.float32)}
    src = source("k_div", division_kernel(n), inputs, out, n // 256, 256, constants=DIVISORS)
    got = runner.run_source(src, {**inputs, **out}, mode)["out"]
    x = inputs["xs"]
    with np.errstate(all="ignore"):
        for k, c in enumerate(DIVISORS.values()):
            c32 = np.float32(c)
            want = x / c32 if mode == "optimized" else x * (np.float32(1) / c32)
            assert same_bits(got[k], want.astype(np.float32)), (c, mode)


@pytest.mark.gpu
@pytest.mark.parametrize("name", ["three_c", "div_c1"])
def test_the_divisor_is_recognised_by_its_name_only(name):
    x = rng().standard_normal(256).astype(np.float32)
    body = tile(256, [ld("v", "x", T), ld("c", name, num(0)), Assign(name="r", op="reciprocal", args=("c",), dtype=None),
                      Assign(name="y", op="multiply", args=("v", "r"), dtype=None), st("out", (T,), "y")])
    inputs, out = {"x": x, name: np.array([3], np.float32)}, {"out": np.zeros(256, np.float32)}
    got = runner.run_source(source("k_div", body, inputs, out, 1, 256, constants={name: 3.0}), {**inputs, **out}, "optimized")["out"]
    product, quotient = x * (np.float32(1) / np.float32(3)), x / np.float32(3)
    assert not np.array_equal(product, quotient)
    assert same_bits(got, quotient if name == "div_c1" else product)
