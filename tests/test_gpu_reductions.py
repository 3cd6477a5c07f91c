"""GPU parity of the reduction family (array sum, row softmax) and of the statement lowering.

Everything goes through compile_file / Lowerer -> ptxas -> libemmyb200.so (the C ABI); the
expected values come from the oracle (oracle/ir_oracle.py) or from the golden outputs of the
reference's own interpreter (tests/golden).
"""

import json
from pathlib import Path

import numpy as np
import pytest

from emmy_ptx import ir, problems, runner
from helpers import margin, oracle_problem, same_bits, source

pytestmark = pytest.mark.gpu
MODES = ("optimized", "strict", "plain")
GOLDEN = [c for c in json.loads((Path(__file__).parent / "golden" / "oracle_cases.json").read_text())
          if c["name"].startswith(("rand_cooperative", "rand_shared_reduction", "rand_attention", "rand_pointwise", "self_",
                                   "wl_", "ex_r01", "ex_a01"))]


@pytest.mark.parametrize("mode", MODES)
@pytest.mark.parametrize("n,grid,block,final_block", [(4096 * 3, 5, 128, 64), (1 << 20, 148, 256, 256), (1 << 16, 1, 32, 32),
                                                        (100_000, 7, 64, 32)])
def test_array_sum_small(tmp_path, mode, n, grid, block, final_block):
    p = problems.array_sum(n=n, grid=grid, block=block, final_block=final_block, ident="t")
    prob = runner.Problem(problems.write(p, tmp_path), mode)
    got = prob.run()
    want = oracle_problem(p, prob.host)
    if mode == "strict":  # the IR's own order of operations: bit for bit
        assert same_bits(prob.outputs()["sum__partial"], want["sum__partial"])
        assert same_bits(got["sum_1"].reshape(()), want["sum_1"])
    else:
        assert margin(got["sum_1"].reshape(()), want["sum_1"], 1e-5, 1e-5 * np.sqrt(n)) <= 1


@pytest.mark.parametrize("mode", MODES)
@pytest.mark.parametrize("rows,cols,block", [(6, 1024, 64), (33, 4096, 256), (5, 512, 128), (3, 96, 32)])
def test_row_softmax_small(tmp_path, mode, rows, cols, block):
    p = problems.row_softmax(rows=rows, cols=cols, block=block, ident="t")
    prob = runner.Problem(problems.write(p, tmp_path), mode)
    got = prob.run()["softmax"]
    want = oracle_problem(p, prob.host)["softmax"]
    assert margin(got, want, 1e-5, 1e-9) <= 1  # exp within its 2 ulp, then sums
    assert np.allclose(got.sum(axis=1), 1.0, atol=1e-5)


@pytest.mark.parametrize("mode", MODES)
def test_row_softmax_extreme_values(tmp_path, mode):
    p = problems.row_softmax(rows=4, cols=1024, block=64, ident="t")
    folder = problems.write(p, tmp_path)
    x = np.random.default_rng(3).standard_normal((4, 1024)).astype(np.float32)
    x[0] *= 50          # one dominant element
    x[1] = -1e4         # all equal, far below zero
    x[2, 5] = 88.0      # exponent range
    x[3] = 0.0
    prob = runner.Problem(folder, mode, inputs={"x": x})
    got = prob.run()["softmax"]
    want = oracle_problem(p, {"x": x})["softmax"]
    assert margin(got, want, 1e-5, 1e-9) <= 1


def test_array_sum_full_size_strict_is_bit_exact():
    folder = Path(runner.__file__).resolve().parent.parent / "problems" / "r_sum_16m"
    prob = runner.Problem(folder, "strict")
    got = prob.run()
    p = problems.array_sum()
    want = oracle_problem(p, prob.host)
    assert same_bits(prob.outputs()["sum__partial"], want["sum__partial"])
    assert same_bits(got["sum_1"].reshape(()), want["sum_1"])
    exact = float(np.sum(prob.host["x"].astype(np.float64)))
    fast = runner.Problem(folder, "optimized").run()["sum_1"]
    assert abs(float(fast.reshape(-1)[0]) - exact) <= 1e-5 * np.sqrt(1 << 24)
    # linearity: the sum of 2x is twice the sum, exactly (a power of two scales every partial)
    twice = runner.Problem(folder, "strict", inputs={"x": prob.host["x"] * np.float32(2)}).run()["sum_1"]
    assert same_bits(twice, got["sum_1"] * np.float32(2))


def test_row_softmax_full_size_sampled_rows_and_properties():
    folder = Path(runner.__file__).resolve().parent.parent / "problems" / "f_softmax_8192x4096"
    prob = runner.Problem(folder, "optimized")
    got = prob.run()["softmax"]
    rows = [0, 1, 777, 4095, 4096, 8191]
    p = problems.row_softmax()
    want = oracle_problem(p, prob.host, blocks=rows)["softmax"]
    assert margin(got[rows], want[rows], 1e-5, 1e-9) <= 1
    assert np.allclose(got.sum(axis=1, dtype=np.float64), 1.0, atol=1e-5)
    x = prob.host["x"]
    assert np.array_equal(got.argmax(axis=1), x.argmax(axis=1))
    # shift invariance: softmax(x + c) == softmax(x) up to the rounding of x + c
    whole = np.exp(x.astype(np.float64) - x.max(axis=1, keepdims=True))
    whole /= whole.sum(axis=1, keepdims=True)
    assert margin(got, whole, 1e-5, 1e-9) <= 1


@pytest.mark.parametrize("mode", MODES)
@pytest.mark.parametrize("case", GOLDEN, ids=lambda c: c["name"])
def test_golden_kernels_of_the_reference_interpreter(golden, case, mode):
    """The reference's random kernel families and examples, lowered in every mode, against the
    outputs its own interpreter gave (strict: sums bit for bit; others within rounding,
    tests/test_oracle.py:256-280 of the reference)."""
    name = case["name"]
    _, arrays = golden[name]
    body = [ir.parse(s) for s in case["body"]]
    inputs = {k: arrays[f"{name}/in/{k}"] for k in case["inputs"]}
    want = {k: arrays[f"{name}/out/{k}"] for k in case["outputs"]}
    src = source("k_case", body, inputs, {k: np.zeros_like(v) for k, v in want.items()}, case["grid"], case["block"])
    got = runner.run_source(src, {**inputs, **{k: np.zeros_like(v) for k, v in want.items()}}, mode)
    uses_exp = "'exp'" in "".join(case["body"]) or "'erf'" in "".join(case["body"])
    exact_family = name.startswith(("rand_pointwise", "self_integers"))  # typed arithmetic: every lowering must match exactly
    for k, w in want.items():
        if (mode == "strict" or exact_family) and not uses_exp:
            assert same_bits(got[k], w), (name, k)
        else:
            tol = 1e-4 if uses_exp else 1e-5
            g, w64 = got[k].astype(np.float64), w.astype(np.float64)
            if w.dtype == np.float16:
                tol = 2e-3
            assert np.allclose(g, w64, rtol=tol, atol=tol / 10 * max(1.0, float(np.abs(w64).max()))), (name, k)


def test_rows_pipeline_gives_the_same_softmax(tmp_path):
    """Slices of rows copied in, computed and copied out on several streams: the same bits as one launch."""
    import torch
    p = problems.row_softmax(rows=96, cols=1024, block=64, ident="t")
    prob = runner.Problem(problems.write(p, tmp_path), "optimized")
    whole = prob.run()["softmax"]
    run = prob.rows_pipeline(chunks=5, streams=3)
    assert run is not None
    x = torch.from_numpy(prob.host["x"]).pin_memory()
    out = torch.zeros(96, 1024).pin_memory()
    prob.tensors["softmax"].zero_()
    run({"x": x}, {"softmax": out})
    torch.cuda.synchronize()
    assert same_bits(out.numpy(), whole)
    assert runner.Problem(problems.write(problems.array_sum(n=4096, grid=4, block=128, final_block=64, ident="s"), tmp_path),
                          "optimized").rows_pipeline() is None


@pytest.mark.parametrize("mode", MODES)
@pytest.mark.parametrize("n,grid,block,copies", [(1 << 18, 512, 128, 2), (1 << 16, 4, 256, 1), (1 << 20, 1024, 256, 4), (4096, 1, 128, 1)])
def test_array_sum_in_the_scalar_spelling(tmp_path, mode, n, grid, block, copies):
    """emmy's own form of the cooperative sum (scalar strided loads, unrolled copies): regrouped into 16-byte chunks in
    the optimizing mode (tolerance of a reassociated sum), the IR's order bit for bit under --strict and --plain."""
    p = problems.array_sum_scalar(n=n, grid=grid, block=block, copies=copies, ident="t")
    prob = runner.Problem(problems.write(p, tmp_path), mode)
    if mode != "plain":
        assert all(k.launch_info["family"] == "reduce" for k in prob.kernels[1:])
        assert prob.kernels[0].launch_info["family"] == ("reduce" if mode == "optimized" or copies == 1 else "statements")
    got = prob.run()
    want = oracle_problem(p, prob.host)
    if mode == "optimized":
        assert margin(got["sum_1"].reshape(()), want["sum_1"], 1e-5, 1e-5 * np.sqrt(n)) <= 1
        exact = float(np.sum(prob.host["x"].astype(np.float64)))
        assert abs(float(got["sum_1"].reshape(-1)[0]) - exact) <= 1e-5 * np.sqrt(n)
    else:
        assert same_bits(prob.outputs()["sum__partial"], want["sum__partial"])
        assert same_bits(got["sum_1"].reshape(()), want["sum_1"])


@pytest.mark.parametrize("mode", MODES)
def test_a_regrouped_fold_keeps_its_arithmetic(mode):
    """Sum of squares times a block-uniform weight, in the scalar spelling: the body's arithmetic travels with the
    element to its new thread. Integer-valued inputs make every order of additions exact."""
    from emmy_ptx.ir import Accum, Assign, Axis, BinaryExpr, Cond, Let, Literal, Load, StridedLoop, Tile, Var, Write, datatype
    f32 = datatype("f32")
    rows, cols, block = 6, 2048, 128
    x = np.random.default_rng(5).integers(-8, 9, (rows, cols)).astype(np.float32)
    w = np.arange(1, rows + 1, dtype=np.float32)
    loop = StridedLoop(axis=Axis(name="a", extent=cols), start=Var(name="t"), step=Literal(value=block, dtype="int"), body=(
        Load(names=("v",), input="x", index=(Var(name="r"), Var(name="a")), dtype=None),
        Assign(name="sq", op="multiply", args=("v", "v"), dtype=f32),
        Assign(name="ws", op="multiply", args=("sq", "wr"), dtype=f32),
        Accum(name="s", value="ws", op="add", dtype=f32, axes=(), base=None)), unroll=False, end=None, seed=True)
    body = (Tile(axes=(Axis(name="r", extent=rows), Axis(name="t", extent=block)), body=(
        Load(names=("wr",), input="w", index=(Var(name="r"),), dtype=None), loop, *problems._block_combine("s", "add", block),
        Cond(cond=BinaryExpr(op="==", left=Var(name="t"), right=Literal(value=0, dtype="int")),
             body=(Write(output="out", index=(Var(name="r"),), values=("s",), value_dtype=f32),), else_body=())),
        block_threads=block, aux_threads=0, raster_axes=None, raster_group=None, raster_orient="m"),)
    src = source("k_wsq", body, {"x": x, "w": w}, {"out": np.zeros(rows, np.float32)}, rows, block)
    got = runner.run_source(src, {"x": x, "w": w, "out": np.zeros(rows, np.float32)}, mode)["out"]
    assert same_bits(got, ((x.astype(np.float64) ** 2).sum(axis=1) * w).astype(np.float32))
    if mode == "optimized":
        from emmy_ptx.lower import Lowerer
        assert any("contiguous 16-byte chunks" in r for r in Lowerer(src).run().remarks)
