"""GPU parity of the pointwise (elementwise streaming) template: runs of four cells per access, the arithmetic of the
statement lowering. Every mode must give the oracle's values: bit for bit where the body is IEEE basic arithmetic
(the reference's rule for its pointwise family, tests/test_oracle.py:256-262), within the math routines' 2 ulp where
it calls tanh. All launches go through libemmyb200.so."""

import numpy as np
import pytest

from emmy_ptx import problems, runner
from emmy_ptx.ir import Assign, Axis, Let, Literal, Load, Tile, Var, Write, datatype
from helpers import margin, oracle_problem, same_bits, source
from oracle import ir_oracle

pytestmark = pytest.mark.gpu
MODES = ("optimized", "strict", "plain")


@pytest.mark.parametrize("mode", MODES)
@pytest.mark.parametrize("rows,cols,block", [(8, 1024, 256), (3, 4100, 100), (1, 256, 256), (257, 36, 36), (2048, 4096, 256)])
def test_bias_relu_residual_is_bit_exact(tmp_path, mode, rows, cols, block):
    """Whole CTAs, a ragged last CTA, one partly filled CTA, rows shorter than a CTA's cells, four runs per thread."""
    p = problems.bias_relu_residual(rows=rows, cols=cols, block=block, ident="t")
    prob = runner.Problem(problems.write(p, tmp_path), mode, canary=True)
    assert prob.kernels[0].launch_info["family"] == ("statements" if mode == "plain" else "pointwise")
    got = prob.run()["y"]
    prob.check_canaries()
    want = oracle_problem(p, prob.host)["y"]
    assert same_bits(got, want)
    x, b, r = prob.host["x"], prob.host["bias"], prob.host["res"]
    assert same_bits(got, np.maximum(x + b, np.float32(0)) + r)


@pytest.mark.parametrize("mode", MODES)
def test_bias_gelu_against_the_oracle(tmp_path, mode):
    p = problems.bias_gelu(rows=16, cols=2048, ident="t")
    prob = runner.Problem(problems.write(p, tmp_path), mode)
    got = prob.run()["y"]
    want = oracle_problem(p, prob.host)["y"]
    assert margin(got, want, 1e-5, 1e-6) <= 1
    z = (prob.host["x"] + prob.host["bias"]).astype(np.float64)
    exact = 0.5 * z * (1 + np.tanh(np.sqrt(2 / np.pi) * (z + 0.044715 * z ** 3)))
    assert margin(got, exact, 1e-5, 1e-6) <= 1


def test_bias_gelu_full_size_sampled_rows_and_streams(tmp_path):
    """The bench's workload: sampled rows against the oracle, the whole output against the f64 expression; the three
    lowerings of the template agree bit for bit on it (strict differs from optimized only by FMA contraction)."""
    from pathlib import Path
    folder = Path(runner.__file__).resolve().parent.parent / "problems" / "e_bias_gelu_8192x4096"
    prob = runner.Problem(folder, "strict")
    got = prob.run()["y"]
    p = problems.bias_gelu()
    rows = [0, 1, 4095, 8191]
    blocks = [b for r in rows for b in range(r * 16, r * 16 + 16)]  # 16 blocks of 256 threads per row in the IR's launch
    want = oracle_problem(p, prob.host, blocks=blocks)["y"]
    assert margin(got[rows], want[rows], 1e-5, 1e-6) <= 1
    z = (prob.host["x"] + prob.host["bias"]).astype(np.float64)
    exact = 0.5 * z * (1 + np.tanh(np.sqrt(2 / np.pi) * (z + 0.044715 * z ** 3)))
    assert margin(got, exact, 1e-5, 1e-6) <= 1


@pytest.mark.parametrize("mode", MODES)
def test_typed_arithmetic_with_broadcasts_and_wide_outputs(mode):
    """f32, i32 and u32 streams, a row-broadcast operand, a value indexed by an outer axis, f64 and i32 outputs at a
    literal leading index (the shape of the reference's pointwise family, tests/test_oracle.py:111-156): bit for bit."""
    f32, i32, u32, f64 = (datatype(n) for n in ("f32", "i32", "u32", "f64"))
    rows, cols = 5, 64
    rng = np.random.default_rng(11)
    xf = (rng.standard_normal((rows, cols)) * 10).astype(np.float32)
    xf[0, :6] = [0.0, -0.0, 3e30, -3e30, 1e-40, 16777217.0]
    xi = rng.integers(-2**31, 2**31, (rows, cols), dtype=np.int64).astype(np.int32)
    yi = rng.integers(1, 50, cols).astype(np.int32)
    xu = rng.integers(0, 2**32, (rows, cols), dtype=np.uint64).astype(np.uint32)
    sc = rng.standard_normal(rows).astype(np.float32)
    r, c = Var(name="r"), Var(name="c")
    lit = lambda v: Literal(value=v, dtype="int")  # noqa: E731
    stmts = (Load(names=("f0",), input="xf", index=(r, c), dtype=None), Load(names=("i0",), input="xi", index=(r, c), dtype=i32),
             Load(names=("i1",), input="yi", index=(c,), dtype=i32), Load(names=("u0",), input="xu", index=(r, c), dtype=u32),
             Load(names=("s0",), input="sc", index=(r,), dtype=None), Let(name="two", value=lit(2), dtype=None),
             Assign(name="a", op="multiply", args=("f0", "s0"), dtype=f32), Assign(name="b", op="maximum", args=("a", "f0"), dtype=f32),
             Assign(name="q", op="floor_divide", args=("i0", "i1"), dtype=i32), Assign(name="m", op="remainder", args=("i0", "i1"), dtype=i32),
             Assign(name="sh", op="right_shift", args=("u0", "two"), dtype=u32), Assign(name="rc", op="reciprocal", args=("b",), dtype=f32),
             Write(output="of", index=(lit(0), r, c), values=("a",)), Write(output="of", index=(lit(1), r, c), values=("b",)),
             Write(output="of", index=(lit(2), r, c), values=("rc",)), Write(output="of", index=(lit(3), r, c), values=("sh",)),
             Write(output="oi", index=(lit(0), r, c), values=("q",)), Write(output="oi", index=(lit(1), r, c), values=("m",)))
    body = (Tile(axes=(Axis(name="r", extent=rows), Axis(name="c", extent=cols)), body=stmts, block_threads=64, aux_threads=0,
                 raster_axes=None, raster_group=None, raster_orient="m"),)
    inputs = {"xf": xf, "xi": xi, "yi": yi, "xu": xu, "sc": sc}
    outs = {"of": np.zeros((4, rows, cols), np.float64), "oi": np.zeros((2, rows, cols), np.int32)}
    src = source("k_typed", body, inputs, outs, rows, 64)
    if mode != "plain":
        from emmy_ptx.lower import Lowerer
        assert Lowerer(src, strict=mode == "strict").run().family == "pointwise"
    got = runner.run_source(src, {**inputs, **{k: v.copy() for k, v in outs.items()}}, mode)
    want = {**{k: v.copy() for k, v in inputs.items()}, **{k: v.copy() for k, v in outs.items()}}
    ir_oracle.run(body, want, rows, 64)
    for k in outs:
        assert same_bits(got[k], want[k]), k
