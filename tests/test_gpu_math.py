"""Accuracy of the single-precision exp, log and tanh routines (csrc/templates/emb_math.cuh) on the GPU.

The ranges and targets are the reference's (tools/mathtest.py:130-145: exp on [0,1] and [1,104], tanh on [0,0.6]
and [0.6,12], log on three ranges; README.md:206: exp and tanh within 2 ulp, log within 1 ulp, measured against the
correctly rounded result). Each function runs through the statement lowering as a one-Assign pointwise kernel.
"""

import numpy as np
import pytest

from emmy_ptx import runner
from emmy_ptx.ir import Assign, Axis, Load, Tile, Var, Write
from helpers import source

pytestmark = pytest.mark.gpu
N = 1 << 20


def ulps(got, x, fn):
    exact = fn(x.astype(np.float64))
    want = exact.astype(np.float32)
    spacing = np.spacing(np.abs(want)).astype(np.float64)
    return float(np.max(np.abs(got.astype(np.float64) - exact) / spacing))


def run(op, x):
    i = Var(name="i")
    body = (Tile(axes=(Axis(name="i", extent=x.size),), body=(
        Load(names=("v",), input="x", index=(i,)), Assign(name="r", op=op, args=("v",)),
        Write(output="out", index=(i,), values=("r",)))),)
    src = source("k_math", body, {"x": x}, {"out": np.zeros_like(x)}, x.size // 256, 256)
    return runner.run_source(src, {"x": x, "out": np.zeros_like(x)}, "strict")["out"]


@pytest.mark.parametrize("op,fn,lo,hi,limit", [
    ("exp", np.exp, 0.0, 1.0, 2.0), ("exp", np.exp, 1.0, 88.0, 2.0), ("exp", np.exp, -87.0, 0.0, 2.0),
    ("tanh", np.tanh, 0.0, 0.6, 2.0), ("tanh", np.tanh, 0.6, 12.0, 2.0), ("tanh", np.tanh, -12.0, -0.6, 2.0),
    ("log", np.log, 0.5, 2.0, 1.0), ("log", np.log, 1e-30, 1.0, 1.0), ("log", np.log, 1.0, 1e30, 1.0)])
def test_ulp_error(op, fn, lo, hi, limit):
    rng = np.random.default_rng(17)
    if op == "log" and hi / max(lo, 1e-38) > 1e6:
        x = np.exp(rng.uniform(np.log(lo), np.log(hi), N)).astype(np.float32)
    else:
        x = rng.uniform(lo, hi, N).astype(np.float32)
    err = ulps(run(op, x), x, fn)
    assert err <= limit, (op, lo, hi, err)


def test_special_values():
    x = np.array([0.0, -0.0, np.inf, -np.inf, np.nan, 1e-45, -104.0, 89.0] + [1.0] * 248, np.float32)
    e = run("exp", x)
    assert e[0] == 1 and e[1] == 1 and np.isinf(e[2]) and e[3] == 0 and np.isnan(e[4]) and e[5] == 1 and e[6] == 0 and np.isinf(e[7])
    t = run("tanh", x)
    assert t[0] == 0 and np.signbit(t[1]) and t[2] == 1 and t[3] == -1 and np.isnan(t[4])
    g = run("log", x)
    assert np.isneginf(g[0]) and np.isneginf(g[1]) and np.isinf(g[2]) and np.isnan(g[3]) and np.isnan(g[4])
    assert abs(g[5] - np.log(np.float64(np.float32(1e-45)))) < 1e-4
