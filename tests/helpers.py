"""Shared helpers of the tests: building a KernelSource in memory, running the oracle on a problem."""

from __future__ import annotations

import numpy as np

from emmy_ptx.frontend import Buffer, KernelSource, Launch

DTYPE_NAME = {np.dtype(np.float32): "f32", np.dtype(np.float64): "f64", np.dtype(np.float16): "f16",
              np.dtype(np.int32): "i32", np.dtype(np.uint32): "u32", np.dtype(np.int64): "i64", np.dtype(np.uint8): "u8"}


def dtype_name(a: np.ndarray) -> str:
    if a.dtype.name == "bfloat16":
        return "bf16"
    return DTYPE_NAME[a.dtype]


def source(name, body, inputs: dict, outputs: dict, grid: int, block: int, constants: dict | None = None) -> KernelSource:
    buffers = {n: Buffer(n, tuple(a.shape), dtype_name(a)) for n, a in {**inputs, **outputs}.items()}
    return KernelSource(name, tuple(body), tuple(inputs) + tuple(outputs), buffers, Launch(grid, block, 0),
                        frozenset(outputs), constants=dict(constants or {}))


def same_bits(got, want) -> bool:
    """NaN matches NaN, everything else bit for bit (tests/test_oracle.py:256-262 of the reference)."""
    got, want = np.ascontiguousarray(got), np.ascontiguousarray(want)
    if got.dtype != want.dtype or got.shape != want.shape:
        return False
    raw = {1: np.uint8, 2: np.uint16, 4: np.uint32, 8: np.uint64}[got.dtype.itemsize]
    eq = got.view(raw) == want.view(raw)
    if got.dtype.kind == "f":
        eq = eq | (np.isnan(got) & np.isnan(want))
    return bool(eq.all())


def margin(got, want, rtol: float, atol: float) -> float:
    """max |got - want| / (atol + rtol |want|): at most 1 passes (the reference's rule,
    tools/run_suite.py:97-104)."""
    got, want = np.asarray(got, np.float64), np.asarray(want, np.float64)
    return float(np.max(np.abs(got - want) / (atol + rtol * np.abs(want)))) if got.size else 0.0


def stated_margin(got, want, rtol: float, name: str | None = None) -> float:
    """The margin at a STATED tolerance, exactly as the reference's runner judges a problem
    (tools/run_suite.py:97-104: max |got - want| / (atol + rtol |want|)) with atol = rtol * RMS(want) over the whole
    compared set: nothing added for the output format's last place, no per-row scale. With ``name`` and the
    environment variable EMB_MARGIN_REPORT set, the value is appended to that file (one JSON object per line), which
    is how the table of measured margins is made."""
    import json
    import os
    want64 = np.asarray(want, np.float64)
    value = margin(got, want64, rtol, rtol * float(np.sqrt(np.mean(want64 ** 2))) if want64.size else 0.0)
    report = os.environ.get("EMB_MARGIN_REPORT")
    if name and report:
        with open(report, "a") as f:
            f.write(json.dumps(dict(case=name, rtol=rtol, margin=value, cells=int(want64.size))) + "\n")
    return value


def oracle_problem(problem: dict, host: dict, blocks=None) -> dict:
    """Run every kernel of an authored problem (emmy_ptx.problems) through the oracle."""
    from emmy_ptx import runner
    from oracle import ir_oracle
    bufs = {k: v.copy() for k, v in host.items()}
    for kern in problem["kernels"]:
        name, shape, dt = kern["output"]
        bufs[name] = np.zeros(shape, runner.numpy_dtype(dt))
        ir_oracle.run(kern["body"], bufs, kern["grid"], kern["block"], blocks=blocks)
    return bufs
