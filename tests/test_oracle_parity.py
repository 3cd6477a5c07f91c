"""oracle/ir_oracle.py against outputs of the reference's own interpreter (tests/golden/make_golden.py)."""

import json
from pathlib import Path

import numpy as np
import pytest

from emmy_ptx import ir
from oracle import ir_oracle

CASES = [c["name"] for c in json.loads((Path(__file__).parent / "golden" / "oracle_cases.json").read_text())]


def same_bits(got, want) -> bool:
    """NaN matches NaN; everything else bit for bit, the sign of a zero included
    (the reference's rule, tests/test_oracle.py:256-262)."""
    got, want = np.ascontiguousarray(got), np.ascontiguousarray(want)
    if got.dtype != want.dtype or got.shape != want.shape:
        return False
    raw = {2: np.uint16, 4: np.uint32, 8: np.uint64, 1: np.uint8}[got.dtype.itemsize]
    eq = got.view(raw) == want.view(raw)
    if got.dtype.kind == "f":
        eq |= np.isnan(got) & np.isnan(want)
    return bool(eq.all())


def run_case(case, arrays, **kw):
    name = case["name"]
    body = [ir.parse(s) for s in case["body"]]
    bufs = {k: arrays[f"{name}/in/{k}"].copy() for k in case["inputs"]}
    want = {k: arrays[f"{name}/out/{k}"] for k in case["outputs"]}
    bufs.update({k: np.zeros_like(v) for k, v in want.items()})
    ir_oracle.run(body, bufs, case["grid"], case["block"], blocks=case["blocks"], **kw)
    return bufs, want


@pytest.mark.parametrize("name", CASES)
def test_restated_interpreter_matches_the_reference_bit_for_bit(golden, name):
    case, arrays = golden[name]
    bufs, want = run_case(case, arrays)
    for k, w in want.items():
        assert same_bits(bufs[k], w), (name, k)


@pytest.mark.parametrize("name", [n for n in CASES if n.startswith(("ex_", "wl_", "rand_attention", "rand_shared"))])
def test_trip_by_trip_loops_give_the_same_as_the_vectorised_dot_products(golden, name, monkeypatch):
    """The reference's order, one trip after the other, against the all-trips-at-once evaluation."""
    monkeypatch.setattr(ir_oracle, "VECTOR_LOOPS", False)
    case, arrays = golden[name]
    bufs, want = run_case(case, arrays)
    for k, w in want.items():
        assert same_bits(bufs[k], w), (name, k)


@pytest.mark.parametrize("name", ["ex_a01_attention", "wl_sum_partial", "wl_softmax", "wl_attention"])
def test_block_at_a_time_order_gives_the_same(golden, name):
    case, arrays = golden[name]
    bufs, want = run_case(case, arrays, batch=1)
    for k, w in want.items():
        assert same_bits(bufs[k], w), (name, k)


def test_shipped_examples_meet_their_expected_answers(golden):
    """The reference's expected.npz (float64 numpy, rounded once) within each problem's own tolerance."""
    tol = {"ex_r01_array_sum": (1e-4, 1e-4), "ex_a01_attention": (1e-3, 1e-4), "ex_k_gelu_mlp": (1e-3, 1e-3)}
    for name, (rtol, atol) in tol.items():
        case, arrays = golden[name]
        bufs, _ = run_case(case, arrays)
        for k in case["expected"]:
            want = arrays[f"{name}/expected/{k}"]
            got = bufs[k].reshape(want.shape)
            if case["blocks"] is not None:  # only the cells of the sampled blocks were computed
                cells = np.concatenate([np.arange(b * case["block"], (b + 1) * case["block"]) for b in case["blocks"]])
                lanes = 8  # k_gelu_mlp: 8 lanes share one output cell
                cells = np.unique(cells // lanes)
                got, want = got.reshape(-1)[cells], want.reshape(-1)[cells]
            assert np.allclose(got, want, rtol=rtol, atol=atol), name


def test_tree_leaves_its_slab_and_broadcasts_the_root(golden):
    case, arrays = golden["self_tree_slab"]
    bufs, _ = run_case(case, arrays)
    assert np.array_equal(bufs["out"][0], np.full(128, 10, np.float32))
    assert np.array_equal(bufs["out"][1], np.tile(np.array([10, 6, 3, 4], np.float32), 32))


def test_bf16_and_e4m3_extension():
    """bf16 loads and the e4m3 decode, which the reference's table lacks: against ml_dtypes by hand."""
    import ml_dtypes
    from emmy_ptx import problems
    rng = np.random.default_rng(5)
    t, d, h, lanes = 4, 16, 32, 8
    p = problems.gelu_mlp(tokens=t, d_model=d, hidden=h, lanes=lanes, block=64)
    x = rng.standard_normal((t, d)).astype(ml_dtypes.bfloat16)
    c1 = rng.integers(0, 256, (d, h)).astype(np.uint8)
    c2 = rng.integers(0, 256, (h, d)).astype(np.uint8)
    c1[c1 & 0x7F == 0x7F] = 0x3A  # keep NaN codes out of the product
    c2[c2 & 0x7F == 0x7F] = 0x3A
    bufs = {"x": x, "w1": c1, "w2": c2, "w1_scale": np.array([2.0 ** -9], np.float32),
            "w2_scale": np.array([2.0 ** -8], np.float32), "gelu_half": np.array([0.5], np.float32),
            "gelu_c": np.array([problems.GELU_C], np.float32), "gelu_k": np.array([problems.GELU_K], np.float32),
            "gelu_one": np.array([1.0], np.float32), "mlp": np.zeros((t, d), ml_dtypes.bfloat16)}
    k = p["kernels"][0]
    ir_oracle.run(k["body"], bufs, k["grid"], k["block"])
    w1 = c1.view(ml_dtypes.float8_e4m3fn).astype(np.float64) * 2.0 ** -9
    w2 = c2.view(ml_dtypes.float8_e4m3fn).astype(np.float64) * 2.0 ** -8
    hp = x.astype(np.float64) @ w1
    g = 0.5 * hp * (1 + np.tanh(problems.GELU_C * (hp + problems.GELU_K * hp ** 3)))
    want = g @ w2
    got = bufs["mlp"].astype(np.float64)
    assert np.allclose(got, want, rtol=2e-2, atol=2e-2 * np.sqrt(np.mean(want ** 2)))
    assert np.array_equal(ir_oracle.apply("from_f8e4m3", [np.array([0x7E, 0x01, 0x80, 0xC0], np.uint8)], "f32"),
                          np.array([448.0, 2.0 ** -9, -0.0, -2.0], np.float32))
