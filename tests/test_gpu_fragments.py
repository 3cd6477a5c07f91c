"""GPU parity of the tensor-core (fragment) form: the statement path (cp.async, ldmatrix, mma.sync as the schedule
says) and the tcgen05 template the proved schedules go to, against the oracle's fragment extension and the
reference's expected values."""

import json

import numpy as np
import pytest

from emmy_ptx import fragproblems, problems, runner
from helpers import margin, source
from oracle import fragment_oracle
from test_fragments import CASES, GOLDEN, masked_bias_tail, one_warp_tile, run_chain, tile_inputs

pytestmark = pytest.mark.gpu
RTOL = 2e-3 + 2.0 ** -10  # the stated f16 tolerance plus one unit in the last place (both sides round an f32 sum once)


def close(got, want):
    want = np.asarray(want, np.float64)
    return margin(got, want, RTOL, RTOL * float(np.sqrt(np.mean(want ** 2)))) <= 1


@pytest.mark.parametrize("mode", ["optimized", "plain", "strict"])
def test_the_shipped_example(mode):
    """examples/m_f16_128 of the reference (two kernels: split-K partials, then their fold): expected.npz at the
    example's rtol = atol = 1e-2, and the oracle's run of the same schedule."""
    prob = runner.Problem(GOLDEN, mode)
    family = prob.kernels[0].launch_info["family"]
    assert family == ("tensorcore" if mode == "optimized" else "statements")
    assert ("tcgen05.mma" if mode == "optimized" else "mma.sync") in prob.kernels[0].ptx
    meta = json.loads((GOLDEN / "meta.json").read_text())
    want = np.load(GOLDEN / "expected.npz")["matmul"]
    oracle = run_chain(GOLDEN)
    for _ in range(2):
        out = prob.run()
        assert margin(out["matmul"], want, meta["rtol"], meta["atol"]) <= 1
        assert close(out["matmul"], oracle["matmul"])
        assert close(out["matmul__partial"], oracle["matmul__partial"])


@pytest.mark.parametrize("mode", ["optimized", "plain"])
@pytest.mark.parametrize("case", CASES + [dict(m=512, n=768, k=1024, splits=2), dict(m=384, n=512, k=512, splits=1, b_layout="nk", dtype="bf16")],
                         ids=lambda c: "-".join(f"{k}{v}" for k, v in c.items()) or "example-sized")
def test_authored_schedules(tmp_path, case, mode):
    """Staged and unstaged schedules, both B layouts, f16 and bf16, ragged edges through the clamps and guards: the
    proved ones on the tcgen05 template (optimized), all of them statement by statement (plain)."""
    p = fragproblems.fragment_matmul(**case)
    prob = runner.Problem(problems.write(p, tmp_path), mode)
    got = prob.run()
    a, b = prob.host["x0"].astype(np.float64), prob.host["x1"].astype(np.float64)
    want = a @ (b if case.get("b_layout", "kn") == "kn" else b.T)
    k_slab = case.get("k", 128) // case.get("splits", 2)
    provable = case.get("staged", True) or not case.get("guarded", True)
    big_enough = case.get("m", 128) * case.get("n", 128) >= 8192
    if mode == "optimized" and provable and big_enough and (case.get("splits", 2) == 1 or k_slab % 64 == 0):
        assert prob.kernels[0].launch_info["family"] == "tensorcore"
    if mode == "plain":
        assert prob.kernels[0].launch_info["family"] == "statements"
    assert close(got["matmul"], want)
    if case.get("m", 128) * case.get("n", 128) <= 1 << 17:
        assert close(got["matmul__partial"], run_chain(p, prob.host)["matmul__partial"])


def test_one_warp_tile_with_coordinate_mask_bias_and_f16_accumulator():
    a, bt, prod, bias = tile_inputs()
    inputs, out = {"a": a, "bt": bt, "bias": bias}, {"out": np.zeros((16, 8), np.float32)}
    body = one_warp_tile("f16", masked_bias_tail())
    got = runner.run_source(source("k_tile", body, inputs, out, 1, 32), {**inputs, **out}, "optimized")["out"]
    want = {**inputs, "out": np.zeros((16, 8), np.float32)}
    fragment_oracle.run(body, want, 1, 32)
    assert np.allclose(got, want["out"], rtol=2e-3, atol=2e-3)
    rows, cols = np.indices((16, 8))
    assert np.allclose(got, np.where(cols > rows, -1.0, prod.astype(np.float16)) + bias, rtol=2e-3, atol=2e-3)


def test_one_warp_tile_added_atomically_twice():
    from emmy_ptx.ir import RegStore
    L = problems.I
    a, bt, prod, _ = tile_inputs()
    tail = tuple(RegStore(dst_buffer="out", dst_index=(L(0), L(0)), frag="acc", shape=(16, 8, 16), atomic=True) for _ in range(2))
    inputs, out = {"a": a, "bt": bt}, {"out": np.zeros((16, 8), np.float16)}
    got = runner.run_source(source("k_tile", one_warp_tile("f32", tail), inputs, out, 1, 32), {**inputs, **out}, "plain")["out"]
    assert np.allclose(got.astype(np.float64), 2 * prod, rtol=5e-3, atol=5e-3)


@pytest.mark.parametrize("mode", ["optimized", "strict"])
def test_attention_tile_in_fragments(mode):
    """Row reductions across the four lanes of a row, per-row operands, exp, the repack of two accumulators into an A
    operand: against the oracle's run of the same statements and the f64 softmax(Q K^T) V."""
    from test_fragments import attention_inputs, attention_tile
    q, k, v, want = attention_inputs()
    inputs, out = {"q": q, "k": k, "v": v}, {"out": np.zeros((16, 8), np.float32)}
    got = runner.run_source(source("k_tile", attention_tile(), inputs, out, 1, 32), {**inputs, **out}, mode)["out"]
    ref = {**inputs, "out": np.zeros((16, 8), np.float32)}
    fragment_oracle.run(attention_tile(), ref, 1, 32)
    assert np.allclose(got, ref["out"], rtol=1e-3, atol=1e-3)
    assert np.allclose(got, want, rtol=2e-3, atol=2e-3)


def test_zero_prologue_clears_another_kernels_accumulator():
    from test_fragments import zero_prologue_kernel
    arrays = {"acc": np.full(40, 7.0, np.float32), "tally": np.zeros(8, np.float32)}
    src = source("k_zero", zero_prologue_kernel(33), {}, arrays, 1, 64)
    got = runner.run_source(src, arrays, "optimized")
    assert (got["acc"][:33] == 0).all() and (got["acc"][33:] == 7.0).all() and (got["tally"] == 8).all()


def test_regstore_epilogue_and_guards():
    from test_fragments import epilogue_expected, epilogue_tile
    a, bt, prod, _ = tile_inputs()
    inputs, out = {"a": a, "bt": bt}, {"out": np.full((16, 8), -7.0, np.float32)}
    got = runner.run_source(source("k_tile", epilogue_tile(), inputs, out, 1, 32), {**inputs, **out}, "optimized")["out"]
    assert np.allclose(got, epilogue_expected(prod), rtol=1e-3, atol=1e-3)


def test_b_read_transposed_from_a_k_by_n_slab():
    from test_fragments import kn_inputs, kn_tile
    a, b, want = kn_inputs()
    inputs, out = {"a": a, "b": b}, {"out": np.zeros((16, 8), np.float32)}
    got = runner.run_source(source("k_tile", kn_tile(), inputs, out, 1, 32), {**inputs, **out}, "plain")["out"]
    assert np.allclose(got, want, rtol=1e-5, atol=1e-5)
