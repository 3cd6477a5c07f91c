"""GPU parity of the GELU-MLP template (e4m3 weight decode, two tcgen05 matmuls, GELU in the first epilogue)."""

from pathlib import Path

import numpy as np
import pytest

from emmy_ptx import problems, runner
from helpers import oracle_problem

pytestmark = pytest.mark.gpu
RTOL = 3e-2  # the stated tolerance for per-tensor-scaled fp8 weights


def check(got, want, rtol=RTOL):
    want64, got64 = np.asarray(want, np.float64), np.asarray(got, np.float64)
    atol = rtol * np.sqrt(np.mean(want64 ** 2))
    m = float(np.max(np.abs(got64 - want64) / (atol + rtol * np.abs(want64))))
    assert m <= 1, m
    return m


def reference(host):
    """The float64 expression the problem's `code` names."""
    import ml_dtypes
    w1 = host["w1"].view(ml_dtypes.float8_e4m3fn).astype(np.float64) * float(host["w1_scale"][0])
    w2 = host["w2"].view(ml_dtypes.float8_e4m3fn).astype(np.float64) * float(host["w2_scale"][0])
    h = host["x"].astype(np.float64) @ w1
    g = 0.5 * h * (1 + np.tanh(problems.GELU_C * (h + problems.GELU_K * h ** 3)))
    return g @ w2


@pytest.mark.parametrize("tokens,d_model,hidden", [(128, 256, 256), (256, 512, 1024), (200, 264, 328)])
def test_mlp_small_against_the_oracle(tmp_path, tokens, d_model, hidden):
    block = 64
    p = problems.gelu_mlp(tokens=tokens, d_model=d_model, hidden=hidden, lanes=8, block=block, ident="t")
    prob = runner.Problem(problems.write(p, tmp_path), "optimized")
    assert prob.kernels[0].launch_info["family"] == "clusters" and len(prob.launches) == 4  # decode x 2, two matmuls
    got = prob.run()["mlp"]
    grid = p["kernels"][0]["grid"]
    blocks = sorted(set(np.random.default_rng(3).integers(0, grid, 48).tolist()) | {0, grid - 1})
    want = oracle_problem(p, prob.host, blocks=blocks)["mlp"].reshape(-1)
    cells = np.concatenate([np.arange(b * block // 8, (b + 1) * block // 8) for b in blocks])
    # bf16 output of sums of O(100) terms: well inside the fp8 tolerance; the measured margin is far below 1
    assert check(got.reshape(-1)[cells], want[cells]) < 0.5
    check(got, reference(prob.host))


@pytest.mark.parametrize("tokens,d_model,hidden", [(256, 512, 1024), (128, 128, 1024), (200, 1024, 2048), (384, 2048, 2048),
                                                   (128 * 19, 256, 2048)])
def test_mlp_fused_in_clusters_against_the_oracle(tmp_path, monkeypatch, tokens, d_model, hidden):
    """The cluster-fused template (hidden chunks exchanged through distributed shared memory): 64, 16, 128 and 256
    columns of y per CTA, one and two rounds of chunks, token rows past the end of the last tile, and more token
    tiles than clusters (a cluster then reuses its tensor memory and barriers for a second tile). Checked against
    the oracle on sampled CTAs, against the f64 expression everywhere, and against the two-matmul chain of the same
    problem; a second launch must find every barrier, the tensor memory and the peers as the first one did."""
    block = 64
    p = problems.gelu_mlp(tokens=tokens, d_model=d_model, hidden=hidden, lanes=8, block=block, ident="t")
    folder = problems.write(p, tmp_path)
    monkeypatch.setenv("EMMY_PTX_PREFER", "dsmem")  # (the chain is the default: it is the faster one on this GPU)
    prob = runner.Problem(folder, "optimized", canary=True)
    info = prob.kernels[0].launch_info
    assert info["family"] == "clusters" and info["cluster"] == 8 and len(prob.launches) == 3  # decode x 2, one fused kernel
    assert "ld.shared::cluster" in prob.kernels[0].ptx and "tcgen05.mma" in prob.kernels[0].ptx
    got = prob.run()["mlp"]
    prob.check_canaries()
    grid = p["kernels"][0]["grid"]
    blocks = sorted(set(np.random.default_rng(3).integers(0, grid, 12).tolist()) | {0, grid - 1})
    want = oracle_problem(p, prob.host, blocks=blocks)["mlp"].reshape(-1)
    cells = np.concatenate([np.arange(b * block // 8, (b + 1) * block // 8) for b in blocks])
    assert check(got.reshape(-1)[cells], want[cells]) < 0.5
    check(got, reference(prob.host))
    again = prob.run()["mlp"]
    assert np.array_equal(again.view(np.uint16), got.view(np.uint16))
    monkeypatch.delenv("EMMY_PTX_PREFER")
    chain = runner.Problem(folder, "optimized")
    assert len(chain.launches) == 4
    assert check(got, chain.run()["mlp"].astype(np.float64)) < 0.5


def test_mlp_statement_lowering_matches_too(tmp_path):
    p = problems.gelu_mlp(tokens=8, d_model=64, hidden=64, lanes=8, block=64, ident="t")
    prob = runner.Problem(problems.write(p, tmp_path), "strict")
    assert prob.kernels[0].launch_info["family"] == "statements"
    got = prob.run()["mlp"]
    want = oracle_problem(p, prob.host)["mlp"]
    check(got, want, rtol=2e-3 + 2.0 ** -8)


def test_mlp_full_size_sampled_cells_and_cross_check():
    import torch
    folder = Path(runner.__file__).resolve().parent.parent / "problems" / "k_mlp_gelu_tanh_16384x4096x16384"
    prob = runner.Problem(folder, "optimized")
    got = prob.run()["mlp"]
    p = problems.gelu_mlp()
    blocks = [123457]  # 256 threads = 32 output cells; every thread walks 2048 hidden units of 4096-long dot products
    want = oracle_problem(p, prob.host, blocks=blocks)["mlp"].reshape(-1)
    cells = np.arange(blocks[0] * 32, blocks[0] * 32 + 32)
    check(got.reshape(-1)[cells], want[cells])
    # the whole tensor against f32 matmuls on the same device (a cross-check, not the oracle)
    x = prob.tensors["x"].float()
    w1 = prob.tensors["w1"].view(torch.float8_e4m3fn).float() * prob.tensors["w1_scale"]
    w2 = prob.tensors["w2"].view(torch.float8_e4m3fn).float() * prob.tensors["w2_scale"]
    ref = (torch.nn.functional.gelu(x @ w1, approximate="tanh") @ w2).cpu().numpy()
    check(got, ref)


@pytest.mark.parametrize("d_model,hidden", [(256, 256), (200, 264)])
def test_weight_decode_of_every_code(tmp_path, d_model, hidden):
    """The MLP's weight decode kernels (e4m3 codes [k][n] -> bf16 [n][k]) on weights that hold every one of the 256 codes:
    the streaming 64 x 128 path (w1, shapes that divide), the 64 x 64 path beside the first matmul (w2) and on ragged
    shapes. Every e4m3 value is a bf16 value, so the decoded scratch buffers are compared bit for bit with the definition
    (ml_dtypes, as tests/test_fp8.py), NaN codes as NaN."""
    import ml_dtypes
    import torch
    p = problems.gelu_mlp(tokens=128, d_model=d_model, hidden=hidden, lanes=8, block=64, ident="t")
    folder = problems.write(p, tmp_path)
    host = dict(runner.Problem(folder, "optimized").host)
    rng = np.random.default_rng(1)
    for name in ("w1", "w2"):
        codes = np.resize(rng.permutation(np.repeat(np.arange(256, dtype=np.uint8), 4)), host[name].size)
        host[name] = codes.reshape(host[name].shape)
    prob = runner.Problem(folder, "optimized", inputs=host)
    prob.run()
    scratch = {k.split(".")[-1]: v for k, v in prob.tensors.items() if "." in k}
    for name, key in (("w1", "w1t"), ("w2", "w2t")):
        want = host[name].view(ml_dtypes.float8_e4m3fn).astype(np.float32).T
        got = scratch[key].view(torch.bfloat16).reshape(want.shape).float().cpu().numpy()
        nan = np.isnan(want)
        assert nan.sum() >= 8 and np.array_equal(np.isnan(got), nan)
        assert np.array_equal(got[~nan].view(np.uint32), want[~nan].view(np.uint32))  # (signed zeros included)
