"""Every family on small and ragged shapes with its output and intermediate buffers between poisoned guard zones:
nothing may be written outside a buffer, and nothing of a final output may be left unwritten (the buffers start as
NaN). The host-side stand-in for a memory checker."""

import numpy as np
import pytest

from emmy_ptx import fragproblems, problems, runner, tcfamilies

pytestmark = pytest.mark.gpu

CASES = {
    "sum": lambda: problems.array_sum(n=1 << 16, grid=24, block=256, ident="t"),
    "softmax": lambda: problems.row_softmax(rows=37, cols=1024, block=256, ident="t"),
    "matmul": lambda: problems.matmul_f16(m=200, n=264, k=72, block=64, ident="t"),
    "matmul-bf16": lambda: problems.matmul_f16(m=384, n=256, k=1024, block=256, dtype="bf16", ident="t"),
    "matmul-e4m3": lambda: problems.matmul_fp8(m=200, n=264, k=144, block=64, ident="t"),
    "attention": lambda: problems.attention(batch=1, heads=2, seq=320, dim=128, causal=True, ident="t"),
    "mlp": lambda: problems.gelu_mlp(tokens=192, d_model=256, hidden=512, ident="t"),
    "fragments": lambda: fragproblems.fragment_matmul(m=256, n=384, k=512, splits=2, b_layout="nk", ident="t"),
    "fragments-ragged": lambda: fragproblems.fragment_matmul(m=100, n=60, k=80, splits=2, staged=False, ident="t"),
}


@pytest.mark.parametrize("mode", ["optimized", "plain"])
@pytest.mark.parametrize("case", sorted(CASES))
def test_kernels_stay_inside_their_buffers_and_fill_them(tmp_path, case, mode):
    folder = problems.write(CASES[case](), tmp_path)
    want = runner.Problem(folder, mode).run()
    prob = runner.Problem(folder, mode, canary=True)
    for _ in range(2):
        got = prob.run()
        prob.check_canaries()
        for name, value in got.items():
            assert not np.isnan(np.asarray(value).astype(np.float32)).any(), f"{name}: elements left unwritten"
            assert value.tobytes() == want[name].tobytes(), f"{name}: differs from the run without guard zones"


def test_matmul_on_cta_pairs_stays_inside(tmp_path, monkeypatch):
    monkeypatch.setattr(tcfamilies, "GEMM_PAIR_MIN_TILES", 1)
    folder = problems.write(problems.matmul_f16(m=200, n=264, k=72, block=64, ident="t"), tmp_path)
    prob = runner.Problem(folder, "optimized", canary=True)
    assert prob.kernels[0].launch_info["cluster"] == 2
    got = prob.run()["matmul"]
    prob.check_canaries()
    assert not np.isnan(got.astype(np.float32)).any()
