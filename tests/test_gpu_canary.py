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


@pytest.mark.parametrize("workload,sizes", [("mlp", dict(tokens=512, d_model=256, hidden=512)), ("matmul", dict(m=512, n=256, k=128)),
                                             ("attention", dict(batch=2, heads=2, seq=256, dim=128))])
def test_a_problem_run_in_slices_gives_the_whole_problems_output(tmp_path, workload, sizes):
    """pipeline.ChunkedProblem: the units cut in four slices, each compiled for its size, copies and kernels on three
    streams, the resident operands uploaded once and their preparation (the MLP's weight decode) run once per call.
    Slices fall on tile boundaries, so the bits are the whole problem's."""
    import torch
    from emmy_ptx import multi, pipeline
    kw = multi.plan(workload, 0, 1, sizes)["kwargs"]
    whole_problem = problems.WORKLOADS[workload](ident="whole", **kw)
    prob = runner.Problem(problems.write(whole_problem, tmp_path), "optimized")
    out_name = whole_problem["kernels"][-1]["output"][0]
    whole = prob.run()[out_name]
    chunked = pipeline.ChunkedProblem(workload, dict(sizes), prob.host, "optimized", 0, chunks=4, streams=3, root=tmp_path / "slices")
    if workload == "mlp":
        assert len(chunked.prepare) == 2 and all(len(work) == 2 for _, _, work in chunked.parts)  # decode once, two matmuls per slice
    pinned = {n: prob.tensors[n].cpu().pin_memory() for n in chunked.plans[0]["slices"]}
    dev_out = prob.tensors[out_name]
    host_out = {out_name: torch.zeros(dev_out.shape, dtype=dev_out.dtype).pin_memory()}
    for _ in range(2):  # a second call reuses everything
        host_out[out_name].zero_()
        chunked.run(pinned, host_out)
        torch.cuda.synchronize()
        chunked.check_status()
        got = runner.to_numpy(host_out[out_name], prob.dtypes[out_name])
        assert np.array_equal(got.view(np.uint16), whole.view(np.uint16))


def test_the_full_size_mlp_in_the_benchs_slices_gives_the_whole_problems_output():
    """The headline workload the way bench.py's end-to-end leg runs it: pipeline.slice_count slices (eight) on four streams,
    matmuls on CTA pairs, the weight decode once per call; the bits are the whole problem's."""
    import torch
    from pathlib import Path
    from emmy_ptx import multi, pipeline
    folder = Path(runner.__file__).resolve().parent.parent / "problems" / "k_mlp_gelu_tanh_16384x4096x16384"
    prob = runner.Problem(folder, "optimized")
    whole = prob.run()["mlp"]
    units = multi.plan("mlp", 0, 1)["units"]
    chunked = pipeline.ChunkedProblem("mlp", dict(multi.FULL_SIZES["mlp"]), prob.host, "optimized", 0,
                                      chunks=pipeline.slice_count(units), streams=4)
    assert len(chunked.parts) == 8 and len(chunked.prepare) == 2
    pinned = {n: prob.tensors[n].cpu().pin_memory() for n in chunked.plans[0]["slices"]}
    host_out = {"mlp": torch.zeros(prob.tensors["mlp"].shape, dtype=prob.tensors["mlp"].dtype).pin_memory()}
    for _ in range(2):
        host_out["mlp"].zero_()
        chunked.run(pinned, host_out)
        torch.cuda.synchronize()
        chunked.check_status()
        got = runner.to_numpy(host_out["mlp"], prob.dtypes["mlp"])
        assert np.array_equal(got.view(np.uint16), whole.view(np.uint16))
