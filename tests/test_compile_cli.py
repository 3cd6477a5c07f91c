"""The compile.py command line and compile_file modes (the contract of the reference's tests/test_compile.py)."""

import json
import re
import shutil
import subprocess
import sys
from pathlib import Path

import pytest

import emmy_ptx
from emmy_ptx import compile_file, lower, problems

ROOT = Path(__file__).resolve().parents[1]
PTXAS = shutil.which("ptxas") or "/usr/local/cuda/bin/ptxas"


@pytest.fixture(scope="module")
def folder(tmp_path_factory):
    root = tmp_path_factory.mktemp("problems")
    out = {}
    out["sum"] = problems.write(problems.array_sum(n=4096, grid=4, block=128, final_block=64, ident="sum"), root)
    out["softmax"] = problems.write(problems.row_softmax(rows=8, cols=512, block=64, ident="softmax"), root)
    out["matmul"] = problems.write(problems.matmul_f16(m=16, n=16, k=32, block=128, ident="matmul"), root)
    out["attention"] = problems.write(problems.attention(batch=1, heads=1, seq=16, dim=32, ident="attention"), root)
    out["mlp"] = problems.write(problems.gelu_mlp(tokens=4, d_model=16, hidden=32, lanes=8, block=64, ident="mlp"), root)
    return out


def cli(*args):
    return subprocess.run([sys.executable, str(ROOT / "compile.py"), *args], capture_output=True, text=True)


KERNELS = [("sum", "k_sum__partial"), ("sum", "k_sum_1_reduce"), ("softmax", "k_softmax_reduce"), ("matmul", "k_matmul"),
           ("attention", "k_attention"), ("mlp", "k_mlp_gelu")]


@pytest.mark.parametrize("flags", [(), ("--strict",), ("--plain",)], ids=["optimized", "strict", "plain"])
@pytest.mark.parametrize("problem,entry", KERNELS)
def test_kernel_compiles_to_well_formed_ptx(folder, tmp_path, problem, entry, flags):
    ir = folder[problem] / f"{entry}.ir.json"
    r = cli(*flags, str(ir))
    assert r.returncode == 0, r.stderr
    ptx = r.stdout
    kernel = next(k for k in json.loads((ir.parent / "meta.json").read_text())["kernels"] if k["entry"] == entry)
    assert ptx.lstrip().startswith("//") and "\n.version " in ptx and "\n.target sm_100a" in ptx
    assert ptx.isascii()
    params = re.search(rf"\.visible \.entry {re.escape(entry)}\(([^)]*)\)", ptx).group(1)
    assert re.findall(r"\.param \.u64 p_(\w+)", params) == kernel["arg_order"]
    assert re.search(r"\.maxntid \d+, 1, 1", ptx)
    out = tmp_path / "k.ptx"
    out.write_text(ptx)
    a = subprocess.run([PTXAS, "-arch=sm_100a", str(out), "-o", str(tmp_path / "k.cubin")], capture_output=True, text=True)
    assert a.returncode == 0, a.stderr


def test_usage_errors_give_rc_2_and_a_clean_stdout(folder):
    ir = str(folder["sum"] / "k_sum__partial.ir.json")
    for args in ((), (ir, ir), ("--fast", ir)):
        r = cli(*args)
        assert r.returncode == 2 and r.stdout == "" and r.stderr.startswith("usage:")


def test_a_failing_compilation_gives_rc_1_a_traceback_and_a_clean_stdout(tmp_path):
    bad = tmp_path / "k.ir.json"
    bad.write_text(json.dumps({"inputs": [], "outputs": [], "nodes": {}}))
    r = cli(str(bad))
    assert r.returncode == 1 and r.stdout == "" and "Traceback" in r.stderr and "expected exactly one KernelOp" in r.stderr


def test_templates_are_chosen_where_the_pattern_matches(folder, capsys):
    compile_file(str(folder["sum"] / "k_sum__partial.ir.json"), report=True)
    assert "block reduction template" in capsys.readouterr().err
    compile_file(str(folder["softmax"] / "k_softmax_reduce.ir.json"), report=True)
    assert "row softmax template" in capsys.readouterr().err
    compile_file(str(folder["softmax"] / "k_softmax_reduce.ir.json"), report=True, plain=True)
    err = capsys.readouterr().err
    assert "template" not in err and "lowered plainly" in err


def test_a_failing_rewrite_falls_back_to_the_plain_lowering(folder, monkeypatch, capsys):
    def unforeseen(*a):
        raise RuntimeError("an IR shape no rewrite foresaw")

    monkeypatch.setattr(lower.families, "match_reduce", unforeseen)
    ir = str(folder["sum"] / "k_sum__partial.ir.json")
    assert compile_file(ir).split("\n", 4)[4] == compile_file(ir, plain=True).split("\n", 4)[4]
    err = capsys.readouterr().err
    assert "RuntimeError: an IR shape no rewrite foresaw" in err and "without the optional rewrites" in err


def test_a_module_too_long_for_the_runner_falls_back(folder, monkeypatch, capsys):
    monkeypatch.setattr(emmy_ptx, "PTX_LIMIT", 100)
    ir = str(folder["sum"] / "k_sum__partial.ir.json")
    assert "lowered plainly" in compile_file(ir)
    assert "more than the runner accepts" in capsys.readouterr().err


@pytest.mark.parametrize("flags", [{}, {"strict": True}, {"plain": True}], ids=["optimized", "strict", "plain"])
def test_report_lists_the_decisions_and_changes_no_ptx(folder, flags, capsys):
    ir = str(folder["sum"] / "k_sum_1_reduce.ir.json")
    ptx = compile_file(ir, **flags)
    capsys.readouterr()
    assert compile_file(ir, report=True, **flags) == ptx
    err = capsys.readouterr().err
    assert err.startswith("k_sum_1_reduce: 1 block x 64 threads") and "\n  PTX: " in err and "instructions:" in err
    assert "launch hints: .maxntid" in err and ("lowered plainly" in err) == bool(flags.get("plain"))


def test_unknown_names_in_the_disable_list_are_refused(monkeypatch):
    monkeypatch.setenv("EMMY_PTX_DISABLE", "reduce,nonsense")
    with pytest.raises(ValueError, match="unknown rewrite"):
        lower.disabled_rewrites()
    monkeypatch.setenv("EMMY_PTX_DISABLE", "reduce,tree")
    assert lower.disabled_rewrites() == {"reduce", "tree"}


def test_meta_wins_over_the_ir_and_is_optional(folder, tmp_path, capsys):
    from emmy_ptx import frontend
    src = frontend.load(folder["sum"] / "k_sum__partial.ir.json")
    assert src.params == ("x", "sum__partial") and src.launch == frontend.Launch(4, 128, 0) and src.written == {"sum__partial"}
    lone = tmp_path / "k_sum__partial.ir.json"
    lone.write_text((folder["sum"] / "k_sum__partial.ir.json").read_text())
    src = frontend.load(lone)
    assert "deriving parameters and launch from the IR" in capsys.readouterr().err
    assert src.params == ("x", "sum__partial") and src.launch.block == 128 and src.launch.grid == 4


def test_one_wave_hint_and_cluster_request_are_in_the_module(tmp_path):
    """`.minnctapersm 1` iff the grid fits in one wave of the 148 SMs (reference emmy_ptx/lower.py:104-106, with its
    TARGET_SMS of another GPU), switched off by EMMY_PTX_DISABLE=hint; a kernel on CTA pairs asks for its cluster."""
    import os
    import subprocess
    import sys
    problems_dir = ROOT / "emmy-ptx-compiler_b200" / "problems"

    def compile_(ir, **env):
        r = subprocess.run([sys.executable, str(ROOT / "compile.py"), "--report", str(ir)], capture_output=True, text=True,
                           env={**os.environ, **env})
        assert r.returncode == 0, r.stderr
        return r.stdout, r.stderr

    ptx, report = compile_(problems_dir / "r_sum_16m" / "k_sum_1_reduce.ir.json")  # one block
    assert ".minnctapersm 1" in ptx and ".minnctapersm 1 (the grid fits in one wave)" in report
    ptx, report = compile_(problems_dir / "r_sum_16m" / "k_sum_1_reduce.ir.json", EMMY_PTX_DISABLE="hint")
    assert ".minnctapersm" not in ptx and "one wave" not in report
    ptx, report = compile_(problems_dir / "f_softmax_8192x4096" / "k_softmax_reduce.ir.json")  # 8192 blocks
    assert "one wave" not in report
    ptx, report = compile_(problems_dir / "m_f16_8192" / "k_matmul.ir.json")
    assert ".reqnctapercluster 2, 1, 1" in ptx and ".reqnctapercluster 2" in report


def test_the_reference_arm_of_the_bench_runs_on_the_host_alone(tmp_path):
    """`bench.py --impl reference` times the CPU interpreter (the oracle port) on a bounded sample and prints one JSON line
    with the contract's keys; it needs no GPU. The array sum keeps the sample small."""
    import json
    import subprocess
    import sys
    from pathlib import Path
    root = Path(__file__).resolve().parent.parent
    r = subprocess.run([sys.executable, str(root / "bench.py"), "--impl", "reference", "--workload", "sum", "--steps", "1"],
                       capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    line = json.loads(r.stdout.strip().splitlines()[-1])
    assert line["impl"] == "reference" and line["unit"] == "us" and line["higher_is_better"] is False and line["value"] > 0
    assert line["cpu_baseline"]["kind"] == "port" and line["cpu_baseline"]["cores"] >= 1 and "CTAs" in line["cpu_baseline"]["sample"]
    assert line["e2e"] == dict(value=line["value"], unit="us", h2d_bytes_per_step=0, d2h_bytes_per_step=0)
