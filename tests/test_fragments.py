"""The tensor-core (fragment) form on the CPU: the oracle's extension against the reference's shipped example,
the three lowering modes through the CLI, and what the matmul proof accepts and refuses."""

import json
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest

from emmy_ptx import families, fragmatch, fragproblems, frontend, ir, problems, runner
from helpers import margin
from oracle import fragment_oracle

GOLDEN = Path(__file__).resolve().parent / "golden" / "m_f16_128"
ROOT = Path(__file__).resolve().parent.parent


def run_chain(problem_or_folder, host=None):
    """Every kernel of a chain through the fragment oracle; (buffers, meta)."""
    if isinstance(problem_or_folder, dict):
        p = problem_or_folder
        bufs = {k: v.copy() for k, v in host.items()}
        for kern in p["kernels"]:
            name, shape, dt = kern["output"]
            bufs[name] = np.zeros(shape, runner.numpy_dtype(dt))
            fragment_oracle.run(kern["body"], bufs, kern["grid"], kern["block"])
        return bufs
    meta = json.loads((problem_or_folder / "meta.json").read_text())
    bufs = runner.host_inputs([a for k in meta["kernels"] for a in k["args"]])
    for k in meta["kernels"]:
        for a in k["args"]:
            bufs.setdefault(a["name"], np.zeros(a["shape"], runner.numpy_dtype(a["dtype"])))
        fragment_oracle.run(frontend.load(problem_or_folder / f"{k['entry']}.ir.json").body, bufs, k["grid"][0], k["block"][0])
    return bufs


def test_the_shipped_example_meets_its_expected_values():
    """examples/m_f16_128 of the reference: expected.npz at the example's own rtol = atol = 1e-2, and the f64
    product of the same seeded inputs to half a unit in the last place of f16."""
    meta = json.loads((GOLDEN / "meta.json").read_text())
    bufs = run_chain(GOLDEN)
    want = np.load(GOLDEN / "expected.npz")["matmul"]
    assert margin(bufs["matmul"], want, meta["rtol"], meta["atol"]) <= 1
    exact = (bufs["x0"].astype(np.float64) @ bufs["x1"].astype(np.float64)).astype(np.float16)
    assert np.mean(bufs["matmul"] == exact) > 0.99  # all but results that sit on a rounding boundary


def test_the_example_reads_back_as_it_was_written():
    graph = json.loads((GOLDEN / "k_matmul__partial.ir.json").read_text())
    body = next(n for n in graph["nodes"].values() if n["op"] == "KernelOp")["op_fields"]["body"]
    assert [repr(ir.parse(s)) for s in body] == body


@pytest.mark.parametrize("mode,has,family", [((), "tcgen05.mma", "tensorcore"), (("--plain",), "mma.sync", "statements"),
                                             (("--strict",), "mma.sync", "statements")])
def test_cli_lowers_the_example_in_every_mode(mode, has, family):
    r = subprocess.run([sys.executable, str(ROOT / "compile.py"), "--report", *mode, str(GOLDEN / "k_matmul__partial.ir.json")],
                       capture_output=True, text=True)
    assert r.returncode == 0, r.stderr
    assert has in r.stdout and f'"family":"{family}"' in r.stdout
    assert ".param .u64 p_x1" in r.stdout and "launch hints: .maxntid" in r.stderr
    if family == "statements":
        assert "ldmatrix" in r.stdout and "cp.async.cg" in r.stdout and "tcgen05" not in r.stdout
    else:
        assert "proved to be matmul__partial = x0 [128 x 128] times x1 [K x N, N = 128] in 2 K-slabs of 64" in r.stderr


CASES = [dict(), dict(m=256, n=384, k=512, splits=2, b_layout="nk"), dict(m=64, n=96, k=128, splits=1, dtype="bf16"),
         dict(m=128, n=128, k=96, splits=3), dict(m=40, n=60, k=72, splits=1, staged=False),
         dict(m=100, n=60, k=80, splits=2, staged=False, b_layout="nk"),
         dict(m=128, n=256, k=256, splits=2, staged=False, guarded=False, b_layout="nk", dtype="bf16")]


@pytest.mark.parametrize("case", CASES, ids=lambda c: "-".join(f"{k}{v}" for k, v in c.items()) or "example-sized")
def test_authored_schedules_compute_the_product(case, tmp_path):
    """The generator's schedules (staged through swizzled shared memory, or read from global memory with clamps and
    zero fill) through the oracle against the f64 product: f32 accumulation, one rounding to f16."""
    p = fragproblems.fragment_matmul(**case)
    meta = json.loads((problems.write(p, tmp_path) / "meta.json").read_text())
    host = runner.host_inputs([a for k in meta["kernels"] for a in k["args"]])
    bufs = run_chain(p, host)
    a, b = bufs["x0"].astype(np.float64), bufs["x1"].astype(np.float64)
    want = a @ (b if case.get("b_layout", "kn") == "kn" else b.T)
    rtol = 2e-3
    assert margin(bufs["matmul"], want, rtol, rtol * float(np.sqrt(np.mean(want ** 2)))) <= 1


def partial_source(tmp_path, **case):
    folder = problems.write(fragproblems.fragment_matmul(**case), tmp_path)
    return frontend.load(folder / "k_matmul__partial.ir.json")


def test_the_proof_takes_schedules_in_both_layouts_and_without_staging(tmp_path):
    for case, text in [(dict(m=256, n=384, k=512, splits=2, b_layout="nk"), "x1 [N x K, N = 384] in 2 K-slabs of 256"),
                       (dict(m=128, n=256, k=128, splits=1, staged=False, guarded=False), "x1 [K x N, N = 256]")]:
        plan = fragmatch.match_fragment_matmul(partial_source(tmp_path, **case), False)
        assert plan.family == "tensorcore" and text in plan.remarks[0]
        assert "gemm_tn_kernel" in plan.source


def rewrite(src, change):
    """``src`` with ``change(statement) -> statement or None`` applied to every statement of the Tile."""
    def walk(stmts):
        out = []
        for s in stmts:
            new = change(s)
            s = s if new is None else new
            for field in ("body", "else_body"):
                if isinstance(getattr(s, field, None), tuple):
                    s = s.replace(**{field: walk(getattr(s, field))})
            out.append(s)
        return tuple(out)
    return frontend.KernelSource(src.name, walk(src.body), src.params, src.buffers, src.launch, src.written, src.constants,
                                 src.meta, src.path)


def refusal(src, strict=False) -> str:
    with pytest.raises(families.Refusal) as e:
        fragmatch.match_fragment_matmul(src, strict)
    return str(e.value)


def test_the_proof_refuses_what_is_not_the_product(tmp_path):
    src = partial_source(tmp_path)
    P, L = problems.B, problems.I
    assert "sum a K-slice in their own order" in refusal(src, strict=True)

    # the two stored fragments swapped: each lands on the other's columns
    def swap(s):
        if ir.kind(s) == "RegStore":
            return s.replace(frag="_c0_[1]" if s.frag == "_c0_[0]" else "_c0_[0]")
    assert "stored somewhere other than C[row of A, column of B]" in refusal(rewrite(src, swap))

    # B's fills shifted by one K-step against A's
    def shift(s):
        if ir.kind(s) == "CpAsyncCopy" and s.src == "x1":
            return s.replace(src_index=(P("+", s.src_index[0], L(32)), s.src_index[1]))
    assert "a B operand whose k does not run with A's" in refusal(rewrite(src, shift))

    # only the first half of every slab is summed
    def halve(s):
        if ir.kind(s) == "StridedLoop" and s.axis.name == "_ks":
            return s.replace(end=L(32))
    assert "does not sum each k of its slab exactly once" in refusal(rewrite(src, halve))

    # the slab index moves the output but not the operands' k
    def pin(s):
        if ir.kind(s) == "RegStore":
            return s.replace(dst_index=(P("*", s.dst_index[0], L(1)),) + tuple(s.dst_index[1:]))
        if ir.kind(s) == "CpAsyncCopy":
            return s.replace(src_index=tuple(_without(e, "_a2_ks") for e in s.src_index))
    assert "moves k differently from the output's slab" in refusal(rewrite(src, pin))

    # an atomic store, a guard: not this proof's business
    assert "an atomic add" in refusal(rewrite(src, lambda s: s.replace(atomic=True) if ir.kind(s) == "RegStore" else None))
    guarded = partial_source(tmp_path, m=40, n=60, k=72, splits=1, staged=False)
    assert "a block axis in the gmem_guard" in refusal(guarded)

    # the last fragment stored a second time
    tile = src.body[0]
    again = frontend.KernelSource(src.name, (tile.replace(body=tile.body + (tile.body[-1],)),), src.params, src.buffers, src.launch,
                                  src.written, src.constants, src.meta, src.path)
    assert "stored twice" in refusal(again)

    # a block axis inside a quotient
    def divide(s):
        if ir.kind(s) == "RegStore":
            return s.replace(dst_index=(s.dst_index[0], P("/", P("*", s.dst_index[1], L(2)), L(2)), s.dst_index[2]))
    assert "other than as a multiple added on" in refusal(rewrite(src, divide))


def _without(e, name):
    """``e`` with variable ``name`` replaced by 0."""
    k = ir.kind(e)
    if k == "Var":
        return problems.I(0) if e.name == name else e
    if k == "BinaryExpr":
        return e.replace(left=_without(e.left, name), right=_without(e.right, name))
    if k == "TernaryExpr":
        return e.replace(cond=_without(e.cond, name), if_true=_without(e.if_true, name), if_false=_without(e.if_false, name))
    return e


def one_warp_tile(acc_dtype: str, tail: tuple):
    """The reference's one-warp test kernel (tests/test_gpu_lowering.py:437-461): A (16 x 16) and B stored N x K
    (8 x 16) staged in shared memory by plain stores, ldmatrix x4 / x2, one mma into ``acc``, then ``tail``."""
    from emmy_ptx.ir import Axis, LdmatrixLoad, Load, MmaSyncPtx, RegFragment, Smem, Sync, Tile, Write, datatype
    P, L, V = problems.B, problems.I, problems.V
    lane, shape, f16 = V("_lane"), (16, 8, 16), datatype("f16")

    def at(cols, j):
        per = 16 // cols
        return (P("/", lane, L(per)), P("+", P("*", P("%", lane, L(per)), L(cols)), L(j)))

    fill = []
    for name, src, cols in (("a_s", "a", 8), ("b_s", "bt", 4)):
        for j in range(cols):
            fill += [Load(names=(f"{name}{j}",), input=src, index=at(cols, j), dtype=None),
                     Write(output=name, index=at(cols, j), values=(f"{name}{j}",), value_dtype=None)]
    return (Tile(axes=(Axis(name="_lane", extent=32),), body=(
        Smem(name="a_s", extents=(16, 16), dtype="__half", align=16), Smem(name="b_s", extents=(8, 16), dtype="__half", align=16),
        *fill, Sync(barrier_id=0, count=None, warp=False),
        RegFragment(name="fa", role="a", shape=shape, dtype=f16), RegFragment(name="fb", role="b", shape=shape, dtype=f16),
        RegFragment(name="acc", role="c", shape=shape, dtype=datatype(acc_dtype)),
        LdmatrixLoad(frag="fa", src_buffer="a_s", src_index=(L(0), L(0)), role="a", ldm=16),
        LdmatrixLoad(frag="fb", src_buffer="b_s", src_index=(L(0), L(0)), role="b", ldm=16, b_trans=True),
        MmaSyncPtx(c_frag="acc", a_frag="fa", b_frag="fb", shape=shape, c_dtype=acc_dtype),
        *tail), block_threads=32, aux_threads=0, raster_axes=None, raster_group=None, raster_orient="m"),)


def tile_inputs():
    rng = np.random.default_rng(11)
    a = (rng.standard_normal((16, 16)) / 4).astype(np.float16)
    bt = (rng.standard_normal((8, 16)) / 4).astype(np.float16)
    return a, bt, a.astype(np.float64) @ bt.astype(np.float64).T, rng.standard_normal((16, 8)).astype(np.float32)


def masked_bias_tail():
    from emmy_ptx.ir import ElementwiseImpl, FragmentApply, FragmentPromote, Literal, RegFragment, RegStore, datatype
    P, L, V = problems.B, problems.I, problems.V
    shape = (16, 8, 16)
    return (RegFragment(name="c", role="c", shape=shape, dtype=datatype("f32")),
            FragmentPromote(dst="c", src="acc"),
            FragmentApply(out="c", op=ElementwiseImpl("where"), args=(P(">", V("__fcol"), V("__frow")), Literal(value=-1.0, dtype="float"), "c"),
                          kinds=("coord", "uniform", "frag"), in_place=True, row_base=L(0), col_base=L(0)),
            FragmentApply(out="c", op=ElementwiseImpl("add"), args=("c", ("bias", (V("__frow"), V("__fcol")))), kinds=("frag", "gmem"),
                          in_place=True, row_base=L(0), col_base=L(0)),
            RegStore(dst_buffer="out", dst_index=(L(0), L(0)), frag="c", shape=shape))


def test_one_warp_tile_with_coordinate_mask_bias_and_f16_accumulator():
    """tests/test_gpu_lowering.py:464-483 of the reference, through the oracle: an f16-accumulate mma folded into an
    f32 fragment, a mask from each element's coordinates (column > row becomes -1) and a bias read at them."""
    a, bt, prod, bias = tile_inputs()
    bufs = {"a": a, "bt": bt, "bias": bias, "out": np.zeros((16, 8), np.float32)}
    fragment_oracle.run(one_warp_tile("f16", masked_bias_tail()), bufs, 1, 32)
    rows, cols = np.indices((16, 8))
    want = np.where(cols > rows, -1.0, prod.astype(np.float16)) + bias
    assert np.allclose(bufs["out"], want, rtol=2e-3, atol=2e-3)


def test_one_warp_tile_added_atomically_twice():
    """tests/test_gpu_lowering.py:486-496: the f32 tile stored twice into an f16 output with atomic adds."""
    from emmy_ptx.ir import RegStore
    L = problems.I
    a, bt, prod, _ = tile_inputs()
    tail = tuple(RegStore(dst_buffer="out", dst_index=(L(0), L(0)), frag="acc", shape=(16, 8, 16), atomic=True) for _ in range(2))
    bufs = {"a": a, "bt": bt, "out": np.zeros((16, 8), np.float16)}
    fragment_oracle.run(one_warp_tile("f32", tail), bufs, 1, 32)
    assert np.allclose(bufs["out"].astype(np.float64), 2 * prod, rtol=5e-3, atol=5e-3)


def attention_tile():
    """One warp, one 16-query tile against 16 keys, entirely in fragments: S = Q K^T on two accumulators, the row
    maximum and the row sum by FragmentRowReduce, exp(S - max) by FragmentApply with per-row operands, the weights
    repacked into an A operand (FragmentRepack), O = P V, the division by the row sum, RegStore."""
    from emmy_ptx.ir import (Axis, ElementwiseImpl, FragmentApply, FragmentRepack, FragmentRowReduce, LdmatrixLoad, MmaSyncPtx,
                             RegFragment, RegStore, Tile, datatype)
    L = problems.I
    shape, f16, f32 = (16, 8, 16), datatype("f16"), datatype("f32")
    body = [RegFragment(name="q", role="a", shape=shape, dtype=f16), RegFragment(name="kf", role="b", shape=shape, dtype=f16, count=2),
            RegFragment(name="s", role="c", shape=shape, dtype=f32, count=2), RegFragment(name="p", role="a", shape=shape, dtype=f16),
            RegFragment(name="vf", role="b", shape=shape, dtype=f16), RegFragment(name="o", role="c", shape=shape, dtype=f32),
            LdmatrixLoad(frag="q", src_buffer="q", src_index=(L(0), L(0)), role="a", staged=False)]
    for r in (0, 1):  # keys 8r .. 8r + 7: K is stored [key, d], the mma's column-major B as it stands
        body += [LdmatrixLoad(frag=f"kf[{r}]", src_buffer="k", src_index=(L(8 * r), L(0)), role="b", staged=False, b_trans=True),
                 MmaSyncPtx(c_frag=f"s[{r}]", a_frag="q", b_frag=f"kf[{r}]", shape=shape)]
    body += [FragmentRowReduce(frags=("s[0]", "s[1]"), op=ElementwiseImpl("maximum"), top="m_top", bot="m_bot")]
    body += [FragmentApply(out=f"s[{r}]", op=ElementwiseImpl("subtract"), args=(f"s[{r}]", ("m_top", "m_bot")), kinds=("frag", "row"),
                           in_place=True, post=(ElementwiseImpl("exp"),)) for r in (0, 1)]
    body += [FragmentRowReduce(frags=("s[0]", "s[1]"), op=ElementwiseImpl("add"), top="l_top", bot="l_bot"),
             FragmentRepack(frag="p", srcs=("s[0]", "s[1]"), ab_dtype="f16"),
             LdmatrixLoad(frag="vf", src_buffer="v", src_index=(L(0), L(0)), role="b", staged=False),  # V is [key, d]: K x N
             MmaSyncPtx(c_frag="o", a_frag="p", b_frag="vf", shape=shape),
             FragmentApply(out="o", op=ElementwiseImpl("divide"), args=("o", ("l_top", "l_bot")), kinds=("frag", "row"), in_place=True),
             RegStore(dst_buffer="out", dst_index=(L(0), L(0)), frag="o", shape=shape)]
    return (Tile(axes=(Axis(name="_lane", extent=32),), body=tuple(body), block_threads=32, aux_threads=0, raster_axes=None,
                 raster_group=None, raster_orient="m"),)


def attention_inputs():
    rng = np.random.default_rng(5)
    q, k, v = (rng.standard_normal(s).astype(np.float16) for s in ((16, 16), (16, 16), (16, 8)))
    s = q.astype(np.float64) @ k.astype(np.float64).T
    w = np.exp(s - s.max(1, keepdims=True))
    return q, k, v, (w / w.sum(1, keepdims=True)) @ v.astype(np.float64)


def test_attention_tile_in_fragments():
    q, k, v, want = attention_inputs()
    bufs = {"q": q, "k": k, "v": v, "out": np.zeros((16, 8), np.float32)}
    fragment_oracle.run(attention_tile(), bufs, 1, 32)
    assert np.allclose(bufs["out"], want, rtol=2e-3, atol=2e-3)  # the weights are rounded to f16 for the second mma


def zero_prologue_kernel(words: int):
    """CTA 0 zeroes the first ``words`` 32-bit words of ``acc``; every thread then adds 1 to acc[thread % 8] atomically."""
    from emmy_ptx.ir import Axis, Let, Literal, Tile, Write, ZeroPrologue, datatype
    P, L, V = problems.B, problems.I, problems.V
    return (Tile(axes=(Axis(name="a0", extent=64),), body=(
        ZeroPrologue(dst="acc", words=words), Let(name="one", value=Literal(value=1.0, dtype="float"), dtype=datatype("f32")),
        Write(output="tally", index=(P("%", V("a0"), L(8)),), values=("one",), value_dtype=None, atomic=True)),
        block_threads=64, aux_threads=0, raster_axes=None, raster_group=None, raster_orient="m"),)


def test_zero_prologue_clears_another_kernels_accumulator():
    bufs = {"acc": np.full(40, 7.0, np.float32), "tally": np.zeros(8, np.float32)}
    fragment_oracle.run(zero_prologue_kernel(33), bufs, 1, 64)
    assert (bufs["acc"][:33] == 0).all() and (bufs["acc"][33:] == 7.0).all() and (bufs["tally"] == 8).all()


def epilogue_tile():
    """The one-warp tile stored through a fused epilogue with row and column guards: y = relu(acc) + (row of the element
    in the tile), bound as the reference binds it (the fragment's element under the epilogue's parameter name, emmy's
    __M__ / __N__ for the element's coordinates; emmy_ptx/tensorcore.py:432-452). Rows >= 13 and columns >= 6 are not
    stored."""
    from emmy_ptx.ir import Assign, KNOWN, Let, RegStore, datatype
    L, V = problems.I, problems.V
    f32 = datatype("f32")
    epilogue = KNOWN["Epilogue"](params=("e0",), results=("y",), body=(
        Assign(name="r", op="relu", args=("e0",), dtype=None), Let(name="mrow", value=V("__M__"), dtype=f32),
        Assign(name="y", op="add", args=("r", "mrow"), dtype=None)))
    tail = (RegStore(dst_buffer="out", dst_index=(L(0), L(0)), frag="acc", shape=(16, 8, 16), epilogue=epilogue,
                     m_guard=(L(0), L(13)), n_guard=(L(0), L(6))),)
    return one_warp_tile("f32", tail)


def epilogue_expected(prod):
    rows, cols = np.indices((16, 8))
    want = np.maximum(prod, 0) + rows
    return np.where((rows < 13) & (cols < 6), want, -7.0)


def test_regstore_epilogue_and_guards():
    a, bt, prod, _ = tile_inputs()
    bufs = {"a": a, "bt": bt, "out": np.full((16, 8), -7.0, np.float32)}
    fragment_oracle.run(epilogue_tile(), bufs, 1, 32)
    assert np.allclose(bufs["out"], epilogue_expected(prod), rtol=1e-3, atol=1e-3)


def kn_tile():
    """One warp, B kept K x N (16 x 8) in shared memory and read with ldmatrix .x2.trans (the single-fragment form of
    the K x N slab), A read straight from global memory."""
    from emmy_ptx.ir import Axis, LdmatrixLoad, Load, MmaSyncPtx, RegFragment, RegStore, Smem, Sync, Tile, Write, datatype
    P, L, V = problems.B, problems.I, problems.V
    lane, shape, f16 = V("_lane"), (16, 8, 16), datatype("f16")
    fill = []
    for j in range(4):  # lane l stages row l / 2, columns (l % 2) * 4 + j of the 16 x 8 slab
        at = (P("/", lane, L(2)), P("+", P("*", P("%", lane, L(2)), L(4)), L(j)))
        fill += [Load(names=(f"b{j}",), input="b", index=at, dtype=None), Write(output="b_s", index=at, values=(f"b{j}",), value_dtype=None)]
    return (Tile(axes=(Axis(name="_lane", extent=32),), body=(
        Smem(name="b_s", extents=(16, 8), dtype="__half", align=16), *fill, Sync(barrier_id=0, count=None, warp=False),
        RegFragment(name="fa", role="a", shape=shape, dtype=f16), RegFragment(name="fb", role="b", shape=shape, dtype=f16),
        RegFragment(name="acc", role="c", shape=shape, dtype=datatype("f32")),
        LdmatrixLoad(frag="fa", src_buffer="a", src_index=(L(0), L(0)), role="a", staged=False),
        LdmatrixLoad(frag="fb", src_buffer="b_s", src_index=(L(0), L(0)), role="b", ldm=8, b_trans=False),
        MmaSyncPtx(c_frag="acc", a_frag="fa", b_frag="fb", shape=shape),
        RegStore(dst_buffer="out", dst_index=(L(0), L(0)), frag="acc", shape=shape)),
        block_threads=32, aux_threads=0, raster_axes=None, raster_group=None, raster_orient="m"),)


def kn_inputs():
    rng = np.random.default_rng(17)
    a = (rng.standard_normal((16, 16)) / 4).astype(np.float16)
    b = (rng.standard_normal((16, 8)) / 4).astype(np.float16)
    return a, b, a.astype(np.float64) @ b.astype(np.float64)


def test_b_read_transposed_from_a_k_by_n_slab():
    a, b, want = kn_inputs()
    bufs = {"a": a, "b": b, "out": np.zeros((16, 8), np.float32)}
    fragment_oracle.run(kn_tile(), bufs, 1, 32)
    assert np.allclose(bufs["out"], want, rtol=1e-5, atol=1e-5)


def test_the_proof_over_a_grid_of_shapes(tmp_path):
    """Every staged schedule the generator writes is a matmul: the proof must accept it exactly when the template's own
    limits allow (result of at least 8192 cells, K slabs of whole 64s when there are several), and name the shapes."""
    import itertools
    for m, n, k, splits, layout, dtype in itertools.product((32, 128, 272), (64, 160), (128, 384), (1, 2), ("kn", "nk"), ("f16", "bf16")):
        if (m % 16) or (n % 32) or ((k // splits) % 32) or (layout == "kn" and dtype == "bf16" and m == 32):
            continue
        src = partial_source(tmp_path, m=m, n=n, k=k, splits=splits, b_layout=layout, dtype=dtype)
        fits = m * n >= 8192 and (splits == 1 or (k // splits) % 64 == 0)
        try:
            plan = fragmatch.match_fragment_matmul(src, False)
        except families.Refusal as r:
            assert not fits, (m, n, k, splits, layout, dtype, str(r))
            assert "too small" in str(r) or "multiples of 64" in str(r)
            continue
        assert fits, (m, n, k, splits, layout, dtype)
        assert f"x0 [{m} x {k}]" in plan.remarks[0] and f"N = {n}]" in plan.remarks[0]
        assert ("K x N" if layout == "kn" else "N x K") in plan.remarks[0]
        assert f"emb::GemmShape{{{m}, {n}, {k}, {splits}}}" in plan.source
