"""The tensor-core matchers: what they take, what their launch header carries, and when they refuse."""

import json
import re

import pytest

from emmy_ptx import compile_file, families, frontend, ir, problems, tcfamilies


def load(tmp_path, problem, entry):
    return frontend.load(problems.write(problem, tmp_path) / f"{entry}.ir.json")


def rebuilt(src, edit):
    tile = src.body[0]
    return frontend.KernelSource(src.name, (tile.replace(body=tuple(edit(list(tile.body)))),), src.params, src.buffers,
                                 src.launch, src.written, src.constants, src.meta)


def launch_of(ptx):
    return json.loads(re.search(r"^// launch: (.*)$", ptx, re.M).group(1))


def test_matmul_is_taken_and_described(tmp_path):
    folder = problems.write(problems.matmul_f16(m=256, n=512, k=128, ident="m"), tmp_path)
    ptx = compile_file(str(folder / "k_matmul.ir.json"))
    li = launch_of(ptx)
    assert li["family"] == "tensorcore" and li["block"] == [192, 1, 1] and li["grid"] == [4, 1, 1]
    kinds = [p["kind"] for p in li["params"]]
    assert kinds == ["buffer", "buffer", "buffer", "tmap", "tmap", "status"]
    a, b = li["params"][3], li["params"][4]
    assert a["dims"] == [128, 256] and a["box"] == [64, 128] and b["dims"] == [128, 512] and b["box"] == [64, 256]
    assert "tcgen05.mma" in ptx and "cp.async.bulk.tensor.2d" in ptx and "multicast" not in ptx.split("\n.version")[1]
    assert launch_of(compile_file(str(folder / "k_matmul.ir.json"), strict=True))["family"] == "statements"


def test_matmul_refusals(tmp_path):
    src = load(tmp_path, problems.matmul_f16(m=256, n=512, k=128, ident="m"), "k_matmul")
    with pytest.raises(families.Refusal, match="own order"):
        tcfamilies.match_matmul(src, True)
    # B indexed [k, n] while the buffer is [N, K]: the index and the storage disagree
    def swap(b):
        loop = b[0]
        lb = loop.body[1]
        return [loop.replace(body=(loop.body[0], lb.replace(index=(lb.index[1], lb.index[0])), *loop.body[2:])), b[1]]
    with pytest.raises(families.Refusal, match="buffer shapes do not fit the cells"):
        tcfamilies.match_matmul(rebuilt(src, swap), False)
    # an f16 product (no dtype on the multiply) is not the f32 accumulation the tensor cores do
    def f16_product(b):
        loop = b[0]
        mul = loop.body[2]
        return [loop.replace(body=(*loop.body[:2], mul.replace(dtype=None), loop.body[3])), b[1]]
    with pytest.raises(families.Refusal, match="f32 multiply"):
        tcfamilies.match_matmul(rebuilt(src, f16_product), False)
    odd = load(tmp_path, problems.matmul_f16(m=256, n=512, k=100, ident="odd"), "k_matmul")
    with pytest.raises(families.Refusal, match="16 bytes"):
        tcfamilies.match_matmul(odd, False)


def test_attention_is_taken_and_refused(tmp_path, monkeypatch):
    monkeypatch.delenv("EMMY_PTX_PREFER", raising=False)
    src = load(tmp_path, problems.attention(batch=1, heads=2, seq=256, dim=128, ident="a"), "k_attention")
    plan = tcfamilies.match_attention(src, False)
    # the default form: 64-key tiles, a producer warp, one issuer warp per query tile, one softmax warp group per query tile
    assert plan.family == "blocking" and plan.grid == 2 and plan.block == 32 * 3 + 256
    assert "attention_fwd_kernel64<2, true, false, 0, false, 128, 1>" in plan.source
    assert plan.smem_bytes == 2 * 32768 + 2 * 4 * 16384 + 1024 + 512
    full = load(tmp_path, problems.attention(batch=1, heads=1, seq=128, dim=128, causal=False, ident="b"), "k_attention")
    plan = tcfamilies.match_attention(full, False)
    assert plan.block == 32 * 2 + 128 and "attention_fwd_kernel64<1, false, false" in plan.source
    with pytest.raises(families.Refusal, match="own order"):
        tcfamilies.match_attention(src, True)
    # any key count is taken: a partial last tile, rows past the end read as zeros through three-dimensional tensor maps
    short = load(tmp_path, problems.attention(batch=1, heads=3, seq=96, dim=128, ident="c"), "k_attention")
    plan = tcfamilies.match_attention(short, False)
    assert "attention_fwd_kernel64<1, true, false" in plan.source and any("not a multiple of the 128-key tile" in r for r in plan.remarks)
    maps = {q["name"]: q for q in plan.extra_params if q["kind"] == "tmap"}
    assert all(q["dims"] == [128, 96, 3] and q["strides_bytes"] == [256, 96 * 256] for q in maps.values())
    assert maps["q"]["box"] == [64, 128, 1] and maps["k"]["box"] == maps["v"]["box"] == [64, 64, 1]
    # an additive per-key mask and the scale as the reciprocal of a division's constant
    masked = load(tmp_path, problems.attention(batch=1, heads=1, seq=256, dim=128, causal=False, mask=True, scale_as="reciprocal", ident="e"),
                  "k_attention")
    plan = tcfamilies.match_attention(masked, False)
    assert "attention_fwd_kernel64<2, false, false, 0, true, 128, 1>" in plan.source and ", p_mask);" in plan.source
    assert "0.12751" in plan.source and "11.3137" in plan.source  # log2(e) / sqrt(128) and sqrt(128), from the constant's value
    narrow = load(tmp_path, problems.attention(batch=1, heads=1, seq=128, dim=64, ident="d"), "k_attention")
    plan = tcfamilies.match_attention(narrow, False)
    assert plan.source.count(", 64, 1>(&tmap_q") == 1 and plan.smem_bytes == 16384 + 2 * 4 * 8192 + 1024 + 512
    # the other forms, on request: 128-key tiles (one score buffer per query tile, one issuer); two threads per query row
    monkeypatch.setenv("EMMY_PTX_PREFER", "keys128")
    plan = tcfamilies.match_attention(src, False)
    assert plan.block == 320 and "attention_fwd_kernel<2, true, false, 4, false, false, 128>" in plan.source
    assert all(q["box"] == [64, 128, 1] for q in plan.extra_params if q["kind"] == "tmap")
    assert tcfamilies.match_attention(narrow, False).smem_bytes == 5 * 16384 + 1280
    monkeypatch.setenv("EMMY_PTX_PREFER", "onepass")  # the one-pass maximum exists on 128-key tiles only
    assert "attention_fwd_kernel<2, true, false, 4, false, true, 128>" in tcfamilies.match_attention(src, False).source
    monkeypatch.setenv("EMMY_PTX_PREFER", "split2")
    plan = tcfamilies.match_attention(src, False)
    assert plan.block == 32 * 3 + 512 and "attention_fwd_kernel64<2, true, false, 0, false, 128, 2>" in plan.source
    assert plan.smem_bytes == 2 * 32768 + 2 * 4 * 16384 + 1024 + 512 + 4096
    monkeypatch.delenv("EMMY_PTX_PREFER")
    # work-item order: longest first over all heads while every head's K and V fit L2 together, else head by head
    assert "f, 1}, status" in tcfamilies.match_attention(src, False).source
    big = load(tmp_path, problems.attention(batch=8, heads=32, seq=4096, dim=128, ident="big"), "k_attention")
    assert "f, 0}, status" in tcfamilies.match_attention(big, False).source
    shard = load(tmp_path, problems.attention(batch=1, heads=32, seq=4096, dim=128, ident="shard"), "k_attention")
    assert "f, 1}, status" in tcfamilies.match_attention(shard, False).source
    assert "f, 0}, status" in tcfamilies.match_attention(full, False).source  # (not causal: every item is as long as the next)
    odd = load(tmp_path, problems.attention(batch=1, heads=1, seq=128, dim=32, ident="d32"), "k_attention")
    with pytest.raises(families.Refusal, match="head dimension"):
        tcfamilies.match_attention(odd, False)
    # the maximum must move LAST: an update that moves m before the sums read it is not the online softmax
    def early_max(b):
        loop = next(s for s in b if ir.kind(s) == "StridedLoop")
        body = list(loop.body)
        body.insert(2, body.pop())
        return [loop.replace(body=tuple(body)) if s is loop else s for s in b]
    with pytest.raises(families.Refusal, match="maximum does not move last"):
        tcfamilies.match_attention(rebuilt(src, early_max), False)


def test_mlp_is_taken_with_its_chain_and_refused(tmp_path):
    src = load(tmp_path, problems.gelu_mlp(tokens=128, d_model=256, hidden=512, lanes=8, block=64, ident="k"), "k_mlp_gelu")
    plan = tcfamilies.match_mlp(src, False)
    assert plan.family == "clusters" and [p["entry"] for p in plan.pre] == ["k_mlp_gelu__w1", "k_mlp_gelu__h", "k_mlp_gelu__w2"]
    assert [bool(p.get("pdl")) for p in plan.pre] == [False, False, True] and "griddepcontrol.launch_dependents" in plan.source
    scratch = {p["name"]: p["bytes"] for pre in plan.pre for p in pre["params"] if p["kind"] == "scratch"}
    assert scratch == {"w1t": 512 * 256 * 2, "w2t": 256 * 512 * 2, "h": 128 * 512 * 2}
    # the decode that runs alone streams 64 x 128 tiles; the one that runs beside the first matmul keeps 64 x 64 tiles
    assert plan.pre[0]["grid"] == [(256 // 64) * (512 // 128), 1, 1] and "dequant_transpose_e4m3<false, true>" in plan.source
    assert plan.pre[2]["grid"] == [(512 // 64) * (256 // 64), 1, 1] and "dequant_transpose_e4m3<true, false>" in plan.source
    ragged = load(tmp_path, problems.gelu_mlp(tokens=128, d_model=160, hidden=320, lanes=8, block=64, ident="r"), "k_mlp_gelu")
    plan_r = tcfamilies.match_mlp(ragged, False)
    assert plan_r.pre[0]["grid"] == [3 * 5, 1, 1] and "dequant_transpose_e4m3<false, false>" in plan_r.source
    with pytest.raises(families.Refusal, match="own order"):
        tcfamilies.match_mlp(src, True)
    # a different activation constant is not the tanh-form GELU
    wrong = frontend.KernelSource(src.name, src.body, src.params, src.buffers, src.launch, src.written,
                                  {**src.constants, "gelu_k": 0.05}, src.meta)
    with pytest.raises(families.Refusal, match="constants or wiring"):
        tcfamilies.match_mlp(wrong, False)


def test_tensor_maps_are_proved_on_the_host():
    """Row strides, box extents and the inner coordinates a template will ask for are checked before anything runs
    (an inner coordinate that is not a multiple of 16 bytes is an illegal instruction at run time)."""
    ok = tcfamilies.tmap("a", "a", "f16", (4096, 128), (8192,), (64, 128))
    assert ok["box"] == [64, 128] and ok["swizzle"] == "128B"
    for bad, why in ((dict(strides_bytes=(8190,)), "row stride"), (dict(box=(64, 512)), "outside 1..256"),
                     (dict(box=(32, 128)), "swizzle span"), (dict(step=(4, 128)), "coordinates")):
        args = dict(name="a", buffer="a", dtype="f16", dims=(4096, 128), strides_bytes=(8192,), box=(64, 128))
        args.update(bad)
        with pytest.raises(families.Refusal, match=why):
            tcfamilies.tmap(**args)


def test_matmul_keeps_an_epilogue_and_takes_either_b_layout(tmp_path):
    """The statements between the loop and the Write become a per-cell function of the template; B [K, N] is read
    MN-major on lone CTAs; an epilogue that reads a value of the loop's last trip is refused."""
    from emmy_ptx import frontend, problems, tcfamilies
    from emmy_ptx.families import Refusal
    from emmy_ptx.ir import Assign, datatype
    import pytest
    for layout in ("nk", "kn"):
        folder = problems.write(problems.matmul_bias_relu(m=256, n=512, k=128, b_layout=layout, ident=layout), tmp_path)
        src = frontend.load(folder / "k_matmul_bias_relu.ir.json")
        plan = tcfamilies.match_matmul(src, False)
        assert "auto cell_ = [&](float acc_, int row_, int col_) -> float {" in plan.source and "decltype(cell_)" in plan.source
        assert ("MN-major" in " ".join(plan.remarks)) == (layout == "kn")
        b_map = next(p for p in plan.extra_params if p.get("name") == "b")
        assert b_map["box"] == ([64, 64] if layout == "kn" else [64, 256])
    tile = src.body[0]
    body = list(tile.body)
    leak = Assign(name="z", op="add", args=("acc0", "in0"), dtype=datatype("f32"))
    bad = frontend.KernelSource(src.name, (tile.replace(body=tuple([body[0], leak] + body[1:])),), src.params, src.buffers, src.launch,
                                src.written, src.constants)
    with pytest.raises(Refusal, match="last trip"):
        tcfamilies.match_matmul(bad, False)
