"""The reduction and softmax matchers: what they take, and the legality conditions that make them refuse."""

import pytest

from emmy_ptx import families, frontend, ir, problems
from emmy_ptx.ir import Assign, Load, Write


def src_of(tmp_path, problem, entry):
    folder = problems.write(problem, tmp_path)
    return frontend.load(folder / f"{entry}.ir.json")


def rebuilt(src, edit):
    """``src`` with its Tile body passed through ``edit`` (a function list -> list)."""
    tile = src.body[0]
    return frontend.KernelSource(src.name, (tile.replace(body=tuple(edit(list(tile.body)))),), src.params, src.buffers,
                                 src.launch, src.written, src.constants)


@pytest.fixture
def sum_src(tmp_path):
    return src_of(tmp_path, problems.array_sum(n=8192, grid=4, block=128, final_block=64, ident="s"), "k_sum__partial")


@pytest.fixture
def softmax_src(tmp_path):
    return src_of(tmp_path, problems.row_softmax(rows=4, cols=1024, block=64, ident="f"), "k_softmax_reduce")


def test_the_authored_kernels_are_taken(sum_src, softmax_src):
    for strict in (False, True):
        plan = families.match_reduce(sum_src, strict)
        assert plan.family == "reduce" and "emb::strided_fold<4, emb::OpAdd" in plan.source
        assert ("true>" in plan.source.split("strided_fold")[1].split("(")[0]) == strict
        assert families.match_softmax(softmax_src, strict).family == "softmax"
    with pytest.raises(families.Refusal):
        families.match_softmax(sum_src, False)


def test_the_reference_example_form_is_taken(tmp_path):
    """One-name loads with step = block, the shape of examples/r01_array_sum."""
    src = src_of(tmp_path, problems.array_sum(n=1024, grid=1, block=128, final_block=128, ident="r"), "k_sum_1_reduce")
    assert "emb::strided_fold<1," in families.match_reduce(src, True).source


def refuses(src, why, fn=families.match_reduce):
    with pytest.raises(families.Refusal, match=why):
        fn(src, False)


def test_reduction_legality(sum_src):
    # the slab is read after the tree (the reference's _tree_refusal)
    peek = Load(names=("left",), input="acc0_smem", index=(ir.Var(name="warp"),))
    refuses(rebuilt(sum_src, lambda b: b + [peek]), "slab is read after")
    # warp redefined (combine_refusal: lane and warp unshadowed)
    let = ir.Let(name="warp", value=ir.Literal(value=0, dtype="int"))
    refuses(rebuilt(sum_src, lambda b: [b[0], let] + b[1:]), "redefined|butterfly")
    # no barrier between the slab's writes and the tree
    refuses(rebuilt(sum_src, lambda b: [s for s in b if ir.kind(s) != "Sync"]), "slab, barrier and tree")
    # the kernel writes the buffer it folds
    aliased = frontend.KernelSource(sum_src.name, sum_src.body, sum_src.params, sum_src.buffers, sum_src.launch,
                                    frozenset({"x", "sum__partial"}), {})
    refuses(aliased, "writes the buffer it folds")
    # a run that is not provably aligned: start (g*B + t)*4 + 1
    def shift(b):
        loop = b[0]
        start = ir.BinaryExpr(op="+", left=loop.start, right=ir.Literal(value=1, dtype="int"))
        return [loop.replace(start=start)] + b[1:]
    refuses(rebuilt(sum_src, shift), "not provably aligned")
    # the butterfly combines another state
    def other_state(b):
        ws = b[1]
        return [b[0], ws.replace(state=("zz",))] + b[2:]
    refuses(rebuilt(sum_src, other_state), "other states")
    # an unseeded loop continues an earlier value: not a pure fold
    refuses(rebuilt(sum_src, lambda b: [b[0].replace(seed=False)] + b[1:]), "not seeded")
    # threads outside the Tile
    wide = frontend.KernelSource(sum_src.name, sum_src.body, sum_src.params, sum_src.buffers,
                                 frontend.Launch(5, 128, 0), sum_src.written, {})
    refuses(wide, "threads outside the Tile")


def test_softmax_legality(softmax_src):
    # phase 3 multiplies by something else than the reciprocal of the sum
    def wrong_scale(b):
        l3 = b[-1]
        body = list(l3.body)
        body[3] = Assign(name=body[3].name, op="multiply", args=(body[2].name, "m"), dtype=body[3].dtype)
        return b[:-1] + [l3.replace(body=tuple(body))]
    refuses(rebuilt(softmax_src, wrong_scale), "no e \\* inv", families.match_softmax)
    # output written elsewhere than the cells read
    def moved(b):
        l3 = b[-1]
        w = l3.body[-1]
        idx = (w.index[0], ir.BinaryExpr(op="+", left=w.index[1], right=ir.Literal(value=4, dtype="int")))
        return b[:-1] + [l3.replace(body=l3.body[:-1] + (Write(output=w.output, index=idx, values=w.values),))]
    refuses(rebuilt(softmax_src, moved), "does not write the row's cells", families.match_softmax)
    # a row too long for the registers of one CTA
    big = problems.row_softmax(rows=2, cols=64 * 4 * 32, block=64, ident="big")
    src = frontend.KernelSource("k", big["kernels"][0]["body"], ("x", "softmax"),
                                {"x": frontend.Buffer("x", (2, 8192), "f32"), "softmax": frontend.Buffer("softmax", (2, 8192), "f32")},
                                frontend.Launch(2, 64, 0), frozenset({"softmax"}))
    refuses(src, "values of the row", families.match_softmax)


# ---------------------------------------------------------------- the regroup rewrite (scalar strided fold -> 16-byte chunks)


def lowered(src, **flags):
    from emmy_ptx.lower import Lowerer
    return Lowerer(src, **flags).run()


def test_the_scalar_spelling_is_regrouped_unless_strict_or_disabled(tmp_path):
    """emmy's own form (one-name loads, start = rank, step = copies * B): chunks of four in the optimizing mode only."""
    p = problems.array_sum_scalar(n=1 << 18, grid=512, block=128, copies=2, ident="sc")
    for entry in ("k_sum__partial", "k_sum_1_reduce"):
        src = src_of(tmp_path, p, entry)
        plan = families.match_reduce(src, False)
        assert "emb::strided_fold<4, emb::OpAdd" in plan.source and "v_a1_co * 4LL, 512LL" in plan.source
        assert any("contiguous 16-byte chunks" in r for r in plan.remarks)
        off = families.match_reduce(src, False, disable=frozenset({"regroup"})) if entry == "k_sum_1_reduce" else None
        if off is not None:
            assert "emb::strided_fold<1," in off.source and any("not regrouped: disabled" in r for r in off.remarks)
    # strict keeps the IR's order: one copy stays on the scalar template, two copies go to the statement lowering
    assert "emb::strided_fold<1," in families.match_reduce(src_of(tmp_path, p, "k_sum_1_reduce"), True).source
    with pytest.raises(families.Refusal, match="unrolled fold that is not regrouped"):
        families.match_reduce(src_of(tmp_path, p, "k_sum__partial"), True)


def test_a_fold_of_computed_values_is_regrouped_with_its_arithmetic(tmp_path):
    p = problems.array_sum_scalar(n=1 << 14, grid=2, block=128, copies=1, ident="sq")
    src = src_of(tmp_path, p, "k_sum__partial")
    def squared(b):
        loop = b[0]
        ld, acc = loop.body
        sq = Assign(name="sq", op="multiply", args=(ld.names[0], ld.names[0]), dtype=ir.datatype("f32"))
        return [loop.replace(body=(ld, sq, acc.replace(value="sq")))] + b[1:]
    plan = families.match_reduce(rebuilt(src, squared), False)
    assert "auto map_ = [&](float in_) -> float {" in plan.source and ", map_);" in plan.source


@pytest.mark.parametrize("name,why", [("weight", "w may differ between the cooperating threads"),
                                       ("row_of_thread", "an outer index moves with the loop or with the thread"),
                                       ("copies", "do not compute alike")])
def test_regroup_hazards_are_refused_with_the_reason(name, why):
    """Three of the reference's hazard kernels reach the regroup analysis (the other three are no block-wide fold at all):
    each must be kept strided, and say why (emmy_ptx/regroup.py:75-147,192-233, emmy_ptx/lower.py:250-272)."""
    import numpy as np
    from helpers import source
    from test_regroup_hazards import hazards
    body, inputs, threads, answer = hazards()[name]
    src = source("k_hazard", body, inputs, {"out": np.zeros(answer.shape, np.float32)}, 1, threads)
    kernel = lowered(src)
    assert any("not regrouped" in r and why in r for r in kernel.remarks), kernel.remarks
    assert "strided_fold<4" not in kernel.cuda_source


def test_a_maximum_of_sums_is_not_regrouped(tmp_path):
    """The butterfly combines with another operation than the loop folds with: the partial sums are observed."""
    p = problems.array_sum_scalar(n=1 << 14, grid=2, block=32, copies=1, ident="mx")
    src = src_of(tmp_path, p, "k_sum__partial")
    def max_of_sums(b):
        ws = b[1]
        c = ws.combine_states[0]
        return [b[0], ws.replace(combine_states=(Assign(name=c.name, op="maximum", args=tuple(c.args), dtype=None),))] + b[2:]
    plan = families.match_reduce(rebuilt(src, max_of_sums), False)
    assert "strided_fold<1," in plan.source and any("butterfly combines with maximum" in r for r in plan.remarks)


# ---------------------------------------------------------------- the pointwise template


def test_pointwise_kernels_take_the_streaming_template(tmp_path):
    for make, entry, streams in ((problems.bias_gelu, "k_bias_gelu", 2), (problems.bias_relu_residual, "k_bias_relu_res", 3)):
        src = src_of(tmp_path, make(rows=8, cols=1024, ident=entry), entry)
        for strict in (False, True):
            plan = families.match_pointwise(src, strict)
            assert plan.family == "pointwise" and plan.block == 256 and plan.grid == 8
            assert plan.source.count("emb::load_run(") == streams and plan.source.count("emb::store_run(") == 1
        assert plan.rows == dict(count=8, ctas_per_row=1, buffers={"x": 4096, "bias": 0, "y": 4096, **({"res": 4096} if streams == 3 else {})})


def test_pointwise_legality(tmp_path):
    src = src_of(tmp_path, problems.bias_relu_residual(rows=4, cols=512, ident="p"), "k_bias_relu_res")
    refuse = lambda s, why: refuses(s, why, families.match_pointwise)  # noqa: E731
    # a name read before it is defined would carry the previous cell's value
    refuse(rebuilt(src, lambda b: [Assign(name="z0", op="add", args=("o", "o"), dtype=ir.datatype("f32"))] + b), "read before it is defined")
    # lane moves with the thread, and the template re-deals the cells
    refuse(rebuilt(src, lambda b: b[:-1] + [Assign(name="o", op="add", args=("o", "lane"), dtype=ir.datatype("f32")), b[-1]]), "lane or warp")
    # a Write that is not at [.., innermost axis]
    def transposed(b):
        w = b[-1]
        return b[:-1] + [Write(output=w.output, index=(w.index[1], w.index[0]), values=w.values)]
    refuse(rebuilt(src, transposed), "not one value at")
    # an innermost axis that is not a multiple of four
    odd = src_of(tmp_path, problems.bias_relu_residual(rows=256, cols=6, block=256, ident="odd"), "k_bias_relu_res")
    refuse(odd, "not a multiple of 4")
    # a loop makes it another family's
    refuse(src_of(tmp_path, problems.row_softmax(rows=4, cols=512, block=64, ident="sm"), "k_softmax_reduce"), "statements other than")
