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
