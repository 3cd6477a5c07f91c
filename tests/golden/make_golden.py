"""Generate tests/golden/oracle_cases.{json,npz}: outputs of the REFERENCE's own interpreter.

Run in the build container only (it reads the reference checkout, which does
not travel): ``python tests/golden/make_golden.py <path-to-reference>``.

The reference's tests/oracle.py is imported unchanged. It needs three symbols
of the absent emmy-ml package; a stand-in provides them from the reference's own
restatements (emmy_ptx/common.py:55-60 identities and canonical names,
emmy_ptx/elementwise.py:56-64 the promotion rule). Every case is then run by
that interpreter, and its inputs, serialized IR and outputs are stored; the
parity tests run oracle/ir_oracle.py on the same cases and compare bit for bit.

Cases: the three oracle-runnable shipped examples (their IR bodies are stored
as fixture data, with the values of their expected.npz), the interpreter's own
three self-tests (tests/test_oracle.py:60-105) rebuilt with this repository's
node classes, seeded random kernels of the reference's four random families
(tests/test_oracle.py:111-231: pointwise, shared_reduction, cooperative,
attention), and small instances of this repository's five workload IRs.
"""

from __future__ import annotations

import json
import sys
import types
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
REPO = HERE.parent.parent
sys.path.insert(0, str(REPO / "emmy-ptx-compiler_b200"))

from emmy_ptx import ir, problems  # noqa: E402
from emmy_ptx.ir import (Accum, Assign, Axis, BinaryExpr, Cond, Init, Let, Literal, Load, Loop, Smem,  # noqa: E402
                         StridedLoop, Sync, Tile, TreeHalve, Var, WarpShuffle, Write, datatype)

F32, I32, U32, BOOL = (datatype(n) for n in ("f32", "i32", "u32", "bool"))


def reference_oracle(ref: Path):
    identity = {"add": 0.0, "multiply": 1.0, "maximum": -1e30, "minimum": 1e30}
    canon = {"add": "add", "sum": "add", "multiply": "multiply", "prod": "multiply", "maximum": "maximum",
             "amax": "maximum", "fmax": "maximum", "minimum": "minimum", "fmin": "minimum"}
    int_dtypes = {"i16", "i32", "i64", "u8", "u16", "u32", "u64"}
    int_ops = {"add", "subtract", "multiply", "floor_divide", "remainder", "mod", "left_shift", "right_shift",
               "bitwise_and", "bitwise_or", "bitwise_xor", "bitwise_count"}
    width = {"u8": 8, "i16": 16, "u16": 16, "i32": 32, "u32": 32, "i64": 64, "u64": 64}

    class ElementwiseImpl:
        def __init__(self, name):
            self.name, self.identity = name, identity[name]

    def dtype_promote(op, dtypes):
        if dtypes and op in int_ops and all(d in int_dtypes for d in dtypes):
            s = max((width[d] for d in dtypes if d.startswith("i")), default=0)
            u = max((width[d] for d in dtypes if d.startswith("u")), default=0)
            return f"u{u}" if u >= s else f"i{s}"
        if dtypes and all(d == "f16" for d in dtypes):
            return "f16"
        return "f32"

    for name in ("emmy", "emmy.compiler", "emmy.compiler.ir", "emmy.compiler.ir.elementwise", "emmy.compiler.ir.stmt",
                 "emmy.compiler.ir.stmt.base"):
        sys.modules[name] = types.ModuleType(name)
    sys.modules["emmy.compiler.ir.elementwise"].ElementwiseImpl = ElementwiseImpl
    sys.modules["emmy.compiler.ir.elementwise"].reduce_canon = lambda n: canon.get(n, n)
    sys.modules["emmy.compiler.ir.stmt.base"].dtype_promote = dtype_promote
    sys.path.insert(0, str(ref / "tests"))
    import oracle
    return oracle


def I(v):  # noqa: E743
    return Literal(value=int(v), dtype="int")


def B(op, a, b):
    return BinaryExpr(op=op, left=a, right=b)


def V(n):
    return Var(name=n)


# ---------------------------------------------------------------- cases


def selftests():
    t = V("t")
    warps = B(">>", t, I(5))
    add = (Assign(name="s", op="add", args=("s", "sb")),)
    body = (Tile(axes=(Axis(name="t", extent=128),), block_threads=128, body=(
        Smem(name="partials", extents=(4,), dtype="float"), Init(name="s", identity=0.0, dtype=F32),
        Let(name="v", value=B("+", warps, I(1))),
        Cond(cond=B("==", B("&", t, I(31)), I(0)), body=(Write(output="partials", index=(warps,), values=("v",)),)),
        Sync(),
        TreeHalve(bufs=("partials",), state=("s",), state_b=("sb",), combine_states=add, length=4, tid_var="t"),
        Load(names=("slot",), input="partials", index=(B("&", t, I(3)),)),
        Write(output="out", index=(I(0), t), values=("s",)), Write(output="out", index=(I(1), t), values=("slot",)))),)
    yield "self_tree_slab", body, {}, {"out": np.zeros((2, 128), np.float32)}, 1, 128

    x = np.zeros(128, np.float32)
    x[:4] = 1
    mx = (Assign(name="s", op="maximum", args=("s", "sb")),)
    body = (Tile(axes=(Axis(name="t", extent=32),), block_threads=32, body=(
        StridedLoop(axis=Axis(name="i", extent=128), start=t, step=I(32), body=(
            Load(names=("v",), input="x", index=(V("i"),)), Accum(name="s", value="v"))),
        WarpShuffle(state=("s",), state_b=("sb",), combine_states=mx, length=32),
        Write(output="out", index=(t,), values=("s",)))),)
    yield "self_max_of_lane_sums", body, {"x": x}, {"out": np.zeros(32, np.float32)}, 1, 32

    a = np.array([-7, 7, 2**31 - 1, -2**31], np.int32)
    u = np.array([0xFFFFFFFF, 7, 0x80000000, 3], np.uint32)
    i = V("i")
    body = (Tile(axes=(Axis(name="i", extent=4),), body=(
        Load(names=("a",), input="xa", index=(i,), dtype=I32), Load(names=("u",), input="xu", index=(i,), dtype=U32),
        Let(name="three", value=I(3)), Let(name="one", value=I(1)),
        Assign(name="fd", op="floor_divide", args=("a", "three"), dtype=I32),
        Assign(name="wrap", op="add", args=("a", "one"), dtype=I32),
        Assign(name="sh", op="right_shift", args=("u", "one"), dtype=U32), Assign(name="eq", op="equal", args=("a", "a")),
        Write(output="out", index=(I(0), i), values=("fd",)), Write(output="out", index=(I(1), i), values=("wrap",)),
        Write(output="out", index=(I(2), i), values=("sh",)), Write(output="out", index=(I(3), i), values=("eq",)))),)
    yield "self_integers", body, {"xa": a, "xu": u}, {"out": np.zeros((4, 4), np.float64)}, 1, 4


def pointwise(rng):
    n = 256
    xs = rng.standard_normal(n).astype(np.float32) * 10
    xs[:6] = [0.0, -0.0, 3e30, -3e30, 1e-40, 16777217.0]
    inputs = {"xf": xs, "yf": rng.standard_normal(n).astype(np.float32),
              "xi": rng.integers(-2**31, 2**31, n, dtype=np.int64).astype(np.int32),
              "yi": np.where(rng.random(n) < 0.5, rng.integers(-50, 50, n), 16777217).astype(np.int32),
              "xu": rng.integers(0, 2**32, n, dtype=np.uint64).astype(np.uint32)}
    inputs["yi"][inputs["yi"] == 0] = 3
    i = V("i")
    stmts = [Load(names=("f0",), input="xf", index=(i,)), Load(names=("f1",), input="yf", index=(i,)),
             Load(names=("i0",), input="xi", index=(i,), dtype=I32), Load(names=("i1",), input="yi", index=(i,), dtype=I32),
             Load(names=("u0",), input="xu", index=(i,), dtype=U32),
             Let(name="nz", value=Literal(value=-0.0, dtype="float"), dtype=F32), Let(name="big", value=I(16777217)),
             Let(name="two", value=I(2))]
    pool = {"f": ["f0", "f1", "nz"], "i": ["i0", "i1", "big", "two"], "u": ["u0"]}
    ops = [("f", "add", 2), ("f", "subtract", 2), ("f", "multiply", 2), ("f", "maximum", 2), ("f", "minimum", 2),
           ("f", "abs", 1), ("f", "negative", 1), ("f", "reciprocal", 1), ("i", "add", 2), ("i", "multiply", 2),
           ("i", "floor_divide", 2), ("i", "remainder", 2), ("i", "bitwise_xor", 2), ("i", "maximum", 2),
           ("u", "right_shift", 2), ("u", "floor_divide", 2), ("u", "remainder", 2)]
    made = []
    for k in range(8):
        kind, op, arity = ops[rng.integers(len(ops))]
        if kind == "u":
            args = ("u0", "two")
        elif op in ("floor_divide", "remainder"):
            args = (str(rng.choice(pool["i"][:3])), "i1")
        else:
            args = tuple(str(rng.choice(pool[kind])) for _ in range(arity))
        name = f"v{k}"
        stmts.append(Assign(name=name, op=op, args=args, dtype={"f": F32, "i": I32, "u": U32}[kind]))
        stmts += [Let(name=f"b{k}", value=V(name), dtype=BOOL), Assign(name=f"d{k}", op="add", args=(name, name), dtype=BOOL)]
        pool[kind].append(name)
        made += [name, f"b{k}", f"d{k}"]
        if rng.random() < 0.4:
            kind2 = str(rng.choice(["f", "i"]))
            cmp_op = str(rng.choice(["equal", "not_equal", "less", "greater_equal"]))
            stmts.append(Assign(name=f"c{k}", op=cmp_op, args=tuple(str(rng.choice(pool[kind2])) for _ in range(2))))
            stmts.append(Assign(name=f"w{k}", op="where", args=(f"c{k}", "f0", "f1"), dtype=F32))
            made += [f"c{k}", f"w{k}"]
    stmts += [Write(output="out", index=(I(j), i), values=(name,)) for j, name in enumerate(made)]
    return (Tile(axes=(Axis(name="i", extent=n),), body=tuple(stmts)),), inputs, {"out": np.zeros((len(made), n), np.float64)}, 1, n


def shared_reduction(rng):
    cols = int(rng.choice([4, 8, 16, 32]))
    rows, trips = 256 // cols, int(rng.choice([24, 50, 64, 97]))
    op = str(rng.choice(["add", "maximum", "minimum"]))
    inputs = {"x": rng.standard_normal((rows, trips)).astype(np.float32),
              "y": rng.standard_normal(trips).astype(np.float32), "z": rng.standard_normal(cols).astype(np.float32)}
    body = (Tile(axes=(Axis(name="r", extent=rows), Axis(name="c", extent=cols)), body=(
        Loop(axis=Axis(name="k", extent=trips), body=(
            Load(names=("xv",), input="x", index=(V("r"), V("k"))), Load(names=("yv",), input="y", index=(V("k"),)),
            Assign(name="p", op="multiply", args=("xv", "yv")), Accum(name="acc", value="p", op=op))),
        Load(names=("zc",), input="z", index=(V("c"),)), Assign(name="o", op="add", args=("acc", "zc")),
        Write(output="out", index=(V("r"), V("c")), values=("o",)))),)
    return body, inputs, {"out": np.zeros((rows, cols), np.float64)}, 1, 256


def cooperative(rng):
    block = int(rng.choice([32, 64, 128, 256]))
    n = block * 4 * int(rng.integers(1, 5))
    fold, combine = str(rng.choice(["add", "maximum"])), str(rng.choice(["add", "maximum", "minimum"]))
    peek = block > 32 and rng.random() < 0.5
    inputs = {"x": rng.standard_normal(n).astype(np.float32)}
    t = V("t")
    comb = (Assign(name="s", op=combine, args=("s", "sb")),)
    stmts = [StridedLoop(axis=Axis(name="i", extent=n), start=t, step=I(block), body=(
                 Load(names=("v",), input="x", index=(V("i"),)), Accum(name="s", value="v", op=fold))),
             WarpShuffle(state=("s",), state_b=("sb",), combine_states=comb, length=min(block, 32))]
    outputs = {"out": np.zeros(block, np.float64)}
    if block > 32:
        warps = block // 32
        stmts += [Let(name="warp", value=B(">>", t, I(5))), Smem(name="slab", extents=(warps,), dtype="float"),
                  Cond(cond=B("==", B("&", t, I(31)), I(0)), body=(Write(output="slab", index=(V("warp"),), values=("s",)),)),
                  Sync(), TreeHalve(bufs=("slab",), state=("s",), state_b=("sb",), combine_states=comb, length=warps,
                                    tid_var="warp")]
        if peek:
            stmts += [Load(names=("left",), input="slab", index=(B("&", t, I(warps - 1)),)),
                      Write(output="peek", index=(t,), values=("left",))]
            outputs["peek"] = np.zeros(block, np.float64)
    stmts.append(Write(output="out", index=(t,), values=("s",)))
    return (Tile(axes=(Axis(name="t", extent=block),), block_threads=block, body=tuple(stmts)),), inputs, outputs, 1, block


def attention(rng):
    rows, cols = int(rng.choice([4, 8, 16])), int(rng.choice([4, 8, 16, 32]))
    d, keys = int(rng.choice([8, 16, 32])), int(rng.choice([16, 33, 44, 64, 100]))
    mask = np.where(rng.random(keys) < 0.2, -1e4, 0.0).astype(np.float32)
    inputs = {"q": rng.standard_normal((rows, d)).astype(np.float32), "kt": rng.standard_normal((d, keys)).astype(np.float32),
              "v": rng.standard_normal((keys, cols)).astype(np.float32), "mask": mask}
    scale = float(np.float32(1 / np.sqrt(d)))
    loop = Loop(axis=Axis(name="t", extent=keys), body=(
        Loop(axis=Axis(name="k", extent=d), body=(
            Load(names=("qk",), input="q", index=(V("r"), V("k"))), Load(names=("kk",), input="kt", index=(V("k"), V("t"))),
            Assign(name="p", op="multiply", args=("qk", "kk")), Accum(name="dot", value="p"))),
        Load(names=("mk",), input="mask", index=(V("t"),)),
        Let(name="scale", value=Literal(value=scale, dtype="float"), dtype=F32),
        Assign(name="s0", op="multiply", args=("dot", "scale")), Assign(name="s", op="add", args=("s0", "mk")),
        Let(name="one", value=Literal(value=1.0, dtype="float"), dtype=F32),
        Assign(name="gn", op="maximum", args=("s", "m")), Assign(name="dg", op="subtract", args=("m", "gn")),
        Assign(name="alpha", op="exp", args=("dg",)), Assign(name="dgo", op="subtract", args=("s", "gn")),
        Assign(name="beta", op="exp", args=("dgo",)), Assign(name="la", op="multiply", args=("alpha", "l")),
        Assign(name="lb", op="multiply", args=("beta", "one")), Accum(name="l", value="lb", base="la"),
        Assign(name="oa", op="multiply", args=("o", "alpha")), Load(names=("vv",), input="v", index=(V("t"), V("c"))),
        Assign(name="ob", op="multiply", args=("vv", "beta")), Accum(name="o", value="ob", base="oa"),
        Accum(name="m", value="s", op="maximum")))
    body = (Tile(axes=(Axis(name="r", extent=rows), Axis(name="c", extent=cols)), body=(
        loop, Assign(name="inv", op="reciprocal", args=("l",)), Assign(name="res", op="multiply", args=("o", "inv")),
        Write(output="out", index=(V("r"), V("c")), values=("res",)))),)
    return body, inputs, {"out": np.zeros((rows, cols), np.float64)}, 1, rows * cols


def workloads(rng):
    """Small instances of the five workload IRs (f32/f16 only: the reference has no bf16 or fp8)."""
    p = problems.array_sum(n=4096 * 3, grid=5, block=128, final_block=64)
    x = rng.uniform(-1, 1, 4096 * 3).astype(np.float32)
    yield "wl_sum_partial", p["kernels"][0]["body"], {"x": x}, {"sum__partial": np.zeros(5, np.float32)}, 5, 128
    part = rng.standard_normal(5).astype(np.float32)
    yield "wl_sum_final", p["kernels"][1]["body"], {"sum__partial": part}, {"sum_1": np.zeros((), np.float32)}, 1, 64
    p = problems.row_softmax(rows=6, cols=1024, block=64)
    x = rng.standard_normal((6, 1024)).astype(np.float32) * 3
    yield "wl_softmax", p["kernels"][0]["body"], {"x": x}, {"softmax": np.zeros((6, 1024), np.float32)}, 6, 64
    p = problems.matmul_f16(m=16, n=32, k=64, block=128)
    a = (rng.standard_normal((16, 64)) / 8).astype(np.float16)
    b = (rng.standard_normal((32, 64)) / 8).astype(np.float16)
    yield "wl_matmul", p["kernels"][0]["body"], {"a": a, "b": b}, {"matmul": np.zeros((16, 32), np.float16)}, 4, 128
    p = problems.attention(batch=1, heads=2, seq=24, dim=32)
    qkv = {n: rng.standard_normal((1, 2, 24, 32)).astype(np.float16) for n in "qkv"}
    yield "wl_attention", p["kernels"][0]["body"], qkv, {"attn": np.zeros((1, 2, 24, 32), np.float16)}, 48, 32


def shipped_examples(ref: Path):
    """The reference's own example problems the interpreter can run, inputs by their meta.json seeds."""
    for folder, blocks in (("r01_array_sum", None), ("a01_attention", None), ("k_gelu_mlp", [0, 1, 777, 2048, 4095])):
        meta = json.loads((ref / "examples" / folder / "meta.json").read_text())["kernels"][0]
        graph = json.loads((ref / "examples" / folder / f"{meta['entry']}.ir.json").read_text())
        body = tuple(ir.parse(s) for s in graph["nodes"][meta["node"]]["op_fields"]["body"])
        # a Tile with raster axes but no raster group is not rasterized (emmy_ptx/cells.py:315); the
        # interpreter refuses on the axes alone (tests/oracle.py:124), so they are cleared
        body = tuple(s.replace(raster_axes=None) if ir.kind(s) == "Tile" and s.raster_group is None else s for s in body)
        inputs, outputs = {}, {}
        for a in meta["args"]:
            dt = {"f32": np.float32}[a["dtype"]]
            if a.get("output"):
                shape = tuple(graph["nodes"][meta["node"]]["outputs"][0]["shape"])
                outputs[a["name"]] = np.zeros(shape, dt)
            elif "data" in a:
                inputs[a["name"]] = np.array(a["data"], dt).reshape(a["shape"])
            else:
                inputs[a["name"]] = np.random.default_rng(a["seed"]).standard_normal(a["shape"]).astype(dt)
        expected = dict(np.load(ref / "examples" / folder / "expected.npz"))
        yield f"ex_{folder}", body, inputs, outputs, int(meta["grid"][0]), int(meta["block"][0]), blocks, expected


def main():
    if len(sys.argv) != 2:
        raise SystemExit("usage: python tests/golden/make_golden.py <path to the reference checkout>")
    ref = Path(sys.argv[1])
    oracle = reference_oracle(ref)
    cases, arrays = [], {}

    def record(name, body, inputs, outputs, grid, block, blocks=None, expected=None):
        bufs = {**{k: v.copy() for k, v in inputs.items()}, **{k: v.copy() for k, v in outputs.items()}}
        if blocks is None:
            oracle.run(list(body), bufs, grid, block)
        else:
            for b in blocks:
                oracle._Block(bufs, b, block).run(list(body))
        case = dict(name=name, body=[repr(s) for s in body], grid=grid, block=block, blocks=blocks,
                    inputs=sorted(inputs), outputs=sorted(outputs), expected=sorted(expected or ()))
        for k, v in inputs.items():
            arrays[f"{name}/in/{k}"] = v
        for k in outputs:
            arrays[f"{name}/out/{k}"] = bufs[k]
        for k, v in (expected or {}).items():
            arrays[f"{name}/expected/{k}"] = v
        cases.append(case)
        print(name, {k: bufs[k].reshape(-1)[:3] for k in outputs})

    for case in shipped_examples(ref):
        record(*case)
    for case in selftests():
        record(*case)
    for family in (pointwise, shared_reduction, cooperative, attention):
        for seed in range(6):
            rng = np.random.default_rng(1000 * seed + len(family.__name__))
            record(f"rand_{family.__name__}_{seed}", *family(rng))
    for case in workloads(np.random.default_rng(2026)):
        record(*case)
    (HERE / "oracle_cases.json").write_text(json.dumps(cases, indent=0))
    np.savez_compressed(HERE / "oracle_cases.npz", **arrays)
    print(len(cases), "cases")


if __name__ == "__main__":
    main()
