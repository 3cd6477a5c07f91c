"""Kernel-IR node classes, a reader for their serialized form, and a printer.

The IR files carry each kernel body as a list of strings, every string one
Python constructor expression with keyword arguments, e.g.::

    Tile(axes=(Axis(name='t', extent=Dim(128), window=None),), body=(...), block_threads=128, ...)

(reference: examples/r01_array_sum/k_sum_1_reduce.ir.json, field
``nodes.<id>.op_fields.body``; the reference hands the strings to the
third-party emmy package, emmy_ptx/frontend.py:54). This module reads them
with ``ast`` instead: no ``eval``, only calls of the known node names, tuples
and literals. ``repr`` of a node gives the same constructor form back, which is
how the shipped problems are authored.

Attribute names are the ones the serialized form uses, so code written against
emmy's node objects (the reference's interpreter, tests/oracle.py:72-268)
can walk these too.
"""

from __future__ import annotations

import ast

import numpy as np

_MISSING = object()


class Node:
    """A record with named fields in a fixed order; ``repr`` is its constructor call."""

    _fields: tuple = ()  # (name, default) pairs; a default of _MISSING makes the field required
    _positional: bool = False  # repr passes the fields positionally (Dim, ElementwiseImpl)
    _children: tuple = ()  # names of the fields holding nested statement tuples

    def __init__(self, *args, **kw):
        names = [f for f, _ in self._fields]
        if len(args) > len(names):
            raise TypeError(f"{type(self).__name__}: too many arguments")
        for name, value in zip(names, args):
            if name in kw:
                raise TypeError(f"{type(self).__name__}: {name} given twice")
            kw[name] = value
        for name, default in self._fields:
            if name in kw:
                value = kw.pop(name)
            elif default is _MISSING:
                raise TypeError(f"{type(self).__name__}: missing {name}")
            else:
                value = default
            object.__setattr__(self, name, value)
        self._extra = tuple(kw)  # fields this reader has no declaration for keep their order
        for name, value in kw.items():
            object.__setattr__(self, name, value)
        self._coerce()

    def _coerce(self) -> None:
        pass

    def field_names(self):
        return tuple(f for f, _ in self._fields) + self._extra

    def items(self):
        return tuple((f, getattr(self, f)) for f in self.field_names())

    def replace(self, **kw):
        d = dict(self.items())
        d.update(kw)
        return type(self)(**d)

    def nested(self):
        """The statement tuples nested in this statement (loop and branch bodies)."""
        return tuple(tuple(getattr(self, c) or ()) for c in self._children)

    def __repr__(self) -> str:
        if self._positional:
            return f"{type(self).__name__}({', '.join(_show(v) for _, v in self.items())})"
        return f"{type(self).__name__}({', '.join(f'{k}={_show(v)}' for k, v in self.items())})"

    def __eq__(self, other) -> bool:
        return type(other) is type(self) and self.items() == other.items()

    def __hash__(self) -> int:
        return hash((type(self).__name__, repr(self)))


def _show(v) -> str:
    if isinstance(v, np.dtype):
        return f"dtype('{v.name}')"
    if isinstance(v, tuple):
        return "(" + ", ".join(_show(x) for x in v) + ("," if len(v) == 1 else "") + ")"
    return repr(v)


# ---------------------------------------------------------------- leaves and expressions


class Dim(Node):
    _fields = (("value", _MISSING),)
    _positional = True

    def as_static(self) -> int:
        return int(self.value)


class DataType(Node):
    _fields = (("name", _MISSING), ("np", None), ("nbytes", None))


NUMPY_OF = {"f32": "float32", "f64": "float64", "f16": "float16", "i8": "int8", "i16": "int16", "i32": "int32",
            "i64": "int64", "u8": "uint8", "u16": "uint16", "u32": "uint32", "u64": "uint64", "bool": "bool"}
NBYTES = {"f32": 4, "f64": 8, "f16": 2, "bf16": 2, "i8": 1, "i16": 2, "i32": 4, "i64": 8, "u8": 1, "u16": 2,
          "u32": 4, "u64": 8, "bool": 1, "f8e4m3": 1, "f8e5m2": 1}


def datatype(name) -> DataType | None:
    """The DataType of an emmy dtype name (None stays None, a DataType is kept)."""
    if name is None or isinstance(name, DataType):
        return name
    # bf16 and the fp8 formats have no numpy dtype of their own: they travel as u16 / u8 codes
    np_name = NUMPY_OF.get(name, {"bf16": "uint16", "f8e4m3": "uint8", "f8e5m2": "uint8"}.get(name))
    return DataType(name=name, np=np.dtype(np_name), nbytes=NBYTES[name])


class ElementwiseImpl(Node):
    _fields = (("name", _MISSING),)
    _positional = True


def _op(v):
    return ElementwiseImpl(v) if isinstance(v, str) else v


class Var(Node):
    _fields = (("name", _MISSING),)


class Literal(Node):
    _fields = (("value", _MISSING), ("dtype", None))

    def _coerce(self):
        if self.dtype is None:
            self.dtype = "int" if isinstance(self.value, int) and not isinstance(self.value, bool) else "float"


class BinaryExpr(Node):
    _fields = (("op", _MISSING), ("left", _MISSING), ("right", _MISSING))


class TernaryExpr(Node):
    _fields = (("cond", _MISSING), ("if_true", _MISSING), ("if_false", _MISSING))


class CastExpr(Node):
    _fields = (("dtype", _MISSING), ("expr", _MISSING))


class Window(Node):
    _fields = (("parent", None), ("base", None), ("bound", None), ("partition", None))


class Axis(Node):
    _fields = (("name", _MISSING), ("extent", _MISSING), ("window", None))

    def _coerce(self):
        if isinstance(self.extent, int):
            self.extent = Dim(self.extent)


# ---------------------------------------------------------------- statements


class Tile(Node):
    _fields = (("axes", _MISSING), ("body", ()), ("block_threads", None), ("aux_threads", 0), ("raster_axes", None),
               ("raster_group", None), ("raster_orient", "m"))
    _children = ("body",)


class Loop(Node):
    _fields = (("axis", _MISSING), ("body", ()), ("unroll", False), ("seed", True))
    _children = ("body",)


class StridedLoop(Node):
    _fields = (("axis", _MISSING), ("start", _MISSING), ("step", _MISSING), ("body", ()), ("unroll", False),
               ("end", None), ("seed", True))
    _children = ("body",)


class Cond(Node):
    _fields = (("cond", _MISSING), ("body", ()), ("else_body", ()))
    _children = ("body", "else_body")


class Load(Node):
    _fields = (("names", None), ("input", _MISSING), ("index", ()), ("dtype", None))

    def __init__(self, *args, name=None, **kw):  # emmy also spells a one-value load ``name=``
        if name is not None:
            kw["names"] = (name,)
        super().__init__(*args, **kw)

    def _coerce(self):
        self.dtype = datatype(self.dtype)


class Write(Node):
    _fields = (("output", _MISSING), ("index", ()), ("values", _MISSING), ("value_dtype", None), ("atomic", False),
               ("swizzle", "NONE"))

    def _coerce(self):
        if isinstance(self.values, str):
            self.values = (self.values,)
        self.value_dtype = datatype(self.value_dtype)


class Assign(Node):
    _fields = (("name", _MISSING), ("op", _MISSING), ("args", _MISSING), ("dtype", None))

    def _coerce(self):
        self.op, self.dtype = _op(self.op), datatype(self.dtype)


class Accum(Node):
    _fields = (("name", _MISSING), ("value", _MISSING), ("op", "add"), ("dtype", None), ("axes", ()), ("base", None))

    def _coerce(self):
        self.op = _op(self.op)
        self.dtype = datatype(self.dtype if self.dtype is not None else "f32")


class Let(Node):
    _fields = (("name", _MISSING), ("value", _MISSING), ("dtype", None))

    def _coerce(self):
        self.dtype = datatype(self.dtype)


class Init(Node):
    _fields = (("name", _MISSING), ("identity", _MISSING), ("dtype", "f32"))

    def _coerce(self):
        self.dtype = datatype(self.dtype)


class SelectBranch(Node):
    _fields = (("value", _MISSING), ("select", None))


class Select(Node):
    _fields = (("name", _MISSING), ("branches", _MISSING))


class Smem(Node):
    _fields = (("name", _MISSING), ("extents", _MISSING), ("dtype", "float"), ("align", 0))


class Sync(Node):
    _fields = (("barrier_id", 0), ("count", None), ("warp", False))


class WarpShuffle(Node):
    _fields = (("state", _MISSING), ("state_b", _MISSING), ("combine_states", _MISSING), ("length", 32),
               ("dtype", None))

    def _coerce(self):
        self.dtype = datatype(self.dtype if self.dtype is not None else "f32")


class TreeHalve(Node):
    _fields = (("bufs", _MISSING), ("state", _MISSING), ("state_b", _MISSING), ("combine_states", _MISSING),
               ("length", _MISSING), ("tid_var", _MISSING), ("dtype", None), ("barrier_id", 0),
               ("barrier_count", None), ("inner", None))

    def _coerce(self):
        self.dtype = datatype(self.dtype if self.dtype is not None else "f32")


KNOWN = {c.__name__: c for c in (
    Dim, DataType, ElementwiseImpl, Var, Literal, BinaryExpr, TernaryExpr, CastExpr, Window, Axis, Tile, Loop,
    StridedLoop, Cond, Load, Write, Assign, Accum, Let, Init, SelectBranch, Select, Smem, Sync, WarpShuffle,
    TreeHalve)}

# ---------------------------------------------------------------- the tensor-core (fragment) form
#
# emmy's warp-level statements for mma.sync m16n8k16 and the asynchronous copies that feed them, with the fields
# and defaults the reference's lowering reads (emmy_ptx/tensorcore.py:147-420, emmy_ptx/lower.py:1057-1102).


class CpAsyncCopy(Node):
    _fields = (("smem", _MISSING), ("smem_index", _MISSING), ("src", _MISSING), ("src_index", _MISSING), ("nbytes", 16),
               ("swizzle", "NONE"), ("lane_index", None), ("lane_rows", None))


class CpAsyncCommit(Node):
    _fields = ()


class CpAsyncWait(Node):
    _fields = (("group", 0),)


class RegFragment(Node):
    _fields = (("name", _MISSING), ("role", _MISSING), ("shape", (16, 8, 16)), ("dtype", "f16"), ("count", 1), ("nregs", None))

    def _coerce(self):
        self.dtype = datatype(self.dtype)


class LdmatrixLoad(Node):
    _fields = (("frag", _MISSING), ("src_buffer", _MISSING), ("src_index", _MISSING), ("role", _MISSING), ("ldm", 0),
               ("swizzle", "NONE"), ("staged", True), ("gmem_guard", None), ("k_zero", None), ("b_trans", False),
               ("pair_frag", None), ("byte_slab", False), ("scale_buffer", None), ("scale_index", ()), ("scale_ldm", 0),
               ("fragment_layout", "m16n8k16"), ("fragment_index", 0))


class MmaSyncPtx(Node):
    _fields = (("c_frag", _MISSING), ("a_frag", _MISSING), ("b_frag", _MISSING), ("shape", (16, 8, 16)), ("ab_dtype", "f16"),
               ("c_dtype", "f32"), ("b_row_major", False), ("sfa_frag", None), ("sfb_frag", None))

    @property
    def block_scaled(self) -> bool:
        return self.sfa_frag is not None or self.sfb_frag is not None


class RegStore(Node):
    _fields = (("dst_buffer", _MISSING), ("dst_index", _MISSING), ("frag", _MISSING), ("shape", (16, 8, 16)), ("ldm", 0),
               ("epilogue", None), ("extra_frags", ()), ("m_guard", None), ("n_guard", None), ("atomic", False),
               ("fragment_layout", "m16n8k16"), ("volta_interleaved", False), ("fragment_index", (0, 0)),
               ("swizzle", "NONE"), ("row_dim", None), ("col_dim", None))


class FragmentApply(Node):
    _fields = (("out", _MISSING), ("op", _MISSING), ("args", _MISSING), ("kinds", _MISSING), ("in_place", False),
               ("row_base", None), ("col_base", None), ("post", ()), ("layout", None))


class FragmentRowReduce(Node):
    _fields = (("frags", _MISSING), ("op", _MISSING), ("top", _MISSING), ("bot", _MISSING), ("layout", None))


class FragmentRepack(Node):
    _fields = (("frag", _MISSING), ("srcs", _MISSING), ("ab_dtype", "f16"), ("fragment_layout", "m16n8k16"))


class FragmentPromote(Node):
    _fields = (("dst", _MISSING), ("src", _MISSING))


class ZeroPrologue(Node):
    """CTA 0 zeroes ``words`` 32-bit words of ``dst``, another kernel's accumulator (emmy_ptx/lower.py:1240-1259)."""
    _fields = (("dst", _MISSING), ("words", _MISSING))


FRAGMENT_FORM = ("CpAsyncCopy", "CpAsyncCommit", "CpAsyncWait", "RegFragment", "LdmatrixLoad", "MmaSyncPtx", "RegStore",
                 "FragmentApply", "FragmentRowReduce", "FragmentRepack", "FragmentPromote")
KNOWN["ZeroPrologue"] = ZeroPrologue
for _cls in (CpAsyncCopy, CpAsyncCommit, CpAsyncWait, RegFragment, LdmatrixLoad, MmaSyncPtx, RegStore, FragmentApply,
             FragmentRowReduce, FragmentRepack, FragmentPromote):
    KNOWN[_cls.__name__] = _cls
# read and printed like the rest, taken by no lowering here
for _name in ("FuncCallExpr", "Builtin", "FlatIndex", "FragmentLayout", "Epilogue"):
    KNOWN[_name] = type(_name, (Node,), {})


def fragment_ref(ref: str) -> tuple:
    """``name`` or ``name[i]`` as (name, index): the index an int, a variable name, or None."""
    if ref.endswith("]") and "[" in ref:
        name, _, index = ref[:-1].partition("[")
        return name, (int(index) if index.isdigit() else index)
    return ref, None


# ---------------------------------------------------------------- reader


class IRSyntaxError(ValueError):
    """A body string that is not a constructor expression of known node names."""


def parse(text: str) -> Node:
    """One serialized statement (a constructor expression) as a node tree."""
    try:
        tree = ast.parse(text, mode="eval")
    except SyntaxError as e:
        raise IRSyntaxError(f"not an expression: {e}") from None
    return _build(tree.body)


def _build(n):
    if isinstance(n, ast.Constant):
        return n.value
    if isinstance(n, ast.Tuple):
        return tuple(_build(e) for e in n.elts)
    if isinstance(n, ast.List):
        return [_build(e) for e in n.elts]
    if isinstance(n, ast.UnaryOp) and isinstance(n.op, (ast.USub, ast.UAdd)):
        v = _build(n.operand)
        if not isinstance(v, (int, float)):
            raise IRSyntaxError("a sign on something that is not a number")
        return -v if isinstance(n.op, ast.USub) else v
    if isinstance(n, ast.Name):
        if n.id in ("inf", "nan"):
            return float(n.id)
        raise IRSyntaxError(f"bare name {n.id!r}")
    if isinstance(n, ast.Call) and isinstance(n.func, ast.Name):
        name = n.func.id
        args = [_build(a) for a in n.args]
        kw = {k.arg: _build(k.value) for k in n.keywords}
        if name == "dtype":
            return np.dtype(*args)
        if name == "float" and len(args) == 1:  # float('inf'), float('-inf'), float('nan')
            return float(args[0])
        if name not in KNOWN:
            if args:  # a record this reader has no declaration for is taken by its keywords alone
                raise IRSyntaxError(f"unknown node {name!r}")
            KNOWN[name] = type(name, (Node,), {})
        return KNOWN[name](*args, **kw)
    raise IRSyntaxError(f"unexpected syntax {ast.dump(n)[:80]}")


# ---------------------------------------------------------------- walking


def walk(stmts):
    """Every statement of ``stmts`` and below, outer before inner, in program order."""
    for s in stmts:
        yield s
        for child in s.nested():
            yield from walk(child)


def kind(node) -> str:
    return type(node).__name__


def dtype_name(d) -> str | None:
    """The emmy dtype name of a DataType, a name, or None."""
    return None if d is None else getattr(d, "name", d)


def expr_vars(e) -> set:
    """Names an index or condition expression reads."""
    k = kind(e)
    if k == "Var":
        return {e.name}
    if k == "BinaryExpr":
        return expr_vars(e.left) | expr_vars(e.right)
    if k == "TernaryExpr":
        return expr_vars(e.cond) | expr_vars(e.if_true) | expr_vars(e.if_false)
    if k == "CastExpr":
        return expr_vars(e.expr)
    return set()


def show_expr(e) -> str:
    """An expression in C-like text (for remarks and listings)."""
    k = kind(e)
    if k == "Var":
        return e.name
    if k == "Literal":
        return repr(e.value)
    if k == "BinaryExpr":
        return f"({show_expr(e.left)} {e.op} {show_expr(e.right)})"
    if k == "TernaryExpr":
        return f"({show_expr(e.cond)} ? {show_expr(e.if_true)} : {show_expr(e.if_false)})"
    if k == "CastExpr":
        return f"({dtype_name(e.dtype)}){show_expr(e.expr)}"
    return repr(e)


def listing(stmts, depth: int = 1) -> str:
    """The indented text form of a body, in the style of the ``*.ir.txt`` files beside the examples."""
    pad, out = "    " * depth, []
    for s in stmts:
        k = kind(s)
        if k == "Tile":
            n = 1
            for a in s.axes:
                n *= a.extent.as_static()
            out.append(f"{pad}Tile[{', '.join(a.name for a in s.axes)}] (N={n})")
        elif k == "Loop":
            out.append(f"{pad}for {s.axis.name} in 0..{s.axis.extent.as_static()}")
        elif k == "StridedLoop":
            end = show_expr(s.end) if s.end is not None else s.axis.extent.as_static()
            out.append(f"{pad}for {s.axis.name} in {show_expr(s.start)}..{end}:{show_expr(s.step)}")
        elif k == "Cond":
            out.append(f"{pad}if ({show_expr(s.cond)}):")
        elif k == "Load":
            out.append(f"{pad}{', '.join(s.names)} = load {s.input}[{', '.join(show_expr(i) for i in s.index)}]")
        elif k == "Write":
            out.append(f"{pad}{s.output}[{', '.join(show_expr(i) for i in s.index)}] = {', '.join(s.values)}")
        elif k == "Assign":
            out.append(f"{pad}{dtype_name(s.dtype) or ''} {s.name} = {s.op.name}({', '.join(s.args)})".replace(f"{pad} ", pad))
        elif k == "Accum":
            out.append(f"{pad}{dtype_name(s.dtype)} {s.name} <- {s.op.name}({s.base or s.name}, {s.value})")
        elif k == "Let":
            out.append(f"{pad}{dtype_name(s.dtype) or 'int'} {s.name} = {show_expr(s.value)}")
        elif k == "Smem":
            out.append(f"{pad}Smem {s.dtype} {s.name}[{', '.join(str(e) for e in s.extents)}]")
        elif k == "Sync":
            out.append(f"{pad}Sync")
        elif k == "WarpShuffle":
            out.append(f"{pad}WarpShuffle({', '.join(s.state)}, length={s.length})")
        elif k == "TreeHalve":
            out.append(f"{pad}TreeHalve({', '.join(s.state)}, length={s.length}, tid={s.tid_var})")
        else:
            out.append(f"{pad}{k}(...)")
        if k == "Cond":
            out.append(listing(s.body, depth + 1))
            if s.else_body:
                out.append(f"{pad}else:")
                out.append(listing(s.else_body, depth + 1))
        else:
            for child in s.nested():
                if child:
                    out.append(listing(child, depth + 1))
    return "\n".join(x for x in out if x)
