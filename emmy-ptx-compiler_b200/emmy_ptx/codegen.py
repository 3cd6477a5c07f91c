"""The statement-by-statement lowering: Kernel IR (SIMT subset) -> one CUDA C++ kernel.

This is the backend's counterpart of the reference's plain lowering, "one rule
per statement, in the IR's order, without the optional rewrites"
(emmy_ptx/__init__.py:33-37, emmy_ptx/lower.py:181-198): every kernel the
templates do not take (or that is compiled with ``--plain``) goes through here,
so there is always device code and never a host fallback. The statement subset
is the interpreter's (tests/oracle.py:21-23) and the meaning of every statement
is the interpreter's too:

  * all threads of a block run each statement together under a mask
    (tests/oracle.py:112-118); a name that was never defined reads as zero
    (:65-70), so every name is a zero-initialised local here;
  * a Tile decodes the global thread index row-major over its axes and masks
    the threads beyond its cells (:121-132);
  * a loop with ``seed`` sets the accumulators of its own body to the reduction
    identity first (:134-141);
  * WarpShuffle is a butterfly over aligned lane groups (:238-245); TreeHalve
    folds its shared slab level by level, leaves it so and broadcasts the root
    (:247-268).

The few rewrites applied here unless ``plain`` keep every result bit for bit
(the reference allows exactly those under ``--strict``, compile.py:12-16):
16-byte global accesses for a multi-name Load or Write whose alignment is
proved from the index expression, and the tree folded by every thread in
registers behind its single barrier (emmy_ptx/lower.py:1334-1350, legal when
nothing reads the slab afterwards, :1385-1402). ``strict`` additionally keeps
nvcc from contracting a multiply and an add into an FMA (emmy_ptx/lower.py:953).
"""

from __future__ import annotations

import math

from . import clusterize, fragcode, ir
from .ir import dtype_name, kind

CTYPE = {"f32": "float", "f64": "double", "f16": "__half", "bf16": "__nv_bfloat16", "i8": "signed char",
         "i16": "short", "i32": "int", "i64": "long long", "u8": "unsigned char", "u16": "unsigned short",
         "u32": "unsigned", "u64": "unsigned long long", "bool": "unsigned char", "f8e4m3": "unsigned char",
         "f8e5m2": "unsigned char"}
SMEM_TYPE = {"float": "f32", "double": "f64", "int": "i32", "unsigned": "u32", "unsigned int": "u32", "__half": "f16",
             "__nv_bfloat16": "bf16"}
IDENTITY = {"add": 0.0, "multiply": 1.0, "maximum": -1e30, "minimum": 1e30}  # emmy_ptx/common.py:55-56
CANON = {"add": "add", "sum": "add", "multiply": "multiply", "prod": "multiply", "maximum": "maximum", "amax": "maximum",
         "fmax": "maximum", "minimum": "minimum", "fmin": "minimum"}  # emmy_ptx/common.py:57-60
INT_DTYPES = {"i16", "i32", "i64", "u8", "u16", "u32", "u64"}
INT_OPS = {"add", "subtract", "multiply", "floor_divide", "remainder", "mod", "left_shift", "right_shift", "bitwise_and",
           "bitwise_or", "bitwise_xor", "bitwise_count"}
WIDTH = {"u8": 8, "i16": 16, "u16": 16, "i32": 32, "u32": 32, "i64": 64, "u64": 64}
COMPARE = {"equal": "==", "not_equal": "!=", "greater": ">", "less": "<", "greater_equal": ">=", "less_equal": "<="}
CROSS_THREAD = ("WarpShuffle", "TreeHalve", "Sync") + fragcode.WARP_WIDE


class CodegenError(Exception):
    """IR outside what this lowering takes."""


def promote(op: str, dtypes: list) -> str:
    """emmy's result-type rule (emmy_ptx/elementwise.py:56-64)."""
    if dtypes and op in INT_OPS and all(d in INT_DTYPES for d in dtypes):
        signed = max((WIDTH[d] for d in dtypes if d[0] == "i"), default=0)
        unsigned = max((WIDTH[d] for d in dtypes if d[0] == "u"), default=0)
        return f"u{unsigned}" if unsigned >= signed else f"i{signed}"
    if dtypes and all(d == "f16" for d in dtypes):
        return "f16"
    return "f32"


def c_float(v: float, dtype: str = "f32") -> str:
    if math.isnan(v):
        return "__int_as_float(0x7fc00000)"
    if math.isinf(v):
        return ("-" if v < 0 else "") + "__int_as_float(0x7f800000)"
    text = repr(float(v))
    return text + ("f" if dtype != "f64" else "")


def divisor_constant(name) -> bool:
    """Is ``name`` a ConstantOp emmy made for the divisor of a source division: a scalar argument of a ``div`` node
    (``<node>_c<k>``) or a mean's element count (``<out>_count``)? (emmy_ptx/lower.py:1598-1604 of the reference)"""
    import re
    return bool(name) and (re.fullmatch(r"(div|divide|true_divide|truediv)(_\d+)?_c\d+", name) is not None or name.endswith("_count"))


def has_cross_thread(stmts) -> bool:
    return any(kind(s) in CROSS_THREAD for s in ir.walk(stmts))


def divisible(e, k: int, facts: dict) -> bool:
    """Is the integer expression a multiple of ``k`` for every thread? ``facts`` maps a loop
    variable to (start, step) and a Tile axis to None."""
    t = kind(e)
    if t == "Literal":
        return isinstance(e.value, int) and e.value % k == 0
    if t == "Var":
        f = facts.get(e.name)
        return f is not None and divisible(f[0], k, facts) and divisible(f[1], k, facts)
    if t == "BinaryExpr":
        if e.op in ("+", "-"):
            return divisible(e.left, k, facts) and divisible(e.right, k, facts)
        if e.op == "*":
            return divisible(e.left, k, facts) or divisible(e.right, k, facts)
    return False


class Emitter(fragcode.FragmentStatements):
    def __init__(self, src, plain: bool = False, strict: bool = False):
        self.const_from: dict = {}  # IR name -> the compile-time constant buffer it was loaded from
        self.reciprocal_of: dict = {}  # IR name -> value of the source divisor it is the reciprocal of
        self.frags: dict = {}  # fragment name -> (role, element dtype, members, registers)
        self.frag_decls: list = []
        self.smem_align: dict = {}
        self.src, self.plain, self.strict = src, plain, strict
        self.lines: list = []
        self.depth = 1
        self.vars: dict = {"lane": "i32", "warp": "i32"}  # IR name -> emmy dtype of the value
        self.shared: dict = {}  # name -> (dtype, extents)
        self.facts: dict = {}
        self.remarks: list = []
        self.guards = 0
        self.loop_depth = 0
        self.body = src.body
        self.cluster = 1  # blocks per thread-block cluster the kernel asks for

    # ------------------------------------------------------------ text

    def emit(self, text: str) -> None:
        self.lines.append("    " * self.depth + text)

    def var(self, name: str, dtype: str) -> str:
        old = self.vars.get(name)
        if old is not None and old != dtype:
            raise CodegenError(f"{name!r} is defined as {old} and as {dtype}")
        self.vars[name] = dtype
        return f"v_{name}"

    def use(self, name: str) -> tuple:
        if name not in self.vars:
            self.vars[name] = "f32"  # read before any definition: zero, as a float
        return f"v_{name}", self.vars[name]

    def remark(self, text: str) -> None:
        self.remarks.append(text)

    # ------------------------------------------------------------ expressions

    def expr(self, e) -> tuple:
        """(C text, 'int' | 'float' | 'bool'): integers are 64-bit, floats double, as the interpreter's."""
        t = kind(e)
        if t == "Var":
            code, dt = self.use(e.name)
            if dt in ("f32", "f64", "f16", "bf16"):
                return f"(double){self.to_float(code, dt)}", "float"
            return f"(long long){code}", "int"
        if t == "Literal":
            if isinstance(e.value, int) and not isinstance(e.value, bool):
                return f"{e.value}LL", "int"
            return c_float(float(e.value), "f64"), "float"
        if t == "BinaryExpr":
            (a, ka), (b, kb) = self.expr(e.left), self.expr(e.right)
            if e.op in ("+", "-", "*", "/", "%"):
                if e.op == "%" and "float" in (ka, kb):
                    raise CodegenError("% on floats")
                if e.op in ("/", "%") and ka != "float" and kb != "float":
                    return f"emb::trunc_{'div' if e.op == '/' else 'mod'}({a}, {b})", "int"
                return f"({a} {e.op} {b})", "float" if "float" in (ka, kb) else "int"
            if e.op in ("<", "<=", ">", ">=", "==", "!="):
                return f"({a} {e.op} {b})", "bool"
            if e.op in ("&&", "||"):
                return f"(({a}) != 0 {e.op} ({b}) != 0)", "bool"
            if e.op in ("&", "|", "^", "<<", ">>"):
                if "float" in (ka, kb):
                    raise CodegenError(f"{e.op} on floats")
                return f"((long long){a} {e.op} (long long){b})", "int"
            raise CodegenError(f"operator {e.op}")
        if t == "TernaryExpr":
            (c, _), (a, ka), (b, kb) = self.expr(e.cond), self.expr(e.if_true), self.expr(e.if_false)
            k = "float" if "float" in (ka, kb) else "int"
            ct = "double" if k == "float" else "long long"
            return f"(({c}) != 0 ? ({ct}){a} : ({ct}){b})", k
        if t == "CastExpr":
            a, _ = self.expr(e.expr)
            dt = dtype_name(e.dtype)
            return f"({'double' if dt[0] == 'f' else 'long long'})({CTYPE[dt]})({a})", "float" if dt[0] == "f" else "int"
        raise CodegenError(f"expression {t}")

    def truth(self, e) -> str:
        code, _ = self.expr(e)
        return f"(({code}) != 0)"

    def flat(self, shape, index) -> str:
        if len(index) > len(shape):
            raise CodegenError("more indices than dimensions")
        out = "0LL"
        for e, n in zip(index, shape):
            code, k = self.expr(e)
            if k == "float":
                code = f"(long long)({code})"
            out = f"({out} * {int(n)}LL + {code})" if out != "0LL" else code
        return out

    # ------------------------------------------------------------ conversions

    @staticmethod
    def to_float(code: str, dt: str) -> str:
        if dt == "f16":
            return f"__half2float({code})"
        if dt == "bf16":
            return f"__bfloat162float({code})"
        return code

    def convert(self, code: str, src: str, dst: str) -> str:
        """``code`` of emmy dtype ``src`` as a value of ``dst`` (numpy's astype / C's conversion)."""
        if src == dst:
            return code
        if dst == "bool":
            return f"(unsigned char)({self.to_float(code, src)} != 0)"
        wide = self.to_float(code, src)
        if dst == "f16":
            return f"__float2half_rn((float){wide})" if src != "f64" else f"__double2half({wide})"
        if dst == "bf16":
            return f"__float2bfloat16_rn((float){wide})"
        return f"({CTYPE[dst]})({wide})"

    # ------------------------------------------------------------ elementwise

    def apply(self, op: str, args: list, out: str) -> str:
        """C text of ``op(*args)`` in result dtype ``out``; ``args`` are (code, dtype) pairs
        (the rules of tests/oracle.py:335-353)."""
        if out == "bool" and op not in COMPARE:
            inner = "i32" if op in ("floor_divide", "remainder", "mod", "left_shift", "right_shift", "bitwise_xor",
                                    "bitwise_count") else "f32"
            return f"(unsigned char)(({self.apply(op, args, inner)}) != 0)"
        if op in COMPARE:
            (a, da), (b, db) = args
            return self.convert(f"({self.to_float(a, da)} {COMPARE[op]} {self.to_float(b, db)})", "i32", out)
        if op in ("to_f8e4m3", "to_f8e5m2"):  # the result is the byte code, whatever 8-bit type carries it
            code = f"emb::{op}({self.convert(args[0][0], args[0][1], 'f32')})"
            return code if out in ("f8e4m3", "f8e5m2", "u8") else self.convert(code, "u8", out)
        if out in ("f8e4m3", "f8e5m2"):
            raise CodegenError(f"{op} with an fp8 result")
        work = "f32" if out in ("f16", "bf16") else out  # halves are computed in float and rounded once
        T = CTYPE[work]
        c = [self.convert(code, dt, work) for code, dt in args]
        if op == "where":
            cond = f"({self.to_float(args[0][0], args[0][1])} != 0)"
            r = f"({cond} ? {c[1]} : {c[2]})"
        elif op in ("from_f8e4m3", "from_f8e5m2"):
            r = self.convert(f"emb::{op}((unsigned){args[0][0]})", "f32", work)
        elif work in ("f32", "f64"):
            suffix = "f" if work == "f32" else ""
            table = {
                "add": "emb::add({0}, {1})", "subtract": "emb::sub({0}, {1})", "multiply": "emb::mul({0}, {1})",
                "divide": "emb::div({0}, {1})", "maximum": "emb::maximum({0}, {1})", "minimum": "emb::minimum({0}, {1})",
                "negative": "(-{0})", "abs": f"fabs{suffix}({{0}})", "copy": "{0}", "pad": "{0}",
                "square": "emb::mul({0}, {0})", "reciprocal": "emb::rcp({0})", "relu": f"emb::maximum({{0}}, ({T})0)",
                "sqrt": "emb::sqrt_({0})",
            }
            single = {"exp": "emb::exp_f32({0})", "log": "emb::log_f32({0})", "tanh": "emb::tanh_f32({0})",
                      "erf": "erff({0})", "sin": "sinf({0})", "cos": "cosf({0})",
                      "sigmoid": "emb::rcp(emb::add(1.0f, emb::exp_f32(emb::sub(0.0f, {0}))))",
                      "rsqrt": "emb::rcp(emb::sqrt_({0}))", "pow": "powf({0}, {1})"}
            double = {"exp": "exp({0})", "log": "log({0})", "tanh": "tanh({0})", "erf": "erf({0})", "sin": "sin({0})",
                      "cos": "cos({0})", "sigmoid": "(1.0 / (1.0 + exp(-{0})))", "rsqrt": "(1.0 / sqrt({0}))",
                      "pow": "pow({0}, {1})"}
            fmt = table.get(op) or (single if work == "f32" else double).get(op)
            if fmt is None:
                raise CodegenError(f"elementwise op {op} on {work}")
            r = fmt.format(*c)
        elif work in INT_DTYPES or work == "i8":
            C = CTYPE[{"u8": "u32", "u16": "u32", "i8": "i32", "i16": "i32"}.get(work, work)]
            c = [f"({C}){x}" for x in c]
            table = {"add": "emb::add({0}, {1})", "subtract": "emb::sub({0}, {1})", "multiply": "emb::mul({0}, {1})",
                     "maximum": "emb::maximum({0}, {1})", "minimum": "emb::minimum({0}, {1})",
                     "floor_divide": "emb::floor_divide({0}, {1})", "remainder": "emb::remainder({0}, {1})",
                     "mod": "emb::remainder({0}, {1})", "left_shift": "({0} << {1})", "right_shift": "({0} >> {1})",
                     "bitwise_and": "({0} & {1})", "bitwise_or": "({0} | {1})", "bitwise_xor": "({0} ^ {1})",
                     "negative": "emb::sub(({2})0, {0})", "abs": "({0} < 0 ? emb::sub(({2})0, {0}) : {0})", "copy": "{0}",
                     "pad": "{0}", "square": "emb::mul({0}, {0})", "bitwise_count": "__popcll((unsigned long long){0})",
                     "relu": "emb::maximum({0}, ({2})0)"}
            fmt = table.get(op)
            if fmt is None:
                raise CodegenError(f"elementwise op {op} on {work}")
            r = f"({T})" + fmt.format(*((c + [C, C])[:2] + [C]))
        else:
            raise CodegenError(f"elementwise result type {out}")
        return self.convert(r, work, out) if work != out else r

    # ------------------------------------------------------------ statements

    def block(self, stmts, guard) -> None:
        """Emit ``stmts`` for the threads where ``guard`` (a C bool expression or None) holds."""
        run: list = []

        def flush():
            if not run:
                return
            if guard is not None:
                self.emit(f"if ({guard}) {{")
                self.depth += 1
            for s in run:
                getattr(self, "s_" + kind(s))(s)
            if guard is not None:
                self.depth -= 1
                self.emit("}")
            run.clear()

        for s in stmts:
            k = kind(s)
            if not hasattr(self, "s_" + k) and not hasattr(self, "x_" + k):
                raise CodegenError(f"statement {k}")
            if k == "Smem":
                self.s_Smem(s)
            elif k in CROSS_THREAD or (k in ("Loop", "Cond", "StridedLoop", "Tile") and any(has_cross_thread(c) for c in s.nested())):
                flush()
                getattr(self, "x_" + k)(s, guard)
            else:
                run.append(s)
        flush()

    def conj(self, guard, cond: str) -> str:
        return cond if guard is None else f"({guard} && {cond})"

    def new_guard(self, value: str) -> str:
        self.guards += 1
        name = f"g{self.guards}"
        self.emit(f"const bool {name} = {value};")
        return name

    # Tile: always at the top, handled with or without cross-thread statements inside
    def s_Tile(self, s) -> None:
        self.x_Tile(s, None)

    def x_Tile(self, s, guard) -> None:
        block = self.src.launch.block
        if s.raster_axes and s.raster_group is not None:
            raise CodegenError("rasterized Tile")
        if s.aux_threads or (s.block_threads not in (None, block)):
            raise CodegenError("banded or partial-block Tile")
        extents = [a.extent.as_static() for a in s.axes]
        cells = math.prod(extents)
        self.emit(f"const long long gid = (long long)blockIdx.x * {block} + threadIdx.x;")
        stride = 1
        for axis, n in zip(reversed(s.axes), reversed(extents)):
            name = self.var(axis.name, "i64")
            term = "gid" if stride == 1 else f"(gid / {stride}LL)"
            self.emit(f"{name} = {term} % {n}LL;")
            self.facts[axis.name] = None
            stride *= n
        inside = None
        if cells != self.src.launch.grid * block:
            inside = self.new_guard(self.conj(guard, f"(gid < {cells}LL)"))
            for axis in s.axes:  # masked threads keep zero
                self.emit(f"if (!{inside}) v_{axis.name} = 0;")
        plan = None
        if not self.plain and inside is None and guard is None and "clusters" not in getattr(self, "disable", ()):
            plan = clusterize.plan(s, self.src.launch.grid, block)
            if isinstance(plan, str):
                if any(kind(t) in ("Loop", "StridedLoop") for t in s.body):
                    self.remark(f"clusters: not used ({plan})")
                plan = None
        if plan is None:
            self.block(s.body, inside if inside is not None else guard)
        else:
            self.clustered(plan, block)

    def clustered(self, p, block: int) -> None:
        """The Tile body with loop ``p.loop`` split over a cluster of 8: every block computes its eighth of
        the iterations of the column-free part and stashes the results; after a cluster barrier every block
        runs all iterations of its own part on values read from the owners' shared memory."""
        self.cluster = clusterize.CLUSTER
        nv, var = len(p.values), p.loop.axis.name
        self.block(p.before, None)
        self.emit("cooperative_groups::cluster_group emb_cluster = cooperative_groups::this_cluster();")
        self.emit("const unsigned emb_rank = emb_cluster.block_rank();")
        self.emit(f"__shared__ float emb_stash[{p.slots * block * nv}];")
        start, _ = self.expr(p.start)
        v = self.var(var, "i64")
        self.seed(p.loop)
        self.loop_depth += 1
        self.emit(f"for (long long k_ = 0; k_ < {p.slots}LL; ++k_) {{")
        self.depth += 1
        self.emit(f"{v} = {start} + {p.step}LL * ((long long)emb_rank * {p.slots}LL + k_);")
        self.block(p.shared, None)
        for i, name in enumerate(p.values):
            code, dt = self.use(name)
            self.emit(f"emb_stash[(k_ * {block} + threadIdx.x) * {nv} + {i}] = {self.convert(code, dt, 'f32')};")
        self.depth -= 1
        self.emit("}")
        self.emit("emb_cluster.sync();")
        self.emit(f"for (long long j_ = 0; j_ < {p.trips}LL; ++j_) {{")
        self.depth += 1
        self.emit(f"{v} = {start} + {p.step}LL * j_;")
        self.emit(f"const float* peer_ = emb_cluster.map_shared_rank(emb_stash, (unsigned)(j_ / {p.slots}LL));")
        for i, name in enumerate(p.values):
            self.emit(f"{self.var(name, 'f32')} = peer_[((j_ % {p.slots}LL) * {block} + threadIdx.x) * {nv} + {i}];")
        self.block(p.own, None)
        self.depth -= 1
        self.emit("}")
        self.loop_depth -= 1
        self.emit("emb_cluster.sync();  // nobody leaves while a peer may still read its stash")
        self.remark(f"clusters of {clusterize.CLUSTER}: the column-free part of the loop over {var} ({p.trips} iterations per thread) "
                    f"is computed once per cluster, {p.slots} iterations per block, and {nv} value(s) per iteration pass through "
                    f"distributed shared memory ({p.slots * block * nv * 4} B stash per block)")
        self.block(p.after, None)

    def seed(self, loop) -> None:
        if not loop.seed:
            return
        for st in loop.body:
            if kind(st) == "Accum":
                dt = dtype_name(st.dtype) or "f32"
                op = CANON.get(st.op.name, st.op.name)
                if op not in IDENTITY:
                    raise CodegenError(f"no identity for {op}")
                value = IDENTITY[op]
                text = c_float(value, dt) if dt in ("f32", "f64") else self.convert(c_float(value), "f32", dt)
                self.emit(f"{self.var(st.name, dt)} = {text};")

    def s_Loop(self, s) -> None:
        self.seed(s)
        v = self.var(s.axis.name, "i64")
        n = s.axis.extent.as_static()
        if s.unroll:
            self.emit("#pragma unroll")
        self.emit(f"for ({v} = 0; {v} < {n}LL; ++{v}) {{")
        self.depth += 1
        self.loop_depth += 1
        self.block(s.body, None)
        self.loop_depth -= 1
        self.depth -= 1
        self.emit("}")
        self.emit(f"{v} = {max(n - 1, 0)}LL;")  # the name keeps its last value

    def x_Loop(self, s, guard) -> None:
        if guard is not None:
            self.emit(f"if ({guard}) {{")
            self.depth += 1
        self.seed(s)
        if guard is not None:
            self.depth -= 1
            self.emit("}")
        n = s.axis.extent.as_static()
        v = self.var(s.axis.name, "i64")
        it = f"it_{s.axis.name}"
        self.emit(f"for (long long {it} = 0; {it} < {n}LL; ++{it}) {{")
        self.depth += 1
        self.loop_depth += 1
        self.emit(f"if ({guard or 'true'}) {v} = {it};")
        self.block(s.body, guard)
        self.loop_depth -= 1
        self.depth -= 1
        self.emit("}")

    def s_StridedLoop(self, s) -> None:
        self.seed(s)
        v = self.var(s.axis.name, "i64")
        (start, _), (step, _) = self.expr(s.start), self.expr(s.step)
        if s.end is not None:
            end, _ = self.expr(s.end)
            self.emit(f"{self.var(s.axis.name + '_end', 'i64')} = {end};")
            end = f"v_{s.axis.name}_end"
        else:
            end = f"{s.axis.extent.as_static()}LL"
        self.facts[s.axis.name] = (s.start, s.step)
        last = f"last_{s.axis.name}"
        self.emit(f"long long {last} = {v};")
        self.emit(f"for (long long i_ = {start}, step_ = {step}; i_ < {end}; i_ += step_) {{")
        self.depth += 1
        self.loop_depth += 1
        self.emit(f"{v} = i_; {last} = i_;")
        self.block(s.body, None)
        self.loop_depth -= 1
        self.depth -= 1
        self.emit("}")
        self.emit(f"{v} = {last};")

    def x_StridedLoop(self, s, guard) -> None:
        """A strided loop around cross-thread statements: every thread of the block must make the same trips, which
        literal bounds guarantee (the K loops of the fragment form); threads outside ``guard`` walk along idle."""
        if not (kind(s.start) == "Literal" and kind(s.step) == "Literal" and (s.end is None or kind(s.end) == "Literal")):
            raise CodegenError("a cross-thread statement inside a strided loop whose bounds are not literals")
        if guard is not None:
            self.emit(f"if ({guard}) {{")
            self.depth += 1
        self.seed(s)
        if guard is not None:
            self.depth -= 1
            self.emit("}")
        v = self.var(s.axis.name, "i64")
        end = int(s.end.value) if s.end is not None else int(s.axis.extent.as_static())
        it = f"it_{s.axis.name}"
        if s.unroll:
            self.emit("#pragma unroll")
        self.emit(f"for (long long {it} = {int(s.start.value)}LL; {it} < {end}LL; {it} += {int(s.step.value)}LL) {{")
        self.depth += 1
        self.loop_depth += 1
        self.emit(f"{v} = {it};" if guard is None else f"if ({guard}) {v} = {it};")
        self.block(s.body, guard)
        self.loop_depth -= 1
        self.depth -= 1
        self.emit("}")

    def s_Cond(self, s) -> None:
        self.emit(f"if {self.truth(s.cond)} {{")
        self.depth += 1
        self.block(s.body, None)
        self.depth -= 1
        if s.else_body:
            self.emit("} else {")
            self.depth += 1
            self.block(s.else_body, None)
            self.depth -= 1
        self.emit("}")

    def x_Cond(self, s, guard) -> None:
        c = self.new_guard(self.truth(s.cond))
        self.block(s.body, self.new_guard(self.conj(guard, c)))
        if s.else_body:
            self.block(s.else_body, self.new_guard(self.conj(guard, f"!{c}")))

    def s_Let(self, s) -> None:
        code, k = self.expr(s.value)
        dt = dtype_name(s.dtype)
        if dt is None:
            if k == "float":
                dt = "f64"
            elif kind(s.value) == "Literal" and not -2**31 <= s.value.value < 2**31:
                dt = "i64"
            else:
                dt = "i32"  # an int, as C declares it
        if dt == "bool":
            self.emit(f"{self.var(s.name, dt)} = (unsigned char)(({code}) != 0);")
        else:
            self.emit(f"{self.var(s.name, dt)} = {self.convert(code, 'f64' if k == 'float' else 'i64', dt)};")

    def s_Init(self, s) -> None:
        dt = dtype_name(s.dtype)
        self.emit(f"{self.var(s.name, dt)} = {self.convert(c_float(float(s.identity), 'f64'), 'f64', dt)};")

    def s_Assign(self, s) -> None:
        args = [self.use(a) for a in s.args]
        out = dtype_name(s.dtype) or promote(s.op.name, [dt for _, dt in args])
        quotient = self.constant_quotient(s, out)
        self.reciprocal_of.pop(s.name, None)
        self.const_from.pop(s.name, None)
        if s.op.name == "reciprocal" and len(s.args) == 1 and divisor_constant(self.const_from.get(s.args[0])):
            self.reciprocal_of[s.name] = float(self.src.constants[self.const_from[s.args[0]]])
        if quotient is not None:
            (x, dx), c = quotient
            self.emit(f"{self.var(s.name, out)} = {self.convert(f'__fdiv_rn({self.convert(x, dx, 'f32')}, {c_float(c)})', 'f32', out)};")
            self.remark("x * reciprocal(c), where emmy split the source's x / c, computed as the correctly rounded x / c "
                        "(the divisor is a ConstantOp of a division)")
            return
        self.emit(f"{self.var(s.name, out)} = {self.apply(s.op.name, args, out)};")

    def constant_quotient(self, s, out: str):
        """((x code, x dtype), c) when the Assign multiplies x by the reciprocal of a source divisor c outside every loop
        with an f32 or f16 result: emmy turns the source's ``x / c`` into ``x * reciprocal(c)``, which can be an ulp from
        the correctly rounded quotient numpy gives (pointwise problems compare at rtol = 0). Recognised, as in the
        reference (emmy_ptx/lower.py:898-930,1598-1604), by the NAME of the constant (``div_c1``, ``*_count``): a
        convention, not a proof. Not under --strict or --plain, not for a power-of-two c (its reciprocal is exact)."""
        if (s.op.name != "multiply" or len(s.args) != 2 or self.strict or self.plain or self.loop_depth or out not in ("f32", "f16")
                or "quotient" in getattr(self, "disable", ())):
            return None
        for i in (0, 1):
            c = self.reciprocal_of.get(s.args[i])
            if c is None or c == 0.0 or not math.isfinite(c):
                continue
            if math.frexp(c)[0] in (0.5, -0.5):
                return None
            return self.use(s.args[1 - i]), c
        return None

    def s_Accum(self, s) -> None:
        if s.name not in self.vars:
            self.vars[s.name] = dtype_name(s.dtype) or "f32"
        acc, dt = self.use(s.name)
        base = self.use(s.base) if s.base is not None else (acc, dt)
        op = CANON.get(s.op.name, s.op.name)
        if op not in ("add", "subtract", "multiply", "divide", "maximum", "minimum"):
            op = "add"  # unknown combines fold additively (tests/oracle.py:193)
        self.emit(f"{acc} = {self.apply(op, [base, self.use(s.value)], dt)};")

    def s_Select(self, s) -> None:
        branches = list(s.branches)
        out = self.convert(*self.use(branches[-1].value), "f32")
        for br in reversed(branches[:-1]):
            out = f"({self.truth(br.select)} ? {self.convert(*self.use(br.value), 'f32')} : {out})"
        self.emit(f"{self.var(s.name, 'f32')} = {out};")

    def s_Smem(self, s) -> None:
        if s.name in self.shared:
            return
        ctype = getattr(s, "dtype", None) or "float"
        dt = SMEM_TYPE.get(ctype, ctype)
        if dt not in CTYPE:
            raise CodegenError(f"shared array of {ctype}")
        self.shared[s.name] = (dt, tuple(int(n) for n in s.extents))
        self.smem_align[s.name] = max(16, int(getattr(s, "align", 0) or 0))

    def memory(self, name: str) -> tuple:
        """(C array, element dtype, shape, is_shared, read_only)"""
        if name in self.shared:
            dt, shape = self.shared[name]
            return f"s_{name}", dt, shape, True, False
        buf = self.src.buffers.get(name)
        if buf is None:
            raise CodegenError(f"unknown buffer {name!r}")
        return f"p_{name}", buf.dtype, buf.shape, False, name not in self.src.written

    @staticmethod
    def value_dtype(mem_dtype: str) -> str:
        return {"f8e4m3": "u8", "f8e5m2": "u8"}.get(mem_dtype, mem_dtype)

    def s_Load(self, s) -> None:
        arr, dt, shape, shared, readonly = self.memory(s.input)
        idx = self.flat(shape, s.index)
        vdt = self.value_dtype(dt)
        out = dtype_name(s.dtype) or vdt
        n = len(s.names)
        for name in s.names:  # what these names held is gone
            self.const_from.pop(name, None)
            self.reciprocal_of.pop(name, None)
        if (not self.plain and not shared and readonly and n in (2, 4) and dt == "f32" and out == "f32"
                and self.aligned(shape, s.index, n)):
            vec = f"float{n}"
            self.emit("{")
            self.emit(f"    const {vec} q_ = __ldg(reinterpret_cast<const {vec}*>({arr} + {idx}));")
            for name, field in zip(s.names, "xyzw"):
                self.emit(f"    {self.var(name, 'f32')} = q_.{field};")
            self.emit("}")
            self.remark(f"{n * 4}-byte global load of {s.input}")
            return
        if len(s.names) == 1 and s.input in getattr(self.src, "constants", {}):
            self.const_from[s.names[0]] = s.input
        for k, name in enumerate(s.names):
            elem = f"{arr}[{idx} + {k}]" if k else f"{arr}[{idx}]"
            if not shared and readonly and dt in ("f32", "f64", "i32", "u32", "i64", "u64", "u8", "i8", "i16", "u16"):
                elem = f"__ldg(&{elem})"
            self.emit(f"{self.var(name, out)} = {self.convert(elem, vdt, out)};")

    def aligned(self, shape, index, n: int) -> bool:
        if not index or len(index) != len(shape):
            return False
        inner_ok = divisible(index[-1], n, self.facts)
        rows_ok = len(shape) == 1 or all(int(d) % n == 0 for d in shape[-1:])
        return inner_ok and rows_ok

    def s_Write(self, s) -> None:
        arr, dt, shape, shared, _ = self.memory(s.output)
        idx = self.flat(shape, s.index) if s.index else "0LL"
        vdt = self.value_dtype(dt)
        vals = [self.use(v) for v in s.values]
        n = len(vals)
        if (not self.plain and not shared and not s.atomic and n in (2, 4) and dt == "f32"
                and all(d == "f32" for _, d in vals) and self.aligned(shape, s.index, n)):
            self.emit(f"*reinterpret_cast<float{n}*>({arr} + {idx}) = make_float{n}({', '.join(c for c, _ in vals)});")
            self.remark(f"{n * 4}-byte global store to {s.output}")
            return
        for k, (code, d) in enumerate(vals):
            value = self.convert(code, d, vdt)
            target = f"{arr}[{idx} + {k}]" if k else f"{arr}[{idx}]"
            if s.atomic:
                if dt not in ("f32", "f64", "i32", "u32", "u64", "f16"):
                    raise CodegenError(f"atomic add on {dt}")
                self.emit(f"atomicAdd(&{target}, {value});")
            else:
                self.emit(f"{target} = {value};")

    def s_ZeroPrologue(self, s) -> None:
        """CTA 0 zeroes ``words`` 32-bit words of another kernel's accumulator (emmy_ptx/lower.py:1240-1259 of the reference)."""
        arr, _, _, shared, _ = self.memory(s.dst)
        if shared:
            raise CodegenError("ZeroPrologue of a shared array")
        self.emit(f"if (blockIdx.x == 0) for (long long z_ = threadIdx.x; z_ < {int(s.words)}LL; z_ += {self.src.launch.block}) "
                  f"reinterpret_cast<unsigned*>({arr})[z_] = 0u;")

    # ------------------------------------------------------------ cross-thread statements

    def x_Sync(self, s, guard) -> None:
        if s.warp:
            self.emit("__syncwarp();")
        else:
            self.emit("__syncthreads();")

    def combine(self, program, guard) -> None:
        if guard is not None:
            self.emit(f"if ({guard}) {{")
            self.depth += 1
        for a in program:
            self.s_Assign(a)
        if guard is not None:
            self.depth -= 1
            self.emit("}")

    def x_WarpShuffle(self, s, guard) -> None:
        length = int(s.length)
        if length & (length - 1) or length > 32:
            raise CodegenError(f"WarpShuffle over {length} lanes")
        width = length // 2
        while width:
            for st, sb in zip(s.state, s.state_b):
                code, dt = self.use(st)
                if dt not in ("f32", "f64", "i32", "u32", "i64", "u64", "f16"):
                    raise CodegenError(f"shuffle of {dt}")
                other = self.var(sb, dt)
                take = f"__shfl_xor_sync(emb_warp, {code}, {width})"
                self.emit(f"{{ const {CTYPE[dt]} t_ = {take}; if ({guard or 'true'}) {other} = t_; }}")
            self.combine(s.combine_states, guard)
            width //= 2

    def x_TreeHalve(self, s, guard) -> None:
        for b in s.bufs:
            if b not in self.shared:
                raise CodegenError("TreeHalve over a slab that is not shared memory")
        length = int(s.length)
        refusal = self.tree_refusal(s)
        if not self.plain and refusal is None:
            return self.one_barrier_tree(s, guard, length)
        if not self.plain:
            self.remark(f"tree over {s.bufs[0]} kept with a barrier per level: {refusal}")
        t, _ = self.use(s.tid_var)
        t = f"(long long){t}"
        if s.inner is not None:
            iv, _ = self.use(s.inner[0])
            slot = lambda k: f"(({k}) * {int(s.inner[1])}LL + (long long){iv})"  # noqa: E731
        else:
            slot = lambda k: f"({k})"  # noqa: E731
        half = length // 2
        while half:
            active = self.new_guard(self.conj(guard, f"({t} < {half}LL)"))
            self.emit(f"if ({active}) {{")
            self.depth += 1
            for st, sb, buf in zip(s.state, s.state_b, s.bufs):
                dt = self.shared[buf][0]
                self.emit(f"{self.var(st, dt)} = s_{buf}[{slot(t)}];")
                self.emit(f"{self.var(sb, dt)} = s_{buf}[{slot(f'{t} + {half}LL')}];")
            for a in s.combine_states:
                self.s_Assign(a)
            for st, buf in zip(s.state, s.bufs):
                self.emit(f"s_{buf}[{slot(t)}] = {self.use(st)[0]};")
            self.depth -= 1
            self.emit("}")
            self.emit("__syncthreads();")
            half //= 2
        for st, buf in zip(s.state, s.bufs):
            self.emit(f"if ({guard or 'true'}) {self.use(st)[0]} = s_{buf}[{slot('0LL')}];")

    def tree_refusal(self, s):
        """Why the tree may not be folded in registers behind one barrier (None: it may):
        the conditions of emmy_ptx/lower.py:1385-1402."""
        if self.loop_depth:
            return "the tree is inside a loop"
        if s.inner is not None:
            return "the tree has an inner index"
        if len(s.state) != 1 or int(s.length) > 32 or int(s.length) < 1:
            return "more than one state or more than 32 partials"
        seen = False
        for st in ir.walk(self.body):
            if st is s:
                seen = True
            elif seen and kind(st) == "Load" and st.input in s.bufs:
                return "the slab is read after the tree"
            elif seen and kind(st) == "TreeHalve" and set(st.bufs) & set(s.bufs):
                return "another tree uses the slab"
        return None

    def one_barrier_tree(self, s, guard, length: int) -> None:
        st, buf = s.state[0], s.bufs[0]
        dt = self.shared[buf][0]
        other = s.state_b[0]
        self.emit("{")
        self.depth += 1
        self.emit(f"{CTYPE[dt]} w_[{length}];")
        self.emit(f"for (int k_ = 0; k_ < {length}; ++k_) w_[k_] = s_{buf}[k_];")
        self.emit(f"{CTYPE[dt]} keep_ = {self.var(st, dt)};")
        half = length // 2
        while half:
            for t in range(half):
                self.emit(f"{self.var(st, dt)} = w_[{t}]; {self.var(other, dt)} = w_[{t + half}];")
                for a in s.combine_states:
                    self.s_Assign(a)
                self.emit(f"w_[{t}] = v_{st};")
            half //= 2
        self.emit(f"v_{st} = ({guard or 'true'}) ? w_[0] : keep_;")
        self.depth -= 1
        self.emit("}")
        self.remark(f"tree over {buf}: every thread folds the {length} partials behind one barrier")


def signature(src) -> str:
    parts = []
    for name in src.params:
        buf = src.buffers.get(name)
        if buf is None:
            raise CodegenError(f"parameter {name!r} has no buffer")
        const = "" if name in src.written else "const "
        parts.append(f"{const}{CTYPE[buf.dtype]}* __restrict__ p_{name}")
    return ", ".join(parts)


PRELUDE = """#include <cooperative_groups.h>
#include "emb_ops.cuh"
namespace emb {
__device__ __forceinline__ long long trunc_div(long long a, long long b) { return b == 0 ? a : a / b; }
__device__ __forceinline__ long long trunc_mod(long long a, long long b) { return b == 0 ? 0 : a % b; }
template <class T> __device__ __forceinline__ T zero() { return T(0); }
}
"""


def dependent_launch(src) -> tuple:
    """(waits, triggers): does the kernel read another kernel's ``intermediate`` output, and is its
    own output one (``final`` false)? From meta.json (examples/m_f16_128/meta.json shows the chain)."""
    meta = getattr(src, "meta", None)
    if not meta:
        return False, False
    waits = any(a.get("intermediate") for a in meta.get("args", ()))
    return waits, not meta.get("final", True)


def pdl_prologue(src, enabled: bool) -> list:
    """Programmatic dependent launch: let the next kernel of the chain be scheduled now, and wait for
    the previous one before touching its results."""
    if not enabled:
        return []
    waits, triggers = dependent_launch(src)
    out = []
    if triggers:
        out.append('    asm volatile("griddepcontrol.launch_dependents;");')
    if waits:
        out.append('    asm volatile("griddepcontrol.wait;" ::: "memory");')
    return out


def generate(src, plain: bool = False, strict: bool = False, disable=()) -> tuple:
    """(CUDA source, remarks, cluster size) of the statement-by-statement lowering of ``src``."""
    em = Emitter(src, plain, strict)
    em.disable = frozenset(disable)
    em.block(src.body, None)
    decls = [f"    {CTYPE[dt]} v_{name} = emb::zero<{CTYPE[dt]}>();" for name, dt in em.vars.items() if name not in ("lane", "warp")]
    smem = [f"    __shared__ __align__({em.smem_align.get(name, 16)}) {CTYPE[dt]} s_{name}[{math.prod(shape)}];"
            for name, (dt, shape) in em.shared.items()]
    attrs = f"__cluster_dims__({em.cluster}, 1, 1) " if em.cluster > 1 else ""
    head = [f"#define EMB_STRICT {int(strict)}", PRELUDE + ('#include "emb_frag.cuh"\n' if em.frags else ""),
            f'extern "C" __global__ void {attrs}__launch_bounds__({src.launch.block}) {src.name}({signature(src)}) {{',
            "    const unsigned emb_warp = __activemask();",
            "    int v_lane = threadIdx.x & 31, v_warp = threadIdx.x >> 5;",
            "    (void)emb_warp; (void)v_lane; (void)v_warp;"] + pdl_prologue(src, not plain)
    return "\n".join(head + smem + decls + em.frag_decls + em.lines + ["}"]) + "\n", em.remarks, em.cluster
