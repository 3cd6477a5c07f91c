"""TEST INFRASTRUCTURE, NOT PRODUCT: a CPU restatement of the reference's Kernel-IR interpreter.

Only the tests, ``__graft_entry__.smoke()`` and the CPU-baseline legs of
``bench.py`` may import this module; no product code path may. It checks what
the GPU kernels compute and is never the thing shipped or measured as the
product.

What it restates: the reference's independent numpy interpreter of emmy
Kernel IR, tests/oracle.py (``run`` :44-49, ``_Block`` :52-268, ``apply``
:335-353), which runs a kernel body statement by statement with every thread
of a block in lockstep and is the definition of "right answer" for the
reference's own GPU tests (tests/test_oracle.py:267-280). That file needs
three symbols of the third-party package emmy-ml 0.3.11 (requirements.txt:2),
which is not available; the reference itself restates all three and those
restatements are what is followed here:

  * reduction identities, emmy's ElementwiseImpl table: emmy_ptx/common.py:55-56
  * reduction-name canonicalisation:                    emmy_ptx/common.py:57-60
  * result-dtype rule ``dtype_promote``:                emmy_ptx/elementwise.py:56-64

Differences of form, none of result: a value here is an array over
(blocks, threads) rather than over one block's threads, so that many CTAs are
interpreted by one numpy call per statement (blocks never see each other's
shared memory, and global writes land in block order, as when the reference
runs its blocks one after another). Kernels in which one block reads global
memory that another block of the same launch wrote are outside what this
batched form reproduces; ``run(..., batch=1)`` is the reference's block-at-a-time
order and serves those.

Extensions, stated as such wherever results are reported: the reference's
dtype table (tests/oracle.py:34-35) has no bf16 and no fp8. bf16 is added with
ml_dtypes.bfloat16; fp8-e4m3 values travel as u8 byte codes and are decoded by
the op ``from_f8e4m3`` (reference semantics: emmy_ptx/elementwise.py:100-129,
docs/DESIGN.md:619-628: value = byte code, 0x7f/0xff NaN, exact widening).

Parity pin: tests/golden/ holds outputs of the reference's own tests/oracle.py
(imported unchanged in the build container, with a three-symbol stand-in for
emmy) for the shipped examples, the interpreter's three self-tests
(tests/test_oracle.py:60-105) and seeded random kernels of its four families;
tests/test_oracle_parity.py compares this module with them bit for bit.
"""

from __future__ import annotations

import math

import numpy as np

try:  # only the bf16 / fp8 extension needs it
    import ml_dtypes
except ImportError:  # pragma: no cover
    ml_dtypes = None

WARP = 32

NP = {"f32": np.float32, "f64": np.float64, "f16": np.float16, "i16": np.int16, "i32": np.int32, "i64": np.int64,
      "u8": np.uint8, "u16": np.uint16, "u32": np.uint32, "u64": np.uint64, "bool": np.bool_}
if ml_dtypes is not None:
    NP["bf16"] = ml_dtypes.bfloat16  # extension (see the module text)
NP["f8e4m3"] = NP["f8e5m2"] = np.uint8  # extension: fp8 values travel as their byte codes
_NAME_OF = {np.dtype(v): k for k, v in NP.items()}
# C type names an Smem declaration may carry (tests/oracle.py:36)
C_TYPES = {"float": "f32", "double": "f64", "int": "i32", "unsigned": "u32", "unsigned int": "u32", "__half": "f16",
           "__nv_bfloat16": "bf16"}

# emmy_ptx/common.py:55-60
IDENTITY = {"add": 0.0, "multiply": 1.0, "maximum": -1e30, "minimum": 1e30}
REDUCE_CANON = {"add": "add", "sum": "add", "multiply": "multiply", "prod": "multiply", "maximum": "maximum",
                "amax": "maximum", "fmax": "maximum", "minimum": "minimum", "fmin": "minimum"}

# emmy_ptx/elementwise.py:28-38
_INT_DTYPES = frozenset({"i16", "i32", "i64", "u8", "u16", "u32", "u64"})
_INT_OPS = frozenset({"add", "subtract", "multiply", "floor_divide", "remainder", "mod", "left_shift", "right_shift",
                      "bitwise_and", "bitwise_or", "bitwise_xor", "bitwise_count"})
_WIDTH = {"u8": 8, "i16": 16, "u16": 16, "i32": 32, "u32": 32, "i64": 64, "u64": 64}


# Evaluate dot-product loops all trips at once (same additions, same order; see _Blocks.vector_loop).
VECTOR_LOOPS = True


class Unsupported(Exception):
    """An IR form outside the interpreter's subset (tests/oracle.py:40-41)."""


class _PerBlock(Exception):
    """A decision the reference takes per block came out differently across the batch."""


def promote(op: str, dtypes: list) -> str:
    """Result dtype of ``op`` on operands of ``dtypes`` (emmy_ptx/elementwise.py:56-64)."""
    if dtypes and op in _INT_OPS and all(d in _INT_DTYPES for d in dtypes):
        signed = max((_WIDTH[d] for d in dtypes if d[0] == "i"), default=0)
        unsigned = max((_WIDTH[d] for d in dtypes if d[0] == "u"), default=0)
        return f"u{unsigned}" if unsigned >= signed else f"i{signed}"
    if dtypes and all(d == "f16" for d in dtypes):
        return "f16"
    return "f32"


def reduce_canon(op: str) -> str:
    return REDUCE_CANON.get(op, op)


def run(body, buffers: dict, grid: int, block: int, blocks=None, batch: int | None = None) -> dict:
    """Run ``body`` on ``grid`` blocks of ``block`` threads and return ``buffers``
    (global name -> array, outputs included), updated in place (tests/oracle.py:44-49).

    ``blocks`` limits the run to those block indices (blocks are independent, so the
    cells they write are exactly what the full launch writes there). ``batch`` is how
    many blocks are interpreted together; None picks a size that keeps a value near a
    million elements.
    """
    ids = np.arange(grid, dtype=np.int64) if blocks is None else np.asarray(sorted(blocks), np.int64)
    if batch is None:
        # keep a value near a million elements, counting the extra axis of a vectorised inner loop
        widest = max([1] + [int(st.axis.extent.as_static()) for st in _all_statements(body)
                            if type(st).__name__ == "Loop"]) if VECTOR_LOOPS else 1
        batch = max(1, (1 << 20) // max(1, block * widest))
    for lo in range(0, len(ids), batch):
        part = ids[lo:lo + batch]
        try:
            _Blocks(buffers, part, block).run(body)
        except _PerBlock:
            if len(part) == 1:
                raise
            for b in part:
                _Blocks(buffers, np.asarray([b], np.int64), block).run(body)
    return buffers


def _name(d):
    return None if d is None else getattr(d, "name", d)


def _all_statements(stmts):
    for st in stmts:
        yield st
        for field in ("body", "else_body"):
            child = getattr(st, field, None)
            if isinstance(child, (tuple, list)):
                yield from _all_statements(child)


class _Blocks:
    """A batch of blocks in lockstep; every value is an array of shape (blocks, threads)."""

    def __init__(self, globals_: dict, ctaids: np.ndarray, block: int):
        self.globals = globals_
        self.nb, self.block = len(ctaids), block
        self.shape = (self.nb, block)
        self.ctaid = ctaids.reshape(-1, 1)
        self.tid = np.broadcast_to(np.arange(block, dtype=np.int64), self.shape)
        self.row = np.broadcast_to(np.arange(self.nb, dtype=np.int64).reshape(-1, 1), self.shape)
        self.shared: dict = {}  # name -> (blocks, size) array
        self.shared_shape: dict = {}
        # lane and warp are names a kernel may use without binding them (tests/oracle.py:58-61)
        self.env = {"lane": (self.tid & 31).astype(np.int32), "warp": (self.tid >> 5).astype(np.int32)}

    # ------------------------------------------------------------ values

    def bind(self, name, value, mask):
        """Masked definition: threads outside ``mask`` keep what they had (zero if nothing),
        converted to the new value's type (tests/oracle.py:65-70)."""
        value = np.broadcast_to(np.asarray(value), self.shape)
        old = self.env.get(name)
        if old is None:
            old = np.zeros(self.shape, value.dtype)
        elif old.dtype != value.dtype:
            old = old.astype(value.dtype)
        self.env[name] = np.where(mask, value, old)

    def ev(self, e):
        """An index or condition expression; C's truncating / and % on integers (tests/oracle.py:72-100)."""
        k = type(e).__name__
        if k == "Var":
            return self.env[e.name]
        if k == "Literal":
            v = e.value
            is_int = isinstance(v, (int, np.integer)) and not isinstance(v, bool)
            return np.full(self.shape, v, np.int64 if is_int else np.float64)
        if k == "BinaryExpr":
            a, b = self.ev(e.left), self.ev(e.right)
            if e.op in ("/", "%") and a.dtype.kind in "iu" and b.dtype.kind in "iu":
                q = np.trunc(a / np.where(b == 0, 1, b)).astype(np.int64)
                return q if e.op == "/" else a - q * b
            fn = _EXPR_OPS.get(e.op)
            if fn is None:
                raise Unsupported(f"operator {e.op}")
            return fn(a, b)
        if k == "TernaryExpr":
            return np.where(_truth(self.ev(e.cond)), self.ev(e.if_true), self.ev(e.if_false))
        if k == "CastExpr":
            return self.ev(e.expr).astype(NP[_name(e.dtype)])
        raise Unsupported(f"expression {k}")

    def flat_index(self, shape, index):
        """Row-major element index (tests/oracle.py:106-110)."""
        idx = np.zeros(self.shape, np.int64)
        for e, n in zip(index, shape):
            idx = idx * int(n) + self.ev(e).astype(np.int64)
        return idx

    def extents_of(self, name):
        return self.shared_shape[name] if name in self.shared else self.globals[name].shape

    # ------------------------------------------------------------ statements

    def run(self, stmts, mask=None):
        mask = np.ones(self.shape, bool) if mask is None else mask
        for s in stmts:
            fn = getattr(self, "do_" + type(s).__name__, None)
            if fn is None:
                raise Unsupported(f"statement {type(s).__name__}")
            fn(s, mask)

    def do_Tile(self, s, mask):  # tests/oracle.py:121-132
        if s.raster_axes or s.aux_threads or (s.block_threads not in (None, self.block)):
            raise Unsupported("rasterized, banded or partial-block Tile")
        extents = [int(a.extent.as_static()) for a in s.axes]
        gid = self.ctaid * self.block + self.tid
        mask = mask & (gid < math.prod(extents))
        stride = 1
        for axis, n in zip(reversed(s.axes), reversed(extents)):
            self.bind(axis.name, (gid // stride) % n, mask)
            stride *= n
        self.run(s.body, mask)

    def seed(self, loop, mask):  # tests/oracle.py:134-141
        if not loop.seed:
            return
        for st in loop.body:
            if type(st).__name__ == "Accum":
                identity = IDENTITY[reduce_canon(st.op.name)]
                self.bind(st.name, np.asarray(identity).astype(NP[_name(st.dtype) or "f32"]), mask)

    def do_Loop(self, s, mask):  # tests/oracle.py:143-147
        if VECTOR_LOOPS and self.vector_loop(s, mask):
            return
        self.seed(s, mask)
        for i in range(int(s.axis.extent.as_static())):
            self.bind(s.axis.name, np.int64(i), mask)
            self.run(s.body, mask)

    def vector_loop(self, s, mask) -> bool:
        """A seeded loop whose body only loads, computes and ends in ONE plain sum (a dot product):
        all trips are evaluated at once along an extra axis, and the sum is taken by
        ``np.cumsum`` in the accumulator's type, which adds strictly left to right from the
        identity 0, i.e. performs the very additions of the trip-by-trip loop in the same order
        (the parity tests run both forms and compare bit for bit). Returns False when the loop is
        not of that shape; the caller then runs it trip by trip."""
        n = int(s.axis.extent.as_static())
        body = list(s.body)
        if not s.seed or n < 4 or not body or type(body[-1]).__name__ != "Accum":
            return False
        acc = body[-1]
        if reduce_canon(acc.op.name) != "add" or acc.base is not None or (_name(acc.dtype) or "f32") not in ("f32", "f64"):
            return False
        defined, read = [], set()
        for st in body[:-1]:
            k = type(st).__name__
            if k == "Load":
                defined += list(st.names)
                for e in st.index:
                    read |= _expr_names(e)
            elif k == "Assign":
                defined.append(st.name)
                read |= set(st.args)
            else:
                return False
        if acc.name in defined or acc.name in read or acc.value not in defined or s.axis.name in defined:
            return False
        sub = _Blocks.__new__(_Blocks)
        sub.globals, sub.nb, sub.block, sub.shape = self.globals, self.nb, self.block * n, (self.nb, self.block * n)
        sub.ctaid = self.ctaid
        sub.tid = np.repeat(self.tid, n, axis=1)
        sub.row = np.broadcast_to(np.arange(self.nb, dtype=np.int64).reshape(-1, 1), sub.shape)
        sub.shared, sub.shared_shape = self.shared, self.shared_shape
        sub.env = {k: np.repeat(v, n, axis=1) for k, v in self.env.items() if k in read and k not in defined}
        sub.env[s.axis.name] = np.broadcast_to(np.tile(np.arange(n, dtype=np.int64), self.block), sub.shape)
        wide = np.repeat(mask, n, axis=1)
        sub.run(body[:-1], wide)
        t = NP[_name(acc.dtype) or "f32"]
        v = sub.env[acc.value].reshape(self.nb, self.block, n).astype(t)
        zero = np.zeros((self.nb, self.block, 1), t)
        total = np.cumsum(np.concatenate([zero, v], axis=2), axis=2, dtype=t)[:, :, -1]
        self.bind(acc.name, total, mask)
        for name in defined:  # the names keep their last trip's values, the loop variable its last index
            self.bind(name, sub.env[name].reshape(self.nb, self.block, n)[:, :, -1], mask)
        self.bind(s.axis.name, np.int64(n - 1), mask)
        return True

    def do_StridedLoop(self, s, mask):  # tests/oracle.py:149-166
        self.seed(s, mask)
        start, step = self.ev(s.start).astype(np.int64), self.ev(s.step).astype(np.int64)
        if s.end is not None:
            end = self.ev(s.end).astype(np.int64)
            self.bind(f"{s.axis.name}_end", end, mask)
        else:
            end = np.full(self.shape, int(s.axis.extent.as_static()), np.int64)
        trip = 0
        while True:
            v = start + trip * step
            active = mask & (v < end)
            if not active.any():
                return
            self.bind(s.axis.name, v, active)
            self.run(s.body, active)
            trip += 1

    def do_Cond(self, s, mask):  # tests/oracle.py:168-171
        c = _truth(self.ev(s.cond))
        self.run(s.body, mask & c)
        self.run(s.else_body, mask & ~c)

    def do_Let(self, s, mask):  # tests/oracle.py:173-179
        v = self.ev(s.value)
        if s.dtype is not None:
            v = v.astype(NP[_name(s.dtype)])
        elif v.dtype == np.int64:
            fits = np.all((v >= -2**31) & (v < 2**31), axis=1)  # the reference decides block by block
            if fits.all():
                v = v.astype(np.int32)  # an int, as C declares it
            elif fits.any():
                raise _PerBlock
        self.bind(s.name, v, mask)

    def do_Init(self, s, mask):  # tests/oracle.py:181-182
        self.bind(s.name, np.asarray(s.identity).astype(NP[_name(s.dtype)]), mask)

    def do_Assign(self, s, mask):  # tests/oracle.py:184-187
        args = [self.env[a] for a in s.args]
        out = _name(s.dtype) or promote(s.op.name, [_NAME_OF[a.dtype] for a in args])
        self.bind(s.name, apply(s.op.name, args, out), mask)

    def do_Accum(self, s, mask):  # tests/oracle.py:189-193
        acc = self.env[s.name]
        base = self.env[s.base] if s.base is not None else acc
        op = reduce_canon(s.op.name)
        self.bind(s.name, apply(op if op in _BINARY else "add", [base, self.env[s.value]], _NAME_OF[acc.dtype]), mask)

    def do_Select(self, s, mask):  # tests/oracle.py:195-200
        branches = list(s.branches)
        out = self.env[branches[-1].value].astype(np.float32)
        for br in reversed(branches[:-1]):
            out = np.where(_truth(self.ev(br.select)), self.env[br.value].astype(np.float32), out)
        self.bind(s.name, out, mask)

    def do_Smem(self, s, mask):  # tests/oracle.py:202-206
        if s.name not in self.shared:
            ctype = getattr(s, "dtype", None) or "float"
            extents = tuple(int(n) for n in s.extents)
            self.shared[s.name] = np.zeros((self.nb, math.prod(extents)), NP[C_TYPES.get(ctype, ctype)])
            self.shared_shape[s.name] = extents

    def do_Load(self, s, mask):  # tests/oracle.py:211-220
        idx = self.flat_index(self.extents_of(s.input), s.index)
        for k, name in enumerate(s.names):
            safe = np.where(mask, idx + k, 0)
            if s.input in self.shared:
                v = self.shared[s.input][self.row, safe]
            else:
                v = self.globals[s.input].reshape(-1)[safe]
            if s.dtype is not None:
                v = v.astype(NP[_name(s.dtype)])
            self.bind(name, v, mask)

    def do_Write(self, s, mask):  # tests/oracle.py:222-231
        idx = self.flat_index(self.extents_of(s.output), s.index)
        shared = s.output in self.shared
        mem = self.shared[s.output] if shared else self.globals[s.output].reshape(-1)
        if not shared and not self.globals[s.output].flags.c_contiguous:
            raise Unsupported("a global buffer that is not contiguous")
        for k, name in enumerate(s.values):
            v = self.env[name].astype(mem.dtype)
            where = (self.row[mask], idx[mask] + k) if shared else idx[mask] + k
            if s.atomic:
                np.add.at(mem, where, v[mask])
            else:
                mem[where] = v[mask]

    def do_Sync(self, s, mask):
        pass  # lockstep execution is a barrier after every statement

    def combine(self, program, mask):
        for a in program:
            self.do_Assign(a, mask)

    def do_WarpShuffle(self, s, mask):  # tests/oracle.py:238-245
        width = int(s.length) // 2
        while width:
            partner = self.tid ^ width
            for st, sb in zip(s.state, s.state_b):
                self.bind(sb, np.take_along_axis(self.env[st], partner, axis=1), mask)
            self.combine(s.combine_states, mask)
            width //= 2

    def do_TreeHalve(self, s, mask):  # tests/oracle.py:247-268
        bufs = [self.shared[b] if b in self.shared else None for b in s.bufs]
        if any(b is None for b in bufs):
            raise Unsupported("TreeHalve over a slab that is not shared memory")
        t = self.env[s.tid_var].astype(np.int64)
        if s.inner is not None:
            iv, scale = self.env[s.inner[0]].astype(np.int64), int(s.inner[1])
            slot = lambda k: k * scale + iv  # noqa: E731
        else:
            slot = lambda k: k  # noqa: E731
        half = int(s.length) // 2
        while half:
            active = mask & (t < half)
            mine, theirs = np.where(active, slot(t), 0), np.where(active, slot(t + half), 0)
            for st, sb, buf in zip(s.state, s.state_b, bufs):
                self.bind(st, buf[self.row, mine], active)
                self.bind(sb, buf[self.row, theirs], active)
            self.combine(s.combine_states, active)
            for st, buf in zip(s.state, bufs):
                buf[self.row[active], mine[active]] = self.env[st][active].astype(buf.dtype)
            half //= 2
        root = np.where(mask, slot(np.zeros(self.shape, np.int64)), 0)
        for st, buf in zip(s.state, bufs):
            self.bind(st, buf[self.row, root], mask)


def _expr_names(e) -> set:
    k = type(e).__name__
    if k == "Var":
        return {e.name}
    if k == "BinaryExpr":
        return _expr_names(e.left) | _expr_names(e.right)
    if k == "TernaryExpr":
        return _expr_names(e.cond) | _expr_names(e.if_true) | _expr_names(e.if_false)
    if k == "CastExpr":
        return _expr_names(e.expr)
    return set()


def _truth(v):
    return v if v.dtype == bool else v.astype(bool)


_EXPR_OPS = {"+": np.add, "-": np.subtract, "*": np.multiply, "/": np.divide, "<": np.less, "<=": np.less_equal,
             ">": np.greater, ">=": np.greater_equal, "==": np.equal, "!=": np.not_equal, "&&": np.logical_and,
             "||": np.logical_or, "&": np.bitwise_and, "|": np.bitwise_or, "^": np.bitwise_xor,
             "<<": np.left_shift, ">>": np.right_shift}


# ---------------------------------------------------------------- elementwise operations (tests/oracle.py:271-353)


def _in_double(fn):
    """A transcendental: computed in double, rounded once to the result type (tests/oracle.py:282-287)."""
    def f(t, *xs):
        with np.errstate(all="ignore"):
            return fn(*(np.asarray(x).astype(np.float64) for x in xs)).astype(t)
    return f


_erf = np.vectorize(math.erf, otypes=[np.float64])


def _is_float(a, b):
    return np.issubdtype(np.result_type(a, b), np.floating) or (
        ml_dtypes is not None and ml_dtypes.bfloat16 in (np.asarray(a).dtype, np.asarray(b).dtype))


def fmax(a, b):
    """CUDA's fmaxf on floats: a NaN gives the other operand and -0 < +0 (tests/oracle.py:294-299)."""
    if not _is_float(a, b):
        return np.maximum(a, b)
    r = np.fmax(a, b)
    both_zero = (a == 0) & (b == 0)
    return np.where(both_zero & ~(np.signbit(a) & np.signbit(b)), np.abs(r), r)


def fmin(a, b):
    """CUDA's fminf on floats (tests/oracle.py:302-307)."""
    if not _is_float(a, b):
        return np.minimum(a, b)
    r = np.fmin(a, b)
    both_zero = (a == 0) & (b == 0)
    return np.where(both_zero & (np.signbit(a) | np.signbit(b)), -np.abs(r), r)


def _decode_e4m3(t, code):
    """Extension: an e4m3 byte code to its value (emmy_ptx/elementwise.py:100-110; 0x7f and 0xff are NaN)."""
    if ml_dtypes is None:
        raise Unsupported("from_f8e4m3 needs ml_dtypes")
    byte = (np.asarray(code).astype(np.int64) & 0xFF).astype(np.uint8)
    return byte.view(ml_dtypes.float8_e4m3fn).astype(np.float32).astype(t)


_F8 = {"e4m3": ("float8_e4m3fn", 448.0), "e5m2": ("float8_e5m2", 57344.0)}


def _decode_f8(fmt):
    """Extension: ``from_f8<fmt>``, a byte code to its value, exactly (emmy_ptx/elementwise.py:100-110: e4m3's 0x7f / 0xff are
    NaN, e5m2's infinities and NaNs stay)."""
    def fn(t, code):
        if ml_dtypes is None:
            raise Unsupported("the fp8 operations need ml_dtypes")
        byte = (np.asarray(code).astype(np.int64) & 0xFF).astype(np.uint8)
        return byte.view(getattr(ml_dtypes, _F8[fmt][0])).astype(np.float32).astype(t)
    return fn


def _encode_f8(fmt):
    """Extension: ``to_f8<fmt>``, f32 to a byte code: round to nearest even, saturate to the largest finite value
    (infinities too), NaN to 0x7f (emmy_ptx/elementwise.py:113-123, one ``cvt.rn.satfinite``)."""
    def fn(t, x):
        if ml_dtypes is None:
            raise Unsupported("the fp8 operations need ml_dtypes")
        name, largest = _F8[fmt]
        x = np.asarray(x).astype(np.float32)
        codes = np.clip(x, -largest, largest).astype(getattr(ml_dtypes, name)).view(np.uint8)
        return np.where(np.isnan(x), np.uint8(0x7F), codes).astype(np.uint8)
    return fn


def _cast_then(fn):
    """A unary computed in the result type: convert the operand first, then apply ``fn``."""
    return lambda t, x: fn(x.astype(t), t)


# one-operand operations (tests/oracle.py:310-322): arithmetic ones in the result type, transcendental ones in double
_UNARY = {name: _cast_then(fn) for name, fn in {
    "negative": lambda v, t: np.negative(v),
    "abs": lambda v, t: np.abs(v),
    "copy": lambda v, t: v,
    "pad": lambda v, t: v,
    "square": lambda v, t: np.multiply(v, v),
    "reciprocal": lambda v, t: np.divide(t(1), v),
    "relu": lambda v, t: fmax(v, t(0)),
    "sqrt": lambda v, t: np.sqrt(v),
}.items()}
_UNARY.update({name: _in_double(fn) for name, fn in {
    "exp": np.exp, "log": np.log, "tanh": np.tanh, "sin": np.sin, "cos": np.cos, "erf": _erf,
    "sigmoid": lambda x: 1 / (1 + np.exp(-x)), "rsqrt": lambda x: 1 / np.sqrt(x),
}.items()})
_UNARY["bitwise_count"] = lambda t, x: np.bitwise_count(x).astype(t)
_UNARY["from_f8e4m3"] = _decode_e4m3  # extension
_UNARY["from_f8e5m2"] = _decode_f8("e5m2")  # extension
_UNARY["to_f8e4m3"], _UNARY["to_f8e5m2"] = _encode_f8("e4m3"), _encode_f8("e5m2")  # extensions

# two-operand operations (tests/oracle.py:323-328), computed on operands converted to the result type
_BINARY = dict(add=np.add, subtract=np.subtract, multiply=np.multiply, divide=np.divide, maximum=fmax, minimum=fmin,
               floor_divide=np.floor_divide, remainder=np.remainder, mod=np.remainder, left_shift=np.left_shift,
               right_shift=np.right_shift, bitwise_and=np.bitwise_and, bitwise_or=np.bitwise_or, bitwise_xor=np.bitwise_xor)
# operations emmy renders on integers only: for a bool result they are computed in i32, all others in f32 (:329-330)
_INTEGER_ONLY = frozenset("floor_divide remainder mod left_shift right_shift bitwise_xor bitwise_count".split())
# comparisons happen in the operands' common type; the result is the test's 0 or 1 (:331-332)
_COMPARE = dict(equal=np.equal, not_equal=np.not_equal, greater=np.greater, less=np.less, greater_equal=np.greater_equal,
                less_equal=np.less_equal)


def apply(op: str, args: list, out: str):
    """``op(*args)`` in result dtype ``out`` (tests/oracle.py:335-353)."""
    if out == "bool" and op not in _COMPARE:  # computed as a number, then converted as C converts to bool
        return apply(op, args, "i32" if op in _INTEGER_ONLY else "f32").astype(np.bool_)
    t = NP[out]
    with np.errstate(all="ignore"):
        if op in _COMPARE:
            return _COMPARE[op](*args).astype(t)
        if op == "where":
            return np.where(args[0].astype(bool), args[1].astype(t), args[2].astype(t))
        if op in _UNARY:
            return np.asarray(_UNARY[op](t, args[0])).astype(t)
        if op in _BINARY:
            return np.asarray(_BINARY[op](args[0].astype(t), args[1].astype(t))).astype(t)
        if op == "pow":
            return _in_double(np.power)(t, *args)
    raise Unsupported(f"elementwise op {op}")
