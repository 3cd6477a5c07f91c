"""A fragment-form schedule recognised as a matmul, and proved to be one, before it goes to the tcgen05 template.

emmy hands tensor-core kernels over as warp-level schedules: cp.async fills of swizzled shared slabs, ldmatrix,
mma.sync m16n8k16 on 16 x 8 tiles, RegStore (examples/m_f16_128/k_matmul__partial.ir.txt of the reference; its
lowering, emmy_ptx/tensorcore.py:165-452, keeps that schedule instruction for instruction). On sm_100a the
same product belongs on tcgen05 with TMA and tensor memory, whose tiling has nothing in common with the
schedule's. So the schedule is not translated; what it COMPUTES is established and handed to the template:

  1. The Tile's axes split into thread axes (inside a block) and block axes; every global index (cp.async source,
     global fragment load, RegStore target) must be ``sum(c_v * block axis v) + (an expression free of block
     axes)``, and block axes may appear nowhere else. Then block b does what block 0 does, shifted by the c_v.
  2. Block 0 is RUN, on provenance instead of numbers: every shared-memory element and fragment register carries
     (buffer, flat index) of the global element it holds, through the swizzles, the ldmatrix lane maps and the mma
     fragment layouts (PTX ISA, "Matrix Fragments for mma.m16n8k16"). Every mma must multiply A[m, k] with
     B[k, n] for one row m per accumulator row, one column n per accumulator column and the same k on both sides;
     every stored element C[s, m, n] must have accumulated exactly the products of row m and column n over each k
     of its slab once.
  3. The shifts of step 1 must move A's rows with C's rows, B's columns with C's columns, both operands' k with
     the slab index, and the blocks' tiles must cover C exactly once.

Anything else - guards, epilogues, atomics, fragments computed on, a shape the template does not take - is a
refusal with its reason, and the kernel runs on the statement path as its schedule says.
"""

from __future__ import annotations

import math

import numpy as np

from . import ir
from .families import Plan, Refusal, need, single_tile
from .ir import dtype_name, expr_vars, kind

C_ROW, C_COL = (0, 0, 1, 1), (0, 1, 0, 1)
SWIZZLE_MASK = {"B32": 1, "B64": 3, "B128": 7}
MAX_TRACE_MMAS = 1 << 18  # mma statements executed by block 0: bounds the work of the proof
MAX_BLOCKS = 1 << 22


def swizzled(e, mode):
    base, _, shift = (mode or "NONE").partition("@")
    mask = SWIZZLE_MASK.get(base)
    if mask is None:
        return e
    return e ^ (((e >> (int(shift) if shift else 6)) & mask) << 3)


# ---------------------------------------------------------------- step 1: block axes enter affinely


def block_coefficients(expr, block_axes: frozenset):
    """{block axis: coefficient} if ``expr`` is sum(c_v * v) + (something free of block axes); else None."""
    if not (expr_vars(expr) & block_axes):
        return {}
    k = kind(expr)
    if k == "Var":
        return {expr.name: 1}
    if k == "BinaryExpr" and expr.op == "+":
        a, b = block_coefficients(expr.left, block_axes), block_coefficients(expr.right, block_axes)
        if a is None or b is None:
            return None
        return {v: a.get(v, 0) + b.get(v, 0) for v in set(a) | set(b)}
    if k == "BinaryExpr" and expr.op == "*":
        for lit, other in ((expr.left, expr.right), (expr.right, expr.left)):
            if kind(lit) == "Literal" and isinstance(lit.value, int) and not isinstance(lit.value, bool):
                inner = block_coefficients(other, block_axes)
                return None if inner is None else {v: c * lit.value for v, c in inner.items()}
    return None


def exprs_of(value):
    """Every expression node reachable in a field value (tuples and (lo, hi) guards included)."""
    if isinstance(value, ir.Node):
        if kind(value) in ("Var", "Literal", "BinaryExpr", "TernaryExpr", "CastExpr"):
            yield value
    elif isinstance(value, (tuple, list)):
        for v in value:
            yield from exprs_of(v)


# ---------------------------------------------------------------- step 2: block 0 on provenance


class Trace:
    def __init__(self, src, thread_axes, block_axes, block: int):
        self.src, self.block, self.warps = src, block, block // 32
        tid = np.arange(block, dtype=np.int64)
        self.tid = tid
        lane = tid & 31
        self.g, self.t, self.warp_base = lane >> 2, lane & 3, tid - lane
        self.env = {"lane": lane, "warp": tid >> 5}
        stride = 1
        for axis, n in reversed(thread_axes):
            self.env[axis] = (tid // stride) % n
            stride *= n
        for axis, _ in block_axes:
            self.env[axis] = np.zeros(block, np.int64)
        self.names = list(src.buffers)  # buffer id = position
        self.smem: dict = {}  # name -> (shape, buffer ids, flat indices)
        self.frags: dict = {}  # name -> (role, buffer ids, flat indices), arrays (threads, members, registers, 2)
        self.acc: dict = {}  # (fragment, member) -> dict(rows, cols, ks, a, b)
        self.b_layouts = {"kn", "nk"}
        self.stores: list = []
        self.mmas = 0

    def ev(self, e):
        k = kind(e)
        if k == "Var":
            need(e.name in self.env, f"{e.name} is not an index the proof can follow")
            return self.env[e.name]
        if k == "Literal":
            need(isinstance(e.value, int) and not isinstance(e.value, bool), "a float in an index")
            return np.int64(e.value)
        if k == "BinaryExpr":
            a, b = self.ev(e.left), self.ev(e.right)
            if e.op == "+":
                return a + b
            if e.op == "-":
                return a - b
            if e.op == "*":
                return a * b
            if e.op in ("/", "%"):
                need(np.all(np.asarray(b) != 0), "a division by zero in an index")
                q = np.trunc(np.asarray(a) / np.asarray(b)).astype(np.int64)
                return q if e.op == "/" else a - q * b
            cmp = {"<": np.less, "<=": np.less_equal, ">": np.greater, ">=": np.greater_equal, "==": np.equal,
                   "!=": np.not_equal}.get(e.op)
            need(cmp is not None, f"operator {e.op} in an index")
            return cmp(a, b).astype(np.int64)
        if k == "TernaryExpr":
            return np.where(np.asarray(self.ev(e.cond)) != 0, self.ev(e.if_true), self.ev(e.if_false))
        raise Refusal(f"expression {k} in an index")

    def flat(self, shape, index):
        need(len(index) == len(shape), "an index with fewer coordinates than its buffer has dimensions")
        out = np.zeros(self.block, np.int64)
        for e, n in zip(index, shape):
            out = out * int(n) + self.ev(e)
        return out

    def member(self, ref):
        name, index = ir.fragment_ref(ref)
        need(name in self.frags, f"{ref} is not a declared fragment")
        if index is None:
            i = 0
        elif isinstance(index, int):
            i = index
        else:
            v = np.unique(np.asarray(self.ev(ir.Var(name=index))))
            need(len(v) == 1, f"fragment index {index} differs between threads")
            i = int(v[0])
        return name, i

    # statements

    def run(self, stmts):
        for s in stmts:
            fn = getattr(self, "t_" + kind(s), None)
            need(fn is not None, f"a {kind(s)} statement in the schedule")
            fn(s)

    def t_RegFragment(self, s):
        need(tuple(s.shape) == (16, 8, 16) and s.nregs is None, "a fragment that is not m16n8k16")
        if s.role == "c":
            need(dtype_name(s.dtype) == "f32", "an f16 accumulator")
            self.frags[s.name] = ("c", None, None)
            for i in range(int(s.count)):
                self.acc[(s.name, i)] = None
        else:
            shape = (self.block, int(s.count), {"a": 4, "b": 2}[s.role], 2)
            self.frags[s.name] = (s.role, np.full(shape, -1, np.int64), np.zeros(shape, np.int64))

    def t_Smem(self, s):
        n = math.prod(int(e) for e in s.extents)
        self.smem[s.name] = (tuple(int(e) for e in s.extents), np.full(n, -1, np.int64), np.zeros(n, np.int64))

    def t_CpAsyncCopy(self, s):
        need(s.smem in self.smem and s.src in self.src.buffers, "a cp.async that is not global to shared")
        shape, ids, flats = self.smem[s.smem]
        buf = self.src.buffers[s.src]
        dst = self.flat(shape, s.smem_index)
        if s.lane_index is not None:
            dst = dst + self.ev(s.lane_index[0]) * shape[-1] + self.ev(s.lane_index[1])
        dst = swizzled(dst, s.swizzle)
        src = self.flat(buf.shape, s.src_index)
        size = {"f16": 2, "bf16": 2}.get(buf.dtype)
        need(size is not None, f"a cp.async of {buf.dtype} elements")
        n = int(s.nbytes) // size
        need(dst.min() >= 0 and dst.max() + n <= len(ids), "a cp.async past the end of its slab")
        for j in range(n):
            ids[dst + j] = self.names.index(s.src)
            flats[dst + j] = src + j

    def t_CpAsyncCommit(self, s):
        pass

    t_CpAsyncWait = t_Sync = t_CpAsyncCommit

    def loop(self, s, values):
        for v in values:
            self.env[s.axis.name] = np.full(self.block, v, np.int64)
            self.run(s.body)

    def t_Loop(self, s):
        self.loop(s, range(int(s.axis.extent.as_static())))

    def t_StridedLoop(self, s):
        need(kind(s.start) == "Literal" and kind(s.step) == "Literal" and (s.end is None or kind(s.end) == "Literal"),
             "a loop whose bounds are not literals")
        end = int(s.end.value) if s.end is not None else int(s.axis.extent.as_static())
        need(int(s.step.value) > 0, "a loop that does not advance")
        self.loop(s, range(int(s.start.value), end, int(s.step.value)))

    def t_LdmatrixLoad(self, s):
        need(s.fragment_layout == "m16n8k16" and not s.byte_slab and s.scale_buffer is None, "an operand that is not 16-bit m16n8k16")
        name, i = self.member(s.frag)
        role, ids, flats = self.frags[name]
        need(role == s.role and role in ("a", "b"), "an operand load into an accumulator")
        lane = self.tid & 31
        low16, low8, half, bit3 = lane & 15, lane & 7, lane >> 4, (lane >> 3) & 1
        if not s.staged:
            need(s.gmem_guard is None and s.k_zero is None, "a guarded global fragment load")
            need(s.src_buffer in self.src.buffers, "a global fragment load from shared memory")
            buf = self.src.buffers[s.src_buffer]
            ldm = int(s.ldm) or int(buf.shape[-1])
            base, t2 = self.flat(buf.shape, s.src_index), 2 * self.t
            for reg in range(4 if role == "a" else 2):
                for h in (0, 1):
                    if role == "a":
                        at = (self.g + 8 * (reg & 1)) * ldm + t2 + 8 * (reg >> 1) + h
                    elif s.b_trans:
                        at = self.g * ldm + t2 + 8 * reg + h
                    else:
                        at = (t2 + 8 * reg + h) * ldm + self.g
                    ids[:, i, reg, h] = self.names.index(s.src_buffer)
                    flats[:, i, reg, h] = base + at
            return
        need(s.src_buffer in self.smem, "ldmatrix from something that is not a shared slab")
        shape, sids, sflats = self.smem[s.src_buffer]
        ldm = int(s.ldm) or shape[-1]
        dests = [(name, i, 0), (name, i, 1)]
        if s.pair_frag is not None:
            pname, pi = self.member(s.pair_frag)
            dests += [(pname, pi, 0), (pname, pi, 1)]
            trans, elem = (False, (low8 + half * 8) * ldm + 8 * bit3) if s.b_trans else (True, low16 * ldm + 8 * half)
        elif role == "a":
            trans, elem, dests = False, low16 * ldm + 8 * half, [(name, i, r) for r in range(4)]
        elif s.b_trans:
            trans, elem = False, low8 * ldm + 8 * bit3
        else:
            trans, elem = True, low16 * ldm
        addr = swizzled(self.flat(shape, s.src_index) + elem, s.swizzle)
        for m, (fname, fi, reg) in enumerate(dests):
            _, fids, fflats = self.frags[fname]
            for h in (0, 1):
                row_lane, col = (2 * self.t + h, self.g) if trans else (self.g, 2 * self.t + h)
                at = addr[self.warp_base + 8 * m + row_lane] + col
                need(at.min() >= 0 and at.max() < len(sids), "an ldmatrix row past the end of its slab")
                fids[:, fi, reg, h] = sids[at]
                fflats[:, fi, reg, h] = sflats[at]

    def operand(self, ref, role):
        """(buffer id, flat indices as per-warp matrices): A (warps, 16 m, 16 k), B (warps, 16 k, 8 n)."""
        name, i = self.member(ref)
        r, ids, flats = self.frags[name]
        need(r == role, f"{ref} is not a {role} operand")
        ids, flats = ids[:, i], flats[:, i]
        need(ids.min() >= 0 and ids.min() == ids.max(), "an operand register that holds nothing, or elements of two buffers")
        f = flats.reshape(self.warps, 8, 4, -1, 2)  # (warp, g, t, register, half)
        if role == "a":
            out = np.zeros((self.warps, 16, 16), np.int64)
            for reg in range(4):
                for h in (0, 1):
                    out[:, 8 * (reg & 1):8 * (reg & 1) + 8, 8 * (reg >> 1) + h:8 * (reg >> 1) + 8:2] = f[:, :, :, reg, h]
        else:
            out = np.zeros((self.warps, 16, 8), np.int64)
            for reg in range(2):
                for h in (0, 1):
                    out[:, 8 * reg + h:8 * reg + 8:2, :] = np.swapaxes(f[:, :, :, reg, h], 1, 2)
        return int(ids.min()), out

    def t_MmaSyncPtx(self, s):
        need(tuple(s.shape) == (16, 8, 16) and not s.block_scaled and not s.b_row_major and s.c_dtype == "f32"
             and s.ab_dtype in ("f16", "bf16"), "an mma that is not m16n8k16 row.col with an f32 accumulator")
        self.mmas += 1
        need(self.mmas <= MAX_TRACE_MMAS, "more mma steps per block than the proof follows")
        cname, ci = self.member(s.c_frag)
        need(self.frags[cname][0] == "c", f"{s.c_frag} is not an accumulator")
        a_id, a = self.operand(s.a_frag, "a")
        b_id, b = self.operand(s.b_frag, "b")
        A, B = self.src.buffers[self.names[a_id]], self.src.buffers[self.names[b_id]]
        need(len(A.shape) == 2 and len(B.shape) == 2, "an operand buffer that is not a matrix")
        rows, ks = np.divmod(a, int(A.shape[1]))
        need((rows == rows[:, :, :1]).all() and (ks == ks[:, :1, :]).all(), "an A operand that is not rows x consecutive k of one matrix")
        rows, ks = rows[:, :, 0], ks[:, 0, :]
        cols = None
        for layout in sorted(self.b_layouts):
            bk, bn = np.divmod(b, int(B.shape[1])) if layout == "kn" else np.divmod(b, int(B.shape[1]))[::-1]
            if (bk == ks[:, :, None]).all() and (bn == bn[:, :1, :]).all():
                cols = bn[:, 0, :]
            else:
                self.b_layouts = self.b_layouts - {layout}
        need(cols is not None and self.b_layouts, "a B operand whose k does not run with A's")
        state = self.acc[(cname, ci)]
        need(state != "stored", "an accumulator that is summed into again after it was stored")
        if state is None:
            self.acc[(cname, ci)] = dict(rows=rows, cols=cols, ks=[ks], a=a_id, b=b_id)
        else:
            need(state["a"] == a_id and state["b"] == b_id and (state["rows"] == rows).all() and (state["cols"] == cols).all(),
                 "an accumulator that sums products of different rows or columns")
            state["ks"].append(ks)

    def t_RegStore(self, s):
        need(s.epilogue is None and not s.extra_frags and s.m_guard is None and s.n_guard is None and not s.atomic
             and s.fragment_layout == "m16n8k16" and not s.volta_interleaved and (s.swizzle or "NONE") == "NONE",
             "a RegStore with an epilogue, a guard, an atomic add or a swizzle")
        need(s.dst_buffer in self.src.buffers and s.dst_buffer not in self.smem, "a RegStore into shared memory")
        cname, ci = self.member(s.frag)
        state = self.acc.get((cname, ci))
        need(state is not None and state != "stored", "a stored accumulator that no mma wrote, or one stored twice")
        shape = self.src.buffers[s.dst_buffer].shape
        ldm = int(s.ldm) or (math.prod(shape[s.row_dim + 1:]) if s.row_dim is not None else int(shape[-1]))
        ldn = math.prod(shape[s.col_dim + 1:]) if s.col_dim is not None else 1
        base = self.flat(shape, s.dst_index)
        dst = np.zeros((self.warps, 16, 8), np.int64)
        for i in range(4):
            at = (base + (self.g + 8 * C_ROW[i]) * ldm + (2 * self.t + C_COL[i]) * ldn).reshape(self.warps, 8, 4)
            dst[:, 8 * C_ROW[i]:8 * C_ROW[i] + 8, C_COL[i]::2] = at
        self.stores.append(dict(buffer=s.dst_buffer, dst=dst, **state))
        self.acc[(cname, ci)] = "stored"


# ---------------------------------------------------------------- the matcher


def match_fragment_matmul(src, strict: bool) -> Plan:
    from . import tcfamilies
    tile = single_tile(src)
    stmts = list(ir.walk(tile.body))
    need(any(kind(s) == "MmaSyncPtx" for s in stmts), "no mma statements")
    need(not strict, "the tensor cores sum a K-slice in their own order (--strict keeps the schedule's mma steps)")
    block, grid = src.launch.block, src.launch.grid
    need(block % 32 == 0 and not tile.aux_threads and tile.block_threads in (None, block), "a partial-block or banded Tile")
    need(not (tile.raster_axes and tile.raster_group is not None), "a rasterized Tile")

    # thread axes and block axes
    thread_axes, block_axes, stride = [], [], 1
    for axis in reversed(tile.axes):
        n = int(axis.extent.as_static())
        if stride * n <= block and block % (stride * n) == 0:
            thread_axes.insert(0, (axis.name, n))
        elif stride % block == 0:
            block_axes.insert(0, (axis.name, n))
        else:
            raise Refusal(f"axis {axis.name} straddles the block boundary")
        stride *= n
    need(math.prod(n for _, n in thread_axes) == block and math.prod(n for _, n in block_axes) == grid and grid <= MAX_BLOCKS,
         "the Tile's cells are not exactly the launch's threads")
    block_names = frozenset(a for a, _ in block_axes)

    # step 1
    global_index = {"CpAsyncCopy": "src_index", "RegStore": "dst_index"}
    coefficients: dict = {}  # buffer -> per dimension {axis: coefficient}
    for s in stmts:
        k = kind(s)
        field = global_index.get(k) or ("src_index" if k == "LdmatrixLoad" and not s.staged else None)
        for name, value in s.items():
            if name in ("body", "else_body"):
                continue
            if name == field:
                buffer = getattr(s, {"CpAsyncCopy": "src", "RegStore": "dst_buffer", "LdmatrixLoad": "src_buffer"}[k])
                dims = [block_coefficients(e, block_names) for e in value]
                need(all(d is not None for d in dims), f"a block axis enters the index of {buffer} other than as a multiple added on")
                dims = [{v: c for v, c in d.items() if c} for d in dims]
                need(coefficients.setdefault(buffer, dims) == dims, f"two accesses of {buffer} move differently with the block")
            else:
                for e in exprs_of(value):
                    need(not (expr_vars(e) & block_names), f"a block axis in the {name} of a {k}")

    # step 2
    trace = Trace(src, thread_axes, block_axes, block)
    trace.run(tile.body)
    need(trace.stores, "nothing is stored")
    need(all(v in (None, "stored") for v in trace.acc.values()), "an accumulator that is summed but never stored")
    outs = {st["buffer"] for st in trace.stores}
    a_ids, b_ids = {st["a"] for st in trace.stores}, {st["b"] for st in trace.stores}
    need(len(outs) == 1 and len(a_ids) == 1 and len(b_ids) == 1, "more than one product")
    out_name, a_name, b_name = outs.pop(), trace.names[a_ids.pop()], trace.names[b_ids.pop()]
    A, B, C = src.buffers[a_name], src.buffers[b_name], src.buffers[out_name]
    need(a_name not in src.written and b_name not in src.written, "the kernel writes an operand")
    need(len(trace.b_layouts) == 1, "B's layout is ambiguous")
    layout = next(iter(trace.b_layouts))
    M, K = (int(d) for d in A.shape)
    N = int(B.shape[1] if layout == "kn" else B.shape[0])
    need(int(B.shape[0] if layout == "kn" else B.shape[1]) == K, "A and B disagree about K")
    need(len(C.shape) in (2, 3) and tuple(C.shape[-2:]) == (M, N), "the output is not [M, N] or [slabs, M, N]")
    S = int(C.shape[0]) if len(C.shape) == 3 else 1
    need(K % S == 0, "K does not split evenly into the output's slabs")
    k_slab = K // S
    cells = {}
    for st in trace.stores:
        ks = np.concatenate(st["ks"], axis=1)  # (warps, every k this accumulator summed)
        need(ks.shape[1] == k_slab and (np.sort(ks, axis=1) == np.arange(k_slab)).all(),
             "an accumulator does not sum each k of its slab exactly once")
        flat = st["dst"]
        slab, rest = np.divmod(flat, M * N)
        row, col = np.divmod(rest, N)
        need((slab == 0).all() and (row == st["rows"][:, :, None]).all() and (col == st["cols"][:, None, :]).all(),
             "a product is stored somewhere other than C[row of A, column of B]")
        for r, c in zip(row.reshape(-1).tolist(), col.reshape(-1).tolist()):
            need((r, c) not in cells, "an output element is stored twice")
            cells[(r, c)] = True
    tile_m, tile_n = 1 + max(r for r, _ in cells), 1 + max(c for _, c in cells)
    need(len(cells) == tile_m * tile_n, "a block's output is not a full rectangle")

    # step 3
    def moves(buffer, dim, axis):
        return coefficients.get(buffer, [{}] * 8)[dim].get(axis, 0)

    a_row, a_k = 0, 1
    b_k, b_n = (0, 1) if layout == "kn" else (1, 0)
    c_dims = len(C.shape)
    offsets = np.zeros((grid, 3), np.int64)
    ids = np.arange(grid, dtype=np.int64)
    stride = grid
    for axis, n in block_axes:
        stride //= n
        value = (ids // stride) % n
        cm, cn = moves(out_name, c_dims - 2, axis), moves(out_name, c_dims - 1, axis)
        cs = moves(out_name, 0, axis) if c_dims == 3 else 0
        need(moves(a_name, a_row, axis) == cm and moves(b_name, b_n, axis) == cn, f"block axis {axis} moves an operand and the output differently")
        need(moves(a_name, a_k, axis) == moves(b_name, b_k, axis) == cs * k_slab, f"block axis {axis} moves k differently from the output's slab")
        offsets += value[:, None] * np.array([cs, cm, cn], np.int64)
    need(M % tile_m == 0 and N % tile_n == 0, "the block tiles do not divide the output")
    want = np.stack(np.meshgrid(np.arange(S), np.arange(0, M, tile_m), np.arange(0, N, tile_n), indexing="ij"), -1).reshape(-1, 3)
    seen = np.unique(offsets, axis=0)  # sorted by slab, then row, then column, as ``want`` is
    need(len(want) == grid and seen.shape == want.shape and (seen == want).all(), "the blocks do not cover the output exactly once")

    # the template
    need(A.dtype == B.dtype and A.dtype in ("f16", "bf16"), "the operands are not both f16 or both bf16")
    need(C.dtype == "f32" or C.dtype == A.dtype, "the output is neither f32 nor the operands' type")
    need(K % 8 == 0 and (layout == "nk" or N % 8 == 0), "an operand's row stride is not a multiple of 16 bytes")
    need(S == 1 or k_slab % 64 == 0, "K slabs that are not multiples of 64")
    need(M * N >= 128 * 256 // 4, "too small for a 128 x 256 tensor-core tile")
    bf16 = A.dtype == "bf16"
    tiles = math.ceil(M / 128) * math.ceil(N / 256) * S
    grid_t = min(tcfamilies.TARGET_SMS, tiles)
    stage = (128 + 256) * 128
    smem = tcfamilies.GEMM_STAGES * stage + 1024 + 256
    flags = f"{str(bf16).lower()}, emb::EPI_NONE, false, {str(layout == 'kn').lower()}, {str(C.dtype == 'f32').lower()}"
    call = [f"    emb::gemm_tn_kernel<{tcfamilies.GEMM_STAGES}, {tcfamilies.GEMM_GROUP_M}, {flags}>(&tmap_a, &tmap_b, p_{out_name}, "
            f"emb::GemmShape{{{M}, {N}, {K}, {S}}}, status);"]
    extra_sig = ["const __grid_constant__ CUtensorMap tmap_a", "const __grid_constant__ CUtensorMap tmap_b", "unsigned* __restrict__ status"]
    source = tcfamilies.wrapper(src, '#include "emb_gemm.cuh"', call, extra_sig, 192)
    b_map = (tcfamilies.tmap("b", b_name, B.dtype, (N, K), (N * 2,), (64, 64)) if layout == "kn"
             else tcfamilies.tmap("b", b_name, B.dtype, (K, N), (K * 2,), (64, 256)))
    extra = [tcfamilies.tmap("a", a_name, A.dtype, (K, M), (K * 2,), (64, 128)), b_map, dict(kind="status", name="status")]
    slabs = f" in {S} K-slabs of {k_slab}" if S > 1 else ""
    remarks = [f"fragment-form schedule proved to be {out_name} = {a_name} [{M} x {K}] times {b_name} "
               f"[{'K x N' if layout == 'kn' else 'N x K'}, N = {N}]{slabs}: {trace.mmas} mma.sync steps of block 0 followed on "
               f"provenance, {grid} blocks of {tile_m} x {tile_n} cover the output once",
               f"tensor-core matmul template instead of the schedule: {tiles} tiles of 128 x 256 on {grid_t} persistent CTAs "
               f"(TMA, tcgen05.mma, f32 accumulation in tensor memory){', B read through an MN-major descriptor' if layout == 'kn' else ''}"
               f"{', f32 partial slabs out' if C.dtype == 'f32' else ''}"]
    return Plan("tensorcore", source, remarks, grid=grid_t, block=192, smem_bytes=smem, extra_params=extra)
