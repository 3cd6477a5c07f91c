"""TEST INFRASTRUCTURE, NOT PRODUCT: the oracle extended to emmy's tensor-core (fragment) form.

Only the tests and the CPU-baseline legs of ``bench.py`` may import this module; no product code path may.

The reference's interpreter (tests/oracle.py) refuses the fragment statements, so its own check of a
fragment-form kernel is the example's ``expected.npz`` alone (examples/m_f16_128). What is restated here
instead is the meaning the reference's LOWERING gives each statement, on the lane maps of the PTX ISA's
"Matrix Fragments for mma.m16n8k16" that it follows:

  * RegFragment, LdmatrixLoad (shared slab with ``ldmatrix`` x4 / x2 / .trans, or the global-memory loader
    with its clamp and zero fill), MmaSyncPtx, FragmentApply / RowReduce / Repack / Promote, RegStore:
    emmy_ptx/tensorcore.py:147-452
  * CpAsyncCopy, CpAsyncCommit, CpAsyncWait: emmy_ptx/lower.py:1057-1102; the XOR swizzle of a slab index
    ``e ^ (((e >> shift) & mask) << 3)``: emmy_ptx/lower.py:1538-1553

An EXTENSION of the oracle, stated as such wherever results are reported. Parity pin: the shipped fragment-form
example against its ``expected.npz`` (tests/golden/), at the example's own rtol = atol = 1e-2; nothing pins
it more tightly, because the order in which an mma sums its 16 products is the hardware's. Here an mma is
``round_f32(c + sum of the exact products in float64)``.

Asynchronous copies complete where they are issued: the kernels this form comes from wait for a copy
group and pass a barrier before any thread reads what it brought, so lockstep execution sees the same data.
"""

from __future__ import annotations

import math

import numpy as np

from . import ir_oracle
from .ir_oracle import NP, C_TYPES, Unsupported, _Blocks, _name, apply

# element i of a lane's C fragment: row g + 8 * C_ROW[i], column 2t + C_COL[i] (g = lane / 4, t = lane % 4)
C_ROW, C_COL = (0, 0, 1, 1), (0, 1, 0, 1)
SWIZZLE_MASK = {"B32": 1, "B64": 3, "B128": 7}


def run(body, buffers: dict, grid: int, block: int, blocks=None, batch: int | None = None) -> dict:
    """ir_oracle.run for bodies that may hold fragment statements."""
    ids = np.arange(grid, dtype=np.int64) if blocks is None else np.asarray(sorted(blocks), np.int64)
    batch = batch or max(1, (1 << 16) // max(1, block))
    for lo in range(0, len(ids), batch):
        _FragmentBlocks(buffers, ids[lo:lo + batch], block).run(body)
    return buffers


def swizzled(e, mode: str):
    base, _, shift = (mode or "NONE").partition("@")
    mask = SWIZZLE_MASK.get(base)
    if mask is None:
        return e
    return e ^ (((e >> (int(shift) if shift else 6)) & mask) << 3)


def _ref(ref: str):
    if ref.endswith("]") and "[" in ref:
        name, _, index = ref[:-1].partition("[")
        return name, index
    return ref, None


class _FragmentBlocks(_Blocks):
    def __init__(self, globals_, ctaids, block):
        super().__init__(globals_, ctaids, block)
        if block % 32:
            raise Unsupported("fragment statements need whole warps")
        self.frags: dict = {}  # name -> (role, element dtype name, array (blocks, threads, count, regs[, 2]))
        lane = self.tid & 31
        self.g, self.t = lane >> 2, lane & 3
        self.warp_base = self.tid - lane

    # a Tile with raster axes but no raster group is not rasterised (the reference's cells.py needs both)
    def do_Tile(self, s, mask):
        if getattr(s, "raster_group", None) is None and s.raster_axes:
            s = s.replace(raster_axes=None)
        super().do_Tile(s, mask)

    # ------------------------------------------------------------ fragments

    def member(self, ref: str):
        name, index = _ref(ref)
        role, dt, data = self.frags[name]
        if index is None:
            i = 0
        elif index.isdigit():
            i = int(index)
        else:
            v = np.unique(self.env[index])
            if len(v) != 1:
                raise Unsupported(f"fragment index {index} differs between threads")
            i = int(v[0])
        return role, dt, data[:, :, i]

    def do_RegFragment(self, s, mask):  # tensorcore.py:147-161
        if tuple(s.shape) != (16, 8, 16):
            raise Unsupported("only m16n8k16 fragments")
        dt = _name(s.dtype)
        if s.role == "c":
            regs = (4,) if dt == "f32" else (2, 2)
        else:
            regs = ({"a": 4, "b": 2}[s.role], 2)
        self.frags[s.name] = (s.role, dt, np.zeros(self.shape + (int(s.count),) + regs, NP[dt]))

    # ------------------------------------------------------------ copies

    def do_CpAsyncCopy(self, s, mask):  # lower.py:1057-1083
        smem = self.shared[s.smem]
        shape = self.shared_shape[s.smem]
        dst = self.flat_index(shape, s.smem_index)
        if s.lane_index is not None:
            row, col = (self.ev(e).astype(np.int64) for e in s.lane_index)
            dst = dst + row * int(shape[-1]) + col
        dst = swizzled(dst, s.swizzle)
        src = self.flat_index(self.globals[s.src].shape, s.src_index)
        flat = self.globals[s.src].reshape(-1)
        n = int(s.nbytes) // flat.dtype.itemsize
        rows = self.row[mask]
        for j in range(n):
            smem[rows, dst[mask] + j] = flat[src[mask] + j]

    def do_CpAsyncCommit(self, s, mask):
        pass

    def do_CpAsyncWait(self, s, mask):
        pass

    # ------------------------------------------------------------ operands

    def do_LdmatrixLoad(self, s, mask):  # tensorcore.py:165-208
        if s.fragment_layout != "m16n8k16" or s.byte_slab or s.scale_buffer is not None:
            raise Unsupported("only 16-bit m16n8k16 operands")
        if not s.staged:
            return self.fragment_from_global(s, mask)
        slab, shape = self.shared[s.src_buffer], self.shared_shape[s.src_buffer]
        ldm = int(s.ldm) or int(shape[-1])
        lane = self.tid & 31
        low16, low8, half, bit3 = lane & 15, lane & 7, lane >> 4, (lane >> 3) & 1
        dests = [(s.frag, 0), (s.frag, 1)]
        if s.pair_frag is not None:
            dests += [(s.pair_frag, 0), (s.pair_frag, 1)]
            if s.b_trans:
                trans, elem = False, (low8 + half * 8) * ldm + 8 * bit3
            else:
                trans, elem = True, low16 * ldm + 8 * half
        elif s.role == "a":
            trans, elem, dests = False, low16 * ldm + 8 * half, [(s.frag, i) for i in range(4)]
        elif s.b_trans:
            trans, elem = False, low8 * ldm + 8 * bit3
        else:
            trans, elem = True, low16 * ldm
        addr = swizzled(self.flat_index(shape, s.src_index) + elem, s.swizzle)  # each lane's 16-byte row
        for m, (ref, reg) in enumerate(dests):  # matrix m: its eight rows come from lanes 8m .. 8m + 7
            _, _, data = self.member(ref)
            for h in (0, 1):
                if trans:  # register = matrix[2t + h][g]
                    row_lane, col = 2 * self.t + h, self.g
                else:  # register = matrix[g][2t + h]
                    row_lane, col = self.g, 2 * self.t + h
                row_addr = np.take_along_axis(addr, self.warp_base + 8 * m + row_lane, axis=1)
                v = slab[self.row, np.where(mask, row_addr + col, 0)]
                data[:, :, reg, h] = np.where(mask, v, data[:, :, reg, h])

    def fragment_from_global(self, s, mask):  # tensorcore.py:210-262
        buf = self.globals[s.src_buffer]
        flat = buf.reshape(-1)
        ldm = int(s.ldm) or int(buf.shape[-1])
        base = self.flat_index(buf.shape, s.src_index)
        _, dt, data = self.member(s.frag)

        def left(guard):
            return None if guard is None else (self.ev(guard[1]) - self.ev(guard[0])).astype(np.int64)

        lanes_left, k_left = left(s.gmem_guard), left(s.k_zero)

        def clamp(x):
            return x if lanes_left is None else np.minimum(x, np.maximum(lanes_left - 1, 0))

        t2 = 2 * self.t
        pairs = []
        if s.role == "a":
            for i in range(4):
                r, k = clamp(self.g + 8 * (i & 1)), t2 + 8 * (i >> 1)
                pairs.append(((r * ldm + k, k), (r * ldm + k + 1, k + 1)))
        else:
            n = clamp(self.g)
            for i in range(2):
                k = t2 + 8 * i
                if s.b_trans:
                    pairs.append(((n * ldm + k, k), (n * ldm + k + 1, k + 1)))
                else:
                    pairs.append(((k * ldm + n, k), ((k + 1) * ldm + n, k + 1)))
        for reg, halves in enumerate(pairs):
            for h, (at, k) in enumerate(halves):
                live = mask if k_left is None else mask & (k < k_left)  # an element past a masked K is zero, never read
                v = np.where(live, flat[np.where(live, base + at, 0)].astype(NP[dt]), np.zeros((), NP[dt]))
                data[:, :, reg, h] = np.where(mask, v, data[:, :, reg, h])

    # ------------------------------------------------------------ the mma

    def warp_tiles(self, frag, role):
        """A fragment as per-warp matrices in float64: (blocks, warps, rows, cols)."""
        nb, nw = self.nb, self.block // 32
        f = frag.astype(np.float64).reshape((nb, nw, 8, 4) + frag.shape[2:])  # (.., g, t, regs[, halves])
        if role == "a":  # A[g + 8 (i & 1), 2t + h + 8 (i >> 1)]
            out = np.zeros((nb, nw, 16, 16))
            for i in range(4):
                for h in (0, 1):
                    out[:, :, 8 * (i & 1):8 * (i & 1) + 8, 8 * (i >> 1) + h:8 * (i >> 1) + 8:2] = f[..., i, h]
            return out
        if role == "b":  # B[2t + h + 8 i, g]
            out = np.zeros((nb, nw, 16, 8))
            for i in range(2):
                for h in (0, 1):
                    out[:, :, 8 * i + h:8 * i + 8:2, :] = np.swapaxes(f[..., i, h], 2, 3)
            return out
        out = np.zeros((nb, nw, 16, 8))  # C[g + 8 C_ROW[i], 2t + C_COL[i]]
        c = f.reshape(f.shape[:4] + (4,))
        for i in range(4):
            out[:, :, 8 * C_ROW[i]:8 * C_ROW[i] + 8, C_COL[i]::2] = c[..., i]
        return out

    def do_MmaSyncPtx(self, s, mask):  # tensorcore.py:274-292
        if tuple(s.shape) != (16, 8, 16) or s.block_scaled or s.b_row_major or s.ab_dtype not in ("f16", "bf16"):
            raise Unsupported("only m16n8k16 f16 / bf16 row.col")
        if not mask.all():
            raise Unsupported("an mma under a mask")
        (_, cdt, c), (_, _, a), (_, _, b) = (self.member(r) for r in (s.c_frag, s.a_frag, s.b_frag))
        d = self.warp_tiles(a, "a") @ self.warp_tiles(b, "b") + self.warp_tiles(c, "c")
        d = d.astype(np.float32)
        nb, nw = self.nb, self.block // 32
        lanes = np.zeros((nb, nw, 8, 4, 4), np.float32)
        for i in range(4):
            lanes[..., i] = d[:, :, 8 * C_ROW[i]:8 * C_ROW[i] + 8, C_COL[i]::2]
        c[...] = lanes.reshape(c.shape if cdt == "f32" else (nb, self.block, 4)).astype(NP[cdt]).reshape(c.shape)

    # ------------------------------------------------------------ C-fragment arithmetic

    def c_elements(self, ref):
        _, dt, data = self.member(ref)
        if dt != "f32":
            raise Unsupported("arithmetic on an f16 accumulator")
        return data

    def do_FragmentApply(self, s, mask):  # tensorcore.py:296-318,326-350
        values = []
        for i in range(4):
            saved = {n: self.env.get(n) for n in ("__frow", "__fcol")}
            if s.row_base is not None:
                self.env["__frow"] = (self.ev(s.row_base) + self.g + 8 * C_ROW[i]).astype(np.int64)
            if s.col_base is not None:
                self.env["__fcol"] = (self.ev(s.col_base) + 2 * self.t + C_COL[i]).astype(np.int64)
            args = []
            for a, k in zip(s.args, s.kinds):
                if k == "frag":
                    args.append(self.c_elements(a)[:, :, i])
                elif k == "row":
                    args.append(self.env[a[C_ROW[i]]])
                elif k == "uniform":
                    args.append(self.env[a] if isinstance(a, str) else self.ev(a).astype(np.float32))
                elif k == "coord":
                    args.append(ir_oracle._truth(self.ev(a)))
                elif k == "gmem":
                    name, index = a
                    g = self.globals[name]
                    args.append(g.reshape(-1)[np.where(mask, self.flat_index(g.shape, index), 0)].astype(np.float32))
                else:
                    raise Unsupported(f"operand kind {k}")
            v = apply(s.op.name, args, "f32")
            for post in s.post:
                v = apply(post.name, [v], "f32")
            values.append(v)
            for n, old in saved.items():
                if old is None:
                    self.env.pop(n, None)
                else:
                    self.env[n] = old
        if s.in_place:
            data = self.c_elements(s.out)
            for i, v in enumerate(values):
                data[:, :, i] = np.where(mask, v, data[:, :, i])
        else:
            self.frags[s.out] = ("c", "f32", np.stack(values, axis=-1)[:, :, None, :].astype(np.float32))

    def do_FragmentRowReduce(self, s, mask):  # tensorcore.py:352-369
        frags = [self.c_elements(f) for f in s.frags]
        rows = []
        for r in (0, 1):
            parts = [f[:, :, i] for f in frags for i in range(4) if C_ROW[i] == r]
            acc = parts[0]
            for p in parts[1:]:
                acc = apply(s.op.name, [acc, p], "f32")
            rows.append(acc)
        xors = tuple(getattr(s.layout, "reduce_xors", None) or (1, 2))
        for distance in xors:
            for r in (0, 1):
                other = np.take_along_axis(rows[r], self.tid ^ int(distance), axis=1)
                rows[r] = apply(s.op.name, [rows[r], other], "f32")
        self.bind(s.top, rows[0], mask)
        self.bind(s.bot, rows[1], mask)

    def do_FragmentRepack(self, s, mask):  # tensorcore.py:371-378
        c0, c1 = (self.c_elements(x) for x in s.srcs)
        _, dt, data = self.member(s.frag)
        for reg, (src, lo) in enumerate(((c0, 0), (c0, 2), (c1, 0), (c1, 2))):
            for h in (0, 1):
                data[:, :, reg, h] = np.where(mask, src[:, :, lo + h].astype(NP[dt]), data[:, :, reg, h])

    def do_FragmentPromote(self, s, mask):  # tensorcore.py:380-390
        dst = self.c_elements(s.dst)
        _, dt, src = self.member(s.src)
        if dt == "f32":
            raise Unsupported("FragmentPromote of an f32 accumulator")
        for i in range(2):
            for j in range(2):
                k = 2 * i + j
                dst[:, :, k] = np.where(mask, dst[:, :, k] + src[:, :, i, j].astype(np.float32), dst[:, :, k])
        src[...] = np.where(mask[:, :, None, None], np.zeros((), src.dtype), src)

    # ------------------------------------------------------------ the store

    def do_RegStore(self, s, mask):  # tensorcore.py:394-452
        if s.fragment_layout != "m16n8k16" or s.volta_interleaved:
            raise Unsupported("only m16n8k16 fragments")
        shared = s.dst_buffer in self.shared
        shape = self.shared_shape[s.dst_buffer] if shared else self.globals[s.dst_buffer].shape
        mem = self.shared[s.dst_buffer] if shared else self.globals[s.dst_buffer].reshape(-1)
        ldm = int(s.ldm) or (math.prod(shape[s.row_dim + 1:]) if s.row_dim is not None else int(shape[-1]))
        ldn = math.prod(shape[s.col_dim + 1:]) if s.col_dim is not None else 1
        base = self.flat_index(shape, s.dst_index)
        frags = [self.member(s.frag)] + [self.member(x) for x in s.extra_frags]
        for i in range(4):
            row, col = self.g + 8 * C_ROW[i], 2 * self.t + C_COL[i]

            def element(f):
                _, dt, data = f
                return data[:, :, i] if dt == "f32" else data[:, :, i // 2, i % 2]

            if s.epilogue is None:
                v = element(frags[0])
            else:
                epi = s.epilogue
                for param, f in zip(epi.params, frags):
                    self.env[param] = element(f).astype(np.float32)
                self.env["__M__"], self.env["__N__"] = row.astype(np.int64), col.astype(np.int64)
                self.run(tuple(epi.body), mask)
                v = self.env[epi.results[0]]
            ok = mask.copy()
            for guard, coord in ((s.m_guard, row), (s.n_guard, col)):
                if guard is not None:
                    ok &= (self.ev(guard[0]) + coord) < self.ev(guard[1])
            at = swizzled(base + row * ldm + col * ldn, s.swizzle)
            where = (self.row[ok], at[ok]) if shared else at[ok]
            out = v.astype(np.float32).astype(mem.dtype)
            if s.atomic:
                np.add.at(mem, where, out[ok])
            else:
                mem[where] = out[ok]

    def do_ZeroPrologue(self, s, mask):  # lower.py:1240-1259: CTA 0 zeroes 32-bit words of another kernel's accumulator
        if (self.ctaid == 0).any():
            flat = self.globals[s.dst].reshape(-1)
            flat.view(np.uint8)[:4 * int(s.words)] = 0

    def do_Smem(self, s, mask):
        if s.name not in self.shared:
            ctype = getattr(s, "dtype", None) or "float"
            extents = tuple(int(n) for n in s.extents)
            # room for a swizzled index, which stays inside the slab's power-of-two span
            self.shared[s.name] = np.zeros((self.nb, math.prod(extents)), NP[C_TYPES.get(ctype, ctype)])
            self.shared_shape[s.name] = extents
