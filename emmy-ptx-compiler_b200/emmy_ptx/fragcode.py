"""Statement rules for the IR's tensor-core (fragment) form, mixed into ``codegen.Emitter``.

The statement-by-statement path for emmy's warp-level statements: every statement becomes the instruction
the reference lowers it to (emmy_ptx/tensorcore.py:147-452 for RegFragment, LdmatrixLoad, MmaSyncPtx,
FragmentApply / RowReduce / Repack / Promote and RegStore; emmy_ptx/lower.py:1057-1102 for the asynchronous
copies), written as CUDA C++ around inline PTX (csrc/templates/emb_frag.cuh), so a fragment-form kernel runs
exactly as its schedule says. ``fragmatch`` sends the schedules it can prove to be matmuls to the tcgen05
template instead; this path is what --plain and --strict get, and every schedule that is not recognised.

A fragment is a register array ``f_<name>[count][registers]``: four (A) or two (B) 32-bit registers of two
16-bit elements, four floats for an f32 accumulator, two packed registers for an f16 one. ``name[i]`` with i
a loop variable is resolved by the C++ compiler once the loop is unrolled, as the reference unrolls such loops
whatever their size.
"""

from __future__ import annotations

import math

from . import ir
from .ir import dtype_name, kind

C_ROW, C_COL = (0, 0, 1, 1), (0, 1, 0, 1)  # element i of a lane's C fragment: row g + 8 C_ROW[i], column 2t + C_COL[i]
SWIZZLE_MASK = {"B32": 1, "B64": 3, "B128": 7}
WARP_WIDE = ("LdmatrixLoad", "MmaSyncPtx", "FragmentRowReduce")  # need every lane of the warp


class FragmentStatements:
    """Needs the host class's emit / expr / flat / memory / use / var / apply / convert / block and CodegenError."""

    def fragment_error(self, text: str):
        from .codegen import CodegenError
        return CodegenError(text)

    def swz(self, code: str, mode) -> str:
        base, _, shift = (mode or "NONE").partition("@")
        mask = SWIZZLE_MASK.get(base)
        if mask is None:
            return code
        return f"emb::frag::swizzle<{int(shift) if shift else 6}, {mask}>({code})"

    def member(self, ref: str) -> tuple:
        """(C text of the member's register array, role, element dtype, registers)"""
        name, index = ir.fragment_ref(ref)
        if name not in self.frags:
            raise self.fragment_error(f"{ref!r} is not a declared fragment")
        role, dt, count, n = self.frags[name]
        if index is None:
            i = "0"
        elif isinstance(index, int):
            if index >= count:
                raise self.fragment_error(f"{ref!r}: the fragment has {count} members")
            i = str(index)
        else:
            i = f"(int){self.use(index)[0]}"
        return f"f_{name}[{i}]", role, dt, n

    def whole_warps(self, guard, what: str) -> None:
        if guard is not None:
            raise self.fragment_error(f"{what} under a condition that differs between threads")

    # ------------------------------------------------------------ declaration

    def s_RegFragment(self, s) -> None:
        if tuple(s.shape) != (16, 8, 16):
            raise self.fragment_error(f"RegFragment {s.name}: shape {s.shape} (only m16n8k16)")
        dt = dtype_name(s.dtype)
        wide = s.role == "c" and dt == "f32"
        n = s.nregs if s.nregs is not None else {"a": 4, "b": 2, "c": 4 if wide else 2}[s.role]
        if n == 0:
            raise self.fragment_error(f"RegFragment {s.name}: block-scale registers")
        if s.name not in self.frags:
            self.frag_decls.append(f"    {'float' if wide else 'uint32_t'} f_{s.name}[{int(s.count)}][{n}];")
        self.frags[s.name] = (s.role, dt, int(s.count), n)
        if s.role == "c":  # an accumulator starts at zero
            self.emit("#pragma unroll")
            self.emit(f"for (int i_ = 0; i_ < {int(s.count) * n}; ++i_) (&f_{s.name}[0][0])[i_] = 0;")

    # ------------------------------------------------------------ asynchronous copies

    def s_CpAsyncCopy(self, s) -> None:
        arr, dt, shape, shared, _ = self.memory(s.smem)
        src, sdt, sshape, sshared, _ = self.memory(s.src)
        if not shared or sshared:
            raise self.fragment_error("cp.async must copy from a global buffer into a shared array")
        if int(s.nbytes) not in (4, 8, 16):
            raise self.fragment_error(f"cp.async of {s.nbytes} bytes")
        dst = self.flat(shape, s.smem_index)
        if s.lane_index is not None:
            (row, _), (col, _) = (self.expr(e) for e in s.lane_index)
            dst = f"({dst} + (long long)({row}) * {int(shape[-1])}LL + (long long)({col}))"
        self.emit(f"emb::frag::cp_async<{int(s.nbytes)}>(&{arr}[{self.swz(dst, s.swizzle)}], &{src}[{self.flat(sshape, s.src_index)}]);")

    def s_CpAsyncCommit(self, s) -> None:
        self.emit("emb::frag::cp_async_commit();")

    def s_CpAsyncWait(self, s) -> None:
        self.emit(f"emb::frag::cp_async_wait<{int(s.group)}>();")

    # ------------------------------------------------------------ operands

    def x_LdmatrixLoad(self, s, guard) -> None:
        if s.fragment_layout != "m16n8k16" or s.byte_slab or s.scale_buffer is not None:
            raise self.fragment_error("LdmatrixLoad: only 16-bit m16n8k16 operands")
        if not s.staged:
            return self.fragment_from_global(s, guard)
        self.whole_warps(guard, "ldmatrix")
        arr, dt, shape, shared, _ = self.memory(s.src_buffer)
        if not shared:
            raise self.fragment_error(f"ldmatrix reads shared memory, not {s.src_buffer!r}")
        ldm = int(s.ldm) or int(shape[-1])
        lane = "(long long)v_lane"
        low16, low8, half, bit3 = f"({lane} & 15)", f"({lane} & 7)", f"({lane} >> 4)", f"(({lane} >> 3) & 1)"
        f, _, _, _ = self.member(s.frag)
        if s.pair_frag is not None:  # two B fragments side by side in one x4
            p, _, _, _ = self.member(s.pair_frag)
            dests = [f"{f}[0]", f"{f}[1]", f"{p}[0]", f"{p}[1]"]
            if s.b_trans:  # an N x K slab
                op, elem = "x4", f"(({low8} + {half} * 8) * {ldm}LL + {bit3} * 8)"
            else:  # a K x N slab, transposed on the way; the second fragment 8 columns on
                op, elem = "x4_trans", f"({low16} * {ldm}LL + {half} * 8)"
        elif s.role == "a":
            op, elem, dests = "x4", f"({low16} * {ldm}LL + {half} * 8)", [f"{f}[{i}]" for i in range(4)]
        elif s.b_trans:
            op, elem, dests = "x2", f"({low8} * {ldm}LL + {bit3} * 8)", [f"{f}[0]", f"{f}[1]"]
        else:
            op, elem, dests = "x2_trans", f"({low16} * {ldm}LL)", [f"{f}[0]", f"{f}[1]"]
        addr = self.swz(f"({self.flat(shape, s.src_index)} + {elem})", s.swizzle)
        self.emit(f"emb::frag::ldmatrix_{op}({', '.join(dests)}, &{arr}[{addr}]);")

    def fragment_from_global(self, s, guard) -> None:
        """Each lane reads its own elements of the A (16 x 16) or B (16 x 8) tile in the lane map ldmatrix would
        give and packs them in pairs; a masked tile clamps the lane's row (A) or column (B) into range, elements
        past a masked K are zero (emmy_ptx/tensorcore.py:210-262)."""
        arr, dt, shape, shared, _ = self.memory(s.src_buffer)
        f, _, fdt, n = self.member(s.frag)
        if dt != fdt and fdt != "f16":
            raise self.fragment_error(f"a {dt} element cannot fill a {fdt} fragment")
        ldm = int(s.ldm) or int(shape[-1])
        self.emit(f"if ({guard or 'true'}) {{")
        self.depth += 1
        self.emit(f"const long long base_ = {self.flat(shape, s.src_index)};")
        self.emit("const long long g_ = v_lane >> 2, t2_ = (v_lane & 3) * 2;")

        def left(guard_, name):
            if guard_ is None:
                return None
            (lo, _), (hi, _) = self.expr(guard_[0]), self.expr(guard_[1])
            self.emit(f"const long long {name} = (long long)({hi}) - (long long)({lo});")
            return name

        lanes_left, k_left = left(s.gmem_guard, "lanes_left_"), left(s.k_zero, "k_left_")

        def clamp(x):
            return x if lanes_left is None else f"min({x}, max({lanes_left} - 1, 0LL))"

        pairs = []
        if s.role == "a":
            for i in range(4):
                r, k = clamp(f"(g_ + {8 * (i & 1)})"), f"(t2_ + {8 * (i >> 1)})"
                pairs.append(((f"({r} * {ldm}LL + {k})", k), (f"({r} * {ldm}LL + {k} + 1)", f"({k} + 1)")))
        else:
            col = clamp("g_")
            for i in range(2):
                k = f"(t2_ + {8 * i})"
                if s.b_trans:
                    pairs.append(((f"({col} * {ldm}LL + {k})", k), (f"({col} * {ldm}LL + {k} + 1)", f"({k} + 1)")))
                else:
                    pairs.append(((f"({k} * {ldm}LL + {col})", k), (f"(({k} + 1) * {ldm}LL + {col})", f"({k} + 1)")))
        ctype = "__nv_bfloat16" if fdt == "bf16" else "__half"
        for reg, halves in enumerate(pairs):
            parts = []
            for at, k in halves:
                v = self.convert(f"{arr}[base_ + {at}]", dt, fdt)
                if k_left is not None:
                    v = f"(({k} < {k_left}) ? {v} : {self.convert('0.0f', 'f32', fdt)})"
                parts.append(f"({ctype})({v})")
            self.emit(f"{f}[{reg}] = emb::frag::pack({parts[0]}, {parts[1]});")
        self.depth -= 1
        self.emit("}")

    # ------------------------------------------------------------ the mma

    def x_MmaSyncPtx(self, s, guard) -> None:
        if tuple(s.shape) != (16, 8, 16) or s.block_scaled or s.b_row_major or s.ab_dtype not in ("f16", "bf16"):
            raise self.fragment_error(f"MmaSyncPtx: m{s.shape} {s.ab_dtype} is not supported")
        self.whole_warps(guard, "mma.sync")
        (c, _, _, _), (a, _, _, _), (b, _, _, _) = (self.member(r) for r in (s.c_frag, s.a_frag, s.b_frag))
        if s.c_dtype == "f32":
            self.emit(f"emb::frag::mma_f32<{'true' if s.ab_dtype == 'bf16' else 'false'}>({c}, {a}, {b});")
        elif s.c_dtype == "f16" and s.ab_dtype == "f16":
            self.emit(f"emb::frag::mma_f16({c}, {a}, {b});")
        else:
            raise self.fragment_error(f"MmaSyncPtx: a {s.c_dtype} accumulator for {s.ab_dtype}")

    # ------------------------------------------------------------ C-fragment arithmetic

    def c_element(self, ref: str, i: int) -> str:
        f, _, dt, _ = self.member(ref)
        if dt != "f32":
            raise self.fragment_error("arithmetic on an f16 accumulator")
        return f"{f}[{i}]"

    def s_FragmentApply(self, s) -> None:
        layout = s.layout
        if layout is not None and (getattr(layout, "n_elems", 4) != 4 or tuple(getattr(layout, "elem_row", C_ROW)) != C_ROW):
            raise self.fragment_error("FragmentApply: only the m16n8 C layout")
        self.emit("{")
        self.depth += 1
        self.emit("float out_[4];")
        self.emit("const long long g_ = v_lane >> 2, t2_ = (v_lane & 3) * 2;")
        for i in range(4):
            if s.row_base is not None:
                self.emit(f"{self.var('__frow', 'i64')} = (long long)({self.expr(s.row_base)[0]}) + g_ + {8 * C_ROW[i]};")
            if s.col_base is not None:
                self.emit(f"{self.var('__fcol', 'i64')} = (long long)({self.expr(s.col_base)[0]}) + t2_ + {C_COL[i]};")
            args = []
            for a, k in zip(s.args, s.kinds):
                if k == "frag":
                    args.append((self.c_element(a, i), "f32"))
                elif k == "row":
                    args.append(self.use(a[C_ROW[i]]))
                elif k == "uniform":
                    if isinstance(a, str):
                        args.append(self.use(a))
                    else:
                        code, kd = self.expr(a)
                        args.append((f"(float)({code})", "f32") if kd == "float" else (code, "i64"))
                elif k == "coord":
                    args.append((f"(unsigned char){self.truth(a)}", "bool"))
                elif k == "gmem":
                    name, index = a
                    arr, dt, shape, _, _ = self.memory(name)
                    args.append((self.convert(f"{arr}[{self.flat(shape, index)}]", self.value_dtype(dt), "f32"), "f32"))
                else:
                    raise self.fragment_error(f"FragmentApply: operand kind {k!r}")
            v = self.apply(s.op.name, args, "f32")
            for post in s.post:
                v = self.apply(post.name, [(v, "f32")], "f32")
            self.emit(f"out_[{i}] = {v};")
        if not s.in_place:
            if s.out not in self.frags:
                self.frag_decls.append(f"    float f_{s.out}[1][4];")
            self.frags[s.out] = ("c", "f32", 1, 4)
        for i in range(4):
            self.emit(f"{self.c_element(s.out, i)} = out_[{i}];")
        self.depth -= 1
        self.emit("}")

    def x_FragmentRowReduce(self, s, guard) -> None:
        self.whole_warps(guard, "a row reduction across lanes")
        xors = tuple(getattr(s.layout, "reduce_xors", None) or (1, 2))
        self.emit("{")
        self.depth += 1
        for r in (0, 1):
            parts = [(self.c_element(f, i), "f32") for f in s.frags for i in range(4) if C_ROW[i] == r]
            self.emit(f"float row{r}_ = {parts[0][0]};")
            for p in parts[1:]:
                self.emit(f"row{r}_ = {self.apply(s.op.name, [(f'row{r}_', 'f32'), p], 'f32')};")
        for distance in xors:
            for r in (0, 1):
                self.emit(f"{{ const float o_ = __shfl_xor_sync(0xffffffffu, row{r}_, {int(distance)}); "
                          f"row{r}_ = {self.apply(s.op.name, [(f'row{r}_', 'f32'), ('o_', 'f32')], 'f32')}; }}")
        self.emit(f"{self.var(s.top, 'f32')} = row0_; {self.var(s.bot, 'f32')} = row1_;")
        self.depth -= 1
        self.emit("}")

    def s_FragmentRepack(self, s) -> None:
        if s.fragment_layout != "m16n8k16" or len(s.srcs) != 2 or s.ab_dtype not in ("f16", "bf16"):
            raise self.fragment_error("FragmentRepack: only two m16n8k16 C fragments into f16 or bf16")
        f, _, _, _ = self.member(s.frag)
        bf = "true" if s.ab_dtype == "bf16" else "false"
        for reg, (src, lo) in enumerate(((s.srcs[0], 0), (s.srcs[0], 2), (s.srcs[1], 0), (s.srcs[1], 2))):
            self.emit(f"{f}[{reg}] = emb::frag::pack_f32<{bf}>({self.c_element(src, lo)}, {self.c_element(src, lo + 1)});")

    def s_FragmentPromote(self, s) -> None:
        src, _, sdt, _ = self.member(s.src)
        if sdt == "f32":
            raise self.fragment_error("FragmentPromote of an f32 accumulator")
        for i in range(2):
            for j in range(2):
                dst = self.c_element(s.dst, 2 * i + j)
                self.emit(f"{dst} = emb::add({dst}, emb::frag::half_of({src}[{i}], {j}));")
            self.emit(f"{src}[{i}] = 0;")

    # ------------------------------------------------------------ the store

    def s_RegStore(self, s) -> None:
        from .codegen import divisible
        if s.fragment_layout != "m16n8k16" or s.volta_interleaved:
            raise self.fragment_error("RegStore: only m16n8k16 fragments")
        arr, dt, shape, shared, _ = self.memory(s.dst_buffer)
        if dt not in ("f32", "f16"):
            raise self.fragment_error(f"RegStore into a {dt} buffer")
        frags = [self.member(s.frag)] + [self.member(x) for x in s.extra_frags]
        ldm = int(s.ldm) or (math.prod(shape[s.row_dim + 1:]) if s.row_dim is not None else int(shape[-1]))
        ldn = math.prod(shape[s.col_dim + 1:]) if s.col_dim is not None else 1

        def element(f, i):
            text, _, fdt, _ = f
            return f"{text}[{i}]" if fdt == "f32" else f"emb::frag::half_of({text}[{i // 2}], {i % 2})"

        self.emit("{")
        self.depth += 1
        self.emit(f"const long long base_ = {self.flat(shape, s.dst_index)};")
        self.emit("const long long g_ = v_lane >> 2, t2_ = (v_lane & 3) * 2;")
        rows = [f"(g_ + {8 * C_ROW[i]})" for i in range(4)]
        cols = [f"(t2_ + {C_COL[i]})" for i in range(4)]
        ctype = {"f32": "float", "f16": "__half"}[dt]
        for i in range(4):
            if s.epilogue is None:
                v = element(frags[0], i)
            else:
                epi = s.epilogue
                for param, f in zip(epi.params, frags):
                    self.emit(f"{self.var(param, 'f32')} = {element(f, i)};")
                self.emit(f"{self.var('__M__', 'i64')} = {rows[i]}; {self.var('__N__', 'i64')} = {cols[i]};")
                self.block(tuple(epi.body), None)
                v = self.convert(*self.use(epi.results[0]), "f32")
            self.emit(f"const {ctype} val{i}_ = {self.convert(v, 'f32', dt)};")
            conds = []
            for guard, coord in ((s.m_guard, rows[i]), (s.n_guard, cols[i])):
                if guard is not None:
                    (start, _), (bound, _) = self.expr(guard[0]), self.expr(guard[1])
                    conds.append(f"((long long)({start}) + {coord} < (long long)({bound}))")
            self.emit(f"const bool ok{i}_ = {' && '.join(conds) if conds else 'true'};")
        last = s.dst_index[-1] if len(s.dst_index) == len(shape) else None
        even = last is not None and int(shape[-1]) % 2 == 0 and ldm % 2 == 0 and divisible(last, 2, self.facts)
        paired = ldn == 1 and s.n_guard is None and even and not s.atomic and (s.swizzle or "NONE") in ("NONE",)
        for i in ((0, 2) if paired else range(4)):
            at = self.swz(f"(base_ + {rows[i]} * {ldm}LL + {cols[i]} * {ldn}LL)", s.swizzle)
            if paired:  # a row's two neighbouring columns as one store
                vec = "float2" if dt == "f32" else "__half2"
                make = f"make_float2(val{i}_, val{i + 1}_)" if dt == "f32" else f"__halves2half2(val{i}_, val{i + 1}_)"
                self.emit(f"if (ok{i}_) *reinterpret_cast<{vec}*>(&{arr}[{at}]) = {make};")
            elif s.atomic:
                self.emit(f"if (ok{i}_) atomicAdd(&{arr}[{at}], val{i}_);")
            else:
                self.emit(f"if (ok{i}_) {arr}[{at}] = val{i}_;")
        self.depth -= 1
        self.emit("}")


def uses_fragments(body) -> bool:
    return any(kind(s) in ir.FRAGMENT_FORM for s in ir.walk(body))
