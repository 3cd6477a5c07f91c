"""``compile.py --report``: what the lowering decided for a kernel, and a static profile of its PTX.

The output contract is the reference's (emmy_ptx/report.py:76-87): first line
``<entry>: <n> block(s) x <threads> threads[, N B of dynamic shared memory]; lowered <mode>``,
then every remark once (with its count when repeated), last ``  PTX: <n> instructions: ...`` by
kind. The kinds counted here are the ones that matter on sm_100a: tensor-core (tcgen05) and
tensor-memory instructions, TMA copies and mbarrier operations next to the classic ones.
"""

from __future__ import annotations

import re
from collections import Counter

KINDS = (
    ("FMA", "FMAs", r"fma\.\S*f(16|32|64)"),
    ("other float op", "other float ops", r"(add|sub|mul|div|max|min|neg|abs|cvt)\.\S*(f16|bf16|f32|f64)"),
    ("special function", "special functions", r"(ex2|lg2|rcp|sqrt|rsqrt|sin|cos|tanh)\."),
    ("global load", "global loads", r"ld\.global"),
    ("shared load", "shared loads", r"ld\.shared"),
    ("global store", "global stores", r"st\.global"),
    ("shared store", "shared stores", r"st\.shared"),
    ("atomic", "atomics", r"(red|atom)\."),
    ("TMA copy", "TMA copies", r"cp\.async\.bulk"),
    ("mbarrier op", "mbarrier ops", r"mbarrier\."),
    ("tcgen05 mma", "tcgen05 mma", r"tcgen05\.mma"),
    ("tensor-memory access", "tensor-memory accesses", r"tcgen05\.(ld|st|cp)"),
    ("shuffle", "shuffles", r"shfl\."),
    ("warp reduction", "warp reductions", r"redux\."),
    ("barrier", "barriers", r"(bar|barrier)\."),
    ("branch", "branches", r"bra\b"),
)


def instruction_lines(ptx: str):
    for line in ptx.splitlines():
        text = line.strip()
        if not text or text.startswith(("//", ".", "{", "}", "$", "(", ")")) or text.endswith(":"):
            continue
        yield re.sub(r"^@!?%p\d+\s+", "", text)


def profile(ptx: str) -> str:
    counts, vectors, total = Counter(), Counter(), 0
    for text in instruction_lines(ptx):
        total += 1
        op = text.split(None, 1)[0]
        for one, _, pattern in KINDS:
            if re.match(pattern, op):
                counts[one] += 1
                if ".v2." in op or ".v4." in op or ".v8." in op:
                    vectors[one] += 1
                break
    parts = []
    for one, many, _ in KINDS:
        if counts[one]:
            vec = f" ({vectors[one]} vector)" if vectors[one] else ""
            parts.append(f"{counts[one]} {one if counts[one] == 1 else many}{vec}")
    return f"{total} instructions: " + ", ".join(parts)


def report(src, kernel, ptx: str, mode: str) -> str:
    launch = kernel.launch
    grid, block, smem = launch["grid"][0], launch["block"][0], launch["smem_bytes"]
    blocks = "1 block" if grid == 1 else f"{grid} blocks"
    dyn = f", {smem} B of dynamic shared memory" if smem else ""
    out = [f"{kernel.name}: {blocks} x {block} threads{dyn}; lowered {mode}"]
    counts = Counter(kernel.remarks)
    for text in dict.fromkeys(kernel.remarks):
        out.append(f"  {text}" + (f"  (x{counts[text]})" if counts[text] > 1 else ""))
    out.append(f"  PTX: {profile(ptx)}")
    return "\n".join(out)
