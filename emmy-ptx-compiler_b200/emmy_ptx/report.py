"""``compile.py --report``: the lowering's decisions for one kernel and a static census of its PTX, on stderr.

Output contract (the reference's emmy_ptx/report.py:76-87, checked by its tests/test_compile.py:83-98):

    <entry>: <n> block(s) x <threads> threads[, <bytes> B of dynamic shared memory]; lowered <mode>
      <remark>                      one line per distinct remark, in order of first appearance, "(xN)" when repeated
      PTX: <count> instructions: <count> <kind>, ...

The census counts what matters on sm_100a: tensor-core (tcgen05) and tensor-memory instructions, TMA copies and
mbarrier operations, warp reductions, next to loads, stores, float arithmetic, special functions and branches.
"""

from __future__ import annotations

import re

# (label for one, label for several, pattern the opcode must start with), in print order; first match wins
CENSUS = [
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
    ("cp.async copy", "cp.async copies", r"cp\.async\.(ca|cg)"),
    ("ldmatrix", "ldmatrix", r"ldmatrix\."),
    ("warp mma", "warp mma", r"mma\.sync"),
    ("tcgen05 mma", "tcgen05 mma", r"tcgen05\.mma"),
    ("tensor-memory access", "tensor-memory accesses", r"tcgen05\.(ld|st|cp)"),
    ("shuffle", "shuffles", r"shfl\."),
    ("warp reduction", "warp reductions", r"redux\."),
    ("barrier", "barriers", r"(bar|barrier)\."),
    ("branch", "branches", r"bra\b"),
]
_NOT_CODE = ("//", ".", "{", "}", "$", "(", ")")


def opcodes(ptx: str):
    """The opcode of every instruction line of a module (directives, labels, braces and comments skipped)."""
    for raw in ptx.splitlines():
        line = raw.strip()
        if line and not line.startswith(_NOT_CODE) and not line.endswith(":"):
            yield re.sub(r"^@!?%p\d+\s+", "", line).split(None, 1)[0]


def profile(ptx: str) -> str:
    tally = {one: [0, 0] for one, _, _ in CENSUS}  # label -> [count, of which vector accesses]
    total = 0
    for op in opcodes(ptx):
        total += 1
        hit = next((one for one, _, pattern in CENSUS if re.match(pattern, op)), None)
        if hit is not None:
            tally[hit][0] += 1
            tally[hit][1] += bool(re.search(r"\.v[248]\.", op))
    shown = []
    for one, several, _ in CENSUS:
        count, vectors = tally[one]
        if count:
            shown.append(f"{count} {one if count == 1 else several}" + (f" ({vectors} vector)" if vectors else ""))
    return f"{total} instructions: " + ", ".join(shown)


def report(src, kernel, ptx: str, mode: str) -> str:
    shape = kernel.launch
    blocks, threads, dynamic = shape["grid"][0], shape["block"][0], shape["smem_bytes"]
    first = f"{kernel.name}: {'1 block' if blocks == 1 else f'{blocks} blocks'} x {threads} threads"
    if dynamic:
        first += f", {dynamic} B of dynamic shared memory"
    lines = [first + f"; lowered {mode}"]
    seen = {}
    for remark in kernel.remarks:
        seen[remark] = seen.get(remark, 0) + 1
    lines += [f"  {remark}" + (f"  (x{n})" if n > 1 else "") for remark, n in seen.items()]
    lines.append(f"  PTX: {profile(ptx)}")
    return "\n".join(lines)
