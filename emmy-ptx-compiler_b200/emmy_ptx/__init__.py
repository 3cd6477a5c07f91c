"""emmy_ptx for B200: a backend that compiles Emmy Kernel IR to PTX for sm_100a.

Same entry points as the reference package (emmy_ptx/__init__.py:17-29)::

    frontend.load      IR json + meta.json           -> KernelSource
    lower.Lowerer      kernel family or statements   -> Kernel (CUDA template instantiation, nvcc -ptx)
    Kernel.render      nvcc's PTX                    -> the module text with the contract's header and parameters
"""

from __future__ import annotations

import sys
import traceback

from .frontend import load
from .lower import Lowerer
from .report import report as _report

PTX_LIMIT = 2_000_000  # characters of PTX a runner accepts (emmy_ptx/ptx.py:35)
PTX_VERSION = "8.8"  # CUDA 12.9's ISA: tcgen05, TMA and sm_100a
TARGET = "sm_100a"
EXPLORE_PTX_CHARS = 250_000  # emmy_ptx/__init__.py:24


def compile_file(ir_path: str, plain: bool = False, strict: bool = False, report: bool = False,
                 bulk_copy: bool = False, explore: bool = False) -> str:
    """Compile one ``*.ir.json`` file and return the PTX module text.

    The modes are the reference's (emmy_ptx/__init__.py:28-85). Optimized: a kernel
    family's template where the pattern and the legality checks pass. ``strict``: only
    what keeps every floating-point result bit for bit as the IR's own order and rounding
    give it (for the reductions the template in its in-order form; no FMA contraction).
    ``plain``: every statement by its own rule, nothing else. Should the optimized
    lowering raise, or give more than PTX_LIMIT characters, the kernel is lowered again
    plainly, with the traceback and a warning on stderr. ``report`` writes the decisions
    and a PTX profile to stderr and changes no PTX. ``bulk_copy`` is accepted and changes
    nothing: the tensor-core templates always load through the TMA unit. ``explore`` is
    accepted: the templates are rolled loops, there is no unrolling to scale down, and the
    report says so when the size target is missed."""
    src = load(ir_path)
    mode = "strictly" if strict else "optimized"
    if not plain:
        try:
            kernel = Lowerer(src, strict=strict, bulk_copy=bulk_copy).run()
            ptx = kernel.render(PTX_VERSION, TARGET)
            if explore and len(ptx) > EXPLORE_PTX_CHARS:
                kernel.remarks.append(f"compile budget (--explore): target not met: {len(ptx)} characters remain, more than "
                                      f"{EXPLORE_PTX_CHARS} (the templates have no optional unrolling to give up)")
            if len(ptx) <= PTX_LIMIT:
                if report:
                    print(_report(src, kernel, ptx, mode), file=sys.stderr)
                return ptx
            print(f"warning: {src.name}: {len(ptx)} characters of PTX, more than the runner accepts", file=sys.stderr)
        except Exception:  # noqa: BLE001 - whatever failed, the plain lowering may still succeed
            traceback.print_exc(file=sys.stderr)
        print(f"warning: {src.name}: lowering it again without the optional rewrites", file=sys.stderr)
        mode = "plainly (the fallback)"
    else:
        mode = "plainly" + (" and strictly" if strict else "")
    kernel = Lowerer(src, plain=True, strict=strict).run()
    ptx = kernel.render(PTX_VERSION, TARGET)
    if len(ptx) > PTX_LIMIT:
        print(f"error: {src.name}: even the plain lowering gives {len(ptx)} characters of PTX, more than the "
              f"runner's {PTX_LIMIT}", file=sys.stderr)
    if report:
        print(_report(src, kernel, ptx, mode), file=sys.stderr)
    return ptx
