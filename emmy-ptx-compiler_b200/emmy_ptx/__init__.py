"""emmy_ptx for B200: Emmy Kernel IR to PTX for sm_100a.

The package keeps the reference's entry points (its emmy_ptx/__init__.py:17-29): ``compile_file``, ``load``,
``Lowerer``, ``PTX_LIMIT``, ``PTX_VERSION``, ``TARGET``. Behind them::

    frontend.load     *.ir.json + meta.json                    -> KernelSource      (ir.py reads the statements)
    lower.Lowerer     a kernel-family template, or statements  -> Kernel            (CUDA C++ instantiation, nvcc -ptx)
    Kernel.render     nvcc's PTX                               -> the module text   (header, launch line, p_<buffer> parameters)
"""

from __future__ import annotations

import sys
import traceback

from .frontend import load
from .lower import Lowerer
from .report import report as _report

PTX_LIMIT = 2_000_000     # characters of PTX a runner accepts (the reference's emmy_ptx/ptx.py:35)
PTX_VERSION = "8.8"       # the ISA of CUDA 12.9: tcgen05, TMA, sm_100a
TARGET = "sm_100a"
EXPLORE_PTX_CHARS = 250_000  # the module size --explore aims at (the reference's emmy_ptx/__init__.py:24)


def _say(text: str) -> None:
    print(text, file=sys.stderr)


def _attempt(src, strict: bool, bulk_copy: bool, explore: bool):
    """The optimizing lowering: (kernel, module text), or None after saying on stderr why it is not used."""
    try:
        kernel = Lowerer(src, strict=strict, bulk_copy=bulk_copy).run()
        text = kernel.render(PTX_VERSION, TARGET)
    except Exception:  # noqa: BLE001 - an IR shape a template or rewrite did not foresee must not cost the kernel its PTX
        traceback.print_exc(file=sys.stderr)
        return None
    if explore and len(text) > EXPLORE_PTX_CHARS:
        kernel.remarks.append(f"compile budget (--explore): target not met: {len(text)} characters remain, more than "
                              f"{EXPLORE_PTX_CHARS} (the templates have no optional unrolling to give up)")
    if len(text) > PTX_LIMIT:
        _say(f"warning: {src.name}: {len(text)} characters of PTX, more than the runner accepts")
        return None
    return kernel, text


def compile_file(ir_path: str, plain: bool = False, strict: bool = False, report: bool = False,
                 bulk_copy: bool = False, explore: bool = False) -> str:
    """The PTX module text of one ``*.ir.json`` file.

    Modes as in the reference (its emmy_ptx/__init__.py:28-85). By default a kernel family's template is used
    where its pattern and legality checks pass. ``strict`` keeps only what leaves every floating-point result bit
    for bit as the IR's order and rounding give it. ``plain`` lowers statement by statement and nothing else. If
    the default lowering raises, or its module is longer than PTX_LIMIT, the traceback or a warning goes to
    stderr and the kernel is lowered plainly instead (a safety net for the lowering, not a check of its code).
    ``report`` prints decisions and a PTX profile on stderr without changing the PTX. ``bulk_copy`` and
    ``explore`` are accepted: TMA loads are always on in the tensor-core templates, and there is no optional
    unrolling whose budget could be scaled (the report says so when the size target is missed).
    """
    src = load(ir_path)
    if plain:
        how = "plainly and strictly" if strict else "plainly"
    else:
        done = _attempt(src, strict, bulk_copy, explore)
        if done is not None:
            kernel, text = done
            if report:
                _say(_report(src, kernel, text, "strictly" if strict else "optimized"))
            return text
        _say(f"warning: {src.name}: lowering it again without the optional rewrites")
        how = "plainly (the fallback)"
    kernel = Lowerer(src, plain=True, strict=strict).run()
    text = kernel.render(PTX_VERSION, TARGET)
    if len(text) > PTX_LIMIT:
        _say(f"error: {src.name}: even the plain lowering gives {len(text)} characters of PTX, more than the runner's {PTX_LIMIT}")
    if report:
        _say(_report(src, kernel, text, how))
    return text
