#!/usr/bin/env python3
"""B200 (sm_100a) backend of the Emmy Kernel-IR compiler: one ``*.ir.json`` in, one PTX module out.

    python compile.py [--strict] [--plain] [--report] [--bulk-copy] [--explore] path/to/<kernel>.ir.json > out.ptx

Drop-in for the reference's command line (its compile.py:30-47): the same five switches, exactly one
path, PTX and only PTX on stdout, everything else on stderr, and the same exit codes

    0  compiled
    1  the compilation raised; the traceback is on stderr and stdout stays empty
    2  bad command line (unknown switch, no path or more than one); the usage line is on stderr

``meta.json`` is looked up next to the IR file (parameter order and launch geometry).

    --strict     keep every floating-point result bit for bit what the IR's own order of operations gives:
                 reductions fold in order, nothing is contracted to an FMA, the tensor-core templates stand back
    --plain      lower statement by statement, with no kernel template and no optional rewrite
    --report     say on stderr what was decided and profile the PTX; the PTX itself does not change
    --bulk-copy  kept for compatibility (the tensor-core templates always load through TMA)
    --explore    kept for compatibility (there is no optional unrolling to trade for module size)
"""

from __future__ import annotations

import sys
import traceback
from pathlib import Path

HERE = Path(__file__).resolve().parent
sys.path.insert(0, str(HERE / "emmy-ptx-compiler_b200"))

SWITCHES = {"--strict": "strict", "--plain": "plain", "--report": "report", "--bulk-copy": "bulk_copy", "--explore": "explore"}
USAGE = "usage: python compile.py " + " ".join(f"[{s}]" for s in SWITCHES) + " <kernel>.ir.json > out.ptx"


class UsageError(Exception):
    pass


def parse(arguments: list) -> tuple:
    """(path, keyword options of compile_file) from the command line, or UsageError."""
    options = {name: False for name in SWITCHES.values()}
    paths = []
    for word in arguments:
        if not word.startswith("--"):
            paths.append(word)
        elif word in SWITCHES:
            options[SWITCHES[word]] = True
        else:
            raise UsageError(word)
    if len(paths) != 1:
        raise UsageError("path")
    return paths[0], options


def main(argv: list) -> int:
    try:
        path, options = parse(argv[1:])
    except UsageError:
        sys.stderr.write(USAGE + "\n")
        return 2
    from emmy_ptx import compile_file
    try:
        module_text = compile_file(path, **options)
    except Exception:  # whatever it was: report it, and leave stdout untouched
        traceback.print_exc(file=sys.stderr)
        return 1
    sys.stdout.write(module_text)
    return 0


if __name__ == "__main__":
    raise SystemExit(main(sys.argv))
