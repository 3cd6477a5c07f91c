#!/usr/bin/env python3
"""Compile one Emmy Kernel-IR file to PTX for NVIDIA B200 (sm_100a).

    python compile.py [--strict] [--plain] [--report] [--bulk-copy] [--explore] path/to/<kernel>.ir.json > out.ptx

The command line of the reference's compile.py, flag for flag (compile.py:30-47):
PTX goes to stdout and nothing else does; diagnostics go to stderr; exit code 0
on success, 1 when the compilation raised (traceback on stderr, stdout empty),
2 on a usage error. ``meta.json`` must sit next to the IR file (parameter order,
launch geometry).

--strict     only lowerings that keep every floating-point result bit for bit what
             the IR's own order of operations gives (reductions in order, no FMA)
--plain      one rule per statement, no template and no optional rewrite
--report     the lowering's decisions and a PTX profile on stderr
--bulk-copy  accepted for compatibility; TMA loads are always on in the templates
--explore    accepted for compatibility; reports when the module size target is missed
"""

import sys
import traceback
from pathlib import Path

sys.path.insert(0, str(Path(__file__).resolve().parent / "emmy-ptx-compiler_b200"))

from emmy_ptx import compile_file  # noqa: E402

FLAGS = ("--strict", "--plain", "--report", "--bulk-copy", "--explore")
USAGE = "usage: python compile.py [--strict] [--plain] [--report] [--bulk-copy] [--explore] <kernel>.ir.json > out.ptx"


def main(argv) -> int:
    flags = {a for a in argv[1:] if a.startswith("--")}
    paths = [a for a in argv[1:] if not a.startswith("--")]
    if len(paths) != 1 or flags - set(FLAGS):
        print(USAGE, file=sys.stderr)
        return 2
    try:
        ptx = compile_file(paths[0], plain="--plain" in flags, strict="--strict" in flags, report="--report" in flags,
                           bulk_copy="--bulk-copy" in flags, explore="--explore" in flags)
    except Exception:  # stdout must stay clean
        traceback.print_exc(file=sys.stderr)
        return 1
    sys.stdout.write(ptx)
    return 0


if __name__ == "__main__":
    sys.exit(main(sys.argv))
