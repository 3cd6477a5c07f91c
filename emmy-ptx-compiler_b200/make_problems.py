#!/usr/bin/env python3
"""Write the five full-size workload problems (IR files and meta.json) under problems/."""
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
sys.path.insert(0, str(HERE))

from emmy_ptx import problems  # noqa: E402

if __name__ == "__main__":
    for folder in problems.write_all(sys.argv[1] if len(sys.argv) > 1 else HERE / "problems"):
        print(folder)
