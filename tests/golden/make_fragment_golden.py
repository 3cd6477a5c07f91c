"""Generate tests/golden/m_f16_128/: the reference's shipped fragment-form example as fixture data.

Run in the build container only (it reads the reference checkout, which does not travel):
``python tests/golden/make_fragment_golden.py <path-to-reference>``.

examples/m_f16_128 is the one kernel chain the reference ships in emmy's tensor-core (fragment) form: a
split-K matmul on mma.sync fragments fed by cp.async (k_matmul__partial) and the fold of its two slabs
(k_matmul). The reference's interpreter cannot run fragment statements, so the example's own expected.npz
(made in float64, rtol = atol = 1e-2 in its meta.json) is what pins them. Stored here as data: the two
serialized IR graphs, meta.json and expected.npz, byte for byte. Before writing, the fragment extension of the
oracle is run on them and must meet the example's tolerance.
"""

from __future__ import annotations

import json
import shutil
import sys
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
REPO = HERE.parent.parent
sys.path.insert(0, str(REPO / "emmy-ptx-compiler_b200"))
sys.path.insert(0, str(REPO))

FILES = ("k_matmul__partial.ir.json", "k_matmul.ir.json", "meta.json", "expected.npz")


def main(ref: Path) -> None:
    from emmy_ptx import frontend
    from oracle import fragment_oracle
    src_dir, out = ref / "examples" / "m_f16_128", HERE / "m_f16_128"
    out.mkdir(exist_ok=True)
    for name in FILES:
        shutil.copyfile(src_dir / name, out / name)
    meta = json.loads((out / "meta.json").read_text())
    types = {"f16": np.float16, "f32": np.float32}
    bufs = {}
    for k in meta["kernels"]:
        for a in k["args"]:
            if "seed" in a:
                bufs[a["name"]] = np.random.default_rng(a["seed"]).standard_normal(a["shape"]).astype(types[a["dtype"]])
            else:
                bufs.setdefault(a["name"], np.zeros(a["shape"], types[a["dtype"]]))
    for k in meta["kernels"]:
        fragment_oracle.run(frontend.load(out / f"{k['entry']}.ir.json").body, bufs, k["grid"][0], k["block"][0])
    want = np.load(out / "expected.npz")["matmul"].astype(np.float64)
    err = np.abs(bufs["matmul"].astype(np.float64) - want) / (meta["atol"] + meta["rtol"] * np.abs(want))
    print(f"fragment oracle against expected.npz: margin {err.max():.4f} (<= 1 passes)")
    assert err.max() <= 1


if __name__ == "__main__":
    if len(sys.argv) != 2:
        raise SystemExit("usage: python tests/golden/make_fragment_golden.py <path to the reference checkout>")
    main(Path(sys.argv[1]))
