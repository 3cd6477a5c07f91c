"""nvcc and ptxas as subprocesses, with a content-addressed cache.

The lowering instantiates a CUDA C++ kernel template (a few generated lines
that include a header of ``csrc/templates``) and asks nvcc for its PTX
(``nvcc -ptx -arch=sm_100a``); the runner then assembles the PTX with ptxas,
as the reference's remote runner does behind ``POST /compile``
(tools/run_suite.py:77-80), and loads the cubin. Both steps are pure functions
of their input text, so their results are kept under ``_cache/`` beside the
package, named by a hash of the input, the flags and every template header.
"""

from __future__ import annotations

import hashlib
import os
import re
import shutil
import subprocess
import tempfile
from pathlib import Path

PACKAGE_ROOT = Path(__file__).resolve().parent.parent
TEMPLATES = PACKAGE_ROOT / "csrc" / "templates"
CACHE = Path(os.environ.get("EMMY_B200_CACHE", PACKAGE_ROOT / "_cache"))
ARCH = "sm_100a"
GENCODE = ("-gencode", "arch=compute_100a,code=sm_100a")


class ToolchainError(RuntimeError):
    """nvcc or ptxas refused the input; the message carries their stderr."""


def _tool(name: str) -> str:
    path = os.environ.get(name.upper()) or shutil.which(name) or f"/usr/local/cuda/bin/{name}"
    if not Path(path).exists():
        raise ToolchainError(f"{name} not found (set ${name.upper()} or put it on PATH)")
    return path


def _templates_digest() -> str:
    h = hashlib.sha256()
    for f in sorted(TEMPLATES.glob("*.cuh")):
        h.update(f.name.encode())
        h.update(f.read_bytes())
    return h.hexdigest()


_DIGEST = None


def _key(*parts) -> str:
    global _DIGEST
    if _DIGEST is None:
        _DIGEST = _templates_digest()
    h = hashlib.sha256(_DIGEST.encode())
    for p in parts:
        h.update(b"\0")
        h.update(p if isinstance(p, bytes) else str(p).encode())
    return h.hexdigest()[:32]


def _atomic_write(path: Path, data: bytes) -> None:
    path.parent.mkdir(parents=True, exist_ok=True)
    fd, tmp = tempfile.mkstemp(dir=path.parent)
    with os.fdopen(fd, "wb") as f:
        f.write(data)
    os.replace(tmp, path)


def cuda_to_ptx(source: str, flags: tuple = ()) -> str:
    """PTX text of one generated ``.cu`` translation unit."""
    flags = ("-O3", "-std=c++17", "-lineinfo", "-diag-suppress", "186,550,177", *flags)
    cached = CACHE / f"{_key('ptx', source, *flags)}.ptx"
    if cached.exists():
        return cached.read_text()
    with tempfile.TemporaryDirectory() as tmp:
        cu = Path(tmp) / "kernel.cu"
        cu.write_text(source)
        out = Path(tmp) / "kernel.ptx"
        r = subprocess.run([_tool("nvcc"), "-ptx", *GENCODE, *flags, f"-I{TEMPLATES}", str(cu), "-o", str(out)],
                           capture_output=True, text=True)
        if r.returncode != 0:
            raise ToolchainError(f"nvcc failed:\n{r.stderr[-4000:]}")
        ptx = out.read_text()
    _atomic_write(cached, ptx.encode())
    return ptx


def assemble(ptx: str) -> tuple:
    """``(cubin bytes, info)`` for a PTX module; ``info`` maps each entry to the resources ptxas
    reports with ``-v``: registers, spill bytes, shared memory, barriers."""
    key = _key("cubin", ptx)
    cubin, log = CACHE / f"{key}.cubin", CACHE / f"{key}.ptxas.txt"
    if not (cubin.exists() and log.exists()):
        with tempfile.TemporaryDirectory() as tmp:
            src, out = Path(tmp) / "k.ptx", Path(tmp) / "k.cubin"
            src.write_text(ptx)
            r = subprocess.run([_tool("ptxas"), f"-arch={ARCH}", "-v", "-lineinfo", str(src), "-o", str(out)],
                               capture_output=True, text=True)
            if r.returncode != 0:
                raise ToolchainError(f"ptxas failed:\n{r.stderr[-4000:]}")
            _atomic_write(cubin, out.read_bytes())
            _atomic_write(log, r.stderr.encode())
    return cubin.read_bytes(), parse_ptxas_log(log.read_text())


def parse_ptxas_log(text: str) -> dict:
    info, entry = {}, None
    for line in text.splitlines():
        m = re.search(r"Compiling entry function '(\w+)'", line)
        if m:
            entry = m.group(1)
            info[entry] = dict(registers=0, spill_stores=0, spill_loads=0, smem=0, barriers=0, stack=0)
            continue
        if entry is None:
            continue
        m = re.search(r"(\d+) bytes stack frame, (\d+) bytes spill stores, (\d+) bytes spill loads", line)
        if m:
            info[entry].update(stack=int(m.group(1)), spill_stores=int(m.group(2)), spill_loads=int(m.group(3)))
        m = re.search(r"Used (\d+) registers", line)
        if m:
            info[entry]["registers"] = int(m.group(1))
            b = re.search(r"used (\d+) barriers", line)
            s = re.search(r"(\d+) bytes smem", line)
            info[entry]["barriers"] = int(b.group(1)) if b else 0
            info[entry]["smem"] = int(s.group(1)) if s else 0
    return info
