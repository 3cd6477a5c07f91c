"""ctypes binding of libemmyb200.so (include/emmy_b200.h): module load, launch, timing, tensor maps.

There is no fallback: if the library is missing or the machine has no CUDA
driver, the calls raise. Device memory belongs to the caller (torch tensors).
"""

from __future__ import annotations

import ctypes
from pathlib import Path

LIB_NAME = "libemmyb200.so"
LIB_PATH = Path(__file__).resolve().parent.parent / LIB_NAME

DTYPE_CODE = {"u8": 0, "f8e4m3": 0, "f8e5m2": 0, "i8": 0, "f16": 1, "bf16": 2, "f32": 3, "u16": 4, "i16": 4, "u32": 5, "i32": 5}
SWIZZLE_CODE = {"none": 0, "32B": 1, "64B": 2, "128B": 3}


class EmbError(RuntimeError):
    """A call into libemmyb200.so failed; ``code`` is its return value."""

    def __init__(self, code: int, text: str):
        super().__init__(f"libemmyb200: {text} (code {code})")
        self.code = code


class LaunchDesc(ctypes.Structure):
    _fields_ = [("fn", ctypes.c_void_p), ("grid", ctypes.c_uint32 * 3), ("block", ctypes.c_uint32 * 3),
                ("cluster_x", ctypes.c_uint32), ("smem_bytes", ctypes.c_uint32),
                ("params", ctypes.POINTER(ctypes.c_void_p)), ("nparams", ctypes.c_int32), ("flags", ctypes.c_uint32)]

LAUNCH_PDL = 1


_lib = None


def library() -> ctypes.CDLL:
    """The shared library, loaded once. Built by ``__graft_entry__.build()`` (nvcc)."""
    global _lib
    if _lib is None:
        if not LIB_PATH.exists():
            raise EmbError(-100, f"{LIB_PATH} is missing: build it first (python -c 'import __graft_entry__ as g; g.build()')")
        lib = ctypes.CDLL(str(LIB_PATH))
        lib.emb_last_error.restype = ctypes.c_char_p
        lib.emb_module_load.argtypes = [ctypes.c_void_p, ctypes.c_size_t, ctypes.POINTER(ctypes.c_void_p)]
        lib.emb_module_unload.argtypes = [ctypes.c_void_p]
        lib.emb_get_function.argtypes = [ctypes.c_void_p, ctypes.c_char_p, ctypes.POINTER(ctypes.c_void_p)]
        lib.emb_function_info.argtypes = [ctypes.c_void_p] + [ctypes.POINTER(ctypes.c_int)] * 4
        lib.emb_launch.argtypes = [ctypes.POINTER(LaunchDesc), ctypes.c_void_p]
        lib.emb_launch_chain.argtypes = [ctypes.POINTER(LaunchDesc), ctypes.c_int, ctypes.c_void_p]
        lib.emb_time_chain.argtypes = [ctypes.POINTER(LaunchDesc), ctypes.c_int, ctypes.c_void_p, ctypes.c_int, ctypes.c_int,
                                       ctypes.c_void_p, ctypes.c_size_t, ctypes.POINTER(ctypes.c_float)]
        lib.emb_time_rotating.argtypes = [ctypes.POINTER(LaunchDesc), ctypes.c_int, ctypes.c_int, ctypes.c_void_p, ctypes.c_int,
                                          ctypes.c_int, ctypes.c_int, ctypes.POINTER(ctypes.c_float)]
        lib.emb_tensor_map.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int, ctypes.c_int,
                                       ctypes.POINTER(ctypes.c_uint64), ctypes.POINTER(ctypes.c_uint64),
                                       ctypes.POINTER(ctypes.c_uint32), ctypes.c_int]
        _lib = lib
    return _lib


def check(code: int) -> None:
    if code != 0:
        raise EmbError(code, library().emb_last_error().decode(errors="replace"))


def init(device: int = 0) -> None:
    check(library().emb_init(int(device)))


class Module:
    """A loaded module image (PTX text or cubin bytes)."""

    def __init__(self, image: bytes | str):
        data = image.encode() + b"\0" if isinstance(image, str) else bytes(image)
        self._image = ctypes.create_string_buffer(data, len(data))
        self.handle = ctypes.c_void_p()
        check(library().emb_module_load(self._image, len(data), ctypes.byref(self.handle)))

    def function(self, entry: str) -> "Function":
        fn = ctypes.c_void_p()
        check(library().emb_get_function(self.handle, entry.encode(), ctypes.byref(fn)))
        return Function(self, entry, fn)

    def unload(self) -> None:
        if self.handle:
            check(library().emb_module_unload(self.handle))
            self.handle = ctypes.c_void_p()


class Function:
    def __init__(self, module: Module, entry: str, handle):
        self.module, self.entry, self.handle = module, entry, handle

    def info(self) -> dict:
        v = [ctypes.c_int() for _ in range(4)]
        check(library().emb_function_info(self.handle, *(ctypes.byref(x) for x in v)))
        return dict(registers=v[0].value, static_smem=v[1].value, local_bytes=v[2].value, max_threads=v[3].value)


class TensorMap:
    """128 bytes of CUtensorMap in 64-byte aligned host storage."""

    def __init__(self, base: int, dtype: str, dims, strides_bytes, box, swizzle: str = "128B"):
        self._raw = ctypes.create_string_buffer(128 + 64)
        addr = ctypes.addressof(self._raw)
        self.address = (addr + 63) & ~63
        rank = len(dims)
        d = (ctypes.c_uint64 * rank)(*dims)
        s = (ctypes.c_uint64 * max(rank - 1, 1))(*strides_bytes) if rank > 1 else None
        b = (ctypes.c_uint32 * rank)(*box)
        check(library().emb_tensor_map(ctypes.c_void_p(self.address), ctypes.c_void_p(base), DTYPE_CODE[dtype], rank, d, s, b,
                                       SWIZZLE_CODE[swizzle]))


class Launch:
    """One kernel launch with its parameter storage kept alive."""

    def __init__(self, fn: Function, grid, block, cluster: int, smem_bytes: int, params: list, flags: int = 0):
        """``params``: an int (a device pointer) or a TensorMap per kernel parameter."""
        self.fn = fn
        self._keep = []
        n = len(params)
        self._slots = (ctypes.c_void_p * max(n, 1))()
        for i, p in enumerate(params):
            if isinstance(p, TensorMap):
                self._keep.append(p)
                self._slots[i] = p.address  # the parameter's value IS the 128 bytes at this address
            else:
                cell = ctypes.c_uint64(int(p))
                self._keep.append(cell)
                self._slots[i] = ctypes.addressof(cell)
        self.desc = LaunchDesc(fn.handle, (ctypes.c_uint32 * 3)(*grid), (ctypes.c_uint32 * 3)(*block), int(cluster),
                               int(smem_bytes), ctypes.cast(self._slots, ctypes.POINTER(ctypes.c_void_p)), n, int(flags))
        self.buffers: list = []  # names of the buffers the launch reads or writes (filled by who binds it)
        self.scratch: list = []  # keys of its scratch buffers

    def scratch_names(self) -> set:
        """The bare names of the launch's scratch buffers (a tensor map over a scratch buffer names it so)."""
        return {key.split(".", 1)[1] for key in self.scratch}


def _chain(launches):
    arr = (LaunchDesc * len(launches))()
    for i, l in enumerate(launches):
        arr[i] = l.desc
    return arr


def launch(launches, stream: int = 0) -> None:
    """Enqueue the launches in order on ``stream`` (a cudaStream_t handle as an int)."""
    launches = list(launches)
    check(library().emb_launch_chain(_chain(launches), len(launches), ctypes.c_void_p(stream)))


def time_chain(launches, stream: int = 0, warmup: int = 3, iters: int = 20, flush=None) -> list:
    """Microseconds of each of ``iters`` runs of the chain (CUDA events on ``stream``), after
    ``warmup`` runs. ``flush`` = (device pointer, bytes) of a buffer overwritten before each timed
    run to evict L2."""
    launches = list(launches)
    out = (ctypes.c_float * iters)()
    ptr, size = flush if flush else (0, 0)
    check(library().emb_time_chain(_chain(launches), len(launches), ctypes.c_void_p(stream), warmup, iters,
                                   ctypes.c_void_p(ptr), size, out))
    return list(out)


def time_rotating(sets, stream: int = 0, warmup: int = 3, iters: int = 20, batch: int = 1) -> list:
    """Microseconds per run of each of ``iters`` batches of ``batch`` consecutive runs, run i using
    ``sets[i % len(sets)]`` (each a list of launches bound to its own buffers): with the sets
    together larger than L2, every run is cold."""
    sets = [list(s) for s in sets]
    flat = [l for s in sets for l in s]
    out = (ctypes.c_float * iters)()
    check(library().emb_time_rotating(_chain(flat), len(sets[0]), len(sets), ctypes.c_void_p(stream), warmup, iters, batch, out))
    return list(out)
