"""ctypes binding of the native sm_100a library (``lib/libsnu1_b200.so``).

The library has a plain C ABI: every entry point takes raw device pointers and
a stream handle and returns 0 or a negative error code; the message is fetched
with ``snu1_last_error``.  Kernels report device-side problems (a wait that ran
out of time) through a status word that :func:`check_status` reads.
"""
from __future__ import annotations

import ctypes
import os
from pathlib import Path

import torch

_LIB = None
_LIB_PATH = Path(__file__).resolve().parent.parent / "lib" / "libsnu1_b200.so"

c_void_p = ctypes.c_void_p
c_int = ctypes.c_int
c_ll = ctypes.c_longlong
c_float = ctypes.c_float


class NativeLibraryError(RuntimeError):
    pass


def lib_path() -> Path:
    return _LIB_PATH


def available() -> bool:
    return _LIB_PATH.exists()


def load():
    """Loads the library (once).  Raises when it has not been built."""
    global _LIB
    if _LIB is not None:
        return _LIB
    if not _LIB_PATH.exists():
        raise NativeLibraryError(
            f"{_LIB_PATH} is missing: run `python -m sensenova_u1_b200.build` "
            "(the CUDA ops of this package have no fallback on a GPU box)")
    lib = ctypes.CDLL(os.fspath(_LIB_PATH))
    lib.snu1_last_error.restype = ctypes.c_char_p
    _LIB = lib
    return lib


def ptr(t) -> int | None:
    if t is None:
        return None
    return t.data_ptr()


def stream() -> int:
    return torch.cuda.current_stream().cuda_stream


# kernels launched per entry point (for launch accounting)
_KERNELS = {"attn_bwd": 3, "attn_build_tiles": 4}
LAUNCHES = 0


def call(name: str, *args) -> None:
    """Calls ``snu1_<name>`` and raises on a non-zero return code."""
    global LAUNCHES
    LAUNCHES += _KERNELS.get(name, 1)
    lib = load()
    fn = getattr(lib, "snu1_" + name)
    rc = fn(*args)
    if rc != 0:
        msg = lib.snu1_last_error()
        raise NativeLibraryError(f"snu1_{name} failed ({rc}): {msg.decode() if msg else ''}")


_ROLE = {1: "TMA producer", 2: "MMA issuer (accumulator)", 3: "MMA issuer (operands)",
         4: "epilogue", 5: "softmax", 6: "correction", 7: "peer flag", 8: "expert-parallel plan"}


def check_status() -> None:
    """Synchronises the device and raises if a kernel reported a problem."""
    lib = load()
    out = c_int(0)
    rc = lib.snu1_read_status(ctypes.byref(out))
    if rc != 0:
        raise NativeLibraryError(f"snu1_read_status failed: {lib.snu1_last_error().decode()}")
    v = out.value
    if v != 0:
        code, where = v & 0xff, v >> 8
        what = {1: "a wait on an mbarrier ran out of time",
                2: "a size limit was exceeded on the device (e.g. expert receive buffer too small)",
                3: "a wait on a peer flag ran out of time"}.get(code, f"code {code}")
        raise NativeLibraryError(f"kernel status: {what} (role: {_ROLE.get(where, where)})")
