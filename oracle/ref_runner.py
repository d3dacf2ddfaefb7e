"""Test infrastructure: runs the reference's own emitted CPU code (oracle/_ref/libsofie_ref.so, built
by oracle/build_ref.py from the unmodified reference generator) on the seeded parity cases."""
from __future__ import annotations

import ctypes as C
from pathlib import Path

import numpy as np

REF_DIR = Path(__file__).resolve().parent / "_ref"
LIB = REF_DIR / "libsofie_ref.so"
_lib = None


def available() -> bool:
    return LIB.exists()


def lib():
    global _lib
    if _lib is None:
        _lib = C.CDLL(str(LIB))
        _lib.ref_blas_config.restype = C.c_char_p
        _lib.ref_get_threads.restype = C.c_int
    return _lib


def set_threads(n: int) -> None:
    lib().ref_set_threads(C.c_int(n))


def threads() -> int:
    return lib().ref_get_threads()


def blas_config() -> str:
    return lib().ref_blas_config().decode()


def infer(case: str, x: np.ndarray, out_elems: int) -> np.ndarray:
    """One Session::infer of the emitted header of `case` (the Session is built on first use from
    the .dat file the reference generator wrote)."""
    fn = getattr(lib(), f"ref_{case}_infer")
    fn.restype = C.c_long
    x = np.ascontiguousarray(x, np.float32)
    y = np.empty(out_elems, np.float32)
    n = fn(str(REF_DIR / f"{case}.dat").encode(), x.ctypes.data_as(C.c_void_p), y.ctypes.data_as(C.c_void_p),
           C.c_long(out_elems))
    if n != out_elems:
        raise RuntimeError(f"reference case {case}: expected {out_elems} outputs, the emitted code returned {n}")
    return y
