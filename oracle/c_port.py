"""ctypes wrapper around the C port of the oracle (oracle/attnres_oracle.c).

TEST INFRASTRUCTURE ONLY; see attnres_oracle.py.  ``build()`` runs the Makefile
beside this file; the wrappers take and return BF16 bit patterns (uint16 arrays).
"""
from __future__ import annotations

import ctypes
import subprocess
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
LIBRARY = HERE / "_build" / "libattnres_oracle.so"
_lib = None


def build() -> Path:
    # Rebuild when the library is missing or older than its source.
    if not LIBRARY.exists() or LIBRARY.stat().st_mtime < (HERE / "attnres_oracle.c").stat().st_mtime:
        subprocess.run(["make", "-C", str(HERE), "-s"], check=True)
    return LIBRARY


def _load():
    global _lib
    if _lib is None:
        build()
        lib = ctypes.CDLL(str(LIBRARY))
        u16 = np.ctypeslib.ndpointer(dtype=np.uint16, flags="C_CONTIGUOUS")
        lib.attnres_oracle_threads.restype = ctypes.c_int
        lib.attnres_oracle_forward.restype = None
        lib.attnres_oracle_forward.argtypes = [u16, u16, ctypes.c_int, ctypes.c_int64, ctypes.c_int,
                                               ctypes.c_int, ctypes.c_float, ctypes.c_float, u16]
        lib.attnres_oracle_backward.restype = None
        lib.attnres_oracle_backward.argtypes = [u16, u16, u16, ctypes.c_int, ctypes.c_int64,
                                                ctypes.c_int, ctypes.c_int, ctypes.c_float,
                                                ctypes.c_float, u16, u16]
        _lib = lib
    return _lib


def threads() -> int:
    return int(_load().attnres_oracle_threads())


def forward(values: np.ndarray, query: np.ndarray, eps: float, scale: float) -> np.ndarray:
    S, N, D = values.shape
    out = np.empty((N, D), dtype=np.uint16)
    _load().attnres_oracle_forward(np.ascontiguousarray(values), np.ascontiguousarray(query),
                                   S, N, D, query.shape[0], eps, scale, out)
    return out


def backward(values: np.ndarray, query: np.ndarray, upstream: np.ndarray, eps: float,
             scale: float):
    S, N, D = values.shape
    dv = np.empty((S, N, D), dtype=np.uint16)
    dq = np.empty((query.shape[0],), dtype=np.uint16)
    _load().attnres_oracle_backward(np.ascontiguousarray(values), np.ascontiguousarray(query),
                                    np.ascontiguousarray(upstream), S, N, D, query.shape[0],
                                    eps, scale, dv, dq)
    return dv, dq
