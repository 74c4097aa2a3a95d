"""ctypes front-end of ``oracle/rode_oracle.c`` (TEST INFRASTRUCTURE, never the product path).

Every function takes and returns numpy arrays.  The algorithms and the reference lines
they restate are documented in ``rode_oracle.c``.
"""
from __future__ import annotations

import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "librode_oracle.so")
_lib = None


def build(force: bool = False) -> str:
    """Compile ``rode_oracle.c`` with the Makefile beside it (gcc, OpenMP)."""
    if force or not os.path.exists(_LIB_PATH) or os.path.getmtime(_LIB_PATH) < os.path.getmtime(
        os.path.join(_HERE, "rode_oracle.c")
    ):
        subprocess.run(["make", "-C", _HERE, os.path.join(_HERE, "librode_oracle.so")], check=True,
                       capture_output=True)
    return _LIB_PATH


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        if not os.path.exists(_LIB_PATH):
            build()
        _lib = ctypes.CDLL(_LIB_PATH)
    return _lib


def _p(a: np.ndarray):
    return a.ctypes.data_as(ctypes.c_void_p)


def _i32(a) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=np.int32)


def _f32(a) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=np.float32)


def max_threads() -> int:
    """Host threads this process may run on.  Not OpenMP's own default: launchers such as
    torchrun export OMP_NUM_THREADS=1, and the functions here take the count explicitly."""
    try:
        return max(1, len(os.sched_getaffinity(0)))
    except AttributeError:  # platforms without sched_getaffinity
        return max(1, os.cpu_count() or int(lib().rode_oracle_max_threads()))


def preprocess_count(row_ptr, seg_len: int, k_block: int, vec_len: int):
    row_ptr = _i32(row_ptr)
    nb, nr = ctypes.c_int(0), ctypes.c_int(0)
    lib().rode_oracle_preprocess_count(seg_len, k_block, vec_len, len(row_ptr) - 1, _p(row_ptr),
                                       ctypes.byref(nb), ctypes.byref(nr))
    return nb.value, nr.value


def preprocess(row_ptr, seg_len: int, k_block: int, vec_len: int):
    """Returns (block_r_ind[n_blk], st_off[n_blk+1], residue_r_ind[n_res], n_blk, n_res)."""
    row_ptr = _i32(row_ptr)
    m = len(row_ptr) - 1
    cb, cr = preprocess_count(row_ptr, seg_len, k_block, vec_len)
    blk = np.empty(max(cb, 1), np.int32)
    st = np.empty(cb + 1, np.int32)
    res = np.empty(max(cr, 1), np.int32)
    nb, nr = ctypes.c_int(0), ctypes.c_int(0)
    lib().rode_oracle_preprocess(seg_len, k_block, vec_len, m, _p(row_ptr), _p(blk), _p(st), _p(res),
                                 ctypes.byref(nb), ctypes.byref(nr))
    assert nb.value == cb and nr.value == cr
    return blk[:cb].copy(), st, res[:cr].copy(), cb, cr


def sddmm_f32(row_ptr, col, val, lhs, rhs, threads: int = 1) -> np.ndarray:
    row_ptr, col, val, lhs, rhs = _i32(row_ptr), _i32(col), _f32(val), _f32(lhs), _f32(rhs)
    out = np.zeros(len(val), np.float32)
    lib().rode_oracle_sddmm_f32(len(row_ptr) - 1, lhs.shape[1], _p(row_ptr), _p(col), _p(val), _p(lhs),
                                _p(rhs), _p(out), int(threads))
    return out


def sddmm_f64acc(row_ptr, col, val, lhs, rhs, threads: int = 1) -> np.ndarray:
    row_ptr, col, val, lhs, rhs = _i32(row_ptr), _i32(col), _f32(val), _f32(lhs), _f32(rhs)
    out = np.zeros(len(val), np.float64)
    lib().rode_oracle_sddmm_f64acc(len(row_ptr) - 1, lhs.shape[1], _p(row_ptr), _p(col), _p(val), _p(lhs),
                                   _p(rhs), _p(out), int(threads))
    return out


def spmm_f32(row_ptr, col, val, B, threads: int = 1) -> np.ndarray:
    row_ptr, col, val, B = _i32(row_ptr), _i32(col), _f32(val), _f32(B)
    m, n = len(row_ptr) - 1, B.shape[1]
    C = np.empty((m, n), np.float32)
    lib().rode_oracle_spmm_f32(m, n, _p(row_ptr), _p(col), _p(val), _p(B), _p(C), int(threads))
    return C


def spmm_f64acc(row_ptr, col, val, B, threads: int = 1) -> np.ndarray:
    row_ptr, col, val, B = _i32(row_ptr), _i32(col), _f32(val), _f32(B)
    m, n = len(row_ptr) - 1, B.shape[1]
    C = np.empty((m, n), np.float64)
    lib().rode_oracle_spmm_f64acc(m, n, _p(row_ptr), _p(col), _p(val), _p(B), _p(C), int(threads))
    return C


def spmm_f64(row_ptr, col, val, B, threads: int = 1) -> np.ndarray:
    row_ptr, col = _i32(row_ptr), _i32(col)
    val = np.ascontiguousarray(val, dtype=np.float64)
    B = np.ascontiguousarray(B, dtype=np.float64)
    m, n = len(row_ptr) - 1, B.shape[1]
    C = np.empty((m, n), np.float64)
    lib().rode_oracle_spmm_f64(m, n, _p(row_ptr), _p(col), _p(val), _p(B), _p(C), int(threads))
    return C
