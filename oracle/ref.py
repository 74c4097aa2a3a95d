"""ctypes front-end of the reference's own code compiled into ``oracle/_ref``.

TEST INFRASTRUCTURE: used to pin the C restatement (``oracle/cpu.py``), to generate the
fixtures under ``tests/golden`` and, on a GPU, to compare the new kernels with the
reference kernels on the same inputs.  The libraries are built from the reference checkout
by ``make -C oracle ref`` and are absent where that never ran; ``available()`` says so.

The reference functions have C++ linkage; the mangled names below are the Itanium-ABI
names of exactly these declarations:

  RoDe_SDDMM/main.cu:65    void sddmm_cpu_reference(int m,int n,int k,int nnz,const int*,const int*,
                                const float*,const float*,const float*,float*)
  RoDe_SDDMM/main.cu:114   void RoDe_preprocess(int SegmentLength,int vectorLen,int KBLOCK,int M,
                                const int*,int*,int*,int*,int&,int&)
  RoDe_SDDMM/RoDeSddmm.h:4,8   RoDeSDDMM_n32 / RoDeSDDMM_n128
  RoDe_SpMM/RoDeSpmm.h:4-14    RoDeSpmm_n32 / RoDeSpmm_n128 (float and double overloads)
"""
from __future__ import annotations

import ctypes
import os

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_SDDMM = os.path.join(_HERE, "_ref", "libref_sddmm.so")
_SPMM = os.path.join(_HERE, "_ref", "libref_spmm.so")
_libs = {}

SYM_PREPROCESS = "_Z15RoDe_preprocessiiiiPKiPiS1_S1_RiS2_"
SYM_SDDMM_CPU = "_Z19sddmm_cpu_referenceiiiiPKiS0_PKfS2_S2_Pf"
SYM_SDDMM_N32 = "_Z13RoDeSDDMM_n32iiiiPKiS0_S0_S0_S0_PKfS2_S2_PfP11CUstream_stS5_"
SYM_SDDMM_N128 = "_Z14RoDeSDDMM_n128iiiiPKiS0_S0_S0_S0_PKfS2_S2_PfP11CUstream_stS5_"
SYM_SPMM_N32_F = "_Z12RoDeSpmm_n32iiiiPKfPKiS2_S2_S2_S2_S0_PfP11CUstream_stS5_"
SYM_SPMM_N128_F = "_Z13RoDeSpmm_n128iiiiPKfPKiS2_S2_S2_S2_S0_PfP11CUstream_stS5_"
SYM_SPMM_N32_D = "_Z12RoDeSpmm_n32iiiiPKdPKiS2_S2_S2_S2_S0_PdP11CUstream_stS5_"
SYM_SPMM_N128_D = "_Z13RoDeSpmm_n128iiiiPKdPKiS2_S2_S2_S2_S0_PdP11CUstream_stS5_"


def available() -> bool:
    return os.path.exists(_SDDMM) and os.path.exists(_SPMM)


def _lib(path: str) -> ctypes.CDLL:
    if path not in _libs:
        _libs[path] = ctypes.CDLL(path)
    return _libs[path]


def _p(a: np.ndarray):
    return a.ctypes.data_as(ctypes.c_void_p)


def preprocess(row_ptr, seg_len: int, k_block: int, vec_len: int):
    """The reference's host RoDe_preprocess (note its argument order: seg, vec, k_block)."""
    row_ptr = np.ascontiguousarray(row_ptr, np.int32)
    m = len(row_ptr) - 1
    nnz = int(row_ptr[-1])
    cap = nnz // seg_len + m + 8
    blk = np.zeros(cap, np.int32)
    st = np.zeros(cap + 1, np.int32)
    res = np.zeros(max(m, 1), np.int32)
    nb, nr = ctypes.c_int(0), ctypes.c_int(0)
    fn = getattr(_lib(_SDDMM), SYM_PREPROCESS)
    fn.restype = None
    fn(ctypes.c_int(seg_len), ctypes.c_int(vec_len), ctypes.c_int(k_block), ctypes.c_int(m), _p(row_ptr),
       _p(blk), _p(st), _p(res), ctypes.byref(nb), ctypes.byref(nr))
    return blk[: nb.value].copy(), st[: nb.value + 1].copy(), res[: nr.value].copy(), nb.value, nr.value


def sddmm_cpu(row_ptr, col, val, lhs, rhs, n_cols: int) -> np.ndarray:
    """The reference's sddmm_cpu_reference (single thread, fp32)."""
    row_ptr = np.ascontiguousarray(row_ptr, np.int32)
    col = np.ascontiguousarray(col, np.int32)
    val = np.ascontiguousarray(val, np.float32)
    lhs = np.ascontiguousarray(lhs, np.float32)
    rhs = np.ascontiguousarray(rhs, np.float32)
    out = np.zeros(len(val), np.float32)
    fn = getattr(_lib(_SDDMM), SYM_SDDMM_CPU)
    fn.restype = None
    fn(ctypes.c_int(len(row_ptr) - 1), ctypes.c_int(n_cols), ctypes.c_int(lhs.shape[1]), ctypes.c_int(len(val)),
       _p(row_ptr), _p(col), _p(val), _p(lhs), _p(rhs), _p(out))
    return out


# ---- GPU entry points of the reference: device pointers as integers, streams as handles ----

def _vp(x):
    return ctypes.c_void_p(int(x))


def sddmm_gpu(k: int, m1, m2, n, blk, res, st, row_ptr, col, val, lhs, rhs, out, stream1, stream2) -> None:
    """RoDeSDDMM_n32 (k == 32) or RoDeSDDMM_n128 (k == 128) on device pointers.

    The reference skips a kernel whose stream handle is null (RoDeSddmm.cu:503,509), so
    both streams must be real (non-default) streams."""
    assert k in (32, 128)
    fn = getattr(_lib(_SDDMM), SYM_SDDMM_N32 if k == 32 else SYM_SDDMM_N128)
    fn.restype = None
    fn(ctypes.c_int(m1), ctypes.c_int(m2), ctypes.c_int(n), ctypes.c_int(k), _vp(blk), _vp(res), _vp(st),
       _vp(row_ptr), _vp(col), _vp(val), _vp(lhs), _vp(rhs), _vp(out), _vp(stream1), _vp(stream2))


def spmm_gpu(variant: int, double: bool, m1, m2, k, n, val, col, row_ptr, blk, res, st, B, C, stream1,
             stream2) -> None:
    """RoDeSpmm_n32 (variant 32) / RoDeSpmm_n128 (variant 128), float or double overload.

    Preconditions taken from reading the kernels (never call outside them):
    m1 > 0 and m2 > 0 (a zero-sized grid is an invalid launch, RoDeSpmm.cu:499-508);
    n a multiple of 32 (variant 32) or 64 (variant 128); max(col) * n * sizeof(T) < 2**31
    (byte offsets are formed in int, RoDeSpmm.cu:153,287); C zero-filled; st has m1+1 entries."""
    assert variant in (32, 128) and m1 > 0 and m2 > 0
    sym = {(32, False): SYM_SPMM_N32_F, (128, False): SYM_SPMM_N128_F,
           (32, True): SYM_SPMM_N32_D, (128, True): SYM_SPMM_N128_D}[(variant, bool(double))]
    fn = getattr(_lib(_SPMM), sym)
    fn.restype = None
    fn(ctypes.c_int(m1), ctypes.c_int(m2), ctypes.c_int(k), ctypes.c_int(n), _vp(val), _vp(col), _vp(row_ptr),
       _vp(blk), _vp(res), _vp(st), _vp(B), _vp(C), _vp(stream1), _vp(stream2))
