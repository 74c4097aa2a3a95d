"""ctypes binding of the C ABI in ``include/rode_b200.h`` (``librode_b200.so``).

torch is used only for device memory and streams: every function takes CUDA tensors (or
raw device addresses) and hands plain pointers and sizes to the library.  There is no CPU
path here: if the library is missing, loading fails loudly.
"""
from __future__ import annotations

import ctypes
import os
from dataclasses import dataclass
from typing import Optional

import torch

_PKG = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_PKG, "librode_b200.so")

RODE_OK = 0
RODE_ERR_INVALID_ARGUMENT = 1
RODE_ERR_WORKSPACE = 2
RODE_ERR_CUDA = 3
RODE_ERR_NO_DEVICE = 4

# Every symbol include/rode_b200.h declares.
C_ABI_SYMBOLS = (
    "rode_last_error", "rode_version", "rode_preprocess_workspace_bytes", "rode_preprocess_capacity",
    "rode_preprocess", "rode_preprocess_noalloc", "rode_preprocess_cpu", "rode_spmm_workspace_bytes", "rode_spmm_f32", "rode_spmm_f64",
    "rode_sddmm_f32", "rode_hot_columns_workspace_bytes", "rode_hot_columns_words", "rode_hot_columns",
    "rode_spmm_f32_hot", "rode_spmm_f64_hot",
)
# Itanium-ABI names of the C++ entry points declared in RoDeSpmm.h / RoDeSddmm.h /
# RoDePreprocess.h; identical to the names the reference's own objects export.
CPP_SYMBOLS = {
    "RoDeSpmm_n32_f32": "_Z12RoDeSpmm_n32iiiiPKfPKiS2_S2_S2_S2_S0_PfP11CUstream_stS5_",
    "RoDeSpmm_n128_f32": "_Z13RoDeSpmm_n128iiiiPKfPKiS2_S2_S2_S2_S0_PfP11CUstream_stS5_",
    "RoDeSpmm_n32_f64": "_Z12RoDeSpmm_n32iiiiPKdPKiS2_S2_S2_S2_S0_PdP11CUstream_stS5_",
    "RoDeSpmm_n128_f64": "_Z13RoDeSpmm_n128iiiiPKdPKiS2_S2_S2_S2_S0_PdP11CUstream_stS5_",
    "RoDeSDDMM_n32": "_Z13RoDeSDDMM_n32iiiiPKiS0_S0_S0_S0_PKfS2_S2_PfP11CUstream_stS5_",
    "RoDeSDDMM_n64": "_Z13RoDeSDDMM_n64iiiiPKiS0_S0_S0_S0_PKfS2_S2_PfP11CUstream_stS5_",
    "RoDeSDDMM_n128": "_Z14RoDeSDDMM_n128iiiiPKiS0_S0_S0_S0_PKfS2_S2_PfP11CUstream_stS5_",
    "RoDe_preprocess": "_Z15RoDe_preprocessiiiiPKiPiS1_S1_S1_S1_",
    "RoDe_preprocess_cpu": "_Z19RoDe_preprocess_cpuiiiiPKiPiS1_S1_RiS2_",
}


class RodeError(RuntimeError):
    def __init__(self, status: int, message: str):
        super().__init__(f"rode_b200 status {status}: {message}")
        self.status = status


_lib: Optional[ctypes.CDLL] = None


def load() -> ctypes.CDLL:
    """Load ``librode_b200.so`` (built by ``python -m rode_b200.build``).  No fallback."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise RuntimeError(
            f"{LIB_PATH} is missing: build it with `python -m rode_b200.build` (nvcc, sm_100a). "
            "rode_b200 has no CPU or PyTorch fallback."
        )
    lib = ctypes.CDLL(LIB_PATH)
    vp, ci, sz = ctypes.c_void_p, ctypes.c_int, ctypes.c_size_t
    lib.rode_last_error.restype = ctypes.c_char_p
    lib.rode_version.restype = ctypes.c_char_p
    lib.rode_preprocess_workspace_bytes.argtypes = [ci, ctypes.POINTER(sz)]
    lib.rode_preprocess_capacity.argtypes = [ci, ci, ci, ctypes.c_longlong, ctypes.POINTER(ctypes.c_longlong)]
    lib.rode_preprocess.argtypes = [ci, ci, ci, ci, vp, vp, vp, vp, vp, vp, vp, sz, vp]
    lib.rode_preprocess_noalloc.argtypes = [ci, ci, ci, ci, vp, vp, vp, vp, vp, vp, vp]
    lib.rode_preprocess_cpu.argtypes = [ci, ci, ci, ci, vp, vp, vp, vp, vp, vp]
    lib.rode_spmm_workspace_bytes.argtypes = [ci, ci, ci, ctypes.POINTER(sz)]
    lib.rode_spmm_f32.argtypes = [ci, ci, ci, ci, vp, vp, vp, vp, vp, vp, vp, vp, vp, sz, vp, vp]
    lib.rode_spmm_f64.argtypes = lib.rode_spmm_f32.argtypes
    lib.rode_sddmm_f32.argtypes = [ci, ci, ci, ci, vp, vp, vp, vp, vp, vp, vp, vp, vp, vp, vp]
    lib.rode_hot_columns_workspace_bytes.argtypes = [ci, ctypes.POINTER(sz)]
    lib.rode_hot_columns_words.argtypes = [ci, ctypes.POINTER(sz)]
    lib.rode_hot_columns.argtypes = [ctypes.c_longlong, ci, vp, sz, sz, vp, vp, sz, vp]
    lib.rode_spmm_f32_hot.argtypes = [ci, ci, ci, ci, vp, vp, vp, vp, vp, vp, vp, vp, vp, sz, vp, vp, vp]
    lib.rode_spmm_f64_hot.argtypes = lib.rode_spmm_f32_hot.argtypes
    for name in ("rode_preprocess_workspace_bytes", "rode_preprocess_capacity", "rode_preprocess",
                 "rode_preprocess_noalloc", "rode_preprocess_cpu", "rode_spmm_workspace_bytes", "rode_spmm_f32", "rode_spmm_f64",
                 "rode_sddmm_f32", "rode_hot_columns_workspace_bytes", "rode_hot_columns_words", "rode_hot_columns",
                 "rode_spmm_f32_hot", "rode_spmm_f64_hot"):
        getattr(lib, name).restype = ci
    _lib = lib
    return lib


def check(status: int) -> None:
    if status != RODE_OK:
        raise RodeError(status, load().rode_last_error().decode())


def version() -> str:
    return load().rode_version().decode()


def _ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


def _stream(s) -> Optional[int]:
    if s is None:
        return None
    if isinstance(s, torch.cuda.Stream):
        return s.cuda_stream or None
    return int(s) or None


def _dev_i32(t: torch.Tensor, name: str) -> torch.Tensor:
    if not (t.is_cuda and t.dtype == torch.int32 and t.is_contiguous()):
        raise ValueError(f"{name} must be a contiguous CUDA int32 tensor")
    return t


# ---------------------------------------------------------------------------------------
@dataclass
class RodeMeta:
    """Row-decomposition metadata on the device (outputs of the preprocessing)."""

    block_r_ind: torch.Tensor   # int32[max(m1, 1)]
    st_off: torch.Tensor        # int32[m1 + 1]
    residue_r_ind: torch.Tensor  # int32[max(m2, 1)]
    m1: int
    m2: int
    seg_len: int
    k_block: int
    vec_len: int


def preprocess_workspace_bytes(M: int) -> int:
    out = ctypes.c_size_t(0)
    check(load().rode_preprocess_workspace_bytes(M, ctypes.byref(out)))
    return out.value


def preprocess_capacity(seg_len: int, vec_len: int, M: int, nnz: int) -> int:
    out = ctypes.c_longlong(0)
    check(load().rode_preprocess_capacity(seg_len, vec_len, M, nnz, ctypes.byref(out)))
    return out.value


def preprocess_raw(seg_len, k_block, vec_len, M, row_ptr, block_r_ind, st_off, residue_r_ind, n_blk, n_res,
                   workspace, workspace_bytes, stream=None) -> None:
    """rode_preprocess on raw device addresses (ints) or tensors' data_ptr()."""
    check(load().rode_preprocess(seg_len, k_block, vec_len, M, row_ptr, block_r_ind, st_off, residue_r_ind, n_blk,
                                 n_res, workspace, workspace_bytes, _stream(stream)))


def preprocess_noalloc_raw(seg_len, k_block, vec_len, M, row_ptr, block_r_ind, st_off, residue_r_ind, n_blk, n_res,
                           stream=None) -> None:
    """rode_preprocess_noalloc on raw device addresses: the variant for callers that cannot
    allocate device memory (scratch is a fixed array inside the library, M <= 2**24)."""
    check(load().rode_preprocess_noalloc(seg_len, k_block, vec_len, M, row_ptr, block_r_ind, st_off, residue_r_ind,
                                         n_blk, n_res, _stream(stream)))


def preprocess(row_ptr: torch.Tensor, nnz: int, seg_len: int = 512, k_block: int = 32, vec_len: int = 4,
               stream=None, trim: bool = True) -> RodeMeta:
    """Device-side row decomposition of a CSR row pointer (int32 CUDA tensor [M+1]).

    Allocates outputs at the capacity bound, runs the two kernels on ``stream`` (default:
    torch's current stream), reads the two counts back (one 8-byte D2H copy, which
    synchronises the stream) and returns views trimmed to the counts."""
    _dev_i32(row_ptr, "row_ptr")
    M = row_ptr.numel() - 1
    dev = row_ptr.device
    cap = preprocess_capacity(seg_len, vec_len, M, int(nnz))
    with torch.cuda.device(dev):
        if stream is None:
            stream = torch.cuda.current_stream(dev)
        with torch.cuda.stream(stream) if isinstance(stream, torch.cuda.Stream) else _null():
            blk = torch.empty(max(cap, 1), dtype=torch.int32, device=dev)
            st = torch.empty(cap + 1, dtype=torch.int32, device=dev)
            res = torch.empty(max(M, 1), dtype=torch.int32, device=dev)
            counts = torch.empty(2, dtype=torch.int32, device=dev)
            ws_bytes = preprocess_workspace_bytes(M)
            ws = torch.empty(ws_bytes, dtype=torch.uint8, device=dev)
            preprocess_raw(seg_len, k_block, vec_len, M, row_ptr.data_ptr(), blk.data_ptr(), st.data_ptr(),
                           res.data_ptr(), counts.data_ptr(), counts.data_ptr() + 4, ws.data_ptr(), ws_bytes,
                           stream)
            m1, m2 = (int(x) for x in counts.cpu().tolist())
    if trim:
        blk, st, res = blk[: max(m1, 1)], st[: m1 + 1], res[: max(m2, 1)]
    return RodeMeta(blk, st, res, m1, m2, seg_len, k_block, vec_len)


class _null:
    def __enter__(self):
        return self

    def __exit__(self, *a):
        return False


def preprocess_cpu(row_ptr: torch.Tensor, seg_len: int = 512, k_block: int = 32, vec_len: int = 4):
    """rode_preprocess_cpu on a HOST int32 tensor (the reference's RoDe_preprocess_cpu API).

    Returns host tensors (block_r_ind[m1], st_off[m1+1], residue_r_ind[m2], m1, m2)."""
    if row_ptr.is_cuda or row_ptr.dtype != torch.int32:
        raise ValueError("row_ptr must be a CPU int32 tensor")
    row_ptr = row_ptr.contiguous()
    M = row_ptr.numel() - 1
    nnz = int(row_ptr[-1]) if M >= 0 and row_ptr.numel() > 0 else 0
    cap = preprocess_capacity(seg_len, vec_len, M, nnz)
    blk = torch.empty(max(cap, 1), dtype=torch.int32)
    st = torch.empty(cap + 1, dtype=torch.int32)
    res = torch.empty(max(M, 1), dtype=torch.int32)
    nb, nr = ctypes.c_int(0), ctypes.c_int(0)
    check(load().rode_preprocess_cpu(seg_len, k_block, vec_len, M, row_ptr.data_ptr(), blk.data_ptr(), st.data_ptr(),
                                     res.data_ptr(), ctypes.addressof(nb), ctypes.addressof(nr)))
    return blk[: nb.value].clone(), st[: nb.value + 1].clone(), res[: nr.value].clone(), nb.value, nr.value


# ---------------------------------------------------------------------------------------
def spmm_workspace_bytes(m1: int, n: int, elem_size: int = 4) -> int:
    out = ctypes.c_size_t(0)
    check(load().rode_spmm_workspace_bytes(m1, n, elem_size, ctypes.byref(out)))
    return out.value


def spmm_raw(dtype, m1, m2, k, n, values, col, row_ptr, blk, res, st, B, C, workspace, workspace_bytes,
             stream1=None, stream2=None, hot=None) -> None:
    """rode_spmm_f32 / _f64 on raw device addresses; with ``hot`` (address of a popularity
    bitmap from ``hot_columns``) the _hot entry points."""
    if hot is None:
        fn = load().rode_spmm_f32 if dtype == torch.float32 else load().rode_spmm_f64
        check(fn(m1, m2, k, n, values, col, row_ptr, blk, res, st, B, C, workspace, workspace_bytes,
                 _stream(stream1), _stream(stream2)))
    else:
        fn = load().rode_spmm_f32_hot if dtype == torch.float32 else load().rode_spmm_f64_hot
        check(fn(m1, m2, k, n, values, col, row_ptr, blk, res, st, B, C, workspace, workspace_bytes, hot,
                 _stream(stream1), _stream(stream2)))


def hot_columns_raw(nnz, n_cols, col, dense_row_bytes, budget_bytes, bitmap, workspace, workspace_bytes,
                    stream=None) -> None:
    check(load().rode_hot_columns(nnz, n_cols, col, dense_row_bytes, budget_bytes, bitmap, workspace,
                                  workspace_bytes, _stream(stream)))


def hot_columns(col: torch.Tensor, n_cols: int, dense_row_bytes: int, budget_bytes: int = 0,
                stream=None) -> Optional[torch.Tensor]:
    """Popularity bitmap of the columns for ``spmm(..., hot=...)`` (rode_hot_columns), or None
    when the library finds that marks would not help on this matrix.  Reads the flag word back
    (4-byte D2H copy, synchronises the stream)."""
    _dev_i32(col, "col")
    dev = col.device
    words, need = ctypes.c_size_t(0), ctypes.c_size_t(0)
    check(load().rode_hot_columns_words(n_cols, ctypes.byref(words)))
    check(load().rode_hot_columns_workspace_bytes(n_cols, ctypes.byref(need)))
    with torch.cuda.device(dev):
        if stream is None:
            stream = torch.cuda.current_stream(dev)
        with torch.cuda.stream(stream) if isinstance(stream, torch.cuda.Stream) else _null():
            bitmap = torch.empty(words.value, dtype=torch.int32, device=dev)
            ws = torch.empty(need.value, dtype=torch.uint8, device=dev)
            hot_columns_raw(col.numel(), n_cols, col.data_ptr(), dense_row_bytes, budget_bytes, bitmap.data_ptr(),
                            ws.data_ptr(), need.value, stream)
            useful = int(bitmap[-1].item())
    return bitmap if useful else None


def spmm(meta: RodeMeta, row_ptr: torch.Tensor, col: torch.Tensor, values: torch.Tensor, B: torch.Tensor,
         C: Optional[torch.Tensor] = None, workspace: Optional[torch.Tensor] = None, stream1=None,
         stream2=None, hot: Optional[torch.Tensor] = None) -> torch.Tensor:
    """C = S @ B through rode_spmm_f32 / rode_spmm_f64.  Asynchronous on the two streams
    (default: torch's current stream for both).  ``C`` defaults to a fresh zero tensor.
    ``hot``: popularity bitmap from ``hot_columns`` (same results, fewer DRAM bytes)."""
    M = row_ptr.numel() - 1
    k, n = B.shape
    if values.dtype not in (torch.float32, torch.float64) or B.dtype != values.dtype:
        raise ValueError("values and B must both be float32 or float64")
    if not (B.is_cuda and B.is_contiguous() and values.is_contiguous() and col.is_contiguous()):
        raise ValueError("contiguous CUDA tensors required")
    dev = B.device
    with torch.cuda.device(dev):
        cur = torch.cuda.current_stream(dev)
        s1 = cur if stream1 is None else stream1
        s2 = cur if stream2 is None else stream2
        if C is None:
            C = torch.zeros((M, n), dtype=B.dtype, device=dev)
        need = spmm_workspace_bytes(meta.m1, n, B.element_size())
        if workspace is None and need:
            workspace = torch.empty(need, dtype=torch.uint8, device=dev)
            # the buffer goes back to torch's allocator when this function returns: tell the
            # allocator which other streams still use it, or a call enqueued right afterwards
            # could be handed the same memory while this call's kernels run
            for s in (s1, s2):
                if isinstance(s, torch.cuda.Stream) and s != cur:
                    workspace.record_stream(s)
        ws_bytes = 0 if workspace is None else workspace.numel() * workspace.element_size()
        spmm_raw(B.dtype, meta.m1, meta.m2, k, n, values.data_ptr(), col.data_ptr(), row_ptr.data_ptr(),
                 meta.block_r_ind.data_ptr(), meta.residue_r_ind.data_ptr(), meta.st_off.data_ptr(), B.data_ptr(),
                 C.data_ptr(), _ptr(workspace), ws_bytes, s1, s2, hot=_ptr(hot))
    return C


def sddmm_raw(m1, m2, n, k, blk, res, st, row_ptr, col, values, lhs, rhs, out, stream1=None, stream2=None) -> None:
    check(load().rode_sddmm_f32(m1, m2, n, k, blk, res, st, row_ptr, col, values, lhs, rhs, out, _stream(stream1),
                                _stream(stream2)))


def sddmm(meta: RodeMeta, row_ptr: torch.Tensor, col: torch.Tensor, values: torch.Tensor, lhs: torch.Tensor,
          rhs: torch.Tensor, out: Optional[torch.Tensor] = None, stream1=None, stream2=None) -> torch.Tensor:
    """out[e] = values[e] * <lhs[row(e)], rhs[col(e)]> through rode_sddmm_f32."""
    k = lhs.shape[1]
    if lhs.dtype != torch.float32 or rhs.dtype != torch.float32 or values.dtype != torch.float32:
        raise ValueError("float32 tensors required")
    if rhs.shape[1] != k:
        raise ValueError("lhs and rhs must have the same number of columns")
    dev = lhs.device
    with torch.cuda.device(dev):
        cur = torch.cuda.current_stream(dev)
        s1 = cur if stream1 is None else stream1
        s2 = cur if stream2 is None else stream2
        if out is None:
            out = torch.zeros(values.numel(), dtype=torch.float32, device=dev)
        sddmm_raw(meta.m1, meta.m2, rhs.shape[0], k, meta.block_r_ind.data_ptr(), meta.residue_r_ind.data_ptr(),
                  meta.st_off.data_ptr(), row_ptr.data_ptr(), col.data_ptr(), values.data_ptr(), lhs.data_ptr(),
                  rhs.data_ptr(), out.data_ptr(), s1, s2)
    return out
