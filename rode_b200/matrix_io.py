"""Matrix ingest: Matrix Market files -> CSR in the layout the RoDe entry points take.

The reference's preprocessing benchmark loads ``.mtx`` files through a matrix layer whose
sources are not part of it (``Preprocess_opt/_preprocess.cu:406-415`` uses
``SPC::SparseMatrix(file, SPC::SORTED, 1)`` and ``SPC::CudaSparseMatrix<float>``; its
``utils/`` directory holds only a CMake file).  This module supplies that step: a reader for
the Matrix Market coordinate format and a COO -> CSR conversion (rows sorted, columns
ascending inside a row, duplicate entries summed) that runs on whatever device the index
tensors live on, so a file can be decomposed and multiplied without leaving the GPU.
"""
from __future__ import annotations

import numpy as np
import torch

from .workloads import CSR


def read_matrix_market(path: str):
    """Parses a Matrix Market *coordinate* file.  Returns (m, n, rows, cols, vals) with
    0-based int64 numpy indices and float32 values; `pattern` files get values 1.0,
    `symmetric` / `skew-symmetric` files are expanded to both triangles."""
    with open(path, "r") as f:
        header = f.readline().strip().split()
        if len(header) < 5 or header[0].lower() != "%%matrixmarket" or header[1].lower() != "matrix":
            raise ValueError(f"{path}: not a Matrix Market matrix file")
        layout, field, symmetry = header[2].lower(), header[3].lower(), header[4].lower()
        if layout != "coordinate":
            raise ValueError(f"{path}: only the coordinate format is supported, got {layout}")
        if field not in ("real", "integer", "pattern", "double"):
            raise ValueError(f"{path}: unsupported field {field}")
        if symmetry not in ("general", "symmetric", "skew-symmetric"):
            raise ValueError(f"{path}: unsupported symmetry {symmetry}")
        line = f.readline()
        while line and (line.startswith("%") or not line.strip()):
            line = f.readline()
        m, n, nnz = (int(x) for x in line.split()[:3])
        cols_per_line = 2 if field == "pattern" else 3
        data = np.loadtxt(f, dtype=np.float64, ndmin=2, comments="%") if nnz > 0 else np.zeros((0, cols_per_line))
    if data.shape[0] != nnz or (nnz > 0 and data.shape[1] < cols_per_line):
        raise ValueError(f"{path}: expected {nnz} entries of {cols_per_line} fields, found {data.shape}")
    rows = data[:, 0].astype(np.int64) - 1
    cols = data[:, 1].astype(np.int64) - 1
    vals = np.ones(nnz, np.float32) if field == "pattern" else data[:, 2].astype(np.float32)
    if nnz and (rows.min() < 0 or rows.max() >= m or cols.min() < 0 or cols.max() >= n):
        raise ValueError(f"{path}: index out of range")
    if symmetry != "general":
        off = rows != cols
        sign = -1.0 if symmetry == "skew-symmetric" else 1.0
        rows, cols, vals = (np.concatenate([rows, cols[off]]), np.concatenate([cols, rows[off]]),
                            np.concatenate([vals, (sign * vals[off]).astype(np.float32)]))
    return m, n, rows, cols, vals


def write_matrix_market(path: str, A: CSR) -> None:
    """Writes a CSR matrix as a general real coordinate file (1-based indices)."""
    rp = A.row_ptr.cpu().numpy().astype(np.int64)
    rows = np.repeat(np.arange(A.m, dtype=np.int64), np.diff(rp))
    cols = A.col.cpu().numpy().astype(np.int64)
    vals = A.val.cpu().numpy()
    with open(path, "w") as f:
        f.write("%%MatrixMarket matrix coordinate real general\n")
        f.write(f"{A.m} {A.n} {len(cols)}\n")
        for r, c, v in zip(rows, cols, vals):
            f.write(f"{r + 1} {c + 1} {float(v)!r}\n")


def coo_to_csr(rows: torch.Tensor, cols: torch.Tensor, vals: torch.Tensor, m: int, n: int) -> CSR:
    """COO -> CSR on the tensors' device: entries sorted by (row, column), duplicates summed.
    Index tensors may be int32 or int64; the result has int32 indices and float32 values."""
    dev = rows.device
    keys = rows.to(torch.int64) * n + cols.to(torch.int64)
    order = torch.argsort(keys)
    keys = keys[order]
    uniq, inverse = torch.unique_consecutive(keys, return_inverse=True)
    summed = torch.zeros(uniq.numel(), dtype=torch.float32, device=dev)
    summed.index_add_(0, inverse, vals.to(torch.float32)[order])
    out_rows = torch.div(uniq, n, rounding_mode="floor")
    counts = torch.bincount(out_rows, minlength=m)
    row_ptr = torch.zeros(m + 1, dtype=torch.int64, device=dev)
    torch.cumsum(counts, 0, out=row_ptr[1:])
    if int(row_ptr[-1]) >= 2**31:
        raise ValueError("nnz does not fit int32")
    return CSR(m, n, row_ptr.to(torch.int32), (uniq - out_rows * n).to(torch.int32).contiguous(), summed)


def load_matrix_market(path: str, device="cpu") -> CSR:
    """Reads a Matrix Market file and returns it as CSR on `device` (conversion runs there)."""
    m, n, rows, cols, vals = read_matrix_market(path)
    dev = torch.device(device)
    return coo_to_csr(torch.from_numpy(rows).to(dev), torch.from_numpy(cols).to(dev), torch.from_numpy(vals).to(dev), m, n)


def row_swizzle(row_ptr: torch.Tensor) -> torch.Tensor:
    """Row order by decreasing length (stable): the Sputnik-style load-balancing
    preprocessing the reference times beside RoDe's (Preprocess_opt/_preprocess.cu:71-104).
    Comparator only; the RoDe kernels do not use it."""
    lens = (row_ptr[1:] - row_ptr[:-1]).to(torch.int64)
    return torch.argsort(lens, descending=True, stable=True).to(torch.int32)
