"""Python entry of the RoDe SDDMM / SpMM path on B200.

Drop-in for the reference's ``RoDe_SDDMM/rode_sddmm.py``: the same public names
(``RoDeCSR``, ``rode_sddmm``, ``torch_sddmm_reference``, ``compare_results``), constructor
arguments and attributes, on top of the compiled module ``rode_sddmm_cuda`` (this package's
torch binding of ``librode_b200.so``).

What differs from the reference wrapper:
  * the row decomposition runs on the GPU (the reference loops on the CPU at every
    construction and uploads three arrays, ``rode_sddmm.py:82-98``);
  * ``k`` may also be 64, and ``rode_spmm`` is added (the reference exposes no SpMM in Python);
  * ``rode_sddmm`` does not block the host: it launches on torch's current stream.
"""
from __future__ import annotations

import torch

from . import rode_sddmm_cuda  # compiled binding; importing fails loudly if it was not built


class RoDeCSR:
    """CSR sparse matrix plus the RoDe row-decomposition metadata
    (mirrors ``RoDe_SDDMM/rode_sddmm.py:12-191``).

    Attributes: ``m, n, k, nnz, device, row_offsets_cpu, row_offsets, column_indices, values,
    block_indices, st_offsets, residue_indices, m1, m2``.
    """

    # (seg_length, k_block, vec_len) per hidden width, as in rode_sddmm.py:35-38 (32 and 128);
    # every other width (any multiple of 4 up to 256, which the reference does not serve) uses
    # the long segments of width 32.
    CONFIGS = {
        32: {"seg_length": 512, "k_block": 32, "vec_len": 4},
        64: {"seg_length": 512, "k_block": 32, "vec_len": 4},
        128: {"seg_length": 32, "k_block": 32, "vec_len": 4},
    }
    MAX_K = 256

    @classmethod
    def config_for(cls, k: int) -> dict:
        if k <= 0 or k % 4 != 0 or k > cls.MAX_K:
            raise ValueError(f"k must be a multiple of 4, at most {cls.MAX_K}, got {k}")
        return cls.CONFIGS.get(k, cls.CONFIGS[32])

    def __init__(self, row_offsets: torch.Tensor, column_indices: torch.Tensor, values: torch.Tensor,
                 device: torch.device, m: int, n: int, k: int = 128):
        self.config_for(k)
        self.m = m
        self.n = n
        self.k = k
        self.nnz = values.numel()
        self.device = torch.device(device)
        if self.device.type != "cuda":
            raise ValueError("RoDeCSR needs a CUDA device; rode_b200 has no CPU path")
        if self.device.index is None:  # "cuda" -> "cuda:<current>", so that tensor.device compares equal
            self.device = torch.device("cuda", torch.cuda.current_device())
        self.row_offsets = row_offsets.to(dtype=torch.int32, device=self.device).contiguous()
        self.row_offsets_cpu = row_offsets.to(dtype=torch.int32, device="cpu").contiguous()
        self.column_indices = column_indices.to(dtype=torch.int32, device=self.device).contiguous()
        self.values = values.to(dtype=torch.float32, device=self.device).contiguous()
        self._preprocess()

    def _preprocess(self):
        config = self.config_for(self.k)
        with torch.cuda.device(self.device):
            blk, st, res, m1, m2 = rode_sddmm_cuda.preprocess(
                self.row_offsets, self.nnz, config["seg_length"], config["k_block"], config["vec_len"])
        self.block_indices = blk
        self.st_offsets = st
        self.residue_indices = res
        self.m1 = m1
        self.m2 = m2

    @classmethod
    def from_random(cls, m: int, n: int, nnz_per_row: int, device: torch.device, k: int = 128) -> "RoDeCSR":
        """Random matrix with about ``m * nnz_per_row`` distinct entries and normal values
        (same construction as ``rode_sddmm.py:100-144``: random coordinates, duplicates removed)."""
        nnz_raw = m * nnz_per_row
        coords = torch.randint(0, m, (nnz_raw,)) * n + torch.randint(0, n, (nnz_raw,))
        coords = torch.unique(coords)
        rows = torch.div(coords, n, rounding_mode="floor")
        cols = coords - rows * n
        row_offsets = torch.zeros(m + 1, dtype=torch.int64)
        row_offsets[1:] = torch.cumsum(torch.bincount(rows, minlength=m), 0)
        values = torch.randn(coords.numel(), dtype=torch.float32)
        return cls(row_offsets.to(torch.int32), cols.to(torch.int32), values, device, m, n, k)

    def to_torch_sparse_csr(self) -> torch.Tensor:
        """torch sparse CSR tensor without explicit zeros (``rode_sddmm.py:146-185`` drops
        entries whose value is 0, the padding of the reference's C++ generators)."""
        keep = self.values != 0
        rows = torch.repeat_interleave(torch.arange(self.m, device=self.device),
                                       (self.row_offsets[1:] - self.row_offsets[:-1]).long())
        crow = torch.zeros(self.m + 1, dtype=torch.int64, device=self.device)
        crow[1:] = torch.cumsum(torch.bincount(rows[keep], minlength=self.m), 0)
        return torch.sparse_csr_tensor(crow, self.column_indices[keep].long(), self.values[keep],
                                       size=(self.m, self.n), device=self.device)

    def __repr__(self) -> str:
        return (f"RoDeCSR(m={self.m}, n={self.n}, nnz={self.nnz}, k={self.k}, "
                f"m1={self.m1}, m2={self.m2}, device={self.device})")


def _check_dense(name: str, t: torch.Tensor, shape, sparse: RoDeCSR):
    if tuple(t.shape) != tuple(shape):
        raise ValueError(f"{name} shape must be {tuple(shape)}, got {tuple(t.shape)}")
    assert t.is_cuda and t.device == sparse.device, f"{name} must be on {sparse.device}, got {t.device}"
    assert t.dtype == torch.float32, f"{name} must be float32, got {t.dtype}"


def rode_sddmm(sparse_matrix: RoDeCSR, lhs: torch.Tensor, rhs: torch.Tensor) -> torch.Tensor:
    """out = S ⊙ (lhs @ rhs^T) sampled at the stored entries of S; returns values [nnz]
    (mirrors ``rode_sddmm.py:194-248``)."""
    m, n, k = sparse_matrix.m, sparse_matrix.n, sparse_matrix.k
    _check_dense("lhs_matrix", lhs, (m, k), sparse_matrix)
    _check_dense("rhs_matrix", rhs, (n, k), sparse_matrix)
    return rode_sddmm_cuda.sddmm_forward(
        sparse_matrix.block_indices, sparse_matrix.residue_indices, sparse_matrix.st_offsets, sparse_matrix.m1,
        sparse_matrix.m2, sparse_matrix.row_offsets, sparse_matrix.column_indices, sparse_matrix.values, m, n,
        lhs.contiguous(), rhs.contiguous(), k)


def rode_spmm(sparse_matrix: RoDeCSR, dense: torch.Tensor, hints: bool = True) -> torch.Tensor:
    """C = S @ dense for dense [n, width], width a multiple of 4.  Needs metadata from
    seg_length 512 (k = 32 or 64 at construction); the reference has no Python SpMM.

    ``hints``: gather popular columns' rows with an L2 policy that keeps them resident
    (same results, fewer DRAM bytes on skewed matrices).  The popularity bitmap is built on
    the first call for a given width and cached on ``sparse_matrix``."""
    if sparse_matrix.config_for(sparse_matrix.k)["k_block"] != 32:
        raise ValueError("SpMM needs k_block = 32 metadata")
    if dense.dim() != 2 or dense.shape[0] != sparse_matrix.n:
        raise ValueError(f"dense must be ({sparse_matrix.n}, width), got {tuple(dense.shape)}")
    assert dense.is_cuda and dense.device == sparse_matrix.device and dense.dtype == torch.float32
    hot = None
    if hints and dense.shape[1] % 128 == 0:
        cache = sparse_matrix.__dict__.setdefault("_hot_columns", {})
        row_bytes = dense.shape[1] * dense.element_size()
        if row_bytes not in cache:
            cache[row_bytes] = rode_sddmm_cuda.hot_columns(sparse_matrix.column_indices, sparse_matrix.n, row_bytes)
        hot = cache[row_bytes]
    return rode_sddmm_cuda.spmm_forward(
        sparse_matrix.block_indices, sparse_matrix.residue_indices, sparse_matrix.st_offsets, sparse_matrix.m1,
        sparse_matrix.m2, sparse_matrix.row_offsets, sparse_matrix.column_indices, sparse_matrix.values,
        sparse_matrix.m, sparse_matrix.n, dense.contiguous(), hot)


def torch_sddmm_reference(sparse_csr: torch.Tensor, lhs_matrix: torch.Tensor, rhs_matrix: torch.Tensor) -> torch.Tensor:
    """The comparison the reference's tests use (``rode_sddmm.py:251-304``):
    ``torch.sparse.sampled_addmm`` with beta = 0 samples lhs @ rhs^T on the pattern, and the
    samples are multiplied by the stored values.  Test helper, not a fallback."""
    sampled = torch.sparse.sampled_addmm(sparse_csr, lhs_matrix, rhs_matrix.T, beta=0.0, alpha=1.0)
    return torch.sparse_csr_tensor(sampled.crow_indices(), sampled.col_indices(),
                                   sampled.values() * sparse_csr.values(), size=sampled.shape,
                                   device=sampled.device, dtype=sampled.dtype)


def compare_results(rode_output: torch.Tensor, torch_sparse_output: torch.Tensor, rode_csr: RoDeCSR,
                    tolerance: float = 1e-3) -> dict:
    """Same report as ``rode_sddmm.py:307-378``: entries with a zero stored value are left
    out, an element fails when both its absolute and its relative error exceed ``tolerance``."""
    torch_values = torch_sparse_output.values().to(torch.float32).cpu()
    rode_values = rode_output[rode_csr.values != 0].to(torch.float32).cpu()
    if rode_values.numel() != torch_values.numel():
        return {"passed": False,
                "error": f"Size mismatch: RoDe={rode_values.numel()}, Torch={torch_values.numel()}",
                "mae": float("inf"), "mean_rel": float("inf"), "max_abs": float("inf"), "max_rel": float("inf"),
                "error_count": -1, "total_count": rode_values.numel()}
    diff = (rode_values - torch_values).abs()
    rel = diff / (torch_values.abs() + 1e-8)
    errors = int(((diff > tolerance) & (rel > tolerance)).sum())
    n = max(diff.numel(), 1)
    return {"passed": errors == 0, "mae": float(diff.sum() / n), "mean_rel": float(rel.sum() / n),
            "max_abs": float(diff.max()) if diff.numel() else 0.0, "max_rel": float(rel.max()) if rel.numel() else 0.0,
            "error_count": errors, "total_count": rode_values.numel()}
