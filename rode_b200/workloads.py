"""Seeded synthetic sparse matrices for the RoDe hot path (benchmark and test inputs).

The reference measures nothing on a public dataset; its drivers draw random CSR matrices
(``RoDe_SDDMM/rode_sddmm.py:100-144`` ``RoDeCSR.from_random``, ``RoDe_SDDMM/main.cu:181-234``).
The generators here produce the five benchmark matrix families at any scale, on the CPU or
on a CUDA device, from ``torch`` random streams with a fixed seed.  All return int32 CSR
with ascending, distinct columns per row and no padding entries, so about three quarters
of the rows start at an offset that is not a multiple of four.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch


@dataclass
class CSR:
    m: int
    n: int
    row_ptr: torch.Tensor  # int32 [m+1]
    col: torch.Tensor      # int32 [nnz]
    val: torch.Tensor      # float32 [nnz]

    @property
    def nnz(self) -> int:
        return int(self.col.numel())

    def to(self, device) -> "CSR":
        return CSR(self.m, self.n, self.row_ptr.to(device), self.col.to(device), self.val.to(device))

    def rows(self, r0: int, r1: int) -> "CSR":
        """Rows [r0, r1) as a CSR of their own (row pointer re-based to 0, columns kept)."""
        lo, hi = int(self.row_ptr[r0]), int(self.row_ptr[r1])
        rp = (self.row_ptr[r0 : r1 + 1] - lo).to(torch.int32)
        return CSR(r1 - r0, self.n, rp.contiguous(), self.col[lo:hi].contiguous(), self.val[lo:hi].contiguous())


def _gen(device, seed: int) -> torch.Generator:
    g = torch.Generator(device=device)
    g.manual_seed(seed)
    return g


def _uniform(shape, lo: float, hi: float, device, gen) -> torch.Tensor:
    return torch.rand(shape, generator=gen, device=device, dtype=torch.float32) * (hi - lo) + lo


def dense(rows: int, cols: int, device="cpu", seed: int = 1, dtype=torch.float32) -> torch.Tensor:
    """Dense operand, uniform in [-1, 1)."""
    return _uniform((rows, cols), -1.0, 1.0, device, _gen(device, seed)).to(dtype)


def _row_ptr_from_lengths(lengths: torch.Tensor) -> torch.Tensor:
    rp = torch.zeros(lengths.numel() + 1, dtype=torch.int64, device=lengths.device)
    torch.cumsum(lengths, 0, out=rp[1:])
    if int(rp[-1]) >= 2**31:
        raise ValueError("nnz does not fit int32")
    return rp


def _from_sorted_keys(keys: torch.Tensor, m: int, n: int, val_lo: float, val_hi: float, gen) -> CSR:
    """keys = row * n + col, ascending and distinct."""
    rows = torch.div(keys, n, rounding_mode="floor")
    cols = (keys - rows * n).to(torch.int32)
    counts = torch.bincount(rows, minlength=m)
    rp = _row_ptr_from_lengths(counts).to(torch.int32)
    val = _uniform((keys.numel(),), val_lo, val_hi, keys.device, gen)
    return CSR(m, n, rp, cols.contiguous(), val)


def _distinct_columns(lengths: torch.Tensor, n: int, gen) -> torch.Tensor:
    """For every row i, ``lengths[i]`` distinct uniform columns in [0, n), as ascending keys
    row * n + col.  Duplicates are re-drawn until none are left (lengths[i] <= n/2)."""
    device = lengths.device
    m = lengths.numel()
    row_of = torch.repeat_interleave(torch.arange(m, device=device, dtype=torch.int64), lengths)
    total = row_of.numel()
    keys = row_of * n + torch.randint(0, n, (total,), generator=gen, device=device, dtype=torch.int64)
    for _ in range(200):
        keys, _ = torch.sort(keys)
        dup = torch.zeros(total, dtype=torch.bool, device=device)
        dup[1:] = keys[1:] == keys[:-1]
        n_dup = int(dup.sum())
        if n_dup == 0:
            return keys
        rows = torch.div(keys[dup], n, rounding_mode="floor")
        keys[dup] = rows * n + torch.randint(0, n, (n_dup,), generator=gen, device=device, dtype=torch.int64)
    raise RuntimeError("could not draw distinct columns")


def _rescale_lengths(raw: torch.Tensor, mean: float, cap: int, floor: int) -> torch.Tensor:
    """Scale positive draws so that the rounded, clipped lengths have the wanted mean."""
    lo, hi = 0.0, 1.0
    def lengths(f):
        return torch.clamp(torch.round(raw * f), floor, cap).to(torch.int64)
    while float(lengths(hi).double().mean()) < mean and hi < 1e12:
        hi *= 2.0
    for _ in range(60):
        mid = 0.5 * (lo + hi)
        if float(lengths(mid).double().mean()) < mean:
            lo = mid
        else:
            hi = mid
    return lengths(hi)


# ---------------------------------------------------------------------------------------
def bernoulli(m: int = 4096, n: int = 4096, p: float = 0.01, device="cpu", seed: int = 11) -> CSR:
    """Every entry non-zero independently with probability p; values 1.0."""
    g = _gen(device, seed)
    mask = torch.rand((m, n), generator=g, device=device) < p
    keys = torch.nonzero(mask.reshape(-1)).reshape(-1)  # ascending row * n + col
    out = _from_sorted_keys(keys, m, n, 0.0, 1.0, g)
    out.val = torch.ones_like(out.val)
    return out


def zipf_rows(m: int = 65536, n: int = 65536, alpha: float = 1.6, cap: int = 16384, mean: float = 16.0,
              device="cpu", seed: int = 22) -> CSR:
    """Heavy-tailed row lengths: Zipf(alpha) draws capped at ``cap`` and rescaled to the wanted
    mean; distinct uniform columns, ascending; values uniform [-1, 1)."""
    g = _gen(device, seed)
    # Inverse-CDF sampling of a continuous power law with the Zipf tail exponent, floored:
    # P(X >= x) ~ x^-(alpha-1) for x >= 1.
    u = torch.rand(m, generator=g, device=device, dtype=torch.float64).clamp_min(1e-12)
    raw = torch.floor(u.pow(-1.0 / (alpha - 1.0))).clamp(max=float(cap))
    lengths = _rescale_lengths(raw, mean, min(cap, n // 2), 1)
    keys = _distinct_columns(lengths, n, g)
    return _from_sorted_keys(keys, m, n, -1.0, 1.0, g)


def stencil27(grid: int = 128, device="cpu", seed: int = 33) -> CSR:
    """27-point stencil on a grid^3 lattice (no wrap-around); values uniform [0.5, 1.5)."""
    g = _gen(device, seed)
    m = grid**3
    idx = torch.arange(m, device=device, dtype=torch.int64)
    z, y, x = idx // (grid * grid), (idx // grid) % grid, idx % grid
    keys = []
    for dz in (-1, 0, 1):
        for dy in (-1, 0, 1):
            for dx in (-1, 0, 1):
                ok = ((z + dz >= 0) & (z + dz < grid) & (y + dy >= 0) & (y + dy < grid) & (x + dx >= 0)
                      & (x + dx < grid))
                nb = idx + (dz * grid + dy) * grid + dx
                keys.append((idx * m + nb)[ok])
    keys, _ = torch.sort(torch.cat(keys))
    return _from_sorted_keys(keys, m, m, 0.5, 1.5, g)


def pareto_rows(m: int = 1 << 20, n: int = 1 << 20, shape: float = 1.2, mean: float = 32.0, cap: int = 200000,
                device="cpu", seed: int = 44) -> CSR:
    """Power-law degrees: Pareto(shape) draws scaled to the wanted mean and capped; distinct
    uniform columns; values uniform [-1, 1)."""
    g = _gen(device, seed)
    u = torch.rand(m, generator=g, device=device, dtype=torch.float64).clamp_min(1e-12)
    raw = u.pow(-1.0 / shape)
    lengths = _rescale_lengths(raw, mean, min(cap, n // 2), 0)
    keys = _distinct_columns(lengths, n, g)
    return _from_sorted_keys(keys, m, n, -1.0, 1.0, g)


def rmat(scale: int = 23, edge_factor: int = 16, a: float = 0.57, b: float = 0.19, c: float = 0.19,
         device="cpu", seed: int = 55, chunk: int = 1 << 25) -> CSR:
    """R-MAT graph with 2^scale vertices and edge_factor * 2^scale edges before removal of
    duplicates; rows sorted; values uniform [-1, 1)."""
    g = _gen(device, seed)
    n = 1 << scale
    total = edge_factor * n
    parts = []
    for start in range(0, total, chunk):
        cnt = min(chunk, total - start)
        rows = torch.zeros(cnt, dtype=torch.int64, device=device)
        cols = torch.zeros(cnt, dtype=torch.int64, device=device)
        for _ in range(scale):
            r = torch.rand(cnt, generator=g, device=device)
            row_bit = r >= (a + b)                    # quadrants c, d
            col_bit = ((r >= a) & (r < a + b)) | (r >= a + b + c)  # quadrants b, d
            rows = (rows << 1) | row_bit
            cols = (cols << 1) | col_bit
        parts.append(torch.unique(rows * n + cols))
    keys = torch.unique(torch.cat(parts)) if len(parts) > 1 else parts[0]
    return _from_sorted_keys(keys, n, n, -1.0, 1.0, g)


# ---------------------------------------------------------------------------------------
def partition_rows(row_ptr: torch.Tensor, parts: int, row_weight: float = 0.0):
    """Contiguous row ranges of equal cost, cost(row) = nnz(row) + row_weight.

    row_weight = 0 is the plain nnz-balanced partition: cut p lies at the first row whose
    offset reaches nnz * p / parts.  A positive row_weight also counts the per-row work
    (one row of the result is written per sparse row, as costly as gathering one dense row
    for a nonzero), which matters when the ranges differ a lot in their number of rows.
    Returns ``parts + 1`` row indices (first 0, last M)."""
    rp = row_ptr.to(torch.float64).cpu() if row_weight else row_ptr.to(torch.int64).cpu()
    m = rp.numel() - 1
    if row_weight:
        cost = rp + row_weight * torch.arange(m + 1, dtype=torch.float64)
        total = float(cost[-1])
        targets = torch.tensor([total * p / parts for p in range(1, parts)], dtype=torch.float64)
    else:
        cost = rp
        nnz = int(rp[-1])
        targets = torch.tensor([(nnz * p) // parts for p in range(1, parts)], dtype=torch.int64)
    cuts = torch.searchsorted(cost, targets, right=False).clamp(0, m).tolist() if parts > 1 else []
    bounds = [0] + [int(c) for c in cuts] + [m]
    for i in range(1, len(bounds)):
        bounds[i] = max(bounds[i], bounds[i - 1])
    return bounds
