"""Shared checks of the parity tests."""
import numpy as np

# Tolerance of the fp32 paths against the fp64-accumulated ground truth: max relative error
# 1e-5, with an absolute floor of 1e-6 near zero.  A sum of T terms of magnitude <= 1 carries
# a rounding error of a few T * 2^-24 whatever the order, so for long rows the absolute
# floor is scaled by the sum of |terms| of the element ("abs_scale").
REL_TOL = 1e-5
ABS_TOL = 1e-6


def tolerance_stats(got, truth, abs_scale=None):
    """How much of the tolerance a result uses.  Returns a dict with
    ``worst_ratio``  max over elements of err / allowed (allowed = the rule of
                     assert_close_to_truth; <= 1 means the check passes),
    ``literal_fail`` number of elements that break the literal rule err <= max(1e-5 |truth|, 1e-6),
                     i.e. the rule without the magnitude-scaled floor,
    ``elements``     number of elements compared, ``max_err`` the largest absolute error."""
    got = np.asarray(got, dtype=np.float64)
    truth = np.asarray(truth, dtype=np.float64)
    err = np.abs(got - truth)
    floor = ABS_TOL if abs_scale is None else np.maximum(ABS_TOL, 2.0 ** -22 * np.asarray(abs_scale, np.float64))
    allowed = np.maximum(REL_TOL * np.abs(truth), floor)
    literal = np.maximum(REL_TOL * np.abs(truth), ABS_TOL)
    return {"worst_ratio": float((err / allowed).max()) if err.size else 0.0,
            "literal_fail": int((err > literal).sum()), "elements": int(err.size),
            "max_err": float(err.max()) if err.size else 0.0}


def assert_close_to_truth(got, truth, abs_scale=None, what=""):
    """Checks the tolerance rule above and returns tolerance_stats() of the comparison."""
    got = np.asarray(got, dtype=np.float64)
    truth = np.asarray(truth, dtype=np.float64)
    assert got.shape == truth.shape, f"{what}: shape {got.shape} vs {truth.shape}"
    assert np.all(np.isfinite(got)), f"{what}: non-finite values"
    err = np.abs(got - truth)
    floor = ABS_TOL if abs_scale is None else np.maximum(ABS_TOL, 2.0 ** -22 * np.asarray(abs_scale, np.float64))
    bad = err > np.maximum(REL_TOL * np.abs(truth), floor)
    if bad.any():
        i = np.argmax(err * bad)
        raise AssertionError(
            f"{what}: {bad.sum()} of {bad.size} elements out of tolerance; worst at flat index {i}: "
            f"got {got.flat[i]!r}, truth {truth.flat[i]!r}, err {err.flat[i]:.3e}")
    return tolerance_stats(got, truth, abs_scale)


def spmm_abs_scale(row_ptr, col, val, B):
    """sum_e |val_e| * |B[col_e, :]| per output element (magnitude of the summed terms)."""
    from oracle import cpu

    return cpu.spmm_f64acc(row_ptr, col, np.abs(val), np.abs(B))


def sddmm_abs_scale(row_ptr, col, val, lhs, rhs):
    from oracle import cpu

    return cpu.sddmm_f64acc(row_ptr, col, np.abs(val), np.abs(lhs), np.abs(rhs))


# ---- GPU-side helpers (imported lazily by the gpu tests) ---------------------------------
def gpu_inputs(A, device="cuda"):
    """CSR on the device plus its row-decomposition metadata for both parameter sets."""
    from rode_b200 import capi

    d = A.to(device)
    meta512 = capi.preprocess(d.row_ptr, d.nnz, 512, 32, 4)
    return d, meta512


def run_reference_spmm(d, meta, B, variant):
    """The reference's own SpMM kernels (oracle/_ref) on the same device arrays."""
    import torch

    from oracle import ref

    C = torch.zeros((d.m, B.shape[1]), dtype=B.dtype, device=B.device)
    s1, s2 = torch.cuda.Stream(), torch.cuda.Stream()
    torch.cuda.synchronize()
    ref.spmm_gpu(variant, B.dtype == torch.float64, meta.m1, meta.m2, d.n, B.shape[1], d.val.data_ptr(),
                 d.col.data_ptr(), d.row_ptr.data_ptr(), meta.block_r_ind.data_ptr(), meta.residue_r_ind.data_ptr(),
                 meta.st_off.data_ptr(), B.data_ptr(), C.data_ptr(), s1.cuda_stream, s2.cuda_stream)
    torch.cuda.synchronize()
    return C


def run_reference_sddmm(d, meta, lhs, rhs):
    import torch

    from oracle import ref

    out = torch.zeros(d.nnz, dtype=torch.float32, device=lhs.device)
    s1, s2 = torch.cuda.Stream(), torch.cuda.Stream()
    torch.cuda.synchronize()
    ref.sddmm_gpu(lhs.shape[1], meta.m1, meta.m2, d.n, meta.block_r_ind.data_ptr(), meta.residue_r_ind.data_ptr(),
                  meta.st_off.data_ptr(), d.row_ptr.data_ptr(), d.col.data_ptr(), d.val.data_ptr(), lhs.data_ptr(),
                  rhs.data_ptr(), out.data_ptr(), s1.cuda_stream, s2.cuda_stream)
    torch.cuda.synchronize()
    return out


def sample_rows_csr(A, rows):
    """Host CSR made of the given rows of a (device or host) CSR, for checking a sample of a
    matrix that is too large for the CPU oracle."""
    import numpy as np
    import torch

    rows = torch.as_tensor(rows, dtype=torch.int64, device=A.row_ptr.device)
    rp = A.row_ptr.to(torch.int64)
    lo, hi = rp[rows], rp[rows + 1]
    lens = hi - lo
    new_rp = torch.zeros(rows.numel() + 1, dtype=torch.int64, device=rp.device)
    torch.cumsum(lens, 0, out=new_rp[1:])
    idx = torch.repeat_interleave(lo - new_rp[:-1], lens) + torch.arange(int(new_rp[-1]), device=rp.device)
    return (new_rp.to(torch.int32).cpu().numpy(), A.col[idx].cpu().numpy(), A.val[idx].cpu().numpy(),
            idx.cpu().numpy())
