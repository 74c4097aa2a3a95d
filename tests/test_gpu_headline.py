"""The configuration the benchmark times, checked for parity: R-MAT scale 23 (8,388,608 rows,
about 131 M nonzeros), SpMM with N = 128 through the popularity-hinted entry point with the
library's default budget (the hinted block kernel on a grid of far more than two waves), and
SDDMM with K = 64 on the same matrix.  The matrix is too large for a full CPU pass inside a
test, so a sample of rows (the 16 longest, 64 empty ones, 4096 random ones) is compared with
the fp64-accumulating oracle, and the hinted result must equal the plain one bit for bit."""
import numpy as np
import pytest
import torch

from rode_b200 import capi
from rode_b200 import workloads as W
from tests.helpers import assert_close_to_truth, sample_rows_csr, sddmm_abs_scale, spmm_abs_scale

pytestmark = pytest.mark.gpu

SCALE = 23
N_DENSE = 128
K_SDDMM = 64


@pytest.fixture(scope="module")
def headline():
    A = W.rmat(scale=SCALE, device="cuda")
    meta = capi.preprocess(A.row_ptr, A.nnz, 512, 32, 4)
    lens = (A.row_ptr[1:] - A.row_ptr[:-1]).long()
    g = torch.Generator(device="cuda").manual_seed(1)
    rows = torch.cat([torch.topk(lens, 16).indices, torch.nonzero(lens == 0).flatten()[:64],
                      torch.randint(0, A.m, (4096,), device="cuda", generator=g)]).unique()
    yield A, meta, rows
    del A, meta
    torch.cuda.empty_cache()


def test_headline_spmm_with_default_hints(oracle_cpu, headline, headroom):
    A, meta, rows = headline
    assert A.m == 1 << SCALE and meta.m1 > 2 * 32 * 148      # a block grid of more than two waves
    hot = capi.hot_columns(A.col, A.n, 4 * N_DENSE)          # budget 0 = the library's default
    assert hot is not None, "the library must find the hints useful on this matrix"
    B = W.dense(A.n, N_DENSE, device="cuda", seed=3)
    hinted = capi.spmm(meta, A.row_ptr, A.col, A.val, B, hot=hot)
    torch.cuda.synchronize()
    rp, col, val, _ = sample_rows_csr(A, rows)
    Bh = B.cpu().numpy()
    truth = oracle_cpu.spmm_f64acc(rp, col, val, Bh, threads=oracle_cpu.max_threads())
    scale = spmm_abs_scale(rp, col, val, Bh)
    got = hinted[rows].cpu().numpy()
    headroom(f"5 R-MAT {SCALE} SpMM N={N_DENSE} (hints, row sample)", "ours",
             assert_close_to_truth(got, truth, scale, "headline SpMM sample"))
    lens = rp[1:] - rp[:-1]
    assert np.all(got[lens == 0] == 0.0)                     # empty rows stay as the caller zero-filled them
    del Bh, truth, scale
    plain = capi.spmm(meta, A.row_ptr, A.col, A.val, B)
    torch.cuda.synchronize()
    assert torch.equal(plain, hinted)                        # hints change cache residency only
    del plain, hinted


def test_headline_sddmm_k64(oracle_cpu, headline, headroom):
    A, meta, rows = headline
    lhs = W.dense(A.m, K_SDDMM, device="cuda", seed=5)
    rhs = W.dense(A.n, K_SDDMM, device="cuda", seed=6)
    out = capi.sddmm(meta, A.row_ptr, A.col, A.val, lhs, rhs)
    torch.cuda.synchronize()
    rp, col, val, idx = sample_rows_csr(A, rows)
    lh, rh = lhs[rows].cpu().numpy(), rhs.cpu().numpy()
    truth = oracle_cpu.sddmm_f64acc(rp, col, val, lh, rh, threads=oracle_cpu.max_threads())
    got = out[torch.from_numpy(idx).cuda()].cpu().numpy()
    headroom(f"5 R-MAT {SCALE} SDDMM K={K_SDDMM} (row sample)", "ours",
             assert_close_to_truth(got, truth, sddmm_abs_scale(rp, col, val, lh, rh), "headline SDDMM sample"))
    # every entry is written exactly once: a second run into a NaN-filled buffer leaves no NaN
    out2 = torch.full_like(out, float("nan"))
    capi.sddmm(meta, A.row_ptr, A.col, A.val, lhs, rhs, out=out2)
    torch.cuda.synchronize()
    assert torch.equal(out, out2)
