"""Column popularity hints: the bitmap against a numpy restatement of the selection rule, and
SpMM with hints bit-identical to SpMM without (the hints steer L2 residency only)."""
import numpy as np
import pytest
import torch

from rode_b200 import capi
from rode_b200 import workloads as W
from tests.helpers import assert_close_to_truth, gpu_inputs, sample_rows_csr, spmm_abs_scale

pytestmark = pytest.mark.gpu

BINS = 4096


def _expected(col, n_cols, max_hot):
    """The rule of rode_hot_columns: walk the in-degrees from the highest down (degrees of
    BINS-1 and more count as one), stop before the marked columns exceed max_hot or at
    in-degree 1; useful = the touched columns exceed 1.5 * max_hot and the marked columns get
    at least twice their share of the references."""
    deg = np.bincount(col, minlength=n_cols).astype(np.int64)
    binned = np.minimum(deg, BINS - 1)
    cols_per = np.bincount(binned, minlength=BINS)
    refs_per = np.bincount(binned, weights=deg, minlength=BINS)
    touched, refs = cols_per[1:].sum(), refs_per[1:].sum()
    hot, hot_refs, thr = 0, 0, BINS
    for b in range(BINS - 1, 1, -1):
        if hot + cols_per[b] > max_hot:
            break
        hot += cols_per[b]
        hot_refs += refs_per[b]
        thr = b
    useful = (2 * touched > 3 * max_hot) and hot > 0 and hot_refs * touched >= 2.0 * hot * refs
    return deg >= thr, bool(useful)


def _bitmap(col_dev, n_cols, row_bytes, budget):
    words = (n_cols + 31) // 32 + 1
    ws_bytes = 4 * n_cols + 64 * 1024
    bitmap = torch.full((words,), -1, dtype=torch.int32, device="cuda")
    ws = torch.empty(ws_bytes + 256, dtype=torch.uint8, device="cuda")
    capi.hot_columns_raw(col_dev.numel(), n_cols, col_dev.data_ptr(), row_bytes, budget, bitmap.data_ptr(),
                         ws.data_ptr(), ws_bytes, torch.cuda.current_stream())
    torch.cuda.synchronize()
    raw = bitmap.cpu().numpy().view(np.uint32)
    bits = np.unpackbits(raw[:-1].view(np.uint8), bitorder="little")[:n_cols].astype(bool)
    return bits, int(raw[-1]), bitmap


@pytest.mark.parametrize("family,max_hot", [("rmat", 2000), ("rmat", 64), ("pareto", 500), ("zipf", 100), ("bernoulli", 100000)])
def test_bitmap_follows_the_selection_rule(family, max_hot):
    A = {"rmat": lambda: W.rmat(scale=16), "pareto": lambda: W.pareto_rows(m=20000, n=30000, cap=5000),
         "zipf": lambda: W.zipf_rows(m=8192, n=10007, cap=2048), "bernoulli": lambda: W.bernoulli()}[family]()
    row_bytes = 512
    bits, flag, _ = _bitmap(A.col.cuda(), A.n, row_bytes, max_hot * row_bytes)
    want_bits, want_flag = _expected(A.col.numpy(), A.n, max_hot)
    assert np.array_equal(bits, want_bits)
    assert flag == int(want_flag)


def test_flag_clear_without_skew_and_wrapper_returns_none():
    A = W.pareto_rows(m=20000, n=30000, cap=5000)   # uniform columns: no popular subset
    assert capi.hot_columns(A.col.cuda(), A.n, 512, budget_bytes=1000 * 512) is None


@pytest.mark.parametrize("dtype", [torch.float32, torch.float64])
def test_spmm_with_hints_is_bit_identical(oracle_cpu, dtype):
    A = W.rmat(scale=19)
    d, meta = gpu_inputs(A)
    n = 128 if dtype == torch.float32 else 64
    row_bytes = n * (4 if dtype == torch.float32 else 8)
    hot = capi.hot_columns(d.col, A.n, row_bytes, budget_bytes=20000 * row_bytes)
    assert hot is not None                          # R-MAT columns are strongly skewed
    B = W.dense(A.n, n, seed=9).to(dtype)
    Bd = B.cuda()
    vals = d.val.to(dtype)
    plain = capi.spmm(meta, d.row_ptr, d.col, vals, Bd)
    hinted = capi.spmm(meta, d.row_ptr, d.col, vals, Bd, hot=hot)
    torch.cuda.synchronize()
    assert torch.equal(plain, hinted)
    if dtype == torch.float32:                      # and both are right
        rows = np.random.default_rng(1).choice(A.m, 2000, replace=False)
        rows.sort()
        srp, scol, sval, _ = sample_rows_csr(A, rows)
        truth = oracle_cpu.spmm_f64acc(srp, scol, sval, B.numpy())
        assert_close_to_truth(hinted[torch.from_numpy(rows).cuda()].cpu().numpy(), truth,
                              spmm_abs_scale(srp, scol, sval, B.numpy()), "hinted spmm")


def test_hints_are_ignored_for_widths_without_a_hinted_kernel():
    """The marks act on the 512-byte tile only: with a narrower or a ragged width the hinted entry
    points run the plain kernels and give the same bits."""
    A = W.rmat(scale=18)
    d, meta = gpu_inputs(A)
    hot = capi.hot_columns(d.col, A.n, 512, budget_bytes=10000 * 512)
    assert hot is not None
    for n in (32, 64, 132, 20):
        Bd = W.dense(A.n, n, seed=n).cuda()
        plain = capi.spmm(meta, d.row_ptr, d.col, d.val, Bd)
        hinted = capi.spmm(meta, d.row_ptr, d.col, d.val, Bd, hot=hot)
        torch.cuda.synchronize()
        assert torch.equal(plain, hinted), n


def test_bitmap_with_a_cleared_flag_is_harmless_through_the_c_abi(oracle_cpu):
    """A caller that hands a bitmap straight to rode_spmm_f32_hot without reading its flag
    word: when the library judged the marks useless (flag 0) the kernel gives every row the
    normal cache priority; either way the result is the plain entry point's, bit for bit."""
    A = W.rmat(scale=19)
    d, meta = gpu_inputs(A)
    assert meta.m1 > 2 * 32 * 148                    # large enough for the hinted kernel to be chosen
    n, row_bytes = 128, 512
    bits, flag, bitmap = _bitmap(d.col, A.n, row_bytes, 20000 * row_bytes)
    assert flag == 1
    B = W.dense(A.n, n, seed=9).cuda()
    plain = capi.spmm(meta, d.row_ptr, d.col, d.val, B)
    cleared = bitmap.clone()
    cleared[-1] = 0
    for bm in (bitmap, cleared):
        got = capi.spmm(meta, d.row_ptr, d.col, d.val, B, hot=bm)
        torch.cuda.synchronize()
        assert torch.equal(got, plain)
    with pytest.raises(capi.RodeError):              # the bitmap's length is derived from k
        capi.spmm_raw(torch.float32, meta.m1, meta.m2, 0, n, d.val.data_ptr(), d.col.data_ptr(), d.row_ptr.data_ptr(),
                      meta.block_r_ind.data_ptr(), meta.residue_r_ind.data_ptr(), meta.st_off.data_ptr(),
                      B.data_ptr(), plain.data_ptr(), None, 0, hot=bitmap.data_ptr())


def test_bad_arguments_are_rejected():
    col = torch.zeros(8, dtype=torch.int32, device="cuda")
    bitmap = torch.zeros(4, dtype=torch.int32, device="cuda")
    with pytest.raises(capi.RodeError):
        capi.hot_columns_raw(8, 64, col.data_ptr(), 512, 0, bitmap.data_ptr(), None, 0)       # no workspace
    with pytest.raises(capi.RodeError):
        capi.hot_columns_raw(8, 64, col.data_ptr(), 0, 0, bitmap.data_ptr(), bitmap.data_ptr(), 1 << 20)  # row bytes 0
