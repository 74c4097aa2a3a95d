"""Bounds and alignment sweep in place of a memory checker: every row length 0..130 at every
start alignment 0..3, for every SpMM width and every SDDMM K (both segment lengths the
reference uses), with guard zones around every output that must stay untouched."""
import numpy as np
import pytest
import torch

from rode_b200 import capi
from rode_b200 import workloads as W
from tests.helpers import assert_close_to_truth, sddmm_abs_scale, spmm_abs_scale

pytestmark = pytest.mark.gpu
GUARD = 4096          # elements of guard zone on each side
CANARY = -12345.678


def _sweep_matrix(align: int, ncols: int = 1100, seed: int = 0):
    """Rows of length 0..130 in random order, each followed by a 1-entry row so that starts
    visit every residue mod 4; `align` extra entries in row 0 shift everything."""
    rng = np.random.default_rng(seed + align)
    lens = rng.permutation(np.arange(0, 131))
    lens = np.stack([lens, np.ones_like(lens)], 1).reshape(-1)
    lens = np.concatenate([[align], lens, [513, 0, 1025, 31, 32, 33]])
    rp = np.concatenate([[0], np.cumsum(lens)]).astype(np.int32)
    col = np.concatenate([np.sort(rng.choice(ncols, l, replace=False)) for l in lens]).astype(np.int32)
    val = rng.uniform(-1, 1, len(col)).astype(np.float32)
    return W.CSR(len(lens), ncols, torch.from_numpy(rp), torch.from_numpy(col), torch.from_numpy(val))


def _guarded(shape):
    n = int(np.prod(shape))
    buf = torch.full((n + 2 * GUARD,), CANARY, device="cuda")
    body = buf[GUARD:GUARD + n].view(*shape) if n else buf[GUARD:GUARD].view(*shape)
    return buf, body


def _guards_intact(buf, n):
    return bool((buf[:GUARD] == CANARY).all()) and bool((buf[GUARD + n:] == CANARY).all())


@pytest.mark.parametrize("align", [0, 1, 2, 3])
def test_spmm_all_lengths_and_alignments(oracle_cpu, align):
    A = _sweep_matrix(align)
    d = A.to("cuda")
    rp, col, val = A.row_ptr.numpy(), A.col.numpy(), A.val.numpy()
    # segment length 512 is what the reference's SpMM uses; 32 (its SDDMM K = 128 setting) cuts
    # rows into many more segments and exercises the workspace / fix-up path much harder
    for seg, n in ((512, 32), (512, 64), (512, 128), (512, 96), (32, 32), (32, 128), (64, 64)):
        meta = capi.preprocess(d.row_ptr, d.nnz, seg, 32, 4)
        B = W.dense(A.n, n, seed=n)
        buf, C = _guarded((A.m, n))
        C.zero_()
        ws_bytes = capi.spmm_workspace_bytes(meta.m1, n, 4)
        wbuf, ws = _guarded((max(ws_bytes // 4, 1),))
        capi.spmm(meta, d.row_ptr, d.col, d.val, B.cuda(), C=C, workspace=ws)
        torch.cuda.synchronize()
        truth = oracle_cpu.spmm_f64acc(rp, col, val, B.numpy())
        assert_close_to_truth(C.cpu().numpy(), truth, spmm_abs_scale(rp, col, val, B.numpy()), f"align={align} seg={seg} n={n}")
        assert _guards_intact(buf, A.m * n) and _guards_intact(wbuf, max(ws_bytes // 4, 1))


@pytest.mark.parametrize("align", [0, 1, 2, 3])
def test_sddmm_all_lengths_and_alignments(oracle_cpu, align):
    A = _sweep_matrix(align, seed=100)
    d = A.to("cuda")
    rp, col, val = A.row_ptr.numpy(), A.col.numpy(), A.val.numpy()
    for k, seg in ((32, 512), (64, 512), (128, 32), (128, 512), (32, 32)):
        meta = capi.preprocess(d.row_ptr, d.nnz, seg, 32, 4)
        lhs, rhs = W.dense(A.m, k, seed=k), W.dense(A.n, k, seed=k + 1)
        buf, out = _guarded((A.nnz,))
        capi.sddmm(meta, d.row_ptr, d.col, d.val, lhs.cuda(), rhs.cuda(), out=out)
        torch.cuda.synchronize()
        truth = oracle_cpu.sddmm_f64acc(rp, col, val, lhs.numpy(), rhs.numpy())
        # every entry written (no canary left) and correct
        assert_close_to_truth(out.cpu().numpy(), truth, sddmm_abs_scale(rp, col, val, lhs.numpy(), rhs.numpy()),
                              f"align={align} k={k} seg={seg}")
        assert _guards_intact(buf, A.nnz)


def test_preprocess_outputs_stay_inside_their_counts():
    A = _sweep_matrix(3, seed=7).to("cuda")
    for seg in (512, 32):
        cap = capi.preprocess_capacity(seg, 4, A.m, A.nnz)
        bbuf, blk = _guarded((cap,))
        sbuf, st = _guarded((cap + 1,))
        rbuf, res = _guarded((A.m,))
        blk_i, st_i, res_i = (torch.full(t.shape, -1, dtype=torch.int32, device="cuda") for t in (blk, st, res))
        cnt = torch.zeros(2, dtype=torch.int32, device="cuda")
        ws_bytes = capi.preprocess_workspace_bytes(A.m)
        ws = torch.empty(ws_bytes, dtype=torch.uint8, device="cuda")
        capi.preprocess_raw(seg, 32, 4, A.m, A.row_ptr.data_ptr(), blk_i.data_ptr(), st_i.data_ptr(), res_i.data_ptr(),
                            cnt.data_ptr(), cnt.data_ptr() + 4, ws.data_ptr(), ws_bytes, torch.cuda.current_stream())
        torch.cuda.synchronize()
        m1, m2 = cnt.cpu().tolist()
        assert m1 <= cap and bool((blk_i[m1:] == -1).all()) and bool((st_i[m1 + 1:] == -1).all())
        assert bool((res_i[m2:] == -1).all()) and bool((blk_i[:m1] >= 0).all()) and bool((res_i[:m2] >= 0).all())
