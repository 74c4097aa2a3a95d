"""SDDMM through the C ABI against the reference fixtures, the CPU oracle (fp64-accumulated
ground truth), the reference's own kernels where built, and size-independent properties."""
import ctypes
import os

import numpy as np
import pytest
import torch

from oracle import ref
from rode_b200 import capi
from rode_b200 import workloads as W
from tests.helpers import assert_close_to_truth, run_reference_sddmm, sample_rows_csr, sddmm_abs_scale

pytestmark = pytest.mark.gpu
SEG_FOR_K = {32: 512, 64: 512, 128: 32}   # RoDe_SDDMM/rode_sddmm.py:35-38 (K = 64 follows K = 32)


def _run(A, lhs, rhs, k):
    d = A.to("cuda")
    meta = capi.preprocess(d.row_ptr, d.nnz, SEG_FOR_K[k], 32, 4)
    out = capi.sddmm(meta, d.row_ptr, d.col, d.val, lhs.cuda(), rhs.cuda())
    torch.cuda.synchronize()
    return d, meta, out


def _check(oracle_cpu, A, lhs, rhs, out, what):
    rp, col, val = A.row_ptr.numpy(), A.col.numpy(), A.val.numpy()
    truth = oracle_cpu.sddmm_f64acc(rp, col, val, lhs.numpy(), rhs.numpy(), threads=oracle_cpu.max_threads())
    return assert_close_to_truth(out.cpu().numpy(), truth,
                                 sddmm_abs_scale(rp, col, val, lhs.numpy(), rhs.numpy()), what)


def test_sddmm_matches_reference_fixtures(golden_dir):
    g = np.load(os.path.join(golden_dir, "sddmm_golden.npz"))
    for case in sorted({k.split("/")[0] for k in g.files}):
        a = {k: g[f"{case}/{k}"] for k in ("row_ptr", "col", "val", "lhs", "rhs", "out")}
        A = W.CSR(len(a["row_ptr"]) - 1, a["rhs"].shape[0], torch.from_numpy(a["row_ptr"]),
                  torch.from_numpy(a["col"]), torch.from_numpy(a["val"]))
        k = a["lhs"].shape[1]
        _, _, out = _run(A, torch.from_numpy(a["lhs"]), torch.from_numpy(a["rhs"]), k)
        # the fixture is the reference's fp32 CPU result; both sides are within the tolerance
        # of the exact value, so compare with twice the scaled floor
        scale = sddmm_abs_scale(a["row_ptr"], a["col"], a["val"], a["lhs"], a["rhs"])
        assert_close_to_truth(out.cpu().numpy(), a["out"].astype(np.float64), 2 * scale, case)


@pytest.mark.parametrize("k", [32, 64, 128])
def test_sddmm_families_against_oracle_and_reference(oracle_cpu, headroom, k):
    fams = {
        "bernoulli": W.bernoulli(),
        "zipf": W.zipf_rows(m=4096, n=4096, cap=4096),
        "stencil": W.stencil27(12),
        "pareto": W.pareto_rows(m=4096, n=8192, cap=3000),
        "rmat": W.rmat(scale=12),
    }
    for name, A in fams.items():
        lhs, rhs = W.dense(A.m, k, seed=5), W.dense(A.n, k, seed=6)
        d, meta, out = _run(A, lhs, rhs, k)
        stats = _check(oracle_cpu, A, lhs, rhs, out, f"{name} k={k}")
        config1 = name == "bernoulli" and k == 32
        if config1:
            headroom("1 Bernoulli 4096^2 SDDMM K=32 (all elements)", "ours", stats)
        assert torch.equal(out, capi.sddmm(meta, d.row_ptr, d.col, d.val, lhs.cuda(), rhs.cuda()))
        if ref.available() and k in (32, 128) and meta.m1 > 0 and meta.m2 > 0:
            oref = run_reference_sddmm(d, meta, lhs.cuda(), rhs.cuda())
            stats = _check(oracle_cpu, A, lhs, rhs, oref, f"reference {name} k={k}")
            if config1:
                headroom("1 Bernoulli 4096^2 SDDMM K=32 (all elements)", "reference kernels", stats)


def test_sddmm_edge_cases(oracle_cpu):
    def csr(lens, ncols, seed=0):
        rng = np.random.default_rng(seed)
        lens = np.asarray(lens)
        rp = np.concatenate([[0], np.cumsum(lens)]).astype(np.int32)
        col = np.concatenate([np.sort(rng.choice(ncols, l, replace=False)) for l in lens] + [np.zeros(0, np.int64)])
        val = rng.uniform(-1, 1, len(col)).astype(np.float32)
        return W.CSR(len(lens), ncols, torch.from_numpy(rp), torch.from_numpy(col.astype(np.int32)),
                     torch.from_numpy(val))

    cases = {
        "empty rows only": csr([0] * 37, 64),
        "single long row": csr([20000], 30000),
        "unaligned long rows": csr([3, 16384, 1, 1025, 2, 513, 0, 0, 545], 20000),
        "block only": csr([32, 64, 512, 1024, 96], 4096),
        "segment edges": csr([511, 512, 513, 1, 543, 544, 545, 31, 32, 33, 0, 1023, 1024, 1025, 63, 64, 65], 2048),
        "one entry": csr([1], 8),
    }
    for name, A in cases.items():
        for k in (32, 64, 128):
            lhs, rhs = W.dense(A.m, k, seed=7), W.dense(A.n, k, seed=8)
            d = A.to("cuda")
            meta = capi.preprocess(d.row_ptr, d.nnz, SEG_FOR_K[k], 32, 4)
            out0 = torch.full((max(A.nnz, 1),), float("nan"), device="cuda")[: A.nnz]
            out = capi.sddmm(meta, d.row_ptr, d.col, d.val, lhs.cuda(), rhs.cuda(), out=out0)
            if A.nnz:
                _check(oracle_cpu, A, lhs, rhs, out, f"{name} k={k}")   # every entry written exactly once


def test_reference_signature_entry_points(oracle_cpu):
    lib = capi.load()
    A = W.pareto_rows(m=4096, n=8192, cap=3000)
    vp = ctypes.c_void_p
    s1, s2 = torch.cuda.Stream(), torch.cuda.Stream()
    for name, k in (("RoDeSDDMM_n32", 32), ("RoDeSDDMM_n64", 64), ("RoDeSDDMM_n128", 128)):
        fn = getattr(lib, capi.CPP_SYMBOLS[name])
        fn.restype = None
        lhs, rhs = W.dense(A.m, k, seed=5), W.dense(A.n, k, seed=6)
        d = A.to("cuda")
        meta = capi.preprocess(d.row_ptr, d.nnz, SEG_FOR_K[k], 32, 4)
        l, r = lhs.cuda(), rhs.cuda()
        out = torch.zeros(A.nnz, device="cuda")
        torch.cuda.synchronize()
        fn(meta.m1, meta.m2, A.n, k, vp(meta.block_r_ind.data_ptr()), vp(meta.residue_r_ind.data_ptr()),
           vp(meta.st_off.data_ptr()), vp(d.row_ptr.data_ptr()), vp(d.col.data_ptr()), vp(d.val.data_ptr()),
           vp(l.data_ptr()), vp(r.data_ptr()), vp(out.data_ptr()), vp(s1.cuda_stream), vp(s2.cuda_stream))
        s1.synchronize()
        s2.synchronize()
        _check(oracle_cpu, A, lhs, rhs, out, name)


@pytest.mark.parametrize("family,k", [("stencil", 64), ("pareto", 32), ("pareto", 128), ("rmat", 64)])
def test_sddmm_full_size_properties(oracle_cpu, headroom, family, k):
    """Full-size matrices: a sample of rows against the oracle, and linearity in lhs."""
    A = {"stencil": lambda: W.stencil27(128, device="cuda"),
         "pareto": lambda: W.pareto_rows(device="cuda"),
         "rmat": lambda: W.rmat(scale=22, device="cuda")}[family]()
    meta = capi.preprocess(A.row_ptr, A.nnz, SEG_FOR_K[k], 32, 4)
    lhs1 = W.dense(A.m, k, device="cuda", seed=5)
    rhs = W.dense(A.n, k, device="cuda", seed=6)
    out1 = capi.sddmm(meta, A.row_ptr, A.col, A.val, lhs1, rhs)
    lens = (A.row_ptr[1:] - A.row_ptr[:-1]).long()
    g = torch.Generator(device="cuda").manual_seed(1)
    rows = torch.cat([torch.topk(lens, 8).indices, torch.randint(0, A.m, (4096,), device="cuda", generator=g)]).unique()
    rp, col, val, idx = sample_rows_csr(A, rows)
    lh, rh = lhs1[rows].cpu().numpy(), rhs.cpu().numpy()
    truth = oracle_cpu.sddmm_f64acc(rp, col, val, lh, rh, threads=oracle_cpu.max_threads())
    scale = sddmm_abs_scale(rp, col, val, lh, rh)
    idx_d = torch.from_numpy(idx).cuda()
    what = {"stencil": "3 stencil 128^3", "pareto": "4 Pareto 2^20", "rmat": "R-MAT 22"}[family] + f" SDDMM K={k} (row sample)"
    headroom(what, "ours", assert_close_to_truth(out1[idx_d].cpu().numpy(), truth, scale, f"{family} k={k} sample"))
    # the reference's kernels where they can run (K = 32 or 128, both lists non-empty, 32-bit offsets)
    if ref.available() and k in (32, 128) and meta.m1 > 0 and meta.m2 > 0 and (A.n - 1) * k < 2**29:
        oref = run_reference_sddmm(A, meta, lhs1, rhs)
        headroom(what, "reference kernels",
                 assert_close_to_truth(oref[idx_d].cpu().numpy(), truth, scale, f"{family} k={k} sample, reference"))
        del oref
    lhs2 = W.dense(A.m, k, device="cuda", seed=9)
    out2 = capi.sddmm(meta, A.row_ptr, A.col, A.val, lhs2, rhs)
    out3 = capi.sddmm(meta, A.row_ptr, A.col, A.val, 2 * lhs1 - lhs2, rhs)
    assert (out3 - (2 * out1 - out2)).abs().max().item() <= 1e-4


@pytest.mark.parametrize("k", [4, 36, 96, 160, 192, 252, 256])
def test_sddmm_other_widths(oracle_cpu, k):
    """Every K that is a multiple of 4 up to 256 behind the one entry point, on metadata of
    either segment length (the reference serves 32 and 128 only)."""
    A = W.pareto_rows(m=3000, n=5000, cap=2500, seed=13)
    lhs, rhs = W.dense(A.m, k, seed=5), W.dense(A.n, k, seed=6)
    d = A.to("cuda")
    for seg in (512, 32):
        meta = capi.preprocess(d.row_ptr, d.nnz, seg, 32, 4)
        out0 = torch.full((A.nnz,), float("nan"), device="cuda")
        out = capi.sddmm(meta, d.row_ptr, d.col, d.val, lhs.cuda(), rhs.cuda(), out=out0)
        torch.cuda.synchronize()
        _check(oracle_cpu, A, lhs, rhs, out, f"k={k} seg={seg}")


def test_sddmm_rejects_unsupported_widths():
    A = W.bernoulli(m=64, n=64).to("cuda")
    meta = capi.preprocess(A.row_ptr, A.nnz)
    for k in (0, 6, 260):
        x = torch.zeros((64, max(k, 1)), device="cuda")
        with pytest.raises(capi.RodeError):
            capi.sddmm_raw(meta.m1, meta.m2, 64, k, meta.block_r_ind.data_ptr(), meta.residue_r_ind.data_ptr(),
                           meta.st_off.data_ptr(), A.row_ptr.data_ptr(), A.col.data_ptr(), A.val.data_ptr(),
                           x.data_ptr(), x.data_ptr(), x.data_ptr())


@pytest.mark.parametrize("k", [32, 64])
def test_sddmm_row_mode_every_entry(oracle_cpu, k):
    """A residue list long enough for the residue kernel to give its warps 32 rows each, with
    rows of every length from 0 to 31 mixed at random and a ragged last warp: warps whose rows
    are long take the row mode (one lane group per row), the others the stream; every entry of
    the result is checked, and a NaN-filled output shows entries written never or twice."""
    m, n = 520_001, 60_000
    g = torch.Generator().manual_seed(77)
    lens = torch.randint(0, 32, (m,), generator=g)
    lens[torch.rand(m, generator=g) < 0.2] = 0                 # empty rows in between
    dense_part = slice(100_000, 200_000)                       # a stretch of long rows only
    lens[dense_part] = torch.randint(20, 32, (100_000,), generator=g)
    rp = torch.zeros(m + 1, dtype=torch.int64)
    torch.cumsum(lens, 0, out=rp[1:])
    nnz = int(rp[-1])
    # ascending distinct columns per row: a random start plus a stride, modulo nothing (n is large enough)
    row_of = torch.repeat_interleave(torch.arange(m), lens)
    pos = torch.arange(nnz) - rp[:-1][row_of]
    start = torch.randint(0, n - 32 * 40, (m,), generator=g)
    stride = torch.randint(1, 40, (m,), generator=g)
    col = (start[row_of] + pos * stride[row_of]).to(torch.int32)
    val = torch.rand(nnz, generator=g) * 2 - 1
    A = W.CSR(m, n, rp.to(torch.int32), col, val)
    lhs, rhs = W.dense(m, k, seed=5), W.dense(n, k, seed=6)
    d = A.to("cuda")
    meta = capi.preprocess(d.row_ptr, d.nnz, 512, 32, 4)
    assert meta.m2 > 31 * 4 * 24 * 148      # enough rows for 32 per warp on a 148-SM part
    out0 = torch.full((nnz,), float("nan"), device="cuda")
    out = capi.sddmm(meta, d.row_ptr, d.col, d.val, lhs.cuda(), rhs.cuda(), out=out0)
    torch.cuda.synchronize()
    _check(oracle_cpu, A, lhs, rhs, out, f"row mode k={k}")


def test_sddmm_calls_on_different_stream_pairs_run_side_by_side():
    """Large block grids run as one resident wave whose warps claim segments from a counter that
    the library keeps per pair of streams: two calls on different pairs, in flight together,
    must not disturb each other, and repeated calls on one pair reuse its counter."""
    A = W.rmat(scale=21, device="cuda")
    meta = capi.preprocess(A.row_ptr, A.nnz, 512, 32, 4)
    assert meta.m1 > 16 * 32 * 148         # enough segments for the block kernel to run as a persistent grid
    k = 64
    lhs, rhs = W.dense(A.m, k, device="cuda", seed=5), W.dense(A.n, k, device="cuda", seed=6)
    want = capi.sddmm(meta, A.row_ptr, A.col, A.val, lhs, rhs)
    torch.cuda.synchronize()
    pairs = [(torch.cuda.Stream(), torch.cuda.Stream()) for _ in range(3)]
    outs = [torch.full((A.nnz,), float("nan"), device="cuda") for _ in pairs]
    for _ in range(2):                       # second round: every pair uses its counter again
        for (s1, s2), out in zip(pairs, outs):
            out.fill_(float("nan"))
        torch.cuda.synchronize()
        for (s1, s2), out in zip(pairs, outs):
            capi.sddmm(meta, A.row_ptr, A.col, A.val, lhs, rhs, out=out, stream1=s1, stream2=s2)
        torch.cuda.synchronize()
        for out in outs:
            assert torch.equal(out, want)
