"""SpMM through the C ABI against the CPU oracle (fp64-accumulated ground truth), the
reference's own kernels where they are built, and size-independent properties."""
import ctypes

import numpy as np
import pytest
import torch

from oracle import ref
from rode_b200 import capi
from rode_b200 import workloads as W
from tests.helpers import (assert_close_to_truth, gpu_inputs, run_reference_spmm, sample_rows_csr, spmm_abs_scale)

pytestmark = pytest.mark.gpu


def _small_families():
    return {
        "bernoulli": W.bernoulli(),                                   # config 1 at full size
        "zipf": W.zipf_rows(m=4096, n=4096, cap=4096, mean=16),       # split rows
        "stencil": W.stencil27(12),                                   # residue only, m1 == 0
        "pareto": W.pareto_rows(m=4096, n=8192, cap=3000),
        "rmat": W.rmat(scale=12),                                     # many empty rows
    }


def _check_against_truth(oracle_cpu, A, B_host, C_dev, what):
    rp, col, val = A.row_ptr.numpy(), A.col.numpy(), A.val.numpy()
    truth = oracle_cpu.spmm_f64acc(rp, col, val, B_host, threads=oracle_cpu.max_threads())
    return assert_close_to_truth(C_dev.cpu().numpy(), truth, spmm_abs_scale(rp, col, val, B_host), what)


@pytest.mark.parametrize("n", [32, 64, 128])
def test_spmm_families_against_oracle_and_reference(oracle_cpu, headroom, n):
    for name, A in _small_families().items():
        d, meta = gpu_inputs(A)
        B = W.dense(A.n, n, seed=3)
        Bd = B.cuda()
        C = capi.spmm(meta, d.row_ptr, d.col, d.val, Bd)
        torch.cuda.synchronize()
        stats = _check_against_truth(oracle_cpu, A, B.numpy(), C, f"{name} n={n}")
        config1 = name == "bernoulli" and n == 32
        if config1:
            headroom("1 Bernoulli 4096^2 SpMM N=32 (all elements)", "ours", stats)
        # deterministic: no floating-point atomics
        C2 = capi.spmm(meta, d.row_ptr, d.col, d.val, Bd)
        assert torch.equal(C, C2)
        # the reference's own kernels on the same inputs (needs both kernels to have work)
        if ref.available() and meta.m1 > 0 and meta.m2 > 0 and n in (32, 128):
            Cref = run_reference_spmm(d, meta, Bd, n)
            stats = _check_against_truth(oracle_cpu, A, B.numpy(), Cref, f"reference {name} n={n}")
            if config1:
                headroom("1 Bernoulli 4096^2 SpMM N=32 (all elements)", "reference kernels", stats)
            scale = spmm_abs_scale(A.row_ptr.numpy(), A.col.numpy(), A.val.numpy(), B.numpy())
            assert_close_to_truth(C.cpu().numpy(), Cref.cpu().numpy().astype(np.float64), 2 * scale,
                                  f"ours vs reference {name} n={n}")


@pytest.mark.parametrize("n", [96, 160, 256])
def test_spmm_other_widths(oracle_cpu, n):
    A = W.pareto_rows(m=2048, n=3000, cap=1400, seed=9)
    d, meta = gpu_inputs(A)
    B = W.dense(A.n, n, seed=4)
    C = capi.spmm(meta, d.row_ptr, d.col, d.val, B.cuda())
    _check_against_truth(oracle_cpu, A, B.numpy(), C, f"n={n}")


def test_spmm_widths_the_tiles_do_not_divide(oracle_cpu):
    """Any multiple of 4 columns behind the one entry point (the reference serves multiples of its
    32- or 64-wide tile only): the narrowest lane-group shape that covers the row, or 512-byte tiles
    whose last one is partly empty.  A small matrix (small-grid kernels, one warp per residue row)
    and one whose grids fill the GPU (batched and per-group residue kernels); C sits inside a larger
    buffer whose guard words must survive."""
    matrices = {
        "zipf 2048 (small grids)": W.zipf_rows(m=2048, n=2048, cap=2048),
        "pareto 65536 (full grids)": W.pareto_rows(m=1 << 16, n=1 << 16, cap=20000, seed=5),
    }
    for name, A in matrices.items():
        d, meta = gpu_inputs(A)
        assert meta.m1 > 0 and meta.m2 > 0
        rp = A.row_ptr.numpy()
        assert ((rp[1:] - rp[:-1]) > 600).any()  # rows cut into several segments: the fix-up grid runs
        for n in (4, 8, 12, 20, 28, 36, 44, 100, 132, 200, 260):
            B = W.dense(A.n, n, seed=n)
            guard = 64
            buf = torch.zeros(A.m * n + guard, device="cuda")
            buf[A.m * n:] = 12345.0
            C = buf[:A.m * n].view(A.m, n)
            capi.spmm(meta, d.row_ptr, d.col, d.val, B.cuda(), C=C)
            torch.cuda.synchronize()
            assert bool((buf[A.m * n:] == 12345.0).all()), f"{name} n={n}: wrote past the end of C"
            _check_against_truth(oracle_cpu, A, B.numpy(), C, f"{name} n={n}")
    # double: 16-byte vectors hold two columns
    A = matrices["zipf 2048 (small grids)"]
    d, meta = gpu_inputs(A)
    for n in (4, 12, 20, 36, 68, 132):
        B = W.dense(A.n, n, seed=n, dtype=torch.float64)
        C = capi.spmm(meta, d.row_ptr, d.col, d.val.double(), B.cuda())
        truth = oracle_cpu.spmm_f64(A.row_ptr.numpy(), A.col.numpy(), A.val.numpy().astype(np.float64), B.numpy())
        assert np.allclose(C.cpu().numpy(), truth, rtol=1e-12, atol=1e-12), n
    # not a multiple of 4: refused
    for n in (6, 30, 130):
        with pytest.raises(capi.RodeError):
            capi.spmm(meta, d.row_ptr, d.col, d.val, torch.zeros((A.n, n), device="cuda"))


def test_spmm_operands_aligned_to_16_bytes_only(oracle_cpu):
    """The 128-byte tile uses 32-byte loads when B, C and the workspace are 32-byte aligned and the
    16-byte shapes otherwise (other lane groups, so another summation order): both against the oracle."""
    A = W.pareto_rows(m=20000, n=20000, cap=3000, seed=11)
    d, meta = gpu_inputs(A)
    for n in (32, 96):
        B = W.dense(A.n, n, seed=12)
        Bd = B.cuda()
        assert Bd.data_ptr() % 32 == 0
        C_wide = capi.spmm(meta, d.row_ptr, d.col, d.val, Bd)
        _check_against_truth(oracle_cpu, A, B.numpy(), C_wide, f"32-byte aligned n={n}")
        buf_b = torch.empty(A.n * n + 4, device="cuda")
        B16 = buf_b[4:].view(A.n, n)
        B16.copy_(Bd)
        buf_c = torch.zeros(A.m * n + 4, device="cuda")
        C16 = buf_c[4:].view(A.m, n)
        assert B16.data_ptr() % 32 == 16 and C16.data_ptr() % 32 == 16
        capi.spmm(meta, d.row_ptr, d.col, d.val, B16, C=C16)
        _check_against_truth(oracle_cpu, A, B.numpy(), C16, f"16-byte aligned n={n}")
        assert float(buf_c[:4].abs().sum()) == 0.0


def test_spmm_edge_cases(oracle_cpu):
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
        "block only (m2 == 0)": csr([32, 64, 512, 1024, 96], 4096),
        "exact segment edges": csr([511, 512, 513, 1, 543, 544, 545, 31, 32, 33, 0, 1023, 1024, 1025], 2048),
        "one entry": csr([1], 8),
    }
    for name, A in cases.items():
        d, meta = gpu_inputs(A)
        if name.startswith("block only"):
            assert meta.m2 == 0 and meta.m1 > 0
        for n in (32, 128):
            B = W.dense(A.n, n, seed=6)
            # rows with a nonzero are written, not accumulated: start from garbage there; rows
            # without one are never touched and stay as the caller zero-filled them
            C0 = torch.zeros((A.m, n), device="cuda")
            nonempty = (d.row_ptr[1:] > d.row_ptr[:-1])
            C0[nonempty] = float("nan")
            C = capi.spmm(meta, d.row_ptr, d.col, d.val, B.cuda(), C=C0)
            _check_against_truth(oracle_cpu, A, B.numpy(), C, f"{name} n={n}")
    # M == 0: nothing to launch
    empty = W.CSR(0, 8, torch.zeros(1, dtype=torch.int32), torch.zeros(0, dtype=torch.int32), torch.zeros(0))
    d, meta = gpu_inputs(empty)
    assert (meta.m1, meta.m2) == (0, 0)
    assert capi.spmm(meta, d.row_ptr, d.col, d.val, torch.zeros((8, 32), device="cuda")).shape == (0, 32)


def test_spmm_fp64(oracle_cpu):
    A = W.zipf_rows(m=2048, n=2048, cap=2048)
    d, meta = gpu_inputs(A)
    for n in (32, 128, 48):
        B = W.dense(A.n, n, seed=8, dtype=torch.float64)
        C = capi.spmm(meta, d.row_ptr, d.col, d.val.double(), B.cuda())
        truth = oracle_cpu.spmm_f64(A.row_ptr.numpy(), A.col.numpy(), A.val.numpy().astype(np.float64), B.numpy())
        assert np.allclose(C.cpu().numpy(), truth, rtol=1e-12, atol=1e-12)
    # the reference's double kernels need double values: run them explicitly
    if ref.available():
        B = W.dense(A.n, 32, seed=8, dtype=torch.float64).cuda()
        dd = W.CSR(d.m, d.n, d.row_ptr, d.col, d.val.double())
        Cref = run_reference_spmm(dd, meta, B, 32)
        C = capi.spmm(meta, d.row_ptr, d.col, dd.val, B)
        assert torch.allclose(C, Cref, rtol=1e-11, atol=1e-11)


def test_reference_signature_entry_points(oracle_cpu):
    """RoDeSpmm_n32 / RoDeSpmm_n128 with the reference's argument order, library-owned workspace."""
    lib = capi.load()
    A = W.zipf_rows(m=4096, n=4096, cap=4096)
    d, meta = gpu_inputs(A)
    s1, s2 = torch.cuda.Stream(), torch.cuda.Stream()
    vp = ctypes.c_void_p
    for name, n in (("RoDeSpmm_n32_f32", 32), ("RoDeSpmm_n128_f32", 128), ("RoDeSpmm_n32_f32", 96)):
        fn = getattr(lib, capi.CPP_SYMBOLS[name])
        fn.restype = None
        B = W.dense(A.n, n, seed=2)
        Bd = B.cuda()
        C = torch.zeros((A.m, n), device="cuda")
        torch.cuda.synchronize()
        fn(meta.m1, meta.m2, A.n, n, vp(d.val.data_ptr()), vp(d.col.data_ptr()), vp(d.row_ptr.data_ptr()),
           vp(meta.block_r_ind.data_ptr()), vp(meta.residue_r_ind.data_ptr()), vp(meta.st_off.data_ptr()),
           vp(Bd.data_ptr()), vp(C.data_ptr()), vp(s1.cuda_stream), vp(s2.cuda_stream))
        s1.synchronize()
        s2.synchronize()
        _check_against_truth(oracle_cpu, A, B.numpy(), C, name)


def test_reference_signature_double_overloads(oracle_cpu):
    """The two `double` overloads of RoDeSpmm_n32 / RoDeSpmm_n128 (RoDe_SpMM/RoDeSpmm.h:10-14),
    called through their mangled names with the reference's argument order."""
    lib = capi.load()
    A = W.zipf_rows(m=4096, n=4096, cap=4096)
    d, meta = gpu_inputs(A)
    vals = d.val.double()
    s1, s2 = torch.cuda.Stream(), torch.cuda.Stream()
    vp = ctypes.c_void_p
    for name, n in (("RoDeSpmm_n32_f64", 32), ("RoDeSpmm_n128_f64", 128), ("RoDeSpmm_n128_f64", 64)):
        fn = getattr(lib, capi.CPP_SYMBOLS[name])
        fn.restype = None
        B = W.dense(A.n, n, seed=2, dtype=torch.float64)
        Bd = B.cuda()
        C = torch.zeros((A.m, n), device="cuda", dtype=torch.float64)
        torch.cuda.synchronize()
        fn(meta.m1, meta.m2, A.n, n, vp(vals.data_ptr()), vp(d.col.data_ptr()), vp(d.row_ptr.data_ptr()),
           vp(meta.block_r_ind.data_ptr()), vp(meta.residue_r_ind.data_ptr()), vp(meta.st_off.data_ptr()),
           vp(Bd.data_ptr()), vp(C.data_ptr()), vp(s1.cuda_stream), vp(s2.cuda_stream))
        s1.synchronize()
        s2.synchronize()
        truth = oracle_cpu.spmm_f64(A.row_ptr.numpy(), A.col.numpy(), A.val.numpy().astype(np.float64), B.numpy())
        assert np.allclose(C.cpu().numpy(), truth, rtol=1e-12, atol=1e-12), name


def test_work_enqueued_after_spmm_sees_the_block_kernel_results():
    """Stream order after a call without split rows.  The fix-up grid is a programmatic
    dependent of the block grid and its warps leave early when their segments hold no split
    row; its first CTA nevertheless waits for the block grid, so the fix-up grid cannot
    complete, and nothing enqueued behind it can start, before the block grid has finished.
    Checked with a block grid that runs for milliseconds: an asynchronous copy of C to the
    host right behind the call, on the same stream, must see every row."""
    A = W.pareto_rows(cap=500, device="cuda")             # 2^20 rows, none longer than one segment
    meta = capi.preprocess(A.row_ptr, A.nnz)
    seg_rows = meta.block_r_ind[: meta.m1].long()
    assert meta.m1 > 0 and meta.m2 > 0
    assert int(torch.unique(seg_rows).numel()) == meta.m1  # one segment per row: no split rows
    n = 128
    B = W.dense(A.n, n, device="cuda", seed=3)
    stream = torch.cuda.Stream()
    host = torch.empty((A.m, n), dtype=torch.float32).pin_memory()
    done = torch.cuda.Event()
    for attempt in range(3):
        C = torch.zeros((A.m, n), device="cuda")
        host.fill_(float("nan"))
        torch.cuda.synchronize()
        with torch.cuda.stream(stream):
            capi.spmm(meta, A.row_ptr, A.col, A.val, B, C=C, stream1=stream, stream2=stream)
            host.copy_(C, non_blocking=True)
            done.record(stream)
        done.synchronize()
        early = host.clone()
        torch.cuda.synchronize()
        assert torch.equal(early, C.cpu()), f"attempt {attempt}: the copy overtook the block kernel"
    want = capi.spmm(meta, A.row_ptr, A.col, A.val, B)     # a second, fully synchronised run
    torch.cuda.synchronize()
    assert torch.equal(early, want.cpu())


def test_spmm_full_size_heavy_tail_config(oracle_cpu, headroom):
    """Config 2 at full size (65536 x 65536 Zipf rows, N = 128): every element checked, ours
    and the reference's own kernels."""
    A = W.zipf_rows(device="cuda")
    meta = capi.preprocess(A.row_ptr, A.nnz)
    B = W.dense(A.n, 128, device="cuda", seed=3)
    C = capi.spmm(meta, A.row_ptr, A.col, A.val, B)
    h = A.to("cpu")
    what = "2 Zipf 65536^2 SpMM N=128 (all elements)"
    headroom(what, "ours", _check_against_truth(oracle_cpu, h, B.cpu().numpy(), C, "config 2"))
    if ref.available() and meta.m1 > 0 and meta.m2 > 0:
        Cref = run_reference_spmm(A, meta, B, 128)
        headroom(what, "reference kernels",
                 _check_against_truth(oracle_cpu, h, B.cpu().numpy(), Cref, "config 2, reference kernels"))


@pytest.mark.parametrize("family,n", [("stencil", 64), ("pareto", 128), ("rmat", 128)])
def test_spmm_full_size_properties(oracle_cpu, headroom, family, n):
    """Full-size matrices: linearity in B, and exact agreement with the oracle on a sample of
    rows (longest rows, empty rows and a random draw)."""
    A = {"stencil": lambda: W.stencil27(128, device="cuda"),
         "pareto": lambda: W.pareto_rows(device="cuda"),
         "rmat": lambda: W.rmat(scale=22, device="cuda")}[family]()
    meta = capi.preprocess(A.row_ptr, A.nnz)
    B1 = W.dense(A.n, n, device="cuda", seed=3)
    C1 = capi.spmm(meta, A.row_ptr, A.col, A.val, B1)
    # sample of rows against the oracle
    lens = (A.row_ptr[1:] - A.row_ptr[:-1]).long()
    g = torch.Generator(device="cuda").manual_seed(1)
    rows = torch.cat([torch.topk(lens, 16).indices, torch.nonzero(lens == 0).flatten()[:64],
                      torch.randint(0, A.m, (4096,), device="cuda", generator=g)]).unique()
    rp, col, val, _ = sample_rows_csr(A, rows)
    Bh = B1.cpu().numpy()
    truth = oracle_cpu.spmm_f64acc(rp, col, val, Bh, threads=oracle_cpu.max_threads())
    scale = spmm_abs_scale(rp, col, val, Bh)
    what = {"stencil": "3 stencil 128^3", "pareto": "4 Pareto 2^20", "rmat": "R-MAT 22"}[family] + f" SpMM N={n} (row sample)"
    headroom(what, "ours", assert_close_to_truth(C1[rows].cpu().numpy(), truth, scale, f"{family} sample"))
    # the reference's kernels where their preconditions hold (both lists non-empty, 32-bit byte offsets)
    if ref.available() and meta.m1 > 0 and meta.m2 > 0 and n in (32, 128) and (A.n - 1) * n * 4 < 2**31:
        Cref = run_reference_spmm(A, meta, B1, n)
        headroom(what, "reference kernels",
                 assert_close_to_truth(Cref[rows].cpu().numpy(), truth, scale, f"{family} sample, reference kernels"))
        del Cref
    # linearity: S(2 B1 - B2) == 2 S B1 - S B2 up to rounding of the combination
    B2 = W.dense(A.n, n, device="cuda", seed=4)
    C2 = capi.spmm(meta, A.row_ptr, A.col, A.val, B2)
    C3 = capi.spmm(meta, A.row_ptr, A.col, A.val, 2 * B1 - B2)
    resid = (C3 - (2 * C1 - C2)).abs().max().item()
    assert resid <= 1e-3 * max(1.0, C1.abs().max().item()), resid
    del C2, C3


def test_spmm_matches_reference_kernel_fixtures(oracle_cpu, golden_dir):
    """tests/golden/spmm_golden.npz: outputs of the reference's own SpMM kernels."""
    import os

    g = np.load(os.path.join(golden_dir, "spmm_golden.npz"))
    for case in sorted({k.split("/")[0] for k in g.files}):
        a = {k: g[f"{case}/{k}"] for k in ("row_ptr", "col", "val", "B", "C")}
        A = W.CSR(len(a["row_ptr"]) - 1, a["B"].shape[0], torch.from_numpy(a["row_ptr"]), torch.from_numpy(a["col"]),
                  torch.from_numpy(a["val"]))
        d, meta = gpu_inputs(A)
        C = capi.spmm(meta, d.row_ptr, d.col, d.val, torch.from_numpy(a["B"]).cuda())
        scale = spmm_abs_scale(a["row_ptr"], a["col"], a["val"], a["B"])
        assert_close_to_truth(C.cpu().numpy(), a["C"].astype(np.float64), 2 * scale, case)


def test_spmm_persistent_grids_on_stream_pairs_in_flight_together():
    """Grids of more than two waves run as one resident wave whose warps claim their work from
    counters at the end of the workspace.  Calls with workspaces of their own (C ABI), and calls
    through the reference's signature (library-owned workspaces, one per pair of streams), on
    different stream pairs and in flight together, must all give the result of a lone call."""
    lib = capi.load()
    A = W.rmat(scale=22, device="cuda")
    meta = capi.preprocess(A.row_ptr, A.nnz)
    # enough segments and enough bundles of 32 residue rows for both kernels to run as persistent grids
    assert meta.m1 > 16 * 32 * 148 and meta.m2 > 16 * 32 * 32 * 148
    n = 128
    B = W.dense(A.n, n, device="cuda", seed=3)
    want = capi.spmm(meta, A.row_ptr, A.col, A.val, B)
    torch.cuda.synchronize()
    pairs = [(torch.cuda.Stream(), torch.cuda.Stream()) for _ in range(4)]
    outs = [torch.zeros((A.m, n), device="cuda") for _ in pairs]
    fn = getattr(lib, capi.CPP_SYMBOLS["RoDeSpmm_n128_f32"])
    fn.restype = None
    vp = ctypes.c_void_p
    for _ in range(2):                       # second round: buffers and counters are used again
        for out in outs:
            out.zero_()
        torch.cuda.synchronize()
        for i, ((s1, s2), out) in enumerate(zip(pairs, outs)):
            if i % 2 == 0:
                capi.spmm(meta, A.row_ptr, A.col, A.val, B, C=out, stream1=s1, stream2=s2)
            else:
                fn(meta.m1, meta.m2, A.n, n, vp(A.val.data_ptr()), vp(A.col.data_ptr()), vp(A.row_ptr.data_ptr()),
                   vp(meta.block_r_ind.data_ptr()), vp(meta.residue_r_ind.data_ptr()), vp(meta.st_off.data_ptr()),
                   vp(B.data_ptr()), vp(out.data_ptr()), vp(s1.cuda_stream), vp(s2.cuda_stream))
        torch.cuda.synchronize()
        for out in outs:
            assert torch.equal(out, want)
