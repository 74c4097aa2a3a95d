"""GPU row decomposition through the C ABI: bit-exact against the reference fixtures and the
CPU oracle, on the reference's parameter sets, edge cases and the benchmark matrix families."""
import ctypes
import os

import numpy as np
import pytest
import torch

from rode_b200 import capi
from rode_b200 import workloads as W

pytestmark = pytest.mark.gpu
PARAMS = ((512, 32, 4), (32, 32, 4))


def _gpu(rp_np, seg, kb, vec):
    rp = torch.from_numpy(np.ascontiguousarray(rp_np, np.int32)).cuda()
    meta = capi.preprocess(rp, int(rp_np[-1]), seg, kb, vec)
    return (meta.block_r_ind[: meta.m1].cpu().numpy(), meta.st_off.cpu().numpy(),
            meta.residue_r_ind[: meta.m2].cpu().numpy(), meta.m1, meta.m2)


def _same(got, want):
    assert (got[3], got[4]) == (want[3], want[4])
    for g, w in zip(got[:3], want[:3]):
        assert np.array_equal(g, w)


def test_gpu_preprocess_matches_reference_fixtures(golden_dir):
    g = np.load(os.path.join(golden_dir, "preprocess_golden.npz"))
    for case in sorted({k.split("/")[0] for k in g.files}):
        rp = g[f"{case}/row_ptr"]
        for seg, kb, vec in PARAMS:
            tag = f"{case}/{seg}_{kb}_{vec}"
            want = (g[f"{tag}/block_r_ind"], g[f"{tag}/st_off"], g[f"{tag}/residue_r_ind"],
                    *g[f"{tag}/counts"].tolist())
            _same(_gpu(rp, seg, kb, vec), want)


@pytest.mark.parametrize("family", ["bernoulli", "zipf", "stencil", "pareto", "rmat"])
def test_gpu_preprocess_matches_oracle_on_matrix_families(oracle_cpu, family):
    A = {"bernoulli": lambda: W.bernoulli(device="cuda"),
         "zipf": lambda: W.zipf_rows(device="cuda"),
         "stencil": lambda: W.stencil27(128, device="cuda"),
         "pareto": lambda: W.pareto_rows(device="cuda"),
         "rmat": lambda: W.rmat(scale=21, device="cuda")}[family]()
    rp = A.row_ptr.cpu().numpy()
    for seg, kb, vec in PARAMS + ((64, 32, 4), (1024, 64, 8)):
        _same(_gpu(rp, seg, kb, vec), oracle_cpu.preprocess(rp, seg, kb, vec))


def test_gpu_preprocess_tile_boundaries_and_long_rows(oracle_cpu):
    rng = np.random.default_rng(5)
    for m in (1, 2, 1023, 1024, 1025, 2047, 2048, 2049, 4097, 6145):
        lens = rng.integers(0, 70, m)
        lens[rng.integers(0, m)] = 300000          # hundreds of segments in one row
        lens[-1] = 5000                            # long last row
        rp = np.concatenate([[0], np.cumsum(lens)]).astype(np.int32)
        # the last two sets are not powers of two: they take the kernels' generic division path
        for seg, kb, vec in PARAMS + ((96, 24, 3), (480, 60, 5)):
            _same(_gpu(rp, seg, kb, vec), oracle_cpu.preprocess(rp, seg, kb, vec))


def test_gpu_preprocess_more_tiles_than_one_scan_pass(oracle_cpu):
    """More tiles (of 2048 rows) than the 2048 that the last CTA's scan takes per pass."""
    rng = np.random.default_rng(6)
    m = 8192 * 1024 + 5000
    lens = rng.integers(0, 40, m)
    lens[rng.integers(0, m, 50)] = 3000
    rp = np.concatenate([[0], np.cumsum(lens)]).astype(np.int32)
    _same(_gpu(rp, 512, 32, 4), oracle_cpu.preprocess(rp, 512, 32, 4))


def test_gpu_preprocess_tiles_with_more_segments_than_the_staging_holds(oracle_cpu):
    """A tile's segments are put in order in shared memory (2048 entries), rows of more than 8
    segments by whole warps.  Tiles with more segments take the direct path; tiles next to them the
    staged one."""
    rng = np.random.default_rng(8)
    m = 5 * 2048 + 77
    lens = rng.integers(0, 70, m)
    lens[100:420] = rng.integers(290, 900, 320)        # tile 0: 320 long rows, > 2048 segments at seg 32
    lens[2048 + 5: 2048 + 40] = 330                     # tile 1: a few long rows, staged
    lens[3 * 2048: 3 * 2048 + 2048] = 33                # tile 3: exactly one segment per row (2048: still staged)
    lens[4 * 2048 + 9] = 70000                          # tile 4: one row of 2188 segments at seg 32
    rp = np.concatenate([[0], np.cumsum(lens)]).astype(np.int32)
    for seg, kb, vec in PARAMS + ((64, 32, 4), (96, 24, 3)):
        _same(_gpu(rp, seg, kb, vec), oracle_cpu.preprocess(rp, seg, kb, vec))


def test_reference_signature_entry_point(oracle_cpu):
    """RoDe_preprocess(N_SEG, blockX, vecLen, M, device pointers...) as the reference declares
    it, with buffers sized the way the reference's callers size them
    (Preprocess_opt/_preprocess.cu:426-432: nnz / N_SEG + M entries, M for the residue list)
    plus guard words: like the reference's device version it writes the n_blk segments and the
    n_res rows and nothing else -- in particular no end sentinel st_off[n_blk]."""
    lib = capi.load()
    fn = getattr(lib, capi.CPP_SYMBOLS["RoDe_preprocess"])
    fn.restype = None
    vp = ctypes.c_void_p
    guard = 8
    # second case: fewer nonzeros than one segment and every row at least 32 long, so n_blk
    # equals the reference-sized capacity nnz / N_SEG + M and a sentinel would land one past it
    full_rows = W.CSR(7, 4096, torch.arange(0, 8 * 64, 64, dtype=torch.int32), None, None)
    for A in (W.pareto_rows(m=50000, n=50000, cap=20000, device="cuda"), full_rows):
        rp = A.row_ptr.cuda()
        nnz = int(rp[-1])
        cap = nnz // 512 + A.m
        blk = torch.full((cap + guard,), -1, dtype=torch.int32, device="cuda")
        st = torch.full((cap + guard,), -1, dtype=torch.int32, device="cuda")
        res = torch.full((A.m + guard,), -1, dtype=torch.int32, device="cuda")
        cnt = torch.zeros(2, dtype=torch.int32, device="cuda")
        torch.cuda.synchronize()
        fn(512, 32, 4, A.m, vp(rp.data_ptr()), vp(blk.data_ptr()), vp(st.data_ptr()), vp(res.data_ptr()),
           vp(cnt.data_ptr()), vp(cnt.data_ptr() + 4))
        torch.cuda.synchronize()
        m1, m2 = cnt.cpu().tolist()
        want = oracle_cpu.preprocess(rp.cpu().numpy(), 512, 32, 4)
        assert (m1, m2) == (want[3], want[4]) and m1 <= cap
        if A is full_rows:
            assert m1 == cap
        assert np.array_equal(blk[:m1].cpu().numpy(), want[0])
        assert np.array_equal(st[:m1].cpu().numpy(), want[1][:m1])
        assert np.array_equal(res[:m2].cpu().numpy(), want[2])
        # nothing is written past the counts
        assert bool((blk[m1:] == -1).all()) and bool((st[m1:] == -1).all()) and bool((res[m2:] == -1).all())
