"""The CPU oracle against the reference: golden fixtures (always) and the reference's own
compiled code (where oracle/_ref was built).  No GPU."""
import numpy as np
import pytest

from oracle import ref

PARAMS = ((512, 32, 4), (32, 32, 4))


def _golden(golden_dir, name):
    import os

    return np.load(os.path.join(golden_dir, name))


def test_preprocess_oracle_matches_reference_fixtures(oracle_cpu, golden_dir):
    g = _golden(golden_dir, "preprocess_golden.npz")
    cases = sorted({k.split("/")[0] for k in g.files})
    assert len(cases) >= 8
    for case in cases:
        rp = g[f"{case}/row_ptr"]
        for seg, kb, vec in PARAMS:
            tag = f"{case}/{seg}_{kb}_{vec}"
            blk, st, res, nb, nr = oracle_cpu.preprocess(rp, seg, kb, vec)
            assert [nb, nr] == g[f"{tag}/counts"].tolist(), tag
            assert np.array_equal(blk, g[f"{tag}/block_r_ind"]), tag
            assert np.array_equal(st, g[f"{tag}/st_off"]), tag
            assert np.array_equal(res, g[f"{tag}/residue_r_ind"]), tag
            assert oracle_cpu.preprocess_count(rp, seg, kb, vec) == (nb, nr)


def test_sddmm_oracle_matches_reference_fixtures(oracle_cpu, golden_dir):
    g = _golden(golden_dir, "sddmm_golden.npz")
    cases = sorted({k.split("/")[0] for k in g.files})
    assert len(cases) == 4
    for case in cases:
        a = {k: g[f"{case}/{k}"] for k in ("row_ptr", "col", "val", "lhs", "rhs", "out")}
        for threads in (1, 3):
            got = oracle_cpu.sddmm_f32(a["row_ptr"], a["col"], a["val"], a["lhs"], a["rhs"], threads=threads)
            # same arithmetic in the same order: bit-exact
            assert np.array_equal(got, a["out"]), case


@pytest.mark.skipif(not ref.available(), reason="oracle/_ref not built (no reference checkout)")
def test_oracle_matches_reference_code_on_random_inputs(oracle_cpu):
    rng = np.random.default_rng(7)
    for trial in range(40):
        m = int(rng.integers(1, 400))
        lens = np.minimum((rng.pareto(1.1, m) * rng.integers(1, 40)).astype(np.int64), 5000)
        rp = np.concatenate([[0], np.cumsum(lens)]).astype(np.int32)
        for seg, kb, vec in PARAMS:
            o = oracle_cpu.preprocess(rp, seg, kb, vec)
            r = ref.preprocess(rp, seg, kb, vec)
            assert (o[3], o[4]) == (r[3], r[4])
            for x, y in zip(o[:3], r[:3]):
                assert np.array_equal(x, y)
    for k in (32, 128):
        m, n = 70, 90
        lens = rng.integers(0, 40, m)
        rp = np.concatenate([[0], np.cumsum(lens)]).astype(np.int32)
        col = np.concatenate([np.sort(rng.choice(n, l, replace=False)) for l in lens]).astype(np.int32)
        val = rng.uniform(-1, 1, len(col)).astype(np.float32)
        lhs = rng.uniform(-1, 1, (m, k)).astype(np.float32)
        rhs = rng.uniform(-1, 1, (n, k)).astype(np.float32)
        assert np.array_equal(oracle_cpu.sddmm_f32(rp, col, val, lhs, rhs), ref.sddmm_cpu(rp, col, val, lhs, rhs, n))


def test_preprocess_oracle_exhaustive_small_rows(oracle_cpu):
    """Every row length 0..130 at every start alignment, against the definition written out
    independently in Python (pure-Python loop, small case)."""
    def spec(rp, seg, kb, vec):
        blk, st, res = [], [], []
        for i in range(len(rp) - 1):
            off = int(rp[i]); pad = off % vec; a = int(rp[i + 1]) - off + pad
            first = True
            while a > seg:
                blk.append(i); st.append(off)
                off = off + seg - pad if first else off + seg
                first = False
                a -= seg
            if a > 0:
                if a >= kb:
                    blk.append(i); st.append(off)
                if a % kb:
                    res.append(i)
        st.append(int(rp[-1]))
        return blk, st, res

    for align in range(4):
        lens = np.concatenate([[align], np.repeat(np.arange(0, 131), 1)])
        # interleave single-element rows so that consecutive rows shift the alignment
        lens = np.stack([lens, np.full_like(lens, 1)], 1).reshape(-1)
        rp = np.concatenate([[0], np.cumsum(lens)]).astype(np.int32)
        for seg, kb, vec in ((32, 32, 4), (64, 32, 4), (512, 32, 4)):
            blk, st, res, nb, nr = oracle_cpu.preprocess(rp, seg, kb, vec)
            eb, es, er = spec(rp, seg, kb, vec)
            assert blk.tolist() == eb and st.tolist() == es and res.tolist() == er


def test_spmm_oracle_against_dense_numpy(oracle_cpu):
    """The SpMM oracle is an ordinary CSR product: compare with a dense matmul in fp64."""
    rng = np.random.default_rng(3)
    m, kk, n = 60, 50, 32
    dense = rng.uniform(-1, 1, (m, kk)) * (rng.uniform(0, 1, (m, kk)) < 0.2)
    dense[5] = 0  # an empty row
    rp = np.concatenate([[0], np.cumsum((dense != 0).sum(1))]).astype(np.int32)
    col = np.concatenate([np.nonzero(r)[0] for r in dense]).astype(np.int32)
    val = dense[dense != 0].astype(np.float32)
    B = rng.uniform(-1, 1, (kk, n)).astype(np.float32)
    truth = dense.astype(np.float32).astype(np.float64) @ B.astype(np.float64)
    assert np.allclose(oracle_cpu.spmm_f64acc(rp, col, val, B), truth, rtol=1e-12, atol=1e-12)
    assert np.allclose(oracle_cpu.spmm_f32(rp, col, val, B, threads=2), truth, rtol=1e-5, atol=1e-5)
    assert np.allclose(oracle_cpu.spmm_f64(rp, col, val, B), truth, rtol=1e-12, atol=1e-12)
    assert np.array_equal(oracle_cpu.spmm_f32(rp, col, val, B)[5], np.zeros(n, np.float32))


def test_spmm_oracle_matches_reference_kernel_fixtures(oracle_cpu, golden_dir):
    """spmm_golden.npz holds results of the reference's own GPU SpMM kernels (generated by
    tests/golden/make_golden_gpu.py); the fp32 oracle and the fp64 ground truth agree with
    them within the tolerance of the parity tests."""
    import os

    from tests.helpers import assert_close_to_truth, spmm_abs_scale

    path = os.path.join(golden_dir, "spmm_golden.npz")
    if not os.path.exists(path):
        pytest.skip("spmm_golden.npz not generated yet (needs a GPU run of make_golden_gpu.py)")
    g = np.load(path)
    cases = sorted({k.split("/")[0] for k in g.files})
    assert len(cases) >= 3
    for case in cases:
        a = {k: g[f"{case}/{k}"] for k in ("row_ptr", "col", "val", "B", "C")}
        truth = oracle_cpu.spmm_f64acc(a["row_ptr"], a["col"], a["val"], a["B"])
        scale = spmm_abs_scale(a["row_ptr"], a["col"], a["val"], a["B"])
        assert_close_to_truth(a["C"], truth, scale, f"reference kernels, {case}")
        assert_close_to_truth(oracle_cpu.spmm_f32(a["row_ptr"], a["col"], a["val"], a["B"]), a["C"].astype(np.float64),
                              2 * scale, f"oracle vs reference kernels, {case}")
