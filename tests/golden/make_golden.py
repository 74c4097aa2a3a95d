"""Generates the fixtures in this directory by running the REFERENCE's own code.

Run once in a checkout that has the reference sources (they are compiled by
``make -C oracle ref`` into ``oracle/_ref``):

    python tests/golden/make_golden.py

* preprocess_golden.npz  inputs (CSR row pointers) and the outputs of the reference's host
                         function RoDe_preprocess (RoDe_SDDMM/main.cu:114-163) for the two
                         parameter sets it uses, (512, 32, 4) and (32, 32, 4).
* sddmm_golden.npz       small seeded SDDMM problems and the outputs of the reference's
                         sddmm_cpu_reference (RoDe_SDDMM/main.cu:65-91), K = 32 and 128.

SpMM fixtures cannot be produced here (the reference has no CPU SpMM); they are produced
on a GPU by make_golden_gpu.py from the reference's SpMM kernels.
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))

from oracle import ref  # noqa: E402


def row_ptr_cases(rng):
    cases = {}
    # every aligned length 0..1100 at every start alignment: lengths shuffled so that the
    # running offset visits all residues mod 4
    lens = np.concatenate([np.arange(0, 1101), np.arange(0, 140), np.arange(500, 560), np.arange(1020, 1060)])
    rng.shuffle(lens)
    cases["sweep"] = np.concatenate([[0], np.cumsum(lens)]).astype(np.int32)
    cases["empty_matrix"] = np.zeros(1, np.int32)                      # M = 0
    cases["all_empty_rows"] = np.zeros(50, np.int32)                   # 49 empty rows
    cases["single_long"] = np.array([0, 20000], np.int32)
    cases["unaligned_long"] = np.array([0, 3, 3 + 16384, 3 + 16384 + 1], np.int32)
    cases["short_only"] = np.concatenate([[0], np.cumsum(rng.integers(0, 31, 3000))]).astype(np.int32)
    heavy = np.minimum((rng.pareto(1.2, 5000) * 6).astype(np.int64), 9000)
    cases["heavy_tail"] = np.concatenate([[0], np.cumsum(heavy)]).astype(np.int32)
    cases["exact_multiples"] = np.concatenate([[0], np.cumsum([32, 64, 512, 1024, 480, 544, 31, 33, 0, 512])]).astype(
        np.int32)
    return cases


def main():
    assert ref.available(), "build oracle/_ref first: make -C oracle ref"
    rng = np.random.default_rng(20240607)
    out = {}
    for name, rp in row_ptr_cases(rng).items():
        out[f"{name}/row_ptr"] = rp
        for seg, kb, vec in ((512, 32, 4), (32, 32, 4)):
            blk, st, res, nb, nr = ref.preprocess(rp, seg, kb, vec)
            tag = f"{name}/{seg}_{kb}_{vec}"
            out[f"{tag}/block_r_ind"] = blk
            out[f"{tag}/st_off"] = st
            out[f"{tag}/residue_r_ind"] = res
            out[f"{tag}/counts"] = np.array([nb, nr], np.int32)
    np.savez_compressed(os.path.join(HERE, "preprocess_golden.npz"), **out)

    out = {}
    for name, (m, n, k, mean_len) in {"k32_small": (96, 150, 32, 9), "k128_small": (64, 80, 128, 20),
                                      "k32_long": (8, 1200, 32, 560), "k128_ragged": (200, 64, 128, 3)}.items():
        lens = np.minimum(rng.poisson(mean_len, m), n)
        lens[rng.integers(0, m, max(1, m // 10))] = 0          # some empty rows
        rp = np.concatenate([[0], np.cumsum(lens)]).astype(np.int32)
        col = np.concatenate([np.sort(rng.choice(n, l, replace=False)) for l in lens] + [np.zeros(0, np.int64)])
        col = col.astype(np.int32)
        val = rng.uniform(-1, 1, len(col)).astype(np.float32)
        lhs = rng.uniform(-1, 1, (m, k)).astype(np.float32)
        rhs = rng.uniform(-1, 1, (n, k)).astype(np.float32)
        got = ref.sddmm_cpu(rp, col, val, lhs, rhs, n)
        for key, arr in dict(row_ptr=rp, col=col, val=val, lhs=lhs, rhs=rhs, out=got).items():
            out[f"{name}/{key}"] = arr
    np.savez_compressed(os.path.join(HERE, "sddmm_golden.npz"), **out)
    print("wrote fixtures to", HERE)


if __name__ == "__main__":
    main()
