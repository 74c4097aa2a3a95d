"""Generates spmm_golden.npz by running the REFERENCE's own SpMM kernels on a GPU.

The reference has no CPU SpMM, so the SpMM fixtures come from its GPU entry points
(RoDe_SpMM/RoDeSpmm.h:4-14) compiled into oracle/_ref, fed with metadata from the
reference's host RoDe_preprocess (RoDe_SDDMM/main.cu:114-163).  Run once on a machine with a
GPU and oracle/_ref built:

    python tests/golden/make_golden_gpu.py [output_dir]

Each case stores the inputs and the reference's C (fp32; its atomicAdd order is not
deterministic, so consumers compare within the tolerance, not bit for bit).
"""
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))

from oracle import ref  # noqa: E402


def main():
    assert ref.available() and torch.cuda.is_available()
    out_dir = sys.argv[1] if len(sys.argv) > 1 else HERE
    rng = np.random.default_rng(20240611)
    out = {}
    cases = {"n32_mixed": (160, 400, 32, [0, 1, 5, 31, 32, 33, 64, 100, 511, 512, 513, 700, 1100]),
             "n128_mixed": (96, 300, 128, [0, 3, 17, 31, 32, 40, 95, 600, 1030]),
             "n128_short": (300, 64, 128, [0, 1, 2, 3, 7, 12, 36])}
    for name, (m, k, n, palette) in cases.items():
        lens = np.minimum(rng.choice(palette, m), k)
        lens[0] = min(max(palette), k)
        rp = np.concatenate([[0], np.cumsum(lens)]).astype(np.int32)
        col = np.concatenate([np.sort(rng.choice(k, l, replace=False)) for l in lens]).astype(np.int32)
        val = rng.uniform(-1, 1, len(col)).astype(np.float32)
        B = rng.uniform(-1, 1, (k, n)).astype(np.float32)
        blk, st, res, m1, m2 = ref.preprocess(rp, 512, 32, 4)
        assert m1 > 0 and m2 > 0
        d = {k_: torch.from_numpy(v).cuda() for k_, v in dict(rp=rp, col=col, val=val, B=B, blk=blk, st=st, res=res).items()}
        C = torch.zeros((m, n), device="cuda")
        s1, s2 = torch.cuda.Stream(), torch.cuda.Stream()
        torch.cuda.synchronize()
        ref.spmm_gpu(32 if n == 32 else 128, False, m1, m2, k, n, d["val"].data_ptr(), d["col"].data_ptr(),
                     d["rp"].data_ptr(), d["blk"].data_ptr(), d["res"].data_ptr(), d["st"].data_ptr(), d["B"].data_ptr(),
                     C.data_ptr(), s1.cuda_stream, s2.cuda_stream)
        torch.cuda.synchronize()
        for key, arr in dict(row_ptr=rp, col=col, val=val, B=B, C=C.cpu().numpy()).items():
            out[f"{name}/{key}"] = arr
    np.savez_compressed(os.path.join(out_dir, "spmm_golden.npz"), **out)
    print("wrote", os.path.join(out_dir, "spmm_golden.npz"))


if __name__ == "__main__":
    main()
