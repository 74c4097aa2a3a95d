"""Preprocessing benchmark on a matrix file, after the reference's Preprocess_opt main
(Preprocess_opt/_preprocess.cu:383-512): times the row-swizzle comparator and the RoDe row
decomposition on the GPU (CUDA events) and on the host (the library's host twin), and - which
the reference's main does not do - checks that the GPU and host results are identical.

    python -m rode_b200.preprocess_bench matrix.mtx [--iters 20] [--seg 512]

Prints one CSV line: name,rows,nnz,swizzle_gpu_ms,rode_gpu_ms,swizzle_cpu_ms,rode_cpu_ms,m1,m2
"""
from __future__ import annotations

import argparse
import os
import time

import torch

from . import capi, matrix_io


def main(argv=None) -> int:
    p = argparse.ArgumentParser()
    p.add_argument("path")
    p.add_argument("--iters", type=int, default=20)
    p.add_argument("--seg", type=int, default=512)
    args = p.parse_args(argv)
    if not torch.cuda.is_available():
        raise SystemExit("needs a CUDA device; rode_b200 has no CPU path")
    A = matrix_io.load_matrix_market(args.path, "cuda")
    rp = A.row_ptr

    def gpu_ms(fn):
        fn()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(args.iters):
            fn()
        b.record()
        torch.cuda.synchronize()
        return a.elapsed_time(b) / args.iters

    # device buffers once, as the reference's main does; raw entry point inside the loop
    cap = capi.preprocess_capacity(args.seg, 4, A.m, A.nnz)
    blk = torch.empty(max(cap, 1), dtype=torch.int32, device="cuda")
    st = torch.empty(cap + 1, dtype=torch.int32, device="cuda")
    res = torch.empty(max(A.m, 1), dtype=torch.int32, device="cuda")
    cnt = torch.zeros(2, dtype=torch.int32, device="cuda")
    ws_bytes = capi.preprocess_workspace_bytes(A.m)
    ws = torch.empty(ws_bytes, dtype=torch.uint8, device="cuda")
    rode_gpu = gpu_ms(lambda: capi.preprocess_raw(args.seg, 32, 4, A.m, rp.data_ptr(), blk.data_ptr(), st.data_ptr(),
                                                  res.data_ptr(), cnt.data_ptr(), cnt.data_ptr() + 4, ws.data_ptr(),
                                                  ws_bytes, torch.cuda.current_stream()))
    swz_gpu = gpu_ms(lambda: matrix_io.row_swizzle(rp))
    m1, m2 = cnt.cpu().tolist()

    rp_host = rp.cpu()
    t0 = time.perf_counter()
    host = capi.preprocess_cpu(rp_host, args.seg, 32, 4)
    rode_cpu = (time.perf_counter() - t0) * 1e3
    t0 = time.perf_counter()
    matrix_io.row_swizzle(rp_host)
    swz_cpu = (time.perf_counter() - t0) * 1e3

    same = (host[3], host[4]) == (m1, m2) and torch.equal(host[0], blk[:m1].cpu()) and torch.equal(
        host[1], st[: m1 + 1].cpu()) and torch.equal(host[2], res[:m2].cpu())
    if not same:
        raise SystemExit("GPU and host row decompositions differ")
    name = os.path.splitext(os.path.basename(args.path))[0]
    print(f"{name},{A.m},{A.nnz},{swz_gpu:.6f},{rode_gpu:.6f},{swz_cpu:.6f},{rode_cpu:.6f},{m1},{m2}")
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
