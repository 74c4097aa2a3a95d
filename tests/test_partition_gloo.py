"""The N > 1 path on CPU: two gloo ranks partition the rows nnz-balanced, each handles its
slice independently (host preprocessing twin + oracle product stand in for the GPU work),
and the gathered result equals the single-rank result.  Exercises what the multi-GPU bench
does around the kernels: partition, slice re-basing, one broadcast, no data-path collective."""
import os
import socket

import numpy as np
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from rode_b200 import workloads as W


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _rank_main(rank, world, port, out_dir):
    import sys

    sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    from oracle import cpu
    from rode_b200 import capi

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        n_vert = 1 << 11
        if rank == 0:
            A = W.rmat(scale=11, edge_factor=12, seed=9, chunk=1 << 13)
            sizes = torch.tensor([A.nnz])
        else:
            A, sizes = None, torch.zeros(1, dtype=torch.int64)
        dist.broadcast(sizes, 0)
        nnz = int(sizes[0])
        row_ptr = A.row_ptr if rank == 0 else torch.empty(n_vert + 1, dtype=torch.int32)
        col = A.col if rank == 0 else torch.empty(nnz, dtype=torch.int32)
        val = A.val if rank == 0 else torch.empty(nnz, dtype=torch.float32)
        X = W.dense(n_vert, 32, seed=3) if rank == 0 else torch.empty((n_vert, 32))
        for t in (row_ptr, col, val, X):     # the one set-up broadcast
            dist.broadcast(t, 0)
        full = W.CSR(n_vert, n_vert, row_ptr, col, val)
        bounds = W.partition_rows(row_ptr, world)
        mine = full.rows(bounds[rank], bounds[rank + 1])
        # per-rank preprocessing of the re-based slice agrees with the oracle
        blk, st, res, m1, m2 = capi.preprocess_cpu(mine.row_ptr, 512, 32, 4)
        want = cpu.preprocess(mine.row_ptr.numpy(), 512, 32, 4)
        assert (m1, m2) == (want[3], want[4]) and np.array_equal(st.numpy(), want[1])
        C = cpu.spmm_f32(mine.row_ptr.numpy(), mine.col.numpy(), mine.val.numpy(), X.numpy())
        np.save(os.path.join(out_dir, f"C{rank}.npy"), C)
        np.save(os.path.join(out_dir, f"nnz{rank}.npy"), np.array([mine.nnz, nnz, bounds[rank], bounds[rank + 1]]))
        if rank == 0:
            np.save(os.path.join(out_dir, "C_full.npy"), cpu.spmm_f32(row_ptr.numpy(), col.numpy(), val.numpy(), X.numpy()))
        dist.barrier()
    finally:
        dist.destroy_process_group()


def test_two_ranks_reproduce_the_single_rank_result(tmp_path, built_library, oracle_cpu):
    world = 2
    mp.spawn(_rank_main, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    parts = [np.load(tmp_path / f"C{r}.npy") for r in range(world)]
    meta = [np.load(tmp_path / f"nnz{r}.npy") for r in range(world)]
    full = np.load(tmp_path / "C_full.npy")
    assert np.array_equal(np.concatenate(parts, 0), full)           # same arithmetic per row: bit-exact
    assert sum(int(m[0]) for m in meta) == int(meta[0][1])          # slices cover every nonzero once
    assert meta[0][3] == meta[1][2] and meta[0][2] == 0 and meta[1][3] == full.shape[0]
    share = [int(m[0]) / int(m[1]) for m in meta]
    assert abs(share[0] - 0.5) < 0.05, share                         # nnz-balanced
