"""Synthetic matrix families and the nnz-balanced row partition (host logic, no GPU)."""
import numpy as np
import torch

from rode_b200 import workloads as W


def _check_csr(A):
    rp = A.row_ptr.numpy().astype(np.int64)
    col = A.col.numpy().astype(np.int64)
    assert rp[0] == 0 and rp[-1] == len(col) == A.val.numel() and np.all(np.diff(rp) >= 0)
    assert A.row_ptr.dtype == torch.int32 and A.col.dtype == torch.int32 and A.val.dtype == torch.float32
    assert col.min(initial=0) >= 0 and col.max(initial=0) < A.n
    starts = np.zeros(len(col) + 1, bool)
    starts[rp] = True
    if len(col) > 1:
        assert np.all((np.diff(col) > 0) | starts[1:-1]), "columns must ascend strictly inside a row"


def test_families_are_valid_seeded_csr():
    fams = {
        "bernoulli": lambda s: W.bernoulli(512, 512, 0.02, seed=s),
        "zipf": lambda s: W.zipf_rows(m=2048, n=2048, cap=1024, seed=s),
        "stencil": lambda s: W.stencil27(9, seed=s),
        "pareto": lambda s: W.pareto_rows(m=2048, n=4096, cap=1500, seed=s),
        "rmat": lambda s: W.rmat(scale=11, edge_factor=8, seed=s, chunk=1 << 12),
    }
    for name, make in fams.items():
        a, b, c = make(5), make(5), make(6)
        _check_csr(a)
        assert torch.equal(a.row_ptr, b.row_ptr) and torch.equal(a.col, b.col) and torch.equal(a.val, b.val), name
        if name != "stencil":
            assert not (a.nnz == c.nnz and torch.equal(a.col, c.col)), name


def test_family_shapes():
    s = W.stencil27(8)
    assert s.nnz == (3 * 8 - 2) ** 3 and int(np.diff(s.row_ptr.numpy()).max()) == 27
    assert float(s.val.min()) >= 0.5 and float(s.val.max()) < 1.5
    z = W.zipf_rows(m=8192, n=8192, cap=2048)
    lens = np.diff(z.row_ptr.numpy())
    assert abs(lens.mean() - 16) < 0.5 and lens.max() > 200 and lens.min() >= 1
    p = W.pareto_rows(m=8192, n=8192, cap=3000)
    lens = np.diff(p.row_ptr.numpy())
    assert abs(lens.mean() - 32) < 1 and lens.max() <= 3000
    b = W.bernoulli(1024, 1024, 0.01)
    assert abs(b.nnz / 1024**2 - 0.01) < 0.002 and float(b.val.min()) == 1.0
    r = W.rmat(scale=12, edge_factor=16)
    assert r.m == 4096 and 0.5 * 16 * 4096 < r.nnz <= 16 * 4096


def test_partition_is_nnz_balanced_and_covers_all_rows():
    A = W.rmat(scale=13, edge_factor=16)
    for parts in (1, 2, 3, 4, 8):
        b = W.partition_rows(A.row_ptr, parts)
        assert b[0] == 0 and b[-1] == A.m and len(b) == parts + 1 and b == sorted(b)
        rp = A.row_ptr.numpy().astype(np.int64)
        per = np.diff(rp[b])
        longest = int(np.diff(rp).max())
        assert per.sum() == A.nnz and per.max() - A.nnz / parts <= longest + 1
        sub = A.rows(b[0], b[1])
        assert sub.m == b[1] and int(sub.row_ptr[-1]) == sub.nnz and sub.row_ptr[0] == 0
    # degenerate: more parts than rows with entries
    tiny = W.CSR(3, 4, torch.tensor([0, 0, 5, 5], dtype=torch.int32), torch.arange(5, dtype=torch.int32) % 4,
                 torch.ones(5))
    assert W.partition_rows(tiny.row_ptr, 4)[-1] == 3


def test_row_weighted_partition_trades_nnz_for_rows():
    A = W.rmat(scale=14, edge_factor=16)
    rp = A.row_ptr.numpy().astype(np.int64)
    plain = W.partition_rows(A.row_ptr, 8, 0.0)
    weighted = W.partition_rows(A.row_ptr, 8, 2.0)
    assert plain[0] == weighted[0] == 0 and plain[-1] == weighted[-1] == A.m and weighted == sorted(weighted)

    def cost(b, w):
        return [(rp[b[i + 1]] - rp[b[i]]) + w * (b[i + 1] - b[i]) for i in range(8)]

    # the weighted cut equalises nnz + 2 * rows; the plain cut equalises nnz and leaves the last
    # ranks with far more rows (R-MAT rows thin out towards high indices)
    cw = cost(weighted, 2.0)
    assert max(cw) / (sum(cw) / 8) < 1.05
    assert max(cost(plain, 2.0)) > max(cw)
    assert (plain[-1] - plain[-2]) > (weighted[-1] - weighted[-2])
