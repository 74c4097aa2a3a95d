"""Matrix Market ingest and COO -> CSR conversion (CPU), plus the file-driven preprocessing
benchmark on a GPU."""
import numpy as np
import pytest
import torch

from rode_b200 import matrix_io
from rode_b200 import workloads as W


def test_round_trip_and_sorted_csr(tmp_path):
    A = W.pareto_rows(m=300, n=500, cap=200, seed=4)
    path = tmp_path / "a.mtx"
    matrix_io.write_matrix_market(str(path), A)
    B = matrix_io.load_matrix_market(str(path))
    assert (B.m, B.n, B.nnz) == (A.m, A.n, A.nnz)
    assert torch.equal(B.row_ptr, A.row_ptr) and torch.equal(B.col, A.col)
    assert torch.allclose(B.val, A.val, rtol=0, atol=0)


def test_symmetric_pattern_duplicates_and_comments(tmp_path):
    path = tmp_path / "s.mtx"
    path.write_text("%%MatrixMarket matrix coordinate pattern symmetric\n% a comment\n\n4 4 4\n1 1\n3 1\n4 2\n4 4\n")
    S = matrix_io.load_matrix_market(str(path))
    dense = torch.zeros(4, 4)
    for i in range(4):
        for e in range(int(S.row_ptr[i]), int(S.row_ptr[i + 1])):
            dense[i, int(S.col[e])] = S.val[e]
    want = torch.tensor([[1., 0, 1, 0], [0, 0, 0, 1], [1, 0, 0, 0], [0, 1, 0, 1]])
    assert torch.equal(dense, want)
    path.write_text("%%MatrixMarket matrix coordinate real general\n2 3 4\n2 3 1.5\n1 1 2\n2 3 0.25\n1 2 -1\n")
    D = matrix_io.load_matrix_market(str(path))
    assert D.row_ptr.tolist() == [0, 2, 3] and D.col.tolist() == [0, 1, 2] and D.val.tolist() == [2.0, -1.0, 1.75]
    path.write_text("%%MatrixMarket matrix coordinate real skew-symmetric\n2 2 1\n2 1 3\n")
    K = matrix_io.load_matrix_market(str(path))
    assert K.col.tolist() == [1, 0] and K.val.tolist() == [-3.0, 3.0]
    path.write_text("%%MatrixMarket matrix array real general\n2 2\n1\n2\n3\n4\n")
    with pytest.raises(ValueError):
        matrix_io.load_matrix_market(str(path))


def test_row_swizzle_orders_rows_by_length():
    rp = torch.tensor([0, 3, 3, 10, 12, 12, 20], dtype=torch.int32)
    assert matrix_io.row_swizzle(rp).tolist() == [5, 2, 0, 3, 1, 4]


@pytest.mark.gpu
def test_file_to_gpu_pipeline_and_benchmark(tmp_path, capsys, oracle_cpu):
    from rode_b200 import capi, preprocess_bench

    A = W.zipf_rows(m=3000, n=3000, cap=3000, seed=8)
    path = tmp_path / "z.mtx"
    matrix_io.write_matrix_market(str(path), A)
    G = matrix_io.load_matrix_market(str(path), "cuda")           # conversion on the device
    assert G.row_ptr.is_cuda and torch.equal(G.row_ptr.cpu(), A.row_ptr) and torch.equal(G.col.cpu(), A.col)
    meta = capi.preprocess(G.row_ptr, G.nnz)
    B = W.dense(A.n, 32, seed=2)
    C = capi.spmm(meta, G.row_ptr, G.col, G.val, B.cuda())
    truth = oracle_cpu.spmm_f64acc(A.row_ptr.numpy(), A.col.numpy(), A.val.numpy(), B.numpy())
    assert np.allclose(C.cpu().numpy(), truth, rtol=1e-5, atol=1e-4)
    assert preprocess_bench.main([str(path), "--iters", "3"]) == 0
    line = capsys.readouterr().out.strip().splitlines()[-1].split(",")
    assert line[0] == "z" and int(line[1]) == 3000 and int(line[2]) == A.nnz and len(line) == 9


@pytest.mark.gpu
def test_row_swizzle_on_the_device_matches_a_stable_host_sort():
    """The Sputnik-style comparator (Preprocess_opt/_preprocess.cu:71-104) on a device row
    pointer: rows by decreasing length, ties in row order."""
    A = W.pareto_rows(m=200000, n=200000, cap=30000, device="cuda", seed=17)
    order = matrix_io.row_swizzle(A.row_ptr)
    assert order.is_cuda and order.dtype == torch.int32
    lens = np.diff(A.row_ptr.cpu().numpy().astype(np.int64))
    want = np.argsort(-lens, kind="stable")
    assert np.array_equal(order.cpu().numpy(), want.astype(np.int32))
