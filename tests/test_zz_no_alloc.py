"""rode_preprocess_noalloc: the preprocessing entry point for callers that cannot allocate
device memory at call time (a process whose GPU memory is owned by its own pool, or a loop
that cannot afford the device-wide synchronisation of cudaMalloc / cudaFree).  Its scratch is
a fixed array inside the library, so every call shares it; the test therefore makes two calls
in a row (a larger matrix first, a smaller one second, so stale scratch would show) and
compares each with the workspace-taking entry point, bit for bit, through the C ABI.
This file is collected last on purpose."""
import numpy as np
import pytest
import torch

from rode_b200 import capi
from rode_b200 import workloads as W


def _run(entry, A, seg, kb, vec):
    """Calls one of the two entry points on raw device addresses; returns host copies."""
    cap = capi.preprocess_capacity(seg, vec, A.m, A.nnz)
    blk = torch.full((max(cap, 1),), -7, dtype=torch.int32, device="cuda")
    st = torch.full((cap + 1,), -7, dtype=torch.int32, device="cuda")
    res = torch.full((max(A.m, 1),), -7, dtype=torch.int32, device="cuda")
    cnt = torch.zeros(2, dtype=torch.int32, device="cuda")
    stream = torch.cuda.current_stream()
    if entry == "noalloc":
        capi.preprocess_noalloc_raw(seg, kb, vec, A.m, A.row_ptr.data_ptr(), blk.data_ptr(), st.data_ptr(),
                                    res.data_ptr(), cnt.data_ptr(), cnt.data_ptr() + 4, stream)
    else:
        ws_bytes = capi.preprocess_workspace_bytes(A.m)
        ws = torch.empty(ws_bytes, dtype=torch.uint8, device="cuda")
        capi.preprocess_raw(seg, kb, vec, A.m, A.row_ptr.data_ptr(), blk.data_ptr(), st.data_ptr(), res.data_ptr(),
                            cnt.data_ptr(), cnt.data_ptr() + 4, ws.data_ptr(), ws_bytes, stream)
    torch.cuda.synchronize()
    return blk.cpu().numpy(), st.cpu().numpy(), res.cpu().numpy(), cnt.cpu().tolist()


@pytest.mark.gpu
def test_noalloc_matches_workspace_entry_point_on_two_calls_in_a_row():
    big = W.pareto_rows(m=300000, n=300000, cap=40000, device="cuda", seed=71)      # 293 tiles
    small = W.zipf_rows(m=5000, n=8192, cap=4096, device="cuda", seed=72)           # 5 tiles
    for A, (seg, kb, vec) in ((big, (512, 32, 4)), (small, (32, 32, 4)), (big, (32, 32, 4))):
        got = _run("noalloc", A, seg, kb, vec)
        want = _run("workspace", A, seg, kb, vec)
        assert got[3] == want[3] and got[3][0] > 0 and got[3][1] > 0
        for g, w in zip(got[:3], want[:3]):
            assert np.array_equal(g, w)       # integer outputs: bit-exact, untouched tails included


def test_noalloc_rejects_sizes_beyond_its_scratch(built_library):
    lib = capi.load()
    too_many = (1 << 24) + 1
    rc = lib.rode_preprocess_noalloc(512, 32, 4, too_many, 16, 16, 16, 16, 16, 16, None)
    assert rc == capi.RODE_ERR_INVALID_ARGUMENT
    msg = lib.rode_last_error().decode()
    assert "16777216" in msg and "rode_preprocess" in msg
