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


def _outputs(A, seg, vec):
    cap = capi.preprocess_capacity(seg, vec, A.m, A.nnz)
    return (torch.full((max(cap, 1),), -7, dtype=torch.int32, device="cuda"),
            torch.full((cap + 1,), -7, dtype=torch.int32, device="cuda"),
            torch.full((max(A.m, 1),), -7, dtype=torch.int32, device="cuda"),
            torch.zeros(2, dtype=torch.int32, device="cuda"))


def _run(entry, A, seg, kb, vec, stream=None):
    """Calls one of the two entry points on raw device addresses; returns host copies."""
    blk, st, res, cnt = _outputs(A, seg, vec)
    if stream is None:
        stream = torch.cuda.current_stream()
    else:
        stream.wait_stream(torch.cuda.current_stream())   # the fills above ran on the current stream
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
    # the same on a stream of the caller's own
    side = torch.cuda.Stream()
    got = _run("noalloc", small, 512, 32, 4, stream=side)
    want = _run("workspace", small, 512, 32, 4)
    assert got[3] == want[3] and all(np.array_equal(g, w) for g, w in zip(got[:3], want[:3]))


@pytest.mark.gpu
def test_noalloc_leaves_the_device_memory_as_it_found_it():
    """The point of the entry point: a call obtains no device memory.  With the outputs
    allocated beforehand, the free memory the driver reports is the same before and after a
    call (the first call on the device has already looked up the built-in scratch's address)."""
    A = W.pareto_rows(m=300000, n=300000, cap=40000, device="cuda", seed=71)
    blk, st, res, cnt = _outputs(A, 512, 4)
    stream = torch.cuda.current_stream()

    def call():
        capi.preprocess_noalloc_raw(512, 32, 4, A.m, A.row_ptr.data_ptr(), blk.data_ptr(), st.data_ptr(),
                                    res.data_ptr(), cnt.data_ptr(), cnt.data_ptr() + 4, stream)
        torch.cuda.synchronize()

    call()                                                # set-up call of this device, if none came before
    free_before, _ = torch.cuda.mem_get_info()
    reserved_before = torch.cuda.memory_reserved()
    for _ in range(3):
        call()
    free_after, _ = torch.cuda.mem_get_info()
    assert free_after == free_before                      # nothing obtained from the driver
    assert torch.cuda.memory_reserved() == reserved_before  # nor from torch's allocator
    assert cnt.cpu().tolist()[0] > 0


def test_noalloc_rejects_sizes_beyond_its_scratch(built_library):
    lib = capi.load()
    too_many = (1 << 24) + 1
    rc = lib.rode_preprocess_noalloc(512, 32, 4, too_many, 16, 16, 16, 16, 16, 16, None)
    assert rc == capi.RODE_ERR_INVALID_ARGUMENT
    msg = lib.rode_last_error().decode()
    assert "16777216" in msg and "rode_preprocess" in msg
