"""The C-ABI library loads without a GPU, exports what include/*.h declares, validates its
arguments before touching CUDA, and its host preprocessing twin matches the oracle."""
import ctypes
import os
import re

import numpy as np
import pytest
import torch

from rode_b200 import capi

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_library_exports_every_declared_symbol(built_library):
    lib = ctypes.CDLL(built_library)
    header = open(os.path.join(ROOT, "include", "rode_b200.h")).read()
    header = re.sub(r"/\*.*?\*/", "", header, flags=re.S)
    declared = set(re.findall(r"\b(rode_[a-z0-9_]+)\s*\(", header))
    assert declared == set(capi.C_ABI_SYMBOLS)
    for name in declared:
        assert hasattr(lib, name), name
    # the reference-signature C++ entry points (RoDeSpmm.h, RoDeSddmm.h, RoDePreprocess.h)
    for name, mangled in capi.CPP_SYMBOLS.items():
        assert hasattr(lib, mangled), name


def test_cpp_symbol_names_equal_the_reference_objects():
    """A program linked against the reference's objects resolves against this library:
    the mangled names are the same strings."""
    from oracle import ref

    assert capi.CPP_SYMBOLS["RoDeSpmm_n32_f32"] == ref.SYM_SPMM_N32_F
    assert capi.CPP_SYMBOLS["RoDeSpmm_n128_f32"] == ref.SYM_SPMM_N128_F
    assert capi.CPP_SYMBOLS["RoDeSpmm_n32_f64"] == ref.SYM_SPMM_N32_D
    assert capi.CPP_SYMBOLS["RoDeSpmm_n128_f64"] == ref.SYM_SPMM_N128_D
    assert capi.CPP_SYMBOLS["RoDeSDDMM_n32"] == ref.SYM_SDDMM_N32
    assert capi.CPP_SYMBOLS["RoDeSDDMM_n128"] == ref.SYM_SDDMM_N128


def test_version_and_sizes(built_library):
    assert re.fullmatch(r"\d+\.\d+\.\d+", capi.version())
    assert capi.preprocess_workspace_bytes(0) == 8
    assert capi.preprocess_workspace_bytes(1024) == 16      # the CTA counter + one tile of 2048 rows
    assert capi.preprocess_workspace_bytes(1025) == 16
    # one partial row per block segment, rounded up to 256 bytes, plus 256 bytes of claim counters
    assert capi.spmm_workspace_bytes(10, 128, 4) == 10 * 128 * 4 + 256
    assert capi.spmm_workspace_bytes(3, 32, 4) == 512 + 256
    assert capi.spmm_workspace_bytes(0, 128, 8) == 256
    assert capi.preprocess_capacity(512, 4, 100, 5000) == (5000 + 300) // 512 + 100


def test_argument_errors_are_reported_not_raised_by_cuda(built_library):
    lib = capi.load()
    # bad parameter relations
    assert lib.rode_preprocess(500, 32, 4, 10, 16, 16, 16, 16, 16, 16, 16, 64, None) == capi.RODE_ERR_INVALID_ARGUMENT
    assert b"seg_len" in lib.rode_last_error()
    # null row pointer
    assert lib.rode_preprocess(512, 32, 4, 10, None, 16, 16, 16, 16, 16, 16, 64, None) == capi.RODE_ERR_INVALID_ARGUMENT
    # workspace too small
    assert lib.rode_preprocess(512, 32, 4, 5000, 16, 16, 16, 16, 16, 16, 16, 8, None) == capi.RODE_ERR_WORKSPACE
    # unsupported widths
    assert lib.rode_spmm_f32(1, 1, 8, 22, 16, 16, 16, 16, 16, 16, 16, 16, None, 0, None, None) == capi.RODE_ERR_INVALID_ARGUMENT
    assert lib.rode_sddmm_f32(1, 1, 8, 50, 16, 16, 16, 16, 16, 16, 16, 16, 16, None, None) == capi.RODE_ERR_INVALID_ARGUMENT
    assert lib.rode_sddmm_f32(1, 1, 8, 260, 16, 16, 16, 16, 16, 16, 16, 16, 16, None, None) == capi.RODE_ERR_INVALID_ARGUMENT
    # misaligned dense operands (16-byte alignment is part of the contract)
    assert lib.rode_spmm_f32(1, 1, 8, 32, 16, 16, 16, 16, 16, 16, 24, 16, None, 0, None, None) == capi.RODE_ERR_INVALID_ARGUMENT
    assert b"aligned" in lib.rode_last_error()
    assert lib.rode_sddmm_f32(1, 1, 8, 32, 16, 16, 16, 16, 16, 16, 16, 20, 16, None, None) == capi.RODE_ERR_INVALID_ARGUMENT
    # negative counts
    assert lib.rode_spmm_f32(-1, 0, 8, 32, 16, 16, 16, 16, 16, 16, 16, 16, None, 0, None, None) == capi.RODE_ERR_INVALID_ARGUMENT
    assert lib.rode_preprocess(512, 32, 4, -5, 16, 16, 16, 16, 16, 16, 16, 64, None) == capi.RODE_ERR_INVALID_ARGUMENT
    # missing workspace for split rows
    assert lib.rode_spmm_f32(4, 0, 8, 32, 16, 16, 16, 16, 16, 16, 16, 16, None, 0, None, None) == capi.RODE_ERR_WORKSPACE
    with pytest.raises(capi.RodeError):
        capi.check(capi.RODE_ERR_WORKSPACE)
    # nothing to do is not an error and needs no device
    assert lib.rode_spmm_f32(0, 0, 8, 32, None, None, None, None, None, None, None, None, None, 0, None, None) == 0
    assert lib.rode_sddmm_f32(0, 0, 8, 32, None, None, None, None, None, None, None, None, None, None, None) == 0


def test_hot_columns_sizes_and_argument_errors(built_library):
    """Host arithmetic and argument checks of the popularity-hint entry points (no device)."""
    lib = capi.load()
    words, need = ctypes.c_size_t(0), ctypes.c_size_t(0)
    assert lib.rode_hot_columns_words(0, ctypes.byref(words)) == 0 and words.value == 1
    assert lib.rode_hot_columns_words(32, ctypes.byref(words)) == 0 and words.value == 2
    assert lib.rode_hot_columns_words(33, ctypes.byref(words)) == 0 and words.value == 3
    assert lib.rode_hot_columns_workspace_bytes(1000, ctypes.byref(need)) == 0
    assert need.value >= 4 * 1000 + 2 * 4096 * 4 and need.value % 256 == 0
    assert lib.rode_hot_columns_words(-1, ctypes.byref(words)) == capi.RODE_ERR_INVALID_ARGUMENT
    # row bytes 0, null bitmap, missing / short / misaligned workspace
    assert lib.rode_hot_columns(10, 64, 256, 0, 0, 256, 256, 1 << 20, None) == capi.RODE_ERR_INVALID_ARGUMENT
    assert lib.rode_hot_columns(10, 64, 256, 512, 0, None, 256, 1 << 20, None) == capi.RODE_ERR_INVALID_ARGUMENT
    assert lib.rode_hot_columns(10, 64, 256, 512, 0, 256, None, 0, None) == capi.RODE_ERR_WORKSPACE
    assert lib.rode_hot_columns(10, 64, 256, 512, 0, 256, 256, 16, None) == capi.RODE_ERR_WORKSPACE
    assert lib.rode_hot_columns(10, 64, 256, 512, 1, 256, 264, 1 << 20, None) == capi.RODE_ERR_WORKSPACE
    assert b"aligned" in lib.rode_last_error()
    # the hinted SpMM entry points validate like the plain ones
    assert lib.rode_spmm_f32_hot(1, 1, 8, 22, 16, 16, 16, 16, 16, 16, 16, 16, None, 0, 16, None, None) == capi.RODE_ERR_INVALID_ARGUMENT
    assert lib.rode_spmm_f64_hot(0, 0, 8, 32, None, None, None, None, None, None, None, None, None, 0, None, None, None) == 0


def test_host_preprocess_twin_matches_oracle_and_fixtures(built_library, oracle_cpu, golden_dir):
    g = np.load(os.path.join(golden_dir, "preprocess_golden.npz"))
    for case in sorted({k.split("/")[0] for k in g.files}):
        rp = g[f"{case}/row_ptr"]
        for seg, kb, vec in ((512, 32, 4), (32, 32, 4)):
            blk, st, res, nb, nr = capi.preprocess_cpu(torch.from_numpy(rp.copy()), seg, kb, vec)
            tag = f"{case}/{seg}_{kb}_{vec}"
            assert [nb, nr] == g[f"{tag}/counts"].tolist()
            assert np.array_equal(blk.numpy(), g[f"{tag}/block_r_ind"])
            assert np.array_equal(st.numpy(), g[f"{tag}/st_off"])
            assert np.array_equal(res.numpy(), g[f"{tag}/residue_r_ind"])


def test_missing_library_fails_loudly(monkeypatch, tmp_path):
    monkeypatch.setattr(capi, "_lib", None)
    monkeypatch.setattr(capi, "LIB_PATH", str(tmp_path / "absent.so"))
    with pytest.raises(RuntimeError, match="no CPU or PyTorch fallback"):
        capi.load()
