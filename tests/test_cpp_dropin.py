"""A C++ program written against the reference's declarations builds against include/ and
links with librode_b200.so (CPU: compile and link only; GPU: run it)."""
import os
import shutil
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
SRC = os.path.join(ROOT, "tests", "cpp", "dropin_main.cu")


def _build(built_library, out_dir):
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    exe = os.path.join(out_dir, "dropin_main")
    lib_dir = os.path.dirname(built_library)
    cmd = [nvcc, "-O2", "-std=c++17", "-gencode", "arch=compute_100a,code=sm_100a", SRC, "-I", os.path.join(ROOT, "include"),
           "-L", lib_dir, "-lrode_b200", "-Xlinker", "-rpath", "-Xlinker", lib_dir, "-o", exe]
    res = subprocess.run(cmd, capture_output=True, text=True)
    assert res.returncode == 0, res.stdout + res.stderr
    return exe


def test_reference_style_program_compiles_and_links(built_library, tmp_path):
    exe = _build(built_library, str(tmp_path))
    assert os.path.exists(exe)
    syms = subprocess.run(["nm", "-u", exe], capture_output=True, text=True).stdout
    for name in ("RoDeSpmm_n32", "RoDeSDDMM_n32", "RoDe_preprocess", "RoDe_preprocess_cpu"):
        assert name in syms, name      # resolved from the shared library, not compiled in


@pytest.mark.gpu
def test_reference_style_program_runs(built_library, tmp_path):
    exe = _build(built_library, str(tmp_path))
    res = subprocess.run([exe], capture_output=True, text=True, timeout=120)
    assert res.returncode == 0 and res.stdout.startswith("PASS"), res.stdout + res.stderr
