"""bench.py's command line on CPU: the reference arm prints exactly one JSON line with the
agreed keys (whole passes over the workload's matrix, oracle port on the host threads, the
step and warm-up counts it was given), the product arm refuses to run without a GPU instead
of falling back, and the record of measured DRAM traffic is only used for the kernel sources
it was captured from."""
import json
import os
import subprocess
import sys

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _run(*args, env=None):
    e = dict(os.environ)
    e.update(env or {})
    return subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), *args], capture_output=True, text=True,
                          env=e, timeout=600)


def test_reference_arm_prints_one_json_line(oracle_cpu):
    res = _run("--impl", "reference", "--scale", "14", "--steps", "2", "--warmup", "1")
    assert res.returncode == 0, res.stderr
    lines = [l for l in res.stdout.splitlines() if l.strip()]
    assert len(lines) == 1
    d = json.loads(lines[0])
    assert d["impl"] == "reference" and d["unit"] == "GFLOP/s" and d["value"] > 0 and d["higher_is_better"] is True
    assert d["cpu_baseline"]["kind"] == "port" and d["cpu_baseline"]["cores"] >= 1 and d["cpu_baseline"]["sample"]
    assert d["e2e"] == {"value": d["value"], "unit": "GFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}
    assert d["config"]["workload"] == "rmat14_spmm_n128" and d["steps"] == 2 and d["warmup"] == 1
    assert d["config"]["rows"] == 1 << 14 and d["config"]["n"] == 128 and d["config"]["nnz"] > 0
    assert str(d["config"]["nnz"]) in d["cpu_baseline"]["sample"]      # whole passes over that very matrix


def test_reference_arm_uses_all_cores_under_a_launcher_that_sets_omp_threads(oracle_cpu):
    """torchrun exports OMP_NUM_THREADS=1; the reference arm must still use the host's cores."""
    res = _run("--impl", "reference", "--scale", "12", "--steps", "1", "--warmup", "1", env={"OMP_NUM_THREADS": "1"})
    assert res.returncode == 0, res.stderr
    d = json.loads(res.stdout.strip().splitlines()[-1])
    assert d["cpu_baseline"]["cores"] == len(os.sched_getaffinity(0))


def test_reference_arm_other_ranks_exit_silently():
    res = _run("--impl", "reference", "--gpus", "2", "--scale", "12", "--steps", "1", env={"RANK": "1", "WORLD_SIZE": "2"})
    assert res.returncode == 0 and res.stdout.strip() == ""


def test_product_arm_needs_a_gpu():
    if torch.cuda.is_available():
        return
    res = _run("--steps", "1")
    assert res.returncode != 0 and "no CPU path" in (res.stderr + res.stdout)


def test_traffic_record_is_tied_to_the_kernel_sources(tmp_path, monkeypatch):
    sys.path.insert(0, ROOT)
    import bench

    digest = bench.kernel_source_digest()
    rec = {"commit": "abc1234", "kernel_source_digest": digest,
           "captures": {"rmat23_n128_hints": {"kernel": "rode::spmm_block<...>", "launches": 1,
                                              "dram_bytes_per_launch": 123}}}
    path = tmp_path / "traffic.json"
    path.write_text(json.dumps(rec))
    monkeypatch.setattr(bench, "TRAFFIC_FILE", str(path))
    value, source = bench.measured_traffic(23, True)
    assert value == 123 and "abc1234" in source
    assert bench.measured_traffic(23, False)[0] is None          # no capture of the plain kernel
    assert bench.measured_traffic(21, True)[0] is None
    rec["kernel_source_digest"] = "0" * 16                          # the sources changed since the capture
    path.write_text(json.dumps(rec))
    value, why = bench.measured_traffic(23, True)
    assert value is None and "changed" in why
    monkeypatch.setattr(bench, "TRAFFIC_FILE", str(tmp_path / "missing.json"))
    assert bench.measured_traffic(23, True)[0] is None

