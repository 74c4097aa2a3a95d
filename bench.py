#!/usr/bin/env python
"""Benchmark of the RoDe hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Headline workload: SpMM, N = 128, fp32, on an R-MAT scale-23 graph (8,388,608 vertices,
edge factor 16, a/b/c/d = 0.57/0.19/0.19/0.05, duplicates removed), rows nnz-balanced over
the ranks, dense operand broadcast once at set-up.  One "step" is one pass of the hot path
(block, fix-up and residue kernels) over the rank's rows.  `value` is whole-job
GFLOP/s = 2 * nnz * N / (max over ranks of the device time per step).

The same line carries: `roofline` (dominant kernel, algorithmic bytes / measured time
against the measured HBM copy bandwidth), `e2e` (host buffers -> H2D -> preprocessing ->
SpMM -> D2H every step), `sddmm` (K = 64 on the same matrix), `cpu_baseline` (CPU oracle on
the host cores, N = 1 only) and, at N = 1, `configs`: the other benchmark matrices with the
reference's own kernels (compiled for sm_100a into oracle/_ref) timed beside ours.

`--hints on` (default) lets the SpMM use the library's column popularity hints where the
library finds them useful (built once at set-up like the preprocessing, and again in every
end-to-end step because the matrix arrives with the step); `--hints off` runs the plain
entry point.  `hints` in the line says what was used and what the pass cost.

`--impl reference` times the CPU implementation (the oracle's restatement of CSR SpMM; the
reference has no CPU SpMM of its own) on all host threads and prints the same line shape.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import torch  # noqa: E402

N_DENSE = 128
K_SDDMM = 64
METRIC = "SpMM GFLOP/s (2*nnz*N), fp32"
FALLBACK_HBM_GBS = 6650.0
# Measured DRAM traffic of one rode::spmm_block launch (ncu, single-pass capture of the two DRAM
# byte counters).  The file records which build of the SpMM sources the capture saw; when the
# sources have changed since, the number no longer describes the kernel that is timed here and
# `traffic` is reported as null.
TRAFFIC_FILE = os.path.join(ROOT, "profiles", "spmm_block_dram_traffic.json")
KERNEL_SOURCES = ("rode_b200/csrc/rode_spmm.cu", "rode_b200/csrc/rode_common.cuh")


def kernel_source_digest() -> str:
    import hashlib

    h = hashlib.sha256()
    for rel in KERNEL_SOURCES:
        with open(os.path.join(ROOT, rel), "rb") as f:
            h.update(f.read())
    return h.hexdigest()[:16]


def measured_traffic(scale: int, hints: bool):
    """(bytes per launch, description) from the capture record, or (None, why not)."""
    try:
        with open(TRAFFIC_FILE) as f:
            rec = json.load(f)
    except Exception:
        return None, "no capture record"
    if rec.get("kernel_source_digest") != kernel_source_digest():
        return None, "the SpMM sources changed after the last ncu capture; no DRAM byte count for this build"
    key = f"rmat{scale}_n{N_DENSE}_{'hints' if hints else 'plain'}"
    entry = rec.get("captures", {}).get(key)
    if entry is None:
        return None, f"no capture of {key}"
    return int(entry["dram_bytes_per_launch"]), (f"ncu dram__bytes_read.sum + dram__bytes_write.sum of "
                                                 f"{entry['kernel']}, {entry['launches']} launch(es), "
                                                 f"captured at commit {rec.get('commit', '?')}")


def parse_args():
    p = argparse.ArgumentParser()
    p.add_argument("--gpus", type=int, default=1)
    p.add_argument("--steps", type=int, default=20)
    p.add_argument("--warmup", type=int, default=3)
    p.add_argument("--impl", default="ours", choices=["ours", "reference"])
    p.add_argument("--scale", type=int, default=23, help="R-MAT scale of the headline workload")
    p.add_argument("--no-extra", action="store_true", help="skip the secondary configs and the CPU baseline")
    p.add_argument("--e2e-steps", type=int, default=20)
    p.add_argument("--repeats", type=int, default=0,
                   help="timed repeats of the --steps loop (0 = at least 10 and at least one second of device time)")
    p.add_argument("--e2e-row-weight", type=float, default=64.0,
                   help="multi-GPU partition of the end-to-end run: cost of a row = its nnz + this; 64 balances the "
                        "bytes a rank moves over PCIe (8 B per nonzero in, 4*N = 512 B per row out)")
    p.add_argument("--row-weight", type=float, default=2.0,
                   help="multi-GPU partition: cost of a row = its nnz + this (0 = plain nnz-balanced)")
    p.add_argument("--hints", choices=["on", "off"], default="on",
                   help="column popularity hints for the SpMM gathers (rode_hot_columns); on = use them where the "
                        "library finds them useful")
    p.add_argument("--hint-budget-mb", type=float, default=0.0,
                   help="bytes of dense rows the hints may mark, in MB (0 = the library's default)")
    p.add_argument("--only", choices=["spmm", "sddmm", "preprocess"], default=None,
                   help="small single-op run (one family, one width) for profiling and A/B timing; for "
                        "preprocess --width is the segment length (512 or 32)")
    p.add_argument("--family", default="rmat", choices=["bernoulli", "zipf", "stencil", "pareto", "rmat"])
    p.add_argument("--width", type=int, default=128, help="N of SpMM / K of SDDMM for --only")
    p.add_argument("--size", type=float, default=1.0, help="row-count factor of the family for --only")
    return p.parse_args()


def measured_peak():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return FALLBACK_HBM_GBS, "fallback"


# ---------------------------------------------------------------------------------------
class ClockSampler:
    """nvidia-smi clock/throttle samples while the timed region runs (read-only query)."""

    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index = index
        self.proc = None
        self.path = f"/tmp/rode_clocks_{os.getpid()}.csv"

    def start(self):
        try:
            self.out = open(self.path, "w")
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                                          "-i", str(self.index), "-lms", "20"], stdout=self.out,
                                         stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        self.out.close()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in open(self.path):
            f = [x.strip() for x in line.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                mx.append(float(f[2]))
            except ValueError:
                continue
            for name, flag in zip(names, f[5:9]):
                if flag.lower().startswith("active"):
                    reasons.add(name)
        try:
            os.remove(self.path)
        except OSError:
            pass
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no samples"]}
        return {"sm_mhz": statistics.median(sm), "sm_max_mhz": max(mx), "reasons": sorted(reasons),
                "samples": len(sm)}


# ---------------------------------------------------------------------------------------
def spmm_bmin(nnz, m, n_dense, k_touched):
    return 8 * nnz + 4 * (m + 1) + 4 * n_dense * k_touched + 4 * n_dense * m


def sddmm_bmin(nnz, m, k, m_nonempty, k_touched):
    return 12 * nnz + 4 * (m + 1) + 4 * k * m_nonempty + 4 * k * k_touched


def distinct_count(t: torch.Tensor) -> int:
    if t.numel() == 0:
        return 0
    s, _ = torch.sort(t)
    return int((s[1:] != s[:-1]).sum()) + 1


def time_loop(fn, steps, warmup, stream, flush=None):
    """Average device milliseconds per call of fn over `steps` calls (after `warmup`), with
    CUDA events on `stream`.  With `flush`, a buffer larger than L2 is rewritten before each
    call and every call is timed by its own event pair (median reported)."""
    for _ in range(warmup):
        if flush is not None:
            flush.add_(1.0)
        fn()
    torch.cuda.synchronize()
    if flush is None:
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record(stream)
        for _ in range(steps):
            fn()
        b.record(stream)
        torch.cuda.synchronize()
        return a.elapsed_time(b) / steps
    times = []
    for _ in range(steps):
        flush.add_(1.0)
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record(stream)
        fn()
        b.record(stream)
        torch.cuda.synchronize()
        times.append(a.elapsed_time(b))
    return statistics.median(times)


def time_preprocess(row_ptr, nnz, seg, iters, peak_gbs, with_host=True, with_swizzle=True):
    """Device time of the preprocessing kernels (raw entry point, buffers allocated
    once), the host twin's single-thread time, and the HBM roofline of the device version:
    algorithmic bytes = row pointer read once + outputs written once."""
    from rode_b200 import capi

    dev = row_ptr.device
    M = row_ptr.numel() - 1
    cap = capi.preprocess_capacity(seg, 4, M, nnz)
    blk = torch.empty(max(cap, 1), dtype=torch.int32, device=dev)
    st = torch.empty(cap + 1, dtype=torch.int32, device=dev)
    res = torch.empty(max(M, 1), dtype=torch.int32, device=dev)
    cnt = torch.zeros(2, dtype=torch.int32, device=dev)
    ws_bytes = capi.preprocess_workspace_bytes(M)
    ws = torch.empty(ws_bytes, dtype=torch.uint8, device=dev)
    stream = torch.cuda.current_stream(dev)

    def run():
        capi.preprocess_raw(seg, 32, 4, M, row_ptr.data_ptr(), blk.data_ptr(), st.data_ptr(), res.data_ptr(),
                            cnt.data_ptr(), cnt.data_ptr() + 4, ws.data_ptr(), ws_bytes, stream)

    ms = time_loop(run, iters, 3, stream)
    m1, m2 = cnt.cpu().tolist()
    algo = 4 * (M + 1) + 8 * m1 + 4 + 4 * m2 + 8
    out = {"seg_len": seg, "rows": M, "m1": m1, "m2": m2, "gpu_ms": ms, "algorithmic_bytes": algo,
           "algorithmic_gbs": algo / ms / 1e6, "frac_of_measured_hbm": algo / ms / 1e6 / peak_gbs}
    if with_swizzle:
        # the comparator the reference times beside its own preprocessing: rows sorted by
        # decreasing length (Preprocess_opt/_preprocess.cu:71-104, a thrust sort_by_key there)
        from rode_b200 import matrix_io

        out["swizzle_gpu_ms"] = time_loop(lambda: matrix_io.row_swizzle(row_ptr), min(iters, 10), 2, stream)
        out["swizzle_over_rode"] = out["swizzle_gpu_ms"] / ms
    if with_host:
        rp_host = row_ptr.cpu()
        t0 = time.perf_counter()
        capi.preprocess_cpu(rp_host, seg, 32, 4)
        out["host_single_thread_ms"] = (time.perf_counter() - t0) * 1e3
    return out


def time_hot_columns(col, n_cols, row_bytes, iters):
    """Device time of the column-popularity pass (raw entry point, buffers allocated once) and
    what it marked."""
    import ctypes

    import numpy as np
    from rode_b200 import capi

    dev = col.device
    words, need = ctypes.c_size_t(0), ctypes.c_size_t(0)
    capi.check(capi.load().rode_hot_columns_words(n_cols, ctypes.byref(words)))
    capi.check(capi.load().rode_hot_columns_workspace_bytes(n_cols, ctypes.byref(need)))
    bitmap = torch.empty(words.value, dtype=torch.int32, device=dev)
    ws = torch.empty(need.value, dtype=torch.uint8, device=dev)
    stream = torch.cuda.current_stream(dev)

    def run():
        capi.hot_columns_raw(col.numel(), n_cols, col.data_ptr(), row_bytes, 0, bitmap.data_ptr(), ws.data_ptr(),
                             need.value, stream)

    ms = time_loop(run, iters, 3, stream)
    raw = bitmap.cpu().numpy().view(np.uint32)
    marked = int(np.unpackbits(raw[:-1].view(np.uint8)).sum())
    return {"gpu_ms": ms, "useful": bool(raw[-1]), "marked_columns": marked, "marked_bytes": marked * row_bytes,
            "budget": "60 % of the device's L2"}


class NumaBinding:
    """Context manager: while it is entered the process runs on the CPUs of the NUMA node the
    given GPU hangs on (read from sysfs), so that host memory allocated and first touched inside
    lands on that node.  Does nothing where the node cannot be determined."""

    def __init__(self, device):
        self.cpus, self.node, self.saved = None, None, None
        try:
            prop = torch.cuda.get_device_properties(device)
            bus = f"{prop.pci_domain_id:04x}:{prop.pci_bus_id:02x}:{prop.pci_device_id:02x}.0"
            with open(f"/sys/bus/pci/devices/{bus}/numa_node") as f:
                node = int(f.read().strip())
            if node < 0:
                return
            with open(f"/sys/devices/system/node/node{node}/cpulist") as f:
                cpus = set()
                for part in f.read().strip().split(","):
                    lo, _, hi = part.partition("-")
                    cpus.update(range(int(lo), int(hi or lo) + 1))
            allowed = os.sched_getaffinity(0)
            if cpus & allowed:
                self.cpus, self.node = cpus & allowed, node
        except Exception:
            pass

    def __enter__(self):
        if self.cpus:
            self.saved = os.sched_getaffinity(0)
            os.sched_setaffinity(0, self.cpus)
        return self

    def __exit__(self, *exc):
        if self.saved is not None:
            os.sched_setaffinity(0, self.saved)
            self.saved = None
        return False


class ForkJoin:
    """Runs the two-stream entry points so that one timing stream sees all of the work:
    block work on the current stream, residue work on a side stream forked from and joined
    back into it."""

    def __init__(self, device):
        self.cur = torch.cuda.current_stream(device)
        self.side = torch.cuda.Stream(device)
        self.fork = torch.cuda.Event()
        self.join = torch.cuda.Event()

    def run(self, launch):
        self.fork.record(self.cur)
        self.side.wait_event(self.fork)
        launch(self.cur, self.side)
        self.join.record(self.side)
        self.cur.wait_event(self.join)


# ---------------------------------------------------------------------------------------
def headline_matrix(scale: int, device):
    from rode_b200 import workloads as W

    return W.rmat(scale=scale, device=device)


def reference_arm(args, rank, world):
    """CPU implementation on the host cores: the oracle's CSR SpMM (the reference ships no
    CPU SpMM), all threads, whole passes over the SAME matrix and dense operand as the GPU arm
    (same generator, seed, scale and width); `--steps` timed passes after `--warmup` untimed
    ones.  Only rank 0 works; the other ranks of a multi-process launch leave at once."""
    if rank != 0:
        return None
    from oracle import cpu
    from rode_b200 import workloads as W

    threads = cpu.max_threads()
    # the generator draws the same matrix on either device type only from the same kind of
    # random stream, so it runs where the GPU arm runs it (on the GPU when one is visible)
    gen_dev = torch.device("cuda", 0) if torch.cuda.is_available() else torch.device("cpu")
    A = headline_matrix(args.scale, gen_dev)
    B = W.dense(A.n, N_DENSE, device=gen_dev, seed=3).cpu().numpy()
    rp, col, val = A.row_ptr.cpu().numpy(), A.col.cpu().numpy(), A.val.cpu().numpy()
    m, n_cols, nnz = A.m, A.n, A.nnz
    del A
    if gen_dev.type == "cuda":
        torch.cuda.empty_cache()
    warm = max(0, args.warmup)
    for _ in range(warm):
        cpu.spmm_f32(rp, col, val, B, threads=threads)
    steps = max(1, args.steps)
    times = []
    for _ in range(steps):
        t0 = time.perf_counter()
        out = cpu.spmm_f32(rp, col, val, B, threads=threads)
        times.append((time.perf_counter() - t0) * 1e3)
    ms = sum(times) / steps
    gflops = 2.0 * nnz * N_DENSE / (ms * 1e-3) / 1e9
    sample = (f"whole passes over the headline matrix (R-MAT scale {args.scale}, nnz {nnz}, N={N_DENSE}), "
              f"{ms / 1e3:.3f} s per pass, matrix drawn on {gen_dev.type}")
    line = {
        "impl": "reference", "metric": METRIC, "value": gflops, "unit": "GFLOP/s", "n_gpus": args.gpus,
        "steps": steps, "warmup": warm, "ms_per_step": ms, "ms_per_step_median": statistics.median(times),
        "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": f"rmat{args.scale}_spmm_n{N_DENSE}", "rows": m, "nnz": nnz, "n": N_DENSE},
        "cpu_baseline": {"value": gflops, "unit": "GFLOP/s", "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": gflops, "unit": "GFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "checksum": float(out.astype("float64").sum()),
    }
    return line


# ---------------------------------------------------------------------------------------
def secondary_configs(peak_gbs, steps, warmup):
    """The other benchmark matrices at N = 1: ours and, where its preconditions hold, the
    reference's own kernels compiled for sm_100a (oracle/_ref), on the same device arrays."""
    from oracle import ref
    from rode_b200 import capi
    from rode_b200 import workloads as W

    dev = torch.device("cuda", torch.cuda.current_device())
    fj = ForkJoin(dev)
    flush = torch.zeros(64 * 1024 * 1024, device=dev)  # 256 MB > L2
    out = {}
    have_ref = ref.available()
    specs = [
        ("cfg1_bernoulli4096", lambda: W.bernoulli(device=dev), [("spmm", 32), ("sddmm", 32)]),
        ("cfg2_zipf65536", lambda: W.zipf_rows(device=dev), [("spmm", 128)]),
        ("cfg3_stencil128", lambda: W.stencil27(128, device=dev), [("spmm", 64), ("sddmm", 64)]),
        ("cfg4_pareto1m", lambda: W.pareto_rows(device=dev), [("spmm", 32), ("spmm", 128), ("sddmm", 32),
                                                              ("sddmm", 128), ("spmm_f64", 32), ("spmm_f64", 128)]),
    ]
    for name, make, ops in specs:
        A = make()
        k_touched = distinct_count(A.col)
        lens = A.row_ptr[1:] - A.row_ptr[:-1]
        m_nonempty = int((lens > 0).sum())
        for op, width in ops:
            seg = 32 if (op == "sddmm" and width == 128) else 512
            meta = capi.preprocess(A.row_ptr, A.nnz, seg, 32, 4)
            entry = {"nnz": A.nnz, "m1": meta.m1, "m2": meta.m2}
            pre = time_preprocess(A.row_ptr, A.nnz, seg, 10, peak_gbs, with_host=False)
            entry["preprocess_gpu_ms"] = pre["gpu_ms"]
            entry["swizzle_gpu_ms"] = pre["swizzle_gpu_ms"]
            if op in ("spmm", "spmm_f64"):
                dt = torch.float64 if op == "spmm_f64" else torch.float32
                esz = 8 if op == "spmm_f64" else 4
                B = W.dense(A.n, width, device=dev, seed=3, dtype=dt)
                vals = A.val.to(dt)
                C = torch.zeros((A.m, width), device=dev, dtype=dt)
                need = capi.spmm_workspace_bytes(meta.m1, width, esz)
                ws = torch.empty(max(need, 16), dtype=torch.uint8, device=dev)

                def ours(s1, s2):
                    capi.spmm_raw(dt, meta.m1, meta.m2, A.n, width, vals.data_ptr(), A.col.data_ptr(),
                                  A.row_ptr.data_ptr(), meta.block_r_ind.data_ptr(), meta.residue_r_ind.data_ptr(),
                                  meta.st_off.data_ptr(), B.data_ptr(), C.data_ptr(), ws.data_ptr(), need, s1, s2)

                def theirs(s1, s2):
                    ref.spmm_gpu(32 if width == 32 else 128, op == "spmm_f64", meta.m1, meta.m2, A.n, width,
                                 vals.data_ptr(), A.col.data_ptr(), A.row_ptr.data_ptr(), meta.block_r_ind.data_ptr(),
                                 meta.residue_r_ind.data_ptr(), meta.st_off.data_ptr(), B.data_ptr(), C.data_ptr(),
                                 s1.cuda_stream, s2.cuda_stream)

                bmin = (spmm_bmin(A.nnz, A.m, width, k_touched) if esz == 4 else
                        12 * A.nnz + 4 * (A.m + 1) + 8 * width * k_touched + 8 * width * A.m)
                # the reference's kernels: both grids non-empty, width 32 or a multiple of 64,
                # and byte offsets col * n * sizeof(T) below 2^31
                ref_ok = (have_ref and meta.m1 > 0 and meta.m2 > 0 and width in (32, 128)
                          and (A.n - 1) * width * esz < 2**31)
            else:
                lhs = W.dense(A.m, width, device=dev, seed=5)
                rhs = W.dense(A.n, width, device=dev, seed=6)
                res = torch.zeros(A.nnz, device=dev)

                def ours(s1, s2):
                    capi.sddmm_raw(meta.m1, meta.m2, A.n, width, meta.block_r_ind.data_ptr(),
                                   meta.residue_r_ind.data_ptr(), meta.st_off.data_ptr(), A.row_ptr.data_ptr(),
                                   A.col.data_ptr(), A.val.data_ptr(), lhs.data_ptr(), rhs.data_ptr(), res.data_ptr(),
                                   s1, s2)

                def theirs(s1, s2):
                    ref.sddmm_gpu(width, meta.m1, meta.m2, A.n, meta.block_r_ind.data_ptr(),
                                  meta.residue_r_ind.data_ptr(), meta.st_off.data_ptr(), A.row_ptr.data_ptr(),
                                  A.col.data_ptr(), A.val.data_ptr(), lhs.data_ptr(), rhs.data_ptr(), res.data_ptr(),
                                  s1.cuda_stream, s2.cuda_stream)

                bmin = sddmm_bmin(A.nnz, A.m, width, m_nonempty, k_touched)
                # the reference SDDMM skips a kernel on a null stream and has K = 32 / 128 only
                ref_ok = have_ref and width in (32, 128) and meta.m1 > 0 and meta.m2 > 0 and (A.n - 1) * width < 2**29
            # context column: the vendor library through torch (cuSPARSE SpMM / sampled_addmm)
            lib_ms = None
            try:
                csr_t = torch.sparse_csr_tensor(A.row_ptr.long(), A.col.long(), A.val, size=(A.m, A.n))
                if op == "spmm_f64":
                    raise RuntimeError("fp64 comparison with the vendor library not timed")
                if op == "spmm":
                    lib_fn = lambda: torch.sparse.mm(csr_t, B)  # noqa: E731
                else:
                    rhs_t = rhs.t()
                    lib_fn = lambda: torch.sparse.sampled_addmm(csr_t, lhs, rhs_t, beta=0.0)  # noqa: E731
                lib_ms = time_loop(lib_fn, min(steps, 5), 2, fj.cur, flush)
                del csr_t
            except Exception as exc:  # library path unavailable for this shape: leave the column empty
                entry["vendor_library_error"] = str(exc)[:120]
            ms = time_loop(lambda: fj.run(ours), steps, warmup, fj.cur, flush)
            if lib_ms is not None:
                entry.update({"vendor_library_ms": lib_ms, "speedup_vs_vendor_library": lib_ms / ms})
            entry.update({"ms": ms, "gflops": 2.0 * A.nnz * width / ms / 1e6, "bmin_bytes": bmin,
                          "algorithmic_gbs": bmin / ms / 1e6, "frac_of_measured_hbm": bmin / ms / 1e6 / peak_gbs})
            if ms < 0.2:
                # launch-bound sizes: the same three launches captured once in a CUDA graph and replayed
                try:
                    cap_stream, cap_side = torch.cuda.Stream(dev), torch.cuda.Stream(dev)
                    graph = torch.cuda.CUDAGraph()
                    torch.cuda.synchronize()
                    with torch.cuda.graph(graph, stream=cap_stream):
                        cap_side.wait_stream(cap_stream)
                        ours(cap_stream, cap_side)
                        cap_stream.wait_stream(cap_side)
                    entry["graph_replay_ms"] = time_loop(graph.replay, steps, warmup, fj.cur, flush)
                    del graph
                except Exception as exc:
                    entry["graph_replay_error"] = str(exc)[:160]
                    torch.cuda.synchronize()
            if ref_ok:
                side1 = torch.cuda.Stream(dev)  # the reference needs two real (non-null) streams

                def run_theirs():
                    fj.fork.record(fj.cur)
                    side1.wait_event(fj.fork)
                    fj.side.wait_event(fj.fork)
                    theirs(side1, fj.side)
                    e1, e2 = torch.cuda.Event(), torch.cuda.Event()
                    e1.record(side1)
                    e2.record(fj.side)
                    fj.cur.wait_event(e1)
                    fj.cur.wait_event(e2)

                rms = time_loop(run_theirs, steps, warmup, fj.cur, flush)
                entry.update({"reference_kernels_ms": rms, "speedup_vs_reference_kernels": rms / ms})
            out[f"{name}_{op}{'_' if op.endswith('64') else ''}{width}"] = entry
            torch.cuda.synchronize()
        del A
        torch.cuda.empty_cache()
    return out


def make_family(name, device, scale=23, size=1.0):
    from rode_b200 import workloads as W

    if name == "bernoulli":
        return W.bernoulli(device=device)
    if name == "zipf":
        m = int(65536 * size)
        return W.zipf_rows(m=m, n=m, device=device)
    if name == "stencil":
        return W.stencil27(max(4, int(round(128 * size ** (1.0 / 3.0)))), device=device)
    if name == "pareto":
        m = int((1 << 20) * size)
        return W.pareto_rows(m=m, n=m, device=device)
    return W.rmat(scale=scale, device=device)


def single_op(args):
    """One family, one op, one width on cuda:0: `warmup` untimed and `steps` timed launches of
    the entry point and nothing else (a run small enough to profile)."""
    from rode_b200 import capi
    from rode_b200 import workloads as W

    capi.load()
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    peak_gbs, peak_kind = measured_peak()
    A = make_family(args.family, dev, args.scale, args.size)
    width = args.width
    if args.only == "preprocess":
        # `steps` calls back to back on pre-allocated buffers (the raw entry point), as the full run times it
        seg = width if width in (32, 512) else 512
        pre = time_preprocess(A.row_ptr, A.nnz, seg, args.steps, peak_gbs, with_host=False, with_swizzle=False)
        return {"only": "preprocess", "family": args.family, **pre, "peak_kind": peak_kind}
    seg = 32 if (args.only == "sddmm" and width == 128) else 512
    meta = capi.preprocess(A.row_ptr, A.nnz, seg, 32, 4)
    fj = ForkJoin(dev)
    k_touched = distinct_count(A.col)
    lens = A.row_ptr[1:] - A.row_ptr[:-1]
    if args.only == "spmm":
        B = W.dense(A.n, width, device=dev, seed=3)
        C = torch.zeros((A.m, width), device=dev)
        need = capi.spmm_workspace_bytes(meta.m1, width, 4)
        ws = torch.empty(max(need, 16), dtype=torch.uint8, device=dev)
        hot = (capi.hot_columns(A.col, A.n, 4 * width, budget_bytes=int(args.hint_budget_mb * 1e6))
               if args.hints == "on" else None)
        hot_ptr = None if hot is None else hot.data_ptr()

        def launch(s1, s2):
            capi.spmm_raw(torch.float32, meta.m1, meta.m2, A.n, width, A.val.data_ptr(), A.col.data_ptr(),
                          A.row_ptr.data_ptr(), meta.block_r_ind.data_ptr(), meta.residue_r_ind.data_ptr(),
                          meta.st_off.data_ptr(), B.data_ptr(), C.data_ptr(), ws.data_ptr(), need, s1, s2,
                          hot=hot_ptr)

        bmin = spmm_bmin(A.nnz, A.m, width, k_touched)
    else:
        lhs = W.dense(A.m, width, device=dev, seed=5)
        rhs = W.dense(A.n, width, device=dev, seed=6)
        res = torch.zeros(A.nnz, device=dev)

        def launch(s1, s2):
            capi.sddmm_raw(meta.m1, meta.m2, A.n, width, meta.block_r_ind.data_ptr(), meta.residue_r_ind.data_ptr(),
                           meta.st_off.data_ptr(), A.row_ptr.data_ptr(), A.col.data_ptr(), A.val.data_ptr(),
                           lhs.data_ptr(), rhs.data_ptr(), res.data_ptr(), s1, s2)

        bmin = sddmm_bmin(A.nnz, A.m, width, int((lens > 0).sum()), k_touched)
    flush = torch.zeros(64 * 1024 * 1024, device=dev)
    ms = time_loop(lambda: fj.run(launch), args.steps, args.warmup, fj.cur, flush)
    return {"only": args.only, "family": args.family, "width": width, "rows": A.m, "nnz": A.nnz,
            "hints": bool(args.only == "spmm" and hot is not None),
            "m1": meta.m1, "m2": meta.m2, "ms": ms, "gflops": 2.0 * A.nnz * width / ms / 1e6,
            "bmin_bytes": bmin, "algorithmic_gbs": bmin / ms / 1e6,
            "frac": bmin / ms / 1e6 / peak_gbs, "peak_kind": peak_kind, "k_touched": k_touched}


# ---------------------------------------------------------------------------------------
class QuietStdout:
    """Everything the process (or a library underneath it, e.g. NCCL's version banner) writes
    to file descriptor 1 goes to stderr; only the final JSON line goes to the real stdout."""

    def __init__(self):
        sys.stdout.flush()
        self.saved = os.dup(1)
        os.dup2(2, 1)

    def emit(self, text: str):
        sys.stdout.flush()
        os.dup2(self.saved, 1)
        print(text, flush=True)


def main():
    args = parse_args()
    console = QuietStdout()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        line = reference_arm(args, rank, world)
        if line is not None:
            console.emit(json.dumps(line))
        return
    if args.only is not None:
        console.emit(json.dumps(single_op(args)))
        return

    import torch.distributed as dist

    from rode_b200 import capi
    from rode_b200 import workloads as W

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (B200); there is no CPU path")
    capi.load()  # fails loudly when librode_b200.so is missing
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(x: float) -> float:
        if world == 1:
            return x
        t = torch.tensor([x], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t)

    def sum_over_ranks(x: float) -> float:
        if world == 1:
            return x
        t = torch.tensor([x], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.SUM)
        return float(t)

    peak_gbs, peak_kind = measured_peak()

    # ---- set-up: rank 0 draws the matrix and the dense operands; one broadcast each -------
    t_setup = time.perf_counter()
    n_vert = 1 << args.scale
    if rank == 0:
        A = headline_matrix(args.scale, dev)
        sizes = torch.tensor([A.nnz], dtype=torch.int64, device=dev)
    else:
        A = None
        sizes = torch.zeros(1, dtype=torch.int64, device=dev)
    if world > 1:
        dist.broadcast(sizes, 0)
    nnz = int(sizes[0])
    if rank == 0:
        row_ptr, col, val = A.row_ptr, A.col, A.val
        X = W.dense(n_vert, N_DENSE, device=dev, seed=3)
        rhs = W.dense(n_vert, K_SDDMM, device=dev, seed=6)
    else:
        row_ptr = torch.empty(n_vert + 1, dtype=torch.int32, device=dev)
        col = torch.empty(nnz, dtype=torch.int32, device=dev)
        val = torch.empty(nnz, dtype=torch.float32, device=dev)
        X = torch.empty((n_vert, N_DENSE), dtype=torch.float32, device=dev)
        rhs = torch.empty((n_vert, K_SDDMM), dtype=torch.float32, device=dev)
    broadcast_ms = None
    if world > 1:
        for t in (row_ptr, col, val, rhs):
            dist.broadcast(t, 0)
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        dist.broadcast(X, 0)  # the dense operand of the headline op: one NCCL broadcast
        e1.record()
        torch.cuda.synchronize()
        broadcast_ms = e0.elapsed_time(e1)
    full = W.CSR(n_vert, n_vert, row_ptr, col, val)
    bounds = W.partition_rows(row_ptr, world, args.row_weight)
    r0, r1 = bounds[rank], bounds[rank + 1]
    mine = full.rows(r0, r1)
    # The end-to-end run is bound by PCIe, not by the kernels, so its rows are cut by the bytes
    # a rank moves per step (8 B per nonzero in, 4*N B per row of C out) instead of by kernel cost.
    if world > 1 and args.e2e_row_weight != args.row_weight:
        e2e_bounds = W.partition_rows(row_ptr, world, args.e2e_row_weight)
        e2e_r0, e2e_r1 = e2e_bounds[rank], e2e_bounds[rank + 1]
        mine_e2e = full.rows(e2e_r0, e2e_r1)
    else:
        e2e_r0, e2e_r1, mine_e2e = r0, r1, mine
    if world > 1:
        del full, row_ptr, col, val
        torch.cuda.empty_cache()
    my_nnz, my_rows = mine.nnz, mine.m
    meta = capi.preprocess(mine.row_ptr, my_nnz, 512, 32, 4)
    preprocess_info = time_preprocess(mine.row_ptr, my_nnz, 512, 20, peak_gbs, with_host=(world == 1))
    C = torch.zeros((my_rows, N_DENSE), dtype=torch.float32, device=dev)
    ws_bytes = capi.spmm_workspace_bytes(meta.m1, N_DENSE, 4)
    ws = torch.empty(max(ws_bytes, 16), dtype=torch.uint8, device=dev)
    fj = ForkJoin(dev)
    # column popularity bitmap of this rank's rows (set-up, like the preprocessing; timed below)
    hot = (capi.hot_columns(mine.col, n_vert, 4 * N_DENSE, budget_bytes=int(args.hint_budget_mb * 1e6))
           if args.hints == "on" else None)
    hot_ptr = None if hot is None else hot.data_ptr()
    hints_info = {"requested": args.hints == "on", "used": hot is not None}
    if args.hints == "on":
        hints_info.update(time_hot_columns(mine.col, n_vert, 4 * N_DENSE, 10))
    setup_s = time.perf_counter() - t_setup

    def spmm_launch(s1, s2, m1=None, m2=None):
        capi.spmm_raw(torch.float32, meta.m1 if m1 is None else m1, meta.m2 if m2 is None else m2, n_vert, N_DENSE,
                      mine.val.data_ptr(), mine.col.data_ptr(), mine.row_ptr.data_ptr(), meta.block_r_ind.data_ptr(),
                      meta.residue_r_ind.data_ptr(), meta.st_off.data_ptr(), X.data_ptr(), C.data_ptr(),
                      ws.data_ptr(), ws_bytes, s1, s2, hot=hot_ptr)

    def step():
        fj.run(spmm_launch)

    # ---- timed region -------------------------------------------------------------------
    # EXACTLY `steps` steps between a barrier + synchronize on both sides, timed with CUDA
    # events on the launching stream, max over ranks; the whole bracket is repeated and the
    # median repeat reported, so that the timed region spans at least a second and one slow
    # repeat (clock ramp, power cap) does not decide the number.
    warm = max(args.warmup, 3)
    for _ in range(warm):
        step()
    barrier()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)

    def timed_repeat():
        barrier()
        a.record(fj.cur)
        for _ in range(args.steps):
            step()
        b.record(fj.cur)
        barrier()
        return max_over_ranks(a.elapsed_time(b) / args.steps)

    first = timed_repeat()                      # also sizes the number of repeats
    repeats = args.repeats if args.repeats > 0 else max(10, int(1000.0 / max(first * args.steps, 1e-3)) + 1)
    repeats = min(repeats, 200)
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    repeat_ms = [timed_repeat() for _ in range(repeats)]
    clocks = sampler.stop() if rank == 0 else None
    ms_step = statistics.median(repeat_ms)
    launches_per_step = (2 if meta.m1 > 0 else 0) + (1 if meta.m2 > 0 else 0)
    gflops = 2.0 * nnz * N_DENSE / ms_step / 1e6
    timing = {"repeats": repeats, "steps_per_repeat": args.steps, "ms_per_step_of_each_repeat": repeat_ms,
              "ms_per_step_min": min(repeat_ms), "ms_per_step_max": max(repeat_ms),
              "timed_region_s": sum(repeat_ms) * args.steps / 1e3,
              # time x clock: comparable between boxes whose power cap settles at different clocks
              "ms_per_step_x_sm_mhz": (ms_step * clocks["sm_mhz"]) if clocks and clocks.get("sm_mhz") else None}

    # ---- per-kernel timing and the roofline of the dominant kernel ---------------------------
    lens = (mine.row_ptr[1:] - mine.row_ptr[:-1]).to(torch.int64)
    aligned = lens + (mine.row_ptr[:-1] % 4)
    in_block = aligned >= 32                                   # rows finished by spmm_block
    rows_block = int(in_block.sum())
    nnz_block = int(lens[in_block].sum())
    entry_in_block = torch.repeat_interleave(in_block, lens)
    kt_block = distinct_count(mine.col[entry_in_block])
    kt_all = distinct_count(mine.col)
    del entry_in_block
    block_bytes = 8 * nnz_block + 4 * N_DENSE * kt_block + 4 * N_DENSE * rows_block
    ms_block = time_loop(lambda: spmm_launch(fj.cur, fj.cur, m2=0), args.steps, 3, fj.cur) if meta.m1 > 0 else 0.0
    ms_residue = time_loop(lambda: spmm_launch(fj.cur, fj.cur, m1=0), args.steps, 3, fj.cur) if meta.m2 > 0 else 0.0
    ms_block = max_over_ranks(ms_block)
    ms_residue = max_over_ranks(ms_residue)
    block_bytes_all = sum_over_ranks(float(block_bytes))
    step_bytes_all = sum_over_ranks(float(spmm_bmin(my_nnz, my_rows, N_DENSE, kt_all)))
    roofline = {
        "kernel": ("rode::spmm_block<float,32> (timed with spmm_fixup, which follows it on the same stream)"
                   + ("; dense rows of popular columns gathered with L2 evict_last" if hot is not None else "")),
        "bound": "hbm", "achieved": block_bytes_all / world / ms_block / 1e6 if ms_block else None,
        "peak": peak_gbs, "unit": "GB/s", "peak_kind": f"of {peak_kind}",
        "frac": (block_bytes_all / world / ms_block / 1e6 / peak_gbs) if ms_block else None,
        "traffic": None, "algorithmic_bytes_per_launch": block_bytes_all / world, "ms_per_launch": ms_block,
        "residue_kernel_ms": ms_residue,
        # upper bracket of the traffic model: every gather counted (no reuse of dense rows at all)
        "no_reuse": {"bytes_per_launch": (8 * nnz_block + 4 * N_DENSE * nnz_block + 4 * N_DENSE * rows_block),
                     "achieved": ((8 * nnz_block + 4 * N_DENSE * nnz_block + 4 * N_DENSE * rows_block) / ms_block / 1e6
                                  if ms_block else None),
                     "note": "rank 0's launch; bytes requested from L1/L2/HBM, of which `traffic` reach DRAM"},
        "step": {"algorithmic_bytes": step_bytes_all, "achieved": step_bytes_all / ms_step / 1e6,
                 "frac": step_bytes_all / ms_step / 1e6 / (peak_gbs * world),
                 "note": "B_min = 8*nnz + 4*(M+1) + 4*N*K_touched + 4*N*M counts a C row for every row of the "
                         "matrix; the kernels store only the rows that have a nonzero"},
    }
    if world == 1 and not args.hint_budget_mb:
        traffic, source = measured_traffic(args.scale, hot is not None)
        roofline["traffic"] = traffic
        roofline["traffic_source"] = source
        roofline["traffic_gbs"] = traffic / ms_block / 1e6 if traffic and ms_block else None
    # What this access order can reach at best with an ideal cache of the L2's size: the C most
    # referenced dense rows (C = L2 bytes / row bytes) are fetched once and then always hit, every
    # other reference misses.  A lower bound of the block kernel's DRAM bytes that, unlike B_min,
    # knows that the gathers of a row-major pass cannot all be served from a 126 MB cache.
    if meta.m1 > 0:
        l2_bytes = torch.cuda.get_device_properties(dev).L2_cache_size
        cached = l2_bytes // (4 * N_DENSE)
        deg = torch.bincount(mine.col[torch.repeat_interleave(in_block, lens)].long(), minlength=1)
        deg_sorted, _ = torch.sort(deg[deg > 0], descending=True)
        refs_total = int(deg_sorted.sum())
        refs_cached = int(deg_sorted[:cached].sum())
        cols_cached = int(min(cached, deg_sorted.numel()))
        floor_bytes = (8 * nnz_block + 4 * N_DENSE * (cols_cached + refs_total - refs_cached)
                       + 4 * N_DENSE * rows_block)
        roofline["floor_model"] = {
            "bytes_per_launch": floor_bytes, "cache_bytes": l2_bytes, "cached_columns": cols_cached,
            "references_served_from_cache": refs_cached / max(refs_total, 1),
            "ms_at_peak": floor_bytes / peak_gbs / 1e6,
            "frac": (floor_bytes / ms_block / 1e6 / peak_gbs) if ms_block else None,
            "note": "ideal-cache lower bound of DRAM bytes for a row-major pass: the most referenced dense rows "
                    "that fit the whole L2 are read once, every other gather misses; rank 0's launch"}
        del deg, deg_sorted

    # ---- SDDMM K = 64 on the same rows ---------------------------------------------------------
    lhs = W.dense(n_vert, K_SDDMM, device=dev, seed=5)[r0:r1].contiguous()
    out = torch.zeros(my_nnz, dtype=torch.float32, device=dev)

    def sddmm_launch(s1, s2):
        capi.sddmm_raw(meta.m1, meta.m2, n_vert, K_SDDMM, meta.block_r_ind.data_ptr(), meta.residue_r_ind.data_ptr(),
                       meta.st_off.data_ptr(), mine.row_ptr.data_ptr(), mine.col.data_ptr(), mine.val.data_ptr(),
                       lhs.data_ptr(), rhs.data_ptr(), out.data_ptr(), s1, s2)

    barrier()
    ms_sddmm = max_over_ranks(time_loop(lambda: fj.run(sddmm_launch), args.steps, 3, fj.cur))
    sddmm_bytes = sum_over_ranks(float(sddmm_bmin(my_nnz, my_rows, K_SDDMM, int((lens > 0).sum()), kt_all)))
    sddmm = {"metric": "SDDMM GFLOP/s (2*nnz*K), fp32", "k": K_SDDMM, "ms_per_step": ms_sddmm,
             "value": 2.0 * nnz * K_SDDMM / ms_sddmm / 1e6, "unit": "GFLOP/s", "algorithmic_bytes": sddmm_bytes,
             "algorithmic_gbs": sddmm_bytes / ms_sddmm / 1e6,
             "frac_of_measured_hbm": sddmm_bytes / ms_sddmm / 1e6 / (peak_gbs * world)}
    del lhs, out

    # ---- end to end: host buffers in, host result out, every step -----------------------------
    # Host side of the job: every rank holds its CSR slice and, at N > 1, 1/N of the dense
    # operand's rows in pinned memory; the operand is assembled on the GPUs by one all-gather
    # over NVLink per step instead of N full copies over PCIe.
    del C
    src = mine_e2e
    e_nnz, e_rows = src.nnz, src.m
    # The pinned host buffers are allocated and first touched while this process is bound to the
    # CPUs of the GPU's own NUMA node, so that their pages sit in the memory next to the GPU's
    # PCIe root (otherwise the copies of half the GPUs of a two-socket host cross the socket link).
    numa = NumaBinding(dev)
    with numa:
        h_rp, h_col, h_val = (t.cpu().pin_memory() for t in (src.row_ptr, src.col, src.val))
        shard = n_vert // world
        h_X = X[rank * shard:(rank + 1) * shard].cpu().pin_memory() if world > 1 else X.cpu().pin_memory()
        h_C = torch.zeros((e_rows, N_DENSE), dtype=torch.float32).pin_memory()
    h2d = sum(t.numel() * t.element_size() for t in (h_rp, h_col, h_val, h_X))
    d2h = h_C.numel() * 4
    # workspace for the split rows of the end-to-end slice (an application knows its matrix: sized once)
    if src is mine:
        ws_e, ws_e_bytes = ws, ws_bytes
    else:
        ws_e_bytes = capi.spmm_workspace_bytes(capi.preprocess(src.row_ptr, e_nnz, 512, 32, 4).m1, N_DENSE, 4)
        ws_e = torch.empty(max(ws_e_bytes, 16), dtype=torch.uint8, device=dev)
    # Software pipeline over steps: two sets of device input buffers and two result buffers,
    # one copy-in stream, the compute streams, one copy-out stream.  Step i+1's H2D runs while
    # step i computes and step i's result goes back (PCIe is full duplex).
    s_in, s_out = torch.cuda.Stream(dev), torch.cuda.Stream(dev)
    bufs = []
    for _ in range(2):
        bufs.append({
            "rp": torch.empty_like(src.row_ptr), "col": torch.empty_like(src.col), "val": torch.empty_like(src.val),
            "X": (torch.empty((shard, N_DENSE), dtype=torch.float32, device=dev) if world > 1 else torch.empty_like(X)),
            "C": torch.empty((e_rows, N_DENSE), dtype=torch.float32, device=dev),
            "in_ready": torch.cuda.Event(), "in_free": torch.cuda.Event(), "out_ready": torch.cuda.Event(),
            "out_free": torch.cuda.Event(),
        })
    d_X_full = torch.empty_like(X) if world > 1 else None

    def copy_in(i):
        bf = bufs[i % 2]
        s_in.wait_event(bf["in_free"])          # the compute of step i-2 is done with this set
        with torch.cuda.stream(s_in):
            bf["rp"].copy_(h_rp, non_blocking=True)
            bf["col"].copy_(h_col, non_blocking=True)
            bf["val"].copy_(h_val, non_blocking=True)
            bf["X"].copy_(h_X, non_blocking=True)
            bf["in_ready"].record(s_in)

    def compute_and_copy_out(i):
        bf = bufs[i % 2]
        fj.cur.wait_event(bf["in_ready"])
        fj.cur.wait_event(bf["out_free"])       # the D2H of step i-2 is done with this C
        if world > 1:
            dist.all_gather_into_tensor(d_X_full, bf["X"])
        dense_x = d_X_full if world > 1 else bf["X"]
        m = capi.preprocess(bf["rp"], e_nnz, 512, 32, 4)    # device-side row decomposition (reads 2 counts back)
        # the matrix arrived with this step, so its popularity bitmap is built in this step too
        h = (capi.hot_columns(bf["col"], n_vert, 4 * N_DENSE, budget_bytes=int(args.hint_budget_mb * 1e6))
             if args.hints == "on" else None)
        bf["C"].zero_()                                       # the API's contract: C arrives zero-filled

        def launch(s1, s2):
            capi.spmm_raw(torch.float32, m.m1, m.m2, n_vert, N_DENSE, bf["val"].data_ptr(), bf["col"].data_ptr(),
                          bf["rp"].data_ptr(), m.block_r_ind.data_ptr(), m.residue_r_ind.data_ptr(),
                          m.st_off.data_ptr(), dense_x.data_ptr(), bf["C"].data_ptr(), ws_e.data_ptr(), ws_e_bytes,
                          s1, s2, hot=None if h is None else h.data_ptr())

        fj.run(launch)
        bf["in_free"].record(fj.cur)
        bf["out_ready"].record(fj.cur)
        s_out.wait_event(bf["out_ready"])
        with torch.cuda.stream(s_out):
            h_C.copy_(bf["C"], non_blocking=True)
            bf["out_free"].record(s_out)

    def e2e_run(steps):
        copy_in(0)
        for i in range(steps):
            if i + 1 < steps:
                copy_in(i + 1)
            compute_and_copy_out(i)
        fj.cur.wait_event(bufs[(steps - 1) % 2]["out_free"])   # the last result is on the host

    e2e_run(1)
    # each direction alone, all ranks at once (what the host's PCIe and memory give N concurrent copies)
    def alone(fn):
        barrier()
        a.record(fj.cur)
        with torch.cuda.stream(fj.cur):
            fn()
        b.record(fj.cur)
        barrier()
        return a.elapsed_time(b)

    def all_inputs():
        for name, h in (("rp", h_rp), ("col", h_col), ("val", h_val), ("X", h_X)):
            bufs[0][name].copy_(h, non_blocking=True)

    ms_h2d_alone = alone(all_inputs)
    ms_d2h_alone = alone(lambda: h_C.copy_(bufs[0]["C"], non_blocking=True))

    # both directions at once, on the two copy streams of the pipeline: what the host gives a
    # step whose copy-in overlaps the previous step's copy-out
    def both_directions():
        s_in.wait_stream(fj.cur)
        s_out.wait_stream(fj.cur)
        with torch.cuda.stream(s_in):
            for name, h in (("rp", h_rp), ("col", h_col), ("val", h_val), ("X", h_X)):
                bufs[1][name].copy_(h, non_blocking=True)
        with torch.cuda.stream(s_out):
            h_C.copy_(bufs[0]["C"], non_blocking=True)
        fj.cur.wait_stream(s_in)
        fj.cur.wait_stream(s_out)

    ms_duplex = alone(both_directions)
    barrier()
    a.record(fj.cur)
    e2e_run(args.e2e_steps)
    b.record(fj.cur)
    barrier()
    ms_e2e_mine = a.elapsed_time(b) / args.e2e_steps
    ms_e2e = max_over_ranks(ms_e2e_mine)
    # every rank's share, gathered on all ranks (rank 0 prints it)
    mine_row = torch.tensor([e_rows, e_nnz, h2d, d2h, ms_e2e_mine, ms_h2d_alone, ms_d2h_alone, ms_duplex],
                            dtype=torch.float64, device=dev)
    if world > 1:
        table = [torch.empty_like(mine_row) for _ in range(world)]
        dist.all_gather(table, mine_row)
    else:
        table = [mine_row]
    per_rank = [{"rank": i, "rows": int(t[0]), "nnz": int(t[1]), "h2d_bytes": int(t[2]), "d2h_bytes": int(t[3]),
                 "ms_per_step": float(t[4]), "h2d_alone_ms": float(t[5]), "h2d_alone_gbs": float(t[2] / t[5] / 1e6),
                 "d2h_alone_ms": float(t[6]), "d2h_alone_gbs": float(t[3] / t[6] / 1e6) if float(t[6]) > 0 else None,
                 "both_directions_ms": float(t[7]), "both_directions_gbs": float((t[2] + t[3]) / t[7] / 1e6)}
                for i, t in enumerate(table)]
    slowest = max(per_rank, key=lambda r: r["ms_per_step"])
    e2e = {"value": 2.0 * nnz * N_DENSE / ms_e2e / 1e6, "unit": "GFLOP/s", "ms_per_step": ms_e2e,
           "h2d_bytes_per_step": int(sum(r["h2d_bytes"] for r in per_rank)),
           "d2h_bytes_per_step": int(sum(r["d2h_bytes"] for r in per_rank)),
           "bytes_are": "sums over all ranks; per_rank has each rank's share",
           "steps": args.e2e_steps, "per_rank": per_rank,
           "host_buffers_numa_node": numa.node,
           "slowest_rank": {"rank": slowest["rank"],
                            "bound_by": ("h2d" if slowest["h2d_alone_ms"] >= slowest["d2h_alone_ms"] else "d2h"),
                            "copy_floor_ms": slowest["both_directions_ms"],
                            "note": "bound_by = the longer of the rank's two copy directions, each timed alone with "
                                    "all ranks copying at once; copy_floor_ms = one step's copy-in and copy-out "
                                    "issued together: a pipelined step cannot be shorter than that"},
           "partition": (f"contiguous rows, cost nnz + {args.e2e_row_weight}*rows (balances PCIe bytes per rank)"
                         if world > 1 else "one rank"),
           "includes": ("every step: H2D of the rank's CSR slice + dense operand from pinned memory, device "
                        "preprocessing, popularity pass, C zero-fill, SpMM, D2H of the rank's C rows; steps are "
                        "software-pipelined (step i+1's H2D overlaps step i's compute and D2H)" if world == 1 else
                        "every step, per rank: H2D of its CSR slice + 1/N of the dense operand from pinned memory, "
                        "NCCL all-gather of the operand, device preprocessing, popularity pass, C zero-fill, SpMM, "
                        "D2H of its C rows; steps are software-pipelined")}
    checksum = float(h_C.double().sum())

    # ---- CPU baseline (rank 0, single-GPU run only) ----------------------------------------------
    cpu_baseline = None
    configs = None
    if world == 1 and not args.no_extra:
        from oracle import cpu

        threads = cpu.max_threads()
        # all host threads: whole passes over the headline matrix for about 10 s
        rp_h, col_h, val_h, X_h = h_rp.numpy(), h_col.numpy(), h_val.numpy(), h_X.numpy()
        passes, t0 = 0, time.perf_counter()
        while passes < 40 and (passes == 0 or time.perf_counter() - t0 < 10.0):
            cpu.spmm_f32(rp_h, col_h, val_h, X_h, threads=threads)
            passes += 1
        dt = (time.perf_counter() - t0) / passes
        # one thread (how the reference's own CPU code runs): the first 2^18 rows, one pass
        rows_1 = min(e_rows, 1 << 18)
        nnz_1 = int(rp_h[rows_1])
        t1 = time.perf_counter()
        cpu.spmm_f32(rp_h[: rows_1 + 1], col_h[:nnz_1], val_h[:nnz_1], X_h, threads=1)
        dt1 = time.perf_counter() - t1
        cpu_baseline = {"value": 2.0 * e_nnz * N_DENSE / dt / 1e9, "unit": "GFLOP/s", "cores": threads, "kind": "port",
                        "sample": f"{passes} full passes over the headline matrix (nnz {e_nnz}), {dt:.3f} s per pass",
                        "single_thread_value": 2.0 * nnz_1 * N_DENSE / dt1 / 1e9,
                        "single_thread_sample": f"rows 0..{rows_1} (nnz {nnz_1}), one pass, {dt1:.2f} s",
                        "note": "the reference has no CPU SpMM; this is the oracle's CSR SpMM with OpenMP over rows"}
        del h_rp, h_col, h_val, h_X, h_C, bufs
        torch.cuda.empty_cache()
        configs = secondary_configs(peak_gbs, min(args.steps, 10), 3)

    if rank == 0:
        line = {
            "metric": METRIC, "value": gflops, "unit": "GFLOP/s", "n_gpus": world, "steps": args.steps,
            "warmup": warm, "ms_per_step": ms_step, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": f"rmat{args.scale}_spmm_n{N_DENSE}", "rows": n_vert, "nnz": nnz, "n": N_DENSE,
                       "partition": (f"nnz-balanced contiguous rows over {world} rank(s)" if not args.row_weight else
                                     f"contiguous rows over {world} rank(s), cost nnz + {args.row_weight}*rows"),
                       "rank0_rows": my_rows, "rank0_nnz": my_nnz,
                       "l2": "inputs larger than L2 (dense operand 4.3 GB, CSR 1 GB); no flush between steps",
                       "m1_rank0": meta.m1, "m2_rank0": meta.m2},
            "clocks": clocks, "timing": timing,
            "gpu_launches": launches_per_step * args.steps, "gpu_launches_note": "per repeat of the timed loop",
            "nnz_per_s": nnz / ms_step * 1e3,
            "roofline": roofline, "e2e": e2e, "sddmm": sddmm, "preprocess": preprocess_info, "hints": hints_info,
            "cpu_baseline": cpu_baseline,
            "broadcast_ms": broadcast_ms, "setup_s": setup_s, "checksum": checksum,
        }
        if configs is not None:
            line["configs"] = configs
        console.emit(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
