#!/usr/bin/env python
"""Benchmark of the compressed matrix-multiply path: t(y) %*% X on DDC column groups (rows/s).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--rows R]

One step = one left vector-matrix product over one resident batch of synthetic input: a
10,000,000 x 200 matrix of single-column DDC groups (256 N(0,1) dictionary values per column, uniform
ids, MapToByte) per GPU. With N > 1 every rank holds its own 10M-row shard of an (N * 10M)-row matrix
(weak scaling) and a step ends in an all-reduce of the 200 partial sums.

Prints one JSON line: value = rows/s with inputs resident in HBM, e2e = the same product through the
host-buffer C-ABI call (left vector copied host->device and result device->host inside the timed region),
roofline = HBM bytes of the dominant kernel against the measured copy bandwidth, cpu_baseline = the CPU
restatement of the reference algorithm on the host cores. `--impl reference` times that CPU path alone.
"""
from __future__ import annotations

import argparse
import ctypes as C
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

METRIC = "compressed t(y)%*%X rows/s"
UNIT = "rows/s"
N_COLS = 200
CPU_SAMPLE_ROWS = 2_000_000


def measured_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        with open(p) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.idx = gpu_index
        self.proc = None
        self.lines = []

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-i", str(self.idx), "-lms", "100"], stdout=subprocess.PIPE, text=True)
            self.t = threading.Thread(target=self._read, daemon=True)
            self.t.start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=2)
        except Exception:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        for ln in self.lines:
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                mx.append(float(f[2]))
            except ValueError:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def cpu_reference_rate(rows: int, steps: int, warmup: int):
    """The CPU restatement of the reference's LMM (CLALibLeftMultBy) on a bounded sample, all host threads."""
    from oracle import oracle as o
    from systemds_b200 import datagen
    o.build()
    cmb, y = datagen.config2(nRows=rows, nCols=N_COLS)
    # every host thread this process may run on, named explicitly: torchrun exports OMP_NUM_THREADS=1 to its
    # ranks, which would otherwise shrink the OpenMP default and with it the baseline
    om = o.OracleMatrix(cmb, threads=len(os.sched_getaffinity(0)))
    for _ in range(warmup):
        om.lmm(y)
    ts = []
    for _ in range(steps):
        t0 = time.perf_counter()
        om.lmm(y)
        ts.append(time.perf_counter() - t0)
    return rows / float(np.mean(ts)), float(np.mean(ts)) * 1e3, om.k


def run_reference(args, rank):
    if rank != 0:
        return
    rate, ms, cores = cpu_reference_rate(CPU_SAMPLE_ROWS, args.steps, args.warmup)
    sample = f"{CPU_SAMPLE_ROWS} x {N_COLS} rows of the same workload per step"
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": rate, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f64", "data": "synthetic",
        "config": {"workload": "configs[1]: t(y)%*%X, X 10,000,000 x 200 DDC (256 values/column, MapToByte), y N(0,1)",
                   "note": "CPU restatement of the reference's CLALibLeftMultBy (no JVM on this box); OpenMP over the "
                           "reference's task split"},
        "cpu_baseline": {"value": rate, "unit": UNIT, "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": rate, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--rows", type=int, default=10_000_000, help="rows per GPU (default: the benchmark configuration)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-also", action="store_true", help="skip the secondary X%%*%%v measurement")
    ap.add_argument("--extras", action="store_true",
                    help="also time scaled-down versions of the other benchmark configurations (mixed-group X%%*%%V, "
                         "t(X)%%*%%X, the lmCG step); adds about a minute of host-side data generation")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if args.impl == "reference":
        run_reference(args, rank)
        return

    import torch
    import torch.distributed as dist
    from systemds_b200 import datagen, native
    from systemds_b200.native import check

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the compressed products have no CPU path")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    L = native.lib()

    # ---- workload: this rank's shard ----------------------------------------------------------------
    n = args.rows
    shard_rows = ((n + datagen.BLOCK - 1) // datagen.BLOCK) * datagen.BLOCK  # shards start on generator blocks
    cmb, y_host = datagen.config2(nRows=n, nCols=N_COLS, row0=rank * shard_rows)
    cmb.to_device(local_rank)
    h = cmb.handle()
    check(L.cla_set_profile(h, 1))
    index_bytes = cmb.index_bytes()
    y_pin = torch.from_numpy(y_host.reshape(-1)).pin_memory()
    y_dev = y_pin.to(dev, non_blocking=True)
    out_dev = torch.zeros(N_COLS, dtype=torch.float64, device=dev)
    out_pin = torch.zeros(N_COLS, dtype=torch.float64).pin_memory()
    stream = torch.cuda.current_stream()
    sptr = C.c_void_p(stream.cuda_stream)
    torch.cuda.synchronize()

    def step():
        check(L.cla_lmm_dev(h, C.c_void_p(y_dev.data_ptr()), 1, C.c_void_p(out_dev.data_ptr()), sptr))
        if world > 1:
            dist.all_reduce(out_dev)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(args.warmup):
        step()
    barrier()
    st0 = cmb.stats()
    sampler = ClockSampler(local_rank)
    sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    e0.record()
    for _ in range(args.steps):
        step()
    e1.record()
    barrier()
    ms_total = e0.elapsed_time(e1)
    st1 = cmb.stats()

    # ---- e2e: host buffers through the plugin-facing call ---------------------------------------------
    y_np = y_pin.numpy()
    out_np = out_pin.numpy()
    for _ in range(2):
        check(L.cla_lmm(h, C.c_void_p(y_np.ctypes.data), 1, C.c_void_p(out_np.ctypes.data)))
    barrier()
    t0 = time.perf_counter()
    e2e_steps = max(3, min(args.steps, 10))
    for _ in range(e2e_steps):
        check(L.cla_lmm(h, C.c_void_p(y_np.ctypes.data), 1, C.c_void_p(out_np.ctypes.data)))
        if world > 1:
            t = torch.from_numpy(out_np).to(dev)
            dist.all_reduce(t)
            out_np[:] = t.cpu().numpy()
    barrier()
    e2e_ms = (time.perf_counter() - t0) * 1e3 / e2e_steps
    clocks = sampler.stop()

    times = torch.tensor([ms_total, e2e_ms], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
    ms_total, e2e_ms = float(times[0]), float(times[1])
    ms_step = ms_total / args.steps
    total_rows = n * world
    value = total_rows / (ms_step * 1e-3)

    # ---- roofline of the dominant kernel (this rank) ---------------------------------------------------
    peak, peak_kind = measured_peaks()
    k_ms = (st1["main_kernel_ms"] - st0["main_kernel_ms"]) / max(1, st1["main_kernel_count"] - st0["main_kernel_count"])
    alg_bytes = index_bytes + n * 8 + N_COLS * 8  # maps + dictionaries, left vector, result
    achieved = alg_bytes / (k_ms * 1e-3) / 1e9 if k_ms > 0 else None
    roofline = {"bound": "hbm", "kernel": "k_lmm_vec_u8", "achieved": achieved, "peak": peak, "unit": "GB/s",
                "frac": (achieved / peak) if achieved else None, "peak_source": f"of {peak_kind}",
                "kernel_ms": k_ms, "algorithmic_bytes": alg_bytes,
                # dram__bytes_read.sum + dram__bytes_write.sum of one launch, from the ncu capture of a 2,000,000-row
                # case scaled by rows (traffic grows in proportion to rows); see profiles/k_lmm_vec_u8_config2.md
                "traffic": 485.1e6 * (n / 2_000_000.0)}

    result = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f64",
        "data": "synthetic",
        "config": {"workload": "configs[1]: t(y)%*%X, X 10,000,000 x 200 per GPU, single-column DDC, 256 N(0,1) values "
                               "per column, uniform ids, MapToByte; y N(0,1)",
                   "rows_per_gpu": n, "cols": N_COLS, "parallelism": f"row-sharded x{world}" if world > 1 else "single GPU",
                   "l2": "inputs (2.08 GB per step) larger than L2; no flush needed"},
        "roofline": roofline,
        "e2e": {"value": total_rows / (e2e_ms * 1e-3), "unit": UNIT, "h2d_bytes_per_step": n * 8,
                "d2h_bytes_per_step": N_COLS * 8 + 8, "ms_per_step": e2e_ms, "steps": e2e_steps,
                "timer": "host wall clock around the synchronous C-ABI call (pinned buffers)"},
        "gpu_launches": int(st1["kernel_launches"] - st0["kernel_launches"]),
        "clocks": clocks,
    }

    # ---- secondary: X %*% v on configs[0] (1,000,000 x 100, 16 values/column), L2 flushed between iterations ----
    if rank == 0 and not args.no_also:
        result["also"] = {"rmm_config0": bench_rmm_config0(L, dev, sptr, peak)}
    if rank == 0 and args.extras:
        result["also"] = dict(result.get("also", {}), **bench_extras(L, dev, sptr, peak))
    # ---- CPU baseline (rank 0 only) ----
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        rate, ms, cores = cpu_reference_rate(CPU_SAMPLE_ROWS, 3, 1)
        result["cpu_baseline"] = {"value": rate, "unit": UNIT, "cores": cores, "kind": "port",
                                  "sample": f"{CPU_SAMPLE_ROWS} x {N_COLS} rows of the same workload, mean of 3 runs "
                                            f"({ms:.0f} ms each)"}
    if rank == 0:
        print(json.dumps(result))
    cmb.free()
    if world > 1:
        dist.destroy_process_group()


def bench_rmm_config0(L, dev, sptr, peak):
    """X %*% v, 1,000,000 x 100 single-column DDC with 16 values per column (MapToUByte)."""
    import torch
    from systemds_b200 import datagen
    from systemds_b200.native import check
    cmb, v = datagen.config1()
    cmb.to_device(dev.index)
    h = cmb.handle()
    check(L.cla_set_profile(h, 1))
    v_dev = torch.from_numpy(v.reshape(-1)).to(dev)
    out = torch.zeros(cmb.rlen, dtype=torch.float64, device=dev)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    for _ in range(3):
        check(L.cla_rmm_dev(h, C.c_void_p(v_dev.data_ptr()), 100, 1, C.c_void_p(out.data_ptr()), sptr))
    torch.cuda.synchronize()
    st0 = cmb.stats()
    iters = 20
    for _ in range(iters):
        flush.fill_(1)  # evict the 100 MB of maps from L2
        check(L.cla_rmm_dev(h, C.c_void_p(v_dev.data_ptr()), 100, 1, C.c_void_p(out.data_ptr()), sptr))
    torch.cuda.synchronize()
    st1 = cmb.stats()
    k_ms = (st1["main_kernel_ms"] - st0["main_kernel_ms"]) / max(1, st1["main_kernel_count"] - st0["main_kernel_count"])
    alg = cmb.index_bytes() + cmb.rlen * 8 + 100 * 8
    ach = alg / (k_ms * 1e-3) / 1e9
    res = {"metric": "compressed X%*%v rows/s", "value": cmb.rlen / (k_ms * 1e-3), "unit": "rows/s", "kernel_ms": k_ms,
           "roofline": {"bound": "hbm", "kernel": "k_rmm_vec_u8", "achieved": ach, "peak": peak, "unit": "GB/s",
                        "frac": ach / peak, "algorithmic_bytes": alg},
           "l2": "256 MB buffer written between iterations (inputs are 100 MB, below L2)"}
    cmb.free()
    return res


def _time_dev(fn, iters=5):
    import torch
    fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / iters


def bench_extras(L, dev, sptr, peak):
    """Scaled-down versions of configs[2..4] (same shapes per row, fewer rows), device-resident operands."""
    import torch
    from systemds_b200 import datagen
    from systemds_b200.native import check
    P = lambda t: C.c_void_p(t.data_ptr())  # noqa: E731
    out = {}
    dm, df = C.c_double(0), C.c_double(0)
    check(L.cla_measure_fp64_peaks(dev.index, C.byref(dm), C.byref(df)))
    out["fp64_peaks_measured"] = {"dmma_m8n8k4_TFLOPs": dm.value, "dfma_TFLOPs": df.value,
                                  "how": "back-to-back independent instructions, 4 CTAs of 256 threads per SM, CUDA events"}
    # configs[0] with ten times the rows: the steady state of the X %*% v kernel (configs[0] itself is 17 us of HBM time)
    n = 10_000_000
    cmb, v = datagen.config1(nRows=n)
    cmb.to_device(dev.index)
    h = cmb.handle()
    vd = torch.from_numpy(v.reshape(-1)).to(dev)
    od = torch.empty(n, dtype=torch.float64, device=dev)
    ms = _time_dev(lambda: check(L.cla_rmm_dev(h, P(vd), 100, 1, P(od), sptr)))
    alg0 = cmb.index_bytes() + n * 8
    out["rmm_config0_x10"] = {"workload": f"configs[0] shape at {n} rows (100 DDC columns, 16 values, MapToUByte)", "ms": ms,
                              "rows_per_s": n / (ms * 1e-3), "algorithmic_GBps": alg0 / (ms * 1e-3) / 1e9,
                              "hbm_frac": alg0 / (ms * 1e-3) / 1e9 / peak}
    cmb.free()
    del vd, od
    # configs[2]: mixed groups, X %*% V with 64 columns
    n = 1_000_000
    cmb, V = datagen.config3(nRows=n)
    cmb.to_device(dev.index)
    h = cmb.handle()
    Vd = torch.from_numpy(V).to(dev)
    Od = torch.empty((n, 64), dtype=torch.float64, device=dev)
    ms = _time_dev(lambda: check(L.cla_rmm_dev(h, P(Vd), 500, 64, P(Od), sptr)))
    alg = cmb.index_bytes() + n * 64 * 8 + V.nbytes
    out["rmm_mixed_config2"] = {"workload": f"configs[2] at {n} rows: 500 columns (40% DDC, 30% SDCZeros, 20% RLE, 10% dense), V 500x64",
                                "ms": ms, "rows_per_s": n / (ms * 1e-3), "algorithmic_GBps": alg / (ms * 1e-3) / 1e9,
                                "hbm_frac": alg / (ms * 1e-3) / 1e9 / peak}
    yd = torch.randn(n, dtype=torch.float64, device=dev)
    od = torch.empty(500, dtype=torch.float64, device=dev)
    ms = _time_dev(lambda: check(L.cla_lmm_dev(h, P(yd), 1, P(od), sptr)))
    algl = cmb.index_bytes() + n * 8
    out["lmm_mixed_config2"] = {"workload": "t(y) %*% X on the same matrix", "ms": ms, "rows_per_s": n / (ms * 1e-3),
                                "algorithmic_GBps": algl / (ms * 1e-3) / 1e9, "hbm_frac": algl / (ms * 1e-3) / 1e9 / peak}
    del Vd, Od
    Dd = torch.empty((n, 500), dtype=torch.float64, device=dev)
    ms = _time_dev(lambda: check(L.cla_decompress_dev(h, P(Dd), sptr)))
    algd = cmb.index_bytes() + n * 500 * 8
    out["decompress_mixed_config2"] = {"workload": "decompress of the same matrix into a device buffer (4 GB)", "ms": ms,
                                       "rows_per_s": n / (ms * 1e-3), "algorithmic_GBps": algd / (ms * 1e-3) / 1e9,
                                       "hbm_frac": algd / (ms * 1e-3) / 1e9 / peak}
    cmb.free()
    del Dd
    # configs[3]: t(X) %*% X, 100 DDC columns with 1000 values (MapToChar), Zipf ids
    n = 2_000_000
    cmb = datagen.config4(nRows=n)
    cmb.to_device(dev.index)
    h = cmb.handle()
    Cd = torch.empty((100, 100), dtype=torch.float64, device=dev)
    ms = _time_dev(lambda: check(L.cla_tsmm_dev(h, P(Cd), sptr)))
    flops = 2.0 * n * 100 * 101 / 2
    out["tsmm_config3"] = {"workload": f"configs[3] at {n} rows: 100 DDC columns, 1000 values, MapToChar, Zipf(1.1)",
                           "ms": ms, "rows_per_s": n / (ms * 1e-3), "algorithmic_TFLOPs": flops / (ms * 1e-3) / 1e12,
                           "dmma_peak_TFLOPs": dm.value, "dmma_frac": flops / (ms * 1e-3) / 1e12 / dm.value,
                           "note": "peak = measured back-to-back DMMA rate (fp64_peaks_measured)"}
    cmb.free()
    # configs[4]: lmCG step w = t(X) (X v) + 1e-3 v on one shard
    n = 2_000_000
    cmb, v = datagen.config5(nRows=n)
    cmb.to_device(dev.index)
    h = cmb.handle()
    vd = torch.from_numpy(v.reshape(-1)).to(dev)
    wd = torch.empty(1000, dtype=torch.float64, device=dev)
    ud = torch.empty(n, dtype=torch.float64, device=dev)

    def step():
        check(L.cla_mmchain_dev(h, P(vd), None, 0, P(wd), P(ud), sptr))
        wd.add_(vd, alpha=1e-3)

    ms = _time_dev(step)
    alg5 = 2 * cmb.index_bytes() + 2 * n * 8
    out["lmcg_step_config4"] = {"workload": f"configs[4] shard at {n} rows x 1000 columns (cardinality 2..255): w = t(X)(Xv) + 1e-3 v",
                                "ms": ms, "rows_per_s": n / (ms * 1e-3), "algorithmic_GBps": alg5 / (ms * 1e-3) / 1e9,
                                "hbm_frac": alg5 / (ms * 1e-3) / 1e9 / peak}
    cmb.free()
    return out


if __name__ == "__main__":
    main()
