#!/usr/bin/env python
"""Benchmark of the compressed matrix-multiply path on the five benchmark workloads.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload 0..4] [--rows R]

The headline line (and the default, --workload 1) is t(y) %*% X on a 10,000,000 x 200 matrix of single-column DDC
groups (256 N(0,1) dictionary values per column, uniform ids, MapToByte) per GPU. One step = one product over one
resident batch of synthetic input. With N > 1 every rank holds its own shard (weak scaling: N x the rows) and a step
ends in the all-reduce the product needs (none for X %*% V, whose result stays row-partitioned).

Workloads (--workload; the other four are timed as well and reported under "also", at every N):
  0  X %*% v         1,000,000 x 100   DDC, 16 values, MapToUByte
  1  t(y) %*% X      10,000,000 x 200  DDC, 256 values, MapToByte                         (all-reduce of 200 doubles)
  2  X %*% V         10,000,000 x 500  40% DDC(4) / 30% SDCZeros / 20% RLE / 10% dense; V 500 x 64
  3  t(X) %*% X      20,000,000 x 100  DDC, 1000 values, MapToChar, Zipf(1.1) ids          (all-reduce of 100 x 100)
  4  lmCG step       12,500,000 x 1000 per GPU (100M rows on 8 GPUs): w = t(X)(X v) + 1e-3 v, DDC, cardinality 2..255
                                                                                           (all-reduce of 1000 doubles)

Prints one JSON line: value = rows/s with inputs resident in HBM (max over ranks of the CUDA-event time of K steps),
e2e = the same product through the host-buffer C-ABI call (operands copied host->device and the result
device->host inside the timed region), roofline = algorithmic bytes (or flops) of the dominant kernel over its
CUDA-event duration against the measured peak, cpu_baseline = the CPU restatement of the reference algorithm on the
host cores. `--impl reference` times that CPU path alone. `--decompress` adds the time of cla_decompress_dev of the
main workload's matrix into a device buffer (bytes written per second against the copy bandwidth). With N > 1 the sums
over the ranks run through the library's kernel over peer memory (`--allreduce nccl` switches to NCCL); `--strong` splits
the workload's rows over the N GPUs instead of giving each GPU all of them.
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

UNIT = "rows/s"
DEFAULT_ROWS = {0: 1_000_000, 1: 10_000_000, 2: 10_000_000, 3: 20_000_000, 4: 12_500_000}
CPU_ROWS = {0: 1_000_000, 1: 10_000_000, 2: 500_000, 3: 200_000, 4: 500_000}  # bounded CPU samples (1: the full workload)
METRICS = {0: "compressed X%*%v rows/s", 1: "compressed t(y)%*%X rows/s", 2: "compressed X%*%V (64 columns) rows/s",
           3: "compressed t(X)%*%X rows/s", 4: "compressed lmCG step t(X)%*%(X%*%v)+1e-3*v rows/s"}
DESCS = {
    0: "configs[0]: X%*%v, X 1,000,000 x 100 per GPU, single-column DDC, 16 N(0,1) values per column, uniform ids, "
       "MapToUByte; v N(0,1)",
    1: "configs[1]: t(y)%*%X, X 10,000,000 x 200 per GPU, single-column DDC, 256 N(0,1) values per column, uniform ids, "
       "MapToByte; y N(0,1)",
    2: "configs[2]: X%*%V, X 10,000,000 x 500 per GPU: 200 DDC columns (4 values), 150 SDCZeros columns (5% listed rows, "
       "8 values), 100 RLE columns (32 values, geometric runs of mean 1000), one dense 50-column group; V 500 x 64 N(0,1)",
    3: "configs[3]: t(X)%*%X, X 20,000,000 x 100 per GPU, single-column DDC, 1000 U(-1,1) values, MapToChar, Zipf(1.1) ids",
    4: "configs[4]: lmCG inner step w = t(X)%*%(X%*%v) + 1e-3*v, X 12,500,000 x 1000 per GPU (100,000,000 rows on 8 GPUs), "
       "single-column DDC, cardinality uniform in [2, 255] (MapToBit / MapToUByte / MapToByte), N(0,1) values, uniform ids",
}
# dram__bytes_read.sum + dram__bytes_write.sum of one launch of the dominant kernel, per matrix row, from ncu captures of
# scaled-down cases (traffic grows in proportion to the rows); None = not captured
TRAFFIC_PER_ROW = {0: 134.6, 1: 223.45, 2: 1846.0, 3: 202.95, 4: 2170.5}


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
                                          "-i", str(self.idx), "-lms", "50"], stdout=subprocess.PIPE, text=True)
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


# ---- CPU arm: the restatement of the reference algorithm ------------------------------------------------
def cpu_reference_rate(workload: int, rows: int, steps: int, warmup: int):
    """The CPU restatement of the reference's product for `workload` on `rows` rows, all host threads.
    Returns (rows/s, ms per step, threads)."""
    from oracle import oracle as o
    from systemds_b200 import datagen
    o.build()
    # every host thread this process may run on, named explicitly: torchrun exports OMP_NUM_THREADS=1 to its
    # ranks, which would otherwise shrink the OpenMP default and with it the baseline
    threads = len(os.sched_getaffinity(0))
    if workload == 0:
        cmb, v = datagen.config1(nRows=rows)
        om = o.OracleMatrix(cmb, threads=threads)
        fn = lambda: om.rmm(v)  # noqa: E731
    elif workload == 1:
        cmb, y = datagen.config2(nRows=rows, nCols=200)
        om = o.OracleMatrix(cmb, threads=threads)
        fn = lambda: om.lmm(y)  # noqa: E731
    elif workload == 2:
        cmb, V = datagen.config3(nRows=rows)
        om = o.OracleMatrix(cmb, threads=threads)
        fn = lambda: om.rmm(V)  # noqa: E731
    elif workload == 3:
        cmb = datagen.config4(nRows=rows)
        om = o.OracleMatrix(cmb, threads=threads)
        fn = lambda: om.tsmm()  # noqa: E731
    else:
        cmb, v = datagen.config5(nRows=rows)
        om = o.OracleMatrix(cmb, threads=threads)
        fn = lambda: om.mmchain(v) + 1e-3 * v.reshape(-1, 1)  # noqa: E731
    for _ in range(warmup):
        fn()
    ts = []
    for _ in range(steps):
        t0 = time.perf_counter()
        fn()
        ts.append(time.perf_counter() - t0)
    return rows / float(np.mean(ts)), float(np.mean(ts)) * 1e3, om.k


def run_reference(args, rank):
    if rank != 0:
        return
    w = args.workload
    rows = CPU_ROWS[w] if args.rows is None else min(args.rows, CPU_ROWS[w])
    rate, ms, cores = cpu_reference_rate(w, rows, args.steps, args.warmup)
    full = rows == DEFAULT_ROWS[w]
    sample = (f"the full workload ({rows} rows) per step" if full else
              f"{rows} rows of the same workload per step (rows/s does not depend on the row count)")
    print(json.dumps({
        "impl": "reference", "metric": METRICS[w], "value": rate, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f64", "data": "synthetic",
        "config": {"workload": DESCS[w], "rows_per_step": rows,
                   "note": "CPU restatement of the reference's CLALib* algorithm (no JVM on this box); OpenMP over the "
                           "reference's task split"},
        "cpu_baseline": {"value": rate, "unit": UNIT, "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": rate, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


# ---- host placement -------------------------------------------------------------------------------------
def bind_to_gpu_numa_node(local_rank: int):
    """Pins this process to the CPUs of the NUMA node its GPU hangs off, so that the pinned host buffers (first
    touched here) and the copy-issuing thread are local to the GPU's PCIe root. Returns (node, previous affinity)
    or (None, previous affinity) when the topology cannot be read."""
    prev = os.sched_getaffinity(0)
    try:
        import torch
        p = torch.cuda.get_device_properties(local_rank)
        bdf = f"{p.pci_domain_id:04x}:{p.pci_bus_id:02x}:{p.pci_device_id:02x}.0"
        with open(f"/sys/bus/pci/devices/{bdf}/numa_node") as f:
            node = int(f.read().strip())
        if node < 0:
            return None, prev
        with open(f"/sys/devices/system/node/node{node}/cpulist") as f:
            cpus = set()
            for part in f.read().strip().split(","):
                a, _, b = part.partition("-")
                cpus.update(range(int(a), int(b or a) + 1))
        cpus &= prev
        if cpus:
            os.sched_setaffinity(0, cpus)
            return node, prev
    except Exception:
        pass
    return None, prev


# ---- the workloads on the device --------------------------------------------------------------------------
class Workload:
    """One benchmark workload on this rank's GPU: build() generates the shard and uploads it, step() enqueues one
    product (and its all-reduce) on the current stream, e2e_step() runs it through the host-buffer call."""

    def __init__(self, idx, rows, rank, local_rank, world, dev, L, host_gen=False):
        self.idx, self.n, self.rank, self.local_rank, self.world, self.dev, self.L = idx, rows, rank, local_rank, world, dev, L
        self.host_gen = host_gen
        self.cmb = None

    def P(self, t):
        return C.c_void_p(t.data_ptr())

    comm = None          # shared by all workloads of this process (one buffer of 10,000 doubles per rank)
    comm_note = "nccl"

    @classmethod
    def setup_allreduce(cls, rank, local_rank, world, dev, kind):
        """The exchange that ends a step on N > 1 GPUs: the library's kernel over peer memory (checked once against
        NCCL on a random vector), or NCCL when that is asked for or the peer setup fails."""
        import torch
        import torch.distributed as dist
        if world == 1 or kind == "nccl":
            return
        from systemds_b200.comm import HANDLE_BYTES, PeerAllReduce, torch_exchange

        def all_ok(flag):  # every stage is agreed on by all ranks, so no rank waits in a collective the others skipped
            f = torch.tensor([int(flag)], device=dev)
            dist.all_reduce(f, op=dist.ReduceOp.MIN)
            return int(f[0]) == 1

        c, err = None, None
        try:
            c = PeerAllReduce(rank, world, local_rank, 10000, connect=False)
        except Exception as e:  # noqa: BLE001
            err = e
        handles = torch_exchange(dev)(c.handle_bytes if c is not None else bytes(HANDLE_BYTES))
        stage = all_ok(c is not None)
        if stage:
            try:
                c.connect(handles=handles)
            except Exception as e:  # noqa: BLE001
                err = e
            stage = all_ok(err is None)
        ok = 0
        if stage:
            g = torch.Generator(device=dev)
            g.manual_seed(1234 + rank)
            x = torch.randn(10000, dtype=torch.float64, device=dev, generator=g)
            y = x.clone()
            dist.all_reduce(y)
            try:
                c(x.data_ptr(), 10000, torch.cuda.current_stream().cuda_stream)
                c.status()
                ok = int(bool(((x - y).abs() <= 1e-12 * (x.abs() + y.abs()) + 1e-15).all()))
            except Exception as e:  # noqa: BLE001
                err = e
        if err is not None:
            cls.comm_note = f"nccl (peer setup failed: {type(err).__name__}: {str(err)[:80]})"
        cls.comm = c
        t = torch.tensor([ok], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MIN)
        if int(t[0]) == 1:
            cls.comm_note = "cla_allreduce_dev: one kernel per rank over NVLink peer memory (stores + flags, rank-ordered sum)"
        else:
            if cls.comm is not None:
                cls.comm.close()
            cls.comm = None
            if cls.comm_note == "nccl":
                cls.comm_note = "nccl (peer result did not match)"

    def allreduce(self, t):
        import torch.distributed as dist
        if Workload.comm is not None:
            Workload.comm(t.data_ptr(), t.numel(), self.sptr.value or 0)
        else:
            dist.all_reduce(t)

    def build(self):
        import torch
        from systemds_b200 import datagen, datagen_dev
        from systemds_b200.native import check
        n, dev, i = self.n, self.dev, self.idx
        row0 = self.rank * (((n + datagen.BLOCK - 1) // datagen.BLOCK) * datagen.BLOCK)  # shards start on generator blocks
        stream = torch.cuda.current_stream()
        self.sptr = C.c_void_p(stream.cuda_stream)
        f64 = torch.float64
        if i == 0:
            self.cmb, v = datagen_dev.config1(nRows=n, row0=row0, device=self.local_rank)
            self.v_host = np.ascontiguousarray(v.reshape(-1))
            self.v = torch.from_numpy(self.v_host).to(dev)
            self.out = torch.zeros(n, dtype=f64, device=dev)
        elif i == 1:
            if self.host_gen:  # the same arrays the CPU oracle can read
                self.cmb, y = datagen.config2(nRows=n, nCols=200, row0=row0)
                self.y_pin = torch.from_numpy(y.reshape(-1)).pin_memory()
                self.y = self.y_pin.to(dev, non_blocking=True)
            else:
                self.cmb, self.y = datagen_dev.config2(nRows=n, row0=row0, device=self.local_rank)
                self.y_pin = None
            self.out = torch.zeros(200, dtype=f64, device=dev)
        elif i == 2:
            self.cmb, V = datagen_dev.config3(nRows=n, row0=row0, device=self.local_rank)
            self.V_host = np.ascontiguousarray(V)
            self.V = torch.from_numpy(self.V_host).to(dev)
            self.out = torch.empty((n, 64), dtype=f64, device=dev)
        elif i == 3:
            self.cmb = datagen_dev.config4(nRows=n, row0=row0, device=self.local_rank)
            self.out = torch.zeros((100, 100), dtype=f64, device=dev)
        else:
            self.cmb, v = datagen_dev.config5(nRows=n, row0=row0, device=self.local_rank)
            self.v_host = np.ascontiguousarray(v.reshape(-1))
            self.v = torch.from_numpy(self.v_host).to(dev)
            self.out = torch.zeros(1000, dtype=f64, device=dev)
            self.u = torch.empty(n, dtype=f64, device=dev)
        torch.cuda.synchronize()
        self.cmb.to_device(self.local_rank)
        datagen_dev.release_sources(self.cmb)
        torch.cuda.empty_cache()
        self.h = self.cmb.handle()
        check(self.L.cla_set_profile(self.h, 1))
        self.index_bytes = self.cmb.index_bytes()
        torch.cuda.synchronize()
        return self

    # one product with device-resident operands, on the current stream
    def step(self):
        from systemds_b200.native import check
        L, h, P, s = self.L, self.h, self.P, self.sptr
        if self.idx == 0:
            check(L.cla_rmm_dev(h, P(self.v), 100, 1, P(self.out), s))
        elif self.idx == 1:
            check(L.cla_lmm_dev(h, P(self.y), 1, P(self.out), s))
            if self.world > 1:
                self.allreduce(self.out)
        elif self.idx == 2:
            check(L.cla_rmm_dev(h, P(self.V), 500, 64, P(self.out), s))
        elif self.idx == 3:
            check(L.cla_tsmm_dev(h, P(self.out), s))
            if self.world > 1:
                self.allreduce(self.out)
        else:
            check(L.cla_mmchain_dev(h, P(self.v), None, 0, P(self.out), P(self.u), s))
            if self.world > 1:
                self.allreduce(self.out)
            self.out.add_(self.v, alpha=1e-3)  # after the reduce, once (scripts/builtin/lmCG.dml: q = t(X) %*% (X %*% p) + lambda * p)

    @property
    def needs_l2_flush(self):
        return self.idx == 0 and self.index_bytes < (126 << 20)

    def algorithmic(self, dmma_peak):
        """(bound, work per launch, unit scale, peak, unit, kernel): bytes for the HBM-bound products, flops for TSMM."""
        n, ib = self.n, self.index_bytes
        if self.idx == 0:
            return "hbm", ib + n * 8 + 100 * 8, "k_rmm_vec_f"
        if self.idx == 1:
            return "hbm", ib + n * 8 + 200 * 8, "k_lmm_vec_u8"
        if self.idx == 2:
            return "hbm", ib + n * 64 * 8 + 500 * 64 * 8, "k_rmm_dmma3"
        if self.idx == 3:
            return "tensor", 2.0 * n * 100 * 101 / 2, "k_tsmm_tri16"
        return "hbm", 2 * ib + 2 * n * 8 + 2 * 1000 * 8, "k_rmm_vec_b + k_lmm_vec_u8"

    # the same product through the host-buffer call (pinned operands prepared by e2e_prepare)
    def e2e_prepare(self, pinned=True):
        import torch
        mk = (lambda a: torch.from_numpy(a).pin_memory().numpy()) if pinned else (lambda a: a.copy())
        n = self.n
        if self.idx == 0:
            self.e_in, self.e_out = mk(self.v_host), mk(np.zeros(n))
            self.h2d, self.d2h = 100 * 8, n * 8 + 8
        elif self.idx == 1:
            yh = self.y_pin.numpy() if (pinned and self.y_pin is not None) else mk(self.y.cpu().numpy())
            self.e_in, self.e_out = yh, mk(np.zeros(200))
            self.h2d, self.d2h = n * 8, 200 * 8 + 8
        elif self.idx == 2:
            self.e_in, self.e_out = mk(self.V_host), mk(np.zeros((n, 64)))
            self.h2d, self.d2h = 500 * 64 * 8, n * 64 * 8 + 8
        elif self.idx == 3:
            self.e_in, self.e_out = None, mk(np.zeros((100, 100)))
            self.h2d, self.d2h = 0, 100 * 100 * 8 + 8
        else:
            self.e_in, self.e_out = mk(self.v_host), mk(np.zeros(1000))
            self.h2d, self.d2h = 1000 * 8, 1000 * 8 + 8

    def e2e_step(self):
        import torch
        import torch.distributed as dist
        from systemds_b200.native import check
        L, h = self.L, self.h
        a = lambda x: C.c_void_p(x.ctypes.data)  # noqa: E731
        if self.idx == 0:
            check(L.cla_rmm(h, a(self.e_in), 100, 1, a(self.e_out)))
        elif self.idx == 1:
            check(L.cla_lmm(h, a(self.e_in), 1, a(self.e_out)))
        elif self.idx == 2:
            check(L.cla_rmm(h, a(self.e_in), 500, 64, a(self.e_out)))
        elif self.idx == 3:
            check(L.cla_tsmm(h, a(self.e_out)))
        else:
            check(L.cla_mmchain(h, a(self.e_in), None, 0, a(self.e_out)))
        if self.world > 1 and self.idx in (1, 3, 4):  # the partial results of the shards add up
            t = torch.from_numpy(self.e_out).to(self.dev)
            self.allreduce(t)
            self.e_out[...] = t.cpu().numpy()
        if self.idx == 4:
            self.e_out += 1e-3 * self.e_in

    def free(self):
        import torch
        if self.cmb is not None:
            self.cmb.free()
        for k in ("cmb", "v", "y", "y_pin", "V", "out", "u", "e_in", "e_out"):
            self.__dict__.pop(k, None)
        self.cmb = None
        torch.cuda.empty_cache()


def barrier(world):
    import torch
    import torch.distributed as dist
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()


def time_steps(wl: Workload, steps: int, warmup: int, world: int):
    """CUDA-event time of `steps` steps after `warmup`, max over ranks; plus the library's own event time of the
    dominant kernel(s) per step and the launch count. Workloads smaller than L2 get a 256 MB write between steps
    and are timed step by step (the flush is outside the timed events)."""
    import torch
    import torch.distributed as dist
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=wl.dev) if wl.needs_l2_flush else None
    for _ in range(warmup):
        wl.step()
    barrier(world)
    st0 = wl.cmb.stats()
    if flush is None:
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier(world)
        e0.record()
        for _ in range(steps):
            wl.step()
        e1.record()
        barrier(world)
        ms_total = e0.elapsed_time(e1)
    else:
        ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(steps)]
        barrier(world)
        for a, b in ev:
            flush.fill_(1)
            a.record()
            wl.step()
            b.record()
        barrier(world)
        ms_total = sum(a.elapsed_time(b) for a, b in ev)
    st1 = wl.cmb.stats()
    t = torch.tensor([ms_total], dtype=torch.float64, device=wl.dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    k_ms = (st1["main_kernel_ms"] - st0["main_kernel_ms"]) / steps
    launches = int(st1["kernel_launches"] - st0["kernel_launches"])
    if Workload.comm is not None and wl.idx in (1, 3, 4):
        launches += steps  # k_peer_allreduce, once per step
    return float(t[0]) / steps, k_ms, launches


def roofline_of(wl: Workload, k_ms: float, hbm_peak: float, peak_kind: str, dmma_peak: float):
    bound, work, kernel = wl.algorithmic(dmma_peak)
    if k_ms <= 0:
        return {"bound": bound, "kernel": kernel, "achieved": None, "peak": None, "frac": None}
    if bound == "hbm":
        ach = work / (k_ms * 1e-3) / 1e9
        r = {"bound": "hbm", "kernel": kernel, "achieved": ach, "peak": hbm_peak, "unit": "GB/s", "frac": ach / hbm_peak,
             "peak_source": f"of {peak_kind}", "frac_of_nominal_8000_GBs": ach / 8000.0, "kernel_ms": k_ms,
             "algorithmic_bytes": work}
        if wl.idx == 2:  # this product is bound by the FP64 tensor pipe long before HBM: say so next to the HBM figure
            fl = 2.0 * wl.n * 250 * 64
            r["dmma"] = {"algorithmic_TFLOPs": fl / (k_ms * 1e-3) / 1e12, "peak_TFLOPs": dmma_peak,
                         "frac": fl / (k_ms * 1e-3) / 1e12 / dmma_peak,
                         "note": "250 dense-operand columns (200 DDC + 50 uncompressed) x 64 x 2 flop per row on DMMA m8n8k4"}
    else:
        ach = work / (k_ms * 1e-3) / 1e12
        r = {"bound": "tensor", "kernel": kernel, "achieved": ach, "peak": dmma_peak, "unit": "TFLOP/s",
             "frac": ach / dmma_peak, "peak_source": "FP64 DMMA rate measured by cla_measure_fp64_peaks (back-to-back "
             "independent m8n8k4, CUDA events); MEASURED_PEAKS.json holds no FP64 figure", "kernel_ms": k_ms,
             "algorithmic_flops": work}
    tr = TRAFFIC_PER_ROW.get(wl.idx)
    r["traffic"] = tr * wl.n if tr else None
    return r


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", type=int, default=1, choices=[0, 1, 2, 3, 4],
                    help="which of the five benchmark workloads the main line measures (default 1: t(y)%%*%%X)")
    ap.add_argument("--rows", type=int, default=None, help="rows per GPU (default: the workload's benchmark size)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-also", action="store_true", help="skip the other four workloads")
    ap.add_argument("--also-steps", type=int, default=20)
    ap.add_argument("--strong", action="store_true",
                    help="strong scaling: the workload's rows are split over the N GPUs instead of each GPU holding all of them")
    ap.add_argument("--allreduce", default="peer", choices=["peer", "nccl"],
                    help="N > 1: the library's exchange over peer memory (default) or NCCL")
    ap.add_argument("--decompress", action="store_true",
                    help="also time cla_decompress_dev of the main workload's matrix into a device buffer (one GPU)")
    ap.add_argument("--also-rows-scale", type=float, default=1.0, help="scale the rows of the 'also' workloads (profiling aid)")
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
    from systemds_b200 import native
    from systemds_b200.native import check

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the compressed products have no CPU path")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    numa_node, full_affinity = bind_to_gpu_numa_node(local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    L = native.lib()
    hbm_peak, peak_kind = measured_peaks()
    dm, df = C.c_double(0), C.c_double(0)
    check(L.cla_measure_fp64_peaks(local_rank, C.byref(dm), C.byref(df)))
    dmma_peak = dm.value

    Workload.setup_allreduce(rank, local_rank, world, dev, args.allreduce)
    w = args.workload
    n = args.rows or DEFAULT_ROWS[w]
    if args.strong:
        n = max(4096, n // world)
    # the main workload keeps host-generated arrays when the CPU baseline will read them (workload 1 on one GPU)
    main = Workload(w, n, rank, local_rank, world, dev, L, host_gen=(w == 1)).build()

    sampler = ClockSampler(local_rank)
    sampler.start()
    ms_step, k_ms, launches = time_steps(main, args.steps, args.warmup, world)
    total_rows = n * world
    value = total_rows / (ms_step * 1e-3)

    # ---- e2e: host buffers through the plugin-facing call; pinned (the bench contract) and pageable (what a JVM
    #      hands over through GetPrimitiveArrayCritical) ----
    e2e = {}
    e2e_steps = max(3, min(args.steps, 10))
    for kind in ("pinned", "pageable"):
        main.e2e_prepare(pinned=(kind == "pinned"))
        for _ in range(2):
            main.e2e_step()
        barrier(world)
        t0 = time.perf_counter()
        for _ in range(e2e_steps):
            main.e2e_step()
        barrier(world)
        ms = (time.perf_counter() - t0) * 1e3 / e2e_steps
        t = torch.tensor([ms], dtype=torch.float64, device=dev)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e[kind] = float(t[0])
    clocks = sampler.stop()

    result = {
        "metric": METRICS[w], "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": ms_step, "higher_is_better": True, "scaling": "strong" if args.strong else "weak", "vs_baseline": None, "dtype": "f64",
        "data": "synthetic",
        "config": {"workload": DESCS[w], "rows_per_gpu": n,
                   "parallelism": f"row-sharded x{world}" if world > 1 else "single GPU",
                   "allreduce": Workload.comm_note if world > 1 else None,
                   "l2": ("256 MB buffer written between timed steps (inputs are below the 126 MB L2)" if main.needs_l2_flush
                          else f"inputs ({main.index_bytes / 1e9:.2f} GB per step) larger than L2; no flush needed"),
                   "host": {"numa_node": numa_node, "cpus": len(os.sched_getaffinity(0))}},
        "roofline": roofline_of(main, k_ms, hbm_peak, peak_kind, dmma_peak),
        "e2e": {"value": total_rows / (e2e["pinned"] * 1e-3), "unit": UNIT, "h2d_bytes_per_step": main.h2d,
                "d2h_bytes_per_step": main.d2h, "ms_per_step": e2e["pinned"], "steps": e2e_steps,
                "timer": "host wall clock around the synchronous C-ABI call (pinned host buffers, max over ranks)",
                "pageable": {"value": total_rows / (e2e["pageable"] * 1e-3), "ms_per_step": e2e["pageable"],
                             "note": "the same call with ordinary (pageable) host arrays, as a JVM heap array is"}},
        "gpu_launches": launches,
        "clocks": clocks,
        "fp64_peaks_measured": {"dmma_m8n8k4_TFLOPs": dm.value, "dfma_TFLOPs": df.value},
    }

    # ---- CPU baseline (rank 0, one GPU): the same arrays for workload 1, a bounded sample otherwise ----
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        os.sched_setaffinity(0, full_affinity)
        if w == 1 and main.host_gen:
            from oracle import oracle as o
            o.build()
            om = o.OracleMatrix(main.cmb, threads=len(full_affinity))
            y = main.y_pin.numpy().reshape(1, -1)
            om.lmm(y)
            ts = []
            for _ in range(3):
                t0 = time.perf_counter()
                om.lmm(y)
                ts.append(time.perf_counter() - t0)
            rate, ms, cores, rows = n / float(np.mean(ts)), float(np.mean(ts)) * 1e3, om.k, n
            del om
        else:
            rows = min(n, CPU_ROWS[w])
            rate, ms, cores = cpu_reference_rate(w, rows, 3, 1)
        result["cpu_baseline"] = {"value": rate, "unit": UNIT, "cores": cores, "kind": "port",
                                  "sample": (f"the full workload, {rows} rows" if rows == n else f"{rows} rows of the same workload")
                                            + f", mean of 3 runs ({ms:.0f} ms each)"}
    # ---- decompress of the same matrix into a device buffer (the output stream is the bound: 8 bytes per cell) ----
    if args.decompress and world == 1:
        cols = main.cmb.clen
        dense = torch.empty((n, cols), dtype=torch.float64, device=dev)
        dec = lambda: check(L.cla_decompress_dev(main.h, C.c_void_p(dense.data_ptr()), main.sptr))  # noqa: E731
        for _ in range(3):
            dec()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        e0.record()
        for _ in range(args.also_steps):
            dec()
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / args.also_steps
        wr = n * cols * 8
        result["decompress"] = {"ms": ms, "rows": n, "cols": cols, "written_GBs": wr / (ms * 1e-3) / 1e9,
                                "frac": wr / (ms * 1e-3) / 1e9 / hbm_peak, "peak_source": f"of {peak_kind}",
                                "algorithmic_bytes": wr + main.index_bytes,
                                "note": "cla_decompress_dev into a device buffer; frac = bytes written / time / copy bandwidth"}
        del dense
    main.free()

    # ---- the other workloads, every rank, same sharding ----
    if not args.no_also:
        also = {}
        for i in range(5):
            if i == w:
                continue
            rows = max(4096, int(DEFAULT_ROWS[i] * args.also_rows_scale) // (world if args.strong else 1))
            wl = Workload(i, rows, rank, local_rank, world, dev, L).build()
            ms_i, k_i, launches_i = time_steps(wl, args.also_steps, 5, world)
            also[f"workload{i}"] = {"metric": METRICS[i], "workload": DESCS[i], "rows_per_gpu": rows,
                                    "value": rows * world / (ms_i * 1e-3), "unit": UNIT, "ms_per_step": ms_i,
                                    "steps": args.also_steps, "gpu_launches": launches_i,
                                    "roofline": roofline_of(wl, k_i, hbm_peak, peak_kind, dmma_peak),
                                    "l2": "256 MB written between steps" if wl.needs_l2_flush else "inputs larger than L2"}
            wl.free()
        result["also"] = also
    if rank == 0:
        print(json.dumps(result))
    if Workload.comm is not None:
        Workload.comm.status()
        Workload.comm.close()
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
