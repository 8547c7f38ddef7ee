#!/usr/bin/env python
"""Benchmark of the hash groupby-aggregate path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl b2|reference] [--config 2] [--rows R]

A "step" is one complete ``GroupBy(keys).aggregate(requests)`` call over one batch of synthetic input
(table sizing + init, the fused aggregate pass, the group-count read-back, output allocation and
finalisation).  At N = 1 the workload is configuration C2 of the benchmark specification (100M rows, composite
int32 keys, float32 values with 2 % nulls, dropna() then mean, ~10K groups).  At N > 1 every rank
holds its own C2-sized shard (weak scaling), aggregates it, hash-partitions its partial aggregates
by owner, exchanges them with one all-to-all over NCCL and merges / finalises the groups it owns.

Prints ONE JSON line (rank 0):  value = rows/s with inputs resident in HBM;  e2e = rows/s from
pinned HOST buffers (H2D of the inputs and D2H of the results inside the timed region);  roofline =
algorithmic bytes of the fused kernel / its CUDA-event duration against the measured HBM copy peak;
cpu_baseline = the CPU oracle on this host.  ``--impl reference`` times the reference's CPU path
stand-in (the oracle port on all host threads; libcudf itself cannot be built offline).
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

import numpy as np  # noqa: E402

import workloads  # noqa: E402

METRIC = "groupby-aggregate rows/sec"
FALLBACK_HBM_GBS = 6650.0
# DRAM bytes per input row of k_aggregate on C2, from the ncu capture summarised in
# profiles/k_aggregate_c2.md (20M-row case: (243.74 + 3.89) MB / 20M rows), scaled by the rows of a launch
C2_TRAFFIC_BYTES_PER_ROW = 12.38


def measured_peak():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return FALLBACK_HBM_GBS, "fallback"


def workload_desc(cfg: int, rows: int) -> str:
    d = {1: "C1: int64 key U[0,1000), f64 value 5% nulls, sum/count/mean",
         2: "C2: keys (int32 U[0,100), int32 U[0,100)), f32 value 2% nulls, dropna() then mean, ~10K groups",
         3: "C3: int64 key U[0,100M), int64 value, sum/min/max/count",
         4: "C4: int64 key Zipf(1.1) over 10M ids, f64 LogNormal value 1% nulls, sum/mean/var",
         5: "C5: keys (string 8-32 B pool 1M, int32 U[0,16)), f64 + int32 values 3% nulls, sum/count/mean/min/max"}
    return f"{d[cfg]}; {rows} rows per GPU"


class ClockSampler:
    """Samples SM clock and throttle reasons of one GPU through NVML while a region runs."""

    def __init__(self, index: int, period: float = 0.02):
        self.index, self.period = index, period
        self.samples, self.reasons = [], set()
        self.max_mhz = None
        self._stop = threading.Event()
        self._thread = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self.nv = None

    def _run(self):
        nv = self.nv
        names = {"hw_slowdown": 0x8, "sw_power_cap": 0x4, "hw_thermal_slowdown": 0x40, "sw_thermal_slowdown": 0x20,
                 "hw_power_brake_slowdown": 0x80}
        while not self._stop.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM))
                try:
                    r = nv.nvmlDeviceGetCurrentClocksEventReasons(self.h)
                except Exception:
                    r = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
                for k, bit in names.items():
                    if r & bit:
                        self.reasons.add(k)
            except Exception:
                pass
            time.sleep(self.period)

    def __enter__(self):
        if self.nv:
            self._thread = threading.Thread(target=self._run, daemon=True)
            self._thread.start()
        return self

    def __exit__(self, *a):
        self._stop.set()
        if self._thread:
            self._thread.join()

    def summary(self):
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons), "samples": 0}
        return {"sm_mhz": statistics.median(self.samples), "sm_max_mhz": self.max_mhz,
                "reasons": sorted(self.reasons), "samples": len(self.samples)}


def oracle_rows_per_s(w, threads: int, repeats: int = 1):
    from oracle import oracle
    best = None
    for _ in range(repeats):
        t0 = time.perf_counter()
        oracle.groupby(w.keys, w.requests, w.null_policy, row_filters=[f.mask for f in w.row_filters],
                       threads=threads)
        dt = time.perf_counter() - t0
        best = dt if best is None else min(best, dt)
    return w.rows / best, best


def run_reference(args):
    """The reference arm: the reference's CPU implementation of the path on the host cores.  libcudf
    cannot be compiled offline, so this is the oracle port, on every host thread, on a bounded
    sample of the same workload per step."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    cores = os.cpu_count() or 1
    sample_rows = min(args.rows, 20_000_000)
    w = workloads.make(args.config, sample_rows)
    for _ in range(args.warmup):
        oracle_rows_per_s(w, cores)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        oracle_rows_per_s(w, cores)
    dt = time.perf_counter() - t0
    value = sample_rows * args.steps / dt
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": "rows/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt / args.steps * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f64", "data": "synthetic",
        "config": {"workload": workload_desc(args.config, args.rows)},
        "cpu_baseline": {"value": value, "unit": "rows/s", "cores": cores, "kind": "port",
                         "sample": f"first {sample_rows} rows of the workload per step, {cores} threads"},
        "e2e": {"value": value, "unit": "rows/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


def run_b2(args):
    import torch
    import torch.distributed as dist

    import cudf_b200 as cb
    from cudf_b200.aggregation import Aggregation
    from cudf_b200.distributed import DistributedGroupBy
    from cudf_b200.types import Kind

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)

    w = workloads.make(args.config, args.rows, rank=rank)
    host_cols = {}

    def pinned(hc):
        if id(hc) not in host_cols:
            host_cols[id(hc)] = hc
        return hc

    # ---- resident inputs
    dev = {}
    for hc in w.keys + [v for v, _ in w.requests] + w.row_filters:
        if id(hc) not in dev:
            dev[id(hc)] = cb.Column.from_host(pinned(hc), device)
    torch.cuda.synchronize()
    keys = cb.Table([dev[id(k)] for k in w.keys])
    reqs = [cb.GroupByRequest(dev[id(v)], [Aggregation(Kind(a)) for a in aggs]) for v, aggs in w.requests]
    filt = [dev[id(f)] for f in w.row_filters]

    kept = []  # --reuse-groupby: one DistributedGroupBy for all steps (it sizes its tables from its previous call)

    def step_resident():
        if world == 1:
            gb = cb.GroupBy(keys, w.null_policy, row_filters=filt)
        elif args.reuse_groupby and kept:
            gb = kept[0]
        else:
            gb = DistributedGroupBy(keys, w.null_policy, row_filters=filt, strategy=args.strategy)
            if args.reuse_groupby:
                kept.append(gb)
        return gb.aggregate(reqs)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    sampler = ClockSampler(local)
    launches, kernel_ms, groups = 0, [], 0
    for _ in range(max(args.warmup, 3)):
        out = step_resident()
    groups = out[0].num_rows()
    barrier()
    with sampler:
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        ev0.record()
        for _ in range(args.steps):
            out = step_resident()
            st = cb.last_call_stats()
            launches += st.kernel_launches
            kernel_ms.append(st.aggregate_kernel_ms)
        ev1.record()
        barrier()
        ms = ev0.elapsed_time(ev1)
        if world > 1:
            t = torch.tensor([ms], device=device)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())

        # ---- end to end from pinned host buffers
        pin = {}
        for hc in w.keys + [v for v, _ in w.requests] + w.row_filters:
            if id(hc) in pin:
                continue
            bufs = {}
            for name in ("data", "mask", "offsets"):
                arr = getattr(hc, name)
                if arr is not None:
                    bufs[name] = torch.from_numpy(np.ascontiguousarray(arr).view(np.uint8).reshape(-1)).pin_memory()
            pin[id(hc)] = bufs
        h2d_bytes = sum(t.numel() for b in pin.values() for t in b.values())

        def upload(hc):
            b = pin[id(hc)]
            d = {k: t.to(device, non_blocking=True) for k, t in b.items()}
            return cb.Column(hc.type_id, hc.size, d.get("data"), d.get("mask"), hc.offset,
                             -1 if hc.mask is not None else 0, d.get("offsets"),
                             cb.TypeId.INT64 if hc.offsets is not None and hc.offsets.dtype == np.int64 else cb.TypeId.INT32)

        d2h_bytes = 0

        def step_e2e():
            nonlocal d2h_bytes
            cols = {}
            for hc in w.keys + [v for v, _ in w.requests] + w.row_filters:
                if id(hc) not in cols:
                    cols[id(hc)] = upload(hc)
            k = cb.Table([cols[id(x)] for x in w.keys])
            r = [cb.GroupByRequest(cols[id(v)], [Aggregation(Kind(a)) for a in aggs]) for v, aggs in w.requests]
            f = [cols[id(x)] for x in w.row_filters]
            gb = cb.GroupBy(k, w.null_policy, row_filters=f) if world == 1 else \
                DistributedGroupBy(k, w.null_policy, row_filters=f, strategy=args.strategy)
            ok, orr = gb.aggregate(r)
            got = 0
            for c in ok.columns() + [c for t in orr for c in t.columns()]:
                for t in (c.data, c.mask, c.offsets):
                    if t is not None:
                        got += t.cpu().numel()
            d2h_bytes = got

        e2e_steps = max(2, min(args.steps, 10))
        step_e2e()
        barrier()
        ee0, ee1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        ee0.record()
        for _ in range(e2e_steps):
            step_e2e()
        ee1.record()
        barrier()
        e2e_ms = ee0.elapsed_time(ee1)
        if world > 1:
            t = torch.tensor([e2e_ms], device=device)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            e2e_ms = float(t.item())

    total_rows = w.rows * world
    value = total_rows * args.steps / (ms / 1e3)
    e2e_value = total_rows * e2e_steps / (e2e_ms / 1e3)

    line = None
    if rank == 0:
        peak, peak_kind = measured_peak()
        in_bytes = w.input_bytes()
        out_bytes = workloads.output_bytes(w, groups)
        alg_bytes = in_bytes + out_bytes
        kms = statistics.mean(kernel_ms) if kernel_ms else float("nan")
        achieved = alg_bytes / (kms / 1e3) / 1e9 if kms and kms > 0 else None
        line = {
            "metric": METRIC, "value": value, "unit": "rows/s", "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": ms / args.steps, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "f64", "data": "synthetic",
            "config": {"workload": workload_desc(args.config, w.rows), "groups_rank0": groups,
                       "strategy": "single GPU" if world == 1 else f"{args.strategy} shuffle over NCCL all-to-all"
                                   + (", one DistributedGroupBy reused across steps" if args.reuse_groupby else ""),
                       "l2": f"inputs ({in_bytes / 1e6:.0f} MB per GPU) larger than the 126 MB L2; no flush needed",
                       "algorithmic_bytes_per_step": alg_bytes},
            "clocks": sampler.summary(),
            "e2e": {"value": e2e_value, "unit": "rows/s", "h2d_bytes_per_step": h2d_bytes,
                    "d2h_bytes_per_step": d2h_bytes, "steps": e2e_steps, "ms_per_step": e2e_ms / e2e_steps},
            "gpu_launches": launches,
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s",
                         "frac": (achieved / peak) if achieved else None,
                         "traffic": (C2_TRAFFIC_BYTES_PER_ROW * w.rows) if args.config == 2 else None,
                         "kernel": "k_aggregate", "kernel_ms": kms, "peak_kind": f"of {peak_kind}",
                         "step_GBps": alg_bytes / (ms / args.steps / 1e3) / 1e9},
        }
        if world == 1 and not args.no_cpu_baseline:
            sample_rows = min(w.rows, 50_000_000)
            ws = workloads.make(args.config, sample_rows) if sample_rows != w.rows else w
            v, secs = oracle_rows_per_s(ws, 1)
            line["cpu_baseline"] = {"value": v, "unit": "rows/s", "cores": 1, "kind": "port",
                                    "sample": f"{sample_rows} rows of the same workload, one run of {secs:.1f} s, "
                                              f"single-thread oracle ({os.cpu_count()} cores on the host)"}
        else:
            line["cpu_baseline"] = None
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="b2", choices=["b2", "reference"])
    ap.add_argument("--config", type=int, default=2)
    ap.add_argument("--rows", type=int, default=0, help="rows per GPU (0 = the configuration's full size)")
    ap.add_argument("--strategy", default="partials", choices=["partials", "rows"])
    ap.add_argument("--reuse-groupby", action="store_true",
                    help="N > 1: keep one DistributedGroupBy across the steps instead of a fresh one per step")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    args = ap.parse_args()
    if args.rows <= 0:
        args.rows = workloads.FULL_ROWS[args.config]
    if args.impl == "reference":
        run_reference(args)
    else:
        run_b2(args)


if __name__ == "__main__":
    main()
