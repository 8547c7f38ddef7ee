#!/usr/bin/env python
"""Benchmark of the hash groupby-aggregate path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl b2|reference] [--config 2] [--rows R]

A "step" is one complete ``GroupBy(keys).aggregate(requests)`` call over one batch of synthetic input
(table sizing + init, the fused aggregate pass, the group-count read-back, output allocation and
finalisation).  At N = 1 the workload is configuration C2 of the benchmark specification (100M rows, composite
int32 keys, float32 values with 2 % nulls, dropna() then mean, ~10K groups).  At N > 1 every rank
holds its own C2-sized shard (weak scaling), aggregates it, hash-partitions its partial aggregates
by owner, exchanges them with one all-to-all over NCCL and merges / finalises the groups it owns.

Prints ONE JSON line (rank 0):
  value        rows/s with inputs resident in HBM (CUDA events around K steps, max over ranks);
  e2e          rows/s from pinned HOST buffers (H2D of the inputs and D2H of the results in the timed region);
  roofline     algorithmic bytes of the fused kernel / its CUDA-event duration against the measured HBM copy peak;
  cpu_baseline pandas (what cudf.pandas runs when it falls back to the CPU) on one host core, plus the
               multi-threaded C++ oracle port as a second figure;
  parity       checks of the LAST timed step's result computed after the timed region (every N);
  configs      N = 1: one entry per other configuration (C1, C3, C4, C5) at full size, inputs generated
               on the device: ms per call (median of 5), kernel ms, algorithmic bytes, fraction of the peak;
  c3_strong    (N > 1) the 500M-row all-distinct configuration split over the N ranks, rows shuffled by key
               before the local aggregate, every group checked exactly
  c4_strong    the 1B-row skewed configuration split by rows over the N ranks (1B/N rows each), a fresh
               distributed groupby per step: ms per step (max over ranks) and rows/s, with its own parity.
``--impl reference`` times the reference's CPU path (pandas, single-threaded by construction) on a
bounded sample of the same workload; libcudf itself cannot be built offline.
"""
from __future__ import annotations

import argparse
import gc
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
# DRAM bytes per input row of the fused kernel on C2, from an ncu capture of a 20M-row launch
# ((dram__bytes_read.sum + dram__bytes_write.sum) / rows); DRAM traffic grows with the rows, the fixed
# part (table init, merge) is below 1 %
C2_TRAFFIC_BYTES_PER_ROW = 12.38
C2_TRAFFIC_SOURCE = "ncu capture of a 20M-row launch x rows of this launch"


def measured_peak():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return FALLBACK_HBM_GBS, "fallback"


WORKLOADS = {1: "C1: int64 key U[0,1000), f64 value 5% nulls, sum/count/mean",
             2: "C2: keys (int32 U[0,100), int32 U[0,100)), f32 value 2% nulls, dropna() then mean, ~10K groups",
             3: "C3: int64 key U[0,100M), int64 value, sum/min/max/count",
             4: "C4: int64 key Zipf(1.1) over 10M ids, f64 LogNormal value 1% nulls, sum/mean/var",
             5: "C5: keys (string 8-32 B pool 1M, int32 U[0,16)), f64 + int32 values 3% nulls, sum/count/mean/min/max"}


def workload_desc(cfg: int, rows: int) -> str:
    return f"{WORKLOADS[cfg]}; {rows} rows per GPU"


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


# ------------------------------------------------------------------------------------ CPU arms
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


def pandas_frame(w):
    """The host workload as the DataFrame a cudf.pandas user would hold: nulls as NaN / pd.NA."""
    import pandas as pd
    from cudf_b200.types import TypeId, is_floating
    cols, names = {}, []

    def add(name, hc):
        if name in cols:
            return
        if hc.type_id == TypeId.STRING:
            cols[name] = pd.array(hc.to_pylist(), dtype="str")
        elif hc.mask is None:
            cols[name] = hc.values()
        elif is_floating(hc.type_id):
            v = hc.values().copy()
            v[~hc.valid()] = np.nan
            cols[name] = v
        else:
            cols[name] = pd.array(hc.values(), dtype=str(hc.values().dtype).replace("int", "Int").replace("uInt", "UInt"))
            cols[name][~hc.valid()] = pd.NA
    key_names = [f"K{i}" for i in range(len(w.keys))]
    for nme, k in zip(key_names, w.keys):
        add(nme, k)
    val_names, seen = [], {}
    for v, _ in w.requests:
        if id(v) not in seen:
            seen[id(v)] = f"V{len(seen)}"
            add(seen[id(v)], v)
        val_names.append(seen[id(v)])
    return pd.DataFrame(cols, copy=False), key_names, val_names


PANDAS_AGG = {0: "sum", 3: "min", 4: "max", 5: "count", 6: "size", 10: "mean", 12: "var", 13: "std"}


def pandas_groupby(w, df, key_names, val_names):
    """The pandas expression of the workload: what cudf.pandas executes on its CPU fallback
    (python/cudf/cudf/pandas/fast_slow_proxy.py:1568-1585)."""
    if w.row_filters:   # C2: df.dropna().groupby(["A", "B"]).mean()
        return df.dropna().groupby(key_names).mean()
    spec = {}
    for name, (_, aggs) in zip(val_names, w.requests):
        spec.setdefault(name, [])
        spec[name] += [PANDAS_AGG[int(a[0] if isinstance(a, tuple) else a)] for a in aggs]
    return df.groupby(key_names, dropna=True).agg(spec)


def pandas_rows_per_s(w, repeats: int = 1):
    df, key_names, val_names = pandas_frame(w)
    best, groups = None, 0
    for _ in range(repeats):
        t0 = time.perf_counter()
        out = pandas_groupby(w, df, key_names, val_names)
        dt = time.perf_counter() - t0
        groups = len(out)
        best = dt if best is None else min(best, dt)
    return w.rows / best, best, groups


def pandas_version():
    try:
        import pandas
        return pandas.__version__
    except Exception:
        return None


def run_reference(args):
    """The reference arm: the reference's CPU implementation of the path on the host cores.  libcudf
    cannot be compiled offline; its CPU path is pandas through the cudf.pandas fallback, which is
    single-threaded for a groupby whatever the core count.  Each step is a bounded sample of the
    workload; the multi-threaded C++ oracle port is timed once beside it as a second figure."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    cores = os.cpu_count() or 1
    sample_rows = min(args.rows, 10_000_000)
    w = workloads.make(args.config, sample_rows)
    use_pandas = pandas_version() is not None
    df = key_names = val_names = None
    if use_pandas:
        df, key_names, val_names = pandas_frame(w)

    def step():
        if use_pandas:
            pandas_groupby(w, df, key_names, val_names)
        else:
            oracle_rows_per_s(w, cores)
    for _ in range(args.warmup):
        step()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        step()
    dt = time.perf_counter() - t0
    value = sample_rows * args.steps / dt
    port_value, _ = oracle_rows_per_s(w, cores)
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": "rows/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt / args.steps * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32->f64", "data": "synthetic",
        "config": {"workload": workload_desc(args.config, args.rows)},
        "cpu_baseline": {"value": value, "unit": "rows/s", "cores": 1 if use_pandas else cores,
                         "kind": "reference" if use_pandas else "port",
                         "engine": f"pandas {pandas_version()} (the CPU path of cudf.pandas), single-threaded; "
                                   f"{cores} cores on the host" if use_pandas else "C++ oracle port",
                         "sample": f"first {sample_rows} rows of the workload per step",
                         "port_value": port_value, "port_cores": cores,
                         "port_note": "C++ restatement of the reference's rules on every host thread, same sample"},
        "e2e": {"value": value, "unit": "rows/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------------------ GPU arm helpers
def _tensor(col, torch_dtype):
    import torch
    nbytes = col.size * torch.empty(0, dtype=torch_dtype).element_size()
    return col.data[:nbytes].view(torch_dtype)


def _all_reduce(t, op="sum"):
    import torch.distributed as dist
    if dist.is_initialized() and dist.get_world_size() > 1:
        dist.all_reduce(t, op={"sum": dist.ReduceOp.SUM, "max": dist.ReduceOp.MAX, "min": dist.ReduceOp.MIN}[op])
    return t


def parity_c2(raw, out):
    """Checks one finished C2 result against an independent torch computation on the same inputs:
    owned key sets disjoint across ranks, their union = the distinct keys of all ranks' inputs, and
    every owned group's mean within the fp32-source tolerance of an fp64 index_add reference that is
    all-reduced over the ranks.  (The mean request carries no count; Σ count is checked through the
    reference: a wrong count would show in the mean.)"""
    import torch
    a, b, v, valid = raw["a"], raw["b"], raw["v"], raw["valid"]
    keys, res = out
    ka, kb = _tensor(keys.columns()[0], torch.int32), _tensor(keys.columns()[1], torch.int32)
    gid = ka.to(torch.int64) * 100 + kb.to(torch.int64)
    mean = _tensor(res[0].columns()[0], torch.float64)
    rid = (a.to(torch.int64) * 100 + b.to(torch.int64))[valid]
    ref_sum = _all_reduce(torch.zeros(10_000, dtype=torch.float64, device=a.device).index_add_(0, rid, v[valid].double()))
    ref_cnt = _all_reduce(torch.bincount(rid, minlength=10_000))
    owned = _all_reduce(torch.bincount(gid, minlength=10_000))
    in_range = bool(((gid >= 0) & (gid < 10_000)).all())
    disjoint = int(owned.max()) <= 1
    union_ok = bool(((owned > 0) == (ref_cnt > 0)).all())
    ref_mean = ref_sum[gid] / ref_cnt[gid]
    err = ((mean - ref_mean).abs() / ref_mean.abs())
    max_err = float(_all_reduce(err.max().reshape(1).clone(), "max")) if gid.numel() else 0.0
    checks = {"keys_in_range": in_range, "owned_key_sets_disjoint": disjoint, "union_equals_input_keys": union_ok,
              "groups_total": int((owned > 0).sum()), "groups_expected": int((ref_cnt > 0).sum()),
              "rows_counted_by_reference": int(ref_cnt.sum()), "max_rel_err_mean": max_err, "rtol": 1e-5}
    ok = in_range and disjoint and union_ok and max_err < 1e-5
    return {"ok": bool(ok), "what": "last timed step vs fp64 torch reference, all-reduced over ranks", **checks}


def parity_c4(raw, out):
    """C4 (sum, mean, var on f64 with nulls; int64 Zipf keys over 10M ids): Σ count is not requested,
    so counts are checked through the per-group reference; owned key sets disjoint; union = input keys;
    Σ of the owned sums = Σ of the valid inputs; per-group sum / mean / variance against fp64 torch
    index_add references all-reduced over the ranks (1e-11, the variance relative to Σx²/(n-1))."""
    import torch
    k, v, valid, distinct = raw["k"], raw["v"], raw["valid"], raw["distinct"]
    keys, res = out
    ok_keys = _tensor(keys.columns()[0], torch.int64)
    s, mean, var = (_tensor(res[0].columns()[i], torch.float64) for i in range(3))
    kv, vv = k[valid], v[valid]
    ref_sum = _all_reduce(torch.zeros(distinct, dtype=torch.float64, device=k.device).index_add_(0, kv, vv))
    ref_sq = _all_reduce(torch.zeros(distinct, dtype=torch.float64, device=k.device).index_add_(0, kv, vv * vv))
    ref_cnt = _all_reduce(torch.bincount(kv, minlength=distinct))
    present = _all_reduce(torch.bincount(k, minlength=distinct).clamp_(max=1), "max")
    owned = _all_reduce(torch.bincount(ok_keys, minlength=distinct))
    disjoint = int(owned.max()) <= 1
    union_ok = bool(((owned > 0) == (present > 0)).all())
    c = ref_cnt[ok_keys]
    has = c > 0
    total_got = float(_all_reduce(s[has].sum().reshape(1).clone()))
    total_ref = float(ref_sum.sum())
    rel_total = abs(total_got - total_ref) / abs(total_ref)
    e_sum = float(_all_reduce(((s[has] - ref_sum[ok_keys][has]).abs() / ref_sum[ok_keys][has]).max().reshape(1).clone(), "max"))
    e_mean = float(_all_reduce(((mean[has] - ref_sum[ok_keys][has] / c[has]).abs() / mean[has]).max().reshape(1).clone(), "max"))
    many = c > 1
    cm = c[many].double()
    ref_var = (ref_sq[ok_keys][many] - ref_sum[ok_keys][many] ** 2 / cm) / (cm - 1)
    scale = ref_sq[ok_keys][many] / (cm - 1)
    e_var = float(_all_reduce(((var[many] - ref_var).abs() / scale).max().reshape(1).clone(), "max"))
    ok = disjoint and union_ok and rel_total < 1e-9 and e_sum < 1e-11 and e_mean < 1e-11 and e_var < 1e-11
    return {"ok": bool(ok), "owned_key_sets_disjoint": disjoint, "union_equals_input_keys": union_ok,
            "groups_total": int((owned > 0).sum()), "groups_expected": int((present > 0).sum()),
            "rel_err_total_sum": rel_total, "max_rel_err_sum": e_sum, "max_rel_err_mean": e_mean,
            "max_err_var_over_scale": e_var, "rtol": 1e-11}


def parity_c3(raw, out, total_rows):
    """C3 (sum, min, max, count of an int64 column; int64 keys U[0,100M)): owned key sets disjoint, union =
    input keys, and every owned group's sum / min / max / count equal — integers, exactly — to torch
    references over all ranks' inputs (index_add / scatter_reduce / bincount on 100M-entry arrays, all-reduced)."""
    import torch
    k, v = raw["k"], raw["v"]
    domain = 100_000_000
    keys, res = out
    ok_keys = _tensor(keys.columns()[0], torch.int64)
    cols = res[0].columns()
    s, mn, mx = (_tensor(cols[i], torch.int64) for i in range(3))
    cnt = _tensor(cols[3], torch.int32).to(torch.int64)
    ref_cnt = _all_reduce(torch.bincount(k, minlength=domain))
    ref_sum = _all_reduce(torch.zeros(domain, dtype=torch.int64, device=k.device).index_add_(0, k, v))
    ref_min = _all_reduce(torch.full((domain,), 2**62, dtype=torch.int64, device=k.device).scatter_reduce_(0, k, v, "amin"), "min")
    ref_max = _all_reduce(torch.full((domain,), -2**62, dtype=torch.int64, device=k.device).scatter_reduce_(0, k, v, "amax"), "max")
    owned = _all_reduce(torch.bincount(ok_keys, minlength=domain))
    disjoint = int(owned.max()) <= 1
    union_ok = bool(((owned > 0) == (ref_cnt > 0)).all())
    bad = ((s != ref_sum[ok_keys]) | (mn != ref_min[ok_keys]) | (mx != ref_max[ok_keys]) | (cnt != ref_cnt[ok_keys])).sum()
    bad = int(_all_reduce(bad.reshape(1).clone()).item())
    rows = int(_all_reduce(cnt.sum().reshape(1).clone()).item())
    ok = disjoint and union_ok and bad == 0 and rows == total_rows
    return {"ok": bool(ok), "owned_key_sets_disjoint": disjoint, "union_equals_input_keys": union_ok,
            "groups_total": int((owned > 0).sum()), "groups_expected": int((ref_cnt > 0).sum()),
            "groups_with_a_wrong_sum_min_max_or_count": bad, "rows_counted": rows, "rows_expected": total_rows}


def time_calls(fn, n, barrier):
    """n calls of fn, each bracketed by CUDA events on the current stream: list of ms."""
    import torch
    ms = []
    for _ in range(n):
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        ms.append(e0.elapsed_time(e1))
    return ms


def run_other_configs(peak, which=(1, 5, 3, 4)):
    """N = 1: the other configurations at full size, inputs generated on the device."""
    import torch
    import cudf_b200 as cb
    out = {}
    for cfg in which:
        try:
            w = workloads.make_device(cfg)
            reqs = w.groupby_requests()
            keys = cb.Table(w.keys)
            res = {}

            def call():
                res["out"] = cb.GroupBy(keys, row_filters=w.row_filters).aggregate(reqs)
                res["stats"] = cb.last_call_stats()
            call()
            kms, calls = [], []
            for _ in range(5):
                calls += time_calls(call, 1, torch.cuda.synchronize)
                kms.append(res["stats"].aggregate_kernel_ms)
            groups = res["out"][0].num_rows()
            key_chars = sum(c.data.numel() for c in res["out"][0].columns() if c.type_id == cb.TypeId.STRING and c.data is not None)
            alg = w.input_bytes + workloads.device_output_bytes(w, groups, key_chars)
            ms = statistics.median(calls)
            k = statistics.median(kms)
            out[f"C{cfg}"] = {"workload": WORKLOADS[cfg], "rows": w.rows, "groups": groups, "ms_per_call": ms,
                              "ms_per_call_min": min(calls), "rows_per_s": w.rows / (ms / 1e3), "kernel_ms": k,
                              "table_attempts": res["stats"].table_attempts, "algorithmic_bytes": alg,
                              "GBps_call": alg / (ms / 1e3) / 1e9, "frac_call": alg / (ms / 1e3) / 1e9 / peak,
                              "GBps_kernel": alg / (k / 1e3) / 1e9 if k > 0 else None,
                              "frac": alg / (k / 1e3) / 1e9 / peak if k > 0 else None,
                              "calls": 5, "data": "generated on the device, seeded"}
            if cfg == 3:
                # cudf::hash_partition of the same rows into 8 destinations (the pre-step of a row exchange
                # between 8 ranks): reads the table twice (hash pass, gather), writes it once
                try:
                    from cudf_b200.partition import hash_partition
                    table = cb.Table(w.keys + [v for v, _ in w.requests])
                    pres = {}

                    def part():
                        pres["out"] = hash_partition(table, [0], 8)
                    part()
                    pms = statistics.median(time_calls(part, 5, torch.cuda.synchronize))
                    tbytes = w.input_bytes
                    out["hash_partition_C3_rows_8_parts"] = {
                        "rows": w.rows, "partitions": 8, "ms_per_call": pms, "table_bytes": tbytes,
                        "GBps_3x_table_bytes": 3 * tbytes / (pms / 1e3) / 1e9, "frac": 3 * tbytes / (pms / 1e3) / 1e9 / peak,
                        "rows_per_partition_min_max": [int(min(np.diff(pres["out"][1]))), int(max(np.diff(pres["out"][1])))]}
                    del pres, table
                except Exception as e:
                    out["hash_partition_C3_rows_8_parts"] = {"error": f"{type(e).__name__}: {e}"}
            del w, reqs, keys, res
        except Exception as e:  # one configuration must not take the headline line down
            out[f"C{cfg}"] = {"error": f"{type(e).__name__}: {e}"}
        torch.cuda.empty_cache()
    return out


def run_c4_strong(world, rank, device, steps, reuse):
    """The 1B-row skewed configuration split by rows over the ranks; a fresh (distributed) groupby per
    step unless ``reuse``.  Returns the entry (rank 0) after checking the last step's result."""
    import torch
    import torch.distributed as dist
    import cudf_b200 as cb
    from cudf_b200.distributed import DistributedGroupBy
    total = workloads.FULL_ROWS[4]
    n = total // world
    w = workloads.make_device(4, n, device=device, rank=rank)
    keys = cb.Table(w.keys)
    reqs = w.groupby_requests()
    kept, res, kms = [], {}, []

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def step():
        if world == 1:
            gb = cb.GroupBy(keys)
            res["out"] = gb.aggregate(reqs)
            kms.append(cb.last_call_stats().aggregate_kernel_ms)
            return
        elif reuse and kept:
            gb = kept[0]
        else:
            gb = DistributedGroupBy(keys, strategy="partials")
            if reuse:
                kept.append(gb)
        res["out"] = gb.aggregate(reqs)
    for _ in range(2):
        step()
    ms = time_calls(step, steps, barrier)
    t = torch.tensor(ms, device=device, dtype=torch.float64)
    _all_reduce(t, "max")
    ms = [float(x) for x in t.tolist()]
    par = parity_c4(w.raw, res["out"])
    groups = int(_all_reduce(torch.tensor([res["out"][0].num_rows()], device=device)).item())
    med = statistics.median(ms)
    entry = {"workload": WORKLOADS[4], "rows_total": n * world, "rows_per_gpu": n, "n_gpus": world, "steps": steps,
             "fresh_groupby_per_step": not reuse, "ms_per_step": med, "ms_per_step_min": min(ms), "ms_per_step_max": max(ms),
             "rows_per_s": n * world / (med / 1e3), "groups": groups, "scaling": "strong", "parity": par}
    if world == 1 and kms:   # one GPU: this is configuration C4 at full size, with its kernel figures
        peak, _ = measured_peak()
        alg = w.input_bytes + workloads.device_output_bytes(w, groups)
        k = statistics.median(kms[-steps:])
        entry.update({"kernel_ms": k, "algorithmic_bytes": alg, "GBps_call": alg / (med / 1e3) / 1e9,
                      "frac_call": alg / (med / 1e3) / 1e9 / peak, "frac": alg / (k / 1e3) / 1e9 / peak if k > 0 else None})
    return entry


def run_c3_strong(world, rank, device, steps):
    """N > 1: the 500M-row all-distinct configuration split by rows over the ranks, the ROWS shuffled by key
    (hash_partition + one all-to-all per column) before a local aggregate; a fresh object per step."""
    import torch
    import torch.distributed as dist
    import cudf_b200 as cb
    from cudf_b200.distributed import DistributedGroupBy
    n = workloads.FULL_ROWS[3] // world
    w = workloads.make_device(3, n, device=device, rank=rank)
    keys = cb.Table(w.keys)
    reqs = w.groupby_requests()
    res = {}

    def barrier():
        dist.barrier()
        torch.cuda.synchronize()

    def step():
        res["out"] = DistributedGroupBy(keys, strategy="rows").aggregate(reqs)
    for _ in range(2):
        step()
    ms = time_calls(step, steps, barrier)
    t = torch.tensor(ms, device=device, dtype=torch.float64)
    _all_reduce(t, "max")
    ms = [float(x) for x in t.tolist()]
    par = parity_c3(w.raw, res["out"], n * world)
    med = statistics.median(ms)
    return {"workload": WORKLOADS[3], "strategy": "rows shuffled by key, then a local aggregate", "rows_total": n * world,
            "rows_per_gpu": n, "n_gpus": world, "steps": steps, "ms_per_step": med, "ms_per_step_min": min(ms),
            "ms_per_step_max": max(ms), "rows_per_s": n * world / (med / 1e3), "groups": par["groups_total"],
            "scaling": "strong", "parity": par}


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

    # ---- resident inputs
    dev = {}
    for hc in w.keys + [v for v, _ in w.requests] + w.row_filters:
        if id(hc) not in dev:
            dev[id(hc)] = cb.Column.from_host(hc, device)
    torch.cuda.synchronize()
    keys = cb.Table([dev[id(k)] for k in w.keys])
    reqs = [cb.GroupByRequest(dev[id(v)], [Aggregation(Kind(a)) for a in aggs]) for v, aggs in w.requests]
    filt = [dev[id(f)] for f in w.row_filters]

    kept = []  # --reuse-groupby: one DistributedGroupBy for all steps (it sizes its tables from its previous call)

    def step_resident():
        if world == 1:
            gb = cb.GroupBy(keys, w.null_policy, row_filters=filt, table_variant=args.table_variant)
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
    warmup = max(args.warmup, 3)
    for _ in range(warmup):
        out = step_resident()
    groups = out[0].num_rows()
    barrier()
    with sampler:
        events = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps + 1)]
        # the interpreter's cyclic garbage collector is paused while steps are timed, as timeit does: a
        # collection inside one rank's step stalls every rank of that step
        gc.collect()
        gc.disable()
        barrier()
        events[0].record()
        for i in range(args.steps):
            out = step_resident()
            st = cb.last_call_stats()
            launches += st.kernel_launches
            kernel_ms.append(st.aggregate_kernel_ms)
            events[i + 1].record()
        barrier()
        gc.enable()
        ms = events[0].elapsed_time(events[-1])
        per_step = torch.tensor([events[i].elapsed_time(events[i + 1]) for i in range(args.steps)], device=device,
                                dtype=torch.float64)
        if world > 1:
            t = torch.tensor([ms], device=device)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
            dist.all_reduce(per_step, op=dist.ReduceOp.MAX)
        per_step = sorted(float(x) for x in per_step.tolist())

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

    # ---- parity of the last timed step (outside the timed region, every N)
    parity = None
    if args.config == 2:
        try:
            raw = {"a": _tensor(dev[id(w.keys[0])], torch.int32), "b": _tensor(dev[id(w.keys[1])], torch.int32),
                   "v": _tensor(dev[id(w.requests[0][0])], torch.float32),
                   "valid": torch.from_numpy(w.requests[0][0].valid()).to(device)}
            parity = parity_c2(raw, out)
        except Exception as e:
            parity = {"ok": False, "error": f"{type(e).__name__}: {e}"}

    total_rows = w.rows * world
    value = total_rows * args.steps / (ms / 1e3)
    e2e_value = total_rows * e2e_steps / (e2e_ms / 1e3)
    in_bytes = w.input_bytes()
    out_bytes = workloads.output_bytes(w, groups)
    del dev, keys, reqs, filt, out, pin
    torch.cuda.empty_cache()

    # ---- the skewed 1B-row configuration, rows split over the ranks (every N), then the other configs (N = 1)
    c4 = None
    if not args.no_c4:
        try:
            c4 = run_c4_strong(world, rank, device, 5, args.reuse_groupby)
            if args.reuse_groupby is False and world > 1 and args.c4_reuse_too:
                c4["reused_groupby"] = run_c4_strong(world, rank, device, 5, True)
        except Exception as e:
            c4 = {"error": f"{type(e).__name__}: {e}"}
        torch.cuda.empty_cache()
    c3 = None
    if world > 1 and not args.no_c4:
        try:
            c3 = run_c3_strong(world, rank, device, 5)
        except Exception as e:
            c3 = {"error": f"{type(e).__name__}: {e}"}
        torch.cuda.empty_cache()

    if rank == 0:
        peak, peak_kind = measured_peak()
        alg_bytes = in_bytes + out_bytes
        kms = statistics.mean(kernel_ms) if kernel_ms else float("nan")
        achieved = alg_bytes / (kms / 1e3) / 1e9 if kms and kms > 0 else None
        line = {
            "metric": METRIC, "value": value, "unit": "rows/s", "n_gpus": world, "steps": args.steps,
            "warmup": warmup, "ms_per_step": ms / args.steps, "ms_per_step_min": per_step[0],
            "ms_per_step_median": per_step[len(per_step) // 2], "ms_per_step_max": per_step[-1],
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32->f64", "data": "synthetic",
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
                         "traffic_source": C2_TRAFFIC_SOURCE if args.config == 2 else None,
                         "kernel": "k_aggregate_lean" if args.config == 2 else "k_aggregate", "kernel_ms": kms,
                         "peak_kind": f"of {peak_kind}",
                         "step_GBps": alg_bytes / (ms / args.steps / 1e3) / 1e9},
            "parity": parity,
            "c4_strong": c4,
        }
        if c3 is not None:
            line["c3_strong"] = c3
        if world == 1 and not args.no_configs:
            # C4 at full size on one GPU is the c4_strong entry above
            line["configs"] = run_other_configs(peak, (1, 5, 3) if c4 and "error" not in c4 else (1, 5, 3, 4))
        if world == 1 and not args.no_cpu_baseline:
            sample_rows = min(w.rows, 50_000_000)
            ws = workloads.make(args.config, sample_rows) if sample_rows != w.rows else w
            pv, psecs = oracle_rows_per_s(ws, os.cpu_count() or 1)
            base = {"port_value": pv, "port_cores": os.cpu_count() or 1,
                    "port_note": f"C++ restatement of the reference's rules on every host thread, {psecs:.1f} s"}
            if pandas_version() is not None:
                v, secs, pg = pandas_rows_per_s(ws)
                base.update({"value": v, "unit": "rows/s", "cores": 1, "kind": "reference",
                             "engine": f"pandas {pandas_version()} (the CPU path of cudf.pandas), single-threaded; "
                                       f"{os.cpu_count()} cores on the host",
                             "sample": f"{sample_rows} rows of the same workload, one run of {secs:.1f} s, {pg} groups"})
            else:
                v1, s1 = oracle_rows_per_s(ws, 1)
                base.update({"value": v1, "unit": "rows/s", "cores": 1, "kind": "port",
                             "sample": f"{sample_rows} rows of the same workload, one run of {s1:.1f} s, single-thread oracle"})
            line["cpu_baseline"] = base
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
    ap.add_argument("--c4-reuse-too", action="store_true", help="N > 1: also report c4_strong with a reused object")
    ap.add_argument("--table-variant", type=int, default=0,
                    help="N = 1: the engine's table_variant option for the resident steps (0 = auto; see include/b2_groupby.h)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-configs", action="store_true", help="skip the full-size C1/C3/C4/C5 block (N = 1)")
    ap.add_argument("--no-c4", action="store_true", help="skip the c4_strong block")
    args = ap.parse_args()
    if args.rows <= 0:
        args.rows = workloads.FULL_ROWS[args.config]
    if args.impl == "reference":
        run_reference(args)
    else:
        run_b2(args)


if __name__ == "__main__":
    main()
