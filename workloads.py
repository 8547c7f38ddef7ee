"""Seeded synthetic inputs of the five benchmark configurations (C1-C5 of the benchmark specification).

No public dataset is involved: these generators ARE the workloads.  Every generator is
counter-seeded (seed = 42 + config index, optionally + rank) and produces Arrow-layout host columns
(numpy) so that the CUDA engine and the CPU oracle read identical bytes.  ``n`` scales a config
down for parity tests; the distributions stay the same.

  C1  key int64 U[0,1000); value f64 N(0,1), 5 % nulls; sum, count, mean
  C2  keys (int32 U[0,100), int32 U[0,100)); value f32 U(0,1000), 2 % nulls; dropna() then mean
  C3  key int64 U[0,100M); value int64 U[-1e9,1e9]; sum, min, max, count
  C4  key int64 Zipf(s=1.1) over 10M ids; value f64 LogNormal(0,1), 1 % nulls; sum, mean, var
  C5  keys (string len U{8..32} from a pool of 1M, int32 U[0,16)); values f64 N(100,15) and
      int32 U[0,1e6), 3 % nulls each; sum, count, mean, min, max on both
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import List, Sequence, Tuple

import numpy as np

from cudf_b200.types import HostColumn, Kind, NullPolicy, TypeId, pack_mask

FULL_ROWS = {1: 10_000_000, 2: 100_000_000, 3: 500_000_000, 4: 1_000_000_000, 5: 200_000_000}


@dataclass
class Workload:
    name: str
    keys: List[HostColumn]
    requests: List[Tuple[HostColumn, Sequence]]
    null_policy: NullPolicy = NullPolicy.EXCLUDE
    row_filters: List[HostColumn] = field(default_factory=list)  # fused dropna(): columns whose nulls drop the row
    rows: int = 0

    def input_bytes(self) -> int:
        """Algorithmic input bytes: keys + values + validity bitmasks, each read once."""
        total = 0
        seen = set()
        for c in self.keys + [v for v, _ in self.requests]:
            if id(c) in seen:
                continue
            seen.add(id(c))
            if c.type_id == TypeId.STRING:
                total += int(c.offsets[-1]) + c.offsets.itemsize * (c.size + 1)
            else:
                total += c.size * c.data.itemsize
            if c.mask is not None:
                total += (c.size + 7) // 8
        return total


def _valid(rng, n, null_frac):
    return rng.random(n) >= null_frac


def zipf_keys(rng, n: int, distinct: int, s: float = 1.1) -> np.ndarray:
    """Zipf(s) over ranks 1..distinct by inverse CDF, ranks mapped to ids by a seeded permutation."""
    w = np.arange(1, distinct + 1, dtype=np.float64) ** (-s)
    cdf = np.cumsum(w)
    cdf /= cdf[-1]
    ranks = np.searchsorted(cdf, rng.random(n), side="left").astype(np.int64)
    np.minimum(ranks, distinct - 1, out=ranks)
    ids = rng.permutation(distinct).astype(np.int64)
    return ids[ranks]


def string_pool(rng, pool: int):
    """``pool`` distinct-ish random [a-z0-9] strings, length uniform in 8..32: (chars, offsets)."""
    alphabet = np.frombuffer(b"abcdefghijklmnopqrstuvwxyz0123456789", dtype=np.uint8)
    lens = rng.integers(8, 33, pool).astype(np.int64)
    offs = np.zeros(pool + 1, dtype=np.int64)
    np.cumsum(lens, out=offs[1:])
    chars = alphabet[rng.integers(0, 36, int(offs[-1]))]
    return chars, offs


def gather_strings(chars: np.ndarray, offs: np.ndarray, idx: np.ndarray, large_offsets: bool) -> HostColumn:
    lens = (offs[1:] - offs[:-1])[idx]
    out_offs = np.zeros(idx.size + 1, dtype=np.int64)
    np.cumsum(lens, out=out_offs[1:])
    total = int(out_offs[-1])
    # position of every output byte inside the pool
    src = np.repeat(offs[:-1][idx] - out_offs[:-1], lens) + np.arange(total, dtype=np.int64)
    out_chars = chars[src]
    return HostColumn(TypeId.STRING, idx.size, out_chars, None, 0,
                      out_offs if large_offsets else out_offs.astype(np.int32))


def make(config: int, n: int = 0, rank: int = 0, scale_domain: bool = False) -> Workload:
    """Workload of configuration ``config`` (1..5) with ``n`` rows (0 = full size).

    ``scale_domain`` shrinks the key domain with n (same rows-per-group ratio as the full config);
    otherwise the full-size key domain is kept, so a small n sees proportionally more groups."""
    full = FULL_ROWS[config]
    n = n or full
    rng = np.random.default_rng([42 + config, rank])
    ratio = n / full if scale_domain else 1.0
    if config == 1:
        k = HostColumn.from_numpy(rng.integers(0, max(2, int(1000 * ratio)), n).astype(np.int64))
        v = HostColumn.from_numpy(rng.standard_normal(n), valid=_valid(rng, n, 0.05))
        return Workload("C1", [k], [(v, [Kind.SUM, Kind.COUNT_VALID, Kind.MEAN])], rows=n)
    if config == 2:
        dom = max(2, int(round(100 * ratio ** 0.5)))
        a = HostColumn.from_numpy(rng.integers(0, dom, n).astype(np.int32))
        b = HostColumn.from_numpy(rng.integers(0, dom, n).astype(np.int32))
        v = HostColumn.from_numpy((rng.random(n) * 1000).astype(np.float32), valid=_valid(rng, n, 0.02))
        # df.dropna().groupby(["A","B"]).mean(): rows with a null anywhere are dropped first
        return Workload("C2", [a, b], [(v, [Kind.MEAN])], row_filters=[v], rows=n)
    if config == 3:
        k = HostColumn.from_numpy(rng.integers(0, max(2, int(100_000_000 * ratio)), n).astype(np.int64))
        v = HostColumn.from_numpy(rng.integers(-1_000_000_000, 1_000_000_001, n).astype(np.int64))
        return Workload("C3", [k], [(v, [Kind.SUM, Kind.MIN, Kind.MAX, Kind.COUNT_VALID])], rows=n)
    if config == 4:
        k = HostColumn.from_numpy(zipf_keys(rng, n, max(2, int(10_000_000 * ratio))))
        v = HostColumn.from_numpy(rng.lognormal(0.0, 1.0, n), valid=_valid(rng, n, 0.01))
        return Workload("C4", [k], [(v, [Kind.SUM, Kind.MEAN, Kind.VARIANCE])], rows=n)
    if config == 5:
        pool = max(2, int(1_000_000 * ratio))
        chars, offs = string_pool(np.random.default_rng([42 + config, 777]), pool)
        idx = rng.integers(0, pool, n)
        s = gather_strings(chars, offs, idx, large_offsets=n >= 100_000_000)
        k2 = HostColumn.from_numpy(rng.integers(0, 16, n).astype(np.int32))
        v1 = HostColumn.from_numpy(100.0 + 15.0 * rng.standard_normal(n), valid=_valid(rng, n, 0.03))
        v2 = HostColumn.from_numpy(rng.integers(0, 1_000_000, n).astype(np.int32), valid=_valid(rng, n, 0.03))
        aggs = [Kind.SUM, Kind.COUNT_VALID, Kind.MEAN, Kind.MIN, Kind.MAX]
        return Workload("C5", [s, k2], [(v1, aggs), (v2, aggs)], rows=n)
    raise ValueError(f"unknown config {config}")


def output_bytes(w: Workload, groups: int) -> int:
    """Algorithmic output bytes: one key row and one result element per aggregation per group."""
    from cudf_b200.types import result_type, type_width
    per = 0
    for k in w.keys:
        per += 28 if k.type_id == TypeId.STRING else k.data.itemsize  # ≈20 B chars + 8 B offset
    for v, aggs in w.requests:
        for a in aggs:
            kind = a[0] if isinstance(a, tuple) else a
            per += type_width(result_type(v.type_id, kind))
    return groups * per


# ------------------------------------------------------------------------------------ device side
# The same five configurations generated on the GPU with seeded torch generators (full sizes take
# seconds instead of minutes, and the host never holds the 16 GB of C4).  The distributions are the
# ones above; the streams differ from the numpy ones, so a device workload is checked against
# computations on its own tensors, never against a host workload of the same seed.
def mask_words(valid):
    """bool tensor -> cudf bitmask words (int32 tensor, LSB first), padded by 64 bytes."""
    import torch
    n = valid.numel()
    pad = (-n) % 32
    v = torch.cat([valid, torch.zeros(pad, dtype=torch.bool, device=valid.device)]) if pad else valid
    w = (v.view(-1, 32).to(torch.int64) << torch.arange(32, device=valid.device, dtype=torch.int64)).sum(1)
    w = torch.where(w >= 2**31, w - 2**32, w).to(torch.int32)
    return torch.cat([w, torch.zeros(16, dtype=torch.int32, device=valid.device)])


@dataclass
class DeviceWorkload:
    name: str
    rows: int
    keys: list                      # cudf_b200.Column
    requests: list                  # (cudf_b200.Column, [Kind, ...])
    row_filters: list = field(default_factory=list)
    raw: dict = field(default_factory=dict)   # the generating tensors, for independent checks
    input_bytes: int = 0            # keys + values + validity bitmasks, each read once

    def groupby_requests(self):
        import cudf_b200 as cb
        from cudf_b200.aggregation import Aggregation
        return [cb.GroupByRequest(v, [Aggregation(Kind(a)) for a in aggs]) for v, aggs in self.requests]


def make_device(config: int, n: int = 0, device="cuda", rank: int = 0) -> DeviceWorkload:
    """Configuration ``config`` (1..5) with ``n`` rows (0 = full size) generated on ``device``;
    seed = 42 + config (+ 1000 * rank), like the host generators."""
    import torch
    import cudf_b200 as cb
    n = n or FULL_ROWS[config]
    g = torch.Generator(device=device).manual_seed(42 + config + 1000 * rank)
    col = cb.Column.from_tensor

    def nullable(t, frac):
        valid = torch.rand(n, device=device, generator=g) >= frac
        c = col(t, mask_words(valid))
        return c, valid

    if config == 1:
        k = torch.randint(0, 1000, (n,), device=device, dtype=torch.int64, generator=g)
        v = torch.randn(n, device=device, dtype=torch.float64, generator=g)
        vc, valid = nullable(v, 0.05)
        return DeviceWorkload("C1", n, [col(k)], [(vc, [Kind.SUM, Kind.COUNT_VALID, Kind.MEAN])], [],
                              {"k": k, "v": v, "valid": valid}, n * 16 + (n + 7) // 8)
    if config == 2:
        a = torch.randint(0, 100, (n,), device=device, dtype=torch.int32, generator=g)
        b = torch.randint(0, 100, (n,), device=device, dtype=torch.int32, generator=g)
        v = torch.rand(n, device=device, generator=g) * 1000
        vc, valid = nullable(v, 0.02)
        return DeviceWorkload("C2", n, [col(a), col(b)], [(vc, [Kind.MEAN])], [vc],
                              {"a": a, "b": b, "v": v, "valid": valid}, n * 12 + (n + 7) // 8)
    if config == 3:
        k = torch.randint(0, 100_000_000, (n,), device=device, dtype=torch.int64, generator=g)
        v = torch.randint(-1_000_000_000, 1_000_000_001, (n,), device=device, dtype=torch.int64, generator=g)
        return DeviceWorkload("C3", n, [col(k)], [(col(v), [Kind.SUM, Kind.MIN, Kind.MAX, Kind.COUNT_VALID])], [],
                              {"k": k, "v": v}, n * 16)
    if config == 4:
        distinct = 10_000_000
        w = torch.arange(1, distinct + 1, device=device, dtype=torch.float64) ** (-1.1)
        cdf = torch.cumsum(w, 0)
        cdf /= cdf[-1].clone()
        # the id permutation is shared by all ranks (one key space), the draws are per rank
        perm = torch.randperm(distinct, device=device, generator=torch.Generator(device=device).manual_seed(42 + config))
        k = torch.empty(n, dtype=torch.int64, device=device)
        chunk = 100_000_000
        for lo in range(0, n, chunk):
            m = min(chunk, n - lo)
            u = torch.rand(m, device=device, dtype=torch.float64, generator=g)
            r = torch.searchsorted(cdf, u).clamp_(max=distinct - 1)
            k[lo:lo + m] = perm[r]
            del u, r
        del w, cdf, perm
        v = torch.empty(n, dtype=torch.float64, device=device)
        v.log_normal_(0.0, 1.0, generator=g)
        vc, valid = nullable(v, 0.01)
        return DeviceWorkload("C4", n, [col(k)], [(vc, [Kind.SUM, Kind.MEAN, Kind.VARIANCE])], [],
                              {"k": k, "v": v, "valid": valid, "distinct": distinct}, n * 16 + (n + 7) // 8)
    if config == 5:
        pool = 1_000_000
        gp = torch.Generator(device=device).manual_seed(42 + config + 777)   # the pool is shared by all ranks
        plen = torch.randint(8, 33, (pool,), device=device, generator=gp)
        poff = torch.zeros(pool + 1, dtype=torch.int64, device=device)
        poff[1:] = torch.cumsum(plen, 0)
        alphabet = torch.tensor(list(b"abcdefghijklmnopqrstuvwxyz0123456789"), dtype=torch.uint8, device=device)
        pchars = alphabet[torch.randint(0, 36, (int(poff[-1]),), device=device, generator=gp)]
        idx = torch.randint(0, pool, (n,), device=device, generator=g)
        lens = plen[idx]
        offs = torch.zeros(n + 1, dtype=torch.int64, device=device)
        offs[1:] = torch.cumsum(lens, 0)
        total = int(offs[-1])
        chars = torch.empty(total, dtype=torch.uint8, device=device)
        chunk = 20_000_000
        for lo in range(0, n, chunk):
            hi = min(n, lo + chunk)
            b0, b1 = int(offs[lo]), int(offs[hi])
            src = torch.repeat_interleave(poff[idx[lo:hi]] - offs[lo:hi], lens[lo:hi]) + torch.arange(b0, b1, device=device)
            chars[b0:b1] = pchars[src]
            del src
        large = total > 0x7FFFFFFF   # INT64 offsets beyond the reference's large-strings threshold
        o = offs if large else offs.to(torch.int32)
        scol = cb.Column(TypeId.STRING, n, chars, None, 0, 0, o.view(torch.uint8), TypeId.INT64 if large else TypeId.INT32)
        k2 = torch.randint(0, 16, (n,), device=device, dtype=torch.int32, generator=g)
        v1 = 100.0 + 15.0 * torch.randn(n, device=device, dtype=torch.float64, generator=g)
        v2 = torch.randint(0, 1_000_000, (n,), device=device, dtype=torch.int32, generator=g)
        c1, val1 = nullable(v1, 0.03)
        c2, val2 = nullable(v2, 0.03)
        aggs = [Kind.SUM, Kind.COUNT_VALID, Kind.MEAN, Kind.MIN, Kind.MAX]
        nbytes = total + (8 if large else 4) * (n + 1) + n * 4 + n * 8 + n * 4 + 2 * ((n + 7) // 8)
        return DeviceWorkload("C5", n, [scol, col(k2)], [(c1, aggs), (c2, aggs)], [],
                              {"idx": idx, "k2": k2, "v1": v1, "v2": v2, "val1": val1, "val2": val2,
                               "pool_chars": pchars, "pool_offsets": poff}, nbytes)
    raise ValueError(f"unknown config {config}")


def device_output_bytes(w: DeviceWorkload, groups: int, key_chars: int = 0) -> int:
    """Algorithmic output bytes of a device workload: key columns + one element per aggregation per group."""
    from cudf_b200.types import result_type, type_width
    per = 0
    for k in w.keys:
        per += 4 if k.type_id == TypeId.STRING else type_width(k.type_id)   # strings: offsets here, chars below
    for v, aggs in w.requests:
        for a in aggs:
            per += type_width(result_type(v.type_id, a))
    return groups * per + key_chars
