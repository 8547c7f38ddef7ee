"""The benchmark configurations at their FULL benchmark sizes on one B200, inputs generated on the
device (seeded torch generators), checked against an independent sort-based computation in torch
(exact for integers) and through size-independent properties (group count, Σ counts, Σ sums,
min <= mean <= max, idempotence of re-aggregating the result)."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _mask_words(valid):
    """bool tensor -> cudf bitmask words (int32 tensor), LSB first."""
    import torch
    n = valid.numel()
    pad = (-n) % 32
    v = torch.cat([valid, torch.zeros(pad, dtype=torch.bool, device=valid.device)]) if pad else valid
    w = (v.view(-1, 32).to(torch.int64) << torch.arange(32, device=valid.device, dtype=torch.int64)).sum(1)
    w = torch.where(w >= 2**31, w - 2**32, w).to(torch.int32)
    return torch.cat([w, torch.zeros(16, dtype=torch.int32, device=valid.device)])


def _agg(keys, reqs, **opts):
    import cudf_b200 as cb
    gb = cb.GroupBy(cb.Table(keys), **opts)
    out_keys, out = gb.aggregate(reqs)
    return out_keys, out, cb.last_call_stats()


def _typed(col, dtype):
    return col.data[: col.size * dtype.itemsize].view(dtype) if hasattr(dtype, "itemsize") else None


def _tensor(col, torch_dtype):
    import torch
    nbytes = col.size * torch.empty(0, dtype=torch_dtype).element_size()
    return col.data[:nbytes].view(torch_dtype)


def test_c2_full_size_100m_rows():
    import torch
    import cudf_b200 as cb
    from cudf_b200 import aggregation as agg
    g = torch.Generator(device="cuda").manual_seed(44)
    n = 100_000_000
    a = torch.randint(0, 100, (n,), device="cuda", dtype=torch.int32, generator=g)
    b = torch.randint(0, 100, (n,), device="cuda", dtype=torch.int32, generator=g)
    v = torch.rand(n, device="cuda", generator=g) * 1000
    valid = torch.rand(n, device="cuda", generator=g) >= 0.02
    mask = _mask_words(valid)
    vc = cb.Column.from_tensor(v, mask)
    keys, out, st = _agg([cb.Column.from_tensor(a), cb.Column.from_tensor(b)],
                         [cb.GroupByRequest(vc, [agg.mean(), agg.count(), agg.sum()])], row_filters=[vc])
    assert st.used_shared_table and st.table_attempts == 1
    G = keys.num_rows()
    assert G == 10_000
    ka, kb = _tensor(keys.columns()[0], torch.int32), _tensor(keys.columns()[1], torch.int32)
    gid = (ka.to(torch.int64) * 100 + kb.to(torch.int64))
    assert torch.unique(gid).numel() == G
    mean, cnt, s = (_tensor(out[0].columns()[i], t) for i, t in enumerate((torch.float64, torch.int32, torch.float32)))
    assert int(cnt.sum()) == int(valid.sum())
    # independent computation: dense bincount in fp64
    rid = a.to(torch.int64) * 100 + b.to(torch.int64)
    ref_sum = torch.zeros(10_000, dtype=torch.float64, device="cuda").index_add_(0, rid[valid], v[valid].double())
    ref_cnt = torch.bincount(rid[valid], minlength=10_000)
    order = torch.argsort(gid)
    assert torch.equal(cnt[order].to(torch.int64), ref_cnt)
    ref_mean = ref_sum / ref_cnt
    assert float(((mean[order] - ref_mean).abs() / ref_mean.abs()).max()) < 1e-5   # fp32 source tolerance
    assert float(((s[order].double() - ref_sum).abs() / ref_sum.abs()).max()) < 1e-5


def test_c3_full_size_500m_rows_bit_exact():
    import torch
    import cudf_b200 as cb
    from cudf_b200 import aggregation as agg
    g = torch.Generator(device="cuda").manual_seed(45)
    n = 500_000_000
    k = torch.randint(0, 100_000_000, (n,), device="cuda", dtype=torch.int64, generator=g)
    v = torch.randint(-1_000_000_000, 1_000_000_001, (n,), device="cuda", dtype=torch.int64, generator=g)
    keys, out, st = _agg([cb.Column.from_tensor(k)],
                         [cb.GroupByRequest(cb.Column.from_tensor(v), [agg.sum(), agg.min(), agg.max(), agg.count()])])
    G = keys.num_rows()
    ok = _tensor(keys.columns()[0], torch.int64)
    s, mn, mx = (_tensor(out[0].columns()[i], torch.int64) for i in range(3))
    cnt = _tensor(out[0].columns()[3], torch.int32)
    # properties
    assert int(cnt.sum()) == n
    assert int(s.sum()) == int(v.sum())
    assert bool((mn <= mx).all())
    # exact check against a sort-based computation on a slice of the key space (bounded memory)
    sel = k < 5_000_000
    ks, vs = k[sel], v[sel]
    uk, inv = torch.unique(ks, return_inverse=True)
    ref_sum = torch.zeros(uk.numel(), dtype=torch.int64, device="cuda").index_add_(0, inv, vs)
    ref_cnt = torch.bincount(inv, minlength=uk.numel())
    ref_min = torch.full((uk.numel(),), 2**62, dtype=torch.int64, device="cuda").scatter_reduce_(0, inv, vs, "amin")
    ref_max = torch.full((uk.numel(),), -2**62, dtype=torch.int64, device="cuda").scatter_reduce_(0, inv, vs, "amax")
    osel = ok < 5_000_000
    order = torch.argsort(ok[osel])
    assert torch.equal(ok[osel][order], uk)
    assert torch.equal(s[osel][order], ref_sum)
    assert torch.equal(cnt[osel][order].to(torch.int64), ref_cnt)
    assert torch.equal(mn[osel][order], ref_min) and torch.equal(mx[osel][order], ref_max)
    assert G == int(torch.unique(k).numel())


def test_c4_full_size_1b_rows_zipf():
    import torch
    import cudf_b200 as cb
    from cudf_b200 import aggregation as agg
    g = torch.Generator(device="cuda").manual_seed(46)
    n, distinct = 1_000_000_000, 10_000_000
    w = torch.arange(1, distinct + 1, device="cuda", dtype=torch.float64) ** (-1.1)
    cdf = torch.cumsum(w, 0)
    cdf /= cdf[-1].clone()
    perm = torch.randperm(distinct, device="cuda", generator=g)
    k = torch.empty(n, dtype=torch.int64, device="cuda")
    chunk = 100_000_000
    for lo in range(0, n, chunk):
        u = torch.rand(chunk, device="cuda", dtype=torch.float64, generator=g)
        r = torch.searchsorted(cdf, u).clamp_(max=distinct - 1)
        k[lo:lo + chunk] = perm[r]
        del u, r
    v = torch.empty(n, dtype=torch.float64, device="cuda")
    v.log_normal_(0.0, 1.0, generator=g)
    valid = torch.rand(n, device="cuda", generator=g) >= 0.01
    mask = _mask_words(valid)
    keys, out, st = _agg([cb.Column.from_tensor(k)],
                         [cb.GroupByRequest(cb.Column.from_tensor(v, mask), [agg.sum(), agg.mean(), agg.variance(), agg.count()])])
    G = keys.num_rows()
    ok = _tensor(keys.columns()[0], torch.int64)
    s, mean, var = (_tensor(out[0].columns()[i], torch.float64) for i in range(3))
    cnt = _tensor(out[0].columns()[3], torch.int32)
    assert torch.unique(ok).numel() == G
    assert int(cnt.sum()) == int(valid.sum())
    total = float(torch.where(valid, v, torch.zeros_like(v)).sum())
    smask = ~torch.isnan(s)
    nullmask_s = out[0].columns()[0].mask
    got_total = float(s[cnt > 0].sum())
    assert abs(got_total - total) <= 1e-9 * total
    # independent per-group computation (dense by id, fp64 atomics in torch)
    ref_sum = torch.zeros(distinct, dtype=torch.float64, device="cuda").index_add_(0, k[valid], v[valid])
    ref_sq = torch.zeros(distinct, dtype=torch.float64, device="cuda").index_add_(0, k[valid], v[valid] ** 2)
    ref_cnt = torch.bincount(k[valid], minlength=distinct)
    has = cnt > 0
    kk = ok[has]
    assert torch.equal(cnt[has].to(torch.int64), ref_cnt[kk])
    rel = ((s[has] - ref_sum[kk]).abs() / ref_sum[kk]).max()
    assert float(rel) < 1e-11
    many = has & (cnt > 1)
    km = ok[many]
    c = ref_cnt[km].double()
    ref_var = (ref_sq[km] - ref_sum[km] ** 2 / c) / (c - 1)
    scale = ref_sq[km] / (c - 1)
    assert float(((var[many] - ref_var).abs() / scale).max()) < 1e-11
    assert float(((mean[has] - ref_sum[kk] / ref_cnt[kk]).abs() / mean[has]).max()) < 1e-11


def test_c5_full_size_200m_rows_string_keys():
    import torch
    import cudf_b200 as cb
    from cudf_b200 import aggregation as agg
    from cudf_b200.types import TypeId
    g = torch.Generator(device="cuda").manual_seed(47)
    n, pool = 200_000_000, 1_000_000
    plen = torch.randint(8, 33, (pool,), device="cuda", generator=g)
    poff = torch.zeros(pool + 1, dtype=torch.int64, device="cuda")
    poff[1:] = torch.cumsum(plen, 0)
    alphabet = torch.tensor(list(b"abcdefghijklmnopqrstuvwxyz0123456789"), dtype=torch.uint8, device="cuda")
    pchars = alphabet[torch.randint(0, 36, (int(poff[-1]),), device="cuda", generator=g)]
    idx = torch.randint(0, pool, (n,), device="cuda", generator=g)
    lens = plen[idx]
    offs = torch.zeros(n + 1, dtype=torch.int64, device="cuda")
    offs[1:] = torch.cumsum(lens, 0)
    total = int(offs[-1])
    assert total > 2**31  # forces INT64 offsets, like the reference's large-strings mode
    chars = torch.empty(total, dtype=torch.uint8, device="cuda")
    chunk = 20_000_000
    for lo in range(0, n, chunk):
        hi = min(n, lo + chunk)
        b0, b1 = int(offs[lo]), int(offs[hi])
        src = torch.repeat_interleave(poff[idx[lo:hi]] - offs[lo:hi], lens[lo:hi]) + torch.arange(b0, b1, device="cuda")
        chars[b0:b1] = pchars[src]
        del src
    k2 = torch.randint(0, 16, (n,), device="cuda", dtype=torch.int32, generator=g)
    v1 = 100.0 + 15.0 * torch.randn(n, device="cuda", dtype=torch.float64, generator=g)
    v2 = torch.randint(0, 1_000_000, (n,), device="cuda", dtype=torch.int32, generator=g)
    val1 = torch.rand(n, device="cuda", generator=g) >= 0.03
    val2 = torch.rand(n, device="cuda", generator=g) >= 0.03
    scol = cb.Column(TypeId.STRING, n, chars, None, 0, 0, offs.view(torch.uint8), TypeId.INT64)
    aggs = [agg.sum(), agg.count(), agg.mean(), agg.min(), agg.max()]
    keys, out, st = _agg([scol, cb.Column.from_tensor(k2)],
                         [cb.GroupByRequest(cb.Column.from_tensor(v1, _mask_words(val1)), aggs),
                          cb.GroupByRequest(cb.Column.from_tensor(v2, _mask_words(val2)), aggs)])
    G = keys.num_rows()
    gid = idx * 16 + k2.to(torch.int64)
    assert G == int(torch.unique(gid).numel())
    c1 = _tensor(out[0].columns()[1], torch.int32)
    c2 = _tensor(out[1].columns()[1], torch.int32)
    assert int(c1.sum()) == int(val1.sum()) and int(c2.sum()) == int(val2.sum())
    s2 = _tensor(out[1].columns()[0], torch.int64)
    assert int(s2[c2 > 0].sum()) == int(v2[val2].to(torch.int64).sum())
    mn1, mx1, mean1 = (_tensor(out[0].columns()[i], torch.float64) for i in (3, 4, 2))
    h = c1 > 0
    assert bool((mn1[h] <= mean1[h] + 1e-9).all()) and bool((mean1[h] <= mx1[h] + 1e-9).all())
    # output strings: offsets child is INT32 (16M keys x ~20 B < 2 GiB) and every key has length 8..32
    kcol = keys.columns()[0]
    ooffs = _tensor(type("C", (), {"data": kcol.offsets, "size": G + 1})(), torch.int32 if kcol.offsets_type == TypeId.INT32 else torch.int64)
    ol = ooffs[1:] - ooffs[:-1]
    assert int(ol.min()) >= 8 and int(ol.max()) <= 32
