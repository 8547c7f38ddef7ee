"""The benchmark configurations at their FULL benchmark sizes on one B200, inputs generated on the
device (workloads.make_device: seeded torch generators), every group checked against an
independent computation in torch (index_add / bincount / scatter_reduce over the generating
tensors: exact for integers, fp64 for floats) plus size-independent properties (group count,
Σ counts, Σ sums, min <= mean <= max)."""
import pytest

import workloads
from cudf_b200.types import Kind

pytestmark = pytest.mark.gpu


def _agg(w, extra=None, **opts):
    import cudf_b200 as cb
    from cudf_b200.aggregation import Aggregation
    reqs = [cb.GroupByRequest(v, [Aggregation(Kind(a)) for a in (extra[i] if extra else aggs)])
            for i, (v, aggs) in enumerate(w.requests)]
    gb = cb.GroupBy(cb.Table(w.keys), row_filters=w.row_filters, **opts)
    out_keys, out = gb.aggregate(reqs)
    return out_keys, out, cb.last_call_stats()


def _tensor(col, torch_dtype):
    import torch
    nbytes = col.size * torch.empty(0, dtype=torch_dtype).element_size()
    return col.data[:nbytes].view(torch_dtype)


@pytest.mark.parametrize("variant", [0, 5])
def test_c2_full_size_100m_rows(variant):
    """variant 0: tiles through registers; 5: through the bulk-copy shared-memory ring."""
    import torch
    w = workloads.make_device(2)
    a, b, v, valid = (w.raw[k] for k in ("a", "b", "v", "valid"))
    keys, out, st = _agg(w, extra=[[Kind.MEAN, Kind.COUNT_VALID, Kind.SUM]], table_variant=variant)
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
    w = workloads.make_device(3)
    n, k, v = w.rows, w.raw["k"], w.raw["v"]
    keys, out, st = _agg(w)
    G = keys.num_rows()
    ok = _tensor(keys.columns()[0], torch.int64)
    s, mn, mx = (_tensor(out[0].columns()[i], torch.int64) for i in range(3))
    cnt = _tensor(out[0].columns()[3], torch.int32)
    # properties
    assert int(cnt.sum()) == n
    assert int(s.sum()) == int(v.sum())
    assert bool((mn <= mx).all())
    # every group, exactly, against dense references over the key domain [0, 100M)
    dom = 100_000_000
    ref_cnt = torch.bincount(k, minlength=dom)
    assert G == int((ref_cnt > 0).sum())
    assert torch.equal(cnt.to(torch.int64), ref_cnt[ok])
    del ref_cnt
    ref = torch.zeros(dom, dtype=torch.int64, device="cuda").index_add_(0, k, v)
    assert torch.equal(s, ref[ok])
    ref.fill_(2**62).scatter_reduce_(0, k, v, "amin")
    assert torch.equal(mn, ref[ok])
    ref.fill_(-2**62).scatter_reduce_(0, k, v, "amax")
    assert torch.equal(mx, ref[ok])
    assert torch.unique(ok).numel() == G


def test_c4_full_size_1b_rows_zipf():
    import torch
    w = workloads.make_device(4)
    k, v, valid, distinct = (w.raw[x] for x in ("k", "v", "valid", "distinct"))
    keys, out, st = _agg(w, extra=[[Kind.SUM, Kind.MEAN, Kind.VARIANCE, Kind.COUNT_VALID]])
    G = keys.num_rows()
    ok = _tensor(keys.columns()[0], torch.int64)
    s, mean, var = (_tensor(out[0].columns()[i], torch.float64) for i in range(3))
    cnt = _tensor(out[0].columns()[3], torch.int32)
    assert torch.unique(ok).numel() == G
    assert G == int(torch.bincount(k, minlength=distinct).clamp_(max=1).sum())
    assert int(cnt.sum()) == int(valid.sum())
    total = float(torch.where(valid, v, torch.zeros_like(v)).sum())
    got_total = float(s[cnt > 0].sum())
    assert abs(got_total - total) <= 1e-9 * total
    # independent per-group computation (dense by id, fp64 atomics in torch)
    ref_sum = torch.zeros(distinct, dtype=torch.float64, device="cuda").index_add_(0, k[valid], v[valid])
    ref_sq = torch.zeros(distinct, dtype=torch.float64, device="cuda").index_add_(0, k[valid], v[valid] ** 2)
    ref_cnt = torch.bincount(k[valid], minlength=distinct)
    has = cnt > 0
    kk = ok[has]
    assert torch.equal(cnt.to(torch.int64), ref_cnt[ok])
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
    """Every group: the output string equals the pool string of its id, and Σ, n, min, max of both value
    columns (int32 exact, float64 to 1e-12 of the group's Σ|x| scale — all values are positive here, so that is
    the strict relative error) against scatter references keyed on (pool id, k2)."""
    import torch
    from cudf_b200.types import TypeId
    w = workloads.make_device(5)
    n = w.rows
    idx, k2, v1, v2, val1, val2 = (w.raw[x] for x in ("idx", "k2", "v1", "v2", "val1", "val2"))
    pchars, poff = w.raw["pool_chars"], w.raw["pool_offsets"]
    assert w.keys[0].offsets_type == TypeId.INT64   # > 2 GiB of chars: the reference's large-strings mode
    keys, out, st = _agg(w)
    G = keys.num_rows()
    gid_in = idx * 16 + k2.to(torch.int64)
    dom = 16_000_000
    present = torch.bincount(gid_in, minlength=dom)
    assert G == int((present > 0).sum())
    del present
    # ---- identify every output group: the pool id of its string by (length, 64-bit polynomial hash), then verify bytes
    kcol = keys.columns()[0]
    odt = torch.int32 if kcol.offsets_type == TypeId.INT32 else torch.int64
    ooffs = kcol.offsets[: (G + 1) * (4 if odt == torch.int32 else 8)].view(odt).to(torch.int64)
    olen = ooffs[1:] - ooffs[:-1]
    assert int(olen.min()) >= 8 and int(olen.max()) <= 32

    def poly_hash(chars, offs):
        lens = offs[1:] - offs[:-1]
        h = torch.zeros(lens.numel(), dtype=torch.int64, device="cuda")
        for j in range(32):
            take = lens > j
            c = chars[(offs[:-1] + j).clamp_(max=chars.numel() - 1)].to(torch.int64)
            h = torch.where(take, h * 1000003 + c + 1, h)
        return h * 64 + lens
    ph = poly_hash(pchars, poff)
    sorted_ph, pid_of = torch.sort(ph)
    oh = poly_hash(kcol.data, ooffs)
    pos = torch.searchsorted(sorted_ph, oh).clamp_(max=sorted_ph.numel() - 1)
    assert torch.equal(sorted_ph[pos], oh)          # every output string's hash is a pool string's hash
    pid = pid_of[pos]
    # bytes equal (guards against hash collisions and against a wrong pool id among equal hashes of equal strings)
    plen = poff[1:] - poff[:-1]
    assert torch.equal(plen[pid], olen)
    for j in range(32):
        take = olen > j
        a = kcol.data[(ooffs[:-1] + j)[take]]
        b = pchars[(poff[:-1][pid] + j)[take]]
        assert torch.equal(a, b)
    ok2 = _tensor(keys.columns()[1], torch.int32).to(torch.int64)
    # pool strings may repeat (random 8-char strings collide with negligible probability, but be exact):
    # map every input pool id to the FIRST pool id holding the same string
    first_of = torch.empty_like(pid_of)
    uniq_h, inv = torch.unique(ph, return_inverse=True)
    first = torch.full((uniq_h.numel(),), ph.numel(), dtype=torch.int64, device="cuda").scatter_reduce_(
        0, inv, torch.arange(ph.numel(), device="cuda"), "amin")
    first_of = first[inv]
    gid_out = first_of[pid] * 16 + ok2
    gid_in = first_of[idx] * 16 + k2.to(torch.int64)
    assert torch.unique(gid_out).numel() == G
    # ---- value columns
    s1, c1, m1, mn1, mx1 = (_tensor(out[0].columns()[i], t) for i, t in
                            enumerate((torch.float64, torch.int32, torch.float64, torch.float64, torch.float64)))
    s2, c2, m2, mn2, mx2 = (_tensor(out[1].columns()[i], t) for i, t in
                            enumerate((torch.int64, torch.int32, torch.float64, torch.int32, torch.int32)))
    assert int(c1.sum()) == int(val1.sum()) and int(c2.sum()) == int(val2.sum())
    # int32 column: exact
    g2, x2 = gid_in[val2], v2[val2].to(torch.int64)
    ref = torch.bincount(g2, minlength=dom)
    assert torch.equal(c2.to(torch.int64), ref[gid_out])
    h2 = c2 > 0
    ref = torch.zeros(dom, dtype=torch.int64, device="cuda").index_add_(0, g2, x2)
    assert torch.equal(s2[h2], ref[gid_out][h2])
    ref_sum2 = ref[gid_out][h2].double()
    ref.fill_(2**40).scatter_reduce_(0, g2, x2, "amin")
    assert torch.equal(mn2[h2].to(torch.int64), ref[gid_out][h2])
    ref.fill_(-1).scatter_reduce_(0, g2, x2, "amax")
    assert torch.equal(mx2[h2].to(torch.int64), ref[gid_out][h2])
    assert float(((m2[h2] - ref_sum2 / c2[h2]).abs() / m2[h2].abs().clamp_(min=1e-300)).max()) < 1e-12
    del ref, g2, x2
    # float64 column: 1e-12 (values ~N(100, 15): sums do not cancel)
    g1, x1 = gid_in[val1], v1[val1]
    refc = torch.bincount(g1, minlength=dom)
    assert torch.equal(c1.to(torch.int64), refc[gid_out])
    h1 = c1 > 0
    reff = torch.zeros(dom, dtype=torch.float64, device="cuda").index_add_(0, g1, x1)
    rs = reff[gid_out][h1]
    assert float(((s1[h1] - rs).abs() / rs.abs()).max()) < 1e-12
    assert float(((m1[h1] - rs / c1[h1]).abs() / m1[h1].abs()).max()) < 1e-12
    reff.fill_(float("inf")).scatter_reduce_(0, g1, x1, "amin")
    assert torch.equal(mn1[h1], reff[gid_out][h1])
    reff.fill_(float("-inf")).scatter_reduce_(0, g1, x1, "amax")
    assert torch.equal(mx1[h1], reff[gid_out][h1])
    assert bool((mn1[h1] <= m1[h1] + 1e-9).all()) and bool((m1[h1] <= mx1[h1] + 1e-9).all())
