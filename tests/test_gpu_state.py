"""Partial-aggregate state (pack / merge / finalize), batch-wise updates and the row-level hash
partition on ONE GPU, emulating the ranks of a multi-GPU run: the merge of partials must equal a
one-shot groupby (the rules of cpp/tests/groupby/streaming_groupby_test.cpp:300,884,912,942)."""
import numpy as np
import pytest

import workloads
from cudf_b200.types import HostColumn, Kind, NullPolicy, TypeId
from oracle import oracle
from tests import helpers as H

pytestmark = pytest.mark.gpu


def _device_objects(keys, requests, policy, lo, hi, **opts):
    import cudf_b200 as cb
    from cudf_b200.aggregation import Aggregation

    def cut(c):
        valid = c.valid()[lo:hi] if c.mask is not None else None
        return HostColumn.from_numpy(c.values()[lo:hi], valid, type_id=c.type_id)

    dk = cb.Table([cb.Column.from_host(cut(k)) for k in keys])
    cache = {}
    reqs = []
    for v, aggs in requests:
        if id(v) not in cache:
            cache[id(v)] = cb.Column.from_host(cut(v))
        reqs.append(cb.GroupByRequest(cache[id(v)], [Aggregation(Kind(a[0]), a[1]) if isinstance(a, tuple)
                                                     else Aggregation(Kind(a)) for a in aggs]))
    return cb.GroupBy(dk, policy, **opts), reqs


def _to_host(res):
    okeys, ores = res
    return [c.to_host() for c in okeys.columns()], [[c.to_host() for c in t.columns()] for t in ores]


def _concat(parts):
    """Union of per-rank results (disjoint groups)."""
    keys = [HostColumn.from_numpy(np.concatenate([p[0][k].values() for p in parts]),
                                  np.concatenate([p[0][k].valid() for p in parts]) if parts[0][0][k].mask is not None else None,
                                  type_id=parts[0][0][k].type_id) for k in range(len(parts[0][0]))]
    res = []
    for q in range(len(parts[0][1])):
        row = []
        for a in range(len(parts[0][1][q])):
            cols = [p[1][q][a] for p in parts]
            valid = np.concatenate([c.valid() for c in cols]) if cols[0].mask is not None else None
            row.append(HostColumn.from_numpy(np.concatenate([c.values() for c in cols]), valid, type_id=cols[0].type_id))
        res.append(row)
    return keys, res


AGGS = [Kind.SUM, Kind.COUNT_VALID, Kind.COUNT_ALL, Kind.MEAN, Kind.MIN, Kind.MAX, Kind.VARIANCE, Kind.M2]


@pytest.mark.parametrize("ranks", [2, 4])
@pytest.mark.parametrize("config", [1, 2, 4])
def test_emulated_ranks_partials_shuffle_equals_one_shot(config, ranks):
    import cudf_b200 as cb
    n = 240_000
    w = workloads.make(config, n, scale_domain=(config == 4))
    reqs = [(v, AGGS) for v, _ in w.requests]
    filt = []  # row filters are per-shard views; leave them out of this emulation
    states, packed = [], []
    for r in range(ranks):
        gb, dreqs = _device_objects(w.keys, reqs, w.null_policy, r * n // ranks, (r + 1) * n // ranks)
        st = cb.GroupByState(gb, dreqs)
        st.update()
        records, counts = st.pack(ranks)
        assert sum(counts) == st.num_groups()
        packed.append((records, counts, st.record_bytes))
        states.append((st, gb, dreqs))
    parts = []
    for dst in range(ranks):
        st, gb, dreqs = states[dst]
        st.reset()
        for records, counts, rb in packed:
            start = sum(counts[:dst]) * rb
            st.merge(records[start:start + counts[dst] * rb], counts[dst])
        parts.append(_to_host(st.finalize()))
    got = _concat(parts)
    exp = oracle.groupby(w.keys, reqs, w.null_policy)
    H.assert_same_result(got, exp, reqs, scales=H.result_scales(w.keys, reqs, w.null_policy))
    # ownership is disjoint: no key on two ranks
    assert got[0][0].size == exp[0][0].size


def test_finishers_over_partial_columns():
    """b2_finish_partial against the same formulas in numpy: mean (FLOAT64, and a duration by integer division),
    M2, variance and standard deviation with their validity (n - ddof > 0), counts as INT32, the validity alone."""
    import cudf_b200 as cb
    from cudf_b200.partials import _finish
    rng = np.random.default_rng(12)
    n = 5000
    cnt = rng.integers(0, 6, n).astype(np.int64)
    x = [rng.standard_normal(c) * 10 for c in cnt]
    s = np.array([v.sum() for v in x])
    ss = np.array([(v * v).sum() for v in x])
    dev = lambda a, t=None: cb.Column.from_host(HostColumn.from_numpy(a, type_id=t))
    c_col, s_col, ss_col = dev(cnt), dev(s), dev(ss)
    mean = _finish(Kind.MEAN, 0, TypeId.FLOAT64, s_col, c_col, None, True).to_host()
    ok = cnt > 0
    assert np.array_equal(mean.valid(), ok) and mean.null_count == int((~ok).sum())
    assert np.allclose(mean.values()[ok], s[ok] / cnt[ok], rtol=1e-15, atol=0)
    for kind, ddof in ((Kind.M2, 0), (Kind.VARIANCE, 1), (Kind.VARIANCE, 0), (Kind.STD, 2)):
        got = _finish(kind, ddof, TypeId.FLOAT64, s_col, c_col, ss_col, True).to_host()
        m2 = np.where(ok, ss - s * s / np.maximum(cnt, 1), 0.0)
        if kind == Kind.M2:
            assert got.mask is None and np.allclose(got.values(), m2, rtol=1e-14, atol=1e-12)
            continue
        good = ok & (cnt - ddof > 0)
        var = m2[good] / (cnt[good] - ddof)
        assert np.array_equal(got.valid(), good) and got.null_count == int((~good).sum())
        assert np.allclose(got.values()[good], var if kind == Kind.VARIANCE else np.sqrt(var), rtol=1e-14, atol=1e-12)
    counts32 = _finish(Kind.COUNT_VALID, 0, TypeId.INT32, None, dev(cnt.astype(np.int32)), None, False).to_host()
    assert counts32.type_id == TypeId.INT32 and np.array_equal(counts32.values(), cnt.astype(np.int32))
    carrier = _finish(None, 0, TypeId.INT8, None, c_col, None, True)
    assert carrier.null_count == int((~ok).sum())
    total = rng.integers(-10**6, 10**6, n).astype(np.int64)
    dur = _finish(Kind.MEAN, 0, TypeId.DURATION_SECONDS, dev(total, TypeId.DURATION_SECONDS), c_col, None, False).to_host()
    q = np.trunc(total[ok] / cnt[ok]).astype(np.int64)   # C++ integer division truncates towards zero
    assert dur.type_id == TypeId.DURATION_SECONDS and np.array_equal(dur.values()[ok], q)


def test_pack_into_the_largest_number_of_destinations():
    """b2_state_pack accepts up to 4096 destinations; the scatter kernel then needs 64 KB of dynamic shared
    memory (beyond the 48 KB default).  All records merged back into one state give the one-shot result."""
    import cudf_b200 as cb
    w = workloads.make(3, 20_000, scale_domain=True)
    reqs = [(v, AGGS) for v, _ in w.requests]
    gb, dreqs = _device_objects(w.keys, reqs, w.null_policy, 0, 20_000)
    st = cb.GroupByState(gb, dreqs)
    st.update()
    records, counts = st.pack(4096)
    assert len(counts) == 4096 and sum(counts) == st.num_groups() and max(counts) < 40
    total = sum(counts)
    st.reset()
    st.merge(records[: total * st.record_bytes], total)
    got = _to_host(st.finalize())
    exp = oracle.groupby(w.keys, reqs, w.null_policy)
    H.assert_same_result(got, exp, reqs, scales=H.result_scales(w.keys, reqs, w.null_policy))


@pytest.mark.parametrize("estimate", [3, 4000, 6000, 10**7])
def test_merge_into_a_table_sized_from_an_estimate(estimate):
    """An empty state sized from an estimate of the distinct keys: too small an estimate (3, 4000 for
    5000 keys) must fall back to the full-size table without losing or doubling a record."""
    import cudf_b200 as cb
    rng = np.random.default_rng(43)
    n = 200_000
    k = HostColumn.from_numpy(rng.integers(0, 5000, n).astype(np.int64))
    v = HostColumn.from_numpy(rng.standard_normal(n), valid=rng.random(n) > 0.1)
    reqs = [(v, AGGS)]
    packed = []
    for r in range(4):
        gb, dreqs = _device_objects([k], reqs, NullPolicy.EXCLUDE, r * n // 4, (r + 1) * n // 4)
        st = cb.GroupByState(gb, dreqs)
        st.update()
        records, counts = st.pack(1)
        packed.append((records, counts[0], st, gb, dreqs))
    import torch
    allrec = torch.cat([p[0][: p[1] * p[2].record_bytes] for p in packed])
    total = sum(p[1] for p in packed)
    st = packed[0][2]
    st.reset(expected_groups=estimate)
    st.merge(allrec, total)
    assert st.num_groups() == 5000
    got = _to_host(st.finalize())
    exp = oracle.groupby([k], reqs, NullPolicy.EXCLUDE)
    H.assert_same_result(got, exp, reqs, scales=H.result_scales([k], reqs, NullPolicy.EXCLUDE))


def test_batchwise_updates_equal_one_shot():
    import cudf_b200 as cb
    rng = np.random.default_rng(41)
    n = 300_000
    # (an int64 key with nulls under INCLUDE needs 65 bits: such states are row-keyed and take one update)
    k = HostColumn.from_numpy(rng.integers(0, 5000, n).astype(np.int32), valid=rng.random(n) > 0.02)
    v = HostColumn.from_numpy(rng.standard_normal(n), valid=rng.random(n) > 0.1)
    # SUM_OVERFLOW of a 64-bit column through batches: its two exact-sum cells add up like any other
    # (some groups of ~60 values of up to 2^58 leave the int64 range, others do not)
    w = HostColumn.from_numpy(rng.integers(0, 2 ** 58, n, dtype=np.int64) * np.where(k.values() % 2 == 0, 1, -1),
                              valid=rng.random(n) > 0.1)
    reqs = [(v, AGGS), (w, [Kind.SUM_OVERFLOW, Kind.COUNT_VALID])]
    for policy in (NullPolicy.EXCLUDE, NullPolicy.INCLUDE):
        st = None
        for b in range(3):
            gb, dreqs = _device_objects([k], reqs, policy, b * n // 3, (b + 1) * n // 3)
            if st is None:
                st = cb.GroupByState(gb, dreqs)
            st.update(gb, dreqs)
        got = _to_host(st.finalize())
        exp = oracle.groupby([k], reqs, policy)
        H.assert_same_result(got, exp, reqs, scales=H.result_scales([k], reqs, policy))


@pytest.mark.parametrize("dtype", [np.float64, np.float32])
def test_batchwise_mean_after_a_lean_first_batch(dtype):
    """Σ and n of one float column: the first batch of a fresh state runs the lean kernel over the sampled key
    box, the later batches the generic kernel on the same table (keys outside the first batch's box included)."""
    import cudf_b200 as cb
    rng = np.random.default_rng(43)
    n = 300_000
    keys = rng.integers(0, 800, n).astype(np.int64)
    keys[n // 3:] += rng.integers(0, 3, n - n // 3) * 5000      # later batches bring keys far outside the box
    k = HostColumn.from_numpy(keys)
    v = HostColumn.from_numpy(rng.standard_normal(n).astype(dtype), valid=rng.random(n) > 0.1)
    reqs = [(v, [Kind.SUM, Kind.COUNT_VALID, Kind.MEAN])]
    st = None
    for b in range(3):
        gb, dreqs = _device_objects([k], reqs, NullPolicy.EXCLUDE, b * n // 3, (b + 1) * n // 3)
        if st is None:
            st = cb.GroupByState(gb, dreqs)
        st.update(gb, dreqs)
    got = _to_host(st.finalize())
    exp = oracle.groupby([k], reqs)
    H.assert_same_result(got, exp, reqs, scales=H.result_scales([k], reqs, NullPolicy.EXCLUDE))


def test_state_with_string_keys_reports_unsupported_for_pack():
    import cudf_b200 as cb
    from cudf_b200 import aggregation as agg
    s = cb.Column.from_host(HostColumn.from_strings(["a", "b", "a", "c"] * 100))
    v = cb.Column.from_host(HostColumn.from_numpy(np.arange(400, dtype=np.int32)))
    gb = cb.GroupBy(cb.Table([s]))
    st = cb.GroupByState(gb, [cb.GroupByRequest(v, [agg.sum()])])
    st.update()
    assert st.num_groups() == 3
    with pytest.raises(cb.UnsupportedError):
        st.pack(2)
    keys, res = _to_host(st.finalize())
    assert sorted(keys[0].to_pylist()) == [b"a", b"b", b"c"]


@pytest.mark.parametrize("nparts", [1, 2, 8, 13])
def test_hash_partition_rows(nparts):
    import cudf_b200 as cb
    from cudf_b200.partition import hash_partition
    rng = np.random.default_rng(42)
    n = 100_003
    a = HostColumn.from_numpy(rng.integers(0, 1000, n).astype(np.int64))
    b = HostColumn.from_numpy(rng.integers(-5, 5, n).astype(np.int32))
    v = HostColumn.from_numpy(rng.standard_normal(n), valid=rng.random(n) > 0.2)
    w = HostColumn.from_numpy(rng.integers(0, 255, n).astype(np.uint8))
    table = cb.Table([cb.Column.from_host(c) for c in (a, b, v, w)])
    out, offsets = hash_partition(table, 2, nparts)
    assert offsets[0] == 0 and offsets[-1] == n and len(offsets) == nparts + 1
    cols = [c.to_host() for c in out.columns()]
    ka, kb = cols[0].values(), cols[1].values()
    # every key lands in exactly one partition
    part_of = np.repeat(np.arange(nparts), np.diff(offsets))
    keyid = ka * 100 + kb
    first = {}
    order = np.argsort(keyid, kind="stable")
    sk, sp = keyid[order], part_of[order]
    change = np.flatnonzero(np.diff(sk)) + 1
    for seg in np.split(sp, change):
        assert seg.min() == seg.max()
    # the rows are a permutation of the input, validity travelling with the values
    def rows(cols4):
        vv = np.where(cols4[2].valid(), cols4[2].values(), np.nan)
        return sorted(zip(cols4[0].values().tolist(), cols4[1].values().tolist(),
                          [None if np.isnan(x) else x for x in vv.tolist()], cols4[3].values().tolist()),
                      key=lambda t: (t[0], t[1], t[3], -1e300 if t[2] is None else t[2]))
    assert rows(cols) == rows([a, b, v, w])
    assert cols[2].null_count == v.null_count


def test_rows_strategy_matches_partials_on_emulated_ranks():
    """hash_partition of raw rows, then per-partition groupby == one-shot groupby."""
    import cudf_b200 as cb
    from cudf_b200.aggregation import Aggregation
    from cudf_b200.partition import hash_partition
    w = workloads.make(3, 200_000, scale_domain=True)
    table = cb.Table([cb.Column.from_host(c) for c in (w.keys[0], w.requests[0][0])])
    out, offsets = hash_partition(table, 1, 4)
    parts = []
    for p in range(4):
        lo, hi = offsets[p], offsets[p + 1]
        kc, vc = out.columns()
        k = cb.Column(kc.type_id, hi - lo, kc.data[lo * 8:hi * 8].clone(), None, 0, 0)
        v = cb.Column(vc.type_id, hi - lo, vc.data[lo * 8:hi * 8].clone(), None, 0, 0)
        gb = cb.GroupBy(cb.Table([k]))
        parts.append(_to_host(gb.aggregate([cb.GroupByRequest(v, [Aggregation(Kind(a)) for a in w.requests[0][1]])])))
    got = _concat(parts)
    exp = oracle.groupby(w.keys, w.requests)
    H.assert_same_result(got, exp, w.requests)


@pytest.mark.parametrize("ranks", [2, 8])
def test_fixed_chunk_exchange_equals_one_shot(ranks):
    """pack_chunks / merge_chunks (the equal-split all-to-all form) on emulated ranks."""
    import torch
    import cudf_b200 as cb
    n, chunk = 160_000, 8192
    w = workloads.make(2, n)
    reqs = [(v, AGGS) for v, _ in w.requests]
    sent, keep = [], []
    for r in range(ranks):
        gb, dreqs = _device_objects(w.keys, reqs, w.null_policy, r * n // ranks, (r + 1) * n // ranks)
        st = cb.GroupByState(gb, dreqs)
        st.update()
        sent.append(st.pack_chunks(ranks, chunk))
        keep.append((st, gb, dreqs))
    cb_bytes = keep[0][0].chunk_bytes(chunk)
    parts = []
    for dst in range(ranks):
        recv = torch.cat([s[dst * cb_bytes:(dst + 1) * cb_bytes] for s in sent])  # what all_to_all delivers
        _, gb, dreqs = keep[dst]
        merged = cb.GroupByState(gb, dreqs)
        merged.merge_chunks(recv, ranks, chunk)
        parts.append(_to_host(merged.finalize()))
    got = _concat(parts)
    exp = oracle.groupby(w.keys, reqs, w.null_policy)
    H.assert_same_result(got, exp, reqs, scales=H.result_scales(w.keys, reqs, w.null_policy))


def test_fixed_chunk_overflow_is_reported_to_every_receiver():
    import torch
    import cudf_b200 as cb
    n = 50_000
    w = workloads.make(2, n)
    reqs = [(v, [Kind.SUM]) for v, _ in w.requests]
    gb, dreqs = _device_objects(w.keys, reqs, w.null_policy, 0, n)
    st = cb.GroupByState(gb, dreqs)
    st.update()
    ranks, chunk = 4, 64   # ~2500 groups per destination do not fit 64 records
    send = st.pack_chunks(ranks, chunk)
    cbytes = st.chunk_bytes(chunk)
    for dst in range(ranks):
        merged = cb.GroupByState(gb, dreqs)
        merged.merge_chunks(send[dst * cbytes:(dst + 1) * cbytes].clone(), 1, chunk)
        with pytest.raises(cb.LogicError, match="chunk overflow"):
            merged.finalize()


def test_hash_partition_with_string_and_nullable_columns():
    import cudf_b200 as cb
    from cudf_b200.partition import hash_partition
    rng = np.random.default_rng(43)
    n = 50_001
    words = ["", "a", "bb", "año", "x" * 37, "hello", "₹1", None]
    pick = rng.integers(0, len(words), n)
    s = HostColumn.from_strings([words[i] for i in pick])
    k2 = HostColumn.from_numpy(rng.integers(0, 5, n).astype(np.int32))
    v = HostColumn.from_numpy(rng.standard_normal(n), valid=rng.random(n) > 0.3)
    table = cb.Table([cb.Column.from_host(c) for c in (s, k2, v)])
    for nparts in (1, 3, 8):
        out, offsets = hash_partition(table, 2, nparts)
        assert offsets[0] == 0 and offsets[-1] == n
        hs, hk, hv = (c.to_host() for c in out.columns())
        got = sorted(zip([x if x is not None else b"\xff" for x in hs.to_pylist()], hk.values().tolist(),
                         [(-1e300 if x is None else x) for x in hv.to_pylist()]))
        exp = sorted(zip([x if x is not None else b"\xff" for x in s.to_pylist()], k2.values().tolist(),
                         [(-1e300 if x is None else x) for x in v.to_pylist()]))
        assert got == exp
        # a key lives in one partition only
        part_of = np.repeat(np.arange(nparts), np.diff(offsets))
        seen = {}
        for key, p in zip(zip(hs.to_pylist(), hk.values().tolist()), part_of.tolist()):
            assert seen.setdefault(key, p) == p


def test_row_exchange_with_strings_and_nulls_single_rank_group():
    """exchange_rows over a one-rank NCCL group (every partition comes back to this rank), then the
    groupby on the received columns equals the one-shot result: C5-shaped input."""
    import os
    import torch
    import torch.distributed as dist
    import cudf_b200 as cb
    from cudf_b200.aggregation import Aggregation
    from cudf_b200.distributed import exchange_rows
    from cudf_b200.partition import hash_partition
    w = workloads.make(5, 60_000)
    created = False
    if not dist.is_initialized():
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29541")
        dist.init_process_group("nccl", rank=0, world_size=1, device_id=torch.device("cuda", 0))
        created = True
    try:
        cols = [cb.Column.from_host(c) for c in w.keys + [v for v, _ in w.requests]]
        parts, offsets = hash_partition(cb.Table(cols), len(w.keys), 1)
        recv = exchange_rows(parts, offsets, 1)
        gb = cb.GroupBy(cb.Table(recv[:2]))
        reqs = [cb.GroupByRequest(recv[2 + i], [Aggregation(Kind(a)) for a in aggs]) for i, (_, aggs) in enumerate(w.requests)]
        got = _to_host(gb.aggregate(reqs))
    finally:
        if created:
            dist.destroy_process_group()
    exp = oracle.groupby(w.keys, w.requests)
    H.assert_same_result(got, exp, w.requests, scales=H.result_scales(w.keys, w.requests, w.null_policy))


@pytest.mark.parametrize("ranks", [2, 3])
def test_partial_table_shuffle_for_string_keys_equals_one_shot(ranks):
    """Keys that do not pack into 64 bits travel as a TABLE of partial aggregates: local aggregate, hash
    partition of the partial table by key, (emulated) exchange, reduction groupby, finalisers — the steps of
    DistributedGroupBy's partials strategy for string keys, with the all-to-all replaced by host slicing."""
    import cudf_b200 as cb
    from cudf_b200.partials import PartialTable
    from cudf_b200.partition import hash_partition
    n = 60_000
    w = workloads.make(5, n)
    kinds = [Kind.SUM, Kind.COUNT_VALID, Kind.COUNT_ALL, Kind.MEAN, Kind.MIN, Kind.MAX, Kind.VARIANCE, Kind.STD, Kind.M2]
    reqs = [(v, kinds) for v, _ in w.requests]
    nkeys = len(w.keys)

    def cut(c, lo, hi):
        if c.type_id == TypeId.STRING:
            return HostColumn.from_strings(c.to_pylist()[lo:hi])
        return HostColumn.from_numpy(c.values()[lo:hi], c.valid()[lo:hi] if c.mask is not None else None, type_id=c.type_id)

    specs = [(q, k, 1) for q in range(len(reqs)) for k in kinds]
    outgoing = []  # per rank: (host columns of the partitioned partial table, offsets)
    tables = []
    for r in range(ranks):
        lo, hi = r * n // ranks, (r + 1) * n // ranks
        pt = PartialTable(specs, w.null_policy)
        pt.add_batch([cb.Column.from_host(cut(k, lo, hi)) for k in w.keys],
                     {q: cb.Column.from_host(cut(v, lo, hi)) for q, (v, _) in enumerate(reqs)})
        parts, offsets = hash_partition(cb.Table(pt.keys + pt.columns()), nkeys, ranks)
        outgoing.append(([c.to_host() for c in parts.columns()], offsets))
        tables.append(pt)
    got_parts = []
    for dst in range(ranks):
        recv = []
        for ci in range(len(outgoing[0][0])):
            pieces = [cut(cols[ci], offs[dst], offs[dst + 1]) for cols, offs in outgoing]
            if pieces[0].type_id == TypeId.STRING:
                merged = HostColumn.from_strings([x for p in pieces for x in p.to_pylist()])
            else:
                valid = np.concatenate([p.valid() for p in pieces]) if any(p.mask is not None for p in pieces) else None
                merged = HostColumn.from_numpy(np.concatenate([p.values() for p in pieces]), valid, type_id=pieces[0].type_id)
            recv.append(cb.Column.from_host(merged))
        pt = tables[dst]
        pt.reduce_rows(recv[:nkeys], recv[nkeys:])
        keys, flat = pt.finalize(detect_nulls=True)
        res, i = [], 0
        for _ in reqs:
            res.append([c.to_host() for c in flat[i:i + len(kinds)]])
            i += len(kinds)
        got_parts.append(([k.to_host() for k in keys], res))

    def cat(cols):
        if cols[0].type_id == TypeId.STRING:
            return HostColumn.from_strings([x for c in cols for x in c.to_pylist()])
        valid = np.concatenate([c.valid() for c in cols]) if any(c.mask is not None for c in cols) else None
        return HostColumn.from_numpy(np.concatenate([c.values() for c in cols]), valid, type_id=cols[0].type_id)
    got = ([cat([p[0][k] for p in got_parts]) for k in range(nkeys)],
           [[cat([p[1][q][a] for p in got_parts]) for a in range(len(kinds))] for q in range(len(reqs))])
    exp = oracle.groupby(w.keys, reqs, w.null_policy)
    H.assert_same_result(got, exp, reqs, check_nullable=False, scales=H.result_scales(w.keys, reqs, w.null_policy))
    assert got[0][0].size == exp[0][0].size  # ownership is disjoint
