"""Shared helpers of the parity tests: golden-case decoding, key sorting, column comparison."""
from __future__ import annotations

import json
import math
import os
from typing import List, Sequence

import numpy as np

from cudf_b200.types import (HostColumn, Kind, NullPolicy, STORAGE_DTYPE, TypeId, int128_array, is_floating, pack_mask,
                             result_type)

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "reference_known_answers.json")

# north_star tolerances: float sum/mean/var within 1e-12 (fp64 sources) or 1e-5 (fp32 sources)
RTOL_F64 = 1e-12
RTOL_F32 = 1e-5
# A float result is held to the STRICT relative tolerance |got - exp| <= rtol * |exp| whenever
# |exp| >= STRICT_FROM * (error scale of its group: Σ|x| for sums and means, Σx²/(n - ddof) for
# variances; for a standard deviation the ratio of the variances decides); only results that
# cancellation drove below that are compared relative to the scale.  The threshold is the point
# where the strict tolerance, rtol * |exp|, is 9 unit roundoffs of the SOURCE type times the scale:
# 1e-3 for fp64 sources (1e-15 * scale against 2^-53), 5.4e-2 for fp32 sources (5.4e-7 * scale
# against 2^-24).  Below it a sum accumulated in the source's own precision, in any order (the
# reference adds fp32 values with fp32 atomics), cannot be told from a wrong one by the result alone.
STRICT_FROM = 1e-3
STRICT_FROM_F32 = STRICT_FROM * (2.0 ** -24 / RTOL_F32) / (2.0 ** -53 / RTOL_F64)
# one record per compared float column: what, values compared, values held to the strict tolerance,
# the largest strict relative error among those, values that only pass through the scaled bound, the
# largest error relative to the scale among them (printed by the parity tests; also appended to
# $B2_TEST_LOG_DIR/parity_stats.jsonl when that variable names a directory)
PARITY_STATS: list = []


def record_parity_stats(label: str):
    """Tags the records collected since the last call with ``label``, prints and appends them to the stats file."""
    recs = [dict(r, config=label) for r in PARITY_STATS]
    PARITY_STATS.clear()
    for r in recs:
        print(f"[parity] {label}: {r['what']}: {r['n']} values, strict {r['strict_n']} (max rel err {r['strict_max']:.3e}, "
              f"rtol {r['rtol']:g}), scaled-only {r['scaled_n']} (max err/scale {r['scaled_max']:.3e})")
    log_dir = os.environ.get("B2_TEST_LOG_DIR")
    if log_dir and os.path.isdir(log_dir):
        try:
            with open(os.path.join(log_dir, "parity_stats.jsonl"), "a", encoding="utf-8") as f:
                for r in recs:
                    f.write(json.dumps(r) + "\n")
        except OSError:
            pass
    return recs


def load_golden() -> list:
    with open(GOLDEN, encoding="utf-8") as f:
        return json.load(f)["cases"]


def _num(x):
    if isinstance(x, str):
        return {"inf": math.inf, "-inf": -math.inf, "nan": math.nan}[x]
    return x


def make_column(values: Sequence, type_name: str, offset: int = 0, scale: int = 0) -> HostColumn:
    """Column of the named type from a Python list where ``None`` is a null element."""
    t = TypeId[type_name]
    valid = np.array([v is not None for v in values], dtype=bool)
    if t == TypeId.STRING:
        return HostColumn.from_strings(list(values))
    filled = [0 if v is None else _num(v) for v in values]
    if t == TypeId.DECIMAL128:
        arr = int128_array(filled)
    elif is_floating(t) or all(-2 ** 63 <= v < 2 ** 63 for v in filled):
        arr = np.array(filled, dtype=np.float64 if is_floating(t) else np.int64).astype(STORAGE_DTYPE[t])
    else:  # a value outside int64 (a 128-bit extreme listed for a narrower type never is)
        arr = np.array([v & (2 ** 64 - 1) for v in filled], dtype=np.uint64).astype(STORAGE_DTYPE[t])
    return HostColumn.from_numpy(arr, None if valid.all() and len(values) else (valid if len(values) else None),
                                 type_id=t, offset=offset, scale=scale)


def sort_order(keys: List[HostColumn]) -> np.ndarray:
    """Permutation that sorts the groups by key (nulls first), the way the reference's tests sort
    a result before comparing it (cpp/tests/groupby/groupby_test_util.cpp:83-90)."""
    n = keys[0].size if keys else 0
    if n == 0:
        return np.zeros(0, dtype=np.int64)
    cols = []
    for k in reversed(keys):
        v = k.valid()
        if k.type_id == TypeId.STRING:
            py = k.to_pylist()
            ranks = {s: i for i, s in enumerate(sorted(set(x for x in py if x is not None)))}
            vals = np.array([ranks[x] if x is not None else -1 for x in py], dtype=np.int64)
        else:
            vals = k.values().copy()
            if is_floating(k.type_id):
                nan = np.isnan(vals)
                vals = np.where(nan, 0.0, vals) + 0.0  # -0 -> +0; NaN keys sort after all numbers
                cols.append(np.where(v, vals, 0.0))
                cols.append((nan & v).astype(np.int8))
                cols.append(v.astype(np.int8))
                continue
        vals = np.where(v, vals, vals.dtype.type(0))
        cols.append(vals)
        cols.append(v.astype(np.int8))
    return np.lexsort(cols)


def take(col: HostColumn, order: np.ndarray) -> list:
    py = col.to_pylist()
    return [py[i] for i in order]


def assert_column_equal(got: HostColumn, exp: HostColumn, order_got, order_exp, rtol: float, what: str,
                        check_nullable: bool = False, scale=None, strict_power: int = 1,
                        strict_from: float = STRICT_FROM):
    assert TypeId(got.type_id) == TypeId(exp.type_id), f"{what}: type {got.type_id!r} != {exp.type_id!r}"
    assert got.size == exp.size, f"{what}: size {got.size} != {exp.size}"
    assert getattr(got, "scale", 0) == getattr(exp, "scale", 0), f"{what}: decimal scale differs"
    if got.size == 0:
        return
    if check_nullable:
        assert (got.mask is None) == (exp.mask is None), f"{what}: nullability differs"
    vg, ve = got.valid()[order_got], exp.valid()[order_exp]
    assert np.array_equal(vg, ve), f"{what}: validity differs at {np.flatnonzero(vg != ve)[:8]}"
    assert got.null_count == exp.null_count, f"{what}: null_count {got.null_count} != {exp.null_count}"
    if got.type_id == TypeId.STRUCT:   # SUM_OVERFLOW: {sum in the source type, overflow flag}, the mask on the struct
        assert len(got.children) == 2 and len(exp.children) == 2, f"{what}: a struct of two children"
        (gs, gf), (es, ef) = got.children, exp.children
        assert gs.mask is None and gf.mask is None, f"{what}: the children carry no masks"
        assert TypeId(gs.type_id) == TypeId(es.type_id) and TypeId(gf.type_id) == TypeId.BOOL8, f"{what}: child types"
        assert gs.scale == es.scale, f"{what}: decimal scale of the sum child differs"
        assert gs.size == got.size and gf.size == got.size, f"{what}: child sizes"
        fa, fb = gf.values()[order_got] != 0, ef.values()[order_exp] != 0
        assert np.array_equal(fa, fb), f"{what}: overflow flags differ at {np.flatnonzero(fa != fb)[:8]}"
        # the sum of a group that overflowed is not specified by the reference; a null struct holds 0 / false
        sa, sb = gs.values()[order_got], es.values()[order_exp]
        cmp = ~fa
        bad = np.flatnonzero(sa[cmp] != sb[cmp])
        assert bad.size == 0, f"{what}: {bad.size} sums differ; first {sa[cmp][bad[:8]]} vs {sb[cmp][bad[:8]]}"
        return
    if got.type_id == TypeId.STRING:   # MIN / MAX of strings
        ga, gb = take(got, order_got), take(exp, order_exp)
        assert ga == gb, f"{what}: {[x for x, y in zip(ga, gb) if x != y][:4]} vs {[y for x, y in zip(ga, gb) if x != y][:4]}"
        return
    a, b = got.values()[order_got][vg], exp.values()[order_exp][ve]
    if is_floating(got.type_id):
        a, b = a.astype(np.float64), b.astype(np.float64)
        nan_a, nan_b = np.isnan(a), np.isnan(b)
        if strict_power == 2 and scale is not None and not np.array_equal(nan_a, nan_b):
            # A standard deviation is the root of Σx² − (Σx)²/n: where that difference is zero up to rounding, the
            # sign of the rounding decides between 0 and NaN — in the reference too (no clamp in
            # cpp/src/groupby/common/m2_var_std.cu:152-188), by the order its atomics happened to add in.  Such a
            # position passes when the side that is a number is zero within the tolerance of the variance.
            one = nan_a ^ nan_b
            number = np.where(nan_a, b, a)[one]
            sc_one = np.asarray(scale, dtype=np.float64)[order_exp][ve][one]
            assert (number ** 2 <= rtol * sc_one ** 2 + 1e-300).all(), f"{what}: NaN positions differ"
            a, b = np.where(one, np.nan, a), np.where(one, np.nan, b)
            nan_a = nan_b = np.isnan(a)
        assert np.array_equal(nan_a, nan_b), f"{what}: NaN positions differ"
        inf = np.isinf(a) | np.isinf(b)
        assert np.array_equal(a[inf], b[inf]), f"{what}: infinities differ"
        fin = ~(nan_a | inf)
        err = np.abs(a[fin] - b[fin])
        mag = np.maximum(np.abs(a[fin]), np.abs(b[fin]))
        if scale is None:
            strict = np.ones(err.size, dtype=bool)
            sc = mag
        else:
            sc = np.asarray(scale, dtype=np.float64)[order_exp][ve][fin]
            # (a standard deviation is the root of a difference: its conditioning is that of the variance)
            strict = mag ** strict_power >= strict_from * sc ** strict_power
        # strict: relative to the result itself; the rest: relative to the group's error scale
        tol = rtol * np.where(strict, mag, np.maximum(mag, sc)) + 1e-300
        bad = np.flatnonzero(err > tol)
        with np.errstate(divide="ignore", invalid="ignore"):
            rel = np.where(mag > 0, err / mag, 0.0)
            rel_sc = np.where(sc > 0, err / np.maximum(mag, sc), 0.0)
        PARITY_STATS.append({"what": what, "n": int(err.size), "strict_n": int(strict.sum()),
                             "strict_max": float(rel[strict].max()) if strict.any() else 0.0,
                             "scaled_n": int((~strict).sum()),
                             "scaled_max": float(rel_sc[~strict].max()) if (~strict).any() else 0.0, "rtol": rtol})
        assert bad.size == 0, (f"{what}: {bad.size} values beyond rtol {rtol}; first {a[fin][bad[:4]]} vs "
                               f"{b[fin][bad[:4]]} (strict: {strict[bad[:4]]})")
    else:
        bad = np.flatnonzero(a != b)
        assert bad.size == 0, f"{what}: {bad.size} values differ; first {a[bad[:8]]} vs {b[bad[:8]]}"


def assert_keys_equal(got: List[HostColumn], exp: List[HostColumn], order_got, order_exp):
    assert len(got) == len(exp)
    for i, (a, b) in enumerate(zip(got, exp)):
        assert TypeId(a.type_id) == TypeId(b.type_id), f"key column {i}: type differs"
        assert a.size == b.size, f"key column {i}: {a.size} vs {b.size} groups"
        if a.size == 0:
            continue
        if a.type_id == TypeId.STRING:
            ga, gb = take(a, order_got), take(b, order_exp)
            assert ga == gb, f"key column {i}: {ga[:8]} vs {gb[:8]}"
            continue
        va, vb = a.valid()[order_got], b.valid()[order_exp]
        assert np.array_equal(va, vb), f"key column {i}: validity differs"
        xa, xb = a.values()[order_got][va], b.values()[order_exp][vb]
        if is_floating(a.type_id):
            # +0 == -0 and NaN == NaN as keys
            assert np.array_equal(np.isnan(xa), np.isnan(xb)), f"key column {i}: NaN keys differ"
            ok = ~np.isnan(xa)
            assert np.array_equal(xa[ok] + 0.0, xb[ok] + 0.0), f"key column {i}: values differ"
        else:
            bad = np.flatnonzero(xa != xb)
            assert bad.size == 0, f"key column {i}: {bad.size} keys differ; first {xa[bad[:8]]} vs {xb[bad[:8]]}"


def rtol_for(source_type: int) -> float:
    return RTOL_F32 if TypeId(source_type) == TypeId.FLOAT32 else RTOL_F64


def strict_from_for(source_type: int) -> float:
    return STRICT_FROM_F32 if TypeId(source_type) == TypeId.FLOAT32 else STRICT_FROM


def golden_instances(case: dict):
    """Expands a golden case into (id, keys column, values column, kind, ddof, policy,
    expected keys column, expected values column)."""
    kind = Kind[case["agg"]]
    policy = NullPolicy[case["null_policy"]]
    for vt in case["value_types"]:
        if vt != "STRING" and any(isinstance(v, (int, float)) and v < 0 for v in case["vals"] if v is not None) \
                and vt.startswith("UINT"):
            continue
        keys = make_column(case["keys"], case["key_type"])
        scale = case.get("scale", 0)
        vals = make_column(case["vals"], vt, scale=scale)
        rt = result_type(TypeId[vt], kind)   # (COUNT and ARGMIN / ARGMAX of strings are INT32, their MIN / MAX strings)
        ekeys = make_column(case["expect_keys"], case["key_type"])
        if kind == Kind.SUM_OVERFLOW:
            # a struct: children without masks (0 / false where the struct is null; "?" = a sum the reference's
            # test does not look at), the validity on the struct
            ev = case["expect_vals"]
            sums = make_column([0 if v is None or v == "?" else v for v in ev], vt, scale=scale)
            flags = HostColumn.from_numpy(np.array(case["expect_overflow"], dtype=np.uint8), type_id=TypeId.BOOL8)
            valid = np.array([v is not None for v in ev], dtype=bool)
            evals = HostColumn(TypeId.STRUCT, len(ev), None, None if valid.all() else pack_mask(valid), 0, None, 0,
                               [sums, flags])
            yield f'{case["name"]}[{vt}]', keys, vals, kind, case["ddof"], policy, ekeys, evals
            continue
        evals = make_column(case["expect_vals"], rt.name, scale=scale if rt.name.startswith("DECIMAL") else 0)
        yield f'{case["name"]}[{vt}]', keys, vals, kind, case["ddof"], policy, ekeys, evals


# ------------------------------------------------------------------------------------ GPU side
def gpu_groupby(keys: Sequence[HostColumn], requests, null_policy=NullPolicy.EXCLUDE, row_filters=(), **opts):
    """Runs the CUDA engine through its public host API (which calls the C ABI) on host columns.
    ``requests`` is a list of (values HostColumn, [kind | (kind, ddof), ...])."""
    import cudf_b200 as cb
    from cudf_b200.aggregation import Aggregation

    dkeys = cb.Table([cb.Column.from_host(k) for k in keys])
    dreqs = []
    cache = {}
    for vals, aggs in requests:
        if id(vals) not in cache:
            cache[id(vals)] = cb.Column.from_host(vals)
        al = [Aggregation(Kind(a[0]), a[1]) if isinstance(a, tuple) else Aggregation(Kind(a)) for a in aggs]
        dreqs.append(cb.GroupByRequest(cache[id(vals)], al))
    filt = [cb.Column.from_host(f) for f in row_filters]
    gb = cb.GroupBy(dkeys, null_policy, row_filters=filt, **opts)
    okeys, ores = gb.aggregate(dreqs)
    return [c.to_host() for c in okeys.columns()], [[c.to_host() for c in t.columns()] for t in ores]


def result_scales(keys, requests, null_policy, row_filters=(), row_filter_offsets=()):
    """Per request, the magnitudes that bound the rounding error of its floating-point results, in
    the oracle's group order: (Σ|x|, Σx², n).  A sum of n floats is only determined up to
    ~eps·Σ|x| (any summation order, the reference's atomics included), and Σx² − (Σx)²/n up to
    ~eps·Σx², so the north-star tolerances are applied relative to these, not to a result that
    cancellation may have driven towards zero."""
    from oracle import oracle
    reqs = []
    for vals, _ in requests:
        if vals.type_id in (TypeId.STRING, TypeId.DECIMAL128) or vals.type_id not in STORAGE_DTYPE:
            x = np.zeros(vals.size)
        else:
            x = vals.values().astype(np.float64)
        x = np.where(np.isfinite(x), x, 0.0)
        valid = vals.valid() if vals.mask is not None else None
        reqs.append((HostColumn.from_numpy(np.abs(x), valid), [Kind.SUM, Kind.COUNT_VALID]))
        reqs.append((HostColumn.from_numpy(x * x, valid), [Kind.SUM]))
    _, res = oracle.groupby(keys, reqs, null_policy, row_filters=row_filters, row_filter_offsets=row_filter_offsets)
    out = []
    for q in range(len(requests)):
        sa = np.where(res[2 * q][0].valid(), res[2 * q][0].values(), 0.0)
        n = res[2 * q][1].values().astype(np.float64)
        ss = np.where(res[2 * q + 1][0].valid(), res[2 * q + 1][0].values(), 0.0)
        out.append((sa, ss, n))
    return out


def reorder_scales(scales, from_keys, to_keys):
    """Scales given in the group order of ``from_keys`` re-expressed in the group order of ``to_keys``
    (same key set, different order)."""
    of, ot = sort_order(from_keys), sort_order(to_keys)
    out = []
    for triple in scales:
        new = []
        for arr in triple:
            a = np.empty_like(arr)
            a[ot] = arr[of]
            new.append(a)
        out.append(tuple(new))
    return out


def _scale_for(kind, ddof, sa, ss, n):
    kind = Kind(kind)
    df = np.maximum(n - ddof, 1.0)
    if kind == Kind.SUM:
        return sa
    if kind == Kind.MEAN:
        return sa / np.maximum(n, 1.0)
    if kind in (Kind.SUM_OF_SQUARES, Kind.M2):
        return ss
    if kind == Kind.VARIANCE:
        return ss / df
    if kind == Kind.STD:
        return np.sqrt(ss / df)
    return np.zeros_like(sa)


def assert_same_result(got, exp, requests, check_nullable=True, scales=None):
    """Compares two (keys, results) pairs after sorting both by key: keys, counts, integer results
    bit-exact; float results within the north-star tolerance of their SOURCE type (1e-12 for
    fp64 sources, 1e-5 for fp32), relative to max(|result|, error scale of the group) below the strict threshold when
    ``scales`` (from result_scales, in ``exp``'s group order) is given."""
    gk, gr = got
    ek, er = exp
    og, oe = sort_order(gk), sort_order(ek)
    assert gk[0].size == ek[0].size, f"group count {gk[0].size} != {ek[0].size}"
    assert_keys_equal(gk, ek, og, oe)
    for q, (vals, aggs) in enumerate(requests):
        for a in range(len(aggs)):
            kind, ddof = (aggs[a] if isinstance(aggs[a], tuple) else (aggs[a], 1))
            scale = None
            if scales is not None and is_floating(er[q][a].type_id):
                scale = _scale_for(kind, ddof, *scales[q])
            assert_column_equal(gr[q][a], er[q][a], og, oe, rtol_for(vals.type_id), f"request {q} agg {aggs[a]}",
                                check_nullable=check_nullable, scale=scale, strict_power=2 if Kind(kind) == Kind.STD else 1,
                                strict_from=strict_from_for(vals.type_id))
