"""Parity of the CUDA engine (through its host API and C ABI) with the CPU oracle on seeded inputs:
the five benchmark configurations at oracle-sized row counts, every table path, and the edge
cases the reference's tests pin (empty / ragged sizes, nulls, slices, collisions, NaN)."""
import numpy as np
import pytest

import workloads
from cudf_b200.types import HostColumn, Kind, NullPolicy, TypeId
from oracle import oracle
from tests import helpers as H

pytestmark = pytest.mark.gpu

ALL_AGGS = [Kind.SUM, Kind.COUNT_VALID, Kind.COUNT_ALL, Kind.MEAN, Kind.MIN, Kind.MAX, Kind.SUM_OF_SQUARES,
            Kind.M2, Kind.VARIANCE, (Kind.STD, 2)]


def check(keys, requests, policy=NullPolicy.EXCLUDE, row_filters=(), **opts):
    got = H.gpu_groupby(keys, requests, policy, row_filters=row_filters, **opts)
    fm = [f.mask for f in row_filters if f.mask is not None]
    fo = [f.offset for f in row_filters if f.mask is not None]
    exp = oracle.groupby(keys, requests, policy, row_filters=fm, row_filter_offsets=fo)
    H.assert_same_result(got, exp, requests, scales=H.result_scales(keys, requests, policy, fm, fo))
    return got


@pytest.mark.parametrize("config,n", [(1, 400_000), (2, 600_000), (3, 300_000), (4, 500_000), (5, 120_000)])
@pytest.mark.parametrize("variant", [0, 1, 2, 3, 5, 6, 8])
def test_benchmark_configs_match_oracle(config, n, variant):
    """Variants: 0 auto, 1 global table only, 2 auto without fixed-point float sums, 3 hashed shared table,
    5 the bulk-copy tile ring (C2), 6 the partitioned path whatever the size (C1 / C4: hot keys folded by the
    counting pass, float sums as fixed-point limbs), 8 STRING keys through dictionary ids (C5)."""
    H.PARITY_STATS.clear()
    w = workloads.make(config, n, scale_domain=(config in (3, 4)))
    check(w.keys, w.requests, w.null_policy, w.row_filters, table_variant=variant)
    H.record_parity_stats(f"C{config} {n} rows, table_variant {variant}")


def test_config1_full_size_10m_rows_against_the_oracle():
    """C1 at its full 10M rows: every group against the CPU oracle, strict 1e-12 wherever the sum is
    not cancelled below 1e-3 of Σ|x|."""
    H.PARITY_STATS.clear()
    w = workloads.make(1)
    assert w.rows == 10_000_000
    got = check(w.keys, w.requests, w.null_policy, w.row_filters)
    assert got[0][0].size == 1000
    H.record_parity_stats("C1 full size (10M rows)")


def test_five_key_columns():
    """More than 4 key columns (the reference switches to cached row hashes there,
    cpp/src/groupby/hash/compute_groupby.cu:68-91): packed when the widths allow, row keys otherwise."""
    rng = np.random.default_rng(5)
    n = 60_000
    narrow = [HostColumn.from_numpy(rng.integers(0, 4, n).astype(dt)) for dt in (np.int8, np.int16, np.uint8, np.int8, np.int16)]
    v = HostColumn.from_numpy(rng.standard_normal(n), valid=rng.random(n) > 0.1)
    w = HostColumn.from_numpy(rng.integers(-50, 50, n).astype(np.int32))
    got = check(narrow, [(v, ALL_AGGS), (w, [Kind.SUM, Kind.MIN, Kind.MAX])])
    assert got[0][0].size == 4 ** 5
    wide = [HostColumn.from_numpy(rng.integers(0, 3, n).astype(np.int64), valid=rng.random(n) > 0.05) for _ in range(5)]
    check(wide, [(v, ALL_AGGS)])                       # 5 x 8 bytes: row keys
    check(wide, [(v, ALL_AGGS)], NullPolicy.INCLUDE)
    six = wide + [HostColumn.from_numpy(rng.random(n).round(1))]   # a float column among six
    check(six, [(w, [Kind.SUM, Kind.COUNT_ALL])], NullPolicy.INCLUDE)


def test_two_string_key_columns():
    """Two STRING key columns, UTF-8 content, nulls under both policies
    (cpp/tests/groupby/keys_tests.cpp:306-321 has one; the row comparator is column-wise)."""
    rng = np.random.default_rng(6)
    n = 40_000
    words = ["", "a", "año", "aa", "añejo", "b", "日本", "日本語", "z" * 40, "ab"]
    s1 = HostColumn.from_strings([None if rng.random() < 0.05 else words[i] for i in rng.integers(0, len(words), n)])
    s2 = HostColumn.from_strings([words[i] for i in rng.integers(0, 4, n)])
    k3 = HostColumn.from_numpy(rng.integers(0, 3, n).astype(np.int16))
    v = HostColumn.from_numpy(rng.standard_normal(n).astype(np.float32), valid=rng.random(n) > 0.2)
    for policy in (NullPolicy.EXCLUDE, NullPolicy.INCLUDE):
        for variant in (0, 8):
            got = check([s1, s2, k3], [(v, ALL_AGGS)], policy, table_variant=variant)
            assert got[0][0].size == (len(words) + (policy == NullPolicy.INCLUDE)) * 4 * 3


@pytest.mark.parametrize("variant", [0, 2, 6])
@pytest.mark.parametrize("vtype", ["f64", "f32"])
def test_float_sums_as_fixed_point_limbs(variant, vtype):
    """Σx / n / Σx² of one float column: the partitioned path (variant 6) folds the hot keys in its counting
    pass and keeps every shared-memory sum as fixed-point limbs; variants 0 and 2 are the table path on the same
    input.  Skewed keys, values of both signs, zeros, denormals, and magnitudes far outside the window the sampled
    maximum places — those are added to fp64 cells instead, and the result must not care."""
    rng = np.random.default_rng(77)
    n = 300_000
    ranks = np.minimum((rng.pareto(1.1, n) * 3).astype(np.int64), 200_000)
    k = HostColumn.from_numpy(ranks * 7919 % 1_000_003)
    x = rng.standard_normal(n) * np.exp(rng.standard_normal(n) * 2)
    x[rng.random(n) < 0.01] = 0.0
    x[rng.random(n) < 0.002] *= 1e-30      # far below the window
    x[rng.random(n) < 0.002] *= 1e25       # far above it
    x[rng.random(n) < 0.0005] = 5e-324     # denormal
    if vtype == "f32":
        x = x.astype(np.float32)
    v = HostColumn.from_numpy(x, valid=rng.random(n) > 0.05)
    aggs = [Kind.SUM, Kind.COUNT_VALID, Kind.MEAN, Kind.SUM_OF_SQUARES, Kind.VARIANCE]
    check([k], [(v, aggs)], table_variant=variant)
    check([k], [(v, [Kind.SUM])], table_variant=variant)                       # Σx alone, no count cell
    k_few = HostColumn.from_numpy(rng.integers(0, 50, n).astype(np.int32))     # a dense key box
    check([k_few], [(v, aggs)], table_variant=variant)


def test_string_keys_through_dictionary_ids():
    """table_variant 8: every STRING key column is replaced by dictionary ids before the packed-key
    aggregate and gathered back afterwards.  A dictionary that outgrows its first table (60K distinct strings
    in 200K rows), a sliced nullable column under both policies, INT64 offsets, an all-null column."""
    import cudf_b200 as cb
    rng = np.random.default_rng(61)
    n = 200_000
    pool = [("k%05d" % i) * (1 + i % 4) for i in range(60_000)]
    s = HostColumn.from_strings([pool[i] for i in rng.integers(0, len(pool), n)])
    k2 = HostColumn.from_numpy(rng.integers(0, 3, n).astype(np.int8))
    v = HostColumn.from_numpy(rng.standard_normal(n), valid=rng.random(n) > 0.1)
    w = HostColumn.from_numpy(rng.integers(-9, 9, n).astype(np.int64))
    reqs = [(v, ALL_AGGS), (w, [Kind.SUM, Kind.MIN, Kind.MAX, Kind.COUNT_ALL])]
    got = check([s, k2], reqs, table_variant=8)
    assert cb.last_call_stats().kernel_launches >= 4     # two dictionary attempts + the aggregate
    assert got[0][0].size > 100_000
    # a slice (element offset 5) of a nullable column with INT64 offsets
    m = 50_000
    words = ["", "x", "xy", "año", "日本語", "q" * 70]
    full = HostColumn.from_strings([None if rng.random() < 0.1 else words[i] for i in rng.integers(0, len(words), m + 9)],
                                   large_offsets=True)
    sl = HostColumn(TypeId.STRING, m, full.data, full.mask, 5, full.offsets)
    kk = HostColumn.from_numpy(rng.integers(0, 4, m).astype(np.int32), valid=rng.random(m) > 0.05)
    vv = HostColumn.from_numpy(rng.integers(-1000, 1000, m).astype(np.int32), valid=rng.random(m) > 0.2)
    for policy in (NullPolicy.EXCLUDE, NullPolicy.INCLUDE):
        got = check([kk, sl], [(vv, [Kind.SUM, Kind.MEAN, Kind.MIN, Kind.MAX, Kind.COUNT_VALID])], policy, table_variant=8)
        assert got[0][0].size == (len(words) + (policy == NullPolicy.INCLUDE)) * (4 + (policy == NullPolicy.INCLUDE))
    nothing = HostColumn.from_strings([None] * 1000)
    one = HostColumn.from_numpy(np.ones(1000, np.int32))
    assert check([nothing], [(one, [Kind.SUM])], NullPolicy.EXCLUDE, table_variant=8)[0][0].size == 0
    assert check([nothing], [(one, [Kind.SUM])], NullPolicy.INCLUDE, table_variant=8)[0][0].size == 1


def test_config2_full_domain_uses_compact_shared_table():
    import cudf_b200 as cb
    w = workloads.make(2, 1_500_000)
    got = check(w.keys, w.requests, w.null_policy, w.row_filters)
    st = cb.last_call_stats()
    assert st.used_shared_table and st.table_attempts == 1
    assert got[0][0].size == 10_000


@pytest.mark.parametrize("n", [0, 1, 2, 31, 32, 33, 127, 128, 129, 1023, 1024, 1025, 4095, 4096, 4097, 12289])
def test_ragged_sizes(n):
    rng = np.random.default_rng(n)
    k = HostColumn.from_numpy(rng.integers(0, 7, n).astype(np.int32), valid=rng.random(n) > 0.1)
    v = HostColumn.from_numpy(rng.standard_normal(n), valid=rng.random(n) > 0.2)
    check([k], [(v, ALL_AGGS)])
    check([k], [(v, ALL_AGGS)], NullPolicy.INCLUDE)


@pytest.mark.parametrize("vt", ["INT8", "INT16", "INT32", "INT64", "UINT8", "UINT16", "UINT32", "UINT64",
                                "FLOAT32", "FLOAT64", "BOOL8"])
def test_value_types_all_aggregations(vt):
    rng = np.random.default_rng(11)
    n = 50_000
    t = TypeId[vt]
    if vt.startswith("FLOAT"):
        vals = (rng.standard_normal(n) * 100).astype(np.float32 if vt == "FLOAT32" else np.float64)
    elif vt == "BOOL8":
        vals = rng.integers(0, 2, n).astype(np.uint8)
    elif vt == "UINT64":
        vals = rng.integers(0, 2**63, n).astype(np.uint64) * 2 + 1
    else:
        info = np.iinfo(getattr(np, vt.lower()))
        vals = rng.integers(max(info.min, -10**9), min(info.max, 10**9), n).astype(getattr(np, vt.lower()))
    k = HostColumn.from_numpy(rng.integers(-50, 50, n).astype(np.int16))
    v = HostColumn.from_numpy(vals, valid=rng.random(n) > 0.3, type_id=t)
    aggs = [a for a in ALL_AGGS]
    check([k], [(v, aggs)])
    v2 = HostColumn.from_numpy(vals, type_id=t)  # no nulls: results are not nullable
    check([k], [(v2, aggs)])


@pytest.mark.parametrize("kt", ["INT8", "INT16", "INT32", "INT64", "UINT8", "UINT32", "UINT64", "FLOAT32", "FLOAT64",
                                "BOOL8", "TIMESTAMP_DAYS", "TIMESTAMP_NANOSECONDS", "DURATION_SECONDS"])
@pytest.mark.parametrize("policy", [NullPolicy.EXCLUDE, NullPolicy.INCLUDE])
def test_key_types(kt, policy):
    rng = np.random.default_rng(3)
    n = 20_000
    raw = rng.integers(0, 2 if kt == "BOOL8" else 40, n)
    k = HostColumn.from_numpy(raw, valid=rng.random(n) > 0.05, type_id=TypeId[kt])
    v = HostColumn.from_numpy(rng.integers(-1000, 1000, n).astype(np.int32), valid=rng.random(n) > 0.1)
    check([k], [(v, [Kind.SUM, Kind.MIN, Kind.MAX, Kind.COUNT_VALID, Kind.COUNT_ALL, Kind.MEAN])], policy)


def test_float_keys_zero_nan_equivalence():
    # +0 == -0 and NaN == NaN as keys (cpp/include/cudf/detail/row_operator/equality.cuh:59-89)
    keys = np.array([0.0, -0.0, np.nan, np.nan, 1.5, -1.5, 1.5, np.inf, -np.inf, np.inf] * 50, dtype=np.float64)
    vals = np.arange(keys.size, dtype=np.int64)
    got = check([HostColumn.from_numpy(keys)], [(HostColumn.from_numpy(vals), [Kind.SUM, Kind.COUNT_VALID])])
    assert got[0][0].size == 6
    check([HostColumn.from_numpy(keys.astype(np.float32))], [(HostColumn.from_numpy(vals), [Kind.SUM])])


def test_key_equal_to_empty_sentinel():
    # an int64 key of -1 has the bit pattern the table uses for "empty slot"
    rng = np.random.default_rng(9)
    n = 100_000
    k = rng.integers(-3, 3, n).astype(np.int64)
    v = rng.integers(-100, 100, n).astype(np.int64)
    for variant in (0, 1):
        got = check([HostColumn.from_numpy(k)], [(HostColumn.from_numpy(v), [Kind.SUM, Kind.MIN, Kind.COUNT_VALID])],
                    table_variant=variant)
        assert got[0][0].size == 6
    ku = np.where(rng.random(n) < 0.5, np.uint64(2**64 - 1), np.uint64(5)).astype(np.uint64)
    check([HostColumn.from_numpy(ku)], [(HostColumn.from_numpy(v), [Kind.SUM])])


def test_composite_keys_with_nulls_include_and_exclude():
    rng = np.random.default_rng(21)
    n = 80_000
    a = HostColumn.from_numpy(rng.integers(0, 5, n).astype(np.int8), valid=rng.random(n) > 0.2)
    b = HostColumn.from_numpy(rng.integers(0, 4, n).astype(np.int32), valid=rng.random(n) > 0.2)
    c = HostColumn.from_numpy(rng.integers(0, 3, n).astype(np.int16))
    v = HostColumn.from_numpy(rng.standard_normal(n).astype(np.float32), valid=rng.random(n) > 0.5)
    for policy in (NullPolicy.EXCLUDE, NullPolicy.INCLUDE):
        check([a, b, c], [(v, [Kind.SUM, Kind.MEAN, Kind.COUNT_VALID, Kind.COUNT_ALL, Kind.MAX])], policy)


def test_wide_composite_keys_use_row_comparison():
    # 3 x int64 = 192 key bits: cannot be packed, rows are compared column by column
    rng = np.random.default_rng(22)
    n = 60_000
    ks = [HostColumn.from_numpy(rng.integers(0, 6, n).astype(np.int64), valid=rng.random(n) > 0.1) for _ in range(3)]
    v = HostColumn.from_numpy(rng.integers(0, 100, n).astype(np.int32))
    for policy in (NullPolicy.EXCLUDE, NullPolicy.INCLUDE):
        check(ks, [(v, [Kind.SUM, Kind.COUNT_VALID])], policy)


def test_string_keys_with_nulls_and_duplicates():
    rng = np.random.default_rng(23)
    words = ["", "a", "ab", "abc", "abd", "año", "₹1", "x" * 40, "x" * 41, "hello world", None]
    n = 30_000
    pick = rng.integers(0, len(words), n)
    s = HostColumn.from_strings([words[i] for i in pick])
    k2 = HostColumn.from_numpy(rng.integers(0, 3, n).astype(np.int32))
    v = HostColumn.from_numpy(rng.standard_normal(n), valid=rng.random(n) > 0.1)
    for policy in (NullPolicy.EXCLUDE, NullPolicy.INCLUDE):
        check([s, k2], [(v, [Kind.SUM, Kind.COUNT_VALID, Kind.MIN, Kind.MAX, Kind.MEAN])], policy)
    s64 = HostColumn.from_strings([words[i] for i in pick], large_offsets=True)
    check([s64], [(v, [Kind.SUM])])


def test_sliced_inputs():
    # views with a non-zero element offset (cudf::slice): data and validity bits both shift
    rng = np.random.default_rng(24)
    n = 10_000
    kraw = rng.integers(0, 9, n).astype(np.int32)
    vraw = rng.standard_normal(n)
    kv, vv = rng.random(n) > 0.1, rng.random(n) > 0.1
    for off in (1, 10, 32, 45):
        k = HostColumn.from_numpy(kraw, valid=kv, offset=off)
        v = HostColumn.from_numpy(vraw, valid=vv, offset=off + 3)
        check([k], [(v, ALL_AGGS)])
        check([k], [(v, ALL_AGGS)], NullPolicy.INCLUDE)


def test_high_cardinality_grows_the_table():
    import cudf_b200 as cb
    rng = np.random.default_rng(25)
    n = 1_400_000
    k = HostColumn.from_numpy(rng.permutation(n).astype(np.int64) * 7919)  # all distinct
    v = HostColumn.from_numpy(rng.integers(-5, 5, n).astype(np.int64))
    got = check([k], [(v, [Kind.SUM, Kind.MIN, Kind.MAX, Kind.COUNT_VALID])])
    assert got[0][0].size == n
    assert cb.last_call_stats().table_attempts == 2  # the speculative table overflowed, the estimated one fit
    got = check([k], [(v, [Kind.SUM])], expected_groups=n)
    assert cb.last_call_stats().table_attempts == 1


def test_skewed_keys_hot_group():
    w = workloads.make(4, 800_000, scale_domain=True)
    check(w.keys, w.requests)
    # one key holds 90 % of the rows
    rng = np.random.default_rng(26)
    n = 500_000
    k = np.where(rng.random(n) < 0.9, 7, rng.integers(0, 100_000, n)).astype(np.int64)
    v = HostColumn.from_numpy(rng.lognormal(0, 1, n), valid=rng.random(n) > 0.01)
    check([HostColumn.from_numpy(k)], [(v, [Kind.SUM, Kind.MEAN, Kind.VARIANCE, Kind.MIN, Kind.MAX])])


def test_dense_key_box_with_outliers_and_negative_keys():
    # the shared-memory slot of a key is its position in a box found from a row sample; keys the
    # sample missed (here: 30 far-away keys at unsampled rows) must still aggregate exactly
    rng = np.random.default_rng(31)
    n = 2_000_000
    a = rng.integers(-40, 40, n).astype(np.int32)
    b = rng.integers(1000, 1050, n).astype(np.int64)
    odd = rng.choice(n, 30, replace=False)
    a[odd] = rng.integers(-2**31, 2**31 - 1, 30)
    b[odd[:10]] = rng.integers(-2**62, 2**62, 10)
    v = HostColumn.from_numpy(rng.standard_normal(n).astype(np.float32), valid=rng.random(n) > 0.1)
    w = HostColumn.from_numpy(rng.integers(-100, 100, n).astype(np.int64), valid=rng.random(n) > 0.1)
    ka = HostColumn.from_numpy(a, valid=rng.random(n) > 0.01)
    kb = HostColumn.from_numpy(b)
    for policy in (NullPolicy.EXCLUDE, NullPolicy.INCLUDE):
        check([ka, kb], [(v, [Kind.MEAN])], policy)
        check([ka, kb], [(v, [Kind.SUM, Kind.MIN, Kind.MAX]), (w, [Kind.SUM, Kind.COUNT_ALL, Kind.VARIANCE])], policy)


def test_float32_sum_spills_to_fp64():
    # one group with far more than 1024 addends per CTA exercises the fp32 -> fp64 spill of the
    # compact shared-memory layout; the mean must stay within the fp32 tolerance of the exact one
    rng = np.random.default_rng(27)
    n = 3_000_000
    k = HostColumn.from_numpy(np.zeros(n, dtype=np.int32))
    k2 = HostColumn.from_numpy((rng.random(n) < 0.001).astype(np.int32))
    v = HostColumn.from_numpy((rng.random(n) * 1000).astype(np.float32), valid=rng.random(n) > 0.02)
    check([k, k2], [(v, [Kind.MEAN])], row_filters=[v])
    check([k, k2], [(v, [Kind.SUM, Kind.COUNT_VALID])])


def test_float64_mean_keeps_its_sum_as_fixed_point_limbs():
    """Σ and n of one FLOAT64 column over a sampled key box: the lean kernel keeps each partial sum as
    fixed-point limbs whose window comes from the sampled values.  Register tiles (4), the bulk-copy ring (5)
    and auto (0); values far outside the window, zeros, denormals, infinities and NaN (added to the fp64
    cells directly); a group with many thousand addends per CTA (the limbs are emptied every 1024); nullable
    keys under both policies and keys the sample missed; a box that only the generic kernel's table holds
    (8000 keys), and one that neither holds (40000 keys)."""
    rng = np.random.default_rng(83)
    n = 1_500_000
    x = rng.standard_normal(n) * np.exp(rng.standard_normal(n))
    x[rng.random(n) < 0.01] = 0.0
    x[rng.random(n) < 0.001] *= 1e-30
    x[rng.random(n) < 0.001] *= 1e25
    x[rng.random(n) < 0.0005] = 5e-324
    k = rng.integers(0, 1000, n).astype(np.int64)
    x[(k == 5) & (rng.random(n) < 0.01)] = np.inf
    x[(k == 6) & (rng.random(n) < 0.01)] = -np.inf
    x[(k == 7) & (rng.random(n) < 0.01)] = np.nan
    v = HostColumn.from_numpy(x, valid=rng.random(n) > 0.05)
    aggs = [Kind.SUM, Kind.COUNT_VALID, Kind.MEAN]
    for variant in (0, 4, 5):
        got = check([HostColumn.from_numpy(k)], [(v, aggs)], table_variant=variant)
        assert got[0][0].size == 1000
        check([HostColumn.from_numpy(k)], [(v, [Kind.MEAN])], row_filters=[v], table_variant=variant)
    # one group takes 99.9 % of the rows
    hot = HostColumn.from_numpy((rng.random(n) < 0.001).astype(np.int32))
    zero = HostColumn.from_numpy(np.zeros(n, dtype=np.int64))
    check([zero, hot], [(v, aggs)])
    tame = HostColumn.from_numpy(rng.standard_normal(n) * 1e-3 + 1.0)        # every value inside the window
    check([zero, hot], [(tame, aggs)])
    # nullable keys, keys far outside the sampled box
    a = rng.integers(-40, 40, n).astype(np.int32)
    b = rng.integers(1000, 1012, n).astype(np.int64)
    odd = rng.choice(n, 30, replace=False)
    a[odd] = rng.integers(-2**31, 2**31 - 1, 30)
    b[odd[:10]] = rng.integers(-2**62, 2**62, 10)
    ka = HostColumn.from_numpy(a, valid=rng.random(n) > 0.01)
    for policy in (NullPolicy.EXCLUDE, NullPolicy.INCLUDE):
        check([ka, HostColumn.from_numpy(b)], [(v, aggs)], policy)
    # key boxes wider than the limbs' table
    for distinct in (8000, 40_000):
        wide = HostColumn.from_numpy(rng.integers(0, distinct, n).astype(np.int32))
        assert check([wide], [(v, aggs)])[0][0].size == distinct


@pytest.mark.parametrize("vtype", ["INT8", "INT16", "INT32", "INT64", "DECIMAL32", "DECIMAL64"])
def test_sum_overflow_struct_results(vtype):
    """SUM_OVERFLOW (cpp/tests/groupby/sum_overflow_tests.cpp): a struct {sum in the source type, overflow flag}
    per group.  Values large enough that some groups leave the source type's range and others do not, null
    values (groups without a valid value give a null struct), both null policies, beside SUM / MEAN of the same
    column, on the table paths and the partitioned path; then 5000 groups of ten ones (MultiBlock, :440)."""
    t = TypeId[vtype]
    rng = np.random.default_rng(91)
    n = 300_000
    dt = np.dtype(H.STORAGE_DTYPE[t])
    info = np.iinfo(dt)
    k = HostColumn.from_numpy(rng.integers(0, 3000, n).astype(np.int32), valid=rng.random(n) > 0.02)
    # ~100 rows per group: magnitudes up to max / 40 overflow in some groups only; one sign per group,
    # so that every arrival order of the reference gives the same flag
    sign = np.where((k.values() % 3) == 0, -1, 1)
    mag = rng.integers(0, int(info.max) // 40, n, dtype=np.int64)
    x = (sign * mag).astype(dt)
    valid = rng.random(n) > 0.1
    valid[k.values() == 17] = False          # a group without a valid value
    scale = -2 if vtype.startswith("DECIMAL") else 0
    v = HostColumn.from_numpy(x, valid=valid, type_id=t, scale=scale)
    for policy in (NullPolicy.EXCLUDE, NullPolicy.INCLUDE):
        for variant in (0, 1, 3, 6):
            got = check([k], [(v, [Kind.SUM_OVERFLOW, Kind.SUM, Kind.COUNT_VALID])], policy, table_variant=variant)
            st = got[1][0][0]
            assert st.type_id == TypeId.STRUCT and st.null_count == 1 and st.children[0].scale == scale
            flags = st.children[1].values()
            assert 0 < int(flags.sum()) < flags.size
    ones = HostColumn.from_numpy(np.ones(50_000, dtype=dt), type_id=t, scale=scale)
    k5 = HostColumn.from_numpy((np.arange(50_000) % 5000).astype(np.int32))
    got = check([k5], [(ones, [Kind.SUM_OVERFLOW])])
    assert (got[1][0][0].children[0].values() == 10).all() and not got[1][0][0].children[1].values().any()


def test_decimal128_sums():
    """SUM and SUM_OVERFLOW of DECIMAL128 values (the reference serves them on its hash path,
    cpp/src/groupby/hash/groupby.cu:82-85; cpp/tests/groupby/sum_tests.cpp:220-247,250-290 sums a DECIMAL128
    column beside an INT32 column): 16-byte elements read as two word columns, four exact chunk sums per
    group.  Magnitudes up to 2^120 with one sign per group, so that some groups leave the 128-bit range; null
    values, a sliced column, both null policies, the table paths and the partitioned path.  MIN of DECIMAL128
    is the reference's sort path: not served."""
    import cudf_b200 as cb
    from cudf_b200 import aggregation as agg
    from cudf_b200.types import int128_array, int128_list
    rng = np.random.default_rng(101)
    n = 120_000
    kv = rng.integers(0, 400, n).astype(np.int32)
    k = HostColumn.from_numpy(kv, valid=rng.random(n) > 0.02)
    hi = rng.integers(0, 2 ** 56, n, dtype=np.int64).tolist()
    lo = rng.integers(0, 2 ** 63, n, dtype=np.int64).tolist()
    sign = np.where(kv % 3 == 0, -1, 1).tolist()
    small = (kv % 5 == 0).tolist()                     # every fifth group stays far inside the range
    ints = [sg * (l if sm else ((h << 64) | l)) for h, l, sg, sm in zip(hi, lo, sign, small)]
    valid = rng.random(n) > 0.1
    valid[kv == 17] = False
    d = HostColumn.from_numpy(int128_array(ints), valid=valid, type_id=TypeId.DECIMAL128, offset=3, scale=-4)
    w = HostColumn.from_numpy(rng.integers(-100, 100, n).astype(np.int32))
    reqs = [(w, [Kind.SUM]), (d, [Kind.SUM, Kind.SUM_OVERFLOW, Kind.COUNT_VALID])]
    for policy in (NullPolicy.EXCLUDE, NullPolicy.INCLUDE):
        for variant in (0, 1, 3, 6):
            got = check([k], reqs, policy, table_variant=variant)
            total, st = got[1][1][0], got[1][1][1]
            assert total.type_id == TypeId.DECIMAL128 and total.scale == -4 and st.children[0].scale == -4
            flags = st.children[1].values()[st.valid()]
            assert 0 < int(flags.sum()) < flags.size
    # one group against Python integers
    gk, gr = H.gpu_groupby([k], reqs)
    g0 = int(np.flatnonzero(gk[0].values() == 5)[0])
    exact = sum(v for v, kk, ok, kok in zip(ints, kv.tolist(), valid.tolist(), k.valid().tolist()) if kk == 5 and ok and kok)
    assert int128_list(gr[1][0].values())[g0] == exact
    kk = cb.Column.from_host(k)
    with pytest.raises(cb.UnsupportedError):
        cb.GroupBy(cb.Table([kk])).aggregate([cb.GroupByRequest(cb.Column.from_host(d), [agg.min()])])


def test_sum_overflow_rejects_bool_and_unsigned_values():
    # cpp/tests/groupby/sum_overflow_tests.cpp:495-561: cudf::logic_error for BOOL8, UINT32, UINT64
    import cudf_b200 as cb
    from cudf_b200 import aggregation as agg
    k = cb.Column.from_host(HostColumn.from_numpy(np.array([1, 1, 1], dtype=np.int32)))
    gb = cb.GroupBy(cb.Table([k]))
    for vals in (np.array([True, False, True]), np.array([1, 2, 3], dtype=np.uint32), np.array([1, 2, 3], dtype=np.uint64),
                 np.array([1.0, 2.0, 3.0])):
        v = cb.Column.from_host(HostColumn.from_numpy(vals))
        with pytest.raises(cb.LogicError, match="Invalid type/aggregation combination."):
            gb.aggregate([cb.GroupByRequest(v, [agg.sum_overflow()])])


def test_dictionary_values_are_looked_up_by_key():
    """DICTIONARY32 value columns with fixed-width keys: the results are those of the column of looked-up keys, in
    the keys' type (cpp/include/cudf/detail/aggregation/device_aggregators.cuh:189-220,
    cpp/src/groupby/hash/output_utils.cu:65-66).  The reference's own vectors (mean_tests.cpp:128-147,
    max_tests.cpp:226-246, count_tests.cpp:185-207), then nullable and sliced dictionaries with INT8 / INT32 /
    UINT32 / INT64 indices against the oracle on the decoded column; a dictionary of strings is not served."""
    import cudf_b200 as cb
    from cudf_b200 import aggregation as agg
    k = HostColumn.from_numpy(np.array([1, 2, 3, 1, 2, 2, 1, 3, 3, 2], dtype=np.int32))
    gk, gr = H.gpu_groupby([k], [(HostColumn.from_dictionary(np.arange(10, dtype=np.int16)), [Kind.MEAN])])
    order = H.sort_order(gk)
    assert H.take(gk[0], order) == [1, 2, 3] and H.take(gr[0][0], order) == [9.0 / 3, 19.0 / 4, 17.0 / 3]
    big = np.array([0xABC, 0xBBB, 0xF1, 0xAAA, 0xFFF, 0xBAA, 0xAAA, 0x01, 0xF1, 0xEEE], dtype=np.int64)
    gk, gr = H.gpu_groupby([k], [(HostColumn.from_dictionary(big), [Kind.MAX, Kind.MIN])])
    order = H.sort_order(gk)
    assert gr[0][0].type_id == TypeId.INT64 and H.take(gr[0][0], order) == [0xABC, 0xFFF, 0xF1]
    assert H.take(gr[0][1], order) == [0xAAA, 0xBAA, 0x01]
    sk = HostColumn.from_strings(["1", "3", "3", "5", "5", "0"])
    gk, gr = H.gpu_groupby([sk], [(HostColumn.from_dictionary(np.ones(6, dtype=np.int32)), [Kind.COUNT_VALID])])
    order = H.sort_order(gk)
    assert H.take(gk[0], order) == [b"0", b"1", b"3", b"5"] and H.take(gr[0][0], order) == [1, 1, 2, 2]

    rng = np.random.default_rng(97)
    n = 200_000
    keys = HostColumn.from_numpy(rng.integers(0, 500, n).astype(np.int32))
    pool = rng.standard_normal(120)
    x = pool[rng.integers(0, pool.size, n)]
    valid = rng.random(n) > 0.1
    for index_type, offset in ((TypeId.INT8, 0), (TypeId.INT32, 3), (TypeId.UINT32, 0), (TypeId.INT64, 64)):
        d = HostColumn.from_dictionary(x, valid=valid, index_type=index_type, offset=offset)
        plain = HostColumn.from_numpy(x, valid=valid)
        reqs_d = [(d, ALL_AGGS), (d, [Kind.SUM])]
        reqs_p = [(plain, ALL_AGGS), (plain, [Kind.SUM])]
        got = H.gpu_groupby([keys], reqs_d)
        exp = oracle.groupby([keys], reqs_p)
        H.assert_same_result(got, exp, reqs_p, scales=H.result_scales([keys], reqs_p, NullPolicy.EXCLUDE))
    ints = rng.integers(-50, 50, n).astype(np.int32)
    di = HostColumn.from_dictionary(ints, valid=valid)
    pi = HostColumn.from_numpy(ints, valid=valid)
    got = H.gpu_groupby([keys], [(di, [Kind.SUM, Kind.SUM_OVERFLOW, Kind.PRODUCT, Kind.ARGMIN])], table_variant=6)
    exp = oracle.groupby([keys], [(pi, [Kind.SUM, Kind.SUM_OVERFLOW, Kind.PRODUCT, Kind.ARGMIN])])
    H.assert_same_result(got, exp, [(pi, [Kind.SUM, Kind.SUM_OVERFLOW, Kind.PRODUCT, Kind.ARGMIN])])
    # the same indices and keys under two different masks in one call
    valid2 = rng.random(n) > 0.5
    full = cb.Column.from_host(HostColumn.from_dictionary(ints))     # every row's index is meaningful
    m1 = cb.Column.from_host(pi).mask
    m2 = cb.Column.from_host(HostColumn.from_numpy(ints, valid=valid2)).mask
    c1 = cb.Column(TypeId.DICTIONARY32, n, None, m1, 0, int(n - valid.sum()), children=full.children)
    c2 = cb.Column(TypeId.DICTIONARY32, n, None, m2, 0, int(n - valid2.sum()), children=full.children)
    dk = cb.Table([cb.Column.from_host(keys)])
    okeys, ores = cb.GroupBy(dk).aggregate([cb.GroupByRequest(c1, [agg.sum()]), cb.GroupByRequest(c2, [agg.sum()])])
    got = ([c.to_host() for c in okeys.columns()], [[c.to_host() for c in t.columns()] for t in ores])
    p2 = HostColumn.from_numpy(ints, valid=valid2)
    H.assert_same_result(got, oracle.groupby([keys], [(pi, [Kind.SUM]), (p2, [Kind.SUM])]), [(pi, [Kind.SUM]), (p2, [Kind.SUM])])


def _string_dictionary(strings, index_type=TypeId.INT32):
    uniq = sorted(set(s for s in strings if s is not None), key=lambda s: s.encode())
    pos = {s: i for i, s in enumerate(uniq)}
    idx = np.array([pos.get(s, 0) for s in strings]).astype(H.STORAGE_DTYPE[TypeId(index_type)])
    valid = np.array([s is not None for s in strings], dtype=bool)
    return HostColumn(TypeId.DICTIONARY32, len(strings), None, None if valid.all() else H.pack_mask(valid), 0, None, 0,
                      [HostColumn.from_numpy(idx, type_id=index_type), HostColumn.from_strings(uniq)]), uniq


def test_dictionaries_of_strings_take_part_through_their_indices():
    """The keys of a dictionary column are sorted and unique, so MIN / MAX / ARGMIN / ARGMAX of its strings are
    those of its indices; MIN / MAX come back as dictionary columns over the same keys
    (cpp/tests/groupby/max_tests.cpp:198-224, min_tests.cpp:190-216, argmax_tests.cpp:145-170,
    argmin_tests.cpp:146-171).  Other aggregations of such a column are not served."""
    import cudf_b200 as cb
    from cudf_b200 import aggregation as agg
    k = HostColumn.from_numpy(np.array([1, 2, 3, 1, 2, 2, 1, 3, 3, 2], dtype=np.int32))

    def strings_of(col, order):
        idx, keys = col.children
        words = keys.to_pylist()
        return [words[i].decode() if ok else None for i, ok in zip(idx.values()[order].tolist(), col.valid()[order].tolist())]

    d, uniq = _string_dictionary(["año", "bit", "₹1", "aaa", "zit", "bat", "aaa", "$1", "₹1", "wut"], TypeId.UINT32)
    gk, gr = H.gpu_groupby([k], [(d, [Kind.MAX, Kind.MIN, Kind.COUNT_VALID])])
    order = H.sort_order(gk)
    assert gr[0][0].type_id == TypeId.DICTIONARY32 and gr[0][0].children[0].type_id == TypeId.UINT32
    assert [w.decode() for w in gr[0][0].children[1].to_pylist()] == uniq         # the keys are the input's
    assert strings_of(gr[0][0], order) == ["año", "zit", "₹1"] and strings_of(gr[0][1], order) == ["aaa", "bat", "$1"]
    assert H.take(gr[0][2], order) == [3, 4, 3]
    d, _ = _string_dictionary(["año", "bit", "₹1", "aaa", "zit", "bat", "aab", "$1", "€1", "wut"])
    gk, gr = H.gpu_groupby([k], [(d, [Kind.ARGMAX, Kind.ARGMIN])])
    order = H.sort_order(gk)
    assert H.take(gr[0][0], order) == [0, 4, 2] and H.take(gr[0][1], order) == [3, 5, 7]
    # many rows, nulls, a group without a valid value: against the oracle on the plain strings
    rng = np.random.default_rng(103)
    n = 60_000
    pool = ["w%04d" % i for i in range(3000)] + ["", "é", "日本"]
    words = [None if rng.random() < 0.1 else pool[i] for i in rng.integers(0, len(pool), n)]
    kv = rng.integers(0, 700, n).astype(np.int32)
    for i in np.flatnonzero(kv == 13):
        words[i] = None
    d, _ = _string_dictionary(words)
    plain = HostColumn.from_strings(words)
    keys = HostColumn.from_numpy(kv)
    gk, gr = H.gpu_groupby([keys], [(d, [Kind.MIN, Kind.MAX, Kind.ARGMIN, Kind.COUNT_VALID])])
    ek, er = oracle.groupby([keys], [(plain, [Kind.MIN, Kind.MAX, Kind.ARGMIN, Kind.COUNT_VALID])])
    og, oe = H.sort_order(gk), H.sort_order(ek)
    H.assert_keys_equal(gk, ek, og, oe)
    for a in (0, 1):
        exp = [w.decode() if w is not None else None for w in H.take(er[0][a], oe)]
        assert strings_of(gr[0][a], og) == exp and gr[0][a].null_count == 1
    assert H.take(gr[0][2], og) == H.take(er[0][2], oe) and H.take(gr[0][3], og) == H.take(er[0][3], oe)
    kk = cb.Column.from_host(k)
    d, _ = _string_dictionary(["a", "b"] * 5)
    with pytest.raises(cb.UnsupportedError):
        cb.GroupBy(cb.Table([kk])).aggregate([cb.GroupByRequest(cb.Column.from_host(d), [agg.sum()])])


def test_dictionary_key_columns_group_by_their_indices():
    """DICTIONARY32 key columns (cpp/tests/groupby/keys_tests.cpp:324-347): the keys of a dictionary are unique, so
    rows group by their indices, and the finished key column is a dictionary over the same keys.  The reference's
    vector, then a nullable dictionary of strings beside an INT8 key and a dictionary of FLOAT64 under both null
    policies, against the oracle on the plain columns."""
    def decode(col):
        idx, keys = col.children
        words = keys.to_pylist()
        return [words[i] if ok else None for i, ok in zip(idx.values().tolist(), col.valid().tolist())]

    d, uniq = _string_dictionary(["aaa", "año", "₹1", "aaa", "año", "año", "aaa", "₹1", "₹1", "año"])
    v = HostColumn.from_numpy(np.arange(10, dtype=np.int32))
    gk, gr = H.gpu_groupby([d], [(v, [Kind.SUM])])
    assert gk[0].type_id == TypeId.DICTIONARY32 and [w.decode() for w in gk[0].children[1].to_pylist()] == uniq
    got = dict(zip([w.decode() for w in decode(gk[0])], gr[0][0].values().tolist()))
    assert got == {"aaa": 9, "año": 19, "₹1": 17}

    rng = np.random.default_rng(107)
    n = 80_000
    pool = ["k%03d" % i for i in range(400)] + ["", "é"]
    words = [None if rng.random() < 0.05 else pool[i] for i in rng.integers(0, len(pool), n)]
    d, _ = _string_dictionary(words, TypeId.UINT16)
    k2 = HostColumn.from_numpy(rng.integers(0, 3, n).astype(np.int8))
    x = rng.standard_normal(n)
    val = HostColumn.from_numpy(x, valid=rng.random(n) > 0.1)
    fpool = rng.standard_normal(50)
    fvals = fpool[rng.integers(0, 50, n)]
    fvalid = rng.random(n) > 0.03
    fd = HostColumn.from_dictionary(fvals, valid=fvalid)
    reqs = [(val, ALL_AGGS)]
    for policy in (NullPolicy.EXCLUDE, NullPolicy.INCLUDE):
        gk, gr = H.gpu_groupby([d, k2, fd], reqs, policy)
        plain = [HostColumn.from_strings(words), k2, HostColumn.from_numpy(fvals, valid=fvalid)]
        ek, er = oracle.groupby(plain, reqs, policy)
        assert gk[0].type_id == TypeId.DICTIONARY32 and gk[2].type_id == TypeId.DICTIONARY32
        f_dec = decode(gk[2])
        back = [HostColumn.from_strings([None if w is None else w.decode() for w in decode(gk[0])]), gk[1],
                HostColumn.from_numpy(np.array([0.0 if f is None else f for f in f_dec]),
                                      valid=np.array([f is not None for f in f_dec]) if policy == NullPolicy.INCLUDE else None)]
        H.assert_same_result((back, gr), (ek, er), reqs, check_nullable=False,
                             scales=H.result_scales(plain, reqs, policy))


def test_min_max_with_nan_and_infinity_terminate():
    # cpp/tests/groupby/min_tests.cpp:518-541, max_tests.cpp:526-549: all-NaN groups must not hang
    keys = HostColumn.from_numpy(np.array([1, 1, 2, 2, 2], dtype=np.int32))
    vals = HostColumn.from_numpy(np.array([np.nan, np.nan, 1.0, -np.inf, np.inf]))
    gk, gr = H.gpu_groupby([keys], [(vals, [Kind.MIN, Kind.MAX])])
    order = H.sort_order(gk)
    assert gk[0].size == 2
    assert H.take(gr[0][0], order)[1] == -np.inf and H.take(gr[0][1], order)[1] == np.inf


def test_multiple_requests_and_duplicates():
    # cpp/tests/groupby/keys_tests.cpp:355-409: repeated aggregations / repeated columns
    rng = np.random.default_rng(28)
    n = 40_000
    k = HostColumn.from_numpy(rng.integers(0, 50, n).astype(np.int32))
    v1 = HostColumn.from_numpy(rng.integers(0, 100, n).astype(np.int32))
    v2 = HostColumn.from_numpy(rng.standard_normal(n), valid=rng.random(n) > 0.2)
    check([k], [(v1, [Kind.SUM, Kind.SUM]), (v1, [Kind.SUM, Kind.MAX]), (v2, [Kind.MEAN, Kind.STD]), (v2, [Kind.MIN])])


def test_many_value_columns_generic_shared_layout():
    rng = np.random.default_rng(29)
    n = 200_000
    k = HostColumn.from_numpy(rng.integers(0, 300, n).astype(np.int32))
    reqs = []
    for i in range(6):
        v = HostColumn.from_numpy(rng.standard_normal(n) * (i + 1), valid=rng.random(n) > 0.1 * i if i else None)
        reqs.append((v, [Kind.SUM, Kind.MIN, Kind.MAX, Kind.MEAN, Kind.VARIANCE]))
    check([k], reqs)


def test_row_filters_drop_rows():
    rng = np.random.default_rng(30)
    n = 100_000
    k = HostColumn.from_numpy(rng.integers(0, 20, n).astype(np.int32))
    v = HostColumn.from_numpy(rng.standard_normal(n), valid=rng.random(n) > 0.3)
    w = HostColumn.from_numpy(rng.integers(0, 9, n).astype(np.int64), valid=rng.random(n) > 0.3)
    check([k], [(v, [Kind.SUM, Kind.COUNT_ALL]), (w, [Kind.SUM, Kind.COUNT_VALID])], row_filters=[v, w])


@pytest.mark.parametrize("policy", [NullPolicy.EXCLUDE, NullPolicy.INCLUDE])
def test_decimal_values_and_keys_keep_type_and_scale(policy):
    """Fixed point columns are aggregated on their integer representation; SUM / MIN / MAX results
    and decimal keys keep type and scale; a DECIMAL32 sum wraps at 32 bits like the reference's
    int32 accumulator (cpp/include/cudf/detail/aggregation/aggregation.hpp:956-963)."""
    rng = np.random.default_rng(77)
    n = 200_000
    k = HostColumn.from_numpy(rng.integers(-500, 500, n).astype(np.int64), valid=rng.random(n) > 0.01,
                              type_id=TypeId.DECIMAL64, scale=-3)
    v32 = HostColumn.from_numpy(rng.integers(-2**30, 2**30, n).astype(np.int32), valid=rng.random(n) > 0.1,
                                type_id=TypeId.DECIMAL32, scale=-2)
    v64 = HostColumn.from_numpy(rng.integers(-10**12, 10**12, n).astype(np.int64), type_id=TypeId.DECIMAL64, scale=4)
    reqs = [(v32, [Kind.SUM, Kind.MIN, Kind.MAX, Kind.COUNT_VALID]), (v64, [Kind.SUM, Kind.MIN, Kind.MAX, Kind.COUNT_ALL])]
    gkeys, gres = check([k], reqs, policy)
    assert gkeys[0].type_id == TypeId.DECIMAL64 and gkeys[0].scale == -3
    assert [c.type_id for c in gres[0]] == [TypeId.DECIMAL32, TypeId.DECIMAL32, TypeId.DECIMAL32, TypeId.INT32]
    assert [c.scale for c in gres[0]] == [-2, -2, -2, 0]
    assert [c.scale for c in gres[1]] == [4, 4, 4, 0]


def test_error_statuses_mirror_the_reference():
    import cudf_b200 as cb
    from cudf_b200 import aggregation as agg
    k = cb.Column.from_host(HostColumn.from_numpy(np.arange(4, dtype=np.int32)))
    v5 = cb.Column.from_host(HostColumn.from_numpy(np.arange(5, dtype=np.int32)))
    s = cb.Column.from_host(HostColumn.from_strings(["a", "b", "c", "d"]))
    gb = cb.GroupBy(cb.Table([k]))
    with pytest.raises(cb.LogicError, match="Size mismatch between request values and groupby keys."):
        gb.aggregate([cb.GroupByRequest(v5, [agg.sum()])])
    # CUDF_EXPECTS with the default exception type: cudf::logic_error (cpp/src/groupby/groupby.cu:185-201)
    with pytest.raises(cb.LogicError, match="Invalid type/aggregation combination."):
        gb.aggregate([cb.GroupByRequest(s, [agg.sum()])])
    # fixed point: SUM / MIN / MAX are served, PRODUCT throws (cpp/tests/groupby/sum_tests.cpp:245-246)
    d = cb.Column.from_host(HostColumn.from_numpy(np.arange(4, dtype=np.int32), type_id=TypeId.DECIMAL32, scale=-2))
    with pytest.raises(cb.LogicError, match="Invalid type/aggregation combination."):
        gb.aggregate([cb.GroupByRequest(d, [agg.product()])])
    with pytest.raises(cb.UnsupportedError):
        gb.aggregate([cb.GroupByRequest(d, [agg.mean()])])
    with pytest.raises(cb.UnsupportedError):
        gb.aggregate([cb.GroupByRequest(k, [agg.median()])])
    with pytest.raises(cb.UnsupportedError):
        gb.aggregate([cb.GroupByRequest(s, [agg.nth_element(0)])])
    # MIN / MAX of strings are served by the hash path (cpp/src/groupby/hash/hash_compound_agg_finalizer.cu:39-91)
    assert gb.aggregate([cb.GroupByRequest(s, [agg.min()])])[1][0].columns()[0].size == 4


def test_results_are_deterministic_for_integers():
    w = workloads.make(3, 400_000, scale_domain=True)
    a = H.gpu_groupby(w.keys, w.requests)
    b = H.gpu_groupby(w.keys, w.requests)
    oa, ob = H.sort_order(a[0]), H.sort_order(b[0])
    for x, y in zip(a[1][0], b[1][0]):
        assert H.take(x, oa) == H.take(y, ob)


# ------------------------------------------------------------------------------------ partitioned path
def _partition_inputs(seed, n, domain, nullable_keys=False):
    rng = np.random.default_rng(seed)
    # int64 keys include -1, whose bits equal the empty-slot marker; nullable keys are int32 so that key +
    # null flag still pack into 64 bits under INCLUDE
    kv = rng.integers(-1, domain, n).astype(np.int32 if nullable_keys else np.int64)
    k = HostColumn.from_numpy(kv, valid=(rng.random(n) > 0.02) if nullable_keys else None)
    v1 = HostColumn.from_numpy(rng.integers(-10**9, 10**9, n).astype(np.int64))
    v2 = HostColumn.from_numpy(rng.lognormal(0, 1, n), valid=rng.random(n) > 0.05)
    v3 = HostColumn.from_numpy(rng.integers(-100, 100, n).astype(np.int16), valid=rng.random(n) > 0.3)
    return k, v1, v2, v3


@pytest.mark.parametrize("table_bytes", [0, 16384])
@pytest.mark.parametrize("policy", [NullPolicy.EXCLUDE, NullPolicy.INCLUDE])
def test_partitioned_path_matches_oracle(table_bytes, policy):
    """table_variant 6 forces the radix-partitioned path; 16 KB tables force its second level
    (300K groups / 128 per bucket = 12 digit bits)."""
    import cudf_b200 as cb
    k, v1, v2, v3 = _partition_inputs(21, 700_000, 400_000, nullable_keys=True)
    reqs = [(v1, [Kind.SUM, Kind.MIN, Kind.MAX, Kind.COUNT_VALID]), (v2, [Kind.SUM, Kind.MEAN, Kind.VARIANCE, Kind.COUNT_ALL]),
            (v3, [Kind.SUM, Kind.MIN, Kind.MAX, Kind.MEAN, (Kind.STD, 0), Kind.SUM_OF_SQUARES])]
    got = check([k], reqs, policy, table_variant=6, shared_table_bytes=table_bytes)
    st = cb.last_call_stats()
    assert st.table_attempts == 1 and not st.used_shared_table      # one partitioned pass, no table fallback
    assert got[0][0].size > 300_000


@pytest.mark.parametrize("table_bytes", [0, 16384])
def test_partitioned_path_int64_keys_with_the_empty_marker_key(table_bytes):
    import cudf_b200 as cb
    k, v1, v2, v3 = _partition_inputs(25, 600_000, 400_000)
    assert (k.values() == -1).any()
    check([k], [(v1, [Kind.SUM, Kind.MIN, Kind.MAX, Kind.COUNT_VALID]), (v2, [Kind.MEAN, Kind.M2]), (v3, [Kind.SUM, Kind.COUNT_ALL])],
          table_variant=6, shared_table_bytes=table_bytes)
    st = cb.last_call_stats()
    assert st.table_attempts == 1 and not st.used_shared_table


def test_partitioned_path_composite_keys_and_row_filters():
    rng = np.random.default_rng(22)
    n = 500_000
    a = HostColumn.from_numpy(rng.integers(0, 3000, n).astype(np.int32))
    b = HostColumn.from_numpy(rng.integers(-50, 50, n).astype(np.int16), valid=rng.random(n) > 0.1)
    v = HostColumn.from_numpy(rng.standard_normal(n).astype(np.float32), valid=rng.random(n) > 0.2)
    for policy in (NullPolicy.EXCLUDE, NullPolicy.INCLUDE):
        check([a, b], [(v, ALL_AGGS)], policy, row_filters=[v], table_variant=6)
    check([a, b], [(v, ALL_AGGS)], table_variant=6, shared_table_bytes=20000)


def test_partitioned_path_falls_back_when_the_hint_is_far_too_low():
    """A hint of 1000 groups for 300K: buckets overflow their shared-memory tables, the attempt is
    discarded and the global table takes over — same result."""
    import cudf_b200 as cb
    k, v1, v2, _ = _partition_inputs(23, 600_000, 400_000)
    got = check([k], [(v1, [Kind.SUM, Kind.MAX]), (v2, [Kind.MEAN])], table_variant=6, expected_groups=1000)
    assert got[0][0].size > 250_000


def test_partitioned_path_few_rows_and_skew():
    rng = np.random.default_rng(24)
    for n in (1, 5, 4097, 70_000):
        k = HostColumn.from_numpy(np.where(rng.random(n) < 0.5, 7, rng.integers(0, 50_000, n)).astype(np.int64))
        v = HostColumn.from_numpy(rng.standard_normal(n), valid=rng.random(n) > 0.1)
        check([k], [(v, ALL_AGGS)], table_variant=6)


# ------------------------------------------------------------------------------------ ARGMIN / ARGMAX, MIN / MAX of strings
def test_argmin_argmax_and_string_min_max():
    """Row-index accumulators (cpp/src/groupby/hash/extract_single_pass_aggs.cpp:39-60): the first row of the
    extreme value wins on ties, so the result is the oracle's whatever the arrival order on the GPU."""
    rng = np.random.default_rng(31)
    n = 80_000
    words = ["", "a", "aa", "año", "b", "日本", "日本語", "z" * 40, "ab", "abc", "abd", "Ab", "$1", "€1", "₹1"]
    k = HostColumn.from_numpy(rng.integers(0, 700, n).astype(np.int32), valid=rng.random(n) > 0.05)
    vi = HostColumn.from_numpy(rng.integers(-20, 20, n).astype(np.int16), valid=rng.random(n) > 0.3)      # many ties
    vf = HostColumn.from_numpy(rng.integers(-50, 50, n).astype(np.float64) / 4)
    vu = HostColumn.from_numpy(rng.integers(0, 2**63, n).astype(np.uint64) * np.uint64(2))
    vs = HostColumn.from_strings([None if rng.random() < 0.2 else words[i] + words[j]
                                  for i, j in zip(rng.integers(0, len(words), n), rng.integers(0, len(words), n))])
    reqs = [(vi, [Kind.ARGMIN, Kind.ARGMAX, Kind.MIN, Kind.SUM, Kind.COUNT_VALID]), (vf, [Kind.ARGMAX, Kind.ARGMIN, Kind.MEAN]),
            (vu, [Kind.ARGMIN, Kind.ARGMAX]), (vs, [Kind.MIN, Kind.MAX, Kind.ARGMIN, Kind.ARGMAX, Kind.COUNT_VALID])]
    for policy in (NullPolicy.EXCLUDE, NullPolicy.INCLUDE):
        got = check([k], reqs, policy)
        assert TypeId(got[1][3][0].type_id) == TypeId.STRING and TypeId(got[1][3][2].type_id) == TypeId.INT32
    # string keys with string values, and an empty input
    ks = HostColumn.from_strings([words[i] for i in rng.integers(0, len(words), n)])
    check([ks, k], [(vs, [Kind.MAX, Kind.MIN]), (vi, [Kind.ARGMIN])], NullPolicy.INCLUDE)
    empty = HostColumn.from_numpy(np.zeros(0, np.int32))
    got = check([empty], [(HostColumn.from_strings([]), [Kind.MIN, Kind.ARGMAX])])
    assert got[1][0][0].size == 0 and TypeId(got[1][0][0].type_id) == TypeId.STRING


def test_row_index_accumulators_stay_inside_one_batch():
    """A row index means nothing in another batch or on another rank: states refuse them."""
    import cudf_b200 as cb
    from cudf_b200 import aggregation as agg
    from cudf_b200.groupby import GroupByState
    rng = np.random.default_rng(32)
    k = cb.Column.from_host(HostColumn.from_numpy(rng.integers(0, 10, 1000).astype(np.int32)))
    v = cb.Column.from_host(HostColumn.from_numpy(rng.integers(0, 100, 1000).astype(np.int32)))
    gb = cb.GroupBy(cb.Table([k]))
    st = GroupByState(gb, [cb.GroupByRequest(v, [agg.argmin()])])
    st.update()
    with pytest.raises(cb.UnsupportedError):
        st.update()
    with pytest.raises(cb.UnsupportedError):
        st.pack(2)
    keys, res = st.finalize()
    assert keys.num_rows() == 10
