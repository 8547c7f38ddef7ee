"""Seeded random schemas against the oracle: key and value columns of mixed types, null masks, slices, row filters,
null policies, aggregation lists valid for each value type, and the table paths."""
import numpy as np
import pytest

from cudf_b200.types import HostColumn, Kind, NullPolicy, STORAGE_DTYPE, TypeId, int128_array
from oracle import oracle
from tests import helpers as H

pytestmark = pytest.mark.gpu

INT_AGGS = [Kind.SUM, Kind.MIN, Kind.MAX, Kind.COUNT_VALID, Kind.COUNT_ALL, Kind.MEAN, Kind.SUM_OF_SQUARES, Kind.PRODUCT,
            Kind.VARIANCE, (Kind.STD, 0), Kind.M2, Kind.ARGMIN, Kind.ARGMAX]
FLOAT_AGGS = [Kind.SUM, Kind.MIN, Kind.MAX, Kind.COUNT_VALID, Kind.COUNT_ALL, Kind.MEAN, Kind.SUM_OF_SQUARES,
              Kind.VARIANCE, (Kind.STD, 2), Kind.M2, Kind.ARGMIN, Kind.ARGMAX]
DEC_AGGS = [Kind.SUM, Kind.SUM_OVERFLOW, Kind.MIN, Kind.MAX, Kind.COUNT_VALID, Kind.COUNT_ALL, Kind.ARGMIN, Kind.ARGMAX]
DEC128_AGGS = [Kind.SUM, Kind.SUM_OVERFLOW, Kind.COUNT_VALID, Kind.COUNT_ALL]
STR_AGGS = [Kind.MIN, Kind.MAX, Kind.ARGMIN, Kind.ARGMAX, Kind.COUNT_VALID]
KEY_TYPES = ["INT8", "INT16", "INT32", "INT64", "UINT32", "UINT64", "BOOL8", "FLOAT32", "FLOAT64", "DECIMAL64",
             "TIMESTAMP_DAYS", "DURATION_SECONDS", "STRING"]
VAL_TYPES = ["INT8", "INT16", "INT32", "INT64", "UINT8", "UINT32", "FLOAT32", "FLOAT64", "DECIMAL32", "DECIMAL64",
             "DECIMAL128", "STRING", "DICT_INT16", "DICT_FLOAT64"]


def _mask(rng, n, nullable):
    return (rng.random(n) > rng.choice([0.02, 0.3])) if nullable else None


def _key_column(rng, tname, n):
    card = int(rng.choice([2, 7, 40, 300]))
    offset = int(rng.choice([0, 0, 3, 32]))
    valid = _mask(rng, n, rng.random() < 0.5)
    if tname == "STRING":
        pool = ["", "a", "é", "日本"] + ["key%d" % i + "x" * (i % 40) for i in range(card)]
        words = [pool[i] for i in rng.integers(0, len(pool), n)]
        if valid is not None:
            words = [w if ok else None for w, ok in zip(words, valid.tolist())]
        return HostColumn.from_strings(words)
    t = TypeId[tname]
    if tname in ("FLOAT32", "FLOAT64"):
        pool = np.concatenate([rng.standard_normal(card), [0.0, -0.0, np.nan, np.inf]])
        vals = pool[rng.integers(0, pool.size, n)]
    elif tname == "BOOL8":
        vals = rng.integers(0, 2, n)
    else:
        lo = 0 if tname.startswith("UINT") else -(card // 2)
        vals = rng.integers(lo, lo + card, n)
        if tname in ("INT64", "UINT64", "DECIMAL64") and rng.random() < 0.5:
            vals = vals.astype(np.int64) * (2 ** 40 + 12345)        # spread over more than 32 bits
    return HostColumn.from_numpy(np.asarray(vals).astype(STORAGE_DTYPE[t]), valid=valid, type_id=t, offset=offset,
                                 scale=-2 if tname.startswith("DECIMAL") else 0)


def _value_column(rng, tname, n):
    """(column for the engine, plain column for the oracle, aggregations)"""
    offset = int(rng.choice([0, 0, 5]))
    valid = _mask(rng, n, rng.random() < 0.7)
    if tname == "STRING":
        pool = ["v%d" % i + "y" * (i % 37) for i in range(500)] + ["", "zz", "日本語"]
        words = [pool[i] for i in rng.integers(0, len(pool), n)]
        if valid is not None:
            words = [w if ok else None for w, ok in zip(words, valid.tolist())]
        c = HostColumn.from_strings(words)
        return c, c, STR_AGGS
    if tname.startswith("DICT_"):
        t = TypeId[tname[5:]]
        pool = rng.standard_normal(60) if tname.endswith("FLOAT64") else rng.integers(-300, 300, 60)
        vals = np.asarray(pool[rng.integers(0, 60, n)]).astype(STORAGE_DTYPE[t])
        plain = HostColumn.from_numpy(vals, valid=valid, type_id=t)
        d = HostColumn.from_dictionary(vals, valid=valid, index_type=rng.choice([TypeId.INT32, TypeId.UINT8]), offset=offset)
        return d, plain, (FLOAT_AGGS if tname.endswith("FLOAT64") else INT_AGGS)
    t = TypeId[tname]
    if tname == "DECIMAL128":
        ints = [int(a) * 2 ** 70 + int(b) for a, b in zip(rng.integers(-2 ** 40, 2 ** 40, n), rng.integers(0, 2 ** 62, n))]
        c = HostColumn.from_numpy(int128_array(ints), valid=valid, type_id=t, offset=offset, scale=3)
        return c, c, DEC128_AGGS
    if tname in ("FLOAT32", "FLOAT64"):
        vals = rng.standard_normal(n) * np.exp(rng.standard_normal(n))
        aggs = FLOAT_AGGS
    else:
        info = np.iinfo(np.dtype(STORAGE_DTYPE[t]))
        # (integers stay below 2^20 so that Σx² cannot wrap in its int64 cell: a wrapped Σx² makes M2 / VARIANCE / STD
        # garbage in the reference too, and which garbage depends on the arithmetic's last bit)
        span = min(int(info.max), 2 ** 40 if tname.startswith("DECIMAL") else 2 ** 20)
        vals = rng.integers(max(int(info.min), -span), span, n)
        aggs = DEC_AGGS if tname.startswith("DECIMAL") else INT_AGGS + ([Kind.SUM_OVERFLOW] if not tname.startswith("UINT") else [])
    c = HostColumn.from_numpy(np.asarray(vals).astype(STORAGE_DTYPE[t]), valid=valid, type_id=t, offset=offset,
                              scale=-1 if tname.startswith("DECIMAL") else 0)
    return c, c, aggs


@pytest.mark.parametrize("seed", range(48))
def test_random_schema_matches_oracle(seed):
    rng = np.random.default_rng(1000 + seed)
    n = int(rng.choice([1, 37, 1500, 6000, 40_000]))
    keys = [_key_column(rng, str(rng.choice(KEY_TYPES)), n) for _ in range(int(rng.integers(1, 4)))]
    reqs_gpu, reqs_cpu = [], []
    for _ in range(int(rng.integers(1, 4))):
        c, plain, aggs = _value_column(rng, str(rng.choice(VAL_TYPES)), n)
        pick = [aggs[i] for i in sorted(rng.choice(len(aggs), size=int(rng.integers(1, min(6, len(aggs)) + 1)), replace=False))]
        reqs_gpu.append((c, pick))
        reqs_cpu.append((plain, pick))
    policy = NullPolicy.INCLUDE if rng.random() < 0.5 else NullPolicy.EXCLUDE
    filters = []
    first = reqs_gpu[0][0]
    if rng.random() < 0.3 and first.mask is not None and first.type_id != TypeId.DICTIONARY32:
        filters = [first]
    opts = {"table_variant": int(rng.choice([0, 0, 1, 2, 3, 6]))}
    if rng.random() < 0.25:
        opts["shared_table_bytes"] = int(rng.choice([16384, 40000, 100000]))
    got = H.gpu_groupby(keys, reqs_gpu, policy, row_filters=filters, **opts)
    fm = [f.mask for f in filters]
    fo = [f.offset for f in filters]
    exp = oracle.groupby(keys, reqs_cpu, policy, row_filters=fm, row_filter_offsets=fo)
    H.assert_same_result(got, exp, reqs_cpu, scales=H.result_scales(keys, reqs_cpu, policy, fm, fo))
