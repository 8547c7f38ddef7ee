"""CPU checks of the oracle's exact sums (SUM_OVERFLOW, DECIMAL128) against Python integers, and of the host-side
helpers that build 16-byte and dictionary columns."""
import numpy as np
import pytest

from cudf_b200.types import HostColumn, Kind, NullPolicy, TypeId, int128_array, int128_list
from oracle import oracle
from tests import helpers as H


def test_int128_storage_round_trip():
    vals = [0, 1, -1, 2 ** 64, -(2 ** 64) - 5, 2 ** 127 - 1, -(2 ** 127), 123456789 * 10 ** 20]
    arr = int128_array(vals)
    assert arr.dtype.itemsize == 16 and int128_list(arr) == vals
    assert int128_list(int128_array([2 ** 127, 2 ** 128 + 3])) == [-(2 ** 127), 3]     # wraps modulo 2^128


def test_dictionary_column_decodes_to_its_values():
    rng = np.random.default_rng(3)
    x = rng.integers(-5, 5, 1000).astype(np.int16)
    valid = rng.random(1000) > 0.2
    d = HostColumn.from_dictionary(x, valid=valid, index_type=TypeId.UINT8, offset=5)
    idx, keys = d.children
    assert d.type_id == TypeId.DICTIONARY32 and d.offset == 5 and idx.size == 1005 and idx.offset == 0
    assert np.array_equal(np.sort(keys.values()), keys.values()) and len(set(keys.values().tolist())) == keys.size
    looked_up = keys.values()[idx.data[5:]]
    assert np.array_equal(looked_up[valid], x[valid]) and np.array_equal(d.valid(), valid)


@pytest.mark.parametrize("vtype,bits", [("INT8", 8), ("INT32", 32), ("INT64", 64), ("DECIMAL64", 64), ("DECIMAL128", 128)])
@pytest.mark.parametrize("threads", [1, 4])
def test_sum_overflow_is_the_exact_sum_leaving_the_range(vtype, bits, threads):
    """The flag of a group is "the exact sum of its valid values is not representable in the source type", its sum
    the exact sum wrapped to that type: what the reference's add-and-check gives in every arrival order when the
    values of a group share a sign (cpp/include/cudf/detail/aggregation/device_aggregators.cuh:136-160)."""
    rng = np.random.default_rng(bits + threads)
    n = 40_000
    kv = rng.integers(0, 300, n)
    top = 2 ** (bits - 1)
    # ~130 values per group of up to 1/40 of the type's range (every fourth group: a thousandth of that)
    mags = [int(h) * top // (2 ** 62 * 40) // (1000 if kk % 4 == 0 else 1)
            for h, kk in zip(rng.integers(0, 2 ** 62, n).tolist(), kv.tolist())]
    vals = [m if kk % 2 else -m for m, kk in zip(mags, kv.tolist())]
    valid = rng.random(n) > 0.1
    k = HostColumn.from_numpy(kv.astype(np.int32))
    v = H.make_column([x if ok else None for x, ok in zip(vals, valid.tolist())], vtype)
    okeys, ores = oracle.groupby([k], [(v, [Kind.SUM_OVERFLOW])], NullPolicy.EXCLUDE, threads=threads)
    st = ores[0][0]
    sums = int128_list(st.children[0].values()) if bits == 128 else st.children[0].values().tolist()
    flags = st.children[1].values().tolist()
    seen_true = seen_false = 0
    for g, key in enumerate(okeys[0].values().tolist()):
        exact = sum(x for x, kk, ok in zip(vals, kv.tolist(), valid.tolist()) if kk == key and ok)
        over = not (-top <= exact < top)
        assert bool(flags[g]) == over
        assert sums[g] == ((exact + top) % (2 * top)) - top
        seen_true += over
        seen_false += not over
    assert seen_false > 0 and seen_true > 0
