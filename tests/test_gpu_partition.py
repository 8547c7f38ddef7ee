"""``hash_partition`` against the properties the reference's own tests check
(cpp/tests/partitioning/hash_partition_test.cpp): empty results for zero partitions / rows / hashed
columns, partition counts beyond shared memory, output = permutation of the input with validity
preserved, and a partition assignment that depends on the hashed columns only."""
import numpy as np
import pytest

from cudf_b200.types import HostColumn, TypeId

pytestmark = pytest.mark.gpu


def _table(cols):
    import cudf_b200 as cb
    return cb.Table([cb.Column.from_host(c) for c in cols])


def _three_columns():
    return [HostColumn.from_numpy(np.arange(1, 9, dtype=np.float32)),
            HostColumn.from_numpy(np.arange(1, 9, dtype=np.int16)),
            HostColumn.from_strings(["a", "bb", "ccc", "d", "ee", "fff", "gg", "h"])]


def _assert_empty_like(out, cols, offsets, nparts):
    assert out.num_columns() == len(cols)
    assert all(c.size == 0 for c in out.columns())
    assert [c.type_id for c in out.columns()] == [c.type_id for c in cols]
    assert offsets == [0] * (nparts + 1)


def test_zero_partitions_gives_an_empty_table():  # hash_partition_test.cpp:72-88
    from cudf_b200.partition import hash_partition
    cols = _three_columns()
    out, offsets = hash_partition(_table(cols), [2], 0)
    _assert_empty_like(out, cols, offsets, 0)


def test_zero_rows():  # hash_partition_test.cpp:90-106
    from cudf_b200.partition import hash_partition
    cols = [HostColumn.from_numpy(np.zeros(0, np.float32)), HostColumn.from_numpy(np.zeros(0, np.int16)),
            HostColumn.from_strings([])]
    out, offsets = hash_partition(_table(cols), [2], 3)
    _assert_empty_like(out, cols, offsets, 3)


def test_zero_columns_and_nothing_to_hash():  # hash_partition_test.cpp:108-142
    import cudf_b200 as cb
    from cudf_b200.partition import hash_partition
    out, offsets = hash_partition(cb.Table([]), [], 3)
    assert out.num_columns() == 0 and offsets == [0, 0, 0, 0]
    cols = _three_columns()
    out, offsets = hash_partition(_table(cols), [], 3)
    _assert_empty_like(out, cols, offsets, 3)


def _partitions_exceeding_shared_memory():
    import torch
    return torch.cuda.get_device_properties(0).shared_memory_per_block_optin // 4 + 10


def test_more_partitions_than_shared_memory():  # hash_partition_test.cpp:172-187
    from cudf_b200.partition import hash_partition
    n, nparts = 48 * 1024, _partitions_exceeding_shared_memory()
    bools = HostColumn.from_numpy(np.ones(n, dtype=np.uint8), type_id=TypeId.BOOL8)
    out, offsets = hash_partition(_table([bools]), [0], nparts)
    assert out.num_columns() == 1 and out.columns()[0].size == n
    assert len(offsets) == nparts + 1 and offsets[0] == 0 and offsets[-1] == n
    # one distinct key: all rows in one partition
    assert sorted(np.diff(offsets).tolist())[-1] == n


def test_large_partition_count_is_a_permutation():  # hash_partition_test.cpp:189-209
    from cudf_b200.partition import hash_partition
    n, nparts = 1000, _partitions_exceeding_shared_memory()
    col = HostColumn.from_numpy(np.arange(n, dtype=np.int32))
    out, offsets = hash_partition(_table([col]), [0], nparts)
    assert offsets == sorted(offsets) and offsets[0] == 0 and offsets[-1] == n and len(offsets) == nparts + 1
    assert sorted(out.columns()[0].to_host().values().tolist()) == list(range(n))


def test_large_partition_count_mixed_types_and_nulls():  # hash_partition_test.cpp:211-260
    from cudf_b200.partition import hash_partition
    n, nparts = 200, _partitions_exceeding_shared_memory()
    valid = np.arange(n) % 4 != 0
    ints = HostColumn.from_numpy(np.arange(n, dtype=np.int32), valid=valid)
    floats = HostColumn.from_numpy(np.arange(n, dtype=np.float32))
    strings = HostColumn.from_strings([str(i) if valid[i] else None for i in range(n)])
    out, offsets = hash_partition(_table([ints, floats, strings]), [0, 1], nparts)
    cols = [c.to_host() for c in out.columns()]
    assert [c.size for c in cols] == [n, n, n]
    assert offsets == sorted(offsets) and offsets[0] == 0 and offsets[-1] == n and len(offsets) == nparts + 1
    assert cols[0].null_count == n // 4 and cols[2].null_count == n // 4
    # rows stay together: the float column still identifies the row
    f = cols[1].values().astype(np.int64)
    assert sorted(f.tolist()) == list(range(n))
    iv, sv = cols[0].to_pylist(), cols[2].to_pylist()
    for j, r in enumerate(f.tolist()):
        assert iv[j] == (r if valid[r] else None)
        assert sv[j] == (str(r).encode() if valid[r] else None)


def test_nullable_strings_without_nulls():  # hash_partition_test.cpp:286-298
    from cudf_b200.partition import hash_partition
    s = HostColumn.from_strings(["a", "bb", "ccc", "d"])
    s.mask = np.full(16, 0xFFFFFFFF, dtype=np.uint32)  # a mask with every bit set
    out, offsets = hash_partition(_table([s]), [0], 3)
    col = out.columns()[0]
    assert col.null_count == 0 and sorted(col.to_host().to_pylist()) == [b"a", b"bb", b"ccc", b"d"]


def test_only_the_hashed_columns_decide():  # hash_partition_test.cpp:300-324
    from cudf_b200.partition import hash_partition
    rng = np.random.default_rng(5)
    n = 10_000
    to_hash = HostColumn.from_numpy(rng.integers(0, 500, n).astype(np.int32))
    first = HostColumn.from_numpy(rng.standard_normal(n))
    second = HostColumn.from_numpy(rng.integers(0, 9, n).astype(np.int64))
    out1, off1 = hash_partition(_table([to_hash, first]), [0], 3)
    out2, off2 = hash_partition(_table([second, to_hash]), [1], 3)   # hashed column in another position
    assert off1 == off2
    a, b = out1.columns()[0].to_host().values(), out2.columns()[1].to_host().values()
    for p in range(3):  # same keys in every partition (the order inside a partition is unspecified)
        assert sorted(a[off1[p]:off1[p + 1]].tolist()) == sorted(b[off2[p]:off2[p + 1]].tolist())


# ------------------------------------------------------------------------------------ against the oracle
def _comparable(x):
    """NaN compares unequal to itself: rows are compared through a stand-in."""
    return "nan" if isinstance(x, float) and x != x else x


def _rows_of(cols, lo, hi):
    """The rows [lo, hi) of host columns as a sorted list of tuples (None = null)."""
    lists = [[_comparable(x) for x in c.to_pylist()[lo:hi]] for c in cols]
    return sorted(zip(*lists), key=repr)


def _check_against_oracle(cols, hashed, nparts, **kw):
    """Every partition holds exactly the rows the reference's rule assigns to it (as a multiset: the order
    inside a partition is unspecified), validity and null counts included."""
    from cudf_b200.partition import hash_partition
    from oracle import partition_oracle as PO
    out, offsets = hash_partition(_table(cols), hashed, nparts, **kw)
    got = [c.to_host() for c in out.columns()]
    n = cols[0].size
    assert len(offsets) == nparts + 1 and offsets[0] == 0 and offsets[-1] == n and offsets == sorted(offsets)
    part = PO.partition_of_rows([cols[i] for i in hashed], nparts, kw.get("hash_function", PO.HASH_MURMUR3), kw.get("seed", 0))
    assert np.array_equal(np.diff(offsets), np.bincount(part, minlength=nparts))
    src = [[_comparable(x) for x in c.to_pylist()] for c in cols]
    for p in range(nparts):
        rows = np.flatnonzero(part == p)
        exp = sorted(zip(*[[l[i] for i in rows] for l in src]), key=repr)
        assert _rows_of(got, offsets[p], offsets[p + 1]) == exp, f"partition {p}"
    for g, c in zip(got, cols):
        assert g.null_count == c.null_count and TypeId(g.type_id) == TypeId(c.type_id)
    return offsets


def _mixed_table(seed, n):
    rng = np.random.default_rng(seed)
    words = ["", "a", "año", "日本語", "z" * 37, "ab", "abc", "abcd", "abcde"]
    return [HostColumn.from_numpy(rng.integers(-500, 500, n).astype(np.int32), valid=rng.random(n) > 0.1),
            HostColumn.from_strings([None if rng.random() < 0.07 else words[i] + str(i) for i in rng.integers(0, len(words), n)]),
            HostColumn.from_numpy(rng.choice([0.0, -0.0, np.nan, 1.5, -2.25, np.inf], n)),
            HostColumn.from_strings([words[i] for i in rng.integers(0, len(words), n)]),
            HostColumn.from_numpy(rng.integers(0, 3, n).astype(np.uint8), type_id=TypeId.BOOL8),
            HostColumn.from_numpy(rng.integers(-2**60, 2**60, n).astype(np.int64)),
            HostColumn.from_numpy(rng.integers(0, 2**16, n).astype(np.uint16)),
            HostColumn.from_numpy(rng.standard_normal(n).astype(np.float32), valid=rng.random(n) > 0.5)]


@pytest.mark.parametrize("nparts", [1, 2, 3, 8, 13, 1000])
def test_partition_assignment_is_the_references_murmur3(nparts):
    cols = _mixed_table(1, 3000)
    _check_against_oracle(cols, [0], nparts)
    _check_against_oracle(cols, [1, 2], nparts)                       # a nullable STRING and a float column
    _check_against_oracle(cols, [3, 1, 4, 5, 6, 7, 0, 2], nparts)     # two STRING columns among eight


def test_custom_seed_changes_the_assignment_deterministically():  # hash_partition_test.cpp:341-364
    cols = _mixed_table(2, 2000)
    a = _check_against_oracle(cols, [2, 3], 7, seed=12345)
    b = _check_against_oracle(cols, [2, 3], 7, seed=12345)
    c = _check_against_oracle(cols, [2, 3], 7, seed=0)
    assert a == b and a != c


def test_identity_hash():  # cpp/src/partitioning/partitioning.cu:856-874, hash_partition_test.cpp:326-339
    import cudf_b200 as cb
    from cudf_b200.partition import HASH_IDENTITY, hash_partition
    rng = np.random.default_rng(3)
    n = 5000
    cols = [HostColumn.from_numpy(rng.integers(0, 10_000, n).astype(np.int32)),
            HostColumn.from_numpy(rng.integers(-5, 5, n).astype(np.int64), valid=rng.random(n) > 0.2),
            HostColumn.from_strings([str(i) for i in range(n)])]
    off = _check_against_oracle(cols, [0], 10, hash_function=HASH_IDENTITY)
    out, _ = hash_partition(_table(cols), [0], 10, hash_function=HASH_IDENTITY)
    v = out.columns()[0].to_host().values()
    for p in range(10):   # identity: the key itself decides, value % partitions
        assert (v[off[p]:off[p + 1]] % 10 == p).all()
    _check_against_oracle(cols, [0, 1], 6, hash_function=HASH_IDENTITY)
    with pytest.raises(cb.LogicError, match="IdentityHash does not support this data type"):
        hash_partition(_table(cols), [2], 3, hash_function=HASH_IDENTITY)
    with pytest.raises(cb.LogicError, match="Unsupported hash function"):
        hash_partition(_table(cols), [0], 3, hash_function=9)


def test_argument_errors():  # hash_partition_test.cpp:48-70
    import cudf_b200 as cb
    from cudf_b200.partition import hash_partition
    cols = _three_columns()
    with pytest.raises(IndexError):                    # std::out_of_range in the reference
        hash_partition(_table(cols), [-1], 3)
    with pytest.raises(IndexError):
        hash_partition(_table(cols), [3], 3)
    short = HostColumn.from_numpy(np.arange(1, 10, dtype=np.int16))
    with pytest.raises(ValueError, match="same number of rows"):   # std::invalid_argument in the reference
        hash_partition(cb.Table([cb.Column.from_host(cols[0]), cb.Column.from_host(short)]), [1], 3)


def test_partition_of_many_rows_matches_the_oracle_counts():
    """2M rows, 8 destinations (the shape of a row exchange between 8 ranks): counts per partition are the oracle's."""
    from cudf_b200.partition import hash_partition
    from oracle import partition_oracle as PO
    rng = np.random.default_rng(4)
    n = 2_000_000
    k = HostColumn.from_numpy(rng.integers(0, 10**12, n).astype(np.int64))
    v = HostColumn.from_numpy(rng.standard_normal(n), valid=rng.random(n) > 0.01)
    out, offsets = hash_partition(_table([k, v]), [0], 8)
    part = PO.partition_of_rows([k], 8)
    assert np.array_equal(np.diff(offsets), np.bincount(part, minlength=8))
    got_k = out.columns()[0].to_host().values()
    for p in range(8):
        assert np.array_equal(np.sort(got_k[offsets[p]:offsets[p + 1]]), np.sort(k.values()[part == p]))
