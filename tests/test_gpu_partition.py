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
