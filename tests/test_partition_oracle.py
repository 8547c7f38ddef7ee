"""The CPU restatement of cudf::hash_partition's row -> partition rule, pinned: MurmurHash3_x86_32 against
the published test vectors of the algorithm (SMHasher's verification strings and the values quoted in its
public descriptions), the vectorised fixed-width form against the scalar form, and the combination rules
(null = UINT32_MAX, hash_combine order, float normalisation, BOOL8 as 0/1) the reference states."""
import numpy as np

from cudf_b200.types import HostColumn, TypeId
from oracle import partition_oracle as PO

PUBLISHED = [  # (bytes, seed, MurmurHash3_x86_32)
    (b"", 0, 0x00000000), (b"", 1, 0x514E28B7), (b"", 0xFFFFFFFF, 0x81F16F39),
    (b"\xff\xff\xff\xff", 0, 0x76293B50), (b"\x21\x43\x65\x87", 0, 0xF55B516B), (b"\x21\x43\x65\x87", 0x5082EDEE, 0x2362F9DE),
    (b"\x21\x43\x65", 0, 0x7E4A8634), (b"\x21\x43", 0, 0xA0F7B07A), (b"\x21", 0, 0x72661CF4),
    (b"\x00\x00\x00\x00", 0, 0x2362F9DE), (b"\x00\x00\x00", 0, 0x85F0B427), (b"\x00\x00", 0, 0x30F4C306), (b"\x00", 0, 0x514E28B7),
    (b"a", 0x9747b28c, 0x7FA09EA6), (b"aa", 0x9747b28c, 0x5D211726), (b"aaa", 0x9747b28c, 0x283E0130), (b"aaaa", 0x9747b28c, 0x5A97808A),
    (b"abc", 0, 0xB3DD93FA), (b"abc", 0x9747b28c, 0xC84A62DD), (b"hello", 0, 0x248BFA47),
    (b"Hello, world!", 0x9747b28c, 0x24884CBA), (b"The quick brown fox jumps over the lazy dog", 0x9747b28c, 0x2FA826CD),
    (b"The quick brown fox jumps over the lazy dog", 0, 0x2E4FF723),
]


def test_murmur3_x86_32_published_vectors():
    for data, seed, expect in PUBLISHED:
        assert PO.murmur3_x86_32(data, seed) == expect, (data, seed)


def test_vectorised_fixed_width_form_equals_the_scalar_form():
    rng = np.random.default_rng(3)
    for dt in (np.int8, np.uint8, np.int16, np.uint16, np.int32, np.uint32, np.int64, np.uint64, np.float32, np.float64):
        v = (rng.standard_normal(200) * 1000).astype(dt) if np.dtype(dt).kind == "f" else \
            rng.integers(np.iinfo(dt).min, np.iinfo(dt).max, 200, dtype=dt, endpoint=True)
        for seed in (0, 42, 0xFFFFFFFF):
            got = PO._murmur_fixed(v, seed)
            exp = np.array([PO.murmur3_x86_32(x.tobytes(), seed) for x in v], dtype=np.uint32)
            assert np.array_equal(got, exp), dt


def test_null_bool_float_and_combine_rules():
    # nulls hash to UINT32_MAX whatever lies under them (murmurhash3_x86_32_test.cpp:53-109)
    a = HostColumn.from_numpy(np.array([0, 100, -100], np.int32), valid=np.array([True, False, True]))
    b = HostColumn.from_numpy(np.array([0, -200, -100], np.int32), valid=np.array([True, False, True]))
    assert np.array_equal(PO.element_hashes(a), PO.element_hashes(b))
    assert PO.element_hashes(a)[1] == 0xFFFFFFFF
    # BOOL8: any non-zero byte is true (murmurhash3_x86_32_test.cpp:32-50)
    t1 = HostColumn.from_numpy(np.array([0, 1, 1, 1, 0], np.uint8), type_id=TypeId.BOOL8)
    t2 = HostColumn.from_numpy(np.array([0, 1, 2, 255, 0], np.uint8), type_id=TypeId.BOOL8)
    assert np.array_equal(PO.element_hashes(t1), PO.element_hashes(t2))
    # floats: -0 == +0, every NaN alike (hash_functions.cuh:31-37)
    f = HostColumn.from_numpy(np.array([0.0, -0.0, np.nan, -np.nan], np.float64))
    h = PO.element_hashes(f)
    assert h[0] == h[1] and h[2] == h[3]
    # hash_combine folds left to right starting from the first column's hash (row_operator/hashing.cuh:120-133)
    x = HostColumn.from_numpy(np.array([7], np.int32))
    y = HostColumn.from_strings(["ab"])
    hx, hy = int(PO.element_hashes(x)[0]), int(PO.element_hashes(y)[0])
    expect = (hx ^ ((hy + 0x9e3779b9 + ((hx << 6) & 0xFFFFFFFF) + (hx >> 2)) & 0xFFFFFFFF)) & 0xFFFFFFFF
    assert int(PO.row_hashes([x, y])[0]) == expect
    # identity hash: the value itself (partitioning.cu:856-874)
    ids = HostColumn.from_numpy(np.array([0, 5, 12, -1], np.int64))
    assert PO.partition_of_rows([ids], 5, PO.HASH_IDENTITY).tolist() == [0, 0, 2, 0xFFFFFFFF % 5]
