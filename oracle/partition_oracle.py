"""CPU restatement of the row -> partition assignment of ``cudf::hash_partition``.

TEST INFRASTRUCTURE ONLY: imported by tests/ to check the CUDA path; nothing under cudf_b200/
imports it.

Rules restated (reference file:line):
  * partition = row hash % num_partitions (a bit mask when num_partitions is a power of two: the same
    value) — cpp/src/partitioning/partitioning.cu:54-92;
  * row hash = hash of the first hashed column, folded left to right with
    ``hash_combine(lhs, rhs) = lhs ^ (rhs + 0x9e3779b9 + (lhs << 6) + (lhs >> 2))`` —
    cpp/include/cudf/detail/row_operator/hashing.cuh:106-134, cpp/include/cudf/hashing/detail/hashing.hpp:83-86;
  * element hash (HASH_MURMUR3) = MurmurHash3_x86_32(bytes of the element, seed): fixed-width values by
    their storage bytes (BOOL8 as the byte 0/1, floats with -0 -> +0 and one NaN), strings by their UTF-8
    bytes — cpp/include/cudf/hashing/detail/murmurhash3_x86_32.cuh:22-76,
    cpp/include/cudf/hashing/detail/hash_functions.cuh:31-37; a null element hashes to UINT32_MAX —
    row_operator/hashing.cuh:52-75;
  * element hash (HASH_IDENTITY) = the numeric element cast to uint32 — partitioning.cu:856-874.

MurmurHash3_x86_32 itself lives in cuCollections (cuco::murmurhash3_32, un-vendored in the reference
tree, version pinned only by rapids-cmake); it is the published algorithm of Austin Appleby
(SMHasher, public domain), restated here and pinned by the published test vectors in
tests/test_partition_oracle.py.
"""
from __future__ import annotations

import numpy as np

from cudf_b200.types import HostColumn, STORAGE_DTYPE, TypeId

HASH_IDENTITY, HASH_MURMUR3 = 0, 1
M32 = 0xFFFFFFFF


def _rotl(x, r):
    return ((x << r) | (x >> (32 - r))) & M32


def murmur3_x86_32(data: bytes, seed: int = 0) -> int:
    """MurmurHash3_x86_32 of a byte string (scalar form, used for strings and for the test vectors)."""
    c1, c2 = 0xcc9e2d51, 0x1b873593
    h = seed & M32
    n = len(data)
    for i in range(0, n - n % 4, 4):
        k = int.from_bytes(data[i:i + 4], "little")
        k = (k * c1) & M32
        k = _rotl(k, 15)
        k = (k * c2) & M32
        h ^= k
        h = _rotl(h, 13)
        h = (h * 5 + 0xe6546b64) & M32
    tail = data[n - n % 4:]
    if tail:
        k = int.from_bytes(tail, "little")
        k = (k * c1) & M32
        k = _rotl(k, 15)
        k = (k * c2) & M32
        h ^= k
    h ^= n
    h ^= h >> 16
    h = (h * 0x85ebca6b) & M32
    h ^= h >> 13
    h = (h * 0xc2b2ae35) & M32
    h ^= h >> 16
    return h


def _murmur_fixed(values: np.ndarray, seed: int) -> np.ndarray:
    """Vectorised MurmurHash3_x86_32 over the storage bytes of fixed-width values (1, 2, 4 or 8 bytes)."""
    raw = np.ascontiguousarray(values)
    nbytes = raw.dtype.itemsize
    b = raw.view(np.uint8).reshape(-1, nbytes).astype(np.uint64)
    c1, c2 = np.uint64(0xcc9e2d51), np.uint64(0x1b873593)
    m = np.uint64(M32)

    def rotl(x, r):
        return ((x << np.uint64(r)) | (x >> np.uint64(32 - r))) & m
    h = np.full(b.shape[0], seed & M32, dtype=np.uint64)
    for blk in range(nbytes // 4):
        k = b[:, 4 * blk] | (b[:, 4 * blk + 1] << np.uint64(8)) | (b[:, 4 * blk + 2] << np.uint64(16)) | (b[:, 4 * blk + 3] << np.uint64(24))
        k = (k * c1) & m
        k = rotl(k, 15)
        k = (k * c2) & m
        h ^= k
        h = rotl(h, 13)
        h = (h * np.uint64(5) + np.uint64(0xe6546b64)) & m
    rem = nbytes % 4
    if rem:
        k = np.zeros(b.shape[0], dtype=np.uint64)
        for j in range(rem):
            k |= b[:, nbytes - rem + j] << np.uint64(8 * j)
        k = (k * c1) & m
        k = rotl(k, 15)
        k = (k * c2) & m
        h ^= k
    h ^= np.uint64(nbytes)
    h ^= h >> np.uint64(16)
    h = (h * np.uint64(0x85ebca6b)) & m
    h ^= h >> np.uint64(13)
    h = (h * np.uint64(0xc2b2ae35)) & m
    h ^= h >> np.uint64(16)
    return h.astype(np.uint32)


def element_hashes(col: HostColumn, hash_function: int = HASH_MURMUR3, seed: int = 0) -> np.ndarray:
    n = col.size
    valid = col.valid()
    if col.type_id == TypeId.STRING:
        if hash_function == HASH_IDENTITY:
            raise ValueError("IdentityHash does not support this data type")
        o = col.offsets[col.offset:col.offset + n + 1].astype(np.int64)
        raw = col.data.tobytes()
        out = np.array([murmur3_x86_32(raw[o[i]:o[i + 1]], seed) if valid[i] else M32 for i in range(n)], dtype=np.uint32)
        return out
    v = col.values().copy()
    if v.dtype.kind == "f":
        v = np.where(v == 0, v.dtype.type(0), v)                      # -0 -> +0
        v = np.where(np.isnan(v), np.array(np.nan, dtype=v.dtype), v)  # one NaN
    if col.type_id == TypeId.BOOL8:
        v = (v != 0).astype(np.uint8)
    if hash_function == HASH_IDENTITY:
        if v.dtype.kind == "f":
            with np.errstate(invalid="ignore"):
                h = np.where(np.isfinite(v) & (v > 0), np.minimum(v, 4294967295.0), 0).astype(np.uint64).astype(np.uint32)
        else:
            h = v.astype(np.int64).astype(np.uint64).astype(np.uint32) if v.dtype.kind != "u" else v.astype(np.uint64).astype(np.uint32)
    else:
        h = _murmur_fixed(v, seed)
    return np.where(valid, h, np.uint32(M32)).astype(np.uint32)


def row_hashes(columns, hash_function: int = HASH_MURMUR3, seed: int = 0) -> np.ndarray:
    h = element_hashes(columns[0], hash_function, seed).astype(np.uint64)
    m = np.uint64(M32)
    for c in columns[1:]:
        r = element_hashes(c, hash_function, seed).astype(np.uint64)
        h = (h ^ ((r + np.uint64(0x9e3779b9) + ((h << np.uint64(6)) & m) + (h >> np.uint64(2))) & m)) & m
    return h.astype(np.uint32)


def partition_of_rows(columns, num_partitions: int, hash_function: int = HASH_MURMUR3, seed: int = 0) -> np.ndarray:
    """Partition index of every row (the order of rows inside a partition is unspecified)."""
    return (row_hashes(columns, hash_function, seed).astype(np.uint64) % np.uint64(num_partitions)).astype(np.int64)
