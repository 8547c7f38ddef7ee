// b2_device.cuh — device-side data model of the groupby engine: the plan a kernel receives,
// row loading, key packing / hashing / equality, and the accumulator-cell operations.
//
// Data layout in HBM
//   * inputs: Arrow-layout columns exactly as cudf::column_view describes them
//     (cpp/include/cudf/column/column_view.hpp:236-243): element i at data[offset+i], validity bit
//     offset+i of the uint32 mask words, LSB first (cpp/include/cudf/utilities/bit.hpp:47-104).
//   * hash table: an array of slots of `stride` 8-byte cells, AoS so that one probe touches one or
//     two 32-byte sectors:  cell 0 = key cell, cells 1.. = accumulators.
//       packed keys : key cell = all fixed-width key columns concatenated into <= 64 bits
//                     (+ one null bit per nullable column under null_policy::INCLUDE);
//       row keys    : key cell = (32-bit hash tag << 32) | representative row index, equality
//                     decided by comparing the rows' key columns (what the reference does for every
//                     key, cpp/src/groupby/hash/helpers.cuh:87-93,
//                     cpp/include/cudf/detail/row_operator/equality.cuh:59-89).
//     An unused slot has key cell == EMPTY; the one packed key whose bits equal EMPTY lives in an
//     extra slot at index `capacity`.  Behind it an optional dense region of `dense_slots` slots is
//     addressed directly by a key's position in the sampled key box (no probing): the CTAs merge
//     their dense shared-memory tables into it with coalesced atomics.
#pragma once
#include <cstddef>
#include <cstdint>
#include <cuda_runtime.h>

namespace b2 {

using u64 = unsigned long long;
using i64 = long long;
using u32 = unsigned int;

constexpr u64 EMPTY = 0xFFFFFFFFFFFFFFFFull;

constexpr int MAX_KEYS    = 16;
constexpr int MAX_VALS    = 16;
constexpr int MAX_CELLS   = 40;
constexpr int MAX_FILTERS = 8;

enum KeyMode : int { KM_PACKED = 0, KM_ROWS = 1 };

// type classes used on the device (host maps b2_type_id onto these)
enum ValClass : int {
  VC_I8 = 0, VC_I16, VC_I32, VC_I64, VC_U8, VC_U16, VC_U32, VC_U64, VC_F32, VC_F64, VC_BOOL,
  VC_STRING, VC_NONE /* only the validity mask is used (COUNT of a non-numeric column) */,
  // the two 64-bit words of a 16-byte element (DECIMAL128 values take two value slots: `data` points at the word)
  VC_U64X2 /* low word */, VC_I64X2 /* high word */
};

// accumulator cell operations; the decomposition of the requested aggregations into these follows
// cpp/src/groupby/hash/extract_single_pass_aggs.cpp:63-109
enum CellOp : int {
  OP_SUM_I = 0, OP_SUM_F, OP_SSQ_I, OP_SSQ_F, OP_MIN_I, OP_MIN_U, OP_MIN_F, OP_MAX_I, OP_MAX_U,
  OP_MAX_F, OP_CNT_V, OP_CNT_A, OP_PROD_I, OP_PROD_F,
  // the cell holds the ROW of the smallest / largest value seen so far (all-ones = none yet): ARGMIN /
  // ARGMAX themselves, and MIN / MAX of STRING values, which the reference computes as ARGMIN / ARGMAX
  // followed by a gather (cpp/src/groupby/hash/extract_single_pass_aggs.cpp:39-60)
  OP_ARGMIN, OP_ARGMAX,
  // SUM_OVERFLOW of a 64-bit source: Σ(v >> 32) and Σ(v & 0xFFFFFFFF), each exact in 64 bits for fewer than 2^31
  // rows, so that the finisher knows the exact sum and whether it fits the source type
  OP_SUM_HI, OP_SUM_LO,
  OP_SUM_HIU  // Σ(v >> 32) of an unsigned word (the low word of a DECIMAL128 value)
};
__host__ __device__ __forceinline__ bool is_arg_op(int op) { return op == OP_ARGMIN || op == OP_ARGMAX; }
constexpr unsigned long long ARG_NONE = 0xFFFFFFFFFFFFFFFFull;

struct DKeyCol {
  const unsigned char* data;
  const u32* mask;      // nullptr = no nulls
  const void* offsets;  // strings
  i64 offset;           // element offset of the view
  int vclass;           // ValClass
  int width;            // bytes (fixed width)
  int shift;            // packed mode: bit position of the value
  int nullbit;          // packed mode + INCLUDE + nullable: bit position of the null flag, else -1
  int offs64;           // strings: 1 = INT64 offsets
  int is_signed;        // fixed width: values order as signed integers
};

struct DValCol {
  const unsigned char* data;
  const u32* mask;
  const void* offsets;  // STRING values (MIN / MAX / ARGMIN / ARGMAX of strings): the offsets child
  i64 offset;
  int vclass;
  int offs64;           // ... typed INT64
};

struct DCell {
  unsigned char op;   // CellOp
  unsigned char col;  // value column index
};

struct DPlan {
  i64 nrows;
  int nkeys, nvals, ncells, key_mode;
  int include_nulls;  // null_policy::INCLUDE
  int nfilters;
  int stride;         // cells per slot = 1 + ncells
  int flags;          // PF_* below
  DKeyCol keys[MAX_KEYS];
  DValCol vals[MAX_VALS];
  DCell cells[MAX_CELLS];
  const u32* filters[MAX_FILTERS];
  i64 filter_offsets[MAX_FILTERS];
};

enum PlanFlags : int {
  PF_VEC_KEYS = 1,  // every key column may be read 4 rows at a time with one 16-byte load
  PF_VEC_VAL0 = 2,  // value column 0 likewise (the compact "Σ and n of one float column" layouts)
  PF_FAST     = 4,  // every key column is 4 or 8 bytes wide and every mask / filter offset is a
                    // multiple of 4, so the validity bits of 4 consecutive rows never straddle a mask word
  PF_BULK     = 8,  // value column 0's validity can be tiled with 16-byte-aligned bulk copies: mask
                    // pointer 16-byte aligned and offset a multiple of 128 bits (or no mask at all)
  PF_F64MEAN  = 16  // the cells are Σ and n of one FLOAT64 column: the key-box sampler also records the
                    // largest exponent among the sampled values (the window of the fixed-point limbs)
};

// Dense key mapping of one aggregate pass, derived on the device by sample_dense_box: when the keys
// seen in a sample span a small box [min_k, min_k + range_k) per key column, a key's shared-memory
// slot is its position in that box — no probing and no key storage.  Keys outside the box (the
// sample missed them) take the global-table path, so the result stays exact.
struct DDense {
  int enabled;
  u32 total;               // slots of one copy = product of ranges
  u32 copies;              // replicas of the table in shared memory (warp w uses copy w % copies):
                           // few groups mean many rows per slot, and same-address atomics serialise
  u32 vexp;                // PF_F64MEAN: 1 + the largest biased exponent among the sampled values, 0 = none seen
  i64 min[MAX_KEYS];
  u64 range[MAX_KEYS];     // includes one extra value for "null" on nullable INCLUDE columns
  u32 mult[MAX_KEYS];
};

// control block shared by the kernels of one table
struct DCtrl {
  u32 overflow;      // set when the table ran out of room or a probe sequence hit its limit
  u32 special_used;  // the slot of the key whose bits equal EMPTY is in use
  u64 nclaimed;      // slots claimed in [0, capacity)
  u64 claim_limit;   // nclaimed above this sets overflow
  u64 out_cursor;    // finalize: next dense output index
  u64 stat_smem_rows;
  u64 stat_gmem_rows;
  u64 done_ctas;     // CTAs of the lean fused kernel that finished their merge (the last one counts the groups)
  u64 chunk_overflow;  // a sender of merged chunks had more records than a chunk holds
  u64 dense_slots;     // slots after the special slot that are addressed directly by dense-box position
  u32 error;           // a bounded wait inside a kernel ran out (1: staged-tile ring of the lean kernel)
  u32 pad0;
  u64 t_phase[5];      // CTA 0 of the fused kernel: %globaltimer at start, after sampling, after the
                       // shared-table init, after the row loop, after the merge (diagnostics)
  DDense dense;
  u32 null_counts[80];  // finalize: nulls per result column [0, 64) and per key column [64, 80)
};

// ---------------------------------------------------------------------------------- table addressing
// Slots 0..cap (hashed region + the special slot at `cap`) are array-of-structures: {key, cells...},
// `stride` words each, so that one probe touches one or two sectors.  The `dense` slots behind them
// (addressed by key-box position, never probed) are structure-of-arrays: all keys, then all cells 0,
// all cells 1, ... so that consecutive threads merging consecutive box positions update consecutive
// words (4 updates per 32-byte sector instead of one request per slot).
struct SlotRef {
  u64* key;    // the key cell
  u64* cells;  // cell c is cells[c * step]
  i64 step;
};
__device__ __forceinline__ SlotRef slot_ref(u64* tbl, i64 cap, int stride, i64 dense, i64 s)
{
  if (s <= cap) {
    u64* p = tbl + s * stride;
    return SlotRef{p, p + 1, 1};
  }
  u64* p = tbl + (cap + 1) * stride + (s - cap - 1);
  return SlotRef{p, p + dense, dense};
}

// ---------------------------------------------------------------------------------- hashing
__host__ __device__ __forceinline__ u64 mix64(u64 x)
{
  x ^= x >> 33; x *= 0xff51afd7ed558ccdull;
  x ^= x >> 33; x *= 0xc4ceb9fe1a85ec53ull;
  x ^= x >> 33;
  return x;
}
// second, independent hash: decides the owner partition/rank of a key so that the keys one rank
// receives still spread over its whole table
__host__ __device__ __forceinline__ u64 owner_hash(u64 h) { return mix64(h * 0x9E3779B97F4A7C15ull + 0x7F4A7C15ull); }
__host__ __device__ __forceinline__ u32 owner_of(u64 h, u32 nparts)
{
  return (u32)(((owner_hash(h) >> 32) * (u64)nparts) >> 32);
}
__device__ __forceinline__ u32 reduce32(u32 h, u32 n) { return __umulhi(h, n); }
__device__ __forceinline__ u64 reduce64(u64 h, u64 n) { return __umul64hi(h, n); }

// ---------------------------------------------------------------------------------- bit tests
__device__ __forceinline__ bool bit_valid(const u32* mask, i64 i)
{
  return (__ldg(mask + (i >> 5)) >> (i & 31)) & 1u;
}

// validity bits of 4 consecutive elements starting at bit `pos` (`nvalid` of them exist)
__device__ __forceinline__ u32 valid_nibble(const u32* mask, i64 pos, int nvalid)
{
  const u32 sh  = (u32)pos & 31u;
  const u32* w  = mask + (pos >> 5);
  u32 bits      = __ldg(w) >> sh;
  if (sh + (u32)nvalid > 32u) bits |= __ldg(w + 1) << (32u - sh);
  return bits & 0xFu;
}

// a row takes part unless a row filter (fused drop_nulls) or, under EXCLUDE, a null key says no
// (cpp/src/groupby/common/utils.cpp:14-32)
__device__ __forceinline__ bool row_active(const DPlan& P, i64 row)
{
  bool ok = true;
  for (int f = 0; f < P.nfilters; ++f) ok = ok && bit_valid(P.filters[f], P.filter_offsets[f] + row);
  if (!P.include_nulls) {
    for (int k = 0; k < P.nkeys; ++k)
      if (P.keys[k].mask) ok = ok && bit_valid(P.keys[k].mask, P.keys[k].offset + row);
  }
  return ok;
}

// ---------------------------------------------------------------------------------- packed keys
__device__ __forceinline__ u64 load_fixed_bits(const unsigned char* data, i64 idx, int width)
{
  switch (width) {
    case 1: return (u64) * (data + idx);
    case 2: return (u64)__ldg((const unsigned short*)data + idx);
    case 4: return (u64)__ldg((const u32*)data + idx);
    default: return (u64)__ldg((const u64*)data + idx);
  }
}

__device__ __forceinline__ u64 pack_key(const DPlan& P, i64 row)
{
  u64 key = 0;
  for (int k = 0; k < P.nkeys; ++k) {
    const DKeyCol& c = P.keys[k];
    const i64 idx    = c.offset + row;
    if (c.nullbit >= 0 && !bit_valid(c.mask, idx)) {
      key |= 1ull << c.nullbit;  // null == null whatever the payload
    } else {
      key |= load_fixed_bits(c.data, idx, c.width) << c.shift;
    }
  }
  return key;
}

// ---------------------------------------------------------------------------------- row keys
__device__ __forceinline__ i64 str_offset(const DKeyCol& c, i64 idx)
{
  return c.offs64 ? (i64)__ldg((const i64*)c.offsets + idx) : (i64)__ldg((const int*)c.offsets + idx);
}

// canonical bits of a fixed-width key element: -0 -> +0 and one NaN, so that hashing agrees with
// equality (cpp/include/cudf/hashing/detail/hash_functions.cuh:31-37)
__device__ __forceinline__ u64 canonical_bits(const DKeyCol& c, i64 idx)
{
  u64 b = load_fixed_bits(c.data, idx, c.width);
  if (c.vclass == VC_F32) {
    float f = __uint_as_float((u32)b);
    if (f == 0.0f) b = 0;
    if (f != f) b = 0x7fc00000u;
  } else if (c.vclass == VC_F64) {
    double d = __longlong_as_double((i64)b);
    if (d == 0.0) b = 0;
    if (d != d) b = 0x7ff8000000000000ull;
  }
  return b;
}

// up to 8 bytes starting at an arbitrarily aligned address, as a little-endian word; bytes beyond
// `nbytes` are zero.  Reads whole aligned 8-byte words (one or two), never a word without a wanted byte.
__device__ __forceinline__ u64 load_bytes8(const unsigned char* p, int nbytes)
{
  const unsigned long long a = (unsigned long long)p;
  const u64* w  = (const u64*)(a & ~7ull);
  const int sh  = (int)(a & 7ull) * 8;
  u64 v = __ldg(w) >> sh;
  if (sh != 0 && (sh >> 3) + nbytes > 8) v |= __ldg(w + 1) << (64 - sh);
  return nbytes >= 8 ? v : (v & ((1ull << (8 * nbytes)) - 1ull));
}

__device__ inline u64 hash_bytes(const unsigned char* p, i64 len, u64 h)
{
  // 8 bytes per step; the tail is zero padded and the length mixed in, so "ab" != "ab\0"
  for (i64 i = 0; i < len; i += 8) {
    const int nb = (int)(len - i < 8 ? len - i : 8);
    h = mix64(h ^ load_bytes8(p + i, nb)) + 0x9E3779B97F4A7C15ull;
  }
  return mix64(h ^ ((u64)len << 56));
}

__device__ inline bool bytes_equal(const unsigned char* a, const unsigned char* b, i64 len)
{
  for (i64 i = 0; i < len; i += 8) {
    const int nb = (int)(len - i < 8 ? len - i : 8);
    if (load_bytes8(a + i, nb) != load_bytes8(b + i, nb)) return false;
  }
  return true;
}

__device__ inline u64 hash_row(const DPlan& P, i64 row)
{
  u64 h = 0x243F6A8885A308D3ull;
  for (int k = 0; k < P.nkeys; ++k) {
    const DKeyCol& c = P.keys[k];
    const i64 idx    = c.offset + row;
    if (c.mask && !bit_valid(c.mask, idx)) {
      h = mix64(h ^ 0xA5A5A5A5DEADBEEFull) + k;  // null element
    } else if (c.vclass == VC_STRING) {
      const i64 b = str_offset(c, idx), e = str_offset(c, idx + 1);
      h = hash_bytes(c.data + b, e - b, h);
    } else {
      h = mix64(h ^ canonical_bits(c, idx)) + 0x9E3779B97F4A7C15ull;
    }
  }
  return mix64(h);
}

// row i == row j over the key columns; null == null (nulls only reach here under INCLUDE),
// NaN == NaN, +0 == -0, strings byte-wise with equal length
// (cpp/include/cudf/detail/row_operator/equality.cuh:59-89,243-261, string_view.cuh:306-326)
__device__ inline bool rows_equal(const DPlan& P, i64 a, i64 b)
{
  if (a == b) return true;
  for (int k = 0; k < P.nkeys; ++k) {
    const DKeyCol& c = P.keys[k];
    const i64 ia = c.offset + a, ib = c.offset + b;
    if (c.mask) {
      const bool va = bit_valid(c.mask, ia), vb = bit_valid(c.mask, ib);
      if (va != vb) return false;
      if (!va) continue;
    }
    if (c.vclass == VC_STRING) {
      const i64 ba = str_offset(c, ia), ea = str_offset(c, ia + 1);
      const i64 bb = str_offset(c, ib), eb = str_offset(c, ib + 1);
      if (ea - ba != eb - bb) return false;
      if (!bytes_equal(c.data + ba, c.data + bb, ea - ba)) return false;
    } else {
      if (canonical_bits(c, ia) != canonical_bits(c, ib)) return false;
    }
  }
  return true;
}

// ---------------------------------------------------------------------------------- the reference's row hash
// cudf::hash_partition assigns row -> hash(row) % partitions with MurmurHash3_x86_32 per element
// (cpp/include/cudf/hashing/detail/murmurhash3_x86_32.cuh:22-76: the published algorithm of Austin
// Appleby over the element's bytes, seeded), a null element hashing to UINT32_MAX
// (cpp/include/cudf/detail/row_operator/hashing.cuh:52-75), the first column's hash folded with the
// others by boost's hash_combine (cpp/include/cudf/hashing/detail/hashing.hpp:83-86); floats hash
// with -0 -> +0 and one NaN, BOOL8 as the byte 0 / 1.  HASH_IDENTITY casts the numeric element to
// uint32 instead (cpp/src/partitioning/partitioning.cu:856-874).
__host__ __device__ __forceinline__ u32 rotl32(u32 x, int r) { return (x << r) | (x >> (32 - r)); }

__host__ __device__ inline u32 murmur3_x86_32(const unsigned char* data, i64 len, u32 seed)
{
  const u32 c1 = 0xcc9e2d51u, c2 = 0x1b873593u;
  u32 h = seed;
  const i64 nblocks = len / 4;
  for (i64 i = 0; i < nblocks; ++i) {
    u32 k = (u32)data[4 * i] | ((u32)data[4 * i + 1] << 8) | ((u32)data[4 * i + 2] << 16) | ((u32)data[4 * i + 3] << 24);
    k *= c1; k = rotl32(k, 15); k *= c2;
    h ^= k; h = rotl32(h, 13); h = h * 5u + 0xe6546b64u;
  }
  const unsigned char* tail = data + 4 * nblocks;
  u32 k = 0;
  switch (len & 3) {
    case 3: k ^= (u32)tail[2] << 16;
    case 2: k ^= (u32)tail[1] << 8;
    case 1: k ^= (u32)tail[0];
            k *= c1; k = rotl32(k, 15); k *= c2; h ^= k;
  }
  h ^= (u32)len;
  h ^= h >> 16; h *= 0x85ebca6bu; h ^= h >> 13; h *= 0xc2b2ae35u; h ^= h >> 16;
  return h;
}
// the same over a value held in a register (little endian, `nbytes` = 1, 2, 4 or 8): whole 4-byte blocks go
// through the block round directly, 1 or 2 bytes are the tail
__host__ __device__ __forceinline__ u32 murmur3_x86_32_value(u64 v, int nbytes, u32 seed)
{
  const u32 c1 = 0xcc9e2d51u, c2 = 0x1b873593u;
  u32 h = seed;
  auto block = [&](u32 k) {
    k *= c1; k = rotl32(k, 15); k *= c2;
    h ^= k; h = rotl32(h, 13); h = h * 5u + 0xe6546b64u;
  };
  if (nbytes >= 4) block((u32)v);
  if (nbytes == 8) block((u32)(v >> 32));
  if (nbytes < 4) {
    u32 k = (u32)v & (nbytes == 1 ? 0xFFu : 0xFFFFu);
    k *= c1; k = rotl32(k, 15); k *= c2;
    h ^= k;
  }
  h ^= (u32)nbytes;
  h ^= h >> 16; h *= 0x85ebca6bu; h ^= h >> 13; h *= 0xc2b2ae35u; h ^= h >> 16;
  return h;
}
__host__ __device__ __forceinline__ u32 hash_combine32(u32 lhs, u32 rhs)
{
  return lhs ^ (rhs + 0x9e3779b9u + (lhs << 6) + (lhs >> 2));
}

enum RefHash : int { RH_IDENTITY = 0, RH_MURMUR3 = 1, RH_ENGINE = 2 /* this engine's own 64-bit mix */ };

__device__ inline u32 ref_element_hash(const DKeyCol& c, i64 row, int kind, u32 seed)
{
  const i64 idx = c.offset + row;
  if (c.mask && !bit_valid(c.mask, idx)) return 0xFFFFFFFFu;
  if (c.vclass == VC_STRING) {
    const i64 b = str_offset(c, idx), e = str_offset(c, idx + 1);
    return murmur3_x86_32(c.data + b, e - b, seed);
  }
  u64 bits = canonical_bits(c, idx);  // -0 -> +0, one NaN
  if (c.vclass == VC_BOOL) bits = bits != 0;
  if (kind == RH_IDENTITY) {
    switch (c.vclass) {
      case VC_F32: return (u32)__uint_as_float((u32)bits);
      case VC_F64: return (u32)__longlong_as_double((i64)bits);
      default: return (u32)bits;  // integers: the low 32 bits, as static_cast<uint32_t> gives
    }
  }
  return murmur3_x86_32_value(bits, c.width, seed);
}

__device__ inline u32 ref_row_hash(const DPlan& P, i64 row, int kind, u32 seed)
{
  u32 h = ref_element_hash(P.keys[0], row, kind, seed);
  for (int k = 1; k < P.nkeys; ++k) h = hash_combine32(h, ref_element_hash(P.keys[k], row, kind, seed));
  return h;
}

// ---------------------------------------------------------------------------------- values
// A value is carried as 64 bits: integers sign/zero-extended to int64, floats widened to double.
__device__ __forceinline__ u64 load_value(const DValCol& c, i64 row)
{
  const i64 idx = c.offset + row;
  switch (c.vclass) {
    case VC_I8: return (u64)(i64) * ((const signed char*)c.data + idx);
    case VC_I16: return (u64)(i64)__ldg((const short*)c.data + idx);
    case VC_I32: return (u64)(i64)__ldg((const int*)c.data + idx);
    case VC_I64: case VC_U64: return __ldg((const u64*)c.data + idx);
    case VC_U8: return (u64) * (c.data + idx);
    case VC_BOOL: return (u64)(*(c.data + idx) != 0);
    case VC_U16: return (u64)__ldg((const unsigned short*)c.data + idx);
    case VC_U32: return (u64)__ldg((const u32*)c.data + idx);
    case VC_F32: return (u64)__double_as_longlong((double)__ldg((const float*)c.data + idx));
    case VC_F64: return __ldg((const u64*)c.data + idx);
    case VC_U64X2: case VC_I64X2: return __ldg((const u64*)c.data + 2 * idx);
    default: return 0;
  }
}
__device__ __forceinline__ bool value_valid(const DValCol& c, i64 row)
{
  return c.mask == nullptr || bit_valid(c.mask, c.offset + row);
}

// order-preserving map double -> u64 (so float min/max are single integer atomics instead of the
// reference's compare-and-swap loop, cpp/include/cudf/detail/utilities/device_atomics.cuh:226-337;
// a NaN can never make the loop spin: cpp/tests/groupby/min_tests.cpp:518-541)
__host__ __device__ __forceinline__ u64 f64_ordered(u64 bits)
{
  return (bits >> 63) ? ~bits : (bits | 0x8000000000000000ull);
}
__host__ __device__ __forceinline__ u64 f64_unordered(u64 enc)
{
  return (enc >> 63) ? (enc & 0x7FFFFFFFFFFFFFFFull) : ~enc;
}

// identity of a cell (cpp/include/cudf/detail/aggregation/aggregation.cuh:121-174,
// cpp/include/cudf/detail/utilities/device_operators.cuh:51-83,114-139,172-197)
__host__ __device__ __forceinline__ u64 cell_identity(int op)
{
  switch (op) {
    case OP_MIN_I: return 0x7FFFFFFFFFFFFFFFull;
    case OP_MIN_U: case OP_MIN_F: return 0xFFFFFFFFFFFFFFFFull;
    case OP_MAX_I: return 0x8000000000000000ull;
    case OP_PROD_I: return 1ull;
    case OP_PROD_F: return 0x3FF0000000000000ull;  // 1.0
    case OP_ARGMIN: case OP_ARGMAX: return ARG_NONE;
    default: return 0ull;                          // sums, counts, MAX_U, MAX_F
  }
}

// fold one input value into a cell (cpp/include/cudf/detail/aggregation/device_aggregators.cuh:
// 99-112 SUM/MIN/MAX, :309-361 SUM_OF_SQUARES/COUNT)
__device__ __forceinline__ void cell_update(u64* cell, int op, u64 v)
{
  switch (op) {
    case OP_SUM_I: atomicAdd(cell, v); break;
    case OP_SUM_HI: atomicAdd(cell, (u64)((i64)v >> 32)); break;
    case OP_SUM_LO: atomicAdd(cell, v & 0xFFFFFFFFull); break;
    case OP_SUM_HIU: atomicAdd(cell, v >> 32); break;
    case OP_SUM_F: atomicAdd((double*)cell, __longlong_as_double((i64)v)); break;
    case OP_SSQ_I: atomicAdd(cell, v * v); break;
    case OP_SSQ_F: { const double d = __longlong_as_double((i64)v); atomicAdd((double*)cell, d * d); break; }
    case OP_MIN_I: atomicMin((i64*)cell, (i64)v); break;
    case OP_MIN_U: atomicMin(cell, v); break;
    case OP_MIN_F: atomicMin(cell, f64_ordered(v)); break;
    case OP_MAX_I: atomicMax((i64*)cell, (i64)v); break;
    case OP_MAX_U: atomicMax(cell, v); break;
    case OP_MAX_F: atomicMax(cell, f64_ordered(v)); break;
    case OP_CNT_V: case OP_CNT_A: atomicAdd(cell, 1ull); break;
    case OP_PROD_I: {
      u64 old = *cell, assumed;
      do { assumed = old; old = atomicCAS(cell, assumed, assumed * v); } while (old != assumed);
      break;
    }
    case OP_PROD_F: {
      u64 old = *cell, assumed;
      do {
        assumed = old;
        const double r = __longlong_as_double((i64)assumed) * __longlong_as_double((i64)v);
        old = atomicCAS(cell, assumed, (u64)__double_as_longlong(r));
      } while (old != assumed);
      break;
    }
    default: break;
  }
}

// ---- ARGMIN / ARGMAX cells: row of the extreme value -------------------------------------------------
// value at row a <, ==, > value at row b of one value column: -1, 0, +1; 2 when a NaN makes them
// unordered.  Strings compare byte-wise, the shorter one first when one is a prefix of the other
// (cpp/include/cudf/strings/string_view.cuh:306-321: UTF-8 byte order is code point order).
__device__ inline int value_compare(const DValCol& c, i64 a, i64 b)
{
  const i64 ia = c.offset + a, ib = c.offset + b;
  if (c.vclass == VC_STRING) {
    const i64 ba = c.offs64 ? __ldg((const i64*)c.offsets + ia) : (i64)__ldg((const int*)c.offsets + ia);
    const i64 ea = c.offs64 ? __ldg((const i64*)c.offsets + ia + 1) : (i64)__ldg((const int*)c.offsets + ia + 1);
    const i64 bb = c.offs64 ? __ldg((const i64*)c.offsets + ib) : (i64)__ldg((const int*)c.offsets + ib);
    const i64 eb = c.offs64 ? __ldg((const i64*)c.offsets + ib + 1) : (i64)__ldg((const int*)c.offsets + ib + 1);
    const i64 la = ea - ba, lb = eb - bb, n = la < lb ? la : lb;
    for (i64 i = 0; i < n; ++i) {
      const unsigned char x = c.data[ba + i], y = c.data[bb + i];
      if (x != y) return x < y ? -1 : 1;
    }
    return la < lb ? -1 : (la > lb ? 1 : 0);
  }
  const u64 x = load_value(c, a), y = load_value(c, b);
  if (c.vclass == VC_F32 || c.vclass == VC_F64) {
    const double dx = __longlong_as_double((i64)x), dy = __longlong_as_double((i64)y);
    if (dx != dx || dy != dy) return 2;
    return dx < dy ? -1 : (dx > dy ? 1 : 0);
  }
  if (c.vclass == VC_U64) return x < y ? -1 : (x > y ? 1 : 0);
  return (i64)x < (i64)y ? -1 : ((i64)x > (i64)y ? 1 : 0);
}

// Folds row `row` into an ARGMIN / ARGMAX cell: the row replaces the cell's row when its value is
// strictly better, or equal with a smaller row index — so the result is the FIRST row holding the
// extreme value whatever the order of arrival (the reference keeps whichever equal value arrived first,
// cpp/include/cudf/detail/aggregation/device_aggregators.cuh:222-263; its tests use distinct values).
// A NaN never replaces anything and is never replaced by a smaller / larger number that arrives later
// only if it arrived first — the comparisons with NaN are false, as in the reference.
__device__ inline void arg_update(u64* cell, int op, const DValCol& c, i64 row)
{
  u64 old = *(volatile u64*)cell;
  for (;;) {
    if (old != ARG_NONE) {
      const int cmp = value_compare(c, row, (i64)old);
      const bool better = op == OP_ARGMIN ? cmp == -1 : cmp == 1;
      if (!(better || (cmp == 0 && (u64)row < old))) return;
    }
    const u64 prev = atomicCAS(cell, old, (u64)row);
    if (prev == old) return;
    old = prev;
  }
}

// partial (+) partial in registers: the operator cell_merge applies atomically
__device__ __forceinline__ u64 cell_combine(int op, u64 a, u64 b)
{
  switch (op) {
    case OP_SUM_I: case OP_SSQ_I: case OP_CNT_V: case OP_CNT_A: case OP_SUM_HI: case OP_SUM_LO: case OP_SUM_HIU: return a + b;
    case OP_SUM_F: case OP_SSQ_F:
      return (u64)__double_as_longlong(__longlong_as_double((i64)a) + __longlong_as_double((i64)b));
    case OP_MIN_I: return (i64)a < (i64)b ? a : b;
    case OP_MIN_U: case OP_MIN_F: return a < b ? a : b;
    case OP_MAX_I: return (i64)a > (i64)b ? a : b;
    case OP_MAX_U: case OP_MAX_F: return a > b ? a : b;
    case OP_PROD_I: return a * b;
    case OP_PROD_F:
      return (u64)__double_as_longlong(__longlong_as_double((i64)a) * __longlong_as_double((i64)b));
    default: return a;
  }
}

// fold a partial cell (same representation as the table's) into a cell: the merge of partial
// aggregates (cpp/src/groupby/streaming_groupby/merge.cu:30-61)
__device__ __forceinline__ void cell_merge(u64* cell, int op, u64 part)
{
  switch (op) {
    case OP_SUM_I: case OP_SSQ_I: case OP_CNT_V: case OP_CNT_A: case OP_SUM_HI: case OP_SUM_LO: case OP_SUM_HIU: atomicAdd(cell, part); break;
    case OP_SUM_F: case OP_SSQ_F: atomicAdd((double*)cell, __longlong_as_double((i64)part)); break;
    case OP_MIN_I: atomicMin((i64*)cell, (i64)part); break;
    case OP_MIN_U: case OP_MIN_F: atomicMin(cell, part); break;
    case OP_MAX_I: atomicMax((i64*)cell, (i64)part); break;
    case OP_MAX_U: case OP_MAX_F: atomicMax(cell, part); break;
    case OP_PROD_I: cell_update(cell, OP_PROD_I, part); break;
    case OP_PROD_F: cell_update(cell, OP_PROD_F, part); break;
    default: break;
  }
}

}  // namespace b2
