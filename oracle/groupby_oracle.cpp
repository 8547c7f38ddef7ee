// groupby_oracle.cpp — CPU restatement of the reference's hash groupby-aggregate semantics.
//
// TEST INFRASTRUCTURE ONLY.  This file is the checker the parity tests, the smoke test and the
// benchmark's CPU-baseline leg compare the CUDA engine against.  Nothing in the shipped library
// links, imports or calls it.
//
// Parity pin: checked against the known-answer vectors of the reference's own groupby unit tests
// (tests/golden/reference_known_answers.json, transcribed case by case with file:line) by
// tests/test_oracle_golden.py.
//
// What is restated, with the reference location each rule follows (paths inside NVIDIA/cudf):
//  * which rows take part: null_policy EXCLUDE drops a row with a null in any key column
//    (cpp/src/groupby/common/utils.cpp:14-32, cpp/src/groupby/hash/groupby.cu:43); INCLUDE keeps
//    them and null == null (cpp/src/groupby/hash/groupby.cu:41).
//  * key equality: integers ==; floats == plus NaN == NaN, so +0 and -0 are one group
//    (cpp/include/cudf/detail/row_operator/equality.cuh:59-89,243-261,
//    cpp/include/cudf/hashing/detail/hash_functions.cuh:31-37); strings byte-wise
//    (cpp/include/cudf/strings/string_view.cuh:306-326).  The output key of a group is the key of
//    one of its rows (cpp/src/groupby/hash/compute_groupby.cu:104-111); here: the first.
//  * decomposition MEAN -> SUM + COUNT_VALID; M2/VAR/STD -> SUM_OF_SQUARES + SUM + COUNT_VALID
//    (cpp/src/groupby/hash/extract_single_pass_aggs.cpp:63-109).
//  * per-element update: null values skipped, COUNT_ALL counts rows
//    (cpp/include/cudf/detail/aggregation/device_aggregators.cuh:99-112,309-361,428-446).
//  * result types (cpp/include/cudf/detail/aggregation/aggregation.hpp:884-1013): SUM /
//    SUM_OF_SQUARES / PRODUCT of integers -> INT64 (wrapping), of floats -> same type; MIN/MAX ->
//    source type; COUNT -> INT32; MEAN/M2/VARIANCE/STD -> FLOAT64.
//  * MEAN = double(sum)/double(count), null iff count == 0
//    (cpp/src/groupby/hash/hash_compound_agg_finalizer.cu:93-133).
//  * M2 = Σx² − (Σx)²/n, 0 (valid) when n == 0; VAR = M2/(n−ddof), STD = sqrt(VAR), null iff
//    n == 0 or n−ddof <= 0 (cpp/src/groupby/common/m2_var_std.cu:49-59,160-187).
//  * result validity: a SUM/MIN/MAX/PRODUCT/SUM_OF_SQUARES result column carries a mask only when
//    its source has nulls; a group with no valid value is null
//    (cpp/src/groupby/hash/output_utils.cu:61-68, device_aggregators.cuh:440-442).
//
// Floating-point sums are accumulated in long double so that the oracle is more accurate than
// either GPU implementation (the reference's own summation order is unspecified: atomics).
//
// Build: see oracle/Makefile.  C interface at the bottom, used through ctypes by oracle/oracle.py.

#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstring>
#include <limits>
#include <memory>
#include <string>
#include <thread>
#include <unordered_map>
#include <vector>

namespace {

enum TypeId : int32_t {
  T_EMPTY = 0, T_INT8, T_INT16, T_INT32, T_INT64, T_UINT8, T_UINT16, T_UINT32, T_UINT64,
  T_FLOAT32, T_FLOAT64, T_BOOL8, T_TS_DAYS, T_TS_S, T_TS_MS, T_TS_US, T_TS_NS,
  T_DUR_DAYS, T_DUR_S, T_DUR_MS, T_DUR_US, T_DUR_NS, T_DICT32, T_STRING, T_LIST,
  T_DEC32, T_DEC64,  // fixed point: the integer representation; the scale is metadata the caller keeps
  T_DEC128, T_STRUCT // (DECIMAL128 is not served; STRUCT is the result type of SUM_OVERFLOW)
};
enum Kind : int32_t {
  K_SUM = 0, K_PRODUCT = 2, K_MIN = 3, K_MAX = 4, K_COUNT_VALID = 5, K_COUNT_ALL = 6,
  K_SUMSQ = 9, K_MEAN = 10, K_M2 = 11, K_VAR = 12, K_STD = 13, K_ARGMAX = 16, K_ARGMIN = 17,
  K_SUM_OVERFLOW = 1
};

struct Col {  // host-memory mirror of a column_view
  int32_t type_id;
  int32_t size;
  const void* data;
  const uint32_t* mask;
  int32_t offset;
  const void* offsets;    // STRING only
  int32_t offsets_type;   // T_INT32 or T_INT64
};
struct Agg { int32_t kind; int32_t ddof; };
struct Req { Col values; int32_t naggs; const Agg* aggs; };

inline bool bit(const uint32_t* m, int64_t i) { return !m || ((m[i >> 5] >> (i & 31)) & 1u); }

int width_of(int32_t t)
{
  switch (t) {
    case T_INT8: case T_UINT8: case T_BOOL8: return 1;
    case T_INT16: case T_UINT16: return 2;
    case T_INT32: case T_UINT32: case T_FLOAT32: case T_TS_DAYS: case T_DUR_DAYS: case T_DEC32: return 4;
    case T_INT64: case T_UINT64: case T_FLOAT64: case T_TS_S: case T_TS_MS: case T_TS_US:
    case T_TS_NS: case T_DUR_S: case T_DUR_MS: case T_DUR_US: case T_DUR_NS: case T_DEC64: return 8;
    case T_DEC128: return 16;
    default: return 0;
  }
}
bool is_float(int32_t t) { return t == T_FLOAT32 || t == T_FLOAT64; }
bool is_duration(int32_t t) { return t >= T_DUR_DAYS && t <= T_DUR_NS; }
bool is_timestamp(int32_t t) { return t >= T_TS_DAYS && t <= T_TS_NS; }
bool is_decimal(int32_t t) { return t == T_DEC32 || t == T_DEC64; }

// value of element i as (int64 bit pattern | double)
struct Val { int64_t i; double f; unsigned __int128 w; };  // w: a DECIMAL128 element (two's complement)
inline Val load(const Col& c, int64_t r)
{
  const int64_t k = (int64_t)c.offset + r;
  Val v{0, 0.0, 0};
  switch (c.type_id) {
    case T_INT8: v.i = ((const int8_t*)c.data)[k]; break;
    case T_INT16: v.i = ((const int16_t*)c.data)[k]; break;
    case T_INT32: case T_TS_DAYS: case T_DUR_DAYS: case T_DEC32: v.i = ((const int32_t*)c.data)[k]; break;
    case T_INT64: case T_TS_S: case T_TS_MS: case T_TS_US: case T_TS_NS: case T_DUR_S:
    case T_DUR_MS: case T_DUR_US: case T_DUR_NS: case T_DEC64: v.i = ((const int64_t*)c.data)[k]; break;
    case T_UINT8: v.i = ((const uint8_t*)c.data)[k]; break;
    case T_BOOL8: v.i = ((const uint8_t*)c.data)[k] != 0; break;
    case T_UINT16: v.i = ((const uint16_t*)c.data)[k]; break;
    case T_UINT32: v.i = ((const uint32_t*)c.data)[k]; break;
    case T_UINT64: v.i = (int64_t)((const uint64_t*)c.data)[k]; break;
    case T_FLOAT32: v.f = ((const float*)c.data)[k]; break;
    case T_FLOAT64: v.f = ((const double*)c.data)[k]; break;
    case T_DEC128: std::memcpy(&v.w, (const char*)c.data + k * 16, 16); break;
    default: break;
  }
  return v;
}

// canonical key bytes of one key element: equal keys <=> equal bytes
inline void append_key(std::string& out, const Col& c, int64_t r, bool include_nulls)
{
  const int64_t k = (int64_t)c.offset + r;
  const bool valid = bit(c.mask, k);
  if (include_nulls) out.push_back(valid ? 1 : 0);
  if (!valid) return;  // null == null whatever the payload
  if (c.type_id == T_STRING) {
    int64_t b, e;
    if (c.offsets_type == T_INT64) { b = ((const int64_t*)c.offsets)[k]; e = ((const int64_t*)c.offsets)[k + 1]; }
    else { b = ((const int32_t*)c.offsets)[k]; e = ((const int32_t*)c.offsets)[k + 1]; }
    const uint32_t len = (uint32_t)(e - b);
    out.append((const char*)&len, 4);
    out.append((const char*)c.data + b, (size_t)len);
  } else if (c.type_id == T_FLOAT32) {
    float f = ((const float*)c.data)[k];
    if (f == 0.0f) f = 0.0f;                                   // -0 -> +0
    if (f != f) f = std::numeric_limits<float>::quiet_NaN();   // one NaN
    out.append((const char*)&f, 4);
  } else if (c.type_id == T_FLOAT64) {
    double f = ((const double*)c.data)[k];
    if (f == 0.0) f = 0.0;
    if (f != f) f = std::numeric_limits<double>::quiet_NaN();
    out.append((const char*)&f, 8);
  } else if (c.type_id == T_BOOL8) {
    out.push_back(((const uint8_t*)c.data)[k] != 0);
  } else {
    const int w = width_of(c.type_id);
    out.append((const char*)c.data + k * w, (size_t)w);
  }
}

struct Acc {  // per (group, request): every simple accumulator the supported kinds decompose into
  int64_t count = 0;     // COUNT_VALID
  int64_t isum = 0;      // SUM of integral sources, wraps like int64
  int64_t isumsq = 0;    // Σ (int64)x*(int64)x, wraps
  int64_t iprod = 1;
  long double fsum = 0;  // float sources
  long double fsumsq = 0;
  long double fprod = 1;
  int64_t imin = 0, imax = 0;  // signed or unsigned compare depending on the source type
  double fmin = 0, fmax = 0;
  // ARGMIN / ARGMAX (and MIN / MAX of strings, which the reference computes as ARGMIN / ARGMAX + gather,
  // cpp/src/groupby/hash/extract_single_pass_aggs.cpp:39-60): row of the extreme valid value, the first
  // such row on ties; -1 = no valid value (ARGMIN_SENTINEL, cpp/include/cudf/detail/aggregation/aggregation.hpp)
  int64_t argmin = -1, argmax = -1;
  // SUM_OVERFLOW: the exact sum.  The reference adds in the source type and raises the flag when an add wraps
  // (cpp/include/cudf/detail/aggregation/device_aggregators.cuh:136-160); which adds wrap depends on the order
  // the rows arrive in.  "The exact sum does not fit the source type" is the flag every arrival order gives when
  // the values of a group share a sign (the reference's tests, cpp/tests/groupby/sum_overflow_tests.cpp:260-378),
  // and the flag of the order that alternates signs otherwise; the sum of a flagged group is not specified there.
  __int128 xsum = 0;
  // DECIMAL128: Σ of the low words and Σ of the (signed) high words, each exact; the sum is their combination
  // modulo 2^128 like the reference's __int128 adds, and it left the range iff hi128 + (lo128 >> 64) is no int64
  unsigned __int128 lo128 = 0;
  __int128 hi128 = 0;
};

struct Group {
  int64_t first_row;
  int64_t rows = 0;  // COUNT_ALL
};

struct OutCol {
  int32_t type_id = 0;
  int64_t size = 0;
  std::vector<uint8_t> data;
  std::vector<uint32_t> mask;  // empty => not nullable
  int64_t null_count = 0;
  std::vector<int64_t> offsets;  // STRING keys (always int64 here)
  // STRUCT results (SUM_OVERFLOW): `data` is child 0 (the sum, typed child_type), `data2` child 1 (BOOL8)
  int32_t child_type = 0;
  std::vector<uint8_t> data2;
};

struct Result {
  int64_t ngroups = 0;
  std::vector<OutCol> keys;
  std::vector<std::vector<OutCol>> results;
  std::string error;
};

template <typename T>
void put(OutCol& c, int64_t g, T v) { std::memcpy(c.data.data() + g * sizeof(T), &v, sizeof(T)); }
void set_null(OutCol& c, int64_t g)
{
  c.mask[g >> 5] &= ~(1u << (g & 31));
  c.null_count++;
}
void alloc(OutCol& c, int32_t type, int64_t n, int w, bool nullable)
{
  c.type_id = type; c.size = n; c.data.assign((size_t)(n * w), 0);
  if (nullable) c.mask.assign((size_t)((n + 31) / 32), 0xFFFFFFFFu);
}

int32_t result_type(int32_t src, int32_t kind)
{
  switch (kind) {
    case K_COUNT_VALID: case K_COUNT_ALL: case K_ARGMAX: case K_ARGMIN: return T_INT32;
    case K_MIN: case K_MAX: return src;
    case K_SUM:
      // fixed point sums keep their type (aggregation.hpp:956-963): a DECIMAL32 sum wraps at 32 bits
      if (is_float(src) || is_duration(src) || is_decimal(src) || src == T_DEC128) return src;
      return T_INT64;
    case K_SUMSQ: case K_PRODUCT: return is_float(src) ? src : T_INT64;
    case K_MEAN: return is_duration(src) ? src : T_FLOAT64;
    case K_SUM_OVERFLOW: return T_STRUCT;  // {sum: src, overflow: BOOL8} (aggregation.hpp:990-995)
    default: return T_FLOAT64;  // M2, VAR, STD
  }
}

// 0 ok, 1 invalid type/agg combination (cpp/src/groupby/groupby.cu:188-201)
int check_combo(int32_t src, int32_t kind)
{
  const bool numeric = (src >= T_INT8 && src <= T_BOOL8);
  switch (kind) {
    case K_COUNT_VALID: case K_COUNT_ALL: return 0;
    case K_MIN: case K_MAX: case K_ARGMIN: case K_ARGMAX:
      return (numeric || is_timestamp(src) || is_duration(src) || is_decimal(src) || src == T_STRING) ? 0 : 1;
    // PRODUCT of decimals throws (sum_tests.cpp:245-246); DECIMAL128 sums run on the hash path
    // (cpp/src/groupby/hash/groupby.cu:82-85), its other aggregations on the sort path (not restated here)
    case K_SUM: return (numeric || is_duration(src) || is_decimal(src) || src == T_DEC128) ? 0 : 1;
    case K_MEAN: return (numeric || is_duration(src)) ? 0 : 1;
    case K_SUM_OVERFLOW:  // signed integers and decimals (aggregation.hpp:980-988)
      return (src == T_INT8 || src == T_INT16 || src == T_INT32 || src == T_INT64 || is_decimal(src) || src == T_DEC128) ? 0 : 1;
    case K_SUMSQ: case K_PRODUCT: case K_M2: case K_VAR: case K_STD: return numeric ? 0 : 1;
    default: return 1;
  }
}

// value at row a vs value at row b of one column: -1, 0, +1, or 2 when a NaN makes them unordered
// (strings: byte-wise, cpp/include/cudf/strings/string_view.cuh:306-321)
int compare_rows(const Col& c, int64_t a, int64_t b)
{
  if (c.type_id == T_STRING) {
    auto off = [&](int64_t i) {
      return c.offsets_type == T_INT64 ? ((const int64_t*)c.offsets)[c.offset + i] : (int64_t)((const int32_t*)c.offsets)[c.offset + i];
    };
    const int64_t ba = off(a), la = off(a + 1) - ba, bb = off(b), lb = off(b + 1) - bb;
    const int r = std::memcmp((const char*)c.data + ba, (const char*)c.data + bb, (size_t)std::min(la, lb));
    if (r != 0) return r < 0 ? -1 : 1;
    return la < lb ? -1 : (la > lb ? 1 : 0);
  }
  const Val x = load(c, a), y = load(c, b);
  if (is_float(c.type_id)) {
    if (x.f != x.f || y.f != y.f) return 2;
    return x.f < y.f ? -1 : (x.f > y.f ? 1 : 0);
  }
  if (c.type_id == T_UINT64) return (uint64_t)x.i < (uint64_t)y.i ? -1 : ((uint64_t)x.i > (uint64_t)y.i ? 1 : 0);
  return x.i < y.i ? -1 : (x.i > y.i ? 1 : 0);
}

struct Partial {  // one thread's table over a contiguous row range
  std::unordered_map<std::string, int64_t> index;
  std::vector<Group> groups;
  std::vector<Acc> accs;  // groups x nreqs
};

void aggregate_range(Partial& P, int64_t lo, int64_t hi, const Col* keys, int nkeys, bool include,
                     const Req* reqs, int nreqs, const uint32_t* const* filters,
                     const int32_t* filter_offsets, int nfilters)
{
  std::string kb;
  for (int64_t r = lo; r < hi; ++r) {
    bool take = true;
    for (int f = 0; f < nfilters && take; ++f)
      take = bit(filters[f], (int64_t)(filter_offsets ? filter_offsets[f] : 0) + r);
    if (!take) continue;
    if (!include)
      for (int k = 0; k < nkeys && take; ++k) take = bit(keys[k].mask, (int64_t)keys[k].offset + r);
    if (!take) continue;
    kb.clear();
    for (int k = 0; k < nkeys; ++k) append_key(kb, keys[k], r, include);
    auto it = P.index.find(kb);
    int64_t g;
    if (it == P.index.end()) {
      g = (int64_t)P.groups.size();
      P.index.emplace(kb, g);
      P.groups.push_back(Group{r, 0});
      P.accs.resize(P.accs.size() + (size_t)nreqs);
    } else {
      g = it->second;
    }
    P.groups[(size_t)g].rows++;
    for (int q = 0; q < nreqs; ++q) {
      const Col& vc = reqs[q].values;
      if (!bit(vc.mask, (int64_t)vc.offset + r)) continue;  // null value: skipped
      Acc& a = P.accs[(size_t)(g * nreqs + q)];
      // rows arrive in ascending order: a strict comparison keeps the first row of equal values
      if (a.argmin < 0 || compare_rows(vc, r, a.argmin) == -1) a.argmin = r;
      if (a.argmax < 0 || compare_rows(vc, r, a.argmax) == 1) a.argmax = r;
      if (vc.type_id == T_STRING) { a.count++; continue; }
      const Val v = load(vc, r);
      const bool first = a.count == 0;
      a.count++;
      if (vc.type_id == T_DEC128) {
        a.lo128 += (unsigned __int128)(uint64_t)v.w;
        a.hi128 += (__int128)(int64_t)(uint64_t)(v.w >> 64);
      } else if (is_float(vc.type_id)) {
        a.fsum += v.f;
        a.fsumsq += (long double)v.f * (long double)v.f;
        a.fprod *= v.f;
        // DeviceMin/DeviceMax: min(a,b) = a < b ? a : b, applied in row order
        if (first) { a.fmin = v.f; a.fmax = v.f; }
        else { a.fmin = (v.f < a.fmin) ? v.f : a.fmin; a.fmax = (v.f > a.fmax) ? v.f : a.fmax; }
      } else {
        a.isum = (int64_t)((uint64_t)a.isum + (uint64_t)v.i);
        a.xsum += (__int128)v.i;
        a.isumsq = (int64_t)((uint64_t)a.isumsq + (uint64_t)v.i * (uint64_t)v.i);
        a.iprod = (int64_t)((uint64_t)a.iprod * (uint64_t)v.i);
        if (first) { a.imin = v.i; a.imax = v.i; }
        else if (vc.type_id == T_UINT64) {
          if ((uint64_t)v.i < (uint64_t)a.imin) a.imin = v.i;
          if ((uint64_t)v.i > (uint64_t)a.imax) a.imax = v.i;
        } else {
          if (v.i < a.imin) a.imin = v.i;
          if (v.i > a.imax) a.imax = v.i;
        }
      }
    }
  }
}

void merge_acc(Acc& d, const Acc& s, const Col& vc)
{
  const int32_t vtype = vc.type_id;
  if (s.count == 0) return;
  // `s` covers later rows than `d`: strict comparisons keep the first row of equal values
  if (s.argmin >= 0 && (d.argmin < 0 || compare_rows(vc, s.argmin, d.argmin) == -1)) d.argmin = s.argmin;
  if (s.argmax >= 0 && (d.argmax < 0 || compare_rows(vc, s.argmax, d.argmax) == 1)) d.argmax = s.argmax;
  const bool first = d.count == 0;
  d.count += s.count;
  d.isum = (int64_t)((uint64_t)d.isum + (uint64_t)s.isum);
  d.xsum += s.xsum;
  d.lo128 += s.lo128;
  d.hi128 += s.hi128;
  d.isumsq = (int64_t)((uint64_t)d.isumsq + (uint64_t)s.isumsq);
  d.iprod = (int64_t)((uint64_t)d.iprod * (uint64_t)s.iprod);
  d.fsum += s.fsum; d.fsumsq += s.fsumsq; d.fprod *= s.fprod;
  if (first) { d.imin = s.imin; d.imax = s.imax; d.fmin = s.fmin; d.fmax = s.fmax; return; }
  if (vtype == T_UINT64) {
    if ((uint64_t)s.imin < (uint64_t)d.imin) d.imin = s.imin;
    if ((uint64_t)s.imax > (uint64_t)d.imax) d.imax = s.imax;
  } else {
    if (s.imin < d.imin) d.imin = s.imin;
    if (s.imax > d.imax) d.imax = s.imax;
  }
  d.fmin = (s.fmin < d.fmin) ? s.fmin : d.fmin;
  d.fmax = (s.fmax > d.fmax) ? s.fmax : d.fmax;
}

void write_typed(OutCol& c, int64_t g, int32_t type, int64_t iv, long double fv)
{
  switch (type) {
    case T_INT8: put<int8_t>(c, g, (int8_t)iv); break;
    case T_UINT8: case T_BOOL8: put<uint8_t>(c, g, (uint8_t)iv); break;
    case T_INT16: put<int16_t>(c, g, (int16_t)iv); break;
    case T_UINT16: put<uint16_t>(c, g, (uint16_t)iv); break;
    case T_INT32: case T_TS_DAYS: case T_DUR_DAYS: case T_DEC32: put<int32_t>(c, g, (int32_t)iv); break;
    case T_UINT32: put<uint32_t>(c, g, (uint32_t)iv); break;
    case T_FLOAT32: put<float>(c, g, (float)fv); break;
    case T_FLOAT64: put<double>(c, g, (double)fv); break;
    default: put<int64_t>(c, g, iv); break;  // all 8-byte integer-backed types
  }
}

Result* run(const Col* keys, int nkeys, int null_policy, const Req* reqs, int nreqs,
            const uint32_t* const* filters, const int32_t* filter_offsets, int nfilters,
            int nthreads)
{
  auto res = std::make_unique<Result>();
  if (nkeys <= 0) { res->error = "no key columns"; return res.release(); }
  const int64_t n = keys[0].size;
  for (int q = 0; q < nreqs; ++q) {
    if (reqs[q].values.size != n) {
      res->error = "Size mismatch between request values and groupby keys.";
      return res.release();
    }
    for (int a = 0; a < reqs[q].naggs; ++a)
      if (check_combo(reqs[q].values.type_id, reqs[q].aggs[a].kind)) {
        res->error = "Invalid type/aggregation combination.";
        return res.release();
      }
  }
  const bool include = null_policy == 1;

  nthreads = std::max(1, nthreads);
  if (n < 100000) nthreads = 1;
  std::vector<Partial> parts((size_t)nthreads);
  if (nthreads == 1) {
    aggregate_range(parts[0], 0, n, keys, nkeys, include, reqs, nreqs, filters, filter_offsets, nfilters);
  } else {
    std::vector<std::thread> th;
    for (int t = 0; t < nthreads; ++t) {
      const int64_t lo = n * t / nthreads, hi = n * (t + 1) / nthreads;
      th.emplace_back([&, t, lo, hi] {
        aggregate_range(parts[(size_t)t], lo, hi, keys, nkeys, include, reqs, nreqs, filters,
                        filter_offsets, nfilters);
      });
    }
    for (auto& t : th) t.join();
    Partial& D = parts[0];
    for (int t = 1; t < nthreads; ++t) {
      Partial& S = parts[(size_t)t];
      for (auto& kv : S.index) {
        auto it = D.index.find(kv.first);
        int64_t g;
        if (it == D.index.end()) {
          g = (int64_t)D.groups.size();
          D.index.emplace(kv.first, g);
          D.groups.push_back(Group{S.groups[(size_t)kv.second].first_row, 0});
          D.accs.resize(D.accs.size() + (size_t)nreqs);
        } else g = it->second;
        D.groups[(size_t)g].rows += S.groups[(size_t)kv.second].rows;
        for (int q = 0; q < nreqs; ++q)
          merge_acc(D.accs[(size_t)(g * nreqs + q)], S.accs[(size_t)(kv.second * nreqs + q)], reqs[q].values);
      }
      S = Partial{};
    }
  }
  const Partial& P = parts[0];
  const int64_t G = (int64_t)P.groups.size();
  res->ngroups = G;

  // ---- keys: gather the representative rows verbatim
  res->keys.resize((size_t)nkeys);
  for (int k = 0; k < nkeys; ++k) {
    const Col& c = keys[k];
    OutCol& o = res->keys[(size_t)k];
    const bool nullable = include && c.mask != nullptr;
    if (c.type_id == T_STRING) {
      o.type_id = T_STRING; o.size = G; o.offsets.assign((size_t)G + 1, 0);
      if (nullable) o.mask.assign((size_t)((G + 31) / 32), 0xFFFFFFFFu);
      for (int64_t g = 0; g < G; ++g) {
        const int64_t r = (int64_t)c.offset + P.groups[(size_t)g].first_row;
        int64_t b = 0, e = 0;
        if (bit(c.mask, r)) {
          if (c.offsets_type == T_INT64) { b = ((const int64_t*)c.offsets)[r]; e = ((const int64_t*)c.offsets)[r + 1]; }
          else { b = ((const int32_t*)c.offsets)[r]; e = ((const int32_t*)c.offsets)[r + 1]; }
        } else if (nullable) set_null(o, g);
        o.data.insert(o.data.end(), (const uint8_t*)c.data + b, (const uint8_t*)c.data + e);
        o.offsets[(size_t)g + 1] = (int64_t)o.data.size();
      }
    } else {
      const int w = width_of(c.type_id);
      alloc(o, c.type_id, G, w, nullable);
      for (int64_t g = 0; g < G; ++g) {
        const int64_t r = (int64_t)c.offset + P.groups[(size_t)g].first_row;
        if (bit(c.mask, r)) std::memcpy(o.data.data() + g * w, (const char*)c.data + r * w, (size_t)w);
        else if (nullable) set_null(o, g);
      }
    }
  }

  // ---- results
  res->results.resize((size_t)nreqs);
  for (int q = 0; q < nreqs; ++q) {
    const int32_t st = reqs[q].values.type_id;
    // has_nulls() in the reference means null_count > 0, not "a mask is allocated"
    bool src_has_nulls = false;
    if (reqs[q].values.mask != nullptr)
      for (int64_t r = 0; r < n && !src_has_nulls; ++r)
        src_has_nulls = !bit(reqs[q].values.mask, (int64_t)reqs[q].values.offset + r);
    const bool flt = is_float(st);
    res->results[(size_t)q].resize((size_t)reqs[q].naggs);
    for (int a = 0; a < reqs[q].naggs; ++a) {
      const int32_t kind = reqs[q].aggs[a].kind;
      const int32_t ddof = reqs[q].aggs[a].ddof;
      const int32_t rt = result_type(st, kind);
      OutCol& o = res->results[(size_t)q][(size_t)a];
      bool nullable = src_has_nulls;
      if (kind == K_COUNT_VALID || kind == K_COUNT_ALL || kind == K_M2) nullable = false;
      if (kind == K_VAR || kind == K_STD) nullable = true;  // n - ddof <= 0 can always occur
      if (rt == T_STRING) {
        // MIN / MAX of strings: gather of the ARGMIN / ARGMAX rows, null where there is none
        // (cpp/src/groupby/hash/hash_compound_agg_finalizer.cu:39-76)
        const Col& c = reqs[q].values;
        o.type_id = T_STRING;
        o.size = G;
        o.offsets.assign((size_t)G + 1, 0);
        if (nullable) o.mask.assign((size_t)((G + 31) / 32), 0xFFFFFFFFu);
        for (int64_t g = 0; g < G; ++g) {
          const Acc& A = P.accs[(size_t)(g * nreqs + q)];
          const int64_t r = kind == K_MIN ? A.argmin : A.argmax;
          if (r < 0) {
            if (nullable) set_null(o, g);
          } else {
            int64_t b, e;
            if (c.offsets_type == T_INT64) { b = ((const int64_t*)c.offsets)[c.offset + r]; e = ((const int64_t*)c.offsets)[c.offset + r + 1]; }
            else { b = ((const int32_t*)c.offsets)[c.offset + r]; e = ((const int32_t*)c.offsets)[c.offset + r + 1]; }
            o.data.insert(o.data.end(), (const uint8_t*)c.data + b, (const uint8_t*)c.data + e);
          }
          o.offsets[(size_t)g + 1] = (int64_t)o.data.size();
        }
        continue;
      }
      if (kind == K_SUM_OVERFLOW) {
        // children without masks, values of a null struct 0 / false (sum_overflow_tests.cpp:200-211)
        const int w = width_of(st);
        alloc(o, T_STRUCT, G, w, nullable);
        o.child_type = st;
        o.data2.assign((size_t)G, 0);
        for (int64_t g = 0; g < G; ++g) {
          const Acc& A = P.accs[(size_t)(g * nreqs + q)];
          if (A.count == 0) { if (nullable) set_null(o, g); continue; }
          if (st == T_DEC128) {
            const __int128 top = A.hi128 + (__int128)(uint64_t)(A.lo128 >> 64);
            const unsigned __int128 sum = ((unsigned __int128)(uint64_t)top << 64) | (uint64_t)A.lo128;
            std::memcpy(o.data.data() + g * 16, &sum, 16);
            o.data2[(size_t)g] = (top < -((__int128)1 << 63) || top > (((__int128)1 << 63) - 1)) ? 1 : 0;
            continue;
          }
          const __int128 lo = -((__int128)1 << (8 * w - 1)), hi = ((__int128)1 << (8 * w - 1)) - 1;
          const int64_t wrapped = (int64_t)(uint64_t)A.xsum;  // low bits; write_typed narrows
          write_typed(o, g, st, wrapped, 0);
          o.data2[(size_t)g] = (A.xsum < lo || A.xsum > hi) ? 1 : 0;
        }
        continue;
      }
      alloc(o, rt, G, width_of(rt), nullable);
      for (int64_t g = 0; g < G; ++g) {
        const Acc& A = P.accs[(size_t)(g * nreqs + q)];
        const int64_t cnt = A.count;
        switch (kind) {
          case K_COUNT_VALID: put<int32_t>(o, g, (int32_t)cnt); break;
          case K_COUNT_ALL: put<int32_t>(o, g, (int32_t)P.groups[(size_t)g].rows); break;
          case K_SUM:
            if (cnt == 0) { if (nullable) set_null(o, g); break; }
            if (rt == T_DEC128) {
              const __int128 top = A.hi128 + (__int128)(uint64_t)(A.lo128 >> 64);
              const unsigned __int128 sum = ((unsigned __int128)(uint64_t)top << 64) | (uint64_t)A.lo128;
              std::memcpy(o.data.data() + g * 16, &sum, 16);
              break;
            }
            write_typed(o, g, rt, A.isum, A.fsum); break;
          case K_SUMSQ:
            if (cnt == 0) { if (nullable) set_null(o, g); break; }
            write_typed(o, g, rt, A.isumsq, A.fsumsq); break;
          case K_PRODUCT:
            if (cnt == 0) { if (nullable) set_null(o, g); break; }
            write_typed(o, g, rt, A.iprod, A.fprod); break;
          case K_MIN:
            if (cnt == 0) { if (nullable) set_null(o, g); break; }
            write_typed(o, g, rt, A.imin, A.fmin); break;
          case K_MAX:
            if (cnt == 0) { if (nullable) set_null(o, g); break; }
            write_typed(o, g, rt, A.imax, A.fmax); break;
          case K_ARGMIN: case K_ARGMAX: {
            const int64_t r = kind == K_ARGMIN ? A.argmin : A.argmax;
            if (r < 0) { if (nullable) set_null(o, g); break; }
            put<int32_t>(o, g, (int32_t)r);
            break;
          }
          case K_MEAN: {
            if (cnt == 0) { if (nullable) set_null(o, g); break; }
            if (is_duration(st)) { write_typed(o, g, rt, A.isum / cnt, 0); break; }
            const long double s = flt ? A.fsum : (long double)(double)A.isum;
            put<double>(o, g, (double)(s / (long double)cnt));
            break;
          }
          case K_M2: case K_VAR: case K_STD: {
            long double m2 = 0;
            if (cnt > 0) {
              const long double ss = flt ? A.fsumsq : (long double)(double)A.isumsq;
              const long double s = flt ? A.fsum : (long double)(double)A.isum;
              m2 = ss - s * s / (long double)cnt;
            }
            if (kind == K_M2) { put<double>(o, g, (double)m2); break; }
            const int64_t df = cnt - ddof;
            if (cnt == 0 || df <= 0) { set_null(o, g); break; }
            const long double var = m2 / (long double)df;
            put<double>(o, g, kind == K_VAR ? (double)var : (double)std::sqrt(var));
            break;
          }
          default: break;
        }
      }
    }
  }
  return res.release();
}

}  // namespace

extern "C" {

struct orc_col {
  int32_t type_id; int32_t size; const void* data; const uint32_t* mask; int32_t offset;
  int32_t offsets_type; const void* offsets;
};
struct orc_agg { int32_t kind; int32_t ddof; };
struct orc_req { orc_col values; int32_t naggs; const orc_agg* aggs; };

static Col to_col(const orc_col& c) { return Col{c.type_id, c.size, c.data, c.mask, c.offset, c.offsets, c.offsets_type}; }

void* orc_groupby(const orc_col* keys, int32_t nkeys, int32_t null_policy, const orc_req* reqs,
                  int32_t nreqs, const uint32_t* const* filters, const int32_t* filter_offsets,
                  int32_t nfilters, int32_t nthreads)
{
  std::vector<Col> k; for (int i = 0; i < nkeys; ++i) k.push_back(to_col(keys[i]));
  std::vector<Req> r;
  for (int i = 0; i < nreqs; ++i) r.push_back(Req{to_col(reqs[i].values), reqs[i].naggs, (const Agg*)reqs[i].aggs});
  return run(k.data(), nkeys, null_policy, r.data(), nreqs, filters, filter_offsets, nfilters, nthreads);
}
const char* orc_error(void* h) { auto* r = (Result*)h; return r->error.empty() ? nullptr : r->error.c_str(); }
int64_t orc_num_groups(void* h) { return ((Result*)h)->ngroups; }
static OutCol* pick(void* h, int32_t req, int32_t idx)
{
  auto* r = (Result*)h;
  return req < 0 ? &r->keys[(size_t)idx] : &r->results[(size_t)req][(size_t)idx];
}
// req < 0 selects key column idx; otherwise result idx of request req
int32_t orc_col_type(void* h, int32_t req, int32_t idx) { return pick(h, req, idx)->type_id; }
int64_t orc_col_bytes(void* h, int32_t req, int32_t idx) { return (int64_t)pick(h, req, idx)->data.size(); }
const void* orc_col_data(void* h, int32_t req, int32_t idx) { return pick(h, req, idx)->data.data(); }
const uint32_t* orc_col_mask(void* h, int32_t req, int32_t idx)
{
  auto* c = pick(h, req, idx); return c->mask.empty() ? nullptr : c->mask.data();
}
int64_t orc_col_null_count(void* h, int32_t req, int32_t idx) { return pick(h, req, idx)->null_count; }
// STRUCT results: the type of child 0 (whose bytes orc_col_data returns) and the BOOL8 bytes of child 1
int32_t orc_col_child_type(void* h, int32_t req, int32_t idx) { return pick(h, req, idx)->child_type; }
const void* orc_col_data2(void* h, int32_t req, int32_t idx) { return pick(h, req, idx)->data2.data(); }
int64_t orc_col_bytes2(void* h, int32_t req, int32_t idx) { return (int64_t)pick(h, req, idx)->data2.size(); }
const int64_t* orc_col_offsets(void* h, int32_t req, int32_t idx)
{
  auto* c = pick(h, req, idx); return c->offsets.empty() ? nullptr : c->offsets.data();
}
void orc_free(void* h) { delete (Result*)h; }

}  // extern "C"
