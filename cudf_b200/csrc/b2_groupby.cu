// b2_groupby.cu — host side of the engine and the C ABI declared in include/b2_groupby.h.
//
// Host flow of one aggregate call (reference flow: cpp/src/groupby/groupby.cu:219-236 →
// cpp/src/groupby/hash/groupby.cu:134-147 → compute_groupby.cu:51-155):
//   validate → plan (key packing, accumulator cells, outputs) → size the global table →
//   k_table_init → k_aggregate → read the control block (ONE stream sync: group count and the
//   overflow flag) → allocate outputs from the caller's allocator → k_finalize → null counts.
// Without a hint the first table is small and speculative; if it overflows, a HyperLogLog pass over the
// keys sizes the table for the repeated pass (B2_TRACE=1 prints the phases of a call to stderr).
#include "../../include/b2_groupby.h"
#include "b2_kernels.cuh"
#include "b2_lean.cuh"
#include "b2_partition.cuh"

#include <dlfcn.h>
#include <nccl.h>

#include <algorithm>
#include <cmath>
#include <cstdio>
#include <chrono>
#include <cstring>
#include <functional>
#include <memory>
#include <mutex>
#include <string>
#include <vector>

using namespace b2;

namespace {

thread_local std::string g_last_error;
thread_local b2_call_stats g_stats{};

struct Err {
  b2_status code;
  std::string msg;
};
#define B2_FAIL(code, msg) throw Err{code, msg}
#define CUDA_TRY(expr)                                                                          \
  do {                                                                                          \
    cudaError_t e_ = (expr);                                                                    \
    if (e_ != cudaSuccess) {                                                                    \
      B2_FAIL(e_ == cudaErrorMemoryAllocation ? B2_OUT_OF_MEMORY : B2_CUDA_ERROR,               \
              std::string("CUDA error at " #expr ": ") + cudaGetErrorName(e_) + " " +           \
                cudaGetErrorString(e_));                                                        \
    }                                                                                           \
  } while (0)

template <typename F>
b2_status guarded(F&& f)
{
  try {
    f();
    return B2_SUCCESS;
  } catch (const Err& e) {
    g_last_error = e.msg;
    return e.code;
  } catch (const std::bad_alloc&) {
    g_last_error = "host allocation failed";
    return B2_OUT_OF_MEMORY;
  } catch (const std::exception& e) {
    g_last_error = e.what();
    return B2_INTERNAL_ERROR;
  }
}

// ------------------------------------------------------------------------------ device facts
struct DeviceInfo {
  int sms = 0;
  int smem_optin = 0;
};
const DeviceInfo& device_info()
{
  static thread_local int cached_dev = -1;
  static thread_local DeviceInfo info;
  int dev = 0;
  CUDA_TRY(cudaGetDevice(&dev));
  if (dev != cached_dev) {
    CUDA_TRY(cudaDeviceGetAttribute(&info.sms, cudaDevAttrMultiProcessorCount, dev));
    CUDA_TRY(cudaDeviceGetAttribute(&info.smem_optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev));
    cached_dev = dev;
  }
  return info;
}

// The library's own temporaries come from the device's default stream-ordered pool.  The first
// allocation a thread makes on a device tells that pool to keep freed memory cached between calls
// (the default threshold returns it to the driver at every synchronisation).  Entry points that
// allocate nothing never get here.
void keep_pool_cached()
{
  static thread_local int tuned_dev = -1;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev == tuned_dev) return;
  cudaMemPool_t pool;
  if (cudaDeviceGetDefaultMemPool(&pool, dev) == cudaSuccess) {
    unsigned long long keep = ~0ull;
    cudaMemPoolSetAttribute(pool, cudaMemPoolAttrReleaseThreshold, &keep);
  }
  tuned_dev = dev;
}

// ------------------------------------------------------------------------------ memory
void* default_alloc(size_t bytes, void* stream, void*)
{
  void* p = nullptr;
  if (bytes == 0) bytes = 8;
  keep_pool_cached();
  if (cudaMallocAsync(&p, bytes, (cudaStream_t)stream) != cudaSuccess) { cudaGetLastError(); return nullptr; }
  return p;
}
void default_free(void* p, size_t, void* stream, void*)
{
  if (p) cudaFreeAsync(p, (cudaStream_t)stream);
}
b2_allocator resolve(const b2_allocator* a)
{
  if (a && a->allocate && a->deallocate) return *a;
  return b2_allocator{default_alloc, default_free, nullptr};
}

struct Scratch {  // stream-ordered temporary, freed on scope exit
  void* p = nullptr;
  size_t bytes = 0;
  cudaStream_t stream = nullptr;
  Scratch() = default;
  Scratch(size_t n, cudaStream_t s) : bytes(n), stream(s)
  {
    p = default_alloc(n, s, nullptr);
    if (!p) B2_FAIL(B2_OUT_OF_MEMORY, "out of device memory allocating " + std::to_string(n) + " bytes of scratch");
    g_stats.scratch_bytes += (int64_t)n;
  }
  Scratch(Scratch&& o) noexcept { *this = std::move(o); }
  Scratch& operator=(Scratch&& o) noexcept
  {
    release();
    p = o.p; bytes = o.bytes; stream = o.stream; o.p = nullptr;
    return *this;
  }
  Scratch(const Scratch&) = delete;
  Scratch& operator=(const Scratch&) = delete;
  void release() { if (p) { cudaFreeAsync(p, stream); p = nullptr; } }
  ~Scratch() { release(); }
};

// ------------------------------------------------------------------------------ type facts
bool is_float_t(int t) { return t == B2_FLOAT32 || t == B2_FLOAT64; }
bool is_duration_t(int t) { return t >= B2_DURATION_DAYS && t <= B2_DURATION_NANOSECONDS; }
bool is_timestamp_t(int t) { return t >= B2_TIMESTAMP_DAYS && t <= B2_TIMESTAMP_NANOSECONDS; }
bool is_numeric_t(int t) { return t >= B2_INT8 && t <= B2_BOOL8; }
// DECIMAL32/64 are served as their integer representation + scale; DECIMAL128 is not (no 16-byte atomics here)
bool is_decimal_t(int t) { return t == B2_DECIMAL32 || t == B2_DECIMAL64; }
// DECIMAL128 values: SUM and SUM_OVERFLOW only, like the reference's hash path (cpp/src/groupby/hash/groupby.cu:82-85);
// a column takes two value slots, its low and its high words.  The second slot carries this internal type.
constexpr int VT_DEC128_HIGH = 1000;

int width_of(int t)
{
  switch (t) {
    case B2_INT8: case B2_UINT8: case B2_BOOL8: return 1;
    case B2_INT16: case B2_UINT16: return 2;
    case B2_INT32: case B2_UINT32: case B2_FLOAT32: case B2_TIMESTAMP_DAYS: case B2_DURATION_DAYS:
    case B2_DECIMAL32: return 4;
    case B2_INT64: case B2_UINT64: case B2_FLOAT64: case B2_TIMESTAMP_SECONDS: case B2_TIMESTAMP_MILLISECONDS:
    case B2_TIMESTAMP_MICROSECONDS: case B2_TIMESTAMP_NANOSECONDS: case B2_DURATION_SECONDS:
    case B2_DURATION_MILLISECONDS: case B2_DURATION_MICROSECONDS: case B2_DURATION_NANOSECONDS:
    case B2_DECIMAL64: return 8;
    default: return 0;
  }
}
int vclass_of(int t)
{
  switch (t) {
    case B2_INT8: return VC_I8;
    case B2_INT16: return VC_I16;
    case B2_INT32: case B2_TIMESTAMP_DAYS: case B2_DURATION_DAYS: case B2_DECIMAL32: return VC_I32;
    case B2_UINT8: return VC_U8;
    case B2_UINT16: return VC_U16;
    case B2_UINT32: return VC_U32;
    case B2_UINT64: return VC_U64;
    case B2_FLOAT32: return VC_F32;
    case B2_FLOAT64: return VC_F64;
    case B2_BOOL8: return VC_BOOL;
    case B2_STRING: return VC_STRING;
    case B2_DECIMAL128: return VC_U64X2;
    case VT_DEC128_HIGH: return VC_I64X2;
    default: return width_of(t) == 8 ? VC_I64 : VC_NONE;
  }
}

// result element type: cpp/include/cudf/detail/aggregation/aggregation.hpp:884-1013
int result_type(int src, int kind)
{
  switch (kind) {
    case B2_AGG_COUNT_VALID: case B2_AGG_COUNT_ALL: case B2_AGG_ARGMAX: case B2_AGG_ARGMIN: return B2_INT32;
    case B2_AGG_MIN: case B2_AGG_MAX: return src;
    case B2_AGG_SUM: return (is_float_t(src) || is_duration_t(src) || is_decimal_t(src) || src == B2_DECIMAL128) ? src : B2_INT64;  // decimals keep type and scale
    case B2_AGG_SUM_OVERFLOW: return B2_STRUCT;  // {sum: the source type, overflow: BOOL8} (aggregation.hpp:990-995)
    case B2_AGG_SUM_OF_SQUARES: case B2_AGG_PRODUCT: return is_float_t(src) ? src : B2_INT64;
    case B2_AGG_MEAN: return is_duration_t(src) ? src : B2_FLOAT64;
    default: return B2_FLOAT64;
  }
}

// 0 = served here, 1 = invalid combination (the reference throws), 2 = valid in the reference but
// only its sort path / ARGMIN path serves it
int classify_request(int src, int kind)
{
  switch (kind) {
    case B2_AGG_COUNT_VALID: case B2_AGG_COUNT_ALL: return 0;
    case B2_AGG_MIN: case B2_AGG_MAX: case B2_AGG_ARGMAX: case B2_AGG_ARGMIN:
      // MIN / MAX of strings run as ARGMIN / ARGMAX + gather, like the reference's
      // (cpp/src/groupby/hash/extract_single_pass_aggs.cpp:39-60, hash_compound_agg_finalizer.cu:39-76)
      if (is_numeric_t(src) || is_timestamp_t(src) || is_duration_t(src) || is_decimal_t(src) || src == B2_STRING) return 0;
      if (src == B2_DECIMAL128 || src == B2_DICTIONARY32 || src == B2_STRUCT || src == B2_LIST) return 2;
      return 1;
    case B2_AGG_SUM:
      // decimal SUM / MIN / MAX run on the hash path of the reference too
      // (cpp/tests/groupby/sum_tests.cpp:220-248, min_tests.cpp:271-292, max_tests.cpp:279-300)
      if (is_numeric_t(src) || is_duration_t(src) || is_decimal_t(src) || src == B2_DECIMAL128) return 0;
      if (src == B2_DICTIONARY32) return 2;
      return 1;
    case B2_AGG_SUM_OVERFLOW:
      // signed integers and decimals (cpp/include/cudf/detail/aggregation/aggregation.hpp:980-995,
      // cpp/tests/groupby/sum_overflow_tests.cpp:495-561: BOOL8 and the unsigned types throw)
      if (src == B2_INT8 || src == B2_INT16 || src == B2_INT32 || src == B2_INT64 || is_decimal_t(src) ||
          src == B2_DECIMAL128)
        return 0;
      return 1;
    case B2_AGG_MEAN:
      if (is_numeric_t(src) || is_duration_t(src)) return 0;
      if (src == B2_DECIMAL32 || src == B2_DECIMAL64 || src == B2_DECIMAL128 || src == B2_DICTIONARY32) return 2;
      return 1;
    case B2_AGG_SUM_OF_SQUARES: case B2_AGG_PRODUCT: case B2_AGG_M2: case B2_AGG_VARIANCE: case B2_AGG_STD:
      if (is_numeric_t(src)) return 0;
      if (src == B2_DICTIONARY32) return 2;
      return 1;
    default:
      return (kind >= 0 && kind <= 40) ? 2 : 1;  // other reference kinds: sort path
  }
}

// ------------------------------------------------------------------------------ views
struct ColView {  // deep copy of a b2_column_view (children included)
  b2_column_view v{};
  std::vector<ColView> kids;
  std::vector<b2_column_view> kid_views;
  explicit ColView(const b2_column_view& in) : v(in)
  {
    for (int i = 0; i < in.num_children; ++i) kids.emplace_back(in.children[i]);
    for (auto& k : kids) kid_views.push_back(k.v);
    v.children = kid_views.empty() ? nullptr : kid_views.data();
  }
  ColView(const ColView& o) : ColView(o.v) {}
  ColView& operator=(const ColView& o)
  {
    if (this != &o) { ColView t(o.v); v = t.v; kids = t.kids; kid_views.clear(); for (auto& k : kids) kid_views.push_back(k.v); v.children = kid_views.empty() ? nullptr : kid_views.data(); }
    return *this;
  }
};

}  // namespace

// ------------------------------------------------------------------------------ objects
struct b2_groupby {
  std::vector<ColView> keys;
  int null_policy = B2_NULL_EXCLUDE;
  int64_t expected_groups = 0;
  int table_variant = 0;
  int shared_table_bytes = 0;
  std::vector<const uint32_t*> filters;
  std::vector<int32_t> filter_offsets;
};

namespace {

struct OutSpec {  // one requested aggregation → one result column
  int req, agg;
  int kind;      // OutKind
  int rtype;     // b2_type_id of the result
  int ctype = 0; // OK_SUMOVF: type of the struct's sum child (the source type)
  int scale = 0; // decimal results: the source column's scale
  int c_a = -1, c_b = -1, c_cnt = -1;
  int ddof = 1;
  int src_float = 0;
  bool nullable = false;
};

struct Schema {  // everything that is fixed by (key types, requests): cells and outputs
  int key_mode = KM_PACKED;
  int nkeys = 0;
  int include_nulls = 0;
  int key_types[MAX_KEYS]{};
  int key_width[MAX_KEYS]{};
  int key_shift[MAX_KEYS]{};
  int key_nullbit[MAX_KEYS]{};
  bool key_nullable[MAX_KEYS]{};
  int key_scale[MAX_KEYS]{};  // decimal keys keep their scale
  int nvals = 0;
  int val_types[MAX_VALS]{};
  int ncells = 0;
  DCell cells[MAX_CELLS]{};
  std::vector<OutSpec> outs;
  std::vector<int> req_nouts;
  std::vector<int> req_val;  // request → value column slot
  bool f32mean = false;      // cells == {Σ of a FLOAT32 column, n of it}: compact shared-memory layout
  bool f64mean = false;      // cells == {Σ of a FLOAT64 column, n of it}: the lean kernel keeps Σ as fixed-point limbs
  bool fixed = false;        // cells ⊆ {Σx, n, Σx²} of ONE float column: the partitioned path folds hot keys and keeps fixed-point cells
  bool has_arg = false;      // some cell holds a row index (ARGMIN / ARGMAX, MIN / MAX of strings): such cells
                             // live in the global table of ONE aggregate call only (no shared-memory copies,
                             // no partial records: a row index means nothing outside its batch)
};

}  // namespace

struct b2_groupby_state {
  Schema sc;
  DPlan plan{};          // schema part filled; pointers filled per update
  u64* table = nullptr;  // (cap + 1) * stride cells
  int64_t cap = 0;
  int64_t dense_slots = 0;  // directly addressed slots behind the special slot
  DCtrl* ctrl = nullptr;
  DCtrl host_ctrl{};     // last read-back
  bool ctrl_fresh = false;
  bool has_rows = false;     // a row-keyed table references the rows of one update
  std::vector<ColView> row_keys;  // key views of that update (row-key mode output gather)
  int64_t expected_groups = 0;
  cudaStream_t last_stream = nullptr;
  // a state filled by the partitioned path holds its finished groups as a compact list instead of a
  // table: structure-of-arrays, word w of group g at groups[w * groups_cap + g], word 0 = key cell
  Scratch groups;
  int64_t groups_cap = 0;
  int64_t groups_n = -1;  // -1 = no list
  // One-shot calls: the first table attempt may leave its control block unread, so that the result columns
  // are allocated (for `deferred_bound` groups) and k_finalize is enqueued while the fused kernel still runs,
  // and ONE synchronisation reads group count, overflow flags and null counts together.
  bool deferred = false;
  bool deferred_lean = false;    // the lean kernel ran alone in that attempt
  int64_t deferred_cap = 0;      // capacity of that attempt's table
  int64_t deferred_bound = 0;    // most groups that attempt can leave in the table without raising its overflow flag
};

namespace {

// ------------------------------------------------------------------------------ planning
void validate_requests(const b2_groupby& gb, const b2_aggregation_request* reqs, int nreqs)
{
  if (nreqs < 0 || (nreqs > 0 && !reqs)) B2_FAIL(B2_INVALID_ARGUMENT, "requests is null");
  const int n = gb.keys.empty() ? 0 : gb.keys[0].v.size;
  for (int r = 0; r < nreqs; ++r) {
    // cpp/src/groupby/groupby.cu:225-229
    if (reqs[r].values.size != n) B2_FAIL(B2_LOGIC_ERROR, "Size mismatch between request values and groupby keys.");
    if (reqs[r].num_aggregations < 0 || (reqs[r].num_aggregations > 0 && !reqs[r].aggregations))
      B2_FAIL(B2_INVALID_ARGUMENT, "aggregations is null");
  }
  bool unsupported = false;
  for (int r = 0; r < nreqs; ++r)
    for (int a = 0; a < reqs[r].num_aggregations; ++a) {
      const int c = classify_request(reqs[r].values.type_id, reqs[r].aggregations[a].kind);
      // cpp/src/groupby/groupby.cu:188-201
      if (c == 1) B2_FAIL(B2_LOGIC_ERROR, "Invalid type/aggregation combination.");  // CUDF_EXPECTS default: cudf::logic_error
      if (c == 2) unsupported = true;
    }
  if (unsupported)
    B2_FAIL(B2_UNSUPPORTED, "request is served by the reference's sort-based groupby, not by the hash path");
}

Schema make_schema(const b2_groupby& gb, const b2_aggregation_request* reqs, int nreqs)
{
  Schema sc;
  sc.nkeys = (int)gb.keys.size();
  if (sc.nkeys == 0) B2_FAIL(B2_LOGIC_ERROR, "groupby needs at least one key column");
  if (sc.nkeys > MAX_KEYS) B2_FAIL(B2_UNSUPPORTED, "more than 16 key columns");
  sc.include_nulls = gb.null_policy == B2_NULL_INCLUDE;

  bool packed = true;
  int bits = 0;
  for (int k = 0; k < sc.nkeys; ++k) {
    const b2_column_view& c = gb.keys[k].v;
    const int w = width_of(c.type_id);
    if (c.type_id == B2_STRING) {
      if (c.size > 0 && (c.num_children < 1 || !c.children ||
                         (c.children[0].type_id != B2_INT32 && c.children[0].type_id != B2_INT64)))
        B2_FAIL(B2_INVALID_ARGUMENT, "STRING key column needs an INT32 or INT64 offsets child");
      packed = false;
    } else if (w == 0) {
      B2_FAIL(B2_UNSUPPORTED, "key column type is not served by the hash path of this engine");
    } else if (is_float_t(c.type_id)) {
      packed = false;  // keys compare by value (+0 == -0, NaN == NaN) but are output verbatim
    }
    sc.key_types[k] = c.type_id;
    sc.key_scale[k] = c.scale;
    sc.key_width[k] = w;
    sc.key_shift[k] = bits;
    sc.key_nullable[k] = c.null_mask != nullptr;
    bits += 8 * w;
  }
  for (int k = 0; k < sc.nkeys; ++k) {
    sc.key_nullbit[k] = -1;
    if (sc.include_nulls && sc.key_nullable[k]) sc.key_nullbit[k] = bits++;
  }
  if (bits > 64) packed = false;
  sc.key_mode = packed ? KM_PACKED : KM_ROWS;

  // value columns: identical views share one slot
  struct VKey { const void* d; const void* m; int off, type; };
  std::vector<VKey> seen;
  struct Need { bool sum = false, cnt = false, ssq = false, mn = false, mx = false, prod = false, nulls = false,
                amin = false, amax = false, ovf8 = false; };
  std::vector<Need> need;
  sc.req_val.resize((size_t)nreqs);
  bool need_cnt_all = false;
  for (int r = 0; r < nreqs; ++r) {
    const b2_column_view& v = reqs[r].values;
    int slot = -1;
    for (size_t i = 0; i < seen.size(); ++i)
      if (seen[i].d == v.data && seen[i].m == v.null_mask && seen[i].off == v.offset && seen[i].type == v.type_id)
        slot = (int)i;
    if (slot < 0) {
      if ((int)seen.size() >= MAX_VALS) B2_FAIL(B2_UNSUPPORTED, "more than 16 distinct value columns");
      slot = (int)seen.size();
      seen.push_back(VKey{v.data, v.null_mask, v.offset, v.type_id});
      need.emplace_back();
      sc.val_types[slot] = v.type_id;
      if (v.type_id == B2_DECIMAL128) {  // the slot of the high words follows
        if ((int)seen.size() >= MAX_VALS) B2_FAIL(B2_UNSUPPORTED, "more than 16 distinct value columns");
        seen.push_back(VKey{nullptr, nullptr, -1, VT_DEC128_HIGH});
        need.emplace_back();
        sc.val_types[slot + 1] = VT_DEC128_HIGH;
      }
    }
    sc.req_val[(size_t)r] = slot;
    Need& nd = need[(size_t)slot];
    const bool has_nulls = v.null_mask != nullptr && v.null_count != 0;
    nd.nulls = nd.nulls || has_nulls;
    for (int a = 0; a < reqs[r].num_aggregations; ++a) {
      switch (reqs[r].aggregations[a].kind) {
        case B2_AGG_SUM: nd.sum = true; break;
        // SUM_OVERFLOW: sources of up to 32 bits share the int64 Σ cell of SUM (it cannot wrap below 2^31 rows);
        // a 64-bit source gets two cells that hold its exact sum
        case B2_AGG_SUM_OVERFLOW:
          if (width_of(v.type_id) == 8) nd.ovf8 = true; else nd.sum = true;  // (DECIMAL128: the four cells of its SUM)
          break;
        case B2_AGG_COUNT_VALID: nd.cnt = true; break;
        case B2_AGG_COUNT_ALL: need_cnt_all = true; break;
        case B2_AGG_MIN: if (v.type_id == B2_STRING) nd.amin = true; else nd.mn = true; break;
        case B2_AGG_MAX: if (v.type_id == B2_STRING) nd.amax = true; else nd.mx = true; break;
        case B2_AGG_ARGMIN: nd.amin = true; break;
        case B2_AGG_ARGMAX: nd.amax = true; break;
        case B2_AGG_PRODUCT: nd.prod = true; break;
        case B2_AGG_SUM_OF_SQUARES: nd.ssq = true; break;
        case B2_AGG_MEAN: nd.sum = nd.cnt = true; break;
        default: nd.sum = nd.cnt = nd.ssq = true; break;  // M2, VARIANCE, STD
      }
    }
  }
  sc.nvals = (int)seen.size();

  // cells, per value column in the order Σ, n, Σx², min, max, Π; the row count last
  struct CellIdx { int sum = -1, cnt = -1, ssq = -1, mn = -1, mx = -1, prod = -1, amin = -1, amax = -1, hi = -1, lo = -1; };
  std::vector<CellIdx> idx((size_t)sc.nvals);
  auto add_cell = [&](int op, int col) {
    if (sc.ncells >= MAX_CELLS) B2_FAIL(B2_UNSUPPORTED, "too many accumulators in one aggregate call");
    sc.cells[sc.ncells] = DCell{(unsigned char)op, (unsigned char)col};
    return sc.ncells++;
  };
  for (int s = 0; s < sc.nvals; ++s) {
    Need& nd = need[(size_t)s];
    const int t = sc.val_types[s];
    const bool f = is_float_t(t);
    const bool uns = t == B2_UINT64;
    if (nd.nulls && (nd.sum || nd.ssq || nd.mn || nd.mx || nd.prod || nd.ovf8)) nd.cnt = true;  // decides validity
    if (nd.amin) { idx[(size_t)s].amin = add_cell(OP_ARGMIN, s); sc.has_arg = true; }
    if (nd.amax) { idx[(size_t)s].amax = add_cell(OP_ARGMAX, s); sc.has_arg = true; }
    if (nd.sum && t == B2_DECIMAL128) {
      // four exact chunk sums over the two word slots, adjacent and in this order (sum128 on the device)
      idx[(size_t)s].sum = add_cell(OP_SUM_LO, s);
      add_cell(OP_SUM_HIU, s);
      add_cell(OP_SUM_LO, s + 1);
      add_cell(OP_SUM_HI, s + 1);
    } else if (nd.sum) {
      idx[(size_t)s].sum = add_cell(f ? OP_SUM_F : OP_SUM_I, s);
    }
    if (nd.cnt) idx[(size_t)s].cnt = add_cell(OP_CNT_V, s);
    if (nd.ssq) idx[(size_t)s].ssq = add_cell(f ? OP_SSQ_F : OP_SSQ_I, s);
    if (nd.mn) idx[(size_t)s].mn = add_cell(f ? OP_MIN_F : uns ? OP_MIN_U : OP_MIN_I, s);
    if (nd.mx) idx[(size_t)s].mx = add_cell(f ? OP_MAX_F : uns ? OP_MAX_U : OP_MAX_I, s);
    if (nd.prod) idx[(size_t)s].prod = add_cell(f ? OP_PROD_F : OP_PROD_I, s);
    if (nd.ovf8) { idx[(size_t)s].hi = add_cell(OP_SUM_HI, s); idx[(size_t)s].lo = add_cell(OP_SUM_LO, s); }
  }
  int cnt_all = -1;
  if (need_cnt_all) cnt_all = add_cell(OP_CNT_A, 0);

  // outputs
  sc.req_nouts.resize((size_t)nreqs);
  for (int r = 0; r < nreqs; ++r) {
    const int s = sc.req_val[(size_t)r];
    const int t = reqs[r].values.type_id;
    const bool f = is_float_t(t);
    const bool has_nulls = reqs[r].values.null_mask != nullptr && reqs[r].values.null_count != 0;
    const CellIdx& ci = idx[(size_t)s];
    sc.req_nouts[(size_t)r] = reqs[r].num_aggregations;
    for (int a = 0; a < reqs[r].num_aggregations; ++a) {
      OutSpec o;
      o.req = r; o.agg = a;
      const int kind = reqs[r].aggregations[a].kind;
      o.rtype = result_type(t, kind);
      o.scale = (is_decimal_t(o.rtype) || o.rtype == B2_DECIMAL128) ? reqs[r].values.scale : 0;
      o.ddof = reqs[r].aggregations[a].ddof;
      o.src_float = f;
      o.c_cnt = has_nulls ? ci.cnt : -1;
      o.nullable = has_nulls;  // cpp/src/groupby/hash/output_utils.cu:61-68
      switch (kind) {
        case B2_AGG_COUNT_VALID: o.kind = OK_COUNT; o.c_a = ci.cnt; o.c_cnt = -1; o.nullable = false; break;
        case B2_AGG_COUNT_ALL: o.kind = OK_COUNT; o.c_a = cnt_all; o.c_cnt = -1; o.nullable = false; break;
        case B2_AGG_SUM_OVERFLOW:
          o.kind = OK_SUMOVF; o.ctype = t; o.scale = (is_decimal_t(t) || t == B2_DECIMAL128) ? reqs[r].values.scale : 0;
          if (width_of(t) == 8) { o.c_a = ci.hi; o.c_b = ci.lo; } else { o.c_a = ci.sum; }
          break;
        case B2_AGG_SUM: o.kind = t == B2_DECIMAL128 ? OK_SUM128 : f ? OK_FLT : OK_INT; o.c_a = ci.sum; break;
        case B2_AGG_SUM_OF_SQUARES: o.kind = f ? OK_FLT : OK_INT; o.c_a = ci.ssq; break;
        case B2_AGG_PRODUCT: o.kind = f ? OK_FLT : OK_INT; o.c_a = ci.prod; break;
        case B2_AGG_MIN:
          if (t == B2_STRING) { o.kind = OK_STRARG; o.c_a = ci.amin; o.c_cnt = -1; }
          else { o.kind = f ? OK_MINMAX_F : OK_INT; o.c_a = ci.mn; }
          break;
        case B2_AGG_MAX:
          if (t == B2_STRING) { o.kind = OK_STRARG; o.c_a = ci.amax; o.c_cnt = -1; }
          else { o.kind = f ? OK_MINMAX_F : OK_INT; o.c_a = ci.mx; }
          break;
        case B2_AGG_ARGMIN: o.kind = OK_ARG; o.c_a = ci.amin; o.c_cnt = -1; break;
        case B2_AGG_ARGMAX: o.kind = OK_ARG; o.c_a = ci.amax; o.c_cnt = -1; break;
        case B2_AGG_MEAN: o.kind = OK_MEAN; o.c_a = ci.sum; o.c_cnt = ci.cnt; break;
        case B2_AGG_M2: o.kind = OK_M2; o.c_a = ci.sum; o.c_b = ci.ssq; o.c_cnt = ci.cnt; o.nullable = false; break;
        case B2_AGG_VARIANCE: o.kind = OK_VAR; o.c_a = ci.sum; o.c_b = ci.ssq; o.c_cnt = ci.cnt; o.nullable = true; break;
        default: o.kind = OK_STD; o.c_a = ci.sum; o.c_b = ci.ssq; o.c_cnt = ci.cnt; o.nullable = true; break;
      }
      sc.outs.push_back(o);
    }
  }
  if ((int)sc.outs.size() > MAX_OUTS) B2_FAIL(B2_UNSUPPORTED, "more than 64 aggregations in one aggregate call");
  sc.f32mean = sc.key_mode == KM_PACKED && sc.ncells == 2 && sc.cells[0].op == OP_SUM_F && sc.cells[1].op == OP_CNT_V &&
               sc.cells[0].col == sc.cells[1].col && sc.val_types[sc.cells[0].col] == B2_FLOAT32;
  sc.f64mean = sc.key_mode == KM_PACKED && sc.ncells == 2 && sc.cells[0].op == OP_SUM_F && sc.cells[1].op == OP_CNT_V &&
               sc.cells[0].col == sc.cells[1].col && sc.val_types[sc.cells[0].col] == B2_FLOAT64;
  if (sc.key_mode == KM_PACKED && !sc.f32mean && sc.nvals == 1 && is_float_t(sc.val_types[0]) && sc.ncells >= 1) {
    sc.fixed = true;
    for (int c = 0; c < sc.ncells; ++c) {
      const int op = sc.cells[c].op;
      sc.fixed = sc.fixed && (op == OP_SUM_F || op == OP_CNT_V || op == OP_SSQ_F);
    }
  }
  return sc;
}

// schema part of the device plan
void fill_plan_schema(DPlan& P, const Schema& sc)
{
  std::memset(&P, 0, sizeof(P));
  P.nkeys = sc.nkeys; P.nvals = sc.nvals; P.ncells = sc.ncells; P.key_mode = sc.key_mode;
  P.include_nulls = sc.include_nulls; P.stride = 1 + sc.ncells;
  for (int k = 0; k < sc.nkeys; ++k) {
    P.keys[k].vclass = vclass_of(sc.key_types[k]);
    P.keys[k].width = sc.key_width[k];
    P.keys[k].shift = sc.key_shift[k];
    P.keys[k].nullbit = sc.key_nullbit[k];
    const int t = sc.key_types[k];
    P.keys[k].is_signed = !(t == B2_UINT8 || t == B2_UINT16 || t == B2_UINT32 || t == B2_UINT64 || t == B2_BOOL8);
  }
  for (int s = 0; s < sc.nvals; ++s) P.vals[s].vclass = vclass_of(sc.val_types[s]);
  for (int c = 0; c < sc.ncells; ++c) P.cells[c] = sc.cells[c];
}

// pointer part: the views of one update
void bind_plan_inputs(DPlan& P, const Schema& sc, const b2_groupby& gb, const b2_aggregation_request* reqs, int nreqs)
{
  if ((int)gb.keys.size() != sc.nkeys) B2_FAIL(B2_LOGIC_ERROR, "key schema differs from the state's");
  P.nrows = gb.keys[0].v.size;
  for (int k = 0; k < sc.nkeys; ++k) {
    const b2_column_view& c = gb.keys[k].v;
    if (c.type_id != sc.key_types[k]) B2_FAIL(B2_LOGIC_ERROR, "key schema differs from the state's");
    if (sc.key_mode == KM_PACKED && sc.key_nullbit[k] < 0 && sc.include_nulls && c.null_mask)
      B2_FAIL(B2_LOGIC_ERROR, "key column gained a null mask after the state was created");
    P.keys[k].data = (const unsigned char*)c.data;
    P.keys[k].mask = c.null_mask;
    P.keys[k].offset = c.offset;
    P.keys[k].offsets = nullptr;
    P.keys[k].offs64 = 0;
    if (c.type_id == B2_STRING && c.num_children > 0) {
      const b2_column_view& o = c.children[0];
      P.keys[k].offsets = (const unsigned char*)o.data + (size_t)o.offset * (o.type_id == B2_INT64 ? 8 : 4);
      P.keys[k].offs64 = o.type_id == B2_INT64;
    }
  }
  std::vector<bool> bound((size_t)sc.nvals, false);
  for (int r = 0; r < nreqs; ++r) {
    const int s = sc.req_val[(size_t)r];
    const b2_column_view& v = reqs[r].values;
    if (v.type_id != sc.val_types[s]) B2_FAIL(B2_LOGIC_ERROR, "request schema differs from the state's");
    if (bound[(size_t)s]) continue;
    bound[(size_t)s] = true;
    P.vals[s].data = (const unsigned char*)v.data;
    P.vals[s].mask = (v.null_mask && v.null_count != 0) ? v.null_mask : nullptr;
    P.vals[s].offset = v.offset;
    P.vals[s].offsets = nullptr;
    P.vals[s].offs64 = 0;
    if (v.type_id == B2_DECIMAL128) {  // the high words: the same rows, 8 bytes further
      P.vals[s + 1] = P.vals[s];
      P.vals[s + 1].data = v.data ? (const unsigned char*)v.data + 8 : nullptr;
      P.vals[s + 1].vclass = VC_I64X2;
      bound[(size_t)s + 1] = true;
    }
    if (v.type_id == B2_STRING) {
      if (v.size > 0 && (v.num_children < 1 || !v.children ||
                         (v.children[0].type_id != B2_INT32 && v.children[0].type_id != B2_INT64)))
        B2_FAIL(B2_INVALID_ARGUMENT, "STRING values column needs an INT32 or INT64 offsets child");
      if (v.num_children > 0 && v.children) {
        const b2_column_view& o = v.children[0];
        P.vals[s].offsets = (const unsigned char*)o.data + (size_t)o.offset * (o.type_id == B2_INT64 ? 8 : 4);
        P.vals[s].offs64 = o.type_id == B2_INT64;
      }
    }
  }
  // 16-byte vector loads of 4 consecutive rows need aligned column starts
  auto aligned = [](const void* base, int64_t offset, int width) {
    const uintptr_t a = (uintptr_t)base + (uintptr_t)offset * (uintptr_t)width;
    return a % (uintptr_t)std::min(16, 4 * width) == 0;
  };
  P.flags = 0;
  if (sc.key_mode == KM_PACKED) {
    bool ok = true;
    for (int k = 0; k < sc.nkeys; ++k) ok = ok && aligned(P.keys[k].data, P.keys[k].offset, P.keys[k].width);
    if (ok) P.flags |= PF_VEC_KEYS;
  }
  if (sc.f32mean && aligned(P.vals[sc.cells[0].col].data, P.vals[sc.cells[0].col].offset, 4)) P.flags |= PF_VEC_VAL0;
  if (sc.f64mean && aligned(P.vals[sc.cells[0].col].data, P.vals[sc.cells[0].col].offset, 8)) P.flags |= PF_VEC_VAL0;
  if (sc.f64mean) P.flags |= PF_F64MEAN;
  P.nfilters = (int)gb.filters.size();
  bool fast = true;
  for (int f = 0; f < P.nfilters; ++f) {
    P.filters[f] = gb.filters[(size_t)f];
    P.filter_offsets[f] = gb.filter_offsets[(size_t)f];
    fast = fast && (P.filter_offsets[f] % 4 == 0);
  }
  for (int k = 0; k < sc.nkeys; ++k)
    fast = fast && (P.keys[k].width == 4 || P.keys[k].width == 8) && (!P.keys[k].mask || P.keys[k].offset % 4 == 0);
  for (int v = 0; v < sc.nvals; ++v) fast = fast && (!P.vals[v].mask || P.vals[v].offset % 4 == 0);
  if (fast) P.flags |= PF_FAST;
  if (sc.f32mean || sc.f64mean) {
    const DValCol& vc = P.vals[sc.cells[0].col];
    if (!vc.mask || ((uintptr_t)vc.mask % 16 == 0 && vc.offset % 128 == 0)) P.flags |= PF_BULK;
  }
}

// ------------------------------------------------------------------------------ table management
constexpr int64_t DENSE_REGION_SLOTS = 32768;  // >= the largest dense box the shared memory can hold
// whether table_variant 0 (auto) runs the lean kernel with the cp.async.bulk tile ring (variant 5)
// or with register tiles (variant 4)
constexpr bool LEAN_STAGED_BY_DEFAULT = true;
constexpr int64_t LEAN_DIRECT_SMEM = 136 * 1024;  // table of the register-tile variant: 17K slots
// B2_TRACE=1 in the environment prints phase times to stderr (each mark synchronises the stream, so
// the traced call itself is slower)
struct Trace {
  bool on;
  cudaStream_t stream;
  std::chrono::steady_clock::time_point t0;
  explicit Trace(cudaStream_t s) : on(getenv("B2_TRACE") != nullptr), stream(s)
  {
    if (on) { cudaStreamSynchronize(stream); t0 = std::chrono::steady_clock::now(); }
  }
  void mark(const char* what)
  {
    if (!on) return;
    cudaStreamSynchronize(stream);
    const auto t1 = std::chrono::steady_clock::now();
    fprintf(stderr, "[b2]   %-28s %8.3f ms\n", what, std::chrono::duration<double, std::milli>(t1 - t0).count());
    t0 = t1;
  }
};

int grid_for(int64_t items, int block, int per_sm)
{
  const int64_t want = (items + block - 1) / block;
  const int64_t cap = (int64_t)device_info().sms * per_sm;
  return (int)std::max<int64_t>(1, std::min(want, cap));
}

// small tables: one slot per thread so that the chunks cover all SMs; large ones: 8 per thread
void launch_finalize(const DPlan& P, const DOutPlan& O, const u64* table, int64_t cap, int64_t nslots, DCtrl* ctrl,
                     cudaStream_t stream)
{
  const int64_t big = (int64_t)device_info().sms * 8 * FIN_BLOCK * FIN_ITEMS;
  if (nslots >= big) k_finalize<FIN_ITEMS><<<grid_for((nslots + FIN_ITEMS - 1) / FIN_ITEMS, FIN_BLOCK, 8), FIN_BLOCK, 0, stream>>>(P, O, table, cap, ctrl);
  else k_finalize<1><<<grid_for(nslots, FIN_BLOCK, 8), FIN_BLOCK, 0, stream>>>(P, O, table, cap, ctrl);
}

void free_table(b2_groupby_state& st, cudaStream_t stream)
{
  if (st.table) { cudaFreeAsync(st.table, stream); st.table = nullptr; }
  st.cap = 0;
}

void alloc_table(b2_groupby_state& st, int64_t cap, double max_load, cudaStream_t stream, bool dense_region = false,
                 u32 cap_dense = 0, u32 cap_lean = 0)
{
  free_table(st, stream);
  if (cap > 0x7FFFFFF0ll) B2_FAIL(B2_UNSUPPORTED, "hash table would need more than 2^31 slots");
  st.dense_slots = (dense_region && st.sc.key_mode == KM_PACKED) ? DENSE_REGION_SLOTS : 0;
  const size_t bytes = (size_t)(cap + 1 + st.dense_slots) * (size_t)st.plan.stride * 8;
  st.table = (u64*)default_alloc(bytes, stream, nullptr);
  if (!st.table) B2_FAIL(B2_OUT_OF_MEMORY, "out of device memory allocating a " + std::to_string(bytes) + "-byte hash table");
  g_stats.scratch_bytes += (int64_t)bytes;
  st.cap = cap;
  if (!st.ctrl) {
    st.ctrl = (DCtrl*)default_alloc(sizeof(DCtrl), stream, nullptr);
    if (!st.ctrl) B2_FAIL(B2_OUT_OF_MEMORY, "out of device memory");
  }
  DCtrl h{};
  h.claim_limit = (u64)((double)cap * max_load);
  st.host_ctrl = h;
  static_assert(sizeof(DCtrl) / 4 <= 256, "the control block is initialised by one CTA of k_table_init");
  h.dense_slots = (u64)st.dense_slots;
  st.host_ctrl = h;
  // the key box of the fused pass is sampled here too (needs a dense region, packed keys and enough rows)
  if (st.dense_slots == 0 || st.plan.nrows < SAMPLE_ROWS) cap_dense = 0;
  k_table_init<<<grid_for((cap + 1 + st.dense_slots) * st.plan.stride / 2 + 1, TABLE_INIT_BLOCK, 16), TABLE_INIT_BLOCK, 0, stream>>>(
    st.table, cap + 1 + st.dense_slots, st.plan, st.ctrl, h.claim_limit, h.dense_slots, cap_dense, cap_lean);
  CUDA_TRY(cudaGetLastError());
  g_stats.kernel_launches++;
  g_stats.table_capacity = cap;
  st.ctrl_fresh = true;
}

void read_ctrl(b2_groupby_state& st, cudaStream_t stream)
{
  if (st.ctrl_fresh || !st.ctrl) return;
  CUDA_TRY(cudaMemcpyAsync(&st.host_ctrl, st.ctrl, sizeof(DCtrl), cudaMemcpyDeviceToHost, stream));
  CUDA_TRY(cudaStreamSynchronize(stream));
  st.ctrl_fresh = true;
}

int64_t num_groups(const b2_groupby_state& st) { return (int64_t)st.host_ctrl.nclaimed + (st.host_ctrl.special_used ? 1 : 0); }

// the opt-in to more than 48 KB of dynamic shared memory is an attribute of a function on ONE device
template <typename Kernel>
void allow_shared(Kernel kern, size_t smem, size_t (&configured)[64])
{
  int dev = 0;
  CUDA_TRY(cudaGetDevice(&dev));
  if (smem > 48 * 1024 && smem > configured[dev & 63]) {
    CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    configured[dev & 63] = smem;
  }
}

template <int KM, int LAYOUT>
void launch_aggregate(const DPlan& P, u64* tbl, int64_t cap, DCtrl* ctrl, int S, int fill_limit, size_t smem,
                      cudaStream_t stream, u32 cap_dense = 0, u32 region_slots = 0, int lean_first = 0)
{
  auto kern = k_aggregate<KM, LAYOUT>;
  static thread_local size_t configured[64] = {};
  allow_shared(kern, smem, configured);
  const int64_t tile = (int64_t)AGG_BLOCK * AGG_ROWS;
  const int grid = (int)std::max<int64_t>(1, std::min<int64_t>((P.nrows + tile - 1) / tile, device_info().sms));
  kern<<<grid, AGG_BLOCK, smem, stream>>>(P, tbl, cap, ctrl, S, fill_limit, cap_dense, region_slots, lean_first);
  CUDA_TRY(cudaGetLastError());
  g_stats.kernel_launches++;
}

template <int NK, bool K8, bool STAGED, bool KEY_MASKS, bool V8>
void launch_lean(const DPlan& P, u64* tbl, int64_t cap, DCtrl* ctrl, size_t smem, cudaStream_t stream, u32 region_slots)
{
  auto kern = k_aggregate_lean<NK, K8, STAGED, KEY_MASKS, V8>;
  static thread_local size_t configured[64] = {};
  allow_shared(kern, smem, configured);
  kern<<<device_info().sms, 1024, smem, stream>>>(P, tbl, cap, ctrl, region_slots);
  CUDA_TRY(cudaGetLastError());
  g_stats.kernel_launches++;
}

struct EventPair {  // times the fused kernel on the caller's stream; read after the call's sync
  cudaEvent_t a = nullptr, b = nullptr;
  EventPair() { cudaEventCreate(&a); cudaEventCreate(&b); }
  ~EventPair() { if (a) cudaEventDestroy(a); if (b) cudaEventDestroy(b); }
};
EventPair& kernel_events()
{
  // events belong to the device that was current when they were created: one pair per device
  static thread_local std::unique_ptr<EventPair> ev[64];
  int dev = 0;
  cudaGetDevice(&dev);
  if (!ev[dev & 63]) ev[dev & 63] = std::make_unique<EventPair>();
  return *ev[dev & 63];
}

// How the fused pass uses shared memory for one (schema, inputs, options) combination: decided on the
// host before the table is initialised, because the key-box sampler inside k_table_init needs the slot budget.
struct SharedPlan {
  int layout = SL_NONE;
  int S = 0, fill_limit = 0;  // hashed mode
  size_t smem = 0;            // dynamic shared memory of the kernels
  u32 cap_dense = 0;          // slots a dense key box may use (0 = no box)
  u32 cap_lean = 0;           // slots of the lean kernel's table when that is fewer than cap_dense (0 = the same)
  bool lean = false;          // k_aggregate_lean runs in front of k_aggregate
  bool staged = false;        // ... with the cp.async.bulk tile ring
  size_t lean_smem = 0;       // dynamic shared memory of k_aggregate_lean
};

SharedPlan plan_shared(const b2_groupby_state& st, const b2_groupby& gb)
{
  const Schema& sc = st.sc;
  const DPlan& P = st.plan;
  SharedPlan sp;
  if (gb.table_variant == 1 || sc.has_arg) return sp;
  const int budget = gb.shared_table_bytes > 0 ? std::min(gb.shared_table_bytes, device_info().smem_optin - 1024)
                                               : device_info().smem_optin - 1024;
  const int cell_bytes = sc.f32mean ? 8 : 8 * sc.ncells;  // accumulators of one slot
  sp.S = budget / (8 + cell_bytes) - 1;                   // hashed mode: key cell + accumulators
  if (sp.S < 256) { sp.S = 0; return sp; }
  sp.layout = sc.f32mean ? SL_F32MEAN : SL_GENERIC;
  sp.fill_limit = (int)(sp.S * SMEM_FILL);
  sp.smem = (size_t)budget;
  if (sc.key_mode != KM_PACKED || gb.table_variant == 3) return sp;
  // dense mode: accumulators + one occupancy bit per slot
  sp.cap_dense = (u32)std::min<int64_t>(DENSE_REGION_SLOTS, ((int64_t)budget - 64) * 8 / ((int64_t)cell_bytes * 8 + 1));
  // the lean kernel: Σ and n of one FLOAT32 / FLOAT64 column, 1..3 key columns of 4 or 8 bytes, aligned vector loads
  const int need = PF_FAST | PF_VEC_KEYS | PF_VEC_VAL0;
  if ((sc.f32mean || sc.f64mean) && sc.nkeys <= 3 && (P.flags & need) == need && P.nrows >= SAMPLE_ROWS && P.nrows < 0xFFFF0000ll) {
    sp.lean = true;
    // bits of one slot: fp32 sum + count + occupancy bit, or the limbs of a FLOAT64 sum + count + occupancy bit
    const int64_t slot_bits = sc.f64mean ? (4 * FX_LIMBS + 4) * 8 + 1 : 65;
    const u32 cap_generic = sp.cap_dense;
    // Register tiles arrive through L1, which is what the shared-memory carve-out leaves of the SM's
    // 256 KB: with the whole opt-in taken, ~24 KB of L1 cannot hold the lines of the loads in flight
    // (32 warps x 3 vector loads x 2 tiles) and the row loop slows down by a third.  So this variant
    // takes a table of at most LEAN_DIRECT_SMEM and leaves the rest to L1; wider key boxes go to the
    // generic kernel.
    sp.lean_smem = (size_t)std::min<int64_t>(budget, gb.shared_table_bytes > 0 ? budget : LEAN_DIRECT_SMEM);
    sp.cap_dense = (u32)std::min<int64_t>(DENSE_REGION_SLOTS, ((int64_t)sp.lean_smem - 256) * 8 / slot_bits);
    // the staged variant needs room for its tile ring, flat 16-byte-aligned tiles, and validity that is
    // either absent or the value column's own mask (also when used as the row filter)
    const DValCol& vc = P.vals[sc.cells[0].col];
    bool bulk_ok = (P.flags & PF_BULK) != 0;
    for (int k = 0; k < sc.nkeys; ++k) bulk_ok = bulk_ok && P.keys[k].mask == nullptr;
    bulk_ok = bulk_ok && (P.nfilters == 0 || (P.nfilters == 1 && P.filters[0] == vc.mask && P.filter_offsets[0] == vc.offset));
    int64_t row_bytes = sc.f64mean ? 8 : 4;
    for (int k = 0; k < sc.nkeys; ++k) row_bytes += sc.key_width[k];
    const int64_t ring = (int64_t)LEAN_STAGES * ((int64_t)LEAN_STAGED_CONSUMERS * LEAN_ROWS * row_bytes + LEAN_MASK_BYTES);
    const int64_t staged_cap = ((int64_t)budget - ring - 512) * 8 / slot_bits;
    const bool want_staged = gb.table_variant == 5 || (gb.table_variant == 0 && LEAN_STAGED_BY_DEFAULT);
    if (want_staged && bulk_ok && staged_cap >= 1024) {
      sp.staged = true;
      sp.lean_smem = (size_t)budget;  // bulk copies land in shared memory directly: L1 is not in their way
      sp.cap_dense = (u32)std::min<int64_t>(DENSE_REGION_SLOTS, staged_cap);
    }
    // FLOAT64: the generic kernel's 16-byte slots hold a wider key box than the limbs do; such a box is left
    // to it (the lean kernel declines).  FLOAT32: both tables have 8-byte slots, the lean capacity serves both.
    if (sc.f64mean && cap_generic > sp.cap_dense) { sp.cap_lean = sp.cap_dense; sp.cap_dense = cap_generic; }
  }
  return sp;
}

// One pass of the fused kernel over the bound inputs into st.table.  With `try_lean` the lean kernel
// runs alone and the function returns true: it declines on the device when the sampled key box did not
// fit, which the caller sees in the control block it reads anyway (dense.enabled == 0) and answers
// with a second call without `try_lean`.
bool run_aggregate(b2_groupby_state& st, const b2_groupby& gb, cudaStream_t stream, const SharedPlan& sp, bool try_lean)
{
  const Schema& sc = st.sc;
  g_stats.used_shared_table = sp.layout != SL_NONE;
  const DPlan& P = st.plan;
  const u32 cap_dense = st.dense_slots > 0 && P.nrows >= SAMPLE_ROWS ? sp.cap_dense : 0;
  EventPair& ev = kernel_events();
  cudaEventRecord(ev.a, stream);
  const bool lean = try_lean && sp.lean && cap_dense > 0;
  if (lean) {
    bool k8 = false;  // any 8-byte key column?
    for (int k = 0; k < sc.nkeys; ++k) k8 = k8 || sc.key_width[k] == 8;
    bool key_masks = false;
    for (int k = 0; k < sc.nkeys; ++k) key_masks = key_masks || P.keys[k].mask != nullptr;
    // (the staged variant is only planned when no key column carries a mask)
#define B2_LEAN_V(N, W, V)                                                                                         \
    do {                                                                                                           \
      if (sp.staged) launch_lean<N, W, true, false, V>(P, st.table, st.cap, st.ctrl, sp.lean_smem, stream, (u32)st.dense_slots);  \
      else if (key_masks) launch_lean<N, W, false, true, V>(P, st.table, st.cap, st.ctrl, sp.lean_smem, stream, (u32)st.dense_slots); \
      else launch_lean<N, W, false, false, V>(P, st.table, st.cap, st.ctrl, sp.lean_smem, stream, (u32)st.dense_slots);    \
    } while (0)
#define B2_LEAN(N, W) do { if (sc.f64mean) B2_LEAN_V(N, W, true); else B2_LEAN_V(N, W, false); } while (0)
    switch (sc.nkeys) {
      case 1: if (k8) B2_LEAN(1, true); else B2_LEAN(1, false); break;
      case 2: if (k8) B2_LEAN(2, true); else B2_LEAN(2, false); break;
      default: if (k8) B2_LEAN(3, true); else B2_LEAN(3, false); break;
    }
#undef B2_LEAN
#undef B2_LEAN_V
    cudaEventRecord(ev.b, stream);
    st.ctrl_fresh = false;
    return true;
  }
  if (sc.key_mode == KM_PACKED) {
    if (sp.layout == SL_F32MEAN) launch_aggregate<KM_PACKED, SL_F32MEAN>(P, st.table, st.cap, st.ctrl, sp.S, sp.fill_limit, sp.smem, stream, cap_dense, (u32)st.dense_slots, 0);
    else if (sp.layout == SL_GENERIC) launch_aggregate<KM_PACKED, SL_GENERIC>(P, st.table, st.cap, st.ctrl, sp.S, sp.fill_limit, sp.smem, stream, cap_dense, (u32)st.dense_slots);
    else launch_aggregate<KM_PACKED, SL_NONE>(P, st.table, st.cap, st.ctrl, 0, 0, 0, stream);
  } else {
    if (sp.layout == SL_GENERIC) launch_aggregate<KM_ROWS, SL_GENERIC>(P, st.table, st.cap, st.ctrl, sp.S, sp.fill_limit, sp.smem, stream);
    else launch_aggregate<KM_ROWS, SL_NONE>(P, st.table, st.cap, st.ctrl, 0, 0, 0, stream);
  }
  cudaEventRecord(ev.b, stream);
  st.ctrl_fresh = false;
  return false;
}

int64_t hll_estimate(const u32* regs);

// distinct keys among the participating rows, from a HyperLogLog pass (k_hll); synchronises the stream
int64_t estimate_groups(const b2_groupby_state& st, cudaStream_t stream)
{
  Scratch regs(HLL_REGS * sizeof(u32), stream);
  CUDA_TRY(cudaMemsetAsync(regs.p, 0, regs.bytes, stream));
  const int grid = (int)std::max<int64_t>(1, std::min<int64_t>((st.plan.nrows + 4095) / 4096, (int64_t)device_info().sms * 2));
  k_hll<<<grid, 1024, 0, stream>>>(st.plan, (u32*)regs.p);
  CUDA_TRY(cudaGetLastError());
  g_stats.kernel_launches++;
  std::vector<u32> h(HLL_REGS);
  CUDA_TRY(cudaMemcpyAsync(h.data(), regs.p, regs.bytes, cudaMemcpyDeviceToHost, stream));
  CUDA_TRY(cudaStreamSynchronize(stream));
  return hll_estimate(h.data());
}

int64_t hll_estimate(const u32* regs)
{
  const double m = (double)HLL_REGS;
  double sum = 0.0;
  int zeros = 0;
  for (int i = 0; i < HLL_REGS; ++i) { sum += std::ldexp(1.0, -(int)regs[i]); zeros += regs[i] == 0; }
  const double alpha = 0.7213 / (1.0 + 1.079 / m);
  double e = alpha * m * m / sum;
  if (e <= 2.5 * m && zeros > 0) e = m * std::log(m / (double)zeros);  // small-range correction
  return (int64_t)e;
}

// out[0..n] = exclusive scan of in[0..n-1] (out[n] = the total), three launches
void device_exclusive_scan(const i64* in, int64_t n, i64* out, cudaStream_t stream)
{
  const int64_t per = (int64_t)SCAN_BLOCK * SCAN_ITEMS;
  const int nblocks = (int)std::max<int64_t>(1, (n + per - 1) / per);
  Scratch totals((size_t)(nblocks + 1) * sizeof(i64), stream), bases((size_t)(nblocks + 1) * sizeof(i64), stream);
  k_scan_block_totals<<<nblocks, SCAN_BLOCK, 0, stream>>>(in, n, (i64*)totals.p);
  k_exclusive_scan<<<1, 1024, 0, stream>>>((const i64*)totals.p, (i64*)bases.p, nblocks);
  k_scan_apply<<<nblocks, SCAN_BLOCK, 0, stream>>>(in, n, (const i64*)bases.p, out);
  CUDA_TRY(cudaGetLastError());
  g_stats.kernel_launches += 3;
}

// ------------------------------------------------------------------------------ partitioned path
// Below this many groups the global table (a few tens of MB) lives in L2 and the fused pass wins.
constexpr int64_t RP_MIN_GROUPS = 1 << 19;
constexpr int64_t RP_MIN_ROWS   = 1 << 22;

// Aggregates the bound inputs by radix partition + per-bucket shared-memory tables (b2_partition.cuh).
// `hint` > 0: the expected number of groups (no HyperLogLog registers are kept).  Returns false, leaving
// the state empty, when this path does not apply or gave up (too few groups, a bucket overflowed its
// table, the group list overflowed): the caller then uses the global table, sized from *estimate.
bool aggregate_partitioned(b2_groupby_state& st, const b2_groupby& gb, cudaStream_t stream, int64_t hint, int64_t* estimate)
{
  const Schema& sc = st.sc;
  const DPlan& P = st.plan;
  const bool forced = gb.table_variant == 6;
  if (sc.key_mode != KM_PACKED || sc.ncells < 1 || sc.has_arg) return false;
  Trace trace(stream);
  const int sms = device_info().sms;
  EventPair& ev = kernel_events();
  cudaEventRecord(ev.a, stream);

  // 1. rows per top-level digit, and the number of groups
  constexpr int TOP = 1 << RP_BITS_TOP;
  Scratch counters((size_t)TOP * 8 + (size_t)HLL_REGS * 4, stream);
  CUDA_TRY(cudaMemsetAsync(counters.p, 0, counters.bytes, stream));
  u64* d_hist = (u64*)counters.p;
  u32* d_hll  = (u32*)(d_hist + TOP);
  const int cgrid = (int)std::max<int64_t>(1, std::min<int64_t>((P.nrows + 4 * RP_BLOCK - 1) / (4 * RP_BLOCK), (int64_t)sms * 2));
  // skewed inputs: the hottest keys of a Σx / n / Σx² aggregate are folded by the counting pass itself
  const bool with_hot = sc.fixed && gb.table_variant != 2;
  Scratch hot_mem;
  DHot hot{};
  if (with_hot) {
    const size_t b_ckeys = (size_t)HOT_COUNT_SLOTS * 8, b_ccnt = (size_t)HOT_COUNT_SLOTS * 4, b_keys = (size_t)HOT_SLOTS * 8,
                 b_ids = (size_t)HOT_SLOTS * 2, b_info = 16 + 256 * 4, b_acc = (size_t)HOT_MAX * HOT_ACC_WORDS * 8;
    const size_t b_mask = ((size_t)(P.nrows + 31) / 32 + 2) * 4;  // (written for every quad before it is read)
    hot_mem = Scratch(b_ckeys + b_keys + b_ccnt + b_ids + b_info + b_acc + b_mask, stream);
    unsigned char* m = (unsigned char*)hot_mem.p;
    u64* ckeys = (u64*)m;
    hot.keys = (u64*)(m + b_ckeys);
    u32* ccnt = (u32*)(m + b_ckeys + b_keys);
    hot.ids = (unsigned short*)(m + b_ckeys + b_keys + b_ccnt);
    hot.info = (u32*)(m + b_ckeys + b_keys + b_ccnt + b_ids);
    hot.acc = (u64*)(m + b_ckeys + b_keys + b_ccnt + b_ids + b_info);
    hot.row_mask = (u32*)(m + b_ckeys + b_keys + b_ccnt + b_ids + b_info + b_acc);
    CUDA_TRY(cudaMemsetAsync(m, 0xFF, b_ckeys + b_keys, stream));
    CUDA_TRY(cudaMemsetAsync(ccnt, 0, b_ccnt + b_ids + b_info + b_acc, stream));
    k_hot_sample<<<sms, 256, 0, stream>>>(P, ckeys, ccnt, hot.info);
    k_hot_hist<<<sms, 256, 0, stream>>>(ccnt, hot.info + 4);
    k_hot_select<<<sms, 256, 0, stream>>>(ckeys, ccnt, hot.info + 4, hot);
    CUDA_TRY(cudaGetLastError());
    g_stats.kernel_launches += 3;
    static thread_local size_t configured[2][64] = {};
    allow_shared(k_rp_count<false, true>, rp_count_hot_smem(), configured[0]);
    allow_shared(k_rp_count<true, true>, rp_count_hot_smem(), configured[1]);
    if (hint > 0) k_rp_count<false, true><<<std::min(cgrid, sms), RP_BLOCK, rp_count_hot_smem(), stream>>>(P, d_hist, d_hll, hot);
    else k_rp_count<true, true><<<std::min(cgrid, sms), RP_BLOCK, rp_count_hot_smem(), stream>>>(P, d_hist, d_hll, hot);
  } else if (hint > 0) {
    k_rp_count<false, false><<<cgrid, RP_BLOCK, 0, stream>>>(P, d_hist, d_hll, hot);
  } else {
    k_rp_count<true, false><<<cgrid, RP_BLOCK, 0, stream>>>(P, d_hist, d_hll, hot);
  }
  CUDA_TRY(cudaGetLastError());
  g_stats.kernel_launches++;
  std::vector<u64> h_hist(TOP);
  std::vector<u32> h_hll(HLL_REGS);
  CUDA_TRY(cudaMemcpyAsync(h_hist.data(), d_hist, (size_t)TOP * 8, cudaMemcpyDeviceToHost, stream));
  if (hint <= 0) CUDA_TRY(cudaMemcpyAsync(h_hll.data(), d_hll, (size_t)HLL_REGS * 4, cudaMemcpyDeviceToHost, stream));
  u32 h_hot[2] = {0, 0};  // number of hot keys, exponent info
  if (with_hot) CUDA_TRY(cudaMemcpyAsync(h_hot, hot.info, sizeof(h_hot), cudaMemcpyDeviceToHost, stream));
  CUDA_TRY(cudaStreamSynchronize(stream));
  const int nhot = (int)std::min<u32>(h_hot[0], (u32)HOT_MAX);
  int64_t active = 0;  // rows that go through the partitions (the rows of hot keys are folded already)
  for (u64 c : h_hist) active += (int64_t)c;
  int64_t est = hint > 0 ? hint : hll_estimate(h_hll.data());
  est = std::max<int64_t>(1, std::min(est, active));
  if (estimate) *estimate = est;
  trace.mark("partition: histogram + estimate");
  if (active == 0 && nhot == 0) return false;
  if (!forced && est < RP_MIN_GROUPS) return false;
  // Heavy skew (one key holding several per cent of the rows) would put that key's rows into one bucket
  // and serialise them on one shared-memory slot: the fused pass with its hot-key cache serves such inputs.
  {
    u64 top = 0;
    for (u64 c : h_hist) top = std::max(top, c);
    if (!forced && (double)top > 8.0 * (double)active / TOP + 4096.0) return false;
  }

  // 2. digits: buckets of about half a shared-memory table each (two CTAs of the aggregate kernel per SM)
  const int slot_bytes = (with_hot ? RPA_FIXED_SLOT_BYTES : 8 * (1 + sc.ncells)) + RPA_INDEX_BYTES;
  int budget = std::min((device_info().smem_optin - 2048), 110 * 1024);
  if (gb.shared_table_bytes > 0) budget = std::min(budget, std::max(gb.shared_table_bytes, 257 * slot_bytes));
  int slots = 256;
  while ((int64_t)(2 * slots + 1) * slot_bytes <= budget) slots *= 2;
  if ((int64_t)(slots + 1) * slot_bytes > budget) return false;  // too many accumulators for a useful table
  int T = 0;
  while (((double)est * 1.05) / (double)(1ll << T) > 0.5 * slots) ++T;
  T = std::max(T, 1);
  if (T > 2 * RP_MAX_BITS) return false;
  int b1 = T <= RP_MAX_BITS ? T : (T + 1) / 2, b2 = T - b1;
  const int F1 = 1 << b1, F2 = 1 << b2;
  const int64_t nbuckets = (int64_t)F1 * F2;

  try {
    // 3. level 1
    int words = 1 + sc.nvals, valid_word = -1;
    for (int v = 0; v < sc.nvals; ++v) if (P.vals[v].mask) valid_word = 1 + sc.nvals;
    if (valid_word >= 0) ++words;
    std::vector<u64> h_start((size_t)F1 + 1);
    {
      u64 run = 0;
      const int fold = TOP / F1;
      for (int d = 0; d < F1; ++d) {
        h_start[(size_t)d] = run;
        for (int j = 0; j < fold; ++j) run += h_hist[(size_t)d * fold + j];
      }
      h_start[(size_t)F1] = run;
    }
    Scratch bounds1((size_t)(2 * F1 + 2) * 8, stream);  // [F1 + 1] starts, [F1] cursors
    u64* d_start1 = (u64*)bounds1.p;
    u64* d_cur1   = d_start1 + F1 + 1;
    CUDA_TRY(cudaMemcpyAsync(d_start1, h_start.data(), (size_t)(F1 + 1) * 8, cudaMemcpyHostToDevice, stream));
    CUDA_TRY(cudaMemcpyAsync(d_cur1, h_start.data(), (size_t)F1 * 8, cudaMemcpyHostToDevice, stream));
    Scratch recA((size_t)words * (size_t)std::max<int64_t>(active, 1) * 8, stream);
    DScatter D1{DRecords{(u64*)recA.p, active, words, valid_word}, d_cur1, 64 - b1, F1};
    const int sgrid = (int)std::max<int64_t>(1, std::min<int64_t>((P.nrows + RP_TILE - 1) / RP_TILE, (int64_t)sms * 2));
    {
      static thread_local size_t configured[64] = {};
      allow_shared(k_rp_scatter, rp_tile_smem(F1), configured);
    }
    k_rp_scatter<<<sgrid, RPS_BLOCK, rp_tile_smem(F1), stream>>>(P, D1, nhot > 0 ? hot.row_mask : nullptr);
    CUDA_TRY(cudaGetLastError());
    g_stats.kernel_launches++;
    trace.mark("partition: level-1 scatter");

    // 4. level 2
    Scratch recB, bounds2, tiles;
    DRecords src{(u64*)recA.p, active, words, valid_word};
    const u64* b_start = d_start1;
    const u64* b_end   = d_cur1;
    if (b2 > 0) {
      tiles = Scratch((size_t)(F1 + 1) * 4, stream);
      k_rp_tiles<<<1, 1024, 0, stream>>>(d_start1, d_cur1, F1, (u32*)tiles.p);
      bounds2 = Scratch((size_t)(3 * nbuckets + 2) * 8, stream);  // [nb] counts, [nb + 1] starts, [nb] cursors
      u64* d_hist2  = (u64*)bounds2.p;
      u64* d_start2 = d_hist2 + nbuckets;
      u64* d_cur2   = d_start2 + nbuckets + 1;
      CUDA_TRY(cudaMemsetAsync(d_hist2, 0, (size_t)nbuckets * 8, stream));
      DLevel2 L{src, d_start1, d_cur1, (const u32*)tiles.p, F1};
      const int shift2 = 64 - b1 - b2;
      const int64_t max_tiles = active / RP_TILE + F1;
      const int g2 = (int)std::max<int64_t>(1, std::min<int64_t>(max_tiles, (int64_t)sms * 2));
      k_rp_count2<<<g2, RP_BLOCK, 0, stream>>>(L, shift2, F2, d_hist2);
      CUDA_TRY(cudaGetLastError());
      device_exclusive_scan((const i64*)d_hist2, nbuckets, (i64*)d_start2, stream);
      CUDA_TRY(cudaMemcpyAsync(d_cur2, d_start2, (size_t)nbuckets * 8, cudaMemcpyDeviceToDevice, stream));
      recB = Scratch((size_t)words * (size_t)std::max<int64_t>(active, 1) * 8, stream);
      DScatter D2{DRecords{(u64*)recB.p, active, words, valid_word}, d_cur2, shift2, F2};
      {
        static thread_local size_t configured[64] = {};
        allow_shared(k_rp_scatter2, rp_tile_smem(F2), configured);
      }
      k_rp_scatter2<<<(int)std::max<int64_t>(1, std::min<int64_t>(max_tiles, (int64_t)sms * 2)), RPS_BLOCK, rp_tile_smem(F2), stream>>>(L, D2);
      CUDA_TRY(cudaGetLastError());
      g_stats.kernel_launches += 3;
      src.rec = (u64*)recB.p;
      b_start = d_start2;
      b_end   = d_cur2;
      trace.mark("partition: level-2 count + scatter");
    }

    // 5. one shared-memory aggregate per bucket
    const int64_t gcap = std::min<int64_t>(active, (int64_t)((double)est * (hint > 0 ? 1.25 : 1.08)) + 65536) + HOT_MAX;
    Scratch groups((size_t)(1 + sc.ncells) * (size_t)gcap * 8, stream);
    if (!st.ctrl) {
      st.ctrl = (DCtrl*)default_alloc(sizeof(DCtrl), stream, nullptr);
      if (!st.ctrl) B2_FAIL(B2_OUT_OF_MEMORY, "out of device memory");
    }
    CUDA_TRY(cudaMemsetAsync(st.ctrl, 0, sizeof(DCtrl), stream));
    Scratch work(8, stream);
    CUDA_TRY(cudaMemsetAsync(work.p, 0, 8, stream));
    DBuckets B{src, b_start, b_end, nbuckets, slots, (u64*)groups.p, gcap, (u64*)work.p};
    const size_t smem = (size_t)(slots + 1) * slot_bytes;
    static thread_local size_t configured[2][64] = {};
    const int agrid = (int)std::min<int64_t>(nbuckets, (int64_t)sms * 2);
    if (with_hot) {
      allow_shared(k_rp_aggregate<true>, smem, configured[1]);
      k_rp_aggregate<true><<<agrid, RPA_BLOCK, smem, stream>>>(P, B, st.ctrl, hot.info + 1);
    } else {
      allow_shared(k_rp_aggregate<false>, smem, configured[0]);
      k_rp_aggregate<false><<<agrid, RPA_BLOCK, smem, stream>>>(P, B, st.ctrl, nullptr);
    }
    CUDA_TRY(cudaGetLastError());
    g_stats.kernel_launches++;
    if (nhot > 0) {
      k_rp_append_hot<<<HOT_SLOTS / 256, 256, 0, stream>>>(P, hot, (u64*)groups.p, gcap, st.ctrl);
      CUDA_TRY(cudaGetLastError());
      g_stats.kernel_launches++;
    }
    cudaEventRecord(ev.b, stream);
    st.ctrl_fresh = false;
    read_ctrl(st, stream);
    trace.mark("partition: bucket aggregate");
    {
      float ms = 0.f;
      if (cudaEventElapsedTime(&ms, ev.a, ev.b) == cudaSuccess) g_stats.aggregate_kernel_ms += ms;
      else cudaGetLastError();
    }
    if (getenv("B2_TRACE"))
      fprintf(stderr, "[b2] partitioned: %lld rows through the partitions, %d hot keys, estimate %lld groups, digits %d + %d, %d slots per bucket, %lld groups, overflow %d\n",
              (long long)active, nhot, (long long)est, b1, b2, slots, (long long)st.host_ctrl.out_cursor, (int)st.host_ctrl.overflow);
    if (st.host_ctrl.overflow) return false;
    st.groups = std::move(groups);
    st.groups_cap = gcap;
    st.groups_n = (int64_t)st.host_ctrl.out_cursor;
    g_stats.table_capacity = nbuckets * slots;
    return true;
  } catch (const Err& e) {
    if (e.code != B2_OUT_OF_MEMORY) throw;
    return false;  // not enough memory for the record buffers: the table path needs less
  }
}

constexpr int64_t SPECULATIVE_CAP = 1 << 17;  // first table when nothing is known about the cardinality
constexpr double MAX_LOAD = 0.70;

// aggregates the bound inputs into an EMPTY state, growing the table until it fits
constexpr int64_t DEFER_MAX_GROUPS = 1 << 20;  // over-allocation a deferred first attempt may cost per result column

void add_kernel_ms()
{
  float ms = 0.f;
  if (cudaEventElapsedTime(&ms, kernel_events().a, kernel_events().b) == cudaSuccess) g_stats.aggregate_kernel_ms += ms;
  else cudaGetLastError();
}

// `defer`: the first table attempt may return with its control block unread (st.deferred; see the state);
// `resume`: continue such an attempt after finalize_state read the control block and found it wanting.
void aggregate_fresh(b2_groupby_state& st, const b2_groupby& gb, cudaStream_t stream, bool may_partition = false,
                     bool defer = false, bool resume = false)
{
  const int64_t n = st.plan.nrows;
  const int64_t hint = st.expected_groups > 0 ? st.expected_groups : gb.expected_groups;
  const int64_t full = std::max<int64_t>(1024, (int64_t)((double)n / 0.6) + 64);  // groups <= rows
  // the partitioned path serves one-shot aggregates over packed keys with very many groups
  may_partition = may_partition && st.sc.key_mode == KM_PACKED && gb.table_variant != 1 && gb.table_variant != 7 &&
                  (gb.table_variant == 6 || n >= RP_MIN_ROWS);
  int64_t known = 0;  // groups estimated by a partitioned attempt that gave up
  if (!resume && may_partition && (gb.table_variant == 6 || hint >= RP_MIN_GROUPS)) {
    g_stats.table_attempts = 1;
    if (aggregate_partitioned(st, gb, stream, hint, &known)) return;
    may_partition = false;
  }
  int64_t cap;
  if (hint > 0) cap = std::min(full, std::max<int64_t>(1024, (int64_t)((double)hint / 0.5) + 64));
  else if (known > 0) cap = std::min(full, (int64_t)((double)known * 1.10 / 0.6) + 1024);
  else if (n <= SPECULATIVE_CAP / 2) cap = std::max<int64_t>(1024, 2 * n + 64);
  else cap = SPECULATIVE_CAP;
  defer = defer && !resume && st.sc.key_mode == KM_PACKED && !st.sc.has_arg && !getenv("B2_TRACE");
  for (int attempt = 1;; ++attempt) {
    g_stats.table_attempts = attempt;
    Trace trace(stream);
    const SharedPlan sp = plan_shared(st, gb);
    bool lean_ran;
    if (resume && attempt == 1) {
      cap = st.deferred_cap;
      lean_ran = st.deferred_lean;
    } else {
      alloc_table(st, cap, cap >= full ? 1.0 : MAX_LOAD, stream, gb.table_variant != 1 && gb.table_variant != 3, sp.cap_dense,
                  sp.cap_lean);
      trace.mark("table allocation + init");
      lean_ran = run_aggregate(st, gb, stream, sp, true);
      const int64_t bound = std::min<int64_t>(n, (int64_t)st.host_ctrl.claim_limit + 1 + st.dense_slots);
      if (defer && attempt == 1 && bound <= DEFER_MAX_GROUPS) {
        st.deferred = true;
        st.deferred_lean = lean_ran;
        st.deferred_cap = cap;
        st.deferred_bound = bound;
        return;
      }
    }
    read_ctrl(st, stream);
    if (st.host_ctrl.error) B2_FAIL(B2_INTERNAL_ERROR, "a bounded wait inside the fused aggregate kernel ran out");
    if (lean_ran && !st.host_ctrl.dense.enabled) {
      // the key box did not fit the lean kernel's table: it did nothing; the generic kernel takes the input
      float ms = 0.f;
      if (cudaEventElapsedTime(&ms, kernel_events().a, kernel_events().b) == cudaSuccess) g_stats.aggregate_kernel_ms += ms;
      else cudaGetLastError();
      if (st.host_ctrl.dense.total != 0) {
        // ... but it fits the generic kernel's (the sampler kept it, switched off): switch it on
        static const int one = 1;
        CUDA_TRY(cudaMemcpyAsync(&st.ctrl->dense.enabled, &one, sizeof(int), cudaMemcpyHostToDevice, stream));
      }
      run_aggregate(st, gb, stream, sp, false);
      read_ctrl(st, stream);
    }
    {
      float ms = 0.f;
      if (cudaEventElapsedTime(&ms, kernel_events().a, kernel_events().b) == cudaSuccess) g_stats.aggregate_kernel_ms += ms;
      else cudaGetLastError();
      if (getenv("B2_TRACE") && st.host_ctrl.t_phase[4] > st.host_ctrl.t_phase[0]) {
        const u64* t = st.host_ctrl.t_phase;
        fprintf(stderr, "[b2]   CTA 0: sample %.1f us, shared init %.1f us, row loop %.1f us, merge %.1f us\n",
                (t[1] > t[0] ? t[1] - t[0] : 0) * 1e-3, ((t[1] > t[0] ? t[2] - t[1] : t[2] - t[0])) * 1e-3, (t[3] - t[2]) * 1e-3,
                (t[4] - t[3]) * 1e-3);
      }
      if (getenv("B2_TRACE")) fprintf(stderr, "[b2] attempt %d cap %lld kernel %.3f ms overflow %d claimed %llu, rows folded in shared memory %llu, in the global table %llu\n", attempt, (long long)cap, ms, (int)st.host_ctrl.overflow, (unsigned long long)st.host_ctrl.nclaimed, (unsigned long long)st.host_ctrl.stat_smem_rows, (unsigned long long)st.host_ctrl.stat_gmem_rows);
    }
    if (!st.host_ctrl.overflow) break;
    if (cap >= full) B2_FAIL(B2_INTERNAL_ERROR, "hash table overflow at full capacity");
    if (attempt == 1) {
      // the speculative table was too small: count the distinct keys (HyperLogLog, one pass over the
      // key columns) and size the table for them — or, with very many groups, leave the table for the
      // partitioned path (its first pass keeps the HyperLogLog registers too)
      int64_t est = 0;
      if (may_partition) {
        free_table(st, stream);
        if (aggregate_partitioned(st, gb, stream, 0, &est)) return;
        may_partition = false;
      }
      if (est <= 0) est = estimate_groups(st, stream);
      trace.mark("HyperLogLog estimate");
      cap = std::min(full, std::max<int64_t>(cap * 16, (int64_t)((double)est * 1.10 / 0.6) + 1024));
    } else {
      cap = (cap * 4 < full) ? cap * 4 : full;  // the estimate fell short (it is within a few percent: rare)
    }
  }
}

// all groups of a table as packed records, destination-major by owner; counts on the host
void pack_table(b2_groupby_state& st, int nparts, cudaStream_t stream, Scratch& out, std::vector<int64_t>& counts)
{
  if (st.sc.has_arg)
    B2_FAIL(B2_UNSUPPORTED, "ARGMIN / ARGMAX and MIN / MAX of strings hold row indices of one batch: no partial records");
  if (st.sc.key_mode != KM_PACKED)
    B2_FAIL(B2_UNSUPPORTED, "partial records of string / float / wide keys are not transferable; partition the rows instead");
  counts.assign((size_t)nparts, 0);
  if (st.groups_n >= 0) {
    // a finished group list (the partitioned path): counts, then the records, with the same kernel
    const int64_t G = st.groups_n;
    Scratch dcounts((size_t)nparts * 2 * sizeof(u64), stream);
    CUDA_TRY(cudaMemsetAsync(dcounts.p, 0, dcounts.bytes, stream));
    u64* d_counts = (u64*)dcounts.p;
    u64* d_cursor = d_counts + nparts;
    const int grid = grid_for(std::max<int64_t>(G, 1), 256, 8);
    const size_t smem = (size_t)nparts * 2 * sizeof(u64);
    if (smem > 48 * 1024) CUDA_TRY(cudaFuncSetAttribute(k_pack_list, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    k_pack_list<<<grid, 256, smem, stream>>>((const u64*)st.groups.p, st.groups_cap, G, st.plan.stride, nparts, d_counts, nullptr);
    CUDA_TRY(cudaGetLastError());
    std::vector<u64> h((size_t)nparts);
    CUDA_TRY(cudaMemcpyAsync(h.data(), d_counts, (size_t)nparts * sizeof(u64), cudaMemcpyDeviceToHost, stream));
    CUDA_TRY(cudaStreamSynchronize(stream));
    std::vector<u64> starts((size_t)nparts);
    u64 run = 0;
    for (int p = 0; p < nparts; ++p) { starts[(size_t)p] = run; run += h[(size_t)p]; counts[(size_t)p] = (int64_t)h[(size_t)p]; }
    if ((int64_t)run != G) B2_FAIL(B2_INTERNAL_ERROR, "pack: group count mismatch");
    CUDA_TRY(cudaMemcpyAsync(d_cursor, starts.data(), (size_t)nparts * sizeof(u64), cudaMemcpyHostToDevice, stream));
    out = Scratch(std::max<size_t>(8, (size_t)G * st.plan.stride * 8), stream);
    k_pack_list<<<grid, 256, smem, stream>>>((const u64*)st.groups.p, st.groups_cap, G, st.plan.stride, nparts, d_cursor, (u64*)out.p);
    CUDA_TRY(cudaGetLastError());
    CUDA_TRY(cudaStreamSynchronize(stream));  // `starts` is read by the copy above
    g_stats.kernel_launches += 2;
    return;
  }
  if (!st.table) { out = Scratch(8, stream); return; }
  read_ctrl(st, stream);
  const int64_t G = num_groups(st);
  Scratch dcounts((size_t)nparts * 2 * sizeof(u64), stream);
  CUDA_TRY(cudaMemsetAsync(dcounts.p, 0, dcounts.bytes, stream));
  u64* d_counts = (u64*)dcounts.p;
  u64* d_cursor = d_counts + nparts;
  const int grid = grid_for(st.cap + 1 + st.dense_slots, 256, 8);
  k_pack_count<<<grid, 256, (size_t)nparts * sizeof(u64), stream>>>(st.table, st.cap, st.plan.stride, nparts, st.ctrl, d_counts);
  CUDA_TRY(cudaGetLastError());
  std::vector<u64> h((size_t)nparts);
  CUDA_TRY(cudaMemcpyAsync(h.data(), d_counts, (size_t)nparts * sizeof(u64), cudaMemcpyDeviceToHost, stream));
  CUDA_TRY(cudaStreamSynchronize(stream));
  std::vector<u64> starts((size_t)nparts);
  u64 run = 0;
  for (int p = 0; p < nparts; ++p) { starts[(size_t)p] = run; run += h[(size_t)p]; counts[(size_t)p] = (int64_t)h[(size_t)p]; }
  if ((int64_t)run != G) B2_FAIL(B2_INTERNAL_ERROR, "pack: group count mismatch");
  CUDA_TRY(cudaMemcpyAsync(d_cursor, starts.data(), (size_t)nparts * sizeof(u64), cudaMemcpyHostToDevice, stream));
  out = Scratch(std::max<size_t>(8, (size_t)G * st.plan.stride * 8), stream);
  const size_t scatter_smem = (size_t)nparts * 2 * sizeof(u64);
  if (scatter_smem > 48 * 1024)  // up to 4096 destinations x 16 bytes: beyond the default limit
    CUDA_TRY(cudaFuncSetAttribute(k_pack_scatter, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)scatter_smem));
  k_pack_scatter<<<grid, 256, scatter_smem, stream>>>(st.table, st.cap, st.plan.stride, nparts, st.ctrl, d_cursor,
                                                                          (u64*)out.p);
  CUDA_TRY(cudaGetLastError());
  CUDA_TRY(cudaStreamSynchronize(stream));  // `starts` is read by the copy above
  g_stats.kernel_launches += 2;
}

void merge_records(b2_groupby_state& st, const u64* recs, int64_t nrecs, cudaStream_t stream)
{
  if (st.sc.has_arg)
    B2_FAIL(B2_UNSUPPORTED, "ARGMIN / ARGMAX and MIN / MAX of strings hold row indices of one batch: no partial records");
  if (st.sc.key_mode != KM_PACKED)
    B2_FAIL(B2_UNSUPPORTED, "partial records of string / float / wide keys are not transferable; partition the rows instead");
  if (nrecs <= 0) return;
  read_ctrl(st, stream);
  const int64_t G = st.table ? num_groups(st) : 0;
  const int64_t need = std::max<int64_t>(1024, (int64_t)((double)(G + nrecs) / 0.6) + 64);
  auto run_merge = [&] {
    k_merge<<<grid_for(nrecs, 256, 8), 256, 0, stream>>>(st.plan, st.table, st.cap, st.ctrl, recs, nrecs);
    CUDA_TRY(cudaGetLastError());
    g_stats.kernel_launches++;
    st.ctrl_fresh = false;
    read_ctrl(st, stream);
  };
  if (!st.table) {
    // An empty state with an estimate of the distinct keys among the records (records of the same key
    // from several senders): a table sized for the estimate stays in L2 and is cheaper to finalise
    // than one sized for one group per record.  The records are still all here, so an estimate that
    // turns out too small only costs a second pass into the full-size table.
    const int64_t hinted = st.expected_groups > 0 ? (int64_t)((double)st.expected_groups / 0.5) + 64 : 0;
    if (hinted > 0 && hinted < need) {
      alloc_table(st, std::max<int64_t>(1024, hinted), 0.85, stream);
      run_merge();
      if (!st.host_ctrl.overflow) return;
    }
    alloc_table(st, std::max<int64_t>(need, hinted), 1.0, stream);
  } else if (st.cap < need) {
    // grow: move the present groups into a larger table
    Scratch old;
    std::vector<int64_t> cnt;
    pack_table(st, 1, stream, old, cnt);
    alloc_table(st, need * 2, 1.0, stream);
    if (cnt[0] > 0) {
      k_merge<<<grid_for(cnt[0], 256, 8), 256, 0, stream>>>(st.plan, st.table, st.cap, st.ctrl, (const u64*)old.p, cnt[0]);
      CUDA_TRY(cudaGetLastError());
      g_stats.kernel_launches++;
    }
  } else {
    // the existing table stays; its claim limit must allow the new records
    DCtrl h = st.host_ctrl;
    h.claim_limit = (u64)st.cap;
    CUDA_TRY(cudaMemcpyAsync(&st.ctrl->claim_limit, &h.claim_limit, sizeof(u64), cudaMemcpyHostToDevice, stream));
    CUDA_TRY(cudaStreamSynchronize(stream));
  }
  run_merge();
  if (st.host_ctrl.overflow) B2_FAIL(B2_INTERNAL_ERROR, "hash table overflow while merging partial records");
}

// ------------------------------------------------------------------------------ outputs
struct OwnedGuard {  // frees partially built results on failure
  b2_groupby_result* r;
  bool armed = true;
  ~OwnedGuard() { if (armed && r) b2_result_free(r); }
};

void* out_alloc(const b2_allocator& al, size_t bytes, cudaStream_t stream)
{
  void* p = al.allocate(bytes ? bytes : 8, stream, al.ctx);
  if (!p) B2_FAIL(B2_OUT_OF_MEMORY, "the allocator returned null for " + std::to_string(bytes) + " bytes");
  return p;
}

void init_owned(b2_owned_column& c, int type_id, int64_t n, bool nullable, const b2_allocator& al, cudaStream_t stream)
{
  std::memset(&c, 0, sizeof(c));
  c.type_id = type_id;
  c.size = (int32_t)n;
  const int w = type_id == B2_DECIMAL128 ? 16 : width_of(type_id);
  if (w > 0) {
    // results narrower than 4 bytes are padded to whole words like the reference's
    // (cpp/src/groupby/hash/output_utils.cu:71-82)
    c.data_bytes = ((size_t)n * w + 3) / 4 * 4;
    c.data = out_alloc(al, c.data_bytes, stream);
  }
  if (nullable) {
    c.null_mask_bytes = (size_t)((n + 511) / 512) * 64;  // 64-byte padded, cpp/include/cudf/null_mask.hpp:52-57
    if (c.null_mask_bytes == 0) c.null_mask_bytes = 64;
    c.null_mask = (uint32_t*)out_alloc(al, c.null_mask_bytes, stream);
    CUDA_TRY(cudaMemsetAsync(c.null_mask, 0xFF, c.null_mask_bytes, stream));
  }
}

// STRING column of the strings at rows `rows` (-1 = none) of `kc`: lengths -> offsets by scan -> bytes.
// `c` has its type, size and (optional) null mask set; chars and the offsets child are allocated here.
// Synchronises the stream once (the total size decides between INT32 and INT64 offsets).
void gather_strings(const DKeyCol& kc, const int* rows, int64_t G, b2_owned_column& c, u32* null_counter,
                    const b2_allocator& al, cudaStream_t stream)
{
  Scratch lens((size_t)(G + 1) * sizeof(i64), stream), offs((size_t)(G + 1) * sizeof(i64), stream);
  k_string_lengths<<<grid_for(G, 256, 8), 256, 0, stream>>>(kc, rows, G, (i64*)lens.p, c.null_mask, null_counter);
  CUDA_TRY(cudaGetLastError());
  device_exclusive_scan((const i64*)lens.p, G, (i64*)offs.p, stream);
  i64 total = 0;
  CUDA_TRY(cudaMemcpyAsync(&total, (i64*)offs.p + G, sizeof(i64), cudaMemcpyDeviceToHost, stream));
  CUDA_TRY(cudaStreamSynchronize(stream));
  // INT64 offsets once the chars pass the reference's large-strings threshold (cpp/src/strings/utilities.cu:150-157)
  const bool big = total > 0x7FFFFFFFll;
  c.data_bytes = (size_t)std::max<i64>(total, 1);
  c.data = out_alloc(al, c.data_bytes, stream);
  c.num_children = 1;
  c.children = (b2_owned_column*)std::calloc(1, sizeof(b2_owned_column));
  b2_owned_column& oc = c.children[0];
  oc.type_id = big ? B2_INT64 : B2_INT32;
  oc.size = (int32_t)(G + 1);
  oc.data_bytes = (size_t)(G + 1) * (big ? 8 : 4);
  oc.data = out_alloc(al, oc.data_bytes, stream);
  if (big) k_string_copy<i64><<<grid_for(G * 4, 256, 8), 256, 0, stream>>>(kc, rows, G, (const i64*)offs.p, (i64*)oc.data, (unsigned char*)c.data);
  else k_string_copy<int><<<grid_for(G * 4, 256, 8), 256, 0, stream>>>(kc, rows, G, (const i64*)offs.p, (int*)oc.data, (unsigned char*)c.data);
  CUDA_TRY(cudaGetLastError());
  g_stats.kernel_launches += 5;
}

// a STRING column without rows: one zero offset
void empty_strings(b2_owned_column& c, const b2_allocator& al, cudaStream_t stream)
{
  c.num_children = 1;
  c.children = (b2_owned_column*)std::calloc(1, sizeof(b2_owned_column));
  c.children[0].type_id = B2_INT32;
  c.children[0].size = 1;
  c.children[0].data_bytes = 4;
  c.children[0].data = out_alloc(al, 4, stream);
  CUDA_TRY(cudaMemsetAsync(c.children[0].data, 0, 4, stream));
}

// `resume` (one-shot calls): continues the aggregate when a deferred first attempt turns out to have failed.
void finalize_state(b2_groupby_state& st, cudaStream_t stream, const b2_allocator* allocator, b2_groupby_result* out,
                    const std::function<void()>* resume = nullptr)
{
  const Schema& sc = st.sc;
  const b2_allocator al = resolve(allocator);
  std::memset(out, 0, sizeof(*out));
  out->allocator = al;
  out->stream = stream;
  OwnedGuard guard{out};

  Trace trace(stream);
  // A deferred first attempt: nothing has been read back yet.  The columns are allocated for the most groups
  // that attempt can hold, k_finalize is enqueued behind the fused kernel, and one synchronisation tells
  // whether the attempt stood (then the columns are cut to the group count) or has to be continued.
  const bool speculative = st.deferred && st.table != nullptr && st.groups_n < 0;
  if (!speculative) read_ctrl(st, stream);
  const bool listed = st.groups_n >= 0;  // the partitioned path left a compact group list, not a table
  if (!speculative) {
    if (st.table && st.host_ctrl.chunk_overflow >= 2) B2_FAIL(B2_INTERNAL_ERROR, "the local aggregate failed on another rank");
    if (st.table && st.host_ctrl.chunk_overflow) B2_FAIL(B2_LOGIC_ERROR, "partial-record chunk overflow");
    if (st.table && st.host_ctrl.overflow) B2_FAIL(B2_INTERNAL_ERROR, "hash table overflow while merging partial records");
  }
  // (speculative: G is the number of rows the columns are allocated for until the control block is read)
  int64_t G = speculative ? st.deferred_bound : listed ? st.groups_n : st.table ? num_groups(st) : 0;
  if (G > 0x7FFFFFFFll) B2_FAIL(B2_UNSUPPORTED, "more than 2^31-1 groups");
  out->num_groups = (int32_t)G;
  out->num_keys = sc.nkeys;
  out->keys = (b2_owned_column*)std::calloc((size_t)std::max(1, sc.nkeys), sizeof(b2_owned_column));
  const int nreqs = (int)sc.req_nouts.size();
  out->num_requests = nreqs;
  out->num_results = (int32_t*)std::calloc((size_t)std::max(1, nreqs), sizeof(int32_t));
  out->results = (b2_owned_column**)std::calloc((size_t)std::max(1, nreqs), sizeof(b2_owned_column*));
  for (int r = 0; r < nreqs; ++r) {
    out->num_results[r] = sc.req_nouts[(size_t)r];
    out->results[r] = (b2_owned_column*)std::calloc((size_t)std::max(1, sc.req_nouts[(size_t)r]), sizeof(b2_owned_column));
  }

  // result columns
  auto plan = std::make_unique<DOutPlan>();
  std::memset(plan.get(), 0, sizeof(DOutPlan));
  plan->nouts = (int)sc.outs.size();
  plan->max_groups = speculative ? G : 0;
  std::vector<Scratch> arg_rows(sc.outs.size());  // MIN / MAX of strings: the winning row of every group
  for (size_t i = 0; i < sc.outs.size(); ++i) {
    const OutSpec& o = sc.outs[i];
    b2_owned_column& c = out->results[o.req][o.agg];
    if (o.kind == OK_STRARG) {
      std::memset(&c, 0, sizeof(c));
      c.type_id = B2_STRING;
      c.size = (int32_t)G;
      if (o.nullable) {
        c.null_mask_bytes = (size_t)std::max<int64_t>(1, (G + 511) / 512) * 64;
        c.null_mask = (uint32_t*)out_alloc(al, c.null_mask_bytes, stream);
        CUDA_TRY(cudaMemsetAsync(c.null_mask, 0xFF, c.null_mask_bytes, stream));
      }
      arg_rows[i] = Scratch(std::max<size_t>(8, (size_t)G * sizeof(int)), stream);
    } else if (o.kind == OK_SUMOVF) {
      // a STRUCT column: no data of its own, the struct-level mask, children {sum, overflow} without masks
      // (cpp/tests/groupby/sum_overflow_tests.cpp:200-211)
      init_owned(c, B2_STRUCT, G, o.nullable, al, stream);
      c.num_children = 2;
      c.children = (b2_owned_column*)std::calloc(2, sizeof(b2_owned_column));
      init_owned(c.children[0], o.ctype, G, false, al, stream);
      c.children[0].scale = o.scale;
      init_owned(c.children[1], B2_BOOL8, G, false, al, stream);
    } else {
      init_owned(c, o.rtype, G, o.nullable, al, stream);
    }
    c.scale = o.kind == OK_SUMOVF ? 0 : o.scale;
    DOutCol& d = plan->outs[i];
    d.data = o.kind == OK_STRARG ? arg_rows[i].p : o.kind == OK_SUMOVF ? c.children[0].data : c.data;
    d.data2 = o.kind == OK_SUMOVF ? c.children[1].data : nullptr;
    d.mask = c.null_mask; d.kind = o.kind; d.rclass = vclass_of(o.kind == OK_SUMOVF ? o.ctype : o.rtype);
    d.c_a = o.c_a; d.c_b = o.c_b; d.c_cnt = o.c_cnt; d.ddof = o.ddof; d.src_float = o.src_float;
    d.null_slot = (int)i;
  }
  // key columns
  Scratch rep_rows;
  for (int k = 0; k < sc.nkeys; ++k) {
    b2_owned_column& c = out->keys[k];
    const bool nullable = sc.include_nulls && sc.key_nullable[k];
    if (sc.key_types[k] == B2_STRING) {
      std::memset(&c, 0, sizeof(c));
      c.type_id = B2_STRING;
      c.size = (int32_t)G;
      if (nullable) {
        c.null_mask_bytes = (size_t)std::max<int64_t>(1, (G + 511) / 512) * 64;
        c.null_mask = (uint32_t*)out_alloc(al, c.null_mask_bytes, stream);
        CUDA_TRY(cudaMemsetAsync(c.null_mask, 0xFF, c.null_mask_bytes, stream));
      }
    } else {
      init_owned(c, sc.key_types[k], G, nullable, al, stream);
      c.scale = sc.key_scale[k];
    }
    plan->kdata[k] = c.data;
    plan->kmask[k] = c.null_mask;
  }
  // the null counters live in the control block (a state without a table or group list has no groups)
  static_assert(sizeof(DCtrl::null_counts) == (MAX_OUTS + MAX_KEYS) * sizeof(u32), "null counters of the control block");
  if (G > 0) {
    if (!st.ctrl) B2_FAIL(B2_INTERNAL_ERROR, "groups without a control block");
    CUDA_TRY(cudaMemsetAsync(st.ctrl->null_counts, 0, sizeof(DCtrl::null_counts), stream));
    plan->null_counts = st.ctrl->null_counts;
  }
  if (sc.key_mode == KM_ROWS) {
    rep_rows = Scratch(std::max<size_t>(8, (size_t)G * sizeof(int)), stream);
    plan->rep_rows = (int*)rep_rows.p;
  }

  std::vector<u32> h_nulls(MAX_OUTS + MAX_KEYS, 0);
  trace.mark("finalize: output allocation");
  if (G > 0) {
    if (listed) {
      k_finalize_records<<<grid_for(G, 256, 16), 256, 0, stream>>>(st.plan, *plan, (const u64*)st.groups.p, st.groups_cap, G);
    } else {
      CUDA_TRY(cudaMemsetAsync(&st.ctrl->out_cursor, 0, sizeof(u64), stream));
      launch_finalize(st.plan, *plan, st.table, st.cap, st.cap + 1 + st.dense_slots, st.ctrl, stream);
    }
    CUDA_TRY(cudaGetLastError());
    g_stats.kernel_launches++;
    trace.mark("finalize: k_finalize");

    if (speculative) {
      CUDA_TRY(cudaMemcpyAsync(&st.host_ctrl, st.ctrl, sizeof(DCtrl), cudaMemcpyDeviceToHost, stream));
      CUDA_TRY(cudaStreamSynchronize(stream));
      st.ctrl_fresh = true;
      st.deferred = false;
      const DCtrl& h = st.host_ctrl;
      const bool stood = !h.overflow && !h.error && !h.chunk_overflow && !(st.deferred_lean && !h.dense.enabled);
      if (stood) add_kernel_ms();  // (a continued attempt adds its kernel times itself)
      if (!stood || num_groups(st) > G) {
        b2_result_free(out);  // (the guard then finds nothing left to free)
        guard.armed = false;
        if (!stood) {
          if (!resume) B2_FAIL(B2_INTERNAL_ERROR, "a deferred table attempt failed and cannot be continued");
          (*resume)();
        }
        finalize_state(st, stream, allocator, out);
        return;
      }
      G = num_groups(st);
      out->num_groups = (int32_t)G;
      for (int k = 0; k < sc.nkeys; ++k) { out->keys[k].size = (int32_t)G; out->keys[k].null_count = (int32_t)h.null_counts[MAX_OUTS + k]; }
      for (size_t i = 0; i < sc.outs.size(); ++i) {
        b2_owned_column& c = out->results[sc.outs[i].req][sc.outs[i].agg];
        c.size = (int32_t)G;
        c.null_count = (int32_t)h.null_counts[i];
        for (int ch = 0; ch < c.num_children && sc.outs[i].kind == OK_SUMOVF; ++ch) c.children[ch].size = (int32_t)G;
      }
      guard.armed = false;
      return;
    }

    if (sc.key_mode == KM_ROWS) {
      if ((int)st.row_keys.size() != sc.nkeys) B2_FAIL(B2_INTERNAL_ERROR, "row-keyed state without bound key views");
      for (int k = 0; k < sc.nkeys; ++k) {
        b2_owned_column& c = out->keys[k];
        const DKeyCol& kc = st.plan.keys[k];
        if (sc.key_types[k] != B2_STRING) {
          DGather gth{kc.data, kc.mask, kc.offset, kc.width, (unsigned char*)c.data, c.null_mask,
                      plan->null_counts + MAX_OUTS + k};
          k_gather_fixed<<<grid_for(G, 256, 8), 256, 0, stream>>>(gth, plan->rep_rows, G);
          CUDA_TRY(cudaGetLastError());
          g_stats.kernel_launches++;
          continue;
        }
        gather_strings(kc, plan->rep_rows, G, c, plan->null_counts + MAX_OUTS + k, al, stream);
        trace.mark("finalize: key strings");
      }
    }
    // MIN / MAX of strings: gather the winning rows' strings (cpp/src/groupby/hash/hash_compound_agg_finalizer.cu:39-76)
    for (size_t i = 0; i < sc.outs.size(); ++i) {
      const OutSpec& o = sc.outs[i];
      if (o.kind != OK_STRARG) continue;
      const DValCol& vc = st.plan.vals[sc.req_val[(size_t)o.req]];
      DKeyCol kc{};
      kc.data = vc.data; kc.mask = nullptr; kc.offsets = vc.offsets; kc.offset = vc.offset; kc.vclass = VC_STRING; kc.offs64 = vc.offs64;
      gather_strings(kc, (const int*)arg_rows[i].p, G, out->results[o.req][o.agg], plan->null_counts + i, al, stream);
    }
    CUDA_TRY(cudaMemcpyAsync(h_nulls.data(), st.ctrl->null_counts, sizeof(DCtrl::null_counts), cudaMemcpyDeviceToHost, stream));
    CUDA_TRY(cudaStreamSynchronize(stream));
    trace.mark("finalize: key gather + nulls");
  } else {
    // empty result: STRING columns still carry a one-entry offsets child
    for (int k = 0; k < sc.nkeys; ++k)
      if (sc.key_types[k] == B2_STRING) empty_strings(out->keys[k], al, stream);
    for (const OutSpec& o : sc.outs)
      if (o.kind == OK_STRARG) empty_strings(out->results[o.req][o.agg], al, stream);
    CUDA_TRY(cudaStreamSynchronize(stream));
  }
  for (size_t i = 0; i < sc.outs.size(); ++i) out->results[sc.outs[i].req][sc.outs[i].agg].null_count = (int32_t)h_nulls[i];
  for (int k = 0; k < sc.nkeys; ++k) out->keys[k].null_count = (int32_t)h_nulls[(size_t)MAX_OUTS + k];
  guard.armed = false;
}

b2_groupby_state* make_state(const b2_groupby& gb, const b2_aggregation_request* reqs, int nreqs)
{
  validate_requests(gb, reqs, nreqs);
  auto st = std::make_unique<b2_groupby_state>();
  st->sc = make_schema(gb, reqs, nreqs);
  fill_plan_schema(st->plan, st->sc);
  st->expected_groups = gb.expected_groups;
  return st.release();
}

void update_state(b2_groupby_state& st, const b2_groupby& gb, const b2_aggregation_request* reqs, int nreqs,
                  cudaStream_t stream, bool may_partition = false, bool defer = false)
{
  validate_requests(gb, reqs, nreqs);
  if ((int)st.sc.req_val.size() != nreqs) B2_FAIL(B2_LOGIC_ERROR, "request list differs from the state's");
  st.last_stream = stream;
  if (gb.keys[0].v.size == 0) return;
  if (st.groups_n >= 0) B2_FAIL(B2_INTERNAL_ERROR, "a finished group list takes no further updates");
  if (!st.table) {
    bind_plan_inputs(st.plan, st.sc, gb, reqs, nreqs);
    aggregate_fresh(st, gb, stream, may_partition, defer);
    if (st.sc.key_mode == KM_ROWS) { st.has_rows = true; st.row_keys = gb.keys; }
    return;
  }
  if (st.sc.key_mode != KM_PACKED)
    B2_FAIL(B2_UNSUPPORTED, "a state keyed on string / float / wide keys takes one update only");
  if (st.sc.has_arg)
    B2_FAIL(B2_UNSUPPORTED, "a state with ARGMIN / ARGMAX or MIN / MAX of strings takes one update only");
  // batch-local table, then merge (a failed pass must not leave half a batch in the state)
  b2_groupby_state tmp;
  tmp.sc = st.sc;
  tmp.plan = st.plan;
  bind_plan_inputs(tmp.plan, tmp.sc, gb, reqs, nreqs);
  try {
    aggregate_fresh(tmp, gb, stream);
    Scratch recs;
    std::vector<int64_t> cnt;
    pack_table(tmp, 1, stream, recs, cnt);
    merge_records(st, (const u64*)recs.p, cnt[0], stream);
  } catch (...) {
    free_table(tmp, stream);
    if (tmp.ctrl) cudaFreeAsync(tmp.ctrl, stream);
    throw;
  }
  free_table(tmp, stream);
  if (tmp.ctrl) cudaFreeAsync(tmp.ctrl, stream);
}

// ------------------------------------------------------------------------------ string keys through a dictionary
// One-shot aggregates of many rows keyed on STRING columns (plus fixed-width ones): every string column is
// first replaced by the id of its string in a dictionary (k_dict_encode), so that the keys
// pack into one 64-bit cell and the packed-key paths (fused shared-memory tables, the partitioned path)
// serve the call; the finished id column of the result is turned back into strings by gathering the
// representative rows.  Worth it while a column's distinct strings are few enough for its dictionary (and
// the representatives' bytes) to stay cached: the table is tried at 2^22 slots, then once larger, then the
// call goes the row-key way as before.  The groups and every result are the same either way.
constexpr int64_t DICT_MIN_ROWS   = 1 << 21;
constexpr int64_t DICT_FIRST_CAP  = 1 << 22;
constexpr int64_t DICT_SECOND_CAP = 1 << 26;
constexpr double DICT_MAX_LOAD    = 0.7;

struct EncodedKeys {
  bool active = false;
  b2_groupby gb;                  // the caller's groupby with id columns in place of the string columns
  std::vector<int> cols;          // key indices that were strings
  std::vector<Scratch> tables;    // per such column: the dictionary (cells, pool of string prefixes, first rows)
  std::vector<const int*> first_rows;  // ... and where its first rows start
  std::vector<Scratch> ids;       // per such column: UINT32 ids, element offset as the string column's
};

bool encode_string_keys(const b2_groupby& gb, cudaStream_t stream, EncodedKeys& ek)
{
  if (gb.table_variant != 0 && gb.table_variant != 8) return false;
  const int64_t n = gb.keys[0].v.size;
  if (n == 0 || (gb.table_variant == 0 && n < DICT_MIN_ROWS)) return false;
  int bits = 0, nstr = 0;
  for (const ColView& k : gb.keys) {
    const b2_column_view& c = k.v;
    if (c.type_id == B2_STRING) {
      if (c.num_children < 1 || !c.children) return false;
      bits += 32; ++nstr;
    } else {
      const int w = width_of(c.type_id);
      if (w == 0 || is_float_t(c.type_id)) return false;
      bits += 8 * w;
    }
    if (gb.null_policy == B2_NULL_INCLUDE && c.null_mask) ++bits;
  }
  if (nstr == 0 || bits > 64) return false;

  Trace trace(stream);
  Scratch ctrl(sizeof(DCtrl), stream);
  ek.gb = gb;
  for (size_t k = 0; k < gb.keys.size(); ++k) {
    const b2_column_view& c = gb.keys[k].v;
    if (c.type_id != B2_STRING) continue;
    auto plan = std::make_unique<DPlan>();
    std::memset(plan.get(), 0, sizeof(DPlan));
    plan->nrows = n; plan->nkeys = 1; plan->key_mode = KM_ROWS; plan->stride = 1;
    DKeyCol& kc = plan->keys[0];
    kc.data = (const unsigned char*)c.data; kc.mask = c.null_mask; kc.offset = c.offset; kc.vclass = VC_STRING; kc.nullbit = -1;
    const b2_column_view& o = c.children[0];
    kc.offsets = (const unsigned char*)o.data + (size_t)o.offset * (o.type_id == B2_INT64 ? 8 : 4);
    kc.offs64 = o.type_id == B2_INT64;

    Scratch ids((size_t)(c.offset + n) * sizeof(u32), stream);
    Scratch table;
    const int* first_rows = nullptr;
    int64_t cap = 1024;
    while (cap < std::min<int64_t>(DICT_FIRST_CAP, std::max<int64_t>(n / 8, 1024))) cap *= 2;
    bool done = false;
    for (int attempt = 0; attempt < 2 && !done; ++attempt) {
      if (attempt == 1) {
        int64_t cap2 = cap;
        while (cap2 < std::min<int64_t>(DICT_SECOND_CAP, 2 * n)) cap2 *= 2;
        if (cap2 == cap) break;
        cap = cap2;
      }
      // cells, then the pool of string prefixes (one entry per id; ids lost to races for a cell stay unused,
      // so the pool holds as many entries as the table has cells), then the first rows
      const int64_t pool_cap = std::min<int64_t>(cap, (int64_t)DICT_ID_MASK - 1);
      table = Scratch((size_t)cap * 8 + (size_t)pool_cap * 32 + (size_t)pool_cap * 4, stream);
      CUDA_TRY(cudaMemsetAsync(table.p, 0xFF, (size_t)cap * sizeof(u64), stream));
      DDict D{(u64*)table.p, cap, (u64*)table.p + cap, (int*)((u64*)table.p + cap + pool_cap * 4), pool_cap};
      DCtrl h{};
      h.claim_limit = (u64)((double)cap * DICT_MAX_LOAD);
      CUDA_TRY(cudaMemcpyAsync(ctrl.p, &h, sizeof(DCtrl), cudaMemcpyHostToDevice, stream));
      const int grid = grid_for((n + DICT_ROWS - 1) / DICT_ROWS, DICT_BLOCK, 8);
      k_dict_encode<<<grid, DICT_BLOCK, 0, stream>>>(*plan, D, (DCtrl*)ctrl.p, (u32*)ids.p);
      first_rows = D.first_row;
      CUDA_TRY(cudaGetLastError());
      g_stats.kernel_launches++;
      CUDA_TRY(cudaMemcpyAsync(&h, ctrl.p, sizeof(DCtrl), cudaMemcpyDeviceToHost, stream));
      CUDA_TRY(cudaStreamSynchronize(stream));
      done = h.overflow == 0;
    }
    if (!done) return false;
    trace.mark("string key -> dictionary ids");

    ColView& dst = ek.gb.keys[k];
    b2_column_view v{};
    v.type_id = B2_UINT32; v.size = c.size; v.data = ids.p; v.null_mask = c.null_mask; v.null_count = c.null_count; v.offset = c.offset;
    dst = ColView(v);
    ek.cols.push_back((int)k);
    ek.tables.push_back(std::move(table));
    ek.first_rows.push_back(first_rows);
    ek.ids.push_back(std::move(ids));
  }
  ek.gb.table_variant = 0;
  ek.active = true;
  return true;
}

// The id key columns of a finished result become the STRING columns the caller asked for.
void restore_string_keys(const EncodedKeys& ek, const b2_groupby& gb, cudaStream_t stream, b2_groupby_result* out)
{
  const b2_allocator al = resolve(&out->allocator);
  const int64_t G = out->num_groups;
  OwnedGuard guard{out};
  for (size_t i = 0; i < ek.cols.size(); ++i) {
    const int k = ek.cols[i];
    b2_owned_column idc = out->keys[k];  // UINT32 ids (+ the null mask of the key under INCLUDE)
    b2_owned_column& c = out->keys[k];
    std::memset(&c, 0, sizeof(c));
    c.type_id = B2_STRING;
    c.size = (int32_t)G;
    c.null_mask = idc.null_mask; c.null_mask_bytes = idc.null_mask_bytes; c.null_count = idc.null_count;
    idc.null_mask = nullptr;
    struct IdFree {
      b2_owned_column& c; const b2_allocator& al; cudaStream_t s;
      ~IdFree() { if (c.data) al.deallocate(c.data, c.data_bytes, s, al.ctx); }
    } id_free{idc, al, stream};
    if (G == 0) { empty_strings(c, al, stream); continue; }
    const b2_column_view& src = gb.keys[(size_t)k].v;
    DKeyCol kc{};
    kc.data = (const unsigned char*)src.data; kc.mask = nullptr; kc.offset = src.offset; kc.vclass = VC_STRING; kc.nullbit = -1;
    const b2_column_view& o = src.children[0];
    kc.offsets = (const unsigned char*)o.data + (size_t)o.offset * (o.type_id == B2_INT64 ? 8 : 4);
    kc.offs64 = o.type_id == B2_INT64;
    Scratch rows((size_t)G * sizeof(int), stream);
    k_dict_rows<<<grid_for(G, 256, 8), 256, 0, stream>>>((const u32*)idc.data, c.null_mask, ek.first_rows[i], G, (int*)rows.p);
    CUDA_TRY(cudaGetLastError());
    g_stats.kernel_launches++;
    // the mask travels as it is: gather_strings must neither clear bits nor count (rows of null keys are -1)
    u32* mask = c.null_mask;
    c.null_mask = nullptr;
    gather_strings(kc, (const int*)rows.p, G, c, nullptr, al, stream);
    c.null_mask = mask;
  }
  CUDA_TRY(cudaStreamSynchronize(stream));  // the id columns and dictionaries are released behind this call
  guard.armed = false;
}

}  // namespace

// ------------------------------------------------------------------------------ no-allocation variant
// Scratch of b2_groupby_aggregate_noalloc: table + control block + null counters.  Lives in the
// library image on every device that loads it.  In host code this name is only a handle for
// cudaGetSymbolAddress; kernels get the device address looked up below.
static __device__ __align__(256) unsigned char g_noalloc_scratch[B2_NOALLOC_SCRATCH_BYTES];

namespace {
constexpr int MAX_DEVICES = 64;
unsigned char* g_noalloc_addr[MAX_DEVICES] = {};
std::mutex g_noalloc_mutex;

// device address of the scratch array on the current device (looked up once per device)
unsigned char* noalloc_scratch()
{
  int dev = 0;
  CUDA_TRY(cudaGetDevice(&dev));
  if (dev < 0 || dev >= MAX_DEVICES) B2_FAIL(B2_UNSUPPORTED, "device ordinal beyond 63");
  std::lock_guard<std::mutex> lock(g_noalloc_mutex);
  if (!g_noalloc_addr[dev]) {
    void* p = nullptr;
    CUDA_TRY(cudaGetSymbolAddress(&p, g_noalloc_scratch));
    g_noalloc_addr[dev] = (unsigned char*)p;
  }
  return g_noalloc_addr[dev];
}
}  // namespace

extern "C" b2_status b2_groupby_aggregate_noalloc(b2_groupby* gb, const b2_aggregation_request* requests,
                                                  int32_t num_requests, void* stream_, int32_t max_groups,
                                                  void* const* key_data, uint32_t* const* key_masks,
                                                  void* const* result_data, uint32_t* const* result_masks,
                                                  int32_t* num_groups_out, int32_t* null_counts_out)
{
  return guarded([&] {
    cudaStream_t stream = (cudaStream_t)stream_;
    if (!gb || !key_data || !result_data || !num_groups_out || max_groups < 1)
      B2_FAIL(B2_INVALID_ARGUMENT, "null argument or max_groups < 1");
    *num_groups_out = 0;
    g_stats = b2_call_stats{};
    if (gb->keys.empty()) B2_FAIL(B2_LOGIC_ERROR, "groupby needs at least one key column");
    validate_requests(*gb, requests, num_requests);
    Schema sc = make_schema(*gb, requests, num_requests);
    if (sc.key_mode != KM_PACKED)
      B2_FAIL(B2_UNSUPPORTED, "the no-allocation variant serves keys that pack into 64 bits (no string / float / wide keys)");
    for (const OutSpec& o : sc.outs) {
      if (o.kind == OK_STRARG) B2_FAIL(B2_UNSUPPORTED, "the no-allocation variant does not serve MIN / MAX of strings (their size is not known in advance)");
      if (o.kind == OK_SUMOVF) B2_FAIL(B2_UNSUPPORTED, "the no-allocation variant does not serve SUM_OVERFLOW (a struct result)");
      if (o.kind == OK_SUM128) B2_FAIL(B2_UNSUPPORTED, "the no-allocation variant does not serve DECIMAL128 values");
    }
    DPlan P;
    fill_plan_schema(P, sc);
    bind_plan_inputs(P, sc, *gb, requests, num_requests);

    // carve the scratch array: [control block | null counters | table]
    unsigned char* base = noalloc_scratch();
    const size_t ctrl_bytes = (sizeof(DCtrl) + 255) / 256 * 256;
    const size_t nulls_bytes = ((MAX_OUTS + MAX_KEYS) * sizeof(u32) + 255) / 256 * 256;
    const int64_t cap = 2 * (int64_t)max_groups;
    const size_t table_bytes = (size_t)(cap + 1) * P.stride * 8;
    if (ctrl_bytes + nulls_bytes + table_bytes > B2_NOALLOC_SCRATCH_BYTES)
      B2_FAIL(B2_INVALID_ARGUMENT, "max_groups = " + std::to_string(max_groups) + " needs a " + std::to_string(table_bytes) +
                                     "-byte table; the fixed scratch array holds " +
                                     std::to_string(B2_NOALLOC_SCRATCH_BYTES - ctrl_bytes - nulls_bytes) + " bytes (" +
                                     std::to_string((B2_NOALLOC_SCRATCH_BYTES - ctrl_bytes - nulls_bytes) / ((size_t)P.stride * 8) / 2 - 1) +
                                     " groups for this request)");
    DCtrl* ctrl = (DCtrl*)base;
    u32* null_counts = (u32*)(base + ctrl_bytes);
    u64* table = (u64*)(base + ctrl_bytes + nulls_bytes);
    for (int k = 0; k < sc.nkeys; ++k) {
      if (!key_data[k]) B2_FAIL(B2_INVALID_ARGUMENT, "key_data entry is null");
      if (sc.include_nulls && sc.key_nullable[k] && (!key_masks || !key_masks[k]))
        B2_FAIL(B2_INVALID_ARGUMENT, "a nullable key column needs a key_masks entry");
    }
    for (size_t i = 0; i < sc.outs.size(); ++i) {
      if (!result_data[i]) B2_FAIL(B2_INVALID_ARGUMENT, "result_data entry is null");
      if (sc.outs[i].nullable && (!result_masks || !result_masks[i]))
        B2_FAIL(B2_INVALID_ARGUMENT, "a nullable result column needs a result_masks entry");
    }

    // everything the kernels read is written first: the previous call's contents are irrelevant.
    // The control block is reset on the device (claim limit = max_groups: one more claim than that
    // sets the overflow flag), so nothing is copied from the host before the kernels run.
    DCtrl h{};
    CUDA_TRY(cudaMemsetAsync(null_counts, 0, nulls_bytes, stream));
    k_table_init<<<grid_for((cap + 1) * P.stride / 2 + 1, 256, 16), 256, 0, stream>>>(table, cap + 1, P, ctrl, (u64)max_groups);
    CUDA_TRY(cudaGetLastError());
    int64_t G = 0;
    if (P.nrows > 0) {
      launch_aggregate<KM_PACKED, SL_NONE>(P, table, cap, ctrl, 0, 0, 0, stream);
      CUDA_TRY(cudaMemcpyAsync(&h, ctrl, sizeof(DCtrl), cudaMemcpyDeviceToHost, stream));
      CUDA_TRY(cudaStreamSynchronize(stream));
      G = (int64_t)h.nclaimed + (h.special_used ? 1 : 0);
      if (h.overflow || G > max_groups) B2_FAIL(B2_LOGIC_ERROR, "the input holds more than max_groups groups");
    }
    g_stats.kernel_launches += 1;

    auto plan = std::make_unique<DOutPlan>();
    std::memset(plan.get(), 0, sizeof(DOutPlan));
    plan->nouts = (int)sc.outs.size();
    const size_t mask_bytes = (size_t)((max_groups + 31) / 32) * 4;
    for (size_t i = 0; i < sc.outs.size(); ++i) {
      const OutSpec& o = sc.outs[i];
      DOutCol& d = plan->outs[i];
      d.data = result_data[i];
      d.mask = o.nullable ? result_masks[i] : nullptr;
      d.kind = o.kind; d.rclass = vclass_of(o.rtype);
      d.c_a = o.c_a; d.c_b = o.c_b; d.c_cnt = o.c_cnt; d.ddof = o.ddof; d.src_float = o.src_float;
      d.null_slot = (int)i;
      if (d.mask) CUDA_TRY(cudaMemsetAsync(d.mask, 0xFF, mask_bytes, stream));
    }
    for (int k = 0; k < sc.nkeys; ++k) {
      plan->kdata[k] = key_data[k];
      plan->kmask[k] = (sc.include_nulls && sc.key_nullable[k]) ? key_masks[k] : nullptr;
      if (plan->kmask[k]) CUDA_TRY(cudaMemsetAsync(plan->kmask[k], 0xFF, mask_bytes, stream));
    }
    plan->null_counts = null_counts;
    u32 h_nulls[MAX_OUTS + MAX_KEYS] = {};
    if (G > 0) {
      launch_finalize(P, *plan, table, cap, cap + 1, ctrl, stream);
      CUDA_TRY(cudaGetLastError());
      g_stats.kernel_launches += 1;
      if (null_counts_out) CUDA_TRY(cudaMemcpyAsync(h_nulls, null_counts, sizeof(h_nulls), cudaMemcpyDeviceToHost, stream));
    }
    CUDA_TRY(cudaStreamSynchronize(stream));
    *num_groups_out = (int32_t)G;
    if (null_counts_out) {
      for (int k = 0; k < sc.nkeys; ++k) null_counts_out[k] = (int32_t)h_nulls[MAX_OUTS + k];
      for (size_t i = 0; i < sc.outs.size(); ++i) null_counts_out[sc.nkeys + i] = (int32_t)h_nulls[i];
    }
  });
}

// ================================================================================ C ABI
extern "C" {

b2_status b2_groupby_create(const b2_column_view* keys, int32_t num_keys, int32_t null_policy,
                            const b2_groupby_options* options, b2_groupby** out)
{
  return guarded([&] {
    if (!out) B2_FAIL(B2_INVALID_ARGUMENT, "out is null");
    *out = nullptr;
    if (num_keys < 0 || (num_keys > 0 && !keys)) B2_FAIL(B2_INVALID_ARGUMENT, "keys is null");
    if (null_policy != B2_NULL_EXCLUDE && null_policy != B2_NULL_INCLUDE) B2_FAIL(B2_INVALID_ARGUMENT, "bad null_policy");
    auto gb = std::make_unique<b2_groupby>();
    for (int k = 0; k < num_keys; ++k) {
      if (keys[k].size != keys[0].size) B2_FAIL(B2_LOGIC_ERROR, "key columns differ in size");
      gb->keys.emplace_back(keys[k]);
    }
    gb->null_policy = null_policy;
    if (options) {
      gb->expected_groups = options->expected_groups;
      gb->table_variant = options->table_variant;
      gb->shared_table_bytes = options->shared_table_bytes;
      if (options->num_row_filters > MAX_FILTERS) B2_FAIL(B2_UNSUPPORTED, "more than 8 row filters");
      for (int f = 0; f < options->num_row_filters; ++f) {
        if (!options->row_filter_masks || !options->row_filter_masks[f]) continue;
        gb->filters.push_back(options->row_filter_masks[f]);
        gb->filter_offsets.push_back(options->row_filter_offsets ? options->row_filter_offsets[f] : 0);
      }
    }
    *out = gb.release();
  });
}

void b2_groupby_destroy(b2_groupby* gb) { delete gb; }

// DICTIONARY32 value columns with fixed-width keys, decoded once into plain columns of the keys' type (the
// reference resolves the key at every update and produces results of the keys' type:
// cpp/src/groupby/hash/output_utils.cu:65-66, cpp/tests/groupby/mean_tests.cpp:128-147, max_tests.cpp:226-246).
// A dictionary of strings takes part through its indices: the keys of a dictionary column are sorted and unique
// (cpp/include/cudf/dictionary/dictionary_column_view.hpp:29-38), so MIN / MAX / ARGMIN / ARGMAX of the strings are
// those of the indices; MIN / MAX results are handed back as dictionary columns over a copy of the same keys, like
// the reference's (cpp/tests/groupby/max_tests.cpp:198-224, min_tests.cpp:190-216).  Other aggregations of a
// dictionary of strings are not served.
struct DecodedValues {
  struct Wrap { int req; b2_column_view keys; };
  std::vector<b2_aggregation_request> reqs;
  std::vector<Scratch> bufs;
  std::vector<Wrap> wraps;  // requests whose MIN / MAX results are indices into these keys
};
const b2_aggregation_request* decode_dictionary_values(const b2_aggregation_request* reqs, int nreqs, cudaStream_t stream,
                                                       DecodedValues& dv)
{
  bool any = false;
  for (int r = 0; reqs && r < nreqs; ++r) any = any || reqs[r].values.type_id == B2_DICTIONARY32;
  if (!any) return reqs;
  dv.reqs.assign(reqs, reqs + nreqs);
  struct Seen { const void* idx; const void* keys; const void* mask; int off; void* buf; };
  std::vector<Seen> seen;
  for (int r = 0; r < nreqs; ++r) {
    b2_column_view& v = dv.reqs[(size_t)r].values;
    if (v.type_id != B2_DICTIONARY32) continue;
    // children {indices, keys} (cpp/include/cudf/dictionary/dictionary_column_view.hpp:56-57)
    if (v.num_children != 2 || !v.children) B2_FAIL(B2_INVALID_ARGUMENT, "a DICTIONARY32 column needs its indices and keys children");
    const b2_column_view& ix = v.children[0];
    const b2_column_view& ky = v.children[1];
    const int iw = width_of(ix.type_id), w = width_of(ky.type_id);
    const bool int_index = ix.type_id >= B2_INT8 && ix.type_id <= B2_UINT64;
    if (!int_index || iw == 0) B2_FAIL(B2_INVALID_ARGUMENT, "dictionary indices must be an integer column");
    if (ix.size < v.size || (v.size > 0 && !ix.data) || (ky.size > 0 && !ky.data) || ky.size < 0)
      B2_FAIL(B2_INVALID_ARGUMENT, "dictionary children do not cover the column");
    if (ky.type_id == B2_STRING) {
      bool by_index = ix.offset == 0 && ky.null_mask == nullptr;
      for (int a = 0; a < reqs[r].num_aggregations && reqs[r].aggregations; ++a) {
        const int kind = reqs[r].aggregations[a].kind;
        by_index = by_index && (kind == B2_AGG_MIN || kind == B2_AGG_MAX || kind == B2_AGG_ARGMIN || kind == B2_AGG_ARGMAX ||
                                kind == B2_AGG_COUNT_VALID || kind == B2_AGG_COUNT_ALL);
      }
      if (!by_index) continue;  // validate_requests reports the column as not served
      dv.wraps.push_back(DecodedValues::Wrap{r, ky});
      v.type_id = ix.type_id; v.scale = 0; v.data = ix.data; v.num_children = 0; v.children = nullptr;
      continue;
    }
    if (w == 0 || ky.type_id == B2_DICTIONARY32) continue;  // other keys: validate_requests reports them
    void* buf = nullptr;
    for (const Seen& sn : seen)
      if (sn.idx == ix.data && sn.keys == ky.data && sn.mask == v.null_mask && sn.off == v.offset) buf = sn.buf;
    if (!buf) {
      dv.bufs.emplace_back(std::max<size_t>(8, (size_t)((int64_t)v.offset + v.size) * (size_t)w), stream);
      buf = dv.bufs.back().p;
      seen.push_back(Seen{ix.data, ky.data, v.null_mask, v.offset, buf});
      if (v.size > 0) {
        DDictDecode D{};
        D.indices = (const unsigned char*)ix.data; D.index_width = iw;
        D.index_signed = ix.type_id >= B2_INT8 && ix.type_id <= B2_INT64;
        D.index_offset = (i64)v.offset + ix.offset;
        D.keys = (const unsigned char*)ky.data; D.keys_offset = ky.offset; D.nkeys = ky.size; D.width = w;
        D.mask = v.null_mask; D.mask_offset = v.offset;
        D.dst = (unsigned char*)buf + (size_t)v.offset * (size_t)w;
        k_dict_decode<<<grid_for(v.size, 256, 8), 256, 0, stream>>>(D, (i64)v.size);
        CUDA_TRY(cudaGetLastError());
        g_stats.kernel_launches++;
      }
    }
    // the decoded column keeps the dictionary column's mask and element offset
    v.type_id = ky.type_id; v.scale = ky.scale; v.data = buf; v.num_children = 0; v.children = nullptr;
  }
  return dv.reqs.data();
}

// A finished column of dictionary indices `c` becomes child 0 of a DICTIONARY32 column whose child 1 is a copy of
// the dictionary's keys `ky`; the validity stays on the parent (cpp/include/cudf/dictionary/dictionary_column_view.hpp:56-57).
void make_dictionary_column(b2_owned_column& c, const b2_column_view& ky, const b2_allocator& al, cudaStream_t stream)
{
  b2_owned_column* kids = (b2_owned_column*)std::calloc(2, sizeof(b2_owned_column));
  if (!kids) B2_FAIL(B2_OUT_OF_MEMORY, "out of host memory");
  kids[0] = c;  // the indices: data of the finished column, no mask of their own
  kids[0].null_mask = nullptr; kids[0].null_mask_bytes = 0; kids[0].null_count = 0;
  b2_owned_column parent{};
  parent.type_id = B2_DICTIONARY32; parent.size = c.size; parent.null_count = c.null_count;
  parent.null_mask = c.null_mask; parent.null_mask_bytes = c.null_mask_bytes;
  parent.num_children = 2; parent.children = kids;
  c = parent;  // (from here on b2_result_free releases the children with the rest)
  if (ky.type_id != B2_STRING) {
    const int w = width_of(ky.type_id);
    init_owned(kids[1], ky.type_id, ky.size, false, al, stream);
    kids[1].scale = ky.scale;
    if (ky.size > 0)
      CUDA_TRY(cudaMemcpyAsync(kids[1].data, (const unsigned char*)ky.data + (size_t)ky.offset * (size_t)w, (size_t)ky.size * (size_t)w,
                               cudaMemcpyDeviceToDevice, stream));
    return;
  }
  kids[1].type_id = B2_STRING; kids[1].size = ky.size;
  if (ky.size > 0) {
    if (ky.num_children < 1 || !ky.children) B2_FAIL(B2_INVALID_ARGUMENT, "STRING keys of a dictionary need their offsets child");
    const b2_column_view& o = ky.children[0];
    DKeyCol kc{};
    kc.data = (const unsigned char*)ky.data; kc.mask = nullptr; kc.offset = ky.offset; kc.vclass = VC_STRING; kc.nullbit = -1;
    kc.offsets = (const unsigned char*)o.data + (size_t)o.offset * (o.type_id == B2_INT64 ? 8 : 4);
    kc.offs64 = o.type_id == B2_INT64;
    Scratch rows((size_t)ky.size * sizeof(int), stream);
    k_iota<<<grid_for(ky.size, 256, 8), 256, 0, stream>>>((int*)rows.p, (i64)ky.size);
    CUDA_TRY(cudaGetLastError());
    gather_strings(kc, (const int*)rows.p, ky.size, kids[1], nullptr, al, stream);
  } else {
    empty_strings(kids[1], al, stream);
  }
}

// MIN / MAX results of a dictionary of strings: the winning indices, handed back as dictionary columns
void wrap_dictionary_results(const DecodedValues& dv, const b2_aggregation_request* reqs, b2_groupby_result* out,
                             const b2_allocator* allocator, cudaStream_t stream)
{
  const b2_allocator al = resolve(allocator);
  for (const DecodedValues::Wrap& w : dv.wraps)
    for (int a = 0; a < reqs[w.req].num_aggregations; ++a) {
      const int kind = reqs[w.req].aggregations[a].kind;
      if (kind == B2_AGG_MIN || kind == B2_AGG_MAX) make_dictionary_column(out->results[w.req][a], w.keys, al, stream);
    }
  if (!dv.wraps.empty()) CUDA_TRY(cudaStreamSynchronize(stream));
}

// DICTIONARY32 key columns (cpp/tests/groupby/keys_tests.cpp:324-347): the keys of a dictionary are unique, so rows
// group by their indices; the finished key column is handed back as a dictionary over a copy of the same keys.
struct DictKeys {
  b2_groupby gb;                              // the groupby with the indices in place of the dictionary columns
  std::vector<std::pair<int, ColView>> wraps; // key column, the dictionary's keys child
};
bool substitute_dictionary_keys(const b2_groupby& gb, DictKeys& dk)
{
  bool any = false;
  for (const ColView& c : gb.keys) any = any || c.v.type_id == B2_DICTIONARY32;
  if (!any) return false;
  dk.gb = gb;
  for (size_t k = 0; k < dk.gb.keys.size(); ++k) {
    const b2_column_view v = dk.gb.keys[k].v;
    if (v.type_id != B2_DICTIONARY32) continue;
    if (v.num_children != 2 || !v.children) B2_FAIL(B2_INVALID_ARGUMENT, "a DICTIONARY32 column needs its indices and keys children");
    const b2_column_view ix = v.children[0];
    const b2_column_view& ky = v.children[1];
    const bool int_index = ix.type_id >= B2_INT8 && ix.type_id <= B2_UINT64;
    if (!int_index || ix.offset != 0 || ix.size < v.size || (v.size > 0 && !ix.data))
      B2_FAIL(B2_INVALID_ARGUMENT, "dictionary indices must be an unsliced integer column that covers the dictionary column");
    if (ky.type_id != B2_STRING && width_of(ky.type_id) == 0) B2_FAIL(B2_UNSUPPORTED, "dictionary keys of this type are not served");
    dk.wraps.emplace_back((int)k, ColView(ky));
    b2_column_view nv = v;
    nv.type_id = ix.type_id; nv.scale = 0; nv.data = ix.data; nv.num_children = 0; nv.children = nullptr;
    dk.gb.keys[k] = ColView(nv);
  }
  return true;
}

b2_status b2_groupby_aggregate(b2_groupby* gb, const b2_aggregation_request* requests, int32_t num_requests,
                               void* stream, const b2_allocator* allocator, b2_groupby_result* out)
{
  return guarded([&] {
    if (!gb || !out) B2_FAIL(B2_INVALID_ARGUMENT, "null argument");
    g_stats = b2_call_stats{};
    std::memset(out, 0, sizeof(*out));
    if (gb->keys.empty()) B2_FAIL(B2_LOGIC_ERROR, "groupby needs at least one key column");
    device_info();
    if (num_requests < 0 || (num_requests > 0 && !requests)) B2_FAIL(B2_INVALID_ARGUMENT, "requests is null");
    DecodedValues dv;  // (lives until the results are finished)
    requests = decode_dictionary_values(requests, num_requests, (cudaStream_t)stream, dv);
    validate_requests(*gb, requests, num_requests);
    DictKeys dk;
    const b2_groupby& base = substitute_dictionary_keys(*gb, dk) ? dk.gb : *gb;
    EncodedKeys ek;
    const b2_groupby& use = encode_string_keys(base, (cudaStream_t)stream, ek) ? ek.gb : base;
    std::unique_ptr<b2_groupby_state, void (*)(b2_groupby_state*)> st(make_state(use, requests, num_requests),
                                                                      b2_state_destroy);
    update_state(*st, use, requests, num_requests, (cudaStream_t)stream, /*may_partition=*/true, /*defer=*/true);
    const std::function<void()> resume = [&] { aggregate_fresh(*st, use, (cudaStream_t)stream, true, false, /*resume=*/true); };
    finalize_state(*st, (cudaStream_t)stream, allocator, out, &resume);
    if (ek.active) restore_string_keys(ek, base, (cudaStream_t)stream, out);
    if (!dv.wraps.empty() || !dk.wraps.empty()) {
      OwnedGuard guard{out};  // a failure below frees what was finished
      wrap_dictionary_results(dv, requests, out, allocator, (cudaStream_t)stream);
      const b2_allocator al = resolve(allocator);
      for (auto& w : dk.wraps) make_dictionary_column(out->keys[w.first], w.second.v, al, (cudaStream_t)stream);
      if (!dk.wraps.empty()) CUDA_TRY(cudaStreamSynchronize((cudaStream_t)stream));
      guard.armed = false;
    }
  });
}

void b2_result_free(b2_groupby_result* r)
{
  if (!r) return;
  const b2_allocator al = resolve(&r->allocator);
  auto free_col = [&](b2_owned_column& c, auto&& self) -> void {
    if (c.data) al.deallocate(c.data, c.data_bytes, r->stream, al.ctx);
    if (c.null_mask) al.deallocate(c.null_mask, c.null_mask_bytes, r->stream, al.ctx);
    for (int i = 0; i < c.num_children; ++i) self(c.children[i], self);
    std::free(c.children);
    c = b2_owned_column{};
  };
  if (r->keys) for (int k = 0; k < r->num_keys; ++k) free_col(r->keys[k], free_col);
  std::free(r->keys);
  if (r->results)
    for (int q = 0; q < r->num_requests; ++q) {
      if (!r->results[q]) continue;
      for (int a = 0; a < r->num_results[q]; ++a) free_col(r->results[q][a], free_col);
      std::free(r->results[q]);
    }
  std::free(r->results);
  std::free(r->num_results);
  std::memset(r, 0, sizeof(*r));
}

b2_status b2_state_create(const b2_groupby* gb, const b2_aggregation_request* requests, int32_t num_requests,
                          b2_groupby_state** out)
{
  return guarded([&] {
    if (!gb || !out) B2_FAIL(B2_INVALID_ARGUMENT, "null argument");
    *out = nullptr;
    if (gb->keys.empty()) B2_FAIL(B2_LOGIC_ERROR, "groupby needs at least one key column");
    *out = make_state(*gb, requests, num_requests);
  });
}

b2_status b2_state_update(b2_groupby_state* st, const b2_groupby* gb, const b2_aggregation_request* requests,
                          int32_t num_requests, void* stream)
{
  return guarded([&] {
    if (!st || !gb) B2_FAIL(B2_INVALID_ARGUMENT, "null argument");
    g_stats = b2_call_stats{};
    device_info();
    update_state(*st, *gb, requests, num_requests, (cudaStream_t)stream);
  });
}

int32_t b2_state_record_bytes(const b2_groupby_state* st) { return st ? st->plan.stride * 8 : 0; }

b2_status b2_state_pack(b2_groupby_state* st, int32_t num_parts, void* stream, const b2_allocator* allocator,
                        void** records_out, size_t* records_bytes, int64_t* counts)
{
  return guarded([&] {
    if (!st || !records_out || !records_bytes || !counts || num_parts < 1 || num_parts > 4096)
      B2_FAIL(B2_INVALID_ARGUMENT, "bad argument");
    device_info();
    std::vector<int64_t> c;
    Scratch recs;
    pack_table(*st, num_parts, (cudaStream_t)stream, recs, c);
    int64_t total = 0;
    for (int p = 0; p < num_parts; ++p) { counts[p] = c[(size_t)p]; total += c[(size_t)p]; }
    const b2_allocator al = resolve(allocator);
    *records_bytes = (size_t)total * st->plan.stride * 8;
    *records_out = out_alloc(al, *records_bytes, (cudaStream_t)stream);
    if (total > 0) {
      CUDA_TRY(cudaMemcpyAsync(*records_out, recs.p, *records_bytes, cudaMemcpyDeviceToDevice, (cudaStream_t)stream));
      CUDA_TRY(cudaStreamSynchronize((cudaStream_t)stream));
    }
  });
}

int64_t b2_state_chunk_bytes(const b2_groupby_state* st, int64_t chunk_records)
{
  return st ? 16 + chunk_records * (int64_t)st->plan.stride * 8 : 0;
}

b2_status b2_state_pack_chunks(b2_groupby_state* st, int32_t num_parts, int64_t chunk_records, void* stream_, void* out)
{
  return guarded([&] {
    cudaStream_t stream = (cudaStream_t)stream_;
    // a table whose first attempt has not been read back: the kernel itself marks the chunks if it failed
    const int check = (st && st->deferred) ? (st->deferred_lean ? 3 : 1) : 0;
    if (!st || !out || num_parts < 1 || num_parts > 4096 || chunk_records < 1) B2_FAIL(B2_INVALID_ARGUMENT, "bad argument");
    if (st->sc.key_mode != KM_PACKED || st->sc.has_arg)
      B2_FAIL(B2_UNSUPPORTED, "partial records of string / float / wide keys (or of row-index accumulators) are not transferable; partition the rows instead");
    device_info();
    const int64_t chunk_words = 2 + chunk_records * st->plan.stride;
    if (!st->table) {  // no groups: empty chunks
      for (int p = 0; p < num_parts; ++p)
        CUDA_TRY(cudaMemsetAsync((u64*)out + p * chunk_words, 0, 16, stream));
      return;
    }
    Scratch cursors((size_t)(num_parts + 1) * sizeof(u64), stream);  // per destination + the ticket of the last CTA
    CUDA_TRY(cudaMemsetAsync(cursors.p, 0, cursors.bytes, stream));
    const int grid = grid_for(st->cap + 1 + st->dense_slots, 256, 8);
    k_pack_chunks<<<grid, 256, 0, stream>>>(st->table, st->cap, st->plan.stride, num_parts, st->ctrl, (u64*)cursors.p,
                                            (u64*)out, chunk_records, check);
    CUDA_TRY(cudaGetLastError());
    g_stats.kernel_launches += 1;
  });
}

b2_status b2_state_merge_chunks(b2_groupby_state* st, const void* chunks, int32_t num_chunks, int64_t chunk_records,
                                void* stream_)
{
  return guarded([&] {
    cudaStream_t stream = (cudaStream_t)stream_;
    if (!st || !chunks || num_chunks < 1 || chunk_records < 1) B2_FAIL(B2_INVALID_ARGUMENT, "bad argument");
    if (st->sc.key_mode != KM_PACKED || st->sc.has_arg)
      B2_FAIL(B2_UNSUPPORTED, "partial records of string / float / wide keys (or of row-index accumulators) are not transferable; partition the rows instead");
    if (st->table) B2_FAIL(B2_LOGIC_ERROR, "b2_state_merge_chunks needs an empty state");
    device_info();
    st->last_stream = stream;
    const int64_t worst = (int64_t)num_chunks * chunk_records;
    alloc_table(*st, std::max<int64_t>(1024, (int64_t)((double)worst / 0.6) + 64), 1.0, stream);
    k_merge_chunks<<<grid_for(worst, 256, 8), 256, 0, stream>>>(st->plan, st->table, st->cap, st->ctrl,
                                                                (const u64*)chunks, num_chunks, chunk_records);
    CUDA_TRY(cudaGetLastError());
    g_stats.kernel_launches++;
    st->ctrl_fresh = false;
  });
}

b2_status b2_state_merge(b2_groupby_state* st, const void* records, int64_t num_records, void* stream)
{
  return guarded([&] {
    if (!st || (num_records > 0 && !records)) B2_FAIL(B2_INVALID_ARGUMENT, "bad argument");
    device_info();
    merge_records(*st, (const u64*)records, num_records, (cudaStream_t)stream);
  });
}

b2_status b2_state_reset(b2_groupby_state* st, int64_t expected_groups, void* stream)
{
  return guarded([&] {
    if (!st) B2_FAIL(B2_INVALID_ARGUMENT, "null argument");
    free_table(*st, (cudaStream_t)stream);
    st->groups.release();
    st->groups_n = -1;
    st->groups_cap = 0;
    st->deferred = false;
    st->host_ctrl = DCtrl{};
    st->ctrl_fresh = true;
    st->has_rows = false;
    st->row_keys.clear();
    st->expected_groups = expected_groups;
  });
}

b2_status b2_state_num_groups(b2_groupby_state* st, void* stream, int64_t* out)
{
  return guarded([&] {
    if (!st || !out) B2_FAIL(B2_INVALID_ARGUMENT, "null argument");
    *out = 0;
    if (!st->table) return;
    read_ctrl(*st, (cudaStream_t)stream);
    if (st->host_ctrl.chunk_overflow) B2_FAIL(B2_LOGIC_ERROR, "partial-record chunk overflow");
    *out = num_groups(*st);
  });
}

b2_status b2_state_finalize(b2_groupby_state* st, void* stream, const b2_allocator* allocator, b2_groupby_result* out)
{
  return guarded([&] {
    if (!st || !out) B2_FAIL(B2_INVALID_ARGUMENT, "null argument");
    device_info();
    finalize_state(*st, (cudaStream_t)stream, allocator, out);
  });
}

void b2_state_destroy(b2_groupby_state* st)
{
  if (!st) return;
  if (st->table) cudaFreeAsync(st->table, st->last_stream);
  if (st->ctrl) cudaFreeAsync(st->ctrl, st->last_stream);
  delete st;
}

b2_status b2_hash_partition(const b2_column_view* columns, int32_t num_columns, int32_t num_key_columns,
                            int32_t num_parts, int32_t hash_function, uint32_t seed, void* stream_,
                            const b2_allocator* allocator, b2_owned_column* out_columns, int64_t* offsets)
{
  return guarded([&] {
    cudaStream_t stream = (cudaStream_t)stream_;
    if (!offsets || num_columns < 0 || (num_columns > 0 && (!columns || !out_columns)) || num_key_columns < 0 ||
        num_key_columns > num_columns || num_parts < 0 || num_parts > (1 << 20))
      B2_FAIL(B2_INVALID_ARGUMENT, "bad argument");
    // cpp/src/partitioning/partitioning.cu:938-945
    if (hash_function != B2_HASH_IDENTITY && hash_function != B2_HASH_MURMUR3)
      B2_FAIL(B2_LOGIC_ERROR, "Unsupported hash function in hash_partition");
    if (num_columns > MAX_PART_COLS) B2_FAIL(B2_UNSUPPORTED, "more than 32 columns");
    if (num_key_columns > MAX_KEYS) B2_FAIL(B2_UNSUPPORTED, "more than 16 columns to hash");
    device_info();
    const b2_allocator al = resolve(allocator);
    // nothing to hash, or nowhere to put the rows: an empty table of the same column types and
    // num_parts + 1 zero offsets (cpp/src/partitioning/partitioning.cu:885-888,
    // cpp/tests/partitioning/hash_partition_test.cpp:72-142)
    const bool empty_result = num_key_columns == 0 || num_parts == 0 || num_columns == 0 || columns[0].size == 0;
    const int64_t n = empty_result ? 0 : columns[0].size;
    for (int c = 0; c < num_columns; ++c) {
      // cpp/src/partitioning/partitioning.cu:934-937 (std::invalid_argument there)
      if (!empty_result && columns[c].size != n)
        B2_FAIL(B2_INVALID_ARGUMENT, "Input table and key table must have same number of rows, or key table should have no columns.");
      if (columns[c].type_id == B2_STRING) {
        if (n > 0 && (columns[c].num_children < 1 || !columns[c].children))
          B2_FAIL(B2_INVALID_ARGUMENT, "STRING column needs an offsets child");
      } else if (width_of(columns[c].type_id) == 0) {
        B2_FAIL(B2_UNSUPPORTED, "hash_partition serves fixed-width and STRING columns");
      }
      // cpp/src/partitioning/partitioning.cu:890-894
      if (c < num_key_columns && num_parts > 0 && hash_function == B2_HASH_IDENTITY && !is_numeric_t(columns[c].type_id))
        B2_FAIL(B2_LOGIC_ERROR, "IdentityHash does not support this data type");
    }
    for (int c = 0; c < num_columns; ++c) std::memset(&out_columns[c], 0, sizeof(b2_owned_column));
    for (int p = 0; p <= num_parts; ++p) offsets[p] = 0;
    struct Guard {
      b2_owned_column* cols; int n; const b2_allocator* al; cudaStream_t s; bool armed = true;
      ~Guard() { if (armed) for (int i = 0; i < n; ++i) b2_column_free(&cols[i], al, s); }
    } guard{out_columns, num_columns, &al, stream};

    if (empty_result) {
      for (int c = 0; c < num_columns; ++c) {
        b2_owned_column& oc = out_columns[c];
        if (columns[c].type_id == B2_STRING) {
          oc.type_id = B2_STRING;
        } else {
          init_owned(oc, columns[c].type_id, 0, false, al, stream);
        }
        oc.scale = columns[c].scale;
      }
      guard.armed = false;
      return;
    }

    // hashing plan over the key columns (their descriptors; nulls hash as nulls)
    b2_groupby gb;
    for (int k = 0; k < num_key_columns; ++k) gb.keys.emplace_back(columns[k]);
    gb.null_policy = B2_NULL_INCLUDE;
    DPlan P{};
    {
      Schema sc = make_schema(gb, nullptr, 0);
      fill_plan_schema(P, sc);
      bind_plan_inputs(P, sc, gb, nullptr, 0);
    }
    DPartPlan Q{};
    Q.nparts = num_parts;
    Q.hash_kind = hash_function == B2_HASH_IDENTITY ? RH_IDENTITY : RH_MURMUR3;
    Q.seed = seed;
    const int64_t want = std::max<int64_t>(1, (n + 8191) / 8192);
    int grid = (int)std::min<int64_t>(want, (int64_t)device_info().sms * 4);
    // per-CTA counters fit shared memory up to 4096 partitions; beyond that they live in global memory,
    // with fewer CTAs so that grid x partitions stays bounded (hash_partition_test.cpp:172-187)
    Q.counters_in_global = num_parts > 4096;
    if (Q.counters_in_global) grid = (int)std::max<int64_t>(1, std::min<int64_t>(grid, (int64_t)(1 << 22) / num_parts));
    Q.rows_per_cta = ((n + grid - 1) / grid + PART_BLOCK - 1) / PART_BLOCK * PART_BLOCK;
    const size_t cells = (size_t)grid * num_parts;
    const size_t smem = Q.counters_in_global ? 0 : (size_t)num_parts * 4;

    // 1. rows per (partition, CTA), 2. their starts by one exclusive scan, 3. the permutation
    Scratch counts(cells * 8, stream), starts((cells + 1) * 8, stream), d_offsets((size_t)(num_parts + 1) * 8, stream);
    // columns the placing kernel moves itself (fixed width, no null mask); the others go through the permutation
    auto direct = std::make_unique<DDirectCols>();
    std::memset(direct.get(), 0, sizeof(DDirectCols));
    std::vector<bool> is_direct((size_t)num_columns, false);
    bool need_perm = false;
    for (int c = 0; c < num_columns; ++c) {
      const b2_column_view& in = columns[c];
      if (in.type_id != B2_STRING && in.null_mask == nullptr) {
        b2_owned_column& oc = out_columns[c];
        init_owned(oc, in.type_id, n, false, al, stream);
        oc.scale = in.scale;
        const int w = width_of(in.type_id);
        const int i = direct->n++;
        direct->width[i] = w;
        direct->src[i] = (const unsigned char*)in.data + (size_t)in.offset * w;
        direct->dst[i] = (unsigned char*)oc.data;
        is_direct[(size_t)c] = true;
      } else {
        need_perm = true;
      }
    }
    Scratch cta_scratch, perm;
    if (need_perm) perm = Scratch((size_t)n * 4, stream);
    if (Q.counters_in_global) {
      cta_scratch = Scratch(cells * 4, stream);
      CUDA_TRY(cudaMemsetAsync(cta_scratch.p, 0, cta_scratch.bytes, stream));
    }
    k_partition_count<<<grid, PART_BLOCK, smem, stream>>>(P, Q, (i64*)counts.p, (u32*)cta_scratch.p);
    CUDA_TRY(cudaGetLastError());
    device_exclusive_scan((const i64*)counts.p, (int64_t)cells, (i64*)starts.p, stream);
    k_partition_offsets<<<grid_for(num_parts + 1, 256, 4), 256, 0, stream>>>((const i64*)starts.p, num_parts, grid, (i64*)d_offsets.p);
    CUDA_TRY(cudaMemcpyAsync(offsets, d_offsets.p, (size_t)(num_parts + 1) * 8, cudaMemcpyDeviceToHost, stream));
    if (Q.counters_in_global) CUDA_TRY(cudaMemsetAsync(cta_scratch.p, 0, cta_scratch.bytes, stream));
    k_partition_perm<<<grid, PART_BLOCK, smem, stream>>>(P, Q, (const i64*)starts.p, (u32*)cta_scratch.p, (int*)perm.p, *direct);
    CUDA_TRY(cudaGetLastError());
    g_stats.kernel_launches += 3;

    // 4. every column gathered by the permutation
    Scratch null_scratch(8, stream);
    for (int c = 0; c < num_columns; ++c) {
      if (is_direct[(size_t)c]) continue;
      const b2_column_view& in = columns[c];
      b2_owned_column& oc = out_columns[c];
      const bool nullable = in.null_mask != nullptr;
      if (in.type_id != B2_STRING) {
        init_owned(oc, in.type_id, n, nullable, al, stream);
        oc.scale = in.scale;
        oc.null_count = nullable ? in.null_count : 0;
        const int g = grid_for(n, 256, 16);
        switch (width_of(in.type_id)) {
          case 1: k_gather_column<unsigned char><<<g, 256, 0, stream>>>((const unsigned char*)in.data, in.null_mask, in.offset, (const int*)perm.p, n, (unsigned char*)oc.data, oc.null_mask); break;
          case 2: k_gather_column<unsigned short><<<g, 256, 0, stream>>>((const unsigned short*)in.data, in.null_mask, in.offset, (const int*)perm.p, n, (unsigned short*)oc.data, oc.null_mask); break;
          case 4: k_gather_column<u32><<<g, 256, 0, stream>>>((const u32*)in.data, in.null_mask, in.offset, (const int*)perm.p, n, (u32*)oc.data, oc.null_mask); break;
          default: k_gather_column<u64><<<g, 256, 0, stream>>>((const u64*)in.data, in.null_mask, in.offset, (const int*)perm.p, n, (u64*)oc.data, oc.null_mask); break;
        }
        CUDA_TRY(cudaGetLastError());
        g_stats.kernel_launches++;
        continue;
      }
      // STRING: lengths -> offsets by scan -> bytes (any number of STRING columns)
      oc.type_id = B2_STRING;
      oc.size = (int32_t)n;
      oc.null_count = nullable ? in.null_count : 0;
      if (nullable) {
        oc.null_mask_bytes = (size_t)std::max<int64_t>(1, (n + 511) / 512) * 64;
        oc.null_mask = (uint32_t*)out_alloc(al, oc.null_mask_bytes, stream);
        CUDA_TRY(cudaMemsetAsync(oc.null_mask, 0xFF, oc.null_mask_bytes, stream));
      }
      DKeyCol kc{};
      kc.data = (const unsigned char*)in.data;
      kc.mask = in.null_mask;
      kc.offset = in.offset;
      kc.vclass = VC_STRING;
      const b2_column_view& o = in.children[0];
      kc.offsets = (const unsigned char*)o.data + (size_t)o.offset * (o.type_id == B2_INT64 ? 8 : 4);
      kc.offs64 = o.type_id == B2_INT64;
      Scratch lens((size_t)(n + 1) * 8, stream), offs((size_t)(n + 1) * 8, stream);
      CUDA_TRY(cudaMemsetAsync(null_scratch.p, 0, 8, stream));
      k_string_lengths<<<grid_for(n, 256, 8), 256, 0, stream>>>(kc, (const int*)perm.p, n, (i64*)lens.p, oc.null_mask, (u32*)null_scratch.p);
      CUDA_TRY(cudaGetLastError());
      device_exclusive_scan((const i64*)lens.p, n, (i64*)offs.p, stream);
      i64 total = 0;
      CUDA_TRY(cudaMemcpyAsync(&total, (i64*)offs.p + n, 8, cudaMemcpyDeviceToHost, stream));
      CUDA_TRY(cudaStreamSynchronize(stream));
      const bool big = total > 0x7FFFFFFFll;  // cpp/src/strings/utilities.cu:150-157
      oc.data_bytes = (size_t)std::max<i64>(total, 1);
      oc.data = out_alloc(al, oc.data_bytes, stream);
      oc.num_children = 1;
      oc.children = (b2_owned_column*)std::calloc(1, sizeof(b2_owned_column));
      oc.children[0].type_id = big ? B2_INT64 : B2_INT32;
      oc.children[0].size = (int32_t)(n + 1);
      oc.children[0].data_bytes = (size_t)(n + 1) * (big ? 8 : 4);
      oc.children[0].data = out_alloc(al, oc.children[0].data_bytes, stream);
      if (big) k_string_copy<i64><<<grid_for(n * 4, 256, 8), 256, 0, stream>>>(kc, (const int*)perm.p, n, (const i64*)offs.p, (i64*)oc.children[0].data, (unsigned char*)oc.data);
      else k_string_copy<int><<<grid_for(n * 4, 256, 8), 256, 0, stream>>>(kc, (const int*)perm.p, n, (const i64*)offs.p, (int*)oc.children[0].data, (unsigned char*)oc.data);
      CUDA_TRY(cudaGetLastError());
      g_stats.kernel_launches += 5;
    }
    CUDA_TRY(cudaStreamSynchronize(stream));
    if (offsets[num_parts] != n) B2_FAIL(B2_INTERNAL_ERROR, "hash_partition: row count mismatch");
    guard.armed = false;
  });
}

b2_status b2_mask_to_bytes(const uint32_t* mask, int64_t offset, int64_t size, void* stream, uint8_t* out)
{
  return guarded([&] {
    if (!mask || !out || size < 0) B2_FAIL(B2_INVALID_ARGUMENT, "bad argument");
    if (size == 0) return;
    device_info();
    k_mask_to_bytes<<<grid_for(size, 256, 16), 256, 0, (cudaStream_t)stream>>>(mask, offset, size, out);
    CUDA_TRY(cudaGetLastError());
  });
}

b2_status b2_bytes_to_mask(const uint8_t* bytes, int64_t size, void* stream, uint32_t* mask, int32_t* null_count_device)
{
  return guarded([&] {
    if (!bytes || !mask || !null_count_device || size < 0) B2_FAIL(B2_INVALID_ARGUMENT, "bad argument");
    CUDA_TRY(cudaMemsetAsync(null_count_device, 0, 4, (cudaStream_t)stream));
    if (size == 0) return;
    device_info();
    k_bytes_to_mask<<<grid_for(size, 256, 16), 256, 0, (cudaStream_t)stream>>>(bytes, size, mask, (u32*)null_count_device);
    CUDA_TRY(cudaGetLastError());
  });
}

b2_status b2_finish_partial(int32_t kind, int32_t ddof, int32_t result_type_id, const b2_column_view* sum,
                            const b2_column_view* count, const b2_column_view* sum_sq, int32_t nullable,
                            void* stream_, const b2_allocator* allocator, b2_owned_column* out)
{
  return guarded([&] {
    cudaStream_t stream = (cudaStream_t)stream_;
    if (!count || !out) B2_FAIL(B2_INVALID_ARGUMENT, "null argument");
    if (width_of(count->type_id) == 0 || is_float_t(count->type_id) || is_decimal_t(count->type_id))
      B2_FAIL(B2_DATA_TYPE_ERROR, "count must be an integer column");
    DFinish F{};
    switch (kind) {
      case B2_AGG_COUNT_VALID: F.kind = FK_COUNT; result_type_id = B2_INT32; nullable = 0; break;
      case B2_AGG_MEAN: F.kind = FK_MEAN; break;
      case B2_AGG_M2: F.kind = FK_M2; result_type_id = B2_FLOAT64; nullable = 0; break;
      case B2_AGG_VARIANCE: F.kind = FK_VAR; result_type_id = B2_FLOAT64; nullable = 1; break;
      case B2_AGG_STD: F.kind = FK_STD; result_type_id = B2_FLOAT64; nullable = 1; break;
      case -1: F.kind = FK_VALID_ONLY; nullable = 1; break;
      default: B2_FAIL(B2_INVALID_ARGUMENT, "kind is not a finisher over partial columns");
    }
    const bool needs_sum = F.kind == FK_MEAN || F.kind == FK_M2 || F.kind == FK_VAR || F.kind == FK_STD;
    const bool needs_ssq = F.kind == FK_M2 || F.kind == FK_VAR || F.kind == FK_STD;
    auto view = [&](const b2_column_view* c, const char* what) {
      if (!c) B2_FAIL(B2_INVALID_ARGUMENT, std::string(what) + " column is missing");
      if (c->size != count->size) B2_FAIL(B2_INVALID_ARGUMENT, std::string(what) + " and count differ in size");
      if (width_of(c->type_id) == 0 || is_decimal_t(c->type_id)) B2_FAIL(B2_DATA_TYPE_ERROR, std::string(what) + " must be a numeric, timestamp or duration column");
      DValCol v{};
      v.data = (const unsigned char*)c->data; v.mask = nullptr; v.offset = c->offset; v.vclass = vclass_of(c->type_id);
      return v;
    };
    F.cnt = view(count, "count");
    if (needs_sum) F.sum = view(sum, "sum");
    if (needs_ssq) F.ssq = view(sum_sq, "sum of squares");
    F.ddof = ddof;
    F.int_mean = F.kind == FK_MEAN && !is_float_t(result_type_id);
    if (F.kind == FK_MEAN && !is_float_t(result_type_id) && !is_duration_t(result_type_id))
      B2_FAIL(B2_DATA_TYPE_ERROR, "a mean is FLOAT64 or, for durations, the duration type");
    device_info();
    const b2_allocator al = resolve(allocator);
    const int64_t n = count->size;
    std::memset(out, 0, sizeof(*out));
    if (F.kind == FK_VALID_ONLY) {
      out->type_id = B2_INT8;  // (no values: a carrier for the mask)
      out->size = (int32_t)n;
      out->null_mask_bytes = (size_t)std::max<int64_t>(1, (n + 511) / 512) * 64;
      out->null_mask = (uint32_t*)out_alloc(al, out->null_mask_bytes, stream);
    } else {
      init_owned(*out, result_type_id, n, nullable != 0, al, stream);
    }
    F.rclass = vclass_of(result_type_id);
    F.out = out->data;
    F.out_mask = out->null_mask;
    Scratch nulls(8, stream);
    CUDA_TRY(cudaMemsetAsync(nulls.p, 0, 8, stream));
    F.null_count = (u32*)nulls.p;
    try {
      if (n > 0) {
        k_finish_partial<<<grid_for(n, 256, 8), 256, 0, stream>>>(F, n);
        CUDA_TRY(cudaGetLastError());
      }
      u32 h = 0;
      CUDA_TRY(cudaMemcpyAsync(&h, nulls.p, 4, cudaMemcpyDeviceToHost, stream));
      CUDA_TRY(cudaStreamSynchronize(stream));
      out->null_count = (int32_t)h;
    } catch (...) {
      b2_column_free(out, &al, stream);
      throw;
    }
  });
}

void b2_column_free(b2_owned_column* c, const b2_allocator* allocator, void* stream)
{
  if (!c) return;
  const b2_allocator al = resolve(allocator);
  if (c->data) al.deallocate(c->data, c->data_bytes, stream, al.ctx);
  if (c->null_mask) al.deallocate(c->null_mask, c->null_mask_bytes, stream, al.ctx);
  for (int i = 0; i < c->num_children; ++i) b2_column_free(&c->children[i], allocator, stream);
  std::free(c->children);
  std::memset(c, 0, sizeof(*c));
}

// ------------------------------------------------------------------------------ multi-GPU (NCCL)
}  // extern "C" (reopened below)

namespace {

// the NCCL entry points this library uses, resolved at run time
struct NcclApi {
  void* handle = nullptr;
  ncclResult_t (*GetUniqueId)(ncclUniqueId*) = nullptr;
  ncclResult_t (*CommInitRank)(ncclComm_t*, int, ncclUniqueId, int) = nullptr;
  ncclResult_t (*CommDestroy)(ncclComm_t) = nullptr;
  ncclResult_t (*GroupStart)() = nullptr;
  ncclResult_t (*GroupEnd)() = nullptr;
  ncclResult_t (*Send)(const void*, size_t, ncclDataType_t, int, ncclComm_t, cudaStream_t) = nullptr;
  ncclResult_t (*Recv)(void*, size_t, ncclDataType_t, int, ncclComm_t, cudaStream_t) = nullptr;
  ncclResult_t (*AllGather)(const void*, void*, size_t, ncclDataType_t, ncclComm_t, cudaStream_t) = nullptr;
  const char* (*GetErrorString)(ncclResult_t) = nullptr;
};

const NcclApi& nccl_api()
{
  static NcclApi api;
  static std::once_flag once;
  static std::string failure;
  std::call_once(once, [] {
    const char* override_path = getenv("B2_NCCL_LIB");
    void* h = nullptr;
    if (override_path && *override_path) h = dlopen(override_path, RTLD_NOW | RTLD_GLOBAL);
    if (!h) h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_NOLOAD);  // the copy the host process already uses
    if (!h) h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
    if (!h) { failure = std::string("cannot load libnccl.so.2: ") + dlerror(); return; }
    api.handle = h;
    auto sym = [&](const char* name) {
      void* p = dlsym(h, name);
      if (!p && failure.empty()) failure = std::string("libnccl.so.2 lacks ") + name;
      return p;
    };
    api.GetUniqueId    = (decltype(api.GetUniqueId))sym("ncclGetUniqueId");
    api.CommInitRank   = (decltype(api.CommInitRank))sym("ncclCommInitRank");
    api.CommDestroy    = (decltype(api.CommDestroy))sym("ncclCommDestroy");
    api.GroupStart     = (decltype(api.GroupStart))sym("ncclGroupStart");
    api.GroupEnd       = (decltype(api.GroupEnd))sym("ncclGroupEnd");
    api.Send           = (decltype(api.Send))sym("ncclSend");
    api.Recv           = (decltype(api.Recv))sym("ncclRecv");
    api.AllGather      = (decltype(api.AllGather))sym("ncclAllGather");
    api.GetErrorString = (decltype(api.GetErrorString))sym("ncclGetErrorString");
  });
  if (!failure.empty()) B2_FAIL(B2_UNSUPPORTED, failure);
  return api;
}

#define NCCL_TRY(expr)                                                                            \
  do {                                                                                            \
    ncclResult_t r_ = (expr);                                                                     \
    if (r_ != ncclSuccess)                                                                        \
      B2_FAIL(B2_CUDA_ERROR, std::string("NCCL error at " #expr ": ") + nccl_api().GetErrorString(r_)); \
  } while (0)

void rethrow(b2_status s)
{
  if (s != B2_SUCCESS) throw Err{s, g_last_error};
}

constexpr int64_t MULTI_CHUNK_RECORDS = 16384;  // records per destination of the fixed-size exchange
constexpr int64_t MULTI_CHUNK_LIMIT   = 64ll << 20;  // bytes all chunks of one rank may take

}  // namespace

struct b2_comm {
  ncclComm_t comm = nullptr;
  int rank = 0, nranks = 1;
  bool owned = false;
};

namespace {

// all-to-all of equal-sized pieces
void exchange_equal(const b2_comm& c, const unsigned char* send, unsigned char* recv, size_t piece, cudaStream_t stream)
{
  const NcclApi& n = nccl_api();
  NCCL_TRY(n.GroupStart());
  for (int r = 0; r < c.nranks; ++r) {
    NCCL_TRY(n.Send(send + (size_t)r * piece, piece, ncclUint8, r, c.comm, stream));
    NCCL_TRY(n.Recv(recv + (size_t)r * piece, piece, ncclUint8, r, c.comm, stream));
  }
  NCCL_TRY(n.GroupEnd());
}

// A rank whose local pass failed still takes part in the exchange — with chunks (or a count row) that
// carry a failure mark — so that every rank leaves the call with an error instead of one rank
// leaving while its peers wait in the collective.
constexpr u64 CHUNK_MARK_OVERFLOW = 1, CHUNK_MARK_FAILED = 2;

struct RedoExact {};  // the fixed-size exchange did not hold: every rank repeats it with exact sizes

// reads back a first table attempt that was left unread and, if it failed, continues the aggregate
void resolve_deferred(b2_groupby_state& st, const b2_groupby& gb, cudaStream_t stream)
{
  if (!st.deferred) return;
  st.deferred = false;
  st.ctrl_fresh = false;
  read_ctrl(st, stream);
  const DCtrl& h = st.host_ctrl;
  if (!h.overflow && !h.error && !(st.deferred_lean && !h.dense.enabled)) { add_kernel_ms(); return; }
  aggregate_fresh(st, gb, stream, /*may_partition=*/true, /*defer=*/false, /*resume=*/true);
}

void aggregate_multi(b2_comm& c, b2_groupby& gb, const b2_aggregation_request* reqs, int nreqs, cudaStream_t stream,
                     const b2_allocator* allocator, b2_groupby_result* out)
{
  const NcclApi& n = nccl_api();
  // what can fail before any communication fails on every rank alike (same schema everywhere)
  std::unique_ptr<b2_groupby_state, void (*)(b2_groupby_state*)> local(make_state(gb, reqs, nreqs), b2_state_destroy);
  if (local->sc.key_mode != KM_PACKED || local->sc.has_arg)
    B2_FAIL(B2_UNSUPPORTED, "partial records of string / float / wide keys (or of row-index accumulators) are not transferable; partition the rows instead");
  const int W = c.nranks;
  const int64_t chunk_bytes = b2_state_chunk_bytes(local.get(), MULTI_CHUNK_RECORDS);
  const int64_t chunk_words = chunk_bytes / 8;
  bool failed = false;
  Err failure{B2_SUCCESS, ""};
  // With chunk-sized states the local attempt is not read back before the exchange: k_pack_chunks marks its
  // chunks if the attempt failed, and the one synchronisation of the call comes after the merged table's
  // finalize kernel has been enqueued.
  const bool chunked = chunk_bytes * W <= MULTI_CHUNK_LIMIT;
  try {
    update_state(*local, gb, reqs, nreqs, stream, /*may_partition=*/true, /*defer=*/chunked);
  } catch (const Err& e) {
    failed = true;
    failure = e;
    cudaGetLastError();
  }

  // ---- small states: fixed-size chunks, no host round trip before the exchange.  Every rank takes
  // this branch or none does (the condition depends on the schema and the rank count only); a rank
  // whose groups cannot fit whatever their split sends marked chunks without packing anything.
  if (chunked) {
    Scratch send((size_t)chunk_bytes * W, stream), recv((size_t)chunk_bytes * W, stream);
    // (a group list is what the partitioned path leaves: half a million groups at least, never chunk-sized)
    const bool hopeless = !failed && (local->groups_n >= 0 ||
                                      (local->table && local->ctrl_fresh && num_groups(*local) > (int64_t)W * MULTI_CHUNK_RECORDS));
    if (failed || hopeless) {
      const u64 head[2] = {0, failed ? CHUNK_MARK_FAILED : CHUNK_MARK_OVERFLOW};
      for (int r = 0; r < W; ++r)
        CUDA_TRY(cudaMemcpyAsync((u64*)send.p + (size_t)r * chunk_words, head, 16, cudaMemcpyHostToDevice, stream));
      CUDA_TRY(cudaStreamSynchronize(stream));  // `head` is a stack object
    } else {
      rethrow(b2_state_pack_chunks(local.get(), W, MULTI_CHUNK_RECORDS, stream, send.p));
    }
    exchange_equal(c, (const unsigned char*)send.p, (unsigned char*)recv.p, (size_t)chunk_bytes, stream);
    if (failed) {
      CUDA_TRY(cudaStreamSynchronize(stream));
      throw failure;
    }
    std::unique_ptr<b2_groupby_state, void (*)(b2_groupby_state*)> merged(make_state(gb, reqs, nreqs), b2_state_destroy);
    rethrow(b2_state_merge_chunks(merged.get(), recv.p, W, MULTI_CHUNK_RECORDS, stream));
    // the merged table is finalized before anything is read back (at most W chunks of groups); a marked chunk
    // shows in its control block, which that one synchronisation reads
    merged->deferred = true;
    merged->deferred_lean = false;
    merged->deferred_cap = merged->cap;
    merged->deferred_bound = std::min<int64_t>((int64_t)W * MULTI_CHUNK_RECORDS, (int64_t)merged->host_ctrl.claim_limit + 1);
    const std::function<void()> redo = [] { throw RedoExact{}; };
    try {
      finalize_state(*merged, stream, allocator, out, &redo);
      return;
    } catch (const RedoExact&) {
      if (merged->host_ctrl.chunk_overflow >= CHUNK_MARK_FAILED) B2_FAIL(B2_INTERNAL_ERROR, "the local aggregate failed on another rank");
      if (merged->host_ctrl.chunk_overflow < CHUNK_MARK_OVERFLOW) B2_FAIL(B2_INTERNAL_ERROR, "hash table overflow while merging partial-record chunks");
    }
    // every rank read a marked chunk: all of them go on to the exact-size exchange
  }
  if (!failed) {
    try {
      resolve_deferred(*local, gb, stream);
    } catch (const Err& e) {
      failed = true;
      failure = e;
      cudaGetLastError();
    }
  }

  // ---- exact sizes: count matrix (with a status word per rank) by all-gather, then variable send / recv
  Scratch records;
  std::vector<int64_t> counts((size_t)W + 1, 0);
  if (!failed) {
    try {
      std::vector<int64_t> cnt;
      pack_table(*local, W, stream, records, cnt);
      std::copy(cnt.begin(), cnt.end(), counts.begin());
    } catch (const Err& e) {
      failed = true;
      failure = e;
      cudaGetLastError();
      std::fill(counts.begin(), counts.end(), 0);
    }
  }
  counts[(size_t)W] = failed ? 1 : 0;
  const int row = W + 1;
  Scratch dcounts((size_t)row * 8, stream), dmatrix((size_t)W * row * 8, stream);
  CUDA_TRY(cudaMemcpyAsync(dcounts.p, counts.data(), (size_t)row * 8, cudaMemcpyHostToDevice, stream));
  NCCL_TRY(n.AllGather(dcounts.p, dmatrix.p, (size_t)row, ncclInt64, c.comm, stream));
  std::vector<int64_t> matrix((size_t)W * row);
  CUDA_TRY(cudaMemcpyAsync(matrix.data(), dmatrix.p, (size_t)W * row * 8, cudaMemcpyDeviceToHost, stream));
  CUDA_TRY(cudaStreamSynchronize(stream));
  if (failed) throw failure;
  for (int r = 0; r < W; ++r)
    if (matrix[(size_t)r * row + W] != 0) B2_FAIL(B2_INTERNAL_ERROR, "the local aggregate failed on another rank");
  const size_t rb = (size_t)local->plan.stride * 8;
  int64_t nrecv = 0;
  std::vector<int64_t> recv_counts((size_t)W);
  for (int r = 0; r < W; ++r) { recv_counts[(size_t)r] = matrix[(size_t)r * row + c.rank]; nrecv += recv_counts[(size_t)r]; }
  Scratch recv(std::max<size_t>(8, (size_t)nrecv * rb), stream);
  NCCL_TRY(n.GroupStart());
  {
    size_t soff = 0, roff = 0;
    for (int r = 0; r < W; ++r) {
      if (counts[(size_t)r] > 0) NCCL_TRY(n.Send((const unsigned char*)records.p + soff, (size_t)counts[(size_t)r] * rb, ncclUint8, r, c.comm, stream));
      if (recv_counts[(size_t)r] > 0) NCCL_TRY(n.Recv((unsigned char*)recv.p + roff, (size_t)recv_counts[(size_t)r] * rb, ncclUint8, r, c.comm, stream));
      soff += (size_t)counts[(size_t)r] * rb;
      roff += (size_t)recv_counts[(size_t)r] * rb;
    }
  }
  NCCL_TRY(n.GroupEnd());
  // the local table is no longer needed; the merged one is sized for the records received
  rethrow(b2_state_reset(local.get(), std::max<int64_t>(nrecv, 1), stream));
  merge_records(*local, (const u64*)recv.p, nrecv, stream);
  finalize_state(*local, stream, allocator, out);
}

}  // namespace

extern "C" {

b2_status b2_comm_unique_id(uint8_t id[B2_COMM_ID_BYTES])
{
  return guarded([&] {
    if (!id) B2_FAIL(B2_INVALID_ARGUMENT, "id is null");
    static_assert(sizeof(ncclUniqueId) == B2_COMM_ID_BYTES, "NCCL unique id size");
    ncclUniqueId u;
    NCCL_TRY(nccl_api().GetUniqueId(&u));
    std::memcpy(id, &u, sizeof(u));
  });
}

b2_status b2_comm_create(const uint8_t id[B2_COMM_ID_BYTES], int32_t rank, int32_t num_ranks, b2_comm** out)
{
  return guarded([&] {
    if (!out) B2_FAIL(B2_INVALID_ARGUMENT, "out is null");
    *out = nullptr;
    if (!id || num_ranks < 1 || rank < 0 || rank >= num_ranks) B2_FAIL(B2_INVALID_ARGUMENT, "bad rank / num_ranks / id");
    ncclUniqueId u;
    std::memcpy(&u, id, sizeof(u));
    auto c = std::make_unique<b2_comm>();
    NCCL_TRY(nccl_api().CommInitRank(&c->comm, num_ranks, u, rank));
    c->rank = rank; c->nranks = num_ranks; c->owned = true;
    *out = c.release();
  });
}

b2_status b2_comm_adopt(void* nccl_comm, int32_t rank, int32_t num_ranks, b2_comm** out)
{
  return guarded([&] {
    if (!out) B2_FAIL(B2_INVALID_ARGUMENT, "out is null");
    *out = nullptr;
    if (!nccl_comm || num_ranks < 1 || rank < 0 || rank >= num_ranks) B2_FAIL(B2_INVALID_ARGUMENT, "bad communicator / rank / num_ranks");
    nccl_api();
    auto c = std::make_unique<b2_comm>();
    c->comm = (ncclComm_t)nccl_comm; c->rank = rank; c->nranks = num_ranks; c->owned = false;
    *out = c.release();
  });
}

void b2_comm_destroy(b2_comm* comm)
{
  if (!comm) return;
  if (comm->owned && comm->comm) {
    try { nccl_api().CommDestroy(comm->comm); } catch (...) {}
  }
  delete comm;
}

b2_status b2_groupby_aggregate_multi(b2_comm* comm, b2_groupby* gb, const b2_aggregation_request* requests,
                                     int32_t num_requests, void* stream, const b2_allocator* allocator,
                                     b2_groupby_result* out)
{
  return guarded([&] {
    if (!comm || !gb || !out) B2_FAIL(B2_INVALID_ARGUMENT, "null argument");
    g_stats = b2_call_stats{};
    std::memset(out, 0, sizeof(*out));
    if (gb->keys.empty()) B2_FAIL(B2_LOGIC_ERROR, "groupby needs at least one key column");
    device_info();
    aggregate_multi(*comm, *gb, requests, num_requests, (cudaStream_t)stream, allocator, out);
  });
}

const char* b2_last_error(void) { return g_last_error.c_str(); }
const char* b2_version(void) { return "b2-groupby 0.1 (sm_100a)"; }
void b2_get_last_stats(b2_call_stats* out) { if (out) *out = g_stats; }

}  // extern "C"
