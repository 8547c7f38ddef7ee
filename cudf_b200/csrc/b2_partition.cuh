// b2_partition.cuh — the high-cardinality path: radix partition of the rows by key hash into
// buckets whose groups fit a shared-memory table, then one shared-memory aggregate per bucket.
//
// Replaces the global-memory branch of the reference (compute_global_memory_aggs.cuh:74-187: one
// probe of a global cuco set + one global atomic per row and aggregation) for inputs with millions of
// groups.  There every row costs a random read-modify-write of a 32-byte sector per accumulator; here
// the rows are moved twice at most, sequentially, and every atomic is a shared-memory atomic:
//
//   k_rp_count      one pass over the key columns: rows per level-1 digit (the top 10 bits of the key
//                   hash) and, when the number of groups is not known, the HyperLogLog registers
//   k_rp_scatter    rows -> records {key, value words, validity word}, written to the region of their
//                   level-1 digit (structure-of-arrays record buffer; CTA-local counting per tile,
//                   one global cursor reservation per digit and tile)
//   k_rp_count2 /   second level inside every level-1 partition (only when one level leaves more
//   k_rp_scatter2   groups per bucket than a shared-memory table holds)
//   k_rp_aggregate  one CTA per bucket at a time: open-addressing table in shared memory, the
//                   bucket's records folded with shared-memory atomics, the finished groups appended
//                   to a compact record list (structure-of-arrays)
//   k_finalize_records  record list -> output columns (the finishers of k_finalize)
//
// Packed keys only (all key columns fixed-width non-float, at most 64 bits together).
#pragma once
#include "b2_kernels.cuh"

namespace b2 {

constexpr int RP_BLOCK    = 1024;                // threads per CTA of the counting kernels
// The scatter kernels run as two 512-thread CTAs per SM (each stages a 4096-row tile in ~90 KB of shared
// memory) that overlap each other's barriers and memory round trips.
constexpr int RPS_BLOCK   = 512;
constexpr int RP_ROWS     = 8;                   // rows per thread per tile: two groups of 4 consecutive rows
constexpr int RP_TILE     = RPS_BLOCK * RP_ROWS; // 4096 rows
constexpr int RP_BITS_TOP = 10;                  // resolution of the first histogram
constexpr int RP_MAX_BITS = 9;                   // widest digit of one level (512 destinations)
constexpr u64 RP_SALT     = 0x9FB21C651E98DF25ull;
constexpr int RPA_BLOCK   = 512;                 // threads per CTA of the bucket aggregate (2 CTAs per SM)
constexpr int RPA_BATCH   = 4;                   // records per thread whose loads are issued together

__device__ __forceinline__ u64 rp_hash(u64 key) { return mix64(key ^ RP_SALT); }

// packed keys + activity of 4 consecutive rows starting at row0 (`nv` of them exist)
__device__ __forceinline__ void rp_keys4(const DPlan& P, i64 row0, int nv, u64 (&kk)[4], u32& act)
{
  act = nv >= 4 ? 0xFu : (nv > 0 ? (1u << nv) - 1u : 0u);
  if (nv == 4 && (P.flags & PF_VEC_KEYS)) {
    packed_keys4(P, row0, kk, act);
  } else {
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      kk[j] = 0;
      if (!((act >> j) & 1u)) continue;
      if (!row_active(P, row0 + j)) { act &= ~(1u << j); continue; }
      kk[j] = pack_key(P, row0 + j);
    }
  }
}


// ------------------------------------------------------------------------------ hot keys (skewed inputs)
// A key that holds a visible share of the rows would put all its records into one bucket and serialise them
// on one shared-memory slot.  For aggregates whose cells are Σx / n / Σx² of one float column the hottest
// keys are therefore taken out before the rows are partitioned:
//   k_hot_sample   256K evenly spaced rows -> occurrences per key (a global counting table), and the
//                  largest magnitude among the sampled values (places the fixed-point windows)
//   k_hot_hist /   the keys seen most often (at most HOT_MAX, at least 3 times each) -> the hot set: an
//   k_hot_select
//                  open-addressing table of HOT_SLOTS key cells and a dense id per key
//   k_rp_count<..., HOT>  folds the rows of hot keys into per-CTA fixed-point accumulators (fx_split /
//                  fx_add: native 32-bit shared-memory atomics, which keep their rate on hot addresses) and
//                  counts only the other rows into the digit histogram; k_rp_scatter skips hot rows
//   k_rp_append_hot  the hot keys' finished cells -> the group list
// Hot and cold keys are disjoint, so the list is the union of both parts.
constexpr int HOT_SAMPLES    = 1 << 18;
constexpr int HOT_COUNT_SLOTS = 1 << 19;  // counting table of the sampler
constexpr int HOT_MAX        = 2048;      // keys in the hot set
constexpr int HOT_SLOTS      = 4096;      // its table (load <= 1/2)
constexpr u32 HOT_MIN_COUNT  = 3;         // occurrences among the samples that make a key hot
constexpr int HOT_ACC_WORDS  = 4;         // global accumulators per hot key: n, Σx, Σx², seen

struct DHot {
  u64* keys;        // [HOT_SLOTS] hot-set table, EMPTY = free
  unsigned short* ids;  // [HOT_SLOTS] dense id of the key in the same slot
  u32* info;        // [0] number of hot keys, [1] 1 + largest biased exponent among the sampled values,
                    // [4, 260) keys per occurrence count (k_hot_hist)
  u64* acc;         // [HOT_MAX][HOT_ACC_WORDS] finished accumulators (filled by k_rp_count)
  u32* row_mask;    // one bit per row: the row's key is hot (written by k_rp_count, read by k_rp_scatter)
};

__device__ __forceinline__ int hot_find(const u64* hk, u64 key, u64 h)
{
  u32 idx = (u32)h & (HOT_SLOTS - 1);
  for (int p = 0; p < HOT_SLOTS; ++p) {
    const u64 k = hk[idx];
    if (k == key) return (int)idx;
    if (k == EMPTY) return -1;
    idx = (idx + 1u) & (HOT_SLOTS - 1);
  }
  return -1;
}

__global__ void __launch_bounds__(256) k_hot_sample(const __grid_constant__ DPlan P, u64* __restrict__ ckeys,
                                                    u32* __restrict__ ccnt, u32* __restrict__ info)
{
  const i64 nsamp  = P.nrows < HOT_SAMPLES ? P.nrows : HOT_SAMPLES;
  const i64 stride = P.nrows / (nsamp > 0 ? nsamp : 1);
  u32 emax = 0;
  for (i64 i = (i64)blockIdx.x * blockDim.x + threadIdx.x; i < nsamp; i += (i64)gridDim.x * blockDim.x) {
    const i64 row = i * stride + (stride > 1 ? (i64)(((u64)i * 7919ull) % (u64)stride) : 0);
    if (!row_active(P, row)) continue;
    const u64 key = pack_key(P, row);
    if (key != EMPTY) {
      u32 idx = (u32)(rp_hash(key) >> 20) & (HOT_COUNT_SLOTS - 1);
      for (int p = 0; p < 64; ++p) {  // (a sample that finds no slot in 64 probes is dropped: it is only a sample)
        u64 k = ckeys[idx];
        if (k == EMPTY) {
          k = atomicCAS(ckeys + idx, EMPTY, key);
          if (k == EMPTY) k = key;
        }
        if (k == key) { atomicAdd(ccnt + idx, 1u); break; }
        idx = (idx + 1u) & (HOT_COUNT_SLOTS - 1);
      }
    }
    if (value_valid(P.vals[0], row)) {
      const u32 e = (u32)((load_value(P.vals[0], row) >> 52) & 0x7FFu);
      if (e != 0x7FFu && e + 1u > emax) emax = e + 1u;
    }
  }
  emax = __reduce_max_sync(0xFFFFFFFFu, emax);
  if ((threadIdx.x & 31) == 0 && emax) atomicMax(info + 1, emax);
}

// keys per (clamped) occurrence count: `hist` = 256 zeroed words
__global__ void __launch_bounds__(256) k_hot_hist(const u32* __restrict__ ccnt, u32* __restrict__ hist)
{
  __shared__ u32 s_hist[256];
  s_hist[threadIdx.x] = 0;
  __syncthreads();
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < HOT_COUNT_SLOTS; i += gridDim.x * blockDim.x) {
    const u32 c = ccnt[i];
    if (c >= HOT_MIN_COUNT) atomicAdd(&s_hist[c < 255u ? c : 255u], 1u);
  }
  __syncthreads();
  if (s_hist[threadIdx.x]) atomicAdd(&hist[threadIdx.x], s_hist[threadIdx.x]);
}

// `hot.keys` arrives filled with EMPTY, `hot.info[0]` (the id counter, then the number of hot keys) zero.
// Every CTA derives the same threshold from the histogram: the smallest count from which on at most HOT_MAX
// keys qualify.
__global__ void __launch_bounds__(256) k_hot_select(const u64* __restrict__ ckeys, const u32* __restrict__ ccnt,
                                                    const u32* __restrict__ hist, DHot hot)
{
  __shared__ u32 s_min;
  if (threadIdx.x == 0) {
    u32 total = 0, t = 256;
    while (t > HOT_MIN_COUNT && total + hist[t - 1] <= (u32)HOT_MAX) { --t; total += hist[t]; }
    s_min = t;
  }
  __syncthreads();
  const u32 tmin = s_min;
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < HOT_COUNT_SLOTS; i += gridDim.x * blockDim.x) {
    const u32 c = ccnt[i];
    if ((c < 255u ? c : 255u) < tmin) continue;
    const u64 key = ckeys[i];
    const u32 id = atomicAdd(hot.info, 1u);  // (at most HOT_MAX keys qualify: tmin bounds them)
    if (id >= (u32)HOT_MAX) continue;
    u32 idx = (u32)rp_hash(key) & (HOT_SLOTS - 1);
    for (;;) {
      const u64 old = atomicCAS(hot.keys + idx, EMPTY, key);
      if (old == EMPTY) { hot.ids[idx] = (unsigned short)id; break; }
      idx = (idx + 1u) & (HOT_SLOTS - 1);  // terminates: at most HOT_MAX keys in HOT_SLOTS slots
    }
  }
}

// ------------------------------------------------------------------------------ level-1 histogram (+ HyperLogLog)
// With HOT the kernel also carries the hot set (dynamic shared memory: keys, ids, then per hot key an
// addend count, the limbs of Σx and of Σx², and a "seen" bit): rows of hot keys are folded here and left out
// of the histogram.  P.cells are Σx / n / Σx² of value column 0 in that case.
constexpr int HOT_STRIDE = HOT_MAX + 1;  // words between the limbs of one key: odd, so that they lie in different banks
constexpr size_t rp_count_hot_smem() { return (size_t)HOT_SLOTS * 10 + (size_t)HOT_MAX * 4 + (size_t)HOT_STRIDE * 8 * FX_LIMBS + HOT_MAX / 8; }

template <bool WITH_HLL, bool HOT>
__global__ void __launch_bounds__(RP_BLOCK, 1) k_rp_count(const __grid_constant__ DPlan P, u64* __restrict__ hist,
                                                       u32* __restrict__ hll, const DHot hot)
{
  extern __shared__ __align__(16) unsigned char rp_hot_smem[];
  __shared__ u32 s_hist[1 << RP_BITS_TOP];
  __shared__ u32 s_regs[WITH_HLL ? HLL_REGS : 1];
  u64* hk = (u64*)rp_hot_smem;                              // [HOT_SLOTS]
  unsigned short* hid = (unsigned short*)(hk + HOT_SLOTS);  // [HOT_SLOTS]
  u32* hcnt = (u32*)(hid + HOT_SLOTS);                      // [HOT_MAX]
  int* hlx  = (int*)(hcnt + HOT_MAX);                       // [FX_LIMBS][HOT_STRIDE]
  int* hlq  = hlx + FX_LIMBS * HOT_STRIDE;                  // [FX_LIMBS][HOT_STRIDE]
  u32* hseen = (u32*)(hlq + FX_LIMBS * HOT_STRIDE);         // [HOT_MAX / 32]
  int nh = 0, bx = FX_NEVER, bq = FX_NEVER;
  for (int i = threadIdx.x; i < (1 << RP_BITS_TOP); i += blockDim.x) s_hist[i] = 0;
  if (WITH_HLL) for (int i = threadIdx.x; i < HLL_REGS; i += blockDim.x) s_regs[i] = 0;
  if (HOT) {
    nh = (int)min(hot.info[0], (u32)HOT_MAX);
    if (hot.info[1]) {
      const int emax = (int)hot.info[1] - 1;
      bx = emax + FX_HEADROOM - FX_MAX_SHIFT;
      bq = 2 * emax - 1023 + 1 + 2 * FX_HEADROOM - FX_MAX_SHIFT;
    }
    if (nh > 0) {
      for (int i = threadIdx.x; i < HOT_SLOTS; i += blockDim.x) { hk[i] = hot.keys[i]; hid[i] = hot.ids[i]; }
      for (int i = threadIdx.x; i < HOT_MAX + 2 * FX_LIMBS * HOT_STRIDE + HOT_MAX / 32; i += blockDim.x) hcnt[i] = 0;
    }
  }
  __syncthreads();
  int c_sum = -1, c_cnt = -1, c_ssq = -1;
  if (HOT)
    for (int c = 0; c < P.ncells; ++c) {
      if (P.cells[c].op == OP_SUM_F) c_sum = c;
      if (P.cells[c].op == OP_CNT_V) c_cnt = c;
      if (P.cells[c].op == OP_SSQ_F) c_ssq = c;
    }
  const i64 nquads = (P.nrows + 3) / 4;
  // (whole warps stay in the loop — a lane beyond the last quad has no rows — because the hot-row mask of
  // 8 consecutive quads is put together with shuffles)
  for (i64 q = (i64)blockIdx.x * blockDim.x + threadIdx.x; q - (threadIdx.x & 31) < nquads; q += (i64)gridDim.x * blockDim.x) {
    u64 kk[4];
    u32 act;
    const int nv = (int)max((i64)0, min((i64)4, P.nrows - q * 4));
    rp_keys4(P, q * 4, nv, kk, act);
    u64 hh[4];
    int hs[4];
    u32 hotm = 0;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      hh[j] = rp_hash(kk[j]);
      hs[j] = -1;
      if (HOT && nh > 0 && ((act >> j) & 1u) && kk[j] != EMPTY) {
        hs[j] = hot_find(hk, kk[j], hh[j]);
        if (hs[j] >= 0) hotm |= 1u << j;
      }
    }
    if (HOT && nh > 0) {
      // bit r of word w of the row mask = row 32 w + r: this quad's four bits sit at 4 (q mod 8) of word q / 8
      u32 w = hotm << (4 * (threadIdx.x & 7));
      w |= __shfl_xor_sync(0xFFFFFFFFu, w, 1);
      w |= __shfl_xor_sync(0xFFFFFFFFu, w, 2);
      w |= __shfl_xor_sync(0xFFFFFFFFu, w, 4);
      if ((threadIdx.x & 7) == 0 && q < nquads) hot.row_mask[q >> 3] = w;
    }
    if (HOT && hotm) {
      const DValCol& vc = P.vals[0];
      u32 vn = hotm;
      if (vc.mask) vn &= valid_nibble(vc.mask, vc.offset + q * 4, nv);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        if (!((hotm >> j) & 1u)) continue;
        const int id = (int)hid[hs[j]];
        if (!((hseen[id >> 5] >> (id & 31)) & 1u)) atomicOr(&hseen[id >> 5], 1u << (id & 31));
        if (!((vn >> j) & 1u)) continue;
        const u64 xb = load_value(vc, q * 4 + j);
        const double d = __longlong_as_double((i64)xb);
        int qx = 0, qq = 0;
        u32 lx[4], lq[4];
        bool fits = c_sum < 0 || fx_split(xb, bx, qx, lx);
        if (fits && c_ssq >= 0) fits = fx_split((u64)__double_as_longlong(d * d), bq, qq, lq);
        u64* acc = hot.acc + (size_t)id * HOT_ACC_WORDS;
        if (!fits) {  // outside the fixed-point window: straight to the fp64 accumulators
          atomicAdd(acc, 1ull);
          if (c_sum >= 0) atomicAdd((double*)(acc + 1), d);
          if (c_ssq >= 0) atomicAdd((double*)(acc + 2), d * d);
          continue;
        }
        if (c_sum >= 0) fx_add(hlx, HOT_STRIDE, id, (xb >> 63) != 0, qx, lx);
        if (c_ssq >= 0) fx_add(hlq, HOT_STRIDE, id, false, qq, lq);
        const u32 old = atomicAdd(hcnt + id, 1u);
        if (((old + 1u) & (FX_FLUSH - 1u)) == 0u) {
          if (c_sum >= 0) atomicAdd((double*)(acc + 1), fx_take(hlx, HOT_STRIDE, id, bx));
          if (c_ssq >= 0) atomicAdd((double*)(acc + 2), fx_take(hlq, HOT_STRIDE, id, bq));
        }
      }
    }
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      if (!((act >> j) & 1u) || ((hotm >> j) & 1u)) continue;
      atomicAdd(&s_hist[hh[j] >> (64 - RP_BITS_TOP)], 1u);
      if (WITH_HLL) {
        const u64 h = hh[j] * 0x9E3779B97F4A7C15ull;  // (the partition hash, re-spread: these registers are only ever read alone)
        const u32 idx  = (u32)(h >> (64 - HLL_BITS));
        const u32 rank = (u32)__clzll((i64)((h << HLL_BITS) | (1ull << (HLL_BITS - 1)))) + 1u;
        if (s_regs[idx] < rank) atomicMax(&s_regs[idx], rank);
      }
    }
  }
  __syncthreads();
  for (int i = threadIdx.x; i < (1 << RP_BITS_TOP); i += blockDim.x)
    if (s_hist[i]) atomicAdd(&hist[i], (u64)s_hist[i]);
  if (WITH_HLL)
    for (int i = threadIdx.x; i < HLL_REGS; i += blockDim.x)
      if (s_regs[i]) atomicMax(&hll[i], s_regs[i]);
  if (HOT && nh > 0) {
    // CTAs start at different ids so that they do not all hit the same accumulators at once
    const int rot = (int)(((u64)blockIdx.x * 2654435761ull) % (u64)nh);
    for (int i0 = threadIdx.x; i0 < nh; i0 += blockDim.x) {
      const int id = i0 + rot < nh ? i0 + rot : i0 + rot - nh;
      u64* acc = hot.acc + (size_t)id * HOT_ACC_WORDS;
      const u32 n = hcnt[id];
      if (n) {
        atomicAdd(acc, (u64)n);
        if (c_sum >= 0) atomicAdd((double*)(acc + 1), fx_take(hlx, HOT_STRIDE, id, bx));
        if (c_ssq >= 0) atomicAdd((double*)(acc + 2), fx_take(hlq, HOT_STRIDE, id, bq));
      }
      if (((hseen[id >> 5] >> (id & 31)) & 1u) && acc[3] == 0) acc[3] = 1;
    }
  }
}

// the hot keys' finished cells join the group list (one thread per hot-set slot)
__global__ void k_rp_append_hot(const __grid_constant__ DPlan P, const DHot hot, u64* __restrict__ out, i64 out_cap, DCtrl* ctrl)
{
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= HOT_SLOTS) return;
  const u64 key = hot.keys[i];
  if (key == EMPTY) return;
  const u64* acc = hot.acc + (size_t)hot.ids[i] * HOT_ACC_WORDS;
  if (acc[3] == 0) return;  // sampled, but no participating row (cannot happen with samples taken from the rows)
  const u64 g = atomicAdd(&ctrl->out_cursor, 1ull);
  if (g >= (u64)out_cap) { ctrl->overflow = 1; return; }
  out[g] = key;
  for (int c = 0; c < P.ncells; ++c) {
    const int op = P.cells[c].op;
    out[(i64)(1 + c) * out_cap + g] = op == OP_CNT_V ? acc[0] : op == OP_SUM_F ? acc[1] : acc[2];
  }
}

// ------------------------------------------------------------------------------ records
// A record buffer holds `cap` records, structure-of-arrays: word w of record i at rec[w * cap + i].
// Word 0 is the packed key, words 1..nvals the value columns in their 64-bit carried form
// (load_value), the last word (if any value column is nullable) the validity bits of the values.
struct DRecords {
  u64* rec;
  i64 cap;
  int words;       // words per record
  int valid_word;  // index of the validity word, -1 = every value is valid
};

struct DScatter {
  DRecords dst;
  u64* cursors;  // [partitions] next free record of every destination (start offsets, advanced)
  int shift;     // digit = (hash >> shift) & (fan - 1)
  int fan;       // destinations per source partition (a power of two, <= 1 << RP_MAX_BITS)
};

// Both scatter levels sort a tile by digit in shared memory before writing it: every thread learns
// its records' ranks inside their digits (shared-memory atomics), the digits' runs are reserved with one
// global atomic each, the records are placed run by run in a staging array, and the staging array is
// copied out in order — consecutive threads write consecutive records of a run.  (Written straight from
// registers, every 8-byte word was an L2 write request of its own — 106 M requests for 60 M rows — and
// the level-1 pass crawled at 0.6 TB/s with DRAM 14 % busy.)
struct RpTile {
  u32* hist;   // [fan] records per digit, then cleared
  u32* off;    // [fan + 1] first staging position of every digit
  u64* base;   // [fan] first global record of every digit's run
  u64* keys;   // [RP_TILE] staged keys
  u64* vals;   // [RP_TILE] staged values (records of two words)
  unsigned short* dig;  // [RP_TILE] digit of every staged record
  unsigned short* src;  // [RP_TILE] position of the record inside the source tile (records of other shapes)
};
__host__ __device__ constexpr size_t rp_tile_smem(int fan) { return (size_t)fan * 4 + (size_t)(fan + 1) * 4 + (size_t)fan * 8 + (size_t)RP_TILE * (8 + 8 + 2 + 2) + 64; }

__device__ __forceinline__ RpTile rp_tile_carve(unsigned char* smem, int fan)
{
  RpTile t;
  t.keys = (u64*)smem;
  t.vals = t.keys + RP_TILE;
  t.base = t.vals + RP_TILE;
  t.hist = (u32*)(t.base + fan);
  t.off  = t.hist + fan;
  t.dig  = (unsigned short*)(t.off + fan + 1);
  t.src  = t.dig + RP_TILE;
  return t;
}

// after phase A (hist filled): staging offsets by an exclusive scan over the digits, one global
// reservation per digit with records, counters cleared.  `fan` <= blockDim.x.  Ends with a barrier.
__device__ __forceinline__ void rp_tile_plan(const RpTile& t, u64* cursors, int fan)
{
  __shared__ u32 s_warp[RPS_BLOCK / 32];
  const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
  const u32 c = (int)threadIdx.x < fan ? t.hist[threadIdx.x] : 0u;
  u32 v = c;
  for (int d = 1; d < 32; d <<= 1) { const u32 x = __shfl_up_sync(0xFFFFFFFFu, v, d); if (lane >= d) v += x; }
  if (lane == 31) s_warp[wid] = v;
  __syncthreads();
  if (wid == 0) {
    u32 w = lane < RPS_BLOCK / 32 ? s_warp[lane] : 0u;
    for (int d = 1; d < 32; d <<= 1) { const u32 x = __shfl_up_sync(0xFFFFFFFFu, w, d); if (lane >= d) w += x; }
    if (lane < RPS_BLOCK / 32) s_warp[lane] = w;
  }
  __syncthreads();
  if ((int)threadIdx.x < fan) {
    const u32 excl = (wid ? s_warp[wid - 1] : 0u) + v - c;
    t.off[threadIdx.x] = excl;
    t.hist[threadIdx.x] = 0;
    if (c) t.base[threadIdx.x] = atomicAdd(&cursors[threadIdx.x], (u64)c);
    if ((int)threadIdx.x == fan - 1) t.off[fan] = excl + c;
  }
  __syncthreads();
}

// level 1: input rows -> records in the region of their digit
// (`hot_rows`: one bit per row, set for the rows whose keys k_rp_count folded already — they are left out here)
__global__ void __launch_bounds__(RPS_BLOCK, 2) k_rp_scatter(const __grid_constant__ DPlan P, const DScatter D,
                                                          const u32* __restrict__ hot_rows)
{
  extern __shared__ __align__(16) unsigned char rp_stage[];
  const RpTile t = rp_tile_carve(rp_stage, D.fan);
  // one value column is the common case: its values are loaded together with the keys and staged with them
  // (a null value as a flag beside the staged digit); other shapes stage the key and the row, and gather the
  // value words at copy-out
  const bool one = P.nvals == 1;
  const bool nullable = one && D.dst.valid_word >= 0;
  for (int i = threadIdx.x; i < D.fan; i += blockDim.x) t.hist[i] = 0;
  __syncthreads();
  const i64 ntiles = (P.nrows + RP_TILE - 1) / RP_TILE;
  const u32 dmask = (u32)D.fan - 1u;
  for (i64 tile = blockIdx.x; tile < ntiles; tile += gridDim.x) {
    const i64 tile0 = tile * RP_TILE;
    u64 kk[RP_ROWS], vv[RP_ROWS];
    u32 rank[RP_ROWS];
    u32 act = 0, vok = 0xFFFFFFFFu;
    // phase A: keys (and values), digits, ranks inside the tile
#pragma unroll
    for (int g = 0; g < RP_ROWS / 4; ++g) {
      const i64 row0 = tile0 + (i64)g * (RP_TILE / (RP_ROWS / 4)) + (i64)threadIdx.x * 4;
      const int nv = (int)max((i64)0, min((i64)4, P.nrows - row0));
      u64 k4[4];
      u32 a4;
      rp_keys4(P, row0, nv, k4, a4);
      if (hot_rows && nv > 0) a4 &= ~(__ldg(hot_rows + (row0 >> 5)) >> (row0 & 31));  // (row0 is a multiple of 4)
      act |= a4 << (4 * g);
      if (nullable && nv > 0) vok = (vok & ~(0xFu << (4 * g))) | (valid_nibble(P.vals[0].mask, P.vals[0].offset + row0, nv) << (4 * g));
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        kk[4 * g + j] = k4[j];
        vv[4 * g + j] = (one && j < nv) ? load_value(P.vals[0], row0 + j) : 0ull;
      }
    }
#pragma unroll
    for (int j = 0; j < RP_ROWS; ++j) {
      rank[j] = 0;
      if ((act >> j) & 1u) {
        const u32 d = (u32)(rp_hash(kk[j]) >> D.shift) & dmask;
        rank[j] = (d << 16) | atomicAdd(&t.hist[d], 1u);  // a tile holds 4096 rows: the rank fits 16 bits
      }
    }
    __syncthreads();
    rp_tile_plan(t, D.cursors, D.fan);
    // phase C: place the records run by run
#pragma unroll
    for (int j = 0; j < RP_ROWS; ++j) {
      if (!((act >> j) & 1u)) continue;
      const u32 d = rank[j] >> 16;
      const u32 pos = t.off[d] + (rank[j] & 0xFFFFu);
      t.keys[pos] = kk[j];
      t.dig[pos]  = (unsigned short)(d | (((vok >> j) & 1u) ? 0u : 0x8000u));  // (digits stay below 2^RP_MAX_BITS)
      if (one) t.vals[pos] = vv[j];
      else t.src[pos] = (unsigned short)((j >> 2) * (RP_TILE / (RP_ROWS / 4)) + (int)threadIdx.x * 4 + (j & 3));
    }
    __syncthreads();
    // phase D: copy out in staging order
    const u32 ntile = t.off[D.fan];
    for (u32 pos = threadIdx.x; pos < ntile; pos += blockDim.x) {
      const u32 dg = t.dig[pos], d = dg & 0x7FFFu;
      const i64 at = (i64)t.base[d] + (i64)(pos - t.off[d]);
      D.dst.rec[at] = t.keys[pos];
      if (one) {
        D.dst.rec[D.dst.cap + at] = t.vals[pos];
        if (nullable) D.dst.rec[(i64)D.dst.valid_word * D.dst.cap + at] = (u64)((dg >> 15) ^ 1u);
      } else {
        const i64 row = tile0 + t.src[pos];
        u64 vbits = 0;
        for (int v = 0; v < P.nvals; ++v) {
          const DValCol& vc = P.vals[v];
          const bool ok = value_valid(vc, row);
          vbits |= (u64)ok << v;
          D.dst.rec[(i64)(1 + v) * D.dst.cap + at] = ok ? load_value(vc, row) : 0ull;
        }
        if (D.dst.valid_word >= 0) D.dst.rec[(i64)D.dst.valid_word * D.dst.cap + at] = vbits;
      }
    }
    __syncthreads();  // the staging arrays are rewritten by the next tile
  }
}

// Level 2 works on the tiles of the level-1 partitions: tile t belongs to the partition p with
// tile_start[p] <= t < tile_start[p + 1] and covers records [start[p] + j * RP_TILE, ...) of it.
struct DLevel2 {
  DRecords src;
  const u64* src_start;   // [parts + 1] first record of every source partition
  const u64* src_end;     // [parts] one past its last record (the advanced level-1 cursors)
  const u32* tile_start;  // [parts + 1] first tile of every source partition
  int parts;
};

__device__ __forceinline__ int rp_partition_of_tile(const u32* tile_start, int parts, u32 tile)
{
  int lo = 0, hi = parts;  // tile_start[lo] <= tile < tile_start[hi]
  while (hi - lo > 1) {
    const int mid = (lo + hi) >> 1;
    if (__ldg(tile_start + mid) <= tile) lo = mid; else hi = mid;
  }
  return lo;
}

// rows per (source partition, level-2 digit)
__global__ void __launch_bounds__(RP_BLOCK, 1) k_rp_count2(const DLevel2 L, int shift, int fan, u64* __restrict__ hist2)
{
  __shared__ u32 s_hist[1 << RP_MAX_BITS];
  for (int i = threadIdx.x; i < fan; i += blockDim.x) s_hist[i] = 0;
  __syncthreads();
  const u32 ntiles = __ldg(L.tile_start + L.parts);
  const u32 dmask = (u32)fan - 1u;
  for (u32 tile = blockIdx.x; tile < ntiles; tile += gridDim.x) {
    const int p = rp_partition_of_tile(L.tile_start, L.parts, tile);
    const i64 lo = (i64)L.src_start[p] + (i64)(tile - __ldg(L.tile_start + p)) * RP_TILE;
    const i64 hi = min((i64)L.src_end[p], lo + RP_TILE);
    for (i64 i = lo + threadIdx.x; i < hi; i += blockDim.x)
      atomicAdd(&s_hist[(u32)(rp_hash(__ldg(L.src.rec + i)) >> shift) & dmask], 1u);
    __syncthreads();
    for (int d = threadIdx.x; d < fan; d += blockDim.x) {
      const u32 c = s_hist[d];
      s_hist[d] = 0;
      if (c) atomicAdd(&hist2[(i64)p * fan + d], (u64)c);
    }
    __syncthreads();
  }
}

__global__ void __launch_bounds__(RPS_BLOCK, 2) k_rp_scatter2(const DLevel2 L, const DScatter D)
{
  extern __shared__ __align__(16) unsigned char rp_stage[];
  const RpTile t = rp_tile_carve(rp_stage, D.fan);
  for (int i = threadIdx.x; i < D.fan; i += blockDim.x) t.hist[i] = 0;
  __syncthreads();
  const u32 ntiles = __ldg(L.tile_start + L.parts);
  const u32 dmask = (u32)D.fan - 1u;
  // key + one value (+ its validity word): the value is loaded and staged with the key, the validity as a
  // flag beside the staged digit; records of other shapes are copied word by word from their source position
  const bool nullable = L.src.words == 3 && L.src.valid_word == 2;
  const bool staged = L.src.words == 2 || nullable;
  for (u32 tile = blockIdx.x; tile < ntiles; tile += gridDim.x) {
    const int p = rp_partition_of_tile(L.tile_start, L.parts, tile);
    const i64 lo = (i64)L.src_start[p] + (i64)(tile - __ldg(L.tile_start + p)) * RP_TILE;
    const i64 hi = min((i64)L.src_end[p], lo + RP_TILE);
    u64 kk[RP_ROWS], vv[RP_ROWS];
    u32 rank[RP_ROWS];
    u32 vok = 0xFFFFFFFFu;
#pragma unroll
    for (int j = 0; j < RP_ROWS; ++j) {
      const i64 i = lo + (i64)j * RPS_BLOCK + threadIdx.x;
      kk[j] = 0; vv[j] = 0;
      if (i < hi) {
        kk[j] = __ldg(L.src.rec + i);
        if (staged) vv[j] = __ldg(L.src.rec + L.src.cap + i);
        if (nullable && !(__ldg(L.src.rec + 2 * L.src.cap + i) & 1ull)) vok &= ~(1u << j);
      }
    }
#pragma unroll
    for (int j = 0; j < RP_ROWS; ++j) {
      const i64 i = lo + (i64)j * RPS_BLOCK + threadIdx.x;
      rank[j] = 0xFFFFFFFFu;
      if (i < hi) {
        const u32 d = (u32)(rp_hash(kk[j]) >> D.shift) & dmask;
        rank[j] = (d << 16) | atomicAdd(&t.hist[d], 1u);
      }
    }
    __syncthreads();
    rp_tile_plan(t, D.cursors + (i64)p * D.fan, D.fan);
#pragma unroll
    for (int j = 0; j < RP_ROWS; ++j) {
      if (rank[j] == 0xFFFFFFFFu) continue;
      const u32 d = rank[j] >> 16;
      const u32 pos = t.off[d] + (rank[j] & 0xFFFFu);
      t.keys[pos] = kk[j];
      t.dig[pos]  = (unsigned short)(d | (((vok >> j) & 1u) ? 0u : 0x8000u));
      if (staged) t.vals[pos] = vv[j];
      else t.src[pos] = (unsigned short)(j * RPS_BLOCK + (int)threadIdx.x);
    }
    __syncthreads();
    const u32 ntile = t.off[D.fan];
    for (u32 pos = threadIdx.x; pos < ntile; pos += blockDim.x) {
      const u32 dg = t.dig[pos], d = dg & 0x7FFFu;
      const i64 at = (i64)t.base[d] + (i64)(pos - t.off[d]);
      D.dst.rec[at] = t.keys[pos];
      if (staged) {
        D.dst.rec[D.dst.cap + at] = t.vals[pos];
        if (nullable) D.dst.rec[2 * D.dst.cap + at] = (u64)((dg >> 15) ^ 1u);
      } else {
        const i64 i = lo + t.src[pos];
        for (int w = 1; w < L.src.words; ++w) D.dst.rec[(i64)w * D.dst.cap + at] = __ldg(L.src.rec + (i64)w * L.src.cap + i);
      }
    }
    __syncthreads();
  }
}

// tiles per source partition from its record count (one thread per partition), then scanned on the device
__global__ void k_rp_tiles(const u64* __restrict__ start, const u64* __restrict__ end, int parts, u32* __restrict__ tile_start)
{
  // single CTA: exclusive scan of ceil(count / RP_TILE)
  __shared__ u32 s_sum[1024];
  u32 mine = 0;
  const int per = (parts + (int)blockDim.x - 1) / (int)blockDim.x;
  const int lo = threadIdx.x * per, hi = min(parts, lo + per);
  for (int p = lo; p < hi; ++p) mine += (u32)((end[p] - start[p] + RP_TILE - 1) / RP_TILE);
  s_sum[threadIdx.x] = mine;
  __syncthreads();
  for (int d = 1; d < (int)blockDim.x; d <<= 1) {
    const u32 t = threadIdx.x >= (u32)d ? s_sum[threadIdx.x - d] : 0u;
    __syncthreads();
    s_sum[threadIdx.x] += t;
    __syncthreads();
  }
  u32 run = s_sum[threadIdx.x] - mine;
  for (int p = lo; p < hi; ++p) {
    tile_start[p] = run;
    run += (u32)((end[p] - start[p] + RP_TILE - 1) / RP_TILE);
  }
  if (threadIdx.x == blockDim.x - 1) tile_start[parts] = s_sum[threadIdx.x];
}

// ------------------------------------------------------------------------------ bucket aggregate
struct DBuckets {
  DRecords src;
  const u64* start;  // [buckets] first record of every bucket
  const u64* end;    // [buckets] one past its last record
  i64 nbuckets;
  int slots;         // shared-memory table slots (a power of two); slot `slots` holds the key whose bits equal EMPTY
  u64* out;          // finished groups, structure-of-arrays: word w of group g at out[w * out_cap + g]; word 0 = key
  i64 out_cap;
  u64* next_bucket;  // work counter
};

// FIXED (the cells are Σx / n / Σx² of one float column): a slot keeps its sums as fixed-point limbs plus one
// fp64 cell each for what does not fit the limbs' window (and for the limbs' periodic flushes), and its count
// as 32 bits — nine native 32-bit atomics per record instead of three 64-bit ones, which shared memory only
// does as compare-and-swap loops.  `vexp` = 1 + the largest biased exponent among the sampled values.
constexpr int RPA_FIXED_SLOT_BYTES = 8 + 8 + 8 + 4 + 8 * FX_LIMBS;
constexpr int RPA_INDEX_BYTES = 2;  // per slot: the claim-order index

template <bool FIXED>
__global__ void __launch_bounds__(RPA_BLOCK, 2) k_rp_aggregate(const __grid_constant__ DPlan P, const DBuckets B, DCtrl* ctrl,
                                                            const u32* __restrict__ vexp)
{
  extern __shared__ __align__(16) unsigned char rp_smem[];
  __shared__ i64 s_bucket;
  __shared__ u32 s_count, s_fail, s_special;
  __shared__ u64 s_outbase;
  const int S  = B.slots;
  const int NS = S + 1;
  u64* skeys  = (u64*)rp_smem;   // [NS]
  u64* scells = skeys + NS;      // [ncells][NS]
  // FIXED: [NS] fp64 Σx beside the limbs, [NS] the same for Σx², [NS] counts, limbs of Σx, limbs of Σx²
  double* fex = (double*)scells;
  double* feq = fex + NS;
  u32* fcnt   = (u32*)(feq + NS);
  int* flx    = (int*)(fcnt + NS);
  int* flq    = flx + FX_LIMBS * NS;
  // slots in the order they were claimed: the finished groups are written in that order, consecutive
  // threads to consecutive list entries, without scanning the table for occupied slots
  unsigned short* sidx = FIXED ? (unsigned short*)(flq + FX_LIMBS * NS) : (unsigned short*)(scells + (size_t)P.ncells * NS);
  int fx_bx = FX_NEVER, fx_bq = FX_NEVER, c_sum = -1, c_cnt = -1, c_ssq = -1;
  if (FIXED) {
    const u32 ve = __ldg(vexp);
    if (ve) {
      const int emax = (int)ve - 1;
      fx_bx = emax + FX_HEADROOM - FX_MAX_SHIFT;
      fx_bq = 2 * emax - 1023 + 1 + 2 * FX_HEADROOM - FX_MAX_SHIFT;
    }
    for (int c = 0; c < P.ncells; ++c) {
      if (P.cells[c].op == OP_SUM_F) c_sum = c;
      if (P.cells[c].op == OP_CNT_V) c_cnt = c;
      if (P.cells[c].op == OP_SSQ_F) c_ssq = c;
    }
  }
  const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
  const u32 smask = (u32)S - 1u;
  // a bucket whose groups fill the table beyond this gives up (the caller falls back to the global table)
  const u32 fill_limit = (u32)S - (u32)(S >> 3);

  for (;;) {
    __syncthreads();
    if (threadIdx.x == 0) { s_bucket = (i64)atomicAdd(B.next_bucket, 1ull); s_count = 0; s_fail = 0; s_special = 0; }
    __syncthreads();
    const i64 b = s_bucket;
    if (b >= B.nbuckets) break;
    const i64 lo = (i64)B.start[b], hi = (i64)B.end[b];
    if (hi <= lo) continue;
    // clear the table
    for (int i = threadIdx.x; i < NS; i += blockDim.x) skeys[i] = EMPTY;
    if (FIXED) {
      for (int i = threadIdx.x; i < 2 * NS; i += blockDim.x) scells[i] = 0;                       // fex, feq
      for (int i = threadIdx.x; i < (1 + 2 * FX_LIMBS) * NS; i += blockDim.x) fcnt[i] = 0;        // fcnt, flx, flq
    } else {
      for (int c = 0; c < P.ncells; ++c) {
        const u64 id = cell_identity(P.cells[c].op);
        for (int i = threadIdx.x; i < NS; i += blockDim.x) scells[(size_t)c * NS + i] = id;
      }
    }
    __syncthreads();
    // fold the records, RPA_BATCH per thread at a time: all loads of a batch are issued before the first
    // probe, so that a batch costs one DRAM round trip instead of one per record and word
    for (i64 base = lo; base < hi; base += (i64)RPA_BATCH * blockDim.x) {
      u64 keys[RPA_BATCH], vbits[RPA_BATCH], vals[RPA_BATCH];
      const bool one_col = B.src.words - (B.src.valid_word >= 0 ? 1 : 0) == 2;  // a single value column: prefetch it too
#pragma unroll
      for (int j = 0; j < RPA_BATCH; ++j) {
        const i64 i = base + (i64)j * blockDim.x + threadIdx.x;
        keys[j] = 0; vbits[j] = ~0ull; vals[j] = 0;
        if (i < hi) {
          keys[j] = __ldg(B.src.rec + i);
          if (B.src.valid_word >= 0) vbits[j] = __ldg(B.src.rec + (i64)B.src.valid_word * B.src.cap + i);
          if (one_col) vals[j] = __ldg(B.src.rec + B.src.cap + i);
        }
      }
      // slots of the batch's records
      int slots[RPA_BATCH];
#pragma unroll
      for (int j = 0; j < RPA_BATCH; ++j) {
        const i64 i = base + (i64)j * blockDim.x + threadIdx.x;
        const u64 key = keys[j];
        int slot = -1;
        if (i < hi) {
          if (key == EMPTY) {
            slot = S;
            s_special = 1;
          } else {
            u32 idx = (u32)rp_hash(key) & smask;
            for (int p = 0; p < S; ++p) {
              u64 k = *(volatile u64*)(skeys + idx);
              if (k == EMPTY) {
                if (*(volatile u32*)&s_count >= fill_limit) break;
                k = atomicCAS(skeys + idx, EMPTY, key);
                if (k == EMPTY) { sidx[atomicAdd(&s_count, 1u)] = (unsigned short)idx; k = key; }
              }
              if (k == key) { slot = (int)idx; break; }
              idx = (idx + 1u) & smask;
            }
          }
          if (slot < 0) s_fail = 1;
        }
        slots[j] = slot;
      }
      // The lanes left the probe loops at different iterations: bring them back together, then go
      // through the accumulators cell by cell — the operator is decoded once per cell and batch (not
      // once per record), and each update is ONE predicated atomic for the whole warp.  (Diverged,
      // each lane's atomics were issued on their own: 11.5 of 32 lanes active on average.)
      __syncwarp();
      if (FIXED) {
#pragma unroll
        for (int j = 0; j < RPA_BATCH; ++j) {
          if (slots[j] < 0 || !(vbits[j] & 1ull)) continue;
          const int s = slots[j];
          const u64 xb = vals[j];
          const double d = __longlong_as_double((i64)xb);
          int qx = 0, qq = 0;
          u32 lx[4], lq[4];
          bool fits = c_sum < 0 || fx_split(xb, fx_bx, qx, lx);
          if (fits && c_ssq >= 0) fits = fx_split((u64)__double_as_longlong(d * d), fx_bq, qq, lq);
          if (!fits) {
            if (c_sum >= 0) atomicAdd(fex + s, d);
            if (c_ssq >= 0) atomicAdd(feq + s, d * d);
            atomicAdd(fcnt + s, 1u);
            continue;
          }
          if (c_sum >= 0) fx_add(flx, NS, s, (xb >> 63) != 0, qx, lx);
          if (c_ssq >= 0) fx_add(flq, NS, s, false, qq, lq);
          const u32 old = atomicAdd(fcnt + s, 1u);
          if (((old + 1u) & (FX_FLUSH - 1u)) == 0u) {
            if (c_sum >= 0) atomicAdd(fex + s, fx_take(flx, NS, s, fx_bx));
            if (c_ssq >= 0) atomicAdd(feq + s, fx_take(flq, NS, s, fx_bq));
          }
        }
      }
      int cur = one_col ? 0 : -1;
      for (int c = 0; !FIXED && c < P.ncells; ++c) {
        const int op = P.cells[c].op, col = P.cells[c].col;
        if (op != OP_CNT_A && col != cur) {  // (the cells of a value column are adjacent)
          cur = col;
#pragma unroll
          for (int j = 0; j < RPA_BATCH; ++j) {
            const i64 i = base + (i64)j * blockDim.x + threadIdx.x;
            vals[j] = i < hi ? __ldg(B.src.rec + (i64)(1 + col) * B.src.cap + i) : 0ull;
          }
        }
        u64* cell = scells + (size_t)c * NS;
        u32 ok = 0;  // records of the batch that update this cell
#pragma unroll
        for (int j = 0; j < RPA_BATCH; ++j)
          if (slots[j] >= 0 && (op == OP_CNT_A || ((vbits[j] >> col) & 1ull))) ok |= 1u << j;
#define B2_RPA_APPLY(EXPR)                                                        \
        _Pragma("unroll") for (int j = 0; j < RPA_BATCH; ++j)                     \
          if ((ok >> j) & 1u) { u64* p = cell + slots[j]; const u64 v = vals[j]; EXPR; }
        // 64-bit shared-memory atomics run as compare-and-swap loops; what can be said in 32 bits is:
        // a count stays below 2^32 inside a bucket; an integer sum is its low word (the add that wraps it
        // carries into the high word) — both exact; a minimum or maximum is only attempted by a value that
        // improves on what the cell holds at that moment (the cell moves one way only).
        switch (op) {
          case OP_SUM_I:
            B2_RPA_APPLY(const u32 lo = (u32)v; const u32 old = atomicAdd((u32*)p, lo);
                         const u32 hi = (u32)(v >> 32) + ((u32)(old + lo) < old ? 1u : 0u);
                         if (hi) atomicAdd((u32*)p + 1, hi))
            break;
          case OP_CNT_V: case OP_CNT_A: B2_RPA_APPLY((void)v; atomicAdd((u32*)p, 1u)) break;
          case OP_SUM_F: B2_RPA_APPLY(atomicAdd((double*)p, __longlong_as_double((i64)v))) break;
          case OP_SSQ_I: B2_RPA_APPLY(atomicAdd(p, v * v)) break;
          case OP_SSQ_F: B2_RPA_APPLY(const double d = __longlong_as_double((i64)v); atomicAdd((double*)p, d * d)) break;
          case OP_MIN_I: B2_RPA_APPLY(if ((i64)v < *(volatile i64*)p) atomicMin((i64*)p, (i64)v)) break;
          case OP_MAX_I: B2_RPA_APPLY(if ((i64)v > *(volatile i64*)p) atomicMax((i64*)p, (i64)v)) break;
          case OP_MIN_U: B2_RPA_APPLY(if (v < *(volatile u64*)p) atomicMin(p, v)) break;
          case OP_MAX_U: B2_RPA_APPLY(if (v > *(volatile u64*)p) atomicMax(p, v)) break;
          case OP_MIN_F: B2_RPA_APPLY(const u64 o = f64_ordered(v); if (o < *(volatile u64*)p) atomicMin(p, o)) break;
          case OP_MAX_F: B2_RPA_APPLY(const u64 o = f64_ordered(v); if (o > *(volatile u64*)p) atomicMax(p, o)) break;
          default: B2_RPA_APPLY(cell_update(p, op, v)) break;  // products: compare-and-swap loops
        }
#undef B2_RPA_APPLY
      }
    }
    __syncthreads();
    if (s_fail) { if (threadIdx.x == 0) ctrl->overflow = 1; continue; }
    // compact the occupied slots into the group list
    const u32 ngroups = s_count + s_special;
    if (threadIdx.x == 0) {
      s_outbase = atomicAdd(&ctrl->out_cursor, (u64)ngroups);
      if (s_outbase + ngroups > (u64)B.out_cap) ctrl->overflow = 1;
    }
    __syncthreads();
    if (s_outbase + ngroups > (u64)B.out_cap) continue;
    for (u32 pos = threadIdx.x; pos < ngroups; pos += blockDim.x) {
      const int i = pos < s_count ? (int)sidx[pos] : S;  // (the special slot, if used, comes last)
      const i64 g = (i64)s_outbase + pos;
      B.out[g] = i < S ? skeys[i] : EMPTY;
      if (FIXED) {
        if (c_cnt >= 0) B.out[(i64)(1 + c_cnt) * B.out_cap + g] = (u64)fcnt[i];
        if (c_sum >= 0) B.out[(i64)(1 + c_sum) * B.out_cap + g] = (u64)__double_as_longlong(fex[i] + fx_take(flx, NS, i, fx_bx));
        if (c_ssq >= 0) B.out[(i64)(1 + c_ssq) * B.out_cap + g] = (u64)__double_as_longlong(feq[i] + fx_take(flq, NS, i, fx_bq));
      } else {
        for (int c = 0; c < P.ncells; ++c) B.out[(i64)(1 + c) * B.out_cap + g] = scells[(size_t)c * NS + i];
      }
    }
  }
}

// group list -> output columns
__global__ void __launch_bounds__(256) k_finalize_records(const __grid_constant__ DPlan P, const __grid_constant__ DOutPlan O,
                                                          const u64* __restrict__ groups, i64 cap, i64 ngroups)
{
  for (i64 g = (i64)blockIdx.x * blockDim.x + threadIdx.x; g < ngroups; g += (i64)gridDim.x * blockDim.x)
    write_group(P, O, groups[g], groups + cap + g, cap, g);
}

}  // namespace b2
