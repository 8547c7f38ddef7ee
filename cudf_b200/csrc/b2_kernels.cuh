// b2_kernels.cuh — the CUDA kernels of the groupby engine (sm_100a).
//
//   k_table_init     identity-fills a table with linear 16-byte stores (replaces the per-column
//                    thrust::fill of cpp/src/aggregation/aggregation.cu:87-97 and the cuco slot memset)
//   k_aggregate      ONE fused pass over keys + values + bitmasks: a per-CTA shared-memory table
//                    (direct-indexed key box sampled in the kernel, or a 2-probe hashed cache) in
//                    front of the global-memory table
//                    (replaces mapping_indices_kernel + single_pass_shmem_aggs_kernel +
//                    the global-memory functors: cpp/src/groupby/hash/compute_mapping_indices.cuh:92-151,
//                    compute_shared_memory_aggs.cu:260-353, single_pass_functors.cuh:86-157)
//   k_hll            HyperLogLog pass over the key columns: sizes the table after the small
//                    speculative one overflowed (the reference sizes by rows: compute_groupby.cu:93-102)
//   k_finalize       compaction of occupied slots + key decode + compound finalisers + result
//                    null masks in one pass (replaces retrieve_all, key gather, binary DIV,
//                    m2/var/std tabulate and null-count kernels: output_utils.cu:139-224,
//                    hash_compound_agg_finalizer.cu:93-186, common/m2_var_std.cu:49-59,160-187)
//   k_gather_fixed, k_string_lengths, k_scan_*, k_string_copy
//                    key gather for row-keyed tables (fixed width and strings)
//   k_pack_* / k_merge / k_merge_chunks
//                    hash partition of partial records by owner and merge of partial records
//                    (cpp/src/partitioning/partitioning.cu:120-337, streaming_groupby/merge.cu:91-142)
//   k_partition_count / k_partition_scatter, k_mask_to_bytes / k_bytes_to_mask
//                    row-level hash partition of a table (cudf::hash_partition) and the validity
//                    conversions a row exchange needs
#pragma once
#include "b2_device.cuh"
#include <type_traits>

namespace b2 {

constexpr int AGG_BLOCK      = 1024;  // threads per CTA of the fused kernel (one CTA per SM)
constexpr int LEAN_ROWS      = 4;     // rows per thread per tile of k_aggregate_lean (1024 threads; 512 measured
                                      // 1.6x slower: too few warps to cover the shared-memory atomics' latency)
constexpr int AGG_ROWS       = 4;     // rows per thread per tile
// The shared-memory table is a cache: a key that finds neither itself nor a free slot within
// SMEM_PROBES slots of its home goes to the global table, and the CTA's merge adds both parts up.
// A short limit keeps warps converged: with 48 probes and a 75 % fill every lookup of an uncached key
// walked a long cluster while the other 31 lanes waited (125M Zipf rows: 21.7 ms; limit 2: 8.0 ms).
constexpr int SMEM_PROBES    = 2;
constexpr double SMEM_FILL   = 0.9;   // the table takes no new keys beyond this fill
constexpr int GMEM_PROBES    = 2048;  // probe limit of the global table before "overflow"
constexpr u32 F32_SPILL_AT   = 1024;  // packed {f32 sum, u32 n} cells spill to fp64 at this count
constexpr int SLOT_NONE      = -1;

enum SmemLayout : int { SL_NONE = 0, SL_GENERIC = 1, SL_F32MEAN = 2 };

// ------------------------------------------------------------------------------ float sums as fixed-point limbs
// 64-bit shared-memory atomics (fp64 adds among them) run as compare-and-swap loops: measured 420 G adds/s
// per GPU on spread-out addresses and 33 G/s when an eighth of them hit one slot (hot keys), against 2.2 T/s
// and 1.2 T/s for native 32-bit adds.  The partitioned path therefore keeps Σx and Σx² of a float column as
// FX_LIMBS signed 32-bit words per slot, word i counting units of 2^(B - 1075 + 18 i): a value's 53-bit
// mantissa, shifted to its place, is cut into at most four 18-bit pieces and each piece is added to its word
// with one native atomic.  The pieces add up exactly; nothing is rounded until a slot is emptied (fx_take),
// which turns its words into one double.  Every FX_FLUSH-th addend of a slot empties it, so that no word
// overflows.  B comes from the largest magnitude among sampled rows: a value whose bits do not fit the
// 108-bit window (zero fits; denormals, infinities, NaN and values more than 2^FX_HEADROOM above or about
// 2^47 below the sampled maximum do not) is added to an fp64 cell instead, so the result does not depend
// on the sample — only the speed does.
constexpr int FX_LIMB_BITS = 18;
constexpr int FX_LIMBS     = 6;
constexpr int FX_MAX_SHIFT = FX_LIMB_BITS * (FX_LIMBS - 4) + FX_LIMB_BITS - 1;  // 53: four pieces end in the last word
constexpr int FX_HEADROOM  = 6;     // the window reaches 2^6 above the sampled maximum
// addends of a slot between flushes.  A word holds 2^13 pieces of 18 bits; every thread that takes a multiple of
// FX_FLUSH empties the slot before it adds anything else, so what can pile up beyond FX_FLUSH is what the other
// threads of the CTA add meanwhile: the lean kernel's tile ring lets them run at most two tiles (7936 rows)
// ahead of a stalled warp only if that warp stalls for microseconds; 1024 + 7167 is the room there is.
constexpr u32 FX_FLUSH     = 1024;
constexpr int FX_NEVER     = 1 << 20;  // window base with which no value fits (nothing was sampled)

// pieces of |x| in units of 2^(B - 1075), piece i for word q + i; false when x does not fit the window that
// starts at B.  32-bit arithmetic throughout: the mantissa as chunks of 18 + 18 + 17 bits, shifted by r < 18.
__device__ __forceinline__ bool fx_split(u64 bits, int B, int& q, u32 (&l)[4])
{
  const u32 lo = (u32)bits, hi = (u32)(bits >> 32);
  const int e = (int)((hi >> 20) & 0x7FFu);
  if (e == 0) {  // zero adds nothing; denormals go the slow way
    q = 0; l[0] = l[1] = l[2] = l[3] = 0;
    return (bits << 1) == 0;
  }
  const int shift = e - B;
  if (e == 0x7FF || shift < 0 || shift > FX_MAX_SHIFT) return false;
  q = (shift * 57) >> 10;  // shift / 18 for 0 <= shift < 64
  const int r = shift - FX_LIMB_BITS * q, rr = FX_LIMB_BITS - r;  // 1 <= rr <= 18
  const u32 m0 = lo & 0x3FFFFu;
  const u32 m1 = __funnelshift_r(lo, hi, 18) & 0x3FFFFu;
  const u32 m2 = ((hi & 0xFFFFFu) | 0x100000u) >> 4;
  l[0] = (m0 << r) & 0x3FFFFu;
  l[1] = ((m1 << r) | (m0 >> rr)) & 0x3FFFFu;
  l[2] = ((m2 << r) | (m1 >> rr)) & 0x3FFFFu;
  l[3] = m2 >> rr;
  return true;
}
// (the limb arrays live in shared memory: 32-bit shared addresses and reductions that return nothing)
// (`limbs_saddr`: the shared-memory address of word 0 of slot 0)
__device__ __forceinline__ void fx_add_s(u32 limbs_saddr, int ns, int slot, bool neg, int q, const u32 (&l)[4])
{
  const u32 base = limbs_saddr + 4u * (u32)(q * ns + slot);
#pragma unroll
  for (int i = 0; i < 4; ++i)
    if (l[i]) {
      const int v = neg ? -(int)l[i] : (int)l[i];
      asm volatile("red.shared.add.s32 [%0], %1;" ::"r"(base + 4u * (u32)(i * ns)), "r"(v) : "memory");
    }
}
__device__ __forceinline__ void fx_add(int* limbs, int ns, int slot, bool neg, int q, const u32 (&l)[4])
{
  fx_add_s((u32)__cvta_generic_to_shared(limbs), ns, slot, neg, q, l);
}
// empties the limbs of one slot and returns their value
__device__ __noinline__ double fx_take(int* limbs, int ns, int slot, int B)
{
  double acc = 0.0;
  for (int i = FX_LIMBS - 1; i >= 0; --i) acc = acc * 262144.0 + (double)atomicExch(limbs + (size_t)i * ns + slot, 0);
  return acc == 0.0 ? 0.0 : ldexp(acc, B - 1075);
}

// ------------------------------------------------------------------------------ table init
__device__ __forceinline__ void sample_dense_box(const DPlan& P, u32 cap_slots, u32 cap_lean, DDense* out);

// Must be launched with TABLE_INIT_BLOCK threads per CTA.  With `cap_dense` > 0 the last CTA also
// samples the key box of the fused kernels that follow on the stream (sample_dense_box) into the
// control block: one CTA's 1024 reads here instead of the same 1024 reads by every CTA of the fused
// kernel (148 CTAs queueing on the same sectors cost 6.5 us of that kernel).  `cap_lean` > 0: a lean kernel
// follows whose table holds fewer slots than the generic kernel's `cap_dense`.
constexpr int TABLE_INIT_BLOCK = 256;
__global__ void __launch_bounds__(TABLE_INIT_BLOCK)
k_table_init(u64* __restrict__ tbl, i64 nslots, const __grid_constant__ DPlan P, DCtrl* ctrl, u64 claim_limit,
             u64 dense_slots = 0, u32 cap_dense = 0, u32 cap_lean = 0)
{
  const bool sampling = ctrl && cap_dense > 0;
  if (ctrl && blockIdx.x == 0 && threadIdx.x < sizeof(DCtrl) / 4) {
    // a fresh control block: all zero except the claim limit (and the key box, which the sampling CTA writes)
    u32 v = 0;
    if (threadIdx.x == offsetof(DCtrl, claim_limit) / 4) v = (u32)claim_limit;
    if (threadIdx.x == offsetof(DCtrl, claim_limit) / 4 + 1) v = (u32)(claim_limit >> 32);
    if (threadIdx.x == offsetof(DCtrl, dense_slots) / 4) v = (u32)dense_slots;
    const bool in_box = threadIdx.x >= offsetof(DCtrl, dense) / 4 && threadIdx.x < (offsetof(DCtrl, dense) + sizeof(DDense)) / 4;
    if (!(sampling && in_box)) ((u32*)ctrl)[threadIdx.x] = v;
  }
  if (sampling && blockIdx.x == gridDim.x - 1) sample_dense_box(P, cap_dense, cap_lean, &ctrl->dense);
  // the table is written as one linear run of 8-byte words, two per thread and step (16-byte stores):
  // word w belongs to cell (w mod stride) of slot (w div stride); cell 0 is the key
  __shared__ u64 s_init[MAX_CELLS + 1];
  const u32 stride = (u32)P.stride;
  if (threadIdx.x <= (u32)P.ncells) s_init[threadIdx.x] = threadIdx.x == 0 ? EMPTY : cell_identity(P.cells[threadIdx.x - 1].op);
  __syncthreads();
  const i64 nwords = nslots * (i64)stride;
  const i64 aos    = (nslots - (i64)dense_slots) * (i64)stride;  // words of the hashed region + special slot
  const i64 span   = (i64)blockDim.x * 2;
  for (i64 base = (i64)blockIdx.x * span; base < nwords; base += (i64)gridDim.x * span) {
    const u32 c0 = (u32)(base % stride);  // same for the whole CTA: one 64-bit division per step
    const i64 w  = base + 2 * (i64)threadIdx.x;
    const u32 c  = (c0 + 2u * threadIdx.x) % stride;
    const u32 c1 = c + 1u == stride ? 0u : c + 1u;
    if (w >= nwords) continue;
    // the dense region is structure-of-arrays: word r of it belongs to cell r / dense_slots
    // (the index is clamped so that a load the compiler hoists above the select stays in bounds)
    const u64 dz = dense_slots ? dense_slots : 1;
    u64 q0 = (u64)(w - aos) / dz, q1 = (u64)(w + 1 - aos) / dz;
    q0 = q0 < stride ? q0 : 0;
    q1 = q1 < stride ? q1 : 0;
    const u64 v0 = w < aos ? s_init[c] : s_init[q0];
    if (w + 1 < nwords) {
      const u64 v1 = w + 1 < aos ? s_init[c1] : s_init[q1];
      *(ulonglong2*)(tbl + w) = make_ulonglong2(v0, v1);
    } else {
      tbl[w] = v0;
    }
  }
}

// ------------------------------------------------------------------------------ probing
// Long probe chains: every 8th probe looks at the overflow flag and gives up when it is set (the table
// is over its claim limit and this attempt will be discarded); every 64th probe also publishes this
// CTA's unreported claims, so that a table that fills up within the first wave of tiles — before any
// CTA reaches its per-tile bookkeeping — is noticed.
__device__ __forceinline__ bool probe_gave_up(int p, DCtrl* ctrl, int* s_new)
{
  if ((p & 7) != 7) return false;
  if ((p & 63) == 63) {
    const int c = atomicExch(s_new, 0);
    if (c) {
      const u64 tot = atomicAdd(&ctrl->nclaimed, (u64)c) + (u64)c;
      if (tot > ctrl->claim_limit) ctrl->overflow = 1;
    }
  }
  return *(volatile u32*)&ctrl->overflow != 0;
}

// Global table, packed keys.  Returns the slot index, or -1 after setting ctrl->overflow.
__device__ __forceinline__ i64 gmem_find_insert_packed(u64* tbl, i64 cap, int stride, u64 key, u64 h,
                                                       DCtrl* ctrl, int* s_new)
{
  if (key == EMPTY) {
    if (ctrl->special_used == 0) ctrl->special_used = 1;
    return cap;
  }
  i64 idx = (i64)reduce64(h, (u64)cap);
  for (int p = 0; p < GMEM_PROBES; ++p) {
    u64* kp = tbl + idx * stride;
    u64 k   = *(volatile u64*)kp;
    if (k == key) return idx;
    if (k == EMPTY) {
      const u64 old = atomicCAS(kp, EMPTY, key);
      if (old == EMPTY) { atomicAdd(s_new, 1); return idx; }
      if (old == key) return idx;
    }
    if (probe_gave_up(p, ctrl, s_new)) return -1;
    if (++idx == cap) idx = 0;
  }
  ctrl->overflow = 1;
  return -1;
}

// Same, when the key cell of the home slot `idx` was already loaded (`k`): the loads of several rows
// are issued together so that their DRAM latencies overlap, then each row finishes here.
__device__ __forceinline__ i64 gmem_finish_packed(u64* tbl, i64 cap, int stride, u64 key, i64 idx, u64 k,
                                                  DCtrl* ctrl, int* s_new)
{
  for (int p = 0; p < GMEM_PROBES; ++p) {
    u64* kp = tbl + idx * stride;
    if (p > 0) k = *(volatile u64*)kp;
    if (k == key) return idx;
    if (k == EMPTY) {
      const u64 old = atomicCAS(kp, EMPTY, key);
      if (old == EMPTY) { atomicAdd(s_new, 1); return idx; }
      if (old == key) return idx;
    }
    if (probe_gave_up(p, ctrl, s_new)) return -1;
    if (++idx == cap) idx = 0;
  }
  ctrl->overflow = 1;
  return -1;
}

// Global table, row keys: key cell = (tag << 32) | representative row.
__device__ __forceinline__ i64 gmem_find_insert_rows(const DPlan& P, u64* tbl, i64 cap, int stride, i64 row,
                                                     u64 h, DCtrl* ctrl, int* s_new)
{
  const u64 tag  = h & 0xFFFFFFFF00000000ull;
  const u64 mine = tag | (u64)(u32)row;
  i64 idx        = (i64)reduce64(h, (u64)cap);
  for (int p = 0; p < GMEM_PROBES; ++p) {
    u64* kp = tbl + idx * stride;
    u64 k   = *(volatile u64*)kp;
    if (k == EMPTY) {
      k = atomicCAS(kp, EMPTY, mine);
      if (k == EMPTY) { atomicAdd(s_new, 1); return idx; }
    }
    if ((k & 0xFFFFFFFF00000000ull) == tag && rows_equal(P, row, (i64)(u32)k)) return idx;
    if (probe_gave_up(p, ctrl, s_new)) return -1;
    if (++idx == cap) idx = 0;
  }
  ctrl->overflow = 1;
  return -1;
}

// Shared-memory table (S slots + the special slot at index S).  Returns -1 when the key is not
// cached and may not be inserted (table closed) — the caller then goes to the global table.
template <int KM>
__device__ __forceinline__ int smem_find_insert(const DPlan& P, u64* skeys, int S, int fill_limit, int* s_fill,
                                                u64 key, u64 h, i64 row)
{
  if (KM == KM_PACKED && key == EMPTY) {
    if (skeys[S] == EMPTY) skeys[S] = 0;
    return S;
  }
  const u64 tag  = h & 0xFFFFFFFF00000000ull;
  const u64 mine = (KM == KM_PACKED) ? key : (tag | (u64)(u32)row);
  int idx        = (int)reduce32((u32)(h >> 11), (u32)S);
  for (int p = 0; p < SMEM_PROBES; ++p) {
    u64 k = *(volatile u64*)(skeys + idx);
    if (k == EMPTY) {
      if (*(volatile int*)s_fill >= fill_limit) return -1;
      k = atomicCAS(skeys + idx, EMPTY, mine);
      if (k == EMPTY) { atomicAdd(s_fill, 1); return idx; }
    }
    if (KM == KM_PACKED) {
      if (k == key) return idx;
    } else {
      if ((k & 0xFFFFFFFF00000000ull) == tag && rows_equal(P, row, (i64)(u32)k)) return idx;
    }
    if (++idx == S) idx = 0;
  }
  return -1;
}

// ------------------------------------------------------------------------------ dense key box
// ordered value of key column k inside a packed key
__device__ __forceinline__ i64 key_field(const DKeyCol& c, u64 key)
{
  u64 v = key >> c.shift;
  if (c.width < 8) {
    const int sh = 64 - 8 * c.width;
    v <<= sh;
    v = c.is_signed ? (u64)((i64)v >> sh) : (v >> sh);
  }
  return (i64)v;
}

// slot of a packed key inside the sampled box, -1 when the key lies outside it
__device__ __forceinline__ int dense_index(const DPlan& P, const DDense& D, u64 key)
{
  u32 idx = 0;
  for (int k = 0; k < P.nkeys; ++k) {
    const DKeyCol& c = P.keys[k];
    u64 f;
    if (c.nullbit >= 0 && ((key >> c.nullbit) & 1ull)) {
      f = D.range[k] - 1;
    } else {
      f = (u64)(key_field(c, key) - D.min[k]);
      if (f >= D.range[k] - (c.nullbit >= 0 ? 1ull : 0ull)) return -1;
    }
    idx += (u32)f * D.mult[k];
  }
  return (int)idx;
}

// inverse of dense_index
__device__ __forceinline__ u64 dense_key(const DPlan& P, const DDense& D, u32 idx)
{
  u64 key = 0;
  for (int k = 0; k < P.nkeys; ++k) {
    const DKeyCol& c = P.keys[k];
    const u64 f = (u64)((idx / D.mult[k]) % (u32)D.range[k]);  // ranges fit 32 bits (their product does)
    if (c.nullbit >= 0 && f == D.range[k] - 1) {
      key |= 1ull << c.nullbit;
    } else {
      const u64 v = (u64)((i64)f + D.min[k]);
      key |= (c.width == 8 ? v : (v & ((1ull << (8 * c.width)) - 1ull))) << c.shift;
    }
  }
  return key;
}

__device__ __forceinline__ void prefetch_l2(const void* p)
{
  asm volatile("prefetch.global.L2 [%0];" ::"l"(p));
}

// One CTA (the last one of k_table_init) looks at 1024 evenly spaced rows and derives the dense key
// box, or disables it when the box would not fit `cap_slots` shared-memory slots.  The fused kernels
// read the box from the control block, so there is no host round trip.  Keys outside the box are
// still aggregated correctly, through the global table.  With `cap_lean` > 0 a box of more than
// `cap_lean` slots that still fits `cap_slots` is written with enabled = 0 and its total kept: the lean
// kernel declines it, and the host enables it for the generic kernel it launches instead.  Must be called
// by all TABLE_INIT_BLOCK threads of the CTA.
constexpr int SAMPLE_ROWS = 1024;
constexpr int SAMPLE_PER_THREAD = SAMPLE_ROWS / 256;
__device__ __forceinline__ void sample_dense_box(const DPlan& P, u32 cap_slots, u32 cap_lean, DDense* out)
{
  __shared__ i64 s_min[MAX_KEYS], s_max[MAX_KEYS];
  __shared__ u32 s_vexp;
  if (threadIdx.x < MAX_KEYS) { s_min[threadIdx.x] = 0x7FFFFFFFFFFFFFFFll; s_max[threadIdx.x] = (i64)0x8000000000000000ull; }
  if (threadIdx.x == 0) s_vexp = 0;
  __syncthreads();
  const i64 nsamp  = P.nrows < SAMPLE_ROWS ? P.nrows : SAMPLE_ROWS;
  const i64 stride = P.nrows / (nsamp > 0 ? nsamp : 1);
  if (P.key_mode == KM_PACKED) {
    // Column by column, the 4 loads of a column issued together: the number of dependent DRAM round
    // trips is the number of columns and masks, not 4 x that (row-major order serialised every load
    // behind the previous one's use and cost 24 us per launch).
    i64 rows[SAMPLE_PER_THREAD];
    u32 ok = 0;  // bit j: sample j of this thread takes part
#pragma unroll
    for (int j = 0; j < SAMPLE_PER_THREAD; ++j) {
      const i64 i = (i64)threadIdx.x + (i64)j * blockDim.x;
      rows[j] = i < nsamp ? i * stride + (stride > 1 ? (i64)(((u64)i * 7919ull) % (u64)stride) : 0) : 0;
      if (i < nsamp) ok |= 1u << j;
    }
    for (int f = 0; f < P.nfilters; ++f) {
      u32 w[SAMPLE_PER_THREAD];
#pragma unroll
      for (int j = 0; j < SAMPLE_PER_THREAD; ++j) w[j] = __ldg(P.filters[f] + ((P.filter_offsets[f] + rows[j]) >> 5));
#pragma unroll
      for (int j = 0; j < SAMPLE_PER_THREAD; ++j)
        if (!((w[j] >> ((P.filter_offsets[f] + rows[j]) & 31)) & 1u)) ok &= ~(1u << j);
    }
    for (int k = 0; k < P.nkeys; ++k) {
      const DKeyCol& c = P.keys[k];
      u32 valid = (1u << SAMPLE_PER_THREAD) - 1u;
      if (c.mask) {
        u32 w[SAMPLE_PER_THREAD];
#pragma unroll
        for (int j = 0; j < SAMPLE_PER_THREAD; ++j) w[j] = __ldg(c.mask + ((c.offset + rows[j]) >> 5));
#pragma unroll
        for (int j = 0; j < SAMPLE_PER_THREAD; ++j)
          if (!((w[j] >> ((c.offset + rows[j]) & 31)) & 1u)) valid &= ~(1u << j);
        if (!P.include_nulls) ok &= valid;  // EXCLUDE: a null key drops the row (for every column)
      }
      u64 bits[SAMPLE_PER_THREAD];
#pragma unroll
      for (int j = 0; j < SAMPLE_PER_THREAD; ++j) bits[j] = load_fixed_bits(c.data, c.offset + rows[j], c.width);
      const int sh = 64 - 8 * c.width;
      i64 lo = 0x7FFFFFFFFFFFFFFFll, hi = (i64)0x8000000000000000ull;
#pragma unroll
      for (int j = 0; j < SAMPLE_PER_THREAD; ++j) {
        if (!((ok >> j) & 1u) || !((valid >> j) & 1u)) continue;
        const i64 v = c.is_signed ? ((i64)(bits[j] << sh) >> sh) : (i64)bits[j];
        lo = v < lo ? v : lo;
        hi = v > hi ? v : hi;
      }
      for (int d = 16; d > 0; d >>= 1) {
        const i64 ol = __shfl_xor_sync(0xFFFFFFFFu, lo, d), oh = __shfl_xor_sync(0xFFFFFFFFu, hi, d);
        lo = ol < lo ? ol : lo;
        hi = oh > hi ? oh : hi;
      }
      if ((threadIdx.x & 31) == 0 && lo <= hi) { atomicMin(&s_min[k], lo); atomicMax(&s_max[k], hi); }
    }
    if (P.flags & PF_F64MEAN) {
      // the largest exponent among the sampled FLOAT64 values places the window of the fixed-point limbs
      // (zeros, denormals, infinities and NaN say nothing about it; a null's payload is not looked at)
      const DValCol& vc = P.vals[P.cells[0].col];
      u64 bits[SAMPLE_PER_THREAD];
      u32 w[SAMPLE_PER_THREAD];
#pragma unroll
      for (int j = 0; j < SAMPLE_PER_THREAD; ++j) {
        bits[j] = __ldg((const u64*)vc.data + vc.offset + rows[j]);
        w[j]    = vc.mask ? __ldg(vc.mask + ((vc.offset + rows[j]) >> 5)) >> ((vc.offset + rows[j]) & 31) : 1u;
      }
      u32 emax = 0;
#pragma unroll
      for (int j = 0; j < SAMPLE_PER_THREAD; ++j) {
        const u32 e = (u32)(bits[j] >> 52) & 0x7FFu;
        if (((ok >> j) & 1u) && (w[j] & 1u) && e != 0u && e != 0x7FFu && e + 1u > emax) emax = e + 1u;
      }
      emax = __reduce_max_sync(0xFFFFFFFFu, emax);
      if ((threadIdx.x & 31) == 0 && emax) atomicMax(&s_vexp, emax);
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    DDense& D = *out;
    for (int k = 0; k < MAX_KEYS; ++k) { D.min[k] = 0; D.range[k] = 0; D.mult[k] = 0; }
    D.enabled = 0;
    D.total   = 0;
    D.copies  = 1;
    D.vexp    = s_vexp;
    bool ok   = P.key_mode == KM_PACKED && nsamp >= SAMPLE_ROWS && cap_slots > 0;
    for (int pass = 0; pass < 2 && ok && !D.enabled; ++pass) {  // pass 0: padded box, pass 1: tight box
      u64 total = 1;
      bool fits = true;
      for (int k = 0; k < P.nkeys && fits; ++k) {
        i64 lo = s_min[k], hi = s_max[k];
        if (lo > hi) { lo = 0; hi = 0; }
        const u64 span = (u64)(hi - lo);
        if (span >= (u64)cap_slots) { fits = false; break; }
        u64 pad = pass == 0 ? (span / 8 + 1 < 64 ? span / 8 + 1 : 64) : 0;
        if (lo < (i64)0x8000000000000000ull + (i64)pad || hi > 0x7FFFFFFFFFFFFFFFll - (i64)pad) pad = 0;
        D.min[k]   = lo - (i64)pad;
        D.range[k] = span + 1 + 2 * pad + (P.keys[k].nullbit >= 0 ? 1 : 0);
        D.mult[k]  = (u32)total;
        total *= D.range[k];
        if (total > (u64)cap_slots) fits = false;
      }
      if (fits) {
        const bool lean_too = cap_lean == 0 || total <= (u64)cap_lean;
        D.enabled = lean_too ? 1 : 0;
        D.total   = (u32)total;
        const u32 r = (cap_lean != 0 && lean_too ? cap_lean : cap_slots) / (u32)total;
        D.copies  = r < 1 ? 1u : (r > 32u ? 32u : r);
        // (a padded box that only the generic table holds: the tight one may still fit the lean table)
      }
    }
  }
  __syncthreads();
}

// shared-memory atomics on 32-bit shared addresses (native on sm_100a; measured at ~73 % of the
// HBM roofline for one float add + one count add per row into a direct-indexed table)
__device__ __forceinline__ void sred_add_f32(u32 saddr, float v)
{
  asm volatile("red.shared.add.f32 [%0], %1;" ::"r"(saddr), "f"(v) : "memory");
}
__device__ __forceinline__ u32 satom_add_u32(u32 saddr, u32 v)
{
  u32 old;
  asm volatile("atom.shared.add.u32 %0, [%1], %2;" : "=r"(old) : "r"(saddr), "r"(v) : "memory");
  return old;
}
// 4 validity bits at a position that is a multiple of 4
__device__ __forceinline__ u32 nibble_aligned(const u32* mask, u32 pos)
{
  return (__ldg(mask + (pos >> 5)) >> (pos & 31u)) & 0xFu;
}

// ------------------------------------------------------------------------------ fused aggregate
// ONE pass over keys + values + bitmasks.  Each thread takes 4 consecutive rows per tile (16-byte
// vector loads when the columns allow, validity read as 4-bit nibbles of the mask words).  Each CTA
// owns a shared-memory table in front of the global table:
//   dense mode  : slot = position of the key in the sampled key box (sample_dense_box), accumulators
//                 only, no probing;
//   hashed mode : open addressing with linear probing on the 64-bit key cell, first come first
//                 cached until `fill_limit`; a CTA whose cache stops paying off turns it off.
// Rows whose key is not in shared memory go to the global table with global atomics.  At the end
// every CTA merges its table into the global one.  There is no barrier inside the row loop.
__device__ __forceinline__ u64 global_timer_ns()
{
  u64 t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

template <int KM, int LAYOUT>
__global__ void __launch_bounds__(AGG_BLOCK, 1)
k_aggregate(const __grid_constant__ DPlan P, u64* __restrict__ tbl, i64 cap, DCtrl* ctrl, int S_hash, int fill_limit,
            u32 cap_dense, u32 region_slots, int lean_first)
{
  extern __shared__ __align__(128) unsigned char smem_raw[];
  __shared__ int s_fill, s_new, s_cache_on, s_abort, s_hit, s_miss;
  __shared__ DDense s_dense;

  const int stride = P.stride;
  const int tid    = threadIdx.x;
  const i64 dense_slots = (i64)region_slots;  // structure-of-arrays slots behind the special slot
  const bool timekeeper = blockIdx.x == 0 && tid == 0;
  const u64 t_start = timekeeper ? global_timer_ns() : 0;
  if (LAYOUT != SL_NONE && KM == KM_PACKED && cap_dense > 0) {
    // the key box sampled by k_table_init, which precedes this kernel on the stream
    for (int i = tid; i < (int)(sizeof(DDense) / 4); i += blockDim.x) ((u32*)&s_dense)[i] = ((const u32*)&ctrl->dense)[i];
  } else if (tid == 0) {
    s_dense.enabled = 0;
  }
  if (tid == 0) { s_fill = 0; s_new = 0; s_cache_on = (LAYOUT != SL_NONE); s_abort = 0; s_hit = 0; s_miss = 0; }
  __syncthreads();
  // k_aggregate_lean ran in front of this kernel and, having found a key box, took the whole input
  if (lean_first && s_dense.enabled) return;
  if (timekeeper) { ctrl->t_phase[0] = t_start; ctrl->t_phase[1] = global_timer_ns(); }
  const bool dense = (LAYOUT != SL_NONE) && KM == KM_PACKED && s_dense.enabled;
  const int S      = dense ? (int)s_dense.total : S_hash;  // slots (hashed mode: + the special slot at S)
  const int NS     = dense ? S * (int)s_dense.copies : S + 1;  // allocated slots per array
  // dense mode: this warp's replica of the table
  const u32 copy_off = dense ? (u32)((threadIdx.x >> 5) % s_dense.copies) * (u32)S : 0u;
  // global slot of dense-box position i: the dense region behind the special slot (the one key whose
  // bits equal EMPTY cannot mark a key cell as used and goes to the special slot instead)
  auto dense_gslot = [&](u32 i) -> i64 { return dense_key(P, s_dense, i) == EMPTY ? cap : cap + 1 + (i64)i; };

  // shared-memory arrays
  u64* skeys  = (u64*)smem_raw;                            // hashed mode only: [NS]
  u64* scells = dense ? (u64*)smem_raw : skeys + NS;       // SL_GENERIC: [ncells][NS]
  float* ssum = (float*)scells;                            // SL_F32MEAN: [NS] fp32 partial sums
  u32* scnt   = (u32*)(ssum + NS);                         // SL_F32MEAN: [NS] counts
  u32* socc   = (u32*)(scells + (size_t)(LAYOUT == SL_F32MEAN ? 1 : P.ncells) * NS);  // dense mode: occupancy bits
  if (LAYOUT != SL_NONE) {
    if (!dense) for (int i = tid; i < NS; i += blockDim.x) skeys[i] = EMPTY;
    if (LAYOUT == SL_GENERIC) {
      for (int c = 0; c < P.ncells; ++c) {
        const u64 id = cell_identity(P.cells[c].op);
        for (int i = tid; i < NS; i += blockDim.x) scells[(size_t)c * NS + i] = id;
      }
    } else {
      for (int i = tid; i < NS; i += blockDim.x) scells[i] = 0;  // {sum, count} arrays together
    }
    if (dense) for (int i = tid; i < (NS + 31) / 32; i += blockDim.x) socc[i] = 0;
  }
  __syncthreads();
  if (timekeeper) ctrl->t_phase[2] = global_timer_ns();

  u32 my_hit = 0, my_miss = 0, tot_hit = 0, tot_miss = 0;
  const i64 rows_done = 0;

  const i64 tile_rows = (i64)blockDim.x * AGG_ROWS;
  const i64 ntiles    = (P.nrows - rows_done + tile_rows - 1) / tile_rows;

  for (i64 tile = blockIdx.x; tile < ntiles; tile += gridDim.x) {
    if (*(volatile int*)&s_abort) break;
    const i64 row0 = rows_done + tile * tile_rows + (i64)tid * AGG_ROWS;
    const int nv   = (int)max((i64)0, min((i64)AGG_ROWS, P.nrows - row0));
    const bool cache_on = (LAYOUT != SL_NONE) && (dense || *(volatile int*)&s_cache_on);

    // ---- loads first, all independent of each other, so that one DRAM round trip covers the tile
    const bool full = nv == AGG_ROWS;
    const bool vec  = KM == KM_PACKED && full && (P.flags & PF_VEC_KEYS);
    u32 act = nv > 0 ? ((1u << nv) - 1u) : 0u;
    int sl[AGG_ROWS];
    u64 kk[AGG_ROWS];
    u32 di[AGG_ROWS];   // dense mode: slot inside the key box
    u32 dout = 0;       // dense mode: rows whose key lies outside the box
#pragma unroll
    for (int j = 0; j < AGG_ROWS; ++j) { sl[j] = SLOT_NONE; kk[j] = 0; di[j] = copy_off; }
    float fx[AGG_ROWS] = {0.f, 0.f, 0.f, 0.f};  // SL_F32MEAN: the values
    u32 fvn = 0xFu;                              // SL_F32MEAN: their validity
    if (LAYOUT == SL_F32MEAN && full && (P.flags & PF_VEC_VAL0)) {
      const DValCol& vc = P.vals[P.cells[0].col];
      const float4 q = __ldg((const float4*)((const float*)vc.data + vc.offset + row0));
      fx[0] = q.x; fx[1] = q.y; fx[2] = q.z; fx[3] = q.w;
      if (vc.mask) fvn = valid_nibble(vc.mask, vc.offset + row0, nv);
    }
    if (vec) {
      for (int k = 0; k < P.nkeys; ++k) {
        const DKeyCol& c = P.keys[k];
        const unsigned char* src = c.data + (c.offset + row0) * c.width;
        u64 f[AGG_ROWS];
        if (c.width == 4) {
          const uint4 q = __ldg((const uint4*)src);
          f[0] = q.x; f[1] = q.y; f[2] = q.z; f[3] = q.w;
        } else if (c.width == 8) {
          const ulonglong2 q0 = __ldg((const ulonglong2*)src), q1 = __ldg((const ulonglong2*)src + 1);
          f[0] = q0.x; f[1] = q0.y; f[2] = q1.x; f[3] = q1.y;
        } else if (c.width == 2) {
          const uint2 q = __ldg((const uint2*)src);
          f[0] = q.x & 0xFFFFu; f[1] = q.x >> 16; f[2] = q.y & 0xFFFFu; f[3] = q.y >> 16;
        } else {
          const u32 q = __ldg((const u32*)src);
          f[0] = q & 0xFFu; f[1] = (q >> 8) & 0xFFu; f[2] = (q >> 16) & 0xFFu; f[3] = q >> 24;
        }
        u32 vn = 0xFu;
        if (c.mask) {
          vn = valid_nibble(c.mask, c.offset + row0, nv);
          if (!P.include_nulls) act &= vn;  // EXCLUDE: a null key drops the row
        }
        const int sh = 64 - 8 * c.width;
#pragma unroll
        for (int j = 0; j < AGG_ROWS; ++j) {
          const bool isnull = c.nullbit >= 0 && !((vn >> j) & 1u);
          kk[j] |= isnull ? (1ull << c.nullbit) : (f[j] << c.shift);
          if (dense) {
            const i64 ov = c.is_signed ? ((i64)(f[j] << sh) >> sh) : (i64)f[j];
            u64 d = (u64)(ov - s_dense.min[k]);
            const u64 lim = s_dense.range[k] - (c.nullbit >= 0 ? 1ull : 0ull);
            if (isnull) d = lim;
            else if (d >= lim) dout |= 1u << j;
            di[j] += (u32)d * s_dense.mult[k];
          }
        }
      }
    } else if (act && !P.include_nulls) {
      for (int k = 0; k < P.nkeys; ++k)
        if (P.keys[k].mask) act &= valid_nibble(P.keys[k].mask, P.keys[k].offset + row0, nv);
    }
    if (act)
      for (int f = 0; f < P.nfilters; ++f) act &= valid_nibble(P.filters[f], P.filter_offsets[f] + row0, nv);

    // ---- phase A: keys -> slots
    if (act) {
      if (!vec) {
#pragma unroll
        for (int j = 0; j < AGG_ROWS; ++j)
          if ((act >> j) & 1u) {
            kk[j] = (KM == KM_PACKED) ? pack_key(P, row0 + j) : hash_row(P, row0 + j);
            if (dense) {
              const int s = dense_index(P, s_dense, kk[j]);
              if (s < 0) dout |= 1u << j; else di[j] = copy_off + (u32)s;
            }
          }
      }
      // shared-memory table first
      u32 miss = 0;
      u64 hh[AGG_ROWS];
#pragma unroll
      for (int j = 0; j < AGG_ROWS; ++j) {
        hh[j] = 0;
        if (!((act >> j) & 1u)) continue;
        int s = -1;
        if (dense) {
          if (!((dout >> j) & 1u)) {
            s = (int)di[j];
            if (!((socc[s >> 5] >> (s & 31)) & 1u)) atomicOr(&socc[s >> 5], 1u << (s & 31));
          }
        } else {
          hh[j] = (KM == KM_PACKED) ? mix64(kk[j]) : kk[j];
          if (cache_on) s = smem_find_insert<KM>(P, skeys, S, fill_limit, &s_fill, kk[j], hh[j], row0 + j);
        }
        if (s >= 0) {
          sl[j] = s;
          ++my_hit;
        } else {
          if (dense) hh[j] = mix64(kk[j]);
          miss |= 1u << j;
          ++my_miss;
        }
      }
      // then the global table: the home slots of all my missing rows are loaded together (their
      // DRAM latencies overlap), then each row finishes its probe sequence
      if (miss) {
        if (KM == KM_PACKED) {
          i64 gi[AGG_ROWS];
          u64 gk[AGG_ROWS];
#pragma unroll
          for (int j = 0; j < AGG_ROWS; ++j) {
            gi[j] = (i64)reduce64(hh[j], (u64)cap);
            gk[j] = 0;
            if (((miss >> j) & 1u) && kk[j] != EMPTY) gk[j] = *(volatile u64*)(tbl + gi[j] * stride);
          }
#pragma unroll
          for (int j = 0; j < AGG_ROWS; ++j) {
            if (!((miss >> j) & 1u)) continue;
            i64 g;
            if (kk[j] == EMPTY) {
              if (ctrl->special_used == 0) ctrl->special_used = 1;
              g = cap;
            } else {
              g = gmem_finish_packed(tbl, cap, stride, kk[j], gi[j], gk[j], ctrl, &s_new);
            }
            if (g >= 0) sl[j] = -2 - (int)g;
          }
        } else {
#pragma unroll
          for (int j = 0; j < AGG_ROWS; ++j) {
            if (!((miss >> j) & 1u)) continue;
            const i64 g = gmem_find_insert_rows(P, tbl, cap, stride, row0 + j, hh[j], ctrl, &s_new);
            if (g >= 0) sl[j] = -2 - (int)g;
          }
        }
      }
    }
    __syncwarp();  // reconverge after the divergent probe loops before the accumulate phase

    // ---- phase B: fold the values
    if (LAYOUT == SL_F32MEAN) {
      // cells: [0] = Σx of a FLOAT32 column, [1] = n of the same column
      const DValCol& vc = P.vals[P.cells[0].col];
      if (act) {
        u32 vn = act;
        float x[AGG_ROWS];
        if (full && (P.flags & PF_VEC_VAL0)) {
          vn &= fvn;
#pragma unroll
          for (int j = 0; j < AGG_ROWS; ++j) x[j] = fx[j];
        } else {
          if (vc.mask) vn &= valid_nibble(vc.mask, vc.offset + row0, nv);
#pragma unroll
          for (int j = 0; j < AGG_ROWS; ++j) x[j] = ((vn >> j) & 1u) ? __ldg((const float*)vc.data + vc.offset + row0 + j) : 0.f;
        }
#pragma unroll
        for (int j = 0; j < AGG_ROWS; ++j) {
          if (sl[j] == SLOT_NONE || !((vn >> j) & 1u)) continue;
          if (sl[j] >= 0) {
            atomicAdd(ssum + sl[j], x[j]);
            const u32 old = atomicAdd(scnt + sl[j], 1u);
            if (((old + 1u) & (F32_SPILL_AT - 1u)) == 0u) {
              // every F32_SPILL_AT-th addend moves the fp32 partial of this key to the fp64 global
              // cell, so that no fp32 sum ever holds many more addends than that
              const float part = atomicExch(ssum + sl[j], 0.f);
              i64 g;
              if (dense) {
                g = dense_gslot((u32)sl[j] - copy_off);
              } else {
                const u64 key = sl[j] == S ? EMPTY : skeys[sl[j]];
                g = gmem_find_insert_packed(tbl, cap, stride, key, mix64(key), ctrl, &s_new);
              }
              if (g >= 0) atomicAdd((double*)slot_ref(tbl, cap, stride, dense_slots, g).cells, (double)part);
            }
          } else {
            u64* slot = tbl + (i64)(-2 - sl[j]) * stride;
            atomicAdd((double*)(slot + 1), (double)x[j]);
            atomicAdd(slot + 2, 1ull);
          }
        }
      }
    } else {
      int cur_col = -1;
      u64 v[AGG_ROWS];
      u32 vn = 0;
      for (int c = 0; c < P.ncells; ++c) {
        const int op  = P.cells[c].op;
        const int col = P.cells[c].col;
        if (op != OP_CNT_A && col != cur_col) {
          cur_col = col;
          const DValCol& vc = P.vals[col];
          vn = act;
          if (vn && vc.mask) vn &= valid_nibble(vc.mask, vc.offset + row0, nv);
#pragma unroll
          for (int j = 0; j < AGG_ROWS; ++j) v[j] = ((vn >> j) & 1u) && sl[j] != SLOT_NONE ? load_value(vc, row0 + j) : 0;
        }
        const u32 use = (op == OP_CNT_A) ? act : vn;
#pragma unroll
        for (int j = 0; j < AGG_ROWS; ++j) {
          if (sl[j] == SLOT_NONE || !((use >> j) & 1u)) continue;
          // two call sites so that each atomic knows its address space (shared vs global reduction)
          if (is_arg_op(op)) arg_update(tbl + (i64)(-2 - sl[j]) * stride + 1 + c, op, P.vals[col], row0 + j);  // (global table only)
          else if (LAYOUT == SL_GENERIC && sl[j] >= 0) cell_update(scells + (size_t)c * NS + sl[j], op, v[j]);
          else {
            const SlotRef slot = slot_ref(tbl, cap, stride, dense_slots, (i64)(-2 - sl[j]));
            cell_update(slot.cells + (i64)c * slot.step, op, v[j]);
          }
        }
      }
    }

    // ---- bookkeeping by one lane per CTA, no barrier: claims, overflow, cache pay-off
    if (LAYOUT != SL_NONE && !dense) {
      const u32 wh = __reduce_add_sync(0xFFFFFFFFu, my_hit), wm = __reduce_add_sync(0xFFFFFFFFu, my_miss);
      if ((tid & 31) == 0) { if (wh) atomicAdd(&s_hit, (int)wh); if (wm) atomicAdd(&s_miss, (int)wm); }
      tot_hit += my_hit; tot_miss += my_miss;
      my_hit = 0; my_miss = 0;
    }
    if (tid == 0) {
      const int c = atomicExch(&s_new, 0);
      if (c) {
        const u64 tot = atomicAdd(&ctrl->nclaimed, (u64)c) + (u64)c;
        if (tot > ctrl->claim_limit) ctrl->overflow = 1;
      }
      if (*(volatile u32*)&ctrl->overflow) s_abort = 1;
      if (LAYOUT != SL_NONE && !dense && s_cache_on && s_fill >= fill_limit) {
        const int h = atomicExch(&s_hit, 0), m = atomicExch(&s_miss, 0);
        if (m > 3 * h && m > 1024) s_cache_on = 0;
      }
    }
  }

  // ---- statistics: rows folded in shared memory / sent to the global table
  tot_hit  = __reduce_add_sync(0xFFFFFFFFu, tot_hit + my_hit);
  tot_miss = __reduce_add_sync(0xFFFFFFFFu, tot_miss + my_miss);
  if ((tid & 31) == 0) {
    if (tot_hit) atomicAdd(&ctrl->stat_smem_rows, (u64)tot_hit);
    if (tot_miss) atomicAdd(&ctrl->stat_gmem_rows, (u64)tot_miss);
  }

  // ---- merge this CTA's table into the global table
  __syncthreads();
  if (timekeeper) ctrl->t_phase[3] = global_timer_ns();
  if (LAYOUT != SL_NONE && !s_abort) {
    // CTAs start their merge at different slots so that they do not all hit the same global cells at once
    const int NM  = dense ? S : NS;  // dense mode: one pass over box positions, replicas reduced on the fly
    const int rot = (int)(((u64)blockIdx.x * 2654435761ull) % (u64)NM);
    int dense_new = 0;  // dense-region key cells this thread was the first to claim
    if (dense) {
      // Dense mode: the replicas of a box position are reduced in registers, then ONE merge into the
      // dense region of the global table: no hashing, consecutive threads -> consecutive words of the
      // structure-of-arrays region.  The key cell is claimed with an unconditional exchange (every
      // CTA writes the same key there).  Four positions per step: their exchanges and reductions are
      // all issued before the first returned key is looked at, so a step waits for one L2 round trip
      // instead of four (one position per step: 21 us for 15.9K positions).
      constexpr int MB = 4;
      const int copies = (int)s_dense.copies;
      for (int base = tid; base < NM; base += MB * (int)blockDim.x) {
        u64 olds[MB];
#pragma unroll
        for (int u = 0; u < MB; ++u) {
          olds[u] = 0;  // anything but EMPTY: "not newly claimed"
          const int i0 = base + u * (int)blockDim.x;
          if (i0 >= NM) continue;
          const int i = i0 + rot < NM ? i0 + rot : i0 + rot - NM;
          bool present = false;
          for (int r = 0; r < copies; ++r) {
            const int q = r * S + i;
            present = present || ((socc[q >> 5] >> (q & 31)) & 1u) || (LAYOUT == SL_F32MEAN && scnt[q] != 0u);
          }
          if (!present) continue;
          const u64 key = dense_key(P, s_dense, (u32)i);
          i64 g;
          if (key == EMPTY) {
            g = cap;
            if (ctrl->special_used == 0) ctrl->special_used = 1;
          } else {
            g = cap + 1 + (i64)i;
          }
          const SlotRef slot = slot_ref(tbl, cap, stride, dense_slots, g);
          if (key != EMPTY) olds[u] = atomicExch(slot.key, key);
          if (LAYOUT == SL_F32MEAN) {
            double sum = 0.0;
            u64 n = 0;
            for (int r = 0; r < copies; ++r) { sum += (double)ssum[r * S + i]; n += scnt[r * S + i]; }
            if (n) { atomicAdd((double*)slot.cells, sum); atomicAdd(slot.cells + slot.step, n); }
          } else {
            for (int c = 0; c < P.ncells; ++c) {
              const int op = P.cells[c].op;
              u64 a = cell_identity(op);
              for (int r = 0; r < copies; ++r) a = cell_combine(op, a, scells[(size_t)c * NS + r * S + i]);
              if (a != cell_identity(op)) cell_merge(slot.cells + (i64)c * slot.step, op, a);
            }
          }
        }
#pragma unroll
        for (int u = 0; u < MB; ++u) dense_new += olds[u] == EMPTY ? 1 : 0;
      }
    }
    for (int i0 = tid; !dense && i0 < NM; i0 += blockDim.x) {
      const int i = i0 + rot < NM ? i0 + rot : i0 + rot - NM;
      u64 key = skeys[i];
      if (key == EMPTY) continue;
      if (i == S) key = EMPTY;  // the special slot holds the key whose bits equal EMPTY
      i64 g;
      if (KM == KM_PACKED) {
        g = gmem_find_insert_packed(tbl, cap, stride, key, mix64(key), ctrl, &s_new);
      } else {
        const i64 row = (i64)(u32)key;
        g = gmem_find_insert_rows(P, tbl, cap, stride, row, hash_row(P, row), ctrl, &s_new);
      }
      if (g < 0) continue;
      u64* slot = tbl + g * stride;
      if (LAYOUT == SL_F32MEAN) {
        const u32 n = scnt[i];
        if (n) {
          atomicAdd((double*)(slot + 1), (double)ssum[i]);
          atomicAdd(slot + 2, (u64)n);
        }
      } else {
        for (int c = 0; c < P.ncells; ++c) {
          const int op = P.cells[c].op;
          const u64 a  = scells[(size_t)c * NS + i];
          if (a != cell_identity(op)) cell_merge(slot + 1 + c, op, a);
        }
      }
    }
    if (dense_new) atomicAdd(&s_new, dense_new);
  }
  __syncthreads();
  if (tid == 0) {
    if (s_new) {
      const u64 tot = atomicAdd(&ctrl->nclaimed, (u64)s_new) + (u64)s_new;
      if (tot > ctrl->claim_limit) ctrl->overflow = 1;
    }
    if (timekeeper) ctrl->t_phase[4] = global_timer_ns();
  }
}

// ------------------------------------------------------------------------------ cardinality estimate
// HyperLogLog over the keys of all participating rows (one streaming pass over the key columns):
// 2^13 registers, each the largest "leading zeros + 1" seen among the hashes that select it.  The host
// turns the registers into a distinct-count estimate (±~1 %) that sizes the table after the small
// speculative table overflowed — instead of growing it by trial and error.
constexpr int HLL_BITS = 13;  // 8192 registers (32 KB of static shared memory), standard error 1.15 %
constexpr int HLL_REGS = 1 << HLL_BITS;

// packed keys of 4 consecutive rows through one vector load per key column (requires PF_VEC_KEYS and
// a full group of 4 rows); clears the bits of dropped rows in `act`
__device__ __forceinline__ void packed_keys4(const DPlan& P, i64 row0, u64 (&kk)[4], u32& act)
{
#pragma unroll
  for (int j = 0; j < 4; ++j) kk[j] = 0;
  for (int k = 0; k < P.nkeys; ++k) {
    const DKeyCol& c = P.keys[k];
    const unsigned char* src = c.data + (c.offset + row0) * c.width;
    u64 f[4];
    if (c.width == 4) {
      const uint4 q = __ldg((const uint4*)src);
      f[0] = q.x; f[1] = q.y; f[2] = q.z; f[3] = q.w;
    } else if (c.width == 8) {
      const ulonglong2 q0 = __ldg((const ulonglong2*)src), q1 = __ldg((const ulonglong2*)src + 1);
      f[0] = q0.x; f[1] = q0.y; f[2] = q1.x; f[3] = q1.y;
    } else if (c.width == 2) {
      const uint2 q = __ldg((const uint2*)src);
      f[0] = q.x & 0xFFFFu; f[1] = q.x >> 16; f[2] = q.y & 0xFFFFu; f[3] = q.y >> 16;
    } else {
      const u32 q = __ldg((const u32*)src);
      f[0] = q & 0xFFu; f[1] = (q >> 8) & 0xFFu; f[2] = (q >> 16) & 0xFFu; f[3] = q >> 24;
    }
    u32 vn = 0xFu;
    if (c.mask) {
      vn = valid_nibble(c.mask, c.offset + row0, 4);
      if (!P.include_nulls) act &= vn;  // EXCLUDE: a null key drops the row
    }
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const bool isnull = c.nullbit >= 0 && !((vn >> j) & 1u);
      kk[j] |= isnull ? (1ull << c.nullbit) : (f[j] << c.shift);
    }
  }
  for (int f = 0; f < P.nfilters; ++f) act &= valid_nibble(P.filters[f], P.filter_offsets[f] + row0, 4);
}

__global__ void __launch_bounds__(1024) k_hll(const __grid_constant__ DPlan P, u32* __restrict__ regs)
{
  __shared__ u32 s_regs[HLL_REGS];
  for (int i = threadIdx.x; i < HLL_REGS; i += blockDim.x) s_regs[i] = 0;
  __syncthreads();
  auto fold = [&](u64 h) {
    const u32 idx  = (u32)(h >> (64 - HLL_BITS));
    const u32 rank = (u32)__clzll((i64)((h << HLL_BITS) | (1ull << (HLL_BITS - 1)))) + 1u;
    if (s_regs[idx] < rank) atomicMax(&s_regs[idx], rank);
  };
  const i64 nquads = (P.key_mode == KM_PACKED && (P.flags & PF_VEC_KEYS)) ? P.nrows / 4 : 0;
  for (i64 q = (i64)blockIdx.x * blockDim.x + threadIdx.x; q < nquads; q += (i64)gridDim.x * blockDim.x) {
    u64 kk[4];
    u32 act = 0xFu;
    packed_keys4(P, q * 4, kk, act);
#pragma unroll
    for (int j = 0; j < 4; ++j)
      if ((act >> j) & 1u) fold(mix64(kk[j] ^ 0x5bd1e9955bd1e995ull));
  }
  for (i64 row = nquads * 4 + (i64)blockIdx.x * blockDim.x + threadIdx.x; row < P.nrows; row += (i64)gridDim.x * blockDim.x) {
    if (!row_active(P, row)) continue;
    fold((P.key_mode == KM_PACKED) ? mix64(pack_key(P, row) ^ 0x5bd1e9955bd1e995ull) : hash_row(P, row));
  }
  __syncthreads();
  for (int i = threadIdx.x; i < HLL_REGS; i += blockDim.x)
    if (s_regs[i]) atomicMax(&regs[i], s_regs[i]);
}

// ------------------------------------------------------------------------------ string keys -> dictionary ids
// A STRING key column is replaced by the id of its string in a dictionary, so that (id, other keys) packs into
// one 64-bit key cell and the packed-key paths serve the aggregate.  The dictionary is an open-addressing
// table of 8-byte cells {hash tag(30) | clamped length(8) | id(26)} plus, per id, the first 32 bytes of the
// string in a dense pool (ids are handed out in order of arrival: the pool of a column with few distinct
// strings is a few contiguous megabytes that stay in L2, where the first rows' own strings — scattered over
// the column — do not) and the first row that held it (for the bytes beyond 32, and for the output).  A probe
// that finds its tag and length compares against the pool entry.  `P` holds the one string column as its only
// key.  ids[P.keys[0].offset + row] = id (0 for a null row: its null bit or its exclusion decides, not the
// payload).  CTAs stop at their next tile once the table or the pool is over its limit.
constexpr int DICT_BLOCK  = 256;
constexpr int DICT_ROWS   = 4;   // rows per thread and tile, strided by the block so that loads coalesce
constexpr int DICT_INLINE = 32;  // string bytes kept in the pool
constexpr u64 DICT_ID_MASK = (1ull << 26) - 1ull;

struct DDict {
  u64* cells;      // [cap], EMPTY = free
  i64 cap;
  u64* pool;       // [pool_cap][4]
  int* first_row;  // [pool_cap]
  i64 pool_cap;    // <= 2^26 - 2
};

// id of the string [p, p + len) of row `row`, inserting it when new; -1 after an overflow
// (`w` = the string's first DICT_INLINE bytes, zero padded)
__device__ __forceinline__ i64 dict_find_insert(const DPlan& P, const DDict& D, const u64 (&w)[4], i64 len, i64 row, u64 h,
                                                DCtrl* ctrl, int* s_new)
{
  const u64 head = ((h >> 34) << 34) | ((u64)(len < 255 ? len : 255) << 26);
  i64 idx = (i64)reduce64(h, (u64)D.cap);
  for (int probe = 0; probe < GMEM_PROBES; ++probe) {
    u64 k = *(volatile u64*)(D.cells + idx);
    if (k == EMPTY) {
      // the entry is written before the cell that publishes it; a thread that loses the race for the cell
      // leaves its id unused
      const u64 id = atomicAdd(&ctrl->out_cursor, 1ull);
      if (id >= (u64)D.pool_cap) { ctrl->overflow = 1; return -1; }
      u64* e = D.pool + id * 4;
      e[0] = w[0]; e[1] = w[1]; e[2] = w[2]; e[3] = w[3];
      D.first_row[id] = (int)row;
      __threadfence();
      k = atomicCAS(D.cells + idx, EMPTY, head | id);
      if (k == EMPTY) { atomicAdd(s_new, 1); return (i64)id; }
    }
    if (((k ^ head) & ~DICT_ID_MASK) == 0) {  // same tag and (clamped) length
      const u64 id = k & DICT_ID_MASK;
      const ulonglong2* e = (const ulonglong2*)(D.pool + id * 4);
      const ulonglong2 e0 = __ldcg(e), e1 = __ldcg(e + 1);
      bool same = e0.x == w[0] && e0.y == w[1] && e1.x == w[2] && e1.y == w[3];
      if (same && len > DICT_INLINE) same = rows_equal(P, row, (i64)__ldcg(D.first_row + id));
      if (same) return (i64)id;
    }
    if (probe_gave_up(probe, ctrl, s_new)) return -1;
    if (++idx == D.cap) idx = 0;
  }
  ctrl->overflow = 1;
  return -1;
}

__global__ void __launch_bounds__(DICT_BLOCK) k_dict_encode(const __grid_constant__ DPlan P, const DDict D, DCtrl* ctrl,
                                                            u32* __restrict__ ids)
{
  __shared__ int s_new;
  __shared__ u32 s_stop;
  if (threadIdx.x == 0) { s_new = 0; s_stop = 0; }
  __syncthreads();
  const DKeyCol& c = P.keys[0];
  constexpr i64 TILE = (i64)DICT_BLOCK * DICT_ROWS;
  for (i64 base = (i64)blockIdx.x * TILE; base < P.nrows; base += (i64)gridDim.x * TILE) {
    // offsets of the tile's rows first (one coalesced pass), then hash and probe row by row
    i64 b[DICT_ROWS], e[DICT_ROWS];
    bool live[DICT_ROWS];
#pragma unroll
    for (int j = 0; j < DICT_ROWS; ++j) {
      const i64 row = base + (i64)j * DICT_BLOCK + threadIdx.x;
      live[j] = row < P.nrows && !(c.mask && !bit_valid(c.mask, c.offset + row));
      b[j] = e[j] = 0;
      if (live[j]) { b[j] = str_offset(c, c.offset + row); e[j] = str_offset(c, c.offset + row + 1); }
    }
#pragma unroll
    for (int j = 0; j < DICT_ROWS; ++j) {
      const i64 row = base + (i64)j * DICT_BLOCK + threadIdx.x;
      if (row >= P.nrows) continue;
      u32 id = 0;
      if (live[j]) {
        // the first 32 bytes once, as four zero-padded words: hashed from registers (every lane takes the same four
        // steps whatever its string's length) and compared against the pool entry; longer strings hash their rest
        const unsigned char* p = c.data + b[j];
        const i64 len = e[j] - b[j];
        u64 w[4];
        u64 h = 0x243F6A8885A308D3ull;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const i64 left = len - 8 * i;
          w[i] = left > 0 ? load_bytes8(p + 8 * i, (int)(left < 8 ? left : 8)) : 0ull;
          h = mix64(h ^ w[i]) + 0x9E3779B97F4A7C15ull;
        }
        if (len > DICT_INLINE) h = hash_bytes(p + DICT_INLINE, len - DICT_INLINE, h);
        h = mix64(mix64(h ^ ((u64)len << 56)));
        const i64 s = dict_find_insert(P, D, w, len, row, h, ctrl, &s_new);
        if (s >= 0) id = (u32)s;
      }
      ids[c.offset + row] = id;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      const int n = s_new;
      s_new = 0;
      if (n) {
        const u64 tot = atomicAdd(&ctrl->nclaimed, (u64)n) + (u64)n;
        if (tot > ctrl->claim_limit) ctrl->overflow = 1;
      }
      s_stop = *(volatile u32*)&ctrl->overflow;
    }
    __syncthreads();
    if (s_stop) return;
  }
}

// ids of the finished groups -> the first rows that held their strings (-1 for a null key)
__global__ void k_dict_rows(const u32* __restrict__ ids, const u32* __restrict__ id_mask, const int* __restrict__ first_row,
                            i64 ngroups, int* __restrict__ rows)
{
  for (i64 g = (i64)blockIdx.x * blockDim.x + threadIdx.x; g < ngroups; g += (i64)gridDim.x * blockDim.x)
    rows[g] = (id_mask && !bit_valid(id_mask, g)) ? -1 : first_row[ids[g]];
}

// ------------------------------------------------------------------------------ dictionary values
// DICTIONARY32 value columns (cpp/include/cudf/detail/aggregation/device_aggregators.cuh:189-220: the reference
// looks the key up at every update): values[i] = keys[indices[i]] written out once, so that the aggregate passes
// see a plain column of the keys' type.  Null rows (their index may be anything) are written as zero.
struct DDictDecode {
  const unsigned char* indices; int index_width; int index_signed; i64 index_offset;  // element offset of row 0
  const unsigned char* keys; i64 keys_offset; i64 nkeys; int width;
  const u32* mask; i64 mask_offset;  // the dictionary column's validity (nullptr = all valid)
  unsigned char* dst;                // element 0 of the decoded rows
};
__global__ void __launch_bounds__(256) k_dict_decode(const DDictDecode D, i64 n)
{
  for (i64 i = (i64)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (i64)gridDim.x * blockDim.x) {
    u64 v = 0;
    if (!D.mask || bit_valid(D.mask, D.mask_offset + i)) {
      const u64 raw = load_fixed_bits(D.indices, D.index_offset + i, D.index_width);
      const int sh  = 64 - 8 * D.index_width;
      const i64 idx = D.index_signed ? ((i64)(raw << sh) >> sh) : (i64)raw;
      if (idx >= 0 && idx < D.nkeys) v = load_fixed_bits(D.keys, D.keys_offset + idx, D.width);
    }
    switch (D.width) {
      case 1: D.dst[i] = (unsigned char)v; break;
      case 2: ((unsigned short*)D.dst)[i] = (unsigned short)v; break;
      case 4: ((u32*)D.dst)[i] = (u32)v; break;
      default: ((u64*)D.dst)[i] = v; break;
    }
  }
}

__global__ void __launch_bounds__(256) k_iota(int* __restrict__ p, i64 n)
{
  for (i64 i = (i64)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (i64)gridDim.x * blockDim.x) p[i] = (int)i;
}

// ------------------------------------------------------------------------------ finalize
enum OutKind : int {
  OK_COUNT = 0,  // int32 from a count cell
  OK_INT,        // integer cell (Σ, Σx², Π, min, max of integers) stored in the result width
  OK_FLT,        // double cell (Σ, Σx², Π of floats) stored as FLOAT32/FLOAT64
  OK_MINMAX_F,   // ordered-encoded double cell
  OK_MEAN, OK_M2, OK_VAR, OK_STD,
  OK_ARG,        // ARGMIN / ARGMAX: the row held by the cell as INT32, null when none
  OK_STRARG,     // MIN / MAX of strings: the row (or -1) into a scratch array the host gathers the strings by
  OK_SUMOVF,     // SUM_OVERFLOW: the sum in the source type into `data`, "the exact sum does not fit it" into `data2`
  OK_SUM128      // SUM of DECIMAL128: 16-byte elements from the four exact-sum cells c_a .. c_a + 3
};

struct DOutCol {
  void* data;
  void* data2;    // OK_SUMOVF: the BOOL8 overflow child
  u32* mask;      // nullptr = result not nullable
  int kind;       // OutKind
  int rclass;     // ValClass of the result element type
  int c_a;        // primary cell (Σx for MEAN/M2/VAR/STD)
  int c_b;        // Σx² for M2/VAR/STD
  int c_cnt;      // count cell deciding validity, -1 = always valid
  int ddof;
  int src_float;  // the Σ cells hold doubles
  int null_slot;  // index into null_counts
};

constexpr int MAX_OUTS = 64;

struct DOutPlan {
  int nouts;
  int pad;
  DOutCol outs[MAX_OUTS];
  void* kdata[MAX_KEYS];   // packed mode: decoded key columns
  u32* kmask[MAX_KEYS];
  int* rep_rows;           // row-key mode: representative row per group
  u32* null_counts;        // [MAX_OUTS + MAX_KEYS]
  i64 max_groups;          // > 0: the output columns hold this many rows; groups beyond them are not written
                           // (the host compares the cursor with it afterwards)
};

__device__ __forceinline__ void store_int(void* data, i64 g, int rclass, u64 v)
{
  switch (rclass) {
    case VC_I8: case VC_U8: case VC_BOOL: ((unsigned char*)data)[g] = (unsigned char)v; break;
    case VC_I16: case VC_U16: ((unsigned short*)data)[g] = (unsigned short)v; break;
    case VC_I32: case VC_U32: ((u32*)data)[g] = (u32)v; break;
    default: ((u64*)data)[g] = v; break;
  }
}
__device__ __forceinline__ void store_flt(void* data, i64 g, int rclass, double v)
{
  if (rclass == VC_F32) ((float*)data)[g] = (float)v;
  else ((double*)data)[g] = v;
}
__device__ __forceinline__ void clear_bit(u32* mask, i64 g, u32* counter)
{
  atomicAnd(mask + (g >> 5), ~(1u << (g & 31)));
  atomicAdd(counter, 1u);
}

// The sum of a DECIMAL128 column from its four exact cells {Σ(lo & 0xFFFFFFFF), Σ(lo >> 32), Σ(hi & 0xFFFFFFFF),
// Σ(hi >> 32, signed)} (cell i at c[i * cstep]; each exact below 2^31 rows): the low and high words of the sum
// modulo 2^128, and whether the exact sum leaves the 128-bit range.
__device__ __forceinline__ bool sum128(const u64* c, i64 cstep, u64& lo, u64& hi)
{
  const unsigned __int128 a = (unsigned __int128)c[0] + ((unsigned __int128)c[cstep] << 32);                  // < 2^96
  const __int128 b = (__int128)c[2 * cstep] + (__int128)(i64)c[3 * cstep] * ((__int128)1 << 32) + (__int128)(u64)(a >> 64);
  lo = (u64)a;
  hi = (u64)b;
  return b < -((__int128)1 << 63) || b > (((__int128)1 << 63) - 1);
}

// One finished group -> output row g: key columns decoded from the key cell (packed keys) or the
// representative row noted (row keys), then every requested aggregation from the accumulator cells
// (cell c at cells[c * cstep]): COUNT as INT32, MEAN = Σx / n, M2 = Σx² − (Σx)²/n, VAR = M2 / (n − ddof),
// STD = sqrt(VAR); results without a valid input are nulled and counted.
__device__ __forceinline__ void write_group(const DPlan& P, const DOutPlan& O, u64 key, const u64* cells, i64 cstep, i64 g)
{
  if (P.key_mode == KM_PACKED) {
    for (int k = 0; k < P.nkeys; ++k) {
      const DKeyCol& c = P.keys[k];
      if (c.nullbit >= 0 && ((key >> c.nullbit) & 1ull)) {
        clear_bit(O.kmask[k], g, O.null_counts + MAX_OUTS + k);
        store_int(O.kdata[k], g, c.width == 1 ? VC_U8 : c.width == 2 ? VC_U16 : c.width == 4 ? VC_U32 : VC_U64, 0);
      } else {
        const u64 v = (c.width == 8) ? (key >> c.shift) : ((key >> c.shift) & ((1ull << (8 * c.width)) - 1ull));
        store_int(O.kdata[k], g, c.width == 1 ? VC_U8 : c.width == 2 ? VC_U16 : c.width == 4 ? VC_U32 : VC_U64, v);
      }
    }
  } else {
    O.rep_rows[g] = (int)(u32)key;
  }
  for (int o = 0; o < O.nouts; ++o) {
    const DOutCol& oc = O.outs[o];
    const i64 n = oc.c_cnt >= 0 ? (i64)cells[(i64)(oc.c_cnt) * cstep] : 1;
    bool valid  = n > 0;
    switch (oc.kind) {
      case OK_COUNT: ((int*)oc.data)[g] = (int)cells[(i64)(oc.c_a) * cstep]; valid = true; break;
      case OK_INT: store_int(oc.data, g, oc.rclass, valid ? cells[(i64)(oc.c_a) * cstep] : 0); break;
      case OK_FLT: store_flt(oc.data, g, oc.rclass, valid ? __longlong_as_double((i64)cells[(i64)(oc.c_a) * cstep]) : 0.0); break;
      case OK_MINMAX_F:
        store_flt(oc.data, g, oc.rclass, valid ? __longlong_as_double((i64)f64_unordered(cells[(i64)(oc.c_a) * cstep])) : 0.0);
        break;
      case OK_ARG: case OK_STRARG: {
        const u64 r = cells[(i64)(oc.c_a) * cstep];
        valid = r != ARG_NONE;
        ((int*)oc.data)[g] = valid ? (int)r : (oc.kind == OK_ARG ? 0 : -1);
        break;
      }
      case OK_SUMOVF: {
        // The exact sum is Σ(v >> 32) · 2^32 + Σ(v & 0xFFFFFFFF) for a 64-bit source (cells c_a, c_b), the one
        // int64 cell otherwise.  The reference raises the flag when an add wraps in the source type
        // (cpp/include/cudf/detail/aggregation/device_aggregators.cuh:136-160), which depends on the order the
        // rows arrive in; "the exact sum does not fit" is what every order gives when a group's values share a
        // sign, and what the order that alternates signs gives otherwise.
        bool ovf = false;
        u64 sum  = 0;
        if (oc.rclass == VC_U64X2) {  // DECIMAL128
          u64 lo = 0, hi = 0;
          if (valid) ovf = sum128(cells + (i64)(oc.c_a) * cstep, cstep, lo, hi);
          ((u64*)oc.data)[2 * g] = lo;
          ((u64*)oc.data)[2 * g + 1] = hi;
          ((unsigned char*)oc.data2)[g] = ovf ? 1 : 0;
          break;
        }
        if (valid) {
          if (oc.c_b >= 0) {
            const u64 lo = cells[(i64)(oc.c_b) * cstep];
            const i64 t  = (i64)cells[(i64)(oc.c_a) * cstep] + (i64)(lo >> 32);
            ovf = t < -2147483648ll || t > 2147483647ll;
            sum = ((u64)t << 32) | (lo & 0xFFFFFFFFull);
          } else {
            const i64 v    = (i64)cells[(i64)(oc.c_a) * cstep];
            const int bits = oc.rclass == VC_I8 ? 8 : oc.rclass == VC_I16 ? 16 : 32;
            ovf = v < -(1ll << (bits - 1)) || v > (1ll << (bits - 1)) - 1;
            sum = (u64)v;
          }
        }
        store_int(oc.data, g, oc.rclass, sum);
        ((unsigned char*)oc.data2)[g] = ovf ? 1 : 0;
        break;
      }
      case OK_SUM128: {
        u64 lo = 0, hi = 0;
        if (valid) sum128(cells + (i64)(oc.c_a) * cstep, cstep, lo, hi);
        ((u64*)oc.data)[2 * g] = lo;
        ((u64*)oc.data)[2 * g + 1] = hi;
        break;
      }
      case OK_MEAN: {
        if (oc.rclass != VC_F64) {  // durations: integer division in the source type
          store_int(oc.data, g, oc.rclass, valid ? (u64)((i64)cells[(i64)(oc.c_a) * cstep] / n) : 0);
          break;
        }
        const double s = oc.src_float ? __longlong_as_double((i64)cells[(i64)(oc.c_a) * cstep]) : (double)(i64)cells[(i64)(oc.c_a) * cstep];
        ((double*)oc.data)[g] = valid ? s / (double)n : 0.0;
        break;
      }
      default: {  // M2, VAR, STD
        double m2 = 0.0;
        if (n > 0) {
          const double s  = oc.src_float ? __longlong_as_double((i64)cells[(i64)(oc.c_a) * cstep]) : (double)(i64)cells[(i64)(oc.c_a) * cstep];
          const double ss = oc.src_float ? __longlong_as_double((i64)cells[(i64)(oc.c_b) * cstep]) : (double)(i64)cells[(i64)(oc.c_b) * cstep];
          m2 = ss - s * s / (double)n;
        }
        if (oc.kind == OK_M2) { ((double*)oc.data)[g] = m2; valid = true; break; }
        const i64 df = n - oc.ddof;
        valid        = n > 0 && df > 0;
        const double var = valid ? m2 / (double)df : 0.0;
        ((double*)oc.data)[g] = (oc.kind == OK_VAR) ? var : sqrt(var);
        break;
      }
    }
    if (!valid && oc.mask) clear_bit(oc.mask, g, O.null_counts + oc.null_slot);
  }
}

constexpr int FIN_BLOCK = 256;
constexpr int FIN_ITEMS = 8;  // slots per thread per chunk (1 for small tables, which otherwise fill few SMs)

// Occupied slots are compacted chunk by chunk: a CTA counts the occupied slots of its chunk
// (FIN_BLOCK x FIN_ITEMS slots), reserves that many output rows with ONE atomic on the cursor, and its
// threads write their groups at the reserved positions.  (One reservation per warp and 32 slots made
// the single cursor the bottleneck of large tables: 6M atomics on one address for 200M slots.)
template <int ITEMS>
__global__ void __launch_bounds__(FIN_BLOCK) k_finalize(const __grid_constant__ DPlan P, const __grid_constant__ DOutPlan O,
                                                        const u64* __restrict__ tbl, i64 cap, DCtrl* ctrl)
{
  __shared__ u32 s_wcount[FIN_BLOCK / 32];
  __shared__ u32 s_ballot[FIN_BLOCK / 32][ITEMS];
  __shared__ u64 s_base;
  const int stride = P.stride;
  const i64 dense  = (i64)ctrl->dense_slots;
  const i64 nslots = cap + 1 + dense;
  const i64 chunk  = (i64)FIN_BLOCK * ITEMS;
  const i64 nchunks = (nslots + chunk - 1) / chunk;
  const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
  for (i64 ch = blockIdx.x; ch < nchunks; ch += gridDim.x) {
    u32 wtotal = 0;
#pragma unroll
    for (int j = 0; j < ITEMS; ++j) {
      const i64 s = ch * chunk + (i64)j * FIN_BLOCK + threadIdx.x;
      bool occ = false;
      if (s < nslots && s != cap) occ = *slot_ref(const_cast<u64*>(tbl), cap, stride, dense, s).key != EMPTY;
      else if (s == cap) occ = ctrl->special_used != 0;
      const u32 m = __ballot_sync(0xFFFFFFFFu, occ);
      if (lane == 0) s_ballot[wid][j] = m;
      wtotal += __popc(m);
    }
    if (lane == 0) s_wcount[wid] = wtotal;
    __syncthreads();
    if (threadIdx.x == 0) {
      u32 tot = 0;
      for (int w = 0; w < FIN_BLOCK / 32; ++w) { const u32 c = s_wcount[w]; s_wcount[w] = tot; tot += c; }
      s_base = tot ? atomicAdd(&ctrl->out_cursor, (u64)tot) : 0ull;
    }
    __syncthreads();
    u64 next = s_base + s_wcount[wid];  // first output row of this warp's groups
#pragma unroll 1
    for (int j = 0; j < ITEMS; ++j) {
      const u32 m = s_ballot[wid][j];
      const i64 g = (i64)next + __popc(m & ((1u << lane) - 1u));
      next += __popc(m);
      if (!((m >> lane) & 1u)) continue;
      if (O.max_groups > 0 && g >= O.max_groups) continue;
      const i64 s = ch * chunk + (i64)j * FIN_BLOCK + threadIdx.x;
      const SlotRef ref = slot_ref(const_cast<u64*>(tbl), cap, stride, dense, s);
      write_group(P, O, s == cap ? EMPTY : *ref.key, ref.cells, ref.step, g);
    }
    __syncthreads();  // the shared arrays are rewritten by the next chunk
  }
}

// ------------------------------------------------------------------------------ finishers over partial columns
// Partial aggregates that travel as columns (string / float / wide keys between ranks and batches: Σx, n, Σx²
// per group) are finished here: mean, M2, variance, standard deviation, counts as INT32 — the formulas of
// write_group (cpp/src/groupby/hash/hash_compound_agg_finalizer.cu:93-186, common/m2_var_std.cu:57) — and the
// validity of a result from n.
struct DFinish {
  int kind;        // FK_* below
  int ddof;
  int rclass;      // ValClass of the result
  int int_mean;    // mean by integer division in the source type (durations)
  DValCol sum, cnt, ssq;
  void* out;
  u32* out_mask;   // nullptr = not nullable
  u32* null_count;
};
enum FinishKind : int { FK_COUNT = 0, FK_MEAN, FK_M2, FK_VAR, FK_STD, FK_VALID_ONLY };

__device__ __forceinline__ double carried_as_double(const DValCol& c, u64 v)
{
  if (c.vclass == VC_F32 || c.vclass == VC_F64) return __longlong_as_double((i64)v);
  if (c.vclass == VC_U64) return (double)v;
  return (double)(i64)v;
}

__global__ void k_finish_partial(const DFinish F, i64 n)
{
  const u32 lane = threadIdx.x & 31u;
  const i64 nround = (n + 31) / 32 * 32;
  for (i64 g = (i64)blockIdx.x * blockDim.x + threadIdx.x; g < nround; g += (i64)gridDim.x * blockDim.x) {
    bool valid = false;
    if (g < n) {
      const i64 c = (i64)load_value(F.cnt, g);
      valid = c > 0;
      switch (F.kind) {
        case FK_COUNT: store_int(F.out, g, F.rclass, (u64)c); valid = true; break;
        case FK_MEAN: {
          const u64 sv = load_value(F.sum, g);
          if (F.int_mean) store_int(F.out, g, F.rclass, (u64)((i64)sv / (c > 0 ? c : 1)));
          else store_flt(F.out, g, F.rclass, carried_as_double(F.sum, sv) / (double)(c > 0 ? c : 1));
          break;
        }
        case FK_M2: case FK_VAR: case FK_STD: {
          const double s = carried_as_double(F.sum, load_value(F.sum, g)), ss = carried_as_double(F.ssq, load_value(F.ssq, g));
          const double m2 = c > 0 ? ss - s * s / (double)c : 0.0;
          if (F.kind == FK_M2) { store_flt(F.out, g, F.rclass, m2); valid = true; break; }
          const i64 df = c - F.ddof;
          valid = c > 0 && df > 0;
          const double var = valid ? m2 / (double)df : 0.0;
          store_flt(F.out, g, F.rclass, F.kind == FK_VAR ? var : sqrt(var));
          break;
        }
        default: break;  // FK_VALID_ONLY: the mask alone
      }
    }
    if (F.out_mask) {
      const u32 word = __ballot_sync(0xFFFFFFFFu, valid);
      if (lane == 0) {
        F.out_mask[g >> 5] = word;
        const i64 here = n - g < 32 ? n - g : 32;  // rows of this word
        const u32 nulls = (u32)here - (u32)__popc(word);
        if (nulls && F.null_count) atomicAdd(F.null_count, nulls);
      }
    }
  }
}

// ------------------------------------------------------------------------------ key gather (row keys)
struct DGather {
  const unsigned char* src; const u32* src_mask; i64 src_offset; int width;
  unsigned char* dst; u32* dst_mask; u32* null_counter;
};

__global__ void k_gather_fixed(DGather G, const int* __restrict__ rows, i64 ngroups)
{
  for (i64 g = (i64)blockIdx.x * blockDim.x + threadIdx.x; g < ngroups; g += (i64)gridDim.x * blockDim.x) {
    const i64 idx = G.src_offset + rows[g];
    if (G.src_mask && !bit_valid(G.src_mask, idx)) {
      if (G.dst_mask) clear_bit(G.dst_mask, g, G.null_counter);
      for (int b = 0; b < G.width; ++b) G.dst[g * G.width + b] = 0;
    } else {
      for (int b = 0; b < G.width; ++b) G.dst[g * G.width + b] = G.src[idx * G.width + b];
    }
  }
}

// string lengths of the representative rows (0 for a null), then offsets by scan, then the bytes
__global__ void k_string_lengths(DKeyCol c, const int* __restrict__ rows, i64 ngroups, i64* __restrict__ lens,
                                 u32* dst_mask, u32* null_counter)
{
  for (i64 g = (i64)blockIdx.x * blockDim.x + threadIdx.x; g < ngroups; g += (i64)gridDim.x * blockDim.x) {
    const i64 idx = c.offset + rows[g];
    i64 len = 0;
    if (rows[g] < 0) {
      // no row (a string MIN / MAX of a group without a valid value: nulled by the finisher already)
    } else if (c.mask && !bit_valid(c.mask, idx)) {
      if (dst_mask) clear_bit(dst_mask, g, null_counter);
    } else {
      len = str_offset(c, idx + 1) - str_offset(c, idx);
    }
    lens[g] = len;
  }
}

// single-CTA exclusive scan over n int64 (n = number of groups; one pass, 1024 threads)
__global__ void __launch_bounds__(1024) k_exclusive_scan(const i64* __restrict__ in, i64* __restrict__ out, i64 n)
{
  __shared__ i64 s_warp[32];
  __shared__ i64 s_carry;
  if (threadIdx.x == 0) s_carry = 0;
  __syncthreads();
  const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
  for (i64 base = 0; base < n; base += blockDim.x) {
    const i64 i = base + threadIdx.x;
    const i64 x = i < n ? in[i] : 0;
    i64 v = x;
    for (int d = 1; d < 32; d <<= 1) { const i64 t = __shfl_up_sync(0xFFFFFFFFu, v, d); if (lane >= d) v += t; }
    if (lane == 31) s_warp[wid] = v;
    __syncthreads();
    if (wid == 0) {
      i64 wv = s_warp[lane];
      for (int d = 1; d < 32; d <<= 1) { const i64 t = __shfl_up_sync(0xFFFFFFFFu, wv, d); if (lane >= d) wv += t; }
      s_warp[lane] = wv;
    }
    __syncthreads();
    const i64 prefix = s_carry + (wid ? s_warp[wid - 1] : 0) + (v - x);
    if (i < n) out[i] = prefix;
    __syncthreads();
    if (threadIdx.x == blockDim.x - 1) s_carry += s_warp[31];
    __syncthreads();
  }
  if (threadIdx.x == 0) out[n] = s_carry;
}

// exclusive scan of many elements in three steps: per-block totals, scan of the totals (one CTA),
// per-block scan with the block's base added
constexpr int SCAN_BLOCK = 1024;
constexpr int SCAN_ITEMS = 4;  // elements per thread
__global__ void __launch_bounds__(SCAN_BLOCK) k_scan_block_totals(const i64* __restrict__ in, i64 n, i64* __restrict__ totals)
{
  __shared__ i64 s_warp[32];
  const i64 base = (i64)blockIdx.x * SCAN_BLOCK * SCAN_ITEMS;
  i64 v = 0;
  for (int j = 0; j < SCAN_ITEMS; ++j) {
    const i64 i = base + (i64)threadIdx.x * SCAN_ITEMS + j;
    if (i < n) v += in[i];
  }
  for (int d = 16; d > 0; d >>= 1) v += __shfl_xor_sync(0xFFFFFFFFu, v, d);
  if ((threadIdx.x & 31) == 0) s_warp[threadIdx.x >> 5] = v;
  __syncthreads();
  if (threadIdx.x < 32) {
    i64 w = s_warp[threadIdx.x];
    for (int d = 16; d > 0; d >>= 1) w += __shfl_xor_sync(0xFFFFFFFFu, w, d);
    if (threadIdx.x == 0) totals[blockIdx.x] = w;
  }
}
__global__ void __launch_bounds__(SCAN_BLOCK)
k_scan_apply(const i64* __restrict__ in, i64 n, const i64* __restrict__ block_bases, i64* __restrict__ out)
{
  __shared__ i64 s_warp[32];
  const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
  const i64 base = (i64)blockIdx.x * SCAN_BLOCK * SCAN_ITEMS;
  i64 x[SCAN_ITEMS], mine = 0;
  for (int j = 0; j < SCAN_ITEMS; ++j) {
    const i64 i = base + (i64)threadIdx.x * SCAN_ITEMS + j;
    x[j] = i < n ? in[i] : 0;
    mine += x[j];
  }
  i64 v = mine;
  for (int d = 1; d < 32; d <<= 1) { const i64 t = __shfl_up_sync(0xFFFFFFFFu, v, d); if (lane >= d) v += t; }
  if (lane == 31) s_warp[wid] = v;
  __syncthreads();
  if (wid == 0) {
    i64 w = s_warp[lane];
    for (int d = 1; d < 32; d <<= 1) { const i64 t = __shfl_up_sync(0xFFFFFFFFu, w, d); if (lane >= d) w += t; }
    s_warp[lane] = w;
  }
  __syncthreads();
  i64 run = block_bases[blockIdx.x] + (wid ? s_warp[wid - 1] : 0) + (v - mine);
  for (int j = 0; j < SCAN_ITEMS; ++j) {
    const i64 i = base + (i64)threadIdx.x * SCAN_ITEMS + j;
    if (i < n) out[i] = run;
    run += x[j];
  }
  if (blockIdx.x == gridDim.x - 1 && threadIdx.x == SCAN_BLOCK - 1) out[n] = run;
}

template <typename OffT>
__global__ void k_string_copy(DKeyCol c, const int* __restrict__ rows, i64 ngroups, const i64* __restrict__ offs,
                              OffT* __restrict__ out_offs, unsigned char* __restrict__ chars)
{
  // four lanes per string, 8 bytes per lane and step (key strings are short: a warp per string left most of
  // its lanes idle); the source is read as aligned words, the destination written byte by byte
  const int sub = threadIdx.x & 3;
  const i64 s0 = ((i64)blockIdx.x * blockDim.x + threadIdx.x) >> 2;
  const i64 ns = ((i64)gridDim.x * blockDim.x) >> 2;
  for (i64 g = s0; g <= ngroups; g += ns) {
    if (sub == 0) out_offs[g] = (OffT)offs[g];
    if (g == ngroups) break;
    const i64 len = offs[g + 1] - offs[g];
    if (len == 0) continue;
    const i64 idx = c.offset + rows[g];
    const unsigned char* src = c.data + str_offset(c, idx);
    unsigned char* dst = chars + offs[g];
    for (i64 b = (i64)sub * 8; b < len; b += 32) {
      const int nb = (int)(len - b < 8 ? len - b : 8);
      u64 v = load_bytes8(src + b, nb);
      for (int i = 0; i < nb; ++i) { dst[b + i] = (unsigned char)v; v >>= 8; }
    }
  }
}

// ------------------------------------------------------------------------------ partial records
// owner partition of every occupied slot: counts, then scatter into destination-major order
// Lanes of a warp headed for the same destination add to its counter ONCE (with few destinations
// every lane of a CTA would otherwise hit the same two or eight shared-memory words).  Returns this
// lane's position among the destination's records as counted by `counter`, or nothing useful for
// lanes with `dest` = NO_DEST.  Must be called by all 32 lanes.
constexpr u32 NO_DEST = 0xFFFFFFFFu;
__device__ __forceinline__ u64 warp_add_by_dest(u64* counters, u32 dest)
{
  const u32 lane  = threadIdx.x & 31u;
  const u32 peers = __match_any_sync(0xFFFFFFFFu, dest);
  const int lead  = __ffs(peers) - 1;
  u64 base = 0;
  if (dest != NO_DEST && (int)lane == lead) base = atomicAdd(&counters[dest], (u64)__popc(peers));
  base = __shfl_sync(0xFFFFFFFFu, base, lead);
  return base + (u64)__popc(peers & ((1u << lane) - 1u));
}

__global__ void k_pack_count(const u64* __restrict__ tbl, i64 cap, int stride, int nparts, const DCtrl* ctrl,
                             u64* __restrict__ counts)
{
  extern __shared__ u64 s_cnt[];
  for (int p = threadIdx.x; p < nparts; p += blockDim.x) s_cnt[p] = 0;
  __syncthreads();
  const i64 last = cap + (i64)ctrl->dense_slots;
  const u32 lane = threadIdx.x & 31u;
  for (i64 s0 = (i64)blockIdx.x * blockDim.x + (threadIdx.x - lane); s0 <= last; s0 += (i64)gridDim.x * blockDim.x) {
    const i64 s = s0 + lane;
    u32 dest = NO_DEST;
    if (s <= last) {
      const u64 key = s != cap ? *slot_ref(const_cast<u64*>(tbl), cap, stride, last - cap, s).key : EMPTY;
      const bool occ = s != cap ? key != EMPTY : ctrl->special_used != 0;
      if (occ) dest = owner_of(mix64(key), (u32)nparts);
    }
    warp_add_by_dest(s_cnt, dest);
  }
  __syncthreads();
  for (int p = threadIdx.x; p < nparts; p += blockDim.x)
    if (s_cnt[p]) atomicAdd(&counts[p], s_cnt[p]);
}

// Scatter of the occupied slots into destination-major order.  Each CTA owns a contiguous range of
// slots: it counts its records per destination in shared memory, reserves its output ranges with ONE
// global atomic per destination, then scatters with shared-memory cursors (one global atomic per
// record on a handful of addresses serialised: 3.5 ms for 5.4M records).
__global__ void __launch_bounds__(256)
k_pack_scatter(const u64* __restrict__ tbl, i64 cap, int stride, int nparts, const DCtrl* ctrl,
               u64* __restrict__ cursors /* start offsets, advanced */, u64* __restrict__ out)
{
  extern __shared__ u64 s_pack[];  // [nparts] counts, then [nparts] bases
  u64* s_cnt  = s_pack;
  u64* s_base = s_pack + nparts;
  const i64 last  = cap + (i64)ctrl->dense_slots;
  const i64 per   = (last + 1 + gridDim.x - 1) / gridDim.x;
  const i64 lo    = (i64)blockIdx.x * per;
  const i64 hi    = min(last + 1, lo + per);
  const u32 lane  = threadIdx.x & 31u;
  auto dest_of = [&](i64 s, u64& key) -> u32 {
    if (s >= hi) return NO_DEST;
    key = s != cap ? *slot_ref(const_cast<u64*>(tbl), cap, stride, last - cap, s).key : EMPTY;
    const bool occ = s != cap ? key != EMPTY : ctrl->special_used != 0;
    return occ ? owner_of(mix64(key), (u32)nparts) : NO_DEST;
  };
  for (int p = threadIdx.x; p < nparts; p += blockDim.x) s_cnt[p] = 0;
  __syncthreads();
  for (i64 s0 = lo + (threadIdx.x - lane); s0 < hi; s0 += blockDim.x) {
    u64 key = 0;
    warp_add_by_dest(s_cnt, dest_of(s0 + lane, key));
  }
  __syncthreads();
  for (int p = threadIdx.x; p < nparts; p += blockDim.x) {
    s_base[p] = s_cnt[p] ? atomicAdd(&cursors[p], s_cnt[p]) : 0;
    s_cnt[p]  = 0;
  }
  __syncthreads();
  for (i64 s0 = lo + (threadIdx.x - lane); s0 < hi; s0 += blockDim.x) {
    const i64 s = s0 + lane;
    u64 key = 0;
    const u32 p = dest_of(s, key);
    const u64 r = warp_add_by_dest(s_cnt, p);
    if (p == NO_DEST) continue;
    const u64 pos = s_base[p] + r;
    u64* dst = out + pos * stride;
    const SlotRef src = slot_ref(const_cast<u64*>(tbl), cap, stride, last - cap, s);
    dst[0] = key;
    for (int c = 1; c < stride; ++c) dst[c] = src.cells[(i64)(c - 1) * src.step];
  }
}

// The same for a state that holds its groups as a list (structure-of-arrays: word w of group g at
// groups[w * gcap + g]) — what the partitioned path leaves: CTA-contiguous ranges of the list, one global
// reservation per destination and CTA, records written in destination-major order.
__global__ void __launch_bounds__(256)
k_pack_list(const u64* __restrict__ groups, i64 gcap, i64 ngroups, int stride, int nparts, u64* __restrict__ cursors,
            u64* __restrict__ out /* nullptr: only count into `cursors` */)
{
  extern __shared__ u64 s_pack[];  // [nparts] counts, then [nparts] bases
  u64* s_cnt  = s_pack;
  u64* s_base = s_pack + nparts;
  const i64 per  = (ngroups + gridDim.x - 1) / gridDim.x;
  const i64 lo   = (i64)blockIdx.x * per;
  const i64 hi   = min(ngroups, lo + per);
  const u32 lane = threadIdx.x & 31u;
  for (int p = threadIdx.x; p < nparts; p += blockDim.x) s_cnt[p] = 0;
  __syncthreads();
  for (i64 g0 = lo + (threadIdx.x - lane); g0 < hi; g0 += blockDim.x) {
    const i64 g = g0 + lane;
    warp_add_by_dest(s_cnt, g < hi ? owner_of(mix64(groups[g]), (u32)nparts) : NO_DEST);
  }
  __syncthreads();
  for (int p = threadIdx.x; p < nparts; p += blockDim.x) {
    s_base[p] = s_cnt[p] ? atomicAdd(&cursors[p], s_cnt[p]) : 0;
    s_cnt[p]  = 0;
  }
  if (!out) return;
  __syncthreads();
  for (i64 g0 = lo + (threadIdx.x - lane); g0 < hi; g0 += blockDim.x) {
    const i64 g = g0 + lane;
    const u64 key = g < hi ? groups[g] : 0;
    const u32 p = g < hi ? owner_of(mix64(key), (u32)nparts) : NO_DEST;
    const u64 r = warp_add_by_dest(s_cnt, p);
    if (p == NO_DEST) continue;
    u64* dst = out + (s_base[p] + r) * stride;
    dst[0] = key;
    for (int c = 1; c < stride; ++c) dst[c] = groups[(i64)c * gcap + g];
  }
}

// Slot of a packed key in a table that may hold a dense region (a table filled by the fused kernel in
// dense mode keeps the in-box keys there): in-box keys are addressed directly, the rest is hashed, so
// that a key never ends up in both regions.
__device__ __forceinline__ i64 table_slot_packed(const DPlan& P, u64* tbl, i64 cap, int stride, u64 key, DCtrl* ctrl,
                                                 int* s_new)
{
  if (ctrl->dense_slots != 0 && ctrl->dense.enabled && key != EMPTY) {
    const int di = dense_index(P, ctrl->dense, key);
    if (di >= 0) {
      const i64 g = cap + 1 + (i64)di;
      u64* kp = slot_ref(tbl, cap, stride, (i64)ctrl->dense_slots, g).key;
      if (*(volatile u64*)kp == EMPTY && atomicCAS(kp, EMPTY, key) == EMPTY) atomicAdd(s_new, 1);
      return g;
    }
  }
  return gmem_find_insert_packed(tbl, cap, stride, key, mix64(key), ctrl, s_new);
}

// fixed-size chunks: chunk d = { count, overflow, records[chunk_records] }.  One launch: every occupied
// slot takes the next position of its destination's chunk (records beyond the chunk's capacity are not
// written); the last CTA to finish writes the headers — the counts, or, when any destination
// overflowed, the overflow mark in EVERY chunk, so that every receiver learns of it.
// `cursors` ([nparts] counters + one ticket word) must arrive zeroed.
// `check`: the table comes from an aggregate attempt whose control block the host has not read — bit 0: an
// attempt that overflowed or hit an error marks every chunk like an overflow (the receivers then make all
// ranks repeat the exchange with exact sizes, and this rank continues its aggregate first); bit 1: so does
// a lean fused kernel that declined its input (no key box).
__global__ void __launch_bounds__(256)
k_pack_chunks(const u64* __restrict__ tbl, i64 cap, int stride, int nparts, const DCtrl* ctrl, u64* __restrict__ cursors,
              u64* __restrict__ out, i64 chunk_records, int check)
{
  __shared__ int s_last;
  const i64 chunk_words = 2 + chunk_records * stride;
  const i64 last = cap + (i64)ctrl->dense_slots;
  const u32 lane = threadIdx.x & 31u;
  for (i64 s0 = (i64)blockIdx.x * blockDim.x + (threadIdx.x - lane); s0 <= last; s0 += (i64)gridDim.x * blockDim.x) {
    const i64 s = s0 + lane;
    u32 dest = NO_DEST;
    u64 key = 0;
    SlotRef src{nullptr, nullptr, 0};
    if (s <= last) {
      src = slot_ref(const_cast<u64*>(tbl), cap, stride, last - cap, s);
      key = s != cap ? *src.key : EMPTY;
      const bool occ = s != cap ? key != EMPTY : ctrl->special_used != 0;
      if (occ) dest = owner_of(mix64(key), (u32)nparts);
    }
    const u64 pos = warp_add_by_dest(cursors, dest);  // lanes of one destination reserve together
    if (dest == NO_DEST || pos >= (u64)chunk_records) continue;
    u64* dst = out + (i64)dest * chunk_words + 2 + (i64)pos * stride;
    dst[0] = key;
    for (int c = 1; c < stride; ++c) dst[c] = src.cells[(i64)(c - 1) * src.step];
  }
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) s_last = atomicAdd(&cursors[nparts], 1ull) == (u64)gridDim.x - 1;
  __syncthreads();
  if (!s_last) return;
  __threadfence();
  __shared__ int s_over;
  if (threadIdx.x == 0) s_over = 0;
  __syncthreads();
  for (int p = threadIdx.x; p < nparts; p += blockDim.x)
    if (__ldcg(&cursors[p]) > (u64)chunk_records) s_over = 1;
  __syncthreads();
  bool over = s_over != 0;
  if ((check & 1) && (ctrl->overflow != 0 || ctrl->error != 0)) over = true;
  if ((check & 2) && ctrl->dense.enabled == 0) over = true;
  for (int p = threadIdx.x; p < nparts; p += blockDim.x) {
    out[(i64)p * chunk_words]     = over ? 0ull : __ldcg(&cursors[p]);
    out[(i64)p * chunk_words + 1] = over ? 1ull : 0ull;
  }
}

__global__ void __launch_bounds__(256)
k_merge_chunks(const __grid_constant__ DPlan P, u64* __restrict__ tbl, i64 cap, DCtrl* ctrl,
               const u64* __restrict__ chunks, int nchunks, i64 chunk_records)
{
  __shared__ int s_new;
  if (threadIdx.x == 0) s_new = 0;
  __syncthreads();
  const int stride = P.stride;
  const i64 chunk_words = 2 + chunk_records * stride;
  const i64 total = (i64)nchunks * chunk_records;
  for (i64 i = (i64)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (i64)gridDim.x * blockDim.x) {
    const i64 c = i / chunk_records, r = i - c * chunk_records;
    const u64* chunk = chunks + c * chunk_words;
    if (r == 0 && chunk[1] != 0) atomicMax(&ctrl->chunk_overflow, chunk[1]);  // 1 = too many records, 2 = the sender failed
    if ((u64)r >= chunk[0] || chunk[1] != 0) continue;
    const u64* rec = chunk + 2 + r * stride;
    const u64 key  = rec[0];
    const i64 g    = table_slot_packed(P, tbl, cap, stride, key, ctrl, &s_new);
    if (g < 0) continue;
    const SlotRef slot = slot_ref(tbl, cap, stride, (i64)ctrl->dense_slots, g);
    for (int k = 0; k < P.ncells; ++k) {
      const int op = P.cells[k].op;
      const u64 a  = rec[1 + k];
      if (a != cell_identity(op)) cell_merge(slot.cells + (i64)k * slot.step, op, a);
    }
  }
  __syncthreads();
  if (threadIdx.x == 0 && s_new) {
    const u64 tot = atomicAdd(&ctrl->nclaimed, (u64)s_new) + (u64)s_new;
    if (tot > ctrl->claim_limit) ctrl->overflow = 1;
  }
}

// merge packed partial records into a table (packed keys)
__global__ void __launch_bounds__(256)
k_merge(const __grid_constant__ DPlan P, u64* __restrict__ tbl, i64 cap, DCtrl* ctrl, const u64* __restrict__ recs,
        i64 nrecs)
{
  __shared__ int s_new;
  if (threadIdx.x == 0) s_new = 0;
  __syncthreads();
  const int stride = P.stride;
  for (i64 r = (i64)blockIdx.x * blockDim.x + threadIdx.x; r < nrecs; r += (i64)gridDim.x * blockDim.x) {
    const u64* rec = recs + r * stride;
    const u64 key  = rec[0];
    const i64 g    = table_slot_packed(P, tbl, cap, stride, key, ctrl, &s_new);
    if (g < 0) continue;
    const SlotRef slot = slot_ref(tbl, cap, stride, (i64)ctrl->dense_slots, g);
    for (int c = 0; c < P.ncells; ++c) {
      const int op = P.cells[c].op;
      const u64 a  = rec[1 + c];
      if (a != cell_identity(op)) cell_merge(slot.cells + (i64)c * slot.step, op, a);
    }
  }
  __syncthreads();
  if (threadIdx.x == 0 && s_new) {
    const u64 tot = atomicAdd(&ctrl->nclaimed, (u64)s_new) + (u64)s_new;
    if (tot > ctrl->claim_limit) ctrl->overflow = 1;
  }
}


// ------------------------------------------------------------------------------ row hash partition
// cudf::hash_partition (cpp/src/partitioning/partitioning.cu:120-337,569-750): partition of a row =
// row hash % partitions, the hash being the reference's (ref_row_hash: MurmurHash3_x86_32 + hash_combine,
// or the identity hash).  Three steps: rows per (partition, CTA) -> exclusive scan on the device ->
// permutation "output position -> input row" -> gather of every column by that permutation (the
// reference's general path gathers too, :750; its shared-memory fast path is limited to fixed-width
// tables and 1024 partitions, :253-337).  Rows keep their input order inside a (partition, CTA) run
// only up to the order of the shared-memory atomics: the order inside a partition is unspecified.
constexpr int PART_BLOCK    = 512;
constexpr int MAX_PART_COLS = 32;

struct DPartPlan {
  int nparts;
  int hash_kind;   // RefHash
  u32 seed;
  int counters_in_global;  // per-CTA partition counters live in global memory (more partitions than shared memory holds)
  i64 rows_per_cta;
};

__device__ __forceinline__ u32 row_partition(const DPlan& P, const DPartPlan& Q, i64 row)
{
  const u32 h = ref_row_hash(P, row, Q.hash_kind, Q.seed);
  return (Q.nparts & (Q.nparts - 1)) == 0 ? (h & (u32)(Q.nparts - 1)) : h % (u32)Q.nparts;
}

// counts[p * gridDim.x + cta] = rows of this CTA's slice that go to partition p (partition-major, so that
// one exclusive scan over the array gives every (partition, CTA) run its start)
__global__ void __launch_bounds__(PART_BLOCK)
k_partition_count(const __grid_constant__ DPlan P, const DPartPlan Q, i64* __restrict__ counts, u32* __restrict__ cta_scratch)
{
  extern __shared__ u32 s_hist[];
  const bool in_global = Q.counters_in_global != 0;
  u32* hist = in_global ? cta_scratch + (size_t)blockIdx.x * Q.nparts : s_hist;  // (global slices arrive zeroed)
  if (!in_global) for (int p = threadIdx.x; p < Q.nparts; p += blockDim.x) hist[p] = 0;
  __syncthreads();
  const i64 lo = (i64)blockIdx.x * Q.rows_per_cta;
  const i64 hi = min(P.nrows, lo + Q.rows_per_cta);
  const u32 lane = threadIdx.x & 31u;
  // four rows per thread and step, their loads in flight together
  for (i64 r0 = lo + (threadIdx.x - lane); r0 < hi; r0 += 4 * (i64)blockDim.x) {
    u32 p[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const i64 r = r0 + (i64)u * blockDim.x + lane;
      p[u] = r < hi ? row_partition(P, Q, r) : NO_DEST;
    }
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      // lanes headed for the same partition add once (with few partitions every lane would hit the same words)
      const u32 peers = __match_any_sync(0xFFFFFFFFu, p[u]);
      if (p[u] != NO_DEST && (int)lane == __ffs(peers) - 1) atomicAdd(&hist[p[u]], (u32)__popc(peers));
    }
  }
  __syncthreads();
  for (int p = threadIdx.x; p < Q.nparts; p += blockDim.x) counts[(size_t)p * gridDim.x + blockIdx.x] = (i64)hist[p];
}

// offsets[p] = start of partition p (its first (partition, CTA) run), offsets[nparts] = the row count
__global__ void k_partition_offsets(const i64* __restrict__ starts, int nparts, int grid, i64* __restrict__ offsets)
{
  for (int p = blockIdx.x * blockDim.x + threadIdx.x; p <= nparts; p += gridDim.x * blockDim.x)
    offsets[p] = starts[(size_t)p * grid];  // (p == nparts reads the scan's closing total)
}

// Fixed-width columns without a null mask are moved by the kernel that places the rows: it reads them in row
// order (coalesced) and writes each row to its output position — the rows of one partition inside a warp go
// to consecutive positions — instead of being gathered through the permutation afterwards, which reads every
// sector of a source column once per partition that has a row in it.
struct DDirectCols {
  int n;
  int width[MAX_PART_COLS];
  const unsigned char* src[MAX_PART_COLS];  // first element of the view
  unsigned char* dst[MAX_PART_COLS];
};

// perm[output position] = input row (when `perm` is given), and the direct columns moved
__global__ void __launch_bounds__(PART_BLOCK)
k_partition_perm(const __grid_constant__ DPlan P, const DPartPlan Q, const i64* __restrict__ starts, u32* __restrict__ cta_scratch,
                 int* __restrict__ perm, const __grid_constant__ DDirectCols D)
{
  extern __shared__ u32 s_cur[];
  const bool in_global = Q.counters_in_global != 0;
  u32* cur = in_global ? cta_scratch + (size_t)blockIdx.x * Q.nparts : s_cur;  // (global slices arrive zeroed)
  if (!in_global) for (int p = threadIdx.x; p < Q.nparts; p += blockDim.x) cur[p] = 0;
  __syncthreads();
  const i64 lo = (i64)blockIdx.x * Q.rows_per_cta;
  const i64 hi = min(P.nrows, lo + Q.rows_per_cta);
  const u32 lane = threadIdx.x & 31u;
  for (i64 r0 = lo + (threadIdx.x - lane); r0 < hi; r0 += blockDim.x) {
    const i64 r = r0 + lane;
    const u32 p = r < hi ? row_partition(P, Q, r) : NO_DEST;
    const u32 peers = __match_any_sync(0xFFFFFFFFu, p);
    const int lead  = __ffs(peers) - 1;
    u32 base = 0;
    if (p != NO_DEST && (int)lane == lead) base = atomicAdd(&cur[p], (u32)__popc(peers));
    base = __shfl_sync(0xFFFFFFFFu, base, lead);
    if (p == NO_DEST) continue;
    const i64 d = starts[(size_t)p * gridDim.x + blockIdx.x] + (i64)base + __popc(peers & ((1u << lane) - 1u));
    if (perm) perm[d] = (int)r;
    for (int c = 0; c < D.n; ++c) {
      switch (D.width[c]) {
        case 8: ((u64*)D.dst[c])[d] = __ldg((const u64*)D.src[c] + r); break;
        case 4: ((u32*)D.dst[c])[d] = __ldg((const u32*)D.src[c] + r); break;
        case 2: ((unsigned short*)D.dst[c])[d] = __ldg((const unsigned short*)D.src[c] + r); break;
        default: D.dst[c][d] = D.src[c][r]; break;
      }
    }
  }
}

// out[i] = src[offset + perm[i]] for a fixed-width column (W bytes per element), validity gathered into whole
// mask words by ballot
template <typename T>
__global__ void k_gather_column(const T* __restrict__ src, const u32* __restrict__ src_mask, i64 src_offset,
                                const int* __restrict__ perm, i64 n, T* __restrict__ dst, u32* __restrict__ dst_mask)
{
  const u32 lane = threadIdx.x & 31u;
  const i64 nround = (n + 31) / 32 * 32;
  for (i64 i = (i64)blockIdx.x * blockDim.x + threadIdx.x; i < nround; i += (i64)gridDim.x * blockDim.x) {
    bool valid = false;
    if (i < n) {
      const i64 idx = src_offset + perm[i];
      dst[i] = src[idx];
      valid = !src_mask || bit_valid(src_mask, idx);
    }
    if (dst_mask) {
      const u32 word = __ballot_sync(0xFFFFFFFFu, valid);
      if (lane == 0) dst_mask[i >> 5] = word;
    }
  }
}

// validity bitmask <-> one byte per row (a row exchange moves validity as bytes: partitions start at
// arbitrary bit positions)
__global__ void k_mask_to_bytes(const u32* __restrict__ mask, i64 offset, i64 n, unsigned char* __restrict__ out)
{
  for (i64 i = (i64)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (i64)gridDim.x * blockDim.x)
    out[i] = bit_valid(mask, offset + i) ? 1 : 0;
}
__global__ void k_bytes_to_mask(const unsigned char* __restrict__ bytes, i64 n, u32* __restrict__ mask, u32* null_count)
{
  const i64 nwords = (n + 31) / 32;
  const int lane = threadIdx.x & 31;
  const i64 warp0 = ((i64)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const i64 nwarps = ((i64)gridDim.x * blockDim.x) >> 5;
  u32 nulls = 0;
  for (i64 w = warp0; w < nwords; w += nwarps) {
    const i64 i = w * 32 + lane;
    const bool v = i < n && bytes[i] != 0;
    const u32 word = __ballot_sync(0xFFFFFFFFu, v);
    if (lane == 0) {
      mask[w] = word;
      const int valid_bits = (int)min((i64)32, n - w * 32);
      nulls += (u32)(valid_bits - __popc(word));
    }
  }
  if (lane == 0 && nulls) atomicAdd(null_count, nulls);
}

}  // namespace b2
