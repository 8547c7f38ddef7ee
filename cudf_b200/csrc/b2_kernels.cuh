// b2_kernels.cuh — the CUDA kernels of the groupby engine (sm_100a).
//
//   k_table_init     identity-fills a table (replaces the per-column thrust::fill of
//                    cpp/src/aggregation/aggregation.cu:87-97 and the cuco slot memset)
//   k_aggregate      ONE fused pass over keys + values + bitmasks: per-CTA shared-memory
//                    open-addressing table in front of the global-memory table
//                    (replaces mapping_indices_kernel + single_pass_shmem_aggs_kernel +
//                    the global-memory functors: cpp/src/groupby/hash/compute_mapping_indices.cuh:92-151,
//                    compute_shared_memory_aggs.cu:260-353, single_pass_functors.cuh:86-157)
//   k_finalize       compaction of occupied slots + key decode + compound finalisers + result
//                    null masks in one pass (replaces retrieve_all, key gather, binary DIV,
//                    m2/var/std tabulate and null-count kernels: output_utils.cu:139-224,
//                    hash_compound_agg_finalizer.cu:93-186, common/m2_var_std.cu:49-59,160-187)
//   k_gather_*       key gather for row-keyed tables (fixed width and strings)
//   k_pack_* / k_merge   hash partition of partial records by owner and merge of partial records
//                    (cpp/src/partitioning/partitioning.cu:120-337, streaming_groupby/merge.cu:91-142)
#pragma once
#include "b2_device.cuh"

namespace b2 {

constexpr int AGG_BLOCK      = 1024;  // threads per CTA of the fused kernel (one CTA per SM)
constexpr int AGG_ROWS       = 4;     // rows per thread per tile
constexpr int SMEM_PROBES    = 48;    // probe limit of the shared-memory table
constexpr int GMEM_PROBES    = 2048;  // probe limit of the global table before "overflow"
constexpr u32 F32_SPILL_AT   = 1024;  // packed {f32 sum, u32 n} cells spill to fp64 at this count
constexpr int SLOT_NONE      = -1;

enum SmemLayout : int { SL_NONE = 0, SL_GENERIC = 1, SL_F32MEAN = 2 };

// ------------------------------------------------------------------------------ table init
__global__ void k_table_init(u64* __restrict__ tbl, i64 nslots, const __grid_constant__ DPlan P)
{
  const int stride = P.stride;
  for (i64 s = (i64)blockIdx.x * blockDim.x + threadIdx.x; s < nslots; s += (i64)gridDim.x * blockDim.x) {
    u64* slot = tbl + s * stride;
    slot[0]   = EMPTY;
    for (int c = 0; c < P.ncells; ++c) slot[1 + c] = cell_identity(P.cells[c].op);
  }
}

// ------------------------------------------------------------------------------ probing
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

// ------------------------------------------------------------------------------ fused aggregate
// One pass over the input.  Each CTA owns a shared-memory table (cache) of S slots; a row whose key
// is cached is folded into shared memory, every other row goes to the global table.  The cache
// fills first-come until `fill_limit`; a CTA whose cache stops paying off (mostly misses) turns it
// off.  At the end each CTA merges its cache into the global table.
template <int KM, int LAYOUT>
__global__ void __launch_bounds__(AGG_BLOCK, 1)
k_aggregate(const __grid_constant__ DPlan P, u64* __restrict__ tbl, i64 cap, DCtrl* ctrl, int S, int fill_limit)
{
  extern __shared__ __align__(16) unsigned char smem_raw[];
  __shared__ int s_fill, s_new, s_cache_on, s_abort, s_hit, s_miss;

  u64* skeys  = (u64*)smem_raw;            // [S+1]
  u64* scells = skeys + (S + 1);           // SL_GENERIC: [ncells][S+1]; SL_F32MEAN: [S+1] packed {f32,u32}
  const int stride = P.stride;
  const int tid    = threadIdx.x;

  if (LAYOUT != SL_NONE) {
    for (int i = tid; i <= S; i += blockDim.x) skeys[i] = EMPTY;
    if (LAYOUT == SL_GENERIC) {
      for (int c = 0; c < P.ncells; ++c) {
        const u64 id = cell_identity(P.cells[c].op);
        for (int i = tid; i <= S; i += blockDim.x) scells[(size_t)c * (S + 1) + i] = id;
      }
    } else {
      for (int i = tid; i <= S; i += blockDim.x) scells[i] = 0;
    }
  }
  if (tid == 0) { s_fill = 0; s_new = 0; s_cache_on = (LAYOUT != SL_NONE); s_abort = 0; s_hit = 0; s_miss = 0; }
  __syncthreads();

  const i64 tile_rows = (i64)blockDim.x * AGG_ROWS;
  const i64 ntiles    = (P.nrows + tile_rows - 1) / tile_rows;

  for (i64 tile = blockIdx.x; tile < ntiles; tile += gridDim.x) {
    const i64 base = tile * tile_rows;
    const bool cache_on = (LAYOUT != SL_NONE) && s_cache_on;

    // ---- phase A: key -> slot
    int sl[AGG_ROWS];
    u64 kk[AGG_ROWS];
    bool act[AGG_ROWS];
#pragma unroll
    for (int j = 0; j < AGG_ROWS; ++j) {
      const i64 row = base + (i64)j * blockDim.x + tid;
      act[j]        = row < P.nrows && row_active(P, row);
      kk[j]         = 0;
      if (act[j]) kk[j] = (KM == KM_PACKED) ? pack_key(P, row) : hash_row(P, row);
    }
    int n_hit = 0, n_miss = 0;
#pragma unroll
    for (int j = 0; j < AGG_ROWS; ++j) {
      sl[j] = SLOT_NONE;
      if (!act[j]) continue;
      const i64 row = base + (i64)j * blockDim.x + tid;
      const u64 h   = (KM == KM_PACKED) ? mix64(kk[j]) : kk[j];
      int s = -1;
      if (cache_on) s = smem_find_insert<KM>(P, skeys, S, fill_limit, &s_fill, kk[j], h, row);
      if (s >= 0) {
        sl[j] = s;
        ++n_hit;
      } else {
        const i64 g = (KM == KM_PACKED) ? gmem_find_insert_packed(tbl, cap, stride, kk[j], h, ctrl, &s_new)
                                        : gmem_find_insert_rows(P, tbl, cap, stride, row, h, ctrl, &s_new);
        if (g >= 0) sl[j] = -2 - (int)g;
        ++n_miss;
      }
    }

    // ---- phase B: fold the values
    if (LAYOUT == SL_F32MEAN) {
      // cells: [0] = Σx of a FLOAT32 column, [1] = n of the same column
      const DValCol& vc = P.vals[P.cells[0].col];
#pragma unroll
      for (int j = 0; j < AGG_ROWS; ++j) {
        if (sl[j] == SLOT_NONE) continue;
        const i64 row = base + (i64)j * blockDim.x + tid;
        if (!value_valid(vc, row)) continue;
        const float x = __ldg((const float*)vc.data + vc.offset + row);
        if (sl[j] >= 0) {
          u64* cell = scells + sl[j];
          u64 old = *(volatile u64*)cell, assumed, next;
          float spill_sum = 0.f;
          bool spill;
          do {
            assumed         = old;
            const float s   = __uint_as_float((u32)assumed) + x;
            const u32 n     = (u32)(assumed >> 32) + 1u;
            spill           = n >= F32_SPILL_AT;
            spill_sum       = s;
            next            = spill ? 0ull : (((u64)n << 32) | (u64)__float_as_uint(s));
            old             = atomicCAS(cell, assumed, next);
          } while (old != assumed);
          if (spill) {
            // move the fp32 partial of this key to the fp64 global cells so that no fp32 sum
            // ever holds more than F32_SPILL_AT addends
            const u64 key = skeys[sl[j]];
            const i64 g   = (sl[j] == S) ? cap
                                         : gmem_find_insert_packed(tbl, cap, stride, key, mix64(key), ctrl, &s_new);
            if (sl[j] == S && ctrl->special_used == 0) ctrl->special_used = 1;
            if (g >= 0) {
              atomicAdd((double*)(tbl + g * stride + 1), (double)spill_sum);
              atomicAdd(tbl + g * stride + 2, (u64)F32_SPILL_AT);
            }
          }
        } else {
          u64* slot = tbl + (i64)(-2 - sl[j]) * stride;
          atomicAdd((double*)(slot + 1), (double)x);
          atomicAdd(slot + 2, 1ull);
        }
      }
    } else {
      int cur_col = -1;
      u64 v[AGG_ROWS];
      bool ok[AGG_ROWS];
      for (int c = 0; c < P.ncells; ++c) {
        const int op  = P.cells[c].op;
        const int col = P.cells[c].col;
        if (op != OP_CNT_A && col != cur_col) {
          cur_col = col;
          const DValCol& vc = P.vals[col];
#pragma unroll
          for (int j = 0; j < AGG_ROWS; ++j) {
            const i64 row = base + (i64)j * blockDim.x + tid;
            ok[j]         = sl[j] != SLOT_NONE && value_valid(vc, row);
            v[j]          = ok[j] ? load_value(vc, row) : 0;
          }
        }
#pragma unroll
        for (int j = 0; j < AGG_ROWS; ++j) {
          if (sl[j] == SLOT_NONE) continue;
          if (op != OP_CNT_A && !ok[j]) continue;
          u64* cell = (LAYOUT == SL_GENERIC && sl[j] >= 0) ? scells + (size_t)c * (S + 1) + sl[j]
                                                          : tbl + (i64)(-2 - sl[j]) * stride + 1 + c;
          cell_update(cell, op, v[j]);
        }
      }
    }

    // ---- per-tile bookkeeping: claims, overflow, cache pay-off
    n_hit  = __reduce_add_sync(0xFFFFFFFFu, n_hit);
    n_miss = __reduce_add_sync(0xFFFFFFFFu, n_miss);
    if ((tid & 31) == 0) { if (n_hit) atomicAdd(&s_hit, n_hit); if (n_miss) atomicAdd(&s_miss, n_miss); }
    __syncthreads();
    if (tid == 0) {
      if (s_new) {
        const u64 tot = atomicAdd(&ctrl->nclaimed, (u64)s_new) + (u64)s_new;
        if (tot > ctrl->claim_limit) ctrl->overflow = 1;
        s_new = 0;
      }
      if (*(volatile u32*)&ctrl->overflow) s_abort = 1;
      if (LAYOUT != SL_NONE && s_cache_on && s_fill >= fill_limit && s_miss > 3 * s_hit) s_cache_on = 0;
      atomicAdd(&ctrl->stat_smem_rows, (u64)s_hit);
      atomicAdd(&ctrl->stat_gmem_rows, (u64)s_miss);
      s_hit = 0; s_miss = 0;
    }
    __syncthreads();
    if (s_abort) break;
  }

  // ---- merge this CTA's cache into the global table
  if (LAYOUT != SL_NONE) {
    __syncthreads();
    if (!s_abort) {
      for (int i = tid; i <= S; i += blockDim.x) {
        const u64 k = skeys[i];
        if (k == EMPTY) continue;
        i64 g;
        if (i == S) {
          g = cap;
          if (ctrl->special_used == 0) ctrl->special_used = 1;
        } else if (KM == KM_PACKED) {
          g = gmem_find_insert_packed(tbl, cap, stride, k, mix64(k), ctrl, &s_new);
        } else {
          const i64 row = (i64)(u32)k;
          g = gmem_find_insert_rows(P, tbl, cap, stride, row, hash_row(P, row), ctrl, &s_new);
        }
        if (g < 0) continue;
        u64* slot = tbl + g * stride;
        if (LAYOUT == SL_F32MEAN) {
          const u64 a = scells[i];
          const u32 n = (u32)(a >> 32);
          if (n) {
            atomicAdd((double*)(slot + 1), (double)__uint_as_float((u32)a));
            atomicAdd(slot + 2, (u64)n);
          }
        } else {
          for (int c = 0; c < P.ncells; ++c) {
            const int op = P.cells[c].op;
            const u64 a  = scells[(size_t)c * (S + 1) + i];
            if (a != cell_identity(op)) cell_merge(slot + 1 + c, op, a);
          }
        }
      }
    }
    __syncthreads();
    if (tid == 0 && s_new) {
      const u64 tot = atomicAdd(&ctrl->nclaimed, (u64)s_new) + (u64)s_new;
      if (tot > ctrl->claim_limit) ctrl->overflow = 1;
    }
  }
}

// ------------------------------------------------------------------------------ finalize
enum OutKind : int {
  OK_COUNT = 0,  // int32 from a count cell
  OK_INT,        // integer cell (Σ, Σx², Π, min, max of integers) stored in the result width
  OK_FLT,        // double cell (Σ, Σx², Π of floats) stored as FLOAT32/FLOAT64
  OK_MINMAX_F,   // ordered-encoded double cell
  OK_MEAN, OK_M2, OK_VAR, OK_STD
};

struct DOutCol {
  void* data;
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

__global__ void k_finalize(const __grid_constant__ DPlan P, const __grid_constant__ DOutPlan O,
                           const u64* __restrict__ tbl, i64 cap, DCtrl* ctrl)
{
  const int stride = P.stride;
  const i64 nslots = cap + 1;
  const i64 nwarp_iters = (nslots + 31) / 32;
  const int lane = threadIdx.x & 31;
  const i64 warp0 = ((i64)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const i64 nwarps = ((i64)gridDim.x * blockDim.x) >> 5;
  for (i64 w = warp0; w < nwarp_iters; w += nwarps) {
    const i64 s = w * 32 + lane;
    u64 key = EMPTY;
    bool occ = false;
    if (s < cap) { key = tbl[s * stride]; occ = key != EMPTY; }
    else if (s == cap) { occ = ctrl->special_used != 0; }
    const u32 m = __ballot_sync(0xFFFFFFFFu, occ);
    if (m == 0) continue;
    u64 base = 0;
    if (lane == 0) base = atomicAdd(&ctrl->out_cursor, (u64)__popc(m));
    base = __shfl_sync(0xFFFFFFFFu, base, 0);
    if (!occ) continue;
    const i64 g = (i64)base + __popc(m & ((1u << lane) - 1u));
    const u64* cells = tbl + s * stride + 1;

    // keys
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

    // results
    for (int o = 0; o < O.nouts; ++o) {
      const DOutCol& oc = O.outs[o];
      const i64 n = oc.c_cnt >= 0 ? (i64)cells[oc.c_cnt] : 1;
      bool valid  = n > 0;
      switch (oc.kind) {
        case OK_COUNT: ((int*)oc.data)[g] = (int)cells[oc.c_a]; valid = true; break;
        case OK_INT: store_int(oc.data, g, oc.rclass, valid ? cells[oc.c_a] : 0); break;
        case OK_FLT: store_flt(oc.data, g, oc.rclass, valid ? __longlong_as_double((i64)cells[oc.c_a]) : 0.0); break;
        case OK_MINMAX_F:
          store_flt(oc.data, g, oc.rclass, valid ? __longlong_as_double((i64)f64_unordered(cells[oc.c_a])) : 0.0);
          break;
        case OK_MEAN: {
          if (oc.rclass != VC_F64) {  // durations: integer division in the source type
            store_int(oc.data, g, oc.rclass, valid ? (u64)((i64)cells[oc.c_a] / n) : 0);
            break;
          }
          const double s = oc.src_float ? __longlong_as_double((i64)cells[oc.c_a]) : (double)(i64)cells[oc.c_a];
          ((double*)oc.data)[g] = valid ? s / (double)n : 0.0;
          break;
        }
        default: {  // M2, VAR, STD
          double m2 = 0.0;
          if (n > 0) {
            const double s  = oc.src_float ? __longlong_as_double((i64)cells[oc.c_a]) : (double)(i64)cells[oc.c_a];
            const double ss = oc.src_float ? __longlong_as_double((i64)cells[oc.c_b]) : (double)(i64)cells[oc.c_b];
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
    if (c.mask && !bit_valid(c.mask, idx)) {
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

template <typename OffT>
__global__ void k_string_copy(DKeyCol c, const int* __restrict__ rows, i64 ngroups, const i64* __restrict__ offs,
                              OffT* __restrict__ out_offs, unsigned char* __restrict__ chars)
{
  // one warp per string
  const int lane = threadIdx.x & 31;
  const i64 warp0 = ((i64)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const i64 nwarps = ((i64)gridDim.x * blockDim.x) >> 5;
  for (i64 g = warp0; g <= ngroups; g += nwarps) {
    if (lane == 0) out_offs[g] = (OffT)offs[g];
    if (g == ngroups) break;
    const i64 len = offs[g + 1] - offs[g];
    if (len == 0) continue;
    const i64 idx = c.offset + rows[g];
    const unsigned char* src = c.data + str_offset(c, idx);
    unsigned char* dst = chars + offs[g];
    for (i64 b = lane; b < len; b += 32) dst[b] = src[b];
  }
}

// ------------------------------------------------------------------------------ partial records
// owner partition of every occupied slot: counts, then scatter into destination-major order
__global__ void k_pack_count(const u64* __restrict__ tbl, i64 cap, int stride, int nparts, const DCtrl* ctrl,
                             u64* __restrict__ counts)
{
  extern __shared__ u64 s_cnt[];
  for (int p = threadIdx.x; p < nparts; p += blockDim.x) s_cnt[p] = 0;
  __syncthreads();
  for (i64 s = (i64)blockIdx.x * blockDim.x + threadIdx.x; s <= cap; s += (i64)gridDim.x * blockDim.x) {
    const u64 key = s < cap ? tbl[s * stride] : EMPTY;
    const bool occ = s < cap ? key != EMPTY : ctrl->special_used != 0;
    if (occ) atomicAdd(&s_cnt[owner_of(mix64(key), (u32)nparts)], 1ull);
  }
  __syncthreads();
  for (int p = threadIdx.x; p < nparts; p += blockDim.x)
    if (s_cnt[p]) atomicAdd(&counts[p], s_cnt[p]);
}

__global__ void k_pack_scatter(const u64* __restrict__ tbl, i64 cap, int stride, int nparts, const DCtrl* ctrl,
                               u64* __restrict__ cursors /* start offsets, advanced */, u64* __restrict__ out)
{
  for (i64 s = (i64)blockIdx.x * blockDim.x + threadIdx.x; s <= cap; s += (i64)gridDim.x * blockDim.x) {
    const u64 key = s < cap ? tbl[s * stride] : EMPTY;
    const bool occ = s < cap ? key != EMPTY : ctrl->special_used != 0;
    if (!occ) continue;
    const u64 pos = atomicAdd(&cursors[owner_of(mix64(key), (u32)nparts)], 1ull);
    u64* dst = out + pos * stride;
    const u64* src = tbl + s * stride;
    dst[0] = key;
    for (int c = 1; c < stride; ++c) dst[c] = src[c];
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
    const i64 g    = gmem_find_insert_packed(tbl, cap, stride, key, mix64(key), ctrl, &s_new);
    if (g < 0) continue;
    u64* slot = tbl + g * stride;
    for (int c = 0; c < P.ncells; ++c) {
      const int op = P.cells[c].op;
      const u64 a  = rec[1 + c];
      if (a != cell_identity(op)) cell_merge(slot + 1 + c, op, a);
    }
  }
  __syncthreads();
  if (threadIdx.x == 0 && s_new) {
    const u64 tot = atomicAdd(&ctrl->nclaimed, (u64)s_new) + (u64)s_new;
    if (tot > ctrl->claim_limit) ctrl->overflow = 1;
  }
}


// ------------------------------------------------------------------------------ row hash partition
// cudf::hash_partition for fixed-width tables (cpp/src/partitioning/partitioning.cu:120-337):
// pass 1 counts rows per (CTA, partition); the host turns the counts into CTA-major start offsets
// inside each partition; pass 2 recomputes the partition of each row and scatters every column.
constexpr int PART_BLOCK    = 512;
constexpr int MAX_PART_COLS = 32;

struct DPartCol {
  const unsigned char* src; const u32* mask; i64 offset; int width; int pad;
  unsigned char* dst; u32* dst_mask;
};
struct DPartPlan {
  int ncols; int nparts;
  i64 rows_per_cta;
  DPartCol cols[MAX_PART_COLS];
};

__device__ __forceinline__ u32 row_partition(const DPlan& P, i64 row, u32 nparts)
{
  const u64 h = (P.key_mode == KM_PACKED) ? mix64(pack_key(P, row)) : hash_row(P, row);
  return owner_of(h, nparts);
}

__global__ void __launch_bounds__(PART_BLOCK)
k_partition_count(const __grid_constant__ DPlan P, DPartPlan Q, u32* __restrict__ cta_counts /* [grid][nparts] */)
{
  extern __shared__ u32 s_hist[];
  for (int p = threadIdx.x; p < Q.nparts; p += blockDim.x) s_hist[p] = 0;
  __syncthreads();
  const i64 lo = (i64)blockIdx.x * Q.rows_per_cta;
  const i64 hi = min(P.nrows, lo + Q.rows_per_cta);
  for (i64 r = lo + threadIdx.x; r < hi; r += blockDim.x) atomicAdd(&s_hist[row_partition(P, r, (u32)Q.nparts)], 1u);
  __syncthreads();
  for (int p = threadIdx.x; p < Q.nparts; p += blockDim.x) cta_counts[(size_t)blockIdx.x * Q.nparts + p] = s_hist[p];
}

__global__ void __launch_bounds__(PART_BLOCK)
k_partition_scatter(const __grid_constant__ DPlan P, const __grid_constant__ DPartPlan Q,
                    const i64* __restrict__ cta_starts /* [grid][nparts] */)
{
  extern __shared__ u32 s_hist[];  // cursor inside this CTA's share of each partition
  for (int p = threadIdx.x; p < Q.nparts; p += blockDim.x) s_hist[p] = 0;
  __syncthreads();
  const i64 lo = (i64)blockIdx.x * Q.rows_per_cta;
  const i64 hi = min(P.nrows, lo + Q.rows_per_cta);
  for (i64 r = lo + threadIdx.x; r < hi; r += blockDim.x) {
    const u32 p   = row_partition(P, r, (u32)Q.nparts);
    const i64 dst = cta_starts[(size_t)blockIdx.x * Q.nparts + p] + atomicAdd(&s_hist[p], 1u);
    for (int c = 0; c < Q.ncols; ++c) {
      const DPartCol& col = Q.cols[c];
      const i64 idx = col.offset + r;
      switch (col.width) {
        case 1: col.dst[dst] = col.src[idx]; break;
        case 2: ((unsigned short*)col.dst)[dst] = ((const unsigned short*)col.src)[idx]; break;
        case 4: ((u32*)col.dst)[dst] = ((const u32*)col.src)[idx]; break;
        default: ((u64*)col.dst)[dst] = ((const u64*)col.src)[idx]; break;
      }
      if (col.dst_mask && bit_valid(col.mask, idx)) atomicOr(col.dst_mask + (dst >> 5), 1u << (dst & 31));
    }
  }
}

}  // namespace b2
