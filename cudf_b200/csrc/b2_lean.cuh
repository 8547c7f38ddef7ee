// b2_lean.cuh — the lean instantiation of the fused aggregate pass: "Σ and n of one FLOAT32 or FLOAT64
// column" (a mean) over 1..3 fixed-width key columns whose sampled key box fits shared memory.
//
//   k_aggregate_lean<NK, K8, STAGED, KEY_MASKS, V8>
//     replaces mapping_indices_kernel + single_pass_shmem_aggs_kernel for this shape
//     (cpp/src/groupby/hash/compute_mapping_indices.cuh:92-151, compute_shared_memory_aggs.cu:260-353).
//
// It is a kernel of its own, not a branch of k_aggregate, so that its register allocation is decided
// by its row loop alone: everything rare (keys outside the sampled box, rows whose value is null,
// the fp32 -> fp64 spill of a long partial sum, the ragged end of the input) lives in __noinline__
// functions.  One CTA per SM, 4 consecutive rows per thread per tile, two native shared-memory
// atomics per row into the CTA's direct-indexed table {fp32 partial sum, u32 count}.
//
//   V8 = true : the value column is FLOAT64.  A 64-bit floating-point add in shared memory is a
//               compare-and-swap loop, so the partial sum of a slot is kept as FX_LIMBS signed 32-bit words
//               of fixed point instead (fx_split / fx_add_s): a row costs up to four native 32-bit adds and
//               its count, and the partial sums are exact.  The window of the limbs comes from the largest
//               exponent the key-box sampler saw; a value outside it (or a denormal, an infinity, NaN) is
//               added to the fp64 cell of the global table directly, as a rare row.
//
//   STAGED = false : tiles go global -> registers with 16-byte ld.global.nc, the next tile's vectors
//                    are loaded into a second register set while the current tile is folded;
//   STAGED = true  : one producer warp streams key / value / validity tiles into a shared-memory
//                    ring with cp.async.bulk (no multicast, no tensor map: the columns are flat)
//                    completing on an mbarrier per stage; 31 consumer warps read the tiles from
//                    shared memory.  Every wait is bounded; a wait that runs out sets ctrl->error.
//
// The key box comes from the control block: the sampler runs in k_table_init, which precedes this
// kernel on the stream.  If the box did not fit, the kernel returns at once and the generic
// k_aggregate (always launched behind it) takes the whole input.
#pragma once
#include "b2_kernels.cuh"

namespace b2 {

constexpr int LEAN_STAGED_CONSUMERS = 992;  // 31 consumer warps; warp 31 is the producer
constexpr int LEAN_STAGES           = 2;
constexpr int LEAN_MASK_BYTES       = 512;  // validity bytes of one staged tile, padded
constexpr int LEAN_WAIT_TRIES       = 1 << 20;

// ------------------------------------------------------------------------------ mbarrier / bulk copy
__device__ __forceinline__ void mbar_init(u32 bar, u32 count)
{
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(u32 bar, u32 bytes)
{
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(u32 bar)
{
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(u32 bar, u32 parity)
{
  u32 ok;
  asm volatile("{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}"
               : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
  return ok != 0;
}
// bounded: false when the phase did not complete within LEAN_WAIT_TRIES attempts
__device__ __forceinline__ bool mbar_wait(u32 bar, u32 parity)
{
  for (int i = 0; i < LEAN_WAIT_TRIES; ++i)
    if (mbar_try_wait(bar, parity)) return true;
  return false;
}
// flat global -> shared copy of `bytes` (a multiple of 16; both addresses 16-byte aligned) that
// reports its bytes to `bar`
__device__ __forceinline__ void bulk_g2s(u32 dst, const void* src, u32 bytes, u32 bar)
{
  asm volatile("cp.async.bulk.shared::cta.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}

// ------------------------------------------------------------------------------ rare paths
struct LeanRare {  // what the rare paths need: this CTA's table and the global one
  float* ssum;  // fp32 partial sums, or (V8) the limbs: word i of slot s at ((int*)ssum)[i * nsp + s]
  int nsp, fx_base;
  u32* socc; int* s_new;
  u64* tbl; i64 cap; i64 region; int stride; int special_pos;
  DCtrl* ctrl; const DDense* box;
};

// reports this CTA's unreported slot claims of the hashed region
__device__ __forceinline__ void lean_report_claims(const LeanRare& L)
{
  const int c = atomicExch(L.s_new, 0);
  if (c) {
    const u64 tot = atomicAdd(&L.ctrl->nclaimed, (u64)c) + (u64)c;
    if (tot > L.ctrl->claim_limit) L.ctrl->overflow = 1;
  }
}

// global slot of box position `pos`
__device__ __forceinline__ SlotRef lean_box_slot(const LeanRare& L, u32 pos)
{
  const i64 g = (int)pos == L.special_pos ? L.cap : L.cap + 1 + (i64)pos;
  return slot_ref(L.tbl, L.cap, L.stride, L.region, g);
}

// a row that cannot be folded in shared memory: its key lies outside the sampled box (global hashed
// region), its FLOAT64 value does not fit the window of the limbs, or it belongs to the ragged end of
// the input (in-box keys go to the dense region directly)
__device__ __noinline__ void lean_slow_row(const DPlan& P, const LeanRare& L, i64 row, bool check_active)
{
  if (check_active && !row_active(P, row)) return;
  if (*(volatile u32*)&L.ctrl->overflow) return;  // this attempt will be discarded
  const u64 key = pack_key(P, row);
  const int di  = key != EMPTY ? dense_index(P, *L.box, key) : -1;
  SlotRef ref;
  if (di >= 0) {
    ref = lean_box_slot(L, (u32)di);
    if ((int)di != L.special_pos && *(volatile u64*)ref.key == EMPTY) *(volatile u64*)ref.key = key;
  } else {
    const i64 g = gmem_find_insert_packed(L.tbl, L.cap, L.stride, key, mix64(key), L.ctrl, L.s_new);
    lean_report_claims(L);
    if (g < 0) return;
    ref = slot_ref(L.tbl, L.cap, L.stride, L.region, g);
  }
  const DValCol& vc = P.vals[P.cells[0].col];
  if (value_valid(vc, row)) {
    const double x = vc.vclass == VC_F64 ? __ldg((const double*)vc.data + vc.offset + row)
                                         : (double)__ldg((const float*)vc.data + vc.offset + row);
    atomicAdd((double*)ref.cells, x);
    atomicAdd(ref.cells + ref.step, 1ull);
  }
}

// the rare rows of one 4-row group: active rows whose value is null (the group exists, nothing is
// added) and active rows whose key lies outside the box or whose value lies outside the limbs' window (`bad`)
__device__ __noinline__ void lean_rare_rows(const DPlan& P, const LeanRare& L, u32 rare, u32 bad, i64 r0, u32 d0, u32 d1,
                                            u32 d2, u32 d3)
{
  const u32 ds[4] = {d0, d1, d2, d3};
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    if (!((rare >> j) & 1u)) continue;
    if (!((bad >> j) & 1u)) {
      const u32 s = ds[j];
      if (!((L.socc[s >> 5] >> (s & 31u)) & 1u)) atomicOr(&L.socc[s >> 5], 1u << (s & 31u));
    } else {
      lean_slow_row(P, L, r0 + j, false);
    }
  }
}

// every F32_SPILL_AT-th addend of a shared-memory slot moves its fp32 partial sum to the fp64 global
// cell, so that no fp32 sum ever holds many more addends than that
__device__ __noinline__ void lean_spill(const LeanRare& L, u32 slot, u32 copy_off)
{
  const float part = atomicExch(L.ssum + slot, 0.f);
  atomicAdd((double*)lean_box_slot(L, slot - copy_off).cells, (double)part);
}
// V8: every FX_FLUSH-th addend of a slot empties its limbs into the fp64 global cell, so that no word overflows
__device__ __noinline__ void lean_flush(const LeanRare& L, u32 slot, u32 copy_off)
{
  atomicAdd((double*)lean_box_slot(L, slot - copy_off).cells, fx_take((int*)L.ssum, L.nsp, (int)slot, L.fx_base));
}

// ------------------------------------------------------------------------------ the kernel
template <int NK, bool K8, bool STAGED, bool KEY_MASKS, bool V8>
__global__ void __launch_bounds__(1024, 1)
k_aggregate_lean(const __grid_constant__ DPlan P, u64* __restrict__ tbl, i64 cap, DCtrl* ctrl, u32 region_slots)
{
  extern __shared__ __align__(128) unsigned char smem_raw[];
  __shared__ DDense s_dense;
  __shared__ int s_new, s_last;
  __shared__ __align__(8) u64 s_bars[2 * LEAN_STAGES];

  const int tid = threadIdx.x;
  const bool timekeeper = blockIdx.x == 0 && tid == 0;
  if (timekeeper) ctrl->t_phase[0] = global_timer_ns();
  // the key box sampled by k_table_init
  for (int i = tid; i < (int)(sizeof(DDense) / 4); i += blockDim.x) ((u32*)&s_dense)[i] = ((const u32*)&ctrl->dense)[i];
  if (tid == 0) { s_new = 0; s_last = 0; }
  __syncthreads();
  if (!s_dense.enabled) return;  // no box: the generic kernel behind this one takes the input
  if (timekeeper) ctrl->t_phase[1] = global_timer_ns();

  const int stride  = P.stride;
  const int S       = (int)s_dense.total;
  const int copies  = (int)s_dense.copies;
  const int NS      = S * copies;
  const int NSP     = (NS + 3) & ~3;  // arrays padded to 16 bytes
  const u32 copy_off = (u32)((tid >> 5) % copies) * (u32)S;

  constexpr int SUM_WORDS = V8 ? FX_LIMBS : 1;  // 32-bit words of one slot's partial sum
  constexpr u32 VB = V8 ? 8u : 4u;              // bytes of one value
  float* ssum = (float*)smem_raw;               // [NSP] fp32 partial sums; V8: [FX_LIMBS][NSP] limbs
  u32* scnt   = (u32*)(ssum + SUM_WORDS * NSP); // [NSP] counts
  u32* socc   = scnt + NSP;                     // [(NS + 31) / 32] groups seen through a null value only
  const int nocc = (NS + 31) / 32;
  unsigned char* stage0 = smem_raw + (((size_t)((SUM_WORDS + 1) * NSP + nocc) * 4 + 127) & ~(size_t)127);
  // V8: the window of the limbs, from the largest exponent the sampler saw
  const int fx_base = V8 && s_dense.vexp ? (int)s_dense.vexp - 1 + FX_HEADROOM - FX_MAX_SHIFT : FX_NEVER;

  {
    const int nwords = (SUM_WORDS + 1) * NSP + nocc, nquads = nwords / 4;  // the arrays start 16-byte aligned
    for (int i = tid; i < nquads; i += blockDim.x) ((uint4*)smem_raw)[i] = make_uint4(0, 0, 0, 0);
    for (int i = 4 * nquads + tid; i < nwords; i += blockDim.x) ((u32*)smem_raw)[i] = 0;
  }

  const DValCol& vc = P.vals[P.cells[0].col];
  const u32 ssum_a = (u32)__cvta_generic_to_shared(ssum), scnt_a = (u32)__cvta_generic_to_shared(scnt);
  const bool filt_is_val = P.nfilters == 1 && P.filters[0] == vc.mask && P.filter_offsets[0] == vc.offset;

  // position of the key whose bits equal EMPTY inside the box (it lives in the special slot), or -1
  int special_pos = -1;
  {
    int bits = 0;
    for (int k = 0; k < P.nkeys; ++k) bits += 8 * P.keys[k].width + (P.keys[k].nullbit >= 0 ? 1 : 0);
    if (bits == 64) special_pos = dense_index(P, s_dense, EMPTY);
  }
  // bytes of key column k: a constant when no column is 8 bytes wide, so the offsets below fold away
  auto kwidth = [&](int k) -> u32 { return K8 ? (u32)P.keys[k].width : 4u; };
  LeanRare L{ssum, NSP, fx_base, socc, &s_new, tbl, cap, (i64)region_slots, stride, special_pos, ctrl, &s_dense};

  // the key box in registers: the shared-memory atomics below clobber memory for the compiler, so
  // anything left in s_dense would be re-read from shared memory in every tile
  using box_t = typename std::conditional<K8, u64, u32>::type;  // 32 bits when every key column is 4 bytes wide
  box_t bmin[NK], blim[NK];
  u32 bmul[NK];
  bool bnull[NK], bexcl[NK], bw4[NK];
#pragma unroll
  for (int k = 0; k < NK; ++k) {
    const DKeyCol& c = P.keys[k];
    // KEY_MASKS = false: no key column carries a mask, so nothing about nulls survives compilation
    bnull[k] = KEY_MASKS && c.nullbit >= 0;
    bexcl[k] = KEY_MASKS && c.mask && !P.include_nulls;
    bw4[k]   = !K8 || c.width == 4;
    bmin[k]  = (box_t)s_dense.min[k];
    blim[k]  = (box_t)(s_dense.range[k] - (bnull[k] ? 1ull : 0ull));
    bmul[k]  = s_dense.mult[k];
  }

  if (STAGED && tid == 0) {
    const u32 bar0 = (u32)__cvta_generic_to_shared(s_bars);
    for (int s = 0; s < LEAN_STAGES; ++s) {
      mbar_init(bar0 + 8u * s, 1);                                              // "full": the producer's expect_tx
      mbar_init(bar0 + 8u * (LEAN_STAGES + s), LEAN_STAGED_CONSUMERS / 32);     // "empty": one arrival per consumer warp
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  if (timekeeper) ctrl->t_phase[2] = global_timer_ns();

  // folds one group of 4 consecutive rows starting at row r0
  // (the values: four floats in qa, or — V8 — four doubles in qa and qb)
  auto fold = [&](i64 r0, const uint4 (&ka)[NK], const uint4 (&kb)[NK], const u32 (&kn)[NK], const uint4& qa, const uint4& qb,
                  u32 vn, u32 act) {
    u32 d0 = copy_off, d1 = copy_off, d2 = copy_off, d3 = copy_off, bad = 0;
#pragma unroll
    for (int k = 0; k < NK; ++k) {
      if (bexcl[k]) act &= kn[k];
      const u32 mult = bmul[k];
      u32 x0, x1, x2, x3, o;
      if (bw4[k]) {
        const u32 mn = (u32)bmin[k];
        const u32 lim = (u32)blim[k];
        x0 = ka[k].x - mn; x1 = ka[k].y - mn; x2 = ka[k].z - mn; x3 = ka[k].w - mn;
        o = (x0 >= lim ? 1u : 0u) | (x1 >= lim ? 2u : 0u) | (x2 >= lim ? 4u : 0u) | (x3 >= lim ? 8u : 0u);
        if (bnull[k]) {
          if (!(kn[k] & 1u)) x0 = lim; if (!(kn[k] & 2u)) x1 = lim; if (!(kn[k] & 4u)) x2 = lim; if (!(kn[k] & 8u)) x3 = lim;
          o &= kn[k];
        }
      } else {
        const u64 mn = (u64)bmin[k];
        const u64 lim = (u64)blim[k];
        const u64 y0 = (((u64)ka[k].y << 32) | ka[k].x) - mn, y1 = (((u64)ka[k].w << 32) | ka[k].z) - mn;
        const u64 y2 = (((u64)kb[k].y << 32) | kb[k].x) - mn, y3 = (((u64)kb[k].w << 32) | kb[k].z) - mn;
        o = (y0 >= lim ? 1u : 0u) | (y1 >= lim ? 2u : 0u) | (y2 >= lim ? 4u : 0u) | (y3 >= lim ? 8u : 0u);
        x0 = (u32)y0; x1 = (u32)y1; x2 = (u32)y2; x3 = (u32)y3;
        if (bnull[k]) {
          if (!(kn[k] & 1u)) x0 = (u32)lim; if (!(kn[k] & 2u)) x1 = (u32)lim; if (!(kn[k] & 4u)) x2 = (u32)lim; if (!(kn[k] & 8u)) x3 = (u32)lim;
          o &= kn[k];
        }
      }
      bad |= o;
      d0 += x0 * mult; d1 += x1 * mult; d2 += x2 * mult; d3 += x3 * mult;
    }
    const u32 take = act & ~bad & vn;  // rows folded in shared memory
    // the four rows' shared-memory atomics are issued back to back; the counts they return are
    // looked at afterwards, so that the warp waits for one round trip, not four
    u32 o0 = 0, o1 = 0, o2 = 0, o3 = 0;
    if (!V8) {
      if (take & 1u) { sred_add_f32(ssum_a + 4u * d0, __uint_as_float(qa.x)); o0 = satom_add_u32(scnt_a + 4u * d0, 1u); }
      if (take & 2u) { sred_add_f32(ssum_a + 4u * d1, __uint_as_float(qa.y)); o1 = satom_add_u32(scnt_a + 4u * d1, 1u); }
      if (take & 4u) { sred_add_f32(ssum_a + 4u * d2, __uint_as_float(qa.z)); o2 = satom_add_u32(scnt_a + 4u * d2, 1u); }
      if (take & 8u) { sred_add_f32(ssum_a + 4u * d3, __uint_as_float(qa.w)); o3 = satom_add_u32(scnt_a + 4u * d3, 1u); }
    } else {
      // a value that does not fit the window joins the rare rows (its bit moves from `take` to `bad`)
      auto add8 = [&](u32 bit, u32 d, u32 lo, u32 hi, u32& o) {
        if (!(take & bit)) return;
        int q;
        u32 l[4];
        if (fx_split(((u64)hi << 32) | lo, fx_base, q, l)) {
          fx_add_s(ssum_a, NSP, (int)d, (hi >> 31) != 0u, q, l);
          o = satom_add_u32(scnt_a + 4u * d, 1u);
        } else {
          bad |= bit;
        }
      };
      add8(1u, d0, qa.x, qa.y, o0);
      add8(2u, d1, qa.z, qa.w, o1);
      add8(4u, d2, qb.x, qb.y, o2);
      add8(8u, d3, qb.z, qb.w, o3);
    }
    constexpr u32 EVERY = V8 ? FX_FLUSH : F32_SPILL_AT;
    if ((((o0 + 1u) & (EVERY - 1u)) == 0u) | (((o1 + 1u) & (EVERY - 1u)) == 0u) |
        (((o2 + 1u) & (EVERY - 1u)) == 0u) | (((o3 + 1u) & (EVERY - 1u)) == 0u)) {
      // (rows not taken keep o = 0)
      if (((o0 + 1u) & (EVERY - 1u)) == 0u) { if (V8) lean_flush(L, d0, copy_off); else lean_spill(L, d0, copy_off); }
      if (((o1 + 1u) & (EVERY - 1u)) == 0u) { if (V8) lean_flush(L, d1, copy_off); else lean_spill(L, d1, copy_off); }
      if (((o2 + 1u) & (EVERY - 1u)) == 0u) { if (V8) lean_flush(L, d2, copy_off); else lean_spill(L, d2, copy_off); }
      if (((o3 + 1u) & (EVERY - 1u)) == 0u) { if (V8) lean_flush(L, d3, copy_off); else lean_spill(L, d3, copy_off); }
    }
    const u32 rare = act & (bad | ~vn);
    if (rare) lean_rare_rows(P, L, rare, bad, r0, d0, d1, d2, d3);
  };

  if (!STAGED) {
    // ---- tiles from global memory into registers
    const u32 tile_rows = 1024u * LEAN_ROWS;
    const u32 nfull     = (u32)(P.nrows / tile_rows);
    auto load_tile = [&](u32 tile, uint4& qa, uint4& qb, u32& vn, u32& act, uint4 (&ka)[NK], uint4 (&kb)[NK], u32 (&kn)[NK]) {
      const u32 r0 = tile * tile_rows + (u32)tid * LEAN_ROWS;
      const u32 ve = (u32)vc.offset + r0;
      const uint4* vp = (const uint4*)(vc.data + (u64)ve * VB);
      qa = __ldg(vp);
      if (V8) qb = __ldg(vp + 1);
      else qb = make_uint4(0, 0, 0, 0);
      vn = vc.mask ? nibble_aligned(vc.mask, ve) : 0xFu;
      act = 0xFu;
      if (filt_is_val) act = vn;
      else for (int f = 0; f < P.nfilters; ++f) act &= nibble_aligned(P.filters[f], (u32)P.filter_offsets[f] + r0);
#pragma unroll
      for (int k = 0; k < NK; ++k) {
        const DKeyCol& c = P.keys[k];
        const u32 e = (u32)c.offset + r0;
        kn[k] = (KEY_MASKS && c.mask) ? nibble_aligned(c.mask, e) : 0xFu;
        const uint4* kp = (const uint4*)(c.data + (u64)e * kwidth(k));
        ka[k] = __ldg(kp);
        if (K8 && c.width == 8) kb[k] = __ldg(kp + 1);
        else kb[k] = make_uint4(0, 0, 0, 0);
      }
    };
    uint4 qa, qb, nqa, nqb;
    u32 vn = 0, act = 0, nvn = 0, nact = 0;
    uint4 ka[NK], kb[NK], nka[NK], nkb[NK];
    u32 kn[NK], nkn[NK];
    // Register prefetch of the next tile pays off with 4-byte keys; with 8-byte key columns the second
    // set of vector registers costs more than it hides, and the tile after is requested into L2 instead
    constexpr bool PREFETCH = !K8 && !V8;
    if (PREFETCH && blockIdx.x < nfull) load_tile(blockIdx.x, qa, qb, vn, act, ka, kb, kn);
    for (u32 tile = blockIdx.x; tile < nfull; tile += gridDim.x) {
      const u32 next = tile + gridDim.x;
      if (!PREFETCH) {
        load_tile(tile, qa, qb, vn, act, ka, kb, kn);
        if (next < nfull) {
          const u32 fr0 = next * tile_rows + (u32)tid * LEAN_ROWS;
          prefetch_l2(vc.data + (u64)((u32)vc.offset + fr0) * VB);
#pragma unroll
          for (int k = 0; k < NK; ++k) prefetch_l2(P.keys[k].data + (u64)((u32)P.keys[k].offset + fr0) * kwidth(k));
        }
      }
      if (PREFETCH && next < nfull) load_tile(next, nqa, nqb, nvn, nact, nka, nkb, nkn);
      fold((i64)tile * tile_rows + (i64)tid * LEAN_ROWS, ka, kb, kn, qa, qb, vn, act);
      if (PREFETCH) {
        qa = nqa; qb = nqb; vn = nvn; act = nact;
#pragma unroll
        for (int k = 0; k < NK; ++k) { ka[k] = nka[k]; kb[k] = nkb[k]; kn[k] = nkn[k]; }
      }
    }
  } else {
    // ---- tiles through the shared-memory ring.  Stage layout: [key column 0 | .. | key column NK-1 |
    // value column | validity bytes of the value column].  The host only selects this variant when
    // there are no key masks and the only row filter (if any) is the value column's own mask.
    constexpr u32 TR = LEAN_STAGED_CONSUMERS * LEAN_ROWS;
    const u32 nfull  = (u32)(P.nrows / TR);
    u32 col_off[NK + 1];
    u32 off = 0;
#pragma unroll
    for (int k = 0; k < NK; ++k) { col_off[k] = off; off += TR * kwidth(k); }
    col_off[NK] = off;
    const u32 mask_off = off + TR * VB;
    const u32 stage_bytes = mask_off + LEAN_MASK_BYTES;
    const u32 bar0 = (u32)__cvta_generic_to_shared(s_bars);
    const u32 stage_a = (u32)__cvta_generic_to_shared(stage0);
    bool failed = false;
    if (tid >= LEAN_STAGED_CONSUMERS) {
      if (tid == LEAN_STAGED_CONSUMERS) {  // one lane issues every copy
        u32 it = 0;
        for (u32 tile = blockIdx.x; tile < nfull; tile += gridDim.x, ++it) {
          const u32 s = it % LEAN_STAGES, round = it / LEAN_STAGES;
          if (round > 0 && !mbar_wait(bar0 + 8u * (LEAN_STAGES + s), (round - 1) & 1u)) { failed = true; break; }
          const u32 dst = stage_a + s * stage_bytes;
          const u64 r0  = (u64)tile * TR;
          const u32 full = bar0 + 8u * s;
          mbar_expect_tx(full, mask_off + (vc.mask ? TR / 8u : 0u));
#pragma unroll
          for (int k = 0; k < NK; ++k)
            bulk_g2s(dst + col_off[k], P.keys[k].data + ((u64)P.keys[k].offset + r0) * kwidth(k), TR * kwidth(k), full);
          bulk_g2s(dst + col_off[NK], vc.data + ((u64)vc.offset + r0) * VB, TR * VB, full);
          if (vc.mask) bulk_g2s(dst + mask_off, (const unsigned char*)vc.mask + (((u64)vc.offset + r0) >> 3), TR / 8u, full);
        }
        // the copies still in flight must land before this CTA's shared memory is reused or released
        if (failed) {
          for (u32 s = 0; s < LEAN_STAGES && s < it; ++s) {
            const u32 last = it - 1 - ((it - 1 - s) % LEAN_STAGES);  // last iteration that used stage s
            mbar_wait(bar0 + 8u * s, (last / LEAN_STAGES) & 1u);
          }
        }
      }
    } else {
      u32 it = 0;
      for (u32 tile = blockIdx.x; tile < nfull; tile += gridDim.x, ++it) {
        const u32 s = it % LEAN_STAGES, round = it / LEAN_STAGES;
        if (!mbar_wait(bar0 + 8u * s, round & 1u)) { failed = true; break; }
        const unsigned char* st = stage0 + (size_t)s * stage_bytes;
        const u32 e = (u32)tid * LEAN_ROWS;  // element inside the tile
        uint4 ka[NK], kb[NK];
        u32 kn[NK];
#pragma unroll
        for (int k = 0; k < NK; ++k) {
          kn[k] = 0xFu;
          const uint4* kp = (const uint4*)(st + col_off[k] + (size_t)e * kwidth(k));
          ka[k] = kp[0];
          if (K8 && P.keys[k].width == 8) kb[k] = kp[1];
          else kb[k] = make_uint4(0, 0, 0, 0);
        }
        const uint4* vp = (const uint4*)(st + col_off[NK] + (size_t)e * VB);
        const uint4 qa = vp[0];
        const uint4 qb = V8 ? vp[1] : make_uint4(0, 0, 0, 0);
        const u32 vn = vc.mask ? ((*(const u32*)(st + mask_off + (e >> 5) * 4u)) >> (e & 31u)) & 0xFu : 0xFu;
        const u32 act = filt_is_val ? vn : 0xFu;
        __syncwarp();
        if ((tid & 31) == 0) mbar_arrive(bar0 + 8u * (LEAN_STAGES + s));  // the stage's data is in registers
        fold((i64)tile * TR + e, ka, kb, kn, qa, qb, vn, act);
      }
    }
    if (failed) ctrl->error = 1;
  }

  // ---- the ragged end of the input, row by row (the row count of the full tiles is worked out again here
  // rather than kept in registers through the row loop; the same goes for the table's shape in the merge)
  constexpr i64 TILE_ROWS = (STAGED ? LEAN_STAGED_CONSUMERS : 1024) * LEAN_ROWS;
  const i64 rows_done = P.nrows / TILE_ROWS * TILE_ROWS;
  for (i64 r = rows_done + (i64)blockIdx.x * blockDim.x + tid; r < P.nrows; r += (i64)gridDim.x * blockDim.x)
    lean_slow_row(P, L, r, true);

  // ---- merge this CTA's table into the dense region of the global table: the replicas of a box
  // position are reduced in registers, then Σ and n are added with reductions that return nothing
  // (no round trip), and the key cell is written with a plain store — every CTA writes the same key.
  __syncthreads();
  if (timekeeper) ctrl->t_phase[3] = global_timer_ns();
  {
    // position -> key without divisions (dense_key divides twice per key column: 13 us of this merge for
    // 16 positions per thread): mixed-radix decode with one reciprocal per column, exact because
    // positions and ranges stay below 2^15
    const int S = (int)s_dense.total, copies = (int)s_dense.copies, NSP = (S * copies + 3) & ~3;
    const int special_pos = L.special_pos;
    const float* ssum = (const float*)smem_raw;
    const u32* scnt   = (const u32*)(ssum + SUM_WORDS * NSP);
    const u32* socc   = scnt + NSP;
    u32 rng[NK], magic[NK];
#pragma unroll
    for (int k = 0; k < NK; ++k) {
      rng[k]   = (u32)s_dense.range[k];
      magic[k] = rng[k] > 1u ? (u32)(0x100000000ull / rng[k]) + 1u : 0u;
    }
    auto box_key = [&](u32 idx) -> u64 {
      u64 key = 0;
      u32 rem = idx;
#pragma unroll
      for (int k = 0; k < NK; ++k) {
        const u32 q = rng[k] > 1u ? __umulhi(rem, magic[k]) : rem;
        const u32 f = rem - q * rng[k];
        rem = q;
        const DKeyCol& c = P.keys[k];
        if (bnull[k] && f == rng[k] - 1u) {
          key |= 1ull << c.nullbit;
        } else {
          const u64 v = (u64)((i64)f + s_dense.min[k]);
          key |= (c.width == 8 ? v : (v & ((1ull << (8 * c.width)) - 1ull))) << c.shift;
        }
      }
      return key;
    };
    const int rot = (int)(((u64)blockIdx.x * 2654435761ull) % (u64)S);
    for (int i0 = tid; i0 < S; i0 += blockDim.x) {
      const int i = i0 + rot < S ? i0 + rot : i0 + rot - S;
      double sum = 0.0;
      u64 n = 0;
      bool present = false;
      i64 words[SUM_WORDS] = {};  // V8: the replicas' limbs, added word by word (exact)
      for (int r = 0; r < copies; ++r) {
        const int q = r * S + i;
        const u32 c = scnt[q];
        present = present || c != 0u || ((socc[q >> 5] >> (q & 31)) & 1u);
        if (V8) {
#pragma unroll
          for (int w = 0; w < SUM_WORDS; ++w) words[w] += (i64)((const int*)ssum)[w * NSP + q];
        } else {
          sum += (double)ssum[q];
        }
        n += c;
      }
      if (!present) continue;
      if (V8) {
        double acc = 0.0;
#pragma unroll
        for (int w = SUM_WORDS - 1; w >= 0; --w) acc = acc * 262144.0 + (double)words[w];
        sum = acc == 0.0 ? 0.0 : ldexp(acc, fx_base - 1075);
      }
      const SlotRef ref = lean_box_slot(L, (u32)i);
      // (an unconditional store: reading the cell first would put an L2 round trip into every iteration)
      if (i == special_pos) { if (ctrl->special_used == 0) ctrl->special_used = 1; }
      else *ref.key = box_key((u32)i);
      if (n) { atomicAdd((double*)ref.cells, sum); atomicAdd(ref.cells + ref.step, n); }
    }
  }
  lean_report_claims(L);

  // ---- the last CTA to finish counts the groups of the dense region (their key cells were written
  // with plain stores, so nobody counted them on the way)
  __threadfence();
  __syncthreads();
  if (tid == 0) s_last = atomicAdd(&ctrl->done_ctas, 1ull) == (u64)gridDim.x - 1;
  __syncthreads();
  if (s_last) {
    __threadfence();
    const int S = (int)s_dense.total, special_pos = L.special_pos;
    int mine = 0;
    for (int i = tid; i < S; i += blockDim.x) {
      if (i == special_pos) continue;
      const u64* kp = slot_ref(tbl, cap, stride, (i64)region_slots, cap + 1 + (i64)i).key;
      mine += __ldcg(kp) != EMPTY ? 1 : 0;
    }
    mine = __reduce_add_sync(0xFFFFFFFFu, mine);
    if ((tid & 31) == 0 && mine) atomicAdd(&s_new, mine);
    __syncthreads();
    if (tid == 0 && s_new) {
      const u64 tot = atomicAdd(&ctrl->nclaimed, (u64)s_new) + (u64)s_new;
      if (tot > ctrl->claim_limit + (u64)S) ctrl->overflow = 1;
    }
  }
  if (timekeeper) ctrl->t_phase[4] = global_timer_ns();
}

}  // namespace b2
