// Attention-forward kernel for sm_100a whose score products run ahead of the softmax.
//
// Same work decomposition as the persistent kernel (one CTA per SM, work item = two adjacent
// 128-row q tiles of one head, items handed out from a global counter), but the kv axis is cut
// into tiles of 64 keys and every q-tile stage owns TWO score buffers in tensor memory:
//
//   TMEM columns  S[0][0] [0,64)  S[0][1] [64,128)  S[1][0] [128,192)  S[1][1] [192,256)
//                 O[0] [256,256+D)                   O[1] [384,384+D)
//
// The fp16 P tile of kv tile n overwrites the first 32 columns of the score buffer n & 1, and
// S(n+1) = Q K(n+1)^T goes to the other buffer. With a single buffer per stage the next score
// product has to wait until P(n) V(n) has read P(n), so every stage runs the dependent chain
// scores -> softmax -> P V -> scores; here the tensor pipe computes S(n+1) while the softmax of
// tile n is still running, and the softmax warps find their next tile ready when they finish one.
// The price is a score product with N = 64, which is bound by the shared-memory reads of its
// operands (48 instead of 32 clocks per K = 16 step), i.e. 640 instead of 512 tensor clocks per
// 64 keys and q tile.
//
// Roles (16 warps):
//   warps 0-3 / 4-7  softmax of q tile 0 / 1, one thread per score row
//   warps 8-11       correction: rescales O in TMEM when a row's reference max moved; epilogue
//   warp 12 / 13     tensor-core issuer of q tile 0 / 1 (one thread each)
//   warp 14          TMA producer: Q tiles, the K/V ring, work-item claim and broadcast
//   warp 15          idle
//
// Replaces the reference's forward_kernel, Schedule and SMem (src/flash_forward.h:22-366),
// apply_mask (src/mask.h:10-84) and apply_softmax (src/softmax.h:9-86).
#pragma once
#include <type_traits>

#include "fwd_params.h"
#include "fwd_persistent.cuh"  // ItemGeom, decode_item, exp2_poly_pair
#include "ptx.cuh"

// Registers per thread after setmaxnreg: 8 softmax warps, 4 correction warps, 4 others;
// 256 * softmax + 128 * correction + 128 * others <= 65536.
#ifndef FA_RA_REG_SOFTMAX
#define FA_RA_REG_SOFTMAX 144
#define FA_RA_REG_CORR 112
#define FA_RA_REG_MISC 112
#endif
// Of every 8 pairs of scores, this many take 2^x from the polynomial on the FMA pipe.
#ifndef FA_RA_EMU_PAIRS
#define FA_RA_EMU_PAIRS 0
#endif

// Bring-up profile (compile with -DFA_RA_PROF and pass a dbg buffer): CTA 0 accumulates the clocks its roles
// spend between stamps; slot meaning is at the call sites.
#ifdef FA_RA_PROF
#define RA_PROF_DECL uint32_t prof_acc[8] = {0, 0, 0, 0, 0, 0, 0, 0}; uint32_t prof_last = static_cast<uint32_t>(clock());
#define RA_PROF(slot) do { const uint32_t t_now = static_cast<uint32_t>(clock()); prof_acc[slot] += t_now - prof_last; prof_last = t_now; } while (0)
#define RA_PROF_DUMP(base) do { if (blockIdx.x == 0 && p.dbg != nullptr) { long long* out = reinterpret_cast<long long*>(p.dbg) + 48 + (base); for (int i = 0; i < 8; ++i) out[i] = prof_acc[i]; } } while (0)
#else
#define RA_PROF_DECL
#define RA_PROF(slot) do { } while (0)
#define RA_PROF_DUMP(base) do { } while (0)
#endif

namespace fa {

template <int D>
struct RunaheadCfg {
  static constexpr int kThreads = 512;
  static constexpr int kBn = 64;                                  // keys per kv tile
  static constexpr int kQBytes = kBlockM * D * 2;                 // one Q tile
  static constexpr int kQPanelBytes = kBlockM * kPanel * 2;       // 128 rows x 128 B
  static constexpr int kKvBytes = kBn * D * 2;                    // one K or V tile
  static constexpr int kKvPanelBytes = kBn * kPanel * 2;          // 64 rows x 128 B
  static constexpr int kStages = (D == 128) ? 9 : 16;             // ring slots, each one K or one V tile
  static constexpr int kOffQ = 0;
  static constexpr int kOffKV = 2 * kQBytes;
  static constexpr int kOffAlpha = kOffKV + kStages * kKvBytes;   // float[2 stages][2 buffers][128]
  static constexpr int kOffRowSum = kOffAlpha + 4 * kBlockM * 4;  // float[2][128]
  static constexpr int kOffBars = kOffRowSum + 2 * kBlockM * 4;
  static constexpr int kNumBars = 30 + 2 * kStages;
  static constexpr int kOffMisc = kOffBars + kNumBars * 8;
  static constexpr int kSmemBytes = kOffMisc + 16;  // TMEM base, abort flag, two work-item slots
  static constexpr uint32_t kTmemCols = 512;
  static constexpr uint32_t kColS = 0;    // + stage * 128 + buffer * 64
  static constexpr uint32_t kColO = 256;  // + stage * 128
  static constexpr float kLazyLog2 = 8.f;
};

// 2^x of `NP` pairs of scores -> packed fp16x2 words; adds the exponentials into two partial row sums.
template <int NP, bool kAllowPoly>
__device__ __forceinline__ void ra_exp_pairs(const float* sc, uint64_t scale2, uint64_t negms2, uint32_t* pk,
                                             uint64_t& lsum_a, uint64_t& lsum_b) {
#pragma unroll
  for (int c = 0; c < NP; ++c) {
    float x0, x1, e0, e1;
    f2_unpack(f2_fma(f2_pack(sc[2 * c], sc[2 * c + 1]), scale2, negms2), x0, x1);
    if (kAllowPoly && (c % 8) < FA_RA_EMU_PAIRS) {
      exp2_poly_pair(x0, x1, e0, e1);
    } else {
      e0 = ex2_approx(x0);
      e1 = ex2_approx(x1);
    }
    if (c & 1) lsum_b = f2_add(lsum_b, f2_pack(e0, e1));
    else lsum_a = f2_add(lsum_a, f2_pack(e0, e1));
    pk[c] = pack_f16x2(e0, e1);
  }
}

template <int D, bool kAlibi, bool kLse = false>
__global__ void __launch_bounds__(512, 1)
fwd_runahead_kernel(const __grid_constant__ CUtensorMap mapQ, const __grid_constant__ CUtensorMap mapK,
                    const __grid_constant__ CUtensorMap mapV, const FwdParams p) {
  using Cfg = RunaheadCfg<D>;
  constexpr int BN = Cfg::kBn;
  extern __shared__ __align__(1024) uint8_t smem[];

  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int lane = tid & 31;

  if ((smem_u32(smem) & 1023u) != 0) {  // swizzled tiles need a 1024-byte aligned base
    if (tid == 0) atomicExch(p.status, 2);
    return;
  }

  uint8_t* sQ = smem + Cfg::kOffQ;
  uint8_t* sKV = smem + Cfg::kOffKV;
  float* sAlpha = reinterpret_cast<float*>(smem + Cfg::kOffAlpha);
  float* sRowSum = reinterpret_cast<float*>(smem + Cfg::kOffRowSum);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + Cfg::kOffBars);
  uint64_t* q_full = bars;             // [2]    TMA -> MMA
  uint64_t* q_empty = bars + 2;        // [2]    MMA -> TMA
  uint64_t* s_full = bars + 4;         // [2][2] MMA -> softmax: score tile in buffer b
  uint64_t* p_full = bars + 8;         // [2][2] softmax (P written) + correction (O rescaled) -> MMA
  uint64_t* alpha_ready = bars + 12;   // [2][2] softmax -> correction: rescale factors in smem
  uint64_t* l_ready = bars + 16;       // [2]    softmax -> correction: final row sums in smem
  uint64_t* l_empty = bars + 18;       // [2]    correction -> softmax: row sums read
  uint64_t* o_done = bars + 20;        // [2]    MMA -> correction: P.V of a tile has landed in O
  uint64_t* item_full = bars + 22;     // [2]    producer -> all roles: next work item id published
  uint64_t* item_empty = bars + 24;    // [2]    all roles -> producer: id slot read
  uint64_t* kv_full = bars + 30;       // [kStages] TMA -> both MMA warps
  uint64_t* kv_empty = bars + 30 + Cfg::kStages;  // [kStages] both MMA warps -> TMA
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + Cfg::kOffMisc);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  volatile int* s_item = reinterpret_cast<volatile int*>(tmem_slot + 2);  // [2]
  constexpr uint32_t kItemReaders = 14;  // 8 softmax warps + 4 correction warps + 2 MMA threads

  if (warp == 15) {
    tmem_alloc(tmem_slot, Cfg::kTmemCols);
    tmem_relinquish();
  }
  if (tid == 0) {
#pragma unroll
    for (int s = 0; s < 2; ++s) {
      mbar_init(&q_full[s], 1);
      mbar_init(&q_empty[s], 1);
      mbar_init(&l_ready[s], 4);
      mbar_init(&l_empty[s], 4);
      mbar_init(&o_done[s], 1);
      mbar_init(&item_full[s], 1);
      mbar_init(&item_empty[s], kItemReaders);
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      mbar_init(&s_full[i], 1);
      mbar_init(&p_full[i], 8);  // one arrival per softmax warp and per correction warp
      mbar_init(&alpha_ready[i], 4);
    }
    for (int i = 0; i < Cfg::kStages; ++i) {
      mbar_init(&kv_full[i], 1);
      mbar_init(&kv_empty[i], 2);  // one arrival per MMA warp
    }
    *abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == 14 && lane == 0) {
    prefetch_tensormap(&mapQ);
    prefetch_tensormap(&mapK);
    prefetch_tensormap(&mapV);
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  const int N = p.seqlen;
  const int wl = p.window_left;
  const int wr = eff_window_right(p.causal, p.window_right);

  // Every consuming warp reads the k-th work item id from slot k & 1 once the producer has published it,
  // and releases the slot. -1 ends the walk (also after a give-up).
  auto take_item = [&](uint32_t& n_items) -> int {
    const uint32_t slot = n_items & 1u;
    if (!mbar_wait_warp(&item_full[slot], (n_items >> 1) & 1u, abort_flag)) return -1;
    const int it = s_item[slot];
    __syncwarp();
    if (lane == 0) mbar_arrive(&item_empty[slot]);
    ++n_items;
    return it;
  };
  auto take_item_thread = [&](uint32_t& n_items) -> int {  // same, for a role that is a single thread
    const uint32_t slot = n_items & 1u;
    if (!mbar_wait(&item_full[slot], (n_items >> 1) & 1u, abort_flag)) return -1;
    const int it = s_item[slot];
    mbar_arrive(&item_empty[slot]);
    ++n_items;
    return it;
  };

  if (warp < 8) {
    // =====================================================================================
    // softmax: stage s = warp / 4, row = tid % 128
    // =====================================================================================
    reg_inc<FA_RA_REG_SOFTMAX>();
    const int s = warp >> 2;
    const int row_l = tid & 127;
    const uint32_t lane_base = static_cast<uint32_t>(warp & 3) * 32u;
    const uint32_t tS0 = tmem_addr(tmem_base, lane_base, Cfg::kColS + s * 128);
    // With ALiBi the scores are moved to the biased log2 domain right after the TMEM load, and
    // everything downstream works with a unit scale.
    const float sl2 = kAlibi ? 1.f : p.scale_log2;
    const uint64_t scale2 = f2_pack(sl2, sl2);
    uint32_t n = 0;       // kv tiles this stage has processed since the kernel started
    uint32_t n_rows = 0;  // items in which this stage had rows
    uint32_t n_items = 0;
    bool ok = true;
    RA_PROF_DECL
    while (ok) {
      const int item = take_item(n_items);
      if (item < 0) break;
      const ItemGeom g = decode_item<BN>(item, p);
      RA_PROF(0);  // item hand-over
      const int q_r0 = s ? g.r0[1] : g.r0[0];
      const int q_r1 = s ? g.r1[1] : g.r1[0];
      const int j_lo = s ? g.lo[1] : g.lo[0];
      const int j_hi = s ? g.hi[1] : g.hi[0];
      if (q_r1 < q_r0) continue;
      const int row = q_r0 + row_l;
      float slope_l2 = 0.f;
      if (kAlibi) slope_l2 = p.alibi_slopes[g.bh % p.heads] * 1.4426950408889634f;
      float m_run = -INFINITY;  // true running max of the raw scores
      float m_used = 0.f;       // max the exponentials are currently taken against
      float l_run = 0.f;
      for (int j = j_lo; j < j_hi; ++j) {
        const uint32_t b = n & 1u;
        if (!mbar_wait_warp(&s_full[s * 2 + b], (n >> 1) & 1u, abort_flag)) { ok = false; break; }
        ++n;
        tc_fence_after();
        RA_PROF(1);  // waiting for scores
        const int kv0 = j * BN;
        const uint32_t tS = tS0 + b * BN;
        float* alpha_slot = sAlpha + (s * 2 + b) * kBlockM + row_l;
        // One body, instantiated twice: tiles cut by a mask boundary (or by the end of the sequence) take the
        // per-element predicate and MUFU-only exponentials, all others carry none of that code.
        auto tile_body = [&](auto masked_tag) {
          constexpr bool kMasked = decltype(masked_tag)::value;
#ifdef FA_RA_FAKE  // bring-up only: measures the load + tensor pipeline without the softmax work
          *alpha_slot = 1.f;
          l_run = 1.f;
          __syncwarp();
          if (lane == 0) { mbar_arrive(&alpha_ready[s * 2 + b]); mbar_arrive(&p_full[s * 2 + b]); }
          return;
#endif
          uint32_t r0[32], r1[32];
          tmem_ld32(tS + 0, r0);
          tmem_ld32(tS + 32, r1);
          tmem_wait_ld();
          tmem_ld_fence(r0);
          tmem_ld_fence(r1);
          float sc[BN];
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            sc[i] = __uint_as_float(r0[i]);
            sc[32 + i] = __uint_as_float(r1[i]);
          }
          if (kAlibi) {  // s * scale - slope * |i - j|, in log2 units (reference: src/mask.h:21-26, src/main.cu:200-207)
            const float rel = static_cast<float>(row - kv0);
#pragma unroll
            for (int c = 0; c < BN; ++c)
              sc[c] = fmaf(sc[c], p.scale_log2, -slope_l2 * fabsf(rel - static_cast<float>(c)));
          }
          if (kMasked) {
            const int c_lo = (wl >= 0) ? row - wl - kv0 : -1;
            int c_hi = N - 1 - kv0;
            if (wr >= 0) c_hi = min(c_hi, row + wr - kv0);
#pragma unroll
            for (int c = 0; c < BN; ++c)
              if (c < c_lo || c > c_hi) sc[c] = -INFINITY;
          }
          // The exponentials of the first 32 keys are taken against the reference max of the previous tile
          // while the row max of this tile is still being reduced: nearly always the reference stays where it
          // is (lazy rescale: it moves only when the true max has grown by more than kLazyLog2, so P stays
          // below 2^8, or when no finite score was seen before), and the max is off the critical path. When a
          // row of the warp does move its reference (always on the first tile of an item), the 32
          // exponentials are taken again.
          uint64_t lsum_a = 0ull, lsum_b = 0ull;
          uint32_t pk[32];
          {
            const float neg_ms0 = -m_used * sl2;
            ra_exp_pairs<16, !kMasked>(sc, scale2, f2_pack(neg_ms0, neg_ms0), pk, lsum_a, lsum_b);
          }
          float mx0 = m_run, mx1 = -INFINITY, mx2 = -INFINITY, mx3 = -INFINITY;
#pragma unroll
          for (int c = 0; c < BN; c += 8) {
            mx0 = max3(mx0, sc[c], sc[c + 1]);
            mx1 = max3(mx1, sc[c + 2], sc[c + 3]);
            mx2 = max3(mx2, sc[c + 4], sc[c + 5]);
            mx3 = max3(mx3, sc[c + 6], sc[c + 7]);
          }
          const float m_new = max3(mx0, mx1, fmaxf(mx2, mx3));
          const bool fresh = (m_run == -INFINITY);
          const bool move = fresh || (m_new - m_used) * sl2 > Cfg::kLazyLog2;
          float alpha = 1.f;
          m_run = m_new;
          if (__any_sync(0xffffffffu, move)) {
            const float m_next = move ? ((m_new == -INFINITY) ? 0.f : m_new) : m_used;
            alpha = fresh ? 1.f : ex2_approx((m_used - m_next) * sl2);
            m_used = m_next;
            lsum_a = 0ull;
            lsum_b = 0ull;
            const float neg_ms1 = -m_used * sl2;
            ra_exp_pairs<16, !kMasked>(sc, scale2, f2_pack(neg_ms1, neg_ms1), pk, lsum_a, lsum_b);
          }
          *alpha_slot = alpha;
          __syncwarp();
          if (lane == 0) mbar_arrive(&alpha_ready[s * 2 + b]);
          const float neg_ms = -m_used * sl2;
          ra_exp_pairs<16, !kMasked>(sc + 32, scale2, f2_pack(neg_ms, neg_ms), pk + 16, lsum_a, lsum_b);
          tmem_st32(tS, pk);  // P over the first 32 columns of this score buffer
          float l0, l1;
          f2_unpack(f2_add(lsum_a, lsum_b), l0, l1);
          l_run = l_run * alpha + (l0 + l1);
          tmem_wait_st();
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(&p_full[s * 2 + b]);
        };
        if (kv_tile_needs_mask(kv0, q_r0, q_r1, wl, wr, N, BN)) tile_body(std::true_type{});
        else tile_body(std::false_type{});
        RA_PROF(2);  // softmax of a tile
      }
      if (!ok) break;
      // the correction warps must have read the previous item's row sums before they are overwritten
      if (!mbar_wait_warp(&l_empty[s], (n_rows & 1u) ^ 1u, abort_flag)) break;
      ++n_rows;
      sRowSum[s * kBlockM + row_l] = l_run;
      __syncwarp();
      if (lane == 0) mbar_arrive(&l_ready[s]);
      // l_run = sum over visible keys of 2^((score - m_used) * sl2), so the natural-log sum of exponentials is
      // ln2 * (m_used * sl2 + log2(l_run)).
      if (kLse && row < N)
        p.lse[static_cast<size_t>(g.bh) * N + row] =
            (l_run > 0.f) ? 0.6931471805599453f * fmaf(m_used, sl2, __log2f(l_run)) : -INFINITY;
      RA_PROF(3);  // row-sum hand-over
    }
    if (warp == 0 && lane == 0) RA_PROF_DUMP(0);
    if (warp == 4 && lane == 0) RA_PROF_DUMP(8);
  } else if (warp < 12) {
    // =====================================================================================
    // correction + epilogue: row = tid % 128 of both stages
    // =====================================================================================
    reg_dec<FA_RA_REG_CORR>();
    const int row_l = tid & 127;
    const uint32_t lane_base = static_cast<uint32_t>(warp & 3) * 32u;
    uint32_t n_t[2] = {0, 0};  // kv tiles per stage since the kernel started
    uint32_t n_l[2] = {0, 0};  // items per stage with rows
    uint32_t n_items = 0;
    bool ok = true;
    while (ok) {
      const int item = take_item(n_items);
      if (item < 0) break;
      const ItemGeom g = decode_item<BN>(item, p);
      for (int j = g.lo_all; j < g.hi_all && ok; ++j) {
#pragma unroll
        for (int s = 0; s < 2; ++s) {
          if (j < g.lo[s] || j >= g.hi[s]) continue;
          const uint32_t b = n_t[s] & 1u;
          if (!mbar_wait_warp(&alpha_ready[s * 2 + b], (n_t[s] >> 1) & 1u, abort_flag)) { ok = false; break; }
          const float alpha = sAlpha[(s * 2 + b) * kBlockM + row_l];
          if (j > g.lo[s] && __any_sync(0xffffffffu, alpha != 1.f)) {
            // the P.V product of this stage's previous tile must have landed before O is touched
            if (!mbar_wait_warp(&o_done[s], (n_t[s] - 1u) & 1u, abort_flag)) { ok = false; break; }
            tc_fence_after();
            const uint32_t tO = tmem_addr(tmem_base, lane_base, Cfg::kColO + s * 128);
#pragma unroll
            for (int c = 0; c < D / 32; ++c) {
              uint32_t r[32];
              tmem_ld32(tO + c * 32, r);
              tmem_wait_ld();
              tmem_ld_fence(r);
#pragma unroll
              for (int i = 0; i < 32; ++i) r[i] = __float_as_uint(__uint_as_float(r[i]) * alpha);
              tmem_st32(tO + c * 32, r);
            }
            tmem_wait_st();
          }
          ++n_t[s];
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(&p_full[s * 2 + b]);
        }
      }
      if (!ok) break;
#pragma unroll
      for (int s = 0; s < 2; ++s) {
        if (g.r1[s] < g.r0[s]) continue;
        if (!mbar_wait_warp(&l_ready[s], n_l[s] & 1u, abort_flag)) { ok = false; break; }
        ++n_l[s];
        const float l = sRowSum[s * kBlockM + row_l];
        __syncwarp();
        if (lane == 0) mbar_arrive(&l_empty[s]);
        if (!mbar_wait_warp(&o_done[s], (n_t[s] - 1u) & 1u, abort_flag)) { ok = false; break; }
        tc_fence_after();
        const float inv_l = (l > 0.f) ? 1.f / l : 0.f;
        const int row = g.r0[s] + row_l;
        const uint32_t tO = tmem_addr(tmem_base, lane_base, Cfg::kColO + s * 128);
        __half* orow = p.O + (static_cast<size_t>(g.bh) * N + row) * D;
#pragma unroll
        for (int c = 0; c < D / 32; ++c) {
          uint32_t r[32];
          tmem_ld32(tO + c * 32, r);
          tmem_wait_ld();
          tmem_ld_fence(r);
          if (row < N) {
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              uint4 v;
              v.x = pack_f16x2(__uint_as_float(r[i * 8 + 0]) * inv_l, __uint_as_float(r[i * 8 + 1]) * inv_l);
              v.y = pack_f16x2(__uint_as_float(r[i * 8 + 2]) * inv_l, __uint_as_float(r[i * 8 + 3]) * inv_l);
              v.z = pack_f16x2(__uint_as_float(r[i * 8 + 4]) * inv_l, __uint_as_float(r[i * 8 + 5]) * inv_l);
              v.w = pack_f16x2(__uint_as_float(r[i * 8 + 6]) * inv_l, __uint_as_float(r[i * 8 + 7]) * inv_l);
              *reinterpret_cast<uint4*>(orow + c * 32 + i * 8) = v;
            }
          }
        }
      }
    }
  } else {
    reg_dec<FA_RA_REG_MISC>();
    if (warp < 14 && lane == 0) {
      // ===================================================================================
      // tensor-core issuer of stage s: one thread walks the schedule of its q tile. Per kv tile n
      // the order on the tensor pipe is S(n+1) = Q K(n+1)^T into the free score buffer, then
      // O += P(n) V(n); tcgen05 operations of one thread execute in issue order, so S(n+2) never
      // overwrites P(n) before P(n) V(n) has read it.
      // ===================================================================================
      const int s = warp - 12;
      constexpr uint32_t idesc_qk = umma_idesc_f16(kBlockM, BN, 0, 0);
      constexpr uint32_t idesc_pv = umma_idesc_f16(kBlockM, D, 0, 1);
      const uint64_t kdesc0 = umma_desc_sw128(0, 16, 1024);                  // K-major tiles (Q, K)
      const uint64_t vdesc0 = umma_desc_sw128(0, Cfg::kKvPanelBytes, 1024);  // MN-major tile (V)
      const uint32_t kv_addr = smem_u32(sKV);
      const uint64_t qdesc = kdesc0 + ((smem_u32(sQ) + s * Cfg::kQBytes) >> 4);
      const uint32_t colS = tmem_base + Cfg::kColS + s * 128;
      const uint32_t colO = tmem_base + Cfg::kColO + s * 128;
      uint32_t ring_slot = 0, ring_par = 0;  // ring position of K tile lo_all of the current item
      uint32_t n = 0;                        // kv tiles of this stage since the kernel started
      uint32_t n_q = 0, n_items = 0;
      bool ok = true;
      RA_PROF_DECL
      auto advance = [](uint32_t& slot, uint32_t& par, uint32_t k) {
        slot += k;
        while (slot >= static_cast<uint32_t>(Cfg::kStages)) { slot -= Cfg::kStages; par ^= 1u; }
      };
      while (ok) {
        const int item = take_item_thread(n_items);
        if (item < 0) break;
        const ItemGeom g = decode_item<BN>(item, p);
        RA_PROF(0);  // item hand-over
        const bool rows = g.r1[s] >= g.r0[s];
        const int lo = rows ? g.lo[s] : g.lo_all;
        const int hi = rows ? g.hi[s] : g.lo_all;
        // a tile this stage does not read is released as soon as it has landed
        auto skip_tiles = [&](uint32_t slot, uint32_t par, int count) {
          for (int i = 0; i < 2 * count && ok; ++i) {
            if (!mbar_wait(&kv_full[slot], par, abort_flag)) { ok = false; break; }
            mbar_arrive(&kv_empty[slot]);
            advance(slot, par, 1);
          }
        };
        skip_tiles(ring_slot, ring_par, lo - g.lo_all);
        uint32_t slot_k = ring_slot, par_k = ring_par;
        advance(slot_k, par_k, 2u * static_cast<uint32_t>(lo - g.lo_all));  // K_lo
        uint32_t slot_v = slot_k, par_v = par_k;
        advance(slot_v, par_v, 1);                                          // V_lo
        auto issue_qk = [&](int j, uint32_t buf) {  // S[buf] = Q K_j^T
          if (!mbar_wait(&kv_full[slot_k], par_k, abort_flag)) { ok = false; return; }
          tc_fence_after();
          RA_PROF(1);  // waiting for K
          const uint64_t kdesc = kdesc0 + ((kv_addr + slot_k * Cfg::kKvBytes) >> 4);
#pragma unroll
          for (int k = 0; k < D / 16; ++k) {
            const uint32_t off_q = ((k / 4) * Cfg::kQPanelBytes + (k % 4) * 32) >> 4;
            const uint32_t off_k = ((k / 4) * Cfg::kKvPanelBytes + (k % 4) * 32) >> 4;
#ifndef FA_RA_NOQK
            umma_ss(colS + buf * BN, qdesc + off_q, kdesc + off_k, idesc_qk, k > 0 ? 1u : 0u);
#endif
          }
          umma_commit(&s_full[s * 2 + buf]);
          umma_commit(&kv_empty[slot_k]);
          if (j + 1 == hi) umma_commit(&q_empty[s]);
          advance(slot_k, par_k, 2);
          RA_PROF(2);  // issuing the score product
        };
        if (ok && lo < hi) {
          if (!mbar_wait(&q_full[s], n_q & 1u, abort_flag)) { ok = false; break; }
          ++n_q;
          issue_qk(lo, n & 1u);
          for (int j = lo; j < hi && ok; ++j) {
            const uint32_t buf = n & 1u;
            if (j + 1 < hi) issue_qk(j + 1, buf ^ 1u);
            if (!ok) break;
            // O += P(n) V_j
            if (!mbar_wait(&kv_full[slot_v], par_v, abort_flag)) { ok = false; break; }
            RA_PROF(3);  // waiting for V
            if (!mbar_wait(&p_full[s * 2 + buf], (n >> 1) & 1u, abort_flag)) { ok = false; break; }
            tc_fence_after();
            RA_PROF(4);  // waiting for P
            const uint64_t vdesc = vdesc0 + ((kv_addr + slot_v * Cfg::kKvBytes) >> 4);
#pragma unroll
            for (int kk = 0; kk < BN / 16; ++kk)
#ifndef FA_RA_NOPV
              umma_ts(colO, colS + buf * BN + kk * 8, vdesc + kk * (2048 >> 4), idesc_pv, (kk > 0 || j > lo) ? 1u : 0u);
#endif
            umma_commit(&kv_empty[slot_v]);
            umma_commit(&o_done[s]);
            advance(slot_v, par_v, 2);
            ++n;
            RA_PROF(5);  // issuing P.V
          }
        }
        if (!ok) break;
        {  // tiles behind this stage's range (slot_k is K_hi by now, or K_lo when the stage had nothing to do)
          skip_tiles(slot_k, par_k, g.hi_all - hi);
          advance(ring_slot, ring_par, 2u * static_cast<uint32_t>(g.hi_all - g.lo_all));
          RA_PROF(6);  // releasing tiles outside the range
        }
      }
      RA_PROF_DUMP(16 + 8 * s);
    } else if (warp == 14 && lane == 0) {
      // ===================================================================================
      // TMA producer
      // ===================================================================================
      uint32_t it = 0;
      uint32_t n_q[2] = {0, 0};
      uint32_t n_pub = 0;
      bool ok = true;
      int next = (static_cast<int>(blockIdx.x) < p.num_items) ? static_cast<int>(blockIdx.x) : -1;
      while (ok) {
        const int item = next;
        {  // publish the id to the other roles
          const uint32_t slot = n_pub & 1u;
          if (!mbar_wait(&item_empty[slot], ((n_pub >> 1) & 1u) ^ 1u, abort_flag)) { ok = false; break; }
          s_item[slot] = item;
          mbar_arrive(&item_full[slot]);
          ++n_pub;
        }
        if (item < 0) break;
        // claim the following item now; the value is not needed before this item's loads are issued
        next = static_cast<int>(gridDim.x) + atomicAdd(p.sched, 1);
        if (next >= p.num_items) next = -1;
        const ItemGeom g = decode_item<BN>(item, p);
#pragma unroll
        for (int s = 0; s < 2; ++s) {
          if (g.r1[s] < g.r0[s]) continue;
          if (!mbar_wait(&q_empty[s], (n_q[s] & 1) ^ 1, abort_flag)) { ok = false; break; }
          ++n_q[s];
          mbar_arrive_expect_tx(&q_full[s], Cfg::kQBytes);
          tma_load_4d(sQ + s * Cfg::kQBytes, &mapQ, &q_full[s], 0, g.r0[s], 0, g.bh);
        }
        for (int j = g.lo_all; j < g.hi_all && ok; ++j) {
#pragma unroll
          for (int t = 0; t < 2; ++t) {
            const uint32_t slot = it % Cfg::kStages;
            if (!mbar_wait(&kv_empty[slot], ((it / Cfg::kStages) & 1) ^ 1, abort_flag)) { ok = false; break; }
            mbar_arrive_expect_tx(&kv_full[slot], Cfg::kKvBytes);
            tma_load_4d(sKV + slot * Cfg::kKvBytes, t == 0 ? &mapK : &mapV, &kv_full[slot], 0, j * BN, 0, g.bh);
            ++it;
          }
        }
      }
      if (!ok) {
        // give-up path: let loads that are still in flight land before the CTA retires
        for (int i = 0; i < 64; ++i) __nanosleep(2000);
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (tid == 0) {
    if (*abort_flag != 0) atomicExch(p.status, 1);
    // the last CTA to finish puts the scheduler words back to zero for the next launch
    if (atomicAdd(p.sched + 1, 1) == static_cast<int>(gridDim.x) - 1) {
      p.sched[0] = 0;
      p.sched[1] = 0;
      __threadfence();
    }
  }
  if (warp == 15) tmem_dealloc(tmem_base, Cfg::kTmemCols);
}

}  // namespace fa
