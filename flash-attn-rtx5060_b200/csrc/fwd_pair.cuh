// CTA-pair variant of the warp-specialised attention-forward kernel (head_dim 128, sm_100a).
//
// Two CTAs on the two SMs of a TPC form a cluster and share every K/V tile: each CTA loads only
// half of it (CTA r: keys [64r, 64r+64) of the K tile, head-dim columns [64r, 64r+64) of the V
// tile), and one tcgen05.mma.cta_group::2 instruction, issued by the even CTA, multiplies the
// q tiles of BOTH CTAs (M = 256) against the whole tile, each tensor core reading the B halves
// from both shared memories. Per CTA this halves the L2 -> shared-memory fill traffic and the
// shared-memory operand reads of B, which bound the one-CTA kernel (fwd_persistent.cuh).
//
// A work item is four adjacent 128-row q tiles of one (batch, head): stage s of CTA r owns tile
// 4*quad + 2*s + r. Roles per CTA are those of the one-CTA kernel (softmax 0-3 / 4-7, correction
// and epilogue 8-11, producer 13); warp 12 of the even CTA issues the MMAs for the pair, warp 12
// of the odd CTA forwards "my half has landed" to the even CTA. Barriers that the tensor pipe
// signals (S ready, O ready, slot free) are multicast to both CTAs by tcgen05.commit; barriers
// that gate an MMA collect arrivals from both CTAs in the even CTA's shared memory.
// No multicast TMA is used. Work items are assigned statically, in a serpentine over the
// cost-ordered item list, so the two CTAs of a pair need no run-time agreement on the next item.
#pragma once
#include "fwd_params.h"
#include "fwd_persistent.cuh"
#include "ptx.cuh"

namespace fa {

struct PairCfg {
  static constexpr int D = 128;
  static constexpr int kThreads = 512;
  static constexpr int kQTileBytes = kBlockM * D * 2;     // 32 KiB, two 16 KiB panels
  static constexpr int kSlotBytes = 16384;                // half a K tile (64 keys x 128) or half a V tile (128 keys x 64)
  static constexpr int kKPanelBytes = 64 * kPanel * 2;    // 8 KiB: 64 keys x 128 B
  static constexpr int kStages = 10;
  static constexpr int kOffQ = 0;
  static constexpr int kOffKV = 2 * kQTileBytes;
  static constexpr int kOffAlpha = kOffKV + kStages * kSlotBytes;  // float[2][128]
  static constexpr int kOffRowSum = kOffAlpha + 2 * kBlockM * 4;   // float[2][128]
  static constexpr int kOffBars = kOffRowSum + 2 * kBlockM * 4;
  static constexpr int kNumBars = 18 + 3 * kStages;
  static constexpr int kOffMisc = kOffBars + kNumBars * 8;
  static constexpr int kSmemBytes = kOffMisc + 16;
  static constexpr uint32_t kTmemCols = 512;
  static constexpr uint32_t kColS0 = 0, kColS1 = 128, kColO0 = 256, kColO1 = 384;
  static constexpr float kLazyLog2 = 8.f;
};

struct PairGeom {
  int bh, quad;
  bool on[2];        // stage has rows at all (its even tile starts inside the sequence)
  int r0[2], r1[2];  // this CTA's q rows per stage (virtual rows past the end of the sequence are never stored)
  int lo[2], hi[2];  // kv-tile range of the stage = union over the two CTAs' tiles
  int lo_all, hi_all;
};

// Same item order as the one-CTA kernel (heads in L2-sized groups, inside a group from the last
// quad to the first), with four q tiles per item.
__device__ __forceinline__ PairGeom decode_pair_item(int item, const FwdParams& p, int rank) {
  PairGeom g;
  const int per_group = p.head_group * p.num_q_pairs;  // num_q_pairs holds the number of quads here
  const int grp = item / per_group;
  const int r = item - grp * per_group;
  const int heads_here = min(p.head_group, p.bh - grp * p.head_group);
  const int pr = r / heads_here;
  g.bh = grp * p.head_group + (r - pr * heads_here);
  g.quad = p.num_q_pairs - 1 - pr;
  const int wr = eff_window_right(p.causal, p.window_right);
  g.lo_all = 0x7fffffff;
  g.hi_all = 0;
#pragma unroll
  for (int s = 0; s < 2; ++s) {
    const int a0 = (4 * g.quad + 2 * s) * kBlockM;  // first row of the even CTA's tile
    const int b0 = a0 + kBlockM;                    // first row of the odd CTA's tile
    g.on[s] = a0 < p.seqlen;
    g.r0[s] = rank ? b0 : a0;
    g.r1[s] = g.r0[s] + kBlockM - 1;
    if (g.r1[s] > p.seqlen - 1 && g.r0[s] < p.seqlen) g.r1[s] = p.seqlen - 1;
    if (!g.on[s]) {
      g.lo[s] = g.hi[s] = 0;
    } else {
      const int last = min((b0 < p.seqlen ? b0 : a0) + kBlockM, p.seqlen) - 1;
      g.lo[s] = kv_tile_begin(a0, p.window_left);
      g.hi[s] = kv_tile_end(last, wr, p.seqlen);
      g.lo_all = min(g.lo_all, g.lo[s]);
      g.hi_all = max(g.hi_all, g.hi[s]);
    }
  }
  return g;
}

// i-th item of cluster c out of G clusters: a serpentine over the cost-ordered list, so that every
// cluster gets a similar mix of long and short items. Returns -1 when the list is exhausted for
// this round, -2 when all rounds are done.
__device__ __forceinline__ int pair_item(int round, int c, int G, int num_items) {
  if (round * G >= num_items) return -2;
  const int idx = round * G + ((round & 1) ? (G - 1 - c) : c);
  return idx < num_items ? idx : -1;
}

template <bool kAlibi>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(512, 1)
fwd_pair_kernel(const __grid_constant__ CUtensorMap mapQ, const __grid_constant__ CUtensorMap mapKh,
                const __grid_constant__ CUtensorMap mapVh, const FwdParams p) {
  using Cfg = PairCfg;
  constexpr int D = Cfg::D;
  extern __shared__ __align__(1024) uint8_t smem[];

  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int lane = tid & 31;
  const int rank = static_cast<int>(cluster_ctarank());
  const int cluster_id = blockIdx.x >> 1;
  const int num_clusters = gridDim.x >> 1;

  // (uniform over the cluster: both CTAs get the same dynamic shared-memory offset)
  const bool misaligned = (smem_u32(smem) & 1023u) != 0;

  uint8_t* sQ = smem + Cfg::kOffQ;
  uint8_t* sKV = smem + Cfg::kOffKV;
  float* sAlpha = reinterpret_cast<float*>(smem + Cfg::kOffAlpha);
  float* sRowSum = reinterpret_cast<float*>(smem + Cfg::kOffRowSum);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + Cfg::kOffBars);
  uint64_t* q_full = bars;            // [2] own TMA -> MMA / relay
  uint64_t* q_empty = bars + 2;       // [2] MMA (multicast) -> own TMA
  uint64_t* s_full = bars + 4;        // [2] MMA (multicast) -> own softmax
  uint64_t* p_full = bars + 6;        // [2] even CTA only: softmax + correction warps of BOTH CTAs -> MMA
  uint64_t* alpha_ready = bars + 8;   // [2] own softmax -> own correction
  uint64_t* l_ready = bars + 10;      // [2] own softmax -> own correction
  uint64_t* o_full = bars + 12;       // [2] MMA (multicast) -> own correction
  uint64_t* p_full2 = bars + 14;      // [2] unused (P is handed over whole: every hand-off crosses the pair)
  uint64_t* q_peer = bars + 16;       // [2] even CTA only: the odd CTA's Q tile has landed
  uint64_t* kv_full = bars + 18;                       // [kStages] own TMA -> MMA / relay
  uint64_t* kv_empty = bars + 18 + Cfg::kStages;       // [kStages] MMA (multicast) -> own TMA
  uint64_t* kv_peer = bars + 18 + 2 * Cfg::kStages;    // [kStages] even CTA only: the odd CTA's half has landed
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + Cfg::kOffMisc);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  if (warp == 12) {
    tmem_alloc(tmem_slot, Cfg::kTmemCols);  // each CTA allocates all of its own TMEM: same base in both
    tmem_relinquish();
  }
  if (tid == 0) {
#pragma unroll
    for (int s = 0; s < 2; ++s) {
      mbar_init(&q_full[s], 1);
      mbar_init(&q_empty[s], 1);
      mbar_init(&s_full[s], 1);
      mbar_init(&p_full[s], 16);  // 4 softmax + 4 correction warps of each CTA
      mbar_init(&p_full2[s], 8);
      mbar_init(&alpha_ready[s], 4);
      mbar_init(&l_ready[s], 4);
      mbar_init(&o_full[s], 1);
      mbar_init(&q_peer[s], 1);
    }
    for (int i = 0; i < Cfg::kStages; ++i) {
      mbar_init(&kv_full[i], 1);
      mbar_init(&kv_empty[i], 1);
      mbar_init(&kv_peer[i], 1);
    }
    *abort_flag = misaligned ? 1 : 0;
    fence_mbar_init();
  }
  if (warp == 13 && lane == 0) {
    prefetch_tensormap(&mapQ);
    prefetch_tensormap(&mapKh);
    prefetch_tensormap(&mapVh);
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();  // the peer's barriers exist before anyone arrives on them
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  const int N = p.seqlen;
  const int wl = p.window_left;
  const int wr = eff_window_right(p.causal, p.window_right);
  // barriers of the even CTA that both CTAs arrive on
  const uint32_t p_full_even[2] = {mapa_u32(smem_u32(&p_full[0]), 0), mapa_u32(smem_u32(&p_full[1]), 0)};

  if (misaligned) {
    // swizzled tiles need a 1024-byte aligned base; nothing was issued, fall through to the common exit
  } else if (warp < 8) {
    // =====================================================================================
    // softmax: stage s = warp / 4, row = tid % 128 of this CTA's tile of that stage
    // =====================================================================================
    reg_inc<168>();
    const int s = warp >> 2;
    const int row_l = tid & 127;
    const uint32_t lane_base = static_cast<uint32_t>(warp & 3) * 32u;
    const uint32_t tS = tmem_addr(tmem_base, lane_base, s == 0 ? Cfg::kColS0 : Cfg::kColS1);
    const float sl2 = kAlibi ? 1.f : p.scale_log2;
    const uint64_t scale2 = f2_pack(sl2, sl2);
    uint32_t n_s = 0;
    bool ok = true;
    for (int round = 0; ok; ++round) {
      const int item = pair_item(round, cluster_id, num_clusters, p.num_items);
      if (item == -2) break;
      if (item < 0) continue;
      const PairGeom g = decode_pair_item(item, p, rank);
      const bool on = s ? g.on[1] : g.on[0];
      if (!on) continue;
      const int q_r0 = s ? g.r0[1] : g.r0[0];
      const int q_r1 = s ? g.r1[1] : g.r1[0];
      const int j_lo = s ? g.lo[1] : g.lo[0];
      const int j_hi = s ? g.hi[1] : g.hi[0];
      const int row = q_r0 + row_l;
      float slope_l2 = 0.f;
      if (kAlibi) slope_l2 = p.alibi_slopes[g.bh % p.heads] * 1.4426950408889634f;
      float m_run = -INFINITY;
      float m_used = 0.f;
      float l_run = 0.f;
      for (int j = j_lo; j < j_hi; ++j) {
        if (!mbar_wait_warp(&s_full[s], n_s & 1, abort_flag)) { ok = false; break; }
        ++n_s;
        tc_fence_after();
#ifdef FA_PAIR_FAKE  // bring-up only: the load + tensor pipeline of the pair without the softmax work
        sAlpha[s * kBlockM + row_l] = 1.f;
        __syncwarp();
        if (lane == 0) { mbar_arrive(&alpha_ready[s]); mbar_arrive_cluster(p_full_even[s]); }
        l_run = 1.f;
        continue;
#endif
        uint32_t r0[32], r1[32], r2[32], r3[32];
        tmem_ld32(tS + 0, r0);
        tmem_ld32(tS + 32, r1);
        tmem_ld32(tS + 64, r2);
        tmem_ld32(tS + 96, r3);
        tmem_wait_ld();
        tmem_ld_fence(r0);
        tmem_ld_fence(r1);
        tmem_ld_fence(r2);
        tmem_ld_fence(r3);
        float sc[kBlockN];
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          sc[i] = __uint_as_float(r0[i]);
          sc[32 + i] = __uint_as_float(r1[i]);
          sc[64 + i] = __uint_as_float(r2[i]);
          sc[96 + i] = __uint_as_float(r3[i]);
        }
        const int kv0 = j * kBlockN;
        if (kAlibi) {
          const float rel = static_cast<float>(row - kv0);
#pragma unroll
          for (int c = 0; c < kBlockN; ++c)
            sc[c] = fmaf(sc[c], p.scale_log2, -slope_l2 * fabsf(rel - static_cast<float>(c)));
        }
        // The stage's kv range is the union over the pair, so a tile may lie wholly outside this
        // CTA's visible range: the predicate then masks every column and P is zero.
        const bool masked = kv_tile_needs_mask(kv0, q_r0, q_r1, wl, wr, N);
        if (masked) {
          const int c_lo = (wl >= 0) ? row - wl - kv0 : -1;
          int c_hi = N - 1 - kv0;
          if (wr >= 0) c_hi = min(c_hi, row + wr - kv0);
#pragma unroll
          for (int c = 0; c < kBlockN; ++c)
            if (c < c_lo || c > c_hi) sc[c] = -INFINITY;
        }
        float mx0 = m_run, mx1 = -INFINITY, mx2 = -INFINITY, mx3 = -INFINITY;
#pragma unroll
        for (int c = 0; c < kBlockN; c += 8) {
          mx0 = max3(mx0, sc[c], sc[c + 1]);
          mx1 = max3(mx1, sc[c + 2], sc[c + 3]);
          mx2 = max3(mx2, sc[c + 4], sc[c + 5]);
          mx3 = max3(mx3, sc[c + 6], sc[c + 7]);
        }
        const float m_new = max3(mx0, mx1, fmaxf(mx2, mx3));
        float alpha = 1.f;
        if (m_run == -INFINITY) {
          m_used = (m_new == -INFINITY) ? 0.f : m_new;
        } else if ((m_new - m_used) * sl2 > Cfg::kLazyLog2) {
          alpha = ex2_approx((m_used - m_new) * sl2);
          m_used = m_new;
        }
        m_run = m_new;
        sAlpha[s * kBlockM + row_l] = alpha;
        __syncwarp();
        if (lane == 0) mbar_arrive(&alpha_ready[s]);

        const float neg_ms = -m_used * sl2;
        const uint64_t negms2 = f2_pack(neg_ms, neg_ms);
        uint64_t lsum_a = 0ull, lsum_b = 0ull;
        uint32_t pk0[32], pk1[32];
        if (masked) exp_half_tile<false>(sc, scale2, negms2, pk0, lsum_a, lsum_b);
        else exp_half_tile<true>(sc, scale2, negms2, pk0, lsum_a, lsum_b);
        tmem_st32(tS + 0, pk0);
        tmem_wait_st();
        tc_fence_before();
        __syncwarp();
        if (masked) exp_half_tile<false>(sc + 64, scale2, negms2, pk1, lsum_a, lsum_b);
        else exp_half_tile<true>(sc + 64, scale2, negms2, pk1, lsum_a, lsum_b);
        tmem_st32(tS + 32, pk1);
        float l0, l1;
        f2_unpack(f2_add(lsum_a, lsum_b), l0, l1);
        l_run = l_run * alpha + (l0 + l1);
        tmem_wait_st();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive_cluster(p_full_even[s]);  // the whole P tile is in TMEM
      }
      if (!ok) break;
      sRowSum[s * kBlockM + row_l] = l_run;
      __syncwarp();
      if (lane == 0) mbar_arrive(&l_ready[s]);
    }
  } else if (warp < 12) {
    // =====================================================================================
    // correction + epilogue for this CTA's rows of both stages
    // =====================================================================================
    reg_dec<96>();
    const int row_l = tid & 127;
    const uint32_t lane_base = static_cast<uint32_t>(warp & 3) * 32u;
    uint32_t n_alpha[2] = {0, 0}, n_l[2] = {0, 0}, n_o[2] = {0, 0};
    bool ok = true;
    for (int round = 0; ok; ++round) {
      const int item = pair_item(round, cluster_id, num_clusters, p.num_items);
      if (item == -2) break;
      if (item < 0) continue;
      const PairGeom g = decode_pair_item(item, p, rank);
      for (int j = g.lo_all; j < g.hi_all && ok; ++j) {
#pragma unroll
        for (int s = 0; s < 2; ++s) {
          if (!g.on[s] || j < g.lo[s] || j >= g.hi[s]) continue;
          if (!mbar_wait_warp(&alpha_ready[s], n_alpha[s] & 1, abort_flag)) { ok = false; break; }
          ++n_alpha[s];
          const float alpha = sAlpha[s * kBlockM + row_l];
          if (j > g.lo[s] && __any_sync(0xffffffffu, alpha != 1.f)) {
            tc_fence_after();
            const uint32_t tO = tmem_addr(tmem_base, lane_base, s == 0 ? Cfg::kColO0 : Cfg::kColO1);
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
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive_cluster(p_full_even[s]);
        }
      }
      if (!ok) break;
#pragma unroll
      for (int s = 0; s < 2; ++s) {
        if (!g.on[s]) continue;
        if (!mbar_wait_warp(&l_ready[s], n_l[s] & 1, abort_flag)) { ok = false; break; }
        ++n_l[s];
        const float l = sRowSum[s * kBlockM + row_l];
        if (!mbar_wait_warp(&o_full[s], n_o[s] & 1, abort_flag)) { ok = false; break; }
        ++n_o[s];
        tc_fence_after();
        const float inv_l = (l > 0.f) ? 1.f / l : 0.f;
        const int row = g.r0[s] + row_l;
        const uint32_t tO = tmem_addr(tmem_base, lane_base, s == 0 ? Cfg::kColO0 : Cfg::kColO1);
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
    reg_dec<80>();
    if (warp == 12 && rank == 0) {
      // ===================================================================================
      // tensor-core issuer of the pair (even CTA)
      // ===================================================================================
      constexpr uint32_t idesc_qk = umma_idesc_f16(2 * kBlockM, kBlockN, 0, 0);
      constexpr uint32_t idesc_pv = umma_idesc_f16(2 * kBlockM, D, 0, 1);
      const uint64_t kdesc0 = umma_desc_sw128(0, 16, 1024);  // K-major tiles (Q, K half)
      const uint64_t vdesc0 = umma_desc_sw128(0, 16, 1024);  // MN-major V half: one 64-wide atom along N
      const uint32_t q_addr = smem_u32(sQ);
      const uint32_t kv_addr = smem_u32(sKV);
      const uint64_t qdesc[2] = {kdesc0 + (q_addr >> 4), kdesc0 + ((q_addr + Cfg::kQTileBytes) >> 4)};
      uint32_t it_base = 0;
      uint32_t n_p[2] = {0, 0}, n_q[2] = {0, 0};
      bool ok = true;
      for (int round = 0; ok; ++round) {
        const int item = pair_item(round, cluster_id, num_clusters, p.num_items);
        if (item == -2) break;
        if (item < 0) continue;
        const PairGeom g = decode_pair_item(item, p, rank);
        for (int j = g.lo_all - 1; j < g.hi_all && ok; ++j) {
#pragma unroll
          for (int s = 0; s < 2; ++s) {
            const bool act_j = g.on[s] && (j >= g.lo[s] && j < g.hi[s]);
            const bool act_n = g.on[s] && (j + 1 >= g.lo[s] && j + 1 < g.hi[s]);
            const bool other_j = (s == 0) && g.on[1] && (j >= g.lo[1] && j < g.hi[1]);
            const bool other_n = (s == 0) && g.on[1] && (j + 1 >= g.lo[1] && j + 1 < g.hi[1]);
            const bool v_seen = (s == 1) && g.on[0] && (j >= g.lo[0] && j < g.hi[0]);
            const bool k_seen = (s == 1) && g.on[0] && (j + 1 >= g.lo[0] && j + 1 < g.hi[0]);
            const uint32_t colS = (s == 0) ? Cfg::kColS0 : Cfg::kColS1;
            const uint32_t colO = (s == 0) ? Cfg::kColO0 : Cfg::kColO1;
            if (act_j) {  // O_s += P_s(j) V_j for both CTAs
              const uint32_t it = it_base + 2u * (j - g.lo_all) + 1u;
              const uint32_t slot = it % Cfg::kStages;
              const uint32_t par = (it / Cfg::kStages) & 1u;
              const uint64_t vdesc = vdesc0 + ((kv_addr + slot * Cfg::kSlotBytes) >> 4);
              if (!v_seen) {
                if (!mbar_wait_warp(&kv_full[slot], par, abort_flag)) { ok = false; break; }
                if (!mbar_wait_cluster_warp(&kv_peer[slot], par, abort_flag)) { ok = false; break; }
              }
              if (!mbar_wait_cluster_warp(&p_full[s], n_p[s] & 1, abort_flag)) { ok = false; break; }
              tc_fence_after();
              if (elect_one()) {
                umma_ts_2cta(tmem_base + colO, tmem_base + colS, vdesc, idesc_pv, (j > g.lo[s]) ? 1u : 0u);
#pragma unroll
                for (int kk = 1; kk < 4; ++kk)
                  umma_ts_2cta(tmem_base + colO, tmem_base + colS + kk * 8, vdesc + kk * (2048 >> 4), idesc_pv, 1u);
              }
              __syncwarp();
              ++n_p[s];
              if (elect_one()) {
#pragma unroll
                for (int kk = 4; kk < 8; ++kk)
                  umma_ts_2cta(tmem_base + colO, tmem_base + colS + kk * 8, vdesc + kk * (2048 >> 4), idesc_pv, 1u);
                if (!other_j) umma_commit_2cta(&kv_empty[slot], 3);
                if (j + 1 == g.hi[s]) umma_commit_2cta(&o_full[s], 3);
              }
              __syncwarp();
            }
            if (act_n) {  // S_s = Q_s K_{j+1}^T for both CTAs
              const uint32_t it = it_base + 2u * (j + 1 - g.lo_all);
              const uint32_t slot = it % Cfg::kStages;
              const uint32_t par = (it / Cfg::kStages) & 1u;
              if (j + 1 == g.lo[s]) {
                if (!mbar_wait_warp(&q_full[s], n_q[s] & 1, abort_flag)) { ok = false; break; }
                if (!mbar_wait_cluster_warp(&q_peer[s], n_q[s] & 1, abort_flag)) { ok = false; break; }
                ++n_q[s];
              }
              if (!k_seen) {
                if (!mbar_wait_warp(&kv_full[slot], par, abort_flag)) { ok = false; break; }
                if (!mbar_wait_cluster_warp(&kv_peer[slot], par, abort_flag)) { ok = false; break; }
              }
              tc_fence_after();
              const uint64_t kdesc = kdesc0 + ((kv_addr + slot * Cfg::kSlotBytes) >> 4);
              if (elect_one()) {
#pragma unroll
                for (int k = 0; k < D / 16; ++k) {
                  const uint32_t offq = ((k / 4) * (kBlockM * kPanel * 2) + (k % 4) * 32) >> 4;
                  const uint32_t offk = ((k / 4) * Cfg::kKPanelBytes + (k % 4) * 32) >> 4;
                  umma_ss_2cta(tmem_base + colS, qdesc[s] + offq, kdesc + offk, idesc_qk, k > 0 ? 1u : 0u);
                }
                umma_commit_2cta(&s_full[s], 3);
                if (!other_n) umma_commit_2cta(&kv_empty[slot], 3);
                if (j + 2 == g.hi[s]) umma_commit_2cta(&q_empty[s], 3);
              }
              __syncwarp();
            }
          }
        }
        it_base += 2u * (g.hi_all - g.lo_all);
      }
    } else if (warp == 12 && rank == 1 && lane == 0) {
      // ===================================================================================
      // odd CTA: tell the issuer when this CTA's Q tiles and K/V halves have landed
      // ===================================================================================
      uint32_t it = 0;
      uint32_t n_q[2] = {0, 0};
      bool ok = true;
      for (int round = 0; ok; ++round) {
        const int item = pair_item(round, cluster_id, num_clusters, p.num_items);
        if (item == -2) break;
        if (item < 0) continue;
        const PairGeom g = decode_pair_item(item, p, rank);
#pragma unroll
        for (int s = 0; s < 2; ++s) {
          if (!g.on[s]) continue;
          if (!mbar_wait(&q_full[s], n_q[s] & 1, abort_flag)) { ok = false; break; }
          ++n_q[s];
          mbar_arrive_cluster(mapa_u32(smem_u32(&q_peer[s]), 0));
        }
        for (int j = g.lo_all; j < g.hi_all && ok; ++j) {
#pragma unroll
          for (int t = 0; t < 2; ++t) {
            const uint32_t slot = it % Cfg::kStages;
            if (!mbar_wait(&kv_full[slot], (it / Cfg::kStages) & 1u, abort_flag)) { ok = false; break; }
            mbar_arrive_cluster(mapa_u32(smem_u32(&kv_peer[slot]), 0));
            ++it;
          }
        }
      }
    } else if (warp == 13 && lane == 0) {
      // ===================================================================================
      // TMA producer: own Q tiles, own half of every K and V tile
      // ===================================================================================
      uint32_t it = 0;
      uint32_t n_q[2] = {0, 0};
      bool ok = true;
      for (int round = 0; ok; ++round) {
        const int item = pair_item(round, cluster_id, num_clusters, p.num_items);
        if (item == -2) break;
        if (item < 0) continue;
        const PairGeom g = decode_pair_item(item, p, rank);
#pragma unroll
        for (int s = 0; s < 2; ++s) {
          if (!g.on[s]) continue;
          if (!mbar_wait(&q_empty[s], (n_q[s] & 1) ^ 1, abort_flag)) { ok = false; break; }
          ++n_q[s];
          mbar_arrive_expect_tx(&q_full[s], Cfg::kQTileBytes);
          tma_load_4d(sQ + s * Cfg::kQTileBytes, &mapQ, &q_full[s], 0, g.r0[s], 0, g.bh);
        }
        for (int j = g.lo_all; j < g.hi_all && ok; ++j) {
#pragma unroll
          for (int t = 0; t < 2; ++t) {
            const uint32_t slot = it % Cfg::kStages;
            if (!mbar_wait(&kv_empty[slot], ((it / Cfg::kStages) & 1) ^ 1, abort_flag)) { ok = false; break; }
            mbar_arrive_expect_tx(&kv_full[slot], Cfg::kSlotBytes);
            if (t == 0)  // keys [64*rank, 64*rank + 64) of the K tile, all 128 head-dim columns
              tma_load_4d(sKV + slot * Cfg::kSlotBytes, &mapKh, &kv_full[slot], 0, j * kBlockN + 64 * rank, 0, g.bh);
            else         // all 128 keys of the V tile, head-dim columns [64*rank, 64*rank + 64)
              tma_load_4d(sKV + slot * Cfg::kSlotBytes, &mapVh, &kv_full[slot], 0, j * kBlockN, rank, g.bh);
            ++it;
          }
        }
      }
      if (!ok) {
        for (int i = 0; i < 64; ++i) __nanosleep(2000);  // give-up path: let loads in flight land
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  // Neither CTA may retire (or free its TMEM) while the pair's MMAs or remote arrivals can still
  // touch it.
  cluster_sync_all();
  if (tid == 0 && *abort_flag != 0) atomicExch(p.status, misaligned ? 2 : 1);
  if (warp == 12) tmem_dealloc(tmem_base, Cfg::kTmemCols);
}

}  // namespace fa
