// CTA-pair attention forward with the scores computed two kv tiles ahead (head_dim 128, sm_100a).
//
// Two CTAs on the two SMs of a TPC form a cluster. Each CTA owns ONE 128-row q tile of a work item
// (CTA r: tile 2*pair + r of a (batch, head)); one tcgen05.mma.cta_group::2 instruction issued by the
// even CTA multiplies both q tiles (M = 256) against a K or V tile of which each CTA holds half in
// its shared memory, so the per-CTA fill traffic and the B-operand reads are half those of the
// one-CTA kernel (fwd_persistent.cuh).
//
// Tensor memory per CTA: S_a [0,128), S_b [128,256), O [256,384), P_a [384,448), P_b [448,512).
// With two score buffers and P in columns of its own, S(t+2) = Q K(t+2)^T depends only on the
// softmax threads having READ S(t), not on P(t)V(t): the tensor pipe computes scores two tiles
// ahead of the softmax, and the only serial chain left is the softmax itself. Every hand-off that
// crosses the pair (P ready, S buffer free) therefore has a full softmax tile of slack.
//
// Tiles of the whole item list of a cluster are numbered t = 0, 1, ...; tile t uses score buffer,
// P buffer and alpha slot t & 1, K ring slot 2t and V ring slot 2t + 1 (mod kStages).
// Roles per CTA (384 threads): warps 0-3 softmax (thread = q row), 4-7 correction + epilogue,
// warp 8 tensor-core issuer (even CTA) / "my half has landed" relay (odd CTA), warp 9 TMA producer.
// No multicast TMA is used. Work items are assigned statically (serpentine over the cost-ordered
// list), so the two CTAs need no run-time agreement on the next item.
#pragma once
#include "fwd_pair.cuh"
#include "fwd_params.h"
#include "fwd_persistent.cuh"
#include "ptx.cuh"

namespace fa {

// Bring-up only: with FA_AHEAD_PROF one thread per role of cluster 0's even CTA adds the clocks it spends in each
// phase into p.dbg (64-bit counters, 16 per role).
#ifdef FA_AHEAD_PROF
#define FA_AP_DECL long long ap_t = clock64(); long long ap_acc[8] = {0, 0, 0, 0, 0, 0, 0, 0}
#define FA_AP(i) { const long long ap_n = clock64(); ap_acc[i] += ap_n - ap_t; ap_t = ap_n; }
#define FA_AP_STORE(cond, role) if ((cond) && p.dbg != nullptr) { for (int ap_i = 0; ap_i < 8; ++ap_i) \
    reinterpret_cast<long long*>(p.dbg)[(role) * 16 + ap_i] = ap_acc[ap_i]; }
#else
#define FA_AP_DECL
#define FA_AP(i)
#define FA_AP_STORE(cond, role)
#endif

struct AheadCfg {
  static constexpr int D = 128;
  static constexpr int kThreads = 384;
  static constexpr int kQTileBytes = kBlockM * D * 2;   // 32 KiB, two 16 KiB panels
  static constexpr int kSlotBytes = 16384;              // half a K tile (64 keys x 128) or half a V tile (128 keys x 64)
  static constexpr int kKPanelBytes = 64 * kPanel * 2;  // 8 KiB: 64 keys x 128 B
  static constexpr int kStages = 10;
  static constexpr int kOffQ = 0;                                  // two Q buffers (item parity)
  static constexpr int kOffKV = 2 * kQTileBytes;
  static constexpr int kOffAlpha = kOffKV + kStages * kSlotBytes;  // float[2][128], by t & 1
  static constexpr int kOffRowSum = kOffAlpha + 2 * kBlockM * 4;   // float[2][128], by item parity
  static constexpr int kOffBars = kOffRowSum + 2 * kBlockM * 4;
  static constexpr int kNumBars = 20 + 3 * kStages;
  static constexpr int kOffMisc = kOffBars + kNumBars * 8;
  static constexpr int kSmemBytes = kOffMisc + 16;
  static constexpr uint32_t kTmemCols = 512;
  static constexpr uint32_t kColS = 0, kColO = 256, kColP = 384;  // S buffer b at kColS + 128 b, P buffer b at kColP + 64 b
  static constexpr float kLazyLog2 = 8.f;
  static constexpr int kRegSoftmax = 232, kRegCorr = 104, kRegMisc = 80;
};

struct AheadGeom {
  int bh;
  int r0, r1;  // this CTA's q rows (r0 may lie past the end of the sequence: the tile is then computed on
               // zero-filled Q and never stored)
  int lo, hi;  // kv-tile range of the item = union over the two CTAs' tiles
};

// Same item order as the one-CTA kernel: heads in L2-sized groups, inside a group from the last
// pair of q tiles to the first.
__device__ __forceinline__ AheadGeom decode_ahead_item(int item, const FwdParams& p, int rank) {
  AheadGeom g;
  const int per_group = p.head_group * p.num_q_pairs;
  const int grp = item / per_group;
  const int r = item - grp * per_group;
  const int heads_here = min(p.head_group, p.bh - grp * p.head_group);
  const int pr = r / heads_here;
  g.bh = grp * p.head_group + (r - pr * heads_here);
  const int pair = p.num_q_pairs - 1 - pr;
  const int wr = eff_window_right(p.causal, p.window_right);
  const int a0 = 2 * pair * kBlockM;  // first row of the even CTA's tile (always inside the sequence)
  const int b0 = a0 + kBlockM;        // first row of the odd CTA's tile
  g.r0 = rank ? b0 : a0;
  g.r1 = g.r0 + kBlockM - 1;
  if (g.r1 > p.seqlen - 1 && g.r0 < p.seqlen) g.r1 = p.seqlen - 1;
  const int last = min((b0 < p.seqlen ? b0 : a0) + kBlockM, p.seqlen) - 1;
  g.lo = kv_tile_begin(a0, p.window_left);
  g.hi = kv_tile_end(last, wr, p.seqlen);
  return g;
}

// Position in the cluster's tile stream: item after item, kv tile after kv tile.
struct AheadCursor {
  int round, j;
  uint32_t t, n_item;
  bool valid;
  AheadGeom g;
  __device__ __forceinline__ void next_item(const FwdParams& p, int rank, int cluster_id, int num_clusters) {
    for (;;) {
      ++round;
      const int item = pair_item(round, cluster_id, num_clusters, p.num_items);
      if (item == -2) { valid = false; return; }
      if (item < 0) continue;
      g = decode_ahead_item(item, p, rank);
      j = g.lo;
      ++n_item;
      valid = true;
      return;
    }
  }
  __device__ __forceinline__ void start(const FwdParams& p, int rank, int cluster_id, int num_clusters) {
    round = -1;
    t = 0;
    n_item = 0xffffffffu;
    next_item(p, rank, cluster_id, num_clusters);
  }
  __device__ __forceinline__ void advance(const FwdParams& p, int rank, int cluster_id, int num_clusters) {
    ++j;
    ++t;
    if (j >= g.hi) next_item(p, rank, cluster_id, num_clusters);
  }
};

template <bool kAlibi>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(384, 1)
fwd_pair_ahead_kernel(const __grid_constant__ CUtensorMap mapQ, const __grid_constant__ CUtensorMap mapKh,
                      const __grid_constant__ CUtensorMap mapVh, const FwdParams p) {
  using Cfg = AheadCfg;
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
  uint64_t* q_full = bars;            // [2] own TMA -> issuer / relay                    (by item parity)
  uint64_t* q_empty = bars + 2;       // [2] issuer (multicast) -> own TMA               (by item parity)
  uint64_t* q_peer = bars + 4;        // [2] even CTA only: the odd CTA's Q tile has landed
  uint64_t* s_full = bars + 6;        // [2] issuer (multicast) -> own softmax            (by t & 1)
  uint64_t* s_free = bars + 8;        // [2] even CTA only: softmax warps of BOTH CTAs have read S -> issuer
  uint64_t* p_full = bars + 10;       // [2] even CTA only: softmax + correction warps of BOTH CTAs -> issuer
  uint64_t* p_free = bars + 12;       // [2] issuer (multicast): P(t) V(t) has completed -> own softmax, correction
  uint64_t* alpha_ready = bars + 14;  // [2] own softmax -> own correction
  uint64_t* l_ready = bars + 16;      // own softmax -> own correction (once per item)
  uint64_t* o_full = bars + 17;       // issuer (multicast) -> own correction (once per item)
  uint64_t* o_empty = bars + 18;      // even CTA only: correction warps of BOTH CTAs have read O -> issuer
  uint64_t* kv_full = bars + 20;                       // [kStages] own TMA -> issuer / relay
  uint64_t* kv_empty = bars + 20 + Cfg::kStages;       // [kStages] issuer (multicast) -> own TMA
  uint64_t* kv_peer = bars + 20 + 2 * Cfg::kStages;    // [kStages] even CTA only: the odd CTA's half has landed
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + Cfg::kOffMisc);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  if (warp == 8) {
    tmem_alloc(tmem_slot, Cfg::kTmemCols);  // each CTA allocates all of its own TMEM: same base in both
    tmem_relinquish();
  }
  if (tid == 0) {
#pragma unroll
    for (int b = 0; b < 2; ++b) {
      mbar_init(&q_full[b], 1);
      mbar_init(&q_empty[b], 1);
      mbar_init(&q_peer[b], 1);
      mbar_init(&s_full[b], 1);
      mbar_init(&s_free[b], 8);   // 4 softmax warps of each CTA
      mbar_init(&p_full[b], 16);  // 4 softmax + 4 correction warps of each CTA
      mbar_init(&p_free[b], 1);
      mbar_init(&alpha_ready[b], 4);
    }
    mbar_init(l_ready, 4);
    mbar_init(o_full, 1);
    mbar_init(o_empty, 8);  // 4 correction warps of each CTA
    for (int i = 0; i < Cfg::kStages; ++i) {
      mbar_init(&kv_full[i], 1);
      mbar_init(&kv_empty[i], 1);
      mbar_init(&kv_peer[i], 1);
    }
    *abort_flag = misaligned ? 1 : 0;
    fence_mbar_init();
  }
  if (warp == 9 && lane == 0) {
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
  const uint32_t s_free_even[2] = {mapa_u32(smem_u32(&s_free[0]), 0), mapa_u32(smem_u32(&s_free[1]), 0)};
  const uint32_t p_full_even[2] = {mapa_u32(smem_u32(&p_full[0]), 0), mapa_u32(smem_u32(&p_full[1]), 0)};
  const uint32_t o_empty_even = mapa_u32(smem_u32(o_empty), 0);

  if (misaligned) {
    // swizzled tiles need a 1024-byte aligned base; nothing was issued, fall through to the common exit
  } else if (warp < 4) {
    // =====================================================================================
    // softmax: thread = q row of this CTA's tile, kv tiles in sequence
    // =====================================================================================
    reg_inc<Cfg::kRegSoftmax>();
    const int row_l = tid & 127;
    const uint32_t lane_base = static_cast<uint32_t>(warp & 3) * 32u;
    const float sl2 = kAlibi ? 1.f : p.scale_log2;
    const uint64_t scale2 = f2_pack(sl2, sl2);
    uint32_t t = 0, n_item = 0;
    bool ok = true;
    FA_AP_DECL;
    for (int round = 0; ok; ++round) {
      const int item = pair_item(round, cluster_id, num_clusters, p.num_items);
      if (item == -2) break;
      if (item < 0) continue;
      const AheadGeom g = decode_ahead_item(item, p, rank);
      const int row = g.r0 + row_l;
      float slope_l2 = 0.f;
      if (kAlibi) slope_l2 = p.alibi_slopes[g.bh % p.heads] * 1.4426950408889634f;
      float m_run = -INFINITY;  // true running max of the raw scores
      float m_used = 0.f;       // max the exponentials are currently taken against
      float l_run = 0.f;
      for (int j = g.lo; j < g.hi; ++j, ++t) {
        const uint32_t b = t & 1u, ph = (t >> 1) & 1u;
        const uint32_t tS = tmem_addr(tmem_base, lane_base, Cfg::kColS + 128u * b);
        const uint32_t tP = tmem_addr(tmem_base, lane_base, Cfg::kColP + 64u * b);
        FA_AP(0);
        if (!mbar_wait_warp(&s_full[b], ph, abort_flag)) { ok = false; break; }
        tc_fence_after();
        FA_AP(1);
#ifdef FA_AHEAD_FAKE  // bring-up only: the load + tensor pipeline of the pair without the softmax work
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive_peer(s_free_even[b]);
        if (!mbar_wait_warp(&p_free[b], ph ^ 1u, abort_flag)) { ok = false; break; }
        sAlpha[b * kBlockM + row_l] = 1.f;
        __syncwarp();
        if (lane == 0) { mbar_arrive(&alpha_ready[b]); mbar_arrive_peer(p_full_even[b]); }
        l_run = 1.f;
        continue;
#endif
        const int kv0 = j * kBlockN;
        // One body, instantiated twice: tiles cut by a mask boundary (or by the end of the sequence, or lying
        // wholly outside this CTA's visible range, since the item's kv range is the union over the pair)
        // take the per-element predicate and MUFU-only exponentials, all others carry none of that code.
        auto tile_body = [&](auto masked_tag) -> bool {
          constexpr bool kMasked = decltype(masked_tag)::value;
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
          // the scores are in registers: the buffer may take S(t + 2)
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive_peer(s_free_even[b]);
          FA_AP(2);
          float sc[kBlockN];
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            sc[i] = __uint_as_float(r0[i]);
            sc[32 + i] = __uint_as_float(r1[i]);
            sc[64 + i] = __uint_as_float(r2[i]);
            sc[96 + i] = __uint_as_float(r3[i]);
          }
          if (kAlibi) {  // s * scale - slope * |i - j|, in log2 units (reference: src/mask.h:21-26, src/main.cu:200-207)
            const float rel = static_cast<float>(row - kv0);
#pragma unroll
            for (int c = 0; c < kBlockN; ++c)
              sc[c] = fmaf(sc[c], p.scale_log2, -slope_l2 * fabsf(rel - static_cast<float>(c)));
          }
          if (kMasked) {
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
          // Lazy rescale, branch-free (as in the one-CTA kernel): the reference max moves only when the true
          // max has grown by more than kLazyLog2 or when no finite score was seen before.
          const bool fresh = (m_run == -INFINITY);
          const bool move = fresh || (m_new - m_used) * sl2 > Cfg::kLazyLog2;
          const float m_next = move ? ((m_new == -INFINITY) ? 0.f : m_new) : m_used;
          float alpha = ex2_approx((m_used - m_next) * sl2);
          alpha = fresh ? 1.f : alpha;
          m_used = m_next;
          m_run = m_new;
          // P(t - 2) V(t - 2) has completed: its P buffer and alpha slot (read by the correction warps before
          // they let that product start) may be overwritten.
          FA_AP(3);
          if (!mbar_wait_warp(&p_free[b], ph ^ 1u, abort_flag)) return false;
          FA_AP(4);
          sAlpha[b * kBlockM + row_l] = alpha;
          __syncwarp();
          if (lane == 0) mbar_arrive(&alpha_ready[b]);

          const float neg_ms = -m_used * sl2;
          const uint64_t negms2 = f2_pack(neg_ms, neg_ms);
          uint64_t lsum_a = 0ull, lsum_b = 0ull;
          uint32_t pk0[32], pk1[32];
          // masked tiles hold -inf scores, which only the MUFU path maps to 0
          exp_half_tile<!kMasked>(sc, scale2, negms2, pk0, lsum_a, lsum_b);
          tmem_st32(tP + 0, pk0);
          exp_half_tile<!kMasked>(sc + 64, scale2, negms2, pk1, lsum_a, lsum_b);
          tmem_st32(tP + 32, pk1);
          float l0, l1;
          f2_unpack(f2_add(lsum_a, lsum_b), l0, l1);
          l_run = l_run * alpha + (l0 + l1);
          FA_AP(5);
          tmem_wait_st();
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive_peer(p_full_even[b]);  // the whole P tile is in TMEM
          FA_AP(6);
          return true;
        };
        if (kv_tile_needs_mask(kv0, g.r0, g.r1, wl, wr, N)) ok = tile_body(std::true_type{});
        else ok = tile_body(std::false_type{});
        if (!ok) break;
      }
      if (!ok) break;
      sRowSum[(n_item & 1u) * kBlockM + row_l] = l_run;
      __syncwarp();
      if (lane == 0) mbar_arrive(l_ready);
      ++n_item;
    }
    FA_AP_STORE(blockIdx.x == 0 && tid == 0, 0);
  } else if (warp < 8) {
    // =====================================================================================
    // correction + epilogue for this CTA's rows
    // =====================================================================================
    reg_dec<Cfg::kRegCorr>();
    const int row_l = tid & 127;
    const uint32_t lane_base = static_cast<uint32_t>(warp & 3) * 32u;
    const uint32_t tO = tmem_addr(tmem_base, lane_base, Cfg::kColO);
    uint32_t t = 0, n_item = 0;
    bool ok = true;
    for (int round = 0; ok; ++round) {
      const int item = pair_item(round, cluster_id, num_clusters, p.num_items);
      if (item == -2) break;
      if (item < 0) continue;
      const AheadGeom g = decode_ahead_item(item, p, rank);
      for (int j = g.lo; j < g.hi && ok; ++j, ++t) {
        const uint32_t b = t & 1u, ph = (t >> 1) & 1u;
        if (!mbar_wait_warp(&alpha_ready[b], ph, abort_flag)) { ok = false; break; }
        const float alpha = sAlpha[b * kBlockM + row_l];
        if (j > g.lo && __any_sync(0xffffffffu, alpha != 1.f)) {
          // O may be rescaled only between P(t-1) V(t-1) and P(t) V(t): wait for the former to complete
          if (!mbar_wait_warp(&p_free[b ^ 1u], ((t - 1u) >> 1) & 1u, abort_flag)) { ok = false; break; }
          tc_fence_after();
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
        if (lane == 0) mbar_arrive_peer(p_full_even[b]);
      }
      if (!ok) break;
      if (!mbar_wait_warp(l_ready, n_item & 1u, abort_flag)) break;
      const float l = sRowSum[(n_item & 1u) * kBlockM + row_l];
      if (!mbar_wait_warp(o_full, n_item & 1u, abort_flag)) break;
      ++n_item;
      tc_fence_after();
      const float inv_l = (l > 0.f) ? 1.f / l : 0.f;
      const int row = g.r0 + row_l;
      __half* orow = p.O + (static_cast<size_t>(g.bh) * N + row) * D;
#pragma unroll
      for (int c = 0; c < D / 32; ++c) {
        uint32_t r[32];
        tmem_ld32(tO + c * 32, r);
        tmem_wait_ld();
        tmem_ld_fence(r);
        if (c == D / 32 - 1) {  // O is in registers: the next item's first P V may overwrite it
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive_peer(o_empty_even);
        }
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
  } else {
    reg_dec<Cfg::kRegMisc>();
    if (warp == 8 && rank == 0) {
      // ===================================================================================
      // tensor-core issuer of the pair (even CTA). Two cursors walk the same tile stream: the
      // score cursor runs two tiles ahead of the P V cursor, across item boundaries.
      // ===================================================================================
      constexpr uint32_t idesc_qk = umma_idesc_f16(2 * kBlockM, kBlockN, 0, 0);
      constexpr uint32_t idesc_pv = umma_idesc_f16(2 * kBlockM, D, 0, 1);
      const uint64_t kdesc0 = umma_desc_sw128(0, 16, 1024);  // K-major tiles (Q, K half)
      const uint64_t vdesc0 = umma_desc_sw128(0, 16, 1024);  // MN-major V half: one 64-wide atom along N
      const uint32_t q_addr = smem_u32(sQ);
      const uint32_t kv_addr = smem_u32(sKV);
      bool ok = true;
      FA_AP_DECL;

      auto wait_slot = [&](uint32_t it) -> bool {  // both halves of ring entry `it` have landed
        const uint32_t slot = it % Cfg::kStages, par = (it / Cfg::kStages) & 1u;
        if (!mbar_wait_warp(&kv_full[slot], par, abort_flag)) return false;
        FA_AP(it & 1u ? 4 : 1);
        const bool landed = mbar_wait_warp(&kv_peer[slot], par, abort_flag);
        FA_AP(7);
        return landed;
      };
      auto issue_scores = [&](const AheadCursor& c) -> bool {  // S(t) = Q K(t)^T for both CTAs
        const uint32_t b = c.t & 1u, ph = (c.t >> 1) & 1u, qb = c.n_item & 1u;
        if (c.j == c.g.lo) {
          const uint32_t qph = (c.n_item >> 1) & 1u;
          if (!mbar_wait_warp(&q_full[qb], qph, abort_flag)) return false;
          if (!mbar_wait_warp(&q_peer[qb], qph, abort_flag)) return false;
        }
        FA_AP(0);
        if (!wait_slot(2u * c.t)) return false;
        if (!mbar_wait_warp(&s_free[b], ph ^ 1u, abort_flag)) return false;  // S(t - 2) has been read
        tc_fence_after();
        FA_AP(2);
        const uint32_t slot = (2u * c.t) % Cfg::kStages;
        const uint64_t kdesc = kdesc0 + ((kv_addr + slot * Cfg::kSlotBytes) >> 4);
        const uint64_t qdesc = kdesc0 + ((q_addr + qb * Cfg::kQTileBytes) >> 4);
        if (elect_one()) {
#pragma unroll
          for (int k = 0; k < D / 16; ++k) {
            const uint32_t offq = ((k / 4) * (kBlockM * kPanel * 2) + (k % 4) * 32) >> 4;
            const uint32_t offk = ((k / 4) * Cfg::kKPanelBytes + (k % 4) * 32) >> 4;
            umma_ss_2cta(tmem_base + Cfg::kColS + 128u * b, qdesc + offq, kdesc + offk, idesc_qk, k > 0 ? 1u : 0u);
          }
          umma_commit_2cta(&s_full[b], 3);
          umma_commit_2cta(&kv_empty[slot], 3);
          if (c.j + 1 == c.g.hi) umma_commit_2cta(&q_empty[qb], 3);
        }
        __syncwarp();
        FA_AP(3);
        return true;
      };
      auto issue_pv = [&](const AheadCursor& c) -> bool {  // O += P(t) V(t) for both CTAs
        const uint32_t b = c.t & 1u, ph = (c.t >> 1) & 1u;
        if (!wait_slot(2u * c.t + 1u)) return false;
        if (c.j == c.g.lo) {  // the previous item's O has been read by the epilogue
          if (!mbar_wait_warp(o_empty, (c.n_item & 1u) ^ 1u, abort_flag)) return false;
        }
        if (!mbar_wait_warp(&p_full[b], ph, abort_flag)) return false;
        tc_fence_after();
        FA_AP(5);
        const uint32_t slot = (2u * c.t + 1u) % Cfg::kStages;
        const uint64_t vdesc = vdesc0 + ((kv_addr + slot * Cfg::kSlotBytes) >> 4);
        const uint32_t tP = tmem_base + Cfg::kColP + 64u * b;
        if (elect_one()) {
          umma_ts_2cta(tmem_base + Cfg::kColO, tP, vdesc, idesc_pv, (c.j > c.g.lo) ? 1u : 0u);
#pragma unroll
          for (int kk = 1; kk < 8; ++kk)
            umma_ts_2cta(tmem_base + Cfg::kColO, tP + kk * 8, vdesc + kk * (2048 >> 4), idesc_pv, 1u);
          umma_commit_2cta(&kv_empty[slot], 3);
          umma_commit_2cta(&p_free[b], 3);
          if (c.j + 1 == c.g.hi) umma_commit_2cta(o_full, 3);
        }
        __syncwarp();
        FA_AP(6);
        return true;
      };

      AheadCursor cs, cp;
      cs.start(p, rank, cluster_id, num_clusters);
      cp = cs;
      for (int i = 0; i < 2 && ok && cs.valid; ++i) {  // scores of the first two tiles
        ok = issue_scores(cs);
        cs.advance(p, rank, cluster_id, num_clusters);
      }
      while (ok && cp.valid) {
        // S(t + 2) first: it only waits for the softmax to have READ S(t), which happens early in
        // tile t, so it completes while that softmax is still running.
        if (cs.valid) {
          ok = issue_scores(cs);
          cs.advance(p, rank, cluster_id, num_clusters);
          if (!ok) break;
        }
        ok = issue_pv(cp);
        cp.advance(p, rank, cluster_id, num_clusters);
      }
      FA_AP_STORE(blockIdx.x == 0 && lane == 0, 1);
    } else if (warp == 8 && rank == 1 && lane == 0) {
      // ===================================================================================
      // odd CTA: tell the issuer when this CTA's Q tile and K/V halves have landed
      // ===================================================================================
      uint32_t it = 0, n_item = 0;
      bool ok = true;
      for (int round = 0; ok; ++round) {
        const int item = pair_item(round, cluster_id, num_clusters, p.num_items);
        if (item == -2) break;
        if (item < 0) continue;
        const AheadGeom g = decode_ahead_item(item, p, rank);
        const uint32_t qb = n_item & 1u;
        if (!mbar_wait(&q_full[qb], (n_item >> 1) & 1u, abort_flag)) break;
        ++n_item;
        mbar_arrive_peer(mapa_u32(smem_u32(&q_peer[qb]), 0));
        for (int j = g.lo; j < g.hi && ok; ++j) {
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            const uint32_t slot = it % Cfg::kStages;
            if (!mbar_wait(&kv_full[slot], (it / Cfg::kStages) & 1u, abort_flag)) { ok = false; break; }
            mbar_arrive_peer(mapa_u32(smem_u32(&kv_peer[slot]), 0));
            ++it;
          }
        }
      }
    } else if (warp == 9 && lane == 0) {
      // ===================================================================================
      // TMA producer: own Q tile, own half of every K and V tile
      // ===================================================================================
      uint32_t it = 0, n_item = 0;
      bool ok = true;
      for (int round = 0; ok; ++round) {
        const int item = pair_item(round, cluster_id, num_clusters, p.num_items);
        if (item == -2) break;
        if (item < 0) continue;
        const AheadGeom g = decode_ahead_item(item, p, rank);
        const uint32_t qb = n_item & 1u;
        if (!mbar_wait(&q_empty[qb], ((n_item >> 1) & 1u) ^ 1u, abort_flag)) break;
        ++n_item;
        mbar_arrive_expect_tx(&q_full[qb], Cfg::kQTileBytes);
        tma_load_4d(sQ + qb * Cfg::kQTileBytes, &mapQ, &q_full[qb], 0, g.r0, 0, g.bh);
        for (int j = g.lo; j < g.hi && ok; ++j) {
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            const uint32_t slot = it % Cfg::kStages;
            if (!mbar_wait(&kv_empty[slot], ((it / Cfg::kStages) & 1u) ^ 1u, abort_flag)) { ok = false; break; }
            mbar_arrive_expect_tx(&kv_full[slot], Cfg::kSlotBytes);
            if (h == 0)  // keys [64*rank, 64*rank + 64) of the K tile, all 128 head-dim columns
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
  if (warp == 8) tmem_dealloc(tmem_base, Cfg::kTmemCols);
}

}  // namespace fa
