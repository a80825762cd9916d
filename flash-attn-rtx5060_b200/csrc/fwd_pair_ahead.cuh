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
// softmax threads having READ S(t), not on P(t)V(t): the tensor pipe computes scores two to three
// tiles ahead of the P V products, and the only serial chain left is the softmax itself. Every hand-off that
// crosses the pair (P ready, S buffer free) therefore has a full softmax tile of slack.
//
// Tiles of the whole item list of a cluster are numbered t = 0, 1, ...; tile t uses score buffer and
// P buffer t & 1, alpha slot t & 3, K ring slot 2t and V ring slot 2t + 1 (mod kStages).
// Roles per CTA (512 threads): warps 0-3 and 4-7 are two softmax groups (thread = q row in both) that
// take the kv tiles alternately (group w owns the tiles with t & 1 == w), so that the TMEM loads, stores
// and waits of one tile overlap the exponentials of the next; the reference max of a row travels from
// tile to tile through shared memory, each group keeps a partial row sum, and the epilogue adds the two.
// Warps 8-11 correction + epilogue; in the even CTA warp 12 issues the score products and warp 14 the P V
// products for the pair, in the odd CTA warp 12 forwards "my half has landed"; warp 13 TMA producer.
// No multicast TMA is used. Work items are assigned statically (serpentine over the cost-ordered
// list), so the two CTAs need no run-time agreement on the next item.
#pragma once
#include "fwd_params.h"
#include "fwd_persistent.cuh"
#include "ptx.cuh"

namespace fa {

struct AheadCfg {
  static constexpr int D = 128;
  static constexpr int kThreads = 512;
  static constexpr int kQTileBytes = kBlockM * D * 2;   // 32 KiB, two 16 KiB panels
  static constexpr int kSlotBytes = 16384;              // half a K tile (64 keys x 128) or half a V tile (128 keys x 64)
  static constexpr int kKPanelBytes = 64 * kPanel * 2;  // 8 KiB: 64 keys x 128 B
  // even: a ring slot then always holds the same kind of tile (K or V), so each of the two issuing warps sees
  // every phase of the slots it waits on
  static constexpr int kStages = 8;
  static constexpr int kOffQ = 0;                                  // two Q buffers (item parity)
  static constexpr int kOffKV = 2 * kQTileBytes;
  static constexpr int kOffAlpha = kOffKV + kStages * kSlotBytes;  // float[4][128], by t & 3
  static constexpr int kOffRowMax = kOffAlpha + 4 * kBlockM * 4;   // float[2][128], by t & 1: reference max after tile t
  static constexpr int kOffRowSum = kOffRowMax + 2 * kBlockM * 4;  // float[2 item parity][2 groups][2: sum, max][128]
  static constexpr int kOffBars = kOffRowSum + 8 * kBlockM * 4;
  static constexpr int kNumBars = 40 + 3 * kStages;
  static constexpr int kOffMisc = kOffBars + kNumBars * 8;
  static constexpr int kSmemBytes = kOffMisc + 16;
  static constexpr uint32_t kTmemCols = 512;
  static constexpr uint32_t kColS = 0, kColO = 256, kColP = 384;  // S buffer b at kColS + 128 b, P buffer b at kColP + 64 b
  static constexpr float kLazyLog2 = 8.f;
  static constexpr int kRegSoftmax = 184, kRegCorr = 80, kRegMisc = 64;  // 8*32*184 + 4*32*80 + 4*32*64 = 64 Ki registers
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

// i-th item of cluster c out of G clusters: a serpentine over the cost-ordered list, so that every
// cluster gets a similar mix of long and short items. Returns -1 when the list is exhausted for
// this round, -2 when all rounds are done.
__device__ __forceinline__ int pair_item(int round, int c, int G, int num_items) {
  if (round * G >= num_items) return -2;
  const int idx = round * G + ((round & 1) ? (G - 1 - c) : c);
  return idx < num_items ? idx : -1;
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
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(512, 1)
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
  float* sRowMax = reinterpret_cast<float*>(smem + Cfg::kOffRowMax);
  float* sRowSum = reinterpret_cast<float*>(smem + Cfg::kOffRowSum);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + Cfg::kOffBars);
  uint64_t* q_full = bars;            // [2] own TMA -> issuer / relay                    (by item parity)
  uint64_t* q_empty = bars + 2;       // [2] issuer (multicast) -> own TMA               (by item parity)
  uint64_t* q_peer = bars + 4;        // [2] even CTA only: the odd CTA's Q tile has landed
  uint64_t* s_full = bars + 6;        // [2] issuer (multicast) -> own softmax            (by t & 1)
  uint64_t* s_free = bars + 8;        // [2] even CTA only: softmax warps of BOTH CTAs have read S -> issuer
  uint64_t* p_full = bars + 10;       // [2] even CTA only: softmax + correction warps of BOTH CTAs -> issuer
  uint64_t* p_free = bars + 12;       // [2] issuer (multicast): P(t) V(t) has completed -> own softmax, correction
  uint64_t* l_ready = bars + 18;      // [2] own softmax group -> own correction (once per item and group)
  uint64_t* o_full = bars + 15;       // issuer (multicast) -> own correction (once per item)
  uint64_t* o_empty = bars + 16;      // even CTA only: correction warps of BOTH CTAs have read O -> issuer
  uint64_t* m_ready = bars + 20;      // [2][4] softmax warp q of the group owning tile t -> warp q of the other group
  uint64_t* e_done = bars + 28;       // [2][4] same pairing: "my exponentials of tile t are done", the MUFU is yours
  uint64_t* alpha_ready = bars + 36;  // [4] own softmax -> own correction (by t & 3)
  uint64_t* kv_full = bars + 40;                       // [kStages] own TMA -> issuer / relay
  uint64_t* kv_empty = bars + 40 + Cfg::kStages;       // [kStages] issuer (multicast) -> own TMA
  uint64_t* kv_peer = bars + 40 + 2 * Cfg::kStages;    // [kStages] even CTA only: the odd CTA's half has landed
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + Cfg::kOffMisc);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  if (warp == 12) {
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
    }
    for (int i = 0; i < 4; ++i) mbar_init(&alpha_ready[i], 4);
    for (int i = 0; i < 8; ++i) {
      mbar_init(&m_ready[i], 1);
      mbar_init(&e_done[i], 1);
    }
    mbar_init(&l_ready[0], 4);
    mbar_init(&l_ready[1], 4);
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
  const uint32_t s_free_even[2] = {mapa_u32(smem_u32(&s_free[0]), 0), mapa_u32(smem_u32(&s_free[1]), 0)};
  const uint32_t p_full_even[2] = {mapa_u32(smem_u32(&p_full[0]), 0), mapa_u32(smem_u32(&p_full[1]), 0)};
  const uint32_t o_empty_even = mapa_u32(smem_u32(o_empty), 0);

  if (misaligned) {
    // swizzled tiles need a 1024-byte aligned base; nothing was issued, fall through to the common exit
  } else if (warp < 8) {
    // =====================================================================================
    // softmax: group w = warp / 4 owns the kv tiles with t & 1 == w; thread = q row
    // =====================================================================================
    reg_inc<Cfg::kRegSoftmax>();
    const uint32_t w = static_cast<uint32_t>(warp >> 2);
    const int row_l = tid & 127;
    const uint32_t lane_base = static_cast<uint32_t>(warp & 3) * 32u;
    const uint32_t tS = tmem_addr(tmem_base, lane_base, Cfg::kColS + 128u * w);
    const uint32_t tP = tmem_addr(tmem_base, lane_base, Cfg::kColP + 64u * w);
    uint64_t* m_mine = &m_ready[w * 4 + (warp & 3)];          // I publish the reference max of my tiles here
    uint64_t* m_other = &m_ready[(w ^ 1u) * 4 + (warp & 3)];  // the other group's warp of the same rows
    uint64_t* e_mine = &e_done[w * 4 + (warp & 3)];
    uint64_t* e_other = &e_done[(w ^ 1u) * 4 + (warp & 3)];
    const float sl2 = kAlibi ? 1.f : p.scale_log2;
    const uint64_t scale2 = f2_pack(sl2, sl2);
    uint32_t t = 0, n_item = 0;
    bool ok = true;
    for (int round = 0; ok; ++round) {
      const int item = pair_item(round, cluster_id, num_clusters, p.num_items);
      if (item == -2) break;
      if (item < 0) continue;
      const AheadGeom g = decode_ahead_item(item, p, rank);
      const int row = g.r0 + row_l;
      float slope_l2 = 0.f;
      if (kAlibi) slope_l2 = p.alibi_slopes[g.bh % p.heads] * 1.4426950408889634f;
      // This group's share of the row: sum of exponentials taken against m_known, over its own tiles.
      float m_known = 0.f;
      float l_part = 0.f;
      for (int j = g.lo; j < g.hi; ++j, ++t) {
        if ((t & 1u) != w) continue;
        const uint32_t ph = (t >> 1) & 1u;
        if (!mbar_wait_warp(&s_full[w], ph, abort_flag)) { ok = false; break; }
        tc_fence_after();
#ifdef FA_AHEAD_FAKE  // bring-up only: the load + tensor pipeline of the pair without the softmax work
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive_peer(s_free_even[w]);
        if (t > 0 && !mbar_wait_warp(m_other, ((t - 1u) >> 1) & 1u, abort_flag)) { ok = false; break; }
        __syncwarp();
        if (lane == 0) mbar_arrive(m_mine);
        if (t > 0 && !mbar_wait_warp(e_other, ((t - 1u) >> 1) & 1u, abort_flag)) { ok = false; break; }
        if (lane == 0) mbar_arrive(e_mine);
        if (!mbar_wait_warp(&p_free[w], ph ^ 1u, abort_flag)) { ok = false; break; }
        sAlpha[(t & 3u) * kBlockM + row_l] = 1.f;
        __syncwarp();
        if (lane == 0) { mbar_arrive(&alpha_ready[t & 3u]); mbar_arrive_peer(p_full_even[w]); }
        l_part = 0.5f;
        continue;
#endif
        const int kv0 = j * kBlockN;
        const bool first = (j == g.lo);
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
          if (lane == 0) mbar_arrive_peer(s_free_even[w]);
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
          float mx0 = -INFINITY, mx1 = -INFINITY, mx2 = -INFINITY, mx3 = -INFINITY;
#pragma unroll
          for (int c = 0; c < kBlockN; c += 8) {
            mx0 = max3(mx0, sc[c], sc[c + 1]);
            mx1 = max3(mx1, sc[c + 2], sc[c + 3]);
            mx2 = max3(mx2, sc[c + 4], sc[c + 5]);
            mx3 = max3(mx3, sc[c + 6], sc[c + 7]);
          }
          const float m_tile = max3(mx0, mx1, fmaxf(mx2, mx3));
          // Reference max after the previous tile, from the group that owns it. Every publication is waited
          // for, also across item boundaries (where its value is not used), so the two groups take strict
          // turns on these barriers. NaN marks "no finite score seen in this row so far".
          float m_prev = __int_as_float(0x7fc00000);
          if (t > 0) {
            if (!mbar_wait_warp(m_other, ((t - 1u) >> 1) & 1u, abort_flag)) return false;
            if (!first) m_prev = sRowMax[(w ^ 1u) * kBlockM + row_l];
          }
          // Lazy rescale: the reference max moves only when this tile's max exceeds it by more than kLazyLog2
          // (P then stays below 2^8, well inside fp16), or when the row had no finite score before.
          const bool fresh = !(m_prev == m_prev);
          const bool move = fresh ? (m_tile != -INFINITY) : ((m_tile - m_prev) * sl2 > Cfg::kLazyLog2);
          const float m_ref = move ? m_tile : m_prev;  // stays NaN while the row is still empty
          sRowMax[w * kBlockM + row_l] = m_ref;
          __syncwarp();
          if (lane == 0) mbar_arrive(m_mine);
          const bool empty = !(m_ref == m_ref);
          const float m_use = empty ? 0.f : m_ref;     // exponentials of an empty row: exp2(-inf - 0) = 0
          float alpha = (fresh || empty) ? 1.f : ex2_approx((m_prev - m_ref) * sl2);
          // my partial sum moves from the reference I last used to the current one
          const float shift = (l_part > 0.f) ? ex2_approx((m_known - m_use) * sl2) : 0.f;
          m_known = m_use;
          // The alpha slot is reused every fourth tile: the correction warps read alpha(t - 4) before P(t - 4) V(t - 4)
          // started, and this group waited for that product to complete during its previous tile.
          sAlpha[(t & 3u) * kBlockM + row_l] = alpha;
          __syncwarp();
          if (lane == 0) mbar_arrive(&alpha_ready[t & 3u]);
          // The two warps that share an SM sub-partition (same rows, one per group) take turns on its MUFU:
          // without this the groups settle into running their exponentials at the same time at half rate
          // each, and their loads, maxima and waits at the same time too, so nothing overlaps.
          if (t > 0 && !mbar_wait_warp(e_other, ((t - 1u) >> 1) & 1u, abort_flag)) return false;
          // P(t - 2) V(t - 2) has completed: its P buffer may be overwritten.
          if (!mbar_wait_warp(&p_free[w], ph ^ 1u, abort_flag)) return false;
          const float neg_ms = -m_use * sl2;
          const uint64_t negms2 = f2_pack(neg_ms, neg_ms);
          uint64_t lsum_a = 0ull, lsum_b = 0ull;
          uint32_t pk0[32], pk1[32];
          // masked tiles hold -inf scores, which only the MUFU path maps to 0
          exp_half_tile(sc, scale2, negms2, pk0, lsum_a, lsum_b);
          tmem_st32(tP + 0, pk0);
          exp_half_tile(sc + 64, scale2, negms2, pk1, lsum_a, lsum_b);
          __syncwarp();
          if (lane == 0) mbar_arrive(e_mine);
          float l0, l1;
          f2_unpack(f2_add(lsum_a, lsum_b), l0, l1);
          l_part = l_part * shift + (l0 + l1);
          tmem_st32(tP + 32, pk1);
          tmem_wait_st();
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive_peer(p_full_even[w]);  // the whole P tile is in TMEM
          return true;
        };
        if (kv_tile_needs_mask(kv0, g.r0, g.r1, wl, wr, N)) ok = tile_body(std::true_type{});
        else ok = tile_body(std::false_type{});
        if (!ok) break;
      }
      if (!ok) break;
      float* part = sRowSum + ((n_item & 1u) * 2u + w) * 2u * kBlockM;
      part[row_l] = l_part;
      part[kBlockM + row_l] = m_known;
      __syncwarp();
      if (lane == 0) mbar_arrive(&l_ready[w]);
      ++n_item;
    }
  } else if (warp < 12) {
    // =====================================================================================
    // correction + epilogue for this CTA's rows
    // =====================================================================================
    reg_dec<Cfg::kRegCorr>();
    const int row_l = tid & 127;
    const uint32_t lane_base = static_cast<uint32_t>(warp & 3) * 32u;
    const uint32_t tO = tmem_addr(tmem_base, lane_base, Cfg::kColO);
    const float sl2 = kAlibi ? 1.f : p.scale_log2;
    uint32_t t = 0, n_item = 0;
    bool ok = true;
    for (int round = 0; ok; ++round) {
      const int item = pair_item(round, cluster_id, num_clusters, p.num_items);
      if (item == -2) break;
      if (item < 0) continue;
      const AheadGeom g = decode_ahead_item(item, p, rank);
      for (int j = g.lo; j < g.hi && ok; ++j, ++t) {
        const uint32_t b = t & 1u;
        if (!mbar_wait_warp(&alpha_ready[t & 3u], (t >> 2) & 1u, abort_flag)) { ok = false; break; }
        const float alpha = sAlpha[(t & 3u) * kBlockM + row_l];
        // O may be rescaled only between P(t-1) V(t-1) and P(t) V(t): wait for the former to complete. The wait is
        // taken for every tile, needed or not, so that every phase of these barriers is observed in turn.
        if (t > 0 && !mbar_wait_warp(&p_free[b ^ 1u], ((t - 1u) >> 1) & 1u, abort_flag)) { ok = false; break; }
        if (j > g.lo && __any_sync(0xffffffffu, alpha != 1.f)) {
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
      if (!mbar_wait_warp(&l_ready[0], n_item & 1u, abort_flag)) break;
      if (!mbar_wait_warp(&l_ready[1], n_item & 1u, abort_flag)) break;
      // Row sum = the two groups' partial sums brought to the reference O was accumulated against, which is
      // the one the owner of the last tile ended with.
      const uint32_t own = (t - 1u) & 1u;
      const float* part_own = sRowSum + ((n_item & 1u) * 2u + own) * 2u * kBlockM;
      const float* part_oth = sRowSum + ((n_item & 1u) * 2u + (own ^ 1u)) * 2u * kBlockM;
      const float l_oth = part_oth[row_l];
      float l = part_own[row_l];
      if (l_oth > 0.f) l += l_oth * ex2_approx((part_oth[kBlockM + row_l] - part_own[kBlockM + row_l]) * sl2);
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
    if ((warp == 12 || warp == 14) && rank == 0) {
      // ===================================================================================
      // tensor-core issuers of the pair (even CTA)
      // ===================================================================================
      constexpr uint32_t idesc_qk = umma_idesc_f16(2 * kBlockM, kBlockN, 0, 0);
      constexpr uint32_t idesc_pv = umma_idesc_f16(2 * kBlockM, D, 0, 1);
      const uint64_t kdesc0 = umma_desc_sw128(0, 16, 1024);  // K-major tiles (Q, K half)
      const uint64_t vdesc0 = umma_desc_sw128(0, 16, 1024);  // MN-major V half: one 64-wide atom along N
      const uint32_t q_addr = smem_u32(sQ);
      const uint32_t kv_addr = smem_u32(sKV);
      bool ok = true;

      auto wait_slot = [&](uint32_t it) -> bool {  // both halves of ring entry `it` have landed
        const uint32_t slot = it % Cfg::kStages, par = (it / Cfg::kStages) & 1u;
        if (!mbar_wait_warp(&kv_full[slot], par, abort_flag)) return false;
        const bool landed = mbar_wait_warp(&kv_peer[slot], par, abort_flag);
        return landed;
      };
      auto issue_scores = [&](const AheadCursor& c) -> bool {  // S(t) = Q K(t)^T for both CTAs
        const uint32_t b = c.t & 1u, ph = (c.t >> 1) & 1u, qb = c.n_item & 1u;
        if (c.j == c.g.lo) {
          const uint32_t qph = (c.n_item >> 1) & 1u;
          if (!mbar_wait_warp(&q_full[qb], qph, abort_flag)) return false;
          if (!mbar_wait_warp(&q_peer[qb], qph, abort_flag)) return false;
        }
        if (!wait_slot(2u * c.t)) return false;
        if (!mbar_wait_warp(&s_free[b], ph ^ 1u, abort_flag)) return false;  // S(t - 2) has been read
        tc_fence_after();
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
        return true;
      };

      // Two issuing warps, one per kind of product: S(t) = Q K(t)^T needs "K(t) has landed" and "S(t - 2) has been
      // read", P(t) V(t) needs "V(t) has landed" and "P(t) is ready". The two chains share nothing but the tensor
      // pipe, so neither ever waits behind an instruction of the other that is not ready yet.
      AheadCursor c;
      c.start(p, rank, cluster_id, num_clusters);
      if (warp == 12) {
        while (ok && c.valid) {
          ok = issue_scores(c);
          c.advance(p, rank, cluster_id, num_clusters);
        }
      } else {
        while (ok && c.valid) {
          ok = issue_pv(c);
          c.advance(p, rank, cluster_id, num_clusters);
        }
      }
    } else if (warp == 12 && rank == 1 && lane == 0) {
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
    } else if (warp == 13 && lane == 0) {
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
  if (warp == 12) tmem_dealloc(tmem_base, Cfg::kTmemCols);
}

}  // namespace fa
