// Warp-specialised persistent attention-forward kernel for sm_100a.
//
// One CTA per SM walks a list of work items; a work item is a pair of adjacent 128-row q tiles
// of one (batch, head). Roles (16 warps):
//   warps 0-3   softmax of q tile 0: one thread per score row (TMEM lane), exp2 online softmax
//   warps 4-7   softmax of q tile 1
//   warps 8-11  correction: rescales the running output in TMEM when a row max moved, and the
//               epilogue (O / l -> fp16 -> the warp's staging area in shared memory -> one TMA store)
//   warp 12     tensor-core issuer: the warp walks the schedule, one elected lane issues tcgen05.mma
//   warp 13     TMA producer: Q tiles and the K/V tile ring
//   warps 14-15 idle (they only donate registers)
// TMEM columns: S0 [0,128) S1 [128,256) O0 [256,256+D) O1 [384,384+D); the fp16 P tile of a
// stage overwrites the first 64 columns of its own S and is handed to the tensor pipe in two
// halves of 64 keys, so that P.V starts while the second half is still being exponentiated.
//
// Replaces the reference's forward_kernel, Schedule and SMem (src/flash_forward.h:22-366),
// apply_mask (src/mask.h:10-84) and apply_softmax (src/softmax.h:9-86): same function, but
// the contractions run on tcgen05 with TMEM accumulators, the two q tiles ping-pong so that
// the tensor pipe works on one while the other is in softmax, masks touch only boundary
// tiles, kv tiles outside a q tile's visible range are never loaded for it, and the output
// is rescaled lazily.
#pragma once
#include <type_traits>

#include "fwd_params.h"
#include "ptx.cuh"

// Registers per thread after setmaxnreg: 8 softmax warps, 4 correction warps, 4 others; the three
// numbers must satisfy 256 * softmax + 128 * correction + 128 * others <= 65536.
#ifndef FA_REG_SOFTMAX
#define FA_REG_SOFTMAX 184
#define FA_REG_CORR 72
#define FA_REG_MISC 72
#endif



namespace fa {

template <int D>
struct PersistentCfg {
  static constexpr int kThreads = 512;
  static constexpr int kTileBytes = kBlockN * D * 2;
  static constexpr int kPanelBytes = kBlockN * kPanel * 2;
  static constexpr int kStages = (D == 128) ? 4 : 8;  // ring slots, each one K or one V tile
  static constexpr int kOffQ = 0;
  static constexpr int kOffKV = 2 * kTileBytes;
  // Output staging: each correction warp owns 32 rows, laid out [panel][row][64] with the 128-byte swizzle, the
  // source of its TMA store.
  static constexpr int kOffOut = kOffKV + kStages * kTileBytes;
  static constexpr int kOutWarpBytes = 32 * D * 2;
  static constexpr int kOffAlpha = kOffOut + 4 * kOutWarpBytes;  // float[2][128]
  static constexpr int kOffRowSum = kOffAlpha + 2 * kBlockM * 4;   // float[2][128]
  static constexpr int kOffBars = kOffRowSum + 2 * kBlockM * 4;
  static constexpr int kNumBars = 20 + 2 * kStages;
  static constexpr int kOffMisc = kOffBars + kNumBars * 8;
  static constexpr int kOffGeom = kOffMisc + 16;     // TMEM base, abort flag (+ 8 spare bytes)
  static constexpr int kSmemBytes = kOffGeom + 2 * 64;  // two work-item slots: the item's decoded geometry and its id
  static constexpr uint32_t kTmemCols = 512;
  static constexpr uint32_t kColS0 = 0, kColS1 = 128, kColO0 = 256, kColO1 = 384;
  // softmax threshold (in log2 units) below which a larger row max does not trigger a rescale
  static constexpr float kLazyLog2 = 8.f;
};

// Work item -> geometry. Every role decodes the same item the same way.
struct ItemGeom {
  int bh, pair;
  int r0[2], r1[2];  // first / last q row of each stage's tile (r1 < r0: stage has no rows)
  int lo[2], hi[2];  // visible kv-tile range of each stage, [lo, hi); empty when no rows
  int lo_all, hi_all;
};

// Work-item order. Heads are taken in groups of `head_group` (sized on the host so that the K/V of
// a group stays in L2); inside a group the items run pair-major from the last (under a causal mask
// the longest) q pair to the first. CTAs claim items in this order from a global counter, so CTAs
// that run together read the same few heads, and the items handed out last are the cheapest ones
// of the last group: the tail stays short.
template <int BN = kBlockN>
__device__ __forceinline__ ItemGeom decode_item(int item, const FwdParams& p) {
  ItemGeom g;
  const int per_group = p.head_group * p.num_q_pairs;
  const int grp = item / per_group;
  const int r = item - grp * per_group;
  const int heads_here = min(p.head_group, p.bh - grp * p.head_group);
  const int pr = r / heads_here;
  g.bh = grp * p.head_group + (r - pr * heads_here);
  g.pair = p.num_q_pairs - 1 - pr;
  const int wr = eff_window_right(p.causal, p.window_right);
  g.lo_all = 0x7fffffff;
  g.hi_all = 0;
#pragma unroll
  for (int s = 0; s < 2; ++s) {
    g.r0[s] = g.pair * 2 * kBlockM + s * kBlockM;
    if (g.r0[s] >= p.seqlen) {
      g.r1[s] = g.r0[s] - 1;
      g.lo[s] = g.hi[s] = 0;
    } else {
      g.r1[s] = min(g.r0[s] + kBlockM, p.seqlen) - 1;
      g.lo[s] = kv_tile_begin(g.r0[s], p.window_left, BN);
      g.hi[s] = kv_tile_end(g.r1[s], wr, p.seqlen, BN);
      g.lo_all = min(g.lo_all, g.lo[s]);
      g.hi_all = max(g.hi_all, g.hi[s]);
    }
  }
  return g;
}

// exp2 of 64 scores (32 pairs) -> 32 packed fp16x2 words; adds the exponentials into two
// (even, odd) pairs of partial row sums.
__device__ __forceinline__ void exp_half_tile(const float* sc, uint64_t scale2, uint64_t negms2, uint32_t (&pk)[32],
                                              uint64_t& lsum_a, uint64_t& lsum_b) {
#pragma unroll
  for (int c = 0; c < 32; ++c) {
    float x0, x1, e0, e1;
    f2_unpack(f2_fma(f2_pack(sc[2 * c], sc[2 * c + 1]), scale2, negms2), x0, x1);
    e0 = ex2_approx(x0);
    e1 = ex2_approx(x1);
    if (c & 1) lsum_b = f2_add(lsum_b, f2_pack(e0, e1));
    else lsum_a = f2_add(lsum_a, f2_pack(e0, e1));
    pk[c] = pack_f16x2(e0, e1);
  }
}

// Same for 32 scores (16 pairs) -> the first 16 words of pk.
__device__ __forceinline__ void exp_quarter_tile(const float* sc, uint64_t scale2, uint64_t negms2, uint32_t* pk,
                                                 uint64_t& lsum_a, uint64_t& lsum_b) {
#pragma unroll
  for (int c = 0; c < 16; ++c) {
    float x0, x1, e0, e1;
    f2_unpack(f2_fma(f2_pack(sc[2 * c], sc[2 * c + 1]), scale2, negms2), x0, x1);
    e0 = ex2_approx(x0);
    e1 = ex2_approx(x1);
    if (c & 1) lsum_b = f2_add(lsum_b, f2_pack(e0, e1));
    else lsum_a = f2_add(lsum_a, f2_pack(e0, e1));
    pk[c] = pack_f16x2(e0, e1);
  }
}

// Philox-4x32 with 10 rounds (Salmon et al., "Parallel random numbers: as easy as 1, 2, 3"): a keyed bijection of a
// 128-bit counter. Stateless, so the keep mask of dropout depends only on (seed, head, row, column) and is the same
// whatever tile shape or schedule computes it. (The reference keeps ONE generator state per q tile, copies it into
// every thread of the CTA, so all threads draw the same numbers, and stores it back: src/flash_forward.h:185-186,
// :248-265, :361-363. That flaw is not reproduced.)
__device__ __forceinline__ void philox4x32_10(uint32_t k0, uint32_t k1, uint32_t c0, uint32_t c1, uint32_t c2,
                                              uint32_t c3, uint32_t (&out)[4]) {
#pragma unroll
  for (int r = 0; r < 10; ++r) {
    const uint32_t hi0 = __umulhi(0xD2511F53u, c0), lo0 = 0xD2511F53u * c0;
    const uint32_t hi1 = __umulhi(0xCD9E8D57u, c2), lo1 = 0xCD9E8D57u * c2;
    c0 = hi1 ^ c1 ^ k0;
    c1 = lo1;
    c2 = hi0 ^ c3 ^ k1;
    c3 = lo0;
    k0 += 0x9E3779B9u;
    k1 += 0xBB67AE85u;
  }
  out[0] = c0; out[1] = c1; out[2] = c2; out[3] = c3;
}

// Zeroes the dropped elements of 32 packed fp16 pairs (64 consecutive columns starting at global column `col0`, a
// multiple of 16) of query row `row` of head `bh`. One Philox call serves 16 columns: byte t of its 16 output bytes
// (little endian over the four words) decides column 16 * block + t.
__device__ __forceinline__ void dropout_mask_64(uint32_t (&pk)[32], const FwdParams& p, int bh, int row, int col0) {
  const uint32_t thr4 = p.drop_keep_thr * 0x01010101u;
#pragma unroll
  for (int blk = 0; blk < 4; ++blk) {
    uint32_t r[4];
    philox4x32_10(p.seed_lo, p.seed_hi, static_cast<uint32_t>(col0 / 16 + blk), static_cast<uint32_t>(row),
                  static_cast<uint32_t>(bh), 0u, r);
#pragma unroll
    for (int w = 0; w < 4; ++w) {
      const uint32_t keep = __vcmpltu4(r[w], thr4);                // 0xff in every byte below the threshold
      pk[blk * 8 + 2 * w] &= __byte_perm(keep, 0u, 0x1100);        // columns 4w, 4w+1
      pk[blk * 8 + 2 * w + 1] &= __byte_perm(keep, 0u, 0x3322);    // columns 4w+2, 4w+3
    }
  }
}

template <int D, bool kAlibi, bool kLse = false, bool kDropout = false>
__global__ void __launch_bounds__(512, 1)
fwd_persistent_kernel(const __grid_constant__ CUtensorMap mapQ, const __grid_constant__ CUtensorMap mapK,
                      const __grid_constant__ CUtensorMap mapV, const __grid_constant__ CUtensorMap mapO,
                      const FwdParams p) {
  using Cfg = PersistentCfg<D>;
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
  uint64_t* q_full = bars;            // [2] TMA -> MMA
  uint64_t* q_empty = bars + 2;       // [2] MMA -> TMA
  uint64_t* s_full = bars + 4;        // [2] MMA -> softmax: S tile in TMEM
  uint64_t* p_full = bars + 6;        // [2] softmax (first half of P) + correction (O rescaled) -> MMA
  uint64_t* alpha_ready = bars + 8;   // [2] softmax -> correction: rescale factors in smem
  uint64_t* l_ready = bars + 10;      // [2] softmax -> correction: final row sums in smem
  uint64_t* o_full = bars + 12;       // [2] MMA -> correction: last P.V of the item landed
  uint64_t* p_full2 = bars + 14;      // [2] softmax -> MMA: second half of P written
  uint64_t* item_full = bars + 16;    // [2] producer -> all roles: next work item id published
  uint64_t* item_empty = bars + 18;   // [2] all roles -> producer: id slot read
  uint64_t* kv_full = bars + 20;      // [kStages] TMA -> MMA
  uint64_t* kv_empty = bars + 20 + Cfg::kStages;  // [kStages] MMA -> TMA
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + Cfg::kOffMisc);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  // [2][16]: ItemGeom of the published item in words 0..11, its id (-1: no more items) in word 12
  volatile int* s_geom = reinterpret_cast<volatile int*>(smem + Cfg::kOffGeom);
  constexpr uint32_t kItemReaders = 13;  // 8 softmax warps + 4 correction warps + the MMA warp

  if (warp == 12) {
    tmem_alloc(tmem_slot, Cfg::kTmemCols);
    tmem_relinquish();
  }
  if (tid == 0) {
#pragma unroll
    for (int s = 0; s < 2; ++s) {
      mbar_init(&q_full[s], 1);
      mbar_init(&q_empty[s], 1);
      mbar_init(&s_full[s], 1);
      mbar_init(&p_full[s], 8);  // one arrival per softmax warp and per correction warp
      mbar_init(&p_full2[s], 4);
      mbar_init(&alpha_ready[s], 4);
      mbar_init(&l_ready[s], 4);
      mbar_init(&o_full[s], 1);
      mbar_init(&item_full[s], 1);
      mbar_init(&item_empty[s], kItemReaders);
    }
    for (int i = 0; i < Cfg::kStages; ++i) {
      mbar_init(&kv_full[i], 1);
      mbar_init(&kv_empty[i], 1);
    }
    *abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == 13 && lane == 0) {
    prefetch_tensormap(&mapQ);
    prefetch_tensormap(&mapK);
    prefetch_tensormap(&mapV);
    prefetch_tensormap(&mapO);
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  const int N = p.seqlen;
  const int wl = p.window_left;
  const int wr = eff_window_right(p.causal, p.window_right);

  // Every consuming warp reads the k-th work item (id and geometry, decoded once by the producer) from slot
  // k & 1 once the producer has published it, and releases the slot. -1 ends the walk (also after a give-up).
  auto take_item = [&](uint32_t& n_items, ItemGeom& g) -> int {
    const uint32_t slot = n_items & 1u;
    if (!mbar_wait_warp(&item_full[slot], (n_items >> 1) & 1u, abort_flag)) return -1;
    const volatile int* w = s_geom + slot * 16;
    const int it = w[12];
    g.bh = w[0]; g.pair = w[1];
    g.r0[0] = w[2]; g.r0[1] = w[3]; g.r1[0] = w[4]; g.r1[1] = w[5];
    g.lo[0] = w[6]; g.lo[1] = w[7]; g.hi[0] = w[8]; g.hi[1] = w[9];
    g.lo_all = w[10]; g.hi_all = w[11];
    __syncwarp();
    if (lane == 0) mbar_arrive(&item_empty[slot]);
    ++n_items;
    return it;
  };

  if (warp < 8) {
    // =====================================================================================
    // softmax: stage s = warp / 4, row = tid % 128
    // =====================================================================================
    reg_inc<FA_REG_SOFTMAX>();
    const int s = warp >> 2;
    const int row_l = tid & 127;
    const uint32_t lane_base = static_cast<uint32_t>(warp & 3) * 32u;
    const uint32_t tS = tmem_addr(tmem_base, lane_base, s == 0 ? Cfg::kColS0 : Cfg::kColS1);
    // With ALiBi the scores are moved to the biased log2 domain right after the TMEM load, and
    // everything downstream works with a unit scale.
    const float sl2 = kAlibi ? 1.f : p.scale_log2;
    const uint64_t scale2 = f2_pack(sl2, sl2);
    uint32_t n_s = 0;  // completed s_full phases
    uint32_t n_items = 0;
    bool ok = true;
    while (ok) {
      ItemGeom g;
      const int item = take_item(n_items, g);
      if (item < 0) break;
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
        if (!mbar_wait_warp(&s_full[s], n_s & 1, abort_flag)) { ok = false; break; }
        ++n_s;
        tc_fence_after();
        const int kv0 = j * kBlockN;
        // One body, instantiated twice: tiles cut by a mask boundary (or by the end of the sequence) take the
        // per-element predicate, all others carry none of that code. (Blanking a cut tile in tensor memory first
        // and sharing one body saved 10 KB of instructions but made every tile 4 % slower: the body then
        // starts behind a merge point instead of directly behind the wait.)
        auto tile_body = [&](auto masked_tag) {
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
            // Visible columns of this row: c_lo <= c <= c_hi, i.e. |c - mid| <= half. The predicate is applied on the
            // FMA pipe, which the softmax leaves nearly idle, instead of as two integer compares and a select per
            // element: t = saturate(|c - mid| - half) is 0 for a visible column and 1 for a hidden one (both
            // operands are multiples of 1/2, so the difference is exact), and sc - kHidden * t leaves a visible
            // score bit for bit as it is and puts a hidden one near -3e38, where its exponential is 0 for any scale the
            // host accepts.
            const int c_lo = (wl >= 0) ? row - wl - kv0 : -(1 << 20);
            int c_hi = N - 1 - kv0;
            if (wr >= 0) c_hi = min(c_hi, row + wr - kv0);
            const float mid = 0.5f * static_cast<float>(c_lo + c_hi);
            const float half = 0.5f * static_cast<float>(c_hi - c_lo);  // negative: no visible column at all
            constexpr float kHidden = 3.0e38f;
  #pragma unroll
            for (int c = 0; c < kBlockN; ++c) {
              const float t = __saturatef(fabsf(static_cast<float>(c) - mid) - half);
              sc[c] = fmaf(t, -kHidden, sc[c]);
            }
          }
          // The exponentials of the first 32 keys are taken against the reference the previous tile left while
          // the row max of this tile is still being reduced: nearly always the reference stays where it is (lazy
          // rescale), so the max leaves the critical path. When a row of the warp does move its reference
          // (always on the first tile of an item), the 32 exponentials are taken again.
          uint64_t lsum_a = 0ull, lsum_b = 0ull;
          uint32_t pk0[32], pk1[32];
          {
            const float neg_ms0 = -m_used * sl2;
            exp_quarter_tile(sc, scale2, f2_pack(neg_ms0, neg_ms0), pk0, lsum_a, lsum_b);
          }
          float mx0 = m_run, mx1 = -INFINITY, mx2 = -INFINITY, mx3 = -INFINITY;
  #pragma unroll
          for (int c = 0; c < kBlockN; c += 8) {
            mx0 = max3(mx0, sc[c], sc[c + 1]);
            mx1 = max3(mx1, sc[c + 2], sc[c + 3]);
            mx2 = max3(mx2, sc[c + 4], sc[c + 5]);
            mx3 = max3(mx3, sc[c + 6], sc[c + 7]);
          }
          float m_new = max3(mx0, mx1, fmaxf(mx2, mx3));
          if (kMasked && m_new < -1.0e37f) m_new = -INFINITY;  // nothing visible so far (hidden scores sit near -3e38)
          // The reference moves when the true max has grown past it by more than kLazyLog2 (P then stays below
          // 2^8, well inside fp16), and always on the first tile that shows a finite score: the reference then IS
          // the row max, so the largest term of the row is exactly 1 in fp16 (a row with a single visible key
          // returns that key's V bit for bit).
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
            exp_quarter_tile(sc, scale2, f2_pack(neg_ms1, neg_ms1), pk0, lsum_a, lsum_b);
          }
          // (no hand-over on the first tile of an item: there is nothing to rescale yet, and the correction warps
          // may still be in the previous item's epilogue)
          sAlpha[s * kBlockM + row_l] = alpha;
          __syncwarp();
          if (lane == 0 && j != j_lo) mbar_arrive(&alpha_ready[s]);
          const float neg_ms = -m_used * sl2;
          const uint64_t negms2 = f2_pack(neg_ms, neg_ms);
          exp_quarter_tile(sc + 32, scale2, negms2, pk0 + 16, lsum_a, lsum_b);
          if (kDropout) dropout_mask_64(pk0, p, g.bh, row, kv0);  // the row sum keeps every exponential
          tmem_st32(tS + 0, pk0);
          tmem_wait_st();
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(&p_full[s]);  // P of keys 0..63 is in TMEM
          exp_half_tile(sc + 64, scale2, negms2, pk1, lsum_a, lsum_b);
          if (kDropout) dropout_mask_64(pk1, p, g.bh, row, kv0 + 64);
          tmem_st32(tS + 32, pk1);
          float l0, l1;
          f2_unpack(f2_add(lsum_a, lsum_b), l0, l1);
          l_run = l_run * alpha + (l0 + l1);
          tmem_wait_st();
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(&p_full2[s]);  // P of keys 64..127
        };
        if (kv_tile_needs_mask(kv0, q_r0, q_r1, wl, wr, N)) tile_body(std::true_type{});
        else tile_body(std::false_type{});
      }
      if (!ok) break;
      // The row sums of the previous item may still be unread when this item is a single tile. The last tile's
      // p_full phase completes only after the correction warps have arrived on it, and on an item's first tile
      // they do that after their epilogue of the previous item, which reads the sums first.
      if (!mbar_wait_warp(&p_full[s], (n_s - 1) & 1, abort_flag)) break;
      sRowSum[s * kBlockM + row_l] = l_run;
      __syncwarp();
      if (lane == 0) mbar_arrive(&l_ready[s]);
      // l_run = sum over visible keys of 2^((score - m_used) * sl2), so the natural-log sum of exponentials is
      // ln2 * (m_used * sl2 + log2(l_run)).
      if (kLse && row < N)
        p.lse[static_cast<size_t>(g.bh) * N + row] =
            (l_run > 0.f) ? 0.6931471805599453f * fmaf(m_used, sl2, __log2f(l_run)) : -INFINITY;
    }
  } else if (warp < 12) {
    // =====================================================================================
    // correction + epilogue: row = tid % 128 of both stages
    // =====================================================================================
    reg_dec<FA_REG_CORR>();
    const int row_l = tid & 127;
    const uint32_t lane_base = static_cast<uint32_t>(warp & 3) * 32u;
    uint8_t* out_stage = smem + Cfg::kOffOut + (warp & 3) * Cfg::kOutWarpBytes;
    uint32_t n_alpha[2] = {0, 0}, n_l[2] = {0, 0}, n_o[2] = {0, 0};
    uint32_t n_items = 0;
    // The first P.V product of an item overwrites O, so it has to wait until the epilogue of the previous item
    // has read O. That hand-off is the correction warps' arrival on p_full for the item's first tile; it is made
    // right after the epilogue (there is nothing to rescale on a first tile), so the next item's first product
    // does not wait for these warps to come round to it.
    bool arrived_early[2] = {false, false};
    bool ok = true;
    while (ok) {
      ItemGeom g;
      const int item = take_item(n_items, g);
      if (item < 0) break;
      bool epi_pending[2] = {g.r1[0] >= g.r0[0], g.r1[1] >= g.r0[1]};
      // O / l -> fp16 -> global for stage s, then the early arrival for the next item's first tile
      auto epilogue = [&](auto stage_tag) {
        constexpr int s = decltype(stage_tag)::value;
        epi_pending[s] = false;
        if (!mbar_wait_warp(&l_ready[s], n_l[s] & 1, abort_flag)) { ok = false; return; }
        ++n_l[s];
        const float l = sRowSum[s * kBlockM + row_l];
        if (!mbar_wait_warp(&o_full[s], n_o[s] & 1, abort_flag)) { ok = false; return; }
        ++n_o[s];
        tc_fence_after();
        const float inv_l = ((l > 0.f) ? 1.f / l : 0.f) * (kDropout ? p.drop_scale : 1.f);
        const uint32_t tO = tmem_addr(tmem_base, lane_base, s == 0 ? Cfg::kColO0 : Cfg::kColO1);
        // The rows go to the warp's staging area and from there to global memory as one TMA store: issued as plain
        // stores (each lane its own row, 16 bytes at a time) they kept the load/store unit busy for about 2000
        // clocks per tile, and the barrier traffic of every other warp of the SM queued behind them.
        if (lane == 0) tma_store_wait_read();  // the previous store of this warp has read the staging area
        __syncwarp();
        // 16 columns at a time, the load of the next chunk in flight while this one is converted and stored.
        // (Rolled up: this path runs once per item and stage, and instructions that are rarely executed are
        // fetched slowly; unrolling it eightfold made the change-over between items slower, not faster.)
        uint32_t ra[16], rb[16];
        tmem_ld16(tO, ra);
  #pragma unroll 2
        for (int c = 0; c < D / 16; ++c) {
          uint32_t (&cur)[16] = (c & 1) ? rb : ra;
          uint32_t (&nxt)[16] = (c & 1) ? ra : rb;
          tmem_wait_ld();
          tmem_ld_fence16(cur);
          if (c + 1 < D / 16) tmem_ld16(tO + (c + 1) * 16, nxt);
          // columns 16c .. 16c+15 are 16-byte units 2(c%4), 2(c%4)+1 of panel c/4; unit u of row r sits at u ^ (r%8)
          uint8_t* prow = out_stage + (c >> 2) * (32 * 128) + lane * 128;
  #pragma unroll
          for (int i = 0; i < 2; ++i) {
            uint4 v;
            v.x = pack_f16x2(__uint_as_float(cur[i * 8 + 0]) * inv_l, __uint_as_float(cur[i * 8 + 1]) * inv_l);
            v.y = pack_f16x2(__uint_as_float(cur[i * 8 + 2]) * inv_l, __uint_as_float(cur[i * 8 + 3]) * inv_l);
            v.z = pack_f16x2(__uint_as_float(cur[i * 8 + 4]) * inv_l, __uint_as_float(cur[i * 8 + 5]) * inv_l);
            v.w = pack_f16x2(__uint_as_float(cur[i * 8 + 6]) * inv_l, __uint_as_float(cur[i * 8 + 7]) * inv_l);
            const int unit = ((c & 3) * 2 + i) ^ (lane & 7);
            *reinterpret_cast<uint4*>(prow + unit * 16) = v;
          }
        }
        fence_proxy_async_smem();
        // O of this stage has been read: let the next item's first product overwrite it
        tc_fence_before();
        __syncwarp();
        if (lane == 0) {
          const int row0 = g.r0[s] + static_cast<int>(lane_base);
          if (row0 < N) {  // rows of the box beyond the sequence are clipped by the store
            tma_store_4d(&mapO, out_stage, 0, row0, 0, g.bh);
            tma_store_commit();
          }
          mbar_arrive(&p_full[s]);
        }
        arrived_early[s] = true;
      };
      for (int j = g.lo_all; j < g.hi_all && ok; ++j) {
        // a stage that has run out of tiles is finished first, while the other stage is still in its softmax
        if (epi_pending[0] && j >= g.hi[0]) epilogue(std::integral_constant<int, 0>{});
        if (epi_pending[1] && j >= g.hi[1]) epilogue(std::integral_constant<int, 1>{});
        if (!ok) break;
#pragma unroll
        for (int s = 0; s < 2; ++s) {
          if (j < g.lo[s] || j >= g.hi[s]) continue;
          if (j == g.lo[s]) {  // first tile of the item: nothing to rescale, and no factors are handed over
            const bool done = arrived_early[s];
            arrived_early[s] = false;
            if (done) continue;
          } else {
            if (!mbar_wait_warp(&alpha_ready[s], n_alpha[s] & 1, abort_flag)) { ok = false; break; }
            ++n_alpha[s];
            const float alpha = sAlpha[s * kBlockM + row_l];
            if (__any_sync(0xffffffffu, alpha != 1.f)) {
              tc_fence_after();
              const uint32_t tO = tmem_addr(tmem_base, lane_base, s == 0 ? Cfg::kColO0 : Cfg::kColO1);
#pragma unroll 1
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
          }
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(&p_full[s]);
        }
      }
      if (!ok) break;
      if (epi_pending[0]) epilogue(std::integral_constant<int, 0>{});
      if (ok && epi_pending[1]) epilogue(std::integral_constant<int, 1>{});
    }
    if (lane == 0) tma_store_wait_all();  // also on the give-up path: stores in flight read this CTA's shared memory
  } else {
    reg_dec<FA_REG_MISC>();
    if (warp == 12) {
      // ===================================================================================
      // tensor-core issuer. The whole warp walks the schedule and waits, so that addresses and
      // descriptors are warp-uniform values; one elected lane issues the tcgen05 instructions.
      // ===================================================================================
      constexpr uint32_t idesc_qk = umma_idesc_f16(kBlockM, kBlockN, 0, 0);
      constexpr uint32_t idesc_pv = umma_idesc_f16(kBlockM, D, 0, 1);
      // Descriptors are built once; per instruction only the 16-byte-unit start address moves.
      const uint64_t kdesc0 = umma_desc_sw128(0, 16, 1024);               // K-major tiles (Q, K)
      const uint64_t vdesc0 = umma_desc_sw128(0, Cfg::kPanelBytes, 1024);  // MN-major tile (V)
      const uint32_t q_addr = smem_u32(sQ);
      const uint32_t kv_addr = smem_u32(sKV);
      const uint64_t qdesc[2] = {kdesc0 + (q_addr >> 4), kdesc0 + ((q_addr + Cfg::kTileBytes) >> 4)};
      uint32_t ring_slot = 0, ring_par = 0;  // ring position (slot, phase parity) of K tile lo_all of the current item
      uint32_t n_p[2] = {0, 0}, n_q[2] = {0, 0};
      uint32_t n_items = 0;
      bool ok = true;
      while (ok) {
        ItemGeom g;
        const int item = take_item(n_items, g);
        if (item < 0) break;
        // Ring positions are carried along instead of recomputed: (slot_v, par_v) is where V_j lives,
        // (slot_k, par_k) where K_{j+1} lives. Rounds in which both stages have a P.V for tile j and a
        // score tile j+1 ("interior", nearly all of a long sequence) take a branch-free body; the first
        // and last rounds of an item take the general one.
        uint32_t slot_k = ring_slot, par_k = ring_par;  // K_{lo_all}
        uint32_t slot_v = 0, par_v = 0;                 // set when j reaches lo_all
        auto advance = [](uint32_t& slot, uint32_t& par, uint32_t n) {
          slot += n;
          if (slot >= static_cast<uint32_t>(Cfg::kStages)) { slot -= Cfg::kStages; par ^= 1u; }
        };
        // interior rounds in_lo <= j < in_hi: for both stages tile j is neither the first (its P.V accumulates)
        // nor among the last two (no Q release, no final commit), and tile j+1 exists
        const int in_lo = max(g.lo[0], g.lo[1]) + 1;
        const int in_hi = min(g.hi[0], g.hi[1]) - 2;
        auto round_body = [&](auto interior_tag, int j) {
          constexpr bool kInterior = decltype(interior_tag)::value;
#pragma unroll
          for (int s = 0; s < 2; ++s) {
            const bool act_j = kInterior || (j >= g.lo[s] && j < g.hi[s]);
            const bool act_n = kInterior || (j + 1 >= g.lo[s] && j + 1 < g.hi[s]);
            const bool other_j = (s == 0) && (kInterior || (j >= g.lo[1] && j < g.hi[1]));          // stage 1 still needs V_j
            const bool other_n = (s == 0) && (kInterior || (j + 1 >= g.lo[1] && j + 1 < g.hi[1]));  // stage 1 still needs K_j+1
            // stage 0 already waited for this tile in the same round
            const bool v_seen = (s == 1) && (kInterior || (j >= g.lo[0] && j < g.hi[0]));
            const bool k_seen = (s == 1) && (kInterior || (j + 1 >= g.lo[0] && j + 1 < g.hi[0]));
            const uint32_t colS = (s == 0) ? Cfg::kColS0 : Cfg::kColS1;
            const uint32_t colO = (s == 0) ? Cfg::kColO0 : Cfg::kColO1;
            if (act_j) {  // O_s += P_s(j) V_j, in two halves of 64 keys as P arrives
              const uint64_t vdesc = vdesc0 + ((kv_addr + slot_v * Cfg::kTileBytes) >> 4);
              if (!v_seen && !mbar_wait_warp(&kv_full[slot_v], par_v, abort_flag)) { ok = false; return; }
              if (!mbar_wait_warp(&p_full[s], n_p[s] & 1, abort_flag)) { ok = false; return; }
              tc_fence_after();
              if (elect_one()) {
                umma_ts(tmem_base + colO, tmem_base + colS, vdesc, idesc_pv, (kInterior || j > g.lo[s]) ? 1u : 0u);
#pragma unroll
                for (int kk = 1; kk < 4; ++kk)
                  umma_ts(tmem_base + colO, tmem_base + colS + kk * 8, vdesc + kk * (2048 >> 4), idesc_pv, 1u);
              }
              __syncwarp();
              if (!mbar_wait_warp(&p_full2[s], n_p[s] & 1, abort_flag)) { ok = false; return; }
              ++n_p[s];
              tc_fence_after();
              if (elect_one()) {
#pragma unroll
                for (int kk = 4; kk < 8; ++kk)
                  umma_ts(tmem_base + colO, tmem_base + colS + kk * 8, vdesc + kk * (2048 >> 4), idesc_pv, 1u);
                if (!other_j) umma_commit(&kv_empty[slot_v]);
                if (!kInterior && j + 1 == g.hi[s]) umma_commit(&o_full[s]);
              }
              __syncwarp();
            }
            if (act_n) {  // S_s = Q_s K_{j+1}^T
              if (!kInterior && j + 1 == g.lo[s]) {
                if (!mbar_wait_warp(&q_full[s], n_q[s] & 1, abort_flag)) { ok = false; return; }
                ++n_q[s];
              }
              if (!k_seen && !mbar_wait_warp(&kv_full[slot_k], par_k, abort_flag)) { ok = false; return; }
              tc_fence_after();
              const uint64_t kdesc = kdesc0 + ((kv_addr + slot_k * Cfg::kTileBytes) >> 4);
              if (elect_one()) {
#pragma unroll
                for (int k = 0; k < D / 16; ++k) {
                  const uint32_t off = ((k / 4) * Cfg::kPanelBytes + (k % 4) * 32) >> 4;
                  umma_ss(tmem_base + colS, qdesc[s] + off, kdesc + off, idesc_qk, k > 0 ? 1u : 0u);
                }
                umma_commit(&s_full[s]);
                if (!other_n) umma_commit(&kv_empty[slot_k]);
                if (!kInterior && j + 2 == g.hi[s]) umma_commit(&q_empty[s]);
              }
              __syncwarp();
            }
          }
        };
        for (int j = g.lo_all - 1; j < g.hi_all && ok; ++j) {
          if (j >= in_lo && j < in_hi) round_body(std::true_type{}, j);
          else round_body(std::false_type{}, j);
          // V_{j+1} sits right after K_{j+1}; K_{j+2} two positions after K_{j+1}
          slot_v = slot_k;
          par_v = par_k;
          advance(slot_v, par_v, 1);
          advance(slot_k, par_k, 2);
        }
        {  // the next item's K_{lo_all} follows this item's last V
          uint32_t n = 2u * static_cast<uint32_t>(g.hi_all - g.lo_all);
          while (n >= static_cast<uint32_t>(Cfg::kStages)) { n -= Cfg::kStages; ring_par ^= 1u; }
          advance(ring_slot, ring_par, n);
        }
      }
    } else if (warp == 13 && lane == 0) {
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
        ItemGeom g;
        if (item >= 0) g = decode_item(item, p);
        {  // publish the item to the other roles
          const uint32_t slot = n_pub & 1u;
          if (!mbar_wait(&item_empty[slot], ((n_pub >> 1) & 1u) ^ 1u, abort_flag)) { ok = false; break; }
          volatile int* w = s_geom + slot * 16;
          if (item >= 0) {
            w[0] = g.bh; w[1] = g.pair;
            w[2] = g.r0[0]; w[3] = g.r0[1]; w[4] = g.r1[0]; w[5] = g.r1[1];
            w[6] = g.lo[0]; w[7] = g.lo[1]; w[8] = g.hi[0]; w[9] = g.hi[1];
            w[10] = g.lo_all; w[11] = g.hi_all;
          }
          w[12] = item;
          mbar_arrive(&item_full[slot]);
          ++n_pub;
        }
        if (item < 0) break;
        // claim the following item now; the value is not needed before this item's loads are issued
        next = static_cast<int>(gridDim.x) + atomicAdd(p.sched, 1);
        if (next >= p.num_items) next = -1;
#pragma unroll
        for (int s = 0; s < 2; ++s) {
          if (g.r1[s] < g.r0[s]) continue;
          if (!mbar_wait(&q_empty[s], (n_q[s] & 1) ^ 1, abort_flag)) { ok = false; break; }
          ++n_q[s];
          mbar_arrive_expect_tx(&q_full[s], Cfg::kTileBytes);
          tma_load_4d(sQ + s * Cfg::kTileBytes, &mapQ, &q_full[s], 0, g.r0[s], 0, g.bh);
        }
        for (int j = g.lo_all; j < g.hi_all && ok; ++j) {
#pragma unroll
          for (int t = 0; t < 2; ++t) {
            const uint32_t slot = it % Cfg::kStages;
            if (!mbar_wait(&kv_empty[slot], ((it / Cfg::kStages) & 1) ^ 1, abort_flag)) { ok = false; break; }
#ifdef FA_TEST_WITHHOLD_LOAD  // test build only: CTA 0 never loads its fourth tile, so that a bounded wait runs out
            if (blockIdx.x == 0 && (p.variant & 2) != 0 && it == 3) {
              ++it;
              continue;
            }
#endif
            {
              mbar_arrive_expect_tx(&kv_full[slot], Cfg::kTileBytes);
              tma_load_4d(sKV + slot * Cfg::kTileBytes, t == 0 ? &mapK : &mapV, &kv_full[slot], 0, j * kBlockN, 0, g.bh);
            }
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
  if (warp == 12) tmem_dealloc(tmem_base, Cfg::kTmemCols);
}

}  // namespace fa
