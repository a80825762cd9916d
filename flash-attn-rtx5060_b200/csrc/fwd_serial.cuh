// Serial bring-up kernel for the attention forward: one CTA of 128 threads per 128-row q tile,
// no overlap between load, tensor work and softmax. It exercises exactly the building blocks
// of the warp-specialised kernel (TMA 128B-swizzled tiles, tcgen05.mma SS for S = Q K^T,
// tcgen05.ld of S one row per thread, exp2 online softmax, P as the TMEM A operand of
// tcgen05.mma TS for O += P V with V read MN-major), so it is the cross-check for that
// kernel on the GPU and the place where a layout assumption can be tested in isolation.
// It computes the same function as the reference's forward_kernel (src/flash_forward.h:78-366)
// with the two-sided window of this library's ABI.
#pragma once
#include "fwd_params.h"
#include "ptx.cuh"

namespace fa {

template <int D>
struct SerialCfg {
  static constexpr int kTileBytes = kBlockN * D * 2;       // one Q / K / V tile
  static constexpr int kPanelBytes = kBlockN * kPanel * 2;  // 16 KiB: 128 rows x 128 B
  static constexpr int kPBytes = kBlockM * kBlockN * 2;     // P staged in smem (variant bit0)
  static constexpr int kSmemBytes = 3 * kTileBytes + kPBytes + 64 + 1024;  // + barriers + alignment slack
  static constexpr uint32_t kTmemCols = 512;
  static constexpr uint32_t kColS = 0, kColP = 128, kColO = 256;
};

template <int D>
__global__ void __launch_bounds__(128, 1)
fwd_serial_kernel(const __grid_constant__ CUtensorMap mapQ, const __grid_constant__ CUtensorMap mapK,
                  const __grid_constant__ CUtensorMap mapV, const FwdParams p) {
  using Cfg = SerialCfg<D>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem;
  uint8_t* sK = sQ + Cfg::kTileBytes;
  uint8_t* sV = sK + Cfg::kTileBytes;
  uint8_t* sP = sV + Cfg::kTileBytes;
  uint64_t* bar_load = reinterpret_cast<uint64_t*>(sP + Cfg::kPBytes);
  uint64_t* bar_mma = bar_load + 1;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bar_load + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int qt = blockIdx.x;
  const int bh = blockIdx.y;
  const int N = p.seqlen;
  const bool p_via_smem = (p.variant & 1) != 0;

  if (warp == 0) {
    tmem_alloc(tmem_slot, Cfg::kTmemCols);
    tmem_relinquish();
  }
  if (tid == 0) {
    mbar_init(bar_load, 1);
    mbar_init(bar_mma, 1);
    *abort_flag = 0;
    fence_mbar_init();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t lane_base = static_cast<uint32_t>(warp) * 32u;
  const uint32_t tS = tmem_addr(tmem_base, lane_base, Cfg::kColS);
  const uint32_t tP = tmem_addr(tmem_base, lane_base, Cfg::kColP);
  const uint32_t tO = tmem_addr(tmem_base, lane_base, Cfg::kColO);

  const int r0 = qt * kBlockM;
  const int r1 = min(r0 + kBlockM, N) - 1;
  const int row = r0 + tid;  // this thread's query row
  const int wl = p.window_left;
  const int wr = eff_window_right(p.causal, p.window_right);
  const int j_lo = kv_tile_begin(r0, wl);
  const int j_hi = kv_tile_end(r1, wr, N);

  constexpr uint32_t idesc_qk = umma_idesc_f16(kBlockM, kBlockN, 0, 0);
  constexpr uint32_t idesc_pv = umma_idesc_f16(kBlockM, D, 0, 1);

  uint32_t ph_load = 0, ph_mma = 0;
  bool ok = true;

  if (tid == 0) {
    mbar_arrive_expect_tx(bar_load, Cfg::kTileBytes);
    tma_load_4d(sQ, &mapQ, bar_load, 0, r0, 0, bh);
  }
  ok = __syncthreads_and(mbar_wait(bar_load, ph_load, abort_flag) && ok);
  ph_load ^= 1;

  float m_run = -INFINITY;  // running row max of the raw (unscaled) scores
  float l_run = 0.f;        // running row sum of exp2((s - m) * scale_log2)

  for (int j = j_lo; j < j_hi && ok; ++j) {
    const int kv0 = j * kBlockN;
    if (tid == 0) {
      mbar_arrive_expect_tx(bar_load, 2 * Cfg::kTileBytes);
      tma_load_4d(sK, &mapK, bar_load, 0, kv0, 0, bh);
      tma_load_4d(sV, &mapV, bar_load, 0, kv0, 0, bh);
    }
    ok = __syncthreads_and(mbar_wait(bar_load, ph_load, abort_flag) && ok);
    ph_load ^= 1;

    // ---- S = Q K^T ----
    if (tid == 0) {
      tc_fence_after();
      const uint32_t qa = smem_u32(sQ), ka = smem_u32(sK);
#pragma unroll
      for (int k = 0; k < D / 16; ++k) {
        const uint32_t off = (k / 4) * Cfg::kPanelBytes + (k % 4) * 32;
        umma_ss(tmem_base + Cfg::kColS, umma_desc_sw128(qa + off, 16, 1024), umma_desc_sw128(ka + off, 16, 1024),
                idesc_qk, k > 0);
      }
      umma_commit(bar_mma);
    }
    ok = __syncthreads_and(mbar_wait(bar_mma, ph_mma, abort_flag) && ok);
    ph_mma ^= 1;
    tc_fence_after();
    if (!ok) break;

    // ---- one score row per thread ----
    float s[kBlockN];
#pragma unroll
    for (int c = 0; c < kBlockN / 32; ++c) {
      uint32_t r[32];
      tmem_ld32(tS + c * 32, r);
      tmem_wait_ld();
#pragma unroll
      for (int i = 0; i < 32; ++i) s[c * 32 + i] = __uint_as_float(r[i]);
    }
    if (p.dbg != nullptr && qt == 0 && bh == 0 && j == j_lo) {
      for (int c = 0; c < kBlockN; ++c) p.dbg[tid * kBlockN + c] = s[c];
    }
    if (kv_tile_needs_mask(kv0, r0, r1, wl, wr, N)) {
      const int c_lo = (wl >= 0) ? row - wl - kv0 : -1;
      int c_hi = N - 1 - kv0;
      if (wr >= 0) c_hi = min(c_hi, row + wr - kv0);
#pragma unroll
      for (int c = 0; c < kBlockN; ++c)
        if (c < c_lo || c > c_hi) s[c] = -INFINITY;
    }
    float m_new = m_run;
#pragma unroll
    for (int c = 0; c < kBlockN; ++c) m_new = fmaxf(m_new, s[c]);
    const float m_use = (m_new == -INFINITY) ? 0.f : m_new;  // fully masked so far: exp2(-inf) = 0, no NaN
    const float alpha = ex2_approx((m_run - m_use) * p.scale_log2);  // m_run = -inf -> 0
    const float neg_ms = -m_use * p.scale_log2;
    float l_tile = 0.f;
    uint32_t pk[kBlockN / 2];
#pragma unroll
    for (int c = 0; c < kBlockN; c += 2) {
      const float e0 = ex2_approx(fmaf(s[c], p.scale_log2, neg_ms));
      const float e1 = ex2_approx(fmaf(s[c + 1], p.scale_log2, neg_ms));
      l_tile += e0 + e1;
      pk[c / 2] = pack_f16x2(e0, e1);
    }
    l_run = l_run * alpha + l_tile;
    m_run = m_new;

    if (p_via_smem) {
      // K-major, 128B-swizzled image: [kv panel][q row][64 fp16]; 16-byte chunk index XOR (row & 7)
#pragma unroll
      for (int c = 0; c < 16; ++c) {
        uint4 v = make_uint4(pk[c * 4], pk[c * 4 + 1], pk[c * 4 + 2], pk[c * 4 + 3]);
        uint8_t* dst = sP + (c / 8) * Cfg::kPanelBytes + tid * 128 + (((c % 8) ^ (tid & 7)) << 4);
        *reinterpret_cast<uint4*>(dst) = v;
      }
      fence_proxy_async_smem();
    } else {
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        uint32_t r[32];
#pragma unroll
        for (int i = 0; i < 32; ++i) r[i] = pk[c * 32 + i];
        tmem_st32(tP + c * 32, r);
      }
    }
    if (j > j_lo) {  // rescale the running output
#pragma unroll
      for (int c = 0; c < D / 32; ++c) {
        uint32_t r[32];
        tmem_ld32(tO + c * 32, r);
        tmem_wait_ld();
#pragma unroll
        for (int i = 0; i < 32; ++i) r[i] = __float_as_uint(__uint_as_float(r[i]) * alpha);
        tmem_st32(tO + c * 32, r);
      }
    }
    tmem_wait_st();
    tc_fence_before();
    __syncthreads();

    // ---- O += P V ----
    if (tid == 0) {
      tc_fence_after();
      const uint32_t va = smem_u32(sV), pa = smem_u32(sP);
#pragma unroll
      for (int kk = 0; kk < kBlockN / 16; ++kk) {
        const uint64_t vdesc = umma_desc_sw128(va + kk * 2048, Cfg::kPanelBytes, 1024);
        const uint32_t acc = (j > j_lo || kk > 0) ? 1u : 0u;
        if (p_via_smem) {
          const uint32_t off = (kk / 4) * Cfg::kPanelBytes + (kk % 4) * 32;
          umma_ss(tmem_base + Cfg::kColO, umma_desc_sw128(pa + off, 16, 1024), vdesc, idesc_pv, acc);
        } else {
          umma_ts(tmem_base + Cfg::kColO, tmem_base + Cfg::kColP + kk * 8, vdesc, idesc_pv, acc);
        }
      }
      umma_commit(bar_mma);
    }
    ok = __syncthreads_and(mbar_wait(bar_mma, ph_mma, abort_flag) && ok);
    ph_mma ^= 1;
    tc_fence_after();

    if (ok && p.dbg != nullptr && qt == 0 && bh == 0 && j == j_lo) {
      for (int c = 0; c < D / 32; ++c) {
        uint32_t r[32];
        tmem_ld32(tO + c * 32, r);
        tmem_wait_ld();
        for (int i = 0; i < 32; ++i) p.dbg[kBlockM * kBlockN + tid * D + c * 32 + i] = __uint_as_float(r[i]);
      }
    }
  }

  // ---- epilogue: O / l -> fp16 -> global ----
  if (ok) {
    const float inv_l = (l_run > 0.f) ? 1.f / l_run : 0.f;
    __half* orow = p.O + (static_cast<size_t>(bh) * N + row) * D;
#pragma unroll
    for (int c = 0; c < D / 32; ++c) {
      uint32_t r[32];
      tmem_ld32(tO + c * 32, r);
      tmem_wait_ld();
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
  } else if (tid == 0) {
    atomicExch(p.status, 1);
    // a give-up leaves at most one TMA load in flight; let it land before the CTA retires
    for (int i = 0; i < 64; ++i) __nanosleep(2000);
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem_base, Cfg::kTmemCols);
}

}  // namespace fa
