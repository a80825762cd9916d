// Parameter block and tile geometry shared by the attention-forward kernels and the host
// launcher. Replaces the reference's by-value `mykernelParamType` (include/utils.h:143-165
// of the reference); fields the reference declares but never reads (L, M, seed, split_num)
// are dropped, the window is two-sided, and a status word is added so that a device-side
// wait that runs out of time is reported to the host instead of hanging.
#pragma once
#include <cuda_fp16.h>
#include <cstdint>

namespace fa {

constexpr int kBlockM = 128;  // q rows per tensor-core tile (one TMEM lane per row)
constexpr int kBlockN = 128;  // kv rows per tile
constexpr int kPanel = 64;    // fp16 elements per 128-byte swizzle row

struct FwdParams {
  __half* O;         // [bh][seqlen][head_dim], head_dim contiguous
  int seqlen;        // N
  int bh;            // batch * heads
  float scale_log2;  // softmax_scale * log2(e)
  int causal;        // key j is visible to query i only if j <= i
  int window_left;   // j >= i - window_left   (< 0: unbounded)
  int window_right;  // j <= i + window_right  (< 0: unbounded); forced to 0 by `causal`
  int* status;       // device word, 0 = ok; set non-zero when a bounded wait gave up
  float* dbg;        // optional bring-up dump (serial kernel only), else nullptr
  int variant;       // bit0 (serial kernel): P through shared memory instead of TMEM; bit1 (test build of the
                     // persistent kernel only): CTA 0 withholds one tile so that a bounded wait runs out
  // persistent kernel only
  int num_q_pairs;   // ceil(seqlen / 256)
  int num_items;     // bh * num_q_pairs
  int head_group;    // heads whose items are interleaved pair-major in the work-item order
  const float* alibi_slopes;  // optional, one slope per head (device); the score of (i, j) gets
                              // -slope * |i - j| after scaling, as the reference does (src/mask.h:21-26)
  int heads;         // heads per batch entry (indexes alibi_slopes)
  float* lse;        // optional [bh][seqlen] output: natural-log sum of exp(scaled, biased scores) over the
                     // visible keys of each row (-inf for a row without visible keys); nullptr = not written
                     // (persistent kernel only).
                     // The reference declares L/M outputs (src/flash_forward.h:602-603) but never writes them.
  // dropout on the attention probabilities (persistent kernel, its own instantiation): element (b*h, i, j) is kept
  // when byte (j % 16) of Philox-4x32-10(key = seed, counter = {j / 16, i, b*h, 0}) is below drop_keep_thr
  unsigned drop_keep_thr;   // 1..255 = round(256 * (1 - p)); 0 = every element dropped
  unsigned seed_lo, seed_hi;
  float drop_scale;         // 256 / drop_keep_thr: the kept elements' 1 / (1 - p), folded into the epilogue
  int* sched;        // device scratch, two words that are 0 between launches: [0] next work item to
                     // hand out (beyond the first gridDim.x), [1] CTAs that have finished
};

// Visible key range of query row i is [i - wl, i + wr] ∩ [0, N-1] with "unbounded" for
// negative values. These helpers give the kv-tile range a block of q rows [r0, r1] touches
// (same bounds as the reference's Schedule::next, src/flash_forward.h:52-61, extended to a
// one-sided window) and whether a given kv tile is cut by a boundary and needs the
// per-element predicate.
__host__ __device__ inline int eff_window_right(int causal, int wr) { return causal ? 0 : wr; }

// `bn` is the number of keys per kv tile (128 in the kernels that keep one score tile per q tile, 64 in the
// kernel that double-buffers its score tiles).
__host__ __device__ inline int kv_tile_begin(int r0, int wl, int bn = kBlockN) {
  if (wl < 0) return 0;
  int lo = r0 - wl;
  return lo <= 0 ? 0 : lo / bn;
}
__host__ __device__ inline int kv_tile_end(int r1, int wr_eff, int seqlen, int bn = kBlockN) {  // exclusive
  int hi = seqlen - 1;
  if (wr_eff >= 0 && r1 + wr_eff < hi) hi = r1 + wr_eff;
  return hi / bn + 1;
}
__host__ __device__ inline bool kv_tile_needs_mask(int kv0, int r0, int r1, int wl, int wr_eff, int seqlen,
                                                   int bn = kBlockN) {
  if (kv0 + bn > seqlen) return true;                          // ragged tail
  if (wr_eff >= 0 && kv0 + bn - 1 > r0 + wr_eff) return true;  // right / causal boundary
  if (wl >= 0 && kv0 < r1 - wl) return true;                   // left window boundary
  return false;
}

}  // namespace fa
