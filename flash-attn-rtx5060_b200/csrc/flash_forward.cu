// Host side of libflashfwd_b200.so: argument checks, TMA descriptors, kernel dispatch and the
// status word. Declared in include/flash_forward_b200.h. This is the replacement for the
// reference's run_flash_attention / run_kernel / create_tensor_map
// (src/flash_forward.h:593-665, :369-590 and include/utils.h:168-186 of the reference):
// same inputs, but asynchronous on a caller stream, on the current device, re-entrant
// (descriptors are per-call kernel parameters, not globals), and with status codes in place
// of exit/abort/throw.
#include <cuda.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <atomic>
#include <mutex>

#include "../../include/flash_forward_b200.h"
#include "fwd_params.h"
#include "fwd_pair_ahead.cuh"
#include "fwd_persistent.cuh"
#include "fwd_serial.cuh"

namespace {

thread_local char g_err[512] = "";

int fail(int code, const char* fmt, const char* a = "", const char* b = "") {
  snprintf(g_err, sizeof(g_err), fmt, a, b);
  return code;
}
int fail_cuda(const char* what, cudaError_t e) {
  snprintf(g_err, sizeof(g_err), "%s: %s", what, cudaGetErrorString(e));
  return FA_CUDA_ERROR;
}

using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// The driver entry point is looked up at run time so that the library links against the CUDA
// runtime only and can be loaded (for symbol checks) on a machine without a driver.
EncodeTiledFn encode_tiled_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  });
  return fn;
}

constexpr int kMaxDevices = 64;
// Each launch of the persistent kernel takes the next pair of scheduler words round-robin, so
// that launches in flight on different streams do not share a work counter. The kernel leaves
// its pair at zero; a pair is reused after kSchedSlots further launches on the device, and a
// launch that reuses a pair last used on ANOTHER stream first makes its stream wait for that
// earlier launch (an event per pair), so two launches never run on one pair side by side.
constexpr int kSchedSlots = 64;
constexpr size_t kDeviceWords = 4 + 2 * kSchedSlots;
struct DeviceState {
  std::mutex mu;
  bool probed = false;
  bool is_sm100 = false;
  int num_sms = 0;
  int* status = nullptr;  // device words: [0] status, then kSchedSlots pairs of scheduler words
  unsigned next_sched = 0;
  cudaEvent_t slot_done[kSchedSlots] = {};     // recorded behind the last launch that used the pair
  cudaStream_t slot_stream[kSchedSlots] = {};  // the stream of that launch
  bool slot_used[kSchedSlots] = {};
  bool attr_set[16] = {};
};

// Hands out the scheduler words for one launch on `st`. Call with s->mu held; `*slot_out` is passed to
// sched_release() right after the launch, under the same lock.
int sched_acquire(DeviceState* s, cudaStream_t st, int** words, int* slot_out) {
  cudaError_t e;
  // A captured launch would keep its pair of words for every replay, while the pairs are handed out in turn to
  // later launches: two kernels could then share one work counter. The entry point with a caller-chosen slot
  // (flash_forward_noalloc) is the one to capture.
  cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
  if ((e = cudaStreamIsCapturing(st, &cap)) != cudaSuccess) return fail_cuda("cudaStreamIsCapturing", e);
  if (cap != cudaStreamCaptureStatusNone)
    return fail(FA_UNSUPPORTED, "this entry point cannot be captured into a CUDA graph; capture flash_forward_noalloc");
  const int slot = (int)(s->next_sched++ % kSchedSlots);
  if (!s->slot_done[slot] &&
      (e = cudaEventCreateWithFlags(&s->slot_done[slot], cudaEventDisableTiming)) != cudaSuccess)
    return fail_cuda("cudaEventCreate(scheduler slot)", e);
  if (s->slot_used[slot] && s->slot_stream[slot] != st &&
      (e = cudaStreamWaitEvent(st, s->slot_done[slot], 0)) != cudaSuccess)
    return fail_cuda("cudaStreamWaitEvent(scheduler slot)", e);
  *words = s->status + 4 + 2 * slot;
  *slot_out = slot;
  return FA_OK;
}
int sched_release(DeviceState* s, cudaStream_t st, int slot) {
  cudaError_t e = cudaEventRecord(s->slot_done[slot], st);
  if (e != cudaSuccess) return fail_cuda("cudaEventRecord(scheduler slot)", e);
  s->slot_stream[slot] = st;
  s->slot_used[slot] = true;
  return FA_OK;
}
DeviceState g_dev[kMaxDevices];

int device_state(DeviceState** out) {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return fail_cuda("cudaGetDevice", e);
  if (dev < 0 || dev >= kMaxDevices) return fail(FA_UNSUPPORTED, "device ordinal out of range");
  DeviceState& s = g_dev[dev];
  std::lock_guard<std::mutex> lk(s.mu);
  if (!s.probed) {
    int major = 0, sms = 0;
    if ((e = cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev)) != cudaSuccess)
      return fail_cuda("cudaDeviceGetAttribute", e);
    if ((e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev)) != cudaSuccess)
      return fail_cuda("cudaDeviceGetAttribute", e);
    s.is_sm100 = (major == 10);
    s.num_sms = sms;
    if (s.is_sm100) {
      if ((e = cudaMalloc(&s.status, kDeviceWords * sizeof(int))) != cudaSuccess)
        return fail_cuda("cudaMalloc(status)", e);
      if ((e = cudaMemset(s.status, 0, kDeviceWords * sizeof(int))) != cudaSuccess)
        return fail_cuda("cudaMemset(status)", e);
    }
    s.probed = true;
  }
  *out = &s;
  return FA_OK;
}

// 4-D map over one [bh][seqlen][head_dim] fp16 tensor: {64 contiguous elements, row, 64-wide
// panel, head}. One box = 128 rows x all panels of one head, landing in shared memory as
// [panel][row][64] with the 128-byte swizzle a UMMA descriptor expects. Out-of-range rows of
// a ragged last tile read as zero.
int make_map(CUtensorMap* map, const void* base, int bh, int seqlen, int head_dim, int box_rows, int box_panels = 0) {
  if (box_panels <= 0) box_panels = head_dim / 64;
  EncodeTiledFn enc = encode_tiled_fn();
  if (!enc) return fail(FA_CUDA_ERROR, "cuTensorMapEncodeTiled entry point not available");
  cuuint64_t dims[4] = {64, (cuuint64_t)seqlen, (cuuint64_t)(head_dim / 64), (cuuint64_t)bh};
  cuuint64_t strides[3] = {(cuuint64_t)head_dim * 2, 128, (cuuint64_t)seqlen * head_dim * 2};
  cuuint32_t box[4] = {64, (cuuint32_t)box_rows, (cuuint32_t)box_panels, 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 4, const_cast<void*>(base), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    snprintf(g_err, sizeof(g_err), "cuTensorMapEncodeTiled failed with CUresult %d", (int)r);
    return FA_CUDA_ERROR;
  }
  return FA_OK;
}

template <typename K>
int ensure_smem_attr(DeviceState* s, int slot, K kernel, int bytes) {
  std::lock_guard<std::mutex> lk(s->mu);
  if (s->attr_set[slot]) return FA_OK;
  cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
  if (e != cudaSuccess) return fail_cuda("cudaFuncSetAttribute(MaxDynamicSharedMemorySize)", e);
  s->attr_set[slot] = true;
  return FA_OK;
}

template <int D>
int launch_serial(DeviceState* s, const CUtensorMap& mq, const CUtensorMap& mk, const CUtensorMap& mv,
                  const fa::FwdParams& p, cudaStream_t st) {
  using Cfg = fa::SerialCfg<D>;
  int rc = ensure_smem_attr(s, D == 64 ? 0 : 1, fa::fwd_serial_kernel<D>, Cfg::kSmemBytes);
  if (rc != FA_OK) return rc;
  dim3 grid((p.seqlen + fa::kBlockM - 1) / fa::kBlockM, p.bh);
  fa::fwd_serial_kernel<D><<<grid, 128, Cfg::kSmemBytes, st>>>(mq, mk, mv, p);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return fail_cuda("launch fwd_serial_kernel", e);
  return FA_OK;
}

// CTA-pair kernel with scores computed two tiles ahead (head_dim 128): one q tile per CTA, items are
// pairs of q tiles as in the one-CTA kernel, assigned statically to the clusters.
int launch_pair_ahead(DeviceState* s, const void* q, const void* k, const void* v, const fa::FwdParams& p,
                      cudaStream_t st) {
  using Cfg = fa::AheadCfg;
  const bool alibi = p.alibi_slopes != nullptr;
  int rc = alibi ? ensure_smem_attr(s, 7, fa::fwd_pair_ahead_kernel<true>, Cfg::kSmemBytes)
                 : ensure_smem_attr(s, 6, fa::fwd_pair_ahead_kernel<false>, Cfg::kSmemBytes);
  if (rc != FA_OK) return rc;
  CUtensorMap mq, mkh, mvh;
  if ((rc = make_map(&mq, q, p.bh, p.seqlen, 128, fa::kBlockM)) != FA_OK) return rc;
  if ((rc = make_map(&mkh, k, p.bh, p.seqlen, 128, 64)) != FA_OK) return rc;             // half a K tile: 64 keys
  if ((rc = make_map(&mvh, v, p.bh, p.seqlen, 128, fa::kBlockN, 1)) != FA_OK) return rc;  // half a V tile: one 64-wide panel
  int clusters = s->num_sms / 2;
  if (p.num_items < clusters) clusters = p.num_items;
  if (alibi) fa::fwd_pair_ahead_kernel<true><<<2 * clusters, Cfg::kThreads, Cfg::kSmemBytes, st>>>(mq, mkh, mvh, p);
  else fa::fwd_pair_ahead_kernel<false><<<2 * clusters, Cfg::kThreads, Cfg::kSmemBytes, st>>>(mq, mkh, mvh, p);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return fail_cuda("launch fwd_pair_ahead_kernel", e);
  return FA_OK;
}

template <int D, bool kAlibi, bool kLse, bool kDropout = false>
int launch_persistent_as(DeviceState* s, const CUtensorMap& mq, const CUtensorMap& mk, const CUtensorMap& mv,
                         const CUtensorMap& mo,
                         const fa::FwdParams& p, cudaStream_t st) {
  using Cfg = fa::PersistentCfg<D>;
  // attribute slots 2..5, 8..11 and 12..15: one per instantiation
  constexpr int slot = (kDropout ? 12 : (kLse ? 8 : 2)) + (kAlibi ? 2 : 0) + (D == 64 ? 0 : 1);
  int rc = ensure_smem_attr(s, slot, fa::fwd_persistent_kernel<D, kAlibi, kLse, kDropout>, Cfg::kSmemBytes);
  if (rc != FA_OK) return rc;
  int grid = p.num_items < s->num_sms ? p.num_items : s->num_sms;
  fa::FwdParams pp = p;
  std::lock_guard<std::mutex> lk(s->mu);
  int sched_slot = 0;
  if ((rc = sched_acquire(s, st, &pp.sched, &sched_slot)) != FA_OK) return rc;
  fa::fwd_persistent_kernel<D, kAlibi, kLse, kDropout><<<grid, Cfg::kThreads, Cfg::kSmemBytes, st>>>(mq, mk, mv, mo, pp);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return fail_cuda("launch fwd_persistent_kernel", e);
  return sched_release(s, st, sched_slot);
}

// The ALiBi bias, the log-sum-exp output and dropout are compiled in only where asked for, so the plain
// forward carries none of their arithmetic or live values.
template <int D>
int launch_persistent(DeviceState* s, const CUtensorMap& mq, const CUtensorMap& mk, const CUtensorMap& mv,
                      const CUtensorMap& mo,
                      const fa::FwdParams& p, cudaStream_t st, bool dropout) {
  const bool alibi = p.alibi_slopes != nullptr, lse = p.lse != nullptr;
  if (dropout) return alibi ? launch_persistent_as<D, true, false, true>(s, mq, mk, mv, mo, p, st)
                            : launch_persistent_as<D, false, false, true>(s, mq, mk, mv, mo, p, st);
  if (alibi) return lse ? launch_persistent_as<D, true, true>(s, mq, mk, mv, mo, p, st)
                        : launch_persistent_as<D, true, false>(s, mq, mk, mv, mo, p, st);
  return lse ? launch_persistent_as<D, false, true>(s, mq, mk, mv, mo, p, st)
             : launch_persistent_as<D, false, false>(s, mq, mk, mv, mo, p, st);
}

// ---- host-buffer entry point -----------------------------------------------------------
// Per device: three streams (upload, compute, download) and the events that chain them.
struct HostPipe {
  std::mutex mu;  // one flash_forward_host call at a time per device: the calls share the streams and events below
  bool ready = false;
  cudaStream_t up = nullptr, run = nullptr, down = nullptr;
  cudaEvent_t in_ready[2] = {}, done[2] = {}, out_done[2] = {};
};
HostPipe g_pipe[kMaxDevices];

int host_pipe(HostPipe** out) {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return fail_cuda("cudaGetDevice", e);
  if (dev < 0 || dev >= kMaxDevices) return fail(FA_UNSUPPORTED, "device ordinal out of range");
  HostPipe& hp = g_pipe[dev];
  std::lock_guard<std::mutex> lk(hp.mu);
  if (!hp.ready) {
    if ((e = cudaStreamCreateWithFlags(&hp.up, cudaStreamNonBlocking)) != cudaSuccess ||
        (e = cudaStreamCreateWithFlags(&hp.run, cudaStreamNonBlocking)) != cudaSuccess ||
        (e = cudaStreamCreateWithFlags(&hp.down, cudaStreamNonBlocking)) != cudaSuccess)
      return fail_cuda("cudaStreamCreate", e);
    for (int i = 0; i < 2; ++i) {
      if ((e = cudaEventCreateWithFlags(&hp.in_ready[i], cudaEventDisableTiming)) != cudaSuccess ||
          (e = cudaEventCreateWithFlags(&hp.done[i], cudaEventDisableTiming)) != cudaSuccess ||
          (e = cudaEventCreateWithFlags(&hp.out_done[i], cudaEventDisableTiming)) != cudaSuccess)
        return fail_cuda("cudaEventCreate", e);
    }
    hp.ready = true;
  }
  *out = &hp;
  return FA_OK;
}

// ---- allocation-free entry point ---------------------------------------------------------
// Scratch of flash_forward_noalloc: a fixed block in the library's own device image instead of
// memory obtained from cudaMalloc. kNoAllocSlots slots of four ints each:
//   word 0 status (set non-zero when a bounded wait inside the kernel gave up),
//   words 2-3 the persistent kernel's work counter and finished-CTA counter.
// 256 bytes per GPU that loads the library, held until the process exits.
constexpr int kNoAllocSlots = 16;
static __device__ __align__(256) int g_noalloc_scratch[kNoAllocSlots * 4];

// Host-side record of the set-up done once per device for the allocation-free path. In host code
// `g_noalloc_scratch` is only a handle for the runtime; the device address the kernel needs comes
// from cudaGetSymbolAddress, asked with that device current.
struct NoAllocState {
  std::mutex mu;
  bool ready = false;
  int num_sms = 0;
  int* scratch = nullptr;  // device address of g_noalloc_scratch on this device
  bool attr_set[2] = {};
};
NoAllocState g_noalloc[kMaxDevices];

int noalloc_state(NoAllocState** out) {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return fail_cuda("cudaGetDevice", e);
  if (dev < 0 || dev >= kMaxDevices) return fail(FA_UNSUPPORTED, "device ordinal out of range");
  NoAllocState& s = g_noalloc[dev];
  std::lock_guard<std::mutex> lk(s.mu);
  if (!s.ready) {
    int major = 0, sms = 0;
    if ((e = cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev)) != cudaSuccess)
      return fail_cuda("cudaDeviceGetAttribute", e);
    if ((e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev)) != cudaSuccess)
      return fail_cuda("cudaDeviceGetAttribute", e);
    if (major != 10) return fail(FA_UNSUPPORTED, "this library runs on compute capability 10.x (B200) only");
    void* ptr = nullptr;
    if ((e = cudaGetSymbolAddress(&ptr, g_noalloc_scratch)) != cudaSuccess)
      return fail_cuda("cudaGetSymbolAddress(g_noalloc_scratch)", e);
    s.scratch = static_cast<int*>(ptr);
    s.num_sms = sms;
    s.ready = true;
  }
  *out = &s;
  return FA_OK;
}

template <int D>
int launch_persistent_noalloc(NoAllocState* s, const CUtensorMap& mq, const CUtensorMap& mk, const CUtensorMap& mv,
                              const CUtensorMap& mo,
                              const fa::FwdParams& p, cudaStream_t st) {
  using Cfg = fa::PersistentCfg<D>;
  {
    std::lock_guard<std::mutex> lk(s->mu);
    bool& done = s->attr_set[D == 64 ? 0 : 1];
    if (!done) {
      cudaError_t e = cudaFuncSetAttribute(fa::fwd_persistent_kernel<D, false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                           Cfg::kSmemBytes);
      if (e != cudaSuccess) return fail_cuda("cudaFuncSetAttribute(MaxDynamicSharedMemorySize)", e);
      done = true;
    }
  }
  const int grid = p.num_items < s->num_sms ? p.num_items : s->num_sms;
  fa::fwd_persistent_kernel<D, false><<<grid, Cfg::kThreads, Cfg::kSmemBytes, st>>>(mq, mk, mv, mo, p);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return fail_cuda("launch fwd_persistent_kernel", e);
  return FA_OK;
}

}  // namespace

// Heads per scheduling group of the persistent kernel. Without a mask all items cost the same and head-major
// order (1) shares K/V best. With a causal mask or a window the item costs differ, and interleaving the heads of
// a group pair-major keeps the tail short. Three measured constraints (B200): the K and V rows that a group
// keeps live (the whole head, or the window span) should stay within ~64 MB (the 126 MB L2 holds two copies of
// what both dies read: the long-context workload read K/V from DRAM 2.2 times with 96 MB in flight, 1.5 times
// with 64 MB, 1.1 times with 48 MB, at the same speed; the 8192-row config is 0.6 % faster with 64 MB than
// with 48); a group needs about two items per CTA to balance; and the groups must be of even size (64 heads in
// groups of 12 leave a last group of 4 heads, too few items for 148 CTAs: -4 %).
static int pick_head_group(int bh, int seqlen, int head_dim, int causal, int window_left, int window_right,
                           int num_q_pairs, int num_sms) {
  if (!causal && window_left < 0 && window_right < 0) return 1;
  const int wr = causal ? 0 : window_right;
  long long span = seqlen;
  if (window_left >= 0 && wr >= 0) {
    span = (long long)window_left + wr + 2 * fa::kBlockM;
    if (span > seqlen) span = seqlen;
  }
  const double span_bytes = 4.0 * (double)span * head_dim;  // K and V rows, fp16
  int grp_l2 = (int)(64.0 * 1024 * 1024 / span_bytes);
  const int grp_bal = (2 * num_sms + num_q_pairs - 1) / num_q_pairs;
  int grp = grp_l2 < 16 ? grp_l2 : 16;
  if (grp < grp_bal) grp = grp_bal;
  if (grp > 16) grp = 16;
  if (grp < 1) grp = 1;
  if (grp > bh) grp = bh;
  const int groups = (bh + grp - 1) / grp;
  return (bh + groups - 1) / groups;
}

// A window that reaches past either end of the sequence for every row is no window. Mapping it to
// "unbounded" (-1) here keeps the tile arithmetic (row - window_left, row + window_right) inside int
// for every legal argument, INT_MAX included.
static inline int norm_window(int w, int seqlen) { return (w < 0 || w >= seqlen) ? -1 : w; }

extern "C" {

const char* flash_forward_last_error(void) { return g_err; }

double flash_forward_flops(int batch, int heads, int seqlen, int head_dim, int is_causal, int window_left,
                           int window_right) {
  const double bh = (double)batch * heads, n = seqlen, d = head_dim;
  window_left = norm_window(window_left, seqlen);
  window_right = norm_window(window_right, seqlen);
  const int wr = fa::eff_window_right(is_causal, window_right);
  if (window_left < 0 && window_right < 0) return (is_causal ? 2.0 : 4.0) * bh * n * n * d;
  double pairs = 0;  // exact count of visible (query, key) pairs of one head
  for (int i = 0; i < seqlen; ++i) {
    int lo = window_left >= 0 ? i - window_left : 0;
    int hi = wr >= 0 ? i + wr : seqlen - 1;
    if (lo < 0) lo = 0;
    if (hi > seqlen - 1) hi = seqlen - 1;
    if (hi >= lo) pairs += hi - lo + 1;
  }
  return 4.0 * bh * pairs * d;
}

int flash_forward_head_group(int batch_heads, int seqlen, int head_dim, int is_causal, int window_left,
                             int window_right, int num_sms) {
  if (batch_heads <= 0 || seqlen <= 0 || (head_dim != 64 && head_dim != 128) || num_sms <= 0) return 0;
  const int pairs = (seqlen + 2 * fa::kBlockM - 1) / (2 * fa::kBlockM);
  return pick_head_group(batch_heads, seqlen, head_dim, is_causal ? 1 : 0, norm_window(window_left, seqlen),
                         norm_window(window_right, seqlen), pairs, num_sms);
}

int flash_forward_kv_range(int seqlen, int is_causal, int window_left, int window_right, int row_begin,
                           int row_end, int* tile_begin, int* tile_end, int* masked_tiles) {
  if (seqlen <= 0 || row_begin < 0 || row_end < row_begin || row_end >= seqlen || !tile_begin || !tile_end ||
      !masked_tiles)
    return fail(FA_INVALID_ARG, "bad row range");
  const int wl = norm_window(window_left, seqlen);
  const int wr = fa::eff_window_right(is_causal, norm_window(window_right, seqlen));
  *tile_begin = fa::kv_tile_begin(row_begin, wl);
  *tile_end = fa::kv_tile_end(row_end, wr, seqlen);
  int masked = 0;
  for (int j = *tile_begin; j < *tile_end; ++j)
    masked += fa::kv_tile_needs_mask(j * fa::kBlockN, row_begin, row_end, wl, wr, seqlen) ? 1 : 0;
  *masked_tiles = masked;
  return FA_OK;
}

static int forward_impl(const void* q, const void* k, const void* v, void* o, int batch, int heads, int seqlen,
                        int head_dim, float softmax_scale, int is_causal, int window_left, int window_right,
                        const float* alibi_slopes, void* stream, int kernel, int variant, float* dbg,
                        float* lse = nullptr, float dropout_prob = 0.f, unsigned long long seed = 0) {
  if (!q || !k || !v || !o) return fail(FA_INVALID_ARG, "null tensor pointer");
  if (reinterpret_cast<uintptr_t>(lse) & 3) return fail(FA_INVALID_ARG, "lse must be 4-byte aligned");
  if (lse && kernel != 0) return fail(FA_UNSUPPORTED, "only the default kernel writes the log-sum-exp");
  if (alibi_slopes && kernel == 1) return fail(FA_UNSUPPORTED, "the serial kernel has no ALiBi path");
  if (batch <= 0 || heads <= 0 || seqlen <= 0) return fail(FA_INVALID_ARG, "batch, heads and seqlen must be positive");
  if (head_dim != 64 && head_dim != 128) return fail(FA_UNSUPPORTED, "head_dim must be 64 or 128");
  if ((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(k) | reinterpret_cast<uintptr_t>(v) |
       reinterpret_cast<uintptr_t>(o)) & 15)
    return fail(FA_INVALID_ARG, "tensor pointers must be 16-byte aligned");
  if ((long long)batch * heads > 0x7fffffffLL) return fail(FA_INVALID_ARG, "batch*heads overflows int");
  if (kernel < 0 || kernel > 2) return fail(FA_INVALID_ARG, "kernel must be 0 (default), 1 (serial) or 2 (CTA pair)");
  if (kernel == 2 && head_dim != 128) return fail(FA_UNSUPPORTED, "the CTA-pair kernel needs head_dim 128");
  if (!(softmax_scale == softmax_scale)) return fail(FA_INVALID_ARG, "softmax_scale is NaN");
  // (hidden scores are pushed to about -3e38 before the scale is applied: a scale this small would bring them back)
  if (softmax_scale > 3.0e38f || (softmax_scale > 0.f && softmax_scale < 1.0e-30f))
    return fail(FA_INVALID_ARG, "softmax_scale must be a finite value of at least 1e-30 (or <= 0 for 1/sqrt(head_dim))");
  if (!(dropout_prob >= 0.f && dropout_prob <= 1.f)) return fail(FA_INVALID_ARG, "dropout_prob must lie in [0, 1]");
  // keep threshold in 1/256 steps (nearest); a probability below 1/512 keeps everything and takes the plain kernel
  const unsigned keep_thr = (unsigned)rintf(256.f * (1.f - dropout_prob));
  const bool dropout = keep_thr < 256u;
  if (dropout && kernel != 0) return fail(FA_UNSUPPORTED, "only the default kernel has dropout");
  if (dropout && lse) return fail(FA_UNSUPPORTED, "dropout and the log-sum-exp output are not combined");

  DeviceState* s = nullptr;
  int rc = device_state(&s);
  if (rc != FA_OK) return rc;
  if (!s->is_sm100) return fail(FA_UNSUPPORTED, "this library runs on compute capability 10.x (B200) only");

  const int bh = batch * heads;
  if (softmax_scale <= 0.f) softmax_scale = 1.0f / sqrtf((float)head_dim);

  fa::FwdParams p;
  memset(&p, 0, sizeof(p));
  p.O = static_cast<__half*>(o);
  p.seqlen = seqlen;
  p.bh = bh;
  p.scale_log2 = softmax_scale * 1.4426950408889634f;
  p.causal = is_causal ? 1 : 0;
  p.window_left = norm_window(window_left, seqlen);
  p.window_right = norm_window(window_right, seqlen);
  p.status = s->status;
  p.dbg = dbg;
  p.variant = variant;
  p.alibi_slopes = alibi_slopes;
  p.lse = lse;
  p.heads = heads;
  p.drop_keep_thr = dropout ? keep_thr : 256u;
  p.seed_lo = (unsigned)(seed & 0xffffffffull);
  p.seed_hi = (unsigned)(seed >> 32);
  p.drop_scale = (dropout && keep_thr > 0) ? 256.f / (float)keep_thr : (dropout ? 0.f : 1.f);
  p.num_q_pairs = (seqlen + 2 * fa::kBlockM - 1) / (2 * fa::kBlockM);
  if ((long long)bh * p.num_q_pairs > 0x7fffffffLL) return fail(FA_INVALID_ARG, "too many work items");
  p.num_items = bh * p.num_q_pairs;
  p.head_group = pick_head_group(bh, seqlen, head_dim, p.causal, p.window_left, p.window_right, p.num_q_pairs, s->num_sms);

  CUtensorMap mq, mk, mv, mo;
  if ((rc = make_map(&mq, q, bh, seqlen, head_dim, fa::kBlockM)) != FA_OK) return rc;
  if ((rc = make_map(&mk, k, bh, seqlen, head_dim, fa::kBlockN)) != FA_OK) return rc;
  if ((rc = make_map(&mv, v, bh, seqlen, head_dim, fa::kBlockN)) != FA_OK) return rc;
  if ((rc = make_map(&mo, o, bh, seqlen, head_dim, 32)) != FA_OK) return rc;  // one correction warp's rows per store

  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (kernel == 2) return launch_pair_ahead(s, q, k, v, p, st);
  if (kernel == 1) {
    return head_dim == 64 ? launch_serial<64>(s, mq, mk, mv, p, st) : launch_serial<128>(s, mq, mk, mv, p, st);
  }
  return head_dim == 64 ? launch_persistent<64>(s, mq, mk, mv, mo, p, st, dropout)
                        : launch_persistent<128>(s, mq, mk, mv, mo, p, st, dropout);
}

int flash_forward_ex(const void* q, const void* k, const void* v, void* o, int batch, int heads, int seqlen,
                     int head_dim, float softmax_scale, int is_causal, int window_left, int window_right,
                     void* stream, int kernel, int variant, float* dbg) {
  return forward_impl(q, k, v, o, batch, heads, seqlen, head_dim, softmax_scale, is_causal, window_left, window_right,
                      nullptr, stream, kernel, variant, dbg);
}

int flash_forward(const void* q, const void* k, const void* v, void* o, int batch, int heads, int seqlen,
                  int head_dim, float softmax_scale, int is_causal, int window_left, int window_right,
                  void* stream) {
  return forward_impl(q, k, v, o, batch, heads, seqlen, head_dim, softmax_scale, is_causal, window_left, window_right,
                      nullptr, stream, 0, 0, nullptr);
}

int flash_forward_alibi(const void* q, const void* k, const void* v, void* o, int batch, int heads, int seqlen,
                        int head_dim, float softmax_scale, int is_causal, int window_left, int window_right,
                        const float* alibi_slopes, void* stream) {
  if (!alibi_slopes) return fail(FA_INVALID_ARG, "alibi_slopes is null");
  return forward_impl(q, k, v, o, batch, heads, seqlen, head_dim, softmax_scale, is_causal, window_left, window_right,
                      alibi_slopes, stream, 0, 0, nullptr);
}

int flash_forward_lse(const void* q, const void* k, const void* v, void* o, float* lse, int batch, int heads,
                      int seqlen, int head_dim, float softmax_scale, int is_causal, int window_left, int window_right,
                      const float* alibi_slopes, void* stream) {
  if (!lse) return fail(FA_INVALID_ARG, "lse is null");
  return forward_impl(q, k, v, o, batch, heads, seqlen, head_dim, softmax_scale, is_causal, window_left, window_right,
                      alibi_slopes, stream, 0, 0, nullptr, lse);
}

int flash_forward_dropout(const void* q, const void* k, const void* v, void* o, int batch, int heads, int seqlen,
                          int head_dim, float softmax_scale, int is_causal, int window_left, int window_right,
                          const float* alibi_slopes, float dropout_prob, unsigned long long seed, void* stream) {
  return forward_impl(q, k, v, o, batch, heads, seqlen, head_dim, softmax_scale, is_causal, window_left, window_right,
                      alibi_slopes, stream, 0, 0, nullptr, nullptr, dropout_prob, seed);
}

double flash_forward_dropout_keep_probability(float dropout_prob) {
  if (!(dropout_prob >= 0.f && dropout_prob <= 1.f)) return -1.0;
  const unsigned keep_thr = (unsigned)rintf(256.f * (1.f - dropout_prob));
  return keep_thr >= 256u ? 1.0 : keep_thr / 256.0;
}

int flash_forward_multi_gpu(int num_slabs, const int* devices, const void* const* q, const void* const* k,
                            const void* const* v, void* const* o, const int* slab_heads, int seqlen, int head_dim,
                            float softmax_scale, int is_causal, int window_left, int window_right,
                            void* const* streams, int wait) {
  if (num_slabs <= 0 || !devices || !q || !k || !v || !o || !slab_heads)
    return fail(FA_INVALID_ARG, "num_slabs must be positive and the per-slab arrays non-null");
  int prev = 0;
  cudaError_t e = cudaGetDevice(&prev);
  if (e != cudaSuccess) return fail_cuda("cudaGetDevice", e);
  int rc = FA_OK;
  // Enqueue on every device first (the launches are asynchronous, so the devices run side by side),
  // then, if asked, wait for each and read its status word.
  for (int i = 0; i < num_slabs && rc == FA_OK; ++i) {
    if (slab_heads[i] == 0) continue;  // a device may be left without work
    if ((e = cudaSetDevice(devices[i])) != cudaSuccess) { rc = fail_cuda("cudaSetDevice", e); break; }
    rc = forward_impl(q[i], k[i], v[i], o[i], 1, slab_heads[i], seqlen, head_dim, softmax_scale, is_causal, window_left,
                      window_right, nullptr, streams ? streams[i] : nullptr, 0, 0, nullptr);
  }
  for (int i = 0; wait && i < num_slabs && rc == FA_OK; ++i) {
    if (slab_heads[i] == 0) continue;
    if ((e = cudaSetDevice(devices[i])) != cudaSuccess) { rc = fail_cuda("cudaSetDevice", e); break; }
    rc = flash_forward_check(streams ? streams[i] : nullptr);
  }
  cudaSetDevice(prev);
  return rc;
}

int flash_forward_check(void* stream) {
  DeviceState* s = nullptr;
  int rc = device_state(&s);
  if (rc != FA_OK) return rc;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  cudaError_t e = cudaStreamSynchronize(st);
  if (e != cudaSuccess) return fail_cuda("cudaStreamSynchronize", e);
  if (!s->status) return FA_OK;
  int host = 0;
  if ((e = cudaMemcpy(&host, s->status, sizeof(int), cudaMemcpyDeviceToHost)) != cudaSuccess)
    return fail_cuda("cudaMemcpy(status)", e);
  if (host != 0) {
    // Only the status word is cleared: the scheduler words belong to launches that may still be running on other
    // streams, and a kernel that gave up still leaves its own pair at zero (every CTA reaches the final count).
    cudaMemset(s->status, 0, sizeof(int));
    snprintf(g_err, sizeof(g_err), "a wait inside the attention kernel ran out of time (status word %d)", host);
    return FA_DEVICE_TIMEOUT;
  }
  return FA_OK;
}

int run_flash_attention_c(int B, int N, int S, int d, void* Q, void* K, void* V, void* O, void* L, void* M,
                          int Is_dropout, int Is_causal, int Is_local, int Has_alibi, int window_size,
                          float* alibi_slopes, float dropout_prob, void* states) {
  (void)L; (void)M; (void)states;
  // The reference draws from curand states that its driver seeds with 48 (src/main.cu:93-95) and that advance from
  // call to call. Here the mask is a function of (seed, head, row, column); the seed starts at 48 and moves on with
  // every call that uses dropout, so repeated calls draw fresh masks as they do in the reference.
  static std::atomic<unsigned long long> dropout_calls{0};
  if (Is_dropout && !(dropout_prob >= 0.f && dropout_prob <= 1.f)) return fail(FA_INVALID_ARG, "dropout_prob must lie in [0, 1]");
  const float drop_p = Is_dropout ? dropout_prob : 0.f;
  const unsigned long long seed = 48ull + (Is_dropout ? dropout_calls.fetch_add(1) : 0ull);
  if (Has_alibi && !alibi_slopes) return fail(FA_INVALID_ARG, "Has_alibi needs alibi_slopes");
  if (Is_local && window_size < 0) return fail(FA_INVALID_ARG, "Is_local needs window_size >= 0");
  const int wl = Is_local ? window_size : -1;
  const int wr = Is_local ? window_size : -1;
  cudaEvent_t t0, t1;
  cudaError_t e;
  if ((e = cudaEventCreate(&t0)) != cudaSuccess) return fail_cuda("cudaEventCreate", e);
  if ((e = cudaEventCreate(&t1)) != cudaSuccess) { cudaEventDestroy(t0); return fail_cuda("cudaEventCreate", e); }
  cudaEventRecord(t0, 0);
  int rc = forward_impl(Q, K, V, O, B, N, S, d, 0.f, Is_causal, wl, wr, Has_alibi ? alibi_slopes : nullptr, nullptr, 0,
                        0, nullptr, nullptr, drop_p, seed);
  cudaEventRecord(t1, 0);
  if (rc == FA_OK) rc = flash_forward_check(nullptr);
  float ms = 0.f;
  if (rc == FA_OK && cudaEventSynchronize(t1) == cudaSuccess && cudaEventElapsedTime(&ms, t0, t1) == cudaSuccess)
    printf("TIME: %f\n", ms);
  cudaEventDestroy(t0);
  cudaEventDestroy(t1);
  return rc;
}

size_t flash_forward_host_workspace_bytes(int seqlen, int head_dim, int chunk_heads) {
  if (seqlen <= 0 || head_dim <= 0 || chunk_heads <= 0) return 0;
  return (size_t)2 * 4 * (size_t)chunk_heads * seqlen * head_dim * 2;
}

int flash_forward_host(const void* q_host, const void* k_host, const void* v_host, void* o_host, int batch,
                       int heads, int seqlen, int head_dim, float softmax_scale, int is_causal, int window_left,
                       int window_right, void* workspace, size_t workspace_bytes, int chunk_heads) {
  if (!q_host || !k_host || !v_host || !o_host) return fail(FA_INVALID_ARG, "null host pointer");
  if (batch <= 0 || heads <= 0 || seqlen <= 0) return fail(FA_INVALID_ARG, "batch, heads and seqlen must be positive");
  if (head_dim != 64 && head_dim != 128) return fail(FA_UNSUPPORTED, "head_dim must be 64 or 128");
  if (chunk_heads <= 0) return fail(FA_INVALID_ARG, "chunk_heads must be positive");
  if (!workspace || workspace_bytes < flash_forward_host_workspace_bytes(seqlen, head_dim, chunk_heads))
    return fail(FA_INVALID_ARG, "device workspace is null or smaller than flash_forward_host_workspace_bytes()");
  if (reinterpret_cast<uintptr_t>(workspace) & 255) return fail(FA_INVALID_ARG, "workspace must be 256-byte aligned");
  HostPipe* hp = nullptr;
  int rc = host_pipe(&hp);
  if (rc != FA_OK) return rc;

  std::lock_guard<std::mutex> pipe_lock(hp->mu);
  const long long bh = (long long)batch * heads;
  const size_t head_bytes = (size_t)seqlen * head_dim * 2;
  const size_t slot_bytes = (size_t)chunk_heads * head_bytes;
  char* ws = static_cast<char*>(workspace);
  auto dev_ptr = [&](int slot, int tensor) { return ws + ((size_t)slot * 4 + tensor) * slot_bytes; };
  const char* src[3] = {static_cast<const char*>(q_host), static_cast<const char*>(k_host),
                        static_cast<const char*>(v_host)};
  cudaError_t e = cudaSuccess;
  const char* what = nullptr;  // the CUDA call that failed, if any
#define FA_TRY(call)                                  \
  if (!what && (e = (call)) != cudaSuccess) what = #call
  int n = 0;
  for (long long h0 = 0; h0 < bh && !what && rc == FA_OK; h0 += chunk_heads, ++n) {
    const int slot = n & 1;
    const int nh = (int)((bh - h0 < chunk_heads) ? (bh - h0) : chunk_heads);
    const size_t bytes = (size_t)nh * head_bytes;
    // the slot is free once the download that used it two chunks ago has finished
    if (n >= 2) FA_TRY(cudaStreamWaitEvent(hp->up, hp->out_done[slot], 0));
    for (int t = 0; t < 3; ++t)
      FA_TRY(cudaMemcpyAsync(dev_ptr(slot, t), src[t] + (size_t)h0 * head_bytes, bytes, cudaMemcpyHostToDevice, hp->up));
    FA_TRY(cudaEventRecord(hp->in_ready[slot], hp->up));
    FA_TRY(cudaStreamWaitEvent(hp->run, hp->in_ready[slot], 0));
    if (n >= 2) FA_TRY(cudaStreamWaitEvent(hp->run, hp->out_done[slot], 0));
    if (what) break;
    rc = flash_forward(dev_ptr(slot, 0), dev_ptr(slot, 1), dev_ptr(slot, 2), dev_ptr(slot, 3), 1, nh, seqlen, head_dim,
                       softmax_scale, is_causal, window_left, window_right, hp->run);
    if (rc != FA_OK) break;
    FA_TRY(cudaEventRecord(hp->done[slot], hp->run));
    FA_TRY(cudaStreamWaitEvent(hp->down, hp->done[slot], 0));
    FA_TRY(cudaMemcpyAsync(static_cast<char*>(o_host) + (size_t)h0 * head_bytes, dev_ptr(slot, 3), bytes,
                           cudaMemcpyDeviceToHost, hp->down));
    FA_TRY(cudaEventRecord(hp->out_done[slot], hp->down));
  }
#undef FA_TRY
  // Whatever happened, nothing of this call may still be in flight when it returns: the copies read and write the
  // caller's host buffers and workspace.
  char saved[sizeof(g_err)];
  memcpy(saved, g_err, sizeof(saved));  // the message of a failed flash_forward() above
  const cudaError_t e_up = cudaStreamSynchronize(hp->up);
  const int rc_run = flash_forward_check(hp->run);
  const cudaError_t e_down = cudaStreamSynchronize(hp->down);
  if (rc != FA_OK) {
    memcpy(g_err, saved, sizeof(saved));
    return rc;
  }
  if (what) return fail_cuda(what, e);
  if (e_up != cudaSuccess) return fail_cuda("cudaStreamSynchronize(upload stream)", e_up);
  if (rc_run != FA_OK) return rc_run;
  if (e_down != cudaSuccess) return fail_cuda("cudaStreamSynchronize(download stream)", e_down);
  return FA_OK;
}

int flash_forward_noalloc(const void* q, const void* k, const void* v, void* o, int batch, int heads, int seqlen,
                          int head_dim, float softmax_scale, int is_causal, int window_left, int window_right,
                          void* stream, int slot, int wait) {
  if (!q || !k || !v || !o) return fail(FA_INVALID_ARG, "null tensor pointer");
  if (batch <= 0 || heads <= 0 || seqlen <= 0) return fail(FA_INVALID_ARG, "batch, heads and seqlen must be positive");
  if (head_dim != 64 && head_dim != 128) return fail(FA_UNSUPPORTED, "head_dim must be 64 or 128");
  if ((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(k) | reinterpret_cast<uintptr_t>(v) |
       reinterpret_cast<uintptr_t>(o)) & 15)
    return fail(FA_INVALID_ARG, "tensor pointers must be 16-byte aligned");
  if (slot < 0 || slot >= kNoAllocSlots) {
    snprintf(g_err, sizeof(g_err),
             "scratch slot %d is outside the %d slots (256 bytes) that the library's static device scratch holds",
             slot, kNoAllocSlots);
    return FA_INVALID_ARG;
  }
  if (!(softmax_scale == softmax_scale)) return fail(FA_INVALID_ARG, "softmax_scale is NaN");
  // (hidden scores are pushed to about -3e38 before the scale is applied: a scale this small would bring them back)
  if (softmax_scale > 3.0e38f || (softmax_scale > 0.f && softmax_scale < 1.0e-30f))
    return fail(FA_INVALID_ARG, "softmax_scale must be a finite value of at least 1e-30 (or <= 0 for 1/sqrt(head_dim))");
  const long long bh_ll = (long long)batch * heads;
  const int pairs = (seqlen + 2 * fa::kBlockM - 1) / (2 * fa::kBlockM);
  // the work counter in the scratch is a 32-bit int to which the kernel adds the grid size
  if (bh_ll > 0x7fffffffLL || bh_ll * pairs > 0x7fffffffLL - 65536) {
    snprintf(g_err, sizeof(g_err),
             "batch*heads*ceil(seqlen/256) = %lld work items do not fit the 32-bit work counter of the static scratch",
             bh_ll * pairs);
    return FA_INVALID_ARG;
  }

  NoAllocState* s = nullptr;
  int rc = noalloc_state(&s);
  if (rc != FA_OK) return rc;
  if (softmax_scale <= 0.f) softmax_scale = 1.0f / sqrtf((float)head_dim);
  const int bh = (int)bh_ll;
  int* words = s->scratch + slot * 4;

  fa::FwdParams p;
  memset(&p, 0, sizeof(p));
  p.O = static_cast<__half*>(o);
  p.seqlen = seqlen;
  p.bh = bh;
  p.scale_log2 = softmax_scale * 1.4426950408889634f;
  p.causal = is_causal ? 1 : 0;
  p.window_left = norm_window(window_left, seqlen);
  p.window_right = norm_window(window_right, seqlen);
  p.status = words;
  p.sched = words + 2;
  p.num_q_pairs = pairs;
  p.num_items = bh * pairs;
  p.head_group = pick_head_group(bh, seqlen, head_dim, p.causal, p.window_left, p.window_right, pairs, s->num_sms);

  CUtensorMap mq, mk, mv, mo;
  if ((rc = make_map(&mq, q, bh, seqlen, head_dim, fa::kBlockM)) != FA_OK) return rc;
  if ((rc = make_map(&mk, k, bh, seqlen, head_dim, fa::kBlockN)) != FA_OK) return rc;
  if ((rc = make_map(&mv, v, bh, seqlen, head_dim, fa::kBlockN)) != FA_OK) return rc;
  if ((rc = make_map(&mo, o, bh, seqlen, head_dim, 32)) != FA_OK) return rc;  // one correction warp's rows per store

  cudaStream_t st = static_cast<cudaStream_t>(stream);
  // The slot keeps whatever the previous call left; status and both counters must start at zero.
  cudaError_t e = cudaMemsetAsync(words, 0, 4 * sizeof(int), st);
  if (e != cudaSuccess) return fail_cuda("cudaMemsetAsync(scratch slot)", e);
  rc = head_dim == 64 ? launch_persistent_noalloc<64>(s, mq, mk, mv, mo, p, st)
                      : launch_persistent_noalloc<128>(s, mq, mk, mv, mo, p, st);
  if (rc != FA_OK || !wait) return rc;

  if ((e = cudaStreamSynchronize(st)) != cudaSuccess) return fail_cuda("cudaStreamSynchronize", e);
  int host = 0;
  if ((e = cudaMemcpy(&host, words, sizeof(int), cudaMemcpyDeviceToHost)) != cudaSuccess)
    return fail_cuda("cudaMemcpy(status)", e);
  if (host != 0) {
    snprintf(g_err, sizeof(g_err), "a wait inside the attention kernel ran out of time (status word %d)", host);
    return FA_DEVICE_TIMEOUT;
  }
  return FA_OK;
}

int flash_forward_noalloc_check(void* stream, int slot) {
  if (slot < 0 || slot >= kNoAllocSlots) return fail(FA_INVALID_ARG, "scratch slot out of range");
  NoAllocState* s = nullptr;
  int rc = noalloc_state(&s);
  if (rc != FA_OK) return rc;
  cudaError_t e = cudaStreamSynchronize(static_cast<cudaStream_t>(stream));
  if (e != cudaSuccess) return fail_cuda("cudaStreamSynchronize", e);
  int host = 0;
  if ((e = cudaMemcpy(&host, s->scratch + slot * 4, sizeof(int), cudaMemcpyDeviceToHost)) != cudaSuccess)
    return fail_cuda("cudaMemcpy(status)", e);
  if (host != 0) {
    snprintf(g_err, sizeof(g_err), "a wait inside the attention kernel ran out of time (status word %d)", host);
    return FA_DEVICE_TIMEOUT;
  }
  return FA_OK;
}

int flash_forward_shutdown(void) {
  int prev = 0;
  if (cudaGetDevice(&prev) != cudaSuccess) prev = -1;
  for (int d = 0; d < kMaxDevices; ++d) {
    DeviceState& s = g_dev[d];
    std::lock_guard<std::mutex> lk(s.mu);
    if (s.status) {
      cudaSetDevice(d);
      cudaFree(s.status);
      s.status = nullptr;
    }
    s.probed = false;
    for (bool& b : s.attr_set) b = false;
    for (int i = 0; i < kSchedSlots; ++i) {
      if (s.slot_done[i]) {
        cudaSetDevice(d);
        cudaEventDestroy(s.slot_done[i]);
        s.slot_done[i] = nullptr;
      }
      s.slot_used[i] = false;
      s.slot_stream[i] = nullptr;
    }
    s.next_sched = 0;
    {  // a device reset after this call invalidates the scratch address and the kernel attributes: look them up again
      NoAllocState& na = g_noalloc[d];
      std::lock_guard<std::mutex> lk2(na.mu);
      na.ready = false;
      na.scratch = nullptr;
      na.attr_set[0] = na.attr_set[1] = false;
    }
    HostPipe& hp = g_pipe[d];
    std::lock_guard<std::mutex> lkp(hp.mu);
    if (hp.ready) {
      cudaSetDevice(d);
      cudaStreamDestroy(hp.up);
      cudaStreamDestroy(hp.run);
      cudaStreamDestroy(hp.down);
      for (int i = 0; i < 2; ++i) {
        cudaEventDestroy(hp.in_ready[i]);
        cudaEventDestroy(hp.done[i]);
        cudaEventDestroy(hp.out_done[i]);
      }
      hp.up = hp.run = hp.down = nullptr;
      for (int i = 0; i < 2; ++i) hp.in_ready[i] = hp.done[i] = hp.out_done[i] = nullptr;
      hp.ready = false;
    }
  }
  if (prev >= 0) cudaSetDevice(prev);
  return FA_OK;
}

}  // extern "C"
