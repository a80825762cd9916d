/* C ABI of the B200 (sm_100a) attention-forward library, libflashfwd_b200.so.
 *
 * Plain pointers and sizes only: no C++ types, no torch types. All tensor pointers are device
 * pointers on the calling thread's current CUDA device. Layout of Q, K, V, O: fp16, contiguous
 * [batch][heads][seqlen][head_dim] with head_dim fastest, the layout the reference's host entry
 * point takes (src/main.cu:173,182 and src/flash_forward.h:378 of the reference).
 *
 * Every function returns an FA_* status code; none of them exits, aborts or throws (the
 * reference does all three: include/utils.h:16-23, src/flash_forward.h:384-387, :588).
 */
#ifndef FLASH_FORWARD_B200_H
#define FLASH_FORWARD_B200_H

#include <stddef.h>

#ifdef __cplusplus
extern "C" {
#endif

enum {
  FA_OK = 0,
  FA_INVALID_ARG = 1,    /* null or misaligned pointer, non-positive size */
  FA_UNSUPPORTED = 2,    /* head_dim not 64/128, a combination a kernel lacks, device is not sm_100 */
  FA_CUDA_ERROR = 3,     /* a CUDA runtime/driver call failed; see flash_forward_last_error() */
  FA_DEVICE_TIMEOUT = 4  /* a bounded wait inside the kernel gave up (status word set) */
};

/* Attention forward O = softmax(scale * Q K^T + mask) V, asynchronous on `stream`.
 *
 * Replaces the launch path of the reference: run_flash_attention (src/flash_forward.h:593-665)
 * -> run_kernel (src/flash_forward.h:369-590) -> forward_kernel (src/flash_forward.h:78-366),
 * with the argument list the reference's call site uses (src/main.cu:99) reduced to what the
 * path reads: Q/K/V/O, batch, heads, seqlen, head_dim, softmax scale, causal flag, window.
 *
 *   softmax_scale <= 0  -> 1/sqrt(head_dim)  (what the reference hard-codes, :639); a positive scale has to be
 *                          finite and at least 1e-30 (FA_INVALID_ARG otherwise)
 *   is_causal != 0      -> key j visible to query i only if j <= i
 *   window_left  >= 0   -> key j visible only if j >= i - window_left   (< 0: unbounded)
 *   window_right >= 0   -> key j visible only if j <= i + window_right  (< 0: unbounded)
 *                          (any value up to INT_MAX is legal; a window of seqlen or more is unbounded)
 *   stream              -> a cudaStream_t passed as void* (NULL = default stream)
 *
 * head_dim must be 64 or 128 (reference: src/flash_forward.h:588). seqlen may be any positive
 * value (the reference silently requires a multiple of 128). Pointers must be 16-byte aligned.
 * The call returns once the kernel is enqueued; use flash_forward_check() to learn whether a
 * device-side wait timed out.
 *
 * Launches in flight: every launch takes one of 64 pairs of scheduler words (device scratch of a
 * few hundred bytes, allocated on the first call per device) in turn. Launches on one stream are
 * ordered anyway; when a pair is reused by a launch on ANOTHER stream, that stream is first made to
 * wait (cudaStreamWaitEvent) for the earlier launch, so any number of launches may be queued on any
 * number of streams. A call whose stream is being captured into a CUDA graph is refused with
 * FA_UNSUPPORTED: a captured launch would keep its pair for every replay. flash_forward_noalloc, whose
 * scratch slot the caller chooses, is the entry point to capture.
 */
int flash_forward(const void* q, const void* k, const void* v, void* o, int batch, int heads, int seqlen,
                  int head_dim, float softmax_scale, int is_causal, int window_left, int window_right,
                  void* stream);

/* The same forward with the reference's ALiBi bias: the scaled score of (query i, key j) of head h
 * gets -alibi_slopes[h] * |i - j| before the masks (src/mask.h:21-26,49-54,71-83 on the GPU side,
 * src/main.cu:200-207 on the CPU side; the reference's own slopes are negative, src/main.cu:41).
 * alibi_slopes: `heads` floats in device memory. All other arguments as for flash_forward(). */
int flash_forward_alibi(const void* q, const void* k, const void* v, void* o, int batch, int heads, int seqlen,
                        int head_dim, float softmax_scale, int is_causal, int window_left, int window_right,
                        const float* alibi_slopes, void* stream);

/* The forward that also returns the log-sum-exp of every query row:
 *   lse[(b*heads + h)*seqlen + i] = ln( sum over visible keys j of exp(scale * q_i.k_j + bias_ij) )
 * in fp32, device memory, batch*heads*seqlen floats. With O it is what a caller needs to merge
 * attention over disjoint key ranges, or to start a backward pass. The reference's signature carries
 * two outputs for this (`half* L`, `half* M`, src/flash_forward.h:602-603) and its parameter block has
 * the fields (include/utils.h:149-150), but they are never assigned and its kernel never writes
 * them; this entry point is the working form of that output, so its parity is pinned
 * by the definition above (tests compare with an fp64 evaluation), not by reference vectors.
 * alibi_slopes may be NULL (no bias). All other arguments as for flash_forward(). */
int flash_forward_lse(const void* q, const void* k, const void* v, void* o, float* lse, int batch, int heads,
                      int seqlen, int head_dim, float softmax_scale, int is_causal, int window_left, int window_right,
                      const float* alibi_slopes, void* stream);

/* The forward with dropout on the attention probabilities, the reference's Is_dropout / dropout_prob
 * (src/flash_forward.h:248-265): after the softmax, each probability is dropped with probability p or
 * scaled by 1/(1-p); the softmax normalisation itself uses all probabilities.
 *
 * The keep mask is a pure function of (seed, batch*heads index, query row, key column): a key column is
 * kept when its byte of Philox-4x32-10(key = seed, counter = {column / 16, row, batch*heads index, 0}) is
 * below round(256 * (1 - p)). p is therefore applied in steps of 1/256 (flash_forward_dropout_keep_probability()
 * returns the keep probability actually used); p < 1/512 runs the plain forward, bit for bit. The same seed
 * gives the same mask on any GPU and for any sharding of the (batch, head) axis only if the caller passes whole
 * tensors; a slab call numbers its heads from 0.
 *
 * What differs from the reference, on purpose: the reference holds one curand state per q tile, copies it into
 * every thread of the CTA (all threads draw the same numbers) and writes it back (src/flash_forward.h:185-186,
 * :361-363; src/init_curand_states.h:7-14); it skips its own verification when dropout is on (src/main.cu:103).
 * Its random stream is not reproduced; the statistics and the arithmetic are.
 * alibi_slopes may be NULL. All other arguments as for flash_forward(). */
int flash_forward_dropout(const void* q, const void* k, const void* v, void* o, int batch, int heads, int seqlen,
                          int head_dim, float softmax_scale, int is_causal, int window_left, int window_right,
                          const float* alibi_slopes, float dropout_prob, unsigned long long seed, void* stream);

/* Keep probability flash_forward_dropout() uses for `dropout_prob` (a multiple of 1/256; 1.0 when nothing is
 * dropped), or -1 when dropout_prob is outside [0, 1]. Needs no GPU. */
double flash_forward_dropout_keep_probability(float dropout_prob);

/* Several GPUs from one host thread. Every (batch, head) is an independent problem (the reference's CPU
 * path loops over them, src/main.cu:179-186, and on its GPU a work item touches only its own head's
 * rows, src/flash_forward.h:128,:134), so the heads are cut into slabs and each slab runs on its own
 * device with no exchange between devices. Slab i: device ordinal devices[i], tensors q[i], k[i], v[i],
 * o[i] resident on that device and laid out [slab_heads[i]][seqlen][head_dim], stream streams[i]
 * (streams may be NULL: default streams). A slab with 0 heads is skipped; two slabs may name the same
 * device. All launches are enqueued before anything is waited for; wait != 0 then synchronises each
 * stream and reads each device's status word. The calling thread's current device is restored.
 * The reference is single-GPU (device 0 hard-coded, src/flash_forward.h:374,:615). */
int flash_forward_multi_gpu(int num_slabs, const int* devices, const void* const* q, const void* const* k,
                            const void* const* v, void* const* o, const int* slab_heads, int seqlen, int head_dim,
                            float softmax_scale, int is_causal, int window_left, int window_right,
                            void* const* streams, int wait);

/* Same operation with an explicit kernel choice, for tests and bring-up:
 *   kernel  0 = default (warp-specialised persistent kernel), 1 = serial one-tile-per-CTA kernel,
 *           2 = CTA-pair kernel (cta_group::2 MMA over a cluster of two CTAs, head_dim 128 only)
 *   variant kernel-specific switches (serial kernel: bit0 stages P in shared memory; bit1 is read only by the
 *           test build of the library, where it makes one CTA withhold a tile so that a wait runs out)
 *   dbg     optional device buffer of 128*128 + 128*head_dim floats receiving the raw first
 *           score tile and first P.V product of q tile 0 / head 0 (serial kernel), else NULL
 * No counterpart in the reference (it has a single kernel).
 */
int flash_forward_ex(const void* q, const void* k, const void* v, void* o, int batch, int heads, int seqlen,
                     int head_dim, float softmax_scale, int is_causal, int window_left, int window_right,
                     void* stream, int kernel, int variant, float* dbg);

/* The same forward for callers that hold Q, K, V and want O in HOST memory: the flow of the
 * reference's driver (src/main.cu:83-85 upload, :99 run, :101 download) as one blocking call.
 * The (batch, head) axis is cut into chunks of `chunk_heads` heads; upload, kernel and download
 * of successive chunks overlap on three internal streams through a two-slot device workspace
 * of flash_forward_host_workspace_bytes() bytes that the caller provides (256-byte aligned).
 * Pinned host buffers give full overlap; pageable ones work but serialise. Returns after O is
 * complete in o_host, with FA_DEVICE_TIMEOUT if a device-side wait gave up. */
int flash_forward_host(const void* q_host, const void* k_host, const void* v_host, void* o_host, int batch,
                       int heads, int seqlen, int head_dim, float softmax_scale, int is_causal, int window_left,
                       int window_right, void* workspace, size_t workspace_bytes, int chunk_heads);
size_t flash_forward_host_workspace_bytes(int seqlen, int head_dim, int chunk_heads);

/* Waits for `stream`, then reads and clears the current device's status word. Returns FA_OK,
 * FA_DEVICE_TIMEOUT, or FA_CUDA_ERROR. Replaces the reference's CUDA_CHECK(cudaDeviceSynchronize())
 * + exit (src/flash_forward.h:654-655). There is ONE status word per device, not per stream: a
 * time-out raised by a launch on another stream of the device is reported (and consumed) by whichever
 * check comes first. Like flash_forward() it allocates the device's scratch on first use; hosts that
 * must not allocate use flash_forward_noalloc() and flash_forward_noalloc_check(). */
int flash_forward_check(void* stream);

/* The reference's host entry point, positional argument for positional argument
 * (src/flash_forward.h:593-612; `N` is the number of heads and `S` the sequence length there).
 * Blocking, prints "TIME: <ms>" like src/flash_forward.h:664. Mapping:
 *   Is_local  -> window_left = window_right = window_size (symmetric, :640-641; mask.h:55)
 *   Is_causal -> window_right = 0 (both masks apply when both flags are set, mask.h:15,:43)
 *   L, M      -> ignored (the reference never reads them)
 *   Has_alibi -> alibi_slopes (device, one float per head) is applied as in flash_forward_alibi()
 *   Is_dropout -> flash_forward_dropout() with dropout_prob; `states` is ignored (the reference's curand states
 *                 are seeded with 48 by its driver, src/main.cu:93-95, and advance from call to call: here the
 *                 seed starts at 48 and is incremented by every call that uses dropout)
 * Unlike the reference it runs on the current device and returns a status instead of exiting. */
int run_flash_attention_c(int B, int N, int S, int d, void* Q, void* K, void* V, void* O, void* L, void* M,
                          int Is_dropout, int Is_causal, int Is_local, int Has_alibi, int window_size,
                          float* alibi_slopes, float dropout_prob, void* states);

/* Heads per scheduling group that the default kernel would use for batch_heads = batch*heads problems of this
 * shape on a GPU with num_sms SMs (1 = head-major order). Host logic only, for tests and tuning; the reference
 * schedules q tiles in natural order (src/flash_forward.h:43-64) and has no such notion. 0 on bad arguments. */
int flash_forward_head_group(int batch_heads, int seqlen, int head_dim, int is_causal, int window_left,
                             int window_right, int num_sms);

/* Message for the last non-OK status returned on the calling thread ("" if none). */
const char* flash_forward_last_error(void);

/* Algorithmic work of one call, the count the throughput figures use: 4*B*H*N^2*d without a
 * window, exactly half of that when causal; with a window, 4 * head_dim * (visible query-key
 * pairs) summed over batch*heads. Needs no GPU. */
double flash_forward_flops(int batch, int heads, int seqlen, int head_dim, int is_causal, int window_left,
                           int window_right);

/* Host-side view of the kernel's tile plan: the kv tiles (128 keys each) that query rows
 * [row_begin, row_end] read are [*tile_begin, *tile_end), of which *masked_tiles are cut by a
 * mask boundary or by the end of the sequence and take the per-element predicate; all others
 * run unmasked. Same bounds as the reference's Schedule::next (src/flash_forward.h:52-61),
 * extended to a two-sided window. Needs no GPU. */
int flash_forward_kv_range(int seqlen, int is_causal, int window_left, int window_right, int row_begin,
                           int row_end, int* tile_begin, int* tile_end, int* masked_tiles);

/* Attention forward for callers that must not allocate device memory. No counterpart in the
 * reference. flash_forward() above obtains its few words of device scratch (status word, work
 * counters) from cudaMalloc on the first call per device. Some hosts cannot afford that call:
 * a serving process whose device memory is handed out entirely by its own pool, where a stray
 * cudaMalloc can fail or fragment the pool; a latency-critical loop, because cudaMalloc
 * synchronises the whole device; a plug-in that runs under an allocator hook which forbids
 * raw allocations. For them this entry point runs the same persistent kernel with its scratch
 * in a fixed 256-byte array that is part of the library's device image (every GPU that loads
 * the library holds those 256 bytes until the process exits). It calls no cudaMalloc, cudaFree
 * or other allocating routine.
 *
 *   slot  which of the 16 four-word scratch slots this call uses, 0..15. Anything else is
 *         rejected with FA_INVALID_ARG; so is a problem whose work-item count
 *         batch*heads*ceil(seqlen/256) does not fit the slot's 32-bit work counter.
 *   wait  0: return once the work is enqueued on `stream` (flash_forward_noalloc_check() reads the
 *         slot's status later; flash_forward_check() is NOT for these hosts, it allocates);
 *         non-zero: block until the kernel has finished and return FA_DEVICE_TIMEOUT if its status
 *         word was set.
 *
 * All other arguments as for flash_forward(). A slot keeps the contents the last call left in it;
 * every call first clears its slot on `stream`. Calls that use the same slot must not overlap on
 * the GPU (they would share one work counter and race); calls on different slots may.
 * The first call on a device performs a one-time set-up (looks up the scratch array's device
 * address, sets the kernel's shared-memory attribute); make that first call before any stream
 * capture begins. */
int flash_forward_noalloc(const void* q, const void* k, const void* v, void* o, int batch, int heads, int seqlen,
                          int head_dim, float softmax_scale, int is_causal, int window_left, int window_right,
                          void* stream, int slot, int wait);

/* Status of the last flash_forward_noalloc() call on scratch slot `slot` of the current device: waits
 * for `stream`, reads the slot's status word (a 4-byte device-to-host copy; nothing is allocated) and
 * returns FA_OK or FA_DEVICE_TIMEOUT. The word is cleared by the next call on that slot. No counterpart
 * in the reference. */
int flash_forward_noalloc_check(void* stream, int slot);

/* Frees the per-device status words, events and streams this library created, and forgets what it
 * learned about each device (scratch addresses, kernel attributes), so that it can be used again
 * after a device reset. Optional. */
int flash_forward_shutdown(void);

#ifdef __cplusplus
}
#endif
#endif /* FLASH_FORWARD_B200_H */
