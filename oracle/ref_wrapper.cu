// Builds the reference's own CPU attention into oracle/_ref/libref_attention.so: TEST
// INFRASTRUCTURE. The reference translation unit (src/main.cu of the reference) is included
// from where it lies, unmodified, with its main() renamed; nothing of it is copied into this
// repository. Only attention_forward_cpu (src/main.cu:159-268) is ever called.
//
// The reference TU also defines its GPU launch path, which references the driver entry point
// cuTensorMapEncodeTiled. That path is never called from here, so the symbol is satisfied by
// a local definition that reports failure: the library then loads on machines without a
// CUDA driver.
#ifndef REFERENCE_MAIN_CU
#error "pass -DREFERENCE_MAIN_CU=\"<reference>/src/main.cu\""
#endif
#define main reference_main_unused
#include REFERENCE_MAIN_CU
#undef main

#include <thread>
#include <vector>
#include <atomic>

extern "C" CUresult CUDAAPI cuTensorMapEncodeTiled(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                                   const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                                   const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                                   CUtensorMapL2promotion, CUtensorMapFloatOOBfill) {
  return CUDA_ERROR_NOT_SUPPORTED;
}

// The reference function as it is: single thread, all heads, dense N^2.
extern "C" void ref_attention_forward_cpu(const void* q, const void* k, const void* v, float softmax_scale,
                                          int batch, int heads, int seqlen, int head_dim, void* out, int causal,
                                          int window_size, const float* alibi_slopes) {
  attention_forward_cpu(static_cast<const half*>(q), static_cast<const half*>(k), static_cast<const half*>(v),
                        softmax_scale, batch, heads, seqlen, head_dim, static_cast<half*>(out), causal != 0,
                        window_size, alibi_slopes);
}

// The same unmodified function called once per head (batch = heads = 1 on that head's slice)
// from `nthreads` host threads: the "all host cores" figure of the CPU baseline.
extern "C" void ref_attention_forward_cpu_mt(const void* q, const void* k, const void* v, float softmax_scale,
                                             int batch, int heads, int seqlen, int head_dim, void* out, int causal,
                                             int window_size, const float* alibi_slopes, int nthreads) {
  const size_t hs = static_cast<size_t>(seqlen) * head_dim;
  const int bh_total = batch * heads;
  std::atomic<int> next{0};
  auto work = [&]() {
    for (;;) {
      const int bh = next.fetch_add(1);
      if (bh >= bh_total) break;
      attention_forward_cpu(static_cast<const half*>(q) + bh * hs, static_cast<const half*>(k) + bh * hs,
                            static_cast<const half*>(v) + bh * hs, softmax_scale, 1, 1, seqlen, head_dim,
                            static_cast<half*>(out) + bh * hs, causal != 0, window_size,
                            alibi_slopes ? alibi_slopes + (bh % heads) : nullptr);
    }
  };
  if (nthreads < 1) nthreads = 1;
  std::vector<std::thread> pool;
  for (int t = 1; t < nthreads; ++t) pool.emplace_back(work);
  work();
  for (auto& t : pool) t.join();
}
