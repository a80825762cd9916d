/* Drop-in for the reference's src/flash_forward.h: the same function, name and positional arguments
 * (src/flash_forward.h:593-612 of the reference), implemented by libflashfwd_b200.so. The reference's
 * caller, src/main.cu, includes "flash_forward.h" (line 13) and calls run_flash_attention once (line 99);
 * with this directory on the include path in place of the reference's own header it compiles unchanged:
 *
 *   nvcc -O2 main.cu -I include/reference_shim -I include -I <reference>/include -I <reference>/src \
 *        -L flash-attn-rtx5060_b200 -lflashfwd_b200
 *
 * Behaviour kept: blocking call, "TIME: <ms>" on stdout, exit on any error (the reference exits through
 * CUDA_CHECK, include/utils.h:16-23). */
#ifndef FLASH_FORWARD_REFERENCE_SHIM_H
#define FLASH_FORWARD_REFERENCE_SHIM_H

#include <cuda_fp16.h>
#include <curand_kernel.h>

#include <cstdio>
#include <cstdlib>

#include "flash_forward_b200.h"

inline void run_flash_attention(const int B, const int N /* heads */, const int S /* sequence length */, const int d,
                                half* Q, half* K, half* V, half* O, half* L = nullptr, half* M = nullptr,
                                bool Is_dropout = false, bool Is_causal = false, bool Is_local = false,
                                bool Has_alibi = false, int window_size = 0, float* alibi_slopes = nullptr,
                                float dropout_prob = 0, curandStatePhilox4_32_10_t* states = nullptr) {
  const int rc = run_flash_attention_c(B, N, S, d, Q, K, V, O, L, M, Is_dropout, Is_causal, Is_local, Has_alibi,
                                       window_size, alibi_slopes, dropout_prob, states);
  if (rc != FA_OK) {
    std::fprintf(stderr, "run_flash_attention: %s\n", flash_forward_last_error());
    std::exit(EXIT_FAILURE);
  }
}

#endif /* FLASH_FORWARD_REFERENCE_SHIM_H */
