#pragma once
#include "fwd_params.h"
#include "ptx.cuh"
namespace fa {
template <int D> struct PersistentCfg { static constexpr int kThreads = 512; static constexpr int kSmemBytes = 1024; };
template <int D>
__global__ void fwd_persistent_kernel(const __grid_constant__ CUtensorMap mapQ, const __grid_constant__ CUtensorMap mapK,
                  const __grid_constant__ CUtensorMap mapV, const FwdParams p) { if (threadIdx.x==0 && blockIdx.x==0) atomicExch(p.status, 99); }
}
