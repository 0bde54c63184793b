// Shared host/device helpers of the ICTC B200 library.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>
#include "../../include/ictc_b200.h"

namespace ictc {

void set_error(const char* fmt, ...);

// Device address of the status word that kernels with bounded waits report through (ictc_kernel_status).
int* kernel_status_word();

// Records a CUDA launch error (if any) and maps it to the C-ABI return code.
inline int finish_launch(const char* what) {
  cudaError_t err = cudaGetLastError();
  if (err != cudaSuccess) {
    set_error("%s: %s", what, cudaGetErrorString(err));
    return ICTC_ERR_LAUNCH;
  }
  return ICTC_OK;
}

constexpr int kWarp = 32;

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// Read-only loads that go through the non-coherent path.
__device__ __forceinline__ float ldg(const float* p) { return __ldg(p); }
__device__ __forceinline__ int64_t ldg(const int64_t* p) { return __ldg(reinterpret_cast<const long long*>(p)); }

}  // namespace ictc
