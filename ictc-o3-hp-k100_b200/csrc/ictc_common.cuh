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

// Sums N per-lane values over the warp with recursive halving: at every level a lane keeps half of the values and
// hands the other half to its partner, so 9 values cost 5 + 3 + 2 + 1 + 1 = 12 shuffles instead of 9 x 5.  On return
// the lane holds the total of value `idx` in `out` when `size >= 1` (exactly N lanes do); the order of the additions is
// fixed, so the result is reproducible.
template <int N, int OFF> struct WarpReduceScatter {
  static __device__ __forceinline__ void run(const float (&v)[N], int lane, int& idx, int& size, float& out) {
    constexpr int H = (N + 1) / 2;
    float w[H];
    const bool upper = (lane & OFF) != 0;
#pragma unroll
    for (int t = 0; t < H; ++t) {
      const float hi = (H + t < N) ? v[H + t < N ? H + t : 0] : 0.f;
      const float recv = __shfl_xor_sync(0xffffffffu, upper ? v[t] : hi, OFF);
      w[t] = (upper ? hi : v[t]) + recv;
    }
    idx += upper ? H : 0;
    size = upper ? (size > H ? size - H : 0) : (size < H ? size : H);
    WarpReduceScatter<H, OFF / 2>::run(w, lane, idx, size, out);
  }
};
template <int N> struct WarpReduceScatter<N, 0> {
  static __device__ __forceinline__ void run(const float (&v)[N], int, int&, int&, float& out) { out = v[0]; }
};
template <int N> __device__ __forceinline__ float warp_reduce_scatter(const float (&v)[N], int lane, int& idx, bool& valid) {
  int size = N;
  float out;
  idx = 0;
  WarpReduceScatter<N, 16>::run(v, lane, idx, size, out);
  valid = size >= 1;
  return out;
}

// Read-only loads that go through the non-coherent path.
__device__ __forceinline__ float ldg(const float* p) { return __ldg(p); }
__device__ __forceinline__ int64_t ldg(const int64_t* p) { return __ldg(reinterpret_cast<const long long*>(p)); }

}  // namespace ictc
