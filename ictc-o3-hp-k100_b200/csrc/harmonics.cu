// Component-normalised Cartesian direction harmonics (degrees 0..2) and their analytic first and
// second derivatives.  Y_h(n) = sum_terms coeff * nx^a ny^b nz^c with the polynomial terms of the
// frozen ICTC basis as literals (reference math: ictc_o3/basis/ictd_irreps.py:1153-1208; kernel it
// replaces: ictc_o3/backends/k100/hip_direction_harmonics.py:11-56).  One thread per edge.
#include "ictc_common.cuh"
#include "generated/harmonics_tables.cuh"

namespace ictc {

// x^a for a compile-time exponent a in {0,1,2}
template <int A> __device__ __forceinline__ float ipow(float x) { return A == 0 ? 1.f : (A == 1 ? x : x * x); }
// d/dx x^a
template <int A> __device__ __forceinline__ float dpow(float x) { return A == 0 ? 0.f : (A == 1 ? 1.f : 2.f * x); }
// d2/dx2 x^a
template <int A> __device__ __forceinline__ float ddpow(float) { return A == 2 ? 2.f : 0.f; }

// MODE 0: value.  MODE 1: dn = J^T gy.  MODE 2: dgy = J hn and dn2 = sum_h gy_h H_h hn.
template <int MODE>
__global__ void harmonics_kernel(int hdim, int64_t E, const float* __restrict__ n, const float* __restrict__ gy,
                                 const float* __restrict__ hn, float* __restrict__ y, float* __restrict__ dn,
                                 float* __restrict__ dgy) {
  const int64_t e = int64_t(blockIdx.x) * blockDim.x + threadIdx.x;
  if (e >= E) return;
  const float x = n[e * 3 + 0], yy = n[e * 3 + 1], z = n[e * 3 + 2];
  constexpr int HD = (ICTC_HARM_LMAX + 1) * (ICTC_HARM_LMAX + 1);
  if (MODE == 0) {
    float val[HD];
#pragma unroll
    for (int h = 0; h < HD; ++h) val[h] = 0.f;
#define ICTC_T(h, a, b, c, cf) val[h] = fmaf(cf, ipow<a>(x) * ipow<b>(yy) * ipow<c>(z), val[h]);
    ICTC_HARM_TERMS(ICTC_T)
#undef ICTC_T
#pragma unroll
    for (int h = 0; h < HD; ++h)
      if (h < hdim) y[e * hdim + h] = val[h];
    return;
  }
  float g[HD];
#pragma unroll
  for (int h = 0; h < HD; ++h) g[h] = h < hdim ? gy[e * hdim + h] : 0.f;
  if (MODE == 1) {
    float d0 = 0.f, d1 = 0.f, d2 = 0.f;
#define ICTC_T(h, a, b, c, cf)                                   \
  d0 = fmaf(g[h] * (cf), dpow<a>(x) * ipow<b>(yy) * ipow<c>(z), d0); \
  d1 = fmaf(g[h] * (cf), ipow<a>(x) * dpow<b>(yy) * ipow<c>(z), d1); \
  d2 = fmaf(g[h] * (cf), ipow<a>(x) * ipow<b>(yy) * dpow<c>(z), d2);
    ICTC_HARM_TERMS(ICTC_T)
#undef ICTC_T
    dn[e * 3 + 0] = d0;
    dn[e * 3 + 1] = d1;
    dn[e * 3 + 2] = d2;
    return;
  }
  const float h0 = hn[e * 3 + 0], h1 = hn[e * 3 + 1], h2 = hn[e * 3 + 2];
  float jh[HD];
#pragma unroll
  for (int h = 0; h < HD; ++h) jh[h] = 0.f;
  float d0 = 0.f, d1 = 0.f, d2 = 0.f;
#define ICTC_T(h, a, b, c, cf)                                                                         \
  {                                                                                                    \
    const float px = ipow<a>(x), py = ipow<b>(yy), pz = ipow<c>(z);                                     \
    const float qx = dpow<a>(x), qy = dpow<b>(yy), qz = dpow<c>(z);                                     \
    jh[h] = fmaf(cf, h0 * qx * py * pz + h1 * px * qy * pz + h2 * px * py * qz, jh[h]);                 \
    const float s = g[h] * (cf);                                                                       \
    d0 = fmaf(s, h0 * ddpow<a>(x) * py * pz + h1 * qx * qy * pz + h2 * qx * py * qz, d0);               \
    d1 = fmaf(s, h0 * qx * qy * pz + h1 * px * ddpow<b>(yy) * pz + h2 * px * qy * qz, d1);              \
    d2 = fmaf(s, h0 * qx * py * qz + h1 * px * qy * qz + h2 * px * py * ddpow<c>(z), d2);               \
  }
  ICTC_HARM_TERMS(ICTC_T)
#undef ICTC_T
  if (dgy) {
#pragma unroll
    for (int h = 0; h < HD; ++h)
      if (h < hdim) dgy[e * hdim + h] = jh[h];
  }
  if (dn) {
    dn[e * 3 + 0] = d0;
    dn[e * 3 + 1] = d1;
    dn[e * 3 + 2] = d2;
  }
}

static int check_lmax(int lmax, int64_t E) {
  if (lmax < 0 || lmax > ICTC_HARM_LMAX) {
    set_error("direction harmonics are compiled for lmax <= %d (got %d)", ICTC_HARM_LMAX, lmax);
    return ICTC_ERR_BAD_SPEC;
  }
  if (E < 0) { set_error("num_edges < 0"); return ICTC_ERR_BAD_ARG; }
  if ((E + 255) / 256 > 2147483647LL) { set_error("too many edges"); return ICTC_ERR_TOO_LARGE; }
  return ICTC_OK;
}

}  // namespace ictc

using namespace ictc;

extern "C" {

int ictc_harmonics_forward(int lmax, int64_t E, const float* n, float* y, void* stream) {
  if (int rc = check_lmax(lmax, E)) return rc;
  if (E == 0) return ICTC_OK;
  if (!n || !y) { set_error("n and y must not be NULL"); return ICTC_ERR_BAD_ARG; }
  harmonics_kernel<0><<<(unsigned)((E + 255) / 256), 256, 0, (cudaStream_t)stream>>>((lmax + 1) * (lmax + 1), E, n,
                                                                                    nullptr, nullptr, y, nullptr, nullptr);
  return finish_launch("harmonics_forward");
}

int ictc_harmonics_vjp(int lmax, int64_t E, const float* n, const float* gy, float* dn, void* stream) {
  if (int rc = check_lmax(lmax, E)) return rc;
  if (E == 0) return ICTC_OK;
  if (!n || !gy || !dn) { set_error("n, gy and dn must not be NULL"); return ICTC_ERR_BAD_ARG; }
  harmonics_kernel<1><<<(unsigned)((E + 255) / 256), 256, 0, (cudaStream_t)stream>>>((lmax + 1) * (lmax + 1), E, n, gy,
                                                                                    nullptr, nullptr, dn, nullptr);
  return finish_launch("harmonics_vjp");
}

int ictc_harmonics_second(int lmax, int64_t E, const float* n, const float* gy, const float* hn, float* dn2,
                          float* dgy, void* stream) {
  if (int rc = check_lmax(lmax, E)) return rc;
  if (E == 0 || (!dn2 && !dgy)) return ICTC_OK;
  if (!n || !gy || !hn) { set_error("n, gy and hn must not be NULL"); return ICTC_ERR_BAD_ARG; }
  harmonics_kernel<2><<<(unsigned)((E + 255) / 256), 256, 0, (cudaStream_t)stream>>>((lmax + 1) * (lmax + 1), E, n, gy,
                                                                                    hn, nullptr, dn2, dgy);
  return finish_launch("harmonics_second");
}

}  // extern "C"
