// Fused edge-geometry, radial-basis, activation and force-assembly kernels of the force engine.
//
// These are the element-wise ends of the model that the reference leaves to a chain of PyTorch
// operators: edge vectors / lengths / unit vectors (mace_ictc/models/mace/backbone.py:941-952), the
// Bessel basis with polynomial envelope (mace_ictc/models/radial_basis.py:11-92), the direction
// harmonics (ictc_o3/basis/ictd_irreps.py:1153-1208), SiLU * 1.679 (mace_ictc/models/mace/layers.py:307-314)
// and the position gradient scatter of autograd.  One kernel each way instead of ~30 launches.
#include "ictc_common.cuh"
#include "generated/harmonics_tables.cuh"

namespace ictc {

template <int A> __device__ __forceinline__ float ipw(float x) { return A == 0 ? 1.f : (A == 1 ? x : x * x); }
template <int A> __device__ __forceinline__ float dpw(float x) { return A == 0 ? 0.f : (A == 1 ? 1.f : 2.f * x); }

constexpr int kRadialMax = 16;

struct GeomArgs {
  const float* pos;          // [N,3]
  const int64_t* src;        // [E]
  const int64_t* dst;        // [E]
  const float* shifts;       // [E,3] lattice units or null
  float box[3];
  float r_max;
  int num_basis, p;
  int64_t E;
  float* sh;                 // [E,9]
  float* rb;                 // [E,num_basis]
  float* unit;               // [E,3]
  float* length;             // [E]
  const float* dsh;          // backward inputs
  const float* drb;
  float* dvec;               // [E,3]
};

__device__ __forceinline__ void envelope(float r, float r_max, int p, float& env, float& denv) {
  const float u = r / r_max;
  if (!(r < r_max)) { env = 0.f; denv = 0.f; return; }
  const float pf = float(p);
  const float up = powf(u, float(p - 1));   // u^(p-1)
  const float a = (pf + 1.f) * (pf + 2.f) * 0.5f, b = pf * (pf + 2.f), c = pf * (pf + 1.f) * 0.5f;
  env = 1.f - a * up * u + b * up * u * u - c * up * u * u * u;
  denv = (-a * pf * up + b * (pf + 1.f) * up * u - c * (pf + 2.f) * up * u * u) / r_max;
}

__global__ void geom_forward_kernel(GeomArgs a) {
  const int64_t e = int64_t(blockIdx.x) * blockDim.x + threadIdx.x;
  if (e >= a.E) return;
  const int64_t i = a.dst[e], j = a.src[e];
  float v[3];
#pragma unroll
  for (int k = 0; k < 3; ++k) {
    v[k] = a.pos[3 * i + k] - a.pos[3 * j + k];
    if (a.shifts) v[k] += a.shifts[3 * e + k] * a.box[k];
  }
  const float r = sqrtf(v[0] * v[0] + v[1] * v[1] + v[2] * v[2]);
  const float rc = fmaxf(r, 1e-8f);
  const float x = v[0] / rc, y = v[1] / rc, z = v[2] / rc;
  a.unit[3 * e + 0] = x;
  a.unit[3 * e + 1] = y;
  a.unit[3 * e + 2] = z;
  a.length[e] = r;
  float val[9];
#pragma unroll
  for (int h = 0; h < 9; ++h) val[h] = 0.f;
#define ICTC_T(h, aa, bb, cc, cf) val[h] = fmaf(cf, ipw<aa>(x) * ipw<bb>(y) * ipw<cc>(z), val[h]);
  ICTC_HARM_TERMS(ICTC_T)
#undef ICTC_T
#pragma unroll
  for (int h = 0; h < 9; ++h) a.sh[9 * e + h] = val[h];
  float env, denv;
  envelope(r, a.r_max, a.p, env, denv);
  const float pref = sqrtf(2.f / a.r_max) / fmaxf(r, 1e-12f);
  const float w = 3.14159265358979323846f / a.r_max;
  for (int k = 0; k < a.num_basis; ++k) a.rb[e * a.num_basis + k] = pref * sinf(r * (w * float(k + 1))) * env;
}

__global__ void geom_backward_kernel(GeomArgs a) {
  const int64_t e = int64_t(blockIdx.x) * blockDim.x + threadIdx.x;
  if (e >= a.E) return;
  const float x = a.unit[3 * e], y = a.unit[3 * e + 1], z = a.unit[3 * e + 2];
  const float r = a.length[e];
  const float rc = fmaxf(r, 1e-8f);
  // harmonics: du = J^T dsh
  float g[9];
#pragma unroll
  for (int h = 0; h < 9; ++h) g[h] = a.dsh[9 * e + h];
  float d0 = 0.f, d1 = 0.f, d2 = 0.f;
#define ICTC_T(h, aa, bb, cc, cf)                                        \
  d0 = fmaf(g[h] * (cf), dpw<aa>(x) * ipw<bb>(y) * ipw<cc>(z), d0);       \
  d1 = fmaf(g[h] * (cf), ipw<aa>(x) * dpw<bb>(y) * ipw<cc>(z), d1);       \
  d2 = fmaf(g[h] * (cf), ipw<aa>(x) * ipw<bb>(y) * dpw<cc>(z), d2);
  ICTC_HARM_TERMS(ICTC_T)
#undef ICTC_T
  // radial basis: dr = sum_k drb_k * d(rb_k)/dr
  float env, denv;
  envelope(r, a.r_max, a.p, env, denv);
  const float rs = fmaxf(r, 1e-12f);
  const float pref = sqrtf(2.f / a.r_max);
  const float w = 3.14159265358979323846f / a.r_max;
  float dr = 0.f;
  for (int k = 0; k < a.num_basis; ++k) {
    const float wk = w * float(k + 1);
    float s, c;
    sincosf(r * wk, &s, &c);
    const float f = pref * s / rs;                      // bessel value
    const float df = pref * (wk * c / rs - s / (rs * rs));
    dr = fmaf(a.drb[e * a.num_basis + k], df * env + f * denv, dr);
  }
  const float dot = x * d0 + y * d1 + z * d2;
  a.dvec[3 * e + 0] = dr * x + (d0 - dot * x) / rc;
  a.dvec[3 * e + 1] = dr * y + (d1 - dot * y) / rc;
  a.dvec[3 * e + 2] = dr * z + (d2 - dot * z) / rc;
}

// grad[i] = sum_{e: dst(e)=i} dvec[e] - sum_{e: src(e)=i} dvec[e]; fixed CSR order, no atomics.
__global__ void position_gradient_kernel(int64_t n, int64_t n_dst_rows, const int64_t* __restrict__ dst_rowptr,
                                         const int64_t* __restrict__ src_rowptr, const int64_t* __restrict__ src_order,
                                         const float* __restrict__ dvec, float* grad) {
  const int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= n) return;
  float gx = 0.f, gy = 0.f, gz = 0.f;
  if (i < n_dst_rows) {
    for (int64_t e = dst_rowptr[i]; e < dst_rowptr[i + 1]; ++e) {
      gx += dvec[3 * e];
      gy += dvec[3 * e + 1];
      gz += dvec[3 * e + 2];
    }
  }
  for (int64_t k = src_rowptr[i]; k < src_rowptr[i + 1]; ++k) {
    const int64_t e = src_order ? src_order[k] : k;
    gx -= dvec[3 * e];
    gy -= dvec[3 * e + 1];
    gz -= dvec[3 * e + 2];
  }
  grad[3 * i] = gx;
  grad[3 * i + 1] = gy;
  grad[3 * i + 2] = gz;
}

// y = silu(x) * scale ; backward: dx = dy * scale * sigmoid(x) * (1 + x * (1 - sigmoid(x)))
__global__ void silu_forward_kernel(int64_t n, float scale, const float* __restrict__ x, float* y) {
  const int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const float v = x[i];
  y[i] = v / (1.f + expf(-v)) * scale;
}
__global__ void silu_backward_kernel(int64_t n, float scale, const float* __restrict__ x, const float* __restrict__ dy,
                                     float* dx) {
  const int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const float v = x[i];
  const float s = 1.f / (1.f + expf(-v));
  dx[i] = dy[i] * scale * s * (1.f + v * (1.f - s));
}

// Whole-row layout conversion between mul_ir (block [C][m]) and ir_mul (block [m][C]) for a row made of
// degree blocks, each holding `count` path slots.  One thread per output element: writes are coalesced,
// reads are strided by at most 2l+1 floats and stay inside one cache line group.
constexpr int kLayoutBlocks = 8;
struct LayoutArgs {
  int64_t rows;
  int width, C, nblocks;
  int count[kLayoutBlocks], m[kLayoutBlocks], off[kLayoutBlocks + 1];
};

// One block per group of rows: a row is read as it lies in memory (coalesced) into shared memory, and written in the
// other order from there (the transposed reads hit shared memory with odd strides 2l+1, or stride C across the
// 2l+1 <= 5 components: no bank conflicts worth mentioning), so both global accesses are contiguous.
__global__ void __launch_bounds__(256) layout_copy_kernel(LayoutArgs a, const float* __restrict__ in,
                                                          float* __restrict__ out, int to_ir_mul) {
  extern __shared__ float layout_row[];
  for (int64_t r = blockIdx.x; r < a.rows; r += gridDim.x) {
    const float* src_row = in + r * a.width;
    for (int col = threadIdx.x; col < a.width; col += blockDim.x) layout_row[col] = src_row[col];
    __syncthreads();
    float* dst_row = out + r * a.width;
    for (int col = threadIdx.x; col < a.width; col += blockDim.x) {
      int b = 0;
      while (b + 1 < a.nblocks && col >= a.off[b + 1]) ++b;
      const int m = a.m[b], C = a.C;
      const int rel = col - a.off[b];
      const int slot = rel / (C * m), q = rel - slot * (C * m);
      // output index q -> (outer, inner) of the OUTPUT block; the input block is its transpose
      const int outer = to_ir_mul ? q / C : q / m, inner = to_ir_mul ? q - outer * C : q - outer * m;
      const int src = to_ir_mul ? inner * m + outer : inner * C + outer;
      dst_row[col] = layout_row[a.off[b] + slot * C * m + src];
    }
    __syncthreads();
  }
}

}  // namespace ictc

using namespace ictc;

extern "C" {

static int geom_fill(GeomArgs& a, const float* pos, const int64_t* src, const int64_t* dst, const float* shifts,
                     const float* host_box, float r_max, int num_basis, int p, int64_t E) {
  if (E < 0 || num_basis < 1 || num_basis > kRadialMax || p < 2 || !(r_max > 0)) {
    set_error("edge geometry: invalid arguments");
    return ICTC_ERR_BAD_ARG;
  }
  if ((E + 255) / 256 > 2147483647LL) { set_error("edge geometry: too many edges"); return ICTC_ERR_TOO_LARGE; }
  a.pos = pos; a.src = src; a.dst = dst; a.shifts = shifts;
  for (int k = 0; k < 3; ++k) a.box[k] = host_box ? host_box[k] : 0.f;
  a.r_max = r_max; a.num_basis = num_basis; a.p = p; a.E = E;
  return ICTC_OK;
}

int ictc_edge_geometry_forward(const float* pos, const int64_t* src, const int64_t* dst, const float* shifts,
                               const float* host_box, float r_max, int num_basis, int p, int64_t num_edges,
                               float* sh, float* rb, float* unit, float* length, void* stream) {
  GeomArgs a{};
  if (int rc = geom_fill(a, pos, src, dst, shifts, host_box, r_max, num_basis, p, num_edges)) return rc;
  if (num_edges == 0) return ICTC_OK;
  if (!pos || !src || !dst || !sh || !rb || !unit || !length) { set_error("edge geometry: NULL buffer"); return ICTC_ERR_BAD_ARG; }
  a.sh = sh; a.rb = rb; a.unit = unit; a.length = length;
  geom_forward_kernel<<<(unsigned)((num_edges + 255) / 256), 256, 0, (cudaStream_t)stream>>>(a);
  return finish_launch("edge_geometry_forward");
}

int ictc_edge_geometry_backward(const float* unit, const float* length, float r_max, int num_basis, int p,
                                int64_t num_edges, const float* dsh, const float* drb, float* dvec, void* stream) {
  GeomArgs a{};
  if (int rc = geom_fill(a, nullptr, nullptr, nullptr, nullptr, nullptr, r_max, num_basis, p, num_edges)) return rc;
  if (num_edges == 0) return ICTC_OK;
  if (!unit || !length || !dsh || !drb || !dvec) { set_error("edge geometry backward: NULL buffer"); return ICTC_ERR_BAD_ARG; }
  a.unit = const_cast<float*>(unit); a.length = const_cast<float*>(length); a.dsh = dsh; a.drb = drb; a.dvec = dvec;
  geom_backward_kernel<<<(unsigned)((num_edges + 255) / 256), 256, 0, (cudaStream_t)stream>>>(a);
  return finish_launch("edge_geometry_backward");
}

int ictc_position_gradient(int64_t num_rows, int64_t num_dst_rows, const int64_t* dst_rowptr,
                           const int64_t* src_rowptr, const int64_t* src_order, const float* dvec, float* grad,
                           void* stream) {
  if (num_rows < 0 || num_dst_rows < 0 || num_dst_rows > num_rows) { set_error("position gradient: sizes"); return ICTC_ERR_BAD_ARG; }
  if (num_rows == 0) return ICTC_OK;
  if (!dst_rowptr || !src_rowptr || !grad) { set_error("position gradient: NULL buffer"); return ICTC_ERR_BAD_ARG; }
  position_gradient_kernel<<<(unsigned)((num_rows + 127) / 128), 128, 0, (cudaStream_t)stream>>>(
      num_rows, num_dst_rows, dst_rowptr, src_rowptr, src_order, dvec, grad);
  return finish_launch("position_gradient");
}

int ictc_silu_forward(int64_t n, float scale, const float* x, float* y, void* stream) {
  if (n < 0 || (n > 0 && (!x || !y))) { set_error("silu: invalid arguments"); return ICTC_ERR_BAD_ARG; }
  if (n == 0) return ICTC_OK;
  silu_forward_kernel<<<(unsigned)((n + 255) / 256), 256, 0, (cudaStream_t)stream>>>(n, scale, x, y);
  return finish_launch("silu_forward");
}

int ictc_silu_backward(int64_t n, float scale, const float* x, const float* dy, float* dx, void* stream) {
  if (n < 0 || (n > 0 && (!x || !dy || !dx))) { set_error("silu backward: invalid arguments"); return ICTC_ERR_BAD_ARG; }
  if (n == 0) return ICTC_OK;
  silu_backward_kernel<<<(unsigned)((n + 255) / 256), 256, 0, (cudaStream_t)stream>>>(n, scale, x, dy, dx);
  return finish_launch("silu_backward");
}

int ictc_layout_copy(int64_t rows, int channels, int num_blocks, const int* host_counts, const int* host_ms,
                     const float* in, float* out, int to_ir_mul, void* stream) {
  if (rows < 0 || channels < 1 || num_blocks < 1 || num_blocks > kLayoutBlocks || !host_counts || !host_ms) {
    set_error("layout copy: invalid arguments");
    return ICTC_ERR_BAD_ARG;
  }
  LayoutArgs a;
  a.rows = rows; a.C = channels; a.nblocks = num_blocks;
  int off = 0;
  for (int b = 0; b < num_blocks; ++b) {
    if (host_counts[b] < 0 || host_ms[b] < 1) { set_error("layout copy: invalid block"); return ICTC_ERR_BAD_ARG; }
    a.count[b] = host_counts[b]; a.m[b] = host_ms[b]; a.off[b] = off;
    off += host_counts[b] * host_ms[b] * channels;
  }
  a.off[num_blocks] = off;
  a.width = off;
  const int64_t total = rows * int64_t(off);
  if (total == 0) return ICTC_OK;
  if (!in || !out) { set_error("layout copy: NULL buffer"); return ICTC_ERR_BAD_ARG; }
  const size_t smem = size_t(off) * sizeof(float);
  if (smem > 200 * 1024) { set_error("layout copy: rows of %d floats do not fit shared memory", off); return ICTC_ERR_TOO_LARGE; }
  if (smem > 48 * 1024) {
    const cudaError_t attr = cudaFuncSetAttribute(layout_copy_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem));
    if (attr != cudaSuccess) { set_error("layout copy smem: %s", cudaGetErrorString(attr)); return ICTC_ERR_LAUNCH; }
  }
  const int64_t blocks = rows < 148 * 8 * 4 ? rows : 148 * 8 * 4;       // a few waves of row-looping blocks
  layout_copy_kernel<<<(unsigned)blocks, 256, smem, (cudaStream_t)stream>>>(a, in, out, to_ir_mul);
  return finish_launch("layout_copy");
}

}  // extern "C"
