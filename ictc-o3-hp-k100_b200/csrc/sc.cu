// Per-species symmetric contraction (correlation 3, input lmax 2) and its derivatives.
//
// y[n,c,l,m] = sum_nu sum_p W_nu^l[species(n), p, c] * sum U_nu^l[m, i1..i_nu, p] * prod_k x[n,c,i_k]
// (reference recursion: ictc_o3/ops/_mace_symmetric_contraction.py:298-354; U tensors:
// ictc_o3/basis/ictd_irreps.py:1535-1557).  The polynomial is emitted as straight-line code with the
// symmetrised couplings as literals (generated/sc_code.cuh); one thread evaluates one (node, channel)
// pair, lanes run over channels so weight-bank and ir_mul feature accesses are coalesced.
// Kernels replaced: circuit<BACK>, circuit (training modes) and reduce_weights of
// ictc_o3/backends/k100/hip_circuit.py:28-257.
//
// Mixed second derivatives use first-order dual numbers on the same generated code: with
// Phi = <gy, F(x,W)>, the cotangents (hx, hW) of (dPhi/dx, dPhi/dW) give
// Psi = d/de Phi(x + e*hx, W + e*hW); dPsi/dgy is the tangent of F and dPsi/dx, dPsi/dW are the
// tangent parts of the first-adjoint kernels.
#include "ictc_common.cuh"

namespace ictc {

struct Dual { float v, d; };

template <class T> __device__ __forceinline__ T zero();
template <> __device__ __forceinline__ float zero<float>() { return 0.f; }
template <> __device__ __forceinline__ Dual zero<Dual>() { return Dual{0.f, 0.f}; }
__device__ __forceinline__ float mul(float a, float b) { return a * b; }
__device__ __forceinline__ float add(float a, float b) { return a + b; }
__device__ __forceinline__ float madd(float c, float a, float b) { return fmaf(c, a, b); }
__device__ __forceinline__ float fmadd(float a, float b, float c) { return fmaf(a, b, c); }
__device__ __forceinline__ float scale(float c, float a) { return c * a; }
__device__ __forceinline__ Dual mul(Dual a, Dual b) { return Dual{a.v * b.v, fmaf(a.v, b.d, a.d * b.v)}; }
__device__ __forceinline__ Dual add(Dual a, Dual b) { return Dual{a.v + b.v, a.d + b.d}; }
__device__ __forceinline__ Dual madd(float c, Dual a, Dual b) { return Dual{fmaf(c, a.v, b.v), fmaf(c, a.d, b.d)}; }
__device__ __forceinline__ Dual fmadd(Dual a, Dual b, Dual c) {
  return Dual{fmaf(a.v, b.v, c.v), fmaf(a.v, b.d, fmaf(a.d, b.v, c.d))};
}
__device__ __forceinline__ Dual scale(float c, Dual a) { return Dual{c * a.v, c * a.d}; }

#include "generated/sc_code.cuh"

template <class T> __device__ __forceinline__ T make(float v, float d);
template <> __device__ __forceinline__ float make<float>(float v, float) { return v; }
template <> __device__ __forceinline__ Dual make<Dual>(float v, float d) { return Dual{v, d}; }
__device__ __forceinline__ float primal(float a) { return a; }
__device__ __forceinline__ float primal(Dual a) { return a.v; }
__device__ __forceinline__ float tangent(float) { return 0.f; }
__device__ __forceinline__ float tangent(Dual a) { return a.d; }

struct ScArgs {
  const float* x;        // [N, 9*C]
  const float* hx;       // tangent of x or null
  const int64_t* species;  // [N]
  const float* w;        // [S, NW, C]
  const float* hw;       // tangent of w or null
  const float* gy;       // [N, NY*C] cotangent of y
  float* y;              // forward output / tangent output
  float* gx;             // [N, 9*C]
  float* partial;        // [chunks, S, NW, C] weight-gradient partial sums
  int64_t N;
  int C, S;
  int ir_mul;            // 0: degree blocks stored [C, 2l+1] (mul_ir); 1: [2l+1, C]
};

// flat offset of component (l, m) of channel c inside a row of `nl` degrees
__device__ __forceinline__ int comp_offset(int l, int m, int c, int C, int ir_mul) {
  return l * l * C + (ir_mul ? m * C + c : c * (2 * l + 1) + m);
}

template <class T> __device__ __forceinline__ void load_row(const float* p, const float* hp, int64_t row, int width,
                                                            int nl, int c, int C, int ir_mul, T* out) {
  const float* r = p + row * int64_t(width) * C;
  const float* hr = hp ? hp + row * int64_t(width) * C : nullptr;
  int k = 0;
  for (int l = 0; l < nl; ++l)
    for (int m = 0; m < 2 * l + 1; ++m, ++k) {
      const int off = comp_offset(l, m, c, C, ir_mul);
      out[k] = make<T>(r[off], hr ? hr[off] : 0.f);
    }
}

template <class T> struct WeightLoader {
  const float* w;
  const float* hw;
  int C;
  __device__ __forceinline__ T operator()(int idx) const { return make<T>(w[idx * C], hw ? hw[idx * C] : 0.f); }
};

// MODE 0: y = F(x,W) (T = float) or its tangent (T = Dual).
// MODE 1: gx = dPhi/dx (float) or its tangent (Dual).
template <class T, int LT, int MODE>
__global__ void __launch_bounds__(128) sc_node_kernel(ScArgs a) {
  constexpr int NY = (LT + 1) * (LT + 1);
  const int64_t idx = int64_t(blockIdx.x) * blockDim.x + threadIdx.x;
  if (idx >= a.N * a.C) return;
  const int64_t n = idx / a.C;
  const int c = int(idx % a.C);
  T x[9];
#pragma unroll
  for (int i = 0; i < 9; ++i) x[i] = zero<T>();
  load_row<T>(a.x, a.hx, n, 9, 3, c, a.C, a.ir_mul, x);
  const int64_t s = a.species[n];
  constexpr int NW = LT == 0 ? ICTC_SC_NW_LT0 : ICTC_SC_NW_LT2;
  WeightLoader<T> w{a.w + (s * NW) * a.C + c, a.hw ? a.hw + (s * NW) * a.C + c : nullptr, a.C};
  if (MODE == 0) {
    T y[NY];
    if (LT == 0) sc_forward_lt0<T>(x, w, reinterpret_cast<T(&)[1]>(y));
    else sc_forward_lt2<T>(x, w, reinterpret_cast<T(&)[9]>(y));
    float* out = a.y + n * int64_t(NY) * a.C;
    int k = 0;
    for (int l = 0; l <= LT; ++l)
      for (int m = 0; m < 2 * l + 1; ++m, ++k) {
        const float val = sizeof(T) == sizeof(float) ? primal(y[k]) : tangent(y[k]);
        out[comp_offset(l, m, c, a.C, a.ir_mul)] = val;
      }
  } else {
    T gy[NY], gx[9];
    load_row<T>(a.gy, nullptr, n, NY, LT + 1, c, a.C, a.ir_mul, gy);
    if (LT == 0) sc_xgrad_lt0<T>(x, w, reinterpret_cast<T(&)[1]>(gy), gx);
    else sc_xgrad_lt2<T>(x, w, reinterpret_cast<T(&)[9]>(gy), gx);
    float* out = a.gx + n * int64_t(9) * a.C;
    int k = 0;
    for (int l = 0; l < 3; ++l)
      for (int m = 0; m < 2 * l + 1; ++m, ++k) {
        const float val = sizeof(T) == sizeof(float) ? primal(gx[k]) : tangent(gx[k]);
        out[comp_offset(l, m, c, a.C, a.ir_mul)] = val;
      }
  }
}

// Weight gradient, stage 1: block = C threads (one per channel) walks a chunk of kScChunk nodes and
// accumulates dPhi/dW per species in shared memory (each thread owns its channel column, so there is
// no race and the order is fixed); the chunk's partial sums go to `partial`.
constexpr int kScChunk = 64;

template <class T, int LT>
__global__ void sc_wgrad_kernel(ScArgs a) {
  constexpr int NY = (LT + 1) * (LT + 1);
  constexpr int NW = LT == 0 ? ICTC_SC_NW_LT0 : ICTC_SC_NW_LT2;
  extern __shared__ float acc[];   // [S][NW][C]
  const int c = threadIdx.x;
  for (int i = c; i < a.S * NW * a.C; i += blockDim.x) acc[i] = 0.f;
  __syncthreads();
  const int64_t first = int64_t(blockIdx.x) * kScChunk;
  const int64_t last = first + kScChunk < a.N ? first + kScChunk : a.N;
  for (int64_t n = first; n < last; ++n) {
    T x[9], gy[NY];
    load_row<T>(a.x, a.hx, n, 9, 3, c, a.C, a.ir_mul, x);
    load_row<T>(a.gy, nullptr, n, NY, LT + 1, c, a.C, a.ir_mul, gy);
    float* col = acc + (a.species[n] * NW) * a.C + c;
    const int C = a.C;
    auto sink = [col, C](int idx, T val) {
      col[idx * C] += sizeof(T) == sizeof(float) ? primal(val) : tangent(val);
    };
    if (LT == 0) sc_wgrad_lt0<T>(x, reinterpret_cast<T(&)[1]>(gy), sink);
    else sc_wgrad_lt2<T>(x, reinterpret_cast<T(&)[9]>(gy), sink);
  }
  __syncthreads();
  float* out = a.partial + int64_t(blockIdx.x) * a.S * NW * a.C;
  for (int i = c; i < a.S * NW * a.C; i += blockDim.x) out[i] = acc[i];
}

// Stage 2: fixed-order sum of the chunk partials.
__global__ void sc_wreduce_kernel(const float* __restrict__ partial, int64_t chunks, int64_t width, float* out) {
  const int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= width) return;
  float s = 0.f;
  for (int64_t k = 0; k < chunks; ++k) s += partial[k * width + i];
  out[i] = s;
}

static int sc_check(int lmax, int target_lmax, int C, int64_t N, int S) {
  if (lmax != 2 || (target_lmax != 0 && target_lmax != 2)) {
    set_error("symmetric contraction kernels are compiled for lmax 2 and target_lmax 0 or 2 (got %d, %d)", lmax,
              target_lmax);
    return ICTC_ERR_BAD_SPEC;
  }
  if (C < 1 || N < 0 || S < 1) { set_error("symmetric contraction: invalid sizes"); return ICTC_ERR_BAD_ARG; }
  if ((N * C + 127) / 128 > 2147483647LL) { set_error("symmetric contraction: too many rows"); return ICTC_ERR_TOO_LARGE; }
  return ICTC_OK;
}

template <class T, int MODE> static int launch_node(int target_lmax, const ScArgs& a, cudaStream_t st) {
  const unsigned blocks = unsigned((a.N * a.C + 127) / 128);
  if (target_lmax == 0) sc_node_kernel<T, 0, MODE><<<blocks, 128, 0, st>>>(a);
  else sc_node_kernel<T, 2, MODE><<<blocks, 128, 0, st>>>(a);
  return finish_launch("sc_node_kernel");
}

template <class T> static int launch_wgrad(int target_lmax, const ScArgs& a, float* gw, cudaStream_t st) {
  const int nw = target_lmax == 0 ? ICTC_SC_NW_LT0 : ICTC_SC_NW_LT2;
  const size_t smem = size_t(a.S) * nw * a.C * sizeof(float);
  if (a.C > 1024 || smem > 200 * 1024) {
    set_error("symmetric contraction weight gradient: species*weights*channels = %zu bytes exceeds the 200 KB "
              "shared-memory accumulator", smem);
    return ICTC_ERR_TOO_LARGE;
  }
  const int64_t chunks = (a.N + kScChunk - 1) / kScChunk;
  const int64_t width = int64_t(a.S) * nw * a.C;
  if (chunks > 0) {
    auto kernel = target_lmax == 0 ? sc_wgrad_kernel<T, 0> : sc_wgrad_kernel<T, 2>;
    cudaError_t err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (err != cudaSuccess) { set_error("sc_wgrad smem: %s", cudaGetErrorString(err)); return ICTC_ERR_LAUNCH; }
    kernel<<<(unsigned)chunks, a.C, smem, st>>>(a);
  }
  sc_wreduce_kernel<<<(unsigned)((width + 255) / 256), 256, 0, st>>>(a.partial, chunks, width, gw);
  return finish_launch("sc_wgrad");
}

}  // namespace ictc

using namespace ictc;

extern "C" {

int ictc_sc_num_weights(int lmax, int target_lmax) {
  if (lmax != 2) return ICTC_ERR_BAD_SPEC;
  if (target_lmax == 0) return ICTC_SC_NW_LT0;
  if (target_lmax == 2) return ICTC_SC_NW_LT2;
  return ICTC_ERR_BAD_SPEC;
}

int64_t ictc_sc_scratch_bytes(int lmax, int target_lmax, int C, int64_t N, int S) {
  const int nw = ictc_sc_num_weights(lmax, target_lmax);
  if (nw < 0 || C < 1 || N < 0 || S < 1) return 0;
  return ((N + kScChunk - 1) / kScChunk) * int64_t(S) * nw * C * 4 + 16;
}

int ictc_sc_forward(int lmax, int target_lmax, int C, int64_t N, int S, int ir_mul, const float* x,
                    const int64_t* species, const float* w, float* y, void* stream) {
  if (int rc = sc_check(lmax, target_lmax, C, N, S)) return rc;
  if (N == 0) return ICTC_OK;
  if (!x || !species || !w || !y) { set_error("sc_forward: NULL buffer"); return ICTC_ERR_BAD_ARG; }
  ScArgs a{};
  a.x = x; a.species = species; a.w = w; a.y = y; a.N = N; a.C = C; a.S = S; a.ir_mul = ir_mul;
  return launch_node<float, 0>(target_lmax, a, (cudaStream_t)stream);
}

int ictc_sc_adjoint(int lmax, int target_lmax, int C, int64_t N, int S, int ir_mul, const float* x,
                    const int64_t* species, const float* w, const float* gy, float* gx, float* gw, void* scratch,
                    void* stream) {
  if (int rc = sc_check(lmax, target_lmax, C, N, S)) return rc;
  if (!gx && !gw) return ICTC_OK;
  if (N > 0 && (!x || !species || !w || !gy)) { set_error("sc_adjoint: NULL buffer"); return ICTC_ERR_BAD_ARG; }
  if (gw && !scratch) { set_error("sc_adjoint: the weight gradient needs scratch"); return ICTC_ERR_BAD_ARG; }
  ScArgs a{};
  a.x = x; a.species = species; a.w = w; a.gy = gy; a.gx = gx; a.partial = (float*)scratch;
  a.N = N; a.C = C; a.S = S; a.ir_mul = ir_mul;
  if (gx && N > 0)
    if (int rc = launch_node<float, 1>(target_lmax, a, (cudaStream_t)stream)) return rc;
  if (gw) return launch_wgrad<float>(target_lmax, a, gw, (cudaStream_t)stream);
  return ICTC_OK;
}

int ictc_sc_second(int lmax, int target_lmax, int C, int64_t N, int S, int ir_mul, const float* x,
                   const int64_t* species, const float* w, const float* gy, const float* hx, const float* hw,
                   float* dgy, float* dx, float* dw, void* scratch, void* stream) {
  if (int rc = sc_check(lmax, target_lmax, C, N, S)) return rc;
  if (!dgy && !dx && !dw) return ICTC_OK;
  if (N > 0 && (!x || !species || !w || !gy)) { set_error("sc_second: NULL buffer"); return ICTC_ERR_BAD_ARG; }
  if (dw && !scratch) { set_error("sc_second: the weight gradient needs scratch"); return ICTC_ERR_BAD_ARG; }
  ScArgs a{};
  a.x = x; a.hx = hx; a.species = species; a.w = w; a.hw = hw; a.gy = gy; a.partial = (float*)scratch;
  a.N = N; a.C = C; a.S = S; a.ir_mul = ir_mul;
  cudaStream_t st = (cudaStream_t)stream;
  if (dgy && N > 0) {
    a.y = dgy;
    if (int rc = launch_node<Dual, 0>(target_lmax, a, st)) return rc;
  }
  if (dx && N > 0) {
    a.gx = dx;
    if (int rc = launch_node<Dual, 1>(target_lmax, a, st)) return rc;
  }
  if (dw) return launch_wgrad<Dual>(target_lmax, a, dw, st);
  return ICTC_OK;
}

}  // extern "C"
