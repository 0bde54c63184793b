// Radial gate MLP (num_basis -> 64 -> 64 -> 64 -> P*C, bias-free, SiLU * 1.679 between layers) on the
// tensor cores, forward and input-gradient, one kernel each.
//
// Reference: the `fc` stack of the interaction block (mace_ictc/models/mace/layers.py:825-835) evaluated by
// F.linear / torch.mm per layer (ictc_o3/ops/streamed_gate_message.py:112-116 tiles its last layer).
// The reference forbids TF32 (ictc_o3/backends/k100/fp32_policy.py:6-11), so every product here is an
// error-compensated split: x = x_big + x_small with both parts representable in TF32, and
// a*b ~= a_small*b_big + a_big*b_small + a_big*b_big accumulated in fp32 (relative error ~2^-21, checked
// against an fp64 evaluation in the tests).  The three partial products are `mma.sync.m16n8k8` TF32
// instructions.
//
// Work split: a block owns a tile of 128 edges, each of its 8 warps owns 16 rows and carries them
// through all four layers, so activations never leave the warp (registers -> a warp-private shared
// buffer -> A fragments of the next layer).  The three small weight matrices stay in shared memory for
// the life of the (persistent) block; the wide last layer is streamed through shared memory in 64-column
// chunks, split into big/small parts while it is staged.  The forward pass can store the three hidden
// pre-activations for the backward kernel, which then needs no recomputation.
#include "ictc_common.cuh"

namespace ictc {

constexpr int kH = 64;                 // hidden width
constexpr int kTileRows = 128;         // rows per block tile
constexpr int kMlpWarps = 8;
constexpr int kWS = 72;                // row stride of weight tiles in float2 {big, small}
constexpr int kAS = 72;                // row stride of the warp activation buffer in floats
constexpr float kSiluScale = 1.6791767923989418f;

__device__ __forceinline__ float to_tf32(float x) {
  unsigned r;
  asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(r) : "f"(x));
  return __uint_as_float(r);
}
__device__ __forceinline__ float2 split_tf32(float x) {
  const float big = to_tf32(x);
  return make_float2(big, to_tf32(x - big));
}
__device__ __forceinline__ void mma_tf32(float (&c)[4], const float (&a)[4], float b0, float b1) {
  asm("mma.sync.aligned.m16n8k8.row.col.f32.tf32.tf32.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(__float_as_uint(a[0])), "r"(__float_as_uint(a[1])), "r"(__float_as_uint(a[2])),
                 "r"(__float_as_uint(a[3])), "r"(__float_as_uint(b0)), "r"(__float_as_uint(b1)));
}
__device__ __forceinline__ float silu_s(float v) { return v / (1.f + expf(-v)) * kSiluScale; }
__device__ __forceinline__ float dsilu_s(float v) {
  const float s = 1.f / (1.f + expf(-v));
  return kSiluScale * s * (1.f + v * (1.f - s));
}

// A fragment (16 x 8 slice of the activations, k-slice `ks`) from a warp buffer [16][kAS], optionally
// through the activation.  Within a k-slice lane t holds the k indices 2t and 2t+1 (any k order is
// valid as long as B uses the same one), so the two values are adjacent in memory.
template <bool ACT>
__device__ __forceinline__ void load_a(const float* buf, int ks, int g, int t, float (&big)[4], float (&small)[4]) {
  const float2 lo = *reinterpret_cast<const float2*>(buf + g * kAS + ks * 8 + 2 * t);
  const float2 hi = *reinterpret_cast<const float2*>(buf + (g + 8) * kAS + ks * 8 + 2 * t);
  float v[4] = {lo.x, hi.x, lo.y, hi.y};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float x = ACT ? silu_s(v[i]) : v[i];
    big[i] = to_tf32(x);
    small[i] = to_tf32(x - big[i]);
  }
}

// acc[nt] += A(16 x K) * W^T for NT column tiles of 8; W tile in shared memory as [n][k] float2 {big, small}.
template <int NT, int KS, bool ACT>
__device__ __forceinline__ void warp_gemm(const float* abuf, const float2* w, int g, int t, float (&acc)[NT][4]) {
#pragma unroll
  for (int ks = 0; ks < KS; ++ks) {
    float ab[4], as[4];
    load_a<ACT>(abuf, ks, g, t, ab, as);
    float4 b[NT];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) b[nt] = *reinterpret_cast<const float4*>(w + (nt * 8 + g) * kWS + ks * 8 + 2 * t);
    // three passes over independent accumulators: small*big, big*small, big*big
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) mma_tf32(acc[nt], as, b[nt].x, b[nt].z);
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) mma_tf32(acc[nt], ab, b[nt].y, b[nt].w);
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) mma_tf32(acc[nt], ab, b[nt].x, b[nt].z);
  }
}

template <int NT> __device__ __forceinline__ void zero_acc(float (&acc)[NT][4]) {
#pragma unroll
  for (int nt = 0; nt < NT; ++nt)
#pragma unroll
    for (int i = 0; i < 4; ++i) acc[nt][i] = 0.f;
}

// C fragments (16 x 64) -> warp buffer [16][kAS]
__device__ __forceinline__ void store_c(float* buf, int g, int t, const float (&acc)[8][4]) {
#pragma unroll
  for (int nt = 0; nt < 8; ++nt) {
    *reinterpret_cast<float2*>(buf + g * kAS + nt * 8 + 2 * t) = make_float2(acc[nt][0], acc[nt][1]);
    *reinterpret_cast<float2*>(buf + (g + 8) * kAS + nt * 8 + 2 * t) = make_float2(acc[nt][2], acc[nt][3]);
  }
}

// Stages a [rows x 64] weight tile W[n][k] (row stride ld floats, k contiguous) into shared {big, small}.
__device__ __forceinline__ void stage_weight(float2* dst, const float* src, int rows, int64_t ld, int kvalid) {
  for (int idx = threadIdx.x; idx < rows * kH; idx += blockDim.x) {
    const int n = idx / kH, k = idx % kH;
    const float v = k < kvalid ? src[n * ld + k] : 0.f;
    dst[n * kWS + k] = split_tf32(v);
  }
}

// Copies a [64 x 64] tile of pre-split weights (float2 {big, small}, row stride ld elements) into shared
// memory with 16-byte asynchronous copies.
__device__ __forceinline__ void stage_split_async(float2* dst, const float2* src, int64_t ld) {
  for (int idx = threadIdx.x; idx < kH * (kH / 2); idx += blockDim.x) {
    const int n = idx / (kH / 2), k = (idx % (kH / 2)) * 2;
    const unsigned d = static_cast<unsigned>(__cvta_generic_to_shared(dst + n * kWS + k));
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(d), "l"(src + n * ld + k) : "memory");
  }
  asm volatile("cp.async.commit_group;" ::: "memory");
}
__device__ __forceinline__ void wait_async() { asm volatile("cp.async.wait_group 0;" ::: "memory"); }

struct MlpArgs {
  const float* rb;      // [E, nb]
  const float* w0;      // [64, nb]
  const float* w1;      // [64, 64]
  const float* w2;      // [64, 64]
  const float2* w3;     // pre-split {big, small}: forward [nout, 64]; backward W3^T [64, nout]
  float* gates;         // [E, nout]
  float* z1;            // [E, 64] pre-activations (optional in forward, required in backward)
  float* z2;
  float* z3;
  const float* dgates;  // [rows, nout]
  const int64_t* pair_a;  // optional: row u of the MLP reads dgates[pair_a[u]] + dgates[pair_b[u]] (pair_b < 0: none)
  const int64_t* pair_b;
  float* drb;           // [E, nb]
  const float* da3;     // backward, optional [E, 64]: gradient of the last hidden activation computed elsewhere
  int64_t E;
  int nb, nout;
};

// ------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(kMlpWarps * 32, 1) radial_mlp_forward_kernel(MlpArgs a) {
  extern __shared__ __align__(16) unsigned char mlp_smem[];
  float2* w0s = reinterpret_cast<float2*>(mlp_smem);                // [64][kWS] (k < nb used)
  float2* w1s = w0s + kH * kWS;
  float2* w2s = w1s + kH * kWS;
  float2* w3s = w2s + kH * kWS;                                     // 2 x [64][kWS]
  float* act = reinterpret_cast<float*>(w3s + 2 * kH * kWS);        // [warps][16][kAS]
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
  float* mine = act + warp * 16 * kAS;
  stage_weight(w0s, a.w0, kH, a.nb, a.nb);
  stage_weight(w1s, a.w1, kH, kH, kH);
  stage_weight(w2s, a.w2, kH, kH, kH);
  __syncthreads();
  const int chunks = a.nout / kH;
  const int64_t tiles = (a.E + kTileRows - 1) / kTileRows;
  for (int64_t tile = blockIdx.x; tile < tiles; tile += gridDim.x) {
    const int64_t row0 = tile * kTileRows + warp * 16;
    const int64_t r_lo = row0 + g, r_hi = row0 + g + 8;
    const bool ok_lo = r_lo < a.E, ok_hi = r_hi < a.E;
    // first chunk of the last layer is staged while the hidden layers run
    if (a.gates) stage_split_async(w3s, a.w3, kH);
    // ---- layer 0: radial basis rows into the warp buffer (zero padded to 8 columns)
    for (int idx = lane; idx < 16 * 8; idx += 32) {
      const int r = idx / 8, k = idx % 8;
      const int64_t row = row0 + r;
      mine[r * kAS + k] = (row < a.E && k < a.nb) ? a.rb[row * a.nb + k] : 0.f;
    }
    __syncwarp();
    float acc[8][4];
    zero_acc<8>(acc);
    warp_gemm<8, 1, false>(mine, w0s, g, t, acc);
    __syncwarp();
    if (a.z1) {
#pragma unroll
      for (int nt = 0; nt < 8; ++nt) {
        if (ok_lo) *reinterpret_cast<float2*>(a.z1 + r_lo * kH + nt * 8 + 2 * t) = make_float2(acc[nt][0], acc[nt][1]);
        if (ok_hi) *reinterpret_cast<float2*>(a.z1 + r_hi * kH + nt * 8 + 2 * t) = make_float2(acc[nt][2], acc[nt][3]);
      }
    }
    store_c(mine, g, t, acc);
    __syncwarp();
    // ---- layer 1
    zero_acc<8>(acc);
    warp_gemm<8, 8, true>(mine, w1s, g, t, acc);
    __syncwarp();
    if (a.z2) {
#pragma unroll
      for (int nt = 0; nt < 8; ++nt) {
        if (ok_lo) *reinterpret_cast<float2*>(a.z2 + r_lo * kH + nt * 8 + 2 * t) = make_float2(acc[nt][0], acc[nt][1]);
        if (ok_hi) *reinterpret_cast<float2*>(a.z2 + r_hi * kH + nt * 8 + 2 * t) = make_float2(acc[nt][2], acc[nt][3]);
      }
    }
    store_c(mine, g, t, acc);
    __syncwarp();
    // ---- layer 2
    zero_acc<8>(acc);
    warp_gemm<8, 8, true>(mine, w2s, g, t, acc);
    __syncwarp();
    if (a.z3) {
#pragma unroll
      for (int nt = 0; nt < 8; ++nt) {
        if (ok_lo) *reinterpret_cast<float2*>(a.z3 + r_lo * kH + nt * 8 + 2 * t) = make_float2(acc[nt][0], acc[nt][1]);
        if (ok_hi) *reinterpret_cast<float2*>(a.z3 + r_hi * kH + nt * 8 + 2 * t) = make_float2(acc[nt][2], acc[nt][3]);
      }
    }
    if (!a.gates) continue;                              // hidden layers only: the wide layer runs elsewhere
    store_c(mine, g, t, acc);
    __syncwarp();
    // ---- layer 3: A fragments of the last hidden activation stay in registers for all chunks
    float ab[8][4], as[8][4];
#pragma unroll
    for (int ks = 0; ks < 8; ++ks) load_a<true>(mine, ks, g, t, ab[ks], as[ks]);
    wait_async();
    __syncthreads();                                     // chunk 0 staged by everyone
    for (int ch = 0; ch < chunks; ++ch) {
      const float2* wc = w3s + (ch & 1) * kH * kWS;
      if (ch + 1 < chunks) stage_split_async(w3s + ((ch + 1) & 1) * kH * kWS, a.w3 + int64_t(ch + 1) * kH * kH, kH);
      zero_acc<8>(acc);
#pragma unroll
      for (int ks = 0; ks < 8; ++ks) {
        float4 b[8];
#pragma unroll
        for (int nt = 0; nt < 8; ++nt) b[nt] = *reinterpret_cast<const float4*>(wc + (nt * 8 + g) * kWS + ks * 8 + 2 * t);
#pragma unroll
        for (int nt = 0; nt < 8; ++nt) mma_tf32(acc[nt], as[ks], b[nt].x, b[nt].z);
#pragma unroll
        for (int nt = 0; nt < 8; ++nt) mma_tf32(acc[nt], ab[ks], b[nt].y, b[nt].w);
#pragma unroll
        for (int nt = 0; nt < 8; ++nt) mma_tf32(acc[nt], ab[ks], b[nt].x, b[nt].z);
      }
#pragma unroll
      for (int nt = 0; nt < 8; ++nt) {
        const int col = ch * kH + nt * 8 + 2 * t;
        if (ok_lo) *reinterpret_cast<float2*>(a.gates + r_lo * a.nout + col) = make_float2(acc[nt][0], acc[nt][1]);
        if (ok_hi) *reinterpret_cast<float2*>(a.gates + r_hi * a.nout + col) = make_float2(acc[nt][2], acc[nt][3]);
      }
      wait_async();
      __syncthreads();                                   // next chunk staged, this one free to overwrite
    }
  }
}

// ------------------------------------------------------------------------------------------------
// drb = d(gates)/d(rb)^T dgates, with the stored pre-activations.  Weight tiles are the transposes:
// w3 = W3^T [64][nout], w2 = W2^T, w1 = W1^T (all [n = input unit][k = output unit]), w0 = W0^T [nb][64].
__global__ void __launch_bounds__(kMlpWarps * 32, 1) radial_mlp_backward_kernel(MlpArgs a) {
  extern __shared__ __align__(16) unsigned char mlp_smem[];
  float2* w0s = reinterpret_cast<float2*>(mlp_smem);                // [8][kWS]  (n = basis index, k = hidden)
  float2* w1s = w0s + 8 * kWS;
  float2* w2s = w1s + kH * kWS;
  float2* w3s = w2s + kH * kWS;                                     // 2 x [64][kWS]
  float* act = reinterpret_cast<float*>(w3s + 2 * kH * kWS);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
  float* mine = act + warp * 16 * kAS;
  for (int idx = threadIdx.x; idx < 8 * kH; idx += blockDim.x) {
    const int n = idx / kH, k = idx % kH;
    w0s[n * kWS + k] = split_tf32(n < a.nb ? a.w0[n * kH + k] : 0.f);
  }
  stage_weight(w1s, a.w1, kH, kH, kH);
  stage_weight(w2s, a.w2, kH, kH, kH);
  __syncthreads();
  const int chunks = a.nout / kH;
  const int64_t tiles = (a.E + kTileRows - 1) / kTileRows;
  for (int64_t tile = blockIdx.x; tile < tiles; tile += gridDim.x) {
    const int64_t row0 = tile * kTileRows + warp * 16;
    const int64_t r_lo = row0 + g, r_hi = row0 + g + 8;
    const bool ok_lo = r_lo < a.E, ok_hi = r_hi < a.E;
    const int64_t c_lo = ok_lo ? r_lo : 0, c_hi = ok_hi ? r_hi : 0;   // clamped rows for loads
    const int64_t da_lo = a.pair_a ? a.pair_a[c_lo] : c_lo, da_hi = a.pair_a ? a.pair_a[c_hi] : c_hi;
    const int64_t db_lo = a.pair_b ? a.pair_b[c_lo] : -1, db_hi = a.pair_b ? a.pair_b[c_hi] : -1;
    float acc[8][4];
    zero_acc<8>(acc);
    if (a.da3) {
#pragma unroll
      for (int nt = 0; nt < 8; ++nt) {
        const int col = nt * 8 + 2 * t;
        const float2 lo = ok_lo ? *reinterpret_cast<const float2*>(a.da3 + r_lo * kH + col) : make_float2(0.f, 0.f);
        const float2 hi = ok_hi ? *reinterpret_cast<const float2*>(a.da3 + r_hi * kH + col) : make_float2(0.f, 0.f);
        acc[nt][0] = lo.x; acc[nt][1] = lo.y; acc[nt][2] = hi.x; acc[nt][3] = hi.y;
      }
    } else {
      stage_split_async(w3s, a.w3, a.nout);
      wait_async();
      __syncthreads();
    }
    // ---- da3 = dgates @ W3 : K = nout streamed in 64-wide chunks, A fragments straight from global
    for (int ch = 0; ch < (a.da3 ? 0 : chunks); ++ch) {
      const float2* wc = w3s + (ch & 1) * kH * kWS;
      if (ch + 1 < chunks) stage_split_async(w3s + ((ch + 1) & 1) * kH * kWS, a.w3 + (ch + 1) * kH, a.nout);
#pragma unroll
      for (int ks = 0; ks < 8; ++ks) {
        const int col = ch * kH + ks * 8 + 2 * t;
        float2 lo = *reinterpret_cast<const float2*>(a.dgates + da_lo * a.nout + col);
        float2 hi = *reinterpret_cast<const float2*>(a.dgates + da_hi * a.nout + col);
        if (db_lo >= 0) {
          const float2 o = *reinterpret_cast<const float2*>(a.dgates + db_lo * a.nout + col);
          lo.x += o.x;
          lo.y += o.y;
        }
        if (db_hi >= 0) {
          const float2 o = *reinterpret_cast<const float2*>(a.dgates + db_hi * a.nout + col);
          hi.x += o.x;
          hi.y += o.y;
        }
        if (!ok_lo) lo = make_float2(0.f, 0.f);
        if (!ok_hi) hi = make_float2(0.f, 0.f);
        const float v[4] = {lo.x, hi.x, lo.y, hi.y};
        float ab[4], as[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          ab[i] = to_tf32(v[i]);
          as[i] = to_tf32(v[i] - ab[i]);
        }
        float4 b[8];
#pragma unroll
        for (int nt = 0; nt < 8; ++nt) b[nt] = *reinterpret_cast<const float4*>(wc + (nt * 8 + g) * kWS + ks * 8 + 2 * t);
#pragma unroll
        for (int nt = 0; nt < 8; ++nt) mma_tf32(acc[nt], as, b[nt].x, b[nt].z);
#pragma unroll
        for (int nt = 0; nt < 8; ++nt) mma_tf32(acc[nt], ab, b[nt].y, b[nt].w);
#pragma unroll
        for (int nt = 0; nt < 8; ++nt) mma_tf32(acc[nt], ab, b[nt].x, b[nt].z);
      }
      __syncthreads();
    }
    // ---- through the three hidden layers: d z = d a * silu'(z), d a_prev = d z @ W
    const float* zs[3] = {a.z3, a.z2, a.z1};
    const float2* ws[2] = {w2s, w1s};
#pragma unroll
    for (int layer = 0; layer < 3; ++layer) {
#pragma unroll
      for (int nt = 0; nt < 8; ++nt) {
        const int col = nt * 8 + 2 * t;
        const float2 zl = *reinterpret_cast<const float2*>(zs[layer] + c_lo * kH + col);
        const float2 zh = *reinterpret_cast<const float2*>(zs[layer] + c_hi * kH + col);
        acc[nt][0] *= dsilu_s(zl.x);
        acc[nt][1] *= dsilu_s(zl.y);
        acc[nt][2] *= dsilu_s(zh.x);
        acc[nt][3] *= dsilu_s(zh.y);
      }
      __syncwarp();
      store_c(mine, g, t, acc);
      __syncwarp();
      if (layer < 2) {
        zero_acc<8>(acc);
        warp_gemm<8, 8, false>(mine, ws[layer], g, t, acc);
      }
    }
    // ---- drb = dz1 @ W0 : one column tile of 8
    float out[1][4];
    zero_acc<1>(out);
    warp_gemm<1, 8, false>(mine, w0s, g, t, out);
    __syncwarp();
    const int col = 2 * t;
    if (ok_lo) {
      if (col < a.nb) a.drb[r_lo * a.nb + col] = out[0][0];
      if (col + 1 < a.nb) a.drb[r_lo * a.nb + col + 1] = out[0][1];
    }
    if (ok_hi) {
      if (col < a.nb) a.drb[r_hi * a.nb + col] = out[0][2];
      if (col + 1 < a.nb) a.drb[r_hi * a.nb + col + 1] = out[0][3];
    }
  }
}

static int mlp_check(int64_t E, int nb, int nout) {
  if (E < 0 || nb < 1 || nb > 8 || nout < kH || nout % kH) {
    set_error("radial mlp: needs 1..8 basis functions and an output width that is a multiple of 64 (got %d, %d)", nb,
              nout);
    return ICTC_ERR_BAD_SPEC;
  }
  return ICTC_OK;
}

static int mlp_grid() {
  int dev = 0, sms = 148;
  if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  return sms;
}

}  // namespace ictc

using namespace ictc;

__global__ void split_tf32_kernel(int64_t n, const float* __restrict__ src, float2* dst) {
  const int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i < n) dst[i] = split_tf32(src[i]);
}

extern "C" {

int ictc_split_tf32(int64_t n, const float* src, float* dst_pairs, void* stream) {
  if (n < 0 || (n > 0 && (!src || !dst_pairs))) { set_error("split_tf32: invalid arguments"); return ICTC_ERR_BAD_ARG; }
  if (n == 0) return ICTC_OK;
  split_tf32_kernel<<<(unsigned)((n + 255) / 256), 256, 0, (cudaStream_t)stream>>>(n, src,
                                                                                reinterpret_cast<float2*>(dst_pairs));
  return finish_launch("split_tf32");
}

int ictc_radial_mlp_forward(int64_t num_edges, int num_basis, int num_out, const float* rb, const float* w0,
                            const float* w1, const float* w2, const float* w3_split, float* gates, float* z1,
                            float* z2, float* z3, void* stream) {
  if (int rc = mlp_check(num_edges, num_basis, num_out)) return rc;
  if (num_edges == 0) return ICTC_OK;
  if (!rb || !w0 || !w1 || !w2 || (gates && !w3_split) || (!gates && !z3)) {
    set_error("radial mlp: NULL buffer");
    return ICTC_ERR_BAD_ARG;
  }
  MlpArgs a{};
  a.rb = rb; a.w0 = w0; a.w1 = w1; a.w2 = w2; a.w3 = reinterpret_cast<const float2*>(w3_split); a.gates = gates; a.z1 = z1; a.z2 = z2; a.z3 = z3;
  a.E = num_edges; a.nb = num_basis; a.nout = num_out;
  const size_t smem = size_t(5 * kH * kWS) * sizeof(float2) + size_t(kMlpWarps * 16 * kAS) * sizeof(float);
  static const cudaError_t attr = cudaFuncSetAttribute(radial_mlp_forward_kernel,
                                                       cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (attr != cudaSuccess) { set_error("radial mlp smem: %s", cudaGetErrorString(attr)); return ICTC_ERR_LAUNCH; }
  const int64_t tiles = (num_edges + kTileRows - 1) / kTileRows;
  const int grid = (int)(tiles < mlp_grid() ? tiles : mlp_grid());
  radial_mlp_forward_kernel<<<grid, kMlpWarps * 32, smem, (cudaStream_t)stream>>>(a);
  return finish_launch("radial_mlp_forward");
}

int ictc_radial_mlp_backward_paired(int64_t num_rows, int num_basis, int num_out, const float* dgates,
                                    const int64_t* pair_a, const int64_t* pair_b, const float* w0t, const float* w1t,
                                    const float* w2t, const float* w3t_split, const float* z1, const float* z2,
                                    const float* z3, float* drb, void* stream);

int ictc_radial_mlp_backward(int64_t num_edges, int num_basis, int num_out, const float* dgates, const float* w0t,
                             const float* w1t, const float* w2t, const float* w3t_split, const float* z1,
                             const float* z2, const float* z3, float* drb, void* stream) {
  return ictc_radial_mlp_backward_paired(num_edges, num_basis, num_out, dgates, nullptr, nullptr, w0t, w1t, w2t,
                                         w3t_split, z1, z2, z3, drb, stream);
}

static int mlp_backward_launch(int64_t num_edges, int num_basis, int num_out, const float* dgates, const float* da3,
                               const int64_t* pair_a, const int64_t* pair_b, const float* w0t, const float* w1t,
                               const float* w2t, const float* w3t_split, const float* z1, const float* z2,
                               const float* z3, float* drb, void* stream);

int ictc_radial_mlp_backward_paired(int64_t num_edges, int num_basis, int num_out, const float* dgates,
                                    const int64_t* pair_a, const int64_t* pair_b, const float* w0t, const float* w1t,
                                    const float* w2t, const float* w3t_split, const float* z1, const float* z2,
                                    const float* z3, float* drb, void* stream) {
  if (!dgates || !w3t_split) { set_error("radial mlp backward: NULL buffer"); return ICTC_ERR_BAD_ARG; }
  return mlp_backward_launch(num_edges, num_basis, num_out, dgates, nullptr, pair_a, pair_b, w0t, w1t, w2t, w3t_split,
                             z1, z2, z3, drb, stream);
}

int ictc_radial_mlp_hidden_forward(int64_t num_edges, int num_basis, const float* rb, const float* w0, const float* w1,
                                   const float* w2, float* z1, float* z2, float* z3, void* stream) {
  return ictc_radial_mlp_forward(num_edges, num_basis, kH, rb, w0, w1, w2, nullptr, nullptr, z1, z2, z3, stream);
}

int ictc_radial_mlp_hidden_backward(int64_t num_edges, int num_basis, const float* da3, const float* w0t,
                                    const float* w1t, const float* w2t, const float* z1, const float* z2,
                                    const float* z3, float* drb, void* stream) {
  if (!da3) { set_error("radial mlp hidden backward: NULL buffer"); return ICTC_ERR_BAD_ARG; }
  return mlp_backward_launch(num_edges, num_basis, kH, nullptr, da3, nullptr, nullptr, w0t, w1t, w2t, nullptr, z1, z2,
                             z3, drb, stream);
}

static int mlp_backward_launch(int64_t num_edges, int num_basis, int num_out, const float* dgates, const float* da3,
                               const int64_t* pair_a, const int64_t* pair_b, const float* w0t, const float* w1t,
                               const float* w2t, const float* w3t_split, const float* z1, const float* z2,
                               const float* z3, float* drb, void* stream) {
  if (int rc = mlp_check(num_edges, num_basis, num_out)) return rc;
  if (num_edges == 0) return ICTC_OK;
  if (!w0t || !w1t || !w2t || !z1 || !z2 || !z3 || !drb) {
    set_error("radial mlp backward: NULL buffer");
    return ICTC_ERR_BAD_ARG;
  }
  MlpArgs a{};
  a.w0 = w0t; a.w1 = w1t; a.w2 = w2t; a.w3 = reinterpret_cast<const float2*>(w3t_split); a.dgates = dgates; a.drb = drb;
  a.da3 = da3;
  a.pair_a = pair_a; a.pair_b = pair_b;
  a.z1 = const_cast<float*>(z1); a.z2 = const_cast<float*>(z2); a.z3 = const_cast<float*>(z3);
  a.E = num_edges; a.nb = num_basis; a.nout = num_out;
  const size_t smem = size_t(8 * kWS + 4 * kH * kWS) * sizeof(float2) + size_t(kMlpWarps * 16 * kAS) * sizeof(float);
  static const cudaError_t attr = cudaFuncSetAttribute(radial_mlp_backward_kernel,
                                                       cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (attr != cudaSuccess) { set_error("radial mlp smem: %s", cudaGetErrorString(attr)); return ICTC_ERR_LAUNCH; }
  const int64_t tiles = (num_edges + kTileRows - 1) / kTileRows;
  const int grid = (int)(tiles < mlp_grid() ? tiles : mlp_grid());
  radial_mlp_backward_kernel<<<grid, kMlpWarps * 32, smem, (cudaStream_t)stream>>>(a);
  return finish_launch("radial_mlp_backward");
}

}  // extern "C"
