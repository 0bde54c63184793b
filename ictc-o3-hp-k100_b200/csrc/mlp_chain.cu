// Hidden layers of the radial gate MLP (num_basis -> 64 -> 64 -> 64, bias-free, scaled SiLU) as a chain through
// tensor memory: forward (pre-activations z1..z3) and input gradient (drb from da3 = dE/d silu(z3)).
//
// Reference: the `fc` stack of the interaction block (mace_ictc/models/mace/layers.py:825-835) evaluated by
// F.linear per layer, and its autograd backward.  TF32 is forbidden by the reference
// (ictc_o3/backends/k100/fp32_policy.py:6-11): the 64 x 64 layers are three-term split TF32 tcgen05.mma products,
// the narrow first / last layer (K or N = num_basis <= 8) is plain fp32 FMA.
//
// One persistent CTA per SM keeps two 128-row tiles in flight (two TMEM slots), so that the serial chain
// MMA -> tcgen05.ld -> activation -> tcgen05.st -> MMA of one tile overlaps with the other tile's.
//   warp 1       allocates TMEM and issues the MMAs of both slots in a fixed order;
//   warps 2-9    chain threads of slot 0, warps 10-17 of slot 1: thread = (row, half of the 64 hidden units);
//                they read the accumulator, store the pre-activation (forward) or multiply by silu'(z) (backward),
//                split the next A operand and write it back to TMEM.
// TMEM per slot (192 columns): A big [0,64) | A small [64,128) | accumulator [128,192).
// The weights of the two 64 x 64 layers stay in shared memory in the B-operand layout (64 KB), the narrow layer's
// as a plain [64][8] table.  Every mbarrier wait is bounded and reports through the library's status word.
#include "tc05.cuh"

namespace ictc {
namespace chain {

using namespace tc;

constexpr int kThreads = 18 * 32;
constexpr int kSlotCols = 192;
constexpr int kSlotWarps = 8;
constexpr int kTableBytes = 64 * 8 * 4;            // narrow layer [64][8]
constexpr int kXchgBytes = 2 * kRows * 8 * 4;       // partial drb rows of both slots
constexpr int kBarOffset = 2 * kWStageBytes + kTableBytes + kXchgBytes;
constexpr int kSmem = kBarOffset + 256;            // W(a) | W(b) | W0 table | drb exchange | barriers

struct Args {
  const float* in;     // forward: rb [E, nb]; backward: da3 [E, 64]
  const float* w0;     // [64, nb] (forward: W0; backward: W0 as well, used as dz1 @ W0)
  const float* wa;     // packed 64 x 64 operand of the first MMA layer (forward: W1, backward: W2 transposed use)
  const float* wb;     // packed operand of the second MMA layer (forward: W2, backward: W1 transposed use)
  float* z1;           // forward outputs / backward inputs [E, 64]
  float* z2;
  float* z3;
  float* drb;          // backward output [E, nb]
  const int64_t* rows; // optional row index: forward reads rb[rows[r]], backward writes / adds to drb[rows[r]]
  const int64_t* in_a; // backward, optional: row r starts from in[in_a[r]] + in[in_b[r]] (in_b[r] < 0: first term only)
  const int64_t* in_b;
  int accumulate;      // backward: drb[...] += instead of =
  const int64_t* limit; // optional device scalar: only min(E, *limit) rows are processed (recorded graphs)
  int64_t E;
  int nb;
  int* status;
};

struct Barriers {
  unsigned long long a_ready[2], h_full[2], w_full, x_full[8], x_free[8];
  unsigned tmem_base;
  volatile int failed;   // polled inside wait loops by other warps: every read must go to shared memory
};

__device__ __forceinline__ void give_up(Barriers* b, int* status, int code) {
  b->failed = 1;
  if (status) atomicExch(status, code);
}
__device__ __forceinline__ void stg256(float* p, const float* v) {
  asm volatile("st.global.v8.f32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"l"(p), "f"(v[0]), "f"(v[1]), "f"(v[2]),
               "f"(v[3]), "f"(v[4]), "f"(v[5]), "f"(v[6]), "f"(v[7])
               : "memory");
}

// Common prologue: barriers, TMEM, weights.  Returns the TMEM base address.
__device__ __forceinline__ unsigned setup(const Args& a, unsigned char* smem, Barriers* bar, float* w0s) {
  const int warp = threadIdx.x >> 5;
  if (threadIdx.x == 0) {
    for (int i = 0; i < 2; ++i) {
      mbar_init(saddr(&bar->a_ready[i]), kSlotWarps * 32);
      mbar_init(saddr(&bar->h_full[i]), 1);
    }
    mbar_init(saddr(&bar->w_full), 1);
    for (int i = 0; i < 8; ++i) {
      mbar_init(saddr(&bar->x_full[i]), 32);
      mbar_init(saddr(&bar->x_free[i]), 32);
    }
    bar->failed = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    mbar_expect_tx(saddr(&bar->w_full), 2 * kWStageBytes);
    bulk_g2s(saddr(smem), a.wa, kWStageBytes, saddr(&bar->w_full));
    bulk_g2s(saddr(smem + kWStageBytes), a.wb, kWStageBytes, saddr(&bar->w_full));
  }
  for (int i = threadIdx.x; i < 64 * 8; i += blockDim.x) {
    const int n = i >> 3, k = i & 7;
    w0s[i] = k < a.nb ? a.w0[n * a.nb + k] : 0.f;
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(saddr(&bar->tmem_base)),
                 "r"(512u)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  return bar->tmem_base;
}

__device__ __forceinline__ void teardown(unsigned tmem) {
  tc_fence_before();
  __syncthreads();
  if ((threadIdx.x >> 5) == 1) {
    __syncwarp();
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(512u) : "memory");
  }
}

// MMA issue of both kernels: per pair of tiles, layer A for slot 0 and 1, then layer B for slot 0 and 1.
__device__ __forceinline__ void mma_loop(const Args& a, Barriers* bar, unsigned char* smem, unsigned tmem,
                                         int64_t my_tiles) {
  if (!mbar_wait(saddr(&bar->w_full), 0)) { give_up(bar, a.status, 41); return; }
  unsigned phase[2] = {0, 0};
  for (int64_t i = 0; i < my_tiles && !bar->failed; i += 2) {
    for (int layer = 0; layer < 2; ++layer) {
      const unsigned w_big = saddr(smem + layer * kWStageBytes), w_small = w_big + kWPartBytes;
      for (int s = 0; s < 2; ++s) {
        if (i + s >= my_tiles) continue;
        if (!mbar_wait(saddr(&bar->a_ready[s]), phase[s] & 1)) { give_up(bar, a.status, 42); return; }
        ++phase[s];
        tc_fence_after();
        const unsigned base = tmem + s * kSlotCols;
        issue_block(base + 2 * kK, base, w_big, w_small, true);
        umma_commit(saddr(&bar->h_full[s]));
      }
    }
  }
}

// ------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(kThreads, 1) mlp_chain_forward_kernel(Args a) {
  extern __shared__ __align__(128) unsigned char chain_smem[];
  float* w0s = reinterpret_cast<float*>(chain_smem + 2 * kWStageBytes);
  Barriers* bar = reinterpret_cast<Barriers*>(chain_smem + kBarOffset);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t nrows = a.limit ? (ldg(a.limit) < a.E ? ldg(a.limit) : a.E) : a.E;
  const int64_t tiles = (nrows + kRows - 1) / kRows;
  const int64_t my_tiles = blockIdx.x < tiles ? (tiles - blockIdx.x + gridDim.x - 1) / gridDim.x : 0;
  const unsigned tmem = setup(a, chain_smem, bar, w0s);

  if (warp == 1) {
    if (lane == 0) mma_loop(a, bar, chain_smem, tmem, my_tiles);
  } else if (warp >= 2) {
    const int s = (warp - 2) / kSlotWarps, q = warp & 3, half = ((warp - 2) % kSlotWarps) >> 2;
    const int row = q * 32 + lane;
    const unsigned lane_base = tmem + (unsigned(q * 32) << 16) + s * kSlotCols;
    const unsigned t_big = lane_base + half * 32, t_acc = lane_base + 2 * kK + half * 32;
    unsigned phase = 0;
    for (int64_t i = s; i < my_tiles; i += 2) {
      const int64_t g = (blockIdx.x + i * gridDim.x) * kRows + row;
      const bool valid = g < nrows;
      // ---- layer 0 in fp32: z1[n] = sum_k rb[k] W0[n][k] for this thread's 32 units
      float rb[8];
#pragma unroll
      const int64_t src_row = (valid && a.rows) ? __ldg(reinterpret_cast<const long long*>(a.rows + g)) : g;
#pragma unroll
      for (int k = 0; k < 8; ++k) rb[k] = (valid && k < a.nb) ? __ldg(a.in + src_row * a.nb + k) : 0.f;
      float x[32];
#pragma unroll
      for (int n = 0; n < 32; ++n) {
        const float4 wl = *reinterpret_cast<const float4*>(w0s + (half * 32 + n) * 8);
        const float4 wh = *reinterpret_cast<const float4*>(w0s + (half * 32 + n) * 8 + 4);
        float acc = rb[0] * wl.x;
        acc = fmaf(rb[1], wl.y, acc);
        acc = fmaf(rb[2], wl.z, acc);
        acc = fmaf(rb[3], wl.w, acc);
        acc = fmaf(rb[4], wh.x, acc);
        acc = fmaf(rb[5], wh.y, acc);
        acc = fmaf(rb[6], wh.z, acc);
        x[n] = fmaf(rb[7], wh.w, acc);
      }
      bool ok = true;
#pragma unroll 1
      for (int layer = 0; layer < 3; ++layer) {
        if (layer > 0) {
          if (bar->failed || !mbar_wait(saddr(&bar->h_full[s]), phase & 1)) { give_up(bar, a.status, 43); ok = false; break; }
          ++phase;
          tc_fence_after();
          tmem_ld32(t_acc, x);
        }
        if (valid) {
          float* z = (layer == 0 ? a.z1 : layer == 1 ? a.z2 : a.z3) + g * kK + half * 32;
#pragma unroll
          for (int j = 0; j < 4; ++j) stg256(z + j * 8, x + j * 8);
        }
        if (layer == 2) break;
#pragma unroll
        for (int n = 0; n < 32; ++n) x[n] = silu_s(x[n]);
        store_split_tmem(t_big, t_big + kK, x);
        tc_fence_before();
        mbar_arrive(saddr(&bar->a_ready[s]));
      }
      if (!ok) break;
      tc_fence_before();
    }
  }
  teardown(tmem);
}

// ------------------------------------------------------------------------------------------------
// backward: t3 = da3 * silu'(z3);  da2 = t3 @ W2;  t2 = da2 * silu'(z2);  da1 = t2 @ W1;  t1 = da1 * silu'(z1);
// drb = t1 @ W0.  (wa = W2 packed for x @ W2, wb = W1 packed for x @ W1.)
__global__ void __launch_bounds__(kThreads, 1) mlp_chain_backward_kernel(Args a) {
  extern __shared__ __align__(128) unsigned char chain_smem[];
  float* w0s = reinterpret_cast<float*>(chain_smem + 2 * kWStageBytes);
  float* xchg = w0s + 64 * 8;                                         // [128][8] partial drb of the upper half
  Barriers* bar = reinterpret_cast<Barriers*>(chain_smem + kBarOffset);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t nrows = a.limit ? (ldg(a.limit) < a.E ? ldg(a.limit) : a.E) : a.E;
  const int64_t tiles = (nrows + kRows - 1) / kRows;
  const int64_t my_tiles = blockIdx.x < tiles ? (tiles - blockIdx.x + gridDim.x - 1) / gridDim.x : 0;
  const unsigned tmem = setup(a, chain_smem, bar, w0s);

  if (warp == 1) {
    if (lane == 0) mma_loop(a, bar, chain_smem, tmem, my_tiles);
  } else if (warp >= 2) {
    const int s = (warp - 2) / kSlotWarps, q = warp & 3, half = ((warp - 2) % kSlotWarps) >> 2;
    const int row = q * 32 + lane;
    const unsigned lane_base = tmem + (unsigned(q * 32) << 16) + s * kSlotCols;
    const unsigned t_big = lane_base + half * 32, t_acc = lane_base + 2 * kK + half * 32;
    // the two warps that share rows (same slot and quarter) add their halves through shared memory
    const unsigned x_full = saddr(&bar->x_full[s * 4 + q]), x_free = saddr(&bar->x_free[s * 4 + q]);
    float* slot_x = xchg + (s * kRows + row) * 8;
    unsigned phase = 0, xphase = 0;
    for (int64_t i = s; i < my_tiles; i += 2) {
      const int64_t g = (blockIdx.x + i * gridDim.x) * kRows + row;
      const bool valid = g < nrows;
      float x[32], z[32];
      bool ok = true;
#pragma unroll 1
      for (int layer = 0; layer < 3; ++layer) {
        // silu'(z) of this layer: issue the loads before waiting for the accumulator
        if (valid) {
#pragma unroll
          for (int j = 0; j < 4; ++j)
            ldg256((layer == 0 ? a.z3 : layer == 1 ? a.z2 : a.z1) + g * kK + half * 32 + j * 8, z + j * 8);
        } else {
#pragma unroll
          for (int n = 0; n < 32; ++n) z[n] = 0.f;
        }
        if (layer == 0) {
          if (valid) {
            const int64_t ra = a.in_a ? ldg(a.in_a + g) : g;
#pragma unroll
            for (int j = 0; j < 4; ++j) ldg256(a.in + ra * kK + half * 32 + j * 8, x + j * 8);
            const int64_t rb = a.in_b ? ldg(a.in_b + g) : -1;
            if (rb >= 0) {
              float y[32];
#pragma unroll
              for (int j = 0; j < 4; ++j) ldg256(a.in + rb * kK + half * 32 + j * 8, y + j * 8);
#pragma unroll
              for (int n = 0; n < 32; ++n) x[n] += y[n];
            }
          } else {
#pragma unroll
            for (int n = 0; n < 32; ++n) x[n] = 0.f;
          }
        } else {
          if (bar->failed || !mbar_wait(saddr(&bar->h_full[s]), phase & 1)) { give_up(bar, a.status, 44); ok = false; break; }
          ++phase;
          tc_fence_after();
          tmem_ld32(t_acc, x);
        }
#pragma unroll
        for (int n = 0; n < 32; ++n) x[n] *= dsilu_s(z[n]);
        if (layer == 2) break;
        store_split_tmem(t_big, t_big + kK, x);
        tc_fence_before();
        mbar_arrive(saddr(&bar->a_ready[s]));
      }
      if (!ok) break;
      tc_fence_before();
      // ---- drb[k] = sum_n t1[n] W0[n][k]: partial sums over this thread's 32 units, halves added through smem
      float p[8];
#pragma unroll
      for (int k = 0; k < 8; ++k) p[k] = 0.f;
#pragma unroll
      for (int n = 0; n < 32; ++n) {
        const float4 wl = *reinterpret_cast<const float4*>(w0s + (half * 32 + n) * 8);
        const float4 wh = *reinterpret_cast<const float4*>(w0s + (half * 32 + n) * 8 + 4);
        p[0] = fmaf(x[n], wl.x, p[0]);
        p[1] = fmaf(x[n], wl.y, p[1]);
        p[2] = fmaf(x[n], wl.z, p[2]);
        p[3] = fmaf(x[n], wl.w, p[3]);
        p[4] = fmaf(x[n], wh.x, p[4]);
        p[5] = fmaf(x[n], wh.y, p[5]);
        p[6] = fmaf(x[n], wh.z, p[6]);
        p[7] = fmaf(x[n], wh.w, p[7]);
      }
      if (half == 1) {
        if (bar->failed || !mbar_wait(x_free, (xphase & 1) ^ 1u)) { give_up(bar, a.status, 45); break; }
        *reinterpret_cast<float4*>(slot_x) = make_float4(p[0], p[1], p[2], p[3]);
        *reinterpret_cast<float4*>(slot_x + 4) = make_float4(p[4], p[5], p[6], p[7]);
        mbar_arrive(x_full);
      } else {
        if (bar->failed || !mbar_wait(x_full, xphase & 1)) { give_up(bar, a.status, 46); break; }
        const float4 lo = *reinterpret_cast<const float4*>(slot_x), hi = *reinterpret_cast<const float4*>(slot_x + 4);
        mbar_arrive(x_free);
        p[0] += lo.x; p[1] += lo.y; p[2] += lo.z; p[3] += lo.w;
        p[4] += hi.x; p[5] += hi.y; p[6] += hi.z; p[7] += hi.w;
        if (valid) {
          float* o = a.drb + (a.rows ? __ldg(reinterpret_cast<const long long*>(a.rows + g)) : g) * a.nb;
#pragma unroll
          for (int k = 0; k < 8; ++k)
            if (k < a.nb) o[k] = a.accumulate ? o[k] + p[k] : p[k];
        }
      }
      ++xphase;
    }
  }
  teardown(tmem);
}

static int grid_size(int64_t rows) {
  int dev = 0, sms = 148;
  if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const int64_t tiles = (rows + kRows - 1) / kRows;
  return int(tiles < sms ? tiles : sms);
}

}  // namespace chain
}  // namespace ictc

using namespace ictc;

extern "C" {

int ictc_mlp_chain_forward(int64_t num_edges, int num_basis, const float* rb, const int64_t* rb_rows, const float* w0,
                           const float* w1_packed, const float* w2_packed, float* z1, float* z2, float* z3,
                           const int64_t* row_limit, void* stream) {
  if (num_edges < 0 || num_basis < 1 || num_basis > 8) {
    set_error("mlp chain: needs 1..8 basis functions (got %d)", num_basis);
    return ICTC_ERR_BAD_SPEC;
  }
  if (num_edges == 0) return ICTC_OK;
  if (!rb || !w0 || !w1_packed || !w2_packed || !z1 || !z2 || !z3) { set_error("mlp chain forward: NULL buffer"); return ICTC_ERR_BAD_ARG; }
  if ((reinterpret_cast<uintptr_t>(z1) | reinterpret_cast<uintptr_t>(z2) | reinterpret_cast<uintptr_t>(z3) |
       reinterpret_cast<uintptr_t>(w1_packed) | reinterpret_cast<uintptr_t>(w2_packed)) & 31) {
    set_error("mlp chain forward: buffers must be 32-byte aligned");
    return ICTC_ERR_BAD_ARG;
  }
  static const cudaError_t attr = cudaFuncSetAttribute(chain::mlp_chain_forward_kernel,
                                                       cudaFuncAttributeMaxDynamicSharedMemorySize, chain::kSmem);
  if (attr != cudaSuccess) { set_error("mlp chain smem: %s", cudaGetErrorString(attr)); return ICTC_ERR_LAUNCH; }
  chain::Args a{};
  a.in = rb; a.rows = rb_rows; a.limit = row_limit; a.w0 = w0; a.wa = w1_packed; a.wb = w2_packed; a.z1 = z1; a.z2 = z2; a.z3 = z3; a.E = num_edges; a.nb = num_basis;
  a.status = kernel_status_word();
  chain::mlp_chain_forward_kernel<<<chain::grid_size(num_edges), chain::kThreads, chain::kSmem, (cudaStream_t)stream>>>(a);
  return finish_launch("mlp_chain_forward");
}

int ictc_mlp_chain_backward(int64_t num_edges, int num_basis, const float* da3, const float* w0, const float* w1t_packed,
                            const float* w2t_packed, const float* z1, const float* z2, const float* z3, float* drb,
                            const int64_t* drb_rows, int accumulate, const int64_t* row_limit, void* stream) {
  return ictc_mlp_chain_backward_paired(num_edges, num_basis, da3, nullptr, nullptr, w0, w1t_packed, w2t_packed, z1, z2,
                                        z3, drb, drb_rows, accumulate, row_limit, stream);
}

int ictc_mlp_chain_backward_paired(int64_t num_edges, int num_basis, const float* da3, const int64_t* pair_a,
                                   const int64_t* pair_b, const float* w0, const float* w1t_packed,
                                   const float* w2t_packed, const float* z1, const float* z2, const float* z3,
                                   float* drb, const int64_t* drb_rows, int accumulate, const int64_t* row_limit,
                                   void* stream) {
  if (num_edges < 0 || num_basis < 1 || num_basis > 8) {
    set_error("mlp chain: needs 1..8 basis functions (got %d)", num_basis);
    return ICTC_ERR_BAD_SPEC;
  }
  if (num_edges == 0) return ICTC_OK;
  if (!da3 || !w0 || !w1t_packed || !w2t_packed || !z1 || !z2 || !z3 || !drb) { set_error("mlp chain backward: NULL buffer"); return ICTC_ERR_BAD_ARG; }
  if ((reinterpret_cast<uintptr_t>(z1) | reinterpret_cast<uintptr_t>(z2) | reinterpret_cast<uintptr_t>(z3) |
       reinterpret_cast<uintptr_t>(da3) | reinterpret_cast<uintptr_t>(w1t_packed) | reinterpret_cast<uintptr_t>(w2t_packed)) & 31) {
    set_error("mlp chain backward: buffers must be 32-byte aligned");
    return ICTC_ERR_BAD_ARG;
  }
  static const cudaError_t attr = cudaFuncSetAttribute(chain::mlp_chain_backward_kernel,
                                                       cudaFuncAttributeMaxDynamicSharedMemorySize, chain::kSmem);
  if (attr != cudaSuccess) { set_error("mlp chain smem: %s", cudaGetErrorString(attr)); return ICTC_ERR_LAUNCH; }
  chain::Args a{};
  a.in = da3; a.w0 = w0; a.wa = w2t_packed; a.wb = w1t_packed; a.z1 = const_cast<float*>(z1); a.z2 = const_cast<float*>(z2);
  a.z3 = const_cast<float*>(z3); a.drb = drb; a.in_a = pair_a; a.in_b = pair_b; a.rows = drb_rows; a.limit = row_limit; a.accumulate = accumulate ? 1 : 0; a.E = num_edges; a.nb = num_basis;
  a.status = kernel_status_word();
  chain::mlp_chain_backward_kernel<<<chain::grid_size(num_edges), chain::kThreads, chain::kSmem, (cudaStream_t)stream>>>(a);
  return finish_launch("mlp_chain_backward");
}

}  // extern "C"
