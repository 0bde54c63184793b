// Weight gradient of a row-wise linear map on the 5th-generation tensor cores (tcgen05 + TMEM):
//
//   dW[o, i] = sum_r  grad[r, o] * rows[r, i]        o < NO (multiple of 64, at most 768),  i < 64,  r < R
//
// the contraction runs over the ROWS (edges or atoms, millions), so both operands are "transposed" with respect to
// their row-major storage.  Reference: the dW / db branch of the training gate (ictc_o3/ops/training_gate_message.py:
// 120-186, `hidden^T @ dgates` accumulated over edge tiles) and the weight gradients of the per-degree channel
// linears (ictc_o3/operators.py:609-628 under autograd).
//
// One persistent CTA per SM owns a contiguous range of row stages (split-K over the CTAs) and keeps the whole
// [NO x 64] partial result in TMEM: up to six [128 x 64] fp32 accumulators = 384 columns.  A stage is 8 * KS rows
// (KS = 4, 2 or 1 K = 8 steps for NO <= 128, <= 256, larger).  Pipeline of one CTA:
//   * warp 1 streams the stage's rows of `grad` and `rows` as they lie in memory into a 4-deep raw ring with one
//     cp.async.bulk per row and operand (no multicast), completing on mbarriers: the HBM latency is covered by the
//     ring, not by registers;
//   * 16 transform warps read the raw rows from shared memory, split each value into two TF32-representable parts
//     and write them TRANSPOSED into a 2-deep operand ring in the canonical K-major no-swizzle layout (K = row
//     index r): element (f, k) of an operand with F feature rows lives at byte (k / 4) * F * 16 + f * 16 + (k % 4) * 4,
//     i.e. one thread writes one 16-byte chunk = four consecutive rows of one feature.  fence.proxy.async orders
//     these generic writes before the MMA's reads;
//   * one thread of warp 0 issues, per K = 8 step and 128-feature tile, the three MMAs small*big + big*small +
//     big*big (fp32-level accuracy, the reference forbids plain TF32: ictc_o3/backends/k100/fp32_policy.py:6-11)
//     and commits the operand stage back to the transform warps.
// At the end four warps read the accumulators (thread = feature row) and store the CTA's partial result; a second
// small kernel adds the partial results in a fixed order, so the gradient is bitwise repeatable.
// Every mbarrier wait is bounded; a wait that runs out raises the library's status word and the CTA leaves through
// the common exit (TMEM is always released).
#include "tc05.cuh"

namespace ictc {
namespace wg {

using namespace tc;

constexpr int kWorkWarps = 16, kWorkers = kWorkWarps * 32;
constexpr int kThreads = (2 + kWorkWarps) * 32;         // warp 0: TMEM owner + MMA issuer, warp 1: row stream
constexpr int kRawStages = 4, kOpStages = 2;
constexpr int kMaxTiles = 6;                            // 6 x 128 features
constexpr int kAPart = 2 * kRows * 16;                  // one part (big or small) of one 128-feature tile, K = 8: 4 KB
constexpr int kBPart = 2 * kK * 16;                     // one part of the 64-feature operand, K = 8: 2 KB
constexpr int kItemsMax = 4;                            // 16-byte chunks per transform thread and stage

__host__ __device__ constexpr int tiles_of(int no) { return (no + kRows - 1) / kRows; }
__host__ __device__ constexpr int ksteps_of(int no) { return tiles_of(no) == 1 ? 4 : (tiles_of(no) == 2 ? 2 : 1); }
__host__ __device__ constexpr int kstep_bytes(int no) { return tiles_of(no) * 2 * kAPart + 2 * kBPart; }
__host__ __device__ constexpr int raw_pitch(int no) { return (no + kK) * 4; }          // one raw row: grad | rows
__host__ __device__ constexpr int raw_bytes(int no) { return 8 * ksteps_of(no) * raw_pitch(no); }
__host__ __device__ constexpr int op_bytes(int no) { return ksteps_of(no) * kstep_bytes(no); }

struct Args {
  const float* grad;      // [R, *] row stride grad_ld, NO columns used
  const float* rows;      // [R, *] row stride rows_ld, 64 columns used
  float* partial;         // [grid, tiles * 128, 64]
  int64_t R, grad_ld, rows_ld;
  int NO;
  int* status;
};

struct Barriers {
  unsigned long long raw_full[kRawStages], raw_empty[kRawStages], op_full[kOpStages], op_empty[kOpStages], done;
  unsigned tmem_base;
  volatile int failed;
};

constexpr int smem_bytes(int no) { return kRawStages * raw_bytes(no) + kOpStages * op_bytes(no) + int(sizeof(Barriers)) + 128; }

__device__ __forceinline__ void umma_tf32_ss(unsigned d_tmem, uint64_t a_desc, uint64_t b_desc, unsigned accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "n"(kIdesc), "r"(accumulate)
      : "memory");
}

__device__ __forceinline__ void give_up(Barriers* b, int* status, int code) {
  b->failed = 1;
  if (status) atomicExch(status, code);
}

__global__ void __launch_bounds__(kThreads, 1) weight_grad_kernel(Args a) {
  extern __shared__ __align__(128) unsigned char wg_smem[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tiles = tiles_of(a.NO), ks_n = ksteps_of(a.NO), stage_rows = 8 * ks_n;
  const int raw_b = raw_bytes(a.NO), op_b = op_bytes(a.NO), ks_b = kstep_bytes(a.NO), pitch = raw_pitch(a.NO);
  unsigned char* raw = wg_smem;
  unsigned char* ops = wg_smem + kRawStages * raw_b;
  Barriers* bar = reinterpret_cast<Barriers*>(ops + kOpStages * op_b);
  const int64_t stages_total = (a.R + stage_rows - 1) / stage_rows;
  const int64_t per = (stages_total + gridDim.x - 1) / gridDim.x;
  const int64_t s0 = min(int64_t(blockIdx.x) * per, stages_total), s1 = min(s0 + per, stages_total);
  const int64_t mine = s1 - s0;

  if (threadIdx.x == 0) {
    for (int i = 0; i < kRawStages; ++i) {
      mbar_init(saddr(&bar->raw_full[i]), 1);
      mbar_init(saddr(&bar->raw_empty[i]), kWorkWarps);
    }
    for (int i = 0; i < kOpStages; ++i) {
      mbar_init(saddr(&bar->op_full[i]), kWorkWarps);
      mbar_init(saddr(&bar->op_empty[i]), 1);
    }
    mbar_init(saddr(&bar->done), 1);
    bar->failed = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 0) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(saddr(&bar->tmem_base)),
                 "r"(512u)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const unsigned tmem = bar->tmem_base;

  if (warp == 0) {
    // ---- MMA issue: per operand stage ks_n K = 8 steps, three products per feature tile
    if (lane == 0) {
      bool ok = true;
      for (int64_t it = 0; it < mine && !bar->failed; ++it) {
        const int s = int(it % kOpStages);
        if (!mbar_wait(saddr(&bar->op_full[s]), unsigned((it / kOpStages) & 1))) {
          give_up(bar, a.status, 41);
          ok = false;
          break;
        }
        tc_fence_after();
        for (int ks = 0; ks < ks_n; ++ks) {
          const unsigned base = saddr(ops + s * op_b + ks * ks_b);
          const unsigned b_big = base + tiles * 2 * kAPart;
          const uint64_t db_big = smem_desc(b_big, kK * 16, 128), db_small = smem_desc(b_big + kBPart, kK * 16, 128);
          for (int j = 0; j < tiles; ++j) {
            const unsigned a_big = base + j * 2 * kAPart;
            const uint64_t da_big = smem_desc(a_big, kRows * 16, 128), da_small = smem_desc(a_big + kAPart, kRows * 16, 128);
            const unsigned d = tmem + j * kChunk;
            umma_tf32_ss(d, da_small, db_big, (it == 0 && ks == 0) ? 0u : 1u);
            umma_tf32_ss(d, da_big, db_small, 1u);
            umma_tf32_ss(d, da_big, db_big, 1u);
          }
        }
        umma_commit(saddr(&bar->op_empty[s]));
      }
      if (ok && mine > 0 && !bar->failed) umma_commit(saddr(&bar->done));
    }
  } else if (warp == 1) {
    // ---- row stream: lane r copies rows r, r + 32, ... of the stage (one bulk copy per row and operand)
    for (int64_t it = 0; it < mine && !bar->failed; ++it) {
      const int s = int(it % kRawStages);
      if (!mbar_wait(saddr(&bar->raw_empty[s]), unsigned((it / kRawStages) & 1) ^ 1u)) {
        give_up(bar, a.status, 44);
        break;
      }
      const int64_t r0 = (s0 + it) * stage_rows;
      const int valid = int(min(int64_t(stage_rows), a.R - r0));
      const unsigned fb = saddr(&bar->raw_full[s]);
      if (lane == 0) mbar_expect_tx(fb, unsigned(valid) * unsigned(pitch));
      __syncwarp();
      // raw stage = [stage_rows x NO] block of grad, then [stage_rows x 64] block of rows; an operand stored without
      // row padding arrives as ONE copy (small per-row copies are bound by the copy engine's request rate)
      const unsigned gdst = saddr(raw + s * raw_b), xdst = gdst + unsigned(stage_rows) * unsigned(a.NO) * 4u;
      if (a.grad_ld == a.NO) {
        if (lane == 0) bulk_g2s(gdst, a.grad + r0 * a.grad_ld, unsigned(valid) * unsigned(a.NO) * 4u, fb);
      } else {
        for (int r = lane; r < valid; r += 32)
          bulk_g2s(gdst + unsigned(r) * unsigned(a.NO) * 4u, a.grad + (r0 + r) * a.grad_ld, unsigned(a.NO) * 4u, fb);
      }
      if (a.rows_ld == kK) {
        if (lane == 1) bulk_g2s(xdst, a.rows + r0 * a.rows_ld, unsigned(valid) * kK * 4u, fb);
      } else {
        for (int r = lane; r < valid; r += 32)
          bulk_g2s(xdst + unsigned(r) * kK * 4u, a.rows + (r0 + r) * a.rows_ld, kK * 4u, fb);
      }
    }
  } else {
    // ---- transform: thread = up to kItemsMax 16-byte chunks (K step, feature, four consecutive rows) per stage
    const int pt = threadIdx.x - 64;
    const int per_k = tiles * 2 * kRows + 2 * kK, a_items = tiles * 2 * kRows, items = ks_n * per_k;
    int src_off[kItemsMax], src_step[kItemsMax], dst_off[kItemsMax], part[kItemsMax], row0[kItemsMax];
    bool used[kItemsMax];
#pragma unroll
    for (int i = 0; i < kItemsMax; ++i) {
      const int id = pt + i * kWorkers;
      used[i] = id < items;
      const int ks = id / per_k, rem = id - ks * per_k;
      const bool is_a = rem < a_items;
      const int q = is_a ? rem / (tiles * kRows) : (rem - a_items) / kK;
      const int f = is_a ? rem - q * (tiles * kRows) : (rem - a_items) - q * kK;
      row0[i] = ks * 8 + 4 * q;
      src_step[i] = (is_a ? a.NO : kK) * 4;
      src_off[i] = (is_a ? 0 : stage_rows * a.NO * 4) + row0[i] * src_step[i] + f * 4;
      dst_off[i] = ks * ks_b + (is_a ? (f / kRows) * 2 * kAPart + q * (kRows * 16) + (f % kRows) * 16
                                     : tiles * 2 * kAPart + q * (kK * 16) + f * 16);
      part[i] = is_a ? kAPart : kBPart;
      if (is_a && f >= a.NO) src_off[i] = -1;       // padding feature of the last tile: zeros
    }
    for (int64_t it = 0; it < mine; ++it) {
      const int rs = int(it % kRawStages), os = int(it % kOpStages);
      if (bar->failed || !mbar_wait(saddr(&bar->raw_full[rs]), unsigned((it / kRawStages) & 1)) ||
          !mbar_wait(saddr(&bar->op_empty[os]), unsigned((it / kOpStages) & 1) ^ 1u)) {
        give_up(bar, a.status, 42);
        break;
      }
      const int valid = int(min(int64_t(stage_rows), a.R - (s0 + it) * stage_rows));
      const unsigned char* in = raw + rs * raw_b;
      unsigned char* out = ops + os * op_b;
#pragma unroll
      for (int i = 0; i < kItemsMax; ++i) {
        if (!used[i]) continue;
        float v[4];
#pragma unroll
        for (int j = 0; j < 4; ++j)
          v[j] = (src_off[i] >= 0 && row0[i] + j < valid) ? *reinterpret_cast<const float*>(in + src_off[i] + j * src_step[i]) : 0.f;
        float4 big, small;
        big.x = to_tf32(v[0]); small.x = to_tf32(v[0] - big.x);
        big.y = to_tf32(v[1]); small.y = to_tf32(v[1] - big.y);
        big.z = to_tf32(v[2]); small.z = to_tf32(v[2] - big.z);
        big.w = to_tf32(v[3]); small.w = to_tf32(v[3] - big.w);
        *reinterpret_cast<float4*>(out + dst_off[i]) = big;
        *reinterpret_cast<float4*>(out + dst_off[i] + part[i]) = small;
      }
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // generic writes -> visible to the MMA's reads
      __syncwarp();
      if (lane == 0) {                 // one arrival per warp: 512 single arrivals per stage cost more than the stage
        mbar_arrive(saddr(&bar->op_full[os]));
        mbar_arrive(saddr(&bar->raw_empty[rs]));
      }
    }
    // ---- epilogue: warps 2-5 cover the four lane quarters of TMEM (quarter = warp % 4)
    if (warp <= 5) {
      const int qd = warp & 3;
      float* outp = a.partial + int64_t(blockIdx.x) * tiles * kRows * kK;
      bool have = mine > 0;
      if (have && (bar->failed || !mbar_wait(saddr(&bar->done), 0u))) {
        give_up(bar, a.status, 43);
        have = false;
      }
      tc_fence_after();
      for (int j = 0; j < tiles; ++j) {
        float v0[32], v1[32];
        if (have) {
          const unsigned taddr = tmem + (unsigned(qd * 32) << 16) + j * kChunk;
          tmem_ld32(taddr, v0);
          tmem_ld32(taddr + 32, v1);
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) v0[i] = v1[i] = 0.f;
        }
        float4* o = reinterpret_cast<float4*>(outp + (int64_t(j) * kRows + qd * 32 + lane) * kK);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          o[i] = make_float4(v0[4 * i], v0[4 * i + 1], v0[4 * i + 2], v0[4 * i + 3]);
          o[8 + i] = make_float4(v1[4 * i], v1[4 * i + 1], v1[4 * i + 2], v1[4 * i + 3]);
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) {
    __syncwarp();
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(512u) : "memory");
  }
}

// dW[o, i] = sum over the CTAs' partial results, in CTA order.
__global__ void weight_grad_reduce_kernel(const float* __restrict__ partial, int parts, int tiles, int NO, float* dw,
                                          int64_t dw_ld) {
  const int idx = blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= NO * kK) return;
  const int o = idx / kK, i = idx % kK;
  const int64_t pitch = int64_t(tiles) * kRows * kK;
  float s = 0.f;
  for (int b = 0; b < parts; ++b) s += partial[b * pitch + idx];
  dw[o * dw_ld + i] = s;
}

static int grid_size(int64_t rows) {
  int dev = 0, sms = 148;
  if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const int64_t stages = (rows + 7) / 8;
  return int(stages < sms ? (stages < 1 ? 1 : stages) : sms);
}

}  // namespace wg
}  // namespace ictc

using namespace ictc;

extern "C" {

int64_t ictc_weight_grad_workspace(int64_t num_rows, int num_out) {
  if (num_rows < 0 || num_out < 64 || num_out % 64 || num_out > wg::kMaxTiles * tc::kRows) return -1;
  const int tiles = (num_out + tc::kRows - 1) / tc::kRows;
  return int64_t(wg::grid_size(num_rows)) * tiles * tc::kRows * tc::kK * int64_t(sizeof(float));
}

int ictc_weight_grad_tc(int64_t num_rows, int num_out, const float* grad, int64_t grad_ld, const float* rows,
                        int64_t rows_ld, float* dweight, int64_t dweight_ld, float* workspace, void* stream) {
  if (num_rows < 0 || num_out < 64 || num_out % 64 || num_out > wg::kMaxTiles * tc::kRows || grad_ld < num_out ||
      rows_ld < tc::kK || dweight_ld < tc::kK) {
    set_error("weight grad: need 64 <= num_out <= %d, a multiple of 64, and row strides covering the columns (got %d)",
              wg::kMaxTiles * tc::kRows, num_out);
    return ICTC_ERR_BAD_SPEC;
  }
  if (!grad || !rows || !dweight || !workspace) { set_error("weight grad: NULL buffer"); return ICTC_ERR_BAD_ARG; }
  if (((reinterpret_cast<uintptr_t>(workspace) | reinterpret_cast<uintptr_t>(grad) | reinterpret_cast<uintptr_t>(rows)) & 15) ||
      (grad_ld & 3) || (rows_ld & 3)) {
    set_error("weight grad: buffers must be 16-byte aligned and row strides multiples of 4 floats (bulk copies)");
    return ICTC_ERR_BAD_ARG;
  }
  const int tiles = wg::tiles_of(num_out);
  const int smem = wg::smem_bytes(num_out);
  constexpr int smem_max = wg::smem_bytes(wg::kMaxTiles * tc::kRows);
  static_assert(smem_max <= 227 * 1024 && wg::smem_bytes(64) <= smem_max && wg::smem_bytes(256) <= smem_max &&
                wg::smem_bytes(384) <= smem_max, "weight grad: shared-memory plan");
  static const cudaError_t attr = cudaFuncSetAttribute(wg::weight_grad_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                       smem_max);
  if (attr != cudaSuccess) { set_error("weight grad smem: %s", cudaGetErrorString(attr)); return ICTC_ERR_LAUNCH; }
  const int grid = wg::grid_size(num_rows);
  wg::Args a{};
  a.grad = grad; a.rows = rows; a.partial = workspace; a.R = num_rows; a.grad_ld = grad_ld; a.rows_ld = rows_ld;
  a.NO = num_out; a.status = kernel_status_word();
  wg::weight_grad_kernel<<<grid, wg::kThreads, smem, (cudaStream_t)stream>>>(a);
  if (int rc = finish_launch("weight_grad")) return rc;
  const int n = num_out * tc::kK;
  wg::weight_grad_reduce_kernel<<<(n + 255) / 256, 256, 0, (cudaStream_t)stream>>>(workspace, grid, tiles, num_out,
                                                                                 dweight, dweight_ld);
  return finish_launch("weight_grad_reduce");
}

}  // extern "C"
