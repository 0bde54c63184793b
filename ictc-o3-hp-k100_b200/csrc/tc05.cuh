// tcgen05 / TMEM / mbarrier helpers shared by the tensor-core kernels of the radial gate MLP and the channel
// linears (inline PTX for sm_100a).  Operand conventions:
//  * B operand in shared memory, canonical K-major no-swizzle layout: element (n, k) of a [64 x 64] part at byte
//    (k / 4) * 1024 + n * 16 + (k % 4) * 4 (descriptor: LBO 1024 B between the two K chunks of a K = 8 MMA,
//    SBO 128 B between 8-row core matrices);
//  * A operand in TMEM: lane = tile row, column = k;  accumulator in TMEM: lane = row, column = n;
//  * fp32-level products through a three-term TF32 split: x = big + small, a*b ~ small*big + big*small + big*big.
#pragma once
#include "ictc_common.cuh"

namespace ictc {
namespace tc {

constexpr int kRows = 128;             // tile rows = UMMA M
constexpr int kK = 64;                 // hidden width
constexpr int kChunk = 64;             // weight chunk: 64 units (N of the forward MMA, K step of the backward)
constexpr int kWPartBytes = kChunk * kK * 4;        // 16 KB
constexpr int kWStageBytes = 2 * kWPartBytes;       // big + small
constexpr long long kWaitCycles = 2000000000LL;     // ~1 s
constexpr float kSiluScale = 1.6791767923989418f;

// instruction descriptor: D fp32, A and B TF32, both K-major, M = 128, N = 64
constexpr uint32_t kIdesc = (1u << 4) | (2u << 7) | (2u << 10) | (uint32_t(kChunk >> 3) << 17) | (uint32_t(kRows >> 4) << 24);

__device__ __forceinline__ unsigned saddr(const void* p) { return static_cast<unsigned>(__cvta_generic_to_shared(p)); }
__device__ __forceinline__ void mbar_init(unsigned bar, unsigned count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive(unsigned bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(unsigned bar, unsigned bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try(unsigned bar, unsigned parity) {
  unsigned done;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(done)
      : "r"(bar), "r"(parity)
      : "memory");
  return done != 0;
}
__device__ __forceinline__ bool mbar_wait(unsigned bar, unsigned parity) {
  if (mbar_try(bar, parity)) return true;
  const long long start = clock64();
  while (!mbar_try(bar, parity))
    if (clock64() - start > kWaitCycles) return false;
  return true;
}
__device__ __forceinline__ void bulk_g2s(unsigned dst, const void* src, unsigned bytes, unsigned bar) {
  asm volatile("cp.async.bulk.shared::cta.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
               "l"(src), "r"(bytes), "r"(bar)
               : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// K-major, no swizzle (layout type 0), descriptor version 1
__device__ __forceinline__ uint64_t smem_desc(unsigned addr, unsigned lbo_bytes, unsigned sbo_bytes) {
  return uint64_t((addr & 0x3FFFFu) >> 4) | (uint64_t(lbo_bytes >> 4) << 16) | (uint64_t(sbo_bytes >> 4) << 32) |
         (1ull << 46);
}
__device__ __forceinline__ void umma_commit(unsigned bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tmem_ld32(unsigned taddr, float (&v)[32]) {
  unsigned r[32];
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
        "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
        "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
  for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
}

__device__ __forceinline__ float to_tf32(float x) {
  unsigned r;
  asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(r) : "f"(x));
  return __uint_as_float(r);
}
// Logistic function from the hardware exp2 and reciprocal approximations (each within ~2 units in the last place;
// the exponent product adds |v| * 6e-8): relative error below 1e-6 where the function is not saturated, which is
// inside the fp32 noise of the surrounding three-term TF32 products and a fraction of the cost of expf and a division.
__device__ __forceinline__ float sigmoid_fast(float v) {
  float t, r;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(t) : "f"(v * -1.4426950408889634f));
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(1.f + t));
  return r;
}
__device__ __forceinline__ float silu_s(float v) { return v * sigmoid_fast(v) * kSiluScale; }
__device__ __forceinline__ float dsilu_s(float v) {
  const float s = sigmoid_fast(v);
  return kSiluScale * s * fmaf(v, 1.f - s, 1.f);
}

__device__ __forceinline__ void umma_tf32_ts(unsigned d_tmem, unsigned a_tmem, uint64_t b_desc, unsigned accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::tf32 [%0], [%1], %2, %3, p;\n\t}"
      ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "n"(kIdesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void tmem_st32(unsigned taddr, const unsigned (&r)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
      "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
      "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]),
      "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]),
      "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
      : "memory");
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
// 32-byte read-only load that bypasses L1 (every thread streams its own row)
__device__ __forceinline__ void ldg256(const float* p, float* v) {
  asm volatile("ld.global.nc.L1::no_allocate.v8.f32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
               : "=f"(v[0]), "=f"(v[1]), "=f"(v[2]), "=f"(v[3]), "=f"(v[4]), "=f"(v[5]), "=f"(v[6]), "=f"(v[7])
               : "l"(p));
}

// Splits 32 values of one row and writes the two parts into the TMEM A operand (lane = row, column = k).
__device__ __forceinline__ void store_split_tmem(unsigned t_big, unsigned t_small, const float (&x)[32]) {
  unsigned b[32], sm[32];
#pragma unroll
  for (int i = 0; i < 32; ++i) {
    const float big = to_tf32(x[i]);
    b[i] = __float_as_uint(big);
    sm[i] = __float_as_uint(to_tf32(x[i] - big));
  }
  tmem_st32(t_big, b);
  tmem_st32(t_small, sm);
  tmem_st_wait();
}

// The 24 MMAs of one [128 x 64] x [64 x 64]^T product: small*big, big*small, big*big over 8 K steps.
// A comes from TMEM (big part at a_tmem, small part 64 columns further), B from shared memory.  The issuing
// thread is a single lane, so the per-MMA instruction count matters: descriptors are advanced by adding the
// K-step offset to a base descriptor (the start-address field never overflows inside one stage).
__device__ __forceinline__ void issue_block(unsigned d_tmem, unsigned a_tmem, unsigned w_big, unsigned w_small,
                                            bool first) {
  const uint64_t desc_big = smem_desc(w_big, kChunk * 16, 128), desc_small = smem_desc(w_small, kChunk * 16, 128);
  constexpr uint64_t kStep = (2 * kChunk * 16) >> 4;        // two 16-byte K chunks per MMA
#pragma unroll
  for (int ks = 0; ks < kK / 8; ++ks) umma_tf32_ts(d_tmem, a_tmem + kK + ks * 8, desc_big + ks * kStep, (first && ks == 0) ? 0u : 1u);
#pragma unroll
  for (int ks = 0; ks < kK / 8; ++ks) umma_tf32_ts(d_tmem, a_tmem + ks * 8, desc_small + ks * kStep, 1u);
#pragma unroll
  for (int ks = 0; ks < kK / 8; ++ks) umma_tf32_ts(d_tmem, a_tmem + ks * 8, desc_big + ks * kStep, 1u);
}

}  // namespace tc
}  // namespace ictc
