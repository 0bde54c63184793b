// Wide last layer of the radial gate MLP on the 5th-generation tensor cores (tcgen05 + TMEM).
//
//   forward :  gates[r, :] = act(z3[r, :]) @ W3^T            K = 64,    N = P*C (192 or 704)
//   backward:  da3[r, :]   = (dG[a(r), :] + dG[b(r), :]) @ W3   K = P*C,  N = 64
//
// Reference: last `F.linear` of the interaction block's radial stack (mace_ictc/models/mace/layers.py:825-835),
// tiled per edge chunk by ictc_o3/ops/streamed_gate_message.py:112-116, and its input gradient
// (streamed_gate_message.py:224-260).  The reference forbids TF32 (ictc_o3/backends/k100/fp32_policy.py:6-11),
// so every operand is split into two TF32-representable parts, x = x_big + x_small, and a product is the sum of
// the three tcgen05.mma passes big*big + big*small + small*big into one fp32 TMEM accumulator.
//
// One persistent CTA per SM works on tiles of 128 rows.  Warp roles:
//   warp 0      streams pre-packed 64-unit weight chunks (32 KB: big and small part) into a 2-stage ring
//               with cp.async.bulk, completing on mbarriers;
//   warp 1      allocates TMEM and issues the MMAs (one thread), committing to mbarriers;
//   warps 2-9   epilogue (forward: two groups taking alternate chunks; backward: warps 2-5 only):
//               tcgen05.ld (thread = row), then coalesced row stores;
//   warps 10-17 A-operand producers: global rows -> (activation | pair sum) -> split -> tcgen05.st into TMEM
//               (the A operand is read from TMEM: lane = row, column = k; no shared memory for A at all).
// Shared-memory layout of the B operand: element (n, k) of a [64 x 64] part lives at byte
// (k / 4) * 1024 + n * 16 + (k % 4) * 4, i.e. 16-byte K chunks, each chunk row-contiguous (canonical K-major
// no-swizzle layout).  In descriptor terms: 8-row core matrices of 128 contiguous bytes, stride between core
// matrices along n (SBO) 128 B, stride between the two K chunks of one K = 8 MMA (LBO) 1024 B.
// Every mbarrier wait is bounded; a wait that runs out raises the library's status word and the CTA leaves
// through the common exit (TMEM is always released).
#include "tc05.cuh"

namespace ictc {
namespace gg {

using namespace tc;

constexpr int kThreads = 18 * 32;
constexpr int kProducerWarp0 = 10, kProducerWarps = 8;   // warps 2-5 and 6-9: two epilogue groups
constexpr int kStagePitch = 272;                    // bytes per staged output row (256 + 16: conflict-free)

struct Args {
  const float* in;        // forward: z3 [rows, 64]; backward: dgates [*, nout]
  const float* w;         // packed chunks, 8192 floats each
  float* out;             // forward: gates [rows, nout]; backward: da3 [rows, 64]
  const int64_t* pair_a;  // backward, optional
  const int64_t* pair_b;
  int64_t rows;
  const int64_t* limit;   // optional device scalar: only min(rows, *limit) rows are processed (recorded graphs)
  // Row windows (plain matrices only).  With `begin` (device scalar) the launch covers the window
  // [*begin, min(*begin + rows, *limit)) of a longer row list: local row g = 0.. stands for list entry *begin + g.
  const int64_t* begin;
  const int64_t* in_index;   // forward: local row g reads in[in_index[*begin + g]] (null: in[*begin + g])
  const int64_t* out_index;  // backward: local row g is written to out[out_index[*begin + g]] (null: out[*begin + g])
  int nout;
  int act;                // forward: apply the scaled SiLU to the input
  int* status;
  // Row addressing (units: floats).  Row g is sub-row g % mm of node g / mm; its 64-float block number b
  // (the only block of the 64-wide side, chunk c * cs of the wide side) starts at
  //   base + (g / mm) * ld + (b + g % mm) * 64.
  // Plain matrices: mm = 1, ld = row length, cs = 1.  Per-degree feature blocks [node][path slot][m][C]:
  // mm = 2l+1, ld = node stride, cs = mm (the slot-major layout is read and written in place).
  int in_mm, out_mm, in_cs, out_cs;
  int64_t in_ld, out_ld;
};

__device__ __forceinline__ int64_t row_offset(int64_t g, int mm, int64_t ld) {
  if (mm == 1) return g * ld;
  const int64_t node = g / mm;
  return node * ld + (g - node * mm) * kK;
}

constexpr int kWStages = 4;      // weight ring
constexpr int kAStagesBwd = 3;   // TMEM A ring of the backward kernel

struct Barriers {
  unsigned long long w_full[kWStages], w_empty[kWStages], a_full[4], a_empty[4], d_full[4], d_empty[4];
  unsigned tmem_base;
  volatile int failed;   // polled inside wait loops by other warps: every read must go to shared memory
  volatile long long progress;   // backward: chunks finished by the first producer warp (read by the prefetch warps)
};

__device__ __forceinline__ void give_up(Barriers* b, int* status, int code) {
  b->failed = 1;
  if (status) atomicExch(status, code);
}

// ------------------------------------------------------------------------------------------------
// forward.  Shared memory: W ring (4 x 32 KB) | output staging (2 x 34 KB) | barriers.
// TMEM (512 columns): accumulator ring 4 x 64 | A operand of two tiles, each big (64) + small (64).
constexpr int kFwdSmem = kWStages * kWStageBytes + 2 * kRows * kStagePitch + 256;

__global__ void __launch_bounds__(kThreads, 1) gate_gemm_forward_kernel(Args a) {
  extern __shared__ __align__(128) unsigned char gg_smem[];
  unsigned char* w_buf = gg_smem;
  unsigned char* stage = w_buf + kWStages * kWStageBytes;
  Barriers* bar = reinterpret_cast<Barriers*>(stage + 2 * kRows * kStagePitch);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int chunks = a.nout / kChunk;
  const int64_t base = a.begin ? ldg(a.begin) : 0;
  int64_t nrows = a.limit ? ldg(a.limit) - base : a.rows;
  nrows = nrows < 0 ? 0 : (nrows < a.rows ? nrows : a.rows);
  const int64_t tiles = (nrows + kRows - 1) / kRows;
  const int64_t my_tiles = blockIdx.x < tiles ? (tiles - blockIdx.x + gridDim.x - 1) / gridDim.x : 0;

  if (threadIdx.x == 0) {
    for (int i = 0; i < kWStages; ++i) {
      mbar_init(saddr(&bar->w_full[i]), 1);
      mbar_init(saddr(&bar->w_empty[i]), 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(saddr(&bar->a_full[i]), kProducerWarps * 32);
      mbar_init(saddr(&bar->a_empty[i]), 1);
    }
    for (int i = 0; i < 4; ++i) {
      mbar_init(saddr(&bar->d_full[i]), 1);
      mbar_init(saddr(&bar->d_empty[i]), 128);
    }
    bar->failed = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
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
  const unsigned tmem = bar->tmem_base;
  const unsigned tmem_a = tmem + 4 * kChunk;       // A operands start after the accumulator ring

  if (warp == 0) {
    // ---- weight chunk stream
    if (lane == 0) {
      int64_t it = 0;
      for (int64_t t = 0; t < my_tiles && !bar->failed; ++t) {
        for (int c = 0; c < chunks; ++c, ++it) {
          const int s = int(it % kWStages);
          if (!mbar_wait(saddr(&bar->w_empty[s]), unsigned((it / kWStages) & 1) ^ 1u)) { give_up(bar, a.status, 21); break; }
          mbar_expect_tx(saddr(&bar->w_full[s]), kWStageBytes);
          bulk_g2s(saddr(w_buf + s * kWStageBytes), a.w + int64_t(c) * (kWStageBytes / 4), kWStageBytes,
                   saddr(&bar->w_full[s]));
        }
      }
    }
  } else if (warp == 1) {
    // ---- MMA issue
    if (lane == 0) {
      int64_t it = 0;
      for (int64_t t = 0; t < my_tiles && !bar->failed; ++t) {
        const int ab = int(t & 1);
        if (!mbar_wait(saddr(&bar->a_full[ab]), unsigned((t >> 1) & 1))) { give_up(bar, a.status, 22); break; }
        tc_fence_after();
        bool ok = true;
        for (int c = 0; c < chunks; ++c, ++it) {
          const int s = int(it % kWStages), d = int(it & 3);
          if (!mbar_wait(saddr(&bar->w_full[s]), unsigned((it / kWStages) & 1)) ||
              !mbar_wait(saddr(&bar->d_empty[d]), unsigned((it >> 2) & 1) ^ 1u)) {
            give_up(bar, a.status, 23);
            ok = false;
            break;
          }
          tc_fence_after();
          const unsigned w_big = saddr(w_buf + s * kWStageBytes), w_small = w_big + kWPartBytes;
          issue_block(tmem + d * kChunk, tmem_a + ab * 2 * kK, w_big, w_small, true);
          umma_commit(saddr(&bar->w_empty[s]));
          umma_commit(saddr(&bar->d_full[d]));
        }
        if (!ok) break;
        umma_commit(saddr(&bar->a_empty[ab]));
      }
    }
  } else if (warp < kProducerWarp0) {
    // ---- epilogue, two groups of four warps that take alternate chunks: tcgen05.ld gives thread = row; the
    // warp's 32 rows go through a padded staging buffer and leave as coalesced 256-byte row segments (two rows
    // per store instruction)
    const int q = warp & 3;                         // TMEM lane quarter this warp may read
    const int group = (warp - 2) >> 2;
    const int row = q * 32 + lane;
    unsigned char* gstage = stage + group * (kRows * kStagePitch);
    unsigned char* mine = gstage + row * kStagePitch;
    const unsigned char* warp_rows = gstage + q * 32 * kStagePitch;
    const int mm = a.out_mm;
    int64_t it = 0;
    for (int64_t t = 0; t < my_tiles; ++t) {
      const int64_t row0 = (blockIdx.x + t * gridDim.x) * kRows + q * 32;
      // rows 2i + (lane >> 4) of this warp are stored by this lane: walk their offsets without dividing
      const int64_t g0 = row0 + (lane >> 4);
      const int64_t node0 = mm == 1 ? g0 : g0 / mm;
      const int sub0 = mm == 1 ? 0 : int(g0 - node0 * mm);
      const int64_t off0 = node0 * a.out_ld + sub0 * kK + (lane & 15) * 4;
      bool ok = true;
      for (int c = 0; c < chunks; ++c, ++it) {
        if (int(it & 1) != group) continue;
        const int d = int(it & 3);
        if (bar->failed || !mbar_wait(saddr(&bar->d_full[d]), unsigned((it >> 2) & 1))) {
          give_up(bar, a.status, 24);
          ok = false;
          break;
        }
        tc_fence_after();
        float v0[32], v1[32];
        const unsigned taddr = tmem + (unsigned(q * 32) << 16) + d * kChunk;
        tmem_ld32(taddr, v0);
        tmem_ld32(taddr + 32, v1);
        tc_fence_before();
        mbar_arrive(saddr(&bar->d_empty[d]));
        __syncwarp();                                // the previous chunk's read-back is complete
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          *reinterpret_cast<float4*>(mine + j * 16) = make_float4(v0[4 * j], v0[4 * j + 1], v0[4 * j + 2], v0[4 * j + 3]);
          *reinterpret_cast<float4*>(mine + 128 + j * 16) =
              make_float4(v1[4 * j], v1[4 * j + 1], v1[4 * j + 2], v1[4 * j + 3]);
        }
        __syncwarp();
        float* base = a.out + int64_t(c) * a.out_cs * kChunk;
        int64_t off = off0;
        int sub = sub0;
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          const int r = 2 * i + (lane >> 4);
          const float4 v = *reinterpret_cast<const float4*>(warp_rows + r * kStagePitch + (lane & 15) * 16);
          if (row0 + r < nrows) __stcs(reinterpret_cast<float4*>(base + off), v);
          if (mm == 1) {
            off += 2 * a.out_ld;
          } else {
            sub += 2;
            off += 2 * kK;
            while (sub >= mm) { sub -= mm; off += a.out_ld - int64_t(mm) * kK; }
          }
        }
      }
      if (!ok) break;
    }
  } else {
    // ---- A producers: thread = (row, half of the 64 columns); z3 -> activation -> split -> TMEM
    const int q = warp & 3, half = (warp - kProducerWarp0) >> 2;
    const int row = q * 32 + lane;
    for (int64_t t = 0; t < my_tiles; ++t) {
      const int ab = int(t & 1);
      const int64_t g = (blockIdx.x + t * gridDim.x) * kRows + row;
      float x[32];
      if (g < nrows) {
        const int64_t srow = a.in_index ? ldg(a.in_index + base + g) : base + g;
#pragma unroll
        for (int j = 0; j < 4; ++j) ldg256(a.in + row_offset(srow, a.in_mm, a.in_ld) + half * 32 + j * 8, x + j * 8);
      } else {
#pragma unroll
        for (int i = 0; i < 32; ++i) x[i] = 0.f;
      }
      if (a.act) {
#pragma unroll
        for (int i = 0; i < 32; ++i) x[i] = silu_s(x[i]);
      }
      if (bar->failed) break;
      if (!mbar_wait(saddr(&bar->a_empty[ab]), unsigned((t >> 1) & 1) ^ 1u)) { give_up(bar, a.status, 25); break; }
      tc_fence_after();
      const unsigned t_big = tmem_a + (unsigned(q * 32) << 16) + ab * 2 * kK + half * 32;
      store_split_tmem(t_big, t_big + kK, x);
      tc_fence_before();
      mbar_arrive(saddr(&bar->a_full[ab]));
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(512u) : "memory");
  }
}

// ------------------------------------------------------------------------------------------------
// backward.  Shared memory: W ring (4 x 32 KB) | barriers.  TMEM: two accumulators [128 x 64] that alternate
// between tiles | A ring of three stages (big + small, 128 columns each); K runs over the nout / 64 chunks.
constexpr int kBwdSmem = kWStages * kWStageBytes + 256;

__global__ void __launch_bounds__(kThreads, 1) gate_gemm_backward_kernel(Args a) {
  extern __shared__ __align__(128) unsigned char gg_smem[];
  unsigned char* w_buf = gg_smem;
  Barriers* bar = reinterpret_cast<Barriers*>(w_buf + kWStages * kWStageBytes);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int chunks = a.nout / kChunk;
  const int64_t base = a.begin ? ldg(a.begin) : 0;
  int64_t nrows = a.limit ? ldg(a.limit) - base : a.rows;
  nrows = nrows < 0 ? 0 : (nrows < a.rows ? nrows : a.rows);
  const int64_t tiles = (nrows + kRows - 1) / kRows;
  const int64_t my_tiles = blockIdx.x < tiles ? (tiles - blockIdx.x + gridDim.x - 1) / gridDim.x : 0;

  if (threadIdx.x == 0) {
    for (int i = 0; i < kWStages; ++i) {
      mbar_init(saddr(&bar->w_full[i]), 1);
      mbar_init(saddr(&bar->w_empty[i]), 1);
    }
    for (int i = 0; i < kAStagesBwd; ++i) {
      mbar_init(saddr(&bar->a_full[i]), kProducerWarps * 32);
      mbar_init(saddr(&bar->a_empty[i]), 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(saddr(&bar->d_full[i]), 1);
      mbar_init(saddr(&bar->d_empty[i]), 128);
    }
    bar->failed = 0;
    bar->progress = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
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
  const unsigned tmem = bar->tmem_base;
  const unsigned tmem_a = tmem + 2 * kChunk;

  if (warp == 0) {
    if (lane == 0) {
      int64_t it = 0;
      for (int64_t t = 0; t < my_tiles && !bar->failed; ++t) {
        for (int c = 0; c < chunks; ++c, ++it) {
          const int s = int(it % kWStages);
          if (!mbar_wait(saddr(&bar->w_empty[s]), unsigned((it / kWStages) & 1) ^ 1u)) { give_up(bar, a.status, 31); break; }
          mbar_expect_tx(saddr(&bar->w_full[s]), kWStageBytes);
          bulk_g2s(saddr(w_buf + s * kWStageBytes), a.w + int64_t(c) * (kWStageBytes / 4), kWStageBytes,
                   saddr(&bar->w_full[s]));
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      int64_t it = 0;
      for (int64_t t = 0; t < my_tiles && !bar->failed; ++t) {
        const int d = int(t & 1);
        if (!mbar_wait(saddr(&bar->d_empty[d]), unsigned((t >> 1) & 1) ^ 1u)) { give_up(bar, a.status, 32); break; }
        bool ok = true;
        for (int c = 0; c < chunks; ++c, ++it) {
          const int s = int(it % kWStages), sa = int(it % kAStagesBwd);
          if (!mbar_wait(saddr(&bar->w_full[s]), unsigned((it / kWStages) & 1)) ||
              !mbar_wait(saddr(&bar->a_full[sa]), unsigned((it / kAStagesBwd) & 1))) {
            give_up(bar, a.status, 33);
            ok = false;
            break;
          }
          tc_fence_after();
          const unsigned w_big = saddr(w_buf + s * kWStageBytes), w_small = w_big + kWPartBytes;
          issue_block(tmem + d * kChunk, tmem_a + sa * 2 * kK, w_big, w_small, c == 0);
          umma_commit(saddr(&bar->w_empty[s]));
          umma_commit(saddr(&bar->a_empty[sa]));
        }
        if (!ok) break;
        umma_commit(saddr(&bar->d_full[d]));
      }
    }
  } else if (warp < 6) {
    const int q = warp & 3;
    const int row = q * 32 + lane;
    for (int64_t t = 0; t < my_tiles; ++t) {
      const int d = int(t & 1);
      const int64_t grow = (blockIdx.x + t * gridDim.x) * kRows + row;
      if (bar->failed || !mbar_wait(saddr(&bar->d_full[d]), unsigned((t >> 1) & 1))) { give_up(bar, a.status, 34); break; }
      tc_fence_after();
      float v0[32], v1[32];
      const unsigned taddr = tmem + (unsigned(q * 32) << 16) + d * kChunk;
      tmem_ld32(taddr, v0);
      tmem_ld32(taddr + 32, v1);
      tc_fence_before();
      mbar_arrive(saddr(&bar->d_empty[d]));
      if (grow < nrows) {
        const int64_t orow = a.out_index ? ldg(a.out_index + base + grow) : base + grow;
        float4* o = reinterpret_cast<float4*>(a.out + row_offset(orow, a.out_mm, a.out_ld));
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          o[j] = make_float4(v0[4 * j], v0[4 * j + 1], v0[4 * j + 2], v0[4 * j + 3]);
          o[8 + j] = make_float4(v1[4 * j], v1[4 * j + 1], v1[4 * j + 2], v1[4 * j + 3]);
        }
      }
    }
  } else if (warp < kProducerWarp0) {
    // ---- warps 6-9: L2 prefetch of the rows a few chunks ahead of the producers, across tile boundaries
    // (thread = row).  They follow the producers through a progress counter and never wait when they are behind.
    const int q = warp & 3;
    const int row = q * 32 + lane;
    constexpr int kAhead = 2;
    const int64_t cstep = int64_t(a.in_cs) * kChunk;
    int64_t pf_tile = 0;
    int pf_chunk = 0;
    const float* pa = nullptr;
    const float* pb = nullptr;
    auto enter_tile = [&]() {
      pa = pb = nullptr;
      if (pf_tile >= my_tiles) return;
      const int64_t g = (blockIdx.x + pf_tile * gridDim.x) * kRows + row;
      if (g >= nrows) return;
      const int64_t ra = a.pair_a ? __ldg(reinterpret_cast<const long long*>(a.pair_a + g)) : g;
      const int64_t rb = a.pair_b ? __ldg(reinterpret_cast<const long long*>(a.pair_b + g)) : -1;
      pa = a.in + row_offset(ra, a.in_mm, a.in_ld);
      if (rb >= 0) pb = a.in + row_offset(rb, a.in_mm, a.in_ld);
    };
    auto advance = [&]() {
      if (pf_tile >= my_tiles) return;
      if (pa) {
        asm volatile("prefetch.global.L2 [%0];" ::"l"(pa + pf_chunk * cstep));
        asm volatile("prefetch.global.L2 [%0];" ::"l"(pa + pf_chunk * cstep + 32));
      }
      if (pb) {
        asm volatile("prefetch.global.L2 [%0];" ::"l"(pb + pf_chunk * cstep));
        asm volatile("prefetch.global.L2 [%0];" ::"l"(pb + pf_chunk * cstep + 32));
      }
      if (++pf_chunk == chunks) {
        pf_chunk = 0;
        ++pf_tile;
        enter_tile();
      }
    };
    enter_tile();
    for (int k = 0; k < kAhead; ++k) advance();
    const int64_t total = my_tiles * chunks;
    for (int64_t it = 0; it < total; ++it) {
      advance();
      const long long start = clock64();
      bool ok = true;
      while (bar->progress <= it && !bar->failed) {
        if (clock64() - start > kWaitCycles) { ok = false; break; }
        __nanosleep(64);
      }
      if (!ok || bar->failed) break;
    }
  } else {
    // ---- A producers: thread = (row, half of a 64-column chunk); (dG[a] + dG[b]) -> split -> TMEM ring
    const int q = warp & 3, half = (warp - kProducerWarp0) >> 2;
    const int row = q * 32 + lane;
    int64_t it = 0;
    for (int64_t t = 0; t < my_tiles; ++t) {
      const int64_t g = (blockIdx.x + t * gridDim.x) * kRows + row;
      const int64_t ra = g < nrows ? (a.pair_a ? __ldg(reinterpret_cast<const long long*>(a.pair_a + g)) : g) : -1;
      const int64_t rb = (g < nrows && a.pair_b) ? __ldg(reinterpret_cast<const long long*>(a.pair_b + g)) : -1;
      const float* pa = a.in + row_offset(ra >= 0 ? ra : 0, a.in_mm, a.in_ld) + half * 32;
      const float* pb = a.in + row_offset(rb >= 0 ? rb : 0, a.in_mm, a.in_ld) + half * 32;
      const int64_t cstep = int64_t(a.in_cs) * kChunk;
      bool ok = true;
      for (int c = 0; c < chunks; ++c, ++it) {
        const int sa = int(it % kAStagesBwd);
        float x[32];
        if (ra >= 0) {
#pragma unroll
          for (int j = 0; j < 4; ++j) ldg256(pa + c * cstep + j * 8, x + j * 8);
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) x[i] = 0.f;
        }
        if (rb >= 0) {
          float y[32];
#pragma unroll
          for (int j = 0; j < 4; ++j) ldg256(pb + c * cstep + j * 8, y + j * 8);
#pragma unroll
          for (int i = 0; i < 32; ++i) x[i] += y[i];
        }
        if (bar->failed || !mbar_wait(saddr(&bar->a_empty[sa]), unsigned((it / kAStagesBwd) & 1) ^ 1u)) {
          give_up(bar, a.status, 35);
          ok = false;
          break;
        }
        tc_fence_after();
        const unsigned t_big = tmem_a + (unsigned(q * 32) << 16) + sa * 2 * kK + half * 32;
        store_split_tmem(t_big, t_big + kK, x);
        tc_fence_before();
        mbar_arrive(saddr(&bar->a_full[sa]));
        if (warp == kProducerWarp0 && lane == 0) bar->progress = it + 1;
      }
      if (!ok) break;
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(512u) : "memory");
  }
}

// Packs W3 [nout, 64] into 64-unit chunks in the shared-memory operand layout, big part then small part.
// transpose = 0 (forward B operand):  block(n, k) = W3[c*64 + n][k]
// transpose = 1 (backward B operand): block(n, k) = W3[c*64 + k][n]
__global__ void gate_pack_kernel(int nout, const float* __restrict__ w, int transpose, float* out) {
  const int idx = blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= nout * kK) return;
  const int c = idx / (kChunk * kK), rem = idx % (kChunk * kK), n = rem / kK, k = rem % kK;
  const float v = transpose ? w[(c * kChunk + k) * kK + n] : w[(c * kChunk + n) * kK + k];
  const float big = to_tf32(v), small = to_tf32(v - big);
  const int off = (k / 4) * (kChunk * 4) + n * 4 + (k % 4);
  out[c * (2 * kChunk * kK) + off] = big;
  out[c * (2 * kChunk * kK) + kChunk * kK + off] = small;
}

static int grid_size(int64_t rows) {
  int dev = 0, sms = 148;
  if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const int64_t tiles = (rows + kRows - 1) / kRows;
  return int(tiles < sms ? tiles : sms);
}

static int check_common(int64_t rows, int nout) {
  if (rows < 0 || nout < kChunk || nout % kChunk) {
    set_error("gate gemm: the gate width must be a positive multiple of 64 (got %d)", nout);
    return ICTC_ERR_BAD_SPEC;
  }
  return ICTC_OK;
}

}  // namespace gg
}  // namespace ictc

using namespace ictc;

extern "C" {

int ictc_gate_pack_weights(int num_out, const float* w3, int transpose, float* packed, void* stream) {
  if (int rc = gg::check_common(0, num_out)) return rc;
  if (!w3 || !packed) { set_error("gate pack: NULL buffer"); return ICTC_ERR_BAD_ARG; }
  const int n = num_out * gg::kK;
  gg::gate_pack_kernel<<<(n + 255) / 256, 256, 0, (cudaStream_t)stream>>>(num_out, w3, transpose ? 1 : 0, packed);
  return finish_launch("gate_pack");
}

int ictc_gate_gemm_forward(int64_t num_rows, int num_out, const float* z3, const float* w_packed, float* gates,
                           int apply_silu, const int64_t* row_limit, void* stream) {
  if (int rc = gg::check_common(num_rows, num_out)) return rc;
  if (num_rows == 0) return ICTC_OK;
  if (!z3 || !w_packed || !gates) { set_error("gate gemm forward: NULL buffer"); return ICTC_ERR_BAD_ARG; }
  if ((reinterpret_cast<uintptr_t>(z3) | reinterpret_cast<uintptr_t>(w_packed) | reinterpret_cast<uintptr_t>(gates)) & 31) {
    set_error("gate gemm forward: buffers must be 32-byte aligned");
    return ICTC_ERR_BAD_ARG;
  }
  static const cudaError_t attr = cudaFuncSetAttribute(gg::gate_gemm_forward_kernel,
                                                       cudaFuncAttributeMaxDynamicSharedMemorySize, gg::kFwdSmem);
  if (attr != cudaSuccess) { set_error("gate gemm smem: %s", cudaGetErrorString(attr)); return ICTC_ERR_LAUNCH; }
  gg::Args a{};
  a.in = z3; a.w = w_packed; a.out = gates; a.rows = num_rows; a.limit = row_limit; a.nout = num_out; a.act = apply_silu ? 1 : 0;
  a.in_mm = a.out_mm = a.in_cs = a.out_cs = 1; a.in_ld = gg::kK; a.out_ld = num_out;
  a.status = kernel_status_word();
  gg::gate_gemm_forward_kernel<<<gg::grid_size(num_rows), gg::kThreads, gg::kFwdSmem, (cudaStream_t)stream>>>(a);
  return finish_launch("gate_gemm_forward");
}

int ictc_gate_gemm_backward(int64_t num_rows, int num_out, const float* dgates, const int64_t* pair_a,
                            const int64_t* pair_b, const float* w_packed_t, float* da3, const int64_t* row_limit,
                            void* stream) {
  if (int rc = gg::check_common(num_rows, num_out)) return rc;
  if (num_rows == 0) return ICTC_OK;
  if (!dgates || !w_packed_t || !da3) { set_error("gate gemm backward: NULL buffer"); return ICTC_ERR_BAD_ARG; }
  if ((reinterpret_cast<uintptr_t>(dgates) | reinterpret_cast<uintptr_t>(w_packed_t) | reinterpret_cast<uintptr_t>(da3)) & 31) {
    set_error("gate gemm backward: buffers must be 32-byte aligned");
    return ICTC_ERR_BAD_ARG;
  }
  static const cudaError_t attr = cudaFuncSetAttribute(gg::gate_gemm_backward_kernel,
                                                       cudaFuncAttributeMaxDynamicSharedMemorySize, gg::kBwdSmem);
  if (attr != cudaSuccess) { set_error("gate gemm smem: %s", cudaGetErrorString(attr)); return ICTC_ERR_LAUNCH; }
  gg::Args a{};
  a.in = dgates; a.w = w_packed_t; a.out = da3; a.pair_a = pair_a; a.pair_b = pair_b; a.rows = num_rows; a.limit = row_limit; a.nout = num_out;
  a.in_mm = a.out_mm = a.in_cs = a.out_cs = 1; a.in_ld = num_out; a.out_ld = gg::kK;
  a.status = kernel_status_word();
  gg::gate_gemm_backward_kernel<<<gg::grid_size(num_rows), gg::kThreads, gg::kBwdSmem, (cudaStream_t)stream>>>(a);
  return finish_launch("gate_gemm_backward");
}


int ictc_gate_gemm_forward_rows(int64_t capacity, int num_out, const float* z3, const int64_t* row_index,
                                const int64_t* row_begin, const int64_t* row_end, const float* w_packed, float* gates,
                                int apply_silu, void* stream) {
  if (int rc = gg::check_common(capacity, num_out)) return rc;
  if (capacity == 0) return ICTC_OK;
  if (!z3 || !w_packed || !gates || !row_begin || !row_end) { set_error("gate gemm forward rows: NULL buffer"); return ICTC_ERR_BAD_ARG; }
  if ((reinterpret_cast<uintptr_t>(z3) | reinterpret_cast<uintptr_t>(w_packed) | reinterpret_cast<uintptr_t>(gates)) & 31) {
    set_error("gate gemm forward rows: buffers must be 32-byte aligned");
    return ICTC_ERR_BAD_ARG;
  }
  static const cudaError_t attr = cudaFuncSetAttribute(gg::gate_gemm_forward_kernel,
                                                       cudaFuncAttributeMaxDynamicSharedMemorySize, gg::kFwdSmem);
  if (attr != cudaSuccess) { set_error("gate gemm smem: %s", cudaGetErrorString(attr)); return ICTC_ERR_LAUNCH; }
  gg::Args a{};
  a.in = z3; a.w = w_packed; a.out = gates; a.rows = capacity; a.limit = row_end; a.begin = row_begin; a.in_index = row_index;
  a.nout = num_out; a.act = apply_silu ? 1 : 0;
  a.in_mm = a.out_mm = a.in_cs = a.out_cs = 1; a.in_ld = gg::kK; a.out_ld = num_out;
  a.status = kernel_status_word();
  gg::gate_gemm_forward_kernel<<<gg::grid_size(capacity), gg::kThreads, gg::kFwdSmem, (cudaStream_t)stream>>>(a);
  return finish_launch("gate_gemm_forward_rows");
}

int ictc_gate_gemm_backward_rows(int64_t capacity, int num_out, const float* dgates, const int64_t* row_begin,
                                 const int64_t* row_end, const int64_t* out_index, const float* w_packed_t, float* da3,
                                 void* stream) {
  if (int rc = gg::check_common(capacity, num_out)) return rc;
  if (capacity == 0) return ICTC_OK;
  if (!dgates || !w_packed_t || !da3 || !row_begin || !row_end) { set_error("gate gemm backward rows: NULL buffer"); return ICTC_ERR_BAD_ARG; }
  if ((reinterpret_cast<uintptr_t>(dgates) | reinterpret_cast<uintptr_t>(w_packed_t) | reinterpret_cast<uintptr_t>(da3)) & 31) {
    set_error("gate gemm backward rows: buffers must be 32-byte aligned");
    return ICTC_ERR_BAD_ARG;
  }
  static const cudaError_t attr = cudaFuncSetAttribute(gg::gate_gemm_backward_kernel,
                                                       cudaFuncAttributeMaxDynamicSharedMemorySize, gg::kBwdSmem);
  if (attr != cudaSuccess) { set_error("gate gemm smem: %s", cudaGetErrorString(attr)); return ICTC_ERR_LAUNCH; }
  gg::Args a{};
  a.in = dgates; a.w = w_packed_t; a.out = da3; a.rows = capacity; a.limit = row_end; a.begin = row_begin; a.out_index = out_index;
  a.nout = num_out;
  a.in_mm = a.out_mm = a.in_cs = a.out_cs = 1; a.in_ld = num_out; a.out_ld = gg::kK;
  a.status = kernel_status_word();
  gg::gate_gemm_backward_kernel<<<gg::grid_size(capacity), gg::kThreads, gg::kBwdSmem, (cudaStream_t)stream>>>(a);
  return finish_launch("gate_gemm_backward_rows");
}


int ictc_channel_linear_tc(int64_t num_rows, int k_chunks, int n_chunks, const float* in, int in_mm, int64_t in_ld,
                           const float* w_packed, float* out, int out_mm, int64_t out_ld, void* stream) {
  if (num_rows < 0 || k_chunks < 1 || n_chunks < 1 || (k_chunks > 1 && n_chunks > 1) || in_mm < 1 || out_mm < 1 ||
      in_ld < 0 || out_ld < 0) {
    set_error("channel linear: one side must be 64 wide, the other a multiple of 64 (got %d x %d chunks)", k_chunks,
              n_chunks);
    return ICTC_ERR_BAD_SPEC;
  }
  if (num_rows == 0) return ICTC_OK;
  if (!in || !w_packed || !out) { set_error("channel linear: NULL buffer"); return ICTC_ERR_BAD_ARG; }
  if (((reinterpret_cast<uintptr_t>(in) | reinterpret_cast<uintptr_t>(w_packed) | reinterpret_cast<uintptr_t>(out)) & 31) ||
      (in_ld & 7) || (out_ld & 7)) {
    set_error("channel linear: buffers must be 32-byte aligned and strides multiples of 8 floats");
    return ICTC_ERR_BAD_ARG;
  }
  gg::Args a{};
  a.in = in; a.w = w_packed; a.out = out; a.rows = num_rows; a.status = kernel_status_word();
  a.in_mm = in_mm; a.out_mm = out_mm; a.in_ld = in_ld; a.out_ld = out_ld;
  a.in_cs = in_mm; a.out_cs = out_mm;
  if (k_chunks == 1) {
    static const cudaError_t attr = cudaFuncSetAttribute(gg::gate_gemm_forward_kernel,
                                                         cudaFuncAttributeMaxDynamicSharedMemorySize, gg::kFwdSmem);
    if (attr != cudaSuccess) { set_error("channel linear smem: %s", cudaGetErrorString(attr)); return ICTC_ERR_LAUNCH; }
    a.nout = n_chunks * gg::kChunk;
    gg::gate_gemm_forward_kernel<<<gg::grid_size(num_rows), gg::kThreads, gg::kFwdSmem, (cudaStream_t)stream>>>(a);
  } else {
    static const cudaError_t attr = cudaFuncSetAttribute(gg::gate_gemm_backward_kernel,
                                                         cudaFuncAttributeMaxDynamicSharedMemorySize, gg::kBwdSmem);
    if (attr != cudaSuccess) { set_error("channel linear smem: %s", cudaGetErrorString(attr)); return ICTC_ERR_LAUNCH; }
    a.nout = k_chunks * gg::kChunk;
    gg::gate_gemm_backward_kernel<<<gg::grid_size(num_rows), gg::kThreads, gg::kBwdSmem, (cudaStream_t)stream>>>(a);
  }
  return finish_launch("channel_linear_tc");
}

}  // extern "C"
