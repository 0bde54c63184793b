// Graph-message kernels with TMA-staged rows (C = 32 or 64, 16-byte aligned buffers).
//
// Same arithmetic as tp_fast_kernels.cuh.  The wide operands of an edge — its gate row and the
// gathered feature row (forward) or cotangent row (adjoint) — are contiguous in memory, so one lane
// fetches each of them with a single bulk asynchronous copy (cp.async.bulk, global -> shared, no
// multicast) into a warp-private ring of STAGES slots and the warp picks them up from shared memory
// when an mbarrier reports the bytes have landed.  The ring keeps several edges' worth of HBM
// requests in flight per warp without holding them in registers, which is what the latency-bound
// register version lacked.  Index chains (order -> edge -> neighbour row) and the harmonics of the
// next edge are fetched ahead of use.
//
// Every mbarrier wait is bounded: when a wait runs out the warp records the fact in a device error
// word, waits (bounded again) for its outstanding copies and leaves.  The host reads the word with
// ictc_kernel_status().
#pragma once
#include "tp_fast_kernels.cuh"

namespace ictc {

constexpr long long kWaitCycles = 2000000000LL;   // about one second at the SM clock

__device__ __forceinline__ unsigned smem_addr(const void* p) {
  return static_cast<unsigned>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ void mbar_init(unsigned bar, unsigned count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(unsigned bar, unsigned bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void bulk_g2s(unsigned dst, const void* src, unsigned bytes, unsigned bar) {
  asm volatile("cp.async.bulk.shared::cta.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
               "l"(src), "r"(bytes), "r"(bar)
               : "memory");
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
// Bounded wait for the phase with the given parity; false when the time limit ran out.
__device__ __forceinline__ bool mbar_wait(unsigned bar, unsigned parity) {
  if (mbar_try(bar, parity)) return true;
  const long long start = clock64();
  while (!mbar_try(bar, parity))
    if (clock64() - start > kWaitCycles) return false;
  return true;
}

template <int CPL> __device__ __forceinline__ Vec<CPL> lds_vec(const unsigned char* p);
template <> __device__ __forceinline__ Vec<1> lds_vec<1>(const unsigned char* p) {
  return Vec<1>{*reinterpret_cast<const float*>(p)};
}
template <> __device__ __forceinline__ Vec<2> lds_vec<2>(const unsigned char* p) {
  return Vec<2>{*reinterpret_cast<const unsigned long long*>(p)};
}

// Only the gate rows (a pure HBM stream) go through the ring; the gathered feature / cotangent rows are mostly L2
// hits and are loaded straight into registers.  Staging the 8,960-byte cotangent row of the 35-slot product in the
// ring as well (two stages, which leaves room for 8 warps per SM) was measured slower (6.99 against 6.42 ms at
// 4.3 M edges): without any memory traffic the adjoint still needs 68 % of its time, it is bound by the FP32 pipe
// and by dependent-issue latency at 3 warps per scheduler, not by the row loads.
constexpr bool kStageRows = false;

#ifndef ICTC_TMA_WARPS
#define ICTC_TMA_WARPS 1
#endif
#ifndef ICTC_TMA_MIN_WARPS
#define ICTC_TMA_MIN_WARPS 12
#endif
// Warps (= owner rows) per block and the resident warps per SM the kernels are compiled for (12 warps of 32 lanes cap
// the registers at 168 per thread).  One warp per block: a block ends with its row, no warp waits for a longer row.
constexpr int kTmaWarps = ICTC_TMA_WARPS;
constexpr int kTmaMinBlocks = ICTC_TMA_MIN_WARPS / ICTC_TMA_WARPS;
#ifndef ICTC_TMA_MIN_WARPS_ADJ
#define ICTC_TMA_MIN_WARPS_ADJ 12
#endif
constexpr int kTmaMinWarpsAdj = ICTC_TMA_MIN_WARPS_ADJ;

template <class S, class F, int CPL, int STAGES, bool ADJ> struct TmaLayout {
  static constexpr int C = 32 * CPL;
  static constexpr int R = (F::NB + 31) / 32, NBP = R * 32;
  static constexpr unsigned GATE_BYTES = S::NP * C * 4;
  static constexpr unsigned ROW_BYTES = kStageRows ? (ADJ ? S::NO : S::NX) * C * 4 : 0;
  static constexpr unsigned SLOT_BYTES = GATE_BYTES + ROW_BYTES;
  static constexpr unsigned GEO_BYTES = 2 * NBP * sizeof(Vec<CPL>);
  static constexpr unsigned BAR_OFF = STAGES * SLOT_BYTES;
  static constexpr unsigned GEO_OFF = BAR_OFF + ((STAGES * 8 + 15) / 16) * 16;
  // adjoint only: per-lane harmonic-gradient partial sums of RED_EDGES edges, one padded row of 32 lanes per
  // (edge, harmonic); lane r later adds up row r
  static constexpr int RED_EDGES = 32 / S::NH, RED_PITCH = 36;
  static constexpr unsigned RED_OFF = GEO_OFF + GEO_BYTES;
  static constexpr unsigned RED_BYTES = ADJ ? RED_EDGES * S::NH * RED_PITCH * 4 : 0;
  static constexpr unsigned WARP_BYTES = ((RED_OFF + RED_BYTES + 127) / 128) * 128;
  static constexpr unsigned BLOCK_BYTES = WARP_BYTES * kTmaWarps;
};

// ------------------------------------------------------------------------------------------------
template <class S, class F, int CPL, int STAGES>
__global__ void __launch_bounds__(kTmaWarps * 32, kTmaMinBlocks) tp_graph_forward_tma_kernel(TpArgs a) {
  using V = Vec<CPL>;
  using L = TmaLayout<S, F, CPL, STAGES, false>;
  constexpr int C = L::C;
  extern __shared__ __align__(128) unsigned char tma_smem[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t n = int64_t(blockIdx.x) * kTmaWarps + warp;
  if (n >= a.N) return;
  unsigned char* mine = tma_smem + warp * L::WARP_BYTES;
  const unsigned bars = smem_addr(mine + L::BAR_OFF);
  V* geo = reinterpret_cast<V*>(mine + L::GEO_OFF);
  if (lane == 0) {
#pragma unroll
    for (int s = 0; s < STAGES; ++s) mbar_init(bars + s * 8, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncwarp();
  BTerm bt[L::R];
#pragma unroll
  for (int r = 0; r < L::R; ++r) bt[r] = (r * 32 + lane < F::NB) ? F::fb(r * 32 + lane) : BTerm{0, 0.f, 0, 0.f};
  V acc[S::NO];
#pragma unroll
  for (int k = 0; k < S::NO; ++k) acc[k] = V::dup(0.f);
  const int64_t begin = ldg(a.rowptr + n), end = ldg(a.rowptr + n + 1);
  // edge ids and row numbers fit 32 bits (checked by the launcher): 32 x 32 -> 64-bit multiplies form the addresses
  auto edge_at = [&](int64_t it) -> int { return int(a.order ? ldg(a.order + it) : it); };
  auto row_at = [&](int e) -> int { return int(ldg(a.nbr + e)); };
  auto issue = [&](int slot, int e, int s, int64_t pos) {
    if (lane == 0) {
      const unsigned bar = bars + slot * 8;
      unsigned char* dst = mine + slot * L::SLOT_BYTES;
      mbar_expect_tx(bar, L::SLOT_BYTES);
      const int64_t gr = gate_row_of(a, e, pos);
      bulk_g2s(smem_addr(dst), a.g + gr * (S::NP * C), L::GATE_BYTES, bar);
      if (kStageRows) bulk_g2s(smem_addr(dst + L::GATE_BYTES), a.x + int64_t(s) * (S::NX * C), L::ROW_BYTES, bar);
    }
  };
  // prologue: fill the ring
#pragma unroll
  for (int k = 0; k < STAGES; ++k)
    if (begin + k < end) {
      const int e = edge_at(begin + k);
      issue(k, e, row_at(e), begin + k);
    }
  // (edge id, sender) of the edge that will be issued at the END of this iteration, started early
  int e_pf = 0, s_pf = 0;
  if (begin + STAGES < end) {
    e_pf = edge_at(begin + STAGES);
    s_pf = row_at(e_pf);
  }
  int e_cur = begin < end ? edge_at(begin) : 0;
  int r_cur = begin < end ? row_at(e_cur) : 0;
  float shv = (begin < end && lane < S::NH) ? ldg(a.sh + int64_t(e_cur) * S::NH + lane) : 0.f;
  int slot = 0, buf = 0;
  unsigned parity = 0;
  for (int64_t it = begin; it < end; ++it, buf ^= 1) {
    const int e = e_cur;
    const float sh_now = shv;
    V ge[S::NP], x[S::NX];
    if (!kStageRows) {
      const float* xp = a.x + int64_t(r_cur) * (S::NX * C) + lane * CPL;
#pragma unroll
      for (int i = 0; i < S::NX; ++i) x[i] = V::load(xp + i * C);
    }
    // start the index/harmonic loads of later edges before blocking on this edge's data
    int e_pf2 = 0, s_pf2 = 0;
    if (it + 1 < end) {
      e_cur = edge_at(it + 1);
      r_cur = row_at(e_cur);
      shv = lane < S::NH ? ldg(a.sh + int64_t(e_cur) * S::NH + lane) : 0.f;
    }
    if (it + STAGES + 1 < end) {
      e_pf2 = edge_at(it + STAGES + 1);
      s_pf2 = row_at(e_pf2);
    }
    V* sb = geo + buf * L::NBP;
    build_geometry<F::NB, CPL, L::R>(bt, sh_now, lane, sb);
    if (!mbar_wait(bars + slot * 8, parity)) {
      if (lane == 0 && a.status) atomicExch(a.status, 1);
      // drain the copies that are still in flight into this warp's shared memory before leaving: slots below
      // `slot` were consumed and refilled in this round (their copy completes the NEXT phase), the others
      // hold this round's copies; a slot is waited for only if an edge was really issued into it
      for (int s = 0; s < STAGES; ++s) {
        const bool refilled = s < slot;
        const int64_t owner = it - slot + s + (refilled ? STAGES : 0);
        if (owner < end) mbar_wait(bars + s * 8, refilled ? parity ^ 1u : parity);
      }
      return;
    }
    const unsigned char* base = mine + slot * L::SLOT_BYTES + lane * (CPL * 4);
#pragma unroll
    for (int p = 0; p < S::NP; ++p) ge[p] = lds_vec<CPL>(base + p * (C * 4));
    if (kStageRows) {
#pragma unroll
      for (int i = 0; i < S::NX; ++i) x[i] = lds_vec<CPL>(base + L::GATE_BYTES + i * (C * 4));
    }
    if (a.mask || a.w) {
      const V mu = V::dup(a.mask ? ldg(a.mask + e) : 1.f);
#pragma unroll
      for (int p = 0; p < S::NP; ++p) {
        ge[p] = vmul(ge[p], mu);
        if (a.w) ge[p] = vmul(ge[p], V::load(a.w + p * C + lane * CPL));
      }
    }
    __syncwarp();   // geometry visible; every lane has read its slot data into registers
    F::forward(x, ge, sb, acc);
    // the slot's values were consumed by the arithmetic above: refill it for edge it + STAGES
    if (it + STAGES < end) issue(slot, e_pf, s_pf, it + STAGES);
    e_pf = e_pf2;
    s_pf = s_pf2;
    if (++slot == STAGES) {
      slot = 0;
      parity ^= 1;
    }
  }
  float* op = a.out + n * (S::NO * C) + lane * CPL;
#pragma unroll
  for (int k = 0; k < S::NO; ++k) acc[k].store(op + k * C);
}

// ------------------------------------------------------------------------------------------------
// PLAIN: no edge mask and no path weights (decided on the host), so the per-path scaling code is not compiled in.
template <class S, class F, int CPL, int STAGES, bool GRAPH, bool NEEDX, bool NEEDH, bool NEEDG, bool PLAIN>
__global__ void __launch_bounds__(kTmaWarps * 32, kTmaMinWarpsAdj / kTmaWarps) tp_adjoint_tma_kernel(TpArgs a) {
  using V = Vec<CPL>;
  using L = TmaLayout<S, F, CPL, STAGES, true>;
  constexpr int C = L::C;
  extern __shared__ __align__(128) unsigned char tma_smem[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t owner = int64_t(blockIdx.x) * kTmaWarps + warp;
  if (owner >= (GRAPH ? a.N : a.E)) return;
  unsigned char* mine = tma_smem + warp * L::WARP_BYTES;
  const unsigned bars = smem_addr(mine + L::BAR_OFF);
  V* geo = reinterpret_cast<V*>(mine + L::GEO_OFF);
  if (lane == 0) {
#pragma unroll
    for (int s = 0; s < STAGES; ++s) mbar_init(bars + s * 8, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncwarp();
  BTerm bt[L::R];
#pragma unroll
  for (int r = 0; r < L::R; ++r) bt[r] = (r * 32 + lane < F::NB) ? F::ap(r * 32 + lane) : BTerm{0, 0.f, 0, 0.f};
  V x[S::NX], dx[S::NX];
  {
    const float* xp = a.x + owner * (S::NX * C) + lane * CPL;
#pragma unroll
    for (int i = 0; i < S::NX; ++i) {
      x[i] = V::load(xp + i * C);
      dx[i] = V::dup(0.f);
    }
  }
  int64_t begin = owner, end = owner + 1;
  if (GRAPH) {
    begin = ldg(a.rowptr + owner);
    end = ldg(a.rowptr + owner + 1);
  }
  auto edge_at = [&](int64_t it) -> int { return int((GRAPH && a.order) ? ldg(a.order + it) : it); };
  auto row_of = [&](int e) -> int { return GRAPH ? int(ldg(a.nbr + e)) : e; };
  auto issue = [&](int slot, int e, int d, int64_t pos) {
    if (lane == 0) {
      const unsigned bar = bars + slot * 8;
      unsigned char* dst = mine + slot * L::SLOT_BYTES;
      mbar_expect_tx(bar, L::SLOT_BYTES);
      const int64_t gr = gate_row_of(a, e, pos);
      bulk_g2s(smem_addr(dst), a.g + gr * (S::NP * C), L::GATE_BYTES, bar);
      if (kStageRows) bulk_g2s(smem_addr(dst + L::GATE_BYTES), a.v + int64_t(d) * (S::NO * C), L::ROW_BYTES, bar);
    }
  };
#pragma unroll
  for (int k = 0; k < STAGES; ++k)
    if (begin + k < end) {
      const int e = edge_at(begin + k);
      issue(k, e, row_of(e), begin + k);
    }
  int e_pf = 0, d_pf = 0;
  if (begin + STAGES < end) {
    e_pf = edge_at(begin + STAGES);
    d_pf = row_of(e_pf);
  }
  int e_cur = begin < end ? edge_at(begin) : 0;
  int r_cur = begin < end ? row_of(e_cur) : 0;
  float shv = (begin < end && lane < S::NH) ? ldg(a.sh + int64_t(e_cur) * S::NH + lane) : 0.f;
  int slot = 0, buf = 0;
  unsigned parity = 0;
  float* red = reinterpret_cast<float*>(mine + L::RED_OFF);
  int batch_edge[L::RED_EDGES];
  int batch = 0;
  for (int64_t it = begin; it < end; ++it, buf ^= 1) {
    const int e = e_cur;
    const float sh_now = shv;
    static_assert(!kStageRows, "the path-major adjoint reads the cotangent row from global memory");
    const float* vp = a.v + int64_t(r_cur) * (S::NO * C) + lane * CPL;     // this edge's cotangent row, read slot by slot
    int e_pf2 = 0, d_pf2 = 0;
    if (it + 1 < end) {
      e_cur = edge_at(it + 1);
      r_cur = row_of(e_cur);
      shv = lane < S::NH ? ldg(a.sh + int64_t(e_cur) * S::NH + lane) : 0.f;
    }
    if (it + STAGES + 1 < end) {
      e_pf2 = edge_at(it + STAGES + 1);
      d_pf2 = row_of(e_pf2);
    }
    V* sb = geo + buf * L::NBP;
    build_geometry<F::NB, CPL, L::R>(bt, sh_now, lane, sb);
    if (!mbar_wait(bars + slot * 8, parity)) {
      if (lane == 0 && a.status) atomicExch(a.status, 2);
      for (int s = 0; s < STAGES; ++s) {     // drain, as in the forward kernel
        const bool refilled = s < slot;
        const int64_t owner = it - slot + s + (refilled ? STAGES : 0);
        if (owner < end) mbar_wait(bars + s * 8, refilled ? parity ^ 1u : parity);
      }
      return;
    }
    const unsigned char* base = mine + slot * L::SLOT_BYTES + lane * (CPL * 4);
    const bool scaled = !PLAIN && (a.mask || a.w);
    const V mu = V::dup((scaled && a.mask) ? ldg(a.mask + e) : 1.f);
    auto scale_of = [&](int p) -> V { return a.w ? vmul(mu, V::load(a.w + p * C + lane * CPL)) : mu; };
    auto gate = [&](int p) -> V {
      const V g = lds_vec<CPL>(base + p * (C * 4));
      if (PLAIN) return g;
      return scaled ? vmul(g, scale_of(p)) : g;
    };
    int dgr = e;            // row of this edge's gate gradient (negative: outside the caller's window, not stored)
    if (NEEDG && a.dg_base) {
      const int64_t r = it - ldg(a.dg_base);
      dgr = (r >= 0 && r < a.dg_cap) ? int(r) : -1;
    }
    float* dgp = a.dg + int64_t(dgr < 0 ? 0 : dgr) * (S::NP * C) + lane * CPL;
    auto store_dg = [&](int p, V val) {
      if (PLAIN) {
        if (dgr >= 0) val.store(dgp + p * C);
      } else if (dgr >= 0) {
        (scaled ? vmul(val, scale_of(p)) : val).store(dgp + p * C);
      }
    };
    __syncwarp();   // geometry visible to every lane
    V dshv[S::NH];
#pragma unroll
    for (int j = 0; j < S::NH; ++j) dshv[j] = V::dup(0.f);
    auto cot = [&](int k) -> V { return V::load(vp + k * C); };      // slot k of the cotangent row
    F::template adjoint_fused<NEEDX, NEEDH, NEEDG>(x, cot, gate, sb, dx, dshv, store_dg);
    __syncwarp();   // every lane is done with the slot and the geometry buffer
    if (NEEDH) {
      // The sum over the 32 lanes goes through shared memory: every lane parks its NH partial sums in column `lane`
      // of the batch buffer; once RED_EDGES edges are in (or the row ends) lane r adds up row r = (edge, harmonic)
      // with eight 16-byte loads, in a fixed order.
#pragma unroll
      for (int j = 0; j < S::NH; ++j) red[(batch * S::NH + j) * L::RED_PITCH + lane] = dshv[j].hsum();
#pragma unroll
      for (int k = 0; k < L::RED_EDGES; ++k)
        if (batch == k) batch_edge[k] = e;      // unrolled so that the array stays in registers
      if (++batch == L::RED_EDGES || it + 1 == end) {
        __syncwarp();
        if (lane < batch * S::NH) {
          const float4* row = reinterpret_cast<const float4*>(red + lane * L::RED_PITCH);
          float tot = 0.f;
#pragma unroll
          for (int q = 0; q < 8; ++q) {
            const float4 t = row[q];
            tot += (t.x + t.y) + (t.z + t.w);
          }
          const int b = lane / S::NH;
          int eb = batch_edge[0];
#pragma unroll
          for (int k = 1; k < L::RED_EDGES; ++k) eb = b == k ? batch_edge[k] : eb;
          a.dsh[int64_t(eb) * S::NH + (lane - b * S::NH)] = tot;
        }
        batch = 0;
        __syncwarp();
      }
    }
    if (it + STAGES < end) issue(slot, e_pf, d_pf, it + STAGES);
    e_pf = e_pf2;
    d_pf = d_pf2;
    if (++slot == STAGES) {
      slot = 0;
      parity ^= 1;
    }
  }
  if (NEEDX) {
    float* dxp = a.dx + owner * (S::NX * C) + lane * CPL;
#pragma unroll
    for (int i = 0; i < S::NX; ++i) dx[i].store(dxp + i * C);
  }
}

// ---------------------------------------------------------------------------------------- launchers
inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

template <class K> int set_smem(K kernel, unsigned bytes) {
  cudaError_t err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
  if (err != cudaSuccess) {
    set_error("cudaFuncSetAttribute(%u bytes): %s", bytes, cudaGetErrorString(err));
    return ICTC_ERR_LAUNCH;
  }
  return ICTC_OK;
}

constexpr int kFwdStages = 4, kAdjStages = 4;

template <class S, class F, int CPL> int launch_graph_forward_tma(const TpArgs& a, cudaStream_t st) {
  using L = TmaLayout<S, F, CPL, kFwdStages, false>;
  auto kernel = tp_graph_forward_tma_kernel<S, F, CPL, kFwdStages>;
  static const int attr = set_smem(kernel, L::BLOCK_BYTES);
  if (attr != ICTC_OK) return attr;
  const int64_t blocks = (a.N + kTmaWarps - 1) / kTmaWarps;
  kernel<<<(unsigned)blocks, kTmaWarps * 32, L::BLOCK_BYTES, st>>>(a);
  return finish_launch("tp_graph_forward_tma");
}

template <class S, class F, int CPL, bool GRAPH, bool NX_, bool NH_, bool NG_, bool PLAIN>
int launch_adjoint_tma_plain(const TpArgs& a, cudaStream_t st) {
  using L = TmaLayout<S, F, CPL, kAdjStages, true>;
  auto kernel = tp_adjoint_tma_kernel<S, F, CPL, kAdjStages, GRAPH, NX_, NH_, NG_, PLAIN>;
  static const int attr = set_smem(kernel, L::BLOCK_BYTES);
  if (attr != ICTC_OK) return attr;
  const int64_t owners = GRAPH ? a.N : a.E;
  const int64_t blocks = (owners + kTmaWarps - 1) / kTmaWarps;
  kernel<<<(unsigned)blocks, kTmaWarps * 32, L::BLOCK_BYTES, st>>>(a);
  return finish_launch("tp_adjoint_tma");
}

template <class S, class F, int CPL, bool GRAPH, bool NX_, bool NH_, bool NG_>
int launch_adjoint_tma_one(const TpArgs& a, cudaStream_t st) {
  // the unscaled sender-row sweep is the molecular-dynamics case and gets its own instantiation
  if (GRAPH && !a.mask && !a.w) return launch_adjoint_tma_plain<S, F, CPL, GRAPH, NX_, NH_, NG_, GRAPH>(a, st);
  return launch_adjoint_tma_plain<S, F, CPL, GRAPH, NX_, NH_, NG_, false>(a, st);
}

template <class S, class F, int CPL, bool GRAPH> int launch_adjoint_tma_g(const TpArgs& a, cudaStream_t st) {
  const int key = (a.dx ? 4 : 0) | (a.dsh ? 2 : 0) | (a.dg ? 1 : 0);
  switch (key) {
    case 1: return launch_adjoint_tma_one<S, F, CPL, GRAPH, false, false, true>(a, st);
    case 2: return launch_adjoint_tma_one<S, F, CPL, GRAPH, false, true, false>(a, st);
    case 3: return launch_adjoint_tma_one<S, F, CPL, GRAPH, false, true, true>(a, st);
    case 4: return launch_adjoint_tma_one<S, F, CPL, GRAPH, true, false, false>(a, st);
    case 5: return launch_adjoint_tma_one<S, F, CPL, GRAPH, true, false, true>(a, st);
    case 6: return launch_adjoint_tma_one<S, F, CPL, GRAPH, true, true, false>(a, st);
    case 7: return launch_adjoint_tma_one<S, F, CPL, GRAPH, true, true, true>(a, st);
    default: return ICTC_OK;
  }
}

template <class S, int ID> int graph_forward_dispatch_tma(const TpArgs& a, cudaStream_t st) {
  if (a.N > 0 && a.E > 0 && a.E <= 2147483647LL && (a.C == 32 || a.C == 64) && a.N <= 2147483647LL &&
      aligned16(a.x) && aligned16(a.g) && aligned8(a.out) && (!a.w || aligned8(a.w))) {
    if (a.C == 64) return launch_graph_forward_tma<S, TpFast<ID, 2>, 2>(a, st);
    return launch_graph_forward_tma<S, TpFast<ID, 1>, 1>(a, st);
  }
  return graph_forward_dispatch<S, ID>(a, st);
}

template <class S, int ID> int adjoint_dispatch_tma(const TpArgs& a, bool graph, cudaStream_t st) {
  const int64_t owners = graph ? a.N : a.E;
  if (owners > 0 && a.E > 0 && a.E <= 2147483647LL && (a.C == 32 || a.C == 64) && owners <= 2147483647LL &&
      a.N <= 2147483647LL &&
      aligned16(a.g) && aligned16(a.v) && aligned8(a.x) && (!a.w || aligned8(a.w)) && (!a.dx || aligned8(a.dx)) &&
      (!a.dg || aligned8(a.dg))) {
    if (a.C == 64)
      return graph ? launch_adjoint_tma_g<S, TpFast<ID, 2>, 2, true>(a, st)
                   : launch_adjoint_tma_g<S, TpFast<ID, 2>, 2, false>(a, st);
    return graph ? launch_adjoint_tma_g<S, TpFast<ID, 1>, 1, true>(a, st)
                 : launch_adjoint_tma_g<S, TpFast<ID, 1>, 1, false>(a, st);
  }
  return adjoint_dispatch<S, ID>(a, graph, st);
}

template <class S, int ID> TpOps make_ops_tma() {
  return TpOps{S::NX, S::NH, S::NP, S::NO, S::NNZ, &launch_edge_forward<S>, &graph_forward_dispatch_tma<S, ID>,
               &adjoint_dispatch_tma<S, ID>};
}

}  // namespace ictc
