// Gated Clebsch-Gordan tensor product in the ICTC basis: device bodies and kernels.
//
// Math (per edge e, path p=(l1,l2,l3), channel c; reference: ictc_o3/basis/ictd_irreps.py:2849-2971,
// kernel form ictc_o3/backends/k100/generated_cartesian_message.py:179-224):
//   t[k]    = sum_{(i,j)} C[i,j,k] * x[i] * sh[j]            (sparse couplings, literals in code)
//   out[k] += t[k] * ge[p(k)],   ge[p] = g[e,p,c] * w[p,c] * mask[e]
// First adjoint with cotangent v:
//   zq[(i,p)] = sum_{(j,k) in p} C[i,j,k] * sh[j] * v[k]
//   dx[i]    += sum_p zq[(i,p)] * ge[p]
//   dg[p]     = w[p] * mask * sum_i x[i] * zq[(i,p)]
//   dsh[j]    = sum_c sum_{(i,k)} C[i,j,k] * x[i] * v[k] * ge[p(k)]
//
// Thread mapping: one lane = one channel, so every feature/gate/output access of a warp is one
// coalesced 128-byte line and the harmonics of an edge are warp-uniform (broadcast loads).
// The graph kernels own an output row per warp and walk a CSR segment, so the scatter-sum needs no
// atomics and its summation order is fixed.
#pragma once
#include "ictc_common.cuh"
#include "generated/tp_spec_tables.cuh"

namespace ictc {

template <int ID> struct TpSpec;

#define ICTC_M_COUPLE_F(i, j, k, p, c) t[k] = (x[i] * sh[j]) * (c);
#define ICTC_M_COUPLE_A(i, j, k, p, c) t[k] = fmaf(x[i] * sh[j], (c), t[k]);
#define ICTC_M_GATE(k, p) acc[k] = fmaf(t[k], ge[p], acc[k]);
#define ICTC_M_ZQ_F(q, j, k, c) zq[q] = (sh[j] * v[k]) * (c);
#define ICTC_M_ZQ_A(q, j, k, c) zq[q] = fmaf(sh[j] * v[k], (c), zq[q]);
#define ICTC_M_DX(q, i, p) dx[i] = fmaf(zq[q], ge[p], dx[i]);
#define ICTC_M_DG_F(q, i, p) dg[p] = x[i] * zq[q];
#define ICTC_M_DG_A(q, i, p) dg[p] = fmaf(x[i], zq[q], dg[p]);
#define ICTC_M_VG(k, p) vg[k] = v[k] * ge[p];
#define ICTC_M_DSH_F(i, j, k, p, c) dsh[j] = (x[i] * vg[k]) * (c);
#define ICTC_M_DSH_A(i, j, k, p, c) dsh[j] = fmaf(x[i] * vg[k], (c), dsh[j]);

#define ICTC_TP_DEFINE(S)                                                                            \
  template <> struct TpSpec<ICTC_TP_##S##_ID> {                                                      \
    static constexpr int NX = ICTC_TP_##S##_NX, NH = ICTC_TP_##S##_NH, NP = ICTC_TP_##S##_NP,        \
                         NO = ICTC_TP_##S##_NO, NQ = ICTC_TP_##S##_NQ, NNZ = ICTC_TP_##S##_NNZ;      \
    static __device__ __forceinline__ void couple(const float (&x)[NX], const float (&sh)[NH],      \
                                                  float (&t)[NO]) {                                  \
      ICTC_TP_##S##_BYK(ICTC_M_COUPLE_F, ICTC_M_COUPLE_A)                                            \
    }                                                                                                \
    static __device__ __forceinline__ void gate_acc(const float (&t)[NO], const float (&ge)[NP],    \
                                                    float (&acc)[NO]) {                              \
      ICTC_TP_##S##_OUTP(ICTC_M_GATE)                                                                \
    }                                                                                                \
    static __device__ __forceinline__ void zq(const float (&sh)[NH], const float (&v)[NO],          \
                                              float (&zq)[NQ]) {                                     \
      ICTC_TP_##S##_BYQ(ICTC_M_ZQ_F, ICTC_M_ZQ_A)                                                    \
    }                                                                                                \
    static __device__ __forceinline__ void dx_acc(const float (&zq)[NQ], const float (&ge)[NP],     \
                                                  float (&dx)[NX]) {                                 \
      ICTC_TP_##S##_QLIST(ICTC_M_DX)                                                                 \
    }                                                                                                \
    static __device__ __forceinline__ void dgate(const float (&x)[NX], const float (&zq)[NQ],       \
                                                 float (&dg)[NP]) {                                  \
      ICTC_TP_##S##_QBYP(ICTC_M_DG_F, ICTC_M_DG_A)                                                   \
    }                                                                                                \
    static __device__ __forceinline__ void dharm(const float (&x)[NX], const float (&v)[NO],        \
                                                 const float (&ge)[NP], float (&dsh)[NH]) {          \
      float vg[NO];                                                                                  \
      ICTC_TP_##S##_OUTP(ICTC_M_VG)                                                                  \
      _Pragma("unroll") for (int j = 0; j < NH; ++j) dsh[j] = 0.f;                                   \
      ICTC_TP_##S##_BYJ(ICTC_M_DSH_F, ICTC_M_DSH_A)                                                  \
    }                                                                                                \
  };

struct TpArgs {
  const float* x;       // [rows, NX*C]
  const float* sh;      // [E, NH]
  const float* w;       // [NP*C] or null
  const float* g;       // [E, NP*C]
  const float* mask;    // [E] or null
  const float* v;       // cotangent of out (adjoint only)
  float* out;           // forward output
  float* dx;            // adjoint outputs (nullable)
  float* dsh;
  float* dg;
  const int64_t* nbr;     // forward: src[E]; adjoint: dst[E]   (graph kernels)
  const int64_t* rowptr;  // CSR over the owner of the reduction
  const int64_t* order;   // CSR edge order or null (identity)
  const int64_t* grow;    // row of every edge in the gate table, or null (row = edge id)
  int64_t N, E;
  int C;
  int* status;          // device status word for kernels with bounded waits (may be null)
  // Chunked evaluation (graph kernels; all optional).  A chunk is a range of owner rows whose gate rows, and for
  // the adjoint gate-gradient rows, live in a buffer that covers only the chunk's edges.
  const int64_t* g_base;   // device scalar subtracted from the gate row; rows are then clamped to [0, g_cap)
  const int64_t* dg_base;  // device scalar: the gate gradient of the edge at CSR position q goes to row q - *dg_base
                           // (rows outside [0, dg_cap) are not stored); null: row = edge id
  int64_t g_cap, dg_cap;
  int g_by_pos;            // gate row = CSR position of the edge instead of grow[e] / e
};

// Row of edge e, found at position `pos` of the owner's CSR walk, in the gate table.
__device__ __forceinline__ int64_t gate_row_of(const TpArgs& a, int64_t e, int64_t pos) {
  int64_t r = a.g_by_pos ? pos : (a.grow ? ldg(a.grow + e) : e);
  if (a.g_base) {
    r -= ldg(a.g_base);
    r = r < 0 ? 0 : (r >= a.g_cap ? a.g_cap - 1 : r);
  }
  return r;
}
// Row of the edge's gate gradient; negative: outside the caller's buffer, do not store.
__device__ __forceinline__ int64_t dg_row_of(const TpArgs& a, int64_t e, int64_t pos) {
  if (!a.dg_base) return e;
  const int64_t r = pos - ldg(a.dg_base);
  return (r >= 0 && r < a.dg_cap) ? r : -1;
}

// ---------------------------------------------------------------------------------------------
// Edge-owned forward: one warp per (edge, 32-channel tile).
template <class S>
__global__ void __launch_bounds__(128) tp_edge_forward_kernel(TpArgs a) {
  const int tiles = (a.C + kWarp - 1) / kWarp;
  const int64_t wid = (int64_t(blockIdx.x) * blockDim.x + threadIdx.x) / kWarp;
  if (wid >= a.E * tiles) return;
  const int64_t e = wid / tiles;
  const int c = int(wid % tiles) * kWarp + (threadIdx.x & 31);
  if (c >= a.C) return;
  float x[S::NX], sh[S::NH], ge[S::NP], t[S::NO], acc[S::NO];
  const float mu = a.mask ? ldg(a.mask + e) : 1.f;
#pragma unroll
  for (int i = 0; i < S::NX; ++i) x[i] = ldg(a.x + (e * S::NX + i) * a.C + c);
#pragma unroll
  for (int j = 0; j < S::NH; ++j) sh[j] = ldg(a.sh + e * S::NH + j);
#pragma unroll
  for (int p = 0; p < S::NP; ++p) {
    float gv = ldg(a.g + (e * S::NP + p) * a.C + c) * mu;
    ge[p] = a.w ? gv * ldg(a.w + p * a.C + c) : gv;
  }
#pragma unroll
  for (int k = 0; k < S::NO; ++k) acc[k] = 0.f;
  S::couple(x, sh, t);
  S::gate_acc(t, ge, acc);
#pragma unroll
  for (int k = 0; k < S::NO; ++k) a.out[(e * S::NO + k) * a.C + c] = acc[k];
}

// ---------------------------------------------------------------------------------------------
// Receiver-owned graph forward: one warp per (receiver, 32-channel tile) walks the receiver's CSR
// segment and keeps the NO output components of its channel in registers.
template <class S>
__global__ void __launch_bounds__(128) tp_graph_forward_kernel(TpArgs a) {
  const int tiles = (a.C + kWarp - 1) / kWarp;
  const int64_t wid = (int64_t(blockIdx.x) * blockDim.x + threadIdx.x) / kWarp;
  if (wid >= a.N * tiles) return;
  const int64_t n = wid / tiles;
  const int c = int(wid % tiles) * kWarp + (threadIdx.x & 31);
  if (c >= a.C) return;
  float wv[S::NP], acc[S::NO];
#pragma unroll
  for (int p = 0; p < S::NP; ++p) wv[p] = a.w ? ldg(a.w + p * a.C + c) : 1.f;
#pragma unroll
  for (int k = 0; k < S::NO; ++k) acc[k] = 0.f;
  const int64_t begin = ldg(a.rowptr + n), end = ldg(a.rowptr + n + 1);
  for (int64_t it = begin; it < end; ++it) {
    const int64_t e = a.order ? ldg(a.order + it) : it;
    const int64_t s = ldg(a.nbr + e);
    const float mu = a.mask ? ldg(a.mask + e) : 1.f;
    float x[S::NX], sh[S::NH], ge[S::NP], t[S::NO];
#pragma unroll
    for (int i = 0; i < S::NX; ++i) x[i] = ldg(a.x + (s * S::NX + i) * a.C + c);
#pragma unroll
    for (int j = 0; j < S::NH; ++j) sh[j] = ldg(a.sh + e * S::NH + j);
    const int64_t gr = gate_row_of(a, e, it);
#pragma unroll
    for (int p = 0; p < S::NP; ++p) ge[p] = ldg(a.g + (gr * S::NP + p) * a.C + c) * (wv[p] * mu);
    S::couple(x, sh, t);
    S::gate_acc(t, ge, acc);
  }
#pragma unroll
  for (int k = 0; k < S::NO; ++k) a.out[(n * S::NO + k) * a.C + c] = acc[k];
}

// ---------------------------------------------------------------------------------------------
// Adjoint, shared by the edge-owned and the sender-owned (graph) variants.
//   GRAPH = false: block = all channel tiles of ONE edge (rows of x/v/dx are edge rows).
//   GRAPH = true : block = all channel tiles of ONE sender node; it walks the sender's out-edges,
//                  gathers v at dst[e] and reduces dx in registers.
// dsh needs a sum over channels: warp shuffle inside a tile, then a fixed-order sum over the tiles
// through shared memory (kChunk edges per round), so the result is bitwise reproducible.
constexpr int kAdjChunk = 16;
constexpr int kMaxTiles = 32;  // block = 32*tiles threads <= 1024

template <class S, bool GRAPH, bool NEEDX, bool NEEDH, bool NEEDG>
__global__ void tp_adjoint_kernel(TpArgs a) {
  extern __shared__ float smem[];  // [tiles][kAdjChunk][NH] when NEEDH && tiles > 1
  const int tiles = blockDim.x / kWarp;
  const int tile = threadIdx.x / kWarp, lane = threadIdx.x & 31;
  const int c = tile * kWarp + lane;
  const bool on = c < a.C;
  const int cc = on ? c : 0;  // inactive lanes read channel 0 and contribute nothing
  const int64_t owner = blockIdx.x;
  float wv[S::NP], x[S::NX], dx[S::NX];
#pragma unroll
  for (int p = 0; p < S::NP; ++p) wv[p] = a.w ? ldg(a.w + p * a.C + cc) : 1.f;
#pragma unroll
  for (int i = 0; i < S::NX; ++i) {
    x[i] = ldg(a.x + (owner * S::NX + i) * a.C + cc);
    dx[i] = 0.f;
  }
  int64_t begin, end;
  if (GRAPH) {
    begin = ldg(a.rowptr + owner);
    end = ldg(a.rowptr + owner + 1);
  } else {
    begin = owner;
    end = owner + 1;
  }
  for (int64_t base = begin; base < end; base += kAdjChunk) {
    const int cnt = int(end - base < kAdjChunk ? end - base : kAdjChunk);
    for (int q = 0; q < cnt; ++q) {
      const int64_t e = (GRAPH && a.order) ? ldg(a.order + base + q) : base + q;
      const int64_t vrow = GRAPH ? ldg(a.nbr + e) : e;
      const int64_t gr = gate_row_of(a, e, base + q);
      const int64_t dgr = dg_row_of(a, e, base + q);
      const float mu = a.mask ? ldg(a.mask + e) : 1.f;
      float sh[S::NH], ge[S::NP], v[S::NO];
#pragma unroll
      for (int j = 0; j < S::NH; ++j) sh[j] = ldg(a.sh + e * S::NH + j);
#pragma unroll
      for (int p = 0; p < S::NP; ++p) ge[p] = ldg(a.g + (gr * S::NP + p) * a.C + cc) * (wv[p] * mu);
#pragma unroll
      for (int k = 0; k < S::NO; ++k) v[k] = on ? ldg(a.v + (vrow * S::NO + k) * a.C + cc) : 0.f;
      if (NEEDX || NEEDG) {
        float zq[S::NQ];
        S::zq(sh, v, zq);
        if (NEEDX) S::dx_acc(zq, ge, dx);
        if (NEEDG) {
          float dg[S::NP];
          S::dgate(x, zq, dg);
          if (on && dgr >= 0) {
#pragma unroll
            for (int p = 0; p < S::NP; ++p) a.dg[(dgr * S::NP + p) * a.C + c] = dg[p] * (wv[p] * mu);
          }
        }
      }
      if (NEEDH) {
        float dsh[S::NH];
        S::dharm(x, v, ge, dsh);
#pragma unroll
        for (int j = 0; j < S::NH; ++j) dsh[j] = warp_sum(dsh[j]);
        if (tiles == 1) {
          if (lane == 0) {
#pragma unroll
            for (int j = 0; j < S::NH; ++j) a.dsh[e * S::NH + j] = dsh[j];
          }
        } else if (lane == 0) {
#pragma unroll
          for (int j = 0; j < S::NH; ++j) smem[(tile * kAdjChunk + q) * S::NH + j] = dsh[j];
        }
      }
    }
    if (NEEDH && tiles > 1) {
      __syncthreads();
      for (int idx = threadIdx.x; idx < cnt * S::NH; idx += blockDim.x) {
        const int q = idx / S::NH, j = idx % S::NH;
        float sum = 0.f;
        for (int tt = 0; tt < tiles; ++tt) sum += smem[(tt * kAdjChunk + q) * S::NH + j];
        const int64_t e = (GRAPH && a.order) ? ldg(a.order + base + q) : base + q;
        a.dsh[e * S::NH + j] = sum;
      }
      __syncthreads();
    }
  }
  if (NEEDX && on) {
#pragma unroll
    for (int i = 0; i < S::NX; ++i) a.dx[(owner * S::NX + i) * a.C + c] = dx[i];
  }
}

// ---------------------------------------------------------------------------------------------
// Host launchers of one spec, reached through a table so that every spec compiles in its own
// translation unit.
struct TpOps {
  int nx, nh, np, no, nnz;
  int (*edge_forward)(const TpArgs&, cudaStream_t);
  int (*graph_forward)(const TpArgs&, cudaStream_t);
  int (*adjoint)(const TpArgs&, bool graph, cudaStream_t);
};

template <class S> int launch_edge_forward(const TpArgs& a, cudaStream_t st) {
  if (a.E == 0) return ICTC_OK;
  const int64_t tiles = (a.C + kWarp - 1) / kWarp;
  const int64_t blocks = (a.E * tiles + 3) / 4;
  if (blocks > 2147483647LL) { set_error("edge forward: too many rows"); return ICTC_ERR_TOO_LARGE; }
  tp_edge_forward_kernel<S><<<(unsigned)blocks, 128, 0, st>>>(a);
  return finish_launch("tp_edge_forward");
}

template <class S> int launch_graph_forward(const TpArgs& a, cudaStream_t st) {
  if (a.N == 0) return ICTC_OK;
  const int64_t tiles = (a.C + kWarp - 1) / kWarp;
  const int64_t blocks = (a.N * tiles + 3) / 4;
  if (blocks > 2147483647LL) { set_error("graph forward: too many rows"); return ICTC_ERR_TOO_LARGE; }
  tp_graph_forward_kernel<S><<<(unsigned)blocks, 128, 0, st>>>(a);
  return finish_launch("tp_graph_forward");
}

template <class S, bool GRAPH, bool NX_, bool NH_, bool NG_>
int launch_adjoint_one(const TpArgs& a, cudaStream_t st) {
  const int tiles = (a.C + kWarp - 1) / kWarp;
  const int64_t owners = GRAPH ? a.N : a.E;
  const size_t smem = (NH_ && tiles > 1) ? size_t(tiles) * kAdjChunk * S::NH * sizeof(float) : 0;
  tp_adjoint_kernel<S, GRAPH, NX_, NH_, NG_><<<(unsigned)owners, tiles * kWarp, smem, st>>>(a);
  return finish_launch("tp_adjoint");
}

template <class S, bool GRAPH> int launch_adjoint_g(const TpArgs& a, cudaStream_t st) {
  const int key = (a.dx ? 4 : 0) | (a.dsh ? 2 : 0) | (a.dg ? 1 : 0);
  switch (key) {
    case 1: return launch_adjoint_one<S, GRAPH, false, false, true>(a, st);
    case 2: return launch_adjoint_one<S, GRAPH, false, true, false>(a, st);
    case 3: return launch_adjoint_one<S, GRAPH, false, true, true>(a, st);
    case 4: return launch_adjoint_one<S, GRAPH, true, false, false>(a, st);
    case 5: return launch_adjoint_one<S, GRAPH, true, false, true>(a, st);
    case 6: return launch_adjoint_one<S, GRAPH, true, true, false>(a, st);
    case 7: return launch_adjoint_one<S, GRAPH, true, true, true>(a, st);
    default: return ICTC_OK;
  }
}

template <class S> int launch_adjoint(const TpArgs& a, bool graph, cudaStream_t st) {
  const int64_t owners = graph ? a.N : a.E;
  if (owners == 0) return ICTC_OK;
  if (owners > 2147483647LL) { set_error("adjoint: too many rows"); return ICTC_ERR_TOO_LARGE; }
  if ((a.C + kWarp - 1) / kWarp > kMaxTiles) { set_error("adjoint: channels > %d", kMaxTiles * kWarp); return ICTC_ERR_TOO_LARGE; }
  return graph ? launch_adjoint_g<S, true>(a, st) : launch_adjoint_g<S, false>(a, st);
}

template <class S> TpOps make_ops() {
  return TpOps{S::NX, S::NH, S::NP, S::NO, S::NNZ, &launch_edge_forward<S>, &launch_graph_forward<S>,
               &launch_adjoint<S>};
}

}  // namespace ictc
