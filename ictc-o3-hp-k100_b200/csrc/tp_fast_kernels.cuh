// Fast graph-message kernels for channel counts of exactly one warp row (C = 32 or C = 64).
//
// Differences to the generic kernels in tp_kernels.cuh:
//  * Per-edge geometry.  b[i,k] = sum_j C[i,j,k] sh[j] is identical for every channel of an edge, so
//    the warp computes its NB (= 83 for lmax 2) entries once per edge, three per lane, parks them in a
//    warp-private shared-memory buffer and every lane reads them back with 16-byte broadcast loads.
//    The per-channel work drops from (products + 93 coupling FMAs) to NB FMAs.
//  * Two channels per lane for C = 64, computed with Blackwell's packed fp32 instructions
//    (fma.rn.f32x2 / mul.rn.f32x2): one issue slot does both channels and every feature / gate / output
//    access is a 64-bit load or store, 256 contiguous bytes per warp.
//  * The channel count is a compile-time constant, so row offsets are immediates in the loads.
//  * The next edge's index chain (order -> edge id -> neighbour row) is fetched one iteration ahead.
// The harmonic adjoint keeps the literal couplings (packed as {c,c} pairs in constant memory).
#pragma once
#include "tp_kernels.cuh"

namespace ictc {

struct BTerm { int j1; float c1; int j2; float c2; };

template <int CPL> struct Vec;

template <> struct Vec<1> {
  float v;
  static __device__ __forceinline__ Vec dup(float s) { return Vec{s}; }
  static __device__ __forceinline__ Vec load(const float* p) { return Vec{__ldg(p)}; }
  __device__ __forceinline__ void store(float* p) const { *p = v; }
  __device__ __forceinline__ float hsum() const { return v; }
};
__device__ __forceinline__ Vec<1> vmul(Vec<1> a, Vec<1> b) { return Vec<1>{a.v * b.v}; }
__device__ __forceinline__ Vec<1> vfma(Vec<1> a, Vec<1> b, Vec<1> c) { return Vec<1>{fmaf(a.v, b.v, c.v)}; }

template <> struct Vec<2> {
  unsigned long long v;
  static __device__ __forceinline__ Vec dup(float s) {
    Vec r;
    asm("mov.b64 %0, {%1, %1};" : "=l"(r.v) : "f"(s));
    return r;
  }
  static __device__ __forceinline__ Vec load(const float* p) {
    return Vec{__ldg(reinterpret_cast<const unsigned long long*>(p))};
  }
  __device__ __forceinline__ void store(float* p) const { *reinterpret_cast<unsigned long long*>(p) = v; }
  __device__ __forceinline__ float hsum() const {
    float lo, hi;
    asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
    return lo + hi;
  }
};
__device__ __forceinline__ Vec<2> vmul(Vec<2> a, Vec<2> b) {
  Vec<2> r;
  asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(r.v) : "l"(a.v), "l"(b.v));
  return r;
}
__device__ __forceinline__ Vec<2> vfma(Vec<2> a, Vec<2> b, Vec<2> c) {
  Vec<2> r;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r.v) : "l"(a.v), "l"(b.v), "l"(c.v));
  return r;
}

// 16-byte chunk of the shared geometry buffer: 4 entries (CPL=1) or 2 entries (CPL=2).
template <int CPL> struct Chunk;
template <> struct Chunk<1> {
  float4 c;
  static constexpr int PER = 4;
  __device__ __forceinline__ void load(const Vec<1>* base, int e) { c = *reinterpret_cast<const float4*>(base + e); }
  template <int I> __device__ __forceinline__ Vec<1> get() const {
    return Vec<1>{I == 0 ? c.x : (I == 1 ? c.y : (I == 2 ? c.z : c.w))};
  }
};
template <> struct Chunk<2> {
  ulonglong2 c;
  static constexpr int PER = 2;
  __device__ __forceinline__ void load(const Vec<2>* base, int e) { c = *reinterpret_cast<const ulonglong2*>(base + e); }
  template <int I> __device__ __forceinline__ Vec<2> get() const { return Vec<2>{I == 0 ? c.x : c.y}; }
};

// Packed coupling constants of the harmonic adjoint, per channel packing.
template <int ID, int CPL> struct TpConst;

#define ICTC_M_BT(j1, c1, j2, c2) BTerm{j1, c1, j2, c2},
#define ICTC_M_C32(c) c,
#define ICTC_M_C64(c) c,
#define ICTC_GETB(e) (ch.template get<(e) % Chunk<CPL>::PER>())
#define ICTC_LDB(e) if ((e) % Chunk<CPL>::PER == 0) ch.load(sb, (e));
#define ICTC_M_FB_F(e, i) ICTC_LDB(e) t = vmul(x[i], ICTC_GETB(e));
#define ICTC_M_FB_A(e, i) ICTC_LDB(e) t = vfma(x[i], ICTC_GETB(e), t);
#define ICTC_M_FB_K(k, p) acc[k] = vfma(t, ge[p], acc[k]);
#define ICTC_M_AB_F(e, k) ICTC_LDB(e) z = vmul(ICTC_GETB(e), v[k]);
#define ICTC_M_AB_A(e, k) ICTC_LDB(e) z = vfma(ICTC_GETB(e), v[k], z);
#define ICTC_M_AB_Q(i, p)                         \
  if (NEEDX) dx[i] = vfma(z, ge[p], dx[i]);       \
  if (NEEDG) dg[p] = vfma(x[i], z, dg[p]);
#define ICTC_M_VG2(k, p) vg[k] = vmul(v[k], ge[p]);
// path-major fused adjoint (see the ADJP program in the generated tables)
#define ICTC_M_P_PB(p) gp = gate(p); dgp = Vec<CPL>::dup(0.f);
#define ICTC_M_P_VL(k) v[k] = cot(k);
#define ICTC_M_P_ZF(e, k) ICTC_LDB(e) z = vmul(ICTC_GETB(e), v[k]);
#define ICTC_M_P_ZA(e, k) ICTC_LDB(e) z = vfma(ICTC_GETB(e), v[k], z);
#define ICTC_M_P_Q(i, p)                         \
  if (NEEDX) dx[i] = vfma(z, gp, dx[i]);         \
  if (NEEDG) dgp = vfma(x[i], z, dgp);
#define ICTC_M_P_VG(k, p) if (NEEDH) vg[k] = vmul(v[k], gp);
#define ICTC_M_P_DF(i, k) if (NEEDH) { Vec<CPL> s = vmul(x[i], vg[k]);
#define ICTC_M_P_DA(i, k) s = vfma(x[i], vg[k], s);
#define ICTC_M_P_DE(t, j) dsh[j] = vfma(s, Vec<CPL>{K::c[t]}, dsh[j]); }
#define ICTC_M_P_PE(p) if (NEEDG) store_dg(p, dgp);
#define ICTC_M_DSHT_F(t, i, j, k, p) dsh[j] = vmul(vmul(x[i], vg[k]), Vec<CPL>{K::c[t]});
#define ICTC_M_DSHT_A(t, i, j, k, p) dsh[j] = vfma(vmul(x[i], vg[k]), Vec<CPL>{K::c[t]}, dsh[j]);

#define ICTC_TP_FAST_DEFINE(S)                                                                          \
  __device__ const BTerm kFB_##S[] = {ICTC_TP_##S##_FB_TAB(ICTC_M_BT)};                                 \
  __device__ const BTerm kAB_##S[] = {ICTC_TP_##S##_AB_TAB(ICTC_M_BT)};                                 \
  __device__ const BTerm kAP_##S[] = {ICTC_TP_##S##_AP_TAB(ICTC_M_BT)};                                 \
  __constant__ float kC32_##S[] = {ICTC_TP_##S##_CLIST(ICTC_M_C32)};                                    \
  __constant__ unsigned long long kC64_##S[] = {ICTC_TP_##S##_CLIST64(ICTC_M_C64)};                     \
  template <> struct TpConst<ICTC_TP_##S##_ID, 1> { static constexpr const float* c = kC32_##S; };      \
  template <> struct TpConst<ICTC_TP_##S##_ID, 2> { static constexpr const unsigned long long* c = kC64_##S; }; \
  template <int CPL> struct TpFast<ICTC_TP_##S##_ID, CPL> {                                             \
    using Base = TpSpec<ICTC_TP_##S##_ID>;                                                              \
    using K = TpConst<ICTC_TP_##S##_ID, CPL>;                                                           \
    using V = Vec<CPL>;                                                                                 \
    static constexpr int NB = ICTC_TP_##S##_NB;                                                         \
    static __device__ __forceinline__ BTerm fb(int idx) { return kFB_##S[idx]; }                        \
    static __device__ __forceinline__ BTerm ab(int idx) { return kAB_##S[idx]; }                        \
    static __device__ __forceinline__ BTerm ap(int idx) { return kAP_##S[idx]; }                        \
    static __device__ __forceinline__ void forward(const V (&x)[Base::NX], const V (&ge)[Base::NP],     \
                                                   const V* sb, V (&acc)[Base::NO]) {                   \
      Chunk<CPL> ch;                                                                                    \
      V t;                                                                                              \
      ICTC_TP_##S##_FB(ICTC_M_FB_F, ICTC_M_FB_A, ICTC_M_FB_K)                                           \
    }                                                                                                   \
    template <bool NEEDX, bool NEEDG>                                                                   \
    static __device__ __forceinline__ void adjoint_xg(const V (&x)[Base::NX], const V (&v)[Base::NO],   \
                                                      const V (&ge)[Base::NP], const V* sb,             \
                                                      V (&dx)[Base::NX], V (&dg)[Base::NP]) {           \
      Chunk<CPL> ch;                                                                                    \
      V z;                                                                                              \
      ICTC_TP_##S##_AB(ICTC_M_AB_F, ICTC_M_AB_A, ICTC_M_AB_Q)                                           \
    }                                                                                                   \
    /* Path-major adjoint of one edge: dx (accumulated), dsh (accumulated) and the gate gradient of every   \
       path (handed to store_dg as soon as it is complete).  cot(k): this lane's part of cotangent slot k;   \
       gate(p): this lane's gate of path p; sb: geometry in AP order.  Only one path's slots are live. */ \
    template <bool NEEDX, bool NEEDH, bool NEEDG, class CotF, class GateF, class StoreF>                \
    static __device__ __forceinline__ void adjoint_fused(const V (&x)[Base::NX], CotF cot,              \
                                                         GateF gate, const V* sb, V (&dx)[Base::NX],    \
                                                         V (&dsh)[Base::NH], StoreF store_dg) {         \
      Chunk<CPL> ch;                                                                                    \
      V z, gp, dgp;                                                                                     \
      V v[Base::NO], vg[Base::NO];                                                                      \
      ICTC_TP_##S##_ADJP(ICTC_M_P_PB, ICTC_M_P_VL, ICTC_M_P_ZF, ICTC_M_P_ZA, ICTC_M_P_Q, ICTC_M_P_VG,   \
                         ICTC_M_P_DF, ICTC_M_P_DA, ICTC_M_P_DE, ICTC_M_P_PE)                            \
    }                                                                                                   \
    static __device__ __forceinline__ void dharm(const V (&x)[Base::NX], const V (&v)[Base::NO],        \
                                                 const V (&ge)[Base::NP], V (&dsh)[Base::NH]) {         \
      V vg[Base::NO];                                                                                   \
      ICTC_TP_##S##_OUTP(ICTC_M_VG2)                                                                    \
      _Pragma("unroll") for (int j = 0; j < Base::NH; ++j) dsh[j] = V::dup(0.f);                        \
      ICTC_TP_##S##_BYJT(ICTC_M_DSHT_F, ICTC_M_DSHT_A)                                                  \
    }                                                                                                   \
  };

template <int ID, int CPL> struct TpFast;

// Builds the NB geometry entries of one edge in the warp-private buffer `sb` (R rounds of 32 lanes).
template <int NB, int CPL, int R>
__device__ __forceinline__ void build_geometry(const BTerm (&bt)[R], float shv, int lane, Vec<CPL>* sb) {
#pragma unroll
  for (int r = 0; r < R; ++r) {
    const float a = __shfl_sync(0xffffffffu, shv, bt[r].j1);
    const float b = __shfl_sync(0xffffffffu, shv, bt[r].j2);
    const float val = fmaf(bt[r].c2, b, bt[r].c1 * a);
    if (r * 32 + lane < NB) sb[r * 32 + lane] = Vec<CPL>::dup(val);
  }
}

constexpr int kFastWarps = 4;  // warps (= owners) per block

// Receiver-owned forward, one warp per receiver row, C = 32 * CPL channels.
template <class S, class F, int CPL>
__global__ void __launch_bounds__(kFastWarps * 32) tp_graph_forward_fast_kernel(TpArgs a) {
  using V = Vec<CPL>;
  constexpr int C = 32 * CPL, R = (F::NB + 31) / 32, NBP = R * 32;
  __shared__ __align__(16) V sbuf[kFastWarps][2][NBP];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t n = int64_t(blockIdx.x) * kFastWarps + warp;
  if (n >= a.N) return;
  BTerm bt[R];
#pragma unroll
  for (int r = 0; r < R; ++r) bt[r] = (r * 32 + lane < F::NB) ? F::fb(r * 32 + lane) : BTerm{0, 0.f, 0, 0.f};
  V acc[S::NO];
#pragma unroll
  for (int k = 0; k < S::NO; ++k) acc[k] = V::dup(0.f);
  const int64_t begin = ldg(a.rowptr + n), end = ldg(a.rowptr + n + 1);
  int64_t e_next = 0, s_next = 0;
  if (begin < end) {
    e_next = a.order ? ldg(a.order + begin) : begin;
    s_next = ldg(a.nbr + e_next);
  }
  int buf = 0;
  for (int64_t it = begin; it < end; ++it, buf ^= 1) {
    const int64_t e = e_next, s = s_next;
    if (it + 1 < end) {
      e_next = a.order ? ldg(a.order + it + 1) : it + 1;
      s_next = ldg(a.nbr + e_next);
    }
    const float shv = lane < S::NH ? ldg(a.sh + e * S::NH + lane) : 0.f;
    const float* gp = a.g + gate_row_of(a, e, it) * (S::NP * C) + lane * CPL;
    const float* xp = a.x + s * (S::NX * C) + lane * CPL;
    V ge[S::NP], x[S::NX];
#pragma unroll
    for (int p = 0; p < S::NP; ++p) ge[p] = V::load(gp + p * C);
#pragma unroll
    for (int i = 0; i < S::NX; ++i) x[i] = V::load(xp + i * C);
    V* sb = sbuf[warp][buf];
    build_geometry<F::NB, CPL, R>(bt, shv, lane, sb);
    if (a.mask || a.w) {
      const V mu = V::dup(a.mask ? ldg(a.mask + e) : 1.f);
#pragma unroll
      for (int p = 0; p < S::NP; ++p) {
        ge[p] = vmul(ge[p], mu);
        if (a.w) ge[p] = vmul(ge[p], V::load(a.w + p * C + lane * CPL));
      }
    }
    __syncwarp();
    F::forward(x, ge, sb, acc);
  }
  float* op = a.out + n * (S::NO * C) + lane * CPL;
#pragma unroll
  for (int k = 0; k < S::NO; ++k) acc[k].store(op + k * C);
}

// Sender-owned (GRAPH) or edge-owned adjoint, one warp per owner row, C = 32 * CPL channels.
template <class S, class F, int CPL, bool GRAPH, bool NEEDX, bool NEEDH, bool NEEDG>
__global__ void __launch_bounds__(kFastWarps * 32) tp_adjoint_fast_kernel(TpArgs a) {
  using V = Vec<CPL>;
  constexpr int C = 32 * CPL, R = (F::NB + 31) / 32, NBP = R * 32;
  __shared__ __align__(16) V sbuf[kFastWarps][2][NBP];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t owner = int64_t(blockIdx.x) * kFastWarps + warp;
  if (owner >= (GRAPH ? a.N : a.E)) return;
  BTerm bt[R];
#pragma unroll
  for (int r = 0; r < R; ++r) bt[r] = (r * 32 + lane < F::NB) ? F::ab(r * 32 + lane) : BTerm{0, 0.f, 0, 0.f};
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
  int64_t e_next = 0, d_next = 0;
  if (begin < end) {
    e_next = (GRAPH && a.order) ? ldg(a.order + begin) : begin;
    d_next = GRAPH ? ldg(a.nbr + e_next) : e_next;
  }
  int buf = 0;
  for (int64_t it = begin; it < end; ++it, buf ^= 1) {
    const int64_t e = e_next, d = d_next;
    if (it + 1 < end) {
      e_next = (GRAPH && a.order) ? ldg(a.order + it + 1) : it + 1;
      d_next = GRAPH ? ldg(a.nbr + e_next) : e_next;
    }
    const float shv = lane < S::NH ? ldg(a.sh + e * S::NH + lane) : 0.f;
    const float* gp = a.g + gate_row_of(a, e, it) * (S::NP * C) + lane * CPL;
    const float* vp = a.v + d * (S::NO * C) + lane * CPL;
    V ge[S::NP], v[S::NO], scale[S::NP];
#pragma unroll
    for (int p = 0; p < S::NP; ++p) ge[p] = V::load(gp + p * C);
#pragma unroll
    for (int k = 0; k < S::NO; ++k) v[k] = V::load(vp + k * C);
    V* sb = sbuf[warp][buf];
    if (NEEDX || NEEDG) build_geometry<F::NB, CPL, R>(bt, shv, lane, sb);
    const bool scaled = a.mask || a.w;
    if (scaled) {
      const V mu = V::dup(a.mask ? ldg(a.mask + e) : 1.f);
#pragma unroll
      for (int p = 0; p < S::NP; ++p) {
        scale[p] = a.w ? vmul(mu, V::load(a.w + p * C + lane * CPL)) : mu;
        ge[p] = vmul(ge[p], scale[p]);
      }
    }
    if (NEEDX || NEEDG) {
      __syncwarp();
      V dg[S::NP];
#pragma unroll
      for (int p = 0; p < S::NP; ++p) dg[p] = V::dup(0.f);
      F::template adjoint_xg<NEEDX, NEEDG>(x, v, ge, sb, dx, dg);
      if (NEEDG) {
        const int64_t dgr = dg_row_of(a, e, it);
        if (dgr >= 0) {
          float* dgp = a.dg + dgr * (S::NP * C) + lane * CPL;
#pragma unroll
          for (int p = 0; p < S::NP; ++p) (scaled ? vmul(dg[p], scale[p]) : dg[p]).store(dgp + p * C);
        }
      }
    }
    if (NEEDH) {
      V dshv[S::NH];
      F::dharm(x, v, ge, dshv);
      if constexpr (S::NP <= 4) {
        // few paths: the reduction is a large share of the per-edge work, use the 12-shuffle recursive halving
        float part[S::NH];
#pragma unroll
        for (int j = 0; j < S::NH; ++j) part[j] = dshv[j].hsum();
        int which;
        bool holder;
        const float tot = warp_reduce_scatter<S::NH>(part, lane, which, holder);
        if (holder) a.dsh[e * S::NH + which] = tot;
      } else {
        // many paths: the kernel is at its register limit, the plain butterfly keeps fewer values live
        float mine_sum = 0.f;
#pragma unroll
        for (int j = 0; j < S::NH; ++j) {
          const float tot = warp_sum(dshv[j].hsum());
          if (lane == j) mine_sum = tot;
        }
        if (lane < S::NH) a.dsh[e * S::NH + lane] = mine_sum;
      }
    }
  }
  if (NEEDX) {
    float* dxp = a.dx + owner * (S::NX * C) + lane * CPL;
#pragma unroll
    for (int i = 0; i < S::NX; ++i) dx[i].store(dxp + i * C);
  }
}

// ---------------------------------------------------------------------------------------- launchers
inline bool aligned8(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 7) == 0; }

template <class S, class F, int CPL> int launch_graph_forward_fast(const TpArgs& a, cudaStream_t st) {
  const int64_t blocks = (a.N + kFastWarps - 1) / kFastWarps;
  tp_graph_forward_fast_kernel<S, F, CPL><<<(unsigned)blocks, kFastWarps * 32, 0, st>>>(a);
  return finish_launch("tp_graph_forward_fast");
}

template <class S, class F, int CPL, bool GRAPH, bool NX_, bool NH_, bool NG_>
int launch_adjoint_fast_one(const TpArgs& a, cudaStream_t st) {
  const int64_t owners = GRAPH ? a.N : a.E;
  const int64_t blocks = (owners + kFastWarps - 1) / kFastWarps;
  tp_adjoint_fast_kernel<S, F, CPL, GRAPH, NX_, NH_, NG_><<<(unsigned)blocks, kFastWarps * 32, 0, st>>>(a);
  return finish_launch("tp_adjoint_fast");
}

template <class S, class F, int CPL, bool GRAPH> int launch_adjoint_fast_g(const TpArgs& a, cudaStream_t st) {
  const int key = (a.dx ? 4 : 0) | (a.dsh ? 2 : 0) | (a.dg ? 1 : 0);
  switch (key) {
    case 1: return launch_adjoint_fast_one<S, F, CPL, GRAPH, false, false, true>(a, st);
    case 2: return launch_adjoint_fast_one<S, F, CPL, GRAPH, false, true, false>(a, st);
    case 3: return launch_adjoint_fast_one<S, F, CPL, GRAPH, false, true, true>(a, st);
    case 4: return launch_adjoint_fast_one<S, F, CPL, GRAPH, true, false, false>(a, st);
    case 5: return launch_adjoint_fast_one<S, F, CPL, GRAPH, true, false, true>(a, st);
    case 6: return launch_adjoint_fast_one<S, F, CPL, GRAPH, true, true, false>(a, st);
    case 7: return launch_adjoint_fast_one<S, F, CPL, GRAPH, true, true, true>(a, st);
    default: return ICTC_OK;
  }
}

// Fast path applies when C is 32 or 64 and (for C = 64) every row pointer is 8-byte aligned.
template <class S, int ID> int graph_forward_dispatch(const TpArgs& a, cudaStream_t st) {
  if (a.N > 0 && (a.N + kFastWarps - 1) / kFastWarps <= 2147483647LL) {
    if (a.C == 64 && aligned8(a.x) && aligned8(a.g) && aligned8(a.out) && (!a.w || aligned8(a.w)))
      return launch_graph_forward_fast<S, TpFast<ID, 2>, 2>(a, st);
    if (a.C == 32) return launch_graph_forward_fast<S, TpFast<ID, 1>, 1>(a, st);
  }
  return launch_graph_forward<S>(a, st);
}

template <class S, int ID> int adjoint_dispatch(const TpArgs& a, bool graph, cudaStream_t st) {
  const int64_t owners = graph ? a.N : a.E;
  if (owners > 0 && (owners + kFastWarps - 1) / kFastWarps <= 2147483647LL) {
    const bool al = aligned8(a.x) && aligned8(a.g) && aligned8(a.v) && (!a.w || aligned8(a.w)) &&
                    (!a.dx || aligned8(a.dx)) && (!a.dg || aligned8(a.dg));
    if (a.C == 64 && al)
      return graph ? launch_adjoint_fast_g<S, TpFast<ID, 2>, 2, true>(a, st)
                   : launch_adjoint_fast_g<S, TpFast<ID, 2>, 2, false>(a, st);
    if (a.C == 32)
      return graph ? launch_adjoint_fast_g<S, TpFast<ID, 1>, 1, true>(a, st)
                   : launch_adjoint_fast_g<S, TpFast<ID, 1>, 1, false>(a, st);
  }
  return launch_adjoint<S>(a, graph, st);
}

template <class S, int ID> TpOps make_ops_fast() {
  return TpOps{S::NX, S::NH, S::NP, S::NO, S::NNZ, &launch_edge_forward<S>, &graph_forward_dispatch<S, ID>,
               &adjoint_dispatch<S, ID>};
}

}  // namespace ictc
