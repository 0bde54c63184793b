// Host build of the GENERATED symmetric-contraction code (csrc/generated/sc_code.cuh) in double precision.
// Test infrastructure: the same straight-line source the CUDA kernels compile (csrc/sc.cu) is compiled here with g++
// for T = double, so the CPU suite can pin the kernel arithmetic on the vectors of the reference's own recursion
// (mace_ictc/models/mace/products.py:845-949) without a GPU.  Layouts as in csrc/sc.cu: features [N, 9*C] with degree
// blocks [C, 2l+1] (mul_ir), weight bank [S, NW, C].
#include <cstdint>
#define __device__
#define __forceinline__ inline

template <class T> T zero();
template <> inline double zero<double>() { return 0.0; }
static inline double mul(double a, double b) { return a * b; }
static inline double add(double a, double b) { return a + b; }
static inline double madd(float c, double a, double b) { return double(c) * a + b; }
static inline double fmadd(double a, double b, double c) { return a * b + c; }
static inline double scale(float c, double a) { return double(c) * a; }

#include "generated/sc_code.cuh"

namespace {
int offset(int l, int m, int c, int C) { return l * l * C + c * (2 * l + 1) + m; }
void load(const double* row, int nl, int c, int C, double* out) {
  int k = 0;
  for (int l = 0; l < nl; ++l)
    for (int m = 0; m < 2 * l + 1; ++m, ++k) out[k] = row[offset(l, m, c, C)];
}
void store(double* row, int nl, int c, int C, const double* in) {
  int k = 0;
  for (int l = 0; l < nl; ++l)
    for (int m = 0; m < 2 * l + 1; ++m, ++k) row[offset(l, m, c, C)] = in[k];
}
struct Weights {
  const double* w;
  int C;
  double operator()(int idx) const { return w[idx * C]; }
};
}  // namespace

extern "C" {

int sc_host_num_weights(int lt) { return lt == 0 ? ICTC_SC_NW_LT0 : ICTC_SC_NW_LT2; }

// mode 0: y = F(x, W); mode 1: gx = d<gy, F>/dx; mode 2: gw += d<gy, F>/dW  (gw [S, NW, C], zeroed by the caller)
void sc_host(int lt, int mode, int64_t N, int C, const double* x, const int64_t* species, const double* w,
             const double* gy, double* y, double* gx, double* gw) {
  const int ny = (lt + 1) * (lt + 1), nw = sc_host_num_weights(lt);
  for (int64_t n = 0; n < N; ++n)
    for (int c = 0; c < C; ++c) {
      double xv[9], gyv[9] = {0}, out[9];
      load(x + n * 9 * C, 3, c, C, xv);
      if (mode) load(gy + n * ny * C, lt + 1, c, C, gyv);
      Weights wl{w + species[n] * nw * C + c, C};
      if (mode == 0) {
        if (lt == 0) sc_forward_lt0<double>(xv, wl, reinterpret_cast<double(&)[1]>(out));
        else sc_forward_lt2<double>(xv, wl, reinterpret_cast<double(&)[9]>(out));
        store(y + n * ny * C, lt + 1, c, C, out);
      } else if (mode == 1) {
        if (lt == 0) sc_xgrad_lt0<double>(xv, wl, reinterpret_cast<double(&)[1]>(gyv), reinterpret_cast<double(&)[9]>(out));
        else sc_xgrad_lt2<double>(xv, wl, reinterpret_cast<double(&)[9]>(gyv), reinterpret_cast<double(&)[9]>(out));
        store(gx + n * 9 * C, 3, c, C, out);
      } else {
        double* col = gw + species[n] * nw * C + c;
        auto sink = [col, C](int idx, double val) { col[idx * C] += val; };
        if (lt == 0) sc_wgrad_lt0<double>(xv, reinterpret_cast<double(&)[1]>(gyv), sink);
        else sc_wgrad_lt2<double>(xv, reinterpret_cast<double(&)[9]>(gyv), sink);
      }
    }
}

}  // extern "C"
