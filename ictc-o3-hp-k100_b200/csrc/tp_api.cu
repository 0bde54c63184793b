// C-ABI entry points of the tensor product / graph message kernels and library-wide helpers.
#include <stdarg.h>
#include <string.h>
#include "tp_tma_kernels.cuh"

namespace ictc {

__device__ int g_kernel_error = 0;

static thread_local char g_error[512] = "";

void set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_error, sizeof(g_error), fmt, ap);
  va_end(ap);
}

#define ICTC_DECL_OPS(S, a, b, c) TpOps tp_ops_##S();
ICTC_TP_SPEC_LIST(ICTC_DECL_OPS)

struct SpecEntry { int lin, ledge, lout; TpOps ops; };

static const SpecEntry* spec_table(int* count) {
#define ICTC_ENTRY(S, a, b, c) SpecEntry{a, b, c, tp_ops_##S()},
  static const SpecEntry table[] = {ICTC_TP_SPEC_LIST(ICTC_ENTRY)};
  *count = int(sizeof(table) / sizeof(table[0]));
  return table;
}

static const TpOps* find_ops(int spec) {
  int count;
  const SpecEntry* t = spec_table(&count);
  if (spec < 0 || spec >= count) {
    set_error("tensor-product spec %d is not compiled into this library", spec);
    return nullptr;
  }
  return &t[spec].ops;
}

// Device address of the status word of the current device (looked up once per device).
int* kernel_status_word() {
  static int* cache[64] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
  if (!cache[dev]) {
    void* p = nullptr;
    if (cudaGetSymbolAddress(&p, g_kernel_error) == cudaSuccess) cache[dev] = static_cast<int*>(p);
  }
  return cache[dev];
}

// A wait that nothing will ever satisfy: the same bounded polling loop as the kernels' mbarrier waits, with a short
// limit.  It gives up, records `code` in the status word and returns normally.
__global__ void bounded_wait_selftest_kernel(long long limit_cycles, int* status, int code) {
  __shared__ __align__(8) unsigned long long bar;
  const unsigned addr = smem_addr(&bar);
  if (threadIdx.x == 0) {
    mbar_init(addr, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  const long long start = clock64();
  bool done = mbar_try(addr, 0);
  while (!done && clock64() - start <= limit_cycles) done = mbar_try(addr, 0);
  if (!done && threadIdx.x == 0 && status) atomicExch(status, code);
}

static bool check(bool ok, const char* what) {
  if (!ok) set_error("invalid argument: %s", what);
  return ok;
}

}  // namespace ictc

using namespace ictc;

extern "C" {

const char* ictc_last_error(void) { return g_error; }
const char* ictc_version(void) { return "ictc_b200 sm_100a"; }

int ictc_kernel_status(int* host_status, int reset) {
  if (!host_status) { set_error("host_status must not be NULL"); return ICTC_ERR_BAD_ARG; }
  cudaError_t err = cudaDeviceSynchronize();
  if (err == cudaSuccess) err = cudaMemcpyFromSymbol(host_status, g_kernel_error, sizeof(int));
  if (err == cudaSuccess && reset) {
    const int zero = 0;
    err = cudaMemcpyToSymbol(g_kernel_error, &zero, sizeof(int));
  }
  if (err != cudaSuccess) {
    set_error("kernel_status: %s", cudaGetErrorString(err));
    return ICTC_ERR_LAUNCH;
  }
  return ICTC_OK;
}

int ictc_tp_spec(int input_lmax, int edge_lmax, int output_lmax) {
  int count;
  const SpecEntry* t = spec_table(&count);
  for (int i = 0; i < count; ++i)
    if (t[i].lin == input_lmax && t[i].ledge == edge_lmax && t[i].lout == output_lmax) return i;
  set_error("no compiled tensor-product kernels for (input_lmax=%d, edge_lmax=%d, output_lmax=%d)", input_lmax,
            edge_lmax, output_lmax);
  return ICTC_ERR_BAD_SPEC;
}

int ictc_tp_spec_info(int spec, int* nx, int* nh, int* np, int* no, int* nnz) {
  const TpOps* o = find_ops(spec);
  if (!o) return ICTC_ERR_BAD_SPEC;
  if (nx) *nx = o->nx;
  if (nh) *nh = o->nh;
  if (np) *np = o->np;
  if (no) *no = o->no;
  if (nnz) *nnz = o->nnz;
  return ICTC_OK;
}

int ictc_tp_edge_forward(int spec, int channels, int64_t num_edges, const float* x, const float* sh, const float* w,
                         const float* g, const float* mask, float* out, void* stream) {
  const TpOps* o = find_ops(spec);
  if (!o) return ICTC_ERR_BAD_SPEC;
  if (!check(channels > 0 && num_edges >= 0, "channels > 0, num_edges >= 0")) return ICTC_ERR_BAD_ARG;
  if (num_edges == 0) return ICTC_OK;
  if (!check(x && sh && g && out, "x, sh, g, out must not be NULL")) return ICTC_ERR_BAD_ARG;
  TpArgs a{};
  a.x = x; a.sh = sh; a.w = w; a.g = g; a.mask = mask; a.out = out; a.E = num_edges; a.N = num_edges; a.C = channels;
  return o->edge_forward(a, (cudaStream_t)stream);
}

int ictc_tp_edge_adjoint(int spec, int channels, int64_t num_edges, const float* x, const float* sh, const float* w,
                         const float* g, const float* mask, const float* v, float* dx, float* dsh, float* dg,
                         void* stream) {
  const TpOps* o = find_ops(spec);
  if (!o) return ICTC_ERR_BAD_SPEC;
  if (!check(channels > 0 && num_edges >= 0, "channels > 0, num_edges >= 0")) return ICTC_ERR_BAD_ARG;
  if (num_edges == 0 || (!dx && !dsh && !dg)) return ICTC_OK;
  if (!check(x && sh && g && v, "x, sh, g, v must not be NULL")) return ICTC_ERR_BAD_ARG;
  TpArgs a{};
  a.x = x; a.sh = sh; a.w = w; a.g = g; a.mask = mask; a.v = v; a.dx = dx; a.dsh = dsh; a.dg = dg;
  a.E = num_edges; a.N = num_edges; a.C = channels; a.status = kernel_status_word();
  return o->adjoint(a, false, (cudaStream_t)stream);
}

int ictc_tp_graph_forward_shared(int spec, int channels, int64_t num_nodes, int64_t num_edges, const float* x,
                                 const float* sh, const float* w, const float* g, const int64_t* gate_row,
                                 const int64_t* src, const int64_t* dst_rowptr, const int64_t* dst_order,
                                 const float* mask, float* out, void* stream);

int ictc_tp_graph_forward(int spec, int channels, int64_t num_nodes, int64_t num_edges, const float* x,
                          const float* sh, const float* w, const float* g, const int64_t* src,
                          const int64_t* dst_rowptr, const int64_t* dst_order, const float* mask, float* out,
                          void* stream) {
  return ictc_tp_graph_forward_shared(spec, channels, num_nodes, num_edges, x, sh, w, g, nullptr, src, dst_rowptr,
                                      dst_order, mask, out, stream);
}

int ictc_tp_graph_forward_shared(int spec, int channels, int64_t num_nodes, int64_t num_edges, const float* x,
                                 const float* sh, const float* w, const float* g, const int64_t* gate_row,
                                 const int64_t* src, const int64_t* dst_rowptr, const int64_t* dst_order,
                                 const float* mask, float* out, void* stream) {
  const TpOps* o = find_ops(spec);
  if (!o) return ICTC_ERR_BAD_SPEC;
  if (!check(channels > 0 && num_edges >= 0 && num_nodes >= 0, "sizes")) return ICTC_ERR_BAD_ARG;
  if (num_nodes == 0) return ICTC_OK;
  if (!check(out && dst_rowptr, "out, dst_rowptr must not be NULL")) return ICTC_ERR_BAD_ARG;
  if (num_edges > 0 && !check(x && sh && g && src, "x, sh, g, src must not be NULL")) return ICTC_ERR_BAD_ARG;
  TpArgs a{};
  a.x = x; a.sh = sh; a.w = w; a.g = g; a.mask = mask; a.out = out; a.nbr = src; a.rowptr = dst_rowptr;
  a.grow = gate_row; a.order = dst_order; a.E = num_edges; a.N = num_nodes; a.C = channels; a.status = kernel_status_word();
  return o->graph_forward(a, (cudaStream_t)stream);
}

int ictc_tp_graph_adjoint_shared(int spec, int channels, int64_t num_nodes, int64_t num_edges, const float* x,
                                 const float* sh, const float* w, const float* g, const int64_t* gate_row,
                                 const int64_t* dst, const int64_t* src_rowptr, const int64_t* src_order,
                                 const float* mask, const float* v, float* dx, float* dsh, float* dg, void* stream);

int ictc_tp_graph_adjoint(int spec, int channels, int64_t num_nodes, int64_t num_edges, const float* x,
                          const float* sh, const float* w, const float* g, const int64_t* dst,
                          const int64_t* src_rowptr, const int64_t* src_order, const float* mask, const float* v,
                          float* dx, float* dsh, float* dg, void* stream) {
  return ictc_tp_graph_adjoint_shared(spec, channels, num_nodes, num_edges, x, sh, w, g, nullptr, dst, src_rowptr,
                                      src_order, mask, v, dx, dsh, dg, stream);
}

int ictc_tp_graph_adjoint_shared(int spec, int channels, int64_t num_nodes, int64_t num_edges, const float* x,
                                 const float* sh, const float* w, const float* g, const int64_t* gate_row,
                                 const int64_t* dst, const int64_t* src_rowptr, const int64_t* src_order,
                                 const float* mask, const float* v, float* dx, float* dsh, float* dg, void* stream) {
  const TpOps* o = find_ops(spec);
  if (!o) return ICTC_ERR_BAD_SPEC;
  if (!check(channels > 0 && num_edges >= 0 && num_nodes >= 0, "sizes")) return ICTC_ERR_BAD_ARG;
  if (num_nodes == 0 || (!dx && !dsh && !dg)) return ICTC_OK;
  if (!check(src_rowptr && x, "x, src_rowptr must not be NULL")) return ICTC_ERR_BAD_ARG;
  if (num_edges > 0 && !check(sh && g && dst && v, "sh, g, dst, v must not be NULL")) return ICTC_ERR_BAD_ARG;
  TpArgs a{};
  a.x = x; a.sh = sh; a.w = w; a.g = g; a.mask = mask; a.v = v; a.dx = dx; a.dsh = dsh; a.dg = dg; a.nbr = dst;
  a.grow = gate_row; a.rowptr = src_rowptr; a.order = src_order; a.E = num_edges; a.N = num_nodes; a.C = channels; a.status = kernel_status_word();
  return o->adjoint(a, true, (cudaStream_t)stream);
}

int ictc_tp_graph_forward_chunk(int spec, int channels, int64_t num_rows, const float* x, const float* sh,
                                const float* w, const float* g, const int64_t* gate_row, const int64_t* g_base,
                                int64_t g_capacity, const int64_t* src, const int64_t* dst_rowptr,
                                const int64_t* dst_order, const float* mask, float* out, void* stream) {
  const TpOps* o = find_ops(spec);
  if (!o) return ICTC_ERR_BAD_SPEC;
  if (!check(channels > 0 && num_rows >= 0 && g_capacity >= 0, "sizes")) return ICTC_ERR_BAD_ARG;
  if (num_rows == 0) return ICTC_OK;
  if (!check(out && dst_rowptr && x && sh && g && src, "x, sh, g, src, dst_rowptr, out must not be NULL")) return ICTC_ERR_BAD_ARG;
  if (!check(!g_base || g_capacity > 0, "g_capacity must be positive when g_base is given")) return ICTC_ERR_BAD_ARG;
  TpArgs a{};
  a.x = x; a.sh = sh; a.w = w; a.g = g; a.mask = mask; a.out = out; a.nbr = src; a.rowptr = dst_rowptr;
  a.grow = gate_row; a.order = dst_order; a.E = 1; a.N = num_rows; a.C = channels; a.status = kernel_status_word();
  a.g_base = g_base; a.g_cap = g_capacity;
  return o->graph_forward(a, (cudaStream_t)stream);
}

int ictc_tp_graph_adjoint_chunk(int spec, int channels, int64_t num_rows, const float* x, const float* sh,
                                const float* w, const float* g, const int64_t* gate_row, int g_by_position,
                                const int64_t* g_base, int64_t g_capacity, const int64_t* dst,
                                const int64_t* src_rowptr, const int64_t* src_order, const float* mask, const float* v,
                                float* dx, float* dsh, float* dg, const int64_t* dg_base, int64_t dg_capacity,
                                void* stream) {
  const TpOps* o = find_ops(spec);
  if (!o) return ICTC_ERR_BAD_SPEC;
  if (!check(channels > 0 && num_rows >= 0 && g_capacity >= 0 && dg_capacity >= 0, "sizes")) return ICTC_ERR_BAD_ARG;
  if (num_rows == 0 || (!dx && !dsh && !dg)) return ICTC_OK;
  if (!check(src_rowptr && x && sh && g && dst && v, "x, sh, g, dst, v, src_rowptr must not be NULL")) return ICTC_ERR_BAD_ARG;
  if (!check(!g_base || g_capacity > 0, "g_capacity must be positive when g_base is given")) return ICTC_ERR_BAD_ARG;
  if (!check(!(dg && dg_base) || dg_capacity > 0, "dg_capacity must be positive when dg_base is given")) return ICTC_ERR_BAD_ARG;
  TpArgs a{};
  a.x = x; a.sh = sh; a.w = w; a.g = g; a.mask = mask; a.v = v; a.dx = dx; a.dsh = dsh; a.dg = dg; a.nbr = dst;
  a.grow = gate_row; a.rowptr = src_rowptr; a.order = src_order; a.E = 1; a.N = num_rows; a.C = channels;
  a.status = kernel_status_word();
  a.g_base = g_base; a.g_cap = g_capacity; a.g_by_pos = g_by_position ? 1 : 0;
  a.dg_base = dg ? dg_base : nullptr; a.dg_cap = dg_capacity;
  return o->adjoint(a, true, (cudaStream_t)stream);
}

int ictc_selftest_bounded_wait(int64_t limit_cycles, int code, void* stream) {
  if (limit_cycles < 1 || limit_cycles > 200000000LL || code == 0) {
    set_error("selftest: limit must be 1..2e8 cycles and the code non-zero");
    return ICTC_ERR_BAD_ARG;
  }
  bounded_wait_selftest_kernel<<<1, 32, 0, (cudaStream_t)stream>>>((long long)limit_cycles, kernel_status_word(), code);
  return finish_launch("selftest_bounded_wait");
}

}  // extern "C"
