// Cell-list neighbour build and velocity-Verlet helpers for the MD step.
//
// Edge convention of the reference's graph fill (lammps_user_mfftorch/src/USER-MFFTORCH/
// pair_mff_torch_kokkos.cpp:661-871): a full neighbour list, edge (src = j neighbour, dst = i centre)
// for every ordered pair with |r_i - r_j + S*box|^2 <= cutoff^2, centres restricted to the first
// `num_centres` rows (owned atoms), edges ordered by (dst, src, shift_x, shift_y, shift_z) — the
// reference's canonical order (:897-911).  The distance test is evaluated in double precision on the
// fp32 coordinates with individually rounded operations (no fused multiply-add), so it is bit-for-bit
// the same predicate a plain CPU loop evaluates.
//
// Phases: (1) cell key per atom -> stable counting sort (the CSR builder of csr.cu), (2) per-centre
// neighbour count, (3) exclusive scan, (4) per-centre fill + in-row sort by (src, shift).
#include "ictc_common.cuh"

extern "C" int ictc_csr_build(const int64_t* keys, int64_t N, int64_t E, int64_t* rowptr, int64_t* order,
                              int32_t* sorted_flag, void* scratch, void* stream);
extern "C" int64_t ictc_csr_scratch_bytes(int64_t N, int64_t E);

namespace ictc {

struct NbGrid {
  double lo[3];       // origin of the cell grid
  double box[3];      // periodic lengths (used for image shifts)
  double inv_w[3];    // 1 / cell width
  int nc[3];          // cells per axis
  int periodic[3];
  double cutsq;
};

__device__ __forceinline__ void cell_of(const NbGrid& g, const float* p, int (&c)[3]) {
#pragma unroll
  for (int a = 0; a < 3; ++a) {
    int v = int(floor((double(p[a]) - g.lo[a]) * g.inv_w[a]));
    c[a] = v < 0 ? 0 : (v >= g.nc[a] ? g.nc[a] - 1 : v);
  }
}

__global__ void nb_cell_key_kernel(NbGrid g, const float* __restrict__ pos, int64_t n, int64_t* keys) {
  const int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= n) return;
  int c[3];
  cell_of(g, pos + 3 * i, c);
  keys[i] = (int64_t(c[0]) * g.nc[1] + c[1]) * g.nc[2] + c[2];
}

// Visits every (neighbour j, image shift) candidate of centre i and calls f(j, sx, sy, sz) for pairs
// inside the cutoff.
template <class F>
__device__ __forceinline__ void nb_visit(const NbGrid& g, const float* __restrict__ pos,
                                         const int64_t* __restrict__ cell_start,
                                         const int64_t* __restrict__ cell_atoms, int64_t i, F f) {
  int c[3];
  cell_of(g, pos + 3 * i, c);
  const double xi = pos[3 * i], yi = pos[3 * i + 1], zi = pos[3 * i + 2];
  for (int ox = -1; ox <= 1; ++ox) {
    int cx = c[0] + ox, sx = 0;
    if (cx < 0 || cx >= g.nc[0]) {
      if (!g.periodic[0]) continue;
      sx = cx < 0 ? -1 : 1;
      cx -= sx * g.nc[0];
    }
    for (int oy = -1; oy <= 1; ++oy) {
      int cy = c[1] + oy, sy = 0;
      if (cy < 0 || cy >= g.nc[1]) {
        if (!g.periodic[1]) continue;
        sy = cy < 0 ? -1 : 1;
        cy -= sy * g.nc[1];
      }
      for (int oz = -1; oz <= 1; ++oz) {
        int cz = c[2] + oz, sz = 0;
        if (cz < 0 || cz >= g.nc[2]) {
          if (!g.periodic[2]) continue;
          sz = cz < 0 ? -1 : 1;
          cz -= sz * g.nc[2];
        }
        const int64_t cell = (int64_t(cx) * g.nc[1] + cy) * g.nc[2] + cz;
        // neighbour image sits at r_j + s*box, so edge_vec = r_i - r_j + (-s)*box
        const double bx = -sx * g.box[0], by = -sy * g.box[1], bz = -sz * g.box[2];
        for (int64_t k = cell_start[cell]; k < cell_start[cell + 1]; ++k) {
          const int64_t j = cell_atoms[k];
          if (j == i && sx == 0 && sy == 0 && sz == 0) continue;
          const double dx = __dadd_rn(__dadd_rn(xi, -double(pos[3 * j])), bx);
          const double dy = __dadd_rn(__dadd_rn(yi, -double(pos[3 * j + 1])), by);
          const double dz = __dadd_rn(__dadd_rn(zi, -double(pos[3 * j + 2])), bz);
          const double rsq = __dadd_rn(__dadd_rn(__dmul_rn(dx, dx), __dmul_rn(dy, dy)), __dmul_rn(dz, dz));
          if (rsq <= g.cutsq) f(j, -sx, -sy, -sz);
        }
      }
    }
  }
}

__global__ void nb_count_kernel(NbGrid g, const float* __restrict__ pos, const int64_t* __restrict__ cell_start,
                                const int64_t* __restrict__ cell_atoms, int64_t centres, int64_t* counts) {
  const int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= centres) return;
  int64_t n = 0;
  nb_visit(g, pos, cell_start, cell_atoms, i, [&](int64_t, int, int, int) { ++n; });
  counts[i + 1] = n;
  if (i == 0) counts[0] = 0;
}

__device__ __forceinline__ int64_t nb_key(int64_t j, int sx, int sy, int sz) {
  return j * 27 + ((sx + 1) * 3 + (sy + 1)) * 3 + (sz + 1);
}

__global__ void nb_fill_kernel(NbGrid g, const float* __restrict__ pos, const int64_t* __restrict__ cell_start,
                               const int64_t* __restrict__ cell_atoms, int64_t centres,
                               const int64_t* __restrict__ rowptr, int64_t capacity, int64_t* src, int64_t* dst,
                               float* shifts, int64_t* keys) {
  const int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= centres) return;
  const int64_t begin = rowptr[i], end = rowptr[i + 1];
  if (end > capacity || begin > end) return;   // offsets must have been clamped to the capacity
  int64_t w = begin;
  nb_visit(g, pos, cell_start, cell_atoms, i, [&](int64_t j, int sx, int sy, int sz) {
    if (w >= end) return;       // row truncated by the capacity clamp: extra neighbours are dropped
    // insertion into the sorted prefix [begin, w) by key (src, shift)
    const int64_t key = nb_key(j, sx, sy, sz);
    int64_t p = w;
    while (p > begin && keys[p - 1] > key) {
      keys[p] = keys[p - 1];
      --p;
    }
    keys[p] = key;
    ++w;
  });
  for (int64_t p = begin; p < end; ++p) {
    const int64_t key = keys[p];
    const int code = int(key % 27);
    src[p] = key / 27;
    dst[p] = i;
    shifts[3 * p + 0] = float(code / 9 - 1);
    shifts[3 * p + 1] = float((code / 3) % 3 - 1);
    shifts[3 * p + 2] = float(code % 3 - 1);
  }
}

// Clamps row offsets to the capacity of fixed-size edge buffers (rows beyond it become empty, the row that
// straddles it is truncated) and raises *overflow when anything had to be clamped.  The flag is sticky (never
// cleared here) so that a host that looks only every few steps still sees an earlier overflow.
__global__ void nb_clamp_kernel(int64_t* rowptr, int64_t n1, int64_t capacity, int32_t* overflow) {
  const int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= n1) return;
  const int64_t v = rowptr[i];
  if (i == n1 - 1 && v > capacity) *overflow = 1;
  if (v > capacity) rowptr[i] = capacity;
}

// Fills the unused tail [count, capacity) of fixed-capacity edge buffers with inert edges so that every
// consumer can run over `capacity` rows without knowing the edge count on the host.
__global__ void nb_pad_kernel(const int64_t* __restrict__ count, int64_t capacity, int64_t pad_src, int64_t pad_dst,
                              int64_t* src, int64_t* dst, float* shifts, int32_t* overflow) {
  const int64_t e = int64_t(blockIdx.x) * blockDim.x + threadIdx.x;
  if (e == 0 && overflow) *overflow = *count > capacity ? 1 : 0;
  if (e >= capacity || e < *count) return;
  src[e] = pad_src;
  dst[e] = pad_dst;
  shifts[3 * e] = shifts[3 * e + 1] = shifts[3 * e + 2] = 0.f;
}

// ---- radial pairing --------------------------------------------------------------------------------
// Edge (j -> i, S) and its reverse (i -> j, -S) have bitwise the same length, so everything that depends
// on the length alone (radial basis, gate MLP) is evaluated once per pair.  `rev` finds the reverse edge by
// binary search in the sorted row of j; an edge is the pair's representative when it has no reverse in the
// list (sender is not a centre) or when its index is the smaller of the two.
__global__ void nb_pair_find_kernel(const int64_t* __restrict__ rowptr, const int64_t* __restrict__ dst,
                                    const int64_t* __restrict__ keys, int64_t centres, int64_t capacity,
                                    const int64_t* __restrict__ count, int64_t* rev, int64_t* flag) {
  const int64_t e = int64_t(blockIdx.x) * blockDim.x + threadIdx.x;
  if (e >= capacity) return;
  if (e >= *count) {
    rev[e] = -1;
    flag[e] = 0;
    return;
  }
  const int64_t key = keys[e];
  const int64_t j = key / 27, i = dst[e];
  int64_t r = -1;
  if (j < centres) {
    const int64_t want = i * 27 + (26 - key % 27);
    int64_t lo = rowptr[j], hi = rowptr[j + 1];
    while (lo < hi) {
      const int64_t mid = (lo + hi) >> 1;
      if (keys[mid] < want) lo = mid + 1; else hi = mid;
    }
    if (lo < rowptr[j + 1] && keys[lo] == want) r = lo;
  }
  rev[e] = r;
  flag[e] = (r < 0 || e < r) ? 1 : 0;
}

// scan = inclusive prefix sum of the representative flags
__global__ void nb_pair_assign_kernel(const int64_t* __restrict__ scan, const int64_t* __restrict__ rev,
                                      int64_t capacity, int64_t unique_capacity, const int64_t* __restrict__ count,
                                      int64_t* gate_row, int64_t* rep_edge, int64_t* other_edge, int64_t* num_unique) {
  const int64_t e = int64_t(blockIdx.x) * blockDim.x + threadIdx.x;
  const int64_t n = *count < capacity ? *count : capacity;
  const int64_t total = n > 0 ? scan[n - 1] : 0;
  if (e == 0) *num_unique = total;
  if (e < capacity) {
    if (e < n) {
      const int64_t r = rev[e];
      const bool rep = r < 0 || e < r;
      const int64_t u = (rep ? scan[e] : scan[r]) - 1;
      // a pair table that is too small is reported through num_unique > unique_capacity; rows stay in range
      gate_row[e] = u < unique_capacity ? u : (unique_capacity > 0 ? unique_capacity - 1 : 0);
      if (rep && u < unique_capacity) {
        rep_edge[u] = e;
        other_edge[u] = r;
      }
    } else {
      gate_row[e] = 0;
    }
  }
  // rows of the pair table beyond the number of pairs point at the last (inert) edge slot
  if (e >= total && e < unique_capacity) {
    rep_edge[e] = capacity - 1;
    other_edge[e] = -1;
  }
}

// ---- velocity Verlet (positions in A, velocities in A/fs, forces in eV/A, masses in amu) ----------
constexpr float kAccel = 9.64853321e-3f;   // 1 eV/(A amu) in A/fs^2

__global__ void md_kick_drift_kernel(int64_t n, float dt, const float* __restrict__ force,
                                     const float* __restrict__ inv_mass, float* vel, float* pos, const float* box,
                                     int drift) {
  const int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const float s = 0.5f * dt * kAccel * inv_mass[i];
#pragma unroll
  for (int a = 0; a < 3; ++a) {
    float v = fmaf(s, force[3 * i + a], vel[3 * i + a]);
    vel[3 * i + a] = v;
    if (drift) {
      float x = fmaf(dt, v, pos[3 * i + a]);
      const float L = box[a];
      if (L > 0.f) {           // periodic axis: wrap into [0, L)
        if (x >= L) x -= L;
        if (x < 0.f) x += L;
        if (x >= L) x = 0.f;   // x was -tiny and x + L rounded to L
      }
      pos[3 * i + a] = x;
    }
  }
}

}  // namespace ictc

using namespace ictc;

extern "C" {

// scratch layout: keys[N] | cell_start[cells+1] | cell_atoms[N] | flag | csr scratch
static int64_t nb_cells(const double* box_len, const double* lo, const double* hi, double cutoff, int* nc) {
  int64_t total = 1;
  for (int a = 0; a < 3; ++a) {
    const double extent = hi[a] - lo[a];
    int n = int(floor(extent / cutoff));
    if (n < 1) n = 1;
    if (n > 1024) n = 1024;
    nc[a] = n;
    total *= n;
  }
  (void)box_len;
  return total;
}

int64_t ictc_neighbor_scratch_bytes(int64_t num_atoms, const double* host_lo, const double* host_hi, double cutoff) {
  if (num_atoms < 0 || !host_lo || !host_hi || !(cutoff > 0)) return 0;
  int nc[3];
  const int64_t cells = nb_cells(nullptr, host_lo, host_hi, cutoff, nc);
  return 8 * (2 * num_atoms + cells + 1 + 8) + ictc_csr_scratch_bytes(cells, num_atoms) + 64;
}

static int nb_setup(int64_t N, const double* lo, const double* hi, const double* box, const int* periodic,
                    double cutoff, NbGrid* g, int64_t* cells) {
  if (N < 0 || !lo || !hi || !box || !periodic || !(cutoff > 0)) {
    set_error("neighbor: invalid arguments");
    return ICTC_ERR_BAD_ARG;
  }
  *cells = nb_cells(box, lo, hi, cutoff, g->nc);
  for (int a = 0; a < 3; ++a) {
    g->lo[a] = lo[a];
    g->box[a] = box[a];
    g->inv_w[a] = g->nc[a] / (hi[a] - lo[a]);
    g->periodic[a] = periodic[a];
    if (periodic[a] && (hi[a] - lo[a]) / g->nc[a] < cutoff && g->nc[a] > 1) {
      set_error("neighbor: cell narrower than the cutoff");
      return ICTC_ERR_BAD_ARG;
    }
    if (periodic[a] && box[a] < cutoff) {
      set_error("neighbor: periodic box shorter than the cutoff needs more than one image per axis");
      return ICTC_ERR_BAD_ARG;
    }
  }
  g->cutsq = cutoff * cutoff;
  if ((N + 255) / 256 > 2147483647LL) { set_error("neighbor: too many atoms"); return ICTC_ERR_TOO_LARGE; }
  return ICTC_OK;
}

struct NbScratch { int64_t *keys, *cell_start, *cell_atoms; int32_t* flag; void* csr; };

static NbScratch nb_carve(void* scratch, int64_t N, int64_t cells) {
  NbScratch s;
  s.keys = reinterpret_cast<int64_t*>(scratch);
  s.cell_start = s.keys + N;
  s.cell_atoms = s.cell_start + cells + 1;
  s.flag = reinterpret_cast<int32_t*>(s.cell_atoms + N);
  s.csr = s.cell_atoms + N + 8;
  return s;
}

int ictc_neighbor_count(const float* pos, int64_t num_atoms, int64_t num_centres, const double* host_lo,
                        const double* host_hi, const double* host_box, const int* host_periodic, double cutoff,
                        int64_t* rowptr, void* scratch, void* stream) {
  NbGrid g;
  int64_t cells;
  if (int rc = nb_setup(num_atoms, host_lo, host_hi, host_box, host_periodic, cutoff, &g, &cells)) return rc;
  if (num_centres < 0 || num_centres > num_atoms || !rowptr || !scratch || (num_atoms > 0 && !pos)) {
    set_error("neighbor_count: invalid arguments");
    return ICTC_ERR_BAD_ARG;
  }
  cudaStream_t st = (cudaStream_t)stream;
  NbScratch s = nb_carve(scratch, num_atoms, cells);
  if (num_atoms > 0)
    nb_cell_key_kernel<<<(unsigned)((num_atoms + 255) / 256), 256, 0, st>>>(g, pos, num_atoms, s.keys);
  if (int rc = ictc_csr_build(s.keys, cells, num_atoms, s.cell_start, s.cell_atoms, s.flag, s.csr, stream)) return rc;
  if (num_centres > 0)
    nb_count_kernel<<<(unsigned)((num_centres + 127) / 128), 128, 0, st>>>(g, pos, s.cell_start, s.cell_atoms,
                                                                          num_centres, rowptr);
  else
    cudaMemsetAsync(rowptr, 0, 8, st);
  return finish_launch("neighbor_count");
}

int ictc_neighbor_fill(const float* pos, int64_t num_atoms, int64_t num_centres, const double* host_lo,
                       const double* host_hi, const double* host_box, const int* host_periodic, double cutoff,
                       const int64_t* rowptr, int64_t capacity, int64_t* src, int64_t* dst, float* shifts,
                       int64_t* edge_keys, void* scratch, void* stream) {
  NbGrid g;
  int64_t cells;
  if (int rc = nb_setup(num_atoms, host_lo, host_hi, host_box, host_periodic, cutoff, &g, &cells)) return rc;
  if (num_centres == 0 || capacity == 0) return ICTC_OK;
  if (!rowptr || !src || !dst || !shifts || !edge_keys || !scratch) {
    set_error("neighbor_fill: NULL buffer");
    return ICTC_ERR_BAD_ARG;
  }
  NbScratch s = nb_carve(scratch, num_atoms, cells);
  nb_fill_kernel<<<(unsigned)((num_centres + 127) / 128), 128, 0, (cudaStream_t)stream>>>(
      g, pos, s.cell_start, s.cell_atoms, num_centres, rowptr, capacity, src, dst, shifts, edge_keys);
  return finish_launch("neighbor_fill");
}

int ictc_neighbor_clamp(int64_t* rowptr, int64_t num_centres, int64_t capacity, int32_t* overflow, void* stream) {
  if (num_centres < 0 || capacity < 0 || !rowptr || !overflow) {
    set_error("neighbor_clamp: invalid arguments");
    return ICTC_ERR_BAD_ARG;
  }
  nb_clamp_kernel<<<(unsigned)((num_centres + 1 + 255) / 256), 256, 0, (cudaStream_t)stream>>>(rowptr, num_centres + 1,
                                                                                             capacity, overflow);
  return finish_launch("neighbor_clamp");
}

int ictc_neighbor_pad(const int64_t* count, int64_t capacity, int64_t pad_src, int64_t pad_dst, int64_t* src,
                      int64_t* dst, float* shifts, int32_t* overflow, void* stream) {
  if (capacity < 0 || !count || (capacity > 0 && (!src || !dst || !shifts))) {
    set_error("neighbor_pad: invalid arguments");
    return ICTC_ERR_BAD_ARG;
  }
  const int64_t blocks = capacity > 0 ? (capacity + 255) / 256 : 1;
  if (blocks > 2147483647LL) { set_error("neighbor_pad: too many edges"); return ICTC_ERR_TOO_LARGE; }
  nb_pad_kernel<<<(unsigned)blocks, 256, 0, (cudaStream_t)stream>>>(count, capacity, pad_src, pad_dst, src, dst,
                                                                    shifts, overflow);
  return finish_launch("neighbor_pad");
}

extern "C" int ictc_inclusive_scan_i64(int64_t* data, int64_t n, void* scratch, void* stream);

int ictc_neighbor_pairs(const int64_t* rowptr, const int64_t* dst, const int64_t* edge_keys, int64_t num_centres,
                        int64_t capacity, int64_t unique_capacity, const int64_t* count, int64_t* rev, int64_t* scan,
                        int64_t* gate_row, int64_t* rep_edge, int64_t* other_edge, int64_t* num_unique,
                        void* scan_scratch, void* stream) {
  if (num_centres < 0 || capacity < 0 || unique_capacity < 0 || !count || !num_unique) {
    set_error("neighbor_pairs: invalid arguments");
    return ICTC_ERR_BAD_ARG;
  }
  const int64_t span = capacity > unique_capacity ? capacity : unique_capacity;
  if (span == 0) return ICTC_OK;
  if (!rowptr || !dst || !edge_keys || !rev || !scan || !gate_row || !rep_edge || !other_edge || !scan_scratch) {
    set_error("neighbor_pairs: NULL buffer");
    return ICTC_ERR_BAD_ARG;
  }
  if ((span + 255) / 256 > 2147483647LL) { set_error("neighbor_pairs: too many edges"); return ICTC_ERR_TOO_LARGE; }
  cudaStream_t st = (cudaStream_t)stream;
  if (capacity > 0) {
    nb_pair_find_kernel<<<(unsigned)((capacity + 255) / 256), 256, 0, st>>>(rowptr, dst, edge_keys, num_centres,
                                                                           capacity, count, rev, scan);
    if (int rc = ictc_inclusive_scan_i64(scan, capacity, scan_scratch, stream)) return rc;
  }
  nb_pair_assign_kernel<<<(unsigned)((span + 255) / 256), 256, 0, st>>>(scan, rev, capacity, unique_capacity, count,
                                                                      gate_row, rep_edge, other_edge, num_unique);
  return finish_launch("neighbor_pairs");
}

int ictc_md_kick(int64_t num_atoms, float dt, const float* force, const float* inv_mass, float* vel, float* pos,
                 const float* box, int drift, void* stream) {
  if (num_atoms < 0 || (num_atoms > 0 && (!force || !inv_mass || !vel || (drift && (!pos || !box))))) {
    set_error("md_kick: invalid arguments");
    return ICTC_ERR_BAD_ARG;
  }
  if (num_atoms == 0) return ICTC_OK;
  md_kick_drift_kernel<<<(unsigned)((num_atoms + 255) / 256), 256, 0, (cudaStream_t)stream>>>(
      num_atoms, dt, force, inv_mass, vel, pos, box, drift);
  return finish_launch("md_kick");
}

}  // extern "C"
