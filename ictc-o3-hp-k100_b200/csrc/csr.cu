// CSR topology from an unsorted int64 key vector (receiver or sender of every edge).
//
// rowptr = exclusive prefix sum of the key histogram; order = edge ids grouped by key, ascending
// inside a row (what a stable sort by key would give), so every reduction that walks a row has a
// fixed summation order.  Integer atomics are used for the histogram and for handing out slots; the
// slot order is then made canonical by ranking the edge ids inside each row.  When the keys are
// already non-decreasing the order is the identity and the ranking pass exits immediately.
// Replaces ictc_o3/backends/k100/generated_csr_forward.py:17-31 (bincount + cumsum + stable argsort)
// and the device counting sort ictc_o3/ops/message_topology.py:15-36.
#include <mutex>
#include "ictc_common.cuh"

namespace ictc {

constexpr int kScanThreads = 256;
constexpr int kScanItems = 8;
constexpr int kScanTile = kScanThreads * kScanItems;  // 2048 values per block

__global__ void csr_init_kernel(int64_t* rowptr, int64_t n1, int32_t* flag) {
  const int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i < n1) rowptr[i] = 0;
  if (i == 0) *flag = 1;
}

__global__ void csr_count_kernel(const int64_t* __restrict__ keys, int64_t E, int64_t N, int64_t* rowptr,
                                 int32_t* flag) {
  const int64_t e = int64_t(blockIdx.x) * blockDim.x + threadIdx.x;
  if (e >= E) return;
  const int64_t k = keys[e];
  if (k < 0 || k >= N) {
    atomicMin(flag, -1);
    return;
  }
  if (e > 0 && keys[e - 1] > k) atomicMin(flag, 0);
  atomicAdd(reinterpret_cast<unsigned long long*>(rowptr + k + 1), 1ULL);
}

// In-place inclusive scan of one 2048-value tile per block; the tile total goes to sums[block].
__global__ void __launch_bounds__(kScanThreads) scan_tile_kernel(int64_t* data, int64_t n, int64_t* sums) {
  __shared__ int64_t warp_tot[kScanThreads / 32];
  const int64_t base = int64_t(blockIdx.x) * kScanTile + int64_t(threadIdx.x) * kScanItems;
  int64_t v[kScanItems];
  int64_t run = 0;
#pragma unroll
  for (int i = 0; i < kScanItems; ++i) {
    v[i] = (base + i < n) ? data[base + i] : 0;
    run += v[i];
    v[i] = run;
  }
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  int64_t inc = run;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const int64_t up = __shfl_up_sync(0xffffffffu, inc, o);
    if (lane >= o) inc += up;
  }
  if (lane == 31) warp_tot[warp] = inc;
  __syncthreads();
  int64_t offset = inc - run;
  for (int w = 0; w < warp; ++w) offset += warp_tot[w];
#pragma unroll
  for (int i = 0; i < kScanItems; ++i)
    if (base + i < n) data[base + i] = v[i] + offset;
  if (sums && threadIdx.x == kScanThreads - 1) sums[blockIdx.x] = offset + run;
}

__global__ void scan_add_kernel(int64_t* data, int64_t n, const int64_t* sums) {
  const int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x;
  const int64_t tile = i / kScanTile;
  if (i < n && tile > 0) data[i] += sums[tile - 1];
}

__global__ void csr_zero_kernel(int64_t* word) { *word = 0; }

__global__ void csr_cursor_kernel(const int64_t* rowptr, int64_t N, int64_t* cursor) {
  const int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i < N) cursor[i] = rowptr[i];
}

__global__ void csr_fill_kernel(const int64_t* __restrict__ keys, int64_t E, int64_t N, int64_t* cursor,
                                int64_t* slots, int64_t* order, const int32_t* flag) {
  const int64_t e = int64_t(blockIdx.x) * blockDim.x + threadIdx.x;
  if (e >= E) return;
  if (*flag == 1) {
    order[e] = e;
    return;
  }
  const int64_t k = keys[e];
  if (k < 0 || k >= N) return;
  const unsigned long long pos = atomicAdd(reinterpret_cast<unsigned long long*>(cursor + k), 1ULL);
  slots[pos] = e;
}

// In-row ordering.  The slot hand-out above leaves the edge ids of a row in arrival order; they are put in
// ascending order (a stable sort of the whole list) by one of two kernels:
//   rows of at most kLongRow edges: one warp per row ranks every id against the row (quadratic, but the row is
//     short and stays in L1);
//   longer rows (listed by the first kernel): one block per row sorts the ids in place with a bitonic network whose every compare-exchange
//     keeps the minimum at the lower index, so positions beyond the row's end act as +infinity and are never
//     touched; O(L log^2 L) instead of O(L^2), which bounds the run time of degenerate inputs (few rows, a
//     million edges).
constexpr int64_t kLongRow = 2048;

__global__ void csr_rank_kernel(const int64_t* __restrict__ rowptr, int64_t N, const int64_t* __restrict__ slots,
                                int64_t* order, const int32_t* flag, int64_t* long_rows, int64_t* long_count) {
  if (*flag == 1) return;
  const int64_t row = (int64_t(blockIdx.x) * blockDim.x + threadIdx.x) / 32;
  if (row >= N) return;
  const int lane = threadIdx.x & 31;
  const int64_t begin = rowptr[row], end = rowptr[row + 1];
  if (end - begin > kLongRow) {                // handed to csr_sort_long_rows_kernel through a list
    if (lane == 0) long_rows[atomicAdd(reinterpret_cast<unsigned long long*>(long_count), 1ULL)] = row;
    return;
  }
  for (int64_t a = begin + lane; a < end; a += 32) {
    const int64_t mine = slots[a];
    int64_t rank = 0;
    for (int64_t b = begin; b < end; ++b) rank += slots[b] < mine;
    order[begin + rank] = mine;
  }
}

// A small fixed grid walks the list of long rows (usually empty: the blocks read one counter and leave).
__global__ void csr_sort_long_rows_kernel(const int64_t* __restrict__ rowptr, int64_t* slots, int64_t* order,
                                          const int32_t* flag, const int64_t* long_rows, const int64_t* long_count) {
  if (*flag == 1) return;
  const int64_t count = *long_count;
  for (int64_t item = blockIdx.x; item < count; item += gridDim.x) {
    const int64_t row = long_rows[item];
    const int64_t begin = rowptr[row], len = rowptr[row + 1] - begin;
    int64_t* v = slots + begin;
    int64_t padded = 1;
    while (padded < len) padded <<= 1;
    for (int64_t k = 2; k <= padded; k <<= 1) {
      for (int64_t j = k >> 1; j > 0; j >>= 1) {
        for (int64_t i = threadIdx.x; i < padded; i += blockDim.x) {
          const int64_t l = (j == (k >> 1)) ? (i ^ (k - 1)) : (i ^ j);     // first step of a stage mirrors the block
          if (l > i && l < len) {
            const int64_t a = v[i], b = v[l];
            if (a > b) { v[i] = b; v[l] = a; }
          }
        }
        __syncthreads();
      }
    }
    for (int64_t i = threadIdx.x; i < len; i += blockDim.x) order[begin + i] = v[i];
    __syncthreads();
  }
}

static int64_t scan_sums_elems(int64_t n) {
  int64_t total = 0;
  while (n > kScanTile) {
    n = (n + kScanTile - 1) / kScanTile;
    total += n;
  }
  return total + 1;
}

// Inclusive scan of data[0..n) using `sums` as scratch for the tile totals of every level.
static void inclusive_scan(int64_t* data, int64_t n, int64_t* sums, cudaStream_t st) {
  if (n <= 0) return;
  const int64_t tiles = (n + kScanTile - 1) / kScanTile;
  scan_tile_kernel<<<(unsigned)tiles, kScanThreads, 0, st>>>(data, n, tiles > 1 ? sums : nullptr);
  if (tiles > 1) {
    inclusive_scan(sums, tiles, sums + tiles, st);
    scan_add_kernel<<<(unsigned)((n + 255) / 256), 256, 0, st>>>(data, n, sums);
  }
}

// ---- built-in scratch for callers that cannot allocate (see ictc_csr_build_static) ----------------
constexpr int64_t kStaticMaxNodes = 1 << 16;   // 65,536 rows
constexpr int64_t kStaticMaxEdges = 1 << 20;   // 1,048,576 edges
constexpr int64_t kStaticElems = kStaticMaxNodes + kStaticMaxEdges + 64;   // + scan totals and padding
static __device__ __align__(256) int64_t g_csr_static_scratch[kStaticElems];   // ~8.9 MB per device

}  // namespace ictc

using namespace ictc;

extern "C" {

int64_t ictc_csr_scratch_bytes(int64_t N, int64_t E) {
  if (N < 0 || E < 0) return 0;
  return 8 * (N + E + scan_sums_elems(N + 1) + 2);
}

// Device address of the built-in scratch on the current device, looked up on first use per device.
static int static_scratch(void** out) {
  static std::mutex lock;
  static void* cache[64] = {};
  int dev = 0;
  cudaError_t err = cudaGetDevice(&dev);
  if (err != cudaSuccess || dev < 0 || dev >= 64) {
    set_error("csr_build_static: cannot identify the current device");
    return ICTC_ERR_LAUNCH;
  }
  std::lock_guard<std::mutex> guard(lock);
  if (!cache[dev]) {
    void* p = nullptr;
    // In host code the array name is only a handle; the kernels need its address on THIS device.
    err = cudaGetSymbolAddress(&p, g_csr_static_scratch);
    if (err != cudaSuccess || !p) {
      set_error("csr_build_static: cudaGetSymbolAddress failed: %s", cudaGetErrorString(err));
      return ICTC_ERR_LAUNCH;
    }
    cache[dev] = p;
  }
  *out = cache[dev];
  return ICTC_OK;
}

int ictc_csr_build(const int64_t* keys, int64_t N, int64_t E, int64_t* rowptr, int64_t* order, int32_t* sorted_flag,
                   void* scratch, void* stream);

int ictc_csr_build_static(const int64_t* keys, int64_t N, int64_t E, int64_t* rowptr, int64_t* order,
                          int32_t* sorted_flag, void* stream) {
  if (N < 0 || E < 0) { set_error("csr_build_static: negative size"); return ICTC_ERR_BAD_ARG; }
  if (N > kStaticMaxNodes || E > kStaticMaxEdges) {
    set_error("csr_build_static: %lld rows / %lld edges exceed the built-in scratch (at most %lld rows and %lld "
              "edges); use ictc_csr_build with caller-owned scratch", (long long)N, (long long)E,
              (long long)kStaticMaxNodes, (long long)kStaticMaxEdges);
    return ICTC_ERR_TOO_LARGE;
  }
  if (ictc_csr_scratch_bytes(N, E) > kStaticElems * 8) {
    set_error("csr_build_static: internal size bound violated");
    return ICTC_ERR_TOO_LARGE;
  }
  void* scratch = nullptr;
  if (int rc = static_scratch(&scratch)) return rc;
  return ictc_csr_build(keys, N, E, rowptr, order, sorted_flag, scratch, stream);
}

// Inclusive scan of an int64 device vector in place (used by the neighbour build for its row offsets).
int64_t ictc_scan_scratch_bytes(int64_t n) { return n < 0 ? 0 : 8 * (scan_sums_elems(n) + 2); }
int ictc_inclusive_scan_i64(int64_t* data, int64_t n, void* scratch, void* stream) {
  if (n < 0 || (n > 0 && (!data || !scratch))) { set_error("scan: invalid arguments"); return ICTC_ERR_BAD_ARG; }
  if ((n + kScanTile - 1) / kScanTile > 2147483647LL) { set_error("scan: too long"); return ICTC_ERR_TOO_LARGE; }
  inclusive_scan(data, n, reinterpret_cast<int64_t*>(scratch), (cudaStream_t)stream);
  return finish_launch("inclusive_scan");
}

int ictc_csr_static_limits(int64_t* max_nodes, int64_t* max_edges) {
  if (max_nodes) *max_nodes = kStaticMaxNodes;
  if (max_edges) *max_edges = kStaticMaxEdges;
  return ICTC_OK;
}

int ictc_csr_build(const int64_t* keys, int64_t N, int64_t E, int64_t* rowptr, int64_t* order, int32_t* sorted_flag,
                   void* scratch, void* stream) {
  if (N < 0 || E < 0) { set_error("csr_build: negative size"); return ICTC_ERR_BAD_ARG; }
  if (!rowptr || !sorted_flag || !scratch || (E > 0 && (!keys || !order))) {
    set_error("csr_build: NULL buffer");
    return ICTC_ERR_BAD_ARG;
  }
  if ((N + 256) / 256 > 2147483647LL || (E + 255) / 256 > 2147483647LL || (N + 7) / 8 > 2147483647LL) {
    set_error("csr_build: too many rows");
    return ICTC_ERR_TOO_LARGE;
  }
  cudaStream_t st = (cudaStream_t)stream;
  int64_t* cursor = reinterpret_cast<int64_t*>(scratch);
  int64_t* slots = cursor + N;
  int64_t* sums = slots + E;
  csr_init_kernel<<<(unsigned)((N + 1 + 255) / 256), 256, 0, st>>>(rowptr, N + 1, sorted_flag);
  if (E > 0) csr_count_kernel<<<(unsigned)((E + 255) / 256), 256, 0, st>>>(keys, E, N, rowptr, sorted_flag);
  inclusive_scan(rowptr, N + 1, sums, st);
  if (E > 0) {
    if (N > 0) csr_cursor_kernel<<<(unsigned)((N + 255) / 256), 256, 0, st>>>(rowptr, N, cursor);
    csr_fill_kernel<<<(unsigned)((E + 255) / 256), 256, 0, st>>>(keys, E, N, cursor, slots, order, sorted_flag);
    if (N > 0) {
      // the cursor array is free again after the fill: it becomes the list of long rows, its counter sits behind
      // the scan totals (the last of the spare words of the scratch)
      int64_t* long_count = sums + scan_sums_elems(N + 1) + 1;
      csr_zero_kernel<<<1, 1, 0, st>>>(long_count);
      csr_rank_kernel<<<(unsigned)((N + 7) / 8), 256, 0, st>>>(rowptr, N, slots, order, sorted_flag, cursor, long_count);
      if (E > kLongRow)        // a row longer than kLongRow can only exist in a list this long
        csr_sort_long_rows_kernel<<<64, 512, 0, st>>>(rowptr, slots, order, sorted_flag, cursor, long_count);
    }
  }
  return finish_launch("csr_build");
}

}  // extern "C"
