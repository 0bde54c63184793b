/*
 * ictc_b200.h — C ABI of the B200 (sm_100a) kernels for the ICTC equivariant hot path.
 *
 * Conventions (all entry points):
 *   - every pointer is a DEVICE pointer unless its name says "host"; buffers are contiguous,
 *     row-major, IEEE fp32; indices are int64; nothing is allocated, freed or synchronised;
 *   - `stream` is a cudaStream_t passed as void* (NULL = the legacy default stream);
 *   - the return value is 0 on success or a negative ICTC_ERR_* code; kernels never trap or abort;
 *   - a NULL output pointer means "this result is not needed" where the comment says so;
 *   - thread-safe for concurrent calls on different streams (no global mutable state except the
 *     entry point that is documented otherwise).
 *
 * Feature rows use the "ir_mul" layout of the reference (ictc_o3/operators.py:283-308):
 * degrees ascending, each degree stored [2l+1, C] with the channel index contiguous.  Output rows:
 * degrees ascending, inside a degree one slot per path (slot order = reference `path_offset`,
 * ictc_o3/basis/ictd_irreps.py:2694-2706), each slot [2l+1, C].  Gates are [E, P, C].
 *
 * Each function names the reference interface it replaces (path inside the reference project).
 */
#ifndef ICTC_B200_H
#define ICTC_B200_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define ICTC_OK 0
#define ICTC_ERR_BAD_SPEC (-1)     /* path set / degree not compiled into this library */
#define ICTC_ERR_BAD_ARG (-2)      /* NULL where a buffer is required, negative size, ... */
#define ICTC_ERR_LAUNCH (-3)       /* CUDA reported a launch error; see ictc_last_error() */
#define ICTC_ERR_TOO_LARGE (-4)    /* size beyond a documented limit */

/* Human-readable description of the last error raised on the calling thread. */
const char* ictc_last_error(void);
/* Device-side status word of the current device: kernels with bounded waits (the TMA-staged graph
 * kernels wait on mbarriers with an iteration limit) record a non-zero code instead of hanging when
 * a wait runs out.  Synchronises the device, copies the word to *host_status (host pointer) and
 * clears it when reset != 0.  0 = every kernel so far completed normally. */
int ictc_kernel_status(int* host_status, int reset);
/* Exercises the give-up path of the bounded waits without any fault: one warp polls an mbarrier on which nothing
 * ever arrives, with the kernels' own polling loop and a limit of `limit_cycles` SM cycles (at most 2e8, about 0.1 s),
 * then records `code` (non-zero) in the status word and returns normally; ictc_kernel_status then reports `code`
 * and the context stays usable.  No counterpart in the reference. */
int ictc_selftest_bounded_wait(int64_t limit_cycles, int code, void* stream);
/* Library build tag, e.g. "ictc_b200 sm_100a". */
const char* ictc_version(void);

/* ------------------------------------------------------------------ tensor-product specs
 * A spec is the natural-parity path set of EdgeTensorProduct.create(input_lmax, edge_lmax,
 * output_lmax) (reference: ictc_o3/operators.py:190-215).  Returns the spec id (>= 0) or
 * ICTC_ERR_BAD_SPEC when that path set has no compiled kernels. */
int ictc_tp_spec(int input_lmax, int edge_lmax, int output_lmax);
/* Sizes of a spec in units of one channel vector: nx feature components, nh harmonics,
 * np paths (= gate blocks), no output components, nnz non-zero couplings. */
int ictc_tp_spec_info(int spec, int* nx, int* nh, int* np, int* no, int* nnz);

/* ------------------------------------------------------------------ edge-wise tensor product
 * Replaces generated_forward with edge-owned rows (src = dst = edge id):
 *   ictc_o3/backends/k100/generated_cartesian_message.py:260-270 (forward branch :179-187),
 *   called from ictc_o3/operators.py:106-127.
 * x [E, nx*C], sh [E, nh], g [E, np*C], w [np*C] or NULL (unit base coefficients),
 * mask [E] or NULL, out [E, no*C] (fully overwritten). */
int ictc_tp_edge_forward(int spec, int channels, int64_t num_edges, const float* x, const float* sh,
                         const float* w, const float* g, const float* mask, float* out, void* stream);

/* First adjoint of the edge-wise product; replaces generated_adjoint for edge-owned rows:
 *   ictc_o3/backends/k100/generated_cartesian_message.py:271-287 (adjoint branch :188-224),
 *   called from ictc_o3/operators.py:129-158.
 * v [E, no*C] is the cotangent of out.  dx [E, nx*C], dsh [E, nh], dg [E, np*C]: each may be NULL
 * when not needed; every non-NULL output is fully overwritten. */
int ictc_tp_edge_adjoint(int spec, int channels, int64_t num_edges, const float* x, const float* sh,
                         const float* w, const float* g, const float* mask, const float* v,
                         float* dx, float* dsh, float* dg, void* stream);

/* ------------------------------------------------------------------ graph message (TP + scatter-sum)
 * out[n] = sum over edges e with dst(e) = n of TP(x[src(e)], sh[e], g[e]) * mask[e].
 * Replaces csr_forward / generated_forward with node-owned rows:
 *   ictc_o3/backends/k100/generated_csr_forward.py:136-157, generated_cartesian_message.py:260-270,
 *   driven by ictc_o3/ops/rematerialized_message.py:166-205.
 * The receiver CSR (dst_rowptr [N+1], dst_order [E] or NULL when the edge list is already sorted by
 * receiver) comes from ictc_csr_build.  Each receiver row is reduced by one warp in CSR order: no
 * atomics, bitwise reproducible.  x [N, nx*C], out [N, no*C] (fully overwritten, zero rows for
 * receivers without edges). */
int ictc_tp_graph_forward(int spec, int channels, int64_t num_nodes, int64_t num_edges, const float* x,
                          const float* sh, const float* w, const float* g, const int64_t* src,
                          const int64_t* dst_rowptr, const int64_t* dst_order, const float* mask,
                          float* out, void* stream);

/* First adjoint of the graph message; replaces generated_adjoint + source_adjoint:
 *   ictc_o3/backends/k100/generated_cartesian_message.py:271-287, generated_csr_adjoint.py:63-79,
 *   generated_csr_fused_adjoint.py:13-120, driven by ictc_o3/ops/rematerialized_message.py:25-83.
 * One traversal owned by the SENDER: dx[s] is reduced over the out-edges of s in sender-CSR order
 * (src_rowptr [N+1], src_order [E] or NULL when edges are sorted by sender), dg and dsh are written
 * per edge.  v [N, no*C] is the cotangent of out, gathered at dst[e].  dx [N, nx*C], dsh [E, nh],
 * dg [E, np*C]; each may be NULL; non-NULL outputs are fully overwritten. */
int ictc_tp_graph_adjoint(int spec, int channels, int64_t num_nodes, int64_t num_edges, const float* x,
                          const float* sh, const float* w, const float* g, const int64_t* dst,
                          const int64_t* src_rowptr, const int64_t* src_order, const float* mask,
                          const float* v, float* dx, float* dsh, float* dg, void* stream);

/* Variants with a shared gate table: gate_row [E] names, for every edge, its row in g (several edges may
 * share one row, see ictc_neighbor_pairs); NULL = row e.  dg of the adjoint stays per edge [E, np*C].
 * No counterpart in the reference. */
int ictc_tp_graph_forward_shared(int spec, int channels, int64_t num_nodes, int64_t num_edges, const float* x,
                                 const float* sh, const float* w, const float* g, const int64_t* gate_row,
                                 const int64_t* src, const int64_t* dst_rowptr, const int64_t* dst_order,
                                 const float* mask, float* out, void* stream);
int ictc_tp_graph_adjoint_shared(int spec, int channels, int64_t num_nodes, int64_t num_edges, const float* x,
                                 const float* sh, const float* w, const float* g, const int64_t* gate_row,
                                 const int64_t* dst, const int64_t* src_rowptr, const int64_t* src_order,
                                 const float* mask, const float* v, float* dx, float* dsh, float* dg, void* stream);

/* Chunked graph message: the same kernels over a range of owner rows, with the gates (and, for the adjoint, the
 * gate gradients) of the chunk's edges in buffers that cover the chunk only, so that no [E, np*C] table has to
 * exist whole.  Follows the reference's bounded-memory gate streaming: gates of an edge tile are produced, consumed
 * and dropped, and recomputed for the reverse sweep (ictc_o3/ops/streamed_gate_message.py:112-116, 193-221; tile
 * sizes mace_ictc/interfaces/lammps_hp.py:163-172).
 * forward: num_rows receiver rows; dst_rowptr points at the chunk's first of num_rows + 1 CSR entries (entries keep
 *   their global values), out at the chunk's first output row; x, sh, src are the whole arrays.  Gate row of edge e =
 *   (gate_row ? gate_row[e] : e) - *g_base, clamped to [0, g_capacity); g_base is a DEVICE scalar (normally the
 *   chunk's first CSR entry itself), NULL = 0 and no clamp.
 * adjoint: num_rows sender rows; src_rowptr, x and dx point at the chunk's first row; dst, v, sh, dsh are whole.
 *   g_by_position != 0: gate row = q - *g_base for the edge at position q of the sender CSR order (gate_row is
 *   ignored).  dg_base (DEVICE scalar) != NULL: the gate gradient of the edge at position q is stored in row
 *   q - *dg_base of dg when that lies in [0, dg_capacity) and dropped otherwise; NULL: row = edge id as in
 *   ictc_tp_graph_adjoint.  Capacities make an under-sized buffer safe: results are then incomplete, never out of
 *   bounds; the caller compares the chunk's edge count with its capacity. */
int ictc_tp_graph_forward_chunk(int spec, int channels, int64_t num_rows, const float* x, const float* sh,
                                const float* w, const float* g, const int64_t* gate_row, const int64_t* g_base,
                                int64_t g_capacity, const int64_t* src, const int64_t* dst_rowptr,
                                const int64_t* dst_order, const float* mask, float* out, void* stream);
int ictc_tp_graph_adjoint_chunk(int spec, int channels, int64_t num_rows, const float* x, const float* sh,
                                const float* w, const float* g, const int64_t* gate_row, int g_by_position,
                                const int64_t* g_base, int64_t g_capacity, const int64_t* dst,
                                const int64_t* src_rowptr, const int64_t* src_order, const float* mask, const float* v,
                                float* dx, float* dsh, float* dg, const int64_t* dg_base, int64_t dg_capacity,
                                void* stream);

/* ------------------------------------------------------------------ CSR topology
 * Counting sort of edges by an int64 key in [0, num_nodes): rowptr [N+1], order [E] (edge ids,
 * ascending inside a row, i.e. a stable sort), *sorted_flag (device int32) = 1 when the keys were
 * already non-decreasing (then order is the identity).  Replaces
 *   ictc_o3/backends/k100/generated_csr_forward.py:17-31 and the device counting sort
 *   ictc_o3/ops/message_topology.py:15-36.
 * scratch: device buffer of ictc_csr_scratch_bytes(N, E) bytes owned by the caller.
 * Keys outside [0, N) are ignored by the count and set *sorted_flag to -1. */
int64_t ictc_csr_scratch_bytes(int64_t num_nodes, int64_t num_edges);
int ictc_csr_build(const int64_t* keys, int64_t num_nodes, int64_t num_edges, int64_t* rowptr,
                   int64_t* order, int32_t* sorted_flag, void* scratch, void* stream);

/* ictc_csr_build without any allocation by anyone: same result as ictc_csr_build, but the scratch is
 * a fixed array built into the library (about 8.9 MB of device memory on every GPU that loads the
 * library, held until the process exits), so the caller passes inputs and outputs only.
 * No counterpart in the reference; added for hosts that cannot call cudaMalloc where the topology is
 * rebuilt, e.g. an MD driver that re-sorts its edges every few steps inside a loop where an
 * allocation would stall the whole device, or a plugin host that hands out all device memory at
 * start-up and offers no allocator afterwards.
 * Limits: num_nodes <= 65,536 and num_edges <= 1,048,576 (ictc_csr_static_limits reports them);
 * larger sizes return ICTC_ERR_TOO_LARGE and change nothing.
 * The first call on each device looks up the device address of the built-in array (one
 * cudaGetSymbolAddress with that device current); make that first call before any stream capture
 * begins.  The entry point itself calls no cudaMalloc / cudaFree or any allocating routine.
 * All calls on a device share the one array and it keeps whatever the previous call left there;
 * nothing in it needs to start at zero (every part is written before it is read within a call),
 * but two calls whose kernels overlap on the GPU (different streams) race on it: serialise them. */
int ictc_csr_build_static(const int64_t* keys, int64_t num_nodes, int64_t num_edges, int64_t* rowptr,
                          int64_t* order, int32_t* sorted_flag, void* stream);
int ictc_csr_static_limits(int64_t* host_max_nodes, int64_t* host_max_edges);

/* In-place inclusive prefix sum of an int64 device vector (row offsets of variable-length rows).
 * scratch: ictc_scan_scratch_bytes(n) bytes. */
int64_t ictc_scan_scratch_bytes(int64_t n);
int ictc_inclusive_scan_i64(int64_t* data, int64_t n, void* scratch, void* stream);

/* ------------------------------------------------------------------ neighbour list and MD integrator
 * Full neighbour list of the first num_centres atoms among num_atoms rows of pos [N,3] (fp32):
 * edge (src = j, dst = i) for every ordered pair with |r_i - r_j + S*box|^2 <= cutoff^2, evaluated in
 * double precision on the fp32 coordinates (each operation rounded separately), ordered by
 * (dst, src, S_x, S_y, S_z).  Semantics of the reference's graph fill and canonical edge order:
 *   lammps_user_mfftorch/src/USER-MFFTORCH/pair_mff_torch_kokkos.cpp:661-871, 897-911.
 * host_lo/host_hi: bounds of the cell grid (HOST double[3]; all atoms lie inside), host_box: periodic
 * lengths, host_periodic: int[3] flags; an axis that is not periodic gets no image shifts.
 * Step 1 ictc_neighbor_count writes per-centre counts to rowptr[1..centres] (rowptr[0] = 0); the caller
 * turns them into offsets with ictc_inclusive_scan_i64 and sizes the edge buffers from
 * rowptr[centres].  Step 2 ictc_neighbor_fill (same positions, same scratch, untouched in between)
 * writes src, dst [E], shifts [E,3] (fp32, lattice units, edge_vec = pos[dst] - pos[src] + shifts*box)
 * and uses edge_keys [E] as work space.  Rows that would exceed `capacity` edges are skipped.
 * scratch: ictc_neighbor_scratch_bytes() bytes. */
int64_t ictc_neighbor_scratch_bytes(int64_t num_atoms, const double* host_lo, const double* host_hi, double cutoff);
int ictc_neighbor_count(const float* pos, int64_t num_atoms, int64_t num_centres, const double* host_lo,
                        const double* host_hi, const double* host_box, const int* host_periodic, double cutoff,
                        int64_t* rowptr, void* scratch, void* stream);
int ictc_neighbor_fill(const float* pos, int64_t num_atoms, int64_t num_centres, const double* host_lo,
                       const double* host_hi, const double* host_box, const int* host_periodic, double cutoff,
                       const int64_t* rowptr, int64_t capacity, int64_t* src, int64_t* dst, float* shifts,
                       int64_t* edge_keys, void* scratch, void* stream);
/* Fixed-capacity edge buffers, step 0: after the prefix sum, clamp the row offsets to `capacity` so that
 * ictc_neighbor_fill and every consumer stay inside the buffers; *overflow (device int32) is set to 1 when the
 * list did not fit (rows were dropped: the caller must redo the step with a larger capacity) and is never
 * cleared by this call, so the caller zeroes it and may poll it every few steps. */
int ictc_neighbor_clamp(int64_t* rowptr, int64_t num_centres, int64_t capacity, int32_t* overflow, void* stream);
/* Fixed-capacity edge buffers: after ictc_neighbor_fill, rows [*count, capacity) of src/dst/shifts are set
 * to the inert edge (pad_src, pad_dst, zero shift) and *overflow (device int32, may be NULL) tells
 * whether *count exceeded the capacity.  `count` is a DEVICE pointer (normally &rowptr[num_centres]).
 * This lets a whole MD step run without the host ever learning the edge count (CUDA-graph replay). */
int ictc_neighbor_pad(const int64_t* count, int64_t capacity, int64_t pad_src, int64_t pad_dst, int64_t* src,
                      int64_t* dst, float* shifts, int32_t* overflow, void* stream);
/* Radial pairing of a neighbour list built by ictc_neighbor_fill (edge_keys = its work array, untouched
 * since): the edge (j -> i, S) and its reverse (i -> j, -S) have bitwise the same length, so length-only
 * quantities (radial basis, gate MLP) are evaluated once per pair.  Outputs: gate_row [capacity] = pair id
 * of every edge, rep_edge / other_edge [unique_capacity] = the representative edge of each pair and its
 * reverse (-1 when the reverse is not in the list, e.g. the sender is a ghost), *num_unique (device) =
 * number of pairs.  Rows of the pair table beyond *num_unique name the last edge slot (capacity - 1).
 * rev, scan [capacity]: work arrays; scan_scratch: ictc_scan_scratch_bytes(capacity) bytes.
 * No counterpart in the reference (it evaluates the radial MLP per directed edge). */
int ictc_neighbor_pairs(const int64_t* rowptr, const int64_t* dst, const int64_t* edge_keys, int64_t num_centres,
                        int64_t capacity, int64_t unique_capacity, const int64_t* count, int64_t* rev, int64_t* scan,
                        int64_t* gate_row, int64_t* rep_edge, int64_t* other_edge, int64_t* num_unique,
                        void* scan_scratch, void* stream);
/* Half step of velocity Verlet: vel += dt/2 * F/m (A, fs, eV, amu); with drift != 0 also
 * pos += dt * vel, wrapped into [0, box) on axes with box > 0.  The reference leaves integration to
 * LAMMPS `fix nve` (examples/in.hco); this is the stand-alone equivalent. */
int ictc_md_kick(int64_t num_atoms, float dt, const float* force, const float* inv_mass, float* vel, float* pos,
                 const float* box, int drift, void* stream);

/* ------------------------------------------------------------------ fused element-wise ends of the model
 * Edge geometry: vec = pos[dst] - pos[src] + shifts*box, length, unit vector, direction harmonics
 * (lmax 2, [E,9]) and the Bessel radial basis with polynomial envelope of order p ([E,num_basis]) in one
 * pass; the backward pass turns cotangents of the harmonics and of the radial basis into d/dvec.
 * Replaces the operator chain of mace_ictc/models/mace/backbone.py:941-973 (radial_basis.py:11-92,
 * ictc_o3/basis/ictd_irreps.py:1153-1208).  host_box: HOST float[3] (ignored when shifts is NULL). */
int ictc_edge_geometry_forward(const float* pos, const int64_t* src, const int64_t* dst, const float* shifts,
                               const float* host_box, float r_max, int num_basis, int p, int64_t num_edges,
                               float* sh, float* rb, float* unit, float* length, void* stream);
int ictc_edge_geometry_backward(const float* unit, const float* length, float r_max, int num_basis, int p,
                                int64_t num_edges, const float* dsh, const float* drb, float* dvec, void* stream);
/* grad[i] = sum_{dst(e)=i} dvec[e] - sum_{src(e)=i} dvec[e] for the first num_rows atoms; edges are sorted
 * by receiver (dst_rowptr over the first num_dst_rows rows) and grouped by sender through the sender CSR.
 * Atomic-free replacement of autograd's index_add scatter (the reference's add_forces,
 * pair_mff_torch_kokkos.cpp:1130-1160). */
int ictc_position_gradient(int64_t num_rows, int64_t num_dst_rows, const int64_t* dst_rowptr,
                           const int64_t* src_rowptr, const int64_t* src_order, const float* dvec, float* grad,
                           void* stream);
/* y = silu(x)*scale and its first derivative; replaces run(x,g,h,y,z,scale,mode,...) modes 0/1 of
 * ictc_o3/backends/k100/hip_activation.py:27-38. */
int ictc_silu_forward(int64_t n, float scale, const float* x, float* y, void* stream);
int ictc_silu_backward(int64_t n, float scale, const float* x, const float* dy, float* dx, void* stream);
/* Whole-row conversion between the model-native mul_ir layout (every block [C, 2l+1], channel outer) and the
 * kernel-native ir_mul layout (every block [2l+1, C], channel contiguous) in one launch.  A row is a sequence of
 * num_blocks degree blocks; block b holds host_counts[b] path slots of host_ms[b] components each (HOST int
 * arrays, at most 8 blocks).  to_ir_mul != 0: in is mul_ir, out is ir_mul; 0: the reverse.  in and out must
 * not overlap.  Replaces the `fused_pack` conversion kernel of ictc_o3/ops/message_layout.py:25-93
 * (copy_layout, ictc_o3/backends/k100/hip_message_layout.py:27-34). */
int ictc_layout_copy(int64_t rows, int channels, int num_blocks, const int* host_counts, const int* host_ms,
                     const float* in, float* out, int to_ir_mul, void* stream);

/* Radial gate MLP num_basis -> 64 -> 64 -> 64 -> num_out (bias-free, SiLU * 1.6791767923989418 between layers; the
 * `fc` stack of the interaction block, mace_ictc/models/mace/layers.py:825-835) runs as two kernels: the hidden
 * layers as a chain through tensor memory (ictc_mlp_chain_*, below) and the wide last layer as a tcgen05 GEMM.
 * Last layer (tiled per edge chunk in the reference by ictc_o3/ops/streamed_gate_message.py:112-116; input
 * gradient streamed_gate_message.py:224-260) as
 * tcgen05.mma TF32 products with a three-term operand split (fp32-level accuracy), accumulators in TMEM.
 * ictc_gate_pack_weights: W3 [num_out, 64] -> `packed` [2 * num_out * 64] floats in the shared-memory operand
 *   layout, 64-unit chunks, transpose = 0 for the forward, 1 for the backward.  num_out % 64 == 0.
 * ictc_gate_gemm_forward: gates[r, :] = act(z3[r, :]) @ W3^T, act = scaled SiLU when apply_silu != 0.
 * ictc_gate_gemm_backward: da3[r, :] = (dgates[pair_a[r], :] + dgates[pair_b[r], :]) @ W3; pair_a == NULL means
 *   row r itself, pair_b == NULL or pair_b[r] < 0 means no second row.
 * row_limit (may be NULL): DEVICE scalar; only min(num_rows, *row_limit) rows are processed, so a recorded step whose
 *   buffers have a fixed capacity does no work for the unused tail.
 * All buffers 32-byte aligned.  Bounded waits report through ictc_kernel_status (codes 21-25, 31-35). */
int ictc_gate_pack_weights(int num_out, const float* w3, int transpose, float* packed, void* stream);
int ictc_gate_gemm_forward(int64_t num_rows, int num_out, const float* z3, const float* w_packed, float* gates,
                           int apply_silu, const int64_t* row_limit, void* stream);
int ictc_gate_gemm_backward(int64_t num_rows, int num_out, const float* dgates, const int64_t* pair_a,
                            const int64_t* pair_b, const float* w_packed_t, float* da3, const int64_t* row_limit,
                            void* stream);
/* The same two products over a window of a longer row list (one edge chunk of the streamed gate evaluation,
 * reference as above): the launch covers list entries [*row_begin, min(*row_begin + capacity, *row_end)), both
 * DEVICE scalars (normally two entries of a CSR row-offset array), local row r = entry *row_begin + r.
 * forward : gates[r, :] = act(z3[row_index[*row_begin + r], :]) @ W3^T   (row_index NULL: z3[*row_begin + r]);
 * backward: da3[out_index[*row_begin + r], :] = dgates[r, :] @ W3        (out_index NULL: da3[*row_begin + r]). */
int ictc_gate_gemm_forward_rows(int64_t capacity, int num_out, const float* z3, const int64_t* row_index,
                                const int64_t* row_begin, const int64_t* row_end, const float* w_packed, float* gates,
                                int apply_silu, void* stream);
int ictc_gate_gemm_backward_rows(int64_t capacity, int num_out, const float* dgates, const int64_t* row_begin,
                                 const int64_t* row_end, const int64_t* out_index, const float* w_packed_t, float* da3,
                                 void* stream);

/* Per-degree channel linear map on the same tcgen05 kernels (reference: ictc_o3/operators.py:609-628
 * channel_linear; mace_ictc/models/mace/layers.py:21-87 linear_up / message_linear; products.py:817): rows are
 * (node, component) pairs with 64 contiguous channels, out = in @ W with fp32-level accuracy (three-term TF32).
 * Exactly one side is 64 wide: k_chunks == 1 gives N = 64 * n_chunks outputs per row, n_chunks == 1 contracts
 * K = 64 * k_chunks inputs.  Row g is component g % mm of node g / mm; the 64-float block b of that row on the
 * wide side starts at base + (g / mm) * ld + (b * mm + g % mm) * 64 (the path-slot-major layout
 * [node][slot][component][channel] of the tensor-product output, read or written in place), the block of the
 * 64-wide side at base + (g / mm) * ld + (g % mm) * 64.  mm = 1 with ld = row length is a plain matrix.
 * w_packed comes from ictc_gate_pack_weights: W given as [64 * n_chunks, 64] (out unit major) with
 * transpose = 0 when k_chunks == 1, as [64 * k_chunks, 64] (in unit major) with transpose = 1 otherwise.
 * Buffers 32-byte aligned, ld a multiple of 8. */
int ictc_channel_linear_tc(int64_t num_rows, int k_chunks, int n_chunks, const float* in, int in_mm, int64_t in_ld,
                           const float* w_packed, float* out, int out_mm, int64_t out_ld, void* stream);

/* Weight gradient of a row-wise linear map, dW[o, i] = sum_r grad[r, o] * rows[r, i], contracted over the rows on
 * the tensor cores with fp32-level accuracy (three-term TF32) and a fixed summation order (reference: the dW branch
 * of the training gate, ictc_o3/ops/training_gate_message.py:120-186, and the weight gradients of channel_linear,
 * ictc_o3/operators.py:609-628, under autograd).  num_out is a multiple of 64 up to 768, `rows` contributes 64
 * columns; grad_ld / rows_ld / dweight_ld are row strides in floats, so a wider `rows` or `dweight` is covered by
 * one call per 64-column block.  `workspace` holds ictc_weight_grad_workspace(num_rows, num_out) bytes (16-byte
 * aligned; negative result: unsupported size). */
int64_t ictc_weight_grad_workspace(int64_t num_rows, int num_out);
int ictc_weight_grad_tc(int64_t num_rows, int num_out, const float* grad, int64_t grad_ld, const float* rows,
                        int64_t rows_ld, float* dweight, int64_t dweight_ld, float* workspace, void* stream);

/* Hidden layers of the gate MLP as a chain through tensor memory (same reference as the last layer above):
 * the two 64 x 64 layers are three-term TF32 tcgen05.mma products with the activations kept in TMEM, the
 * num_basis-wide layer is fp32 FMA.  w1_packed / w2_packed come from ictc_gate_pack_weights(64, W, 0, ...),
 * w1t_packed / w2t_packed from ictc_gate_pack_weights(64, W, 1, ...); w0 is the plain [64, num_basis] matrix.
 * forward: rb rows -> pre-activations z1, z2, z3 [E, 64]; row r reads rb[rb_rows[r]] (rb_rows NULL: rb[r]).
 * backward: da3 [E, 64] (gradient of silu(z3)) and z1..z3 -> drb; row r is written (accumulate == 0) or added
 *   (accumulate != 0) to drb[drb_rows[r]] (drb_rows NULL: drb[r]); a row index that repeats (the inert padding
 *   rows of a fixed-capacity pair table) receives an unspecified one of its results.
 * row_limit: as for ictc_gate_gemm_forward.
 * z*, da3 and the packed weights 32-byte aligned.  Bounded waits report codes 41-46. */
int ictc_mlp_chain_forward(int64_t num_edges, int num_basis, const float* rb, const int64_t* rb_rows, const float* w0,
                           const float* w1_packed, const float* w2_packed, float* z1, float* z2, float* z3,
                           const int64_t* row_limit, void* stream);
int ictc_mlp_chain_backward(int64_t num_edges, int num_basis, const float* da3, const float* w0, const float* w1t_packed,
                            const float* w2t_packed, const float* z1, const float* z2, const float* z3, float* drb,
                            const int64_t* drb_rows, int accumulate, const int64_t* row_limit, void* stream);
/* ictc_mlp_chain_backward over a pair table: row r starts from da3[pair_a[r]] + da3[pair_b[r]] (pair_b[r] < 0:
 * the first term only; both NULL: da3[r]), i.e. the two edges of a radial pair add their gradients as they are
 * read.  No counterpart in the reference (it has no pairing). */
int ictc_mlp_chain_backward_paired(int64_t num_edges, int num_basis, const float* da3, const int64_t* pair_a,
                                   const int64_t* pair_b, const float* w0, const float* w1t_packed,
                                   const float* w2t_packed, const float* z1, const float* z2, const float* z3,
                                   float* drb, const int64_t* drb_rows, int accumulate, const int64_t* row_limit,
                                   void* stream);

/* ------------------------------------------------------------------ direction harmonics
 * Component-normalised Cartesian harmonics of unit vectors, degrees 0..lmax (lmax <= 2 here).
 * Replaces the harmonics<MODE> kernel run(n,g,h,y,dn,dg,mode,needn,needg):
 *   ictc_o3/backends/k100/hip_direction_harmonics.py:11-56 (math: ictc_o3/basis/ictd_irreps.py:1153-1208).
 * forward: n [E,3] -> y [E,(lmax+1)^2].
 * vjp:     dn[e,a] = sum_h gy[e,h] dY_h/dn_a                        (MODE 1)
 * second:  given tangent hn [E,3] on the vjp output: dgy[e,h] = sum_a hn_a dY_h/dn_a,
 *          dn2[e,a] = sum_h gy_h sum_b hn_b d2Y_h/dn_a dn_b          (MODE 2); either may be NULL. */
int ictc_harmonics_forward(int lmax, int64_t num_edges, const float* n, float* y, void* stream);
int ictc_harmonics_vjp(int lmax, int64_t num_edges, const float* n, const float* gy, float* dn, void* stream);
int ictc_harmonics_second(int lmax, int64_t num_edges, const float* n, const float* gy, const float* hn,
                          float* dn2, float* dgy, void* stream);

/* ------------------------------------------------------------------ symmetric contraction
 * Per-species symmetric contraction of correlation 3 over lmax-2 node features:
 *   y[n,c,l,m] = sum_nu sum_p W_nu^l[species(n),p,c] sum U_nu^l[m,i1..i_nu,p] prod_k x[n,c,i_k]
 * Replaces the SC circuit kernels run(x, bank, g, idx, out, backward), the training-mode run(...) and
 * reduce(...):  ictc_o3/backends/k100/hip_circuit.py:115-125, 223-255 (math:
 * ictc_o3/ops/_mace_symmetric_contraction.py:298-354 with U from ictc_o3/basis/ictd_irreps.py:1535-1557).
 * Only lmax = 2 and target_lmax in {0, 2} are compiled.
 *   x  [N, 9*C]   node features; ir_mul = 0: degree blocks [C, 2l+1] (the reference's mul_ir rows),
 *                 ir_mul = 1: degree blocks [2l+1, C]
 *   w  [S, NW, C] packed weight bank, NW = ictc_sc_num_weights(); block order (l_out, nu = 1,2,3, p)
 *   y  [N, (target_lmax+1)^2 * C] in the same block convention as x
 * adjoint: gy is the cotangent of y; gx [N, 9*C] and gw [S, NW, C] may each be NULL.
 * second : mixed second derivatives.  With Phi = <gy, y>, gx = dPhi/dx, gw = dPhi/dw and cotangents
 *          hx (of gx, may be NULL) and hw (of gw, may be NULL):  Psi = <hx, gx> + <hw, gw>;
 *          dgy = dPsi/dgy, dx = dPsi/dx, dw = dPsi/dw (each may be NULL).
 * scratch: device buffer of ictc_sc_scratch_bytes() bytes, needed when gw / dw is requested (chunk
 *          partial sums of the weight gradient, reduced in fixed order: no float atomics). */
int ictc_sc_num_weights(int lmax, int target_lmax);
int64_t ictc_sc_scratch_bytes(int lmax, int target_lmax, int channels, int64_t num_nodes, int num_species);
int ictc_sc_forward(int lmax, int target_lmax, int channels, int64_t num_nodes, int num_species, int ir_mul,
                    const float* x, const int64_t* species, const float* w, float* y, void* stream);
int ictc_sc_adjoint(int lmax, int target_lmax, int channels, int64_t num_nodes, int num_species, int ir_mul,
                    const float* x, const int64_t* species, const float* w, const float* gy, float* gx,
                    float* gw, void* scratch, void* stream);
int ictc_sc_second(int lmax, int target_lmax, int channels, int64_t num_nodes, int num_species, int ir_mul,
                   const float* x, const int64_t* species, const float* w, const float* gy, const float* hx,
                   const float* hw, float* dgy, float* dx, float* dw, void* scratch, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* ICTC_B200_H */
