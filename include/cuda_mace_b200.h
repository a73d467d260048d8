/*
 * C-ABI of the B200 (sm_100a) invariant-MACE energy+force hot path.
 *
 * Every entry point takes plain device pointers and sizes, launches on the stream it is
 * given, returns 0 on success or one of the CMACE_ERR_* codes, never throws and never
 * allocates unless stated (only the *_plan_create calls allocate).  cmace_last_error()
 * returns a thread-local description of the last failure.
 *
 * Each declaration names the entry point of the cuda-mace project it replaces (paths relative
 * to that project).  Layouts are the reference's: node features X [N, C]; per-edge harmonics
 * Y [16, E] (component-major); radial weights R [E, 4, C]; messages [N, 16, C]; all row-major
 * and contiguous; indices int32; edges sorted by receiver.
 * C (channels) must be a multiple of 32.  Offsets are 64-bit throughout.
 */
#ifndef CUDA_MACE_B200_H
#define CUDA_MACE_B200_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define CMACE_OK 0
#define CMACE_ERR_ARG 1         /* bad size, null or misaligned pointer */
#define CMACE_ERR_CUDA 2        /* a CUDA runtime call or launch failed */
#define CMACE_ERR_UNSUPPORTED 3 /* shape outside what the kernels cover */

typedef void *cmace_stream_t; /* a cudaStream_t */

const char *cmace_last_error(void);
int cmace_abi_version(void);

/* ---- topology -------------------------------------------------------------------------
 * Replaces jit_calculate_first_occurences (jit_wrappers/src/invariant_message_passing_wrapper.cpp:19-70,
 * kernel cuda/src/invariant_message_passing_impl.cu:8-72).  row_ptr[n]..row_ptr[n+1] is the
 * edge range of receiver n; receivers without edges get an empty range (the reference leaves
 * theirs unwritten).  row_ptr has nnodes+1 entries. */
int cmace_receiver_csr(const int32_t *receiver, int64_t nedges, int64_t nnodes, int32_t *row_ptr,
                       cmace_stream_t stream);

/* Sender-side ordering used by the node backward; stands in for the reference's N x N reverse-edge
 * table (invariant_message_passing_wrapper.cpp:91-93, impl.cu:112-116).  perm lists the edge ids
 * grouped by sender (stable), send_ptr [nnodes+1] the group bounds.  workspace must hold
 * cmace_sender_order_workspace_bytes(nedges) bytes. */
int64_t cmace_sender_order_workspace_bytes(int64_t nedges);
int cmace_sender_order(const int32_t *sender, int64_t nedges, int64_t nnodes, int32_t *perm,
                       int32_t *send_ptr, void *workspace, int64_t workspace_bytes,
                       cmace_stream_t stream);

/* Groups nodes by chemical element for ElementalLinear; stands in for the per-element
 * torch::where + host sync of jit_elemental_linear (jit_wrappers/src/linear_wrapper.cpp:137-143).
 * node_order [nnodes] lists node ids grouped by element, elem_start [nelements+1] the bounds;
 * workspace as for cmace_sender_order with nedges = nnodes. */
int cmace_group_by_element(const int32_t *elem, int64_t nnodes, int nelements, int32_t *node_order,
                           int32_t *elem_start, void *workspace, int64_t workspace_bytes,
                           cmace_stream_t stream);

/* ---- neighbour list on the device (orthorhombic cell, cell list) -----------------------------------
 * The step before the hot path: upstream builds the list on the host (matscipy / ASE; the reference's tests use
 * tests/test_utils.py:97-105) and the reference recomputes the receiver offsets on every call
 * (src/invariant_message_passing.cpp:22); no counterpart inside the reference library.
 * Full list, receivers = the first nrecv atoms, sorted by receiver:
 *   vector(e) = pos[sender[e]] - pos[receiver[e]] + shift_idx[e] * (lx, ly, lz),  |vector| < r_cut.
 * pos [natoms,3] float64; (lox,loy,loz) + (lx,ly,lz) the box (for a non-periodic axis: the range the atoms
 * lie in); pbc_mask bit d = axis d periodic (then lx >= r_cut).  Sequence:
 *   1. cmace_nl_cell_ids_f64            -> cell_id [natoms]
 *   2. cmace_sender_order(cell_id, natoms, cmace_nl_num_cells(...), perm, cell_ptr [ncells+1], ...)
 *   3. cmace_nl_count_f64               -> count [nrecv]
 *   4. cmace_exclusive_scan_i32 over count[0..nrecv] (count[nrecv] = 0) -> row_ptr [nrecv+1]; E = row_ptr[nrecv]
 *   5. cmace_nl_fill_f64                -> sender [E], receiver [E], shift_idx [E,3] int8 and/or shifts [E,3]
 * row_ptr is the receiver CSR cmace_imp_* take.  The edges of a receiver come out in a fixed order. */
int64_t cmace_nl_num_cells(double lx, double ly, double lz, double r_cut);
int cmace_nl_cell_ids_f64(const double *pos, int64_t natoms, double lox, double loy, double loz, double lx,
                          double ly, double lz, int pbc_mask, double r_cut, int32_t *cell_id,
                          cmace_stream_t stream);
int cmace_nl_count_f64(const double *pos, int64_t natoms, int64_t nrecv, double lox, double loy, double loz,
                       double lx, double ly, double lz, int pbc_mask, double r_cut, const int32_t *perm,
                       const int32_t *cell_ptr, int32_t *count, cmace_stream_t stream);
int64_t cmace_scan_workspace_bytes(int64_t n);
int cmace_exclusive_scan_i32(const int32_t *in, int64_t n, int32_t *out, void *workspace,
                             int64_t workspace_bytes, cmace_stream_t stream);
int cmace_nl_fill_f64(const double *pos, int64_t natoms, int64_t nrecv, double lox, double loy, double loz,
                      double lx, double ly, double lz, int pbc_mask, double r_cut, const int32_t *perm,
                      const int32_t *cell_ptr, const int32_t *row_ptr, int32_t *sender, int32_t *receiver,
                      int8_t *shift_idx, double *shifts, cmace_stream_t stream);

/* ---- per-edge basis: spherical harmonics (+ Bessel x cutoff) -----------------------------
 * cmace_sph_* replace jit_spherical_harmonics / jit_spherical_harmonics_backward
 * (jit_wrappers/src/spherical_harmonics_wrapper.cpp:15-137, kernels
 * cuda/src/spherical_harmonics_impl.cu:21-334): xyz [E,3] -> Y [16,E], normalised input,
 * e3nn component order, sqrt(4 pi) scaling.  The backward recomputes the derivatives from xyz
 * instead of reading a saved dY [16,3,E].
 * cmace_edge_basis_* additionally emit the radial basis B [E, nbessel] =
 * sqrt(2/r_max) sin(n pi r/r_max)/r * polynomial cutoff(p), which the reference obtains from
 * upstream MACE's radial_embedding before tabulating it (models/InvariantMACE.py:226-240).
 * Pass B / gB = NULL to skip the radial part. */
int cmace_sph_fwd_f32(const float *xyz, int64_t nedges, float *Y, cmace_stream_t stream);
int cmace_sph_fwd_f64(const double *xyz, int64_t nedges, double *Y, cmace_stream_t stream);
int cmace_sph_bwd_f32(const float *xyz, const float *gY, int64_t nedges, float *gxyz,
                      cmace_stream_t stream);
int cmace_sph_bwd_f64(const double *xyz, const double *gY, int64_t nedges, double *gxyz,
                      cmace_stream_t stream);
int cmace_edge_basis_fwd_f32(const float *xyz, int64_t nedges, double r_max, int nbessel, int p,
                             float *Y, float *B, cmace_stream_t stream);
int cmace_edge_basis_fwd_f64(const double *xyz, int64_t nedges, double r_max, int nbessel, int p,
                             double *Y, double *B, cmace_stream_t stream);
int cmace_edge_basis_bwd_f32(const float *xyz, const float *gY, const float *gB, int64_t nedges,
                             double r_max, int nbessel, int p, float *gxyz, cmace_stream_t stream);
int cmace_edge_basis_bwd_f64(const double *xyz, const double *gY, const double *gB, int64_t nedges,
                             double r_max, int nbessel, int p, double *gxyz, cmace_stream_t stream);

/* ---- edge vectors and their position gradient ---------------------------------------------------
 * vec[e] = pos[sender[e]] - pos[receiver[e]] + shifts[e] (float64 arithmetic, stored in the kernels' precision;
 * shifts may be NULL) and its adjoint grad_pos[n] = sum_{sender = n} g[e] - sum_{receiver = n} g[e], which is
 * minus the force when g is the energy gradient with respect to the edge vectors.  The reference leaves both to
 * torch (get_edge_vectors_and_lengths, models/InvariantMACE.py:297-304, and autograd's index_add).  The adjoint
 * walks the receiver-sorted list (row_ptr [nrecv+1] from cmace_receiver_csr) and the sender grouping (perm,
 * send_ptr [nsend+1] from cmace_sender_order), one warp per atom, float64 sums in a fixed order: no atomics.
 * pos and grad_pos are [nsend,3] float64; receivers index the first nrecv atoms. */
int cmace_edge_vectors_fwd_f32(const double *pos, const int32_t *sender, const int32_t *receiver,
                               const double *shifts, int64_t nedges, float *vec, cmace_stream_t stream);
int cmace_edge_vectors_fwd_f64(const double *pos, const int32_t *sender, const int32_t *receiver,
                               const double *shifts, int64_t nedges, double *vec, cmace_stream_t stream);
int cmace_edge_vectors_bwd_f32(const float *g, const int32_t *row_ptr, const int32_t *perm,
                               const int32_t *send_ptr, int64_t nrecv, int64_t nsend, double *grad_pos,
                               cmace_stream_t stream);
int cmace_edge_vectors_bwd_f64(const double *g, const int32_t *row_ptr, const int32_t *perm,
                               const int32_t *send_ptr, int64_t nrecv, int64_t nsend, double *grad_pos,
                               cmace_stream_t stream);

/* ---- cubic spline of the radial weights ----------------------------------------------------
 * Replace jit_evaluate_spline / jit_backward_spline (jit_wrappers/src/cubic_spline_wrapper.cpp:14-153,
 * kernels cuda/src/cubic_spline_impl.cu:5-107).  coeffs [nintervals, 4, noutputs]; R [E, noutputs];
 * R is zero for r > r_max.  The backward recomputes dR/dr instead of reading a saved table. */
int cmace_spline_fwd_f32(const float *r, const float *r_knots, const float *coeffs, int64_t nedges,
                         int nintervals, int noutputs, double r_width, double r_max, float *R,
                         cmace_stream_t stream);
int cmace_spline_fwd_f64(const double *r, const double *r_knots, const double *coeffs,
                         int64_t nedges, int nintervals, int noutputs, double r_width, double r_max,
                         double *R, cmace_stream_t stream);
int cmace_spline_bwd_f32(const float *r, const float *r_knots, const float *coeffs, const float *gR,
                         int64_t nedges, int nintervals, int noutputs, double r_width, double r_max,
                         float *gr, cmace_stream_t stream);
int cmace_spline_bwd_f64(const double *r, const double *r_knots, const double *coeffs,
                         const double *gR, int64_t nedges, int nintervals, int noutputs,
                         double r_width, double r_max, double *gr, cmace_stream_t stream);

/* ---- invariant message passing ------------------------------------------------------------
 * cmace_imp_fwd_* replace jit_forward_message_passing (invariant_message_passing_wrapper.cpp:72-155,
 * kernel impl.cu:74-165): out[i,lm,c] = sum_{e in row i} X[sender[e],c] * Y[lm,e] * R[e,l(lm),c].
 * Every row of out is written (zeros for receivers without edges).
 * cmace_imp_bwd_edge_* + cmace_imp_bwd_node_* replace jit_backward_message_passing
 * (wrapper :157-284, kernels impl.cu:167-399).  The edge pass writes gradY [16,E], gradR [E,4,C] unless
 * gradR == NULL (a caller that forms the radial-weight gradient on the fly, cmace_gemm3x_gradr_f32),
 * and, when T != NULL, the per-edge sender contribution T [E,C]; the node pass sums T over each
 * sender's group into gradX [N,C].  A warp covers 32*VEC channels (VEC = 4, 2 or 1 scalars per
 * lane, the widest that divides C/32 within 16 bytes); when C needs several such chunks (e.g.
 * float64 with C = 128) each chunk writes its own partial of gradY into gradY_partial, a scratch
 * of cmace_imp_bwd_scratch_elems(...) scalars, and a second small kernel sums them.  Pass NULL
 * when that query returns 0. */
int cmace_imp_fwd_f32(const float *X, const float *Y, const float *R, const int32_t *sender,
                      const int32_t *row_ptr, int64_t nnodes, int64_t nedges, int channels,
                      float *out, cmace_stream_t stream);
int cmace_imp_fwd_f64(const double *X, const double *Y, const double *R, const int32_t *sender,
                      const int32_t *row_ptr, int64_t nnodes, int64_t nedges, int channels,
                      double *out, cmace_stream_t stream);
int64_t cmace_imp_bwd_scratch_elems(int64_t nedges, int channels, int is_f64);
/* float32 with 128 channels runs the edge pass with the R rows staged through shared memory by bulk copies.
 * Its waits on the copies are bounded (about 0.2 s); cmace_imp_staged_stalled() synchronises, returns 1 if one
 * of them gave up since the last call (the results of that launch are then incomplete) and clears the flag. */
int cmace_imp_staged_stalled(void);
int cmace_imp_bwd_edge_f32(const float *X, const float *Y, const float *R, const float *G,
                           const int32_t *sender, const int32_t *row_ptr, int64_t nnodes,
                           int64_t nedges, int channels, float *gradR, float *gradY, float *T,
                           float *gradY_partial, cmace_stream_t stream);
int cmace_imp_bwd_edge_f64(const double *X, const double *Y, const double *R, const double *G,
                           const int32_t *sender, const int32_t *row_ptr, int64_t nnodes,
                           int64_t nedges, int channels, double *gradR, double *gradY, double *T,
                           double *gradY_partial, cmace_stream_t stream);
/* No counterpart in the reference.  Same computation as cmace_imp_bwd_edge_f64 for callers that cannot
 * allocate device memory where they call from (a plugin inside a framework whose memory pool is fixed, a
 * thread that must stay out of the allocator): the gradY partials live in a 16 MiB array that is part of
 * the library image (every GPU that loads the library carries it until exit), so no scratch pointer is
 * passed and nothing is allocated or freed, by this library or by any other.  Limits and rules:
 *  - at most cmace_imp_bwd_edge_f64_noalloc_max_elems() = 2 Mi scratch doubles, i.e.
 *    cmace_imp_bwd_scratch_elems(nedges, channels, 1) must not exceed it (65 536 edges at C = 128);
 *    larger calls fail with CMACE_ERR_UNSUPPORTED and a message;
 *  - the first call on each device looks up the array's device address (that device must be current);
 *    make that first call outside any stream capture;
 *  - all calls share the one array: calls that overlap on the GPU (different streams, or several host
 *    threads) race on it; issue them on one stream or serialise them. */
int64_t cmace_imp_bwd_edge_f64_noalloc_max_elems(void);
int cmace_imp_bwd_edge_f64_noalloc(const double *X, const double *Y, const double *R, const double *G,
                                   const int32_t *sender, const int32_t *row_ptr, int64_t nnodes,
                                   int64_t nedges, int channels, double *gradR, double *gradY, double *T,
                                   cmace_stream_t stream);
int cmace_imp_bwd_node_f32(const float *T, const int32_t *perm, const int32_t *send_ptr,
                           int64_t nnodes, int channels, float *gradX, cmace_stream_t stream);
int cmace_imp_bwd_node_f64(const double *T, const int32_t *perm, const int32_t *send_ptr,
                           int64_t nnodes, int channels, double *gradX, cmace_stream_t stream);

/* ---- Linear / ElementalLinear -------------------------------------------------------------
 * Replace jit_linear and jit_elemental_linear (jit_wrappers/src/linear_wrapper.cpp:23-191, kernels
 * cuda/src/linear_impl.cu:16-255): out[n, l^2+m, :] = scale * X[n, l^2+m, :] @ W[z_n, l].
 * X [N,16,K]; W [nelements,4,K,Nout]; out [N,16,Nout].  The reference hard-codes
 * scale = 1/sqrt(K) (linear_impl.cu:33); pass that for the forward.  For Linear pass
 * nelements = 1 and node_order = elem_start = NULL.  For ElementalLinear pass the outputs of
 * cmace_group_by_element (node_order may be NULL when the nodes are already stored grouped by element:
 * element z owns nodes elem_start[z] .. elem_start[z+1] - 1).  The backward of both is the same call with the transposed weights,
 * as in the reference (src/linear.cpp:29-44, :77-93), and with the FORWARD's scale (the
 * reference re-derives it from the transposed shape, which is only right for K = Nout).
 * One launch, no host synchronisation.  The float64 entry point runs on the FP64 tensor cores (mma.sync
 * m8n8k4.f64) when K and Nout are even and the pointers 16-byte aligned, otherwise on an FMA tile kernel. */
int cmace_linear_f32(const float *X, const float *W, const int32_t *node_order,
                     const int32_t *elem_start, int nelements, int64_t nnodes, int K, int Nout,
                     double scale, float *out, cmace_stream_t stream);
int cmace_linear_f64(const double *X, const double *W, const int32_t *node_order,
                     const int32_t *elem_start, int nelements, int64_t nnodes, int K, int Nout,
                     double scale, double *out, cmace_stream_t stream);

/* Plain float64 product out[M,N] = scale * A[M,K] @ B[K,N] on the FP64 tensor cores (the tile loop of
 * cmace_linear_f64 with the identity row map; FMA tile kernel for odd K or N).  Serves the radial multilayer
 * perceptron and the node products [N,C] x [C,C] of the float64 model, which the reference leaves to
 * torch.matmul (models/InvariantMACE.py:41-53 linear_matmul) or tabulates in float32 (:226-240). */
int cmace_gemm_f64(const double *A, const double *B, int64_t M, int K, int N, double scale, double *out,
                   cmace_stream_t stream);

/* ---- float32 tensor-core path (tcgen05, kind::tf32 with a 3-term hi/lo split, TMEM accumulator) -----
 * The reference runs Linear / ElementalLinear on wmma TF32 with the same 3-term error compensation
 * (cuda/src/linear_impl.cu:85-101).  Weights are packed once into the shared-memory image the tensor
 * core reads: Bt [nmat, N, K] is the TRANSPOSE of each [K, N] weight matrix (K contiguous), i.e. W_T for
 * the forward of Linear and W for its backward.  packed needs cmace_gemm_packed_floats(nmat, N, K) floats.
 * cmace_linear_tc_f32 has the contract of cmace_linear_f32 (Nout <= 128), with one addition: for nelements > 1
 * node_order may be NULL when the nodes are STORED grouped by element (element z owns the nodes
 * elem_start[z] .. elem_start[z+1] - 1); without a gather list the rows move by TMA.  cmace_gemm3x_f32 is the plain
 * out[M,N] = scale * A[M,K] @ B used for the radial multilayer perceptron (which upstream MACE evaluates
 * with torch and the reference replaces by its spline table, models/InvariantMACE.py:226-240).
 * status: optional device int32, set non-zero if a bounded wait inside the kernel timed out. */
int64_t cmace_gemm_packed_floats(int nmat, int N, int K);
int cmace_gemm_pack_weights_f32(const float *Bt, int nmat, int N, int K, float *packed,
                                cmace_stream_t stream);
int cmace_gemm3x_f32(const float *A, const float *packed, int64_t M, int K, int N, double scale,
                     float *out, int32_t *status, cmace_stream_t stream);
int cmace_linear_tc_f32(const float *X, const float *packed, const int32_t *node_order,
                        const int32_t *elem_start, int nelements, int64_t nnodes, int K, int Nout,
                        double scale, float *out, int32_t *status, cmace_stream_t stream);

/* Gradient of the last hidden radial activations without a gradR array (no counterpart in the reference, whose
 * backward writes gradR [E,4,C] for its spline kernel, invariant_message_passing_impl.cu:283-291):
 *   out[e, :] = sum_{l,c} gradR[e,l,c] * W[:, l*C + c],   gradR[e,l,c] = X[sender[e],c] * sum_{m in l} Y[m,e] * G[receiver[e],m,c]
 * i.e. cmace_gemm3x_f32 applied to the radial-weight gradient of cmace_imp_bwd_edge_f32, whose rows are formed in
 * the producer warps of the tensor-core kernel instead of being read from memory (call the edge pass with
 * gradR = NULL for gradY and T).  X [Ns,C], G [Nr,16,C], Y [16,E], sender / receiver [E] sorted by receiver,
 * C in {32,64,96,128}; packed = cmace_gemm_pack_weights_f32 of Bt = W [N, 4C] (the last radial layer, N its input
 * width, 32 <= N <= 128, a multiple of 4); out [E, N]. */
/* No counterpart in the reference.  Launches one warp that waits, with the bounded wait the tensor-core kernels
 * use, on a barrier nothing completes; after limit_seconds (0 < limit <= 1) the kernel writes `code` (non-zero)
 * into *status (if it still holds 0) and returns.  The context stays usable: this is how a caller (or a test)
 * exercises the time-out reporting without hanging or faulting the GPU. */
int cmace_bounded_wait_probe(int32_t *status, int code, double limit_seconds, cmace_stream_t stream);

int cmace_gemm3x_gradr_f32(const float *X, const float *G, const float *Y, const int32_t *sender,
                           const int32_t *receiver, const float *packed, int64_t nedges, int channels, int N,
                           float *out, int32_t *status, cmace_stream_t stream);

/* ---- hidden layers of the radial multilayer perceptron in one kernel (float32) ---------------------
 * basis [E, nb] -> h3 = silu(silu(silu(basis W1) W2) W3) [E, 64], nb in {8, 16, 24, 32}, hidden width 64: the
 * network upstream MACE evaluates with torch (e3nn FullyConnectedNet) and the reference tabulates into its
 * spline (models/InvariantMACE.py:226-240), without its last, linear layer.  The activations stay in shared /
 * tensor memory between the layers.  Weights are packed with cmace_gemm_pack_weights_f32 (nmat = 1):
 * forward packed_wK from Bt = W_K^T [64, in]; backward packed_wKt from Bt = W_K [in, 64].  The normalisation
 * constants (1/sqrt(fan_in), second moment of the activation) are folded into the weights by the caller.
 * saved: cmace_radial_hidden_saved_floats(E) floats written by the forward (activation derivatives, tiled) and
 * read by the backward; NULL in the forward when no backward follows. */
int64_t cmace_radial_hidden_saved_floats(int64_t nedges);
int cmace_radial_hidden_fwd_f32(const float *basis, int nb, const float *packed_w1, const float *packed_w2,
                                const float *packed_w3, int64_t nedges, float *h3, float *saved,
                                int32_t *status, cmace_stream_t stream);
int cmace_radial_hidden_bwd_f32(const float *grad_h3, const float *saved, const float *packed_w3t,
                                const float *packed_w2t, const float *packed_w1t, int nb, int64_t nedges,
                                float *grad_basis, int32_t *status, cmace_stream_t stream);

/* ---- message passing with the last radial layer formed on the fly (float32) --------------------------
 * out[i,lm,c] = sum_e X[sender(e),c] * Y[lm,e] * R[e,l,c] with R = H @ W, H [E,K] (K = 32 or 64) the last hidden
 * activations of the radial perceptron and W [K,4C] its last layer: cmace_imp_fwd_f32 applied to the product
 * without a separate pass that writes and re-reads R [E,4,C] (no counterpart in the reference, which reads R from
 * its spline kernel's output, models/InvariantMACE.py:101-113).  C in {32,64,96,128}.
 * packed_w: cmace_gemm_pack_weights_f32 of Bt [C/32, 128, K] with Bt[q, l*32 + j, :] = W[:, l*C + q*32 + j].
 * sender, receiver: the edge list sorted by receiver (the receiver list itself, not the CSR).
 * R: optional output [E,4,C] for a later backward pass (cmace_imp_bwd_edge_f32), or NULL.
 * out is zero-filled by the call; partial sums are combined with float atomics. */
int cmace_imp_radial_fused_fwd_f32(const float *X, const float *Y, const float *H, const float *packed_w,
                                   const int32_t *sender, const int32_t *receiver, int64_t nnodes,
                                   int64_t nedges, int nchannels, int K, float *out, float *R,
                                   int32_t *status, cmace_stream_t stream);

/* ---- symmetric contraction (correlation 3, invariant output) ------------------------------
 * Replace jit_symmetric_contraction_forward / _backward
 * (jit_wrappers/src/symmetric_contraction_wrapper.cpp:15-205, kernels
 * cuda/src/symmetric_contraction_impl.cu:6-234).  The plan is built once from HOST copies of the
 * reference's sparse U tables (layout of cuda_mace/ops/symmetric_contraction.py:91-187; the values
 * are taken as double so that a float64 caller keeps full precision, a float32 table is simply
 * widened); it symmetrises them into a list of monomial terms kept in device memory.
 * forward: out [N,C] (the reference returns the same data shaped [N,1,C]);
 * backward: gradX[n,i,c] = gout[n,c] * d out[n,c] / d X[n,i,c], recomputed from X (the reference
 * reads a saved [N,16,C] derivative written by its forward).
 * X [N,16,C]; atom_types [N] int32; W3 [nelements,w3,C], W2 [nelements,w2,C], W1 [nelements,w1,C]
 * (slice of the output irrep 0 of the reference's [nlout,Z,w,C] buffers). */
typedef struct cmace_symcon_plan cmace_symcon_plan;
int cmace_symcon_plan_create(int u3_max_nonzero, const int16_t *u3_num_nonzero /*[16,16]*/,
                             const int32_t *u3_indices /*[maxnz,16,16]*/,
                             const double *u3_values /*[maxnz,16,16]*/,
                             const int16_t *u2_num_nonzero /*[16,16]*/,
                             const int16_t *u2_indices /*[16,16]*/,
                             const double *u2_values /*[16,16]*/, int w3_size, int w2_size,
                             int w1_size, cmace_symcon_plan **plan);
void cmace_symcon_plan_destroy(cmace_symcon_plan *plan);
int cmace_symcon_plan_nterms(const cmace_symcon_plan *plan);
int cmace_symcon_plan_nclasses(const cmace_symcon_plan *plan);
/* 1 when the tables were recognised as the canonical l_max = 3 couplings (up to one scale per path) and the
 * build-time generated register kernel is used instead of the table-driven one. */
int cmace_symcon_plan_is_canonical(const cmace_symcon_plan *plan);
int cmace_symcon_fwd_f32(const cmace_symcon_plan *plan, const float *X, const int32_t *atom_types,
                         const float *W3, const float *W2, const float *W1, int nelements,
                         int64_t nnodes, int channels, float *out, cmace_stream_t stream);
int cmace_symcon_fwd_f64(const cmace_symcon_plan *plan, const double *X, const int32_t *atom_types,
                         const double *W3, const double *W2, const double *W1, int nelements,
                         int64_t nnodes, int channels, double *out, cmace_stream_t stream);
int cmace_symcon_bwd_f32(const cmace_symcon_plan *plan, const float *X, const int32_t *atom_types,
                         const float *W3, const float *W2, const float *W1, const float *gout,
                         int nelements, int64_t nnodes, int channels, float *gradX,
                         cmace_stream_t stream);
int cmace_symcon_bwd_f64(const cmace_symcon_plan *plan, const double *X, const int32_t *atom_types,
                         const double *W3, const double *W2, const double *W1, const double *gout,
                         int nelements, int64_t nnodes, int channels, double *gradX,
                         cmace_stream_t stream);

#ifdef __cplusplus
}
#endif
#endif
