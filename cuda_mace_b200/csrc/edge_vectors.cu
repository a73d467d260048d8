// Edge vectors from atom positions, and the position gradient (minus the forces) from the gradient of the edge vectors.
//
//   forward    vec[e] = pos[sender[e]] - pos[receiver[e]] + shift[e]          (float64 arithmetic, stored as T)
//   backward   grad pos[n] = sum_{e: sender[e] = n} g[e]  -  sum_{e: receiver[e] = n} g[e]
//
// The reference leaves both to torch (get_edge_vectors_and_lengths, models/InvariantMACE.py:297-304: index_select,
// subtraction, and autograd's index_add with atomics in the backward).  Here the backward walks the two edge
// groupings the message passing already owns -- the receiver-sorted edge list (row_ptr) and the sender-grouped
// permutation (perm, send_ptr) -- one warp per atom, float64 accumulation in a fixed order: no atomics, bitwise
// reproducible, one launch instead of about ten.
#include "common.cuh"

namespace cmace {

template <typename T>
__global__ void __launch_bounds__(256)
    edge_vectors_fwd_kernel(const double *__restrict__ pos, const int32_t *__restrict__ sender,
                            const int32_t *__restrict__ receiver, const double *__restrict__ shifts, int64_t nedges,
                            T *__restrict__ vec) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;   // one component of one edge
  if (i >= nedges * 3) return;
  const int64_t e = i / 3;
  const int c = (int)(i - e * 3);
  double v = __dsub_rn(pos[(int64_t)sender[e] * 3 + c], pos[(int64_t)receiver[e] * 3 + c]);
  if (shifts) v = __dadd_rn(v, shifts[i]);
  vec[i] = (T)v;
}

template <typename T>
__global__ void __launch_bounds__(256)
    edge_vectors_bwd_kernel(const T *__restrict__ g, const int32_t *__restrict__ row_ptr,
                            const int32_t *__restrict__ perm, const int32_t *__restrict__ send_ptr, int64_t nrecv,
                            int64_t nsend, double *__restrict__ grad_pos) {
  const int64_t n = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;   // one warp per atom
  const int lane = threadIdx.x & 31;
  if (n >= nsend) return;
  double ax = 0.0, ay = 0.0, az = 0.0;
  for (int k = send_ptr[n] + lane; k < send_ptr[n + 1]; k += 32) {
    const int64_t e = perm[k];
    ax += (double)g[e * 3];
    ay += (double)g[e * 3 + 1];
    az += (double)g[e * 3 + 2];
  }
  if (n < nrecv) {
    for (int64_t e = row_ptr[n] + lane; e < row_ptr[n + 1]; e += 32) {
      ax -= (double)g[e * 3];
      ay -= (double)g[e * 3 + 1];
      az -= (double)g[e * 3 + 2];
    }
  }
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) {
    ax += __shfl_xor_sync(0xffffffffu, ax, off);
    ay += __shfl_xor_sync(0xffffffffu, ay, off);
    az += __shfl_xor_sync(0xffffffffu, az, off);
  }
  if (lane == 0) {
    grad_pos[n * 3] = ax;
    grad_pos[n * 3 + 1] = ay;
    grad_pos[n * 3 + 2] = az;
  }
}

template <typename T>
static int edge_vectors_fwd(const double *pos, const int32_t *sender, const int32_t *receiver, const double *shifts,
                            int64_t nedges, T *vec, cmace_stream_t stream) {
  if (nedges < 0) return fail(CMACE_ERR_ARG, "cmace_edge_vectors_fwd: bad size");
  if (nedges == 0) return CMACE_OK;
  if (!pos || !sender || !receiver || !vec) return fail(CMACE_ERR_ARG, "cmace_edge_vectors_fwd: null pointer");
  const int64_t blocks = (nedges * 3 + 255) / 256;
  if (blocks > 0x7fffffffLL) return fail(CMACE_ERR_UNSUPPORTED, "cmace_edge_vectors_fwd: too many edges");
  edge_vectors_fwd_kernel<T><<<(unsigned)blocks, 256, 0, (cudaStream_t)stream>>>(pos, sender, receiver, shifts, nedges, vec);
  return check_launch("cmace_edge_vectors_fwd");
}

template <typename T>
static int edge_vectors_bwd(const T *g, const int32_t *row_ptr, const int32_t *perm, const int32_t *send_ptr,
                            int64_t nrecv, int64_t nsend, double *grad_pos, cmace_stream_t stream) {
  if (nrecv < 0 || nsend < 0 || nrecv > nsend) return fail(CMACE_ERR_ARG, "cmace_edge_vectors_bwd: bad size");
  if (nsend == 0) return CMACE_OK;
  if (!g || !row_ptr || !perm || !send_ptr || !grad_pos)
    return fail(CMACE_ERR_ARG, "cmace_edge_vectors_bwd: null pointer");
  const int64_t blocks = (nsend * 32 + 255) / 256;
  if (blocks > 0x7fffffffLL) return fail(CMACE_ERR_UNSUPPORTED, "cmace_edge_vectors_bwd: too many atoms");
  edge_vectors_bwd_kernel<T><<<(unsigned)blocks, 256, 0, (cudaStream_t)stream>>>(g, row_ptr, perm, send_ptr, nrecv, nsend,
                                                                                grad_pos);
  return check_launch("cmace_edge_vectors_bwd");
}

}  // namespace cmace

using namespace cmace;

extern "C" {
int cmace_edge_vectors_fwd_f32(const double *pos, const int32_t *sender, const int32_t *receiver, const double *shifts,
                               int64_t nedges, float *vec, cmace_stream_t stream) {
  return edge_vectors_fwd<float>(pos, sender, receiver, shifts, nedges, vec, stream);
}
int cmace_edge_vectors_fwd_f64(const double *pos, const int32_t *sender, const int32_t *receiver, const double *shifts,
                               int64_t nedges, double *vec, cmace_stream_t stream) {
  return edge_vectors_fwd<double>(pos, sender, receiver, shifts, nedges, vec, stream);
}
int cmace_edge_vectors_bwd_f32(const float *g, const int32_t *row_ptr, const int32_t *perm, const int32_t *send_ptr,
                               int64_t nrecv, int64_t nsend, double *grad_pos, cmace_stream_t stream) {
  return edge_vectors_bwd<float>(g, row_ptr, perm, send_ptr, nrecv, nsend, grad_pos, stream);
}
int cmace_edge_vectors_bwd_f64(const double *g, const int32_t *row_ptr, const int32_t *perm, const int32_t *send_ptr,
                               int64_t nrecv, int64_t nsend, double *grad_pos, cmace_stream_t stream) {
  return edge_vectors_bwd<double>(g, row_ptr, perm, send_ptr, nrecv, nsend, grad_pos, stream);
}
}
