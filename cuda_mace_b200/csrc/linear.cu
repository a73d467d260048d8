// Per-l channel mixing:  out[n, l^2+m, :] = scale * X[n, l^2+m, :] @ W[z_n, l],  scale = 1/sqrt(K).
//
// One launch covers the four l blocks and, for ElementalLinear, all chemical elements: the rows
// (node, m) of one (element, l) pair form a dense GEMM problem of (#nodes of the element)*(2l+1)
// rows, and every CTA takes one TILE_M x TILE_N output tile of one such problem.  Tiles are
// located on the device from the element group bounds, so there is no host synchronisation and
// no per-element launch.  This file holds the shared-memory tiled FMA kernel used for float64 and
// as the float32 fallback; rows are gathered, so no intermediate re-layout of X is needed.
#include "common.cuh"

namespace cmace {

constexpr int TILE_M = 64, TILE_N = 64, KSTEP = 16, LIN_THREADS = 256;

template <typename T>
__global__ void __launch_bounds__(LIN_THREADS)
    linear_tile_kernel(const T *__restrict__ X, const T *__restrict__ W,
                       const int32_t *__restrict__ node_order, const int32_t *__restrict__ elem_start,
                       int nelements, int64_t nnodes, int K, int Nout, T scale, T *__restrict__ out) {
  __shared__ T As[KSTEP][TILE_M + 4];
  __shared__ T Bs[KSTEP][TILE_N];
  __shared__ int64_t row_of[TILE_M];

  const int l = blockIdx.y;
  const int nl = 2 * l + 1;
  const int n0 = blockIdx.z * TILE_N;

  // which (element, tile) this CTA owns
  int z = 0;
  int64_t tile = blockIdx.x, seg_begin = 0, seg_count = 0;
  for (; z < nelements; z++) {
    seg_begin = elem_start ? elem_start[z] : 0;
    seg_count = elem_start ? (int64_t)elem_start[z + 1] - seg_begin : nnodes;
    const int64_t tiles = (seg_count * nl + TILE_M - 1) / TILE_M;
    if (tile < tiles) break;
    tile -= tiles;
  }
  if (z >= nelements) return;

  const int tid = threadIdx.x;
  if (tid < TILE_M) {
    const int64_t rl = tile * TILE_M + tid;
    int64_t grow = -1;
    if (rl < seg_count * nl) {
      const int64_t slot = seg_begin + rl / nl;
      const int64_t node = node_order ? (int64_t)node_order[slot] : slot;
      grow = node * 16 + l * l + (rl % nl);
    }
    row_of[tid] = grow;
  }
  __syncthreads();

  const T *Wz = W + ((int64_t)(z * 4 + l) * K) * Nout;
  const int ty = tid / 16, tx = tid % 16;
  T acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; i++)
#pragma unroll
    for (int j = 0; j < 4; j++) acc[i][j] = T(0);

  const int arow = tid / 4, ak = (tid % 4) * 4;   // A tile: 64 rows x 16 k, 4 consecutive k per thread
  const int bk = tid / 16, bc = (tid % 16) * 4;   // B tile: 16 k x 64 cols, 4 consecutive cols per thread
  const int64_t agrow = row_of[arow];

  for (int k0 = 0; k0 < K; k0 += KSTEP) {
#pragma unroll
    for (int q = 0; q < 4; q++) {
      const int k = k0 + ak + q;
      As[ak + q][arow] = (agrow >= 0 && k < K) ? X[agrow * K + k] : T(0);
    }
#pragma unroll
    for (int q = 0; q < 4; q++) {
      const int k = k0 + bk, c = n0 + bc + q;
      Bs[bk][bc + q] = (k < K && c < Nout) ? Wz[(int64_t)k * Nout + c] : T(0);
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < KSTEP; kk++) {
      T a[4], b[4];
#pragma unroll
      for (int i = 0; i < 4; i++) a[i] = As[kk][ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; j++) b[j] = Bs[kk][tx * 4 + j];
#pragma unroll
      for (int i = 0; i < 4; i++)
#pragma unroll
        for (int j = 0; j < 4; j++) acc[i][j] = fma(a[i], b[j], acc[i][j]);
    }
    __syncthreads();
  }

#pragma unroll
  for (int i = 0; i < 4; i++) {
    const int64_t grow = row_of[ty * 4 + i];
    if (grow < 0) continue;
#pragma unroll
    for (int j = 0; j < 4; j++) {
      const int c = n0 + tx * 4 + j;
      if (c < Nout) out[grow * Nout + c] = acc[i][j] * scale;
    }
  }
}

template <typename T>
static int linear(const T *X, const T *W, const int32_t *node_order, const int32_t *elem_start,
                  int nelements, int64_t nnodes, int K, int Nout, double scale, T *out,
                  cmace_stream_t stream) {
  if (nnodes < 0 || K < 1 || Nout < 1 || nelements < 1) return fail(CMACE_ERR_ARG, "cmace_linear: bad size");
  if (nnodes == 0) return CMACE_OK;
  if (!X || !W || !out) return fail(CMACE_ERR_ARG, "cmace_linear: null pointer");
  if ((nelements > 1) != (node_order != nullptr) || (node_order != nullptr) != (elem_start != nullptr))
    return fail(CMACE_ERR_ARG, "cmace_linear: node_order and elem_start go together with nelements > 1");
  const int64_t max_tiles = (nnodes * 7 + TILE_M - 1) / TILE_M + nelements;
  if (max_tiles > 0x7fffffffLL) return fail(CMACE_ERR_UNSUPPORTED, "cmace_linear: too many rows");
  dim3 grid((unsigned)max_tiles, 4, (unsigned)((Nout + TILE_N - 1) / TILE_N));
  linear_tile_kernel<T><<<grid, LIN_THREADS, 0, (cudaStream_t)stream>>>(
      X, W, node_order, elem_start, nelements, nnodes, K, Nout, (T)scale, out);
  return check_launch("cmace_linear");
}

}  // namespace cmace

using namespace cmace;

extern "C" {
int cmace_linear_f32(const float *X, const float *W, const int32_t *node_order, const int32_t *elem_start,
                     int nelements, int64_t nnodes, int K, int Nout, double scale, float *out,
                     cmace_stream_t stream) {
  return linear<float>(X, W, node_order, elem_start, nelements, nnodes, K, Nout, scale, out, stream);
}
int cmace_linear_f64(const double *X, const double *W, const int32_t *node_order, const int32_t *elem_start,
                     int nelements, int64_t nnodes, int K, int Nout, double scale, double *out,
                     cmace_stream_t stream) {
  return linear<double>(X, W, node_order, elem_start, nelements, nnodes, K, Nout, scale, out, stream);
}
}
