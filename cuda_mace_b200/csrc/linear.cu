// Per-l channel mixing:  out[n, l^2+m, :] = scale * X[n, l^2+m, :] @ W[z_n, l],  scale = 1/sqrt(K).
//
// One launch covers the four l blocks and, for ElementalLinear, all chemical elements: the rows
// (node, m) of one (element, l) pair form a dense GEMM problem of (#nodes of the element)*(2l+1)
// rows, and every CTA takes one TILE_M x TILE_N output tile of one such problem.  Tiles are
// located on the device from the element group bounds, so there is no host synchronisation and
// no per-element launch.  This file holds the float64 tensor-core (DMMA) kernel and the shared-memory tiled
// FMA kernel that serves odd sizes and float32 callers that do not use the tcgen05 path; rows are gathered,
// so no intermediate re-layout of X is needed.  The same two kernels with the identity row map are the plain float64
// product cmace_gemm_f64 (radial multilayer perceptron and node products of the float64 model).
#include "common.cuh"

namespace cmace {

constexpr int TILE_M = 64, TILE_N = 64, KSTEP = 16, LIN_THREADS = 256;

// PLAIN: one dense product out[M, Nout] = scale * X[M, K] @ W[K, Nout] (nnodes = M rows, no l blocks, no elements).
template <typename T, bool PLAIN>
__global__ void __launch_bounds__(LIN_THREADS)
    linear_tile_kernel(const T *__restrict__ X, const T *__restrict__ W,
                       const int32_t *__restrict__ node_order, const int32_t *__restrict__ elem_start,
                       int nelements, int64_t nnodes, int K, int Nout, T scale, T *__restrict__ out) {
  __shared__ T As[KSTEP][TILE_M + 4];
  __shared__ T Bs[KSTEP][TILE_N];
  __shared__ int64_t row_of[TILE_M];

  const int l = PLAIN ? 0 : blockIdx.y;
  const int nl = 2 * l + 1;
  const int n0 = blockIdx.z * TILE_N;

  // which (element, tile) this CTA owns
  int z = 0;
  int64_t tile = blockIdx.x, seg_begin = 0, seg_count = 0;
  if (!PLAIN) {
    for (; z < nelements; z++) {
      seg_begin = elem_start ? elem_start[z] : 0;
      seg_count = elem_start ? (int64_t)elem_start[z + 1] - seg_begin : nnodes;
      const int64_t tiles = (seg_count * nl + TILE_M - 1) / TILE_M;
      if (tile < tiles) break;
      tile -= tiles;
    }
    if (z >= nelements) return;
  }

  const int tid = threadIdx.x;
  if (tid < TILE_M) {
    const int64_t rl = tile * TILE_M + tid;
    int64_t grow = -1;
    if (PLAIN) {
      if (rl < nnodes) grow = rl;
    } else if (rl < seg_count * nl) {
      const int64_t slot = seg_begin + rl / nl;
      const int64_t node = node_order ? (int64_t)node_order[slot] : slot;
      grow = node * 16 + l * l + (rl % nl);
    }
    row_of[tid] = grow;
  }
  __syncthreads();

  const T *Wz = PLAIN ? W : W + ((int64_t)(z * 4 + l) * K) * Nout;
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

// ---- float64 on the tensor cores (DMMA) -----------------------------------------------------------
// Same tile bookkeeping, 128 x 128 output tile per CTA, 16 warps of 32 x 32 (4 x 4 mma.sync m8n8k4 f64 tiles,
// 32 accumulator doubles per thread).  A rows (gathered) and W rows arrive through a 3-stage cp.async ring of
// 16-wide K slices; the row strides (20 and 132 doubles) make the fragment loads of both operands conflict-free:
// a fragment load touches 8 rows x 4 consecutive doubles (A) or 4 rows x 8 columns (B), and 2 * stride mod 32 = 8
// spreads the rows of each half-warp over all 32 banks.  Fragment layout of mma.m8n8k4.f64: A[lane/4][lane%4],
// B[lane%4][lane/4], C[lane/4][2*(lane%4) + {0,1}].
// The operator is bound by the FP64 tensor rate at K = Nout = 128 (16 flop/B against a machine balance of ~6).
// TN: columns of the output tile, 128 or 64 (the radial perceptron's hidden layers are 64 wide: a 128-column tile would
// spend half of its instructions on padding); the 16 warps form a 4 x 4 grid of 32 x TN/4 pieces in both cases.
constexpr int DM_TILE = 128, DM_K = 16, DM_THREADS = 512, DM_STAGES = 3;
constexpr int DM_AS = DM_K + 4;                                // row stride of the A slice in doubles
template <int TN>
struct DmGeom {
  static constexpr int BS = TN + 4;                            // row stride of the B slice in doubles
  static constexpr int STAGE_DOUBLES = DM_TILE * DM_AS + DM_K * BS;
  static constexpr int SMEM_BYTES = DM_STAGES * STAGE_DOUBLES * 8;
  static constexpr int B_COPIES = DM_K * TN / 2 / DM_THREADS;  // 16-byte chunks of a B slice per thread
  static constexpr int NJ = TN / 32;                           // 8-column MMA tiles per warp
};

__device__ __forceinline__ void cp_async_16_zfill(void *dst, const void *src, bool valid) {
  const uint32_t d = (uint32_t)__cvta_generic_to_shared(dst);
  const int n = valid ? 16 : 0;   // 0 source bytes: the 16 destination bytes are zero-filled
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(d), "l"(src), "r"(n) : "memory");
}

template <bool PLAIN, int TN>
__global__ void __launch_bounds__(DM_THREADS, 1)
    linear_dmma_kernel(const double *__restrict__ X, const double *__restrict__ W,
                       const int32_t *__restrict__ node_order, const int32_t *__restrict__ elem_start,
                       int nelements, int64_t nnodes, int K, int Nout, double scale, double *__restrict__ out) {
  extern __shared__ __align__(16) double dm_smem[];
  __shared__ int64_t row_of[DM_TILE];

  const int l = PLAIN ? 0 : blockIdx.y;
  const int nl = 2 * l + 1;
  using Geo = DmGeom<TN>;
  constexpr int DM_BS = Geo::BS, DM_STAGE_DOUBLES = Geo::STAGE_DOUBLES;
  const int n0 = blockIdx.z * TN;

  int z = 0;
  int64_t tile = blockIdx.x, seg_begin = 0, seg_count = 0;
  if (!PLAIN) {
    for (; z < nelements; z++) {
      seg_begin = elem_start ? elem_start[z] : 0;
      seg_count = elem_start ? (int64_t)elem_start[z + 1] - seg_begin : nnodes;
      const int64_t tiles = (seg_count * nl + DM_TILE - 1) / DM_TILE;
      if (tile < tiles) break;
      tile -= tiles;
    }
    if (z >= nelements) return;
  }

  const int tid = threadIdx.x;
  if (tid < DM_TILE) {
    const int64_t rl = tile * DM_TILE + tid;
    int64_t grow = -1;
    if (PLAIN) {
      if (rl < nnodes) grow = rl;
    } else if (rl < seg_count * nl) {
      const int64_t slot = seg_begin + rl / nl;
      const int64_t node = node_order ? (int64_t)node_order[slot] : slot;
      grow = node * 16 + l * l + (rl % nl);
    }
    row_of[tid] = grow;
  }
  __syncthreads();

  const double *Wz = PLAIN ? W : W + ((int64_t)(z * 4 + l) * K) * Nout;
  // copy assignments: 1024 16-byte chunks per operand and K slice, two per thread
  int64_t a_src[2];
  int a_dst[2], a_k[2], b_dst[Geo::B_COPIES], b_k[Geo::B_COPIES], b_c[Geo::B_COPIES];
#pragma unroll
  for (int i = 0; i < 2; i++) {
    const int c = tid + DM_THREADS * i;
    const int ar = c >> 3, ach = c & 7;              // A: 128 rows x 8 chunks
    a_src[i] = row_of[ar] >= 0 ? row_of[ar] * K + ach * 2 : -1;
    a_k[i] = ach * 2;
    a_dst[i] = ar * DM_AS + ach * 2;
  }
#pragma unroll
  for (int i = 0; i < Geo::B_COPIES; i++) {
    const int c = tid + DM_THREADS * i;
    const int bk = c / (TN / 2), bch = c % (TN / 2);   // B: 16 K rows x TN/2 chunks
    b_k[i] = bk;
    b_c[i] = n0 + bch * 2;
    b_dst[i] = DM_TILE * DM_AS + bk * DM_BS + bch * 2;
  }
  auto load_slice = [&](int kt) {
    double *st = dm_smem + (kt % DM_STAGES) * DM_STAGE_DOUBLES;
    const int k0 = kt * DM_K;
#pragma unroll
    for (int i = 0; i < 2; i++) {
      const bool av = a_src[i] >= 0 && k0 + a_k[i] < K;
      cp_async_16_zfill(st + a_dst[i], av ? X + a_src[i] + k0 : X, av);
    }
#pragma unroll
    for (int i = 0; i < Geo::B_COPIES; i++) {
      const bool bv = k0 + b_k[i] < K && b_c[i] < Nout;
      cp_async_16_zfill(st + b_dst[i], bv ? Wz + (int64_t)(k0 + b_k[i]) * Nout + b_c[i] : W, bv);
    }
  };

  const int warp = tid >> 5, lane = tid & 31;
  constexpr int NJ = Geo::NJ;
  const int wm = (warp >> 2) * 32, wn = (warp & 3) * (TN / 4);
  const int fr = lane >> 2, fk = lane & 3;
  double acc[4][NJ][2];
#pragma unroll
  for (int i = 0; i < 4; i++)
#pragma unroll
    for (int j = 0; j < NJ; j++) acc[i][j][0] = acc[i][j][1] = 0.0;

  const int nk = (K + DM_K - 1) / DM_K;
#pragma unroll
  for (int s = 0; s < DM_STAGES - 1; s++) {
    if (s < nk) load_slice(s);
    asm volatile("cp.async.commit_group;" ::: "memory");
  }
  for (int kt = 0; kt < nk; kt++) {
    asm volatile("cp.async.wait_group %0;" ::"n"(DM_STAGES - 2) : "memory");
    __syncthreads();   // slice kt has landed for every thread, and everybody is done with slice kt - 1
    if (kt + DM_STAGES - 1 < nk) load_slice(kt + DM_STAGES - 1);
    asm volatile("cp.async.commit_group;" ::: "memory");
    const double *As = dm_smem + (kt % DM_STAGES) * DM_STAGE_DOUBLES;
    const double *Bs = As + DM_TILE * DM_AS;
#pragma unroll
    for (int kk = 0; kk < DM_K; kk += 4) {
      double a[4], b[NJ];
#pragma unroll
      for (int i = 0; i < 4; i++) a[i] = As[(wm + i * 8 + fr) * DM_AS + kk + fk];
#pragma unroll
      for (int j = 0; j < NJ; j++) b[j] = Bs[(kk + fk) * DM_BS + wn + j * 8 + fr];
#pragma unroll
      for (int i = 0; i < 4; i++)
#pragma unroll
        for (int j = 0; j < NJ; j++)
          asm volatile("mma.sync.aligned.m8n8k4.row.col.f64.f64.f64.f64 {%0, %1}, {%2}, {%3}, {%0, %1};"
                       : "+d"(acc[i][j][0]), "+d"(acc[i][j][1])
                       : "d"(a[i]), "d"(b[j]));
    }
  }
  asm volatile("cp.async.wait_group 0;" ::: "memory");

#pragma unroll
  for (int i = 0; i < 4; i++) {
    const int64_t grow = row_of[wm + i * 8 + fr];
    if (grow < 0) continue;
#pragma unroll
    for (int j = 0; j < NJ; j++) {
      const int c = n0 + wn + j * 8 + 2 * fk;
      if (c < Nout)   // Nout is even: both columns or none
        *reinterpret_cast<double2 *>(out + grow * Nout + c) = make_double2(acc[i][j][0] * scale, acc[i][j][1] * scale);
    }
  }
}

static int linear_dmma(const double *X, const double *W, const int32_t *node_order, const int32_t *elem_start,
                       int nelements, int64_t nnodes, int K, int Nout, double scale, double *out,
                       cmace_stream_t stream) {
  static bool attr_set = false;
  if (!attr_set) {
    if (cudaFuncSetAttribute(linear_dmma_kernel<false, 128>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             DmGeom<128>::SMEM_BYTES) != cudaSuccess)
      return fail(CMACE_ERR_CUDA, "cmace_linear_f64: cannot reserve shared memory");
    attr_set = true;
  }
  const int64_t max_tiles = (nnodes * 7 + DM_TILE - 1) / DM_TILE + nelements;
  if (max_tiles > 0x7fffffffLL) return fail(CMACE_ERR_UNSUPPORTED, "cmace_linear: too many rows");
  dim3 grid((unsigned)max_tiles, 4, (unsigned)((Nout + DM_TILE - 1) / DM_TILE));
  linear_dmma_kernel<false, 128><<<grid, DM_THREADS, DmGeom<128>::SMEM_BYTES, (cudaStream_t)stream>>>(
      X, W, node_order, elem_start, nelements, nnodes, K, Nout, scale, out);
  return check_launch("cmace_linear_f64");
}

// out[M, N] = scale * A[M, K] @ B[K, N], float64: the DMMA tile loop with the identity row map; the FMA tile kernel
// when the 16-byte copies of the tensor-core path cannot be aligned (odd K or N).
static int gemm_f64(const double *A, const double *B, int64_t M, int K, int N, double scale, double *out,
                    cmace_stream_t stream) {
  if (M < 0 || K < 1 || N < 1) return fail(CMACE_ERR_ARG, "cmace_gemm_f64: bad size");
  if (M == 0) return CMACE_OK;
  if (!A || !B || !out) return fail(CMACE_ERR_ARG, "cmace_gemm_f64: null pointer");
  if (K % 2 == 0 && N % 2 == 0 && aligned16(A) && aligned16(B) && aligned16(out)) {
    static bool attr_set = false;
    if (!attr_set) {
      if (cudaFuncSetAttribute(linear_dmma_kernel<true, 128>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                               DmGeom<128>::SMEM_BYTES) != cudaSuccess ||
          cudaFuncSetAttribute(linear_dmma_kernel<true, 64>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                               DmGeom<64>::SMEM_BYTES) != cudaSuccess)
        return fail(CMACE_ERR_CUDA, "cmace_gemm_f64: cannot reserve shared memory");
      attr_set = true;
    }
    const int64_t tiles = (M + DM_TILE - 1) / DM_TILE;
    if (tiles > 0x7fffffffLL) return fail(CMACE_ERR_UNSUPPORTED, "cmace_gemm_f64: too many rows");
    if (N <= 64) {   // narrow output: 64-column tiles
      dim3 grid((unsigned)tiles, 1, 1);
      linear_dmma_kernel<true, 64><<<grid, DM_THREADS, DmGeom<64>::SMEM_BYTES, (cudaStream_t)stream>>>(
          A, B, nullptr, nullptr, 1, M, K, N, scale, out);
    } else {
      dim3 grid((unsigned)tiles, 1, (unsigned)((N + DM_TILE - 1) / DM_TILE));
      linear_dmma_kernel<true, 128><<<grid, DM_THREADS, DmGeom<128>::SMEM_BYTES, (cudaStream_t)stream>>>(
          A, B, nullptr, nullptr, 1, M, K, N, scale, out);
    }
    return check_launch("cmace_gemm_f64");
  }
  const int64_t tiles = (M + TILE_M - 1) / TILE_M;
  if (tiles > 0x7fffffffLL) return fail(CMACE_ERR_UNSUPPORTED, "cmace_gemm_f64: too many rows");
  dim3 grid((unsigned)tiles, 1, (unsigned)((N + TILE_N - 1) / TILE_N));
  linear_tile_kernel<double, true><<<grid, LIN_THREADS, 0, (cudaStream_t)stream>>>(A, B, nullptr, nullptr, 1, M, K, N,
                                                                                   scale, out);
  return check_launch("cmace_gemm_f64");
}

template <typename T>
static int linear(const T *X, const T *W, const int32_t *node_order, const int32_t *elem_start,
                  int nelements, int64_t nnodes, int K, int Nout, double scale, T *out,
                  cmace_stream_t stream) {
  if (nnodes < 0 || K < 1 || Nout < 1 || nelements < 1) return fail(CMACE_ERR_ARG, "cmace_linear: bad size");
  if (nnodes == 0) return CMACE_OK;
  if (!X || !W || !out) return fail(CMACE_ERR_ARG, "cmace_linear: null pointer");
  // (node_order may be NULL for nelements > 1: the nodes are then stored grouped by element)
  if ((nelements > 1) != (elem_start != nullptr) || (node_order != nullptr && elem_start == nullptr))
    return fail(CMACE_ERR_ARG, "cmace_linear: elem_start goes with nelements > 1, node_order only with elem_start");
  if constexpr (sizeof(T) == 8) {
    // tensor-core path whenever its 16-byte copies are aligned: even K and Nout, 16-byte aligned bases
    if (K % 2 == 0 && Nout % 2 == 0 && aligned16(X) && aligned16(W) && aligned16(out))
      return linear_dmma(X, W, node_order, elem_start, nelements, nnodes, K, Nout, scale, out, stream);
  }
  const int64_t max_tiles = (nnodes * 7 + TILE_M - 1) / TILE_M + nelements;
  if (max_tiles > 0x7fffffffLL) return fail(CMACE_ERR_UNSUPPORTED, "cmace_linear: too many rows");
  dim3 grid((unsigned)max_tiles, 4, (unsigned)((Nout + TILE_N - 1) / TILE_N));
  linear_tile_kernel<T, false><<<grid, LIN_THREADS, 0, (cudaStream_t)stream>>>(
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
int cmace_gemm_f64(const double *A, const double *B, int64_t M, int K, int N, double scale, double *out,
                   cmace_stream_t stream) {
  return gemm_f64(A, B, M, K, N, scale, out, stream);
}
}
