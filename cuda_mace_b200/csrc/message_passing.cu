// Invariant message passing: receiver-sorted gather * product * segmented sum, and its backward.
//
//   out[i, lm, c] = sum_{e in row(i)} X[sender[e], c] * Y[lm, e] * R[e, l(lm), c]
//
// Work split: one warp owns one receiver row and a chunk of 32*VEC channels (lane <-> VEC
// consecutive channels, 16-byte loads).  The warp walks the receiver's contiguous edge range,
// keeps all 16 (l,m) accumulators of its channels in registers and writes each output once:
// no atomics, a fixed summation order, and R (the dominant HBM stream, E*4*C scalars) is read
// exactly once with full 128-byte lines.  Y [16, E] is component-major, so the 16 values of an
// edge are fetched by 16 lanes (two edges per 32-lane load) and broadcast with shuffles.
//
// Backward, edge pass (same mapping, G[i] = d loss / d out[i] held in registers):
//   u[l, c]      = sum_{m in l} Y[m, e] * G[i, m, c]
//   gradR[e,l,c] = X[s, c] * u[l, c]
//   T[e, c]      = sum_l u[l, c] * R[e, l, c]                (sender contribution of edge e)
//   gradY[m, e]  = sum_c G[i, m, c] * R[e, l, c] * X[s, c]   (16-value warp transpose-reduce)
// Backward, node pass: gradX[s, c] = sum over the edges sent by s of T[e, c], walking the
// sender-grouped edge permutation; again one warp per node, no atomics.
#include "common.cuh"

namespace cmace {

constexpr int kWarpsPerBlock = 4;

template <typename T, int VEC>
__global__ void __launch_bounds__(kWarpsPerBlock * 32)
    imp_fwd_kernel(const T *__restrict__ X, const T *__restrict__ Y, const T *__restrict__ R,
                   const int32_t *__restrict__ sender, const int32_t *__restrict__ row_ptr,
                   int64_t nnodes, int64_t nedges, int C, T *__restrict__ out) {
  const int lane = threadIdx.x & 31;
  const int64_t node = (int64_t)blockIdx.x * kWarpsPerBlock + (threadIdx.x >> 5);
  if (node >= nnodes) return;
  const int c0 = blockIdx.y * (32 * VEC) + lane * VEC;
  const int64_t e0 = row_ptr[node], e1 = row_ptr[node + 1];

  T acc[16][VEC];
#pragma unroll
  for (int m = 0; m < 16; m++)
#pragma unroll
    for (int v = 0; v < VEC; v++) acc[m][v] = T(0);

  const int ylm = lane & 15, yedge = lane >> 4;
  for (int64_t e = e0; e < e1; e += 2) {
    // second edge of the pair: clamp to a valid edge, its harmonics are zeroed below
    const int64_t eb = (e + 1 < e1) ? e + 1 : e;
    const int64_t ey = yedge ? eb : e;
    T yv = __ldg(Y + (int64_t)ylm * nedges + ey);
    if (yedge && e + 1 >= e1) yv = T(0);
    const int64_t sa = sender[e], sb = sender[eb];
    T xa[VEC], xb[VEC], ra[4][VEC], rb[4][VEC];
    load_vec<T, VEC>(xa, X + sa * C + c0);
    load_vec<T, VEC>(xb, X + sb * C + c0);
#pragma unroll
    for (int l = 0; l < 4; l++) {
      load_vec_stream<T, VEC>(ra[l], R + (e * 4 + l) * C + c0);
      load_vec_stream<T, VEC>(rb[l], R + (eb * 4 + l) * C + c0);
    }
#pragma unroll
    for (int l = 0; l < 4; l++)
#pragma unroll
      for (int v = 0; v < VEC; v++) {
        ra[l][v] *= xa[v];
        rb[l][v] *= xb[v];
      }
#pragma unroll
    for (int m = 0; m < 16; m++) {
      const T ya = __shfl_sync(0xffffffffu, yv, m);
      const T yb = __shfl_sync(0xffffffffu, yv, 16 + m);
#pragma unroll
      for (int v = 0; v < VEC; v++) {
        acc[m][v] = fma(ya, ra[l_of_lm(m)][v], acc[m][v]);
        acc[m][v] = fma(yb, rb[l_of_lm(m)][v], acc[m][v]);
      }
    }
  }
  T *o = out + node * 16 * C + c0;
#pragma unroll
  for (int m = 0; m < 16; m++) store_vec<T, VEC>(o + m * C, acc[m]);
}

// Sum of p[m] over the 32 lanes for all 16 m at once: after the call every lane holds the
// total of component (lane >> 1).  16 shuffles instead of 16 * 5.
template <typename T>
__device__ __forceinline__ T warp_reduce16(T (&p)[16], int lane) {
  T q8[8], q4[4], q2[2];
  {
    const bool up = lane & 16;
#pragma unroll
    for (int i = 0; i < 8; i++) {
      const T send = up ? p[i] : p[i + 8];
      const T keep = up ? p[i + 8] : p[i];
      q8[i] = keep + __shfl_xor_sync(0xffffffffu, send, 16);
    }
  }
  {
    const bool up = lane & 8;
#pragma unroll
    for (int i = 0; i < 4; i++) {
      const T send = up ? q8[i] : q8[i + 4];
      const T keep = up ? q8[i + 4] : q8[i];
      q4[i] = keep + __shfl_xor_sync(0xffffffffu, send, 8);
    }
  }
  {
    const bool up = lane & 4;
#pragma unroll
    for (int i = 0; i < 2; i++) {
      const T send = up ? q4[i] : q4[i + 2];
      const T keep = up ? q4[i + 2] : q4[i];
      q2[i] = keep + __shfl_xor_sync(0xffffffffu, send, 4);
    }
  }
  const bool up = lane & 2;
  const T send = up ? q2[0] : q2[1];
  const T keep = up ? q2[1] : q2[0];
  T r = keep + __shfl_xor_sync(0xffffffffu, send, 2);
  r += __shfl_xor_sync(0xffffffffu, r, 1);
  return r;
}

template <typename T, int VEC>
__global__ void __launch_bounds__(kWarpsPerBlock * 32)
    imp_bwd_edge_kernel(const T *__restrict__ X, const T *__restrict__ Y, const T *__restrict__ R,
                        const T *__restrict__ G, const int32_t *__restrict__ sender,
                        const int32_t *__restrict__ row_ptr, int64_t nnodes, int64_t nedges, int C,
                        T *__restrict__ gradR, T *__restrict__ gradY_out, T *__restrict__ Tout) {
  const int lane = threadIdx.x & 31;
  const int64_t node = (int64_t)blockIdx.x * kWarpsPerBlock + (threadIdx.x >> 5);
  if (node >= nnodes) return;
  const int c0 = blockIdx.y * (32 * VEC) + lane * VEC;
  const int64_t e0 = row_ptr[node], e1 = row_ptr[node + 1];
  if (e0 >= e1) return;
  // with several channel chunks each chunk writes its own [16, E] partial of gradY
  T *gy = gradY_out + (int64_t)blockIdx.y * 16 * nedges;

  T g[16][VEC];
#pragma unroll
  for (int m = 0; m < 16; m++) load_vec<T, VEC>(g[m], G + (node * 16 + m) * C + c0);

  const int ylm = lane & 15, yedge = lane >> 4;
  for (int64_t e = e0; e < e1; e += 2) {
    const int64_t eb = (e + 1 < e1) ? e + 1 : e;
    const T yv = __ldg(Y + (int64_t)ylm * nedges + (yedge ? eb : e));
    // loads of both edges of the pair are issued before either is consumed
    const int64_t s2[2] = {sender[e], sender[eb]};
    T xx[2][VEC], rr[2][4][VEC];
#pragma unroll
    for (int h = 0; h < 2; h++) {
      load_vec<T, VEC>(xx[h], X + s2[h] * C + c0);
#pragma unroll
      for (int l = 0; l < 4; l++) load_vec_stream<T, VEC>(rr[h][l], R + ((h ? eb : e) * 4 + l) * C + c0);
    }
#pragma unroll
    for (int h = 0; h < 2; h++) {
      const int64_t ee = h ? eb : e;
      if (h && e + 1 >= e1) break;  // warp-uniform
      T(&x)[VEC] = xx[h];
      T(&r)[4][VEC] = rr[h];
      T u[4][VEC], p[16];
#pragma unroll
      for (int l = 0; l < 4; l++)
#pragma unroll
        for (int v = 0; v < VEC; v++) u[l][v] = T(0);
#pragma unroll
      for (int m = 0; m < 16; m++) {
        const T y = __shfl_sync(0xffffffffu, yv, 16 * h + m);
        T pm = T(0);
#pragma unroll
        for (int v = 0; v < VEC; v++) {
          u[l_of_lm(m)][v] = fma(y, g[m][v], u[l_of_lm(m)][v]);
          pm = fma(g[m][v], r[l_of_lm(m)][v] * x[v], pm);
        }
        p[m] = pm;
      }
      T t[VEC];
#pragma unroll
      for (int v = 0; v < VEC; v++) t[v] = T(0);
#pragma unroll
      for (int l = 0; l < 4; l++) {
        T gr[VEC];
#pragma unroll
        for (int v = 0; v < VEC; v++) {
          t[v] = fma(u[l][v], r[l][v], t[v]);
          gr[v] = x[v] * u[l][v];
        }
        store_vec_stream<T, VEC>(gradR + (ee * 4 + l) * C + c0, gr);
      }
      if (Tout != nullptr) store_vec<T, VEC>(Tout + ee * C + c0, t);
      const T tot = warp_reduce16(p, lane);
      if ((lane & 1) == 0) gy[(int64_t)(lane >> 1) * nedges + ee] = tot;
    }
  }
}

// gradY[m, e] = sum over chunks of partial[chunk, m, e]
template <typename T>
__global__ void sum_partials_kernel(const T *__restrict__ partial, int nchunks, int64_t n,
                                    T *__restrict__ out) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  T s = T(0);
  for (int k = 0; k < nchunks; k++) s += partial[(int64_t)k * n + i];
  out[i] = s;
}

template <typename T, int VEC>
__global__ void __launch_bounds__(kWarpsPerBlock * 32)
    imp_bwd_node_kernel(const T *__restrict__ Tin, const int32_t *__restrict__ perm,
                        const int32_t *__restrict__ send_ptr, int64_t nnodes, int C,
                        T *__restrict__ gradX) {
  const int lane = threadIdx.x & 31;
  const int64_t node = (int64_t)blockIdx.x * kWarpsPerBlock + (threadIdx.x >> 5);
  if (node >= nnodes) return;
  const int c0 = blockIdx.y * (32 * VEC) + lane * VEC;
  const int64_t k0 = send_ptr[node], k1 = send_ptr[node + 1];
  T acc[VEC], acc2[VEC];
#pragma unroll
  for (int v = 0; v < VEC; v++) acc[v] = acc2[v] = T(0);
  int64_t k = k0;
  for (; k + 1 < k1; k += 2) {
    const int64_t ea = perm[k], eb = perm[k + 1];
    T a[VEC], b[VEC];
    load_vec<T, VEC>(a, Tin + ea * C + c0);
    load_vec<T, VEC>(b, Tin + eb * C + c0);
#pragma unroll
    for (int v = 0; v < VEC; v++) {
      acc[v] += a[v];
      acc2[v] += b[v];
    }
  }
  if (k < k1) {
    T a[VEC];
    load_vec<T, VEC>(a, Tin + (int64_t)perm[k] * C + c0);
#pragma unroll
    for (int v = 0; v < VEC; v++) acc[v] += a[v];
  }
#pragma unroll
  for (int v = 0; v < VEC; v++) acc[v] += acc2[v];
  store_vec<T, VEC>(gradX + node * C + c0, acc);
}

// ------------------------------------------------------------------------------------------
// host side
// ------------------------------------------------------------------------------------------
template <typename T>
static int check_common(const void *a, const void *b, const void *c, int64_t nnodes, int64_t nedges,
                        int C, const char *what) {
  if (nnodes < 0 || nedges < 0) return fail(CMACE_ERR_ARG, "%s: negative size", what);
  if (C <= 0 || C % 32 != 0)
    return fail(CMACE_ERR_UNSUPPORTED, "%s: channels must be a positive multiple of 32, got %d", what, C);
  if (nnodes > 0x7fffffffLL / kWarpsPerBlock * kWarpsPerBlock)
    return fail(CMACE_ERR_UNSUPPORTED, "%s: too many nodes", what);
  if (!aligned16(a) || !aligned16(b) || !aligned16(c))
    return fail(CMACE_ERR_ARG, "%s: pointers must be 16-byte aligned", what);
  return CMACE_OK;
}

template <typename T, int VEC>
static void launch_fwd(const T *X, const T *Y, const T *R, const int32_t *sender,
                       const int32_t *row_ptr, int64_t nnodes, int64_t nedges, int C, T *out,
                       cudaStream_t st) {
  dim3 grid((unsigned)((nnodes + kWarpsPerBlock - 1) / kWarpsPerBlock), C / (32 * VEC));
  imp_fwd_kernel<T, VEC><<<grid, kWarpsPerBlock * 32, 0, st>>>(X, Y, R, sender, row_ptr, nnodes,
                                                                nedges, C, out);
}

template <typename T>
static int imp_fwd(const T *X, const T *Y, const T *R, const int32_t *sender, const int32_t *row_ptr,
                   int64_t nnodes, int64_t nedges, int C, T *out, cmace_stream_t stream) {
  int rc = check_common<T>(X, R, out, nnodes, nedges, C, "cmace_imp_fwd");
  if (rc) return rc;
  if (nnodes == 0) return CMACE_OK;
  if (!out || !row_ptr || (nedges > 0 && (!X || !R || !Y || !sender)))
    return fail(CMACE_ERR_ARG, "cmace_imp_fwd: null pointer");
  cudaStream_t st = (cudaStream_t)stream;
  switch (pick_vec<T>(C)) {
    case 4:
      if constexpr (sizeof(T) == 4) launch_fwd<T, 4>(X, Y, R, sender, row_ptr, nnodes, nedges, C, out, st);
      break;
    case 2: launch_fwd<T, 2>(X, Y, R, sender, row_ptr, nnodes, nedges, C, out, st); break;
    default: launch_fwd<T, 1>(X, Y, R, sender, row_ptr, nnodes, nedges, C, out, st); break;
  }
  return check_launch("cmace_imp_fwd");
}

template <typename T, int VEC>
static void launch_bwd_edge(const T *X, const T *Y, const T *R, const T *G, const int32_t *sender,
                            const int32_t *row_ptr, int64_t nnodes, int64_t nedges, int C, T *gradR,
                            T *gy, T *Tout, cudaStream_t st) {
  dim3 grid((unsigned)((nnodes + kWarpsPerBlock - 1) / kWarpsPerBlock), C / (32 * VEC));
  imp_bwd_edge_kernel<T, VEC><<<grid, kWarpsPerBlock * 32, 0, st>>>(X, Y, R, G, sender, row_ptr,
                                                                     nnodes, nedges, C, gradR, gy, Tout);
}

template <typename T>
static int imp_bwd_edge(const T *X, const T *Y, const T *R, const T *G, const int32_t *sender,
                        const int32_t *row_ptr, int64_t nnodes, int64_t nedges, int C, T *gradR,
                        T *gradY, T *Tout, T *partial, cmace_stream_t stream) {
  int rc = check_common<T>(X, R, G, nnodes, nedges, C, "cmace_imp_bwd_edge");
  if (rc) return rc;
  if (nnodes == 0 || nedges == 0) return CMACE_OK;
  if (!X || !Y || !R || !G || !sender || !row_ptr || !gradR || !gradY)
    return fail(CMACE_ERR_ARG, "cmace_imp_bwd_edge: null pointer");
  if (!aligned16(gradR) || (Tout && !aligned16(Tout)))
    return fail(CMACE_ERR_ARG, "cmace_imp_bwd_edge: outputs must be 16-byte aligned");
  const int vec = pick_vec<T>(C);
  const int nchunks = C / (32 * vec);
  if (nchunks > 1 && !partial)
    return fail(CMACE_ERR_ARG, "cmace_imp_bwd_edge: gradY_partial scratch required for %d chunks", nchunks);
  T *gy = nchunks > 1 ? partial : gradY;
  cudaStream_t st = (cudaStream_t)stream;
  switch (vec) {
    case 4:
      if constexpr (sizeof(T) == 4)
        launch_bwd_edge<T, 4>(X, Y, R, G, sender, row_ptr, nnodes, nedges, C, gradR, gy, Tout, st);
      break;
    case 2: launch_bwd_edge<T, 2>(X, Y, R, G, sender, row_ptr, nnodes, nedges, C, gradR, gy, Tout, st); break;
    default: launch_bwd_edge<T, 1>(X, Y, R, G, sender, row_ptr, nnodes, nedges, C, gradR, gy, Tout, st); break;
  }
  rc = check_launch("cmace_imp_bwd_edge");
  if (rc) return rc;
  if (nchunks > 1) {
    const int64_t n = 16 * nedges;
    sum_partials_kernel<T><<<(unsigned)((n + 255) / 256), 256, 0, st>>>(partial, nchunks, n, gradY);
    rc = check_launch("cmace_imp_bwd_edge(sum)");
  }
  return rc;
}

template <typename T, int VEC>
static void launch_bwd_node(const T *Tin, const int32_t *perm, const int32_t *send_ptr, int64_t nnodes,
                            int C, T *gradX, cudaStream_t st) {
  dim3 grid((unsigned)((nnodes + kWarpsPerBlock - 1) / kWarpsPerBlock), C / (32 * VEC));
  imp_bwd_node_kernel<T, VEC><<<grid, kWarpsPerBlock * 32, 0, st>>>(Tin, perm, send_ptr, nnodes, C, gradX);
}

template <typename T>
static int imp_bwd_node(const T *Tin, const int32_t *perm, const int32_t *send_ptr, int64_t nnodes,
                        int C, T *gradX, cmace_stream_t stream) {
  int rc = check_common<T>(Tin, gradX, gradX, nnodes, 0, C, "cmace_imp_bwd_node");
  if (rc) return rc;
  if (nnodes == 0) return CMACE_OK;
  if (!send_ptr || !gradX) return fail(CMACE_ERR_ARG, "cmace_imp_bwd_node: null pointer");
  cudaStream_t st = (cudaStream_t)stream;
  switch (pick_vec<T>(C)) {
    case 4:
      if constexpr (sizeof(T) == 4) launch_bwd_node<T, 4>(Tin, perm, send_ptr, nnodes, C, gradX, st);
      break;
    case 2: launch_bwd_node<T, 2>(Tin, perm, send_ptr, nnodes, C, gradX, st); break;
    default: launch_bwd_node<T, 1>(Tin, perm, send_ptr, nnodes, C, gradX, st); break;
  }
  return check_launch("cmace_imp_bwd_node");
}

// ---- variant without caller scratch -------------------------------------------------------------
// Some callers cannot hand over scratch memory because they cannot allocate on the device at the point
// of the call: a plugin running inside another framework's memory pool that is already sized, or a
// host thread that must not call into an allocator while the device is busy.  For those, the float64
// edge backward keeps its per-chunk gradY partials in a fixed array in the library image.
constexpr int64_t kStaticScratchElems = 2 * 1024 * 1024;  // doubles: 16 MiB, e.g. 65 536 edges at C = 128
static __device__ __align__(256) double g_static_gradY_partial[kStaticScratchElems];

// device address of the array, looked up once per device (index = CUDA device ordinal)
static double *static_scratch_address(int *err) {
  static double *addr[64] = {nullptr};
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess || dev < 0 || dev >= 64) {
    *err = 1;
    return nullptr;
  }
  if (addr[dev] == nullptr) {
    // the array's name is a host-side handle, not a device pointer: ask the runtime for the address
    // on the device that is current now
    double *p = nullptr;
    e = cudaGetSymbolAddress(reinterpret_cast<void **>(&p), g_static_gradY_partial);
    if (e != cudaSuccess || p == nullptr) {
      *err = 1;
      return nullptr;
    }
    addr[dev] = p;
  }
  *err = 0;
  return addr[dev];
}

}  // namespace cmace

using namespace cmace;

extern "C" {

int cmace_imp_fwd_f32(const float *X, const float *Y, const float *R, const int32_t *sender,
                      const int32_t *row_ptr, int64_t nnodes, int64_t nedges, int channels, float *out,
                      cmace_stream_t stream) {
  return imp_fwd<float>(X, Y, R, sender, row_ptr, nnodes, nedges, channels, out, stream);
}
int cmace_imp_fwd_f64(const double *X, const double *Y, const double *R, const int32_t *sender,
                      const int32_t *row_ptr, int64_t nnodes, int64_t nedges, int channels, double *out,
                      cmace_stream_t stream) {
  return imp_fwd<double>(X, Y, R, sender, row_ptr, nnodes, nedges, channels, out, stream);
}
int64_t cmace_imp_bwd_scratch_elems(int64_t nedges, int channels, int is_f64) {
  if (channels <= 0 || channels % 32 != 0) return 0;
  const int vec = is_f64 ? pick_vec<double>(channels) : pick_vec<float>(channels);
  const int nchunks = channels / (32 * vec);
  return nchunks > 1 ? (int64_t)nchunks * 16 * nedges : 0;
}
int cmace_imp_bwd_edge_f32(const float *X, const float *Y, const float *R, const float *G,
                           const int32_t *sender, const int32_t *row_ptr, int64_t nnodes, int64_t nedges,
                           int channels, float *gradR, float *gradY, float *T, float *gradY_partial,
                           cmace_stream_t stream) {
  return imp_bwd_edge<float>(X, Y, R, G, sender, row_ptr, nnodes, nedges, channels, gradR, gradY, T,
                             gradY_partial, stream);
}
int cmace_imp_bwd_edge_f64(const double *X, const double *Y, const double *R, const double *G,
                           const int32_t *sender, const int32_t *row_ptr, int64_t nnodes, int64_t nedges,
                           int channels, double *gradR, double *gradY, double *T, double *gradY_partial,
                           cmace_stream_t stream) {
  return imp_bwd_edge<double>(X, Y, R, G, sender, row_ptr, nnodes, nedges, channels, gradR, gradY, T,
                              gradY_partial, stream);
}
int64_t cmace_imp_bwd_edge_f64_noalloc_max_elems(void) { return kStaticScratchElems; }

int cmace_imp_bwd_edge_f64_noalloc(const double *X, const double *Y, const double *R, const double *G,
                                   const int32_t *sender, const int32_t *row_ptr, int64_t nnodes, int64_t nedges,
                                   int channels, double *gradR, double *gradY, double *T, cmace_stream_t stream) {
  const int64_t need = cmace_imp_bwd_scratch_elems(nedges, channels, 1);
  if (need > kStaticScratchElems)
    return fail(CMACE_ERR_UNSUPPORTED,
                "cmace_imp_bwd_edge_f64_noalloc: %lld scratch elements needed, the built-in array holds %lld "
                "(reduce the number of edges per call or use cmace_imp_bwd_edge_f64 with your own scratch)",
                (long long)need, (long long)kStaticScratchElems);
  int err = 0;
  double *scratch = need > 0 ? static_scratch_address(&err) : nullptr;
  if (err) return fail(CMACE_ERR_CUDA, "cmace_imp_bwd_edge_f64_noalloc: cudaGetSymbolAddress failed");
  if (need > 0) {
    // the array keeps the previous call's contents; the part this call sums over starts from zero
    cudaError_t e = cudaMemsetAsync(scratch, 0, (size_t)need * sizeof(double), (cudaStream_t)stream);
    if (e != cudaSuccess)
      return fail(CMACE_ERR_CUDA, "cmace_imp_bwd_edge_f64_noalloc: %s", cudaGetErrorString(e));
  }
  return imp_bwd_edge<double>(X, Y, R, G, sender, row_ptr, nnodes, nedges, channels, gradR, gradY, T, scratch,
                              stream);
}

int cmace_imp_bwd_node_f32(const float *T, const int32_t *perm, const int32_t *send_ptr, int64_t nnodes,
                           int channels, float *gradX, cmace_stream_t stream) {
  return imp_bwd_node<float>(T, perm, send_ptr, nnodes, channels, gradX, stream);
}
int cmace_imp_bwd_node_f64(const double *T, const int32_t *perm, const int32_t *send_ptr, int64_t nnodes,
                           int channels, double *gradX, cmace_stream_t stream) {
  return imp_bwd_node<double>(T, perm, send_ptr, nnodes, channels, gradX, stream);
}
}
