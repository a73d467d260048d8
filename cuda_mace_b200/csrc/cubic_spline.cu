// Cubic-spline evaluation of the tabulated radial weights R[e, j] = a + b x + c x^2 + d x^3 with
// x = r_e - knot(floor(r_e / h)), zero beyond r_max, and its backward gr[e] = sum_j dR/dr * gR[e, j].
// One warp per edge; lanes move VEC consecutive outputs with one 16-byte access.  The
// coefficient table (nintervals x 4 x noutputs) stays L2 resident; R / gR are streamed once.
// The backward recomputes dR/dr from the table rather than reading a saved [E, noutputs] tensor.
#include "common.cuh"

namespace cmace {

template <typename T>
__device__ __forceinline__ bool spline_locate(T r, const T *__restrict__ knots, int nint, T h, T r_max,
                                              int &idx, T &x) {
  if (r > r_max) return false;
  idx = (int)(r / h);
  idx = idx < 0 ? 0 : (idx >= nint ? nint - 1 : idx);
  x = r - knots[idx];
  return true;
}

template <typename T, int VEC>
__global__ void __launch_bounds__(128)
    spline_fwd_kernel(const T *__restrict__ r, const T *__restrict__ knots, const T *__restrict__ coeffs,
                      int64_t E, int nint, int nout, T h, T r_max, T *__restrict__ R) {
  const int lane = threadIdx.x & 31;
  const int64_t e = (int64_t)blockIdx.x * 4 + (threadIdx.x >> 5);
  if (e >= E) return;
  int idx = 0;
  T x = T(0);
  const bool inside = spline_locate<T>(r[e], knots, nint, h, r_max, idx, x);
  const T *cf = coeffs + (int64_t)idx * 4 * nout;
  for (int j = lane * VEC; j < nout; j += 32 * VEC) {
    T o[VEC];
    if (inside) {
      T a[VEC], b[VEC], c[VEC], d[VEC];
      load_vec<T, VEC>(a, cf + j);
      load_vec<T, VEC>(b, cf + nout + j);
      load_vec<T, VEC>(c, cf + 2 * nout + j);
      load_vec<T, VEC>(d, cf + 3 * nout + j);
#pragma unroll
      for (int v = 0; v < VEC; v++) o[v] = a[v] + x * (b[v] + x * (c[v] + x * d[v]));
    } else {
#pragma unroll
      for (int v = 0; v < VEC; v++) o[v] = T(0);
    }
    store_vec<T, VEC>(R + e * nout + j, o);
  }
}

template <typename T, int VEC>
__global__ void __launch_bounds__(128)
    spline_bwd_kernel(const T *__restrict__ r, const T *__restrict__ knots, const T *__restrict__ coeffs,
                      const T *__restrict__ gR, int64_t E, int nint, int nout, T h, T r_max,
                      T *__restrict__ gr) {
  const int lane = threadIdx.x & 31;
  const int64_t e = (int64_t)blockIdx.x * 4 + (threadIdx.x >> 5);
  if (e >= E) return;
  int idx = 0;
  T x = T(0);
  const bool inside = spline_locate<T>(r[e], knots, nint, h, r_max, idx, x);
  T acc = T(0);
  if (inside) {
    const T *cf = coeffs + (int64_t)idx * 4 * nout;
    for (int j = lane * VEC; j < nout; j += 32 * VEC) {
      T b[VEC], c[VEC], d[VEC], g[VEC];
      load_vec<T, VEC>(b, cf + nout + j);
      load_vec<T, VEC>(c, cf + 2 * nout + j);
      load_vec<T, VEC>(d, cf + 3 * nout + j);
      load_vec_stream<T, VEC>(g, gR + e * nout + j);
#pragma unroll
      for (int v = 0; v < VEC; v++) acc = fma(b[v] + x * (T(2) * c[v] + T(3) * x * d[v]), g[v], acc);
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
  if (lane == 0) gr[e] = acc;
}

template <typename T>
static int spline_check(const void *coeffs, const void *R, int64_t E, int nint, int nout, double h,
                        const char *what) {
  if (E < 0 || nint < 1 || nout < 1 || !(h > 0)) return fail(CMACE_ERR_ARG, "%s: bad size", what);
  if (!aligned16(coeffs) || !aligned16(R)) return fail(CMACE_ERR_ARG, "%s: pointers must be 16-byte aligned", what);
  return CMACE_OK;
}

template <typename T>
static int spline_fwd(const T *r, const T *knots, const T *coeffs, int64_t E, int nint, int nout, double h,
                      double r_max, T *R, cmace_stream_t stream) {
  int rc = spline_check<T>(coeffs, R, E, nint, nout, h, "cmace_spline_fwd");
  if (rc) return rc;
  if (E == 0) return CMACE_OK;
  if (!r || !knots || !coeffs || !R) return fail(CMACE_ERR_ARG, "cmace_spline_fwd: null pointer");
  constexpr int W = 16 / sizeof(T);
  const unsigned grid = (unsigned)((E + 3) / 4);
  cudaStream_t st = (cudaStream_t)stream;
  if (nout % W == 0)
    spline_fwd_kernel<T, W><<<grid, 128, 0, st>>>(r, knots, coeffs, E, nint, nout, (T)h, (T)r_max, R);
  else
    spline_fwd_kernel<T, 1><<<grid, 128, 0, st>>>(r, knots, coeffs, E, nint, nout, (T)h, (T)r_max, R);
  return check_launch("cmace_spline_fwd");
}

template <typename T>
static int spline_bwd(const T *r, const T *knots, const T *coeffs, const T *gR, int64_t E, int nint,
                      int nout, double h, double r_max, T *gr, cmace_stream_t stream) {
  int rc = spline_check<T>(coeffs, gR, E, nint, nout, h, "cmace_spline_bwd");
  if (rc) return rc;
  if (E == 0) return CMACE_OK;
  if (!r || !knots || !coeffs || !gR || !gr) return fail(CMACE_ERR_ARG, "cmace_spline_bwd: null pointer");
  constexpr int W = 16 / sizeof(T);
  const unsigned grid = (unsigned)((E + 3) / 4);
  cudaStream_t st = (cudaStream_t)stream;
  if (nout % W == 0)
    spline_bwd_kernel<T, W><<<grid, 128, 0, st>>>(r, knots, coeffs, gR, E, nint, nout, (T)h, (T)r_max, gr);
  else
    spline_bwd_kernel<T, 1><<<grid, 128, 0, st>>>(r, knots, coeffs, gR, E, nint, nout, (T)h, (T)r_max, gr);
  return check_launch("cmace_spline_bwd");
}

}  // namespace cmace

using namespace cmace;

extern "C" {
int cmace_spline_fwd_f32(const float *r, const float *k, const float *c, int64_t E, int nint, int nout,
                         double h, double r_max, float *R, cmace_stream_t s) {
  return spline_fwd<float>(r, k, c, E, nint, nout, h, r_max, R, s);
}
int cmace_spline_fwd_f64(const double *r, const double *k, const double *c, int64_t E, int nint, int nout,
                         double h, double r_max, double *R, cmace_stream_t s) {
  return spline_fwd<double>(r, k, c, E, nint, nout, h, r_max, R, s);
}
int cmace_spline_bwd_f32(const float *r, const float *k, const float *c, const float *gR, int64_t E,
                         int nint, int nout, double h, double r_max, float *gr, cmace_stream_t s) {
  return spline_bwd<float>(r, k, c, gR, E, nint, nout, h, r_max, gr, s);
}
int cmace_spline_bwd_f64(const double *r, const double *k, const double *c, const double *gR, int64_t E,
                         int nint, int nout, double h, double r_max, double *gr, cmace_stream_t s) {
  return spline_bwd<double>(r, k, c, gR, E, nint, nout, h, r_max, gr, s);
}
}
