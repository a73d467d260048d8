// Per-edge basis kernels: real spherical harmonics to l=3 (output Y [16, E]) and, optionally,
// the Bessel x polynomial-cutoff radial basis (output B [E, nbessel]); one thread per edge.
// Both are pure streams (27 scalars written per 3 read), so the kernels only have to keep the
// stores coalesced: consecutive threads write consecutive e of each Y row, and each thread writes
// its nbessel contiguous B values.  The backward recomputes every derivative from xyz, which
// removes the reference's saved dY [16,3,E] table (3x the size of Y) from the HBM traffic.
#include "common.cuh"
#include "edge_math.cuh"

namespace cmace {

constexpr int kMaxBessel = 16;

template <typename T>
__global__ void __launch_bounds__(256)
    edge_basis_fwd_kernel(const T *__restrict__ xyz, int64_t E, T r_max, int nb, int p,
                          T *__restrict__ Y, T *__restrict__ B) {
  const int64_t e = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (e >= E) return;
  const T v0 = xyz[e * 3 + 0], v1 = xyz[e * 3 + 1], v2 = xyz[e * 3 + 2];
  T y[16], b[kMaxBessel];
  edge_basis_fwd_one<T>(v0, v1, v2, r_max, nb, p, y, B != nullptr ? b : nullptr);
#pragma unroll
  for (int m = 0; m < 16; m++) Y[(int64_t)m * E + e] = y[m];
  if (B != nullptr)
    for (int n = 0; n < nb; n++) B[e * nb + n] = b[n];
}

template <typename T>
__global__ void __launch_bounds__(256)
    edge_basis_bwd_kernel(const T *__restrict__ xyz, const T *__restrict__ gY,
                          const T *__restrict__ gB, int64_t E, T r_max, int nb, int p,
                          T *__restrict__ gxyz) {
  const int64_t e = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (e >= E) return;
  const T v0 = xyz[e * 3 + 0], v1 = xyz[e * 3 + 1], v2 = xyz[e * 3 + 2];
  T g[16], gb[kMaxBessel];
#pragma unroll
  for (int m = 0; m < 16; m++) g[m] = gY[(int64_t)m * E + e];
  if (gB != nullptr)
    for (int n = 0; n < nb; n++) gb[n] = gB[e * nb + n];
  T o0, o1, o2;
  edge_basis_bwd_one<T>(v0, v1, v2, g, gB != nullptr ? gb : nullptr, r_max, nb, p, o0, o1, o2);
  gxyz[e * 3 + 0] = o0;
  gxyz[e * 3 + 1] = o1;
  gxyz[e * 3 + 2] = o2;
}

template <typename T>
static int edge_fwd(const T *xyz, int64_t E, double r_max, int nb, int p, T *Y, T *B,
                    cmace_stream_t stream) {
  if (E < 0) return fail(CMACE_ERR_ARG, "cmace_edge_basis_fwd: negative size");
  if (E == 0) return CMACE_OK;
  if (!xyz || !Y) return fail(CMACE_ERR_ARG, "cmace_edge_basis_fwd: null pointer");
  if (B && (nb < 1 || nb > kMaxBessel || p < 1 || !(r_max > 0)))
    return fail(CMACE_ERR_UNSUPPORTED, "cmace_edge_basis_fwd: nbessel in 1..%d, p >= 1, r_max > 0", kMaxBessel);
  edge_basis_fwd_kernel<T><<<(unsigned)((E + 255) / 256), 256, 0, (cudaStream_t)stream>>>(
      xyz, E, (T)r_max, nb, p, Y, B);
  return check_launch("cmace_edge_basis_fwd");
}

template <typename T>
static int edge_bwd(const T *xyz, const T *gY, const T *gB, int64_t E, double r_max, int nb, int p,
                    T *gxyz, cmace_stream_t stream) {
  if (E < 0) return fail(CMACE_ERR_ARG, "cmace_edge_basis_bwd: negative size");
  if (E == 0) return CMACE_OK;
  if (!xyz || !gY || !gxyz) return fail(CMACE_ERR_ARG, "cmace_edge_basis_bwd: null pointer");
  if (gB && (nb < 1 || nb > kMaxBessel || p < 1 || !(r_max > 0)))
    return fail(CMACE_ERR_UNSUPPORTED, "cmace_edge_basis_bwd: nbessel in 1..%d, p >= 1, r_max > 0", kMaxBessel);
  edge_basis_bwd_kernel<T><<<(unsigned)((E + 255) / 256), 256, 0, (cudaStream_t)stream>>>(
      xyz, gY, gB, E, (T)r_max, nb, p, gxyz);
  return check_launch("cmace_edge_basis_bwd");
}

}  // namespace cmace

using namespace cmace;

extern "C" {
int cmace_sph_fwd_f32(const float *xyz, int64_t E, float *Y, cmace_stream_t s) {
  return edge_fwd<float>(xyz, E, 1.0, 0, 1, Y, nullptr, s);
}
int cmace_sph_fwd_f64(const double *xyz, int64_t E, double *Y, cmace_stream_t s) {
  return edge_fwd<double>(xyz, E, 1.0, 0, 1, Y, nullptr, s);
}
int cmace_sph_bwd_f32(const float *xyz, const float *gY, int64_t E, float *gxyz, cmace_stream_t s) {
  return edge_bwd<float>(xyz, gY, nullptr, E, 1.0, 0, 1, gxyz, s);
}
int cmace_sph_bwd_f64(const double *xyz, const double *gY, int64_t E, double *gxyz, cmace_stream_t s) {
  return edge_bwd<double>(xyz, gY, nullptr, E, 1.0, 0, 1, gxyz, s);
}
int cmace_edge_basis_fwd_f32(const float *xyz, int64_t E, double r_max, int nb, int p, float *Y, float *B,
                             cmace_stream_t s) {
  return edge_fwd<float>(xyz, E, r_max, nb, p, Y, B, s);
}
int cmace_edge_basis_fwd_f64(const double *xyz, int64_t E, double r_max, int nb, int p, double *Y,
                             double *B, cmace_stream_t s) {
  return edge_fwd<double>(xyz, E, r_max, nb, p, Y, B, s);
}
int cmace_edge_basis_bwd_f32(const float *xyz, const float *gY, const float *gB, int64_t E, double r_max,
                             int nb, int p, float *gxyz, cmace_stream_t s) {
  return edge_bwd<float>(xyz, gY, gB, E, r_max, nb, p, gxyz, s);
}
int cmace_edge_basis_bwd_f64(const double *xyz, const double *gY, const double *gB, int64_t E, double r_max,
                             int nb, int p, double *gxyz, cmace_stream_t s) {
  return edge_bwd<double>(xyz, gY, gB, E, r_max, nb, p, gxyz, s);
}
}
