// Per-edge math shared by the device kernels and a host-compiled check library:
// real spherical harmonics to l=3 of the normalised edge vector and their vector-Jacobian
// product, Bessel radial basis with polynomial cutoff and its derivative.
//
// Conventions (same as spherical_harmonics_impl.cu:62-125 of the cuda-mace project): the
// harmonic's axes (X, Y, Z) are the input's components (2, 0, 1), components are ordered
// (l, m) with m = -l..l, and scaled by sqrt(4 pi) so that sum_m Y_lm^2 = 2l+1.
// Written as homogeneous polynomials P_lm of the unit vector u = v/|v|, which gives
//   dY_lm/dv_a = ( dP_lm/du_a (u) - l * P_lm(u) * u_a ) / |v| .
#pragma once

#if defined(__CUDACC__)
#define CMACE_HD __host__ __device__ __forceinline__
#else
#define CMACE_HD inline
#endif

#include <cmath>

namespace cmace {

template <typename T>
struct ShConst {
  static constexpr T s3 = T(1.7320508075688772935);    // sqrt(3)
  static constexpr T s5 = T(2.2360679774997896964);    // sqrt(5)
  static constexpr T s7 = T(2.6457513110645905905);    // sqrt(7)
  static constexpr T s15 = T(3.8729833462074168852);   // sqrt(15)
  static constexpr T s105 = T(10.246950765959598383);  // sqrt(105)
  static constexpr T a = T(2.0916500663351888699);     // sqrt(35/8)
  static constexpr T b = T(1.6201851746019650785);     // sqrt(21/8)
};

// out[16] = Y_lm of the unit vector with harmonic axes (X, Y, Z)
template <typename T>
CMACE_HD void sph_l3(T X, T Y, T Z, T (&out)[16]) {
  using K = ShConst<T>;
  const T X2 = X * X, Y2 = Y * Y, Z2 = Z * Z;
  out[0] = T(1);
  out[1] = K::s3 * Y;
  out[2] = K::s3 * Z;
  out[3] = K::s3 * X;
  out[4] = K::s15 * X * Y;
  out[5] = K::s15 * Y * Z;
  out[6] = T(0.5) * K::s5 * (T(2) * Z2 - X2 - Y2);
  out[7] = K::s15 * X * Z;
  out[8] = T(0.5) * K::s15 * (X2 - Y2);
  const T q = T(4) * Z2 - X2 - Y2;
  out[9] = K::a * Y * (T(3) * X2 - Y2);
  out[10] = K::s105 * X * Y * Z;
  out[11] = K::b * Y * q;
  out[12] = T(0.5) * K::s7 * Z * (T(2) * Z2 - T(3) * X2 - T(3) * Y2);
  out[13] = K::b * X * q;
  out[14] = T(0.5) * K::s105 * Z * (X2 - Y2);
  out[15] = K::a * X * (X2 - T(3) * Y2);
}

// Vector-Jacobian product: given g[16] = d loss / d Y_lm returns (GX, GY, GZ) with
// G_a = sum_lm g_lm * ( dP_lm/da - l P_lm a ), a in harmonic axes; the caller divides by |v|.
template <typename T>
CMACE_HD void sph_l3_vjp(T X, T Y, T Z, const T (&g)[16], T &GX, T &GY, T &GZ) {
  using K = ShConst<T>;
  const T X2 = X * X, Y2 = Y * Y, Z2 = Z * Z;
  T P[16];
  sph_l3(X, Y, Z, P);
  // S = sum_lm l * g_lm * P_lm
  T S = T(0);
#pragma unroll
  for (int m = 1; m < 4; m++) S += g[m] * P[m];
  T S2 = T(0), S3 = T(0);
#pragma unroll
  for (int m = 4; m < 9; m++) S2 += g[m] * P[m];
#pragma unroll
  for (int m = 9; m < 16; m++) S3 += g[m] * P[m];
  S += T(2) * S2 + T(3) * S3;
  const T q = T(4) * Z2 - X2 - Y2;
  GX = g[3] * K::s3 + g[4] * K::s15 * Y - g[6] * K::s5 * X + g[7] * K::s15 * Z + g[8] * K::s15 * X +
       g[9] * T(6) * K::a * X * Y + g[10] * K::s105 * Y * Z - g[11] * T(2) * K::b * X * Y -
       g[12] * T(3) * K::s7 * X * Z + g[13] * K::b * (q - T(2) * X2) + g[14] * K::s105 * X * Z +
       g[15] * T(3) * K::a * (X2 - Y2);
  GY = g[1] * K::s3 + g[4] * K::s15 * X + g[5] * K::s15 * Z - g[6] * K::s5 * Y - g[8] * K::s15 * Y +
       g[9] * T(3) * K::a * (X2 - Y2) + g[10] * K::s105 * X * Z + g[11] * K::b * (q - T(2) * Y2) -
       g[12] * T(3) * K::s7 * Y * Z - g[13] * T(2) * K::b * X * Y - g[14] * K::s105 * Y * Z -
       g[15] * T(6) * K::a * X * Y;
  GZ = g[2] * K::s3 + g[5] * K::s15 * Y + g[6] * T(2) * K::s5 * Z + g[7] * K::s15 * X +
       g[10] * K::s105 * X * Y + g[11] * T(8) * K::b * Y * Z +
       g[12] * T(1.5) * K::s7 * (T(2) * Z2 - X2 - Y2) + g[13] * T(8) * K::b * X * Z +
       g[14] * T(0.5) * K::s105 * (X2 - Y2);
  GX -= S * X;
  GY -= S * Y;
  GZ -= S * Z;
}

// Polynomial cutoff of order p at x = r/r_max and its derivative with respect to x:
//   f = 1 - (p+1)(p+2)/2 x^p + p(p+2) x^(p+1) - p(p+1)/2 x^(p+2)   for x < 1, else 0,
// evaluated in the equivalent factored form (1-x)^3 * sum_{k<p} (k+1)(k+2)/2 x^k, which has no
// cancellation near the cutoff.
template <typename T>
CMACE_HD void poly_cutoff(T x, int p, T &f, T &df) {
  if (!(x < T(1))) {
    f = T(0);
    df = T(0);
    return;
  }
  T S = T(0), dS = T(0);
  for (int k = p - 1; k >= 0; k--) {  // Horner, value and derivative
    dS = dS * x + S;
    S = S * x + T(0.5) * T((k + 1) * (k + 2));
  }
  const T u = T(1) - x, u2 = u * u;
  f = u2 * u * S;
  df = u2 * (u * dS - T(3) * S);
}

// Radial basis b_n(r) = sqrt(2/r_max) sin(n pi r / r_max) / r * f(r/r_max), n = 1..nb (nb <= 16),
// and optionally db_n/dr.  sin/cos of the multiples come from the angle-addition recurrence.
template <typename T>
CMACE_HD void bessel_cutoff(T r, T r_max, int nb, int p, T *b, T *db) {
  const T kPi = T(3.14159265358979323846);
  const T pref = sqrt(T(2) / r_max);
  const T w = kPi / r_max;
  const T th = w * r;
  const T s1 = sin(th), c1 = cos(th);
  T f, df;
  poly_cutoff(r / r_max, p, f, df);
  df = df / r_max;  // d f / d r
  const T ir = T(1) / r;
  T s = s1, c = c1;
  for (int n = 1; n <= nb; n++) {
    const T base = pref * s * ir;
    b[n - 1] = base * f;
    if (db != nullptr) {
      // d/dr [ sin(n w r) / r ] = n w cos(n w r) / r - sin(n w r) / r^2
      const T dbase = pref * (T(n) * w * c - s * ir) * ir;
      db[n - 1] = dbase * f + base * df;
    }
    const T sn = s * c1 + c * s1;
    c = c * c1 - s * s1;
    s = sn;
  }
}

// ---- whole per-edge bodies, shared by the kernels and the host check library -------------------

template <typename T>
CMACE_HD T inv_sqrt(T x) {
#if defined(__CUDA_ARCH__)
  return rsqrt(x);
#else
  return T(1) / std::sqrt(x);
#endif
}

// v[3] -> y[16] (and b[nb] when b != nullptr)
template <typename T>
CMACE_HD void edge_basis_fwd_one(T v0, T v1, T v2, T r_max, int nb, int p, T (&y)[16], T *b) {
  const T r2 = v0 * v0 + v1 * v1 + v2 * v2;
  const T ir = inv_sqrt(r2);
  sph_l3<T>(v2 * ir, v0 * ir, v1 * ir, y);
  if (b != nullptr) bessel_cutoff<T>(r2 * ir, r_max, nb, p, b, nullptr);
}

// d loss / d v from g[16] = d loss / d Y and (optionally) gb[nb] = d loss / d B
template <typename T>
CMACE_HD void edge_basis_bwd_one(T v0, T v1, T v2, const T (&g)[16], const T *gb, T r_max, int nb, int p,
                                 T &o0, T &o1, T &o2) {
  const T r2 = v0 * v0 + v1 * v1 + v2 * v2;
  const T ir = inv_sqrt(r2);
  const T X = v2 * ir, Y = v0 * ir, Z = v1 * ir;
  T GX, GY, GZ;
  sph_l3_vjp<T>(X, Y, Z, g, GX, GY, GZ);
  // back to the input's component order: component 0 <-> Y axis, 1 <-> Z, 2 <-> X
  o0 = GY * ir;
  o1 = GZ * ir;
  o2 = GX * ir;
  if (gb != nullptr) {
    T b[16], db[16];
    bessel_cutoff<T>(r2 * ir, r_max, nb, p, b, db);
    T gr = T(0);
    for (int n = 0; n < nb; n++) gr += gb[n] * db[n];
    // d r / d v_a = v_a / r
    o0 += gr * Y;
    o1 += gr * Z;
    o2 += gr * X;
  }
}

}  // namespace cmace
