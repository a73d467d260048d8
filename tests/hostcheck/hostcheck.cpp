// Host-compiled copy of the per-edge math (edge_math.cuh), so that the formulas the kernels run
// can be checked on a machine without a GPU.  Loops over edges on the CPU; same layouts as the
// device entry points (xyz [E,3], Y [16,E], B [E,nb]).
#include <cstdint>

#include "edge_math.cuh"   // found through -I cuda_mace_b200/csrc (tests/conftest.py builds this file)

using namespace cmace;

extern "C" {
void hc_edge_basis_fwd_f64(const double *xyz, int64_t E, double r_max, int nb, int p, double *Y, double *B) {
  for (int64_t e = 0; e < E; e++) {
    double y[16], b[16];
    edge_basis_fwd_one<double>(xyz[e * 3], xyz[e * 3 + 1], xyz[e * 3 + 2], r_max, nb, p, y, B ? b : nullptr);
    for (int m = 0; m < 16; m++) Y[m * E + e] = y[m];
    if (B)
      for (int n = 0; n < nb; n++) B[e * nb + n] = b[n];
  }
}
void hc_edge_basis_bwd_f64(const double *xyz, const double *gY, const double *gB, int64_t E, double r_max, int nb,
                           int p, double *gxyz) {
  for (int64_t e = 0; e < E; e++) {
    double g[16];
    for (int m = 0; m < 16; m++) g[m] = gY[m * E + e];
    edge_basis_bwd_one<double>(xyz[e * 3], xyz[e * 3 + 1], xyz[e * 3 + 2], g, gB ? gB + e * nb : nullptr, r_max, nb,
                               p, gxyz[e * 3], gxyz[e * 3 + 1], gxyz[e * 3 + 2]);
  }
}
void hc_edge_basis_fwd_f32(const float *xyz, int64_t E, float r_max, int nb, int p, float *Y, float *B) {
  for (int64_t e = 0; e < E; e++) {
    float y[16], b[16];
    edge_basis_fwd_one<float>(xyz[e * 3], xyz[e * 3 + 1], xyz[e * 3 + 2], r_max, nb, p, y, B ? b : nullptr);
    for (int m = 0; m < 16; m++) Y[m * E + e] = y[m];
    if (B)
      for (int n = 0; n < nb; n++) B[e * nb + n] = b[n];
  }
}
}

#include "symcon_plan.hpp"

extern "C" {
// Builds the contraction program on the host and evaluates it for N nodes x C channels.
// X [N,16,C], atom_types [N], W3 [Z,w3,C], W2 [Z,w2,C], W1 [Z,w1,C] -> out [N,C], grad [N,16,C].
// info[0..4] = nclass3, nclass2, nterms3, nterms2, canonical-match flag.  use_canonical selects the generated
// straight-line code when the tables match the build-time canonical ones.  Returns 0 on success.
int hc_symcon_f64(int maxnz, const int16_t *u3_num, const int32_t *u3_idx, const double *u3_val,
                  const int16_t *u2_num, const int16_t *u2_idx, const double *u2_val, int w3, int w2, int w1,
                  const double *X, const int32_t *atom_types, const double *W3, const double *W2, const double *W1,
                  int64_t N, int C, double *out, double *grad, int32_t *info, int use_canonical) {
  SymconProgram pg;
  std::string err;
  if (!build_symcon_program(maxnz, u3_num, u3_idx, u3_val, u2_num, u2_idx, u2_val, w3, w2, w1, pg, err)) return 1;
  info[0] = pg.nclass3; info[1] = pg.nclass2; info[2] = (int)pg.packed3.size(); info[3] = (int)pg.packed2.size();
  info[4] = pg.canonical ? 1 : 0;
  std::vector<double> a(w3), b(w2);
  for (int64_t n = 0; n < N; n++)
    for (int c = 0; c < C; c++) {
      const int z = atom_types[n];
      double x[16], g[16];
      for (int i = 0; i < 16; i++) x[i] = X[(n * 16 + i) * C + c];
      for (int p = 0; p < w3; p++) a[p] = W3[((int64_t)z * w3 + p) * C + c];
      for (int p = 0; p < w2; p++) b[p] = W2[((int64_t)z * w2 + p) * C + c];
      const double w1v = W1[(int64_t)z * w1 * C + c];
      out[n * C + c] = (use_canonical && pg.canonical) ? eval_symcon_canonical(pg, x, a.data(), b.data(), w1v, g)
                                                       : eval_symcon_program(pg, x, a.data(), b.data(), w1v, g);
      for (int i = 0; i < 16; i++) grad[(n * 16 + i) * C + c] = g[i];
    }
  return 0;
}
}
