// Host-side construction of the symmetric-contraction program from the reference's sparse U
// tables (layout of cuda_mace/ops/symmetric_contraction.py:91-187).  Plain C++ so that the same
// code is compiled into the CUDA library and into the host check library.
//
// Cubic part: per coupling path p the form B_p(x) = sum U3[i,j,k,p] x_i x_j x_k is reduced to
// monomials x_a x_b x_c (a<=b<=c); proportional forms are merged into classes; for every class the
// gradient terms  dB_q/dx_i = sum coef * x_j * x_k  are listed grouped by i.  Quadratic part alike.
#pragma once
#include <cmath>
#include <cstdint>
#include <map>
#include <string>
#include <vector>

#include "symcon_canonical.inc"

namespace cmace {

struct SymconProgram {
  int nclass3 = 0, nclass2 = 0;
  std::vector<int32_t> seg3, seg2;        // [17] term ranges per differentiated index i
  std::vector<int32_t> class3, class2;    // [w3], [w2] class of each path
  std::vector<double> scale3, scale2;     // [w3], [w2] form_p = scale_p * form_class
  std::vector<int32_t> packed3, packed2;  // j | k << 8 | class << 16   /   j | class << 16
  std::vector<double> coef3, coef2;
  // When the forms equal the build-time canonical ones up to a scale per class, the generated
  // straight-line kernel can be used: form_p = canon_scale_p * canonical_form[canon_class_p].
  bool canonical = false;
  std::vector<int32_t> canon_class3, canon_class2;
  std::vector<double> canon_scale3, canon_scale2;
};


struct Mono {
  int a, b, c;
  bool operator<(const Mono &o) const { return a != o.a ? a < o.a : (b != o.b ? b < o.b : c < o.c); }
};
typedef std::map<Mono, double> Poly;

// Finds the build-time canonical class a form is proportional to (form = sigma * canonical); -1 if none.
template <int W>
inline int match_canonical(const Poly &form, const int (*monos)[W], const double *coefs, const int *starts,
                           int nclass, double &sigma) {
  for (int q = 0; q < nclass; q++) {
    if ((int)form.size() != starts[q + 1] - starts[q]) continue;
    bool ok = true;
    double s = 0.0;
    for (int t = starts[q]; t < starts[q + 1] && ok; t++) {
      const Mono m{monos[t][0], monos[t][1], W == 3 ? monos[t][W - 1] : 0};
      auto it = form.find(m);
      if (it == form.end()) { ok = false; break; }
      const double ratio = it->second / coefs[t];
      if (s == 0.0) s = ratio;
      if (std::fabs(ratio - s) > 1e-5 * std::fabs(s)) ok = false;
    }
    if (ok) { sigma = s; return q; }
  }
  return -1;
}

// Groups proportional polynomials: cls[p] = class id, scale[p] with poly_p = scale[p] * poly_rep.
inline void classify(const std::vector<Poly> &polys, std::vector<int> &cls, std::vector<double> &scale,
                     std::vector<int> &reps) {
  const int n = (int)polys.size();
  cls.assign(n, -1);
  scale.assign(n, 0.0);
  reps.clear();
  for (int p = 0; p < n; p++) {
    if (polys[p].empty()) continue;  // path that never occurs: its weight is unused
    for (size_t r = 0; r < reps.size() && cls[p] < 0; r++) {
      const Poly &a = polys[reps[r]], &b = polys[p];
      if (a.size() != b.size()) continue;
      double s = 0.0;
      bool ok = true;
      auto ia = a.begin();
      auto ib = b.begin();
      for (; ia != a.end(); ++ia, ++ib) {
        if (ia->first < ib->first || ib->first < ia->first) { ok = false; break; }
        const double ratio = ib->second / ia->second;
        if (s == 0.0) s = ratio;
        if (std::fabs(ratio - s) > 1e-6 * std::fabs(s)) { ok = false; break; }
      }
      if (ok) {
        cls[p] = (int)r;
        scale[p] = s;
      }
    }
    if (cls[p] < 0) {
      cls[p] = (int)reps.size();
      scale[p] = 1.0;
      reps.push_back(p);
    }
  }
}

inline bool build_symcon_program(int maxnz, const int16_t *u3_num, const int32_t *u3_idx, const double *u3_val,
                                 const int16_t *u2_num, const int16_t *u2_idx, const double *u2_val, int w3,
                                 int w2, int w1, SymconProgram &prog, std::string &err) {
  if (!u3_num || !u3_idx || !u3_val || !u2_num || !u2_idx || !u2_val) { err = "null pointer"; return false; }
  if (maxnz < 0 || w3 < 1 || w3 > 255 || w2 < 1 || w2 > 255 || w1 < 1) { err = "bad sizes"; return false; }
  std::vector<Poly> poly3(w3), poly2(w2);
  for (int i = 0; i < 16; i++)
    for (int j = 0; j < 16; j++) {
      const int n = u3_num[i * 16 + j];
      if (n < 0 || n > maxnz) { err = "U3_num_nonzero exceeds the table depth"; return false; }
      for (int t = 0; t < n; t++) {
        const int32_t pk = u3_idx[(t * 16 + i) * 16 + j];
        const int p = pk & 0xff, k = (pk >> 8) & 0xff;
        if (p >= w3 || k >= 16) { err = "U3 index out of range"; return false; }
        int m[3] = {i, j, k};
        if (m[0] > m[1]) std::swap(m[0], m[1]);
        if (m[1] > m[2]) std::swap(m[1], m[2]);
        if (m[0] > m[1]) std::swap(m[0], m[1]);
        poly3[p][Mono{m[0], m[1], m[2]}] += u3_val[(t * 16 + i) * 16 + j];
      }
      if (u2_num[i * 16 + j] > 0) {
        const int p = u2_idx[i * 16 + j];
        if (p < 0 || p >= w2) { err = "U2 index out of range"; return false; }
        poly2[p][Mono{i < j ? i : j, i < j ? j : i, 0}] += u2_val[i * 16 + j];
      }
    }
  for (auto *polys : {&poly3, &poly2})
    for (auto &P : *polys)
      for (auto it = P.begin(); it != P.end();) it = (std::fabs(it->second) < 1e-14) ? P.erase(it) : std::next(it);

  std::vector<int> cls3, cls2, reps3, reps2;
  std::vector<double> sc3, sc2;
  classify(poly3, cls3, sc3, reps3);
  classify(poly2, cls2, sc2, reps2);

  struct Term { int j, k, q; double coef; };
  std::vector<std::vector<Term>> t3(16), t2(16);
  for (size_t q = 0; q < reps3.size(); q++)
    for (auto &kv : poly3[reps3[q]]) {
      const int m[3] = {kv.first.a, kv.first.b, kv.first.c};
      for (int s = 0; s < 3; s++) {
        if (s > 0 && m[s] == m[s - 1]) continue;  // each distinct index once
        int mult = 0, rest[3], nr = 0;
        bool removed = false;
        for (int u = 0; u < 3; u++) {
          if (m[u] == m[s]) mult++;
          if (m[u] == m[s] && !removed) { removed = true; continue; }
          rest[nr++] = m[u];
        }
        t3[m[s]].push_back(Term{rest[0], rest[1], (int)q, kv.second * mult});
      }
    }
  for (size_t q = 0; q < reps2.size(); q++)
    for (auto &kv : poly2[reps2[q]]) {
      const int a = kv.first.a, b = kv.first.b;
      if (a == b) {
        t2[a].push_back(Term{a, 0, (int)q, 2.0 * kv.second});
      } else {
        t2[a].push_back(Term{b, 0, (int)q, kv.second});
        t2[b].push_back(Term{a, 0, (int)q, kv.second});
      }
    }

  prog = SymconProgram();
  prog.nclass3 = (int)reps3.size();
  prog.nclass2 = (int)reps2.size();
  prog.seg3.assign(17, 0);
  prog.seg2.assign(17, 0);
  for (int i = 0; i < 16; i++) {
    prog.seg3[i] = (int)prog.packed3.size();
    for (auto &t : t3[i]) { prog.packed3.push_back(t.j | (t.k << 8) | (t.q << 16)); prog.coef3.push_back(t.coef); }
    prog.seg2[i] = (int)prog.packed2.size();
    for (auto &t : t2[i]) { prog.packed2.push_back(t.j | (t.q << 16)); prog.coef2.push_back(t.coef); }
  }
  prog.seg3[16] = (int)prog.packed3.size();
  prog.seg2[16] = (int)prog.packed2.size();
  for (int p = 0; p < w3; p++) { prog.class3.push_back(cls3[p] < 0 ? 0 : cls3[p]); prog.scale3.push_back(cls3[p] < 0 ? 0.0 : sc3[p]); }
  for (int p = 0; p < w2; p++) { prog.class2.push_back(cls2[p] < 0 ? 0 : cls2[p]); prog.scale2.push_back(cls2[p] < 0 ? 0.0 : sc2[p]); }

  // canonical matching
  prog.canonical = true;
  std::vector<int> cq3(reps3.size()), cq2(reps2.size());
  std::vector<double> sg3(reps3.size()), sg2(reps2.size());
  for (size_t q = 0; q < reps3.size() && prog.canonical; q++) {
    cq3[q] = match_canonical<3>(poly3[reps3[q]], canon::kMono3, canon::kCoef3, canon::kClassStart3, canon::NCLASS3, sg3[q]);
    if (cq3[q] < 0) prog.canonical = false;
  }
  for (size_t q = 0; q < reps2.size() && prog.canonical; q++) {
    cq2[q] = match_canonical<2>(poly2[reps2[q]], canon::kMono2, canon::kCoef2, canon::kClassStart2, canon::NCLASS2, sg2[q]);
    if (cq2[q] < 0) prog.canonical = false;
  }
  if (prog.canonical) {
    for (int p = 0; p < w3; p++) {
      prog.canon_class3.push_back(cls3[p] < 0 ? 0 : cq3[cls3[p]]);
      prog.canon_scale3.push_back(cls3[p] < 0 ? 0.0 : sc3[p] * sg3[cls3[p]]);
    }
    for (int p = 0; p < w2; p++) {
      prog.canon_class2.push_back(cls2[p] < 0 ? 0 : cq2[cls2[p]]);
      prog.canon_scale2.push_back(cls2[p] < 0 ? 0.0 : sc2[p] * sg2[cls2[p]]);
    }
  }
  return true;
}

// Reference evaluation of a program for one (node, channel): x[16], per-path weights.
// Returns the output value and, when grad != nullptr, d out / d x_i.  Mirrors the device loop.
inline double eval_symcon_program(const SymconProgram &pg, const double *x, const double *W3, const double *W2,
                                  double w1, double *grad) {
  std::vector<double> weff(pg.nclass3 + pg.nclass2, 0.0);
  for (size_t p = 0; p < pg.class3.size(); p++) weff[pg.class3[p]] += pg.scale3[p] * W3[p];
  for (size_t p = 0; p < pg.class2.size(); p++) weff[pg.nclass3 + pg.class2[p]] += pg.scale2[p] * W2[p];
  double acc = 0.0;
  for (int i = 0; i < 16; i++) {
    double d3 = 0.0, d2 = 0.0;
    for (int t = pg.seg3[i]; t < pg.seg3[i + 1]; t++) {
      const int pk = pg.packed3[t];
      d3 += pg.coef3[t] * weff[pk >> 16] * x[pk & 0xff] * x[(pk >> 8) & 0xff];
    }
    for (int t = pg.seg2[i]; t < pg.seg2[i + 1]; t++) {
      const int pk = pg.packed2[t];
      d2 += pg.coef2[t] * weff[pg.nclass3 + (pk >> 16)] * x[pk & 0xff];
    }
    const double d1 = i == 0 ? w1 : 0.0;
    if (grad) grad[i] = d1 + d2 + d3;
    acc += x[i] * (d1 + 0.5 * d2 + d3 / 3.0);
  }
  return acc;
}

// Same result through the generated straight-line code (requires pg.canonical).
inline double eval_symcon_canonical(const SymconProgram &pg, const double *x, const double *W3, const double *W2,
                                    double w1, double *grad) {
  double w3[canon::NCLASS3] = {0}, w2[canon::NCLASS2] = {0}, xx[16], g[16], value;
  for (size_t p = 0; p < pg.canon_class3.size(); p++) w3[pg.canon_class3[p]] += pg.canon_scale3[p] * W3[p];
  for (size_t p = 0; p < pg.canon_class2.size(); p++) w2[pg.canon_class2[p]] += pg.canon_scale2[p] * W2[p];
  for (int i = 0; i < 16; i++) xx[i] = x[i];
  canon::eval<double>(xx, w3, w2, w1, g, value);
  if (grad)
    for (int i = 0; i < 16; i++) grad[i] = g[i];
  return value;
}

}  // namespace cmace
