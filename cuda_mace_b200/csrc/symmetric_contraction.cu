// Symmetric contraction, correlation 3, invariant (L=0) output:
//
//   out[n,c] = sum_ijk T3[z_n,i,j,k,c] x_i x_j x_k + sum_ij T2[z_n,i,j,c] x_i x_j + W1[z_n,0,c] x_0,
//   T3 = sum_p U3[i,j,k,p] W3[z,p,c],  T2 = sum_p U2[i,j,p] W2[z,p,c],  x_i = X[n,i,c].
//
// The plan turns the reference's sparse U tables into a symmetrised program.  Per coupling path p
// the cubic form B_p(x) = sum U3[i,j,k,p] x_i x_j x_k only depends on the monomials x_a x_b x_c
// (a<=b<=c), so permuted index triples are merged, and paths whose forms are proportional are
// merged into one class q with an effective weight Weff[q] = sum_p s_p W[p].  For each class the
// kernel evaluates the gradient D_q[i] = dB_q/dx_i term by term; Euler's identity then gives the
// value for free, out = sum_i x_i (W1 d_i0 + 1/2 sum_q2 Weff2 D2_q[i] + 1/3 sum_q3 Weff3 D3_q[i]),
// and the same loop yields the exact input gradient, so the backward recomputes from X instead of
// reading a saved [N,16,C] derivative.
//
// Mapping: lane <-> channel, one warp per (node, 32-channel chunk); the node's 16 components and
// the effective weights sit in shared memory (conflict-free, lane-major), the program is read
// with warp-uniform addresses.  No atomics; every output element has one writer.
#include <cmath>
#include <cstdlib>
#include <string>
#include <vector>

#include "common.cuh"
#include "symcon_plan.hpp"

struct cmace_symcon_plan {
  int w3 = 0, w2 = 0, w1 = 0;
  int nclass3 = 0, nclass2 = 0;
  int nterms3 = 0, nterms2 = 0;
  // device arrays
  int32_t *d_ints = nullptr;   // [seg3 (17)] [seg2 (17)] [class3 (w3)] [class2 (w2)] [packed3] [packed2]
  double *d_f64 = nullptr;     // [scale3 (w3)] [scale2 (w2)] [coef3] [coef2]
  float *d_f32 = nullptr;      // same layout in float
  int ints_total = 0, reals_total = 0;
  // canonical fast path: per path, class of the generated program and scale (device copies follow the
  // generic arrays: ints [.. | canon_class3 (w3) | canon_class2 (w2)], reals [.. | canon_scale3 | canon_scale2])
  bool canonical = false;
  int canon_int_off = 0, canon_real_off = 0;
};

namespace cmace {

constexpr int SC_WARPS = 4;

struct PlanView {
  const int32_t *seg3, *seg2, *class3, *class2, *packed3, *packed2;
  int w3, w2, w1, nclass3, nclass2, nterms3, nterms2;
};

template <typename T>
struct RealView {
  const T *scale3, *scale2, *coef3, *coef2;
};

template <typename T, bool BWD>
__global__ void __launch_bounds__(SC_WARPS * 32)
    symcon_kernel(PlanView pv, RealView<T> rv, const T *__restrict__ X,
                  const int32_t *__restrict__ atom_types, const T *__restrict__ W3,
                  const T *__restrict__ W2, const T *__restrict__ W1, const T *__restrict__ gout,
                  int nelements, int64_t nnodes, int C, T *__restrict__ out) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  // layout: [xs: SC_WARPS*16*32 T] [weff: SC_WARPS*(nclass3+nclass2)*32 T] [coef3][coef2] [packed3][packed2][seg3][seg2]
  T *xs_all = reinterpret_cast<T *>(smem_raw);
  const int nq = pv.nclass3 + pv.nclass2;
  T *weff_all = xs_all + SC_WARPS * 16 * 32;
  T *s_coef3 = weff_all + SC_WARPS * nq * 32;
  T *s_coef2 = s_coef3 + pv.nterms3;
  int32_t *s_packed3 = reinterpret_cast<int32_t *>(s_coef2 + pv.nterms2);
  int32_t *s_packed2 = s_packed3 + pv.nterms3;
  int32_t *s_seg3 = s_packed2 + pv.nterms2;
  int32_t *s_seg2 = s_seg3 + 17;

  for (int t = threadIdx.x; t < pv.nterms3; t += blockDim.x) {
    s_coef3[t] = rv.coef3[t];
    s_packed3[t] = pv.packed3[t];
  }
  for (int t = threadIdx.x; t < pv.nterms2; t += blockDim.x) {
    s_coef2[t] = rv.coef2[t];
    s_packed2[t] = pv.packed2[t];
  }
  if (threadIdx.x < 17) {
    s_seg3[threadIdx.x] = pv.seg3[threadIdx.x];
    s_seg2[threadIdx.x] = pv.seg2[threadIdx.x];
  }
  __syncthreads();

  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  T *xs = xs_all + warp * 16 * 32;
  T *weff = weff_all + warp * nq * 32;
  const int nchunks = C / 32;
  const int64_t nitems = nnodes * nchunks;
  const int64_t stride = (int64_t)gridDim.x * SC_WARPS;

  for (int64_t item = (int64_t)blockIdx.x * SC_WARPS + warp; item < nitems; item += stride) {
    const int64_t node = item / nchunks;
    const int c = (int)(item % nchunks) * 32 + lane;
    const int z = atom_types[node];
    const T *xrow = X + node * 16 * C + c;
#pragma unroll
    for (int i = 0; i < 16; i++) xs[i * 32 + lane] = xrow[(int64_t)i * C];
    for (int q = 0; q < nq; q++) weff[q * 32 + lane] = T(0);
    for (int p = 0; p < pv.w3; p++)
      weff[pv.class3[p] * 32 + lane] += rv.scale3[p] * W3[((int64_t)z * pv.w3 + p) * C + c];
    for (int p = 0; p < pv.w2; p++)
      weff[(pv.nclass3 + pv.class2[p]) * 32 + lane] += rv.scale2[p] * W2[((int64_t)z * pv.w2 + p) * C + c];
    const T w1 = W1[(int64_t)z * pv.w1 * C + c];
    T go = T(0);
    if (BWD) go = gout[node * C + c];
    __syncwarp();

    T acc = T(0);
#pragma unroll 1
    for (int i = 0; i < 16; i++) {
      T d3 = T(0), d2 = T(0);
      for (int t = s_seg3[i]; t < s_seg3[i + 1]; t++) {
        const int pk = s_packed3[t];
        d3 = fma(s_coef3[t] * weff[(pk >> 16) * 32 + lane],
                 xs[(pk & 0xff) * 32 + lane] * xs[((pk >> 8) & 0xff) * 32 + lane], d3);
      }
      for (int t = s_seg2[i]; t < s_seg2[i + 1]; t++) {
        const int pk = s_packed2[t];
        d2 = fma(s_coef2[t] * weff[(pv.nclass3 + (pk >> 16)) * 32 + lane], xs[(pk & 0xff) * 32 + lane], d2);
      }
      const T d1 = (i == 0) ? w1 : T(0);
      if (BWD) {
        out[(node * 16 + i) * C + c] = go * (d1 + d2 + d3);
      } else {
        acc = fma(xs[i * 32 + lane], d1 + T(0.5) * d2 + d3 * T(1.0 / 3.0), acc);
      }
    }
    if (!BWD) out[node * C + c] = acc;
    __syncwarp();
  }
}

// ---- generated straight-line path -----------------------------------------------------------
// Used when the caller's tables are the canonical l_max=3 couplings (up to a scale per path).  One thread
// per (node, channel): the node's 16 components, the 12 effective class weights and the 16 gradient
// components stay in registers; the effective weights of every element are combined once per CTA into
// shared memory (each thread its own channel column), then nodes are streamed: 16 coalesced loads in,
// 1 (forward) or 16 (backward) coalesced stores out.  HBM-bound: s*17*N*C bytes forward, s*33*N*C backward.
template <typename T, bool BWD>
__global__ void __launch_bounds__(128)
    symcon_canon_kernel(const int32_t *__restrict__ cclass3, const int32_t *__restrict__ cclass2,
                        const T *__restrict__ cscale3, const T *__restrict__ cscale2, int w3, int w2, int w1,
                        const T *__restrict__ X, const int32_t *__restrict__ atom_types, const T *__restrict__ W3,
                        const T *__restrict__ W2, const T *__restrict__ W1, const T *__restrict__ gout,
                        int nelements, int64_t nnodes, int C, T *__restrict__ out) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  T *weff = reinterpret_cast<T *>(smem_raw);  // [nelements][13][blockDim.x]
  constexpr int NW = canon::NCLASS3 + canon::NCLASS2 + 1;
  const int CH = blockDim.x;
  const int c = blockIdx.y * CH + threadIdx.x;
  for (int z = 0; z < nelements; z++) {
    T acc[NW];
#pragma unroll
    for (int q = 0; q < NW; q++) acc[q] = T(0);
    for (int p = 0; p < w3; p++) {
      const T v = cscale3[p] * W3[((int64_t)z * w3 + p) * C + c];
      const int q = cclass3[p];
#pragma unroll
      for (int u = 0; u < canon::NCLASS3; u++) acc[u] += (u == q) ? v : T(0);
    }
    for (int p = 0; p < w2; p++) {
      const T v = cscale2[p] * W2[((int64_t)z * w2 + p) * C + c];
      const int q = cclass2[p];
#pragma unroll
      for (int u = 0; u < canon::NCLASS2; u++) acc[canon::NCLASS3 + u] += (u == q) ? v : T(0);
    }
    acc[NW - 1] = W1[(int64_t)z * w1 * C + c];
#pragma unroll
    for (int q = 0; q < NW; q++) weff[(z * NW + q) * CH + threadIdx.x] = acc[q];
  }
  // each thread reads back only what it wrote: no barrier needed

  for (int64_t node = blockIdx.x; node < nnodes; node += gridDim.x) {
    const int z = atom_types[node];
    T x[16], g[16], w3r[canon::NCLASS3], w2r[canon::NCLASS2], value;
    const T *xrow = X + node * 16 * C + c;
#pragma unroll
    for (int i = 0; i < 16; i++) x[i] = __ldcs(xrow + (int64_t)i * C);
    const T *wz = weff + (int64_t)z * NW * CH + threadIdx.x;
#pragma unroll
    for (int q = 0; q < canon::NCLASS3; q++) w3r[q] = wz[q * CH];
#pragma unroll
    for (int q = 0; q < canon::NCLASS2; q++) w2r[q] = wz[(canon::NCLASS3 + q) * CH];
    const T w1r = wz[(NW - 1) * CH];
    canon::eval<T>(x, w3r, w2r, w1r, g, value);
    if (BWD) {
      const T go = gout[node * C + c];
      T *orow = out + node * 16 * C + c;
#pragma unroll
      for (int i = 0; i < 16; i++) __stcs(orow + (int64_t)i * C, go * g[i]);
    } else {
      out[node * C + c] = value;
    }
  }
}

}  // namespace cmace

using namespace cmace;

extern "C" {

int cmace_symcon_plan_create(int maxnz, const int16_t *u3_num, const int32_t *u3_idx, const double *u3_val,
                             const int16_t *u2_num, const int16_t *u2_idx, const double *u2_val,
                             int w3, int w2, int w1, cmace_symcon_plan **out_plan) {
  if (!out_plan) return fail(CMACE_ERR_ARG, "cmace_symcon_plan_create: null pointer");
  SymconProgram prog;
  std::string err;
  if (!build_symcon_program(maxnz, u3_num, u3_idx, u3_val, u2_num, u2_idx, u2_val, w3, w2, w1, prog, err))
    return fail(CMACE_ERR_ARG, "cmace_symcon_plan_create: %s", err.c_str());

  cmace_symcon_plan *plan = new cmace_symcon_plan();
  plan->w3 = w3; plan->w2 = w2; plan->w1 = w1;
  plan->nclass3 = prog.nclass3;
  plan->nclass2 = prog.nclass2;
  plan->nterms3 = (int)prog.packed3.size();
  plan->nterms2 = (int)prog.packed2.size();

  std::vector<int32_t> ints;
  ints.insert(ints.end(), prog.seg3.begin(), prog.seg3.end());
  ints.insert(ints.end(), prog.seg2.begin(), prog.seg2.end());
  ints.insert(ints.end(), prog.class3.begin(), prog.class3.end());
  ints.insert(ints.end(), prog.class2.begin(), prog.class2.end());
  ints.insert(ints.end(), prog.packed3.begin(), prog.packed3.end());
  ints.insert(ints.end(), prog.packed2.begin(), prog.packed2.end());
  std::vector<double> reals;
  reals.insert(reals.end(), prog.scale3.begin(), prog.scale3.end());
  reals.insert(reals.end(), prog.scale2.begin(), prog.scale2.end());
  reals.insert(reals.end(), prog.coef3.begin(), prog.coef3.end());
  reals.insert(reals.end(), prog.coef2.begin(), prog.coef2.end());
  plan->canonical = prog.canonical;
  plan->canon_int_off = (int)ints.size();
  plan->canon_real_off = (int)reals.size();
  if (prog.canonical) {
    ints.insert(ints.end(), prog.canon_class3.begin(), prog.canon_class3.end());
    ints.insert(ints.end(), prog.canon_class2.begin(), prog.canon_class2.end());
    reals.insert(reals.end(), prog.canon_scale3.begin(), prog.canon_scale3.end());
    reals.insert(reals.end(), prog.canon_scale2.begin(), prog.canon_scale2.end());
  }
  std::vector<float> reals32(reals.begin(), reals.end());
  plan->ints_total = (int)ints.size();
  plan->reals_total = (int)reals.size();

  cudaError_t e = cudaMalloc(&plan->d_ints, ints.size() * sizeof(int32_t));
  if (e == cudaSuccess) e = cudaMalloc(&plan->d_f64, reals.size() * sizeof(double));
  if (e == cudaSuccess) e = cudaMalloc(&plan->d_f32, reals.size() * sizeof(float));
  if (e == cudaSuccess) e = cudaMemcpy(plan->d_ints, ints.data(), ints.size() * sizeof(int32_t), cudaMemcpyHostToDevice);
  if (e == cudaSuccess) e = cudaMemcpy(plan->d_f64, reals.data(), reals.size() * sizeof(double), cudaMemcpyHostToDevice);
  if (e == cudaSuccess) e = cudaMemcpy(plan->d_f32, reals32.data(), reals32.size() * sizeof(float), cudaMemcpyHostToDevice);
  if (e != cudaSuccess) {
    cmace_symcon_plan_destroy(plan);
    return fail(CMACE_ERR_CUDA, "cmace_symcon_plan_create: %s", cudaGetErrorString(e));
  }
  *out_plan = plan;
  return CMACE_OK;
}

void cmace_symcon_plan_destroy(cmace_symcon_plan *plan) {
  if (!plan) return;
  cudaFree(plan->d_ints);
  cudaFree(plan->d_f64);
  cudaFree(plan->d_f32);
  delete plan;
}

int cmace_symcon_plan_nterms(const cmace_symcon_plan *plan) { return plan ? plan->nterms3 + plan->nterms2 : 0; }
int cmace_symcon_plan_nclasses(const cmace_symcon_plan *plan) { return plan ? plan->nclass3 + plan->nclass2 : 0; }
int cmace_symcon_plan_is_canonical(const cmace_symcon_plan *plan) { return plan && plan->canonical ? 1 : 0; }
}

namespace cmace {

// CMACE_SYMCON_GENERIC=1 in the environment forces the table-driven kernel (tests compare both)
static bool force_generic() {
  const char *e = getenv("CMACE_SYMCON_GENERIC");
  return e != nullptr && e[0] == '1';
}

template <typename T, bool BWD>
static int symcon_launch(const cmace_symcon_plan *plan, const T *X, const int32_t *atom_types, const T *W3,
                         const T *W2, const T *W1, const T *gout, int nelements, int64_t nnodes, int C, T *out,
                         cmace_stream_t stream, const char *what) {
  if (!plan) return fail(CMACE_ERR_ARG, "%s: null plan", what);
  if (nnodes < 0 || nelements < 1) return fail(CMACE_ERR_ARG, "%s: bad size", what);
  if (C <= 0 || C % 32 != 0) return fail(CMACE_ERR_UNSUPPORTED, "%s: channels must be a multiple of 32", what);
  if (nnodes == 0) return CMACE_OK;
  if (!X || !atom_types || !W3 || !W2 || !W1 || !out || (BWD && !gout)) return fail(CMACE_ERR_ARG, "%s: null pointer", what);
  const T *reals = sizeof(T) == 8 ? reinterpret_cast<const T *>(plan->d_f64) : reinterpret_cast<const T *>(plan->d_f32);
  if (plan->canonical && !force_generic()) {
    // channel chunk per CTA: the whole row when C <= 128, else 128-wide chunks
    const int CH = C <= 128 ? C : 128;
    constexpr int NW = canon::NCLASS3 + canon::NCLASS2 + 1;
    const size_t smem = sizeof(T) * (size_t)nelements * NW * CH;
    if (C % CH == 0 && smem <= 160 * 1024) {
      auto kern = symcon_canon_kernel<T, BWD>;
      if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return fail(CMACE_ERR_CUDA, "%s: %s", what, cudaGetErrorString(e));
      }
      int per_sm = (int)((200 * 1024) / (smem + 1024));
      per_sm = per_sm < 1 ? 1 : (per_sm > 12 ? 12 : per_sm);
      int64_t blocks = (int64_t)148 * per_sm;
      if (blocks > nnodes) blocks = nnodes;
      dim3 grid((unsigned)blocks, (unsigned)(C / CH));
      const int32_t *ci = plan->d_ints + plan->canon_int_off;
      const T *cr = reals + plan->canon_real_off;
      kern<<<grid, CH, smem, (cudaStream_t)stream>>>(ci, ci + plan->w3, cr, cr + plan->w3, plan->w3, plan->w2, plan->w1, X,
                                                     atom_types, W3, W2, W1, gout, nelements, nnodes, C, out);
      return check_launch(what);
    }
  }
  PlanView pv;
  const int32_t *ip = plan->d_ints;
  pv.seg3 = ip; ip += 17;
  pv.seg2 = ip; ip += 17;
  pv.class3 = ip; ip += plan->w3;
  pv.class2 = ip; ip += plan->w2;
  pv.packed3 = ip; ip += plan->nterms3;
  pv.packed2 = ip;
  pv.w3 = plan->w3; pv.w2 = plan->w2; pv.w1 = plan->w1;
  pv.nclass3 = plan->nclass3; pv.nclass2 = plan->nclass2;
  pv.nterms3 = plan->nterms3; pv.nterms2 = plan->nterms2;
  RealView<T> rv;
  const T *rp = sizeof(T) == 8 ? reinterpret_cast<const T *>(plan->d_f64) : reinterpret_cast<const T *>(plan->d_f32);
  rv.scale3 = rp; rp += plan->w3;
  rv.scale2 = rp; rp += plan->w2;
  rv.coef3 = rp; rp += plan->nterms3;
  rv.coef2 = rp;
  const size_t smem = sizeof(T) * (size_t)(SC_WARPS * 16 * 32 + SC_WARPS * (pv.nclass3 + pv.nclass2) * 32 +
                                           pv.nterms3 + pv.nterms2) +
                      sizeof(int32_t) * (size_t)(pv.nterms3 + pv.nterms2 + 34);
  if (smem > 200 * 1024) return fail(CMACE_ERR_UNSUPPORTED, "%s: contraction program too large (%zu bytes)", what, smem);
  auto kern = symcon_kernel<T, BWD>;
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return fail(CMACE_ERR_CUDA, "%s: %s", what, cudaGetErrorString(e));
  }
  const int64_t nitems = nnodes * (C / 32);
  int64_t blocks = (nitems + SC_WARPS - 1) / SC_WARPS;
  const int64_t cap = 148 * 16;  // a few waves of resident CTAs; items are strided over the grid
  if (blocks > cap) blocks = cap;
  kern<<<(unsigned)blocks, SC_WARPS * 32, smem, (cudaStream_t)stream>>>(pv, rv, X, atom_types, W3, W2, W1, gout,
                                                                       nelements, nnodes, C, out);
  return check_launch(what);
}

}  // namespace cmace

extern "C" {
int cmace_symcon_fwd_f32(const cmace_symcon_plan *plan, const float *X, const int32_t *atom_types, const float *W3,
                         const float *W2, const float *W1, int nelements, int64_t nnodes, int channels, float *out,
                         cmace_stream_t stream) {
  return symcon_launch<float, false>(plan, X, atom_types, W3, W2, W1, nullptr, nelements, nnodes, channels, out,
                                     stream, "cmace_symcon_fwd");
}
int cmace_symcon_fwd_f64(const cmace_symcon_plan *plan, const double *X, const int32_t *atom_types, const double *W3,
                         const double *W2, const double *W1, int nelements, int64_t nnodes, int channels,
                         double *out, cmace_stream_t stream) {
  return symcon_launch<double, false>(plan, X, atom_types, W3, W2, W1, nullptr, nelements, nnodes, channels, out,
                                      stream, "cmace_symcon_fwd");
}
int cmace_symcon_bwd_f32(const cmace_symcon_plan *plan, const float *X, const int32_t *atom_types, const float *W3,
                         const float *W2, const float *W1, const float *gout, int nelements, int64_t nnodes,
                         int channels, float *gradX, cmace_stream_t stream) {
  return symcon_launch<float, true>(plan, X, atom_types, W3, W2, W1, gout, nelements, nnodes, channels, gradX,
                                    stream, "cmace_symcon_bwd");
}
int cmace_symcon_bwd_f64(const cmace_symcon_plan *plan, const double *X, const int32_t *atom_types, const double *W3,
                         const double *W2, const double *W1, const double *gout, int nelements, int64_t nnodes,
                         int channels, double *gradX, cmace_stream_t stream) {
  return symcon_launch<double, true>(plan, X, atom_types, W3, W2, W1, gout, nelements, nnodes, channels, gradX,
                                     stream, "cmace_symcon_bwd");
}
}
