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
#include <cstdlib>

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
        if (gradR != nullptr) store_vec_stream<T, VEC>(gradR + (ee * 4 + l) * C + c0, gr);
      }
      if (Tout != nullptr) store_vec<T, VEC>(Tout + ee * C + c0, t);
      const T tot = warp_reduce16(p, lane);
      if ((lane & 1) == 0) gy[(int64_t)(lane >> 1) * nedges + ee] = tot;
    }
  }
}

// ---- edge pass with the R rows staged through shared memory (float32, 128 channels) -------------------------
// The kernel above keeps the loads of one pair of edges in flight per warp, and the register budget allows 12
// warps per SM: about 48 KB in flight, not enough to cover HBM latency at full bandwidth.  Here every warp owns a
// ring of BS_SLOTS shared-memory slots; one lane starts, BS_SLOTS edges ahead of where the warp computes, a bulk
// copy of the edge's four R rows (2 KB, contiguous) and of its sender's feature row (512 B) that completes on the
// slot's mbarrier.  160 KB per SM are then on their way from HBM at any time, independent of registers.
// The arithmetic per edge is that of imp_bwd_edge_kernel.  Everything this pass writes is per edge (gradY, T, gradR),
// so the edge list is cut into equal contiguous pieces, one per warp of a persistent grid, wherever the receiver
// boundaries fall (a warp reloads G when its edges move on to the next receiver): the warps finish together
// whatever the degrees are, which matters most for small systems (3 000 atoms: 2 368 warps, 0.139 -> 0.10 ms).
// Every wait is bounded and sets *stalled when it gives up.  Measured at 64 000 atoms: 3.36 ms with
// the register-prefetch kernel, 3.38 ms with 8 warps x 8 slots (two warps per scheduler cannot hide the latency of
// their own instruction chains), 3.06 ms with 16 warps x 4 slots, 3.22 ms with 16 x 5 (the modulo by 5).
constexpr int BS_WARPS = 16;
constexpr int BS_SLOTS = 4;
constexpr int BS_C = 128;
constexpr int BS_R_BYTES = 4 * BS_C * 4;
constexpr int BS_SLOT_BYTES = BS_R_BYTES + BS_C * 4;
constexpr long long BS_TIMEOUT_CYCLES = 400000000LL;   // bound of every wait, about 0.2 s

// position in a warp's piece [e, end) of the receiver-sorted edge list: edge e belongs to receiver `node`, whose
// edges end at e1; e = -1 when the piece is exhausted
struct EdgeCursor {
  int64_t node, e, e1, end;
};

// first = first edge of the piece: the receiver is found by bisection in row_ptr [nnodes + 1]
__device__ __forceinline__ void cursor_start(EdgeCursor &c, const int32_t *__restrict__ row_ptr, int64_t nnodes,
                                             int64_t first, int64_t end) {
  c.end = end;
  if (first >= end) {
    c.e = c.e1 = -1;
    c.node = 0;
    return;
  }
  int64_t lo = 0, hi = nnodes;   // invariant: row_ptr[lo] <= first < row_ptr[hi]
  while (hi - lo > 1) {
    const int64_t mid = (lo + hi) >> 1;
    if (row_ptr[mid] <= first) lo = mid;
    else hi = mid;
  }
  c.node = lo;
  c.e = first;
  c.e1 = row_ptr[lo + 1];
}
__device__ __forceinline__ void cursor_next(EdgeCursor &c, const int32_t *__restrict__ row_ptr) {
  if (++c.e >= c.end) {
    c.e = -1;
    return;
  }
  while (c.e >= c.e1) c.e1 = row_ptr[++c.node + 1];   // receivers without edges are stepped over
}

// WANT_T / WANT_GR: whether T [E,C] and gradR [E,4,C] are written.  With neither (the first layer of a model whose
// radial gradient is formed inside the GEMM) u[l,c] is not needed at all, and Y is not read: gradY does not depend
// on it.
template <bool WANT_T, bool WANT_GR>
__global__ void __launch_bounds__(BS_WARPS * 32, 1)
    imp_bwd_edge_staged_kernel(const float *__restrict__ X, const float *__restrict__ Y, const float *__restrict__ R,
                               const float *__restrict__ G, const int32_t *__restrict__ sender,
                               const int32_t *__restrict__ row_ptr, int64_t nnodes, int64_t nedges,
                               float *__restrict__ gradR, float *__restrict__ gy, float *__restrict__ Tout,
                               int *__restrict__ stalled) {
  extern __shared__ __align__(128) unsigned char bs_smem[];
  __shared__ __align__(8) uint64_t bs_bars[BS_WARPS][BS_SLOTS];
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
  const uint32_t ring = (uint32_t)__cvta_generic_to_shared(bs_smem) + (uint32_t)w * BS_SLOTS * BS_SLOT_BYTES;
  const uint32_t bar0 = (uint32_t)__cvta_generic_to_shared(&bs_bars[w][0]);
  if (lane == 0) {
    for (int s = 0; s < BS_SLOTS; s++)
      asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar0 + 8 * s), "r"(1));
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncwarp();

  const int64_t nwarps = (int64_t)gridDim.x * BS_WARPS, wid = (int64_t)blockIdx.x * BS_WARPS + w;
  const int64_t per = (nedges + nwarps - 1) / nwarps;
  const int64_t e_first = wid * per, e_end = e_first + per < nedges ? e_first + per : nedges;
  EdgeCursor ic, cc;   // where copies are issued, where the warp computes
  cursor_start(ic, row_ptr, nnodes, e_first, e_end);
  cc = ic;
  int64_t chunk_base = -64;
  int snd = 0;
  uint32_t icount = 0, ccount = 0;

  auto issue_one = [&]() {
    if (ic.e < 0) return;
    // sender indices of the issue stream, 32 at a time
    if (ic.e >= chunk_base + 32) {
      chunk_base = ic.e;
      snd = (ic.e + lane < ic.end) ? sender[ic.e + lane] : 0;
    }
    const int s = __shfl_sync(0xffffffffu, snd, (int)(ic.e - chunk_base));
    if (lane == 0) {
      const uint32_t slot = ring + (icount % BS_SLOTS) * BS_SLOT_BYTES, bar = bar0 + 8 * (icount % BS_SLOTS);
      asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(BS_SLOT_BYTES) : "memory");
      asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(slot),
                   "l"(R + ic.e * (4 * BS_C)), "r"(BS_R_BYTES), "r"(bar)
                   : "memory");
      asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                       slot + BS_R_BYTES),
                   "l"(X + (int64_t)s * BS_C), "r"(BS_C * 4), "r"(bar)
                   : "memory");
    }
    icount++;
    cursor_next(ic, row_ptr);
  };
  for (int i = 0; i < BS_SLOTS; i++) issue_one();

  const int c0 = lane * 4;
  const int ylm = lane & 15;
  constexpr bool WANT_U = WANT_T || WANT_GR;
  unsigned long long g2[16][2];   // G[node, m, c0 .. c0 + 3] as two register pairs
  int64_t g_node = -1;
  float yv_next = (WANT_U && cc.e >= 0) ? __ldg(Y + (int64_t)ylm * nedges + cc.e) : 0.f;
  while (cc.e >= 0) {
    const int64_t e = cc.e, node = cc.node;
    EdgeCursor nc = cc;
    cursor_next(nc, row_ptr);
    const float yv = yv_next;
    if (WANT_U && nc.e >= 0) yv_next = __ldg(Y + (int64_t)ylm * nedges + nc.e);
    if (node != g_node) {
      g_node = node;
#pragma unroll
      for (int m = 0; m < 16; m++) {
        const ulonglong2 v = __ldg(reinterpret_cast<const ulonglong2 *>(G + (node * 16 + m) * BS_C + c0));
        g2[m][0] = v.x;
        g2[m][1] = v.y;
      }
    }
    // wait for the edge's slot
    const uint32_t slot = ring + (ccount % BS_SLOTS) * BS_SLOT_BYTES, bar = bar0 + 8 * (ccount % BS_SLOTS);
    const uint32_t parity = (ccount / BS_SLOTS) & 1u;
    {
      uint32_t ok = 0;
      const long long t0 = clock64();
      for (;;) {
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(ok)
            : "r"(bar), "r"(parity)
            : "memory");
        if (ok || clock64() - t0 > BS_TIMEOUT_CYCLES) break;
      }
      if (!__all_sync(0xffffffffu, ok != 0)) {
        // Give up on this warp's receivers, but not before the copies it still has in flight have landed: they
        // target this CTA's shared memory, which must stay allocated until they complete.  Slots ccount + 1 ..
        // icount - 1 are outstanding; each gets one more bounded wait.
        if (lane == 0 && stalled) atomicExch(stalled, 1);
        for (uint32_t k = ccount + 1; k < icount; k++) {
          const uint32_t kbar = bar0 + 8 * (k % BS_SLOTS), kpar = (k / BS_SLOTS) & 1u;
          uint32_t done = 0;
          const long long t1 = clock64();
          do {
            asm volatile(
                "{\n\t.reg .pred p;\n\t"
                "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
                "selp.u32 %0, 1, 0, p;\n\t}"
                : "=r"(done)
                : "r"(kbar), "r"(kpar)
                : "memory");
          } while (!done && clock64() - t1 < BS_TIMEOUT_CYCLES);
        }
        break;
      }
    }
    unsigned long long x2[2], r2[4][2], rx2[4][2];
    asm volatile("ld.shared.v2.b64 {%0, %1}, [%2];" : "=l"(x2[0]), "=l"(x2[1]) : "r"(slot + BS_R_BYTES + lane * 16));
#pragma unroll
    for (int l = 0; l < 4; l++) {
      asm volatile("ld.shared.v2.b64 {%0, %1}, [%2];"
                   : "=l"(r2[l][0]), "=l"(r2[l][1])
                   : "r"(slot + l * (BS_C * 4) + lane * 16));
      rx2[l][0] = mul2(r2[l][0], x2[0]);
      rx2[l][1] = mul2(r2[l][1], x2[1]);
    }
    unsigned long long u2[4][2];
    float p[16];
#pragma unroll
    for (int l = 0; l < 4; l++) u2[l][0] = u2[l][1] = 0ull;
#pragma unroll
    for (int m = 0; m < 16; m++) {
      const int l = l_of_lm(m);
      if (WANT_U) {
        const float y = __shfl_sync(0xffffffffu, yv, m);
        const unsigned long long yy = pack2(y, y);
        u2[l][0] = fma2(yy, g2[m][0], u2[l][0]);
        u2[l][1] = fma2(yy, g2[m][1], u2[l][1]);
      }
      const unsigned long long pm = fma2(g2[m][1], rx2[l][1], mul2(g2[m][0], rx2[l][0]));
      float pa, pb;
      unpack2(pm, pa, pb);
      p[m] = pa + pb;
    }
    float t[4] = {0.f, 0.f, 0.f, 0.f};
    if (WANT_T) {
      unsigned long long t2[2] = {0ull, 0ull};
#pragma unroll
      for (int l = 0; l < 4; l++) {
        t2[0] = fma2(u2[l][0], r2[l][0], t2[0]);
        t2[1] = fma2(u2[l][1], r2[l][1], t2[1]);
      }
      unpack2(t2[0], t[0], t[1]);
      unpack2(t2[1], t[2], t[3]);
    }
    if (WANT_GR) {
#pragma unroll
      for (int l = 0; l < 4; l++) {
        float gr[4];
        unpack2(mul2(x2[0], u2[l][0]), gr[0], gr[1]);
        unpack2(mul2(x2[1], u2[l][1]), gr[2], gr[3]);
        store_vec_stream<float, 4>(gradR + (e * 4 + l) * BS_C + c0, gr);
      }
    }
    // every value read from the slot has been consumed by now: the next copy may go into it
    __syncwarp();
    ccount++;
    issue_one();
    if (WANT_T) store_vec<float, 4>(Tout + e * BS_C + c0, t);
    const float tot = warp_reduce16(p, lane);
    if ((lane & 1) == 0) gy[(int64_t)(lane >> 1) * nedges + e] = tot;
    cc = nc;
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

static __device__ int g_staged_stall;   // set when a bounded wait of the staged edge pass gave up
static int *staged_stall_flag() {
  static int *per_device[64] = {nullptr};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
  if (per_device[dev] == nullptr) {
    int *p = nullptr;
    if (cudaGetSymbolAddress(reinterpret_cast<void **>(&p), g_staged_stall) == cudaSuccess) per_device[dev] = p;
  }
  return per_device[dev];
}

template <typename T>
static int imp_bwd_edge(const T *X, const T *Y, const T *R, const T *G, const int32_t *sender,
                        const int32_t *row_ptr, int64_t nnodes, int64_t nedges, int C, T *gradR,
                        T *gradY, T *Tout, T *partial, cmace_stream_t stream) {
  int rc = check_common<T>(X, R, G, nnodes, nedges, C, "cmace_imp_bwd_edge");
  if (rc) return rc;
  if (nnodes == 0 || nedges == 0) return CMACE_OK;
  if (!X || !Y || !R || !G || !sender || !row_ptr || !gradY)
    return fail(CMACE_ERR_ARG, "cmace_imp_bwd_edge: null pointer");
  if ((gradR && !aligned16(gradR)) || (Tout && !aligned16(Tout)))
    return fail(CMACE_ERR_ARG, "cmace_imp_bwd_edge: outputs must be 16-byte aligned");
  const int vec = pick_vec<T>(C);
  const int nchunks = C / (32 * vec);
  if (nchunks > 1 && !partial)
    return fail(CMACE_ERR_ARG, "cmace_imp_bwd_edge: gradY_partial scratch required for %d chunks", nchunks);
  T *gy = nchunks > 1 ? partial : gradY;
  cudaStream_t st = (cudaStream_t)stream;
  if constexpr (sizeof(T) == 4) {
    if (C == BS_C && aligned16(R) && aligned16(X) && aligned16(G)) {
      static int num_sms = 0;
      if (num_sms == 0) {
        int dev = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&num_sms, cudaDevAttrMultiProcessorCount, dev);
        if (num_sms <= 0) num_sms = 148;
      }
      const size_t smem = (size_t)BS_WARPS * BS_SLOTS * BS_SLOT_BYTES;
      int64_t blocks = (nedges + BS_WARPS * 8 - 1) / (BS_WARPS * 8);   // at least a few edges a warp
      blocks = blocks < num_sms ? blocks : num_sms;
      auto launch = [&](auto kernel) -> int {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return fail(CMACE_ERR_CUDA, "cmace_imp_bwd_edge: %s", cudaGetErrorString(e));
        kernel<<<(unsigned)blocks, BS_WARPS * 32, smem, st>>>(X, Y, R, G, sender, row_ptr, nnodes, nedges, gradR, gy,
                                                              Tout, staged_stall_flag());
        return check_launch("cmace_imp_bwd_edge");
      };
      if (Tout && gradR) return launch(imp_bwd_edge_staged_kernel<true, true>);
      if (Tout) return launch(imp_bwd_edge_staged_kernel<true, false>);
      if (gradR) return launch(imp_bwd_edge_staged_kernel<false, true>);
      return launch(imp_bwd_edge_staged_kernel<false, false>);
    }
  }
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

int cmace_imp_staged_stalled(void) {
  int *flag = staged_stall_flag();
  int v = 0;
  if (flag == nullptr) return 0;
  if (cudaMemcpy(&v, flag, sizeof(int), cudaMemcpyDeviceToHost) != cudaSuccess) return -1;
  if (v != 0) cudaMemset(flag, 0, sizeof(int));
  return v;
}

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
