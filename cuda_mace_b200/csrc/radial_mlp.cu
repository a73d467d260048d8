// Hidden layers of the radial multilayer perceptron in one kernel (float32, tensor cores):
//
//   forward    basis [E, nb]  ->  h3 = silu(silu(silu(basis W1) W2) W3)   [E, 64]
//   backward   grad h3 [E, 64] -> grad basis [E, nb]
//
// (the 1/sqrt(fan_in) factors and the normalisation constant of the activation are folded into the weights by
// the caller).  The activations never leave the SM: a layer's accumulator is read from tensor memory, activated,
// split into the hi / lo TF32 images and written to shared memory as the next layer's A operand.  Every product
// uses the 3-term split  Ahi*Bhi + Ahi*Blo + Alo*Bhi  with the float32 accumulator in tensor memory, three
// tcgen05.mma per K step into the same columns (one tensor-memory load per value in the elementwise phase).
// The forward stores the activation derivatives d_k = silu'(z_k) (three [E, 64] arrays in a tiled layout that
// both kernels access with coalesced 16-byte transfers); the backward is then three products with an
// elementwise factor between them and needs no special-function work.
//
// One CTA per SM, two independent groups of eight warps.  A group works on one 128-edge tile at a time and
// runs its layers one after the other (write A, barrier, one thread issues the MMAs, everybody waits for
// their completion, read the accumulator); while one group waits for the tensor core the other one does
// its elementwise phase.  The weights (80 KB forward, 72 KB backward) are loaded into shared memory once.
// Every mbarrier wait is bounded: on a time-out the group records a code in *status and leaves its loop.
#include <cstring>

#include "common.cuh"
#include "tc_ptx.cuh"

namespace cmace {

constexpr int RH_H = 64;                    // hidden width
constexpr int RH_TILE = 128;                // edges per tile
constexpr int RH_GROUP_THREADS = 256;       // eight warps
constexpr int RH_THREADS = 2 * RH_GROUP_THREADS;
constexpr int RH_A_SLAB = RH_TILE * 128;    // one image (hi or lo) of one 32-column K block: 16 KB
constexpr int RH_A_GROUP = 4 * RH_A_SLAB;   // two K blocks x (hi, lo)
constexpr int RH_W_SMALL = 2 * 64 * 128;    // packed [nb <= 32, 64]: one K block, hi + lo images of 64 rows
constexpr int RH_W_BIG = 2 * RH_W_SMALL;    // packed [64, 64]: two K blocks
constexpr int RH_TMEM_COLS = 128;           // two groups x 64 accumulator columns

struct RadialArgs {
  const float *in;        // forward: basis [E, nb]; backward: grad h3 [E, 64]
  float *out;             // forward: h3 [E, 64]; backward: grad basis [E, nb]
  float4 *dsave;          // [tiles][3][16][128] float4: activation derivatives
  const float *w[3];      // packed weights in the order the kernel uses them
  int32_t *status;
  int64_t E;
  int nb;
  int npad_last;          // backward: rows per image of the last packed matrix
};

__device__ __forceinline__ void group_sync(int group) {
  asm volatile("bar.sync %0, %1;" ::"r"(group + 1), "r"(RH_GROUP_THREADS) : "memory");
}

__device__ __forceinline__ void tmem_ld8(uint32_t taddr, uint32_t (&r)[8]) {
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
               : "r"(taddr)
               : "memory");
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// One layer's products for a 128-row tile: A images at sA (per K block: hi slab, lo slab), packed weights at sB
// (per K block: hi image then lo image of npad rows).  The three terms Ahi*Bhi + Ahi*Blo + Alo*Bhi accumulate into
// the same npad columns, so the elementwise phase reads each value once and needs no addition.
__device__ __forceinline__ void issue_layer(uint32_t d_tmem, uint32_t sA, uint32_t sB, int K, int npad) {
  const uint32_t idesc = umma_idesc_tf32(RH_TILE, npad);
  const uint32_t b_image = (uint32_t)npad * 128u, b_block = 2u * b_image;
  for (int k0 = 0, kb = 0; k0 < K; k0 += 32, kb++) {
    const uint64_t a_hi = umma_desc_sw128(sA + kb * 2 * RH_A_SLAB);
    const uint64_t a_lo = umma_desc_sw128(sA + kb * 2 * RH_A_SLAB + RH_A_SLAB);
    const uint64_t b_hi = umma_desc_sw128(sB + kb * b_block);
    const uint64_t b_lo = umma_desc_sw128(sB + kb * b_block + b_image);
    int ksteps = (K - k0) / 8;
    ksteps = ksteps > 4 ? 4 : ksteps;
    for (int j = 0; j < ksteps; j++) {
      // K step j starts 32 bytes = 2 address units further into every row
      umma_tf32(d_tmem, a_hi + (uint64_t)(2 * j), b_hi + (uint64_t)(2 * j), idesc, (kb | j) != 0);
      umma_tf32_acc(d_tmem, a_hi + (uint64_t)(2 * j), b_lo + (uint64_t)(2 * j), idesc);
      umma_tf32_acc(d_tmem, a_lo + (uint64_t)(2 * j), b_hi + (uint64_t)(2 * j), idesc);
    }
  }
}

__device__ __forceinline__ void store_split(uint32_t s_hi, float4 a) {
  // raw values are the hi image (the tensor core ignores the low 13 mantissa bits), lo = tf32(a - trunc(a))
  float4 lo;
  lo.x = to_tf32(a.x - __uint_as_float(__float_as_uint(a.x) & 0xFFFFE000u));
  lo.y = to_tf32(a.y - __uint_as_float(__float_as_uint(a.y) & 0xFFFFE000u));
  lo.z = to_tf32(a.z - __uint_as_float(__float_as_uint(a.z) & 0xFFFFE000u));
  lo.w = to_tf32(a.w - __uint_as_float(__float_as_uint(a.w) & 0xFFFFE000u));
  asm volatile("st.shared.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(s_hi), "f"(a.x), "f"(a.y), "f"(a.z), "f"(a.w) : "memory");
  asm volatile("st.shared.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(s_hi + RH_A_SLAB), "f"(lo.x), "f"(lo.y), "f"(lo.z),
               "f"(lo.w)
               : "memory");
}

__device__ __forceinline__ void l2_prefetch(const void *p, uint32_t bytes) {
  asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(p), "r"(bytes) : "memory");
}

__device__ __forceinline__ void silu_both(float z, float &a, float &d) {
  const float s = sigmoid_fast(z);
  a = z * s;
  d = s * fmaf(z, 1.0f - s, 1.0f);
}

template <bool BACKWARD>
__global__ void __launch_bounds__(RH_THREADS, 1) radial_hidden_kernel(const RadialArgs g) {
  extern __shared__ __align__(1024) unsigned char smem[];
  __shared__ __align__(8) uint64_t bars[3];
  __shared__ uint32_t tmem_base_slot;

  const uint32_t smem_base = (smem_u32(smem) + 1023u) & ~1023u;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int group = warp >> 3, gw = warp & 7, gtid = tid & (RH_GROUP_THREADS - 1);
  const uint32_t wbar = smem_u32(&bars[0]);
  const uint32_t mma_bar = smem_u32(&bars[1 + group]);

  // weights: forward W1 (one K block), W2, W3; backward W3^T, W2^T, W1^T (narrow)
  const uint32_t w_bytes[3] = {BACKWARD ? (uint32_t)RH_W_BIG : (uint32_t)RH_W_SMALL, (uint32_t)RH_W_BIG,
                               BACKWARD ? 2u * 2u * (uint32_t)g.npad_last * 128u : (uint32_t)RH_W_BIG};
  const uint32_t sW[3] = {smem_base, smem_base + w_bytes[0], smem_base + w_bytes[0] + w_bytes[1]};
  const uint32_t sA = smem_base + w_bytes[0] + w_bytes[1] + w_bytes[2] + group * RH_A_GROUP;

  if (tid == 0) {
    mbar_init(wbar, 1);
    mbar_init(wbar + 8, 1);
    mbar_init(wbar + 16, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 0) tmem_alloc(smem_u32(&tmem_base_slot), RH_TMEM_COLS);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_acc = tmem_base_slot + group * RH_H;

  if (tid == 0) {
    mbar_arrive_expect_tx(wbar, w_bytes[0] + w_bytes[1] + w_bytes[2]);
    for (int i = 0; i < 3; i++)
      for (uint32_t off = 0; off < w_bytes[i]; off += 8192u) {
        const uint32_t n = w_bytes[i] - off < 8192u ? w_bytes[i] - off : 8192u;
        bulk_copy_g2s(sW[i] + off, reinterpret_cast<const unsigned char *>(g.w[i]) + off, n, wbar);
      }
  }
  bool ok = warp_wait(wbar, 0, lane);
  if (!ok && lane == 0 && g.status) atomicCAS(g.status, 0, 11);

  const int q = gw & 3, h = gw >> 2;      // tensor-memory lane quarter, column half (= K block of the next layer)
  const int r = q * 32 + lane;            // row of the tile this thread owns in the elementwise phases
  const uint32_t t_row = tmem_acc + ((uint32_t)(q * 32) << 16);
  const uint32_t a_row = sA + h * 2 * RH_A_SLAB;   // hi slab of K block h
  uint32_t phase = 0;
  const int64_t ntiles = (g.E + RH_TILE - 1) / RH_TILE;
  const int nchunks = g.nb / 4;           // 16-byte chunks per row of the basis

  // one layer = start_layer (barrier, MMAs issued by one thread) ... finish_layer (wait for them); whatever is
  // placed between the two overlaps with the tensor core: the global loads of the next elementwise phase
  auto start_layer = [&](uint32_t sB, int K, int npad) {
    tc_fence_before();
    fence_proxy_async();
    group_sync(group);
    if (gtid == 0) {
      tc_fence_after();
      issue_layer(tmem_acc, sA, sB, K, npad);
      umma_commit(mma_bar);
    }
  };
  auto finish_layer = [&]() -> bool {
    const bool got = warp_wait(mma_bar, phase, lane);
    phase ^= 1;
    tc_fence_after();
    return got;
  };
  const int64_t tile_step = (int64_t)gridDim.x * 2;
  int64_t tile = (int64_t)blockIdx.x * 2 + group;

  if (!BACKWARD) {
    // the basis rows of a tile: one or two 16-byte chunks per thread, fetched one tile ahead
    float4 pre[4];
    auto load_basis = [&](int64_t t) {
#pragma unroll
      for (int i = 0; i < 4; i++) {
        const int idx = gtid + RH_GROUP_THREADS * i;
        const int rr = idx / nchunks, c = idx - rr * nchunks;
        const int64_t ee = t * RH_TILE + rr;
        pre[i] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (t < ntiles && rr < RH_TILE && ee < g.E) pre[i] = __ldg(reinterpret_cast<const float4 *>(g.in + ee * g.nb) + c);
      }
    };
    load_basis(tile);
    for (; ok && tile < ntiles; tile += tile_step) {
      const int64_t e = tile * RH_TILE + r;
      const bool row_ok = e < g.E;
      float4 *dtile = g.dsave + (tile * 3) * 16 * RH_TILE + (h * 8) * RH_TILE + r;   // + (layer*16 + chunk)*128
      // ---- layer 1 operand: the basis rows, raw + residual images, K block 0
#pragma unroll
      for (int i = 0; i < 4; i++) {
        const int idx = gtid + RH_GROUP_THREADS * i;
        const int rr = idx / nchunks, c = idx - rr * nchunks;
        if (rr < RH_TILE) store_split(sA + (uint32_t)sw128_offset(rr, c), pre[i]);
      }
      start_layer(sW[0], g.nb, RH_H);
      load_basis(tile + tile_step);
      if (!(ok = finish_layer())) break;
      for (int layer = 0; layer < 3; layer++) {
uint32_t v[32];
        tmem_ld32_nowait(t_row + 32 * h, v);
        tmem_ld_wait();
#pragma unroll
        for (int c = 0; c < 8; c++) {
          float4 a, d;
          silu_both(__uint_as_float(v[4 * c]), a.x, d.x);
          silu_both(__uint_as_float(v[4 * c + 1]), a.y, d.y);
          silu_both(__uint_as_float(v[4 * c + 2]), a.z, d.z);
          silu_both(__uint_as_float(v[4 * c + 3]), a.w, d.w);
          if (layer < 2)
            store_split(a_row + (uint32_t)sw128_offset(r, c), a);
          else if (row_ok)
            *reinterpret_cast<float4 *>(g.out + e * RH_H + 32 * h + 4 * c) = a;
          if (g.dsave != nullptr) dtile[(layer * 16 + c) * RH_TILE] = d;
        }
        if (layer < 2) {
          start_layer(sW[layer + 1], RH_H, RH_H);
          if (!(ok = finish_layer())) break;
        }
      }
    }
  } else {
    // grad h3 and d3 of a tile are fetched while the previous tile's last product runs; d2 and d1 while the
    // product that precedes their use runs
    float4 pg[8], pd[8];
    auto load_first = [&](int64_t t) {
      const int64_t e = t * RH_TILE + r;
      const float4 *dt = g.dsave + (t * 3 + 2) * 16 * RH_TILE + (h * 8) * RH_TILE + r;
#pragma unroll
      for (int c = 0; c < 8; c++) {
        pg[c] = make_float4(0.f, 0.f, 0.f, 0.f);
        pd[c] = pg[c];
        if (t < ntiles) {
          if (e < g.E) pg[c] = __ldg(reinterpret_cast<const float4 *>(g.in + e * RH_H + 32 * h) + c);
          pd[c] = dt[c * RH_TILE];
        }
      }
    };
    load_first(tile);
    for (; ok && tile < ntiles; tile += tile_step) {
      const int64_t e = tile * RH_TILE + r;
      const bool row_ok = e < g.E;
      const float4 *dtile = g.dsave + (tile * 3) * 16 * RH_TILE + (h * 8) * RH_TILE + r;
      // The phases of a tile wait one after the other for their operands, so HBM latency adds up three times per
      // tile; pulling the group's next tile (96 KB of derivatives, 32 KB of gradient rows, both contiguous) into L2
      // a whole tile ahead shortens every one of those waits.
      if (gtid == 0 && tile + tile_step < ntiles) {   // (two tiles ahead measured slower)
        const int64_t tn = tile + tile_step;
        const char *dsrc = reinterpret_cast<const char *>(g.dsave + tn * 3 * 16 * RH_TILE);
        for (int off = 0; off < 3 * 16 * RH_TILE * 16; off += 32768) l2_prefetch(dsrc + off, 32768);
        const int64_t rows = g.E - tn * RH_TILE < RH_TILE ? g.E - tn * RH_TILE : RH_TILE;
        l2_prefetch(reinterpret_cast<const char *>(g.in + tn * RH_TILE * RH_H), (uint32_t)(rows * RH_H * 4));
      }
      // ---- grad z3 = grad h3 * d3
#pragma unroll
      for (int c = 0; c < 8; c++)
        store_split(a_row + (uint32_t)sw128_offset(r, c),
                    make_float4(pg[c].x * pd[c].x, pg[c].y * pd[c].y, pg[c].z * pd[c].z, pg[c].w * pd[c].w));
      start_layer(sW[0], RH_H, RH_H);
#pragma unroll
      for (int c = 0; c < 8; c++) pd[c] = dtile[(16 + c) * RH_TILE];        // d2
      if (!(ok = finish_layer())) break;
      for (int layer = 1; layer >= 0; layer--) {
uint32_t v[32];
        tmem_ld32_nowait(t_row + 32 * h, v);
        tmem_ld_wait();
#pragma unroll
        for (int c = 0; c < 8; c++) {
          const float4 d = pd[c];
          store_split(a_row + (uint32_t)sw128_offset(r, c),
                      make_float4(__uint_as_float(v[4 * c]) * d.x, __uint_as_float(v[4 * c + 1]) * d.y,
                                  __uint_as_float(v[4 * c + 2]) * d.z, __uint_as_float(v[4 * c + 3]) * d.w));
        }
        start_layer(sW[2 - layer], RH_H, layer == 0 ? g.npad_last : RH_H);
        if (layer == 1) {
#pragma unroll
          for (int c = 0; c < 8; c++) pd[c] = dtile[c * RH_TILE];            // d1
        } else {
          load_first(tile + tile_step);
        }
        if (!(ok = finish_layer())) break;
      }
      if (!ok) break;
      // ---- grad basis: columns [0, nb) of the accumulator
      if (h == 0) {
        for (int c0 = 0; c0 < g.nb; c0 += 8) {
          uint32_t v[8];
          tmem_ld8(t_row + c0, v);
          if (row_ok) {
            float *o = g.out + e * g.nb + c0;
            *reinterpret_cast<float4 *>(o) = make_float4(__uint_as_float(v[0]), __uint_as_float(v[1]),
                                                         __uint_as_float(v[2]), __uint_as_float(v[3]));
            *reinterpret_cast<float4 *>(o + 4) = make_float4(__uint_as_float(v[4]), __uint_as_float(v[5]),
                                                             __uint_as_float(v[6]), __uint_as_float(v[7]));
          }
        }
      }
    }
  }
  if (!ok && lane == 0 && g.status) atomicCAS(g.status, 0, 12);

  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem_base_slot, RH_TMEM_COLS);
}

static int radial_launch(RadialArgs &g, bool backward, const char *what, cudaStream_t st) {
  static int num_sms = 0;
  if (num_sms == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&num_sms, cudaDevAttrMultiProcessorCount, dev);
    if (num_sms <= 0) num_sms = 148;
  }
  const size_t w_total = backward ? (size_t)2 * RH_W_BIG + (size_t)4 * g.npad_last * 128 : (size_t)RH_W_SMALL + 2 * RH_W_BIG;
  const size_t smem = w_total + 2 * (size_t)RH_A_GROUP + 1024;
  auto kern = backward ? radial_hidden_kernel<true> : radial_hidden_kernel<false>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return fail(CMACE_ERR_CUDA, "%s: %s", what, cudaGetErrorString(e));
  const int64_t ntiles = (g.E + RH_TILE - 1) / RH_TILE;
  int64_t blocks = (ntiles + 1) / 2;
  blocks = blocks < num_sms ? blocks : num_sms;
  kern<<<(unsigned)blocks, RH_THREADS, smem, st>>>(g);
  return check_launch(what);
}

}  // namespace cmace

using namespace cmace;

extern "C" {

int64_t cmace_radial_hidden_saved_floats(int64_t nedges) {
  if (nedges < 0) return 0;
  return ((nedges + RH_TILE - 1) / RH_TILE) * 3 * RH_H * RH_TILE;
}

int cmace_radial_hidden_fwd_f32(const float *basis, int nb, const float *packed_w1, const float *packed_w2,
                                const float *packed_w3, int64_t nedges, float *h3, float *saved, int32_t *status,
                                cmace_stream_t stream) {
  if (nedges < 0 || nb < 8 || nb > 32 || nb % 8 != 0)
    return fail(CMACE_ERR_UNSUPPORTED, "cmace_radial_hidden_fwd: the basis size must be 8, 16, 24 or 32");
  if (nedges == 0) return CMACE_OK;
  if (!basis || !packed_w1 || !packed_w2 || !packed_w3 || !h3)
    return fail(CMACE_ERR_ARG, "cmace_radial_hidden_fwd: null pointer");
  if (!aligned16(basis) || !aligned16(packed_w1) || !aligned16(packed_w2) || !aligned16(packed_w3) || !aligned16(h3) ||
      !aligned16(saved))
    return fail(CMACE_ERR_ARG, "cmace_radial_hidden_fwd: pointers must be 16-byte aligned");
  RadialArgs g{};
  g.in = basis; g.out = h3; g.dsave = reinterpret_cast<float4 *>(saved);
  g.w[0] = packed_w1; g.w[1] = packed_w2; g.w[2] = packed_w3;
  g.status = status; g.E = nedges; g.nb = nb; g.npad_last = RH_H;
  return radial_launch(g, false, "cmace_radial_hidden_fwd", (cudaStream_t)stream);
}

int cmace_radial_hidden_bwd_f32(const float *grad_h3, const float *saved, const float *packed_w3t,
                                const float *packed_w2t, const float *packed_w1t, int nb, int64_t nedges,
                                float *grad_basis, int32_t *status, cmace_stream_t stream) {
  if (nedges < 0 || nb < 8 || nb > 32 || nb % 8 != 0)
    return fail(CMACE_ERR_UNSUPPORTED, "cmace_radial_hidden_bwd: the basis size must be 8, 16, 24 or 32");
  if (nedges == 0) return CMACE_OK;
  if (!grad_h3 || !saved || !packed_w3t || !packed_w2t || !packed_w1t || !grad_basis)
    return fail(CMACE_ERR_ARG, "cmace_radial_hidden_bwd: null pointer");
  if (!aligned16(grad_h3) || !aligned16(saved) || !aligned16(packed_w3t) || !aligned16(packed_w2t) ||
      !aligned16(packed_w1t) || !aligned16(grad_basis))
    return fail(CMACE_ERR_ARG, "cmace_radial_hidden_bwd: pointers must be 16-byte aligned");
  RadialArgs g{};
  g.in = grad_h3; g.out = grad_basis; g.dsave = reinterpret_cast<float4 *>(const_cast<float *>(saved));
  g.w[0] = packed_w3t; g.w[1] = packed_w2t; g.w[2] = packed_w1t;
  g.status = status; g.E = nedges; g.nb = nb; g.npad_last = (nb + 15) & ~15;
  return radial_launch(g, true, "cmace_radial_hidden_bwd", (cudaStream_t)stream);
}
}
