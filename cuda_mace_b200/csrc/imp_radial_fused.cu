// Message passing with the last (linear) layer of the radial perceptron computed on the fly (float32):
//
//   R[e, l, c]     = sum_k H[e, k] * W[k, l*C + c]                     H [E, K]: last hidden activations
//   out[i, lm, c]  = sum_{e : receiver(e) = i} X[sender(e), c] * Y[lm, e] * R[e, l(lm), c]
//
// The product runs on the tensor cores with the roles of the operands swapped with respect to a plain GEMM:
// the weight rows (l, c) are the M side and the 128 edges of a tile the N side, so the accumulator in tensor
// memory has the channels on its lanes and the edges on its columns.  That is exactly the layout the
// scatter-sum wants: a thread owns one (l, channel), reads R for consecutive edges straight from tensor
// memory, multiplies with the sender's feature (a coalesced 128-byte row piece per warp and edge) and the
// harmonics, and accumulates the 2l+1 outputs of the current receiver in registers.  R only goes to HBM when
// the caller asks for it (the backward pass reads it); the forward never reads it back.
//
// A CTA owns 32 channels (a "channel quarter" at C = 128) of all four l, i.e. 128 weight rows whose hi / lo
// TF32 images (64 KB at K = 64) stay in shared memory for the whole kernel.  Two groups of sixteen warps each
// work on one 128-edge tile at a time: write the tile's H images, one thread issues the MMAs
// (3-term split accumulated in place, three instructions per K step), the harmonics and edge indices of the tile
// are staged while the tensor core works, then every warp consumes its lane quarter (= its l) for a quarter of
// the edges.  While one group waits for the tensor core the other one is in its scatter phase.
// Partial sums of a receiver whose edges straddle warps, tiles or CTAs are combined with float atomics on
// the zero-filled output, so the result is reproducible to rounding, not bit for bit.
// Every mbarrier wait is bounded: on a time-out the group records a code in *status and leaves its loop.
#include "common.cuh"
#include "tc_ptx.cuh"

namespace cmace {

constexpr int RF_TILE = 128;                 // edges per tile
#ifndef RF_GROUP_WARPS
#define RF_GROUP_WARPS 16   // measured at 64 000 atoms: 3.75 ms with 16 warps per group, 4.32 ms with 8
#endif
constexpr int RF_GROUP_THREADS = RF_GROUP_WARPS * 32;
constexpr int RF_SLICE = RF_TILE / (RF_GROUP_WARPS / 4);   // edges per warp in the scatter phase
constexpr int RF_THREADS = 2 * RF_GROUP_THREADS;
constexpr int RF_SLAB = 128 * 128;           // one image (hi or lo) of one 32-column K block of 128 rows
constexpr int RF_Y_STRIDE = 20;              // staged harmonics per edge: l=0,1 at words 0..3, l=2 at 4..8, l=3 at 12..18
constexpr int RF_STAGE_BYTES = RF_TILE * RF_Y_STRIDE * 4 + RF_TILE * 8;
constexpr int RF_TMEM_COLS = 256;            // two groups x 128 columns (one per edge of the tile)

struct FusedArgs {
  const float *X, *Y, *H, *packed;
  const int32_t *sender, *receiver;
  float *out, *R;
  int32_t *status;
  int64_t E;
  int C, K, nq;
};

__device__ __forceinline__ void rf_group_sync(int group) {
  asm volatile("bar.sync %0, %1;" ::"r"(group + 1), "r"(RF_GROUP_THREADS) : "memory");
}

__device__ __forceinline__ void rf_tmem_ld8(uint32_t taddr, uint32_t (&r)[8]) {
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
               : "r"(taddr)
               : "memory");
}

__device__ __forceinline__ float4 rf_lds4(uint32_t addr) {
  float4 v;
  asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(addr));
  return v;
}
__device__ __forceinline__ float rf_lds1(uint32_t addr) {
  float v;
  asm volatile("ld.shared.f32 %0, [%1];" : "=f"(v) : "r"(addr));
  return v;
}
__device__ __forceinline__ int2 rf_lds_i2(uint32_t addr) {
  int2 v;
  asm volatile("ld.shared.v2.s32 {%0, %1}, [%2];" : "=r"(v.x), "=r"(v.y) : "r"(addr));
  return v;
}

// Adds a receiver's partial sums to the output.  Out of line on purpose: it runs about once per 40 edges, and
// inlined at each of its call sites it made the scatter loop miss the instruction cache.
template <int NM>
__device__ __noinline__ void rf_flush(float *o, int64_t stride, float a0, float a1, float a2, float a3, float a4,
                                      float a5, float a6) {
  atomicAdd(o, a0);
  if (NM > 1) {
    atomicAdd(o + stride, a1);
    atomicAdd(o + 2 * stride, a2);
  }
  if (NM > 3) {
    atomicAdd(o + 3 * stride, a3);
    atomicAdd(o + 4 * stride, a4);
  }
  if (NM > 5) {
    atomicAdd(o + 5 * stride, a5);
    atomicAdd(o + 6 * stride, a6);
  }
}

// one edge of the scatter loop: p = x * r, then the 2l+1 products with the staged harmonics at yaddr
template <int L>
__device__ __forceinline__ void rf_edge(float (&acc)[7], float p, uint32_t yaddr) {
  if (L == 0) {
    acc[0] = fmaf(rf_lds1(yaddr), p, acc[0]);
  } else if (L == 1) {
    const float4 t = rf_lds4(yaddr);
    acc[0] = fmaf(t.y, p, acc[0]);
    acc[1] = fmaf(t.z, p, acc[1]);
    acc[2] = fmaf(t.w, p, acc[2]);
  } else if (L == 2) {
    const float4 t = rf_lds4(yaddr + 16);
    const float u = rf_lds1(yaddr + 32);
    acc[0] = fmaf(t.x, p, acc[0]);
    acc[1] = fmaf(t.y, p, acc[1]);
    acc[2] = fmaf(t.z, p, acc[2]);
    acc[3] = fmaf(t.w, p, acc[3]);
    acc[4] = fmaf(u, p, acc[4]);
  } else {
    const float4 t = rf_lds4(yaddr + 48);
    const float4 u = rf_lds4(yaddr + 64);
    acc[0] = fmaf(t.x, p, acc[0]);
    acc[1] = fmaf(t.y, p, acc[1]);
    acc[2] = fmaf(t.z, p, acc[2]);
    acc[3] = fmaf(t.w, p, acc[3]);
    acc[4] = fmaf(u.x, p, acc[4]);
    acc[5] = fmaf(u.y, p, acc[5]);
    acc[6] = fmaf(u.z, p, acc[6]);
  }
}

// scatter phase of one warp: lane quarter = l, 64 edges (columns col0 .. col0 + 63 of the accumulator).
// Receivers are sorted, so a group of eight edges whose first and last receiver equal the current one needs no
// per-edge boundary test: that is the straight-line path nearly all groups take.
template <int L, int C>
__device__ __forceinline__ void rf_consume(const FusedArgs &g, uint32_t t_row, int col0, int64_t e0, uint32_t s_ys,
                                           uint32_t s_ids, int ch) {
  constexpr int NM = 2 * L + 1;
  float acc[7];
#pragma unroll
  for (int m = 0; m < 7; m++) acc[m] = 0.f;
  int cur = -1;
  const float *xc = g.X + ch;
#pragma unroll 1
  for (int gi = 0; gi < RF_SLICE / 8; gi++) {
    const int col = col0 + 8 * gi;
    uint32_t v[8];
    rf_tmem_ld8(t_row + col, v);
    int2 sr[8];
    float x[8];
    const uint32_t ia = s_ids + col * 8;
#pragma unroll
    for (int k = 0; k < 8; k++) sr[k] = rf_lds_i2(ia + k * 8);
#pragma unroll
    for (int k = 0; k < 8; k++) x[k] = __ldg(xc + (int64_t)sr[k].x * C);
    float *rp = g.R + ((e0 + col) * 4 + L) * C + ch;
    const uint32_t yaddr = s_ys + col * (RF_Y_STRIDE * 4);
    tmem_ld_wait();
    if (cur >= 0 && sr[0].y == cur && sr[7].y == cur) {
      const bool write_r = g.R != nullptr;
#pragma unroll
      for (int k = 0; k < 8; k++) {
        const float r = __uint_as_float(v[k]);
        if (write_r) rp[k * 4 * C] = r;
        rf_edge<L>(acc, x[k] * r, yaddr + k * (RF_Y_STRIDE * 4));
      }
    } else {
#pragma unroll
      for (int k = 0; k < 8; k++) {
        if (sr[k].y != cur) {
          if (cur >= 0)
            rf_flush<NM>(g.out + ((int64_t)cur * 16 + L * L) * C + ch, C, acc[0], acc[1], acc[2], acc[3], acc[4], acc[5],
                         acc[6]);
#pragma unroll
          for (int m = 0; m < 7; m++) acc[m] = 0.f;
          cur = sr[k].y;
        }
        const float r = __uint_as_float(v[k]);
        if (g.R != nullptr && sr[k].y >= 0) rp[k * 4 * C] = r;
        rf_edge<L>(acc, x[k] * r, yaddr + k * (RF_Y_STRIDE * 4));
      }
    }
  }
  if (cur >= 0)
    rf_flush<NM>(g.out + ((int64_t)cur * 16 + L * L) * C + ch, C, acc[0], acc[1], acc[2], acc[3], acc[4], acc[5], acc[6]);
}

template <int C>
__global__ void __launch_bounds__(RF_THREADS, 1)
    imp_radial_fused_kernel(const FusedArgs g, const __grid_constant__ CUtensorMap tmap) {
  extern __shared__ __align__(1024) unsigned char smem[];
  __shared__ __align__(8) uint64_t bars[5];
  __shared__ uint32_t tmem_base_slot;

  const uint32_t smem_base = (smem_u32(smem) + 1023u) & ~1023u;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int group = warp / RF_GROUP_WARPS, gw = warp % RF_GROUP_WARPS, gtid = tid & (RF_GROUP_THREADS - 1);
  const int cq = blockIdx.x % g.nq;                  // channel quarter of this CTA
  const int cta_in_cq = blockIdx.x / g.nq, ctas_per_cq = gridDim.x / g.nq;
  const int k_blocks = (g.K + 31) / 32;
  const uint32_t w_bytes = (uint32_t)k_blocks * 2u * RF_SLAB;
  const uint32_t wbar = smem_u32(&bars[0]);
  const uint32_t mma_bar = smem_u32(&bars[1 + group]);
  const uint32_t tma_bar = smem_u32(&bars[3 + group]);
  const uint32_t sW = smem_base;
  const uint32_t sH = smem_base + w_bytes + group * (k_blocks * 2 * RF_SLAB);
  const uint32_t s_ys = smem_base + w_bytes + 2 * (k_blocks * 2 * RF_SLAB) + group * RF_STAGE_BYTES;
  const uint32_t s_ids = s_ys + RF_TILE * RF_Y_STRIDE * 4;

  if (tid == 0) {
    for (int i = 0; i < 5; i++) mbar_init(wbar + 8 * i, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 0) tmem_alloc(smem_u32(&tmem_base_slot), RF_TMEM_COLS);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_acc = tmem_base_slot + group * 128;

  const int64_t ntiles = (g.E + RF_TILE - 1) / RF_TILE;
  const int64_t tile_step = (int64_t)ctas_per_cq * 2;
  int64_t tile = (int64_t)cta_in_cq * 2 + group;
  // one thread per group starts the asynchronous tile loads of H: raw rows straight into the hi images
  auto start_tile_load = [&](int64_t t) {
    mbar_arrive_expect_tx(tma_bar, (uint32_t)k_blocks * RF_SLAB);
    for (int kb = 0; kb < k_blocks; kb++) tma_load_2d(sH + kb * 2 * RF_SLAB, &tmap, kb * 32, (int)(t * RF_TILE), tma_bar);
  };
  if (tid == 0) {
    const unsigned char *src = reinterpret_cast<const unsigned char *>(g.packed) + (size_t)cq * w_bytes;
    mbar_arrive_expect_tx(wbar, w_bytes);
    for (uint32_t off = 0; off < w_bytes; off += 8192u) bulk_copy_g2s(sW + off, src + off, 8192u, wbar);
  }
  if (gtid == 0 && tile < ntiles) start_tile_load(tile);
  bool ok = warp_wait(wbar, 0, lane);
  if (!ok && lane == 0 && g.status) atomicCAS(g.status, 0, 21);

  const int l = gw & 3, slice = gw >> 2;
  const uint32_t t_row = tmem_acc + ((uint32_t)(l * 32) << 16);
  const int ch = cq * 32 + lane;
  uint32_t phase = 0;

  for (; ok && tile < ntiles; tile += tile_step) {
    const int64_t e0 = tile * RF_TILE;
    // ---- the tile's rows of H have landed as the raw (= hi) image; add the residual image
    if (!(ok = warp_wait(tma_bar, phase, lane))) break;
    for (int kb = 0; kb < k_blocks; kb++) {
#pragma unroll
      for (int i = 0; i < 1024 / RF_GROUP_THREADS; i++) {
        const int cidx = gtid + RF_GROUP_THREADS * i;
        const uint32_t addr = sH + kb * 2 * RF_SLAB + (uint32_t)sw128_offset(cidx >> 3, cidx & 7);
        const float4 a = rf_lds4(addr);
        float4 lo;
        lo.x = to_tf32(a.x - __uint_as_float(__float_as_uint(a.x) & 0xFFFFE000u));
        lo.y = to_tf32(a.y - __uint_as_float(__float_as_uint(a.y) & 0xFFFFE000u));
        lo.z = to_tf32(a.z - __uint_as_float(__float_as_uint(a.z) & 0xFFFFE000u));
        lo.w = to_tf32(a.w - __uint_as_float(__float_as_uint(a.w) & 0xFFFFE000u));
        asm volatile("st.shared.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(addr + RF_SLAB), "f"(lo.x), "f"(lo.y), "f"(lo.z),
                     "f"(lo.w)
                     : "memory");
      }
    }
    tc_fence_before();
    fence_proxy_async();
    rf_group_sync(group);
    if (gtid == 0) {
      tc_fence_after();
      const uint32_t idesc = umma_idesc_tf32(128, RF_TILE);
      for (int k0 = 0, kb = 0; k0 < g.K; k0 += 32, kb++) {
        const uint64_t a_hi = umma_desc_sw128(sW + kb * 2 * RF_SLAB);
        const uint64_t a_lo = umma_desc_sw128(sW + kb * 2 * RF_SLAB + RF_SLAB);
        const uint64_t b_hi = umma_desc_sw128(sH + kb * 2 * RF_SLAB);
        const uint64_t b_lo = umma_desc_sw128(sH + kb * 2 * RF_SLAB + RF_SLAB);
        int ksteps = (g.K - k0) / 8;
        ksteps = ksteps > 4 ? 4 : ksteps;
        for (int j = 0; j < ksteps; j++) {
          // the three terms of the split accumulate in place: Whi*Hhi + Whi*Hlo + Wlo*Hhi
          umma_tf32(tmem_acc, a_hi + (uint64_t)(2 * j), b_hi + (uint64_t)(2 * j), idesc, (kb | j) != 0);
          umma_tf32_acc(tmem_acc, a_hi + (uint64_t)(2 * j), b_lo + (uint64_t)(2 * j), idesc);
          umma_tf32_acc(tmem_acc, a_lo + (uint64_t)(2 * j), b_hi + (uint64_t)(2 * j), idesc);
        }
      }
      umma_commit(mma_bar);
    }
    // ---- while the tensor core works: harmonics and edge indices of the tile into shared memory
    if (gtid < RF_TILE) {
      const int64_t e = e0 + gtid;
      const int2 v = e < g.E ? make_int2(g.sender[e], g.receiver[e]) : make_int2(0, -1);
      asm volatile("st.shared.v2.s32 [%0], {%1, %2};" ::"r"(s_ids + gtid * 8), "r"(v.x), "r"(v.y) : "memory");
    }
#pragma unroll
    for (int i = 0; i < 2048 / RF_GROUP_THREADS; i++) {
      const int idx = gtid + RF_GROUP_THREADS * i;
      const int lm = idx >> 7, el = idx & (RF_TILE - 1);
      const int64_t e = e0 + el;
      const float y = e < g.E ? __ldg(g.Y + (int64_t)lm * g.E + e) : 0.f;
      asm volatile("st.shared.f32 [%0], %1;" ::"r"(s_ys + (el * RF_Y_STRIDE + (lm < 9 ? lm : lm + 3)) * 4), "f"(y) : "memory");
    }
    rf_group_sync(group);
    if (!(ok = warp_wait(mma_bar, phase, lane))) break;
    phase ^= 1;
    tc_fence_after();
    // the H images are free again: fetch the next tile while this one is scattered
    if (gtid == 0 && tile + tile_step < ntiles) start_tile_load(tile + tile_step);
    const int col0 = slice * RF_SLICE;
    if (l == 0) rf_consume<0, C>(g, t_row, col0, e0, s_ys, s_ids, ch);
    else if (l == 1) rf_consume<1, C>(g, t_row, col0, e0, s_ys, s_ids, ch);
    else if (l == 2) rf_consume<2, C>(g, t_row, col0, e0, s_ys, s_ids, ch);
    else rf_consume<3, C>(g, t_row, col0, e0, s_ys, s_ids, ch);
  }
  if (!ok && lane == 0 && g.status) atomicCAS(g.status, 0, 22);

  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem_base_slot, RF_TMEM_COLS);
}

}  // namespace cmace

using namespace cmace;

extern "C" {

int cmace_imp_radial_fused_fwd_f32(const float *X, const float *Y, const float *H, const float *packed_w,
                                   const int32_t *sender, const int32_t *receiver, int64_t nnodes, int64_t nedges,
                                   int nchannels, int K, float *out, float *R, int32_t *status, cmace_stream_t stream) {
  if (nnodes < 0 || nedges < 0) return fail(CMACE_ERR_ARG, "cmace_imp_radial_fused_fwd: negative size");
  if (nchannels < 32 || nchannels > 128 || nchannels % 32 != 0 || (K != 32 && K != 64))
    return fail(CMACE_ERR_UNSUPPORTED, "cmace_imp_radial_fused_fwd: channels must be 32, 64, 96 or 128 and K 32 or 64");
  if (nnodes == 0) return CMACE_OK;
  if (!out) return fail(CMACE_ERR_ARG, "cmace_imp_radial_fused_fwd: null output");
  cudaStream_t st = (cudaStream_t)stream;
  cudaError_t e = cudaMemsetAsync(out, 0, (size_t)nnodes * 16 * nchannels * sizeof(float), st);
  if (e != cudaSuccess) return fail(CMACE_ERR_CUDA, "cmace_imp_radial_fused_fwd: %s", cudaGetErrorString(e));
  if (nedges == 0) return CMACE_OK;
  if (!X || !Y || !H || !packed_w || !sender || !receiver)
    return fail(CMACE_ERR_ARG, "cmace_imp_radial_fused_fwd: null pointer");
  if (!aligned16(H) || !aligned16(packed_w))
    return fail(CMACE_ERR_ARG, "cmace_imp_radial_fused_fwd: H and the packed weights must be 16-byte aligned");
  static int num_sms = 0;
  if (num_sms == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&num_sms, cudaDevAttrMultiProcessorCount, dev);
    if (num_sms <= 0) num_sms = 148;
  }
  FusedArgs g{};
  g.X = X; g.Y = Y; g.H = H; g.packed = packed_w; g.sender = sender; g.receiver = receiver;
  g.out = out; g.R = R; g.status = status; g.E = nedges; g.C = nchannels; g.K = K; g.nq = nchannels / 32;
  const int k_blocks = (K + 31) / 32;
  const size_t smem = (size_t)3 * k_blocks * 2 * RF_SLAB + 2 * RF_STAGE_BYTES + 1024;
  auto kern = nchannels == 128 ? imp_radial_fused_kernel<128>
              : nchannels == 96 ? imp_radial_fused_kernel<96>
              : nchannels == 64 ? imp_radial_fused_kernel<64> : imp_radial_fused_kernel<32>;
  e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return fail(CMACE_ERR_CUDA, "cmace_imp_radial_fused_fwd: %s", cudaGetErrorString(e));
  const int64_t ntiles = (nedges + RF_TILE - 1) / RF_TILE;
  int64_t per_cq = (ntiles + 1) / 2;
  const int64_t cap = num_sms / g.nq > 0 ? num_sms / g.nq : 1;
  per_cq = per_cq < cap ? per_cq : cap;
  CUtensorMap tmap;
  if (int rc = encode_rows_tensor_map(&tmap, H, nedges, K, "cmace_imp_radial_fused_fwd")) return rc;
  kern<<<(unsigned)(per_cq * g.nq), RF_THREADS, smem, st>>>(g, tmap);
  return check_launch("cmace_imp_radial_fused_fwd");
}
}
