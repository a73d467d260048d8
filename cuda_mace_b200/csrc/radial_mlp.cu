// Hidden layers of the radial multilayer perceptron in one kernel (float32, tensor cores):
//
//   forward    basis [E, nb]  ->  h3 = silu(silu(silu(basis W1) W2) W3)   [E, 64]
//   backward   grad h3 [E, 64] -> grad basis [E, nb]
//
// (the 1/sqrt(fan_in) factors and the normalisation constant of the activation are folded into the weights by
// the caller).  The activations never leave the SM: a layer's accumulator is read from tensor memory, activated,
// split into the hi / lo TF32 images and written back as the next layer's A operand.  Every product uses the
// 3-term split  Ahi*Bhi + Ahi*Blo + Alo*Bhi  with the float32 accumulator in tensor memory, three tcgen05.mma per
// K step into the same columns (one tensor-memory load per value in the elementwise phase).
// The forward stores the activation derivatives d_k = silu'(z_k) (three [E, 64] arrays in a tiled layout that
// both kernels access with coalesced 16-byte transfers); the backward is then three products with an
// elementwise factor between them and needs no special-function work.
//
// One CTA per SM, two independent groups of eight warps; the weights (80 KB forward, 72 KB backward) are loaded
// into shared memory once.  A tile's layers form a chain: elementwise phase, hand-over, MMAs, completion,
// accumulator load, next elementwise phase; the fixed latencies of that chain are longer than the arithmetic.
// Both kernels: every group keeps TWO 128-edge tiles in flight and alternates between them, so one tile's
// elementwise phase runs while the other tile's products are on the tensor core.  Four tiles per SM need four
// operand buffers: the raw values (= hi image) of the 64 activations go to shared memory (32 KB a tile), their
// residual image to tensor memory, from where the third product term reads its A operand.  The first thread of
// a group issues its MMAs after the group's barrier: 16 warps per CTA keep the register limit at 128 per thread.
// Every mbarrier wait is bounded: on a time-out the role records a code in *status and leaves its loop.
#include <cstring>

#include "common.cuh"
#include "tc_ptx.cuh"

namespace cmace {

constexpr int RH_H = 64;                    // hidden width
constexpr int RH_TILE = 128;                // edges per tile
constexpr int RH_GROUP_THREADS = 256;       // eight warps
constexpr int RH_THREADS = 2 * RH_GROUP_THREADS;
constexpr int RH_A_SLAB = RH_TILE * 128;    // one image (hi or lo) of one 32-column K block: 16 KB
constexpr int RH_W_SMALL = 2 * 64 * 128;    // packed [nb <= 32, 64]: one K block, hi + lo images of 64 rows
constexpr int RH_W_BIG = 2 * RH_W_SMALL;    // packed [64, 64]: two K blocks
constexpr int RF_SLOT_BYTES = 2 * RH_A_SLAB;  // operand buffer of a tile in flight: raw images of two K blocks
                                              // (first layer: raw and residual image of the basis)
constexpr int RF_TMEM_SLOT = 128;             // tensor-memory columns of a tile in flight: 64 accumulator + 64 residual
constexpr int RF_TMEM_COLS = 4 * RF_TMEM_SLOT;

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

// special-function unit: 2^x and 1/x, about 2 ulp and 1 ulp
__device__ __forceinline__ float ex2_approx(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ float rcp_approx(float x) {
  float y;
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// silu(z) = z s and silu'(z) = s (1 + z (1 - s)), s = 1 / (1 + 2^(-z log2 e)), for two values at once: four
// special-function and six packed instructions per pair.  Large |z| saturate cleanly (s = 0 or 1), no NaN.
__device__ __forceinline__ void silu_both2(unsigned long long z2, unsigned long long &a2, unsigned long long &d2) {
  const unsigned long long one2 = pack2(1.0f, 1.0f);
  float t0, t1;
  unpack2(mul2(z2, pack2(-1.4426950408889634f, -1.4426950408889634f)), t0, t1);
  float n0, n1;
  unpack2(add2(pack2(ex2_approx(t0), ex2_approx(t1)), one2), n0, n1);
  const unsigned long long s2 = pack2(rcp_approx(n0), rcp_approx(n1));
  a2 = mul2(z2, s2);
  d2 = mul2(s2, fma2(z2, fma2(s2, pack2(-1.0f, -1.0f), one2), one2));
}

// The products of one layer for a tile in flight, into npad accumulator columns.  `first` (forward, layer 1): A =
// the basis, raw image in slab 0 and residual image in slab 1 of the tile's buffer, K = nb.  Otherwise K = 64: raw
// images of the two K blocks in the two slabs, residual image in tensor memory (column k of the tile's residual
// region = column k of A).  sB: packed weights, per K block the hi image then the lo image of npad rows.
__device__ __forceinline__ void issue_tile_layer(uint32_t acc, uint32_t lo_tmem, uint32_t sA, uint32_t sB, bool first,
                                                 int nb, int npad) {
  const uint32_t idesc = umma_idesc_tf32(RH_TILE, npad);
  const uint32_t b_image = (uint32_t)npad * 128u;
  if (first) {
    const uint64_t a_hi = umma_desc_sw128(sA), a_lo = umma_desc_sw128(sA + RH_A_SLAB);
    const uint64_t b_hi = umma_desc_sw128(sB), b_lo = umma_desc_sw128(sB + b_image);
    for (int j = 0; j < nb / 8; j++) {
      umma_tf32(acc, a_hi + (uint64_t)(2 * j), b_hi + (uint64_t)(2 * j), idesc, j != 0);
      umma_tf32_acc(acc, a_hi + (uint64_t)(2 * j), b_lo + (uint64_t)(2 * j), idesc);
      umma_tf32_acc(acc, a_lo + (uint64_t)(2 * j), b_hi + (uint64_t)(2 * j), idesc);
    }
    return;
  }
#pragma unroll
  for (int kb = 0; kb < 2; kb++) {
    const uint64_t a_hi = umma_desc_sw128(sA + kb * RH_A_SLAB);
    const uint64_t b_hi = umma_desc_sw128(sB + kb * 2 * b_image);
    const uint64_t b_lo = umma_desc_sw128(sB + kb * 2 * b_image + b_image);
#pragma unroll
    for (int j = 0; j < 4; j++) {
      umma_tf32(acc, a_hi + (uint64_t)(2 * j), b_hi + (uint64_t)(2 * j), idesc, (kb | j) != 0);
      umma_tf32_acc(acc, a_hi + (uint64_t)(2 * j), b_lo + (uint64_t)(2 * j), idesc);
      umma_tf32_ts_acc(acc, lo_tmem + 32u * kb + 8u * j, b_hi + (uint64_t)(2 * j), idesc);
    }
  }
}

// NI: 16-byte chunks of the basis a thread carries per tile (256 threads x NI chunks cover 128 rows of nb floats:
// 1 for nb = 8, 4 up to nb = 32)
template <int NI>
__global__ void __launch_bounds__(RH_THREADS, 1)
    radial_hidden_fwd_kernel(const RadialArgs g, const __grid_constant__ CUtensorMap out_map) {
  extern __shared__ __align__(1024) unsigned char smem[];
  __shared__ __align__(8) uint64_t bars[5];   // weights; done[group][slot]
  __shared__ uint32_t tmem_base_slot;

  const uint32_t smem_base = (smem_u32(smem) + 1023u) & ~1023u;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int group = warp >> 3;
  const uint32_t wbar = smem_u32(&bars[0]);
  const uint32_t done0 = wbar + 8u * (1 + 2 * group);   // + 8 * slot

  const uint32_t w_bytes[3] = {(uint32_t)RH_W_SMALL, (uint32_t)RH_W_BIG, (uint32_t)RH_W_BIG};
  const uint32_t sW[3] = {smem_base, smem_base + w_bytes[0], smem_base + w_bytes[0] + w_bytes[1]};
  const uint32_t sA0 = smem_base + w_bytes[0] + w_bytes[1] + w_bytes[2] + (uint32_t)(2 * group) * RF_SLOT_BYTES;

  if (tid == 0) {
    for (int i = 0; i < 5; i++) mbar_init(wbar + 8u * i, 1);   // weights; done: the commit of a layer's MMAs
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 0) tmem_alloc(smem_u32(&tmem_base_slot), RF_TMEM_COLS);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem0 = tmem_base_slot + (uint32_t)(2 * group) * RF_TMEM_SLOT;   // + slot * RF_TMEM_SLOT; residual at + 64

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

  // the group's tiles: first, first + step, ...; tile number j of the group uses slot j & 1, and the two slots
  // move through their layers side by side
  const int64_t ntiles = (g.E + RH_TILE - 1) / RH_TILE;
  const int64_t step = (int64_t)gridDim.x * 2;
  const int64_t first = (int64_t)blockIdx.x * 2 + group;

  {
    const int gw = warp & 7, gtid = tid & (RH_GROUP_THREADS - 1);
    const int q = gw & 3, h = gw >> 2;      // tensor-memory lane quarter, column half (= K block of the next layer)
    const int r = q * 32 + lane;            // row of the tile this thread owns in the elementwise phases
    const uint32_t lane_field = (uint32_t)(q * 32) << 16;
    const int nchunks = g.nb / 4;           // 16-byte chunks per row of the basis
    uint32_t phase = 0;

    // the basis rows of a tile: up to four 16-byte chunks per thread, fetched a whole pass ahead
    float4 pre[2][NI];
    auto load_basis = [&](int64_t t, float4 (&dst)[NI]) {
#pragma unroll
      for (int i = 0; i < NI; i++) {
        const int idx = gtid + RH_GROUP_THREADS * i;
        const int rr = idx / nchunks, c = idx - rr * nchunks;
        const int64_t ee = t * RH_TILE + rr;
        dst[i] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (t < ntiles && rr < RH_TILE && ee < g.E) dst[i] = __ldg(reinterpret_cast<const float4 *>(g.in + ee * g.nb) + c);
      }
    };
    load_basis(first, pre[0]);
    load_basis(first + step, pre[1]);
    // the whole group has written its part of an operand: its first thread issues the layer's products.  (A warp of
    // its own for the issue made the CTA 18 warps and the register limit 96; with 16 warps and 128 registers the
    // kernel is 9 % faster although the issuing thread's warp is held up.)
    auto hand_over = [&](int s, int layer) {
      fence_proxy_async();
      group_sync(group);
      if (gtid == 0) {
        tc_fence_after();
        const uint32_t acc0 = tmem0 + (uint32_t)s * RF_TMEM_SLOT;
        issue_tile_layer(acc0, acc0 + 64u, sA0 + (uint32_t)s * RF_SLOT_BYTES, sW[layer], layer == 0, g.nb, RH_H);
        umma_commit(done0 + 8u * s);
      }
    };

    for (int64_t t0 = first; ok && t0 < ntiles; t0 += 2 * step) {
      const int nslots = t0 + step < ntiles ? 2 : 1;
      if (t0 != first) {
        // the tile stores of the previous pass read the buffers that are written next
        if (gtid == 0) tma_store_wait_read();
        group_sync(group);
      }
      // ---- first layer's operand: the basis rows, raw image in slab 0, residual image in slab 1
#pragma unroll
      for (int s = 0; s < 2; s++) {
        if (s < nslots) {
          const uint32_t sA = sA0 + (uint32_t)s * RF_SLOT_BYTES;
#pragma unroll
          for (int i = 0; i < NI; i++) {
            const int idx = gtid + RH_GROUP_THREADS * i;
            const int rr = idx / nchunks, c = idx - rr * nchunks;
            if (rr < RH_TILE) store_split(sA + (uint32_t)sw128_offset(rr, c), pre[s][i]);
          }
          tc_fence_before();      // orders this warp's accumulator loads of the previous pass before the new MMAs
          hand_over(s, 0);
        }
      }
      for (int layer = 0; ok && layer < 3; layer++) {
        if (layer == 2) {
          load_basis(t0 + 2 * step, pre[0]);
          load_basis(t0 + 3 * step, pre[1]);
        }
#pragma unroll
        for (int s = 0; s < 2; s++) {
          if (s < nslots && ok) {
            const int64_t tile = t0 + s * step;
            const uint32_t acc = tmem0 + (uint32_t)s * RF_TMEM_SLOT + lane_field;
            const uint32_t a_row = sA0 + (uint32_t)s * RF_SLOT_BYTES + (uint32_t)h * RH_A_SLAB;
            float4 *dtile = g.dsave + ((tile * 3 + layer) * 16 + h * 8) * RH_TILE + r;   // + chunk * 128
            if (!warp_wait(done0 + 8u * s, phase, lane)) {
              if (lane == 0 && g.status) atomicCAS(g.status, 0, 12);
              ok = false;
            } else {
              tc_fence_after();
              uint32_t v[32];
              tmem_ld32_nowait(acc + 32u * h, v);
              tmem_ld_wait();
#pragma unroll
              for (int hh = 0; hh < 2; hh++) {          // 16 columns at a time: one tensor-memory store each
                uint32_t lo[16];
#pragma unroll
                for (int c = 0; c < 4; c++) {
                  const int col = 16 * hh + 4 * c;
                  unsigned long long a01, a23, d01, d23;
                  silu_both2(pack2(__uint_as_float(v[col]), __uint_as_float(v[col + 1])), a01, d01);
                  silu_both2(pack2(__uint_as_float(v[col + 2]), __uint_as_float(v[col + 3])), a23, d23);
                  float4 d;
                  unpack2(d01, d.x, d.y);
                  unpack2(d23, d.z, d.w);
                  if (g.dsave != nullptr) dtile[(4 * hh + c) * RH_TILE] = d;
                  // layers 1, 2: the raw values are the next operand's hi image.  Layer 3: the same swizzled 128-row
                  // x 32-column image is what the tile store of h3 reads (a thread owns a row: stores from registers
                  // would hit 32 different 128-byte lines per instruction, which measured 0.3 ms of a 0.85 ms kernel)
                  asm volatile("st.shared.v2.b64 [%0], {%1, %2};" ::"r"(a_row + (uint32_t)sw128_offset(r, 4 * hh + c)),
                               "l"(a01), "l"(a23)
                               : "memory");
                  if (layer < 2) {
                    // the residual a - trunc(a) is exact in float32 and is read by the tensor core with the same
                    // truncation as the hi image (error below 2^-20 |a|)
                    const unsigned long long l01 = sub2(a01, a01 & 0xFFFFE000FFFFE000ull);
                    const unsigned long long l23 = sub2(a23, a23 & 0xFFFFE000FFFFE000ull);
                    asm("mov.b64 {%0, %1}, %2;" : "=r"(lo[4 * c]), "=r"(lo[4 * c + 1]) : "l"(l01));
                    asm("mov.b64 {%0, %1}, %2;" : "=r"(lo[4 * c + 2]), "=r"(lo[4 * c + 3]) : "l"(l23));
                  }
                }
                if (layer < 2) tmem_st16(acc + 64u + 32u * h + 16u * hh, lo);
              }
              if (layer < 2) {
                tmem_st_wait();
                tc_fence_before();
                hand_over(s, layer + 1);
              } else {
                // h3 [128, 64] of the tile: two 32-column boxes, rows past the end of the array are clipped
                fence_proxy_async();
                group_sync(group);
                if (gtid == 0) {
                  const uint32_t sT = sA0 + (uint32_t)s * RF_SLOT_BYTES;
                  tma_store_2d(&out_map, 0, (int)(tile * RH_TILE), sT);
                  tma_store_2d(&out_map, 32, (int)(tile * RH_TILE), sT + RH_A_SLAB);
                }
              }
            }
          }
        }
        phase ^= 1;
      }
    }
    if (gtid == 0) tma_store_wait_all();
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem_base_slot, RF_TMEM_COLS);
}

// ---- backward ------------------------------------------------------------------------------------------
// Same arrangement as the forward: two tiles in flight per group, raw images in shared memory (32 KB a tile),
// residual images in tensor memory.  A tile goes through four phases:
//   0  operand = grad h3 * d3 (the grad h3 tile was put into the tile's buffer by TMA, a thread multiplies its own
//      row in place), product with W3^T;   1  operand = accumulator * d2, product with W2^T;
//   2  operand = accumulator * d1, product with W1^T (narrow);   3  grad basis = accumulator columns [0, nb).
// The derivatives of the phase a tile enters next are fetched into registers as soon as the current phase has
// consumed its own (32 registers per tile in flight), so they are on their way during the other tile's phase;
// the grad h3 tile of a buffer's next tile is requested in phase 3, when the last product that read the buffer
// has completed.  (Pulling the next pass's derivative arrays into L2 ahead of time measured slower: 0.89 against
// 0.73 ms.  What bounds the kernel is the bytes the register buffers keep in flight: 64 registers x 512 threads,
// in flight for about 70 % of the time.)  The MMAs are issued by the first thread of the group after the group's barrier: the elementwise
// phases are short here (no special functions), and a warp of its own would cost every thread 32 registers.
__global__ void __launch_bounds__(RH_THREADS, 1)
    radial_hidden_bwd_kernel(const RadialArgs g, const __grid_constant__ CUtensorMap in_map) {
  extern __shared__ __align__(1024) unsigned char smem[];
  __shared__ __align__(8) uint64_t bars[9];   // weights; done[group][slot]; grad h3 tile landed [group][slot]
  __shared__ uint32_t tmem_base_slot;

  const uint32_t smem_base = (smem_u32(smem) + 1023u) & ~1023u;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int group = warp >> 3, gw = warp & 7, gtid = tid & (RH_GROUP_THREADS - 1);
  const uint32_t wbar = smem_u32(&bars[0]);
  const uint32_t done0 = wbar + 8u * (1 + 2 * group);   // + 8 * slot
  const uint32_t gin0 = wbar + 8u * (5 + 2 * group);

  // weights: W3^T, W2^T, W1^T (narrow)
  const uint32_t w_bytes[3] = {(uint32_t)RH_W_BIG, (uint32_t)RH_W_BIG, 2u * 2u * (uint32_t)g.npad_last * 128u};
  const uint32_t sW[3] = {smem_base, smem_base + w_bytes[0], smem_base + w_bytes[0] + w_bytes[1]};
  const uint32_t sA0 = smem_base + w_bytes[0] + w_bytes[1] + w_bytes[2] + (uint32_t)(2 * group) * RF_SLOT_BYTES;

  if (tid == 0) {
    for (int i = 0; i < 9; i++) mbar_init(wbar + 8u * i, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 0) tmem_alloc(smem_u32(&tmem_base_slot), RF_TMEM_COLS);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem0 = tmem_base_slot + (uint32_t)(2 * group) * RF_TMEM_SLOT;

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
  const uint32_t lane_field = (uint32_t)(q * 32) << 16;
  const int64_t ntiles = (g.E + RH_TILE - 1) / RH_TILE;
  const int64_t step = (int64_t)gridDim.x * 2;
  const int64_t first = (int64_t)blockIdx.x * 2 + group;

  // grad h3 [128, 64] of a tile into the buffer of slot s: two 32-column boxes, rows past the end read as zero
  auto request_g = [&](int s, int64_t tile) {
    if (tile >= ntiles) return;
    const uint32_t dst = sA0 + (uint32_t)s * RF_SLOT_BYTES, bar = gin0 + 8u * s;
    mbar_arrive_expect_tx(bar, 2u * RH_A_SLAB);
    tma_load_2d(dst, &in_map, 0, (int)(tile * RH_TILE), bar);
    tma_load_2d(dst + RH_A_SLAB, &in_map, 32, (int)(tile * RH_TILE), bar);
  };
  // d_{layer+1} of a tile: this thread's row, its 32 columns (8 chunks of 16 bytes, 512 bytes apart in the tiled array)
  float4 buf[2][8];
  auto load_d = [&](float4 (&dst)[8], int64_t tile, int layer) {
    if (tile >= ntiles) return;
    const float4 *dt = g.dsave + ((tile * 3 + layer) * 16 + h * 8) * RH_TILE + r;
#pragma unroll
    for (int c = 0; c < 8; c++) dst[c] = dt[c * RH_TILE];
  };
  // the whole group has written its part of the operand: one thread issues the layer's products
  auto hand_over = [&](int s, int layer) {
    tmem_st_wait();
    tc_fence_before();
    fence_proxy_async();
    group_sync(group);
    if (gtid == 0) {
      tc_fence_after();
      const uint32_t acc = tmem0 + (uint32_t)s * RF_TMEM_SLOT;
      issue_tile_layer(acc, acc + 64u, sA0 + (uint32_t)s * RF_SLOT_BYTES, sW[layer], false, 0,
                       layer == 2 ? g.npad_last : RH_H);
      umma_commit(done0 + 8u * s);
    }
  };
  // 16 columns of the operand: raw values into the swizzled image, residual into tensor memory
  auto put16 = [&](int s, int hh, const unsigned long long (&a)[8]) {
    const uint32_t a_row = sA0 + (uint32_t)s * RF_SLOT_BYTES + (uint32_t)h * RH_A_SLAB;
    uint32_t lo[16];
#pragma unroll
    for (int c = 0; c < 4; c++) {
      asm volatile("st.shared.v2.b64 [%0], {%1, %2};" ::"r"(a_row + (uint32_t)sw128_offset(r, 4 * hh + c)), "l"(a[2 * c]),
                   "l"(a[2 * c + 1])
                   : "memory");
#pragma unroll
      for (int k = 0; k < 2; k++) {
        const unsigned long long l2 = sub2(a[2 * c + k], a[2 * c + k] & 0xFFFFE000FFFFE000ull);
        asm("mov.b64 {%0, %1}, %2;" : "=r"(lo[4 * c + 2 * k]), "=r"(lo[4 * c + 2 * k + 1]) : "l"(l2));
      }
    }
    tmem_st16(tmem0 + (uint32_t)s * RF_TMEM_SLOT + lane_field + 64u + 32u * h + 16u * hh, lo);
  };

  if (gtid == 0) {
    request_g(0, first);
    request_g(1, first + step);
  }
  load_d(buf[0], first, 2);
  load_d(buf[1], first + step, 2);
  uint32_t done_phase = 0, gin_phase = 0;   // one parity bit each: both slots' barriers complete side by side

  for (int64_t t0 = first; ok && t0 < ntiles; t0 += 2 * step) {
    const int nslots = t0 + step < ntiles ? 2 : 1;
    // ---- phase 0: grad z3 = grad h3 * d3, in place
#pragma unroll
    for (int s = 0; s < 2; s++) {
      if (s < nslots && ok) {
        const int64_t tile = t0 + s * step;
        if (!warp_wait(gin0 + 8u * s, gin_phase, lane)) {
          if (lane == 0 && g.status) atomicCAS(g.status, 0, 14);
          ok = false;
        } else {
          const uint32_t a_row = sA0 + (uint32_t)s * RF_SLOT_BYTES + (uint32_t)h * RH_A_SLAB;
#pragma unroll
          for (int hh = 0; hh < 2; hh++) {
            unsigned long long a[8];
#pragma unroll
            for (int c = 0; c < 4; c++) {
              unsigned long long g01, g23;
              asm volatile("ld.shared.v2.b64 {%0, %1}, [%2];"
                           : "=l"(g01), "=l"(g23)
                           : "r"(a_row + (uint32_t)sw128_offset(r, 4 * hh + c))
                           : "memory");
              const float4 d = buf[s][4 * hh + c];
              a[2 * c] = mul2(g01, pack2(d.x, d.y));
              a[2 * c + 1] = mul2(g23, pack2(d.z, d.w));
            }
            put16(s, hh, a);
          }
          load_d(buf[s], tile, 1);
          hand_over(s, 0);
        }
      }
    }
    gin_phase ^= 1;
    // ---- phases 1 and 2: grad z_k = accumulator * d_k
    for (int k = 1; ok && k < 3; k++) {
#pragma unroll
      for (int s = 0; s < 2; s++) {
        if (s < nslots && ok) {
          const int64_t tile = t0 + s * step;
          if (!warp_wait(done0 + 8u * s, done_phase, lane)) {
            if (lane == 0 && g.status) atomicCAS(g.status, 0, 12);
            ok = false;
          } else {
            tc_fence_after();
            const uint32_t t_row = tmem0 + (uint32_t)s * RF_TMEM_SLOT + lane_field + 32u * h;
#pragma unroll
            for (int hh = 0; hh < 2; hh++) {
              uint32_t v[16];
              tmem_ld16_nowait(t_row + 16u * hh, v);
              tmem_ld_wait();
              unsigned long long a[8];
#pragma unroll
              for (int c = 0; c < 4; c++) {
                const float4 d = buf[s][4 * hh + c];
                a[2 * c] = mul2(pack2(__uint_as_float(v[4 * c]), __uint_as_float(v[4 * c + 1])), pack2(d.x, d.y));
                a[2 * c + 1] = mul2(pack2(__uint_as_float(v[4 * c + 2]), __uint_as_float(v[4 * c + 3])), pack2(d.z, d.w));
              }
              put16(s, hh, a);
            }
            if (k == 1) load_d(buf[s], tile, 0);
            else load_d(buf[s], tile + 2 * step, 2);
            hand_over(s, k);
          }
        }
      }
      done_phase ^= 1;
    }
    // ---- phase 3: grad basis = columns [0, nb) of the accumulator; the buffer is free for its next tile
#pragma unroll
    for (int s = 0; s < 2; s++) {
      if (s < nslots && ok) {
        const int64_t tile = t0 + s * step;
        if (!warp_wait(done0 + 8u * s, done_phase, lane)) {
          if (lane == 0 && g.status) atomicCAS(g.status, 0, 12);
          ok = false;
        } else {
          tc_fence_after();
          if (gtid == 0) request_g(s, tile + 2 * step);
          const int64_t e = tile * RH_TILE + r;
          if (h == 0) {
            const uint32_t t_row = tmem0 + (uint32_t)s * RF_TMEM_SLOT + lane_field;
            for (int c0 = 0; c0 < g.nb; c0 += 8) {
              uint32_t v[8];
              tmem_ld8(t_row + c0, v);
              if (e < g.E) {
                float *o = g.out + e * g.nb + c0;
                *reinterpret_cast<float4 *>(o) = make_float4(__uint_as_float(v[0]), __uint_as_float(v[1]),
                                                             __uint_as_float(v[2]), __uint_as_float(v[3]));
                *reinterpret_cast<float4 *>(o + 4) = make_float4(__uint_as_float(v[4]), __uint_as_float(v[5]),
                                                                 __uint_as_float(v[6]), __uint_as_float(v[7]));
              }
            }
          }
          tc_fence_before();
        }
      }
    }
    done_phase ^= 1;
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem_base_slot, RF_TMEM_COLS);
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
  const size_t smem = w_total + 4 * (size_t)RF_SLOT_BYTES + 1024;
  const int64_t ntiles = (g.E + RH_TILE - 1) / RH_TILE;
  int64_t blocks = (ntiles + 1) / 2;
  blocks = blocks < num_sms ? blocks : num_sms;
  if (ntiles * RH_TILE > 0x7fffffffLL) return fail(CMACE_ERR_UNSUPPORTED, "%s: too many edges", what);
  // the [E, 64] array that moves by TMA as 128-row x 32-column boxes: grad h3 in (backward), h3 out (forward)
  CUtensorMap map;
  if (int rc = encode_rows_tensor_map(&map, backward ? g.in : g.out, g.E, RH_H, what)) return rc;
  if (backward) {
    cudaError_t e = cudaFuncSetAttribute(radial_hidden_bwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return fail(CMACE_ERR_CUDA, "%s: %s", what, cudaGetErrorString(e));
    radial_hidden_bwd_kernel<<<(unsigned)blocks, RH_THREADS, smem, st>>>(g, map);
  } else {
    auto kern = g.nb == 8 ? radial_hidden_fwd_kernel<1> : radial_hidden_fwd_kernel<4>;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return fail(CMACE_ERR_CUDA, "%s: %s", what, cudaGetErrorString(e));
    kern<<<(unsigned)blocks, RH_THREADS, smem, st>>>(g, map);
  }
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
