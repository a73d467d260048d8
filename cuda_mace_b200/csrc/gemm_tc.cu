// float32 GEMM on the 5th-generation tensor cores with a 3-term TF32 split:
//
//   out[row(r), :] = scale * A[row(r), :] @ B          A [M, K] float32, B [K, N] float32
//
// Every float32 operand x is split as x = hi + lo with hi = tf32(x) and lo = tf32(x - hi) (both rounded to
// nearest, so the residual is unbiased), and D = Ahi*Bhi + Alo*Bhi + Ahi*Blo is accumulated in float32 in tensor
// memory, which brings the result to about 2^-21 relative: float32-grade, unlike a single TF32 pass.
// A tcgen05.mma of M=128, K=8 takes 48 cycles at N=64 and 64 cycles at N=128 (measured), so narrow
// instructions waste the pipe: the hi and lo images of B sit back to back and are read as ONE operand of twice the rows, which
// yields Ahi*Bhi and Ahi*Blo from a single instruction (two column ranges of the accumulator, added in the
// epilogue); with Alo*Bhi that is two instructions per K step instead of three.
//
// Structure (one CTA per SM, persistent over 128-row tiles, warp specialised, 18 warps):
//   warp 17    loader (PLAIN row map): per pipeline item one TMA tile load (128 rows x 32 columns of A,
//              128-byte swizzle) straight into the stage's hi image (the tensor core ignores the low 13
//              mantissa bits of a float32, so raw data is the hi operand) and one bulk copy of the matching
//              pre-packed B block (hi and lo images, swizzled by the pack kernel).  Nothing waits in
//              registers for HBM.
//   warps 0-7  converters (PLAIN): read the raw tile back from shared memory and store the residual image
//              lo = tf32(a - trunc(a)) next to it -- or, where tensor memory has room beside the accumulators
//              (kernel variant TS), into a ring of tensor-memory columns, from where the Alo*Bhi product
//              takes its A operand.
//              With the LINEAR row map (gathered rows) the same warps load the row segments into registers
//              themselves, two items ahead, and convert from there.
//   warp 8     MMA issuer: one elected thread issues tcgen05.mma kind::tf32 (M=128, N<=128, K=8),
//              4 K-steps x 3 split terms per stage, and commits to the stage's "empty" barrier and,
//              after the last K block of a tile, to the accumulator's "full" barrier.
//   warps 9-16 epilogue: tcgen05.ld of the accumulator, add the two column ranges, scale, store, release the
//              accumulator.  PLAIN: a warp writes its 32 rows x 32 columns into a swizzled 4 KB staging buffer
//              and one thread stores it by TMA (the engine clips what lies outside the matrix); with
//              N < 32, 16x256b loads stored straight from registers.  LINEAR:
//              32x32b loads (a thread holds one row, 16 columns at a time), transposed through a per-warp
//              shared-memory buffer, stored as 64-byte row pieces.
// Accumulators are double buffered in tensor memory (2 x 256 columns), so the epilogue of tile t
// overlaps the MMAs of tile t+1, and a 3-8 stage shared-memory ring overlaps loads with MMAs.
// Every role walks its tiles with a forward-moving cursor (TileWalker): no division per tile.
//
// Row maps: PLAIN (row r of tile t is r + 128 t; used for the radial multilayer perceptron, N may be
// several 128-column tiles) and LINEAR (rows are the (node, m) pairs of one (element, l) problem of the
// per-l Linear / ElementalLinear operator, with the weight matrix selected per tile).
//
// Every wait on an mbarrier is bounded; on a time-out the role records a code in *status and leaves
// its loop, the others time out in turn, and the CTA still frees its tensor memory and returns.
#include <cuda.h>

#include <cstdlib>
#include <cstring>

#include "common.cuh"
#include "tc_ptx.cuh"

namespace cmace {

constexpr int GT_MAX_STAGES = 8;
constexpr int GT_TILE_M = 128;
constexpr int GT_KBLOCK = 32;                       // floats per K block = one 128-byte swizzle row
constexpr int GT_A_SLAB = GT_TILE_M * 128;          // bytes of one A image (hi or lo) per stage
constexpr int GT_PRODUCER_WARPS = 8;                 // 8 measured best (4: 0.47 ms, 8: 0.36 ms, 16: 0.59 ms on the Linear case)
constexpr int GT_ROWS_PER_THREAD = GT_TILE_M / (GT_PRODUCER_WARPS * 4);  // 8 threads cover one row segment
constexpr int GT_ROW_STEP = GT_PRODUCER_WARPS * 4;                       // rows between a thread's row segments
constexpr int GT_EPILOGUE_WARPS = 8;
constexpr int GT_THREADS = (GT_PRODUCER_WARPS + 1 + GT_EPILOGUE_WARPS + 1) * 32;
constexpr int GT_SMEM_BUDGET = 227 * 1024 - 2048;    // dynamic shared memory (the static barriers count against the same 227 KB)
constexpr int GT_TMEM_COLS = 512;                   // two accumulators of 2 x 128 columns
constexpr int GT_PREFETCH = 2;                      // K blocks of global loads in flight per producer thread
constexpr int GT_EP_STRIDE = 20;                    // floats per row of an epilogue transpose buffer (16 + padding)
constexpr int GT_EP_BYTES = 8 * 32 * GT_EP_STRIDE * 4;  // one buffer per epilogue warp, 20 KB in all
constexpr int GT_EP_TMA_BYTES = 8 * 32 * 128;       // PLAIN with TMA stores: 32 rows x 128 bytes per epilogue warp

// GRADR: the A operand is never in memory.  Row e, column l*C + c of A is the radial-weight gradient of the message
// passing, X[sender(e), c] * sum_{m in l} Y[m, e] * G[receiver(e), m, c]; the producer warps form it on the fly.
enum { GT_MODE_PLAIN = 0, GT_MODE_LINEAR = 1, GT_MODE_GRADR = 2 };

struct GemmArgs {
  const float *A;
  const float *packed;          // [nmat][n_tiles][k_blocks][hi|lo][npad rows x 128 B]
  float *out;
  const int32_t *node_order;    // LINEAR mode, may be null
  const int32_t *elem_start;    // LINEAR mode, may be null
  int32_t *status;              // device int, may be null
  int64_t M;                    // PLAIN: rows; LINEAR: nodes
  int K, N;
  int nelements;
  int mode;
  float scale;
  int n_tiles, k_blocks, npad;  // packing geometry: N tiles of <= 128 columns, npad rows per B image
  int64_t total_tiles;          // upper bound of the tile index space
  int stages, stage_bytes;      // shared-memory ring: depth and bytes per stage (A hi+lo, B hi+lo)
  int b_resident;               // PLAIN: bytes of this CTA's B images kept in shared memory for the whole kernel, or 0
  int a_lo_tmem;                // PLAIN: 1 when the residual image of A lives in tensor memory (kernel variant TS)
  int ep_tma;                   // PLAIN: 1 when the epilogue stores tiles with TMA from a staging buffer
  // GRADR: X [Ns, C] sender features, G [Nr, 16, C] gradient of the messages, Y [16, M] harmonics, edge lists [M]
  const float *gx, *gg, *gy;
  const int32_t *sender, *receiver;
  int C;
  int g_stage_bytes;            // GRADR: shared memory behind the ring and the epilogue buffers for staged G rows
  int b_slots;                  // GRADR: depth of the separate ring of B blocks behind the staged G rows
  int lin_tma;                  // LINEAR: rows move by TMA through rank-3 tensor maps (nodes in storage order)
};

// LINEAR with lin_tma: [nodes, 16, K] in and [nodes, 16, N] out, per l a box of (columns, 2l+1 components, nodes)
struct LinMaps {
  CUtensorMap in[4], out[4];
};
// rows a quarter of a tile (32 tensor-memory lanes) holds: whole nodes only, so that a box covers it
__host__ __device__ constexpr int lin_nodes_per_quarter(int l) { return 32 / (2 * l + 1); }

// ---- tile bookkeeping ----------------------------------------------------------------------------
struct Tile {
  bool valid;
  int64_t row0;       // PLAIN: first row; LINEAR: first local row of the (element, l) problem
  int64_t seg_begin;  // LINEAR: first slot of the element in node_order
  int64_t seg_rows;   // LINEAR: rows of the problem
  int l, nl, mat, ntile;
  int64_t node0;      // LINEAR with lin_tma: first node slot of the tile; quarter q holds nodes node0 + q nq .. + nq - 1
  int64_t node_end;   //   one past the last node of the tile's (element, l) problem
  int nq;
};

// LINEAR: the (l, element) problems in the order their tiles are numbered (l outer, element inner), built once
// per CTA in shared memory.  Every role of the kernel walks its tiles in increasing order, so locating a tile is a
// cursor that moves forward: no division or search per tile (one thread runs the MMA role, and scalar code
// there costs about ten cycles per instruction: a handful of integer divisions per tile used to cost more than
// the tile's MMAs).
constexpr int GT_MAX_PROBLEMS = 512;   // 4 x 128 elements
struct ProblemTable {
  int32_t tile_begin[GT_MAX_PROBLEMS + 1];
  int32_t seg_begin[GT_MAX_PROBLEMS];
  int32_t seg_rows[GT_MAX_PROBLEMS];
};

// filled by all threads of the CTA; the caller synchronises afterwards
__device__ __forceinline__ void build_problem_table(const GemmArgs &g, ProblemTable *tab) {
  const int nprob = 4 * g.nelements;
  for (int p = threadIdx.x; p < nprob; p += blockDim.x) {
    const int l = p / g.nelements, z = p - l * g.nelements;
    const int32_t b = g.elem_start ? g.elem_start[z] : 0;
    const int64_t cnt = g.elem_start ? (int64_t)g.elem_start[z + 1] - b : g.M;
    const uint32_t rows = (uint32_t)(cnt * (2 * l + 1));   // fits 32 bits (checked on the host)
    tab->seg_begin[p] = b;
    tab->seg_rows[p] = (int32_t)rows;
    const uint32_t per_tile = 4u * (uint32_t)lin_nodes_per_quarter(l);   // lin_tma: nodes per tile
    tab->tile_begin[p + 1] = g.lin_tma ? (int32_t)(((uint32_t)cnt + per_tile - 1) / per_tile)
                                       : (int32_t)((rows + GT_TILE_M - 1) / GT_TILE_M);   // count; prefix-summed below
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int32_t acc = 0;
    tab->tile_begin[0] = 0;
    for (int p = 0; p < nprob; p++) {
      acc += tab->tile_begin[p + 1];
      tab->tile_begin[p + 1] = acc;
    }
  }
}

// The tiles of this CTA in increasing order.  PLAIN: tile t = (row tile, column tile) with the column tile fastest,
// or, with resident B images, a fixed column tile per CTA and row tiles blockIdx / n_tiles + j * (CTAs per column tile).
template <int MODE>
struct TileWalker {
  int64_t t, total, rt, rt_step, M;
  int ntile, nt_step, n_tiles;
  const ProblemTable *tab;
  int nprob, nelements, prob, l, z;
  bool started;

  __device__ __forceinline__ TileWalker(const GemmArgs &g, const ProblemTable *tab_) {
    started = false;
    t = blockIdx.x;
    total = g.total_tiles;
    M = g.M;
    n_tiles = g.n_tiles;
    tab = tab_;
    nelements = g.nelements;
    nprob = 4 * g.nelements;
    prob = l = z = 0;
    rt = 0;
    ntile = 0;
    rt_step = 0;
    nt_step = 0;
    if (MODE != GT_MODE_LINEAR) {
      rt = blockIdx.x / (uint32_t)n_tiles;
      ntile = (int)(blockIdx.x - (uint32_t)rt * (uint32_t)n_tiles);
      rt_step = gridDim.x / (uint32_t)n_tiles;
      nt_step = g.b_resident ? 0 : (int)(gridDim.x - (uint32_t)rt_step * (uint32_t)n_tiles);
    }
  }

  // moves to the next tile; false when the CTA has no more
  __device__ __forceinline__ bool next(Tile &T) {
    if (started) {
      t += gridDim.x;
      if (MODE != GT_MODE_LINEAR) {
        rt += rt_step;
        ntile += nt_step;
        if (ntile >= n_tiles) {
          ntile -= n_tiles;
          rt++;
        }
      }
    }
    started = true;
    T.valid = false;
    if (t >= total) return false;
    if (MODE != GT_MODE_LINEAR) {
      T.row0 = rt * GT_TILE_M;
      if (T.row0 >= M) return false;   // padded index space of the resident-B mode: row tiles only grow
      T.seg_begin = 0;
      T.seg_rows = M;
      T.l = 0;
      T.nl = 1;
      T.mat = 0;
      T.ntile = ntile;
      T.valid = true;
      return true;
    }
    while (prob < nprob && t >= tab->tile_begin[prob + 1]) {
      prob++;
      if (++z == nelements) {
        z = 0;
        l++;
      }
    }
    if (prob >= nprob) return false;
    T.row0 = (t - tab->tile_begin[prob]) * GT_TILE_M;
    T.nq = lin_nodes_per_quarter(l);
    T.node0 = tab->seg_begin[prob] + (t - tab->tile_begin[prob]) * 4 * T.nq;
    T.node_end = tab->seg_begin[prob] + tab->seg_rows[prob] / (2 * l + 1);
    T.seg_begin = tab->seg_begin[prob];
    T.seg_rows = tab->seg_rows[prob];
    T.l = l;
    T.nl = 2 * l + 1;
    T.mat = z * 4 + l;
    T.ntile = 0;
    T.valid = true;
    return true;
  }
};

// global row (in units of rows of A / out) of local row r of a tile, or -1
template <int MODE>
__device__ __forceinline__ int64_t global_row(const GemmArgs &g, const Tile &T, int r) {
  const int64_t lr = T.row0 + r;
  if (lr >= T.seg_rows) return -1;
  if (MODE != GT_MODE_LINEAR) return lr;
  // rows of one (element, l) problem fit 32 bits (checked on the host); constant divisors compile to a multiplication
  const uint32_t lr32 = (uint32_t)lr;
  uint32_t q;
  switch (T.l) {
    case 0: q = lr32; break;
    case 1: q = lr32 / 3u; break;
    case 2: q = lr32 / 5u; break;
    default: q = lr32 / 7u; break;
  }
  const int64_t slot = T.seg_begin + q;
  const int64_t node = g.node_order ? (int64_t)g.node_order[slot] : slot;
  return node * 16 + T.l * T.l + (int)(lr32 - q * (uint32_t)T.nl);
}

__device__ __forceinline__ void report(const GemmArgs &g, int code) {
  if (g.status) atomicCAS(g.status, 0, code);
}

// TS: the residual image lo = tf32(a - trunc(a)) of A goes to tensor memory instead of shared memory and the
// Alo*Bhi product reads its A operand from there.  Shared-memory bandwidth is what the roles of this kernel compete
// for; this takes the image's 16 KB store and its 16 KB read by the tensor core out of every pipeline item.  Needs
// room in tensor memory next to the accumulators: two accumulators of 2 npad columns + 32 columns per ring slot.
// CC: compile-time channel count of the GRADR producers (0: read it from the arguments)
// OA: PLAIN with the three product terms in ONE set of accumulator columns (three MMAs per K step instead of two on a
// double-width B operand): two accumulators then take 2 npad columns, which leaves room for the residual images of a
// 128-column tile in tensor memory; [E,64]x[64,512] went from 1.49 to 1.37 ms with it.
// EW: epilogue warps, 8 (two per tensor-memory lane quarter, alternate 32-column chunks) or 4.  GRADR runs with 4:
// its narrow output leaves the epilogue idle most of the time, and 14 warps instead of 18 give every thread 128
// registers instead of 96, which is what its producer warps were short of (2.73 -> 2.35 ms).
template <int MODE, bool TS = false, int CC = 0, int EW = GT_EPILOGUE_WARPS, bool OA = false>
__global__ void __launch_bounds__((GT_PRODUCER_WARPS + 1 + EW + 1) * 32, 1)
    gemm3x_tf32_kernel(const GemmArgs g, const __grid_constant__ CUtensorMap tmap,
                       const __grid_constant__ CUtensorMap tmap_out, const __grid_constant__ LinMaps lin_maps) {
  extern __shared__ __align__(1024) unsigned char smem[];
  __shared__ __align__(8) uint64_t bars[3 * GT_MAX_STAGES + 9];
  __shared__ uint32_t tmem_base_slot;
  __shared__ int32_t tab_words[MODE == GT_MODE_LINEAR ? sizeof(ProblemTable) / 4 : 1];
  const ProblemTable *tab = reinterpret_cast<const ProblemTable *>(tab_words);
  if (MODE == GT_MODE_LINEAR) build_problem_table(g, reinterpret_cast<ProblemTable *>(tab_words));

  // dynamic smem base rounded up to 1024 bytes (the swizzle pattern repeats every 1024 bytes)
  const uint32_t smem_first = (smem_u32(smem) + 1023u) & ~1023u;
  const uint32_t smem_base = smem_first + (uint32_t)g.b_resident;   // the ring starts behind the resident B images
  const uint32_t full_bar = smem_u32(&bars[0]);                 // + 8*s
  const uint32_t empty_bar = smem_u32(&bars[GT_MAX_STAGES]);        // + 8*s
  const uint32_t acc_full = smem_u32(&bars[2 * GT_MAX_STAGES]);     // + 8*a
  const uint32_t acc_empty = smem_u32(&bars[2 * GT_MAX_STAGES + 2]);
  const uint32_t tma_full = smem_u32(&bars[2 * GT_MAX_STAGES + 4]);   // + 8*s, PLAIN: A tile and B block landed
  const uint32_t b_full = smem_u32(&bars[3 * GT_MAX_STAGES + 4]);     // PLAIN with resident B: images landed
  const uint32_t g_full = smem_u32(&bars[3 * GT_MAX_STAGES + 5]);     // + 8*buf, GRADR: staged G rows of a tile landed
  const uint32_t g_empty = smem_u32(&bars[3 * GT_MAX_STAGES + 7]);    // + 8*buf, GRADR: every producer warp is done with them
  const int GT_STAGES = g.stages;
  const uint32_t GT_STAGE_BYTES = (uint32_t)g.stage_bytes;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < GT_STAGES; s++) {
      // LINEAR, GRADR: one arrival per producer warp + the expect_tx arrival of the B copy; PLAIN: converters only
      mbar_init(full_bar + 8 * s, GT_PRODUCER_WARPS + ((MODE == GT_MODE_PLAIN || g.lin_tma) ? 0 : 1));
      mbar_init(tma_full + 8 * s, 1);         // the loader's expect_tx arrival (+ the copies' bytes)
      mbar_init(empty_bar + 8 * s, 1);        // one tcgen05.commit
    }
    for (int a = 0; a < 2; a++) {
      mbar_init(acc_full + 8 * a, 1);         // one tcgen05.commit
      mbar_init(acc_empty + 8 * a, EW);  // one arrival per epilogue warp
    }
    mbar_init(b_full, 1);
    for (int b2 = 0; b2 < 2; b2++) {
      mbar_init(g_full + 8 * b2, 1);                      // the loader's expect_tx arrival (+ the copy's bytes)
      mbar_init(g_empty + 8 * b2, GT_PRODUCER_WARPS);     // one arrival per producer warp
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == GT_PRODUCER_WARPS) tmem_alloc(smem_u32(&tmem_base_slot), GT_TMEM_COLS);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = tmem_base_slot;

  const int k_blocks = g.k_blocks;
  const uint32_t b_image = (uint32_t)g.npad * 128u;  // bytes of one B image
  const uint32_t b_off = TS ? GT_A_SLAB : 2 * GT_A_SLAB;          // the stage's B block follows its A image(s)
  // tensor-memory columns between the accumulators; TS: ring of residual images behind them, 32 columns a slot
  // LINEAR with TS: the three product terms share one set of npad columns (ONE_ACC), which leaves room for the ring
  // of residual images next to two accumulators of 128 columns
  constexpr bool ONE_ACC = (MODE == GT_MODE_LINEAR && TS) || OA;
  const uint32_t acc_stride = ONE_ACC ? (uint32_t)g.npad : (TS ? 2u * (uint32_t)g.npad : 256u);
  const uint32_t lo_ring = tmem_base + (ONE_ACC ? 2u : 4u) * (uint32_t)g.npad;
  const int items = k_blocks;                                     // pipeline items per tile

  if (((MODE == GT_MODE_PLAIN && TS) || (MODE == GT_MODE_LINEAR && TS && g.lin_tma)) && warp < GT_PRODUCER_WARPS) {
    // ================================ converters, residual image to tensor memory ================================
    // A thread owns one row of the tile (the tensor-memory lane its warp may access) and 16 of the K block's 32
    // columns: four 16-byte shared-memory loads (conflict-free: the 128-byte swizzle puts the same logical chunk of
    // eight consecutive rows into eight different bank groups), three ALU operations per float, one tcgen05.st.
    const int q = warp & 3, hf = warp >> 2;
    const int r = q * 32 + lane;
    uint32_t soff[4];
#pragma unroll
    for (int c = 0; c < 4; c++) soff[c] = (uint32_t)sw128_offset(r, 4 * hf + c);
    const uint32_t t_lo = lo_ring + ((uint32_t)(q * 32) << 16) + 16u * (uint32_t)hf;
    int stage = 0;
    uint32_t phase = 0;
    bool ok = true;
    TileWalker<MODE> tiles(g, tab);
    Tile T;
    while (ok && tiles.next(T)) {
      for (int kb = 0; kb < items; kb++) {
        uint32_t got = 1;
        if (lane == 0) got = mbar_wait(tma_full + 8 * stage, phase) ? 1u : 0u;
        got = __shfl_sync(0xffffffffu, got, 0);
        if (!got) {
          report(g, 1);
          ok = false;
          break;
        }
        const uint32_t sA = smem_base + stage * GT_STAGE_BYTES;
        uint32_t lo[16];
#pragma unroll
        for (int c = 0; c < 4; c++) {
          float4 a;
          asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];"
                       : "=f"(a.x), "=f"(a.y), "=f"(a.z), "=f"(a.w)
                       : "r"(sA + soff[c])
                       : "memory");
          lo[4 * c] = __float_as_uint(to_tf32(a.x - __uint_as_float(__float_as_uint(a.x) & 0xFFFFE000u)));
          lo[4 * c + 1] = __float_as_uint(to_tf32(a.y - __uint_as_float(__float_as_uint(a.y) & 0xFFFFE000u)));
          lo[4 * c + 2] = __float_as_uint(to_tf32(a.z - __uint_as_float(__float_as_uint(a.z) & 0xFFFFE000u)));
          lo[4 * c + 3] = __float_as_uint(to_tf32(a.w - __uint_as_float(__float_as_uint(a.w) & 0xFFFFE000u)));
        }
        tmem_st16(t_lo + 32u * (uint32_t)stage, lo);
        tmem_st_wait();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(full_bar + 8 * stage);
        if (++stage == GT_STAGES) {
          stage = 0;
          phase ^= 1;
        }
      }
    }
  } else if (MODE == GT_MODE_PLAIN && warp < GT_PRODUCER_WARPS) {
    // ================================ converters ================================
    // The loader's TMA puts the raw float32 tile straight into the stage's "hi" image: kind::tf32 reads
    // the top 19 bits of each float32 and ignores the low 13 mantissa bits (checked on the hardware), so
    // the raw tile IS the hi operand, hi = trunc_tf32(a).  These warps only add the residual image
    // lo = tf32(a - hi): one shared-memory load, three ALU operations per float and one store per 16 bytes.
    // They are bound by instruction issue, hence the tiny loop.
    const int p = threadIdx.x;       // 0..255
    const int chunk = p & 7;         // 16-byte chunk of the 128-byte row segment
    const int rbase = p >> 3;        // rows rbase + GT_ROW_STEP * i
    uint32_t soff[GT_ROWS_PER_THREAD];
#pragma unroll
    for (int i = 0; i < GT_ROWS_PER_THREAD; i++) soff[i] = (uint32_t)sw128_offset(rbase + GT_ROW_STEP * i, chunk);
    int stage = 0;
    uint32_t phase = 0;
    bool ok = true;
    TileWalker<MODE> tiles(g, tab);
    Tile T;
    while (ok && tiles.next(T)) {
      for (int kb = 0; kb < k_blocks; kb++) {
        uint32_t got = 1;
        if (lane == 0) got = mbar_wait(tma_full + 8 * stage, phase) ? 1u : 0u;
        got = __shfl_sync(0xffffffffu, got, 0);
        if (!got) {
          report(g, 1);
          ok = false;
          break;
        }
        const uint32_t sA = smem_base + stage * GT_STAGE_BYTES;
#pragma unroll
        for (int i = 0; i < GT_ROWS_PER_THREAD; i++) {
          float4 a, lo;
          asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];"
                       : "=f"(a.x), "=f"(a.y), "=f"(a.z), "=f"(a.w)
                       : "r"(sA + soff[i])
                       : "memory");
          lo.x = to_tf32(a.x - __uint_as_float(__float_as_uint(a.x) & 0xFFFFE000u));
          lo.y = to_tf32(a.y - __uint_as_float(__float_as_uint(a.y) & 0xFFFFE000u));
          lo.z = to_tf32(a.z - __uint_as_float(__float_as_uint(a.z) & 0xFFFFE000u));
          lo.w = to_tf32(a.w - __uint_as_float(__float_as_uint(a.w) & 0xFFFFE000u));
          asm volatile("st.shared.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(sA + GT_A_SLAB + soff[i]), "f"(lo.x),
                       "f"(lo.y), "f"(lo.z), "f"(lo.w)
                       : "memory");
        }
        fence_proxy_async();
        __syncwarp();
        if (lane == 0) mbar_arrive(full_bar + 8 * stage);
        if (++stage == GT_STAGES) {
          stage = 0;
          phase ^= 1;
        }
      }
    }
  } else if (MODE == GT_MODE_GRADR && warp < GT_PRODUCER_WARPS) {
    // ================================ producers, operand formed on the fly ================================
    // (always the TS variant, and here BOTH images of A go to tensor memory: the raw values as the hi image, the
    // residual a - trunc(a) as the lo image, 32 columns each per slot.  No shared-memory store, hence no proxy fence
    // in the hand-over: 2.32 -> 2.20 ms with 128 registers a thread; with 96 it had been slower.)
    // A thread owns one row of the tile = one edge e (the tensor-memory lane its warp may write) and 16 of a K
    // block's 32 columns.  K block (l, cb) covers the columns l*C + 32 cb .. + 31 of A; the items of a tile run
    // cb-outer, l-inner (the order of a sum does not matter to the accumulator, the producer only has to fetch the
    // matching B block), so the sender's features x = X[s, 32 cb + 16 hf .. + 15] stay in registers for four items
    // and the next column block's are already on their way.  Per item: q = sum_{m in l} Y[m, e] * G[r, m, same
    // columns], a = x * q.  Y[0..15, e] lives in registers for the whole tile.  The rows of a tile are consecutive
    // edges of the receiver-sorted list, so their receivers form a short contiguous range: the loader warp copies
    // the G rows of that range (8 KB per receiver at C = 128, one contiguous piece) into one of two shared-memory
    // buffers a tile ahead, and the inner loop reads them from there (warp-wide broadcasts); receivers beyond
    // the staged range, when a tile spans many low-degree receivers, are read from global memory.
    // The B blocks are copied by the loader warp into a ring with the same slot index and barriers as the A images;
    // four slots: two accumulators of 2 x 64 columns leave 256 tensor-memory columns for the images.
    const int q4 = warp & 3, hf = warp >> 2;
    const int r = q4 * 32 + lane;
    const int C = CC ? CC : g.C, ncb = C >> 5;
    const uint32_t g_stage0 = smem_base + GT_STAGES * GT_STAGE_BYTES;
    const uint32_t g_half = (uint32_t)g.g_stage_bytes / 2u;
    const int max_staged = (int)(g_half / (uint32_t)(16 * C * 4));
    const uint32_t t_lo = lo_ring + ((uint32_t)(q4 * 32) << 16) + 16u * (uint32_t)hf;
    int stage = 0, pending_stage = -1;
    uint32_t phase = 0;
    bool ok = true;
    auto hand_over = [&]() {
      if (pending_stage < 0) return;
      tmem_st_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(full_bar + 8 * pending_stage);
      pending_stage = -1;
    };
    TileWalker<MODE> tiles(g, tab);
    Tile T;
    for (int t = 0; ok && tiles.next(T); t++) {
      const int buf = t & 1;
      const int64_t e_last = T.row0 + GT_TILE_M - 1 < g.M ? T.row0 + GT_TILE_M - 1 : g.M - 1;
      const int r_first = __ldg(g.receiver + T.row0);
      const int r_count = __ldg(g.receiver + e_last) - r_first + 1;
      const int nstaged = r_count < max_staged ? r_count : max_staged;
      const int64_t e = T.row0 + r;
      const bool in = e < g.M;
      const int64_t ee = in ? e : T.row0;
      const int my_recv = __ldg(g.receiver + ee);
      const float *xrow = g.gx + (int64_t)__ldg(g.sender + ee) * C + 16 * hf;
      float y[16];
#pragma unroll
      for (int m = 0; m < 16; m++) y[m] = in ? __ldg(g.gy + (int64_t)m * g.M + ee) : 0.f;
      const bool staged = my_recv - r_first < nstaged;
      const bool warp_staged = __all_sync(0xffffffffu, staged);
      const uint32_t gs = g_stage0 + buf * g_half + (uint32_t)((my_recv - r_first) * 16 * C + 16 * hf) * 4u;
      const float *gg = g.gg + (int64_t)my_recv * 16 * C + 16 * hf;
      {
        uint32_t got = 1;
        if (lane == 0) got = mbar_wait(g_full + 8 * buf, (uint32_t)(t >> 1) & 1u) ? 1u : 0u;
        if (!__shfl_sync(0xffffffffu, got, 0)) {
          report(g, 8);
          ok = false;
          break;
        }
      }
      // Arithmetic on register pairs: fma.rn.f32x2 / mul.rn.f32x2 / sub.rn.f32x2 handle two floats per instruction,
      // and the inner loop of this role is bound by instruction issue (eight warps feed the tensor core).
      unsigned long long xn2[8];
      {
        const ulonglong2 *xp = reinterpret_cast<const ulonglong2 *>(xrow);
#pragma unroll
        for (int c = 0; c < 4; c++) {
          const ulonglong2 v = __ldg(xp + c);
          xn2[2 * c] = v.x;
          xn2[2 * c + 1] = v.y;
        }
      }
#pragma unroll 1
      for (int cb = 0; ok && cb < ncb; cb++) {
        unsigned long long x2[8];
#pragma unroll
        for (int c = 0; c < 8; c++) x2[c] = xn2[c];
        if (cb + 1 < ncb) {
          const ulonglong2 *xp = reinterpret_cast<const ulonglong2 *>(xrow + 32 * (cb + 1));
#pragma unroll
          for (int c = 0; c < 4; c++) {
            const ulonglong2 v = __ldg(xp + c);
            xn2[2 * c] = v.x;
            xn2[2 * c + 1] = v.y;
          }
        }
#pragma unroll
        for (int l = 0; l < 4; l++) {
          unsigned long long a2[8];
#pragma unroll
          for (int c = 0; c < 8; c++) a2[c] = 0ull;
#pragma unroll
          for (int m = l * l; m < (l + 1) * (l + 1); m++) {
            unsigned long long yy;
            asm("mov.b64 %0, {%1, %1};" : "=l"(yy) : "f"(y[m]));
            unsigned long long gv[8];
            if (warp_staged) {
              const uint32_t ga = gs + (uint32_t)(m * C + 32 * cb) * 4u;
#pragma unroll
              for (int c = 0; c < 4; c++)
                asm("ld.shared.v2.b64 {%0, %1}, [%2];" : "=l"(gv[2 * c]), "=l"(gv[2 * c + 1]) : "r"(ga + 16u * c));
            } else {
              const ulonglong2 *gp = reinterpret_cast<const ulonglong2 *>(gg + m * C + 32 * cb);
#pragma unroll
              for (int c = 0; c < 4; c++) {
                const ulonglong2 v = __ldg(gp + c);
                gv[2 * c] = v.x;
                gv[2 * c + 1] = v.y;
              }
            }
#pragma unroll
            for (int c = 0; c < 8; c++) asm("fma.rn.f32x2 %0, %1, %2, %0;" : "+l"(a2[c]) : "l"(yy), "l"(gv[c]));
          }
#pragma unroll
          for (int c = 0; c < 8; c++) asm("mul.rn.f32x2 %0, %0, %1;" : "+l"(a2[c]) : "l"(x2[c]));
          hand_over();   // the previous item: its stores had this item's arithmetic to complete (with 128 registers
                         // a thread this is 1.5 % faster than handing over at once; with 96 it was slower)
          // the slot (shared-memory image and tensor-memory columns) is free once the MMAs that read it completed
          uint32_t got = 1;
          if (lane == 0) got = mbar_wait(empty_bar + 8 * stage, phase ^ 1) ? 1u : 0u;
          if (!__shfl_sync(0xffffffffu, got, 0)) {
            report(g, 1);
            ok = false;
            break;
          }
          // hi image: the raw values (the tensor core ignores the low 13 mantissa bits of its operands);
          // residual image: a - trunc(a), exact in float32 and at most 2^-10 |a|; it is read with the same truncation,
          // which leaves an error below 2^-20 |a| per element
          uint32_t lo[16], hi[16];
#pragma unroll
          for (int c = 0; c < 4; c++) {
#pragma unroll
            for (int h2 = 0; h2 < 2; h2++) {
              unsigned long long d;
              const unsigned long long tr = a2[2 * c + h2] & 0xFFFFE000FFFFE000ull;
              asm("sub.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a2[2 * c + h2]), "l"(tr));
              asm("mov.b64 {%0, %1}, %2;" : "=r"(lo[4 * c + 2 * h2]), "=r"(lo[4 * c + 2 * h2 + 1]) : "l"(d));
              asm("mov.b64 {%0, %1}, %2;" : "=r"(hi[4 * c + 2 * h2]), "=r"(hi[4 * c + 2 * h2 + 1]) : "l"(a2[2 * c + h2]));
            }
          }
          tmem_st16(t_lo + 32u * (uint32_t)stage, lo);
          tmem_st16(t_lo + 32u * (uint32_t)(GT_STAGES + stage), hi);   // the hi ring follows the lo ring
          pending_stage = stage;
          if (++stage == GT_STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
      }
      // this warp no longer reads the tile's G rows: the loader may overwrite the buffer
      __syncwarp();
      if (lane == 0) mbar_arrive(g_empty + 8 * buf);
    }
    hand_over();
  } else if (MODE == GT_MODE_LINEAR && warp < GT_PRODUCER_WARPS) {
    // ================================ producers ================================
    // Work items are (tile, K block) pairs in the order the MMA warp consumes them.  Loads run
    // GT_PREFETCH items ahead of the conversion in a register ring, so that enough bytes are in flight
    // per SM to cover HBM latency (about a microsecond) independently of the shared-memory ring depth.
    // (LINEAR always runs as the TS variant.)  The residual image goes to tensor memory, which a warp reaches only
    // for the 32 lanes (= rows) of its quarter: warp (q, hf) loads rows 32 q .. 32 q + 31, the 64-byte half hf of
    // their 128-byte K-block segments (4 threads a row, rows (lane >> 2) + 8 i), writes the raw values to the
    // shared-memory image, and then every lane reads ITS row's half back (all of it written by this warp) to form the
    // residuals.
    const int chunk = 4 * (warp >> 2) + (lane & 3);      // 16-byte chunk of the 128-byte row segment
    const int rbase = 32 * (warp & 3) + (lane >> 2);     // rows rbase + row_step * i
    constexpr int row_step = 8;
    // head: the next (tile, K block) item whose loads have not been issued yet
    struct Head {
      Tile T;
      int kb;
      bool valid;
      int64_t grow[GT_ROWS_PER_THREAD];
    } head;
    TileWalker<MODE> tiles(g, tab);
    auto advance = [&]() {
      if (++head.kb < k_blocks && head.valid) return;
      head.kb = 0;
      head.valid = tiles.next(head.T);
      if (!head.valid) return;
#pragma unroll
      for (int i = 0; i < GT_ROWS_PER_THREAD; i++) head.grow[i] = global_row<MODE>(g, head.T, rbase + row_step * i);
    };
    // returns -1 when there is no item left (otherwise the index of the item's B block, which the loader warp copies)
    auto issue = [&](float4 (&v)[GT_ROWS_PER_THREAD]) -> int64_t {
      if (!head.valid) return -1;
      const int k0 = head.kb * GT_KBLOCK + chunk * 4;
#pragma unroll
      for (int i = 0; i < GT_ROWS_PER_THREAD; i++) {
        v[i] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (head.grow[i] >= 0 && k0 < g.K)
          v[i] = __ldg(reinterpret_cast<const float4 *>(g.A + head.grow[i] * g.K + k0));
      }
      const int64_t bblock = (int64_t)(head.T.mat * g.n_tiles + head.T.ntile) * k_blocks + head.kb;
      advance();
      return bblock;
    };
    int stage = 0;
    uint32_t phase = 0;
    // returns false on a timed-out wait
    auto commit = [&](const float4 (&v)[GT_ROWS_PER_THREAD]) -> bool {
      // lane 0 polls the barrier for the warp
      uint32_t got = 1;
      if (lane == 0) got = mbar_wait(empty_bar + 8 * stage, phase ^ 1) ? 1u : 0u;
      got = __shfl_sync(0xffffffffu, got, 0);
      if (!got) {
        report(g, 1);
        return false;
      }
      const uint32_t sA = smem_base + stage * GT_STAGE_BYTES;
      // (the B block of the item is copied by the loader warp into a ring of its own)
#pragma unroll
      for (int i = 0; i < GT_ROWS_PER_THREAD; i++) {
        const uint32_t off = (uint32_t)sw128_offset(rbase + row_step * i, chunk);
        asm volatile("st.shared.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(sA + off), "f"(v[i].x), "f"(v[i].y), "f"(v[i].z),
                     "f"(v[i].w)
                     : "memory");
      }
      __syncwarp();
      const int q = warp & 3, hf = warp >> 2;
      uint32_t lo[16];
#pragma unroll
      for (int c = 0; c < 4; c++) {
        float4 a;
        asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];"
                     : "=f"(a.x), "=f"(a.y), "=f"(a.z), "=f"(a.w)
                     : "r"(sA + (uint32_t)sw128_offset(32 * q + lane, 4 * hf + c))
                     : "memory");
        lo[4 * c] = __float_as_uint(to_tf32(a.x - __uint_as_float(__float_as_uint(a.x) & 0xFFFFE000u)));
        lo[4 * c + 1] = __float_as_uint(to_tf32(a.y - __uint_as_float(__float_as_uint(a.y) & 0xFFFFE000u)));
        lo[4 * c + 2] = __float_as_uint(to_tf32(a.z - __uint_as_float(__float_as_uint(a.z) & 0xFFFFE000u)));
        lo[4 * c + 3] = __float_as_uint(to_tf32(a.w - __uint_as_float(__float_as_uint(a.w) & 0xFFFFE000u)));
      }
      tmem_st16(lo_ring + 32u * (uint32_t)stage + ((uint32_t)(q * 32) << 16) + 16u * (uint32_t)hf, lo);
      tmem_st_wait();
      tc_fence_before();
      fence_proxy_async();
      __syncwarp();
      if (lane == 0) mbar_arrive(full_bar + 8 * stage);
      if (++stage == GT_STAGES) {
        stage = 0;
        phase ^= 1;
      }
      return true;
    };

    head.kb = k_blocks;  // forces advance() to step to the first tile
    head.valid = false;
    advance();
    // register ring: GT_PREFETCH items of global loads in flight per thread
    float4 buf[GT_PREFETCH][GT_ROWS_PER_THREAD];
    int64_t inflight[GT_PREFETCH];
#pragma unroll
    for (int d = 0; d < GT_PREFETCH; d++) inflight[d] = issue(buf[d]);
    for (bool run = true; run;) {
#pragma unroll
      for (int d = 0; d < GT_PREFETCH; d++) {
        if (inflight[d] < 0 || !commit(buf[d])) {
          run = false;
          break;
        }
        inflight[d] = issue(buf[d]);
      }
    }
  } else if (warp == GT_PRODUCER_WARPS + 1 + EW) {
    // ================================ loader ================================
    // PLAIN row map only.  Per pipeline item one thread starts two asynchronous copies that complete on the
    // stage's barrier: the TMA tile load of A (128 rows x 32 columns, 128-byte swizzle, zeros outside the
    // matrix) into the hi image, and the bulk copy of the matching pre-packed B block.  Nothing waits in
    // registers for HBM; the ring depth sets the bytes in flight.
    if (MODE == GT_MODE_GRADR && lane == 0) {
      // Per item the B block of the producers' K block order (cb outer, l inner) into a ring of g.b_slots slots; per
      // tile one bulk copy of the G rows of the NEXT tile's receiver range (contiguous) into the buffer the producers
      // released, issued in the middle of the current tile: by then every producer warp has left the previous tile
      // (they run at most a few items ahead of the tensor core), so this thread never waits long for the buffer.
      const uint32_t g_stage0 = smem_base + GT_STAGES * GT_STAGE_BYTES;
      const uint32_t g_half = (uint32_t)g.g_stage_bytes / 2u;
      const uint32_t b_ring0 = g_stage0 + (uint32_t)g.g_stage_bytes;
      const int per_receiver = 16 * g.C * 4;
      const int max_staged = (int)(g_half / (uint32_t)per_receiver);
      const int ncb = g.C >> 5;
      bool ok = true;
      auto copy_g = [&](const Tile &Tg, int tg) -> bool {
        const int buf = tg & 1;
        if (tg >= 2 && !mbar_wait(g_empty + 8 * buf, ((uint32_t)(tg >> 1) & 1u) ^ 1u)) {
          report(g, 7);
          return false;
        }
        const int64_t e_last = Tg.row0 + GT_TILE_M - 1 < g.M ? Tg.row0 + GT_TILE_M - 1 : g.M - 1;
        const int r_first = __ldg(g.receiver + Tg.row0);
        const int r_count = __ldg(g.receiver + e_last) - r_first + 1;
        const uint32_t bytes = (uint32_t)((r_count < max_staged ? r_count : max_staged) * per_receiver);
        const unsigned char *src = reinterpret_cast<const unsigned char *>(g.gg + (int64_t)r_first * 16 * g.C);
        mbar_arrive_expect_tx(g_full + 8 * buf, bytes);
        for (uint32_t off = 0; off < bytes; off += 8192u) {
          const uint32_t n = bytes - off < 8192u ? bytes - off : 8192u;
          bulk_copy_g2s(g_stage0 + buf * g_half + off, src + off, n, g_full + 8 * buf);
        }
        return true;
      };
      TileWalker<MODE> tiles(g, tab);
      Tile Tc, Tn;
      bool have = tiles.next(Tc);
      if (have) ok = copy_g(Tc, 0);
      int slot = 0;
      uint32_t bphase = 0;
      for (int t = 0; ok && have; t++) {
        const bool have_next = tiles.next(Tn);
        for (int j = 0; ok && j < 4 * ncb; j++) {
          if (j == 2 * ncb && have_next) ok = copy_g(Tn, t + 1);
          if (!ok) break;
          if (!mbar_wait(empty_bar + 8 * slot, bphase ^ 1)) {   // same slot index and barrier as the A image
            report(g, 9);
            ok = false;
            break;
          }
          const int cb = j >> 2, l = j & 3;
          const int kb = l * ncb + cb;
          const unsigned char *bsrc = reinterpret_cast<const unsigned char *>(g.packed) + (int64_t)kb * (2 * (int64_t)b_image);
          mbar_arrive_expect_tx(full_bar + 8 * slot, 2 * b_image);
          bulk_copy_g2s(b_ring0 + (uint32_t)slot * 2u * b_image, bsrc, 2 * b_image, full_bar + 8 * slot);
          if (++slot == g.b_slots) {
            slot = 0;
            bphase ^= 1;
          }
        }
        Tc = Tn;
        have = have_next;
      }
    }
    if (MODE == GT_MODE_LINEAR && TS && g.lin_tma && lane == 0) {
      // Rows by TMA: per item four box loads (one per quarter of the tile: nq whole nodes x 2l+1 components x 32
      // columns land as consecutive 128-byte rows, swizzled, at the quarter's first row) and the B block, all on the
      // slot's tma_full barrier; the converter warps then add the residual image.  Boxes that reach past the last
      // node read zeros.
      const uint32_t b_ring0 = smem_base + GT_STAGES * GT_STAGE_BYTES + (uint32_t)g.g_stage_bytes;
      int slot = 0;
      uint32_t bphase = 0;
      bool ok = true;
      TileWalker<MODE> tiles(g, tab);
      Tile T;
      while (ok && tiles.next(T)) {
        const unsigned char *bsrc = reinterpret_cast<const unsigned char *>(g.packed) +
                                    ((int64_t)(T.mat * g.n_tiles + T.ntile) * k_blocks) * (2 * (int64_t)b_image);
        const uint32_t quarter_bytes = (uint32_t)(T.nq * T.nl) * 128u;
        for (int kb = 0; kb < items; kb++) {
          if (!mbar_wait(empty_bar + 8 * slot, bphase ^ 1)) {
            report(g, 9);
            ok = false;
            break;
          }
          const uint32_t sA = smem_base + slot * GT_STAGE_BYTES, bar = tma_full + 8 * slot;
          mbar_arrive_expect_tx(bar, 4u * quarter_bytes + 2 * b_image);
#pragma unroll
          for (int q = 0; q < 4; q++)
            tma_load_3d(sA + (uint32_t)q * 4096u, &lin_maps.in[T.l], kb * GT_KBLOCK, T.l * T.l, (int)(T.node0 + q * T.nq), bar);
          bulk_copy_g2s(b_ring0 + (uint32_t)slot * 2u * b_image, bsrc + (int64_t)kb * (2 * (int64_t)b_image), 2 * b_image, bar);
          if (++slot == GT_STAGES) {
            slot = 0;
            bphase ^= 1;
          }
        }
      }
    }
    if (MODE == GT_MODE_LINEAR && TS && !g.lin_tma && lane == 0) {
      // Per item the B block of the tile's (l, element) problem into the ring of B blocks, same slot index and
      // barriers as the A images: the copy starts as soon as the slot is released, while the producers still
      // convert the items before it.
      const uint32_t b_ring0 = smem_base + GT_STAGES * GT_STAGE_BYTES + (uint32_t)g.g_stage_bytes;
      int slot = 0;
      uint32_t bphase = 0;
      bool ok = true;
      TileWalker<MODE> tiles(g, tab);
      Tile T;
      while (ok && tiles.next(T)) {
        const unsigned char *bsrc = reinterpret_cast<const unsigned char *>(g.packed) +
                                    ((int64_t)(T.mat * g.n_tiles + T.ntile) * k_blocks) * (2 * (int64_t)b_image);
        for (int kb = 0; kb < items; kb++) {
          if (!mbar_wait(empty_bar + 8 * slot, bphase ^ 1)) {
            report(g, 9);
            ok = false;
            break;
          }
          mbar_arrive_expect_tx(full_bar + 8 * slot, 2 * b_image);
          bulk_copy_g2s(b_ring0 + (uint32_t)slot * 2u * b_image, bsrc + (int64_t)kb * (2 * (int64_t)b_image), 2 * b_image,
                        full_bar + 8 * slot);
          if (++slot == GT_STAGES) {
            slot = 0;
            bphase ^= 1;
          }
        }
      }
    }
    if (MODE == GT_MODE_PLAIN && lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      if (g.b_resident) {
        const unsigned char *src = reinterpret_cast<const unsigned char *>(g.packed) +
                                   ((int64_t)(blockIdx.x % (uint32_t)g.n_tiles) * k_blocks) * (2 * (int64_t)b_image);
        mbar_arrive_expect_tx(b_full, (uint32_t)g.b_resident);
        for (uint32_t off = 0; off < (uint32_t)g.b_resident; off += 8192u) {
          const uint32_t n = (uint32_t)g.b_resident - off < 8192u ? (uint32_t)g.b_resident - off : 8192u;
          bulk_copy_g2s(smem_first + off, src + off, n, b_full);
        }
      }
      TileWalker<MODE> tiles(g, tab);
      Tile T;
      while (ok && tiles.next(T)) {
        const unsigned char *bsrc = reinterpret_cast<const unsigned char *>(g.packed) +
                                    ((int64_t)(T.mat * g.n_tiles + T.ntile) * k_blocks) * (2 * (int64_t)b_image);
        for (int kb = 0; kb < items; kb++) {
          if (!mbar_wait(empty_bar + 8 * stage, phase ^ 1)) {
            report(g, 5);
            ok = false;
            break;
          }
          const uint32_t sA = smem_base + stage * GT_STAGE_BYTES;
          mbar_arrive_expect_tx(tma_full + 8 * stage, g.b_resident ? (uint32_t)GT_A_SLAB : GT_A_SLAB + 2 * b_image);
          tma_load_2d(sA, &tmap, kb * GT_KBLOCK, (int)T.row0, tma_full + 8 * stage);
          if (!g.b_resident)
            bulk_copy_g2s(sA + b_off, bsrc + (int64_t)kb * (2 * (int64_t)b_image), 2 * b_image,
                          tma_full + 8 * stage);
          if (++stage == GT_STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
      }
    }
  } else if (warp == GT_PRODUCER_WARPS) {
    // ================================ MMA issuer ================================
    int stage = 0;
    uint32_t phase = 0;
    uint32_t acc_phase[2] = {0, 0};
    int acc = 0;
    bool ok = true;
    if (MODE == GT_MODE_PLAIN && g.b_resident) {
      uint32_t got = 1;
      if (lane == 0) got = mbar_wait(b_full, 0) ? 1u : 0u;
      if (!__shfl_sync(0xffffffffu, got, 0)) {
        report(g, 6);
        ok = false;
      }
    }
    // One thread runs the whole loop: between two batches of MMAs there is nothing but the barrier test and a few
    // integer operations, no warp-wide shuffle or re-convergence.  Whatever sits between the batches leaves the
    // tensor core idle (the issue of an MMA blocks until the previous ones have drained, so the queue is shallow).
    if (lane != 0) ok = false;
    // low / high words of the operand descriptors (umma_desc_sw128): the low word of stage 0, its step per stage
    const uint64_t d0 = umma_desc_sw128(smem_base);
    const uint32_t desc_hi32 = (uint32_t)(d0 >> 32);
    const uint32_t stage_step = GT_STAGE_BYTES >> 4;
    const uint32_t a_hi_first = (uint32_t)d0;
    const uint32_t a_lo_first = (uint32_t)umma_desc_sw128(smem_base + GT_A_SLAB);
    const uint32_t b_ring_first = (uint32_t)umma_desc_sw128(smem_base + b_off);
    const uint32_t bres_lo32 = (uint32_t)umma_desc_sw128(smem_first), bres_step = (2u * b_image) >> 4;
    uint32_t a_hi_lo32 = a_hi_first, a_lo_lo32 = a_lo_first, b_ring_lo32 = b_ring_first;
    const bool full_k = (g.K % GT_KBLOCK) == 0;
    const uint32_t bb_first = (uint32_t)umma_desc_sw128(smem_base + GT_STAGES * GT_STAGE_BYTES + (uint32_t)g.g_stage_bytes);
    TileWalker<MODE> tiles(g, tab);
    Tile T;
    while (ok && tiles.next(T)) {
      int ncols = g.N - T.ntile * 128;
      ncols = ncols > 128 ? 128 : ncols;
      const int nmma = (ncols + 15) & ~15;
      // B images are npad rows each, hi directly followed by lo: read as one operand of 2 * npad rows,
      // one MMA gives Ahi*Bhi in columns [0, npad) and Ahi*Blo in columns [npad, 2 npad)
      const uint32_t idesc2 = umma_idesc_tf32(GT_TILE_M, 2 * g.npad);
      const uint32_t idesc1 = umma_idesc_tf32(GT_TILE_M, nmma);
      if (!mbar_wait(acc_empty + 8 * acc, acc_phase[acc] ^ 1)) {
        report(g, 2);
        break;
      }
      tc_fence_after();
      const uint32_t d_tmem = tmem_base + acc * acc_stride;
      for (int kb = 0; kb < items; kb++) {
        if (!mbar_wait(full_bar + 8 * stage, phase)) {
          report(g, 3);
          ok = false;
          break;
        }
        tc_fence_after();
        {
          // Operand descriptors: only the low word (address field) changes from stage to stage and from K step to K
          // step (j * 32 bytes = 2 address units); the high word is a constant.  This thread shares its scheduler
          // with busy warps, so every instruction between two MMAs costs issue latency: the low words advance with
          // one add per item, the eight MMAs go back to back.
          const uint32_t b_lo32 = (MODE == GT_MODE_GRADR || MODE == GT_MODE_LINEAR) ? bb_first + (uint32_t)stage * bres_step
                                  : g.b_resident      ? bres_lo32 + (uint32_t)kb * bres_step
                                                      : b_ring_lo32;
          uint64_t ah[4], al[4], bh[4];
#pragma unroll
          for (int j = 0; j < 4; j++) {
            asm("mov.b64 %0, {%1, %2};" : "=l"(ah[j]) : "r"(a_hi_lo32 + 2u * j), "r"(desc_hi32));
            asm("mov.b64 %0, {%1, %2};" : "=l"(al[j]) : "r"(a_lo_lo32 + 2u * j), "r"(desc_hi32));
            asm("mov.b64 %0, {%1, %2};" : "=l"(bh[j]) : "r"(b_lo32 + 2u * j), "r"(desc_hi32));
          }
          const uint32_t a_lo_t = lo_ring + 32u * (uint32_t)stage;   // TS: K step j at + 8 j columns
          if (ONE_ACC) {
            // all three terms into the same npad columns; the B lo image follows the hi image, b_image bytes further
            const uint32_t idescn = umma_idesc_tf32(GT_TILE_M, g.npad);
            int ksteps = (g.K - kb * GT_KBLOCK + 7) / 8;
            ksteps = ksteps > 4 ? 4 : ksteps;
#pragma unroll
            for (int j = 0; j < 4; j++) {
              if (j < ksteps) {
                uint64_t bl;
                asm("mov.b64 %0, {%1, %2};" : "=l"(bl) : "r"(b_lo32 + (b_image >> 4) + 2u * j), "r"(desc_hi32));
                umma_tf32(d_tmem, ah[j], bh[j], idescn, (kb | j) != 0);
                umma_tf32_acc(d_tmem, ah[j], bl, idescn);
                umma_tf32_ts_acc(d_tmem, a_lo_t + 8u * j, bh[j], idescn);
              }
            }
          } else if (full_k && MODE == GT_MODE_GRADR) {
            const uint32_t a_hi_t = a_lo_t + 32u * (uint32_t)GT_STAGES;
#pragma unroll
            for (int j = 0; j < 4; j++) {
              umma_tf32_ts(d_tmem, a_hi_t + 8u * j, bh[j], idesc2, (kb | j) != 0);
              umma_tf32_ts_acc(d_tmem, a_lo_t + 8u * j, bh[j], idesc1);
            }
          } else if (full_k) {
            umma_tf32(d_tmem, ah[0], bh[0], idesc2, kb != 0);
            if (TS) umma_tf32_ts_acc(d_tmem, a_lo_t, bh[0], idesc1);
            else umma_tf32_acc(d_tmem, al[0], bh[0], idesc1);
#pragma unroll
            for (int j = 1; j < 4; j++) {
              umma_tf32_acc(d_tmem, ah[j], bh[j], idesc2);
              if (TS) umma_tf32_ts_acc(d_tmem, a_lo_t + 8u * j, bh[j], idesc1);
              else umma_tf32_acc(d_tmem, al[j], bh[j], idesc1);
            }
          } else {
            int ksteps = (g.K - kb * GT_KBLOCK + 7) / 8;
            ksteps = ksteps > 4 ? 4 : ksteps;
            for (int j = 0; j < ksteps; j++) {
              umma_tf32(d_tmem, ah[j], bh[j], idesc2, (kb | j) != 0);
              if (TS) umma_tf32_ts_acc(d_tmem, a_lo_t + 8u * j, bh[j], idesc1);
              else umma_tf32_acc(d_tmem, al[j], bh[j], idesc1);
            }
          }
          umma_commit(empty_bar + 8 * stage);
          if (kb == k_blocks - 1) umma_commit(acc_full + 8 * acc);
        }
        a_hi_lo32 += stage_step;
        a_lo_lo32 += stage_step;
        b_ring_lo32 += stage_step;
        if (++stage == GT_STAGES) {
          stage = 0;
          phase ^= 1;
          a_hi_lo32 = a_hi_first;
          a_lo_lo32 = a_lo_first;
          b_ring_lo32 = b_ring_first;
        }
      }
      acc_phase[acc] ^= 1;
      acc ^= 1;
    }
  } else {
    // ================================ epilogue ================================
    // Eight warps: two per tensor-memory lane quarter (a warp may only read lanes 32*(warp%4)..+31), the two
    // taking alternate 32-column chunks of the tile.  In LINEAR mode each chunk goes through a per-warp transpose
    // buffer in two 16-column halves so that the global stores are 64-byte row pieces, 8 rows per instruction;
    // in PLAIN mode the buffer does not exist (the launch reserves no bytes for it) and is never touched.
    const int q = warp & 3;                          // tensor-memory lane quarter this warp may read
    const int half = (warp - (GT_PRODUCER_WARPS + 1)) >> 2;  // which alternate chunks this warp takes
    float *ep_buf = reinterpret_cast<float *>(smem + (smem_base - smem_u32(smem)) + GT_STAGES * GT_STAGE_BYTES) +
                    (warp - (GT_PRODUCER_WARPS + 1)) * 32 * GT_EP_STRIDE;
    const int r = q * 32 + lane;            // row of the tile
    uint32_t acc_phase[2] = {0, 0};
    int acc = 0;
    TileWalker<MODE> tiles(g, tab);
    Tile T;
    while (tiles.next(T)) {
      const int64_t grow = global_row<MODE>(g, T, r);
      const int n0 = T.ntile * 128;
      int ncols = g.N - n0;
      ncols = ncols > 128 ? 128 : ncols;
      uint32_t got = 1;
      if (lane == 0) got = mbar_wait(acc_full + 8 * acc, acc_phase[acc]) ? 1u : 0u;
      if (!__shfl_sync(0xffffffffu, got, 0)) {
        report(g, 4);
        break;
      }
      tc_fence_after();
      const uint32_t taddr = tmem_base + acc * acc_stride + ((uint32_t)(q * 32) << 16);
      if (MODE != GT_MODE_LINEAR && g.ep_tma) {
        // Tile store by TMA.  Global stores from registers cost the load/store data pipe one pass per 32-byte sector
        // whatever their shape (64 KB per tile = 2048 passes, the pipe measured 70 % busy on [E,64]x[64,512]); here
        // a warp writes its 32 rows x 32 columns into a swizzled 4 KB staging buffer (eight conflict-free 16-byte
        // stores per thread) and one thread hands the buffer to the copy engine, which clips rows and columns
        // outside the matrix.
        const uint32_t stg = smem_base + GT_STAGES * GT_STAGE_BYTES + (uint32_t)(warp - (GT_PRODUCER_WARPS + 1)) * 4096u;
        for (int c0 = half * 32; c0 < ncols; c0 += 8 * EW) {
          if (lane == 0) tma_store_wait_read();   // the previous store has left the staging buffer
          __syncwarp();
#pragma unroll
          for (int h16 = 0; h16 < 2; h16++) {
            uint32_t v[16], w[16];
            tmem_ld16_nowait(taddr + (uint32_t)(c0 + 16 * h16), v);
            if (OA) {
#pragma unroll
              for (int i = 0; i < 16; i++) w[i] = 0u;
            } else {
              tmem_ld16_nowait(taddr + (uint32_t)(g.npad + c0 + 16 * h16), w);
            }
            tmem_ld_wait();
#pragma unroll
            for (int c = 0; c < 4; c++) {
              const uint32_t dst = stg + (uint32_t)sw128_offset(lane, 4 * h16 + c);
              asm volatile("st.shared.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(dst),
                           "f"((__uint_as_float(v[4 * c]) + __uint_as_float(w[4 * c])) * g.scale),
                           "f"((__uint_as_float(v[4 * c + 1]) + __uint_as_float(w[4 * c + 1])) * g.scale),
                           "f"((__uint_as_float(v[4 * c + 2]) + __uint_as_float(w[4 * c + 2])) * g.scale),
                           "f"((__uint_as_float(v[4 * c + 3]) + __uint_as_float(w[4 * c + 3])) * g.scale)
                           : "memory");
            }
          }
          fence_proxy_async();
          __syncwarp();
          // a box that starts inside the matrix: the engine clips what hangs over, a start outside is never issued
          if (lane == 0 && T.row0 + q * 32 < g.M)
            tma_store_2d(&tmap_out, n0 + c0, (int)T.row0 + q * 32, stg);
        }
      } else if (MODE != GT_MODE_LINEAR) {
        // Straight from tensor memory to global memory, no shared-memory transpose: the 16x256b load shape hands
        // thread t two rows (t/4 and t/4 + 8 of a 16-row half) and, per 8-column block, the two columns
        // 2(t%4), 2(t%4)+1 -- four neighbouring lanes hold 32 contiguous bytes of a row, so an 8-byte store per
        // lane writes whole 32-byte sectors.  Shared memory is the scarce resource of this kernel (at the TF32
        // rate the tensor core's own operand reads take most of its 128 bytes per clock): [E,64]x[64,512] went
        // from 1.98 to 1.79 ms.  With gathered rows (LINEAR) it measured the same as the staged version below.
        for (int c0 = half * 32; c0 < ncols; c0 += 8 * EW) {
#pragma unroll
          for (int hr = 0; hr < 2; hr++) {
            uint32_t v[16], w[16];
            const uint32_t ta = taddr + ((uint32_t)(16 * hr) << 16) + (uint32_t)c0;
            tmem_ld_16x256b_x4(ta, v);                 // Ahi*Bhi + Alo*Bhi
            tmem_ld_16x256b_x4(ta + g.npad, w);        // Ahi*Blo
            tmem_ld_wait();
            const int64_t gra = __shfl_sync(0xffffffffu, grow, 16 * hr + (lane >> 2));
            const int64_t grb = __shfl_sync(0xffffffffu, grow, 16 * hr + 8 + (lane >> 2));
            // One exchange with the neighbouring lane turns the 8-byte pieces into 16-byte ones: the even lane keeps
            // column blocks 0 and 1 and receives its neighbour's halves of them, the odd lane blocks 2 and 3.  A store
            // instruction then writes two whole 32-byte sectors of a row instead of one (the stores of this kernel
            // are bound by the number of requests, not by bytes).
            const bool odd = (lane & 1) != 0;
            float sv[16];
#pragma unroll
            for (int i = 0; i < 16; i++) sv[i] = (__uint_as_float(v[i]) + __uint_as_float(w[i])) * g.scale;
            float4 oa[2], ob[2];
#pragma unroll
            for (int m = 0; m < 2; m++) {
              float rc[4];
#pragma unroll
              for (int x = 0; x < 4; x++)
                rc[x] = __shfl_xor_sync(0xffffffffu, odd ? sv[4 * m + x] : sv[4 * (2 + m) + x], 1);
              oa[m] = odd ? make_float4(rc[0], rc[1], sv[4 * (2 + m)], sv[4 * (2 + m) + 1])
                          : make_float4(sv[4 * m], sv[4 * m + 1], rc[0], rc[1]);
              ob[m] = odd ? make_float4(rc[2], rc[3], sv[4 * (2 + m) + 2], sv[4 * (2 + m) + 3])
                          : make_float4(sv[4 * m + 2], sv[4 * m + 3], rc[2], rc[3]);
            }
            const int cbase = c0 + 2 * (lane & 2) + (odd ? 16 : 0);   // first column of this lane's piece m = 0
            float *pa = g.out + gra * g.N + n0 + cbase;
            float *pb = g.out + grb * g.N + n0 + cbase;
#pragma unroll
            for (int m = 0; m < 2; m++) {
              const bool col_ok = cbase + 8 * m < ncols;
              if (gra >= 0 && col_ok) *reinterpret_cast<float4 *>(pa + 8 * m) = oa[m];
              if (grb >= 0 && col_ok) *reinterpret_cast<float4 *>(pb + 8 * m) = ob[m];
            }
          }
        }
      } else if (MODE == GT_MODE_LINEAR && TS && g.lin_tma) {
        // Tile store by TMA: a warp writes 32 rows x 16 columns into a 2 KB staging buffer (64-byte rows, 64-byte
        // swizzle: conflict-free 16-byte stores) and one thread hands it to the copy engine as a box of
        // (16 columns, 2l+1 components, nq nodes) = the quarter's first nq (2l+1) rows; nodes and columns outside the
        // array are clipped.  This takes the transposes and the row stores (one pass of the load/store pipe per
        // 32-byte sector) out of the epilogue.
        const uint32_t stg = smem_base + GT_STAGES * GT_STAGE_BYTES + (uint32_t)(warp - (GT_PRODUCER_WARPS + 1)) * 2048u;
        // A quarter that reaches past the last node of its problem (the next nodes belong to another element, or
        // lie outside the array) is stored row by row from registers instead: one such tile per problem.
        const int node_q = (int)(T.node0 + q * T.nq);
        const bool whole = node_q + T.nq <= T.node_end;
        for (int c0 = half * 32; c0 < ncols; c0 += 8 * EW) {
#pragma unroll
          for (int h16 = 0; h16 < 2; h16++) {
            const int cc = c0 + 16 * h16;
            if (cc >= ncols) break;  // warp-uniform
            uint32_t v[16];
            tmem_ld16_nowait(taddr + (uint32_t)cc, v);
            tmem_ld_wait();
            if (!whole) {
              const int node = node_q + lane / T.nl, m = lane - (lane / T.nl) * T.nl;
              if (lane < T.nq * T.nl && node < T.node_end) {
                float *o = g.out + ((int64_t)node * 16 + T.l * T.l + m) * g.N + n0 + cc;
#pragma unroll
                for (int c = 0; c < 4; c++)
                  if (cc + 4 * c < ncols)
                    *reinterpret_cast<float4 *>(o + 4 * c) =
                        make_float4(__uint_as_float(v[4 * c]) * g.scale, __uint_as_float(v[4 * c + 1]) * g.scale,
                                    __uint_as_float(v[4 * c + 2]) * g.scale, __uint_as_float(v[4 * c + 3]) * g.scale);
              }
              continue;
            }
            if (lane == 0) tma_store_wait_read();   // the previous store has left the staging buffer
            __syncwarp();
#pragma unroll
            for (int c = 0; c < 4; c++)
              asm volatile("st.shared.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(stg + (uint32_t)sw64_offset(lane, c)),
                           "f"(__uint_as_float(v[4 * c]) * g.scale), "f"(__uint_as_float(v[4 * c + 1]) * g.scale),
                           "f"(__uint_as_float(v[4 * c + 2]) * g.scale), "f"(__uint_as_float(v[4 * c + 3]) * g.scale)
                           : "memory");
            fence_proxy_async();
            __syncwarp();
            if (lane == 0) tma_store_3d(&lin_maps.out[T.l], n0 + cc, T.l * T.l, node_q, stg);
          }
        }
      } else {
        // rows each store instruction of this lane covers (8 rows x 64 bytes): row pointers, once per tile
        float *rowptr[4];
  #pragma unroll
        for (int it = 0; it < 4; it++) {
          const int64_t gr = __shfl_sync(0xffffffffu, grow, it * 8 + (lane >> 2));
          rowptr[it] = gr >= 0 ? g.out + gr * g.N + n0 + (lane & 3) * 4 : nullptr;
        }
        for (int c0 = half * 32; c0 < ncols; c0 += 8 * EW) {
  #pragma unroll
          for (int h16 = 0; h16 < 32; h16 += 16) {
            const int cc = c0 + h16;
            if (cc >= ncols) break;  // warp-uniform
            uint32_t v[16];
            tmem_ld16_nowait(taddr + cc, v);             // all three product terms share these columns
            tmem_ld_wait();
            // lane = row: write the row's 16 values, then read back 8 rows x 64 bytes per instruction
            float *mine = ep_buf + lane * GT_EP_STRIDE;
  #pragma unroll
            for (int i = 0; i < 16; i += 4)
              *reinterpret_cast<float4 *>(mine + i) =
                  make_float4(__uint_as_float(v[i]) * g.scale, __uint_as_float(v[i + 1]) * g.scale,
                              __uint_as_float(v[i + 2]) * g.scale, __uint_as_float(v[i + 3]) * g.scale);
            __syncwarp();
            const bool col_ok = cc + (lane & 3) * 4 < ncols;
  #pragma unroll
            for (int it = 0; it < 4; it++) {
              const int rr = it * 8 + (lane >> 2);
              float4 o = *reinterpret_cast<const float4 *>(ep_buf + rr * GT_EP_STRIDE + (lane & 3) * 4);
              if (rowptr[it] != nullptr && col_ok) {
                *reinterpret_cast<float4 *>(rowptr[it] + cc) = o;
              }
            }
            __syncwarp();
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(acc_empty + 8 * acc);
      acc_phase[acc] ^= 1;
      acc ^= 1;
    }
    // the copy engine still reads this warp's staging buffer and writes its tile: wait before the CTA retires
    if (((MODE != GT_MODE_LINEAR && g.ep_tma) || (MODE == GT_MODE_LINEAR && g.lin_tma)) && lane == 0) tma_store_wait_all();
  }

  tc_fence_before();
  __syncthreads();
  if (warp == GT_PRODUCER_WARPS) tmem_dealloc(tmem_base, GT_TMEM_COLS);
}

// ---- a wait that runs out ---------------------------------------------------------------------------
// One warp waits, with the same bounded wait every role of the kernels above uses, on an mbarrier that nothing ever
// completes; when the wait gives up the kernel records `code` in *status and returns normally.  This is how the
// time-out path is exercised on a GPU without hanging or faulting it (tests, health checks).
__global__ void bounded_wait_probe_kernel(int32_t *status, int code, long long limit_cycles) {
  __shared__ __align__(8) uint64_t bar;
  const uint32_t b = smem_u32(&bar);
  if (threadIdx.x == 0) {
    mbar_init(b, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncwarp();
  uint32_t got = 1;
  if (threadIdx.x == 0) {
    got = mbar_try_wait(b, 0) ? 1u : 0u;
    const long long t0 = clock64();
    while (!got && clock64() - t0 < limit_cycles) got = mbar_try_wait(b, 0) ? 1u : 0u;
  }
  got = __shfl_sync(0xffffffffu, got, 0);
  if (!got && threadIdx.x == 0 && status) atomicCAS(status, 0, code);
}

// ---- weight packing ---------------------------------------------------------------------------------
// Bt [nmat, N, K] (K contiguous, i.e. the transpose of each B) -> per matrix, per N tile, per K block:
// hi image then lo image, each npad rows x 128 bytes in the swizzled layout, zero padded.
__global__ void pack_weights_kernel(const float *__restrict__ Bt, int nmat, int N, int K, int n_tiles, int k_blocks,
                                    int npad, float *__restrict__ packed) {
  const int64_t total = (int64_t)nmat * n_tiles * k_blocks * npad * 8;  // one thread per 16-byte chunk
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= total) return;
  const int c = (int)(i % 8);
  const int r = (int)((i / 8) % npad);
  const int kb = (int)((i / (8 * (int64_t)npad)) % k_blocks);
  const int nt = (int)((i / (8 * (int64_t)npad * k_blocks)) % n_tiles);
  const int m = (int)(i / (8 * (int64_t)npad * k_blocks * n_tiles));
  const int n = nt * 128 + r;
  float hi[4], lo[4];
#pragma unroll
  for (int u = 0; u < 4; u++) {
    const int k = kb * GT_KBLOCK + c * 4 + u;
    const float x = (n < N && r < 128 && k < K) ? Bt[((int64_t)m * N + n) * K + k] : 0.f;
    hi[u] = to_tf32(x);
    lo[u] = to_tf32(x - hi[u]);
  }
  const int64_t image = (int64_t)npad * 32;  // floats per image
  float *base = packed + (((int64_t)(m * n_tiles + nt) * k_blocks + kb) * 2) * image;
  const int off = sw128_offset(r, c) / 4;
  *reinterpret_cast<float4 *>(base + off) = make_float4(hi[0], hi[1], hi[2], hi[3]);
  *reinterpret_cast<float4 *>(base + image + off) = make_float4(lo[0], lo[1], lo[2], lo[3]);
}

struct PackGeom {
  int n_tiles, k_blocks, npad;
  int64_t floats_per_matrix;
};
static PackGeom pack_geom(int N, int K) {
  PackGeom p;
  p.n_tiles = (N + 127) / 128;
  p.k_blocks = (K + GT_KBLOCK - 1) / GT_KBLOCK;
  const int widest = N > 128 ? 128 : N;
  p.npad = (widest + 15) & ~15;
  p.floats_per_matrix = (int64_t)p.n_tiles * p.k_blocks * 2 * p.npad * 32;
  return p;
}

// cuTensorMapEncodeTiled through the runtime's driver entry point (no link-time dependency on libcuda)
typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                  const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static EncodeTiledFn encode_tiled_fn() {
  static EncodeTiledFn fn = nullptr;
  if (fn == nullptr) {
    void *p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  }
  return fn;
}

// Tensor map of a row-major float32 matrix [rows, K] for tile loads of 128 rows x 32 columns with the 128-byte
// swizzle (zeros outside the matrix): the layout of one K block of a tensor-core operand image.
int encode_rows_tensor_map(CUtensorMap *tmap, const float *A, int64_t rows, int K, const char *what) {
  memset(tmap, 0, sizeof(*tmap));
  EncodeTiledFn enc = encode_tiled_fn();
  if (enc == nullptr) return fail(CMACE_ERR_CUDA, "%s: cuTensorMapEncodeTiled is not available", what);
  const cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
  const cuuint64_t strides[1] = {(cuuint64_t)K * 4};
  const cuuint32_t box[2] = {GT_KBLOCK, GT_TILE_M};
  const cuuint32_t estr[2] = {1, 1};
  const CUresult r = enc(tmap, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<float *>(A), dims, strides, box, estr,
                         CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                         CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(CMACE_ERR_CUDA, "%s: cuTensorMapEncodeTiled failed (%d)", what, (int)r);
  return CMACE_OK;
}

// out [rows, N] as 32-row x 32-column boxes (128 bytes per row: one swizzle span) for the epilogue's tile stores
static int encode_out_tensor_map(CUtensorMap *tmap, float *out, int64_t rows, int N, const char *what) {
  memset(tmap, 0, sizeof(*tmap));
  EncodeTiledFn enc = encode_tiled_fn();
  if (enc == nullptr) return fail(CMACE_ERR_CUDA, "%s: cuTensorMapEncodeTiled is not available", what);
  const cuuint64_t dims[2] = {(cuuint64_t)N, (cuuint64_t)rows};
  const cuuint64_t strides[1] = {(cuuint64_t)N * 4};
  const cuuint32_t box[2] = {32, 32};
  const cuuint32_t estr[2] = {1, 1};
  const CUresult r = enc(tmap, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, out, dims, strides, box, estr,
                         CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_NONE,
                         CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(CMACE_ERR_CUDA, "%s: cuTensorMapEncodeTiled (out) failed (%d)", what, (int)r);
  return CMACE_OK;
}

// [nodes, 16, width] float32 as boxes of (box_cols columns, 2l+1 components starting at l^2, nq whole nodes)
static int encode_node_tensor_map(CUtensorMap *tmap, const float *base, int64_t nodes, int width, int l, int box_cols,
                                  CUtensorMapSwizzle swizzle, const char *what) {
  memset(tmap, 0, sizeof(*tmap));
  EncodeTiledFn enc = encode_tiled_fn();
  if (enc == nullptr) return fail(CMACE_ERR_CUDA, "%s: cuTensorMapEncodeTiled is not available", what);
  const cuuint64_t dims[3] = {(cuuint64_t)width, 16, (cuuint64_t)nodes};
  const cuuint64_t strides[2] = {(cuuint64_t)width * 4, (cuuint64_t)width * 64};
  const cuuint32_t box[3] = {(cuuint32_t)box_cols, (cuuint32_t)(2 * l + 1), (cuuint32_t)lin_nodes_per_quarter(l)};
  const cuuint32_t estr[3] = {1, 1, 1};
  const CUresult r = enc(tmap, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3, const_cast<float *>(base), dims, strides, box, estr,
                         CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                         CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(CMACE_ERR_CUDA, "%s: cuTensorMapEncodeTiled (rank 3) failed (%d)", what, (int)r);
  return CMACE_OK;
}

static int gemm_launch(GemmArgs &g, const char *what, cudaStream_t st) {
  static int num_sms = 0;
  if (num_sms == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&num_sms, cudaDevAttrMultiProcessorCount, dev);
    if (num_sms <= 0) num_sms = 148;
  }
  // PLAIN row map with few K blocks: every CTA keeps the B images of one column tile in shared memory and only
  // streams A, instead of fetching the same B block from L2 again for every 128-row tile
  const int b_all = g.k_blocks * 2 * g.npad * 128;
  g.b_resident = (g.mode == GT_MODE_PLAIN && b_all <= 64 * 1024 && num_sms >= g.n_tiles) ? b_all : 0;
  // residual image of A in tensor memory when at least four ring slots fit next to the two accumulators
  const int ts_slots = (GT_TMEM_COLS - 4 * g.npad) / 32;
  g.a_lo_tmem = ((g.mode == GT_MODE_PLAIN && ts_slots >= 4) || g.mode == GT_MODE_GRADR) ? 1 : 0;
  // PLAIN, full K blocks, wide output: one set of accumulator columns for the three terms leaves tensor memory for the
  // residual images where two sets would not
  const int oa_slots = (GT_TMEM_COLS - 2 * g.npad) / 32;
  const bool one_acc = g.mode == GT_MODE_PLAIN && !g.a_lo_tmem && g.K % GT_KBLOCK == 0 && g.N >= 32 && oa_slots >= 4;
  if (one_acc) g.a_lo_tmem = 1;
  // LINEAR: one set of accumulator columns for the three terms, so two accumulators take 2 npad columns
  const int lin_ts_slots = (GT_TMEM_COLS - 2 * g.npad) / 32;
  if (g.mode == GT_MODE_LINEAR) {
    if (lin_ts_slots < 2) return fail(CMACE_ERR_UNSUPPORTED, "%s: no room in tensor memory", what);
    g.a_lo_tmem = 1;
  }
  // rows by TMA when the nodes of every problem are consecutive in storage (no gather list)
  g.lin_tma = (g.mode == GT_MODE_LINEAR && g.a_lo_tmem && g.node_order == nullptr) ? 1 : 0;
  if (g.mode == GT_MODE_GRADR && ts_slots < 4) return fail(CMACE_ERR_UNSUPPORTED, "%s: no room in tensor memory", what);
  g.stage_bytes = (g.a_lo_tmem ? 1 : 2) * GT_A_SLAB + (g.b_resident ? 0 : 2 * g.npad * 128);
  // PLAIN: tile stores by TMA from a 4 KB staging buffer per epilogue warp (N >= 32: the box is 32 columns wide);
  // LINEAR: the transpose buffers of its epilogue
  g.ep_tma = (g.mode != GT_MODE_LINEAR && g.N >= 32) ? 1 : 0;
  const int ep_bytes = g.mode != GT_MODE_LINEAR ? (g.ep_tma ? GT_EP_TMA_BYTES : 0)
                       : g.lin_tma              ? GT_EPILOGUE_WARPS * 2048
                                                : GT_EP_BYTES;
  // the LINEAR variant holds its problem table in static shared memory
  const int budget = GT_SMEM_BUDGET - (g.mode == GT_MODE_LINEAR ? (int)sizeof(ProblemTable) + 1024 : 0);
  g.stages = (budget - ep_bytes - 1024 - g.b_resident) / g.stage_bytes;
  if (g.stages > GT_MAX_STAGES) g.stages = GT_MAX_STAGES;
  if (g.a_lo_tmem && g.mode != GT_MODE_LINEAR && g.stages > (one_acc ? oa_slots : ts_slots)) g.stages = one_acc ? oa_slots : ts_slots;
  g.g_stage_bytes = 0;
  if (g.mode == GT_MODE_LINEAR && g.a_lo_tmem) {
    // ring of A images (raw values only, 16 KB a slot), the epilogue's transpose buffers behind it, then a ring of B
    // blocks with the same slot count
    g.stage_bytes = GT_A_SLAB;
    g.stages = (budget - ep_bytes - 1024) / (GT_A_SLAB + 2 * g.npad * 128);
    if (g.stages > GT_MAX_STAGES) g.stages = GT_MAX_STAGES;
    if (g.stages > lin_ts_slots) g.stages = lin_ts_slots;
    g.b_slots = g.stages;
    g.g_stage_bytes = ep_bytes;   // the kernel finds the B ring behind stages * stage_bytes + g_stage_bytes
  }
  if (g.mode == GT_MODE_GRADR) {
    // Shared memory: a ring of B blocks and the G rows of a tile's receivers twice (the next tile's are copied while
    // this one is consumed).  No A images (they live in tensor memory) and no epilogue staging buffers (the narrow
    // output goes from tensor memory to global memory through registers).
    const int per_receiver = 16 * g.C * 4;
    g.ep_tma = 0;
    g.stage_bytes = 0;       // both images of A live in tensor memory: 64 columns a slot
    g.stages = ts_slots / 2 < 4 ? ts_slots / 2 : 4;
    g.b_slots = g.stages;    // the B blocks share slot index and barriers with the A images
    int left = budget - 1024 - g.stages * g.stage_bytes - g.b_slots * 2 * g.npad * 128;
    while (g.stages > 2 && left < 2 * 4 * per_receiver) {   // keep room for four receivers per buffer
      g.stages--;
      g.b_slots--;
      left += g.stage_bytes + 2 * g.npad * 128;
    }
    if (left < 0) return fail(CMACE_ERR_UNSUPPORTED, "%s: tile does not fit shared memory", what);
    g.g_stage_bytes = (left / (2 * per_receiver)) * 2 * per_receiver;
    if (g.g_stage_bytes < 0) g.g_stage_bytes = 0;
  }
  if (g.stages < 2) return fail(CMACE_ERR_UNSUPPORTED, "%s: tile does not fit shared memory", what);
  const size_t smem = (size_t)g.b_resident + (size_t)g.stages * g.stage_bytes +
                      ((g.mode == GT_MODE_GRADR || (g.mode == GT_MODE_LINEAR && g.a_lo_tmem)) ? 0 : ep_bytes) + 1024 +
                      (size_t)g.g_stage_bytes + (size_t)g.b_slots * 2 * g.npad * 128;
  LinMaps lin_maps;
  memset(&lin_maps, 0, sizeof(lin_maps));
  if (g.lin_tma) {
    for (int l = 0; l < 4; l++) {
      if (int rc = encode_node_tensor_map(&lin_maps.in[l], g.A, g.M, g.K, l, GT_KBLOCK, CU_TENSOR_MAP_SWIZZLE_128B, what)) return rc;
      if (int rc = encode_node_tensor_map(&lin_maps.out[l], g.out, g.M, g.N, l, 16, CU_TENSOR_MAP_SWIZZLE_64B, what)) return rc;
    }
    // tiles hold whole nodes: 128, 40, 24 and 16 of them for l = 0 .. 3
    g.total_tiles = 4 * (int64_t)g.nelements;
    for (int l = 0; l < 4; l++) g.total_tiles += g.M / (4 * lin_nodes_per_quarter(l)) + 1;
  }
  CUtensorMap tmap, tmap_out;
  memset(&tmap, 0, sizeof(tmap));
  memset(&tmap_out, 0, sizeof(tmap_out));
  if (g.mode == GT_MODE_PLAIN) {
    if (int rc = encode_rows_tensor_map(&tmap, g.A, g.M, g.K, what)) return rc;
  }
  if (g.ep_tma) {
    if (int rc = encode_out_tensor_map(&tmap_out, g.out, g.M, g.N, what)) return rc;
  }
  auto kern = g.mode == GT_MODE_LINEAR ? gemm3x_tf32_kernel<GT_MODE_LINEAR, true>
              : g.mode == GT_MODE_GRADR ? (g.C == 128 ? gemm3x_tf32_kernel<GT_MODE_GRADR, true, 128, 4>
                                                       : gemm3x_tf32_kernel<GT_MODE_GRADR, true, 0, 4>)
              : one_acc                ? gemm3x_tf32_kernel<GT_MODE_PLAIN, true, 0, GT_EPILOGUE_WARPS, true>
              : g.a_lo_tmem            ? gemm3x_tf32_kernel<GT_MODE_PLAIN, true>
                                       : gemm3x_tf32_kernel<GT_MODE_PLAIN>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return fail(CMACE_ERR_CUDA, "%s: %s", what, cudaGetErrorString(e));
  if (g.total_tiles > 0x7fffffffLL) return fail(CMACE_ERR_UNSUPPORTED, "%s: too many tiles", what);
  int64_t blocks = g.total_tiles < num_sms ? g.total_tiles : num_sms;
  if (g.b_resident) {
    // CTAs per column tile x column tiles; the tile index space becomes (iterations) x (grid)
    const int64_t row_tiles = g.total_tiles / g.n_tiles;
    int64_t per_col = num_sms / g.n_tiles;
    per_col = per_col < row_tiles ? per_col : row_tiles;
    blocks = per_col * g.n_tiles;
    g.total_tiles = ((row_tiles + per_col - 1) / per_col) * blocks;
  }
  if (blocks < 1) return CMACE_OK;
  const int nthreads = g.mode == GT_MODE_GRADR ? (GT_PRODUCER_WARPS + 1 + 4 + 1) * 32 : GT_THREADS;
  kern<<<(unsigned)blocks, nthreads, smem, st>>>(g, tmap, tmap_out, lin_maps);
  return check_launch(what);
}

}  // namespace cmace

using namespace cmace;

extern "C" {

int64_t cmace_gemm_packed_floats(int nmat, int N, int K) {
  if (nmat < 1 || N < 1 || K < 1) return 0;
  return (int64_t)nmat * pack_geom(N, K).floats_per_matrix;
}

int cmace_gemm_pack_weights_f32(const float *Bt, int nmat, int N, int K, float *packed, cmace_stream_t stream) {
  if (!Bt || !packed || nmat < 1 || N < 1 || K < 1) return fail(CMACE_ERR_ARG, "cmace_gemm_pack_weights: bad argument");
  if (!aligned16(packed)) return fail(CMACE_ERR_ARG, "cmace_gemm_pack_weights: packed must be 16-byte aligned");
  const PackGeom p = pack_geom(N, K);
  const int64_t total = (int64_t)nmat * p.n_tiles * p.k_blocks * p.npad * 8;
  pack_weights_kernel<<<(unsigned)((total + 255) / 256), 256, 0, (cudaStream_t)stream>>>(Bt, nmat, N, K, p.n_tiles,
                                                                                        p.k_blocks, p.npad, packed);
  return check_launch("cmace_gemm_pack_weights");
}

int cmace_gemm3x_f32(const float *A, const float *packed, int64_t M, int K, int N, double scale, float *out,
                     int32_t *status, cmace_stream_t stream) {
  if (M < 0 || K < 1 || N < 1) return fail(CMACE_ERR_ARG, "cmace_gemm3x: bad size");
  if (K % 8 != 0 || N % 4 != 0)
    return fail(CMACE_ERR_UNSUPPORTED, "cmace_gemm3x: K must be a multiple of 8 and N a multiple of 4");
  if (M == 0) return CMACE_OK;
  if (!A || !packed || !out) return fail(CMACE_ERR_ARG, "cmace_gemm3x: null pointer");
  if (!aligned16(A) || !aligned16(packed) || !aligned16(out))
    return fail(CMACE_ERR_ARG, "cmace_gemm3x: pointers must be 16-byte aligned");
  const PackGeom p = pack_geom(N, K);
  GemmArgs g{};
  g.A = A; g.packed = packed; g.out = out; g.status = status;
  g.M = M; g.K = K; g.N = N; g.nelements = 1; g.mode = GT_MODE_PLAIN; g.scale = (float)scale;
  g.n_tiles = p.n_tiles; g.k_blocks = p.k_blocks; g.npad = p.npad;
  g.total_tiles = ((M + GT_TILE_M - 1) / GT_TILE_M) * p.n_tiles;
  return gemm_launch(g, "cmace_gemm3x", (cudaStream_t)stream);
}

int cmace_bounded_wait_probe(int32_t *status, int code, double limit_seconds, cmace_stream_t stream) {
  if (!status || code == 0) return fail(CMACE_ERR_ARG, "cmace_bounded_wait_probe: status pointer and a non-zero code needed");
  if (!(limit_seconds > 0.0) || limit_seconds > 1.0)
    return fail(CMACE_ERR_ARG, "cmace_bounded_wait_probe: the limit must lie in (0, 1] seconds");
  int dev = 0, khz = 0;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&khz, cudaDevAttrClockRate, dev);
  if (khz <= 0) khz = 1965000;
  bounded_wait_probe_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(status, code, (long long)(limit_seconds * 1e3 * khz));
  return check_launch("cmace_bounded_wait_probe");
}

int cmace_gemm3x_gradr_f32(const float *X, const float *G, const float *Y, const int32_t *sender,
                           const int32_t *receiver, const float *packed, int64_t nedges, int channels, int N,
                           float *out, int32_t *status, cmace_stream_t stream) {
  if (nedges < 0 || N < 32 || N > 128 || N % 4 != 0)
    return fail(CMACE_ERR_UNSUPPORTED, "cmace_gemm3x_gradr: the hidden width must be a multiple of 4 in 32..128");
  if (channels < 32 || channels > 128 || channels % 32 != 0)
    return fail(CMACE_ERR_UNSUPPORTED, "cmace_gemm3x_gradr: channels must be 32, 64, 96 or 128");
  if (nedges == 0) return CMACE_OK;
  if (!X || !G || !Y || !sender || !receiver || !packed || !out)
    return fail(CMACE_ERR_ARG, "cmace_gemm3x_gradr: null pointer");
  if (!aligned16(X) || !aligned16(G) || !aligned16(packed) || !aligned16(out))
    return fail(CMACE_ERR_ARG, "cmace_gemm3x_gradr: pointers must be 16-byte aligned");
  const int K = 4 * channels;
  const PackGeom p = pack_geom(N, K);
  GemmArgs g{};
  g.packed = packed; g.out = out; g.status = status;
  g.gx = X; g.gg = G; g.gy = Y; g.sender = sender; g.receiver = receiver; g.C = channels;
  g.M = nedges; g.K = K; g.N = N; g.nelements = 1; g.mode = GT_MODE_GRADR; g.scale = 1.0f;
  g.n_tiles = p.n_tiles; g.k_blocks = p.k_blocks; g.npad = p.npad;
  g.total_tiles = (nedges + GT_TILE_M - 1) / GT_TILE_M;
  return gemm_launch(g, "cmace_gemm3x_gradr", (cudaStream_t)stream);
}

int cmace_linear_tc_f32(const float *X, const float *packed, const int32_t *node_order, const int32_t *elem_start,
                        int nelements, int64_t nnodes, int K, int Nout, double scale, float *out, int32_t *status,
                        cmace_stream_t stream) {
  if (nnodes < 0 || K < 1 || Nout < 1 || nelements < 1) return fail(CMACE_ERR_ARG, "cmace_linear_tc: bad size");
  if (nnodes > 0x7fffffffLL / 16) return fail(CMACE_ERR_UNSUPPORTED, "cmace_linear_tc: too many nodes");
  if (K % 8 != 0 || Nout % 4 != 0 || Nout > 128)
    return fail(CMACE_ERR_UNSUPPORTED, "cmace_linear_tc: K multiple of 8, Nout multiple of 4 and Nout <= 128");
  if (4 * nelements > GT_MAX_PROBLEMS)
    return fail(CMACE_ERR_UNSUPPORTED, "cmace_linear_tc: at most %d elements", GT_MAX_PROBLEMS / 4);
  if (nnodes == 0) return CMACE_OK;
  if (!X || !packed || !out) return fail(CMACE_ERR_ARG, "cmace_linear_tc: null pointer");
  if ((nelements > 1) != (elem_start != nullptr) || (node_order != nullptr && elem_start == nullptr))
    return fail(CMACE_ERR_ARG, "cmace_linear_tc: elem_start goes with nelements > 1, node_order only with elem_start");
  if (!aligned16(X) || !aligned16(packed) || !aligned16(out))
    return fail(CMACE_ERR_ARG, "cmace_linear_tc: pointers must be 16-byte aligned");
  const PackGeom p = pack_geom(Nout, K);
  GemmArgs g{};
  g.A = X; g.packed = packed; g.out = out; g.status = status;
  g.node_order = node_order; g.elem_start = elem_start;
  g.M = nnodes; g.K = K; g.N = Nout; g.nelements = nelements; g.mode = GT_MODE_LINEAR; g.scale = (float)scale;
  g.n_tiles = p.n_tiles; g.k_blocks = p.k_blocks; g.npad = p.npad;
  g.total_tiles = (nnodes * 16 + GT_TILE_M - 1) / GT_TILE_M + 4 * (int64_t)nelements;
  return gemm_launch(g, "cmace_linear_tc", (cudaStream_t)stream);
}
}
