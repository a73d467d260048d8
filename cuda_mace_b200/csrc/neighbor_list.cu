// Neighbour list on the device for an orthorhombic cell (the step before the hot path: upstream builds it on the
// host with matscipy / ASE, tests/test_utils.py:97-105 of the reference).  Full list (both directions), receivers =
// the first nrecv atoms, sorted by receiver, i.e. directly the layout InvariantMessagePassing wants:
//
//   edge e:  vector = pos[sender[e]] - pos[receiver[e]] + shift[e],  |vector| < r_cut
//
// Cell list: atoms are binned into cells of at least r_cut per side (cmace_nl_cell_ids_f64), grouped by cell with
// the same radix-sort routine that groups edges by sender (cmace_sender_order with keys = cell ids), then one
// warp per receiver walks the 27 surrounding cells, 32 candidates at a time, once to count and once to fill
// (ballot + prefix inside the warp, so the edges of a receiver come out in a fixed order and nothing is atomic).
// Periodic axes wrap with a lattice shift; a box of one or two cells per periodic axis still works because each of
// the 27 (cell, shift) pairs is distinct as long as the box is at least r_cut long.  Distances are formed with
// the same operations and in the same order as the host list (no fused multiply-add), so both make the same
// decision for every pair.
#include <cub/device/device_scan.cuh>

#include "common.cuh"

namespace cmace {

struct NlGeom {
  double lo[3], len[3], cell[3], rc2;
  int ncell[3], pbc[3];
};

static int make_geom(NlGeom &g, double lox, double loy, double loz, double lx, double ly, double lz, int pbc_mask,
                     double r_cut, const char *what) {
  const double lo[3] = {lox, loy, loz}, len[3] = {lx, ly, lz};
  if (!(r_cut > 0.0)) return fail(CMACE_ERR_ARG, "%s: r_cut must be positive", what);
  for (int d = 0; d < 3; d++) {
    if (!(len[d] > 0.0)) return fail(CMACE_ERR_ARG, "%s: box lengths must be positive", what);
    g.lo[d] = lo[d];
    g.len[d] = len[d];
    g.pbc[d] = (pbc_mask >> d) & 1;
    int64_t n = (int64_t)(len[d] / r_cut);
    if (n < 1) {
      if (g.pbc[d])
        return fail(CMACE_ERR_UNSUPPORTED, "%s: a periodic axis shorter than r_cut needs more than one image", what);
      n = 1;
    }
    if (n > 1024) n = 1024;
    g.ncell[d] = (int)n;
    g.cell[d] = len[d] / (double)n;
  }
  g.rc2 = r_cut * r_cut;
  return CMACE_OK;
}

// wrapped coordinate, cell index and number of lattice translations removed, along axis d
__device__ __forceinline__ void locate(const NlGeom &g, int d, double x, double &xw, int &c, int &w) {
  w = 0;
  xw = x;
  if (g.pbc[d]) {
    w = (int)floor((x - g.lo[d]) / g.len[d]);
    if (w != 0) xw = x - (double)w * g.len[d];
  }
  int ci = (int)floor((xw - g.lo[d]) / g.cell[d]);
  c = ci < 0 ? 0 : (ci >= g.ncell[d] ? g.ncell[d] - 1 : ci);
}

__global__ void nl_cell_ids_kernel(const double *__restrict__ pos, int64_t natoms, const NlGeom g,
                                   int32_t *__restrict__ cell_id) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= natoms) return;
  int c[3], w;
  double xw;
  for (int d = 0; d < 3; d++) locate(g, d, pos[3 * i + d], xw, c[d], w);
  cell_id[i] = (c[0] * g.ncell[1] + c[1]) * g.ncell[2] + c[2];
}

// One warp per receiver.  FILL = false: count[i] = number of neighbours; FILL = true: writes them at row_ptr[i].
template <bool FILL>
__global__ void __launch_bounds__(128)
    nl_walk_kernel(const double *__restrict__ pos, int64_t nrecv, const NlGeom g, const int32_t *__restrict__ perm,
                   const int32_t *__restrict__ cell_ptr, int32_t *__restrict__ count,
                   const int32_t *__restrict__ row_ptr, int32_t *__restrict__ sender, int32_t *__restrict__ receiver,
                   int8_t *__restrict__ shift_idx, double *__restrict__ shifts) {
  const int lane = threadIdx.x & 31;
  const int64_t i = (int64_t)blockIdx.x * 4 + (threadIdx.x >> 5);
  if (i >= nrecv) return;
  double xi[3];
  int ci[3], wi[3];
  for (int d = 0; d < 3; d++) locate(g, d, pos[3 * i + d], xi[d], ci[d], wi[d]);
  int64_t out = FILL ? (int64_t)row_ptr[i] : 0;
  int total = 0;
  for (int dx = -1; dx <= 1; dx++)
    for (int dy = -1; dy <= 1; dy++)
      for (int dz = -1; dz <= 1; dz++) {
        const int dd[3] = {dx, dy, dz};
        int c[3], S[3];
        bool skip = false;
        for (int d = 0; d < 3; d++) {
          int cc = ci[d] + dd[d];
          S[d] = 0;
          if (cc < 0 || cc >= g.ncell[d]) {
            if (!g.pbc[d]) {
              skip = true;
            } else {
              S[d] = cc < 0 ? -1 : 1;
              cc -= S[d] * g.ncell[d];
            }
          }
          c[d] = cc;
        }
        if (skip) continue;
        const int cf = (c[0] * g.ncell[1] + c[1]) * g.ncell[2] + c[2];
        const double sx = (double)S[0] * g.len[0], sy = (double)S[1] * g.len[1], sz = (double)S[2] * g.len[2];
        const bool same_image = S[0] == 0 && S[1] == 0 && S[2] == 0;
        const int k0 = cell_ptr[cf], k1 = cell_ptr[cf + 1];
        for (int kb = k0; kb < k1; kb += 32) {
          const int k = kb + lane;
          bool hit = false;
          int j = 0, wj[3] = {0, 0, 0};
          if (k < k1) {
            j = perm[k];
            double xj[3];
            int cj;
            for (int d = 0; d < 3; d++) locate(g, d, pos[3 * (int64_t)j + d], xj[d], cj, wj[d]);
            // (x_j + shift) - x_i, squared and summed in the order of the host list, without contraction
            const double ddx = __dsub_rn(__dadd_rn(xj[0], sx), xi[0]);
            const double ddy = __dsub_rn(__dadd_rn(xj[1], sy), xi[1]);
            const double ddz = __dsub_rn(__dadd_rn(xj[2], sz), xi[2]);
            const double d2 = __dadd_rn(__dadd_rn(__dmul_rn(ddx, ddx), __dmul_rn(ddy, ddy)), __dmul_rn(ddz, ddz));
            hit = d2 < g.rc2 && !(same_image && (int64_t)j == i);
          }
          const unsigned m = __ballot_sync(0xffffffffu, hit);
          if (FILL && hit) {
            const int64_t e = out + __popc(m & ((1u << lane) - 1u));
            sender[e] = j;
            receiver[e] = (int32_t)i;
            for (int d = 0; d < 3; d++) {
              const int s = S[d] - wj[d] + wi[d];
              if (shift_idx) shift_idx[3 * e + d] = (int8_t)s;
              if (shifts) shifts[3 * e + d] = (double)s * g.len[d];
            }
          }
          out += __popc(m);
          total += __popc(m);
        }
      }
  if (!FILL && lane == 0) count[i] = total;
}

}  // namespace cmace

using namespace cmace;

extern "C" {

int64_t cmace_nl_num_cells(double lx, double ly, double lz, double r_cut) {
  NlGeom g;
  if (make_geom(g, 0, 0, 0, lx, ly, lz, 0, r_cut, "cmace_nl_num_cells")) return 0;
  return (int64_t)g.ncell[0] * g.ncell[1] * g.ncell[2];
}

int cmace_nl_cell_ids_f64(const double *pos, int64_t natoms, double lox, double loy, double loz, double lx, double ly,
                          double lz, int pbc_mask, double r_cut, int32_t *cell_id, cmace_stream_t stream) {
  NlGeom g;
  if (int rc = make_geom(g, lox, loy, loz, lx, ly, lz, pbc_mask, r_cut, "cmace_nl_cell_ids")) return rc;
  if (natoms < 0) return fail(CMACE_ERR_ARG, "cmace_nl_cell_ids: negative size");
  if (natoms == 0) return CMACE_OK;
  if (!pos || !cell_id) return fail(CMACE_ERR_ARG, "cmace_nl_cell_ids: null pointer");
  nl_cell_ids_kernel<<<(unsigned)((natoms + 255) / 256), 256, 0, (cudaStream_t)stream>>>(pos, natoms, g, cell_id);
  return check_launch("cmace_nl_cell_ids");
}

int cmace_nl_count_f64(const double *pos, int64_t natoms, int64_t nrecv, double lox, double loy, double loz, double lx,
                       double ly, double lz, int pbc_mask, double r_cut, const int32_t *perm, const int32_t *cell_ptr,
                       int32_t *count, cmace_stream_t stream) {
  NlGeom g;
  if (int rc = make_geom(g, lox, loy, loz, lx, ly, lz, pbc_mask, r_cut, "cmace_nl_count")) return rc;
  if (natoms < 0 || nrecv < 0 || nrecv > natoms) return fail(CMACE_ERR_ARG, "cmace_nl_count: bad size");
  if (nrecv == 0) return CMACE_OK;
  if (!pos || !perm || !cell_ptr || !count) return fail(CMACE_ERR_ARG, "cmace_nl_count: null pointer");
  nl_walk_kernel<false><<<(unsigned)((nrecv + 3) / 4), 128, 0, (cudaStream_t)stream>>>(
      pos, nrecv, g, perm, cell_ptr, count, nullptr, nullptr, nullptr, nullptr, nullptr);
  return check_launch("cmace_nl_count");
}

int64_t cmace_scan_workspace_bytes(int64_t n) {
  size_t bytes = 0;
  cub::DeviceScan::ExclusiveSum(nullptr, bytes, (const int32_t *)nullptr, (int32_t *)nullptr, (int)(n < 1 ? 1 : n));
  return (int64_t)bytes + 256;
}

int cmace_exclusive_scan_i32(const int32_t *in, int64_t n, int32_t *out, void *workspace, int64_t workspace_bytes,
                             cmace_stream_t stream) {
  if (n < 0 || n > 0x7ffffffeLL) return fail(CMACE_ERR_ARG, "cmace_exclusive_scan: bad size");
  if (n == 0) return CMACE_OK;
  if (!in || !out || !workspace) return fail(CMACE_ERR_ARG, "cmace_exclusive_scan: null pointer");
  size_t bytes = (size_t)workspace_bytes;
  cudaError_t e = cub::DeviceScan::ExclusiveSum(workspace, bytes, in, out, (int)n, (cudaStream_t)stream);
  if (e != cudaSuccess) return fail(CMACE_ERR_CUDA, "cmace_exclusive_scan: %s", cudaGetErrorString(e));
  return check_launch("cmace_exclusive_scan");
}

int cmace_nl_fill_f64(const double *pos, int64_t natoms, int64_t nrecv, double lox, double loy, double loz, double lx,
                      double ly, double lz, int pbc_mask, double r_cut, const int32_t *perm, const int32_t *cell_ptr,
                      const int32_t *row_ptr, int32_t *sender, int32_t *receiver, int8_t *shift_idx, double *shifts,
                      cmace_stream_t stream) {
  NlGeom g;
  if (int rc = make_geom(g, lox, loy, loz, lx, ly, lz, pbc_mask, r_cut, "cmace_nl_fill")) return rc;
  if (natoms < 0 || nrecv < 0 || nrecv > natoms) return fail(CMACE_ERR_ARG, "cmace_nl_fill: bad size");
  if (nrecv == 0) return CMACE_OK;
  if (!pos || !perm || !cell_ptr || !row_ptr || !sender || !receiver)
    return fail(CMACE_ERR_ARG, "cmace_nl_fill: null pointer");
  nl_walk_kernel<true><<<(unsigned)((nrecv + 3) / 4), 128, 0, (cudaStream_t)stream>>>(
      pos, nrecv, g, perm, cell_ptr, nullptr, row_ptr, sender, receiver, shift_idx, shifts);
  return check_launch("cmace_nl_fill");
}
}
