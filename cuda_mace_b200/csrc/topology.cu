// Topology preprocessing, run once per neighbour list (not per layer or per step):
//  * receiver CSR from the receiver-sorted edge list (empty rows allowed),
//  * sender-grouped edge permutation (stable radix sort of edge ids by sender) + its CSR,
//  * nodes grouped by chemical element (same routine, keys = element index).
#include <cub/device/device_radix_sort.cuh>

#include "common.cuh"

namespace cmace {

char *error_buffer() {
  static thread_local char buf[512] = {0};
  return buf;
}

// keys sorted ascending -> ptr[k] = first position whose key is >= k, for k = 0..nkeys.
// Thread i looks at the boundary between positions i-1 and i and fills every ptr entry whose
// first position is i, so keys that never occur get an empty range.
__global__ void csr_from_sorted_kernel(const int32_t *__restrict__ keys, int64_t n, int64_t nkeys,
                                       int32_t *__restrict__ ptr) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i > n) return;
  int64_t prev = (i == 0) ? -1 : (int64_t)keys[i - 1];
  int64_t cur = (i == n) ? nkeys : (int64_t)keys[i];
  if (cur > nkeys) cur = nkeys;
  if (prev < -1) prev = -1;
  for (int64_t k = prev + 1; k <= cur; k++) ptr[k] = (int32_t)i;
}

__global__ void iota_kernel(int32_t *p, int64_t n) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) p[i] = (int32_t)i;
}

static int64_t align256(int64_t x) { return (x + 255) / 256 * 256; }

static int64_t cub_temp_bytes(int64_t n) {
  size_t bytes = 0;
  cub::DeviceRadixSort::SortPairs(nullptr, bytes, (const int32_t *)nullptr, (int32_t *)nullptr,
                                  (const int32_t *)nullptr, (int32_t *)nullptr, (int)n);
  return (int64_t)bytes;
}

static int group_by_key(const int32_t *keys, int64_t n, int64_t nkeys, int32_t *order, int32_t *ptr,
                        void *workspace, int64_t workspace_bytes, cudaStream_t st, const char *what) {
  if (n < 0 || nkeys < 0 || n > 0x7fffffffLL) return fail(CMACE_ERR_ARG, "%s: bad size", what);
  if (!ptr) return fail(CMACE_ERR_ARG, "%s: null pointer", what);
  if (n > 0) {
    if (!keys || !order || !workspace) return fail(CMACE_ERR_ARG, "%s: null pointer", what);
    const int64_t need = cmace_sender_order_workspace_bytes(n);
    if (workspace_bytes < need)
      return fail(CMACE_ERR_ARG, "%s: workspace of %lld bytes, %lld needed", what,
                  (long long)workspace_bytes, (long long)need);
    char *w = static_cast<char *>(workspace);
    int32_t *keys_sorted = reinterpret_cast<int32_t *>(w);
    int32_t *ids = reinterpret_cast<int32_t *>(w + align256(n * 4));
    void *temp = w + 2 * align256(n * 4);
    size_t temp_bytes = (size_t)(workspace_bytes - 2 * align256(n * 4));
    iota_kernel<<<(unsigned)((n + 255) / 256), 256, 0, st>>>(ids, n);
    int end_bit = 1;
    while (end_bit < 31 && (1LL << end_bit) < nkeys) end_bit++;
    cudaError_t e = cub::DeviceRadixSort::SortPairs(temp, temp_bytes, keys, keys_sorted, ids, order,
                                                    (int)n, 0, end_bit, st);
    if (e != cudaSuccess) return fail(CMACE_ERR_CUDA, "%s: radix sort: %s", what, cudaGetErrorString(e));
    csr_from_sorted_kernel<<<(unsigned)((n + 1 + 255) / 256), 256, 0, st>>>(keys_sorted, n, nkeys, ptr);
  } else {
    csr_from_sorted_kernel<<<1, 256, 0, st>>>(nullptr, 0, nkeys, ptr);
  }
  return check_launch(what);
}

}  // namespace cmace

using namespace cmace;

extern "C" {

const char *cmace_last_error(void) { return error_buffer(); }
int cmace_abi_version(void) { return 1; }

int cmace_receiver_csr(const int32_t *receiver, int64_t nedges, int64_t nnodes, int32_t *row_ptr,
                       cmace_stream_t stream) {
  if (nedges < 0 || nnodes < 0 || nedges > 0x7fffffffLL)
    return fail(CMACE_ERR_ARG, "cmace_receiver_csr: bad size");
  if (!row_ptr || (nedges > 0 && !receiver)) return fail(CMACE_ERR_ARG, "cmace_receiver_csr: null pointer");
  csr_from_sorted_kernel<<<(unsigned)((nedges + 1 + 255) / 256), 256, 0, (cudaStream_t)stream>>>(
      receiver, nedges, nnodes, row_ptr);
  return check_launch("cmace_receiver_csr");
}

int64_t cmace_sender_order_workspace_bytes(int64_t n) {
  if (n <= 0) return 0;
  return 2 * align256(n * 4) + align256(cub_temp_bytes(n));
}

int cmace_sender_order(const int32_t *sender, int64_t nedges, int64_t nnodes, int32_t *perm,
                       int32_t *send_ptr, void *workspace, int64_t workspace_bytes, cmace_stream_t stream) {
  return group_by_key(sender, nedges, nnodes, perm, send_ptr, workspace, workspace_bytes,
                      (cudaStream_t)stream, "cmace_sender_order");
}

int cmace_group_by_element(const int32_t *elem, int64_t nnodes, int nelements, int32_t *node_order,
                           int32_t *elem_start, void *workspace, int64_t workspace_bytes,
                           cmace_stream_t stream) {
  return group_by_key(elem, nnodes, nelements, node_order, elem_start, workspace, workspace_bytes,
                      (cudaStream_t)stream, "cmace_group_by_element");
}
}
