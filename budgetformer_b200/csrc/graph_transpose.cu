// By-key view of the per-epoch attention graph and the balanced dK/dV work list, built on the device.
//
// The attention graph is a CSR over queries (rowptr, col = key per edge).  The dK/dV pass of the edge attention
// walks it by key, so every epoch needs
//   t_rowptr [n+1]   edges per key (prefix sums),
//   t_eid    [E]     edge positions grouped by key, query order kept inside a key (stable => reproducible sums),
//   t_row    [E]     the query of each of those edges,
//   tasks    [T, 4]  (key, first, end, partial slot) work items of at most `chunk` edges,
//   splits   [S, 3]  (key, first slot, number of slots) for keys cut into several items.
// Steps: row id per edge (one warp per query), LSD radix sort of (key, edge id) pairs over only the bits a node id
// needs (cub::DeviceRadixSort: 3 passes for 2.9 M nodes instead of 8 for 64-bit keys), key boundaries read off the
// sorted keys, and two compaction kernels driven by prefix sums.  The reference has no
// counterpart (its attention runs on COO with scatter reductions, e.g. models/gt_dist_node_level.py:224-262).
#include <cuda_runtime.h>
#include <stdint.h>

#include <cub/device/device_radix_sort.cuh>
#include <cub/device/device_scan.cuh>

#include "bf_kernels.h"

namespace {

// one warp per query row (a virtual-node row holds every node: its lanes stride over it)
__global__ void edge_rows_kernel(const int* __restrict__ rowptr, int n, int* __restrict__ erow) {
  const long long gt = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const int row = (int)(gt >> 5), lane = (int)(gt & 31);
  if (row >= n) return;
  const int beg = rowptr[row], end = rowptr[row + 1];
  for (int e = beg + lane; e < end; e += 32) erow[e] = row;
}

__global__ void iota_kernel(int* __restrict__ p, long long n) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) p[i] = (int)i;
}

// t_rowptr[k] = first position in the sorted key array whose key is >= k: position i is that boundary for every key
// in (keys[i-1], keys[i]] (several when keys without edges lie in between); i = n_edges closes the array.
__global__ void key_offsets_kernel(const int* __restrict__ keys_sorted, long long n_edges, int n, int* __restrict__ t_rowptr) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i > n_edges) return;
  const int prev = i == 0 ? -1 : keys_sorted[i - 1];
  const int cur = i == n_edges ? n : keys_sorted[i];
  for (int k = prev + 1; k <= cur; ++k) t_rowptr[k] = (int)i;
}

__global__ void gather_rows_kernel(const int* __restrict__ erow, const int* __restrict__ t_eid, long long n_edges,
                                   int* __restrict__ t_row) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n_edges) t_row[i] = erow[t_eid[i]];
}

// items per key (at least one, so that keys without edges still get their zero gradient written) and partial slots
__global__ void task_counts_kernel(const int* __restrict__ t_rowptr, int n, int chunk, int* __restrict__ n_items,
                                   int* __restrict__ n_slots, int* __restrict__ is_split) {
  const int k = blockIdx.x * blockDim.x + threadIdx.x;
  if (k >= n) return;
  const int deg = t_rowptr[k + 1] - t_rowptr[k];
  const int c = deg <= chunk ? 1 : (deg + chunk - 1) / chunk;
  n_items[k] = c;
  n_slots[k] = c > 1 ? c : 0;
  is_split[k] = c > 1 ? 1 : 0;
}

// One warp per key: lane l writes items l, l+32, ... (hub keys own thousands of items).  The list starts with the
// items of all split keys (full-length items: the long work is scheduled first and runs side by side in a warp),
// followed by the single item of every other key in key order; an item of a split key sits at its partial-slot index.
__global__ void task_fill_kernel(const int* __restrict__ t_rowptr, const int* __restrict__ item_first,
                                 const int* __restrict__ slot_first, const int* __restrict__ split_first, int n,
                                 int chunk, int4* __restrict__ tasks, int* __restrict__ splits) {
  const long long gt = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const int k = (int)(gt >> 5), lane = (int)(gt & 31);
  if (k >= n) return;
  const int beg = t_rowptr[k], end = t_rowptr[k + 1];
  const int cnt = item_first[k + 1] - item_first[k];
  const int s0 = slot_first[k];
  const int total_slots = slot_first[n];
  if (cnt == 1) {
    if (lane == 0) tasks[total_slots + (k - split_first[k])] = make_int4(k, beg, end, -1);
    return;
  }
  for (int c = lane; c < cnt; c += 32) {
    const int b = beg + c * chunk;
    int e = b + chunk;
    if (e > end) e = end;
    tasks[s0 + c] = make_int4(k, b, e, s0 + c);
  }
  if (lane == 0 && cnt > 1) {
    const int s = split_first[k];
    splits[3 * s] = k; splits[3 * s + 1] = s0; splits[3 * s + 2] = cnt;
  }
}

int bits_for(int n) {
  int b = 1;
  while (b < 31 && (1ll << b) < (long long)n) ++b;
  return b;
}

}  // namespace

// Bytes of scratch `bf_graph_transpose` needs for (n, n_edges); the caller allocates it.
extern "C" size_t bf_graph_transpose_scratch(int n, long long n_edges) {
  size_t sort_bytes = 0;
  cub::DeviceRadixSort::SortPairs(nullptr, sort_bytes, (const int*)nullptr, (int*)nullptr, (const int*)nullptr,
                                  (int*)nullptr, n_edges, 0, bits_for(n));
  // keys_out + iota + erow (rounded up to 256 bytes), then the sort's own temporary storage
  return ((3 * (size_t)n_edges * sizeof(int) + 255) & ~(size_t)255) + ((sort_bytes + 255) & ~(size_t)255) + 256;
}

extern "C" int bf_graph_transpose(const int* rowptr, const int* col, int n, long long n_edges, int* t_rowptr, int* t_row,
                                  int* t_eid, void* scratch, size_t scratch_bytes, cudaStream_t st) {
  if (n_edges == 0) return (int)cudaMemsetAsync(t_rowptr, 0, sizeof(int) * ((size_t)n + 1), st);
  int* keys_out = static_cast<int*>(scratch);
  int* iota = keys_out + n_edges;
  int* erow = iota + n_edges;
  const size_t head = (3 * (size_t)n_edges * sizeof(int) + 255) & ~(size_t)255;
  void* sort_tmp = static_cast<uint8_t*>(scratch) + head;
  size_t sort_bytes = scratch_bytes - head;
  const unsigned eb = (unsigned)((n_edges + 255) / 256);
  iota_kernel<<<eb, 256, 0, st>>>(iota, n_edges);
  edge_rows_kernel<<<(unsigned)(((long long)n * 32 + 255) / 256), 256, 0, st>>>(rowptr, n, erow);
  cudaError_t e = cub::DeviceRadixSort::SortPairs(sort_tmp, sort_bytes, col, keys_out, iota, t_eid, n_edges, 0,
                                                  bits_for(n), st);
  if (e != cudaSuccess) return (int)e;
  key_offsets_kernel<<<(unsigned)((n_edges + 1 + 255) / 256), 256, 0, st>>>(keys_out, n_edges, n, t_rowptr);
  gather_rows_kernel<<<eb, 256, 0, st>>>(erow, t_eid, n_edges, t_row);
  return (int)cudaGetLastError();
}

// Phase 1 of the work list: per-key counts and their exclusive prefix sums ([n+1] each, last element = total).
extern "C" int bf_kv_task_counts(const int* t_rowptr, int n, int chunk, int* item_first, int* slot_first,
                                 int* split_first, void* scratch, size_t scratch_bytes, cudaStream_t st) {
  // scratch: three int[n] count arrays followed by the scan's temporary storage
  int* n_items = static_cast<int*>(scratch);
  int* n_slots = n_items + n;
  int* is_split = n_slots + n;
  const size_t head = (3 * (size_t)n * sizeof(int) + 255) & ~(size_t)255;
  void* scan_tmp = static_cast<uint8_t*>(scratch) + head;
  size_t scan_bytes = scratch_bytes - head;
  task_counts_kernel<<<(n + 255) / 256, 256, 0, st>>>(t_rowptr, n, chunk, n_items, n_slots, is_split);
  cudaError_t e;
  // exclusive prefix sums with the total appended: out[0] = 0, out[1..n] = inclusive sums
  for (int which = 0; which < 3; ++which) {
    const int* in = which == 0 ? n_items : which == 1 ? n_slots : is_split;
    int* out = which == 0 ? item_first : which == 1 ? slot_first : split_first;
    e = cudaMemsetAsync(out, 0, sizeof(int), st);
    if (e != cudaSuccess) return (int)e;
    e = cub::DeviceScan::InclusiveSum(scan_tmp, scan_bytes, in, out + 1, n, st);
    if (e != cudaSuccess) return (int)e;
  }
  return (int)cudaGetLastError();
}

extern "C" size_t bf_kv_task_scratch(int n) {
  size_t scan_bytes = 0;
  cub::DeviceScan::InclusiveSum(nullptr, scan_bytes, (const int*)nullptr, (int*)nullptr, n);
  return ((3 * (size_t)n * sizeof(int) + 255) & ~(size_t)255) + ((scan_bytes + 255) & ~(size_t)255) + 256;
}

// Phase 2: write the items and the split list (sizes read back by the caller from the prefix sums).
extern "C" int bf_kv_task_fill(const int* t_rowptr, const int* item_first, const int* slot_first, const int* split_first,
                               int n, int chunk, int* tasks, int* splits, cudaStream_t st) {
  const long long threads = (long long)n * 32;
  const unsigned blocks = (unsigned)((threads + 255) / 256);
  if (blocks > 0)
    task_fill_kernel<<<blocks, 256, 0, st>>>(t_rowptr, item_first, slot_first, split_first, n, chunk,
                                             reinterpret_cast<int4*>(tasks), splits);
  return (int)cudaGetLastError();
}
