// Segment layout (CSR by destination / CSC by source) of a COO edge list, plus the hub-row chunk
// lists the attention kernels use to split very long rows.  Built once per batch on the device.
//
// Contract (checked bit-for-bit by the tests against a stable CPU sort):
//   perm  = stable argsort of the grouping endpoint
//   other = other_endpoint[perm]
//   ptr   = exclusive prefix sum of bincount(grouping endpoint, n_rows)
#include <cub/device/device_radix_sort.cuh>
#include <cub/device/device_scan.cuh>

#include "tgt_common.cuh"

namespace tgt {
namespace {

constexpr int kThreads = 256;

inline int grid_for(int64_t n, int threads = kThreads) {
  int64_t b = (n + threads - 1) / threads;
  const int64_t cap = int64_t(kSmCount) * 32;
  if (b > cap) b = cap;
  if (b < 1) b = 1;
  return int(b);
}

// keys[i] = grouping endpoint of edge i as int32, iota[i] = i; any endpoint outside [0, n_rows)
// raises bit 0 of *flag (the offending edge is clamped so later kernels stay in bounds).
__global__ void extract_keys_kernel(const int64_t* __restrict__ key64,
                                    const int64_t* __restrict__ other64, int64_t n_edges,
                                    int64_t n_rows, int32_t* __restrict__ keys,
                                    int32_t* __restrict__ iota, int32_t* __restrict__ flag) {
  bool bad = false;
  for (int64_t i = blockIdx.x * int64_t(blockDim.x) + threadIdx.x; i < n_edges;
       i += int64_t(gridDim.x) * blockDim.x) {
    int64_t kk = key64[i];
    const int64_t oo = other64[i];
    if (kk < 0 || kk >= n_rows || oo < 0 || oo >= n_rows) {
      bad = true;
      kk = 0;
    }
    keys[i] = int32_t(kk);
    iota[i] = int32_t(i);
  }
  if (__syncthreads_or(bad) && threadIdx.x == 0) atomicOr(flag, 1);
}

// other[i] = other endpoint of the edge that landed at sorted position i; ptr[] from the run
// boundaries of the sorted keys.  Every ptr entry is written exactly once.
__global__ void finalize_kernel(const int32_t* __restrict__ sorted_keys,
                                const int32_t* __restrict__ perm,
                                const int64_t* __restrict__ other64, int64_t n_edges,
                                int64_t n_rows, int32_t* __restrict__ other,
                                int32_t* __restrict__ ptr) {
  for (int64_t i = blockIdx.x * int64_t(blockDim.x) + threadIdx.x; i <= n_edges;
       i += int64_t(gridDim.x) * blockDim.x) {
    if (i < n_edges) {
      int64_t oo = other64[perm[i]];
      if (oo < 0 || oo >= n_rows) oo = 0;  // already flagged by extract_keys_kernel
      other[i] = int32_t(oo);
    }
    // rows (prev, cur] start at sorted position i
    const int32_t prev = (i == 0) ? -1 : sorted_keys[i - 1];
    const int32_t cur = (i == n_edges) ? int32_t(n_rows) : sorted_keys[i];
    for (int32_t r = prev + 1; r <= cur; ++r) ptr[r] = int32_t(i);
  }
}

// Per row: number of chunks (0 unless the row is a hub) and hub indicator; entry n_rows is 0 so the
// exclusive scans below leave the totals there.
__global__ void count_hubs_kernel(const int32_t* __restrict__ ptr, int64_t n_rows,
                                  int32_t chunk_edges, int32_t* __restrict__ n_chunks,
                                  int32_t* __restrict__ is_hub) {
  for (int64_t r = blockIdx.x * int64_t(blockDim.x) + threadIdx.x; r <= n_rows;
       r += int64_t(gridDim.x) * blockDim.x) {
    int32_t c = 0;
    if (r < n_rows) {
      const int32_t deg = ptr[r + 1] - ptr[r];
      if (deg > chunk_edges) c = (deg + chunk_edges - 1) / chunk_edges;
    }
    n_chunks[r] = c;
    is_hub[r] = c > 0;
  }
}

__global__ void write_hubs_kernel(const int32_t* __restrict__ ptr, int64_t n_rows,
                                  int32_t chunk_edges, const int32_t* __restrict__ chunk_off,
                                  const int32_t* __restrict__ hub_off,
                                  int32_t* __restrict__ chunk_row, int32_t* __restrict__ chunk_begin,
                                  int32_t* __restrict__ hub_row, int32_t* __restrict__ hub_chunk_ptr) {
  for (int64_t r = blockIdx.x * int64_t(blockDim.x) + threadIdx.x; r <= n_rows;
       r += int64_t(gridDim.x) * blockDim.x) {
    if (r == n_rows) {
      hub_chunk_ptr[hub_off[r]] = chunk_off[r];  // terminator: hub_chunk_ptr[n_hubs] = n_chunks
      continue;
    }
    const int32_t c0 = chunk_off[r], c1 = chunk_off[r + 1];
    if (c1 == c0) continue;
    const int32_t h = hub_off[r];
    hub_row[h] = int32_t(r);
    hub_chunk_ptr[h] = c0;
    const int32_t begin = ptr[r];
    for (int32_t c = c0; c < c1; ++c) {
      chunk_row[c] = int32_t(r);
      chunk_begin[c] = begin + (c - c0) * chunk_edges;
    }
  }
}

int sort_bits(int64_t n_rows) {
  int bits = 1;
  while ((int64_t(1) << bits) < n_rows) ++bits;
  return bits;
}

struct Workspace {
  size_t keys, sorted, iota, n_chunks, is_hub, chunk_off, hub_off, flag, cub, total;
  size_t cub_bytes;
};

int plan_workspace(int64_t n_rows, int64_t n_edges, Workspace* w) {
  size_t sort_bytes = 0, scan_bytes = 0;
  if (n_edges > 0) {
    cudaError_t e = cub::DeviceRadixSort::SortPairs(
        nullptr, sort_bytes, static_cast<const int32_t*>(nullptr), static_cast<int32_t*>(nullptr),
        static_cast<const int32_t*>(nullptr), static_cast<int32_t*>(nullptr), int(n_edges), 0,
        sort_bits(n_rows));
    if (e != cudaSuccess)
      return set_error(TGT_ERR_CUDA, "cub radix sort size query failed: %s", cudaGetErrorString(e));
  }
  {
    cudaError_t e = cub::DeviceScan::ExclusiveSum(nullptr, scan_bytes,
                                                  static_cast<const int32_t*>(nullptr),
                                                  static_cast<int32_t*>(nullptr), int(n_rows + 1));
    if (e != cudaSuccess)
      return set_error(TGT_ERR_CUDA, "cub scan size query failed: %s", cudaGetErrorString(e));
  }
  const size_t e4 = round_up(size_t(n_edges) * 4, 256), r4 = round_up(size_t(n_rows + 1) * 4, 256);
  size_t off = 0;
  w->keys = off; off += e4;
  w->sorted = off; off += e4;
  w->iota = off; off += e4;
  w->n_chunks = off; off += r4;
  w->is_hub = off; off += r4;
  w->chunk_off = off; off += r4;
  w->hub_off = off; off += r4;
  w->flag = off; off += 256;
  w->cub = off;
  w->cub_bytes = round_up(sort_bytes > scan_bytes ? sort_bytes : scan_bytes, 256) + 256;
  off += w->cub_bytes;
  w->total = off;
  return TGT_OK;
}

}  // namespace
}  // namespace tgt

extern "C" int tgt_edge_layout_sizes(int64_t n_rows, int64_t n_edges, int32_t chunk_edges,
                                     int64_t* max_chunks, int64_t* max_hubs,
                                     size_t* workspace_bytes) {
  using namespace tgt;
  TGT_CHECK_ARG(n_rows >= 0 && n_edges >= 0, "n_rows and n_edges must be >= 0");
  TGT_CHECK_ARG(n_rows < (int64_t(1) << 31) - 1 && n_edges < (int64_t(1) << 31) - 1,
                "n_rows and n_edges must fit in int32");
  TGT_CHECK_ARG(chunk_edges >= 1, "chunk_edges must be >= 1");
  TGT_CHECK_ARG(max_chunks && max_hubs && workspace_bytes, "null output pointer");
  // a hub row of degree g > c has ceil(g/c) <= g/c + 1 < 2g/c chunks; hubs have degree > c
  *max_chunks = 2 * (n_edges / chunk_edges) + 1;
  *max_hubs = n_edges / (int64_t(chunk_edges) + 1) + 1;
  Workspace w;
  const int rc = plan_workspace(n_rows, n_edges, &w);
  if (rc != TGT_OK) return rc;
  *workspace_bytes = w.total;
  return TGT_OK;
}

extern "C" int tgt_edge_layout_build(const int64_t* edge_index, int64_t n_edges, int64_t n_rows,
                                     int group_by, int32_t chunk_edges, int32_t* ptr,
                                     int32_t* other, int32_t* perm, int32_t* chunk_row,
                                     int32_t* chunk_begin, int32_t* hub_row,
                                     int32_t* hub_chunk_ptr, int64_t* counts_host, void* workspace,
                                     size_t workspace_bytes, void* stream_) {
  using namespace tgt;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  TGT_CHECK_ARG(n_rows >= 0 && n_edges >= 0, "n_rows and n_edges must be >= 0");
  TGT_CHECK_ARG(n_rows < (int64_t(1) << 31) - 1 && n_edges < (int64_t(1) << 31) - 1,
                "n_rows and n_edges must fit in int32");
  TGT_CHECK_ARG(group_by == 0 || group_by == 1, "group_by must be 0 (source) or 1 (destination)");
  TGT_CHECK_ARG(chunk_edges >= 1, "chunk_edges must be >= 1");
  TGT_CHECK_ARG(n_edges == 0 || n_rows > 0, "edges given for a graph with no rows");
  TGT_CHECK_ARG(n_edges == 0 || edge_index, "edge_index is null");
  TGT_CHECK_ARG(ptr && counts_host, "ptr / counts_host is null");
  TGT_CHECK_ARG(n_edges == 0 || (other && perm), "other / perm is null");
  TGT_CHECK_ARG(chunk_row && chunk_begin && hub_row && hub_chunk_ptr, "hub arrays are null");
  TGT_CHECK_ARG(workspace, "workspace is null");
  TGT_CHECK_ARG(aligned16(edge_index) && aligned16(workspace), "pointers must be 16-byte aligned");

  Workspace w;
  int rc = plan_workspace(n_rows, n_edges, &w);
  if (rc != TGT_OK) return rc;
  if (workspace_bytes < w.total)
    return set_error(TGT_ERR_WORKSPACE, "workspace holds %zu bytes, %zu needed", workspace_bytes,
                     w.total);

  char* base = static_cast<char*>(workspace);
  int32_t* keys = reinterpret_cast<int32_t*>(base + w.keys);
  int32_t* sorted = reinterpret_cast<int32_t*>(base + w.sorted);
  int32_t* iota = reinterpret_cast<int32_t*>(base + w.iota);
  int32_t* n_chunks = reinterpret_cast<int32_t*>(base + w.n_chunks);
  int32_t* is_hub = reinterpret_cast<int32_t*>(base + w.is_hub);
  int32_t* chunk_off = reinterpret_cast<int32_t*>(base + w.chunk_off);
  int32_t* hub_off = reinterpret_cast<int32_t*>(base + w.hub_off);
  int32_t* flag = reinterpret_cast<int32_t*>(base + w.flag);
  void* cub_tmp = base + w.cub;

  const int64_t* key64 = edge_index + (group_by == 1 ? n_edges : 0);
  const int64_t* other64 = edge_index + (group_by == 1 ? 0 : n_edges);

  TGT_CHECK_CUDA(cudaMemsetAsync(flag, 0, 4, stream));
  if (n_edges > 0) {
    extract_keys_kernel<<<grid_for(n_edges), kThreads, 0, stream>>>(key64, other64, n_edges,
                                                                    n_rows, keys, iota, flag);
    size_t tmp = w.cub_bytes;
    TGT_CHECK_CUDA(cub::DeviceRadixSort::SortPairs(cub_tmp, tmp, keys, sorted, iota, perm,
                                                   int(n_edges), 0, sort_bits(n_rows), stream));
  }
  finalize_kernel<<<grid_for(n_edges + 1), kThreads, 0, stream>>>(sorted, perm, other64, n_edges,
                                                                  n_rows, other, ptr);
  count_hubs_kernel<<<grid_for(n_rows + 1), kThreads, 0, stream>>>(ptr, n_rows, chunk_edges,
                                                                   n_chunks, is_hub);
  {
    size_t tmp = w.cub_bytes;
    TGT_CHECK_CUDA(cub::DeviceScan::ExclusiveSum(cub_tmp, tmp, n_chunks, chunk_off,
                                                 int(n_rows + 1), stream));
    tmp = w.cub_bytes;
    TGT_CHECK_CUDA(
        cub::DeviceScan::ExclusiveSum(cub_tmp, tmp, is_hub, hub_off, int(n_rows + 1), stream));
  }
  write_hubs_kernel<<<grid_for(n_rows + 1), kThreads, 0, stream>>>(
      ptr, n_rows, chunk_edges, chunk_off, hub_off, chunk_row, chunk_begin, hub_row, hub_chunk_ptr);
  TGT_CHECK_CUDA(cudaGetLastError());

  int32_t h_counts[2] = {0, 0};
  int32_t h_flag = 0;
  TGT_CHECK_CUDA(cudaMemcpyAsync(&h_counts[0], chunk_off + n_rows, 4, cudaMemcpyDeviceToHost, stream));
  TGT_CHECK_CUDA(cudaMemcpyAsync(&h_counts[1], hub_off + n_rows, 4, cudaMemcpyDeviceToHost, stream));
  TGT_CHECK_CUDA(cudaMemcpyAsync(&h_flag, flag, 4, cudaMemcpyDeviceToHost, stream));
  TGT_CHECK_CUDA(cudaStreamSynchronize(stream));
  counts_host[0] = h_counts[0];
  counts_host[1] = h_counts[1];
  if (h_flag != 0)
    return set_error(TGT_ERR_INDEX_RANGE, "edge_index holds a node id outside [0, %lld)",
                     static_cast<long long>(n_rows));
  return TGT_OK;
}
