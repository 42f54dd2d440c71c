// Segment layout (CSR by destination / CSC by source) of a COO edge list, built once per batch on
// the device with a stable radix sort.
//
// Contract (checked bit-for-bit by the tests against a stable CPU sort):
//   perm  = stable argsort of the grouping endpoint
//   seg   = grouping endpoint[perm]          (the row of every sorted edge)
//   other = other endpoint[perm]
//   ptr   = exclusive prefix sum of bincount(grouping endpoint, n_rows)
#include <cub/device/device_radix_sort.cuh>

#include "tgt_common.cuh"

namespace tgt {
namespace {

constexpr int kThreads = 256;

inline int grid_for(int64_t n, int threads = kThreads) {
  int64_t b = (n + threads - 1) / threads;
  const int64_t cap = int64_t(sm_count()) * 32;
  if (b > cap) b = cap;
  if (b < 1) b = 1;
  return int(b);
}

// keys[i] = grouping endpoint of edge i as int32, iota[i] = i; any endpoint outside [0, n_rows)
// raises *flag (the offending id is replaced by 0 so the later kernels stay in bounds).
template <typename I>
__global__ void extract_keys_kernel(const I* __restrict__ key64,
                                    const I* __restrict__ other64, int64_t n_edges,
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
template <typename I>
__global__ void finalize_kernel(const int32_t* __restrict__ sorted_keys,
                                const int32_t* __restrict__ perm,
                                const I* __restrict__ other64, int64_t n_edges,
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

int sort_bits(int64_t n_rows) {
  int bits = 1;
  while ((int64_t(1) << bits) < n_rows) ++bits;
  return bits;
}

struct Workspace {
  size_t keys, iota, flag, cub, total, cub_bytes;
};

int plan_workspace(int64_t n_rows, int64_t n_edges, Workspace* w) {
  size_t sort_bytes = 0;
  if (n_edges > 0) {
    cudaError_t e = cub::DeviceRadixSort::SortPairs(
        nullptr, sort_bytes, static_cast<const int32_t*>(nullptr), static_cast<int32_t*>(nullptr),
        static_cast<const int32_t*>(nullptr), static_cast<int32_t*>(nullptr), int(n_edges), 0,
        sort_bits(n_rows));
    if (e != cudaSuccess)
      return set_error(TGT_ERR_CUDA, "cub radix sort size query failed: %s", cudaGetErrorString(e));
  }
  const size_t e4 = round_up(size_t(n_edges) * 4, 256);
  size_t off = 0;
  w->keys = off; off += e4;
  w->iota = off; off += e4;
  w->flag = off; off += 256;
  w->cub = off;
  w->cub_bytes = round_up(sort_bytes, 256) + 256;
  off += w->cub_bytes;
  w->total = off;
  return TGT_OK;
}

}  // namespace
}  // namespace tgt

extern "C" int tgt_edge_layout_sizes(int64_t n_rows, int64_t n_edges, size_t* workspace_bytes) {
  using namespace tgt;
  TGT_CHECK_ARG(n_rows >= 0 && n_edges >= 0, "n_rows and n_edges must be >= 0");
  TGT_CHECK_ARG(n_rows < (int64_t(1) << 31) - 1 && n_edges < (int64_t(1) << 31) - 1,
                "n_rows and n_edges must fit in int32");
  TGT_CHECK_ARG(workspace_bytes, "null output pointer");
  Workspace w;
  const int rc = plan_workspace(n_rows, n_edges, &w);
  if (rc != TGT_OK) return rc;
  *workspace_bytes = w.total;
  return TGT_OK;
}

namespace tgt {
namespace {

// The build for endpoint type I (int64: the reference's edge_index as is; int32: lists prepared on
// the device by tgt_edge_prepare, half the upload and half the reads).
template <typename I>
int build_layout(const I* edge_index, int64_t n_edges, int64_t n_rows, int group_by, int32_t* ptr,
                 int32_t* other, int32_t* perm, int32_t* seg, void* workspace,
                 size_t workspace_bytes, int32_t* deferred_status, cudaStream_t stream) {
  TGT_CHECK_ARG(n_rows >= 0 && n_edges >= 0, "n_rows and n_edges must be >= 0");
  TGT_CHECK_ARG(n_rows < (int64_t(1) << 31) - 1 && n_edges < (int64_t(1) << 31) - 1,
                "n_rows and n_edges must fit in int32");
  TGT_CHECK_ARG(group_by == 0 || group_by == 1, "group_by must be 0 (source) or 1 (destination)");
  TGT_CHECK_ARG(n_edges == 0 || n_rows > 0, "edges given for a graph with no rows");
  TGT_CHECK_ARG(n_edges == 0 || edge_index, "edge_index is null");
  TGT_CHECK_ARG(ptr, "ptr is null");
  TGT_CHECK_ARG(n_edges == 0 || (other && perm && seg), "other / perm / seg is null");
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
  int32_t* iota = reinterpret_cast<int32_t*>(base + w.iota);
  // the range-check result goes to the caller's word when the check is deferred
  int32_t* flag = deferred_status != nullptr ? deferred_status : reinterpret_cast<int32_t*>(base + w.flag);
  void* cub_tmp = base + w.cub;

  const I* key64 = edge_index + (group_by == 1 ? n_edges : 0);
  const I* other64 = edge_index + (group_by == 1 ? 0 : n_edges);

  TGT_CHECK_CUDA(cudaMemsetAsync(flag, 0, 4, stream));
  if (n_edges > 0) {
    extract_keys_kernel<I><<<grid_for(n_edges), kThreads, 0, stream>>>(key64, other64, n_edges,
                                                                       n_rows, keys, iota, flag);
    size_t tmp = w.cub_bytes;
    TGT_CHECK_CUDA(cub::DeviceRadixSort::SortPairs(cub_tmp, tmp, keys, seg, iota, perm,
                                                   int(n_edges), 0, sort_bits(n_rows), stream));
  }
  finalize_kernel<I><<<grid_for(n_edges + 1), kThreads, 0, stream>>>(seg, perm, other64, n_edges,
                                                                     n_rows, other, ptr);
  TGT_CHECK_CUDA(cudaGetLastError());
  if (deferred_status != nullptr) return TGT_OK;  // no synchronisation: the caller reads the word later

  int32_t h_flag = 0;
  TGT_CHECK_CUDA(cudaMemcpyAsync(&h_flag, flag, 4, cudaMemcpyDeviceToHost, stream));
  TGT_CHECK_CUDA(cudaStreamSynchronize(stream));
  if (h_flag != 0)
    return set_error(TGT_ERR_INDEX_RANGE, "edge_index holds a node id outside [0, %lld)",
                     static_cast<long long>(n_rows));
  return TGT_OK;
}

// Batch edge construction on the device (the reference does it on the host for every batch and
// uploads the int64 result): for raw edge e of graph g with endpoints (s, d) over that graph's own
// node ids 0..n-1,
//   fix     (fix_edge_index):            x -> x + 1, and per node i of the graph the two global-token
//                                        edges (i+1 -> 0) and (0 -> i+1) are appended after the raw edges;
//   adjust  (adjust_edge_index_nomerge): x > 0 -> x + (x - 1) / sub_seq_len;
//   flatten (flatten_edge_index_nopad):  x -> x + g * rows_per_graph.
// Output layout per graph: [raw edges | node -> token | token -> node], graphs concatenated, both
// endpoint rows int32 — the order the reference's helpers produce.
struct PrepareParams {
  const int64_t* raw;          // [2, raw_total]
  const int64_t* raw_ptr;      // [graphs + 1] raw edge range of every graph
  const int64_t* node_ptr;     // [graphs + 1] prefix sums of the graphs' node counts (fix only)
  int64_t raw_total, out_total;
  int graphs;
  int fix;                     // 1: add the global token
  int64_t sub_seq_len;         // 0: no adjust
  int64_t rows_per_graph;      // flatten offset per graph
  int32_t* out;                // [2, out_total]
};

__device__ __forceinline__ int graph_of(const int64_t* ptr, int graphs, int64_t i) {
  int lo = 0, hi = graphs;     // largest g with ptr[g] <= i
  while (hi - lo > 1) {
    const int mid = (lo + hi) >> 1;
    if (ptr[mid] <= i) lo = mid; else hi = mid;
  }
  return lo;
}

__global__ void edge_prepare_kernel(const PrepareParams p) {
  for (int64_t i = blockIdx.x * int64_t(blockDim.x) + threadIdx.x; i < p.out_total;
       i += int64_t(gridDim.x) * blockDim.x) {
    // output position i belongs to graph g: out_ptr[g] = raw_ptr[g] + 2 * node_ptr[g]
    int g;
    int64_t s, d;
    if (p.fix) {
      int lo = 0, hi = p.graphs;
      while (hi - lo > 1) {
        const int mid = (lo + hi) >> 1;
        if (p.raw_ptr[mid] + 2 * p.node_ptr[mid] <= i) lo = mid; else hi = mid;
      }
      g = lo;
      const int64_t local = i - (p.raw_ptr[g] + 2 * p.node_ptr[g]);
      const int64_t n_raw = p.raw_ptr[g + 1] - p.raw_ptr[g];
      const int64_t n_nodes = p.node_ptr[g + 1] - p.node_ptr[g];
      if (local < n_raw) {
        s = p.raw[p.raw_ptr[g] + local] + 1;
        d = p.raw[p.raw_total + p.raw_ptr[g] + local] + 1;
      } else if (local < n_raw + n_nodes) {
        s = local - n_raw + 1; d = 0;
      } else {
        s = 0; d = local - n_raw - n_nodes + 1;
      }
    } else {
      g = graph_of(p.raw_ptr, p.graphs, i);
      s = p.raw[i];
      d = p.raw[p.raw_total + i];
    }
    if (p.sub_seq_len > 0) {
      if (s > 0) s += (s - 1) / p.sub_seq_len;
      if (d > 0) d += (d - 1) / p.sub_seq_len;
    }
    const int64_t off = int64_t(g) * p.rows_per_graph;
    p.out[i] = int32_t(s + off);
    p.out[p.out_total + i] = int32_t(d + off);
  }
}

}  // namespace
}  // namespace tgt

extern "C" int tgt_edge_layout_build(const int64_t* edge_index, int64_t n_edges, int64_t n_rows,
                                     int group_by, int32_t* ptr, int32_t* other, int32_t* perm,
                                     int32_t* seg, void* workspace, size_t workspace_bytes,
                                     int32_t* deferred_status, void* stream) {
  return tgt::build_layout<int64_t>(edge_index, n_edges, n_rows, group_by, ptr, other, perm, seg,
                                    workspace, workspace_bytes, deferred_status,
                                    static_cast<cudaStream_t>(stream));
}

extern "C" int tgt_edge_layout_build_i32(const int32_t* edge_index, int64_t n_edges, int64_t n_rows,
                                         int group_by, int32_t* ptr, int32_t* other, int32_t* perm,
                                         int32_t* seg, void* workspace, size_t workspace_bytes,
                                         int32_t* deferred_status, void* stream) {
  return tgt::build_layout<int32_t>(edge_index, n_edges, n_rows, group_by, ptr, other, perm, seg,
                                    workspace, workspace_bytes, deferred_status,
                                    static_cast<cudaStream_t>(stream));
}

extern "C" int tgt_edge_prepare(const int64_t* raw_edges, int64_t raw_total, const int64_t* raw_ptr,
                                const int64_t* node_ptr, int graphs, int add_global_token,
                                int64_t sub_seq_len, int64_t rows_per_graph, int32_t* out,
                                int64_t out_total, void* stream_) {
  using namespace tgt;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  TGT_CHECK_ARG(graphs >= 1 && raw_total >= 0 && out_total >= 0, "graphs must be >= 1, sizes >= 0");
  TGT_CHECK_ARG(add_global_token == 0 || add_global_token == 1, "add_global_token must be 0 or 1");
  TGT_CHECK_ARG(raw_ptr != nullptr, "raw_ptr is null");
  TGT_CHECK_ARG(add_global_token == 0 || node_ptr != nullptr, "node_ptr is needed to add the global token");
  TGT_CHECK_ARG(sub_seq_len >= 0 && rows_per_graph >= 0, "sub_seq_len and rows_per_graph must be >= 0");
  TGT_CHECK_ARG(out_total < (int64_t(1) << 31) - 1 && int64_t(graphs) * rows_per_graph < (int64_t(1) << 31) - 1,
                "edge and row counts must fit in int32");
  if (out_total == 0) return TGT_OK;
  TGT_CHECK_ARG(out != nullptr && (raw_total == 0 || raw_edges != nullptr), "edge pointers are null");
  PrepareParams p;
  p.raw = raw_edges; p.raw_ptr = raw_ptr; p.node_ptr = node_ptr;
  p.raw_total = raw_total; p.out_total = out_total; p.graphs = graphs; p.fix = add_global_token;
  p.sub_seq_len = sub_seq_len; p.rows_per_graph = rows_per_graph; p.out = out;
  edge_prepare_kernel<<<grid_for(out_total), kThreads, 0, stream>>>(p);
  TGT_CHECK_CUDA(cudaGetLastError());
  return TGT_OK;
}
