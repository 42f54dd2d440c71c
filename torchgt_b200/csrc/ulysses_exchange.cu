// Local re-layout kernels around the Ulysses head<->sequence all-to-all, and the global-token
// row fix-ups of the node-level Graphormer layer.  Pure HBM-bound permuted copies: one thread
// moves one 16/8/4/2-byte unit, grid-stride, reads and writes coalesced along the row width.
//
// Staging buffer: stage[world][n_tensors][batch][seq_local][width_local]   ("peer-major")
//   heads-split side: x_t[batch][seq_local][world][width_local]
//   seq-split side:   x_t[batch][world][seq_local][width_local]
#include "tgt_common.cuh"

namespace tgt {
namespace {

constexpr int kThreads = 256;

struct Ptrs3 {
  void* p[3];
};

// One kernel for the four directions: `heads_split` picks the tensor-side layout, `to_stage` the
// copy direction.  All extents are in copy units of type U.
template <typename U>
__global__ void relayout_kernel(Ptrs3 tensors, U* __restrict__ stage, int n_tensors, int64_t batch,
                                int64_t seq_local, int64_t wv, int world, bool heads_split,
                                bool to_stage) {
  const int64_t per_tensor = batch * seq_local * wv;          // units per (peer, tensor)
  const int64_t total = int64_t(world) * n_tensors * per_tensor;
  for (int64_t i = blockIdx.x * int64_t(blockDim.x) + threadIdx.x; i < total;
       i += int64_t(gridDim.x) * blockDim.x) {
    int64_t r = i;
    const int64_t c = r % wv; r /= wv;
    const int64_t l = r % seq_local; r /= seq_local;
    const int64_t b = r % batch; r /= batch;
    const int t = int(r % n_tensors);
    const int peer = int(r / n_tensors);
    int64_t off;
    if (heads_split)
      off = ((b * seq_local + l) * world + peer) * wv + c;
    else
      off = ((b * world + peer) * seq_local + l) * wv + c;
    U* x = static_cast<U*>(tensors.p[t]);
    if (to_stage)
      stage[i] = x[off];
    else
      x[off] = stage[i];
  }
}

int grid_for(int64_t n) {
  int64_t b = (n + kThreads - 1) / kThreads;
  const int64_t cap = int64_t(sm_count()) * 16;
  if (b > cap) b = cap;
  if (b < 1) b = 1;
  return int(b);
}

int elem_size(int dtype) { return dtype == TGT_F32 ? 4 : 2; }

int relayout(const void* t0, const void* t1, const void* t2, int n_tensors, const void* stage,
             int64_t batch, int64_t seq_local, int64_t width_local, int world, int dtype,
             bool heads_split, bool to_stage, cudaStream_t stream) {
  TGT_CHECK_ARG(dtype == TGT_F32 || dtype == TGT_BF16, "dtype must be TGT_F32 or TGT_BF16");
  TGT_CHECK_ARG(n_tensors >= 1 && n_tensors <= 3, "n_tensors must be 1, 2 or 3");
  TGT_CHECK_ARG(batch >= 0 && seq_local >= 0 && width_local >= 1 && world >= 1,
                "batch/seq_local must be >= 0, width_local/world >= 1");
  const void* ts[3] = {t0, t1, t2};
  for (int t = 0; t < 3; ++t)
    TGT_CHECK_ARG((t < n_tensors) == (ts[t] != nullptr), "tensor pointers do not match n_tensors");
  if (batch * seq_local == 0) return TGT_OK;
  TGT_CHECK_ARG(stage != nullptr, "stage is null");
  TGT_CHECK_ARG(aligned16(stage) && aligned16(t0) && aligned16(t1) && aligned16(t2),
                "device pointers must be 16-byte aligned");
  const int64_t row_bytes = width_local * elem_size(dtype);
  Ptrs3 p;
  for (int t = 0; t < 3; ++t) p.p[t] = const_cast<void*>(ts[t]);
  void* st = const_cast<void*>(stage);
  const int64_t units_bytes = int64_t(world) * n_tensors * batch * seq_local * row_bytes;
#define TGT_RELAYOUT(U)                                                                         \
  relayout_kernel<U><<<grid_for(units_bytes / int64_t(sizeof(U))), kThreads, 0, stream>>>(      \
      p, static_cast<U*>(st), n_tensors, batch, seq_local, row_bytes / int64_t(sizeof(U)), world, \
      heads_split, to_stage)
  if (row_bytes % 16 == 0) TGT_RELAYOUT(uint4);
  else if (row_bytes % 8 == 0) TGT_RELAYOUT(uint2);
  else if (row_bytes % 4 == 0) TGT_RELAYOUT(uint32_t);
  else TGT_RELAYOUT(uint16_t);
#undef TGT_RELAYOUT
  TGT_CHECK_CUDA(cudaGetLastError());
  return TGT_OK;
}

// x[b, rows[i], :] = x[b, 0, :]   (one block column per (batch, listed row))
template <typename U>
__global__ void global_rows_broadcast_kernel(U* __restrict__ x, const int32_t* __restrict__ rows,
                                             int n_global, int64_t seq, int64_t wv) {
  const int64_t b = blockIdx.y;
  const int i = blockIdx.x;
  const int64_t row = rows[i];
  if (row == 0) return;
  const U* src = x + b * seq * wv;
  U* dst = x + (b * seq + row) * wv;
  for (int64_t c = threadIdx.x; c < wv; c += blockDim.x) dst[c] = src[c];
}

// dx[b,0,:] = sum_i dx[b, rows[i], :] in list order; other listed rows := 0.
template <typename T>
__global__ void global_rows_reduce_kernel(T* __restrict__ dx, const int32_t* __restrict__ rows,
                                          int n_global, int64_t seq, int64_t width) {
  const int64_t b = blockIdx.x;
  for (int64_t c = threadIdx.x; c < width; c += blockDim.x) {
    float s = 0.f;
    bool row0_listed = false;
    for (int i = 0; i < n_global; ++i) {
      row0_listed |= rows[i] == 0;
      const int64_t off = (b * seq + rows[i]) * width + c;
      float val;
      if constexpr (sizeof(T) == 4) val = dx[off]; else val = __bfloat162float(dx[off]);
      s += val;
      if (rows[i] != 0) {
        if constexpr (sizeof(T) == 4) dx[off] = 0.f; else dx[off] = __float2bfloat16(0.f);
      }
    }
    const int64_t off0 = b * seq * width + c;
    if (!row0_listed) {  // row 0 keeps its own gradient when it was not overwritten
      if constexpr (sizeof(T) == 4) s += dx[off0]; else s += __bfloat162float(dx[off0]);
    }
    if constexpr (sizeof(T) == 4) dx[off0] = s; else dx[off0] = __float2bfloat16(s);
  }
}

}  // namespace
}  // namespace tgt

extern "C" int tgt_a2a_pack_heads(const void* x0, const void* x1, const void* x2, int n_tensors,
                                  void* stage, int64_t batch, int64_t seq_local,
                                  int64_t width_local, int world, int dtype, void* stream) {
  return tgt::relayout(x0, x1, x2, n_tensors, stage, batch, seq_local, width_local, world, dtype,
                       true, true, static_cast<cudaStream_t>(stream));
}

extern "C" int tgt_a2a_unpack_seq(const void* stage, int n_tensors, void* y0, void* y1, void* y2,
                                  int64_t batch, int64_t seq_local, int64_t width_local, int world,
                                  int dtype, void* stream) {
  return tgt::relayout(y0, y1, y2, n_tensors, stage, batch, seq_local, width_local, world, dtype,
                       false, false, static_cast<cudaStream_t>(stream));
}

extern "C" int tgt_a2a_pack_seq(const void* x0, const void* x1, const void* x2, int n_tensors,
                                void* stage, int64_t batch, int64_t seq_local, int64_t width_local,
                                int world, int dtype, void* stream) {
  return tgt::relayout(x0, x1, x2, n_tensors, stage, batch, seq_local, width_local, world, dtype,
                       false, true, static_cast<cudaStream_t>(stream));
}

extern "C" int tgt_a2a_unpack_heads(const void* stage, int n_tensors, void* y0, void* y1, void* y2,
                                    int64_t batch, int64_t seq_local, int64_t width_local,
                                    int world, int dtype, void* stream) {
  return tgt::relayout(y0, y1, y2, n_tensors, stage, batch, seq_local, width_local, world, dtype,
                       true, false, static_cast<cudaStream_t>(stream));
}

extern "C" int tgt_global_rows_broadcast(void* x, const int32_t* global_rows, int n_global,
                                         int64_t batch, int64_t seq, int64_t width, int dtype,
                                         void* stream_) {
  using namespace tgt;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  TGT_CHECK_ARG(dtype == TGT_F32 || dtype == TGT_BF16, "dtype must be TGT_F32 or TGT_BF16");
  TGT_CHECK_ARG(n_global >= 0 && batch >= 0 && seq >= 0 && width >= 1, "negative size");
  if (n_global == 0 || batch == 0 || seq == 0) return TGT_OK;
  TGT_CHECK_ARG(x && global_rows, "x / global_rows is null");
  TGT_CHECK_ARG(batch <= 65535, "batch must be <= 65535");
  const int64_t row_bytes = width * elem_size(dtype);
  dim3 grid(n_global, unsigned(batch));
  if (row_bytes % 16 == 0 && aligned16(x))
    global_rows_broadcast_kernel<uint4><<<grid, 128, 0, stream>>>(
        static_cast<uint4*>(x), global_rows, n_global, seq, row_bytes / 16);
  else
    global_rows_broadcast_kernel<uint16_t><<<grid, 128, 0, stream>>>(
        static_cast<uint16_t*>(x), global_rows, n_global, seq, row_bytes / 2);
  TGT_CHECK_CUDA(cudaGetLastError());
  return TGT_OK;
}

extern "C" int tgt_global_rows_reduce(void* dx, const int32_t* global_rows, int n_global,
                                      int64_t batch, int64_t seq, int64_t width, int dtype,
                                      void* stream_) {
  using namespace tgt;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  TGT_CHECK_ARG(dtype == TGT_F32 || dtype == TGT_BF16, "dtype must be TGT_F32 or TGT_BF16");
  TGT_CHECK_ARG(n_global >= 0 && batch >= 0 && seq >= 0 && width >= 1, "negative size");
  if (n_global == 0 || batch == 0 || seq == 0) return TGT_OK;
  TGT_CHECK_ARG(dx && global_rows, "dx / global_rows is null");
  if (dtype == TGT_F32)
    global_rows_reduce_kernel<float><<<unsigned(batch), 128, 0, stream>>>(
        static_cast<float*>(dx), global_rows, n_global, seq, width);
  else
    global_rows_reduce_kernel<__nv_bfloat16><<<unsigned(batch), 128, 0, stream>>>(
        static_cast<__nv_bfloat16*>(dx), global_rows, n_global, seq, width);
  TGT_CHECK_CUDA(cudaGetLastError());
  return TGT_OK;
}
