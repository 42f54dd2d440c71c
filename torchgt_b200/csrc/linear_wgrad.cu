// Weight and bias gradient of a narrow nn.Linear over many rows: dW[o][i] = sum_r dY[r][o] X[r][i],
// db[o] = sum_r dY[r][o], fp32.  The graph transformers' projections are 64 x 64 (128 x 64 for the node
// encoder) over 64,000 to 870,000 rows (models/graphormer_dist_node_level.py:241-245,281-286,343: linear_q/k/v,
// output_layer, the two FFN layers, node_encoder): a product with a tiny result and a very long reduction,
// which a library GEMM runs split over a few CTAs (66 us at 64,001 rows, plus 25 us for the bias sum).
// Here every CTA walks its share of the rows in chunks staged in shared memory and keeps a 64 x 64 tile of
// dW in registers (8 x 8 per thread, fp32 FMA); the CTAs' tiles are then added in a fixed order by a second
// kernel.  No atomics: results are bitwise reproducible.
#include "tgt_common.cuh"

namespace tgt {
namespace {

constexpr int kWgThreads = 64;
constexpr int kWgTile = 64;        // outputs and inputs per tile
constexpr int kWgChunk = 32;       // rows staged at a time

struct WgradParams {
  const float* dy;   // [rows, out]
  const float* x;    // [rows, in]
  float* partial;    // [gridDim.x][out * in + out]
  int64_t rows;
  int in, out;
};

// 16 bytes global -> shared without passing through registers; bytes = 0 fills the destination with zeros
__device__ __forceinline__ void copy_async_16(void* smem_dst, const void* src, int bytes) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(uint32_t(__cvta_generic_to_shared(smem_dst))),
               "l"(src), "r"(bytes)
               : "memory");
}

// Two warps per CTA; thread (ty, tx) of the 8 x 8 grid owns outputs {4 ty .. 4 ty + 3, 32 + 4 ty .. 32 + 4 ty + 3}
// x inputs {4 tx .. 4 tx + 3, 32 + 4 tx .. 32 + 4 tx + 3}: per staged row four 16-byte shared-memory reads (two of
// them the same address for the eight lanes of a quarter warp, two contiguous over them) feed 64 FMAs, so the
// FMA pipe, not shared memory, sets the pace.  Chunks of 32 rows are double-buffered with asynchronous copies.
__global__ void __launch_bounds__(kWgThreads) linear_wgrad_kernel(const WgradParams p) {
  __shared__ __align__(16) float s_dy[2][kWgChunk][kWgTile];
  __shared__ __align__(16) float s_x[2][kWgChunk][kWgTile];
  const int tid = threadIdx.x;
  const int ty = tid / 8, tx = tid % 8;
  const int tiles_in = p.in / kWgTile;
  const int o0 = (blockIdx.y / tiles_in) * kWgTile, i0 = (blockIdx.y % tiles_in) * kWgTile;
  float acc[8][8];
#pragma unroll
  for (int a = 0; a < 8; ++a)
#pragma unroll
    for (int b = 0; b < 8; ++b) acc[a][b] = 0.f;
  float bias_acc = 0.f;          // thread tid sums column o0 + tid of dY
  const int64_t n_chunks = (p.rows + kWgChunk - 1) / kWgChunk;
  auto stage = [&](int64_t chunk, int buf) {
#pragma unroll
    for (int j = 0; j < kWgChunk * 16 / kWgThreads; ++j) {
      const int u = tid + j * kWgThreads;            // 512 pieces of 16 bytes per operand: 32 rows x 16
      const int r = u / 16, c4 = u % 16;
      const int64_t row = chunk * kWgChunk + r;
      const bool live = row < p.rows;
      const int64_t from = live ? row : 0;
      const bool col = o0 + 4 * c4 < p.out;          // the last tile of outputs may be narrower than 64
      copy_async_16(&s_dy[buf][r][4 * c4], p.dy + from * p.out + (col ? o0 + 4 * c4 : 0), live && col ? 16 : 0);
      copy_async_16(&s_x[buf][r][4 * c4], p.x + from * p.in + i0 + 4 * c4, live ? 16 : 0);
    }
  };
  if (int64_t(blockIdx.x) < n_chunks) stage(blockIdx.x, 0);
  asm volatile("cp.async.commit_group;" ::: "memory");
  int buf = 0;
  for (int64_t chunk = blockIdx.x; chunk < n_chunks; chunk += gridDim.x, buf ^= 1) {
    if (chunk + gridDim.x < n_chunks) stage(chunk + gridDim.x, buf ^ 1);
    asm volatile("cp.async.commit_group;" ::: "memory");
    asm volatile("cp.async.wait_group 1;" ::: "memory");     // this chunk's copies have landed
    __syncthreads();
#pragma unroll 4
    for (int r = 0; r < kWgChunk; ++r) {
      const float4 a0 = *reinterpret_cast<const float4*>(&s_dy[buf][r][4 * ty]);
      const float4 a1 = *reinterpret_cast<const float4*>(&s_dy[buf][r][32 + 4 * ty]);
      const float4 b0 = *reinterpret_cast<const float4*>(&s_x[buf][r][4 * tx]);
      const float4 b1 = *reinterpret_cast<const float4*>(&s_x[buf][r][32 + 4 * tx]);
      const float av[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w};
      const float bv[8] = {b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w};
#pragma unroll
      for (int a = 0; a < 8; ++a)
#pragma unroll
        for (int b = 0; b < 8; ++b) acc[a][b] = fmaf(av[a], bv[b], acc[a][b]);
    }
    if (i0 == 0) {
#pragma unroll 8
      for (int r = 0; r < kWgChunk; ++r) bias_acc += s_dy[buf][r][tid];
    }
    __syncthreads();                                 // the next iteration's copies overwrite this buffer
  }
  asm volatile("cp.async.wait_group 0;" ::: "memory");
  float* out = p.partial + int64_t(blockIdx.x) * (int64_t(p.out) * p.in + p.out);
#pragma unroll
  for (int a = 0; a < 8; ++a) {
    const int o = o0 + (a < 4 ? 4 * ty + a : 32 + 4 * ty + a - 4);
    if (o >= p.out) continue;
    *reinterpret_cast<float4*>(out + int64_t(o) * p.in + i0 + 4 * tx) = make_float4(acc[a][0], acc[a][1], acc[a][2], acc[a][3]);
    *reinterpret_cast<float4*>(out + int64_t(o) * p.in + i0 + 32 + 4 * tx) = make_float4(acc[a][4], acc[a][5], acc[a][6], acc[a][7]);
  }
  if (i0 == 0 && o0 + tid < p.out) out[int64_t(p.out) * p.in + o0 + tid] = bias_acc;
}

// dw[j] = sum over CTAs of partial[cta][j], db likewise (db may be null); sum_partials: fixed association.
__global__ void __launch_bounds__(kPartialSumThreads) linear_wgrad_sum_kernel(const float* __restrict__ partial,
                                                                              int ctas, int n_w, int n_b,
                                                                              float* __restrict__ dw,
                                                                              float* __restrict__ db) {
  __shared__ float s_part[16][32];
  const int i = blockIdx.x * 32 + threadIdx.x % 32;
  const bool live = i < n_w + n_b;
  const float s = sum_partials(partial, ctas, int64_t(n_w) + n_b, i, live, s_part);
  if (threadIdx.x < 32 && live) {
    if (i < n_w) dw[i] = s;
    else if (db != nullptr) db[i - n_w] = s;
  }
}

// inputs in whole tiles of 64; outputs any multiple of 4 (a classifier head of 40 classes, say): the last tile
// of outputs is padded with zero columns that are never stored
bool wgrad_supported(int in, int out) {
  return in >= kWgTile && in % kWgTile == 0 && in <= 1024 && out >= 4 && out % 4 == 0 && out <= 1024;
}
int wgrad_out_tiles(int out) { return (out + kWgTile - 1) / kWgTile; }

int wgrad_grid(int64_t rows, int in, int out) {
  const int tiles = (in / kWgTile) * wgrad_out_tiles(out);
  const int64_t chunks = (rows + kWgChunk - 1) / kWgChunk;
  int64_t g = int64_t(sm_count()) * 4 / tiles;     // about four CTAs (of two warps) per SM over all tiles
  if (g < 1) g = 1;
  if (g > chunks) g = chunks < 1 ? 1 : chunks;
  return int(g);
}

}  // namespace
}  // namespace tgt

extern "C" int tgt_linear_wgrad_scratch_bytes(int64_t rows, int in_features, int out_features, size_t* bytes) {
  using namespace tgt;
  TGT_CHECK_ARG(bytes != nullptr, "bytes is null");
  TGT_CHECK_ARG(rows >= 0, "rows must be >= 0");
  if (!wgrad_supported(in_features, out_features))
    return set_error(TGT_ERR_UNSUPPORTED, "in_features=%d out_features=%d: in_features must be a multiple of 64, out_features of 4, both at most 1024",
                     in_features, out_features);
  *bytes = size_t(wgrad_grid(rows, in_features, out_features)) *
           (size_t(in_features) * out_features + out_features) * sizeof(float);
  return TGT_OK;
}

extern "C" int tgt_linear_wgrad(const float* dy, const float* x, int64_t rows, int in_features, int out_features,
                                float* dw, float* db, void* scratch, size_t scratch_bytes, void* stream_) {
  using namespace tgt;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  TGT_CHECK_ARG(rows >= 0, "rows must be >= 0");
  if (!wgrad_supported(in_features, out_features))
    return set_error(TGT_ERR_UNSUPPORTED, "in_features=%d out_features=%d: in_features must be a multiple of 64, out_features of 4, both at most 1024",
                     in_features, out_features);
  TGT_CHECK_ARG(dw != nullptr, "dw must not be null");
  const size_t n_w = size_t(in_features) * out_features;
  if (rows == 0) {
    TGT_CHECK_CUDA(cudaMemsetAsync(dw, 0, n_w * sizeof(float), stream));
    if (db != nullptr) TGT_CHECK_CUDA(cudaMemsetAsync(db, 0, size_t(out_features) * sizeof(float), stream));
    return TGT_OK;
  }
  TGT_CHECK_ARG(dy && x, "dy and x must not be null");
  TGT_CHECK_ARG(aligned16(dy) && aligned16(x) && aligned16(dw) && aligned16(scratch), "tensors must be 16-byte aligned");
  const int grid = wgrad_grid(rows, in_features, out_features);
  const size_t need = size_t(grid) * (n_w + out_features) * sizeof(float);
  if (scratch == nullptr || scratch_bytes < need)
    return set_error(TGT_ERR_WORKSPACE, "scratch holds %zu bytes, %zu needed", scratch_bytes, need);
  WgradParams p{dy, x, static_cast<float*>(scratch), rows, in_features, out_features};
  const dim3 g(grid, (in_features / kWgTile) * wgrad_out_tiles(out_features));
  linear_wgrad_kernel<<<g, kWgThreads, 0, stream>>>(p);
  const int n = int(n_w) + out_features;
  linear_wgrad_sum_kernel<<<(n + 31) / 32, kPartialSumThreads, 0, stream>>>(p.partial, grid, int(n_w), out_features, dw, db);
  TGT_CHECK_CUDA(cudaGetLastError());
  return TGT_OK;
}
