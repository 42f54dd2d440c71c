// Weight and bias gradient of a narrow nn.Linear over many rows: dW[o][i] = sum_r dY[r][o] X[r][i],
// db[o] = sum_r dY[r][o], fp32.  The graph transformers' projections are 64 x 64 (128 x 64 for the node
// encoder) over 64,000 to 870,000 rows (models/graphormer_dist_node_level.py:241-245,281-286,343: linear_q/k/v,
// output_layer, the two FFN layers, node_encoder): a product with a tiny result and a very long reduction,
// which a library GEMM runs split over a few CTAs (66 us at 64,001 rows, plus 25 us for the bias sum).
// Here every CTA walks its share of the rows in chunks staged in shared memory and keeps a 64 x 64 tile of
// dW in registers (4 x 4 per thread, fp32 FMA); the CTAs' tiles are then added in a fixed order by a second
// kernel.  No atomics: results are bitwise reproducible.
#include "tgt_common.cuh"

namespace tgt {
namespace {

constexpr int kWgThreads = 256;
constexpr int kWgTile = 64;        // outputs and inputs per tile
constexpr int kWgChunk = 32;       // rows staged at a time

struct WgradParams {
  const float* dy;   // [rows, out]
  const float* x;    // [rows, in]
  float* partial;    // [gridDim.x][out * in + out]
  int64_t rows;
  int in, out;
};

__global__ void __launch_bounds__(kWgThreads) linear_wgrad_kernel(const WgradParams p) {
  __shared__ __align__(16) float s_dy[kWgChunk][kWgTile];
  __shared__ __align__(16) float s_x[kWgChunk][kWgTile];
  const int tid = threadIdx.x;
  const int ty = tid / 16, tx = tid % 16;
  const int tiles_in = p.in / kWgTile;
  const int o0 = (blockIdx.y / tiles_in) * kWgTile, i0 = (blockIdx.y % tiles_in) * kWgTile;
  float acc[4][4];
#pragma unroll
  for (int a = 0; a < 4; ++a)
#pragma unroll
    for (int b = 0; b < 4; ++b) acc[a][b] = 0.f;
  float bias_acc = 0.f;          // thread tid < 64 sums column o0 + tid of dY
  const int64_t n_chunks = (p.rows + kWgChunk - 1) / kWgChunk;
  // the loads of the next chunk are issued before the arithmetic of this one
  float4 next_dy[2], next_x[2];
  auto fetch = [&](int64_t chunk) {
#pragma unroll
    for (int j = 0; j < 2; ++j) {
      const int u = tid + j * kWgThreads;            // 512 float4 per operand: 32 rows x 16
      const int r = u / 16, c4 = u % 16;
      const int64_t row = chunk * kWgChunk + r;
      const bool live = chunk < n_chunks && row < p.rows;
      next_dy[j] = live ? __ldg(reinterpret_cast<const float4*>(p.dy + row * p.out + o0) + c4) : make_float4(0.f, 0.f, 0.f, 0.f);
      next_x[j] = live ? __ldg(reinterpret_cast<const float4*>(p.x + row * p.in + i0) + c4) : make_float4(0.f, 0.f, 0.f, 0.f);
    }
  };
  fetch(blockIdx.x);
  for (int64_t chunk = blockIdx.x; chunk < n_chunks; chunk += gridDim.x) {
    __syncthreads();                                 // the previous chunk has been consumed
#pragma unroll
    for (int j = 0; j < 2; ++j) {
      const int u = tid + j * kWgThreads;
      const int r = u / 16, c4 = u % 16;
      *reinterpret_cast<float4*>(&s_dy[r][4 * c4]) = next_dy[j];
      *reinterpret_cast<float4*>(&s_x[r][4 * c4]) = next_x[j];
    }
    __syncthreads();
    fetch(chunk + gridDim.x);
#pragma unroll 8
    for (int r = 0; r < kWgChunk; ++r) {
      const float4 a = *reinterpret_cast<const float4*>(&s_dy[r][4 * ty]);
      const float4 b = *reinterpret_cast<const float4*>(&s_x[r][4 * tx]);
      acc[0][0] = fmaf(a.x, b.x, acc[0][0]); acc[0][1] = fmaf(a.x, b.y, acc[0][1]);
      acc[0][2] = fmaf(a.x, b.z, acc[0][2]); acc[0][3] = fmaf(a.x, b.w, acc[0][3]);
      acc[1][0] = fmaf(a.y, b.x, acc[1][0]); acc[1][1] = fmaf(a.y, b.y, acc[1][1]);
      acc[1][2] = fmaf(a.y, b.z, acc[1][2]); acc[1][3] = fmaf(a.y, b.w, acc[1][3]);
      acc[2][0] = fmaf(a.z, b.x, acc[2][0]); acc[2][1] = fmaf(a.z, b.y, acc[2][1]);
      acc[2][2] = fmaf(a.z, b.z, acc[2][2]); acc[2][3] = fmaf(a.z, b.w, acc[2][3]);
      acc[3][0] = fmaf(a.w, b.x, acc[3][0]); acc[3][1] = fmaf(a.w, b.y, acc[3][1]);
      acc[3][2] = fmaf(a.w, b.z, acc[3][2]); acc[3][3] = fmaf(a.w, b.w, acc[3][3]);
    }
    if (tid < kWgTile) {
#pragma unroll 8
      for (int r = 0; r < kWgChunk; ++r) bias_acc += s_dy[r][tid];
    }
  }
  float* out = p.partial + int64_t(blockIdx.x) * (int64_t(p.out) * p.in + p.out);
#pragma unroll
  for (int a = 0; a < 4; ++a)
    *reinterpret_cast<float4*>(out + int64_t(o0 + 4 * ty + a) * p.in + i0 + 4 * tx) =
        make_float4(acc[a][0], acc[a][1], acc[a][2], acc[a][3]);
  if (tid < kWgTile && i0 == 0) out[int64_t(p.out) * p.in + o0 + tid] = bias_acc;
}

// dw[j] = sum over CTAs of partial[cta][j], db likewise (db may be null).  A block owns 32 consecutive
// values; its warp w adds the CTAs w, w + 8, ... (two running sums), then the eight sums are added in warp
// order: a fixed association, whatever the timing.
__global__ void __launch_bounds__(256) linear_wgrad_sum_kernel(const float* __restrict__ partial, int ctas, int n_w,
                                                               int n_b, float* __restrict__ dw,
                                                               float* __restrict__ db) {
  __shared__ float s_part[8][32];
  const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
  const int i = blockIdx.x * 32 + lane;
  const int64_t pitch = int64_t(n_w) + n_b;
  float s0 = 0.f, s1 = 0.f;
  if (i < n_w + n_b) {
    int b = warp;
    for (; b + 8 < ctas; b += 16) {
      s0 += __ldg(partial + int64_t(b) * pitch + i);
      s1 += __ldg(partial + int64_t(b + 8) * pitch + i);
    }
    if (b < ctas) s0 += __ldg(partial + int64_t(b) * pitch + i);
  }
  s_part[warp][lane] = s0 + s1;
  __syncthreads();
  if (warp == 0 && i < n_w + n_b) {
    float s = s_part[0][lane];
#pragma unroll
    for (int w = 1; w < 8; ++w) s += s_part[w][lane];
    if (i < n_w) dw[i] = s;
    else if (db != nullptr) db[i - n_w] = s;
  }
}

bool wgrad_supported(int in, int out) {
  return in >= kWgTile && out >= kWgTile && in % kWgTile == 0 && out % kWgTile == 0 && in <= 1024 && out <= 1024;
}

int wgrad_grid(int64_t rows, int in, int out) {
  const int tiles = (in / kWgTile) * (out / kWgTile);
  const int64_t chunks = (rows + kWgChunk - 1) / kWgChunk;
  int64_t g = int64_t(sm_count()) * 2 / tiles;     // about two CTAs per SM over all tiles
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
    return set_error(TGT_ERR_UNSUPPORTED, "in_features=%d out_features=%d: both must be multiples of 64, at most 1024",
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
    return set_error(TGT_ERR_UNSUPPORTED, "in_features=%d out_features=%d: both must be multiples of 64, at most 1024",
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
  const dim3 g(grid, (in_features / kWgTile) * (out_features / kWgTile));
  linear_wgrad_kernel<<<g, kWgThreads, 0, stream>>>(p);
  const int n = int(n_w) + out_features;
  linear_wgrad_sum_kernel<<<(n + 31) / 32, 256, 0, stream>>>(p.partial, grid, int(n_w), out_features, dw, db);
  TGT_CHECK_CUDA(cudaGetLastError());
  return TGT_OK;
}
