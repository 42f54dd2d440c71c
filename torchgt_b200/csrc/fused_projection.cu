// The dense layers on either side of the Ulysses exchange, fused with the exchange itself.
//
// What the reference runs per encoder layer around its attention (models/graphormer_dist_node_level.py:
// 301 LayerNorm, :254-257 three nn.Linear, gt_sp/layer.py:41 a `contiguous` copy per chunk and three
// all-to-alls; on the way back :271 the output nn.Linear after gt_sp/utils.py:836 copy_global_token0
// and one more all-to-all) becomes two kernels that compute AND move:
//
//   ln_qkv_push   per tile of rows: LayerNorm -> Q, K, V = xn W^T + b (fp32 FMA, weights resident in
//                 shared memory) -> every head slice is stored straight at its final position in the
//                 slot of the rank that owns those heads (plain stores into peer memory over NVLink;
//                 rows of one tile form one contiguous run per peer and tensor).  No q/k/v tensor, no
//                 pack pass, no collective launch; the NVLink stores of one tile overlap the arithmetic
//                 of the next.
//   pull_out_proj per tile of rows: read this rank's rows of every peer's attention output (contiguous
//                 runs over NVLink; global-token slots read row 0 instead), keep the gathered tile for
//                 the weight gradient, and multiply by the output projection while it is on chip.
//
// Both need the barrier of peer_exchange.cu between producers and consumers (after ln_qkv_push and
// before the attention; after the attention and before pull_out_proj).  Hidden size and projection
// width are compile-time (64, the reference models' size, is built: its three weight matrices fit one SM's
// shared memory twice over); everything else takes the separate kernels.
#include "tgt_common.cuh"

namespace tgt {
namespace {

constexpr int kMaxWorld = 16;
constexpr int kThreads = 256;
constexpr int kTileRows = 32;

struct PeerTable {
  void* p[kMaxWorld];
};

struct QkvParams {
  const float* x;        // [rows_total, HIDDEN]
  const float* gamma;    // [HIDDEN] or null (no LayerNorm)
  const float* beta;
  float eps;
  const float* w[3];     // [OUT, HIDDEN] each (nn.Linear layout)
  const float* b[3];     // [OUT] each
  PeerTable slots;       // q | k | v back to back in every rank's slot
  int64_t tensor_bytes;  // bytes of one gathered tensor in a slot
  int64_t rows_total;    // batch * rows
  int64_t rows;          // rows per batch entry on this rank
  int world, rank;
};

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
  return v;
}

// out[r][c] = sum_k a[r][k] * w[c][k] for the thread's rows {2 ty, 2 ty + 1} and columns {j * 16 + tx}.
// a: [kTileRows][K + 4], w: [COLS][K + 4] in shared memory (the padding keeps quarter-warps of 128-bit
// loads on different banks).
template <int K, int NJ>
__device__ __forceinline__ void tile_gemm(const float* __restrict__ a, const float* __restrict__ w, int ty, int tx,
                                          float (&acc)[2][NJ]) {
  constexpr int LD = K + 4;
#pragma unroll
  for (int i = 0; i < 2; ++i)
#pragma unroll
    for (int j = 0; j < NJ; ++j) acc[i][j] = 0.f;
#pragma unroll 4
  for (int k = 0; k < K; k += 4) {
    const float4 a0 = *reinterpret_cast<const float4*>(a + (2 * ty) * LD + k);
    const float4 a1 = *reinterpret_cast<const float4*>(a + (2 * ty + 1) * LD + k);
#pragma unroll
    for (int j = 0; j < NJ; ++j) {
      const float4 b = *reinterpret_cast<const float4*>(w + (j * 16 + tx) * LD + k);
      acc[0][j] = fmaf(a0.x, b.x, acc[0][j]); acc[0][j] = fmaf(a0.y, b.y, acc[0][j]);
      acc[0][j] = fmaf(a0.z, b.z, acc[0][j]); acc[0][j] = fmaf(a0.w, b.w, acc[0][j]);
      acc[1][j] = fmaf(a1.x, b.x, acc[1][j]); acc[1][j] = fmaf(a1.y, b.y, acc[1][j]);
      acc[1][j] = fmaf(a1.z, b.z, acc[1][j]); acc[1][j] = fmaf(a1.w, b.w, acc[1][j]);
    }
  }
}

// Shared memory: weights (3 OUT x (HIDDEN + 4)), biases, gamma / beta, the input tile, the output tile.
template <int HIDDEN, int OUT>
struct QkvSmem {
  static constexpr int LD = HIDDEN + 4;
  static constexpr int LDO = 3 * OUT + 4;   // row pitch of the output tile (keeps half-warps on different banks)
  static constexpr size_t floats = size_t(3) * OUT * LD + 3 * OUT + 2 * HIDDEN + size_t(kTileRows) * LD +
                                   size_t(kTileRows) * LDO;
};

template <int HIDDEN, int OUT>
__global__ void __launch_bounds__(kThreads) ln_qkv_push_kernel(const QkvParams p) {
  constexpr int LD = HIDDEN + 4;
  constexpr int LDO = QkvSmem<HIDDEN, OUT>::LDO;
  constexpr int NJ = 3 * OUT / 16;                 // output columns per thread
  extern __shared__ __align__(16) float smem[];
  float* s_w = smem;                               // [3 * OUT][LD]
  float* s_b = s_w + 3 * OUT * LD;                 // [3 * OUT]
  float* s_g = s_b + 3 * OUT;                      // gamma, beta
  float* s_x = s_g + 2 * HIDDEN;                   // [kTileRows][LD]
  float* s_o = s_x + kTileRows * LD;               // [kTileRows][LDO]
  const int tid = threadIdx.x;
  for (int i = tid; i < 3 * OUT * HIDDEN; i += kThreads) {
    const int c = i / HIDDEN, k = i % HIDDEN;
    s_w[c * LD + k] = __ldg(p.w[c / OUT] + (c % OUT) * HIDDEN + k);
  }
  for (int i = tid; i < 3 * OUT; i += kThreads) s_b[i] = __ldg(p.b[i / OUT] + i % OUT);
  for (int i = tid; i < HIDDEN; i += kThreads) {
    s_g[i] = p.gamma != nullptr ? __ldg(p.gamma + i) : 1.f;
    s_g[HIDDEN + i] = p.gamma != nullptr ? __ldg(p.beta + i) : 0.f;
  }
  const int warp = tid / 32, lane = tid % 32;
  const int ty = tid / 16, tx = tid % 16;
  const int cols_per_peer = OUT / p.world;         // floats of one head slice
  const int units_per_row = cols_per_peer / 4;     // 16-byte units one peer gets from one row and tensor
  const int64_t n_tiles = (p.rows_total + kTileRows - 1) / kTileRows;
  for (int64_t tile = blockIdx.x; tile < n_tiles; tile += gridDim.x) {
    const int64_t row0 = tile * kTileRows;
    const int n = int(min(int64_t(kTileRows), p.rows_total - row0));
    __syncthreads();                               // the previous tile's stores have read s_o; weights are in place
    for (int i = tid; i < kTileRows * (HIDDEN / 4); i += kThreads) {
      const int r = i / (HIDDEN / 4), k4 = i % (HIDDEN / 4);
      float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
      if (r < n) v = __ldg(reinterpret_cast<const float4*>(p.x + (row0 + r) * HIDDEN) + k4);
      *reinterpret_cast<float4*>(s_x + r * LD + 4 * k4) = v;
    }
    __syncthreads();
    if (p.gamma != nullptr) {
      // LayerNorm, one warp per row: biased variance, as torch.nn.LayerNorm
      for (int r = warp; r < n; r += kThreads / 32) {
        float v[HIDDEN / 32];
        float s = 0.f;
#pragma unroll
        for (int i = 0; i < HIDDEN / 32; ++i) { v[i] = s_x[r * LD + lane + 32 * i]; s += v[i]; }
        const float mean = warp_sum(s) * (1.0f / HIDDEN);
        float q = 0.f;
#pragma unroll
        for (int i = 0; i < HIDDEN / 32; ++i) { v[i] -= mean; q += v[i] * v[i]; }
        const float rstd = 1.0f / sqrtf(warp_sum(q) * (1.0f / HIDDEN) + p.eps);
#pragma unroll
        for (int i = 0; i < HIDDEN / 32; ++i) {
          const int k = lane + 32 * i;
          s_x[r * LD + k] = v[i] * rstd * s_g[k] + s_g[HIDDEN + k];
        }
      }
      __syncthreads();
    }
    float acc[2][NJ];
    tile_gemm<HIDDEN, NJ>(s_x, s_w, ty, tx, acc);
#pragma unroll
    for (int i = 0; i < 2; ++i)
#pragma unroll
      for (int j = 0; j < NJ; ++j) s_o[(2 * ty + i) * LDO + j * 16 + tx] = acc[i][j] + s_b[j * 16 + tx];
    __syncthreads();
    // Store the tile: for every tensor and peer the rows of the tile are one contiguous run on the peer
    // (gathered row = (batch entry * world + rank) * rows + l, row width = one head slice).
    const int units_per_run = kTileRows * units_per_row;
    const int total_units = 3 * p.world * units_per_run;
    for (int u = tid; u < total_units; u += kThreads) {
      const int run = u / units_per_run, in_run = u % units_per_run;
      const int t = run / p.world;
      const int peer = (p.rank + 1 + run % p.world) % p.world;     // start with the next rank
      const int r = in_run / units_per_row, w = in_run % units_per_row;
      if (r >= n) continue;
      const int64_t gi = row0 + r;
      const int64_t bi = gi / p.rows, l = gi % p.rows;
      const int64_t dest_row = (bi * p.world + p.rank) * p.rows + l;
      const float4 val = *reinterpret_cast<const float4*>(s_o + r * LDO + t * OUT + peer * cols_per_peer + 4 * w);
      float4* dst = reinterpret_cast<float4*>(static_cast<char*>(p.slots.p[peer]) + t * p.tensor_bytes) +
                    dest_row * units_per_row + w;
      *dst = val;
    }
  }
}

struct OutProjParams {
  PeerTable slots;       // every rank's attention output [batch][world * rows][OUT / world]
  const float* w;        // [HIDDEN, OUT] (nn.Linear layout: out_features = HIDDEN)
  const float* b;        // [HIDDEN]
  float* ctx;            // [rows_total, OUT] the gathered attention output (kept for the weight gradient)
  float* y;              // [rows_total, HIDDEN]
  const int32_t* alias_rows;
  int n_alias;
  int64_t rows_total, rows;
  int world, rank;
};

template <int HIDDEN, int OUT>
struct OutSmem {
  static constexpr int LD = OUT + 4;
  static constexpr size_t floats = size_t(HIDDEN) * LD + HIDDEN + size_t(kTileRows) * LD;
};

template <int HIDDEN, int OUT>
__global__ void __launch_bounds__(kThreads) pull_out_proj_kernel(const OutProjParams p) {
  constexpr int LD = OUT + 4;
  constexpr int NJ = HIDDEN / 16;
  extern __shared__ __align__(16) float smem[];
  float* s_w = smem;                  // [HIDDEN][LD]
  float* s_b = s_w + HIDDEN * LD;     // [HIDDEN]
  float* s_c = s_b + HIDDEN;          // [kTileRows][LD] gathered tile
  const int tid = threadIdx.x;
  for (int i = tid; i < HIDDEN * OUT; i += kThreads) s_w[(i / OUT) * LD + i % OUT] = __ldg(p.w + i);
  for (int i = tid; i < HIDDEN; i += kThreads) s_b[i] = __ldg(p.b + i);
  const int ty = tid / 16, tx = tid % 16;
  const int cols_per_peer = OUT / p.world;
  const int units_per_row = cols_per_peer / 4;
  const int64_t n_tiles = (p.rows_total + kTileRows - 1) / kTileRows;
  for (int64_t tile = blockIdx.x; tile < n_tiles; tile += gridDim.x) {
    const int64_t row0 = tile * kTileRows;
    const int n = int(min(int64_t(kTileRows), p.rows_total - row0));
    __syncthreads();
    // gather: for every peer the tile's rows are one contiguous run in the peer's slot
    const int units_per_run = kTileRows * units_per_row;
    for (int u = tid; u < p.world * units_per_run; u += kThreads) {
      const int run = u / units_per_run, in_run = u % units_per_run;
      const int peer = (p.rank + 1 + run) % p.world;
      const int r = in_run / units_per_row, w = in_run % units_per_row;
      float4 val = make_float4(0.f, 0.f, 0.f, 0.f);
      if (r < n) {
        const int64_t gi = row0 + r;
        const int64_t bi = gi / p.rows, l = gi % p.rows;
        int64_t src_row = int64_t(p.rank) * p.rows + l;
        for (int j = 0; j < p.n_alias; ++j)
          if (src_row == p.alias_rows[j]) {   // global-token slots take row 0's output
            src_row = 0;
            break;
          }
        val = *(reinterpret_cast<const float4*>(p.slots.p[peer]) + (bi * p.world * p.rows + src_row) * units_per_row + w);
        *(reinterpret_cast<float4*>(p.ctx + gi * OUT + peer * cols_per_peer) + w) = val;
      }
      *reinterpret_cast<float4*>(s_c + r * LD + peer * cols_per_peer + 4 * w) = val;
    }
    __syncthreads();
    float acc[2][NJ];
    tile_gemm<OUT, NJ>(s_c, s_w, ty, tx, acc);
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const int r = 2 * ty + i;
      if (r < n) {
#pragma unroll
        for (int j = 0; j < NJ; ++j) p.y[(row0 + r) * HIDDEN + j * 16 + tx] = acc[i][j] + s_b[j * 16 + tx];
      }
    }
  }
}

int fill_slots(PeerTable* tab, void* const* peers, int world) {
  TGT_CHECK_ARG(world >= 1 && world <= kMaxWorld, "world must be between 1 and 16");
  TGT_CHECK_ARG(peers != nullptr, "peer table is null");
  for (int i = 0; i < kMaxWorld; ++i) tab->p[i] = nullptr;
  for (int i = 0; i < world; ++i) {
    TGT_CHECK_ARG(peers[i] != nullptr && aligned16(peers[i]), "peer pointers must be non-null and 16-byte aligned");
    tab->p[i] = peers[i];
  }
  return TGT_OK;
}

template <typename Kernel>
int launch_grid(Kernel kernel, size_t smem_bytes, int64_t n_tiles, int* grid) {
  TGT_CHECK_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem_bytes)));
  int per_sm = 0;
  TGT_CHECK_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, kThreads, smem_bytes));
  if (per_sm < 1) return set_error(TGT_ERR_UNSUPPORTED, "the fused projection kernel does not fit an SM");
  int64_t g = int64_t(sm_count()) * per_sm;     // persistent CTAs: one wave, tiles dealt round-robin
  if (g > n_tiles) g = n_tiles;
  *grid = int(g < 1 ? 1 : g);
  return TGT_OK;
}

}  // namespace
}  // namespace tgt

extern "C" int tgt_ln_qkv_push(const float* x, const float* gamma, const float* beta, float eps,
                               const float* wq, const float* bq, const float* wk, const float* bk,
                               const float* wv, const float* bv, int hidden, int out_features,
                               void* const* peer_slots, size_t slot_bytes, int64_t batch, int64_t rows,
                               int world, int rank, void* stream_) {
  using namespace tgt;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  TGT_CHECK_ARG(x && wq && bq && wk && bk && wv && bv, "x, the three weights and the three biases must not be null");
  TGT_CHECK_ARG((gamma == nullptr) == (beta == nullptr), "give both LayerNorm parameters or neither");
  TGT_CHECK_ARG(batch >= 1 && rows >= 1, "batch and rows must be positive");
  TGT_CHECK_ARG(rank >= 0 && rank < world, "rank outside the world");
  if (!(hidden == 64 && out_features == 64))
    return set_error(TGT_ERR_UNSUPPORTED, "the fused projection is built for hidden = projection width = 64");
  TGT_CHECK_ARG(out_features % world == 0 && (out_features / world) % 4 == 0,
                "the head slice of one rank must be a whole number of 16-byte units");
  TGT_CHECK_ARG(aligned16(x) && aligned16(wq) && aligned16(wk) && aligned16(wv), "tensors must be 16-byte aligned");
  QkvParams p;
  p.x = x; p.gamma = gamma; p.beta = beta; p.eps = eps;
  p.w[0] = wq; p.w[1] = wk; p.w[2] = wv;
  p.b[0] = bq; p.b[1] = bk; p.b[2] = bv;
  int rc = fill_slots(&p.slots, peer_slots, world);
  if (rc != TGT_OK) return rc;
  p.rows_total = batch * rows; p.rows = rows; p.world = world; p.rank = rank;
  p.tensor_bytes = batch * int64_t(world) * rows * (out_features / world) * 4;
  TGT_CHECK_ARG(size_t(3) * size_t(p.tensor_bytes) <= slot_bytes, "the slot is too small for q, k and v");
  const int64_t n_tiles = (p.rows_total + kTileRows - 1) / kTileRows;
  int grid = 1;
  const size_t smem = QkvSmem<64, 64>::floats * 4;
  rc = launch_grid(ln_qkv_push_kernel<64, 64>, smem, n_tiles, &grid);
  if (rc != TGT_OK) return rc;
  ln_qkv_push_kernel<64, 64><<<grid, kThreads, smem, stream>>>(p);
  TGT_CHECK_CUDA(cudaGetLastError());
  return TGT_OK;
}

extern "C" int tgt_pull_out_proj(void* const* peer_slots, size_t slot_bytes, const float* w, const float* b,
                                 int hidden, int in_features, float* ctx, float* y, int64_t batch,
                                 int64_t rows, int world, int rank, const int32_t* alias_rows, int n_alias,
                                 void* stream_) {
  using namespace tgt;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  TGT_CHECK_ARG(w && b && ctx && y, "w, b, ctx and y must not be null");
  TGT_CHECK_ARG(batch >= 1 && rows >= 1, "batch and rows must be positive");
  TGT_CHECK_ARG(rank >= 0 && rank < world, "rank outside the world");
  if (!(hidden == 64 && in_features == 64))
    return set_error(TGT_ERR_UNSUPPORTED, "the fused projection is built for hidden = projection width = 64");
  TGT_CHECK_ARG(in_features % world == 0 && (in_features / world) % 4 == 0,
                "the head slice of one rank must be a whole number of 16-byte units");
  TGT_CHECK_ARG(n_alias >= 0 && (n_alias == 0 || alias_rows != nullptr), "bad alias row arguments");
  TGT_CHECK_ARG(aligned16(w) && aligned16(ctx) && aligned16(y), "tensors must be 16-byte aligned");
  OutProjParams p;
  int rc = fill_slots(&p.slots, peer_slots, world);
  if (rc != TGT_OK) return rc;
  p.w = w; p.b = b; p.ctx = ctx; p.y = y; p.alias_rows = alias_rows; p.n_alias = n_alias;
  p.rows_total = batch * rows; p.rows = rows; p.world = world; p.rank = rank;
  TGT_CHECK_ARG(size_t(batch) * size_t(world) * size_t(rows) * size_t(in_features / world) * 4 <= slot_bytes,
                "the slot is smaller than the attention output said to live in it");
  const int64_t n_tiles = (p.rows_total + kTileRows - 1) / kTileRows;
  int grid = 1;
  const size_t smem = OutSmem<64, 64>::floats * 4;
  rc = launch_grid(pull_out_proj_kernel<64, 64>, smem, n_tiles, &grid);
  if (rc != TGT_OK) return rc;
  pull_out_proj_kernel<64, 64><<<grid, kThreads, smem, stream>>>(p);
  TGT_CHECK_CUDA(cudaGetLastError());
  return TGT_OK;
}
