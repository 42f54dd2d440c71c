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
static_assert(kTileRows == 4 * (kThreads / 32), "tile_gemm gives every warp four rows of the tile");

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

// out[r][c] = sum_k a[r][k] * w[c][k] for the thread's rows {4 warp .. 4 warp + 3} and columns {j * 32 + lane}.
// a: [kTileRows][K + 4], w: [COLS][K + 4] in shared memory.  Per step of four k a warp reads four row pieces
// (one address for all lanes: one shared-memory wavefront each) and NJ weight pieces (32 different rows whose
// pitch of K + 4 words puts every quarter warp on all 32 banks once: four wavefronts each) for 16 NJ FMAs per
// thread.  With two rows x 16 column groups per warp instead, both halves of the warp fetched the same weight
// pieces and the kernel spent twice the shared-memory wavefronts per FMA (LayerNorm + projections 90 us).
template <int K, int NJ>
__device__ __forceinline__ void tile_gemm(const float* __restrict__ a, const float* __restrict__ w, int warp, int lane,
                                          float (&acc)[4][NJ]) {
  constexpr int LD = K + 4;
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < NJ; ++j) acc[i][j] = 0.f;
#pragma unroll 2
  for (int k = 0; k < K; k += 4) {
    float4 av[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) av[i] = *reinterpret_cast<const float4*>(a + (4 * warp + i) * LD + k);
#pragma unroll
    for (int j = 0; j < NJ; ++j) {
      const float4 b = *reinterpret_cast<const float4*>(w + (j * 32 + lane) * LD + k);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        acc[i][j] = fmaf(av[i].x, b.x, acc[i][j]); acc[i][j] = fmaf(av[i].y, b.y, acc[i][j]);
        acc[i][j] = fmaf(av[i].z, b.z, acc[i][j]); acc[i][j] = fmaf(av[i].w, b.w, acc[i][j]);
      }
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
  constexpr int NJ = 3 * OUT / 32;                 // output columns per thread
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
  const int cols_per_peer = OUT / p.world;         // floats of one head slice
  const int units_per_row = cols_per_peer / 4;     // 16-byte units one peer gets from one row and tensor
  const int64_t n_tiles = (p.rows_total + kTileRows - 1) / kTileRows;
  // A thread owns two 16-byte pieces of the input tile: column piece k4 of rows r_a and r_a + 16; the 16
  // threads with the same r_a are half a warp and hold whole rows, so the LayerNorm is two shuffle sums.  The
  // pieces of the NEXT tile are fetched into registers before the arithmetic of this one.
  static_assert(HIDDEN == 64 && kTileRows == 32 && kThreads == 256, "the tile's pieces are dealt two per thread");
  const int r_a = tid / 16, k4 = tid % 16;
  float4 nx[2];
  auto fetch = [&](int64_t tile) {
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const int64_t row = tile * kTileRows + r_a + 16 * h;
      nx[h] = tile < n_tiles && row < p.rows_total ? __ldg(reinterpret_cast<const float4*>(p.x + row * HIDDEN) + k4)
                                                    : make_float4(0.f, 0.f, 0.f, 0.f);
    }
  };
  auto half_warp_sum = [](float v) {
#pragma unroll
    for (int off = 8; off > 0; off >>= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
    return v;
  };
  // Which pieces of the output tile this thread stores, and where to: the same for every tile (3 * 32 * 16
  // pieces of 16 bytes = 6 per thread), so the divisions are done once.
  constexpr int kStores = 3 * kTileRows * (OUT / 4) / kThreads;
  int st_row[kStores], st_from[kStores];       // row inside the tile; word offset inside s_o
  float4* st_base[kStores];                     // the peer's tensor, at this piece's position inside a row
  {
    const int units_per_run = kTileRows * units_per_row;
#pragma unroll
    for (int j = 0; j < kStores; ++j) {
      const int u = tid + j * kThreads;
      const int run = u / units_per_run, in_run = u % units_per_run;
      const int t = run / p.world;
      const int peer = (p.rank + 1 + run % p.world) % p.world;     // start with the next rank
      const int r = in_run / units_per_row, w = in_run % units_per_row;
      st_row[j] = r;
      st_from[j] = r * LDO + t * OUT + peer * cols_per_peer + 4 * w;
      st_base[j] = reinterpret_cast<float4*>(static_cast<char*>(p.slots.p[peer]) + t * p.tensor_bytes) + w;
    }
  }
  const unsigned rows_u = unsigned(p.rows);
  fetch(blockIdx.x);
  for (int64_t tile = blockIdx.x; tile < n_tiles; tile += gridDim.x) {
    const int64_t row0 = tile * kTileRows;
    const int n = int(min(int64_t(kTileRows), p.rows_total - row0));
    __syncthreads();               // the previous tile's arithmetic has read s_x, its stores s_o; weights are in place
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      float4 v = nx[h];
      if (p.gamma != nullptr) {
        // LayerNorm: biased variance, as torch.nn.LayerNorm
        const float mean = half_warp_sum((v.x + v.y) + (v.z + v.w)) * (1.0f / HIDDEN);
        v.x -= mean; v.y -= mean; v.z -= mean; v.w -= mean;
        const float var = half_warp_sum((v.x * v.x + v.y * v.y) + (v.z * v.z + v.w * v.w)) * (1.0f / HIDDEN);
        const float rstd = 1.0f / sqrtf(var + p.eps);
        const float4 g = *reinterpret_cast<const float4*>(s_g + 4 * k4);
        const float4 bt = *reinterpret_cast<const float4*>(s_g + HIDDEN + 4 * k4);
        v.x = v.x * rstd * g.x + bt.x; v.y = v.y * rstd * g.y + bt.y;
        v.z = v.z * rstd * g.z + bt.z; v.w = v.w * rstd * g.w + bt.w;
      }
      *reinterpret_cast<float4*>(s_x + (r_a + 16 * h) * LD + 4 * k4) = v;
    }
    __syncthreads();
    fetch(tile + gridDim.x);
    float acc[4][NJ];
    tile_gemm<HIDDEN, NJ>(s_x, s_w, warp, lane, acc);
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int j = 0; j < NJ; ++j) s_o[(4 * warp + i) * LDO + j * 32 + lane] = acc[i][j] + s_b[j * 32 + lane];
    __syncthreads();
    // Store the tile: for every tensor and peer the rows of the tile are one contiguous run on the peer
    // (gathered row = (batch entry * world + rank) * rows + l, row width = one head slice).
#pragma unroll
    for (int j = 0; j < kStores; ++j) {
      if (st_row[j] >= n) continue;
      const unsigned gi = unsigned(row0) + unsigned(st_row[j]);
      const unsigned bi = gi / rows_u, l = gi - bi * rows_u;
      const int64_t dest_row = (int64_t(bi) * p.world + p.rank) * p.rows + l;
      st_base[j][dest_row * units_per_row] = *reinterpret_cast<const float4*>(s_o + st_from[j]);
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
  constexpr int NJ = HIDDEN / 32;
  extern __shared__ __align__(16) float smem[];
  float* s_w = smem;                  // [HIDDEN][LD]
  float* s_b = s_w + HIDDEN * LD;     // [HIDDEN]
  float* s_c = s_b + HIDDEN;          // [kTileRows][LD] gathered tile
  const int tid = threadIdx.x;
  for (int i = tid; i < HIDDEN * OUT; i += kThreads) s_w[(i / OUT) * LD + i % OUT] = __ldg(p.w + i);
  for (int i = tid; i < HIDDEN; i += kThreads) s_b[i] = __ldg(p.b + i);
  const int warp = tid / 32, lane = tid % 32;
  const int cols_per_peer = OUT / p.world;
  const int units_per_row = cols_per_peer / 4;
  const int64_t n_tiles = (p.rows_total + kTileRows - 1) / kTileRows;
  // gather: for every peer the tile's rows are one contiguous run in the peer's slot; a thread owns two
  // 16-byte pieces of the tile and fetches those of the NEXT tile (over NVLink) before the arithmetic of this one
  static_assert(OUT == 64 && kTileRows == 32 && kThreads == 256, "the tile's pieces are dealt two per thread");
  const int units_per_run = kTileRows * units_per_row;
  int g_peer[2], g_row[2], g_unit[2];           // the same for every tile
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const int u = tid + h * kThreads;
    const int run = u / units_per_run, in_run = u % units_per_run;
    g_peer[h] = (p.rank + 1 + run) % p.world;
    g_row[h] = in_run / units_per_row;
    g_unit[h] = in_run % units_per_row;
  }
  const unsigned rows_u = unsigned(p.rows);
  float4 nv[2];
  auto fetch = [&](int64_t tile) {
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const int64_t gi64 = tile * kTileRows + g_row[h];
      nv[h] = make_float4(0.f, 0.f, 0.f, 0.f);
      if (tile < n_tiles && gi64 < p.rows_total) {
        const unsigned gi = unsigned(gi64);
        const unsigned bi = gi / rows_u, l = gi - bi * rows_u;
        int64_t src_row = int64_t(p.rank) * p.rows + l;
        for (int j = 0; j < p.n_alias; ++j)
          if (src_row == p.alias_rows[j]) {   // global-token slots take row 0's output
            src_row = 0;
            break;
          }
        nv[h] = *(reinterpret_cast<const float4*>(p.slots.p[g_peer[h]]) +
                  (int64_t(bi) * p.world * p.rows + src_row) * units_per_row + g_unit[h]);
      }
    }
  };
  fetch(blockIdx.x);
  for (int64_t tile = blockIdx.x; tile < n_tiles; tile += gridDim.x) {
    const int64_t row0 = tile * kTileRows;
    const int n = int(min(int64_t(kTileRows), p.rows_total - row0));
    __syncthreads();               // the previous tile's arithmetic has read s_c
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const int r = g_row[h], col = g_peer[h] * cols_per_peer + 4 * g_unit[h];
      if (r < n) *reinterpret_cast<float4*>(p.ctx + (row0 + r) * OUT + col) = nv[h];
      *reinterpret_cast<float4*>(s_c + r * LD + col) = nv[h];
    }
    __syncthreads();
    fetch(tile + gridDim.x);
    float acc[4][NJ];
    tile_gemm<OUT, NJ>(s_c, s_w, warp, lane, acc);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int r = 4 * warp + i;
      if (r < n) {
#pragma unroll
        for (int j = 0; j < NJ; ++j) p.y[(row0 + r) * HIDDEN + j * 32 + lane] = acc[i][j] + s_b[j * 32 + lane];
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
  TGT_CHECK_ARG(batch >= 1 && rows >= 1 && batch * rows < (int64_t(1) << 31), "batch and rows must be positive, batch * rows below 2^31");
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
  TGT_CHECK_ARG(batch >= 1 && rows >= 1 && batch * rows < (int64_t(1) << 31), "batch and rows must be positive, batch * rows below 2^31");
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
