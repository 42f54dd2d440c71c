// LayerNorm over short rows (the hidden size of the graph transformers: 64 values), forward and backward,
// fp32.  It is the operation on both sides of the attention block (models/graphormer_dist_node_level.py:
// 293-311: self_attention_norm before the projections, ffn_norm after the residual; final_ln :395) and the
// backward half of the fused LayerNorm + projection kernel.  With rows this short a row is a few lanes of
// one warp: LPR lanes hold a row as 16-byte pieces, 32 / LPR rows per warp, everything in registers, one
// read of the input and one write of the result (forward), two reads and one write (backward).  The
// parameter gradients are summed per thread over the rows it walks, then per CTA in shared memory, then
// over the CTAs by a second small kernel in a fixed order: no atomics, bitwise reproducible.
#include <type_traits>

#include "tgt_common.cuh"

namespace tgt {
namespace {

constexpr int kLnThreads = 256;
constexpr int kLnMaxPieces = 4;   // 16-byte pieces per lane: rows of up to 32 * 4 * 4 = 512 values

template <int LPR>
__device__ __forceinline__ float row_sum(float x) {
#pragma unroll
  for (int o = LPR / 2; o > 0; o >>= 1) x += __shfl_xor_sync(0xffffffffu, x, o);
  return x;
}

struct LnFwdParams {
  const float* x;
  const float* gamma;
  const float* beta;
  float* y;
  float2* stats;   // [rows] mean, 1 / sqrt(var + eps); may be null
  int64_t rows;
  int hidden;
  float eps;
};

template <int LPR, int PIECES>
__global__ void __launch_bounds__(kLnThreads) layer_norm_fwd_kernel(const LnFwdParams p) {
  constexpr int RPW = 32 / LPR;
  const int lane = threadIdx.x % 32;
  const int sub = lane / LPR, l = lane % LPR;
  const int pieces = p.hidden / 4;
  const int64_t warp = (int64_t(blockIdx.x) * kLnThreads + threadIdx.x) / 32;
  const int64_t n_warps = int64_t(gridDim.x) * (kLnThreads / 32);
  float4 ga[PIECES], be[PIECES];
#pragma unroll
  for (int j = 0; j < PIECES; ++j) {
    const int c = l + j * LPR;
    ga[j] = c < pieces ? __ldg(reinterpret_cast<const float4*>(p.gamma) + c) : make_float4(0.f, 0.f, 0.f, 0.f);
    be[j] = c < pieces ? __ldg(reinterpret_cast<const float4*>(p.beta) + c) : make_float4(0.f, 0.f, 0.f, 0.f);
  }
  const float inv_h = 1.0f / float(p.hidden);
  for (int64_t r0 = warp * RPW; r0 < p.rows; r0 += n_warps * RPW) {   // all lanes of a warp loop together
    const int64_t row = r0 + sub;
    const bool live = row < p.rows;
    float4 v[PIECES];
    float s = 0.f;
#pragma unroll
    for (int j = 0; j < PIECES; ++j) {
      const int c = l + j * LPR;
      v[j] = live && c < pieces ? __ldg(reinterpret_cast<const float4*>(p.x + row * p.hidden) + c)
                                : make_float4(0.f, 0.f, 0.f, 0.f);
      s += (v[j].x + v[j].y) + (v[j].z + v[j].w);
    }
    const float mean = row_sum<LPR>(s) * inv_h;
    float q = 0.f;
#pragma unroll
    for (int j = 0; j < PIECES; ++j) {
      const int c = l + j * LPR;
      if (c < pieces) {
        const float a = v[j].x - mean, b = v[j].y - mean, cc = v[j].z - mean, d = v[j].w - mean;
        q += (a * a + b * b) + (cc * cc + d * d);
      }
    }
    const float rstd = rsqrtf(row_sum<LPR>(q) * inv_h + p.eps);
    if (live) {
#pragma unroll
      for (int j = 0; j < PIECES; ++j) {
        const int c = l + j * LPR;
        if (c < pieces) {
          float4 o;
          o.x = (v[j].x - mean) * rstd * ga[j].x + be[j].x;
          o.y = (v[j].y - mean) * rstd * ga[j].y + be[j].y;
          o.z = (v[j].z - mean) * rstd * ga[j].z + be[j].z;
          o.w = (v[j].w - mean) * rstd * ga[j].w + be[j].w;
          reinterpret_cast<float4*>(p.y + row * p.hidden)[c] = o;
        }
      }
      if (l == 0 && p.stats != nullptr) p.stats[row] = make_float2(mean, rstd);
    }
  }
}

struct LnBwdParams {
  const float* dy;
  const float* x;
  const float* gamma;
  const float2* stats;
  float* dx;
  float* partial;   // [gridDim.x][2][hidden]: this CTA's sums for dgamma, then for dbeta
  int64_t rows;
  int hidden;
};

template <int LPR, int PIECES>
__global__ void __launch_bounds__(kLnThreads) layer_norm_bwd_kernel(const LnBwdParams p) {
  constexpr int RPW = 32 / LPR;
  constexpr int GROUPS = kLnThreads / LPR;       // row slots per CTA
  __shared__ float4 s_sum[GROUPS][LPR];          // one piece of every group, reduced piece by piece
  const int lane = threadIdx.x % 32;
  const int sub = lane / LPR, l = lane % LPR;
  const int group = threadIdx.x / LPR;
  const int pieces = p.hidden / 4;
  const int64_t warp = (int64_t(blockIdx.x) * kLnThreads + threadIdx.x) / 32;
  const int64_t n_warps = int64_t(gridDim.x) * (kLnThreads / 32);
  float4 ga[PIECES], dg[PIECES], db[PIECES];
#pragma unroll
  for (int j = 0; j < PIECES; ++j) {
    const int c = l + j * LPR;
    ga[j] = c < pieces ? __ldg(reinterpret_cast<const float4*>(p.gamma) + c) : make_float4(0.f, 0.f, 0.f, 0.f);
    dg[j] = db[j] = make_float4(0.f, 0.f, 0.f, 0.f);
  }
  const float inv_h = 1.0f / float(p.hidden);
  for (int64_t r0 = warp * RPW; r0 < p.rows; r0 += n_warps * RPW) {
    const int64_t row = r0 + sub;
    const bool live = row < p.rows;
    const float2 st = live ? __ldg(p.stats + row) : make_float2(0.f, 0.f);
    float4 xh[PIECES], g[PIECES];
    float s1 = 0.f, s2 = 0.f;
#pragma unroll
    for (int j = 0; j < PIECES; ++j) {
      const int c = l + j * LPR;
      const bool on = live && c < pieces;
      const float4 xv = on ? __ldg(reinterpret_cast<const float4*>(p.x + row * p.hidden) + c)
                           : make_float4(st.x, st.x, st.x, st.x);
      const float4 d = on ? __ldg(reinterpret_cast<const float4*>(p.dy + row * p.hidden) + c)
                          : make_float4(0.f, 0.f, 0.f, 0.f);
      xh[j] = make_float4((xv.x - st.x) * st.y, (xv.y - st.x) * st.y, (xv.z - st.x) * st.y, (xv.w - st.x) * st.y);
      g[j] = make_float4(d.x * ga[j].x, d.y * ga[j].y, d.z * ga[j].z, d.w * ga[j].w);
      s1 += (g[j].x + g[j].y) + (g[j].z + g[j].w);
      s2 += (g[j].x * xh[j].x + g[j].y * xh[j].y) + (g[j].z * xh[j].z + g[j].w * xh[j].w);
      dg[j].x = fmaf(d.x, xh[j].x, dg[j].x); dg[j].y = fmaf(d.y, xh[j].y, dg[j].y);
      dg[j].z = fmaf(d.z, xh[j].z, dg[j].z); dg[j].w = fmaf(d.w, xh[j].w, dg[j].w);
      db[j].x += d.x; db[j].y += d.y; db[j].z += d.z; db[j].w += d.w;
    }
    const float c1 = row_sum<LPR>(s1) * inv_h;
    const float c2 = row_sum<LPR>(s2) * inv_h;
    if (live) {
#pragma unroll
      for (int j = 0; j < PIECES; ++j) {
        const int c = l + j * LPR;
        if (c < pieces) {
          float4 o;
          o.x = st.y * (g[j].x - c1 - xh[j].x * c2);
          o.y = st.y * (g[j].y - c1 - xh[j].y * c2);
          o.z = st.y * (g[j].z - c1 - xh[j].z * c2);
          o.w = st.y * (g[j].w - c1 - xh[j].w * c2);
          reinterpret_cast<float4*>(p.dx + row * p.hidden)[c] = o;
        }
      }
    }
  }
  // sums over this CTA's row slots, in slot order
  float* out = p.partial + int64_t(blockIdx.x) * 2 * p.hidden;
#pragma unroll
  for (int which = 0; which < 2; ++which) {
#pragma unroll
    for (int j = 0; j < PIECES; ++j) {
      __syncthreads();
      s_sum[group][l] = which == 0 ? dg[j] : db[j];
      __syncthreads();
      const int c = l + j * LPR;
      if (group == 0 && c < pieces) {
        float4 t = s_sum[0][l];
        for (int gq = 1; gq < GROUPS; ++gq) {
          const float4 u = s_sum[gq][l];
          t.x += u.x; t.y += u.y; t.z += u.z; t.w += u.w;
        }
        reinterpret_cast<float4*>(out + which * p.hidden)[c] = t;
      }
    }
  }
}

// dgamma[j] = sum over CTAs of partial[cta][0][j], dbeta likewise (sum_partials: fixed association).
__global__ void __launch_bounds__(kPartialSumThreads) layer_norm_param_grad_kernel(const float* __restrict__ partial,
                                                                                   int ctas, int hidden,
                                                                                   float* __restrict__ dgamma,
                                                                                   float* __restrict__ dbeta) {
  __shared__ float s_part[16][32];
  const int i = blockIdx.x * 32 + threadIdx.x % 32;
  const bool live = i < 2 * hidden;
  const float s = sum_partials(partial, ctas, int64_t(2) * hidden, i, live, s_part);
  if (threadIdx.x < 32 && live) {
    if (i < hidden) dgamma[i] = s;
    else dbeta[i - hidden] = s;
  }
}

// lanes per row (power of two, at most 32) and pieces per lane for a hidden size
bool ln_shape(int hidden, int* lpr, int* pieces) {
  if (hidden < 4 || hidden % 4 != 0 || hidden > 32 * kLnMaxPieces * 4) return false;
  const int n = hidden / 4;
  int l = 1;
  while (l < n && l < 32) l *= 2;
  *lpr = l;
  *pieces = (n + l - 1) / l;
  return true;
}

int ln_grid(int64_t rows, int lpr) {
  const int64_t rows_per_cta = int64_t(kLnThreads / 32) * (32 / lpr);
  const int64_t want = (rows + rows_per_cta - 1) / rows_per_cta;
  const int64_t cap = int64_t(sm_count()) * 4;
  return int(want < cap ? (want < 1 ? 1 : want) : cap);
}

template <class F>
bool ln_dispatch(int lpr, int pieces, F&& f) {
#define TGT_LN_CASE(L, P) \
  if (lpr == L && pieces == P) { f(std::integral_constant<int, L>{}, std::integral_constant<int, P>{}); return true; }
  TGT_LN_CASE(1, 1) TGT_LN_CASE(2, 1) TGT_LN_CASE(4, 1) TGT_LN_CASE(8, 1) TGT_LN_CASE(16, 1)
  TGT_LN_CASE(32, 1) TGT_LN_CASE(32, 2) TGT_LN_CASE(32, 3) TGT_LN_CASE(32, 4)
#undef TGT_LN_CASE
  return false;
}

}  // namespace
}  // namespace tgt

extern "C" int tgt_layer_norm_fwd(const float* x, const float* gamma, const float* beta, float eps,
                                  int64_t rows, int hidden, float* y, float* stats, void* stream_) {
  using namespace tgt;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  int lpr = 0, pieces = 0;
  if (!ln_shape(hidden, &lpr, &pieces))
    return set_error(TGT_ERR_UNSUPPORTED, "hidden=%d: the row must be a multiple of 4 values, at most %d",
                     hidden, 32 * kLnMaxPieces * 4);
  TGT_CHECK_ARG(rows >= 0, "rows must be >= 0");
  if (rows == 0) return TGT_OK;
  TGT_CHECK_ARG(x && gamma && beta && y, "x, gamma, beta and y must not be null");
  TGT_CHECK_ARG(aligned16(x) && aligned16(gamma) && aligned16(beta) && aligned16(y) &&
                    (reinterpret_cast<uintptr_t>(stats) & 7u) == 0,
                "tensors must be 16-byte aligned (stats 8-byte)");
  LnFwdParams p{x, gamma, beta, y, reinterpret_cast<float2*>(stats), rows, hidden, eps};
  const int grid = ln_grid(rows, lpr);
  const bool built = ln_dispatch(lpr, pieces, [&](auto L, auto P) {
    layer_norm_fwd_kernel<decltype(L)::value, decltype(P)::value><<<grid, kLnThreads, 0, stream>>>(p);
  });
  if (!built) return set_error(TGT_ERR_UNSUPPORTED, "no LayerNorm kernel for hidden=%d", hidden);
  TGT_CHECK_CUDA(cudaGetLastError());
  return TGT_OK;
}

extern "C" int tgt_layer_norm_bwd_scratch_bytes(int64_t rows, int hidden, size_t* bytes) {
  using namespace tgt;
  TGT_CHECK_ARG(bytes != nullptr, "bytes is null");
  int lpr = 0, pieces = 0;
  if (!ln_shape(hidden, &lpr, &pieces))
    return set_error(TGT_ERR_UNSUPPORTED, "hidden=%d: the row must be a multiple of 4 values, at most %d",
                     hidden, 32 * kLnMaxPieces * 4);
  TGT_CHECK_ARG(rows >= 0, "rows must be >= 0");
  *bytes = size_t(ln_grid(rows < 1 ? 1 : rows, lpr)) * 2 * size_t(hidden) * sizeof(float);
  return TGT_OK;
}

extern "C" int tgt_layer_norm_bwd(const float* dy, const float* x, const float* gamma, const float* stats,
                                  int64_t rows, int hidden, float* dx, float* dgamma, float* dbeta,
                                  void* scratch, size_t scratch_bytes, void* stream_) {
  using namespace tgt;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  int lpr = 0, pieces = 0;
  if (!ln_shape(hidden, &lpr, &pieces))
    return set_error(TGT_ERR_UNSUPPORTED, "hidden=%d: the row must be a multiple of 4 values, at most %d",
                     hidden, 32 * kLnMaxPieces * 4);
  TGT_CHECK_ARG(rows >= 0, "rows must be >= 0");
  TGT_CHECK_ARG(dgamma && dbeta, "dgamma and dbeta must not be null");
  if (rows == 0) {
    TGT_CHECK_CUDA(cudaMemsetAsync(dgamma, 0, size_t(hidden) * sizeof(float), stream));
    TGT_CHECK_CUDA(cudaMemsetAsync(dbeta, 0, size_t(hidden) * sizeof(float), stream));
    return TGT_OK;
  }
  TGT_CHECK_ARG(dy && x && gamma && stats && dx, "dy, x, gamma, stats and dx must not be null");
  TGT_CHECK_ARG(aligned16(dy) && aligned16(x) && aligned16(gamma) && aligned16(dx) && aligned16(scratch) &&
                    (reinterpret_cast<uintptr_t>(stats) & 7u) == 0,
                "tensors must be 16-byte aligned (stats 8-byte)");
  const int grid = ln_grid(rows, lpr);
  const size_t need = size_t(grid) * 2 * size_t(hidden) * sizeof(float);
  if (scratch == nullptr || scratch_bytes < need)
    return set_error(TGT_ERR_WORKSPACE, "scratch holds %zu bytes, %zu needed", scratch_bytes, need);
  LnBwdParams p{dy, x, gamma, reinterpret_cast<const float2*>(stats), dx, static_cast<float*>(scratch), rows, hidden};
  const bool built = ln_dispatch(lpr, pieces, [&](auto L, auto P) {
    layer_norm_bwd_kernel<decltype(L)::value, decltype(P)::value><<<grid, kLnThreads, 0, stream>>>(p);
  });
  if (!built) return set_error(TGT_ERR_UNSUPPORTED, "no LayerNorm kernel for hidden=%d", hidden);
  layer_norm_param_grad_kernel<<<(2 * hidden + 31) / 32, kPartialSumThreads, 0, stream>>>(p.partial, grid, hidden, dgamma, dbeta);
  TGT_CHECK_CUDA(cudaGetLastError());
  return TGT_OK;
}
