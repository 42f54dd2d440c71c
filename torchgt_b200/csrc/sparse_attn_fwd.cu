// Forward of the topology-aware sparse graph attention: SDDMM -> clamp -> +bias -> exp ->
// running sums of w and w*V -> divide by (Z + 1e-6), fused in one pass over the edges grouped by
// destination.  No [E, H, D] tensor ever exists.
#include "attn_common.cuh"

namespace tgt {
namespace {

struct FwdParams {
  const void* q;
  const void* k;
  const void* v;
  const float* bias;  // original edge order, may be null
  int bias_heads;     // 0, 1 or heads
  void* out;
  float* z;           // [n_rows, heads]
  float* part_acc;    // chunk mode: [n_chunks, heads*head_dim]
  float* part_z;      // chunk mode: [n_chunks, heads]
  tgt_layout L;
  int heads;
  int row_elems;      // heads * head_dim
  float inv_scale;    // 1 / sqrt(head_dim)
  int chunk_mode;
  int lpr_log2;
};

template <typename T, int LPH, int G>
__global__ void __launch_bounds__(kBlockThreads) fwd_kernel(const FwdParams p) {
  constexpr int VEC = Vec16<T>::kElems;
  const Walk w = make_walk<G>(p.L, p.chunk_mode != 0, p.lpr_log2);
  const int col0 = (blockIdx.y * G + w.c) * VEC;           // first element of this lane in the row
  const int head = blockIdx.y * (G / LPH) + w.c / LPH;      // head this lane belongs to
  const T* __restrict__ K = static_cast<const T*>(p.k);
  const T* __restrict__ V = static_cast<const T*>(p.v);

  float q[VEC];
#pragma unroll
  for (int j = 0; j < VEC; ++j) q[j] = 0.f;
  if (w.row >= 0 && !w.is_hub)
    Vec16<T>::load(static_cast<const T*>(p.q) + int64_t(w.row) * p.row_elems + col0, q);

  float acc[VEC];
#pragma unroll
  for (int j = 0; j < VEC; ++j) acc[j] = 0.f;
  float zsum = 0.f;

  const int32_t* __restrict__ other = p.L.other;
  const int32_t* __restrict__ perm = p.L.perm;
  const int bias_stride = p.bias_heads;
  const int bias_off = p.bias_heads > 1 ? head : 0;

  int e = w.begin;
  for (int it = 0; it < w.iters; it += kUnroll) {
    int src[kUnroll];
    float b[kUnroll];
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      const int ee = e + u * w.nslots;
      src[u] = (ee < w.end) ? __ldg(other + ee) : -1;
    }
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      const int ee = e + u * w.nslots;
      b[u] = 0.f;
      if (p.bias != nullptr && src[u] >= 0)
        b[u] = __ldg(p.bias + int64_t(__ldg(perm + ee)) * bias_stride + bias_off);
    }
    float kk[kUnroll][VEC], vv[kUnroll][VEC];
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      if (src[u] >= 0) {
        const int64_t off = int64_t(src[u]) * p.row_elems + col0;
        Vec16<T>::load(K + off, kk[u]);
        Vec16<T>::load(V + off, vv[u]);
      } else {
#pragma unroll
        for (int j = 0; j < VEC; ++j) kk[u][j] = vv[u][j] = 0.f;
      }
    }
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      const float raw = group_sum<LPH>(dot<VEC>(q, kk[u])) * p.inv_scale;
      const float wgt = (src[u] >= 0) ? expf(clamp_score(raw) + b[u]) : 0.f;
      zsum += wgt;
#pragma unroll
      for (int j = 0; j < VEC; ++j) acc[j] = fmaf(wgt, vv[u][j], acc[j]);
    }
    e += kUnroll * w.nslots;
  }

  const int lpr = p.chunk_mode ? 32 : (1 << p.lpr_log2);
#pragma unroll
  for (int j = 0; j < VEC; ++j) acc[j] = slot_sum<G>(acc[j], lpr);
  zsum = slot_sum<G>(zsum, lpr);

  if (w.row < 0 || w.is_hub || w.slot != 0) return;
  if (p.chunk_mode) {
    float* dst = p.part_acc + int64_t(w.chunk) * p.row_elems + col0;
#pragma unroll
    for (int j = 0; j < VEC; j += 4)
      *reinterpret_cast<float4*>(dst + j) = make_float4(acc[j], acc[j + 1], acc[j + 2], acc[j + 3]);
    if (w.c % LPH == 0) p.part_z[int64_t(w.chunk) * p.heads + head] = zsum;
  } else {
    const float inv = 1.0f / (zsum + kZEps);
    float o[VEC];
#pragma unroll
    for (int j = 0; j < VEC; ++j) o[j] = acc[j] * inv;
    Vec16<T>::store(static_cast<T*>(p.out) + int64_t(w.row) * p.row_elems + col0, o);
    if (w.c % LPH == 0) p.z[int64_t(w.row) * p.heads + head] = zsum;
  }
}

// Sum the chunk partials of every hub row in chunk order and finish the row.
// One warp per (hub row, 128-value column tile): lane l owns columns l*4 .. l*4+3 of the tile.
template <typename T>
__global__ void __launch_bounds__(kBlockThreads)
fwd_hub_reduce_kernel(const FwdParams p, int head_dim) {
  const int hub = blockIdx.x * kWarpsPerBlock + (threadIdx.x >> 5);
  if (hub >= p.L.n_hubs) return;
  const int lane = threadIdx.x & 31;
  const int col = (blockIdx.y * 32 + lane) * 4;
  if (col >= p.row_elems) return;
  const int row = __ldg(p.L.hub_row + hub);
  const int c0 = __ldg(p.L.hub_chunk_ptr + hub), c1 = __ldg(p.L.hub_chunk_ptr + hub + 1);
  const int head = col / head_dim;
  float4 a = make_float4(0.f, 0.f, 0.f, 0.f);
  float zsum = 0.f;
  for (int c = c0; c < c1; ++c) {
    const float4 t = *reinterpret_cast<const float4*>(p.part_acc + int64_t(c) * p.row_elems + col);
    a.x += t.x; a.y += t.y; a.z += t.z; a.w += t.w;
    zsum += p.part_z[int64_t(c) * p.heads + head];
  }
  const float inv = 1.0f / (zsum + kZEps);
  T* o = static_cast<T*>(p.out) + int64_t(row) * p.row_elems + col;
  if constexpr (sizeof(T) == 4) {
    *reinterpret_cast<float4*>(o) = make_float4(a.x * inv, a.y * inv, a.z * inv, a.w * inv);
  } else {
    const __nv_bfloat162 lo = __floats2bfloat162_rn(a.x * inv, a.y * inv);
    const __nv_bfloat162 hi = __floats2bfloat162_rn(a.z * inv, a.w * inv);
    uint2 pk;
    pk.x = *reinterpret_cast<const uint32_t*>(&lo);
    pk.y = *reinterpret_cast<const uint32_t*>(&hi);
    *reinterpret_cast<uint2*>(o) = pk;
  }
  if (col % head_dim == 0) p.z[int64_t(row) * p.heads + head] = zsum;
}

}  // namespace

size_t fwd_scratch_bytes(const tgt_layout* L, int heads, int head_dim) {
  const size_t acc = round_up(size_t(L->n_chunks) * heads * head_dim * 4, 256);
  const size_t z = round_up(size_t(L->n_chunks) * heads * 4, 256);
  return acc + z;
}

}  // namespace tgt

extern "C" int tgt_sparse_attn_fwd(const void* q, const void* k, const void* v, const float* bias,
                                   int bias_heads, const tgt_layout* by_dst, void* out, float* z,
                                   int heads, int head_dim, int dtype, void* scratch,
                                   size_t scratch_bytes, void* stream_) {
  using namespace tgt;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  TGT_CHECK_ARG(dtype == TGT_F32 || dtype == TGT_BF16, "dtype must be TGT_F32 or TGT_BF16");
  int rc = check_layout(by_dst, "by_dst");
  if (rc != TGT_OK) return rc;
  HeadSplit hs;
  if (!split_heads(heads, head_dim, dtype, &hs))
    return set_error(TGT_ERR_UNSUPPORTED,
                     "heads=%d head_dim=%d dtype=%d: head_dim must be a power of two multiple of "
                     "16 bytes, at most 512 bytes per head",
                     heads, head_dim, dtype);
  TGT_CHECK_ARG(bias_heads == 0 || bias_heads == 1 || bias_heads == heads,
                "bias_heads must be 0, 1 or heads");
  TGT_CHECK_ARG((bias_heads == 0) == (bias == nullptr), "bias pointer and bias_heads disagree");
  const tgt_layout& L = *by_dst;
  if (L.n_rows == 0) return TGT_OK;
  TGT_CHECK_ARG(q && k && v && out && z, "q/k/v/out/z must not be null");
  TGT_CHECK_ARG(aligned16(q) && aligned16(k) && aligned16(v) && aligned16(out) && aligned16(z) &&
                    aligned16(bias) && aligned16(scratch),
                "device pointers must be 16-byte aligned");
  const size_t need = L.n_chunks > 0 ? fwd_scratch_bytes(&L, heads, head_dim) : 0;
  if (need > 0 && (scratch == nullptr || scratch_bytes < need))
    return set_error(TGT_ERR_WORKSPACE, "scratch holds %zu bytes, %zu needed", scratch_bytes, need);

  FwdParams p;
  p.q = q; p.k = k; p.v = v; p.bias = bias; p.bias_heads = bias_heads;
  p.out = out; p.z = z;
  p.part_acc = static_cast<float*>(scratch);
  p.part_z = need > 0 ? reinterpret_cast<float*>(
                            static_cast<char*>(scratch) +
                            round_up(size_t(L.n_chunks) * heads * head_dim * 4, 256))
                      : nullptr;
  p.L = L;
  p.heads = heads;
  p.row_elems = heads * head_dim;
  p.inv_scale = 1.0f / sqrtf(float(head_dim));
  const double avg_deg = double(L.n_edges) / double(L.n_rows);
  p.lpr_log2 = choose_lpr_log2(hs.g, avg_deg);

#define TGT_LAUNCH_FWD(T, LPH, G)                                                      \
  fwd_kernel<T, LPH, G><<<grid, kBlockThreads, 0, stream>>>(p)

  if (L.n_chunks > 0) {
    p.chunk_mode = 1;
    dim3 grid((L.n_chunks + kWarpsPerBlock - 1) / kWarpsPerBlock, hs.groups);
    TGT_DISPATCH(dtype, hs.lph, hs.g, TGT_LAUNCH_FWD);
  }
  {
    p.chunk_mode = 0;
    const int64_t rows_per_block = int64_t(kWarpsPerBlock) * (32 >> p.lpr_log2);
    dim3 grid(unsigned((L.n_rows + rows_per_block - 1) / rows_per_block), hs.groups);
    TGT_DISPATCH(dtype, hs.lph, hs.g, TGT_LAUNCH_FWD);
  }
  if (L.n_hubs > 0) {
    dim3 grid((L.n_hubs + kWarpsPerBlock - 1) / kWarpsPerBlock, (p.row_elems + 127) / 128);
    if (dtype == TGT_F32)
      fwd_hub_reduce_kernel<float><<<grid, kBlockThreads, 0, stream>>>(p, head_dim);
    else
      fwd_hub_reduce_kernel<__nv_bfloat16><<<grid, kBlockThreads, 0, stream>>>(p, head_dim);
  }
#undef TGT_LAUNCH_FWD
  TGT_CHECK_CUDA(cudaGetLastError());
  return TGT_OK;
}
