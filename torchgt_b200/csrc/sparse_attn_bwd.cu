// Backward of the sparse graph attention in two atomics-free passes that recompute the scores:
//   pass A walks edges grouped by destination: dQ, dbias and the per-row statistics
//          stats[d,h] = { 1/(Z+1e-6), dO_d . O_d };
//   pass B walks edges grouped by source: dK and dV (reads the statistics of each destination).
// With G = dO, inv = 1/(Z+1e-6), w = exp(clamp(raw)+bias):
//   dw = (G_d.V_s - G_d.O_d) * inv_d      dV_s += w * inv_d * G_d      dt = dw * w  (= dbias)
//   da = dt * [-5 <= raw <= 5]            dQ_d += da * K_s / sqrt(D)   dK_s += da * Q_d / sqrt(D)
#include "attn_common.cuh"

namespace tgt {
namespace {

struct BwdParams {
  const void* dout;
  const void* q;
  const void* k;
  const void* v;
  const void* out;
  const float* z;
  const float* bias;
  int bias_heads;
  void* dq;
  void* dk;
  void* dv;
  float* dbias;
  float2* stats;  // [n_rows, heads]
  float* part;    // chunk partials of the running pass
  tgt_layout L;   // by_dst in pass A, by_src in pass B
  int heads;
  int row_elems;
  float inv_scale;
  int chunk_mode;
  int lpr_log2;
};

template <int VEC>
__device__ __forceinline__ void zero(float (&a)[VEC]) {
#pragma unroll
  for (int j = 0; j < VEC; ++j) a[j] = 0.f;
}

template <int VEC>
__device__ __forceinline__ void store_partial(float* dst, const float (&a)[VEC]) {
#pragma unroll
  for (int j = 0; j < VEC; j += 4)
    *reinterpret_cast<float4*>(dst + j) = make_float4(a[j], a[j + 1], a[j + 2], a[j + 3]);
}

// ---- pass A: dQ, dbias, row statistics -----------------------------------------------------
template <typename T, int LPH, int G>
__global__ void __launch_bounds__(kBlockThreads) bwd_dq_kernel(const BwdParams p) {
  constexpr int VEC = Vec16<T>::kElems;
  const Walk w = make_walk<G>(p.L, p.chunk_mode != 0, p.lpr_log2);
  const int col0 = (blockIdx.y * G + w.c) * VEC;
  const int head = blockIdx.y * (G / LPH) + w.c / LPH;
  const T* __restrict__ K = static_cast<const T*>(p.k);
  const T* __restrict__ V = static_cast<const T*>(p.v);

  float q[VEC], g[VEC], o[VEC];
  zero<VEC>(q); zero<VEC>(g); zero<VEC>(o);
  float zrow = 0.f;
  if (w.row >= 0) {
    const int64_t off = int64_t(w.row) * p.row_elems + col0;
    Vec16<T>::load(static_cast<const T*>(p.q) + off, q);
    Vec16<T>::load(static_cast<const T*>(p.dout) + off, g);
    Vec16<T>::load(static_cast<const T*>(p.out) + off, o);
    zrow = __ldg(p.z + int64_t(w.row) * p.heads + head);
  }
  const float inv = 1.0f / (zrow + kZEps);
  const float delta = group_sum<LPH>(dot<VEC>(g, o));
  if (!p.chunk_mode && w.row >= 0 && w.slot == 0 && w.c % LPH == 0)
    p.stats[int64_t(w.row) * p.heads + head] = make_float2(inv, delta);

  float dq[VEC];
  zero<VEC>(dq);
  const int32_t* __restrict__ other = p.L.other;
  const int32_t* __restrict__ perm = p.L.perm;
  const bool need_perm = p.bias != nullptr || p.dbias != nullptr;
  const int bias_stride = p.bias_heads;
  const int bias_off = p.bias_heads > 1 ? head : 0;

  int e = w.begin;
  for (int it = 0; it < w.iters; it += kUnroll) {
    int src[kUnroll], pe[kUnroll];
    float b[kUnroll];
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      const int ee = e + u * w.nslots;
      src[u] = (ee < w.end) ? __ldg(other + ee) : -1;
      pe[u] = (need_perm && ee < w.end) ? __ldg(perm + ee) : 0;
    }
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      b[u] = 0.f;
      if (p.bias != nullptr && src[u] >= 0)
        b[u] = __ldg(p.bias + int64_t(pe[u]) * bias_stride + bias_off);
    }
    float kk[kUnroll][VEC], vv[kUnroll][VEC];
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      if (src[u] >= 0) {
        const int64_t off = int64_t(src[u]) * p.row_elems + col0;
        Vec16<T>::load(K + off, kk[u]);
        Vec16<T>::load(V + off, vv[u]);
      } else {
        zero<VEC>(kk[u]);
        zero<VEC>(vv[u]);
      }
    }
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      const float raw = group_sum<LPH>(dot<VEC>(q, kk[u])) * p.inv_scale;
      const float gv = group_sum<LPH>(dot<VEC>(g, vv[u]));
      const float wgt = expf(clamp_score(raw) + b[u]);
      float dt = (gv - delta) * inv * wgt;
      if (src[u] < 0) dt = 0.f;
      const float da = clamp_passes_grad(raw) ? dt : 0.f;
#pragma unroll
      for (int j = 0; j < VEC; ++j) dq[j] = fmaf(da, kk[u][j], dq[j]);
      if (p.dbias != nullptr) {
        if (p.bias_heads == 1) {
          // every head's dt sits on LPH lanes; the group sum counts it LPH times
          const float s = group_sum<G>(dt) * (1.0f / LPH);
          if (src[u] >= 0 && w.c == 0) p.dbias[pe[u]] = s;
        } else if (src[u] >= 0 && w.c % LPH == 0) {
          p.dbias[int64_t(pe[u]) * bias_stride + head] = dt;
        }
      }
    }
    e += kUnroll * w.nslots;
  }

  const int lpr = p.chunk_mode ? 32 : (1 << p.lpr_log2);
#pragma unroll
  for (int j = 0; j < VEC; ++j) dq[j] = slot_sum<G>(dq[j], lpr);
  if (w.row < 0 || w.is_hub || w.slot != 0) return;
  if (p.chunk_mode) {
    store_partial<VEC>(p.part + int64_t(w.chunk) * p.row_elems + col0, dq);
  } else {
#pragma unroll
    for (int j = 0; j < VEC; ++j) dq[j] *= p.inv_scale;
    Vec16<T>::store(static_cast<T*>(p.dq) + int64_t(w.row) * p.row_elems + col0, dq);
  }
}

// ---- pass B: dK, dV --------------------------------------------------------------------------
template <typename T, int LPH, int G>
__global__ void __launch_bounds__(kBlockThreads) bwd_dkv_kernel(const BwdParams p) {
  constexpr int VEC = Vec16<T>::kElems;
  const Walk w = make_walk<G>(p.L, p.chunk_mode != 0, p.lpr_log2);
  const int col0 = (blockIdx.y * G + w.c) * VEC;
  const int head = blockIdx.y * (G / LPH) + w.c / LPH;
  const T* __restrict__ Q = static_cast<const T*>(p.q);
  const T* __restrict__ DO = static_cast<const T*>(p.dout);

  float k[VEC], v[VEC];
  zero<VEC>(k); zero<VEC>(v);
  if (w.row >= 0 && !w.is_hub) {
    const int64_t off = int64_t(w.row) * p.row_elems + col0;
    Vec16<T>::load(static_cast<const T*>(p.k) + off, k);
    Vec16<T>::load(static_cast<const T*>(p.v) + off, v);
  }

  float dk[VEC], dv[VEC];
  zero<VEC>(dk); zero<VEC>(dv);
  const int32_t* __restrict__ other = p.L.other;
  const int32_t* __restrict__ perm = p.L.perm;
  const int bias_stride = p.bias_heads;
  const int bias_off = p.bias_heads > 1 ? head : 0;

  int e = w.begin;
  for (int it = 0; it < w.iters; it += kUnroll) {
    int dst[kUnroll];
    float b[kUnroll];
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      const int ee = e + u * w.nslots;
      dst[u] = (ee < w.end) ? __ldg(other + ee) : -1;
    }
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      const int ee = e + u * w.nslots;
      b[u] = 0.f;
      if (p.bias != nullptr && dst[u] >= 0)
        b[u] = __ldg(p.bias + int64_t(__ldg(perm + ee)) * bias_stride + bias_off);
    }
    float qq[kUnroll][VEC], gg[kUnroll][VEC];
    float2 st[kUnroll];
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      if (dst[u] >= 0) {
        const int64_t off = int64_t(dst[u]) * p.row_elems + col0;
        Vec16<T>::load(Q + off, qq[u]);
        Vec16<T>::load(DO + off, gg[u]);
        st[u] = __ldg(p.stats + int64_t(dst[u]) * p.heads + head);
      } else {
        zero<VEC>(qq[u]);
        zero<VEC>(gg[u]);
        st[u] = make_float2(0.f, 0.f);
      }
    }
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      const float raw = group_sum<LPH>(dot<VEC>(qq[u], k)) * p.inv_scale;
      const float gv = group_sum<LPH>(dot<VEC>(gg[u], v));
      float wgt = expf(clamp_score(raw) + b[u]);
      if (dst[u] < 0) wgt = 0.f;
      const float dt = (gv - st[u].y) * st[u].x * wgt;
      const float da = clamp_passes_grad(raw) ? dt : 0.f;
      const float wi = wgt * st[u].x;
#pragma unroll
      for (int j = 0; j < VEC; ++j) {
        dv[j] = fmaf(wi, gg[u][j], dv[j]);
        dk[j] = fmaf(da, qq[u][j], dk[j]);
      }
    }
    e += kUnroll * w.nslots;
  }

  const int lpr = p.chunk_mode ? 32 : (1 << p.lpr_log2);
#pragma unroll
  for (int j = 0; j < VEC; ++j) {
    dk[j] = slot_sum<G>(dk[j], lpr);
    dv[j] = slot_sum<G>(dv[j], lpr);
  }
  if (w.row < 0 || w.is_hub || w.slot != 0) return;
  if (p.chunk_mode) {
    float* base = p.part + int64_t(w.chunk) * 2 * p.row_elems + col0;
    store_partial<VEC>(base, dk);
    store_partial<VEC>(base + p.row_elems, dv);
  } else {
#pragma unroll
    for (int j = 0; j < VEC; ++j) dk[j] *= p.inv_scale;
    const int64_t off = int64_t(w.row) * p.row_elems + col0;
    Vec16<T>::store(static_cast<T*>(p.dk) + off, dk);
    Vec16<T>::store(static_cast<T*>(p.dv) + off, dv);
  }
}

// Sum chunk partials of each hub row in chunk order; n_out tensors are interleaved per chunk.
template <typename T>
__global__ void __launch_bounds__(kBlockThreads)
bwd_hub_reduce_kernel(const tgt_layout L, const float* __restrict__ part, int n_out, void* out0,
                      void* out1, float scale0, float scale1, int row_elems) {
  const int hub = blockIdx.x * kWarpsPerBlock + (threadIdx.x >> 5);
  if (hub >= L.n_hubs) return;
  const int lane = threadIdx.x & 31;
  const int col = (blockIdx.y * 32 + lane) * 4;
  if (col >= row_elems) return;
  const int row = __ldg(L.hub_row + hub);
  const int c0 = __ldg(L.hub_chunk_ptr + hub), c1 = __ldg(L.hub_chunk_ptr + hub + 1);
  for (int t = 0; t < n_out; ++t) {
    float4 a = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int c = c0; c < c1; ++c) {
      const float4 x = *reinterpret_cast<const float4*>(
          part + (int64_t(c) * n_out + t) * row_elems + col);
      a.x += x.x; a.y += x.y; a.z += x.z; a.w += x.w;
    }
    const float s = t == 0 ? scale0 : scale1;
    T* o = static_cast<T*>(t == 0 ? out0 : out1) + int64_t(row) * row_elems + col;
    if constexpr (sizeof(T) == 4) {
      *reinterpret_cast<float4*>(o) = make_float4(a.x * s, a.y * s, a.z * s, a.w * s);
    } else {
      const __nv_bfloat162 lo = __floats2bfloat162_rn(a.x * s, a.y * s);
      const __nv_bfloat162 hi = __floats2bfloat162_rn(a.z * s, a.w * s);
      uint2 pk;
      pk.x = *reinterpret_cast<const uint32_t*>(&lo);
      pk.y = *reinterpret_cast<const uint32_t*>(&hi);
      *reinterpret_cast<uint2*>(o) = pk;
    }
  }
}

struct BwdScratch {
  size_t stats, part_a, part_b, total;
};

BwdScratch plan_bwd_scratch(const tgt_layout* by_dst, const tgt_layout* by_src, int heads,
                            int head_dim) {
  BwdScratch s;
  const size_t row = size_t(heads) * head_dim * 4;
  size_t off = 0;
  s.stats = off; off += round_up(size_t(by_dst->n_rows) * heads * 8, 256);
  s.part_a = off; off += round_up(size_t(by_dst->n_chunks) * row, 256);
  s.part_b = off; off += round_up(size_t(by_src->n_chunks) * 2 * row, 256);
  s.total = off;
  return s;
}

}  // namespace

size_t fwd_scratch_bytes(const tgt_layout* L, int heads, int head_dim);

}  // namespace tgt

extern "C" int tgt_sparse_attn_scratch_bytes(const tgt_layout* by_dst, const tgt_layout* by_src,
                                             int heads, int head_dim, int phase, size_t* bytes) {
  using namespace tgt;
  TGT_CHECK_ARG(bytes != nullptr, "bytes is null");
  TGT_CHECK_ARG(heads >= 1 && head_dim >= 1, "heads and head_dim must be >= 1");
  TGT_CHECK_ARG(phase == 0 || phase == 1, "phase must be 0 (forward) or 1 (backward)");
  int rc = check_layout(by_dst, "by_dst");
  if (rc != TGT_OK) return rc;
  if (phase == 0) {
    *bytes = by_dst->n_chunks > 0 ? fwd_scratch_bytes(by_dst, heads, head_dim) : 0;
    return TGT_OK;
  }
  rc = check_layout(by_src, "by_src");
  if (rc != TGT_OK) return rc;
  *bytes = plan_bwd_scratch(by_dst, by_src, heads, head_dim).total;
  return TGT_OK;
}

extern "C" int tgt_sparse_attn_bwd(const void* dout, const void* q, const void* k, const void* v,
                                   const float* bias, int bias_heads, const void* out,
                                   const float* z, const tgt_layout* by_dst,
                                   const tgt_layout* by_src, void* dq, void* dk, void* dv,
                                   float* dbias, int heads, int head_dim, int dtype, void* scratch,
                                   size_t scratch_bytes, void* stream) {
  return tgt_sparse_attn_bwd_passes(dout, q, k, v, bias, bias_heads, out, z, by_dst, by_src, dq, dk,
                                    dv, dbias, heads, head_dim, dtype, scratch, scratch_bytes, stream,
                                    3);
}

extern "C" int tgt_sparse_attn_bwd_passes(const void* dout, const void* q, const void* k,
                                          const void* v, const float* bias, int bias_heads,
                                          const void* out, const float* z, const tgt_layout* by_dst,
                                          const tgt_layout* by_src, void* dq, void* dk, void* dv,
                                          float* dbias, int heads, int head_dim, int dtype,
                                          void* scratch, size_t scratch_bytes, void* stream_,
                                          int passes) {
  using namespace tgt;
  TGT_CHECK_ARG(passes >= 1 && passes <= 3, "passes must be 1 (dQ), 2 (dK/dV) or 3 (both)");
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  TGT_CHECK_ARG(dtype == TGT_F32 || dtype == TGT_BF16, "dtype must be TGT_F32 or TGT_BF16");
  int rc = check_layout(by_dst, "by_dst");
  if (rc != TGT_OK) return rc;
  rc = check_layout(by_src, "by_src");
  if (rc != TGT_OK) return rc;
  TGT_CHECK_ARG(by_dst->n_rows == by_src->n_rows && by_dst->n_edges == by_src->n_edges,
                "by_dst and by_src describe different graphs");
  HeadSplit hs;
  if (!split_heads(heads, head_dim, dtype, &hs))
    return set_error(TGT_ERR_UNSUPPORTED,
                     "heads=%d head_dim=%d dtype=%d: head_dim must be a power of two multiple of "
                     "16 bytes, at most 512 bytes per head",
                     heads, head_dim, dtype);
  TGT_CHECK_ARG(bias_heads == 0 || bias_heads == 1 || bias_heads == heads,
                "bias_heads must be 0, 1 or heads");
  TGT_CHECK_ARG((bias_heads == 0) == (bias == nullptr), "bias pointer and bias_heads disagree");
  TGT_CHECK_ARG(dbias == nullptr || bias != nullptr, "dbias requested without bias");
  if (dbias != nullptr && bias_heads == 1 && hs.groups > 1)
    return set_error(TGT_ERR_UNSUPPORTED,
                     "a per-edge scalar dbias needs all heads in one lane group (heads*head_dim "
                     "<= 512 bytes, heads a power of two); pass a per-head bias instead");
  if (by_dst->n_rows == 0) return TGT_OK;
  TGT_CHECK_ARG(dout && q && k && v && out && z && dq && dk && dv, "tensor pointers must not be null");
  TGT_CHECK_ARG(aligned16(dout) && aligned16(q) && aligned16(k) && aligned16(v) && aligned16(out) &&
                    aligned16(z) && aligned16(dq) && aligned16(dk) && aligned16(dv) &&
                    aligned16(bias) && aligned16(dbias) && aligned16(scratch),
                "device pointers must be 16-byte aligned");
  const BwdScratch sc = plan_bwd_scratch(by_dst, by_src, heads, head_dim);
  if (scratch == nullptr || scratch_bytes < sc.total)
    return set_error(TGT_ERR_WORKSPACE, "scratch holds %zu bytes, %zu needed", scratch_bytes,
                     sc.total);
  char* base = static_cast<char*>(scratch);

  BwdParams p;
  p.dout = dout; p.q = q; p.k = k; p.v = v; p.out = out; p.z = z;
  p.bias = bias; p.bias_heads = bias_heads;
  p.dq = dq; p.dk = dk; p.dv = dv; p.dbias = dbias;
  p.stats = reinterpret_cast<float2*>(base + sc.stats);
  p.heads = heads;
  p.row_elems = heads * head_dim;
  p.inv_scale = 1.0f / sqrtf(float(head_dim));
  const dim3 reduce_y((p.row_elems + 127) / 128);

#define TGT_LAUNCH_DQ(T, LPH, G) bwd_dq_kernel<T, LPH, G><<<grid, kBlockThreads, 0, stream>>>(p)
#define TGT_LAUNCH_DKV(T, LPH, G) bwd_dkv_kernel<T, LPH, G><<<grid, kBlockThreads, 0, stream>>>(p)

  // ---- pass A over destinations
  if (passes & 1) {
    const tgt_layout& L = *by_dst;
    p.L = L;
    p.part = reinterpret_cast<float*>(base + sc.part_a);
    p.lpr_log2 = choose_lpr_log2(hs.g, double(L.n_edges) / double(L.n_rows));
    if (L.n_chunks > 0) {
      p.chunk_mode = 1;
      dim3 grid((L.n_chunks + kWarpsPerBlock - 1) / kWarpsPerBlock, hs.groups);
      TGT_DISPATCH(dtype, hs.lph, hs.g, TGT_LAUNCH_DQ);
    }
    p.chunk_mode = 0;
    const int64_t rows_per_block = int64_t(kWarpsPerBlock) * (32 >> p.lpr_log2);
    dim3 grid(unsigned((L.n_rows + rows_per_block - 1) / rows_per_block), hs.groups);
    TGT_DISPATCH(dtype, hs.lph, hs.g, TGT_LAUNCH_DQ);
    if (L.n_hubs > 0) {
      dim3 rgrid((L.n_hubs + kWarpsPerBlock - 1) / kWarpsPerBlock, reduce_y.x);
      if (dtype == TGT_F32)
        bwd_hub_reduce_kernel<float><<<rgrid, kBlockThreads, 0, stream>>>(
            L, p.part, 1, dq, nullptr, p.inv_scale, 0.f, p.row_elems);
      else
        bwd_hub_reduce_kernel<__nv_bfloat16><<<rgrid, kBlockThreads, 0, stream>>>(
            L, p.part, 1, dq, nullptr, p.inv_scale, 0.f, p.row_elems);
    }
  }
  // ---- pass B over sources
  if (passes & 2) {
    const tgt_layout& L = *by_src;
    p.L = L;
    p.part = reinterpret_cast<float*>(base + sc.part_b);
    p.lpr_log2 = choose_lpr_log2(hs.g, double(L.n_edges) / double(L.n_rows));
    if (L.n_chunks > 0) {
      p.chunk_mode = 1;
      dim3 grid((L.n_chunks + kWarpsPerBlock - 1) / kWarpsPerBlock, hs.groups);
      TGT_DISPATCH(dtype, hs.lph, hs.g, TGT_LAUNCH_DKV);
    }
    p.chunk_mode = 0;
    const int64_t rows_per_block = int64_t(kWarpsPerBlock) * (32 >> p.lpr_log2);
    dim3 grid(unsigned((L.n_rows + rows_per_block - 1) / rows_per_block), hs.groups);
    TGT_DISPATCH(dtype, hs.lph, hs.g, TGT_LAUNCH_DKV);
    if (L.n_hubs > 0) {
      dim3 rgrid((L.n_hubs + kWarpsPerBlock - 1) / kWarpsPerBlock, reduce_y.x);
      if (dtype == TGT_F32)
        bwd_hub_reduce_kernel<float><<<rgrid, kBlockThreads, 0, stream>>>(
            L, p.part, 2, dk, dv, p.inv_scale, 1.0f, p.row_elems);
      else
        bwd_hub_reduce_kernel<__nv_bfloat16><<<rgrid, kBlockThreads, 0, stream>>>(
            L, p.part, 2, dk, dv, p.inv_scale, 1.0f, p.row_elems);
    }
  }
#undef TGT_LAUNCH_DQ
#undef TGT_LAUNCH_DKV
  TGT_CHECK_CUDA(cudaGetLastError());
  return TGT_OK;
}
