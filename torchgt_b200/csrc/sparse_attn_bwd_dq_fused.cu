// Backward of the sparse graph attention, pass A that derives the row statistics itself (see sparse_attn_bwd.cuh).
#include "sparse_attn_bwd.cuh"

namespace tgt {
namespace bwd {
namespace {

// ---- pass A without a statistics pre-pass (no dbias) ---------------------------------------------
template <typename T, int W, int LPH, int G>
struct DqFusedPolicy {
  static constexpr int VEC = Lane<T, W>::kElems;
  static constexpr int NACC = 2 * VEC + 1;  // A1, A2, S
  static constexpr int kUnroll = walk_unroll<T, W, G>();

  const T* __restrict__ q;
  const T* __restrict__ k;
  const T* __restrict__ v;
  const T* __restrict__ dout;
  const float* __restrict__ z;
  const float* __restrict__ bias;
  float2* __restrict__ stats;
  T* __restrict__ dq;
  int bias_stride, bias_off;
  unsigned row_vecs, cvec, q_vecs, kv_vecs, g_vecs;
  int heads, head;
  bool head_leader;
  float inv_scale;

  using Raw = typename Lane<T, W>::Raw;
  struct Operands {
    Raw k, v, q, g;
    float b;
  };
  struct Scalars {
    float wm, wgv_m, wgv;  // mask*w, mask*w*(dO.V), w*(dO.V)
  };

  __device__ __forceinline__ void load(Operands& o, int row, int src, int pe) const {
    const unsigned so = unsigned(src) * kv_vecs + cvec;
    o.k = Lane<T, W>::raw_at(k, so);
    o.v = Lane<T, W>::raw_at(v, so);
    o.q = Lane<T, W>::raw_at(q, unsigned(row) * q_vecs + cvec);
    o.g = Lane<T, W>::raw_at(dout, unsigned(row) * g_vecs + cvec);
    o.b = bias != nullptr ? __ldg(bias + int64_t(pe) * bias_stride + bias_off) : 0.f;
  }
  __device__ __forceinline__ void clear(Operands& o) const {
    o.k = o.v = o.q = o.g = Lane<T, W>::raw_zero();
    o.b = 0.f;
  }
  __device__ __forceinline__ Scalars prep(const Operands& o, bool valid, int) const {
    float a[VEC], b[VEC];
    Lane<T, W>::unpack(o.q, a);
    Lane<T, W>::unpack(o.k, b);
    const float raw = group_sum<LPH>(dot<VEC>(a, b)) * inv_scale;
    Lane<T, W>::unpack(o.g, a);
    Lane<T, W>::unpack(o.v, b);
    const float gv = group_sum<LPH>(dot<VEC>(a, b));
    const float wgt = valid ? fast_exp(clamp_score(raw) + o.b) : 0.f;
    Scalars s;
    s.wgv = wgt * gv;
    s.wm = clamp_passes_grad(raw) ? wgt : 0.f;
    s.wgv_m = s.wm * gv;
    return s;
  }
  __device__ __forceinline__ void accumulate(float (&acc)[NACC], const Operands& o,
                                             const Scalars& s) const {
    float kf[VEC];
    Lane<T, W>::unpack(o.k, kf);
#pragma unroll
    for (int j = 0; j < VEC; ++j) {
      acc[j] = fmaf(s.wgv_m, kf[j], acc[j]);
      acc[VEC + j] = fmaf(s.wm, kf[j], acc[VEC + j]);
    }
    acc[2 * VEC] += s.wgv;
  }
  __device__ __forceinline__ void finalize(int row, const float (&acc)[NACC]) const {
    const float inv = 1.0f / (__ldg(z + int64_t(row) * heads + head) + kZEps);
    const float delta = inv * acc[2 * VEC];
    float o[VEC];
#pragma unroll
    for (int j = 0; j < VEC; ++j) o[j] = (acc[j] - delta * acc[VEC + j]) * (inv * inv_scale);
    Lane<T, W>::store_at(dq, unsigned(row) * row_vecs + cvec, o);
    if (head_leader) stats[int64_t(row) * heads + head] = make_float2(inv, delta);
  }
  __device__ __forceinline__ void zero_row(int row) const {
    float o[VEC];
#pragma unroll
    for (int j = 0; j < VEC; ++j) o[j] = 0.f;
    Lane<T, W>::store_at(dq, unsigned(row) * row_vecs + cvec, o);
  }
};

template <typename T, int W, int LPH, int G>
__device__ __forceinline__ DqFusedPolicy<T, W, LPH, G> make_dq_fused_policy(const BwdParams& p) {
  constexpr int VEC = Lane<T, W>::kElems;
  const int c = threadIdx.x % G;
  DqFusedPolicy<T, W, LPH, G> pol;
  pol.q = static_cast<const T*>(p.q);
  pol.k = static_cast<const T*>(p.k);
  pol.v = static_cast<const T*>(p.v);
  pol.dout = static_cast<const T*>(p.dout);
  pol.z = p.z;
  pol.bias = p.bias;
  pol.stats = p.stats;
  pol.dq = static_cast<T*>(p.dq);
  pol.head = blockIdx.y * (G / LPH) + c / LPH;
  pol.bias_stride = p.bias_heads;
  pol.bias_off = p.bias_heads > 1 ? pol.head : 0;
  pol.row_vecs = unsigned(p.row_elems / VEC);
  pol.q_vecs = unsigned(p.q_row_bytes / W);
  pol.kv_vecs = unsigned(p.kv_row_bytes / W);
  pol.g_vecs = unsigned(p.g_row_bytes / W);
  pol.heads = p.heads;
  pol.cvec = blockIdx.y * G + c;
  pol.head_leader = c % LPH == 0;
  pol.inv_scale = p.inv_scale;
  return pol;
}

template <typename T, int W, int LPH, int G>
__global__ void TGT_WALK_BOUNDS bwd_dq_fused_kernel(const BwdParams p) {
  using Policy = DqFusedPolicy<T, W, LPH, G>;
  __shared__ TileSmem<G, Policy::NACC> sm;
  const Policy pol = make_dq_fused_policy<T, W, LPH, G>(p);
  walk_tile_in<G, Policy>(sm, p.walk, pol);
}

template <typename T, int W, int LPH, int G>
__global__ void __launch_bounds__(kBlockThreads) bwd_dq_fused_stitch_kernel(const BwdParams p) {
  using Policy = DqFusedPolicy<T, W, LPH, G>;
  const Policy pol = make_dq_fused_policy<T, W, LPH, G>(p);
  __shared__ float s_part[kBlockThreads * Policy::NACC];
  stitch_tiles<G, Policy>(p.walk, pol, s_part);
}


}  // namespace

bool launch_dq_fused(const BwdParams& p, int dtype, const HeadSplit& hs, dim3 grid, bool second_kernel, int link,
                     cudaStream_t stream) {
  return dispatch_shape(dtype, hs.w, hs.lph, hs.g, [&](auto sh) {
    using S = decltype(sh);
    launch_chained(bwd_dq_fused_kernel<typename S::T, S::W, S::LPH, S::G>, grid, kBlockThreads, stream, link, p);
    if (second_kernel && grid.x > 1)
      launch_chained(bwd_dq_fused_stitch_kernel<typename S::T, S::W, S::LPH, S::G>, grid, kBlockThreads, stream, kLinkStitch, p);
  });
}

int occupancy_dq_fused(int dtype, const HeadSplit& hs, int* cache_slot) {
  int result = 4;
  dispatch_shape(dtype, hs.w, hs.lph, hs.g, [&](auto sh) {
    using S = decltype(sh);
    result = resident_ctas(bwd_dq_fused_kernel<typename S::T, S::W, S::LPH, S::G>, cache_slot);
  });
  return result;
}

}  // namespace bwd
}  // namespace tgt
