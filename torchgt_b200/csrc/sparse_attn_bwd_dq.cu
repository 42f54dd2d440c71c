// Backward of the sparse graph attention, pass A with per-edge dbias (see sparse_attn_bwd.cuh).
#include "sparse_attn_bwd.cuh"

namespace tgt {
namespace bwd {
namespace {

// ---- pass A: dQ and dbias -----------------------------------------------------------------------
template <typename T, int W, int LPH, int G>
struct DqPolicy {
  static constexpr int VEC = Lane<T, W>::kElems;
  static constexpr int NACC = VEC;
  static constexpr int kUnroll = walk_unroll<T, W, G>();

  const T* __restrict__ q;
  const T* __restrict__ k;
  const T* __restrict__ v;
  const T* __restrict__ dout;
  const float2* __restrict__ stats;
  const float* __restrict__ bias;
  float* __restrict__ dbias;
  T* __restrict__ dq;
  int bias_stride, bias_off;
  unsigned row_vecs, cvec, q_vecs, kv_vecs, g_vecs;
  int heads, head;
  bool head_leader, group_leader;
  float inv_scale;

  using Raw = typename Lane<T, W>::Raw;
  struct Operands {
    Raw k, v, q, g;  // packed 16-byte pieces, unpacked where they are used
    float2 st;
    float b;
  };
  struct Scalars {
    float da;
  };

  __device__ __forceinline__ void load(Operands& o, int row, int src, int pe) const {
    const unsigned so = unsigned(src) * kv_vecs + cvec;
    o.k = Lane<T, W>::raw_at(k, so);
    o.v = Lane<T, W>::raw_at(v, so);
    o.q = Lane<T, W>::raw_at(q, unsigned(row) * q_vecs + cvec);
    o.g = Lane<T, W>::raw_at(dout, unsigned(row) * g_vecs + cvec);
    o.st = __ldg(stats + int64_t(row) * heads + head);
    o.b = bias != nullptr ? __ldg(bias + int64_t(pe) * bias_stride + bias_off) : 0.f;
  }
  __device__ __forceinline__ void clear(Operands& o) const {
    o.k = o.v = o.q = o.g = Lane<T, W>::raw_zero();
    o.st = make_float2(0.f, 0.f);
    o.b = 0.f;
  }
  __device__ __forceinline__ Scalars prep(const Operands& o, bool valid, int pe) const {
    float a[VEC], b[VEC];
    Lane<T, W>::unpack(o.q, a);
    Lane<T, W>::unpack(o.k, b);
    const float raw = group_sum<LPH>(dot<VEC>(a, b)) * inv_scale;
    Lane<T, W>::unpack(o.g, a);
    Lane<T, W>::unpack(o.v, b);
    const float gv = group_sum<LPH>(dot<VEC>(a, b));
    const float wgt = fast_exp(clamp_score(raw) + o.b);
    const float dt = valid ? (gv - o.st.y) * o.st.x * wgt : 0.f;
    if (dbias != nullptr) {
      if (bias_stride == 1) {
        const float s = sum_over_heads<LPH, G>(dt);   // every head's dt sits on all LPH lanes of the head
        if (valid && group_leader) dbias[pe] = s;
      } else if (valid && head_leader) {
        dbias[int64_t(pe) * bias_stride + head] = dt;
      }
    }
    Scalars s;
    s.da = clamp_passes_grad(raw) ? dt : 0.f;
    return s;
  }
  __device__ __forceinline__ void accumulate(float (&acc)[NACC], const Operands& o,
                                             const Scalars& s) const {
    float kf[VEC];
    Lane<T, W>::unpack(o.k, kf);
#pragma unroll
    for (int j = 0; j < VEC; ++j) acc[j] = fmaf(s.da, kf[j], acc[j]);
  }
  __device__ __forceinline__ void finalize(int row, const float (&acc)[NACC]) const {
    float o[VEC];
#pragma unroll
    for (int j = 0; j < VEC; ++j) o[j] = acc[j] * inv_scale;
    Lane<T, W>::store_at(dq, unsigned(row) * row_vecs + cvec, o);
  }
  __device__ __forceinline__ void zero_row(int row) const {
    float o[VEC];
#pragma unroll
    for (int j = 0; j < VEC; ++j) o[j] = 0.f;
    Lane<T, W>::store_at(dq, unsigned(row) * row_vecs + cvec, o);
  }
};

template <typename T, int W, int LPH, int G>
__device__ __forceinline__ DqPolicy<T, W, LPH, G> make_dq_policy(const BwdParams& p) {
  constexpr int VEC = Lane<T, W>::kElems;
  const int c = threadIdx.x % G;
  DqPolicy<T, W, LPH, G> pol;
  pol.q = static_cast<const T*>(p.q);
  pol.k = static_cast<const T*>(p.k);
  pol.v = static_cast<const T*>(p.v);
  pol.dout = static_cast<const T*>(p.dout);
  pol.stats = p.stats;
  pol.bias = p.bias;
  pol.dbias = p.dbias;
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
  pol.group_leader = c == 0;
  pol.inv_scale = p.inv_scale;
  return pol;
}

template <typename T, int W, int LPH, int G>
__global__ void TGT_WALK_BOUNDS bwd_dq_kernel(const BwdParams p) {
  using Policy = DqPolicy<T, W, LPH, G>;
  __shared__ TileSmem<G, Policy::NACC> sm;
  const Policy pol = make_dq_policy<T, W, LPH, G>(p);
  walk_tile_in<G, Policy>(sm, p.walk, pol);
}

template <typename T, int W, int LPH, int G>
__global__ void __launch_bounds__(kBlockThreads) bwd_dq_stitch_kernel(const BwdParams p) {
  using Policy = DqPolicy<T, W, LPH, G>;
  const Policy pol = make_dq_policy<T, W, LPH, G>(p);
  __shared__ float s_part[kBlockThreads * Policy::NACC];
  stitch_tiles<G, Policy>(p.walk, pol, s_part);
}


}  // namespace

bool launch_dq(const BwdParams& p, int dtype, const HeadSplit& hs, dim3 grid, bool second_kernel, int link,
               cudaStream_t stream) {
  return dispatch_shape(dtype, hs.w, hs.lph, hs.g, [&](auto sh) {
    using S = decltype(sh);
    launch_chained(bwd_dq_kernel<typename S::T, S::W, S::LPH, S::G>, grid, kBlockThreads, stream, link, p);
    if (second_kernel && grid.x > 1)
      launch_chained(bwd_dq_stitch_kernel<typename S::T, S::W, S::LPH, S::G>, grid, kBlockThreads, stream, kLinkStitch, p);
  });
}

int occupancy_dq(int dtype, const HeadSplit& hs, int* cache_slot) {
  int result = 4;
  dispatch_shape(dtype, hs.w, hs.lph, hs.g, [&](auto sh) {
    using S = decltype(sh);
    result = resident_ctas(bwd_dq_kernel<typename S::T, S::W, S::LPH, S::G>, cache_slot);
  });
  return result;
}

}  // namespace bwd
}  // namespace tgt
