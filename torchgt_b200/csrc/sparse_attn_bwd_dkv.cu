// Backward of the sparse graph attention, pass B: dK and dV (see sparse_attn_bwd.cuh).
#include "sparse_attn_bwd.cuh"

namespace tgt {
namespace bwd {
namespace {

// ---- pass B: dK and dV --------------------------------------------------------------------------
template <typename T, int W, int LPH, int G>
struct DkvPolicy {
  static constexpr int VEC = Lane<T, W>::kElems;
  static constexpr int NACC = 2 * VEC;  // dK then dV
  static constexpr int kUnroll = walk_unroll<T, W, G>();

  const T* __restrict__ q;
  const T* __restrict__ k;
  const T* __restrict__ v;
  const T* __restrict__ dout;
  const float2* __restrict__ stats;
  const float* __restrict__ bias;
  T* __restrict__ dk;
  T* __restrict__ dv;
  int bias_stride, bias_off;
  unsigned row_vecs, cvec, q_vecs, kv_vecs, g_vecs;
  int heads, head;
  float inv_scale;

  using Raw = typename Lane<T, W>::Raw;
  struct Operands {
    Raw q, g, k, v;  // packed 16-byte pieces, unpacked where they are used
    float2 st;
    float b;
  };
  struct Scalars {
    float da, wi;
  };

  // `row` is the source (K/V row), `dst` the destination whose Q, dO and statistics are gathered
  __device__ __forceinline__ void load(Operands& o, int row, int dst, int pe) const {
    const unsigned ro = unsigned(row) * kv_vecs + cvec;
    o.q = Lane<T, W>::raw_at(q, unsigned(dst) * q_vecs + cvec);
    o.g = Lane<T, W>::raw_at(dout, unsigned(dst) * g_vecs + cvec);
    o.k = Lane<T, W>::raw_at(k, ro);
    o.v = Lane<T, W>::raw_at(v, ro);
    o.st = __ldg(stats + int64_t(dst) * heads + head);
    o.b = bias != nullptr ? __ldg(bias + int64_t(pe) * bias_stride + bias_off) : 0.f;
  }
  __device__ __forceinline__ void clear(Operands& o) const {
    o.k = o.v = o.q = o.g = Lane<T, W>::raw_zero();
    o.st = make_float2(0.f, 0.f);
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
    const float dt = (gv - o.st.y) * o.st.x * wgt;
    Scalars s;
    s.da = clamp_passes_grad(raw) ? dt : 0.f;
    s.wi = wgt * o.st.x;
    return s;
  }
  __device__ __forceinline__ void accumulate(float (&acc)[NACC], const Operands& o,
                                             const Scalars& s) const {
    float qf[VEC], gf[VEC];
    Lane<T, W>::unpack(o.q, qf);
    Lane<T, W>::unpack(o.g, gf);
#pragma unroll
    for (int j = 0; j < VEC; ++j) {
      acc[j] = fmaf(s.da, qf[j], acc[j]);
      acc[VEC + j] = fmaf(s.wi, gf[j], acc[VEC + j]);
    }
  }
  __device__ __forceinline__ void finalize(int row, const float (&acc)[NACC]) const {
    float a[VEC], b[VEC];
#pragma unroll
    for (int j = 0; j < VEC; ++j) {
      a[j] = acc[j] * inv_scale;
      b[j] = acc[VEC + j];
    }
    const unsigned off = unsigned(row) * row_vecs + cvec;
    Lane<T, W>::store_at(dk, off, a);
    Lane<T, W>::store_at(dv, off, b);
  }
  __device__ __forceinline__ void zero_row(int row) const {
    float o[VEC];
#pragma unroll
    for (int j = 0; j < VEC; ++j) o[j] = 0.f;
    const unsigned off = unsigned(row) * row_vecs + cvec;
    Lane<T, W>::store_at(dk, off, o);
    Lane<T, W>::store_at(dv, off, o);
  }
};

template <typename T, int W, int LPH, int G>
__device__ __forceinline__ DkvPolicy<T, W, LPH, G> make_dkv_policy(const BwdParams& p) {
  constexpr int VEC = Lane<T, W>::kElems;
  const int c = threadIdx.x % G;
  DkvPolicy<T, W, LPH, G> pol;
  pol.q = static_cast<const T*>(p.q);
  pol.k = static_cast<const T*>(p.k);
  pol.v = static_cast<const T*>(p.v);
  pol.dout = static_cast<const T*>(p.dout);
  pol.stats = p.stats;
  pol.bias = p.bias;
  pol.dk = static_cast<T*>(p.dk);
  pol.dv = static_cast<T*>(p.dv);
  pol.head = blockIdx.y * (G / LPH) + c / LPH;
  pol.bias_stride = p.bias_heads;
  pol.bias_off = p.bias_heads > 1 ? pol.head : 0;
  pol.row_vecs = unsigned(p.row_elems / VEC);
  pol.q_vecs = unsigned(p.q_row_bytes / W);
  pol.kv_vecs = unsigned(p.kv_row_bytes / W);
  pol.g_vecs = unsigned(p.g_row_bytes / W);
  pol.heads = p.heads;
  pol.cvec = blockIdx.y * G + c;
  pol.inv_scale = p.inv_scale;
  return pol;
}

template <typename T, int W, int LPH, int G>
__global__ void TGT_WALK_BOUNDS bwd_dkv_kernel(const BwdParams p) {
  using Policy = DkvPolicy<T, W, LPH, G>;
  __shared__ TileSmem<G, Policy::NACC> sm;
  const Policy pol = make_dkv_policy<T, W, LPH, G>(p);
  walk_tile_in<G, Policy>(sm, p.walk, pol);
}

template <typename T, int W, int LPH, int G>
__global__ void __launch_bounds__(kBlockThreads) bwd_dkv_stitch_kernel(const BwdParams p) {
  using Policy = DkvPolicy<T, W, LPH, G>;
  const Policy pol = make_dkv_policy<T, W, LPH, G>(p);
  __shared__ float s_part[kBlockThreads * Policy::NACC];
  stitch_tiles<G, Policy>(p.walk, pol, s_part);
}


}  // namespace

bool launch_dkv(const BwdParams& p, int dtype, const HeadSplit& hs, dim3 grid, bool second_kernel, int link,
                cudaStream_t stream) {
  return dispatch_shape(dtype, hs.w, hs.lph, hs.g, [&](auto sh) {
    using S = decltype(sh);
    launch_chained(bwd_dkv_kernel<typename S::T, S::W, S::LPH, S::G>, grid, kBlockThreads, stream, link, p);
    if (second_kernel && grid.x > 1)
      launch_chained(bwd_dkv_stitch_kernel<typename S::T, S::W, S::LPH, S::G>, grid, kBlockThreads, stream, kLinkStitch, p);
  });
}

int occupancy_dkv(int dtype, const HeadSplit& hs, int* cache_slot) {
  int result = 4;
  dispatch_shape(dtype, hs.w, hs.lph, hs.g, [&](auto sh) {
    using S = decltype(sh);
    result = resident_ctas(bwd_dkv_kernel<typename S::T, S::W, S::LPH, S::G>, cache_slot);
  });
  return result;
}

}  // namespace bwd
}  // namespace tgt
