// Forward of the topology-aware sparse graph attention: SDDMM -> clamp -> +bias -> exp ->
// running sums of w and w*V -> divide by (Z + 1e-6), fused in one pass over the edges sorted by
// destination.  No [E, H, D] tensor ever exists.
#include "attn_common.cuh"

namespace tgt {
namespace {

template <typename T, int W, int LPH, int G>
struct FwdPolicy {
  static constexpr int VEC = Lane<T, W>::kElems;
  static constexpr int NACC = VEC + 1;  // w*V and, last, the sum of w
  static constexpr int kUnroll = walk_unroll<T, W, G>();

  const T* __restrict__ q;
  const T* __restrict__ k;
  const T* __restrict__ v;
  const float* __restrict__ bias;  // original edge order, may be null
  T* __restrict__ out;
  float* __restrict__ z;           // [n_rows, heads]
  int bias_stride, bias_off;
  unsigned row_vecs, cvec;         // lane-wide units per (dense) row; this lane's unit inside a row
  unsigned q_vecs, kv_vecs;        // row strides of q and of k / v in lane-wide units
  int heads, head;                 // head count; the head this lane belongs to
  bool z_writer;                   // one lane per head stores Z
  float inv_scale;

  using Raw = typename Lane<T, W>::Raw;
  struct Operands {
    Raw k, v, q;  // packed 16-byte pieces, unpacked where they are used
    float b;
  };
  struct Scalars {
    float w;
  };

  __device__ __forceinline__ void load(Operands& o, int row, int src, int pe) const {
    const unsigned so = unsigned(src) * kv_vecs + cvec;
    o.k = Lane<T, W>::raw_at(k, so);
    o.v = Lane<T, W>::raw_at(v, so);
    o.q = Lane<T, W>::raw_at(q, unsigned(row) * q_vecs + cvec);
    o.b = bias != nullptr ? __ldg(bias + int64_t(pe) * bias_stride + bias_off) : 0.f;
  }
  __device__ __forceinline__ void clear(Operands& o) const {
    o.k = o.v = o.q = Lane<T, W>::raw_zero();
    o.b = 0.f;
  }
  __device__ __forceinline__ Scalars prep(const Operands& o, bool valid, int) const {
    float qf[VEC], kf[VEC];
    Lane<T, W>::unpack(o.q, qf);
    Lane<T, W>::unpack(o.k, kf);
    const float raw = group_sum<LPH>(dot<VEC>(qf, kf)) * inv_scale;
    Scalars s;
    s.w = valid ? fast_exp(clamp_score(raw) + o.b) : 0.f;
    return s;
  }
  __device__ __forceinline__ void accumulate(float (&acc)[NACC], const Operands& o,
                                             const Scalars& s) const {
    float vf[VEC];
    Lane<T, W>::unpack(o.v, vf);
#pragma unroll
    for (int j = 0; j < VEC; ++j) acc[j] = fmaf(s.w, vf[j], acc[j]);
    acc[VEC] += s.w;
  }
  __device__ __forceinline__ void finalize(int row, const float (&acc)[NACC]) const {
    const float inv = 1.0f / (acc[VEC] + kZEps);
    float o[VEC];
#pragma unroll
    for (int j = 0; j < VEC; ++j) o[j] = acc[j] * inv;
    Lane<T, W>::store_at(out, unsigned(row) * row_vecs + cvec, o);
    if (z_writer) z[int64_t(row) * heads + head] = acc[VEC];
  }
  __device__ __forceinline__ void zero_row(int row) const {
    float o[VEC];
#pragma unroll
    for (int j = 0; j < VEC; ++j) o[j] = 0.f;
    Lane<T, W>::store_at(out, unsigned(row) * row_vecs + cvec, o);
    if (z_writer) z[int64_t(row) * heads + head] = 0.f;
  }
};

struct FwdParams {
  const void* q;
  const void* k;
  const void* v;
  const float* bias;
  int bias_heads;
  void* out;
  float* z;
  int heads, row_elems;
  int64_t q_row_bytes, kv_row_bytes;   // distance between consecutive rows of q and of k / v
  float inv_scale;
  SegWalk walk;
};

template <typename T, int W, int LPH, int G>
__device__ __forceinline__ FwdPolicy<T, W, LPH, G> make_policy(const FwdParams& p) {
  constexpr int VEC = Lane<T, W>::kElems;
  const int c = threadIdx.x % G;
  FwdPolicy<T, W, LPH, G> pol;
  pol.q = static_cast<const T*>(p.q);
  pol.k = static_cast<const T*>(p.k);
  pol.v = static_cast<const T*>(p.v);
  pol.bias = p.bias;
  pol.out = static_cast<T*>(p.out);
  pol.z = p.z;
  pol.head = blockIdx.y * (G / LPH) + c / LPH;
  pol.bias_stride = p.bias_heads;
  pol.bias_off = p.bias_heads > 1 ? pol.head : 0;
  pol.row_vecs = unsigned(p.row_elems / VEC);
  pol.q_vecs = unsigned(p.q_row_bytes / W);
  pol.kv_vecs = unsigned(p.kv_row_bytes / W);
  pol.heads = p.heads;
  pol.cvec = blockIdx.y * G + c;
  pol.z_writer = c % LPH == 0;
  pol.inv_scale = p.inv_scale;
  return pol;
}

template <typename T, int W, int LPH, int G>
__global__ void TGT_WALK_BOUNDS fwd_kernel(const FwdParams p) {
  using Policy = FwdPolicy<T, W, LPH, G>;
  __shared__ TileSmem<G, Policy::NACC> sm;
  const Policy pol = make_policy<T, W, LPH, G>(p);
  walk_tile_in<G, Policy>(sm, p.walk, pol);
}

template <typename T, int W, int LPH, int G>
__global__ void __launch_bounds__(kBlockThreads) fwd_stitch_kernel(const FwdParams p) {
  using Policy = FwdPolicy<T, W, LPH, G>;
  const Policy pol = make_policy<T, W, LPH, G>(p);
  __shared__ float s_part[kBlockThreads * Policy::NACC];
  stitch_tiles<G, Policy>(p.walk, pol, s_part);
}

// Resident CTAs per SM of fwd_kernel<T, W, LPH, G> for the run-time triple.
int fwd_resident_ctas(int dtype, const HeadSplit& hs) {
  static int cache[kMaxDevices][2][2][6][6] = {};   // occupancy is a property of the device
  auto log2i = [](int x) { int l = 0; while ((1 << l) < x) ++l; return l; };
  const int dev = current_device();
  int* slot = &cache[dev < 0 ? 0 : dev][hs.w == 32 ? 1 : 0][dtype == TGT_F32 ? 0 : 1][log2i(hs.lph)][log2i(hs.g)];
  int result = 4;
  dispatch_shape(dtype, hs.w, hs.lph, hs.g, [&](auto sh) {
    using S = decltype(sh);
    result = resident_ctas(fwd_kernel<typename S::T, S::W, S::LPH, S::G>, slot);
  });
  return result;
}

}  // namespace

TilePlan plan_tiles(int64_t n_edges, const HeadSplit& hs, int nacc, int ctas_per_sm) {
  TilePlan t;
  t.ge = choose_ge(n_edges, hs.g, ctas_per_sm);
  const int64_t te = int64_t(kBlockThreads / hs.g) * t.ge;
  t.n_tiles = int((n_edges + te - 1) / te);
  t.carry_bytes = round_up(size_t(t.n_tiles) * 2 * size_t(hs.groups) * hs.g * nacc * 4, 256);
  t.counter_bytes = round_up(size_t(t.n_tiles) * hs.groups * 4, 256);
  t.scratch_bytes = t.carry_bytes + t.counter_bytes;
  return t;
}

// Scratch of the forward for lanes of w bytes (0 when that width does not fit the heads).
size_t fwd_scratch_bytes_w(const tgt_layout* L, int heads, int head_dim, int dtype, int w) {
  HeadSplit hs;
  if (!split_heads(heads, head_dim, dtype, w, &hs) || L->n_edges == 0) return 0;
  const int nacc = w / (dtype == TGT_F32 ? 4 : 2) + 1;
  return plan_tiles(L->n_edges, hs, nacc, fwd_resident_ctas(dtype, hs)).scratch_bytes;
}

// What a caller must provide: enough for whichever lane width the call ends up using (the width depends
// on pointer alignment, which the size query does not see).
size_t fwd_scratch_bytes(const tgt_layout* L, int heads, int head_dim, int dtype) {
  size_t need = fwd_scratch_bytes_w(L, heads, head_dim, dtype, 16);
  if (lane_bytes(heads, head_dim, dtype, true, kPassFwd) == 32) {
    const size_t wide = fwd_scratch_bytes_w(L, heads, head_dim, dtype, 32);
    if (wide > need) need = wide;
  }
  return need;
}

}  // namespace tgt

extern "C" int tgt_sparse_attn_fwd(const void* q, const void* k, const void* v, const float* bias,
                                   int bias_heads, const tgt_layout* by_dst, void* out, float* z,
                                   int heads, int head_dim, int dtype, void* scratch,
                                   size_t scratch_bytes, void* stream) {
  const int64_t row_bytes = int64_t(heads) * head_dim * (dtype == TGT_F32 ? 4 : 2);
  return tgt_sparse_attn_fwd_strided(q, row_bytes, k, v, row_bytes, bias, bias_heads, by_dst, out, z,
                                     heads, head_dim, dtype, scratch, scratch_bytes, stream);
}

extern "C" int tgt_sparse_attn_fwd_strided(const void* q, int64_t q_row_bytes, const void* k,
                                           const void* v, int64_t kv_row_bytes, const float* bias,
                                           int bias_heads, const tgt_layout* by_dst, void* out,
                                           float* z, int heads, int head_dim, int dtype,
                                           void* scratch, size_t scratch_bytes, void* stream_) {
  using namespace tgt;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  TGT_CHECK_ARG(dtype == TGT_F32 || dtype == TGT_BF16, "dtype must be TGT_F32 or TGT_BF16");
  int rc = check_layout(by_dst, "by_dst");
  if (rc != TGT_OK) return rc;
  const bool can32 = aligned32(q) && aligned32(k) && aligned32(v) && aligned32(out) && q_row_bytes % 32 == 0 &&
                     kv_row_bytes % 32 == 0;
  HeadSplit hs;
  if (!split_heads(heads, head_dim, dtype, lane_bytes(heads, head_dim, dtype, can32, kPassFwd), &hs))
    return set_error(TGT_ERR_UNSUPPORTED,
                     "heads=%d head_dim=%d dtype=%d: head_dim must be a power of two multiple of "
                     "16 bytes, at most 512 bytes per head",
                     heads, head_dim, dtype);
  TGT_CHECK_ARG(bias_heads == 0 || bias_heads == 1 || bias_heads == heads,
                "bias_heads must be 0, 1 or heads");
  TGT_CHECK_ARG((bias_heads == 0) == (bias == nullptr), "bias pointer and bias_heads disagree");
  const tgt_layout& L = *by_dst;
  if (L.n_rows == 0) return TGT_OK;
  const size_t elem = dtype == TGT_F32 ? 4 : 2;
  const int64_t row_bytes = int64_t(heads) * head_dim * int64_t(elem);
  TGT_CHECK_ARG(q && k && v && out && z, "q/k/v/out/z must not be null");
  TGT_CHECK_ARG(q_row_bytes >= row_bytes && kv_row_bytes >= row_bytes && q_row_bytes % 16 == 0 &&
                    kv_row_bytes % 16 == 0,
                "row strides must be multiples of 16 bytes and at least heads * head_dim elements");
  TGT_CHECK_ARG(uint64_t(L.n_rows) * uint64_t(q_row_bytes > kv_row_bytes ? q_row_bytes : kv_row_bytes) / 16 <
                    (uint64_t(1) << 32),
                "tensors larger than 64 GiB are not supported");
  TGT_CHECK_ARG(aligned16(q) && aligned16(k) && aligned16(v) && aligned16(out) && aligned16(z) &&
                    aligned16(bias) && aligned16(scratch),
                "device pointers must be 16-byte aligned");
  if (L.n_edges == 0) {  // no edges: every row is empty
    TGT_CHECK_CUDA(cudaMemsetAsync(out, 0, size_t(L.n_rows) * heads * head_dim * elem, stream));
    TGT_CHECK_CUDA(cudaMemsetAsync(z, 0, size_t(L.n_rows) * heads * 4, stream));
    return TGT_OK;
  }
  const int nacc = hs.w / int(elem) + 1;
  const TilePlan tp = plan_tiles(L.n_edges, hs, nacc, fwd_resident_ctas(dtype, hs));
  if (scratch == nullptr || scratch_bytes < tp.scratch_bytes)
    return set_error(TGT_ERR_WORKSPACE, "scratch holds %zu bytes, %zu needed", scratch_bytes,
                     tp.scratch_bytes);

  FwdParams p;
  p.q = q; p.k = k; p.v = v; p.bias = bias; p.bias_heads = bias_heads;
  p.out = out; p.z = z;
  p.heads = heads;
  p.row_elems = heads * head_dim;
  p.q_row_bytes = q_row_bytes;
  p.kv_row_bytes = kv_row_bytes;
  p.inv_scale = 1.0f / sqrtf(float(head_dim));
  p.walk.ptr = L.ptr; p.walk.other = L.other; p.walk.perm = L.perm; p.walk.seg = L.seg;
  p.walk.n_rows = int(L.n_rows); p.walk.n_edges = int(L.n_edges);
  p.walk.ge = tp.ge; p.walk.n_tiles = tp.n_tiles;
  p.walk.gcarry = static_cast<float*>(scratch);
  const bool second_kernel = stitch_in_second_kernel(hs.g);
  p.walk.tile_done = second_kernel ? nullptr : reinterpret_cast<int*>(static_cast<char*>(scratch) + tp.carry_bytes);
  p.walk.need_perm = bias != nullptr;
  if (tp.n_tiles > 1 && !second_kernel)
    TGT_CHECK_CUDA(cudaMemsetAsync(p.walk.tile_done, 0, tp.counter_bytes, stream));

  const dim3 grid(tp.n_tiles, hs.groups);
  const bool built = dispatch_shape(dtype, hs.w, hs.lph, hs.g, [&](auto sh) {
    using S = decltype(sh);
    fwd_kernel<typename S::T, S::W, S::LPH, S::G><<<grid, kBlockThreads, 0, stream>>>(p);
    if (second_kernel && tp.n_tiles > 1)
      launch_chained(fwd_stitch_kernel<typename S::T, S::W, S::LPH, S::G>, grid, kBlockThreads, stream, kLinkStitch, p);
  });
  if (!built) return set_error(TGT_ERR_UNSUPPORTED, "no kernel is built for this head layout");
  TGT_CHECK_CUDA(cudaGetLastError());
  return TGT_OK;
}

// ---- forward without any allocation by anybody ---------------------------------------------------
// Some hosts cannot give this library scratch memory at call time: a serving process that handed
// every byte of the GPU to its own arena at start-up, a plug-in living inside such a process, or a
// latency-critical loop that must never reach cudaMalloc (which may stall the whole device).  For
// them the cross-tile carry of the forward pass lives in the module itself.
namespace tgt {
namespace {

constexpr size_t kStaticScratchBytes = size_t(4) << 20;  // 4 MiB per GPU that loads the library
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

void* g_static_scratch_ptr[kMaxDevices] = {};  // device address of the array, per device ordinal

// The array's name is only a handle on the host; the address the kernels need comes from the
// runtime, once per device, with that device current.
int static_scratch_address(void** out) {
  int dev = -1;
  TGT_CHECK_CUDA(cudaGetDevice(&dev));
  if (dev < 0 || dev >= kMaxDevices)
    return set_error(TGT_ERR_UNSUPPORTED, "device ordinal %d is outside the supported range", dev);
  void* p = __atomic_load_n(&g_static_scratch_ptr[dev], __ATOMIC_ACQUIRE);
  if (p == nullptr) {
    TGT_CHECK_CUDA(cudaGetSymbolAddress(&p, g_static_scratch));
    __atomic_store_n(&g_static_scratch_ptr[dev], p, __ATOMIC_RELEASE);
  }
  *out = p;
  return TGT_OK;
}

}  // namespace
}  // namespace tgt

extern "C" int tgt_sparse_attn_fwd_noalloc(const void* q, const void* k, const void* v,
                                           const float* bias, int bias_heads,
                                           const tgt_layout* by_dst, void* out, float* z,
                                           int heads, int head_dim, int dtype, void* stream) {
  using namespace tgt;
  TGT_CHECK_ARG(dtype == TGT_F32 || dtype == TGT_BF16, "dtype must be TGT_F32 or TGT_BF16");
  int rc = check_layout(by_dst, "by_dst");
  if (rc != TGT_OK) return rc;
  HeadSplit hs;
  if (!split_heads(heads, head_dim, dtype, 16, &hs))
    return set_error(TGT_ERR_UNSUPPORTED, "heads=%d head_dim=%d dtype=%d is not supported", heads,
                     head_dim, dtype);
  // size check first: nothing is launched and nothing is looked up for a graph that does not fit
  const size_t need = fwd_scratch_bytes(by_dst, heads, head_dim, dtype);
  if (need > kStaticScratchBytes)
    return set_error(TGT_ERR_WORKSPACE,
                     "this graph needs %zu bytes of carry space, the built-in scratch of "
                     "tgt_sparse_attn_fwd_noalloc holds %zu; use tgt_sparse_attn_fwd with caller "
                     "scratch",
                     need, kStaticScratchBytes);
  void* scratch = nullptr;
  rc = static_scratch_address(&scratch);
  if (rc != TGT_OK) return rc;
  return tgt_sparse_attn_fwd(q, k, v, bias, bias_heads, by_dst, out, z, heads, head_dim, dtype,
                             scratch, kStaticScratchBytes, stream);
}
