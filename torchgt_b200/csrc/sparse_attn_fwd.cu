// Forward of the topology-aware sparse graph attention: SDDMM -> clamp -> +bias -> exp ->
// running sums of w and w*V -> divide by (Z + 1e-6), fused in one pass over the edges sorted by
// destination.  No [E, H, D] tensor ever exists.
#include "attn_common.cuh"

namespace tgt {
namespace {

template <typename T, int LPH, int G>
struct FwdPolicy {
  static constexpr int VEC = Vec16<T>::kElems;
  static constexpr int NACC = VEC + 1;  // w*V and, last, the sum of w
  static constexpr int kUnroll = walk_unroll<T, G>();

  const T* __restrict__ q;
  const T* __restrict__ k;
  const T* __restrict__ v;
  const float* __restrict__ bias;  // original edge order, may be null
  T* __restrict__ out;
  float* __restrict__ z;           // [n_rows, heads]
  int bias_stride, bias_off;
  unsigned row_vecs, cvec;         // 16-byte units per row; this lane's unit inside a row
  int heads, head;                 // head count; the head this lane belongs to
  bool z_writer;                   // one lane per head stores Z
  float inv_scale;

  using Raw = typename Vec16<T>::Raw;
  struct Operands {
    Raw k, v, q;  // packed 16-byte pieces, unpacked where they are used
    float b;
  };
  struct Scalars {
    float w;
  };

  __device__ __forceinline__ void load(Operands& o, int row, int src, int pe) const {
    const unsigned so = unsigned(src) * row_vecs + cvec;
    o.k = Vec16<T>::raw_at(k, so);
    o.v = Vec16<T>::raw_at(v, so);
    o.q = Vec16<T>::raw_at(q, unsigned(row) * row_vecs + cvec);
    o.b = bias != nullptr ? __ldg(bias + int64_t(pe) * bias_stride + bias_off) : 0.f;
  }
  __device__ __forceinline__ void clear(Operands& o) const {
    o.k = o.v = o.q = Vec16<T>::raw_zero();
    o.b = 0.f;
  }
  __device__ __forceinline__ Scalars prep(const Operands& o, bool valid, int) const {
    float qf[VEC], kf[VEC];
    Vec16<T>::unpack(o.q, qf);
    Vec16<T>::unpack(o.k, kf);
    const float raw = group_sum<LPH>(dot<VEC>(qf, kf)) * inv_scale;
    Scalars s;
    s.w = valid ? fast_exp(clamp_score(raw) + o.b) : 0.f;
    return s;
  }
  __device__ __forceinline__ void accumulate(float (&acc)[NACC], const Operands& o,
                                             const Scalars& s) const {
    float vf[VEC];
    Vec16<T>::unpack(o.v, vf);
#pragma unroll
    for (int j = 0; j < VEC; ++j) acc[j] = fmaf(s.w, vf[j], acc[j]);
    acc[VEC] += s.w;
  }
  __device__ __forceinline__ void finalize(int row, const float (&acc)[NACC]) const {
    const float inv = 1.0f / (acc[VEC] + kZEps);
    float o[VEC];
#pragma unroll
    for (int j = 0; j < VEC; ++j) o[j] = acc[j] * inv;
    Vec16<T>::store_at(out, unsigned(row) * row_vecs + cvec, o);
    if (z_writer) z[int64_t(row) * heads + head] = acc[VEC];
  }
  __device__ __forceinline__ void zero_row(int row) const {
    float o[VEC];
#pragma unroll
    for (int j = 0; j < VEC; ++j) o[j] = 0.f;
    Vec16<T>::store_at(out, unsigned(row) * row_vecs + cvec, o);
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
  float inv_scale;
  SegWalk walk;
};

template <typename T, int LPH, int G>
__device__ __forceinline__ FwdPolicy<T, LPH, G> make_policy(const FwdParams& p) {
  constexpr int VEC = Vec16<T>::kElems;
  const int c = threadIdx.x % G;
  FwdPolicy<T, LPH, G> pol;
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
  pol.heads = p.heads;
  pol.cvec = blockIdx.y * G + c;
  pol.z_writer = c % LPH == 0;
  pol.inv_scale = p.inv_scale;
  return pol;
}

template <typename T, int LPH, int G>
__global__ void TGT_WALK_BOUNDS fwd_kernel(const FwdParams p) {
  using Policy = FwdPolicy<T, LPH, G>;
  __shared__ TileSmem<G, Policy::NACC> sm;
  const Policy pol = make_policy<T, LPH, G>(p);
  walk_tile_in<G, Policy>(sm, p.walk, pol);
}

template <typename T, int LPH, int G>
__global__ void __launch_bounds__(kBlockThreads) fwd_stitch_kernel(const FwdParams p) {
  using Policy = FwdPolicy<T, LPH, G>;
  const Policy pol = make_policy<T, LPH, G>(p);
  __shared__ float s_part[kBlockThreads * Policy::NACC];
  stitch_tiles<G, Policy>(p.walk, pol, s_part);
}

// Resident CTAs per SM of fwd_kernel<T, LPH, G> for the run-time triple.
int fwd_resident_ctas(int dtype, const HeadSplit& hs) {
  static int cache[kMaxDevices][2][6][6] = {};   // occupancy is a property of the device
  auto log2i = [](int x) { int l = 0; while ((1 << l) < x) ++l; return l; };
  const int dev = current_device();
  int* slot = &cache[dev < 0 ? 0 : dev][dtype == TGT_F32 ? 0 : 1][log2i(hs.lph)][log2i(hs.g)];
  int result = 4;
#define TGT_OCC_FWD(T, LPH, G) result = resident_ctas(fwd_kernel<T, LPH, G>, slot)
  TGT_DISPATCH(dtype, hs.lph, hs.g, TGT_OCC_FWD);
#undef TGT_OCC_FWD
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

size_t fwd_scratch_bytes(const tgt_layout* L, int heads, int head_dim, int dtype) {
  HeadSplit hs;
  if (!split_heads(heads, head_dim, dtype, &hs) || L->n_edges == 0) return 0;
  const int nacc = (dtype == TGT_F32 ? 4 : 8) + 1;
  return plan_tiles(L->n_edges, hs, nacc, fwd_resident_ctas(dtype, hs)).scratch_bytes;
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
  TGT_CHECK_ARG(uint64_t(L.n_rows) * uint64_t(heads) * head_dim * (dtype == TGT_F32 ? 4 : 2) / 16 <
                    (uint64_t(1) << 32),
                "tensors larger than 64 GiB are not supported");
  TGT_CHECK_ARG(aligned16(q) && aligned16(k) && aligned16(v) && aligned16(out) && aligned16(z) &&
                    aligned16(bias) && aligned16(scratch),
                "device pointers must be 16-byte aligned");
  const size_t elem = dtype == TGT_F32 ? 4 : 2;
  if (L.n_edges == 0) {  // no edges: every row is empty
    TGT_CHECK_CUDA(cudaMemsetAsync(out, 0, size_t(L.n_rows) * heads * head_dim * elem, stream));
    TGT_CHECK_CUDA(cudaMemsetAsync(z, 0, size_t(L.n_rows) * heads * 4, stream));
    return TGT_OK;
  }
  const int nacc = (dtype == TGT_F32 ? 4 : 8) + 1;
  const TilePlan tp = plan_tiles(L.n_edges, hs, nacc, fwd_resident_ctas(dtype, hs));
  if (scratch == nullptr || scratch_bytes < tp.scratch_bytes)
    return set_error(TGT_ERR_WORKSPACE, "scratch holds %zu bytes, %zu needed", scratch_bytes,
                     tp.scratch_bytes);

  FwdParams p;
  p.q = q; p.k = k; p.v = v; p.bias = bias; p.bias_heads = bias_heads;
  p.out = out; p.z = z;
  p.heads = heads;
  p.row_elems = heads * head_dim;
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
#define TGT_LAUNCH_FWD(T, LPH, G)                                          \
  do {                                                                     \
    fwd_kernel<T, LPH, G><<<grid, kBlockThreads, 0, stream>>>(p);          \
    if (second_kernel && tp.n_tiles > 1)                                   \
      fwd_stitch_kernel<T, LPH, G><<<grid, kBlockThreads, 0, stream>>>(p); \
  } while (0)
  TGT_DISPATCH(dtype, hs.lph, hs.g, TGT_LAUNCH_FWD);
#undef TGT_LAUNCH_FWD
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
  if (!split_heads(heads, head_dim, dtype, &hs))
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
