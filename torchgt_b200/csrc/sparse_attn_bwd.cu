// Entry points of the backward of the sparse graph attention: argument checks, scratch planning, the
// streaming row-statistics pre-pass, and the launches of the three passes (sparse_attn_bwd.cuh).
#include "sparse_attn_bwd.cuh"

namespace tgt {
namespace {

using bwd::BwdParams;

// ---- row statistics ---------------------------------------------------------------------------
// One lane per 16-byte chunk of a row; the LPH lanes of a head are adjacent.
template <typename T, int LPH>
__global__ void __launch_bounds__(256) bwd_stats_kernel(const BwdParams p) {
  constexpr int VEC = Vec16<T>::kElems;
  const int64_t idx = blockIdx.x * int64_t(blockDim.x) + threadIdx.x;
  const int chunks = p.row_elems / VEC;
  const int64_t total = p.n_rows * chunks;
  const bool live = idx < total;
  release_dependents();   // pass A stages its edge indices while this kernel drains
  // the arrival counters of both walks, which start only after this kernel has completed: saves the memset
  // node in front of the call
  if (blockIdx.x == 0 && p.clear_words != nullptr)
    for (int i = threadIdx.x; i < p.n_clear_words; i += blockDim.x) p.clear_words[i] = 0;
  float g[VEC], o[VEC];
#pragma unroll
  for (int j = 0; j < VEC; ++j) g[j] = o[j] = 0.f;
  if (live) {
    const int64_t row = idx / chunks, col = idx % chunks;
    Vec16<T>::load(reinterpret_cast<const T*>(static_cast<const char*>(p.dout) + row * p.g_row_bytes) + col * VEC, g);
    Vec16<T>::load(static_cast<const T*>(p.out) + idx * VEC, o);
  }
  const float delta = group_sum<LPH>(dot<VEC>(g, o));
  if (live && (idx % LPH) == 0) {
    const int64_t row = idx / chunks;
    const int head = int(idx % chunks) / LPH;
    const float zr = __ldg(p.z + row * p.heads + head);
    p.stats[row * p.heads + head] = make_float2(1.0f / (zr + kZEps), delta);
  }
}

enum { kWalkDq = 0, kWalkDkv = 1, kWalkDqFused = 2 };

int bwd_resident_ctas(int dtype, const HeadSplit& hs, int which) {
  static int cache[kMaxDevices][2][3][2][6][6] = {};   // occupancy is a property of the device
  auto log2i = [](int x) { int l = 0; while ((1 << l) < x) ++l; return l; };
  const int dev = current_device();
  int* slot = &cache[dev < 0 ? 0 : dev][hs.w == 32 ? 1 : 0][which][dtype == TGT_F32 ? 0 : 1][log2i(hs.lph)][log2i(hs.g)];
  if (which == kWalkDkv) return bwd::occupancy_dkv(dtype, hs, slot);
  if (which == kWalkDqFused) return bwd::occupancy_dq_fused(dtype, hs, slot);
  return bwd::occupancy_dq(dtype, hs, slot);
}

struct BwdScratch {
  size_t stats, carry_a, carry_b, counters, counter_bytes, total;
  TilePlan plan_a, plan_a_fused, plan_b;
};

// hs: lane layout of pass A (by destination), hsb: of pass B (by source); they may use different lane widths
BwdScratch plan_bwd_scratch(const tgt_layout* by_dst, const HeadSplit& hs, const HeadSplit& hsb, int heads,
                            int dtype) {
  BwdScratch s;
  const int vec = hs.w / (dtype == TGT_F32 ? 4 : 2);
  const int vecb = hsb.w / (dtype == TGT_F32 ? 4 : 2);
  s.plan_a = plan_tiles(by_dst->n_edges, hs, vec, bwd_resident_ctas(dtype, hs, kWalkDq));
  s.plan_a_fused = plan_tiles(by_dst->n_edges, hs, 2 * vec + 1, bwd_resident_ctas(dtype, hs, kWalkDqFused));
  s.plan_b = plan_tiles(by_dst->n_edges, hsb, 2 * vecb, bwd_resident_ctas(dtype, hsb, kWalkDkv));
  size_t off = 0;
  s.stats = off; off += round_up(size_t(by_dst->n_rows) * heads * 8, 256);
  s.carry_a = off;
  off += s.plan_a.carry_bytes > s.plan_a_fused.carry_bytes ? s.plan_a.carry_bytes : s.plan_a_fused.carry_bytes;
  s.carry_b = off; off += s.plan_b.carry_bytes;
  // arrival counters of both passes side by side (one memset clears them): pass A first
  s.counters = off;
  const size_t ca = s.plan_a.counter_bytes > s.plan_a_fused.counter_bytes ? s.plan_a.counter_bytes
                                                                           : s.plan_a_fused.counter_bytes;
  s.counter_bytes = ca + s.plan_b.counter_bytes;
  off += s.counter_bytes;
  s.total = off;
  return s;
}

void fill_walk(SegWalk* w, const tgt_layout& L, const TilePlan& tp, float* carry, int* counters,
               bool need_perm) {
  w->ptr = L.ptr; w->other = L.other; w->perm = L.perm; w->seg = L.seg;
  w->n_rows = int(L.n_rows); w->n_edges = int(L.n_edges);
  w->ge = tp.ge; w->n_tiles = tp.n_tiles;
  w->gcarry = carry;
  w->tile_done = counters;
  w->need_perm = need_perm;
}

}  // namespace

size_t fwd_scratch_bytes(const tgt_layout* L, int heads, int head_dim, int dtype);

}  // namespace tgt

extern "C" int tgt_sparse_attn_scratch_bytes(const tgt_layout* by_dst, const tgt_layout* by_src,
                                             int heads, int head_dim, int dtype, int phase,
                                             size_t* bytes) {
  using namespace tgt;
  TGT_CHECK_ARG(bytes != nullptr, "bytes is null");
  TGT_CHECK_ARG(phase == 0 || phase == 1, "phase must be 0 (forward) or 1 (backward)");
  TGT_CHECK_ARG(dtype == TGT_F32 || dtype == TGT_BF16, "dtype must be TGT_F32 or TGT_BF16");
  int rc = check_layout(by_dst, "by_dst");
  if (rc != TGT_OK) return rc;
  HeadSplit hs;
  if (!split_heads(heads, head_dim, dtype, 16, &hs))
    return set_error(TGT_ERR_UNSUPPORTED, "heads=%d head_dim=%d dtype=%d is not supported", heads,
                     head_dim, dtype);
  if (phase == 0) {
    *bytes = fwd_scratch_bytes(by_dst, heads, head_dim, dtype);
    return TGT_OK;
  }
  rc = check_layout(by_src, "by_src");
  if (rc != TGT_OK) return rc;
  // enough for whichever lane width the call ends up using (it depends on pointer alignment)
  size_t need = 0;
  for (int wa = 16; wa <= 32; wa += 16)
    for (int wb = 16; wb <= 32; wb += 16) {
      HeadSplit a, b;
      if ((wa == 32 && lane_bytes(heads, head_dim, dtype, true, kPassDq) != 32) ||
          (wb == 32 && lane_bytes(heads, head_dim, dtype, true, kPassDkv) != 32))
        continue;
      if (!split_heads(heads, head_dim, dtype, wa, &a) || !split_heads(heads, head_dim, dtype, wb, &b)) continue;
      const size_t t = plan_bwd_scratch(by_dst, a, b, heads, dtype).total;
      if (t > need) need = t;
    }
  *bytes = need;
  return TGT_OK;
}

extern "C" int tgt_sparse_attn_bwd(const void* dout, const void* q, const void* k, const void* v,
                                   const float* bias, int bias_heads, const void* out,
                                   const float* z, const tgt_layout* by_dst,
                                   const tgt_layout* by_src, void* dq, void* dk, void* dv,
                                   float* dbias, int heads, int head_dim, int dtype, void* scratch,
                                   size_t scratch_bytes, void* stream) {
  // the statistics pre-pass is only needed when dbias is wanted
  return tgt_sparse_attn_bwd_passes(dout, q, k, v, bias, bias_heads, out, z, by_dst, by_src, dq, dk,
                                    dv, dbias, heads, head_dim, dtype, scratch, scratch_bytes, stream,
                                    dbias != nullptr ? 7 : 6);
}

extern "C" int tgt_sparse_attn_bwd_passes(const void* dout, const void* q, const void* k,
                                          const void* v, const float* bias, int bias_heads,
                                          const void* out, const float* z, const tgt_layout* by_dst,
                                          const tgt_layout* by_src, void* dq, void* dk, void* dv,
                                          float* dbias, int heads, int head_dim, int dtype,
                                          void* scratch, size_t scratch_bytes, void* stream,
                                          int passes) {
  TGT_CHECK_ARG(passes >= 1 && passes <= 7,
                "passes is a bit mask: 1 = row-statistics pre-pass, 2 = dQ/dbias, 4 = dK/dV");
  const int64_t row_bytes = int64_t(heads) * head_dim * (dtype == TGT_F32 ? 4 : 2);
  return tgt_sparse_attn_bwd_strided(dout, row_bytes, q, row_bytes, k, v, row_bytes, bias, bias_heads,
                                     out, z, by_dst, by_src, dq, dk, dv, dbias, heads, head_dim, dtype,
                                     scratch, scratch_bytes, stream, passes);
}

extern "C" int tgt_sparse_attn_bwd_strided(const void* dout, int64_t dout_row_bytes, const void* q,
                                           int64_t q_row_bytes, const void* k, const void* v,
                                           int64_t kv_row_bytes, const float* bias, int bias_heads,
                                           const void* out, const float* z, const tgt_layout* by_dst,
                                           const tgt_layout* by_src, void* dq, void* dk, void* dv,
                                           float* dbias, int heads, int head_dim, int dtype,
                                           void* scratch, size_t scratch_bytes, void* stream_,
                                           int passes) {
  using namespace tgt;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  if (passes == 0) passes = dbias != nullptr ? 7 : 6;
  TGT_CHECK_ARG(passes >= 1 && passes <= 7,
                "passes is a bit mask: 1 = row-statistics pre-pass, 2 = dQ/dbias, 4 = dK/dV (0 = all that are needed)");
  TGT_CHECK_ARG(dtype == TGT_F32 || dtype == TGT_BF16, "dtype must be TGT_F32 or TGT_BF16");
  int rc = check_layout(by_dst, "by_dst");
  if (rc != TGT_OK) return rc;
  rc = check_layout(by_src, "by_src");
  if (rc != TGT_OK) return rc;
  TGT_CHECK_ARG(by_dst->n_rows == by_src->n_rows && by_dst->n_edges == by_src->n_edges,
                "by_dst and by_src describe different graphs");
  const bool can32 = aligned32(dout) && aligned32(q) && aligned32(k) && aligned32(v) && aligned32(dq) &&
                     aligned32(dk) && aligned32(dv) && dout_row_bytes % 32 == 0 && q_row_bytes % 32 == 0 &&
                     kv_row_bytes % 32 == 0;
  HeadSplit hs, hsb;   // lane layouts of pass A (dQ) and pass B (dK/dV)
  if (!split_heads(heads, head_dim, dtype, lane_bytes(heads, head_dim, dtype, can32, kPassDq), &hs) ||
      !split_heads(heads, head_dim, dtype, lane_bytes(heads, head_dim, dtype, can32, kPassDkv), &hsb))
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
  const int64_t n_rows = by_dst->n_rows, n_edges = by_dst->n_edges;
  if (n_rows == 0) return TGT_OK;
  const size_t elem = dtype == TGT_F32 ? 4 : 2;
  const int64_t row_bytes = int64_t(heads) * head_dim * int64_t(elem);
  TGT_CHECK_ARG(dout && q && k && v && z && dq && dk && dv, "tensor pointers must not be null");
  TGT_CHECK_ARG(out != nullptr || !(passes & 1), "out is needed by the row-statistics pre-pass (dbias)");
  TGT_CHECK_ARG(dout_row_bytes >= row_bytes && q_row_bytes >= row_bytes && kv_row_bytes >= row_bytes &&
                    dout_row_bytes % 16 == 0 && q_row_bytes % 16 == 0 && kv_row_bytes % 16 == 0,
                "row strides must be multiples of 16 bytes and at least heads * head_dim elements");
  int64_t widest = dout_row_bytes > q_row_bytes ? dout_row_bytes : q_row_bytes;
  if (kv_row_bytes > widest) widest = kv_row_bytes;
  TGT_CHECK_ARG(uint64_t(n_rows) * uint64_t(widest) / 16 < (uint64_t(1) << 32),
                "tensors larger than 64 GiB are not supported");
  TGT_CHECK_ARG(aligned16(dout) && aligned16(q) && aligned16(k) && aligned16(v) && aligned16(out) &&
                    aligned16(z) && aligned16(dq) && aligned16(dk) && aligned16(dv) &&
                    aligned16(bias) && aligned16(dbias) && aligned16(scratch),
                "device pointers must be 16-byte aligned");
  const size_t tensor_bytes = size_t(n_rows) * heads * head_dim * elem;
  if (n_edges == 0) {  // no edges: all gradients vanish
    if (passes & 2) TGT_CHECK_CUDA(cudaMemsetAsync(dq, 0, tensor_bytes, stream));
    if (passes & 4) {
      TGT_CHECK_CUDA(cudaMemsetAsync(dk, 0, tensor_bytes, stream));
      TGT_CHECK_CUDA(cudaMemsetAsync(dv, 0, tensor_bytes, stream));
    }
    return TGT_OK;
  }
  const BwdScratch sc = plan_bwd_scratch(by_dst, hs, hsb, heads, dtype);
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
  p.q_row_bytes = q_row_bytes;
  p.kv_row_bytes = kv_row_bytes;
  p.g_row_bytes = dout_row_bytes;
  p.n_rows = n_rows;
  p.inv_scale = 1.0f / sqrtf(float(head_dim));

  const bool second_kernel = stitch_in_second_kernel(hs.g);      // pass A
  const bool second_kernel_b = stitch_in_second_kernel(hsb.g);   // pass B
  int* counters_a = second_kernel ? nullptr : reinterpret_cast<int*>(base + sc.counters);
  int* counters_b = second_kernel_b ? nullptr
                                    : reinterpret_cast<int*>(base + sc.counters + sc.counter_bytes -
                                                             sc.plan_b.counter_bytes);
  p.clear_words = nullptr;
  p.n_clear_words = 0;
  if ((passes & 6) && !(second_kernel && second_kernel_b)) {
    if (passes & 1) {   // the statistics kernel clears them on its way
      p.clear_words = reinterpret_cast<int*>(base + sc.counters);
      p.n_clear_words = int(sc.counter_bytes / sizeof(int));
    } else {
      TGT_CHECK_CUDA(cudaMemsetAsync(base + sc.counters, 0, sc.counter_bytes, stream));
    }
  }
  // from here on the kernels of this call follow one another on the stream without anything in between, and
  // each is launched as the dependent of the one before
  int link = 0;
  if (passes & 1) {
    // streaming pre-pass, always with 16-byte lanes
    const int lph16 = head_dim / (dtype == TGT_F32 ? 4 : 8);
    const int64_t lanes = n_rows * (p.row_elems / (dtype == TGT_F32 ? 4 : 8));
    const unsigned blocks = unsigned((lanes + 255) / 256);
    dispatch_shape(dtype, 16, lph16, lph16, [&](auto sh) {
      using S = decltype(sh);
      bwd_stats_kernel<typename S::T, S::LPH><<<blocks, 256, 0, stream>>>(p);
    });
    link = kLinkWalk;
  }
  // one walk kernel per pass, plus the kernel that finishes cross-tile rows when the lane group is narrow
  bool built = true;
  if ((passes & 2) && dbias == nullptr) {
    // pass A that derives the row statistics itself (and leaves them in scratch for pass B)
    fill_walk(&p.walk, *by_dst, sc.plan_a_fused, reinterpret_cast<float*>(base + sc.carry_a), counters_a,
              bias != nullptr);
    const dim3 grid(sc.plan_a_fused.n_tiles, hs.groups);
    built = bwd::launch_dq_fused(p, dtype, hs, grid, second_kernel, link, stream);
    link = second_kernel && grid.x > 1 ? kLinkAfterStitch : kLinkWalk;
  } else if (passes & 2) {
    // pass A with per-edge dbias: uses the statistics of the pre-pass (stage 1)
    fill_walk(&p.walk, *by_dst, sc.plan_a, reinterpret_cast<float*>(base + sc.carry_a), counters_a, true);
    const dim3 grid(sc.plan_a.n_tiles, hs.groups);
    built = bwd::launch_dq(p, dtype, hs, grid, second_kernel, link, stream);
    link = second_kernel && grid.x > 1 ? kLinkAfterStitch : kLinkWalk;
  }
  if (built && (passes & 4)) {
    fill_walk(&p.walk, *by_src, sc.plan_b, reinterpret_cast<float*>(base + sc.carry_b), counters_b,
              bias != nullptr);
    const dim3 grid(sc.plan_b.n_tiles, hsb.groups);
    built = bwd::launch_dkv(p, dtype, hsb, grid, second_kernel_b, link, stream);
  }
  if (!built) return set_error(TGT_ERR_UNSUPPORTED, "no kernel is built for this head layout");
  TGT_CHECK_CUDA(cudaGetLastError());
  return TGT_OK;
}
