// Backward of the sparse graph attention: two passes without floating-point atomics that recompute the scores.
//   pass A: edges sorted by destination -> dQ, and the row statistics
//           stats[d,h] = { inv_d = 1/(Z+1e-6), delta_d = dO_d . O_d } that pass B reads
//   pass B: edges sorted by source      -> dK and dV
// Pass A needs delta_d before the row is complete.  Because O_d = inv_d * sum_e w_e V_s,
// delta_d = inv_d * sum_e w_e (dO_d . V_s) is a sum over the same edges, so the pass accumulates
//   A1 = sum mask w (dO.V) K,  A2 = sum mask w K,  S = sum w (dO.V)
// and finishes the row with delta = inv S, dQ = inv (A1 - delta A2) / sqrt(D): no separate statistics
// pass and no read of O.  Only when dbias is wanted (it needs delta per edge) a streaming pre-pass
// computes the statistics from dO and O first and pass A uses them per edge.
// With G = dO, inv = 1/(Z+1e-6), w = exp(clamp(raw)+bias):
//   dw = (G_d.V_s - G_d.O_d) * inv_d      dV_s += w * inv_d * G_d      dt = dw * w  (= dbias)
//   da = dt * [-5 <= raw <= 5]            dQ_d += da * K_s / sqrt(D)   dK_s += da * Q_d / sqrt(D)
//
// This header holds what the three passes share; each pass's kernels are instantiated in a translation
// unit of their own (sparse_attn_bwd_dq.cu, sparse_attn_bwd_dq_fused.cu, sparse_attn_bwd_dkv.cu) so that
// they compile side by side, and sparse_attn_bwd.cu holds the entry points.
#pragma once

#include "attn_common.cuh"

namespace tgt {
namespace bwd {

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
  int heads, row_elems;
  int64_t q_row_bytes, kv_row_bytes, g_row_bytes;   // distance between rows of q, of k / v and of dout
  int64_t n_rows;
  float inv_scale;
  int* clear_words;      // arrival counters the statistics pre-pass zeroes for the two walks (or null)
  int n_clear_words;
  SegWalk walk;
};

// What sparse_attn_bwd.cu asks of each pass: launch it (plus the kernel that finishes cross-tile rows when
// `second_kernel`; `link` != 0 = the kernel enqueued just before on the stream belongs to the same call, so
// the walk kernel is launched as its dependent, see launch_chained), and the resident CTAs per SM of its walk kernel.  Both return false / 0 when no kernel
// is built for the lane layout.
bool launch_dq(const BwdParams& p, int dtype, const HeadSplit& hs, dim3 grid, bool second_kernel, int link,
               cudaStream_t stream);
bool launch_dq_fused(const BwdParams& p, int dtype, const HeadSplit& hs, dim3 grid, bool second_kernel, int link,
                     cudaStream_t stream);
bool launch_dkv(const BwdParams& p, int dtype, const HeadSplit& hs, dim3 grid, bool second_kernel, int link,
                cudaStream_t stream);
int occupancy_dq(int dtype, const HeadSplit& hs, int* cache_slot);
int occupancy_dq_fused(int dtype, const HeadSplit& hs, int* cache_slot);
int occupancy_dkv(int dtype, const HeadSplit& hs, int* cache_slot);

}  // namespace bwd
}  // namespace tgt
