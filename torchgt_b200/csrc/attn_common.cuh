// Lane mapping and work assignment shared by the sparse-attention kernels.
//
// A row of Q/K/V/O is heads*head_dim values.  Lanes move 16 bytes each (VEC values), so
//   LPH = head_dim / VEC        lanes cover one head,
//   G   = LPH * heads_per_group lanes cover one "head group" of a row (G <= 32),
// and heads that do not fit one group are walked by blockIdx.y.  Within a warp, LPR >= G lanes
// work on one row (LPR is a run-time power of two), so LPR/G edges of that row are in flight per
// step ("slots") and 32/LPR rows share the warp.
//
// Rows with more than chunk_edges edges are not walked in row mode; their chunks are walked in
// chunk mode (one warp per chunk, LPR = 32) into fp32 partials which a small reduce kernel sums in
// chunk order.  No atomics anywhere, so results are bitwise reproducible.
#pragma once

#include "tgt_common.cuh"

namespace tgt {

constexpr int kWarpsPerBlock = 4;
constexpr int kBlockThreads = kWarpsPerBlock * 32;
constexpr int kUnroll = 4;

struct Walk {
  int row;        // row this lane works on (-1: none)
  int begin;      // first edge position of this lane (already offset by its slot)
  int end;        // one past the last edge position of the row/chunk
  int iters;      // warp-uniform number of steps
  int nslots;     // edges in flight per row per step
  int slot;       // this lane's slot
  int c;          // this lane's 16-byte column inside the head group
  int chunk;      // chunk id in chunk mode, else -1
  bool is_hub;    // row mode: the row is a hub and is handled by chunk mode
};

// Work assignment for one lane.  `lpr_log2` is log2(lanes per row) in row mode.
template <int G>
__device__ __forceinline__ Walk make_walk(const tgt_layout& L, bool chunk_mode, int lpr_log2) {
  Walk w;
  const int lane = threadIdx.x & 31;
  const int warp_global = blockIdx.x * kWarpsPerBlock + (threadIdx.x >> 5);
  w.chunk = -1;
  w.is_hub = false;
  int deg = 0;
  if (chunk_mode) {
    w.nslots = 32 / G;
    w.slot = lane / G;
    w.c = lane % G;
    if (warp_global < L.n_chunks) {
      w.chunk = warp_global;
      w.row = __ldg(L.chunk_row + warp_global);
      const int b = __ldg(L.chunk_begin + warp_global);
      const int row_end = __ldg(L.ptr + w.row + 1);
      w.end = min(b + L.chunk_edges, row_end);
      w.begin = b + w.slot;
      deg = w.end - b;
    } else {
      w.row = -1;
      w.begin = w.end = 0;
    }
  } else {
    const int lpr = 1 << lpr_log2;
    const int rpw = 32 >> lpr_log2;
    const int in_row = lane & (lpr - 1);
    w.nslots = lpr / G;
    w.slot = in_row / G;
    w.c = in_row % G;
    const int64_t row = int64_t(warp_global) * rpw + (lane >> lpr_log2);
    if (row < L.n_rows) {
      w.row = int(row);
      const int b = __ldg(L.ptr + row);
      w.end = __ldg(L.ptr + row + 1);
      deg = w.end - b;
      if (deg > L.chunk_edges) {
        w.is_hub = true;
        deg = 0;
        w.end = b;
      }
      w.begin = b + w.slot;
    } else {
      w.row = -1;
      w.begin = w.end = 0;
    }
  }
  const int steps = (deg + w.nslots - 1) / w.nslots;
  w.iters = __reduce_max_sync(0xffffffffu, steps);
  return w;
}

// Sum over the slots of one row (lanes that hold the same column c); LPR lanes per row.
template <int G>
__device__ __forceinline__ float slot_sum(float x, int lpr) {
#pragma unroll
  for (int off = G; off < 32; off <<= 1) {
    const float t = __shfl_xor_sync(0xffffffffu, x, off);
    if (off < lpr) x += t;
  }
  return x;
}

template <int VEC>
__device__ __forceinline__ float dot(const float (&a)[VEC], const float (&b)[VEC]) {
  float s = 0.f;
#pragma unroll
  for (int j = 0; j < VEC; ++j) s = fmaf(a[j], b[j], s);
  return s;
}

__device__ __forceinline__ float clamp_score(float raw) {
  return fminf(fmaxf(raw, kClampLo), kClampHi);
}

__device__ __forceinline__ bool clamp_passes_grad(float raw) {
  return raw >= kClampLo && raw <= kClampHi;
}

// Host-side choice of lanes per row: enough slots for about half the average degree.
inline int choose_lpr_log2(int G, double avg_degree) {
  int lpr = G;
  while (lpr < 32 && double(lpr / G) * 2.0 < avg_degree) lpr <<= 1;
  int l2 = 0;
  while ((1 << l2) < lpr) ++l2;
  return l2;
}

struct HeadSplit {
  int lph;         // lanes per head
  int hpg;         // heads per group
  int g;           // lanes per group
  int groups;      // number of head groups (gridDim.y)
};

// Returns false when (heads, head_dim, dtype) cannot be mapped onto 16-byte lanes.
inline bool split_heads(int heads, int head_dim, int dtype, HeadSplit* hs) {
  const int vec = dtype == TGT_F32 ? 4 : 8;
  if (heads < 1 || head_dim < vec || head_dim % vec != 0) return false;
  const int lph = head_dim / vec;
  if (lph > 32 || (lph & (lph - 1)) != 0) return false;
  int hpg = 1;
  while (hpg * 2 * lph <= 32 && heads % (hpg * 2) == 0) hpg *= 2;
  hs->lph = lph;
  hs->hpg = hpg;
  hs->g = lph * hpg;
  hs->groups = heads / hpg;
  return true;
}

// Expands to `CALL(T, LPH, G)` for the run-time (dtype, lph, g) triple.
#define TGT_DISPATCH_G(T, LPH, g, CALL)                     \
  switch (g) {                                              \
    case 1: if constexpr (LPH <= 1) { CALL(T, LPH, 1); } break;   \
    case 2: if constexpr (LPH <= 2) { CALL(T, LPH, 2); } break;   \
    case 4: if constexpr (LPH <= 4) { CALL(T, LPH, 4); } break;   \
    case 8: if constexpr (LPH <= 8) { CALL(T, LPH, 8); } break;   \
    case 16: if constexpr (LPH <= 16) { CALL(T, LPH, 16); } break; \
    case 32: if constexpr (LPH <= 32) { CALL(T, LPH, 32); } break; \
    default: break;                                         \
  }

#define TGT_DISPATCH_LPH(T, lph, g, CALL)              \
  switch (lph) {                                       \
    case 1: TGT_DISPATCH_G(T, 1, g, CALL) break;       \
    case 2: TGT_DISPATCH_G(T, 2, g, CALL) break;       \
    case 4: TGT_DISPATCH_G(T, 4, g, CALL) break;       \
    case 8: TGT_DISPATCH_G(T, 8, g, CALL) break;       \
    case 16: TGT_DISPATCH_G(T, 16, g, CALL) break;     \
    case 32: TGT_DISPATCH_G(T, 32, g, CALL) break;     \
    default: break;                                    \
  }

#define TGT_DISPATCH(dtype, lph, g, CALL)                       \
  do {                                                          \
    if ((dtype) == TGT_F32) {                                   \
      TGT_DISPATCH_LPH(float, lph, g, CALL)                     \
    } else {                                                    \
      TGT_DISPATCH_LPH(__nv_bfloat16, lph, g, CALL)             \
    }                                                           \
  } while (0)

int check_layout(const tgt_layout* L, const char* name);

}  // namespace tgt
