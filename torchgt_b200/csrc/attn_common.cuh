// Edge-balanced segmented reduction shared by the three sparse-attention kernels.
//
// Lanes move 16 bytes of a row each (VEC values): LPH = head_dim / VEC lanes cover one head and
// G = LPH * heads_per_group lanes ("lane group") cover the heads one CTA column handles; heads that
// do not fit 32 lanes are walked by blockIdx.y.
//
// The edges, sorted by the grouping endpoint ("row"), are cut into tiles of NG * ge consecutive
// edges, one CTA per tile, NG = 128 / G lane groups per CTA.  Lane group g walks ge consecutive
// edges, kUnroll at a time: all gathers of a batch are issued before any arithmetic.  Edge
// positions, not rows, are what is divided, so a row with 100,000 edges and a row with one edge
// cost the same per edge and every lane group does the same amount of work.
//
// A row whose edges lie inside one lane group's range is finished by that group and written once.
// A row that crosses a range boundary leaves partial sums in shared memory ("head" = the range
// starts inside the row, "tail" = the row starts here and runs past the range); after a barrier
// the group that holds the tail adds the heads of the following groups in order.  If the row
// also crosses the tile boundary the CTA writes its sum to a per-tile carry in global memory and
// counts itself in on the row's arrival counter; the CTA that arrives last adds the carries in tile
// order and finishes the row (nobody waits for anybody).  Every sum has a fixed order whichever CTA
// does it: no floating-point atomics, bitwise reproducible results.  Rows without edges are
// zero-filled by the group that walks the gap.
#pragma once

#include <type_traits>

#include "tgt_common.cuh"

namespace tgt {

// Build-time tuning knobs (defaults are what the measurements in the repository use).
#ifndef TGT_UNROLL
#define TGT_UNROLL 4
#endif
// Lane groups up to this width finish the rows that cross tiles in a second kernel; wider ones do it
// inside the walk kernel (the last tile to arrive).  Narrow groups have many small tiles (a thread
// walks 32 edges at G = 2), where the fence and the arrival count of every CTA cost more than one
// extra launch.
#ifndef TGT_STITCH_KERNEL_MAX_G
#define TGT_STITCH_KERNEL_MAX_G 4
#endif
// Which walks use 32-byte lanes when nobody forces a lane width (see lane_bytes()).  Measured on B200
// (fp32, 8-float heads, 64K-node batches and their 2-, 4- and 8-rank head slices, 870K-node batch): the
// forward gains on 128-byte rows (55 -> 50 us), the dQ pass on 64- and 128-byte rows (86 -> 80 us,
// 72 -> 62 us).  On 256-byte rows they tie at 64K nodes and lose 4-5 % at 870K nodes, where K and V no
// longer fit the L2 and the higher occupancy of the 16-byte-lane kernels (64-72 registers) counts; both
// lose on 32-byte rows, and the dK/dV pass, with twice the accumulators per lane, loses 10-40 % everywhere.
#ifndef TGT_WIDE_DEFAULT
#define TGT_WIDE_DEFAULT(pass, row_bytes) \
  ((pass) != kPassDkv && (row_bytes) <= 128 && (row_bytes) >= ((pass) == kPassDq ? 64 : 128))
#endif
// Edges per batch of the walk with 32-byte lanes (their operands take twice the registers).
#ifndef TGT_WIDE_UNROLL
#define TGT_WIDE_UNROLL 2
#endif
#ifdef TGT_MIN_CTAS
#define TGT_WALK_BOUNDS __launch_bounds__(128, TGT_MIN_CTAS)
#else
#define TGT_WALK_BOUNDS __launch_bounds__(128)
#endif

constexpr int kBlockThreads = 128;
constexpr int kUnroll = TGT_UNROLL;  // edges per lane group whose gathers are in flight together
constexpr int kGeStep = 4;           // ge is a multiple of this (and of every batch size below)

// Batch size of the walk for element type T and lane-group width G.  Measured on B200 (fp32, 8-byte to
// 256-byte rows; bf16 128-byte rows): batches of 4 edges are best everywhere except for fp32 rows of
// 16 lanes (the 8 heads x 8 case, two lane groups per warp), where batches of 2 are 9-10 % faster
// (64K benchmark step 176 -> 158 us, 870K step 5.11 -> 4.67 ms); narrower groups lose 20-70 % with 2.
template <typename T, int W, int G>
constexpr int walk_unroll() {
  if (W == 32) return TGT_WIDE_UNROLL;
  return (std::is_same<T, float>::value && G == 16 && TGT_UNROLL == 4) ? 2 : TGT_UNROLL;
}
static_assert(kGeStep % TGT_WIDE_UNROLL == 0, "ge must stay a multiple of the batch size");
static_assert(kGeStep % TGT_UNROLL == 0, "ge must stay a multiple of the batch size");

template <int G>
struct TileGeom {
  static constexpr int NG = kBlockThreads / G;  // lane groups per CTA
  static constexpr int GE_MAX = (2048 / NG) > 128 ? 128 : ((2048 / NG) < 8 ? 8 : (2048 / NG));
  static constexpr int TE_MAX = NG * GE_MAX;    // most edges a tile can hold
};

// What every kernel needs to walk the edges.
struct SegWalk {
  const int32_t* ptr;
  const int32_t* other;
  const int32_t* perm;
  const int32_t* seg;
  int n_rows;
  int n_edges;
  int ge;          // edges per lane group per tile (multiple of kGeStep, <= GE_MAX)
  int n_tiles;
  float* gcarry;   // [n_tiles][2][gridDim.y * G * NACC] cross-tile partial sums
  int* tile_done;  // [gridDim.y][n_tiles] arrivals per row that crosses tiles, indexed by the tile it
                   // starts in; zero when the kernel starts.  Null: a second kernel finishes those rows
  bool need_perm;  // stage perm[] (bias or dbias in original edge order)
};

inline int host_ge_max(int g) {
  const int ng = kBlockThreads / g;
  int m = 2048 / ng;
  return m > 128 ? 128 : (m < 8 ? 8 : m);
}

// Edges per lane group: one balanced wave over the GPU when the graph is small enough, else the
// largest tile.  `ctas_per_sm` is the occupancy the caller expects.
int forced_ge();  // 0 unless tgt_debug_set_tile_edges() overrides the choice

inline int choose_ge(int64_t n_edges, int g, int ctas_per_sm) {
  const int ng = kBlockThreads / g;
  const int ge_max = host_ge_max(g);
  if (forced_ge() > 0) {
    int f = (forced_ge() + kGeStep - 1) / kGeStep * kGeStep;
    return f > ge_max ? ge_max : f;
  }
  // Time is roughly (number of CTA waves) x (work of one tile); a tile costs its ge edges per lane
  // group plus a fixed part (index staging, barriers, stitching) worth about 8 edges.  Few, full
  // waves win; with many waves the tail does not matter and larger tiles amortise the fixed part.
  const int64_t capacity = int64_t(sm_count()) * ctas_per_sm;
  int best = ge_max;
  double best_cost = 1e300;
  for (int ge = (ge_max < 16 ? ge_max : 16); ge <= ge_max; ge += kGeStep) {
    const int64_t tiles = (n_edges + int64_t(ng) * ge - 1) / (int64_t(ng) * ge);
    const int64_t waves = (tiles + capacity - 1) / capacity;
    const double cost = double(waves) * (ge + 8);
    if (cost < best_cost - 1e-9) {
      best_cost = cost;
      best = ge;
    }
  }
  return best;
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

// torch.clamp passes the gradient where the input lies inside [lo, hi], bounds included
__device__ __forceinline__ bool clamp_passes_grad(float raw) {
  return raw >= kClampLo && raw <= kClampHi;
}

// Sum of a per-head value (replicated on the LPH lanes of each head) over the heads of a lane group.
template <int LPH, int G>
__device__ __forceinline__ float sum_over_heads(float x) {
#pragma unroll
  for (int off = LPH; off < G; off <<= 1) x += __shfl_xor_sync(0xffffffffu, x, off);
  return x;
}

// exp(x) for |x| < 80: ex2.approx on the rounded product x*log2(e), corrected for the rounding error
// of that product with one fma (relative error about 2^-22, like expf).  Building with
// -DTGT_EXP_CORRECT=0 drops the correction: four instructions per edge and lane fewer (the 64K
// benchmark step goes from 176 to 170 us), relative error |x| * 1.44 * 2^-24 * ln 2 + 2^-22, i.e. below
// 6e-7 for clamped scores and 5e-6 at |x| = 80; the op-level parity tests still pass with it, but
// gradients that cancel heavily (key-bias gradients of a whole model) move by more than 1e-4.
#ifndef TGT_EXP_CORRECT
#define TGT_EXP_CORRECT 1
#endif
__device__ __forceinline__ float fast_exp(float x) {
  constexpr float kLog2eHi = 1.4426950216293335f;   // log2(e) rounded to fp32
  const float t = x * kLog2eHi;
  float e;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e) : "f"(t));
#if TGT_EXP_CORRECT
  constexpr float kLog2eLo = 1.9259629911e-8f;      // log2(e) - kLog2eHi
  constexpr float kLn2 = 0.6931471805599453f;
  const float r = fmaf(x, kLog2eHi, -t) + x * kLog2eLo;  // what the product lost
  e = fmaf(e, r * kLn2, e);
#endif
  return e;
}

template <int G, class Policy>
__device__ __forceinline__ void finish_row(const SegWalk& w, const Policy& pol, float* s_part, int tile);

// The walk.  Policy supplies:
//   static constexpr int NACC;                     accumulators per lane
//   static constexpr int kUnroll;                  edges per batch (walk_unroll<T, G>())
//   struct Operands;                               what one edge loads
//   void load(Operands&, int row, int other, int perm_e) const;      issue the gathers of one edge
//   void clear(Operands&) const;                                     operands of a padding slot
//   Scalars prep(const Operands&, bool valid, int perm_e) const;     warp-uniform part (shuffles)
//   void accumulate(float (&acc)[NACC], const Operands&, const Scalars&) const;
//   void finalize(int row, const float (&acc)[NACC]) const;          write the finished row
//   void zero_row(int row) const;                                    row without edges
template <int G, class Policy>
__device__ __forceinline__ void walk_tile(const SegWalk& w, const Policy& pol, int32_t* s_other,
                                          int32_t* s_seg, int32_t* s_perm, float* s_carry,
                                          int32_t* s_carry_row, float* s_part, int32_t* s_finish) {
  constexpr int NG = TileGeom<G>::NG;
  constexpr int NACC = Policy::NACC;
  constexpr int kUnroll = Policy::kUnroll;   // edges per batch (shadows the default)
  const int tid = threadIdx.x;
  const int g = tid / G;        // lane group inside the CTA
  const int c = tid % G;        // 16-byte column inside the group
  const int te = NG * w.ge;
  const int64_t t0 = int64_t(blockIdx.x) * te;
  const int n = int(min(int64_t(te), int64_t(w.n_edges) - t0));  // edges in this tile (>= 1)
  release_dependents();   // the next kernel of the call may take this SM's slots as they free up

  // ---- stage the tile's indices.  Tile edge i lives at position i + i / ge: one pad word per
  // lane-group range, so the groups of a warp (which read ranges ge apart) hit different banks.
  // The rows of the edge before and after the tile go to the two words behind the padded array.
  const int ge = w.ge;
  auto pos = [ge](int i) { return i + i / ge; };
  int32_t* s_halo = s_seg + TileGeom<G>::TE_MAX + NG;   // [0] = row before the tile, [1] = row after
  for (int i = tid; i < n; i += kBlockThreads) {
    const int p = pos(i);
    s_seg[p] = __ldg(w.seg + t0 + i);
    s_other[p] = __ldg(w.other + t0 + i);
    if (w.need_perm) s_perm[p] = __ldg(w.perm + t0 + i);
  }
  if (tid == 0) {
    s_halo[0] = t0 == 0 ? -1 : __ldg(w.seg + t0 - 1);
    s_halo[1] = t0 + n >= w.n_edges ? -2 : __ldg(w.seg + t0 + n);
  }
  for (int i = tid; i < 2 * NG; i += kBlockThreads) s_carry_row[i] = -3;  // [g][0] head row, [g][1] tail row
  // the indices are the layout's, complete long before this call; everything below reads or overwrites what
  // the previous kernel of the call works on
  dependent_wait();
  __syncthreads();

  // ---- walk this group's range [gb, ge) of the tile
  const int gb = min(g * w.ge, n);
  const int gend = min(gb + w.ge, n);
  float acc[NACC];
#pragma unroll
  for (int a = 0; a < NACC; ++a) acc[a] = 0.f;
  // row of tile edge i, for i in [-1, n]
  auto row_of = [&](int i) { return i < 0 ? s_halo[0] : (i >= n ? s_halo[1] : s_seg[pos(i)]); };
  int cur = row_of(gb - 1);                          // row of the edge just before the range
  bool own = gb < gend && row_of(gb) == cur;         // the range starts inside row `cur`
  const int gb_pos = pos(gb);                        // the range is contiguous in padded positions
  bool head_pending = own;
  float* my_head = s_carry + (g * 2 + 0) * (G * NACC) + c * NACC;
  float* my_tail = s_carry + (g * 2 + 1) * (G * NACC) + c * NACC;

  // State of the segmented walk, advanced one batch of kUnroll edges at a time.  FULL = every
  // slot of the batch holds an edge of this group's range (all tiles but the last one).
  auto batch = [&](int first, auto full_tag) {
    constexpr bool FULL = decltype(full_tag)::value;
    typename Policy::Operands ops[kUnroll];
    int row[kUnroll], pe[kUnroll];
    bool valid[kUnroll];
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      const int i = first + u;
      valid[u] = FULL || i < gend;
      const int ii = valid[u] ? gb_pos + (i - gb) : 0;
      row[u] = s_seg[ii];
      pe[u] = w.need_perm ? s_perm[ii] : 0;
      if (valid[u]) pol.load(ops[u], row[u], s_other[ii], pe[u]);
      else pol.clear(ops[u]);
    }
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      const typename Policy::Scalars sc = pol.prep(ops[u], valid[u], pe[u]);
      if (valid[u]) {
        if (row[u] != cur) {
          if (own) {
            if (head_pending) {
#pragma unroll
              for (int a = 0; a < NACC; ++a) my_head[a] = acc[a];
              if (c == 0) s_carry_row[g * 2 + 0] = cur;
            } else {
              pol.finalize(cur, acc);
            }
          }
          head_pending = false;
          for (int r = cur + 1; r < row[u]; ++r) pol.zero_row(r);
          cur = row[u];
          own = true;
#pragma unroll
          for (int a = 0; a < NACC; ++a) acc[a] = 0.f;
        }
        pol.accumulate(acc, ops[u], sc);
      }
    }
  };
  if (n == te) {
    // ge is a multiple of the batch size, so every batch of every group is full
    for (int first = gb; first < gend; first += kUnroll) batch(first, std::true_type{});
  } else {
    // last tile: all groups of a warp run the same number of batches (the shuffles inside need
    // the full warp), slots past the group's range are padding
    const int warp_first_group = (tid / 32) * (32 / G);
    const int warp_gb = min(warp_first_group * w.ge, n);
    const int batches = (min(w.ge, n - warp_gb) + kUnroll - 1) / kUnroll;
    for (int b = 0; b < batches; ++b) batch(gb + b * kUnroll, std::false_type{});
  }
  if (gb < gend) {  // close the last row of the range
    const bool cont_out = row_of(gend) == cur;
    if (head_pending) {
#pragma unroll
      for (int a = 0; a < NACC; ++a) my_head[a] = acc[a];
      if (c == 0) s_carry_row[g * 2 + 0] = cur;
    } else if (cont_out) {
#pragma unroll
      for (int a = 0; a < NACC; ++a) my_tail[a] = acc[a];
      if (c == 0) s_carry_row[g * 2 + 1] = cur;
    } else {
      pol.finalize(cur, acc);
    }
    if (t0 + gend == w.n_edges)  // this group owns the last edge: rows after it have no edges
      for (int r = cur + 1; r < w.n_rows; ++r) pol.zero_row(r);
  }
  __syncthreads();

  // ---- stitch rows that cross group boundaries, in group order
  const int last_row = row_of(n - 1);       // row of the tile's last edge
  const bool tile_cont_out = s_halo[1] == last_row;
  const int lanes_all = gridDim.y * G;
  float* tile_carry = w.gcarry + (int64_t(blockIdx.x) * 2) * (int64_t(lanes_all) * NACC) +
                      int64_t(blockIdx.y * G + c) * NACC;
  if (g == 0 && s_halo[0] == row_of(0)) {
    // the tile starts inside a row that began in an earlier tile: sum its heads into the tile's
    // head carry
    const int r = row_of(0);
#pragma unroll
    for (int a = 0; a < NACC; ++a) acc[a] = 0.f;
    for (int j = 0; j < NG && s_carry_row[j * 2] == r; ++j) {
      const float* h = s_carry + (j * 2) * (G * NACC) + c * NACC;
#pragma unroll
      for (int a = 0; a < NACC; ++a) acc[a] += h[a];
    }
#pragma unroll
    for (int a = 0; a < NACC; ++a) tile_carry[a] = acc[a];
  }
  const int r = s_carry_row[g * 2 + 1];
  if (r >= 0) {
    // this group holds the start of row r: add the heads of the groups the row runs through
#pragma unroll
    for (int a = 0; a < NACC; ++a) acc[a] = my_tail[a];
    for (int j = g + 1; j < NG && s_carry_row[j * 2] == r; ++j) {
      const float* h = s_carry + (j * 2) * (G * NACC) + c * NACC;
#pragma unroll
      for (int a = 0; a < NACC; ++a) acc[a] += h[a];
    }
    if (r == last_row && tile_cont_out) {
      float* t = tile_carry + int64_t(lanes_all) * NACC;  // the tile's tail carry
#pragma unroll
      for (int a = 0; a < NACC; ++a) t[a] = acc[a];
    } else {
      pol.finalize(r, acc);
    }
  }

  // ---- rows that cross tile boundaries: every tile such a row touches has written one partial
  // (the tile it starts in a tail carry, the others a head carry) and now counts itself in; the
  // tile that arrives last finishes the row.  A tile touches at most two such rows.
  if (w.n_tiles == 1 || w.tile_done == nullptr) return;
  __threadfence();   // this thread's carries are visible device-wide before the arrival is counted
  __syncthreads();
  if (tid == 0) {
    const int first_row = row_of(0);
    auto arrive = [&](int row) {
      const int start_tile = __ldg(w.ptr + row) / te;
      const int end_tile = (__ldg(w.ptr + row + 1) - 1) / te;
      const int before = atomicAdd(w.tile_done + int64_t(blockIdx.y) * w.n_tiles + start_tile, 1);
      return before == end_tile - start_tile ? start_tile : -1;
    };
    __threadfence();
    s_finish[0] = s_halo[0] == first_row ? arrive(first_row) : -1;              // a head carry was written
    s_finish[1] = (tile_cont_out && s_halo[0] != last_row) ? arrive(last_row) : -1;  // a tail carry
    __threadfence();   // the other tiles' carries are read after their arrivals were seen
  }
  __syncthreads();     // from here on the index arrays are dead: s_part may overlay them
#pragma unroll 1
  for (int f = 0; f < 2; ++f) {
    const int start_tile = s_finish[f];
    if (start_tile >= 0) {
      finish_row<G, Policy>(w, pol, s_part, start_tile);
      __syncthreads();
    }
  }
}

// Finishes the row that starts in `tile` and runs past its end, from the partials all its tiles have
// delivered: that tile's tail carry and the head carries of the following tiles.  The partials are
// dealt round-robin to 128 / G slots, each slot adds its share in tile order, then the slots are
// combined in a fixed tree: the order depends neither on timing nor on which CTA runs this.
template <int G, class Policy>
__device__ __forceinline__ void finish_row(const SegWalk& w, const Policy& pol, float* s_part, int tile) {
  constexpr int NG = TileGeom<G>::NG;
  constexpr int NACC = Policy::NACC;
  const int te = NG * w.ge;
  const int64_t t1 = int64_t(tile + 1) * te;
  const int r = __ldg(w.seg + t1 - 1);
  const int last_tile = (__ldg(w.ptr + r + 1) - 1) / te;
  const int slot = threadIdx.x / G, c = threadIdx.x % G;
  const int lanes_all = gridDim.y * G;
  const int64_t stride = int64_t(lanes_all) * NACC;
  const float* base = w.gcarry + int64_t(blockIdx.y * G + c) * NACC;
  float acc[NACC];
#pragma unroll
  for (int a = 0; a < NACC; ++a) acc[a] = 0.f;
  // partial 0 = tail carry of `tile`, partial i > 0 = head carry of tile + i
  const int n_part = last_tile - tile + 1;
#pragma unroll 4
  for (int i = slot; i < n_part; i += NG) {
    const float* p = base + (int64_t(tile + i) * 2 + (i == 0 ? 1 : 0)) * stride;
#pragma unroll
    for (int a = 0; a < NACC; ++a) acc[a] += __ldcg(p + a);   // written by other CTAs of this launch: read at L2
  }
  // combine the NG slots: halving tree through shared memory
  float* mine = s_part + (slot * G + c) * NACC;
#pragma unroll
  for (int a = 0; a < NACC; ++a) mine[a] = acc[a];
  __syncthreads();
  for (int half = NG / 2; half >= 1; half >>= 1) {
    if (slot < half) {
      const float* o = s_part + ((slot + half) * G + c) * NACC;
#pragma unroll
      for (int a = 0; a < NACC; ++a) mine[a] += o[a];
    }
    __syncthreads();
  }
  if (slot == 0) {
#pragma unroll
    for (int a = 0; a < NACC; ++a) acc[a] = mine[a];
    pol.finalize(r, acc);
  }
}

// Second kernel for narrow lane groups: one CTA per tile; the CTA of the tile in which a row that runs
// past the tile's end STARTS finishes that row.
template <int G, class Policy>
__device__ __forceinline__ void stitch_tiles(const SegWalk& w, const Policy& pol, float* s_part) {
  const int tile = blockIdx.x;
  const int te = TileGeom<G>::NG * w.ge;
  const int64_t t1 = int64_t(tile + 1) * te;
  release_dependents();
  dependent_wait();                                  // the walk kernel's carries; every CTA waits, also those that return
  if (t1 >= w.n_edges) return;                       // last tile: nothing runs past it
  const int r = __ldg(w.seg + t1 - 1);
  if (__ldg(w.seg + t1) != r) return;                // the tile ends on a row boundary
  if (__ldg(w.ptr + r) < t1 - te) return;            // the row started in an earlier tile
  finish_row<G, Policy>(w, pol, s_part, tile);
}

inline bool stitch_in_second_kernel(int g) { return g <= TGT_STITCH_KERNEL_MAX_G; }

struct HeadSplit {
  int w;       // bytes one lane moves: 16 or 32
  int lph;     // lanes per head
  int hpg;     // heads per lane group
  int g;       // lanes per group
  int groups;  // number of head groups (gridDim.y)
};

enum { kPassFwd = 0, kPassDq = 1, kPassDkv = 2 };

// Lane width of the walk kernels: 0 = chosen by the library, 1 = 16-byte lanes, 2 = 32-byte lanes
// wherever the head size allows.  Set by tgt_debug_set_lane_mode().
int lane_mode();

// Bytes per lane for heads of head_dim elements.  32-byte lanes need heads that are whole multiples of
// 32 bytes and 32-byte aligned tensors and strides (`can32`).
inline int lane_bytes(int heads, int head_dim, int dtype, bool can32, int pass) {
  const int head_bytes = head_dim * (dtype == TGT_F32 ? 4 : 2);
  if (!can32 || dtype != TGT_F32 || head_bytes % 32 != 0 || head_bytes > 128) return 16;
  const int mode = lane_mode();
  if (mode == 1) return 16;
  if (mode == 2) return 32;
  return TGT_WIDE_DEFAULT(pass, heads * head_bytes) ? 32 : 16;
}

// Returns false when (heads, head_dim, dtype) cannot be mapped onto lanes of w bytes.
inline bool split_heads(int heads, int head_dim, int dtype, int w, HeadSplit* hs) {
  const int vec = w / (dtype == TGT_F32 ? 4 : 2);
  if (heads < 1 || head_dim < vec || head_dim % vec != 0) return false;
  const int lph = head_dim / vec;
  if (lph > 32 || (lph & (lph - 1)) != 0) return false;
  int hpg = 1;
  while (hpg * 2 * lph <= 32 && heads % (hpg * 2) == 0) hpg *= 2;
  hs->w = w;
  hs->lph = lph;
  hs->hpg = hpg;
  hs->g = lph * hpg;
  hs->groups = heads / hpg;
  return true;
}

// Compile-time shape of one kernel instantiation: element type, bytes per lane, lanes per head, lanes
// per group.
template <typename T_, int W_, int LPH_, int G_>
struct LaneShape {
  using T = T_;
  static constexpr int W = W_, LPH = LPH_, G = G_;
};

// Calls f(LaneShape<...>{}) for the run-time (dtype, w, lph, g); only shapes that can occur are
// instantiated (a group holds whole heads: LPH <= G; 32-byte lanes are built for fp32 heads of up to
// 128 bytes).  Returns false when the combination is not built.
template <typename T, int W, int LPH, class F>
inline bool dispatch_group(int g, F&& f) {
  switch (g) {
    case 1: if constexpr (LPH <= 1) { f(LaneShape<T, W, LPH, 1>{}); return true; } break;
    case 2: if constexpr (LPH <= 2) { f(LaneShape<T, W, LPH, 2>{}); return true; } break;
    case 4: if constexpr (LPH <= 4) { f(LaneShape<T, W, LPH, 4>{}); return true; } break;
    case 8: if constexpr (LPH <= 8) { f(LaneShape<T, W, LPH, 8>{}); return true; } break;
    case 16: if constexpr (LPH <= 16) { f(LaneShape<T, W, LPH, 16>{}); return true; } break;
    case 32: if constexpr (LPH <= 32) { f(LaneShape<T, W, LPH, 32>{}); return true; } break;
    default: break;
  }
  return false;
}

template <typename T, int W, class F>
inline bool dispatch_head(int lph, int g, F&& f) {
  switch (lph) {
    case 1: return dispatch_group<T, W, 1>(g, f);
    case 2: return dispatch_group<T, W, 2>(g, f);
    case 4: return dispatch_group<T, W, 4>(g, f);
    case 8: if constexpr (W == 16) return dispatch_group<T, W, 8>(g, f); else break;
    case 16: if constexpr (W == 16) return dispatch_group<T, W, 16>(g, f); else break;
    case 32: if constexpr (W == 16) return dispatch_group<T, W, 32>(g, f); else break;
    default: break;
  }
  return false;
}

template <class F>
inline bool dispatch_shape(int dtype, int w, int lph, int g, F&& f) {
  if (dtype == TGT_F32) return w == 32 ? dispatch_head<float, 32>(lph, g, f) : dispatch_head<float, 16>(lph, g, f);
  return w == 16 ? dispatch_head<__nv_bfloat16, 16>(lph, g, f) : false;
}

int check_layout(const tgt_layout* L, const char* name);

// Resident CTAs per SM of a walk kernel on the current device (asked from the runtime once per
// instantiation): the tile size is chosen so that one wave of CTAs covers the graph.
template <typename Kernel>
inline int resident_ctas(Kernel kernel, int* cache) {
  if (*cache <= 0) {
    int n = 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, kernel, kBlockThreads, 0) != cudaSuccess || n < 1) {
      cudaGetLastError();
      n = 4;
    }
    *cache = n;
  }
  return *cache;
}

// Tiling of one pass: edges per lane group, number of tiles, bytes of cross-tile carry followed by
// the arrival counters (scratch_bytes = both).
struct TilePlan {
  int ge;
  int n_tiles;
  size_t carry_bytes;
  size_t counter_bytes;
  size_t scratch_bytes;
};
TilePlan plan_tiles(int64_t n_edges, const HeadSplit& hs, int nacc, int ctas_per_sm);

// Shared-memory bytes walk_tile needs (indices + carries), as the kernels declare them.
template <int G, int NACC>
struct TileSmem {
  static constexpr int TE = TileGeom<G>::TE_MAX;
  static constexpr int NG = TileGeom<G>::NG;
  struct Indices {
    int32_t other[TE + NG];
    int32_t seg[TE + NG + 2];   // padded rows + the two halo words
    int32_t perm[TE + NG];
  };
  union {
    Indices idx;                          // while the tile is walked
    float part[kBlockThreads * NACC];     // afterwards: slots of finish_row
  };
  float carry[NG * 2 * G * NACC];
  int32_t carry_row[NG * 2];
  int32_t finish[2];
};

// The call every walk kernel makes.
template <int G, class Policy>
__device__ __forceinline__ void walk_tile_in(TileSmem<G, Policy::NACC>& sm, const SegWalk& w, const Policy& pol) {
  walk_tile<G, Policy>(w, pol, sm.idx.other, sm.idx.seg, sm.idx.perm, sm.carry, sm.carry_row, sm.part, sm.finish);
}

}  // namespace tgt
