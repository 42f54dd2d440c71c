// Ulysses exchange over NVLink peer memory: the head<->sequence all-to-all done by this GPU's own
// kernels instead of a library collective.
//
// Every rank owns peer-visible memory: one small control block and any number of "slots" (landing
// or source buffers) that all peers can address.  The two directions of the exchange move data the
// way NVLink likes it, in long contiguous runs on the wire:
//   sequence -> heads (q, k, v, dO):  PUSH.  Each rank reads its [rows, heads] tensors once (narrow
//       strided pieces, locally) and stores them as contiguous runs at their FINAL position in the
//       destination rank's slot — the split, the transfer and the concatenation of the reference's
//       _SeqAllToAll in one pass.  The attention kernels then read the slot in place.  Several
//       tensors can be interleaved row by row on arrival (K and V of a row side by side), so that
//       one gather serves both.
//   heads -> sequence (attention output, dQ, dK, dV):  PULL.  The producers write into their own
//       slot; after the barrier each rank reads the peers' slots in contiguous runs and stores the
//       narrow pieces locally at their final position.
//   barrier: every rank tells every peer "everything I enqueued before this point is done and
//       visible" and waits for the same from all peers (one flag word per peer pair,
//       release/acquire at system scope).
// A slot may be rewritten (by anybody) only after a barrier that follows the last read of its old
// content on every rank; the host-side bookkeeping that guarantees it lives with the caller.
//
// The general _SeqAllToAll (any tensor, any axis pair) remains available as push -> barrier ->
// fetch, where fetch copies a landed slot into ordinary tensors (and, in "staged" mode, does the
// concatenation that narrow destination runs would make slow on the wire).
//
// Waits are bounded: after `spin_limit` polls the barrier gives up, records the rank it was waiting
// for in a status word the host can read, and returns; the context stays usable.
#include <cstdlib>

#include "tgt_common.cuh"

namespace tgt {
namespace {

constexpr int kMaxWorld = 16;
constexpr int kThreads = 256;

struct PeerTable {
  void* p[kMaxWorld];
};
struct Ptrs3 {
  void* p[3];
};

// Control block of one rank (peer-visible, zero-filled once).
//   flags[j]  : last epoch announced by rank j (written only by rank j)
//   epoch     : number of barriers this rank has passed (local use; lives on the device so that a
//               replayed CUDA graph keeps counting)
struct Control {
  unsigned flags[kMaxWorld];
  unsigned epoch;
  unsigned pad[15];
};

__device__ __forceinline__ unsigned ld_acquire_sys(const unsigned* p) {
  unsigned v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_sys(unsigned* p, unsigned v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

// The copy kernels move "units" of 16 bytes (uint4) or, where every width and address allows it, of 32
// bytes (one 256-bit load / store of sm_100 per unit: half the requests per byte on the wire).
struct alignas(32) Unit32 {
  Raw32 r;
};
template <typename U>
__device__ __forceinline__ U load_unit(const U* p) {
  if constexpr (sizeof(U) == 32) {
    U u;
    u.r = ld_nc_256(p);
    return u;
  } else {
    return *p;
  }
}
template <typename U>
__device__ __forceinline__ void store_unit(U* p, const U& v) {
  if constexpr (sizeof(U) == 32) st_256(p, v.r);
  else *p = v;
}

// Fused split + transfer + concatenate.  Source tensor t is [outer_s][world][ws] in 16-byte units
// (ws units go to each peer from every outer row); the destination tensor on peer r' is
// [outer_g][world][wg] units, this rank filling column block `rank`.  A chunk's flat unit index
// f = a * ws + w maps to (f / wg, f % wg) on the destination.
// With n_weave > 1 the n_weave source tensors arrive as ONE tensor whose rows hold the sources'
// pieces side by side ([.., n_weave * ws] per outer row): the same formulas with ws and wg scaled
// by n_weave, unit w' of a woven row coming from source w' / ws.
template <typename U>
__global__ void push_kernel(Ptrs3 src, PeerTable landing, int n_tensors, int n_weave, int64_t outer_s,
                            int64_t ws, int64_t wg, int world, int rank,
                            const int32_t* __restrict__ alias_rows, int n_alias,
                            int64_t alias_period_units, bool staged) {
  constexpr int kBatch = 4;      // loads in flight per thread before the (posted) remote stores
  constexpr int kBurst = 256;    // consecutive 16-byte units (4 KB) written to one peer by one CTA pass
  const int64_t wsv = ws * n_weave, wgv = wg * n_weave;     // widths of the (woven) arriving tensor
  const int n_virtual = n_tensors / n_weave;                // tensors as they arrive
  const int64_t chunk = outer_s * wsv;                      // units one peer gets per arriving tensor
  const int64_t per_tensor_dst = chunk * world;             // units of one arriving tensor
  // Work is cut into bursts; consecutive bursts go to DIFFERENT peers, starting with the next rank,
  // so at any moment the CTAs of every GPU are spread over all links and no destination is hit by
  // all senders at once.
  const int64_t bursts_per_chunk = (chunk + kBurst - 1) / kBurst;
  const int64_t total = bursts_per_chunk * world * n_virtual * kBurst;
  const int64_t stride = int64_t(gridDim.x) * blockDim.x;
  for (int64_t i0 = blockIdx.x * int64_t(blockDim.x) + threadIdx.x; i0 < total;
       i0 += stride * kBatch) {
    U val[kBatch];
    U* dst[kBatch];
#pragma unroll
    for (int u = 0; u < kBatch; ++u) {
      const int64_t i = i0 + u * stride;
      dst[u] = nullptr;
      if (i >= total) continue;
      const int64_t burst = i / kBurst;
      const int pk = int(burst % world);
      const int tv = int((burst / world) % n_virtual);
      const int64_t f = (burst / (int64_t(world) * n_virtual)) * kBurst + (i % kBurst);
      if (f >= chunk) continue;
      const int peer = (rank + 1 + pk) % world;
      const int64_t a = f / wsv;
      const int64_t wv = f % wsv;
      const int t = tv * n_weave + int(wv / ws);          // source tensor of this unit
      const int64_t w = wv % ws;
      int64_t pos = int64_t(peer) * ws + w;   // unit position inside outer row a of the source
      if (n_alias > 0) {
        // rows listed in alias_rows are read from row 0 of the same outer row instead
        // (copy_global_token0 folded into the transfer); a row is alias_period_units wide
        const int64_t row = pos / alias_period_units;
        for (int j = 0; j < n_alias; ++j)
          if (row == alias_rows[j]) {
            pos = pos % alias_period_units;
            break;
          }
      }
      val[u] = load_unit(static_cast<const U*>(src.p[t]) + (a * world * ws + pos));
      // final position on the destination, or (staged) this rank's contiguous block of the slot
      const int64_t og = f / wgv, o = f % wgv;
      const int64_t where = staged ? int64_t(rank) * chunk + f : (og * world + rank) * wgv + o;
      dst[u] = static_cast<U*>(landing.p[peer]) + tv * per_tensor_dst + where;
    }
#pragma unroll
    for (int u = 0; u < kBatch; ++u)
      if (dst[u] != nullptr) store_unit(dst[u], val[u]);
  }
}

// Transfer + split + concatenate, reading from the peers.  Peer r' holds n_tensors tensors
// [outer][world * rows][wu] (16-byte units) back to back in its slot; this rank gathers
//   y_t[o][l][r' * wu + w] = slot_{r'}_t[o][rank * rows + l][w].
// What is read from one peer for one (t, o) is one contiguous run of rows * wu units.
template <typename U>
__global__ void pull_kernel(Ptrs3 dst, PeerTable slots, int n_tensors, int64_t outer, int64_t rows,
                            int64_t wu, int world, int rank,
                            const int32_t* __restrict__ alias_rows, int n_alias) {
  constexpr int kBatch = 8;      // remote loads in flight per thread
  constexpr int kBurst = 256;    // consecutive 16-byte units (4 KB) read from one peer by one CTA pass
  const int64_t run = rows * wu;                              // units of one contiguous remote run
  const int64_t bursts_per_run = (run + kBurst - 1) / kBurst;
  const int64_t per_tensor_src = outer * world * run;         // units of one tensor in a slot
  const int64_t total = bursts_per_run * world * outer * n_tensors * kBurst;
  const int64_t stride = int64_t(gridDim.x) * blockDim.x;
  for (int64_t i0 = blockIdx.x * int64_t(blockDim.x) + threadIdx.x; i0 < total;
       i0 += stride * kBatch) {
    U val[kBatch];
    U* where[kBatch];
#pragma unroll
    for (int u = 0; u < kBatch; ++u) {
      const int64_t i = i0 + u * stride;
      where[u] = nullptr;
      if (i >= total) continue;
      int64_t burst = i / kBurst;
      const int pk = int(burst % world); burst /= world;          // consecutive bursts: different peers
      const int t = int(burst % n_tensors); burst /= n_tensors;
      const int64_t o = burst % outer; burst /= outer;
      const int64_t f = burst * kBurst + (i % kBurst);            // unit inside the run
      if (f >= run) continue;
      const int peer = (rank + 1 + pk) % world;
      const int64_t l = f / wu, w = f % wu;
      int64_t src_row = int64_t(rank) * rows + l;
      for (int j = 0; j < n_alias; ++j)
        if (src_row == alias_rows[j]) {   // listed rows take the value of row 0 (copy_global_token0)
          src_row = 0;
          break;
        }
      val[u] = load_unit(static_cast<const U*>(slots.p[peer]) + (t * per_tensor_src + (o * world * rows + src_row) * wu + w));
      where[u] = static_cast<U*>(dst.p[t]) + ((o * rows + l) * world + peer) * wu + w;
    }
#pragma unroll
    for (int u = 0; u < kBatch; ++u)
      if (where[u] != nullptr) store_unit(where[u], val[u]);
  }
}

// One block; thread j talks to peer j.
__global__ void barrier_kernel(PeerTable control, int world, int rank, unsigned spin_limit,
                               int* __restrict__ status) {
  Control* mine = static_cast<Control*>(control.p[rank]);
  __shared__ unsigned next;
  if (threadIdx.x == 0) next = mine->epoch + 1;
  __syncthreads();
  const unsigned epoch = next;
  const int j = threadIdx.x;
  if (j < world && j != rank) {
    Control* theirs = static_cast<Control*>(control.p[j]);
    __threadfence_system();
    st_release_sys(&theirs->flags[rank], epoch);             // "everything before this barrier is done"
    unsigned polls = 0;
    // epochs only grow; a difference test survives the 32-bit wrap
    while (int(ld_acquire_sys(&mine->flags[j]) - epoch) < 0) {
      if (++polls >= spin_limit) {
        *reinterpret_cast<volatile int*>(status) = 1 + j;    // gave up waiting for rank j
        break;
      }
      __nanosleep(64);
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) mine->epoch = epoch;
}

// Copy a landed slot into ordinary tensors.  In staged mode the slot holds one contiguous block per
// source rank and the concatenation happens here: output unit j = (og * world + r) * wg + o comes
// from block r, unit og * wg + o.
template <typename U>
__global__ void fetch_kernel(Ptrs3 dst, const U* __restrict__ src, int n_tensors,
                             int64_t units_per_tensor, bool staged, int world, int64_t wg) {
  const int64_t total = units_per_tensor * n_tensors;
  const int64_t chunk = units_per_tensor / world;
  constexpr int kBatch = 4;
  const int64_t stride = int64_t(gridDim.x) * blockDim.x;
  for (int64_t i0 = blockIdx.x * int64_t(blockDim.x) + threadIdx.x; i0 < total; i0 += stride * kBatch) {
    U val[kBatch];
#pragma unroll
    for (int u = 0; u < kBatch; ++u) {
      const int64_t i = i0 + u * stride;
      if (i < total) {
        int64_t from = i;
        if (staged) {
          const int64_t t = i / units_per_tensor, j = i - t * units_per_tensor;
          const int64_t o = j % wg, r = (j / wg) % world, og = j / (wg * world);
          from = t * units_per_tensor + r * chunk + og * wg + o;
        }
        val[u] = src[from];
      }
    }
#pragma unroll
    for (int u = 0; u < kBatch; ++u) {
      const int64_t i = i0 + u * stride;
      if (i < total) {
        const int t = int(i / units_per_tensor);
        static_cast<U*>(dst.p[t])[i - t * units_per_tensor] = val[u];
      }
    }
  }
}

// CTAs per SM of the copy kernels; the environment variable TGT_P2P_CTAS (1..32) overrides the default
// for tuning runs.
int ctas_per_sm() {
  static const int value = [] {
    const char* e = getenv("TGT_P2P_CTAS");
    const int v = e != nullptr ? atoi(e) : 0;
    return v >= 1 && v <= 32 ? v : 8;
  }();
  return value;
}

// 32-byte units in the copy kernels; TGT_P2P_UNIT=16 in the environment keeps them at 16 bytes.
bool wide_units() {
  static const bool value = [] {
    const char* e = getenv("TGT_P2P_UNIT");
    return !(e != nullptr && atoi(e) == 16);
  }();
  return value;
}

int grid_for(int64_t n) {
  int64_t b = (n + kThreads - 1) / kThreads;
  const int64_t cap = int64_t(sm_count()) * ctas_per_sm();
  if (b > cap) b = cap;
  if (b < 1) b = 1;
  return int(b);
}

int fill_table(PeerTable* tab, void* const* peers, int world) {
  TGT_CHECK_ARG(world >= 1 && world <= kMaxWorld, "world must be between 1 and 16");
  TGT_CHECK_ARG(peers != nullptr, "peer table is null");
  for (int i = 0; i < kMaxWorld; ++i) tab->p[i] = nullptr;
  for (int i = 0; i < world; ++i) {
    TGT_CHECK_ARG(peers[i] != nullptr && aligned16(peers[i]), "peer pointers must be non-null and 16-byte aligned");
    tab->p[i] = peers[i];
  }
  return TGT_OK;
}

}  // namespace
}  // namespace tgt

extern "C" size_t tgt_p2p_control_bytes(void) { return sizeof(tgt::Control); }

extern "C" int tgt_p2p_push(const void* x0, const void* x1, const void* x2, int n_tensors,
                            void* const* peer_slots, size_t slot_bytes, int64_t outer_s,
                            int64_t width_s_bytes, int64_t width_g_bytes, int world, int rank,
                            const int32_t* alias_rows, int n_alias, int64_t alias_row_bytes,
                            int mode, void* stream_) {
  using namespace tgt;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  TGT_CHECK_ARG(n_tensors >= 1 && n_tensors <= 3, "n_tensors must be 1, 2 or 3");
  TGT_CHECK_ARG(mode == TGT_PUSH_FINAL || mode == TGT_PUSH_STAGED || mode == TGT_PUSH_WOVEN,
                "mode must be TGT_PUSH_FINAL, TGT_PUSH_STAGED or TGT_PUSH_WOVEN");
  const void* xs[3] = {x0, x1, x2};
  for (int t = 0; t < 3; ++t)
    TGT_CHECK_ARG((t < n_tensors) == (xs[t] != nullptr), "tensor pointers do not match n_tensors");
  TGT_CHECK_ARG(rank >= 0 && rank < world, "rank outside the world");
  TGT_CHECK_ARG(outer_s >= 1 && width_s_bytes >= 16 && width_g_bytes >= 16, "sizes must be positive");
  TGT_CHECK_ARG(width_s_bytes % 16 == 0 && width_g_bytes % 16 == 0,
                "per-peer widths must be multiples of 16 bytes");
  TGT_CHECK_ARG((outer_s * width_s_bytes) % width_g_bytes == 0, "chunk is not a whole number of destination rows");
  TGT_CHECK_ARG(aligned16(x0) && aligned16(x1) && aligned16(x2), "tensors must be 16-byte aligned");
  TGT_CHECK_ARG(size_t(n_tensors) * size_t(outer_s) * size_t(width_s_bytes) * size_t(world) <= slot_bytes,
                "the slot is too small for this exchange");
  TGT_CHECK_ARG(n_alias >= 0 && (n_alias == 0 || (alias_rows != nullptr && alias_row_bytes >= 16 &&
                                                  alias_row_bytes % 16 == 0)),
                "bad alias row arguments");
  TGT_CHECK_ARG(mode != TGT_PUSH_WOVEN || n_alias == 0, "alias rows are not supported with woven rows");
  PeerTable tab;
  int rc = fill_table(&tab, peer_slots, world);
  if (rc != TGT_OK) return rc;
  Ptrs3 src;
  for (int t = 0; t < 3; ++t) src.p[t] = const_cast<void*>(xs[t]);
  // 32-byte units when every width, row and address is a multiple of 32 bytes
  bool wide = wide_units() && width_s_bytes % 32 == 0 && width_g_bytes % 32 == 0 && aligned32(x0) && aligned32(x1) &&
              aligned32(x2) && (n_alias == 0 || alias_row_bytes % 32 == 0);
  for (int i = 0; i < world; ++i) wide = wide && aligned32(tab.p[i]);
  wide = wide && (outer_s * width_s_bytes * world) % 32 == 0;
  const int ub = wide ? 32 : 16;
  const int64_t ws = width_s_bytes / ub, wg = width_g_bytes / ub;
  const int64_t total = ((outer_s * ws + 255) / 256) * 256 * world * n_tensors;
  if (wide)
    push_kernel<Unit32><<<grid_for((total + 3) / 4), kThreads, 0, stream>>>(
        src, tab, n_tensors, mode == TGT_PUSH_WOVEN ? n_tensors : 1, outer_s, ws, wg, world, rank,
        alias_rows, n_alias, n_alias > 0 ? alias_row_bytes / ub : 1, mode == TGT_PUSH_STAGED);
  else
    push_kernel<uint4><<<grid_for((total + 3) / 4), kThreads, 0, stream>>>(
        src, tab, n_tensors, mode == TGT_PUSH_WOVEN ? n_tensors : 1, outer_s, ws, wg, world, rank,
        alias_rows, n_alias, n_alias > 0 ? alias_row_bytes / ub : 1, mode == TGT_PUSH_STAGED);
  TGT_CHECK_CUDA(cudaGetLastError());
  return TGT_OK;
}

extern "C" int tgt_p2p_pull(void* const* peer_slots, size_t slot_bytes, int n_tensors, void* y0,
                            void* y1, void* y2, int64_t outer, int64_t rows, int64_t width_bytes,
                            int world, int rank, const int32_t* alias_rows, int n_alias,
                            void* stream_) {
  using namespace tgt;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  TGT_CHECK_ARG(n_tensors >= 1 && n_tensors <= 3, "n_tensors must be 1, 2 or 3");
  void* ys[3] = {y0, y1, y2};
  for (int t = 0; t < 3; ++t)
    TGT_CHECK_ARG((t < n_tensors) == (ys[t] != nullptr), "tensor pointers do not match n_tensors");
  TGT_CHECK_ARG(rank >= 0 && rank < world, "rank outside the world");
  TGT_CHECK_ARG(outer >= 1 && rows >= 1 && width_bytes >= 16 && width_bytes % 16 == 0,
                "outer and rows must be positive, width_bytes a positive multiple of 16");
  TGT_CHECK_ARG(aligned16(y0) && aligned16(y1) && aligned16(y2), "tensors must be 16-byte aligned");
  TGT_CHECK_ARG(size_t(n_tensors) * size_t(outer) * size_t(world) * size_t(rows) * size_t(width_bytes) <= slot_bytes,
                "the slot is smaller than the tensors said to live in it");
  TGT_CHECK_ARG(n_alias >= 0 && (n_alias == 0 || alias_rows != nullptr), "bad alias row arguments");
  PeerTable tab;
  int rc = fill_table(&tab, peer_slots, world);
  if (rc != TGT_OK) return rc;
  Ptrs3 dst;
  for (int t = 0; t < 3; ++t) dst.p[t] = ys[t];
  bool wide = wide_units() && width_bytes % 32 == 0 && aligned32(y0) && aligned32(y1) && aligned32(y2);
  for (int i = 0; i < world; ++i) wide = wide && aligned32(tab.p[i]);
  wide = wide && (size_t(outer) * size_t(world) * size_t(rows) * size_t(width_bytes)) % 32 == 0;
  const int64_t wu = width_bytes / (wide ? 32 : 16);
  const int64_t total = ((rows * wu + 255) / 256) * 256 * world * outer * n_tensors;
  if (wide)
    pull_kernel<Unit32><<<grid_for((total + 7) / 8), kThreads, 0, stream>>>(dst, tab, n_tensors, outer, rows, wu,
                                                                           world, rank, alias_rows, n_alias);
  else
    pull_kernel<uint4><<<grid_for((total + 7) / 8), kThreads, 0, stream>>>(dst, tab, n_tensors, outer, rows, wu,
                                                                          world, rank, alias_rows, n_alias);
  TGT_CHECK_CUDA(cudaGetLastError());
  return TGT_OK;
}

extern "C" int tgt_p2p_barrier(void* const* peer_control, int world, int rank, uint32_t spin_limit,
                               int32_t* status, void* stream_) {
  using namespace tgt;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  TGT_CHECK_ARG(rank >= 0 && rank < world, "rank outside the world");
  TGT_CHECK_ARG(status != nullptr, "status is null");
  TGT_CHECK_ARG(spin_limit >= 1, "spin_limit must be >= 1");
  PeerTable tab;
  int rc = fill_table(&tab, peer_control, world);
  if (rc != TGT_OK) return rc;
  barrier_kernel<<<1, 32, 0, stream>>>(tab, world, rank, spin_limit, status);
  TGT_CHECK_CUDA(cudaGetLastError());
  return TGT_OK;
}

extern "C" int tgt_p2p_fetch(const void* slot_mine, size_t slot_bytes, int n_tensors, void* y0,
                             void* y1, void* y2, int64_t bytes_per_tensor, int staged, int world,
                             int64_t width_g_bytes, void* stream_) {
  using namespace tgt;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  TGT_CHECK_ARG(n_tensors >= 1 && n_tensors <= 3, "n_tensors must be 1, 2 or 3");
  TGT_CHECK_ARG(staged == 0 || staged == 1, "staged must be 0 or 1");
  TGT_CHECK_ARG(staged == 0 || (world >= 1 && width_g_bytes >= 16 && width_g_bytes % 16 == 0 &&
                                bytes_per_tensor % (int64_t(world) * width_g_bytes) == 0),
                "staged fetch needs world and a destination row width that divide the tensor");
  void* ys[3] = {y0, y1, y2};
  for (int t = 0; t < 3; ++t)
    TGT_CHECK_ARG((t < n_tensors) == (ys[t] != nullptr), "tensor pointers do not match n_tensors");
  TGT_CHECK_ARG(slot_mine != nullptr && aligned16(slot_mine), "slot pointer is null or misaligned");
  TGT_CHECK_ARG(bytes_per_tensor >= 16 && bytes_per_tensor % 16 == 0, "bytes_per_tensor must be a multiple of 16");
  TGT_CHECK_ARG(size_t(bytes_per_tensor) * n_tensors <= slot_bytes, "the slot is smaller than the request");
  TGT_CHECK_ARG(aligned16(y0) && aligned16(y1) && aligned16(y2), "tensors must be 16-byte aligned");
  Ptrs3 dst;
  for (int t = 0; t < 3; ++t) dst.p[t] = ys[t];
  const int64_t units = bytes_per_tensor / 16;
  fetch_kernel<uint4><<<grid_for((units * n_tensors + 3) / 4), kThreads, 0, stream>>>(
      dst, static_cast<const uint4*>(slot_mine), n_tensors, units, staged != 0, staged ? world : 1,
      staged ? width_g_bytes / 16 : 1);
  TGT_CHECK_CUDA(cudaGetLastError());
  return TGT_OK;
}
