/*
 * torchgt_b200 — C ABI of the sparse graph-attention hot path for NVIDIA B200 (sm_100a).
 *
 * One shared library (libtorchgt_b200.so) exports the functions below.  Signatures use only plain
 * pointers and sizes.  Every pointer named "device" must point into CUDA device memory of the
 * current device, be 16-byte aligned and densely packed.  Nothing here allocates device memory
 * unless the comment on the entry point says otherwise: scratch is passed in by the caller after a
 * size query.  Kernels are enqueued on the `stream` argument (a cudaStream_t passed as void*;
 * NULL = legacy default stream) and the calls do not synchronise unless stated.
 *
 * Every function returns TGT_OK (0) or a TGT_ERR_* code; tgt_last_error() gives the message of the
 * last failure on the calling thread.  Argument checks run before any launch.
 *
 * The reference (zxmeng98/torchgt) is pure PyTorch and has no FFI; each entry point below cites the
 * reference Python code it replaces (path inside that project : lines).
 */
#ifndef TORCHGT_B200_H
#define TORCHGT_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(__GNUC__)
#define TGT_API __attribute__((visibility("default")))
#else
#define TGT_API
#endif

#define TGT_OK 0
#define TGT_ERR_INVALID 1      /* null / misaligned pointer, negative size, inconsistent layout   */
#define TGT_ERR_CUDA 2         /* a CUDA runtime call or a launch failed                          */
#define TGT_ERR_UNSUPPORTED 3  /* head_dim / head count / dtype combination not built             */
#define TGT_ERR_WORKSPACE 4    /* scratch or workspace smaller than the size query says           */
#define TGT_ERR_INDEX_RANGE 5  /* edge_index holds a node id outside [0, n_rows)                  */

#define TGT_F32 0
#define TGT_BF16 1

/* bias_heads values: per-edge additive score bias given in ORIGINAL edge order (fp32).           */
#define TGT_BIAS_NONE 0 /* no bias                                                                */
/* 1      -> bias[E]     one value per edge shared by all heads                                   */
/* heads  -> bias[E, H]  one value per edge and head                                              */

/*
 * Edges sorted by one endpoint ("segment layout").  Built by tgt_edge_layout_build.
 *   group_by = 1 : sorted by destination (edge_index row 1) — used by forward and by the dQ pass;
 *                  `other` holds the source of every edge.
 *   group_by = 0 : sorted by source (edge_index row 0) — used by the dK/dV pass; `other` holds the
 *                  destination.
 * Definition (bit-exact contract): perm = stable argsort of the grouping endpoint,
 * seg = grouping endpoint[perm], other = other endpoint[perm],
 * ptr = exclusive prefix sum of bincount(grouping endpoint, n_rows).
 */
typedef struct tgt_layout {
  int64_t n_rows;
  int64_t n_edges;
  const int32_t* ptr;   /* device [n_rows + 1] */
  const int32_t* other; /* device [n_edges]    */
  const int32_t* perm;  /* device [n_edges]    */
  const int32_t* seg;   /* device [n_edges]    */
} tgt_layout;

/* Library version (major * 100 + minor). */
TGT_API int tgt_version(void);

/* Message of the last error returned on this thread ("" if none).  Never NULL. */
TGT_API const char* tgt_last_error(void);

/*
 * Tuning / test knob with no counterpart in the reference: the attention kernels cut the sorted edge
 * list into tiles of (128 / lanes-per-row) * edges_per_lane_group edges.  0 (the default) lets the
 * library choose so that one wave of thread blocks covers the graph; a small value forces many
 * tiles, which the tests use to exercise the cross-tile paths on small graphs.  Process-wide.
 */
TGT_API int tgt_debug_set_tile_edges(int edges_per_lane_group);

/*
 * Tuning / test knob with no counterpart in the reference: how many bytes of a row one lane of the
 * attention kernels moves.  0 (default): the library chooses per head size; 1: 16 bytes (one 128-bit
 * load per piece); 2: 32 bytes wherever it applies — fp32 heads of 32, 64 or 128 bytes in 32-byte
 * aligned tensors — using the 256-bit global loads and stores of sm_100, so that a head of 8 fp32
 * values is one lane and one load.  Results agree to rounding (the order of sums inside a head
 * differs).  Process-wide.
 */
TGT_API int tgt_debug_set_lane_mode(int mode);

/*
 * Tuning / test knob with no counterpart in the reference: which consecutive kernels of one attention call
 * are chained with programmatic dependent launches (the next kernel's CTAs stage their edge indices while
 * the previous kernel drains, then wait for it to complete).  A bit mask: 1 = a walk kernel after the
 * statistics kernel or another walk kernel, 2 = the kernel that finishes cross-tile rows after its walk
 * kernel, 4 = a walk kernel after such a kernel; 0 launches everything one after the other, the default is
 * 1 | 4.  The results are bitwise the same.  Process-wide.
 */
TGT_API int tgt_debug_set_dependent_launch(int links);

/*
 * Bytes of device workspace tgt_edge_layout_build needs.
 * Replaces nothing in the reference (the reference keeps edges as an unsorted COO list).
 */
TGT_API int tgt_edge_layout_sizes(int64_t n_rows, int64_t n_edges, size_t* workspace_bytes);

/*
 * Build one segment layout from the COO edge list the reference's batch packing produces
 * (gt_sp/utils.py:34-58 fix_edge_index / adjust_edge_index_nomerge, gt_sp/utils.py:409-520
 * get_batch_reorder_blockize, data/collator_sp_sparse.py:126-133 flatten_edge_index_nopad):
 * edge_index is a device int64 [2, n_edges] array, row 0 = source (K/V row), row 1 = destination
 * (Q / output row), exactly as consumed by CoreAttention.sparse_attention (attn_module.py:146-147).
 * ptr [n_rows + 1], other, perm, seg [n_edges] are device output buffers.
 * With deferred_status == NULL this call SYNCHRONISES the stream once (it is made once per batch,
 * not per layer) and returns TGT_ERR_INDEX_RANGE if any node id is outside [0, n_rows).  With a
 * device int32 word in deferred_status nothing is synchronised: the word is set to 0, or to 1 if an
 * id was out of range (such ids are replaced by 0 in the layout, so later kernels stay in bounds),
 * and the caller reads it when convenient.
 */
TGT_API int tgt_edge_layout_build(const int64_t* edge_index, int64_t n_edges, int64_t n_rows,
                                  int group_by, int32_t* ptr, int32_t* other, int32_t* perm,
                                  int32_t* seg, void* workspace, size_t workspace_bytes,
                                  int32_t* deferred_status, void* stream);

/*
 * The same build for an int32 [2, n_edges] device edge list (what tgt_edge_prepare writes): half the
 * bytes of the reference's int64 list (main_sp_sparse_node_level.py:178-182 uploads int64 every
 * iteration).  All other arguments and the result are those of tgt_edge_layout_build.
 */
TGT_API int tgt_edge_layout_build_i32(const int32_t* edge_index, int64_t n_edges, int64_t n_rows,
                                      int group_by, int32_t* ptr, int32_t* other, int32_t* perm,
                                      int32_t* seg, void* workspace, size_t workspace_bytes,
                                      int32_t* deferred_status, void* stream);

/*
 * Batch edge construction on the device: the reference's host-side helpers applied in one pass to the
 * RAW edges of a batch of `graphs` graphs (node ids 0..n_g-1 inside each graph), writing an int32
 * [2, out_total] edge list for tgt_edge_layout_build_i32.
 *   add_global_token = 1 : fix_edge_index (gt_sp/utils.py:34-50, data/collator_sp_sparse.py:107-123):
 *                          ids + 1, then per graph the edges (i -> 0), i = 1..n_g, then (0 -> i);
 *   sub_seq_len > 0      : adjust_edge_index_nomerge (gt_sp/utils.py:53-58): id x > 0 becomes
 *                          x + (x - 1) / sub_seq_len (integer division);
 *   rows_per_graph       : flatten_edge_index_nopad (data/collator_sp_sparse.py:126-133): graph g's ids
 *                          are offset by g * rows_per_graph (pass 0 for a single graph).
 * raw_edges: device int64 [2, raw_total], the graphs' raw lists concatenated; raw_ptr: device int64
 * [graphs + 1] edge range of every graph; node_ptr: device int64 [graphs + 1] prefix sums of the node
 * counts (only read with add_global_token).  out_total must equal raw_total (+ 2 * total nodes with
 * add_global_token).  Per graph the output order is [raw | node -> token | token -> node], i.e. the
 * order the reference's helpers produce, so per-edge biases keep their meaning.
 */
TGT_API int tgt_edge_prepare(const int64_t* raw_edges, int64_t raw_total, const int64_t* raw_ptr,
                             const int64_t* node_ptr, int graphs, int add_global_token,
                             int64_t sub_seq_len, int64_t rows_per_graph, int32_t* out,
                             int64_t out_total, void* stream);

/*
 * Bytes of scratch tgt_sparse_attn_fwd (phase 0) / tgt_sparse_attn_bwd (phase 1) need for these
 * layouts (partial sums of rows that cross a tile boundary; row statistics of the backward).
 * by_src may be NULL for phase 0.
 */
TGT_API int tgt_sparse_attn_scratch_bytes(const tgt_layout* by_dst, const tgt_layout* by_src,
                                          int heads, int head_dim, int dtype, int phase,
                                          size_t* bytes);

/*
 * Forward of the topology-aware sparse attention: for every edge e = (s -> d) and head h
 *   raw = sum_j K[s,h,j] * Q[d,h,j] / sqrt(head_dim);  t = clamp(raw, -5, 5) + bias[e(,h)]
 *   w = exp(t);  U[d,h,:] += w * V[s,h,:];  Z[d,h] += w;      out = U / (Z + 1e-6)
 * Replaces CoreAttention.sparse_attention (attn_module.py:133-189) and the sparse_attention_bias
 * copies (models/graphormer_dist_node_level.py:69-127, models/gt_dist_node_level.py:83-142,
 * models/graphormer_dist_graph_level.py:238-292, models/gt_dist_graph_level.py:83-137) including
 * the two torch_scatter.scatter(reduce='add') calls.  No per-edge tensor is materialised.
 * q, k, v, out: device [n_rows, heads, head_dim] of `dtype`; z: device fp32 [n_rows, heads]
 * (saved for backward); bias: device fp32 in ORIGINAL edge order or NULL (see bias_heads).
 * Rows without in-edges produce exactly 0.  Deterministic (every floating-point sum has a fixed order).
 */
TGT_API int tgt_sparse_attn_fwd(const void* q, const void* k, const void* v, const float* bias,
                        int bias_heads, const tgt_layout* by_dst, void* out, float* z, int heads,
                        int head_dim, int dtype, void* scratch, size_t scratch_bytes, void* stream);

/*
 * The same forward for q, k, v whose rows are not densely packed: q_row_bytes and kv_row_bytes are
 * the distances between consecutive rows of q and of k / v (multiples of 16, at least heads *
 * head_dim elements).  With k and v stored side by side per row ([n_rows, 2, heads * head_dim]:
 * v = k + one row width, kv_row_bytes = two row widths — what TGT_PUSH_WOVEN delivers) the K and V
 * pieces of an edge share their cache lines.  out and z are dense.  No counterpart in the reference
 * (its tensors are always contiguous copies: gt_sp/layer.py:41,45).
 */
TGT_API int tgt_sparse_attn_fwd_strided(const void* q, int64_t q_row_bytes, const void* k,
                                        const void* v, int64_t kv_row_bytes, const float* bias,
                                        int bias_heads, const tgt_layout* by_dst, void* out,
                                        float* z, int heads, int head_dim, int dtype, void* scratch,
                                        size_t scratch_bytes, void* stream);

/*
 * Forward for callers that cannot allocate.  No counterpart in the reference.
 *
 * tgt_sparse_attn_fwd needs scratch from its caller.  Some callers have none to give and may not
 * create any: a process whose own arena took the whole GPU at start-up, a plug-in inside such a
 * process, a loop that must never reach cudaMalloc because that call can stall the device.  This
 * entry point computes exactly what tgt_sparse_attn_fwd computes (same kernels, same results) but
 * keeps the scratch in a 4 MiB array that is part of the library image, so the call allocates
 * nothing and neither must the caller; every GPU that loads the library carries those 4 MiB until
 * the process exits.  Inputs and outputs are still the caller's.
 *
 * Limit: the graph's cross-tile carry must fit the 4 MiB (for 8 heads x 8 in fp32 that is about
 * 6.5 million edges); a larger graph is refused with TGT_ERR_WORKSPACE before anything runs.
 * The first call on each device looks the array's device address up (one cudaGetSymbolAddress with
 * that device current) and remembers it; make that first call outside any stream capture.
 * All calls on one GPU share the array: two calls whose kernels can overlap on the GPU (different
 * streams, no ordering between them) race on it and corrupt each other's rows; calls ordered on
 * one stream are safe.  Nothing in the array has to start at zero — every slot that is read was
 * written earlier in the same call — so stale contents of a previous call are harmless.
 */
TGT_API int tgt_sparse_attn_fwd_noalloc(const void* q, const void* k, const void* v,
                                        const float* bias, int bias_heads,
                                        const tgt_layout* by_dst, void* out, float* z, int heads,
                                        int head_dim, int dtype, void* stream);

/*
 * Backward of the same op (the reference has no hand-written backward; this replaces the autograd
 * graph of attn_module.py:141-187: three index_put_(accumulate=True), two gathers and the
 * elementwise chain).  With G = dout, inv = 1/(Z+1e-6):
 *   dw = (G_d . V_s - G_d . O_d) * inv_d;  dV_s += w * inv_d * G_d;  dt = dw * w  (= dbias)
 *   da = dt * [-5 <= raw <= 5];  dQ_d += da * K_s / sqrt(D);  dK_s += da * Q_d / sqrt(D)
 * Pass A walks by_dst (dQ, dbias, per-row statistics), pass B walks by_src (dK, dV); scores are
 * recomputed, nothing per-edge is read from forward.  dbias is device fp32 in ORIGINAL edge order
 * with the shape bias has, or NULL when not wanted.  `out` (the forward result) is read only when
 * dbias is wanted and may be NULL otherwise.  Deterministic (every floating-point sum has a fixed order).
 */
TGT_API int tgt_sparse_attn_bwd(const void* dout, const void* q, const void* k, const void* v,
                        const float* bias, int bias_heads, const void* out, const float* z,
                        const tgt_layout* by_dst, const tgt_layout* by_src, void* dq, void* dk,
                        void* dv, float* dbias, int heads, int head_dim, int dtype, void* scratch,
                        size_t scratch_bytes, void* stream);

/*
 * The same backward with its stages selectable by bit mask: 2 = pass A (dQ and, into `scratch`, the
 * per-row statistics 1/(Z+1e-6) and dO.O that pass B reads), 4 = pass B (dK, dV; needs the statistics
 * a pass A left in the same scratch for the same inputs), 1 = streaming pre-pass that computes the
 * statistics from dO and O — required (in the same or an earlier call) only when dbias is wanted,
 * because dbias needs them per edge before a row is complete.  tgt_sparse_attn_bwd runs 6, or 7 with
 * dbias.  Lets a caller time or overlap the stages; replaces the same reference code.
 */
TGT_API int tgt_sparse_attn_bwd_passes(const void* dout, const void* q, const void* k, const void* v,
                                       const float* bias, int bias_heads, const void* out,
                                       const float* z, const tgt_layout* by_dst,
                                       const tgt_layout* by_src, void* dq, void* dk, void* dv,
                                       float* dbias, int heads, int head_dim, int dtype,
                                       void* scratch, size_t scratch_bytes, void* stream, int passes);

/*
 * tgt_sparse_attn_bwd_passes for inputs whose rows are not densely packed (see
 * tgt_sparse_attn_fwd_strided): row distances of dout, of q and of k / v in bytes.  dq, dk, dv, out
 * and z are dense.  passes = 0 runs what is needed (6, or 7 when dbias is wanted).
 */
TGT_API int tgt_sparse_attn_bwd_strided(const void* dout, int64_t dout_row_bytes, const void* q,
                                        int64_t q_row_bytes, const void* k, const void* v,
                                        int64_t kv_row_bytes, const float* bias, int bias_heads,
                                        const void* out, const float* z, const tgt_layout* by_dst,
                                        const tgt_layout* by_src, void* dq, void* dk, void* dv,
                                        float* dbias, int heads, int head_dim, int dtype,
                                        void* scratch, size_t scratch_bytes, void* stream,
                                        int passes);

/*
 * Ulysses head<->sequence exchange: local re-layout kernels around ONE all-to-all.
 *
 * The reference's _SeqAllToAll (gt_sp/layer.py:30-49, gt_sp/gt_layer.py:30-49) does
 * tensor_split(scatter_idx) + contiguous() per chunk, a list all_to_all, and cat(gather_idx)
 * .contiguous(), once per tensor (q, k, v: gt_sp/layer.py:516-518; context: :545).  Here up to three
 * tensors share one peer-major staging buffer
 *     stage[world][n_tensors][batch][seq_local][width_local]
 * (chunk `peer` is what is sent to / received from that rank), so one collective moves them all.
 * width_local = (heads / world) * head_dim elements; `dtype` only fixes the element size.
 *
 *   tgt_a2a_pack_heads  : x_t [batch, seq_local, world*width_local]  -> stage   (scatter_idx = 2)
 *   tgt_a2a_unpack_seq  : stage -> y_t [batch, world*seq_local, width_local]    (gather_idx  = 1)
 *   tgt_a2a_pack_seq    : x_t [batch, world*seq_local, width_local]  -> stage   (scatter_idx = 1)
 *   tgt_a2a_unpack_heads: stage -> y_t [batch, seq_local, world*width_local]    (gather_idx  = 2)
 *
 * pack_heads + unpack_seq is the q/k/v direction (and the backward of the context direction);
 * pack_seq + unpack_heads is the context direction (and the backward of the q/k/v direction).
 * Unused tensor slots (t >= n_tensors) must be NULL.
 */
TGT_API int tgt_a2a_pack_heads(const void* x0, const void* x1, const void* x2, int n_tensors, void* stage,
                       int64_t batch, int64_t seq_local, int64_t width_local, int world, int dtype,
                       void* stream);
TGT_API int tgt_a2a_unpack_seq(const void* stage, int n_tensors, void* y0, void* y1, void* y2,
                       int64_t batch, int64_t seq_local, int64_t width_local, int world, int dtype,
                       void* stream);
TGT_API int tgt_a2a_pack_seq(const void* x0, const void* x1, const void* x2, int n_tensors, void* stage,
                     int64_t batch, int64_t seq_local, int64_t width_local, int world, int dtype,
                     void* stream);
TGT_API int tgt_a2a_unpack_heads(const void* stage, int n_tensors, void* y0, void* y1, void* y2,
                         int64_t batch, int64_t seq_local, int64_t width_local, int world,
                         int dtype, void* stream);

/*
 * copy_global_token0 (gt_sp/utils.py:817-838): x [batch, seq, width]; every row listed in
 * global_rows (device int32 [n_global], e.g. r*(L+1) for r = 0..P-1) is overwritten in place with
 * row 0 of the same batch entry.  The reference builds and uploads the index tensor on every call;
 * here it stays on the device.
 */
TGT_API int tgt_global_rows_broadcast(void* x, const int32_t* global_rows, int n_global, int64_t batch,
                              int64_t seq, int64_t width, int dtype, void* stream);

/*
 * Backward of tgt_global_rows_broadcast (autograd of the in-place index assignment at
 * gt_sp/utils.py:836): dx[b, 0, :] = sum over listed rows of dx[b, row, :] (summed in list order,
 * fp32 accumulation; plus dx[b, 0, :] itself when row 0 is not listed), then every listed row
 * other than 0 is set to zero.
 */
TGT_API int tgt_global_rows_reduce(void* dx, const int32_t* global_rows, int n_global, int64_t batch,
                           int64_t seq, int64_t width, int dtype, void* stream);

/*
 * Ulysses exchange over NVLink peer memory: the same head<->sequence all-to-all as above, done by this
 * library's kernels reading and writing the other ranks' memory directly instead of by a collective
 * library plus pack / unpack passes.  Replaces _SeqAllToAll.forward (gt_sp/layer.py:30-45) and, with
 * alias rows, copy_global_token0 (gt_sp/utils.py:817-838) in the same pass.
 *
 * Peer-visible memory is the caller's: every rank owns one zero-filled control block of
 * tgt_p2p_control_bytes() bytes and any number of "slots".  A peer table is a host array of `world`
 * pointers (world <= 16), entry i being rank i's block or slot AS SEEN FROM THIS GPU (peer mapping).
 * All ranks make the same calls in the same order with the same sizes.  A slot may be written again
 * only after a tgt_p2p_barrier that follows, in stream order on every rank, the last read of its
 * old content; the barrier counts on the device, so a sequence may be replayed from a CUDA graph.
 *
 * tgt_p2p_push (sequence -> heads: q, k, v, dO): tensor t is [outer_s][world][width_s_bytes] (what
 * _SeqAllToAll splits along scatter_idx); on every destination it lands as
 * [outer_g][world][width_g_bytes] (what cat along gather_idx produces) with this rank's piece in
 * column block `rank`, tensors back to back in the destination's slot.  If n_alias > 0, source rows
 * (of alias_row_bytes each, counted inside one outer row) listed in the device array alias_rows are
 * read from row 0 instead.  mode:
 *   TGT_PUSH_FINAL   every piece is stored at its final position on the destination;
 *   TGT_PUSH_STAGED  this rank's whole chunk is stored as one contiguous block and the concatenation
 *                    is left to tgt_p2p_fetch (for small width_g_bytes: NVLink stores of less than
 *                    128 bytes are slow);
 *   TGT_PUSH_WOVEN   as FINAL, but the n_tensors tensors arrive as ONE tensor whose rows hold the
 *                    sources' pieces side by side ([.., n_tensors * width_s_bytes]): K and V of a row
 *                    next to each other, so that one gather serves both.
 * tgt_p2p_pull (heads -> sequence: attention output, dQ, dK, dV; call it after a barrier): every
 * peer's slot holds n_tensors tensors [outer][world * rows][width_bytes] back to back; this rank
 * reads its rows from all of them, y_t[o][l][r * width_bytes + c] = slot_r_t[o][rank * rows + l][c],
 * into ordinary device tensors.  Source rows listed in alias_rows are read from row 0 of the same o.
 * tgt_p2p_barrier: everything every rank enqueued before it is complete and visible when the kernel
 * ends.  Waits are bounded: after spin_limit polls it gives up, writes 1 + (rank it waited for) to
 * *status (a host-readable, device-writable int32, e.g. pinned memory) and returns; the context
 * stays usable, the data of that step is not.
 * tgt_p2p_fetch: copies n_tensors landed tensors (bytes_per_tensor each) out of this rank's slot into
 * ordinary device tensors; `staged`, `world` and `width_g_bytes` must repeat what the push was given.
 */
#define TGT_PUSH_FINAL 0
#define TGT_PUSH_STAGED 1
#define TGT_PUSH_WOVEN 2
TGT_API size_t tgt_p2p_control_bytes(void);
TGT_API int tgt_p2p_push(const void* x0, const void* x1, const void* x2, int n_tensors,
                         void* const* peer_slots, size_t slot_bytes, int64_t outer_s,
                         int64_t width_s_bytes, int64_t width_g_bytes, int world, int rank,
                         const int32_t* alias_rows, int n_alias, int64_t alias_row_bytes,
                         int mode, void* stream);
TGT_API int tgt_p2p_pull(void* const* peer_slots, size_t slot_bytes, int n_tensors, void* y0,
                         void* y1, void* y2, int64_t outer, int64_t rows, int64_t width_bytes,
                         int world, int rank, const int32_t* alias_rows, int n_alias, void* stream);
TGT_API int tgt_p2p_barrier(void* const* peer_control, int world, int rank, uint32_t spin_limit,
                            int32_t* status, void* stream);
TGT_API int tgt_p2p_fetch(const void* slot_mine, size_t slot_bytes, int n_tensors, void* y0,
                          void* y1, void* y2, int64_t bytes_per_tensor, int staged, int world,
                          int64_t width_g_bytes, void* stream);

/*
 * The dense layers next to the exchange, fused with it (fp32, hidden size = projection width = 64, the
 * reference models' size; other sizes return TGT_ERR_UNSUPPORTED and the caller uses the separate steps).
 *
 * tgt_ln_qkv_push replaces, per encoder layer, LayerNorm (models/graphormer_dist_node_level.py:301), the
 * three projections (:254-257) and the q/k/v all-to-alls with their `contiguous` copies
 * (gt_sp/layer.py:41,516-518): x is this rank's [batch * rows, hidden]; for every tile of rows the kernel
 * normalises (gamma / beta NULL: no LayerNorm), multiplies by the three [out_features, hidden] weights
 * (nn.Linear layout, fp32 FMA), adds the biases and stores every rank's head slice at its final position
 * in that rank's slot (q, k, v back to back, each [batch][world * rows][out_features / world]) — plain
 * stores into peer memory.  Follow it with tgt_p2p_barrier; the attention then reads the slot in place.
 *
 * tgt_pull_out_proj replaces copy_global_token0 (gt_sp/utils.py:817-838), the output all-to-all
 * (gt_sp/layer.py:545) and the output projection (models/graphormer_dist_node_level.py:271): call it
 * after a tgt_p2p_barrier that follows the attention; every peer's slot holds its attention output
 * [batch][world * rows][in_features / world]; the kernel gathers this rank's rows of all of them
 * (rows listed in alias_rows read row 0), writes the gathered [batch * rows, in_features] to ctx (the
 * input of the projection, needed for its weight gradient) and y = ctx W^T + b ([hidden, in_features]
 * weight) to y.
 */
TGT_API int tgt_ln_qkv_push(const float* x, const float* gamma, const float* beta, float eps,
                            const float* wq, const float* bq, const float* wk, const float* bk,
                            const float* wv, const float* bv, int hidden, int out_features,
                            void* const* peer_slots, size_t slot_bytes, int64_t batch, int64_t rows,
                            int world, int rank, void* stream);
TGT_API int tgt_pull_out_proj(void* const* peer_slots, size_t slot_bytes, const float* w, const float* b,
                              int hidden, int in_features, float* ctx, float* y, int64_t batch,
                              int64_t rows, int world, int rank, const int32_t* alias_rows, int n_alias,
                              void* stream);

/*
 * LayerNorm over short rows, fp32, forward and backward: the normalisation on both sides of the attention
 * block (models/graphormer_dist_node_level.py:301,306,395; nn.LayerNorm(hidden) with weight and bias) and
 * the backward of the LayerNorm inside tgt_ln_qkv_push.  hidden must be a multiple of 4, at most 512.
 *   forward:  y = (x - mean) / sqrt(var + eps) * gamma + beta (biased variance, as torch.nn.LayerNorm);
 *             stats (may be NULL) receives [rows][2] = mean, 1 / sqrt(var + eps) for the backward.
 *   backward: dx, dgamma [hidden], dbeta [hidden] from dy, x, gamma and the forward's stats; scratch of
 *             tgt_layer_norm_bwd_scratch_bytes holds per-CTA sums that a second kernel adds in a fixed
 *             order (no atomics: results are bitwise reproducible).
 */
TGT_API int tgt_layer_norm_fwd(const float* x, const float* gamma, const float* beta, float eps, int64_t rows,
                               int hidden, float* y, float* stats, void* stream);
TGT_API int tgt_layer_norm_bwd_scratch_bytes(int64_t rows, int hidden, size_t* bytes);
TGT_API int tgt_layer_norm_bwd(const float* dy, const float* x, const float* gamma, const float* stats,
                               int64_t rows, int hidden, float* dx, float* dgamma, float* dbeta, void* scratch,
                               size_t scratch_bytes, void* stream);

/*
 * Weight and bias gradient of a narrow nn.Linear over many rows, fp32: dw [out_features, in_features] =
 * dy^T x and db [out_features] (may be NULL) = column sums of dy, for dy [rows, out_features] and x [rows,
 * in_features] — the backward of the models' projections and FFN layers (models/graphormer_dist_node_level.py:
 * 241-245,281-286,343) with respect to their parameters.  in_features must be a multiple of 64, out_features
 * of 4, both at most 1024 (TGT_ERR_UNSUPPORTED otherwise: the caller uses a library GEMM).  Per-CTA tiles are added
 * in a fixed order by a second kernel (no atomics, bitwise reproducible); scratch of
 * tgt_linear_wgrad_scratch_bytes holds them.
 */
TGT_API int tgt_linear_wgrad_scratch_bytes(int64_t rows, int in_features, int out_features, size_t* bytes);
TGT_API int tgt_linear_wgrad(const float* dy, const float* x, int64_t rows, int in_features, int out_features,
                             float* dw, float* db, void* scratch, size_t scratch_bytes, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* TORCHGT_B200_H */
