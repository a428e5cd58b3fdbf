/*
 * dsa_b200 -- C ABI of the B200 (sm_100a) DSA decode kernels.
 *
 * One shared library, libdsa_b200.so, replaces the torch extension that the
 * reference JIT-builds from kernels/cuda_fused_sparse_splitk.py (export list
 * :2922-2941, declarations :2228-2303). Every entry point takes raw device
 * pointers, plain sizes and a CUDA stream; nothing here allocates, synchronises
 * with the host or reads a length on the host, so each call can be captured in
 * a CUDA graph (the reference's contract: kernels/cuda_fused_sparse_splitk.py
 * :2399-2499 argument checks, :2531 current stream, caller-owned scratch
 * src/lagged_indexer_dsa/inference/modeling/fused_decode.py:46-119).
 *
 * Conventions
 *   - return value: DSA_OK (0) or a negative dsa_status; dsa_last_error()
 *     returns the message of the calling thread's last failure.
 *   - "row" = one query token. R rows share `rows_per_seq` consecutive rows per
 *     cached sequence: rows_per_seq == 1 is batched decode, rows_per_seq == S
 *     is the reference's S-row single-sequence launch.
 *   - seq_lens[r] (device int32, may be NULL = `ctx`) is the number of causally
 *     visible keys of row r; keys at positions >= seq_lens[r] are masked.
 *   - stream is a cudaStream_t passed as void*.
 *   - all device pointers must be 16-byte aligned.
 */
#ifndef DSA_B200_H_
#define DSA_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define DSA_ABI_VERSION 9

enum dsa_status {
  DSA_OK = 0,
  DSA_ERR_INVALID_ARGUMENT = -1, /* shape / stride / alignment contract broken  */
  DSA_ERR_UNSUPPORTED = -2,      /* valid request outside the compiled geometry */
  DSA_ERR_CUDA = -3,             /* a CUDA runtime/driver call failed           */
  DSA_ERR_DEVICE_TIMEOUT = -4    /* a bounded in-kernel wait gave up            */
};

/* Geometry fixed at compile time, as in the reference kernel
 * (kernels/cuda_fused_sparse_splitk.py:53-55, :2498-2499, :2550). */
#define DSA_LATENT_DIM 576      /* 512 latent + 64 rope, bf16                    */
#define DSA_VALUE_DIM 512
#define DSA_INDEX_DIM 128       /* index key width, e4m3                         */
#define DSA_INDEX_MAX_HEADS 64
#define DSA_HEAD_BLOCK 16       /* MLA heads per attention CTA                   */
#define DSA_PAGE_TOKENS 64
#define DSA_INDEX_PAGE_BYTES 8448 /* 64 x 128 B keys, then 64 x fp32 scales      */
#define DSA_FP8_LATENT_ROW 656  /* 512 e4m3 | 4 x fp32 group scale | 64 bf16     */
#define DSA_TOPK_HIST_BINS 4096 /* first-level histogram bins per row            */

int dsa_abi_version(void);
const char* dsa_last_error(void);
const char* dsa_status_string(int status);

/* Reads and clears the per-device status word. Kernels set a bit in it when one of
 * their bounded waits ran out (DSA_STATUS_*_TIMEOUT) or when they declined to follow a
 * page-table entry outside the pool (DSA_STATUS_BAD_PAGE). Synchronises the device.
 * Returns DSA_OK, DSA_ERR_DEVICE_TIMEOUT when a wait ran out, else
 * DSA_ERR_INVALID_ARGUMENT for a bad page; *detail (optional) receives the raw word. */
#define DSA_STATUS_SCAN_TIMEOUT 1u
#define DSA_STATUS_ATTN_TIMEOUT 2u
#define DSA_STATUS_SELECT_OVERFLOW 4u
#define DSA_STATUS_BAD_PAGE 8u
#define DSA_STATUS_EXCHANGE_TIMEOUT 16u
int dsa_check_device_status(uint32_t* detail);

/* Tracing builds only (compiled with -DDSA_STAMPS): copies the per-CTA phase
 * stamps (SM cycle counters, 16 slots per CTA, first 1024 CTAs) to host_out and
 * clears them; returns the number of words or DSA_ERR_UNSUPPORTED. Counterpart
 * of hide_debug_read (kernels/cuda_fused_sparse_splitk.py:2329-2349). */
int dsa_debug_read_stamps(uint64_t* host_out, int max_words);

/* Test aid for the bounded waits: launches one CTA that waits, for at most
 * limit_ns (0 < limit_ns <= 10 ms) of wall time, on a shared-memory barrier that
 * nothing completes. The wait runs out, the kernel sets DSA_STATUS_ATTN_TIMEOUT
 * and returns; dsa_check_device_status then reports DSA_ERR_DEVICE_TIMEOUT once
 * and clears the word. Nothing faults or hangs: this is the path every kernel of
 * the library takes when one of its waits runs out. */
int dsa_debug_wait_timeout(uint64_t limit_ns, void* stream);

/* ---- (a1) lightning-indexer scan ------------------------------------------
 * logits[r, s] = (sum_h w[r,h] * relu(q[r,h,:] . k[s,:])) * k_scale[s],
 * -inf for s >= seq_lens[r]. Replaces the indexer half of
 * launch_fused_sparse_splitk* with with_select=1
 * (kernels/cuda_fused_sparse_splitk.py:531-647, :1677-1903; host reference
 * ref_indexer_logits_fp8 :2990-2992).
 *
 *   index_q   [R, n_heads, 128] e4m3        index_w  [R, n_heads] fp32
 *   index_k   [n_seq, k_seq_stride, 128] e4m3  (sequence of row r = r / rows_per_seq)
 *   k_scale   [n_seq, scale_seq_stride] fp32
 *   logits    [R, slab_stride] fp32, columns [0, ctx) written
 *   hist      NULL, or [R, DSA_TOPK_HIST_BINS] uint32 that the scan increments
 *             with the top-12-bit bucket of every valid logit (must be zero on
 *             entry; dsa_topk_select re-zeroes it after use)
 *   impl      0 = TMA + tcgen05 FP8 MMA, 1 = legacy mma.sync path (diagnostic,
 *             like the reference's hp_diag_mode bit 2, :1851-1880)
 */
int dsa_indexer_scan_fp8(const uint8_t* index_q, const float* index_w,
                         const uint8_t* index_k, const float* k_scale,
                         const int32_t* seq_lens, float* logits, uint32_t* hist,
                         int R, int rows_per_seq, int n_heads, int64_t ctx,
                         int64_t n_seq, int64_t k_seq_stride, int64_t scale_seq_stride,
                         int64_t slab_stride, int impl, void* stream);

/* Paged form: index keys live in 64-token pages of DSA_INDEX_PAGE_BYTES
 * ([64 x 128 B keys][64 x fp32 scales], kernels/cuda_fused_sparse_splitk.py
 * :540-546, :2428-2429); page_table[r, j] is the pool page of tokens
 * [64 j, 64 j + 64) of row r (rows_per_seq is 1). Replaces the indexer half of
 * launch_fused_sparse_splitk_paged (:2770-2808). */
int dsa_indexer_scan_fp8_paged(const uint8_t* index_q, const float* index_w,
                               const uint8_t* index_k_pages, int64_t num_pages,
                               const int32_t* page_table, int64_t pt_stride,
                               const int32_t* seq_lens, float* logits, uint32_t* hist,
                               int R, int n_heads, int64_t ctx, int64_t slab_stride,
                               void* stream);

/* fp32 form for any head count / key width (src/lagged_indexer_dsa/
 * attention_core.py:27-49 arithmetic, used by the full-sequence layer API). */
int dsa_indexer_scan_f32(const float* index_q, const float* index_w, const float* index_k,
                         const int32_t* seq_lens, float* logits,
                         int R, int rows_per_seq, int n_heads, int head_dim, int64_t ctx,
                         int64_t k_seq_stride, int64_t slab_stride, void* stream);

/* ---- (a3) exact top-k selection -------------------------------------------
 * Indices of the `topk` largest logits[r, 0:min(n, seq_lens[r])), ties broken
 * by lower position, written in ascending position order and padded with
 * `pad_value` (also written for a selected entry whose logit is -inf). Replaces
 * torch.topk on the slab (src/lagged_indexer_dsa/attention_core.py:66-91;
 * inference/modeling/transformer.py:1156) and the in-kernel select
 * (kernels/cuda_fused_sparse_splitk.py:2017-2154).
 *
 *   hist       NULL, or the histogram dsa_indexer_scan_fp8 filled for these
 *              rows (saves the histogram launch; re-zeroed on exit)
 *   index_map  NULL, or [R, n] int32: the value written for position p is
 *              index_map[r, p] (used to merge per-GPU candidate lists)
 *   out_idx    [R, topk] int32        out_val  NULL or [R, topk] fp32
 *   workspace  caller-owned scratch of at least dsa_topk_workspace_bytes(R, n)
 *              bytes, zero before its first use; every call leaves it re-armed
 *              (the reference's self-resetting SelScratch, :2150-2153). Calls
 *              that share a workspace must not overlap on the device.
 *   index_offset is added to positions when index_map is NULL.
 * Limit: n <= 1048576 per row.
 */
int64_t dsa_topk_workspace_bytes(int R, int64_t n);
int dsa_topk_select(const float* logits, const int32_t* seq_lens, uint32_t* hist,
                    const int32_t* index_map, int32_t* out_idx, float* out_val,
                    void* workspace, int64_t workspace_bytes,
                    int R, int64_t n, int64_t slab_stride, int topk,
                    int32_t pad_value, int32_t index_offset, void* stream);

/* ---- candidate exchange of the KV-sequence-sharded indexer -------------------
 * One process per GPU, each scanning its own range of the keys. The reference has no
 * multi-GPU indexer; its closest relative is the per-slice top-m followed by an exact merge
 * inside one GPU (kernels/cuda_fused_sparse_splitk.py:1914-2015), and its serving overlay
 * states the rules for collectives inside a captured graph (persistent buffers, in-place,
 * sglang_overlay/mli-sglang-v0.5.16.patch:2478-2487). Here the exchange is part of the two
 * top-k launches themselves, so a whole sharded step is kernels in stream order:
 *
 *   dsa_topk_select_push   the local top-k of each row; every selected (index + index_offset,
 *                          logit) pair is STORED into slot `rank` of every rank's gather buffers
 *                          (plain stores through peer-mapped pointers over NVLink, no loads from
 *                          peer memory, no multicast), then the row's step number is posted, with
 *                          release at system scope, to flag word [rank][r] of every rank.
 *   dsa_topk_merge_wait    waits until all `world` flags of a row carry its next step number
 *                          (acquire; BOUNDED by wait_limit_ns of wall time: when it runs out the
 *                          kernel sets DSA_STATUS_EXCHANGE_TIMEOUT and finishes, and
 *                          dsa_check_device_status returns DSA_ERR_DEVICE_TIMEOUT), then selects
 *                          the exact top-k of the world * topk candidates, ties to the lower rank /
 *                          position, so every rank ends with the single-GPU selection bit for bit.
 *
 * Buffers of one rank (all zero before the first step, never touched by the host afterwards):
 *   gather_idx int32 / gather_val fp32  [2][R][world][topk]   two step parities
 *   flags  uint32 [world][R]   written by the sources        sent, seen  uint32 [R]  local
 * gather_idx / gather_val / flags given to dsa_topk_select_push are arrays of `world`
 * pointers: entry d is rank d's buffer as THIS process can address it (its own pointer for
 * d == rank, else from dsa_ipc_open). The two launches of a step must be enqueued in this
 * order on every rank, the same number of times; rows of up to 262144 logits. */
int dsa_topk_select_push(const float* logits, const int32_t* seq_lens, uint32_t* hist, int R, int64_t n,
                         int64_t slab_stride, int topk, int32_t pad_value, int32_t index_offset, int world,
                         int rank, void* const* gather_idx, void* const* gather_val, void* const* flags,
                         uint32_t* sent, void* stream);
int dsa_topk_merge_wait(const int32_t* gather_idx, const float* gather_val, const uint32_t* flags,
                        uint32_t* seen, int32_t* out_idx, int R, int world, int topk, int32_t pad_value,
                        int64_t wait_limit_ns, void* stream);
/* ---- all-reduce of a decode activation across the GPUs of a tensor-parallel layer ----
 * The reference sums the partial outputs of its row-parallel projections with
 * dist.all_reduce in fp32 (src/lagged_indexer_dsa/inference/modeling/transformer.py:361-377
 * RowParallelLinear, :3965 MoE / MLP output). At decode that is a [B, hidden] vector of tens
 * of kilobytes; here it is two one-CTA launches in stream order, the same store-and-flag
 * protocol as the candidate exchange above:
 *   dsa_allreduce_push      src [n] (bf16 when src_bf16, else fp32) -> fp32, stored into slot
 *                           `rank` of every rank's slots [2][world][n], then the step number
 *                           is posted to flag word [rank] of every rank.
 *   dsa_allreduce_wait_sum  bounded wait for all `world` flags, then
 *                           out = (residual ? residual : 0) + sum over ranks in rank order
 *                           (bit-identical on every rank); out / residual bf16 when out_bf16.
 *                           With a bf16 residual the sum is rounded to bf16 before the addition.
 * slots / flags given to the push are arrays of `world` pointers as for the candidate
 * exchange; n a multiple of 4. Buffers start zeroed; flags uint32 [world], sent / seen one
 * uint32 each. */
int dsa_allreduce_push(const void* src, int src_bf16, int64_t n, int world, int rank, void* const* slots,
                       void* const* flags, uint32_t* sent, void* stream);
int dsa_allreduce_wait_sum(const float* slots, const uint32_t* flags, uint32_t* seen, const void* residual,
                           void* out, int out_bf16, int64_t n, int world, int64_t wait_limit_ns, void* stream);

/* Set-up of the peer mapping (CUDA IPC; one call per buffer and peer, outside any step):
 * export gives the handle of the allocation that holds `ptr` and ptr's offset inside it,
 * open maps a peer's allocation and returns the address of the same byte, close unmaps it. */
#define DSA_IPC_HANDLE_BYTES 64
int dsa_ipc_export(const void* ptr, void* handle_out /* DSA_IPC_HANDLE_BYTES */, int64_t* offset_out);
int dsa_ipc_open(const void* handle, int64_t offset, void** ptr_out);
int dsa_ipc_close(void* ptr, int64_t offset);

/* ---- top-k for callers that cannot allocate ---------------------------------
 * This entry point has no counterpart in the reference. It is dsa_topk_select
 * (no histogram input, no index map) for hosts that have no way to obtain device
 * memory for scratch: a runtime whose memory pool is closed once serving starts,
 * a plugin that is handed only its input and output buffers, or code running at
 * a point where cudaMalloc is forbidden. Rows of up to 262144 logits (131072
 * on a device that cannot schedule a cluster of 16 CTAs) need no scratch at all
 * (one cluster kernel, shared memory only); for longer rows the
 * scratch is a fixed DSA_TOPK_STATIC_SCRATCH_BYTES array inside the library's
 * device image, so each GPU that loads the library gives up that much memory
 * until the process exits; the call itself performs no cudaMalloc / cudaFree
 * and calls no allocating routine.
 *   - Limit: dsa_topk_workspace_bytes(R, n) <= DSA_TOPK_STATIC_SCRATCH_BYTES
 *     (for rows longer than 262144: one row of up to ~480k logits); larger requests return DSA_ERR_UNSUPPORTED with a message naming
 *     both sizes. Every argument is checked before anything is enqueued.
 *   - The first call on each device looks up the array's device address
 *     (cudaGetSymbolAddress); make that first call before starting any stream
 *     capture. Host threads may make it concurrently (the look-up is locked).
 *   - All calls on a device share the one array and it keeps the previous call's
 *     contents; the part that must start at zero is cleared on `stream` by every
 *     call that uses the array. Two such calls that overlap on the GPU
 *     (different streams, or work replayed concurrently) race on it: serialise them.
 */
#define DSA_TOPK_STATIC_SCRATCH_BYTES (4 * 1024 * 1024)
int dsa_topk_select_static(const float* logits, const int32_t* seq_lens, int32_t* out_idx,
                           float* out_val, int R, int64_t n, int64_t slab_stride, int topk,
                           int32_t pad_value, int32_t index_offset, void* stream);

/* ---- (a4, a5) split-K sparse MLA decode ------------------------------------
 * out[r,h,:] = softmax_j(sm_scale * q[r,h,:] . kv[idx_j,:]) . kv[idx_j,:512]
 * over the entries of indices[r,:] with 0 <= idx < seq_lens[r]. Replaces the
 * attention half of launch_fused_sparse_splitk* and combine_kernel
 * (kernels/cuda_fused_sparse_splitk.py:282-530, :996-1045; host reference
 * ref_sparse_mla :2950-2966).
 *
 *   q        [R, H, 576] bf16 (absorbed queries), H a multiple of 16
 *   kv       kv_fp8 == 0: [n_seq, kv_seq_stride, 576] bf16
 *            kv_fp8 == 1: [n_seq, kv_seq_stride, 656] bytes, rows laid out as
 *            512 e4m3 | 4 fp32 scales (one per 128 dims) | 64 bf16 rope
 *            (:1098-1104), dequantised fp8->f32 * scale -> bf16 RN (:1181-1196)
 *   indices  [R, topk] int32, or NULL to attend every key below seq_lens[r]
 *            (dense cold start; topk is then the key capacity to cover)
 *   part_acc [R, nsplit, H, 512] fp32, part_m / part_l [R, nsplit, H] fp32
 *   out      [R, H, 512] bf16
 * dsa_sparse_mla_decode = partials + combine; the two halves are exported for
 * callers that schedule them separately, as the reference does.
 *
 * Two kernels serve the partials. Launches with H a multiple of 64 and at least
 * 128 tiles of 64 heads x 64 keys (R * H/64 * ceil(topk/64)) run on tcgen05 /
 * tensor memory with 64 heads per CTA; smaller launches and other head counts
 * run on mma.sync with 16 heads per CTA. Both write the same part_* layout;
 * part_m is a base-2 softmax reference of the split (not necessarily its
 * maximum) consistent with part_l and part_acc, which is all
 * dsa_sparse_mla_combine needs. (bf16 partial accumulators were measured: the
 * combine alone gets 1 us faster, the pair of launches 0.2 us slower.)
 */
int dsa_sparse_mla_partials(const void* q, const void* kv, const int32_t* indices,
                            const int32_t* seq_lens, float* part_acc, float* part_m,
                            float* part_l, int R, int rows_per_seq, int H, int topk,
                            int nsplit, float sm_scale, int64_t kv_seq_stride, int kv_fp8,
                            void* stream);
int dsa_sparse_mla_combine(const float* part_acc, const float* part_m, const float* part_l,
                           void* out, int R, int H, int nsplit, void* stream);
int dsa_sparse_mla_decode(const void* q, const void* kv, const int32_t* indices,
                          const int32_t* seq_lens, float* part_acc, float* part_m,
                          float* part_l, void* out, int R, int rows_per_seq, int H, int topk,
                          int nsplit, float sm_scale, int64_t kv_seq_stride, int kv_fp8,
                          void* stream);

/* dsa_sparse_mla_decode for a launch whose operands do NOT depend on the kernel enqueued just
 * before it on the stream: under the lagged schedule (inference/modeling/transformer.py:1140-1190)
 * a layer's attention reads the PREVIOUS layer's selection, so enqueued behind this layer's top-k it
 * can run beside it (and, because the top-k releases its dependents before it waits for the
 * scan, beside the end of the scan too: the operands must depend on neither of the two kernels
 * enqueued before the call). The partials kernel releases its dependents and starts at once, and
 * waits for the kernel before it only before it exits: it completes after that kernel, and whatever
 * is enqueued next sees both. The whole lagged layer then stays one chain of programmatic
 * dependents on one stream (scan -> top-k -> this) instead of two streams and a join. Launches
 * that the tcgen05 kernel serves run as dsa_sparse_mla_decode does. The kernel before it must be
 * one of this library's; behind any other work the call behaves like dsa_sparse_mla_decode. */
int dsa_sparse_mla_decode_beside(const void* q, const void* kv, const int32_t* indices,
                                 const int32_t* seq_lens, float* part_acc, float* part_m,
                                 float* part_l, void* out, int R, int rows_per_seq, int H, int topk,
                                 int nsplit, float sm_scale, int64_t kv_seq_stride, int kv_fp8,
                                 void* stream);

/* ---- (a6) fused indexer + attention launch -----------------------------------
 * One launch whose first CTAs compute the split-K attention partials over
 * `attend_indices` (under the lagged schedule: the PREVIOUS layer's selection)
 * and whose remaining CTAs run this layer's indexer scan into `logits` (+ `hist`),
 * followed by the LSE merge. Same results as dsa_sparse_mla_decode +
 * dsa_indexer_scan_fp8, bit for bit. Replaces launch_fused_sparse_splitk with
 * attn_on=1, with_select=1|2 (kernels/cuda_fused_sparse_splitk.py:178-683,
 * :2634-2655); the top-k stays a separate call. Dense bf16 caches only. */
int dsa_fused_decode(const void* q, const void* kv, const int32_t* attend_indices,
                     const int32_t* attn_seq_lens, float* part_acc, float* part_m, float* part_l,
                     void* out,
                     const uint8_t* index_q, const float* index_w, const uint8_t* index_k,
                     const float* k_scale, const int32_t* index_seq_lens, float* logits, uint32_t* hist,
                     int R, int rows_per_seq, int H, int topk, int nsplit, float sm_scale,
                     int64_t kv_seq_stride, int n_index_heads, int64_t ctx, int64_t n_seq,
                     int64_t k_seq_stride, int64_t scale_seq_stride, int64_t slab_stride, void* stream);

/* fp32 form for any head / latent width (src/lagged_indexer_dsa/
 * attention_core.py:94-160): one pass, no split. indices NULL = dense causal. */
int dsa_sparse_mla_f32(const float* q, const float* kv, const int32_t* indices,
                       const int32_t* seq_lens, float* out, int R, int rows_per_seq, int H,
                       int qk_dim, int v_dim, int topk, float sm_scale,
                       int64_t kv_seq_stride, void* stream);

/* ---- decode-step preparation between the projection GEMVs and the hot path ---
 * dsa_rmsnorm: out = x * rsqrt(mean(x^2) + eps) * weight over rows of `dim`
 * (src/lagged_indexer_dsa/dsa_layer.py:42-52); dtype 0 = fp32, 1 = bf16.
 *
 * dsa_decode_prep: everything the new token needs before scan / attention, in
 * one launch (the reference's stage_fp8_operands chain,
 * inference/modeling/transformer.py:1015-1066, :1137-1144, :3268-3276):
 *   - indexer query heads: RoPE at positions[b], per-head e4m3 quantisation,
 *     index_w = q_scale * w_raw;
 *   - the token's index key: RoPE, e4m3 + scale, written at cache row positions[b];
 *   - the token's latent row: RMSNorm(512) | RoPE(64), written at positions[b];
 *   - the absorbed query: q_full = [q_abs | RoPE(q_pe)].
 * All inputs bf16 ([B,Hidx,128], [B,Hidx], [B,128], [B,576], [B,H,512],
 * [B,H,64] with row stride q_pe_stride elements); rotary tables bf16
 * [cap,64] / [cap,128]; caches as in dsa_indexer_scan_fp8 / dsa_sparse_mla_*. */
int dsa_rmsnorm(const void* x, const void* weight, void* out, int64_t rows, int dim, float eps,
                int dtype, void* stream);
/* The residual addition and the norm that follows it in a decoder layer
 * (src/lagged_indexer_dsa/model.py:137-138) in one launch, bf16 rows of dim <= 8192
 * (a multiple of 8): sum_out = x + delta (rounded to bf16), out = rmsnorm(sum_out). */
int dsa_add_rmsnorm_bf16(const void* x, const void* delta, const void* weight, void* sum_out, void* out,
                         int64_t rows, int dim, float eps, void* stream);
/* dst[0, bytes) = src[0, bytes) by a kernel (16-byte pieces; bytes and both pointers
 * multiples of 16). Either side may be pinned host memory: inside a CUDA graph a kernel
 * node starts sooner than a copy-engine node, which matters for the few KB a decode step
 * brings from the host. No counterpart in the reference. */
int dsa_copy_bytes(void* dst, const void* src, int64_t bytes, void* stream);
/* The same copy, run BESIDE the kernel enqueued just before it on the stream instead of after
 * it: for data that neither of the two kernels enqueued before it writes or reads (a step's
 * queries arriving from the host while the selection is being computed; the top-k releases its
 * dependents before it waits for the scan, so the copy may start while the scan still runs).
 * The copy still completes after the kernel before it, and whatever is enqueued next on the
 * stream sees both. It keeps the stream's chain of
 * programmatic dependents intact where a copy on a forked stream would cost a join. The
 * kernel before it must be one of this library's (they release their dependents early);
 * behind any other work it behaves like dsa_copy_bytes. No counterpart in the reference. */
int dsa_copy_bytes_beside(void* dst, const void* src, int64_t bytes, void* stream);

/* Completion signal for a host that polls instead of calling a stream synchronise:
 * *counter (device) is incremented and its new value posted to *host_flag (pinned
 * host memory) once everything enqueued before it on the stream has completed and its
 * writes to host memory are visible. No counterpart in the reference. */
int dsa_post_epoch(uint32_t* counter, uint32_t* host_flag, void* stream);
/* dsa_copy_bytes (at most 1 MiB, by one CTA) followed by dsa_post_epoch in ONE launch: the
 * last node of a step's graph when a few KB (the selection) still have to reach the host
 * before the signal. It starts as a programmatic dependent of the kernel enqueued before
 * it on the stream and runs once that kernel has completed. beside != 0: the bytes do not
 * come from that kernel (nor from the one before it); they are then copied beside it and only
 * the signal waits for it. No counterpart in the reference. */
int dsa_copy_post_epoch(void* dst, const void* src, int64_t bytes, uint32_t* counter, uint32_t* host_flag,
                        int beside, void* stream);

/* y[b, n] = sum_k w[n, k] x[b, k] for a decode batch of 1..4 rows: bf16 operands, fp32
 * accumulation, w [n, k] row-major streamed once (the projection GEMVs of
 * src/lagged_indexer_dsa/dsa_layer.py:87-125 at decode). k a multiple of 8,
 * batch * k * 2 <= 96 KB; row strides of x and y in elements. */
int dsa_gemv_bf16(const void* w, const void* x, void* y, int batch, int n, int k, int64_t x_stride,
                  int64_t y_stride, void* stream);
/* out = silu(gate) * up over n bf16 elements: the SwiGLU between the MLP's GEMVs
 * (src/lagged_indexer_dsa/dsa_layer.py:194-196), rounded as the two separate operations. */
int dsa_silu_mul_bf16(const void* gate, const void* up, void* out, int64_t n, void* stream);
int dsa_decode_prep(const void* iq_raw, const void* w_raw, const void* ik_raw, const void* kv_a,
                    const void* q_abs, const void* q_pe, int64_t q_pe_stride, const void* kv_norm_w,
                    const void* mla_cos, const void* mla_sin, const void* idx_cos, const void* idx_sin,
                    const int64_t* positions, uint8_t* index_q, float* index_w, void* q_full,
                    uint8_t* cache_index_k, float* cache_k_scale, void* cache_kv,
                    int B, int H, int n_index_heads, int64_t cap, int interleave, float eps,
                    void* stream);

/* Serving-form indexer staging: what the serving model's indexer does to the new
 * token between its projection GEMVs and the scan
 * (src/lagged_indexer_dsa/inference/modeling/transformer.py:1015-1066
 * Indexer.stage_fp8_operands), one launch:
 *   k = LayerNorm(k_raw) (fp32, weight + bias, :418-433); rotary embedding of dims 0..63 of
 *   every query head and of k (:525-547; rope_interleave 1: pairs (2i, 2i+1), 0: pairs
 *   (i, i+32)); 128-point Hadamard rotation times 128^-0.5 (:550-592); act_quant over the 128
 *   dims (inference/modeling/kernels.py:19-117: scale = max(amax, 1e-4) / 448, or its next
 *   power of two when round_scale != 0); index_q <- query bytes, index_w <- w_raw * head_scale *
 *   q_scale * softmax_scale (:1063-1065, head_scale = heads^-0.5); the key's bytes and scale
 *   are appended at positions[b] (:1061-1062) in the dense cache (pages NULL) or in 64-token
 *   pages of DSA_INDEX_PAGE_BYTES addressed through page_table [B, pt_stride]; the pool holds
 *   num_pages pages and pt_stride * 64 >= cap is required. A page-table entry outside
 *   [0, num_pages) is not followed: that token is skipped and a bit is set in the device status
 *   word (dsa_check_device_status). The paged scan treats such an entry the same way (the keys
 *   behind it get logit -inf).
 * q_raw bf16 [B, n_heads, 128]; k_raw bf16 [B, 128]; w_raw fp32 [B, n_heads]; k_norm_weight /
 * k_norm_bias fp32 [128]; rope_cos / rope_sin fp32 [cap, 32] (real / imaginary part of the
 * reference's freqs_cis); positions int64 [B]. Rounding follows the reference's op sequence
 * (bf16 after LayerNorm, after the rotary embedding and after the rotation). */
int dsa_indexer_stage_fp8(const void* q_raw, const void* k_raw, const float* w_raw,
                          const float* k_norm_weight, const float* k_norm_bias, float k_norm_eps,
                          const float* rope_cos, const float* rope_sin, const int64_t* positions,
                          uint8_t* index_q, float* index_w, uint8_t* cache_index_k,
                          float* cache_k_scale, uint8_t* pages, int64_t num_pages,
                          const int32_t* page_table, int64_t pt_stride, int B, int n_heads, int64_t cap,
                          int rope_interleave, int round_scale, float head_scale, float softmax_scale,
                          void* stream);

/* Serving-form latent append: the new token's latent row between wkv_a and the cache
 * (src/lagged_indexer_dsa/inference/modeling/transformer.py:3264-3276): RMSNorm of the 512
 * latent dims (fp32 weight, :380-410), rotary embedding of the 64 rope dims (:525-547),
 * written at row slots[b] of `pool` as
 *   format 0: bf16 [512 | 64];
 *   format 1: bf16 [512 | 64] whose latent dims went through act_quant and back (one e4m3
 *             scale per 128 dims, dequantised, rounded to bf16: what the reference's bf16
 *             cache holds, :3268-3274);
 *   format 2: the serving pool's DSA_FP8_LATENT_ROW bytes: 512 e4m3 | 4 fp32 scales | 64 bf16
 *             (kernels/cuda_fused_sparse_splitk.py:1098-1104), the rows
 *             dsa_sparse_mla_* reads with kv_fp8 = 1.
 * kv_a bf16 [B, 576]; kv_norm_weight fp32 [512]; rope tables fp32 [cap, 32]; positions and
 * slots int64 [B] (slot < 0 or >= n_slots: the row is skipped); round_scale as in
 * dsa_indexer_stage_fp8. */
int dsa_latent_append(const void* kv_a, const float* kv_norm_weight, float eps, const float* rope_cos,
                      const float* rope_sin, const int64_t* positions, const int64_t* slots, void* pool,
                      int B, int64_t cap, int64_t n_slots, int rope_interleave, int format,
                      int round_scale, void* stream);

/* ---- (a7) per-token e4m3 quantisation of index keys / queries --------------
 * scale = max(amax(row), clamp_min) / 448, q = sat(x / scale) -> e4m3 RN
 * (kernels/cuda_fused_sparse_splitk.py:2969-2974). x is fp32 [rows, cols]. */
int dsa_quantize_e4m3_rowwise(const float* x, uint8_t* q_out, float* scale_out,
                              int64_t rows, int cols, float clamp_min, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* DSA_B200_H_ */
