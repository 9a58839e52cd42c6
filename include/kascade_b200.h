/*
 * kascade_b200 — C ABI of the B200 (sm_100a) Kascade sparse-attention kernels.
 *
 * One shared library, libkascade_b200.so, replaces the seven per-kernel shared objects the
 * reference builds at strategy construction (strategies/EfficientKascadeStrategy.py:22-70), each of
 * which exports `init`, `call`, `get_last_error`
 * (kernels/flash_attention/kascade_prefill_cu_kernels/dynamic_alllen_reuse_cp_async_ts32_dim128_gsize4_heads32_groups8_rolling.cu:249-319).
 *
 * Conventions
 *  - every pointer is a DEVICE pointer unless the comment says "host"; fp16 data is IEEE binary16;
 *  - strides are in ELEMENTS, the head dimension D is contiguous and must be 128;
 *  - query heads per KV head (H / G) must be 4, the prefill query tile is 32 queries — the one
 *    shape the reference compiles (README.md:74, file names `ts32_dim128_gsize4`);
 *  - every call is asynchronous on `stream` (a cudaStream_t passed as void*), allocates nothing,
 *    copies nothing between host and device and never synchronises; the caller owns all memory,
 *    including the workspaces whose sizes the *_workspace_bytes functions return;
 *  - return value 0 = launched, non-zero = rejected (nothing launched); the reason is returned by
 *    kb200_last_error() for the calling thread.
 *  - logits are kept in the log2 domain like the reference's kernels
 *    (kernels/flash_attention/recompute_kascade_gqa_prefill.py:266-272):
 *    lse2 = log2(sum_j exp2(s_j * scale * log2 e)).
 */
#ifndef KASCADE_B200_H_
#define KASCADE_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* storage types of activations and KV caches (field `dtype` of the layouts; 0 = fp16, so a zero-initialised
 * layout is fp16).  bf16 is the native type of Qwen3; both go through the same tensor-core path
 * (tcgen05 kind::f16 / mma.sync), probabilities are rounded to the activations' type, accumulation is fp32,
 * outputs are written in the activations' type. */
#define KB200_FP16 0
#define KB200_BF16 1
#define KB200_FP8_E4M3 2   /* KV caches of the decode calls only, see kb200_kv_layout */

#define KB200_HEAD_DIM 128
#define KB200_GROUP_SIZE 4
#define KB200_TILE 32

/* ---- library ---------------------------------------------------------------------------------- */

/* Replaces `init()` of every reference kernel library (…_rolling.cu:249-258): selects nothing,
 * allocates nothing; raises the dynamic shared-memory limits of the kernels on `device` and checks
 * that the device is an sm_100 part.  Must be called once per device before any other call. */
int kb200_init(int device);

/* Replaces `get_last_error()` (…_rolling.cu:245-247).  Thread-local, never NULL. */
const char* kb200_last_error(void);

/* ABI version of this header. */
int kb200_abi_version(void);

/* Every device-side wait of the tensor-core kernels is bounded; a kernel that gives up records a
 * non-zero code in a device status word, releases what it holds and returns.  This call copies
 * that word to *host_out (host pointer) and clears it.  It synchronises the device, so call it at
 * a point where the caller synchronises anyway.  0 = no kernel gave up.  No counterpart in the
 * reference (its kernels spin without a limit). */
int kb200_read_status(int* host_out);

/* Number of tensor-map descriptors the prefill entry points have encoded so far in this process.  The
 * descriptors are kept per (pointer, strides, extents), so a loop over the same buffers stops encoding after
 * its first pass; the counter lets a host check that.  No counterpart in the reference. */
long long kb200_tensor_map_encodes(void);

/* ---- Top-k selection (replaces the torch.topk call sites,
 *      strategies/EfficientKascadeStrategy.py:82,90,111) ---------------------------------------- */

/* Exact Top-k of each row of a fp32 score matrix by radix select.
 *   scores      [rows, row_stride]      only the first n_valid[r] entries of row r are candidates
 *   n_valid     [rows] int32            (NULL: every row has n_cols candidates)
 *   k_row       [rows] int32            budget of row r, capped at k_max (NULL: k_max for every row)
 *   out_idx     [rows, idx_stride] int32, idx_stride >= k_max; receives min(k_row[r], k_max,
 *                                       n_valid[r]) indices in ASCENDING
 *                                       index order; entries beyond that count are left untouched
 *   out_count   [rows] int32            receives that count
 * Ties at the k-th score are resolved towards the lowest index.  NaNs are not supported. */
int kb200_topk_select(const float* scores, int64_t row_stride, int n_cols, const int32_t* n_valid,
                      const int32_t* k_row, int k_max, int32_t* out_idx, int64_t idx_stride,
                      int32_t* out_count, int64_t rows, void* stream);

/* ---- paged decode (replaces kernels/flash_decoding/reuse_kascade_gqa_decode.py:50-134 and
 *      recompute_kascade_gqa_decode.py:49-315; the reference has no paged variant, README.md:135;
 *      the closest signature is reuse_kascade_gqa_decode_with_kvcache.py:160-171) --------------- */

/* Address of the 128-element row of token `pos` of sequence `b`, KV head `g`:
 *   page = block_table ? block_table[b * block_table_stride + pos / page_size] : pos / page_size
 *   base + b * stride_batch + page * stride_page + (pos % page_size) * stride_token + g * stride_head
 * vLLM-style paged cache [num_pages, page_size, G, D]: stride_batch = 0.  Contiguous HF cache
 * [B, G, L, D]: block_table = NULL, stride_batch = G*L*D, stride_page = page_size*D,
 * stride_token = D, stride_head = L*D. */
typedef struct kb200_kv_layout {
  const void* k;              /* fp16 or bf16, see dtype */
  const void* v;              /* same type as k, may be NULL where a call says so */
  int64_t stride_batch;
  int64_t stride_page;
  int64_t stride_token;
  int64_t stride_head;
  const int32_t* block_table; /* [B, block_table_stride] or NULL */
  int32_t block_table_stride;
  int32_t page_size;          /* power of two, >= 1 */
  int32_t dtype;              /* KB200_FP16 / KB200_BF16: type of the cache, of q and of the output of a decode call;
                                 KB200_FP8_E4M3: the cache holds e4m3 bytes (strides in bytes, multiples of 16), q and
                                 the output are fp16 */
  /* FP8 caches: value = stored e4m3 value x scale, one fp32 scale per (page, KV head), K and V separately:
   *   k_scale[b * scale_stride_batch + page * scale_stride_page + g * scale_stride_head]   (page as in the address
   * rule above: physical page with a block table).  The kernels turn the stored bytes into fp16 exactly and
   * apply the scales in fp32 (on the key's logit, on its probability before P.V).  Halves the bytes a decode
   * step moves.  The reference has no quantised cache. */
  const float* k_scale;
  const float* v_scale;
  int64_t scale_stride_batch;
  int64_t scale_stride_page;
  int64_t scale_stride_head;
} kb200_kv_layout;

/* Workspace for kb200_decode_sparse_paged / kb200_decode_anchor_paged (split-K partials). */
size_t kb200_decode_workspace_bytes(int batch, int num_q_heads, int num_splits);
/* Number of splits the library would choose (num_splits = 0) for this problem. */
int kb200_decode_default_splits(int batch, int num_kv_heads, int max_keys);

/* Sparse (reuse-layer) decode: attention of one query token per sequence over the key rows
 * listed in topk_idx.   (K8 + K9 of the reference: reuse_kascade_gqa_decode.py:50-200)
 *   q           [B, H, D] fp16, strides q_stride_b / q_stride_h
 *   topk_idx    [B, G, idx_stride_g…] int32 logical token positions; row of KV head g of
 *               sequence b starts at topk_idx + b*idx_stride_b + g*idx_stride_g
 *   topk_count  [B, G] int32 number of valid entries per row (NULL: k_max everywhere)
 *   head_map    [G] int32: KV head g reads the index row of KV head head_map[g] (NULL: identity)
 *   out         [B, H, D] fp16 contiguous
 *   lse2_out    [B, H] fp32 or NULL
 * Rows with zero valid keys produce zeros. */
int kb200_decode_sparse_paged(const void* q, int64_t q_stride_b, int64_t q_stride_h,
                              const kb200_kv_layout* kv, const int32_t* topk_idx,
                              int64_t idx_stride_b, int64_t idx_stride_g,
                              const int32_t* topk_count, int k_max, const int32_t* head_map,
                              float softmax_scale, void* out, float* lse2_out, void* workspace,
                              size_t workspace_bytes, int batch, int num_q_heads, int num_kv_heads,
                              int num_splits, void* stream);

/* Sparse decode for callers that cannot allocate.  No counterpart in the reference.
 *
 * Some hosts of this library have no way to give it a workspace: an inference server that hands all
 * free HBM to its KV-cache pool at start-up and treats any later cudaMalloc as a bug, a plugin slot
 * whose interface carries only inputs and outputs, a latency-critical loop that must not take the
 * allocator lock.  For them this entry point computes exactly what kb200_decode_sparse_paged
 * computes, with the split partials kept in a fixed array inside the library image instead of a
 * caller-owned workspace.  It calls no cudaMalloc / cudaFree and no allocating library routine.
 *
 *  - Limit: batch * num_q_heads * num_splits <= KB200_NOALLOC_MAX_SLOTS (4.06 MiB of partials, held
 *    by every GPU that loads the library until the process exits).  With num_splits = 0 the library
 *    lowers its own choice until it fits; an explicit num_splits that does not fit is rejected with
 *    a message, nothing is launched.  num_splits = 1 needs no scratch and always fits.
 *  - The first call on a device that uses more than one split looks up the array's device address
 *    (cudaGetSymbolAddress) with that device current, and caches it; make that first call during set-up,
 *    before any stream capture.
 *    The device that is current at the call must be the one that owns the pointers.
 *  - All calls on a device share the one array.  Nothing in it has to start at zero — every slot the
 *    merge step reads is written earlier in the same call — but two calls that overlap on the GPU
 *    (different streams, or different host threads) race on it: serialise them, or use the variant
 *    with a workspace.
 * Arguments as kb200_decode_sparse_paged, without workspace / workspace_bytes. */
#define KB200_NOALLOC_MAX_SLOTS 8192
/* Splits kb200_decode_sparse_paged_noalloc uses for this problem and this num_splits argument
 * (0 = the call would be rejected); with 1 split the call launches one kernel, otherwise two. */
int kb200_decode_noalloc_splits(int batch, int num_q_heads, int num_kv_heads, int k_max, int num_splits);
int kb200_decode_sparse_paged_noalloc(const void* q, int64_t q_stride_b, int64_t q_stride_h,
                                      const kb200_kv_layout* kv, const int32_t* topk_idx,
                                      int64_t idx_stride_b, int64_t idx_stride_g,
                                      const int32_t* topk_count, int k_max, const int32_t* head_map,
                                      float softmax_scale, void* out, float* lse2_out, int batch,
                                      int num_q_heads, int num_kv_heads, int num_splits, void* stream);

/* Anchor-layer decode: dense pass over all seq_lens[b] cached keys.  Writes the scaled base-2
 * logits of every (head, key), the per-head lse2, optionally the dense output, and the pooled
 * post-softmax score  pooled[b,g,j] = sum_{h in group g} exp2(logit[b,h,j] - lse2[b,h])
 * that kb200_topk_select consumes.  (K5 + K6 + K7: recompute_kascade_gqa_decode.py:49-315)
 *   seq_lens    [B] int32
 *   logits      [B, H, logit_stride] fp32 scratch (logit_stride >= max seq len)
 *   pooled      [B, G, logit_stride] fp32
 *   out         [B, H, D] fp16 or NULL (NULL: K only — anchor layers > 0 read no V)
 *   lse2_out    [B, H] fp32 (required) */
int kb200_decode_anchor_paged(const void* q, int64_t q_stride_b, int64_t q_stride_h,
                              const kb200_kv_layout* kv, const int32_t* seq_lens, int max_seq_len,
                              float softmax_scale, float* logits, float* pooled,
                              int64_t logit_stride, void* out, float* lse2_out, void* workspace,
                              size_t workspace_bytes, int batch, int num_q_heads, int num_kv_heads,
                              int num_splits, void* stream);

/* ---- tile prefill (replaces kernels/flash_attention/recompute_kascade_gqa_prefill.py:191-312 and
 *      reuse_kascade_gqa_prefill.py:146-198) --------------------------------------------------- */

/* Token-major activations: element (b, token, head, d) at
 *   base + b*stride_b + token*stride_t + head*stride_h + d. */
typedef struct kb200_act_layout {
  const void* ptr; /* fp16 or bf16, see dtype */
  int64_t stride_b;
  int64_t stride_t;
  int64_t stride_h;
  int32_t dtype;   /* KB200_FP16 / KB200_BF16; q, k and v of a call must agree, `out` is written in the same type */
} kb200_act_layout;

/* Dense causal attention of a whole prompt, one CTA per (32-query tile, KV head, batch).
 *   out   [B, L, H, D] fp16 contiguous, or NULL for the lse-only pass (then v is not read)
 *   lse2  [B, L, H] fp32, or NULL
 * (K1 `prefill` and K2 `compute_scores`: recompute_kascade_gqa_prefill.py:224-312) */
int kb200_prefill_dense(const kb200_act_layout* q, const kb200_act_layout* k,
                        const kb200_act_layout* v, float softmax_scale, void* out, float* lse2,
                        int batch, int seq_len, int num_q_heads, int num_kv_heads, void* stream);

/* Tile-pooled post-softmax scores of an anchor layer:
 *   pooled[b,g,t,j] = sum_{32 queries i of tile t} sum_{4 heads h of group g}
 *                     exp2(q_ih . k_j * scale * log2 e - lse2[b,i,h])      for j < 32*t
 * Entries j >= 32*t of a row are not written (kb200_topk_select is given n_valid = 32*t).
 *   pooled  [B, G, T, row_stride] fp32, T = ceil(L/32), row_stride >= L rounded up to 128
 * (K3 `aggregate`: recompute_kascade_gqa_prefill.py:171-222 and
 *  dynamic_alllen_aggregate_cp_async_ts32_dim128_gsize4_heads32_groups8.cu) */
int kb200_prefill_pool_scores(const kb200_act_layout* q, const kb200_act_layout* k,
                              const float* lse2, float softmax_scale, float* pooled,
                              int64_t row_stride, int batch, int seq_len, int num_q_heads,
                              int num_kv_heads, void* stream);

/* Sparse tile attention of a reuse layer (or of an anchor layer > 0 over its own fresh rows):
 * query i of tile t attends to the keys tile_idx[b, head_map[g], t, 0:tile_count[…]] (all
 * strictly before the tile) and to the keys 32*t .. i of its own tile.
 *   tile_idx    [B, Gi, T, idx_stride] int32, ascending or any order, no duplicates
 *   tile_count  [B, Gi, T] int32
 *   idx_kv_heads  Gi, the number of KV heads the index tensors hold (0: num_kv_heads).  When the
 *               KV heads of a layer are sharded over GPUs, a call covers num_kv_heads local heads
 *               while the index tensors hold the rows of all Gi heads of the anchor layer.
 *   head_map    [num_kv_heads] int32 with values in [0, Gi), or NULL (identity, needs Gi == num_kv_heads)
 *   out         [B, L, H, D] fp16 contiguous;  lse2 [B, L, H] fp32 or NULL
 * (K4 `main_kernel`: reuse_kascade_gqa_prefill.py:146-198 and the two
 *  dynamic_alllen_reuse_cp_async_ts32_dim128_gsize4_heads32_groups8[_rolling].cu) */
int kb200_prefill_sparse(const kb200_act_layout* q, const kb200_act_layout* k,
                         const kb200_act_layout* v, const int32_t* tile_idx, int64_t idx_stride,
                         const int32_t* tile_count, const int32_t* head_map, float softmax_scale,
                         void* out, float* lse2, int batch, int seq_len, int num_q_heads,
                         int num_kv_heads, int idx_kv_heads, void* stream);

/* ---- ragged batches in one launch ---------------------------------------------------------------
 * A batch whose prompts differ in length (left- or right-padded by the tokenizer, or simply of different
 * lengths inside equally sized slots) runs through the same persistent kernels in ONE launch per kernel:
 * sequence b occupies rows seq_start[b] .. seq_start[b] + seq_len[b] - 1 of its slot of max_len rows
 * (element (b, seq_start[b] + token, head, d) of every activation, row seq_start[b] + token of `out`); tiles
 * beyond a sequence's end are skipped, key positions and index rows are relative to the sequence's first
 * token.  The reference has no varlen prefill (README.md:135 lists it as future work; its only length
 * argument is cache_seqlens of kernels/flash_decoding/reuse_kascade_gqa_decode_with_kvcache.py:160-171).
 *   seq_start [B] int32 device, or NULL (every sequence starts at row 0: right padding)
 *   seq_len   [B] int32 device, 0 <= seq_len[b], seq_start[b] + seq_len[b] <= max_len
 * lse2 [B, max_len, H] and pooled [B, G, ceil(max_len/32), row_stride] are indexed by the token / tile number
 * inside the sequence. */
typedef struct kb200_ragged {
  const int32_t* seq_start;
  const int32_t* seq_len;
} kb200_ragged;
int kb200_prefill_dense_ragged(const kb200_act_layout* q, const kb200_act_layout* k,
                               const kb200_act_layout* v, float softmax_scale, void* out, float* lse2,
                               const kb200_ragged* ragged, int batch, int max_len, int num_q_heads,
                               int num_kv_heads, void* stream);
int kb200_prefill_pool_scores_ragged(const kb200_act_layout* q, const kb200_act_layout* k,
                                     const float* lse2, float softmax_scale, float* pooled,
                                     int64_t row_stride, const kb200_ragged* ragged, int batch, int max_len,
                                     int num_q_heads, int num_kv_heads, void* stream);
int kb200_prefill_sparse_ragged(const kb200_act_layout* q, const kb200_act_layout* k,
                                const kb200_act_layout* v, const int32_t* tile_idx, int64_t idx_stride,
                                const int32_t* tile_count, const int32_t* head_map, float softmax_scale,
                                void* out, float* lse2, const kb200_ragged* ragged, int batch, int max_len,
                                int num_q_heads, int num_kv_heads, int idx_kv_heads, void* stream);
/* Budgets of a ragged batch for kb200_topk_select, per sequence by the reference's formulas
 * (strategies/KascadeStrategy.py:127-139) for a prompt of seq_len[b] tokens:
 *   k_b = min(max(128, int(pct/100 * seq_len[b])), seq_len[b]) - 32,
 *   n_valid[b,g,t] = 32*t, k_row[b,g,t] = min(k_cap, rolling ? min(k_b, max(128, floor(pct*32*t/100))) : k_b)
 * for tiles inside the sequence, 0 / 0 for tiles beyond its end.  k_cap = row length of the index tensor. */
int kb200_prefill_budgets_ragged(int32_t* n_valid, int32_t* k_row, const int32_t* seq_len, int batch,
                                 int num_kv_heads, int num_tiles, int k_cap, float pct, int rolling, void* stream);

/* Output fan-out for prompts whose KV heads are sharded over GPUs: the rows a call computes (its
 * num_q_heads heads) are stored by the kernel's epilogue into `count` buffers, each
 * [B, L, total_heads, D] fp16 contiguous, at heads [head_offset, head_offset + num_q_heads).  out[0] is
 * normally this GPU's own buffer, the others are peer GPUs' buffers mapped into this process (CUDA IPC
 * or symmetric memory; plain stores over NVLink, no multicast).  Every GPU then holds all heads of a
 * layer once all GPUs' kernels have finished — the caller synchronises the GPUs before reading.
 * The reference all-gathers nothing (single GPU); this replaces the all-gather of per-head outputs. */
#define KB200_MAX_FANOUT 8
typedef struct kb200_out_fanout {
  void* out[KB200_MAX_FANOUT];
  int32_t count;
  int32_t total_heads;
  int32_t head_offset;
  int32_t multicast;   /* 0: plain addresses.  1: count must be 1 and out[0] is the address of an NVLink multicast
                          object (NVLS: one mapping that stands for the same buffer on every GPU of the group); the
                          epilogue then stores every row ONCE with multimem.st and the NVSwitch delivers it to all
                          GPUs, this one included: the egress of a rank is its own slice, not (GPUs - 1) copies of it. */
} kb200_out_fanout;

/* kb200_prefill_dense / kb200_prefill_sparse with the output rows fanned out (see kb200_out_fanout);
 * all other arguments as in the plain entry points, lse2 (if given) stays local [B, L, num_q_heads]. */
int kb200_prefill_dense_fanout(const kb200_act_layout* q, const kb200_act_layout* k,
                               const kb200_act_layout* v, float softmax_scale,
                               const kb200_out_fanout* fan, float* lse2, int batch, int seq_len,
                               int num_q_heads, int num_kv_heads, void* stream);
int kb200_prefill_sparse_fanout(const kb200_act_layout* q, const kb200_act_layout* k,
                                const kb200_act_layout* v, const int32_t* tile_idx, int64_t idx_stride,
                                const int32_t* tile_count, const int32_t* head_map, float softmax_scale,
                                const kb200_out_fanout* fan, float* lse2, int batch, int seq_len,
                                int num_q_heads, int num_kv_heads, int idx_kv_heads, void* stream);

/* Output exchange by the copy engines, for prompts whose KV heads are sharded over the GPUs of one node
 * (alternative to kb200_out_fanout: from four GPUs on, the NVLink time of a reuse layer exceeds its compute
 * time, and stores issued by the kernel hold it up).  The kernel writes its heads into this GPU's own
 * [rows, pitch] buffer; kb200_peer_push then copies that slice (width_bytes at offset_bytes of every row) into
 * the same place of every peer's buffer: one strided 2-D device-to-device copy per peer, each on the stream the
 * plan names, ordered after everything queued on compute_stream so far (ready_event is recorded there) and
 * followed by a record of done_event[i].  No SM is used; the next layer's kernels run meanwhile.  The caller
 * owns streams and events (cudaStream_t / cudaEvent_t passed as void*), makes the compute stream wait for the
 * done events before it overwrites the slice (kb200_stream_wait_events), and synchronises the GPUs before
 * anyone reads a peer-written buffer.  The reference all-gathers nothing (single GPU). */
typedef struct kb200_push_plan {
  void* dst[KB200_MAX_FANOUT];        /* peers' buffers (mapped into this process), same shape as the source */
  void* stream[KB200_MAX_FANOUT];     /* one copy stream per peer */
  void* done_event[KB200_MAX_FANOUT]; /* recorded on stream[i] after the copy to peer i */
  int32_t count;
} kb200_push_plan;
int kb200_peer_push(const kb200_push_plan* plan, const void* src_base, size_t offset_bytes, size_t pitch_bytes,
                    size_t width_bytes, size_t rows, void* ready_event, void* compute_stream);
/* Makes `stream` wait for `count` events (NULL entries are skipped).  Host-side helper of kb200_peer_push. */
int kb200_stream_wait_events(void* stream, void* const* events, int count);

/* Per-tile budgets of an anchor prefill layer, written on the device for kb200_topk_select:
 *   n_valid[b,g,t] = 32*t,
 *   k_row[b,g,t]   = rolling ? min(k_max, max(128, floor(pct * 32*t / 100))) : k_max
 * (strategies/KascadeStrategy.py:127-139). */
int kb200_prefill_budgets(int32_t* n_valid, int32_t* k_row, int batch, int num_kv_heads,
                          int num_tiles, int k_max, float pct, int rolling, void* stream);

/* ---- KV-cache write path ----------------------------------------------------------------------
 * One pass over the new tokens of every sequence: optional per-head RMS norm of Q and K (Qwen3),
 * rotary position embedding of Q and K, and the append of the new K / V rows to the cache in the layout
 * the attention kernels read.  The reference has no such kernel: it receives rotated q/k/v from the
 * Hugging Face attention module and pays transposes and `.contiguous()` copies before every kernel
 * call (strategies/EfficientKascadeStrategy.py:144-150).  Arithmetic follows the Hugging Face modules
 * step by step in the model's type - fp16 or bf16, the `dtype` of the layouts, which must all agree
 * (LlamaRMSNorm, LlamaRotaryEmbedding, apply_rotary_pos_emb: fp32 norm rounded to that type, gain applied in
 * that type, cos / sin in fp32 rounded to that type, products and sum in that type).
 *   q_in        [B, T, H, D] view, or NULL (then q_out is ignored); q_out [B, T, H, D] contiguous, same type
 *   k_new/v_new [B, T, G, D] views: the rows to append (T = max_new)
 *   start_pos   [B] int32: cache length of each sequence before the append (position of its first new token)
 *   n_new       [B] int32 number of new tokens per sequence (<= max_new), or NULL (= max_new)
 *   kv          the cache (written): paged with a block table that already covers the new positions, or contiguous;
 *               or an FP8 cache (dtype KB200_FP8_E4M3, k_scale / v_scale given by the caller, e.g. calibrated per
 *               layer): a row is stored as value / scale of its page and KV head (fp32 division, saturating at
 *               +-448, round to nearest even) - the bytes the decode entry points read back as byte x scale
 *   q_norm_gain / k_norm_gain  [D] in the same type, or NULL (no norm);  norm_eps
 *   inv_freq    [D/2] fp32 inverse frequencies of the model's rotary embedding (device memory), or NULL
 *               (no rotary);  rope_scale multiplies cos and sin (1 for the default rope type)
 */
int kb200_kv_write(const kb200_act_layout* q_in, void* q_out, const kb200_act_layout* k_new,
                   const kb200_act_layout* v_new, const int32_t* start_pos, const int32_t* n_new,
                   const kb200_kv_layout* kv, const void* q_norm_gain, const void* k_norm_gain,
                   float norm_eps, const float* inv_freq, float rope_scale, int batch, int max_new,
                   int num_q_heads, int num_kv_heads, void* stream);

/* ---- diagnostics ----------------------------------------------------------------------------- */

/* Runs four 128x128x128 fp16 products through the tensor-core paths the prefill kernels rely on
 * (A/B from shared memory K-major; B MN-major; A from tensor memory) and writes the fp32 results:
 *   a, b [128,128] fp16 row-major;  out [4, 128, 128] fp32
 *   out[0] = a . b^T   out[1] = a . b   out[2] = a . b^T (A via tensor memory)   out[3] = a . b (A via tensor memory)
 *   status [4] int32: 0 ok, non-zero = a bounded wait gave up.
 * No counterpart in the reference. */
int kb200_selftest_umma(const void* a, const void* b, float* out, int32_t* status, void* stream);

/* Exercises the give-up path of the bounded device-side waits without hanging anything: one CTA allocates
 * tensor memory, then all its threads wait for at most limit_ns (0 < limit_ns <= 100 ms) on a barrier on
 * which nobody arrives.  The wait runs out, the CTA frees its tensor memory, records `code` (1..255) in the
 * device status word that kb200_read_status returns and clears, and returns.
 *   result [3] int32: code the CTA ended with, threads whose wait returned "gave up", elapsed ns.
 * While the status word is non-zero the tile prefill kernels return at entry; read it to clear it.
 * No counterpart in the reference (its kernels spin without a limit). */
int kb200_selftest_wait_timeout(int32_t* result, uint64_t limit_ns, int code, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* KASCADE_B200_H_ */
