/*
 * omnikv_b200 -- C ABI of the B200 (sm_100a) kernels behind OmniKV's decode-time
 * context selection.
 *
 * The reference (antgroup/OmniKV) has no native boundary: its "plugin API" is
 * Python (modeling/omnikv.py, modeling/spec_cache.py).  Each entry point below
 * names the reference lines whose GPU work it replaces; the Python classes in
 * omnikv_b200/modeling keep the reference's names and call these through ctypes.
 *
 * Conventions
 *   - raw device pointers (tensor.data_ptr()), explicit sizes and ELEMENT strides;
 *   - the caller owns every buffer, workspaces included: nothing here allocates,
 *     frees or synchronises, so every call may be captured in a CUDA graph;
 *   - per-sequence lengths are DEVICE arrays of int32 so that a captured graph can
 *     be replayed while the context grows;
 *   - the last argument is the cudaStream_t to launch on (passed as void*);
 *   - return value: 0 or a negative omnikv_status after host-side validation;
 *     nothing throws or aborts across the boundary;
 *   - head_dim is 128 (Llama-3 8B / 70B); other values return OMNIKV_E_UNSUPPORTED.
 *   - process-wide switches, read ONCE from the environment on first use (the only global state besides the
 *     built-in scratch of omnikv_decode_attn_no_alloc): OMNIKV_PDL=0 launches every kernel without programmatic
 *     dependent launch; OMNIKV_ATTN_TMA=0 keeps dense decode attention on its cp.async variant;
 *     OMNIKV_WINDOW_TMA=0 does the same for the window selector's mma.sync kernels; OMNIKV_WINDOW_TC=0 keeps the
 *     window selector off its tcgen05 kernels; OMNIKV_TOPK_CLUSTER=8 limits omnikv_topk to the portable cluster size.
 *     OMNIKV_ATTN_COOP=0 has every split merge of decode attention done by the last CTA of its group (by default a dense
 *     layer with 64 splits or more on a grid that is resident as a whole merges them across all of its CTAs).
 *     They exist for measurements and fault isolation; results are the same up to the order of fp32 sums.
 */
#ifndef OMNIKV_B200_H_
#define OMNIKV_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define OMNIKV_ABI_VERSION 5

typedef enum {
  OMNIKV_OK = 0,
  OMNIKV_E_BADARG = -1,      /* null pointer, non-positive size, bad stride or alignment */
  OMNIKV_E_UNSUPPORTED = -2, /* shape or dtype outside what the kernels are built for   */
  OMNIKV_E_WORKSPACE = -3,   /* workspace missing or smaller than omnikv_*_workspace_bytes */
  OMNIKV_E_CUDA = -4         /* a CUDA runtime call failed; see omnikv_last_cuda_error()  */
} omnikv_status;

typedef enum { OMNIKV_F32 = 0, OMNIKV_BF16 = 1, OMNIKV_F16 = 2 } omnikv_dtype;

/* Window selectors of modeling/omnikv.py:49-105. */
typedef enum {
  OMNIKV_SEL_SOFTMAX_LAST = 0, /* "softmax_before_last" :49-58  */
  OMNIKV_SEL_UNIFORM = 1,      /* "uniform"             :59-80  */
  OMNIKV_SEL_EXP = 2           /* "exp"                 :81-105 */
} omnikv_window_selector;

int omnikv_abi_version(void);
const char* omnikv_strerror(int status);
/* Text of the last CUDA error seen by this library on the calling thread ("" if none). */
const char* omnikv_last_cuda_error(void);

/* ------------------------------------------------------------------------------------------
 * Decode attention over a list of KV rows, with optional selection-score output.
 *
 * One query token per sequence.  The rows a sequence attends to are the concatenation of
 *   segment A: lenA[b] rows of (kA, vA); row j is cache position idxA[b][j] when idxA is
 *              given, else position j;
 *   segment B: lenB[b] consecutive rows of (kB, vB) starting at position startB[b].
 * out[b,h,:] = softmax_j(q[b,h,:] . K_j * scale) V_j with query head h reading KV head
 * h / (H / KVH).
 *
 *   dense layer  (modeling/spec_cache.py:358-369 + the attention call modeling/omnikv.py:219-227):
 *       A = the whole cache, idxA = NULL, lenA = prompt + decoded tokens; lenB = NULL.
 *   sparse layer (modeling/spec_cache.py:337-356: cat([part_key, tail_k])):
 *       A = prompt rows at the selected indices (replaces the index_select of :297-303 and
 *       the torch.cat of :349-356: no gathered copy is materialised), B = the decode-time tail.
 *   offloaded sparse layer: A = the staged rows written by omnikv_offload_gather (idxA = NULL).
 *   paged pool (omnikv-lightllm/lightllm/common/mem_manager.py:102-104, req_manager.py:12-17): A = the pool
 *       [tokens, 2*KVH, d] (a_stride_b = 0, a_stride_h = d, a_stride_row = 2*KVH*d; V = K + KVH*d),
 *       idxA = req_to_token_indexs, idx_row = b_req_idx, lenA = b_seq_len.
 *
 * score_out (optional): the filter layer's selection score of selector "last"
 * (modeling/omnikv.py:40-46) for free while K streams through: for every position
 * p < score_len[b] of segment A (the position j, not the cache row it maps to),
 * score_out[kvh][b][p] = max over the query heads of KV head kvh of the scaled raw logit.  The max over KV heads is taken by omnikv_topk (n_planes = KVH), or by a
 * MAX all-reduce of the planes when KV heads are sharded over GPUs.
 *
 * out == NULL with score_out != NULL computes scores only (V is never read).
 * ------------------------------------------------------------------------------------------ */
typedef struct {
  int32_t dtype;    /* omnikv_dtype of q, k, v, out */
  int32_t B, H, KVH, head_dim;
  float scale;      /* 1/sqrt(head_dim) */
  const void* q;    /* [B, H, d] */
  int64_t q_stride_b, q_stride_h;
  void* out;        /* [B, H, d], same strides as q; may be NULL (scores only) */
  /* segment A */
  const void* kA;
  const void* vA;
  int64_t a_stride_b, a_stride_h, a_stride_row; /* elements; a row is head_dim contiguous elements */
  const int32_t* idxA; /* device [B, idx_stride] or NULL */
  int64_t idx_stride;
  const int32_t* idx_row; /* device [B] or NULL: batch entry b uses row idx_row[b] of the index table instead of
                             row b (a paged pool shared by requests: the table has one row per request slot) */
  const int32_t* lenA; /* device [B] */
  /* segment B (all NULL / 0 when unused) */
  const void* kB;
  const void* vB;
  int64_t b_stride_b, b_stride_h, b_stride_row;
  const int32_t* startB; /* device [B] */
  const int32_t* lenB;   /* device [B] */
  /* optional score output */
  float* score_out;           /* device [KVH, B, score_stride] or NULL */
  int64_t score_stride;
  const int32_t* score_len;   /* device [B]: positions >= score_len[b] are not written */
  /* split-K */
  int32_t n_splits;           /* >= 1; rows of a sequence are cut into n_splits contiguous chunks */
  void* workspace;            /* omnikv_decode_attn_workspace_bytes(B, H, n_splits) bytes, 16-byte aligned.  Its first
                                 16 KiB are arrival counters (B*KVH <= 4096, n_splits <= 512): they must be ZERO before the first call
                                 that uses this workspace; every call leaves them zero.  Calls that share a workspace
                                 must not overlap on the GPU. */
  size_t workspace_bytes;
  int32_t* status;            /* optional device word: set to 5 if a bounded wait for a KV copy ran out (never
                                 in a healthy run); left untouched otherwise */
  int64_t a_rows;             /* optional: row capacity of segment A's cache (every row < a_rows of every (b, head)
                                 is readable memory).  When given for a 16-bit cache without idxA and without a
                                 segment B, tiles are fetched through a TMA tensor map; 0: unknown */
} omnikv_attn_params;

/* Stream order: the kernel is launched as a programmatic dependent launch (unless OMNIKV_PDL=0).  When the
 * call right before it on the stream is one of this library's weight-streaming calls (omnikv_decode_qkv ...),
 * the kernel reads the lengths, the index list and K/V rows OTHER than the last row of each sequence while
 * that call is still finishing; q, the last row and everything it writes wait for the call to complete.  So
 * such a call may produce q and the newest K/V row (what omnikv_decode_qkv does) but nothing else that this
 * kernel reads.  After any other kernel the launch is ordered like a plain one. */
size_t omnikv_decode_attn_workspace_bytes(int B, int H, int n_splits);
int omnikv_decode_attn(const omnikv_attn_params* p, void* stream);

/* ------------------------------------------------------------------------------------------
 * omnikv_decode_attn_no_alloc: omnikv_decode_attn for callers that have no way to allocate device
 * memory (no counterpart in the reference, whose tensors all come from PyTorch's allocator).
 *
 * Who needs it: code that is handed tensors but no allocator -- an operator plugged into another runtime
 * that owns all device memory, a process whose memory budget is fixed at start-up, a latency-critical loop
 * that must never reach cudaMalloc (which can block and synchronise the device).  The split partials and arrival counters that omnikv_decode_attn
 * takes from the caller's workspace come instead from a fixed array inside the library:
 * OMNIKV_NO_ALLOC_SCRATCH_BYTES (4 MiB) of device memory on every GPU that loads the library, held until
 * the process exits.  p->workspace and p->workspace_bytes are ignored; inputs and outputs are the caller's.
 *
 * Limit: omnikv_decode_attn_workspace_bytes(B, H, n_splits) must not exceed OMNIKV_NO_ALLOC_SCRATCH_BYTES
 * (B * H * n_splits <= 8034, e.g. batch 1, 32 heads, 251 splits); larger problems return OMNIKV_E_WORKSPACE.
 * A call that is refused -- for its size or for any argument omnikv_decode_attn would refuse -- puts nothing on
 * the stream and does not touch the array.  Nothing is allocated or freed, here or in any routine it calls.
 *
 * The first call on a device looks up the array's device address (cudaGetSymbolAddress, with that device
 * current); make that first call outside stream capture.  All calls on a device share the one array: it
 * keeps the previous call's contents (the counters are cleared at the start of every call, on the given
 * stream), and two calls that overlap on the GPU -- different streams, or graphs replayed concurrently --
 * race on it.  Keep them on one stream, or order them with events.  The first call may come from several host
 * threads at once (the address look-up is idempotent and its cache is atomic).  The clearing of the counters is a
 * memset node in front of the kernel, so unlike omnikv_decode_attn this call does not start early behind a
 * preceding weight-streaming call (no programmatic overlap).
 * ------------------------------------------------------------------------------------------ */
#define OMNIKV_NO_ALLOC_SCRATCH_BYTES (4 * 1024 * 1024)
int omnikv_decode_attn_no_alloc(const omnikv_attn_params* p, void* stream);

/* ------------------------------------------------------------------------------------------
 * Window-selector scores (modeling/omnikv.py:49-105), replaces the per-window-query Python
 * loop of matmul + softmax + max + sum and the repeat_kv copy of :38.
 *
 * qw [B, H, W, d]: rotated queries of the observation window, slot W-1 = current token.
 * For every position p < consider_len[b]:
 *   A[h,w,p] = softmax over p' < consider_len[b] of (qw[b,h,w,:] . K[b,h/G,p',:] * scale)
 *   score_out[b][p] = sum_w weight_w * max_h A[h,w,p]
 * with weight_w = 1 (uniform), 2^-(W-1-w) (exp), or only slot W-1 (softmax_before_last).
 * When planes_out is given instead (KV heads sharded over GPUs), planes_out[b][w][p] holds
 * max over the LOCAL heads, to be MAX-all-reduced and folded by omnikv_window_fold.
 * ------------------------------------------------------------------------------------------ */
typedef struct {
  int32_t dtype;
  int32_t B, H, KVH, head_dim, W;
  int32_t selector; /* omnikv_window_selector */
  float scale;
  const void* qw; /* [B, H, W, d] contiguous */
  const void* k;  /* [B, KVH, *, d] */
  int64_t k_stride_b, k_stride_h, k_stride_row;
  const int32_t* consider_len; /* device [B] */
  int32_t max_len;             /* host upper bound of consider_len, sizes the grid */
  float* score_out;            /* device [B, score_stride] or NULL */
  float* planes_out;           /* device [B, W, score_stride] or NULL */
  int64_t score_stride;
  void* workspace;
  size_t workspace_bytes;
  int32_t* status;             /* optional device word: set to 5 if a bounded wait for a K tile ran out */
} omnikv_window_params;

size_t omnikv_score_window_workspace_bytes(int B, int H, int W, int max_len);
int omnikv_score_window(const omnikv_window_params* p, void* stream);
/* score_out[b][p] = sum_w weight_w * planes[b][w][p] (after the MAX all-reduce of the planes). */
int omnikv_window_fold(const float* planes, float* score_out, int B, int W, int64_t score_stride,
                       const int32_t* consider_len, int max_len, int selector, void* stream);

/* ------------------------------------------------------------------------------------------
 * Top-k selector: replaces torch.topk(sorted=True) + torch.sort of the indices,
 * modeling/omnikv.py:47-48, :79, :105, :109.
 *
 * score[b][p] = max over planes pl < n_planes of scores[pl*plane_stride + b*batch_stride + p].
 * For every sequence: kk = min(k[b], len[b]); the kk positions with the largest score are
 * written to idx_out[b][0..kk) in ASCENDING position order (int32); among equal scores the
 * lowest position wins; NaN ranks above +inf (as torch.topk).  Then append_n[b] consecutive
 * positions len[b], len[b]+1, ... are appended (the prompt tokens still inside the observation
 * window, modeling/omnikv.py:199-210); count_out[b] = kk + append_n[b].
 * One thread-block cluster per sequence; radix select with shared-memory histograms.
 * ------------------------------------------------------------------------------------------ */
size_t omnikv_topk_workspace_bytes(int B, int max_len);
int omnikv_topk(const float* scores, int n_planes, int64_t plane_stride, int64_t batch_stride,
                const int32_t* len, const int32_t* k, const int32_t* append_n /* may be NULL */,
                int B, int max_len, int32_t* idx_out, int64_t idx_stride, int32_t* count_out,
                void* workspace, size_t workspace_bytes, void* stream);

/* ------------------------------------------------------------------------------------------
 * Lazy re-gather rule: replaces get_idx_iou_score + the skip test of OmniKVLazyCache.set_out_idx,
 * modeling/spec_cache.py:10-31, :539-548 (cache_cls "lazy"), without the .cpu() round trip.
 *
 * Per sequence b: new_idx[b][0..new_count[b]) is the selection just made, live_idx[b][0..live_count[b]) the
 * one in use (both ascending, no duplicates; live_count = 0: none yet).  With inter = |new & live|:
 * the new list REPLACES the one in use (copied into live_idx, live_count = new_count, applied[b] = 1)
 * unless inter / new_count > skip_threshold (compared in double, as the reference's Python floats), in
 * which case the one in use is kept (applied[b] = 0).  gather_n[b] (optional) = new_count[b] when replaced,
 * else 0: passed as n_idx to omnikv_offload_gather it turns the host gather into a no-op on kept steps.
 * overlap[b] (optional) = inter.  capacity bounds both counts; new_idx and live_idx must not alias.
 * ------------------------------------------------------------------------------------------ */
int omnikv_idx_commit(const int32_t* new_idx, int64_t new_stride, const int32_t* new_count, int32_t* live_idx,
                      int64_t live_stride, int32_t* live_count, int B, int capacity, double skip_threshold,
                      int32_t* applied, int32_t* gather_n /* may be NULL */, int32_t* overlap /* may be NULL */,
                      void* stream);

/* ------------------------------------------------------------------------------------------
 * Offload gather: replaces the CPU index_select + .cuda(non_blocking=True) of
 * modeling/spec_cache.py:293-303 (real_offload).  The prompt KV of the sparse layers of one
 * group lives in PINNED, device-mapped host memory, token-major:
 *     host_kv[token][layer_in_group][K|V][KVH][d]
 * so that one selected token is one contiguous chunk.  The kernel reads the selected chunks
 * straight over the host link with 16-byte loads and writes, per layer, the compact rows
 *     staged[layer_in_group][K|V][KVH][n_idx_capacity][d]
 * that omnikv_decode_attn then reads as segment A with idxA = NULL.
 * host_kv must be a device-visible address of the pinned buffer (cudaHostGetDevicePointer).
 * ------------------------------------------------------------------------------------------ */
int omnikv_offload_gather(const void* host_kv, int64_t token_stride_bytes, int n_layers_in_group,
                          int KVH, int head_dim, int elem_bytes, const int32_t* idx,
                          const int32_t* n_idx /* device [1] */, int n_idx_capacity, void* staged,
                          int n_ctas, void* stream);

/* ------------------------------------------------------------------------------------------
 * Append the current token's K/V rows: replaces the torch.cat re-copy of the whole cache,
 * modeling/spec_cache.py:363-369 (dense) and :343-347 (tail of sparse layers).
 * k_new, v_new [B, KVH, d] are written at row pos[b] of k_cache, v_cache [B, KVH, *, d].
 * ------------------------------------------------------------------------------------------ */
int omnikv_kv_append(int dtype, const void* k_new, const void* v_new, void* k_cache, void* v_cache,
                     int B, int KVH, int head_dim, int64_t new_stride_b, int64_t new_stride_h,
                     int64_t cache_stride_b, int64_t cache_stride_h, int64_t cache_stride_row,
                     const int32_t* pos, void* stream);

/* ------------------------------------------------------------------------------------------
 * Causal prefill attention: the attention of the prompt pass that fills the cache before the first decode step
 * (the reference reaches flash-attn there through transformers' decoder layer, modeling/omnikv.py:219-227, after
 * cache.update has returned the fresh keys, modeling/spec_cache.py:318-336).
 *
 *   out[b, i, h, :] = softmax over keys j <= q_pos0 + i of (q[b,h,i,:] . k[b,h/G,j,:] * scale) . v[b,h/G,j,:]
 *
 * q [B, H, Sq, d], k and v [B, KVH, Skv, d] (Skv >= q_pos0 + Sq; a chunk of queries against a longer cache passes its
 * first position as q_pos0), out [B, Sq, H, d]; all 16-bit of one dtype, element strides given (multiples of 8,
 * rows of d contiguous elements, bases 16-byte aligned), so k and v may be views of a cache or of a fused
 * projection.  tcgen05 kernels: 128 or 2 x 128 queries of a head per CTA, tiles by TMA, accumulators in tensor memory.
 * status (optional device word) is set to 6 if a bounded wait ran out.
 * ------------------------------------------------------------------------------------------ */
typedef struct {
  int32_t dtype; /* OMNIKV_BF16 or OMNIKV_F16 */
  int32_t B, H, KVH, head_dim;
  int32_t Sq, Skv, q_pos0;
  float scale;
  const void* q;
  int64_t q_stride_b, q_stride_h, q_stride_row;
  const void* k;
  int64_t k_stride_b, k_stride_h, k_stride_row;
  const void* v;
  int64_t v_stride_b, v_stride_h, v_stride_row;
  void* out;
  int64_t o_stride_b, o_stride_row, o_stride_h;
  int32_t* status;
  int32_t variant; /* 0: two query tiles per CTA, P and O in tensor memory (default); 1: one query tile per CTA, P
                      through shared memory and O in registers (the first version, kept for fault isolation) */
} omnikv_prefill_params;

int omnikv_prefill_attn(const omnikv_prefill_params* p, void* stream);

/* ------------------------------------------------------------------------------------------
 * A projection of a batched decode step (1..16 tokens) as a stream of its weight matrix on tcgen05:
 *
 *   y[b, n] = sum_k w[n, k] * x'[b, k]      x' = x, or RMSNorm(x, eps) * norm_w when norm_w is given
 *
 *   OMNIKV_EPI_STORE      out[b, n] = y                       (fused QKV projection; out is 16-bit)
 *   OMNIKV_EPI_STORE_F32  out[b, n] = y in fp32               (lm_head logits)
 *   OMNIKV_EPI_RESIDUAL   out[b, n] = residual[b, n] + y      (output and down projection; out may alias residual)
 *   OMNIKV_EPI_SWIGLU     w = [gate rows | up rows] (w_rows = 2 * inter, inter % 64 == 0),
 *                         out[b, j] = silu(y[b, j]) * y[b, inter + j]     for j < inter
 *
 * the third-party decoder modules the reference calls around its selection path (modeling/omnikv.py:156, :219-236,
 * :361-373) when several sequences decode together.  w [w_rows, K] row-major 16-bit (K % 8 == 0, 16-byte aligned),
 * x [n_tokens, K].  The workspace (omnikv_batched_linear_workspace_bytes) starts with 16 KiB of counters that must be
 * ZERO before the first call that uses it; every call leaves them zero; calls that share it must be stream-ordered.
 * Sums over K are taken in a fixed order (results do not depend on scheduling).  status (optional) is set to 7 if a
 * bounded wait ran out.
 * ------------------------------------------------------------------------------------------ */
typedef enum {
  OMNIKV_EPI_STORE = 0,
  OMNIKV_EPI_STORE_F32 = 1,
  OMNIKV_EPI_RESIDUAL = 2,
  OMNIKV_EPI_SWIGLU = 3
} omnikv_epilogue;

typedef struct {
  int32_t dtype; /* OMNIKV_BF16 or OMNIKV_F16: w, x, norm_w, residual, out (except STORE_F32) */
  int32_t n_tokens, w_rows, K;
  const void* w;
  int64_t w_stride_row;
  const void* x;
  int64_t x_stride_tok;
  const void* norm_w; /* [K] or NULL */
  float eps;
  int32_t epilogue; /* omnikv_epilogue */
  const void* residual;
  int64_t residual_stride_tok;
  void* out;
  int64_t out_stride_tok;
  void* workspace;
  size_t workspace_bytes;
  int32_t* status;
} omnikv_batched_linear_params;

size_t omnikv_batched_linear_workspace_bytes(int n_tokens, int w_rows, int K, int epilogue);
int omnikv_batched_linear(const omnikv_batched_linear_params* p, void* stream);

/* The current token of every sequence straight from a fused QKV projection (batched decode):
 * qkv[b] = [H query heads | KVH key heads | KVH value heads] x head_dim.  q and k are rotated (pairs (i, i+64) of
 * a head by rope_pos[b] * inv_freq[i], the rotate_half convention of the reference's decoder; fp32 arithmetic,
 * rounded once), q is written to q_out[b] = [H, head_dim], k and v to row cache_pos[b] of the caches
 * (cache_pos[b] < 0: sequence skipped).  Replaces apply_rotary + the contiguous copies + omnikv_kv_append of the
 * PyTorch path: one launch instead of thirteen. */
int omnikv_rope_append(int dtype, const void* qkv, int64_t qkv_stride_b, int B, int H, int KVH, int head_dim,
                       const float* inv_freq, const int32_t* rope_pos, void* q_out, int64_t q_stride_b,
                       void* k_cache, void* v_cache, int64_t cache_stride_b, int64_t cache_stride_h,
                       int64_t cache_stride_row, const int32_t* cache_pos, void* stream);
/* The observation window's queries of a window selector straight from the q projection: qlin[b][w] = H heads x
 * head_dim (element strides given), every query rotated at rope_pos[b] (the reference rotates all window queries at
 * the current position, modeling/omnikv.py:52-57, :66-71), written as out [B, H, W, head_dim] contiguous: the qw
 * argument of omnikv_score_window.  One launch instead of the transpose and the element-wise rotary kernels. */
int omnikv_rope_window(int dtype, const void* qlin, int64_t stride_b, int64_t stride_w, int B, int W, int H,
                       int head_dim, const float* inv_freq, const int32_t* rope_pos, void* out, void* stream);
/* The residual add and the RMSNorm behind it as one launch (batched decode): h[b] += delta[b] when delta is given
 * (rounded to the residual stream's type), out[b] = RMSNorm(h[b], eps) * norm_w.  Replaces the separate add and norm
 * kernels between the third-party decoder modules (modeling/omnikv.py:229-232 and the next layer's :156). */
int omnikv_add_rms_norm(int dtype, void* h, int64_t h_stride_tok, const void* delta, int64_t delta_stride_tok,
                        const void* norm_w, float eps, void* out, int64_t out_stride_tok, int n_tokens, int hidden,
                        void* stream);
/* act[b][j] = silu(gate_up[b][j]) * gate_up[b][inter + j] for j < inter (SwiGLU of a fused gate/up projection). */
int omnikv_silu_mul(int dtype, const void* gate_up, int64_t gate_up_stride_b, void* act, int64_t act_stride_b,
                    int B, int inter, void* stream);

/* ------------------------------------------------------------------------------------------
 * Batch-1 decode step: weight-streaming kernels with the element-wise work of the decoder layer
 * fused in.  In the reference these are third-party transformers modules called around the hot
 * path (LlamaRMSNorm, q/k/v/o_proj, apply_rotary_pos_emb, LlamaMLP, lm_head: the calls at
 * modeling/omnikv.py:156, :219-236, :361-373) plus the cache append of modeling/spec_cache.py:363-369;
 * at batch 1 they read 75 % of the step's bytes, so they decide the tokens/s the path delivers.
 * 16-bit dtypes only; hidden sizes K in {512, 1024, 1792, 2048, 3584, 4096, 7168, 8192, 14336}.
 * status: device int32, stays 0; a kernel whose bounded wait on a copy ran out writes a code there.
 *
 * omnikv_decode_qkv: x = RMSNorm(h) * norm_w; [q|k|v] = w_qkv x (rows: H q heads, KVH k heads, KVH v
 *   heads, 128 rows each); RoPE at position *rope_pos with inv_freq[64] (rotate_half convention);
 *   q -> q_out [H*128]; k, v -> row *cache_pos of k_cache_seq / v_cache_seq (one sequence's
 *   [KVH, rows, 128] cache with the given element strides).
 * omnikv_decode_gemv_residual: out[N] = (resid ? resid : 0) + w[N,K] x.  out may alias resid.
 * omnikv_decode_gate_up: x = RMSNorm(h) * norm_w; act[i] = silu(w[i] . x) * (w[inter + i] . x).
 * omnikv_decode_logits: x = RMSNorm(h) * norm_w; logits[r] = w_head[r] . x (fp32); token_out (optional)
 *   = row_offset + argmax (lowest index among equal maxima); best_scratch: 8 bytes of device scratch.
 * ------------------------------------------------------------------------------------------ */
/* Tensor parallelism: the SUM all-reduce that follows a row-parallel projection (output projection, MLP down
 * projection; the all_reduce calls of lightllm/common/basemodel/layer_infer/template/
 * transformer_layer_infer_template.py:119-120, :128-129 in the reference's fork) is fused into the kernels on
 * both sides of it, over peer-mapped memory:
 *   producer  omnikv_decode_gemv_residual(tp_out = x): every rank stores its fp32 partial sums straight into
 *             EVERY rank's exchange buffer (plain peer stores over NVLink) as 8-byte entries {value, tag}, one
 *             store per entry, tag = *epoch * 256 + seq + 1: an entry is the old one or the new one, never a mix,
 *             so there is no flag, no fence and nothing after the last row.  `resid` and `out` are unused (may be
 *             NULL).
 *   consumer  omnikv_decode_gate_up / _qkv / _logits(tp_in = x): every thread reads its entries of all ranks until
 *             they carry this exchange's tag (bounded wait), then the activations are h + sum over ranks of the
 *             partials (rank order, the same on every rank), rounded once to the storage type; they are also
 *             written to h_inout (the updated residual stream), which must be a DIFFERENT buffer than h: other
 *             CTAs of the same launch are still reading h.  A consumer does not wait for the completion of the
 *             call before it on the stream (it is launched as a programmatic dependent launch): the only thing it
 *             may need from that call are the local partials, which arrive through the entries.  So the call right
 *             before a consumer must be the producer of its exchange (or any call whose outputs the consumer does
 *             not read), and what else the consumer reads (h, the norm weights) must come from calls at least two
 *             back.
 * peer_base[r]: rank r's exchange buffer (omnikv_tp_exchange_bytes(hidden) bytes, zero before first use) as
 * mapped into THIS process (peer_base[rank] = the local one).  Exchanges alternate between two slots
 * (seq & 1); seq numbers the exchanges of a decode step 0, 1, 2, ... (< 256) and must follow program order, and a
 * step must hold an EVEN number of them (a decoder layer has two), so that the last exchange of a step and the
 * first of the next never share a slot; *epoch is a local device word that every rank bumps once per decode
 * step (it must never repeat: tags identify an exchange for good).  All ranks must issue the same sequence of
 * calls.  world <= 8.  NULL or world <= 1: no exchange.  A consumer takes a residual stream of at most 8192
 * values (OMNIKV_E_UNSUPPORTED above that).  The wait for the peers' entries gives up after two seconds
 * (status 4). */
typedef struct {
  int32_t world, rank;
  void* peer_base[8];
  uint32_t* done_counter; /* TWO local device words, zero before first use: [0] CTAs that have finished (producers),
                             [1] calls made so far on this object (omnikv_tp_allreduce_sum) */
  const uint32_t* epoch;
  int32_t seq;
  int32_t hidden;
} omnikv_tp_exchange;

size_t omnikv_tp_exchange_bytes(int hidden);

/* SUM all-reduce of x[0..n) (bf16 / fp16 / fp32, in place) across the ranks of an exchange, for tensors too small
 * for a ring to pay off (the hidden state of a batched decode step): every rank stores its vector into its slot of
 * EVERY rank's exchange buffer over NVLink and raises a flag; every rank then adds the slots in rank order in
 * fp32 (bit-identical results on all ranks).  Replaces the dist.all_reduce after the output projection and the
 * MLP of the reference's tensor-parallel fork (lightllm/common/basemodel/layer_infer/template/
 * transformer_layer_infer_template.py:119-120, :128-129).  The exchange describes a buffer of
 * omnikv_tp_exchange_bytes(hidden) bytes per rank; n * element size must not exceed hidden * 4 bytes and must be
 * a multiple of 16.  The two slots alternate by a device-side count of the calls made on THIS exchange object
 * (done_counter[1]; seq and epoch are not used), so any number of calls per step -- odd ones too, and replays of a
 * captured step -- is safe as long as every rank issues the same sequence of calls on one stream.  The wait for
 * the peers' flags gives up after two seconds (status 4). */
int omnikv_tp_allreduce_sum(int dtype, void* x, int64_t n, const omnikv_tp_exchange* t, int32_t* status,
                            void* stream);
/* The same exchange as element-wise MAX of fp32 vectors (the filter layers' score planes before the top-k: a step
 * the reference's fork does not have, it selects per rank, lightllm/models/llama_omnikv/triton_kernel/
 * flash_decoding.py:76) and as an all-gather: out[r * n + i] = rank r's x[i] (the vocabulary-sharded logits,
 * lightllm/models/llama_omnikv/layer_infer/post_layer_infer.py:140-148).  Same buffer, size and call-order rules. */
int omnikv_tp_allreduce_max(void* x, int64_t n, const omnikv_tp_exchange* t, int32_t* status, void* stream);
int omnikv_tp_allgather(int dtype, const void* x, int64_t n, void* out, const omnikv_tp_exchange* t, int32_t* status,
                        void* stream);
int omnikv_decode_qkv(int dtype, const void* h, const void* norm_w, float eps, const void* w_qkv, int hidden,
                      int H, int KVH, int head_dim, const float* inv_freq, const int32_t* rope_pos,
                      void* q_out, void* k_cache_seq, void* v_cache_seq, int64_t kv_stride_h,
                      int64_t kv_stride_row, const int32_t* cache_pos, const omnikv_tp_exchange* tp_in,
                      void* h_inout, int32_t* status, void* stream);
int omnikv_decode_gemv_residual(int dtype, const void* w, int N, int K, const void* x, const void* resid,
                                void* out, const omnikv_tp_exchange* tp_out, int32_t* status, void* stream);
int omnikv_decode_gate_up(int dtype, const void* h, const void* norm_w, float eps, const void* w_gate_up,
                          int hidden, int inter, void* act_out, const omnikv_tp_exchange* tp_in, void* h_inout,
                          int32_t* sched, int32_t* status, void* stream);
/* sched (optional): four device int32, zero before the first use (the kernel leaves them zero).  With it the last
 * chunks of the gate/up matrix are handed to whichever SM is ready instead of by a fixed round-robin, which evens
 * out the end of the kernel (SMs do not all stream at the same rate).  Calls sharing one sched buffer must be
 * issued on one stream.  NULL: fixed assignment. */
int omnikv_decode_logits(int dtype, const void* h, const void* norm_w, float eps, const void* w_head,
                         int hidden, int vocab_rows, int row_offset, float* logits,
                         unsigned long long* best_scratch, int64_t* token_out, const omnikv_tp_exchange* tp_in,
                         int32_t* status, void* stream);

/* ------------------------------------------------------------------------------------------
 * omnikv_decode_chain: the weight-streaming phases between two attention calls of a batch-1 decode
 * step in ONE cooperative launch (one CTA per SM, grid-wide barriers between phases):
 *   [h += w_o attn_out] -> [act = silu(gate) * up of RMSNorm(h)] -> [h += w_down act]
 *   -> [next layer's omnikv_decode_qkv on h]  or  [omnikv_decode_logits on h]
 * Same arithmetic as the four single calls above; what it adds is that the weight stream never
 * stops: while the CTAs wait at a barrier or load the next phase's activations, the producer
 * thread keeps copying the next phase's rows into the shared-memory ring.  A phase whose weight
 * pointer is NULL is skipped (w_o; w_gate_up together with w_down; w_qkv; w_head; w_qkv and w_head
 * exclude each other).  Single GPU only: there is no collective between the phases.
 * grid_sync: one device uint32, zero before the first use; the kernel leaves it ready for reuse.
 * chunk_counters: four device int32 that are ZERO when the launch starts (the kernel does not reset them):
 * CTAs then take weight chunks from shared counters as they become ready, which evens out SMs that get
 * less memory bandwidth; NULL: static round-robin assignment.
 * omnikv_decode_chain_supported: 1 when a kernel is built for (dtype, hidden, inter, H), else 0.
 * ------------------------------------------------------------------------------------------ */
typedef struct {
  int32_t dtype, hidden, inter, H, KVH;
  float eps;
  void* h;                 /* [hidden] residual stream, updated in place */
  const void* w_o;         /* [hidden, hidden] or NULL */
  const void* attn_out;    /* [hidden] */
  const void* post_norm_w; /* [hidden] */
  const void* w_gate_up;   /* [2*inter, hidden] or NULL */
  const void* w_down;      /* [hidden, inter] */
  void* act_scratch;       /* [inter] */
  const void* in_norm_w;   /* next layer's input norm [hidden] */
  const void* w_qkv;       /* next layer's [(H+2KVH)*128, hidden] or NULL */
  const float* inv_freq;
  const int32_t* rope_pos;
  void* q_out;
  void* k_cache_seq;
  void* v_cache_seq;
  int64_t kv_stride_h, kv_stride_row;
  const int32_t* cache_pos;
  const void* final_norm_w;
  const void* w_head;      /* [vocab_rows, hidden] or NULL */
  int32_t vocab_rows;
  float* logits;
  unsigned long long* best_scratch;
  int64_t* token_out;      /* may be NULL */
  uint32_t* grid_sync;
  int32_t* chunk_counters; /* may be NULL */
  int32_t* status;
  const void* next_w;      /* optional: the weights the NEXT launch will read first (next layer's w_o); the kernel asks
                              for next_w_bytes of them to be brought into L2 when its own copies are issued */
  size_t next_w_bytes;
} omnikv_chain_params;

int omnikv_decode_chain(const omnikv_chain_params* p, void* stream);
int omnikv_decode_chain_supported(int dtype, int hidden, int inter, int H);

#ifdef __cplusplus
}
#endif
#endif /* OMNIKV_B200_H_ */
