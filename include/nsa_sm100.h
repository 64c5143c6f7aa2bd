/* C ABI of libnsa_sm100.so: hand-written sm_100a kernels for the Native-Sparse-Attention hot path.
 *
 * The reference project has no FFI of its own (its kernels are Triton functions launched from Python), so
 * each entry point below names the reference Python function whose kernel launch it replaces.  The Python
 * package `flash_nsa` in this repository binds these symbols with ctypes and keeps the reference's Python
 * signatures on top of them.
 *
 * Conventions
 *  - every pointer is a DEVICE pointer unless said otherwise; tensors are bf16 (uint16 bit patterns) with a
 *    contiguous innermost dimension, strides are in ELEMENTS;
 *  - `stream` is a cudaStream_t passed as void*; calls only enqueue work, they never synchronise, never
 *    allocate device memory and never free it: every scratch buffer is a caller-provided field;
 *  - return value 0 = ok, negative = NsaStatus; nsa_last_error() gives the message for the calling thread;
 *  - sequences are described by NsaSeqMeta.  A "piece" is a run of local query rows belonging to one
 *    sequence: without context parallelism pieces are the sequences themselves; with it they are the parts
 *    of sequences that fall into this rank's chunks, and piece_off is the position of the first local row
 *    inside its sequence (flash_nsa/utils.py:284-323 builds the same table as cp_cu_seqlens / cp_batch_idx /
 *    cp_offset).  K/V-side tensors always hold whole sequences (x_cu), compressed tensors whole sequences of
 *    compressed rows (y_cu).
 */
#ifndef NSA_SM100_H_
#define NSA_SM100_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum NsaStatus {
  NSA_OK = 0,
  NSA_ERR_BAD_ARG = -1,
  NSA_ERR_UNSUPPORTED_SHAPE = -2,
  NSA_ERR_CUDA = -3,
  NSA_ERR_TIMEOUT = -4
} NsaStatus;

typedef struct NsaSeqMeta {
  const int32_t* piece_cu;  /* [n_pieces+1] local row offsets of the pieces                                */
  const int32_t* piece_seq; /* [n_pieces] sequence id of each piece; NULL = identity                         */
  const int32_t* piece_off; /* [n_pieces] position of the piece's first row in its sequence; NULL = zeros    */
  const int32_t* x_cu;      /* [n_seq+1] token offsets of the sequences in K/V-side tensors                  */
  const int32_t* y_cu;      /* [n_seq+1] offsets of the sequences' compressed rows; may be NULL if unused     */
  /* Paged K/V (inference): when kv_table is set, token row r of sequence s lives at flat cache row
   * kv_table[s*kv_table_stride + r/page_size]*page_size + r%page_size instead of x_cu[s]+r (x_cu then only gives the
   * lengths); cmp_table does the same for compressed rows (y_cu gives their counts).  flash_nsa/inference/*.py
   * address the cache the same way (e.g. inference/compress_attn.py:93-97).                                     */
  const int32_t* kv_table;
  const int32_t* cmp_table;
  int32_t n_pieces;
  int32_t n_seq;
  int32_t max_piece_len; /* longest piece (grid sizing)                                                    */
  int32_t x_maxlen;      /* longest sequence                                                               */
  int32_t y_maxlen;      /* most compressed rows in one sequence                                           */
  int32_t page_size;     /* rows per cache page (paged mode)                                               */
  int32_t kv_table_stride;
  int32_t cmp_table_stride;
} NsaSeqMeta;

typedef struct NsaHyper {
  int32_t kernel_size; /* tokens per compressed row (32)            */
  int32_t stride;      /* distance between compressed rows (16)     */
  int32_t block_size;  /* tokens per selection block (64)           */
  int32_t window;      /* sliding window: keys t-window .. t        */
  int32_t top_n;       /* selected blocks per (token, kv head)      */
  int32_t num_init;    /* forced first blocks                       */
  int32_t num_local;   /* forced blocks ending at the query's block */
  int32_t reserved0;
} NsaHyper;

/* ---- KV compression ------------------------------------------------------------------------------- */
typedef struct NsaPoolParams {
  NsaSeqMeta meta;
  NsaHyper hp;
  const void* x; /* [T,H,D] bf16                                                   */
  void* y;       /* fwd: [Ytot,H,D] bf16 out.  bwd: dy, same shape, bf16 in         */
  float* dx;     /* bwd only: [T,H,D] fp32                                          */
  int64_t x_stride_t, y_stride_t, dx_stride_t; /* token strides (head stride = D)   */
  int32_t H, D;
  int32_t accumulate; /* bwd: 1 = add into dx, 0 = overwrite                        */
  int32_t reserved0;
} NsaPoolParams;
/* replaces mean_pooling_fwd, flash_nsa/ops/compress_kv.py:335-366 */
int nsa_mean_pool_fwd(const NsaPoolParams* p, void* stream);
/* replaces mean_pooling_bwd, flash_nsa/ops/compress_kv.py:368-399 (dx is fp32, as in the fused backward) */
int nsa_mean_pool_bwd(const NsaPoolParams* p, void* stream);

typedef struct NsaBlockParams {
  NsaSeqMeta meta;
  NsaHyper hp;
  const void* x; /* fwd: [T,H,D] bf16 in                                            */
  void* y;       /* fwd: [Ytot,H,kernel_size,D] bf16 out.  bwd: dy (bf16 in)        */
  float* dx;     /* bwd: [T,H,D] fp32                                               */
  int64_t x_stride_t, dx_stride_t;
  int32_t H, D;
  int32_t accumulate;
  int32_t reserved0;
} NsaBlockParams;
/* replaces construct_block_fwd / construct_block_bwd, flash_nsa/ops/compress_kv.py:127-190 */
int nsa_construct_block_fwd(const NsaBlockParams* p, void* stream);
int nsa_construct_block_bwd(const NsaBlockParams* p, void* stream);

typedef struct NsaActParams {
  const void* x;  /* [M,2K] bf16: gate | up                                          */
  void* y;        /* fwd: [M,K] bf16 out                                             */
  const void* dy; /* bwd: [M,K] bf16                                                 */
  void* dx;       /* bwd: [M,2K] bf16 out (may alias x)                              */
  int64_t M;
  int32_t K;
  int32_t kind; /* 0 = swiglu (silu(gate)*up), 1 = sigmoid-mul (sigmoid(gate)*up)    */
} NsaActParams;
/* replaces swiglu_fwd/bwd and sigmoid_mul_fwd/bwd, flash_nsa/ops/act.py:60-94, 174-208 */
int nsa_act_fwd(const NsaActParams* p, void* stream);
int nsa_act_bwd(const NsaActParams* p, void* stream);

/* ---- attention branches ----------------------------------------------------------------------------- */
typedef struct NsaAttnParams {
  NsaSeqMeta meta;
  NsaHyper hp;
  const void* q;     /* [Tq,QH,D] bf16 (local rows)                                                      */
  const void* k;     /* compressed branch: [Ytot,KH,D]; otherwise [Tk,KH,D]                               */
  const void* v;     /* same rows as k, [.,KH,D]                                                          */
  void* o;           /* [Tq,QH,D] bf16; fwd out, bwd in                                                   */
  float* lse;        /* base-2 log-sum-exp of the scaled scores; element (t,h) at t*lse_stride_t+h*lse_stride_h */
  const void* dout;  /* bwd: [Tq,QH,D] bf16                                                               */
  float* delta;      /* bwd scratch, same addressing as lse: rowsum(o*dout), written by the call          */
  void* dq;          /* bwd: [Tq,QH,D] bf16                                                               */
  float* dk;         /* bwd: fp32, same rows as k; results are ADDED (atomics): zero-fill for a fresh result */
  float* dv;         /* bwd: fp32, same rows as v; idem                                                   */
  const int32_t* topk; /* selected branch: [KH,Tq,top_n] int32                                            */
  const int32_t* k2q_offsets; /* selected bwd: CSR offsets from nsa_k2q_index (not read by the kernels: the items carry
                                 their entry ranges; callers that inspect the index use them)                  */
  const int32_t* k2q_tokens;  /* selected bwd: [KH, Tq*top_n] local query rows, cell after cell               */
  const int32_t* k2q_blk_cu;  /* selected bwd: [n_pieces+1] first table row of each piece (as in NsaK2qParams) */
  const int32_t* k2q_items;   /* selected bwd: [KH, k2q_items_cap, 4] work items from nsa_k2q_index (item_rows > 0) */
  int32_t* k2q_n_items;       /* selected bwd: [KH + 2]: items per kv head, then two ticket counters of the backward
                                 kernel (zero between launches: nsa_k2q_index clears them, the kernel restores them),
                                 so two backward launches on one index must not overlap on the GPU              */
  int32_t* status;   /* optional device word: kernels OR a bit into it when a bounded wait on the tensor-core
                        pipeline gives up (NSA_ERR_TIMEOUT condition); never written on success; may be NULL     */
  int64_t q_stride_t, k_stride_t, v_stride_t, o_stride_t, do_stride_t, dq_stride_t, dk_stride_t, dv_stride_t;
  int64_t lse_stride_t, lse_stride_h;
  int64_t topk_stride_h; /* elements between kv heads in topk (= Tq*top_n when contiguous)                */
  int64_t k2q_stride_h;  /* elements between kv heads in k2q_tokens                                       */
  float sm_scale;
  int32_t QH, KH, D;
  int32_t accumulate_dq;   /* bwd: 1 = dq += result, 0 = dq = result                                      */
  int32_t n_q_rows;        /* bwd: total number of local query rows (= piece_cu[n_pieces])                */
  int32_t n_k_rows;        /* bwd: rows of the k / v tensors (bounds of the bulk tensor loads)            */
  int32_t k2q_items_cap;   /* selected bwd: items per kv head that k2q_items can hold (its kv-head stride)   */
  int32_t n_blocks_total;  /* selected bwd: rows of the k2q table per kv head                             */
  int32_t phases;          /* bwd: 0 = run every kernel of the call; otherwise a mask, bit 0 = delta, bit 1 = dK/dV,
                              bit 2 = dQ (lets a profiler time the kernels of one call separately)         */
} NsaAttnParams;

/* compressed attention: replaces cmp_attn_fwd / cmp_attn_bwd, flash_nsa/ops/compress_attn.py:532-741.
 * lse layout of the reference is [QH,T]: pass lse_stride_h = T, lse_stride_t = 1.                        */
int nsa_cmp_attn_fwd(const NsaAttnParams* p, void* stream);
int nsa_cmp_attn_bwd(const NsaAttnParams* p, void* stream);
/* sliding-window attention: replaces swa_fwd / swa_bwd, flash_nsa/ops/sliding_window_attention.py:42-157,
 * i.e. the flash-attn call with window_size=(window,-1), causal=True.                                     */
int nsa_swa_fwd(const NsaAttnParams* p, void* stream);
int nsa_swa_bwd(const NsaAttnParams* p, void* stream);
/* selected-block attention: replaces slc_attn_fwd / slc_attn_bwd, flash_nsa/ops/select_attn.py:440-701.
 * Backward: needs the key-block -> queries index WITH work items (nsa_k2q_index, item_rows > 0; range buckets are
 * optional and only change the order of the work).  dK/dV come from one persistent block-major kernel (one CTA per SM
 * walking the items in order); when dK/dV and dQ are both asked for (phases 0, 6 or 7) the same kernel also adds its
 * dQ tiles into dq with bf16 reductions (the reference's fuse_dqdkdv=True form, select_attn.py:148-335); with
 * accumulate_dq = 0 dq is cleared first.  The last bits of dq then depend on the order of the adds; the environment
 * variable NSA_SLC_BWD_UNFUSED=1 selects the token-major dQ kernel instead (fp32 accumulation, fixed order).        */
int nsa_slc_attn_fwd(const NsaAttnParams* p, void* stream);
int nsa_slc_attn_bwd(const NsaAttnParams* p, void* stream);

/* ---- block importance + top-n ----------------------------------------------------------------------- */
typedef struct NsaTopkParams {
  NsaSeqMeta meta;
  NsaHyper hp;
  const void* q;    /* [Tq,QH,D] bf16                                                                     */
  const void* ck;   /* [Ytot,KH,D] bf16 compressed keys                                                   */
  const float* lse; /* log-sum-exp of the compressed branch (addressing as in NsaAttnParams)              */
  int32_t* topk;    /* out [KH,Tq,top_n]; unused slots keep ignore_index                                  */
  void* probs;      /* optional out [KH,Tq,probs_stride_t] block scores (fp16 or fp32 per quant), or NULL  */
  int32_t* status;  /* optional device word for pipeline time-outs, as in NsaAttnParams                   */
  int64_t q_stride_t, ck_stride_t, lse_stride_t, lse_stride_h, probs_stride_t;
  float sm_scale;
  int32_t QH, KH, D;
  int32_t ignore_index;
  int32_t quant; /* what the selection compares: 0 = fp32 score, 1 = score rounded to fp16,
                    2 = score^3 rounded to fp16 (the reference default below 128K tokens),
                    3 = fp32 score pooled from per-row probabilities rounded to fp16 (the reference's general path) */
  int32_t q_rows;  /* rows of the q tensor and of the ck tensor: bounds of the bulk tensor loads           */
  int32_t ck_rows;
} NsaTopkParams;
/* replaces slc_topk_indices_for_32_16_64 (kernel pair _slc_probs_kernel + _topk_kernel, flash_nsa/ops/topk.py:499-628)
 * and the general pair _attn_probs_kernel + _slc_probs_topk_kernel (topk.py:19-218); scores and selection are fused, no
 * [KH,T,blocks] or [KH,T,rows] scratch is needed.
 * kernel 32 / stride 16 / block 64, quant 0-2: contiguous (non-paged) inputs with top_n - num_init - num_local == 13 run
 * on the TMA + tcgen05 kernel (up to 64 query heads per kv head); paged caches and other list sizes (top_n <= 32) run on
 * the warp-MMA kernel (<= 16 heads per kv head).  Any other kernel_size / stride / block_size, quant 3, or top_n > 32 run on
 * the general warp-MMA kernel (<= 16 heads per kv head; meta.x_maxlen must bound the sequence length: it sizes the
 * per-token score array in shared memory, at most about 5000 blocks).                                               */
int nsa_slc_topk(const NsaTopkParams* p, void* stream);

typedef struct NsaK2qParams {
  NsaSeqMeta meta;
  NsaHyper hp;
  const int32_t* topk; /* [KH,Tq,top_n]                                                                   */
  int32_t* offsets;    /* out [KH, n_cells+1]; also used as the histogram while building                  */
  int32_t* tokens;     /* out [KH, Tq*top_n]                                                              */
  int32_t* cursor;     /* scratch [KH, n_cells] (any contents)                                            */
  const int32_t* blk_cu; /* [n_pieces+1] offsets of each piece's block rows (cdiv(len+off, block_size))    */
  int32_t* items;      /* optional out [KH, items_cap, 4]: work items (block row, first entry, end entry, range), 16-byte
                          aligned; written when item_rows > 0                                             */
  int32_t* n_items;    /* optional out [KH + 2]: items written per kv head; the two extra words are cleared (they are
                          the ticket counters of nsa_slc_attn_bwd)                                       */
  int64_t Tq;
  int32_t KH;
  int32_t n_blocks_total;
  int32_t range_rows;  /* 0: one list per (kv head, block row), n_cells = n_blocks_total.  > 0: lists are split by the
                          range q_row / range_rows of the query row; cell = range * n_blocks_total + block row,
                          n_cells = cdiv(Tq, range_rows) * n_blocks_total                                  */
  int32_t item_rows;   /* > 0: also cut every cell into items of at most item_rows entries, in cell order   */
  int32_t items_cap;   /* capacity of `items` per kv head; Tq*top_n/item_rows + min(n_cells, Tq*top_n) + 1 always suffices */
  int32_t reserved0;
} NsaK2qParams;
/* replaces get_bind_from_find, flash_nsa/ops/topk.py:889-945: for every (kv head, key block) the list of local
 * query rows that selected it, as CSR (counts -> exclusive scan -> fill) instead of a dense table.  Range buckets and
 * work items (no counterpart in the reference) order the backward's work so that concurrently running CTAs touch the
 * q / dO / dq rows of one range, which then stay in L2.                                                    */
int nsa_k2q_index(const NsaK2qParams* p, void* stream);
/* No counterpart in the reference.  Same result as nsa_k2q_index, but the fill cursors live in a 1 MiB array inside
 * the library image instead of `cursor` (which is ignored), so the call needs no scratch allocation at all.
 * For hosts that cannot allocate at the point of the call: an inference server that gave all free device memory to its
 * KV-cache pool at start-up, or code between a framework's caching allocator and a region where cudaMalloc is not
 * allowed.  Limit: KH * n_cells <= 262144 (without range buckets e.g. 4 kv heads and 4 M tokens), larger sizes are refused with
 * NSA_ERR_UNSUPPORTED_SHAPE.  The first call on each device looks up the array's device address: make that call outside
 * any stream capture and at start-up, before the host gives the device's free memory away (the array is materialised
 * when the library's code is first used on a device; n_blocks_total = 0 is enough for that call).  The address cache covers
 * device ordinals 0-63.  All calls on a device share the array: the cursors are cleared at the start of every call, and
 * two calls whose kernels overlap on the GPU (different streams) corrupt each other.                              */
int nsa_k2q_index_static(const NsaK2qParams* p, void* stream);

/* ---- gated combine ---------------------------------------------------------------------------------- */
typedef struct NsaCombineParams {
  const void *a, *b, *c; /* [T,H,D] bf16 branch outputs                                                    */
  const void* w;         /* [T,H,3] bf16 gate logits                                                       */
  void* y;               /* fwd out [T,H,D] bf16                                                           */
  const void* dy;        /* bwd in                                                                         */
  void *da, *db, *dc;    /* bwd out [T,H,D] bf16                                                           */
  void* dw;              /* bwd out [T,H,3] bf16                                                           */
  int64_t a_stride_t, b_stride_t, c_stride_t, w_stride_t, y_stride_t, dy_stride_t, dw_stride_t;
  int64_t T;
  int32_t H, D;
  /* optional bwd out (all three or none): delta_x[t,h] = sum_d x[t,h,d] * dx[t,h,d] in fp32, the row term the branch
   * backward kernels need; a branch backward given this runs with phases = 6 (no delta pass of its own) */
  float *delta_a, *delta_b, *delta_c;
  int64_t delta_a_stride_t, delta_a_stride_h, delta_b_stride_t, delta_b_stride_h, delta_c_stride_t, delta_c_stride_h;
} NsaCombineParams;
/* replaces combine_fwd / combine_bwd, flash_nsa/ops/combine.py:114-177 */
int nsa_combine_fwd(const NsaCombineParams* p, void* stream);
int nsa_combine_bwd(const NsaCombineParams* p, void* stream);

/* ---- paged-KV pooling (inference) ---------------------------------------------------------------------- */
typedef struct NsaPagedPoolParams {
  void* cache0;                /* [pages*page_size, H, D] bf16 cache; pooled rows are written IN PLACE at slot rows */
  void* cache1;                /* optional second cache (V) pooled by the same launch, or NULL                      */
  const int32_t* slot_mapping; /* prefill: one entry per compressed row of the batch; decode: one per sequence;
                                  flat cache row to write, -1 = nothing to write                                    */
  const int32_t* kv_table;     /* [B, table_stride] page ids of the token rows                                      */
  const int32_t* y_cu;         /* prefill: [B+1] offsets of the sequences' compressed rows                          */
  const int32_t* context_lens; /* decode: [B] tokens in the cache, the new one included                             */
  int64_t row_stride;          /* elements between cache rows (H*D)                                                 */
  int32_t B, H, D;
  int32_t page_size, table_stride;
  int32_t y_maxlen;            /* prefill: most compressed rows in one sequence (grid sizing)                       */
  int32_t kernel_size, stride;
  int32_t decode;              /* 0: prefill (every row with a slot), 1: decode (only the window ending at the last token);
                                  nsa_paged_zero_tails: 2 = context_lens are token counts, clear the compressed-row tails */
  int32_t reserved0;
} NsaPagedPoolParams;
/* replaces mean_pooling_prefill / mean_pooling_decode / kv_mean_pooling_decode,
 * flash_nsa/inference/compress_kv.py:191-286 */
int nsa_paged_mean_pool(const NsaPagedPoolParams* p, void* stream);
/* Clears the cache rows [len_b, next multiple of 128) of every sequence b (cache0 and, if given, cache1), where len_b =
 * context_lens[b] counts the rows of the kind kv_table lists (token rows with the token page table and the context
 * lengths; compressed rows with the compressed-row page table and the compressed-row counts).  The TMA-fed prefill kernels
 * read whole 128-row tiles of a page, and rows past a sequence's end may be never-written memory; the reference's kernels
 * mask per row instead (flash_nsa/inference/compress_attn.py:60-120).  Uses cache0, cache1, kv_table, context_lens,
 * row_stride, B, page_size, table_stride; with decode = 2, context_lens holds TOKEN counts and len_b is the number of
 * compressed rows they give, (tokens - kernel_size) / stride + 1. */
int nsa_paged_zero_tails(const NsaPagedPoolParams* p, void* stream);
/* Copies the rows that kv_table lists for every sequence b, rows 0 .. y_cu[b+1] - y_cu[b] - 1, from the paged cache0 into
 * the contiguous buffer cache1 at rows y_cu[b] + j (same row layout).  The prefill scoring uses it on the compressed K rows
 * so that the tcgen05 scoring kernel, whose 128-row tiles start every 124 rows and cannot follow a page table, serves
 * a paged cache too (the reference's paged scoring kernel reads the pages directly, flash_nsa/inference/topk.py:19-190).
 * Uses cache0, cache1, kv_table, y_cu, y_maxlen, row_stride, B, page_size, table_stride. */
int nsa_paged_gather_rows(const NsaPagedPoolParams* p, void* stream);

/* ---- fused paged decode step ---------------------------------------------------------------------------- */
typedef struct NsaDecodeParams {
  const void* q;               /* [B,QH,D] bf16: one new token per sequence                                          */
  void* k_cache;               /* [pages*page_size, KH, D] bf16; also receives the new compressed row (in place)     */
  void* v_cache;               /* same layout                                                                        */
  const void* w;               /* [B,QH,3] bf16 gate logits                                                          */
  void* o;                     /* [B,QH,D] bf16 out                                                                  */
  const int32_t* context_lens; /* [B] tokens in the cache including the new one; 0 = padding row (output zeros)      */
  const int32_t* kv_table;     /* [B, kv_table_stride] pages of the tokens                                           */
  const int32_t* cmp_table;    /* [B, cmp_table_stride] pages of the compressed rows                                 */
  const int32_t* slot_mapping; /* [B] flat cache row for the compressed row completed by this token, -1 = none       */
  int32_t* topk_out;           /* optional [KH,B,top_n] selected blocks (-1 = unused slot), or NULL                  */
  int32_t* status;             /* optional error word (bit 32: a sequence has more compressed rows than y_cap)       */
  NsaHyper hp;
  int64_t q_stride_t, o_stride_t, w_stride_t, cache_stride_t;
  float sm_scale;
  int32_t B, QH, KH, D;
  int32_t page_size, kv_table_stride, cmp_table_stride;
  int32_t y_cap;               /* most compressed rows a sequence may have (sizes the shared-memory score array)      */
  int32_t cache_rows;          /* rows of the flat caches (pages * page_size): bounds of the bulk tensor loads; 0 = unknown
                                  (the kernel then fetches its tiles with per-warp copies)                           */
} NsaDecodeParams;
/* replaces the whole body of nsa_decode, flash_nsa/inference/__init__.py:160-257 (8 launches there): pooling of the new
 * compressed row, compressed attention, block scores + top-n, selected and sliding-window attention, gated combine,
 * one CTA (or one cluster, see below) per (sequence, kv head): a producer warp streams the K/V tiles of the step through a shared-memory ring with
 * bulk tensor loads, six consumer warps work on them.  Needs kernel 32 / stride 16 / block 64 and at most 16 query heads
 * per kv head.                                                                                                      */
int nsa_decode_fused(const NsaDecodeParams* p, void* stream);
/* How many CTAs nsa_decode_fused would give each (sequence, kv head) of this step: 1, or 2 / 4 / 8 (a thread-block cluster
 * that splits the tiles of the step and exchanges scores and partial outputs through distributed shared memory) when the
 * step has few sequences (B * KH * size within the SM count) and kv_table_stride * page_size, the bound on the context
 * lengths the host knows, is at least 4K tokens (sizes 4 and 8) or 16K tokens (size 2); the launch falls back to the next
 * smaller size when the GPU cannot hold all clusters at once.  The reference splits long contexts over CTAs with its num_splits arguments
 * (flash_nsa/inference/__init__.py:160-257); here the library decides.  Reads the sizes (B, KH, D, page_size,
 * kv_table_stride, y_cap, hp), no pointer; asks the device how many clusters it holds, so it needs a current device.  */
int nsa_decode_cluster_size(const NsaDecodeParams* p);

/* ---- context-parallel chunk reorder ------------------------------------------------------------------ */
typedef struct NsaReorderParams {
  const void* x; /* [2*world_size chunks of chunk_bytes bytes]                                            */
  void* y;       /* same size, must not alias x                                                           */
  int64_t chunk_bytes; /* multiple of 16                                                                  */
  int32_t world_size;
  int32_t unshuffle; /* 0: sequential -> rank-major zig-zag; 1: the inverse                               */
} NsaReorderParams;
/* replaces reorder, flash_nsa/ops/reorder.py:43-93 (out of place) */
int nsa_reorder(const NsaReorderParams* p, void* stream);

/* ---- writing new K/V rows into the paged cache (inference caller) -------------------------------------- */
typedef struct NsaStoreKvParams {
  const void *key, *value;     /* [N, H*D] bf16 rows (row strides below), the new tokens of a step                  */
  void *k_cache, *v_cache;     /* [slots, H*D] bf16, rows contiguous                                                 */
  const int32_t* slot_mapping; /* [N] flat cache row of every new token, -1 = skip (padding of a captured graph)     */
  int64_t key_stride, value_stride;
  int32_t N, row_elems;        /* row_elems = H*D, a multiple of 8                                                   */
} NsaStoreKvParams;
/* replaces store_kvcache, nano-vllm/nanovllm/layers/attention.py:123-154 */
int nsa_store_kvcache(const NsaStoreKvParams* p, void* stream);

/* ---- rotary position embedding (demo layers) ---------------------------------------------------------- */
typedef struct NsaRopeParams {
  const void *q, *k;     /* [B,N,QH,D], [B,N,KH,D] bf16; backward: the gradients of qe, ke                          */
  void *qe, *ke;         /* outputs, same shapes; may alias q, k (in place)                                          */
  const void *cos, *sin; /* [B,N,D] bf16 (a broadcast batch has stride 0)                                            */
  int64_t q_stride_b, q_stride_n, q_stride_h, k_stride_b, k_stride_n, k_stride_h;
  int64_t qe_stride_b, qe_stride_n, qe_stride_h, ke_stride_b, ke_stride_n, ke_stride_h;
  int64_t cos_stride_b, cos_stride_n; /* shared by cos and sin                                                       */
  int32_t B, N, QH, KH, D;            /* D % 16 == 0; the last dimension of every tensor is contiguous               */
  int32_t backward;                   /* 0: e1 = x1 cos1 - x2 sin1, e2 = x2 cos2 + x1 sin2 (x1, x2 the halves of a head);
                                         1: the transposed rotation applied to the incoming gradients               */
} NsaRopeParams;
/* replaces fused_apply_rope (forward and backward), flash_nsa/ops/rope.py:5-232 */
int nsa_rope(const NsaRopeParams* p, void* stream);

/* ---- weight gradient of the learned compression ------------------------------------------------------- */
typedef struct NsaWgradParams {
  const void* dy;    /* [rows, n_out] bf16: gradient of the compression's hidden state                       */
  const void* x;     /* [rows, n_in] bf16: the flattened windows (construct_block output, n_in = kernel_size * D) */
  float* main_grad;  /* [n_out, n_in] fp32: the trainer's accumulation buffer; the product is ADDED (atomics)  */
  int32_t* status;   /* optional device word for pipeline time-outs, as in NsaAttnParams                     */
  int64_t rows;
  int64_t dy_stride, x_stride, grad_stride; /* row strides in elements                                       */
  int32_t n_out, n_in;                      /* multiples of 128                                              */
} NsaWgradParams;
/* replaces the accumulating weight-gradient GEMM of weight_grad(), flash_nsa/modules/megatron_level_nsa.py:20-44
 * (apex's wgrad_gemm_accum_fp32, or the reference's Triton gemm(..., acc=True, transpose_a=True), ops/gemm.py:134):
 * main_grad += dy^T x with fp32 accumulation, one launch, split over the rows.                                   */
int nsa_wgrad_accum(const NsaWgradParams* p, void* stream);

/* ---- misc -------------------------------------------------------------------------------------------- */
/* No counterpart in the reference (Triton kernels have no bounded waits).  Runs the give-up path of the bounded pipeline
 * wait that every tcgen05 / TMA kernel here uses, on purpose and with nothing in flight: one warp polls a barrier that
 * nobody arrives on at most `polls` times (1 .. 2^20), then ORs bit 512 into *status and returns.  *waits_failed
 * (optional) receives 1000 * (number of waits that gave up) + the poll budget left for later waits.  The context stays
 * usable; a test calls this to see that a time-out becomes a status bit and not a hang.                              */
int nsa_selftest_wait_timeout(int32_t* status, int32_t polls, int32_t* waits_failed, void* stream);
const char* nsa_last_error(void);
int nsa_version(void);
/* The 16-bit element type this build of the library computes in: 0 = bf16 (libnsa_sm100.so), 1 = IEEE half
 * (libnsa_sm100_f16.so, the same sources compiled with -DNSA_F16; where this header says bf16, that build reads and writes
 * half).  The reference's ops take either type (its tests switch DTYPE, test.py:14); a host loads the library that matches
 * its tensors.                                                                                                        */
int nsa_element_type(void);
/* sizeof() of a parameter struct by name ("NsaAttnParams", ...), 0 if unknown: lets a binding verify its mirror */
int nsa_struct_size(const char* name);

#ifdef __cplusplus
}
#endif
#endif /* NSA_SM100_H_ */
