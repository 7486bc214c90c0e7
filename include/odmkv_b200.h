/*
 * odmkv_b200 -- C ABI of the B200 (sm_100a) implementation of ODM-KV's
 * compress-then-decode path: risk scoring, per-layer Lagrangian bit allocation,
 * Lloyd-Max quantise-and-pack into bit-width banks, and decode attention that reads the
 * packed banks directly.
 *
 * The reference (yiiwang118/ODM-KV) is pure Python/PyTorch and has no FFI; each entry point
 * below names the reference function whose arithmetic it replaces (paths relative to the
 * reference project root).  A Python caller binds these with ctypes.
 *
 * Conventions
 *   - every pointer is a DEVICE pointer unless its comment says "host";
 *   - the library allocates nothing on the device: callers pass outputs and workspaces
 *     (sizes come from the *_workspace_bytes queries, which are pure host arithmetic);
 *   - `stream` is a cudaStream_t passed as void*; all work is enqueued on it and nothing
 *     synchronises unless stated;
 *   - return value: 0 ok; negative = argument / shape / workspace error detected on the host
 *     before any launch; positive = CUDA runtime error code of a failed launch;
 *   - dtype codes for cache tensors: 0 = fp16, 1 = bf16, 2 = fp32;
 *   - head_dim is 128 throughout (the only value the reference's experiments use);
 *   - quantised levels are 2, 3, 4 and 8 bits ("level index" 0..3 in that order); level 16 is
 *     the exact (verbatim) bank and level 0 the evicted list.
 */
#ifndef ODMKV_B200_H
#define ODMKV_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define ODMKV_ABI_VERSION 1
#define ODMKV_HEAD_DIM 128
#define ODMKV_NUM_QLEVELS 4   /* 2, 3, 4, 8 bits */
#define ODMKV_NUM_CLASSES 6   /* evicted, 2, 3, 4, 8, exact-16 (class index = position in this list) */
#define ODMKV_SEG_ALIGN 16    /* every (batch, head) segment of a bank starts on a multiple of 16 slots */
#define ODMKV_TILE 128        /* tokens per quantise tile */
#define ODMKV_MAX_LEVELS 8    /* candidate widths of one Lagrangian problem */

#define ODMKV_OK 0
#define ODMKV_ERR_ARG (-1)
#define ODMKV_ERR_SHAPE (-2)
#define ODMKV_ERR_WORKSPACE (-3)
#define ODMKV_ERR_UNSUPPORTED (-4)
#define ODMKV_ERR_LIMIT (-5)

int odmkv_abi_version(void);
/* host string for a status code returned by any entry point */
const char *odmkv_status_string(int status);

/* ------------------------------------------------------------------------------------------
 * Scorer.  Replaces RiskScorer.score_prefill (kvquant/scorer.py:385-404) together with
 * _expected_core_internals (kvquant/scorer.py:285-318) and _pad_sinks_and_normalize with grain
 * "global" (kvquant/scorer.py:321-325): per sample, softmax over the positions after the sinks
 * of mu.k/sqrt(d), mean over the G query heads of a KV head, then
 * s = (p + eps)^2 (|v|^2 + |k|^2/d |v - o|^2); sink slots receive the maximum over the sample.
 *   K, V   [B, H, T, 128] contiguous, dtype code `dtype`, 16-byte aligned (ODMKV_ERR_ARG otherwise)
 *   mu     [B, H*G, 128] fp32 -- the averaged-RoPE'd mean query (query head index is KV-major)
 *   scores [B, H, T] fp32 out
 * T <= n_sink gives all ones (kvquant/scorer.py:388-389).
 */
size_t odmkv_score_workspace_bytes(int B, int H, int G, int T);
/* Offset (bytes) inside the score workspace of a 32-bit status word: 0 after a clean call, 1 when a bounded wait of
 * a sweep on one of its bulk copies expired (scores invalid).  No counterpart in the reference. */
size_t odmkv_score_status_offset(int B, int H, int G, int T, int n_sink);
int odmkv_score_prefill(const void *K, const void *V, int dtype, const float *mu, int B, int H, int G, int T,
                        int n_sink, float eps, float *scores, void *workspace, size_t workspace_bytes,
                        void *stream);

/* RiskScorer.score_with_attn (kvquant/scorer.py:406-416): same risk formula for R independent
 * rows of T tokens each with externally supplied attention weights p (the decode-buffer flush).
 *   K, V [R, T, 128]; p [R, T] fp32; scores [R, T] fp32 out.  T <= 1024. */
int odmkv_score_with_attn(const void *K, const void *V, int dtype, const float *p, int R, int T, float eps,
                          float *scores, void *stream);

/* ------------------------------------------------------------------------------------------
 * Allocator.  Replaces optimal_scores_to_bits (kvquant/allocator.py:459-663) for P independent
 * problems of n scores each (one problem = one (layer, sample): all KV heads flattened).
 */
typedef struct odmkv_alloc_report {
    double lam;            /* final lambda (the last midpoint) */
    double gap_before;     /* (avg - target) * n_active before gap closure */
    long long counts[ODMKV_MAX_LEVELS]; /* tokens per candidate level after gap closure */
    int n_active;          /* non-sink tokens */
    int evaluations;       /* number of assignment passes (66 when hi = 1 suffices) */
    int moved;             /* tokens moved by gap closure */
    int ties_lambda;       /* tokens whose two adjacent-level costs differ by < 1e-6 at the final lambda */
    int ties_cut;          /* gap-closure cuts that fall between two equal scores */
    int done;              /* 1 when the schedule completed */
} odmkv_alloc_report;

size_t odmkv_alloc_workspace_bytes(int P, int n);
/*   scores    [P, n] fp32
 *   sink_mask [n] uint8 or NULL (shared by all problems; nonzero = pinned to sink_bits)
 *   levels    host int[K] ascending candidate widths, eps host float64[K] (eviction cost already
 *             applied to the 0 level, i.e. allocator.py:550-552 done by the caller)
 *   bits      [P, n] int32 out;  reports [P] out (device)
 * With more than one problem the per-problem sorts run on up to eight helper streams of the library, forked from
 * and joined back into `stream` with events; the first call on a device creates them (host objects only) and must
 * not be made while `stream` is being captured.  One call at a time per device. */
int odmkv_allocate_bits(const float *scores, const uint8_t *sink_mask, int P, int n, const int *levels,
                        const double *eps, int K, double target_avg_bits, int sink_bits, int32_t *bits,
                        odmkv_alloc_report *reports, void *workspace, size_t workspace_bytes, void *stream);

/* Stepwise form for KV heads sharded over ranks: every rank evaluates its shard, the per-level
 * counts (and, during gap closure, the selection histograms) are summed over ranks by the caller
 * (an all-reduce on `exchange`, int64 [P, exchange_len]) between `eval` and `update`.
 * odmkv_alloc_step_* mirror exactly what odmkv_allocate_bits runs internally.
 *   idx_base: global index of this shard's first score inside the flattened problem. */
size_t odmkv_alloc_exchange_len(void);
int odmkv_alloc_begin(const float *scores, const uint8_t *sink_mask, int P, int n_local, long long idx_base,
                      const int *levels, const double *eps, int K, double target_avg_bits, int sink_bits,
                      void *workspace, size_t workspace_bytes, long long *exchange, void *stream);
int odmkv_alloc_eval(void *workspace, long long *exchange, void *stream);
int odmkv_alloc_update(void *workspace, const long long *exchange_reduced, void *stream);
/* host: number of eval/update rounds odmkv_alloc_* needs before odmkv_alloc_finish for K levels */
int odmkv_alloc_num_rounds(int K);
int odmkv_alloc_finish(void *workspace, int32_t *bits, odmkv_alloc_report *reports, void *stream);

/* ------------------------------------------------------------------------------------------
 * Quantise-and-pack.  Replaces TurboQuantAdaptiveKVCacheState.append
 * (kvquant/tq_adaptive_backend.py:350-374), QuantizedBank.append (149-174),
 * TurboQuantMSE.quantize (kvquant/tq_backend.py:185-197) and _pack_indices (103-125).
 *
 * A "chunk" is the packed form of one [B, H, T] block of tokens.  Per class c it holds a bank
 * whose slots are ordered (b, h, t) -- the row order of the reference's mask.nonzero() -- with
 * each (b, h) segment starting on a multiple of 16 slots (padding slots have pos = -1).
 *
 * Step 1 (plan): count classes, lay out segments.
 *   bits      [B, H, T] int32 with values in {0, 2, 3, 4, 8, 16}
 *   seg_start [6, B*H] int32 out, seg_count [6, B*H] int32 out
 *   totals    [6] int32 out (device): padded slots per class -- the caller reads it back to size
 *             the banks
 *   plan workspace keeps per-tile bases for step 2.
 */
size_t odmkv_pack_plan_workspace_bytes(int B, int H, int T);
int odmkv_pack_plan(const int32_t *bits, int B, int H, int T, int32_t *seg_start, int32_t *seg_count,
                    int32_t *totals, void *plan_workspace, size_t plan_workspace_bytes, void *stream);

/* Bank storage of one chunk; all device pointers, sized from `totals` (cap[c] slots, a multiple of 16).
 * Code bytes per slot: 32 (2-bit), 48 (3-bit, a true 3 bits per code), 64 (4-bit), 128 (8-bit).
 * The 8-bit bank is token-major (byte d of a slot = code of coordinate d).  The 2/3/4-bit banks are
 * stored in tiles of 16 slots arranged for the tensor-core fragments of the decode kernel: lane
 * (g, t) = (lane / 4, lane % 4) of a warp owns the 8*b bytes at tile + lane*8*b as 32 little-endian
 * pair fields of 2*b bits; keys: field 4s+2odd+hi = coordinates (32t+4s+2odd, +1) of slot g+8hi;
 * values: field 4m+2hi+a = coordinate 16m+g+8a of slots (2t+8hi, 2t+8hi+1) -- in both cases four consecutive
 * fields are the A registers of one HMMA step.  odmkv_export_bank converts any bank to the reference's byte layout. */
typedef struct odmkv_chunk {
    uint8_t *k_codes[ODMKV_NUM_QLEVELS];
    uint8_t *v_codes[ODMKV_NUM_QLEVELS];
    float *k_norm[ODMKV_NUM_QLEVELS];
    float *v_norm[ODMKV_NUM_QLEVELS];
    int32_t *pos[ODMKV_NUM_QLEVELS];  /* token position t, -1 for padding */
    void *exact_k;                    /* [cap16, 128] cache dtype */
    void *exact_v;
    int32_t *exact_pos;
    int32_t *evicted_pos;             /* [cap0] */
    const int32_t *seg_start;         /* [6, B*H] */
    const int32_t *seg_count;         /* [6, B*H] */
    int32_t cap[ODMKV_NUM_CLASSES];   /* slots allocated per class (>= totals) */
    int32_t B, H, T, t_offset;        /* t_offset is added to every stored position */
} odmkv_chunk;

/* Step 2: norm, normalise, rotate (one ascending fp32 FMA chain per coordinate), nearest centroid
 * (searchsorted + neighbour pick, lower index on ties), pack, write into the banks.
 *   pi_k, pi_v [128, 128] fp32 row-major (y = pi x);  codebooks [4][256] fp32 ascending
 *   (level index li uses the first 2^bits(li) entries). `chunk` is a HOST struct. */
size_t odmkv_quantize_workspace_bytes(const int32_t *cap /* host int32[6], slots per class */);
/* Status of the tensor-core quantise kernel (16-bit caches): 0 when none of its bounded waits has expired on the current
 * device since the library was loaded, 1 otherwise (the codes of that call are invalid); synchronises the device. */
int odmkv_quantize_status(void);
int odmkv_quantize_pack(const void *K, const void *V, int dtype, const int32_t *bits, const float *pi_k,
                        const float *pi_v, const float *codebooks, const odmkv_chunk *chunk,
                        const void *plan_workspace, void *workspace, size_t workspace_bytes, void *stream);

/* Encode-and-pack only: nearest centroid + pack of already rotated coordinates (the stand-in for
 * the absent kvquant/tq_triton.mse_nearest_centroid followed by _pack_indices).
 *   y [n, 128] fp32; codebook [2^bits] fp32; out [n, 16*bits] bytes: the little-endian bit stream of the
 *   128 codes of each row (for 2, 4 and 8 bits this is the reference's byte layout). */
int odmkv_encode_pack(const float *y, long long n, int bits, const float *codebook, uint8_t *out, void *stream);

/* Dequantise a chunk into dense [B, H, T_dense, 128] tensors (positions index the T axis).
 * Replaces TurboQuantMSE.dequantize (kvquant/tq_backend.py:199-203), QuantizedBank.materialize_into
 * (kvquant/tq_adaptive_backend.py:205-242) and ExactBank.materialize_into (66-71).
 *   out_dtype: 0/1/2 as above (fp32 gives the values before the cast to the cache dtype)
 *   include_exact: also scatter the exact bank.  Evicted rows are not touched. */
int odmkv_dequant_chunk(const odmkv_chunk *chunk, int in_dtype, const float *pi_k, const float *pi_v,
                        const float *codebooks, void *K_out, void *V_out, int out_dtype, int T_dense,
                        int include_exact, void *stream);

/* Export one quantised bank in the reference's bank layout (kvquant/tq_adaptive_backend.py:74-174,
 * kvquant/tq_backend.py:103-125): rows compacted in (b, h, t) order, 3-bit codes as nibbles.
 *   class_idx 1..4; indices_k/v [N, ref_bytes] uint8, norms [N] fp32, positions [N, 3] int64;
 *   row_start [B*H] int32 = exclusive prefix sum of seg_count for that class. */
int odmkv_export_bank(const odmkv_chunk *chunk, int class_idx, const int32_t *row_start, uint8_t *indices_k,
                      uint8_t *indices_v, float *norms_k, float *norms_v, int64_t *positions, void *stream);
/* positions of the exact (class 5) or evicted (class 0) list, same row order */
int odmkv_export_positions(const odmkv_chunk *chunk, int class_idx, const int32_t *row_start,
                           int64_t *positions, void *stream);

/* Merge n_src chunks (HOST array, at most 12, same B and H) into the chunk `dst` (HOST struct; banks allocated by the
 * caller from the summed segment counts, each (b, h) segment on a multiple of 16 slots, pos arrays preset to -1 and
 * norms to 0).  Inside every (b, h) segment of every class the tokens of chunk 0 come first, then chunk 1, ...; with
 * chunks in time order that is ascending position, the order the reference's growing banks have
 * (kvquant/tq_adaptive_backend.py:149-174, 481-532: flushed tokens are appended to the banks).
 *   dst_off [n_src, 6, B*H] int32 (device): first destination slot of chunk i inside the destination segment
 *   workspace: odmkv_quantize_workspace_bytes(dst->cap) bytes, 256-byte aligned. */
int odmkv_compact_chunks(const odmkv_chunk *src, int n_src, const odmkv_chunk *dst, const int32_t *dst_off, int dtype,
                         void *workspace, size_t workspace_bytes, void *stream);

/* ------------------------------------------------------------------------------------------
 * Decode attention over packed chunks.  Replaces, for q_len = 1, the attention call the
 * reference's wrapper forwards to after masking evicted keys (kvquant/attention_patch.py:30-55)
 * and the dense dequantised cache it reads: out = softmax(q K_hat^T * scale) V_hat over every
 * stored token of every chunk plus a dense tail of recent tokens, evicted tokens absent.
 *   q    [B, H*G, 128] dtype q_dtype;   out [B, H*G, 128] dtype out_dtype
 *   chunks: HOST array of n_chunks descriptors sharing B and H
 *   tail_k/tail_v [B, H, tail_cap, 128] cache dtype (may be NULL when tail_len = 0): the first
 *   tail_len tokens of every (b, h) are attended exactly
 *   lse  [B, H*G] fp32 out or NULL (log-sum-exp of the scaled logits)
 *   n_splits: partial-result slots per (b, h), at least 1 (odmkv_decode_default_splits gives a good value):
 *   odmkv_decode_attn runs that many CTAs per (b, h), at most 64.
 */
size_t odmkv_decode_workspace_bytes(int B, int H, int G, int n_splits);
int odmkv_decode_default_splits(int B, int H, long long max_tokens_per_head);
int odmkv_decode_attn(const void *q, int q_dtype, const odmkv_chunk *chunks, int n_chunks, int cache_dtype,
                      const void *tail_k, const void *tail_v, int tail_len, int tail_cap, const float *pi_k,
                      const float *pi_v, const float *codebooks, int B, int H, int G, float scale, void *out,
                      int out_dtype, float *lse, int n_splits, void *workspace, size_t workspace_bytes,
                      void *stream);

/* Tensor-core variant of odmkv_decode_attn (same contract and arguments): the 2-, 3- and 4-bit banks
 * are consumed with mma.sync m16n8k16 tiles straight from the tile layout; 8-bit, exact and tail
 * tokens take the CUDA-core kernel in a second launch on a forked stream.  The kernel is persistent: it picks
 * its own grid (one CTA pair per SM, shared evenly by the (b, h) units) such that at most n_splits CTAs overlap one
 * unit; n_splits may go up to 128 and only bounds the workspace.
 *   lut_scales: host float[3] or NULL (= 1.0): per level a factor s such that fp16(c * s) carries the
 *   centroids of the 2-, 3-, 4-bit codebooks with less rounding error; divided out again in fp32. */
int odmkv_decode_attn_mma(const void *q, int q_dtype, const odmkv_chunk *chunks, int n_chunks, int cache_dtype,
                          const void *tail_k, const void *tail_v, int tail_len, int tail_cap, const float *pi_k,
                          const float *pi_v, const float *codebooks, int B, int H, int G, float scale, void *out,
                          int out_dtype, float *lse, int n_splits, void *workspace, size_t workspace_bytes,
                          const float *lut_scales, void *stream);

/* odmkv_decode_attn_mma with the tail length in device memory (no counterpart in the reference, whose decode step
 * concatenates onto dense tensors, transformers/cache_utils.py DynamicLayer.update).  The launch attends
 * min(*tail_len_dev + tail_len_add, tail_cap) tokens of the tail, read when the kernel runs; tail_len_bound
 * (1..tail_cap) is the largest value it may take and only sizes the launch.  A decode step captured into a CUDA
 * graph therefore stays valid while the tail grows: the host replays it and a device counter advances. */
int odmkv_decode_attn_mma_devtail(const void *q, int q_dtype, const odmkv_chunk *chunks, int n_chunks, int cache_dtype,
                                  const void *tail_k, const void *tail_v, const int32_t *tail_len_dev, int tail_len_add,
                                  int tail_len_bound, int tail_cap, const float *pi_k, const float *pi_v,
                                  const float *codebooks, int B, int H, int G, float scale, void *out, int out_dtype,
                                  float *lse, int n_splits, void *workspace, size_t workspace_bytes,
                                  const float *lut_scales, void *stream);

/* Decode attention without a caller-supplied workspace (no counterpart in the reference).  For hosts
 * that cannot allocate device memory on the decode path -- a serving loop with a frozen memory pool, a
 * thread that may not take the driver's allocation lock, a plug-in that only ever receives raw device
 * pointers.  Same arguments and result as odmkv_decode_attn_mma, but the scratch is a device array inside
 * the library: odmkv_decode_attn_noalloc_scratch_bytes() bytes (6 MiB) held by every GPU that loads the
 * library until the process exits.  Sizes whose partials need more (roughly B*H*(n_splits+8)*8 KiB for
 * G <= 4, twice that for G <= 8) return ODMKV_ERR_LIMIT and launch nothing.  The first call on a device
 * resolves the array's address and should come before any stream capture.  All calls on a device share
 * the array: calls that overlap on the GPU race, so keep them on one stream.  It calls no cudaMalloc,
 * cudaFree or other routine that allocates device memory; the first decode call on a device (through any
 * entry point) also creates one helper stream and two events and sets the kernels' shared-memory attribute
 * (host objects only), which is one more reason to make it before a capture. */
size_t odmkv_decode_attn_noalloc_scratch_bytes(void);
int odmkv_decode_attn_noalloc(const void *q, int q_dtype, const odmkv_chunk *chunks, int n_chunks, int cache_dtype,
                              const void *tail_k, const void *tail_v, int tail_len, int tail_cap, const float *pi_k,
                              const float *pi_v, const float *codebooks, int B, int H, int G, float scale, void *out,
                              int out_dtype, float *lse, int n_splits, const float *lut_scales, void *stream);

/* ------------------------------------------------------------------------------------------
 * Column statistics of causal softmax attention.  Replaces _chunked_attention_qk
 * (kvquant/attention_utils.py:160-211), the reference's windowed-attention building block whose column sums feed
 * RiskScorer.score_with_attn (kvquant/scorer.py:406-416): logits q_r.k_j / scale, keys j > r + q_offset hidden from
 * query r (the reference's mask is q_offset = 0; a window of the last Tq positions takes q_offset = Tkv - Tq),
 * softmax over the keys per query, mean over the G query heads of a KV head, and per key the sum, the maximum and
 * the sum of squares of that mean over the queries.
 *   Q [B, H*G, Tq, 128], K [B, H, Tkv, 128]: fp16 or bf16 (dtype code), contiguous, 16-byte aligned
 *   sum_attn, max_attn, sum_sq_attn: [B, H, Tkv] fp32 out
 *   workspace: odmkv_window_stats_workspace_bytes(B, H, G, Tq) bytes; the 32-bit word at
 *   odmkv_window_stats_status_offset(...) is 0 after a clean run, 1 if a bounded wait expired (results invalid)
 * G <= 16.  Runs on the tcgen05 tensor cores (two passes: log-sum-exp per query, then the statistics per key),
 * operand tiles staged by TMA tensor copies where the shapes allow. */
size_t odmkv_window_stats_workspace_bytes(int B, int H, int G, int Tq);
size_t odmkv_window_stats_status_offset(int B, int H, int G, int Tq);
/* how the last call on this process staged its operand tiles: 1 = tensor copies (TMA), 0 = 16-byte copies by the
 * threads (taken when the driver's tensor-map encoder is unavailable, or when forced), -1 = no call yet */
int odmkv_window_stats_last_path(void);
/* on != 0: stage by thread copies even where tensor copies are possible (for testing that path) */
void odmkv_window_stats_force_thread_copies(int on);
int odmkv_window_attn_stats(const void *Q, const void *K, int dtype, int B, int H, int G, int Tq, int Tkv, int q_offset,
                            float scale, float *sum_attn, float *max_attn, float *sum_sq_attn, void *workspace,
                            size_t workspace_bytes, void *stream);

/* ------------------------------------------------------------------------------------------
 * Optional kernel timing (no counterpart in the reference).  When enabled, the launchers bracket
 * their dominant kernel with CUDA events on the launching stream under the names "score",
 * "allocate", "quantize", "decode_main"; odmkv_timing_read waits for the events recorded since the
 * last read and returns their summed duration and count. */
void odmkv_timing_enable(int on);
int odmkv_timing_read(const char *kernel, double *total_ms, long long *launches);

#ifdef __cplusplus
}
#endif
#endif /* ODMKV_B200_H */
