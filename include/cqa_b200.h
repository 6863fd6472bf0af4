/*
 * cqa_b200 — C ABI of the B200 (sm_100a) certified quantised decode-attention path.
 *
 * One shared library, `extern "C"`, plain pointers and sizes.  Unless a
 * parameter is documented as host memory, every pointer is a DEVICE pointer.
 * Every call that launches work takes a `cudaStream_t` passed as `void*`
 * (NULL = legacy default stream), returns 0 on success or a negative
 * `cqa_status` and never throws.  No compute entry point allocates or frees
 * device memory: all buffers, including scratch, belong to the caller.  The
 * one exception is the pair cqa_peer_alloc / cqa_peer_free, which exists to
 * create the exchange buffer that peers map.
 *
 * Geometry is fixed to what the reference's native kernels hard-wire
 * (dotcache/backends/cuda_kernels/certified_blackwell.cpp:110,226): head_dim =
 * d_v = 128, 16 tokens per block ("page"), INT4 group size 16.  gqa_group may
 * be 1, 2, 4 or 8.
 *
 * Citations below name the reference interface each entry point replaces, as
 * file:line inside the reference project (DeanoC/certified-quantised-attention).
 */
#ifndef CQA_B200_H
#define CQA_B200_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define CQA_HEAD_DIM 128
#define CQA_BLOCK 16
#define CQA_GROUP 16
#define CQA_NGROUPS 8
#define CQA_MAX_RANKING_K 32
#define CQA_MAX_SORT_BLOCKS 16384 /* selector limit: quantised blocks per call */
#define CQA_MAX_SPLITS 256        /* Phase-2 splits per KV head */
#define CQA_MAX_DENSE_SPLITS 64   /* dense-recompute chunks per head */

typedef enum cqa_status {
    CQA_OK = 0,
    CQA_ERR_INVALID = -1,   /* bad argument (NULL pointer, unsupported size or dtype) */
    CQA_ERR_CUDA = -2,      /* a CUDA runtime call failed; see cqa_last_error() */
    CQA_ERR_UNSUPPORTED = -3,
    CQA_ERR_TOO_LARGE = -4, /* request exceeds a documented limit */
    CQA_ERR_TIMEOUT = -5    /* a bounded device-side wait ran out */
} cqa_status;

typedef enum cqa_dtype { CQA_F32 = 0, CQA_F16 = 1, CQA_BF16 = 2 } cqa_dtype;

/* One layer's cache arrays (the fields of the reference's TieredKeyCacheLayer,
 * dotcache/kernels/tiered_kv_cache.py:29-132).  Row-major; `cap_tokens` and
 * `max_blocks` are the per-KV-head strides (in token rows / blocks) so the
 * active prefix is addressed in place, without copies. */
typedef struct cqa_cache {
    int32_t kv_heads;
    int32_t gqa_group;
    int32_t t2_dtype;                /* cqa_dtype of keys_t2 / values_t2 */
    int32_t reserved;
    int64_t cap_tokens;              /* rows per KV head in the per-token arrays */
    int64_t max_blocks;              /* blocks per KV head in the per-block arrays */
    int8_t *keys_int8;               /* [KV][cap][128] */
    float *keys_scale;               /* [KV][max_blocks][128] */
    float *keys_zero_points;         /* [KV][max_blocks][128] */
    float *correction;               /* [KV][max_blocks] */
    float *sigma_max;                /* [KV][128] running max of keys_scale over quantised blocks */
    uint8_t *values_int4_packed;     /* [KV][cap][64], low nibble = even channel */
    uint16_t *values_int4_scales;    /* [KV][cap][8] IEEE half bits */
    uint16_t *values_int4_zeros;     /* [KV][cap][8] IEEE half bits */
    float *values_int4_errors;       /* eta_b [KV][max_blocks] */
    float *values_int4_error_sums;   /* [KV][max_blocks] */
    int32_t *values_int4_error_counts; /* [KV][max_blocks] */
    float *values_norm_max;          /* nu_b [KV][max_blocks] */
    void *keys_t2;                   /* Tier-2 keys, [KV][keys_t2_rows][128] of t2_dtype */
    int64_t keys_t2_rows;
    void *values_t2;                 /* Tier-2 values, [KV][values_t2_rows][128] */
    int64_t values_t2_rows;
    const int32_t *key_slots;        /* block -> 16-row slot in keys_t2; NULL = identity */
    const int32_t *value_slots;      /* block -> slot in values_t2; NULL = identity */
    /* Bounded hot tier: when a slot table is given, keys_t2 / values_t2 are scratch arrays of a few thousand
     * blocks and the complete Tier-2 lives in the backing arrays ([KV][t2_backing_rows][128] of t2_dtype, row =
     * token index), typically pinned host memory mapped into the device address space.  Blocks with slot -1 are read
     * from the backing array directly; cqa_hot_tier_update pages them in afterwards. */
    void *keys_t2_backing;
    void *values_t2_backing;
    int64_t t2_backing_rows;
} cqa_cache;

/* Certification knobs (the keyword arguments of certified_attention_layer,
 * dotcache/kernels/certified_attention.py:1065-1097). */
typedef struct cqa_knobs {
    float q_scale;
    float tau_cov;
    float rung1_threshold;       /* < 0 disables Rung-1 expansion */
    float rung1_multiplier;
    float eps_guard;
    float exploration_rate;
    float v_tolerance;
    int32_t k_min;
    int32_t k_max;               /* <= 0: no cap */
    int32_t ranking_r;
    int32_t top_k_fp16_keys;
    int32_t ranking_fallback;    /* bool */
    int32_t rung3_recompute;     /* bool: ranking_fallback_mode == "full" */
    int32_t score_consistency;   /* bool */
    int32_t value_mode_tight;    /* bool: "tight" (1) or "loose" (0) */
    int32_t force_trailing_value_fp16; /* bool */
} cqa_knobs;

/* Per-head results of selection and certification (device memory, one per q head). */
typedef struct cqa_head_cert {
    int32_t k_star;
    int32_t k_star_base;
    int32_t k_star_expanded;
    int32_t rung1_triggered;
    int32_t exploration_blocks;
    int32_t ranking_disagree;    /* top-r ranking disagreement (before the boundary check) */
    int32_t ranking_disagree_r1;
    int32_t ranking_disagree_r3;
    int32_t boundary_triggered;
    int32_t rung3;               /* ranking_disagree | boundary_triggered */
    int32_t consistency_violation;
    int32_t value_promoted_blocks;
    int32_t dense;               /* this head's output comes from the dense FP16 recompute */
    int32_t reserved[3];
    float tail_mass;
    float tau_actual;
    float m_global;
    float total_mass;
    float delta;
    float e_pre;
    float e_val;
    float boundary_ub;           /* max over tail blocks of ell_int8 + delta */
    float ell_fp16_r;            /* r-th largest FP16 log-mass among the re-scored blocks */
    float fp16_top1;             /* largest FP16 block score */
    float fp16_top2;
    float int8_top1;             /* m_b of the best INT8 block */
    int32_t top_blocks[CQA_MAX_RANKING_K];
    float fp16_scores[CQA_MAX_RANKING_K];
    float fp16_logmass[CQA_MAX_RANKING_K];
} cqa_head_cert;

/* Caller-owned scratch and outputs of one layer step.  H = kv_heads*gqa_group,
 * nq = fully quantised blocks, nact = active blocks (nq or nq+1),
 * ld = leading dimension (>= nact) of the [H][ld] arrays. */
typedef struct cqa_workspace {
    int64_t ld;
    float *m_b;                  /* [H][ld] */
    float *s_b;                  /* [H][ld] */
    float *token_scores;         /* [KV][nq][G][16] */
    float *mass_frac;            /* [H][ld] */
    uint8_t *topk_mask;          /* [H][ld] 1 = FP16 keys for this (head, block) */
    uint8_t *value_mask;         /* [H][ld] 1 = FP16 values */
    uint8_t *explore_mask;       /* [H][ld] */
    int32_t *sorted_idx;         /* [H][sel_width] */
    float *sorted_cumsum;        /* [H][sel_width] */
    int32_t sel_width;           /* >= min(expanded k_max, nq); ignored if k_max <= 0 (then ld) */
    int32_t num_splits;          /* Phase-2 splits per KV head */
    int32_t dense_splits;        /* dense recompute splits per head */
    int32_t reserved;
    float *part_m;               /* [H][num_splits] */
    float *part_l;               /* [H][num_splits] */
    float *part_acc;             /* [H][num_splits][128] */
    float *dense_m;              /* [H][dense_splits] */
    float *dense_l;
    float *dense_acc;            /* [H][dense_splits][128] */
    cqa_head_cert *cert;         /* [H] */
    int32_t *any_flags;          /* [5 + H]: any rung1, any rung3, any rung4 (violation), any value promotion,
                                    number of heads flagged for dense recompute, then their ids */
    float *out;                  /* [H][128] float32 */
    int32_t *tickets;            /* [KV + H] merge tickets: zero them once after allocation; kernels leave them at zero */
    /* Sequence-sharded runs only (NULL otherwise). */
    const float *given_fp16;     /* [H][CQA_MAX_RANKING_K][2]: FP16 score and log-mass of each top-list block,
                                    computed by the rank that owns the block (cqa_rescore_owned) and summed over ranks */
    float *partial_out;          /* [H][CQA_PARTIAL_STRIDE]: when set, cqa_attend writes the un-normalised
                                    (max, sum, acc[128]) of its own blocks here instead of the output rows */
    /* Exploration draw when no uniforms are passed (exploration_u == NULL, exploration_rate > 0): one
     * Philox4x32-10 value per (head, block), keyed by rng_seed, counter (block, head, rng_offset).  Callers
     * advance rng_offset by one per call.  Same distribution as the reference's torch.rand draw, not the
     * same stream. */
    uint64_t rng_seed;
    uint64_t rng_offset;
    /* Sequence-sharded selector input straight from the all-gather buffer (0 = plain [row][ld] arrays):
     * m_b, s_b and cqa_cache.values_int4_errors then point at the rows of rank 0 inside a buffer laid out
     * [rank][row][shard_chunk] with shard_rank_stride floats per rank; global block b lives in rank
     * r = min(b / shard_stride, shard_ranks - 1), column b - r * shard_stride. */
    int64_t shard_stride;
    int64_t shard_chunk;
    int64_t shard_rank_stride;
    int32_t shard_ranks;
    int32_t given_ranks;         /* > 1: given_fp16 holds one [H][32][2] array per rank, given_rank_stride floats
                                    apart; the kernel adds them (only the owner of a block contributes non-zero) */
    int64_t given_rank_stride;
    /* With shard_ranks > 0, cqa_cache.sigma_max points at rank 0's row of per-channel scale maxima inside the
     * exchange buffer and the kernel takes the maximum over the ranks' rows (shard_rank_stride apart). */
    /* Peer exchange (cqa_sharded_layer_step): before reading exchanged data the kernel waits, with a bounded
     * spin, until wait_flags[i] >= wait_value for every i < wait_n except i == wait_skip; on a timeout it sets
     * *wait_status to a non-zero code and carries on (the step's result is then invalid, the GPU stays usable). */
    const int32_t *wait_flags;
    int32_t wait_n;
    int32_t wait_skip;
    int32_t wait_value;
    int32_t wait_spins;          /* polls of one flag before giving up; 0 = the default (about half a second) */
    int32_t *wait_status;
    /* Exchange B inside the selector (cqa_sharded_layer_step): the ranking-check CTA of a head re-scores the
     * top-list blocks this rank owns ([peer_first_block, +peer_n_local), local block ids), writes (score, log-mass)
     * into every rank's buffer at peer_xb[r], releases peer_flags_b[r][peer_rank * H + head] = peer_step, waits
     * (bounded) for the other ranks' flags in its own buffer and carries on to the flags.  peer_world = 0: off. */
    float *peer_xb[8];
    int32_t *peer_flags_b[8];
    /* Exchange C from inside cqa_attend: with peer_partial[r] set (r < peer_world), the un-normalised partial rows
     * are written into every rank's buffer (peer_partial[peer_rank] is this rank's own slot and replaces
     * partial_out), and the last merge of the launch releases *peer_flag_c[r] = peer_step on the other ranks. */
    float *peer_partial[8];
    int32_t *peer_flag_c[8];
    int32_t *peer_ticket_c;
    int64_t peer_first_block;
    int64_t peer_n_local;
    int32_t peer_world;
    int32_t peer_rank;
    int32_t peer_step;
    int32_t reserved3;
} cqa_workspace;

#define CQA_PARTIAL_STRIDE 130

const char *cqa_version(void);
/* Text of the last error on the calling thread (host memory, valid until the next call). */
const char *cqa_last_error(void);
/* Number of bounded device-side waits on staged copies that ran out on the current device since the library was
 * loaded (0 in a healthy run; a non-zero count means results of the affected calls are invalid).  Synchronises with
 * the device.  `reset` != 0 clears the counter. */
int cqa_wait_timeouts(int *count, int reset);
/* Kernels this library has launched in this process so far (all threads); `reset` != 0 also sets the count to 0. */
int64_t cqa_launch_count(int reset);

/* Quantise `n_blocks` complete blocks starting at block `first_block` from
 * K/V in `src_dtype` ([KV][src_rows][128], token 0 of the source = token
 * first_block*16 of the cache): INT8 keys (scale, zero point, correction,
 * sigma_max), INT4 values (packed, scales, zeros, eta_b = max over the block,
 * error sums/counts), nu_b, and copies the rows into the Tier-2 arrays
 * (converted to t2_dtype).  Replaces TieredKeyCacheLayer.from_fp16_cache /
 * from_fp16_cache_int4v (tiered_kv_cache.py:135-405) and
 * quantise_int4_grouped_block (int4_group_quantise.py:123-151). */
int cqa_quantize_blocks(const cqa_cache *c, const void *k_src, const void *v_src, int src_dtype,
                        int64_t src_rows, int64_t first_block, int64_t n_blocks, void *stream);

/* Whole-model prefill encode in one call: for each item (one layer's cache) the complete 16-token blocks of
 * its n_tokens source rows are quantised as by cqa_quantize_blocks, straight from the strided
 * [KV][src_rows][128] prefill tensors (no contiguous copy of the aligned prefix), and the ragged remainder
 * (n_tokens % 16 tokens) is appended by ONE launch whose CTAs walk the tokens of their KV head in order, with the
 * arithmetic of cqa_append_token.  `items` is a host array; every item is checked before the first launch.
 * Replaces the per-layer loop of create_tiered_cache_int4v_from_model / create_tiered_cache_from_model
 * (tiered_kv_cache.py:1579-1701), which quantises layer by layer and appends the remainder token by token
 * from Python. */
typedef struct {
    cqa_cache cache;
    const void *k_src;    /* [KV][src_rows][128] of the call's src_dtype (device) */
    const void *v_src;
    int64_t src_rows;     /* rows per KV head in the source tensors */
    int64_t n_tokens;     /* tokens to encode (<= src_rows) */
    int32_t defer_int4;   /* as in cqa_append_token, for the remainder */
    int32_t reserved;
} cqa_prefill_item;
int cqa_prefill_encode(const cqa_prefill_item *items, int n_items, int src_dtype, void *stream);

/* Fused append-and-quantise of one token at position `pos` for every KV head:
 * Tier-2 rows, nu_b, per-token INT4 (unless `defer_int4`), and, when the token
 * completes a block, the block's INT8 keys and (deferred) INT4 values with
 * eta_b = mean of the 16 token errors; poisons the unused INT8 rows of a newly
 * opened block with -127.  k_new/v_new: [KV][128] of `src_dtype`.
 * Replaces TieredKeyCacheLayer.append_token / _quantize_block /
 * _quantize_value_block (tiered_kv_cache.py:545-708, 480-543, 407-453). */
int cqa_append_token(const cqa_cache *c, const void *k_new, const void *v_new, int src_dtype,
                     int64_t pos, int defer_int4, void *stream);

/* Per-token per-group INT4 quantisation of x [T][128] (src_dtype): packed
 * [T][64], scales/zeros [T][8] half, rel_err/abs_err [T] float32.
 * Replaces quantise_int4_grouped (int4_group_quantise.py:22-88). */
int cqa_int4_quantise(const void *x, int src_dtype, int64_t T, uint8_t *packed, uint16_t *scales,
                      uint16_t *zeros, float *rel_err, float *abs_err, void *stream);

/* Phase 1: m_b, S_b [H][ld] for blocks [0, nq) and, if token_scores != NULL,
 * the 16 token scores per (kv, block, head).  q: [H][128] of q_dtype.
 * Replaces score_blocks_cuda (backends/certified_blackwell.py:64-87) and
 * fused_score_certify_multihead (kernels/fused_score_certify.py:398-456). */
int cqa_score_blocks(const cqa_cache *c, const void *q, int q_dtype, int64_t nq, float q_scale,
                     float *m_b, float *s_b, int64_t ld, float *token_scores, void *stream);

/* Adaptive top-K* selection with the Rung-1 expansion and the exploration
 * draw: fills mass_frac, sorted_idx, sorted_cumsum, topk_mask (blocks >= nq up
 * to nact are forced to 1), explore_mask and the selection fields of cert[].
 * exploration_u: [H][u_ld] uniforms in [0,1) or NULL.
 * Replaces adaptive_topk_cuda (backends/certified_blackwell.py:90-107),
 * compute_adaptive_topk_mask and augment_mask_with_exploration
 * (kernels/certified_attention.py:245-444, 882-909, 1299-1535). */
int cqa_select(const cqa_cache *c, const cqa_knobs *knobs, const cqa_workspace *ws, int64_t nq,
               int64_t nact, const float *exploration_u, int64_t u_ld, void *stream);

/* FP16-key block re-score: scores/logmass [H][K] for block ids idx [H][K].
 * Replaces fp16_block_scores_triton (kernels/fp16_block_scores_triton.py:73-146). */
int cqa_fp16_block_scores(const cqa_cache *c, const void *q, int q_dtype, const int32_t *idx, int K,
                          int64_t n_scoring_blocks, float q_scale, float *scores, float *logmass,
                          void *stream);

/* Delta[h] = sum_c |q[h][c]| * sigma_max[kv(h)][c] / (2*sqrt(128)).
 * Replaces compute_delta_bound (kernels/certified_attention.py:912-945) with
 * sigma_max maintained by the quantisers. */
int cqa_delta_bound(const cqa_cache *c, const void *q, int q_dtype, float *delta, void *stream);

/* Ranking / boundary / score-consistency checks and the Rung-2 value check:
 * fills the certificate fields of cert[], value_mask and any_flags.  Must run
 * after cqa_select on the same workspace.
 * Replaces certified_attention.py:1563-1727 and :1940-2034. */
int cqa_certify(const cqa_cache *c, const cqa_knobs *knobs, const cqa_workspace *ws, const void *q,
                int q_dtype, int64_t nq, int64_t nact, void *stream);

/* Phase 2: mixed INT8/FP16-key, INT4/FP16-value split-K attend over blocks
 * [0, nact) with `last_block_valid` valid tokens in the last block, the dense
 * FP16 recompute of heads whose cert[h].dense is set, and the LSE merge into
 * ws->out (one launch; the last CTA per KV head merges).  INT8 blocks reuse
 * ws->token_scores.  ws->num_splits must not exceed nact.
 * Replaces hybrid_mixedv_split_k_cuda (backends/certified_blackwell.py:138-224),
 * selective_attend_multihead_hybrid_{int4v,mixedv,mixedv_split_k}
 * (kernels/selective_attend_triton.py:633-708, 1448-1576),
 * recompute_heads_dense_fp16 and sdpa_attend_with_skip
 * (kernels/certified_attention.py:789-879, 989-1062). */
int cqa_attend(const cqa_cache *c, const cqa_workspace *ws, const void *q, int q_dtype, int64_t nq,
               int64_t nact, int64_t num_tokens, int last_block_valid, float q_scale, void *stream);

/* Dense attention over the Tier-2 keys and values for the heads the attached certificate lists: heads with
 * cert[h].dense set, their number in any_flags[4] and their ids in any_flags[5..]; or every head when any_flags[2]
 * is non-zero.  Only the dense-recompute CTAs of the attend kernel run; rows of listed heads go to ws->out, other
 * rows are left alone.  Needs cert, any_flags, dense_m/dense_l/dense_acc (dense_splits), tickets and out.
 * Replaces recompute_heads_dense_fp16 and sdpa_attend_with_skip called on their own
 * (kernels/certified_attention.py:789-879, 989-1062). */
int cqa_dense_attend(const cqa_cache *c, const cqa_workspace *ws, const void *q, int q_dtype, int64_t num_tokens,
                     float q_scale, void *stream);

/* Limits of cqa_attend_static (the size of its built-in scratch). */
#define CQA_STATIC_MAX_HEADS 64
#define CQA_STATIC_MAX_SPLITS 128
#define CQA_STATIC_MAX_DENSE_SPLITS 64

/* Same work and same result as cqa_attend, for callers that cannot hand over
 * scratch buffers because they are not able to allocate device memory at all:
 * for example a plugin loaded into a serving engine that has already claimed
 * the whole GPU for its own memory pool, or a decode loop in which calling
 * the driver's allocator is off limits because it stalls the device.  This
 * entry point has no counterpart in the reference project.
 *
 * The split partials (m, l, acc[128] per head and split, for Phase 2 and for
 * the dense recompute) live in an array that is part of the library image
 * (about 6.3 MB of device memory on every GPU that loads the library, held
 * until the process exits).  ws->part_m/part_l/part_acc and
 * ws->dense_m/dense_l/dense_acc are ignored and may be NULL; every other
 * field of ws, the inputs and ws->out are the caller's as usual.
 * Limits: kv_heads*gqa_group <= CQA_STATIC_MAX_HEADS, ws->num_splits <=
 * CQA_STATIC_MAX_SPLITS, ws->dense_splits <= CQA_STATIC_MAX_DENSE_SPLITS;
 * anything larger returns CQA_ERR_TOO_LARGE and launches nothing.
 * The call performs no device allocation or free, directly or through a
 * library.  The first call on each device looks up the device address of
 * the array (with that device current); make that first call outside any
 * stream capture.  All calls on a device share the one array and it keeps
 * whatever the previous call left there.  The only part that has to start at
 * zero is the row of merge tickets, and every call clears it itself with a
 * memset queued ahead of its kernel; the partials need no clearing because
 * each call overwrites every partial it later reads.  Two calls whose kernels
 * can overlap on the GPU (different streams) would overwrite each other's
 * partials and tickets: serialise them. */
int cqa_attend_static(const cqa_cache *c, const cqa_workspace *ws, const void *q, int q_dtype, int64_t nq,
                      int64_t nact, int64_t num_tokens, int last_block_valid, float q_scale, void *stream);

/* The whole per-layer chain on one stream: score -> select -> certify ->
 * attend.  No host synchronisation; results stay on the device.
 * Replaces certified_attention_layer (kernels/certified_attention.py:1065-2790)
 * for the adaptive-K*, INT4-value configuration. */
int cqa_layer_step(const cqa_cache *c, const cqa_knobs *knobs, const cqa_workspace *ws, const void *q,
                   int q_dtype, int64_t num_tokens, int64_t nq, const float *exploration_u,
                   int64_t u_ld, void *stream);

/* One decode step of one layer from HOST buffers: copies the packed step inputs
 * [q (H*128) | k_new (KV*128) | v_new (KV*128)] (elements of `dtype`) from `qkv_host`
 * to the device scratch `qkv_dev` (same size), appends the token at position `pos`
 * (cqa_append_token), runs cqa_layer_step on the pos+1 tokens with the H*128 float32
 * output rows going to `out_host`, and waits for the stream.  A pinned `qkv_host` makes the
 * input copy an asynchronous DMA transfer; a pinned `out_host` is written by Phase 2
 * directly (ws->out is then left untouched), any other is filled by a copy from ws->out.  An addition with no reference counterpart: it is
 * cqa_append_token + cqa_layer_step for a caller that holds its activations on the host,
 * in one call (no interpreter between the launches). */
int cqa_decode_step_host(const cqa_cache *c, const cqa_knobs *knobs, const cqa_workspace *ws, const void *qkv_host,
                         void *qkv_dev, int dtype, int64_t pos, int defer_int4, float *out_host, void *stream);

/* The same work queued on `stream` without the final wait: a decoder calls it once per
 * layer and waits on the stream once per token, so the copies and launches of layer l+1
 * are queued while layer l runs.  qkv_host and out_host must stay untouched until the
 * caller has waited on the stream; qkv_dev and the workspace may be shared by the layers
 * (stream order protects them). */
int cqa_decode_step_host_async(const cqa_cache *c, const cqa_knobs *knobs, const cqa_workspace *ws,
                               const void *qkv_host, void *qkv_dev, int dtype, int64_t pos, int defer_int4,
                               float *out_host, void *stream);

/* One decode token of a whole model from host buffers: the inputs of all n_layers entries are
 * copied to the device first (qkv_dev holds n_layers rows of (H + 2 KV) * 128 elements), then
 * each layer's append and layer step are queued in order, then ONE wait on the stream.  When
 * out_host is pinned memory that the device can address, Phase 2 writes the rows into it
 * directly (ws->out of that layer is then left untouched); otherwise they are copied.  No
 * transfer sits between two layers' kernels, and the loop over the layers runs inside the
 * library.  knobs and dtype are shared by the layers; all caches share the head geometry. */
typedef struct cqa_layer_call {
    const cqa_cache *cache;
    const cqa_workspace *ws;
    const void *qkv_host; /* [q | k_new | v_new] of this layer, pinned host memory */
    float *out_host;      /* [H, 128] float32, pinned host memory */
    int64_t pos;          /* tokens already in this layer's cache */
    int32_t defer_int4;
    int32_t reserved;
} cqa_layer_call;

int cqa_decode_token_host(const cqa_layer_call *layers, int n_layers, const cqa_knobs *knobs, void *qkv_dev, int dtype,
                          void *stream);

/* ---- batches: several sequences in one launch of each kernel ----
 * The reference runs batch 1 only (its adapter raises on anything else, dotcache/integrations/llama.py:717-718), so a
 * batch of B sequences costs it B serial kernel chains per layer.  cqa_layer_step_batched puts (sequence, KV head,
 * block range) on the grid of each of the kernels, so that many short sequences fill the GPU together.  Each sequence
 * gets exactly the arithmetic of its own cqa_append_token + cqa_layer_step call: results are bit-identical to the
 * one-sequence entry points when ws.num_splits is the same.  No reference counterpart.
 *
 * One record per sequence; all caches of a call share kv_heads, gqa_group and t2_dtype; every workspace carries the
 * dense scratch.  The exploration draw is the in-kernel one (ws.rng_seed / ws.rng_offset of each record). */
typedef struct cqa_batch_item {
    cqa_cache cache;
    cqa_workspace ws;
    const void *q;        /* [H][128] elements of the call's dtype (device) */
    const void *k_new;    /* [KV][128] key row of the token to append (device); unused when do_append == 0 */
    const void *v_new;
    int64_t pos;          /* tokens in the cache before this step's append (the step attends pos + do_append tokens) */
    int32_t defer_int4;
    int32_t reserved;
} cqa_batch_item;

/* `items_host` (host memory, n_items records) is copied to `items_dev` (device scratch of the same size, 16-byte
 * aligned) on the stream; then, with grid.z = sequence: the fused append (when do_append != 0), Phase 1, the
 * selector / certifier and Phase 2.  Limits: n_items <= 65535, every sequence at least one complete block after the
 * append. */
int cqa_layer_step_batched(const cqa_batch_item *items_host, int n_items, void *items_dev, const cqa_knobs *knobs,
                           int dtype, int do_append, void *stream);

/* ---- sequence sharding: every rank owns a contiguous range of blocks ----
 * The reference runs one cache per process; these entry points let P ranks that each
 * hold the blocks [first_block, first_block + n_local) of one long sequence reproduce
 * the unsharded certificate bit for bit (same selector on the all-gathered m_b / S_b /
 * eta arrays) and merge their Phase-2 partials.  No reference counterpart.
 *
 * cqa_select_certify_local: selector, value check and the top-list search on global
 * arrays (ws->m_b, ws->s_b, c->values_int4_errors cover all blocks of all ranks); stops
 * the ranking check after writing cert[h].top_blocks. */
int cqa_select_certify_local(const cqa_cache *c, const cqa_knobs *knobs, const cqa_workspace *ws, int64_t nq,
                             int64_t nact, const float *exploration_u, int64_t u_ld, void *stream);
/* FP16 re-score of the top-list blocks this rank owns: out[h][i] = (score, log-mass) for
 * cert[h].top_blocks[i] in [first_block, first_block + n_local), zeros otherwise, so a
 * sum over ranks gives every rank all scores.  `c` is the rank's local cache. */
int cqa_rescore_owned(const cqa_cache *c, const cqa_head_cert *cert, const void *q, int q_dtype,
                      int64_t first_block, int64_t n_local, float q_scale, float *out, void *stream);
/* Ranking / boundary / consistency flags from cert[h].top_blocks and ws->given_fp16. */
int cqa_certify_given(const cqa_cache *c, const cqa_knobs *knobs, const cqa_workspace *ws, const void *q,
                      int q_dtype, int64_t nq, int64_t nact, void *stream);
/* Log-sum-exp merge of n_parts partial rows per head ([n_parts][H][CQA_PARTIAL_STRIDE]) into out[H][128]. */
int cqa_merge_partials(const float *parts, int n_parts, int n_heads, float *out, void *stream);

/* ---- peer-memory exchange for the sharded step (one node, up to 8 GPUs) ----
 * Every rank allocates one buffer (cqa_peer_alloc), exports it (cqa_peer_export), the 64-byte handles are exchanged by
 * the host (e.g. torch.distributed all_gather_object) and opened (cqa_peer_import).  Ranks then PUSH their slices into
 * every peer's buffer with plain stores followed by a system-scope release of a per-(exchange, source) flag word;
 * consumers wait on their LOCAL flag words.  No rank ever loads from a peer, no collective library is involved, and
 * every wait is bounded.  Layout of a rank's buffer (floats unless noted), both parities of a step back to back:
 *   xa [2][world][rows][chunk]    Exchange A: m_b rows, S_b rows, eta rows, one row of scale maxima
 *   xb [2][world][H][32][2]       Exchange B: FP16 re-scores of the top list
 *   xc [2][world][H][130]         Exchange C: un-normalised Phase-2 partials
 *   flags int32 [3][world], flags_b int32 [world][H], status int32 [4], tickets int32 [3][world]
 */
#define CQA_MAX_PEERS 8
typedef struct cqa_peers {
    int32_t world, rank;
    int32_t rows;                /* 2H + KV + 1 */
    int32_t n_heads;
    int64_t chunk;               /* columns per row of xa */
    void *base[CQA_MAX_PEERS];   /* every rank's buffer as seen from this process (base[rank] = own) */
} cqa_peers;

int64_t cqa_peer_buffer_bytes(int world, int n_heads, int kv_heads, int64_t chunk);
int cqa_peer_alloc(int64_t bytes, void **ptr);
int cqa_peer_free(void *ptr);
int cqa_peer_export(void *ptr, unsigned char handle[64]);
int cqa_peer_import(const unsigned char handle[64], void **ptr);
int cqa_peer_close(void *ptr);
/* Wait status of this rank's buffer (0 = no bounded wait has timed out; 100 + i = the flag of source rank i did
 * not arrive in time).  Synchronises with the device; `reset` clears it. */
int cqa_peer_status(const cqa_peers *peers, int32_t *status_out, int reset);

/* One sharded layer step with peer-memory exchanges: local Phase 1, push A, global selector (waits for A),
 * owner re-scores pushed to every rank and awaited inside the same kernel (B), local Phase 2, push C, merge (waits for C).
 * `local` is the rank's cache; `global_view` the same descriptor with max_blocks = the global leading dimension
 * (its values_int4_errors and sigma_max are replaced by pointers into the exchange buffer); `wg` is the workspace
 * for the global selector (masks, certificate), `wl` the one for the local Phase 2 (mask pointers offset to the
 * rank's first block).  `step` counts calls from 1 and must be the same on every rank; `push_meta` != 0 when a
 * block completed since the previous call (eta rows and scale maxima are re-sent).  *status is set non-zero if a
 * wait timed out.  No reference counterpart. */
int cqa_sharded_layer_step(const cqa_cache *local, const cqa_cache *global_view, const cqa_knobs *knobs,
                           const cqa_workspace *wg, const cqa_workspace *wl, const cqa_peers *peers, const void *q,
                           int q_dtype, int64_t nq_global, int64_t nact_global, int64_t n_local, int64_t nact_local,
                           int64_t first_block, int64_t num_tokens_local, int last_valid, int64_t step, int push_meta,
                           float *out, void *stream);

/* ---- bounded hot tier (reference: ensure_fp16_{keys,values}_resident, _page_in_fp16_blocks,
 * _prepare_bounded_fp16_key_scratch - tiered_kv_cache.py:986-1537; backends/cuda_pagein.*) ----
 * The reference keeps an LRU on the host, reads the selection back, copies the missing blocks host-to-device and
 * only then attends.  Here the step never waits: kernels read a non-resident block straight from the backing
 * array, and cqa_hot_tier_update, queued after the step, marks the blocks the step used (FP16-key mask, FP16-value
 * mask), takes slots that were not used in this step in clock order, and copies the missed blocks into them, so
 * the next steps find them in HBM.  All bookkeeping is on the device. */
typedef struct cqa_hot_tier {
    int32_t key_capacity_blocks;   /* slots in keys_t2 */
    int32_t value_capacity_blocks; /* slots in values_t2 */
    int32_t max_fill_blocks;       /* page-in budget per call and tier (blocks) */
    int32_t reserved;
    int32_t *key_slots;          /* [max_blocks], the table cqa_cache.key_slots points at */
    int32_t *value_slots;
    int32_t *key_owner;          /* [capacity] block held by a slot, -1 = free */
    int32_t *value_owner;
    int32_t *key_stamp;          /* [capacity] step in which the slot was last used */
    int32_t *value_stamp;
    int32_t *work;               /* [2][2 + 3 * max_blocks] per tier: miss count, fill count, missed blocks, (block, slot) pairs */
    int64_t *counters;           /* [24]: step, clock hands (keys, values), then per tier: hits, misses, page-ins, evictions;
                                    1 spare; entries 12..23 repeat 0..11 as they were before the latest update call */
} cqa_hot_tier;

int cqa_hot_tier_update(const cqa_cache *c, const cqa_workspace *ws, const cqa_hot_tier *ht, int64_t nact,
                        void *stream);

/* Residency request by block id (reference: TieredKeyCacheLayer.ensure_fp16_keys_resident / _values_resident,
 * tiered_kv_cache.py:1218-1537): the `n` distinct blocks `block_ids` (device memory) of tier 0 (keys) or 1 (values) are
 * marked as used; those not resident are paged in from the backing array into slots that were not used in the
 * current step (at most max_fill_blocks per call).  Counters are updated as by cqa_hot_tier_update. */
int cqa_hot_tier_ensure(const cqa_cache *c, const cqa_hot_tier *ht, int tier, const int64_t *block_ids, int64_t n,
                        void *stream);

/* Page-in primitives under the reference's native extension (dotcache/backends/cuda_pagein.py:68-149,
 * cuda_kernels/cuda_pagein_kernel.cu): gather 16-row blocks of a backing array `src` ([KV][src_rows] rows of
 * row_bytes bytes, device memory or pinned host memory) into 16-row slots of the scratch array `dst`
 * ([KV][dst_rows] rows).  Rows at or beyond active_tokens are not copied.
 * cqa_page_in_blocks: (loaded_blocks[i] -> loaded_slots[i]) pairs, after setting slot_table[evicted] = -1 and
 * slot_table[loaded] = slot (slot_table may be NULL).  Lists are device memory.
 * cqa_page_in_by_slots: block i goes to slot block_slots[i] for every i < n_blocks with a slot >= 0. */
int cqa_page_in_blocks(const void *src, int64_t src_rows, void *dst, int64_t dst_rows, int kv_heads, int row_bytes,
                       const int64_t *loaded_blocks, const int32_t *loaded_slots, int64_t n_loaded,
                       const int64_t *evicted_blocks, int64_t n_evicted, int32_t *slot_table, int64_t table_size,
                       int64_t active_tokens, void *stream);
int cqa_page_in_by_slots(const void *src, int64_t src_rows, void *dst, int64_t dst_rows, int kv_heads, int row_bytes,
                         const int32_t *block_slots, int64_t n_blocks, int64_t active_tokens, void *stream);

/* Suggested split counts for a context of `nact` blocks on the current device. */
int cqa_suggest_splits(int kv_heads, int gqa_group, int64_t nact, int *num_splits, int *dense_splits);

#ifdef __cplusplus
}
#endif
#endif /* CQA_B200_H */
