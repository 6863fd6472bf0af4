// C ABI glue: error text, argument checks, the fused per-layer chain.
#include <atomic>
#include <cstdarg>
#include <cstdio>

#include "common.cuh"

namespace cqa {

static thread_local char g_err[512] = "";

void set_error(const char *fmt, ...)
{
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof g_err, fmt, ap);
    va_end(ap);
}

int check_cuda(cudaError_t e, const char *what)
{
    if (e == cudaSuccess) return CQA_OK;
    set_error("%s: %s", what, cudaGetErrorString(e));
    return CQA_ERR_CUDA;
}

int check_launch(const char *what) { return check_cuda(cudaGetLastError(), what); }

static std::atomic<long long> g_launches{0};
void note_launch(int n) { g_launches.fetch_add(n, std::memory_order_relaxed); }

int score_blocks_launch(const cqa_cache *c, const void *q, int q_dtype, long nq, float q_scale, float *m_b,
                        float *s_b, long ld, float *tok, cudaStream_t st, int32_t *zero_words, int n_zero_words,
                        const ScorePush *push);
int select_launch(const cqa_cache *c, const cqa_knobs *kn, const cqa_workspace *ws, long nq, long nact,
                  const float *u, long u_ld, cudaStream_t st);
int certify_launch(const cqa_cache *c, const cqa_knobs *kn, const cqa_workspace *ws, const void *q, int q_dtype,
                   long nq, long nact, cudaStream_t st);
int select_certify_local_launch(const cqa_cache *c, const cqa_knobs *kn, const cqa_workspace *ws, long nq,
                                long nact, const float *u, long u_ld, cudaStream_t st);
int certify_given_launch(const cqa_cache *c, const cqa_knobs *kn, const cqa_workspace *ws, const void *q,
                         int q_dtype, long nq, long nact, cudaStream_t st);
int rescore_owned_launch(const cqa_cache *c, const cqa_head_cert *cert, const void *q, int q_dtype, long first_block,
                         long n_local, float q_scale, float *out, cudaStream_t st);
int merge_partials_launch(const float *parts, int n_parts, int n_heads, float *out, cudaStream_t st);
int selcert_launch(const cqa_cache *c, const cqa_knobs *kn, const cqa_workspace *ws, const void *q, int q_dtype,
                   long nq, long nact, const float *u, long u_ld, int phases, cudaStream_t st);
int attend_launch(const cqa_cache *c, const cqa_workspace *ws, const void *q, int q_dtype, long nq, long nact,
                  long num_tokens, int last_valid, float q_scale, cudaStream_t st, bool chained);

int dense_launch(const cqa_cache *c, const cqa_workspace *ws, const void *q, int q_dtype, long num_tokens, float q_scale,
                 cudaStream_t st);
int score_blocks_batched_launch(const cqa_batch_item *items_dev, int n_items, int kv_heads, int gqa_group, long max_nq,
                                int q_dtype, float q_scale, int do_append, cudaStream_t st);
int selcert_batched_launch(const cqa_batch_item *items_dev, int n_items, int n_heads, long max_nq, const cqa_knobs *kn,
                           int q_dtype, int do_append, cudaStream_t st);
int attend_batched_launch(const cqa_batch_item *items_dev, int n_items, int kv_heads, int gqa_group, int t2_dtype,
                          int max_splits, int q_dtype, float q_scale, int do_append, cudaStream_t st);
int append_batched_launch(const cqa_batch_item *items_dev, int n_items, int kv_heads, int t2_dtype, int src_dtype, cudaStream_t st);
int attend_static_launch(const cqa_cache *c, const cqa_workspace *ws, const void *q, int q_dtype, long nq, long nact,
                         long num_tokens, int last_valid, float q_scale, cudaStream_t st);

static int check_common(const cqa_cache *c, const cqa_workspace *ws, const char *who)
{
    if (!c || !ws) { set_error("%s: NULL cache or workspace", who); return CQA_ERR_INVALID; }
    if (c->kv_heads <= 0 || (c->gqa_group != 1 && c->gqa_group != 2 && c->gqa_group != 4 && c->gqa_group != 8)) {
        set_error("%s: unsupported head layout kv=%d group=%d", who, c->kv_heads, c->gqa_group);
        return CQA_ERR_UNSUPPORTED;
    }
    if (c->t2_dtype < 0 || c->t2_dtype > 2) { set_error("%s: unknown Tier-2 dtype %d", who, c->t2_dtype); return CQA_ERR_INVALID; }
    if (ws->ld <= 0) { set_error("%s: workspace ld must be positive", who); return CQA_ERR_INVALID; }
    return CQA_OK;
}

static int check_select_ws(const cqa_workspace *ws, const char *who)
{
    if (!ws->m_b || !ws->s_b || !ws->mass_frac || !ws->topk_mask || !ws->explore_mask || !ws->sorted_idx ||
        !ws->sorted_cumsum || !ws->cert || !ws->any_flags) {
        set_error("%s: workspace is missing selector buffers", who);
        return CQA_ERR_INVALID;
    }
    return CQA_OK;
}

}  // namespace cqa

using namespace cqa;

extern "C" const char *cqa_version(void) { return "cqa_b200 0.1 (sm_100a)"; }
extern "C" const char *cqa_last_error(void) { return g_err; }
extern "C" int cqa_wait_timeouts(int *count, int reset)
{
    if (!count) { set_error("cqa_wait_timeouts: NULL pointer"); return CQA_ERR_INVALID; }
    int a = 0, b = 0;
    if (score_wait_timeouts(&a, reset) || selcert_wait_timeouts(&b, reset)) {
        set_error("cqa_wait_timeouts: could not read the device counters: %s", cudaGetErrorString(cudaGetLastError()));
        return CQA_ERR_CUDA;
    }
    *count = a + b;
    return CQA_OK;
}

extern "C" int64_t cqa_launch_count(int reset)
{
    return reset ? g_launches.exchange(0, std::memory_order_relaxed) : g_launches.load(std::memory_order_relaxed);
}

extern "C" int cqa_select(const cqa_cache *c, const cqa_knobs *knobs, const cqa_workspace *ws, int64_t nq,
                          int64_t nact, const float *exploration_u, int64_t u_ld, void *stream)
{
    int rc = check_common(c, ws, "cqa_select");
    if (rc) return rc;
    if (!knobs) { set_error("cqa_select: NULL knobs"); return CQA_ERR_INVALID; }
    rc = check_select_ws(ws, "cqa_select");
    if (rc) return rc;
    if (nact < nq || nact > nq + 1 || nact > ws->ld) {
        set_error("cqa_select: nact=%ld inconsistent with nq=%ld (ld=%ld)", (long)nact, (long)nq, (long)ws->ld);
        return CQA_ERR_INVALID;
    }
    if (!(knobs->tau_cov > 0.0f)) { set_error("cqa_select: tau_cov must be positive"); return CQA_ERR_INVALID; }
    if (exploration_u && u_ld < nq) { set_error("cqa_select: exploration_u leading dimension too small"); return CQA_ERR_INVALID; }
    return select_launch(c, knobs, ws, nq, nact, exploration_u, u_ld, (cudaStream_t)stream);
}

extern "C" int cqa_certify(const cqa_cache *c, const cqa_knobs *knobs, const cqa_workspace *ws, const void *q,
                           int q_dtype, int64_t nq, int64_t nact, void *stream)
{
    int rc = check_common(c, ws, "cqa_certify");
    if (rc) return rc;
    if (!knobs || !q) { set_error("cqa_certify: NULL knobs or q"); return CQA_ERR_INVALID; }
    rc = check_select_ws(ws, "cqa_certify");
    if (rc) return rc;
    if (!ws->value_mask) { set_error("cqa_certify: value_mask missing"); return CQA_ERR_INVALID; }
    if (nact < nq || nact > nq + 1 || nact > ws->ld) { set_error("cqa_certify: bad nact"); return CQA_ERR_INVALID; }
    return certify_launch(c, knobs, ws, q, q_dtype, nq, nact, (cudaStream_t)stream);
}

static int decode_step_host(const cqa_cache *c, const cqa_knobs *knobs, const cqa_workspace *ws, const void *qkv_host,
                            void *qkv_dev, int dtype, int64_t pos, int defer_int4, float *out_host, void *stream,
                            bool wait)
{
    if (!c || !knobs || !ws || !qkv_host || !qkv_dev || !out_host) {
        set_error("cqa_decode_step_host: NULL pointer");
        return CQA_ERR_INVALID;
    }
    if (dtype < 0 || dtype > 2) { set_error("cqa_decode_step_host: unknown dtype"); return CQA_ERR_INVALID; }
    if (!ws->out) { set_error("cqa_decode_step_host: workspace has no output rows"); return CQA_ERR_INVALID; }
    const size_t esz = dtype == CQA_F32 ? 4 : 2;
    const size_t H = (size_t)c->kv_heads * c->gqa_group, KV = (size_t)c->kv_heads;
    const size_t n_in = (H + 2 * KV) * D;
    cudaStream_t st = (cudaStream_t)stream;
    int rc = check_cuda(cudaMemcpyAsync(qkv_dev, qkv_host, n_in * esz, cudaMemcpyHostToDevice, st), "copy of step inputs");
    if (rc) return rc;
    char *dev = static_cast<char *>(qkv_dev);
    const void *q = dev, *k_new = dev + H * D * esz, *v_new = dev + (H + KV) * D * esz;
    rc = cqa_append_token(c, k_new, v_new, dtype, pos, defer_int4, stream);
    if (rc) return rc;
    const int64_t num_tokens = pos + 1;
    // Phase 2 writes its rows straight into the caller's buffer when it is pinned memory the device can address
    cqa_workspace w = *ws;
    void *mapped = nullptr;
    if (cudaHostGetDevicePointer(&mapped, out_host, 0) == cudaSuccess && mapped != nullptr)
        w.out = static_cast<float *>(mapped);
    else
        (void)cudaGetLastError();
    rc = cqa_layer_step(c, knobs, &w, q, dtype, num_tokens, num_tokens / BS, nullptr, 0, stream);
    if (rc) return rc;
    if (w.out == ws->out)
        rc = check_cuda(cudaMemcpyAsync(out_host, ws->out, H * D * sizeof(float), cudaMemcpyDeviceToHost, st), "copy of the output");
    if (rc || !wait) return rc;
    return check_cuda(cudaStreamSynchronize(st), "cudaStreamSynchronize");
}

extern "C" int cqa_decode_step_host(const cqa_cache *c, const cqa_knobs *knobs, const cqa_workspace *ws,
                                    const void *qkv_host, void *qkv_dev, int dtype, int64_t pos, int defer_int4,
                                    float *out_host, void *stream)
{
    return decode_step_host(c, knobs, ws, qkv_host, qkv_dev, dtype, pos, defer_int4, out_host, stream, true);
}

extern "C" int cqa_decode_step_host_async(const cqa_cache *c, const cqa_knobs *knobs, const cqa_workspace *ws,
                                          const void *qkv_host, void *qkv_dev, int dtype, int64_t pos, int defer_int4,
                                          float *out_host, void *stream)
{
    return decode_step_host(c, knobs, ws, qkv_host, qkv_dev, dtype, pos, defer_int4, out_host, stream, false);
}

extern "C" int cqa_decode_token_host(const cqa_layer_call *layers, int n_layers, const cqa_knobs *knobs, void *qkv_dev,
                                     int dtype, void *stream)
{
    if (!layers || n_layers <= 0 || !knobs || !qkv_dev) {
        set_error("cqa_decode_token_host: no layers, knobs or staging buffer");
        return CQA_ERR_INVALID;
    }
    if (dtype < 0 || dtype > 2) { set_error("cqa_decode_token_host: unknown dtype"); return CQA_ERR_INVALID; }
    for (int l = 0; l < n_layers; ++l) {
        const cqa_layer_call &c = layers[l];
        if (!c.cache || !c.ws || !c.qkv_host || !c.out_host || !c.ws->out) {
            set_error("cqa_decode_token_host: layer %d has a NULL pointer", l);
            return CQA_ERR_INVALID;
        }
        if (c.cache->kv_heads != layers[0].cache->kv_heads || c.cache->gqa_group != layers[0].cache->gqa_group) {
            set_error("cqa_decode_token_host: layer %d has another head geometry than layer 0", l);
            return CQA_ERR_INVALID;
        }
    }
    const size_t esz = dtype == CQA_F32 ? 4 : 2;
    const size_t H = (size_t)layers[0].cache->kv_heads * layers[0].cache->gqa_group, KV = (size_t)layers[0].cache->kv_heads;
    const size_t row = (H + 2 * KV) * D * esz;
    cudaStream_t st = (cudaStream_t)stream;
    char *dev = static_cast<char *>(qkv_dev);
    // every layer's inputs first (host rows that follow one another go in one transfer), so that no transfer
    // sits between two layers' kernels
    for (int l = 0; l < n_layers;) {
        int r = l + 1;
        while (r < n_layers &&
               static_cast<const char *>(layers[r].qkv_host) == static_cast<const char *>(layers[l].qkv_host) + (size_t)(r - l) * row)
            ++r;
        const int rc = check_cuda(cudaMemcpyAsync(dev + (size_t)l * row, layers[l].qkv_host, (size_t)(r - l) * row,
                                                  cudaMemcpyHostToDevice, st), "copy of step inputs");
        if (rc) return rc;
        l = r;
    }
    for (int l = 0; l < n_layers; ++l) {
        const cqa_layer_call &c = layers[l];
        // Phase 2 writes its rows straight into the caller's pinned buffer when the driver maps it for the device
        cqa_workspace w = *c.ws;
        void *mapped = nullptr;
        if (cudaHostGetDevicePointer(&mapped, c.out_host, 0) == cudaSuccess && mapped != nullptr)
            w.out = static_cast<float *>(mapped);
        else
            (void)cudaGetLastError();
        const char *in = dev + (size_t)l * row;
        int rc = cqa_append_token(c.cache, in + H * D * esz, in + (H + KV) * D * esz, dtype, c.pos, c.defer_int4, stream);
        if (rc) return rc;
        const int64_t num_tokens = c.pos + 1;
        rc = cqa_layer_step(c.cache, knobs, &w, in, dtype, num_tokens, num_tokens / BS, nullptr, 0, stream);
        if (rc) return rc;
        if (w.out == c.ws->out) {
            rc = check_cuda(cudaMemcpyAsync(c.out_host, c.ws->out, H * D * sizeof(float), cudaMemcpyDeviceToHost, st),
                            "copy of the output");
            if (rc) return rc;
        }
    }
    return check_cuda(cudaStreamSynchronize(st), "cudaStreamSynchronize");
}

extern "C" int cqa_select_certify_local(const cqa_cache *c, const cqa_knobs *knobs, const cqa_workspace *ws, int64_t nq,
                                        int64_t nact, const float *exploration_u, int64_t u_ld, void *stream)
{
    int rc = check_common(c, ws, "cqa_select_certify_local");
    if (rc) return rc;
    if (!knobs) { set_error("cqa_select_certify_local: NULL knobs"); return CQA_ERR_INVALID; }
    rc = check_select_ws(ws, "cqa_select_certify_local");
    if (rc) return rc;
    if (!ws->value_mask) { set_error("cqa_select_certify_local: value_mask missing"); return CQA_ERR_INVALID; }
    if (nact < nq || nact > nq + 1 || nact > ws->ld) {
        set_error("cqa_select_certify_local: nact=%ld inconsistent with nq=%ld (ld=%ld)", (long)nact, (long)nq, (long)ws->ld);
        return CQA_ERR_INVALID;
    }
    if (!(knobs->tau_cov > 0.0f)) { set_error("cqa_select_certify_local: tau_cov must be positive"); return CQA_ERR_INVALID; }
    if (exploration_u && u_ld < nq) { set_error("cqa_select_certify_local: exploration_u leading dimension too small"); return CQA_ERR_INVALID; }
    return select_certify_local_launch(c, knobs, ws, nq, nact, exploration_u, u_ld, (cudaStream_t)stream);
}

extern "C" int cqa_rescore_owned(const cqa_cache *c, const cqa_head_cert *cert, const void *q, int q_dtype,
                                 int64_t first_block, int64_t n_local, float q_scale, float *out, void *stream)
{
    if (!c || !cert || !q || !out || !c->keys_t2) { set_error("cqa_rescore_owned: NULL pointer"); return CQA_ERR_INVALID; }
    if (first_block < 0 || n_local < 0 || n_local > c->max_blocks) {
        set_error("cqa_rescore_owned: block range [%ld, +%ld) does not fit the local cache", (long)first_block, (long)n_local);
        return CQA_ERR_INVALID;
    }
    if (q_dtype < 0 || q_dtype > 2) { set_error("cqa_rescore_owned: unknown q dtype"); return CQA_ERR_INVALID; }
    return rescore_owned_launch(c, cert, q, q_dtype, first_block, n_local, q_scale, out, (cudaStream_t)stream);
}

extern "C" int cqa_certify_given(const cqa_cache *c, const cqa_knobs *knobs, const cqa_workspace *ws, const void *q,
                                 int q_dtype, int64_t nq, int64_t nact, void *stream)
{
    int rc = check_common(c, ws, "cqa_certify_given");
    if (rc) return rc;
    if (!knobs || !q) { set_error("cqa_certify_given: NULL knobs or q"); return CQA_ERR_INVALID; }
    rc = check_select_ws(ws, "cqa_certify_given");
    if (rc) return rc;
    if (nact < nq || nact > nq + 1 || nact > ws->ld) { set_error("cqa_certify_given: bad nact"); return CQA_ERR_INVALID; }
    return certify_given_launch(c, knobs, ws, q, q_dtype, nq, nact, (cudaStream_t)stream);
}

extern "C" int cqa_merge_partials(const float *parts, int n_parts, int n_heads, float *out, void *stream)
{
    if (!parts || !out || n_parts <= 0 || n_heads <= 0) { set_error("cqa_merge_partials: bad arguments"); return CQA_ERR_INVALID; }
    return merge_partials_launch(parts, n_parts, n_heads, out, (cudaStream_t)stream);
}

extern "C" int cqa_attend(const cqa_cache *c, const cqa_workspace *ws, const void *q, int q_dtype, int64_t nq,
                          int64_t nact, int64_t num_tokens, int last_block_valid, float q_scale, void *stream)
{
    int rc = check_common(c, ws, "cqa_attend");
    if (rc) return rc;
    if (!q) { set_error("cqa_attend: NULL q"); return CQA_ERR_INVALID; }
    return attend_launch(c, ws, q, q_dtype, nq, nact, num_tokens, last_block_valid, q_scale, (cudaStream_t)stream, false);
}

extern "C" int cqa_dense_attend(const cqa_cache *c, const cqa_workspace *ws, const void *q, int q_dtype,
                                int64_t num_tokens, float q_scale, void *stream)
{
    int rc = check_common(c, ws, "cqa_dense_attend");
    if (rc) return rc;
    if (!q) { set_error("cqa_dense_attend: NULL q"); return CQA_ERR_INVALID; }
    return dense_launch(c, ws, q, q_dtype, num_tokens, q_scale, (cudaStream_t)stream);
}

extern "C" int cqa_attend_static(const cqa_cache *c, const cqa_workspace *ws, const void *q, int q_dtype, int64_t nq,
                                 int64_t nact, int64_t num_tokens, int last_block_valid, float q_scale, void *stream)
{
    int rc = check_common(c, ws, "cqa_attend_static");
    if (rc) return rc;
    if (!q) { set_error("cqa_attend_static: NULL q"); return CQA_ERR_INVALID; }
    return attend_static_launch(c, ws, q, q_dtype, nq, nact, num_tokens, last_block_valid, q_scale,
                                (cudaStream_t)stream);
}

extern "C" int cqa_layer_step(const cqa_cache *c, const cqa_knobs *knobs, const cqa_workspace *ws, const void *q,
                              int q_dtype, int64_t num_tokens, int64_t nq, const float *exploration_u,
                              int64_t u_ld, void *stream)
{
    // every argument check comes before the first launch: a bad call must not write anything on the device
    int rc = check_common(c, ws, "cqa_layer_step");
    if (rc) return rc;
    if (!knobs || !q) { set_error("cqa_layer_step: NULL knobs or q"); return CQA_ERR_INVALID; }
    rc = check_select_ws(ws, "cqa_layer_step");
    if (rc) return rc;
    if (nq <= 0 || num_tokens < nq * BS || num_tokens >= (nq + 1) * BS) {
        set_error("cqa_layer_step: num_tokens=%ld does not match %ld quantised blocks", (long)num_tokens, (long)nq);
        return CQA_ERR_INVALID;
    }
    rc = check_score_args(c, q_dtype, nq, ws->ld, "cqa_layer_step");
    if (rc) return rc;
    const long nact = (num_tokens + BS - 1) / BS;
    const int last_valid = nact == nq ? BS : (int)(num_tokens - nq * BS);
    cudaStream_t st = (cudaStream_t)stream;
    if (!ws->token_scores) { set_error("cqa_layer_step: token_scores missing"); return CQA_ERR_INVALID; }
    if (!(knobs->tau_cov > 0.0f)) { set_error("cqa_layer_step: tau_cov must be positive"); return CQA_ERR_INVALID; }
    if (!ws->value_mask) { set_error("cqa_layer_step: value_mask missing"); return CQA_ERR_INVALID; }
    if (nact > ws->ld || nact > c->max_blocks) { set_error("cqa_layer_step: workspace ld or cache max_blocks too small"); return CQA_ERR_INVALID; }
    if (exploration_u && u_ld < nq) { set_error("cqa_layer_step: exploration_u leading dimension too small"); return CQA_ERR_INVALID; }
    rc = selcert_check(c, knobs, ws, q, nq, 3 | 16);
    if (rc) return rc;
    rc = attend_check(c, ws, nq, nact, last_valid);
    if (rc) return rc;
    const int n_flag_words = 5 + c->kv_heads * c->gqa_group;
    rc = score_blocks_launch(c, q, q_dtype, nq, knobs->q_scale, ws->m_b, ws->s_b, ws->ld, ws->token_scores, st,
                             ws->any_flags, n_flag_words, nullptr);
    if (rc) return rc;
    rc = selcert_launch(c, knobs, ws, q, q_dtype, nq, nact, exploration_u, u_ld, 3 | 16, st);   // select + certify in one launch; flags cleared by the score kernel
    if (rc) return rc;
    return attend_launch(c, ws, q, q_dtype, nq, nact, num_tokens, last_valid, knobs->q_scale, st, true);
}

extern "C" int cqa_layer_step_batched(const cqa_batch_item *items, int n_items, void *items_dev, const cqa_knobs *knobs,
                                      int dtype, int do_append, void *stream)
{
    if (!items || !items_dev || !knobs || n_items <= 0 || n_items > 65535) {
        set_error("cqa_layer_step_batched: NULL pointer or item count %d out of range (1..65535)", n_items);
        return CQA_ERR_INVALID;
    }
    if (dtype < 0 || dtype > 2) { set_error("cqa_layer_step_batched: unknown dtype %d", dtype); return CQA_ERR_INVALID; }
    if ((uintptr_t)items_dev & 15) { set_error("cqa_layer_step_batched: items_dev must be 16-byte aligned"); return CQA_ERR_INVALID; }
    if (!(knobs->tau_cov > 0.0f)) { set_error("cqa_layer_step_batched: tau_cov must be positive"); return CQA_ERR_INVALID; }
    do_append = do_append ? 1 : 0;
    const cqa_cache &c0 = items[0].cache;
    long max_nq = 0;
    int max_splits = 0;
    // every check of every sequence comes before the first copy or launch
    for (int i = 0; i < n_items; ++i) {
        const cqa_batch_item &it = items[i];
        int rc = check_common(&it.cache, &it.ws, "cqa_layer_step_batched");
        if (rc) return rc;
        if (it.cache.kv_heads != c0.kv_heads || it.cache.gqa_group != c0.gqa_group || it.cache.t2_dtype != c0.t2_dtype) {
            set_error("cqa_layer_step_batched: item %d differs from item 0 in head geometry or Tier-2 dtype", i);
            return CQA_ERR_INVALID;
        }
        rc = check_select_ws(&it.ws, "cqa_layer_step_batched");
        if (rc) return rc;
        if (!it.q || !it.ws.token_scores || !it.ws.value_mask) {
            set_error("cqa_layer_step_batched: item %d has no q, token_scores or value_mask", i);
            return CQA_ERR_INVALID;
        }
        if (do_append) {
            rc = append_check(&it.cache, it.k_new, it.v_new, dtype, it.pos);
            if (rc) return rc;
        }
        const long num_tokens = it.pos + do_append;
        const long nq = num_tokens / BS, nact = (num_tokens + BS - 1) / BS;
        if (it.pos < 0 || nq <= 0) {
            set_error("cqa_layer_step_batched: item %d holds %ld tokens; at least one complete block is needed", i, num_tokens);
            return CQA_ERR_INVALID;
        }
        rc = check_score_args(&it.cache, dtype, nq, it.ws.ld, "cqa_layer_step_batched");
        if (rc) return rc;
        if (nact > it.ws.ld || nact > it.cache.max_blocks) {
            set_error("cqa_layer_step_batched: item %d: workspace ld or cache max_blocks too small", i);
            return CQA_ERR_INVALID;
        }
        rc = selcert_check(&it.cache, knobs, &it.ws, it.q, nq, 3 | 16);
        if (rc) return rc;
        rc = attend_check(&it.cache, &it.ws, nq, nact, nact == nq ? BS : (int)(num_tokens - nq * BS));
        if (rc) return rc;
        if (!it.ws.out) { set_error("cqa_layer_step_batched: item %d has no output rows", i); return CQA_ERR_INVALID; }
        if (nq > max_nq) max_nq = nq;
        if (it.ws.num_splits > max_splits) max_splits = it.ws.num_splits;
    }
    cudaStream_t st = (cudaStream_t)stream;
    const cqa_batch_item *dev = static_cast<const cqa_batch_item *>(items_dev);
    int rc = check_cuda(cudaMemcpyAsync(items_dev, items, (size_t)n_items * sizeof(cqa_batch_item), cudaMemcpyHostToDevice, st),
                        "copy of the batch records");
    if (rc) return rc;
    if (do_append) {
        rc = append_batched_launch(dev, n_items, c0.kv_heads, c0.t2_dtype, dtype, st);
        if (rc) return rc;
    }
    rc = score_blocks_batched_launch(dev, n_items, c0.kv_heads, c0.gqa_group, max_nq, dtype, knobs->q_scale, do_append, st);
    if (rc) return rc;
    rc = selcert_batched_launch(dev, n_items, c0.kv_heads * c0.gqa_group, max_nq, knobs, dtype, do_append, st);
    if (rc) return rc;
    return attend_batched_launch(dev, n_items, c0.kv_heads, c0.gqa_group, c0.t2_dtype, max_splits, dtype, knobs->q_scale,
                                 do_append, st);
}

extern "C" int cqa_suggest_splits(int kv_heads, int gqa_group, int64_t nact, int *num_splits, int *dense_splits)
{
    if (kv_heads <= 0 || gqa_group <= 0 || !num_splits || !dense_splits) {
        set_error("cqa_suggest_splits: bad arguments");
        return CQA_ERR_INVALID;
    }
    int dev = 0, sms = 148;
    if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    if (sms <= 0) sms = 148;
    // Phase 2: two resident CTAs per SM, at least 8 blocks (one per warp) per split.
    long target = ((long)sms * CQA_ATT_MIN_CTAS) / kv_heads;
    if (target < 1) target = 1;
    long by_work = (nact + 7) / 8;
    long ns = target < by_work ? target : by_work;
    if (ns > CQA_MAX_SPLITS) ns = CQA_MAX_SPLITS;
    if (ns < 1) ns = 1;
    *num_splits = (int)ns;
    // dense recompute: chunks of about 16 blocks per (flagged head), at most CQA_MAX_DENSE_SPLITS
    long ds = (nact + 15) / 16;
    if (ds > CQA_MAX_DENSE_SPLITS) ds = CQA_MAX_DENSE_SPLITS;
    if (ds < 1) ds = 1;
    *dense_splits = (int)ds;
    return CQA_OK;
}
