// Peer-memory exchanges of the sequence-sharded step (one node, NVLink peers).
//
// Every rank owns one buffer; all ranks map all buffers.  A rank PUSHES its slice of an exchange into every peer's
// buffer with plain stores, then the last CTA of the push makes the stores visible system-wide and releases a flag
// word in the peer's buffer.  Consumers only ever read their own buffer, after waiting (bounded) on their own flag
// words.  Nothing loads from a peer, nothing multicasts, no kernel waits on a kernel of its own GPU.
//
// Buffer layout (all ranks identical; two parities so that step s+1 never overwrites what a slower rank still reads
// from step s):
//   xa [2][world][rows][chunk] f32 | xb [2][world][H][32][2] f32 | xc [2][world][H][130] f32 |
//   flags [3][world] i32 | flags_b [world][H] i32 | status [4] i32 | tickets [3][world] i32
#include <cstring>

#include "common.cuh"
#include "rescore.cuh"

namespace cqa {

int score_blocks_launch(const cqa_cache *c, const void *q, int q_dtype, long nq, float q_scale, float *m_b,
                        float *s_b, long ld, float *tok, cudaStream_t st, int32_t *zero_words, int n_zero_words,
                        const ScorePush *push);
int selcert_launch(const cqa_cache *c, const cqa_knobs *kn, const cqa_workspace *ws, const void *q, int q_dtype,
                   long nq, long nact, const float *u, long u_ld, int phases, cudaStream_t st);
int attend_launch(const cqa_cache *c, const cqa_workspace *ws, const void *q, int q_dtype, long nq, long nact,
                  long num_tokens, int last_valid, float q_scale, cudaStream_t st, bool chained);

struct PeerLayout {
    long xa_parity, xb_parity, xc_parity;      // floats per parity
    long xa, xb, xc, flags, flags_b, status, tickets;   // offsets in 4-byte words
    long words;
    int world, rows, H;
    long chunk;
};

__host__ __device__ inline PeerLayout peer_layout(int world, int H, int rows, long chunk)
{
    PeerLayout L;
    L.world = world; L.rows = rows; L.H = H; L.chunk = chunk;
    L.xa_parity = (long)world * rows * chunk;
    L.xb_parity = (long)world * H * CQA_MAX_RANKING_K * 2;
    L.xc_parity = (long)world * H * CQA_PARTIAL_STRIDE;
    L.xa = 0;
    L.xb = L.xa + 2 * L.xa_parity;
    L.xc = L.xb + 2 * L.xb_parity;
    L.flags = L.xc + 2 * L.xc_parity;
    L.flags_b = L.flags + 3 * world;          // [source rank][head]: Exchange B is per head
    L.status = L.flags_b + (long)world * H;
    L.tickets = L.status + 4;
    L.words = L.tickets + 3 * world;
    return L;
}

struct PeerArgs {
    float *base[CQA_MAX_PEERS];
    int world, rank;
};

// Copy `n_rows` rows (row r has cols(r) floats, at src + r*src_ld) into every peer's buffer at dst_off + r*dst_ld,
// then release flag word `flag_word` (value `step`) on that peer.  Grid (world, PUSH_CTAS): blockIdx.x = peer.
constexpr int PUSH_CTAS = 16, PUSH_THREADS = 256;
__device__ __forceinline__ void push_row(const float *src, float *dst, long cols)
{
    if (((reinterpret_cast<uintptr_t>(src) | reinterpret_cast<uintptr_t>(dst)) & 15) == 0) {
        const float4 *s4 = reinterpret_cast<const float4 *>(src);
        float4 *d4 = reinterpret_cast<float4 *>(dst);
        const long n4 = cols / 4;
        for (long i = threadIdx.x; i < n4; i += PUSH_THREADS) d4[i] = s4[i];
        for (long i = n4 * 4 + threadIdx.x; i < cols; i += PUSH_THREADS) dst[i] = src[i];
    } else {
        for (long i = threadIdx.x; i < cols; i += PUSH_THREADS) dst[i] = src[i];
    }
}
// Rows r >= alt_first_row are written a second time at dst_off_alt (the other parity's copy of slowly changing rows).
__global__ void __launch_bounds__(PUSH_THREADS) peer_push_kernel(PeerArgs pa, const float *src, long src_ld, long dst_off,
                                                                long dst_ld, int n_rows, int rows_a, long cols_a,
                                                                long cols_b, long cols_last, long flag_word,
                                                                long ticket_word, int step, long dst_off_alt,
                                                                int alt_first_row)
{
    const int peer = blockIdx.x;
    if (peer == pa.rank) return;
    float *dst = pa.base[peer] + dst_off;
    // rows [0, rows_a) carry cols_a floats, the last row cols_last, the rows between cols_b
    for (int r = blockIdx.y; r < n_rows; r += PUSH_CTAS) {
        const long cols = r < rows_a ? cols_a : (r == n_rows - 1 ? cols_last : cols_b);
        push_row(src + (long)r * src_ld, dst + (long)r * dst_ld, cols);
        if (dst_off_alt >= 0 && r >= alt_first_row)
            push_row(src + (long)r * src_ld, pa.base[peer] + dst_off_alt + (long)r * dst_ld, cols);
    }
    // One thread per CTA fences after the CTA barrier (the barrier orders the other threads' stores before it); the
    // last CTA for this peer then releases the flag, so everything above is visible there before the flag is.
    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence_system();
        int32_t *tick = reinterpret_cast<int32_t *>(pa.base[pa.rank]) + ticket_word + peer;
        const int t = atomicAdd(tick, 1);
        if (t == PUSH_CTAS - 1) {
            *tick = 0;
            __threadfence_system();   // acquire side of the ticket chain: the other CTAs' fenced stores come first
            st_release_sys(reinterpret_cast<int32_t *>(pa.base[peer]) + flag_word, step);
        }
    }
}

// Exchange C consumer: wait for every rank's partial rows, then the log-sum-exp merge (one CTA per head).
__global__ void __launch_bounds__(D) merge_wait_kernel(const float *parts, int n_parts, int n_heads, float *out,
                                                      const int32_t *flags, int skip, int value, int32_t *status,
                                                      int spins)
{
    grid_dependency_wait();   // this rank's own rows come from the attend kernel before it on the stream
    peer_wait(flags, n_parts, skip, value, status, 1, spins);
    const int h = blockIdx.x, ch = threadIdx.x;
    float M = -INFINITY;
    for (int p = 0; p < n_parts; ++p) M = fmaxf(M, __ldcg(parts + ((long)p * n_heads + h) * CQA_PARTIAL_STRIDE));
    float l = 0.0f, a = 0.0f;
    for (int p = 0; p < n_parts; ++p) {
        const float *row = parts + ((long)p * n_heads + h) * CQA_PARTIAL_STRIDE;
        const float m = __ldcg(row);
        const float sc = m == -INFINITY ? 0.0f : __expf(m - M);
        l = fmaf(__ldcg(row + 1), sc, l);
        a = fmaf(__ldcg(row + 2 + ch), sc, a);
    }
    out[(long)h * D + ch] = a / (l > 0.0f ? l : 1.0f);
}

}  // namespace cqa

using namespace cqa;

extern "C" int64_t cqa_peer_buffer_bytes(int world, int n_heads, int kv_heads, int64_t chunk)
{
    if (world < 1 || world > CQA_MAX_PEERS || n_heads <= 0 || kv_heads <= 0 || chunk <= 0) return -1;
    const PeerLayout L = peer_layout(world, n_heads, 2 * n_heads + kv_heads + 1, chunk);
    return (L.words * 4 + 255) / 256 * 256;
}

extern "C" int cqa_peer_alloc(int64_t bytes, void **ptr)
{
    if (!ptr || bytes <= 0) { set_error("cqa_peer_alloc: bad arguments"); return CQA_ERR_INVALID; }
    int rc = check_cuda(cudaMalloc(ptr, (size_t)bytes), "cudaMalloc(peer buffer)");
    if (rc) return rc;
    return check_cuda(cudaMemset(*ptr, 0, (size_t)bytes), "cudaMemset(peer buffer)");
}

extern "C" int cqa_peer_free(void *ptr) { return check_cuda(cudaFree(ptr), "cudaFree(peer buffer)"); }

extern "C" int cqa_peer_export(void *ptr, unsigned char handle[64])
{
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
    if (!ptr || !handle) { set_error("cqa_peer_export: NULL pointer"); return CQA_ERR_INVALID; }
    cudaIpcMemHandle_t h;
    int rc = check_cuda(cudaIpcGetMemHandle(&h, ptr), "cudaIpcGetMemHandle");
    if (rc) return rc;
    memcpy(handle, &h, 64);
    return CQA_OK;
}

extern "C" int cqa_peer_import(const unsigned char handle[64], void **ptr)
{
    if (!ptr || !handle) { set_error("cqa_peer_import: NULL pointer"); return CQA_ERR_INVALID; }
    cudaIpcMemHandle_t h;
    memcpy(&h, handle, 64);
    return check_cuda(cudaIpcOpenMemHandle(ptr, h, cudaIpcMemLazyEnablePeerAccess), "cudaIpcOpenMemHandle");
}

extern "C" int cqa_peer_close(void *ptr) { return check_cuda(cudaIpcCloseMemHandle(ptr), "cudaIpcCloseMemHandle"); }

extern "C" int cqa_peer_status(const cqa_peers *peers, int32_t *status_out, int reset)
{
    if (!peers || !status_out || peers->world < 1 || peers->rank < 0 || peers->rank >= peers->world ||
        !peers->base[peers->rank]) {
        set_error("cqa_peer_status: bad arguments");
        return CQA_ERR_INVALID;
    }
    const PeerLayout L = peer_layout(peers->world, peers->n_heads, peers->rows, peers->chunk);
    int32_t *st = reinterpret_cast<int32_t *>(peers->base[peers->rank]) + L.status;
    int rc = check_cuda(cudaMemcpy(status_out, st, sizeof(int32_t), cudaMemcpyDeviceToHost), "read of the wait status");
    if (rc) return rc;
    if (reset) rc = check_cuda(cudaMemset(st, 0, sizeof(int32_t)), "reset of the wait status");
    return rc;
}

extern "C" int cqa_sharded_layer_step(const cqa_cache *local, const cqa_cache *global_view, const cqa_knobs *knobs,
                                      const cqa_workspace *wg, const cqa_workspace *wl, const cqa_peers *peers,
                                      const void *q, int q_dtype, int64_t nq_global, int64_t nact_global,
                                      int64_t n_local, int64_t nact_local, int64_t first_block,
                                      int64_t num_tokens_local, int last_valid, int64_t step, int push_meta, float *out,
                                      void *stream)
{
    if (!local || !global_view || !knobs || !wg || !wl || !peers || !q || !out) {
        set_error("cqa_sharded_layer_step: NULL pointer");
        return CQA_ERR_INVALID;
    }
    const int W = peers->world, R = peers->rank, H = peers->n_heads, KV = local->kv_heads;
    if (W < 2 || W > CQA_MAX_PEERS || R < 0 || R >= W || H != KV * local->gqa_group ||
        peers->rows != 2 * H + KV + 1 || peers->chunk < n_local || peers->chunk < (int64_t)KV * D ||
        (peers->chunk & 3) != 0 || step < 1 ||
        step > 0x7fffffff) {
        set_error("cqa_sharded_layer_step: inconsistent peer description");
        return CQA_ERR_INVALID;
    }
    for (int p = 0; p < W; ++p)
        if (!peers->base[p]) { set_error("cqa_sharded_layer_step: peer %d is not mapped", p); return CQA_ERR_INVALID; }
    // every range check of the three kernels comes before the first launch or copy
    if (n_local <= 0 || nact_local < n_local || nact_local > n_local + 1 || nq_global < n_local ||
        nact_global < nq_global || nact_global > nq_global + 1 || first_block < 0 || first_block + n_local > nq_global) {
        set_error("cqa_sharded_layer_step: inconsistent block counts (local %ld/%ld, global %ld/%ld, first %ld)",
                  (long)n_local, (long)nact_local, (long)nq_global, (long)nact_global, (long)first_block);
        return CQA_ERR_INVALID;
    }
    int rc = check_score_args(local, q_dtype, n_local, peers->chunk, "cqa_sharded_layer_step");
    if (rc) return rc;
    if (!wl->token_scores || !wg->cert || !wg->any_flags || !wg->mass_frac || !wg->topk_mask || !wg->explore_mask ||
        !wg->value_mask || !wg->sorted_idx || !wg->sorted_cumsum) {
        set_error("cqa_sharded_layer_step: workspace is missing selector buffers or token scores");
        return CQA_ERR_INVALID;
    }
    if (nact_global > wg->ld || nact_global > global_view->max_blocks) {
        set_error("cqa_sharded_layer_step: %ld global blocks exceed the global leading dimension", (long)nact_global);
        return CQA_ERR_INVALID;
    }
    if (push_meta && (!local->values_int4_errors || !local->sigma_max)) {
        set_error("cqa_sharded_layer_step: eta rows or scale maxima missing");
        return CQA_ERR_INVALID;
    }
    {
        cqa_workspace probe = *wg;
        probe.shard_stride = probe.shard_stride > 0 ? probe.shard_stride : 1;   // the exchange layout replaces ld
        probe.given_fp16 = static_cast<const float *>(peers->base[R]);
        probe.peer_world = W;
        probe.peer_step = (int)step;
        rc = selcert_check(global_view, knobs, &probe, q, nq_global, 1 | 2 | 64);
        if (rc) return rc;
        cqa_workspace lp = *wl;
        lp.partial_out = static_cast<float *>(peers->base[R]);
        rc = attend_check(local, &lp, n_local, nact_local, last_valid);
        if (rc) return rc;
    }
    cudaStream_t st = (cudaStream_t)stream;
    const PeerLayout L = peer_layout(W, H, peers->rows, peers->chunk);
    const int par = (int)(step & 1);
    PeerArgs pa;
    for (int p = 0; p < CQA_MAX_PEERS; ++p) pa.base[p] = p < W ? static_cast<float *>(peers->base[p]) : nullptr;
    pa.world = W;
    pa.rank = R;
    float *own = static_cast<float *>(peers->base[R]);
    int32_t *own_i = reinterpret_cast<int32_t *>(own);
    const long slot = (long)peers->rows * peers->chunk;                 // one rank's rows of xa
    float *xa_par = own + L.xa + par * L.xa_parity;                      // [world][rows][chunk] of this parity
    float *xa_own = xa_par + (long)R * slot;
    const long xb_off = L.xb + par * L.xb_parity + (long)R * H * CQA_MAX_RANKING_K * 2;
    float *xc_par = own + L.xc + par * L.xc_parity;
    float *xc_own = xc_par + (long)R * H * CQA_PARTIAL_STRIDE;

    // 1. Phase 1 on the local blocks, straight into this rank's slot of xa.  On ordinary steps the kernel also stores
    // every result into the other ranks' buffers and its last CTA releases the Exchange-A flags; when eta rows and
    // scale maxima changed (a block completed) the rows go out together through the push kernel instead.
    ScorePush sp = {};
    if (!push_meta) {
        const long row0 = L.xa + par * L.xa_parity + (long)R * slot;
        for (int p = 0; p < W; ++p) {
            sp.mb[p] = pa.base[p] + row0;
            sp.sb[p] = pa.base[p] + row0 + (long)H * peers->chunk;
            sp.flag[p] = reinterpret_cast<int32_t *>(pa.base[p]) + L.flags + 0 * W + R;
        }
        sp.ticket = own_i + L.tickets + 0 * W + R;
        sp.world = W;
        sp.rank = R;
        sp.step = (int)step;
    }
    rc = score_blocks_launch(local, q, q_dtype, n_local, knobs->q_scale, xa_own, xa_own + (long)H * peers->chunk,
                                 peers->chunk, wl->token_scores, st, wg->any_flags, 5 + H, push_meta ? nullptr : &sp);
    if (rc) return rc;
    if (push_meta) {
        // eta rows and the row of scale maxima follow the 2H score rows; both parities get them
        rc = check_cuda(cudaMemcpy2DAsync(xa_own + 2L * H * peers->chunk, peers->chunk * 4, local->values_int4_errors,
                                          local->max_blocks * 4, (size_t)n_local * 4, KV, cudaMemcpyDeviceToDevice, st),
                        "copy of eta rows");
        if (rc) return rc;
        rc = check_cuda(cudaMemcpyAsync(xa_own + (2L * H + KV) * peers->chunk, local->sigma_max, (size_t)KV * D * 4,
                                        cudaMemcpyDeviceToDevice, st), "copy of scale maxima");
        if (rc) return rc;
        dim3 grid(W, PUSH_CTAS);
        peer_push_kernel<<<grid, PUSH_THREADS, 0, st>>>(pa, xa_own, peers->chunk, L.xa + par * L.xa_parity + (long)R * slot,
                                                        peers->chunk, peers->rows, 2 * H, n_local, n_local, (long)KV * D,
                                                        L.flags + 0 * W + R, L.tickets + 0 * W, (int)step,
                                                        L.xa + (par ^ 1) * L.xa_parity + (long)R * slot, 2 * H); note_launch();
        float *other = own + L.xa + (par ^ 1) * L.xa_parity + (long)R * slot + 2L * H * peers->chunk;
        rc = check_cuda(cudaMemcpyAsync(other, xa_own + 2L * H * peers->chunk, (size_t)(KV + 1) * peers->chunk * 4,
                                        cudaMemcpyDeviceToDevice, st), "copy of meta rows to the other parity");
        if (rc) return rc;
    }
    // 3. the global selector and certificate on the exchanged arrays, one launch: it waits for every rank's A; the
    // ranking-check CTA of each head re-scores the top-list blocks this rank owns, pushes them to every rank, waits
    // for the other ranks' rows (Exchange B, per head) and raises the flags
    cqa_workspace g = *wg;
    g.m_b = xa_par;
    g.s_b = xa_par + (long)H * peers->chunk;
    g.shard_chunk = peers->chunk;
    g.shard_rank_stride = slot;
    g.shard_ranks = W;
    g.wait_flags = own_i + L.flags + 0 * W;
    g.wait_n = W;
    g.wait_skip = R;
    g.wait_value = (int)step;
    g.wait_status = own_i + L.status;
    g.partial_out = nullptr;
    g.given_fp16 = own + L.xb + par * L.xb_parity;
    g.given_ranks = W;
    g.given_rank_stride = (long)H * CQA_MAX_RANKING_K * 2;
    for (int p = 0; p < CQA_MAX_PEERS; ++p) {
        g.peer_xb[p] = p < W ? pa.base[p] + xb_off : nullptr;
        g.peer_flags_b[p] = p < W ? reinterpret_cast<int32_t *>(pa.base[p]) + L.flags_b : nullptr;
    }
    g.peer_first_block = first_block;
    g.peer_n_local = n_local;
    g.peer_world = W;
    g.peer_rank = R;
    g.peer_step = (int)step;
    cqa_cache gv = *global_view;
    gv.values_int4_errors = xa_par + 2L * H * peers->chunk;
    gv.sigma_max = xa_par + (2L * H + KV) * peers->chunk;
    rc = selcert_launch(&gv, knobs, &g, q, q_dtype, nq_global, nact_global, nullptr, 0, 1 | 2 | 16 | 64, st);
    if (rc) return rc;
    // 6. Phase 2 over the local blocks; un-normalised partial rows go to this rank's slot of xc
    cqa_workspace l = *wl;
    l.m_b = xa_own;
    l.s_b = xa_own + (long)H * peers->chunk;
    l.shard_stride = 0;
    l.shard_chunk = peers->chunk;
    l.partial_out = xc_own;
    l.wait_flags = nullptr;
    // Exchange C is written by Phase 2 itself: its final merges store the partial rows into every rank's buffer and
    // the last of them releases the flags
    const long xc_slot = L.xc + par * L.xc_parity + (long)R * H * CQA_PARTIAL_STRIDE;
    for (int p = 0; p < CQA_MAX_PEERS; ++p) {
        l.peer_partial[p] = p < W ? pa.base[p] + xc_slot : nullptr;
        l.peer_flag_c[p] = p < W ? reinterpret_cast<int32_t *>(pa.base[p]) + L.flags + 2 * W + R : nullptr;
    }
    l.peer_ticket_c = own_i + L.tickets + 2 * W + R;
    l.peer_world = W;
    l.peer_rank = R;
    l.peer_step = (int)step;
    rc = attend_launch(local, &l, q, q_dtype, n_local, nact_local, num_tokens_local, last_valid, knobs->q_scale, st, true);
    if (rc) return rc;
    // the four kernels are chained by programmatic dependent launch, like the single-GPU step: each one is scheduled
    // while the previous one drains and waits for it on the device (the score kernel cleared the certifier's flags)
    return check_cuda(launch_chained(merge_wait_kernel, dim3(H), dim3(D), 0, st, true, (const float *)xc_par, W, H, out,
                                     (const int32_t *)(own_i + L.flags + 2 * W), R, (int)step, own_i + L.status,
                                     wg->wait_spins), "sharded step kernels");
}
