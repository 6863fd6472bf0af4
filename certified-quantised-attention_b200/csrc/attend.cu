// Phase 2: mixed INT8/FP16-key, INT4/FP16-value split-K attend, the dense
// FP16 recompute of flagged heads, and the log-sum-exp merge.
//
// attend_mixed_kernel: one CTA = (kv head, split of blocks); the G query heads
// of the group share every value load.  A warp owns one 16-token block at a
// time: lane L (mod 16) owns output channels 8L..8L+7, the two half warps take
// 8 tokens each.  Blocks whose (head, block) bit in topk_mask is clear reuse
// the Phase-1 token scores (no second pass over the INT8 keys); promoted
// blocks recompute their scores from the Tier-2 keys.  INT4 values are
// unpacked and dequantised in registers straight into the softmax.V
// accumulation; (head, block) pairs flagged in value_mask read Tier-2 values.
//
// Nothing computed here can change a selection or a certificate flag, so fast
// exponentials are used.
#include <mutex>

#include "common.cuh"

namespace cqa {

constexpr int ATT_WARPS = 8;

__device__ __forceinline__ float fexp(float x) { return __expf(x); }

// Merge (m, l, acc) partials across the warps of a CTA and write one partial.
template <int G>
__device__ __forceinline__ void cta_merge_store(float (&m)[G], float (&l)[G], float (&acc)[G][8], float *sm_m,
                                                float *sm_l, float *sm_acc, float *out_m, float *out_l,
                                                float *out_acc, int head0, int split, int nsplits)
{
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, L = lane & 15;
    // the two half warps hold partial sums over disjoint tokens
#pragma unroll
    for (int g = 0; g < G; ++g)
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[g][i] += __shfl_xor_sync(FULL, acc[g][i], 16);
    if (lane < 16) {
#pragma unroll
        for (int g = 0; g < G; ++g)
#pragma unroll
            for (int i = 0; i < 8; ++i) sm_acc[(warp * G + g) * D + 8 * L + i] = acc[g][i];
    }
    if (lane == 0) {
#pragma unroll
        for (int g = 0; g < G; ++g) { sm_m[warp * G + g] = m[g]; sm_l[warp * G + g] = l[g]; }
    }
    __syncthreads();
    for (int item = threadIdx.x; item < G * D; item += ATT_WARPS * 32) {
        const int g = item / D, ch = item % D;
        float M = -INFINITY;
#pragma unroll
        for (int w = 0; w < ATT_WARPS; ++w) M = fmaxf(M, sm_m[w * G + g]);
        float a = 0.0f, ll = 0.0f;
#pragma unroll
        for (int w = 0; w < ATT_WARPS; ++w) {
            const float mw = sm_m[w * G + g];
            const float sc = mw == -INFINITY ? 0.0f : fexp(mw - M);
            a = fmaf(sm_acc[(w * G + g) * D + ch], sc, a);
            ll = fmaf(sm_l[w * G + g], sc, ll);
        }
        const long p = (long)(head0 + g) * nsplits + split;
        out_acc[p * D + ch] = a;
        if (ch == 0) { out_m[p] = M; out_l[p] = ll; }
    }
}

template <int G, typename T2>
__global__ void __launch_bounds__(ATT_WARPS * 32) attend_mixed_kernel(cqa_cache c, cqa_workspace ws, const void *q,
                                                                     int q_dtype, long nq, long nact,
                                                                     int last_valid, float q_scale,
                                                                     int blocks_per_split)
{
    __shared__ float s_q[G * D];
    __shared__ float s_w[ATT_WARPS][BS][G];        // softmax weights of the current block, [token][head]
    __shared__ float s_sc[ATT_WARPS][G][BS];       // FP16-key logits of the current block
    __shared__ float sm_m[ATT_WARPS * G], sm_l[ATT_WARPS * G];
    __shared__ float sm_acc[ATT_WARPS * G * D];
    const int kv = blockIdx.y, split = blockIdx.x;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, L = lane & 15, hw = lane >> 4;
    const long b_begin = (long)split * blocks_per_split;
    const long b_end = min(nact, b_begin + (long)blocks_per_split);
    for (int i = threadIdx.x; i < G * D; i += ATT_WARPS * 32) s_q[i] = load_q(q, q_dtype, (long)kv * G * D + i);
    __syncthreads();

    float m[G], l[G], acc[G][8];
#pragma unroll
    for (int g = 0; g < G; ++g) {
        m[g] = -INFINITY;
        l[g] = 0.0f;
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[g][i] = 0.0f;
    }
    const T2 *kt2 = reinterpret_cast<const T2 *>(c.keys_t2) + (long)kv * c.keys_t2_rows * D;
    const T2 *vt2 = reinterpret_cast<const T2 *>(c.values_t2) + (long)kv * c.values_t2_rows * D;
    constexpr int NP = (G + 1) / 2;  // score passes: two heads (one per half warp) at a time

    for (long b = b_begin + warp; b < b_end; b += ATT_WARPS) {
        unsigned km = 0, vm = 0;  // bit g: head g uses FP16 keys / FP16 values for this block
#pragma unroll
        for (int g = 0; g < G; ++g) {
            const long o = (long)(kv * G + g) * ws.ld + b;
            km |= (ws.topk_mask[o] || b >= nq) ? (1u << g) : 0u;
            vm |= ws.value_mask[o] ? (1u << g) : 0u;
        }
        const int n_valid = (b == nact - 1) ? last_valid : BS;
        // FP16-key logits for promoted heads
        if (km) {
            long kslot = c.key_slots ? (long)c.key_slots[b] : b;
            if (kslot < 0) kslot = 0;
            float kf[8][8];
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const int t = hw * 8 + i;
                if (t < n_valid) load8<T2>(kt2 + (kslot * BS + t) * D + 8 * L, kf[i]);
                else {
#pragma unroll
                    for (int k = 0; k < 8; ++k) kf[i][k] = 0.0f;
                }
            }
#pragma unroll
            for (int g = 0; g < G; ++g) {
                if (km & (1u << g)) {
                    float qv[8];
                    load8<float>(s_q + g * D + 8 * L, qv);
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        float d = hw_sum(chain8(kf[i], qv));
                        if (L == i) s_sc[warp][g][hw * 8 + i] = d * q_scale;
                    }
                }
            }
            __syncwarp();
        }
        // softmax bookkeeping, two heads per pass
        float alpha[G];
#pragma unroll
        for (int p = 0; p < NP; ++p) {
            const int g = 2 * p + hw;
            const bool gvalid = g < G;
            float s = -INFINITY;
            if (gvalid && L < n_valid) {
                if (km & (1u << g)) s = s_sc[warp][g][L];
                else s = ws.token_scores[(((long)kv * nq + b) * G + g) * BS + L];
            }
            const float bm = hw_max(s);
            const float bm_o = __shfl_xor_sync(FULL, bm, 16);
            // new running max for this lane's head (and the other half's head)
            const int g_o = 2 * p + (hw ^ 1);
            float m_old_mine = 0.0f, m_new_mine = 0.0f;
#pragma unroll
            for (int gg = 0; gg < G; ++gg) {
                if (gg == g || gg == g_o) {
                    const float bmg = (gg == g) ? bm : bm_o;
                    const float mn = fmaxf(m[gg], bmg);
                    alpha[gg] = (mn == -INFINITY || m[gg] == mn) ? 1.0f : fexp(m[gg] - mn);
                    if (gg == g) { m_old_mine = m[gg]; m_new_mine = mn; }
                    m[gg] = mn;
                }
            }
            (void)m_old_mine;
            const float w = (gvalid && s != -INFINITY) ? fexp(s - m_new_mine) : 0.0f;
            if (gvalid) s_w[warp][L][g] = w;
            const float ls = hw_sum(w);
            const float ls_o = __shfl_xor_sync(FULL, ls, 16);
#pragma unroll
            for (int gg = 0; gg < G; ++gg) {
                if (gg == g || gg == g_o) l[gg] = fmaf(l[gg], alpha[gg], (gg == g) ? ls : ls_o);
            }
        }
        __syncwarp();
#pragma unroll
        for (int g = 0; g < G; ++g) {
            if (alpha[g] != 1.0f) {
#pragma unroll
                for (int i = 0; i < 8; ++i) acc[g][i] *= alpha[g];
            }
        }
        // values
        const bool need4 = (vm != ((1u << G) - 1u));
        const bool need16 = vm != 0;
        long vslot = c.value_slots ? (long)c.value_slots[b] : b;
        if (vslot < 0) vslot = 0;
        const long row_base = (long)kv * c.cap_tokens + b * BS;
#pragma unroll 2
        for (int i = 0; i < 8; ++i) {
            const int t = hw * 8 + i;
            if (t >= n_valid) continue;
            float v4[8], v16[8];
            if (need4) {
                const long row = row_base + t;
                const unsigned pk = *reinterpret_cast<const unsigned *>(c.values_int4_packed + row * (D / 2) + 4 * L);
                const float s = __half2float(__ushort_as_half(c.values_int4_scales[row * NG + (L >> 1)]));
                const float z = __half2float(__ushort_as_half(c.values_int4_zeros[row * NG + (L >> 1)]));
#pragma unroll
                for (int k = 0; k < 8; ++k) v4[k] = fmaf((float)((pk >> (4 * k)) & 0xFu), s, z);
            }
            if (need16) load8<T2>(vt2 + (vslot * BS + t) * D + 8 * L, v16);
            float wv[G];
#pragma unroll
            for (int g = 0; g < G; ++g) wv[g] = s_w[warp][t][g];
#pragma unroll
            for (int g = 0; g < G; ++g) {
                if (vm & (1u << g)) {
#pragma unroll
                    for (int k = 0; k < 8; ++k) acc[g][k] = fmaf(wv[g], v16[k], acc[g][k]);
                } else {
#pragma unroll
                    for (int k = 0; k < 8; ++k) acc[g][k] = fmaf(wv[g], v4[k], acc[g][k]);
                }
            }
        }
        __syncwarp();
    }
    cta_merge_store<G>(m, l, acc, sm_m, sm_l, sm_acc, ws.part_m, ws.part_l, ws.part_acc, kv * G, split,
                       ws.num_splits);
}

// Dense attention over the Tier-2 keys/values of heads flagged for recompute
// (per-head Rung 3, or every head when a score-consistency violation was
// raised).  Grid (dense_splits, H); CTAs of unflagged heads return at once.
template <typename T2>
__global__ void __launch_bounds__(ATT_WARPS * 32) dense_attend_kernel(cqa_cache c, cqa_workspace ws, const void *q,
                                                                     int q_dtype, long num_tokens, float q_scale,
                                                                     int blocks_per_split)
{
    const int h = blockIdx.y, split = blockIdx.x;
    if (!(ws.cert[h].dense || ws.any_flags[2])) return;
    __shared__ float sm_m[ATT_WARPS], sm_l[ATT_WARPS];
    __shared__ float sm_acc[ATT_WARPS * D];
    const int kv = h / c.gqa_group;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, L = lane & 15, hw = lane >> 4;
    const long nblk = (num_tokens + BS - 1) / BS;
    const long b_begin = (long)split * blocks_per_split;
    const long b_end = min(nblk, b_begin + (long)blocks_per_split);
    float qv[8];
    load_q8(q, q_dtype, (long)h * D + 8 * L, qv);
    const T2 *kt2 = reinterpret_cast<const T2 *>(c.keys_t2) + (long)kv * c.keys_t2_rows * D;
    const T2 *vt2 = reinterpret_cast<const T2 *>(c.values_t2) + (long)kv * c.values_t2_rows * D;
    float m[1] = {-INFINITY}, l[1] = {0.0f}, acc[1][8];
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[0][i] = 0.0f;
    for (long b = b_begin + warp; b < b_end; b += ATT_WARPS) {
        long kslot = c.key_slots ? (long)c.key_slots[b] : b;
        long vslot = c.value_slots ? (long)c.value_slots[b] : b;
        if (kslot < 0 || vslot < 0) continue;
        float lg[8];
        float bm = -INFINITY;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const long t = b * BS + hw * 8 + i;
            float kf[8];
            if (t < num_tokens) load8<T2>(kt2 + (kslot * BS + hw * 8 + i) * D + 8 * L, kf);
            else {
#pragma unroll
                for (int k = 0; k < 8; ++k) kf[k] = 0.0f;
            }
            const float d = hw_sum(chain8(kf, qv));
            lg[i] = t < num_tokens ? d * q_scale : -INFINITY;
            bm = fmaxf(bm, lg[i]);
        }
        bm = fmaxf(bm, __shfl_xor_sync(FULL, bm, 16));
        const float mn = fmaxf(m[0], bm);
        const float alpha = (mn == -INFINITY || m[0] == mn) ? 1.0f : fexp(m[0] - mn);
        m[0] = mn;
        float ls = 0.0f;
        if (alpha != 1.0f) {
#pragma unroll
            for (int i = 0; i < 8; ++i) acc[0][i] *= alpha;
        }
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            if (lg[i] == -INFINITY) continue;
            const float w = fexp(lg[i] - mn);
            ls += w;
            float vf[8];
            load8<T2>(vt2 + (vslot * BS + hw * 8 + i) * D + 8 * L, vf);
#pragma unroll
            for (int k = 0; k < 8; ++k) acc[0][k] = fmaf(w, vf[k], acc[0][k]);
        }
        ls += __shfl_xor_sync(FULL, ls, 16);
        l[0] = fmaf(l[0], alpha, ls);
    }
    cta_merge_store<1>(m, l, acc, sm_m, sm_l, sm_acc, ws.dense_m, ws.dense_l, ws.dense_acc, h, split,
                       ws.dense_splits);
}

// Final merge of the split partials; picks the dense partials for flagged heads.
__global__ void __launch_bounds__(D) lse_reduce_kernel(cqa_workspace ws)
{
    const int h = blockIdx.x, ch = threadIdx.x;
    const bool dense = ws.cert != nullptr && (ws.cert[h].dense || ws.any_flags[2]);
    const int ns = dense ? ws.dense_splits : ws.num_splits;
    const float *pm = dense ? ws.dense_m : ws.part_m;
    const float *pl = dense ? ws.dense_l : ws.part_l;
    const float *pa = dense ? ws.dense_acc : ws.part_acc;
    float M = -INFINITY;
    for (int s = 0; s < ns; ++s) M = fmaxf(M, pm[(long)h * ns + s]);
    float a = 0.0f, l = 0.0f;
    for (int s = 0; s < ns; ++s) {
        const long p = (long)h * ns + s;
        const float mi = pm[p];
        const float sc = mi == -INFINITY ? 0.0f : fexp(mi - M);
        a = fmaf(pa[p * D + ch], sc, a);
        l = fmaf(pl[p], sc, l);
    }
    ws.out[(long)h * D + ch] = a / (l > 0.0f ? l : 1.0f);
}

template <typename T2>
static int attend_launch_t(const cqa_cache *c, const cqa_workspace *ws, const void *q, int q_dtype, long nq,
                           long nact, long num_tokens, int last_valid, float q_scale, cudaStream_t st)
{
    const int H = c->kv_heads * c->gqa_group;
    const int ns = ws->num_splits;
    const int bps = (int)((nact + ns - 1) / ns);
    dim3 grid((unsigned)ns, (unsigned)c->kv_heads);
    switch (c->gqa_group) {
    case 1: attend_mixed_kernel<1, T2><<<grid, ATT_WARPS * 32, 0, st>>>(*c, *ws, q, q_dtype, nq, nact, last_valid, q_scale, bps); break;
    case 2: attend_mixed_kernel<2, T2><<<grid, ATT_WARPS * 32, 0, st>>>(*c, *ws, q, q_dtype, nq, nact, last_valid, q_scale, bps); break;
    case 4: attend_mixed_kernel<4, T2><<<grid, ATT_WARPS * 32, 0, st>>>(*c, *ws, q, q_dtype, nq, nact, last_valid, q_scale, bps); break;
    case 8: attend_mixed_kernel<8, T2><<<grid, ATT_WARPS * 32, 0, st>>>(*c, *ws, q, q_dtype, nq, nact, last_valid, q_scale, bps); break;
    default: set_error("cqa_attend: unsupported gqa_group %d", c->gqa_group); return CQA_ERR_UNSUPPORTED;
    }
    int rc = check_launch("attend_mixed_kernel");
    if (rc) return rc;
    if (ws->cert && ws->dense_splits > 0 && ws->dense_m && c->keys_t2 && c->values_t2) {
        const long nblk = (num_tokens + BS - 1) / BS;
        const int dbps = (int)((nblk + ws->dense_splits - 1) / ws->dense_splits);
        dim3 dgrid((unsigned)ws->dense_splits, (unsigned)H);
        dense_attend_kernel<T2><<<dgrid, ATT_WARPS * 32, 0, st>>>(*c, *ws, q, q_dtype, num_tokens, q_scale, dbps);
        rc = check_launch("dense_attend_kernel");
        if (rc) return rc;
    }
    lse_reduce_kernel<<<H, D, 0, st>>>(*ws);
    return check_launch("lse_reduce_kernel");
}

int attend_launch(const cqa_cache *c, const cqa_workspace *ws, const void *q, int q_dtype, long nq, long nact,
                  long num_tokens, int last_valid, float q_scale, cudaStream_t st)
{
    if (ws->num_splits <= 0 || !ws->part_m || !ws->part_l || !ws->part_acc || !ws->out || !ws->topk_mask ||
        !ws->value_mask) {
        set_error("cqa_attend: workspace is missing partial buffers, masks or the output");
        return CQA_ERR_INVALID;
    }
    if (nq > 0 && !ws->token_scores) { set_error("cqa_attend: token_scores missing"); return CQA_ERR_INVALID; }
    if (nact <= 0 || nact > ws->ld || nact > c->max_blocks) {
        set_error("cqa_attend: nact=%ld out of range (ld=%ld)", nact, (long)ws->ld);
        return CQA_ERR_INVALID;
    }
    if (last_valid < 1 || last_valid > BS) { set_error("cqa_attend: last_block_valid=%d", last_valid); return CQA_ERR_INVALID; }
    if (!c->keys_t2 || !c->values_t2) {
        set_error("cqa_attend: Tier-2 key/value arrays are required (promoted and trailing blocks read them)");
        return CQA_ERR_INVALID;
    }
    switch (c->t2_dtype) {
    case CQA_F32: return attend_launch_t<float>(c, ws, q, q_dtype, nq, nact, num_tokens, last_valid, q_scale, st);
    case CQA_F16: return attend_launch_t<__half>(c, ws, q, q_dtype, nq, nact, num_tokens, last_valid, q_scale, st);
    case CQA_BF16: return attend_launch_t<__nv_bfloat16>(c, ws, q, q_dtype, nq, nact, num_tokens, last_valid, q_scale, st);
    }
    set_error("cqa_attend: unknown Tier-2 dtype %d", c->t2_dtype);
    return CQA_ERR_INVALID;
}

// ---------------------------------------------------------------------------
// Built-in scratch for cqa_attend_static: split partials for callers that
// cannot allocate device memory.  Layout: [Phase-2 m | l | acc][dense m | l | acc].
constexpr long STATIC_P2 = (long)CQA_STATIC_MAX_HEADS * CQA_STATIC_MAX_SPLITS;
constexpr long STATIC_DN = (long)CQA_STATIC_MAX_HEADS * CQA_STATIC_MAX_DENSE_SPLITS;
constexpr long STATIC_FLOATS = STATIC_P2 * (D + 2) + STATIC_DN * (D + 2);
static __device__ __align__(256) float g_static_partials[STATIC_FLOATS];

// Device address of g_static_partials per device.  In host code the symbol is
// only a handle; the address a kernel can use comes from cudaGetSymbolAddress,
// looked up once per device with that device current.
static float *static_partials_for_current_device(int *rc_out)
{
    constexpr int MAX_DEV = 64;
    static float *addr[MAX_DEV] = {nullptr};
    static std::mutex mu;
    int dev = -1;
    *rc_out = check_cuda(cudaGetDevice(&dev), "cudaGetDevice");
    if (*rc_out) return nullptr;
    if (dev < 0 || dev >= MAX_DEV) {
        set_error("cqa_attend_static: device index %d out of range", dev);
        *rc_out = CQA_ERR_UNSUPPORTED;
        return nullptr;
    }
    std::lock_guard<std::mutex> lock(mu);
    if (!addr[dev]) {
        void *p = nullptr;
        *rc_out = check_cuda(cudaGetSymbolAddress(&p, g_static_partials), "cudaGetSymbolAddress(g_static_partials)");
        if (*rc_out) return nullptr;
        addr[dev] = static_cast<float *>(p);
    }
    return addr[dev];
}

int attend_static_launch(const cqa_cache *c, const cqa_workspace *ws, const void *q, int q_dtype, long nq, long nact,
                         long num_tokens, int last_valid, float q_scale, cudaStream_t st)
{
    const long H = (long)c->kv_heads * c->gqa_group;
    if (H > CQA_STATIC_MAX_HEADS || ws->num_splits > CQA_STATIC_MAX_SPLITS ||
        ws->dense_splits > CQA_STATIC_MAX_DENSE_SPLITS) {
        set_error("cqa_attend_static: %ld heads / %d splits / %d dense splits exceed the built-in scratch "
                  "(limits %d / %d / %d); use cqa_attend with caller-provided partial buffers",
                  H, ws->num_splits, ws->dense_splits, CQA_STATIC_MAX_HEADS, CQA_STATIC_MAX_SPLITS,
                  CQA_STATIC_MAX_DENSE_SPLITS);
        return CQA_ERR_TOO_LARGE;
    }
    int rc = CQA_OK;
    float *base = static_partials_for_current_device(&rc);
    if (rc) return rc;
    cqa_workspace w = *ws;
    w.part_m = base;
    w.part_l = base + STATIC_P2;
    w.part_acc = base + 2 * STATIC_P2;
    float *dn = base + STATIC_P2 * (D + 2);
    w.dense_m = dn;
    w.dense_l = dn + STATIC_DN;
    w.dense_acc = dn + 2 * STATIC_DN;
    return attend_launch(c, &w, q, q_dtype, nq, nact, num_tokens, last_valid, q_scale, st);
}

}  // namespace cqa
