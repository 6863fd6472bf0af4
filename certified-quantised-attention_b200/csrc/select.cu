// Selector and certifier: one CTA of 1024 threads per query head.
//
// cqa_select : block mass fractions, descending order of blocks by mass
//              (ties -> lower block id), sequential cumulative mass, K* with
//              the Rung-1 expansion, exploration draw, FP16-key mask.
// cqa_certify: top-k blocks by m_b, FP16 re-score, ranking / boundary /
//              score-consistency flags, greedy Rung-2 value promotion.
//
// Sums over blocks use the canonical order: 32 consecutive values by a warp
// butterfly, 8 such sums by a butterfly (one 256-block leaf), leaves added
// left to right.  Prefix sums over the sorted order are sequential.
#include "common.cuh"
#include "rescore.cuh"

namespace cqa {

constexpr int SEL_THREADS = 1024;

struct SelShared {
    float red_f[32];
    unsigned long long red_u[32];
    float leaf[4];
    float bcast_f[4];
    int bcast_i[4];
    unsigned long long bcast_u;
    int counter;
};

__device__ __forceinline__ float block_max(float v, SelShared &sh)
{
    v = warp_max(v);
    const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
    __syncthreads();
    if (l == 0) sh.red_f[w] = v;
    __syncthreads();
    float r = sh.red_f[l];
    r = warp_max(r);
    return r;
}

__device__ __forceinline__ unsigned long long warp_max_u64(unsigned long long v)
{
#pragma unroll
    for (int s = 16; s >= 1; s >>= 1) {
        unsigned long long o = __shfl_xor_sync(FULL, v, s);
        v = o > v ? o : v;
    }
    return v;
}
__device__ __forceinline__ unsigned long long block_max_u64(unsigned long long v, SelShared &sh)
{
    v = warp_max_u64(v);
    const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
    __syncthreads();
    if (l == 0) sh.red_u[w] = v;
    __syncthreads();
    return warp_max_u64(sh.red_u[l]);
}

// Canonical sum of vals[0..n) (shared memory, values beyond n read as +0).
// All 1024 threads must call it; the result is returned to every thread.
__device__ float block_canonical_sum(const float *vals, int n, SelShared &sh)
{
    const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
    float total = 0.0f;
    for (int base = 0; base < n; base += SEL_THREADS) {
        const int i = base + threadIdx.x;
        float v = i < n ? vals[i] : 0.0f;
        v = warp_sum(v);  // strides 16,8,4,2,1 over 32 consecutive values
        __syncthreads();
        if (l == 0) sh.red_f[w] = v;
        __syncthreads();
        if (w == 0) {
            float g = sh.red_f[l];
            g = __fadd_rn(g, __shfl_xor_sync(FULL, g, 4));
            g = __fadd_rn(g, __shfl_xor_sync(FULL, g, 2));
            g = __fadd_rn(g, __shfl_xor_sync(FULL, g, 1));
            // lanes 0, 8, 16, 24 hold the four leaf sums of this pass
            float l0 = __shfl_sync(FULL, g, 0), l1 = __shfl_sync(FULL, g, 8);
            float l2 = __shfl_sync(FULL, g, 16), l3 = __shfl_sync(FULL, g, 24);
            if (l == 0) {
                total = __fadd_rn(total, l0);
                if (base + 256 < n) total = __fadd_rn(total, l1);
                if (base + 512 < n) total = __fadd_rn(total, l2);
                if (base + 768 < n) total = __fadd_rn(total, l3);
            }
        }
    }
    __syncthreads();
    if (threadIdx.x == 0) sh.bcast_f[0] = total;
    __syncthreads();
    return sh.bcast_f[0];
}

// In-place descending bitonic sort of n_pad (power of two) 64-bit keys.
__device__ void bitonic_sort_desc(unsigned long long *keys, int n_pad)
{
    for (int k = 2; k <= n_pad; k <<= 1) {
        for (int j = k >> 1; j > 0; j >>= 1) {
            for (int i = threadIdx.x; i < n_pad; i += SEL_THREADS) {
                const int ixj = i ^ j;
                if (ixj > i) {
                    const bool desc = (i & k) == 0;
                    const unsigned long long a = keys[i], b = keys[ixj];
                    if (desc ? (a < b) : (a > b)) {
                        keys[i] = b;
                        keys[ixj] = a;
                    }
                }
            }
            __syncthreads();
        }
    }
}

__device__ __forceinline__ unsigned long long make_key(float v, int idx)
{
    // v >= 0: the bit pattern orders like the value; ties -> lower index first.
    return ((unsigned long long)__float_as_uint(v) << 32) | (unsigned long long)(0xFFFFFFFFu - (unsigned)idx);
}
__device__ __forceinline__ int key_idx(unsigned long long k) { return (int)(0xFFFFFFFFu - (unsigned)(k & 0xFFFFFFFFull)); }
__device__ __forceinline__ float key_val(unsigned long long k) { return __uint_as_float((unsigned)(k >> 32)); }
__device__ __forceinline__ unsigned orderable(float v)
{
    unsigned u = __float_as_uint(v);
    return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

// Dynamic shared memory layout: keys[n_pad] (u64), vals[n_pad] (f32), mask[n_pad] (u8)
__global__ void __launch_bounds__(SEL_THREADS) select_kernel(cqa_cache c, cqa_knobs kn, cqa_workspace ws, long nq,
                                                            long nact, const float *u, long u_ld, int n_pad,
                                                            int hi, int base_width, int two_level)
{
    extern __shared__ __align__(16) unsigned char dsm[];
    unsigned long long *keys = reinterpret_cast<unsigned long long *>(dsm);
    float *vals = reinterpret_cast<float *>(dsm + (size_t)n_pad * 8);
    unsigned char *mask = dsm + (size_t)n_pad * 12;
    __shared__ SelShared sh;
    const int h = blockIdx.x, tid = threadIdx.x;
    const int n = (int)nq;
    const float *mb = ws.m_b + (long)h * ws.ld;
    const float *sb = ws.s_b + (long)h * ws.ld;
    if (tid == 0) sh.counter = 0;

    float mg = -INFINITY;
    for (int b = tid; b < n; b += SEL_THREADS) mg = fmaxf(mg, mb[b]);
    mg = block_max(mg, sh);
    for (int b = tid; b < n; b += SEL_THREADS) {
        float s = fmaxf(sb[b], 1e-30f);
        float lm = __fadd_rn(clog(s), mb[b]);
        vals[b] = cexp(__fsub_rn(lm, mg));
    }
    __syncthreads();
    float total = fmaxf(block_canonical_sum(vals, n, sh), 1e-30f);
    float *mf = ws.mass_frac + (long)h * ws.ld;
    for (int b = tid; b < n_pad; b += SEL_THREADS) {
        if (b < n) {
            float f = __fdiv_rn(vals[b], total);
            mf[b] = f;
            keys[b] = make_key(f, b);
        } else {
            keys[b] = 0ull;
        }
        mask[b] = 0;
    }
    __syncthreads();
    bitonic_sort_desc(keys, n_pad);

    cqa_head_cert *ct = ws.cert + h;
    if (tid == 0) {
        const float tau = kn.tau_cov;
        float cum = 0.0f;
        int ss_e = hi, ss_b = base_width;  // searchsorted results (first j with cum >= tau)
        bool found_e = false, found_b = false;
        float cum_at_b_last = 0.0f;
        int32_t *sidx = ws.sorted_idx + (long)h * ws.sel_width;
        float *scum = ws.sorted_cumsum + (long)h * ws.sel_width;
        for (int j = 0; j < hi; ++j) {
            float v = key_val(keys[j]);
            cum = j == 0 ? v : __fadd_rn(cum, v);
            sidx[j] = key_idx(keys[j]);
            scum[j] = cum;
            if (!found_e && cum >= tau) { ss_e = j; found_e = true; }
            if (j < base_width && !found_b && cum >= tau) { ss_b = j; found_b = true; }
        }
        (void)cum_at_b_last;
        const int lo_e = min(kn.k_min, hi);
        int k_e = min(max(ss_e + 1, lo_e), hi);
        float ta_e = scum[k_e - 1];
        float tl_e = fmaxf(__fsub_rn(1.0f, ta_e), 0.0f);
        int k_star = k_e;
        float ta = ta_e, tl = tl_e;
        int trig = 0, k_b = k_e;
        if (two_level) {
            const int lo_b = min(kn.k_min, base_width);
            k_b = min(max(ss_b + 1, lo_b), base_width);
            float ta_b = scum[k_b - 1];
            float tl_b = fmaxf(__fsub_rn(1.0f, ta_b), 0.0f);
            trig = tl_b > kn.rung1_threshold ? 1 : 0;
            if (!trig) { k_star = k_b; ta = ta_b; tl = tl_b; }
        } else if (kn.rung1_threshold >= 0.0f && kn.k_max > 0) {
            trig = tl_e > kn.rung1_threshold ? 1 : 0;
        }
        ct->k_star = k_star;
        ct->k_star_base = k_b;
        ct->k_star_expanded = k_e;
        ct->rung1_triggered = trig;
        ct->tail_mass = tl;
        ct->tau_actual = ta;
        ct->m_global = mg;
        ct->total_mass = total;
        sh.bcast_i[0] = k_star;
        if (trig) atomicOr(ws.any_flags + 0, 1);
    }
    __syncthreads();
    const int k_star = sh.bcast_i[0];
    for (int j = tid; j < k_star; j += SEL_THREADS) mask[key_idx(keys[j])] = 1;
    __syncthreads();
    unsigned char *tm = ws.topk_mask + (long)h * ws.ld;
    unsigned char *em = ws.explore_mask + (long)h * ws.ld;
    int explored = 0;
    const bool explore_on = kn.exploration_rate > 0.0f && u != nullptr;
    for (int b = tid; b < (int)nact; b += SEL_THREADS) {
        unsigned char m = 1, e = 0;
        if (b < n) {
            m = mask[b];
            if (!m && explore_on && u[(long)h * u_ld + b] < kn.exploration_rate) { m = 1; e = 1; ++explored; }
        }
        tm[b] = m;
        em[b] = e;
    }
    if (explored) atomicAdd(&sh.counter, explored);
    __syncthreads();
    if (tid == 0) ct->exploration_blocks = sh.counter;
}

template <typename T2>
__global__ void __launch_bounds__(SEL_THREADS) certify_kernel(cqa_cache c, cqa_knobs kn, cqa_workspace ws,
                                                             const void *q, int q_dtype, long nq, long nact,
                                                             int n_pad, int rk)
{
    extern __shared__ __align__(16) unsigned char dsm[];
    unsigned long long *keys = reinterpret_cast<unsigned long long *>(dsm);
    float *vals = reinterpret_cast<float *>(dsm + (size_t)n_pad * 8);
    unsigned char *mask = dsm + (size_t)n_pad * 12;
    __shared__ SelShared sh;
    __shared__ int top_idx[CQA_MAX_RANKING_K];
    __shared__ float top_i8[CQA_MAX_RANKING_K], top_f16[CQA_MAX_RANKING_K], top_lm[CQA_MAX_RANKING_K];
    __shared__ float s_delta;
    const int h = blockIdx.x, tid = threadIdx.x, warp = tid >> 5;
    const int kv = h / c.gqa_group;
    const int n = (int)nq;
    const float *mb = ws.m_b + (long)h * ws.ld;
    const float *sb = ws.s_b + (long)h * ws.ld;
    cqa_head_cert *ct = ws.cert + h;
    const bool need_fp16 = (kn.ranking_fallback || kn.score_consistency) && n > 0;
    int rung3 = 0, violation = 0;

    if (need_fp16) {
        // top-rk blocks by m_b, descending, ties -> lower block id
        unsigned long long prev = ~0ull;
        for (int r = 0; r < rk; ++r) {
            unsigned long long best = 0ull;
            for (int b = tid; b < n; b += SEL_THREADS) {
                unsigned long long k = ((unsigned long long)orderable(mb[b]) << 32) |
                                       (unsigned long long)(0xFFFFFFFFu - (unsigned)b);
                if (k < prev && k > best) best = k;
            }
            best = block_max_u64(best, sh);
            if (tid == 0) {
                top_idx[r] = key_idx(best);
                top_i8[r] = mb[key_idx(best)];
            }
            prev = best;
        }
        __syncthreads();
        if (warp < rk) {
            float s, lm;
            fp16_block_score_warp<T2>(c, q, q_dtype, h, (long)top_idx[warp], nq * BS, kn.q_scale, s, lm);
            if ((tid & 31) == 0) { top_f16[warp] = s; top_lm[warp] = lm; }
        } else if (warp == rk) {
            float d = delta_bound_warp(c, q, q_dtype, h);
            if ((tid & 31) == 0) s_delta = d;
        }
        __syncthreads();
        const float delta = s_delta;
        // boundary: max over blocks outside the re-scored set of ell_int8 + delta
        float ub = -INFINITY;
        if (kn.ranking_fallback) {
            for (int b = tid; b < n; b += SEL_THREADS) {
                bool in_top = false;
                for (int r = 0; r < rk; ++r) in_top |= (top_idx[r] == b);
                if (!in_top) {
                    float ell = __fadd_rn(clog(fmaxf(sb[b], 1e-30f)), mb[b]);
                    ub = fmaxf(ub, __fadd_rn(ell, delta));
                }
            }
            ub = block_max(ub, sh);
        }
        if (tid == 0) {
            // rank of the FP16 scores (descending, ties -> lower position)
            int rank16[CQA_MAX_RANKING_K];
            bool used[CQA_MAX_RANKING_K];
            for (int i = 0; i < rk; ++i) used[i] = false;
            for (int p = 0; p < rk; ++p) {
                int bi = -1;
                for (int i = 0; i < rk; ++i)
                    if (!used[i] && (bi < 0 || top_f16[i] > top_f16[bi])) bi = i;
                used[bi] = true;
                rank16[p] = bi;
            }
            int dis_main = 0, dis_r1 = 0, dis_r3 = 0, boundary = 0;
            float ell_r = -INFINITY;
            if (kn.ranking_fallback) {
                const int r_main = min(kn.ranking_r, rk);
                for (int p = 0; p < rk; ++p) {
                    const bool d = rank16[p] != p;
                    if (p < r_main) dis_main |= d;
                    if (p < 1) dis_r1 |= d;
                    if (p < 3) dis_r3 |= d;
                }
                // r-th largest FP16 log-mass
                float tmp[CQA_MAX_RANKING_K];
                for (int i = 0; i < rk; ++i) tmp[i] = top_lm[i];
                for (int p = 0; p < r_main; ++p) {
                    int bi = p;
                    for (int i = p + 1; i < rk; ++i)
                        if (tmp[i] > tmp[bi]) bi = i;
                    float t = tmp[p]; tmp[p] = tmp[bi]; tmp[bi] = t;
                }
                ell_r = r_main > 0 ? tmp[r_main - 1] : -INFINITY;
                boundary = (r_main > 0 && ub > ell_r) ? 1 : 0;
                if (kn.ranking_r <= 0) { dis_main = 0; dis_r1 = 0; dis_r3 = 0; }
            }
            if (kn.score_consistency) {
                const float thr = __fadd_rn(delta, kn.eps_guard);
                for (int i = 0; i < rk; ++i)
                    if (fabsf(__fsub_rn(top_f16[i], top_i8[i])) > thr) violation = 1;
            }
            rung3 = (dis_main | boundary) ? 1 : 0;
            ct->ranking_disagree = dis_main;
            ct->ranking_disagree_r1 = dis_r1;
            ct->ranking_disagree_r3 = dis_r3;
            ct->boundary_triggered = boundary;
            ct->rung3 = rung3;
            ct->consistency_violation = violation;
            ct->delta = delta;
            ct->boundary_ub = ub;
            ct->ell_fp16_r = ell_r;
            ct->fp16_top1 = top_f16[rank16[0]];
            ct->fp16_top2 = rk > 1 ? top_f16[rank16[1]] : top_f16[rank16[0]];
            ct->int8_top1 = top_i8[0];
            for (int i = 0; i < CQA_MAX_RANKING_K; ++i) {
                ct->top_blocks[i] = i < rk ? top_idx[i] : -1;
                ct->fp16_scores[i] = i < rk ? top_f16[i] : 0.0f;
                ct->fp16_logmass[i] = i < rk ? top_lm[i] : 0.0f;
            }
            ct->dense = (kn.ranking_fallback && kn.rung3_recompute && rung3) ? 1 : 0;
            if (rung3) atomicOr(ws.any_flags + 1, 1);
            if (violation) atomicOr(ws.any_flags + 2, 1);
        }
    } else if (tid == 0) {
        ct->ranking_disagree = ct->ranking_disagree_r1 = ct->ranking_disagree_r3 = 0;
        ct->boundary_triggered = ct->rung3 = ct->consistency_violation = ct->dense = 0;
        ct->delta = 0.0f;
        ct->boundary_ub = -INFINITY;
        ct->ell_fp16_r = -INFINITY;
        ct->fp16_top1 = ct->fp16_top2 = ct->int8_top1 = 0.0f;
        for (int i = 0; i < CQA_MAX_RANKING_K; ++i) { ct->top_blocks[i] = -1; ct->fp16_scores[i] = 0.0f; ct->fp16_logmass[i] = 0.0f; }
    }

    // ---- Rung-2 value check
    unsigned char *vm = ws.value_mask + (long)h * ws.ld;
    if (c.values_int4_packed == nullptr || c.values_int4_errors == nullptr) {
        // FP16-value cache: every block reads Tier-2 values.
        for (int b = tid; b < (int)nact; b += SEL_THREADS) vm[b] = 1;
        if (tid == 0) { ct->e_pre = 0.0f; ct->e_val = 0.0f; ct->value_promoted_blocks = 0; }
        return;
    }
    const float *mf = ws.mass_frac + (long)h * ws.ld;
    const float *eta = c.values_int4_errors + (long)kv * c.max_blocks;
    for (int b = tid; b < n_pad; b += SEL_THREADS) {
        vals[b] = b < n ? __fmul_rn(mf[b], eta[b]) : 0.0f;
        mask[b] = 0;
    }
    __syncthreads();
    const float e_pre = block_canonical_sum(vals, n, sh);
    const float excess = fmaxf(__fsub_rn(e_pre, kn.v_tolerance), 0.0f);
    float promoted = 0.0f;
    int n_prom = 0;
    if (kn.value_mode_tight) {
        if (excess > 0.0f) {
            for (int b = tid; b < n_pad; b += SEL_THREADS) keys[b] = b < n ? make_key(vals[b], b) : 0ull;
            __syncthreads();
            bitonic_sort_desc(keys, n_pad);
            if (tid == 0) {
                float cum = 0.0f;
                for (int j = 0; j < n; ++j) {
                    const float v = key_val(keys[j]);
                    cum = j == 0 ? v : __fadd_rn(cum, v);
                    const float cb = __fsub_rn(cum, v);
                    if (!(cb < excess)) break;
                    mask[key_idx(keys[j])] = 1;
                    promoted = cum;
                    ++n_prom;
                }
            }
        }
    } else {
        for (int b = tid; b < n; b += SEL_THREADS) {
            const bool unsafe = eta[b] > kn.v_tolerance;
            mask[b] = unsafe ? 1 : 0;
            if (!unsafe) vals[b] = 0.0f;
        }
        __syncthreads();
        promoted = block_canonical_sum(vals, n, sh);
    }
    __syncthreads();
    int cnt = 0;
    for (int b = tid; b < (int)nact; b += SEL_THREADS) {
        unsigned char m = b < n ? mask[b] : (kn.force_trailing_value_fp16 ? 1 : 0);
        vm[b] = m;
        if (b < n && m) ++cnt;
    }
    if (!kn.value_mode_tight) {
        if (tid == 0) sh.counter = 0;
        __syncthreads();
        if (cnt) atomicAdd(&sh.counter, cnt);
        __syncthreads();
        n_prom = sh.counter;
    }
    if (tid == 0) {
        ct->e_pre = e_pre;
        ct->e_val = fmaxf(__fsub_rn(e_pre, promoted), 0.0f);
        ct->value_promoted_blocks = n_prom;
        if (n_prom > 0) atomicOr(ws.any_flags + 3, 1);
    }
}

static int next_pow2(long n)
{
    int p = 32;
    while (p < n) p <<= 1;
    return p;
}

int select_launch(const cqa_cache *c, const cqa_knobs *kn, const cqa_workspace *ws, long nq, long nact,
                  const float *u, long u_ld, cudaStream_t st)
{
    const int H = c->kv_heads * c->gqa_group;
    if (nq <= 0) { set_error("cqa_select: needs at least one quantised block"); return CQA_ERR_INVALID; }
    if (nq > CQA_MAX_SORT_BLOCKS) {
        set_error("cqa_select: %ld quantised blocks exceed the selector limit %d", nq, CQA_MAX_SORT_BLOCKS);
        return CQA_ERR_TOO_LARGE;
    }
    // Rung-1: one sorted prefix of the expanded width serves both decisions.
    const bool can_expand = kn->rung1_threshold >= 0.0f && kn->k_max > 0;
    long sel_kmax = kn->k_max;
    int two_level = 0;
    if (can_expand) {
        long expanded = (long)ceil((double)kn->k_max * (double)kn->rung1_multiplier);
        if (expanded > nq) expanded = nq;
        if (expanded > kn->k_max) { sel_kmax = expanded; two_level = 1; }
    }
    const int hi = (int)(sel_kmax <= 0 ? nq : (sel_kmax < nq ? sel_kmax : nq));
    const int base_width = two_level ? (int)(kn->k_max < hi ? kn->k_max : hi) : hi;
    if (ws->sel_width < hi) {
        set_error("cqa_select: workspace sel_width %d < required %d", ws->sel_width, hi);
        return CQA_ERR_INVALID;
    }
    const int n_pad = next_pow2(nq);
    const size_t smem = (size_t)n_pad * 13;
    static size_t attr = 0;
    if (smem > attr) {
        int rc = check_cuda(cudaFuncSetAttribute(select_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                 (int)smem),
                            "cudaFuncSetAttribute(select_kernel)");
        if (rc) return rc;
        attr = smem;
    }
    {
        int rc = check_cuda(cudaMemsetAsync(ws->any_flags, 0, 4 * sizeof(int32_t), st), "cudaMemsetAsync(any_flags)");
        if (rc) return rc;
    }
    select_kernel<<<H, SEL_THREADS, smem, st>>>(*c, *kn, *ws, nq, nact, u, u_ld, n_pad, hi, base_width, two_level);
    return check_launch("select_kernel");
}

template <typename T2>
static int certify_launch_t(const cqa_cache *c, const cqa_knobs *kn, const cqa_workspace *ws, const void *q,
                            int q_dtype, long nq, long nact, int rk, cudaStream_t st)
{
    const int H = c->kv_heads * c->gqa_group;
    const int n_pad = next_pow2(nq);
    const size_t smem = (size_t)n_pad * 13;
    static size_t attr = 0;
    if (smem > attr) {
        int rc = check_cuda(cudaFuncSetAttribute(certify_kernel<T2>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                 (int)smem),
                            "cudaFuncSetAttribute(certify_kernel)");
        if (rc) return rc;
        attr = smem;
    }
    certify_kernel<T2><<<H, SEL_THREADS, smem, st>>>(*c, *kn, *ws, q, q_dtype, nq, nact, n_pad, rk);
    return check_launch("certify_kernel");
}

int certify_launch(const cqa_cache *c, const cqa_knobs *kn, const cqa_workspace *ws, const void *q, int q_dtype,
                   long nq, long nact, cudaStream_t st)
{
    if (nq <= 0 || nq > CQA_MAX_SORT_BLOCKS) {
        set_error("cqa_certify: nq=%ld outside [1, %d]", nq, CQA_MAX_SORT_BLOCKS);
        return nq <= 0 ? CQA_ERR_INVALID : CQA_ERR_TOO_LARGE;
    }
    int rk = kn->ranking_r > kn->top_k_fp16_keys ? kn->ranking_r : kn->top_k_fp16_keys;
    if (rk < 4) rk = 4;
    if (rk > nq) rk = (int)nq;
    if (rk > CQA_MAX_RANKING_K - 1) {
        set_error("cqa_certify: ranking set of %d blocks exceeds the limit %d", rk, CQA_MAX_RANKING_K - 1);
        return CQA_ERR_TOO_LARGE;
    }
    const bool need_fp16 = kn->ranking_fallback || kn->score_consistency;
    if (need_fp16 && (!c->keys_t2 || !c->sigma_max)) {
        set_error("cqa_certify: ranking / consistency checks need Tier-2 keys and sigma_max");
        return CQA_ERR_INVALID;
    }
    switch (c->t2_dtype) {
    case CQA_F32: return certify_launch_t<float>(c, kn, ws, q, q_dtype, nq, nact, rk, st);
    case CQA_F16: return certify_launch_t<__half>(c, kn, ws, q, q_dtype, nq, nact, rk, st);
    case CQA_BF16: return certify_launch_t<__nv_bfloat16>(c, kn, ws, q, q_dtype, nq, nact, rk, st);
    }
    set_error("cqa_certify: unknown Tier-2 dtype %d", c->t2_dtype);
    return CQA_ERR_INVALID;
}

}  // namespace cqa
