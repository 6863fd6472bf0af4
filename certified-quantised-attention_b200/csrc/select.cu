// Selector and certifier: one CTA of 1024 threads per query head, everything
// after one round of global loads runs out of shared memory.
//
//   select : block log-masses and mass fractions (canonical sum), the 256
//            heaviest blocks in descending order (ties -> lower block id) by a
//            4-pass radix select plus a one-warp register bitonic sort,
//            sequential cumulative mass, K* with the Rung-1 expansion,
//            exploration draw, FP16-key mask.
//   certify: top-4 blocks by m_b (per-thread lists merged by shuffles), FP16
//            re-score by four warps, Delta, ranking / boundary /
//            score-consistency flags, Rung-2 value check (radix select of the
//            largest mass*eta contributors, sequential greedy prefix; a full
//            block-wide bitonic sort only if 256 contributors are not enough).
//
// cqa_select, cqa_certify and the fused cqa_layer_step all launch the same
// kernel with a phase mask.  Sums over blocks use the canonical order (32
// consecutive values by a warp butterfly, 8 such sums by a butterfly = one
// 256-block leaf, leaves added left to right); prefix sums over the sorted
// order are sequential.
#include "common.cuh"
#include "rescore.cuh"

namespace cqa {

constexpr int SC_THREADS = 1024;
constexpr int SC_WARPS = 32;
constexpr int CAND = 256;          // candidates kept by the radix select
constexpr int PH_SELECT = 1, PH_CERTIFY = 2;

typedef unsigned long long u64;

// Optional phase clocks (compile with -DCQA_PHASE_CLOCKS): thread 0 of every CTA stores the cycle count at
// numbered points; the deltas land in the unused tail of cert[h].fp16_logmass.
#ifdef CQA_PHASE_CLOCKS
#define CQA_CLK(i) do { if (threadIdx.x == 0) phase_clk[i] = clock64(); } while (0)
#else
#define CQA_CLK(i) do { } while (0)
#endif

struct SCShared {
    float red_f[SC_WARPS];
    u64 red_u[SC_WARPS * 4];
    unsigned hist[256];
    float bcast_f[8];
    int bcast_i[8];
    unsigned bcast_u[4];
    int counter;
    int counter2;
};

__device__ __forceinline__ u64 make_key(float v, int idx)
{
    // v >= 0: the bit pattern orders like the value; ties -> lower index first.
    return ((u64)__float_as_uint(v) << 32) | (u64)(0xFFFFFFFFu - (unsigned)idx);
}
__device__ __forceinline__ int key_idx(u64 k) { return (int)(0xFFFFFFFFu - (unsigned)(k & 0xFFFFFFFFull)); }
__device__ __forceinline__ float key_val(u64 k) { return __uint_as_float((unsigned)(k >> 32)); }
__device__ __forceinline__ unsigned orderable(float v)
{
    unsigned u = __float_as_uint(v);
    return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}
__device__ __forceinline__ u64 shfl_xor_u64(u64 v, int m)
{
    unsigned lo = (unsigned)v, hi = (unsigned)(v >> 32);
    lo = __shfl_xor_sync(FULL, lo, m);
    hi = __shfl_xor_sync(FULL, hi, m);
    return ((u64)hi << 32) | lo;
}

__device__ __forceinline__ float block_max(float v, SCShared &sh)
{
    v = warp_max(v);
    const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
    __syncthreads();
    if (l == 0) sh.red_f[w] = v;
    __syncthreads();
    return warp_max(sh.red_f[l]);
}

// Canonical sum of vals[0..n) in shared memory; returns the total to every thread.
// gsum needs ceil(n/32) floats, leaf ceil(n/256).
__device__ __noinline__ float block_canonical_sum(const float *vals, int n, float *gsum, float *leaf, SCShared &sh)
{
    const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
    const int ngroups = (n + 31) >> 5, nleaf = (n + 255) >> 8;
    __syncthreads();
    for (int g = w; g < ngroups; g += SC_WARPS) {
        const int i = g * 32 + l;
        float v = i < n ? vals[i] : 0.0f;
        v = warp_sum(v);
        if (l == 0) gsum[g] = v;
    }
    __syncthreads();
    for (int L = threadIdx.x; L < nleaf; L += SC_THREADS) {
        float p[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) p[i] = (L * 8 + i) < ngroups ? gsum[L * 8 + i] : 0.0f;
#pragma unroll
        for (int s = 4; s >= 1; s >>= 1)
#pragma unroll
            for (int i = 0; i < s; ++i) p[i] = __fadd_rn(p[i], p[i + s]);
        leaf[L] = p[0];
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        float total = 0.0f;
        for (int L = 0; L < nleaf; ++L) total = __fadd_rn(total, leaf[L]);
        sh.bcast_f[0] = total;
    }
    __syncthreads();
    return sh.bcast_f[0];
}

// In-place descending bitonic sort of n_pad (power of two) 64-bit keys by the whole CTA.
__device__ __noinline__ void bitonic_sort_desc(u64 *keys, int n_pad)
{
    for (int k = 2; k <= n_pad; k <<= 1) {
        for (int j = k >> 1; j > 0; j >>= 1) {
            for (int i = threadIdx.x; i < n_pad; i += SC_THREADS) {
                const int ixj = i ^ j;
                if (ixj > i) {
                    const bool desc = (i & k) == 0;
                    const u64 a = keys[i], b = keys[ixj];
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

// One warp sorts 256 keys (descending) held 8 per lane, element index = lane*8 + r: compare-exchange
// distances below 8 stay inside a lane, larger ones cross lanes by shuffles.  Fully unrolled (static
// register indices); called from one place only so the code exists once.
__device__ __noinline__ void warp_sort256_desc(u64 (&e)[8])
{
    const int lane = threadIdx.x & 31;
#pragma unroll
    for (int k = 2; k <= 256; k <<= 1) {
#pragma unroll
        for (int j = k >> 1; j > 0; j >>= 1) {
            if (j >= 8) {
                const int lm = j >> 3;
                const bool lower = (lane & lm) == 0;
#pragma unroll
                for (int r = 0; r < 8; ++r) {
                    const bool desc = (((lane << 3) | r) & k) == 0;
                    const u64 o = shfl_xor_u64(e[r], lm);
                    const bool keep_max = (lower == desc);
                    const bool o_gt = o > e[r];
                    e[r] = (keep_max == o_gt) ? o : e[r];
                }
            } else {
#pragma unroll
                for (int r = 0; r < 8; ++r) {
                    if ((r & j) == 0) {
                        const bool desc = (((lane << 3) | r) & k) == 0;
                        const u64 a = e[r], b = e[r | j];
                        const bool sw = desc ? (a < b) : (a > b);
                        e[r] = sw ? b : a;
                        e[r | j] = sw ? a : b;
                    }
                }
            }
        }
    }
}

// The M = min(CAND, n) largest (value, lower-index-first) entries of vals[0..n), vals >= 0, sorted
// descending into cand[0..CAND) (padding = 0).  Returns M.
__device__ __noinline__ int select_top_sorted(const float *vals, int n, u64 *cand, SCShared &sh)
{
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    __syncthreads();
    if (tid == 0) { sh.counter = 0; sh.counter2 = 0; }
    for (int i = tid; i < CAND; i += SC_THREADS) cand[i] = 0ull;
    __syncthreads();
    const int M = n < CAND ? n : CAND;
    if (n <= CAND) {
        for (int b = tid; b < n; b += SC_THREADS) cand[b] = make_key(vals[b], b);
    } else {
        unsigned prefix = 0u, pmask = 0u;
        int need = M;
        for (int pass = 0; pass < 4; ++pass) {
            const int shift = 24 - 8 * pass;
            if (tid < 256) sh.hist[tid] = 0u;
            __syncthreads();
            for (int b0 = warp * 32; b0 < n; b0 += SC_THREADS) {
                const int b = b0 + lane;
                bool ok = false;
                unsigned digit = 0;
                if (b < n) {
                    const unsigned bits = __float_as_uint(vals[b]);
                    ok = (bits & pmask) == prefix;
                    digit = (bits >> shift) & 255u;
                }
                // one shared-memory atomic per distinct digit in the warp
                const unsigned act = __ballot_sync(FULL, ok);
                if (ok) {
                    const unsigned same = __match_any_sync(act, digit);
                    if (lane == __ffs(same) - 1) atomicAdd(&sh.hist[digit], (unsigned)__popc(same));
                }
            }
            __syncthreads();
            if (warp == 0) {
                // lane l owns bins 8l..8l+7; find the highest bin d with count(bins > d) < need <= count(bins >= d)
                unsigned c[8], tot = 0;
#pragma unroll
                for (int i = 0; i < 8; ++i) { c[i] = sh.hist[lane * 8 + i]; tot += c[i]; }
                unsigned suffix = tot;   // inclusive suffix sum over lanes >= this one
#pragma unroll
                for (int s = 1; s < 32; s <<= 1) {
                    const unsigned o = __shfl_down_sync(FULL, suffix, s);
                    if (lane + s < 32) suffix += o;
                }
                const unsigned above_lane = suffix - tot;   // elements in the bins of higher lanes
                if (above_lane < (unsigned)need && suffix >= (unsigned)need) {
                    unsigned above = above_lane;
                    int d = 7;
                    for (; d > 0; --d) {
                        if (above + c[d] >= (unsigned)need) break;
                        above += c[d];
                    }
                    sh.bcast_u[0] = (unsigned)(lane * 8 + d);
                    sh.bcast_u[1] = above;
                }
            }
            __syncthreads();
            prefix |= sh.bcast_u[0] << shift;
            pmask |= 255u << shift;
            need -= (int)sh.bcast_u[1];
            __syncthreads();
        }
        const unsigned thr = prefix;   // value bits of the M-th largest entry
        const int need_eq = need;      // entries equal to it to take (lowest block ids first)
        int cnt_eq = 0;
        for (int b = tid; b < n; b += SC_THREADS) {
            const unsigned bits = __float_as_uint(vals[b]);
            if (bits > thr) cand[atomicAdd(&sh.counter, 1)] = make_key(vals[b], b);
            else if (bits == thr) ++cnt_eq;
        }
        if (cnt_eq) atomicAdd(&sh.counter2, cnt_eq);
        __syncthreads();
        if (sh.counter2 == need_eq) {
            for (int b = tid; b < n; b += SC_THREADS)
                if (__float_as_uint(vals[b]) == thr) cand[atomicAdd(&sh.counter, 1)] = make_key(vals[b], b);
        } else if (tid == 0) {
            // more equal values than needed (exact ties): take the lowest block ids
            int taken = 0;
            const int base = sh.counter;
            for (int b = 0; b < n && taken < need_eq; ++b)
                if (__float_as_uint(vals[b]) == thr) { cand[base + taken] = make_key(vals[b], b); ++taken; }
        }
    }
    __syncthreads();
    if (warp == 0) {
        u64 e[8];
#pragma unroll
        for (int r = 0; r < 8; ++r) e[r] = cand[lane * 8 + r];
        warp_sort256_desc(e);
#pragma unroll
        for (int r = 0; r < 8; ++r) cand[lane * 8 + r] = e[r];
    }
    __syncthreads();
    return M;
}

// Descending insertion of k into a sorted list of 4.
__device__ __forceinline__ void insert4(u64 (&t)[4], u64 k)
{
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const bool gt = k > t[i];
        const u64 hi = gt ? k : t[i];
        k = gt ? t[i] : k;
        t[i] = hi;
    }
}
// Butterfly merge of per-lane sorted 4-lists: afterwards every lane holds the warp's four largest keys.
__device__ __noinline__ void warp_merge_top4(u64 (&t)[4])
{
#pragma unroll 1
    for (int s = 16; s >= 1; s >>= 1) {
        u64 o[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) o[i] = shfl_xor_u64(t[i], s);
        // keep the 4 largest of two descending lists: max(t[i], o[3-i]) is a bitonic sequence; two more stages sort it
        u64 x[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) x[i] = t[i] > o[3 - i] ? t[i] : o[3 - i];
        u64 a0 = x[0] > x[2] ? x[0] : x[2], a2 = x[0] > x[2] ? x[2] : x[0];
        u64 a1 = x[1] > x[3] ? x[1] : x[3], a3 = x[1] > x[3] ? x[3] : x[1];
        t[0] = a0 > a1 ? a0 : a1;
        t[1] = a0 > a1 ? a1 : a0;
        t[2] = a2 > a3 ? a2 : a3;
        t[3] = a2 > a3 ? a3 : a2;
    }
}

// Dynamic shared memory: A[n_pad] B[n_pad] C[n_pad] (floats), cand[CAND] (u64), cum[CAND], gsum, leaf, mask[n_pad]
// (bytes).  The full-sort fallbacks alias their keys over B and C.
template <typename T2>
__global__ void __launch_bounds__(SC_THREADS) selcert_kernel(cqa_cache c, cqa_knobs kn, cqa_workspace ws, const void *q,
                                                            int q_dtype, long nq, long nact, const float *u, long u_ld,
                                                            int n_pad, int hi, int base_width, int two_level, int rk,
                                                            int phases, int role_base)
{
    extern __shared__ __align__(16) unsigned char dsm[];
    float *A = reinterpret_cast<float *>(dsm);                 // m_b, later mass*eta
    float *B = A + n_pad;                                      // block log-mass ell
    float *C = B + n_pad;                                      // mass, then mass fraction
    u64 *cand = reinterpret_cast<u64 *>(C + n_pad);
    float *cum = reinterpret_cast<float *>(cand + CAND);
    float *gsum = cum + CAND;
    float *leaf = gsum + (n_pad >> 5) + 1;
    unsigned char *mask = reinterpret_cast<unsigned char *>(leaf + (n_pad >> 8) + 2);
    __shared__ SCShared sh;
    __shared__ int top_idx[CQA_MAX_RANKING_K];
    __shared__ float top_i8[CQA_MAX_RANKING_K], top_f16[CQA_MAX_RANKING_K], top_lm[CQA_MAX_RANKING_K];
    __shared__ float s_delta;
    __shared__ u64 s_top[SC_WARPS * 4];

    const int h = blockIdx.x, tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int kv = h / c.gqa_group;
    const int n = (int)nq;
    const float *mb = ws.m_b + (long)h * ws.ld;
    const float *sb = ws.s_b + (long)h * ws.ld;
    float *mf = ws.mass_frac + (long)h * ws.ld;
    cqa_head_cert *ct = ws.cert + h;
    // Three independent roles per head run as separate CTAs (grid.y): 0 = selector, 1 = ranking /
    // boundary / consistency checks, 2 = value check.  Roles 0 and 2 both need the mass fractions and
    // compute them with the same canonical arithmetic, so no CTA waits for another.
    const int role = role_base + (int)blockIdx.y;
    const bool fused = (phases & PH_SELECT) != 0;
    const bool compute_frac = role == 0 || (role == 2 && fused);
    const bool have_int4 = c.values_int4_packed != nullptr && c.values_int4_errors != nullptr;
#ifdef CQA_PHASE_CLOCKS
    long long phase_clk[16];
    for (int i = 0; i < 16; ++i) phase_clk[i] = 0;
#endif
    CQA_CLK(0);

    // ---- one round of global loads, all issued up front: m_b, S_b; the exploration draw (role 0);
    // eta_b and, when only certifying, the mass fractions (role 2)
    const bool explore_on = kn.exploration_rate > 0.0f && u != nullptr;
    const float *eta = have_int4 ? c.values_int4_errors + (long)kv * c.max_blocks : nullptr;
    float mg = -INFINITY;
    for (int b = tid; b < n_pad; b += SC_THREADS) {
        if (b < n) {
            const float m = mb[b];
            const float s = fmaxf(sb[b], 1e-30f);
            unsigned char ebit = 0;
            if (role == 0 && explore_on) ebit = u[(long)h * u_ld + b] < kn.exploration_rate ? 2 : 0;
            if (role == 2) {
                if (!fused) C[b] = mf[b];
                A[b] = eta ? eta[b] : 0.0f;      // role 2 never needs m_b
            } else {
                A[b] = m;
            }
            B[b] = __fadd_rn(clog(s), m);
            mask[b] = ebit;                       // bit 1: exploration candidate, bit 0: selected (set later)
            mg = fmaxf(mg, m);
        } else {
            mask[b] = 0;
        }
    }
    CQA_CLK(1);
    float total = 0.0f;
    if (compute_frac) {
        mg = block_max(mg, sh);
        for (int b = tid; b < n; b += SC_THREADS) C[b] = cexp(__fsub_rn(B[b], mg));
        total = fmaxf(block_canonical_sum(C, n, gsum, leaf, sh), 1e-30f);
        for (int b = tid; b < n_pad; b += SC_THREADS) {
            if (b < n) {
                const float f = __fdiv_rn(C[b], total);
                C[b] = f;
                if (role == 0) mf[b] = f;
            }
        }
    }
    if (role == 0) {
        CQA_CLK(2);
        // the `hi` heaviest blocks, sorted
        int32_t *sidx = ws.sorted_idx + (long)h * ws.sel_width;
        float *scum = ws.sorted_cumsum + (long)h * ws.sel_width;
        const bool narrow = hi <= CAND;
        if (narrow) {
            select_top_sorted(C, n, cand, sh);
            if (tid == 0) {
                // sequential prefix sum, eight values fetched ahead of the dependent adds
                float run = 0.0f;
                for (int j0 = 0; j0 < hi; j0 += 8) {
                    float v[8];
#pragma unroll
                    for (int i = 0; i < 8; ++i) v[i] = key_val(cand[j0 + i]);   // cand is padded to 256
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        run = (j0 + i) == 0 ? v[i] : __fadd_rn(run, v[i]);
                        v[i] = run;
                    }
#pragma unroll
                    for (int i = 0; i < 8; ++i) cum[j0 + i] = v[i];
                }
            }
            __syncthreads();
            for (int j = tid; j < hi; j += SC_THREADS) {
                sidx[j] = key_idx(cand[j]);
                scum[j] = cum[j];
            }
        } else {
            // wide selections (k_max unset or very large): full sort, prefix sums straight to global memory
            u64 *keys = reinterpret_cast<u64 *>(B);   // ell and the fractions are rebuilt below
            __syncthreads();
            for (int b = tid; b < n_pad; b += SC_THREADS) keys[b] = b < n ? make_key(mf[b], b) : 0ull;
            __syncthreads();
            bitonic_sort_desc(keys, n_pad);
            if (tid == 0) {
                float run = 0.0f;
                for (int j = 0; j < hi; ++j) {
                    const float v = key_val(keys[j]);
                    run = j == 0 ? v : __fadd_rn(run, v);
                    scum[j] = run;
                    sidx[j] = key_idx(keys[j]);
                }
            }
            __syncthreads();
        }
        CQA_CLK(3);
        // K*, Rung 1: the prefix sums are non-decreasing, so the first index with cum >= tau is the
        // number of entries below tau (one barrier-wide count each)
        const float *cs = narrow ? cum : scum;
        int ss_e = 0, ss_b = 0;
        {
            int below_e = 0, below_b = 0;
            for (int j = tid; j < hi; j += SC_THREADS) {
                const bool lt = cs[j] < kn.tau_cov;
                below_e += lt ? 1 : 0;
                below_b += (lt && j < base_width) ? 1 : 0;
            }
            if (hi <= SC_THREADS) {
                ss_e = __syncthreads_count(below_e);
                ss_b = __syncthreads_count(below_b);
            } else {
                if (tid == 0) { sh.counter = 0; sh.counter2 = 0; }
                __syncthreads();
                if (below_e) atomicAdd(&sh.counter, below_e);
                if (below_b) atomicAdd(&sh.counter2, below_b);
                __syncthreads();
                ss_e = sh.counter;
                ss_b = sh.counter2;
                __syncthreads();
            }
        }
        if (tid == 0) {
            const int lo_e = min(kn.k_min, hi);
            const int k_e = min(max(ss_e + 1, lo_e), hi);
            const float ta_e = cs[k_e - 1];
            const float tl_e = fmaxf(__fsub_rn(1.0f, ta_e), 0.0f);
            int k_star = k_e, trig = 0, k_b = k_e;
            float ta = ta_e, tl = tl_e;
            if (two_level) {
                const int lo_b = min(kn.k_min, base_width);
                k_b = min(max(ss_b + 1, lo_b), base_width);
                const float ta_b = cs[k_b - 1];
                const float tl_b = fmaxf(__fsub_rn(1.0f, ta_b), 0.0f);
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
            sh.counter = 0;
            if (trig) atomicOr(ws.any_flags + 0, 1);
        }
        __syncthreads();
        const int k_star = sh.bcast_i[0];
        if (narrow) {
            for (int j = tid; j < k_star; j += SC_THREADS) mask[key_idx(cand[j])] |= 1;
        } else {
            for (int j = tid; j < k_star; j += SC_THREADS) mask[sidx[j]] |= 1;
        }
        __syncthreads();
        CQA_CLK(4);
        unsigned char *tm = ws.topk_mask + (long)h * ws.ld;
        unsigned char *em = ws.explore_mask + (long)h * ws.ld;
        int explored = 0;
        for (int b = tid; b < (int)nact; b += SC_THREADS) {
            unsigned char m = 1, e = 0;
            if (b < n) {
                const unsigned char mk = mask[b];
                m = mk & 1;
                if (!m && (mk & 2)) { m = 1; e = 1; ++explored; }
            }
            tm[b] = m;
            em[b] = e;
        }
        if (explored) atomicAdd(&sh.counter, explored);
        __syncthreads();
        if (tid == 0) ct->exploration_blocks = sh.counter;
        if (!narrow) {
            // the full sort overwrote ell and the fractions: rebuild them (each thread re-reads what it wrote)
            for (int b = tid; b < n; b += SC_THREADS) {
                B[b] = __fadd_rn(clog(fmaxf(sb[b], 1e-30f)), A[b]);
                C[b] = mf[b];
            }
        }
    }
    CQA_CLK(5);
    if (role == 0) return;
    __syncthreads();

    // ---- ranking / boundary / score consistency
    const bool need_fp16 = (kn.ranking_fallback || kn.score_consistency) && n > 0;
    if (role == 1 && need_fp16) {
        if (rk <= 4) {
            u64 t4[4] = {0ull, 0ull, 0ull, 0ull};
            for (int b = tid; b < n; b += SC_THREADS)
                insert4(t4, ((u64)orderable(A[b]) << 32) | (u64)(0xFFFFFFFFu - (unsigned)b));
            warp_merge_top4(t4);
            if (lane == 0) {
#pragma unroll
                for (int i = 0; i < 4; ++i) s_top[warp * 4 + i] = t4[i];
            }
            __syncthreads();
            if (warp == 0) {
#pragma unroll
                for (int i = 0; i < 4; ++i) t4[i] = s_top[lane * 4 + i];
                warp_merge_top4(t4);
                if (lane == 0) {
                    for (int r = 0; r < rk; ++r) {
                        top_idx[r] = key_idx(t4[r]);
                        top_i8[r] = A[key_idx(t4[r])];
                    }
                }
            }
        } else {
            u64 prev = ~0ull;
            for (int r = 0; r < rk; ++r) {
                u64 best = 0ull;
                for (int b = tid; b < n; b += SC_THREADS) {
                    const u64 k = ((u64)orderable(A[b]) << 32) | (u64)(0xFFFFFFFFu - (unsigned)b);
                    if (k < prev && k > best) best = k;
                }
#pragma unroll
                for (int s = 16; s >= 1; s >>= 1) {
                    const u64 o = shfl_xor_u64(best, s);
                    best = o > best ? o : best;
                }
                __syncthreads();
                if (lane == 0) sh.red_u[warp] = best;
                __syncthreads();
                best = sh.red_u[lane];
#pragma unroll
                for (int s = 16; s >= 1; s >>= 1) {
                    const u64 o = shfl_xor_u64(best, s);
                    best = o > best ? o : best;
                }
                if (tid == 0) {
                    top_idx[r] = key_idx(best);
                    top_i8[r] = A[key_idx(best)];
                }
                prev = best;
            }
        }
        __syncthreads();
        CQA_CLK(6);
        if (warp < rk) {
            float s, lm;
            fp16_block_score_warp<T2>(c, q, q_dtype, h, (long)top_idx[warp], nq * BS, kn.q_scale, s, lm);
            if (lane == 0) { top_f16[warp] = s; top_lm[warp] = lm; }
        } else if (warp == rk) {
            const float d = delta_bound_warp(c, q, q_dtype, h);
            if (lane == 0) s_delta = d;
        }
        __syncthreads();
        CQA_CLK(7);
        const float delta = s_delta;
        float ub = -INFINITY;
        if (kn.ranking_fallback) {
            for (int b = tid; b < n; b += SC_THREADS) {
                bool in_top = false;
                for (int r = 0; r < rk; ++r) in_top |= (top_idx[r] == b);
                if (!in_top) ub = fmaxf(ub, __fadd_rn(B[b], delta));
            }
            ub = block_max(ub, sh);
        }
        CQA_CLK(8);
        if (tid == 0) {
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
            int dis_main = 0, dis_r1 = 0, dis_r3 = 0, boundary = 0, violation = 0;
            float ell_r = -INFINITY;
            if (kn.ranking_fallback) {
                const int r_main = min(kn.ranking_r, rk);
                for (int p = 0; p < rk; ++p) {
                    const bool d = rank16[p] != p;
                    if (p < r_main) dis_main |= d;
                    if (p < 1) dis_r1 |= d;
                    if (p < 3) dis_r3 |= d;
                }
                float tmp[CQA_MAX_RANKING_K];
                for (int i = 0; i < rk; ++i) tmp[i] = top_lm[i];
                for (int p = 0; p < r_main; ++p) {
                    int bi = p;
                    for (int i = p + 1; i < rk; ++i)
                        if (tmp[i] > tmp[bi]) bi = i;
                    const float t = tmp[p]; tmp[p] = tmp[bi]; tmp[bi] = t;
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
            const int rung3 = (dis_main | boundary) ? 1 : 0;
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
            if (ct->dense) {
                const int slot = atomicAdd(ws.any_flags + 4, 1);
                ws.any_flags[5 + slot] = h;
            }
            if (rung3) atomicOr(ws.any_flags + 1, 1);
            if (violation) atomicOr(ws.any_flags + 2, 1);
        }
    } else if (role == 1 && tid == 0) {
        ct->ranking_disagree = ct->ranking_disagree_r1 = ct->ranking_disagree_r3 = 0;
        ct->boundary_triggered = ct->rung3 = ct->consistency_violation = ct->dense = 0;
        ct->delta = 0.0f;
        ct->boundary_ub = -INFINITY;
        ct->ell_fp16_r = -INFINITY;
        ct->fp16_top1 = ct->fp16_top2 = ct->int8_top1 = 0.0f;
        for (int i = 0; i < CQA_MAX_RANKING_K; ++i) { ct->top_blocks[i] = -1; ct->fp16_scores[i] = 0.0f; ct->fp16_logmass[i] = 0.0f; }
    }

    CQA_CLK(9);
    if (role == 1) return;
    // ---- Rung-2 value check
    unsigned char *vm = ws.value_mask + (long)h * ws.ld;
    if (!have_int4) {
        for (int b = tid; b < (int)nact; b += SC_THREADS) vm[b] = 1;   // FP16-value cache: every block reads Tier 2
        if (tid == 0) { ct->e_pre = 0.0f; ct->e_val = 0.0f; ct->value_promoted_blocks = 0; }
        return;
    }
    __syncthreads();
    for (int b = tid; b < n_pad; b += SC_THREADS) {
        A[b] = b < n ? __fmul_rn(C[b], A[b]) : 0.0f;   // A held eta_b
        mask[b] = 0;
    }
    CQA_CLK(10);
    const float e_pre = block_canonical_sum(A, n, gsum, leaf, sh);
    CQA_CLK(11);
    const float excess = fmaxf(__fsub_rn(e_pre, kn.v_tolerance), 0.0f);
    if (tid == 0) { sh.bcast_f[1] = 0.0f; sh.bcast_i[1] = 0; sh.bcast_i[2] = 1; }
    if (kn.value_mode_tight) {
        if (excess > 0.0f) {
            // greedy promotion over the descending order: the 256 largest contributors first
            const int M = select_top_sorted(A, n, cand, sh);
            CQA_CLK(12);
            if (tid == 0) {
                float run = 0.0f, promoted = 0.0f;
                int n_prom = 0, done = 0;
                for (int j = 0; j < M; ++j) {
                    const float v = key_val(cand[j]);
                    run = j == 0 ? v : __fadd_rn(run, v);
                    if (!(__fsub_rn(run, v) < excess)) { done = 1; break; }
                    mask[key_idx(cand[j])] = 1;
                    promoted = run;
                    ++n_prom;
                }
                if (M == n) done = 1;
                sh.bcast_f[1] = promoted;
                sh.bcast_i[1] = n_prom;
                sh.bcast_i[2] = done;
            }
            __syncthreads();
            if (!sh.bcast_i[2]) {
                // 256 contributors were not enough: sort everything and walk the whole order
                u64 *keys = reinterpret_cast<u64 *>(B);
                for (int b = tid; b < n_pad; b += SC_THREADS) keys[b] = b < n ? make_key(A[b], b) : 0ull;
                __syncthreads();
                bitonic_sort_desc(keys, n_pad);
                if (tid == 0) {
                    float run = 0.0f, promoted = 0.0f;
                    int n_prom = 0;
                    for (int j = 0; j < n; ++j) {
                        const float v = key_val(keys[j]);
                        run = j == 0 ? v : __fadd_rn(run, v);
                        if (!(__fsub_rn(run, v) < excess)) break;
                        mask[key_idx(keys[j])] = 1;
                        promoted = run;
                        ++n_prom;
                    }
                    sh.bcast_f[1] = promoted;
                    sh.bcast_i[1] = n_prom;
                }
            }
        }
    } else {
        __syncthreads();
        int cnt = 0;
        for (int b = tid; b < n; b += SC_THREADS) {
            const bool unsafe = eta[b] > kn.v_tolerance;
            mask[b] = unsafe ? 1 : 0;
            if (!unsafe) A[b] = 0.0f; else ++cnt;
        }
        if (tid == 0) sh.counter = 0;
        __syncthreads();
        if (cnt) atomicAdd(&sh.counter, cnt);
        const float promoted = block_canonical_sum(A, n, gsum, leaf, sh);
        if (tid == 0) { sh.bcast_f[1] = promoted; sh.bcast_i[1] = sh.counter; }
    }
    __syncthreads();
    CQA_CLK(13);
    for (int b = tid; b < (int)nact; b += SC_THREADS)
        vm[b] = b < n ? mask[b] : (kn.force_trailing_value_fp16 ? 1 : 0);
    if (tid == 0) {
        ct->e_pre = e_pre;
        ct->e_val = fmaxf(__fsub_rn(e_pre, sh.bcast_f[1]), 0.0f);
        ct->value_promoted_blocks = sh.bcast_i[1];
        if (sh.bcast_i[1] > 0) atomicOr(ws.any_flags + 3, 1);
#ifdef CQA_PHASE_CLOCKS
        phase_clk[14] = clock64();
        for (int i = 1; i < 15; ++i) ct->fp16_logmass[16 + i] = phase_clk[i] ? (float)(phase_clk[i] - phase_clk[0]) : 0.0f;
#endif
    }
}

static int next_pow2(long n)
{
    int p = 32;
    while (p < n) p <<= 1;
    return p;
}

static size_t selcert_smem(int n_pad)
{
    return (size_t)n_pad * 13 + (size_t)CAND * 12 + ((size_t)(n_pad >> 5) + 1 + (n_pad >> 8) + 2) * 4 + 64;
}

template <typename T2>
static int selcert_launch_t(const cqa_cache *c, const cqa_knobs *kn, const cqa_workspace *ws, const void *q,
                            int q_dtype, long nq, long nact, const float *u, long u_ld, int phases,
                            cudaStream_t st)
{
    const int H = c->kv_heads * c->gqa_group;
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
    if ((phases & PH_SELECT) && ws->sel_width < hi) {
        set_error("cqa_select: workspace sel_width %d < required %d", ws->sel_width, hi);
        return CQA_ERR_INVALID;
    }
    int rk = kn->ranking_r > kn->top_k_fp16_keys ? kn->ranking_r : kn->top_k_fp16_keys;
    if (rk < 4) rk = 4;
    if (rk > nq) rk = (int)nq;
    if (rk > CQA_MAX_RANKING_K - 1) {
        set_error("cqa_certify: ranking set of %d blocks exceeds the limit %d", rk, CQA_MAX_RANKING_K - 1);
        return CQA_ERR_TOO_LARGE;
    }
    const int n_pad = next_pow2(nq);
    const size_t smem = selcert_smem(n_pad);
    static size_t attr = 0;
    if (smem > attr) {
        int rc = check_cuda(cudaFuncSetAttribute(selcert_kernel<T2>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                 (int)smem),
                            "cudaFuncSetAttribute(selcert_kernel)");
        if (rc) return rc;
        attr = smem;
    }
    if (phases & PH_SELECT) {
        int rc = check_cuda(cudaMemsetAsync(ws->any_flags, 0, (5 + H) * sizeof(int32_t), st),
                            "cudaMemsetAsync(any_flags)");
        if (rc) return rc;
    }
    // select only: role 0; certify only: roles 1 and 2; fused: all three
    const int role_base = (phases & PH_SELECT) ? 0 : 1;
    const int n_roles = phases == (PH_SELECT | PH_CERTIFY) ? 3 : (phases == PH_SELECT ? 1 : 2);
    dim3 grid((unsigned)H, (unsigned)n_roles);
    selcert_kernel<T2><<<grid, SC_THREADS, smem, st>>>(*c, *kn, *ws, q, q_dtype, nq, nact, u, u_ld, n_pad, hi,
                                                       base_width, two_level, rk, phases, role_base);
    return check_launch("selcert_kernel");
}

int selcert_launch(const cqa_cache *c, const cqa_knobs *kn, const cqa_workspace *ws, const void *q, int q_dtype,
                   long nq, long nact, const float *u, long u_ld, int phases, cudaStream_t st)
{
    if (nq <= 0) { set_error("selector: needs at least one quantised block"); return CQA_ERR_INVALID; }
    if (nq > CQA_MAX_SORT_BLOCKS) {
        set_error("selector: %ld quantised blocks exceed the limit %d", nq, CQA_MAX_SORT_BLOCKS);
        return CQA_ERR_TOO_LARGE;
    }
    if (phases & PH_CERTIFY) {
        const bool need_fp16 = kn->ranking_fallback || kn->score_consistency;
        if (need_fp16 && (!c->keys_t2 || !c->sigma_max || !q)) {
            set_error("cqa_certify: ranking / consistency checks need q, Tier-2 keys and sigma_max");
            return CQA_ERR_INVALID;
        }
    }
    switch (c->t2_dtype) {
    case CQA_F32: return selcert_launch_t<float>(c, kn, ws, q, q_dtype, nq, nact, u, u_ld, phases, st);
    case CQA_F16: return selcert_launch_t<__half>(c, kn, ws, q, q_dtype, nq, nact, u, u_ld, phases, st);
    case CQA_BF16: return selcert_launch_t<__nv_bfloat16>(c, kn, ws, q, q_dtype, nq, nact, u, u_ld, phases, st);
    }
    set_error("selector: unknown Tier-2 dtype %d", c->t2_dtype);
    return CQA_ERR_INVALID;
}

int select_launch(const cqa_cache *c, const cqa_knobs *kn, const cqa_workspace *ws, long nq, long nact,
                  const float *u, long u_ld, cudaStream_t st)
{
    return selcert_launch(c, kn, ws, nullptr, CQA_F32, nq, nact, u, u_ld, PH_SELECT, st);
}

int certify_launch(const cqa_cache *c, const cqa_knobs *kn, const cqa_workspace *ws, const void *q, int q_dtype,
                   long nq, long nact, cudaStream_t st)
{
    return selcert_launch(c, kn, ws, q, q_dtype, nq, nact, nullptr, 0, PH_CERTIFY, st);
}

}  // namespace cqa
