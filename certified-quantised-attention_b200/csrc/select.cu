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
// Sequence-sharded runs split the ranking check around an exchange: PH_TOP_ONLY stops role 1 once the top
// list is in the certificate; PH_GIVEN resumes it from that list with FP16 scores computed by the ranks that
// own the blocks (ws.given_fp16) and runs role 1 alone.
constexpr int PH_TOP_ONLY = 4, PH_GIVEN = 8;
constexpr int PH_FLAGS_CLEARED = 16;   // the caller already zeroed ws.any_flags on this stream
constexpr int PH_PEER_B = 64;          // role 1 exchanges the FP16 re-scores with the other ranks itself (ws.peer_*)

typedef unsigned long long u64;

// Optional phase clocks (compile with -DCQA_PHASE_CLOCKS): thread 0 of every CTA stores the cycle count at
// numbered points; the deltas land in the unused tail of cert[h].fp16_logmass.
#ifdef CQA_PHASE_CLOCKS
#define CQA_CLK(i) do { if (threadIdx.x == 0) phase_clk[i] = clock64(); } while (0)
#define CQA_CLK_FLUSH(lo, hi) do { if (threadIdx.x == 0) for (int i_ = (lo); i_ <= (hi); ++i_) \
    ct->fp16_logmass[16 + i_] = (float)(phase_clk[i_] - phase_clk[0]); } while (0)
#define CQA_LM_ROWS 16
#define CQA_DBG(i) do { if (threadIdx.x == 0) sh.dbg[i] = clock64(); } while (0)
#else
#define CQA_CLK(i) do { } while (0)
#define CQA_DBG(i) do { } while (0)
#define CQA_CLK_FLUSH(lo, hi) do { } while (0)
#define CQA_LM_ROWS CQA_MAX_RANKING_K
#endif

// One uniform in [0, 1) per (block, head, call): Philox4x32-10 on the counter (block, head, offset) under `seed`.
__device__ __forceinline__ float philox_uniform(unsigned long long seed, unsigned long long offset, unsigned head,
                                                unsigned block)
{
    unsigned c0 = block, c1 = head, c2 = (unsigned)offset, c3 = (unsigned)(offset >> 32);
    unsigned k0 = (unsigned)seed, k1 = (unsigned)(seed >> 32);
#pragma unroll
    for (int r = 0; r < 10; ++r) {
        const unsigned hi0 = __umulhi(0xD2511F53u, c0), lo0 = 0xD2511F53u * c0;
        const unsigned hi1 = __umulhi(0xCD9E8D57u, c2), lo1 = 0xCD9E8D57u * c2;
        const unsigned n0 = hi1 ^ c1 ^ k0, n2 = hi0 ^ c3 ^ k1;
        c0 = n0; c1 = lo1; c2 = n2; c3 = lo0;
        k0 += 0x9E3779B9u;
        k1 += 0xBB67AE85u;
    }
    return (float)(c0 >> 8) * 5.9604644775390625e-08f;   // 2^-24
}

struct SCShared {
    float red_f[SC_WARPS];
    u64 red_u[SC_WARPS * 4];
    int red_i[2][SC_WARPS];
    unsigned char rank_part[4][CAND];
    float vs_f[2][8];
    int vs_i[2][8];
    unsigned short rank_pos[CAND];
#ifdef CQA_PHASE_CLOCKS
    long long dbg[8];
#endif
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

// Sort the CAND keys of cand[] in place, descending, by rank counting: four threads (in four different
// warps) share one key and count the keys above it in a quarter of the list each; every warp reads one
// list entry at a time (a broadcast).  Real keys are distinct and non-zero; zero is padding and ends up
// behind them.
__device__ __forceinline__ void rank_sort_desc(u64 *cand, SCShared &sh)
{
    static_assert(CAND * 4 == SC_THREADS, "one key per four threads");
    const int tid = threadIdx.x;
    const int cidx = tid & (CAND - 1), part = tid >> 8;
    const u64 key = cand[cidx];
    const u64 *seg = cand + part * (CAND / 4);
    int above = 0;
#pragma unroll 8
    for (int j = 0; j < CAND / 4; ++j) above += seg[j] > key ? 1 : 0;
    sh.rank_part[part][cidx] = (unsigned char)above;   // at most 64
    __syncthreads();
    if (part == 0) {
        const int pos = (int)sh.rank_part[0][cidx] + sh.rank_part[1][cidx] + sh.rank_part[2][cidx] + sh.rank_part[3][cidx];
        cand[cidx] = 0ull;
        sh.rank_pos[cidx] = (unsigned short)pos;
    }
    __syncthreads();
    if (part == 0 && key != 0ull) cand[sh.rank_pos[cidx]] = key;
    __syncthreads();
}

// Sum of one int per thread over the CTA with a single barrier: per-warp sums go to one of two
// alternating rows of sh.red_i, so the next call never overwrites a row that is still being read.
__device__ __forceinline__ int block_sum_int(int v, SCShared &sh, int parity)
{
    const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
    v = __reduce_add_sync(FULL, v);
    if (l == 0) sh.red_i[parity][w] = v;
    __syncthreads();
    return __reduce_add_sync(FULL, sh.red_i[parity][l]);
}

// Named barrier for the first VS_THREADS threads of the CTA (the rest do not take part).
constexpr int VS_THREADS = 256, VS_WARPS = VS_THREADS / 32;
__device__ __forceinline__ void vs_barrier() { asm volatile("bar.sync 1, %0;" ::"n"(VS_THREADS) : "memory"); }

// "Column sum" of the entries of vals[0..n) that `pred(bits, index)` admits, and their number; called by
// threads 0..VS_THREADS-1 only, result in every one of them.  Fixed order: thread t adds its entries
// t, t+256, t+512, ... in ascending order; the 32 columns of a warp are combined by the butterfly
// 16,8,4,2,1; the 8 warp sums by the butterfly 4,2,1.  Adding an admitted entry never lowers the result
// (every step is a monotone rounding), which is what the threshold search below relies on.
template <typename Pred>
__device__ __forceinline__ float column_sum(const float *vals, int n, Pred pred, SCShared &sh, int &parity, int &count)
{
    const int tid = threadIdx.x, lane = tid & 31, w = tid >> 5;
    float s = 0.0f;
    int c = 0;
    for (int b = tid; b < n; b += VS_THREADS) {
        const float v = vals[b];
        if (pred(__float_as_uint(v), b)) { s = __fadd_rn(s, v); ++c; }
    }
    s = warp_sum(s);
    c = __reduce_add_sync(FULL, c);
    if (lane == 0) { sh.vs_f[parity][w] = s; sh.vs_i[parity][w] = c; }
    vs_barrier();
    float x = lane < VS_WARPS ? sh.vs_f[parity][lane] : 0.0f;
    int y = lane < VS_WARPS ? sh.vs_i[parity][lane] : 0;
    parity ^= 1;
    x = __fadd_rn(x, __shfl_xor_sync(FULL, x, 4));
    x = __fadd_rn(x, __shfl_xor_sync(FULL, x, 2));
    x = __fadd_rn(x, __shfl_xor_sync(FULL, x, 1));
    count = __reduce_add_sync(FULL, y);
    return __shfl_sync(FULL, x, 0);
}

// The M = min(CAND, n) largest (value, lower-index-first) entries of vals[0..n), vals >= 0, sorted
// descending into cand[0..CAND) (padding = 0).  Returns M.
//
// The value of the M-th largest entry is found bit by bit (most significant first): a bit is kept when
// at least M entries are >= the candidate threshold.  Each step is one pass over the values and one
// barrier, with no shared-memory atomics, and the search stops as soon as a threshold separates exactly
// M entries.  Entries above the threshold are then compacted and ordered by rank counting.
__device__ __noinline__ int select_top_sorted(const float *vals, int n, u64 *cand, SCShared &sh)
{
    const int tid = threadIdx.x, lane = tid & 31;
    CQA_DBG(0);
    __syncthreads();
    CQA_DBG(1);
    if (tid == 0) sh.counter = 0;
    for (int i = tid; i < CAND; i += SC_THREADS) cand[i] = 0ull;
    const int M = n < CAND ? n : CAND;
    if (n <= CAND) {
        __syncthreads();
        for (int b = tid; b < n; b += SC_THREADS) cand[b] = make_key(vals[b], b);
    } else {
        unsigned thr = 0u;
        int n_ge = n;            // entries >= thr
        int parity = 0;
        const int w = tid >> 5;
        // Two bits per step: three candidate thresholds are counted at once.  Only the first 256 threads search
        // (named barrier): a step is a short dependent chain, and with all 32 warps the issue slots of their
        // bookkeeping cost more than the shorter element loops save.
        if (tid < VS_THREADS) {
#pragma unroll 1
            for (int bit = 30; bit >= 0 && n_ge != M; bit -= 2) {
                const bool single = bit == 0;                 // 31 value bits: the last step decides one bit
                const int lo = single ? 0 : bit - 1;
                const unsigned t1 = thr | (1u << lo);                              // 01 (or 1)
                const unsigned t2 = single ? 0xFFFFFFFFu : thr | (2u << lo);       // 10
                const unsigned t3 = single ? 0xFFFFFFFFu : thr | (3u << lo);       // 11
                unsigned l12 = 0, l3 = 0;                     // a thread holds at most 64 entries
                for (int b = tid; b < n; b += VS_THREADS) {
                    const unsigned v = __float_as_uint(vals[b]);
                    l12 += (v >= t1 ? 1u : 0u) + (v >= t2 ? 1u << 16 : 0u);
                    l3 += v >= t3 ? 1u : 0u;
                }
                l12 = __reduce_add_sync(FULL, l12);
                l3 = __reduce_add_sync(FULL, l3);
                if (lane == 0) { sh.vs_i[parity][w] = (int)l12; sh.red_i[parity][w] = (int)l3; }
                vs_barrier();
                const unsigned p12 = lane < VS_WARPS ? (unsigned)sh.vs_i[parity][lane] : 0u;
                const unsigned p3 = lane < VS_WARPS ? (unsigned)sh.red_i[parity][lane] : 0u;
                parity ^= 1;
                const unsigned c12 = __reduce_add_sync(FULL, p12);   // totals stay below 2^15 per field
                const int c3 = (int)__reduce_add_sync(FULL, p3);
                const int c1 = (int)(c12 & 0xFFFFu), c2 = (int)(c12 >> 16);
                if (!single && c3 >= M) { thr = t3; n_ge = c3; }
                else if (!single && c2 >= M) { thr = t2; n_ge = c2; }
                else if (c1 >= M) { thr = t1; n_ge = c1; }
            }
            if (tid == 0) { sh.bcast_u[1] = thr; sh.bcast_i[4] = n_ge; }
        }
        __syncthreads();
        thr = sh.bcast_u[1];
        n_ge = sh.bcast_i[4];
        parity = 0;
        // n_ge == M: the entries >= thr are the answer.  Otherwise thr is the value of the M-th largest
        // entry and several entries equal it: take everything above, then the lowest block ids among the equal.
        const bool ties = n_ge != M;
        CQA_DBG(2);
        __syncthreads();   // cand is zeroed, sh.counter is 0
        for (int b0 = tid - lane; b0 < n; b0 += SC_THREADS) {
            const int b = b0 + lane;
            const unsigned bits = b < n ? __float_as_uint(vals[b]) : 0u;
            const bool take = b < n && (ties ? bits > thr : bits >= thr);
            const unsigned who = __ballot_sync(FULL, take);
            if (who) {
                int base = 0;
                if (lane == 0) base = atomicAdd(&sh.counter, __popc(who));
                base = __shfl_sync(FULL, base, 0);
                if (take) cand[base + __popc(who & ((1u << lane) - 1u))] = make_key(vals[b], b);
            }
        }
        CQA_DBG(3);
        if (ties) {
            // entries equal to the threshold fill the remaining places in block order: an ordered compaction,
            // 1024 consecutive blocks per round (per-warp counts, then an exclusive scan over the warps)
            __syncthreads();
            int taken = sh.counter;
            for (int b0 = 0; b0 < n && taken < M; b0 += SC_THREADS) {
                const int b = b0 + tid;
                const bool eq = b < n && __float_as_uint(vals[b]) == thr;
                const unsigned who = __ballot_sync(FULL, eq);
                if (lane == 0) sh.red_i[parity][w] = __popc(who);
                __syncthreads();
                const int cw = sh.red_i[parity][lane];
                parity ^= 1;
                int incl = cw;   // inclusive scan of the per-warp counts
#pragma unroll
                for (int o = 1; o < 32; o <<= 1) {
                    const int v = __shfl_up_sync(FULL, incl, o);
                    if (lane >= o) incl += v;
                }
                const int before = __shfl_sync(FULL, incl - cw, w);
                const int pos = taken + before + __popc(who & ((1u << lane) - 1u));
                if (eq && pos < M) cand[pos] = make_key(vals[b], b);
                taken += __shfl_sync(FULL, incl, 31);
            }
        }
    }
    __syncthreads();
    CQA_DBG(4);
    rank_sort_desc(cand, sh);
    CQA_DBG(5);
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
// The four largest keys held by a warp, given one descending 4-list per lane (keys distinct, zero is
// padding): four rounds of a warp-wide maximum over the list heads; the lane that wins pops its list.
__device__ __forceinline__ void warp_top4(u64 (&t)[4], u64 (&out)[4])
{
#pragma unroll
    for (int r = 0; r < 4; ++r) {
        u64 best = t[0];
#pragma unroll
        for (int s = 16; s >= 1; s >>= 1) {
            const u64 o = shfl_xor_u64(best, s);
            best = o > best ? o : best;
        }
        out[r] = best;
        if (t[0] == best) { t[0] = t[1]; t[1] = t[2]; t[2] = t[3]; t[3] = 0ull; }
    }
}

// Dynamic shared memory: A[n_pad] B[n_pad] C[n_pad] (floats), cand[CAND] (u64), cum[CAND], gsum, leaf, mask[n_pad]
// (bytes).  The full-sort fallbacks alias their keys over B and C.
#ifdef CQA_WARM_REPEAT
#define CQA_BODY_QUAL __device__ __noinline__   // instrumentation: the body runs twice, the second time with warm code
#else
#define CQA_BODY_QUAL __device__ __forceinline__
#endif
template <typename T2>
CQA_BODY_QUAL void selcert_body(const cqa_cache &c, const cqa_knobs &kn, const cqa_workspace &ws, const void *q,
                                int q_dtype, long nq, long nact, const float *u, long u_ld, int n_pad, int hi,
                                int base_width, int two_level, int rk, int phases, int role_base)
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
    // Plain layout: row h of an [H][ld] array.  Sharded layout: row h of rank r's slot in the all-gather buffer,
    // [rank][row][chunk]; `gcol` maps a global block to its offset from the row start of rank 0.
    const bool sharded_in = ws.shard_stride > 0;
    const long row_ld = sharded_in ? ws.shard_chunk : ws.ld;
    const float *mb = ws.m_b + (long)h * row_ld;
    const float *sb = ws.s_b + (long)h * row_ld;
    auto gcol = [&](int b) -> long {
        if (!sharded_in) return b;
        long r = b / ws.shard_stride;
        if (r > ws.shard_ranks - 1) r = ws.shard_ranks - 1;
        return r * ws.shard_rank_stride + (b - r * ws.shard_stride);
    };
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
    const bool explore_on = kn.exploration_rate > 0.0f;
    const float *eta = have_int4 ? c.values_int4_errors + (long)kv * (sharded_in ? ws.shard_chunk : c.max_blocks) : nullptr;
    float mg = -INFINITY;
    // four blocks per thread and round: all global loads of a round are issued before any is used
    for (int b0 = tid; b0 < n_pad; b0 += 4 * SC_THREADS) {
        float m4[4], s4[4], x4[4];
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const int b = b0 + k * SC_THREADS;
            m4[k] = 0.0f; s4[k] = 1.0f; x4[k] = 0.0f;
            if (b < n) {
                const long gb = gcol(b);
                m4[k] = mb[gb];
                s4[k] = sb[gb];
                if (role == 0) {
                    if (explore_on && u != nullptr) x4[k] = u[(long)h * u_ld + b];
                } else if (role == 2) {
                    x4[k] = eta ? eta[gb] : 0.0f;
                }
            }
        }
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const int b = b0 + k * SC_THREADS;
            if (b >= n_pad) continue;
            if (b < n) {
                const float m = m4[k];
                const float s = fmaxf(s4[k], 1e-30f);
                unsigned char ebit = 0;
                if (role == 0 && explore_on) {
                    const float uv = u != nullptr ? x4[k]
                                                  : philox_uniform(ws.rng_seed, ws.rng_offset, (unsigned)h, (unsigned)b);
                    ebit = uv < kn.exploration_rate ? 2 : 0;
                }
                if (role == 2) {
                    if (!fused) C[b] = mf[b];
                    A[b] = x4[k];                     // eta_b: role 2 never needs m_b
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
                B[b] = __fadd_rn(clog(fmaxf(sb[gcol(b)], 1e-30f)), A[b]);
                C[b] = mf[b];
            }
        }
    }
    CQA_CLK(5);
    if (role == 0) { CQA_CLK_FLUSH(1, 5); return; }
    __syncthreads();

    // ---- ranking / boundary / score consistency
    const bool need_fp16 = (kn.ranking_fallback || kn.score_consistency) && n > 0;
    if (role == 1 && need_fp16) {
        const bool given = (phases & PH_GIVEN) != 0;
        if (given) {
            if (tid < rk) {
                const int b = ct->top_blocks[tid];
                top_idx[tid] = b;
                top_i8[tid] = A[b];
                // one array per rank when the re-scores were pushed (only a block's owner wrote non-zero values)
                float gs = 0.0f, gl = 0.0f;
                const int gr = ws.given_ranks > 1 ? ws.given_ranks : 1;
                for (int r = 0; r < gr; ++r) {
                    const float *g = ws.given_fp16 + r * ws.given_rank_stride + ((long)h * CQA_MAX_RANKING_K + tid) * 2;
                    gs = __fadd_rn(gs, g[0]);
                    gl = __fadd_rn(gl, g[1]);
                }
                top_f16[tid] = gs;
                top_lm[tid] = gl;
            }
        } else if (rk <= 4) {
            u64 t4[4] = {0ull, 0ull, 0ull, 0ull};
            for (int b = tid; b < n; b += SC_THREADS)
                insert4(t4, ((u64)orderable(A[b]) << 32) | (u64)(0xFFFFFFFFu - (unsigned)b));
            CQA_CLK(15);
            u64 w4[4];
            warp_top4(t4, w4);
            if (lane == 0) {
#pragma unroll
                for (int i = 0; i < 4; ++i) s_top[warp * 4 + i] = w4[i];
            }
            __syncthreads();
            if (warp == 0) {
#pragma unroll
                for (int i = 0; i < 4; ++i) t4[i] = s_top[lane * 4 + i];
                warp_top4(t4, w4);
                if (lane == 0) {
                    for (int r = 0; r < rk; ++r) {
                        top_idx[r] = key_idx(w4[r]);
                        top_i8[r] = A[key_idx(w4[r])];
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
        if (phases & PH_TOP_ONLY) {
            if (tid < CQA_MAX_RANKING_K) ct->top_blocks[tid] = tid < rk ? top_idx[tid] : -1;
            return;
        }
        // Boundary bound: max over the blocks outside the top list of (ell_b + delta).  Rounding is monotone,
        // so it equals (max ell_b) + delta; the maximum is taken by the warps that neither re-score a block
        // nor compute delta, while those wait for Tier-2 rows.
        const int ub_first = rk + 1, ub_warps = SC_WARPS - ub_first;
        const bool overlap = ub_warps >= 8;
        float ubm = -INFINITY;
        const bool peer_b = (phases & PH_PEER_B) != 0;
        if (warp < rk) {
            if (peer_b) {
                // re-score the block if this rank owns it (local block ids), zeros otherwise; every rank gets the row
                const long bl = (long)top_idx[warp] - ws.peer_first_block;
                float s = 0.0f, lm = 0.0f;
                if (bl >= 0 && bl < ws.peer_n_local)
                    fp16_block_score_warp<T2>(c, q, q_dtype, h, bl, ws.peer_n_local * BS, kn.q_scale, s, lm);
                if (lane < ws.peer_world) {
                    float *d = ws.peer_xb[lane] + ((long)h * CQA_MAX_RANKING_K + warp) * 2;
                    d[0] = s;
                    d[1] = lm;
                }
            } else if (!given) {
                float s, lm;
                fp16_block_score_warp<T2>(c, q, q_dtype, h, (long)top_idx[warp], nq * BS, kn.q_scale, s, lm);
                if (lane == 0) { top_f16[warp] = s; top_lm[warp] = lm; }
            }
        } else if (warp == rk) {
            const float d = delta_bound_warp(c, q, q_dtype, h, sharded_in ? ws.shard_ranks : 1, ws.shard_rank_stride);
            if (lane == 0) s_delta = d;
        } else if (overlap && kn.ranking_fallback) {
            for (int b = (warp - ub_first) * 32 + lane; b < n; b += ub_warps * 32) {
                bool in_top = false;
                for (int r = 0; r < rk; ++r) in_top |= (top_idx[r] == b);
                if (!in_top) ubm = fmaxf(ubm, B[b]);
            }
        }
        if (overlap) {
            ubm = warp_max(ubm);
            if (lane == 0) sh.red_f[warp] = ubm;
        }
        __syncthreads();
        if (peer_b) {
            // publish this rank's rows of head h, then wait (bounded) for the other ranks' rows and add them up
            if (tid == 0) {
                __threadfence_system();
                for (int p = 0; p < ws.peer_world; ++p)
                    if (p != ws.peer_rank)
                        st_release_sys(ws.peer_flags_b[p] + (long)ws.peer_rank * gridDim.x + h, ws.peer_step);
            }
            peer_wait(ws.peer_flags_b[ws.peer_rank] + h, ws.peer_world, ws.peer_rank, ws.peer_step, ws.wait_status,
                      (long)gridDim.x);
            if (tid < rk) {
                float gs = 0.0f, gl = 0.0f;
                for (int r = 0; r < ws.peer_world; ++r) {
                    const float *g = ws.given_fp16 + r * ws.given_rank_stride + ((long)h * CQA_MAX_RANKING_K + tid) * 2;
                    gs = __fadd_rn(gs, __ldcg(g));
                    gl = __fadd_rn(gl, __ldcg(g + 1));
                }
                top_f16[tid] = gs;
                top_lm[tid] = gl;
            }
            __syncthreads();
        }
        CQA_CLK(7);
        const float delta = s_delta;
        float ub = -INFINITY;
        if (kn.ranking_fallback) {
            if (overlap) {
                ubm = warp_max(sh.red_f[lane]);
            } else {
                for (int b = tid; b < n; b += SC_THREADS) {
                    bool in_top = false;
                    for (int r = 0; r < rk; ++r) in_top |= (top_idx[r] == b);
                    if (!in_top) ubm = fmaxf(ubm, B[b]);
                }
                ubm = block_max(ubm, sh);
            }
            ub = __fadd_rn(ubm, delta);
        }
        CQA_CLK(8);
        if (warp == 1) {
            // the certificate's per-candidate rows do not depend on the flag logic below
            ct->top_blocks[lane] = lane < rk ? top_idx[lane] : -1;
            if (lane < CQA_LM_ROWS) ct->fp16_scores[lane] = lane < rk ? top_f16[lane] : 0.0f;
            if (lane < CQA_LM_ROWS) ct->fp16_logmass[lane] = lane < rk ? top_lm[lane] : 0.0f;
        }
        if (warp == 0) {
            // lane i owns candidate i (candidates are in INT8 order): its position in the stable
            // descending FP16 order, and in the descending FP16 log-mass order
            const bool mine = lane < rk;
            const float f = mine ? top_f16[lane] : 0.0f;
            const float lmv = mine ? top_lm[lane] : 0.0f;
            int pos16 = 0, poslm = 0;
#pragma unroll 1
            for (int j = 0; j < rk; ++j) {
                const float fj = top_f16[j], lj = top_lm[j];
                pos16 += (fj > f || (fj == f && j < lane)) ? 1 : 0;
                poslm += (lj > lmv || (lj == lmv && j < lane)) ? 1 : 0;
            }
            const int r_main = min(kn.ranking_r, rk);
            const bool rf = kn.ranking_fallback && kn.ranking_r > 0;
            const bool d = mine && pos16 != lane;
            const int dis_main = (rf && __any_sync(FULL, d && lane < r_main)) ? 1 : 0;
            const int dis_r1 = (rf && __any_sync(FULL, d && lane < 1)) ? 1 : 0;
            const int dis_r3 = (rf && __any_sync(FULL, d && lane < 3)) ? 1 : 0;
            const unsigned who_r = __ballot_sync(FULL, mine && poslm == r_main - 1);
            const unsigned who_1 = __ballot_sync(FULL, mine && pos16 == 0);
            const unsigned who_2 = __ballot_sync(FULL, mine && pos16 == 1);
            float ell_r = -INFINITY;
            if (kn.ranking_fallback && r_main > 0) ell_r = __shfl_sync(FULL, lmv, __ffs(who_r) - 1);
            const float top1 = __shfl_sync(FULL, f, __ffs(who_1) - 1);
            const float top2 = who_2 ? __shfl_sync(FULL, f, __ffs(who_2) - 1) : top1;
            const int boundary = (kn.ranking_fallback && r_main > 0 && ub > ell_r) ? 1 : 0;
            int violation = 0;
            if (kn.score_consistency) {
                const float thr = __fadd_rn(delta, kn.eps_guard);
                violation = __any_sync(FULL, mine && fabsf(__fsub_rn(f, top_i8[lane])) > thr) ? 1 : 0;
            }
            if (lane == 0) {
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
                ct->fp16_top1 = top1;
                ct->fp16_top2 = top2;
                ct->int8_top1 = top_i8[0];
                const int dense = (kn.ranking_fallback && kn.rung3_recompute && rung3) ? 1 : 0;
                ct->dense = dense;
                if (dense) {
                    const int slot = atomicAdd(ws.any_flags + 4, 1);
                    if (slot < (int)gridDim.x) ws.any_flags[5 + slot] = h;
                }
                if (rung3) atomicOr(ws.any_flags + 1, 1);
                if (violation) atomicOr(ws.any_flags + 2, 1);
            }
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
    if (role == 1) { CQA_CLK_FLUSH(6, 9); CQA_CLK_FLUSH(15, 15); return; }
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
    __syncthreads();
    // Greedy promotion, largest contribution first (ties: lower block id first): block b is promoted while the
    // column sum of the contributions ranked before it is below the excess.  That sum never decreases along the
    // ranking, so the promoted blocks are exactly those with contribution bits >= t0, where t0 is the largest
    // threshold whose admitted set still sums to at least the excess; t0 is found bit by bit by the first 256
    // threads (no sort, no serial walk).  Exact ties at t0 are resolved the same way over the block id.
    if (tid == 0) { sh.bcast_f[1] = 0.0f; sh.bcast_f[2] = 0.0f; sh.bcast_i[1] = 0; sh.bcast_u[0] = 0xFFFFFFFFu; sh.bcast_i[3] = 0; }
    if (tid < VS_THREADS) {
        int parity = 0, cnt = 0;
        const float e_pre_v = column_sum(A, n, [](unsigned, int) { return true; }, sh, parity, cnt);
        const float excess = fmaxf(__fsub_rn(e_pre_v, kn.v_tolerance), 0.0f);
        float promoted = 0.0f;
        int n_prom = 0;
        unsigned t0 = 0xFFFFFFFFu;   // nothing admitted
        int id_bound = 0;
        if (kn.value_mode_tight) {
            if (excess > 0.0f) {
                t0 = 0u;
                int cnt_lo = cnt, cnt_hi = 0;     // entries >= t0, entries >= the upper end of the open range
                float f_lo = e_pre_v;
#pragma unroll 1
                for (int bit = 30; bit >= 0 && cnt_lo - cnt_hi > 1; --bit) {
                    const unsigned trial = t0 | (1u << bit);
                    int c = 0;
                    const float f = column_sum(A, n, [trial](unsigned bits, int) { return bits >= trial; }, sh, parity, c);
                    if (f >= excess) { t0 = trial; cnt_lo = c; f_lo = f; } else { cnt_hi = c; }
                }
                promoted = f_lo;
                n_prom = cnt_lo;
                id_bound = n;                     // every entry equal to t0 is admitted ...
                if (cnt_lo - cnt_hi > 1) {
                    // ... unless several entries equal t0: admit them in block order while the sum stays below
                    int i0 = 0;
#pragma unroll 1
                    for (int bit = 14; bit >= 0; --bit) {
                        const int trial = i0 | (1 << bit);
                        if (trial > n) continue;
                        int c = 0;
                        const unsigned tt = t0;
                        const float g = column_sum(A, n, [tt, trial](unsigned bits, int b) { return bits > tt || (bits == tt && b < trial); }, sh, parity, c);
                        if (g < excess) i0 = trial;
                    }
                    id_bound = i0 + 1;
                    const unsigned tt = t0;
                    const int ib = id_bound;
                    promoted = column_sum(A, n, [tt, ib](unsigned bits, int b) { return bits > tt || (bits == tt && b < ib); }, sh, parity, n_prom);
                }
            }
        } else {
            const float vt = kn.v_tolerance;
            promoted = column_sum(A, n, [eta, vt, &gcol](unsigned, int b) { return eta[gcol(b)] > vt; }, sh, parity, n_prom);
        }
        if (tid == 0) {
            sh.bcast_f[1] = promoted;
            sh.bcast_f[2] = e_pre_v;
            sh.bcast_i[1] = n_prom;
            sh.bcast_u[0] = t0;
            sh.bcast_i[3] = id_bound;
        }
    }
    __syncthreads();
    CQA_CLK(12);
    const float e_pre = sh.bcast_f[2];
    {
        const unsigned t0 = sh.bcast_u[0];
        const int id_bound = sh.bcast_i[3];
        for (int b = tid; b < n; b += SC_THREADS) {
            bool up;
            if (kn.value_mode_tight) {
                const unsigned bits = __float_as_uint(A[b]);
                up = t0 != 0xFFFFFFFFu && (bits > t0 || (bits == t0 && b < id_bound));
            } else {
                up = eta[gcol(b)] > kn.v_tolerance;
            }
            mask[b] = up ? 1 : 0;
        }
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
    }
    CQA_CLK(14);
    CQA_CLK_FLUSH(10, 14);
#ifdef CQA_PHASE_CLOCKS
    if (threadIdx.x == 0) for (int i = 0; i < 6; ++i) ct->fp16_scores[16 + i] = (float)(sh.dbg[i] - phase_clk[0]);
#endif
}

template <typename T2>
__global__ void __launch_bounds__(SC_THREADS) selcert_kernel(cqa_cache c, cqa_knobs kn, cqa_workspace ws, const void *q,
                                                            int q_dtype, long nq, long nact, const float *u, long u_ld,
                                                            int n_pad, int hi, int base_width, int two_level, int rk,
                                                            int phases, int role_base)
{
    grid_dependency_wait();
    peer_wait(ws.wait_flags, ws.wait_n, ws.wait_skip, ws.wait_value, ws.wait_status);
#ifdef CQA_WARM_REPEAT
    selcert_body<T2>(c, kn, ws, q, q_dtype, nq, nact, u, u_ld, n_pad, hi, base_width, two_level, rk, phases, role_base);
    __syncthreads();
#endif
    selcert_body<T2>(c, kn, ws, q, q_dtype, nq, nact, u, u_ld, n_pad, hi, base_width, two_level, rk, phases, role_base);
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
    static size_t granted[SMEM_ATTR_DEVICES] = {};
    const int rc_attr = check_cuda(ensure_dynamic_smem(selcert_kernel<T2>, smem, granted), "cudaFuncSetAttribute(selcert_kernel)");
    if (rc_attr) return rc_attr;
    if ((phases & PH_SELECT) && !(phases & PH_FLAGS_CLEARED)) {
        int rc = check_cuda(cudaMemsetAsync(ws->any_flags, 0, (5 + H) * sizeof(int32_t), st),
                            "cudaMemsetAsync(any_flags)");
        if (rc) return rc;
    }
    // select only: role 0; certify only: roles 1 and 2; fused: all three
    const int role_base = (phases & PH_SELECT) ? 0 : 1;
    int n_roles = (phases & PH_SELECT) ? ((phases & PH_CERTIFY) ? 3 : 1) : 2;
    if (phases & PH_GIVEN) n_roles = 1;   // role 1 alone
    dim3 grid((unsigned)H, (unsigned)n_roles);
    // chained to the score kernel only in the fused step (a memset precedes the launch otherwise)
    const bool chained = (phases & PH_FLAGS_CLEARED) != 0;
    return check_cuda(launch_chained(selcert_kernel<T2>, grid, dim3(SC_THREADS), smem, st, chained, *c, *kn, *ws, q, q_dtype,
                                     nq, nact, u, u_ld, n_pad, hi, base_width, two_level, rk, phases, role_base),
                      "selcert_kernel");
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
        const bool local_keys = !(phases & (PH_TOP_ONLY | PH_GIVEN));
        if ((phases & PH_PEER_B) && (ws->peer_world < 2 || ws->peer_world > 8 || !ws->given_fp16 || ws->peer_step < 1)) {
            set_error("selector: incomplete peer description for the in-kernel exchange");
            return CQA_ERR_INVALID;
        }
        if (need_fp16 && local_keys && (!c->keys_t2 || !c->sigma_max || !q)) {
            set_error("cqa_certify: ranking / consistency checks need q, Tier-2 keys and sigma_max");
            return CQA_ERR_INVALID;
        }
        if (need_fp16 && (phases & PH_GIVEN) && (!ws->given_fp16 || !c->sigma_max || !q)) {
            set_error("cqa_certify_given: needs q, sigma_max and the exchanged FP16 scores");
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

int select_certify_local_launch(const cqa_cache *c, const cqa_knobs *kn, const cqa_workspace *ws, long nq,
                                long nact, const float *u, long u_ld, cudaStream_t st)
{
    return selcert_launch(c, kn, ws, nullptr, CQA_F32, nq, nact, u, u_ld, PH_SELECT | PH_CERTIFY | PH_TOP_ONLY, st);
}

int certify_given_launch(const cqa_cache *c, const cqa_knobs *kn, const cqa_workspace *ws, const void *q,
                         int q_dtype, long nq, long nact, cudaStream_t st)
{
    return selcert_launch(c, kn, ws, q, q_dtype, nq, nact, nullptr, 0, PH_CERTIFY | PH_GIVEN, st);
}

int certify_launch(const cqa_cache *c, const cqa_knobs *kn, const cqa_workspace *ws, const void *q, int q_dtype,
                   long nq, long nact, cudaStream_t st)
{
    return selcert_launch(c, kn, ws, q, q_dtype, nq, nact, nullptr, 0, PH_CERTIFY, st);
}

}  // namespace cqa
