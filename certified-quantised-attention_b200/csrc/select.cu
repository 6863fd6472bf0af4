// Selector and certifier: one CTA of 1024 threads per (query head, role).
//
// A thread owns the blocks b = tid, tid + 1024, ... (at most 16 at the limit of
// 16384 blocks).  The per-block values live in shared-memory arrays and every
// phase is a short rolled loop over them with one CTA barrier: the executed
// code is small on purpose, because ~100 CTAs start the same code at the same
// moment and an unrolled form of these loops was bound by instruction fetch.
//
//   role 0 (select) : exploration bits (drawn before the wait on the score
//            kernel), block masses and mass fractions (canonical sum), the 256
//            heaviest blocks (ties -> lower block id) by a radix search on the
//            float bit patterns, ordered by rank counting; sequential cumulative
//            mass; K* with the Rung-1 expansion; FP16-key mask.
//   role 1 (ranking): query row and Delta (before the wait), top-4 blocks by
//            m_b (per-thread lists merged by shuffles), FP16 re-score of each
//            candidate by eight warps while the boundary maximum is taken,
//            ranking / boundary / score-consistency flags, work list of the
//            dense recompute.
//   role 2 (values) : Rung-2 value check: the promoted blocks are those whose
//            contribution mass*eta is at or above a threshold found by a search
//            over "column sums" (histogram hint, then two bits per step), no sort
//            and no serial walk.
//
// cqa_select, cqa_certify and the fused cqa_layer_step all launch the same
// kernel with a phase mask.  Sums over blocks use the canonical orders
// documented at the functions; prefix sums over the sorted order are
// sequential.
#include "common.cuh"
#include "rescore.cuh"

namespace cqa {

constexpr int SC_THREADS = 1024;
constexpr int SC_WARPS = 32;
constexpr int CAND = 256;          // candidates kept by the top search
constexpr int PH_SELECT = 1, PH_CERTIFY = 2;
// Sequence-sharded runs split the ranking check around an exchange: PH_TOP_ONLY stops role 1 once the top
// list is in the certificate; PH_GIVEN resumes it from that list with FP16 scores computed by the ranks that
// own the blocks (ws.given_fp16) and runs role 1 alone.
constexpr int PH_TOP_ONLY = 4, PH_GIVEN = 8;
constexpr int PH_FLAGS_CLEARED = 16;   // the caller already zeroed ws.any_flags on this stream
constexpr int PH_PEER_B = 64;          // role 1 exchanges the FP16 re-scores with the other ranks itself (ws.peer_*)

typedef unsigned long long u64;

// Philox4x32-10 on the counter (c0, head, offset) under `seed`: four 32-bit words.
__device__ __forceinline__ uint4 philox4(unsigned long long seed, unsigned long long offset, unsigned head, unsigned c0)
{
    unsigned c1 = head, c2 = (unsigned)offset, c3 = (unsigned)(offset >> 32);
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
    return make_uint4(c0, c1, c2, c3);
}
// The exploration draw takes one 16-bit uniform per (block, head, call): the eight blocks a thread owns in a row
// (b, b + 1024, ..., b + 7168) share one Philox call with counter word (b mod 1024) + 1024 * (b div 8192); block
// number i of the eight reads half (i mod 2) of output word i div 2.

__device__ __forceinline__ void cp_async4(float *smem, const float *gmem)
{
    const unsigned sa = (unsigned)__cvta_generic_to_shared(smem);
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;\n" ::"r"(sa), "l"(gmem) : "memory");
}

struct SCShared {
    float red_f[2][SC_WARPS];
    float red_f3[2][3][SC_WARPS];
    unsigned red_u[2][2][SC_WARPS];
    int red_i[2][SC_WARPS];
    unsigned char rank_part[4][CAND];
    unsigned short rank_pos[CAND];
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

// Maximum of one value per thread over the CTA, in every thread; one barrier (rows alternate with `parity`).
__device__ __forceinline__ float cta_max(float v, SCShared &sh, int &parity)
{
    v = warp_max(v);
    const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
    if (l == 0) sh.red_f[parity][w] = v;
    __syncthreads();
    const float r = warp_max(sh.red_f[parity][l]);
    parity ^= 1;
    return r;
}

// Every per-block loop of this kernel is a ROLLED loop over shared-memory arrays ("for k < nk: b = k * 1024 + tid").
// The code of a phase is then a few dozen instructions that stay in the instruction cache, instead of the same
// instructions unrolled once per block a thread owns: with ~100 CTAs starting the same straight-line code at the same
// moment, fetching instructions through the L2 was what bounded the unrolled form.

// Canonical sum of vals[0..n) (shared memory): 32 consecutive values by a warp butterfly (16..1), 8 such sums by a
// butterfly (4,2,1) = one leaf of 256 values, leaves added left to right.  Result in every thread.  gsum needs
// n_pad / 32 floats, leaf n_pad / 256.
__device__ __forceinline__ float cta_canonical_sum(const float *vals, int n, int nk, float *gsum, float *leaf)
{
    const int tid = threadIdx.x, w = tid >> 5, l = tid & 31;
    const int ngroups = (n + 31) >> 5, nleaf = (n + 255) >> 8;
#pragma unroll 1
    for (int k = 0; k < nk; ++k) {
        const int b = k * SC_THREADS + tid;
        const float s = warp_sum(b < n ? vals[b] : 0.0f);
        if (l == 0 && k * SC_WARPS + w < ngroups) gsum[k * SC_WARPS + w] = s;   // groups beyond n hold nothing
    }
    __syncthreads();
    if (tid < nleaf) {
        float p[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) p[i] = (tid * 8 + i) < ngroups ? gsum[tid * 8 + i] : 0.0f;
#pragma unroll
        for (int s = 4; s >= 1; s >>= 1)
#pragma unroll
            for (int i = 0; i < s; ++i) p[i] = __fadd_rn(p[i], p[i + s]);
        leaf[tid] = p[0];
    }
    __syncthreads();
    float total = leaf[0];
#pragma unroll 1
    for (int L = 1; L < nleaf; ++L) total = __fadd_rn(total, leaf[L]);
    return total;
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

// Given hist[0..nbins) (nbins <= 2048, non-negative, total below 2^31), find the highest bin d whose suffix sum
// S(d) = hist[d] + hist[d+1] + ... reaches `need` (need >= 1, S(0) >= need): returns d in every thread, with
// `above` = S(d+1) and `in_bin` = hist[d].  Thread t scans the bins in descending order, two per thread; one
// warp scan, one barrier, a second scan over the warp totals.
__device__ __forceinline__ int find_suffix_crossing(const int *hist, int nbins, int need, SCShared &sh, int &above,
                                                    int &in_bin)
{
    const int tid = threadIdx.x, lane = tid & 31, w = tid >> 5;
    const int r0 = 2 * tid, r1 = 2 * tid + 1;                      // ranks from the top
    const int c0 = r0 < nbins ? hist[nbins - 1 - r0] : 0;
    const int c1 = r1 < nbins ? hist[nbins - 1 - r1] : 0;
    const int local = c0 + c1;
    int incl = local;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const int x = __shfl_up_sync(FULL, incl, o);
        if (lane >= o) incl += x;
    }
    if (lane == 31) sh.red_i[0][w] = incl;
    __syncthreads();
    const int wt = sh.red_i[0][lane];
    int wincl = wt;                                                // inclusive scan of the warp totals
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const int x = __shfl_up_sync(FULL, wincl, o);
        if (lane >= o) wincl += x;
    }
    const int base = __shfl_sync(FULL, wincl - wt, w);
    const int excl = base + incl - local;
    if (excl < need && need <= excl + local) {
        const bool first = excl + c0 >= need;
        sh.bcast_i[4] = nbins - 1 - (first ? r0 : r1);
        sh.bcast_i[5] = first ? excl : excl + c0;
        sh.bcast_i[6] = first ? c0 : c1;
    }
    __syncthreads();
    above = sh.bcast_i[5];
    in_bin = sh.bcast_i[6];
    return sh.bcast_i[4];
}

// Count into hist[digit] the entries that `match`, one shared-memory atomic per entry; when every matching lane of
// a warp has the same digit (heavily tied data) the warp adds its count with a single atomic instead.
__device__ __forceinline__ void hist_add(int *hist, bool match, unsigned digit, int amount = 1)
{
    const unsigned who = __ballot_sync(FULL, match);
    if (who == 0) return;
    const int leader = __ffs(who) - 1;
    const unsigned d0 = __shfl_sync(FULL, digit, leader);
    const unsigned same = __ballot_sync(FULL, match && digit == d0);
    if (same == who && amount == 1) {
        if ((int)(threadIdx.x & 31) == leader) atomicAdd(&hist[d0], __popc(who));
    } else if (match) {
        atomicAdd(&hist[digit], amount);
    }
}

// Bit pattern `thr` of the M-th largest of vals[0..n) (shared memory, values >= 0; 1 <= M < n) and the number n_ge of
// entries at or above it, by a radix search: digits of 11, 11 and 9 bits from the top, each a histogram in shared
// memory (integer atomics) and a scan for the bin that holds the M-th entry.  A pass only counts the entries that
// fell into the previous pass's bin, and the search stops when a bin is taken whole (then n_ge == M and the lower
// bits of thr are zero).  hist: 2048 ints.
__device__ __forceinline__ void radix_threshold(const float *vals, int n, int nk, int M, int *hist, SCShared &sh,
                                                unsigned &thr, int &n_ge)
{
    const int tid = threadIdx.x;
    unsigned prefix = 0;
    int need = M, above_total = 0;
#pragma unroll 1
    for (int pass = 0; pass < 3; ++pass) {
        const int shift = pass == 0 ? 20 : (pass == 1 ? 9 : 0);
        const int nbins = pass == 2 ? 512 : 2048;
        const int up = pass == 0 ? 31 : (pass == 1 ? 20 : 9);        // bits at and above `up` are decided
        hist[2 * tid] = 0;
        hist[2 * tid + 1] = 0;
        __syncthreads();
#pragma unroll 1
        for (int k = 0; k < nk; ++k) {
            const int b = k * SC_THREADS + tid;
            const unsigned x = b < n ? __float_as_uint(vals[b]) : 0u;
            const bool match = b < n && (pass == 0 || (x >> up) == (prefix >> up));
            hist_add(hist, match, (x >> shift) & (unsigned)(nbins - 1));
        }
        __syncthreads();
        int above, in_bin;
        const int d = find_suffix_crossing(hist, nbins, need, sh, above, in_bin);
        prefix |= (unsigned)d << shift;
        above_total += above;
        need -= above;
        __syncthreads();          // hist and the broadcast words are rewritten by the next pass
        if (in_bin == need || pass == 2) {
            thr = prefix;
            n_ge = above_total + in_bin;
            return;
        }
    }
}

// The M = min(CAND, n) largest (value, lower-index-first) entries of vals[0..n) (shared memory, values >= 0), sorted
// descending into cand[0..CAND) (padding = 0).  The value of the M-th largest entry is found by a radix search over
// the bit patterns (radix_threshold); entries above the threshold are then compacted and ordered by rank counting.
__device__ __forceinline__ void select_top_sorted(const float *vals, int n, int nk, u64 *cand, int *hist, SCShared &sh)
{
    const int tid = threadIdx.x, lane = tid & 31, w = tid >> 5;
    if (tid == 0) sh.counter = 0;
    for (int i = tid; i < CAND; i += SC_THREADS) cand[i] = 0ull;
    const int M = n < CAND ? n : CAND;
    if (n <= CAND) {
        __syncthreads();
        if (tid < n) cand[tid] = make_key(vals[tid], tid);
    } else {
        unsigned thr = 0u;
        int n_ge = n;            // entries >= thr
        radix_threshold(vals, n, nk, M, hist, sh, thr, n_ge);
        // n_ge == M: the entries >= thr are the answer.  Otherwise thr is the value of the M-th largest
        // entry and several entries equal it: take everything above, then the lowest block ids among the equal.
        const bool ties = n_ge != M;
        __syncthreads();   // cand is zeroed, sh.counter is 0
        // first the number of entries each thread takes, then one atomic per warp for the base, then the copies
        int mine = 0;
#pragma unroll 1
        for (int k = 0; k < nk; ++k) {
            const int b = k * SC_THREADS + tid;
            const unsigned x = b < n ? __float_as_uint(vals[b]) : 0u;
            mine += (b < n && (ties ? x > thr : x >= thr)) ? 1 : 0;
        }
        int incl = mine;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const int x = __shfl_up_sync(FULL, incl, o);
            if (lane >= o) incl += x;
        }
        const int warp_total = __shfl_sync(FULL, incl, 31);
        int base = 0;
        if (lane == 31 && warp_total > 0) base = atomicAdd(&sh.counter, warp_total);
        base = __shfl_sync(FULL, base, 31);
        int pos = base + incl - mine;
        if (mine) {
#pragma unroll 1
            for (int k = 0; k < nk; ++k) {
                const int b = k * SC_THREADS + tid;
                if (b < n) {
                    const float v = vals[b];
                    const unsigned x = __float_as_uint(v);
                    if (ties ? x > thr : x >= thr) cand[pos++] = make_key(v, b);
                }
            }
        }
        if (ties) {
            // entries equal to the threshold fill the remaining places in block order: an ordered compaction,
            // 1024 consecutive blocks per round (per-warp counts, then an exclusive scan over the warps)
            __syncthreads();
            int taken = sh.counter;
            int par = 0;
            for (int b0 = 0; b0 < n && taken < M; b0 += SC_THREADS) {
                const int b = b0 + tid;
                const bool eq = b < n && __float_as_uint(vals[b]) == thr;
                const unsigned who = __ballot_sync(FULL, eq);
                if (lane == 0) sh.red_i[par][w] = __popc(who);
                __syncthreads();
                const int cw = sh.red_i[par][lane];
                par ^= 1;
                int inc2 = cw;   // inclusive scan of the per-warp counts
#pragma unroll
                for (int o = 1; o < 32; o <<= 1) {
                    const int x = __shfl_up_sync(FULL, inc2, o);
                    if (lane >= o) inc2 += x;
                }
                const int before = __shfl_sync(FULL, inc2 - cw, w);
                const int p = taken + before + __popc(who & ((1u << lane) - 1u));
                if (eq && p < M) cand[p] = make_key(vals[b], b);
                taken += __shfl_sync(FULL, inc2, 31);
            }
        }
    }
    __syncthreads();
    rank_sort_desc(cand, sh);
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

// "Column sums" of the value check for up to three admission thresholds at once: of the entries e[0..n) (shared
// memory), column t (= thread t, 0..1023) adds its admitted
// members t, t + 1024, ... in ascending order; the 32 columns of a warp are combined by the butterfly 16,8,4,2,1 and
// the 32 warp sums by the same butterfly.  f[i] = sum of the entries with bits >= t[i], c[i] = their number; results
// in every thread.  Adding an admitted entry never lowers a sum (every step is a monotone rounding), which is what
// the threshold search relies on.  A threshold of 0xFFFFFFFF admits nothing.
__device__ __forceinline__ void column_sums3(const float *e, int n, int nk, unsigned t1, unsigned t2, unsigned t3,
                                             SCShared &sh, int &parity, float (&f)[3], int (&c)[3])
{
    const int tid = threadIdx.x, lane = tid & 31, w = tid >> 5;
    float s1 = 0.0f, s2 = 0.0f, s3 = 0.0f;
    unsigned n12 = 0, n3 = 0;
#pragma unroll 1
    for (int k = 0; k < nk; ++k) {
        const int b = k * SC_THREADS + tid;
        if (b < n) {
            const float v = e[b];
            const unsigned x = __float_as_uint(v);
            if (x >= t1) { s1 = __fadd_rn(s1, v); n12 += 1u; }
            if (x >= t2) { s2 = __fadd_rn(s2, v); n12 += 1u << 16; }
            if (x >= t3) { s3 = __fadd_rn(s3, v); n3 += 1u; }
        }
    }
    s1 = warp_sum(s1);
    s2 = warp_sum(s2);
    s3 = warp_sum(s3);
    n12 = __reduce_add_sync(FULL, n12);
    n3 = __reduce_add_sync(FULL, n3);
    if (lane == 0) {
        sh.red_f3[parity][0][w] = s1;
        sh.red_f3[parity][1][w] = s2;
        sh.red_f3[parity][2][w] = s3;
        sh.red_u[parity][0][w] = n12;
        sh.red_u[parity][1][w] = n3;
    }
    __syncthreads();
    f[0] = warp_sum(sh.red_f3[parity][0][lane]);
    f[1] = warp_sum(sh.red_f3[parity][1][lane]);
    f[2] = warp_sum(sh.red_f3[parity][2][lane]);
    const unsigned c12 = __reduce_add_sync(FULL, sh.red_u[parity][0][lane]);
    c[2] = (int)__reduce_add_sync(FULL, sh.red_u[parity][1][lane]);
    c[0] = (int)(c12 & 0xFFFFu);
    c[1] = (int)(c12 >> 16);
    parity ^= 1;
}

// One column sum (same order as column_sums3) over the entries with bits > t_gt, or bits == t_gt and block id below
// id_lt.  (t_gt = t - 1, id_lt = 0 admits the entries with bits >= t; t_gt = 0, id_lt = n admits everything.)
__device__ __forceinline__ float column_sum1(const float *e, int n, int nk, unsigned t_gt, int id_lt, SCShared &sh,
                                             int &parity, int &count)
{
    const int tid = threadIdx.x, lane = tid & 31, w = tid >> 5;
    float s = 0.0f;
    unsigned c = 0;
#pragma unroll 1
    for (int k = 0; k < nk; ++k) {
        const int b = k * SC_THREADS + tid;
        if (b < n) {
            const float v = e[b];
            const unsigned x = __float_as_uint(v);
            if (x > t_gt || (x == t_gt && b < id_lt)) { s = __fadd_rn(s, v); ++c; }
        }
    }
    s = warp_sum(s);
    c = __reduce_add_sync(FULL, c);
    if (lane == 0) { sh.red_f3[parity][0][w] = s; sh.red_u[parity][0][w] = c; }
    __syncthreads();
    const float r = warp_sum(sh.red_f3[parity][0][lane]);
    count = (int)__reduce_add_sync(FULL, sh.red_u[parity][0][lane]);
    parity ^= 1;
    return r;
}

template <typename T2>
__device__ __forceinline__ void rescore_block(const cqa_cache &c, const void *q, int q_dtype, int h, long bid,
                                              long n_scoring_tokens, float q_scale, float &s, float &lm, const float *q_row)
{
    fp16_block_score_warp<T2>(c, q, q_dtype, h, bid, n_scoring_tokens, q_scale, s, lm, q_row);
}
// Address of token t of Tier-2 key block `bid` as seen by this lane (its 8 channels), or NULL when the token does not
// take part (beyond the scoring range, or a block held by neither tier).
__device__ __forceinline__ const void *t2_token_row(const cqa_cache &c, int kv, long bid, int t, long n_scoring_tokens)
{
    const int L = threadIdx.x & 15;
    if (bid < 0 || bid * BS + t >= n_scoring_tokens) return nullptr;
    const size_t esz = c.t2_dtype == CQA_F32 ? 4 : 2;
    const char *base = c.t2_dtype == CQA_BF16  ? reinterpret_cast<const char *>(t2_key_block<__nv_bfloat16>(c, kv, bid))
                       : c.t2_dtype == CQA_F16 ? reinterpret_cast<const char *>(t2_key_block<__half>(c, kv, bid))
                                               : reinterpret_cast<const char *>(t2_key_block<float>(c, kv, bid));
    return base ? base + ((size_t)t * D + 8 * L) * esz : nullptr;
}
// The logit of one token, by the 16 lanes of a half warp (same arithmetic as fp16_block_score_warp).
template <typename T2>
__device__ __forceinline__ float token_logit_t(const void *row, const float *q_row, float q_scale)
{
    const int L = threadIdx.x & 15;
    const Raw8<T2> raw = row ? raw_load8<T2>(reinterpret_cast<const T2 *>(row)) : raw_zero8<T2>();
    float kf[8], qv[8];
    raw_to_f(raw, kf);
#pragma unroll
    for (int i = 0; i < 8; ++i) qv[i] = q_row[8 * L + i];
    const float d = hw_sum(chain8(kf, qv));
    return row ? __fmul_rn(d, q_scale) : -INFINITY;
}
__device__ __forceinline__ float token_logit(const cqa_cache &c, const void *row, const float *q_row, float q_scale)
{
    if (c.t2_dtype == CQA_BF16) return token_logit_t<__nv_bfloat16>(row, q_row, q_scale);
    if (c.t2_dtype == CQA_F16) return token_logit_t<__half>(row, q_row, q_scale);
    return token_logit_t<float>(row, q_row, q_scale);
}

// Tier-2 dtype dispatch at run time: the re-score is a few warps of one role, the rest of the kernel does not
// depend on the dtype.
__device__ __noinline__ void rescore_block_any(const cqa_cache &c, const void *q, int q_dtype, int h, long bid,
                                               long n_scoring_tokens, float q_scale, float &s, float &lm,
                                               const float *q_row)
{
    if (c.t2_dtype == CQA_BF16) rescore_block<__nv_bfloat16>(c, q, q_dtype, h, bid, n_scoring_tokens, q_scale, s, lm, q_row);
    else if (c.t2_dtype == CQA_F16) rescore_block<__half>(c, q, q_dtype, h, bid, n_scoring_tokens, q_scale, s, lm, q_row);
    else rescore_block<float>(c, q, q_dtype, h, bid, n_scoring_tokens, q_scale, s, lm, q_row);
}

// Dynamic shared memory: A[n_arr] B[n_arr] C[n_pad] (floats; n_arr = max(n_pad, 2048)), cand[CAND] (u64), cum[CAND],
// gsum, leaf, mask[n_pad] (bytes).  The full-sort fallback aliases its keys over A and B; the radix searches use the
// array that is free at that point as their histogram.
__device__ __forceinline__ void selcert_body(const cqa_cache &c, const cqa_knobs &kn, const cqa_workspace &ws, const void *q,
                                             int q_dtype, long nq, long nact, const float *u, long u_ld, int n_pad, int hi,
                                             int base_width, int two_level, int rk, int phases, int role_base)
{
    extern __shared__ __align__(16) unsigned char dsm[];
    const int n_arr = n_pad > 2048 ? n_pad : 2048;
    float *A = reinterpret_cast<float *>(dsm);                 // m_b; role 2 later: contributions mass * eta
    float *B = A + n_arr;                                      // S_b; then mass / block log-mass / histogram
    float *C = B + n_arr;                                      // uniforms or eta_b; then mass fractions / histogram
    u64 *cand = reinterpret_cast<u64 *>(C + n_pad);
    float *cum = reinterpret_cast<float *>(cand + CAND);
    float *gsum = cum + CAND;
    float *leaf = gsum + (n_pad >> 5) + 1;
    unsigned char *mask = reinterpret_cast<unsigned char *>(leaf + (n_pad >> 8) + 2);
    __shared__ SCShared sh;
    __shared__ int top_idx[CQA_MAX_RANKING_K];
    __shared__ float top_i8[CQA_MAX_RANKING_K], top_f16[CQA_MAX_RANKING_K], top_lm[CQA_MAX_RANKING_K];
    __shared__ float s_delta;
    __shared__ float s_q[D];           // role 1: the head's query row as floats
    __shared__ u64 s_top[SC_WARPS * 4];

    __shared__ __align__(8) uint64_t row_bar;
    if (threadIdx.x == 0) {
        mbar_init(&row_bar, 1);
        mbar_init_fence();
    }
    __syncthreads();   // before the wait on the previous kernel: this part overlaps its tail

    const int h = blockIdx.x, tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int kv = h / c.gqa_group;
    const int n = (int)nq;
    const int nk = (n + SC_THREADS - 1) / SC_THREADS;          // blocks per thread: b = k * 1024 + tid, k < nk
    // Plain layout: row h of an [H][ld] array.  Sharded layout: row h of rank r's slot in the all-gather buffer,
    // [rank][row][chunk]; global block b sits at rank r = min(b / stride, ranks - 1), column b - r * stride.
    const bool sharded_in = ws.shard_stride > 0;
    const long row_ld = sharded_in ? ws.shard_chunk : ws.ld;
    const float *mb = ws.m_b + (long)h * row_ld;
    const float *sb = ws.s_b + (long)h * row_ld;
    // 32-bit arithmetic on purpose: the mapping runs once per block and thread
    const int sh_stride = sharded_in ? (int)ws.shard_stride : 1, sh_last = ws.shard_ranks - 1;
    const long sh_rank_stride = ws.shard_rank_stride;
    float *mf = ws.mass_frac + (long)h * ws.ld;
    cqa_head_cert *ct = ws.cert + h;
    // Three independent roles per head run as separate CTAs (grid.y): 0 = selector, 1 = ranking /
    // boundary / consistency checks, 2 = value check.  Roles 0 and 2 both need the mass fractions and
    // compute them with the same canonical arithmetic, so no CTA waits for another.
    const int role = role_base + (int)blockIdx.y;
    const bool fused = (phases & PH_SELECT) != 0;
    const bool compute_frac = role == 0 || (role == 2 && fused);
    const bool have_int4 = c.values_int4_packed != nullptr && c.values_int4_errors != nullptr;
    int parity = 0;

    // ---- the rows go from global to shared memory without passing through registers:
    // A <- m_b, B <- S_b, C <- eta_b (role 2) or the exploration uniforms (role 0)
    const bool explore_on = role == 0 && kn.exploration_rate > 0.0f;
    const float *eta = have_int4 ? c.values_int4_errors + (long)kv * (sharded_in ? ws.shard_chunk : c.max_blocks) : nullptr;
    const bool frac_given = role == 2 && !fused;
    const float *xsrc = role == 2 ? eta : ((explore_on && u != nullptr) ? u + (long)h * u_ld : nullptr);
    // Rows that start on a 16-byte boundary are fetched by the bulk-copy engine: one thread issues the copies (one
    // per array, or one per array and rank in the sharded layout, whose per-rank pieces are contiguous) and every
    // thread waits on the barrier they report to (bounded).  The last n % 4 blocks and unaligned rows go by 4-byte
    // asynchronous copies, each thread copying the blocks it owns.
    const float *bsrc = frac_given ? mf : sb;
    const int n4 = n & ~3;
    const int nseg = sharded_in ? ws.shard_ranks : 1;
    const int last_first = (nseg - 1) * sh_stride;             // first block of the last piece
    const bool pieces_ok = !sharded_in || (((sh_stride | (int)(sh_rank_stride & 0x7fffffff)) & 3) == 0 && n > last_first);
    const bool bulk = pieces_ok && n4 > 0 &&
                      (((uintptr_t)mb | (uintptr_t)bsrc | (uintptr_t)(xsrc ? xsrc : mb)) & 15u) == 0;
    // Still nothing of the previous kernel has been read: the exploration bits depend on the seed alone and are drawn
    // while that kernel drains.  One Philox call gives the eight 16-bit uniforms of blocks tid + 1024 * (8j .. 8j+7).
    const bool drawn = explore_on && u == nullptr;
    if (drawn) {
        const int nkp = n_pad > SC_THREADS ? n_pad / SC_THREADS : 1;
#pragma unroll 1
        for (int j = 0; j * 8 < nkp; ++j) {
            const uint4 r = philox4(ws.rng_seed, ws.rng_offset, (unsigned)h, (unsigned)tid | ((unsigned)j << 10));
            const unsigned wds[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const int b = (8 * j + i) * SC_THREADS + tid;
                if (8 * j + i < nkp && b < n_pad) {
                    const float uni = (float)((wds[i >> 1] >> ((i & 1) * 16)) & 0xFFFFu) * 1.52587890625e-05f;   // 2^-16
                    mask[b] = (b < n && uni < kn.exploration_rate) ? 2 : 0;   // bit 1: exploration candidate
                }
            }
        }
    }

    // Role 1, also ahead of the wait: the query row and Delta depend on q and on the per-channel scale maxima, both
    // complete before the score kernel started (the scale maxima of a sharded run arrive with the exchange and are
    // read after it).  The re-scoring warps later find q in shared memory and have one round trip to DRAM less.
    const bool rank_checks = role == 1 && (kn.ranking_fallback || kn.score_consistency) && n > 0 && q != nullptr;
    const bool delta_early = rank_checks && !sharded_in && !(phases & PH_TOP_ONLY) && c.sigma_max != nullptr;
    if (rank_checks) {
        if (warp == 0)
            for (int i = lane; i < D; i += 32) s_q[i] = load_q(q, q_dtype, (long)h * D + i);
        if (warp == 1 && delta_early) {
            const float d = delta_bound_warp(c, q, q_dtype, h);
            if (lane == 0) s_delta = d;
        }
    }

    grid_dependency_wait();
    peer_wait(ws.wait_flags, ws.wait_n, ws.wait_skip, ws.wait_value, ws.wait_status, 1, ws.wait_spins);

    if (bulk && tid == 0) {
        const unsigned bar = smem_u32(&row_bar);
        mbar_arrive_expect_tx(bar, (unsigned)n4 * 4u * (xsrc ? 3u : 2u));
#pragma unroll 1
        for (int r = 0; r < nseg; ++r) {
            const int first = r * sh_stride;
            const int cnt = (r == nseg - 1 ? n4 : first + sh_stride) - first;     // blocks of this piece, a multiple of 4
            if (cnt <= 0) continue;
            const long go = sharded_in ? (long)r * sh_rank_stride : 0;
            const unsigned bytes = (unsigned)cnt * 4u;
            bulk_copy_g2s(smem_u32(A + first), mb + go, bytes, bar);
            bulk_copy_g2s(smem_u32(B + first), frac_given ? mf + first : sb + go, bytes, bar);
            if (xsrc) bulk_copy_g2s(smem_u32(C + first), role == 2 ? xsrc + go : xsrc + first, bytes, bar);
        }
    }
#pragma unroll 1
    for (int k = bulk ? n4 / SC_THREADS : 0; k < nk; ++k) {
        const int b = k * SC_THREADS + tid;
        if (b < n && !(bulk && b < n4)) {
            long gb = b;
            if (sharded_in) {
                int r = b / sh_stride;
                if (r > sh_last) r = sh_last;
                gb = (long)r * sh_rank_stride + (b - r * sh_stride);
            }
            cp_async4(A + b, mb + gb);
            // certifying only: the mass fractions were computed by the selector call and take the place of S_b
            cp_async4(B + b, frac_given ? mf + b : sb + gb);
            if (xsrc) cp_async4(C + b, xsrc + (role == 2 ? gb : (long)b));
        }
    }
    asm volatile("cp.async.commit_group;\n" ::: "memory");
    asm volatile("cp.async.wait_group 0;\n" ::: "memory");
    if (bulk) mbar_wait(smem_u32(&row_bar), 0u);
    // each thread reads back only what it copied itself until the next barrier

    // ---- per-block preparation: the head's largest m_b; exploration bits (role 0); block log-masses (role 1)
    float mg = -INFINITY;
    if (role == 0) {
#pragma unroll 1
        for (int k = 0; k < nk; ++k) {
            const int b = k * SC_THREADS + tid;
            if (b < n_pad) {
                if (!drawn)   // bit 1: exploration candidate (uniforms given by the caller), bit 0: selected (set later)
                    mask[b] = (explore_on && b < n && C[b] < kn.exploration_rate) ? 2 : 0;
                if (b < n) mg = fmaxf(mg, A[b]);
            }
        }
    } else {
#pragma unroll 1
        for (int k = 0; k < nk; ++k) {
            const int b = k * SC_THREADS + tid;
            if (b < n) {
                const float m = A[b];
                mg = fmaxf(mg, m);
                if (role == 1) B[b] = __fadd_rn(clog(fmaxf(B[b], 1e-30f)), m);   // block log-mass for the boundary check
            }
        }
    }
    float total = 0.0f;
    if (compute_frac) {
        // mass = S * exp(m - max m) into B, fraction = mass * (1 / total): role 0 into C (and global memory),
        // role 2 straight into the contributions
        mg = cta_max(mg, sh, parity);
#pragma unroll 1
        for (int k = 0; k < nk; ++k) {
            const int b = k * SC_THREADS + tid;
            if (b < n) B[b] = __fmul_rn(fmaxf(B[b], 1e-30f), cexp(__fsub_rn(A[b], mg)));
        }
        total = fmaxf(cta_canonical_sum(B, n, nk, gsum, leaf), 1e-30f);
        const float inv_total = __fdiv_rn(1.0f, total);
#pragma unroll 1
        for (int k = 0; k < nk; ++k) {
            const int b = k * SC_THREADS + tid;
            if (b < n) {
                const float f = __fmul_rn(B[b], inv_total);
                if (role == 0) { C[b] = f; mf[b] = f; }
                else A[b] = __fmul_rn(f, C[b]);           // role 2: contribution = mass fraction * eta_b
            }
        }
    } else if (role == 2) {
#pragma unroll 1
        for (int k = 0; k < nk; ++k) {
            const int b = k * SC_THREADS + tid;
            if (b < n) A[b] = __fmul_rn(B[b], C[b]);
        }
    }
    __syncthreads();

    if (role == 0) {
        // the `hi` heaviest blocks, sorted
        int32_t *sidx = ws.sorted_idx + (long)h * ws.sel_width;
        float *scum = ws.sorted_cumsum + (long)h * ws.sel_width;
        const bool narrow = hi <= CAND;
        if (narrow) {
            select_top_sorted(C, n, nk, cand, reinterpret_cast<int *>(B), sh);
            if (tid < CAND) cum[tid] = key_val(cand[tid]);
            __syncthreads();
            if (tid == 0) {
                // sequential prefix sum in place; 32 values are fetched at a time so that only the additions are serial
                float run = 0.0f;
                float4 *c4 = reinterpret_cast<float4 *>(cum);
#pragma unroll 1
                for (int j0 = 0; j0 < hi; j0 += 32) {
                    float4 v[8];
#pragma unroll
                    for (int i = 0; i < 8; ++i) v[i] = c4[(j0 >> 2) + i];
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        v[i].x = (j0 == 0 && i == 0) ? v[i].x : __fadd_rn(run, v[i].x);
                        v[i].y = __fadd_rn(v[i].x, v[i].y);
                        v[i].z = __fadd_rn(v[i].y, v[i].z);
                        v[i].w = __fadd_rn(v[i].z, v[i].w);
                        run = v[i].w;
                    }
#pragma unroll
                    for (int i = 0; i < 8; ++i) c4[(j0 >> 2) + i] = v[i];
                }
            } else if (tid >= 32 && tid < 32 + CAND) {
                const int j = tid - 32;
                if (j < hi) sidx[j] = key_idx(cand[j]);
            }
            __syncthreads();
            if (tid < hi) scum[tid] = cum[tid];
        } else {
            // wide selections (k_max unset or very large): full sort, prefix sums straight to global memory
            u64 *keys = reinterpret_cast<u64 *>(A);   // m_b and the masses are not needed any more
            for (int b = tid; b < n_pad; b += SC_THREADS) keys[b] = b < n ? make_key(C[b], b) : 0ull;
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
        unsigned char *tm = ws.topk_mask + (long)h * ws.ld;
        unsigned char *em = ws.explore_mask + (long)h * ws.ld;
        int explored = 0;
        // four blocks per thread and store when the rows allow it (mask[] is 4-byte aligned, n_pad a multiple of 32)
        const int n4w = ((((uintptr_t)tm | (uintptr_t)em) & 3u) == 0) ? (n & ~3) : 0;
        const unsigned *mask4 = reinterpret_cast<const unsigned *>(mask);
#pragma unroll 1
        for (int b = 4 * tid; b < n4w; b += 4 * SC_THREADS) {
            const unsigned mk = mask4[b >> 2];
            const unsigned sel = mk & 0x01010101u;                       // selected by K*
            const unsigned exp = ((mk >> 1) & 0x01010101u) & ~sel;       // exploration candidates not already selected
            explored += __popc(exp);
            *reinterpret_cast<unsigned *>(tm + b) = sel | exp;
            *reinterpret_cast<unsigned *>(em + b) = exp;
        }
#pragma unroll 1
        for (int b = n4w + tid; b < (int)nact; b += SC_THREADS) {
            unsigned char mk1 = 1, e = 0;
            if (b < n) {
                const unsigned char mk = mask[b];
                mk1 = mk & 1;
                if (!mk1 && (mk & 2)) { mk1 = 1; e = 1; ++explored; }
            }
            tm[b] = mk1;
            em[b] = e;
        }
        explored = __reduce_add_sync(FULL, explored);
        if (lane == 0 && explored) atomicAdd(&sh.counter, explored);
        __syncthreads();
        if (tid == 0) ct->exploration_blocks = sh.counter;
        return;
    }

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
#pragma unroll 1
            for (int k = 0; k < nk; ++k) {
                const int b = k * SC_THREADS + tid;
                if (b < n) insert4(t4, ((u64)orderable(A[b]) << 32) | (u64)(0xFFFFFFFFu - (unsigned)b));
            }
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
                if (lane == 0) s_top[warp] = best;
                __syncthreads();
                best = s_top[lane];
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
        if (phases & PH_TOP_ONLY) {
            if (tid < CQA_MAX_RANKING_K) ct->top_blocks[tid] = tid < rk ? top_idx[tid] : -1;
            return;
        }
        // Boundary bound: max over the blocks outside the top list of (ell_b + delta).  Rounding is monotone,
        // so it equals (max ell_b) + delta; the maximum is taken by the warps that neither re-score a block
        // nor compute delta, while those wait for Tier-2 rows.
        const int ub_first = rk + 1, ub_warps = SC_WARPS - ub_first;
        const bool peer_b = (phases & PH_PEER_B) != 0;
        // With at most four candidates and Delta already known, a candidate block is re-scored by EIGHT warps (warp
        // 8j + p takes tokens p and p + 8 of candidate j, one per half warp): a single warp walking all 16 tokens is a
        // chain of ~600 dependent instructions behind a DRAM round trip, run once, and was the longest step of this role.
        const bool spread = !given && rk <= 4 && (delta_early || peer_b);
        const bool overlap = spread || ub_warps >= 8;
        float ubm = -INFINITY;
        if (spread) {
            const int j = warp >> 3, part = warp & 7, hw = lane >> 4;
            const int t = part + 8 * hw;
            // sharded by block range: this rank re-scores the candidates it owns (local block ids) and sends zeros for
            // the others, so that the sum over the ranks' rows is the owner's row
            const long bid = j < rk ? (long)top_idx[j] - (peer_b ? ws.peer_first_block : 0) : -1;
            const bool owned = j < rk && (!peer_b || (bid >= 0 && bid < ws.peer_n_local));
            const void *row = owned ? t2_token_row(c, kv, bid, t, peer_b ? ws.peer_n_local * BS : nq * BS) : nullptr;
            if (row && c.key_slots == nullptr) asm volatile("prefetch.global.L2 [%0];" ::"l"(row));   // device memory only
            if (kn.ranking_fallback) {
                // the boundary maximum while the rows are on their way
#pragma unroll 1
                for (int b = tid; b < n; b += SC_THREADS) {
                    bool in_top = false;
                    for (int r = 0; r < rk; ++r) in_top |= (top_idx[r] == b);
                    if (!in_top) ubm = fmaxf(ubm, B[b]);
                }
            }
            float *s_lg = reinterpret_cast<float *>(s_top);          // [4][16] logits, then [4][8] pair sums behind them
            float *s_pair = s_lg + 4 * BS;
            if (j < rk) {
                const float lg = token_logit(c, row, s_q, kn.q_scale);
                if ((lane & 15) == 0) s_lg[j * BS + t] = lg;
            }
            __syncthreads();
            float mx = -INFINITY;
            if (j < rk) {
                const float mine = s_lg[j * BS + t];
                mx = s_lg[j * BS + (lane & 15)];
#pragma unroll
                for (int o = 8; o >= 1; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(FULL, mx, o));
                float e = mine == -INFINITY ? 0.0f : cexp(__fsub_rn(mine, mx));
                e = __fadd_rn(e, __shfl_xor_sync(FULL, e, 16));       // token p + token p + 8
                if (lane == 0) s_pair[j * 8 + part] = e;
            }
            __syncthreads();
            if (j < rk && part == 0) {
                // the 16-token butterfly finished in its fixed order: (i, i+4), then (0,2) and (1,3), then the two
                const float *pp = s_pair + j * 8;
                const float q0 = __fadd_rn(pp[0], pp[4]), q1 = __fadd_rn(pp[1], pp[5]);
                const float q2 = __fadd_rn(pp[2], pp[6]), q3 = __fadd_rn(pp[3], pp[7]);
                const float l = fmaxf(__fadd_rn(__fadd_rn(q0, q2), __fadd_rn(q1, q3)), 1e-30f);
                const float sc = owned ? mx : 0.0f;
                const float lm = !owned ? 0.0f : (mx == -INFINITY ? -INFINITY : __fadd_rn(mx, clog(l)));
                if (peer_b) {
                    if (lane < ws.peer_world) {       // one lane per destination rank
                        float *d = ws.peer_xb[lane] + ((long)h * CQA_MAX_RANKING_K + j) * 2;
                        d[0] = sc;
                        d[1] = lm;
                    }
                } else if (lane == 0) {
                    top_f16[j] = sc;
                    top_lm[j] = lm;
                }
            } else if (warp == 1 && !delta_early) {
                const float d = delta_bound_warp(c, q, q_dtype, h, sharded_in ? ws.shard_ranks : 1, ws.shard_rank_stride);
                if (lane == 0) s_delta = d;
            }
        } else if (warp < rk) {
            if (peer_b) {
                // re-score the block if this rank owns it (local block ids), zeros otherwise; every rank gets the row
                const long bl = (long)top_idx[warp] - ws.peer_first_block;
                float s = 0.0f, lm = 0.0f;
                if (bl >= 0 && bl < ws.peer_n_local)
                    rescore_block_any(c, q, q_dtype, h, bl, ws.peer_n_local * BS, kn.q_scale, s, lm, s_q);
                if (lane < ws.peer_world) {
                    float *d = ws.peer_xb[lane] + ((long)h * CQA_MAX_RANKING_K + warp) * 2;
                    d[0] = s;
                    d[1] = lm;
                }
            } else if (!given) {
                float s, lm;
                rescore_block_any(c, q, q_dtype, h, (long)top_idx[warp], nq * BS, kn.q_scale, s, lm, s_q);
                if (lane == 0) { top_f16[warp] = s; top_lm[warp] = lm; }
            }
        } else if (warp == rk) {
            if (!delta_early) {
                const float d = delta_bound_warp(c, q, q_dtype, h, sharded_in ? ws.shard_ranks : 1, ws.shard_rank_stride);
                if (lane == 0) s_delta = d;
            }
        } else if (overlap && kn.ranking_fallback) {
#pragma unroll 1
            for (int b = (warp - ub_first) * 32 + lane; b < n; b += ub_warps * 32) {
                bool in_top = false;
                for (int r = 0; r < rk; ++r) in_top |= (top_idx[r] == b);
                if (!in_top) ubm = fmaxf(ubm, B[b]);
            }
        }
        if (overlap) {
            ubm = warp_max(ubm);
            if (lane == 0) sh.red_f[0][warp] = ubm;
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
                      (long)gridDim.x, ws.wait_spins);
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
        const float delta = s_delta;
        float ub = -INFINITY;
        if (kn.ranking_fallback) {
            if (overlap) {
                ubm = warp_max(sh.red_f[0][lane]);
            } else {
                for (int b = tid; b < n; b += SC_THREADS) {
                    bool in_top = false;
                    for (int r = 0; r < rk; ++r) in_top |= (top_idx[r] == b);
                    if (!in_top) ubm = fmaxf(ubm, B[b]);
                }
                parity = 1;   // row 0 of red_f is not in use here, keep the two uses apart all the same
                ubm = cta_max(ubm, sh, parity);
            }
            ub = __fadd_rn(ubm, delta);
        }
        if (warp == 1) {
            // the certificate's per-candidate rows do not depend on the flag logic below
            ct->top_blocks[lane] = lane < rk ? top_idx[lane] : -1;
            ct->fp16_scores[lane] = lane < rk ? top_f16[lane] : 0.0f;
            ct->fp16_logmass[lane] = lane < rk ? top_lm[lane] : 0.0f;
        }
        if (warp == 0) {
            // lane i owns candidate i (candidates are in INT8 order): its position in the stable
            // descending FP16 order, and in the descending FP16 log-mass order
            const bool mine = lane < rk;
            const float fs = mine ? top_f16[lane] : 0.0f;
            const float lmv = mine ? top_lm[lane] : 0.0f;
            int pos16 = 0, poslm = 0;
#pragma unroll 1
            for (int j = 0; j < rk; ++j) {
                const float fj = top_f16[j], lj = top_lm[j];
                pos16 += (fj > fs || (fj == fs && j < lane)) ? 1 : 0;
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
            const float top1 = __shfl_sync(FULL, fs, __ffs(who_1) - 1);
            const float top2 = who_2 ? __shfl_sync(FULL, fs, __ffs(who_2) - 1) : top1;
            const int boundary = (kn.ranking_fallback && r_main > 0 && ub > ell_r) ? 1 : 0;
            int violation = 0;
            if (kn.score_consistency) {
                const float thr = __fadd_rn(delta, kn.eps_guard);
                violation = __any_sync(FULL, mine && fabsf(__fsub_rn(fs, top_i8[lane])) > thr) ? 1 : 0;
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
    if (role == 1) return;

    // ---- Rung-2 value check (A holds the contributions mass fraction * eta_b, C still holds eta_b)
    unsigned char *vm = ws.value_mask + (long)h * ws.ld;
    if (!have_int4) {
        for (int b = tid; b < (int)nact; b += SC_THREADS) vm[b] = 1;   // FP16-value cache: every block reads Tier 2
        if (tid == 0) { ct->e_pre = 0.0f; ct->e_val = 0.0f; ct->value_promoted_blocks = 0; }
        return;
    }
    const float *e = A;
    // Greedy promotion, largest contribution first (ties: lower block id first): block b is promoted while the
    // column sum of the contributions ranked before it is below the excess.  That sum never decreases along the
    // ranking, so the promoted blocks are exactly those with contribution bits >= t0, where t0 is the largest
    // threshold whose admitted set still sums to at least the excess (no sort, no serial walk).  Exact ties at t0
    // are resolved the same way over the block id.
    int cnt = 0;
    const float e_pre = column_sum1(e, n, nk, 0u, n, sh, parity, cnt);     // every entry
    const float excess = fmaxf(__fsub_rn(e_pre, kn.v_tolerance), 0.0f);
    float promoted = 0.0f;
    int n_prom = 0;
    unsigned t0 = 0xFFFFFFFFu;   // nothing admitted
    int id_bound = 0;
    if (kn.value_mode_tight) {
        if (excess > 0.0f) {
            t0 = 0u;
            int cnt_lo = cnt, cnt_hi = 0;     // entries >= t0, entries >= the upper end of the open range
            float f_lo = e_pre;
            int bit = 30;
            // A hint first: 2048 bins over the top 11 bits of the contributions, each holding a fixed-point sum of its
            // entries (integer atomics; the scale keeps the total below 2^30).  The bin where the approximate suffix
            // sum crosses the excess is then CHECKED with exact column sums of its two edges; only if the exact sums
            // bracket the excess does the search continue inside the bin (bits 19..0), otherwise it starts from the
            // top as if there had been no hint.  The result never depends on the approximation.
            float emax = 0.0f;
#pragma unroll 1
            for (int k = 0; k < nk; ++k) {
                const int b = k * SC_THREADS + tid;
                if (b < n) emax = fmaxf(emax, e[b]);
            }
            emax = cta_max(emax, sh, parity);
            if (emax > 0.0f && n > 64) {
                int *hsum = reinterpret_cast<int *>(B);
                hsum[2 * tid] = 0;
                hsum[2 * tid + 1] = 0;
                __syncthreads();
                const float sc = __fdiv_rn(1073741824.0f, __fmul_rn((float)n, emax));     // 2^30 / (n * max)
#pragma unroll 1
                for (int k = 0; k < nk; ++k) {
                    const int b = k * SC_THREADS + tid;
                    const float v = b < n ? e[b] : 0.0f;
                    const int qv = (int)__fmul_rn(v, sc);
                    hist_add(hsum, qv > 0, __float_as_uint(v) >> 20, qv);
                }
                __syncthreads();
                const int need = max(1, (int)fminf(__fmul_rn(excess, sc), 1073741824.0f));
                // total of the bins (the crossing search needs need <= total)
                int tot = hsum[2 * tid] + hsum[2 * tid + 1];
                tot = __reduce_add_sync(FULL, tot);
                if (lane == 0) sh.red_i[1][warp] = tot;
                __syncthreads();
                tot = __reduce_add_sync(FULL, sh.red_i[1][lane]);
                if (need <= tot) {
                    int above, in_bin;
                    const int d = find_suffix_crossing(hsum, 2048, need, sh, above, in_bin);
                    const unsigned t_lo = (unsigned)d << 20, t_hi = (unsigned)(d + 1) << 20;
                    float fs[3];
                    int cs3[3];
                    column_sums3(e, n, nk, t_lo, t_hi, 0xFFFFFFFFu, sh, parity, fs, cs3);
                    if (fs[0] >= excess && fs[1] < excess) {
                        t0 = t_lo; cnt_lo = cs3[0]; f_lo = fs[0]; cnt_hi = cs3[1];
                        bit = 19;
                    } else {
                        // the fixed-point sums put the crossing one bin off: look at the neighbour on that side
                        const unsigned t_dn = d > 0 ? (unsigned)(d - 1) << 20 : 0u;
                        const unsigned t_up = d + 2 < 2048 ? (unsigned)(d + 2) << 20 : 0xFFFFFFFFu;
                        float gs[3];
                        int gc[3];
                        column_sums3(e, n, nk, t_dn, t_up, 0xFFFFFFFFu, sh, parity, gs, gc);
                        if (d > 0 && fs[0] < excess && gs[0] >= excess) {
                            t0 = t_dn; cnt_lo = gc[0]; f_lo = gs[0]; cnt_hi = cs3[0];
                            bit = 19;
                        } else if (fs[1] >= excess && gs[1] < excess) {
                            t0 = t_hi; cnt_lo = cs3[1]; f_lo = fs[1]; cnt_hi = gc[1];
                            bit = 19;
                        }
                    }
                }
            }
            // two bits per step: of the three trial thresholds t0 + {1,2,3} << (bit-1), keep the highest whose admitted
            // entries still reach the excess (the sums fall as the threshold rises)
#pragma unroll 1
            for (; bit >= 1 && cnt_lo - cnt_hi > 1; bit -= 2) {
                const unsigned s1 = t0 | (1u << (bit - 1)), s2 = t0 | (2u << (bit - 1)), s3 = t0 | (3u << (bit - 1));
                float fs[3];
                int cs3[3];
                column_sums3(e, n, nk, s1, s2, s3, sh, parity, fs, cs3);
                if (fs[2] >= excess) { t0 = s3; cnt_lo = cs3[2]; f_lo = fs[2]; }
                else if (fs[1] >= excess) { t0 = s2; cnt_lo = cs3[1]; f_lo = fs[1]; cnt_hi = cs3[2]; }
                else if (fs[0] >= excess) { t0 = s1; cnt_lo = cs3[0]; f_lo = fs[0]; cnt_hi = cs3[1]; }
                else cnt_hi = cs3[0];
            }
            if (bit == 0 && cnt_lo - cnt_hi > 1) {      // an odd number of bits was open (search from the top: 31)
                const unsigned trial = t0 | 1u;
                int cc = 0;
                const float fv = column_sum1(e, n, nk, trial - 1u, 0, sh, parity, cc);
                if (fv >= excess) { t0 = trial; cnt_lo = cc; f_lo = fv; } else { cnt_hi = cc; }
            }
            promoted = f_lo;
            n_prom = cnt_lo;
            id_bound = n;                     // every entry equal to t0 is admitted ...
            if (cnt_lo - cnt_hi > 1) {
                // ... unless several entries equal t0: admit them in block order while the sum stays below
                int i0 = 0;
#pragma unroll 1
                for (int bit2 = 14; bit2 >= 0; --bit2) {
                    const int trial = i0 | (1 << bit2);
                    if (trial > n) continue;
                    int cc = 0;
                    const float g = column_sum1(e, n, nk, t0, trial, sh, parity, cc);
                    if (g < excess) i0 = trial;
                }
                id_bound = i0 + 1;
                promoted = column_sum1(e, n, nk, t0, id_bound, sh, parity, n_prom);
            }
        }
    } else {
        // loose mode: every block whose eta_b exceeds the tolerance
        const float vt = kn.v_tolerance;
        const int lane_ = tid & 31, w_ = tid >> 5;
        float s = 0.0f;
        unsigned cc = 0;
#pragma unroll 1
        for (int k = 0; k < nk; ++k) {
            const int b = k * SC_THREADS + tid;
            if (b < n && C[b] > vt) { s = __fadd_rn(s, e[b]); ++cc; }
        }
        s = warp_sum(s);
        cc = __reduce_add_sync(FULL, cc);
        if (lane_ == 0) { sh.red_f3[parity][0][w_] = s; sh.red_u[parity][0][w_] = cc; }
        __syncthreads();
        promoted = warp_sum(sh.red_f3[parity][0][lane_]);
        n_prom = (int)__reduce_add_sync(FULL, sh.red_u[parity][0][lane_]);
        parity ^= 1;
    }
#pragma unroll 1
    for (int k = 0; k < nk; ++k) {
        const int b = k * SC_THREADS + tid;
        if (b < n) {
            unsigned char upb;
            if (kn.value_mode_tight) {
                const unsigned bits = __float_as_uint(e[b]);
                upb = (t0 != 0xFFFFFFFFu && (bits > t0 || (bits == t0 && b < id_bound))) ? 1 : 0;
            } else {
                upb = C[b] > kn.v_tolerance ? 1 : 0;
            }
            vm[b] = upb;
        }
    }
    // the trailing partial block (at most one) lies beyond the blocks the threads own
    if (tid == 0 && (int)nact > n) vm[n] = kn.force_trailing_value_fp16 ? 1 : 0;
    if (tid == 0) {
        ct->e_pre = e_pre;
        ct->e_val = fmaxf(__fsub_rn(e_pre, promoted), 0.0f);
        ct->value_promoted_blocks = n_prom;
        if (n_prom > 0) atomicOr(ws.any_flags + 3, 1);
    }
}

__global__ void __launch_bounds__(SC_THREADS, 1) selcert_kernel(cqa_cache c, cqa_knobs kn, cqa_workspace ws, const void *q,
                                                                int q_dtype, long nq, long nact, const float *u, long u_ld,
                                                                int n_pad, int hi, int base_width, int two_level, int rk,
                                                                int phases, int role_base)
{
    selcert_body(c, kn, ws, q, q_dtype, nq, nact, u, u_ld, n_pad, hi, base_width, two_level, rk, phases, role_base);
}

static __host__ __device__ inline int next_pow2(long n)
{
    int p = 32;
    while (p < n) p <<= 1;
    return p;
}

// Selection widths derived from the knobs (shared by the argument check, the launch and the batched kernel).
struct SelPlan {
    int hi, base_width, two_level, rk;
};
static __host__ __device__ inline SelPlan sel_plan(const cqa_knobs *kn, long nq)
{
    SelPlan p;
    const bool can_expand = kn->rung1_threshold >= 0.0f && kn->k_max > 0;
    long sel_kmax = kn->k_max;
    p.two_level = 0;
    if (can_expand) {
        long expanded = (long)ceil((double)kn->k_max * (double)kn->rung1_multiplier);
        if (expanded > nq) expanded = nq;
        if (expanded > kn->k_max) { sel_kmax = expanded; p.two_level = 1; }
    }
    p.hi = (int)(sel_kmax <= 0 ? nq : (sel_kmax < nq ? sel_kmax : nq));
    p.base_width = p.two_level ? (int)(kn->k_max < p.hi ? kn->k_max : p.hi) : p.hi;
    int rk = kn->ranking_r > kn->top_k_fp16_keys ? kn->ranking_r : kn->top_k_fp16_keys;
    if (rk < 4) rk = 4;
    if (rk > nq) rk = (int)nq;
    p.rk = rk;
    return p;
}

// Sequence blockIdx.z of a batch: the fused selector + certifier (all three roles) with that sequence's sizes.
__global__ void __launch_bounds__(SC_THREADS, 1) selcert_batched_kernel(const cqa_batch_item *items, cqa_knobs kn, int q_dtype,
                                                                        int do_append)
{
    const cqa_batch_item &it = *stage_batch_item(items + blockIdx.z);
    const long num_tokens = it.pos + do_append;
    const long nq = num_tokens / BS, nact = (num_tokens + BS - 1) / BS;
    const SelPlan p = sel_plan(&kn, nq);
    selcert_body(it.cache, kn, it.ws, it.q, q_dtype, nq, nact, nullptr, 0, next_pow2(nq), p.hi, p.base_width, p.two_level,
                      p.rk, PH_SELECT | PH_CERTIFY | PH_FLAGS_CLEARED, 0);
}

static size_t selcert_smem(int n_pad)
{
    const size_t n_arr = n_pad > 2048 ? n_pad : 2048;
    return n_arr * 8 + (size_t)n_pad * 5 + (size_t)CAND * 12 + ((size_t)(n_pad >> 5) + 1 + (n_pad >> 8) + 2) * 4 + 64;
}

// Every argument check of the selector / certifier launch; nothing is launched or copied here.
int selcert_check(const cqa_cache *c, const cqa_knobs *kn, const cqa_workspace *ws, const void *q, long nq, int phases)
{
    if (nq <= 0) { set_error("selector: needs at least one quantised block"); return CQA_ERR_INVALID; }
    if (nq > CQA_MAX_SORT_BLOCKS) {
        set_error("selector: %ld quantised blocks exceed the limit %d", nq, CQA_MAX_SORT_BLOCKS);
        return CQA_ERR_TOO_LARGE;
    }
    if (nq > ws->ld && ws->shard_stride <= 0) { set_error("selector: workspace ld %ld < %ld blocks", (long)ws->ld, nq); return CQA_ERR_INVALID; }
    if (c->t2_dtype < 0 || c->t2_dtype > 2) { set_error("selector: unknown Tier-2 dtype %d", c->t2_dtype); return CQA_ERR_INVALID; }
    const SelPlan p = sel_plan(kn, nq);
    if ((phases & PH_SELECT) && ws->sel_width < p.hi) {
        set_error("cqa_select: workspace sel_width %d < required %d", ws->sel_width, p.hi);
        return CQA_ERR_INVALID;
    }
    if (p.rk > CQA_MAX_RANKING_K - 1) {
        set_error("cqa_certify: ranking set of %d blocks exceeds the limit %d", p.rk, CQA_MAX_RANKING_K - 1);
        return CQA_ERR_TOO_LARGE;
    }
    if (phases & PH_CERTIFY) {
        const bool need_fp16 = kn->ranking_fallback || kn->score_consistency;
        const bool local_keys = !(phases & (PH_TOP_ONLY | PH_GIVEN));
        if ((phases & PH_PEER_B) && (ws->peer_world < 2 || ws->peer_world > 8 || !ws->given_fp16 || ws->peer_step < 1)) {
            set_error("selector: incomplete peer description for the in-kernel exchange");
            return CQA_ERR_INVALID;
        }
        if (need_fp16 && c->sigma_max && ((uintptr_t)c->sigma_max & 15)) {
            set_error("cqa_certify: sigma_max must be 16-byte aligned");
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
    return CQA_OK;
}

static int selcert_launch_v(const cqa_cache *c, const cqa_knobs *kn, const cqa_workspace *ws, const void *q,
                            int q_dtype, long nq, long nact, const float *u, long u_ld, int phases, int n_pad,
                            cudaStream_t st)
{
    const int H = c->kv_heads * c->gqa_group;
    const SelPlan p = sel_plan(kn, nq);
    const size_t smem = selcert_smem(n_pad);
    static size_t granted[SMEM_ATTR_DEVICES] = {};
    const int rc_attr = check_cuda(ensure_dynamic_smem(selcert_kernel, smem, granted), "cudaFuncSetAttribute(selcert_kernel)");
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
    return check_cuda(launch_chained(selcert_kernel, grid, dim3(SC_THREADS), smem, st, chained, *c, *kn, *ws, q, q_dtype,
                                     nq, nact, u, u_ld, n_pad, p.hi, p.base_width, p.two_level, p.rk, phases, role_base),
                      "selcert_kernel");
}

int selcert_launch(const cqa_cache *c, const cqa_knobs *kn, const cqa_workspace *ws, const void *q, int q_dtype,
                   long nq, long nact, const float *u, long u_ld, int phases, cudaStream_t st)
{
    const int rc = selcert_check(c, kn, ws, q, nq, phases);
    if (rc) return rc;
    const int n_pad = next_pow2(nq);
    return selcert_launch_v(c, kn, ws, q, q_dtype, nq, nact, u, u_ld, phases, n_pad, st);
}

// The selector of a batch; `max_nq` = most quantised blocks of any sequence (sizes the shared memory), every item checked by the caller.
int selcert_batched_launch(const cqa_batch_item *items_dev, int n_items, int n_heads, long max_nq, const cqa_knobs *kn,
                           int q_dtype, int do_append, cudaStream_t st)
{
    const int n_pad = next_pow2(max_nq);
    const size_t smem = selcert_smem(n_pad);
    dim3 grid((unsigned)n_heads, 3u, (unsigned)n_items);
    static size_t granted[SMEM_ATTR_DEVICES] = {};
    const int rc = check_cuda(ensure_dynamic_smem(selcert_batched_kernel, smem, granted),
                              "cudaFuncSetAttribute(selcert_batched_kernel)");
    if (rc) return rc;
    return check_cuda(launch_chained(selcert_batched_kernel, grid, dim3(SC_THREADS), smem, st, true, items_dev, *kn, q_dtype,
                                     do_append), "selcert_batched_kernel");
}

int selcert_wait_timeouts(int *count, int reset) { return wait_timeouts_of_this_unit(count, reset); }

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
