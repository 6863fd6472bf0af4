// Phase 1: per-block INT8 Q.K scores (m_b, S_b and the 16 token scores per
// head), the FP16-key block re-score and the Delta bound.
//
// score_blocks_kernel: one CTA = (kv head, run of blocks); each half warp
// owns one 16-token block at a time.  Lane L of the half warp owns channels
// 8L..8L+7 with q*sigma for the G heads of the group in registers, so one
// key byte feeds G fused multiply-adds.  Key rows, scales and zero points are
// staged in shared memory by bulk asynchronous copies (TMA engine: one lane
// issues three copies per block, 2048 + 512 + 512 bytes, which report to an
// mbarrier; warp-private double buffer, no CTA barrier).  Lane L walks the tokens in the order j^L, which
// makes the shared-memory reads conflict free and lets the 16-lane
// reduce-scatter run without selects: afterwards lane L holds token L.
//
// Per token and head:  score = (dot(k_int8, q*sigma) + dot(q, zero)) * q_scale
// with the canonical dot order (two chains per lane, butterfly 8,4,2,1).
#include "common.cuh"
#include "rescore.cuh"

namespace cqa {

constexpr int SCORE_WARPS = 8;
constexpr int BLOCK_BYTES = BS * D;                       // 2048 INT8 key bytes
constexpr int STAGE_HALF = BLOCK_BYTES + 2 * D * 4;       // + scale + zero point = 3072
constexpr int STAGE_WARP = 2 * STAGE_HALF;                // two half warps
constexpr int SCORE_SMEM = SCORE_WARPS * 2 * STAGE_WARP;  // double buffered: 98304

// Issue the copies of one warp stage: blocks b0 (lanes 0-15 consume it) and b0+1 (lanes 16-31).  The two blocks are
// neighbours in every array, so a stage is three bulk copies: 4096 key bytes, 2 x 128 scales, 2 x 128 zero points
// (laid out [keys b0 | keys b0+1 | scales b0 | scales b0+1 | zero points b0 | zero points b0+1]).  An odd tail block
// has no neighbour: then the copies are half as long and both half warps read the first half (the block is scored
// twice, one result is stored).  One lane announces the bytes to the stage's mbarrier and issues the copies.
constexpr int ST_SCALES = 2 * BLOCK_BYTES, ST_ZEROS = ST_SCALES + 2 * D * 4;
__device__ __forceinline__ void score_issue(const cqa_cache &c, int kv, long b_first, long b_last, unsigned stage_addr,
                                            unsigned bar_addr, int lane)
{
    // the addresses are the same for every lane (computed outside the one-lane region, where the compiler can
    // keep them on the uniform datapath); only the copy instructions themselves are issued by one lane
    const unsigned nblk = b_first < b_last ? 2u : 1u;
    const char *k0 = reinterpret_cast<const char *>(c.keys_int8) + ((long)kv * c.cap_tokens + b_first * BS) * D;
    const char *s0 = reinterpret_cast<const char *>(c.keys_scale) + ((long)kv * c.max_blocks + b_first) * (D * 4);
    const char *z0 = reinterpret_cast<const char *>(c.keys_zero_points) + ((long)kv * c.max_blocks + b_first) * (D * 4);
    if (lane == 0) {
        mbar_arrive_expect_tx(bar_addr, nblk * STAGE_HALF);
        bulk_copy_g2s(stage_addr, k0, nblk * BLOCK_BYTES, bar_addr);
        bulk_copy_g2s(stage_addr + ST_SCALES, s0, nblk * (D * 4), bar_addr);
        bulk_copy_g2s(stage_addr + ST_ZEROS, z0, nblk * (D * 4), bar_addr);
    }
}

// 8 signed bytes -> four float pairs, exactly: flip the sign bit (u = k + 128), drop each byte into the
// low mantissa byte of 2^23 with one byte permute, and remove the offset with one packed add per pair.
__device__ __forceinline__ void i8x8_to_f2(uint2 w, float2 (&k)[4])
{
    const unsigned M = 0x4B000000u;
    const float2 off = make_float2(-8388736.0f, -8388736.0f);   // -(2^23 + 128)
    const unsigned x0 = w.x ^ 0x80808080u, x1 = w.y ^ 0x80808080u;
    k[0] = __fadd2_rn(make_float2(__uint_as_float(__byte_perm(x0, M, 0x7440)), __uint_as_float(__byte_perm(x0, M, 0x7441))), off);
    k[1] = __fadd2_rn(make_float2(__uint_as_float(__byte_perm(x0, M, 0x7442)), __uint_as_float(__byte_perm(x0, M, 0x7443))), off);
    k[2] = __fadd2_rn(make_float2(__uint_as_float(__byte_perm(x1, M, 0x7440)), __uint_as_float(__byte_perm(x1, M, 0x7441))), off);
    k[3] = __fadd2_rn(make_float2(__uint_as_float(__byte_perm(x1, M, 0x7442)), __uint_as_float(__byte_perm(x1, M, 0x7443))), off);
}

// chain8 on packed operands: the .x lanes are the even-channel chain, the .y lanes the odd one.
__device__ __forceinline__ float chain8_f2(const float2 (&a)[4], const float2 (&b)[4])
{
    float2 p = __ffma2_rn(a[0], b[0], make_float2(0.0f, 0.0f));
    p = __ffma2_rn(a[1], b[1], p);
    p = __ffma2_rn(a[2], b[2], p);
    p = __ffma2_rn(a[3], b[3], p);
    return __fadd_rn(p.x, p.y);
}

template <int G>
__device__ __forceinline__ void score_blocks_body(const cqa_cache &c, const void *q, int q_dtype, long nq, float q_scale,
                                                  float *m_b, float *s_b, long ld, float *tok, int blocks_per_cta,
                                                  int32_t *zero_words, int n_zero_words, const ScorePush &push)
{
    extern __shared__ __align__(16) char smem[];
    constexpr int GH = G >= 4 ? 4 : G;  // heads per register pass
    const int kv = blockIdx.y;
    grid_dependency_wait();
    // the fused layer step lets this kernel clear the certifier's flag words (one memset launch fewer)
    if (zero_words != nullptr && blockIdx.x == 0 && blockIdx.y == 0)
        for (int i = threadIdx.x; i < n_zero_words; i += SCORE_WARPS * 32) zero_words[i] = 0;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int L = lane & 15, hw = lane >> 4;
    const long b_begin = (long)blockIdx.x * blocks_per_cta;
    const long b_end = min(nq, b_begin + (long)blocks_per_cta);
    const long b_last = b_end - 1;
    char *wbuf = smem + warp * 2 * STAGE_WARP;
    float *s_q = reinterpret_cast<float *>(smem + SCORE_SMEM);   // [G][128] query rows of this KV group
    uint64_t *wbar = reinterpret_cast<uint64_t *>(smem + SCORE_SMEM + G * D * 4) + 2 * warp;   // one per stage
    if (lane == 0) {
        mbar_init(wbar, 1);
        mbar_init(wbar + 1, 1);
        mbar_init_fence();
    }
    __syncwarp();
    const unsigned wbuf_addr = smem_u32(wbuf), wbar_addr = smem_u32(wbar);

    // Blocks of this warp: b_begin + 2*(warp + 8*it) + hw
    const long stride = 2 * SCORE_WARPS;
    long b0 = b_begin + 2 * warp;
    int stage = 0, use = 0;
    if (b0 < b_end) score_issue(c, kv, b0, b_last, wbuf_addr, wbar_addr, lane);
    for (int i = threadIdx.x; i < G * D; i += SCORE_WARPS * 32) s_q[i] = load_q(q, q_dtype, (long)kv * G * D + i);
    __syncthreads();

    for (; b0 < b_end; b0 += stride) {
        const long bn = b0 + stride;
        // the other buffer was read in the previous iteration, which ended with a warp barrier
        if (bn < b_end)
            score_issue(c, kv, bn, b_last, wbuf_addr + (stage ^ 1) * STAGE_WARP, wbar_addr + (stage ^ 1) * 8, lane);
        mbar_wait(wbar_addr + stage * 8, (unsigned)(use >> 1) & 1u);     // this stage's barrier completes one phase per use
        const long b = b0 + hw;
        const bool live = b < b_end;
        const int half = live ? hw : 0;        // an odd tail has one block in the stage
        const char *sbase = wbuf + stage * STAGE_WARP;
        const char *kb = sbase + half * BLOCK_BYTES;
        const float *sc = reinterpret_cast<const float *>(sbase + ST_SCALES) + half * D;
        const float *zp = reinterpret_cast<const float *>(sbase + ST_ZEROS) + half * D;
#pragma unroll
        for (int pass = 0; pass < G / GH; ++pass) {
            float2 qs[GH][4];
            float zq[GH];
            {
                float sg[8], zz[8];
                load8<float>(sc + 8 * L, sg);
                load8<float>(zp + 8 * L, zz);
#pragma unroll
                for (int g = 0; g < GH; ++g) {
                    float qv[8];
                    load8<float>(s_q + (pass * GH + g) * D + 8 * L, qv);
#pragma unroll
                    for (int i = 0; i < 4; ++i)
                        qs[g][i] = make_float2(__fmul_rn(qv[2 * i], sg[2 * i]), __fmul_rn(qv[2 * i + 1], sg[2 * i + 1]));
                    zq[g] = hw_sum(chain8(qv, zz));
                }
            }
            // Tokens are visited in pairs (j^L, (j+8)^L): the first step of the 16-lane reduce-scatter
            // (stride 8) is applied at once, so only 8 partial sums per head stay live.
            float acc[GH][8];
            const char *krow = kb + 8 * L;
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const int t = j ^ L;
                float2 klo[4], khi[4];
                i8x8_to_f2(*reinterpret_cast<const uint2 *>(krow + t * D), klo);
                i8x8_to_f2(*reinterpret_cast<const uint2 *>(krow + (t ^ 8) * D), khi);
#pragma unroll
                for (int g = 0; g < GH; ++g) {
                    const float lo = chain8_f2(klo, qs[g]);
                    const float hi = chain8_f2(khi, qs[g]);
                    acc[g][j] = __fadd_rn(lo, __shfl_xor_sync(FULL, hi, 8));
                }
            }
#pragma unroll
            for (int g = 0; g < GH; ++g) {
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[g][j] = __fadd_rn(acc[g][j], __shfl_xor_sync(FULL, acc[g][j + 4], 4));
#pragma unroll
                for (int j = 0; j < 2; ++j) acc[g][j] = __fadd_rn(acc[g][j], __shfl_xor_sync(FULL, acc[g][j + 2], 2));
                acc[g][0] = __fadd_rn(acc[g][0], __shfl_xor_sync(FULL, acc[g][1], 1));
                const float score = __fmul_rn(__fadd_rn(acc[g][0], zq[g]), q_scale);
                const float mx = hw_max(score);
                const float e = cexp(__fsub_rn(score, mx));
                const float ssum = hw_sum(e);
                if (live) {
                    const int gg = pass * GH + g;
                    if (tok) tok[(((long)kv * nq + b) * G + gg) * BS + L] = score;
                    if (L == 0) {
                        const long o = (long)(kv * G + gg) * ld + b;
                        m_b[o] = mx;
                        s_b[o] = ssum;
                    }
                }
            }
        }
        __syncwarp();
        stage ^= 1;
        ++use;
    }
    if (push.world > 0) {
        // This CTA's results (G rows of b_end - b_begin consecutive blocks, for m_b and for S_b) go to the other ranks
        // as runs of consecutive words, a warp storing 128 contiguous bytes at a time: a remote store of a single word
        // costs a whole link packet, so the rows are not pushed from the scoring loop.  The values are read back
        // from this GPU's L2 after the CTA barrier.
        __syncthreads();
        const int nb = (int)(b_end - b_begin);
        if (nb > 0) {
            for (int i = threadIdx.x; i < 2 * G * nb; i += SCORE_WARPS * 32) {
                const int row = i / nb, col = i - row * nb;              // rows 0..G-1: m_b, G..2G-1: S_b
                const int gg = row < G ? row : row - G;
                const long o = (long)(kv * G + gg) * ld + b_begin + col;
                const float v = __ldcg((row < G ? m_b : s_b) + o);
                for (int p = 0; p < push.world; ++p)
                    if (p != push.rank) (row < G ? push.mb[p] : push.sb[p])[o] = v;
            }
        }
        // the last CTA of the grid tells every rank that this rank's rows have landed
        __syncthreads();
        if (threadIdx.x == 0) {
            __threadfence_system();
            const int t = atomicAdd(push.ticket, 1);
            if (t == (int)(gridDim.x * gridDim.y) - 1) {
                *push.ticket = 0;
                __threadfence_system();   // acquire side of the ticket chain: the other CTAs' fenced stores come first
                for (int p = 0; p < push.world; ++p)
                    if (p != push.rank) st_release_sys(push.flag[p], push.step);
            }
        }
    }
}

template <int G>
__global__ void __launch_bounds__(SCORE_WARPS * 32, 2) score_blocks_kernel(cqa_cache c, const void *q, int q_dtype,
                                                                          long nq, float q_scale, float *m_b,
                                                                          float *s_b, long ld, float *tok,
                                                                          int blocks_per_cta, int32_t *zero_words,
                                                                          int n_zero_words, ScorePush push)
{
    score_blocks_body<G>(c, q, q_dtype, nq, q_scale, m_b, s_b, ld, tok, blocks_per_cta, zero_words, n_zero_words, push);
}

// The same for sequence blockIdx.z of a batch; grid.x is sized for the longest sequence and every sequence splits
// its blocks over all of grid.x.
template <int G>
__global__ void __launch_bounds__(SCORE_WARPS * 32, 2) score_blocks_batched_kernel(const cqa_batch_item *items, int q_dtype,
                                                                                  float q_scale, int do_append)
{
    const cqa_batch_item &it = *stage_batch_item(items + blockIdx.z);
    const long nq = (it.pos + do_append) / BS;
    long bpc = (nq + gridDim.x - 1) / gridDim.x;
    if (bpc < 2) bpc = 2;
    ScorePush none = {};
    score_blocks_body<G>(it.cache, it.q, q_dtype, nq, q_scale, it.ws.m_b, it.ws.s_b, it.ws.ld, it.ws.token_scores, (int)bpc,
                         it.ws.any_flags, 5 + it.cache.kv_heads * G, none);
}

template <typename T2>
__global__ void __launch_bounds__(32) fp16_block_scores_kernel(cqa_cache c, const void *q, int q_dtype,
                                                              const int32_t *idx, int K, long n_scoring_tokens,
                                                              float q_scale, float *scores, float *logmass)
{
    const int h = blockIdx.y, kk = blockIdx.x;
    float s, lm;
    fp16_block_score_warp<T2>(c, q, q_dtype, h, (long)idx[h * K + kk], n_scoring_tokens, q_scale, s, lm);
    if (threadIdx.x == 0) {
        scores[h * K + kk] = s;
        logmass[h * K + kk] = lm;
    }
}

// Sequence-sharded ranking check: one warp per (top-list slot, head); blocks outside this rank's range give zeros.
template <typename T2>
__global__ void __launch_bounds__(32) rescore_owned_kernel(cqa_cache c, const cqa_head_cert *cert, const void *q,
                                                          int q_dtype, long first_block, long n_local, float q_scale,
                                                          float *out)
{
    const int h = blockIdx.y, i = blockIdx.x;
    const long b = (long)cert[h].top_blocks[i] - first_block;
    float s = 0.0f, lm = 0.0f;
    if (cert[h].top_blocks[i] >= 0 && b >= 0 && b < n_local)
        fp16_block_score_warp<T2>(c, q, q_dtype, h, b, n_local * BS, q_scale, s, lm);
    if (threadIdx.x == 0) {
        out[((long)h * CQA_MAX_RANKING_K + i) * 2] = s;
        out[((long)h * CQA_MAX_RANKING_K + i) * 2 + 1] = lm;
    }
}

__global__ void __launch_bounds__(32) delta_bound_kernel(cqa_cache c, const void *q, int q_dtype, float *delta)
{
    float d = delta_bound_warp(c, q, q_dtype, blockIdx.x);
    if (threadIdx.x == 0) delta[blockIdx.x] = d;
}

template <int G>
static int score_launch_g(const cqa_cache *c, const void *q, int q_dtype, long nq, float q_scale, float *m_b,
                          float *s_b, long ld, float *tok, dim3 grid, int bpc, int32_t *zero_words, int n_zero_words,
                          const ScorePush &push, cudaStream_t st)
{
    constexpr int SMEM = SCORE_SMEM + G * D * 4 + SCORE_WARPS * 2 * 8;   // stages, query rows, mbarriers
    static size_t granted[SMEM_ATTR_DEVICES] = {};
    const int rc_attr = check_cuda(ensure_dynamic_smem(score_blocks_kernel<G>, (size_t)SMEM, granted),
                                   "cudaFuncSetAttribute(score_blocks_kernel)");
    if (rc_attr) return rc_attr;
    return check_cuda(launch_chained(score_blocks_kernel<G>, grid, dim3(SCORE_WARPS * 32), SMEM, st, true, *c, q, q_dtype,
                                     nq, q_scale, m_b, s_b, ld, tok, bpc, zero_words, n_zero_words, push),
                      "score_blocks_kernel");
}

// Phase 1 of a batch: `max_nq` = most quantised blocks of any sequence.
int score_blocks_batched_launch(const cqa_batch_item *items_dev, int n_items, int kv_heads, int gqa_group, long max_nq,
                                int q_dtype, float q_scale, int do_append, cudaStream_t st)
{
    int dev = 0, sm_count = 148;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, dev);
    if (sm_count <= 0) sm_count = 148;
    // CTAs per (sequence, KV head): the count that minimises (waves of 2 CTAs per SM) x (blocks per CTA + a fixed
    // start-up cost of about 16 blocks).  One CTA too many per head spills the grid into a second, nearly empty wave
    // (5 instead of 4 CTAs per head cost 9 % of a 128K batch of 8); with many waves the granularity of a
    // one-sequence launch is the best choice again.  The split does not change any result: blocks are independent.
    const long slots = (long)sm_count * 2, heads = (long)kv_heads * n_items;
    long p_max = (slots + kv_heads - 1) / kv_heads;          // what a launch for one sequence uses
    const long by_work = (max_nq + 15) / 16;                  // at least 16 blocks per CTA
    if (p_max > by_work) p_max = by_work;
    if (p_max < 1) p_max = 1;
    long gx = 1;
    double best = 0.0;
    for (long p = 1; p <= p_max; ++p) {
        const long waves = (heads * p + slots - 1) / slots;
        const double cost = (double)waves * ((double)((max_nq + p - 1) / p) + 16.0);
        if (p == 1 || cost < best) { best = cost; gx = p; }
    }
    dim3 grid((unsigned)gx, (unsigned)kv_heads, (unsigned)n_items);
#define CQA_SCORE_BATCH_CASE(GG)                                                                                       \
    case GG: {                                                                                                         \
        constexpr int SMEM = SCORE_SMEM + GG * D * 4 + SCORE_WARPS * 2 * 8;                                            \
        static size_t granted[SMEM_ATTR_DEVICES] = {};                                                                 \
        const int rc = check_cuda(ensure_dynamic_smem(score_blocks_batched_kernel<GG>, (size_t)SMEM, granted),         \
                                  "cudaFuncSetAttribute(score_blocks_batched_kernel)");                                \
        if (rc) return rc;                                                                                             \
        return check_cuda(launch_chained(score_blocks_batched_kernel<GG>, grid, dim3(SCORE_WARPS * 32), SMEM, st, true, \
                                         items_dev, q_dtype, q_scale, do_append), "score_blocks_batched_kernel");      \
    }
    switch (gqa_group) {
        CQA_SCORE_BATCH_CASE(1)
        CQA_SCORE_BATCH_CASE(2)
        CQA_SCORE_BATCH_CASE(4)
        CQA_SCORE_BATCH_CASE(8)
    }
#undef CQA_SCORE_BATCH_CASE
    set_error("cqa_layer_step_batched: unsupported gqa_group %d", gqa_group);
    return CQA_ERR_UNSUPPORTED;
}

int rescore_owned_launch(const cqa_cache *c, const cqa_head_cert *cert, const void *q, int q_dtype, long first_block,
                         long n_local, float q_scale, float *out, cudaStream_t st)
{
    const int H = c->kv_heads * c->gqa_group;
    dim3 grid(CQA_MAX_RANKING_K, (unsigned)H);
    switch (c->t2_dtype) {
    case CQA_F32: rescore_owned_kernel<float><<<grid, 32, 0, st>>>(*c, cert, q, q_dtype, first_block, n_local, q_scale, out); note_launch(); break;
    case CQA_F16: rescore_owned_kernel<__half><<<grid, 32, 0, st>>>(*c, cert, q, q_dtype, first_block, n_local, q_scale, out); note_launch(); break;
    case CQA_BF16: rescore_owned_kernel<__nv_bfloat16><<<grid, 32, 0, st>>>(*c, cert, q, q_dtype, first_block, n_local, q_scale, out); note_launch(); break;
    default: set_error("cqa_rescore_owned: unknown Tier-2 dtype"); return CQA_ERR_INVALID;
    }
    return check_launch("rescore_owned_kernel");
}

int score_blocks_launch(const cqa_cache *c, const void *q, int q_dtype, long nq, float q_scale, float *m_b,
                        float *s_b, long ld, float *tok, cudaStream_t st, int32_t *zero_words, int n_zero_words,
                        const ScorePush *push_in)
{
    ScorePush push = {};
    if (push_in) push = *push_in;
    static int sm_count = 0;
    if (sm_count == 0) {
        int dev = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, dev);
        if (sm_count <= 0) sm_count = 148;
    }
    // two resident CTAs per SM
    long target_ctas = (long)sm_count * 2;
    long per_kv = (target_ctas + c->kv_heads - 1) / c->kv_heads;
    long bpc = (nq + per_kv - 1) / per_kv;
    if (bpc < 2) bpc = 2;
    dim3 grid((unsigned)((nq + bpc - 1) / bpc), (unsigned)c->kv_heads);
    switch (c->gqa_group) {
    case 1: return score_launch_g<1>(c, q, q_dtype, nq, q_scale, m_b, s_b, ld, tok, grid, (int)bpc, zero_words, n_zero_words, push, st);
    case 2: return score_launch_g<2>(c, q, q_dtype, nq, q_scale, m_b, s_b, ld, tok, grid, (int)bpc, zero_words, n_zero_words, push, st);
    case 4: return score_launch_g<4>(c, q, q_dtype, nq, q_scale, m_b, s_b, ld, tok, grid, (int)bpc, zero_words, n_zero_words, push, st);
    case 8: return score_launch_g<8>(c, q, q_dtype, nq, q_scale, m_b, s_b, ld, tok, grid, (int)bpc, zero_words, n_zero_words, push, st);
    }
    set_error("score_blocks: unsupported gqa_group %d", c->gqa_group);
    return CQA_ERR_UNSUPPORTED;
}

}  // namespace cqa

using namespace cqa;

// Range checks shared by every entry point that launches the score kernel (they all run before the launch).
int cqa::check_score_args(const cqa_cache *c, int q_dtype, long nq, long ld, const char *who)
{
    if (!c->keys_int8 || !c->keys_scale || !c->keys_zero_points) {
        set_error("%s: INT8 key arrays missing", who);
        return CQA_ERR_INVALID;
    }
    if (nq < 0 || nq > c->max_blocks || nq * BS > c->cap_tokens || ld < nq) {
        set_error("%s: nq=%ld out of range (max_blocks=%ld, cap_tokens=%ld, ld=%ld)", who, nq, (long)c->max_blocks,
                  (long)c->cap_tokens, ld);
        return CQA_ERR_INVALID;
    }
    if (q_dtype < 0 || q_dtype > 2) { set_error("%s: unknown q dtype %d", who, q_dtype); return CQA_ERR_INVALID; }
    if (((uintptr_t)c->keys_int8 | (uintptr_t)c->keys_scale | (uintptr_t)c->keys_zero_points) & 15) {
        set_error("%s: keys_int8, keys_scale and keys_zero_points must be 16-byte aligned (bulk copies)", who);
        return CQA_ERR_INVALID;
    }
    if (c->gqa_group != 1 && c->gqa_group != 2 && c->gqa_group != 4 && c->gqa_group != 8) {
        set_error("%s: unsupported gqa_group %d", who, c->gqa_group);
        return CQA_ERR_UNSUPPORTED;
    }
    return CQA_OK;
}

extern "C" int cqa_score_blocks(const cqa_cache *c, const void *q, int q_dtype, int64_t nq, float q_scale,
                                float *m_b, float *s_b, int64_t ld, float *token_scores, void *stream)
{
    if (!c || !q || !m_b || !s_b) {
        set_error("cqa_score_blocks: NULL pointer");
        return CQA_ERR_INVALID;
    }
    const int rc = check_score_args(c, q_dtype, nq, ld, "cqa_score_blocks");
    if (rc) return rc;
    if (nq == 0) return CQA_OK;
    return score_blocks_launch(c, q, q_dtype, nq, q_scale, m_b, s_b, ld, token_scores, (cudaStream_t)stream, nullptr, 0,
                               nullptr);
}

int cqa::score_wait_timeouts(int *count, int reset) { return wait_timeouts_of_this_unit(count, reset); }

extern "C" int cqa_fp16_block_scores(const cqa_cache *c, const void *q, int q_dtype, const int32_t *idx, int K,
                                     int64_t n_scoring_blocks, float q_scale, float *scores, float *logmass,
                                     void *stream)
{
    if (!c || !q || !idx || !scores || !logmass || !c->keys_t2) {
        set_error("cqa_fp16_block_scores: NULL pointer");
        return CQA_ERR_INVALID;
    }
    if (K <= 0) return CQA_OK;
    const int H = c->kv_heads * c->gqa_group;
    dim3 grid((unsigned)K, (unsigned)H);
    cudaStream_t st = (cudaStream_t)stream;
    const long nst = n_scoring_blocks * BS;
    switch (c->t2_dtype) {
    case CQA_F32: fp16_block_scores_kernel<float><<<grid, 32, 0, st>>>(*c, q, q_dtype, idx, K, nst, q_scale, scores, logmass); note_launch(); break;
    case CQA_F16: fp16_block_scores_kernel<__half><<<grid, 32, 0, st>>>(*c, q, q_dtype, idx, K, nst, q_scale, scores, logmass); note_launch(); break;
    case CQA_BF16: fp16_block_scores_kernel<__nv_bfloat16><<<grid, 32, 0, st>>>(*c, q, q_dtype, idx, K, nst, q_scale, scores, logmass); note_launch(); break;
    default: set_error("cqa_fp16_block_scores: unknown Tier-2 dtype"); return CQA_ERR_INVALID;
    }
    return check_launch("fp16_block_scores_kernel");
}

extern "C" int cqa_delta_bound(const cqa_cache *c, const void *q, int q_dtype, float *delta, void *stream)
{
    if (!c || !q || !delta || !c->sigma_max) { set_error("cqa_delta_bound: NULL pointer"); return CQA_ERR_INVALID; }
    if ((uintptr_t)c->sigma_max & 15) { set_error("cqa_delta_bound: sigma_max must be 16-byte aligned"); return CQA_ERR_INVALID; }
    const int H = c->kv_heads * c->gqa_group;
    delta_bound_kernel<<<H, 32, 0, (cudaStream_t)stream>>>(*c, q, q_dtype, delta); note_launch();
    return check_launch("delta_bound_kernel");
}
