// Phase 2: mixed INT8/FP16-key, INT4/FP16-value split-K attend, the dense
// FP16 recompute of flagged heads, and the log-sum-exp merge — one launch.
//
// attend_kernel, grid (8 + splits, KV):
//   * CTAs x >= 8: one (kv head, split of blocks).  The G query heads of the
//     group share every value load.  A warp owns one 16-token block at a time;
//     the block's INT4 codes, scales, zeros and cached Phase-1 token scores
//     (1.5 KB + 64 B per head) arrive in a warp-private 4-stage shared-memory
//     ring through 16-byte asynchronous copies, so several blocks per warp are
//     in flight and no CTA barrier sits in the loop.  (The pieces of a block are
//     small here - 1024, 256, 256 and 64 bytes per head - and bulk copies through
//     the TMA engine measured 3-7 % slower for them than per-lane 16-byte copies;
//     the score kernel, whose pieces are 2 KB and 512 bytes, stages by TMA.)  Lane L (mod 16) owns
//     output channels 8L..8L+7; half warp 0 takes the even tokens, half warp 1
//     the odd ones (conflict-free shared-memory reads).  INT4 codes become
//     floats with one logic op and one exact fused multiply-add each (magic
//     number 2^23), scale and zero are folded into the softmax weights, and
//     the accumulation uses packed f32x2 fused multiply-adds.  (head, block)
//     pairs flagged in topk_mask recompute their scores from Tier-2 keys;
//     pairs flagged in value_mask read Tier-2 values.
//   * CTAs x < 8 (dispatched first): a pool of 8*KV CTAs for the dense FP16
//     recompute.  Work units are (flagged head, chunk of blocks), taken from the
//     list the certifier wrote; with no flagged head the pool exits at once.
//   * The last CTA to finish for a kv head (a head, for the dense role) merges
//     the split partials and writes the output rows; no separate merge launch.
//
// Nothing computed here can change a selection or a certificate flag, so fast
// exponentials are used.
#include <mutex>

#include "common.cuh"

namespace cqa {

constexpr int ATT_WARPS = 8;
constexpr int ATT_THREADS = ATT_WARPS * 32;
#ifndef CQA_ATT_STAGES
#define CQA_ATT_STAGES 4
#endif
constexpr int ATT_STAGES = CQA_ATT_STAGES;

__device__ __forceinline__ float fexp(float x) { return __expf(x); }

__device__ __forceinline__ void att_cp16(void *smem, const void *gmem)
{
    unsigned s = (unsigned)__cvta_generic_to_shared(smem);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(s), "l"(gmem) : "memory");
}
__device__ __forceinline__ void att_commit() { asm volatile("cp.async.commit_group;\n" ::: "memory"); }
template <int N>
__device__ __forceinline__ void att_wait()
{
    asm volatile("cp.async.wait_group %0;\n" ::"n"(N) : "memory");
}

template <int G>
struct AttLayout {
    static constexpr int PACKED = 0;
    static constexpr int SCALES = BS * (D / 2);               // 1024
    static constexpr int ZEROS = SCALES + BS * NG * 2;        // 1280
    static constexpr int SCORES = ZEROS + BS * NG * 2;        // 1536
    static constexpr int STAGE = SCORES + G * BS * 4;         // + 64 B per head
    static constexpr int RING = ATT_WARPS * ATT_STAGES * STAGE;
    // cross-warp merge buffers and final-merge scratch (both alias the ring)
    static constexpr int MERGE_A = ATT_WARPS * G * (D + 2) * 4;
    static constexpr int MERGE_B = (2 * G * CQA_MAX_SPLITS + G + 4 + ATT_WARPS * D) * 4;
    static constexpr int MERGE = MERGE_A > MERGE_B ? MERGE_A : MERGE_B;
    static constexpr int RING_BYTES = RING > MERGE ? RING : MERGE;
    // per warp: two weight tiles [16 tokens][GP] of (w, w) pairs (INT4 part, zero where a head reads Tier-2
    // values), two tiles of true weights for those heads, and the FP16-key logits of the block being prepared.
    // A token's row is padded to GP = G + 2 pairs: with the lanes of a head holding tokens sub, sub + LPH, ... the
    // 8-byte stores of a half warp then fall into 16 different bank pairs (rows of G pairs collide four ways).
    static constexpr int GP = G >= 2 ? G + 2 : G;
    static constexpr int W_TILE = BS * GP * 8;
    static constexpr int PER_WARP = 4 * W_TILE + G * BS * 4;
    static constexpr int TOTAL = RING_BYTES + ATT_WARPS * PER_WARP;
};

// Per-lane source pointers of the next block to stage.  A block's stage is 1536 + 64*G bytes = packed codes
// (two 512-byte rounds), scales+zeros (one round: lanes 0-15 scales, 16-31 zeros) and G*64 bytes of token scores.
template <int G>
struct AttIssuer {
    const char *pk, *sz, *sc;   // global sources for this lane
    long b, b_end, nq;          // block to issue next
    bool have4;

    __device__ __forceinline__ void init(const cqa_cache &c, const float *tok, long nq_, int kv, long b0, long bend,
                                         int lane)
    {
        b = b0;
        b_end = bend;
        nq = nq_;
        have4 = c.values_int4_packed != nullptr;
        const long row0 = (long)kv * c.cap_tokens + b0 * BS;
        pk = reinterpret_cast<const char *>(c.values_int4_packed) + row0 * (D / 2) + lane * 16;
        const char *szb = lane < 16 ? reinterpret_cast<const char *>(c.values_int4_scales)
                                    : reinterpret_cast<const char *>(c.values_int4_zeros);
        sz = szb + row0 * NG * 2 + (lane & 15) * 16;
        sc = reinterpret_cast<const char *>(tok + ((long)kv * nq_ + b0) * G * BS) + lane * 16;
    }
    // Stage the block `b` (if any) and advance by one warp stride; always commits one group.  A block without
    // INT4 data (the trailing partial block) gets zeros, so the INT4 arithmetic on it is finite.
    __device__ __forceinline__ void issue(char *stage, int lane)
    {
        using LY = AttLayout<G>;
        if (b < b_end) {
            if (have4 && b < nq) {
                att_cp16(stage + lane * 16, pk);
                att_cp16(stage + 512 + lane * 16, pk + 512);
                att_cp16(stage + LY::SCALES + lane * 16, sz);
                if (lane < 4 * G) att_cp16(stage + LY::SCORES + lane * 16, sc);
            } else {
                const uint4 z = make_uint4(0u, 0u, 0u, 0u);
                *reinterpret_cast<uint4 *>(stage + lane * 16) = z;
                *reinterpret_cast<uint4 *>(stage + 512 + lane * 16) = z;
                *reinterpret_cast<uint4 *>(stage + LY::SCALES + lane * 16) = z;
                if (b < nq && lane < 4 * G) att_cp16(stage + LY::SCORES + lane * 16, sc);
            }
        }
        att_commit();
        b += ATT_WARPS;
        pk += ATT_WARPS * BS * (D / 2);
        sz += ATT_WARPS * BS * NG * 2;
        sc += ATT_WARPS * G * BS * 4;
    }
};

// (a & b) | c in one logic instruction.
__device__ __forceinline__ unsigned and_or(unsigned a, unsigned b, unsigned c)
{
    unsigned d;
    asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}

// Eight INT4 codes of one 32-bit word -> four float pairs, dequantised.  (bits | 2^(23-4j)) reads as
// 2^(23-4j) + code for a nibble at bit 4j of a 16-bit half; one exact packed add removes the offset, one packed
// fused multiply-add applies scale and zero point.
__device__ __forceinline__ void int4x8_dequant(unsigned pk, float2 s2, float2 z2, float2 (&v)[4])
{
    const float2 o01 = make_float2(-8388608.0f, -524288.0f), o23 = make_float2(-32768.0f, -2048.0f);
    const unsigned hi = pk >> 16;
    v[0] = make_float2(__uint_as_float(and_or(pk, 0x000Fu, 0x4B000000u)), __uint_as_float(and_or(pk, 0x00F0u, 0x49000000u)));
    v[1] = make_float2(__uint_as_float(and_or(pk, 0x0F00u, 0x47000000u)), __uint_as_float(and_or(pk, 0xF000u, 0x45000000u)));
    v[2] = make_float2(__uint_as_float(and_or(hi, 0x000Fu, 0x4B000000u)), __uint_as_float(and_or(hi, 0x00F0u, 0x49000000u)));
    v[3] = make_float2(__uint_as_float(and_or(hi, 0x0F00u, 0x47000000u)), __uint_as_float(and_or(hi, 0xF000u, 0x45000000u)));
    v[0] = __ffma2_rn(__fadd2_rn(v[0], o01), s2, z2);
    v[1] = __ffma2_rn(__fadd2_rn(v[1], o23), s2, z2);
    v[2] = __ffma2_rn(__fadd2_rn(v[2], o01), s2, z2);
    v[3] = __ffma2_rn(__fadd2_rn(v[3], o23), s2, z2);
}

// Cross-warp merge of (m, l, acc) inside the CTA, then one partial per head to global memory.
template <int G>
__device__ __forceinline__ void cta_merge_store(float (&m)[G], float (&l)[G], float (&acc)[G][8], float *sm_m,
                                                float *sm_l, float *sm_acc, float *out_m, float *out_l,
                                                float *out_acc, int head0, int split, int nsplits)
{
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, L = lane & 15;
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
    for (int item = threadIdx.x; item < G * D; item += ATT_THREADS) {
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

// Final merge of `ns` split partials of heads [head0, head0+nh) by the last CTA to arrive.
// All 256 threads take part; `sm` is 16-byte aligned scratch of at least 2*nh*ns + nh + 3 + 8*128 floats.
// A thread owns one float4 column of one head and every (256 / (32*nh))-th split.  Its accumulator rows are
// requested first (up to 20 loads in flight per thread), then the (m, l) partials go through shared memory and
// one warp per head turns them into per-split scales while those loads are still travelling; the rows are then
// scaled and summed, the per-thread sums combined through shared memory, normalised and written.
__device__ __forceinline__ void final_merge(const float *pm, const float *pl, const float *pa, int ns, int head0,
                                            int nh, const cqa_workspace &ws, bool dense_role, float *sm, int n_heads_total)
{
    constexpr int BATCH = 20;
    const bool push_c = ws.partial_out != nullptr && ws.peer_world > 0 && ws.peer_partial[0] != nullptr;
    float *s_m = sm, *s_sc = sm + nh * ns, *s_l = s_sc + nh * ns;
    float *s_part = sm + ((2 * nh * ns + nh + 3) & ~3);  // 16-byte aligned for float4 stores
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int nparts = ATT_WARPS / nh;      // nh is 1, 2, 4 or 8
    const int g = warp / nparts, part = warp % nparts;
    const float4 *rows = reinterpret_cast<const float4 *>(pa + (long)(head0 + g) * ns * D) + lane;
    float4 buf[BATCH];
#pragma unroll
    for (int j = 0; j < BATCH; ++j) {
        const int sp = part + j * nparts;
        buf[j] = sp < ns ? __ldcg(rows + (long)sp * (D / 4)) : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    }
    __syncthreads();   // the scratch may still be in use as merge buffers
    for (int i = tid; i < nh * ns; i += ATT_THREADS) {
        s_m[i] = __ldcg(pm + (long)head0 * ns + i);
        s_sc[i] = __ldcg(pl + (long)head0 * ns + i);
    }
    __syncthreads();
    if (warp < nh) {
        float M = -INFINITY;
        for (int sp = lane; sp < ns; sp += 32) M = fmaxf(M, s_m[warp * ns + sp]);
        M = warp_max(M);
        float lsum = 0.0f;
        for (int sp = lane; sp < ns; sp += 32) {
            const float mi = s_m[warp * ns + sp];
            const float sc = mi == -INFINITY ? 0.0f : fexp(mi - M);
            lsum = fmaf(s_sc[warp * ns + sp], sc, lsum);
            s_sc[warp * ns + sp] = sc;
        }
        lsum = warp_sum(lsum);
        if (lane == 0) {
            s_l[warp] = lsum;
            if (ws.partial_out != nullptr) {
                const int h = head0 + warp;
                const bool flagged = ws.cert != nullptr && (ws.cert[h].dense || ws.any_flags[2]);
                if (flagged == dense_role) {
                    if (push_c) {
                        for (int p = 0; p < ws.peer_world; ++p) {
                            ws.peer_partial[p][(long)h * CQA_PARTIAL_STRIDE] = M;
                            ws.peer_partial[p][(long)h * CQA_PARTIAL_STRIDE + 1] = lsum;
                        }
                    } else {
                        ws.partial_out[(long)h * CQA_PARTIAL_STRIDE] = M;
                        ws.partial_out[(long)h * CQA_PARTIAL_STRIDE + 1] = lsum;
                    }
                }
            }
        }
    }
    __syncthreads();
    float4 a = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
#pragma unroll
    for (int j = 0; j < BATCH; ++j) {
        const int sp = part + j * nparts;
        if (sp < ns) {
            const float sc = s_sc[g * ns + sp];
            a.x = fmaf(buf[j].x, sc, a.x);
            a.y = fmaf(buf[j].y, sc, a.y);
            a.z = fmaf(buf[j].z, sc, a.z);
            a.w = fmaf(buf[j].w, sc, a.w);
        }
    }
#pragma unroll 4
    for (int sp = part + BATCH * nparts; sp < ns; sp += nparts) {   // more splits than one batch covers
        const float4 v = __ldcg(rows + (long)sp * (D / 4));
        const float sc = s_sc[g * ns + sp];
        a.x = fmaf(v.x, sc, a.x);
        a.y = fmaf(v.y, sc, a.y);
        a.z = fmaf(v.z, sc, a.z);
        a.w = fmaf(v.w, sc, a.w);
    }
    reinterpret_cast<float4 *>(s_part + warp * D)[lane] = a;
    __syncthreads();
    for (int item = tid; item < nh * D; item += ATT_THREADS) {
        const int gg = item / D, ch = item % D, h = head0 + gg;
        const bool flagged = ws.cert != nullptr && (ws.cert[h].dense || ws.any_flags[2]);
        if (flagged != dense_role) continue;
        float acc = 0.0f;
        for (int p = 0; p < nparts; ++p) acc += s_part[(gg * nparts + p) * D + ch];
        if (ws.partial_out != nullptr) {
            // un-normalised: merged across ranks later
            if (push_c) {
                for (int p = 0; p < ws.peer_world; ++p) ws.peer_partial[p][(long)h * CQA_PARTIAL_STRIDE + 2 + ch] = acc;
            } else {
                ws.partial_out[(long)h * CQA_PARTIAL_STRIDE + 2 + ch] = acc;
            }
            continue;
        }
        const float l = s_l[gg];
        ws.out[(long)h * D + ch] = acc / (l > 0.0f ? l : 1.0f);
    }
    __syncthreads();
    if (push_c && tid == 0) {
        // Exchange C: one arrival per KV head (regular merges) plus one per densely recomputed head; the last one
        // tells every rank that this rank's partial rows have landed
        __threadfence_system();
        int expected = (int)gridDim.y;
        if (ws.dense_splits > 0 && ws.cert != nullptr) expected += ws.any_flags[2] ? n_heads_total : ws.any_flags[4];
        const int t = atomicAdd(ws.peer_ticket_c, 1);
        if (t == expected - 1) {
            *ws.peer_ticket_c = 0;
            __threadfence_system();
            for (int p = 0; p < ws.peer_world; ++p)
                if (p != ws.peer_rank) st_release_sys(ws.peer_flag_c[p], ws.peer_step);
        }
    }
}

// Returns true in every thread of the CTA that took the last ticket.
__device__ __forceinline__ bool take_ticket(int *ticket, int total, int *s_flag)
{
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) {
        const int t = atomicAdd(ticket, 1);
        *s_flag = (t == total - 1) ? 1 : 0;
        if (t == total - 1) *ticket = 0;  // ready for the next launch
    }
    __syncthreads();
    const bool last = *s_flag != 0;
    if (last) __threadfence();
    return last;
}

// Dense FP16 attention of one (head, chunk of blocks) unit; the last unit of a head merges and writes the row.
template <typename T2>
__device__ void dense_unit(const cqa_cache &c, const cqa_workspace &ws, const void *q, int q_dtype, long num_tokens,
                           float q_scale, int h, int chunk, char *smem_raw, int *s_flag)
{
    float *sm_m = reinterpret_cast<float *>(smem_raw);
    float *sm_l = sm_m + ATT_WARPS;
    float *sm_acc = sm_l + ATT_WARPS;
    const int kv = h / c.gqa_group;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, L = lane & 15, hw = lane >> 4;
    const long nblk = (num_tokens + BS - 1) / BS;
    const int ds = ws.dense_splits;
    const long bps = (nblk + ds - 1) / ds;
    const long b_begin = (long)chunk * bps;
    const long b_end = min(nblk, b_begin + bps);
    float qv[8];
    load_q8(q, q_dtype, (long)h * D + 8 * L, qv);
    float m[1] = {-INFINITY}, l[1] = {0.0f}, acc[1][8];
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[0][i] = 0.0f;
    for (long b = b_begin + warp; b < b_end; b += ATT_WARPS) {
        const T2 *kblk = t2_key_block<T2>(c, kv, b), *vblk = t2_value_block<T2>(c, kv, b);
        if (kblk == nullptr || vblk == nullptr) continue;
        // all key and value rows of this half warp's 8 tokens are requested before anything is consumed
        Raw8<T2> kr[8], vr[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const long t = b * BS + hw * 8 + i;
            if (t < num_tokens) {
                kr[i] = raw_load8<T2>(kblk + (hw * 8 + i) * D + 8 * L);
                vr[i] = raw_load8<T2>(vblk + (hw * 8 + i) * D + 8 * L);
            } else {
                kr[i] = raw_zero8<T2>();
                vr[i] = raw_zero8<T2>();
            }
        }
        float lg[8];
        float bm = -INFINITY;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const long t = b * BS + hw * 8 + i;
            float kf[8];
            raw_to_f(kr[i], kf);
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
            const float w = lg[i] == -INFINITY ? 0.0f : fexp(lg[i] - mn);
            ls += w;
            float vf[8];
            raw_to_f(vr[i], vf);
#pragma unroll
            for (int k = 0; k < 8; ++k) acc[0][k] = fmaf(w, vf[k], acc[0][k]);
        }
        ls += __shfl_xor_sync(FULL, ls, 16);
        l[0] = fmaf(l[0], alpha, ls);
    }
    __syncthreads();
    cta_merge_store<1>(m, l, acc, sm_m, sm_l, sm_acc, ws.dense_m, ws.dense_l, ws.dense_acc, h, chunk, ds);
    if (take_ticket(ws.tickets + c.kv_heads + h, ds, s_flag))
        final_merge(ws.dense_m, ws.dense_l, ws.dense_acc, ds, h, 1, ws, true, reinterpret_cast<float *>(smem_raw),
                    c.kv_heads * c.gqa_group);
}

constexpr int DENSE_POOL_X = 8;  // dense-recompute CTAs per KV row of the grid

template <int G, typename T2>
__device__ __forceinline__ void attend_body(const cqa_cache &c, const cqa_workspace &ws, const void *q, int q_dtype, long nq,
                                            long nact, long num_tokens, int last_valid, float q_scale, int blocks_per_split)
{
    using LY = AttLayout<G>;
    extern __shared__ __align__(16) char dsm[];
    __shared__ int s_flag;
    const int kv = blockIdx.y;
    const int ns = ws.num_splits;
    const int pool_x = ws.dense_splits > 0 ? DENSE_POOL_X : 0;
    if ((int)blockIdx.x < pool_x) {
        grid_dependency_wait();   // the list of flagged heads comes from the selector
        // Dense-recompute pool: units are (flagged head, chunk); unflagged steps leave at once.
        const int H = c.kv_heads * G;
        const bool all = ws.any_flags[2] != 0;
        const int n_heads = all ? H : ws.any_flags[4];
        if (n_heads == 0) return;
        const int ds = ws.dense_splits;
        const int pool = c.kv_heads * DENSE_POOL_X;
        for (int u = kv * DENSE_POOL_X + (int)blockIdx.x; u < n_heads * ds; u += pool) {
            const int h = all ? u / ds : ws.any_flags[5 + u / ds];
            dense_unit<T2>(c, ws, q, q_dtype, num_tokens, q_scale, h, u % ds, dsm, &s_flag);
        }
        return;
    }
    // ---- shared memory carve-up
    char *ring = dsm;
    const int split = (int)blockIdx.x - pool_x;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, L = lane & 15, hw = lane >> 4;
    const long b_begin = (long)split * blocks_per_split;
    const long b_end = min(nact, b_begin + (long)blocks_per_split);
    char *wring = ring + warp * ATT_STAGES * LY::STAGE;
    char *wpriv = dsm + LY::RING_BYTES + warp * LY::PER_WARP;
    float2 *w_tiles = reinterpret_cast<float2 *>(wpriv);                       // [2][16][GP] INT4-part weights
    float2 *w16_tiles = reinterpret_cast<float2 *>(wpriv + 2 * LY::W_TILE);    // [2][16][GP] true weights (Tier-2 values)
    float *sc_tile = reinterpret_cast<float *>(wpriv + 4 * LY::W_TILE);        // [G][16] FP16-key logits

    // start the pipeline before anything else
    AttIssuer<G> issuer;
    issuer.init(c, ws.token_scores, nq, kv, b_begin + warp, b_end, lane);
#pragma unroll
    for (int s = 0; s < ATT_STAGES - 1; ++s) issuer.issue(wring + s * LY::STAGE, lane);

    // Blocks of this warp: b_begin + warp + 8*it.  Lane j keeps the key / value promotion bits of the warp's
    // block (it0 + j), one bit per head of the group; they are re-read every 32 blocks.
    const int n_my = b_begin + warp < b_end ? (int)((b_end - b_begin - warp + ATT_WARPS - 1) / ATT_WARPS) : 0;
    // Everything above reads what the append and score kernels wrote (they completed before the selector, the
    // previous kernel of the chain, began); the masks and flags below are the selector's, so wait for it here.
    // CTAs that were scheduled while the selector was still running have their first blocks in flight by now.
    grid_dependency_wait();
    unsigned my_masks = 0;   // km | vm << 8 of block (it0 + lane)
    auto load_masks = [&](int it0) {
        const long b = b_begin + warp + (long)(it0 + lane) * ATT_WARPS;
        unsigned km = 0, vm = 0;
        if (b < b_end) {
#pragma unroll
            for (int g = 0; g < G; ++g) {
                const long o = (long)(kv * G + g) * ws.ld + b;
                km |= (ws.topk_mask[o] || b >= nq) ? (1u << g) : 0u;
                vm |= ws.value_mask[o] ? (1u << g) : 0u;
            }
        }
        my_masks = km | (vm << 8);
    };
    load_masks(0);
    // Largest Phase-1 block maximum over this warp's quantised blocks, per head: the softmax reference point.
    const bool have_mb = ws.m_b != nullptr;
    const long mb_ld = ws.shard_chunk > 0 ? ws.shard_chunk : ws.ld;   // a rank's own rows of the exchange buffer
    float m_init = -INFINITY;
    if (have_mb) {
        float mx[G];
#pragma unroll
        for (int g = 0; g < G; ++g) mx[g] = -INFINITY;
        for (long b = b_begin + warp + (long)lane * ATT_WARPS; b < b_end && b < nq; b += 32 * ATT_WARPS) {
#pragma unroll
            for (int g = 0; g < G; ++g) mx[g] = fmaxf(mx[g], ws.m_b[(long)(kv * G + g) * mb_ld + b]);
        }
#pragma unroll
        for (int g = 0; g < G; ++g) {
            const float v = warp_max(mx[g]);
            if (g == lane / (G >= 8 ? 4 : (G == 4 ? 8 : 16))) m_init = v;
        }
    }

    // Softmax bookkeeping layout: LPH lanes per head, each lane holds TPL tokens of its head `gl`.
    constexpr int LPH = G >= 8 ? 4 : (G == 4 ? 8 : 16);
    constexpr int TPL = BS / LPH;
    constexpr int GP = LY::GP;           // pairs per token row of a weight tile (padded)
    const int gl = lane / LPH, sub = lane % LPH;
    const bool gl_valid = gl < G;

    float2 acc2[G][4];
#pragma unroll
    for (int g = 0; g < G; ++g)
#pragma unroll
        for (int k = 0; k < 4; ++k) acc2[g][k] = make_float2(0.0f, 0.0f);
    float m_mine = m_init;      // running max of head gl (uniform over its LPH lanes)
    float l_mine = 0.0f;        // this lane's share of the running sum of head gl
    const bool have4 = c.values_int4_packed != nullptr;

    // prepare(it): logits -> weights of block `it` into w_tiles[it & 1]; returns this lane's rescale factor for
    // head gl (1 when the running max did not move).
    auto prepare = [&](int it, unsigned masks) -> float {
        const long b = b_begin + warp + (long)it * ATT_WARPS;
        const unsigned km = masks & 0xFFu, vm = (masks >> 8) & 0xFFu;
        const int n_valid = (b == nact - 1) ? last_valid : BS;
        const char *st = wring + (it % ATT_STAGES) * LY::STAGE;
        if (km) {
            // FP16-key logits for promoted heads (rare): Tier-2 rows straight from global memory
            const T2 *kblk = t2_key_block<T2>(c, kv, b);
#pragma unroll 1
            for (int g = 0; g < G; ++g) {
                if (!(km & (1u << g))) continue;
                float qv[8];
                load_q8(q, q_dtype, (long)(kv * G + g) * D + 8 * L, qv);
                Raw8<T2> kr[8];
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    const int t = hw * 8 + i;
                    kr[i] = (t < n_valid && kblk != nullptr) ? raw_load8<T2>(kblk + t * D + 8 * L) : raw_zero8<T2>();
                }
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    float kf[8];
                    raw_to_f(kr[i], kf);
                    const float d = hw_sum(chain8(kf, qv));
                    if (L == i) sc_tile[g * BS + hw * 8 + i] = d * q_scale;
                }
            }
            __syncwarp();
        }
        const float *st_sc = reinterpret_cast<const float *>(st + LY::SCORES);
        float sv_[TPL];
#pragma unroll
        for (int i = 0; i < TPL; ++i) {
            const int t = sub + LPH * i;
            float x = -INFINITY;
            if (gl_valid && t < n_valid) x = ((km >> gl) & 1u) ? sc_tile[gl * BS + t] : st_sc[gl * BS + t];
            sv_[i] = x;
        }
        // The running max starts at the largest Phase-1 block maximum of this warp's blocks, so it can only move
        // when FP16-key logits (or a block without Phase-1 scores) are involved.
        float alpha = 1.0f;
        if (km || !have_mb) {
            float bm = -INFINITY;
#pragma unroll
            for (int i = 0; i < TPL; ++i) bm = fmaxf(bm, sv_[i]);
#pragma unroll
            for (int o = LPH / 2; o >= 1; o >>= 1) bm = fmaxf(bm, __shfl_xor_sync(FULL, bm, o));
            const float m_up = fmaxf(m_mine, bm);
            alpha = (m_up == -INFINITY || m_mine == m_up) ? 1.0f : fexp(m_mine - m_up);
            m_mine = m_up;
        }
        const float m_new = m_mine;
        float2 *wt = w_tiles + (it & 1) * BS * GP;
        const bool v16 = (vm >> gl) & 1u;
        float ls = 0.0f;
#pragma unroll
        for (int i = 0; i < TPL; ++i) {
            const float w = sv_[i] == -INFINITY ? 0.0f : fexp(sv_[i] - m_new);
            ls += w;
            const float w4 = v16 ? 0.0f : w;
            if (gl_valid) wt[(sub + LPH * i) * GP + gl] = make_float2(w4, w4);
        }
        if (vm) {
#pragma unroll
            for (int i = 0; i < TPL; ++i) {
                const float w = sv_[i] == -INFINITY ? 0.0f : fexp(sv_[i] - m_new);
                if (gl_valid) w16_tiles[((it & 1) * BS + sub + LPH * i) * GP + gl] = make_float2(w, w);
            }
        }
        l_mine = fmaf(l_mine, alpha, ls);
        return alpha;
    };

    float alpha_cur = 1.0f;
    if (n_my > 0) {
        att_wait<ATT_STAGES - 2>();
        __syncwarp();
        alpha_cur = prepare(0, __shfl_sync(FULL, my_masks, 0));
    }
    for (int it = 0; it < n_my; ++it) {
        const long b = b_begin + warp + (long)it * ATT_WARPS;
        __syncwarp();   // every lane is done with the slot that is about to be refilled, and with w_tiles[(it+1)&1]
        issuer.issue(wring + ((it + ATT_STAGES - 1) % ATT_STAGES) * LY::STAGE, lane);
        att_wait<ATT_STAGES - 2>();   // block it+1 has landed
        __syncwarp();
        const unsigned masks_cur = __shfl_sync(FULL, my_masks, it & 31);
        const unsigned vm = (masks_cur >> 8) & 0xFFu;
        if ((it & 31) == 31 && it + 1 < n_my) load_masks(it + 1);
        const unsigned masks_next = __shfl_sync(FULL, my_masks, (it + 1) & 31);
        // rescale the accumulators if the running max of any head moved when block `it` was prepared
        if (__any_sync(FULL, alpha_cur != 1.0f)) {
#pragma unroll
            for (int g = 0; g < G; ++g) {
                const float ag = __shfl_sync(FULL, alpha_cur, g * LPH);
                const float2 a2 = make_float2(ag, ag);
#pragma unroll
                for (int k = 0; k < 4; ++k) acc2[g][k] = __fmul2_rn(acc2[g][k], a2);
            }
        }
        const char *st = wring + (it % ATT_STAGES) * LY::STAGE;
        const float2 *wt = w_tiles + (it & 1) * BS * GP;
        // ---- INT4 values of block `it` (zero weights where a head reads Tier-2 values or the token is padding);
        // this half warp takes tokens t = 2i + hw
        if (have4) {
            const unsigned *st_pk = reinterpret_cast<const unsigned *>(st + LY::PACKED);
            const __half *st_s = reinterpret_cast<const __half *>(st + LY::SCALES);
            const __half *st_z = reinterpret_cast<const __half *>(st + LY::ZEROS);
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const int t = 2 * i + hw;
                const unsigned pk = st_pk[t * 16 + L];
                const float sv = __half2float(st_s[t * NG + (L >> 1)]);
                const float zv = __half2float(st_z[t * NG + (L >> 1)]);
                float2 v[4];
                int4x8_dequant(pk, make_float2(sv, sv), make_float2(zv, zv), v);
                float2 w2[G];
                if constexpr (G % 2 == 0) {
#pragma unroll
                    for (int g = 0; g < G; g += 2) {
                        const float4 ww = *reinterpret_cast<const float4 *>(wt + t * GP + g);
                        w2[g] = make_float2(ww.x, ww.y);
                        w2[g + 1] = make_float2(ww.z, ww.w);
                    }
                } else {
                    w2[0] = wt[t * GP];
                }
#pragma unroll
                for (int g = 0; g < G; ++g)
#pragma unroll
                    for (int k = 0; k < 4; ++k) acc2[g][k] = __ffma2_rn(w2[g], v[k], acc2[g][k]);
            }
        }
        // ---- weights of the next block, in the same straight-line stretch so the two interleave
        float alpha_next = 1.0f;
        if (it + 1 < n_my) alpha_next = prepare(it + 1, masks_next);
        // ---- Tier-2 values for the heads that were promoted (rare)
        if (vm) {
            const int n_valid = (b == nact - 1) ? last_valid : BS;
            const T2 *vblk = t2_value_block<T2>(c, kv, b);
            // all eight rows of this half warp are requested before the first is used
            Raw8<T2> vr[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const int t = 2 * i + hw;
                vr[i] = (t < n_valid && vblk != nullptr) ? raw_load8<T2>(vblk + t * D + 8 * L) : raw_zero8<T2>();
            }
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const int t = 2 * i + hw;
                float v16[8];
                raw_to_f(vr[i], v16);
#pragma unroll
                for (int g = 0; g < G; ++g) {
                    if (!(vm & (1u << g))) continue;
                    const float2 w2 = w16_tiles[((it & 1) * BS + t) * GP + g];
#pragma unroll
                    for (int k = 0; k < 4; ++k)
                        acc2[g][k] = __ffma2_rn(w2, make_float2(v16[2 * k], v16[2 * k + 1]), acc2[g][k]);
                }
            }
        }
        alpha_cur = alpha_next;
    }
    att_wait<0>();
    // per-head (m, l) for the CTA merge: l is summed over the lanes of a head first
#pragma unroll
    for (int o = LPH / 2; o >= 1; o >>= 1) l_mine += __shfl_xor_sync(FULL, l_mine, o);
    float m[G], l[G];
    float acc[G][8];
#pragma unroll
    for (int g = 0; g < G; ++g) {
        m[g] = __shfl_sync(FULL, m_mine, (g * LPH) & 31);
        l[g] = __shfl_sync(FULL, l_mine, (g * LPH) & 31);
#pragma unroll
        for (int k = 0; k < 4; ++k) { acc[g][2 * k] = acc2[g][k].x; acc[g][2 * k + 1] = acc2[g][k].y; }
    }
    __syncthreads();  // the ring is reused as merge buffers
    float *sm_m = reinterpret_cast<float *>(ring);
    float *sm_l = sm_m + ATT_WARPS * G;
    float *sm_acc = sm_l + ATT_WARPS * G;
    cta_merge_store<G>(m, l, acc, sm_m, sm_l, sm_acc, ws.part_m, ws.part_l, ws.part_acc, kv * G, split, ns);
    if (take_ticket(ws.tickets + kv, ns, &s_flag))
        final_merge(ws.part_m, ws.part_l, ws.part_acc, ns, kv * G, G, ws, false, reinterpret_cast<float *>(ring),
                    c.kv_heads * G);
}

template <int G, typename T2>
__global__ void __launch_bounds__(ATT_THREADS, CQA_ATT_MIN_CTAS) attend_kernel(cqa_cache c, cqa_workspace ws, const void *q,
                                                               int q_dtype, long nq, long nact, long num_tokens,
                                                               int last_valid, float q_scale, int blocks_per_split)
{
    attend_body<G, T2>(c, ws, q, q_dtype, nq, nact, num_tokens, last_valid, q_scale, blocks_per_split);
}

// Sequence blockIdx.z of a batch.  grid.x = dense pool + the largest split count of the batch; CTAs beyond a
// sequence's own split count have nothing to do.
template <int G, typename T2>
__global__ void __launch_bounds__(ATT_THREADS, CQA_ATT_MIN_CTAS) attend_batched_kernel(const cqa_batch_item *items, int q_dtype,
                                                                                      float q_scale, int do_append)
{
    const cqa_batch_item &it = *stage_batch_item(items + blockIdx.z);
    const long num_tokens = it.pos + do_append;
    const long nq = num_tokens / BS, nact = (num_tokens + BS - 1) / BS;
    const int ns = it.ws.num_splits;
    if ((int)blockIdx.x >= DENSE_POOL_X + ns) return;
    const int last_valid = nact == nq ? BS : (int)(num_tokens - nq * BS);
    attend_body<G, T2>(it.cache, it.ws, it.q, q_dtype, nq, nact, num_tokens, last_valid, q_scale, (int)((nact + ns - 1) / ns));
}

template <int G>
static size_t attend_smem()
{
    using LY = AttLayout<G>;
    size_t dense_bytes = (size_t)(2 * CQA_MAX_DENSE_SPLITS + 8 + 8 * D + 2 * ATT_WARPS + ATT_WARPS * D) * 4;
    size_t mixed = ((size_t)LY::TOTAL + 15) & ~(size_t)15;
    return mixed > dense_bytes ? mixed : dense_bytes;
}

template <int G, typename T2>
static int attend_launch_gt(const cqa_cache *c, const cqa_workspace *ws, const void *q, int q_dtype, long nq,
                            long nact, long num_tokens, int last_valid, float q_scale, cudaStream_t st, bool chained)
{
    const int ns = ws->num_splits;
    const int bps = (int)((nact + ns - 1) / ns);
    const bool dense = ws->cert && ws->dense_splits > 0 && ws->dense_m && ws->dense_l && ws->dense_acc;
    cqa_workspace w = *ws;
    if (!dense) w.dense_splits = 0;
    const size_t smem = attend_smem<G>();
    static size_t granted[SMEM_ATTR_DEVICES] = {};
    const int rc_attr = check_cuda(ensure_dynamic_smem(attend_kernel<G, T2>, smem, granted), "cudaFuncSetAttribute(attend_kernel)");
    if (rc_attr) return rc_attr;
    dim3 grid((unsigned)(ns + (dense ? DENSE_POOL_X : 0)), (unsigned)c->kv_heads);
    return check_cuda(launch_chained(attend_kernel<G, T2>, grid, dim3(ATT_THREADS), smem, st, chained, *c, w, q, q_dtype, nq,
                                     nact, num_tokens, last_valid, q_scale, bps),
                      "attend_kernel");
}

template <typename T2>
static int attend_launch_t(const cqa_cache *c, const cqa_workspace *ws, const void *q, int q_dtype, long nq,
                           long nact, long num_tokens, int last_valid, float q_scale, cudaStream_t st, bool chained)
{
    switch (c->gqa_group) {
    case 1: return attend_launch_gt<1, T2>(c, ws, q, q_dtype, nq, nact, num_tokens, last_valid, q_scale, st, chained);
    case 2: return attend_launch_gt<2, T2>(c, ws, q, q_dtype, nq, nact, num_tokens, last_valid, q_scale, st, chained);
    case 4: return attend_launch_gt<4, T2>(c, ws, q, q_dtype, nq, nact, num_tokens, last_valid, q_scale, st, chained);
    case 8: return attend_launch_gt<8, T2>(c, ws, q, q_dtype, nq, nact, num_tokens, last_valid, q_scale, st, chained);
    }
    set_error("cqa_attend: unsupported gqa_group %d", c->gqa_group);
    return CQA_ERR_UNSUPPORTED;
}

// Argument checks of Phase 2 (also called by the fused step before its first launch).
int attend_check(const cqa_cache *c, const cqa_workspace *ws, long nq, long nact, int last_valid)
{
    if (ws->num_splits <= 0 || !ws->part_m || !ws->part_l || !ws->part_acc || (!ws->out && !ws->partial_out) || !ws->topk_mask ||
        !ws->value_mask || !ws->tickets) {
        set_error("cqa_attend: workspace is missing partial buffers, tickets, masks or the output");
        return CQA_ERR_INVALID;
    }
    if (nq > 0 && !ws->token_scores) { set_error("cqa_attend: token_scores missing"); return CQA_ERR_INVALID; }
    if (((uintptr_t)ws->token_scores | (uintptr_t)c->values_int4_packed | (uintptr_t)c->values_int4_scales |
         (uintptr_t)c->values_int4_zeros) & 15) {
        set_error("cqa_attend: token_scores and the INT4 value arrays must be 16-byte aligned (16-byte copies)");
        return CQA_ERR_INVALID;
    }
    if (nq < 0 || nact <= 0 || nact < nq || nact > ws->ld || nact > c->max_blocks) {
        set_error("cqa_attend: nact=%ld out of range (nq=%ld, ld=%ld, max_blocks=%ld)", nact, nq, (long)ws->ld,
                  (long)c->max_blocks);
        return CQA_ERR_INVALID;
    }
    if (ws->num_splits > CQA_MAX_SPLITS || ws->dense_splits > CQA_MAX_DENSE_SPLITS) {
        set_error("cqa_attend: at most %d splits and %d dense splits", CQA_MAX_SPLITS, CQA_MAX_DENSE_SPLITS);
        return CQA_ERR_TOO_LARGE;
    }
    if (ws->num_splits > nact) { set_error("cqa_attend: more splits (%d) than blocks (%ld)", ws->num_splits, nact); return CQA_ERR_INVALID; }
    if (last_valid < 1 || last_valid > BS) { set_error("cqa_attend: last_block_valid=%d", last_valid); return CQA_ERR_INVALID; }
    if (!c->keys_t2 || !c->values_t2) {
        set_error("cqa_attend: Tier-2 key/value arrays are required (promoted and trailing blocks read them)");
        return CQA_ERR_INVALID;
    }
    // A certificate can flag heads for the dense recompute; their rows are then written by the dense pool only.
    // Without the dense scratch nothing would write them, so that combination is refused instead of leaving
    // stale rows in the output.
    if (ws->cert != nullptr && (ws->dense_splits <= 0 || !ws->dense_m || !ws->dense_l || !ws->dense_acc)) {
        set_error("cqa_attend: a certificate is attached (ws->cert) but the dense-recompute scratch "
                  "(dense_splits, dense_m, dense_l, dense_acc) is missing; pass it, or detach the certificate");
        return CQA_ERR_INVALID;
    }
    if (ws->cert != nullptr && !ws->any_flags) { set_error("cqa_attend: certificate without flag words"); return CQA_ERR_INVALID; }
    if (c->t2_dtype < 0 || c->t2_dtype > 2) { set_error("cqa_attend: unknown Tier-2 dtype %d", c->t2_dtype); return CQA_ERR_INVALID; }
    return CQA_OK;
}

// `chained`: the previous kernel on the stream is the selector of the same fused step, so the kernel may be
// scheduled early and stage its first blocks (written two kernels back) before waiting for the selector.
int attend_launch(const cqa_cache *c, const cqa_workspace *ws, const void *q, int q_dtype, long nq, long nact,
                  long num_tokens, int last_valid, float q_scale, cudaStream_t st, bool chained)
{
    const int rc = attend_check(c, ws, nq, nact, last_valid);
    if (rc) return rc;
    switch (c->t2_dtype) {
    case CQA_F32: return attend_launch_t<float>(c, ws, q, q_dtype, nq, nact, num_tokens, last_valid, q_scale, st, chained);
    case CQA_F16: return attend_launch_t<__half>(c, ws, q, q_dtype, nq, nact, num_tokens, last_valid, q_scale, st, chained);
    default: return attend_launch_t<__nv_bfloat16>(c, ws, q, q_dtype, nq, nact, num_tokens, last_valid, q_scale, st, chained);
    }
}

template <int G, typename T2>
static int attend_batched_launch_gt(const cqa_batch_item *items_dev, int n_items, int kv_heads, int max_splits, int q_dtype,
                                    float q_scale, int do_append, cudaStream_t st)
{
    const size_t smem = attend_smem<G>();
    static size_t granted[SMEM_ATTR_DEVICES] = {};
    const int rc = check_cuda(ensure_dynamic_smem(attend_batched_kernel<G, T2>, smem, granted),
                              "cudaFuncSetAttribute(attend_batched_kernel)");
    if (rc) return rc;
    dim3 grid((unsigned)(DENSE_POOL_X + max_splits), (unsigned)kv_heads, (unsigned)n_items);
    return check_cuda(launch_chained(attend_batched_kernel<G, T2>, grid, dim3(ATT_THREADS), smem, st, true, items_dev, q_dtype,
                                     q_scale, do_append), "attend_batched_kernel");
}

template <typename T2>
static int attend_batched_launch_t(const cqa_batch_item *items_dev, int n_items, int kv_heads, int gqa_group, int max_splits,
                                   int q_dtype, float q_scale, int do_append, cudaStream_t st)
{
    switch (gqa_group) {
    case 1: return attend_batched_launch_gt<1, T2>(items_dev, n_items, kv_heads, max_splits, q_dtype, q_scale, do_append, st);
    case 2: return attend_batched_launch_gt<2, T2>(items_dev, n_items, kv_heads, max_splits, q_dtype, q_scale, do_append, st);
    case 4: return attend_batched_launch_gt<4, T2>(items_dev, n_items, kv_heads, max_splits, q_dtype, q_scale, do_append, st);
    case 8: return attend_batched_launch_gt<8, T2>(items_dev, n_items, kv_heads, max_splits, q_dtype, q_scale, do_append, st);
    }
    set_error("cqa_layer_step_batched: unsupported gqa_group %d", gqa_group);
    return CQA_ERR_UNSUPPORTED;
}

// Phase 2 of a batch; every item was checked by the caller (attend_check) and carries the dense scratch.
int attend_batched_launch(const cqa_batch_item *items_dev, int n_items, int kv_heads, int gqa_group, int t2_dtype,
                          int max_splits, int q_dtype, float q_scale, int do_append, cudaStream_t st)
{
    switch (t2_dtype) {
    case CQA_F32: return attend_batched_launch_t<float>(items_dev, n_items, kv_heads, gqa_group, max_splits, q_dtype, q_scale, do_append, st);
    case CQA_F16: return attend_batched_launch_t<__half>(items_dev, n_items, kv_heads, gqa_group, max_splits, q_dtype, q_scale, do_append, st);
    default: return attend_batched_launch_t<__nv_bfloat16>(items_dev, n_items, kv_heads, gqa_group, max_splits, q_dtype, q_scale, do_append, st);
    }
}

// Dense recompute alone: only the pool CTAs of the kernel are launched (no split CTAs), for the heads the attached
// certificate lists (cert[h].dense with the list in any_flags[5..], or every head when any_flags[2] is set).
template <typename T2>
static int dense_launch_t(const cqa_cache *c, const cqa_workspace *ws, const void *q, int q_dtype, long num_tokens,
                          float q_scale, cudaStream_t st)
{
    cqa_workspace w = *ws;
    w.num_splits = 0;
    const long nblk = (num_tokens + BS - 1) / BS;
    dim3 grid((unsigned)DENSE_POOL_X, (unsigned)c->kv_heads);
#define CQA_DENSE_CASE(GG)                                                                                             \
    case GG: {                                                                                                         \
        const size_t smem = attend_smem<GG>();                                                                         \
        static size_t granted[SMEM_ATTR_DEVICES] = {};                                                                 \
        const int rc = check_cuda(ensure_dynamic_smem(attend_kernel<GG, T2>, smem, granted), "cudaFuncSetAttribute(attend_kernel)"); \
        if (rc) return rc;                                                                                             \
        return check_cuda(launch_chained(attend_kernel<GG, T2>, grid, dim3(ATT_THREADS), smem, st, false, *c, w, q, q_dtype, \
                                         (long)0, nblk, num_tokens, BS, q_scale, 1), "attend_kernel (dense)");         \
    }
    switch (c->gqa_group) {
        CQA_DENSE_CASE(1)
        CQA_DENSE_CASE(2)
        CQA_DENSE_CASE(4)
        CQA_DENSE_CASE(8)
    }
#undef CQA_DENSE_CASE
    set_error("cqa_dense_attend: unsupported gqa_group %d", c->gqa_group);
    return CQA_ERR_UNSUPPORTED;
}

int dense_launch(const cqa_cache *c, const cqa_workspace *ws, const void *q, int q_dtype, long num_tokens, float q_scale,
                 cudaStream_t st)
{
    if (!ws->cert || !ws->any_flags || ws->dense_splits <= 0 || ws->dense_splits > CQA_MAX_DENSE_SPLITS || !ws->dense_m ||
        !ws->dense_l || !ws->dense_acc || !ws->tickets || !ws->out) {
        set_error("cqa_dense_attend: needs cert, any_flags, the dense scratch (1..%d splits), tickets and out",
                  CQA_MAX_DENSE_SPLITS);
        return CQA_ERR_INVALID;
    }
    const bool identity = c->key_slots == nullptr && c->value_slots == nullptr;
    if (num_tokens <= 0 || (num_tokens + BS - 1) / BS > c->max_blocks ||
        (identity && (num_tokens > c->keys_t2_rows || num_tokens > c->values_t2_rows))) {
        set_error("cqa_dense_attend: num_tokens=%ld out of range", num_tokens);
        return CQA_ERR_INVALID;
    }
    if (!c->keys_t2 || !c->values_t2) { set_error("cqa_dense_attend: Tier-2 arrays missing"); return CQA_ERR_INVALID; }
    if (q_dtype < 0 || q_dtype > 2) { set_error("cqa_dense_attend: unknown q dtype"); return CQA_ERR_INVALID; }
    switch (c->t2_dtype) {
    case CQA_F32: return dense_launch_t<float>(c, ws, q, q_dtype, num_tokens, q_scale, st);
    case CQA_F16: return dense_launch_t<__half>(c, ws, q, q_dtype, num_tokens, q_scale, st);
    case CQA_BF16: return dense_launch_t<__nv_bfloat16>(c, ws, q, q_dtype, num_tokens, q_scale, st);
    }
    set_error("cqa_dense_attend: unknown Tier-2 dtype %d", c->t2_dtype);
    return CQA_ERR_INVALID;
}

// Merge of per-rank partial rows (max, sum, acc[128]) of every head: one CTA per head, one thread per channel.
__global__ void __launch_bounds__(D) merge_partials_kernel(const float *parts, int n_parts, int n_heads, float *out)
{
    const int h = blockIdx.x, ch = threadIdx.x;
    float M = -INFINITY;
    for (int p = 0; p < n_parts; ++p) M = fmaxf(M, parts[((long)p * n_heads + h) * CQA_PARTIAL_STRIDE]);
    float l = 0.0f, a = 0.0f;
    for (int p = 0; p < n_parts; ++p) {
        const float *row = parts + ((long)p * n_heads + h) * CQA_PARTIAL_STRIDE;
        const float sc = row[0] == -INFINITY ? 0.0f : fexp(row[0] - M);
        l = fmaf(row[1], sc, l);
        a = fmaf(row[2 + ch], sc, a);
    }
    out[(long)h * D + ch] = a / (l > 0.0f ? l : 1.0f);
}

int merge_partials_launch(const float *parts, int n_parts, int n_heads, float *out, cudaStream_t st)
{
    merge_partials_kernel<<<n_heads, D, 0, st>>>(parts, n_parts, n_heads, out); note_launch();
    return check_launch("merge_partials_kernel");
}

// ---------------------------------------------------------------------------
// Built-in scratch for cqa_attend_static: split partials and merge tickets for
// callers that cannot allocate device memory.
// Layout: [Phase-2 m | l | acc][dense m | l | acc][tickets (int32)].
constexpr long STATIC_P2 = (long)CQA_STATIC_MAX_HEADS * CQA_STATIC_MAX_SPLITS;
constexpr long STATIC_DN = (long)CQA_STATIC_MAX_HEADS * CQA_STATIC_MAX_DENSE_SPLITS;
constexpr long STATIC_TICKETS = 2 * CQA_STATIC_MAX_HEADS;
constexpr long STATIC_FLOATS = STATIC_P2 * (D + 2) + STATIC_DN * (D + 2) + STATIC_TICKETS;
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
    w.tickets = reinterpret_cast<int32_t *>(dn + STATIC_DN * (D + 2));
    // The merge tickets are the only part of the shared array that must start at zero.
    rc = check_cuda(cudaMemsetAsync(w.tickets, 0, STATIC_TICKETS * sizeof(int32_t), st), "cudaMemsetAsync(tickets)");
    if (rc) return rc;
    return attend_launch(c, &w, q, q_dtype, nq, nact, num_tokens, last_valid, q_scale, st, false);
}

}  // namespace cqa
