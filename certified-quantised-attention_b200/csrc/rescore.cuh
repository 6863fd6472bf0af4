// FP16-key block re-score and Delta bound, shared by the stand-alone entry
// points and the certifier kernel.
#pragma once
#include "common.cuh"

namespace cqa {

// ------------------------------------------------------ FP16 block re-score

// One warp scores one (head, block): 16 token logits from Tier-2 keys, then
// m = max, logmass = m + log(max(sum exp(logit - m), 1e-30)).  Tokens with
// block*16+t >= n_scoring_tokens, or of a block held by neither tier, are -inf.
template <typename T2>
__device__ __forceinline__ void fp16_block_score_warp(const cqa_cache &c, const void *q, int q_dtype, int h,
                                                      long bid, long n_scoring_tokens, float q_scale,
                                                      float &score_out, float &logmass_out,
                                                      const float *q_row = nullptr)
{
    const int lane = threadIdx.x & 31, L = lane & 15, hw = lane >> 4;
    const int kv = h / c.gqa_group;
    const bool valid_block = bid >= 0 && bid * BS < n_scoring_tokens;
    const T2 *base = valid_block ? t2_key_block<T2>(c, kv, bid) : nullptr;   // hot slot or backing array
    // q_row: the head's 128 query values already converted to float (shared memory), fetched by the caller ahead of time
    float qv[8];
    if (q_row != nullptr) {
#pragma unroll
        for (int i = 0; i < 8; ++i) qv[i] = q_row[8 * L + i];
    } else {
        load_q8(q, q_dtype, (long)h * D + 8 * L, qv);
    }
    float lg[8];  // this half warp's tokens hw*8 .. hw*8+7 (all lanes hold all 8)
    // issue the eight row loads together, then reduce (small code: this runs once per launch)
    Raw8<T2> raw[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const int t = hw * 8 + i;
        const bool valid = base != nullptr && (bid * BS + t) < n_scoring_tokens;
        raw[i] = valid ? raw_load8<T2>(base + t * D + 8 * L) : raw_zero8<T2>();
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const int t = hw * 8 + i;
        const bool valid = base != nullptr && (bid * BS + t) < n_scoring_tokens;
        float kf[8];
        raw_to_f(raw[i], kf);
        float d = hw_sum(chain8(kf, qv));
        lg[i] = valid ? __fmul_rn(d, q_scale) : -INFINITY;
    }
    float mx = lg[0];
#pragma unroll
    for (int i = 1; i < 8; ++i) mx = fmaxf(mx, lg[i]);
    mx = fmaxf(mx, __shfl_xor_sync(FULL, mx, 16));
    float e[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) e[i] = lg[i] == -INFINITY ? 0.0f : cexp(__fsub_rn(lg[i], mx));
    // butterfly over the 16 tokens: stride 8 pairs token i with i+8 (other half warp)
#pragma unroll
    for (int i = 0; i < 8; ++i) e[i] = __fadd_rn(e[i], __shfl_xor_sync(FULL, e[i], 16));
#pragma unroll
    for (int i = 0; i < 4; ++i) e[i] = __fadd_rn(e[i], e[i + 4]);
    e[0] = __fadd_rn(e[0], e[2]);
    e[1] = __fadd_rn(e[1], e[3]);
    float l = fmaxf(__fadd_rn(e[0], e[1]), 1e-30f);
    score_out = mx;
    logmass_out = mx == -INFINITY ? -INFINITY : __fadd_rn(mx, clog(l));
}

// Delta[h] = dot(|q_h|, sigma_max[kv]) / (2 sqrt(128))
// `ranks` > 1: sigma_max is one row per rank, `rank_stride` floats apart (sequence sharding); the maximum is taken.
__device__ __forceinline__ float delta_bound_warp(const cqa_cache &c, const void *q, int q_dtype, int h, int ranks = 1,
                                                  long rank_stride = 0)
{
    const int L = threadIdx.x & 15, hw = (threadIdx.x >> 4) & 1;
    const int kv = h / c.gqa_group;
    float qa[8], sg[8];
    load_q8(q, q_dtype, (long)h * D + 8 * L, qa);
#pragma unroll
    for (int i = 0; i < 8; ++i) { qa[i] = fabsf(qa[i]); sg[i] = 0.0f; }      // scales are positive
    // the ranks' rows are split over the two half warps and fetched four ranks at a time (a chain of dependent
    // loads, one rank after the other, was several microseconds long with eight ranks)
#pragma unroll 4
    for (int r = hw; r < ranks; r += 2) {
        const float4 *row = reinterpret_cast<const float4 *>(c.sigma_max + (long)r * rank_stride + kv * D + 8 * L);
        const float4 a = row[0], b = row[1];
        sg[0] = fmaxf(sg[0], a.x); sg[1] = fmaxf(sg[1], a.y); sg[2] = fmaxf(sg[2], a.z); sg[3] = fmaxf(sg[3], a.w);
        sg[4] = fmaxf(sg[4], b.x); sg[5] = fmaxf(sg[5], b.y); sg[6] = fmaxf(sg[6], b.z); sg[7] = fmaxf(sg[7], b.w);
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) sg[i] = fmaxf(sg[i], __shfl_xor_sync(0xFFFFFFFFu, sg[i], 16));
    const float denom = 22.627416997969522f;  // 2*sqrt(128) rounded to binary32
    return __fdiv_rn(hw_sum(chain8(qa, sg)), denom);
}


}  // namespace cqa
