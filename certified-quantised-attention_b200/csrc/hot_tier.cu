// Bounded hot tier: device-side residency bookkeeping and page-in of the
// Tier-2 blocks a step used (reference: ensure_fp16_{keys,values}_resident,
// _page_in_fp16_blocks, _prepare_bounded_fp16_key_scratch,
// tiered_kv_cache.py:986-1537; backends/cuda_pagein.*).
//
// The attend and certifier kernels read a non-resident block straight from the
// backing array (pinned host memory), so a miss costs bandwidth, never a wait.
// After the step, three small launches make the next steps faster:
//   mark   one thread per block: the block was used if any head has it in the
//          FP16-key mask (tier 0) / FP16-value mask (tier 1).  Resident ->
//          stamp its slot with the step number (hit); not resident -> append
//          to the miss list.
//   assign one warp per tier walks the slots from the clock hand, takes those
//          not stamped in this step, evicts their owners and hands them to
//          the missed blocks (at most max_fill_blocks per call).
//   fill   one CTA per (assigned block, KV head) copies the 16 rows from the
//          backing array into the slot.
// Everything is stream-ordered; no kernel waits on another.
#include "common.cuh"

namespace cqa {

constexpr int HT_STEP = 0, HT_HAND = 1, HT_TIER0 = 3;   // counters layout: [step, hand_k, hand_v, k:{hit,miss,fill,evict}, v:{...}]

struct HotTierView {
    int32_t *slots, *owner, *stamp, *work;
    int64_t *ctr;   // hits, misses, page-ins, evictions of this tier
    int64_t *hand;
};

__device__ __forceinline__ HotTierView tier_view(const cqa_hot_tier &ht, int tier, long max_blocks)
{
    HotTierView v;
    v.slots = tier == 0 ? ht.key_slots : ht.value_slots;
    v.owner = tier == 0 ? ht.key_owner : ht.value_owner;
    v.stamp = tier == 0 ? ht.key_stamp : ht.value_stamp;
    v.work = ht.work + (long)tier * (2 + 3 * max_blocks);
    v.ctr = ht.counters + HT_TIER0 + 4 * tier;
    v.hand = ht.counters + HT_HAND + tier;
    return v;
}

__global__ void __launch_bounds__(256) hot_mark_kernel(cqa_hot_tier ht, cqa_workspace ws, int n_heads, long nact,
                                                      long max_blocks)
{
    const int tier = blockIdx.y;
    const HotTierView v = tier_view(ht, tier, max_blocks);
    const long b = (long)blockIdx.x * blockDim.x + threadIdx.x;
    if (b >= nact) return;
    const unsigned char *mask = tier == 0 ? ws.topk_mask : ws.value_mask;
    bool used = false;
    for (int h = 0; h < n_heads; ++h) used |= mask[(long)h * ws.ld + b] != 0;
    if (!used) return;
    const int step = (int)ht.counters[HT_STEP];
    const int s = v.slots[b];
    if (s >= 0) {
        v.stamp[s] = step;
        atomicAdd(reinterpret_cast<unsigned long long *>(v.ctr + 0), 1ull);
    } else {
        const int i = atomicAdd(v.work + 0, 1);
        v.work[2 + i] = (int)b;
        atomicAdd(reinterpret_cast<unsigned long long *>(v.ctr + 1), 1ull);
    }
}

__global__ void __launch_bounds__(32) hot_assign_kernel(cqa_hot_tier ht, long max_blocks)
{
    const int tier = blockIdx.x, lane = threadIdx.x;
    const HotTierView v = tier_view(ht, tier, max_blocks);
    const int step = (int)ht.counters[HT_STEP];
    const int cap = tier == 0 ? ht.key_capacity_blocks : ht.value_capacity_blocks;
    int n_miss = v.work[0];
    if (n_miss > ht.max_fill_blocks) n_miss = ht.max_fill_blocks;
    int hand = (int)(*v.hand % cap);
    int given = 0;
    // walk the slots once from the hand, 32 at a time; a slot is free for taking if it was not used in this step
    for (int base = 0; base < cap && given < n_miss; base += 32) {
        const int idx = base + lane;
        int s = hand + idx;
        if (s >= cap) s -= cap;
        const bool ok = idx < cap && v.stamp[s] != step;
        const unsigned who = __ballot_sync(FULL, ok);
        const int rank = given + __popc(who & ((1u << lane) - 1u));
        if (ok && rank < n_miss) {
            const int b = v.work[2 + rank];
            const int old = v.owner[s];
            if (old >= 0) {
                v.slots[old] = -1;
                atomicAdd(reinterpret_cast<unsigned long long *>(v.ctr + 3), 1ull);
            }
            v.owner[s] = b;
            v.slots[b] = s;
            v.stamp[s] = step;
            v.work[2 + max_blocks + 2 * rank] = b;
            v.work[2 + max_blocks + 2 * rank + 1] = s;
        }
        given += __popc(who);
        if (given >= n_miss) {
            // the hand stops behind the last slot taken
            const int taken_in_chunk = n_miss - (given - __popc(who));
            int last = -1;
            unsigned w = who;
            for (int k = 0; k < taken_in_chunk; ++k) { last = __ffs(w) - 1; w &= w - 1; }
            hand = hand + base + last + 1;
        }
    }
    if (given > n_miss) given = n_miss;
    __syncwarp();
    if (lane == 0) {
        if (given < n_miss || n_miss == 0) hand = (int)(*v.hand % cap);   // nothing (more) to take: the hand stays
        *v.hand = hand % cap;
        v.work[1] = given;
        v.ctr[2] += given;
    }
}

template <typename T2>
__global__ void __launch_bounds__(128) hot_fill_kernel(cqa_hot_tier ht, cqa_cache c, long max_blocks)
{
    const int tier = blockIdx.z, kv = blockIdx.y, i = blockIdx.x;
    const HotTierView v = tier_view(ht, tier, max_blocks);
    if (i >= v.work[1]) return;
    const long b = v.work[2 + max_blocks + 2 * i], s = v.work[2 + max_blocks + 2 * i + 1];
    const void *backing = tier == 0 ? c.keys_t2_backing : c.values_t2_backing;
    void *hot = tier == 0 ? c.keys_t2 : c.values_t2;
    const long hot_rows = tier == 0 ? c.keys_t2_rows : c.values_t2_rows;
    const uint4 *src = reinterpret_cast<const uint4 *>(reinterpret_cast<const T2 *>(backing) +
                                                       ((long)kv * c.t2_backing_rows + b * BS) * D);
    uint4 *dst = reinterpret_cast<uint4 *>(reinterpret_cast<T2 *>(hot) + ((long)kv * hot_rows + s * BS) * D);
    constexpr int N16 = BS * D * (int)sizeof(T2) / 16;
    for (int k = threadIdx.x; k < N16; k += 128) dst[k] = src[k];
}

__global__ void hot_finish_kernel(cqa_hot_tier ht, long max_blocks)
{
    // next step; clear the per-step lists
    if (threadIdx.x == 0) {
        ht.counters[HT_STEP] += 1;
        for (int tier = 0; tier < 2; ++tier) {
            int32_t *w = ht.work + (long)tier * (2 + 3 * max_blocks);
            w[0] = 0;
            w[1] = 0;
        }
    }
}

}  // namespace cqa

using namespace cqa;

extern "C" int cqa_hot_tier_update(const cqa_cache *c, const cqa_workspace *ws, const cqa_hot_tier *ht, int64_t nact,
                                   void *stream)
{
    if (!c || !ws || !ht) { set_error("cqa_hot_tier_update: NULL pointer"); return CQA_ERR_INVALID; }
    if (!ht->key_slots || !ht->value_slots || !ht->key_owner || !ht->value_owner || !ht->key_stamp || !ht->value_stamp ||
        !ht->work || !ht->counters || ht->key_capacity_blocks <= 0 || ht->value_capacity_blocks <= 0 ||
        ht->max_fill_blocks <= 0) {
        set_error("cqa_hot_tier_update: incomplete hot-tier state");
        return CQA_ERR_INVALID;
    }
    if (!c->keys_t2_backing || !c->values_t2_backing || !c->keys_t2 || !c->values_t2 || c->key_slots != ht->key_slots ||
        c->value_slots != ht->value_slots) {
        set_error("cqa_hot_tier_update: the cache is not in bounded hot-tier mode (slot tables and backing arrays)");
        return CQA_ERR_INVALID;
    }
    if (!ws->topk_mask || !ws->value_mask || nact <= 0 || nact > c->max_blocks || nact > ws->ld) {
        set_error("cqa_hot_tier_update: bad masks or block count");
        return CQA_ERR_INVALID;
    }
    if (ht->key_capacity_blocks * (int64_t)BS > c->keys_t2_rows ||
        ht->value_capacity_blocks * (int64_t)BS > c->values_t2_rows) {
        set_error("cqa_hot_tier_update: capacity exceeds the scratch arrays");
        return CQA_ERR_INVALID;
    }
    cudaStream_t st = (cudaStream_t)stream;
    const int H = c->kv_heads * c->gqa_group;
    dim3 gm((unsigned)((nact + 255) / 256), 2);
    hot_mark_kernel<<<gm, 256, 0, st>>>(*ht, *ws, H, nact, c->max_blocks);
    hot_assign_kernel<<<2, 32, 0, st>>>(*ht, c->max_blocks);
    dim3 gf((unsigned)ht->max_fill_blocks, (unsigned)c->kv_heads, 2);
    switch (c->t2_dtype) {
    case CQA_F32: hot_fill_kernel<float><<<gf, 128, 0, st>>>(*ht, *c, c->max_blocks); break;
    case CQA_F16: hot_fill_kernel<__half><<<gf, 128, 0, st>>>(*ht, *c, c->max_blocks); break;
    case CQA_BF16: hot_fill_kernel<__nv_bfloat16><<<gf, 128, 0, st>>>(*ht, *c, c->max_blocks); break;
    default: set_error("cqa_hot_tier_update: unknown Tier-2 dtype"); return CQA_ERR_INVALID;
    }
    hot_finish_kernel<<<1, 32, 0, st>>>(*ht, c->max_blocks);
    return check_launch("hot tier kernels");
}
