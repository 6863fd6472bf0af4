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

// The same marking for an explicit list of block ids of one tier (a caller that knows which blocks it is about to
// read asks for them by name; reference: ensure_fp16_keys_resident / ensure_fp16_values_resident).
__global__ void __launch_bounds__(256) hot_mark_list_kernel(cqa_hot_tier ht, int tier, const int64_t *blocks, long n,
                                                           long max_blocks)
{
    const HotTierView v = tier_view(ht, tier, max_blocks);
    const long i = (long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const long b = blocks[i];
    if (b < 0 || b >= max_blocks) return;
    const int step = (int)ht.counters[HT_STEP];
    const int s = v.slots[b];
    if (s >= 0) {
        v.stamp[s] = step;
        atomicAdd(reinterpret_cast<unsigned long long *>(v.ctr + 0), 1ull);
    } else {
        const int k = atomicAdd(v.work + 0, 1);
        v.work[2 + k] = (int)b;
        atomicAdd(reinterpret_cast<unsigned long long *>(v.ctr + 1), 1ull);
    }
}

// Gather of 16-row blocks from a backing array (row = token index) into the slots of a scratch array, 16 bytes per
// thread and step.  grid (blocks, KV).  Rows at or beyond active_tokens are not copied.
__global__ void __launch_bounds__(128) page_in_gather_kernel(const char *src, long src_rows, char *dst, long dst_rows,
                                                            long row_bytes, const int64_t *blocks,
                                                            const int32_t *slots, const int32_t *slot_of_block,
                                                            long active_tokens)
{
    const int kv = blockIdx.y;
    // two addressing forms: (blocks[i], slots[i]) pairs, or block i with slot slot_of_block[i]
    const long b = blocks ? blocks[blockIdx.x] : (long)blockIdx.x;
    const long s = blocks ? (long)slots[blockIdx.x] : (long)slot_of_block[blockIdx.x];
    if (b < 0 || s < 0 || (s + 1) * BS > dst_rows || b * BS >= src_rows) return;
    long rows = active_tokens - b * BS;
    if (rows > BS) rows = BS;
    if (rows <= 0) return;
    const uint4 *from = reinterpret_cast<const uint4 *>(src + ((long)kv * src_rows + b * BS) * row_bytes);
    uint4 *to = reinterpret_cast<uint4 *>(dst + ((long)kv * dst_rows + s * BS) * row_bytes);
    const long n16 = rows * row_bytes / 16;
    for (long k = threadIdx.x; k < n16; k += 128) to[k] = from[k];
}

__global__ void __launch_bounds__(256) slot_table_update_kernel(const int64_t *loaded_blocks, const int32_t *loaded_slots,
                                                               long n_loaded, const int64_t *evicted_blocks,
                                                               long n_evicted, int32_t *table, long table_size)
{
    const long i = (long)blockIdx.x * blockDim.x + threadIdx.x;
    // evictions first, then loads, in two grid-strided halves of the same launch would race when a block is both
    // evicted and loaded; the loads therefore win by being applied by the same thread after its eviction
    if (i < n_evicted) {
        const long b = evicted_blocks[i];
        bool reloaded = false;
        for (long j = 0; j < n_loaded; ++j) reloaded |= loaded_blocks[j] == b;
        if (b >= 0 && b < table_size && !reloaded) table[b] = -1;
    }
    if (i < n_loaded) {
        const long b = loaded_blocks[i];
        if (b >= 0 && b < table_size) table[b] = loaded_slots[i];
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

static int check_hot_tier(const cqa_cache *c, const cqa_hot_tier *ht, const char *who)
{
    if (!ht->key_slots || !ht->value_slots || !ht->key_owner || !ht->value_owner || !ht->key_stamp || !ht->value_stamp ||
        !ht->work || !ht->counters || ht->key_capacity_blocks <= 0 || ht->value_capacity_blocks <= 0 ||
        ht->max_fill_blocks <= 0) {
        set_error("%s: incomplete hot-tier state", who);
        return CQA_ERR_INVALID;
    }
    if (!c->keys_t2_backing || !c->values_t2_backing || !c->keys_t2 || !c->values_t2 || c->key_slots != ht->key_slots ||
        c->value_slots != ht->value_slots) {
        set_error("%s: the cache is not in bounded hot-tier mode (slot tables and backing arrays)", who);
        return CQA_ERR_INVALID;
    }
    if (ht->key_capacity_blocks * (int64_t)BS > c->keys_t2_rows ||
        ht->value_capacity_blocks * (int64_t)BS > c->values_t2_rows) {
        set_error("%s: capacity exceeds the scratch arrays", who);
        return CQA_ERR_INVALID;
    }
    if (c->t2_dtype < 0 || c->t2_dtype > 2) { set_error("%s: unknown Tier-2 dtype", who); return CQA_ERR_INVALID; }
    return CQA_OK;
}

static void launch_fill(const cqa_cache *c, const cqa_hot_tier *ht, cudaStream_t st)
{
    dim3 gf((unsigned)ht->max_fill_blocks, (unsigned)c->kv_heads, 2);
    switch (c->t2_dtype) {
    case CQA_F32: hot_fill_kernel<float><<<gf, 128, 0, st>>>(*ht, *c, c->max_blocks); note_launch(); break;
    case CQA_F16: hot_fill_kernel<__half><<<gf, 128, 0, st>>>(*ht, *c, c->max_blocks); note_launch(); break;
    default: hot_fill_kernel<__nv_bfloat16><<<gf, 128, 0, st>>>(*ht, *c, c->max_blocks); note_launch(); break;
    }
}

extern "C" int cqa_hot_tier_ensure(const cqa_cache *c, const cqa_hot_tier *ht, int tier, const int64_t *block_ids,
                                   int64_t n, void *stream)
{
    if (!c || !ht || (n > 0 && !block_ids)) { set_error("cqa_hot_tier_ensure: NULL pointer"); return CQA_ERR_INVALID; }
    if (tier != 0 && tier != 1) { set_error("cqa_hot_tier_ensure: tier must be 0 (keys) or 1 (values)"); return CQA_ERR_INVALID; }
    if (n < 0 || n > c->max_blocks) { set_error("cqa_hot_tier_ensure: %ld block ids", (long)n); return CQA_ERR_INVALID; }
    const int rc = check_hot_tier(c, ht, "cqa_hot_tier_ensure");
    if (rc) return rc;
    cudaStream_t st = (cudaStream_t)stream;
    // the counters before this call, for callers that report per-call figures
    cudaMemcpyAsync(ht->counters + 12, ht->counters, 12 * sizeof(int64_t), cudaMemcpyDeviceToDevice, st);
    if (n > 0) {
        hot_mark_list_kernel<<<(unsigned)((n + 255) / 256), 256, 0, st>>>(*ht, tier, block_ids, n, c->max_blocks);
        note_launch();
    }
    hot_assign_kernel<<<2, 32, 0, st>>>(*ht, c->max_blocks); note_launch();
    launch_fill(c, ht, st);
    hot_finish_kernel<<<1, 32, 0, st>>>(*ht, c->max_blocks); note_launch();
    return check_launch("hot tier kernels");
}

static const char *device_view(const void *p)
{
    // pinned host memory is addressed through its device alias; device memory as it is
    cudaPointerAttributes at;
    if (cudaPointerGetAttributes(&at, p) == cudaSuccess && at.type == cudaMemoryTypeHost && at.devicePointer)
        return static_cast<const char *>(at.devicePointer);
    (void)cudaGetLastError();
    return static_cast<const char *>(p);
}

extern "C" int cqa_page_in_blocks(const void *src, int64_t src_rows, void *dst, int64_t dst_rows, int kv_heads,
                                  int row_bytes, const int64_t *loaded_blocks, const int32_t *loaded_slots,
                                  int64_t n_loaded, const int64_t *evicted_blocks, int64_t n_evicted,
                                  int32_t *slot_table, int64_t table_size, int64_t active_tokens, void *stream)
{
    if (n_loaded < 0 || n_evicted < 0 || kv_heads <= 0 || row_bytes <= 0 || (row_bytes & 15) != 0 ||
        (n_loaded > 0 && (!src || !dst || !loaded_blocks || !loaded_slots)) || (n_evicted > 0 && !evicted_blocks)) {
        set_error("cqa_page_in_blocks: bad arguments");
        return CQA_ERR_INVALID;
    }
    cudaStream_t st = (cudaStream_t)stream;
    const long n = n_loaded > n_evicted ? n_loaded : n_evicted;
    if (slot_table && n > 0) {
        slot_table_update_kernel<<<(unsigned)((n + 255) / 256), 256, 0, st>>>(loaded_blocks, loaded_slots, n_loaded,
                                                                              evicted_blocks, n_evicted, slot_table, table_size);
        note_launch();
    }
    if (n_loaded > 0) {
        dim3 grid((unsigned)n_loaded, (unsigned)kv_heads);
        page_in_gather_kernel<<<grid, 128, 0, st>>>(device_view(src), src_rows, static_cast<char *>(dst), dst_rows, row_bytes,
                                                    loaded_blocks, loaded_slots, nullptr, active_tokens); note_launch();
    }
    return check_launch("page-in kernels");
}

extern "C" int cqa_page_in_by_slots(const void *src, int64_t src_rows, void *dst, int64_t dst_rows, int kv_heads,
                                    int row_bytes, const int32_t *block_slots, int64_t n_blocks,
                                    int64_t active_tokens, void *stream)
{
    if (n_blocks < 0 || kv_heads <= 0 || row_bytes <= 0 || (row_bytes & 15) != 0 ||
        (n_blocks > 0 && (!src || !dst || !block_slots))) {
        set_error("cqa_page_in_by_slots: bad arguments");
        return CQA_ERR_INVALID;
    }
    if (n_blocks == 0) return CQA_OK;
    dim3 grid((unsigned)n_blocks, (unsigned)kv_heads);
    page_in_gather_kernel<<<grid, 128, 0, (cudaStream_t)stream>>>(device_view(src), src_rows, static_cast<char *>(dst),
                                                                  dst_rows, row_bytes, nullptr, nullptr, block_slots,
                                                                  active_tokens); note_launch();
    return check_launch("page_in_gather_kernel");
}

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
    if (c->t2_dtype < 0 || c->t2_dtype > 2) { set_error("cqa_hot_tier_update: unknown Tier-2 dtype"); return CQA_ERR_INVALID; }
    cudaStream_t st = (cudaStream_t)stream;
    const int H = c->kv_heads * c->gqa_group;
    // counters[12..23] keep the values from before this step, so the host can report per-step figures
    cudaMemcpyAsync(ht->counters + 12, ht->counters, 12 * sizeof(int64_t), cudaMemcpyDeviceToDevice, st);
    dim3 gm((unsigned)((nact + 255) / 256), 2);
    hot_mark_kernel<<<gm, 256, 0, st>>>(*ht, *ws, H, nact, c->max_blocks); note_launch();
    hot_assign_kernel<<<2, 32, 0, st>>>(*ht, c->max_blocks); note_launch();
    launch_fill(c, ht, st);
    hot_finish_kernel<<<1, 32, 0, st>>>(*ht, c->max_blocks); note_launch();
    return check_launch("hot tier kernels");
}
