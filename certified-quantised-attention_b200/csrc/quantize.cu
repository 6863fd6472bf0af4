// Block quantisers: INT8 per-channel keys, INT4 per-token-per-group values,
// error annotations, and the fused append-and-quantise step.
//
// One CTA of 128 threads works on one (kv head, 16-token block).  Keys: thread c
// owns channel c over the 16 tokens.  Values: thread (t, g) owns group g of
// token t (16 channels).  All arithmetic that lands in stored bytes is
// elementwise IEEE; the error norms use the canonical 16-lane dot order.
#include "common.cuh"

namespace cqa {

struct BlockQuantSmem {
    float scale[D];
    float tok_err[BS];
    float tok_vnorm[BS];
};

// Butterfly over the 16 lane-partials of one token held by 8 consecutive
// threads (thread g holds partials 2g and 2g+1).
__device__ __forceinline__ float group8_sum(float pa, float pb)
{
    pa = __fadd_rn(pa, __shfl_xor_sync(FULL, pa, 4));
    pb = __fadd_rn(pb, __shfl_xor_sync(FULL, pb, 4));
    pa = __fadd_rn(pa, __shfl_xor_sync(FULL, pa, 2));
    pb = __fadd_rn(pb, __shfl_xor_sync(FULL, pb, 2));
    pa = __fadd_rn(pa, __shfl_xor_sync(FULL, pa, 1));
    pb = __fadd_rn(pb, __shfl_xor_sync(FULL, pb, 1));
    return __fadd_rn(pa, pb);
}

__device__ __forceinline__ float sumsq16(const float (&x)[16], float &pa, float &pb)
{
    float a[8], b[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) { a[i] = x[i]; b[i] = x[i + 8]; }
    pa = chain8(a, a);
    pb = chain8(b, b);
    return 0.0f;
}

// INT4 quantisation of one (token, group): x[16] -> codes packed in 8 bytes,
// scale, zero, and the group's contribution to |x - deq|^2 (two lane partials).
__device__ __forceinline__ void int4_group(const float (&x)[16], uint2 &packed, float &s, float &z,
                                           float &da, float &db)
{
    float lo = x[0], hi = x[0];
#pragma unroll
    for (int i = 1; i < 16; ++i) { lo = fminf(lo, x[i]); hi = fmaxf(hi, x[i]); }
    float range = fmaxf(__fsub_rn(hi, lo), 1e-8f);
    s = __fdiv_rn(range, 15.0f);
    z = lo;
    float diff[16];
    unsigned code[16];
#pragma unroll
    for (int i = 0; i < 16; ++i) {
        float r = rintf(__fdiv_rn(__fsub_rn(x[i], z), s));
        r = fminf(fmaxf(r, 0.0f), 15.0f);
        code[i] = (unsigned)r;
        float deq = __fadd_rn(__fmul_rn(r, s), z);
        diff[i] = __fsub_rn(x[i], deq);
    }
    unsigned w0 = 0, w1 = 0;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        w0 |= (code[2 * j] | (code[2 * j + 1] << 4)) << (8 * j);
        w1 |= (code[8 + 2 * j] | (code[8 + 2 * j + 1] << 4)) << (8 * j);
    }
    packed = make_uint2(w0, w1);
    sumsq16(diff, da, db);
}

// Quantise one complete block.  ksrc/vsrc: 16 rows of 128 elements of T.
template <typename T>
__device__ void quantize_one_block(const cqa_cache &c, int kv, long blk, const T *ksrc, const T *vsrc,
                                   bool do_keys, bool do_values, bool eta_mean, bool write_nu,
                                   BlockQuantSmem &sm)
{
    const int tid = threadIdx.x;
    const long row0 = (long)kv * c.cap_tokens + blk * BS;
    const long bidx = (long)kv * c.max_blocks + blk;

    if (do_keys) {
        const int ch = tid;
        float x[BS];
#pragma unroll
        for (int t = 0; t < BS; ++t) x[t] = Cvt<T>::to_f(ksrc[t * D + ch]);
        float lo = x[0], hi = x[0];
#pragma unroll
        for (int t = 1; t < BS; ++t) { lo = fminf(lo, x[t]); hi = fmaxf(hi, x[t]); }
        float range = fmaxf(__fsub_rn(hi, lo), 1e-8f);
        float s = __fdiv_rn(range, 255.0f);
        float z = __fdiv_rn(__fadd_rn(lo, hi), 2.0f);
#pragma unroll
        for (int t = 0; t < BS; ++t) {
            float r = rintf(__fdiv_rn(__fsub_rn(x[t], z), s));
            r = fminf(fmaxf(r, -128.0f), 127.0f);
            c.keys_int8[(row0 + t) * D + ch] = (int8_t)r;
        }
        c.keys_scale[bidx * D + ch] = s;
        c.keys_zero_points[bidx * D + ch] = z;
        sm.scale[ch] = s;
        if (c.sigma_max) atomicMax(reinterpret_cast<int *>(c.sigma_max) + kv * D + ch, __float_as_int(s));
    }
    if (do_values) {
        const int t = tid >> 3, g = tid & 7;
        float xm[16], x[16];
        float a[8], b[8];
        load8<T>(vsrc + t * D + g * GS, a);
        load8<T>(vsrc + t * D + g * GS + 8, b);
#pragma unroll
        for (int i = 0; i < 8; ++i) { xm[i] = a[i]; xm[i + 8] = b[i]; }
        // values.to(float16) before quantising (prefill and deferred block paths)
#pragma unroll
        for (int i = 0; i < 16; ++i) x[i] = __half2float(__float2half_rn(xm[i]));
        uint2 packed;
        float s, z, da, db, xa, xb, na, nb;
        int4_group(x, packed, s, z, da, db);
        sumsq16(x, xa, xb);
        sumsq16(xm, na, nb);
        const long row = row0 + t;
        *reinterpret_cast<uint2 *>(c.values_int4_packed + row * (D / 2) + g * 8) = packed;
        c.values_int4_scales[row * NG + g] = __half_as_ushort(__float2half_rn(s));
        c.values_int4_zeros[row * NG + g] = __half_as_ushort(__float2half_rn(z));
        float ae = __fsqrt_rn(group8_sum(da, db));
        float xn = fmaxf(__fsqrt_rn(group8_sum(xa, xb)), 1e-6f);
        float vn = __fsqrt_rn(group8_sum(na, nb));
        if (g == 0) {
            sm.tok_err[t] = __fdiv_rn(ae, xn);
            sm.tok_vnorm[t] = vn;
        }
    }
    __syncthreads();
    if (do_keys && tid < 32) {
        const int L = tid & 15;
        float a[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) a[i] = sm.scale[8 * L + i];
        float n2 = hw_sum(chain8(a, a));
        if (tid == 0) {
            float delta = __fdiv_rn(__fsqrt_rn(n2), 127.0f);
            c.correction[bidx] = cexp(__fmul_rn(2.0f, delta));
        }
    }
    if (do_values && tid == 0) {
        float p[BS];
        float mx = sm.tok_err[0], vmx = sm.tok_vnorm[0];
#pragma unroll
        for (int i = 0; i < BS; ++i) {
            p[i] = sm.tok_err[i];
            mx = fmaxf(mx, p[i]);
            vmx = fmaxf(vmx, sm.tok_vnorm[i]);
        }
#pragma unroll
        for (int s = 8; s >= 1; s >>= 1)
#pragma unroll
            for (int i = 0; i < s; ++i) p[i] = __fadd_rn(p[i], p[i + s]);
        c.values_int4_errors[bidx] = eta_mean ? __fdiv_rn(p[0], 16.0f) : mx;
        c.values_int4_error_sums[bidx] = p[0];
        c.values_int4_error_counts[bidx] = BS;
        if (write_nu) c.values_norm_max[bidx] = vmx;
    }
    __syncthreads();
}

template <typename T>
__global__ void __launch_bounds__(128) quantize_blocks_kernel(cqa_cache c, const T *k_src, const T *v_src,
                                                             long src_rows, long first_block, int copy_t2)
{
    __shared__ BlockQuantSmem sm;
    const int kv = blockIdx.y;
    const long lb = blockIdx.x;
    const long blk = first_block + lb;
    const T *ks = k_src + ((long)kv * src_rows + lb * BS) * D;
    const T *vs = v_src + ((long)kv * src_rows + lb * BS) * D;
    if (copy_t2) {
        // full mirror: the Tier-2 arrays themselves; bounded hot tier: the backing arrays (the scratch starts empty)
        T *kd = c.key_slots ? (c.keys_t2_backing ? reinterpret_cast<T *>(c.keys_t2_backing) + ((long)kv * c.t2_backing_rows + blk * BS) * D : nullptr)
                            : (c.keys_t2 ? reinterpret_cast<T *>(c.keys_t2) + ((long)kv * c.keys_t2_rows + blk * BS) * D : nullptr);
        T *vd = c.value_slots ? (c.values_t2_backing ? reinterpret_cast<T *>(c.values_t2_backing) + ((long)kv * c.t2_backing_rows + blk * BS) * D : nullptr)
                              : (c.values_t2 ? reinterpret_cast<T *>(c.values_t2) + ((long)kv * c.values_t2_rows + blk * BS) * D : nullptr);
        for (int i = threadIdx.x; i < BS * D; i += 128) {
            if (kd) kd[i] = ks[i];
            if (vd) vd[i] = vs[i];
        }
    }
    quantize_one_block<T>(c, kv, blk, ks, vs, true, c.values_int4_packed != nullptr, false, true, sm);
    if (c.values_int4_packed == nullptr && threadIdx.x < 32) {
        // FP16-value caches still carry nu_b.
        const int lane = threadIdx.x, L = lane & 15;
        float vmx = 0.0f;
        for (int t = 0; t < BS; ++t) {
            float a[8];
            load8<T>(vs + t * D + 8 * L, a);
            vmx = fmaxf(vmx, __fsqrt_rn(hw_sum(chain8(a, a))));
        }
        if (lane == 0) c.values_norm_max[(long)kv * c.max_blocks + blk] = vmx;
    }
}

// Fused append-and-quantise of one token.  Grid: KV CTAs of 128 threads.
template <typename T2>
__device__ __forceinline__ void append_token_body(const cqa_cache &c, const void *k_new, const void *v_new, int src_dtype,
                                                  long pos, int defer_int4, long kv_stride = D, long tok_off = 0)
{
    __shared__ BlockQuantSmem sm;
    __shared__ float s_v[D];
    const int kv = blockIdx.x, tid = threadIdx.x;
    const long blk = pos / BS;
    const int pib = (int)(pos % BS);
    const long bidx = (long)kv * c.max_blocks + blk;
    grid_dependency_wait();

    long krow = pos, vrow = pos;
    if (c.key_slots) { int s = c.key_slots[blk]; krow = s < 0 ? -1 : (long)s * BS + pib; }
    if (c.value_slots) { int s = c.value_slots[blk]; vrow = s < 0 ? -1 : (long)s * BS + pib; }

    T2 kq = Cvt<T2>::from_f(load_q(k_new, src_dtype, (long)kv * kv_stride + tok_off + tid));
    T2 vq = Cvt<T2>::from_f(load_q(v_new, src_dtype, (long)kv * kv_stride + tok_off + tid));
    T2 *kt2 = reinterpret_cast<T2 *>(c.keys_t2);
    T2 *vt2 = reinterpret_cast<T2 *>(c.values_t2);
    if (kt2 && krow >= 0) kt2[((long)kv * c.keys_t2_rows + krow) * D + tid] = kq;
    if (vt2 && vrow >= 0) vt2[((long)kv * c.values_t2_rows + vrow) * D + tid] = vq;
    // bounded hot tier: the backing arrays always receive the row (the hot copy above only if the block is resident)
    if (c.key_slots && c.keys_t2_backing)
        reinterpret_cast<T2 *>(c.keys_t2_backing)[((long)kv * c.t2_backing_rows + pos) * D + tid] = kq;
    if (c.value_slots && c.values_t2_backing)
        reinterpret_cast<T2 *>(c.values_t2_backing)[((long)kv * c.t2_backing_rows + pos) * D + tid] = vq;
    s_v[tid] = Cvt<T2>::to_f(vq);
    __syncthreads();

    // nu_b running max with the new token's value norm
    if (tid < 32) {
        const int L = tid & 15;
        float a[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) a[i] = s_v[8 * L + i];
        float vn = __fsqrt_rn(hw_sum(chain8(a, a)));
        if (tid == 0) {
            float old = pib == 0 ? 0.0f : c.values_norm_max[bidx];
            c.values_norm_max[bidx] = fmaxf(old, vn);
        }
    }
    // per-token INT4 (only when quantisation is not deferred to block completion)
    if (c.values_int4_packed && !defer_int4 && tid < 32) {
        const int g = tid & 7;
        float x[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) x[i] = s_v[g * GS + i];
        uint2 packed;
        float s, z, da, db, xa, xb;
        int4_group(x, packed, s, z, da, db);
        sumsq16(x, xa, xb);
        float ae = __fsqrt_rn(group8_sum(da, db));
        float xn = fmaxf(__fsqrt_rn(group8_sum(xa, xb)), 1e-6f);
        if (tid < 8) {
            const long row = (long)kv * c.cap_tokens + pos;
            *reinterpret_cast<uint2 *>(c.values_int4_packed + row * (D / 2) + g * 8) = packed;
            c.values_int4_scales[row * NG + g] = __half_as_ushort(__float2half_rn(s));
            c.values_int4_zeros[row * NG + g] = __half_as_ushort(__float2half_rn(z));
            if (tid == 0) {
                float err = __fdiv_rn(ae, xn);
                float osum = pib == 0 ? 0.0f : c.values_int4_error_sums[bidx];
                int ocnt = pib == 0 ? 0 : c.values_int4_error_counts[bidx];
                float oerr = pib == 0 ? 0.0f : c.values_int4_errors[bidx];
                c.values_int4_error_sums[bidx] = __fadd_rn(osum, err);
                c.values_int4_error_counts[bidx] = ocnt + 1;
                c.values_int4_errors[bidx] = fmaxf(oerr, err);
            }
        }
    }
    if (pib == BS - 1) {
        // The block just filled: quantise it from the Tier-2 rows (this CTA wrote the last one).
        __threadfence_block();
        __syncthreads();
        __threadfence();   // the rows may have gone to the backing arrays only
        const T2 *ks = t2_key_block<T2>(c, kv, blk);
        const T2 *vs = t2_value_block<T2>(c, kv, blk);
        if (ks && vs) {
            quantize_one_block<T2>(c, kv, blk, ks, vs, true,
                                   c.values_int4_packed != nullptr && defer_int4 != 0, true, false, sm);
        }
    } else if (pib == 0) {
        // New block opened: poison the not-yet-written INT8 rows.
        const long row0 = (long)kv * c.cap_tokens + pos;
        for (int t = 1; t < BS; ++t)
            if (pos + t < c.cap_tokens) c.keys_int8[(row0 + t) * D + tid] = (int8_t)-127;
    }
}

template <typename T2>
__global__ void __launch_bounds__(128) append_token_kernel(cqa_cache c, const void *k_new, const void *v_new,
                                                          int src_dtype, long pos, int defer_int4)
{
    append_token_body<T2>(c, k_new, v_new, src_dtype, pos, defer_int4);
}

// The ragged tail of a prefill: tokens [first_pos, first_pos + n_tail) of a [KV][src_rows][128] source, appended one
// after the other by the CTA of their KV head (the per-block running maxima and error sums are read-modify-write, so
// the tokens of one head stay in order; different heads share nothing).
template <typename T2>
__global__ void __launch_bounds__(128) append_tail_kernel(cqa_cache c, const void *k_src, const void *v_src, int src_dtype,
                                                         long src_rows, long first_pos, int n_tail, int defer_int4)
{
    for (int t = 0; t < n_tail; ++t) {
        append_token_body<T2>(c, k_src, v_src, src_dtype, first_pos + t, defer_int4, src_rows * D, (first_pos + t) * D);
        __syncthreads();   // the staging arrays of the body are reused by the next token
    }
}

// One token for every sequence of a batch: grid (KV, sequences).
template <typename T2>
__global__ void __launch_bounds__(128) append_token_batched_kernel(const cqa_batch_item *items, int src_dtype)
{
    const cqa_batch_item &it = *stage_batch_item(items + blockIdx.y);
    append_token_body<T2>(it.cache, it.k_new, it.v_new, src_dtype, it.pos, it.defer_int4);
}

int append_batched_launch(const cqa_batch_item *items_dev, int n_items, int kv_heads, int t2_dtype, int src_dtype, cudaStream_t st)
{
    dim3 grid((unsigned)kv_heads, (unsigned)n_items);
    switch (t2_dtype) {
    case CQA_F32: return check_cuda(launch_chained(append_token_batched_kernel<float>, grid, dim3(128), 0, st, true, items_dev, src_dtype), "append_token_batched_kernel");
    case CQA_F16: return check_cuda(launch_chained(append_token_batched_kernel<__half>, grid, dim3(128), 0, st, true, items_dev, src_dtype), "append_token_batched_kernel");
    default: return check_cuda(launch_chained(append_token_batched_kernel<__nv_bfloat16>, grid, dim3(128), 0, st, true, items_dev, src_dtype), "append_token_batched_kernel");
    }
}

// Stand-alone per-token INT4 quantiser: one 8-thread group per token.
template <typename T>
__global__ void __launch_bounds__(128) int4_quantise_kernel(const T *x, long T_rows, uint8_t *packed,
                                                           uint16_t *scales, uint16_t *zeros,
                                                           float *rel_err, float *abs_err)
{
    const long t = (long)blockIdx.x * 16 + (threadIdx.x >> 3);
    const int g = threadIdx.x & 7;
    const bool live = t < T_rows;
    float xv[16];
    if (live) {
        float a[8], b[8];
        load8<T>(x + t * D + g * GS, a);
        load8<T>(x + t * D + g * GS + 8, b);
#pragma unroll
        for (int i = 0; i < 8; ++i) { xv[i] = a[i]; xv[i + 8] = b[i]; }
    } else {
#pragma unroll
        for (int i = 0; i < 16; ++i) xv[i] = 0.0f;
    }
    uint2 pk;
    float s, z, da, db, xa, xb;
    int4_group(xv, pk, s, z, da, db);
    sumsq16(xv, xa, xb);
    float ae = __fsqrt_rn(group8_sum(da, db));
    float xn = fmaxf(__fsqrt_rn(group8_sum(xa, xb)), 1e-6f);
    if (live) {
        *reinterpret_cast<uint2 *>(packed + t * (D / 2) + g * 8) = pk;
        scales[t * NG + g] = __half_as_ushort(__float2half_rn(s));
        zeros[t * NG + g] = __half_as_ushort(__float2half_rn(z));
        if (g == 0) {
            if (rel_err) rel_err[t] = __fdiv_rn(ae, xn);
            if (abs_err) abs_err[t] = ae;
        }
    }
}

// ------------------------------------------------------------------ launchers

static int valid_cache(const cqa_cache *c)
{
    if (!c || !c->keys_int8 || !c->keys_scale || !c->keys_zero_points) {
        set_error("cqa_cache: NULL key arrays");
        return CQA_ERR_INVALID;
    }
    if (c->kv_heads <= 0 || c->cap_tokens <= 0 || c->max_blocks <= 0) {
        set_error("cqa_cache: bad sizes kv=%d cap=%ld max_blocks=%ld", c->kv_heads, (long)c->cap_tokens,
                  (long)c->max_blocks);
        return CQA_ERR_INVALID;
    }
    if (c->gqa_group != 1 && c->gqa_group != 2 && c->gqa_group != 4 && c->gqa_group != 8) {
        set_error("cqa_cache: gqa_group must be 1, 2, 4 or 8 (got %d)", c->gqa_group);
        return CQA_ERR_UNSUPPORTED;
    }
    return CQA_OK;
}

template <typename T>
static int launch_quantize(const cqa_cache *c, const void *k, const void *v, long src_rows, long first,
                           long n, cudaStream_t st)
{
    const T *ks = reinterpret_cast<const T *>(k), *vs = reinterpret_cast<const T *>(v);
    int copy = 1;
    if (!c->key_slots && !c->value_slots && k == c->keys_t2 && v == c->values_t2 && src_rows == c->keys_t2_rows &&
        first == 0)
        copy = 0;
    const long max_x = 1L << 30;
    for (long off = 0; off < n; off += max_x) {
        long cnt = n - off < max_x ? n - off : max_x;
        dim3 grid((unsigned)cnt, (unsigned)c->kv_heads);
        quantize_blocks_kernel<T><<<grid, 128, 0, st>>>(*c, ks + off * BS * D, vs + off * BS * D, src_rows,
                                                        first + off, copy); note_launch();
    }
    return check_launch("quantize_blocks_kernel");
}

}  // namespace cqa

using namespace cqa;

extern "C" int cqa_quantize_blocks(const cqa_cache *c, const void *k_src, const void *v_src, int src_dtype,
                                   int64_t src_rows, int64_t first_block, int64_t n_blocks, void *stream)
{
    int rc = valid_cache(c);
    if (rc) return rc;
    if (!k_src || !v_src) { set_error("cqa_quantize_blocks: NULL source"); return CQA_ERR_INVALID; }
    if (n_blocks == 0) return CQA_OK;
    if (n_blocks < 0 || first_block < 0 || first_block + n_blocks > c->max_blocks ||
        (first_block + n_blocks) * BS > c->cap_tokens || n_blocks * BS > src_rows) {
        set_error("cqa_quantize_blocks: block range [%ld,+%ld) out of bounds", (long)first_block,
                  (long)n_blocks);
        return CQA_ERR_INVALID;
    }
    if ((c->keys_t2 || c->values_t2) && src_dtype != c->t2_dtype) {
        set_error("cqa_quantize_blocks: source dtype %d must equal the cache's Tier-2 dtype %d", src_dtype,
                  c->t2_dtype);
        return CQA_ERR_UNSUPPORTED;
    }
    cudaStream_t st = (cudaStream_t)stream;
    switch (src_dtype) {
    case CQA_F32: return launch_quantize<float>(c, k_src, v_src, src_rows, first_block, n_blocks, st);
    case CQA_F16: return launch_quantize<__half>(c, k_src, v_src, src_rows, first_block, n_blocks, st);
    case CQA_BF16: return launch_quantize<__nv_bfloat16>(c, k_src, v_src, src_rows, first_block, n_blocks, st);
    }
    set_error("cqa_quantize_blocks: unknown dtype %d", src_dtype);
    return CQA_ERR_INVALID;
}

// Argument checks of the append (shared with the batched step).
int cqa::append_check(const cqa_cache *c, const void *k_new, const void *v_new, int src_dtype, long pos)
{
    int rc = valid_cache(c);
    if (rc) return rc;
    if (!k_new || !v_new) { set_error("cqa_append_token: NULL token"); return CQA_ERR_INVALID; }
    if (pos < 0 || pos >= c->cap_tokens || pos / BS >= c->max_blocks) {
        set_error("cqa_append_token: position %ld beyond capacity %ld", pos, (long)c->cap_tokens);
        return CQA_ERR_TOO_LARGE;
    }
    if (src_dtype < 0 || src_dtype > 2) { set_error("cqa_append_token: unknown dtype"); return CQA_ERR_INVALID; }
    if (c->t2_dtype < 0 || c->t2_dtype > 2) { set_error("cqa_append_token: unknown Tier-2 dtype %d", c->t2_dtype); return CQA_ERR_INVALID; }
    return CQA_OK;
}

extern "C" int cqa_append_token(const cqa_cache *c, const void *k_new, const void *v_new, int src_dtype,
                                int64_t pos, int defer_int4, void *stream)
{
    int rc = append_check(c, k_new, v_new, src_dtype, pos);
    if (rc) return rc;
    cudaStream_t st = (cudaStream_t)stream;
    switch (c->t2_dtype) {
    case CQA_F32: rc = check_cuda(launch_chained(append_token_kernel<float>, dim3(c->kv_heads), dim3(128), 0, st, true, *c, k_new, v_new, src_dtype, pos, defer_int4), "append_token_kernel"); break;
    case CQA_F16: rc = check_cuda(launch_chained(append_token_kernel<__half>, dim3(c->kv_heads), dim3(128), 0, st, true, *c, k_new, v_new, src_dtype, pos, defer_int4), "append_token_kernel"); break;
    case CQA_BF16: rc = check_cuda(launch_chained(append_token_kernel<__nv_bfloat16>, dim3(c->kv_heads), dim3(128), 0, st, true, *c, k_new, v_new, src_dtype, pos, defer_int4), "append_token_kernel"); break;
    default: set_error("cqa_append_token: unknown Tier-2 dtype %d", c->t2_dtype); return CQA_ERR_INVALID;
    }
    return rc;
}

extern "C" int cqa_prefill_encode(const cqa_prefill_item *items, int n_items, int src_dtype, void *stream)
{
    if (!items || n_items <= 0) { set_error("cqa_prefill_encode: no items"); return CQA_ERR_INVALID; }
    if (src_dtype < 0 || src_dtype > 2) { set_error("cqa_prefill_encode: unknown dtype %d", src_dtype); return CQA_ERR_INVALID; }
    // every check before the first launch
    for (int i = 0; i < n_items; ++i) {
        const cqa_prefill_item &it = items[i];
        int rc = valid_cache(&it.cache);
        if (rc) return rc;
        if (!it.k_src || !it.v_src || it.n_tokens < 0 || it.src_rows < it.n_tokens) {
            set_error("cqa_prefill_encode: item %d: bad source (%ld tokens in %ld rows)", i, (long)it.n_tokens, (long)it.src_rows);
            return CQA_ERR_INVALID;
        }
        const long nblk = (it.n_tokens + BS - 1) / BS;
        if (it.n_tokens > it.cache.cap_tokens || nblk > it.cache.max_blocks) {
            set_error("cqa_prefill_encode: item %d: %ld tokens exceed the cache capacity %ld", i, (long)it.n_tokens,
                      (long)it.cache.cap_tokens);
            return CQA_ERR_TOO_LARGE;
        }
        if ((it.cache.keys_t2 || it.cache.values_t2) && src_dtype != it.cache.t2_dtype) {
            set_error("cqa_prefill_encode: item %d: source dtype %d must equal the cache's Tier-2 dtype %d", i, src_dtype,
                      it.cache.t2_dtype);
            return CQA_ERR_UNSUPPORTED;
        }
    }
    cudaStream_t st = (cudaStream_t)stream;
    for (int i = 0; i < n_items; ++i) {
        const cqa_prefill_item &it = items[i];
        const long full = it.n_tokens / BS;
        const int tail = (int)(it.n_tokens - full * BS);
        if (full > 0) {
            int rc = cqa_quantize_blocks(&it.cache, it.k_src, it.v_src, src_dtype, it.src_rows, 0, full, stream);
            if (rc) return rc;
        }
        if (tail > 0) {
            const cqa_cache *c = &it.cache;
            int rc;
            switch (c->t2_dtype) {
            case CQA_F32: rc = check_cuda(launch_chained(append_tail_kernel<float>, dim3(c->kv_heads), dim3(128), 0, st, false, *c, it.k_src, it.v_src, src_dtype, (long)it.src_rows, full * BS, tail, (int)it.defer_int4), "append_tail_kernel"); break;
            case CQA_F16: rc = check_cuda(launch_chained(append_tail_kernel<__half>, dim3(c->kv_heads), dim3(128), 0, st, false, *c, it.k_src, it.v_src, src_dtype, (long)it.src_rows, full * BS, tail, (int)it.defer_int4), "append_tail_kernel"); break;
            default: rc = check_cuda(launch_chained(append_tail_kernel<__nv_bfloat16>, dim3(c->kv_heads), dim3(128), 0, st, false, *c, it.k_src, it.v_src, src_dtype, (long)it.src_rows, full * BS, tail, (int)it.defer_int4), "append_tail_kernel"); break;
            }
            if (rc) return rc;
        }
    }
    return CQA_OK;
}

extern "C" int cqa_int4_quantise(const void *x, int src_dtype, int64_t T, uint8_t *packed, uint16_t *scales,
                                 uint16_t *zeros, float *rel_err, float *abs_err, void *stream)
{
    if (!x || !packed || !scales || !zeros) { set_error("cqa_int4_quantise: NULL pointer"); return CQA_ERR_INVALID; }
    if (T == 0) return CQA_OK;
    if (T < 0) { set_error("cqa_int4_quantise: negative row count"); return CQA_ERR_INVALID; }
    cudaStream_t st = (cudaStream_t)stream;
    unsigned grid = (unsigned)((T + 15) / 16);
    switch (src_dtype) {
    case CQA_F32: int4_quantise_kernel<float><<<grid, 128, 0, st>>>((const float *)x, T, packed, scales, zeros, rel_err, abs_err); note_launch(); break;
    case CQA_F16: int4_quantise_kernel<__half><<<grid, 128, 0, st>>>((const __half *)x, T, packed, scales, zeros, rel_err, abs_err); note_launch(); break;
    case CQA_BF16: int4_quantise_kernel<__nv_bfloat16><<<grid, 128, 0, st>>>((const __nv_bfloat16 *)x, T, packed, scales, zeros, rel_err, abs_err); note_launch(); break;
    default: set_error("cqa_int4_quantise: unknown dtype %d", src_dtype); return CQA_ERR_INVALID;
    }
    return check_launch("int4_quantise_kernel");
}
