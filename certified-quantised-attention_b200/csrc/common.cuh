// Shared device helpers: canonical binary32 arithmetic, loads, error plumbing.
//
// "Canonical" functions fix the exact sequence of IEEE-754 binary32 operations
// (round to nearest even, explicit fused multiply-adds, no contraction, no
// approximate intrinsics) for every value that can change a block selection or
// a certificate flag.  The CPU checker used by the tests follows the same
// sequence, so those values are reproducible bit for bit.
#pragma once

#include <cuda_runtime.h>
#include <cuda_fp16.h>
#include <cuda_bf16.h>
#include <stdint.h>

#include "../../include/cqa_b200.h"

namespace cqa {

constexpr int D = 128;   // head_dim == d_v
constexpr int BS = 16;   // tokens per block
constexpr int GS = 16;   // INT4 group size
constexpr int NG = 8;    // groups per token
constexpr unsigned FULL = 0xffffffffu;

// ---------------------------------------------------------------- exp / log

// exp(x): Cody-Waite reduction, degree-5 polynomial (Cephes coefficients),
// exact power-of-two scaling.  x <= -104 (or NaN) gives 0.
__device__ __forceinline__ float cexp(float x)
{
    if (!(x > -104.0f)) return 0.0f;
    if (x > 88.0f) x = 88.0f;
    float t = __fmul_rn(x, 1.44269504088896341f);
    float n = rintf(t);
    float r = __fmaf_rn(n, -0.693145751953125f, x);
    r = __fmaf_rn(n, -1.42860682030941723212e-6f, r);
    float p = 1.9875691500e-4f;
    p = __fmaf_rn(p, r, 1.3981999507e-3f);
    p = __fmaf_rn(p, r, 8.3334519073e-3f);
    p = __fmaf_rn(p, r, 4.1665795894e-2f);
    p = __fmaf_rn(p, r, 1.6666665459e-1f);
    p = __fmaf_rn(p, r, 5.0000001201e-1f);
    float r2 = __fmul_rn(r, r);
    p = __fmaf_rn(p, r2, r);
    p = __fadd_rn(p, 1.0f);
    int ni = (int)n;
    if (ni < -126) {
        p = __fmul_rn(p, __int_as_float((ni + 64 + 127) << 23));
        return __fmul_rn(p, 5.42101086242752217e-20f);  // 2^-64
    }
    return __fmul_rn(p, __int_as_float((ni + 127) << 23));
}

// log(x) for positive normal x (Cephes logf layout).
__device__ __forceinline__ float clog(float x)
{
    unsigned ix = __float_as_uint(x);
    int e = (int)(ix >> 23) - 126;
    float m = __uint_as_float((ix & 0x007FFFFFu) | 0x3F000000u);
    if (m < 0.707106781186547524f) {
        e -= 1;
        m = __fadd_rn(__fadd_rn(m, m), -1.0f);
    } else {
        m = __fadd_rn(m, -1.0f);
    }
    float z = __fmul_rn(m, m);
    float y = 7.0376836292e-2f;
    y = __fmaf_rn(y, m, -1.1514610310e-1f);
    y = __fmaf_rn(y, m, 1.1676998740e-1f);
    y = __fmaf_rn(y, m, -1.2420140846e-1f);
    y = __fmaf_rn(y, m, 1.4249322787e-1f);
    y = __fmaf_rn(y, m, -1.6668057665e-1f);
    y = __fmaf_rn(y, m, 2.0000714765e-1f);
    y = __fmaf_rn(y, m, -2.4999993993e-1f);
    y = __fmaf_rn(y, m, 3.3333331174e-1f);
    y = __fmul_rn(y, m);
    y = __fmul_rn(y, z);
    float fe = (float)e;
    y = __fmaf_rn(fe, -2.12194440e-4f, y);
    y = __fmaf_rn(z, -0.5f, y);
    float r = __fadd_rn(m, y);
    r = __fmaf_rn(fe, 0.693359375f, r);
    return r;
}

// ------------------------------------------------------------ canonical sums

// Partial of a 128-wide dot product for the 8 channels a lane owns: two fused
// chains (even / odd channels) added at the end.
__device__ __forceinline__ float chain8(const float (&a)[8], const float (&b)[8])
{
    float e = __fmaf_rn(a[0], b[0], 0.0f);
    float o = __fmaf_rn(a[1], b[1], 0.0f);
    e = __fmaf_rn(a[2], b[2], e);
    o = __fmaf_rn(a[3], b[3], o);
    e = __fmaf_rn(a[4], b[4], e);
    o = __fmaf_rn(a[5], b[5], o);
    e = __fmaf_rn(a[6], b[6], e);
    o = __fmaf_rn(a[7], b[7], o);
    return __fadd_rn(e, o);
}

// Butterfly all-reduce over the 16 lanes of a half warp (strides 8,4,2,1).
__device__ __forceinline__ float hw_sum(float p)
{
    p = __fadd_rn(p, __shfl_xor_sync(FULL, p, 8));
    p = __fadd_rn(p, __shfl_xor_sync(FULL, p, 4));
    p = __fadd_rn(p, __shfl_xor_sync(FULL, p, 2));
    p = __fadd_rn(p, __shfl_xor_sync(FULL, p, 1));
    return p;
}
__device__ __forceinline__ float hw_max(float p)
{
    p = fmaxf(p, __shfl_xor_sync(FULL, p, 8));
    p = fmaxf(p, __shfl_xor_sync(FULL, p, 4));
    p = fmaxf(p, __shfl_xor_sync(FULL, p, 2));
    p = fmaxf(p, __shfl_xor_sync(FULL, p, 1));
    return p;
}
// Butterfly all-reduce over a full warp (strides 16,8,4,2,1).
__device__ __forceinline__ float warp_sum(float p)
{
    p = __fadd_rn(p, __shfl_xor_sync(FULL, p, 16));
    return hw_sum(p);
}
__device__ __forceinline__ float warp_max(float p)
{
    p = fmaxf(p, __shfl_xor_sync(FULL, p, 16));
    return hw_max(p);
}

// ------------------------------------------------------------------- loads

template <typename T> struct Cvt;
template <> struct Cvt<float> {
    static __device__ __forceinline__ float to_f(float v) { return v; }
    static __device__ __forceinline__ float from_f(float v) { return v; }
};
template <> struct Cvt<__half> {
    static __device__ __forceinline__ float to_f(__half v) { return __half2float(v); }
    static __device__ __forceinline__ __half from_f(float v) { return __float2half_rn(v); }
};
template <> struct Cvt<__nv_bfloat16> {
    static __device__ __forceinline__ float to_f(__nv_bfloat16 v) { return __bfloat162float(v); }
    static __device__ __forceinline__ __nv_bfloat16 from_f(float v) { return __float2bfloat16_rn(v); }
};

// 8 consecutive elements of type T -> float[8] (16-byte or 32-byte vector loads).
template <typename T>
__device__ __forceinline__ void load8(const T *p, float (&out)[8]);
template <>
__device__ __forceinline__ void load8<float>(const float *p, float (&out)[8])
{
    float4 a = *reinterpret_cast<const float4 *>(p);
    float4 b = *reinterpret_cast<const float4 *>(p + 4);
    out[0] = a.x; out[1] = a.y; out[2] = a.z; out[3] = a.w;
    out[4] = b.x; out[5] = b.y; out[6] = b.z; out[7] = b.w;
}
template <>
__device__ __forceinline__ void load8<__half>(const __half *p, float (&out)[8])
{
    uint4 u = *reinterpret_cast<const uint4 *>(p);
    const __half2 *h = reinterpret_cast<const __half2 *>(&u);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        float2 f = __half22float2(h[i]);
        out[2 * i] = f.x;
        out[2 * i + 1] = f.y;
    }
}
template <>
__device__ __forceinline__ void load8<__nv_bfloat16>(const __nv_bfloat16 *p, float (&out)[8])
{
    uint4 u = *reinterpret_cast<const uint4 *>(p);
    const unsigned *w = reinterpret_cast<const unsigned *>(&u);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        out[2 * i] = __uint_as_float(w[i] << 16);
        out[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
    }
}


// Raw (unconverted) 8-element loads, so many rows can be in flight in few registers.
template <typename T> struct Raw8 { uint4 v; };
template <> struct Raw8<float> { float4 a, b; };
template <typename T>
__device__ __forceinline__ Raw8<T> raw_load8(const T *p)
{
    Raw8<T> r;
    r.v = *reinterpret_cast<const uint4 *>(p);
    return r;
}
template <>
__device__ __forceinline__ Raw8<float> raw_load8<float>(const float *p)
{
    Raw8<float> r;
    r.a = *reinterpret_cast<const float4 *>(p);
    r.b = *reinterpret_cast<const float4 *>(p + 4);
    return r;
}
template <typename T>
__device__ __forceinline__ Raw8<T> raw_zero8()
{
    Raw8<T> r;
    r.v = make_uint4(0u, 0u, 0u, 0u);
    return r;
}
template <>
__device__ __forceinline__ Raw8<float> raw_zero8<float>()
{
    Raw8<float> r;
    r.a = make_float4(0.f, 0.f, 0.f, 0.f);
    r.b = r.a;
    return r;
}
__device__ __forceinline__ void raw_to_f(const Raw8<float> &r, float (&out)[8])
{
    out[0] = r.a.x; out[1] = r.a.y; out[2] = r.a.z; out[3] = r.a.w;
    out[4] = r.b.x; out[5] = r.b.y; out[6] = r.b.z; out[7] = r.b.w;
}
__device__ __forceinline__ void raw_to_f(const Raw8<__half> &r, float (&out)[8])
{
    const __half2 *h = reinterpret_cast<const __half2 *>(&r.v);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        float2 f = __half22float2(h[i]);
        out[2 * i] = f.x;
        out[2 * i + 1] = f.y;
    }
}
__device__ __forceinline__ void raw_to_f(const Raw8<__nv_bfloat16> &r, float (&out)[8])
{
    const unsigned *w = reinterpret_cast<const unsigned *>(&r.v);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        out[2 * i] = __uint_as_float(w[i] << 16);
        out[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
    }
}

// Scalar read of q in its runtime dtype.
__device__ __forceinline__ float load_q(const void *q, int dtype, long idx)
{
    if (dtype == CQA_F32) return reinterpret_cast<const float *>(q)[idx];
    if (dtype == CQA_F16) return __half2float(reinterpret_cast<const __half *>(q)[idx]);
    return __bfloat162float(reinterpret_cast<const __nv_bfloat16 *>(q)[idx]);
}
__device__ __forceinline__ void load_q8(const void *q, int dtype, long idx, float (&out)[8])
{
#pragma unroll
    for (int i = 0; i < 8; ++i) out[i] = load_q(q, dtype, idx + i);
}

// 8 signed bytes -> float[8]
__device__ __forceinline__ void i8x8_to_f(uint2 w, float (&out)[8])
{
    const int8_t *b = reinterpret_cast<const int8_t *>(&w);
#pragma unroll
    for (int i = 0; i < 8; ++i) out[i] = (float)b[i];
}

// ------------------------------------------------------------- Tier-2 block rows

// First row (token 0) of block `b` of KV head `kv` in Tier 2: the hot slot when the block is resident (or when there
// is no slot table: identity), else the backing array; nullptr when neither holds it.
template <typename T2>
__device__ __forceinline__ const T2 *t2_block(const void *hot, long hot_rows, const int32_t *slots, const void *backing,
                                              long backing_rows, int kv, long b)
{
    if (slots == nullptr)
        return hot ? reinterpret_cast<const T2 *>(hot) + ((long)kv * hot_rows + b * BS) * D : nullptr;
    const int s = slots[b];
    if (s >= 0) return reinterpret_cast<const T2 *>(hot) + ((long)kv * hot_rows + (long)s * BS) * D;
    return backing ? reinterpret_cast<const T2 *>(backing) + ((long)kv * backing_rows + b * BS) * D : nullptr;
}
template <typename T2>
__device__ __forceinline__ const T2 *t2_key_block(const cqa_cache &c, int kv, long b)
{
    return t2_block<T2>(c.keys_t2, c.keys_t2_rows, c.key_slots, c.keys_t2_backing, c.t2_backing_rows, kv, b);
}
template <typename T2>
__device__ __forceinline__ const T2 *t2_value_block(const cqa_cache &c, int kv, long b)
{
    return t2_block<T2>(c.values_t2, c.values_t2_rows, c.value_slots, c.values_t2_backing, c.t2_backing_rows, kv, b);
}

// ------------------------------------------------- programmatic dependent launch

// Kernels of the fused decode chain are launched with programmatic stream serialisation: the next kernel's CTAs
// may be scheduled while the previous kernel drains, and wait here until that kernel has completed and its writes
// are visible.  Without the launch attribute the wait returns at once.
__device__ __forceinline__ void grid_dependency_wait()
{
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}

// Every kernel launch of the library is counted (cqa_launch_count), so a caller can check that its calls ran on the
// GPU and how many kernels a step takes.
void note_launch(int n = 1);

// Opt a kernel in to `bytes` of dynamic shared memory on the current device.  The attribute belongs to the
// (function, device) pair, so the largest size already granted is remembered per device ordinal; `granted` is one
// array per kernel instantiation (a function-local static of the caller).
#ifndef CQA_ATT_MIN_CTAS
#define CQA_ATT_MIN_CTAS 2   // resident Phase-2 CTAs per SM that the kernel is built for and the split heuristic assumes
#endif
constexpr int SMEM_ATTR_DEVICES = 64;
template <typename K>
static inline cudaError_t ensure_dynamic_smem(K kernel, size_t bytes, size_t (&granted)[SMEM_ATTR_DEVICES])
{
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    const bool tracked = dev >= 0 && dev < SMEM_ATTR_DEVICES;
    if (tracked && bytes <= granted[dev]) return cudaSuccess;
    e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
    if (e == cudaSuccess && tracked) granted[dev] = bytes;
    return e;
}

// Launch with (or without) the programmatic-serialisation attribute.
template <typename... KArgs, typename... Args>
static inline cudaError_t launch_chained(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st,
                                         bool chained, Args... args)
{
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = chained ? 1 : 0;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    note_launch();
    return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

// ----------------------------------------------------------------- bulk asynchronous copies (TMA) + mbarrier
//
// Page tiles are staged in shared memory by the bulk-copy engine: one lane issues `cp.async.bulk` for each
// contiguous piece of a block (the pieces land without touching a register or the load/store units of the other
// lanes) and the copies report their bytes to an mbarrier that the consuming lanes wait on.  Plain single-CTA
// copies from this GPU's own memory only.  Source and destination must be 16-byte aligned and sizes multiples of
// 16 bytes.  Every wait is bounded: after BULK_WAIT_POLLS unsuccessful polls the waiter records the event in a
// device-global counter (cqa_wait_timeouts) and carries on, so a lost copy can never hang the GPU.

__device__ __forceinline__ unsigned smem_u32(const void *p) { return (unsigned)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t *bar, int count)
{
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
// Makes freshly initialised barriers visible to the copy engine; call once after mbar_init, before the CTA barrier.
__device__ __forceinline__ void mbar_init_fence()
{
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
// One arrival that also announces `bytes` of copies to come.
// The issuing side works on 32-bit shared-memory addresses (smem_u32 of the stage and of its barrier, computed
// once), so a copy costs the instruction itself and an add for each address.
__device__ __forceinline__ void mbar_arrive_expect_tx(unsigned bar_addr, unsigned bytes)
{
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar_addr), "r"(bytes) : "memory");
}
__device__ __forceinline__ void bulk_copy_g2s(unsigned dst_addr, const void *src_gmem, unsigned bytes, unsigned bar_addr)
{
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(dst_addr), "l"(src_gmem), "r"(bytes), "r"(bar_addr)
                 : "memory");
}
// One poll of the barrier's phase.  The hardware may park the thread for up to `suspend_ns` before it answers, so a
// waiting warp issues almost no instructions while its tile is in flight.
__device__ __forceinline__ bool mbar_try_wait(unsigned bar_addr, unsigned parity, unsigned suspend_ns = 20000u)
{
    unsigned ok;
    asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                 : "=r"(ok)
                 : "r"(bar_addr), "r"(parity), "r"(suspend_ns)
                 : "memory");
    return ok != 0;
}
// One counter per translation unit (the library is built without relocatable device code); cqa_wait_timeouts adds
// them up through the accessors that the units using staged copies export.
static __device__ int g_wait_timeouts = 0;
constexpr int BULK_WAIT_POLLS = 50000;
// Wait (bounded) until the phase with this parity of `bar` has completed.  A copy normally lands within a few
// polls.  Once any wait of this unit has run out, later waits give up after a handful of polls, so that a broken
// run ends quickly instead of paying the full limit at every stage.
__device__ __forceinline__ void mbar_wait(unsigned bar_addr, unsigned parity)
{
    if (mbar_try_wait(bar_addr, parity)) return;
    const int limit = *reinterpret_cast<volatile int *>(&g_wait_timeouts) != 0 ? 64 : BULK_WAIT_POLLS;
    for (int polls = 0; polls < limit; ++polls)
        if (mbar_try_wait(bar_addr, parity)) return;
    atomicAdd(&g_wait_timeouts, 1);
}

// Host side: read (and optionally clear) this translation unit's timeout counter on the current device.
static inline int wait_timeouts_of_this_unit(int *count, int reset)
{
    cudaError_t e = cudaMemcpyFromSymbol(count, g_wait_timeouts, sizeof(int));
    if (e == cudaSuccess && reset) {
        const int zero = 0;
        e = cudaMemcpyToSymbol(g_wait_timeouts, &zero, sizeof(int));
    }
    return e == cudaSuccess ? 0 : -1;
}

// ----------------------------------------------------------------- peer exchange flags

__device__ __forceinline__ int ld_acquire_sys(const int32_t *p)
{
    int v;
    asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_release_sys(int32_t *p, int v)
{
    asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

// Exchange A from inside the score kernel: every (head, block) result is also stored into the other ranks' buffers,
// and the last CTA to finish releases the flags.  world == 0: off.
struct ScorePush {
    float *mb[8];        // each rank's rows for this rank's m_b (same leading dimension as the local rows)
    float *sb[8];
    int32_t *flag[8];    // flag word to release on each rank
    int32_t *ticket;     // local counter
    int world, rank, step;
};

// Called by every thread of a CTA before it reads exchanged data: thread 0 waits until flags[i * stride] >= value
// for every i < n except `skip`, then the CTA synchronises.  Every wait is bounded: after `spins` polls (0 = the
// default, about half a second) of one flag the thread records 100 + i in *status and moves on, so the kernel
// always returns and the context stays usable; the step's result is then invalid and the host reads the status.
constexpr int PEER_WAIT_SPINS = 2000000;
__device__ __forceinline__ void peer_wait(const int32_t *flags, int n, int skip, int value, int32_t *status,
                                          long stride = 1, int spins_limit = 0)
{
    if (flags != nullptr && threadIdx.x == 0) {
        const int limit = spins_limit > 0 ? spins_limit : PEER_WAIT_SPINS;
        for (int i = 0; i < n; ++i) {
            if (i == skip) continue;
            int spins = 0;
            while (ld_acquire_sys(flags + i * stride) < value) {
                if (++spins > limit) {
                    if (status) atomicExch(status, 100 + i);
                    break;
                }
                __nanosleep(200);
            }
        }
    }
    __syncthreads();
}

// ----------------------------------------------------------------- batches

// A batched kernel's CTA copies the record of its sequence from global to shared memory once and works from that
// copy (the one-sequence kernels get the same structs as kernel parameters).  Ends with a CTA barrier.
__device__ __forceinline__ const cqa_batch_item *stage_batch_item(const cqa_batch_item *src)
{
    __shared__ __align__(16) cqa_batch_item s_item;
    static_assert(sizeof(cqa_batch_item) % 4 == 0, "record is copied in 32-bit words");
    const int *from = reinterpret_cast<const int *>(src);
    int *to = reinterpret_cast<int *>(&s_item);
    for (int i = threadIdx.x; i < (int)(sizeof(cqa_batch_item) / 4); i += blockDim.x) to[i] = from[i];
    __syncthreads();
    return &s_item;
}

// ----------------------------------------------------------------- errors

void set_error(const char *fmt, ...);
int check_cuda(cudaError_t e, const char *what);
int check_launch(const char *what);

// Argument checks of the three kernels of a layer step, callable on their own so that a fused entry point can
// validate the whole chain before its first launch.
int check_score_args(const cqa_cache *c, int q_dtype, long nq, long ld, const char *who);
int selcert_check(const cqa_cache *c, const cqa_knobs *kn, const cqa_workspace *ws, const void *q, long nq, int phases);
int attend_check(const cqa_cache *c, const cqa_workspace *ws, long nq, long nact, int last_valid);
int append_check(const cqa_cache *c, const void *k_new, const void *v_new, int src_dtype, long pos);
int score_wait_timeouts(int *count, int reset);
int selcert_wait_timeouts(int *count, int reset);

}  // namespace cqa
