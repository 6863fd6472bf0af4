/*
 * CPU oracle for certified quantised decode attention.  TEST INFRASTRUCTURE
 * ONLY: nothing under the product package may link, import or execute this
 * file; it exists to check the CUDA path and to time a CPU baseline.
 *
 * It restates the arithmetic of the reference project
 * (DeanoC/certified-quantised-attention) for one layer's decode step:
 *   - INT8 per-channel-per-block key quantisation
 *       dotcache/kernels/tiered_kv_cache.py:160-192, 480-543
 *   - INT4 per-token-per-group value quantisation and its error annotation
 *       dotcache/kernels/int4_group_quantise.py:42-88, 123-151
 *   - Phase-1 block scores m_b, S_b
 *       dotcache/kernels/fused_score_certify.py:258-292
 *   - FP16 block re-score          dotcache/kernels/fp16_block_scores_triton.py:28-70
 *   - block mass fractions         dotcache/kernels/certified_attention.py:345-350
 *   - Delta bound                  dotcache/kernels/certified_attention.py:912-945
 *   - Phase-2 mixed attend         dotcache/kernels/selective_attend_triton.py:1310-1445, 1245-1272
 *   - dense FP16 recompute         dotcache/kernels/certified_attention.py:789-879
 *
 * Floating-point results that feed a selection or a certificate flag are
 * computed in a CANONICAL ORDER of IEEE-754 binary32 operations (fused
 * multiply-add where written, round-to-nearest-even everywhere, own exp/log
 * built from those operations) so that a GPU kernel that follows the same
 * order reproduces them bit for bit.  The reference itself fixes no order
 * (its Triton, CUDA and CPU back ends associate sums differently), so this
 * canonical order is pinned against the reference by golden vectors with a
 * small tolerance on floats and exact equality on bytes, masks and flags.
 *
 * Attention outputs (Phase 2, dense recompute) are accumulated in double
 * precision here: they are the ground truth the GPU result is compared with
 * under a tolerance.
 *
 * Build: gcc -O2 -shared -fPIC -ffp-contract=off -fno-fast-math -march=x86-64-v3 -fopenmp
 */
#include <math.h>
#include <stdint.h>
#include <string.h>
#include <stdlib.h>

#define D 128          /* head_dim == d_v */
#define BS 16          /* tokens per block */
#define GS 16          /* INT4 group size */
#define NG (D / GS)    /* groups per token */

/* ---------------------------------------------------------------- exp / log */

static inline float f_from_bits(uint32_t u) { float f; memcpy(&f, &u, 4); return f; }
static inline uint32_t f_bits(float f) { uint32_t u; memcpy(&u, &f, 4); return u; }

/* exp(x): Cody-Waite reduction by ln2 (two constants), degree-5 polynomial for
 * exp(r)-1-r over r^2 (Cephes coefficients), scaling by 2^n through the
 * exponent field.  Inputs below -104 give 0. */
#ifdef _OPENMP
#include <omp.h>
#endif
/* Number of OpenMP threads the parallel loops below use (a launcher may have exported OMP_NUM_THREADS=1). */
void cqa_o_set_threads(int n)
{
#ifdef _OPENMP
    if (n > 0) omp_set_num_threads(n);
#else
    (void)n;
#endif
}

int cqa_o_max_threads(void)
{
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

float cqa_o_exp(float x)
{
    if (!(x > -104.0f)) return 0.0f;
    if (x > 88.0f) x = 88.0f;
    float t = x * 1.44269504088896341f;
    float n = rintf(t);
    float r = fmaf(n, -0.693145751953125f, x);
    r = fmaf(n, -1.42860682030941723212e-6f, r);
    float p = 1.9875691500e-4f;
    p = fmaf(p, r, 1.3981999507e-3f);
    p = fmaf(p, r, 8.3334519073e-3f);
    p = fmaf(p, r, 4.1665795894e-2f);
    p = fmaf(p, r, 1.6666665459e-1f);
    p = fmaf(p, r, 5.0000001201e-1f);
    float r2 = r * r;
    p = fmaf(p, r2, r);
    p = p + 1.0f;
    int ni = (int)n;
    if (ni < -126) {
        float s1 = f_from_bits((uint32_t)(ni + 64 + 127) << 23);
        p = p * s1;
        p = p * 5.42101086242752217e-20f; /* 2^-64 */
        return p;
    }
    return p * f_from_bits((uint32_t)(ni + 127) << 23);
}

/* log(x) for positive normal x (Cephes logf layout). */
float cqa_o_log(float x)
{
    uint32_t ix = f_bits(x);
    int e = (int)(ix >> 23) - 126;
    float m = f_from_bits((ix & 0x007FFFFFu) | 0x3F000000u); /* [0.5, 1) */
    if (m < 0.707106781186547524f) {
        e -= 1;
        m = (m + m) - 1.0f;
    } else {
        m = m - 1.0f;
    }
    float z = m * m;
    float y = 7.0376836292e-2f;
    y = fmaf(y, m, -1.1514610310e-1f);
    y = fmaf(y, m, 1.1676998740e-1f);
    y = fmaf(y, m, -1.2420140846e-1f);
    y = fmaf(y, m, 1.4249322787e-1f);
    y = fmaf(y, m, -1.6668057665e-1f);
    y = fmaf(y, m, 2.0000714765e-1f);
    y = fmaf(y, m, -2.4999993993e-1f);
    y = fmaf(y, m, 3.3333331174e-1f);
    y = y * m;
    y = y * z;
    float fe = (float)e;
    y = fmaf(fe, -2.12194440e-4f, y);
    y = fmaf(z, -0.5f, y);
    float r = m + y;
    r = fmaf(fe, 0.693359375f, r);
    return r;
}

/* ------------------------------------------------------------ canonical sums */

/* dot of two 128-vectors.  "Lane" L (0..15) owns channels 8L..8L+7 and runs
 * two fused chains (even and odd channels); the 16 lane partials are then
 * combined by a butterfly with strides 8,4,2,1. */
static inline float dot128(const float *a, const float *b)
{
    float p[16];
    for (int L = 0; L < 16; ++L) {
        const float *x = a + 8 * L, *y = b + 8 * L;
        float e = fmaf(x[0], y[0], 0.0f);
        float o = fmaf(x[1], y[1], 0.0f);
        e = fmaf(x[2], y[2], e); o = fmaf(x[3], y[3], o);
        e = fmaf(x[4], y[4], e); o = fmaf(x[5], y[5], o);
        e = fmaf(x[6], y[6], e); o = fmaf(x[7], y[7], o);
        p[L] = e + o;
    }
    for (int s = 8; s >= 1; s >>= 1)
        for (int i = 0; i < s; ++i) p[i] = p[i] + p[i + s];
    return p[0];
}

/* dot of int8 row with float vector (int8 widened exactly). */
static inline float dot128_i8(const int8_t *k, const float *b)
{
    float a[D];
    for (int c = 0; c < D; ++c) a[c] = (float)k[c];
    return dot128(a, b);
}

static inline float butterfly16(float *p)
{
    for (int s = 8; s >= 1; s >>= 1)
        for (int i = 0; i < s; ++i) p[i] = p[i] + p[i + s];
    return p[0];
}

/* Sum over n values: groups of 32 consecutive values by a butterfly
 * (strides 16..1, missing values are +0), groups of 8 such sums by a
 * butterfly (strides 4,2,1) -> one "leaf" per 256 values; leaves are then
 * added left to right. */
float cqa_o_canonical_sum(const float *x, long n)
{
    float total = 0.0f;
    for (long leaf = 0; leaf * 256 < n; ++leaf) {
        float g[8];
        for (int w = 0; w < 8; ++w) {
            float p[32];
            for (int i = 0; i < 32; ++i) {
                long idx = leaf * 256 + w * 32 + i;
                p[i] = idx < n ? x[idx] : 0.0f;
            }
            for (int s = 16; s >= 1; s >>= 1)
                for (int i = 0; i < s; ++i) p[i] = p[i] + p[i + s];
            g[w] = p[0];
        }
        for (int s = 4; s >= 1; s >>= 1)
            for (int i = 0; i < s; ++i) g[i] = g[i] + g[i + s];
        total = leaf == 0 ? g[0] : total + g[0];
    }
    return total;
}

/* "Column sum" used by the Rung-2 value check: of the values x[i] with include[i] != 0 (all when include is
 * NULL), column t (0..1023) adds its members i = t, t+1024, ... in ascending order; the 32 columns of each group
 * of 32 are combined by a butterfly (strides 16..1), and the 32 group sums by the same butterfly.  Adding a
 * non-negative member never lowers the result. */
float cqa_o_column_sum(const float *x, const unsigned char *include, long n)
{
    float col[1024];
    for (int t = 0; t < 1024; ++t) {
        float s = 0.0f;
        for (long i = t; i < n; i += 1024)
            if (!include || include[i]) s = s + x[i];
        col[t] = s;
    }
    float g[32];
    for (int w = 0; w < 32; ++w) {
        float *p = col + w * 32;
        for (int s = 16; s >= 1; s >>= 1)
            for (int i = 0; i < s; ++i) p[i] = p[i] + p[i + s];
        g[w] = p[0];
    }
    for (int s = 16; s >= 1; s >>= 1)
        for (int i = 0; i < s; ++i) g[i] = g[i] + g[i + s];
    return g[0];
}

/* Leaf sums only (256 values per leaf); used by the sharded merge. */
void cqa_o_leaf_sums(const float *x, long n, float *leaves)
{
    for (long leaf = 0; leaf * 256 < n; ++leaf) {
        long lo = leaf * 256;
        long cnt = n - lo < 256 ? n - lo : 256;
        leaves[leaf] = cqa_o_canonical_sum(x + lo, cnt);
    }
}

/* Sequential (left to right) inclusive prefix sum. */
void cqa_o_seq_cumsum(const float *x, long n, float *out)
{
    float c = 0.0f;
    for (long i = 0; i < n; ++i) {
        c = i == 0 ? x[0] : c + x[i];
        out[i] = c;
    }
}

/* ------------------------------------------------------------- quantisation */

/* INT8 per-channel asymmetric key quantisation of complete blocks.
 * k: [nblk][16][128] float32 (model-dtype values widened exactly).
 * tiered_kv_cache.py:169-192 */
void cqa_o_quant_keys(const float *k, long nblk, int8_t *q, float *scale, float *zp, float *corr)
{
#pragma omp parallel for schedule(static)
    for (long b = 0; b < nblk; ++b) {
        const float *kb = k + b * BS * D;
        float *s = scale + b * D, *z = zp + b * D;
        for (int c = 0; c < D; ++c) {
            float lo = kb[c], hi = kb[c];
            for (int t = 1; t < BS; ++t) {
                float v = kb[t * D + c];
                lo = v < lo ? v : lo;
                hi = v > hi ? v : hi;
            }
            float range = hi - lo;
            if (range < 1e-8f) range = 1e-8f;
            s[c] = range / 255.0f;
            z[c] = (lo + hi) / 2.0f;
        }
        for (int t = 0; t < BS; ++t)
            for (int c = 0; c < D; ++c) {
                float r = rintf((kb[t * D + c] - z[c]) / s[c]);
                if (r < -128.0f) r = -128.0f;
                if (r > 127.0f) r = 127.0f;
                q[(b * BS + t) * D + c] = (int8_t)r;
            }
        float n2 = dot128(s, s);
        float delta = sqrtf(n2) / 127.0f;
        corr[b] = cqa_o_exp(2.0f * delta);
    }
}

/* INT4 per-token per-group asymmetric quantisation with error annotation.
 * x: [T][128] float32.  s,z returned in float32 (caller rounds to half for
 * storage); rel_err uses the float32 s,z.  int4_group_quantise.py:46-77 */
void cqa_o_quant_values_int4(const float *x, long T, uint8_t *packed, float *s_out, float *z_out,
                             float *rel_err, float *abs_err)
{
#pragma omp parallel for schedule(static)
    for (long t = 0; t < T; ++t) {
        const float *xt = x + t * D;
        float diff[D];
        uint8_t code[D];
        for (int g = 0; g < NG; ++g) {
            float lo = xt[g * GS], hi = lo;
            for (int i = 1; i < GS; ++i) {
                float v = xt[g * GS + i];
                lo = v < lo ? v : lo;
                hi = v > hi ? v : hi;
            }
            float range = hi - lo;
            if (range < 1e-8f) range = 1e-8f;
            float s = range / 15.0f;
            float z = lo;
            s_out[t * NG + g] = s;
            z_out[t * NG + g] = z;
            for (int i = 0; i < GS; ++i) {
                float v = xt[g * GS + i];
                float r = rintf((v - z) / s);
                if (r < 0.0f) r = 0.0f;
                if (r > 15.0f) r = 15.0f;
                code[g * GS + i] = (uint8_t)r;
                float deq = r * s;
                deq = deq + z;
                diff[g * GS + i] = v - deq;
            }
        }
        for (int j = 0; j < D / 2; ++j)
            packed[t * (D / 2) + j] = (uint8_t)((code[2 * j] & 0xF) | ((code[2 * j + 1] & 0xF) << 4));
        float ae = sqrtf(dot128(diff, diff));
        float xn = sqrtf(dot128(xt, xt));
        if (xn < 1e-6f) xn = 1e-6f;
        abs_err[t] = ae;
        rel_err[t] = ae / xn;
    }
}

/* Per-token L2 norm.  tiered_kv_cache.py:229-234 */
void cqa_o_row_norms(const float *v, long T, float *out)
{
#pragma omp parallel for schedule(static)
    for (long t = 0; t < T; ++t) out[t] = sqrtf(dot128(v + t * D, v + t * D));
}

/* Sum of 16 values in butterfly order (block error sums). */
void cqa_o_block_sum16(const float *x, long nblk, float *out)
{
    for (long b = 0; b < nblk; ++b) {
        float p[16];
        memcpy(p, x + b * 16, sizeof p);
        out[b] = butterfly16(p);
    }
}

/* ------------------------------------------------------------------ Phase 1 */

/* keys: int8 [KV][cap][128] with kv stride `kstride` (in rows); scale/zp
 * [KV][maxblk][128] with kv stride `sstride` (in blocks).  q [H][128].
 * Outputs m_b,S_b [H][nq]; tok [KV][nq][G][16] (token scores).
 * score = (dot(k, q*sigma) + dot(q, z)) * q_scale.  fused_score_certify.py:268-289 */
void cqa_o_score_blocks(const int8_t *keys, long kstride, const float *scale, const float *zp,
                        long sstride, const float *q, int KV, int G, long nq, float q_scale,
                        float *m_b, float *S_b, float *tok)
{
    int H = KV * G;
    (void)H;
#pragma omp parallel for collapse(2) schedule(static)
    for (int kv = 0; kv < KV; ++kv)
        for (long b = 0; b < nq; ++b) {
            const float *s = scale + (kv * sstride + b) * D;
            const float *z = zp + (kv * sstride + b) * D;
            for (int g = 0; g < G; ++g) {
                int h = kv * G + g;
                const float *qh = q + h * D;
                float qs[D];
                for (int c = 0; c < D; ++c) qs[c] = qh[c] * s[c];
                float zq = dot128(qh, z);
                float sc[BS];
                float mx = -INFINITY;
                for (int t = 0; t < BS; ++t) {
                    const int8_t *kr = keys + ((long)kv * kstride + b * BS + t) * D;
                    float d = dot128_i8(kr, qs);
                    float v = (d + zq) * q_scale;
                    sc[t] = v;
                    mx = v > mx ? v : mx;
                }
                float e[BS];
                for (int t = 0; t < BS; ++t) e[t] = cqa_o_exp(sc[t] - mx);
                m_b[(long)h * nq + b] = mx;
                S_b[(long)h * nq + b] = butterfly16(e);
                if (tok) memcpy(tok + (((long)kv * nq + b) * G + g) * BS, sc, sizeof sc);
            }
        }
}

/* FP16-key block scores for selected (head, block) pairs.
 * keysf: [KV][tstride][128] float32 (Tier-2 keys widened exactly), indexed by
 * slot*16+t.  idx [H][K]; slots [nblocks_slots] (block -> slot, <0 = absent).
 * Tokens at block*16+t >= n_scoring_tokens are invalid (-inf).
 * fp16_block_scores_triton.py:39-70 */
void cqa_o_fp16_block_scores(const float *keysf, long tstride, long scratch_tokens, const float *q,
                             const int32_t *idx, const int32_t *slots, int H, int G, int K,
                             long n_scoring_tokens, float q_scale, float *scores, float *logmass)
{
    for (int h = 0; h < H; ++h)
        for (int kk = 0; kk < K; ++kk) {
            long bid = idx[h * K + kk];
            int valid_block = bid >= 0 && bid * BS < n_scoring_tokens;
            long slot = valid_block ? slots[bid] : -1;
            float lg[BS];
            float mx = -INFINITY;
            for (int t = 0; t < BS; ++t) {
                long ti = slot * BS + t;
                int valid = valid_block && (bid * BS + t) < n_scoring_tokens && slot >= 0 &&
                            ti < scratch_tokens;
                if (valid) {
                    const float *kr = keysf + ((long)(h / G) * tstride + ti) * D;
                    lg[t] = dot128(kr, q + h * D) * q_scale;
                } else {
                    lg[t] = -INFINITY;
                }
                mx = lg[t] > mx ? lg[t] : mx;
            }
            float e[BS];
            for (int t = 0; t < BS; ++t) e[t] = lg[t] == -INFINITY ? 0.0f : cqa_o_exp(lg[t] - mx);
            float l = butterfly16(e);
            if (l < 1e-30f) l = 1e-30f;
            scores[h * K + kk] = mx;
            logmass[h * K + kk] = mx == -INFINITY ? -INFINITY : mx + cqa_o_log(l);
        }
}

/* Block mass fractions per head.  The reference computes mass = exp(log(max(S,1e-30)) + m - max m) and
 * frac = mass / max(sum(mass), 1e-30) (certified_attention.py:345-350) without fixing the rounding of either; the
 * canonical form here is the algebraically equal
 *     mass = max(S,1e-30) * exp(m - max m),  frac = mass * (1 / max(canonical_sum(mass), 1e-30))
 * (one exponential and one multiplication per block, one division per head).
 * Also returns ell = m + log(max(S,1e-30)) (block log-mass, :1683-1686), which the boundary check uses. */
void cqa_o_mass_frac(const float *m_b, const float *S_b, int H, long nq, float *frac, float *ell,
                     float *m_global, float *total_out)
{
#pragma omp parallel for schedule(static)
    for (int h = 0; h < H; ++h) {
        const float *m = m_b + (long)h * nq, *S = S_b + (long)h * nq;
        float mg = -INFINITY;
        for (long b = 0; b < nq; ++b) mg = m[b] > mg ? m[b] : mg;
        float *f = frac + (long)h * nq;
        for (long b = 0; b < nq; ++b) {
            float s = S[b] < 1e-30f ? 1e-30f : S[b];
            if (ell) ell[(long)h * nq + b] = cqa_o_log(s) + m[b];
            f[b] = s * cqa_o_exp(m[b] - mg);
        }
        float tot = cqa_o_canonical_sum(f, nq);
        if (tot < 1e-30f) tot = 1e-30f;
        const float inv = 1.0f / tot;
        for (long b = 0; b < nq; ++b) f[b] = f[b] * inv;
        if (m_global) m_global[h] = mg;
        if (total_out) total_out[h] = tot;
    }
}

/* Delta[h] = dot(|q_h|, sigma_max[kv(h)]) / (2*sqrt(128)).  :912-945 */
void cqa_o_delta_bound(const float *q, const float *sigma_max, int H, int G, float *delta)
{
    const float denom = (float)(2.0 * sqrt(128.0));
    for (int h = 0; h < H; ++h) {
        float a[D];
        for (int c = 0; c < D; ++c) a[c] = fabsf(q[h * D + c]);
        delta[h] = dot128(a, sigma_max + (h / G) * D) / denom;
    }
}

/* ------------------------------------------------------------------ Phase 2 */

/* Mixed attend, double-precision ground truth.
 *   keys int8/scale/zp as in score_blocks; keysf: Tier-2 keys widened to f32
 *   [KV][kf_stride][128] addressed by key_slots[b]*16+t; vpacked [KV][cap][64],
 *   vs,vz [KV][cap][8] float32 (the half-rounded scale/zero widened), kv stride
 *   `vstride` rows; valsf Tier-2 values [KV][vf_stride][128] addressed by
 *   val_slots[b]*16+t.  topk/vmask: [H][nblk] int32.  last_valid: valid tokens
 *   in block nblk-1.  out [H][128] double.
 *   Also returns per-head logsumexp (m + log l) in lse[H] for split merges. */
void cqa_o_attend_mixed(const int8_t *keys, long kstride, const float *scale, const float *zp,
                        long sstride, const float *keysf, long kf_stride, const int32_t *key_slots,
                        const uint8_t *vpacked, const float *vs, const float *vz, long vstride,
                        const float *valsf, long vf_stride, const int32_t *val_slots,
                        const int32_t *topk, const int32_t *vmask, const float *q, int KV, int G,
                        long nblk, int last_valid, float q_scale, double *out, double *lse)
{
    int H = KV * G;
#pragma omp parallel for schedule(dynamic, 1)
    for (int h = 0; h < H; ++h) {
        int kv = h / G;
        const float *qh = q + h * D;
        double *logit = (double *)malloc(sizeof(double) * nblk * BS);
        double mx = -INFINITY;
        for (long b = 0; b < nblk; ++b) {
            int use16 = topk[(long)h * nblk + b] != 0;
            long ks = key_slots[b] < 0 ? 0 : key_slots[b];
            const float *s = scale + (kv * sstride + b) * D;
            const float *z = zp + (kv * sstride + b) * D;
            for (int t = 0; t < BS; ++t) {
                double acc = 0.0;
                if (use16) {
                    const float *kr = keysf + ((long)kv * kf_stride + ks * BS + t) * D;
                    for (int c = 0; c < D; ++c) acc += (double)kr[c] * (double)qh[c];
                } else {
                    const int8_t *kr = keys + ((long)kv * kstride + b * BS + t) * D;
                    for (int c = 0; c < D; ++c)
                        acc += ((double)kr[c] * (double)s[c] + (double)z[c]) * (double)qh[c];
                }
                double v = acc * (double)q_scale;
                if (b == nblk - 1 && t >= last_valid) v = -INFINITY;
                logit[b * BS + t] = v;
                if (v > mx) mx = v;
            }
        }
        double l = 0.0, acc[D];
        for (int c = 0; c < D; ++c) acc[c] = 0.0;
        for (long b = 0; b < nblk; ++b) {
            int v16 = vmask[(long)h * nblk + b] != 0;
            long vslot = val_slots[b] < 0 ? 0 : val_slots[b];
            for (int t = 0; t < BS; ++t) {
                double lg = logit[b * BS + t];
                if (lg == -INFINITY) continue;
                double w = exp(lg - mx);
                l += w;
                if (v16) {
                    const float *vr = valsf + ((long)kv * vf_stride + vslot * BS + t) * D;
                    for (int c = 0; c < D; ++c) acc[c] += w * (double)vr[c];
                } else {
                    long row = (long)kv * vstride + b * BS + t;
                    const uint8_t *pr = vpacked + row * (D / 2);
                    for (int c = 0; c < D; ++c) {
                        int code = (c & 1) ? (pr[c >> 1] >> 4) & 0xF : pr[c >> 1] & 0xF;
                        double val = (double)code * (double)vs[row * NG + c / GS] +
                                     (double)vz[row * NG + c / GS];
                        acc[c] += w * val;
                    }
                }
            }
        }
        double safe_l = l > 0.0 ? l : 1.0;
        for (int c = 0; c < D; ++c) out[h * D + c] = acc[c] / safe_l;
        if (lse) lse[h] = l > 0.0 ? mx + log(l) : -INFINITY;
        free(logit);
    }
}

/* Dense attention over Tier-2 keys/values for listed heads, double precision.
 * keysf/valsf: [KV][stride][128] float32, tokens [0, nt).  :872-878 */
void cqa_o_dense_attend(const float *keysf, long kf_stride, const float *valsf, long vf_stride,
                        const float *q, const int32_t *heads, int nheads, int G, long nt,
                        float q_scale, double *out /* [nheads][128] */)
{
#pragma omp parallel for schedule(dynamic, 1)
    for (int i = 0; i < nheads; ++i) {
        int h = heads[i], kv = h / G;
        const float *qh = q + h * D;
        double *logit = (double *)malloc(sizeof(double) * nt);
        double mx = -INFINITY;
        for (long t = 0; t < nt; ++t) {
            const float *kr = keysf + ((long)kv * kf_stride + t) * D;
            double a = 0.0;
            for (int c = 0; c < D; ++c) a += (double)kr[c] * (double)qh[c];
            a *= (double)q_scale;
            logit[t] = a;
            if (a > mx) mx = a;
        }
        double l = 0.0, acc[D];
        for (int c = 0; c < D; ++c) acc[c] = 0.0;
        for (long t = 0; t < nt; ++t) {
            double w = exp(logit[t] - mx);
            l += w;
            const float *vr = valsf + ((long)kv * vf_stride + t) * D;
            for (int c = 0; c < D; ++c) acc[c] += w * (double)vr[c];
        }
        for (int c = 0; c < D; ++c) out[i * D + c] = acc[c] / l;
        free(logit);
    }
}

/* Single-precision mixed attend used only as the timed CPU baseline (same
 * data movement as the double-precision version, float arithmetic, token
 * scores reused from Phase 1 for INT8 blocks). */
void cqa_o_attend_mixed_f32(const float *tok /* [KV][nq][G][16] */, long nq, const float *keysf,
                            long kf_stride, const int32_t *key_slots, const uint8_t *vpacked,
                            const float *vs, const float *vz, long vstride, const float *valsf,
                            long vf_stride, const int32_t *val_slots, const int32_t *topk,
                            const int32_t *vmask, const float *q, int KV, int G, long nblk,
                            int last_valid, float q_scale, float *out)
{
    int H = KV * G;
#pragma omp parallel for schedule(dynamic, 1)
    for (int h = 0; h < H; ++h) {
        int kv = h / G, g = h % G;
        const float *qh = q + h * D;
        float m = -INFINITY, l = 0.0f, acc[D];
        for (int c = 0; c < D; ++c) acc[c] = 0.0f;
        for (long b = 0; b < nblk; ++b) {
            float sc[BS];
            int use16 = topk[(long)h * nblk + b] != 0 || b >= nq;
            if (use16) {
                long ks = key_slots[b] < 0 ? 0 : key_slots[b];
                for (int t = 0; t < BS; ++t)
                    sc[t] = dot128(keysf + ((long)kv * kf_stride + ks * BS + t) * D, qh) * q_scale;
            } else {
                memcpy(sc, tok + (((long)kv * nq + b) * G + g) * BS, sizeof sc);
            }
            float bm = -INFINITY;
            for (int t = 0; t < BS; ++t) {
                if (b == nblk - 1 && t >= last_valid) sc[t] = -INFINITY;
                bm = sc[t] > bm ? sc[t] : bm;
            }
            float nm = bm > m ? bm : m;
            float alpha = expf(m - nm);
            l *= alpha;
            for (int c = 0; c < D; ++c) acc[c] *= alpha;
            int v16 = vmask[(long)h * nblk + b] != 0;
            long vslot = val_slots[b] < 0 ? 0 : val_slots[b];
            for (int t = 0; t < BS; ++t) {
                float w = expf(sc[t] - nm);
                l += w;
                if (v16) {
                    const float *vr = valsf + ((long)kv * vf_stride + vslot * BS + t) * D;
                    for (int c = 0; c < D; ++c) acc[c] = fmaf(w, vr[c], acc[c]);
                } else {
                    long row = (long)kv * vstride + b * BS + t;
                    const uint8_t *pr = vpacked + row * (D / 2);
                    for (int c = 0; c < D; c += 2) {
                        uint8_t by = pr[c >> 1];
                        float s = vs[row * NG + c / GS], z = vz[row * NG + c / GS];
                        acc[c] = fmaf(w, fmaf((float)(by & 0xF), s, z), acc[c]);
                        acc[c + 1] = fmaf(w, fmaf((float)(by >> 4), s, z), acc[c + 1]);
                    }
                }
            }
            m = nm;
        }
        float safe_l = l > 0.0f ? l : 1.0f;
        for (int c = 0; c < D; ++c) out[h * D + c] = acc[c] / safe_l;
    }
}
