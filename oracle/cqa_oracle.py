"""CPU oracle for certified quantised decode attention (numpy + C).

TEST INFRASTRUCTURE ONLY.  Only the tests, the smoke check and the
benchmark's CPU-baseline leg may import this module; the product package
never does.  It restates, for one layer and one decode step, what the
reference project (DeanoC/certified-quantised-attention) computes in
  dotcache/kernels/tiered_kv_cache.py      (cache build, append_token)
  dotcache/kernels/int4_group_quantise.py  (INT4 values)
  dotcache/kernels/certified_attention.py  (certified_attention_layer)
with the arithmetic-critical parts in `cqa_oracle.c` (canonical IEEE
binary32 operation order) and the control flow here.  Parity of this oracle
with the reference is pinned by the golden vectors under tests/golden/,
which were produced by running the reference's own code (see
tests/golden/make_golden.py).
"""
from __future__ import annotations

import ctypes as C
import math
import os
import subprocess
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
_SO = HERE / "libcqa_oracle.so"
BS = 16
D = 128
NG = 8

f32 = np.float32


def build(force: bool = False) -> Path:
    """Compile cqa_oracle.c into libcqa_oracle.so (gcc)."""
    src = HERE / "cqa_oracle.c"
    if force or not _SO.exists() or _SO.stat().st_mtime < src.stat().st_mtime:
        cmd = [
            "gcc", "-O2", "-shared", "-fPIC", "-ffp-contract=off", "-fno-fast-math",
            "-march=x86-64-v3", "-fopenmp", "-o", str(_SO), str(src), "-lm",
        ]
        subprocess.check_call(cmd)
    return _SO


_lib = None


def lib():
    global _lib
    if _lib is None:
        if not _SO.exists():
            build()
        _lib = C.CDLL(str(_SO))
        _lib.cqa_o_exp.restype = C.c_float
        _lib.cqa_o_exp.argtypes = [C.c_float]
        _lib.cqa_o_log.restype = C.c_float
        _lib.cqa_o_log.argtypes = [C.c_float]
        _lib.cqa_o_canonical_sum.restype = C.c_float
        _lib.cqa_o_column_sum.restype = C.c_float
    return _lib


def set_threads(n: int) -> int:
    """Use `n` OpenMP threads for the parallel loops (a launcher such as torchrun exports OMP_NUM_THREADS=1, which
    would silently serialise them).  Returns the number now in effect."""
    lib().cqa_o_set_threads(C.c_int(int(n)))
    return int(lib().cqa_o_max_threads())


def _p(a):
    return a.ctypes.data_as(C.c_void_p) if a is not None else None


def _c(a, dt):
    return np.ascontiguousarray(a, dtype=dt)


# --------------------------------------------------------------------------- primitives

def exp32(x):
    return f32(lib().cqa_o_exp(C.c_float(float(x))))


def log32(x):
    return f32(lib().cqa_o_log(C.c_float(float(x))))


def canonical_sum(x) -> np.float32:
    x = _c(x, np.float32)
    return f32(lib().cqa_o_canonical_sum(_p(x), C.c_long(x.size)))


def column_sum(x, include=None) -> np.float32:
    """Sum of x[include] in the fixed column order of the Rung-2 value check (1024 columns, butterflies)."""
    x = _c(x, np.float32)
    inc = None if include is None else _c(include, np.uint8)
    return f32(lib().cqa_o_column_sum(_p(x), _p(inc), C.c_long(x.size)))


def leaf_sums(x) -> np.ndarray:
    x = _c(x, np.float32)
    out = np.zeros((x.size + 255) // 256, dtype=np.float32)
    lib().cqa_o_leaf_sums(_p(x), C.c_long(x.size), _p(out))
    return out


def seq_cumsum(x) -> np.ndarray:
    x = _c(x, np.float32)
    out = np.empty_like(x)
    if x.size:
        lib().cqa_o_seq_cumsum(_p(x), C.c_long(x.size), _p(out))
    return out


def quant_keys(k_blocks: np.ndarray):
    """k_blocks [..., nblk*16, 128] float32 -> (int8, scale, zp, corr)."""
    k = _c(k_blocks, np.float32).reshape(-1, BS, D)
    nblk = k.shape[0]
    q = np.empty((nblk, BS, D), dtype=np.int8)
    s = np.empty((nblk, D), dtype=np.float32)
    z = np.empty((nblk, D), dtype=np.float32)
    corr = np.empty((nblk,), dtype=np.float32)
    lib().cqa_o_quant_keys(_p(k), C.c_long(nblk), _p(q), _p(s), _p(z), _p(corr))
    return q, s, z, corr


def quant_values_int4(x: np.ndarray):
    """x [T,128] float32 -> dict like the reference's quantise_int4_grouped
    (int4_group_quantise.py:22-88)."""
    x = _c(x, np.float32).reshape(-1, D)
    T = x.shape[0]
    packed = np.empty((T, D // 2), dtype=np.uint8)
    s = np.empty((T, NG), dtype=np.float32)
    z = np.empty((T, NG), dtype=np.float32)
    rel = np.empty((T,), dtype=np.float32)
    ab = np.empty((T,), dtype=np.float32)
    lib().cqa_o_quant_values_int4(_p(x), C.c_long(T), _p(packed), _p(s), _p(z), _p(rel), _p(ab))
    return dict(data_packed=packed, scales=s.astype(np.float16), zeros=z.astype(np.float16),
                per_token_error=rel, per_token_abs_error=ab)


def row_norms(v: np.ndarray) -> np.ndarray:
    v = _c(v, np.float32).reshape(-1, D)
    out = np.empty((v.shape[0],), dtype=np.float32)
    lib().cqa_o_row_norms(_p(v), C.c_long(v.shape[0]), _p(out))
    return out


def block_sum16(x: np.ndarray) -> np.ndarray:
    x = _c(x, np.float32).reshape(-1, BS)
    out = np.empty((x.shape[0],), dtype=np.float32)
    lib().cqa_o_block_sum16(_p(x), C.c_long(x.shape[0]), _p(out))
    return out


def to_half_f32(x: np.ndarray) -> np.ndarray:
    """float32 -> IEEE half (round to nearest even) -> float32."""
    return np.asarray(x, dtype=np.float32).astype(np.float16).astype(np.float32)


# --------------------------------------------------------------------------- cache

class OracleCache:
    """numpy restatement of TieredKeyCacheLayer in full-mirror mode
    (tiered_kv_cache.py:29-132): Tier-1 INT8 keys / INT4 values plus Tier-2
    originals kept as float32 arrays holding model-dtype values."""

    def __init__(self):
        self.block_size = BS

    @classmethod
    def from_fp16_cache_int4v(cls, keys, values, dtype: str, max_new_tokens: int = 512,
                              defer_int4_append_quantization: bool = True):
        """keys/values [KV, N, 128] float32 arrays whose values are already
        representable in `dtype`; N block aligned.  tiered_kv_cache.py:135-405."""
        self = cls()
        keys = _c(keys, np.float32)
        values = _c(values, np.float32)
        KV, N, d = keys.shape
        assert d == D and N % BS == 0
        self.dtype = dtype
        self.kv_heads, self.head_dim, self.d_v = KV, D, D
        nb = N // BS
        cap = N + max_new_tokens
        max_new_blocks = (max_new_tokens + BS - 1) // BS
        maxblk = nb + max_new_blocks
        self.capacity, self.max_blocks = cap, maxblk
        self.keys_int8 = np.zeros((KV, cap, D), dtype=np.int8)
        self.keys_scale = np.zeros((KV, maxblk, D), dtype=np.float32)
        self.keys_zero_points = np.zeros((KV, maxblk, D), dtype=np.float32)
        self.correction = np.ones((KV, maxblk), dtype=np.float32)
        self.values_norm_max_per_block = np.zeros((KV, maxblk), dtype=np.float32)
        self.keys_t2 = np.zeros((KV, cap, D), dtype=np.float32)
        self.values_t2 = np.zeros((KV, cap, D), dtype=np.float32)
        self.keys_t2[:, :N] = keys
        self.values_t2[:, :N] = values
        if nb:
            q, s, z, corr = quant_keys(keys)
            self.keys_int8[:, :N] = q.reshape(KV, N, D)
            self.keys_scale[:, :nb] = s.reshape(KV, nb, D)
            self.keys_zero_points[:, :nb] = z.reshape(KV, nb, D)
            self.correction[:, :nb] = corr.reshape(KV, nb)
            self.values_norm_max_per_block[:, :nb] = row_norms(values).reshape(KV, nb, BS).max(axis=2)
        self.sigma_max = (self.keys_scale[:, :nb].max(axis=1) if nb
                          else np.zeros((KV, D), dtype=np.float32))
        # INT4 values: values.to(float16) first (tiered_kv_cache.py:322-324).
        self.values_int4_packed = np.zeros((KV, cap, D // 2), dtype=np.uint8)
        self.values_int4_scales = np.zeros((KV, cap, NG), dtype=np.float16)
        self.values_int4_zeros = np.zeros((KV, cap, NG), dtype=np.float16)
        self.values_int4_errors = np.zeros((KV, maxblk), dtype=np.float32)
        self.values_int4_error_sums = np.zeros((KV, maxblk), dtype=np.float32)
        self.values_int4_error_counts = np.zeros((KV, maxblk), dtype=np.int32)
        if nb:
            r = quant_values_int4(to_half_f32(values))
            self.values_int4_packed[:, :N] = r["data_packed"].reshape(KV, N, D // 2)
            self.values_int4_scales[:, :N] = r["scales"].reshape(KV, N, NG)
            self.values_int4_zeros[:, :N] = r["zeros"].reshape(KV, N, NG)
            pte = r["per_token_error"].reshape(KV, nb, BS)
            self.values_int4_errors[:, :nb] = pte.max(axis=2)
            self.values_int4_error_sums[:, :nb] = block_sum16(pte).reshape(KV, nb)
            self.values_int4_error_counts[:, :nb] = BS
        self.defer = bool(defer_int4_append_quantization)
        self.num_tokens = N
        self.num_blocks = nb
        self.num_quantized_blocks = nb
        return self

    # -- append (tiered_kv_cache.py:545-708)
    def append_token(self, k_new, v_new):
        """k_new, v_new: [KV, 1, 128] or [KV, 128] float32 (model-dtype values)."""
        k_new = _c(k_new, np.float32).reshape(self.kv_heads, D)
        v_new = _c(v_new, np.float32).reshape(self.kv_heads, D)
        pos = self.num_tokens
        b, pib = pos // BS, pos % BS
        vn = row_norms(v_new)
        self.values_norm_max_per_block[:, b] = np.maximum(self.values_norm_max_per_block[:, b], vn)
        if not self.defer:
            r = quant_values_int4(v_new)
            self.values_int4_packed[:, pos] = r["data_packed"]
            self.values_int4_scales[:, pos] = r["scales"]
            self.values_int4_zeros[:, pos] = r["zeros"]
            err = r["per_token_error"]
            self.values_int4_error_sums[:, b] = self.values_int4_error_sums[:, b] + err
            self.values_int4_error_counts[:, b] += 1
            self.values_int4_errors[:, b] = np.maximum(self.values_int4_errors[:, b], err)
        self.keys_t2[:, pos] = k_new
        self.values_t2[:, pos] = v_new
        self.num_tokens = pos + 1
        self.num_blocks = (self.num_tokens + BS - 1) // BS
        if pib == BS - 1:
            if self.defer:
                self._quantize_value_block(b)
            self._quantize_block(b)
        if pib == 0 and self.num_tokens < self.aligned_tokens:
            self.keys_int8[:, self.num_tokens:self.aligned_tokens] = -127

    def _quantize_value_block(self, b):
        st, en = b * BS, (b + 1) * BS
        blk = to_half_f32(self.values_t2[:, st:en]).reshape(-1, D)
        r = quant_values_int4(blk)
        KV = self.kv_heads
        self.values_int4_packed[:, st:en] = r["data_packed"].reshape(KV, BS, D // 2)
        self.values_int4_scales[:, st:en] = r["scales"].reshape(KV, BS, NG)
        self.values_int4_zeros[:, st:en] = r["zeros"].reshape(KV, BS, NG)
        s = block_sum16(r["per_token_error"].reshape(KV, BS))
        self.values_int4_errors[:, b] = s / f32(BS)
        self.values_int4_error_sums[:, b] = s
        self.values_int4_error_counts[:, b] = BS

    def _quantize_block(self, b):
        st, en = b * BS, (b + 1) * BS
        q, s, z, corr = quant_keys(self.keys_t2[:, st:en])
        KV = self.kv_heads
        self.keys_int8[:, st:en] = q.reshape(KV, BS, D)
        self.keys_scale[:, b] = s
        self.keys_zero_points[:, b] = z
        self.correction[:, b] = corr
        self.sigma_max = np.maximum(self.sigma_max, s)
        self.num_quantized_blocks = b + 1

    @property
    def aligned_tokens(self):
        return ((self.num_tokens + BS - 1) // BS) * BS

    @property
    def active_blocks(self):
        return (self.num_tokens + BS - 1) // BS

    @property
    def has_trailing_partial_block(self):
        return self.num_tokens > 0 and self.num_tokens % BS != 0

    def v_max_global(self):
        a = self.values_norm_max_per_block[:, :self.active_blocks]
        return float(a.max()) if a.size else 0.0


# --------------------------------------------------------------------------- kernels

def score_blocks(cache: OracleCache, q, gqa_group, q_scale):
    """Phase 1: returns (m_b [H,nq], S_b [H,nq], token_scores [KV,nq,G,16])."""
    KV, G = cache.kv_heads, gqa_group
    H = KV * G
    nq = cache.num_quantized_blocks
    q = _c(q, np.float32)
    m_b = np.empty((H, nq), dtype=np.float32)
    S_b = np.empty((H, nq), dtype=np.float32)
    tok = np.empty((KV, nq, G, BS), dtype=np.float32)
    if nq:
        lib().cqa_o_score_blocks(
            _p(cache.keys_int8), C.c_long(cache.capacity), _p(cache.keys_scale),
            _p(cache.keys_zero_points), C.c_long(cache.max_blocks), _p(q), C.c_int(KV), C.c_int(G),
            C.c_long(nq), C.c_float(q_scale), _p(m_b), _p(S_b), _p(tok))
    return m_b, S_b, tok


def fp16_block_scores(cache: OracleCache, q, idx, gqa_group, q_scale, n_scoring_blocks):
    q = _c(q, np.float32)
    idx = _c(idx, np.int32)
    H, K = idx.shape
    slots = np.arange(max(n_scoring_blocks, 1), dtype=np.int32)
    scores = np.empty((H, K), dtype=np.float32)
    logmass = np.empty((H, K), dtype=np.float32)
    lib().cqa_o_fp16_block_scores(
        _p(cache.keys_t2), C.c_long(cache.capacity), C.c_long(cache.capacity), _p(q), _p(idx),
        _p(slots), C.c_int(H), C.c_int(gqa_group), C.c_int(K),
        C.c_long(n_scoring_blocks * BS), C.c_float(q_scale), _p(scores), _p(logmass))
    return scores, logmass


def mass_frac(m_b, S_b):
    m_b = _c(m_b, np.float32)
    S_b = _c(S_b, np.float32)
    H, nq = m_b.shape
    frac = np.empty((H, nq), dtype=np.float32)
    ell = np.empty((H, nq), dtype=np.float32)
    mg = np.empty((H,), dtype=np.float32)
    tot = np.empty((H,), dtype=np.float32)
    lib().cqa_o_mass_frac(_p(m_b), _p(S_b), C.c_int(H), C.c_long(nq), _p(frac), _p(ell), _p(mg), _p(tot))
    return frac, ell, mg, tot


def delta_bound(q, sigma_max, gqa_group):
    q = _c(q, np.float32)
    sm = _c(sigma_max, np.float32)
    H = q.shape[0]
    out = np.empty((H,), dtype=np.float32)
    lib().cqa_o_delta_bound(_p(q), _p(sm), C.c_int(H), C.c_int(gqa_group), _p(out))
    return out


def attend_mixed(cache: OracleCache, q, gqa_group, q_scale, topk_mask, value_mask, nblk, last_valid):
    """Phase 2 ground truth in float64.  Identity slot tables (full mirror)."""
    q = _c(q, np.float32)
    KV = cache.kv_heads
    H = KV * gqa_group
    topk = _c(topk_mask, np.int32)
    vm = _c(value_mask, np.int32)
    slots = np.arange(max(nblk, 1), dtype=np.int32)
    vs = cache.values_int4_scales.astype(np.float32)
    vz = cache.values_int4_zeros.astype(np.float32)
    out = np.empty((H, D), dtype=np.float64)
    lse = np.empty((H,), dtype=np.float64)
    lib().cqa_o_attend_mixed(
        _p(cache.keys_int8), C.c_long(cache.capacity), _p(cache.keys_scale),
        _p(cache.keys_zero_points), C.c_long(cache.max_blocks), _p(cache.keys_t2),
        C.c_long(cache.capacity), _p(slots), _p(cache.values_int4_packed), _p(vs), _p(vz),
        C.c_long(cache.capacity), _p(cache.values_t2), C.c_long(cache.capacity), _p(slots),
        _p(topk), _p(vm), _p(q), C.c_int(KV), C.c_int(gqa_group), C.c_long(nblk),
        C.c_int(last_valid), C.c_float(q_scale), _p(out), _p(lse))
    return out, lse


def attend_mixed_f32(cache: OracleCache, q, gqa_group, q_scale, tok, topk_mask, value_mask, nblk,
                     last_valid, _vs=None, _vz=None):
    """float32 CPU baseline of Phase 2 (token scores reused from Phase 1)."""
    q = _c(q, np.float32)
    KV = cache.kv_heads
    H = KV * gqa_group
    topk = _c(topk_mask, np.int32)
    vm = _c(value_mask, np.int32)
    slots = np.arange(max(nblk, 1), dtype=np.int32)
    vs = cache.values_int4_scales.astype(np.float32) if _vs is None else _vs
    vz = cache.values_int4_zeros.astype(np.float32) if _vz is None else _vz
    out = np.empty((H, D), dtype=np.float32)
    lib().cqa_o_attend_mixed_f32(
        _p(tok), C.c_long(cache.num_quantized_blocks), _p(cache.keys_t2), C.c_long(cache.capacity),
        _p(slots), _p(cache.values_int4_packed), _p(vs), _p(vz), C.c_long(cache.capacity),
        _p(cache.values_t2), C.c_long(cache.capacity), _p(slots), _p(topk), _p(vm), _p(q),
        C.c_int(KV), C.c_int(gqa_group), C.c_long(nblk), C.c_int(last_valid), C.c_float(q_scale),
        _p(out))
    return out


def dense_attend(cache: OracleCache, q, heads, gqa_group, q_scale):
    q = _c(q, np.float32)
    heads = _c(heads, np.int32)
    out = np.empty((len(heads), D), dtype=np.float64)
    if len(heads):
        lib().cqa_o_dense_attend(
            _p(cache.keys_t2), C.c_long(cache.capacity), _p(cache.values_t2),
            C.c_long(cache.capacity), _p(q), _p(heads), C.c_int(len(heads)), C.c_int(gqa_group),
            C.c_long(cache.num_tokens), C.c_float(q_scale), _p(out))
    return out


# --------------------------------------------------------------------------- selector / certificate

def _searchsorted_left(cum, tau):
    # first index with cum[i] >= tau (cum non-decreasing)
    return int(np.searchsorted(cum, tau, side="left"))


def adaptive_select(m_b, S_b, tau_cov, k_min, k_max, rung1_threshold=0.02, rung1_multiplier=2.0):
    """Adaptive K* with the Rung-1 expansion derived from one sorted prefix.
    certified_attention.py:245-444 and :1299-1441."""
    H, nq = m_b.shape
    frac, ell, mg, tot = mass_frac(m_b, S_b)
    can_expand = (rung1_threshold is not None and rung1_threshold >= 0 and k_max is not None)
    sel_kmax = k_max
    expanded = None
    if can_expand:
        expanded = min(int(math.ceil(int(k_max) * float(rung1_multiplier))), nq)
        if expanded > int(k_max):
            sel_kmax = expanded
    hi = nq if sel_kmax is None else min(int(sel_kmax), nq)
    two_level = can_expand and expanded is not None and expanded > int(k_max)
    tau32 = f32(tau_cov)
    sorted_idx = np.zeros((H, hi), dtype=np.int32)
    sorted_cumsum = np.zeros((H, hi), dtype=np.float32)
    k_star = np.zeros((H,), dtype=np.int32)
    tail = np.zeros((H,), dtype=np.float32)
    tau_act = np.zeros((H,), dtype=np.float32)
    trig = np.zeros((H,), dtype=bool)
    mask = np.zeros((H, nq), dtype=bool)
    kmargin = np.full((H,), np.inf)
    for h in range(H):
        order = np.argsort(-frac[h], kind="stable")[:hi]
        cum = seq_cumsum(frac[h][order])
        sorted_idx[h] = order
        sorted_cumsum[h] = cum
        lo = min(int(k_min), hi)
        k_e = min(max(_searchsorted_left(cum, tau32) + 1, lo), hi)
        ta_e = cum[k_e - 1]
        tl_e = max(f32(1.0) - ta_e, f32(0.0))
        if two_level:
            bw = min(int(k_max), hi)
            lo_b = min(int(k_min), bw)
            k_b = min(max(_searchsorted_left(cum[:bw], tau32) + 1, lo_b), bw)
            ta_b = cum[k_b - 1]
            tl_b = max(f32(1.0) - ta_b, f32(0.0))
            t = bool(tl_b > f32(rung1_threshold))
            trig[h] = t
            k_star[h], tau_act[h], tail[h] = (k_e, ta_e, tl_e) if t else (k_b, ta_b, tl_b)
        else:
            k_star[h], tau_act[h], tail[h] = k_e, ta_e, tl_e
            if rung1_threshold is not None and rung1_threshold >= 0 and k_max is not None:
                trig[h] = bool(tl_e > f32(rung1_threshold))
        mask[h, order[: k_star[h]]] = True
        near = [abs(float(cum[j]) - float(tau32)) for j in (k_star[h] - 2, k_star[h] - 1) if 0 <= j < hi]
        kmargin[h] = min(near) if near else np.inf
    return dict(kstar_margin=kmargin, mass_frac=frac, ell=ell, m_global=mg, total=tot, sorted_idx=sorted_idx,
                sorted_cumsum=sorted_cumsum, k_star=k_star, tail_mass=tail, tau_actual=tau_act,
                rung1_trigger=trig, topk_mask=mask)


def value_check(frac, eta, gqa_group, v_tolerance, mode="tight"):
    """Rung-2 greedy value promotion.  certified_attention.py:1940-2034."""
    H, nq = frac.shape
    kv_idx = np.minimum(np.arange(H) // gqa_group, eta.shape[0] - 1)
    e = (frac * eta[kv_idx][:, :nq]).astype(np.float32)
    e_pre = np.array([column_sum(e[h]) for h in range(H)], dtype=np.float32)
    unsafe = np.zeros((H, nq), dtype=bool)
    promoted = np.zeros((H,), dtype=np.float32)
    margin = np.full((H,), np.inf)
    vt = f32(v_tolerance)
    if mode == "tight":
        # Greedy promotion over the descending order (ties: lower block id first): the entry at position j is
        # promoted while the column sum of the entries before it is below the excess.  The column sum of a prefix
        # never decreases with its length, so the promoted entries are a prefix and its length can be bisected.
        for h in range(H):
            excess = max(e_pre[h] - vt, f32(0.0))
            if not excess > 0:
                continue
            order = np.argsort(-e[h], kind="stable")
            inc = np.zeros(nq, dtype=np.uint8)

            def before(j):
                inc[:] = 0
                inc[order[:j]] = 1
                return column_sum(e[h], inc)

            lo, hi = 0, nq - 1          # position lo is promoted (nothing before it); find the last promoted one
            while lo < hi:
                mid = (lo + hi + 1) // 2
                if before(mid) < excess:
                    lo = mid
                else:
                    hi = mid - 1
            unsafe[h, order[: lo + 1]] = True
            # decision margins at the promotion boundary, relative to the excess: how far the last "still below"
            # and the first "reached" column sums are from the excess they were compared with
            below, reached = before(lo), before(lo + 1)
            margin[h] = min(float(excess - below), float(reached - excess) if lo + 1 < nq else np.inf) / float(excess)
            promoted[h] = reached
    else:
        unsafe = eta[kv_idx][:, :nq] > vt
        for h in range(H):
            promoted[h] = column_sum(e[h], unsafe[h])
    e_val = np.maximum(e_pre - promoted, f32(0.0)).astype(np.float32)
    return dict(e=e, e_pre=e_pre, unsafe=unsafe, promoted=promoted, e_val=e_val, margin=margin)


def layer_step(cache: OracleCache, q, gqa_group, q_scale=None, *, v_tolerance, top_k_fp16_keys=0,
               ranking_fallback=False, ranking_r=1, ranking_fallback_mode="full", tau_cov=None,
               k_min=2, k_max=None, rung1_threshold=0.02, rung1_multiplier=2.0,
               score_consistency_check=True, eps_guard=0.01, exploration_rate=0.0,
               exploration_u=None, value_error_mode="tight", fp16_values=False):
    """One certified decode step for one layer (adaptive K*, INT4-value cache,
    full-mirror Tier-2).  Follows certified_attention.py:1065-2790 for that
    configuration.  Returns a dict with every intermediate.
    `fp16_values`: the cache holds model-dtype values instead of INT4 (from_fp16_cache, tiered_kv_cache.py:135-286):
    there is no value check and every block reads the original values (certified_attention.py:1827-1829)."""
    if q_scale is None:
        q_scale = 1.0 / math.sqrt(D)
    q = _c(q, np.float32)
    KV = cache.kv_heads
    H = KV * gqa_group
    nq = cache.num_quantized_blocks
    nact = cache.active_blocks
    trailing = cache.has_trailing_partial_block
    assert tau_cov is not None and tau_cov > 0 and nq > 0, "oracle covers the adaptive path"
    R = {}
    m_b, S_b, tok = score_blocks(cache, q, gqa_group, q_scale)
    R.update(m_b=m_b, S_b=S_b, token_scores=tok)
    sel = adaptive_select(m_b, S_b, tau_cov, k_min, k_max, rung1_threshold, rung1_multiplier)
    R.update(sel)
    mask = sel["topk_mask"].copy()
    explore = np.zeros_like(mask)
    if exploration_rate > 0.0:
        assert exploration_u is not None
        explore = (~mask) & (np.asarray(exploration_u, dtype=np.float32) < f32(exploration_rate))
        mask = mask | explore
    R["exploration_mask"] = explore
    topk_active = np.zeros((H, nact), dtype=bool)
    topk_active[:, :nq] = mask
    if trailing:
        topk_active[:, nq:] = True
    R["topk_mask_active"] = topk_active

    # ranking / boundary / score consistency (:1563-1727)
    need_fp16 = (ranking_fallback or score_consistency_check) and nq > 0
    disagree = None
    R["rung4"] = False
    delta = None
    if need_fp16:
        rk = min(max(ranking_r, top_k_fp16_keys, 4), nq)
        top_idx = np.stack([np.argsort(-m_b[h], kind="stable")[:rk] for h in range(H)]).astype(np.int32)
        top_int8 = np.take_along_axis(m_b, top_idx, axis=1)
        fp16_s, fp16_l = fp16_block_scores(cache, q, top_idx, gqa_group, q_scale, nq)
        R.update(ranking_k=rk, top_block_indices=top_idx, top_int8_scores=top_int8,
                 fp16_block_scores=fp16_s, fp16_block_log_masses=fp16_l)
        delta = delta_bound(q, cache.sigma_max, gqa_group)
        R["delta_per_head"] = delta
        if ranking_fallback:
            rank16 = np.stack([np.argsort(-fp16_s[h], kind="stable") for h in range(H)])
            diff = rank16 != np.arange(rk)[None, :]
            r_main = min(int(ranking_r), rk)
            disagree = diff[:, :r_main].any(axis=1)
            R["ranking_disagree_r1"] = int(diff[:, :min(1, rk)].any(axis=1).sum())
            R["ranking_disagree_r3"] = int(diff[:, :min(3, rk)].any(axis=1).sum())
            ub = (sel["ell"] + delta[:, None]).astype(np.float32)
            np.put_along_axis(ub, top_idx.astype(np.int64), -np.inf, axis=1)
            kb = min(int(ranking_r), rk)
            ell_r = -np.sort(-fp16_l, axis=1)[:, kb - 1]
            boundary = ub.max(axis=1) > ell_r
            R["boundary_mask"] = boundary
            R["ranking_only_mask"] = disagree.copy()
            disagree = disagree | boundary
            R["ranking_disagree_mask"] = disagree
        if score_consistency_check:
            thr = (delta + f32(eps_guard)).astype(np.float32)
            viol = (np.abs(fp16_s - top_int8).astype(np.float32) > thr[:, None]).any(axis=1)
            R["score_consistency_violation_mask"] = viol
            R["rung4"] = bool(viol.any())
    if R["rung4"]:
        out = dense_attend(cache, q, np.arange(H, dtype=np.int32), gqa_group, q_scale)
        R["output"] = out
        return R

    # value check (:1940-2058)
    if fp16_values:
        vmask = np.ones((H, nact), dtype=bool)
        R.update(e_pre=np.zeros(H, np.float32), e_val=np.zeros(H, np.float32),
                 value_unsafe_mask=np.zeros((H, nq), dtype=bool))
    else:
        vc = value_check(sel["mass_frac"], cache.values_int4_errors[:, :nq], gqa_group, v_tolerance,
                         value_error_mode)
        R.update(e_pre=vc["e_pre"], e_val=vc["e_val"], value_unsafe_mask=vc["unsafe"], value_margin=vc["margin"])
        vmask = np.zeros((H, nact), dtype=bool)
        vmask[:, :nq] = vc["unsafe"]
        if trailing:
            vmask[:, nq:] = True
    R["value_fp16_mask"] = vmask
    last_valid = BS if not trailing else cache.num_tokens - nq * BS
    out, lse = attend_mixed(cache, q, gqa_group, q_scale, topk_active, vmask, nact, last_valid)
    R["phase2_output"] = out.copy()
    R["last_block_valid"] = last_valid
    # Rung 3 (:2584-2605)
    heads = np.zeros((0,), dtype=np.int32)
    if ranking_fallback and ranking_fallback_mode == "full" and disagree is not None:
        heads = np.nonzero(disagree)[0].astype(np.int32)
        if heads.size:
            out[heads] = dense_attend(cache, q, heads, gqa_group, q_scale)
    R["rung3_heads"] = heads
    R["output"] = out
    return R
