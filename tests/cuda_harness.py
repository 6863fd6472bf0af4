"""Shared helpers for the GPU parity tests: build a CUDA cache and an oracle
cache from the same seeded inputs, run one layer step on both, and compare.

Selection-relevant values (packed bytes, block scores, mass fractions, sorted
order, masks, certificate flags) must be bit-identical between the CUDA path
and the CPU oracle; attention outputs agree within OUT_RTOL of the row scale.
"""
from __future__ import annotations

import numpy as np
import torch

import golden_cases as gc  # noqa: F401  (sets sys.path)
from oracle import cqa_oracle as orc
from dotcache.kernels import certified_attention as ca
from dotcache.kernels.tiered_kv_cache import TieredKeyCacheLayer

OUT_RTOL = 1e-3
TORCH_DTYPE = {"float32": torch.float32, "float16": torch.float16, "bfloat16": torch.bfloat16}


def to_dev(a: np.ndarray, dtype: str) -> torch.Tensor:
    return torch.from_numpy(np.ascontiguousarray(a)).to(TORCH_DTYPE[dtype]).cuda()


def make_cuda_cache(k, v, dtype, max_new, defer=True):
    return TieredKeyCacheLayer.from_fp16_cache_int4v(
        to_dev(k, dtype), to_dev(v, dtype), max_new_tokens=max_new, defer_int4_append_quantization=defer)


def make_oracle_cache(k, v, dtype, max_new, defer=True):
    return orc.OracleCache.from_fp16_cache_int4v(k, v, dtype, max_new_tokens=max_new,
                                                 defer_int4_append_quantization=defer)


def bits(a: np.ndarray) -> np.ndarray:
    a = np.ascontiguousarray(a)
    return a.view(np.uint32) if a.dtype == np.float32 else a.view(np.uint16) if a.dtype == np.float16 else a


def assert_bits_equal(a, b, what):
    a = np.ascontiguousarray(a)
    b = np.ascontiguousarray(b)
    assert a.shape == b.shape, f"{what}: shape {a.shape} vs {b.shape}"
    same = bits(a) == bits(b)
    if not same.all():
        bad = np.argwhere(~same)
        i = tuple(bad[0])
        raise AssertionError(f"{what}: {len(bad)} of {a.size} elements differ; first at {i}: "
                             f"cuda={a[i]!r} oracle={b[i]!r}")


def t2_as_f32(t: torch.Tensor) -> np.ndarray:
    return t.float().cpu().numpy()


def compare_caches(cc: TieredKeyCacheLayer, oc: orc.OracleCache, what=""):
    """Every Tier-1 array, the annotations and the Tier-2 rows, bit for bit."""
    assert cc.num_tokens == oc.num_tokens and cc.num_quantized_blocks == oc.num_quantized_blocks
    assert cc.num_blocks == oc.num_blocks
    nt, nq, nb = oc.num_tokens, oc.num_quantized_blocks, oc.num_blocks
    T = nq * 16
    cpu = lambda t: t.cpu().numpy()
    assert_bits_equal(cpu(cc.keys_int8[:, :T]), oc.keys_int8[:, :T], f"{what} keys_int8")
    assert_bits_equal(cpu(cc.keys_scale[:, :nq]), oc.keys_scale[:, :nq], f"{what} keys_scale")
    assert_bits_equal(cpu(cc.keys_zero_points[:, :nq]), oc.keys_zero_points[:, :nq], f"{what} keys_zero_points")
    assert_bits_equal(cpu(cc.correction[:, :nq]), oc.correction[:, :nq], f"{what} correction")
    assert_bits_equal(cpu(cc.keys_scale_max), oc.sigma_max, f"{what} keys_scale_max")
    vt = T if oc.defer else nt
    assert_bits_equal(cpu(cc.values_int4_packed[:, :vt]), oc.values_int4_packed[:, :vt], f"{what} values_int4_packed")
    assert_bits_equal(cpu(cc.values_int4_scales[:, :vt]), oc.values_int4_scales[:, :vt], f"{what} values_int4_scales")
    assert_bits_equal(cpu(cc.values_int4_zeros[:, :vt]), oc.values_int4_zeros[:, :vt], f"{what} values_int4_zeros")
    eb = nq if oc.defer else nb
    assert_bits_equal(cpu(cc.values_int4_errors[:, :eb]), oc.values_int4_errors[:, :eb], f"{what} eta_b")
    assert_bits_equal(cpu(cc.values_int4_error_sums[:, :eb]), oc.values_int4_error_sums[:, :eb], f"{what} error_sums")
    assert np.array_equal(cpu(cc.values_int4_error_counts[:, :eb]), oc.values_int4_error_counts[:, :eb])
    assert_bits_equal(cpu(cc.values_norm_max_per_block[:, :nb]), oc.values_norm_max_per_block[:, :nb], f"{what} nu_b")
    assert_bits_equal(t2_as_f32(cc.keys_fp16_gpu[:, :nt]), oc.keys_t2[:, :nt], f"{what} Tier-2 keys")
    assert_bits_equal(t2_as_f32(cc.values_fp16_gpu[:, :nt]), oc.values_t2[:, :nt], f"{what} Tier-2 values")
    # poison rows of an open block
    if nt % 16:
        at = ((nt + 15) // 16) * 16
        assert (cpu(cc.keys_int8[:, nt:at]) == -127).all(), f"{what} poison rows"


def cuda_step(cc, q_np, dtype, G, knobs, u=None, collect_stats=True):
    q = to_dev(q_np, dtype)
    kw = dict(knobs)
    if u is not None:
        kw["exploration_uniforms"] = torch.from_numpy(np.ascontiguousarray(u))
    out, stats = ca.certified_attention_layer(cc, q, G, None, collect_stats, **kw)
    torch.cuda.synchronize()
    return out.cpu().numpy().copy(), stats


def compare_step(cc, R, out, what="", check_value=True):
    """CUDA workspace of the last step on `cc` against the oracle result R."""
    ws = cc._certified_workspace["cqa_ws"]
    H = ws.H
    nq = cc.num_quantized_blocks
    nact = cc.active_blocks
    cpu = lambda t: t.cpu().numpy()
    assert_bits_equal(cpu(ws.m_b[:, :nq]), R["m_b"], f"{what} m_b")
    assert_bits_equal(cpu(ws.s_b[:, :nq]), R["S_b"], f"{what} S_b")
    G = ws.G
    tok = cpu(ws.token_scores[: cc.kv_heads * nq * G * 16]).reshape(cc.kv_heads, nq, G, 16)
    assert_bits_equal(tok, R["token_scores"], f"{what} token scores")
    cert, flags = ws.read_cert()
    if R.get("rung4"):
        assert flags[2] == 1, f"{what}: Rung-4 flag not raised"
    else:
        assert_bits_equal(cpu(ws.mass_frac[:, :nq]), R["mass_frac"], f"{what} mass_frac")
        W = R["sorted_idx"].shape[1]
        assert np.array_equal(cpu(ws.sorted_idx[:, :W]), R["sorted_idx"]), f"{what} sorted block order"
        assert_bits_equal(cpu(ws.sorted_cumsum[:, :W]), R["sorted_cumsum"], f"{what} sorted cumsum")
        assert np.array_equal(cert["k_star"], R["k_star"]), f"{what} k_star {cert['k_star']} vs {R['k_star']}"
        assert_bits_equal(cert["tail_mass"].astype(np.float32), R["tail_mass"], f"{what} tail_mass")
        assert_bits_equal(cert["tau_actual"].astype(np.float32), R["tau_actual"], f"{what} tau_actual")
        assert np.array_equal(cert["rung1_triggered"].astype(bool), R["rung1_trigger"]), f"{what} rung1"
        assert np.array_equal(cpu(ws.explore_mask[:, :nq]).astype(bool), R["exploration_mask"]), f"{what} exploration"
        assert np.array_equal(cpu(ws.topk_mask[:, :nact]).astype(bool), R["topk_mask_active"]), f"{what} top-K* mask"
    if "top_block_indices" in R:
        rk = R["ranking_k"]
        assert np.array_equal(cert["top_blocks"][:, :rk], R["top_block_indices"]), f"{what} top blocks by m_b"
        assert_bits_equal(cert["fp16_scores"][:, :rk], R["fp16_block_scores"], f"{what} fp16 block scores")
        assert_bits_equal(cert["fp16_logmass"][:, :rk], R["fp16_block_log_masses"], f"{what} fp16 log-mass")
        assert_bits_equal(cert["delta"].astype(np.float32), R["delta_per_head"], f"{what} delta")
    if "ranking_disagree_mask" in R:
        assert np.array_equal(cert["rung3"].astype(bool), R["ranking_disagree_mask"]), f"{what} rung-3 mask"
        assert np.array_equal(cert["boundary_triggered"].astype(bool), R["boundary_mask"]), f"{what} boundary"
        assert np.array_equal(cert["ranking_disagree"].astype(bool), R["ranking_only_mask"]), f"{what} ranking"
        assert int(cert["ranking_disagree_r1"].sum()) == R["ranking_disagree_r1"]
        assert int(cert["ranking_disagree_r3"].sum()) == R["ranking_disagree_r3"]
    if "score_consistency_violation_mask" in R:
        assert np.array_equal(cert["consistency_violation"].astype(bool), R["score_consistency_violation_mask"])
    if not R.get("rung4") and check_value:
        assert np.array_equal(cpu(ws.value_mask[:, :nact]).astype(bool), R["value_fp16_mask"]), f"{what} value mask"
        assert_bits_equal(cert["e_pre"].astype(np.float32), R["e_pre"], f"{what} e_pre")
        assert_bits_equal(cert["e_val"].astype(np.float32), R["e_val"], f"{what} e_val")
        assert np.array_equal(cert["value_promoted_blocks"], R["value_unsafe_mask"].sum(axis=1))
    ref = R["output"]
    scale = np.abs(ref).max(axis=1, keepdims=True)
    err = np.abs(out.astype(np.float64) - ref) / scale
    assert np.all(err <= OUT_RTOL), f"{what} output: max rel err {err.max():.3e} (head {err.max(axis=1).argmax()})"
    return float(err.max())
