"""GPU tests of every reference-named entry point of the package against the CPU oracle: the backend module
(dotcache.backends.certified_blackwell, dotcache.backends.cuda_pagein), the kernel modules that keep the reference's
names (selective_attend_triton, fused_score_certify, fp16_block_scores_triton, int4_group_quantise), the helper
functions of certified_attention, the FP16-value cache (from_fp16_cache / create_tiered_cache_from_model) end to
end, and the bounded device-side wait that runs out.

Block scores, masks and packed bytes are compared bit for bit; attention rows within 1e-3 of the row scale.
"""
from __future__ import annotations

import ctypes as C

import numpy as np
import pytest
import torch

import golden_cases as gc
from cqa_b200 import synth

pytestmark = pytest.mark.gpu

if torch.cuda.is_available():
    import cuda_harness as hz
    from cqa_b200 import _lib
    from dotcache.backends import certified_blackwell as cb
    from dotcache.backends import cuda_pagein as pg
    from dotcache.kernels import certified_attention as ca
    from dotcache.kernels import fp16_block_scores_triton as f16mod
    from dotcache.kernels import fused_score_certify as fsc
    from dotcache.kernels import int4_group_quantise as i4
    from dotcache.kernels import selective_attend_triton as sat
    from dotcache.kernels.tiered_kv_cache import (TieredKeyCacheLayer, create_tiered_cache_from_model,
                                                  create_tiered_cache_int4v_from_model)
    from oracle import cqa_oracle as orc

Q_SCALE = float(1.0 / np.sqrt(128.0))
DTYPE = "bfloat16"


def _caches(seed, n_tokens, planted=8, extra=0, dtype=DTYPE, max_new=64):
    base = synth.make_layer_inputs(seed, n_tokens + extra, dtype=dtype, n_planted_blocks=planted)
    cc = hz.make_cuda_cache(base.k[:, :n_tokens], base.v[:, :n_tokens], dtype, max_new)
    oc = hz.make_oracle_cache(base.k[:, :n_tokens], base.v[:, :n_tokens], dtype, max_new)
    for t in range(n_tokens, n_tokens + extra):
        cc.append_token(hz.to_dev(base.k[:, t:t + 1], dtype), hz.to_dev(base.v[:, t:t + 1], dtype))
        oc.append_token(base.k[:, t:t + 1], base.v[:, t:t + 1])
    return base, cc, oc


def _knobs_struct(**over):
    """The cqa_knobs struct of the paper operating point (exploration off: no uniforms are passed)."""
    kw = dict(q_scale=Q_SCALE, tau_cov=0.995, k_min=2, k_max=128, rung1_threshold=0.02, rung1_multiplier=2.0,
              eps_guard=0.01, exploration_rate=0.0, v_tolerance=0.05, ranking_r=1, top_k_fp16_keys=4,
              ranking_fallback=True, ranking_fallback_mode="full", score_consistency_check=True,
              value_error_mode="tight", force_trailing_value_fp16=True)
    kw.update(over)
    return ca._make_knobs(**kw)


def _rows_close(got, ref, what, tol=1e-3):
    got = np.asarray(got, dtype=np.float64)
    ref = np.asarray(ref, dtype=np.float64)
    scale = np.abs(ref).max(axis=1, keepdims=True)
    err = np.abs(got - ref) / scale
    assert np.all(err <= tol), f"{what}: max relative error {err.max():.3e}"


# ----------------------------------------------------------------------------- Phase 1

def test_score_blocks_cuda_strided_slice_and_token_scores():
    """score_blocks_cuda on slices of a larger cache (`cache.keys_int8[:, :n]`): nothing is copied, the KV-head
    stride goes to the kernel; with and without the token scores."""
    base, cc, oc = _caches(41, 2048)
    q = hz.to_dev(base.q, DTYPE)
    n = cc.num_quantized_blocks * 16
    nb = cc.num_quantized_blocks
    assert cc.keys_int8.shape[1] > n and not cc.keys_int8[:, :n].is_contiguous()
    m_ref, s_ref, tok_ref = orc.score_blocks(oc, base.q, 4, Q_SCALE)
    m_b, s_b, tok = cb.score_blocks_cuda(
        keys_int8=cc.keys_int8[:, :n], keys_scale=cc.keys_scale[:, :nb], keys_zero_points=cc.keys_zero_points[:, :nb],
        q_all=q, gqa_group=4, q_scale=Q_SCALE, return_token_scores=True)
    hz.assert_bits_equal(m_b.cpu().numpy(), m_ref, "m_b")
    hz.assert_bits_equal(s_b.cpu().numpy(), s_ref, "S_b")
    # reference layout of the token scores: [H, nb, 16]
    ref_tok = tok_ref.transpose(0, 2, 1, 3).reshape(32, nb, 16)
    hz.assert_bits_equal(tok.cpu().numpy(), ref_tok, "token scores")
    m2, s2 = cb.score_blocks_cuda(
        keys_int8=cc.keys_int8[:, :n], keys_scale=cc.keys_scale[:, :nb], keys_zero_points=cc.keys_zero_points[:, :nb],
        q_all=q, gqa_group=4, q_scale=Q_SCALE)
    assert torch.equal(m2, m_b) and torch.equal(s2, s_b)
    # a shorter prefix of the same arrays
    half = nb // 2
    m3, s3 = cb.score_blocks_cuda(
        keys_int8=cc.keys_int8[:, :half * 16], keys_scale=cc.keys_scale[:, :half],
        keys_zero_points=cc.keys_zero_points[:, :half], q_all=q, gqa_group=4, q_scale=Q_SCALE)
    hz.assert_bits_equal(m3.cpu().numpy(), m_ref[:, :half], "m_b of the prefix")
    with pytest.raises(RuntimeError):
        cb.score_blocks_cuda(keys_int8=cc.keys_int8.cpu(), keys_scale=cc.keys_scale, keys_zero_points=cc.keys_zero_points,
                             q_all=q, gqa_group=4)


def test_fused_score_certify_multihead():
    base, cc, oc = _caches(42, 1024, dtype="float16")
    q = hz.to_dev(base.q, "float16")
    nb = cc.num_quantized_blocks
    m_ref, s_ref, tok_ref = orc.score_blocks(oc, base.q, 4, Q_SCALE)
    m_b, s_b, skip, tok = fsc.fused_score_certify_multihead(
        cc.keys_int8[:, :nb * 16], cc.keys_scale[:, :nb], cc.keys_zero_points[:, :nb], q, cc.correction[:, :nb], 4,
        q_scale=Q_SCALE, block_epsilon=0.0, return_token_scores=True)
    hz.assert_bits_equal(m_b.cpu().numpy(), m_ref, "m_b")
    hz.assert_bits_equal(s_b.cpu().numpy(), s_ref, "S_b")
    assert skip.dtype == torch.bool and not bool(skip.any())
    hz.assert_bits_equal(tok.cpu().numpy(), tok_ref.transpose(0, 2, 1, 3).reshape(32, nb, 16), "token scores")
    with pytest.raises(NotImplementedError):
        fsc.fused_score_certify_multihead(cc.keys_int8, cc.keys_scale, cc.keys_zero_points, q, cc.correction, 4)


# ----------------------------------------------------------------------------- selector helpers

def test_adaptive_topk_and_mass_helpers():
    base, cc, oc = _caches(43, 4096, planted=16)
    m_ref, s_ref, _ = orc.score_blocks(oc, base.q, 4, Q_SCALE)
    m_b = torch.from_numpy(m_ref).cuda()
    s_b = torch.from_numpy(s_ref).cuda()
    sel = orc.adaptive_select(m_ref, s_ref, 0.995, 2, 128, None, 2.0)
    mask, k_star, tail, tau_a, mass, sidx, k2, scum = cb.adaptive_topk_cuda(m_b=m_b, s_b=s_b, tau_cov=0.995, k_min=2,
                                                                           k_max=128)
    assert np.array_equal(mask.cpu().numpy(), sel["topk_mask"])
    assert np.array_equal(k_star.cpu().numpy(), sel["k_star"]) and torch.equal(k_star, k2)
    hz.assert_bits_equal(tail.cpu().numpy(), sel["tail_mass"], "tail mass")
    hz.assert_bits_equal(tau_a.cpu().numpy(), sel["tau_actual"], "tau actual")
    hz.assert_bits_equal(mass.cpu().numpy(), sel["mass_frac"], "mass fractions")
    assert np.array_equal(sidx.cpu().numpy(), sel["sorted_idx"].astype(np.int64))
    hz.assert_bits_equal(scum.cpu().numpy(), sel["sorted_cumsum"], "sorted cumsum")
    res = ca.compute_adaptive_topk_mask(m_b, s_b, tau_cov=0.9, k_min=4, k_max=None, return_mass_frac=True)
    sel2 = orc.adaptive_select(m_ref, s_ref, 0.9, 4, None, None, 2.0)
    assert np.array_equal(res[0].cpu().numpy(), sel2["topk_mask"])
    assert np.array_equal(res[1].cpu().numpy(), sel2["k_star"])
    frac = ca.compute_block_mass_fraction(m_b, s_b)
    hz.assert_bits_equal(frac.cpu().numpy(), sel["mass_frac"], "compute_block_mass_fraction")
    # residual mass and the value-error bounds (torch reductions over the kernel's mass fractions)
    skip = torch.zeros_like(mask)
    rho, mf, topk_idx = ca.compute_tier2_residual_mass(m_b, s_b, skip, top_k=4, return_details=True)
    top4 = np.argsort(-m_ref, axis=1, kind="stable")[:, :4]
    want_rho = 1.0 - np.take_along_axis(sel["mass_frac"].astype(np.float64), top4, axis=1).sum(axis=1)
    np.testing.assert_allclose(rho.cpu().numpy(), np.clip(want_rho, 0, 1), atol=2e-6)
    assert np.array_equal(np.sort(topk_idx.cpu().numpy(), axis=1), np.sort(top4, axis=1))
    eta = cc.values_int4_errors[:, :cc.num_quantized_blocks]
    eta_q = oc.values_int4_errors[:, :oc.num_quantized_blocks][np.arange(32) // 4].astype(np.float64)
    bound = ca.compute_value_error_bound(mf, topk_idx, skip, eta, 4)
    resid = np.ones_like(sel["mass_frac"], dtype=bool)
    np.put_along_axis(resid, top4, False, axis=1)
    np.testing.assert_allclose(bound.cpu().numpy(), (sel["mass_frac"] * eta_q * resid).sum(axis=1), rtol=1e-4)
    int4_mask = torch.from_numpy(~sel["topk_mask"]).cuda()
    bound_m = ca.compute_value_error_bound_for_mask(mf, int4_mask, eta, 4)
    np.testing.assert_allclose(bound_m.cpu().numpy(), (sel["mass_frac"] * eta_q * ~sel["topk_mask"]).sum(axis=1), rtol=1e-4)


def test_fp16_scores_and_delta_helpers():
    base, cc, oc = _caches(44, 2048, extra=5)
    q = hz.to_dev(base.q, DTYPE)
    nq = cc.num_quantized_blocks
    m_ref, _, _ = orc.score_blocks(oc, base.q, 4, Q_SCALE)
    idx = np.stack([np.argsort(-m_ref[h], kind="stable")[:4] for h in range(32)]).astype(np.int32)
    s_ref, l_ref = orc.fp16_block_scores(oc, base.q, idx, 4, Q_SCALE, nq)
    idx_d = torch.from_numpy(idx).cuda()
    s1, l1 = ca.compute_fp16_block_scores(cc, q, idx_d, nq, 4, Q_SCALE, return_log_mass=True)
    hz.assert_bits_equal(s1.cpu().numpy(), s_ref, "compute_fp16_block_scores")
    hz.assert_bits_equal(l1.cpu().numpy(), l_ref, "compute_fp16_block_scores log-mass")
    s2, l2 = f16mod.fp16_block_scores_triton(cc.keys_fp16_gpu, q, idx_d.long(), num_scoring_blocks=nq, gqa_group=4,
                                             block_size=16, q_scale=Q_SCALE)
    assert torch.equal(s1, s2) and torch.equal(l1, l2)
    # with a slot table: the rows of block b sit in slot perm[b] of a scratch array
    perm = torch.randperm(nq, generator=torch.Generator().manual_seed(3)).to(torch.int32).cuda()
    scratch = torch.zeros_like(cc.keys_fp16_gpu)
    scratch.view(8, -1, 16, 128)[:, perm.long()] = cc.keys_fp16_gpu.view(8, -1, 16, 128)[:, :nq]
    s3, l3 = f16mod.fp16_block_scores_triton(scratch, q, idx_d, num_scoring_blocks=nq, gqa_group=4, block_size=16,
                                             q_scale=Q_SCALE, key_block_slots=perm)
    assert torch.equal(s1, s3) and torch.equal(l1, l3)
    d_ref = orc.delta_bound(base.q, oc.sigma_max, 4)
    d = ca.compute_delta_bound(q, cc.keys_scale[:, :nq], 4, Q_SCALE)
    hz.assert_bits_equal(d.cpu().numpy(), d_ref, "compute_delta_bound")
    # tiny comparison helpers
    viol = ca.score_consistency_violations(torch.from_numpy(np.take_along_axis(m_ref, idx, axis=1)).cuda(), s1, d, 0.01)
    assert viol.shape == (32,) and not bool(viol.any())
    dis = ca.detect_ranking_disagreement(s1, s1, 2)
    assert not bool(dis.any())


# ----------------------------------------------------------------------------- Phase 2 entry points

def _phase2_inputs(cc, oc, base, seed=0):
    """Masks of a certified step (from the oracle), then everything hybrid_mixedv_split_k_cuda takes."""
    knobs = dict(gc.PAPER_KNOBS)
    R = orc.layer_step(oc, base.q, 4, exploration_u=np.random.default_rng(seed).random(
        (32, oc.num_quantized_blocks), dtype=np.float32), **knobs)
    return R


def test_hybrid_mixedv_split_k_cuda_with_slot_tables_and_partial_block():
    base, cc, oc = _caches(45, 4096, planted=16, extra=6)
    q = hz.to_dev(base.q, DTYPE)
    R = _phase2_inputs(cc, oc, base)
    nact, nq = cc.active_blocks, cc.num_quantized_blocks
    last_valid = cc.num_tokens - nq * 16
    assert 0 < last_valid < 16
    topk = torch.from_numpy(R["topk_mask_active"]).cuda()
    vmask = torch.from_numpy(R["value_fp16_mask"]).cuda()
    n = nact * 16
    args = dict(keys_int8=cc.keys_int8[:, :n], keys_scale=cc.keys_scale[:, :nact],
                keys_zero_points=cc.keys_zero_points[:, :nact], q_all=q, gqa_group=4, q_scale=Q_SCALE,
                last_block_valid=last_valid, values_int4_packed=cc.values_int4_packed[:, :n],
                values_int4_scales=cc.values_int4_scales[:, :n], values_int4_zeros=cc.values_int4_zeros[:, :n])
    ws = {}
    out = cb.hybrid_mixedv_split_k_cuda(keys_fp16=cc.keys_fp16_gpu, topk_mask=topk, values_fp16_scratch=cc.values_fp16_gpu,
                                        value_fp16_mask=vmask, value_block_slots=None, workspace=ws, **args)
    _rows_close(out.cpu().numpy(), R["phase2_output"], "hybrid_mixedv_split_k_cuda")
    # the same through permuted slot tables (both tiers), reusing the workspace dict
    g = torch.Generator().manual_seed(5)
    kperm = torch.randperm(nact, generator=g).to(torch.int32).cuda()
    vperm = torch.randperm(nact, generator=g).to(torch.int32).cuda()
    kscr, vscr = torch.zeros_like(cc.keys_fp16_gpu), torch.zeros_like(cc.values_fp16_gpu)
    kscr.view(8, -1, 16, 128)[:, kperm.long()] = cc.keys_fp16_gpu.view(8, -1, 16, 128)[:, :nact]
    vscr.view(8, -1, 16, 128)[:, vperm.long()] = cc.values_fp16_gpu.view(8, -1, 16, 128)[:, :nact]
    out2 = cb.hybrid_mixedv_split_k_cuda(keys_fp16=kscr, key_block_slots=kperm, topk_mask=topk, values_fp16_scratch=vscr,
                                         value_fp16_mask=vmask, value_block_slots=vperm, workspace=ws, **args)
    assert torch.equal(out, out2), "slot tables must not change a bit of the result"
    assert "mixedv_output" in ws and "cqa_tickets" in ws
    # profile counters
    cb.reset_native_profile()
    cb.enable_native_profile(True)
    cb.hybrid_mixedv_split_k_cuda(keys_fp16=cc.keys_fp16_gpu, topk_mask=topk, values_fp16_scratch=cc.values_fp16_gpu,
                                  value_fp16_mask=vmask, value_block_slots=None, workspace=ws, **args)
    cb.enable_native_profile(False)
    prof = cb.native_profile_summary()
    assert prof["calls"] == 1 and prof["total_ms"] > 0
    assert cb.certified_blackwell_available()


def test_hybrid_without_int4_values_reads_fp16_everywhere():
    """values_int4_packed=None: every block takes its values from the FP16 tensor (the FP16-value branch of the
    attend kernel)."""
    base, cc, oc = _caches(46, 2048, planted=8)
    q = hz.to_dev(base.q, DTYPE)
    R = _phase2_inputs(cc, oc, base)
    nb = cc.num_quantized_blocks
    topk = R["topk_mask_active"]
    ones = np.ones_like(topk)
    ref, _ = orc.attend_mixed(oc, base.q, 4, Q_SCALE, topk, ones, nb, 16)
    n = nb * 16
    out = cb.hybrid_mixedv_split_k_cuda(
        keys_int8=cc.keys_int8[:, :n], keys_scale=cc.keys_scale[:, :nb], keys_zero_points=cc.keys_zero_points[:, :nb],
        keys_fp16=cc.keys_fp16_gpu, topk_mask=torch.from_numpy(topk).cuda(), values_int4_packed=None,
        values_int4_scales=None, values_int4_zeros=None, values_fp16_scratch=cc.values_fp16_gpu,
        value_fp16_mask=torch.from_numpy(ones).cuda(), value_block_slots=None, q_all=q, gqa_group=4, q_scale=Q_SCALE)
    _rows_close(out.cpu().numpy(), ref, "FP16 values everywhere")


def test_selective_attend_entry_points():
    """The eight selective_attend_multihead* names against the oracle's Phase 2 with the masks each one implies."""
    base, cc, oc = _caches(47, 2048, planted=8)
    q = hz.to_dev(base.q, DTYPE)
    R = _phase2_inputs(cc, oc, base)
    nb = cc.num_quantized_blocks
    n = nb * 16
    topk_np, vm_np = R["topk_mask_active"], R["value_fp16_mask"]
    topk, vm = torch.from_numpy(topk_np).cuda(), torch.from_numpy(vm_np).cuda()
    zeros, ones = np.zeros_like(topk_np), np.ones_like(topk_np)
    k8, ks, kz = cc.keys_int8[:, :n], cc.keys_scale[:, :nb], cc.keys_zero_points[:, :nb]
    v4 = (cc.values_int4_packed[:, :n], cc.values_int4_scales[:, :n], cc.values_int4_zeros[:, :n])
    kf, vf = cc.keys_fp16_gpu[:, :n], cc.values_fp16_gpu[:, :n]
    no_skip = torch.zeros(32, nb, dtype=torch.int32, device="cuda")

    def ref(topk_m, val_m):
        return orc.attend_mixed(oc, base.q, 4, Q_SCALE, topk_m, val_m, nb, 16)[0]

    common = dict(gqa_group=4, q_scale=Q_SCALE)
    out = sat.selective_attend_multihead_hybrid_mixedv_split_k(k8, ks, kz, kf, topk, *v4, vf, vm, None, q,
                                                               skip_mask_i32=no_skip, last_block_valid=16, **common)
    _rows_close(out.cpu().numpy(), ref(topk_np, vm_np), "hybrid_mixedv_split_k")
    out = sat.selective_attend_multihead_hybrid_mixedv(k8, ks, kz, kf, topk, *v4, vf, vm, None, q, **common)
    _rows_close(out.cpu().numpy(), ref(topk_np, vm_np), "hybrid_mixedv")
    out = sat.selective_attend_multihead_hybrid_int4v(k8, ks, kz, kf, topk, *v4, q, **common)
    _rows_close(out.cpu().numpy(), ref(topk_np, zeros), "hybrid_int4v")
    out = sat.selective_attend_multihead_hybrid_split_k(k8, ks, kz, kf, topk, vf, q, **common)
    _rows_close(out.cpu().numpy(), ref(topk_np, ones), "hybrid_split_k")
    out = sat.selective_attend_multihead_hybrid(k8, ks, kz, kf, topk, vf, q, **common)
    _rows_close(out.cpu().numpy(), ref(topk_np, ones), "hybrid")
    out = sat.selective_attend_multihead_int8k_int4v(k8, ks, kz, *v4, q, **common)
    _rows_close(out.cpu().numpy(), ref(zeros, zeros), "int8k_int4v")
    out = sat.selective_attend_multihead_int8(k8, ks, kz, vf, q, **common)
    _rows_close(out.cpu().numpy(), ref(zeros, ones), "int8")
    with pytest.raises(NotImplementedError):
        sat.selective_attend_multihead(k8, ks, kz)
    with pytest.raises(NotImplementedError):
        sat.selective_attend_multihead_int8(k8, ks, kz, vf, q, skip_mask_i32=torch.ones_like(no_skip), **common)


def test_attend_refuses_certificate_without_dense_scratch():
    """A certificate can flag heads whose rows only the dense pool writes; without dense scratch the call is
    refused instead of returning stale rows for them."""
    base, cc, oc = _caches(48, 1024)
    q = hz.to_dev(base.q, DTYPE)
    ca.certified_attention_layer(cc, q, 4, None, False, **gc.PAPER_KNOBS)
    ws = cc._certified_workspace["cqa_ws"]
    w = _lib.CqaWorkspace.from_buffer_copy(bytes(ws.fill_struct(cc.active_blocks)))
    w.dense_splits = 0
    rc = _lib.lib().cqa_attend(C.byref(cc._desc(4)), C.byref(w), q.data_ptr(), _lib.CQA_BF16, cc.num_quantized_blocks,
                               cc.active_blocks, cc.num_tokens, 16, Q_SCALE, None)
    assert rc == -1 and b"dense-recompute scratch" in _lib.lib().cqa_last_error()
    w.cert = None                                  # detached certificate: the mixed result for every head
    rc = _lib.lib().cqa_attend(C.byref(cc._desc(4)), C.byref(w), q.data_ptr(), _lib.CQA_BF16, cc.num_quantized_blocks,
                               cc.active_blocks, cc.num_tokens, 16, Q_SCALE, None)
    assert rc == 0
    torch.cuda.synchronize()


def test_layer_step_rejects_bad_sizes_before_launching():
    """cqa_layer_step validates every size before its first launch (a short leading dimension would make the score
    kernel write past the rows)."""
    base, cc, oc = _caches(49, 1024)
    q = hz.to_dev(base.q, DTYPE)
    ca.certified_attention_layer(cc, q, 4, None, False, **gc.PAPER_KNOBS)
    ws = cc._certified_workspace["cqa_ws"]
    guard = ws.m_b.clone()
    knobs = _knobs_struct()
    L = _lib.lib()
    nq = cc.num_quantized_blocks
    w = _lib.CqaWorkspace.from_buffer_copy(bytes(ws.fill_struct(cc.active_blocks)))
    w.ld = nq - 1
    rc = L.cqa_layer_step(C.byref(cc._desc(4)), C.byref(knobs), C.byref(w), q.data_ptr(), _lib.CQA_BF16,
                          cc.num_tokens, nq, None, 0, None)
    assert rc == -1
    rc = L.cqa_layer_step(C.byref(cc._desc(4)), C.byref(knobs), C.byref(ws.fill_struct(cc.active_blocks)), q.data_ptr(), 7,
                          cc.num_tokens, nq, None, 0, None)
    assert rc == -1 and b"dtype" in L.cqa_last_error()
    d = cc._desc_copy(4)
    d.max_blocks = nq - 1
    rc = L.cqa_layer_step(C.byref(d), C.byref(knobs), C.byref(ws.fill_struct(cc.active_blocks)), q.data_ptr(),
                          _lib.CQA_BF16, cc.num_tokens, nq, None, 0, None)
    assert rc == -1
    torch.cuda.synchronize()
    assert torch.equal(guard, ws.m_b), "a refused call must not have launched anything"


# ----------------------------------------------------------------------------- dense helpers

def test_dense_recompute_and_sdpa_helpers():
    base, cc, oc = _caches(50, 2048, extra=3)
    q = hz.to_dev(base.q, DTYPE)
    heads = np.array([1, 7, 8, 30], dtype=np.int32)
    ref = orc.dense_attend(oc, base.q, heads, 4, Q_SCALE)
    out = torch.full((32, 128), 7.0, dtype=torch.float32, device="cuda")
    out2, kb, kn, vb, vn = ca.recompute_heads_dense_fp16(cc, q, out, torch.from_numpy(heads).cuda().long(), 4, Q_SCALE)
    assert out2 is out and (kb, kn, vb, vn) == (0, 0, 0, 0)
    got = out.cpu().numpy()
    _rows_close(got[heads], ref, "recompute_heads_dense_fp16")
    untouched = np.setdiff1d(np.arange(32), heads)
    assert (got[untouched] == 7.0).all(), "unlisted heads keep their rows"
    same, *_ = ca.recompute_heads_dense_fp16(cc, q, out, torch.zeros(0, dtype=torch.long, device="cuda"), 4, Q_SCALE)
    assert same is out
    full = ca.sdpa_attend_with_skip(cc, q, torch.zeros(32, cc.active_blocks, dtype=torch.bool, device="cuda"), 4, Q_SCALE)
    ref_all = orc.dense_attend(oc, base.q, np.arange(32, dtype=np.int32), 4, Q_SCALE)
    _rows_close(full.cpu().numpy(), ref_all, "sdpa_attend_with_skip")
    with pytest.raises(NotImplementedError):
        ca.sdpa_attend_with_skip(cc, q, torch.ones(32, cc.active_blocks, dtype=torch.bool, device="cuda"), 4, Q_SCALE)


# ----------------------------------------------------------------------------- INT4 quantiser module

def test_int4_group_quantise_module():
    rng = np.random.default_rng(51)
    x = rng.standard_normal((2, 64, 128)).astype(np.float32)
    xd = torch.from_numpy(x).to(torch.bfloat16).cuda()
    xf = xd.float().cpu().numpy()
    r = i4.quantise_int4_grouped(xd.reshape(-1, 128))
    # the value tier quantises float16 copies of the values (tiered_kv_cache.py:303); the stand-alone quantiser
    # takes its input as it is
    o = orc.quant_values_int4(xf.reshape(-1, 128))
    rel_ref = o["per_token_error"]
    assert np.array_equal(r["data_packed"].cpu().numpy(), o["data_packed"])
    hz.assert_bits_equal(r["scales"].cpu().numpy(), o["scales"], "INT4 scales")
    hz.assert_bits_equal(r["zeros"].cpu().numpy(), o["zeros"], "INT4 zeros")
    hz.assert_bits_equal(r["per_token_error"].cpu().numpy(), rel_ref, "per-token relative error")
    hz.assert_bits_equal(r["per_token_abs_error"].cpu().numpy(), o["per_token_abs_error"], "per-token absolute error")
    assert float(r["error_bound"]) == float(rel_ref.max())
    blk = i4.quantise_int4_grouped_block(xd)
    assert blk["data_packed"].shape == (2, 64, 64) and blk["scales"].shape == (2, 64, 8)
    hz.assert_bits_equal(blk["error_bounds"].cpu().numpy(), rel_ref.reshape(2, 4, 16).max(axis=2), "block error bounds")
    deq = i4.dequantise_int4_grouped(r["data_packed"], r["scales"], r["zeros"])
    assert deq.shape == (128, 128) and deq.dtype == torch.float16
    # dequantised values stay within one quantisation step of the input
    step = r["scales"].float().repeat_interleave(16, dim=-1)
    assert bool(((deq.float() - xd.reshape(-1, 128).float()).abs() <= 0.51 * step + 2e-2).all())
    with pytest.raises(RuntimeError):
        i4.quantise_int4_grouped(xd.reshape(-1, 128).cpu())


# ----------------------------------------------------------------------------- FP16-value cache end to end

class _Layer:
    def __init__(self, k, v):
        self.keys, self.values = k, v


class _PastKV:
    def __init__(self, layers):
        self.layers = layers


@pytest.mark.parametrize("dtype", ["bfloat16", "float16"])
def test_fp16_value_cache_end_to_end(dtype):
    """from_fp16_cache + create_tiered_cache_from_model + certified_attention_layer on a cache without INT4 values
    (the reference's smoke test runs both value modes): selections and flags bit-exact, every block read from the
    model-dtype values, v_format "fp16"."""
    n = 2048 + 11
    base = synth.make_layer_inputs(52, n + 24, dtype=dtype, n_planted_blocks=8)
    kd, vd = hz.to_dev(base.k[:, :n], dtype), hz.to_dev(base.v[:, :n], dtype)
    past = _PastKV([_Layer(kd.unsqueeze(0), vd.unsqueeze(0))])
    caches = create_tiered_cache_from_model(past, [0], max_new_tokens=64)
    cc = caches[0]
    assert cc.values_int4_packed is None and cc.values_fp16 is not None and cc.num_tokens == n
    assert int((cc.keys_int8[:, n:((n + 15) // 16) * 16] == -127).all())
    oc = hz.make_oracle_cache(base.k[:, :2048], base.v[:, :2048], dtype, 64)
    for t in range(2048, n):
        oc.append_token(base.k[:, t:t + 1], base.v[:, t:t + 1])
    direct = TieredKeyCacheLayer.from_fp16_cache(kd[:, :2048].contiguous(), vd[:, :2048].contiguous(), max_new_tokens=64)
    assert torch.equal(direct.keys_int8[:, :2048], cc.keys_int8[:, :2048])
    knobs = dict(gc.PAPER_KNOBS)
    rng = np.random.default_rng(52)
    for step in range(24):
        q, kn, vn = synth.decode_step_inputs(base, step, dtype=dtype)
        cc.append_token(hz.to_dev(kn, dtype), hz.to_dev(vn, dtype))
        oc.append_token(kn, vn)
        if step % 6 != 5:
            continue
        u = rng.random((32, oc.num_quantized_blocks), dtype=np.float32)
        R = orc.layer_step(oc, q, 4, exploration_u=u, fp16_values=True, **knobs)
        out, stats = hz.cuda_step(cc, q, dtype, 4, knobs, u)
        hz.compare_step(cc, R, out, f"fp16-value step {step}", check_value=False)
        ws = cc._certified_workspace["cqa_ws"]
        assert bool((ws.value_mask[:, :cc.active_blocks] == 1).all())
        assert stats["v_format"] == "fp16" and stats["rung2_fired"] is False and "eta_int4" not in stats
    nq, nt = oc.num_quantized_blocks, oc.num_tokens
    hz.assert_bits_equal(cc.keys_int8[:, :nq * 16].cpu().numpy(), oc.keys_int8[:, :nq * 16], "keys_int8")
    hz.assert_bits_equal(cc.values_fp16[:, :nt].float().cpu().numpy(), oc.values_t2[:, :nt], "model-dtype values")
    # the INT4 factory on the same prompt: ragged tail through append_token, poison rows set
    c4 = create_tiered_cache_int4v_from_model(past, [0], max_new_tokens=64)[0]
    assert c4.values_int4_packed is not None and c4.num_tokens == n and c4.num_quantized_blocks == n // 16


@pytest.mark.parametrize("dtype,defer", [("bfloat16", None), ("float32", False)])
def test_whole_model_prefill_encode(dtype, defer):
    """create_tiered_cache_int4v_from_model: three layers with ragged lengths go through ONE library call (complete
    blocks quantised from the strided [1, KV, seq, 128] tensors, the remainder appended by one launch per layer);
    every array equals the oracle cache built block-wise + token by token, and decoding continues from there."""
    lens = [16 * 37 + 11, 16 * 37 + 11, 16 * 37 + 11]
    layers, bases = [], []
    for i, n in enumerate(lens):
        base = synth.make_layer_inputs(70 + i, n + 40, dtype=dtype, n_planted_blocks=4)
        bases.append(base)
        # a [1, KV, seq + 40, 128] buffer of which the first n rows are the prompt: non-trivial KV stride
        kfull, vfull = hz.to_dev(base.k, dtype).unsqueeze(0), hz.to_dev(base.v, dtype).unsqueeze(0)
        layers.append(_Layer(kfull[:, :, :n], vfull[:, :, :n]))
    before = _lib.lib().cqa_launch_count(0)
    caches = create_tiered_cache_int4v_from_model(_PastKV(layers), [0, 1, 2], max_new_tokens=48,
                                                  defer_int4_append_quantization=defer)
    launched = _lib.lib().cqa_launch_count(0) - before
    assert launched == 2 * len(lens), f"{launched} launches for {len(lens)} layers"
    for i, n in enumerate(lens):
        cc, base = caches[i], bases[i]
        al = (n // 16) * 16
        oc = hz.make_oracle_cache(base.k[:, :al], base.v[:, :al], dtype, 48 + n - al, defer=cc._defer_int4_flag())
        for t in range(al, n):
            oc.append_token(base.k[:, t:t + 1], base.v[:, t:t + 1])
        hz.compare_caches(cc, oc, f"layer {i} after the prefill encode")
        for step in range(8):     # crosses the completion of the ragged block
            q, kn, vn = synth.decode_step_inputs(base, step, dtype=dtype)
            cc.append_token(hz.to_dev(kn, dtype), hz.to_dev(vn, dtype))
            oc.append_token(kn, vn)
        hz.compare_caches(cc, oc, f"layer {i} after 8 appends")


def test_prefill_encode_refuses_bad_items():
    base = synth.make_layer_inputs(75, 256, kv_heads=2, dtype="bfloat16")
    cc = hz.make_cuda_cache(base.k, base.v, "bfloat16", 16)
    it = (_lib.CqaPrefillItem * 1)()
    it[0].cache = cc._desc()
    it[0].k_src, it[0].v_src = cc.keys_fp16_gpu.data_ptr(), cc.values_fp16_gpu.data_ptr()
    it[0].src_rows, it[0].n_tokens = 256, 100000          # more tokens than the cache holds
    before = _lib.lib().cqa_launch_count(0)
    rc = _lib.lib().cqa_prefill_encode(it, 1, _lib.CQA_BF16, None)
    assert rc != 0 and _lib.lib().cqa_launch_count(0) == before


# ----------------------------------------------------------------------------- page-in module and residency API

def test_cuda_pagein_module():
    assert pg.cuda_pagein_available() and pg.cuda_pagein_enabled()
    rng = torch.Generator().manual_seed(53)
    kv, nblk, cap = 4, 40, 12
    src = torch.randn(kv, nblk * 16, 128, generator=rng).to(torch.bfloat16).pin_memory()
    dst = torch.zeros(kv, cap * 16, 128, dtype=torch.bfloat16, device="cuda")
    table = torch.full((nblk,), -1, dtype=torch.int32, device="cuda")
    table[3] = 5                                         # block 3 sits in slot 5 and gets evicted below
    loaded = torch.tensor([7, 39, 0], dtype=torch.int64).pin_memory()
    slots = torch.tensor([5, 0, 11], dtype=torch.int32).pin_memory()
    evicted = torch.tensor([3], dtype=torch.int64).pin_memory()
    lb = torch.zeros(8, dtype=torch.int64, device="cuda")
    ls = torch.zeros(8, dtype=torch.int32, device="cuda")
    ev = torch.zeros(8, dtype=torch.int64, device="cuda")
    active = 39 * 16 + 9                                 # block 39 is partial: 9 valid rows
    nbytes = pg.page_in_fp16_blocks_cuda(src_cpu=src, dst_gpu=dst, loaded_blocks_cpu=loaded, loaded_slots_cpu=slots,
                                         evicted_blocks_cpu=evicted, loaded_blocks_gpu=lb, loaded_slots_gpu=ls,
                                         evicted_blocks_gpu=ev, slot_table_gpu=table, block_size=16, active_tokens=active)
    torch.cuda.synchronize()
    assert nbytes == kv * (16 + 9 + 16) * 256
    t = table.cpu().numpy()
    assert t[3] == -1 and t[7] == 5 and t[39] == 0 and t[0] == 11 and (np.delete(t, [0, 3, 7, 39]) == -1).all()
    d = dst.cpu()
    assert torch.equal(d[:, 5 * 16: 6 * 16], src[:, 7 * 16: 8 * 16])
    assert torch.equal(d[:, 11 * 16: 12 * 16], src[:, 0:16])
    assert torch.equal(d[:, 0:9], src[:, 39 * 16: 39 * 16 + 9]) and bool((d[:, 9:16] == 0).all())
    # packed variant: same result
    dst2 = torch.zeros_like(dst)
    table2 = torch.full((nblk,), -1, dtype=torch.int32, device="cuda")
    pg.page_in_fp16_blocks_packed_cuda(src_cpu=src, dst_gpu=dst2, stage_cpu=None, stage_gpu=None, loaded_blocks_cpu=loaded,
                                       loaded_slots_cpu=slots, evicted_blocks_cpu=torch.zeros(0, dtype=torch.int64),
                                       loaded_blocks_gpu=lb, loaded_slots_gpu=ls, evicted_blocks_gpu=ev,
                                       slot_table_gpu=table2, block_size=16, active_tokens=active)
    assert torch.equal(dst2, dst)
    # by slots: every block with a slot is copied
    dst3 = torch.zeros_like(dst)
    pg.page_in_fp16_blocks_by_slots_cuda(src_cpu=src, dst_gpu=dst3, block_slots_gpu=table, block_size=16,
                                         active_tokens=active, n_blocks=nblk)
    assert torch.equal(dst3, dst)
    with pytest.raises(ValueError):
        pg.page_in_fp16_blocks_by_slots_cuda(src_cpu=src.clone(), dst_gpu=dst3, block_slots_gpu=table, block_size=16,
                                             active_tokens=active, n_blocks=nblk)   # pageable host memory


def test_residency_requests_and_step_stats():
    """ensure_fp16_{keys,values}_resident on a bounded hot tier, and the per-step residency keys of the stats dict
    (filled from the device counters)."""
    dtype = DTYPE
    base = synth.make_layer_inputs(54, 4096 + 8, dtype=dtype, n_planted_blocks=8)
    kd, vd = hz.to_dev(base.k[:, :4096], dtype), hz.to_dev(base.v[:, :4096], dtype)
    hot = TieredKeyCacheLayer.from_fp16_cache_int4v(kd, vd, max_new_tokens=64, max_pagein_blocks=32,
                                                    fp16_key_cache_capacity=64, fp16_value_cache_capacity=64)
    full = hz.make_cuda_cache(base.k[:, :4096], base.v[:, :4096], dtype, 64, defer=False)
    assert full.ensure_fp16_keys_resident([1, 2, 3]) == (0, 0, 0, 0)
    blk = 8 * 16 * 128 * 2
    h, m, b, e = hot.ensure_fp16_keys_resident([5, 9, 9, 200])
    assert (h, m, b, e) == (0, 3, 3 * blk, 0)
    h, m, b, e = hot.ensure_fp16_keys_resident(torch.tensor([5, 9, 17]))
    assert (h, m, b, e) == (2, 1, blk, 0)
    h, m, b, e = hot.ensure_fp16_values_resident_batched([0, 1])
    assert (h, m, b, e) == (0, 2, 2 * blk, 0)
    torch.cuda.synchronize()
    sl = hot._hot["key_slots"].cpu().numpy()
    for bid in (5, 9, 17, 200):
        s = sl[bid]
        assert s >= 0 and torch.equal(hot.keys_fp16_gpu[:, s * 16:(s + 1) * 16].cpu(), hot.keys_fp16_cpu[:, bid * 16:(bid + 1) * 16])
    knobs = dict(gc.PAPER_KNOBS)
    seen = []
    for step in range(8):
        q, kn, vn = synth.decode_step_inputs(base, step, dtype=dtype)
        hot.append_token(hz.to_dev(kn, dtype), hz.to_dev(vn, dtype))
        _, stats = hz.cuda_step(hot, q, dtype, 4, knobs, None)
        for key in ("fp16_cache_capacity_blocks", "fp16_cache_resident_blocks", "fp16_cache_hits_step",
                    "fp16_cache_misses_step", "fp16_cache_evictions_step", "fp16_cache_needed_blocks_step",
                    "fp16_cache_hit_rate_step", "fp16_value_cache_hits_step", "fp16_value_cache_misses_step",
                    "fp16_value_cache_hit_rate_step", "h2d_key_bytes", "h2d_total_bytes"):
            assert key in stats, key
        assert stats["fp16_cache_needed_blocks_step"] == stats["fp16_cache_hits_step"] + stats["fp16_cache_misses_step"]
        assert 0 < stats["fp16_cache_resident_blocks"] <= 64
        assert stats["h2d_key_bytes"] % blk == 0
        seen.append((stats["fp16_cache_hits_step"], stats["fp16_cache_misses_step"]))
    assert seen[0][1] > 0, "the first step must miss"
    assert seen[-1][0] > 0, "later steps must hit what the earlier ones paged in"
    tot = hot.hot_tier_counters()
    assert tot["key_hits"] >= sum(s[0] for s in seen)


# ----------------------------------------------------------------------------- bounded device-side wait

def test_bounded_wait_runs_out_and_reports():
    """A kernel that waits on a flag nobody sets gives up after its spin limit, records 100 + i (i = the source it
    waited for) in the status word and finishes; the context stays usable.  One GPU: the flag word is simply never
    written."""
    base, cc, oc = _caches(55, 1024)
    q = hz.to_dev(base.q, DTYPE)
    ca.certified_attention_layer(cc, q, 4, None, False, **gc.PAPER_KNOBS)     # fills m_b / S_b / masks
    ws = cc._certified_workspace["cqa_ws"]
    flags = torch.zeros(4, dtype=torch.int32, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    flags[0] = 1                                                  # source 0 has arrived, source 1 is skipped (self)
    w = _lib.CqaWorkspace.from_buffer_copy(bytes(ws.fill_struct(cc.active_blocks)))
    w.wait_flags, w.wait_n, w.wait_skip, w.wait_value = flags.data_ptr(), 3, 1, 1
    w.wait_spins = 2000                                           # about half a millisecond instead of half a second
    w.wait_status = status.data_ptr()
    knobs = _knobs_struct()
    L = _lib.lib()
    # the selection without any wait, for comparison
    plain = _lib.CqaWorkspace.from_buffer_copy(bytes(ws.fill_struct(cc.active_blocks)))
    assert L.cqa_select(C.byref(cc._desc(4)), C.byref(knobs), C.byref(plain), cc.num_quantized_blocks, cc.active_blocks,
                        None, 0, _lib.current_stream(q.device)) == 0
    torch.cuda.synchronize()
    ref_mask = ws.topk_mask.clone()
    ws.topk_mask.zero_()
    t0 = torch.cuda.Event(enable_timing=True)
    t1 = torch.cuda.Event(enable_timing=True)
    t0.record()
    rc = L.cqa_select(C.byref(cc._desc(4)), C.byref(knobs), C.byref(w), cc.num_quantized_blocks, cc.active_blocks, None, 0,
                      _lib.current_stream(q.device))
    t1.record()
    assert rc == 0
    torch.cuda.synchronize()
    assert int(status.item()) == 102, "the wait for source 2 must have run out"
    assert t0.elapsed_time(t1) < 1000.0
    # the kernel carried on after the timeout and the context is intact: the next call works and agrees
    status.zero_()
    flags[2] = 1
    rc = L.cqa_select(C.byref(cc._desc(4)), C.byref(knobs), C.byref(w), cc.num_quantized_blocks, cc.active_blocks, None, 0,
                      _lib.current_stream(q.device))
    assert rc == 0
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    assert torch.equal(ws.topk_mask, ref_mask), "the selection after a wait equals the selection without one"
    out2, _ = ca.certified_attention_layer(cc, q, 4, None, False, **dict(gc.PAPER_KNOBS, exploration_rate=0.0))
    torch.cuda.synchronize()
    assert bool(torch.isfinite(out2).all())


def test_no_staged_copy_wait_ran_out():
    """After everything above, the library's counter of bounded waits on staged (bulk-copy) tiles that ran out is
    zero: every tile of every score and attend launch arrived."""
    n = C.c_int(-1)
    with torch.cuda.device(0):
        assert _lib.lib().cqa_wait_timeouts(C.byref(n), 0) == 0
    assert n.value == 0


# ----------------------------------------------------------------------------- batches

def test_batched_layer_step_equals_single_sequence_runs():
    """cqa_layer_step_batched: several sequences of different lengths in one launch of each kernel.  Every
    sequence's masks, certificate, appended bytes and output rows equal its own one-sequence run bit for bit (same
    split count), over steps that cross a block completion; an oracle check pins one of them."""
    dtype = DTYPE
    lengths = [1024 + 3, 4096, 2048 + 15, 512]
    knobs = dict(gc.PAPER_KNOBS, exploration_rate=0.0)
    bases = [synth.make_layer_inputs(60 + i, n + 24, dtype=dtype, n_planted_blocks=4) for i, n in enumerate(lengths)]

    def build(i):
        n = lengths[i]
        al = (n // 16) * 16
        c = hz.make_cuda_cache(bases[i].k[:, :al], bases[i].v[:, :al], dtype, 64)
        for t in range(al, n):
            c.append_token(hz.to_dev(bases[i].k[:, t:t + 1], dtype), hz.to_dev(bases[i].v[:, t:t + 1], dtype))
        return c

    solo = [build(i) for i in range(4)]
    batch = [build(i) for i in range(4)]
    oc = hz.make_oracle_cache(bases[1].k[:, :4096], bases[1].v[:, :4096], dtype, 64)
    for step in range(20):
        qs, ks, vs = [], [], []
        for i in range(4):
            q, kn, vn = synth.decode_step_inputs(bases[i], step, dtype=dtype)
            qs.append(q), ks.append(kn.reshape(8, 128)), vs.append(vn.reshape(8, 128))
        oc.append_token(ks[1].reshape(8, 1, 128), vs[1].reshape(8, 1, 128))
        qd = hz.to_dev(np.stack(qs), dtype)
        kd, vd = hz.to_dev(np.stack(ks), dtype), hz.to_dev(np.stack(vs), dtype)
        out_b = ca.certified_attention_batch(batch, qd, 4, None, new_keys=kd, new_values=vd, num_splits=6, **knobs)
        torch.cuda.synchronize()
        for i in range(4):
            solo[i].append_token(kd[i].reshape(8, 1, 128), vd[i].reshape(8, 1, 128))
            ws = solo[i]._certified_workspace.get("cqa_ws") or ca._workspace(solo[i], 32, 4, qd.device)
            # the same split count as the batch call used for this sequence
            nact = solo[i].active_blocks
            want_ns = max(1, min(6, max(1, min(ws.num_splits, (nact + 7) // 8)), nact))
            keep = ws.num_splits
            ws.num_splits = want_ns
            out_s, _ = ca.certified_attention_layer(solo[i], qd[i], 4, None, False, **knobs)
            torch.cuda.synchronize()
            ws.num_splits = keep
            assert torch.equal(out_b[i], out_s), f"step {step} sequence {i}: output rows differ"
            wb = batch[i]._certified_workspace["cqa_ws"]
            for name in ("topk_mask", "value_mask", "explore_mask", "m_b", "s_b", "mass_frac"):
                assert torch.equal(getattr(wb, name)[:, :nact], getattr(ws, name)[:, :nact]), f"{name} seq {i} step {step}"
            cb_, fb = wb.read_cert()
            cs_, fs = ws.read_cert()
            assert fb[:5] == fs[:5]
            for key in ("k_star", "rung3", "dense", "value_promoted_blocks", "delta", "e_val", "tail_mass"):
                assert np.array_equal(np.asarray(cb_[key]).view(np.uint8), np.asarray(cs_[key]).view(np.uint8)), key
            assert batch[i].num_tokens == solo[i].num_tokens
        if step in (0, 15, 19):
            R = orc.layer_step(oc, qs[1], 4, exploration_u=None, **knobs)
            hz.compare_step(batch[1], R, out_b[1].cpu().numpy(), f"batched sequence 1 step {step}")
    for i in range(4):
        for name in ("keys_int8", "keys_scale", "values_int4_packed", "values_int4_errors", "keys_fp16_gpu"):
            assert torch.equal(getattr(batch[i], name), getattr(solo[i], name)), f"{name} of sequence {i}"
    # attend only (no append) on the same caches
    prev = out_b.clone()
    out_n = ca.certified_attention_batch(batch, qd, 4, None, num_splits=6, **knobs)
    torch.cuda.synchronize()
    assert torch.equal(out_n, prev)
