"""Native certified-attention kernels behind the reference's backend API.

Same function names and argument meaning as the reference's
`dotcache/backends/certified_blackwell.py` (score_blocks_cuda:64-87,
adaptive_topk_cuda:90-107, hybrid_mixedv_split_k_cuda:138-224,
reset_native_profile:43-46, native_profile_summary:49-61), implemented over
libcqa_b200.so for sm_100a.  Tensor arguments may be slices of larger
buffers (`cache.keys_int8[:, :n]`): the KV-head stride is passed to the
kernels, nothing is copied.
"""
from __future__ import annotations

import ctypes as C
from typing import Any

import torch

from cqa_b200 import _lib

_PROFILE = {"calls": 0, "partial_ms_total": 0.0, "reduce_ms_total": 0.0}
_PROFILE_ENABLED = False


def certified_blackwell_available() -> bool:
    """True when a CUDA device of compute capability 10.x is present and the library loads."""
    try:
        if not torch.cuda.is_available() or torch.cuda.get_device_capability()[0] != 10:
            return False
        _lib.lib()
    except Exception:
        return False
    return True


def reset_native_profile() -> None:
    _PROFILE.update(calls=0, partial_ms_total=0.0, reduce_ms_total=0.0)


def enable_native_profile(on: bool = True) -> None:
    """Time every hybrid_mixedv_split_k_cuda call with CUDA events (synchronises)."""
    global _PROFILE_ENABLED
    _PROFILE_ENABLED = bool(on)


def native_profile_summary() -> dict:
    calls = int(_PROFILE["calls"])
    p, r = float(_PROFILE["partial_ms_total"]), float(_PROFILE["reduce_ms_total"])
    return {
        "calls": calls, "partial_ms_total": p, "reduce_ms_total": r, "total_ms": p + r,
        "partial_ms_per_call": p / calls if calls else 0.0, "reduce_ms_per_call": r / calls if calls else 0.0,
    }


def _rows_view(t: torch.Tensor, width: int, what: str) -> tuple[torch.Tensor, int]:
    """Return (tensor, kv stride in rows) for a [kv, rows, width] view without copying when possible."""
    if t.dim() != 3 or t.shape[2] != width:
        raise ValueError(f"{what}: expected [kv, rows, {width}], got {tuple(t.shape)}")
    if t.stride(2) != 1 or t.stride(1) != width or (t.shape[0] > 1 and t.stride(0) % width != 0):
        t = t.contiguous()
    kv_stride = t.stride(0) // width if t.shape[0] > 1 else max(int(t.shape[1]), 1)
    return t, int(kv_stride)


def _same_stride(pairs, what):
    strides = {s for _, s in pairs}
    if len(strides) == 1:
        return [t for t, _ in pairs], strides.pop()
    ts = [t.contiguous() for t, _ in pairs]
    return ts, int(ts[0].shape[1])


def score_blocks_cuda(*, keys_int8: Any, keys_scale: Any, keys_zero_points: Any, q_all: Any, gqa_group: int,
                      block_size: int = 16, q_scale: float = 1.0, blocks_per_chunk: int | None = None,
                      return_token_scores: bool = False):
    """Phase-1 scores.  Returns (m_b, S_b) [H, nb] float32 (plus token scores
    [H, nb, 16] when asked).  `blocks_per_chunk` is accepted and ignored (the
    grid is sized from the SM count)."""
    if block_size != 16:
        raise ValueError("block_size must be 16")
    if not keys_int8.is_cuda:
        raise RuntimeError("score_blocks_cuda needs CUDA tensors; there is no CPU fallback")
    k, kstride = _rows_view(keys_int8, 128, "keys_int8")
    (s, z), sstride = _same_stride([_rows_view(keys_scale, 128, "keys_scale"),
                                    _rows_view(keys_zero_points, 128, "keys_zero_points")], "scales")
    kv, n, _ = k.shape
    nb = n // 16
    H = int(q_all.shape[0])
    G = int(gqa_group)
    if H != kv * G:
        raise ValueError("q_all heads must equal kv_heads * gqa_group")
    dev = k.device
    m_b = torch.empty(H, nb, dtype=torch.float32, device=dev)
    s_b = torch.empty(H, nb, dtype=torch.float32, device=dev)
    tok = torch.empty(kv, nb, G, 16, dtype=torch.float32, device=dev) if return_token_scores else None
    if nb:
        d = _lib.CqaCache()
        d.kv_heads, d.gqa_group, d.t2_dtype = kv, G, _lib.CQA_F16
        d.cap_tokens, d.max_blocks = kstride, sstride
        d.keys_int8, d.keys_scale, d.keys_zero_points = k.data_ptr(), s.data_ptr(), z.data_ptr()
        q = q_all.contiguous()
        with torch.cuda.device(dev):
            _lib.check(_lib.lib().cqa_score_blocks(
                C.byref(d), q.data_ptr(), _lib.dtype_code(q.dtype), nb, float(q_scale), m_b.data_ptr(),
                s_b.data_ptr(), nb, _lib.ptr(tok), _lib.current_stream(dev)), "cqa_score_blocks")
    if return_token_scores:
        # [kv, nb, G, 16] -> the reference's [H, nb, 16]
        return m_b, s_b, tok.permute(0, 2, 1, 3).reshape(H, nb, 16)
    return m_b, s_b


def adaptive_topk_cuda(*, m_b: Any, s_b: Any, tau_cov: float, k_min: int, k_max: int):
    """Returns (topk_mask bool, k_star i32, tail_mass, tau_actual, mass_frac,
    sorted_idx i64, k_star, sorted_cumsum) like the reference's native selector."""
    from dotcache.kernels.certified_attention import compute_adaptive_topk_mask

    return tuple(compute_adaptive_topk_mask(
        m_b, s_b, tau_cov=tau_cov, k_min=k_min, k_max=k_max, return_mass_frac=True,
        return_selection_indices=True, return_sorted_cumsum=True))


def hybrid_mixedv_split_k_cuda(*, keys_int8: Any, keys_scale: Any, keys_zero_points: Any, keys_fp16: Any,
                               key_block_slots: Any | None = None, topk_mask: Any,
                               values_int4_packed: Any | None, values_int4_scales: Any | None,
                               values_int4_zeros: Any | None, values_fp16_scratch: Any, value_fp16_mask: Any,
                               value_block_slots: Any | None, q_all: Any, gqa_group: int, block_size: int = 16,
                               group_size: int = 16, q_scale: float = 1.0, last_block_valid: int | None = None,
                               num_splits: int | None = None, int8_token_scores: Any | None = None,
                               workspace: Any | None = None, **_unused: Any):
    """Phase 2: hybrid INT8/FP16 keys, mixed INT4/FP16 values, split-K + merge.
    Returns out [H, 128] float32.  When the last block is partial
    (`last_block_valid` < 16) it is read from the FP16 key tensor, as the
    reference does by forcing its top-K bit."""
    if block_size != 16 or group_size != 16:
        raise ValueError("block_size and group_size must be 16")
    if not keys_int8.is_cuda:
        raise RuntimeError("hybrid_mixedv_split_k_cuda needs CUDA tensors; there is no CPU fallback")
    k, kstride = _rows_view(keys_int8, 128, "keys_int8")
    kv, n, _ = k.shape
    nb = n // 16
    H, G = int(q_all.shape[0]), int(gqa_group)
    lbv = 16 if last_block_valid is None else int(last_block_valid)
    nq = nb if lbv == 16 else nb - 1
    dev = k.device
    (s, z), sstride = _same_stride([_rows_view(keys_scale, 128, "keys_scale"),
                                    _rows_view(keys_zero_points, 128, "keys_zero_points")], "scales")
    kf, kfrows = _rows_view(keys_fp16, 128, "keys_fp16")
    vf, vfrows = _rows_view(values_fp16_scratch, 128, "values_fp16_scratch")
    if kf.dtype != vf.dtype:
        vf = vf.to(kf.dtype)
        vfrows = int(vf.shape[1])
    d = _lib.CqaCache()
    d.kv_heads, d.gqa_group, d.t2_dtype = kv, G, _lib.dtype_code(kf.dtype)
    d.keys_int8, d.keys_scale, d.keys_zero_points = k.data_ptr(), s.data_ptr(), z.data_ptr()
    d.max_blocks = sstride
    keep = [k, s, z, kf, vf]
    if values_int4_packed is not None:
        vp_, vps = _rows_view(values_int4_packed, 64, "values_int4_packed")
        (vs_, vz_), vss = _same_stride([_rows_view(values_int4_scales, 8, "values_int4_scales"),
                                        _rows_view(values_int4_zeros, 8, "values_int4_zeros")], "value scales")
        if not (vps == vss == kstride):
            k, vp_, vs_, vz_ = k.contiguous(), vp_.contiguous(), vs_.contiguous(), vz_.contiguous()
            kstride = int(k.shape[1])
            d.keys_int8 = k.data_ptr()
        d.values_int4_packed, d.values_int4_scales, d.values_int4_zeros = vp_.data_ptr(), vs_.data_ptr(), vz_.data_ptr()
        keep += [k, vp_, vs_, vz_]
    d.cap_tokens = kstride
    d.keys_t2, d.keys_t2_rows = kf.data_ptr(), kfrows
    d.values_t2, d.values_t2_rows = vf.data_ptr(), vfrows
    if key_block_slots is not None:
        ks = key_block_slots.to(torch.int32).contiguous()
        d.key_slots = ks.data_ptr()
        keep.append(ks)
    if value_block_slots is not None:
        vsl = value_block_slots.to(torch.int32).contiguous()
        d.value_slots = vsl.data_ptr()
        keep.append(vsl)
    f32 = dict(dtype=torch.float32, device=dev)
    wsd = workspace if isinstance(workspace, dict) else {}

    def buf(name, shape, dtype=torch.float32):
        t = wsd.get(name)
        if t is None or tuple(t.shape) != tuple(shape) or t.dtype != dtype or t.device != dev:
            t = torch.empty(shape, dtype=dtype, device=dev)
            wsd[name] = t
        return t

    ns, ds = C.c_int(0), C.c_int(0)
    with torch.cuda.device(dev):
        _lib.check(_lib.lib().cqa_suggest_splits(kv, G, nb, C.byref(ns), C.byref(ds)), "cqa_suggest_splits")
    nsplit = int(num_splits) if num_splits else ns.value
    nsplit = max(1, min(nsplit, nb))
    w = _lib.CqaWorkspace()
    w.ld = nb
    tok = buf("cqa_token_scores", (kv, max(nq, 1), G, 16))
    m_b = buf("cqa_m_b", (H, nb))
    s_b = buf("cqa_s_b", (H, nb))
    tk = topk_mask.to(torch.uint8).contiguous()
    vm = value_fp16_mask.to(torch.uint8).contiguous()
    part_m, part_l = buf("mixedv_m_part", (H, nsplit)), buf("mixedv_l_part", (H, nsplit))
    part_acc = buf("mixedv_acc_part", (H, nsplit, 128))
    out = buf("mixedv_output", (H, 128))
    tickets = wsd.get("cqa_tickets")
    if tickets is None or tickets.numel() != kv + H or tickets.device != dev:
        tickets = torch.zeros(kv + H, dtype=torch.int32, device=dev)
        wsd["cqa_tickets"] = tickets
    w.m_b, w.s_b, w.token_scores = m_b.data_ptr(), s_b.data_ptr(), tok.data_ptr()
    w.topk_mask, w.value_mask = tk.data_ptr(), vm.data_ptr()
    w.num_splits, w.dense_splits = nsplit, 0
    w.part_m, w.part_l, w.part_acc, w.out = part_m.data_ptr(), part_l.data_ptr(), part_acc.data_ptr(), out.data_ptr()
    w.tickets = tickets.data_ptr()
    q = q_all.contiguous()
    qd = _lib.dtype_code(q.dtype)
    L = _lib.lib()
    st = _lib.current_stream(dev)
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(2)] if _PROFILE_ENABLED else None
    with torch.cuda.device(dev):
        if ev:
            ev[0].record()
        if nq > 0:
            _lib.check(L.cqa_score_blocks(C.byref(d), q.data_ptr(), qd, nq, float(q_scale), m_b.data_ptr(),
                                          s_b.data_ptr(), nb, tok.data_ptr(), st), "cqa_score_blocks")
        _lib.check(L.cqa_attend(C.byref(d), C.byref(w), q.data_ptr(), qd, nq, nb, nq * 16 + (lbv if nq < nb else 0),
                                lbv, float(q_scale), st), "cqa_attend")
        if ev:
            ev[1].record()
            torch.cuda.synchronize()
            _PROFILE["calls"] += 1
            _PROFILE["partial_ms_total"] += float(ev[0].elapsed_time(ev[1]))
    del keep
    return out
