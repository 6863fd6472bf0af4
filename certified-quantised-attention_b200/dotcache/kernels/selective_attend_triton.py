"""Phase-2 attend entry points under the reference's names
(dotcache/kernels/selective_attend_triton.py).  All of them run the one CUDA
split-K kernel of libcqa_b200.so; the module name is kept for drop-in
imports, nothing here uses Triton.

Block skipping (`skip_mask_i32` with non-zero entries) belongs to the
reference's legacy path and is not built: the paper path always passes an
all-zero mask.
"""
from __future__ import annotations

import torch

from dotcache.backends.certified_blackwell import hybrid_mixedv_split_k_cuda


def _no_skip(skip_mask_i32):
    if skip_mask_i32 is not None and bool(skip_mask_i32.any().item()):
        raise NotImplementedError("block skipping is not built; pass an all-zero skip mask")


def selective_attend_multihead_hybrid_mixedv_split_k(keys_int8, keys_scale, keys_zero_points, keys_fp16, topk_mask,
                                                     values_int4_packed, values_int4_scales, values_int4_zeros,
                                                     values_fp16_scratch, value_fp16_mask, value_block_slots, q_all,
                                                     skip_mask_i32=None, gqa_group=1, block_size=16, group_size=16,
                                                     q_scale=1.0, last_block_valid=None, num_splits=None,
                                                     key_block_slots=None, int8_token_scores=None, workspace=None):
    """Reference: selective_attend_triton.py:1448-1576."""
    _no_skip(skip_mask_i32)
    return hybrid_mixedv_split_k_cuda(
        keys_int8=keys_int8, keys_scale=keys_scale, keys_zero_points=keys_zero_points, keys_fp16=keys_fp16,
        key_block_slots=key_block_slots, topk_mask=topk_mask, values_int4_packed=values_int4_packed,
        values_int4_scales=values_int4_scales, values_int4_zeros=values_int4_zeros,
        values_fp16_scratch=values_fp16_scratch, value_fp16_mask=value_fp16_mask,
        value_block_slots=value_block_slots, q_all=q_all, gqa_group=gqa_group, block_size=block_size,
        group_size=group_size, q_scale=q_scale, last_block_valid=last_block_valid, num_splits=num_splits,
        workspace=workspace)


def selective_attend_multihead_hybrid_mixedv(*args, **kwargs):
    """Reference: selective_attend_triton.py:876-961 (single-program variant; same result)."""
    return selective_attend_multihead_hybrid_mixedv_split_k(*args, **kwargs)


def selective_attend_multihead_hybrid_int4v(keys_int8, keys_scale, keys_zero_points, keys_fp16, topk_mask,
                                            values_int4_packed, values_int4_scales, values_int4_zeros, q_all,
                                            skip_mask_i32=None, gqa_group=1, block_size=16, group_size=16, q_scale=1.0,
                                            last_block_valid=None, key_block_slots=None, workspace=None):
    """Hybrid keys + INT4 values everywhere (reference: selective_attend_triton.py:633-708)."""
    _no_skip(skip_mask_i32)
    vmask = torch.zeros(topk_mask.shape, dtype=torch.uint8, device=topk_mask.device)
    return hybrid_mixedv_split_k_cuda(
        keys_int8=keys_int8, keys_scale=keys_scale, keys_zero_points=keys_zero_points, keys_fp16=keys_fp16,
        key_block_slots=key_block_slots, topk_mask=topk_mask, values_int4_packed=values_int4_packed,
        values_int4_scales=values_int4_scales, values_int4_zeros=values_int4_zeros,
        values_fp16_scratch=keys_fp16, value_fp16_mask=vmask, value_block_slots=None, q_all=q_all,
        gqa_group=gqa_group, block_size=block_size, group_size=group_size, q_scale=q_scale,
        last_block_valid=last_block_valid, workspace=workspace)


def selective_attend_multihead_hybrid_split_k(keys_int8, keys_scale, keys_zero_points, keys_fp16, topk_mask,
                                              values_fp16, q_all, skip_mask_i32=None, gqa_group=1, block_size=16,
                                              q_scale=1.0, last_block_valid=None, num_splits=None,
                                              key_block_slots=None, workspace=None):
    """Hybrid keys + FP16 values (reference: selective_attend_triton.py:1579-1700)."""
    _no_skip(skip_mask_i32)
    vmask = torch.ones(topk_mask.shape, dtype=torch.uint8, device=topk_mask.device)
    return hybrid_mixedv_split_k_cuda(
        keys_int8=keys_int8, keys_scale=keys_scale, keys_zero_points=keys_zero_points, keys_fp16=keys_fp16,
        key_block_slots=key_block_slots, topk_mask=topk_mask, values_int4_packed=None, values_int4_scales=None,
        values_int4_zeros=None, values_fp16_scratch=values_fp16, value_fp16_mask=vmask, value_block_slots=None,
        q_all=q_all, gqa_group=gqa_group, block_size=block_size, q_scale=q_scale,
        last_block_valid=last_block_valid, num_splits=num_splits, workspace=workspace)


def selective_attend_multihead_hybrid(*args, **kwargs):
    """Reference: selective_attend_triton.py:1084-1101 (single-program variant; same result)."""
    return selective_attend_multihead_hybrid_split_k(*args, **kwargs)


def selective_attend_multihead_int8k_int4v(keys_int8, keys_scale, keys_zero_points, values_int4_packed,
                                           values_int4_scales, values_int4_zeros, q_all, skip_mask_i32=None,
                                           gqa_group=1, block_size=16, group_size=16, q_scale=1.0):
    """INT8 keys + INT4 values for every block (reference: selective_attend_triton.py:436-494).
    Needs no FP16 tensors: every block must be complete."""
    _no_skip(skip_mask_i32)
    H = q_all.shape[0]
    nb = keys_int8.shape[1] // 16
    zeros = torch.zeros(H, nb, dtype=torch.uint8, device=q_all.device)
    dummy = torch.zeros(keys_int8.shape[0], 16, 128, dtype=torch.float16, device=q_all.device)
    return hybrid_mixedv_split_k_cuda(
        keys_int8=keys_int8, keys_scale=keys_scale, keys_zero_points=keys_zero_points, keys_fp16=dummy,
        topk_mask=zeros, values_int4_packed=values_int4_packed, values_int4_scales=values_int4_scales,
        values_int4_zeros=values_int4_zeros, values_fp16_scratch=dummy, value_fp16_mask=zeros,
        value_block_slots=None, q_all=q_all, gqa_group=gqa_group, block_size=block_size, group_size=group_size,
        q_scale=q_scale, last_block_valid=16)


def selective_attend_multihead_int8(keys_int8, keys_scale, keys_zero_points, values_fp16, q_all, skip_mask_i32=None,
                                    gqa_group=1, block_size=16, q_scale=1.0):
    """INT8 keys + FP16 values for every block (reference: selective_attend_triton.py:250-301)."""
    _no_skip(skip_mask_i32)
    H = q_all.shape[0]
    nb = keys_int8.shape[1] // 16
    dev = q_all.device
    return hybrid_mixedv_split_k_cuda(
        keys_int8=keys_int8, keys_scale=keys_scale, keys_zero_points=keys_zero_points, keys_fp16=values_fp16,
        topk_mask=torch.zeros(H, nb, dtype=torch.uint8, device=dev), values_int4_packed=None,
        values_int4_scales=None, values_int4_zeros=None, values_fp16_scratch=values_fp16,
        value_fp16_mask=torch.ones(H, nb, dtype=torch.uint8, device=dev), value_block_slots=None, q_all=q_all,
        gqa_group=gqa_group, block_size=block_size, q_scale=q_scale, last_block_valid=16)


def selective_attend_multihead(*_a, **_k):
    """float32-key/value attend of the reference's earliest prototype
    (selective_attend_triton.py:72-153); nothing on the certified path calls it."""
    raise NotImplementedError("float32 K/V attend is not part of the certified path")
