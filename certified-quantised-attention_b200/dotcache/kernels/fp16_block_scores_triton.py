"""FP16 selected-block scores (reference: dotcache/kernels/fp16_block_scores_triton.py:73-146).
The module keeps the reference's name; the kernel is CUDA, not Triton."""
from __future__ import annotations

import ctypes as C

import torch

from cqa_b200 import _lib


def fp16_block_scores_triton(keys: torch.Tensor, q_all: torch.Tensor, block_indices: torch.Tensor, *,
                             num_scoring_blocks: int, gqa_group: int, block_size: int, q_scale: float,
                             key_block_slots: torch.Tensor | None = None):
    """keys [kv, T, 128] (fp16/bf16/fp32), block_indices [H, K] -> (max logits, log-masses) [H, K]."""
    if not (keys.is_cuda and q_all.is_cuda and block_indices.is_cuda):
        raise ValueError("fp16_block_scores_triton requires CUDA tensors")
    if keys.ndim != 3 or q_all.ndim != 2 or block_indices.ndim != 2:
        raise ValueError("invalid tensor ranks for fp16_block_scores_triton")
    if block_size != 16 or keys.shape[2] != 128:
        raise ValueError("block_size must be 16 and head_dim 128")
    H, K = block_indices.shape
    if H != q_all.shape[0]:
        raise ValueError("block_indices head dimension must match q_all")
    dev = q_all.device
    scores = torch.full((H, K), float("-inf"), dtype=torch.float32, device=dev)
    logm = torch.full((H, K), float("-inf"), dtype=torch.float32, device=dev)
    if K == 0 or num_scoring_blocks <= 0:
        return scores, logm
    kc = keys.contiguous()
    d = _lib.CqaCache()
    d.kv_heads, d.gqa_group = int(kc.shape[0]), int(gqa_group)
    d.t2_dtype = _lib.dtype_code(kc.dtype)
    d.cap_tokens, d.max_blocks = int(kc.shape[1]), max(int(num_scoring_blocks), 1)
    d.keys_t2, d.keys_t2_rows = kc.data_ptr(), int(kc.shape[1])
    slots = None
    if key_block_slots is not None:
        slots = torch.full((int(num_scoring_blocks),), -1, dtype=torch.int32, device=dev)
        n = min(int(key_block_slots.numel()), int(num_scoring_blocks))
        slots[:n] = key_block_slots[:n].to(torch.int32)
        d.key_slots = slots.data_ptr()
    idx = block_indices.to(torch.int32).contiguous()
    q = q_all.contiguous()
    with torch.cuda.device(dev):
        _lib.check(_lib.lib().cqa_fp16_block_scores(
            C.byref(d), q.data_ptr(), _lib.dtype_code(q.dtype), idx.data_ptr(), K, int(num_scoring_blocks),
            float(q_scale), scores.data_ptr(), logm.data_ptr(), _lib.current_stream(dev)), "cqa_fp16_block_scores")
    return scores, logm
