"""Phase-1 block scoring (reference: dotcache/kernels/fused_score_certify.py:398-456)."""
from __future__ import annotations

from dotcache.backends.certified_blackwell import score_blocks_cuda

import torch


def fused_score_certify_multihead(K_int8_packed, K_scale, K_zero_points, q_all, correction, gqa_group: int,
                                  block_size: int = 16, q_scale: float = 1.0, block_epsilon: float = 0.001,
                                  return_token_scores: bool = False):
    """Returns (m_b, S_b, skip_mask[, token_scores [H, nb, 16]]).  The legacy
    epsilon skip mask is not built: the paper path always calls this with
    block_epsilon=0.0, for which the mask is all False."""
    if block_epsilon != 0.0:
        raise NotImplementedError("legacy block-epsilon skipping is not built; pass block_epsilon=0.0")
    res = score_blocks_cuda(keys_int8=K_int8_packed, keys_scale=K_scale, keys_zero_points=K_zero_points,
                            q_all=q_all, gqa_group=gqa_group, block_size=block_size, q_scale=q_scale,
                            return_token_scores=return_token_scores)
    m_b, S_b = res[0], res[1]
    skip = torch.zeros(m_b.shape, dtype=torch.bool, device=m_b.device)
    if return_token_scores:
        return m_b, S_b, skip, res[2]
    return m_b, S_b, skip
