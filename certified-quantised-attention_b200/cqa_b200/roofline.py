"""Algorithmic HBM bytes of one certified decode step (one layer, one sequence).

"Algorithmic" means every byte the step needs is counted once, no matter how
often an implementation re-reads it, with GQA sharing (one load serves all the
query heads of a KV group):

  Phase 1   : INT8 keys 128 B/token + per-block scale and zero point 64 B/token
              = 192 B per quantised token per KV head
  Phase 2   : INT4 values 64 B + scale/zero 32 B = 96 B/token for blocks that at
              least one head of the group reads as INT4; FP16 values 256 B/token
              for blocks at least one head reads from Tier 2 (both if the group
              is split); FP16 keys 256 B/token for the per-KV-head union of
              promoted, explored and re-scored blocks; the trailing partial
              block t * 512 B per KV head
  Rung 3/4  : dense FP16 recompute, 512 B/token per KV head that has a flagged head
  small     : block statistics and masks, 40 B per (head, block)

The token-score cache between Phase 1 and Phase 2 (16 B/token/KV head, written
once and read once) is implementation traffic, not algorithmic, and is not
counted.
"""
from __future__ import annotations

import numpy as np

BLOCK = 16


def tier1_floor_bytes(n_tokens: int, kv_heads: int = 8) -> int:
    """Pure Tier-1 floor: 288 B per token per KV head."""
    return int(n_tokens) * kv_heads * 288


def step_bytes(topk_mask: np.ndarray, value_mask: np.ndarray, nq: int, nact: int, last_valid: int,
               gqa_group: int, dense_heads: np.ndarray | None = None, t2_elem: int = 2,
               top_blocks: np.ndarray | None = None) -> dict:
    """Bytes by kernel for one step.

    topk_mask, value_mask: [H, >=nact] 0/1 arrays (FP16-key / FP16-value bits);
    dense_heads: [H] 0/1 (heads recomputed densely); top_blocks: [H, k] block
    ids re-scored with FP16 keys by the ranking check (-1 = unused).
    """
    H = topk_mask.shape[0]
    KV = H // gqa_group
    tm = np.asarray(topk_mask[:, :nq], dtype=bool).reshape(KV, gqa_group, nq)
    vm = np.asarray(value_mask[:, :nq], dtype=bool).reshape(KV, gqa_group, nq)
    row = 128 * t2_elem
    score = KV * nq * BLOCK * 192
    key_union = tm.any(axis=1)
    if top_blocks is not None:
        tb = np.asarray(top_blocks).reshape(KV, -1)
        for kv in range(KV):
            ids = tb[kv][(tb[kv] >= 0) & (tb[kv] < nq)]
            key_union[kv, ids] = True
    fp16_keys = int(key_union.sum()) * BLOCK * row
    v_fp16 = int(vm.any(axis=1).sum()) * BLOCK * row
    v_int4 = int((~vm).any(axis=1).sum()) * BLOCK * 96
    trailing = 0
    if nact > nq:
        trailing = KV * last_valid * 2 * row
    dense = 0
    if dense_heads is not None and np.asarray(dense_heads).any():
        dk = np.asarray(dense_heads, dtype=bool).reshape(KV, gqa_group).any(axis=1)
        dense = int(dk.sum()) * (nq * BLOCK + (last_valid if nact > nq else 0)) * 2 * row
    small = H * nact * 40
    attend = fp16_keys + v_fp16 + v_int4 + trailing
    return {
        "score": int(score), "attend": int(attend), "dense": int(dense), "small": int(small),
        "fp16_key_bytes": int(fp16_keys), "fp16_value_bytes": int(v_fp16), "int4_value_bytes": int(v_int4),
        "total": int(score + attend + dense + small),
    }
