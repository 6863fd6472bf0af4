"""Llama adapter for certified decode attention.

The reference's `dotcache/integrations/llama.py` is a 1900-line harness
(dense/dotcache/certified modes, page caches, profiling); the part that sits
on the certified path is small and is what this module provides, with the
reference's names and argument meaning:

* `CertifiedAttentionState` (llama.py:81-173): the knob carrier with the
  per-layer `TieredKeyCacheLayer` objects and the per-step stats list.
* `CertifiedLlamaAttention._forward_certified` (llama.py:710-797): for a decode
  step of batch 1, project q/k/v, apply RoPE, append the new token to the
  layer's cache, run `certified_attention_layer`, project the output.
* `install_certified_attention` / `remove_certified_attention`: swap the
  `self_attn` modules of a HF `LlamaForCausalLM` (the reference does the same
  swap in `LlamaDotCacheModelAdapter._install_wrappers`).
* `build_certified_state_from_prefill`: INT8-key / INT4-value caches from the
  model's own prefill KV (reference: `create_tiered_cache_int4v_from_model`,
  tiered_kv_cache.py:1579-1641).

* batch > 1 (an addition; the reference raises on it, llama.py:717-718): with
  `CertifiedAttentionState.batch_caches` (one cache per layer and sequence) a
  single-token decode call of B sequences runs each layer's append and
  certified step as ONE batched launch chain (`certified_attention_batch`).

Prefill and any call that is not a single-token decode go through the wrapped
HF attention unchanged.
"""
from __future__ import annotations

from dataclasses import dataclass, field

import torch
from torch import nn

from ..kernels.certified_attention import certified_attention_batch, certified_attention_layer
from ..kernels.tiered_kv_cache import TieredKeyCacheLayer, create_tiered_cache_int4v_from_model


@dataclass
class CertifiedAttentionState:
    """Runtime state of certified attention mode (reference: llama.py:81-173; same fields and defaults)."""

    tiered_caches: dict                      # layer_id -> TieredKeyCacheLayer
    block_size: int = 16
    collect_stats: bool = True               # False during timed runs: no host synchronisation
    append_kv: bool = False                  # append the new token's K/V to the tiered cache during decode
    top_k_fp16_keys: int = 4
    ranking_fallback: bool = False
    ranking_r: int = 1
    ranking_fallback_mode: str = "full"
    tau_cov: float | None = None
    k_min: int = 2
    k_max: int | None = None
    rung1_threshold: float = 0.02
    rung1_multiplier: float = 2.0
    score_consistency_check: bool = True
    score_consistency_interval: int = 1
    eps_guard: float = 0.01
    v_tolerance: float = -1.0                # sentinel: must be set explicitly (paper value 0.05)
    exploration_rate: float = 0.0
    per_kv_group_topk: bool = False
    value_error_mode: str = "tight"
    step_stats: list = None
    _clear_seq: int = 0
    phase_timings: dict | None = None
    _score_consistency_step: int = 0
    # batch > 1 (an addition; the reference raises, llama.py:717-718): layer_id -> list of one cache per sequence.
    # A decode call with B sequences then runs each layer's step as ONE batched launch chain.
    batch_caches: dict | None = None

    def __post_init__(self):
        if self.step_stats is None:
            self.step_stats = []
        if self.v_tolerance < 0.0:
            raise ValueError("CertifiedAttentionState requires an explicit v_tolerance (paper value: 0.05)")
        if self.score_consistency_interval < 1:
            raise ValueError("score_consistency_interval must be at least 1")

    def clear_step_stats(self) -> list[dict]:
        """Return the accumulated per-layer stats and start a new list."""
        out = self.step_stats
        self.step_stats = []
        self._clear_seq += 1
        return out

    def begin_decode_step(self) -> None:
        """Called once per generated token (before the first layer)."""
        self._score_consistency_step += 1

    def score_consistency_enabled_for_layer(self, layer_idx: int) -> bool:
        """The consistency check runs on every `score_consistency_interval`-th decode step."""
        if not self.score_consistency_check:
            return False
        n = self.score_consistency_interval
        return n <= 1 or (self._score_consistency_step % n) == 0


class CertifiedLlamaAttention(nn.Module):
    """Drop-in for a HF `LlamaAttention`: batch-1 single-token decode goes through the certified path, everything
    else through the wrapped module."""

    def __init__(self, base_attention: nn.Module, state: CertifiedAttentionState):
        super().__init__()
        self.base_attention = base_attention
        self.certified_state = state
        self.layer_idx = int(base_attention.layer_idx)
        self.config = base_attention.config

    def _project_qkv(self, hidden_states, position_embeddings):
        from transformers.models.llama import modeling_llama as llama_mod

        base = self.base_attention
        shape = (*hidden_states.shape[:-1], -1, base.head_dim)
        q = base.q_proj(hidden_states).view(shape).transpose(1, 2)
        k = base.k_proj(hidden_states).view(shape).transpose(1, 2)
        v = base.v_proj(hidden_states).view(shape).transpose(1, 2)
        cos, sin = position_embeddings
        q, k = llama_mod.apply_rotary_pos_emb(q, k, cos, sin)
        return q, k, v

    def _forward_certified(self, hidden_states, position_embeddings=None):
        """One decode step of this layer (reference: llama.py:710-797)."""
        if hidden_states.shape[1] != 1:
            raise ValueError("Certified decode mode only supports query_len=1")
        if position_embeddings is None:
            raise ValueError("position_embeddings are required for the Llama attention path")
        st = self.certified_state
        if hidden_states.shape[0] != 1:
            return self._forward_certified_batch(hidden_states, position_embeddings)
        cache = st.tiered_caches.get(self.layer_idx)
        if cache is None:
            raise ValueError(f"No tiered cache for layer {self.layer_idx}")
        q, k, v = self._project_qkv(hidden_states, position_embeddings)
        q_all = q[0, :, 0, :]                                    # [num_q_heads, head_dim], model dtype
        if st.append_kv:
            cache.append_token(k[0], v[0])                       # [kv_heads, 1, head_dim]
        gqa_group = self.config.num_attention_heads // self.config.num_key_value_heads
        context, stats = certified_attention_layer(
            cache, q_all, gqa_group, float(self.base_attention.scaling),
            collect_stats=st.collect_stats,
            v_tolerance=st.v_tolerance, top_k_fp16_keys=st.top_k_fp16_keys,
            ranking_fallback=st.ranking_fallback, ranking_r=st.ranking_r,
            ranking_fallback_mode=st.ranking_fallback_mode, tau_cov=st.tau_cov, k_min=st.k_min, k_max=st.k_max,
            rung1_threshold=st.rung1_threshold, rung1_multiplier=st.rung1_multiplier,
            score_consistency_check=st.score_consistency_enabled_for_layer(self.layer_idx),
            eps_guard=st.eps_guard, exploration_rate=st.exploration_rate, phase_timings=st.phase_timings,
            per_kv_group_topk=st.per_kv_group_topk, value_error_mode=st.value_error_mode,
        )
        if st.collect_stats and stats:
            st.step_stats.append({"layer": self.layer_idx, **stats})
        ctx = context.to(dtype=hidden_states.dtype).reshape(1, 1, -1)
        return self.base_attention.o_proj(ctx), None

    def _forward_certified_batch(self, hidden_states, position_embeddings):
        """One decode step of this layer for B sequences with their own caches: one append and one chain of three
        kernels for the whole batch (certified_attention_batch).  Per-layer stats are not collected here; the
        certificates stay in each cache's workspace."""
        st = self.certified_state
        caches = (st.batch_caches or {}).get(self.layer_idx)
        B = hidden_states.shape[0]
        if caches is None or len(caches) != B:
            raise ValueError(f"No batch of {B} tiered caches for layer {self.layer_idx}")
        q, k, v = self._project_qkv(hidden_states, position_embeddings)
        gqa_group = self.config.num_attention_heads // self.config.num_key_value_heads
        context = certified_attention_batch(
            caches, q[:, :, 0, :], gqa_group, float(self.base_attention.scaling),
            new_keys=k[:, :, 0, :] if st.append_kv else None, new_values=v[:, :, 0, :] if st.append_kv else None,
            v_tolerance=st.v_tolerance, top_k_fp16_keys=st.top_k_fp16_keys,
            ranking_fallback=st.ranking_fallback, ranking_r=st.ranking_r,
            ranking_fallback_mode=st.ranking_fallback_mode, tau_cov=st.tau_cov, k_min=st.k_min, k_max=st.k_max,
            rung1_threshold=st.rung1_threshold, rung1_multiplier=st.rung1_multiplier,
            score_consistency_check=st.score_consistency_enabled_for_layer(self.layer_idx),
            eps_guard=st.eps_guard, exploration_rate=st.exploration_rate, value_error_mode=st.value_error_mode,
        )
        ctx = context.to(dtype=hidden_states.dtype).reshape(B, 1, -1)
        return self.base_attention.o_proj(ctx), None

    def forward(self, hidden_states, position_embeddings=None, attention_mask=None, past_key_values=None, **kwargs):
        st = self.certified_state
        B = hidden_states.shape[0]
        decode = st is not None and hidden_states.shape[1] == 1 and (
            (B == 1 and self.layer_idx in st.tiered_caches)
            or (B > 1 and st.batch_caches is not None and len(st.batch_caches.get(self.layer_idx, ())) == B))
        if decode:
            return self._forward_certified(hidden_states, position_embeddings)
        return self.base_attention(hidden_states, position_embeddings=position_embeddings,
                                   attention_mask=attention_mask, past_key_values=past_key_values, **kwargs)


def install_certified_attention(model: nn.Module, state: CertifiedAttentionState) -> list[CertifiedLlamaAttention]:
    """Wrap every decoder layer's `self_attn` whose layer id has a tiered cache; returns the wrappers."""
    wrappers = []
    for layer in model.model.layers:
        attn = layer.self_attn
        if isinstance(attn, CertifiedLlamaAttention):
            attn.certified_state = state
            wrappers.append(attn)
            continue
        if int(attn.layer_idx) in state.tiered_caches or int(attn.layer_idx) in (state.batch_caches or {}):
            w = CertifiedLlamaAttention(attn, state)
            layer.self_attn = w
            wrappers.append(w)
    return wrappers


def remove_certified_attention(model: nn.Module) -> None:
    for layer in model.model.layers:
        if isinstance(layer.self_attn, CertifiedLlamaAttention):
            layer.self_attn = layer.self_attn.base_attention


def build_certified_state_from_prefill(past_key_values, layer_ids: list[int], *, max_new_tokens: int = 512,
                                       fp16_key_cache_capacity: int | None = None,
                                       fp16_value_cache_capacity: int | None = None,
                                       **state_kwargs) -> CertifiedAttentionState:
    """INT8-key / INT4-value caches from a prefill's KV (one cache per layer; with a batch of prompts one per layer
    and sequence, in `batch_caches`), wrapped in a state with the paper's knobs
    unless overridden: tau_cov 0.995, k in [2, 128], ranking fallback r = 1, v_tolerance 0.05, append_kv on."""
    knobs = dict(append_kv=True, tau_cov=0.995, k_min=2, k_max=128, ranking_fallback=True, ranking_r=1,
                 v_tolerance=0.05, score_consistency_check=False, collect_stats=False)
    knobs.update(state_kwargs)
    batch = _prefill_batch_size(past_key_values, layer_ids[0])
    per_seq = [create_tiered_cache_int4v_from_model(
        past_key_values, layer_ids, max_new_tokens=max_new_tokens, fp16_key_cache_capacity=fp16_key_cache_capacity,
        fp16_value_cache_capacity=fp16_value_cache_capacity, batch_index=b) for b in range(batch)]
    if batch == 1:
        return CertifiedAttentionState(tiered_caches=per_seq[0], **knobs)
    # a batch of prompts (all of the prefill's length): one cache per (layer, sequence)
    return CertifiedAttentionState(tiered_caches={}, batch_caches={l: [c[l] for c in per_seq] for l in layer_ids},
                                   **knobs)


def _prefill_batch_size(past_kv, layer_id: int) -> int:
    if hasattr(past_kv, "layers"):
        return int(past_kv.layers[layer_id].keys.shape[0])
    return int(past_kv[layer_id][0].shape[0])
