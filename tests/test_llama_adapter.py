"""The Llama adapter: a tiny random-init LlamaForCausalLM decodes through the certified path (append + certified
attention per layer) and stays close to its own dense decode; state and stats plumbing follow the reference."""
from __future__ import annotations

import pytest
import torch

from dotcache.integrations.llama import (CertifiedAttentionState, CertifiedLlamaAttention,
                                         build_certified_state_from_prefill, install_certified_attention,
                                         remove_certified_attention)


def test_state_requires_v_tolerance_and_keeps_reference_defaults():
    with pytest.raises(ValueError):
        CertifiedAttentionState(tiered_caches={})
    st = CertifiedAttentionState(tiered_caches={}, v_tolerance=0.05)
    assert (st.block_size, st.top_k_fp16_keys, st.k_min, st.k_max, st.tau_cov) == (16, 4, 2, None, None)
    assert st.rung1_threshold == 0.02 and st.rung1_multiplier == 2.0 and st.value_error_mode == "tight"
    assert st.score_consistency_check and st.score_consistency_enabled_for_layer(0)
    st.step_stats.append({"layer": 0})
    assert st.clear_step_stats() == [{"layer": 0}] and st.step_stats == [] and st._clear_seq == 1
    st2 = CertifiedAttentionState(tiered_caches={}, v_tolerance=0.05, score_consistency_interval=4)
    fired = []
    for _ in range(8):
        st2.begin_decode_step()
        fired.append(st2.score_consistency_enabled_for_layer(3))
    assert fired == [False, False, False, True, False, False, False, True]


@pytest.mark.gpu
def test_tiny_llama_decodes_through_the_certified_path():
    from transformers import LlamaConfig, LlamaForCausalLM

    torch.manual_seed(0)
    cfg = LlamaConfig(vocab_size=512, hidden_size=512, intermediate_size=1024, num_hidden_layers=2,
                      num_attention_heads=4, num_key_value_heads=2, head_dim=128, max_position_embeddings=4096,
                      rms_norm_eps=1e-5, tie_word_embeddings=False)
    model = LlamaForCausalLM(cfg).to(torch.bfloat16).cuda().eval()
    T, steps = 1024 + 5, 20
    ids = torch.randint(0, cfg.vocab_size, (1, T + steps), device="cuda")
    with torch.no_grad():
        pre = model(input_ids=ids[:, :T], use_cache=True)
        past = pre.past_key_values
        # dense decode, token by token, on a copy of the prefill cache
        import copy

        dense_past = copy.deepcopy(past)
        dense_logits = []
        for s in range(steps):
            out = model(input_ids=ids[:, T + s: T + s + 1], past_key_values=dense_past, use_cache=True)
            dense_logits.append(out.logits[0, -1].float())
        state = build_certified_state_from_prefill(past, [0, 1], max_new_tokens=64, collect_stats=True)
        wrappers = install_certified_attention(model, state)
        assert len(wrappers) == 2 and all(isinstance(w, CertifiedLlamaAttention) for w in wrappers)
        cert_logits = []
        for s in range(steps):
            state.begin_decode_step()
            pos = torch.tensor([[T + s]], device="cuda")
            out = model(input_ids=ids[:, T + s: T + s + 1], position_ids=pos, use_cache=False)
            cert_logits.append(out.logits[0, -1].float())
        remove_certified_attention(model)
    assert all(c.num_tokens == T + steps for c in state.tiered_caches.values())
    per_layer = state.clear_step_stats()
    assert len(per_layer) == 2 * steps and {d["layer"] for d in per_layer} == {0, 1}
    assert all("k_star_mean" in d and "e_val_max" in d for d in per_layer)
    for s in range(steps):
        d, c = dense_logits[s], cert_logits[s]
        cos = torch.nn.functional.cosine_similarity(d, c, dim=0).item()
        rel = ((d - c).norm() / d.norm()).item()
        assert cos > 0.999 and rel < 5e-2, f"step {s}: cosine {cos}, relative error {rel}"
        assert d.argmax().item() == c.argmax().item() or (d.max() - d[c.argmax()]).item() < 0.05


@pytest.mark.gpu
def test_tiny_llama_batch_of_two_decodes_in_one_launch_chain_per_layer():
    """Batch 2 (the reference raises on it): every layer's append + certified step is one batched chain of four
    launches for both sequences; logits stay close to the model's own dense batch decode."""
    import copy

    from transformers import LlamaConfig, LlamaForCausalLM

    from cqa_b200 import _lib

    torch.manual_seed(1)
    cfg = LlamaConfig(vocab_size=512, hidden_size=512, intermediate_size=1024, num_hidden_layers=2,
                      num_attention_heads=4, num_key_value_heads=2, head_dim=128, max_position_embeddings=4096,
                      rms_norm_eps=1e-5, tie_word_embeddings=False)
    model = LlamaForCausalLM(cfg).to(torch.bfloat16).cuda().eval()
    T, steps, B = 768 + 9, 12, 2
    ids = torch.randint(0, cfg.vocab_size, (B, T + steps), device="cuda")
    with torch.no_grad():
        past = model(input_ids=ids[:, :T], use_cache=True).past_key_values
        dense_past = copy.deepcopy(past)
        dense_logits = []
        for s in range(steps):
            out = model(input_ids=ids[:, T + s: T + s + 1], past_key_values=dense_past, use_cache=True)
            dense_logits.append(out.logits[:, -1].float())
        state = build_certified_state_from_prefill(past, [0, 1], max_new_tokens=64)
        assert state.batch_caches is not None and all(len(v) == B for v in state.batch_caches.values())
        install_certified_attention(model, state)
        cert_logits, launches = [], []
        for s in range(steps):
            state.begin_decode_step()
            pos = torch.full((B, 1), T + s, device="cuda")
            before = _lib.lib().cqa_launch_count(0)
            out = model(input_ids=ids[:, T + s: T + s + 1], position_ids=pos, use_cache=False)
            launches.append(_lib.lib().cqa_launch_count(0) - before)
            cert_logits.append(out.logits[:, -1].float())
        remove_certified_attention(model)
    assert all(c.num_tokens == T + steps for cs in state.batch_caches.values() for c in cs)
    assert all(n == 2 * 4 for n in launches), launches      # 2 layers x (append, score, selector, attend)
    for s in range(steps):
        for b in range(B):
            d, c = dense_logits[s][b], cert_logits[s][b]
            cos = torch.nn.functional.cosine_similarity(d, c, dim=0).item()
            rel = ((d - c).norm() / d.norm()).item()
            assert cos > 0.999 and rel < 5e-2, f"step {s} sequence {b}: cosine {cos}, relative error {rel}"
