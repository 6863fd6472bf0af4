"""GPU parity tests: the CUDA path (through the C ABI) against the CPU oracle on
the same seeded inputs, and against the golden vectors from the reference."""
from __future__ import annotations

import json

import numpy as np
import pytest
import torch

import golden_cases as gc
from cqa_b200 import synth

pytestmark = pytest.mark.gpu

if torch.cuda.is_available():
    import cuda_harness as hz
    from oracle import cqa_oracle as orc
    from test_oracle_golden import check_cache_snapshot, check_call


def _knobs(**over):
    k = dict(gc.PAPER_KNOBS)
    k.update(over)
    return k


def _oracle_knobs(knobs, u):
    k = dict(knobs)
    k["exploration_u"] = u
    return k


@pytest.mark.parametrize("dtype", ["float32", "float16", "bfloat16"])
def test_prefill_quantisation_bit_exact(dtype):
    base = synth.make_layer_inputs(101, 2048, kv_heads=2, gqa_group=4, dtype=dtype)
    cc = hz.make_cuda_cache(base.k, base.v, dtype, 64)
    oc = hz.make_oracle_cache(base.k, base.v, dtype, 64)
    hz.compare_caches(cc, oc, f"prefill[{dtype}]")


@pytest.mark.parametrize("dtype,defer", [("bfloat16", True), ("float16", False), ("float32", True)])
def test_append_sequence_bit_exact(dtype, defer):
    base = synth.make_layer_inputs(102, 512, kv_heads=3, gqa_group=2, dtype=dtype)
    cc = hz.make_cuda_cache(base.k, base.v, dtype, 64, defer=defer)
    oc = hz.make_oracle_cache(base.k, base.v, dtype, 64, defer=defer)
    for step in range(37):
        _, kn, vn = synth.decode_step_inputs(base, step, dtype=dtype)
        cc.append_token(hz.to_dev(kn, dtype), hz.to_dev(vn, dtype))
        oc.append_token(kn, vn)
        if step in (0, 4, 15, 16, 31, 36):
            torch.cuda.synchronize()
            hz.compare_caches(cc, oc, f"append[{dtype},defer={defer}] step {step}")
    with pytest.raises(ValueError):
        for _ in range(64):
            cc.append_token(hz.to_dev(kn, dtype), hz.to_dev(vn, dtype))


def test_empty_prefill_then_appends():
    """A cache that starts empty: every block arrives through append_token."""
    dtype = "bfloat16"
    base = synth.make_layer_inputs(103, 16, kv_heads=2, gqa_group=4, dtype=dtype)
    cc = hz.make_cuda_cache(base.k[:, :0], base.v[:, :0], dtype, 80)
    oc = hz.make_oracle_cache(base.k[:, :0], base.v[:, :0], dtype, 80)
    knobs = _knobs(exploration_rate=0.0)
    for step in range(50):
        q, kn, vn = synth.decode_step_inputs(base, step, dtype=dtype)
        cc.append_token(hz.to_dev(kn, dtype), hz.to_dev(vn, dtype))
        oc.append_token(kn, vn)
        if step in (15, 16, 30, 31, 47, 49):   # nq = 1, 1, 1, 2, 3, 3 with trailing 0,1,15,0,0,2
            hz.compare_caches(cc, oc, f"step {step}")
            R = orc.layer_step(oc, q, 4, **_oracle_knobs(knobs, None))
            out, _ = hz.cuda_step(cc, q, dtype, 4, knobs)
            hz.compare_step(cc, R, out, f"empty-start step {step}")


@pytest.mark.parametrize("name", gc.available(gc.SMALL_CASES + gc.LARGE_CASES))
def test_golden_case_cuda(name):
    """CUDA against the oracle (bit-exact) and against the reference's stored results."""
    spec, z = gc.load(name)
    H = spec["kv_heads"] * spec["gqa_group"]
    dtype = spec["dtype"]
    oracle_cache = {}

    def mk(k, v, dt, max_new):
        oracle_cache["c"] = hz.make_oracle_cache(k, v, dt, max_new)
        return hz.make_cuda_cache(k, v, dt, max_new)

    def app(cache, k, v):
        cache.append_token(hz.to_dev(k, dtype), hz.to_dev(v, dtype))
        oracle_cache["c"].append_token(k, v)

    def call(cache, q, target, knobs):
        oc = oracle_cache["c"]
        hz.compare_caches(cache, oc, f"{name} call{target}")
        check_cache_snapshot(oc, z, f"call{target}/cache")
        u = gc.exploration_uniforms(spec, target, H, cache.num_quantized_blocks)
        R = orc.layer_step(oc, q, spec["gqa_group"], **_oracle_knobs(knobs, u))
        out, stats = hz.cuda_step(cache, q, dtype, spec["gqa_group"], knobs, u)
        hz.compare_step(cache, R, out, f"{name} call{target}")
        # the oracle result is itself pinned to the reference's golden values
        check_call(R, z, f"call{target}", H, cache.num_quantized_blocks, cache.active_blocks)
        ref_stats = json.loads(str(z[f"call{target}/stats"]))
        for key in ("k_star_min", "k_star_max", "rung1_fired", "rung2_fired", "rung3_fired", "rung4_fired",
                    "v_format", "exploration_blocks", "skipped_blocks", "attended_blocks", "total_blocks",
                    "rung1_triggered_heads", "ranking_k", "boundary_check_triggered_heads"):
            if key in ref_stats:
                assert stats[key] == ref_stats[key], f"stats[{key}]: {stats[key]} vs reference {ref_stats[key]}"
        for key in ("value_fallback_blocks", "value_fallback_head_blocks"):
            assert stats.get(key, 0) == ref_stats.get(key, 0), key
        ref_out = z[f"call{target}/output"].astype(np.float64)
        scale = np.abs(ref_out).max(axis=1, keepdims=True)
        assert np.all(np.abs(out - ref_out) <= hz.OUT_RTOL * scale), "output vs reference out of tolerance"
        return R

    for target, cache, R in gc.replay(spec, mk, app, call):
        pass


@pytest.mark.parametrize("n_tokens,planted,dtype,seed", [
    (32768 + 5, 64, "bfloat16", 7),      # the 32K single-GPU configuration plus a trailing partial block
    (16384, 0, "float16", 8),            # diffuse attention: K* pinned, nearly every value block promoted
])
def test_layer_step_vs_oracle_large(n_tokens, planted, dtype, seed):
    base = synth.make_layer_inputs(seed, n_tokens, dtype=dtype, n_planted_blocks=planted)
    aligned = (n_tokens // 16) * 16
    cc = hz.make_cuda_cache(base.k[:, :aligned], base.v[:, :aligned], dtype, 64)
    oc = hz.make_oracle_cache(base.k[:, :aligned], base.v[:, :aligned], dtype, 64)
    for t in range(aligned, n_tokens):
        cc.append_token(hz.to_dev(base.k[:, t:t + 1], dtype), hz.to_dev(base.v[:, t:t + 1], dtype))
        oc.append_token(base.k[:, t:t + 1], base.v[:, t:t + 1])
    hz.compare_caches(cc, oc, "large prefill")
    rng = np.random.default_rng(seed)
    u = rng.random((32, oc.num_quantized_blocks), dtype=np.float32)
    knobs = _knobs()
    R = orc.layer_step(oc, base.q, 4, **_oracle_knobs(knobs, u))
    out, stats = hz.cuda_step(cc, base.q, dtype, 4, knobs, u)
    err = hz.compare_step(cc, R, out, f"large N={n_tokens}")
    print(f"N={n_tokens} planted={planted}: k*={stats['k_star_mean']:.1f} rung1={stats['rung1_triggered_heads']} "
          f"value_fallback_blocks={stats.get('value_fallback_blocks', 0)} out_err={err:.2e}")


def test_full_size_128k_needles_vs_oracle():
    """The long-context retrieval shape at full size: 131072 tokens, ten needle blocks (cosine 0.95) at depths
    0.0 .. 0.9 among N(0,1) distractors.  Scores, selections and certificates bit-exact against the oracle, output
    within 1e-3; and the size-independent properties of the step: every head's mass fractions sum to one, the
    sorted cumulative mass is non-decreasing, and every needle block outranks every distractor block in the mass
    ranking of the query head it was planted for."""
    dtype = "bfloat16"
    n_tokens = 131072
    depths = [i / 10.0 for i in range(10)]
    base = synth.make_layer_inputs(77, n_tokens, dtype=dtype, n_planted_blocks=10, planted_cos=0.95,
                                   planted_depths=depths)
    cc = hz.make_cuda_cache(base.k, base.v, dtype, 64)
    oc = hz.make_oracle_cache(base.k, base.v, dtype, 64)
    hz.compare_caches(cc, oc, "128K prefill")
    knobs = _knobs(exploration_rate=0.0)
    R = orc.layer_step(oc, base.q, 4, **_oracle_knobs(knobs, None))
    out, stats = hz.cuda_step(cc, base.q, dtype, 4, knobs, None)
    err = hz.compare_step(cc, R, out, "128K needles")
    assert err < 1e-3
    ws = cc._certified_workspace["cqa_ws"]
    nq = cc.num_quantized_blocks
    frac = ws.mass_frac[:, :nq].double().cpu().numpy()
    assert np.allclose(frac.sum(axis=1), 1.0, atol=1e-4)
    cum = ws.sorted_cumsum.cpu().numpy()
    assert (np.diff(cum, axis=1) >= 0).all()
    planted = np.asarray(base.planted_blocks)
    assert len(planted) == 10
    others = np.ones(nq, dtype=bool)
    others[planted] = False
    for i, blk in enumerate(planted):
        for kv in range(8):
            h = int(base.planted_heads[i, kv])
            assert frac[h, blk] > frac[h, others].max(), f"needle block {blk} does not outrank the distractors of head {h}"
    print(f"128K needles: k*={stats['k_star_mean']:.1f} out_err={err:.2e}")


def test_maximum_size_and_one_block_more():
    """The selector's limit: 16384 quantised blocks (262144 tokens; every thread of a selector CTA owns 16 blocks),
    here with two KV heads, exploration on and a trailing partial block.  Bit-exact against the oracle like any other
    size; one block more is refused with CQA_ERR_TOO_LARGE before anything is launched."""
    dtype = "bfloat16"
    n_tokens = 16384 * 16 + 5
    base = synth.make_layer_inputs(78, n_tokens + 16, kv_heads=2, dtype=dtype, n_planted_blocks=24)
    cc = hz.make_cuda_cache(base.k[:, :16384 * 16], base.v[:, :16384 * 16], dtype, 48)
    oc = hz.make_oracle_cache(base.k[:, :16384 * 16], base.v[:, :16384 * 16], dtype, 48)
    for t in range(16384 * 16, n_tokens):
        cc.append_token(hz.to_dev(base.k[:, t:t + 1], dtype), hz.to_dev(base.v[:, t:t + 1], dtype))
        oc.append_token(base.k[:, t:t + 1], base.v[:, t:t + 1])
    knobs = _knobs()
    rng = np.random.default_rng(78)
    u = rng.random((8, oc.num_quantized_blocks), dtype=np.float32)
    R = orc.layer_step(oc, base.q, 4, **_oracle_knobs(knobs, u))
    out, stats = hz.cuda_step(cc, base.q, dtype, 4, knobs, u)
    err = hz.compare_step(cc, R, out, "16384 blocks")
    assert err < 1e-3
    # eleven more tokens complete block 16385: beyond the limit
    for t in range(n_tokens, n_tokens + 11):
        cc.append_token(hz.to_dev(base.k[:, t:t + 1], dtype), hz.to_dev(base.v[:, t:t + 1], dtype))
    assert cc.num_quantized_blocks == 16385
    from cqa_b200 import _lib
    before = _lib.lib().cqa_launch_count(0)
    with pytest.raises((ValueError, RuntimeError), match="exceed the limit"):
        hz.cuda_step(cc, base.q, dtype, 4, knobs, None)
    assert _lib.lib().cqa_launch_count(0) == before


def test_exact_ties_take_lowest_block_ids():
    """Every 16-token block repeats the same keys and values, so all mass fractions and all value-error
    terms tie exactly: the selector, the top-4 list and the value check must break the ties by block id
    exactly as the oracle does (512 blocks, more than the 256 candidates the selector keeps)."""
    dtype = "bfloat16"
    base = synth.make_layer_inputs(21, 8192, dtype=dtype, n_planted_blocks=0)
    k = np.tile(base.k[:, :16], (1, 512, 1)).copy()
    v = np.tile(base.v[:, :16], (1, 512, 1)).copy()
    # a second family of blocks so that two distinct tied values exist
    k[:, 4096:] = np.tile(base.k[:, 16:32], (1, 256, 1))
    v[:, 4096:] = np.tile(base.v[:, 16:32], (1, 256, 1))
    cc = hz.make_cuda_cache(k, v, dtype, 64)
    oc = hz.make_oracle_cache(k, v, dtype, 64)
    rng = np.random.default_rng(21)
    u = rng.random((32, oc.num_quantized_blocks), dtype=np.float32)
    for knobs in (_knobs(), _knobs(v_tolerance=0.0), _knobs(k_max=None, rung1_threshold=-1.0)):
        R = orc.layer_step(oc, base.q, 4, **_oracle_knobs(knobs, u))
        out, _ = hz.cuda_step(cc, base.q, dtype, 4, knobs, u)
        hz.compare_step(cc, R, out, f"ties {knobs['v_tolerance']} {knobs['k_max']}")


@pytest.mark.parametrize("kcap,vcap,planted", [(48, 48, 16), (8, 300, 0), (2000, 24, 8)])
def test_bounded_hot_tier_equals_full_mirror(kcap, vcap, planted):
    """Tier 2 in pinned host memory with a small device scratch: non-resident blocks are read from the backing
    arrays, used blocks are paged in after the step, slots are recycled.  Outputs, certificates and cache bytes
    equal the full-mirror run bit for bit; the scratch always mirrors the backing rows of the blocks it holds."""
    from dotcache.kernels.tiered_kv_cache import TieredKeyCacheLayer

    dtype = "bfloat16"
    n = 4096 + 7
    base = synth.make_layer_inputs(19, n, dtype=dtype, n_planted_blocks=planted)
    aligned = 4096
    knobs = _knobs(exploration_rate=0.02)
    full = hz.make_cuda_cache(base.k[:, :aligned], base.v[:, :aligned], dtype, 96, defer=False)
    kd, vd = hz.to_dev(base.k[:, :aligned], dtype), hz.to_dev(base.v[:, :aligned], dtype)
    hot = TieredKeyCacheLayer.from_fp16_cache_int4v(kd, vd, max_new_tokens=96, max_pagein_blocks=32,
                                                    fp16_key_cache_capacity=kcap, fp16_value_cache_capacity=vcap)
    assert hot.bounded_hot_tier and hot.keys_fp16_cpu.is_pinned()
    assert hot.keys_fp16_gpu.shape[1] == min(kcap, 262) * 16 and hot.values_fp16_gpu.shape[1] == min(vcap, 262) * 16
    for t in range(aligned, n):
        for c in (full, hot):
            c.append_token(hz.to_dev(base.k[:, t:t + 1], dtype), hz.to_dev(base.v[:, t:t + 1], dtype))
    rng = np.random.default_rng(19)
    for step in range(40):
        q, kn, vn = synth.decode_step_inputs(base, step, dtype=dtype)
        for c in (full, hot):
            c.append_token(hz.to_dev(kn, dtype), hz.to_dev(vn, dtype))
        u = rng.random((32, full.num_quantized_blocks), dtype=np.float32)
        o_full, _ = hz.cuda_step(full, q, dtype, 4, knobs, u, collect_stats=False)
        o_hot, _ = hz.cuda_step(hot, q, dtype, 4, knobs, u, collect_stats=False)
        assert np.array_equal(o_full, o_hot), f"step {step}"
        cf, ff = full._certified_workspace["cqa_ws"].read_cert()
        ch, fh = hot._certified_workspace["cqa_ws"].read_cert()
        assert ff[:5] == fh[:5]
        for key in cf:
            assert np.array_equal(np.asarray(cf[key]).view(np.uint8), np.asarray(ch[key]).view(np.uint8)), key
    for name in ("keys_int8", "keys_scale", "values_int4_packed", "values_int4_scales", "values_int4_errors"):
        assert torch.equal(getattr(full, name), getattr(hot, name)), name
    nt = full.num_tokens
    assert torch.equal(full.keys_fp16_gpu[:, :nt].cpu(), hot.keys_fp16_cpu[:, :nt])
    assert torch.equal(full.values_fp16_gpu[:, :nt].cpu(), hot.values_fp16_cpu[:, :nt])
    torch.cuda.synchronize()
    for tier, slots, owner, gpu, cpu_t in (("key", "key_slots", "key_owner", hot.keys_fp16_gpu, hot.keys_fp16_cpu),
                                           ("value", "value_slots", "value_owner", hot.values_fp16_gpu,
                                            hot.values_fp16_cpu)):
        sl = hot._hot[slots].cpu().numpy()
        ow = hot._hot[owner].cpu().numpy()
        res = np.nonzero(sl >= 0)[0]
        assert len(res) > 0
        for b in res:
            assert ow[sl[b]] == b, f"{tier}: owner table disagrees for block {b}"
            lo = b * 16
            hi = min(lo + 16, nt)
            assert torch.equal(gpu[:, sl[b] * 16: sl[b] * 16 + (hi - lo)].cpu(), cpu_t[:, lo:hi]), f"{tier} block {b}"
        assert len(set(sl[res].tolist())) == len(res), f"{tier}: two blocks share a slot"
    ctr = hot.hot_tier_counters()
    assert ctr["steps"] == 40 and ctr["key_misses"] > 0 and ctr["key_pageins"] > 0 and ctr["value_pageins"] >= 0
    assert ctr["key_hits"] > 0, ctr
    # a slot used in the current step is never recycled, so a scratch smaller than one step's working set
    # fills once and then serves hits; misses beyond it are read from the backing arrays every step
    assert ctr["key_pageins"] - ctr["key_evictions"] <= min(kcap, 262)
    assert ctr["value_pageins"] - ctr["value_evictions"] <= min(vcap, 262)


def test_decode_step_from_host_buffers_equals_two_calls():
    """cqa_decode_step_host (pinned host inputs, one library call) gives the bytes and rows of
    append_token + certified_attention_layer."""
    from dotcache.kernels import certified_attention as ca

    dtype = "bfloat16"
    base = synth.make_layer_inputs(17, 4096 + 9, dtype=dtype, n_planted_blocks=8)
    aligned = 4096
    knobs = _knobs(exploration_rate=0.0)
    ca_a = hz.make_cuda_cache(base.k[:, :aligned], base.v[:, :aligned], dtype, 64)
    ca_b = hz.make_cuda_cache(base.k[:, :aligned], base.v[:, :aligned], dtype, 64)
    for t in range(aligned, 4096 + 9):
        for c in (ca_a, ca_b):
            c.append_token(hz.to_dev(base.k[:, t:t + 1], dtype), hz.to_dev(base.v[:, t:t + 1], dtype))
    qkv = torch.empty((32 + 16) * 128, dtype=torch.bfloat16).pin_memory()
    out_host = torch.empty(32, 128, dtype=torch.float32).pin_memory()
    for step in range(20):
        q, kn, vn = synth.decode_step_inputs(base, step, dtype=dtype)
        ca_a.append_token(hz.to_dev(kn, dtype), hz.to_dev(vn, dtype))
        ref, _ = hz.cuda_step(ca_a, q, dtype, 4, knobs, None, collect_stats=False)
        qkv[: 32 * 128] = torch.from_numpy(q).to(torch.bfloat16).reshape(-1)
        qkv[32 * 128: 40 * 128] = torch.from_numpy(kn).to(torch.bfloat16).reshape(-1)
        qkv[40 * 128:] = torch.from_numpy(vn).to(torch.bfloat16).reshape(-1)
        ca.certified_decode_step_host(ca_b, qkv, 4, out_host, **knobs)
        assert ca_b.num_tokens == ca_a.num_tokens and ca_b.num_quantized_blocks == ca_a.num_quantized_blocks
        assert np.array_equal(out_host.numpy(), ref), f"step {step}"
    for name in ("keys_int8", "values_int4_packed", "keys_scale", "values_int4_errors"):
        assert torch.equal(getattr(ca_a, name), getattr(ca_b, name)), name


def test_decode_step_async_layers_one_wait_per_token():
    """cqa_decode_step_host_async queued for three layer caches and waited for once, and cqa_decode_token_host
    (the loop over the layers inside the library), give each layer the rows of the waiting entry point (stream
    order alone protects the shared staging and the copies)."""
    from dotcache.kernels import certified_attention as ca

    dtype = "bfloat16"
    knobs = _knobs(exploration_rate=0.0)
    bases = [synth.make_layer_inputs(31 + l, 4096, dtype=dtype, n_planted_blocks=8) for l in range(3)]
    sync_caches = [hz.make_cuda_cache(b.k, b.v, dtype, 64) for b in bases]
    async_caches = [hz.make_cuda_cache(b.k, b.v, dtype, 64) for b in bases]
    token_caches = [hz.make_cuda_cache(b.k, b.v, dtype, 64) for b in bases]
    n_in = (32 + 16) * 128
    qkv = torch.empty(3, n_in, dtype=torch.bfloat16).pin_memory()
    out_sync = torch.empty(3, 32, 128, dtype=torch.float32).pin_memory()
    out_async = torch.empty(3, 32, 128, dtype=torch.float32).pin_memory()
    out_token = torch.empty(3, 32, 128, dtype=torch.float32).pin_memory()
    for step in range(18):
        for l, b in enumerate(bases):
            q, kn, vn = synth.decode_step_inputs(b, step, dtype=dtype)
            qkv[l, : 32 * 128] = torch.from_numpy(q).to(torch.bfloat16).reshape(-1)
            qkv[l, 32 * 128: 40 * 128] = torch.from_numpy(kn).to(torch.bfloat16).reshape(-1)
            qkv[l, 40 * 128:] = torch.from_numpy(vn).to(torch.bfloat16).reshape(-1)
        out_async.fill_(float("nan"))
        for l in range(3):
            ca.certified_decode_step_host(async_caches[l], qkv[l], 4, out_async[l], wait=False, **knobs)
        torch.cuda.current_stream().synchronize()
        for l in range(3):
            ca.certified_decode_step_host(sync_caches[l], qkv[l], 4, out_sync[l], **knobs)
        assert np.array_equal(out_async.numpy(), out_sync.numpy()), f"step {step}"
        # the same token through the one-call-per-token entry point
        out_token.fill_(float("nan"))
        ca.certified_decode_token_host(token_caches, qkv, 4, out_token, **knobs)
        assert np.array_equal(out_token.numpy(), out_sync.numpy()), f"token call, step {step}"
    for a, b, c in zip(async_caches, sync_caches, token_caches):
        assert a.num_tokens == b.num_tokens == c.num_tokens
        assert torch.equal(a.keys_int8, b.keys_int8) and torch.equal(c.keys_int8, b.keys_int8)
        assert torch.equal(c.values_int4_packed, b.values_int4_packed)


def test_in_kernel_exploration_draw():
    """Without uniforms or a generator the selector draws its own: the rate is respected, the draw is a function
    of torch's seed, the workspace's serial number (so the layers of a model differ) and the per-cache call counter
    only, and explored blocks are never blocks the selector chose."""
    dtype = "bfloat16"
    base = synth.make_layer_inputs(13, 16384, dtype=dtype, n_planted_blocks=32)
    knobs = _knobs(exploration_rate=0.05)
    masks = []
    from dotcache.kernels import certified_attention as ca
    for rep in range(3):
        torch.manual_seed(1234)
        if rep < 2:
            ca._Workspace._serial = 0          # as in a fresh process: the first workspace created
        cc = hz.make_cuda_cache(base.k, base.v, dtype, 16)
        per_call = []
        for call in range(2):
            hz.cuda_step(cc, base.q, dtype, 4, knobs, None)
            ws = cc._certified_workspace["cqa_ws"]
            nq = cc.num_quantized_blocks
            ex = ws.explore_mask[:, :nq].cpu().numpy().astype(bool)
            tk = ws.topk_mask[:, :nq].cpu().numpy().astype(bool)
            cert, _ = ws.read_cert()
            assert (ex <= tk).all(), "explored blocks must be in the key mask"
            assert np.array_equal(ex.sum(axis=1), cert["exploration_blocks"])
            per_call.append(ex)
        masks.append(per_call)
        frac = per_call[0].mean()
        assert 0.035 < frac < 0.065, f"exploration fraction {frac}"
        assert not np.array_equal(per_call[0], per_call[1]), "the call counter must change the draw"
    assert np.array_equal(masks[0][0], masks[1][0]) and np.array_equal(masks[0][1], masks[1][1])
    assert not np.array_equal(masks[2][0], masks[0][0]), "a second workspace (another layer) must draw another set"


def test_decode_loop_bit_exact_selections():
    """48 decode steps (3 block completions) at 4K context: every step's
    selections, flags and appended bytes match the oracle."""
    dtype = "bfloat16"
    base = synth.make_layer_inputs(9, 4096, dtype=dtype, n_planted_blocks=16)
    cc = hz.make_cuda_cache(base.k, base.v, dtype, 64)
    oc = hz.make_oracle_cache(base.k, base.v, dtype, 64)
    knobs = _knobs()
    rng = np.random.default_rng(9)
    for step in range(48):
        q, kn, vn = synth.decode_step_inputs(base, step, dtype=dtype)
        cc.append_token(hz.to_dev(kn, dtype), hz.to_dev(vn, dtype))
        oc.append_token(kn, vn)
        u = rng.random((32, oc.num_quantized_blocks), dtype=np.float32)
        R = orc.layer_step(oc, q, 4, **_oracle_knobs(knobs, u))
        out, _ = hz.cuda_step(cc, q, dtype, 4, knobs, u, collect_stats=(step % 8 == 0))
        hz.compare_step(cc, R, out, f"decode step {step}")
    hz.compare_caches(cc, oc, "after decode loop")


def test_rung3_dense_recompute():
    """ranking_r=4 makes INT8/FP16 ranking disagreements common: the flagged
    heads must come from the dense FP16 recompute, the others from Phase 2."""
    dtype = "bfloat16"
    base = synth.make_layer_inputs(10, 4096 + 7, dtype=dtype)
    al = 4096
    cc = hz.make_cuda_cache(base.k[:, :al], base.v[:, :al], dtype, 32)
    oc = hz.make_oracle_cache(base.k[:, :al], base.v[:, :al], dtype, 32)
    for t in range(al, al + 7):
        cc.append_token(hz.to_dev(base.k[:, t:t + 1], dtype), hz.to_dev(base.v[:, t:t + 1], dtype))
        oc.append_token(base.k[:, t:t + 1], base.v[:, t:t + 1])
    knobs = _knobs(ranking_r=4, exploration_rate=0.0)
    R = orc.layer_step(oc, base.q, 4, **_oracle_knobs(knobs, None))
    assert R["rung3_heads"].size > 0, "test needs at least one flagged head"
    assert R["rung3_heads"].size < 32
    out, stats = hz.cuda_step(cc, base.q, dtype, 4, knobs)
    hz.compare_step(cc, R, out, "rung3")
    assert stats["rung3_fired"] and stats["ranking_fallback_triggered"] == R["rung3_heads"].size
    # "measure" mode detects but does not recompute
    knobs_m = _knobs(ranking_r=4, exploration_rate=0.0, ranking_fallback_mode="measure")
    Rm = orc.layer_step(oc, base.q, 4, **_oracle_knobs(knobs_m, None))
    outm, statsm = hz.cuda_step(cc, base.q, dtype, 4, knobs_m)
    hz.compare_step(cc, Rm, outm, "rung3-measure")
    assert not statsm["rung3_fired"]


def test_rung4_dense_for_all_heads():
    """A negative eps_guard makes the score-consistency check fail on every
    head (host-side fault injection): all heads are recomputed densely."""
    dtype = "float16"
    base = synth.make_layer_inputs(11, 2048, dtype=dtype)
    cc = hz.make_cuda_cache(base.k, base.v, dtype, 32)
    oc = hz.make_oracle_cache(base.k, base.v, dtype, 32)
    knobs = _knobs(eps_guard=-10.0)
    u = np.random.default_rng(1).random((32, 128), dtype=np.float32)
    R = orc.layer_step(oc, base.q, 4, **_oracle_knobs(knobs, u))
    assert R["rung4"]
    out, stats = hz.cuda_step(cc, base.q, dtype, 4, knobs, u)
    hz.compare_step(cc, R, out, "rung4")
    assert stats["rung4_fired"] is True and stats["v_format"] == "fp16" and stats["rung3_fired"] is False


def test_loose_value_mode_and_no_ranking():
    dtype = "bfloat16"
    base = synth.make_layer_inputs(12, 3072, dtype=dtype, n_planted_blocks=8)
    cc = hz.make_cuda_cache(base.k, base.v, dtype, 32)
    oc = hz.make_oracle_cache(base.k, base.v, dtype, 32)
    for kn in (_knobs(value_error_mode="loose", v_tolerance=0.07),
               _knobs(ranking_fallback=False, score_consistency_check=False),
               _knobs(k_max=None, rung1_threshold=0.02),
               _knobs(k_max=16, k_min=4, rung1_multiplier=3.0, tau_cov=0.9)):
        u = np.random.default_rng(2).random((32, 192), dtype=np.float32)
        R = orc.layer_step(oc, base.q, 4, **_oracle_knobs(kn, u))
        out, _ = hz.cuda_step(cc, base.q, dtype, 4, kn, u)
        hz.compare_step(cc, R, out, f"knobs {kn}")


def test_no_stats_path_returns_same_output():
    dtype = "bfloat16"
    base = synth.make_layer_inputs(13, 2048 + 3, dtype=dtype, n_planted_blocks=8)
    cc = hz.make_cuda_cache(base.k[:, :2048], base.v[:, :2048], dtype, 32)
    for t in range(2048, 2051):
        cc.append_token(hz.to_dev(base.k[:, t:t + 1], dtype), hz.to_dev(base.v[:, t:t + 1], dtype))
    knobs = _knobs(exploration_rate=0.0)
    out1, stats = hz.cuda_step(cc, base.q, dtype, 4, knobs, collect_stats=True)
    out2, empty = hz.cuda_step(cc, base.q, dtype, 4, knobs, collect_stats=False)
    assert empty == {} and np.array_equal(out1, out2)
    timings = {}
    out3, _ = hz.cuda_step(cc, base.q, dtype, 4, dict(knobs, phase_timings=timings), collect_stats=False)
    assert np.array_equal(out1, out3)
    assert {"phase1_int8_scoring_us", "adaptive_selection_us", "ranking_check_us", "phase2_fused_attend_us"} <= set(timings)
    for key in ("total_blocks", "skipped_blocks", "skip_rate", "attended_blocks", "v_format", "h2d_total_bytes",
                "vram_fp16_key_cache_bytes", "rung1_fired", "rung2_fired", "rung3_fired", "rung4_fired", "rho_max",
                "eta_int4", "int4_error_bound", "e_val_max", "e_val_pre_rung2_max", "k_star_mean", "tau_cov",
                "tau_cov_actual_mean", "tail_mass_int8_est_max", "exploration_blocks", "v_max_layer",
                "e_key_step_max", "score_consistency_violation_heads", "delta_bound_mean", "ranking_heads_total",
                "ranking_disagree_r1", "ranking_fallback_triggered", "ranking_k", "boundary_check_fired",
                "score_gap_top12_mean", "s_int8_top1_mean", "s_fp16_top1_mean"):
        assert key in stats, key


def test_naive_baseline_matches_oracle_all_int8_int4():
    """Plain INT8K/INT4V attend (no certification) equals Phase 2 with empty masks."""
    dtype = "bfloat16"
    base = synth.make_layer_inputs(14, 2048, dtype=dtype)
    cc = hz.make_cuda_cache(base.k, base.v, dtype, 32)
    oc = hz.make_oracle_cache(base.k, base.v, dtype, 32)
    q = hz.to_dev(base.q, dtype)
    from dotcache.kernels import certified_attention as ca
    out, stats = ca.certified_attention_layer(cc, q, 4, None, False, v_tolerance=0.05, score_consistency_check=False)
    torch.cuda.synchronize()
    z = np.zeros((32, 128), dtype=np.int32)
    ref, _ = orc.attend_mixed(oc, base.q, 4, 1.0 / np.sqrt(128.0), z, z, 128, 16)
    scale = np.abs(ref).max(axis=1, keepdims=True)
    assert stats == {} and np.all(np.abs(out.cpu().numpy() - ref) <= 1e-3 * scale)
