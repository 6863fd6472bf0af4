"""Helpers shared by the parity tests: rebuild the seeded inputs of a golden
case, replay it through the CPU oracle, and load the stored reference results.

The case specifications live inside each .npz (key "spec") exactly as
tests/golden/make_golden.py wrote them, so the tests need nothing from the
reference checkout.
"""
from __future__ import annotations

import hashlib
import json
import sys
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT / "certified-quantised-attention_b200"))
sys.path.insert(0, str(ROOT))

from cqa_b200 import synth  # noqa: E402

GOLDEN_DIR = Path(__file__).resolve().parent / "golden"

PAPER_KNOBS = dict(
    v_tolerance=0.05, top_k_fp16_keys=4, ranking_fallback=True, ranking_r=1,
    ranking_fallback_mode="full", tau_cov=0.995, k_min=2, k_max=128,
    rung1_threshold=0.02, rung1_multiplier=2.0, score_consistency_check=True,
    eps_guard=0.01, exploration_rate=0.02, value_error_mode="tight",
)

SMALL_CASES = ["small_fp32", "small_vtol0", "planted_bf16_append", "planted_fp16_g2"]
LARGE_CASES = ["config1_8k", "planted_8k_bf16", "planted_32k_bf16"]


def available(names):
    return [n for n in names if (GOLDEN_DIR / f"{n}.npz").exists()]


def load(name: str):
    z = np.load(GOLDEN_DIR / f"{name}.npz", allow_pickle=False)
    spec = json.loads(str(z["spec"]))
    return spec, z


def sha_np(a: np.ndarray) -> str:
    return hashlib.sha256(np.ascontiguousarray(a).tobytes()).hexdigest()


def exploration_uniforms(spec, target: int, H: int, nq: int) -> np.ndarray:
    """The uniforms the reference drew: torch CPU generator seeded per call."""
    import torch

    g = torch.Generator(device="cpu")
    g.manual_seed(1000 + spec["seed"] * 100 + target)
    return torch.rand((H, nq), generator=g).numpy()


def case_inputs(spec):
    return synth.make_layer_inputs(
        spec["seed"], spec["n_tokens"], kv_heads=spec["kv_heads"], gqa_group=spec["gqa_group"],
        dtype=spec["dtype"], n_planted_blocks=spec["planted"],
    )


def knobs_for(spec):
    k = dict(PAPER_KNOBS)
    k.update(spec["knobs"])
    return k


def unpack_mask(packed: np.ndarray, ncols: int) -> np.ndarray:
    return np.unpackbits(packed, axis=1)[:, :ncols].astype(bool)


def replay(spec, make_cache, append, layer_call):
    """Drive a cache implementation through the case's append/call schedule.

    make_cache(k_aligned, v_aligned, dtype, max_new_tokens) -> cache
    append(cache, k_new, v_new) -> None
    layer_call(cache, q, target, knobs) -> result
    Yields ("prefill", cache, None) once the prompt is in, then (target, cache, result).
    """
    base = case_inputs(spec)
    n = spec["n_tokens"]
    aligned = (n // 16) * 16
    max_new = spec["appends"] + 16
    cache = make_cache(base.k[:, :aligned], base.v[:, :aligned], spec["dtype"],
                       max_new + (n - aligned))
    for t in range(aligned, n):
        append(cache, base.k[:, t:t + 1], base.v[:, t:t + 1])
    knobs = knobs_for(spec)
    yield "prefill", cache, None
    step = 0
    for target in spec["call_after"]:
        while step < target:
            _, kn, vn = synth.decode_step_inputs(base, step, dtype=spec["dtype"])
            append(cache, kn, vn)
            step += 1
        q = base.q if target == 0 else synth.decode_step_inputs(base, target - 1, dtype=spec["dtype"])[0]
        yield target, cache, layer_call(cache, q, target, knobs)
