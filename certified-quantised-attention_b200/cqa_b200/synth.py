"""Seeded synthetic workloads for certified quantised decode attention.

Everything here is numpy-only so the CPU oracle, the CUDA path, the golden
generator and the benchmark all see bit-identical inputs for a given seed.
The shapes follow the Llama-3.1-8B attention geometry (32 query heads, 8 KV
heads, head_dim 128); the value distributions are N(0,1) with a few fixed
"outlier" key channels scaled up, optionally with planted high-similarity
key blocks so the attention mass is concentrated the way long-context
retrieval data concentrates it.  These are stand-ins for the public text
corpora the reference measures on; no item of any such corpus is used.
"""
from __future__ import annotations

from dataclasses import dataclass, field

import numpy as np

BLOCK = 16


@dataclass
class LayerInputs:
    """One attention layer's decode inputs (all float32 numpy arrays)."""

    q: np.ndarray            # [H, d] query of the first decode step
    k: np.ndarray            # [KV, N, d]
    v: np.ndarray            # [KV, N, d]
    gqa_group: int
    outlier_channels: np.ndarray        # [KV, n_outlier] int64
    planted_blocks: np.ndarray          # [n_planted] int64 block ids (may be empty)
    planted_heads: np.ndarray           # [n_planted, KV] int64 q-head (absolute) each block targets
    seed: int = 0
    meta: dict = field(default_factory=dict)


def round_to_dtype(x: np.ndarray, dtype: str) -> np.ndarray:
    """Round a float32 array to the value set of `dtype`, returned as float32.

    "bfloat16" is round-to-nearest-even on the upper 16 bits; "float16" uses
    numpy's IEEE half conversion.
    """
    x = np.ascontiguousarray(x, dtype=np.float32)
    if dtype == "float32":
        return x
    if dtype == "float16":
        return x.astype(np.float16).astype(np.float32)
    if dtype == "bfloat16":
        u = x.view(np.uint32).astype(np.uint64)
        rounded = (u + 0x7FFF + ((u >> 16) & 1)) & 0xFFFF0000
        return rounded.astype(np.uint32).view(np.float32).reshape(x.shape)
    raise ValueError(f"unsupported dtype {dtype!r}")


def make_layer_inputs(
    seed: int,
    n_tokens: int,
    *,
    kv_heads: int = 8,
    gqa_group: int = 4,
    head_dim: int = 128,
    dtype: str = "float32",
    n_outlier_channels: int = 4,
    outlier_scale: float = 8.0,
    n_planted_blocks: int = 0,
    planted_cos: float = 0.9,
    planted_depths: list[float] | None = None,
) -> LayerInputs:
    """Build Q/K/V for one layer.

    K, V ~ N(0,1); `n_outlier_channels` key channels per KV head (indices
    drawn once from the seed, fixed over tokens) are multiplied by
    `outlier_scale`.  Planted blocks: `n_planted_blocks` block-aligned
    16-token key blocks whose keys (for every KV head) have cosine
    `planted_cos` to the query of one seeded q-head of that KV head's group:
    k = |k| (cos * q_hat + sqrt(1-cos^2) * n_perp).  `planted_depths`
    (fractions of the context) places them at fixed depths instead of
    seeded positions.
    """
    rng = np.random.default_rng(seed)
    H = kv_heads * gqa_group
    q = rng.standard_normal((H, head_dim), dtype=np.float32)
    k = rng.standard_normal((kv_heads, n_tokens, head_dim), dtype=np.float32)
    v = rng.standard_normal((kv_heads, n_tokens, head_dim), dtype=np.float32)
    out_idx = np.stack(
        [rng.choice(head_dim, size=n_outlier_channels, replace=False) for _ in range(kv_heads)]
    ).astype(np.int64) if n_outlier_channels > 0 else np.zeros((kv_heads, 0), dtype=np.int64)
    for kv in range(kv_heads):
        k[kv][:, out_idx[kv]] *= np.float32(outlier_scale)

    nb = n_tokens // BLOCK
    planted = np.zeros((0,), dtype=np.int64)
    planted_heads = np.zeros((0, kv_heads), dtype=np.int64)
    n_plant = len(planted_depths) if planted_depths is not None else int(n_planted_blocks)
    if n_plant > 0 and nb > 0:
        if planted_depths is not None:
            planted = np.array(
                [min(int(d * nb), nb - 1) for d in planted_depths], dtype=np.int64
            )
        else:
            planted = np.sort(rng.choice(nb, size=min(n_plant, nb), replace=False)).astype(np.int64)
        planted_heads = rng.integers(0, gqa_group, size=(len(planted), kv_heads)).astype(np.int64)
        c = np.float32(planted_cos)
        s = np.float32(np.sqrt(max(0.0, 1.0 - float(planted_cos) ** 2)))
        for i, b in enumerate(planted):
            for kv in range(kv_heads):
                h = kv * gqa_group + int(planted_heads[i, kv])
                planted_heads[i, kv] = h
                qh = q[h]
                q_hat = qh / np.linalg.norm(qh)
                blk = k[kv, b * BLOCK:(b + 1) * BLOCK, :]
                norms = np.linalg.norm(blk, axis=1, keepdims=True)
                perp = blk - (blk @ q_hat)[:, None] * q_hat[None, :]
                perp /= np.maximum(np.linalg.norm(perp, axis=1, keepdims=True), 1e-12)
                k[kv, b * BLOCK:(b + 1) * BLOCK, :] = (
                    norms * (c * q_hat[None, :] + s * perp)
                ).astype(np.float32)

    q = round_to_dtype(q, dtype)
    k = round_to_dtype(k, dtype)
    v = round_to_dtype(v, dtype)
    return LayerInputs(
        q=q, k=k, v=v, gqa_group=gqa_group, outlier_channels=out_idx,
        planted_blocks=planted, planted_heads=planted_heads, seed=seed,
        meta=dict(n_tokens=n_tokens, kv_heads=kv_heads, head_dim=head_dim, dtype=dtype,
                  n_outlier_channels=n_outlier_channels, outlier_scale=outlier_scale,
                  n_planted_blocks=int(len(planted)), planted_cos=planted_cos),
    )


def decode_step_inputs(
    base: LayerInputs, step: int, *, dtype: str = "float32", jitter: float = 0.1
) -> tuple[np.ndarray, np.ndarray, np.ndarray]:
    """Seeded per-step (q_t, k_new, v_new) for a decode loop.

    q_t = |q_0| * normalise(q_0 + jitter * eps_t) keeps planted blocks
    relevant across steps; k_new/v_new are fresh N(0,1) tokens with the same
    outlier channels as the prefill keys.  Shapes: q_t [H,d], k_new/v_new
    [KV,1,d].
    """
    rng = np.random.default_rng([base.seed, 7919, step])
    H, d = base.q.shape
    kv = base.k.shape[0]
    eps = rng.standard_normal((H, d), dtype=np.float32)
    qn = np.linalg.norm(base.q, axis=1, keepdims=True)
    qt = base.q + np.float32(jitter) * eps
    qt = qn * qt / np.linalg.norm(qt, axis=1, keepdims=True)
    k_new = rng.standard_normal((kv, 1, d), dtype=np.float32)
    v_new = rng.standard_normal((kv, 1, d), dtype=np.float32)
    scale = np.float32(base.meta.get("outlier_scale", 8.0))
    for h in range(kv):
        k_new[h][:, base.outlier_channels[h]] *= scale
    return (
        round_to_dtype(qt.astype(np.float32), dtype),
        round_to_dtype(k_new, dtype),
        round_to_dtype(v_new, dtype),
    )
