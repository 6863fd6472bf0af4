"""Certified attention for one layer, all heads — B200-native host side.

Mirrors the public surface of the reference's
`dotcache/kernels/certified_attention.py`: `certified_attention_layer`
(:1065-1113) with the same arguments, return value and stats keys
(:2608-2788, Rung-4 variant :1771-1796), and the helper functions other code
imports.  The whole per-layer chain
    Phase-1 INT8 block scores -> adaptive K* (+ Rung 1, exploration)
    -> ranking / boundary / score-consistency checks -> Rung-2 value check
    -> Phase-2 mixed attend -> Rung-3/4 dense recompute -> merge
is four CUDA kernels launched back to back on the current stream by ONE call
into libcqa_b200.so (`cqa_layer_step`), with no host synchronisation; the
certificate lives in a small device struct that is copied to the host only
when `collect_stats` is set.  There is no Triton, PyTorch or CPU compute path.
"""
from __future__ import annotations

import ctypes as C
import math
from typing import Any

import torch

from cqa_b200 import _lib
from dotcache.kernels.tiered_kv_cache import TieredKeyCacheLayer

DEFAULT_V_TOLERANCE = 0.5
TOP_K_BLOCKS = 4
DEFAULT_TAU_COV = 0.995
DEFAULT_K_MIN = 2
DEFAULT_K_MAX: int | None = None
DEFAULT_RUNG1_THRESHOLD = 0.02
DEFAULT_RUNG1_MULTIPLIER = 2.0

_CERT_INT_FIELDS = [f for f, t in _lib.CqaHeadCert._fields_ if t is C.c_int32]
_CERT_F32_FIELDS = [f for f, t in _lib.CqaHeadCert._fields_ if t is C.c_float]


# ----------------------------------------------------------------------------- workspace

class _Workspace:
    """Device buffers for one layer's step, kept in cache._certified_workspace."""

    _serial = 0

    def draw_seed(self) -> int:
        """Key of this workspace's Philox stream: torch.initial_seed() mixed (splitmix64) with the workspace's
        serial number.  Fixed at the first draw."""
        if self.rng_seed is None:
            z = (int(torch.initial_seed()) + 0x9E3779B97F4A7C15 * self.serial) & 0xFFFFFFFFFFFFFFFF
            z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & 0xFFFFFFFFFFFFFFFF
            z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & 0xFFFFFFFFFFFFFFFF
            self.rng_seed = z ^ (z >> 31)
        return self.rng_seed

    def __init__(self, cache: TieredKeyCacheLayer, H: int, G: int, device: torch.device, ld: int | None = None):
        self.H, self.G = H, G
        ld = int(cache.keys_scale.shape[1]) if ld is None else int(ld)
        self.ld = ld
        f32 = dict(dtype=torch.float32, device=device)
        u8 = dict(dtype=torch.uint8, device=device)
        self.m_b = torch.zeros(H, ld, **f32)
        self.s_b = torch.zeros(H, ld, **f32)
        self.token_scores = torch.empty(cache.kv_heads * ld * G * 16, **f32)
        self.mass_frac = torch.zeros(H, ld, **f32)
        self.topk_mask = torch.zeros(H, ld, **u8)
        self.value_mask = torch.zeros(H, ld, **u8)
        self.explore_mask = torch.zeros(H, ld, **u8)
        self.sel_width = 0
        self.sorted_idx = None
        self.sorted_cumsum = None
        ns, ds = C.c_int(0), C.c_int(0)
        with torch.cuda.device(device):
            _lib.check(_lib.lib().cqa_suggest_splits(cache.kv_heads, G, ld, C.byref(ns), C.byref(ds)),
                       "cqa_suggest_splits")
        self.num_splits, self.dense_splits = ns.value, ds.value
        self.part_m = torch.empty(H, self.num_splits, **f32)
        self.part_l = torch.empty(H, self.num_splits, **f32)
        self.part_acc = torch.empty(H, self.num_splits, 128, **f32)
        self.dense_m = torch.empty(H, self.dense_splits, **f32)
        self.dense_l = torch.empty(H, self.dense_splits, **f32)
        self.dense_acc = torch.empty(H, self.dense_splits, 128, **f32)
        # certificate structs followed by the flag words (4 flags, dense-head count and list):
        # one D2H copy reads both
        self.cert_bytes = H * _lib.CERT_BYTES
        self.cert_buf = torch.zeros(self.cert_bytes + 4 * (5 + H), **u8)
        self.out = torch.empty(H, 128, **f32)
        self.tickets = torch.zeros(cache.kv_heads + H, dtype=torch.int32, device=device)
        self.cert_host = None
        self._u_flat = None
        self._step_in = None
        # In-kernel exploration draw: torch's seed mixed with a per-workspace serial number, so that the layers of
        # a model (one workspace each, created in layer order) draw different exploration sets, reproducibly.
        self.rng_seed = None
        self.rng_calls = 0
        _Workspace._serial += 1
        self.serial = _Workspace._serial
        self.struct = _lib.CqaWorkspace()
        self._struct_stale = True

    def ensure_sel_width(self, width: int, device):
        if self.sel_width < width:
            self.sel_width = width
            self.sorted_idx = torch.zeros(self.H, width, dtype=torch.int32, device=device)
            self.sorted_cumsum = torch.zeros(self.H, width, dtype=torch.float32, device=device)

    def step_input_buffer(self, n: int, dtype, device) -> torch.Tensor:
        """Device scratch for the packed (q, k_new, v_new) of cqa_decode_step_host."""
        buf = self._step_in
        if buf is None or buf.numel() != n or buf.dtype != dtype:
            buf = torch.empty(n, dtype=dtype, device=device)
            self._step_in = buf
        return buf

    def uniform_buffer(self, nq: int, device) -> torch.Tensor:
        """A reused [H, nq] float32 view for the exploration draw."""
        if self._u_flat is None or self._u_flat.numel() < self.H * self.ld:
            self._u_flat = torch.empty(self.H * self.ld, dtype=torch.float32, device=device)
        return self._u_flat[: self.H * nq].view(self.H, nq)

    def fill_struct(self, nact: int | None = None) -> _lib.CqaWorkspace:
        """The cqa_workspace struct over these buffers.  Pointers are written once (again after a buffer is
        replaced); per call only the split counts follow `nact`."""
        s = self.struct
        if self._struct_stale:
            s.ld = self.ld
            s.m_b, s.s_b = self.m_b.data_ptr(), self.s_b.data_ptr()
            s.token_scores = self.token_scores.data_ptr()
            s.mass_frac = self.mass_frac.data_ptr()
            s.topk_mask, s.value_mask = self.topk_mask.data_ptr(), self.value_mask.data_ptr()
            s.explore_mask = self.explore_mask.data_ptr()
            s.sorted_idx = _lib.ptr(self.sorted_idx)
            s.sorted_cumsum = _lib.ptr(self.sorted_cumsum)
            s.sel_width = self.sel_width
            s.part_m, s.part_l, s.part_acc = self.part_m.data_ptr(), self.part_l.data_ptr(), self.part_acc.data_ptr()
            s.dense_m, s.dense_l, s.dense_acc = self.dense_m.data_ptr(), self.dense_l.data_ptr(), self.dense_acc.data_ptr()
            s.cert = self.cert_buf.data_ptr()
            s.any_flags = self.cert_buf.data_ptr() + self.cert_bytes
            s.out = self.out.data_ptr()
            s.tickets = self.tickets.data_ptr()
            self._struct_stale = False
        ns, ds = self.num_splits, self.dense_splits
        if nact is not None:
            # never more splits than eight-block groups of work
            ns = max(1, min(ns, (nact + 7) // 8))
            ds = max(1, min(ds, (nact + 15) // 16))
        s.num_splits, s.dense_splits = ns, ds
        return s

    def __setattr__(self, name, value):
        # replacing a buffer (tests and the sharded layer do) makes the cached pointers stale
        if name in ("m_b", "s_b", "token_scores", "mass_frac", "topk_mask", "value_mask", "explore_mask",
                    "sorted_idx", "sorted_cumsum", "part_m", "part_l", "part_acc", "dense_m", "dense_l", "dense_acc",
                    "cert_buf", "out", "tickets", "sel_width"):
            object.__setattr__(self, "_struct_stale", True)
        object.__setattr__(self, name, value)

    def read_cert(self) -> tuple[dict, list]:
        """Copy the certificate structs and flags to the host (synchronises)."""
        host = self.cert_buf.cpu().numpy()
        arr = (_lib.CqaHeadCert * self.H).from_buffer_copy(host[: self.cert_bytes].tobytes())
        import numpy as np

        flags = np.frombuffer(host[self.cert_bytes:].tobytes(), dtype=np.int32).tolist()
        cols: dict[str, Any] = {}
        for f in _CERT_INT_FIELDS + _CERT_F32_FIELDS:
            cols[f] = np.array([getattr(arr[h], f) for h in range(self.H)])
        cols["top_blocks"] = np.array([list(arr[h].top_blocks) for h in range(self.H)])
        cols["fp16_scores"] = np.array([list(arr[h].fp16_scores) for h in range(self.H)], dtype=np.float32)
        cols["fp16_logmass"] = np.array([list(arr[h].fp16_logmass) for h in range(self.H)], dtype=np.float32)
        return cols, flags


def _workspace(cache: TieredKeyCacheLayer, H: int, G: int, device) -> _Workspace:
    ws = cache._certified_workspace.get("cqa_ws")
    if ws is None or ws.H != H or ws.G != G or ws.ld != int(cache.keys_scale.shape[1]):
        ws = _Workspace(cache, H, G, device)
        cache._certified_workspace["cqa_ws"] = ws
    return ws


_KNOBS_CACHE: dict = {}


def _make_knobs(*, q_scale, tau_cov, k_min, k_max, rung1_threshold, rung1_multiplier, eps_guard,
                exploration_rate, v_tolerance, ranking_r, top_k_fp16_keys, ranking_fallback,
                ranking_fallback_mode, score_consistency_check, value_error_mode,
                force_trailing_value_fp16) -> _lib.CqaKnobs:
    """The cqa_knobs struct for these settings (structs are read-only to the library, so one per distinct
    setting is kept and reused)."""
    key = (q_scale, tau_cov, k_min, k_max, rung1_threshold, rung1_multiplier, eps_guard, exploration_rate,
           v_tolerance, ranking_r, top_k_fp16_keys, ranking_fallback, ranking_fallback_mode,
           score_consistency_check, value_error_mode, force_trailing_value_fp16)
    cached = _KNOBS_CACHE.get(key)
    if cached is not None:
        return cached
    if len(_KNOBS_CACHE) > 256:
        _KNOBS_CACHE.clear()
    k = _lib.CqaKnobs()
    k.q_scale = float(q_scale)
    k.tau_cov = float(tau_cov)
    k.rung1_threshold = -1.0 if rung1_threshold is None else float(rung1_threshold)
    k.rung1_multiplier = float(rung1_multiplier)
    k.eps_guard = float(eps_guard)
    k.exploration_rate = float(exploration_rate)
    k.v_tolerance = float(v_tolerance)
    k.k_min = int(k_min)
    k.k_max = 0 if k_max is None else int(k_max)
    k.ranking_r = int(ranking_r)
    k.top_k_fp16_keys = int(top_k_fp16_keys or 0)
    k.ranking_fallback = int(bool(ranking_fallback))
    k.rung3_recompute = int(ranking_fallback_mode == "full")
    k.score_consistency = int(bool(score_consistency_check))
    k.value_mode_tight = int(value_error_mode == "tight")
    k.force_trailing_value_fp16 = int(bool(force_trailing_value_fp16))
    _KNOBS_CACHE[key] = k
    return k


def _selection_width(k_max, rung1_threshold, rung1_multiplier, nq: int) -> int:
    if k_max is None:
        return nq
    w = int(k_max)
    if rung1_threshold is not None and rung1_threshold >= 0:
        w = max(w, min(int(math.ceil(int(k_max) * float(rung1_multiplier))), nq))
    return min(w, nq)


class _PhaseTimer:
    """CUDA-event timing of one phase into `timings[f"{name}_us"]` (reference:
    certified_attention.py:54-80); events are read after one synchronise at the
    end of the layer call."""

    def __init__(self, timings, name, pending):
        self.timings, self.name, self.pending = timings, name, pending

    def __enter__(self):
        if self.timings is not None:
            self.start = torch.cuda.Event(enable_timing=True)
            self.start.record()
        return self

    def __exit__(self, *_):
        if self.timings is not None:
            end = torch.cuda.Event(enable_timing=True)
            end.record()
            self.pending.append((self.name, self.start, end))


# ----------------------------------------------------------------------------- main entry

def certified_decode_step_host(
    cache: TieredKeyCacheLayer,
    qkv_host: torch.Tensor,
    gqa_group: int,
    out_host: torch.Tensor,
    q_scale: float | None = None,
    *,
    v_tolerance: float,
    top_k_fp16_keys: int = 4,
    ranking_fallback: bool = True,
    ranking_r: int = 1,
    ranking_fallback_mode: str = "full",
    tau_cov: float = 0.995,
    k_min: int = DEFAULT_K_MIN,
    k_max: int | None = DEFAULT_K_MAX,
    rung1_threshold: float = DEFAULT_RUNG1_THRESHOLD,
    rung1_multiplier: float = DEFAULT_RUNG1_MULTIPLIER,
    score_consistency_check: bool = False,
    eps_guard: float = 0.01,
    exploration_rate: float = 0.0,
    value_error_mode: str = "tight",
    wait: bool = True,
) -> torch.Tensor:
    """`cache.append_token(k, v)` followed by `certified_attention_layer(cache, q, ...)` for a caller whose step
    inputs live in host memory, as ONE library call (cqa_decode_step_host): `qkv_host` is a pinned 1-D tensor
    [q (H*128) | k_new (KV*128) | v_new (KV*128)] in the cache's model dtype, `out_host` a pinned float32 [H, 128]
    tensor that holds the attention output when the call returns.  An addition (no reference counterpart): it
    removes the interpreter from between the copies and the launches; results equal the two-call sequence.
    With `wait=False` the work is only queued on the current stream (cqa_decode_step_host_async): a decoder calls
    it once per layer, each with its own `qkv_host` and `out_host`, and synchronises the stream once per token."""
    H = cache.kv_heads * int(gqa_group)
    n_in = (H + 2 * cache.kv_heads) * cache.head_dim
    if qkv_host.is_cuda or out_host.is_cuda:
        raise ValueError("certified_decode_step_host takes host tensors (pinned for asynchronous copies)")
    if qkv_host.numel() != n_in or not qkv_host.is_contiguous():
        raise ValueError(f"qkv_host must be a contiguous tensor of {n_in} elements")
    if out_host.dtype != torch.float32 or out_host.numel() != H * cache.head_dim or not out_host.is_contiguous():
        raise ValueError(f"out_host must be a contiguous float32 tensor of {H * cache.head_dim} elements")
    pos = cache.num_tokens
    if pos >= cache.keys_int8.shape[1]:
        raise ValueError(f"cache capacity {cache.keys_int8.shape[1]} exhausted")
    if (pos + 1) // cache.block_size <= 0:
        raise NotImplementedError("the certified path needs at least one complete block")
    device = cache.keys_int8.device
    if q_scale is None:
        q_scale = 1.0 / (cache.head_dim ** 0.5)
    G = int(gqa_group)
    ws = _workspace(cache, H, G, device)
    nq = (pos + 1) // cache.block_size
    knobs = _make_knobs(
        q_scale=q_scale, tau_cov=tau_cov, k_min=k_min, k_max=k_max, rung1_threshold=rung1_threshold,
        rung1_multiplier=rung1_multiplier, eps_guard=eps_guard, exploration_rate=exploration_rate,
        v_tolerance=v_tolerance, ranking_r=ranking_r, top_k_fp16_keys=top_k_fp16_keys,
        ranking_fallback=ranking_fallback, ranking_fallback_mode=ranking_fallback_mode,
        score_consistency_check=score_consistency_check, value_error_mode=value_error_mode,
        force_trailing_value_fp16=True,
    )
    ws.ensure_sel_width(_selection_width(k_max, rung1_threshold, rung1_multiplier, nq), device)
    wstruct = ws.fill_struct((pos + 1 + cache.block_size - 1) // cache.block_size)
    if exploration_rate > 0.0:
        wstruct.rng_seed = ws.draw_seed()
        wstruct.rng_offset = ws.rng_calls
        ws.rng_calls += 1
    stage = ws.step_input_buffer(n_in, qkv_host.dtype, device)
    with _lib.on_device(device):
        entry = _lib.lib().cqa_decode_step_host if wait else _lib.lib().cqa_decode_step_host_async
        _lib.check(entry(
            C.byref(cache._desc(G)), C.byref(knobs), C.byref(wstruct), qkv_host.data_ptr(), stage.data_ptr(),
            _lib.dtype_code(qkv_host.dtype), pos, 1 if cache._defers_int4() else 0, out_host.data_ptr(),
            _lib.current_stream(device)), "cqa_decode_step_host")
        if cache.bounded_hot_tier:
            cache._hot_tier_update(cache._desc(G), wstruct, (pos + 1 + cache.block_size - 1) // cache.block_size,
                                   _lib.current_stream(device))
    cache._advance_after_append(pos)
    return out_host


def certified_decode_token_host(
    caches,
    qkv_host: torch.Tensor,
    gqa_group: int,
    out_host: torch.Tensor,
    q_scale: float | None = None,
    *,
    v_tolerance: float,
    top_k_fp16_keys: int = 4,
    ranking_fallback: bool = True,
    ranking_r: int = 1,
    ranking_fallback_mode: str = "full",
    tau_cov: float = 0.995,
    k_min: int = DEFAULT_K_MIN,
    k_max: int | None = DEFAULT_K_MAX,
    rung1_threshold: float = DEFAULT_RUNG1_THRESHOLD,
    rung1_multiplier: float = DEFAULT_RUNG1_MULTIPLIER,
    score_consistency_check: bool = False,
    eps_guard: float = 0.01,
    exploration_rate: float = 0.0,
    value_error_mode: str = "tight",
) -> torch.Tensor:
    """`certified_decode_step_host` for every layer of a model in ONE library call (cqa_decode_token_host):
    `caches` is the list of the layers' caches, `qkv_host` a pinned [L, (H + 2 KV) * 128] tensor, `out_host` a
    pinned float32 [L, H, 128] tensor that holds every layer's attention rows when the call returns.  The loop over
    the layers runs inside the library, all inputs are copied before the first kernel, Phase 2 writes into `out_host`
    directly when it is pinned, and the stream is waited for once.  Row l equals what
    `certified_decode_step_host(caches[l], qkv_host[l], ...)` returns.  An addition (no reference counterpart)."""
    n_layers = len(caches)
    if n_layers == 0:
        raise ValueError("certified_decode_token_host needs at least one layer cache")
    first = caches[0]
    G = int(gqa_group)
    H = first.kv_heads * G
    n_in = (H + 2 * first.kv_heads) * first.head_dim
    if qkv_host.is_cuda or out_host.is_cuda:
        raise ValueError("certified_decode_token_host takes host tensors (pinned for asynchronous copies)")
    if qkv_host.numel() != n_layers * n_in or not qkv_host.is_contiguous():
        raise ValueError(f"qkv_host must be a contiguous [{n_layers}, {n_in}] tensor")
    if (out_host.dtype != torch.float32 or out_host.numel() != n_layers * H * first.head_dim
            or not out_host.is_contiguous()):
        raise ValueError(f"out_host must be a contiguous float32 [{n_layers}, {H}, {first.head_dim}] tensor")
    device = first.keys_int8.device
    if q_scale is None:
        q_scale = 1.0 / (first.head_dim ** 0.5)
    knobs = _make_knobs(
        q_scale=q_scale, tau_cov=tau_cov, k_min=k_min, k_max=k_max, rung1_threshold=rung1_threshold,
        rung1_multiplier=rung1_multiplier, eps_guard=eps_guard, exploration_rate=exploration_rate,
        v_tolerance=v_tolerance, ranking_r=ranking_r, top_k_fp16_keys=top_k_fp16_keys,
        ranking_fallback=ranking_fallback, ranking_fallback_mode=ranking_fallback_mode,
        score_consistency_check=score_consistency_check, value_error_mode=value_error_mode,
        force_trailing_value_fp16=True,
    )
    # the array of per-layer call records is kept on the first cache and rebuilt when the set of layers changes
    key = (tuple(id(c) for c in caches), G)
    plan = getattr(first, "_decode_token_plan", None)
    if plan is not None and any(c._certified_workspace.get("cqa_ws") is not w for c, w in zip(caches, plan[2])):
        plan = None   # a layer's workspace was replaced since the records were built
    if plan is None or plan[0] != key:
        calls = (_lib.CqaLayerCall * n_layers)()
        spaces = []
        for l, cache in enumerate(caches):
            if (cache.kv_heads, cache.head_dim, cache.keys_int8.device) != (first.kv_heads, first.head_dim, device):
                raise ValueError("all layer caches must share geometry and device")
            ws = _workspace(cache, H, G, device)
            spaces.append(ws)
            calls[l].cache = C.addressof(cache._desc(G))
            calls[l].ws = C.addressof(ws.struct)
        plan = (key, calls, spaces, torch.empty(n_layers * n_in, dtype=qkv_host.dtype, device=device))
        first._decode_token_plan = plan
    _, calls, spaces, stage = plan
    if stage.dtype != qkv_host.dtype:
        raise ValueError("qkv_host changed dtype between calls")
    block = first.block_size
    in_bytes = n_in * qkv_host.element_size()
    out_bytes = H * first.head_dim * 4
    qkv_base, out_base = qkv_host.data_ptr(), out_host.data_ptr()
    explore = exploration_rate > 0.0
    last_pos, width = -1, 0
    positions = []
    for l, cache in enumerate(caches):
        pos = cache.num_tokens
        if pos != last_pos:   # layers of one model normally hold the same number of tokens
            if pos >= cache.keys_int8.shape[1]:
                raise ValueError(f"cache capacity {cache.keys_int8.shape[1]} exhausted")
            nq = (pos + 1) // block
            if nq <= 0:
                raise NotImplementedError("the certified path needs at least one complete block")
            width = _selection_width(k_max, rung1_threshold, rung1_multiplier, nq)
            nblocks = (pos + block) // block
            last_pos = pos
        elif pos >= cache.keys_int8.shape[1]:
            raise ValueError(f"cache capacity {cache.keys_int8.shape[1]} exhausted")
        positions.append(pos)
        ws = spaces[l]
        if ws.sel_width < width:
            ws.ensure_sel_width(width, device)
        wstruct = ws.fill_struct(nblocks)
        if explore:
            wstruct.rng_seed = ws.draw_seed()
            wstruct.rng_offset = ws.rng_calls
            ws.rng_calls += 1
        call = calls[l]
        call.cache = C.addressof(cache._desc(G))
        call.qkv_host = qkv_base + l * in_bytes
        call.out_host = out_base + l * out_bytes
        call.pos = pos
        call.defer_int4 = 1 if cache._defers_int4() else 0
    stream = _lib.current_stream(device)
    with _lib.on_device(device):
        _lib.check(_lib.lib().cqa_decode_token_host(calls, n_layers, C.byref(knobs), stage.data_ptr(),
                                                    _lib.dtype_code(qkv_host.dtype), stream), "cqa_decode_token_host")
        for l, cache in enumerate(caches):
            if cache.bounded_hot_tier:
                cache._hot_tier_update(cache._desc(G), spaces[l].struct, (positions[l] + block) // block, stream)
    for l, cache in enumerate(caches):
        cache._advance_after_append(positions[l])
    return out_host


def _batch_splits(slots: int, heads: int, nact: int, limit: int) -> int:
    """Phase-2 splits per (sequence, KV head) of a batch: the count that minimises (waves of `slots` resident CTAs)
    x (blocks per CTA + the fixed cost of a CTA, worth about 64 blocks: merges, partial rows, ticket).  Rounding the
    per-head share UP to fill the GPU puts a few CTAs into a second, nearly empty wave; this picks the lower count or
    a multi-wave split instead."""
    best_p, best = 1, None
    for p in range(1, max(1, min(limit, nact // 8 if nact >= 8 else 1)) + 1):
        waves = -(-heads * p // slots)
        cost = waves * (-(-nact // p) + 64)
        if best is None or cost < best:
            best_p, best = p, cost
    return best_p


def certified_attention_batch(
    caches,
    q_all: torch.Tensor,
    gqa_group: int,
    q_scale: float | None = None,
    *,
    new_keys: torch.Tensor | None = None,
    new_values: torch.Tensor | None = None,
    num_splits: int | None = None,
    v_tolerance: float,
    top_k_fp16_keys: int = 4,
    ranking_fallback: bool = True,
    ranking_r: int = 1,
    ranking_fallback_mode: str = "full",
    tau_cov: float = 0.995,
    k_min: int = DEFAULT_K_MIN,
    k_max: int | None = DEFAULT_K_MAX,
    rung1_threshold: float = DEFAULT_RUNG1_THRESHOLD,
    rung1_multiplier: float = DEFAULT_RUNG1_MULTIPLIER,
    score_consistency_check: bool = False,
    eps_guard: float = 0.01,
    exploration_rate: float = 0.0,
    value_error_mode: str = "tight",
) -> torch.Tensor:
    """One certified decode step of one layer for a BATCH of sequences, each with its own cache: the (optional)
    append and the three kernels of the step run once, with the sequences on the grid (cqa_layer_step_batched).
    The reference is batch-1 only (its adapter raises otherwise, integrations/llama.py:717-718); a caller with B
    sequences would loop.  An addition, no reference counterpart.

    `caches`: the B layer caches (same head geometry and dtype; lengths may differ).  `q_all`: [B, H, 128] on the
    GPU in the caches' dtype (or float32).  `new_keys` / `new_values`: [B, KV, 128]; when given, every sequence's
    token is appended first (`cache.append_token`) inside the same call.  Returns float32 [B, H, 128]; row b equals
    what `certified_attention_layer(caches[b], q_all[b], ...)` returns when both use the same `num_splits` (the
    split count fixes the summation order of Phase 2).  The tensor is reused by the next call with the same caches.
    Certificates stay in each cache's workspace (`cache._certified_workspace["cqa_ws"].read_cert()`)."""
    B = len(caches)
    if B == 0:
        raise ValueError("certified_attention_batch needs at least one cache")
    if not q_all.is_cuda:
        raise RuntimeError("certified_attention_batch needs CUDA tensors; there is no CPU fallback")
    first = caches[0]
    G = int(gqa_group)
    H = first.kv_heads * G
    KV = first.kv_heads
    if tuple(q_all.shape) != (B, H, first.head_dim):
        raise ValueError(f"q_all must have shape {(B, H, first.head_dim)}, got {tuple(q_all.shape)}")
    do_append = new_keys is not None
    if do_append != (new_values is not None):
        raise ValueError("new_keys and new_values go together")
    if do_append and (tuple(new_keys.shape) != (B, KV, first.head_dim) or tuple(new_values.shape) != (B, KV, first.head_dim)):
        raise ValueError(f"new_keys / new_values must have shape {(B, KV, first.head_dim)}")
    device = q_all.device
    if q_scale is None:
        q_scale = 1.0 / (first.head_dim ** 0.5)
    q = q_all.contiguous()
    if do_append:
        new_keys = new_keys.to(q.dtype).contiguous()
        new_values = new_values.to(q.dtype).contiguous()
    knobs = _make_knobs(
        q_scale=q_scale, tau_cov=tau_cov, k_min=k_min, k_max=k_max, rung1_threshold=rung1_threshold,
        rung1_multiplier=rung1_multiplier, eps_guard=eps_guard, exploration_rate=exploration_rate,
        v_tolerance=v_tolerance, ranking_r=ranking_r, top_k_fp16_keys=top_k_fp16_keys,
        ranking_fallback=ranking_fallback, ranking_fallback_mode=ranking_fallback_mode,
        score_consistency_check=score_consistency_check, value_error_mode=value_error_mode,
        force_trailing_value_fp16=True,
    )
    key = (tuple(id(c) for c in caches), G)
    plan = getattr(first, "_batch_plan", None)
    if plan is None or plan[0] != key:
        items = (_lib.CqaBatchItem * B)()
        items_dev = torch.empty(C.sizeof(items) + 16, dtype=torch.uint8, device=device)
        out = torch.empty(B, H, first.head_dim, dtype=torch.float32, device=device)
        plan = (key, items, items_dev, out)
        first._batch_plan = plan
    _, items, items_dev, out = plan
    esz = q.element_size()
    row_q, row_kv = H * first.head_dim * esz, KV * first.head_dim * esz
    block = first.block_size
    sms = torch.cuda.get_device_properties(device).multi_processor_count
    positions = []
    for b, cache in enumerate(caches):
        if (cache.kv_heads, cache.head_dim, cache.keys_int8.device) != (KV, first.head_dim, first.keys_int8.device):
            raise ValueError("all caches of a batch must share geometry and device")
        pos = cache.num_tokens
        if do_append and pos >= cache.keys_int8.shape[1]:
            raise ValueError(f"cache capacity {cache.keys_int8.shape[1]} exhausted")
        n_tok = pos + (1 if do_append else 0)
        nq, nact = n_tok // block, (n_tok + block - 1) // block
        if nq <= 0:
            raise NotImplementedError("the certified path needs at least one complete block per sequence")
        ws = _workspace(cache, H, G, device)
        ws.ensure_sel_width(_selection_width(k_max, rung1_threshold, rung1_multiplier, nq), device)
        w = ws.fill_struct(nact)
        # splits per sequence: never more than the sequence's own limit (its partial buffers)
        ns = int(num_splits) if num_splits else _batch_splits(2 * sms, KV * B, nact, w.num_splits)
        w.num_splits = max(1, min(ns, w.num_splits, nact))
        if exploration_rate > 0.0:
            w.rng_seed = ws.draw_seed()
            w.rng_offset = ws.rng_calls
            ws.rng_calls += 1
        it = items[b]
        C.memmove(C.byref(it.cache), C.byref(cache._desc(G)), C.sizeof(_lib.CqaCache))
        C.memmove(C.byref(it.ws), C.byref(w), C.sizeof(_lib.CqaWorkspace))
        it.ws.out = out.data_ptr() + b * H * first.head_dim * 4
        it.q = q.data_ptr() + b * row_q
        it.k_new = new_keys.data_ptr() + b * row_kv if do_append else None
        it.v_new = new_values.data_ptr() + b * row_kv if do_append else None
        it.pos = pos
        it.defer_int4 = 1 if cache._defers_int4() else 0
        positions.append(pos)
    dev_ptr = (items_dev.data_ptr() + 15) & ~15
    stream = _lib.current_stream(device)
    with _lib.on_device(device):
        _lib.check(_lib.lib().cqa_layer_step_batched(items, B, dev_ptr, C.byref(knobs), _lib.dtype_code(q.dtype),
                                                     1 if do_append else 0, stream), "cqa_layer_step_batched")
        for b, cache in enumerate(caches):
            if cache.bounded_hot_tier:
                n_tok = positions[b] + (1 if do_append else 0)
                cache._hot_tier_update(cache._desc(G), items[b].ws, (n_tok + block - 1) // block, stream)
    if do_append:
        for b, cache in enumerate(caches):
            cache._advance_after_append(positions[b])
    return out


def certified_attention_layer(
    cache: TieredKeyCacheLayer,
    q_all: torch.Tensor,
    gqa_group: int,
    q_scale: float = None,
    collect_stats: bool = True,
    *,
    v_tolerance: float,
    top_k_fp16_keys: int = 0,
    ranking_fallback: bool = False,
    ranking_r: int = 1,
    ranking_fallback_mode: str = "full",
    tau_cov: float | None = None,
    k_min: int = DEFAULT_K_MIN,
    k_max: int | None = DEFAULT_K_MAX,
    rung1_threshold: float = DEFAULT_RUNG1_THRESHOLD,
    rung1_multiplier: float = DEFAULT_RUNG1_MULTIPLIER,
    score_consistency_check: bool = True,
    eps_guard: float = 0.01,
    exploration_rate: float = 0.0,
    exploration_generator: torch.Generator | None = None,
    phase_timings: dict | None = None,
    per_kv_group_topk: bool = False,
    value_error_mode: str = "tight",
    exploration_uniforms: torch.Tensor | None = None,
) -> tuple[torch.Tensor, dict[str, Any]]:
    """Full certified attention for one layer, all heads.

    Same contract as the reference (certified_attention.py:1065-1113): returns
    (output [num_q_heads, d_v] float32, stats dict).

    ONE DIFFERENCE a drop-in caller must know: the returned tensor is the
    workspace's output buffer of this cache, not a fresh tensor.  The next
    call on the same cache overwrites it (the kernels write their rows there
    without an allocation or a copy per step).  A caller that keeps outputs
    across steps must `.clone()` them; `o_proj(output)` right away, as the
    adapter does, needs nothing.

    `exploration_uniforms` ([H, nq] floats in [0,1)) is an addition: when given
    it replaces the random draw so a run can be replayed exactly.  With an
    `exploration_generator` the draw is the reference's `torch.rand` from that
    generator; with neither, the selector kernel draws (Philox keyed by
    `torch.initial_seed()`, a per-workspace serial number and a per-cache call
    counter, so different layers draw different sets).
    """
    if not q_all.is_cuda:
        raise RuntimeError("certified_attention_layer needs CUDA tensors; there is no CPU fallback")
    if value_error_mode not in ("loose", "tight"):
        raise ValueError(f"value_error_mode must be 'loose' or 'tight', got {value_error_mode!r}")
    if per_kv_group_topk:
        raise NotImplementedError("per_kv_group_topk (experimental per-KV-group selection) is not built")
    if q_scale is None:
        q_scale = 1.0 / (cache.head_dim ** 0.5)
    H = int(q_all.shape[0])
    G = int(gqa_group)
    if H != cache.kv_heads * G or q_all.shape[1] != cache.head_dim:
        raise ValueError(f"q_all shape {tuple(q_all.shape)} does not match {cache.kv_heads} KV heads x group {G}")
    nq = cache.num_quantized_blocks
    nact = cache.active_blocks
    bs = cache.block_size
    device = q_all.device
    has_int4 = cache.values_int4_packed is not None
    adaptive = tau_cov is not None and tau_cov > 0 and nq > 0
    naive = (
        has_int4 and not collect_stats and not (tau_cov is not None and tau_cov > 0)
        and int(top_k_fp16_keys or 0) <= 0 and not ranking_fallback and not score_consistency_check
        and exploration_rate <= 0
    )
    if not adaptive and not naive:
        if nq == 0:
            raise NotImplementedError(
                "no fully quantised block yet: the certified path needs at least 16 cached tokens")
        raise NotImplementedError(
            "only the adaptive-K* paper path (tau_cov > 0) and the plain INT8K/INT4V baseline are built; "
            "the legacy block-skipping paths are not")
    if not has_int4 and cache.values_fp16 is None:
        raise ValueError("No values available in cache")

    q = q_all if q_all.is_contiguous() else q_all.contiguous()
    qd = _lib.dtype_code(q.dtype)
    ws = _workspace(cache, H, G, device)
    L = _lib.lib()
    desc = cache._desc(G)
    stream = _lib.current_stream(device)
    pending: list = []
    trailing = cache.has_trailing_partial_block
    last_valid = bs if not trailing else cache.num_tokens - nq * bs

    if naive:
        # Plain quantised baseline: INT8 scores for every complete block, INT4
        # values, no certification.  (The trailing partial block is served from
        # the exact Tier-2 rows.)
        if nq == 0:
            raise NotImplementedError("baseline attend needs at least one complete block")
        wstruct = ws.fill_struct(nact)
        with _lib.on_device(device), _PhaseTimer(phase_timings, "phase2_fused_attend", pending):
            ws.topk_mask[:, :nact].zero_()
            ws.value_mask[:, :nact].zero_()
            if trailing:
                ws.value_mask[:, nq:nact].fill_(1)
            ws.cert_buf.zero_()
            _lib.check(L.cqa_score_blocks(C.byref(desc), q.data_ptr(), qd, nq, float(q_scale),
                                          ws.m_b.data_ptr(), ws.s_b.data_ptr(), ws.ld,
                                          ws.token_scores.data_ptr(), stream), "cqa_score_blocks")
            _lib.check(L.cqa_attend(C.byref(desc), C.byref(wstruct), q.data_ptr(), qd, nq, nact,
                                    cache.num_tokens, last_valid, float(q_scale), stream), "cqa_attend")
        _flush_timers(phase_timings, pending)
        return ws.out, {}

    force_trailing_value_fp16 = bool(
        trailing and has_int4 and cache.values_fp16_gpu is not None
        and (cache.values_fp16_cpu is not None or cache.fp16_value_cache_capacity is None
             or cache.static_resident_value_cache)
    )
    knobs = _make_knobs(
        q_scale=q_scale, tau_cov=tau_cov, k_min=k_min, k_max=k_max, rung1_threshold=rung1_threshold,
        rung1_multiplier=rung1_multiplier, eps_guard=eps_guard, exploration_rate=exploration_rate,
        v_tolerance=v_tolerance, ranking_r=ranking_r, top_k_fp16_keys=top_k_fp16_keys,
        ranking_fallback=ranking_fallback, ranking_fallback_mode=ranking_fallback_mode,
        score_consistency_check=score_consistency_check, value_error_mode=value_error_mode,
        force_trailing_value_fp16=force_trailing_value_fp16,
    )
    ws.ensure_sel_width(_selection_width(k_max, rung1_threshold, rung1_multiplier, nq), device)
    wstruct = ws.fill_struct(nact)

    u_ptr, u_ld = None, 0
    u_keep = None
    if exploration_rate > 0.0:
        if exploration_uniforms is not None:
            u_keep = exploration_uniforms.to(device=device, dtype=torch.float32).contiguous()
        elif exploration_generator is not None:
            # the reference's draw from the caller's generator (one uniform per (head, complete block))
            u_keep = torch.rand((H, nq), generator=exploration_generator, out=ws.uniform_buffer(nq, device))
        if u_keep is not None:
            if tuple(u_keep.shape) != (H, nq):
                raise ValueError(f"exploration uniforms must have shape {(H, nq)}, got {tuple(u_keep.shape)}")
            u_ptr, u_ld = u_keep.data_ptr(), nq
        else:
            # no generator given: the selector draws in-kernel (Philox keyed by torch's seed and a call counter;
            # same distribution as torch.rand, one launch fewer)
            wstruct.rng_seed = ws.draw_seed()
            wstruct.rng_offset = ws.rng_calls
            ws.rng_calls += 1

    with _lib.on_device(device):
        if phase_timings is None:
            _lib.check(L.cqa_layer_step(C.byref(desc), C.byref(knobs), C.byref(wstruct), q.data_ptr(), qd,
                                        cache.num_tokens, nq, u_ptr, u_ld, stream), "cqa_layer_step")
        else:
            with _PhaseTimer(phase_timings, "phase1_int8_scoring", pending):
                _lib.check(L.cqa_score_blocks(C.byref(desc), q.data_ptr(), qd, nq, float(q_scale),
                                              ws.m_b.data_ptr(), ws.s_b.data_ptr(), ws.ld,
                                              ws.token_scores.data_ptr(), stream), "cqa_score_blocks")
            with _PhaseTimer(phase_timings, "adaptive_selection", pending):
                _lib.check(L.cqa_select(C.byref(desc), C.byref(knobs), C.byref(wstruct), nq, nact, u_ptr, u_ld,
                                        stream), "cqa_select")
            # ranking, boundary, consistency and value checks share one kernel
            with _PhaseTimer(phase_timings, "ranking_check", pending):
                _lib.check(L.cqa_certify(C.byref(desc), C.byref(knobs), C.byref(wstruct), q.data_ptr(), qd, nq,
                                         nact, stream), "cqa_certify")
            with _PhaseTimer(phase_timings, "phase2_fused_attend", pending):
                _lib.check(L.cqa_attend(C.byref(desc), C.byref(wstruct), q.data_ptr(), qd, nq, nact,
                                        cache.num_tokens, last_valid, float(q_scale), stream), "cqa_attend")
        if cache.bounded_hot_tier:
            # queue the residency update (mark the blocks this step used, page the missed ones in)
            cache._hot_tier_update(desc, wstruct, nact, stream)
    _flush_timers(phase_timings, pending)
    output = ws.out
    if not collect_stats:
        return output, {}
    stats = _assemble_stats(
        cache, ws, H, G, nq, nact, has_int4=has_int4, force_trailing=force_trailing_value_fp16,
        tau_cov=tau_cov, rung1_threshold=rung1_threshold, rung1_multiplier=rung1_multiplier,
        exploration_rate=exploration_rate, score_consistency_check=score_consistency_check,
        eps_guard=eps_guard, ranking_fallback=ranking_fallback, ranking_r=ranking_r,
        ranking_fallback_mode=ranking_fallback_mode, top_k_fp16_keys=top_k_fp16_keys,
        value_error_mode=value_error_mode,
    )
    return output, stats


def _flush_timers(timings, pending):
    if timings is None or not pending:
        return
    torch.cuda.synchronize()
    for name, a, b in pending:
        key = f"{name}_us"
        timings[key] = timings.get(key, 0.0) + a.elapsed_time(b) * 1000.0


def _vram_stats(cache: TieredKeyCacheLayer) -> tuple[int, int]:
    kb = 0
    if cache.keys_fp16_gpu is not None:
        kb = cache.kv_heads * cache.num_tokens * cache.head_dim * cache.keys_fp16_gpu.element_size()
    vb = 0
    if cache.values_fp16 is not None:
        vb = cache.kv_heads * cache.num_tokens * cache.d_v * cache.values_fp16.element_size()
    elif cache.values_fp16_gpu is not None:
        vb = cache.values_fp16_gpu.numel() * cache.values_fp16_gpu.element_size()
    return int(kb), int(vb)


def _assemble_stats(cache, ws: _Workspace, H, G, nq, nact, *, has_int4, force_trailing, tau_cov,
                    rung1_threshold, rung1_multiplier, exploration_rate, score_consistency_check, eps_guard,
                    ranking_fallback, ranking_r, ranking_fallback_mode, top_k_fp16_keys,
                    value_error_mode) -> dict[str, Any]:
    """The reference's per-layer stats dict (certified_attention.py:2608-2788)."""
    import numpy as np

    cert, flags = ws.read_cert()
    rung4 = bool(score_consistency_check and flags[2])
    kb, vb = _vram_stats(cache)
    total_blocks = H * cache.num_blocks
    violation_heads = int(cert["consistency_violation"].sum())
    boundary_heads = int(cert["boundary_triggered"].sum())
    rung1_heads = int(cert["rung1_triggered"].sum())
    if rung4:
        # every head was recomputed densely; same keys as the reference's early return (:1771-1796)
        return {
            "total_blocks": total_blocks, "skipped_blocks": 0, "skip_rate": 0.0,
            "attended_blocks": total_blocks, "v_format": "fp16",
            "score_consistency_violation_heads": violation_heads,
            "delta_bound_mean": float(cert["delta"].mean()), "eps_guard": float(eps_guard),
            "h2d_key_bytes": 0, "h2d_key_blocks": 0, "h2d_value_bytes": 0, "h2d_value_blocks": 0,
            "h2d_total_bytes": 0, "vram_fp16_key_cache_bytes": kb, "vram_fp16_value_cache_bytes": vb,
            "rung1_fired": bool(rung1_heads > 0), "rung2_fired": False, "rung3_fired": False,
            "rung4_fired": True, "rung4_violating_heads": violation_heads,
            "boundary_check_triggered_heads": boundary_heads,
            "boundary_check_fired": bool(boundary_heads > 0),
        }
    skipped = int((ws.topk_mask[:, :nact] == 0).sum().item())
    vmask_q = ws.value_mask[:, :nq]
    head_blocks = int(cert["value_promoted_blocks"].sum()) if has_int4 else 0
    union_blocks = int((vmask_q.amax(dim=0) > 0).sum().item()) if (has_int4 and head_blocks) else 0
    if has_int4:
        v_format = "mixed" if (head_blocks or force_trailing) else "int4"
    else:
        v_format = "fp16"
    rung2 = bool(has_int4 and v_format == "mixed")
    dense_heads = int(cert["dense"].sum())
    stats: dict[str, Any] = {
        "total_blocks": total_blocks, "skipped_blocks": skipped,
        "skip_rate": float(skipped) / float(total_blocks), "attended_blocks": total_blocks - skipped,
        "v_format": v_format,
        "h2d_key_bytes": 0, "h2d_key_blocks": 0, "h2d_value_bytes": 0, "h2d_value_blocks": 0,
        "h2d_total_bytes": 0,
    }
    # residency figures of this step: the counters live on the device (csrc/hot_tier.cu keeps the values from
    # before the latest update beside the running totals); a full mirror never misses
    hot = cache.hot_tier_counters(last_call=True) if cache.bounded_hot_tier else {}
    if hot:
        blk_bytes = cache.kv_heads * cache.block_size * cache.head_dim * cache.keys_fp16_gpu.element_size()
        stats["h2d_key_blocks"] = int(hot["key_pageins"])
        stats["h2d_key_bytes"] = int(hot["key_pagein_bytes"])
        stats["h2d_value_blocks"] = int(hot["value_pageins"])
        stats["h2d_value_bytes"] = int(hot["value_pageins"]) * blk_bytes
        stats["h2d_total_bytes"] = stats["h2d_key_bytes"] + stats["h2d_value_bytes"]
    if cache.fp16_key_cache_capacity is not None:
        hits, misses = int(hot.get("key_hits", 0)), int(hot.get("key_misses", 0))
        resident = (int((cache._hot["key_slots"] >= 0).sum().item()) if cache.bounded_hot_tier
                    else int(len(cache._fp16_key_resident)))
        stats.update({
            "fp16_cache_capacity_blocks": int(cache.fp16_key_cache_capacity),
            "fp16_cache_resident_blocks": resident,
            "fp16_cache_hits_step": hits, "fp16_cache_misses_step": misses,
            "fp16_cache_evictions_step": int(hot.get("key_evictions", 0)),
            "fp16_cache_needed_blocks_step": hits + misses,
            "fp16_cache_hit_rate_step": float(hits) / (hits + misses) if (hits + misses) else 0.0,
        })
    if cache.fp16_value_cache_capacity is not None:
        hits, misses = int(hot.get("value_hits", 0)), int(hot.get("value_misses", 0))
        resident = (int((cache._hot["value_slots"] >= 0).sum().item()) if cache.bounded_hot_tier
                    else int(len(cache._fp16_value_resident)))
        stats.update({
            "fp16_value_cache_capacity_blocks": int(cache.fp16_value_cache_capacity),
            "fp16_value_cache_resident_blocks": resident,
            "fp16_value_cache_hits_step": hits, "fp16_value_cache_misses_step": misses,
            "fp16_value_cache_evictions_step": int(hot.get("value_evictions", 0)),
            "fp16_value_cache_needed_blocks_step": hits + misses,
            # a block that finds no free slot is read from the backing array in place: nothing overflows and the
            # attend kernel never falls back to another code path
            "fp16_value_cache_overflow_step": 0, "mixedv_splitk_fallback_step": 0,
            "fp16_value_cache_hit_rate_step": float(hits) / (hits + misses) if (hits + misses) else 0.0,
        })
    stats["vram_fp16_key_cache_bytes"] = kb
    stats["vram_fp16_value_cache_bytes"] = vb
    stats["rung1_fired"] = bool(rung1_heads > 0)
    stats["rung2_fired"] = rung2
    stats["rung3_fired"] = bool(dense_heads > 0)
    stats["rung4_fired"] = False
    if has_int4:
        rho = ws.mass_frac[:, :nq].sum(dim=1)
        rho_max = float(rho.max().item())
        eta_int4 = float(cache.values_int4_errors.max().item())
        stats["rho_max"] = rho_max
        stats["rho_mean"] = float(rho.mean().item())
        stats["eta_int4"] = eta_int4
        stats["int4_error_bound_loose"] = eta_int4 * rho_max
        stats["int4_error_bound"] = stats["int4_error_bound_loose"]
        stats["e_val_max"] = float(cert["e_val"].max())
        stats["e_val_mean"] = float(cert["e_val"].mean())
        stats["value_error_mode"] = value_error_mode
        stats["e_val_pre_rung2_max"] = float(cert["e_pre"].max())
        stats["e_val_pre_rung2_mean"] = float(cert["e_pre"].mean())
        if head_blocks:
            stats["value_fallback_blocks"] = union_blocks
            stats["value_fallback_head_blocks"] = head_blocks
    ks = cert["k_star"]
    stats["k_star_mean"] = float(ks.astype(np.float32).mean())
    stats["k_star_min"] = int(ks.min())
    stats["k_star_max"] = int(ks.max())
    stats["tau_cov"] = float(tau_cov) if tau_cov is not None else 0.0
    stats["tau_cov_actual_mean"] = float(cert["tau_actual"].mean())
    stats["tail_mass_int8_est_mean"] = float(cert["tail_mass"].mean())
    stats["tail_mass_int8_est_max"] = float(cert["tail_mass"].max())
    stats["rung1_triggered_heads"] = rung1_heads
    stats["rung1_threshold"] = float(rung1_threshold) if rung1_threshold is not None else -1.0
    stats["rung1_multiplier"] = float(rung1_multiplier)
    stats["exploration_rate"] = float(exploration_rate)
    stats["exploration_blocks"] = int(cert["exploration_blocks"].sum())
    v_max_layer = cache.v_max_global()
    stats["v_max_layer"] = float(v_max_layer)
    have_delta = (ranking_fallback or score_consistency_check) and nq > 0
    if have_delta and v_max_layer > 0.0:
        e2d = np.exp(2.0 * cert["delta"].astype(np.float32))
        e_key = 2.0 * v_max_layer * e2d * cert["tail_mass"].astype(np.float32) * (e2d - 1.0)
        stats["e_key_step_mean"] = float(e_key.mean())
        stats["e_key_step_max"] = float(e_key.max())
    if score_consistency_check:
        stats["score_consistency_violation_heads"] = violation_heads
        stats["delta_bound_mean"] = float(cert["delta"].mean())
        stats["eps_guard"] = float(eps_guard)
        stats["rung4_fired"] = False
        stats["rung4_violating_heads"] = 0
    if ranking_fallback:
        rk = min(max(int(ranking_r), int(top_k_fp16_keys or 0), 4), nq)
        stats["ranking_heads_total"] = H
        stats["ranking_disagree_r1"] = int(cert["ranking_disagree_r1"].sum())
        stats["ranking_disagree_r3"] = int(cert["ranking_disagree_r3"].sum())
        stats["ranking_fallback_triggered"] = dense_heads
        stats["ranking_r"] = int(ranking_r)
        stats["ranking_k"] = int(rk)
        stats["ranking_fallback_mode"] = ranking_fallback_mode
        stats["boundary_check_triggered_heads"] = boundary_heads
        stats["boundary_check_fired"] = bool(boundary_heads > 0)
        if rk >= 2:
            gap = (cert["fp16_top1"] - cert["fp16_top2"]).astype(np.float32)
            stats["score_gap_top12_mean"] = float(gap.mean())
            stats["score_gap_top12_min"] = float(gap.min())
        stats["s_int8_top1_mean"] = float(cert["int8_top1"].mean())
        stats["s_fp16_top1_mean"] = float(cert["fp16_top1"].mean())
    return stats


# ----------------------------------------------------------------------------- helper API

def _helper_cache_desc(kv_heads: int, gqa_group: int) -> _lib.CqaCache:
    d = _lib.CqaCache()
    d.kv_heads, d.gqa_group, d.t2_dtype = kv_heads, gqa_group, _lib.CQA_F16
    d.cap_tokens, d.max_blocks = 1, 1
    return d


def compute_adaptive_topk_mask(m_b, S_b, tau_cov: float = DEFAULT_TAU_COV, k_min: int = DEFAULT_K_MIN,
                               k_max: int | None = DEFAULT_K_MAX, per_kv_group_topk: bool = False,
                               gqa_group: int = 1, return_mass_frac: bool = False,
                               return_selection_indices: bool = False, defer_mask: bool = False,
                               return_sorted_cumsum: bool = False) -> tuple:
    """Adaptive top-K* selector (reference: certified_attention.py:245-444).

    Returns (topk_mask bool [H,B], k_star int32 [H], tail_mass [H], tau_actual [H]
    [, mass_frac][, sorted_idx int64, k_star][, sorted_cumsum])."""
    if per_kv_group_topk:
        raise NotImplementedError("per_kv_group_topk is not built")
    if not m_b.is_cuda:
        raise RuntimeError("compute_adaptive_topk_mask needs CUDA tensors; there is no CPU fallback")
    H, nb = m_b.shape
    dev = m_b.device
    if nb == 0:
        eb = torch.zeros(H, 0, dtype=torch.bool, device=dev)
        zi = torch.zeros(H, dtype=torch.int32, device=dev)
        zf = torch.zeros(H, dtype=torch.float32, device=dev)
        res = (eb, zi, zf, zf, torch.zeros(H, 0, dtype=torch.float32, device=dev)) if return_mass_frac else (eb, zi, zf, zf)
        if return_selection_indices:
            res = (*res, eb.long(), zi)
        if return_sorted_cumsum:
            res = (*res, torch.zeros(H, 0, dtype=torch.float32, device=dev))
        return res
    m = m_b.to(torch.float32).contiguous()
    s = S_b.to(torch.float32).contiguous()
    hi = nb if k_max is None else min(int(k_max), nb)
    f32 = dict(dtype=torch.float32, device=dev)
    mass = torch.empty(H, nb, **f32)
    topk = torch.empty(H, nb, dtype=torch.uint8, device=dev)
    expl = torch.empty(H, nb, dtype=torch.uint8, device=dev)
    sidx = torch.empty(H, hi, dtype=torch.int32, device=dev)
    scum = torch.empty(H, hi, **f32)
    cert = torch.zeros(H * _lib.CERT_BYTES + 4 * (5 + H), dtype=torch.uint8, device=dev)
    w = _lib.CqaWorkspace()
    w.ld = nb
    w.m_b, w.s_b, w.mass_frac = m.data_ptr(), s.data_ptr(), mass.data_ptr()
    w.topk_mask, w.explore_mask = topk.data_ptr(), expl.data_ptr()
    w.sorted_idx, w.sorted_cumsum, w.sel_width = sidx.data_ptr(), scum.data_ptr(), hi
    w.cert = cert.data_ptr()
    w.any_flags = cert.data_ptr() + H * _lib.CERT_BYTES
    kn = _make_knobs(q_scale=1.0, tau_cov=tau_cov, k_min=k_min, k_max=k_max, rung1_threshold=None,
                     rung1_multiplier=1.0, eps_guard=0.0, exploration_rate=0.0, v_tolerance=0.0, ranking_r=1,
                     top_k_fp16_keys=0, ranking_fallback=False, ranking_fallback_mode="full",
                     score_consistency_check=False, value_error_mode="tight", force_trailing_value_fp16=False)
    d = _helper_cache_desc(H, 1)
    with torch.cuda.device(dev):
        _lib.check(_lib.lib().cqa_select(C.byref(d), C.byref(kn), C.byref(w), nb, nb, None, 0,
                                         _lib.current_stream(dev)), "cqa_select")
    import numpy as np

    host = cert.cpu().numpy()
    arr = (_lib.CqaHeadCert * H).from_buffer_copy(host[: H * _lib.CERT_BYTES].tobytes())
    k_star = torch.tensor([arr[h].k_star for h in range(H)], dtype=torch.int32, device=dev)
    tail = torch.tensor(np.array([arr[h].tail_mass for h in range(H)], dtype=np.float32), device=dev)
    tau_a = torch.tensor(np.array([arr[h].tau_actual for h in range(H)], dtype=np.float32), device=dev)
    mask = torch.empty(H, 0, dtype=torch.bool, device=dev) if defer_mask else topk.bool()
    res = (mask, k_star, tail, tau_a, mass) if return_mass_frac else (mask, k_star, tail, tau_a)
    if return_selection_indices:
        res = (*res, sidx.long(), k_star)
    if return_sorted_cumsum:
        res = (*res, scum)
    return res


def compute_block_mass_fraction(m_b, S_b):
    """Normalised per-block attention mass (reference: certified_attention.py:128-136)."""
    return compute_adaptive_topk_mask(m_b, S_b, tau_cov=1.0, k_min=1, k_max=1, return_mass_frac=True)[4]


def compute_tier2_residual_mass(m_b, S_b, skip_mask, top_k: int = TOP_K_BLOCKS, return_details: bool = False):
    """Per-head residual mass rho = 1 - alpha_K - beta: alpha_K = mass on the top_k blocks by m_b, beta = mass on
    skipped blocks (reference: certified_attention.py:83-125).  The mass fractions come from the selector kernel;
    the [H, top_k] gather and the two row sums are torch reductions over a tensor that already exists."""
    mass_frac = compute_block_mass_fraction(m_b, S_b)
    H, nb = m_b.shape
    k = min(int(top_k), nb)
    topk_idx = m_b.topk(k, dim=1).indices if k else torch.zeros(H, 0, dtype=torch.long, device=m_b.device)
    alpha = mass_frac.gather(1, topk_idx).sum(dim=1)
    beta = (mass_frac * skip_mask.to(mass_frac.dtype)).sum(dim=1)
    rho = (1.0 - alpha - beta).clamp(min=0.0, max=1.0)
    return (rho, mass_frac, topk_idx) if return_details else rho


def _eta_per_q_head(eta_per_block, num_q_heads: int, gqa_group: int, nb: int):
    kv_idx = (torch.arange(num_q_heads, device=eta_per_block.device) // int(gqa_group)).clamp(
        max=eta_per_block.shape[0] - 1)
    return eta_per_block[:, :nb][kv_idx]


def compute_value_error_bound_for_mask(mass_frac, int4_value_mask, eta_per_block, gqa_group: int):
    """[H]: sum over the blocks whose values stay INT4 of mass[h, b] * eta[kv(h), b]
    (reference: certified_attention.py:139-155)."""
    nb = min(mass_frac.shape[1], eta_per_block.shape[1])
    eta_q = _eta_per_q_head(eta_per_block, mass_frac.shape[0], gqa_group, nb)
    return (mass_frac[:, :nb] * int4_value_mask[:, :nb].to(mass_frac.dtype) * eta_q).sum(dim=1)


def compute_value_error_bound(mass_frac, topk_idx, skip_mask, eta_per_block, gqa_group: int):
    """[H]: the same sum over the residual blocks, i.e. neither in `topk_idx` nor skipped
    (reference: certified_attention.py:158-208)."""
    nb = min(mass_frac.shape[1], eta_per_block.shape[1])
    residual = torch.ones(mass_frac.shape[0], nb, dtype=torch.bool, device=mass_frac.device)
    if topk_idx.numel():
        residual.scatter_(1, topk_idx.clamp(max=nb - 1), False)
    residual &= ~skip_mask[:, :nb].bool()
    eta_q = _eta_per_q_head(eta_per_block, mass_frac.shape[0], gqa_group, nb)
    return (mass_frac[:, :nb] * eta_q * residual.to(mass_frac.dtype)).sum(dim=1)


def _dense_rows(cache: TieredKeyCacheLayer, q_all, gqa_group: int, q_scale: float, heads: torch.Tensor | None):
    """Dense attention over the Tier-2 keys and values of `cache` for the listed heads (all heads when `heads` is
    None), by the dense-recompute CTAs of the attend kernel (cqa_dense_attend).  Returns float32 [H, 128]; rows of
    heads that were not listed are undefined."""
    if not q_all.is_cuda:
        raise RuntimeError("dense recompute needs CUDA tensors; there is no CPU fallback")
    G = int(gqa_group)
    H = cache.kv_heads * G
    dev = q_all.device
    ws = _workspace(cache, H, G, dev)
    # a private certificate: only the `dense` marks, the count and the list of heads are read
    buf = torch.zeros(H * _lib.CERT_BYTES + 4 * (5 + H), dtype=torch.uint8, device=dev)
    flags = buf[H * _lib.CERT_BYTES:].view(torch.int32)
    if heads is None:
        flags[2] = 1                                   # "every head": what a score-consistency violation sets
    else:
        hs = heads.to(device=dev, dtype=torch.int32).reshape(-1)
        cert_i32 = buf[: H * _lib.CERT_BYTES].view(torch.int32).view(H, _lib.CERT_BYTES // 4)
        cert_i32[hs.long(), _lib.CqaHeadCert.dense.offset // 4] = 1
        flags[4] = int(hs.numel())
        flags[5: 5 + hs.numel()] = hs
    out = torch.empty(H, 128, dtype=torch.float32, device=dev)
    w = _lib.CqaWorkspace.from_buffer_copy(bytes(ws.fill_struct(cache.active_blocks)))
    w.cert = buf.data_ptr()
    w.any_flags = buf.data_ptr() + H * _lib.CERT_BYTES
    w.out = out.data_ptr()
    q = q_all.contiguous()
    with _lib.on_device(dev):
        _lib.check(_lib.lib().cqa_dense_attend(
            C.byref(cache._desc(G)), C.byref(w), q.data_ptr(), _lib.dtype_code(q.dtype), cache.num_tokens,
            float(q_scale), _lib.current_stream(dev)), "cqa_dense_attend")
    return out


def recompute_heads_dense_fp16(cache: TieredKeyCacheLayer, q_all, output, head_indices, gqa_group: int,
                               q_scale: float):
    """Rung-3 recompute: replace output[h] for the listed heads by dense attention over the cache's Tier-2 keys and
    values (reference: certified_attention.py:789-879).  Returns (output, h2d_key_bytes, h2d_key_blocks,
    h2d_value_bytes, h2d_value_blocks); the byte counts are zero because nothing is staged through the host (with
    a bounded hot tier the kernel reads non-resident blocks from the pinned backing arrays in place)."""
    if head_indices.numel() == 0:
        return output, 0, 0, 0, 0
    rows = _dense_rows(cache, q_all, gqa_group, q_scale, head_indices)
    idx = head_indices.to(device=output.device, dtype=torch.long).reshape(-1)
    output.index_copy_(0, idx, rows.index_select(0, idx).to(output.dtype))
    return output, 0, 0, 0, 0


def sdpa_attend_with_skip(cache: TieredKeyCacheLayer, q_all, skip_mask, gqa_group: int, q_scale: float):
    """Dense attention of every head over the Tier-2 keys and values, float32 [H, 128]
    (reference: certified_attention.py:989-1062, which calls torch SDPA in the model dtype; here the dense CTAs of
    the attend kernel accumulate in float32).  Block skipping (`skip_mask` with True entries) belongs to the
    reference's disabled legacy path and is refused."""
    if skip_mask is not None and bool(skip_mask.any().item()):
        raise NotImplementedError("block skipping is not built; pass an all-False skip mask")
    return _dense_rows(cache, q_all, gqa_group, q_scale, None)


def compute_fp16_block_scores(cache: TieredKeyCacheLayer, q_all, block_indices, num_scoring_blocks: int,
                              gqa_group: int, q_scale: float, return_log_mass: bool = False,
                              keys_fp16_override=None, key_block_slots=None):
    """Per-head FP16-key block max logits (and log-masses) for `block_indices`
    [H, K] (reference: certified_attention.py:447-559)."""
    if keys_fp16_override is not None or key_block_slots is not None:
        raise NotImplementedError("custom FP16 key scratch / slot tables are not built (full mirrors only)")
    H, K = block_indices.shape
    dev = q_all.device
    scores = torch.full((H, K), float("-inf"), dtype=torch.float32, device=dev)
    logm = torch.full((H, K), float("-inf"), dtype=torch.float32, device=dev)
    if K and num_scoring_blocks > 0:
        idx = block_indices.to(torch.int32).contiguous()
        q = q_all.contiguous()
        d = cache._desc(gqa_group)
        with torch.cuda.device(dev):
            _lib.check(_lib.lib().cqa_fp16_block_scores(
                C.byref(d), q.data_ptr(), _lib.dtype_code(q.dtype), idx.data_ptr(), K, int(num_scoring_blocks),
                float(q_scale), scores.data_ptr(), logm.data_ptr(), _lib.current_stream(dev)),
                "cqa_fp16_block_scores")
    return (scores, logm) if return_log_mass else scores


def compute_delta_bound(q_all, key_scales, gqa_group: int, q_scale: float):
    """Per-head Delta bound (reference: certified_attention.py:912-945).
    `key_scales` is [kv, blocks, 128]; its per-channel max over blocks is
    reduced with torch (this helper is not on the decode path, which uses the
    cache's running `keys_scale_max`)."""
    H = q_all.shape[0]
    dev = q_all.device
    if key_scales.numel() == 0:
        return torch.zeros(H, dtype=torch.float32, device=dev)
    smax = key_scales.amax(dim=1).to(torch.float32).contiguous()
    d = _helper_cache_desc(int(smax.shape[0]), int(gqa_group))
    d.sigma_max = smax.data_ptr()
    out = torch.empty(H, dtype=torch.float32, device=dev)
    q = q_all.contiguous()
    with torch.cuda.device(dev):
        _lib.check(_lib.lib().cqa_delta_bound(C.byref(d), q.data_ptr(), _lib.dtype_code(q.dtype),
                                              out.data_ptr(), _lib.current_stream(dev)), "cqa_delta_bound")
    return out


def score_consistency_violations(int8_scores, fp16_scores, delta_per_head, eps_guard: float = 0.01):
    """[H] bool: any |FP16 - INT8| block score above Delta + eps_guard
    (reference: certified_attention.py:948-965).  Tiny [H, K] comparison."""
    if int8_scores.numel() == 0:
        return torch.zeros(int8_scores.shape[0], dtype=torch.bool, device=int8_scores.device)
    diff = (fp16_scores - int8_scores).abs().float()
    return (diff > (delta_per_head + float(eps_guard)).unsqueeze(1)).any(dim=1)


def detect_ranking_disagreement(int8_scores, fp16_scores, r: int):
    """[H] bool: ordered top-r positions differ (reference: certified_attention.py:968-986)."""
    if int8_scores.numel() == 0 or r <= 0:
        return torch.zeros(int8_scores.shape[0], dtype=torch.bool, device=int8_scores.device)
    r_eff = min(r, int8_scores.shape[1])
    a = int8_scores.argsort(dim=1, descending=True)[:, :r_eff]
    b = fp16_scores.argsort(dim=1, descending=True)[:, :r_eff]
    return (a != b).any(dim=1)


def augment_mask_with_exploration(topk_mask, exploration_rate: float, generator=None, count: bool = True):
    """Bernoulli exploration on non-promoted blocks (reference: certified_attention.py:882-909)."""
    if exploration_rate <= 0.0 or topk_mask.numel() == 0:
        return topk_mask, torch.zeros_like(topk_mask), 0
    rand = torch.rand(topk_mask.shape, device=topk_mask.device, generator=generator)
    explore = (~topk_mask) & (rand < float(exploration_rate))
    return topk_mask | explore, explore, (int(explore.sum().item()) if count else 0)


def decide_v_format(rho, eta_int4: float, tolerance: float = DEFAULT_V_TOLERANCE) -> str:
    return "int4" if eta_int4 * rho.max().item() < tolerance else "fp16"


def decide_v_format_tight(e_val_head, tolerance: float = DEFAULT_V_TOLERANCE) -> str:
    return "int4" if e_val_head.max().item() < tolerance else "fp16"
