"""Tiered KV cache for certified decode attention, B200-native.

Mirrors the public surface of the reference's
`dotcache/kernels/tiered_kv_cache.py` (TieredKeyCacheLayer:29-132,
from_fp16_cache:135-286, from_fp16_cache_int4v:289-405, append_token:545-708,
create_tiered_cache*_from_model:1579-1701): same field names, shapes, dtypes
and counters, so callers that read the tensors keep working.  All
quantisation and append work runs in hand-written CUDA through the C ABI of
libcqa_b200.so; there is no PyTorch or CPU compute path.

Tier 1 (INT8 per-channel keys, INT4 per-group values) lives in HBM.  Tier 2
(the model-dtype originals) lives in HBM too by default: a B200 has room for
the full-context originals, so `keys_fp16_gpu` / `values_fp16_gpu` are full
mirrors addressed through identity slot tables.  With hot-tier capacities
below the reserved context (INT4-value caches), Tier 2 is kept in pinned host
memory behind a device scratch of `capacity` blocks; residency tables, clock
replacement and counters live on the device (csrc/hot_tier.cu).
"""
from __future__ import annotations

import ctypes as C
from collections import OrderedDict
from dataclasses import dataclass, field
from typing import Any

import torch

from cqa_b200 import _lib

BLOCK = 16
HEAD_DIM = 128


def _require_cuda(t: torch.Tensor, what: str) -> None:
    if not t.is_cuda:
        raise RuntimeError(
            f"{what} must be a CUDA tensor: this cache runs only on the GPU library "
            "(libcqa_b200.so); there is no CPU fallback"
        )


@dataclass
class TieredKeyCacheLayer:
    """One layer's tiered cache (all KV heads)."""

    keys_int8: torch.Tensor           # [kv, cap, 128] int8
    keys_scale: torch.Tensor          # [kv, max_blocks, 128] f32
    keys_zero_points: torch.Tensor    # [kv, max_blocks, 128] f32
    correction: torch.Tensor          # [kv, max_blocks] f32
    values_fp16: torch.Tensor | None  # [kv, cap, 128] model dtype (FP16-value caches only)
    keys_fp16_cpu: torch.Tensor | None
    kv_heads: int
    num_tokens: int
    head_dim: int
    d_v: int
    block_size: int
    num_blocks: int
    num_quantized_blocks: int = 0
    _pagein_buffer: torch.Tensor | None = None
    _keys_deq_f32: torch.Tensor | None = None
    _values_f32: torch.Tensor | None = None
    values_int4_packed: torch.Tensor | None = None   # [kv, cap, 64] u8
    values_int4_scales: torch.Tensor | None = None   # [kv, cap, 8] f16
    values_int4_zeros: torch.Tensor | None = None    # [kv, cap, 8] f16
    values_int4_errors: torch.Tensor | None = None   # eta_b [kv, max_blocks] f32
    values_int4_error_sums: torch.Tensor | None = None
    values_int4_error_counts: torch.Tensor | None = None
    values_int4_group_size: int = 16
    defer_int4_append_quantization: bool = False
    values_norm_max_per_block: torch.Tensor | None = None  # nu_b [kv, max_blocks] f32
    values_fp16_cpu: torch.Tensor | None = None
    values_fp16_gpu: torch.Tensor | None = None
    fp16_value_cache_capacity: int | None = None
    _fp16_value_resident: "OrderedDict[int, int]" = field(default_factory=OrderedDict)
    _fp16_value_free_slots: list = field(default_factory=list)
    static_resident_value_cache: bool = False
    static_resident_value_prepare_bytes: int = 0
    keys_fp16_gpu: torch.Tensor | None = None
    fp16_key_cache_capacity: int | None = None
    _fp16_key_resident: "OrderedDict[int, int]" = field(default_factory=OrderedDict)
    _fp16_key_free_slots: list = field(default_factory=list)
    static_resident_key_cache: bool = False
    static_resident_key_prepare_bytes: int = 0
    # Running per-channel max of keys_scale over quantised blocks, [kv, 128] f32
    # (what compute_delta_bound reduces every step in the reference,
    # certified_attention.py:938; here the quantisers maintain it).
    keys_scale_max: torch.Tensor | None = None
    gqa_group_hint: int = 1
    _certified_workspace: dict = field(default_factory=dict, repr=False)
    _desc_cache: dict = field(default_factory=dict, repr=False)
    _hot: dict | None = field(default=None, repr=False)     # bounded hot tier: tables, counters, struct

    # ------------------------------------------------------------------ C ABI view

    def _desc(self, gqa_group: int | None = None) -> _lib.CqaCache:
        """The cqa_cache struct over this layer's tensors.  Built once per GQA group and reused: the tensors
        are allocated at construction and never replaced (call `_invalidate_desc` after swapping one)."""
        g = int(gqa_group if gqa_group is not None else self.gqa_group_hint)
        cached = self._desc_cache.get(g)
        if cached is not None:
            return cached
        d = _lib.CqaCache()
        d.kv_heads = self.kv_heads
        d.gqa_group = g
        t2 = self.keys_fp16_gpu
        d.t2_dtype = _lib.dtype_code(t2.dtype) if t2 is not None else _lib.CQA_F16
        d.cap_tokens = int(self.keys_int8.shape[1])
        d.max_blocks = int(self.keys_scale.shape[1])
        d.keys_int8 = _lib.ptr(self.keys_int8)
        d.keys_scale = _lib.ptr(self.keys_scale)
        d.keys_zero_points = _lib.ptr(self.keys_zero_points)
        d.correction = _lib.ptr(self.correction)
        d.sigma_max = _lib.ptr(self.keys_scale_max)
        d.values_int4_packed = _lib.ptr(self.values_int4_packed)
        d.values_int4_scales = _lib.ptr(self.values_int4_scales)
        d.values_int4_zeros = _lib.ptr(self.values_int4_zeros)
        d.values_int4_errors = _lib.ptr(self.values_int4_errors)
        d.values_int4_error_sums = _lib.ptr(self.values_int4_error_sums)
        d.values_int4_error_counts = _lib.ptr(self.values_int4_error_counts)
        d.values_norm_max = _lib.ptr(self.values_norm_max_per_block)
        d.keys_t2 = _lib.ptr(t2)
        d.keys_t2_rows = int(t2.shape[1]) if t2 is not None else 0
        vt2 = self.values_fp16 if self.values_fp16 is not None else self.values_fp16_gpu
        d.values_t2 = _lib.ptr(vt2)
        d.values_t2_rows = int(vt2.shape[1]) if vt2 is not None else 0
        d.key_slots = None      # identity: full mirrors
        d.value_slots = None
        if self._hot is not None:
            # bounded hot tier: the *_gpu arrays are slot scratch, the pinned *_cpu arrays back them
            d.key_slots = self._hot["key_slots"].data_ptr()
            d.value_slots = self._hot["value_slots"].data_ptr()
            d.keys_t2_backing = self.keys_fp16_cpu.data_ptr()
            d.values_t2_backing = self.values_fp16_cpu.data_ptr()
            d.t2_backing_rows = int(self.keys_fp16_cpu.shape[1])
        self._desc_cache[g] = d
        return d

    def _desc_copy(self, gqa_group: int | None = None) -> _lib.CqaCache:
        """A private copy of the descriptor, for callers that override fields."""
        src = self._desc(gqa_group)
        d = _lib.CqaCache()
        C.memmove(C.byref(d), C.byref(src), C.sizeof(d))
        return d

    def _invalidate_desc(self) -> None:
        self._desc_cache.clear()

    # ------------------------------------------------------------------ construction

    @classmethod
    def _allocate(cls, keys: torch.Tensor, values: torch.Tensor, block_size: int, max_pagein_blocks: int,
                  max_new_tokens: int, int4: bool, group_size: int,
                  hot_blocks: tuple[int, int] | None = None) -> "TieredKeyCacheLayer":
        _require_cuda(keys, "keys")
        _require_cuda(values, "values")
        if block_size != BLOCK:
            raise ValueError("block_size must be 16 (fixed by the kernels)")
        if int4 and group_size != 16:
            raise ValueError("INT4 group_size must be 16 (fixed by the kernels)")
        kv, N, hd = keys.shape
        dv = values.shape[2]
        if hd != HEAD_DIM or dv != HEAD_DIM:
            raise ValueError(f"head_dim and d_v must be 128 (got {hd}, {dv})")
        if N % BLOCK != 0:
            raise ValueError("N must be block aligned; append the remainder with append_token")
        if keys.dtype != values.dtype:
            values = values.to(keys.dtype)
        _lib.dtype_code(keys.dtype)
        dev = keys.device
        nb = N // BLOCK
        cap = N + max_new_tokens
        maxblk = nb + (max_new_tokens + BLOCK - 1) // BLOCK
        kvd = keys.dtype
        z = torch.zeros
        self = cls(
            keys_int8=z(kv, cap, hd, dtype=torch.int8, device=dev),
            keys_scale=z(kv, maxblk, hd, dtype=torch.float32, device=dev),
            keys_zero_points=z(kv, maxblk, hd, dtype=torch.float32, device=dev),
            correction=torch.ones(kv, maxblk, dtype=torch.float32, device=dev),
            values_fp16=None,
            keys_fp16_cpu=None,
            kv_heads=kv, num_tokens=N, head_dim=hd, d_v=dv, block_size=BLOCK, num_blocks=nb,
            num_quantized_blocks=nb,
            _pagein_buffer=torch.empty(max_pagein_blocks * BLOCK, hd, dtype=kvd, device=dev),
            values_norm_max_per_block=z(kv, maxblk, dtype=torch.float32, device=dev),
            keys_fp16_gpu=z(kv, cap if hot_blocks is None else hot_blocks[0] * BLOCK, hd, dtype=kvd, device=dev),
            keys_scale_max=z(kv, hd, dtype=torch.float32, device=dev),
        )
        vbuf = z(kv, cap if hot_blocks is None else hot_blocks[1] * BLOCK, dv, dtype=kvd, device=dev)
        if hot_blocks is not None:
            # Bounded hot tier: the complete Tier 2 lives in pinned host memory (device-addressable); the
            # *_gpu arrays above are slot scratch; residency tables and counters live on the device.
            kcap, vcap = hot_blocks
            self.keys_fp16_cpu = torch.zeros(kv, cap, hd, dtype=kvd).pin_memory()
            self.values_fp16_cpu = torch.zeros(kv, cap, dv, dtype=kvd).pin_memory()
            i32 = dict(dtype=torch.int32, device=dev)
            hot = {
                "key_slots": torch.full((maxblk,), -1, **i32), "value_slots": torch.full((maxblk,), -1, **i32),
                "key_owner": torch.full((kcap,), -1, **i32), "value_owner": torch.full((vcap,), -1, **i32),
                "key_stamp": torch.full((kcap,), -1, **i32), "value_stamp": torch.full((vcap,), -1, **i32),
                "work": torch.zeros(2 * (2 + 3 * maxblk), **i32),
                "counters": torch.zeros(24, dtype=torch.int64, device=dev),
            }
            st = _lib.CqaHotTier()
            st.key_capacity_blocks, st.value_capacity_blocks = kcap, vcap
            st.max_fill_blocks = max(1, int(max_pagein_blocks))
            for name in ("key_slots", "value_slots", "key_owner", "value_owner", "key_stamp", "value_stamp", "work",
                         "counters"):
                setattr(st, name, hot[name].data_ptr())
            hot["struct"] = st
            self._hot = hot
            self.fp16_key_cache_capacity = kcap
            self.fp16_value_cache_capacity = vcap
        if int4:
            self.values_int4_packed = z(kv, cap, dv // 2, dtype=torch.uint8, device=dev)
            self.values_int4_scales = z(kv, cap, dv // 16, dtype=torch.float16, device=dev)
            self.values_int4_zeros = z(kv, cap, dv // 16, dtype=torch.float16, device=dev)
            self.values_int4_errors = z(kv, maxblk, dtype=torch.float32, device=dev)
            self.values_int4_error_sums = z(kv, maxblk, dtype=torch.float32, device=dev)
            self.values_int4_error_counts = z(kv, maxblk, dtype=torch.int32, device=dev)
            self.values_int4_group_size = 16
            self.values_fp16_gpu = vbuf
        else:
            self.values_fp16 = vbuf
        self._fp16_key_resident = OrderedDict((i, i) for i in range(nb))
        return self

    def _quantize_prefill(self, keys: torch.Tensor, values: torch.Tensor) -> None:
        N = keys.shape[1]
        if N == 0:
            return
        keys = keys.contiguous()
        values = values.to(keys.dtype).contiguous()
        with torch.cuda.device(keys.device):
            rc = _lib.lib().cqa_quantize_blocks(
                C.byref(self._desc()), keys.data_ptr(), values.data_ptr(), _lib.dtype_code(keys.dtype),
                N, 0, N // BLOCK, _lib.current_stream(keys.device))
        _lib.check(rc, "cqa_quantize_blocks")

    @staticmethod
    def _check_capacity(cap, max_blocks: int, what: str):
        """None = full HBM mirror; a capacity covering the reserved context = static-resident (same layout);
        anything smaller = bounded hot tier (INT4-value caches only)."""
        if cap is None:
            return None
        return max(int(cap), 0)

    @classmethod
    def from_fp16_cache(cls, keys_fp16: torch.Tensor, values_fp16: torch.Tensor, block_size: int = 16,
                        max_pagein_blocks: int = 64, max_new_tokens: int = 512,
                        fp16_key_cache_capacity: int | None = None, _encode: bool = True) -> "TieredKeyCacheLayer":
        """INT8 keys + model-dtype values (reference: tiered_kv_cache.py:135-286).  `_encode=False` only allocates
        (the whole-model constructors encode every layer in one library call afterwards)."""
        self = cls._allocate(keys_fp16, values_fp16, block_size, max_pagein_blocks, max_new_tokens,
                             int4=False, group_size=16)
        cap = cls._check_capacity(fp16_key_cache_capacity, self.keys_scale.shape[1], "fp16_key_cache_capacity")
        if cap is not None and cap < self.keys_scale.shape[1]:
            raise NotImplementedError(
                "a bounded FP16-key scratch is built for the INT4-value cache (from_fp16_cache_int4v) only; "
                "pass None or a capacity that covers the reserved context")
        if _encode:
            self._quantize_prefill(keys_fp16, values_fp16)
        if cap is not None:
            self.fp16_key_cache_capacity = cap
            self.static_resident_key_cache = True
            self._fp16_key_resident = OrderedDict((i, i) for i in range(self.keys_scale.shape[1]))
        return self

    @classmethod
    def from_fp16_cache_int4v(cls, keys_fp16: torch.Tensor, values_fp16: torch.Tensor, block_size: int = 16,
                              group_size: int = 16, max_pagein_blocks: int = 64, max_new_tokens: int = 512,
                              fp16_key_cache_capacity: int | None = None,
                              fp16_value_cache_capacity: int | None = None,
                              defer_int4_append_quantization: bool = False,
                              _encode: bool = True) -> "TieredKeyCacheLayer":
        """INT8 keys + INT4 g16 values (reference: tiered_kv_cache.py:289-405).  `_encode=False` only allocates."""
        nb0 = keys_fp16.shape[1] // BLOCK
        maxblk = nb0 + (max_new_tokens + BLOCK - 1) // BLOCK
        kcap = cls._check_capacity(fp16_key_cache_capacity, maxblk, "fp16_key_cache_capacity")
        vcap = cls._check_capacity(fp16_value_cache_capacity, maxblk, "fp16_value_cache_capacity")
        bounded = (kcap is not None and kcap < maxblk) or (vcap is not None and vcap < maxblk)
        hot_blocks = None
        if bounded:
            if (kcap is not None and kcap < 1) or (vcap is not None and vcap < 1):
                raise ValueError("hot-tier capacities must be at least one block")
            hot_blocks = (min(kcap, maxblk) if kcap is not None else maxblk,
                          min(vcap, maxblk) if vcap is not None else maxblk)
        self = cls._allocate(keys_fp16, values_fp16, block_size, max_pagein_blocks, max_new_tokens,
                             int4=True, group_size=group_size, hot_blocks=hot_blocks)
        if bounded:
            self.defer_int4_append_quantization = bool(defer_int4_append_quantization)
            if _encode:
                self._quantize_prefill(keys_fp16, values_fp16)
            self._fp16_key_resident = OrderedDict()
            self._fp16_value_resident = OrderedDict()
            return self
        self.defer_int4_append_quantization = bool(defer_int4_append_quantization)
        if _encode:
            self._quantize_prefill(keys_fp16, values_fp16)
        if kcap is not None:
            self.fp16_key_cache_capacity = kcap
            self.static_resident_key_cache = True
            self._fp16_key_resident = OrderedDict((i, i) for i in range(maxblk))
        if vcap is not None:
            # A capacity that covers the reserved context is the reference's
            # "static resident" mode, which also defers INT4 append
            # quantisation to block completion (tiered_kv_cache.py:947-952).
            self.fp16_value_cache_capacity = vcap
            self.static_resident_value_cache = True
            self.defer_int4_append_quantization = True
            self._fp16_value_resident = OrderedDict((i, i) for i in range(maxblk))
        return self

    # ------------------------------------------------------------------ append

    def append_token(self, key_fp16: torch.Tensor, value_fp16: torch.Tensor) -> None:
        """Append one token ([kv, 1, 128] each); one fused kernel launch.

        Reference: tiered_kv_cache.py:545-708 (append_token, _quantize_block,
        _quantize_value_block)."""
        pos = self.num_tokens
        if pos >= self.keys_int8.shape[1]:
            raise ValueError(
                f"cache capacity {self.keys_int8.shape[1]} exhausted; build the cache with a larger max_new_tokens")
        _require_cuda(key_fp16, "key")
        k = key_fp16.reshape(self.kv_heads, self.head_dim)
        v = value_fp16.reshape(self.kv_heads, self.d_v)
        if v.dtype != k.dtype:
            v = v.to(k.dtype)
        if not k.is_contiguous():
            k = k.contiguous()
        if not v.is_contiguous():
            v = v.contiguous()
        defer = self._defer_int4_flag()
        dev = k.device
        with _lib.on_device(dev):
            rc = _lib.lib().cqa_append_token(
                C.byref(self._desc()), k.data_ptr(), v.data_ptr(), _lib.dtype_code(k.dtype), pos,
                1 if defer else 0, _lib.current_stream(dev))
        _lib.check(rc, "cqa_append_token")
        self._advance_after_append(pos)

    # ------------------------------------------------------------------ bounded hot tier

    @property
    def bounded_hot_tier(self) -> bool:
        return self._hot is not None

    def _hot_tier_update(self, desc, ws_struct, nact: int, stream: int) -> None:
        """Queue the residency update for the step whose masks are in `ws_struct` (no host wait)."""
        rc = _lib.lib().cqa_hot_tier_update(C.byref(desc), C.byref(ws_struct), C.byref(self._hot["struct"]), nact,
                                            stream)
        _lib.check(rc, "cqa_hot_tier_update")

    def hot_tier_counters(self, last_call: bool = False) -> dict:
        """Residency telemetry (synchronises): hits, misses, page-ins and evictions per tier, and the bytes the
        page-ins moved from the backing arrays.  Totals since construction, or with `last_call` the figures of the
        latest residency update alone (the device keeps the counters as they were before it)."""
        if self._hot is None:
            return {}
        c = self._hot["counters"].cpu().tolist()
        if last_call:
            c = [a - b for a, b in zip(c[:12], c[12:24])]
        blk = BLOCK * self.head_dim * self.keys_fp16_gpu.element_size() * self.kv_heads
        out = {"steps": c[0]}
        for name, o in (("key", 3), ("value", 7)):
            out[f"{name}_hits"], out[f"{name}_misses"] = c[o], c[o + 1]
            out[f"{name}_pageins"], out[f"{name}_evictions"] = c[o + 2], c[o + 3]
            out[f"{name}_pagein_bytes"] = c[o + 2] * blk
        return out

    def _ensure_resident(self, tier: int, block_ids) -> tuple[int, int, int, int]:
        """(hits, misses, bytes paged in, evictions) of one residency request; zeros for a full mirror."""
        if self._hot is None:
            return (0, 0, 0, 0)
        dev = self.keys_int8.device
        ids = block_ids if torch.is_tensor(block_ids) else torch.as_tensor(list(block_ids), dtype=torch.int64)
        ids = torch.unique(ids.to(device=dev, dtype=torch.int64))
        with _lib.on_device(dev):
            rc = _lib.lib().cqa_hot_tier_ensure(C.byref(self._desc()), C.byref(self._hot["struct"]), tier,
                                                ids.data_ptr(), int(ids.numel()), _lib.current_stream(dev))
        _lib.check(rc, "cqa_hot_tier_ensure")
        d = self.hot_tier_counters(last_call=True)
        name = "key" if tier == 0 else "value"
        return (d[f"{name}_hits"], d[f"{name}_misses"], d[f"{name}_pagein_bytes"], d[f"{name}_evictions"])

    def ensure_fp16_keys_resident(self, block_ids) -> tuple[int, int, int, int]:
        """Bring `block_ids` into the bounded FP16 key scratch; returns (hits, misses, bytes, evictions) of this
        call (reference: tiered_kv_cache.py:1218-1304).  A no-op returning zeros for a full mirror.  The residency
        tables live on the device: misses are paged in by kernels from the pinned backing array, slots not used in
        the current step are recycled in clock order, at most `max_pagein_blocks` blocks per call.  Kernels never
        need this call (they read a non-resident block from the backing array); it is a prefetch."""
        return self._ensure_resident(0, block_ids)

    def ensure_fp16_values_resident(self, block_ids) -> tuple[int, int, int, int]:
        """Value-tier twin of ensure_fp16_keys_resident (reference: tiered_kv_cache.py:1387-1463)."""
        return self._ensure_resident(1, block_ids)

    def ensure_fp16_keys_resident_batched(self, block_ids) -> tuple[int, int, int, int]:
        """Reference: tiered_kv_cache.py:1306-1385; the request is always one batched device operation here."""
        return self._ensure_resident(0, block_ids)

    def ensure_fp16_values_resident_batched(self, block_ids) -> tuple[int, int, int, int]:
        """Reference: tiered_kv_cache.py:1465-1537."""
        return self._ensure_resident(1, block_ids)

    def _defers_int4(self) -> bool:
        return bool(
            self.defer_int4_append_quantization
            and self.values_fp16_gpu is not None
            and (self.fp16_value_cache_capacity is None or self.static_resident_value_cache)
        )

    def _defer_int4_flag(self) -> bool:
        """INT4 quantisation of appended values waits for block completion (reference: tiered_kv_cache.py:947-952)."""
        return bool(
            self.defer_int4_append_quantization
            and self.values_fp16_gpu is not None
            and (self.fp16_value_cache_capacity is None or self.static_resident_value_cache)
        )

    def _advance_after_append(self, pos: int) -> None:
        self.num_tokens = pos + 1
        self.num_blocks = (self.num_tokens + BLOCK - 1) // BLOCK
        if pos % BLOCK == BLOCK - 1:
            self.num_quantized_blocks = pos // BLOCK + 1

    # ------------------------------------------------------------------ views / accounting

    @property
    def has_trailing_partial_block(self) -> bool:
        return self.num_tokens > 0 and self.num_tokens % self.block_size != 0

    @property
    def trailing_block_idx(self) -> int | None:
        return self.num_tokens // self.block_size if self.has_trailing_partial_block else None

    @property
    def active_tokens(self) -> int:
        return self.num_tokens

    @property
    def aligned_tokens(self) -> int:
        return ((self.num_tokens + self.block_size - 1) // self.block_size) * self.block_size

    @property
    def active_blocks(self) -> int:
        return (self.num_tokens + self.block_size - 1) // self.block_size

    def keys_int8_active(self) -> torch.Tensor:
        return self.keys_int8[:, :self.aligned_tokens, :]

    def keys_scale_active(self) -> torch.Tensor:
        return self.keys_scale[:, :self.active_blocks, :]

    def keys_zero_points_active(self) -> torch.Tensor:
        return self.keys_zero_points[:, :self.active_blocks, :]

    def correction_active(self) -> torch.Tensor:
        return self.correction[:, :self.active_blocks]

    def values_fp16_active(self):
        return None if self.values_fp16 is None else self.values_fp16[:, :self.aligned_tokens, :]

    def v_max_global(self) -> float:
        if self.values_norm_max_per_block is None:
            return 0.0
        a = self.values_norm_max_per_block[:, :self.active_blocks]
        return float(a.max().item()) if a.numel() else 0.0

    def refresh_keys_scale_max(self) -> None:
        """Recompute keys_scale_max from keys_scale (needed only after a caller
        edits keys_scale by hand)."""
        nq = self.num_quantized_blocks
        if nq:
            self.keys_scale_max.copy_(self.keys_scale[:, :nq].amax(dim=1))
        else:
            self.keys_scale_max.zero_()

    def vram_bytes(self) -> int:
        total = self.keys_int8.nelement()
        total += self.keys_scale.nelement() * 4 + self.keys_zero_points.nelement() * 4
        total += self.correction.nelement() * 4
        if self.values_fp16 is not None:
            total += self.values_fp16.nelement() * self.values_fp16.element_size()
        if self._pagein_buffer is not None:
            total += self._pagein_buffer.nelement() * self._pagein_buffer.element_size()
        if self.values_int4_packed is not None:
            total += self.values_int4_packed.nelement()
            total += self.values_int4_scales.nelement() * 2 + self.values_int4_zeros.nelement() * 2
            total += self.values_int4_errors.nelement() * 4
            total += self.values_int4_error_sums.nelement() * 4
            total += self.values_int4_error_counts.nelement() * 4
        if self.values_fp16_gpu is not None:
            total += self.values_fp16_gpu.nelement() * self.values_fp16_gpu.element_size()
        if self.keys_fp16_gpu is not None:
            total += self.keys_fp16_gpu.nelement() * self.keys_fp16_gpu.element_size()
        return int(total)

    def cpu_bytes(self) -> int:
        total = 0
        if self.keys_fp16_cpu is not None:
            total += self.keys_fp16_cpu.nelement() * self.keys_fp16_cpu.element_size()
        if self.values_fp16_cpu is not None:
            total += self.values_fp16_cpu.nelement() * self.values_fp16_cpu.element_size()
        return int(total)

    def fp16_key_block_slots_gpu(self, n_blocks: int) -> torch.Tensor:
        return self._identity_slots(n_blocks)

    def fp16_value_block_slots_gpu(self, n_blocks: int) -> torch.Tensor:
        return self._identity_slots(n_blocks)

    def _identity_slots(self, n_blocks: int) -> torch.Tensor:
        t = self._certified_workspace.get("identity_slots")
        n = int(self.keys_scale.shape[1])
        if t is None or t.numel() < n:
            t = torch.arange(n, dtype=torch.int32, device=self.keys_int8.device)
            self._certified_workspace["identity_slots"] = t
        return t[: int(n_blocks)]

    def dequantise_int4_values(self) -> torch.Tensor:
        """All INT4 values as float32 [kv, cap, 128] (debug helper; torch ops)."""
        p = self.values_int4_packed
        lo = (p & 0x0F).to(torch.float32)
        hi = ((p >> 4) & 0x0F).to(torch.float32)
        codes = torch.stack([lo, hi], dim=-1).reshape(p.shape[0], p.shape[1], -1)
        s = self.values_int4_scales.float().repeat_interleave(16, dim=-1)
        z = self.values_int4_zeros.float().repeat_interleave(16, dim=-1)
        return codes * s + z


def _layer_kv(past_kv, layer_id: int, batch_index: int = 0):
    if hasattr(past_kv, "layers"):
        return past_kv.layers[layer_id].keys[batch_index], past_kv.layers[layer_id].values[batch_index]
    return past_kv[layer_id][0][batch_index], past_kv[layer_id][1][batch_index]


def _encode_prefill_layers(entries) -> None:
    """entries: (cache, keys [KV, seq, 128], values, seq_len) per layer, caches allocated but empty.  One library
    call per (device, dtype) group quantises every layer's complete blocks straight from the prefill tensors and
    appends each ragged remainder with one launch (reference: the per-layer, per-token loop of
    tiered_kv_cache.py:1579-1701)."""
    groups: dict = {}
    for cache, keys, values, seq_len in entries:
        if values.dtype != keys.dtype:
            values = values.to(keys.dtype)
        # rows of 128 contiguous elements with one row stride per KV head are read in place (a slice of a longer
        # [KV, rows, 128] buffer, as HF caches hand out); anything else is copied once
        def row_stride(t):
            ok = t.stride(2) == 1 and t.stride(1) == HEAD_DIM and t.stride(0) % HEAD_DIM == 0
            return t.stride(0) // HEAD_DIM if ok and t.stride(0) >= t.shape[1] * HEAD_DIM else None
        rk, rv = row_stride(keys), row_stride(values)
        if rk is None or rk != rv:
            keys, values = keys.contiguous(), values.contiguous()
            rk = keys.shape[1]
        groups.setdefault((keys.device, keys.dtype), []).append((cache, keys, values, seq_len, rk))
    for (dev, dtype), group in groups.items():
        items = (_lib.CqaPrefillItem * len(group))()
        for i, (cache, keys, values, seq_len, rows) in enumerate(group):
            items[i].cache = cache._desc()
            items[i].k_src = keys.data_ptr()
            items[i].v_src = values.data_ptr()
            items[i].src_rows = rows
            items[i].n_tokens = seq_len
            items[i].defer_int4 = 1 if cache._defer_int4_flag() else 0
        with _lib.on_device(dev):
            rc = _lib.lib().cqa_prefill_encode(items, len(group), _lib.dtype_code(dtype), _lib.current_stream(dev))
        _lib.check(rc, "cqa_prefill_encode")
        for cache, _k, _v, seq_len, _rows in group:
            cache.num_tokens = seq_len
            cache.num_blocks = (seq_len + BLOCK - 1) // BLOCK
            cache.num_quantized_blocks = seq_len // BLOCK


def create_tiered_cache_int4v_from_model(past_kv, layer_ids: list, block_size: int = 16, group_size: int = 16,
                                         max_new_tokens: int = 512,
                                         fp16_key_cache_capacity: int | None = None,
                                         fp16_value_cache_capacity: int | None = None,
                                         defer_int4_append_quantization: bool | None = None,
                                         batch_index: int = 0) -> dict:
    """Per-layer INT8K/INT4V caches from HF past_key_values, sequence `batch_index` of the prefill's batch
    (reference: tiered_kv_cache.py:1579-1641, which takes sequence 0).  Every layer is allocated first, then all of them are encoded by one
    library call, ragged remainders included."""
    if defer_int4_append_quantization is None:
        defer_int4_append_quantization = fp16_value_cache_capacity is None
    caches, entries = {}, []
    for layer_id in layer_ids:
        keys, values = _layer_kv(past_kv, layer_id, batch_index)
        seq_len = keys.shape[1]
        aligned = (seq_len // block_size) * block_size
        cache = TieredKeyCacheLayer.from_fp16_cache_int4v(
            keys[:, :aligned, :], values[:, :aligned, :],
            block_size=block_size, group_size=group_size,
            max_new_tokens=max_new_tokens + (seq_len - aligned),
            fp16_key_cache_capacity=fp16_key_cache_capacity,
            fp16_value_cache_capacity=fp16_value_cache_capacity,
            defer_int4_append_quantization=bool(defer_int4_append_quantization), _encode=False,
        )
        cache.num_tokens = cache.num_blocks = cache.num_quantized_blocks = 0
        entries.append((cache, keys, values, seq_len))
        caches[layer_id] = cache
    _encode_prefill_layers(entries)
    return caches


def create_tiered_cache_from_model(past_kv, layer_ids: list, block_size: int = 16, max_new_tokens: int = 512,
                                   fp16_key_cache_capacity: int | None = None) -> dict:
    """Per-layer INT8-key / model-dtype-value caches (reference: tiered_kv_cache.py:1644-1701)."""
    caches, entries = {}, []
    for layer_id in layer_ids:
        keys, values = _layer_kv(past_kv, layer_id)
        seq_len = keys.shape[1]
        aligned = (seq_len // block_size) * block_size
        cache = TieredKeyCacheLayer.from_fp16_cache(
            keys[:, :aligned, :], values[:, :aligned, :],
            block_size=block_size, max_new_tokens=max_new_tokens + (seq_len - aligned),
            fp16_key_cache_capacity=fp16_key_cache_capacity, _encode=False,
        )
        cache.num_tokens = cache.num_blocks = cache.num_quantized_blocks = 0
        entries.append((cache, keys, values, seq_len))
        caches[layer_id] = cache
    _encode_prefill_layers(entries)
    return caches
