"""Page-in of Tier-2 blocks under the reference's native-extension names
(dotcache/backends/cuda_pagein.py: cuda_pagein_available:23,
page_in_fp16_blocks_cuda:68, page_in_fp16_blocks_packed_cuda:98,
page_in_fp16_blocks_by_slots_cuda:132), over the gather kernels of
libcqa_b200.so (csrc/hot_tier.cu).

The decode path of this package does not call these: its bounded hot tier
keeps residency on the device (TieredKeyCacheLayer.hot_tier_counters,
cqa_hot_tier_update).  They exist for callers that drive residency from the
host the way the reference does: a host LRU decides which blocks to load and
evict, these functions move the rows and update the device slot table.
"""
from __future__ import annotations

import ctypes as C
from typing import Any

import torch

from cqa_b200 import _lib


def cuda_pagein_enabled() -> bool:
    return True


def cuda_pagein_available() -> bool:
    """True when a CUDA device is present and the library loads."""
    try:
        if not torch.cuda.is_available():
            return False
        _lib.lib()
    except Exception:
        return False
    return True


def _geometry(src_cpu: torch.Tensor, dst_gpu: torch.Tensor):
    if src_cpu.dim() != 3 or dst_gpu.dim() != 3 or src_cpu.shape[0] != dst_gpu.shape[0] \
            or src_cpu.shape[2] != dst_gpu.shape[2] or src_cpu.dtype != dst_gpu.dtype:
        raise ValueError("src_cpu and dst_gpu must be [kv, rows, dim] tensors of the same dtype, kv and dim")
    if not dst_gpu.is_cuda or not dst_gpu.is_contiguous() or not src_cpu.is_contiguous():
        raise ValueError("dst_gpu must be a contiguous CUDA tensor and src_cpu contiguous")
    if not (src_cpu.is_cuda or src_cpu.is_pinned()):
        raise ValueError("src_cpu must be pinned host memory (or a CUDA tensor): the gather kernel reads it in place")
    row_bytes = int(src_cpu.shape[2]) * src_cpu.element_size()
    if row_bytes % 16:
        raise ValueError("rows must be a multiple of 16 bytes")
    return int(src_cpu.shape[0]), int(src_cpu.shape[1]), int(dst_gpu.shape[1]), row_bytes


def _stage(host_list: torch.Tensor, dev_buf: torch.Tensor, dtype) -> tuple[torch.Tensor, int]:
    n = int(host_list.numel())
    if n == 0:
        return dev_buf, 0
    if dev_buf.numel() < n or dev_buf.dtype != dtype or not dev_buf.is_cuda:
        raise ValueError("device index buffer is too small, of the wrong dtype or not on the GPU")
    dev_buf[:n].copy_(host_list.reshape(-1).to(dtype), non_blocking=True)
    return dev_buf, n


def page_in_fp16_blocks_cuda(*, src_cpu: Any, dst_gpu: Any, loaded_blocks_cpu: Any, loaded_slots_cpu: Any,
                             evicted_blocks_cpu: Any, loaded_blocks_gpu: Any, loaded_slots_gpu: Any,
                             evicted_blocks_gpu: Any, slot_table_gpu: Any, block_size: int,
                             active_tokens: int) -> int:
    """Copy block loaded_blocks[i] of `src_cpu` into slot loaded_slots[i] of `dst_gpu`, set
    slot_table[evicted] = -1 and slot_table[loaded] = slot.  The *_cpu index tensors (int64 blocks, int32 slots)
    are staged through the *_gpu buffers.  Returns the bytes moved."""
    if block_size != 16:
        raise ValueError("block_size must be 16")
    kv, src_rows, dst_rows, row_bytes = _geometry(src_cpu, dst_gpu)
    dev = dst_gpu.device
    lb, n_loaded = _stage(loaded_blocks_cpu, loaded_blocks_gpu, torch.int64)
    ls, n_slots = _stage(loaded_slots_cpu, loaded_slots_gpu, torch.int32)
    ev, n_evicted = _stage(evicted_blocks_cpu, evicted_blocks_gpu, torch.int64)
    if n_loaded != n_slots:
        raise ValueError("loaded_blocks and loaded_slots differ in length")
    table = slot_table_gpu
    with torch.cuda.device(dev):
        _lib.check(_lib.lib().cqa_page_in_blocks(
            src_cpu.data_ptr(), src_rows, dst_gpu.data_ptr(), dst_rows, kv, row_bytes,
            lb.data_ptr() if n_loaded else None, ls.data_ptr() if n_loaded else None, n_loaded,
            ev.data_ptr() if n_evicted else None, n_evicted,
            None if table is None else table.data_ptr(), 0 if table is None else int(table.numel()),
            int(active_tokens), _lib.current_stream(dev)), "cqa_page_in_blocks")
    full_rows = 0
    for b in loaded_blocks_cpu.reshape(-1).tolist():
        full_rows += max(0, min(16, int(active_tokens) - int(b) * 16))
    return kv * full_rows * row_bytes


def page_in_fp16_blocks_packed_cuda(*, src_cpu: Any, dst_gpu: Any, stage_cpu: Any = None, stage_gpu: Any = None,
                                    loaded_blocks_cpu: Any, loaded_slots_cpu: Any, evicted_blocks_cpu: Any,
                                    loaded_blocks_gpu: Any, loaded_slots_gpu: Any, evicted_blocks_gpu: Any,
                                    slot_table_gpu: Any, block_size: int, active_tokens: int) -> int:
    """Same result as page_in_fp16_blocks_cuda.  The reference packs the rows into a pinned staging buffer first
    (one large copy instead of many small ones); the gather kernel here reads the pinned source in place, so the
    staging tensors are accepted and left untouched."""
    return page_in_fp16_blocks_cuda(
        src_cpu=src_cpu, dst_gpu=dst_gpu, loaded_blocks_cpu=loaded_blocks_cpu, loaded_slots_cpu=loaded_slots_cpu,
        evicted_blocks_cpu=evicted_blocks_cpu, loaded_blocks_gpu=loaded_blocks_gpu,
        loaded_slots_gpu=loaded_slots_gpu, evicted_blocks_gpu=evicted_blocks_gpu, slot_table_gpu=slot_table_gpu,
        block_size=block_size, active_tokens=active_tokens)


def page_in_fp16_blocks_by_slots_cuda(*, src_cpu: Any, dst_gpu: Any, block_slots_gpu: Any, block_size: int,
                                      active_tokens: int, n_blocks: int) -> None:
    """Copy every block i < n_blocks whose slot block_slots_gpu[i] is >= 0 into that slot of `dst_gpu`."""
    if block_size != 16:
        raise ValueError("block_size must be 16")
    kv, src_rows, dst_rows, row_bytes = _geometry(src_cpu, dst_gpu)
    slots = block_slots_gpu
    if not slots.is_cuda or slots.dtype != torch.int32 or slots.numel() < n_blocks or not slots.is_contiguous():
        raise ValueError("block_slots_gpu must be a contiguous int32 CUDA tensor of at least n_blocks entries")
    dev = dst_gpu.device
    with torch.cuda.device(dev):
        _lib.check(_lib.lib().cqa_page_in_by_slots(
            src_cpu.data_ptr(), src_rows, dst_gpu.data_ptr(), dst_rows, kv, row_bytes, slots.data_ptr(),
            int(n_blocks), int(active_tokens), _lib.current_stream(dev)), "cqa_page_in_by_slots")
