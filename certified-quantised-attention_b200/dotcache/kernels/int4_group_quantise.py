"""Per-group INT4 quantisation of value vectors (group size 16), on the GPU.

Same names and return layout as the reference's
`dotcache/kernels/int4_group_quantise.py` (quantise_int4_grouped:22-88,
dequantise_int4_grouped:91-120, quantise_int4_grouped_block:123-151).
Packing: two codes per byte, low nibble = even channel.
"""
from __future__ import annotations

import ctypes as C

import torch

from cqa_b200 import _lib

GROUP_SIZE = 16


def quantise_int4_grouped(values: torch.Tensor, group_size: int = GROUP_SIZE) -> dict:
    """values [T, 128] (float32/float16/bfloat16, CUDA) -> dict with
    data_packed u8 [T,64], scales/zeros f16 [T,8], per_token_error,
    per_token_abs_error f32 [T], error_bound, abs_error_bound (0-dim)."""
    if group_size != GROUP_SIZE:
        raise ValueError("group_size must be 16 (fixed by the kernels)")
    if not values.is_cuda:
        raise RuntimeError("quantise_int4_grouped needs a CUDA tensor; there is no CPU fallback")
    T, hd = values.shape
    if hd != 128:
        raise ValueError("head_dim must be 128")
    x = values.contiguous()
    dev = x.device
    packed = torch.empty(T, hd // 2, dtype=torch.uint8, device=dev)
    scales = torch.empty(T, hd // 16, dtype=torch.float16, device=dev)
    zeros = torch.empty(T, hd // 16, dtype=torch.float16, device=dev)
    rel = torch.empty(T, dtype=torch.float32, device=dev)
    ab = torch.empty(T, dtype=torch.float32, device=dev)
    with torch.cuda.device(dev):
        _lib.check(_lib.lib().cqa_int4_quantise(
            x.data_ptr(), _lib.dtype_code(x.dtype), T, packed.data_ptr(), scales.data_ptr(), zeros.data_ptr(),
            rel.data_ptr(), ab.data_ptr(), _lib.current_stream(dev)), "cqa_int4_quantise")
    return {
        "data_packed": packed, "scales": scales, "zeros": zeros, "group_size": group_size,
        "per_token_error": rel, "per_token_abs_error": ab,
        "error_bound": rel.max() if T else torch.zeros((), device=dev),
        "abs_error_bound": ab.max() if T else torch.zeros((), device=dev),
    }


def dequantise_int4_grouped(packed: torch.Tensor, scales: torch.Tensor, zeros: torch.Tensor,
                            group_size: int = GROUP_SIZE) -> torch.Tensor:
    """Inverse of the packing, returned as float16 [T, 128] (inspection helper, torch ops)."""
    T = packed.shape[0]
    lo = (packed & 0x0F).to(torch.float32)
    hi = ((packed >> 4) & 0x0F).to(torch.float32)
    codes = torch.stack([lo, hi], dim=-1).reshape(T, -1)
    s = scales.float().repeat_interleave(group_size, dim=-1)
    z = zeros.float().repeat_interleave(group_size, dim=-1)
    return (codes * s + z).half()


def quantise_int4_grouped_block(values: torch.Tensor, block_size: int = 16, group_size: int = GROUP_SIZE) -> dict:
    """[kv, N, 128] -> per-token INT4 data plus per-block error bounds (max) and sums."""
    kv, N, hd = values.shape
    nb = N // block_size
    r = quantise_int4_grouped(values.reshape(kv * N, hd), group_size)
    pte = r["per_token_error"].reshape(kv, nb, block_size)
    pta = r["per_token_abs_error"].reshape(kv, nb, block_size)
    return {
        "data_packed": r["data_packed"].reshape(kv, N, hd // 2),
        "scales": r["scales"].reshape(kv, N, hd // group_size),
        "zeros": r["zeros"].reshape(kv, N, hd // group_size),
        "error_bounds": pte.amax(dim=2), "error_sums": pte.sum(dim=2),
        "abs_error_bounds": pta.amax(dim=2), "group_size": group_size,
    }
