"""ctypes binding of libcqa_b200.so (the C ABI declared in include/cqa_b200.h).

The library is the only compute path: there is no CPU or PyTorch fallback.
`lib()` raises if the shared object is missing or does not export every
declared symbol.
"""
from __future__ import annotations

import ctypes as C
from pathlib import Path

HERE = Path(__file__).resolve().parent
LIB_PATH = HERE / "libcqa_b200.so"

CQA_F32, CQA_F16, CQA_BF16 = 0, 1, 2
MAX_RANKING_K = 32
MAX_SORT_BLOCKS = 16384

SYMBOLS = [
    "cqa_version", "cqa_last_error", "cqa_quantize_blocks", "cqa_append_token", "cqa_int4_quantise",
    "cqa_score_blocks", "cqa_select", "cqa_fp16_block_scores", "cqa_delta_bound", "cqa_certify",
    "cqa_attend", "cqa_attend_static", "cqa_layer_step", "cqa_suggest_splits",
    "cqa_select_certify_local", "cqa_rescore_owned", "cqa_certify_given", "cqa_merge_partials",
    "cqa_decode_step_host", "cqa_decode_step_host_async", "cqa_decode_token_host", "cqa_hot_tier_update",
    "cqa_peer_buffer_bytes", "cqa_peer_alloc", "cqa_peer_free", "cqa_peer_export", "cqa_peer_import", "cqa_peer_close",
    "cqa_sharded_layer_step", "cqa_peer_status",
    "cqa_hot_tier_ensure", "cqa_page_in_blocks", "cqa_page_in_by_slots", "cqa_dense_attend",
    "cqa_launch_count", "cqa_wait_timeouts", "cqa_layer_step_batched", "cqa_prefill_encode",
]
PARTIAL_STRIDE = 130

vp = C.c_void_p


class CqaCache(C.Structure):
    _fields_ = [
        ("kv_heads", C.c_int32), ("gqa_group", C.c_int32), ("t2_dtype", C.c_int32), ("reserved", C.c_int32),
        ("cap_tokens", C.c_int64), ("max_blocks", C.c_int64),
        ("keys_int8", vp), ("keys_scale", vp), ("keys_zero_points", vp), ("correction", vp),
        ("sigma_max", vp), ("values_int4_packed", vp), ("values_int4_scales", vp),
        ("values_int4_zeros", vp), ("values_int4_errors", vp), ("values_int4_error_sums", vp),
        ("values_int4_error_counts", vp), ("values_norm_max", vp),
        ("keys_t2", vp), ("keys_t2_rows", C.c_int64), ("values_t2", vp), ("values_t2_rows", C.c_int64),
        ("key_slots", vp), ("value_slots", vp),
        ("keys_t2_backing", vp), ("values_t2_backing", vp), ("t2_backing_rows", C.c_int64),
    ]


class CqaKnobs(C.Structure):
    _fields_ = [
        ("q_scale", C.c_float), ("tau_cov", C.c_float), ("rung1_threshold", C.c_float),
        ("rung1_multiplier", C.c_float), ("eps_guard", C.c_float), ("exploration_rate", C.c_float),
        ("v_tolerance", C.c_float),
        ("k_min", C.c_int32), ("k_max", C.c_int32), ("ranking_r", C.c_int32),
        ("top_k_fp16_keys", C.c_int32), ("ranking_fallback", C.c_int32), ("rung3_recompute", C.c_int32),
        ("score_consistency", C.c_int32), ("value_mode_tight", C.c_int32),
        ("force_trailing_value_fp16", C.c_int32),
    ]


class CqaHeadCert(C.Structure):
    _fields_ = [
        ("k_star", C.c_int32), ("k_star_base", C.c_int32), ("k_star_expanded", C.c_int32),
        ("rung1_triggered", C.c_int32), ("exploration_blocks", C.c_int32),
        ("ranking_disagree", C.c_int32), ("ranking_disagree_r1", C.c_int32),
        ("ranking_disagree_r3", C.c_int32), ("boundary_triggered", C.c_int32), ("rung3", C.c_int32),
        ("consistency_violation", C.c_int32), ("value_promoted_blocks", C.c_int32), ("dense", C.c_int32),
        ("reserved", C.c_int32 * 3),
        ("tail_mass", C.c_float), ("tau_actual", C.c_float), ("m_global", C.c_float),
        ("total_mass", C.c_float), ("delta", C.c_float), ("e_pre", C.c_float), ("e_val", C.c_float),
        ("boundary_ub", C.c_float), ("ell_fp16_r", C.c_float), ("fp16_top1", C.c_float),
        ("fp16_top2", C.c_float), ("int8_top1", C.c_float),
        ("top_blocks", C.c_int32 * MAX_RANKING_K), ("fp16_scores", C.c_float * MAX_RANKING_K),
        ("fp16_logmass", C.c_float * MAX_RANKING_K),
    ]


class CqaWorkspace(C.Structure):
    _fields_ = [
        ("ld", C.c_int64),
        ("m_b", vp), ("s_b", vp), ("token_scores", vp), ("mass_frac", vp),
        ("topk_mask", vp), ("value_mask", vp), ("explore_mask", vp),
        ("sorted_idx", vp), ("sorted_cumsum", vp),
        ("sel_width", C.c_int32), ("num_splits", C.c_int32), ("dense_splits", C.c_int32),
        ("reserved", C.c_int32),
        ("part_m", vp), ("part_l", vp), ("part_acc", vp),
        ("dense_m", vp), ("dense_l", vp), ("dense_acc", vp),
        ("cert", vp), ("any_flags", vp), ("out", vp), ("tickets", vp),
        ("given_fp16", vp), ("partial_out", vp),
        ("rng_seed", C.c_uint64), ("rng_offset", C.c_uint64),
        ("shard_stride", C.c_int64), ("shard_chunk", C.c_int64), ("shard_rank_stride", C.c_int64),
        ("shard_ranks", C.c_int32), ("given_ranks", C.c_int32), ("given_rank_stride", C.c_int64),
        ("wait_flags", vp), ("wait_n", C.c_int32), ("wait_skip", C.c_int32), ("wait_value", C.c_int32),
        ("wait_spins", C.c_int32), ("wait_status", vp),
        ("peer_xb", vp * 8), ("peer_flags_b", vp * 8), ("peer_partial", vp * 8), ("peer_flag_c", vp * 8),
        ("peer_ticket_c", vp), ("peer_first_block", C.c_int64), ("peer_n_local", C.c_int64),
        ("peer_world", C.c_int32), ("peer_rank", C.c_int32), ("peer_step", C.c_int32), ("reserved3", C.c_int32),
    ]


MAX_PEERS = 8


class CqaPeers(C.Structure):
    _fields_ = [
        ("world", C.c_int32), ("rank", C.c_int32), ("rows", C.c_int32), ("n_heads", C.c_int32),
        ("chunk", C.c_int64), ("base", vp * MAX_PEERS),
    ]


class CqaHotTier(C.Structure):
    _fields_ = [
        ("key_capacity_blocks", C.c_int32), ("value_capacity_blocks", C.c_int32),
        ("max_fill_blocks", C.c_int32), ("reserved", C.c_int32),
        ("key_slots", vp), ("value_slots", vp), ("key_owner", vp), ("value_owner", vp),
        ("key_stamp", vp), ("value_stamp", vp), ("work", vp), ("counters", vp),
    ]


class CqaLayerCall(C.Structure):
    _fields_ = [
        ("cache", vp), ("ws", vp), ("qkv_host", vp), ("out_host", vp),
        ("pos", C.c_int64), ("defer_int4", C.c_int32), ("reserved", C.c_int32),
    ]


class CqaBatchItem(C.Structure):
    _fields_ = [
        ("cache", CqaCache), ("ws", CqaWorkspace), ("q", vp), ("k_new", vp), ("v_new", vp),
        ("pos", C.c_int64), ("defer_int4", C.c_int32), ("reserved", C.c_int32),
    ]


class CqaPrefillItem(C.Structure):
    _fields_ = [
        ("cache", CqaCache), ("k_src", vp), ("v_src", vp), ("src_rows", C.c_int64), ("n_tokens", C.c_int64),
        ("defer_int4", C.c_int32), ("reserved", C.c_int32),
    ]


CERT_BYTES = C.sizeof(CqaHeadCert)

_lib = None


class CqaError(RuntimeError):
    pass


def lib() -> C.CDLL:
    """Load the CUDA library (once).  Fails loudly when it has not been built."""
    global _lib
    if _lib is not None:
        return _lib
    if not LIB_PATH.exists():
        raise CqaError(
            f"{LIB_PATH} is missing: build it with "
            "`python certified-quantised-attention_b200/build.py` (needs nvcc); "
            "this package has no CPU fallback"
        )
    L = C.CDLL(str(LIB_PATH))
    missing = [s for s in SYMBOLS if not hasattr(L, s)]
    if missing:
        raise CqaError(f"{LIB_PATH} does not export {missing}")
    L.cqa_version.restype = C.c_char_p
    L.cqa_last_error.restype = C.c_char_p
    i64, i32, f32 = C.c_int64, C.c_int, C.c_float
    pc, pk, pw = C.POINTER(CqaCache), C.POINTER(CqaKnobs), C.POINTER(CqaWorkspace)
    L.cqa_quantize_blocks.argtypes = [pc, vp, vp, i32, i64, i64, i64, vp]
    L.cqa_append_token.argtypes = [pc, vp, vp, i32, i64, i32, vp]
    L.cqa_int4_quantise.argtypes = [vp, i32, i64, vp, vp, vp, vp, vp, vp]
    L.cqa_score_blocks.argtypes = [pc, vp, i32, i64, f32, vp, vp, i64, vp, vp]
    L.cqa_select.argtypes = [pc, pk, pw, i64, i64, vp, i64, vp]
    L.cqa_fp16_block_scores.argtypes = [pc, vp, i32, vp, i32, i64, f32, vp, vp, vp]
    L.cqa_delta_bound.argtypes = [pc, vp, i32, vp, vp]
    L.cqa_certify.argtypes = [pc, pk, pw, vp, i32, i64, i64, vp]
    L.cqa_attend.argtypes = [pc, pw, vp, i32, i64, i64, i64, i32, f32, vp]
    L.cqa_attend_static.argtypes = [pc, pw, vp, i32, i64, i64, i64, i32, f32, vp]
    L.cqa_layer_step.argtypes = [pc, pk, pw, vp, i32, i64, i64, vp, i64, vp]
    L.cqa_suggest_splits.argtypes = [i32, i32, i64, C.POINTER(C.c_int), C.POINTER(C.c_int)]
    L.cqa_select_certify_local.argtypes = [pc, pk, pw, i64, i64, vp, i64, vp]
    L.cqa_rescore_owned.argtypes = [pc, vp, vp, i32, i64, i64, f32, vp, vp]
    L.cqa_certify_given.argtypes = [pc, pk, pw, vp, i32, i64, i64, vp]
    L.cqa_merge_partials.argtypes = [vp, i32, i32, vp, vp]
    L.cqa_decode_step_host.argtypes = [pc, pk, pw, vp, vp, i32, i64, i32, vp, vp]
    L.cqa_decode_step_host_async.argtypes = [pc, pk, pw, vp, vp, i32, i64, i32, vp, vp]
    L.cqa_decode_token_host.argtypes = [C.POINTER(CqaLayerCall), i32, pk, vp, i32, vp]
    L.cqa_hot_tier_update.argtypes = [pc, pw, C.POINTER(CqaHotTier), i64, vp]
    L.cqa_peer_buffer_bytes.argtypes = [i32, i32, i32, i64]
    L.cqa_peer_alloc.argtypes = [i64, C.POINTER(vp)]
    L.cqa_peer_free.argtypes = [vp]
    L.cqa_peer_export.argtypes = [vp, C.c_char_p]
    L.cqa_peer_import.argtypes = [C.c_char_p, C.POINTER(vp)]
    L.cqa_peer_close.argtypes = [vp]
    L.cqa_peer_status.argtypes = [C.POINTER(CqaPeers), C.POINTER(C.c_int32), i32]
    L.cqa_sharded_layer_step.argtypes = [pc, pc, pk, pw, pw, C.POINTER(CqaPeers), vp, i32, i64, i64, i64, i64, i64, i64,
                                         i32, i64, i32, vp, vp]
    L.cqa_dense_attend.argtypes = [pc, pw, vp, i32, i64, f32, vp]
    L.cqa_hot_tier_ensure.argtypes = [pc, C.POINTER(CqaHotTier), i32, vp, i64, vp]
    L.cqa_page_in_blocks.argtypes = [vp, i64, vp, i64, i32, i32, vp, vp, i64, vp, i64, vp, i64, i64, vp]
    L.cqa_page_in_by_slots.argtypes = [vp, i64, vp, i64, i32, i32, vp, i64, i64, vp]
    for s in SYMBOLS[2:]:
        getattr(L, s).restype = C.c_int
    L.cqa_peer_buffer_bytes.restype = C.c_int64
    L.cqa_prefill_encode.argtypes = [C.POINTER(CqaPrefillItem), i32, i32, vp]
    L.cqa_layer_step_batched.argtypes = [C.POINTER(CqaBatchItem), i32, vp, pk, i32, i32, vp]
    L.cqa_wait_timeouts.argtypes = [C.POINTER(C.c_int), i32]
    L.cqa_launch_count.argtypes = [i32]
    L.cqa_launch_count.restype = C.c_int64
    _lib = L
    return L


def check(rc: int, what: str = "") -> None:
    if rc != 0:
        msg = lib().cqa_last_error().decode("utf-8", "replace")
        if rc in (-1, -3, -4):
            raise ValueError(f"{what}: {msg} (status {rc})")
        raise CqaError(f"{what}: {msg} (status {rc})")


def dtype_code(torch_dtype) -> int:
    import torch

    if torch_dtype == torch.float32:
        return CQA_F32
    if torch_dtype == torch.float16:
        return CQA_F16
    if torch_dtype == torch.bfloat16:
        return CQA_BF16
    raise ValueError(f"unsupported dtype {torch_dtype}; expected float32, float16 or bfloat16")


def ptr(t) -> int | None:
    return None if t is None else t.data_ptr()


def current_stream(device) -> int:
    """Raw cudaStream_t of torch's current stream on `device` (no Stream object is built)."""
    import torch

    idx = device.index if device.index is not None else torch.cuda.current_device()
    return torch._C._cuda_getCurrentRawStream(idx)


class on_device:
    """`with on_device(dev):` makes `dev` the current CUDA device, and is free when it already is."""

    __slots__ = ("idx", "prev")

    def __init__(self, device):
        self.idx = device.index
        self.prev = -1

    def __enter__(self):
        import torch

        if self.idx is not None:
            cur = torch.cuda.current_device()
            if cur != self.idx:
                self.prev = cur
                torch.cuda.set_device(self.idx)
        return self

    def __exit__(self, *exc):
        if self.prev >= 0:
            import torch

            torch.cuda.set_device(self.prev)
        return False
