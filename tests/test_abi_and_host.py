"""CPU-side checks: the C-ABI library loads and exports every declared symbol,
the ctypes structures match the header's layout, and host-side helpers."""
from __future__ import annotations

import ctypes as C
import re
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT / "certified-quantised-attention_b200"))

from cqa_b200 import _lib, roofline, synth  # noqa: E402


def test_library_exports_every_declared_symbol():
    header = (ROOT / "include" / "cqa_b200.h").read_text()
    declared = set(re.findall(r"\b(cqa_[a-z0-9_]+)\s*\(", header))
    assert declared, "no declarations parsed"
    L = _lib.lib()
    for name in sorted(declared):
        assert hasattr(L, name), f"{name} declared in include/cqa_b200.h but not exported"
    assert set(_lib.SYMBOLS) == declared
    assert b"sm_100a" in L.cqa_version()


def test_struct_layout_matches_header(tmp_path):
    src = tmp_path / "sz.c"
    src.write_text(
        '#include <stdio.h>\n#include <stddef.h>\n#include "cqa_b200.h"\n'
        "int main(void){printf(\"%zu %zu %zu %zu %zu %zu %zu\\n\", sizeof(cqa_cache), sizeof(cqa_knobs),"
        " sizeof(cqa_head_cert), sizeof(cqa_workspace), offsetof(cqa_cache, keys_t2),"
        " offsetof(cqa_workspace, cert), offsetof(cqa_head_cert, top_blocks));return 0;}\n")
    exe = tmp_path / "sz"
    subprocess.check_call(["gcc", "-I", str(ROOT / "include"), "-o", str(exe), str(src)])
    got = [int(x) for x in subprocess.check_output([str(exe)]).split()]
    want = [C.sizeof(_lib.CqaCache), C.sizeof(_lib.CqaKnobs), C.sizeof(_lib.CqaHeadCert),
            C.sizeof(_lib.CqaWorkspace), _lib.CqaCache.keys_t2.offset, _lib.CqaWorkspace.cert.offset,
            _lib.CqaHeadCert.top_blocks.offset]
    assert got == want


def test_argument_errors_without_gpu():
    """Argument validation happens before any CUDA call."""
    L = _lib.lib()
    c = _lib.CqaCache()
    assert L.cqa_quantize_blocks(C.byref(c), None, None, 0, 0, 0, 0, None) == -1
    assert b"NULL" in L.cqa_last_error()
    assert L.cqa_int4_quantise(None, 0, 4, None, None, None, None, None, None) == -1
    ns, ds = C.c_int(0), C.c_int(0)
    assert L.cqa_suggest_splits(0, 4, 100, C.byref(ns), C.byref(ds)) == -1
    with pytest.raises(ValueError):
        _lib.check(-1, "x")
    with pytest.raises(_lib.CqaError):
        _lib.check(-2, "x")


def test_host_api_refuses_cpu_tensors():
    import torch
    from dotcache.kernels import certified_attention as ca
    from dotcache.kernels.tiered_kv_cache import TieredKeyCacheLayer
    from dotcache.kernels.int4_group_quantise import quantise_int4_grouped

    k = torch.zeros(2, 32, 128)
    with pytest.raises(RuntimeError, match="no CPU fallback"):
        TieredKeyCacheLayer.from_fp16_cache_int4v(k, k)
    with pytest.raises(RuntimeError, match="no CPU fallback"):
        quantise_int4_grouped(torch.zeros(4, 128))
    with pytest.raises(RuntimeError, match="no CPU fallback"):
        ca.compute_adaptive_topk_mask(torch.zeros(4, 8), torch.ones(4, 8))


def test_selection_width():
    from dotcache.kernels.certified_attention import _selection_width

    assert _selection_width(128, 0.02, 2.0, 2048) == 256
    assert _selection_width(128, 0.02, 2.0, 200) == 200
    assert _selection_width(128, 0.02, 2.0, 64) == 64
    assert _selection_width(128, None, 2.0, 2048) == 128
    assert _selection_width(None, 0.02, 2.0, 2048) == 2048


def test_synth_is_deterministic_and_planted():
    a = synth.make_layer_inputs(3, 1024, kv_heads=2, dtype="bfloat16", n_planted_blocks=4)
    b = synth.make_layer_inputs(3, 1024, kv_heads=2, dtype="bfloat16", n_planted_blocks=4)
    assert np.array_equal(a.k, b.k) and np.array_equal(a.q, b.q)
    # bf16-representable
    assert np.array_equal(synth.round_to_dtype(a.k, "bfloat16"), a.k)
    blk = int(a.planted_blocks[0])
    h = int(a.planted_heads[0, 0])
    kb = a.k[0, blk * 16:(blk + 1) * 16]
    cos = (kb @ a.q[h]) / (np.linalg.norm(kb, axis=1) * np.linalg.norm(a.q[h]))
    assert np.all(np.abs(cos - 0.9) < 0.02)
    q1, k1, v1 = synth.decode_step_inputs(a, 5, dtype="bfloat16")
    q2, _, _ = synth.decode_step_inputs(a, 5, dtype="bfloat16")
    assert np.array_equal(q1, q2) and k1.shape == (2, 1, 128)


def test_roofline_bytes():
    H, nq = 8, 10
    tk = np.zeros((H, nq + 1), dtype=np.uint8)
    vm = np.zeros((H, nq + 1), dtype=np.uint8)
    b = roofline.step_bytes(tk, vm, nq, nq, 16, 4)
    assert b["score"] == 2 * nq * 16 * 192 and b["attend"] == 2 * nq * 16 * 96
    assert b["score"] + b["attend"] == roofline.tier1_floor_bytes(nq * 16, 2)
    tk[0, 3] = 1
    tk[1, 3] = 1          # same KV group: counted once
    vm[5, 7] = 1          # split group: block 7 of kv 1 counts INT4 and FP16
    tk[:, nq] = 1
    vm[:, nq] = 1
    b2 = roofline.step_bytes(tk, vm, nq, nq + 1, 5, 4)
    assert b2["fp16_key_bytes"] == 16 * 256
    assert b2["fp16_value_bytes"] == 16 * 256 and b2["int4_value_bytes"] == 2 * nq * 16 * 96
    assert b2["attend"] == 16 * 256 + 16 * 256 + 2 * nq * 16 * 96 + 2 * 5 * 512


def test_batch_split_policy_avoids_a_nearly_empty_wave():
    """Phase-2 splits per (sequence, KV head) of a batch: never more than the sequence's limit or one split per 8
    blocks, one sequence keeps the one-sequence split, and a batch is never given a count that spills a few CTAs
    into a second wave when one fewer per head fits in one (8 sequences x 8 KV heads on 296 slots: 4, not 5)."""
    from dotcache.kernels.certified_attention import _batch_splits

    slots = 296
    assert _batch_splits(slots, 8, 8193, 37) == 37
    for heads, nact in ((64, 2049), (64, 8193), (256, 2049), (512, 513), (32, 4097)):
        p = _batch_splits(slots, heads, nact, 37)
        assert 1 <= p <= min(37, max(1, nact // 8))
        waves = -(-heads * p // slots)
        fill = heads * p / (waves * slots)
        assert waves >= 4 or fill > 0.8 or p == 1, (heads, nact, p, waves, fill)
    assert _batch_splits(slots, 64, 2049, 37) == 4
    assert _batch_splits(slots, 8, 40, 37) <= 5
