"""cqa_attend_static: the attend entry point for callers that cannot allocate
device memory (its split partials live in an array inside the library).

Collected last on purpose: a run that stops at the first failure has already
run every other test.  The check is that it returns what cqa_attend returns on
the same inputs, twice in a row (the second call finds the first call's
leftovers in the shared array), and that it refuses sizes beyond its limits.
"""
from __future__ import annotations

import ctypes as C

import numpy as np
import pytest
import torch

import golden_cases as gc
from cqa_b200 import _lib, synth

pytestmark = pytest.mark.gpu


def _attend(fn, cache, ws, wstruct, q, nq, nact, last_valid):
    desc = cache._desc(4)
    rc = fn(C.byref(desc), C.byref(wstruct), q.data_ptr(), _lib.dtype_code(q.dtype), nq, nact, cache.num_tokens,
            last_valid, 1.0 / np.sqrt(128.0), _lib.current_stream(q.device))
    _lib.check(rc, "attend")
    torch.cuda.synchronize()
    return ws.out.clone()


def test_static_scratch_attend_matches_caller_scratch_attend():
    import cuda_harness as hz
    from dotcache.kernels import certified_attention as ca

    L = _lib.lib()
    dtype = "bfloat16"
    base = synth.make_layer_inputs(31, 4096 + 6, dtype=dtype, n_planted_blocks=16)
    cc = hz.make_cuda_cache(base.k[:, :4096], base.v[:, :4096], dtype, 64)
    for t in range(4096, 4102):
        cc.append_token(hz.to_dev(base.k[:, t:t + 1], dtype), hz.to_dev(base.v[:, t:t + 1], dtype))
    knobs = dict(gc.PAPER_KNOBS, ranking_r=4)     # r=4: some heads take the dense recompute as well
    for call in range(2):
        q_np, kn, vn = synth.decode_step_inputs(base, call, dtype=dtype)
        cc.append_token(hz.to_dev(kn, dtype), hz.to_dev(vn, dtype))
        q = hz.to_dev(q_np, dtype)
        # one full layer step fills the masks, token scores and certificate in the workspace
        ca.certified_attention_layer(cc, q, 4, None, False, **knobs)
        torch.cuda.synchronize()
        ws = cc._certified_workspace["cqa_ws"]
        nq, nact = cc.num_quantized_blocks, cc.active_blocks
        last_valid = 16 if nact == nq else cc.num_tokens - nq * 16
        wstruct = ws.fill_struct(nact)
        ref = _attend(L.cqa_attend, cc, ws, wstruct, q, nq, nact, last_valid)
        # the static variant must not need the caller's partial buffers at all
        no_scratch = _lib.CqaWorkspace.from_buffer_copy(bytes(wstruct))
        for f in ("part_m", "part_l", "part_acc", "dense_m", "dense_l", "dense_acc", "tickets"):
            setattr(no_scratch, f, None)
        ws.out.zero_()
        got = _attend(L.cqa_attend_static, cc, ws, no_scratch, q, nq, nact, last_valid)
        # same kernel, same split plan, partials merged in split order whatever the scratch: bit for bit
        assert torch.isfinite(got).all()
        assert torch.equal(got, ref), f"call {call}: outputs differ (max {float((got - ref).abs().max()):.3e})"


def test_static_scratch_attend_rejects_oversize():
    import cuda_harness as hz

    L = _lib.lib()
    dtype = "bfloat16"
    base = synth.make_layer_inputs(32, 256, kv_heads=2, dtype=dtype)
    cc = hz.make_cuda_cache(base.k, base.v, dtype, 16)
    w = _lib.CqaWorkspace()
    w.ld = 16
    w.num_splits = 129          # one more than CQA_STATIC_MAX_SPLITS
    q = hz.to_dev(base.q, dtype)
    desc = cc._desc(4)
    rc = L.cqa_attend_static(C.byref(desc), C.byref(w), q.data_ptr(), _lib.CQA_BF16, 16, 16, 256, 16, 0.088, None)
    assert rc == -4 and b"exceed the built-in scratch" in L.cqa_last_error()
