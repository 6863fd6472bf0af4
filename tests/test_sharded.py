"""Sequence sharding: block-range plan, exchange packing (gloo, CPU), and the
sharded CUDA step against the unsharded one (ranks emulated as threads on one
GPU; real NCCL ranks when the box has two or more GPUs)."""
from __future__ import annotations

import os
import socket
import threading

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import golden_cases as gc
from cqa_b200 import synth
from dotcache.kernels.sharded_certified_attention import DistComm, ShardPlan, exchange_rows, global_column

H, KV, G = 32, 8, 4


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


# ----------------------------------------------------------------------------- plan (CPU)

def test_plan_ranges_cover_the_sequence():
    for world, n_tok, new in [(2, 8192, 64), (4, 32768 + 5, 512), (8, 131072, 512), (1, 4096, 16)]:
        plans = [ShardPlan(world, r, n_tok, new) for r in range(world)]
        edges = [p.prefill_token_range() for p in plans]
        assert edges[0][0] == 0 and edges[-1][1] == n_tok
        for a, b in zip(edges, edges[1:]):
            assert a[1] == b[0] and a[1] % 16 == 0
        p = plans[-1]
        nq = (n_tok + new) // 16
        assert sum(pl.local_blocks(nq) for pl in plans) == nq
        assert p.ld >= (n_tok + new + 15) // 16
        assert p.chunk >= max(pl.local_blocks(nq) for pl in plans)
    with pytest.raises(ValueError):
        ShardPlan(8, 0, 32 * 16, 16)


def _gloo_rank(rank, world, port, n_tok, new, ret):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        plan = ShardPlan(world, rank, n_tok, new)
        nq = (n_tok + 40) // 16          # 40 tokens appended so far
        rows = exchange_rows(H, KV)
        n_loc, first = plan.local_blocks(nq), plan.first_block()
        # "global truth": value of row r at global block b is r * 1e4 + b; scale maxima differ per rank
        send = torch.zeros(rows, plan.chunk)
        cols = torch.arange(first, first + n_loc, dtype=torch.float32)
        send[: rows - 1, :n_loc] = torch.arange(rows - 1, dtype=torch.float32)[:, None] * 1e4 + cols[None, :]
        send[rows - 1, : KV * 128] = torch.arange(KV * 128, dtype=torch.float32) * (1 + (rank == 1))
        recv = torch.zeros(world, rows, plan.chunk)
        DistComm().all_gather(recv, send)
        # every global block is found, in every row, at the offset the selector kernel uses
        flat = recv.view(-1)
        ok = True
        for row in (0, H, 2 * H + KV - 1):
            for b in (0, 1, plan.stride - 1, plan.stride, nq // 2, nq - 1):
                ok = ok and float(flat[row * plan.chunk + global_column(plan, rows, b)]) == row * 1e4 + b
        sigma = recv[:, rows - 1, : KV * 128].amax(dim=0)
        ok = ok and bool(torch.equal(sigma, torch.arange(KV * 128, dtype=torch.float32) * (2 if world > 1 else 1)))
        t = torch.tensor([1.0 if ok else 0.0])
        dist.all_reduce(t, op=dist.ReduceOp.MIN)
        if rank == 0:
            ret.put(float(t.item()))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 3])
def test_exchange_a_packing_over_gloo(world):
    """Every rank packs its block range, all-gathers over gloo and rebuilds the same global arrays."""
    ctx = mp.get_context("spawn")
    ret = ctx.SimpleQueue()
    port = _free_port()
    procs = [ctx.Process(target=_gloo_rank, args=(r, world, port, 4096 + 7, 64, ret)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    assert ret.get() == 1.0


# ----------------------------------------------------------------------------- CUDA (one GPU, ranks as threads)

class _ThreadComm:
    """all_gather / all_reduce between threads of one process (one GPU, one stream)."""

    def __init__(self, world):
        self.world, self.barrier, self.slots = world, threading.Barrier(world), [None] * world

    def view(self, rank):
        comm = self

        class V:
            def all_gather(self, out, inp):
                comm.slots[rank] = inp
                comm.barrier.wait()
                for p in range(comm.world):
                    out[p].copy_(comm.slots[p])
                comm.barrier.wait()

            def all_reduce_sum(self, t):
                comm.slots[rank] = t.clone()
                comm.barrier.wait()
                tot = torch.stack(comm.slots).sum(dim=0)
                comm.barrier.wait()
                t.copy_(tot)

        return V()


def _run_sharded_threads(world, k, v, n_prefill, steps, dtype, knobs, us, max_new=64):
    import cuda_harness as hz
    from dotcache.kernels.sharded_certified_attention import ShardedCertifiedLayer

    comm = _ThreadComm(world)
    results = [None] * world
    errors = []

    def rank_main(r):
        try:
            torch.cuda.set_device(0)
            plan = ShardPlan(world, r, n_prefill, max_new)
            lo, hi = plan.prefill_token_range()
            hi_al = lo + ((hi - lo) // 16) * 16
            cache = hz.make_cuda_cache(k[:, lo:hi_al], v[:, lo:hi_al], dtype, max_new if r == plan.last else 0)
            for t in range(hi_al, hi):
                cache.append_token(hz.to_dev(k[:, t:t + 1], dtype), hz.to_dev(v[:, t:t + 1], dtype))
            layer = ShardedCertifiedLayer(plan, cache, G, comm.view(r))
            outs = []
            for i, (q, kn, vn) in enumerate(steps):
                if kn is not None:
                    layer.append_token(hz.to_dev(kn, dtype), hz.to_dev(vn, dtype))
                out, st = layer.step(hz.to_dev(q, dtype), None, exploration_uniforms=torch.from_numpy(us[i]),
                                     collect_stats=True, **knobs)
                torch.cuda.synchronize()
                outs.append((out.cpu().numpy().copy(), st, layer.ws.topk_mask[:, :layer.nact].cpu().numpy().copy(),
                             layer.ws.value_mask[:, :layer.nact].cpu().numpy().copy(),
                             layer.ws.mass_frac[:, :layer.nq].cpu().numpy().copy()))
            results[r] = outs
        except Exception as e:  # pragma: no cover - surfaced below
            errors.append((r, repr(e)))
            comm.barrier.abort()

    threads = [threading.Thread(target=rank_main, args=(r,)) for r in range(world)]
    for t in threads:
        t.start()
    for t in threads:
        t.join(timeout=300)
    assert not errors, errors
    return results


def _knobs(**over):
    kn = dict(gc.PAPER_KNOBS)
    kn.update(over)
    return kn


@pytest.mark.gpu
@pytest.mark.parametrize("world,knobs", [(2, {}), (4, {}), (2, {"ranking_r": 4}), (3, {"score_consistency_check": True,
                                                                                      "eps_guard": -10.0})])
def test_sharded_step_matches_unsharded(world, knobs):
    """Certificates, masks and mass fractions are bit-identical to the one-rank run; outputs agree to 1e-5.
    Covers a ragged prefill, appends across a block completion, Rung 3 (ranking_r=4) and Rung 4 (every head
    recomputed densely)."""
    import cuda_harness as hz

    dtype = "bfloat16"
    n_prefill = 8192 + 5
    base = synth.make_layer_inputs(31, n_prefill, dtype=dtype, n_planted_blocks=16)
    kn = _knobs(**knobs)
    rng = np.random.default_rng(31)
    steps, us = [(base.q, None, None)], []
    for s in range(14):
        steps.append(synth.decode_step_inputs(base, s, dtype=dtype))
    n_tok = n_prefill
    for (q, knew, vnew) in steps:
        n_tok += 0 if knew is None else 1
        us.append(rng.random((H, n_tok // 16), dtype=np.float32))
    # unsharded run
    aligned = (n_prefill // 16) * 16
    cc = hz.make_cuda_cache(base.k[:, :aligned], base.v[:, :aligned], dtype, 64)
    for t in range(aligned, n_prefill):
        cc.append_token(hz.to_dev(base.k[:, t:t + 1], dtype), hz.to_dev(base.v[:, t:t + 1], dtype))
    ref = []
    for i, (q, knew, vnew) in enumerate(steps):
        if knew is not None:
            cc.append_token(hz.to_dev(knew, dtype), hz.to_dev(vnew, dtype))
        out, _ = hz.cuda_step(cc, q, dtype, G, kn, us[i])
        ws = cc._certified_workspace["cqa_ws"]
        cert, flags = ws.read_cert()
        ref.append((out, cert, flags, ws.topk_mask[:, :cc.active_blocks].cpu().numpy().copy(),
                    ws.value_mask[:, :cc.active_blocks].cpu().numpy().copy(),
                    ws.mass_frac[:, :cc.num_quantized_blocks].cpu().numpy().copy()))
    res = _run_sharded_threads(world, base.k, base.v, n_prefill, steps, dtype, kn, us)
    for r in range(world):
        for i, (out, st, tm, vm, mf) in enumerate(res[r]):
            r_out, r_cert, r_flags, r_tm, r_vm, r_mf = ref[i]
            what = f"world {world} rank {r} step {i}"
            assert np.array_equal(tm, r_tm), f"{what}: key mask"
            assert np.array_equal(vm, r_vm), f"{what}: value mask"
            assert np.array_equal(mf.view(np.uint32), r_mf.view(np.uint32)), f"{what}: mass fractions"
            assert st["flags"][:5] == r_flags[:5], f"{what}: flags {st['flags'][:5]} vs {r_flags[:5]}"
            for key, val in r_cert.items():
                got = st["cert"][key]
                if val.dtype.kind == "f":
                    assert np.array_equal(np.asarray(got, np.float32).view(np.uint32),
                                          np.asarray(val, np.float32).view(np.uint32)), f"{what}: cert {key}"
                else:
                    assert np.array_equal(got, val), f"{what}: cert {key}"
            err = np.abs(out - r_out).max() / max(np.abs(r_out).max(), 1e-6)
            assert err < 1e-5, f"{what}: output rel err {err}"


# ----------------------------------------------------------------------------- CUDA, real ranks over NCCL

NCCL_STEPS = 24     # crosses a block completion (step 16): the eta rows and scale maxima are exchanged again there


def _nccl_rank(rank, world, port, ret, exchange="collective"):
    import sys
    from pathlib import Path

    root = Path(__file__).resolve().parents[1]
    for p in (str(root), str(root / "tests"), str(root / "certified-quantised-attention_b200")):
        if p not in sys.path:
            sys.path.insert(0, p)
    import cuda_harness as hz
    from dotcache.kernels.sharded_certified_attention import ShardedCertifiedLayer

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        dtype = "bfloat16"
        n_prefill = 16384
        base = synth.make_layer_inputs(33, n_prefill, dtype=dtype, n_planted_blocks=16)
        kn = dict(gc.PAPER_KNOBS)
        plan = ShardPlan(world, rank, n_prefill, 64)
        lo, hi = plan.prefill_token_range()
        with torch.cuda.device(rank):
            cache = hz.make_cuda_cache(base.k[:, lo:hi], base.v[:, lo:hi], dtype, 64 if rank == plan.last else 0)
            layer = ShardedCertifiedLayer(plan, cache, G, exchange=exchange)
            rng = np.random.default_rng(33)
            outs, ks = [], []
            for s in range(NCCL_STEPS):
                q, knew, vnew = synth.decode_step_inputs(base, s, dtype=dtype)
                layer.append_token(hz.to_dev(knew, dtype).cuda(rank), hz.to_dev(vnew, dtype).cuda(rank))
                u = rng.random((H, layer.nq), dtype=np.float32)
                if exchange == "peer":
                    kn["exploration_rate"] = 0.0
                    out, st = layer.step(hz.to_dev(q, dtype).cuda(rank), None, collect_stats=True, **kn)
                    assert st["peer_status"] == 0, f"rank {rank}: a bounded wait timed out ({st['peer_status']})"
                else:
                    out, st = layer.step(hz.to_dev(q, dtype).cuda(rank), None,
                                         exploration_uniforms=torch.from_numpy(u), collect_stats=True, **kn)
                torch.cuda.synchronize()
                outs.append(out.cpu().numpy().copy())
                ks.append(st["cert"]["k_star"].copy())
            layer.close()
        if rank == 0:
            ret.put((outs, ks))
    finally:
        dist.destroy_process_group()


@pytest.mark.gpu
@pytest.mark.parametrize("exchange", ["collective", "peer"])
def test_sharded_step_over_nccl(exchange):
    """Two (or four) real ranks over NCCL against the one-GPU run.  Skipped on a one-GPU box."""
    import cuda_harness as hz

    n_gpus = torch.cuda.device_count()
    if n_gpus < 2:
        pytest.skip("needs two GPUs")
    world = 4 if n_gpus >= 4 else 2
    ctx = mp.get_context("spawn")
    ret = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_nccl_rank, args=(r, world, port, ret, exchange)) for r in range(world)]
    for p in procs:
        p.start()
    try:
        outs, ks = ret.get(timeout=600)      # a rank that died leaves the queue empty: fail, do not hang
    finally:
        for p in procs:
            p.join(timeout=300)
            if p.is_alive():
                p.kill()
    assert all(p.exitcode == 0 for p in procs), [p.exitcode for p in procs]
    dtype = "bfloat16"
    base = synth.make_layer_inputs(33, 16384, dtype=dtype, n_planted_blocks=16)
    cc = hz.make_cuda_cache(base.k, base.v, dtype, 64)
    rng = np.random.default_rng(33)
    for s in range(NCCL_STEPS):
        q, knew, vnew = synth.decode_step_inputs(base, s, dtype=dtype)
        cc.append_token(hz.to_dev(knew, dtype), hz.to_dev(vnew, dtype))
        u = rng.random((H, cc.num_quantized_blocks), dtype=np.float32)
        knobs = dict(gc.PAPER_KNOBS)
        if exchange == "peer":
            knobs["exploration_rate"] = 0.0
        out, stats = hz.cuda_step(cc, q, dtype, G, knobs, u)
        cert, _ = cc._certified_workspace["cqa_ws"].read_cert()
        assert np.array_equal(cert["k_star"], ks[s])
        err = np.abs(out - outs[s]).max() / max(np.abs(out).max(), 1e-6)
        assert err < 1e-5, f"step {s}: {err}"
