"""Benchmark: certified quantised decode attention, µs per layer per decode step.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
                    [--context 131072] [--layers 8] [--planted 64]

Workload (N=1): the configuration the headline target is stated on - Llama-3.1-8B
attention geometry (32 query heads, 8 KV heads, head_dim 128), batch 1,
context 131072, bf16 Q/K/V ~ N(0,1) with 4 outlier key channels per head (x8)
and 64 planted key blocks (cosine 0.9 to the query), INT8 keys / INT4 g16
values, paper certification knobs; every decode step appends one seeded token
and runs the certified attention chain.  A "step" is one token through
`--layers` independent layer caches (distinct caches, so the working set
between two visits of the same cache is far larger than L2, as in a real
32-layer decode); the metric is step time / layers.  The 32K configuration is
measured in the same run and reported under "ctx32k".

The default run prints ONE JSON line on rank 0.  `value` is the device-timed
number with inputs resident in HBM; `e2e` is the same metric through the public
Python API with host buffers (pinned q/k/v copied in, output copied out every
layer-step).  `roofline` is for the dominant kernel, `cpu_baseline` times the CPU
oracle (a port of the reference's algorithm) on this host.

--impl reference times the reference's own algorithm on the host cores.  The
reference is Python + Triton with no CPU implementation that can travel to this
box, so that arm runs the CPU oracle port (oracle/cqa_oracle.*) with all host
threads on the same workload, with the same --steps / --warmup / --layers.
"""
from __future__ import annotations

import argparse
import json
import math
import os
import subprocess
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
for p in (str(ROOT), str(ROOT / "certified-quantised-attention_b200")):
    if p not in sys.path:
        sys.path.insert(0, p)

import numpy as np

PAPER_KNOBS = dict(
    v_tolerance=0.05, top_k_fp16_keys=4, ranking_fallback=True, ranking_r=1,
    ranking_fallback_mode="full", tau_cov=0.995, k_min=2, k_max=128,
    rung1_threshold=0.02, rung1_multiplier=2.0, score_consistency_check=False,
    eps_guard=0.01, exploration_rate=0.02, value_error_mode="tight",
)
METRIC = "certified_decode_attention_us_per_layer_step"


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=256)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--context", type=int, default=131072)
    ap.add_argument("--second-context", type=int, default=32768,
                    help="a second single-GPU configuration measured in the same run (0 = skip)")
    ap.add_argument("--layers", type=int, default=8)
    ap.add_argument("--planted", type=int, default=64)
    ap.add_argument("--seed", type=int, default=2)
    ap.add_argument("--e2e-steps", type=int, default=64)
    ap.add_argument("--kernel-steps", type=int, default=32)
    ap.add_argument("--cpu-steps", type=int, default=96,
                    help="decode steps of the bounded CPU sample (about 10 s of host work at 128K on 16 threads)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--sharded-context", type=int, default=131072,
                    help="context of the sequence-sharded measurement taken when --gpus > 1 (0 = skip)")
    ap.add_argument("--sharded-steps", type=int, default=64)
    ap.add_argument("--batched-sweep", action="store_true",
                    help="instead of the headline run: batch x context sweep of one layer (batched launch against a loop "
                         "of one-sequence calls, full Tier-2 mirror and a hot tier capped at 2048 tokens)")
    ap.add_argument("--decoder", action="store_true",
                    help="instead of the headline run: a whole random-init Llama-3.1-8B-shaped decoder (32 layers, "
                         "hidden 4096, 32/8 heads, FFN 14336, vocab 128256), a batch of prompts prefilled by the "
                         "model itself, then greedy decoding through the certified path")
    ap.add_argument("--decoder-layers", type=int, default=32)
    ap.add_argument("--decoder-batch", type=int, default=4)
    ap.add_argument("--decoder-prompt", type=int, default=65536)
    ap.add_argument("--decoder-steps", type=int, default=256)
    ap.add_argument("--decoder-dense-steps", type=int, default=8,
                    help="steps of the model's own dense decode (HF cache, torch SDPA) timed for comparison (0 = skip)")
    ap.add_argument("--sharded-peer", type=int, default=1,
                    help="also time the sharded step with peer-memory exchanges (0 = collectives only)")
    return ap.parse_args()


# ----------------------------------------------------------------------------- clocks

class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu, self.proc, self.lines, self.first = gpu_index, None, [], 0

    def mark(self):
        """Samples read so far are dropped from the summary (they precede the timed region)."""
        self.first = len(self.lines)

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "20",
                 "-i", str(self.gpu)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=2)
        except Exception:
            self.proc.kill()
        sm, smax, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        kept = self.lines[self.first:] or self.lines[-1:]
        for ln in kept:
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                smax.append(float(f[2]))
            except ValueError:
                continue
            for name, val in zip(names, f[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": max(smax) if smax else None,
                "samples": len(sm), "reasons": sorted(reasons)}


# ----------------------------------------------------------------------------- workload

def build_inputs(args, n_layers, rank=0, context=None):
    from cqa_b200 import synth

    bases = []
    for l in range(n_layers):
        bases.append(synth.make_layer_inputs(args.seed + 1000 * rank + l, args.context if context is None else context,
                                             dtype="bfloat16", n_planted_blocks=args.planted))
    return bases


def step_tensors(bases, n_steps):
    """[steps][layers] numpy arrays of (q, k_new, v_new)."""
    from cqa_b200 import synth

    out = []
    for s in range(n_steps):
        out.append([synth.decode_step_inputs(b, s, dtype="bfloat16") for b in bases])
    return out


# ----------------------------------------------------------------------------- CPU arm

def cpu_threads() -> int:
    """All host threads, set explicitly: a launcher (torchrun) exports OMP_NUM_THREADS=1."""
    from oracle import cqa_oracle as orc

    return orc.set_threads(os.cpu_count() or 1)


def cpu_baseline(args, base, n_steps, max_new, context=None, layers=1, warmup=1):
    """The CPU oracle port of the reference's algorithm on the host cores: append + Phase 1 + selector +
    certificate + Phase 2 (float32) per layer-step.  A step is `layers` layer-steps (all on ONE layer cache: a
    bounded sample, the host's caches are far smaller than a layer's Tier 1 either way).  Returns the median µs per
    layer-step over `n_steps` steps after `warmup` untimed ones."""
    from cqa_b200 import synth
    from oracle import cqa_oracle as orc

    n = args.context if context is None else context
    aligned = (n // 16) * 16
    oc = orc.OracleCache.from_fp16_cache_int4v(base.k[:, :aligned], base.v[:, :aligned], "bfloat16",
                                               max_new_tokens=max_new)
    for t in range(aligned, n):
        oc.append_token(base.k[:, t:t + 1], base.v[:, t:t + 1])
    vs = oc.values_int4_scales.astype(np.float32)
    vz = oc.values_int4_zeros.astype(np.float32)
    knobs = dict(PAPER_KNOBS)
    times = []
    rng = np.random.default_rng(0)
    s = 0
    for step in range(warmup + n_steps):
        t_step = 0.0
        for _ in range(layers):
            q, kn, vn = synth.decode_step_inputs(base, s, dtype="bfloat16")
            s += 1
            t0 = time.perf_counter()
            oc.append_token(kn, vn)
            if (oc.num_tokens - 1) % 16 == 15:
                vs = oc.values_int4_scales.astype(np.float32)
                vz = oc.values_int4_zeros.astype(np.float32)
            nq = oc.num_quantized_blocks
            nact = oc.active_blocks
            m_b, S_b, tok = orc.score_blocks(oc, q, 4, 1.0 / math.sqrt(128.0))
            sel = orc.adaptive_select(m_b, S_b, knobs["tau_cov"], knobs["k_min"], knobs["k_max"],
                                      knobs["rung1_threshold"], knobs["rung1_multiplier"])
            mask = sel["topk_mask"]
            u = rng.random(mask.shape, dtype=np.float32)
            mask = mask | ((~mask) & (u < np.float32(knobs["exploration_rate"])))
            H = mask.shape[0]
            top_idx = np.stack([np.argsort(-m_b[h], kind="stable")[:4] for h in range(H)]).astype(np.int32)
            orc.fp16_block_scores(oc, q, top_idx, 4, 1.0 / math.sqrt(128.0), nq)
            orc.delta_bound(q, oc.sigma_max, 4)
            vc = orc.value_check(sel["mass_frac"], oc.values_int4_errors[:, :nq], 4, knobs["v_tolerance"])
            tk = np.zeros((H, nact), dtype=np.int32)
            tk[:, :nq] = mask
            vm = np.zeros((H, nact), dtype=np.int32)
            vm[:, :nq] = vc["unsafe"]
            trailing = oc.has_trailing_partial_block
            if trailing:
                tk[:, nq:] = 1
                vm[:, nq:] = 1
            lv = 16 if not trailing else oc.num_tokens - nq * 16
            orc.attend_mixed_f32(oc, q, 4, 1.0 / math.sqrt(128.0), tok, tk, vm, nact, lv, vs, vz)
            t_step += time.perf_counter() - t0
        if step >= warmup:
            times.append(t_step / layers)
    return float(np.median(times)) * 1e6


def workload_text(context, planted):
    return (f"llama3.1-8b attention geometry, batch 1, context {context}, bf16 KV, INT8K/INT4V g16, "
            f"{planted} planted blocks, one appended token per step")


def config_dict(context, planted, layers, world):
    return {"workload": workload_text(context, planted), "context": context, "layers_per_step": layers,
            "kv_heads": 8, "q_heads": 32, "head_dim": 128,
            "knobs": "tau_cov 0.995, k 2..128, r 1, eps_guard 0.01, exploration 0.02, rung1 0.02 x2.0, v_tol 0.05",
            "l2": "working set per step (layers x Tier-1) larger than L2",
            "parallelism": "independent sequences per GPU" if world > 1 else "single GPU"}


# ----------------------------------------------------------------------------- GPU arm

def run_ours(args, rank, world, device_index, context=None, light=False):
    """One single-GPU measurement at `context` (default: --context).  `light`: fewer staged kernel steps and
    end-to-end steps (the second configuration of a run)."""
    import torch
    import torch.distributed as dist

    from cqa_b200 import roofline
    from dotcache.kernels import certified_attention as ca
    from dotcache.kernels.tiered_kv_cache import TieredKeyCacheLayer

    torch.cuda.set_device(device_index)
    dev = torch.device("cuda", device_index)
    from cqa_b200 import _lib as cl

    K, W, NL = args.steps, args.warmup, args.layers
    context = args.context if context is None else context
    e2e_steps = max(2, args.e2e_steps // 4) if light else args.e2e_steps
    kernel_steps = max(1, args.kernel_steps // 8) if light else args.kernel_steps
    total_steps = W + K + e2e_steps + kernel_steps + 4
    bases = build_inputs(args, NL, rank, context)
    n = context
    aligned = (n // 16) * 16
    caches = []
    for b in bases:
        kd = torch.from_numpy(b.k[:, :aligned]).to(torch.bfloat16).to(dev)
        vd = torch.from_numpy(b.v[:, :aligned]).to(torch.bfloat16).to(dev)
        c = TieredKeyCacheLayer.from_fp16_cache_int4v(kd, vd, max_new_tokens=total_steps + (n - aligned) + 16,
                                                      defer_int4_append_quantization=True)
        for t in range(aligned, n):
            c.append_token(torch.from_numpy(b.k[:, t:t + 1]).to(torch.bfloat16).to(dev),
                           torch.from_numpy(b.v[:, t:t + 1]).to(torch.bfloat16).to(dev))
        caches.append(c)
        del kd, vd
    steps = step_tensors(bases, total_steps)
    H = 32
    q_host = torch.empty(total_steps, NL, H, 128, dtype=torch.bfloat16).pin_memory()
    k_host = torch.empty(total_steps, NL, 8, 128, dtype=torch.bfloat16).pin_memory()
    v_host = torch.empty(total_steps, NL, 8, 128, dtype=torch.bfloat16).pin_memory()
    for s in range(total_steps):
        for l in range(NL):
            q, kn, vn = steps[s][l]
            q_host[s, l] = torch.from_numpy(q).to(torch.bfloat16)
            k_host[s, l] = torch.from_numpy(kn.reshape(8, 128)).to(torch.bfloat16)
            v_host[s, l] = torch.from_numpy(vn.reshape(8, 128)).to(torch.bfloat16)
    q_dev, k_dev, v_dev = q_host.to(dev), k_host.to(dev), v_host.to(dev)
    knobs = dict(PAPER_KNOBS)
    q_scale = 1.0 / math.sqrt(128.0)

    def layer_step(s, l, collect=False, timings=None):
        c = caches[l]
        c.append_token(k_dev[s, l], v_dev[s, l])
        return ca.certified_attention_layer(c, q_dev[s, l], 4, q_scale, collect, phase_timings=timings, **knobs)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # the clock sampler starts before the warm-up so that nvidia-smi is already reporting when the timed
    # region begins; samples taken before the region starts are dropped
    sampler = ClockSampler(device_index)
    sampler.start()
    s_idx = 0
    for _ in range(W):
        for l in range(NL):
            layer_step(s_idx, l)
        s_idx += 1
    # ---- timed region: inputs resident in HBM
    barrier()
    sampler.mark()
    launches0 = int(cl.lib().cqa_launch_count(0))
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    t_host = time.perf_counter()
    for _ in range(K):
        for l in range(NL):
            layer_step(s_idx, l)
        s_idx += 1
    host_us = (time.perf_counter() - t_host) * 1e6 / (K * NL)   # CPU time to queue one layer-step
    e1.record()
    barrier()
    gpu_launches = int(cl.lib().cqa_launch_count(0)) - launches0     # kernels the library launched in the timed region
    ms_total = e0.elapsed_time(e1)
    if world > 1:
        t = torch.tensor([ms_total], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms_total = float(t.item())
    ms_per_step = ms_total / K
    # whole-job aggregate: layer-steps of all ranks per unit time (ranks run independent sequences)
    us_per_layer = ms_per_step * 1e3 / (NL * world)

    # ---- end to end: host buffers in, output out, through the host-buffer entry points.  One library call per
    # decode step (cqa_decode_token_host) queues, for each of the NL layers, the H2D copy of the packed q/k/v, the
    # append, the layer step and the D2H copy of the output rows, and waits on the stream once; the host then
    # holds every layer's output.  The per-layer entry point with a stream wait after every layer-step is
    # reported beside it.
    n_in = (H + 16) * 128
    qkv_host = torch.empty(e2e_steps, NL, n_in, dtype=torch.bfloat16).pin_memory()
    for i in range(e2e_steps):
        for l in range(NL):
            qkv_host[i, l, : H * 128] = q_host[s_idx + i, l].reshape(-1)
            qkv_host[i, l, H * 128: (H + 8) * 128] = k_host[s_idx + i, l].reshape(-1)
            qkv_host[i, l, (H + 8) * 128:] = v_host[s_idx + i, l].reshape(-1)
    out_host = torch.empty(NL, H, 128, dtype=torch.float32).pin_memory()
    e2e_rows = [[qkv_host[i, l] for l in range(NL)] for i in range(e2e_steps)]
    out_rows = [out_host[l] for l in range(NL)]
    n_waited = e2e_steps // 2          # first half: one wait per layer-step; second half: one per decode step

    def e2e_loop(first, last, wait_each):
        nonlocal s_idx
        barrier()
        t0 = time.perf_counter()
        for i in range(first, last):
            if wait_each:
                for l in range(NL):
                    ca.certified_decode_step_host(caches[l], e2e_rows[i][l], 4, out_rows[l], q_scale, **knobs)
            else:
                ca.certified_decode_token_host(caches, qkv_host[i], 4, out_host, q_scale, **knobs)
            s_idx += 1
        sec = time.perf_counter() - t0
        if world > 1:
            t = torch.tensor([sec], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            sec = float(t.item())
        return sec * 1e6 / (max(1, last - first) * NL)

    e2e_waited_us = e2e_loop(0, n_waited, True) if n_waited > 0 else None
    e2e_us = e2e_loop(n_waited, e2e_steps, False)
    # the clock record covers both timed regions (device-timed steps and the end-to-end loops)
    clocks = sampler.stop()
    if not bool(torch.isfinite(out_host).all()):
        raise RuntimeError("end-to-end loop returned non-finite attention rows")
    h2d = n_in * 2
    d2h = H * 128 * 4

    # ---- per-kernel timing (staged calls, CUDA events on the launching stream) and algorithmic bytes
    phase = {}
    bytes_acc = {"score": 0, "attend": 0, "dense": 0, "total": 0, "floor": 0}
    n_meas = 0
    sel_stats = {"k_star_mean": [], "value_fallback_blocks": [], "rung3": 0, "fp16_key_bytes": 0,
                 "fp16_value_bytes": 0}
    # A 512 MB fill runs ahead of every staged layer-step: it evicts L2 and keeps the GPU busy while the host
    # queues the four launches, so the events bracket kernel time and not launch latency.
    flush = torch.empty(128 * 1024 * 1024, dtype=torch.float32, device=dev)
    for _ in range(kernel_steps):
        for l in range(NL):
            flush.fill_(1.0)
            layer_step(s_idx, l, collect=False, timings=phase)
            c = caches[l]
            ws = c._certified_workspace["cqa_ws"]
            nq, nact = c.num_quantized_blocks, c.active_blocks
            cert, flags = ws.read_cert()
            lv = 16 if nact == nq else c.num_tokens - nq * 16
            b = roofline.step_bytes(ws.topk_mask[:, :nact].cpu().numpy(), ws.value_mask[:, :nact].cpu().numpy(),
                                    nq, nact, lv, 4, cert["dense"], 2, cert["top_blocks"][:, :4])
            for key in ("score", "attend", "dense", "total"):
                bytes_acc[key] += b[key]
            bytes_acc["floor"] += roofline.tier1_floor_bytes(c.num_tokens)
            sel_stats["k_star_mean"].append(float(cert["k_star"].mean()))
            sel_stats["value_fallback_blocks"].append(int((ws.value_mask[:, :nq].amax(dim=0) > 0).sum().item()))
            sel_stats["rung3"] += int(cert["dense"].sum())
            sel_stats["fp16_key_bytes"] += b["fp16_key_bytes"]
            sel_stats["fp16_value_bytes"] += b["fp16_value_bytes"]
            n_meas += 1
        s_idx += 1
    # ---- the two streaming kernels again, each launched back to back over the NL layer caches (NL x its bytes is
    # larger than L2 at the default sizes) between ONE pair of events: the average launch duration without the
    # event and ramp overhead that an isolated launch carries.  Every workspace still holds its last step's masks.
    import ctypes as C
    L = cl.lib()
    stream = cl.current_stream(dev)
    last_q = [q_dev[s_idx - 1, l] for l in range(NL)]
    rec = []
    for l in range(NL):
        c = caches[l]
        ws = c._certified_workspace["cqa_ws"]
        nq, nact = c.num_quantized_blocks, c.active_blocks
        lv = 16 if nact == nq else c.num_tokens - nq * 16
        rec.append((c._desc(4), ws, ws.fill_struct(nact), nq, nact, c.num_tokens, lv))

    def launch_score(l):
        d, ws, w, nq, nact, ntok, lv = rec[l]
        cl.check(L.cqa_score_blocks(C.byref(d), last_q[l].data_ptr(), cl.dtype_code(last_q[l].dtype), nq, float(q_scale),
                                    ws.m_b.data_ptr(), ws.s_b.data_ptr(), ws.ld, ws.token_scores.data_ptr(), stream),
                 "cqa_score_blocks")

    def launch_attend(l):
        d, ws, w, nq, nact, ntok, lv = rec[l]
        cl.check(L.cqa_attend(C.byref(d), C.byref(w), last_q[l].data_ptr(), cl.dtype_code(last_q[l].dtype), nq, nact,
                              ntok, lv, float(q_scale), stream), "cqa_attend")

    def back_to_back(fn, rounds):
        ea, eb = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        with cl.on_device(dev):
            for l in range(NL):
                fn(l)                       # warm-up of this entry point
            flush.fill_(1.0)                # evicts L2; the launches below are queued while it runs
            ea.record()
            for _ in range(rounds):
                for l in range(NL):
                    fn(l)
            eb.record()
        torch.cuda.synchronize()
        return ea.elapsed_time(eb) * 1e3 / (rounds * NL)

    b2b_rounds = max(1, min(8, kernel_steps * 2))
    b2b_us = {"phase1_int8_scoring": back_to_back(launch_score, b2b_rounds),
              "phase2_fused_attend": back_to_back(launch_attend, b2b_rounds)}
    peaks = {}
    try:
        peaks = json.loads((ROOT / "MEASURED_PEAKS.json").read_text())
    except Exception:
        pass
    peak_gbs = float(peaks.get("hbm_gbs", 6650.0))
    peak_src = "measured (MEASURED_PEAKS.json)" if "hbm_gbs" in peaks else "fallback 6650 GB/s"
    kern_us = {k[:-3]: v / n_meas for k, v in phase.items()}
    stage_of = {"phase1_int8_scoring": "score", "phase2_fused_attend": "attend"}
    dominant = max(stage_of, key=lambda k: b2b_us.get(k, 0.0))
    dom_bytes = bytes_acc[stage_of[dominant]] / n_meas
    if dominant == "phase2_fused_attend":
        dom_bytes += bytes_acc["dense"] / n_meas
    achieved = dom_bytes / (b2b_us[dominant] * 1e-6) / 1e9
    chain_bytes = bytes_acc["total"] / n_meas
    chain_gbs = chain_bytes / (us_per_layer * 1e-6) / 1e9
    roof = {
        "bound": "hbm", "kernel": {"phase1_int8_scoring": "score_blocks_kernel",
                                   "phase2_fused_attend": "attend_kernel"}[dominant],
        "achieved": round(achieved, 1), "peak": peak_gbs, "unit": "GB/s", "frac": round(achieved / peak_gbs, 4),
        "peak_source": peak_src,
        # dram__bytes_read.sum + dram__bytes_write.sum needs a profiler; a bench run does not measure it (the ncu
        # summaries under profiles/ do)
        "traffic": None,
        "algorithmic_bytes_per_launch": int(dom_bytes), "kernel_us": round(b2b_us[dominant], 2),
        "kernel_us_how": "average over %d back-to-back launches on %d layer caches, one event pair" % (b2b_rounds * NL, NL),
        "kernel_us_isolated": round(kern_us[dominant], 2),
        "back_to_back_us": {k: round(v, 2) for k, v in b2b_us.items()},
        "chain": {"algorithmic_bytes_per_layer_step": int(chain_bytes), "us_per_layer_step": round(us_per_layer, 2),
                  "achieved_gbs": round(chain_gbs, 1), "frac": round(chain_gbs / peak_gbs, 4),
                  "frac_of_nominal_8000": round(chain_gbs / 8000.0, 4),
                  "tier1_floor_bytes": int(bytes_acc["floor"] / n_meas)},
        "stage_us": {k: round(v, 2) for k, v in kern_us.items()},
    }
    result = {
        "metric": METRIC, "value": round(us_per_layer, 3), "unit": "us", "n_gpus": world, "steps": K, "warmup": W,
        "ms_per_step": round(ms_per_step, 5), "higher_is_better": False, "scaling": "weak", "vs_baseline": None,
        "dtype": "f32", "data": "synthetic",
        "config": config_dict(context, args.planted, NL, world),
        "tokens_per_s_32layer_equiv": round(1e6 / (32.0 * us_per_layer), 2),
        "e2e": {"value": round(e2e_us, 3), "unit": "us", "h2d_bytes_per_step": h2d * NL, "d2h_bytes_per_step": d2h * NL,
                "tokens_per_s_32layer_equiv": round(1e6 / (32.0 * e2e_us), 2),
                "waits": "one library call and one stream wait per decode step of %d layers" % NL,
                "with_a_wait_per_layer_step": None if e2e_waited_us is None else round(e2e_waited_us, 3)},
        "gpu_launches": gpu_launches,
        "gpu_launches_how": "the library's own launch counter (cqa_launch_count) read before and after the timed region",
        "host_us_per_layer_step": round(host_us, 2),
        "clocks": clocks,
        "roofline": roof,
        "selection": {"k_star_mean": round(float(np.mean(sel_stats["k_star_mean"])), 2),
                      "value_fallback_blocks_mean": round(float(np.mean(sel_stats["value_fallback_blocks"])), 2),
                      "rung3_heads_total": sel_stats["rung3"], "layer_steps_measured": n_meas},
    }
    return result, bases


def run_sharded(args, rank, world, device_index):
    """Config 4: one layer, 128K context with 10 needle blocks (cosine 0.95 at depths 0.0 .. 0.9), sharded by
    block range over the ranks.  Rank 0 also times the same sequence unsharded on its own GPU."""
    import torch
    import torch.distributed as dist

    from cqa_b200 import synth
    from dotcache.kernels import certified_attention as ca
    from dotcache.kernels.sharded_certified_attention import ShardedCertifiedLayer, ShardPlan
    from dotcache.kernels.tiered_kv_cache import TieredKeyCacheLayer

    dev = torch.device("cuda", device_index)
    n, K, W = args.sharded_context, args.sharded_steps, max(3, args.warmup)
    base = synth.make_layer_inputs(args.seed + 77, n, dtype="bfloat16", n_planted_blocks=10, planted_cos=0.95,
                                   planted_depths=[i / 10.0 for i in range(10)])
    steps = [synth.decode_step_inputs(base, s, dtype="bfloat16") for s in range(W + K + 1)]
    to = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(torch.bfloat16).to(dev)
    qs = [to(q) for q, _, _ in steps]
    ks = [to(k.reshape(8, 1, 128)) for _, k, _ in steps]
    vs = [to(v.reshape(8, 1, 128)) for _, _, v in steps]
    knobs = dict(PAPER_KNOBS)
    knobs["exploration_rate"] = 0.0   # the draw must be identical on every rank; off keeps the comparison simple
    plan = ShardPlan(world, rank, n, W + K + 16)
    lo, hi = plan.prefill_token_range()
    cache = TieredKeyCacheLayer.from_fp16_cache_int4v(to(base.k[:, lo:hi]), to(base.v[:, lo:hi]),
                                                      max_new_tokens=(W + K + 16) if rank == plan.last else 0,
                                                      defer_int4_append_quantization=True)
    layer = ShardedCertifiedLayer(plan, cache, 4)

    host_us = {}

    def timed(fn, tag):
        for s in range(W):
            fn(s)
        dist.barrier()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        t_host = time.perf_counter()
        for s in range(W, W + K):
            fn(s)
        host_us[tag] = (time.perf_counter() - t_host) * 1e6 / K    # host time to queue one sharded layer-step
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) * 1e3 / K

    def sharded_step(s):
        layer.append_token(ks[s], vs[s])
        layer.step(qs[s], None, **knobs)

    def parity_record():
        """One more step (index W + K) with the certificate read back: what rank 0 compares with the unsharded run."""
        s = W + K
        layer.append_token(ks[s], vs[s])
        out, st = layer.step(qs[s], None, collect_stats=True, **knobs)
        torch.cuda.synchronize()
        nact = layer.nact
        return {"out": out.float().cpu().numpy().copy(), "k_star": np.asarray(st["cert"]["k_star"]).copy(),
                "rung3": np.asarray(st["cert"]["rung3"]).copy(),
                "topk": layer.ws.topk_mask[:, :nact].cpu().numpy().copy(),
                "vmask": layer.ws.value_mask[:, :nact].cpu().numpy().copy()}

    us = timed(sharded_step, "collective")
    t = torch.tensor([us], device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    us = float(t.item())
    rec_coll = parity_record()
    # the same sequence again with peer-memory exchanges (pushes over NVLink, bounded waits on local flags)
    us_peer, peer_status, rec_peer = None, None, None
    if args.sharded_peer:
        del layer, cache
        torch.cuda.empty_cache()
        cache = TieredKeyCacheLayer.from_fp16_cache_int4v(to(base.k[:, lo:hi]), to(base.v[:, lo:hi]),
                                                          max_new_tokens=(W + K + 16) if rank == plan.last else 0,
                                                          defer_int4_append_quantization=True)
        layer = ShardedCertifiedLayer(plan, cache, 4, exchange="peer")
        us_peer = timed(sharded_step, "peer")
        rec_peer = parity_record()
        peer_status = layer.peer_status()
        t = torch.tensor([us_peer, float(peer_status)], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        us_peer, peer_status = float(t[0].item()), int(t[1].item())
        layer.close()
    single = None
    if rank == 0:
        full = TieredKeyCacheLayer.from_fp16_cache_int4v(to(base.k), to(base.v), max_new_tokens=W + K + 16,
                                                         defer_int4_append_quantization=True)
        q_scale = 1.0 / math.sqrt(128.0)
        for s in range(W):
            full.append_token(ks[s], vs[s])
            ca.certified_attention_layer(full, qs[s], 4, q_scale, False, **knobs)
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for s in range(W, W + K):
            full.append_token(ks[s], vs[s])
            ca.certified_attention_layer(full, qs[s], 4, q_scale, False, **knobs)
        e1.record()
        torch.cuda.synchronize()
        single = e0.elapsed_time(e1) * 1e3 / K
        # the same extra step on the unsharded cache, and the comparison: K*, Rung-3 flags and both masks exact,
        # output rows within 1e-5 of the row scale
        s_par = W + K
        full.append_token(ks[s_par], vs[s_par])
        ref_out, _ = ca.certified_attention_layer(full, qs[s_par], 4, q_scale, False, **knobs)
        torch.cuda.synchronize()
        fws = full._certified_workspace["cqa_ws"]
        fcert, _ = fws.read_cert()
        nact = full.active_blocks
        ref = {"out": ref_out.float().cpu().numpy().copy(), "k_star": np.asarray(fcert["k_star"]),
               "rung3": np.asarray(fcert["rung3"]), "topk": fws.topk_mask[:, :nact].cpu().numpy(),
               "vmask": fws.value_mask[:, :nact].cpu().numpy()}

        def same(rec):
            if rec is None:
                return None
            exact = all(np.array_equal(rec[k], ref[k]) for k in ("k_star", "rung3", "topk", "vmask"))
            scale = np.abs(ref["out"]).max(axis=1, keepdims=True)
            err = float((np.abs(rec["out"] - ref["out"]) / scale).max())
            return {"selections_exact": bool(exact), "output_max_rel_err": err, "ok": bool(exact and err <= 1e-5)}

        par_coll, par_peer = same(rec_coll), same(rec_peer)
    dist.barrier()
    if rank != 0:
        return None
    per_rank_bytes = 2304.0 * n / world
    parity = bool(par_coll["ok"] and (par_peer is None or par_peer["ok"]))
    return {"workload": f"one layer, context {n}, 10 needle blocks (cosine 0.95), block ranges over {world} ranks, "
                        "NCCL all-gather / all-reduce exchanges", "ranks": world, "steps": K,
            "us_per_layer_step": round(us, 2), "single_gpu_us_per_layer_step": round(single, 2),
            "speedup_vs_single_gpu": round(single / us, 3),
            "peer_exchange_us_per_layer_step": None if us_peer is None else round(us_peer, 2),
            "peer_exchange_speedup_vs_single_gpu": None if us_peer is None else round(single / us_peer, 3),
            "peer_exchange_wait_status": peer_status,
            "parity": parity,
            "parity_detail": {"what": "one extra step after the timed ones: K*, Rung-3 flags, FP16-key and FP16-value "
                                      "masks equal to the single-GPU run's, output rows within 1e-5 of the row scale",
                              "collective": par_coll, "peer": par_peer},
            "host_us_per_layer_step": {k: round(v, 2) for k, v in host_us.items()},
            "hbm_floor_us_per_rank": round(per_rank_bytes / 6540.2e3, 2)}


def run_decoder(args, device_index):
    """A whole decoder with random-init bf16 weights: prefill of a batch of uniform-random prompts by the model itself
    (chunked, its own SDPA attention), per-(layer, sequence) certified caches built from that prefill by one library
    call per sequence, then greedy decoding with every layer's attention going through the certified batched step.
    Reports end-to-end decode tokens/s (all sequences) and the model's own dense decode beside it."""
    import torch
    from transformers import DynamicCache, LlamaConfig, LlamaForCausalLM

    from cqa_b200 import _lib as cl
    from dotcache.integrations.llama import (build_certified_state_from_prefill, install_certified_attention,
                                             remove_certified_attention)

    torch.cuda.set_device(device_index)
    dev = torch.device("cuda", device_index)
    torch.manual_seed(args.seed)
    NL, B, P, S = args.decoder_layers, args.decoder_batch, args.decoder_prompt, args.decoder_steps
    cfg = LlamaConfig(vocab_size=128256, hidden_size=4096, intermediate_size=14336, num_hidden_layers=NL,
                      num_attention_heads=32, num_key_value_heads=8, head_dim=128,
                      max_position_embeddings=P + S + 64, rms_norm_eps=1e-5, rope_theta=500000.0,
                      tie_word_embeddings=False)
    with torch.device(dev):
        model = LlamaForCausalLM(cfg).to(torch.bfloat16).eval()
    ids = torch.randint(0, cfg.vocab_size, (B, P), device=dev)
    ev = lambda: torch.cuda.Event(enable_timing=True)
    with torch.no_grad():
        past = DynamicCache()
        t0 = time.perf_counter()
        chunk = 4096
        for c0 in range(0, P, chunk):
            out = model.model(input_ids=ids[:, c0:c0 + chunk], past_key_values=past, use_cache=True)
        tok = model.lm_head(out.last_hidden_state[:, -1:]).argmax(dim=-1)          # [B, 1]
        torch.cuda.synchronize()
        prefill_s = time.perf_counter() - t0
        first_tok = tok.clone()
        dense = None
        if args.decoder_dense_steps > 0:
            e0, e1 = ev(), ev()
            dtok = first_tok.clone()
            for s in range(args.decoder_dense_steps + 2):
                if s == 2:
                    e0.record()
                o = model(input_ids=dtok, past_key_values=past, use_cache=True)
                dtok = o.logits[:, -1:].argmax(dim=-1)
            e1.record()
            torch.cuda.synchronize()
            dense_ms = e0.elapsed_time(e1) / args.decoder_dense_steps
            dense = {"ms_per_step": round(dense_ms, 3), "tokens_per_s": round(B * 1e3 / dense_ms, 1),
                     "what": "the same model's dense decode: HF DynamicCache (grows by concatenation) + torch SDPA, "
                             f"{args.decoder_dense_steps} steps"}
            past.crop(P)
        t0 = time.perf_counter()
        state = build_certified_state_from_prefill(past, list(range(NL)), max_new_tokens=S + 32)
        torch.cuda.synchronize()
        encode_s = time.perf_counter() - t0
        del past, out
        torch.cuda.empty_cache()
        install_certified_attention(model, state)
        warm = 4
        e0, e1 = ev(), ev()
        tok = first_tok
        sampler = ClockSampler(device_index)
        launches0 = 0
        for s in range(warm + S):
            if s == warm:
                torch.cuda.synchronize()
                sampler.start()
                launches0 = cl.lib().cqa_launch_count(0)
                e0.record()
            state.begin_decode_step()
            pos = torch.full((B, 1), P + s, device=dev)
            o = model(input_ids=tok, position_ids=pos, use_cache=False)
            tok = o.logits[:, -1:].argmax(dim=-1)
        e1.record()
        torch.cuda.synchronize()
        clocks = sampler.stop()
        launches = cl.lib().cqa_launch_count(0) - launches0
        remove_certified_attention(model)
        caches = state.batch_caches if state.batch_caches else {l: [c] for l, c in state.tiered_caches.items()}
        # the attention part alone: the batched certified step of every layer in turn (no append), one event pair
        from dotcache.kernels import certified_attention as ca

        qb = torch.randn(B, 32, 128, device=dev).to(torch.bfloat16)
        kn = dict(v_tolerance=state.v_tolerance, top_k_fp16_keys=state.top_k_fp16_keys,
                  ranking_fallback=state.ranking_fallback, ranking_r=state.ranking_r, tau_cov=state.tau_cov,
                  k_min=state.k_min, k_max=state.k_max)
        a0, a1 = ev(), ev()
        for rep in range(3):
            if rep == 1:
                a0.record()
            for l in range(NL):
                if B > 1:
                    ca.certified_attention_batch(caches[l], qb, 4, None, **kn)
                else:
                    ca.certified_attention_layer(caches[l][0], qb[0], 4, None, False, **kn)
        a1.record()
        torch.cuda.synchronize()
        attn_ms = a0.elapsed_time(a1) / 2
    ms = e0.elapsed_time(e1) / S
    tier1 = sum(c.keys_int8.numel() + c.values_int4_packed.numel() for cs in caches.values() for c in cs)
    return {
        "metric": "certified_decode_tokens_per_s", "value": round(B * 1e3 / ms, 1), "unit": "tokens/s", "n_gpus": 1,
        "steps": S, "warmup": warm, "ms_per_step": round(ms, 3), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": f"Llama-3.1-8B-shaped decoder, random-init bf16 weights, {NL} layers, batch {B}, prompt "
                               f"{P} uniform token ids, {S} greedy steps, INT8K/INT4V g16 certified attention in every "
                               "layer (one batched launch chain per layer), projections / MLP / lm_head by torch",
                   "layers": NL, "batch": B, "prompt": P, "knobs": "tau_cov 0.995, k 2..128, r 1, v_tol 0.05"},
        "us_per_sequence_layer_step": round(ms * 1e3 / (NL * B), 2),
        "attention_only": {"ms_per_step": round(attn_ms, 3), "us_per_sequence_layer_step": round(attn_ms * 1e3 / (NL * B), 2),
                           "what": "the certified step of all layers back to back on the final caches, no model around it"},
        "gpu_launches": int(launches), "clocks": clocks,
        "prefill_s": round(prefill_s, 1), "cache_encode_s": round(encode_s, 2),
        "tier1_bytes_int8k_int4v": int(tier1), "dense_decode": dense,
        "hbm_gb_allocated": round(torch.cuda.max_memory_allocated(dev) / 2**30, 1),
    }


def run_batched_sweep(args, device_index):
    """Capped-hot-tier sweep shape (batch x context, one layer): µs per sequence-layer-step of the batched launch
    (cqa_layer_step_batched) against a loop of one-sequence calls on the same caches, with the full Tier-2 mirror
    and with the hot tier capped at 2048 tokens (128 blocks; Tier 2 in pinned host memory), where the residency
    counters give hit rate and page-in bytes per step."""
    import torch

    from cqa_b200 import synth
    from dotcache.kernels import certified_attention as ca
    from dotcache.kernels.tiered_kv_cache import TieredKeyCacheLayer

    torch.cuda.set_device(device_index)
    dev = torch.device("cuda", device_index)
    K, W = max(4, min(args.steps, 32)), max(3, min(args.warmup, 8))
    q_scale = 1.0 / math.sqrt(128.0)
    rows = []
    for context in (8192, 32768, 131072):
        base = synth.make_layer_inputs(args.seed, context, dtype="bfloat16", n_planted_blocks=args.planted)
        kd = torch.from_numpy(base.k).to(torch.bfloat16).to(dev)
        vd = torch.from_numpy(base.v).to(torch.bfloat16).to(dev)
        steps = [synth.decode_step_inputs(base, s, dtype="bfloat16") for s in range(2 * (W + K))]
        for v_tol in (0.05, 0.02):
            knobs = dict(PAPER_KNOBS, v_tolerance=v_tol)
            for capped in (0, 128, 2048):     # blocks of 16 tokens in each hot tier; 0 = full mirror in HBM
                for B in (1, 8, 32, 64):
                    if context == 131072 and B > 8:
                        continue
                    if capped and (B > 8 or v_tol != 0.05 or (capped == 2048 and (B > 1 or context == 8192))):
                        continue     # the pinned backing arrays of larger batches do not fit the time budget of a sweep
                    if not capped and v_tol != 0.05 and B not in (1, 32):
                        continue
                    kw = dict(max_new_tokens=2 * (W + K) + 16, defer_int4_append_quantization=not capped)
                    if capped:
                        kw.update(fp16_key_cache_capacity=capped, fp16_value_cache_capacity=capped, max_pagein_blocks=64)
                    caches = [TieredKeyCacheLayer.from_fp16_cache_int4v(kd, vd, **kw) for _ in range(B)]
                    qs = [torch.from_numpy(np.stack([steps[s][0]] * B)).to(torch.bfloat16).to(dev) for s in range(2 * (W + K))]
                    ks = [torch.from_numpy(np.stack([steps[s][1].reshape(8, 128)] * B)).to(torch.bfloat16).to(dev)
                          for s in range(2 * (W + K))]
                    vs = [torch.from_numpy(np.stack([steps[s][2].reshape(8, 128)] * B)).to(torch.bfloat16).to(dev)
                          for s in range(2 * (W + K))]

                    def batched(s):
                        ca.certified_attention_batch(caches, qs[s], 4, q_scale, new_keys=ks[s], new_values=vs[s], **knobs)

                    def looped(s):
                        for b in range(B):
                            caches[b].append_token(ks[s][b].reshape(8, 1, 128), vs[s][b].reshape(8, 1, 128))
                            ca.certified_attention_layer(caches[b], qs[s][b], 4, q_scale, False, **knobs)

                    def timed(fn, first):
                        for s in range(first, first + W):
                            fn(s)
                        torch.cuda.synchronize()
                        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                        e0.record()
                        for s in range(first + W, first + W + K):
                            fn(s)
                        e1.record()
                        torch.cuda.synchronize()
                        return e0.elapsed_time(e1) * 1e3 / (K * B)

                    us_loop = timed(looped, 0)
                    before = caches[0].hot_tier_counters() if capped else {}
                    us_batch = timed(batched, W + K)
                    row = {"context": context, "batch": B, "v_tolerance": v_tol, "hot_tier_tokens": capped * 16 if capped else None,
                           "us_per_sequence_layer_step_batched": round(us_batch, 2),
                           "us_per_sequence_layer_step_looped": round(us_loop, 2),
                           "speedup_of_batching": round(us_loop / us_batch, 2)}
                    if capped:
                        after = caches[0].hot_tier_counters()
                        d = {k: after[k] - before.get(k, 0) for k in after}
                        n_steps = max(1, d["steps"])
                        for tier in ("key", "value"):
                            tot = d[f"{tier}_hits"] + d[f"{tier}_misses"]
                            row[f"{tier}_hit_rate"] = round(d[f"{tier}_hits"] / tot, 4) if tot else None
                            row[f"{tier}_pagein_bytes_per_step"] = int(d[f"{tier}_pagein_bytes"] / n_steps)
                    rows.append(row)
                    print(json.dumps(row), file=sys.stderr, flush=True)
                    del caches, qs, ks, vs
                    torch.cuda.empty_cache()
        del kd, vd
    return {"metric": "certified_decode_attention_us_per_sequence_layer_step", "unit": "us", "n_gpus": 1,
            "steps": K, "warmup": W, "higher_is_better": False, "data": "synthetic", "dtype": "f32",
            "config": {"workload": "batch x context sweep, one layer, llama3.1-8b attention geometry, bf16 KV, "
                                   "INT8K/INT4V g16, one appended token per sequence and step"},
            "batched_sweep": rows}


def main():
    args = parse_args()
    # Libraries (NCCL prints its version on start-up) write to file descriptor 1; the one JSON line the caller
    # parses goes to the original stdout, everything else to stderr.
    out = os.fdopen(os.dup(1), "w")
    os.dup2(2, 1)
    try:
        return _main(args, out)
    finally:
        out.flush()


def _main(args, out):
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    max_new = args.warmup + args.steps + args.e2e_steps + args.kernel_steps + 64

    if args.impl == "reference":
        if rank != 0:
            return 0
        from cqa_b200 import synth

        cores = cpu_threads()
        base = synth.make_layer_inputs(args.seed, args.context, dtype="bfloat16", n_planted_blocks=args.planted)
        t0 = time.perf_counter()
        us = cpu_baseline(args, base, args.steps, (args.steps + args.warmup) * args.layers + 64, layers=args.layers,
                          warmup=args.warmup)
        sample = (f"{args.steps} decode steps of {args.layers} layer-steps each at context {args.context} (median per "
                  f"layer-step), all on one layer cache, OpenMP over {cores} host threads, after {args.warmup} warm-up steps")
        line = {
            "impl": "reference", "metric": METRIC, "value": round(us, 1), "unit": "us", "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(us * args.layers / 1e3, 3),
            "higher_is_better": False, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": config_dict(args.context, args.planted, args.layers, max(1, args.gpus)),
            "cpu_baseline": {"value": round(us, 1), "unit": "us", "cores": cores, "kind": "port", "sample": sample},
            "e2e": {"value": round(us, 1), "unit": "us", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "note": "the reference has no CPU implementation that runs outside its Python/Triton stack; this arm "
                    "times the CPU oracle port of its algorithm",
            "wall_s": round(time.perf_counter() - t0, 1),
        }
        print(json.dumps(line), file=out, flush=True)
        return 0

    import torch

    if not torch.cuda.is_available():
        print(json.dumps({"error": "no CUDA device: bench.py --impl ours needs a B200; there is no CPU fallback"}), file=out)
        return 1
    if args.decoder:
        if rank == 0:
            print(json.dumps(run_decoder(args, local)), file=out, flush=True)
        return 0
    if args.batched_sweep:
        if rank == 0:
            print(json.dumps(run_batched_sweep(args, local)), file=out, flush=True)
        return 0
    if world > 1:
        import torch.distributed as dist

        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    result, bases = run_ours(args, rank, world, local)
    if args.second_context > 0 and args.second_context != args.context:
        base0 = bases[0]
        del bases
        torch.cuda.empty_cache()
        second, _ = run_ours(args, rank, world, local, context=args.second_context, light=True)
        if rank == 0:
            result[f"ctx{args.second_context // 1024}k"] = {
                k: second[k] for k in ("value", "unit", "ms_per_step", "e2e", "roofline", "host_us_per_layer_step",
                                       "selection", "gpu_launches", "config")}
        bases = [base0]
    if world > 1 and args.sharded_context > 0:
        del bases
        torch.cuda.empty_cache()
        sharded = run_sharded(args, rank, world, local)
        if rank == 0:
            result["sharded"] = sharded
        bases = [None]
    if rank == 0:
        if world == 1 and not args.no_cpu_baseline:
            cores = cpu_threads()
            us = cpu_baseline(args, bases[0], args.cpu_steps, max(max_new, args.cpu_steps + 32))
            result["cpu_baseline"] = {
                "value": round(us, 1), "unit": "us", "cores": cores, "kind": "port",
                "sample": f"{args.cpu_steps} decode steps of one layer at context {args.context} (median), "
                          f"OpenMP over {cores} host threads, after 1 warm-up step"}
        print(json.dumps(result), file=out, flush=True)
    if world > 1:
        import torch.distributed as dist

        dist.barrier()
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
