"""Sequence-sharded certified attention: one long context split by block range
over the ranks of a process group (one process per GPU).

The reference runs one cache per process (its distributed driver,
benchmarks/paper/run_distributed_quality_slice.py, only farms independent
slices out to workers); this module is the sharded form of
certified_attention_layer (kernels/certified_attention.py:1065-2790).

Every rank holds the INT8/INT4 tiers and the Tier-2 originals of a contiguous
range of 16-token blocks.  One layer step:

  1. Phase 1 on the local blocks (cqa_score_blocks).
  2. Exchange A (all-gather): the local m_b / S_b rows, the local eta_b rows and
     the local per-channel scale maxima.  Every rank now holds the global
     arrays and runs the *same* selector, value check and top-list search on
     them (cqa_select_certify_local), so K*, masks and flags are those of the
     unsharded run bit for bit, whatever the number of ranks.
  3. The ranks that own top-list blocks re-score them from their Tier-2 keys
     (cqa_rescore_owned); Exchange B (all-reduce sum, non-owners send zeros).
     Ranking, boundary and consistency flags follow (cqa_certify_given).
  4. Phase 2 over the local blocks with the global masks; the kernel leaves the
     un-normalised (max, sum, acc) of every head (cqa_attend, partial_out).
     Heads flagged for the dense recompute are covered the same way.
  5. Exchange C (all-gather) and the log-sum-exp merge (cqa_merge_partials).

New tokens go to the last rank (it owns the tail of the sequence).
Two transports carry the exchanges: torch.distributed collectives (NCCL on
GPUs; the default, `exchange="collective"`), or pushes into the other ranks'
buffers over NVLink with bounded waits on local flags, all inside one library
call per step (`exchange="peer"`, cqa_sharded_layer_step).  The plan and index
helpers below are device-agnostic so the host logic can be exercised with the
gloo backend on CPU tensors.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass
from typing import Any

import torch
import torch.distributed as dist

from cqa_b200 import _lib
from .certified_attention import _Workspace, _make_knobs, _selection_width
from .tiered_kv_cache import TieredKeyCacheLayer

BLOCK = 16


@dataclass
class ShardPlan:
    """Block ranges of the ranks.  Ranks 0..P-2 own `stride` blocks each, the
    last rank owns the rest of the prefill and everything appended later."""

    world: int
    rank: int
    prefill_tokens: int
    max_new_tokens: int
    stride: int = 0
    sigma_cols: int = 8 * 128     # kv_heads * head_dim: the scale maxima travel as one row of the exchange

    def __post_init__(self):
        nb = self.prefill_tokens // BLOCK
        if self.world < 1 or not (0 <= self.rank < self.world):
            raise ValueError("bad world / rank")
        if self.stride <= 0:
            self.stride = (nb // self.world // 8) * 8
        if self.world > 1 and (self.stride <= 0 or self.stride * (self.world - 1) >= nb):
            raise ValueError(f"{nb} prefill blocks are too few for {self.world} ranks")
        self.prefill_blocks = nb

    @property
    def last(self) -> int:
        return self.world - 1

    def first_block(self, rank: int | None = None) -> int:
        r = self.rank if rank is None else rank
        return r * self.stride if self.world > 1 else 0

    def prefill_token_range(self, rank: int | None = None) -> tuple[int, int]:
        """Tokens of the prefill held by `rank` (the last rank also takes the ragged tail)."""
        r = self.rank if rank is None else rank
        lo = self.first_block(r) * BLOCK
        hi = self.prefill_tokens if r == self.last else (self.first_block(r) + self.stride) * BLOCK
        return lo, hi

    def local_blocks(self, nq_global: int, rank: int | None = None) -> int:
        """Complete blocks held by `rank` when the sequence has nq_global complete blocks."""
        r = self.rank if rank is None else rank
        if r != self.last:
            return self.stride
        return nq_global - self.first_block(r)

    @property
    def last_capacity(self) -> int:
        lo, hi = self.prefill_token_range(self.last)
        return (hi - lo + self.max_new_tokens + BLOCK - 1) // BLOCK + 1

    @property
    def chunk(self) -> int:
        """Columns of one rank's slot in the exchange buffers (a multiple of four: rows stay 16-byte aligned)."""
        return (max(self.stride, self.last_capacity, self.sigma_cols) + 3) // 4 * 4

    @property
    def ld(self) -> int:
        """Leading dimension of the global per-block arrays."""
        return self.first_block(self.last) + self.last_capacity


def exchange_rows(n_heads: int, kv_heads: int) -> int:
    """Rows of the Exchange-A payload: m_b [H], S_b [H], eta [KV], one row of scale maxima."""
    return 2 * n_heads + kv_heads + 1


def global_column(plan: ShardPlan, rows: int, b: int) -> int:
    """Offset of global block `b` from the start of a row of rank 0 in the all-gather buffer
    [rank][row][chunk] (the selector kernel computes the same)."""
    r = min(b // plan.stride, plan.world - 1) if plan.world > 1 else 0
    return r * rows * plan.chunk + (b - r * plan.stride)


class DistComm:
    """The two collectives the sharded step needs, over a torch.distributed process group."""

    def __init__(self, group: dist.ProcessGroup | None = None):
        self.group = group

    def all_gather(self, out: torch.Tensor, inp: torch.Tensor) -> None:
        dist.all_gather_into_tensor(out.view(-1), inp.view(-1), group=self.group)

    def all_reduce_sum(self, t: torch.Tensor) -> None:
        dist.all_reduce(t, op=dist.ReduceOp.SUM, group=self.group)


class ShardedCertifiedLayer:
    """One layer of one sequence, sharded over the ranks of a process group.  `comm` is a DistComm (or
    anything with the same two methods)."""

    def __init__(self, plan: ShardPlan, local_cache: TieredKeyCacheLayer, gqa_group: int, comm=None,
                 exchange: str = "collective"):
        """`exchange`: "collective" = torch.distributed all-gather / all-reduce through `comm`; "peer" = every rank
        pushes its slices into the other ranks' buffers over NVLink and kernels wait on local flags
        (cqa_sharded_layer_step; one node, one process per GPU, at most 8 ranks; the default process group is used
        once, at construction, to exchange the memory handles)."""
        if exchange not in ("collective", "peer"):
            raise ValueError("exchange must be 'collective' or 'peer'")
        self.plan, self.cache, self.G = plan, local_cache, int(gqa_group)
        self.exchange = exchange
        self.comm = comm if comm is not None else DistComm()
        dev = local_cache.keys_int8.device
        self.device = dev
        KV = local_cache.kv_heads
        H = KV * self.G
        self.H, self.KV = H, KV
        if KV * 128 > plan.sigma_cols:
            raise ValueError(f"ShardPlan.sigma_cols={plan.sigma_cols} is too small for {KV} KV heads")
        self.num_tokens = plan.prefill_tokens
        f32 = dict(dtype=torch.float32, device=dev)
        rows = exchange_rows(H, KV)
        self.send = torch.zeros(rows, plan.chunk, **f32)
        self.recv = torch.zeros(plan.world, rows, plan.chunk, **f32)
        self.given = torch.zeros(H, _lib.MAX_RANKING_K, 2, **f32)
        self.partial = torch.zeros(H, _lib.PARTIAL_STRIDE, **f32)
        self.partials = torch.zeros(plan.world, H, _lib.PARTIAL_STRIDE, **f32)
        # masks, certificate and scratch: a workspace sized for the global block count; the selector reads
        # m_b / S_b / eta straight from the all-gather buffer, Phase 2 reads this rank's rows of the send buffer
        self.ws = _Workspace(local_cache, H, self.G, dev, ld=plan.ld)
        self._rows = rows
        esz = 4
        self._p_send = self.send.data_ptr()
        self._p_send_sb = self._p_send + H * plan.chunk * esz
        self._p_recv = self.recv.data_ptr()
        self._p_recv_sb = self._p_recv + H * plan.chunk * esz
        self._p_recv_eta = self._p_recv + 2 * H * plan.chunk * esz
        self._p_recv_sigma = self._p_recv + (2 * H + KV) * plan.chunk * esz
        self.rng_seed, self.rng_calls = 0, 0     # exploration draw: identical on every rank
        self._meta_nq = -1
        self._wg, self._wl = _lib.CqaWorkspace(), _lib.CqaWorkspace()   # private copies: fields are overridden
        self._peers = None
        self._step = 0
        if exchange == "peer":
            self._open_peers()

    # -------------------------------------------------------------- peer buffers
    def _open_peers(self) -> None:
        plan, L = self.plan, _lib.lib()
        if plan.world < 2 or plan.world > _lib.MAX_PEERS:
            raise ValueError(f"peer exchange needs 2..{_lib.MAX_PEERS} ranks")
        with _lib.on_device(self.device):
            nbytes = L.cqa_peer_buffer_bytes(plan.world, self.H, self.KV, plan.chunk)
            own = C.c_void_p()
            _lib.check(L.cqa_peer_alloc(nbytes, C.byref(own)), "cqa_peer_alloc")
            handle = C.create_string_buffer(64)
            _lib.check(L.cqa_peer_export(own, handle), "cqa_peer_export")
            handles = [None] * plan.world
            dist.all_gather_object(handles, bytes(handle.raw))
            st = _lib.CqaPeers()
            st.world, st.rank, st.rows, st.n_heads, st.chunk = plan.world, plan.rank, self._rows, self.H, plan.chunk
            self._imported = []
            for r in range(plan.world):
                if r == plan.rank:
                    st.base[r] = own.value
                else:
                    p = C.c_void_p()
                    _lib.check(L.cqa_peer_import(handles[r], C.byref(p)), "cqa_peer_import")
                    st.base[r] = p.value
                    self._imported.append(p)
            self._peers, self._own_buffer, self._peer_bytes = st, own, nbytes
            dist.barrier()

    def close(self) -> None:
        """Unmap the peers' buffers and free this rank's (call on every rank, after the last step)."""
        if self._peers is None:
            return
        L = _lib.lib()
        torch.cuda.synchronize(self.device)
        dist.barrier()
        with _lib.on_device(self.device):
            for p in self._imported:
                L.cqa_peer_close(p)
            dist.barrier()
            L.cqa_peer_free(self._own_buffer)
        self._peers = None

    def peer_status(self, reset: bool = False) -> int:
        """0 unless a bounded wait of the steps so far timed out (synchronises with the device)."""
        if self._peers is None:
            return 0
        out = C.c_int32(0)
        with _lib.on_device(self.device):
            _lib.check(_lib.lib().cqa_peer_status(C.byref(self._peers), C.byref(out), 1 if reset else 0),
                       "cqa_peer_status")
        return int(out.value)

    # -------------------------------------------------------------- bookkeeping
    @property
    def nq(self) -> int:
        return self.num_tokens // BLOCK

    @property
    def nact(self) -> int:
        return (self.num_tokens + BLOCK - 1) // BLOCK

    def append_token(self, key: torch.Tensor, value: torch.Tensor) -> None:
        """Every rank calls this; only the last rank stores the token."""
        if self.plan.rank == self.plan.last:
            self.cache.append_token(key, value)
        self.num_tokens += 1

    # -------------------------------------------------------------------- step
    def _step_peer(self, q, qd, q_scale, nq_g, nact_g, n_loc, first, is_last, collect_stats, exploration_uniforms,
                   knob_args):
        """The whole step as one library call (cqa_sharded_layer_step): eight launches, no collective library."""
        if exploration_uniforms is not None:
            raise NotImplementedError("the peer exchange draws exploration in-kernel; explicit uniforms are only "
                                      "supported with exchange='collective'")
        plan, cache, ws, G = self.plan, self.cache, self.ws, self.G
        L = _lib.lib()
        knobs = _make_knobs(q_scale=q_scale, force_trailing_value_fp16=True, **knob_args)
        ws.ensure_sel_width(_selection_width(knob_args["k_max"], knob_args["rung1_threshold"],
                                             knob_args["rung1_multiplier"], nq_g), self.device)
        wg = self._wg
        C.memmove(C.byref(wg), C.byref(ws.fill_struct(nact_g)), C.sizeof(wg))
        wg.shard_stride = plan.stride
        wg.rng_seed, wg.rng_offset = self.rng_seed, self.rng_calls
        if knob_args["exploration_rate"] > 0.0:
            self.rng_calls += 1
        nact_l = n_loc + (1 if (is_last and nact_g > nq_g) else 0)
        wl = self._wl
        C.memmove(C.byref(wl), C.byref(ws.fill_struct(nact_l)), C.sizeof(wl))
        wl.topk_mask = ws.topk_mask.data_ptr() + first
        wl.value_mask = ws.value_mask.data_ptr() + first
        wl.explore_mask = ws.explore_mask.data_ptr() + first
        desc_g = cache._desc_copy(G)
        desc_g.max_blocks = plan.ld
        last_valid = BLOCK if nact_l == n_loc else cache.num_tokens - n_loc * BLOCK
        self._step += 1
        push_meta = 1 if self._meta_nq != nq_g else 0
        self._meta_nq = nq_g
        with _lib.on_device(self.device):
            _lib.check(L.cqa_sharded_layer_step(
                C.byref(cache._desc(G)), C.byref(desc_g), C.byref(knobs), C.byref(wg), C.byref(wl),
                C.byref(self._peers), q.data_ptr(), qd, nq_g, nact_g, n_loc, nact_l, first, cache.num_tokens,
                last_valid, self._step, push_meta, ws.out.data_ptr(), _lib.current_stream(self.device)),
                "cqa_sharded_layer_step")
        if not collect_stats:
            return ws.out, {}
        cert, flags = ws.read_cert()
        return ws.out, {"cert": cert, "flags": flags, "peer_status": self.peer_status()}

    def step(self, q_all: torch.Tensor, q_scale: float | None = None, *, v_tolerance: float,
             top_k_fp16_keys: int = 4, ranking_fallback: bool = True, ranking_r: int = 1,
             ranking_fallback_mode: str = "full", tau_cov: float = 0.995, k_min: int = 2, k_max: int | None = 128,
             rung1_threshold: float = 0.02, rung1_multiplier: float = 2.0, score_consistency_check: bool = False,
             eps_guard: float = 0.01, exploration_rate: float = 0.0, value_error_mode: str = "tight",
             exploration_uniforms: torch.Tensor | None = None, collect_stats: bool = False
             ) -> tuple[torch.Tensor, dict[str, Any]]:
        plan, cache, H, KV, G = self.plan, self.cache, self.H, self.KV, self.G
        if q_scale is None:
            q_scale = 1.0 / (cache.head_dim ** 0.5)
        q = q_all if q_all.is_contiguous() else q_all.contiguous()
        qd = _lib.dtype_code(q.dtype)
        L = _lib.lib()
        stream = _lib.current_stream(self.device)
        nq_g, nact_g = self.nq, self.nact
        n_loc = plan.local_blocks(nq_g)
        first = plan.first_block()
        is_last = plan.rank == plan.last
        if is_last and cache.num_quantized_blocks != n_loc:
            raise RuntimeError("local cache and global token count disagree")
        ws = self.ws
        desc_l = cache._desc(G)
        if self.exchange == "peer":
            return self._step_peer(q, qd, q_scale, nq_g, nact_g, n_loc, first, is_last, collect_stats,
                                   exploration_uniforms, dict(
                                       tau_cov=tau_cov, k_min=k_min, k_max=k_max, rung1_threshold=rung1_threshold,
                                       rung1_multiplier=rung1_multiplier, eps_guard=eps_guard,
                                       exploration_rate=exploration_rate, v_tolerance=v_tolerance, ranking_r=ranking_r,
                                       top_k_fp16_keys=top_k_fp16_keys, ranking_fallback=ranking_fallback,
                                       ranking_fallback_mode=ranking_fallback_mode,
                                       score_consistency_check=score_consistency_check,
                                       value_error_mode=value_error_mode))

        with _lib.on_device(self.device):
            # 1. Phase 1 straight into the send buffer (rows 0..H-1 m_b, H..2H-1 S_b)
            _lib.check(L.cqa_score_blocks(C.byref(desc_l), q.data_ptr(), qd, n_loc, float(q_scale),
                                          self._p_send, self._p_send_sb, plan.chunk,
                                          ws.token_scores.data_ptr(), stream), "cqa_score_blocks")
            # eta_b and the scale maxima only change when a block completes
            fresh_meta = self._meta_nq != nq_g
            if fresh_meta:
                self.send[2 * H: 2 * H + KV, :n_loc].copy_(cache.values_int4_errors[:, :n_loc])
                self.send[2 * H + KV, : KV * 128].copy_(cache.keys_scale_max.reshape(-1))
            # 2. Exchange A and the global selector
            self.comm.all_gather(self.recv, self.send)
            self._meta_nq = nq_g
            knobs = _make_knobs(
                q_scale=q_scale, tau_cov=tau_cov, k_min=k_min, k_max=k_max, rung1_threshold=rung1_threshold,
                rung1_multiplier=rung1_multiplier, eps_guard=eps_guard, exploration_rate=exploration_rate,
                v_tolerance=v_tolerance, ranking_r=ranking_r, top_k_fp16_keys=top_k_fp16_keys,
                ranking_fallback=ranking_fallback, ranking_fallback_mode=ranking_fallback_mode,
                score_consistency_check=score_consistency_check, value_error_mode=value_error_mode,
                force_trailing_value_fp16=True,
            )
            ws.ensure_sel_width(_selection_width(k_max, rung1_threshold, rung1_multiplier, nq_g), self.device)
            wg = self._wg
            C.memmove(C.byref(wg), C.byref(ws.fill_struct(nact_g)), C.sizeof(wg))
            wg.given_fp16 = self.given.data_ptr()
            wg.partial_out = None
            wg.m_b, wg.s_b = self._p_recv, self._p_recv_sb
            wg.shard_stride, wg.shard_chunk = plan.stride, plan.chunk
            wg.shard_rank_stride, wg.shard_ranks = self._rows * plan.chunk, plan.world
            desc_g = cache._desc_copy(G)
            desc_g.max_blocks = plan.ld
            desc_g.values_int4_errors = self._p_recv_eta
            desc_g.sigma_max = self._p_recv_sigma      # one row per rank: the kernel takes the maximum
            u_ptr, u_ld, u_keep = None, 0, None
            if exploration_rate > 0.0:
                if exploration_uniforms is not None:
                    u_keep = exploration_uniforms.to(device=self.device, dtype=torch.float32).contiguous()
                    u_ptr, u_ld = u_keep.data_ptr(), nq_g
                else:
                    # in-kernel draw: same seed and call counter on every rank, hence the same exploration set
                    wg.rng_seed = self.rng_seed
                    wg.rng_offset = self.rng_calls
                    self.rng_calls += 1
            _lib.check(L.cqa_select_certify_local(C.byref(desc_g), C.byref(knobs), C.byref(wg), nq_g, nact_g,
                                                  u_ptr, u_ld, stream), "cqa_select_certify_local")
            # 3. owners re-score the top list; Exchange B; flags
            need_fp16 = ranking_fallback or score_consistency_check
            if need_fp16:
                _lib.check(L.cqa_rescore_owned(C.byref(desc_l), ws.cert_buf.data_ptr(), q.data_ptr(), qd, first,
                                               n_loc, float(q_scale), self.given.data_ptr(), stream),
                           "cqa_rescore_owned")
                self.comm.all_reduce_sum(self.given)
            _lib.check(L.cqa_certify_given(C.byref(desc_g), C.byref(knobs), C.byref(wg), q.data_ptr(), qd, nq_g,
                                           nact_g, stream), "cqa_certify_given")
            # 4. Phase 2 over the local blocks, global masks viewed from this rank's first block
            nact_l = n_loc + (1 if (is_last and nact_g > nq_g) else 0)
            wl = self._wl
            C.memmove(C.byref(wl), C.byref(ws.fill_struct(nact_l)), C.sizeof(wl))
            wl.m_b, wl.s_b = self._p_send, self._p_send_sb
            wl.shard_stride, wl.shard_chunk, wl.shard_rank_stride, wl.shard_ranks = 0, plan.chunk, 0, 0
            wl.topk_mask = ws.topk_mask.data_ptr() + first
            wl.value_mask = ws.value_mask.data_ptr() + first
            wl.explore_mask = ws.explore_mask.data_ptr() + first
            wl.partial_out = self.partial.data_ptr()
            wl.given_fp16 = None
            last_valid = BLOCK if nact_l == n_loc else cache.num_tokens - n_loc * BLOCK
            _lib.check(L.cqa_attend(C.byref(desc_l), C.byref(wl), q.data_ptr(), qd, n_loc, nact_l,
                                    cache.num_tokens, last_valid, float(q_scale), stream), "cqa_attend")
            # 5. Exchange C and the merge
            self.comm.all_gather(self.partials, self.partial)
            _lib.check(L.cqa_merge_partials(self.partials.data_ptr(), plan.world, H, ws.out.data_ptr(), stream),
                       "cqa_merge_partials")
        if not collect_stats:
            return ws.out, {}
        cert, flags = ws.read_cert()
        return ws.out, {"cert": cert, "flags": flags}
