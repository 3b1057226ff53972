"""Expert parallelism over peer memory (NVLink loads / stores from inside the kernels, no all-to-all).

The all-to-all transport in :mod:`expert_parallel` packs the routed rows, sends them, re-gathers them into the
padded grouped layout, and does the same three passes on the way back.  Here every rank keeps its token rows,
router weights and a return buffer in memory that the other ranks of the node have mapped (symmetric memory),
and the permutation kernels address that memory directly:

  forward   publish x, router weights, expert ids            (local copies into the shared buffers)
            all-gather the ids and weights (a few hundred KiB; doubles as the "published" barrier)
            route all slots over this rank's experts plus a 'not mine' bin: row_map then names global slots
            gather those rows from their owners                (ck_moe_gather_rows_peer: NVLink loads)
            up projection + activation (router weight folded in; the weights travel with the ids)
            down projection, every result row stored into its owner's return buffer from the GEMM epilogue
                                                               (ck_moe_grouped_linear_scatter_peer: NVLink stores)
            barrier; k-way sum of the local return buffer      (ck_moe_combine_rows)
  backward  the same shape: publish dy, barrier, gather dy rows from their owners, dgrad(down) + activation
            backward, weight grads (local), router-weight grads scattered to their owners, dgrad(up) rows stored
            into the owners' return buffers, barrier, k-way sum.

Rows cross NVLink once per direction, overlapped tile by tile with the GEMM that produces them; no send / receive
staging buffers exist.  Ordering between ranks comes only from stream-ordered NCCL collectives issued between the
phases; no kernel waits on another GPU.  A global flat slot names a routed row: ``g = rank * S + token * k + j``
with ``S = max_tokens * k`` slots per rank.

The reference is single-GPU; the contract is its layer on the concatenated batch (expert weights sharded as in
:func:`expert_parallel.shard_expert_state_dict`).
"""

from __future__ import annotations

import ctypes
from dataclasses import dataclass

import torch
import torch.distributed as dist

from . import _lib
from .moe import combine_rows, cta_pair_kernels, dgates_parts, dgrad_down, reduce_dgates, up_act_fwd, wgrad
from .routing import Routing, route


def _ptr_array(ptrs: list[int]):
    return (ctypes.c_void_p * len(ptrs))(*ptrs)


def _gather_rows_peer(ptrs, S: int, dst, r: Routing, experts: int, fan_out: int, row_begin: int, row_end: int) -> None:
    status = _lib.status_word(dst.device)
    with torch.cuda.device(dst.device), _lib.launch("gather_rows_peer"):
        st = _lib.lib.ck_moe_gather_rows_peer(_ptr_array(ptrs), len(ptrs), S, dst.data_ptr(), r.row_map.data_ptr(),
                                              r.padded_off.data_ptr(), None, experts,
                                              dst.size(0), fan_out, dst.size(1), row_begin, row_end,
                                              _lib.dtype_code(dst.dtype), status.data_ptr(), _lib.stream_ptr())
    _lib.check(st, "ck_moe_gather_rows_peer")


def _linear_scatter_peer(x, w, r: Routing, ptrs, S: int, trans_w: bool) -> None:
    status = _lib.status_word(x.device)
    E = w.size(0)
    N, K = (w.size(2), w.size(1)) if trans_w else (w.size(1), w.size(2))
    assert x.size(1) == K
    with torch.cuda.device(x.device), _lib.launch("grouped_linear_scatter_peer", 1, 2.0 * x.size(0) * N * K):
        st = _lib.lib.ck_moe_grouped_linear_scatter_peer(x.data_ptr(), w.data_ptr(), r.mtile_off.data_ptr(),
                                                         r.row_map.data_ptr(), None, _ptr_array(ptrs),
                                                         len(ptrs), S, E, x.size(0), N, K, int(trans_w),
                                                         _lib.dtype_code(x.dtype), status.data_ptr(), _lib.stream_ptr())
    _lib.check(st, "ck_moe_grouped_linear_scatter_peer")


def _up_act_pull_peer(ptrs, S: int, fan_out: int, w_fc, gate_w, r: Routing, act, h, xg_out, act_kind: int) -> None:
    """Up projection whose producer warps pull the routed rows from their owners (NVLink loads inside the GEMM)."""
    status = _lib.status_word(act.device)
    E, two_i, H = w_fc.shape
    with torch.cuda.device(act.device), _lib.launch("up_act_fwd_peer", 1, 2.0 * act.size(0) * two_i * H):
        st = _lib.lib.ck_moe_up_act_fwd_gather_peer(_ptr_array(ptrs), len(ptrs), S, fan_out, w_fc.data_ptr(), _lib.ptr(gate_w),
                                                    r.row_map.data_ptr(), r.mtile_off.data_ptr(), act.data_ptr(), _lib.ptr(h),
                                                    _lib.ptr(xg_out), E, act.size(0), H, two_i // 2, act_kind,
                                                    _lib.dtype_code(act.dtype), status.data_ptr(), _lib.stream_ptr())
    _lib.check(st, "ck_moe_up_act_fwd_gather_peer")


def _dgrad_down_pull_peer(ptrs, S: int, fan_out: int, w_proj, h, gate_w, r: Routing, dh, dg_part, dyg_out, act_kind: int) -> None:
    status = _lib.status_word(dh.device)
    E, H, I = w_proj.shape
    with torch.cuda.device(dh.device), _lib.launch("dgrad_down_peer", 1, 2.0 * dh.size(0) * H * I):
        st = _lib.lib.ck_moe_dgrad_down_gather_peer(_ptr_array(ptrs), len(ptrs), S, fan_out, w_proj.data_ptr(), h.data_ptr(),
                                                    _lib.ptr(gate_w), r.row_map.data_ptr(), r.mtile_off.data_ptr(), dh.data_ptr(),
                                                    None, _lib.ptr(dg_part), _lib.ptr(dyg_out), E, dh.size(0), H, I, act_kind,
                                                    _lib.dtype_code(dh.dtype), status.data_ptr(), _lib.stream_ptr())
    _lib.check(st, "ck_moe_dgrad_down_gather_peer")


def _scatter_scalars_peer(vals_by_slot, flat, n: int, ptrs, S: int) -> None:
    status = _lib.status_word(vals_by_slot.device)
    with torch.cuda.device(vals_by_slot.device), _lib.launch("peer_scatter_scalars"):
        st = _lib.lib.ck_peer_scatter_scalars(vals_by_slot.data_ptr(), flat.data_ptr(), n, 1, _ptr_array(ptrs), len(ptrs), S,
                                              vals_by_slot.element_size(), status.data_ptr(), _lib.stream_ptr())
    _lib.check(st, "ck_peer_scatter_scalars")


@dataclass
class PeerBuffers:
    """One rank's shared buffers and every rank's address of them (``*_ptrs[r]`` = rank r's buffer as mapped here).

    tokens [max_tokens, H]  x in forward, dy in backward          rows [S, H]  returned expert outputs / input grads
    weights [S]             router weights, dtype of x (local)    dgates [S]   router-weight grads, fp32
    ids [S] int32           published expert ids (``num_experts`` = "no row" on the unused tail)
    ``ids`` and ``weights`` are views into one byte buffer ``published`` (ids first), so one all-gather moves both.
    """

    rank: int
    world: int
    max_tokens: int
    top_k: int
    tokens: torch.Tensor
    rows: torch.Tensor
    weights: torch.Tensor
    dgates: torch.Tensor
    ids: torch.Tensor
    tokens_ptrs: list[int]
    rows_ptrs: list[int]
    dgates_ptrs: list[int]
    published: torch.Tensor | None = None  # uint8 [S * (4 + element size)]: ids | weights, when they share storage

    @property
    def slots(self) -> int:
        return self.max_tokens * self.top_k

    def split_published(self, gathered: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
        """(ids_all int32 [world * S], weights_all [world * S]) from the all-gathered ``published`` buffers."""
        S, esz = self.slots, self.weights.element_size()
        per_rank = gathered.view(self.world, S * (4 + esz))
        ids_all = per_rank[:, : 4 * S].contiguous().view(torch.int32).reshape(-1)
        weights_all = per_rank[:, 4 * S:].contiguous().view(self.weights.dtype).reshape(-1)
        return ids_all, weights_all


def packed_publication(slots: int, dtype: torch.dtype, device: torch.device) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """(published uint8, ids int32 view, weights view): ids and router weights in one buffer, one all-gather for both."""
    esz = torch.empty(0, dtype=dtype).element_size()
    published = torch.empty(slots * (4 + esz), dtype=torch.uint8, device=device)
    return published, published[: 4 * slots].view(torch.int32), published[4 * slots:].view(dtype)


@dataclass
class _Plan:
    routing: Routing   # all ranks' slots routed over [this rank's experts..., "not mine"]; row_map[p] = global flat slot
    rows: int | None   # padded rows of the local experts (a multiple of 128, may be 0); None: not read back (capacity mode)
    cap: int           # rows allocated: max(rows, 128), or the caller's capacity
    split: int         # number of pull windows beyond the first (0: one window)
    edges: list[int] | None            # window w covers the m-tiles [edges[w], edges[w + 1])
    mtile_windows: list[torch.Tensor] | None  # mtile_off clamped to each window
    own_map: torch.Tensor | None = None  # capacity mode: row_map[:cap] with -1 beyond the local experts' rows


class PeerExpertEngine:
    """The per-rank phases; the caller puts a collective between them (see :class:`PeerExpertParallelMoE`)."""

    def __init__(self, buffers: PeerBuffers, num_experts: int, act_kind: int = _lib.CK_ACT_SWIGLU,
                 expert_to_rank: list[int] | None = None, capacity_rows: int | None = None) -> None:
        """``expert_to_rank[e]``: the rank that owns expert e (default: contiguous blocks, rank g owns
        [g E/G, (g+1) E/G)); every rank must own exactly E/G experts, and its weight tensors list them in increasing
        expert id (see :func:`expert_parallel.shard_expert_state_dict`).  ``capacity_rows``: allocate this many padded
        rows per call instead of reading the exact count back from the device (no host synchronisation in the step);
        a call whose routing needs more rows computes nothing and raises CK_DEV_META in the device status word."""
        if num_experts % buffers.world != 0:
            raise ValueError("num_experts must be divisible by the number of ranks")
        self.b = buffers
        self.num_experts = num_experts
        self.local_experts = num_experts // buffers.world
        self.act_kind = act_kind
        self._side: torch.cuda.Stream | None = None
        if expert_to_rank is None:
            expert_to_rank = [e // self.local_experts for e in range(num_experts)]
        if len(expert_to_rank) != num_experts or any(expert_to_rank.count(r) != self.local_experts for r in range(buffers.world)):
            raise ValueError("expert_to_rank must give every rank exactly num_experts / world experts")
        self.expert_to_rank = list(expert_to_rank)
        self.local_expert_ids = [e for e in range(num_experts) if expert_to_rank[e] == buffers.rank]
        # global expert id -> local slot of the routing pass (0 .. E/G - 1), E/G = "not mine"; entry [num_experts] is the
        # padding id of unused slots
        table = [self.local_experts] * (num_experts + 1)
        for slot, e in enumerate(self.local_expert_ids):
            table[e] = slot
        self._local_slot = torch.tensor(table, dtype=torch.int32, device=buffers.tokens.device)
        if capacity_rows is not None:
            capacity_rows = max(_lib.CK_TILE_M, -(-int(capacity_rows) // _lib.CK_TILE_M) * _lib.CK_TILE_M)
        self.capacity_rows = capacity_rows

    # ---- forward -------------------------------------------------------------------------------------
    def publish(self, x: torch.Tensor, router_weights: torch.Tensor, selected_experts: torch.Tensor) -> None:
        b = self.b
        T = x.size(0)
        if T > b.max_tokens:
            raise RuntimeError(f"{T} tokens exceed the shared buffers' {b.max_tokens}")
        _lib.require_cuda(x, router_weights, selected_experts)
        b.tokens[:T].copy_(x)
        b.weights[: T * b.top_k].copy_(router_weights.reshape(-1))
        b.ids[: T * b.top_k].copy_(selected_experts.reshape(-1))
        b.ids[T * b.top_k:].fill_(self.num_experts)

    def plan(self, ids_all: torch.Tensor) -> _Plan:
        """ids_all int32 [world * S]: every rank's published ids, rank-major.  One routing pass over all slots with
        the ids of other ranks' experts folded into a last "not mine" bin: the local experts' segments of the padded
        layout then list global flat slots, in (source rank, token) order inside every expert."""
        epr = self.local_experts
        in_range = (ids_all >= 0) & (ids_all <= self.num_experts)
        loc = self._local_slot[ids_all.clamp(0, self.num_experts).long()]
        r = route(loc, epr + 1)
        # ids outside [0, num_experts] would be "not mine" on every rank and their rows would never be computed
        n_bad = (~in_range).sum(dtype=torch.int32)
        if self.capacity_rows is not None:
            # no read-back: the capacity bounds the allocation, the kernels refuse (CK_DEV_META) when the tile tables
            # describe more rows, and bad ids raise CK_DEV_RANGE in the same status word
            status = _lib.status_word(ids_all.device)
            status.bitwise_or_((n_bad > 0).to(torch.int32) * _lib.CK_DEV_RANGE)
            cap = self.capacity_rows
            own = torch.arange(cap, device=ids_all.device, dtype=torch.int32) < r.padded_off[epr]
            if r.row_map.numel() < cap:
                raise RuntimeError("capacity_rows exceeds the routing pass's own bound")
            own_map = torch.where(own, r.row_map[:cap], -1)
            return _Plan(r, None, cap, 0, None, None, own_map)
        rows, bad = torch.stack([r.padded_off[epr], n_bad]).tolist()  # the one host sync: rows to allocate
        if bad:
            raise RuntimeError(f"{bad} expert ids outside [0, {self.num_experts}) reached the expert-parallel layer")
        # Windows of the padded rows: window w + 1 is pulled on a side stream while the GEMM runs on window w.
        tiles = rows // _lib.CK_TILE_M
        edges = None
        if self.MIN_TILES_TO_SPLIT is not None and tiles >= self.MIN_TILES_TO_SPLIT:
            n_win = max(2, min(self.PULL_WINDOWS, tiles // max(2, self.MIN_TILES_TO_SPLIT // 2)))
            if n_win == 2:  # a quarter first (the exposed pull), the rest beside its GEMM
                edges = [0, min(tiles - 2, max(2, (tiles // 4 + 1) & ~1)), tiles]
            else:           # equal shares, whole CTA pairs
                edges = sorted({min(tiles, ((tiles * w // n_win) + 1) & ~1) for w in range(n_win)} | {0, tiles})
            if len(edges) < 3:
                edges = None
        windows = None
        if edges is not None:
            windows = [r.mtile_off.clamp(min=a, max=b) for a, b in zip(edges[:-1], edges[1:])]
        return _Plan(r, rows, max(rows, _lib.CK_TILE_M), 0 if edges is None else len(edges) - 2, edges, windows)

    # Windowed schedule: the padded rows are cut into PULL_WINDOWS windows; the first is pulled, then window w + 1 is pulled on a
    # side stream WHILE the GEMM runs on window w (only the first pull is exposed).  A pull kernel never becomes resident on an SM that hosts a persistent GEMM CTA (its warps
    # hold the whole register file; tried 128-thread blocks, the shared-memory carve-out, a high-priority stream, the one-CTA
    # flavour: the later kernel always started in the earlier one's tail), so the first-window GEMM is launched on
    # ``SMS - PULL_SMS`` SMs and the pull gets the rest.  That costs the GEMM next to nothing: the layer runs under the
    # board's power cap, and a GEMM on 132 of 148 SMs settles at a higher clock (measured on the Mixtral-shaped layer:
    # 29.02 ms per step on 148 SMs, 29.14 ms on 132, 29.91 ms on 120).  Set MIN_TILES_TO_SPLIT to None for one window.
    MIN_TILES_TO_SPLIT: int | None = 16
    PULL_SMS = 16
    # Two windows: a quarter of the rows, then the rest.  Four equal windows were measured at 4 GPUs: the 64-expert layer
    # 16.18 against 16.20 ms per step (what the extra windows hide, 1.5 ms, the four narrower GEMM launches give back: the
    # ranks' GEMM time rose from 12.7 to 13.9 ms), the 8-expert layer within the spread between runs.
    PULL_WINDOWS = 2

    def _side_stream(self) -> torch.cuda.Stream:
        if self._side is None:
            self._side = torch.cuda.Stream(device=self.b.tokens.device, priority=-1)
        return self._side

    def _pull_then(self, plan: _Plan, dst: torch.Tensor, gemm) -> None:
        """Pulls the padded rows of ``dst`` from their owners and runs ``gemm(mtile_off)`` on them.  With two windows:
        pull A; then pull B on the side stream while gemm(A) runs; gemm(B) once B has landed."""
        b, r = self.b, plan.routing
        if not plan.split:
            _gather_rows_peer(b.tokens_ptrs, b.slots, dst, r, self.local_experts, b.top_k, 0, plan.cap)
            gemm(r.mtile_off)
            return
        main, side = torch.cuda.current_stream(), self._side_stream()
        rows = [e * _lib.CK_TILE_M for e in plan.edges]
        rows[-1] = plan.cap
        n_win = len(plan.mtile_windows)
        _gather_rows_peer(b.tokens_ptrs, b.slots, dst, r, self.local_experts, b.top_k, rows[0], rows[1])
        first_done = torch.cuda.Event()
        first_done.record(main)
        # the later windows are pulled back to back on the side stream, after the first pull (which keeps the whole machine)
        side.wait_event(first_done)
        landed = []
        with torch.cuda.stream(side):
            for w in range(1, n_win):
                _gather_rows_peer(b.tokens_ptrs, b.slots, dst, r, self.local_experts, b.top_k, rows[w], rows[w + 1])
                ev = torch.cuda.Event()
                ev.record(side)
                landed.append(ev)
        dst.record_stream(side)
        # the GEMM of every window but the last runs beside a pull: it leaves PULL_SMS SMs to it
        narrow = max(2, _lib.lib.ck_gemm_sm_budget() - self.PULL_SMS)
        for w in range(n_win):
            if w > 0:
                main.wait_event(landed[w - 1])
            if w + 1 < n_win:
                with _lib.gemm_sm_budget(narrow):
                    gemm(plan.mtile_windows[w])
            else:
                gemm(plan.mtile_windows[w])

    # True: the GEMMs' own producer warp pulls the rows over NVLink (cp.async by row index, CTA-pair kernels) and leaves a
    # local grouped copy behind for the weight gradients.  False (default): a separate pull kernel runs first and the GEMM
    # reads its output with tiled TMA loads -- an A tile is fetched once per n-tile, so pulling inside the GEMM would
    # cross NVLink 56-112 times per row, and the cp.async path is the slower fetch path even locally.
    FUSED_PULL = False

    def fwd_compute(self, plan: _Plan, weights_all: torch.Tensor, w_fc: torch.Tensor, w_proj: torch.Tensor,
                    need_grad: bool):
        """weights_all [world * S]: every rank's published router weights (indexed by global flat slot)."""
        b, r = self.b, plan.routing
        dev, dt = b.tokens.device, b.tokens.dtype
        H = b.tokens.size(1)
        two_i = w_fc.size(1)
        act = torch.empty(plan.cap, two_i // 2, dtype=dt, device=dev)
        h = torch.empty(plan.cap, two_i, dtype=dt, device=dev) if need_grad else None
        if self.FUSED_PULL and cta_pair_kernels() and not plan.split:
            xg = torch.empty(plan.cap, H, dtype=dt, device=dev) if need_grad else None
            _up_act_pull_peer(b.tokens_ptrs, b.slots, b.top_k, w_fc, weights_all, r, act, h, xg, self.act_kind)
        else:
            xg = torch.empty(plan.cap, H, dtype=dt, device=dev)
            self._pull_then(plan, xg, lambda mt: up_act_fwd(xg, w_fc, None, weights_all, r.row_map, mt, act, h, self.act_kind))
        _linear_scatter_peer(act, w_proj, r, b.rows_ptrs, b.slots, False)
        return xg, act, h

    def fwd_finish(self, T: int) -> torch.Tensor:
        b = self.b
        y = torch.empty(T, b.tokens.size(1), dtype=b.tokens.dtype, device=b.tokens.device)
        if T:
            combine_rows(b.rows, None, None, y, b.top_k)
        return y

    # ---- backward ------------------------------------------------------------------------------------
    def bwd_publish(self, dy: torch.Tensor) -> None:
        self.b.tokens[: dy.size(0)].copy_(dy)

    def bwd_compute(self, plan: _Plan, saved, weights_all, w_fc, w_proj, need_wfc: bool, need_wproj: bool, need_x: bool):
        b, r = self.b, plan.routing
        xg, act, h = saved
        dev, dt = act.device, act.dtype
        H = b.tokens.size(1)
        dyg = torch.empty(plan.cap, H, dtype=dt, device=dev)
        dh = torch.empty(plan.cap, w_fc.size(1), dtype=dt, device=dev)
        # router-weight grads by global flat slot: per-part partial sums, added in a fixed order
        dg_part = torch.empty(dgates_parts(w_fc.size(1) // 2), plan.cap, dtype=torch.float32, device=dev)
        if self.FUSED_PULL and cta_pair_kernels() and not plan.split:
            _dgrad_down_pull_peer(b.tokens_ptrs, b.slots, b.top_k, w_proj, h, weights_all, r, dh, dg_part, dyg, self.act_kind)
        else:
            self._pull_then(plan, dyg,
                            lambda mt: dgrad_down(dyg, w_proj, h, weights_all, r.row_map, mt, dh, None, dg_part, self.act_kind))
        dgates = torch.zeros(b.world * b.slots, dtype=torch.float32, device=dev)
        reduce_dgates(dg_part, r.row_map, r.padded_off, self.local_experts, dgates)
        d_wproj = d_wfc = None
        if need_wproj:
            d_wproj = torch.empty_like(w_proj)
            wgrad(dyg, act, r.padded_off, d_wproj)
        if plan.own_map is not None:  # capacity mode: entries beyond the local experts' rows are masked to -1 (skipped)
            _scatter_scalars_peer(dgates, plan.own_map, plan.cap, b.dgates_ptrs, b.slots)
        else:
            _scatter_scalars_peer(dgates, r.row_map, plan.rows, b.dgates_ptrs, b.slots)  # local experts' rows only
        if need_x:
            _linear_scatter_peer(dh, w_fc, r, b.rows_ptrs, b.slots, True)
        if need_wfc:
            d_wfc = torch.empty_like(w_fc)
            wgrad(dh, xg, r.padded_off, d_wfc)
        return d_wfc, d_wproj

    def bwd_finish(self, T: int, need_x: bool):
        b = self.b
        dx = None
        if need_x:
            dx = torch.empty(T, b.tokens.size(1), dtype=b.tokens.dtype, device=b.tokens.device)
            if T:
                combine_rows(b.rows, None, None, dx, b.top_k)
        d_rw = b.dgates[: T * b.top_k].view(T, b.top_k).to(b.tokens.dtype, copy=True)
        return dx, d_rw


class _NcclExchange:
    """Stream-ordered ordering points between the phases: an all-gather of the ids and a one-element all-reduce."""

    def __init__(self, group, device: torch.device) -> None:
        self.group = group
        self.flag = torch.zeros(1, dtype=torch.float32, device=device)

    def all_gather(self, local: torch.Tensor) -> torch.Tensor:
        out = torch.empty(dist.get_world_size(self.group) * local.numel(), dtype=local.dtype, device=local.device)
        dist.all_gather_into_tensor(out, local, group=self.group)
        return out

    def barrier(self) -> None:
        dist.all_reduce(self.flag, group=self.group)


class _PeerExperts(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, router_weights, w_fc, w_proj, selected_experts, engine: PeerExpertEngine, exchange):
        need_grad = any(ctx.needs_input_grad[:4])
        engine.publish(x, router_weights, selected_experts)
        if engine.b.published is not None:
            # ids and router weights share one buffer: a single all-gather, which is also the "everything is published"
            # ordering point
            ids_all, weights_all = engine.b.split_published(exchange.all_gather(engine.b.published))
        else:
            ids_all = exchange.all_gather(engine.b.ids)
            weights_all = exchange.all_gather(engine.b.weights)
        plan = engine.plan(ids_all)
        saved = engine.fwd_compute(plan, weights_all, w_fc, w_proj, need_grad)
        exchange.barrier()
        y = engine.fwd_finish(x.size(0))
        ctx.engine, ctx.exchange, ctx.plan, ctx.tokens = engine, exchange, plan, x.size(0)
        ctx.save_for_backward(w_fc, w_proj, weights_all, *saved)
        return y

    @staticmethod
    def backward(ctx, dy):
        w_fc, w_proj, weights_all, *saved = ctx.saved_tensors
        engine, exchange, plan, T = ctx.engine, ctx.exchange, ctx.plan, ctx.tokens
        need_x, need_rw, need_wfc, need_wproj = ctx.needs_input_grad[:4]
        engine.bwd_publish(dy.contiguous().to(saved[0].dtype))
        exchange.barrier()
        d_wfc, d_wproj = engine.bwd_compute(plan, saved, weights_all, w_fc, w_proj, need_wfc, need_wproj, need_x)
        exchange.barrier()
        dx, d_rw = engine.bwd_finish(T, need_x)
        return dx, (d_rw if need_rw else None), d_wfc, d_wproj, None, None, None


def allocate_symmetric_buffers(max_tokens: int, hidden_size: int, top_k: int, dtype: torch.dtype, group=None,
                               device: torch.device | None = None) -> PeerBuffers:
    """Allocates the shared buffers in symmetric memory and exchanges their addresses (collective over ``group``)."""
    import torch.distributed._symmetric_memory as symm_mem

    group = group if group is not None else dist.group.WORLD
    device = device or torch.device("cuda", torch.cuda.current_device())
    S = max_tokens * top_k

    def shared(shape, dt):
        t = symm_mem.empty(shape, dtype=dt, device=device)
        hdl = symm_mem.rendezvous(t, group)
        return t, [int(p) for p in hdl.buffer_ptrs]

    tokens, tokens_ptrs = shared((max_tokens, hidden_size), dtype)
    rows, rows_ptrs = shared((S, hidden_size), dtype)
    dgates, dgates_ptrs = shared((S,), torch.float32)
    published, ids, weights = packed_publication(S, dtype, device)
    return PeerBuffers(dist.get_rank(group), dist.get_world_size(group), max_tokens, top_k, tokens, rows, weights,
                       dgates, ids, tokens_ptrs, rows_ptrs, dgates_ptrs, published)


class PeerExpertParallelMoE:
    """Callable with the signature of :class:`expert_parallel.ExpertParallelMoE`:
    ``y = ep(x, router_weights, selected_experts, w_fc_local, w_proj_local)`` with GLOBAL expert ids.

    The shared buffers are sized for ``max_tokens`` rows of ``hidden_size`` per rank and are reused by every call
    (forward and backward of one call must finish before the next call's forward starts, which stream order gives)."""

    def __init__(self, num_experts: int, top_k: int, max_tokens: int, hidden_size: int, dtype: torch.dtype, group=None,
                 act_kind: int = _lib.CK_ACT_SWIGLU, buffers: PeerBuffers | None = None, exchange=None,
                 expert_to_rank: list[int] | None = None, capacity_factor: float | None = None) -> None:
        """``capacity_factor``: None reads the exact number of rows this rank's experts received back from the device
        once per call (one host synchronisation); a number allocates ``capacity_factor * max_tokens * top_k`` rows (the
        share of a perfectly balanced routing, times the factor) plus one tile per local expert and never synchronises --
        a batch that routes more rows to this rank is refused on the device (CK_DEV_META, see check_device_status)."""
        self.group = group if group is not None else dist.group.WORLD
        self.buffers = buffers or allocate_symmetric_buffers(max_tokens, hidden_size, top_k, dtype, self.group)
        cap_rows = None
        if capacity_factor is not None:
            world = dist.get_world_size(self.group)
            cap_rows = int(capacity_factor * max_tokens * top_k) + (num_experts // world) * _lib.CK_TILE_M
            cap_rows = min(cap_rows, world * max_tokens * top_k + (num_experts // world) * _lib.CK_TILE_M)
        self.engine = PeerExpertEngine(self.buffers, num_experts, act_kind, expert_to_rank, cap_rows)
        self.exchange = exchange or _NcclExchange(self.group, self.buffers.tokens.device)
        self.top_k = top_k

    def __call__(self, x, router_weights, selected_experts, w_fc_local, w_proj_local):
        return _PeerExperts.apply(x.contiguous(), router_weights, w_fc_local.contiguous(), w_proj_local.contiguous(),
                                  selected_experts.to(torch.int32), self.engine, self.exchange)
