"""Expert parallelism for the MoE expert path: experts block-partitioned over the ranks of a process
group, tokens data-parallel, rows exchanged with all-to-all-v (NCCL over NVLink on GPUs).
(:mod:`peer_parallel` is the faster transport on one node: the kernels read and write the other ranks'
buffers directly; this module is the portable one and the one whose host logic runs on CPU ranks in tests.)

The reference has no multi-GPU path; the contract is the single-process layer on the concatenated
batch.  Rank g owns experts [g*E/G, (g+1)*E/G) and only those slices of ``c_fc.weight`` /
``c_proj.weight`` (so expert weight gradients need no all-reduce).

  forward   local route by global expert id (sorted by expert == sorted by destination rank)
            -> exchange the per-(rank, expert) counts            (all_to_all_single, int64[G * E/G])
            -> gather the token rows in sorted order              (send buffer)
            -> all-to-all-v of the rows                           (dispatch)
            -> local expert computation on the received rows      (the fused grouped-GEMM path, top_k = 1)
            -> all-to-all-v back                                  (return)
            -> router-weighted k-way combine on the source rank
  backward  the mirror image; every exchange step is an autograd function whose backward is the
            reverse exchange.

Overlap (``chunks`` > 1, GPUs): the local tokens are cut into chunks that run the whole pipeline on streams of their own, so
the all-to-all of one chunk travels while the grouped GEMMs of another compute, forward and backward (autograd replays every
op on the stream it ran on).  The persistent GEMM grids own every SM they run on, so the layer lowers their SM budget by
``comm_sms`` for the process (ck_set_gemm_sm_budget): NCCL's kernels then find free SMs instead of waiting for a GEMM's tail.
Under the board's power cap the narrower GEMMs settle at a higher clock and lose next to nothing.

Receive sizes are data dependent: one device-to-host read of the count matrix per call (per chunk).
``expert_fn`` / ``route_fn`` are injectable so the permutation and exchange logic can run on CPU ranks
(gloo) with a CPU expert function in tests.
"""

from __future__ import annotations

from typing import Callable

import torch
import torch.distributed as dist


def _all_to_all_rows(inp: torch.Tensor, out_rows: int, in_splits: list[int], out_splits: list[int], group) -> torch.Tensor:
    out = torch.empty((out_rows,) + tuple(inp.shape[1:]), dtype=inp.dtype, device=inp.device)
    if inp.is_cuda:
        dist.all_to_all_single(out, inp.contiguous(), output_split_sizes=out_splits, input_split_sizes=in_splits, group=group)
    else:
        # gloo has no all_to_all_single with uneven splits on every build: pairwise send / recv
        world, rank = dist.get_world_size(group), dist.get_rank(group)
        ins = list(inp.contiguous().split(in_splits))
        outs = list(out.split(out_splits))
        outs[rank].copy_(ins[rank])
        ops = []
        for peer in range(world):
            if peer == rank:
                continue
            gpeer = dist.get_global_rank(group, peer) if group is not None else peer
            if in_splits[peer] > 0:
                ops.append(dist.P2POp(dist.isend, ins[peer].contiguous(), gpeer, group))
            if out_splits[peer] > 0:
                ops.append(dist.P2POp(dist.irecv, outs[peer], gpeer, group))
        if ops:
            for req in dist.batch_isend_irecv(ops):
                req.wait()
    return out


class _AllToAllRows(torch.autograd.Function):
    """Rows [sum(in_splits), ...] -> [sum(out_splits), ...]; the gradient travels the reverse way."""

    @staticmethod
    def forward(ctx, inp, in_splits, out_splits, group):
        ctx.in_splits, ctx.out_splits, ctx.group = in_splits, out_splits, group
        return _all_to_all_rows(inp, sum(out_splits), in_splits, out_splits, group)

    @staticmethod
    def backward(ctx, grad):
        return _all_to_all_rows(grad.contiguous(), sum(ctx.in_splits), ctx.out_splits, ctx.in_splits, ctx.group), None, None, None


class _GatherSorted(torch.autograd.Function):
    """rows[j] = x[tok[j]]; backward sums the k copies of every token in fp32."""

    @staticmethod
    def forward(ctx, x, tok):
        ctx.save_for_backward(tok)
        ctx.tokens = x.size(0)
        return x.index_select(0, tok)

    @staticmethod
    def backward(ctx, grad):
        (tok,) = ctx.saved_tensors
        acc = torch.zeros(ctx.tokens, grad.size(1), dtype=torch.float32, device=grad.device)
        acc.index_add_(0, tok, grad.float())
        return acc.to(grad.dtype), None


class _CombineSorted(torch.autograd.Function):
    """y[t] = sum_j w[flat_j] * rows[j] over the sorted rows of token t (fp32 accumulation)."""

    @staticmethod
    def forward(ctx, rows, w_flat_sorted, tok, tokens: int):
        ctx.save_for_backward(rows, w_flat_sorted, tok)
        acc = torch.zeros(tokens, rows.size(1), dtype=torch.float32, device=rows.device)
        acc.index_add_(0, tok, rows.float() * w_flat_sorted.float().unsqueeze(1))
        return acc.to(rows.dtype)

    @staticmethod
    def backward(ctx, dy):
        rows, w, tok = ctx.saved_tensors
        dyg = dy.index_select(0, tok)
        d_rows = (dyg.float() * w.float().unsqueeze(1)).to(rows.dtype)
        d_w = (dyg.float() * rows.float()).sum(dim=1).to(w.dtype)
        return d_rows, d_w, None, None


class _GatherSortedCuda(torch.autograd.Function):
    """rows[j] = x[sorted_idx[j] // k] (one streaming kernel); backward = deterministic k-way sum."""

    @staticmethod
    def forward(ctx, x, sorted_idx32, pos32, k: int):
        from .moe import gather_rows_scaled

        ctx.save_for_backward(pos32)
        ctx.k, ctx.tokens = k, x.size(0)
        rows = torch.empty(sorted_idx32.numel(), x.size(1), dtype=x.dtype, device=x.device)
        gather_rows_scaled(x.contiguous(), rows, sorted_idx32, None, k)
        return rows

    @staticmethod
    def backward(ctx, grad):
        from .moe import combine_rows

        (pos32,) = ctx.saved_tensors
        dx = torch.empty(ctx.tokens, grad.size(1), dtype=grad.dtype, device=grad.device)
        combine_rows(grad.contiguous(), pos32, None, dx, ctx.k)
        return dx, None, None, None


class _CombineSortedCuda(torch.autograd.Function):
    """y[t] = sum_j w[t, j] * rows[pos[t*k+j]] with fp32 accumulation; backward = scaled gather + row dots."""

    @staticmethod
    def forward(ctx, rows, w, sorted_idx32, pos32, k: int):
        from .moe import combine_rows

        rows = rows.contiguous()
        w = w.contiguous()
        ctx.save_for_backward(rows, w, sorted_idx32, pos32)
        ctx.k = k
        y = torch.empty(w.size(0), rows.size(1), dtype=rows.dtype, device=rows.device)
        combine_rows(rows, pos32, w.view(-1), y, k)
        return y

    @staticmethod
    def backward(ctx, dy):
        from .moe import gather_rows_scaled, row_dots

        rows, w, sorted_idx32, pos32 = ctx.saved_tensors
        dy = dy.contiguous()
        d_rows = torch.empty_like(rows)
        gather_rows_scaled(dy, d_rows, sorted_idx32, w.view(-1), ctx.k)
        d_w = torch.empty_like(w)
        row_dots(rows, pos32, dy, d_w.view(-1), ctx.k)
        return d_rows, d_w, None, None, None


def _default_route(ids: torch.Tensor, num_experts: int):
    from .routing import route

    r = route(ids, num_experts, with_tile_metadata=False)
    return r.sorted_idx, r.counts


def _default_expert_fn(rows, local_ids, w_fc, w_proj, act_kind):
    from .moe import expert_shard

    return expert_shard(rows, local_ids, w_fc, w_proj, act_kind)


class ExpertParallelMoE:
    """Callable: ``y = ep(x, router_weights, selected_experts, w_fc_local, w_proj_local)``.

    x [T_local, H]; router_weights / selected_experts [T_local, k] with GLOBAL expert ids;
    w_fc_local [E/G, 2I, H], w_proj_local [E/G, H, I]: this rank's experts."""

    def __init__(self, num_experts: int, top_k: int, group=None, act_kind: int = 0,
                 expert_fn: Callable | None = None, route_fn: Callable | None = None, chunks: int = 1,
                 comm_sms: int = 16) -> None:
        """``chunks``: token chunks pipelined on their own streams (1 = everything on the caller's stream); with more than
        one chunk the grouped GEMMs of this PROCESS leave ``comm_sms`` SMs free from now on, for the collectives' kernels."""
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        if num_experts % self.world != 0:
            raise ValueError("num_experts must be divisible by the number of ranks")
        self.num_experts = num_experts
        self.local_experts = num_experts // self.world
        self.top_k = top_k
        self.act_kind = act_kind
        self.expert_fn = expert_fn or _default_expert_fn
        self.route_fn = route_fn or _default_route
        self.chunks = max(1, int(chunks))
        self._streams: list = []
        if self.chunks > 1 and torch.cuda.is_available():
            from . import _lib

            all_sms = torch.cuda.get_device_properties(torch.cuda.current_device()).multi_processor_count
            _lib.lib.ck_set_gemm_sm_budget(max(2, all_sms - int(comm_sms)))

    def __call__(self, x, router_weights, selected_experts, w_fc_local, w_proj_local):
        """Runs the layer; with ``chunks`` > 1 on CUDA tensors, chunk by chunk on side streams (see the module docstring)."""
        T = x.size(0)
        if self.chunks == 1 or not x.is_cuda or T < 2 * self.chunks:
            return self._run(x, router_weights, selected_experts, w_fc_local, w_proj_local)
        if not self._streams:
            self._streams = [torch.cuda.Stream(device=x.device) for _ in range(self.chunks)]
        main = torch.cuda.current_stream()
        ready = main.record_event()
        bounds = [T * c // self.chunks for c in range(self.chunks + 1)]
        outs = []
        for c, st in enumerate(self._streams):
            sl = slice(bounds[c], bounds[c + 1])
            st.wait_event(ready)
            with torch.cuda.stream(st):
                y_c = self._run(x[sl], router_weights[sl], selected_experts[sl], w_fc_local, w_proj_local)
            outs.append(y_c)
        for t in (x, router_weights, selected_experts, w_fc_local, w_proj_local):
            for st in self._streams:
                t.record_stream(st)
        for y_c, st in zip(outs, self._streams):
            main.wait_stream(st)
            y_c.record_stream(main)
        return torch.cat(outs, dim=0)

    def _run(self, x, router_weights, selected_experts, w_fc_local, w_proj_local):
        G, epr, k = self.world, self.local_experts, self.top_k
        T = x.size(0)
        dev = x.device
        flat_ids = selected_experts.reshape(-1)
        sorted_idx32, counts = self.route_fn(flat_ids, self.num_experts)
        on_gpu = dev.type == "cuda"

        # per-(destination rank, local expert) counts -> what every source sends us
        send_counts = counts.to(torch.int64).view(G, epr)
        recv_counts = torch.empty_like(send_counts)
        if dev.type == "cuda":
            dist.all_to_all_single(recv_counts, send_counts.contiguous(), group=self.group)
        else:
            gathered = [torch.empty_like(send_counts) for _ in range(G)]
            dist.all_gather(gathered, send_counts.contiguous(), group=self.group)
            recv_counts = torch.stack([g[self.rank] for g in gathered])
        both = torch.stack([send_counts.sum(1), recv_counts.sum(1)]).cpu()  # the one host sync of the layer
        in_splits, out_splits = both[0].tolist(), both[1].tolist()
        n_recv = sum(out_splits)
        # An id outside [0, num_experts) is skipped by the routing pass and leaves the tail of sorted_idx unwritten:
        # refuse before anything indexes with it.
        if sum(in_splits) != flat_ids.numel():
            raise RuntimeError(f"{flat_ids.numel() - sum(in_splits)} expert ids outside [0, {self.num_experts}) reached "
                               "the expert-parallel layer")
        sorted_idx = sorted_idx32.long()
        if on_gpu:  # inverse permutation: position of flat slot (t*k + j) in the sorted order
            pos32 = torch.empty_like(sorted_idx32)
            pos32[sorted_idx] = torch.arange(sorted_idx32.numel(), device=dev, dtype=torch.int32)
        else:
            tok = sorted_idx // k

        rows = _GatherSortedCuda.apply(x, sorted_idx32, pos32, k) if on_gpu else _GatherSorted.apply(x, tok)
        recv = _AllToAllRows.apply(rows, in_splits, out_splits, self.group)
        # received rows are (source rank major, local expert minor): their local expert ids
        local_ids = torch.repeat_interleave(
            torch.arange(epr, device=dev, dtype=torch.int64).repeat(G), recv_counts.reshape(-1), output_size=n_recv)
        y_recv = self.expert_fn(recv, local_ids, w_fc_local, w_proj_local, self.act_kind)
        y_back = _AllToAllRows.apply(y_recv, out_splits, in_splits, self.group)
        if on_gpu:
            return _CombineSortedCuda.apply(y_back, router_weights, sorted_idx32, pos32, k)
        w_sorted = router_weights.reshape(-1).index_select(0, sorted_idx)
        return _CombineSorted.apply(y_back, w_sorted, tok, T)


def balanced_expert_placement(rows_per_expert, world: int) -> list[int]:
    """``expert_to_rank`` for ``world`` ranks with E / world experts each, balancing the rows per rank: experts in order of
    decreasing load go to the least-loaded rank that still has a free slot (longest-processing-time-first).  The load is
    whatever histogram the caller trusts -- a running count of routed rows per expert, typically."""
    loads = [float(v) for v in rows_per_expert]
    E = len(loads)
    if E % world != 0:
        raise ValueError("the number of experts must be divisible by the number of ranks")
    per_rank = E // world
    total = [0.0] * world
    used = [0] * world
    placement = [0] * E
    for e in sorted(range(E), key=lambda i: (-loads[i], i)):
        r = min((r for r in range(world) if used[r] < per_rank), key=lambda r: (total[r], r))
        placement[e] = r
        total[r] += loads[e]
        used[r] += 1
    return placement


def shard_expert_state_dict(full: dict[str, torch.Tensor], rank: int, world: int,
                            expert_to_rank: list[int] | None = None) -> dict[str, torch.Tensor]:
    """Slices ``c_fc.*`` / ``c_proj.*`` of a full MoE state_dict to the experts rank ``rank`` owns (in increasing expert
    id); ``gate.weight`` (the router) is replicated.  Default ownership: contiguous blocks of E / world experts."""
    out = {}
    for key, v in full.items():
        if key.startswith(("c_fc.", "c_proj.")):
            if expert_to_rank is None:
                epr = v.size(0) // world
                out[key] = v[rank * epr : (rank + 1) * epr].clone()
            else:
                mine = [e for e in range(v.size(0)) if expert_to_rank[e] == rank]
                out[key] = v[mine].clone()
        else:
            out[key] = v.clone()
    return out


def gather_expert_state_dict(local: dict[str, torch.Tensor], group=None,
                             expert_to_rank: list[int] | None = None) -> dict[str, torch.Tensor]:
    """Inverse of :func:`shard_expert_state_dict`: all-gathers the expert slices into a full state_dict."""
    world = dist.get_world_size(group)
    out = {}
    for key, v in local.items():
        if key.startswith(("c_fc.", "c_proj.")):
            parts = [torch.empty_like(v) for _ in range(world)]
            dist.all_gather(parts, v.contiguous(), group=group)
            full = torch.cat(parts, dim=0)
            if expert_to_rank is not None:
                order = [e for r in range(world) for e in range(len(expert_to_rank)) if expert_to_rank[e] == r]
                restored = torch.empty_like(full)
                restored[order] = full
                full = restored
            out[key] = full
        else:
            out[key] = v.clone()
    return out
