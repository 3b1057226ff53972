"""MoE_Cute: the MoE expert layer on hand-written sm_100a kernels.

Constructor, ``forward`` contract and ``state_dict`` layout follow the reference's ``MoE_Torch`` /
``MoE_Triton`` (kernels/scattermoe/torch_implementation.py:63-120,
kernels/scattermoe/triton_implementation/__init__.py:39-103); the expert computation replaces
``scattered_experts`` (kernels/scattermoe/triton_implementation/ops.py:143-316):

  forward   route (count + scan + stable scatter) -> gather rows into the 128-row padded layout
            -> up projection with the GLU activation and the router weight fused in the epilogue
            -> down projection with gather-back + top-k combine fused (fp32 red.add) -> cast
  backward  gather grad rows -> dgrad(down) fused with activation backward and the router-weight
            grad -> wgrad(down) -> dgrad(up) fused with the k-way sum -> wgrad(up)

A gated activation that is SwiGLU (``swiglu_packed_*``) or ``torch.nn.GLU`` and no bias takes this
fused path.  Any other activation callable (or ``add_bias=True``) runs the same grouped GEMM kernels
un-fused, with the permutations expressed as torch indexing so autograd differentiates them.
"""

from __future__ import annotations

from typing import Callable

import torch
import torch.nn as nn
import torch.nn.functional as F

from . import _lib
from . import router as _router
from .routing import Routing, route


# ---------------------------------------------------------------------------------------------------
# thin op wrappers: out-parameter style, opaque to torch.compile
# ---------------------------------------------------------------------------------------------------
def _make_op(name: str, impl: Callable, mutates: set[str]) -> Callable:
    op = torch.library.custom_op(f"cute_kernels_b200::{name}", impl, mutates_args=mutates)

    def call(*args):
        return (op if torch.compiler.is_compiling() else impl)(*args)

    call.__name__ = name
    return call


def _gather_rows_impl(src: torch.Tensor, dst: torch.Tensor, row_map: torch.Tensor, padded_off: torch.Tensor,
                      fan_out: int) -> None:
    _lib.require_cuda(src, dst)
    with torch.cuda.device(src.device), _lib.launch("gather_rows", 1, 0.0):
        st = _lib.lib.ck_moe_gather_rows(src.data_ptr(), dst.data_ptr(), row_map.data_ptr(), padded_off.data_ptr(),
                                         padded_off.numel() - 1, dst.size(0), fan_out, src.size(1),
                                         _lib.dtype_code(src.dtype), _lib.stream_ptr())
    _lib.check(st, "ck_moe_gather_rows")


def _cast_from_f32_impl(src: torch.Tensor, dst: torch.Tensor) -> None:
    _lib.require_cuda(src, dst)
    with torch.cuda.device(src.device), _lib.launch("cast_from_f32", 1, 0.0):
        st = _lib.lib.ck_cast_from_f32(src.data_ptr(), dst.data_ptr(), src.numel(), _lib.dtype_code(dst.dtype),
                                       _lib.stream_ptr())
    _lib.check(st, "ck_cast_from_f32")


def _up_act_fwd_impl(xg: torch.Tensor, wfc: torch.Tensor, gate_w: torch.Tensor | None, row_map: torch.Tensor,
                     mtile_off: torch.Tensor, act: torch.Tensor, h: torch.Tensor | None, act_kind: int) -> None:
    _lib.require_cuda(xg, wfc, act)
    status = _lib.status_word(xg.device)
    E, two_i, H = wfc.shape
    with torch.cuda.device(xg.device), _lib.launch("up_act_fwd", 1, 2.0 * xg.size(0) * two_i * H):
        st = _lib.lib.ck_moe_up_act_fwd(xg.data_ptr(), wfc.data_ptr(), _lib.ptr(gate_w), row_map.data_ptr(),
                                        mtile_off.data_ptr(), act.data_ptr(), _lib.ptr(h), E, xg.size(0), H,
                                        two_i // 2, act_kind, _lib.dtype_code(xg.dtype), status.data_ptr(),
                                        _lib.stream_ptr())
    _lib.check(st, "ck_moe_up_act_fwd")


def _up_act_fwd_gather_impl(x: torch.Tensor, top_k: int, wfc: torch.Tensor, gate_w: torch.Tensor | None,
                            row_map: torch.Tensor, mtile_off: torch.Tensor, act: torch.Tensor, h: torch.Tensor | None,
                            act_kind: int) -> None:
    _lib.require_cuda(x, wfc, act)
    status = _lib.status_word(x.device)
    E, two_i, H = wfc.shape
    with torch.cuda.device(x.device), _lib.launch("up_act_fwd", 1, 2.0 * act.size(0) * two_i * H):
        st = _lib.lib.ck_moe_up_act_fwd_gather(x.data_ptr(), x.size(0), top_k, wfc.data_ptr(), _lib.ptr(gate_w),
                                               row_map.data_ptr(), mtile_off.data_ptr(), act.data_ptr(), _lib.ptr(h), E,
                                               act.size(0), H, two_i // 2, act_kind, _lib.dtype_code(x.dtype),
                                               status.data_ptr(), _lib.stream_ptr())
    _lib.check(st, "ck_moe_up_act_fwd_gather")


def _down_combine_fwd_impl(act: torch.Tensor, wproj: torch.Tensor, row_map: torch.Tensor, mtile_off: torch.Tensor,
                           out32: torch.Tensor, top_k: int) -> None:
    _lib.require_cuda(act, wproj, out32)
    status = _lib.status_word(act.device)
    E, H, I = wproj.shape
    with torch.cuda.device(act.device), _lib.launch("down_combine_fwd", 1, 2.0 * act.size(0) * H * I):
        st = _lib.lib.ck_moe_down_combine_fwd(act.data_ptr(), wproj.data_ptr(), row_map.data_ptr(),
                                              mtile_off.data_ptr(), out32.data_ptr(), E, act.size(0), H, I, top_k,
                                              _lib.dtype_code(act.dtype), status.data_ptr(), _lib.stream_ptr())
    _lib.check(st, "ck_moe_down_combine_fwd")


def _dgrad_down_impl(dyg: torch.Tensor, wproj: torch.Tensor, h: torch.Tensor, gate_w: torch.Tensor | None,
                     row_map: torch.Tensor, mtile_off: torch.Tensor, dh: torch.Tensor, dgates: torch.Tensor | None,
                     act_kind: int) -> None:
    _lib.require_cuda(dyg, wproj, h, dh, dgates)
    status = _lib.status_word(dyg.device)
    E, H, I = wproj.shape
    with torch.cuda.device(dyg.device), _lib.launch("dgrad_down", 1, 2.0 * dyg.size(0) * H * I):
        st = _lib.lib.ck_moe_dgrad_down(dyg.data_ptr(), wproj.data_ptr(), h.data_ptr(), _lib.ptr(gate_w),
                                        row_map.data_ptr(), mtile_off.data_ptr(), dh.data_ptr(), _lib.ptr(dgates), E,
                                        dyg.size(0), H, I, act_kind, _lib.dtype_code(dyg.dtype), status.data_ptr(),
                                        _lib.stream_ptr())
    _lib.check(st, "ck_moe_dgrad_down")


def _dgrad_down_gather_impl(dy: torch.Tensor, top_k: int, wproj: torch.Tensor, h: torch.Tensor,
                            gate_w: torch.Tensor | None, row_map: torch.Tensor, mtile_off: torch.Tensor, dh: torch.Tensor,
                            dgates: torch.Tensor | None, act_kind: int) -> None:
    _lib.require_cuda(dy, wproj, h, dh, dgates)
    status = _lib.status_word(dy.device)
    E, H, I = wproj.shape
    with torch.cuda.device(dy.device), _lib.launch("dgrad_down", 1, 2.0 * dh.size(0) * H * I):
        st = _lib.lib.ck_moe_dgrad_down_gather(dy.data_ptr(), dy.size(0), top_k, wproj.data_ptr(), h.data_ptr(),
                                               _lib.ptr(gate_w), row_map.data_ptr(), mtile_off.data_ptr(), dh.data_ptr(),
                                               _lib.ptr(dgates), E, dh.size(0), H, I, act_kind,
                                               _lib.dtype_code(dy.dtype), status.data_ptr(), _lib.stream_ptr())
    _lib.check(st, "ck_moe_dgrad_down_gather")


def _wgrad_gather_impl(a: torch.Tensor, a_fan: int, b: torch.Tensor, b_fan: int, row_map: torch.Tensor,
                       padded_off: torch.Tensor, dw: torch.Tensor) -> None:
    """dW[e] = A_e^T B_e; an operand with fan > 0 is the un-permuted matrix and is gathered by TMA."""
    _lib.require_cuda(a, b, dw)
    status = _lib.status_word(a.device)
    E, M, N = dw.shape
    assert a.size(1) == M and b.size(1) == N
    cap = row_map.numel()
    with torch.cuda.device(a.device), _lib.launch("wgrad", 1, 2.0 * cap * M * N):
        st = _lib.lib.ck_moe_wgrad_gather(a.data_ptr(), a.size(0), a_fan, b.data_ptr(), b.size(0), b_fan,
                                          row_map.data_ptr(), padded_off.data_ptr(), dw.data_ptr(), E, cap, M, N,
                                          _lib.dtype_code(a.dtype), status.data_ptr(), _lib.stream_ptr())
    _lib.check(st, "ck_moe_wgrad_gather")


def _dgrad_up_impl(dh: torch.Tensor, wfc: torch.Tensor, row_map: torch.Tensor, mtile_off: torch.Tensor,
                   dx32: torch.Tensor, top_k: int) -> None:
    _lib.require_cuda(dh, wfc, dx32)
    status = _lib.status_word(dh.device)
    E, i2, H = wfc.shape
    with torch.cuda.device(dh.device), _lib.launch("dgrad_up", 1, 2.0 * dh.size(0) * H * i2):
        st = _lib.lib.ck_moe_dgrad_up(dh.data_ptr(), wfc.data_ptr(), row_map.data_ptr(), mtile_off.data_ptr(),
                                      dx32.data_ptr(), E, dh.size(0), H, i2, top_k, _lib.dtype_code(dh.dtype),
                                      status.data_ptr(), _lib.stream_ptr())
    _lib.check(st, "ck_moe_dgrad_up")


def _wgrad_impl(a: torch.Tensor, b: torch.Tensor, padded_off: torch.Tensor, dw: torch.Tensor) -> None:
    _lib.require_cuda(a, b, dw)
    status = _lib.status_word(a.device)
    E, M, N = dw.shape
    assert a.size(1) == M and b.size(1) == N and a.size(0) == b.size(0)
    with torch.cuda.device(a.device), _lib.launch("wgrad", 1, 2.0 * a.size(0) * M * N):
        st = _lib.lib.ck_moe_wgrad(a.data_ptr(), b.data_ptr(), padded_off.data_ptr(), dw.data_ptr(), E, a.size(0), M, N,
                                   _lib.dtype_code(a.dtype), status.data_ptr(), _lib.stream_ptr())
    _lib.check(st, "ck_moe_wgrad")


def _grouped_linear_impl(x: torch.Tensor, w: torch.Tensor, mtile_off: torch.Tensor, y: torch.Tensor, trans_w: bool) -> None:
    _lib.require_cuda(x, w, y)
    status = _lib.status_word(x.device)
    E = w.size(0)
    N, K = (w.size(2), w.size(1)) if trans_w else (w.size(1), w.size(2))
    assert x.size(1) == K and y.size(1) == N and x.size(0) == y.size(0)
    with torch.cuda.device(x.device), _lib.launch("grouped_linear", 1, 2.0 * x.size(0) * N * K):
        st = _lib.lib.ck_moe_grouped_linear(x.data_ptr(), w.data_ptr(), mtile_off.data_ptr(), y.data_ptr(), E,
                                            x.size(0), N, K, int(trans_w), _lib.dtype_code(x.dtype),
                                            status.data_ptr(), _lib.stream_ptr())
    _lib.check(st, "ck_moe_grouped_linear")


def _grouped_linear_scatter_impl(x: torch.Tensor, w: torch.Tensor, mtile_off: torch.Tensor, row_map: torch.Tensor,
                                 y: torch.Tensor, trans_w: bool) -> None:
    _lib.require_cuda(x, w, y)
    status = _lib.status_word(x.device)
    E = w.size(0)
    N, K = (w.size(2), w.size(1)) if trans_w else (w.size(1), w.size(2))
    assert x.size(1) == K and y.size(1) == N
    with torch.cuda.device(x.device), _lib.launch("grouped_linear_scatter", 1, 2.0 * x.size(0) * N * K):
        st = _lib.lib.ck_moe_grouped_linear_scatter(x.data_ptr(), w.data_ptr(), mtile_off.data_ptr(), row_map.data_ptr(),
                                                    y.data_ptr(), E, x.size(0), N, K, int(trans_w),
                                                    _lib.dtype_code(x.dtype), status.data_ptr(), _lib.stream_ptr())
    _lib.check(st, "ck_moe_grouped_linear_scatter")


def _gather_rows_scaled_impl(src: torch.Tensor, dst: torch.Tensor, idx: torch.Tensor, coeff: torch.Tensor | None,
                             fan_out: int) -> None:
    _lib.require_cuda(src, dst, idx)
    with torch.cuda.device(src.device), _lib.launch("gather_rows_scaled"):
        st = _lib.lib.ck_moe_gather_rows_scaled(src.data_ptr(), dst.data_ptr(), idx.data_ptr(), _lib.ptr(coeff),
                                                dst.size(0), fan_out, src.size(1), _lib.dtype_code(src.dtype),
                                                _lib.stream_ptr())
    _lib.check(st, "ck_moe_gather_rows_scaled")


def _combine_rows_impl(src: torch.Tensor, pos: torch.Tensor | None, w: torch.Tensor | None, out: torch.Tensor, k: int) -> None:
    _lib.require_cuda(src, out)
    with torch.cuda.device(src.device), _lib.launch("combine_rows"):
        st = _lib.lib.ck_moe_combine_rows(src.data_ptr(), _lib.ptr(pos), _lib.ptr(w), out.data_ptr(), out.size(0), k,
                                          src.size(1), _lib.dtype_code(src.dtype), _lib.stream_ptr())
    _lib.check(st, "ck_moe_combine_rows")


def _row_dots_impl(a: torch.Tensor, pos: torch.Tensor, b: torch.Tensor, dots: torch.Tensor, k: int) -> None:
    _lib.require_cuda(a, pos, b, dots)
    with torch.cuda.device(a.device), _lib.launch("row_dots"):
        st = _lib.lib.ck_moe_row_dots(a.data_ptr(), pos.data_ptr(), b.data_ptr(), dots.data_ptr(), dots.numel(), k,
                                      a.size(1), _lib.dtype_code(a.dtype), _lib.stream_ptr())
    _lib.check(st, "ck_moe_row_dots")


gather_rows = _make_op("moe_gather_rows", _gather_rows_impl, {"dst"})
cast_from_f32 = _make_op("cast_from_f32", _cast_from_f32_impl, {"dst"})
up_act_fwd = _make_op("moe_up_act_fwd", _up_act_fwd_impl, {"act", "h"})
up_act_fwd_gather = _make_op("moe_up_act_fwd_gather", _up_act_fwd_gather_impl, {"act", "h"})
down_combine_fwd = _make_op("moe_down_combine_fwd", _down_combine_fwd_impl, {"out32"})
dgrad_down = _make_op("moe_dgrad_down", _dgrad_down_impl, {"dh", "dgates"})
dgrad_down_gather = _make_op("moe_dgrad_down_gather", _dgrad_down_gather_impl, {"dh", "dgates"})
wgrad_gather = _make_op("moe_wgrad_gather", _wgrad_gather_impl, {"dw"})
dgrad_up = _make_op("moe_dgrad_up", _dgrad_up_impl, {"dx32"})
wgrad = _make_op("moe_wgrad", _wgrad_impl, {"dw"})
grouped_linear = _make_op("moe_grouped_linear", _grouped_linear_impl, {"y"})
grouped_linear_scatter = _make_op("moe_grouped_linear_scatter", _grouped_linear_scatter_impl, {"y"})
gather_rows_scaled = _make_op("moe_gather_rows_scaled", _gather_rows_scaled_impl, {"dst"})
combine_rows = _make_op("moe_combine_rows", _combine_rows_impl, {"out"})
row_dots = _make_op("moe_row_dots", _row_dots_impl, {"dots"})


def _from_f32(src32: torch.Tensor, dtype: torch.dtype) -> torch.Tensor:
    if dtype == torch.float32:
        return src32
    out = torch.empty(src32.shape, dtype=dtype, device=src32.device)
    cast_from_f32(src32, out)
    return out


# ---------------------------------------------------------------------------------------------------
# fused expert computation
# ---------------------------------------------------------------------------------------------------
# Route the permutations through TMA gather4 inside the GEMMs (no grouped copies of x / dy) instead of the
# streaming gather kernel.  Measured on B200 (Mixtral-shaped layer, bf16): the gathered operand is fetched 512
# bytes per TMA operation (four 128-byte swizzle rows), and the up projection drops from 1180 to 446 TFLOP/s, wgrad
# from 1220 to 293; the separate gather costs 0.14 ms per use.  So this stays off unless CK_TMA_GATHER=1.
import os as _os

TMA_GATHER = _os.environ.get("CK_TMA_GATHER", "0") == "1"

class _FusedExperts(torch.autograd.Function):
    """y[t] = sum_j w[t, j] * W_proj[e_tj] @ act(W_fc[e_tj] @ x[t]) with saved-for-backward tensors in the
    padded grouped layout.  Mirrors _ScatteredExperts (ops.py:143-292) for c_fc + activation + c_proj at once."""

    @staticmethod
    def forward(ctx, x, router_weights, w_fc, w_proj, row_map, mtile_off, padded_off, top_k: int, act_kind: int):
        T, H = x.shape
        E, two_i, _ = w_fc.shape
        I = two_i // 2
        cap = row_map.numel()
        dev, dt = x.device, x.dtype
        need_grad = any(ctx.needs_input_grad[:4])

        x = x.contiguous()
        gate_w = router_weights.contiguous().view(-1)
        act = torch.empty(cap, I, dtype=dt, device=dev)
        h = torch.empty(cap, two_i, dtype=dt, device=dev) if need_grad else None
        if TMA_GATHER:
            # the up projection gathers the routed token rows itself (TMA gather4); the grouped copy of x is
            # only built in backward, where the weight gradient contracts over it
            xg = None
            up_act_fwd_gather(x, top_k, w_fc, gate_w, row_map, mtile_off, act, h, act_kind)
        else:
            xg = torch.empty(cap, H, dtype=dt, device=dev)
            gather_rows(x, xg, row_map, padded_off, top_k)
            up_act_fwd(xg, w_fc, gate_w, row_map, mtile_off, act, h, act_kind)
        out32 = torch.zeros(T, H, dtype=torch.float32, device=dev)
        down_combine_fwd(act, w_proj, row_map, mtile_off, out32, top_k)
        y = _from_f32(out32, dt)

        if need_grad:
            ctx.save_for_backward(x if xg is None else xg, act, h, gate_w, w_fc, w_proj, row_map, mtile_off, padded_off)
        ctx.x_is_grouped = xg is not None
        ctx.top_k = top_k
        ctx.act_kind = act_kind
        ctx.tokens = T
        return y

    @staticmethod
    def backward(ctx, dy):
        xg, act, h, gate_w, w_fc, w_proj, row_map, mtile_off, padded_off = ctx.saved_tensors
        top_k, act_kind, T = ctx.top_k, ctx.act_kind, ctx.tokens
        E, two_i, H = w_fc.shape
        cap = row_map.numel()
        dev, dt = dy.device, xg.dtype
        need_x, need_rw, need_wfc, need_wproj = ctx.needs_input_grad[:4]

        dy = dy.contiguous().to(dt)
        dh = torch.empty(cap, two_i, dtype=dt, device=dev)
        dgates = torch.zeros(T * top_k, dtype=torch.float32, device=dev)
        d_wproj = d_wfc = dx = d_rw = None
        if not ctx.x_is_grouped:
            # every permutation is done by TMA gather inside the GEMMs: no grouped copies of x or dy exist
            x = xg
            dgrad_down_gather(dy, top_k, w_proj, h, gate_w, row_map, mtile_off, dh, dgates, act_kind)
            if need_wproj:
                d_wproj = torch.empty_like(w_proj)
                wgrad_gather(dy, top_k, act, 0, row_map, padded_off, d_wproj)
            if need_wfc:
                d_wfc = torch.empty_like(w_fc)
                wgrad_gather(dh, 0, x, top_k, row_map, padded_off, d_wfc)
        else:
            dyg = torch.empty(cap, H, dtype=dt, device=dev)
            gather_rows(dy, dyg, row_map, padded_off, top_k)
            dgrad_down(dyg, w_proj, h, gate_w, row_map, mtile_off, dh, dgates, act_kind)
            if need_wproj:
                d_wproj = torch.empty_like(w_proj)
                wgrad(dyg, act, padded_off, d_wproj)
            if need_wfc:
                d_wfc = torch.empty_like(w_fc)
                wgrad(dh, xg, padded_off, d_wfc)
        if need_x:
            dx32 = torch.zeros(T, H, dtype=torch.float32, device=dev)
            dgrad_up(dh, w_fc, row_map, mtile_off, dx32, top_k)
            dx = _from_f32(dx32, dt)
        if need_rw:
            d_rw = dgates.view(T, top_k).to(dt)
        return dx, d_rw, d_wfc, d_wproj, None, None, None, None, None


class _ExpertShard(torch.autograd.Function):
    """Expert computation on rows that already belong to this rank's experts (expert parallelism): every row is
    computed once, un-weighted, and returned in the caller's row order (scatter store, no fp32 staging)."""

    @staticmethod
    def forward(ctx, rows, w_fc, w_proj, row_map, mtile_off, padded_off, act_kind: int):
        n, H = rows.shape
        two_i = w_fc.size(1)
        cap = row_map.numel()
        dev, dt = rows.device, rows.dtype
        need_grad = any(ctx.needs_input_grad[:3])
        rows = rows.contiguous()
        xg = torch.empty(cap, H, dtype=dt, device=dev)
        gather_rows(rows, xg, row_map, padded_off, 1)
        act = torch.empty(cap, two_i // 2, dtype=dt, device=dev)
        h = torch.empty(cap, two_i, dtype=dt, device=dev) if need_grad else None
        up_act_fwd(xg, w_fc, None, row_map, mtile_off, act, h, act_kind)
        y = torch.empty(n, H, dtype=dt, device=dev)
        grouped_linear_scatter(act, w_proj, mtile_off, row_map, y, False)
        if need_grad:
            ctx.save_for_backward(xg, act, h, w_fc, w_proj, row_map, mtile_off, padded_off)
        ctx.act_kind = act_kind
        ctx.rows = n
        return y

    @staticmethod
    def backward(ctx, dy):
        xg, act, h, w_fc, w_proj, row_map, mtile_off, padded_off = ctx.saved_tensors
        E, two_i, H = w_fc.shape
        cap = row_map.numel()
        dev, dt = dy.device, xg.dtype
        dy = dy.contiguous().to(dt)
        dyg = torch.empty(cap, H, dtype=dt, device=dev)
        gather_rows(dy, dyg, row_map, padded_off, 1)
        dh = torch.empty(cap, two_i, dtype=dt, device=dev)
        dgrad_down(dyg, w_proj, h, None, row_map, mtile_off, dh, None, ctx.act_kind)
        d_rows = d_wfc = d_wproj = None
        if ctx.needs_input_grad[2]:
            d_wproj = torch.empty_like(w_proj)
            wgrad(dyg, act, padded_off, d_wproj)
        if ctx.needs_input_grad[0]:
            d_rows = torch.empty(ctx.rows, H, dtype=dt, device=dev)
            grouped_linear_scatter(dh, w_fc, mtile_off, row_map, d_rows, True)
        if ctx.needs_input_grad[1]:
            d_wfc = torch.empty_like(w_fc)
            wgrad(dh, xg, padded_off, d_wfc)
        return d_rows, d_wfc, d_wproj, None, None, None, None


def expert_shard(rows: torch.Tensor, local_expert_ids: torch.Tensor, w_fc: torch.Tensor, w_proj: torch.Tensor,
                 act_kind: int = _lib.CK_ACT_SWIGLU) -> torch.Tensor:
    """y[i] = W_proj[e_i] @ act(W_fc[e_i] @ rows[i]) for rows already dispatched to this rank's experts."""
    r = route(local_expert_ids.reshape(-1), w_fc.size(0))
    return _ExpertShard.apply(rows, w_fc.contiguous(), w_proj.contiguous(), r.row_map, r.mtile_off, r.padded_off, act_kind)


def fused_experts(x: torch.Tensor, router_weights: torch.Tensor, selected_experts: torch.Tensor, w_fc: torch.Tensor,
                  w_proj: torch.Tensor, top_k: int, act_kind: int = _lib.CK_ACT_SWIGLU) -> torch.Tensor:
    """Functional form of the fused expert path: x [T, H], router_weights [T, k] (dtype of x),
    selected_experts [T, k] (int32/int64), w_fc [E, 2I, H] packed [up | gate], w_proj [E, H, I]."""
    E = w_fc.size(0)
    if x.size(0) == 0:
        return torch.zeros_like(x)
    r = route(selected_experts.reshape(-1), E)
    return _FusedExperts.apply(x, router_weights, w_fc.contiguous(), w_proj.contiguous(), r.row_map, r.mtile_off,
                               r.padded_off, top_k, act_kind)


# ---------------------------------------------------------------------------------------------------
# un-fused path for arbitrary activations / bias
# ---------------------------------------------------------------------------------------------------
class _GroupedLinear(torch.autograd.Function):
    """y[p] = x[p] @ W[e(p)]^T on padded rows; rows past the padded total stay zero."""

    @staticmethod
    def forward(ctx, x, w, mtile_off, padded_off):
        x = x.contiguous()
        w = w.contiguous()
        y = torch.zeros(x.size(0), w.size(1), dtype=x.dtype, device=x.device)
        grouped_linear(x, w, mtile_off, y, False)
        ctx.save_for_backward(x, w, mtile_off, padded_off)
        return y

    @staticmethod
    def backward(ctx, dy):
        x, w, mtile_off, padded_off = ctx.saved_tensors
        dy = dy.contiguous()
        dx = dw = None
        if ctx.needs_input_grad[0]:
            dx = torch.zeros_like(x)
            grouped_linear(dy, w, mtile_off, dx, True)
        if ctx.needs_input_grad[1]:
            dw = torch.empty_like(w)
            wgrad(dy, x, padded_off, dw)
        return dx, dw, None, None


def _act_kind_of(activation_function: Callable, is_glu: bool) -> int | None:
    """Which fused epilogue, if any, implements ``activation_function``."""
    if not is_glu:
        return None
    kind = getattr(activation_function, "_ck_act_kind", None)
    if kind is not None:
        return kind
    if getattr(activation_function, "__name__", "") in ("swiglu_packed_cute", "swiglu_packed_torch"):
        return _lib.CK_ACT_SWIGLU
    if isinstance(activation_function, nn.GLU) and activation_function.dim in (-1,):
        return _lib.CK_ACT_GLU
    return None


class Experts_Cute(nn.Module):
    """Parameter container with the reference's layout: weight [E, out, in], optional bias [E, out]
    (kernels/scattermoe/torch_implementation.py:12-60)."""

    def __init__(self, num_experts: int, in_features: int, out_features: int, add_bias: bool = True,
                 std: float | None = None) -> None:
        super().__init__()
        self.weight = nn.Parameter(torch.empty(num_experts, out_features, in_features))
        self.bias = nn.Parameter(torch.empty(num_experts, out_features)) if add_bias else None
        self.std = std
        self.num_experts = num_experts
        self.in_features = in_features
        self.out_features = out_features
        self.reset_parameters()

    def extra_repr(self) -> str:
        return f"num_experts={self.num_experts}, in_features={self.in_features}, out_features={self.out_features}"

    @torch.no_grad()
    def reset_parameters(self) -> None:
        nn.init.normal_(self.weight, mean=0, std=self.std)
        if self.bias is not None:
            self.bias.zero_()

    def forward(self, x: torch.Tensor, r: Routing, row_expert: torch.Tensor | None = None) -> torch.Tensor:
        y = _GroupedLinear.apply(x, self.weight, r.mtile_off, r.padded_off)
        if self.bias is not None:
            y = y + self.bias[row_expert]
        return y


class MoE_Cute(nn.Module):
    def __init__(
        self,
        num_experts: int,
        num_experts_per_tok: int,
        hidden_size: int,
        intermediate_size: int,
        activation_function: Callable,
        is_glu: bool,
        add_bias: bool,
        std: float,
    ) -> None:
        super().__init__()
        self.num_experts = num_experts
        self.top_k = num_experts_per_tok
        self.hidden_size = hidden_size
        self.intermediate_size = intermediate_size
        self.is_glu = is_glu

        self.gate = nn.Linear(in_features=hidden_size, out_features=num_experts, bias=False)
        self.c_fc = Experts_Cute(num_experts, hidden_size, 2 * intermediate_size if is_glu else intermediate_size,
                                 add_bias=add_bias, std=std)
        self.act = activation_function
        self.c_proj = Experts_Cute(num_experts, intermediate_size, hidden_size, add_bias=add_bias, std=std)
        self._act_kind = _act_kind_of(activation_function, is_glu) if not add_bias else None

    def forward(self, hidden_states: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
        original_shape = hidden_states.shape
        hidden_states = hidden_states.view(-1, self.hidden_size)
        router_logits, router_weights, selected_experts = self._compute_routing_weights(hidden_states)
        hidden_states = self._compute_experts(hidden_states, router_weights, selected_experts)
        return hidden_states.view(original_shape), router_logits

    # the gate projection is a library GEMM; top-k + softmax + int32 ids run as one kernel when the router fits
    # it (up to 256 experts), else as the reference's three torch ops
    def _compute_routing_weights(self, hidden_states: torch.Tensor):
        router_logits = self.gate(hidden_states)
        if router_logits.is_cuda and _router.supported(self.num_experts, self.top_k):
            router_weights, selected_experts = _router.router_topk_softmax(router_logits, self.top_k)
            return router_logits, router_weights, selected_experts
        router_weights, selected_experts = self._get_topk(router_logits)
        router_weights = F.softmax(router_weights.float(), dim=-1).type_as(hidden_states)
        return router_logits, router_weights, selected_experts

    def _get_topk(self, x: torch.Tensor):
        if self.top_k == 1:
            return x.max(dim=-1, keepdim=True)
        return x.topk(self.top_k, dim=-1)

    def _compute_experts(self, hidden_states: torch.Tensor, router_weights: torch.Tensor,
                         selected_experts: torch.Tensor) -> torch.Tensor:
        if self._act_kind is not None:
            return fused_experts(hidden_states, router_weights, selected_experts, self.c_fc.weight, self.c_proj.weight,
                                 self.top_k, self._act_kind)
        return self._compute_experts_unfused(hidden_states, router_weights, selected_experts)

    def _compute_experts_unfused(self, x: torch.Tensor, router_weights: torch.Tensor,
                                 selected_experts: torch.Tensor) -> torch.Tensor:
        T, k = x.size(0), self.top_k
        if T == 0:
            return torch.zeros_like(x)
        r = route(selected_experts.reshape(-1), self.num_experts)
        valid = r.row_map >= 0
        src = r.row_map.clamp(min=0).long()
        tok = src // k
        row_expert = None
        if self.c_fc.bias is not None:
            rows = torch.arange(r.capacity, device=x.device, dtype=torch.int32)
            row_expert = torch.searchsorted(r.padded_off[1:].contiguous(), rows, right=True).clamp(max=self.num_experts - 1)
        vmask = valid.unsqueeze(-1).to(x.dtype)
        xg = x[tok] * vmask
        h = self.c_fc(xg, r, row_expert)
        a = self.act(h) * vmask
        y = self.c_proj(a, r, row_expert)
        w = router_weights.reshape(-1)[src] * valid.to(router_weights.dtype)
        out = torch.zeros(T, self.hidden_size, dtype=torch.float32, device=x.device)
        out = out.index_add(0, tok, (y * w.unsqueeze(-1)).float())
        return out.to(x.dtype)
