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

SwiGLU (``swiglu_packed_*``), ``torch.nn.GLU`` and -- un-gated -- ``torch.nn.GELU(approximate="tanh")`` take this
fused path, with or without biases (``add_bias=True``: the biases are added in the GEMM epilogues, their gradients are
column sums over each expert's rows).  Any other activation callable runs the same grouped GEMM kernels un-fused, with
the permutations expressed as torch indexing so autograd differentiates them.
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
        return (op if _lib.use_custom_op() else impl)(*args)

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


def _up_act_fwd_impl(xg: torch.Tensor, wfc: torch.Tensor, b_fc: torch.Tensor | None, gate_w: torch.Tensor | None,
                     row_map: torch.Tensor, mtile_off: torch.Tensor, act: torch.Tensor, h: torch.Tensor | None,
                     act_kind: int) -> None:
    """``wfc`` is [E, 2I, H] for the gated activations and [E, I, H] for CK_ACT_GELU_TANH; ``act`` is [cap, I]."""
    _lib.require_cuda(xg, wfc, act)
    status = _lib.status_word(xg.device)
    E, n_out, H = wfc.shape
    with torch.cuda.device(xg.device), _lib.launch("up_act_fwd", 1, 2.0 * xg.size(0) * n_out * H):
        st = _lib.lib.ck_moe_up_act_fwd(xg.data_ptr(), wfc.data_ptr(), _lib.ptr(b_fc), _lib.ptr(gate_w), row_map.data_ptr(),
                                        mtile_off.data_ptr(), act.data_ptr(), _lib.ptr(h), E, xg.size(0), H,
                                        act.size(1), act_kind, _lib.dtype_code(xg.dtype), status.data_ptr(),
                                        _lib.stream_ptr())
    _lib.check(st, "ck_moe_up_act_fwd")


def _up_act_fwd_gather_impl(x: torch.Tensor, top_k: int, wfc: torch.Tensor, b_fc: torch.Tensor | None,
                            gate_w: torch.Tensor | None, row_map: torch.Tensor, mtile_off: torch.Tensor, act: torch.Tensor,
                            h: torch.Tensor | None, xg_out: torch.Tensor | None, act_kind: int) -> None:
    """Up projection reading the routed rows of ``x`` by row index inside the GEMM; ``xg_out`` [cap, H] (optional)
    receives the grouped copy of those rows as a by-product."""
    _lib.require_cuda(x, wfc, act)
    status = _lib.status_word(x.device)
    E, n_out, H = wfc.shape
    with torch.cuda.device(x.device), _lib.launch("up_act_fwd", 1, 2.0 * act.size(0) * n_out * H):
        st = _lib.lib.ck_moe_up_act_fwd_gather(x.data_ptr(), x.size(0), top_k, wfc.data_ptr(), _lib.ptr(b_fc), _lib.ptr(gate_w),
                                               row_map.data_ptr(), mtile_off.data_ptr(), act.data_ptr(), _lib.ptr(h),
                                               _lib.ptr(xg_out), E, act.size(0), H, act.size(1), act_kind,
                                               _lib.dtype_code(x.dtype), status.data_ptr(), _lib.stream_ptr())
    _lib.check(st, "ck_moe_up_act_fwd_gather")


def _down_combine_fwd_impl(act: torch.Tensor, wproj: torch.Tensor, b_proj: torch.Tensor | None, gate_w: torch.Tensor | None,
                           row_map: torch.Tensor, mtile_off: torch.Tensor, out32: torch.Tensor, top_k: int) -> None:
    _lib.require_cuda(act, wproj, out32)
    status = _lib.status_word(act.device)
    E, H, I = wproj.shape
    with torch.cuda.device(act.device), _lib.launch("down_combine_fwd", 1, 2.0 * act.size(0) * H * I):
        st = _lib.lib.ck_moe_down_combine_fwd(act.data_ptr(), wproj.data_ptr(), _lib.ptr(b_proj), _lib.ptr(gate_w),
                                              row_map.data_ptr(), mtile_off.data_ptr(), out32.data_ptr(), E, act.size(0), H,
                                              I, top_k, _lib.dtype_code(act.dtype), status.data_ptr(), _lib.stream_ptr())
    _lib.check(st, "ck_moe_down_combine_fwd")


def _dgrad_down_impl(dyg: torch.Tensor, wproj: torch.Tensor, h: torch.Tensor, gate_w: torch.Tensor | None,
                     row_map: torch.Tensor, mtile_off: torch.Tensor, dh: torch.Tensor, dgates: torch.Tensor | None,
                     dgates_part: torch.Tensor | None, act_kind: int) -> None:
    _lib.require_cuda(dyg, wproj, h, dh, dgates, dgates_part)
    status = _lib.status_word(dyg.device)
    E, H, I = wproj.shape
    with torch.cuda.device(dyg.device), _lib.launch("dgrad_down", 1, 2.0 * dyg.size(0) * H * I):
        st = _lib.lib.ck_moe_dgrad_down(dyg.data_ptr(), wproj.data_ptr(), h.data_ptr(), _lib.ptr(gate_w),
                                        row_map.data_ptr(), mtile_off.data_ptr(), dh.data_ptr(), _lib.ptr(dgates),
                                        _lib.ptr(dgates_part), E, dyg.size(0), H, I, act_kind,
                                        _lib.dtype_code(dyg.dtype), status.data_ptr(), _lib.stream_ptr())
    _lib.check(st, "ck_moe_dgrad_down")


def _dgrad_down_gather_impl(dy: torch.Tensor, top_k: int, wproj: torch.Tensor, h: torch.Tensor,
                            gate_w: torch.Tensor | None, row_map: torch.Tensor, mtile_off: torch.Tensor, dh: torch.Tensor,
                            dgates: torch.Tensor | None, dgates_part: torch.Tensor | None, dyg_out: torch.Tensor | None,
                            act_kind: int) -> None:
    _lib.require_cuda(dy, wproj, h, dh, dgates, dgates_part)
    status = _lib.status_word(dy.device)
    E, H, I = wproj.shape
    with torch.cuda.device(dy.device), _lib.launch("dgrad_down", 1, 2.0 * dh.size(0) * H * I):
        st = _lib.lib.ck_moe_dgrad_down_gather(dy.data_ptr(), dy.size(0), top_k, wproj.data_ptr(), h.data_ptr(),
                                               _lib.ptr(gate_w), row_map.data_ptr(), mtile_off.data_ptr(), dh.data_ptr(),
                                               _lib.ptr(dgates), _lib.ptr(dgates_part), _lib.ptr(dyg_out), E, dh.size(0), H,
                                               I, act_kind, _lib.dtype_code(dy.dtype), status.data_ptr(),
                                               _lib.stream_ptr())
    _lib.check(st, "ck_moe_dgrad_down_gather")


def _reduce_dgates_impl(dgates_part: torch.Tensor, row_map: torch.Tensor, padded_off: torch.Tensor, num_experts: int,
                        dgates: torch.Tensor) -> None:
    """dgates[row_map[p]] = sum of the parts of padded row p, added in part order (reproducible), for the padded rows
    of the first ``num_experts`` experts (those the GEMM ran over)."""
    _lib.require_cuda(dgates_part, row_map, dgates)
    with torch.cuda.device(dgates.device), _lib.launch("reduce_dgates"):
        st = _lib.lib.ck_moe_reduce_dgates(dgates_part.data_ptr(), dgates_part.size(0), dgates_part.size(1),
                                           row_map.data_ptr(), padded_off.data_ptr(), num_experts,
                                           dgates.data_ptr(), _lib.stream_ptr())
    _lib.check(st, "ck_moe_reduce_dgates")


@torch.compiler.assume_constant_result
def cta_pair_kernels() -> bool:
    """True when the grouped GEMMs run as CTA pairs (the default), False for the single-CTA flavour.  A process-level
    setting: under torch.compile its value at trace time is baked into the graph."""
    return bool(_lib.lib.ck_gemm_cta_pair())


def dgates_parts(intermediate_size: int) -> int:
    """Rows of the partial router-weight-grad buffer ``[parts, cap]`` that dgrad_down fills
    (ck_moe_dgrad_down_parts: one part per 256-column n-tile, two with the CTA-pair kernels' two epilogue groups)."""
    n_tiles = (intermediate_size + 255) // 256
    return 2 * n_tiles if cta_pair_kernels() else n_tiles


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


def _grouped_linear_scatter_impl(x: torch.Tensor, w: torch.Tensor, bias: torch.Tensor | None, gate_w: torch.Tensor | None,
                                 mtile_off: torch.Tensor, row_map: torch.Tensor, y: torch.Tensor, trans_w: bool) -> None:
    _lib.require_cuda(x, w, y)
    status = _lib.status_word(x.device)
    E = w.size(0)
    N, K = (w.size(2), w.size(1)) if trans_w else (w.size(1), w.size(2))
    assert x.size(1) == K and y.size(1) == N
    with torch.cuda.device(x.device), _lib.launch("grouped_linear_scatter", 1, 2.0 * x.size(0) * N * K):
        st = _lib.lib.ck_moe_grouped_linear_scatter(x.data_ptr(), w.data_ptr(), _lib.ptr(bias), _lib.ptr(gate_w),
                                                    mtile_off.data_ptr(), row_map.data_ptr(), y.data_ptr(), E, x.size(0), N, K,
                                                    int(trans_w), _lib.dtype_code(x.dtype), status.data_ptr(),
                                                    _lib.stream_ptr())
    _lib.check(st, "ck_moe_grouped_linear_scatter")


def _bias_grad_impl(rows: torch.Tensor, row_map: torch.Tensor | None, gate_w: torch.Tensor | None, padded_off: torch.Tensor,
                    out: torch.Tensor) -> None:
    """out[e, :] = sum over expert e's padded rows of (gate_w[row_map[p]] or 1) * rows[p, :]."""
    _lib.require_cuda(rows, padded_off, out)
    with torch.cuda.device(rows.device), _lib.launch("bias_grad"):
        st = _lib.lib.ck_moe_bias_grad(rows.data_ptr(), rows.size(0), rows.size(1), _lib.ptr(row_map), _lib.ptr(gate_w),
                                       padded_off.data_ptr(), out.size(0), out.data_ptr(), _lib.dtype_code(rows.dtype),
                                       _lib.stream_ptr())
    _lib.check(st, "ck_moe_bias_grad")


def _bias_dots_impl(rows: torch.Tensor, bias: torch.Tensor, padded_off: torch.Tensor, part: torch.Tensor) -> None:
    """part[p] = rows[p, :] . bias[expert of p, :] (fp32, one more part of the router-weight-grad buffer)."""
    _lib.require_cuda(rows, bias, padded_off, part)
    with torch.cuda.device(rows.device), _lib.launch("bias_dots"):
        st = _lib.lib.ck_moe_bias_dots(rows.data_ptr(), rows.size(0), rows.size(1), bias.data_ptr(), padded_off.data_ptr(),
                                       bias.size(0), part.data_ptr(), _lib.dtype_code(rows.dtype), _lib.stream_ptr())
    _lib.check(st, "ck_moe_bias_dots")


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
up_act_fwd_gather = _make_op("moe_up_act_fwd_gather", _up_act_fwd_gather_impl, {"act", "h", "xg_out"})
down_combine_fwd = _make_op("moe_down_combine_fwd", _down_combine_fwd_impl, {"out32"})
dgrad_down = _make_op("moe_dgrad_down", _dgrad_down_impl, {"dh", "dgates", "dgates_part"})
dgrad_down_gather = _make_op("moe_dgrad_down_gather", _dgrad_down_gather_impl, {"dh", "dgates", "dgates_part", "dyg_out"})
reduce_dgates = _make_op("moe_reduce_dgates", _reduce_dgates_impl, {"dgates"})
wgrad_gather = _make_op("moe_wgrad_gather", _wgrad_gather_impl, {"dw"})
dgrad_up = _make_op("moe_dgrad_up", _dgrad_up_impl, {"dx32"})
wgrad = _make_op("moe_wgrad", _wgrad_impl, {"dw"})
grouped_linear = _make_op("moe_grouped_linear", _grouped_linear_impl, {"y"})
grouped_linear_scatter = _make_op("moe_grouped_linear_scatter", _grouped_linear_scatter_impl, {"y"})
bias_grad = _make_op("moe_bias_grad", _bias_grad_impl, {"out"})
bias_dots = _make_op("moe_bias_dots", _bias_dots_impl, {"part"})
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
# How the routed rows of x (forward) and of grad_out (backward) reach the GEMMs.
#   "kernel"   (default) a streaming gather kernel builds the grouped copies first; the GEMMs read them with tiled TMA loads.
#   "producer" the up projection and dgrad-down read the rows by row index with their own producer warp (cp.async into
#              the swizzled stages, CTA-pair kernels only) and write the grouped copy out as a by-product for the
#              weight-gradient GEMMs; no separate permutation kernel runs.
#   "tma"      no grouped copies at all: the weight-gradient GEMMs gather their operand with TMA gather4 as well.
# Measured on B200 (Mixtral-shaped layer, bf16, up projection): "kernel" 0.09 ms gather + 5.4 ms GEMM; "producer" 28.7 ms
# (16-byte cp.async delivers about 7 GB/s per SM, a sixth of what the tensor cores consume, whether one warp or two issue
# it, with or without the proxy fence, with a CTA- or cluster-scope acquire); "tma" 17.7 ms (gather4 moves 512 bytes per
# TMA operation).  Every A tile is fetched once per n-tile, 56-112 times in all, so the per-byte cost of the fetch path
# matters far more than the one extra pass of the gather kernel.  The alternatives stay selectable (CK_GATHER_MODE,
# CK_TMA_GATHER=1) and tested.
import os as _os

TMA_GATHER = _os.environ.get("CK_TMA_GATHER", "0") == "1"
GATHER_MODE = _os.environ.get("CK_GATHER_MODE", "")


def _gather_mode() -> str:
    if TMA_GATHER:
        return "tma"
    if GATHER_MODE in ("kernel", "tma"):
        return GATHER_MODE
    if GATHER_MODE == "producer":
        return "producer" if cta_pair_kernels() else "kernel"
    return "kernel"


class _FusedExperts(torch.autograd.Function):
    """y[t] = sum_j w[t, j] * (W_proj[e_tj] @ act(W_fc[e_tj] @ x[t] + b_fc[e_tj]) + b_proj[e_tj]) with saved-for-backward
    tensors in the padded grouped layout.  Mirrors _ScatteredExperts (ops.py:143-292) for c_fc + activation + c_proj at
    once, with the biases of Experts_Torch (torch_implementation.py:41-44) folded into the GEMM epilogues.

    ``act_kind``: CK_ACT_SWIGLU / CK_ACT_GLU (w_fc [E, 2I, H], packed [up | gate]) or CK_ACT_GELU_TANH (w_fc [E, I, H]).
    ``deterministic``: the k rows of every token are stored un-combined ([T*k, H], each written once) and summed in a
    fixed order by a second kernel, instead of fp32 ``red.add`` into one [T, H] buffer from the GEMM epilogue (whose
    order of additions varies from run to run when k > 2)."""

    @staticmethod
    def forward(ctx, x, router_weights, w_fc, w_proj, b_fc, b_proj, row_map, mtile_off, padded_off, top_k: int,
                act_kind: int, deterministic: bool = False):
        T, H = x.shape
        E, n_fc, _ = w_fc.shape
        I = w_proj.size(2)
        cap = row_map.numel()
        dev, dt = x.device, x.dtype
        need_grad = any(ctx.needs_input_grad[:6])
        need_xg = ctx.needs_input_grad[2]  # the weight gradient of the up projection contracts over the grouped rows
        mode = _gather_mode()

        x = x.contiguous()
        gate_w = router_weights.contiguous().view(-1)
        act = torch.empty(cap, I, dtype=dt, device=dev)
        h = torch.empty(cap, n_fc, dtype=dt, device=dev) if need_grad else None
        xg = None
        if mode == "kernel":
            xg = torch.empty(cap, H, dtype=dt, device=dev)
            gather_rows(x, xg, row_map, padded_off, top_k)
            up_act_fwd(xg, w_fc, b_fc, gate_w, row_map, mtile_off, act, h, act_kind)
        else:
            if mode == "producer" and need_xg:
                xg = torch.empty(cap, H, dtype=dt, device=dev)
            up_act_fwd_gather(x, top_k, w_fc, b_fc, gate_w, row_map, mtile_off, act, h, xg, act_kind)
        if deterministic:
            rows = torch.empty(T * top_k, H, dtype=dt, device=dev)
            grouped_linear_scatter(act, w_proj, b_proj, gate_w if b_proj is not None else None, mtile_off, row_map, rows, False)
            y = torch.empty(T, H, dtype=dt, device=dev)
            combine_rows(rows, None, None, y, top_k)
        else:
            out32 = torch.zeros(T, H, dtype=torch.float32, device=dev)
            down_combine_fwd(act, w_proj, b_proj, gate_w if b_proj is not None else None, row_map, mtile_off, out32, top_k)
            y = _from_f32(out32, dt)

        if need_grad:
            ctx.save_for_backward(x, xg, act, h, gate_w, w_fc, w_proj, b_proj, row_map, mtile_off, padded_off)
        ctx.mode = mode
        ctx.top_k = top_k
        ctx.act_kind = act_kind
        ctx.deterministic = deterministic
        ctx.has_b_fc = b_fc is not None
        return y

    @staticmethod
    def backward(ctx, dy):
        x, xg, act, h, gate_w, w_fc, w_proj, b_proj, row_map, mtile_off, padded_off = ctx.saved_tensors
        top_k, act_kind, mode = ctx.top_k, ctx.act_kind, ctx.mode
        T = x.size(0)
        E, n_fc, H = w_fc.shape
        I = w_proj.size(2)
        cap = row_map.numel()
        dev, dt = dy.device, x.dtype
        need_x, need_rw, need_wfc, need_wproj, need_bfc, need_bproj = ctx.needs_input_grad[:6]
        need_bfc = need_bfc and ctx.has_b_fc
        need_bproj = need_bproj and b_proj is not None

        dy = dy.contiguous().to(dt)
        dh = torch.empty(cap, n_fc, dtype=dt, device=dev)
        # router-weight grads: per-(n-tile, epilogue group) partial sums (+ one part for the bias term), added in a fixed
        # order afterwards
        parts = dgates_parts(I)
        dg_part = torch.empty(parts + (1 if b_proj is not None else 0), cap, dtype=torch.float32, device=dev) if need_rw else None
        d_wproj = d_wfc = dx = d_rw = d_bfc = d_bproj = None
        dyg = None
        need_dyg = need_wproj or need_bproj or (need_rw and b_proj is not None)
        if mode == "kernel":
            dyg = torch.empty(cap, H, dtype=dt, device=dev)
            gather_rows(dy, dyg, row_map, padded_off, top_k)
            dgrad_down(dyg, w_proj, h, gate_w, row_map, mtile_off, dh, None, dg_part, act_kind)
        else:
            if mode == "producer" and need_dyg:
                dyg = torch.empty(cap, H, dtype=dt, device=dev)
            dgrad_down_gather(dy, top_k, w_proj, h, gate_w, row_map, mtile_off, dh, None, dg_part, dyg, act_kind)
        if dyg is None and (need_bproj or (need_rw and b_proj is not None)):
            dyg = torch.empty(cap, H, dtype=dt, device=dev)  # "tma" mode with a bias: the bias kernels read grouped rows
            gather_rows(dy, dyg, row_map, padded_off, top_k)
        if need_wproj:
            d_wproj = torch.empty_like(w_proj)
            if dyg is not None:
                wgrad(dyg, act, padded_off, d_wproj)
            else:
                wgrad_gather(dy, top_k, act, 0, row_map, padded_off, d_wproj)
        if need_wfc:
            d_wfc = torch.empty_like(w_fc)
            if xg is not None:
                wgrad(dh, xg, padded_off, d_wfc)
            else:
                wgrad_gather(dh, 0, x, top_k, row_map, padded_off, d_wfc)
        if need_bfc:
            d_bfc = torch.empty(E, n_fc, dtype=dt, device=dev)
            bias_grad(dh, None, None, padded_off, d_bfc)
        if need_bproj:
            d_bproj = torch.empty(E, H, dtype=dt, device=dev)
            bias_grad(dyg, row_map, gate_w, padded_off, d_bproj)
        if need_x:
            if ctx.deterministic:
                rows = torch.empty(T * top_k, H, dtype=dt, device=dev)
                grouped_linear_scatter(dh, w_fc, None, None, mtile_off, row_map, rows, True)
                dx = torch.empty(T, H, dtype=dt, device=dev)
                combine_rows(rows, None, None, dx, top_k)
            else:
                dx32 = torch.zeros(T, H, dtype=torch.float32, device=dev)
                dgrad_up(dh, w_fc, row_map, mtile_off, dx32, top_k)
                dx = _from_f32(dx32, dt)
        if need_rw:
            if b_proj is not None:
                bias_dots(dyg, b_proj, padded_off, dg_part[parts])
            dgates = torch.zeros(T * top_k, dtype=torch.float32, device=dev)
            reduce_dgates(dg_part, row_map, padded_off, E, dgates)
            d_rw = dgates.view(T, top_k).to(dt)
        return dx, d_rw, d_wfc, d_wproj, d_bfc, d_bproj, None, None, None, None, None, None


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
        act = torch.empty(cap, two_i // 2, dtype=dt, device=dev)
        h = torch.empty(cap, two_i, dtype=dt, device=dev) if need_grad else None
        producer = _gather_mode() == "producer" and n > 0
        xg = torch.empty(cap, H, dtype=dt, device=dev) if (need_grad or not producer) else None
        if producer:
            up_act_fwd_gather(rows, 1, w_fc, None, None, row_map, mtile_off, act, h, xg, act_kind)
        else:
            gather_rows(rows, xg, row_map, padded_off, 1)
            up_act_fwd(xg, w_fc, None, None, row_map, mtile_off, act, h, act_kind)
        y = torch.empty(n, H, dtype=dt, device=dev)
        grouped_linear_scatter(act, w_proj, None, None, mtile_off, row_map, y, False)
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
        dh = torch.empty(cap, two_i, dtype=dt, device=dev)
        if _gather_mode() == "producer" and ctx.rows > 0:
            dgrad_down_gather(dy, 1, w_proj, h, None, row_map, mtile_off, dh, None, None, dyg, ctx.act_kind)
        else:
            gather_rows(dy, dyg, row_map, padded_off, 1)
            dgrad_down(dyg, w_proj, h, None, row_map, mtile_off, dh, None, None, ctx.act_kind)
        d_rows = d_wfc = d_wproj = None
        if ctx.needs_input_grad[2]:
            d_wproj = torch.empty_like(w_proj)
            wgrad(dyg, act, padded_off, d_wproj)
        if ctx.needs_input_grad[0]:
            d_rows = torch.empty(ctx.rows, H, dtype=dt, device=dev)
            grouped_linear_scatter(dh, w_fc, None, None, mtile_off, row_map, d_rows, True)
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
                  w_proj: torch.Tensor, top_k: int, act_kind: int = _lib.CK_ACT_SWIGLU, deterministic: bool | None = None,
                  b_fc: torch.Tensor | None = None, b_proj: torch.Tensor | None = None) -> torch.Tensor:
    """Functional form of the fused expert path: x [T, H], router_weights [T, k] (dtype of x),
    selected_experts [T, k] (int32/int64), w_fc [E, 2I, H] packed [up | gate] (or [E, I, H] with
    ``act_kind=CK_ACT_GELU_TANH``), w_proj [E, H, I], optional biases b_fc [E, 2I or I] and b_proj [E, H].

    ``deterministic``: how the k expert outputs of a token (and the k input-gradient rows) are summed.  False: fp32
    ``red.add`` into one [T, H] buffer from the GEMM epilogue (bit-reproducible for k <= 2, where two addends commute; for
    k > 2 the order varies from run to run).  True: every row is stored once ([T*k, H]) and a second kernel sums the k rows
    in slot order (always reproducible).  None (default): True for k > 2, where it is also the faster form (measured on
    the 64-expert top-8 layer: 13.7 against 14.4 ms per step -- k fp32 reductions per element load L2 more than k 16-bit
    stores and one pass over them), False for k <= 2 (28.8 against 29.0 ms on the top-2 layer).
    Router-weight and bias gradients are always summed in a fixed order."""
    E = w_fc.size(0)
    if x.size(0) == 0:
        return torch.zeros_like(x)
    if deterministic is None:
        deterministic = top_k > 2
    r = route(selected_experts.reshape(-1), E)
    return _FusedExperts.apply(x, router_weights, w_fc.contiguous(), w_proj.contiguous(),
                               None if b_fc is None else b_fc.contiguous(), None if b_proj is None else b_proj.contiguous(),
                               r.row_map, r.mtile_off, r.padded_off, top_k, act_kind, deterministic)


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
    kind = getattr(activation_function, "_ck_act_kind", None)
    if kind is not None:
        return kind
    if is_glu:
        if getattr(activation_function, "__name__", "") in ("swiglu_packed_cute", "swiglu_packed_torch"):
            return _lib.CK_ACT_SWIGLU
        if isinstance(activation_function, nn.GLU) and activation_function.dim in (-1,):
            return _lib.CK_ACT_GLU
        return None
    if isinstance(activation_function, nn.GELU) and activation_function.approximate == "tanh":
        return _lib.CK_ACT_GELU_TANH
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
        *,
        check_status: bool = False,
        deterministic: bool | None = None,
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
        self._act_kind = _act_kind_of(activation_function, is_glu)
        # True: every forward ends with one read of the device status word (a stream synchronisation) and raises when
        # a kernel of the step flagged an out-of-range expert id, a bounded wait that ran out or inconsistent tile
        # tables.  False (default): no synchronisation; poll cute_kernels.check_device_status() when convenient.
        self.check_status = check_status
        # how the k expert outputs of a token are summed (see fused_experts): None = in a fixed order for k > 2
        self.deterministic = deterministic
        # False: keep the gate projection a library GEMM (its logits then match F.linear bit for bit)
        self.fuse_router = True

    def forward(self, hidden_states: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
        original_shape = hidden_states.shape
        hidden_states = hidden_states.view(-1, self.hidden_size)
        router_logits, router_weights, selected_experts = self._compute_routing_weights(hidden_states)
        hidden_states = self._compute_experts(hidden_states, router_weights, selected_experts)
        if self.check_status and hidden_states.is_cuda and not torch.compiler.is_compiling():
            _lib.check_device_status(hidden_states.device)
        return hidden_states.view(original_shape), router_logits

    # 16-bit tensors, up to 256 experts, k <= 8: the gate projection runs on the tensor cores with top-k + softmax + int32
    # ids in its epilogue (one launch).  Otherwise the gate projection is a library GEMM and top-k + softmax + ids run as
    # one kernel when the router fits it, else as the reference's three torch ops.
    def _compute_routing_weights(self, hidden_states: torch.Tensor):
        if self.fuse_router and _router.fused_gate_supported(hidden_states, self.gate.weight, self.top_k):
            return _router.router_gate_topk_softmax(hidden_states, self.gate.weight, self.top_k)
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
                                 self.top_k, self._act_kind, self.deterministic, self.c_fc.bias, self.c_proj.bias)
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
