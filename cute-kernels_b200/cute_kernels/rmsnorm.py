"""rmsnorm_cute / fused_residual_add_rmsnorm_cute (reference: kernels/rmsnorm/__init__.py:12-77,
kernels/fused_residual_add_rmsnorm/__init__.py:15-132): the norm that sits in front of the MoE layer in a
transformer block, as HBM-bound sm_100a kernels (csrc/rmsnorm.cu)."""

from __future__ import annotations

import torch

from . import _lib
from .utils import ensure_contiguous


def _rows_and_hidden(x: torch.Tensor) -> tuple[int, int]:
    H = x.size(-1)
    return (x.numel() // H if H else 0), H


def _fwd_impl(x: torch.Tensor, residual: torch.Tensor | None, weight: torch.Tensor | None, output: torch.Tensor,
              added: torch.Tensor | None, inv_rms: torch.Tensor | None, eps: float, multiplier: float) -> None:
    _lib.require_cuda(x, residual, weight, output)
    rows, H = _rows_and_hidden(x)
    with torch.cuda.device(x.device), _lib.launch("rmsnorm_fwd"):
        st = _lib.lib.ck_rmsnorm_fwd(x.data_ptr(), _lib.ptr(residual), _lib.ptr(weight), output.data_ptr(), _lib.ptr(added),
                                     _lib.ptr(inv_rms), rows, H, eps, multiplier, _lib.dtype_code(x.dtype), _lib.stream_ptr())
    _lib.check(st, "ck_rmsnorm_fwd")


def _bwd_impl(a: torch.Tensor, weight: torch.Tensor | None, output_grad: torch.Tensor, added_grad: torch.Tensor | None,
              inv_rms: torch.Tensor | None, x_grad: torch.Tensor, residual_grad: torch.Tensor | None,
              weight_grad_parts: torch.Tensor | None, weight_grad: torch.Tensor | None, eps: float, multiplier: float) -> None:
    _lib.require_cuda(a, weight, output_grad, x_grad)
    rows, H = _rows_and_hidden(a)
    with torch.cuda.device(a.device), _lib.launch("rmsnorm_bwd", 2 if weight_grad is not None else 1):
        st = _lib.lib.ck_rmsnorm_bwd(a.data_ptr(), _lib.ptr(weight), output_grad.data_ptr(), _lib.ptr(added_grad),
                                     _lib.ptr(inv_rms), x_grad.data_ptr(), _lib.ptr(residual_grad), _lib.ptr(weight_grad_parts),
                                     _lib.ptr(weight_grad), rows, H, eps, multiplier, _lib.dtype_code(a.dtype), _lib.stream_ptr())
    _lib.check(st, "ck_rmsnorm_bwd")


def weight_grad_parts(rows: int, hidden: int) -> int:
    """Rows of the fp32 partial buffer ``[parts, hidden]`` the backward kernel writes its per-block weight-gradient sums
    to (mirror of ck_rmsnorm_bwd_parts, kept out of ctypes so torch.compile can trace callers): the backward launches at
    most 4 blocks per SM."""
    if rows <= 0 or hidden <= 0:
        return 1
    return max(1, min(rows, 4 * _sm_count()))


_SM_COUNT: dict[int, int] = {}


@torch.compiler.assume_constant_result
def _sm_count() -> int:
    dev = torch.cuda.current_device()
    if dev not in _SM_COUNT:
        _SM_COUNT[dev] = torch.cuda.get_device_properties(dev).multi_processor_count
    return _SM_COUNT[dev]


_fwd_op = torch.library.custom_op("cute_kernels_b200::rmsnorm_forward", _fwd_impl, mutates_args={"output", "added", "inv_rms"})
_bwd_op = torch.library.custom_op("cute_kernels_b200::rmsnorm_backward", _bwd_impl,
                                  mutates_args={"x_grad", "residual_grad", "weight_grad_parts", "weight_grad"})


def _fwd(*args) -> None:
    (_fwd_op if _lib.use_custom_op() else _fwd_impl)(*args)


def _bwd(*args) -> None:
    (_bwd_op if _lib.use_custom_op() else _bwd_impl)(*args)


def _check_weight(x: torch.Tensor, weight: torch.Tensor | None) -> None:
    if weight is not None:
        assert weight.dim() == 1, "weight should be 1D"
        assert weight.size(-1) == x.size(-1), "hidden size for x and weight tensor is different"
        assert weight.type() == x.type(), "tensors weight and y should have same dtype"


def _weight_grad_buffers(a: torch.Tensor, weight: torch.Tensor | None):
    """(weight_grad in the weight's dtype, fp32 partial-sum workspace) or (None, None) without a weight."""
    if weight is None:
        return None, None
    rows, H = _rows_and_hidden(a)
    return torch.empty_like(weight), torch.empty(weight_grad_parts(rows, H), H, dtype=torch.float32, device=a.device)


class _RMSNorm_Cute(torch.autograd.Function):
    @staticmethod
    @ensure_contiguous
    def forward(ctx, x: torch.Tensor, weight: torch.Tensor | None, eps: float | None, memory_efficient: bool) -> torch.Tensor:
        _check_weight(x, weight)
        if eps is None:
            eps = torch.finfo(x.dtype).eps
        rows, _ = _rows_and_hidden(x)
        output = torch.empty_like(x)
        inv_rms = None if memory_efficient else torch.empty(rows, device=x.device, dtype=torch.float32)
        _fwd(x, None, weight, output, None, inv_rms, float(eps), 1.0)
        ctx.save_for_backward(x, weight, inv_rms)
        ctx.eps = float(eps)
        return output

    @staticmethod
    @ensure_contiguous
    def backward(ctx, output_grad: torch.Tensor):
        x, weight, inv_rms = ctx.saved_tensors
        x_grad = torch.empty_like(x)
        weight_grad, parts = _weight_grad_buffers(x, weight)
        _bwd(x, weight, output_grad, None, inv_rms, x_grad, None, parts, weight_grad, ctx.eps, 1.0)
        return x_grad, weight_grad, None, None


class _FusedResidualAddRMSNorm_Cute(torch.autograd.Function):
    @staticmethod
    @ensure_contiguous
    def forward(ctx, x: torch.Tensor, residual: torch.Tensor, weight: torch.Tensor | None, eps: float | None,
                multiplier: float | None, memory_efficient: bool):
        _check_weight(x, weight)
        assert residual.size() == x.size() and residual.type() == x.type(), "x and residual should match"
        if eps is None:
            eps = torch.finfo(x.dtype).eps
        rows, _ = _rows_and_hidden(x)
        output = torch.empty_like(x)
        added = torch.empty_like(x)
        inv_rms = None if memory_efficient else torch.empty(rows, device=x.device, dtype=torch.float32)
        mult = 1.0 if multiplier is None else float(multiplier)
        _fwd(x, residual, weight, output, added, inv_rms, float(eps), mult)
        ctx.save_for_backward(added, weight, inv_rms)
        ctx.eps = float(eps)
        ctx.multiplier = mult
        return output, added

    @staticmethod
    @ensure_contiguous
    def backward(ctx, output_grad: torch.Tensor, added_grad: torch.Tensor):
        added, weight, inv_rms = ctx.saved_tensors
        x_grad = torch.empty_like(added)
        residual_grad = torch.empty_like(added)
        weight_grad, parts = _weight_grad_buffers(added, weight)
        _bwd(added, weight, output_grad, added_grad, inv_rms, x_grad, residual_grad, parts, weight_grad, ctx.eps, ctx.multiplier)
        return x_grad, residual_grad, weight_grad, None, None, None


def rmsnorm_cute(x: torch.Tensor, weight: torch.Tensor | None, eps: float | None, memory_efficient: bool = False) -> torch.Tensor:
    """RMSNorm over the last dimension: ``x * rsqrt(mean(x^2) + eps) * weight``.

    ``eps=None`` takes ``torch.finfo(x.dtype).eps``; ``memory_efficient=False`` keeps the per-row 1/rms from the forward
    for the backward instead of recomputing it (same arguments as the reference's ``rmsnorm_cute``)."""
    return _RMSNorm_Cute.apply(x, weight, eps, memory_efficient)


def fused_residual_add_rmsnorm_cute(x: torch.Tensor, residual: torch.Tensor, weight: torch.Tensor | None, eps: float | None,
                                    multiplier: float | None = None, memory_efficient: bool = False):
    """``residual' = x * multiplier + residual`` and ``rmsnorm(residual')`` in one pass; returns ``(normed, residual')``."""
    return _FusedResidualAddRMSNorm_Cute.apply(x, residual, weight, eps, multiplier, memory_efficient)
