"""swiglu_cute / swiglu_packed_cute (reference: kernels/swiglu/__init__.py:77-175)."""

import torch

from . import _lib
from .kernel_backend import CutoTuneParameter, KernelBackend, resolve_backend
from .utils import divide_if_divisible, ensure_contiguous


def _swiglu_forward_impl(gate: torch.Tensor, up: torch.Tensor, output: torch.Tensor, rows: int, cols: int,
                         in_stride: int, out_stride: int) -> None:
    _lib.require_cuda(gate, up, output)
    with torch.cuda.device(gate.device), _lib.launch("swiglu_fwd"):
        st = _lib.lib.ck_swiglu_fwd(gate.data_ptr(), up.data_ptr(), output.data_ptr(), rows, cols, in_stride,
                                    out_stride, _lib.dtype_code(gate.dtype), _lib.stream_ptr())
    _lib.check(st, "ck_swiglu_fwd")


def _swiglu_backward_impl(gate: torch.Tensor, up: torch.Tensor, output_grad: torch.Tensor, gate_grad: torch.Tensor,
                          up_grad: torch.Tensor, rows: int, cols: int, in_stride: int, dy_stride: int,
                          grad_stride: int) -> None:
    _lib.require_cuda(gate, up, output_grad, gate_grad, up_grad)
    with torch.cuda.device(gate.device), _lib.launch("swiglu_bwd"):
        st = _lib.lib.ck_swiglu_bwd(gate.data_ptr(), up.data_ptr(), output_grad.data_ptr(), gate_grad.data_ptr(),
                                    up_grad.data_ptr(), rows, cols, in_stride, dy_stride, grad_stride,
                                    _lib.dtype_code(gate.dtype), _lib.stream_ptr())
    _lib.check(st, "ck_swiglu_bwd")


def _swiglu_packed_forward_impl(x: torch.Tensor, output: torch.Tensor, rows: int, cols: int) -> None:
    # up = x[:, :cols], gate = x[:, cols:]; both are passed as pointers into the one packed buffer
    _lib.require_cuda(x, output)
    esz = x.element_size()
    with torch.cuda.device(x.device), _lib.launch("swiglu_fwd"):
        st = _lib.lib.ck_swiglu_fwd(x.data_ptr() + cols * esz, x.data_ptr(), output.data_ptr(), rows, cols, 2 * cols,
                                    cols, _lib.dtype_code(x.dtype), _lib.stream_ptr())
    _lib.check(st, "ck_swiglu_fwd")


def _swiglu_packed_backward_impl(x: torch.Tensor, output_grad: torch.Tensor, x_grad: torch.Tensor, rows: int,
                                 cols: int) -> None:
    _lib.require_cuda(x, output_grad, x_grad)
    esz = x.element_size()
    with torch.cuda.device(x.device), _lib.launch("swiglu_bwd"):
        st = _lib.lib.ck_swiglu_bwd(x.data_ptr() + cols * esz, x.data_ptr(), output_grad.data_ptr(),
                                    x_grad.data_ptr() + cols * esz, x_grad.data_ptr(), rows, cols, 2 * cols, cols,
                                    2 * cols, _lib.dtype_code(x.dtype), _lib.stream_ptr())
    _lib.check(st, "ck_swiglu_bwd")


_swiglu_forward_op = torch.library.custom_op(
    "cute_kernels_b200::swiglu_forward", _swiglu_forward_impl, mutates_args={"output"}
)
_swiglu_backward_op = torch.library.custom_op(
    "cute_kernels_b200::swiglu_backward", _swiglu_backward_impl, mutates_args={"gate_grad", "up_grad"}
)
_swiglu_packed_forward_op = torch.library.custom_op(
    "cute_kernels_b200::swiglu_packed_forward", _swiglu_packed_forward_impl, mutates_args={"output"}
)
_swiglu_packed_backward_op = torch.library.custom_op(
    "cute_kernels_b200::swiglu_packed_backward", _swiglu_packed_backward_impl, mutates_args={"x_grad"}
)


def _fwd(*args):
    (_swiglu_forward_op if _lib.use_custom_op() else _swiglu_forward_impl)(*args)


def _bwd(*args):
    (_swiglu_backward_op if _lib.use_custom_op() else _swiglu_backward_impl)(*args)


class _Swiglu_Cute(torch.autograd.Function):
    @staticmethod
    @ensure_contiguous
    def forward(ctx, gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
        assert gate.size() == up.size(), "tensors gate and up should have same shape"
        assert gate.type() == up.type(), "tensors gate and up should have same dtype"
        ctx.save_for_backward(gate, up)
        output = torch.empty_like(gate)
        n = gate.numel()
        _fwd(gate, up, output, 1, n, n, n)
        return output

    @staticmethod
    @ensure_contiguous
    def backward(ctx, output_grad: torch.Tensor):
        gate, up = ctx.saved_tensors
        gate_grad = torch.empty_like(gate)
        up_grad = torch.empty_like(up)
        n = gate.numel()
        _bwd(gate, up, output_grad, gate_grad, up_grad, 1, n, n, n, n)
        return gate_grad, up_grad


class _SwigluPacked_Cute(torch.autograd.Function):
    """x = [up | gate] along the last dim (kernels/swiglu/torch_implementation.py:21-23)."""

    @staticmethod
    @ensure_contiguous
    def forward(ctx, x: torch.Tensor) -> torch.Tensor:
        ctx.save_for_backward(x)
        cols = divide_if_divisible(x.size(-1), 2)
        output = torch.empty(*x.size()[:-1], cols, device=x.device, dtype=x.dtype)
        rows = x.numel() // (2 * cols) if cols > 0 else 0
        fn = _swiglu_packed_forward_op if _lib.use_custom_op() else _swiglu_packed_forward_impl
        fn(x, output, rows, cols)
        return output

    @staticmethod
    @ensure_contiguous
    def backward(ctx, output_grad: torch.Tensor):
        x: torch.Tensor = ctx.saved_tensors[0]
        cols = x.size(-1) // 2
        rows = x.numel() // (2 * cols) if cols > 0 else 0
        x_grad = torch.empty_like(x)
        fn = _swiglu_packed_backward_op if _lib.use_custom_op() else _swiglu_packed_backward_impl
        fn(x, output_grad, x_grad, rows, cols)
        return x_grad


def swiglu_cute(
    gate: torch.Tensor,
    up: torch.Tensor,
    *,
    kernel_backend_forward: KernelBackend | CutoTuneParameter = CutoTuneParameter(),
    kernel_backend_backward: KernelBackend | CutoTuneParameter = CutoTuneParameter(),
) -> torch.Tensor:
    """Computes ``up * gate * sigmoid(gate)`` (fp32 math, output in the input dtype).

    ``kernel_backend_*`` are accepted for signature compatibility; only CUDA exists here, asking for
    Triton raises ``ValueError``.
    """
    resolve_backend(kernel_backend_forward)
    resolve_backend(kernel_backend_backward)
    return _Swiglu_Cute.apply(gate, up)


def swiglu_packed_cute(x: torch.Tensor) -> torch.Tensor:
    """SwiGLU of a packed tensor: ``x[..., :I] * silu(x[..., I:])`` with ``I = x.size(-1) // 2``."""
    return _SwigluPacked_Cute.apply(x)
