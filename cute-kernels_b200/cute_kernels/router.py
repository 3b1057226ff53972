"""Router tail on one kernel: top-k of the gate logits, softmax over the selected k, int32 expert ids.

The reference runs ``topk`` (``max`` when k == 1), ``softmax(.float())`` and ``type_as`` as separate torch ops
and hands an int64 ``selected_experts`` to the expert path
(kernels/scattermoe/torch_implementation.py:122-135,195-201).  ``router_topk_softmax`` computes the same
``(router_weights, selected_experts)`` pair in one launch and keeps the ids int32, the form the routing kernels
read.  ``router_gate_topk_softmax`` goes one step further and runs the gate projection itself on the tensor cores with
this tail in the GEMM epilogue (16-bit dtypes, up to 256 experts, k <= 8).  Differentiable in the logits: the
backward kernel scatters the softmax gradient of the k selected logits into a zero ``[T, E]`` tensor, which is
what autograd derives for the three torch ops.
"""

from __future__ import annotations

import torch

from . import _lib

MAX_EXPERTS = 256
MAX_TOP_K = 32


def _fwd_impl(logits: torch.Tensor, weights: torch.Tensor, ids: torch.Tensor, top_k: int) -> None:
    _lib.require_cuda(logits, weights, ids)
    with torch.cuda.device(logits.device), _lib.launch("router_topk_softmax"):
        st = _lib.lib.ck_router_topk_softmax(logits.data_ptr(), weights.data_ptr(), ids.data_ptr(), logits.size(0),
                                             logits.size(1), top_k, _lib.dtype_code(logits.dtype), _lib.stream_ptr())
    _lib.check(st, "ck_router_topk_softmax")


def _bwd_impl(weights: torch.Tensor, d_weights: torch.Tensor, ids: torch.Tensor, d_logits: torch.Tensor) -> None:
    _lib.require_cuda(weights, d_weights, ids, d_logits)
    status = _lib.status_word(weights.device)
    with torch.cuda.device(weights.device), _lib.launch("router_topk_softmax_bwd"):
        st = _lib.lib.ck_router_topk_softmax_bwd(weights.data_ptr(), d_weights.data_ptr(), ids.data_ptr(),
                                                 d_logits.data_ptr(), weights.size(0), d_logits.size(1),
                                                 weights.size(1), _lib.dtype_code(weights.dtype), status.data_ptr(),
                                                 _lib.stream_ptr())
    _lib.check(st, "ck_router_topk_softmax_bwd")


_fwd_op = torch.library.custom_op("cute_kernels_b200::router_topk_softmax", _fwd_impl, mutates_args={"weights", "ids"})
_bwd_op = torch.library.custom_op("cute_kernels_b200::router_topk_softmax_bwd", _bwd_impl, mutates_args={"d_logits"})


def _call(op, impl, *args):
    return (op if _lib.use_custom_op() else impl)(*args)


class _RouterTopkSoftmax(torch.autograd.Function):
    @staticmethod
    def forward(ctx, logits: torch.Tensor, top_k: int):
        logits = logits.contiguous()
        T, E = logits.shape
        weights = torch.empty(T, top_k, dtype=logits.dtype, device=logits.device)
        ids = torch.empty(T, top_k, dtype=torch.int32, device=logits.device)
        if T:
            _call(_fwd_op, _fwd_impl, logits, weights, ids, top_k)
        ctx.save_for_backward(weights, ids)
        ctx.num_experts = E
        ctx.mark_non_differentiable(ids)
        return weights, ids

    @staticmethod
    def backward(ctx, d_weights, _d_ids):
        weights, ids = ctx.saved_tensors
        d_logits = torch.empty(weights.size(0), ctx.num_experts, dtype=weights.dtype, device=weights.device)
        if weights.size(0):
            _call(_bwd_op, _bwd_impl, weights, d_weights.contiguous(), ids, d_logits)
        return d_logits, None


# ---- gate projection + router tail in one tensor-core launch ---------------------------------------------
FUSED_MAX_TOP_K = 8


def _gate_fwd_impl(x: torch.Tensor, gate_w: torch.Tensor, logits: torch.Tensor, weights: torch.Tensor, ids: torch.Tensor,
                   top_k: int) -> None:
    _lib.require_cuda(x, gate_w, logits, weights, ids)
    status = _lib.status_word(x.device)
    T, H = x.shape
    E = gate_w.size(0)
    with torch.cuda.device(x.device), _lib.launch("router_gate_topk_softmax", 1, 2.0 * T * H * E):
        st = _lib.lib.ck_router_gate_topk_softmax(x.data_ptr(), gate_w.data_ptr(), logits.data_ptr(), weights.data_ptr(),
                                                  ids.data_ptr(), T, H, E, top_k, _lib.dtype_code(x.dtype), status.data_ptr(),
                                                  _lib.stream_ptr())
    _lib.check(st, "ck_router_gate_topk_softmax")


_gate_fwd_op = torch.library.custom_op("cute_kernels_b200::router_gate_topk_softmax", _gate_fwd_impl,
                                       mutates_args={"logits", "weights", "ids"})


class _GateRouter(torch.autograd.Function):
    """(logits, weights, ids) = router(x @ gate_w^T).  Backward: the softmax / top-k scatter kernel gives the gradient that
    reaches the logits through the weights; added to whatever arrives on the logits themselves (auxiliary losses), it goes
    through the two library GEMMs of a linear layer."""

    @staticmethod
    def forward(ctx, x: torch.Tensor, gate_w: torch.Tensor, top_k: int):
        x = x.contiguous()
        gate_w = gate_w.contiguous()
        T, E = x.size(0), gate_w.size(0)
        logits = torch.empty(T, E, dtype=x.dtype, device=x.device)
        weights = torch.empty(T, top_k, dtype=x.dtype, device=x.device)
        ids = torch.empty(T, top_k, dtype=torch.int32, device=x.device)
        if T:
            _call(_gate_fwd_op, _gate_fwd_impl, x, gate_w, logits, weights, ids, top_k)
        ctx.save_for_backward(x, gate_w, weights, ids)
        ctx.mark_non_differentiable(ids)
        return logits, weights, ids

    @staticmethod
    def backward(ctx, d_logits_direct, d_weights, _d_ids):
        x, gate_w, weights, ids = ctx.saved_tensors
        T, E = x.size(0), gate_w.size(0)
        d_logits = torch.zeros(T, E, dtype=x.dtype, device=x.device)
        if T and d_weights is not None:
            _call(_bwd_op, _bwd_impl, weights, d_weights.contiguous().to(weights.dtype), ids, d_logits)
        if d_logits_direct is not None:
            d_logits = d_logits + d_logits_direct
        dx = d_logits @ gate_w if ctx.needs_input_grad[0] else None
        dw = d_logits.t() @ x if ctx.needs_input_grad[1] else None
        return dx, dw, None


def fused_gate_supported(x: torch.Tensor, gate_w: torch.Tensor, top_k: int) -> bool:
    E, H = gate_w.shape
    return (x.is_cuda and x.dtype in (torch.bfloat16, torch.float16) and gate_w.dtype == x.dtype and H % 8 == 0 and E % 8 == 0
            and E <= MAX_EXPERTS and 0 < top_k <= min(FUSED_MAX_TOP_K, E))


def router_gate_topk_softmax(x: torch.Tensor, gate_w: torch.Tensor, top_k: int):
    """``(router_logits [T, E], router_weights [T, k], selected_experts [T, k] int32)`` from tokens ``x [T, H]`` and the gate
    weight ``[E, H]`` in one tensor-core launch: the gate projection with the top-k / softmax / ids in its epilogue.
    16-bit dtypes, ``H % 8 == 0``, ``E % 8 == 0``, ``E <= 256``, ``k <= 8`` (see :func:`fused_gate_supported`)."""
    if x.dim() != 2 or gate_w.dim() != 2 or x.size(1) != gate_w.size(1):
        raise ValueError("x must be [tokens, H] and gate_w [experts, H]")
    if not fused_gate_supported(x, gate_w, top_k):
        raise ValueError("shape / dtype outside the fused router's range; use gate(x) + router_topk_softmax")
    return _GateRouter.apply(x, gate_w, top_k)


def supported(num_experts: int, top_k: int) -> bool:
    return num_experts <= MAX_EXPERTS and top_k <= MAX_TOP_K


def router_topk_softmax(router_logits: torch.Tensor, top_k: int) -> tuple[torch.Tensor, torch.Tensor]:
    """``(router_weights [T, k] in the logits' dtype, selected_experts [T, k] int32)`` from ``[T, E]`` gate logits.

    Selection is descending by logit with ties to the lower expert index; weights are the fp32 softmax over the
    selected logits rounded to the logits' dtype.  Raises on CPU tensors and when ``E > 256`` or ``k > 32``.
    """
    if router_logits.dim() != 2:
        raise ValueError("router_logits must be [tokens, experts]")
    if not 0 < top_k <= router_logits.size(1):
        raise ValueError("top_k must be in [1, num_experts]")
    return _RouterTopkSoftmax.apply(router_logits, top_k)
