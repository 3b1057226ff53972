"""Router tail on one kernel: top-k of the gate logits, softmax over the selected k, int32 expert ids.

The reference runs ``topk`` (``max`` when k == 1), ``softmax(.float())`` and ``type_as`` as separate torch ops
and hands an int64 ``selected_experts`` to the expert path
(kernels/scattermoe/torch_implementation.py:122-135,195-201).  ``router_topk_softmax`` computes the same
``(router_weights, selected_experts)`` pair in one launch and keeps the ids int32, the form the routing kernels
read.  The gate projection itself stays ``nn.Linear`` (a library GEMM).  Differentiable in the logits: the
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
