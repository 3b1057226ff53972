"""Eager-PyTorch counterparts with the reference's ``*_torch`` / ``MoE_Torch`` names.

The reference package exports a plain-PyTorch implementation next to every kernel
(cute_kernels/__init__.py:15-54: ``MoE_Torch``, ``swiglu_torch``, ``swiglu_packed_torch``, ``continuous_count_torch``,
``rmsnorm_torch``, ``fused_residual_add_rmsnorm_torch``) and code written against it imports those names, usually as
the "expected" side of a comparison.  They are kept here so such imports keep working.  They are ordinary torch code
that runs wherever torch runs; nothing in this package calls them -- no ``*_cute`` function or ``MoE_Cute`` falls back
to them, and the sm_100a kernels raise on CPU tensors instead.
"""

from __future__ import annotations

from typing import Callable

import torch
import torch.nn as nn
import torch.nn.functional as F


def swiglu_torch(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    """``up * silu(gate)`` in fp32, cast back (kernels/swiglu/torch_implementation.py:9-18)."""
    dtype = gate.dtype
    return (up.float() * F.silu(gate.float())).to(dtype)


def swiglu_packed_torch(x: torch.Tensor) -> torch.Tensor:
    """``x = [up | gate]`` along the last dimension (kernels/swiglu/torch_implementation.py:21-23)."""
    up, gate = x.chunk(2, dim=-1)
    return swiglu_torch(gate, up)


def continuous_count_torch(x: torch.Tensor, size: int) -> torch.Tensor:
    """``bincount(minlength=size)`` as uint32 (kernels/continuous_count/torch_implementation.py:9-10)."""
    return x.bincount(minlength=size).to(torch.uint32)


def rmsnorm_torch(x: torch.Tensor, weight: torch.Tensor | None, eps: float) -> torch.Tensor:
    """kernels/rmsnorm/torch_implementation.py:9-10."""
    return F.rms_norm(x, (x.size(-1),), weight=weight, eps=eps)


def fused_residual_add_rmsnorm_torch(x: torch.Tensor, residual: torch.Tensor, weight: torch.Tensor | None, eps: float,
                                     multiplier: float | None = None) -> tuple[torch.Tensor, torch.Tensor]:
    """kernels/fused_residual_add_rmsnorm/torch_implementation.py:9-20."""
    if multiplier not in (None, 1):
        x = x * multiplier
    x = x + residual
    return F.rms_norm(x, (x.size(-1),), weight=weight, eps=eps), x


class Experts_Torch(nn.Module):
    """``weight [E, out, in]``, optional ``bias [E, out]``; one ``F.linear`` per expert over a split of the rows
    (kernels/scattermoe/torch_implementation.py:12-60)."""

    def __init__(self, num_experts: int, in_features: int, out_features: int, add_bias: bool = True, std: float | None = None) -> None:
        super().__init__()
        self.weight = nn.Parameter(torch.empty(num_experts, out_features, in_features))
        self.bias = nn.Parameter(torch.empty(num_experts, out_features)) if add_bias else None
        self.std = std
        self.num_experts = num_experts
        self.in_features = in_features
        self.out_features = out_features
        self.reset_parameters()

    @torch.no_grad()
    def reset_parameters(self) -> None:
        nn.init.normal_(self.weight, mean=0, std=self.std)
        if self.bias is not None:
            self.bias.zero_()

    def forward(self, rows: torch.Tensor | list[torch.Tensor], rows_per_expert: torch.Tensor, return_list: bool = False):
        if isinstance(rows, torch.Tensor):
            rows = rows.split(rows_per_expert.tolist(), dim=0)
        out = [F.linear(r, self.weight[e], None if self.bias is None else self.bias[e]) for e, r in enumerate(rows)]
        return out if return_list else torch.cat(out, dim=0)


class MoE_Torch(nn.Module):
    """The reference's eager MoE layer (kernels/scattermoe/torch_implementation.py:63-201): same constructor, parameters,
    ``state_dict`` and ``(hidden_states, router_logits)`` return as :class:`MoE_Cute`, computed with torch ops."""

    def __init__(self, num_experts: int, num_experts_per_tok: int, hidden_size: int, intermediate_size: int,
                 activation_function: Callable, is_glu: bool, add_bias: bool, std: float) -> None:
        super().__init__()
        self.num_experts = num_experts
        self.top_k = num_experts_per_tok
        self.hidden_size = hidden_size
        self.intermediate_size = intermediate_size
        self.gate = nn.Linear(hidden_size, num_experts, bias=False)
        self.c_fc = Experts_Torch(num_experts, hidden_size, 2 * intermediate_size if is_glu else intermediate_size, add_bias, std)
        self.act = activation_function
        self.c_proj = Experts_Torch(num_experts, intermediate_size, hidden_size, add_bias, std)

    def forward(self, hidden_states: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
        shape = hidden_states.shape
        x = hidden_states.view(-1, self.hidden_size)
        router_logits, router_weights, selected_experts = self._compute_routing_weights(x)
        return self._compute_experts(x, router_weights, selected_experts).view(shape), router_logits

    def _compute_routing_weights(self, x: torch.Tensor):
        router_logits = self.gate(x)
        if self.top_k == 1:
            vals, selected = router_logits.max(dim=-1, keepdim=True)
        else:
            vals, selected = router_logits.topk(self.top_k, dim=-1)
        return router_logits, F.softmax(vals.float(), dim=-1).type_as(x), selected

    def _compute_experts(self, x: torch.Tensor, router_weights: torch.Tensor, selected_experts: torch.Tensor) -> torch.Tensor:
        flat = selected_experts.flatten()
        rows_per_expert = flat.bincount(minlength=self.num_experts)
        order = flat.argsort()
        token_of_row = order // self.top_k
        gates = router_weights.flatten()[order]
        hidden = self.c_fc(x[token_of_row], rows_per_expert, return_list=True)
        hidden = [self.act(h) for h in hidden]
        rows = self.c_proj(hidden, rows_per_expert) * gates.unsqueeze(-1)
        return torch.zeros(x.size(0), self.hidden_size, dtype=rows.dtype, device=rows.device).index_add(0, token_of_row, rows)
