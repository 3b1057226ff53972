"""CPU oracle for the MoE expert path.  TEST INFRASTRUCTURE ONLY.

Nothing under ``cute-kernels_b200/`` imports this file; only ``tests/``, ``__graft_entry__.smoke()`` and
the ``cpu_baseline`` / ``--impl reference`` legs of ``bench.py`` do, as the checker or the timed CPU arm.

Each function restates, in plain numpy / torch-on-CPU, what the reference computes on this path, and
cites the reference file:line it follows.  Parity pinning: ``tests/golden/make_golden.py`` runs the
reference's own ``MoE_Torch``, ``swiglu_torch``, ``swiglu_packed_torch`` and ``continuous_count_torch``
(imported from the reference checkout) on seeded inputs and stores the results under ``tests/golden/``;
``tests/test_oracle_golden.py`` checks every function here against those vectors.
"""

from __future__ import annotations

import math

import numpy as np
import torch
import torch.nn.functional as F

TILE_M = 128


# ---------------------------------------------------------------------------------------------------
# integer path (bit exact)
# ---------------------------------------------------------------------------------------------------
def continuous_count_ref(x: np.ndarray, size: int) -> np.ndarray:
    """kernels/continuous_count/torch_implementation.py:9-10: bincount(minlength=size) as uint32.
    Out-of-range values are dropped (kernels/continuous_count/__init__.py:15-16)."""
    x = np.asarray(x).reshape(-1)
    x = x[(x >= 0) & (x < size)]
    return np.bincount(x, minlength=size).astype(np.uint32)


def route_ref(ids: np.ndarray, num_experts: int) -> dict[str, np.ndarray]:
    """Routing outputs of MoE_Triton._compute_experts (kernels/scattermoe/triton_implementation/__init__.py:82-83:
    sort -> sorted_scattered_idxs, bincount().cumsum() -> END offsets) and of
    MoE_Torch._compute_expert_assignment (kernels/scattermoe/torch_implementation.py:171-193), with the
    sort made stable so the index order is well defined, plus the 128-row padded layout."""
    ids = np.asarray(ids).reshape(-1).astype(np.int64)
    counts = np.bincount(ids, minlength=num_experts).astype(np.int64)
    end = np.cumsum(counts)
    excl = end - counts
    sorted_idx = np.argsort(ids, kind="stable").astype(np.int32)
    tiles = (counts + TILE_M - 1) // TILE_M
    mtile_off = np.concatenate([[0], np.cumsum(tiles)]).astype(np.int32)
    padded_off = (mtile_off.astype(np.int64) * TILE_M).astype(np.int32)
    cap = (ids.size // TILE_M + num_experts) * TILE_M
    row_map = np.full(cap, -1, dtype=np.int32)
    for e in range(num_experts):
        row_map[padded_off[e] : padded_off[e] + counts[e]] = sorted_idx[excl[e] : end[e]]
    return dict(
        counts=counts.astype(np.uint32), excl_off=excl.astype(np.int32), end_off=end.astype(np.int32),
        sorted_idx=sorted_idx, sorted_expert=ids[sorted_idx].astype(np.int32), padded_off=padded_off,
        mtile_off=mtile_off, row_map=row_map,
    )


# ---------------------------------------------------------------------------------------------------
# SwiGLU
# ---------------------------------------------------------------------------------------------------
def swiglu_ref(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    """kernels/swiglu/torch_implementation.py:9-18: fp32 up * silu(gate), cast back."""
    return (up.float() * F.silu(gate.float())).to(gate.dtype)


def swiglu_packed_ref(x: torch.Tensor) -> torch.Tensor:
    """kernels/swiglu/torch_implementation.py:21-23: first half = up, second half = gate."""
    half = x.size(-1) // 2
    return swiglu_ref(x[..., half:], x[..., :half])


def swiglu_backward_ref(gate: torch.Tensor, up: torch.Tensor, dy: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    """kernels/swiglu/cuda_implementation/backward.cu:27-35 (formula of kernels/swiglu/README.md:7-17)."""
    g, u, d = gate.float(), up.float(), dy.float()
    s = torch.sigmoid(g)
    silu = g * s
    return (d * u * (s + silu * (1 - s))).to(gate.dtype), (d * silu).to(gate.dtype)


# ---------------------------------------------------------------------------------------------------
# RMSNorm
# ---------------------------------------------------------------------------------------------------
def rmsnorm_ref(x: torch.Tensor, weight: torch.Tensor | None, eps: float) -> torch.Tensor:
    """kernels/rmsnorm/torch_implementation.py:9-10 (F.rms_norm over the last dimension): statistics and scaling in
    fp32, one rounding to the input dtype at the end."""
    xf = x.float()
    y = xf * torch.rsqrt(xf.pow(2).mean(dim=-1, keepdim=True) + eps)
    if weight is not None:
        y = y * weight.float()
    return y.to(x.dtype)


def fused_residual_add_rmsnorm_ref(x: torch.Tensor, residual: torch.Tensor, weight: torch.Tensor | None, eps: float,
                                   multiplier: float | None = None) -> tuple[torch.Tensor, torch.Tensor]:
    """kernels/fused_residual_add_rmsnorm/torch_implementation.py:9-20: x * multiplier (skipped for None / 1), + residual
    (each a tensor op in the input dtype), the sum is both the new residual stream and the input of the norm."""
    if multiplier not in (None, 1):
        x = x * multiplier
    x = x + residual
    return rmsnorm_ref(x, weight, eps), x


# ---------------------------------------------------------------------------------------------------
# MoE expert layer
# ---------------------------------------------------------------------------------------------------
def routing_weights_ref(router_logits: torch.Tensor, top_k: int, out_dtype: torch.dtype):
    """kernels/scattermoe/torch_implementation.py:122-135,195-201: top-k (max for k == 1), softmax over
    the selected logits in fp32, cast to the activation dtype."""
    if top_k == 1:
        vals, idx = router_logits.max(dim=-1, keepdim=True)
    else:
        vals, idx = router_logits.topk(top_k, dim=-1)
    return F.softmax(vals.float(), dim=-1).to(out_dtype), idx


def moe_experts_ref(x, router_weights, selected_experts, w_fc, w_proj, activation, b_fc=None, b_proj=None):
    """MoE_Torch._compute_experts (kernels/scattermoe/torch_implementation.py:137-169) with
    Experts_Torch.forward (:32-49) inlined: group rows by expert, per-expert linear -> activation ->
    linear, scale by the router weight, index_add back to the token rows."""
    T, H = x.shape
    E = w_fc.size(0)
    k = selected_experts.size(1)
    flat = selected_experts.reshape(-1)
    order = torch.sort(flat, stable=True).indices
    tok = order // k
    counts = torch.bincount(flat, minlength=E).tolist()
    gates = router_weights.reshape(-1)[order]
    rows = x[tok]
    outs = []
    start = 0
    for e in range(E):
        seg = rows[start : start + counts[e]]
        hid = F.linear(seg, w_fc[e], None if b_fc is None else b_fc[e])
        hid = activation(hid)
        outs.append(F.linear(hid, w_proj[e], None if b_proj is None else b_proj[e]))
        start += counts[e]
    y = torch.cat(outs) * gates.unsqueeze(-1)
    return torch.zeros(T, H, dtype=y.dtype, device=y.device).index_add(0, tok, y)


class MoERef(torch.nn.Module):
    """Parameter-compatible restatement of MoE_Torch (kernels/scattermoe/torch_implementation.py:63-120):
    state_dict keys gate.weight [E, H], c_fc.weight [E, 2I or I, H], c_proj.weight [E, H, I] (+ biases)."""

    class _Experts(torch.nn.Module):
        def __init__(self, E, fin, fout, add_bias, std):
            super().__init__()
            self.weight = torch.nn.Parameter(torch.empty(E, fout, fin).normal_(0, std))
            self.bias = torch.nn.Parameter(torch.zeros(E, fout)) if add_bias else None

    def __init__(self, num_experts, num_experts_per_tok, hidden_size, intermediate_size, activation_function, is_glu,
                 add_bias, std):
        super().__init__()
        self.top_k = num_experts_per_tok
        self.hidden_size = hidden_size
        self.gate = torch.nn.Linear(hidden_size, num_experts, bias=False)
        self.c_fc = self._Experts(num_experts, hidden_size, intermediate_size * (2 if is_glu else 1), add_bias, std)
        self.c_proj = self._Experts(num_experts, intermediate_size, hidden_size, add_bias, std)
        self.act = activation_function

    def forward(self, hidden_states, forced_selection=None):
        """``forced_selection`` [T, k] pins the chosen experts (a 16-bit router can break near-ties differently
        from this fp32 one); the router weights are still the softmax of this module's own logits."""
        shape = hidden_states.shape
        x = hidden_states.view(-1, self.hidden_size)
        logits = self.gate(x)
        if forced_selection is None:
            w, idx = routing_weights_ref(logits, self.top_k, x.dtype)
        else:
            idx = forced_selection
            w = F.softmax(logits.gather(1, idx).float(), dim=-1).to(x.dtype)
        y = moe_experts_ref(x, w, idx, self.c_fc.weight, self.c_proj.weight, self.act, self.c_fc.bias, self.c_proj.bias)
        return y.view(shape), logits


# ---------------------------------------------------------------------------------------------------
# seeded synthetic inputs (shapes and distributions of the five benchmark configurations)
# ---------------------------------------------------------------------------------------------------
CONFIGS = {
    "c1_cpu": dict(T=512, H=256, I=512, E=8, k=2, expert_bias=False),
    "c4_mixtral": dict(T=16384, H=4096, I=14336, E=8, k=2, expert_bias=False),
    "c5_finegrained": dict(T=32768, H=2048, I=1408, E=64, k=8, expert_bias=True),
}


def gen_moe_inputs(seed: int, T: int, H: int, I: int, E: int, k: int, expert_bias: bool = False,
                   dtype: torch.dtype = torch.float32) -> dict[str, torch.Tensor]:
    """One generator, fixed draw order, fp32 on CPU then cast: x ~ N(0,1); router logits ~ N(0,1)
    (+ a per-expert N(0,1) bias for the fine-grained config); W_up, W_gate, W_down ~ N(0, 0.02);
    grad_out ~ N(0,1).  c_fc.weight = cat([W_up, W_gate], dim=1) (packed [up | gate])."""
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(T, H, generator=g)
    logits = torch.randn(T, E, generator=g)
    if expert_bias:
        logits = logits + torch.randn(E, generator=g)
    w_up = 0.02 * torch.randn(E, I, H, generator=g)
    w_gate = 0.02 * torch.randn(E, I, H, generator=g)
    w_down = 0.02 * torch.randn(E, H, I, generator=g)
    grad_out = torch.randn(T, H, generator=g)
    w_fc = torch.cat([w_up, w_gate], dim=1)
    router_weights, selected = routing_weights_ref(logits, k, dtype)
    return dict(x=x.to(dtype), router_logits=logits, router_weights=router_weights, selected_experts=selected,
                w_fc=w_fc.to(dtype), w_proj=w_down.to(dtype), grad_out=grad_out.to(dtype))


def gen_ids(seed: int, n: int, E: int, dist: str = "uniform", dtype=np.int32) -> np.ndarray:
    """Expert ids for the count / sort benchmark: uniform over [0, E) or Zipf-skewed p_i ~ 1/(i+1)^1.2."""
    rng = np.random.default_rng(seed)
    if dist == "uniform":
        return rng.integers(0, E, size=n, dtype=np.int64).astype(dtype)
    if dist == "zipf":
        p = 1.0 / np.power(np.arange(1, E + 1, dtype=np.float64), 1.2)
        p /= p.sum()
        return rng.choice(E, size=n, p=p).astype(dtype)
    raise ValueError(dist)


def moe_fwd_bwd_ref(inp: dict[str, torch.Tensor], activation=swiglu_packed_ref, dtype=torch.float32) -> dict[str, torch.Tensor]:
    """fwd + bwd of the expert computation on the inputs of gen_moe_inputs, computed in ``dtype`` on CPU."""
    x = inp["x"].to(dtype).clone().requires_grad_()
    rw = inp["router_weights"].to(dtype).clone().requires_grad_()
    w_fc = inp["w_fc"].to(dtype).clone().requires_grad_()
    w_proj = inp["w_proj"].to(dtype).clone().requires_grad_()
    y = moe_experts_ref(x, rw, inp["selected_experts"], w_fc, w_proj, activation)
    y.backward(inp["grad_out"].to(dtype))
    return dict(y=y.detach(), dx=x.grad, d_router_weights=rw.grad, d_w_fc=w_fc.grad, d_w_proj=w_proj.grad)


def moe_flops(T: int, H: int, I: int, k: int, backward: bool = True) -> float:
    """Algorithmic FLOPs of the six expert GEMMs: 6*k*H*I per token forward, 18*k*H*I forward+backward."""
    return float(T) * (18.0 if backward else 6.0) * k * H * I


def is_close_report(a: torch.Tensor, b: torch.Tensor) -> str:
    d = (a.float() - b.float()).abs()
    return f"max_abs={d.max().item():.3e} ref_max={b.float().abs().max().item():.3e}"
