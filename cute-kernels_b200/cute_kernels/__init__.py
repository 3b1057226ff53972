"""B200-native drop-in for the MoE expert path of cute-kernels.

Public names follow the reference package (cute_kernels/__init__.py:5-58) for this path:
``continuous_count_cute``, ``swiglu_cute``, ``swiglu_packed_cute``, ``rmsnorm_cute``, ``fused_residual_add_rmsnorm_cute``,
``CuteInductor``, ``KernelBackend``, ``CutoTuneParameter``, ``set_seed``, ``ceil_divide`` -- plus ``MoE_Cute``, which takes
the constructor arguments and state_dict of the reference's ``MoE_Torch`` / ``MoE_Triton``.  ``MoE_Triton`` is an alias
of ``MoE_Cute`` (the GPU implementation of the layer); ``MoE_Torch`` and the ``*_torch`` functions are the eager-PyTorch
counterparts the reference exports under those names (:mod:`torch_reference`), never used by the kernels' code paths.
"""

from ._lib import check_device_status
from .continuous_count import continuous_count_cute
from .cute_inductor import CuteInductor, replace_rmsnorm, replace_swiglu_unchunked
from .expert_parallel import (ExpertParallelMoE, balanced_expert_placement, gather_expert_state_dict,
                              shard_expert_state_dict)
from .kernel_backend import CutoTuneParameter, KernelBackend
from .moe import Experts_Cute, MoE_Cute, fused_experts
from .rmsnorm import fused_residual_add_rmsnorm_cute, rmsnorm_cute
from .router import router_gate_topk_softmax, router_topk_softmax
from .routing import Routing, padded_capacity, route
from .swiglu import swiglu_cute, swiglu_packed_cute
from .torch_reference import (Experts_Torch, MoE_Torch, continuous_count_torch, fused_residual_add_rmsnorm_torch,
                              rmsnorm_torch, swiglu_packed_torch, swiglu_torch)
from .utils import ceil_divide, divide_if_divisible, set_seed

MoE_Triton = MoE_Cute  # the reference's name for its GPU implementation of the layer

__all__ = [
    "Experts_Torch", "MoE_Torch", "balanced_expert_placement", "MoE_Triton", "continuous_count_torch", "fused_residual_add_rmsnorm_torch", "rmsnorm_torch",
    "swiglu_packed_torch", "swiglu_torch",
    "CuteInductor", "CutoTuneParameter", "ExpertParallelMoE", "Experts_Cute", "KernelBackend", "MoE_Cute", "Routing", "ceil_divide",
    "check_device_status", "continuous_count_cute", "divide_if_divisible", "fused_experts", "gather_expert_state_dict", "padded_capacity",
    "fused_residual_add_rmsnorm_cute", "replace_rmsnorm", "replace_swiglu_unchunked", "rmsnorm_cute", "route", "router_gate_topk_softmax", "router_topk_softmax", "set_seed", "shard_expert_state_dict", "swiglu_cute", "swiglu_packed_cute",
]
