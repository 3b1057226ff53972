"""B200-native drop-in for the MoE expert path of cute-kernels.

Public names follow the reference package (cute_kernels/__init__.py:5-58) for this path:
``continuous_count_cute``, ``swiglu_cute``, ``swiglu_packed_cute``, ``CuteInductor``, ``KernelBackend``,
``CutoTuneParameter``, ``set_seed``, ``ceil_divide`` -- plus ``MoE_Cute``, which takes the constructor
arguments and state_dict of the reference's ``MoE_Torch`` / ``MoE_Triton``.
"""

from ._lib import check_device_status
from .continuous_count import continuous_count_cute
from .cute_inductor import CuteInductor, replace_swiglu_unchunked
from .expert_parallel import ExpertParallelMoE, gather_expert_state_dict, shard_expert_state_dict
from .kernel_backend import CutoTuneParameter, KernelBackend
from .moe import Experts_Cute, MoE_Cute, fused_experts
from .router import router_topk_softmax
from .routing import Routing, padded_capacity, route
from .swiglu import swiglu_cute, swiglu_packed_cute
from .utils import ceil_divide, divide_if_divisible, set_seed

__all__ = [
    "CuteInductor", "CutoTuneParameter", "ExpertParallelMoE", "Experts_Cute", "KernelBackend", "MoE_Cute", "Routing", "ceil_divide",
    "check_device_status", "continuous_count_cute", "divide_if_divisible", "fused_experts", "gather_expert_state_dict", "padded_capacity",
    "replace_swiglu_unchunked", "route", "router_topk_softmax", "set_seed", "shard_expert_state_dict", "swiglu_cute", "swiglu_packed_cute",
]
