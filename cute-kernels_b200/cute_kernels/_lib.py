"""ctypes binding of libck_b200.so (the C ABI declared in include/ck_b200.h).

The library is built ahead of time (``python __graft_entry__.py`` or ``make -C csrc``); there is no
JIT, no backend search and no CPU fallback: importing this module without the built library raises.
It replaces the reference's ``cute_kernels/jit.py`` (cpp_extension.load on first call) and
``cute_kernels/cutotune`` (runtime search) for the MoE expert path.
"""

from __future__ import annotations

import ctypes
import os

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.environ.get("CK_LIB_PATH") or os.path.join(_HERE, "libck_b200.so")

CK_F32, CK_F16, CK_BF16 = 0, 1, 2
CK_ACT_SWIGLU, CK_ACT_GLU, CK_ACT_GELU_TANH = 0, 1, 2
CK_DEV_RANGE, CK_DEV_TIMEOUT, CK_DEV_META = 1, 2, 4
CK_TILE_M = 128
CK_COUNT_MAX_SIZE = 16384
CK_ROUTE_MAX_EXPERTS = 1024

_vp, _i, _i64 = ctypes.c_void_p, ctypes.c_int, ctypes.c_int64

# name -> (restype, argtypes); must list every symbol include/ck_b200.h declares
PROTOTYPES = {
    "ck_status_string": (ctypes.c_char_p, [_i]),
    "ck_last_cuda_error": (ctypes.c_char_p, []),
    "ck_abi_version": (_i, []),
    "ck_continuous_count": (_i, [_vp, _i, _i64, _i, _vp, _vp]),
    "ck_route_workspace_bytes": (_i64, [_i64, _i]),
    "ck_route_padded_capacity": (_i64, [_i64, _i]),
    "ck_route": (_i, [_vp, _i, _i64, _i, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i64, _vp, _vp]),
    "ck_route_static_max_bytes": (_i64, []),
    "ck_route_static": (_i, [_vp, _i, _i64, _i, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp]),
    "ck_swiglu_fwd": (_i, [_vp, _vp, _vp, _i64, _i64, _i64, _i64, _i, _vp]),
    "ck_swiglu_bwd": (_i, [_vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _i64, _i64, _i, _vp]),
    "ck_moe_gather_rows": (_i, [_vp, _vp, _vp, _vp, _i, _i64, _i, _i64, _i, _vp]),
    "ck_cast_from_f32": (_i, [_vp, _vp, _i64, _i, _vp]),
    "ck_moe_up_act_fwd": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i64, _i, _i, _i, _i, _vp, _vp]),
    "ck_moe_up_act_fwd_gather": (_i, [_vp, _i64, _i, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i64, _i, _i, _i, _i, _vp, _vp]),
    "ck_moe_up_act_fwd_gather_peer": (_i, [_vp, _i, _i64, _i, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i64, _i, _i, _i, _i, _vp, _vp]),
    "ck_moe_down_combine_fwd": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i64, _i, _i, _i, _i, _vp, _vp]),
    "ck_moe_dgrad_down": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i64, _i, _i, _i, _i, _vp, _vp]),
    "ck_moe_dgrad_down_parts": (_i, [_i]),
    "ck_moe_reduce_dgates": (_i, [_vp, _i, _i64, _vp, _vp, _i, _vp, _vp]),
    "ck_moe_dgrad_down_gather": (_i, [_vp, _i64, _i, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i64, _i, _i, _i, _i, _vp, _vp]),
    "ck_moe_dgrad_down_gather_peer": (_i, [_vp, _i, _i64, _i, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i64, _i, _i, _i, _i, _vp, _vp]),
    "ck_moe_wgrad_gather": (_i, [_vp, _i64, _i, _vp, _i64, _i, _vp, _vp, _vp, _i, _i64, _i, _i, _i, _vp, _vp]),
    "ck_moe_dgrad_up": (_i, [_vp, _vp, _vp, _vp, _vp, _i, _i64, _i, _i, _i, _i, _vp, _vp]),
    "ck_moe_wgrad": (_i, [_vp, _vp, _vp, _vp, _i, _i64, _i, _i, _i, _vp, _vp]),
    "ck_moe_grouped_linear": (_i, [_vp, _vp, _vp, _vp, _i, _i64, _i, _i, _i, _i, _vp, _vp]),
    "ck_set_gemm_cta_pair": (_i, [_i]),
    "ck_gemm_cta_pair": (_i, []),
    "ck_set_gemm_sm_budget": (_i, [_i]),
    "ck_gemm_sm_budget": (_i, []),
    "ck_moe_grouped_linear_scatter": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i64, _i, _i, _i, _i, _vp, _vp]),
    "ck_moe_bias_grad": (_i, [_vp, _i64, _i, _vp, _vp, _vp, _i, _vp, _i, _vp]),
    "ck_moe_bias_dots": (_i, [_vp, _i64, _i, _vp, _vp, _i, _vp, _i, _vp]),
    "ck_moe_gather_rows_scaled": (_i, [_vp, _vp, _vp, _vp, _i64, _i, _i64, _i, _vp]),
    "ck_moe_combine_rows": (_i, [_vp, _vp, _vp, _vp, _i64, _i, _i64, _i, _vp]),
    "ck_moe_row_dots": (_i, [_vp, _vp, _vp, _vp, _i64, _i, _i64, _i, _vp]),
    "ck_rmsnorm_fwd": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _i64, _i64, ctypes.c_float, ctypes.c_float, _i, _vp]),
    "ck_rmsnorm_bwd_parts": (_i64, [_i64, _i64]),
    "ck_rmsnorm_bwd": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i64, _i64, ctypes.c_float, ctypes.c_float, _i, _vp]),
    "ck_router_topk_softmax": (_i, [_vp, _vp, _vp, _i64, _i, _i, _i, _vp]),
    "ck_router_topk_softmax_bwd": (_i, [_vp, _vp, _vp, _vp, _i64, _i, _i, _i, _vp, _vp]),
    "ck_router_gate_topk_softmax": (_i, [_vp, _vp, _vp, _vp, _vp, _i64, _i, _i, _i, _i, _vp, _vp]),
    "ck_moe_gather_rows_peer": (_i, [_vp, _i, _i64, _vp, _vp, _vp, _vp, _i, _i64, _i, _i64, _i64, _i64, _i, _vp, _vp]),
    "ck_moe_grouped_linear_scatter_peer": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _i, _i64, _i, _i64, _i, _i, _i, _i, _vp, _vp]),
    "ck_peer_gather_scalars": (_i, [_vp, _i, _i64, _vp, _i64, _vp, _i, _vp, _vp]),
    "ck_peer_scatter_scalars": (_i, [_vp, _vp, _i64, _i, _vp, _i, _i64, _i, _vp, _vp]),
    "ck_test_wait_timeout": (_i, [_i64, _vp, _vp, _vp]),
}


def _load() -> ctypes.CDLL:
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `python __graft_entry__.py` (or `make -C cute-kernels_b200/csrc`). "
            "This package has no fallback path."
        )
    lib = ctypes.CDLL(LIB_PATH)
    for name, (res, args) in PROTOTYPES.items():
        fn = getattr(lib, name)
        fn.restype = res
        fn.argtypes = args
    return lib


lib = _load()

_DTYPE_CODE = {torch.float32: CK_F32, torch.float16: CK_F16, torch.bfloat16: CK_BF16}


def dtype_code(dtype: torch.dtype) -> int:
    try:
        return _DTYPE_CODE[dtype]
    except KeyError:
        raise TypeError(f"unsupported dtype {dtype}: the kernels take float32, float16 and bfloat16") from None


def check(status: int, what: str) -> None:
    """Turns a negative ck_status into a RuntimeError (the reference raises through TORCH_CHECK)."""
    if status == 0:
        return
    name = lib.ck_status_string(int(status)).decode()
    detail = lib.ck_last_cuda_error().decode() if name == "CK_ERR_CUDA" else ""
    raise RuntimeError(f"{what} failed with {name}" + (f": {detail}" if detail else ""))


def require_cuda(*tensors: torch.Tensor) -> None:
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise RuntimeError("cute_kernels (B200) ops take CUDA tensors only; there is no CPU path")


_trace_depth = 0


class tracing:
    """``with tracing():`` -- every op of this package goes through its opaque ``torch.library`` custom op inside the
    block, whatever ``torch.compiler.is_compiling()`` says (a compiler backend that re-traces a captured graph with
    fake tensors, as CuteInductor does when it hands the rewritten graph to inductor, is not "compiling" for dynamo)."""

    def __enter__(self):
        global _trace_depth
        _trace_depth += 1
        return self

    def __exit__(self, *exc):
        global _trace_depth
        _trace_depth -= 1
        return False


def use_custom_op() -> bool:
    """True when a call must be recorded as an opaque custom op instead of launching the kernel right away."""
    return _trace_depth > 0 or torch.compiler.is_compiling()


def stream_ptr() -> int:
    return torch.cuda.current_stream().cuda_stream


def ptr(t: torch.Tensor | None) -> int | None:
    return None if t is None else t.data_ptr()


_status_words: dict[int, torch.Tensor] = {}


def status_word(device: torch.device) -> torch.Tensor:
    """One int32 per device into which kernels OR CK_DEV_* bits."""
    idx = device.index if device.index is not None else torch.cuda.current_device()
    w = _status_words.get(idx)
    if w is None:
        w = torch.zeros(1, dtype=torch.int32, device=torch.device("cuda", idx))
        _status_words[idx] = w
    return w


def check_device_status(device: torch.device | None = None) -> None:
    """Synchronises and raises if any kernel flagged a device-side problem since the last check."""
    if device is None:
        device = torch.device("cuda", torch.cuda.current_device())
    w = status_word(device)
    v = int(w.item())
    if v == 0:
        return
    w.zero_()
    names = [n for bit, n in ((CK_DEV_RANGE, "CK_DEV_RANGE (expert id out of range)"),
                              (CK_DEV_TIMEOUT, "CK_DEV_TIMEOUT (a bounded device wait ran out)"),
                              (CK_DEV_META, "CK_DEV_META (tile metadata exceeds the allocated rows)")) if v & bit]
    raise RuntimeError("device status: " + ", ".join(names))


class gemm_sm_budget:
    """``with gemm_sm_budget(n):`` -- grouped GEMMs launched inside the block occupy at most ``n`` SMs (0 = all), leaving the
    rest to kernels of other streams.  The budget is read when a GEMM is launched, so it only has to cover the launch call;
    it is process-wide (see ck_set_gemm_sm_budget), so do not launch GEMMs from other threads meanwhile."""

    def __init__(self, sms: int) -> None:
        self.sms, self.prev = int(sms), 0

    def __enter__(self):
        self.prev = lib.ck_set_gemm_sm_budget(self.sms)
        return self

    def __exit__(self, *exc):
        lib.ck_set_gemm_sm_budget(self.prev)
        return False


# ---- launch accounting ------------------------------------------------------------------------------
class LaunchLog:
    """Counts this library's kernel launches and, when enabled, brackets each with CUDA events on the
    launching stream so a harness can attribute device time to kernels inside its own timed region."""

    def __init__(self) -> None:
        self.count = 0
        self.record_events = False
        self.events: list[tuple[str, float, "torch.cuda.Event", "torch.cuda.Event"]] = []

    def reset(self) -> None:
        self.count = 0
        self.events = []


launch_log = LaunchLog()


class launch:
    """``with launch("kernel", n_kernels, work): lib.ck_...`` -- bookkeeping around one C-ABI call."""

    __slots__ = ("name", "n", "work", "e0")

    def __init__(self, name: str, n_kernels: int = 1, work: float = 0.0) -> None:
        self.name, self.n, self.work, self.e0 = name, n_kernels, work, None

    def __enter__(self):
        if launch_log.record_events:
            self.e0 = torch.cuda.Event(enable_timing=True)
            self.e0.record()
        return self

    def __exit__(self, *exc):
        launch_log.count += self.n
        if self.e0 is not None:
            e1 = torch.cuda.Event(enable_timing=True)
            e1.record()
            launch_log.events.append((self.name, self.work, self.e0, e1))
        return False
