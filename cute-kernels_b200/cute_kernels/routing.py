"""Routing front end of the MoE: count + exclusive scan + stable scatter in three launches.

Replaces ``selected_experts.flatten().sort()`` + ``bincount`` + ``cumsum`` of the reference
(kernels/scattermoe/triton_implementation/__init__.py:82-83) and the bincount/argsort of
``MoE_Torch._compute_expert_assignment`` (kernels/scattermoe/torch_implementation.py:171-193).
"""

from __future__ import annotations

from dataclasses import dataclass

import torch

from . import _lib


@dataclass
class Routing:
    """Outputs of :func:`route`.

    counts        uint32[E]   bincount(ids, minlength=E)
    excl_offsets  int32[E]    exclusive scan of counts
    end_offsets   int32[E]    inclusive scan (the reference's ``expert_offsets``)
    sorted_idx    int32[n]    torch.sort(ids, stable=True).indices
    sorted_expert int32[n]    ids[sorted_idx]  (None unless requested)
    padded_off    int32[E+1]  start row of every expert in the 128-row padded layout (None w/o metadata)
    mtile_off     int32[E+1]  padded_off / 128
    row_map       int32[cap]  padded row -> flat (token * top_k + slot) index, -1 on pad rows
    """

    counts: torch.Tensor
    excl_offsets: torch.Tensor
    end_offsets: torch.Tensor
    sorted_idx: torch.Tensor
    sorted_expert: torch.Tensor | None
    padded_off: torch.Tensor | None
    mtile_off: torch.Tensor | None
    row_map: torch.Tensor | None

    @property
    def capacity(self) -> int:
        return 0 if self.row_map is None else self.row_map.numel()


def padded_capacity(n: int, num_experts: int) -> int:
    return (n // _lib.CK_TILE_M + num_experts) * _lib.CK_TILE_M


def route_workspace_bytes(n: int, num_experts: int) -> int:
    """Python mirror of ck_route_workspace_bytes (kept out of ctypes so torch.compile can trace callers)."""
    if n <= 0:
        return 256 + num_experts * 4
    slice_len = -(-n // (148 * 4))          # at most 592 slices, one per thread block
    slice_len = -(-slice_len // 4096) * 4096  # whole 4096-id tiles
    return 256 + -(-n // slice_len) * num_experts * 4


def _route_impl(
    ids: torch.Tensor,
    num_experts: int,
    counts: torch.Tensor,
    excl: torch.Tensor,
    end: torch.Tensor,
    sorted_idx: torch.Tensor,
    sorted_expert: torch.Tensor | None,
    padded_off: torch.Tensor | None,
    mtile_off: torch.Tensor | None,
    row_map: torch.Tensor | None,
    workspace: torch.Tensor,
) -> None:
    _lib.require_cuda(ids, counts, sorted_idx, workspace)
    status = _lib.status_word(ids.device)
    with torch.cuda.device(ids.device), _lib.launch("route", 3 if ids.numel() else 1):
        st = _lib.lib.ck_route(
            ids.data_ptr(), int(ids.dtype == torch.int64), ids.numel(), num_experts,
            counts.data_ptr(), excl.data_ptr(), end.data_ptr(), sorted_idx.data_ptr(), _lib.ptr(sorted_expert),
            _lib.ptr(padded_off), _lib.ptr(mtile_off), _lib.ptr(row_map),
            workspace.data_ptr(), workspace.numel(), status.data_ptr(), _lib.stream_ptr(),
        )
    _lib.check(st, "ck_route")


_route_op = torch.library.custom_op(
    "cute_kernels_b200::route",
    _route_impl,
    mutates_args={"counts", "excl", "end", "sorted_idx", "sorted_expert", "padded_off", "mtile_off", "row_map",
                  "workspace"},
)


@torch.no_grad()
def route(ids: torch.Tensor, num_experts: int, *, with_tile_metadata: bool = True,
          with_sorted_expert: bool = False) -> Routing:
    """Stable counting sort of the flat expert ids (int32 or int64, values in [0, num_experts))."""
    assert ids.dim() == 1, "ids should be 1-dimensional"
    assert ids.dtype in (torch.int32, torch.int64)
    if not 0 < num_experts <= _lib.CK_ROUTE_MAX_EXPERTS:
        raise RuntimeError(f"num_experts must be in [1, {_lib.CK_ROUTE_MAX_EXPERTS}]")
    ids = ids.contiguous()
    dev = ids.device
    n = ids.numel()
    i32 = dict(dtype=torch.int32, device=dev)
    counts = torch.empty(num_experts, dtype=torch.uint32, device=dev)
    excl = torch.empty(num_experts, **i32)
    end = torch.empty(num_experts, **i32)
    sorted_idx = torch.empty(n, **i32)
    sorted_expert = torch.empty(n, **i32) if with_sorted_expert else None
    if with_tile_metadata:
        padded_off = torch.empty(num_experts + 1, **i32)
        mtile_off = torch.empty(num_experts + 1, **i32)
        row_map = torch.empty(padded_capacity(n, num_experts), **i32)
    else:
        padded_off = mtile_off = row_map = None
    workspace = torch.empty(route_workspace_bytes(n, num_experts), dtype=torch.uint8, device=dev)
    fn = _route_op if _lib.use_custom_op() else _route_impl
    fn(ids, num_experts, counts, excl, end, sorted_idx, sorted_expert, padded_off, mtile_off, row_map, workspace)
    return Routing(counts, excl, end, sorted_idx, sorted_expert, padded_off, mtile_off, row_map)
