"""CuteInductor: a torch.compile backend that rewrites FX patterns into this package's kernels.

Same constructor and ``compiler(gm, example_inputs)`` entry as the reference
(cute_kernels/cute_inductor/compiler.py:18-47), and its two rewrites:

* ``replace_swiglu_unchunked``: a ``chunk(2, dim=-1)`` whose halves feed ``silu`` and ``mul`` becomes one
  ``swiglu_packed_cute`` call on the un-chunked tensor (cute_kernels/cute_inductor/swiglu_packed.py:16-76; the
  reference version calls an undefined name when the pattern matches, this one inserts the real function);
* ``replace_rmsnorm``: ``torch.rms_norm(input, normalized_shape, weight, eps)`` becomes
  ``rmsnorm_cute(x, weight, eps)`` (cute_kernels/cute_inductor/rmsnorm.py:13-35).
"""

from __future__ import annotations

import operator
import os
from typing import Callable

import torch
import torch.nn.functional as F
from torch._dynamo import lookup_backend
from torch.fx import Node
from torch.fx.graph_module import GraphModule

from . import _lib
from .rmsnorm import rmsnorm_cute
from .swiglu import swiglu_packed_cute

_DEBUG_CUTEINDUCTOR = os.environ.get("DEBUG_CUTEINDUCTOR", "0").lower() in ("1", "true")


def _is_chunk_in_two_on_last_dim(node: Node) -> bool:
    if node.op == "call_method" and node.target == "chunk":
        args = node.args[1:]
    elif node.op == "call_function" and node.target is torch.chunk:
        args = node.args[1:]
    else:
        return False
    chunks = node.kwargs.get("chunks", args[0] if len(args) > 0 else None)
    dim = node.kwargs.get("dim", args[1] if len(args) > 1 else 0)
    return chunks == 2 and dim == -1


def _match_swiglu(chunk: Node) -> Node | None:
    """Returns the final ``mul`` node when ``chunk`` feeds exactly up * silu(gate), else None."""
    getitems = list(chunk.users.keys())
    if len(getitems) != 2:
        return None
    halves = {}
    for g in getitems:
        if not (g.op == "call_function" and g.target is operator.getitem and g.args[1] in (0, 1)):
            return None
        halves[g.args[1]] = g
    if set(halves) != {0, 1}:
        return None
    up, gate = halves[0], halves[1]
    if len(up.users) != 1 or len(gate.users) != 1:
        return None
    silu = next(iter(gate.users))
    if not (silu.op == "call_function" and silu.target is F.silu) or len(silu.users) != 1:
        return None
    out = next(iter(silu.users))
    if not (out.op == "call_function" and out.target in (torch.mul, operator.mul)):
        return None
    if up not in out.all_input_nodes or next(iter(up.users)) is not out:
        return None
    return out


def replace_swiglu_unchunked(gm: GraphModule, node: Node) -> None:
    if not _is_chunk_in_two_on_last_dim(node):
        return
    out = _match_swiglu(node)
    if out is None:
        return
    x = node.kwargs.get("input", node.args[0])
    with gm.graph.inserting_after(out):
        new_node = gm.graph.call_function(swiglu_packed_cute, args=(x,))
    out.replace_all_uses_with(new_node)
    gm.graph.eliminate_dead_code()
    gm.recompile()


def replace_rmsnorm(gm: GraphModule, node: Node) -> None:
    """``rms_norm`` over the last dimension -> ``rmsnorm_cute``.  Arguments may arrive positionally or by keyword
    (``input``, ``normalized_shape``, ``weight``, ``eps``); a normalized_shape of more than one dimension is left alone."""
    if not (node.op == "call_function" and node.target in (torch.rms_norm, F.rms_norm)):
        return
    names = ("input", "normalized_shape", "weight", "eps")
    bound = dict(zip(names, node.args))
    bound.update(node.kwargs)
    shape = bound.get("normalized_shape")
    if "input" not in bound or shape is None or len(shape) != 1:
        return
    with gm.graph.inserting_after(node):
        new_node = gm.graph.call_function(rmsnorm_cute, args=(bound["input"], bound.get("weight"), bound.get("eps")))
    node.replace_all_uses_with(new_node)
    gm.graph.erase_node(node)
    gm.recompile()


class CuteInductor:
    def __init__(self, use_torch_inductor_after_cute_inductor: bool = True,
                 replace_functions: list[Callable] | None = None) -> None:
        self.use_torch_inductor_after_cute_inductor = use_torch_inductor_after_cute_inductor
        self.replace_functions = [replace_rmsnorm, replace_swiglu_unchunked] if replace_functions is None else replace_functions

    def compiler(self, gm: GraphModule, example_inputs: list[torch.Tensor]) -> Callable:
        if _DEBUG_CUTEINDUCTOR:
            print("graph before cute inductor")
            gm.print_readable()
        for replace_function in self.replace_functions:
            for node in list(gm.graph.nodes):
                replace_function(gm, node)
        if _DEBUG_CUTEINDUCTOR:
            print("graph after cute inductor")
            gm.print_readable()
        if self.use_torch_inductor_after_cute_inductor:
            # inductor re-traces the rewritten graph with fake tensors: the kernels must appear as opaque custom ops
            # (the reference wraps this call in enable_cute_tracing(), cute_inductor/compiler.py:28)
            with _lib.tracing():
                return lookup_backend("inductor")(gm, example_inputs)
        return gm.forward
