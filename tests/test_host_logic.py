"""Host-side logic that needs no GPU: API surface, FX rewrite, state_dict compatibility, argument checks."""

import pytest
import torch
import torch.nn.functional as F

import ck_oracle as orc


def test_public_names_of_the_reference_surface():
    import cute_kernels as ck

    for name in ("MoE_Cute", "continuous_count_cute", "swiglu_cute", "swiglu_packed_cute", "CuteInductor",
                 "KernelBackend", "CutoTuneParameter", "set_seed", "ceil_divide"):
        assert hasattr(ck, name), name
    assert ck.ceil_divide(7, 2) == 4
    assert ck.KernelBackend.cuda.value == "cuda" and ck.KernelBackend.triton.value == "triton"


def test_state_dict_is_interchangeable_with_the_reference_layout():
    import cute_kernels as ck

    m = ck.MoE_Cute(8, 2, 64, 128, ck.swiglu_packed_cute, True, False, 0.02)
    sd = m.state_dict()
    assert {k: tuple(v.shape) for k, v in sd.items()} == {
        "gate.weight": (8, 64), "c_fc.weight": (8, 256, 64), "c_proj.weight": (8, 64, 128)}
    r = orc.MoERef(8, 2, 64, 128, orc.swiglu_packed_ref, True, False, 0.02)
    r.load_state_dict(sd)
    m.load_state_dict(r.state_dict())
    mb = ck.MoE_Cute(4, 2, 64, 128, F.gelu, False, True, 0.02)
    assert {k: tuple(v.shape) for k, v in mb.state_dict().items()} == {
        "gate.weight": (4, 64), "c_fc.weight": (4, 128, 64), "c_fc.bias": (4, 128), "c_proj.weight": (4, 64, 128),
        "c_proj.bias": (4, 64)}
    assert abs(m.c_fc.weight.std().item() - 0.02) < 2e-3


def test_fused_path_selection():
    import torch.nn as nn

    import cute_kernels as ck

    mk = lambda act, glu, bias=False: ck.MoE_Cute(4, 2, 64, 64, act, glu, bias, 0.02)._act_kind  # noqa: E731
    assert mk(ck.swiglu_packed_cute, True) == 0
    assert mk(orc.swiglu_packed_ref, True) is None  # unknown callables run un-fused
    assert mk(nn.GLU(), True) == 1
    assert mk(nn.GELU(approximate="tanh"), False) is None
    assert mk(ck.swiglu_packed_cute, True, bias=True) is None


def test_ops_refuse_cpu_tensors():
    import cute_kernels as ck

    x = torch.randn(8, 8)
    with pytest.raises(RuntimeError, match="CUDA tensors only"):
        ck.swiglu_cute(x, x)
    with pytest.raises(RuntimeError, match="CUDA tensors only"):
        ck.swiglu_packed_cute(x)
    with pytest.raises(RuntimeError):
        ck.continuous_count_cute(torch.zeros(10, dtype=torch.int64), 4)


def test_kernel_backend_arguments():
    import cute_kernels as ck
    from cute_kernels.kernel_backend import resolve_backend

    resolve_backend(None)
    resolve_backend(ck.CutoTuneParameter())
    resolve_backend(ck.KernelBackend.cuda)
    with pytest.raises(ValueError):
        resolve_backend(ck.KernelBackend.triton)
    with pytest.raises(ValueError):
        resolve_backend("cuda")


def _swiglu_module(x):
    up, gate = x.chunk(2, dim=-1)
    return up * F.silu(gate)


def test_cute_inductor_rewrites_chunk_silu_mul():
    import cute_kernels as ck

    gm = torch.fx.symbolic_trace(_swiglu_module)
    for node in list(gm.graph.nodes):
        ck.replace_swiglu_unchunked(gm, node)
    targets = [n.target for n in gm.graph.nodes if n.op == "call_function"]
    assert targets == [ck.swiglu_packed_cute]


def test_cute_inductor_leaves_other_graphs_alone():
    import cute_kernels as ck

    def not_swiglu(x):
        a, b = x.chunk(2, dim=-1)
        return a * F.silu(b) + b  # gate has a second user

    def wrong_dim(x):
        a, b = x.chunk(2, dim=0)
        return a * F.silu(b)

    for fn in (not_swiglu, wrong_dim):
        gm = torch.fx.symbolic_trace(fn)
        before = [n.target for n in gm.graph.nodes]
        for node in list(gm.graph.nodes):
            ck.replace_swiglu_unchunked(gm, node)
        assert [n.target for n in gm.graph.nodes] == before


def test_cute_inductor_class_shell():
    import cute_kernels as ck

    ci = ck.CuteInductor(use_torch_inductor_after_cute_inductor=False)
    assert ci.replace_functions == [ck.replace_swiglu_unchunked]
    gm = torch.fx.symbolic_trace(_swiglu_module)
    fwd = ci.compiler(gm, [torch.randn(2, 8)])
    assert callable(fwd)
    assert any(n.target is ck.swiglu_packed_cute for n in gm.graph.nodes)


def test_padded_capacity_bounds_every_routing():
    import numpy as np

    import cute_kernels as ck

    rng = np.random.default_rng(0)
    for _ in range(200):
        E = int(rng.integers(1, 40))
        n = int(rng.integers(0, 5000))
        ids = rng.integers(0, E, size=n)
        r = orc.route_ref(ids, E)
        assert r["padded_off"][-1] <= ck.padded_capacity(n, E) == r["row_map"].size


def test_route_workspace_bytes_mirror_matches_the_library():
    from cute_kernels import _lib
    from cute_kernels.routing import route_workspace_bytes

    for n in (0, 1, 255, 256, 257, 4096, 4097, 32768, 262144, 1 << 20, (1 << 24) + 5, (1 << 27) + 1):
        for E in (1, 8, 64, 72, 1024):
            assert route_workspace_bytes(n, E) == _lib.lib.ck_route_workspace_bytes(n, E), (n, E)


def test_module_traces_under_fullgraph_compile_without_graph_breaks():
    """Dynamo must trace MoE_Cute end to end (custom ops stay opaque).  On a CPU-only machine the trace
    succeeds and the first kernel call then refuses the CPU tensors."""
    import cute_kernels as ck

    m = ck.MoE_Cute(4, 2, 64, 64, ck.swiglu_packed_cute, True, False, 0.02)
    mod = torch.compile(m, fullgraph=True, backend="eager")
    x = torch.randn(16, 64, requires_grad=True)
    if torch.cuda.is_available():
        y, _ = mod.cuda()(x.cuda())
        assert y.shape == (16, 64)
    else:
        try:
            with pytest.raises(RuntimeError, match="CUDA tensors only"):
                mod(x)
        finally:
            # the refusal interrupts the traced graph inside route()'s no_grad region: restore grad mode
            torch.set_grad_enabled(True)
