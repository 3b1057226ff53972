"""Host-side logic that needs no GPU: API surface, FX rewrite, state_dict compatibility, argument checks."""

import pytest
import torch
import torch.nn.functional as F

import ck_oracle as orc


def test_public_names_of_the_reference_surface():
    import cute_kernels as ck

    for name in ("MoE_Cute", "MoE_Torch", "MoE_Triton", "continuous_count_cute", "continuous_count_torch", "swiglu_cute",
                 "swiglu_torch", "swiglu_packed_cute", "swiglu_packed_torch", "rmsnorm_cute", "rmsnorm_torch",
                 "fused_residual_add_rmsnorm_cute", "fused_residual_add_rmsnorm_torch", "CuteInductor", "KernelBackend",
                 "CutoTuneParameter", "set_seed", "ceil_divide"):
        assert hasattr(ck, name), name
    assert ck.ceil_divide(7, 2) == 4
    assert ck.KernelBackend.cuda.value == "cuda" and ck.KernelBackend.triton.value == "triton"
    assert ck.MoE_Triton is ck.MoE_Cute


def test_torch_named_counterparts_match_the_oracle():
    """The eager-PyTorch functions exported under the reference's ``*_torch`` names agree with the oracle (which is
    pinned to the reference's outputs) and share MoE_Cute's state_dict layout."""
    import cute_kernels as ck

    g = torch.Generator().manual_seed(0)
    gate, up = torch.randn(5, 12, generator=g), torch.randn(5, 12, generator=g)
    assert torch.equal(ck.swiglu_torch(gate, up), orc.swiglu_ref(gate, up))
    assert torch.equal(ck.swiglu_packed_torch(torch.cat([up, gate], -1)), orc.swiglu_ref(gate, up))
    ids = torch.randint(0, 9, (100,), generator=g)
    assert ck.continuous_count_torch(ids, 9).tolist() == orc.continuous_count_ref(ids.numpy(), 9).tolist()
    w = torch.randn(12, generator=g)
    torch.testing.assert_close(ck.rmsnorm_torch(gate, w, 1e-5), orc.rmsnorm_ref(gate, w, 1e-5))
    z, r = ck.fused_residual_add_rmsnorm_torch(gate, up, w, 1e-5, 0.9)
    ze, r_e = orc.fused_residual_add_rmsnorm_ref(gate, up, w, 1e-5, 0.9)
    torch.testing.assert_close(z, ze)
    assert torch.equal(r, r_e)
    inp = orc.gen_moe_inputs(2, T=40, H=16, I=24, E=4, k=2)
    m = ck.MoE_Torch(4, 2, 16, 24, ck.swiglu_packed_torch, True, False, 0.02)
    with torch.no_grad():
        m.c_fc.weight.copy_(inp["w_fc"])
        m.c_proj.weight.copy_(inp["w_proj"])
    y = m._compute_experts(inp["x"], inp["router_weights"], inp["selected_experts"])
    ref = orc.moe_experts_ref(inp["x"], inp["router_weights"], inp["selected_experts"], inp["w_fc"], inp["w_proj"], orc.swiglu_packed_ref)
    torch.testing.assert_close(y, ref, rtol=1e-5, atol=1e-6)
    cute = ck.MoE_Cute(4, 2, 16, 24, ck.swiglu_packed_cute, True, False, 0.02)
    cute.load_state_dict(m.state_dict())
    out, logits = m(inp["x"].view(2, 20, 16))
    assert out.shape == (2, 20, 16) and logits.shape == (40, 4)


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
    assert mk(nn.GELU(approximate="tanh"), False) == 2   # the reference tests' un-gated activation is fused too
    assert mk(nn.GELU(), False) is None                  # exact (erf) GELU: un-fused
    assert mk(nn.GELU(approximate="tanh"), True) is None
    assert mk(ck.swiglu_packed_cute, True, bias=True) == 0  # biases ride in the GEMM epilogues


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
    assert ci.replace_functions == [ck.replace_rmsnorm, ck.replace_swiglu_unchunked]
    gm = torch.fx.symbolic_trace(_swiglu_module)
    fwd = ci.compiler(gm, [torch.randn(2, 8)])
    assert callable(fwd)
    assert any(n.target is ck.swiglu_packed_cute for n in gm.graph.nodes)


def test_cute_inductor_rewrites_rms_norm():
    import cute_kernels as ck

    def block(x, w):
        return F.rms_norm(x, (x.size(-1),), weight=w, eps=1e-5) + 1.0

    def two_dims(x):
        return F.rms_norm(x, x.shape[-2:])

    gm = torch.fx.symbolic_trace(lambda x, w: torch.rms_norm(x, [16], w, 1e-5) + 1.0)
    for node in list(gm.graph.nodes):
        ck.replace_rmsnorm(gm, node)
    targets = [n.target for n in gm.graph.nodes if n.op == "call_function"]
    assert ck.rmsnorm_cute in targets and torch.rms_norm not in targets
    new = next(n for n in gm.graph.nodes if n.target is ck.rmsnorm_cute)
    assert len(new.args) == 3 and new.args[2] == 1e-5  # (x, weight, eps): normalized_shape dropped

    # through dynamo: the rewritten graph reaches this library's op, which refuses CPU tensors loudly
    seen = []

    def backend(gm, example_inputs):
        for node in list(gm.graph.nodes):
            ck.replace_rmsnorm(gm, node)
        seen.extend(n.target for n in gm.graph.nodes if n.op == "call_function")
        return gm.forward

    torch._dynamo.reset()
    f = torch.compile(block, backend=backend)
    with pytest.raises(RuntimeError, match="no CPU path"):
        f(torch.randn(4, 16), torch.randn(16))
    assert ck.rmsnorm_cute in seen

    gm2 = torch.fx.symbolic_trace(lambda x: torch.rms_norm(x, [4, 16]))
    before = [n.target for n in gm2.graph.nodes]
    for node in list(gm2.graph.nodes):
        ck.replace_rmsnorm(gm2, node)
    assert [n.target for n in gm2.graph.nodes] == before  # two normalized dims: left alone


def test_cute_inductor_with_inductor_reaches_the_custom_op_on_cpu():
    """With ``use_torch_inductor_after_cute_inductor=True`` the rewritten graph is re-traced by inductor with fake
    tensors: the kernels must be recorded as opaque custom ops.  On a CPU tensor the compiled function then fails at
    run time inside this library (there is no CPU path), not at trace time."""
    import cute_kernels as ck

    torch._dynamo.reset()
    ci = ck.CuteInductor(use_torch_inductor_after_cute_inductor=True)
    f = torch.compile(_swiglu_module, backend=ci.compiler)
    with pytest.raises(RuntimeError, match="no CPU path"):
        f(torch.randn(8, 16, requires_grad=True))


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


def test_balanced_expert_placement_and_state_dict_round_trip():
    import cute_kernels as ck
    from cute_kernels.expert_parallel import shard_expert_state_dict

    loads = [100, 5, 5, 5, 90, 5, 5, 80]
    placement = ck.balanced_expert_placement(loads, 4)
    assert sorted(placement.count(r) for r in range(4)) == [2, 2, 2, 2]
    per_rank = [sum(l for l, r in zip(loads, placement) if r == g) for g in range(4)]
    assert max(per_rank) == 105                      # contiguous blocks would give 105, 10, 95, 85: same bound here ...
    assert max(per_rank) - min(per_rank) <= 100      # ... but the heavy experts land on different ranks
    assert len({placement[0], placement[4], placement[7]}) == 3
    skew = [64, 32, 16, 8, 4, 2, 1, 1]
    pl = ck.balanced_expert_placement(skew, 2)
    assert max(sum(l for l, r in zip(skew, pl) if r == g) for g in range(2)) < sum(skew[:4])
    with pytest.raises(ValueError):
        ck.balanced_expert_placement([1, 2, 3], 2)
    sd = {"gate.weight": torch.zeros(8, 4), "c_fc.weight": torch.arange(8.0).view(8, 1, 1).expand(8, 2, 3).contiguous()}
    for g in range(4):
        local = shard_expert_state_dict(sd, g, 4, placement)
        assert local["c_fc.weight"][:, 0, 0].tolist() == [float(e) for e in range(8) if placement[e] == g]


def test_bench_reference_arm_prints_the_contract_line():
    """`bench.py --impl reference` needs no GPU: it times the CPU port on a bounded sample and prints one JSON line with the
    keys the GPU arm's line carries."""
    import json
    import os
    import subprocess
    import sys

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    out = subprocess.run([sys.executable, os.path.join(root, "bench.py"), "--impl", "reference", "--steps", "1", "--warmup", "0"],
                         capture_output=True, text=True, timeout=600, check=True).stdout.strip().splitlines()
    assert len(out) == 1
    line = json.loads(out[0])
    assert line["impl"] == "reference" and line["metric"] == "moe_fwd_bwd_tokens_per_s" and line["unit"] == "tokens/s"
    assert line["higher_is_better"] is True and line["steps"] == 1 and line["value"] > 0
    assert line["config"]["workload"] == "c4_mixtral_moe_fwd_bwd"
    cpu = line["cpu_baseline"]
    assert cpu["kind"] == "port" and cpu["cores"] >= 1 and cpu["value"] == line["value"] and "sample" in cpu
    assert line["e2e"] == {"value": line["value"], "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}
