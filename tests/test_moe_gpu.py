"""MoE_Cute / fused_experts on the GPU against the CPU oracle and the reference's golden vectors."""

import os

import numpy as np
import pytest
import torch
import torch.nn as nn

import ck_oracle as orc

pytestmark = pytest.mark.gpu

# bf16 outputs and gradients within rtol 2e-2 / atol 2e-2 of the fp32 oracle; fp32 (TF32 tensor cores) and fp16
# use the forward tolerances of the reference's MoE test (tests/kernels/scattermoe_test.py:102-127)
TOL = {torch.bfloat16: dict(rtol=2e-2, atol=2e-2), torch.float16: dict(rtol=4e-3, atol=4e-3),
       torch.float32: dict(rtol=6e-3, atol=6e-3)}


def _run_fused(inp, dtype, act_kind=0):
    from cute_kernels import fused_experts

    x = inp["x"].to(dtype).cuda().requires_grad_()
    rw = inp["router_weights"].to(dtype).cuda().requires_grad_()
    w_fc = inp["w_fc"].to(dtype).cuda().requires_grad_()
    w_proj = inp["w_proj"].to(dtype).cuda().requires_grad_()
    k = inp["selected_experts"].size(1)
    y = fused_experts(x, rw, inp["selected_experts"].cuda(), w_fc, w_proj, k, act_kind)
    y.backward(inp["grad_out"].to(dtype).cuda())
    return dict(y=y.detach(), dx=x.grad, d_router_weights=rw.grad, d_w_fc=w_fc.grad, d_w_proj=w_proj.grad)


def _compare(res, ref, dtype, T):
    inter = res["d_w_proj"].size(-1)
    for key in ("y", "dx", "d_router_weights", "d_w_fc", "d_w_proj"):
        tol = dict(TOL[dtype])
        if key.startswith("d_w"):
            # weight grads sum over the tokens of an expert: absolute error grows with sqrt(rows)
            tol["atol"] = tol["atol"] * max(1.0, (T / 64) ** 0.5)
        if key == "d_router_weights":
            # a dot product over the intermediate size of O(1) terms rounded to the 16-bit dtype
            tol["atol"] = tol["atol"] * max(1.0, (inter / 256) ** 0.5)
        a, b = res[key].float().cpu(), ref[key].float()
        assert a.shape == b.shape, key
        torch.testing.assert_close(a, b, **tol, msg=lambda m, key=key: f"{key}: {m}")


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32, torch.float16])
def test_c1_config_against_fp32_oracle(dtype):
    """512 tokens, hidden 256, intermediate 512, 8 experts, top-2, seed 0: fwd + all five gradients."""
    c = orc.CONFIGS["c1_cpu"]
    inp = orc.gen_moe_inputs(0, **c)
    ref = orc.moe_fwd_bwd_ref(inp)  # fp32 gold on CPU
    res = _run_fused(inp, dtype)
    _compare(res, ref, dtype, c["T"])


@pytest.mark.parametrize("name", ["small", "skew", "c1"])
def test_against_reference_golden(golden_dir, name):
    """Outputs of the reference's MoE_Torch (fp32) stored by tests/golden/make_golden.py."""
    g = np.load(os.path.join(golden_dir, "moe.npz"))
    seed, T, H, I, E, k, bias = (int(v) for v in g[f"{name}_cfg"])
    inp = orc.gen_moe_inputs(seed, T, H, I, E, k, bool(bias))
    res = _run_fused(inp, torch.bfloat16)
    for key, v in res.items():
        v = v.float().cpu()
        if f"{name}_{key}" in g:
            exp, got = torch.from_numpy(g[f"{name}_{key}"]), v
        else:
            flat = v.reshape(-1)
            stride = max(1, flat.numel() // 4096)
            exp, got = torch.from_numpy(g[f"{name}_{key}_sample"]), flat[::stride][:4096]
        tol = dict(TOL[torch.bfloat16])
        if key.startswith("d_w"):
            tol["atol"] *= max(1.0, (T / 64) ** 0.5)
        torch.testing.assert_close(got, exp, **tol, msg=lambda m, key=key: f"{key}: {m}")


@pytest.mark.parametrize("case", [dict(T=1, H=64, I=64, E=4, k=2), dict(T=3, H=576, I=256, E=128, k=8),
                                  dict(T=700, H=128, I=200, E=6, k=4), dict(T=257, H=64, I=72, E=3, k=1),
                                  dict(T=1024, H=512, I=1408, E=16, k=8, expert_bias=True)])
def test_ragged_and_edge_shapes(case):
    """One token (the reference's only MoE test input), many experts, k == 1, N tails, skewed routing."""
    inp = orc.gen_moe_inputs(1, **case)
    ref = orc.moe_fwd_bwd_ref(inp)
    res = _run_fused(inp, torch.bfloat16)
    _compare(res, ref, torch.bfloat16, case["T"])


def test_tma_gather_flavour_matches(monkeypatch):
    """The whole fused layer with every permutation done by TMA gather4 inside the GEMMs."""
    import cute_kernels.moe as moe

    inp = orc.gen_moe_inputs(6, T=700, H=128, I=200, E=6, k=4)
    base = _run_fused(inp, torch.bfloat16)
    monkeypatch.setattr(moe, "TMA_GATHER", True)
    got = _run_fused(inp, torch.bfloat16)
    for key in ("y", "dx", "d_w_fc", "d_w_proj"):
        torch.testing.assert_close(got[key].float(), base[key].float(), rtol=1e-2, atol=1e-3, msg=lambda m, key=key: f"{key}: {m}")
    ref = orc.moe_fwd_bwd_ref(inp)
    _compare(got, ref, torch.bfloat16, 700)


def test_glu_activation_fused():
    inp = orc.gen_moe_inputs(2, T=300, H=128, I=256, E=4, k=2)
    glu = lambda t: t[..., : t.size(-1) // 2] * torch.sigmoid(t[..., t.size(-1) // 2 :])  # noqa: E731
    ref = orc.moe_fwd_bwd_ref(inp, activation=glu)
    res = _run_fused(inp, torch.bfloat16, act_kind=1)
    _compare(res, ref, torch.bfloat16, 300)


def test_run_to_run_determinism_top2():
    """k == 2: the fp32 combine adds two values per element, so results are bit-reproducible; the router-weight
    gradient is summed from per-tile partial sums in a fixed order."""
    inp = orc.gen_moe_inputs(3, T=512, H=256, I=1024, E=8, k=2)
    a = _run_fused(inp, torch.bfloat16)
    b = _run_fused(inp, torch.bfloat16)
    for key in ("y", "dx", "d_router_weights", "d_w_fc", "d_w_proj"):
        assert torch.equal(a[key], b[key]), key


def test_deterministic_option_top8():
    """k > 2 with ``deterministic=True``: the k rows of a token are stored un-combined and summed in a fixed order, so
    every output is bit-reproducible; the values still match the oracle."""
    from cute_kernels import fused_experts

    cfg = dict(T=600, H=256, I=384, E=16, k=8, expert_bias=True)
    inp = orc.gen_moe_inputs(8, **cfg)
    outs = []
    for _ in range(3):
        x = inp["x"].bfloat16().cuda().requires_grad_()
        rw = inp["router_weights"].bfloat16().cuda().requires_grad_()
        w_fc = inp["w_fc"].bfloat16().cuda().requires_grad_()
        w_proj = inp["w_proj"].bfloat16().cuda().requires_grad_()
        y = fused_experts(x, rw, inp["selected_experts"].cuda(), w_fc, w_proj, 8, deterministic=True)
        y.backward(inp["grad_out"].bfloat16().cuda())
        outs.append(dict(y=y.detach(), dx=x.grad, d_router_weights=rw.grad, d_w_fc=w_fc.grad, d_w_proj=w_proj.grad))
    for key in outs[0]:
        assert torch.equal(outs[0][key], outs[1][key]) and torch.equal(outs[0][key], outs[2][key]), key
    _compare(outs[0], orc.moe_fwd_bwd_ref(inp), torch.bfloat16, cfg["T"])


@pytest.mark.parametrize("case", [dict(T=700, H=128, I=200, E=6, k=4), dict(T=1024, H=512, I=1408, E=16, k=8, expert_bias=True),
                                  dict(T=130, H=72, I=64, E=3, k=1)])
def test_gather_modes_agree(monkeypatch, case):
    """Rows read by the GEMM's own producer warps ("producer", with the grouped copy written back for the weight
    gradients) against rows gathered by the separate streaming kernel ("kernel"): the same bits everywhere."""
    import cute_kernels.moe as moe

    inp = orc.gen_moe_inputs(6, **case)
    monkeypatch.setattr(moe, "GATHER_MODE", "kernel")
    base = _run_fused(inp, torch.bfloat16)
    monkeypatch.setattr(moe, "GATHER_MODE", "producer")
    got = _run_fused(inp, torch.bfloat16)
    keys = ("y", "dx", "d_router_weights", "d_w_fc", "d_w_proj") if case["k"] <= 2 else ("d_router_weights", "d_w_fc", "d_w_proj")
    for key in keys:
        assert torch.equal(got[key], base[key]), key
    for key in ("y", "dx"):  # k > 2: the fp32 combine order is not fixed
        torch.testing.assert_close(got[key].float(), base[key].float(), rtol=1e-2, atol=1e-3)
    _compare(got, orc.moe_fwd_bwd_ref(inp), torch.bfloat16, case["T"])


def _modules(E, k, H, I, act_cute, act_ref, is_glu, dtype, add_bias=False):
    from cute_kernels import MoE_Cute

    torch.manual_seed(42)
    m = MoE_Cute(E, k, H, I, act_cute, is_glu, add_bias, 0.02).to(dtype).cuda()
    r = orc.MoERef(E, k, H, I, act_ref, is_glu, add_bias, 0.02)
    if add_bias:
        with torch.no_grad():
            m.c_fc.bias.normal_(0, 0.02)
            m.c_proj.bias.normal_(0, 0.02)
    r.load_state_dict({k_: v.float().cpu() for k_, v in m.state_dict().items()})  # same keys and shapes
    return m, r


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("compiled", [False, True])
def test_module_swiglu_end_to_end(dtype, compiled):
    from cute_kernels import swiglu_packed_cute

    m, r = _modules(8, 2, 256, 512, swiglu_packed_cute, orc.swiglu_packed_ref, True, dtype)
    mod = torch.compile(m, fullgraph=True) if compiled else m
    g = torch.Generator().manual_seed(9)
    x = torch.randn(4, 96, 256, generator=g)
    xk = x.to(dtype).cuda().requires_grad_()
    xr = x.to(dtype).float().requires_grad_()
    y, logits = mod(xk)
    # the 16-bit router may break near-ties differently from the fp32 oracle: pin the oracle to the same experts
    sel = m._compute_routing_weights(xk.detach().view(-1, 256))[2].cpu()
    yr, logits_r = r(xr, forced_selection=sel)
    assert y.shape == xk.shape and logits.shape == (4 * 96, 8)
    torch.testing.assert_close(logits.float().cpu(), logits_r, rtol=2e-2, atol=2e-2)
    torch.testing.assert_close(y.float().cpu(), yr, **TOL[dtype])
    y.sum().backward()
    yr.sum().backward()
    tol = dict(rtol=4e-2, atol=4e-2) if dtype == torch.bfloat16 else TOL[dtype]  # reference dgrad tolerance for bf16
    torch.testing.assert_close(xk.grad.float().cpu(), xr.grad, **tol)
    torch.testing.assert_close(m.gate.weight.grad.float().cpu(), r.gate.weight.grad, rtol=5e-2, atol=5e-2)


@pytest.mark.parametrize("E,k,H,I", [(2, 2, 256, 512), (8, 4, 256, 512), (128, 8, 576, 256)])
@pytest.mark.parametrize("is_glu", [True, False])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
def test_reference_test_matrix(E, k, H, I, is_glu, dtype):
    """The reference's own MoE test (tests/kernels/scattermoe_test.py:16-127): nn.GLU / GELU(tanh) activations,
    one-token input, forward and input-gradient tolerances of that file (hidden sizes scaled down to keep
    the CPU oracle fast; the 128-expert shape is the reference's)."""
    act = nn.GLU() if is_glu else nn.GELU(approximate="tanh")
    m, r = _modules(E, k, H, I, act, act, is_glu, dtype)
    g = torch.Generator().manual_seed(42)
    x = torch.randn(H, generator=g)
    xk = x.to(dtype).cuda().requires_grad_()
    xr = x.to(dtype).float().requires_grad_()
    (y, _), names = _launch_names(lambda: m(xk))
    combine = "down_combine_fwd" in names or ("grouped_linear_scatter" in names and "combine_rows" in names)  # red.add (k <= 2) or row store
    assert "up_act_fwd" in names and combine, f"the module did not take the fused path: {names}"
    sel = m._compute_routing_weights(xk.detach().view(-1, H))[2].cpu()
    yr = r(xr, forced_selection=sel)[0]
    fwd = {torch.float16: 4e-3, torch.bfloat16: 2e-2, torch.float32: 6e-3}[dtype]
    bwd = {torch.float16: 4e-3, torch.bfloat16: 4e-2, torch.float32: 6e-3}[dtype]
    torch.testing.assert_close(y.float().cpu(), yr, atol=fwd, rtol=0)
    y.sum().backward()
    yr.sum().backward()
    torch.testing.assert_close(xk.grad.float().cpu(), xr.grad, atol=bwd, rtol=0)


def _launch_names(fn):
    from cute_kernels import _lib

    _lib.launch_log.reset()
    _lib.launch_log.record_events = True
    try:
        out = fn()
        torch.cuda.synchronize()
        return out, [e[0] for e in _lib.launch_log.events]
    finally:
        _lib.launch_log.record_events = False
        _lib.launch_log.reset()


@pytest.mark.parametrize("act", ["swiglu", "glu", "gelu_tanh"])
@pytest.mark.parametrize("with_bias", [False, True])
@pytest.mark.parametrize("deterministic", [False, True])
def test_fused_activations_and_biases_against_oracle(act, with_bias, deterministic):
    """Every fused epilogue -- gated (SwiGLU, GLU) and un-gated (GELU-tanh, the reference tests' is_glu=False
    activation), with and without the biases of Experts_Torch -- against the fp32 oracle: outputs and every gradient,
    the bias gradients included."""
    from cute_kernels import fused_experts

    T, H, I, E, k = 333, 128, 264, 5, 3
    inp = orc.gen_moe_inputs(13, T=T, H=H, I=I, E=E, k=k, expert_bias=True)
    gelu = nn.GELU(approximate="tanh")
    glu = lambda t: t[..., : t.size(-1) // 2] * torch.sigmoid(t[..., t.size(-1) // 2 :])  # noqa: E731
    act_fn, kind = {"swiglu": (orc.swiglu_packed_ref, 0), "glu": (glu, 1), "gelu_tanh": (gelu, 2)}[act]
    w_fc = inp["w_fc"] if kind != 2 else inp["w_fc"][:, :I].contiguous()
    g = torch.Generator().manual_seed(5)
    b_fc = 0.1 * torch.randn(E, w_fc.size(1), generator=g) if with_bias else None
    b_proj = 0.1 * torch.randn(E, H, generator=g) if with_bias else None

    # the oracle sees the bf16-representable values the kernels get (bias gradients are short sums with cancellation:
    # input rounding would otherwise dominate their near-zero entries)
    leaf = lambda t: None if t is None else t.to(torch.bfloat16).float().requires_grad_()  # noqa: E731
    rx, rrw, rwf, rwp, rbf, rbp = map(leaf, (inp["x"], inp["router_weights"], w_fc, inp["w_proj"], b_fc, b_proj))
    yr = orc.moe_experts_ref(rx, rrw, inp["selected_experts"], rwf, rwp, act_fn, rbf, rbp)
    yr.backward(inp["grad_out"].to(torch.bfloat16).float())

    dt = torch.bfloat16
    dev = lambda t: None if t is None else t.to(dt).cuda().requires_grad_()  # noqa: E731
    x, rw, wf, wp, bf, bp = map(dev, (inp["x"], inp["router_weights"], w_fc, inp["w_proj"], b_fc, b_proj))
    y, names = _launch_names(lambda: fused_experts(x, rw, inp["selected_experts"].cuda(), wf, wp, k, kind, deterministic, bf, bp))
    assert "up_act_fwd" in names
    y.backward(inp["grad_out"].to(dt).cuda())
    res = dict(y=y.detach(), dx=x.grad, d_router_weights=rw.grad, d_w_fc=wf.grad, d_w_proj=wp.grad)
    ref = dict(y=yr.detach(), dx=rx.grad, d_router_weights=rrw.grad, d_w_fc=rwf.grad, d_w_proj=rwp.grad)
    _compare(res, ref, dt, T)
    if with_bias:
        tol = dict(rtol=2e-2, atol=2e-2 * max(1.0, (T / 64) ** 0.5))
        torch.testing.assert_close(bf.grad.float().cpu(), rbf.grad, **tol)
        torch.testing.assert_close(bp.grad.float().cpu(), rbp.grad, **tol)


def test_module_with_bias_takes_the_fused_path():
    act = nn.GELU(approximate="tanh")
    m, r = _modules(4, 2, 128, 256, act, act, False, torch.bfloat16, add_bias=True)
    g = torch.Generator().manual_seed(1)
    x = torch.randn(200, 128, generator=g)
    xk = x.bfloat16().cuda().requires_grad_()
    xr = x.bfloat16().float().requires_grad_()
    (y, _), names = _launch_names(lambda: m(xk))
    assert "up_act_fwd" in names and "grouped_linear" not in names, names
    sel = m._compute_routing_weights(xk.detach())[2].cpu()
    yr = r(xr, forced_selection=sel)[0]
    torch.testing.assert_close(y.float().cpu(), yr, rtol=2e-2, atol=2e-2)
    y.sum().backward()
    yr.sum().backward()
    torch.testing.assert_close(xk.grad.float().cpu(), xr.grad, rtol=4e-2, atol=4e-2)
    torch.testing.assert_close(m.c_proj.bias.grad.float().cpu(), r.c_proj.bias.grad, rtol=4e-2, atol=4e-1)


def test_arbitrary_activation_runs_unfused():
    """An activation callable without a fused epilogue (exact GELU here) still runs, on the grouped GEMM kernels with
    the activation in between as a torch op."""
    act = nn.GELU()
    m, r = _modules(4, 2, 128, 256, act, act, False, torch.bfloat16, add_bias=True)
    g = torch.Generator().manual_seed(2)
    x = torch.randn(150, 128, generator=g)
    xk = x.bfloat16().cuda().requires_grad_()
    xr = x.bfloat16().float().requires_grad_()
    (y, _), names = _launch_names(lambda: m(xk))
    assert "grouped_linear" in names and "up_act_fwd" not in names, names
    sel = m._compute_routing_weights(xk.detach())[2].cpu()
    yr = r(xr, forced_selection=sel)[0]
    torch.testing.assert_close(y.float().cpu(), yr, rtol=2e-2, atol=2e-2)
    y.sum().backward()
    yr.sum().backward()
    torch.testing.assert_close(xk.grad.float().cpu(), xr.grad, rtol=4e-2, atol=4e-2)


def test_inference_mode_skips_saved_activations():
    from cute_kernels import fused_experts

    inp = orc.gen_moe_inputs(4, T=256, H=128, I=128, E=4, k=2)
    ref = orc.moe_experts_ref(inp["x"], inp["router_weights"], inp["selected_experts"], inp["w_fc"], inp["w_proj"],
                              orc.swiglu_packed_ref)
    with torch.no_grad():
        y = fused_experts(inp["x"].bfloat16().cuda(), inp["router_weights"].bfloat16().cuda(),
                          inp["selected_experts"].cuda(), inp["w_fc"].bfloat16().cuda(), inp["w_proj"].bfloat16().cuda(), 2)
    torch.testing.assert_close(y.float().cpu(), ref, rtol=2e-2, atol=2e-2)


def test_linearity_in_grad_out_at_scale():
    """Size-independent property at a larger shape: backward is linear in grad_out (dx(2g) == 2 dx(g))."""
    from cute_kernels import fused_experts

    inp = orc.gen_moe_inputs(5, T=4096, H=1024, I=1408, E=16, k=4, expert_bias=True, dtype=torch.bfloat16)
    dev = {k_: v.cuda() for k_, v in inp.items()}
    outs = []
    for scale in (1.0, 2.0):
        x = dev["x"].clone().requires_grad_()
        w_fc = dev["w_fc"].clone().requires_grad_()
        y = fused_experts(x, dev["router_weights"], dev["selected_experts"], w_fc, dev["w_proj"], 4)
        y.backward(dev["grad_out"] * scale)
        outs.append((x.grad.float(), w_fc.grad.float()))
    torch.testing.assert_close(outs[1][0], 2 * outs[0][0], rtol=2e-2, atol=1e-3)
    torch.testing.assert_close(outs[1][1], 2 * outs[0][1], rtol=2e-2, atol=1e-3)
