"""The oracle against the golden vectors produced by the reference's own torch path (CPU only)."""

import os

import numpy as np
import pytest
import torch

import ck_oracle as orc


@pytest.fixture(scope="module")
def routing(golden_dir):
    return np.load(os.path.join(golden_dir, "routing.npz"))


@pytest.mark.parametrize("name", ["u72_i64", "u72_i32", "zipf64", "tiny"])
def test_routing_oracle_matches_reference(routing, name):
    n, E, dist, isz = routing[f"{name}_meta"]
    ids = orc.gen_ids(7, int(n), int(E), "zipf" if dist else "uniform", np.int64 if isz == 8 else np.int32)
    assert np.array_equal(orc.continuous_count_ref(ids, int(E)), routing[f"{name}_counts"])
    r = orc.route_ref(ids, int(E))
    assert np.array_equal(r["sorted_idx"], routing[f"{name}_sorted_idx"])
    assert np.array_equal(r["end_off"], routing[f"{name}_end_off"])
    assert np.array_equal(r["excl_off"], routing[f"{name}_end_off"] - r["counts"].astype(np.int32))
    # padded layout is self-consistent
    valid = r["row_map"][r["row_map"] >= 0]
    assert np.array_equal(valid, r["sorted_idx"])
    assert np.all(r["padded_off"] % orc.TILE_M == 0) and r["padded_off"][-1] <= r["row_map"].size


def test_count_ignores_out_of_range():
    x = np.array([0, 5, -1, 9, 3, 3, 100], dtype=np.int64)
    assert orc.continuous_count_ref(x, 6).tolist() == [1, 0, 0, 2, 0, 1]


@pytest.mark.parametrize("name,dt", [("f32", torch.float32), ("bf16", torch.bfloat16), ("f16", torch.float16)])
def test_swiglu_oracle_matches_reference(golden_dir, name, dt):
    g = np.load(os.path.join(golden_dir, "swiglu.npz"))
    t = lambda k: torch.from_numpy(g[f"{name}_{k}"]).to(dt)  # noqa: E731
    gate, up, dy = t("gate"), t("up"), t("dy")
    assert torch.equal(orc.swiglu_ref(gate, up), t("out"))
    assert torch.equal(orc.swiglu_packed_ref(torch.cat([up, gate], -1)), t("packed_out"))
    dgate, dup = orc.swiglu_backward_ref(gate, up, dy)
    # the reference backward is autograd of the fp32 formula: equal up to one rounding of the output dtype
    tol = dict(rtol=0, atol=5e-6) if dt == torch.float32 else dict(rtol=1.6e-2, atol=1e-5)
    torch.testing.assert_close(dgate, t("dgate"), **tol)
    torch.testing.assert_close(dup, t("dup"), **tol)
    pdx = t("packed_dx")
    torch.testing.assert_close(torch.cat([dup, dgate], -1), pdx, **tol)


@pytest.mark.parametrize("name", ["small", "skew", "c1"])
def test_moe_oracle_matches_reference(golden_dir, name):
    g = np.load(os.path.join(golden_dir, "moe.npz"))
    seed, T, H, I, E, k, bias = (int(v) for v in g[f"{name}_cfg"])
    inp = orc.gen_moe_inputs(seed, T, H, I, E, k, bool(bias))
    res = orc.moe_fwd_bwd_ref(inp)
    for key, v in res.items():
        v = v.float()
        s = np.array([v.double().sum().item(), v.double().abs().sum().item(), v.double().pow(2).sum().item()])
        np.testing.assert_allclose(s, g[f"{name}_{key}_sum"], rtol=1e-5, atol=1e-6, err_msg=key)
        if f"{name}_{key}" in g:
            np.testing.assert_allclose(v.numpy(), g[f"{name}_{key}"], rtol=1e-5, atol=2e-6, err_msg=key)
        else:
            flat = v.reshape(-1)
            stride = max(1, flat.numel() // 4096)
            np.testing.assert_allclose(flat[::stride][:4096].numpy(), g[f"{name}_{key}_sample"], rtol=1e-5, atol=2e-6, err_msg=key)


@pytest.mark.parametrize("name", ["small", "skew"])
def test_moe_module_oracle_matches_reference_module(golden_dir, name):
    g = np.load(os.path.join(golden_dir, "moe.npz"))
    seed, T, H, I, E, k, bias = (int(v) for v in g[f"{name}_cfg"])
    inp = orc.gen_moe_inputs(seed, T, H, I, E, k, bool(bias))
    m = orc.MoERef(E, k, H, I, orc.swiglu_packed_ref, True, False, 0.02)
    with torch.no_grad():
        m.c_fc.weight.copy_(inp["w_fc"])
        m.c_proj.weight.copy_(inp["w_proj"])
        m.gate.weight.copy_(torch.from_numpy(g[f"{name}_module_gate_w"]))
        y, logits = m(inp["x"])
    np.testing.assert_allclose(logits.numpy(), g[f"{name}_module_logits"], rtol=1e-5, atol=1e-6)
    np.testing.assert_allclose(y.numpy(), g[f"{name}_module_y"], rtol=1e-5, atol=2e-6)


def _rmsnorm_case(g, name, dt):
    t = lambda k: torch.from_numpy(g[f"{name}_{k}"]).to(dt)  # noqa: E731
    mult, has_w = g[f"{name}_meta"]
    return t, (None if mult == 0 else float(mult)), bool(has_w)


@pytest.mark.parametrize("name,dt", [("f32_w", torch.float32), ("f32_now", torch.float32), ("bf16_w", torch.bfloat16),
                                     ("f16_w", torch.float16)])
def test_rmsnorm_oracle_matches_reference(golden_dir, name, dt):
    """rmsnorm_torch / fused_residual_add_rmsnorm_torch of the reference, forward and autograd backward."""
    g = np.load(os.path.join(golden_dir, "rmsnorm.npz"))
    t, mult, has_w = _rmsnorm_case(g, name, dt)
    x = t("x").requires_grad_()
    w = t("w").requires_grad_() if has_w else None
    z = orc.rmsnorm_ref(x, w, 1e-5)
    z.sum().backward()
    exact = dt == torch.float32
    tol = dict(rtol=0, atol=2e-6) if exact else dict(rtol=1.6e-2, atol=1e-5)
    assert torch.equal(z.detach(), t("z")) if not exact else torch.allclose(z.detach(), t("z"), rtol=0, atol=1e-6)
    torch.testing.assert_close(x.grad, t("dx"), **tol)
    if has_w:
        torch.testing.assert_close(w.grad, t("dw"), rtol=tol["rtol"], atol=max(tol["atol"], 2e-5))
    x2 = t("x").requires_grad_()
    res = t("res").requires_grad_()
    w2 = t("w").requires_grad_() if has_w else None
    z2, r2 = orc.fused_residual_add_rmsnorm_ref(x2, res, w2, 1e-5, mult)
    (z2 * 2 + r2 * 3).sum().backward()
    assert torch.equal(r2.detach(), t("fr"))
    assert torch.equal(z2.detach(), t("fz")) if not exact else torch.allclose(z2.detach(), t("fz"), rtol=0, atol=1e-6)
    torch.testing.assert_close(x2.grad, t("fdx"), **tol)
    torch.testing.assert_close(res.grad, t("fdres"), **tol)
    if has_w:
        torch.testing.assert_close(w2.grad, t("fdw"), rtol=tol["rtol"], atol=max(tol["atol"], 4e-5))
