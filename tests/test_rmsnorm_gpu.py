"""rmsnorm_cute / fused_residual_add_rmsnorm_cute on the GPU against the oracle and the reference's golden vectors.

Sizes, dtypes, options and tolerances follow the reference's own tests (tests/kernels/rmsnorm_test.py:17-83,
tests/kernels/fused_residual_add_rmsnorm_test.py:21-104): shapes (size,) and (400, size) for sizes around the powers
of two up to 2^14 + 9 and odd sizes near 3000, eps 1e-5, with / without weight, memory_efficient on / off, eager and
torch.compile(fullgraph=True); losses z.sum() and (2 z + 3 r).sum()."""

import os

import numpy as np
import pytest
import torch

import ck_oracle as orc

pytestmark = pytest.mark.gpu

EPS = 1e-5
SIZES = [1, 2, 7, 8, 33, 64, 100, 257, 1024, 1032, 2049, 3001, 4096, 8200, 16384, 16393]


def _shapes():
    out = []
    for s in SIZES:
        out.append((s,))
        out.append((400, s))
    return out


def _pair(shape, dtype, seed):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(shape, generator=g).to(dtype)
    return x.cuda().requires_grad_(), x.clone().requires_grad_()


@pytest.mark.parametrize("shape", _shapes())
@pytest.mark.parametrize("dtype", [torch.float32, torch.float16, torch.bfloat16])
@pytest.mark.parametrize("has_weight", [True, False])
def test_rmsnorm_matches_oracle(shape, dtype, has_weight):
    from cute_kernels import rmsnorm_cute

    for memory_efficient in (False, True):
        xk, xe = _pair(shape, dtype, 1)
        wk, we = _pair((shape[-1],), dtype, 2) if has_weight else (None, None)
        z = rmsnorm_cute(x=xk, weight=wk, eps=EPS, memory_efficient=memory_efficient)
        ze = orc.rmsnorm_ref(xe, we, EPS)
        z.sum().backward()
        ze.sum().backward()
        if dtype == torch.float32:
            torch.testing.assert_close(z.cpu(), ze, rtol=1.3e-6, atol=1e-5)
            torch.testing.assert_close(xk.grad.cpu(), xe.grad, rtol=1.3e-6, atol=1e-5)
            if has_weight:
                torch.testing.assert_close(wk.grad.cpu(), we.grad, rtol=0, atol=6.5e-5 * max(1.0, (shape[0] if len(shape) > 1 else 1) ** 0.5 / 4))
        else:
            torch.testing.assert_close(z.cpu().float(), ze.float(), rtol=0, atol=1.6e-2)
            torch.testing.assert_close(xk.grad.cpu().float(), xe.grad.float(), rtol=0, atol=9e-2)
            if has_weight:
                torch.testing.assert_close(wk.grad.cpu().float(), we.grad.float(), rtol=1e-2, atol=0.1)


@pytest.mark.parametrize("shape", [(5,), (400, 33), (400, 1024), (400, 3001), (400, 4096), (37, 16393)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("has_weight", [True, False])
@pytest.mark.parametrize("multiplier", [None, 0.9])
def test_fused_residual_add_rmsnorm_matches_oracle(shape, dtype, has_weight, multiplier):
    from cute_kernels import fused_residual_add_rmsnorm_cute

    for memory_efficient in (False, True):
        xk, xe = _pair(shape, dtype, 3)
        rk, re = _pair(shape, dtype, 4)
        wk, we = _pair((shape[-1],), dtype, 5) if has_weight else (None, None)
        z, r = fused_residual_add_rmsnorm_cute(x=xk, residual=rk, weight=wk, eps=EPS, multiplier=multiplier,
                                               memory_efficient=memory_efficient)
        ze, r_e = orc.fused_residual_add_rmsnorm_ref(xe, re, we, EPS, multiplier)
        (z * 2 + r * 3).sum().backward()
        (ze * 2 + r_e * 3).sum().backward()
        if dtype == torch.float32:
            tol = dict(rtol=0, atol=1.6e-4)
            assert torch.equal(r.detach().cpu(), r_e.detach())
        else:
            tol = dict(rtol=2e-2, atol=1e-1)
            assert torch.equal(r.detach().cpu(), r_e.detach())  # the new residual stream: two roundings, the same bits
        torch.testing.assert_close(z.detach().cpu().float(), ze.detach().float(), **tol)
        torch.testing.assert_close(xk.grad.cpu().float(), xe.grad.float(), **tol)
        torch.testing.assert_close(rk.grad.cpu().float(), re.grad.float(), **tol)
        if has_weight:
            wt = dict(rtol=0, atol=1.1e-4 * max(1.0, (shape[0] if len(shape) > 1 else 1) ** 0.5 / 4)) if dtype == torch.float32 else dict(rtol=2e-2, atol=0.5)
            torch.testing.assert_close(wk.grad.cpu().float(), we.grad.float(), **wt)


@pytest.mark.parametrize("name,dt", [("f32_w", torch.float32), ("f32_now", torch.float32), ("bf16_w", torch.bfloat16),
                                     ("f16_w", torch.float16)])
def test_against_reference_golden(golden_dir, name, dt):
    """Outputs of the reference's rmsnorm_torch / fused_residual_add_rmsnorm_torch stored by tests/golden/make_golden.py."""
    from cute_kernels import fused_residual_add_rmsnorm_cute, rmsnorm_cute

    g = np.load(os.path.join(golden_dir, "rmsnorm.npz"))
    t = lambda k: torch.from_numpy(g[f"{name}_{k}"]).to(dt).cuda()  # noqa: E731
    mult, has_w = g[f"{name}_meta"]
    mult = None if mult == 0 else float(mult)
    x = t("x").requires_grad_()
    w = t("w").requires_grad_() if has_w else None
    z = rmsnorm_cute(x, w, EPS)
    z.sum().backward()
    f32 = dt == torch.float32
    tol = dict(rtol=0, atol=2e-5) if f32 else dict(rtol=1.6e-2, atol=1.6e-2)
    torch.testing.assert_close(z.detach(), t("z"), **tol)
    torch.testing.assert_close(x.grad, t("dx"), rtol=tol["rtol"], atol=tol["atol"] if f32 else 9e-2)
    if has_w:
        torch.testing.assert_close(w.grad, t("dw"), rtol=1e-2, atol=6.5e-5 if f32 else 0.1)
    x2, res = t("x").requires_grad_(), t("res").requires_grad_()
    w2 = t("w").requires_grad_() if has_w else None
    z2, r2 = fused_residual_add_rmsnorm_cute(x2, res, w2, EPS, mult)
    (z2 * 2 + r2 * 3).sum().backward()
    assert torch.equal(r2.detach(), t("fr"))
    ftol = dict(rtol=0, atol=1.6e-4) if f32 else dict(rtol=2e-2, atol=1e-1)
    torch.testing.assert_close(z2.detach(), t("fz"), **ftol)
    torch.testing.assert_close(x2.grad, t("fdx"), **ftol)
    torch.testing.assert_close(res.grad, t("fdres"), **ftol)
    if has_w:
        torch.testing.assert_close(w2.grad, t("fdw"), rtol=2e-2, atol=1.1e-4 if f32 else 0.5)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_compiled_fullgraph(dtype):
    from cute_kernels import fused_residual_add_rmsnorm_cute, rmsnorm_cute

    torch._dynamo.reset()
    xk, xe = _pair((64, 1024), dtype, 6)
    rk, re = _pair((64, 1024), dtype, 7)
    wk, we = _pair((1024,), dtype, 8)
    f = torch.compile(rmsnorm_cute, fullgraph=True)
    z = f(x=xk, weight=wk, eps=EPS, memory_efficient=False)
    ze = orc.rmsnorm_ref(xe, we, EPS)
    z.sum().backward()
    ze.sum().backward()
    tol = dict(rtol=0, atol=2e-5) if dtype == torch.float32 else dict(rtol=2e-2, atol=2e-2)
    torch.testing.assert_close(z.detach().cpu().float(), ze.detach().float(), **tol)
    torch.testing.assert_close(xk.grad.cpu().float(), xe.grad.float(), rtol=tol["rtol"], atol=max(tol["atol"], 1e-4))
    f2 = torch.compile(fused_residual_add_rmsnorm_cute, fullgraph=True)
    xk2, xe2 = _pair((64, 1024), dtype, 9)
    z2, r2 = f2(x=xk2, residual=rk, weight=wk, eps=EPS, multiplier=0.9, memory_efficient=True)
    ze2, re2 = orc.fused_residual_add_rmsnorm_ref(xe2, re, we, EPS, 0.9)
    assert torch.equal(r2.detach().cpu(), re2.detach())
    torch.testing.assert_close(z2.detach().cpu().float(), ze2.detach().float(), **tol)


def test_rejects_cpu_and_mismatched_weight():
    from cute_kernels import rmsnorm_cute

    with pytest.raises(RuntimeError):
        rmsnorm_cute(torch.randn(4, 8), None, EPS)
    with pytest.raises(AssertionError):
        rmsnorm_cute(torch.randn(4, 8, device="cuda"), torch.randn(9, device="cuda"), EPS)
    out = rmsnorm_cute(torch.empty(0, 8, device="cuda"), None, None)
    assert out.shape == (0, 8)


def test_replace_rmsnorm_in_a_compiled_block():
    """CuteInductor's second rewrite: torch.rms_norm / F.rms_norm in a traced graph becomes rmsnorm_cute
    (cute_inductor/rmsnorm.py:13-35), and the compiled function launches the RMSNorm kernel."""
    import torch.nn.functional as F

    import cute_kernels as ck
    from cute_kernels import _lib

    torch._dynamo.reset()

    def block(x, w):
        return F.rms_norm(x, (x.size(-1),), weight=w, eps=EPS) * 2.0

    ci = ck.CuteInductor(use_torch_inductor_after_cute_inductor=False)
    f = torch.compile(block, backend=ci.compiler)
    xk, xe = _pair((48, 512), torch.bfloat16, 10)
    wk, we = _pair((512,), torch.bfloat16, 11)
    _lib.launch_log.reset()
    _lib.launch_log.record_events = True
    try:
        z = f(xk, wk)
        torch.cuda.synchronize()
        names = [e[0] for e in _lib.launch_log.events]
    finally:
        _lib.launch_log.record_events = False
        _lib.launch_log.reset()
    assert "rmsnorm_fwd" in names, names
    ze = orc.rmsnorm_ref(xe, we, EPS) * 2.0
    torch.testing.assert_close(z.detach().cpu().float(), ze.detach().float(), rtol=2e-2, atol=2e-2)
    z.sum().backward()
    ze.sum().backward()
    torch.testing.assert_close(xk.grad.cpu().float(), xe.grad.float(), rtol=2e-2, atol=9e-2)
