"""swiglu_cute / swiglu_packed_cute against the oracle (tests/kernels/swiglu_test.py:23-72 of the reference)."""

import os

import numpy as np
import pytest
import torch

import ck_oracle as orc

pytestmark = pytest.mark.gpu

SHAPES = [(1, 1), (3, 5), (7, 8), (17, 33), (64, 64), (129, 257), (1025, 1031), (2048, 3000)]
DTYPES = [torch.float32, torch.float16, torch.bfloat16]


def _pair(shape, dtype, seed):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(shape, generator=g).to(dtype).cuda()
    return x.clone().requires_grad_(), x.clone().requires_grad_()


def _tol(dtype, fwd):
    if dtype == torch.float32:
        return dict(atol=5.5e-6 if fwd else 5e-6, rtol=0)  # the reference's fp32 tolerances
    return dict(atol=None, rtol=None)  # assert_close dtype defaults, as the reference does


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("compiled", [False, True])
def test_swiglu(dtype, compiled):
    from cute_kernels import CutoTuneParameter, KernelBackend, swiglu_cute

    fn = torch.compile(swiglu_cute, fullgraph=True) if compiled else swiglu_cute
    for i, shape in enumerate(SHAPES[: 4 if compiled else None]):
        gk, ge = _pair(shape, dtype, 2 * i)
        uk, ue = _pair(shape, dtype, 2 * i + 1)
        z = fn(gk, uk, kernel_backend_forward=KernelBackend.cuda, kernel_backend_backward=CutoTuneParameter())
        ze = orc.swiglu_ref(ge, ue)
        z.mean().backward()
        ze.mean().backward()
        torch.testing.assert_close(z, ze, **_tol(dtype, True))
        torch.testing.assert_close(gk.grad, ge.grad, **_tol(dtype, False))
        torch.testing.assert_close(uk.grad, ue.grad, **_tol(dtype, False))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("compiled", [False, True])
def test_swiglu_packed(dtype, compiled):
    from cute_kernels import swiglu_packed_cute

    fn = torch.compile(swiglu_packed_cute, fullgraph=True) if compiled else swiglu_packed_cute
    for i, shape in enumerate(SHAPES[: 4 if compiled else None]):
        shape = (shape[0], (shape[1] + 1) // 2 * 2)
        xk, xe = _pair(shape, dtype, 100 + i)
        z = fn(xk)
        ze = orc.swiglu_packed_ref(xe)
        z.mean().backward()
        ze.mean().backward()
        torch.testing.assert_close(z, ze, **_tol(dtype, True))
        torch.testing.assert_close(xk.grad, xe.grad, **_tol(dtype, False))


def test_swiglu_large_random_grad_bf16():
    """Benchmark-shaped slice with an N(0,1) upstream gradient; rtol/atol 2e-2 against the fp32 oracle."""
    from cute_kernels import swiglu_cute

    g = torch.Generator().manual_seed(0)
    gate = torch.randn(2048, 14336, generator=g).bfloat16().cuda().requires_grad_()
    up = torch.randn(2048, 14336, generator=g).bfloat16().cuda().requires_grad_()
    dy = torch.randn(2048, 14336, generator=g).bfloat16().cuda()
    z = swiglu_cute(gate, up)
    z.backward(dy)
    g32, u32, d32 = gate.detach().float(), up.detach().float(), dy.float()
    ref = orc.swiglu_ref(g32, u32)
    dg, du = orc.swiglu_backward_ref(g32, u32, d32)
    torch.testing.assert_close(z.float(), ref, rtol=2e-2, atol=2e-2)
    torch.testing.assert_close(gate.grad.float(), dg, rtol=2e-2, atol=2e-2)
    torch.testing.assert_close(up.grad.float(), du, rtol=2e-2, atol=2e-2)


def test_swiglu_matches_reference_golden(golden_dir):
    from cute_kernels import swiglu_cute, swiglu_packed_cute

    g = np.load(os.path.join(golden_dir, "swiglu.npz"))
    for name, dt in [("f32", torch.float32), ("bf16", torch.bfloat16), ("f16", torch.float16)]:
        t = lambda k: torch.from_numpy(g[f"{name}_{k}"]).to(dt).cuda()  # noqa: E731
        gate, up, dy = t("gate").requires_grad_(), t("up").requires_grad_(), t("dy")
        z = swiglu_cute(gate, up)
        z.backward(dy)
        tol = dict(atol=5.5e-6, rtol=0) if dt == torch.float32 else dict(atol=None, rtol=None)
        torch.testing.assert_close(z, t("out"), **tol)
        torch.testing.assert_close(gate.grad, t("dgate"), **tol)
        torch.testing.assert_close(up.grad, t("dup"), **tol)
        xp = torch.cat([up.detach(), gate.detach()], -1).requires_grad_()
        zp = swiglu_packed_cute(xp)
        zp.backward(dy)
        torch.testing.assert_close(zp, t("packed_out"), **tol)
        torch.testing.assert_close(xp.grad, t("packed_dx"), **tol)


def test_swiglu_rejects_triton_backend_and_cpu():
    from cute_kernels import KernelBackend, swiglu_cute

    x = torch.randn(4, 4, device="cuda")
    with pytest.raises(ValueError):
        swiglu_cute(x, x, kernel_backend_forward=KernelBackend.triton)
    with pytest.raises(RuntimeError):
        swiglu_cute(x.cpu(), x.cpu())
