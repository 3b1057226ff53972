"""CuteInductor as a torch.compile backend on the GPU: the rewritten graph must launch this library's kernels and
match the oracle, forward and backward (reference: cute_kernels/cute_inductor/compiler.py:27-47,
cute_inductor/swiglu_packed.py:16-76, cute_inductor/rmsnorm.py:13-35)."""

import pytest
import torch
import torch.nn.functional as F

import ck_oracle as orc

pytestmark = pytest.mark.gpu


def _chunk_silu_mul(x):
    up, gate = x.chunk(2, dim=-1)
    return up * F.silu(gate)


class _GatedMlp(torch.nn.Module):
    def __init__(self, hidden, inter):
        super().__init__()
        self.fc = torch.nn.Linear(hidden, 2 * inter, bias=False)
        self.proj = torch.nn.Linear(inter, hidden, bias=False)

    def forward(self, x):
        up, gate = self.fc(x).chunk(2, dim=-1)
        return self.proj(up * F.silu(gate))


def _logged(fn):
    """Runs fn() with per-launch logging on and returns (result, names of this library's launches)."""
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


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("after_inductor", [False, True])
def test_compiled_chunk_silu_mul_runs_swiglu_kernels(dtype, after_inductor):
    import cute_kernels as ck

    torch._dynamo.reset()
    ci = ck.CuteInductor(use_torch_inductor_after_cute_inductor=after_inductor)
    fn = torch.compile(_chunk_silu_mul, backend=ci.compiler)
    g = torch.Generator().manual_seed(0)
    x = torch.randn(300, 512, generator=g).to(dtype)
    dy = torch.randn(300, 256, generator=g).to(dtype)
    xk = x.cuda().requires_grad_()

    y, names = _logged(lambda: fn(xk))
    assert "swiglu_fwd" in names, f"the compiled graph did not launch the SwiGLU kernel: {names}"
    _, names_b = _logged(lambda: y.backward(dy.cuda()))
    assert "swiglu_bwd" in names_b, f"the compiled backward did not launch the SwiGLU kernel: {names_b}"

    xr = x.float().requires_grad_()
    yr = orc.swiglu_packed_ref(xr)
    yr.backward(dy.float())
    tol = dict(rtol=2e-2, atol=2e-2) if dtype == torch.bfloat16 else dict(rtol=0, atol=5.5e-6)
    torch.testing.assert_close(y.float().cpu(), yr.detach(), **tol)
    torch.testing.assert_close(xk.grad.float().cpu(), xr.grad, **tol)


def test_compiled_gated_mlp_module():
    import cute_kernels as ck

    torch._dynamo.reset()
    torch.manual_seed(3)
    m = _GatedMlp(128, 256).cuda().bfloat16()
    ref = _GatedMlp(128, 256)
    ref.load_state_dict({k: v.float().cpu() for k, v in m.state_dict().items()})
    ci = ck.CuteInductor(use_torch_inductor_after_cute_inductor=False)
    cm = torch.compile(m, backend=ci.compiler)
    x = torch.randn(4, 50, 128)
    xk = x.bfloat16().cuda().requires_grad_()
    xr = x.bfloat16().float().requires_grad_()
    y, names = _logged(lambda: cm(xk))
    assert "swiglu_fwd" in names
    yr = ref(xr)
    torch.testing.assert_close(y.float().cpu(), yr.detach(), rtol=2e-2, atol=2e-2)
    y.sum().backward()
    yr.sum().backward()
    torch.testing.assert_close(xk.grad.float().cpu(), xr.grad, rtol=4e-2, atol=4e-2)
