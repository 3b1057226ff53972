"""Parity at the benchmarked shapes: the Mixtral-shaped layer (16384 tokens, hidden 4096, intermediate 14336,
8 experts, top-2), the fine-grained layer (32768 tokens, hidden 2048, intermediate 1408, 64 experts, top-8, skewed
routing) and the stand-alone SwiGLU at [16384, 14336], all bf16.

Two checkers per MoE shape, both in fp32 on the same bf16-representable seeded inputs:
  * the CPU oracle on 64 sampled tokens (each token needs only its own k experts): y, dx, d_router_weights;
  * the oracle's expert computation (``ck_oracle.moe_experts_ref``, plain torch) run in fp32 on the GPU over the
    whole batch: all five outputs including the full weight gradients.  It is a checker, not a product path.

Tolerance: |got - ref| <= atol + 2e-2 |ref| with atol = 2e-2 taken relative to the magnitude of the tensor: every
output here is a sum of 4096 - 28672 products of bf16-rounded O(1) terms, so an absolute 2e-2 is meaningless for its
near-zero elements; atol = 2e-2 * max(1, RMS of the reference), with the RMS taken per expert for the weight gradients
(an expert's gradient scales with the number of rows routed to it, and the fine-grained layer's routing is skewed 6:1).
Calibration: a plain torch bf16 run of the same oracle code, measured against the same fp32 reference, must not be more
accurate than the kernels by more than 25 % RMS (on B200 it is 1.3 - 2 x less accurate).
"""

import pytest
import torch

import ck_oracle as orc

pytestmark = pytest.mark.gpu

RTOL = 2e-2
ATOL = 2e-2


def _check(name, got, ref, atol):
    got, ref = got.float(), ref.float()
    assert got.shape == ref.shape, name
    err = (got - ref).abs()
    bound = atol + RTOL * ref.abs()
    worst = (err / bound).max().item()
    assert torch.isfinite(got).all(), f"{name}: non-finite values"
    atol = float(torch.as_tensor(atol).max())
    assert worst <= 1.0, (f"{name}: worst error / bound = {worst:.3f} (atol {atol:.4f}, rtol {RTOL}); max abs err "
                          f"{err.max().item():.4e}, ref rms {ref.pow(2).mean().sqrt().item():.4e}, "
                          f"{(err > bound).float().mean().item():.3e} of the elements out of bound")
    return worst


def _rms_atol(ref):
    return ATOL * max(1.0, ref.float().pow(2).mean().sqrt().item())


def _per_expert_rms_atol(ref):
    """atol tensor [E, 1, 1] for a weight gradient [E, out, in]."""
    rms = ref.float().pow(2).mean(dim=(1, 2), keepdim=True).sqrt()
    return ATOL * rms.clamp(min=1.0)


def _err_rms(got, ref):
    return (got.float() - ref.float()).pow(2).mean().sqrt().item()


def _run_gpu(inp, k):
    from cute_kernels import check_device_status, fused_experts

    x = inp["x"].cuda().requires_grad_()
    rw = inp["router_weights"].cuda().requires_grad_()
    w_fc = inp["w_fc"].cuda().requires_grad_()
    w_proj = inp["w_proj"].cuda().requires_grad_()
    y = fused_experts(x, rw, inp["selected_experts"].cuda(), w_fc, w_proj, k)
    y.backward(inp["grad_out"].cuda())
    torch.cuda.synchronize()
    check_device_status()
    return dict(y=y.detach(), dx=x.grad, d_router_weights=rw.grad, d_w_fc=w_fc.grad, d_w_proj=w_proj.grad)


def _cpu_oracle_on_tokens(inp, tokens):
    """fp32 CPU oracle restricted to ``tokens``: outputs and the gradients that depend on those tokens alone."""
    x = inp["x"][tokens].float().requires_grad_()
    rw = inp["router_weights"][tokens].float().requires_grad_()
    y = orc.moe_experts_ref(x, rw, inp["selected_experts"][tokens], inp["w_fc"].float(), inp["w_proj"].float(),
                            orc.swiglu_packed_ref)
    y.backward(inp["grad_out"][tokens].float())
    return dict(y=y.detach(), dx=x.grad, d_router_weights=rw.grad)


@pytest.mark.parametrize("name", ["c4_mixtral", "c5_finegrained"])
def test_moe_at_benchmark_shape(name):
    cfg = orc.CONFIGS[name]
    T, k = cfg["T"], cfg["k"]
    prev = torch.backends.cuda.matmul.allow_tf32
    torch.backends.cuda.matmul.allow_tf32 = False  # the GPU-side checker multiplies in full fp32
    try:
        inp = orc.gen_moe_inputs(0, dtype=torch.bfloat16, **cfg)  # seeded, generated in fp32 on the CPU, rounded to bf16
        res = _run_gpu(inp, k)

        # (1) CPU oracle on 64 sampled tokens
        g = torch.Generator().manual_seed(1)
        tokens = torch.randperm(T, generator=g)[:64].sort().values
        cpu = _cpu_oracle_on_tokens(inp, tokens)
        for key, ref in cpu.items():
            _check(f"{name} {key} (CPU oracle, 64 tokens)", res[key][tokens.cuda()].cpu(), ref, _rms_atol(ref))

        # (2) the oracle's expert computation in fp32 on the GPU, whole batch, all five outputs
        ref = orc.moe_fwd_bwd_ref({k_: v.cuda() for k_, v in inp.items()}, dtype=torch.float32)
        worst = {}
        for key in ("y", "dx", "d_router_weights"):
            worst[key] = _check(f"{name} {key} (fp32 checker, full)", res[key], ref[key], _rms_atol(ref[key]))
        for key in ("d_w_fc", "d_w_proj"):
            worst[key] = _check(f"{name} {key} (fp32 checker, full)", res[key], ref[key], _per_expert_rms_atol(ref[key]))
        # calibration: the same oracle code run by torch in bf16 is the accuracy a bf16 implementation is expected to have
        cal = orc.moe_fwd_bwd_ref({k_: v.cuda() for k_, v in inp.items()}, dtype=torch.bfloat16)
        for key in ("y", "dx", "d_router_weights", "d_w_fc", "d_w_proj"):
            ours, theirs = _err_rms(res[key], ref[key]), _err_rms(cal[key], ref[key])
            assert ours <= 1.25 * theirs, f"{name} {key}: RMS error {ours:.3e} against {theirs:.3e} for a torch bf16 run"
        # the two checkers agree with each other on the sampled tokens far inside the tolerance
        for key, r_cpu in cpu.items():
            torch.testing.assert_close(ref[key][tokens.cuda()].cpu(), r_cpu, rtol=1e-3, atol=1e-3 * max(1.0, r_cpu.abs().max().item()))
        print(f"\n{name}: worst error / bound per output: " + ", ".join(f"{k_}={v:.3f}" for k_, v in worst.items()))
    finally:
        torch.backends.cuda.matmul.allow_tf32 = prev


def test_swiglu_at_benchmark_shape():
    """[16384, 14336] bf16, N(0,1) gate / up / upstream gradient, forward and backward against the fp32 oracle."""
    from cute_kernels import swiglu_cute

    rows, cols = 16384, 14336
    g = torch.Generator(device="cuda").manual_seed(0)
    mk = lambda: torch.randn(rows, cols, generator=g, device="cuda", dtype=torch.float32).bfloat16()  # noqa: E731
    gate, up, dy = mk().requires_grad_(), mk().requires_grad_(), mk()
    z = swiglu_cute(gate, up)
    z.backward(dy)
    # the oracle in fp32, slab by slab to bound the checker's memory
    step = 2048
    for r0 in range(0, rows, step):
        sl = slice(r0, r0 + step)
        g32, u32, d32 = gate.detach()[sl].float(), up.detach()[sl].float(), dy[sl].float()
        torch.testing.assert_close(z.detach()[sl].float(), orc.swiglu_ref(g32, u32), rtol=RTOL, atol=ATOL)
        dg, du = orc.swiglu_backward_ref(g32, u32, d32)
        torch.testing.assert_close(gate.grad[sl].float(), dg, rtol=RTOL, atol=ATOL)
        torch.testing.assert_close(up.grad[sl].float(), du, rtol=RTOL, atol=ATOL)
