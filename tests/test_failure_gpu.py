"""Failure paths that return a status instead of faulting: the bounded device wait and the status word on the module.

Nothing here hangs, traps or faults a GPU: the wait under test has a 2 ms limit and simply runs out."""

import pytest
import torch

import ck_oracle as orc

pytestmark = pytest.mark.gpu


@pytest.mark.expects_dev_status
def test_bounded_wait_runs_out_sets_timeout_and_context_survives():
    import cute_kernels
    from cute_kernels import _lib

    dev = torch.device("cuda", torch.cuda.current_device())
    status = _lib.status_word(dev)
    cute_kernels.check_device_status()
    result = torch.full((4,), -1, dtype=torch.int32, device=dev)
    limit_ns = 2_000_000
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    st = _lib.lib.ck_test_wait_timeout(limit_ns, result.data_ptr(), status.data_ptr(), _lib.stream_ptr())
    e1.record()
    assert st == 0
    torch.cuda.synchronize()
    ok0, ok1, waited_ns, abort = result.tolist()
    assert ok0 == 0 and ok1 == 0, "both waits must give up"
    assert abort == 1
    assert limit_ns <= waited_ns < 50 * limit_ns
    assert e0.elapsed_time(e1) < 200.0  # the launch ended by itself, in milliseconds
    assert int(status.item()) & _lib.CK_DEV_TIMEOUT
    with pytest.raises(RuntimeError, match="CK_DEV_TIMEOUT"):
        cute_kernels.check_device_status()
    cute_kernels.check_device_status()  # the word was cleared

    # limits outside (0, 100 ms] are refused on the host
    assert _lib.lib.ck_test_wait_timeout(0, result.data_ptr(), status.data_ptr(), _lib.stream_ptr()) == -2
    assert _lib.lib.ck_test_wait_timeout(10**9, result.data_ptr(), status.data_ptr(), _lib.stream_ptr()) == -2

    # the context is intact: a grouped GEMM step right after still matches the oracle
    inp = orc.gen_moe_inputs(11, T=256, H=128, I=128, E=4, k=2)
    ref = orc.moe_experts_ref(inp["x"], inp["router_weights"], inp["selected_experts"], inp["w_fc"], inp["w_proj"],
                              orc.swiglu_packed_ref)
    with torch.no_grad():
        y = cute_kernels.fused_experts(inp["x"].bfloat16().cuda(), inp["router_weights"].bfloat16().cuda(),
                                       inp["selected_experts"].cuda(), inp["w_fc"].bfloat16().cuda(),
                                       inp["w_proj"].bfloat16().cuda(), 2)
    torch.testing.assert_close(y.float().cpu(), ref, rtol=2e-2, atol=2e-2)
    cute_kernels.check_device_status()


@pytest.mark.expects_dev_status
def test_module_check_status_raises_on_a_flagged_step():
    """``MoE_Cute(check_status=True)`` polls the device status word once per forward (one synchronisation) and raises
    when a kernel of the step flagged a problem -- here an expert id outside [0, E) injected behind the router."""
    from cute_kernels import MoE_Cute, check_device_status
    from cute_kernels.swiglu import swiglu_packed_cute

    torch.manual_seed(0)
    m = MoE_Cute(8, 2, 128, 128, swiglu_packed_cute, True, False, 0.02).cuda().bfloat16()
    m.check_status = True
    x = torch.randn(64, 128, device="cuda", dtype=torch.bfloat16)
    y, _ = m(x)  # a clean step passes
    assert torch.isfinite(y.float()).all()

    real = m._compute_routing_weights

    def bad_router(h):
        logits, w, sel = real(h)
        sel = sel.clone()
        sel[3, 1] = 99  # outside [0, 8)
        return logits, w, sel

    m._compute_routing_weights = bad_router
    with pytest.raises(RuntimeError, match="CK_DEV_RANGE"):
        m(x)
    check_device_status()  # cleared by the raise
    m.check_status = False
    m(x)  # silent without the option; the conftest hook is told to expect the flag
    with pytest.raises(RuntimeError, match="CK_DEV_RANGE"):
        check_device_status()
