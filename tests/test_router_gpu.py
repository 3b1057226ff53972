"""Router tail kernel (top-k + softmax + int32 ids) against the oracle's three-op restatement."""

import pytest
import torch

import ck_oracle as orc

pytestmark = pytest.mark.gpu

SHAPES = [(1, 8, 1), (5, 8, 2), (300, 8, 2), (257, 64, 8), (1000, 60, 6), (64, 256, 32), (129, 33, 33 - 1), (7, 3, 3)]


def _logits(T, E, dtype, seed, ties=False):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(T, E, generator=g)
    if ties:
        x = (x * 2).round() / 2  # many equal logits per row
    return x.to(dtype)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
@pytest.mark.parametrize("T,E,k", SHAPES)
def test_router_forward_matches_oracle(dtype, T, E, k):
    from cute_kernels import router_topk_softmax

    logits = _logits(T, E, dtype, 17 * T + E + k)
    w, ids = router_topk_softmax(logits.cuda(), k)
    assert ids.dtype == torch.int32 and w.dtype == dtype and ids.shape == (T, k)
    w_ref, ids_ref = orc.routing_weights_ref(logits, k, dtype)
    # the selected logits (values, in order) are bit-identical; ids may differ only between equal logits
    picked = torch.gather(logits, 1, ids.cpu().long())
    assert torch.equal(picked, torch.gather(logits, 1, ids_ref))
    if dtype == torch.float32:
        assert torch.equal(ids.cpu().long(), ids_ref)
    # no expert twice in a row
    assert (torch.sort(ids.cpu(), dim=1).values.diff(dim=1) > 0).all() or k == 1
    tol = dict(rtol=1e-5, atol=1e-6) if dtype == torch.float32 else dict(rtol=2e-2, atol=2e-2)
    torch.testing.assert_close(w.cpu().float(), w_ref.float(), **tol)


@pytest.mark.parametrize("T,E,k", [(200, 8, 2), (100, 64, 8)])
def test_router_ties_take_lower_index(T, E, k):
    from cute_kernels import router_topk_softmax

    logits = _logits(T, E, torch.float32, 5, ties=True)
    _, ids = router_topk_softmax(logits.cuda(), k)
    # stable descending sort = descending by value, ties by lower index
    exp = torch.sort(logits, dim=1, descending=True, stable=True).indices[:, :k]
    assert torch.equal(ids.cpu().long(), exp)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("T,E,k", [(5, 8, 2), (300, 64, 8), (77, 60, 6), (33, 8, 1)])
def test_router_backward_matches_autograd(dtype, T, E, k):
    from cute_kernels import router_topk_softmax

    logits = _logits(T, E, dtype, 3 * T + E)
    g = torch.Generator().manual_seed(T)
    dw = torch.randn(T, k, generator=g).to(dtype)

    x = logits.cuda().requires_grad_(True)
    w, ids = router_topk_softmax(x, k)
    w.backward(dw.cuda())

    xr = logits.float().requires_grad_(True)
    vals = torch.gather(xr, 1, ids.cpu().long())          # pinned to the kernel's selection
    wr = torch.softmax(vals, dim=-1)
    wr.backward(dw.float())
    tol = dict(rtol=1e-5, atol=1e-6) if dtype == torch.float32 else dict(rtol=2e-2, atol=2e-2)
    torch.testing.assert_close(x.grad.cpu().float(), xr.grad, **tol)
    # exact zeros off the selection
    mask = torch.ones(T, E, dtype=torch.bool)
    mask.scatter_(1, ids.cpu().long(), False)
    assert (x.grad.cpu()[mask] == 0).all()


def test_router_masked_logits_give_distinct_experts():
    from cute_kernels import router_topk_softmax

    logits = torch.full((6, 16), float("-inf"))
    logits[:, 5] = 1.0                      # one live expert, k = 3: the other two picks are masked experts 0 and 1
    logits[3, 9] = 2.0
    w, ids = router_topk_softmax(logits.cuda(), 3)
    ids = ids.cpu()
    assert ids[0].tolist() == [5, 0, 1] and ids[3].tolist() == [9, 5, 0]
    assert (torch.sort(ids, dim=1).values.diff(dim=1) > 0).all()
    torch.testing.assert_close(w.cpu()[0], torch.tensor([1.0, 0.0, 0.0]))


def test_router_rejects_and_empty():
    from cute_kernels import router_topk_softmax

    w, ids = router_topk_softmax(torch.empty(0, 8, device="cuda"), 2)
    assert w.shape == (0, 2) and ids.shape == (0, 2)
    with pytest.raises(RuntimeError):
        router_topk_softmax(torch.randn(4, 512, device="cuda"), 2)       # more experts than the kernel holds
    with pytest.raises(ValueError):
        router_topk_softmax(torch.randn(4, 8, device="cuda"), 9)
    with pytest.raises(Exception):
        router_topk_softmax(torch.randn(4, 8), 2)                          # CPU tensors fail loudly


def test_moe_module_uses_int32_router():
    from cute_kernels import MoE_Cute
    from cute_kernels.swiglu import swiglu_packed_cute

    torch.manual_seed(0)
    m = MoE_Cute(num_experts=8, num_experts_per_tok=2, hidden_size=128, intermediate_size=128,
                 activation_function=swiglu_packed_cute, is_glu=True, add_bias=False, std=0.02).cuda().bfloat16()
    x = torch.randn(64, 128, device="cuda", dtype=torch.bfloat16)
    logits, weights, sel = m._compute_routing_weights(x)
    assert sel.dtype == torch.int32 and weights.dtype == torch.bfloat16
    y, _ = m(x)
    assert torch.isfinite(y.float()).all()


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("E,k", [(8, 2), (64, 8), (40, 6)])
def test_router_nan_rows_give_valid_distinct_ids(dtype, E, k):
    """NaN logits sort as the greatest value (torch.topk's order): an all-NaN row and a partly-NaN row still give k
    distinct ids in [0, E), and the backward pass completes without touching memory outside d_logits."""
    from cute_kernels import router_topk_softmax

    g = torch.Generator().manual_seed(E + k)
    logits = torch.randn(9, E, generator=g)
    logits[2] = float("nan")                       # every logit NaN
    logits[4, 3] = float("nan")                    # one NaN: it must be picked first
    logits[6, 1] = float("nan")
    logits[6, E - 1] = -float("nan")               # sign bit set: still a NaN, still greatest
    x = logits.to(dtype).cuda().requires_grad_()
    w, ids = router_topk_softmax(x, k)
    idc = ids.cpu().long()
    assert ((idc >= 0) & (idc < E)).all()
    assert (torch.sort(idc, dim=1).values.diff(dim=1) > 0).all()
    assert idc[2].tolist() == list(range(k))       # ties between NaNs go to the lower index
    assert idc[4, 0].item() == 3
    assert sorted(idc[6, :2].tolist()) == [1, E - 1]
    # rows without NaN are unaffected
    w_ref, ids_ref = orc.routing_weights_ref(logits.to(dtype)[[0, 1, 3, 5, 7, 8]], k, dtype)
    picked = torch.gather(logits.to(dtype)[[0, 1, 3, 5, 7, 8]], 1, idc[[0, 1, 3, 5, 7, 8]])
    assert torch.equal(picked, torch.gather(logits.to(dtype)[[0, 1, 3, 5, 7, 8]], 1, ids_ref))
    assert torch.isnan(w.detach().float().cpu()[2]).all()
    w.backward(torch.ones_like(w))
    torch.cuda.synchronize()
    assert x.grad.shape == (9, E)
    assert torch.isfinite(x.grad.float().cpu()[[0, 1, 3, 5, 7, 8]]).all()


@pytest.mark.expects_dev_status
def test_router_backward_skips_out_of_range_ids():
    """The backward kernel never writes through an id outside [0, E): it skips the entry and raises CK_DEV_RANGE."""
    import cute_kernels
    from cute_kernels import _lib

    T, E, k = 4, 8, 2
    w = torch.full((T, k), 0.5, device="cuda")
    dw = torch.ones(T, k, device="cuda")
    ids = torch.tensor([[0, 1], [2, 0x7FFFFFFF], [-5, 3], [7, 6]], dtype=torch.int32, device="cuda")
    guard = torch.full((T * E + 64,), 7.0, device="cuda")
    d_logits = guard[:T * E]
    status = _lib.status_word(torch.device("cuda", torch.cuda.current_device()))
    st = _lib.lib.ck_router_topk_softmax_bwd(w.data_ptr(), dw.data_ptr(), ids.data_ptr(), d_logits.data_ptr(), T, E, k,
                                             _lib.CK_F32, status.data_ptr(), _lib.stream_ptr())
    assert st == 0
    torch.cuda.synchronize()
    assert (guard[T * E:] == 7.0).all()
    with pytest.raises(RuntimeError, match="CK_DEV_RANGE"):
        cute_kernels.check_device_status()
    cute_kernels.check_device_status()  # cleared


# ---- gate projection + router tail in one tensor-core launch ---------------------------------------------------
@pytest.mark.parametrize("flavour", ["cta_pair", "single_cta"])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("T,H,E,k", [(1, 64, 8, 2), (130, 256, 8, 2), (1000, 512, 64, 8), (257, 128, 40, 6), (512, 1024, 256, 8),
                                     (384, 72, 8, 1)])
def test_fused_gate_router_matches_linear_plus_router(flavour, dtype, T, H, E, k):
    """logits = F.linear(x, w) within one rounding of the 16-bit type (fp32 accumulation in a different order); weights and
    ids are EXACTLY what the stand-alone router kernel gives on the fused kernel's own logits."""
    from cute_kernels import _lib, router_gate_topk_softmax, router_topk_softmax

    prev = _lib.lib.ck_set_gemm_cta_pair(1 if flavour == "cta_pair" else 0)
    try:
        g = torch.Generator().manual_seed(T + E)
        x = torch.randn(T, H, generator=g).to(dtype).cuda()
        w = (torch.randn(E, H, generator=g) / H**0.5).to(dtype).cuda()
        logits = torch.full((T, E), float("nan"), dtype=dtype, device="cuda")
        logits, weights, ids = router_gate_topk_softmax(x, w, k)
        ref = x.float() @ w.float().t()
        torch.testing.assert_close(logits.float(), ref, rtol=2 ** -7 if dtype == torch.bfloat16 else 2 ** -10, atol=1e-3)
        w2, ids2 = router_topk_softmax(logits, k)
        assert torch.equal(ids, ids2)
        assert torch.equal(weights.view(torch.int16), w2.view(torch.int16))
        assert ids.dtype == torch.int32 and int(ids.min()) >= 0 and int(ids.max()) < E
        import cute_kernels

        cute_kernels.check_device_status()
    finally:
        _lib.lib.ck_set_gemm_cta_pair(prev)


def test_fused_gate_router_gradients_match_autograd():
    from cute_kernels import router_gate_topk_softmax

    T, H, E, k = 300, 256, 16, 4
    g = torch.Generator().manual_seed(5)
    x0 = torch.randn(T, H, generator=g).bfloat16().cuda()
    w0 = (torch.randn(E, H, generator=g) / H**0.5).bfloat16().cuda()
    d_w = torch.randn(T, k, generator=g).bfloat16().cuda()
    d_l = torch.randn(T, E, generator=g).bfloat16().cuda()
    x, w = x0.clone().requires_grad_(), w0.clone().requires_grad_()
    logits, weights, ids = router_gate_topk_softmax(x, w, k)
    torch.autograd.backward([logits, weights], [d_l, d_w])
    # the same computation with torch ops on the same selection
    xr, wr = x0.float().requires_grad_(), w0.float().requires_grad_()
    lr = xr @ wr.t()
    wr_sel = torch.softmax(lr.gather(1, ids.long()), dim=-1)
    torch.autograd.backward([lr, wr_sel], [d_l.float(), d_w.float()])
    torch.testing.assert_close(x.grad.float(), xr.grad, rtol=3e-2, atol=3e-2)
    torch.testing.assert_close(w.grad.float(), wr.grad, rtol=3e-2, atol=3e-2 * T**0.5 / 4)


def test_fused_gate_router_rejects_what_it_cannot_do_and_module_uses_it():
    from cute_kernels import MoE_Cute, _lib, router_gate_topk_softmax
    from cute_kernels.router import fused_gate_supported
    from cute_kernels.swiglu import swiglu_packed_cute

    x = torch.randn(16, 64, device="cuda")
    assert not fused_gate_supported(x, torch.randn(8, 64, device="cuda"), 2)              # fp32: two-step path
    assert not fused_gate_supported(x.bfloat16(), torch.randn(12, 64, device="cuda").bfloat16(), 2)  # E % 8 != 0
    assert not fused_gate_supported(x.bfloat16(), torch.randn(16, 64, device="cuda").bfloat16(), 9)  # k > 8
    with pytest.raises(ValueError):
        router_gate_topk_softmax(x, torch.randn(8, 64, device="cuda"), 2)
    torch.manual_seed(0)
    m = MoE_Cute(num_experts=8, num_experts_per_tok=2, hidden_size=128, intermediate_size=128,
                 activation_function=swiglu_packed_cute, is_glu=True, add_bias=False, std=0.02).cuda().bfloat16()
    xb = torch.randn(200, 128, device="cuda", dtype=torch.bfloat16)
    _lib.launch_log.reset()
    _lib.launch_log.record_events = True
    try:
        logits, weights, sel = m._compute_routing_weights(xb)
        names = [e[0] for e in _lib.launch_log.events]
    finally:
        _lib.launch_log.record_events = False
        _lib.launch_log.reset()
    assert names == ["router_gate_topk_softmax"]
    m.fuse_router = False
    l2, w2, s2 = m._compute_routing_weights(xb)
    torch.testing.assert_close(logits.float(), l2.float(), rtol=2 ** -7, atol=1e-3)
    same = (sel == s2).all(dim=1)
    assert same.float().mean() > 0.98  # a logit that rounds differently may swap two near-equal experts
    assert torch.equal(weights[same].view(torch.int16), w2[same].view(torch.int16)) or \
        torch.allclose(weights[same].float(), w2[same].float(), atol=2e-2)


def test_fused_gate_router_nan_tokens_give_valid_distinct_ids():
    """A token of NaNs gives NaN logits: they sort as the greatest value, the ids stay distinct and inside [0, E), the
    weights are NaN like torch.softmax's, and the other tokens are untouched."""
    from cute_kernels import router_gate_topk_softmax, router_topk_softmax

    T, H, E, k = 200, 128, 16, 4
    g = torch.Generator().manual_seed(9)
    x = torch.randn(T, H, generator=g).bfloat16().cuda()
    w = (torch.randn(E, H, generator=g) / H**0.5).bfloat16().cuda()
    ref_l, ref_w, ref_i = router_gate_topk_softmax(x, w, k)
    x2 = x.clone()
    x2[7] = float("nan")
    x2[130, :5] = float("nan")
    logits, weights, ids = router_gate_topk_softmax(x2, w, k)
    for t in (7, 130):
        assert torch.isnan(logits[t].float()).all()
        row = ids[t].tolist()
        assert len(set(row)) == k and all(0 <= e < E for e in row)
        assert row == list(range(k))  # all keys equal: ties go to the lower expert index
        assert torch.isnan(weights[t].float()).all()
    keep = torch.ones(T, dtype=torch.bool, device="cuda")
    keep[[7, 130]] = False
    assert torch.equal(ids[keep], ref_i[keep]) and torch.equal(weights[keep].view(torch.int16), ref_w[keep].view(torch.int16))
    w2, i2 = router_topk_softmax(logits, k)
    assert torch.equal(i2, ids)
