"""Each grouped-GEMM entry point of the C ABI against an fp32 torch reference of the same op."""

import numpy as np
import pytest
import torch

import ck_oracle as orc

pytestmark = pytest.mark.gpu

@pytest.fixture(params=["cta_pair", "single_cta"], autouse=True)
def gemm_flavour(request):
    """Every test of this file runs on both grouped-GEMM kernel flavours."""
    from cute_kernels import _lib

    prev = _lib.lib.ck_set_gemm_cta_pair(1 if request.param == "cta_pair" else 0)
    yield request.param
    _lib.lib.ck_set_gemm_cta_pair(prev)


TOL = {torch.bfloat16: dict(rtol=2e-2, atol=2e-2), torch.float16: dict(rtol=4e-3, atol=4e-3),
       torch.float32: dict(rtol=6e-3, atol=6e-3)}  # fp32 runs as TF32 on the tensor cores, like the reference's tl.dot


def _routing(counts, k, seed=0):
    """ids with the given per-expert counts, shuffled; returns the device Routing and the oracle dict."""
    from cute_kernels import route

    ids = np.concatenate([np.full(c, e, dtype=np.int64) for e, c in enumerate(counts)])
    np.random.default_rng(seed).shuffle(ids)
    pad = (-ids.size) % k
    if pad:
        ids = np.concatenate([ids, np.zeros(pad, dtype=np.int64)])
    r = route(torch.from_numpy(ids).cuda(), len(counts))
    return ids, r, orc.route_ref(ids, len(counts))


def _row_expert(ref, E):
    cap = ref["row_map"].size
    re = np.full(cap, -1, dtype=np.int64)
    for e in range(E):
        re[ref["padded_off"][e] : ref["padded_off"][e + 1]] = e
    return re


def _padded_rows(ref, cols, dtype, seed, scale=1.0):
    """[cap, cols] activations: random on valid rows, zero on pad rows."""
    cap = ref["row_map"].size
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(cap, cols, generator=g) * scale
    x[torch.from_numpy(ref["row_map"] < 0)] = 0
    return x.to(dtype).cuda()


CASES = [
    # counts per expert, K, N
    ([130, 0, 5], 64, 256),
    ([1, 1, 1, 1], 192, 8),
    ([300, 17, 128, 0, 256], 136, 264),
    ([700, 900], 512, 1024),
]


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
@pytest.mark.parametrize("trans_w", [False, True])
@pytest.mark.parametrize("case", CASES)
def test_grouped_linear(dtype, trans_w, case):
    from cute_kernels import _lib
    from cute_kernels.moe import grouped_linear

    counts, K, N = case
    E = len(counts)
    ids, r, ref = _routing(counts, 1)
    x = _padded_rows(ref, K, dtype, 1)
    g = torch.Generator().manual_seed(2)
    w = (torch.randn(E, K, N, generator=g) if trans_w else torch.randn(E, N, K, generator=g)).mul(0.1).to(dtype).cuda()
    y = torch.full((x.size(0), N), float("nan"), dtype=dtype, device="cuda")
    grouped_linear(x, w, r.mtile_off, y, trans_w)
    re = _row_expert(ref, E)
    total = int(ref["padded_off"][-1])
    xf, wf = x.float().cpu(), w.float().cpu()
    for e in range(E):
        rows = np.nonzero(re[:total] == e)[0]
        if rows.size == 0:
            continue
        exp = xf[rows] @ (wf[e] if trans_w else wf[e].t())
        torch.testing.assert_close(y[rows].float().cpu(), exp, **TOL[dtype])
    assert torch.isnan(y[total:].float()).all()  # rows past the padded total are never written


@pytest.mark.parametrize("split", [1, 2, 3, 5])
@pytest.mark.parametrize("case", [([300, 17, 128, 0, 256], 136, 264), ([700, 900], 512, 1024), ([0, 0, 5], 64, 256)])
def test_grouped_linear_row_windows(case, split):
    """Two calls with clamped copies of mtile_off (m-tiles [0, split) and [split, end)) write exactly what one call writes."""
    from cute_kernels.moe import grouped_linear

    counts, K, N = case
    E = len(counts)
    ids, r, ref = _routing(counts, 1)
    x = _padded_rows(ref, K, torch.bfloat16, 1)
    g = torch.Generator().manual_seed(2)
    w = torch.randn(E, N, K, generator=g).mul(0.1).bfloat16().cuda()
    full = torch.full((x.size(0), N), float("nan"), dtype=torch.bfloat16, device="cuda")
    grouped_linear(x, w, r.mtile_off, full, False)
    y = torch.full_like(full, float("nan"))
    total = int(ref["padded_off"][-1])
    split = min(split, total // 128)                         # the window edge stays inside the padded rows
    grouped_linear(x, w, r.mtile_off.clamp(max=split), y, False)
    lo = split * 128
    assert torch.equal(y[:lo].view(torch.int16), full[:lo].view(torch.int16))
    assert torch.isnan(y[lo:].float()).all()                 # the second window is untouched so far
    grouped_linear(x, w, r.mtile_off.clamp(min=split), y, False)
    assert torch.equal(y[:total].view(torch.int16), full[:total].view(torch.int16))
    assert torch.isnan(y[total:].float()).all()


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
@pytest.mark.parametrize("case", [([130, 0, 5], 64, 256), ([300, 17, 128, 0, 256], 136, 264), ([700, 900], 512, 384)])
def test_wgrad(dtype, case):
    from cute_kernels import _lib
    from cute_kernels.moe import wgrad

    counts, M, N = case
    E = len(counts)
    ids, r, ref = _routing(counts, 1)
    a = _padded_rows(ref, M, dtype, 3)
    b = _padded_rows(ref, N, dtype, 4)
    dw = torch.full((E, M, N), float("nan"), dtype=dtype, device="cuda")
    wgrad(a, b, r.padded_off, dw)
    re = _row_expert(ref, E)
    af, bf = a.float().cpu(), b.float().cpu()
    for e in range(E):
        rows = np.nonzero(re == e)[0]
        exp = af[rows].t() @ bf[rows] if rows.size else torch.zeros(M, N)
        scale = max(1.0, float(rows.size) ** 0.5)
        tol = {k: v * scale for k, v in TOL[dtype].items()}
        torch.testing.assert_close(dw[e].float().cpu(), exp, **tol)


def _moe_problem(counts, H, I, k, dtype, seed=0):
    E = len(counts)
    ids, r, ref = _routing(counts, k, seed)
    T = ids.size // k
    g = torch.Generator().manual_seed(seed + 10)
    x = torch.randn(T, H, generator=g).to(dtype).cuda()
    w_fc = (torch.randn(E, 2 * I, H, generator=g) * 0.05).to(dtype).cuda()
    w_proj = (torch.randn(E, H, I, generator=g) * 0.05).to(dtype).cuda()
    gate_w = torch.rand(T * k, generator=g).to(dtype).cuda()
    return dict(E=E, T=T, H=H, I=I, k=k, ids=ids, r=r, ref=ref, x=x, w_fc=w_fc, w_proj=w_proj, gate_w=gate_w)


MOE_CASES = [([130, 0, 5, 9], 64, 128, 2), ([300, 17, 128, 0, 255], 136, 72, 2), ([513, 700, 64, 3], 256, 320, 4)]


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
@pytest.mark.parametrize("act_kind", [0, 1])
@pytest.mark.parametrize("case", MOE_CASES)
def test_fused_forward_pieces(dtype, act_kind, case):
    """gather -> up projection + activation -> down projection + combine, each checked separately."""
    from cute_kernels import _lib
    from cute_kernels.moe import down_combine_fwd, gather_rows, up_act_fwd

    counts, H, I, k = case
    p = _moe_problem(counts, H, I, k, dtype)
    r, ref, E, T = p["r"], p["ref"], p["E"], p["T"]
    cap = r.capacity
    xg = torch.full((cap, H), float("nan"), dtype=dtype, device="cuda")
    gather_rows(p["x"], xg, r.row_map, r.padded_off, k)
    total = int(ref["padded_off"][-1])
    rm = torch.from_numpy(ref["row_map"][:total].astype(np.int64))
    valid = rm >= 0
    exp_xg = torch.zeros(total, H)
    exp_xg[valid] = p["x"].float().cpu()[rm[valid] // k]
    assert torch.equal(xg[:total].float().cpu(), exp_xg)

    act = torch.full((cap, I), float("nan"), dtype=dtype, device="cuda")
    h = torch.full((cap, 2 * I), float("nan"), dtype=dtype, device="cuda")
    up_act_fwd(xg, p["w_fc"], None, p["gate_w"], r.row_map, r.mtile_off, act, h, act_kind)
    re = torch.from_numpy(_row_expert(ref, E)[:total])
    wf = p["w_fc"].float().cpu()
    exp_h = torch.zeros(total, 2 * I)
    for e in range(E):
        rows = re == e
        exp_h[rows] = exp_xg[rows] @ wf[e].t()
    torch.testing.assert_close(h[:total].float().cpu(), exp_h, **TOL[dtype])
    gw = torch.zeros(total)
    gw[valid] = p["gate_w"].float().cpu()[rm[valid]]
    up_, gate_ = exp_h[:, :I], exp_h[:, I:]
    exp_act = gw[:, None] * up_ * (torch.nn.functional.silu(gate_) if act_kind == 0 else torch.sigmoid(gate_))
    torch.testing.assert_close(act[:total].float().cpu(), exp_act, **TOL[dtype])

    # the same kernel reading x by row index itself (cp.async producer warps on the CTA-pair kernels, TMA gather4 on the
    # single-CTA ones): identical bits on every valid row, and the grouped copy it writes back equals the gather kernel's
    from cute_kernels.moe import cta_pair_kernels, up_act_fwd_gather

    act_g = torch.full((cap, I), float("nan"), dtype=dtype, device="cuda")
    h_g = torch.full((cap, 2 * I), float("nan"), dtype=dtype, device="cuda")
    xg_back = torch.full((cap, H), float("nan"), dtype=dtype, device="cuda") if cta_pair_kernels() else None
    up_act_fwd_gather(p["x"], k, p["w_fc"], None, p["gate_w"], r.row_map, r.mtile_off, act_g, h_g, xg_back, act_kind)
    vrows = valid.cuda()
    assert torch.equal(act_g[:total], act[:total])  # pad rows included: they are weighted by zero
    assert torch.equal(h_g[:total][vrows], h[:total][vrows])
    if xg_back is not None:
        assert torch.equal(xg_back[:total], xg[:total])  # zero pad rows included
        # and without the write-back
        act_g2 = torch.full((cap, I), float("nan"), dtype=dtype, device="cuda")
        up_act_fwd_gather(p["x"], k, p["w_fc"], None, p["gate_w"], r.row_map, r.mtile_off, act_g2, None, None, act_kind)
        assert torch.equal(act_g2[:total], act[:total])

    out32 = torch.zeros(T, H, dtype=torch.float32, device="cuda")
    down_combine_fwd(act, p["w_proj"], None, None, r.row_map, r.mtile_off, out32, k)
    af = act[:total].float().cpu()
    wp = p["w_proj"].float().cpu()
    exp_out = torch.zeros(T, H)
    for e in range(E):
        rows = (re == e) & valid
        exp_out.index_add_(0, rm[rows] // k, af[rows] @ wp[e].t())
    torch.testing.assert_close(out32.cpu(), exp_out, **TOL[dtype])


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("act_kind", [0, 1])
@pytest.mark.parametrize("case", MOE_CASES)
def test_fused_backward_pieces(dtype, act_kind, case):
    from cute_kernels import _lib
    from cute_kernels.moe import dgrad_down, dgrad_up

    counts, H, I, k = case
    p = _moe_problem(counts, H, I, k, dtype, seed=1)
    r, ref, E, T = p["r"], p["ref"], p["E"], p["T"]
    total = int(ref["padded_off"][-1])
    rm = torch.from_numpy(ref["row_map"][:total].astype(np.int64))
    valid = rm >= 0
    re = torch.from_numpy(_row_expert(ref, E)[:total])
    dyg = _padded_rows(ref, H, dtype, 5)
    h = _padded_rows(ref, 2 * I, dtype, 6)
    dh = torch.full((r.capacity, 2 * I), float("nan"), dtype=dtype, device="cuda")
    dgates = torch.zeros(T * k, dtype=torch.float32, device="cuda")
    dgrad_down(dyg, p["w_proj"], h, p["gate_w"], r.row_map, r.mtile_off, dh, dgates, None, act_kind)
    # the reproducible form of the router-weight grad: per-part partial sums, then a fixed-order reduction
    from cute_kernels.moe import dgates_parts, reduce_dgates

    dh_p = torch.full((r.capacity, 2 * I), float("nan"), dtype=dtype, device="cuda")
    part = torch.full((dgates_parts(I), r.capacity), float("nan"), dtype=torch.float32, device="cuda")
    dgrad_down(dyg, p["w_proj"], h, p["gate_w"], r.row_map, r.mtile_off, dh_p, None, part, act_kind)
    dgates_p = torch.zeros(T * k, dtype=torch.float32, device="cuda")
    reduce_dgates(part, r.row_map, r.padded_off, E, dgates_p)
    assert torch.equal(dh_p[:total], dh[:total])
    torch.testing.assert_close(dgates_p, dgates, rtol=1e-5, atol=1e-5 * max(1.0, float(dgates.abs().max())))
    part2 = torch.empty_like(part)
    dgrad_down(dyg, p["w_proj"], h, p["gate_w"], r.row_map, r.mtile_off, dh_p, None, part2, act_kind)
    dgates_p2 = torch.zeros(T * k, dtype=torch.float32, device="cuda")
    reduce_dgates(part2, r.row_map, r.padded_off, E, dgates_p2)
    assert torch.equal(dgates_p2, dgates_p), "router-weight grads must be bit-reproducible"

    wp = p["w_proj"].float().cpu()
    g = torch.zeros(total, I)
    for e in range(E):
        rows = re == e
        g[rows] = dyg[:total].float().cpu()[rows] @ wp[e]
    hf = h[:total].float().cpu()
    up_, gate_ = hf[:, :I], hf[:, I:]
    s = torch.sigmoid(gate_)
    if act_kind == 0:
        a = up_ * gate_ * s
        du_m, dg_m = gate_ * s, up_ * (s + gate_ * s * (1 - s))
    else:
        a = up_ * s
        du_m, dg_m = s, up_ * s * (1 - s)
    gw = torch.zeros(total)
    gw[valid] = p["gate_w"].float().cpu()[rm[valid]]
    exp_dh = torch.cat([gw[:, None] * g * du_m, gw[:, None] * g * dg_m], dim=1)
    torch.testing.assert_close(dh[:total].float().cpu(), exp_dh, **TOL[dtype])
    exp_dg = torch.zeros(T * k)
    exp_dg[rm[valid]] = (a * g).sum(-1)[valid]
    tol = {k_: v * max(1.0, I**0.5 / 4) for k_, v in TOL[dtype].items()}
    torch.testing.assert_close(dgates.cpu(), exp_dg, **tol)

    # the same kernel reading un-permuted grad rows by row index: gather any [T, H] matrix both ways
    from cute_kernels.moe import cta_pair_kernels, dgrad_down_gather, gather_rows, wgrad, wgrad_gather

    dy_any = _padded_rows(ref, H, dtype, 12)[:T].contiguous()
    dyg_k = torch.empty(r.capacity, H, dtype=dtype, device="cuda")
    gather_rows(dy_any, dyg_k, r.row_map, r.padded_off, k)
    dh_k = torch.full((r.capacity, 2 * I), float("nan"), dtype=dtype, device="cuda")
    part_k = torch.empty(dgates_parts(I), r.capacity, dtype=torch.float32, device="cuda")
    dgrad_down(dyg_k, p["w_proj"], h, p["gate_w"], r.row_map, r.mtile_off, dh_k, None, part_k, act_kind)
    dh_g = torch.full((r.capacity, 2 * I), float("nan"), dtype=dtype, device="cuda")
    part_g = torch.empty(dgates_parts(I), r.capacity, dtype=torch.float32, device="cuda")
    dyg_back = torch.full((r.capacity, H), float("nan"), dtype=dtype, device="cuda") if cta_pair_kernels() else None
    dgrad_down_gather(dy_any, k, p["w_proj"], h, p["gate_w"], r.row_map, r.mtile_off, dh_g, None, part_g, dyg_back, act_kind)
    assert torch.equal(dh_g[:total], dh_k[:total])
    assert torch.equal(part_g[:, :total], part_k[:, :total])
    if dyg_back is not None:
        assert torch.equal(dyg_back[:total], dyg_k[:total])
    # wgrad with gathered operands against wgrad on pre-gathered copies
    dy2 = _padded_rows(ref, H, dtype, 8)[:T].contiguous()  # any [T, H] matrix
    dyg2 = torch.empty(r.capacity, H, dtype=dtype, device="cuda")
    gather_rows(dy2, dyg2, r.row_map, r.padded_off, k)
    actz = _padded_rows(ref, I, dtype, 9)
    dw_a = torch.empty(E, H, I, dtype=dtype, device="cuda")
    dw_b = torch.empty(E, H, I, dtype=dtype, device="cuda")
    wgrad(dyg2, actz, r.padded_off, dw_a)
    wgrad_gather(dy2, k, actz, 0, r.row_map, r.padded_off, dw_b)
    assert torch.equal(dw_a, dw_b)
    dw_c = torch.empty(E, I, H, dtype=dtype, device="cuda")
    dw_d = torch.empty(E, I, H, dtype=dtype, device="cuda")
    wgrad(actz, dyg2, r.padded_off, dw_c)
    wgrad_gather(actz, 0, dy2, k, r.row_map, r.padded_off, dw_d)
    assert torch.equal(dw_c, dw_d)

    dh_in = _padded_rows(ref, 2 * I, dtype, 7)
    dx32 = torch.zeros(T, H, dtype=torch.float32, device="cuda")
    dgrad_up(dh_in, p["w_fc"], r.row_map, r.mtile_off, dx32, k)
    wf = p["w_fc"].float().cpu()
    exp_dx = torch.zeros(T, H)
    dhf = dh_in[:total].float().cpu()
    for e in range(E):
        rows = (re == e) & valid
        exp_dx.index_add_(0, rm[rows] // k, dhf[rows] @ wf[e])
    tol = {k_: v * max(1.0, (2 * I) ** 0.5 / 4) for k_, v in TOL[dtype].items()}
    torch.testing.assert_close(dx32.cpu(), exp_dx, **tol)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_swiglu_epilogues_on_the_negative_gate_tail(dtype):
    """Gates in [-12, -3]: the 16-bit epilogues compute sigmoid(x) = 0.5 + 0.5 tanh.approx(x / 2), whose absolute error
    (about 2.4e-4 on the sigmoid) is a large RELATIVE error where silu is tiny.  Forward and backward must stay within
    rtol 2e-2 plus an explicit absolute 4e-3 (|gate| * 2.4e-4 * |up| <= 12 * 2.4e-4 * |up|) of the exact fp32 formulas."""
    from cute_kernels.moe import dgrad_down, gather_rows, up_act_fwd

    counts, H, I, k = [130, 70, 0, 56], 64, 128, 2
    p = _moe_problem(counts, H, I, k, dtype, seed=3)
    r, ref, E, T = p["r"], p["ref"], p["E"], p["T"]
    total = int(ref["padded_off"][-1])
    rm = torch.from_numpy(ref["row_map"][:total].astype(np.int64))
    valid = rm >= 0
    tol = dict(rtol=2e-2, atol=4e-3)

    # forward: feature 0 of every token is 1 and W_gate reads only that feature, so gate[j] = -g_j exactly
    x = p["x"].clone()
    x[:, 0] = 1.0
    g_j = torch.linspace(3.0, 12.0, I)
    w_fc = p["w_fc"].clone()
    w_fc[:, I:, :] = 0
    w_fc[:, I:, 0] = (-g_j).to(dtype).cuda()
    xg = torch.empty(r.capacity, H, dtype=dtype, device="cuda")
    gather_rows(x, xg, r.row_map, r.padded_off, k)
    act = torch.full((r.capacity, I), float("nan"), dtype=dtype, device="cuda")
    h = torch.full((r.capacity, 2 * I), float("nan"), dtype=dtype, device="cuda")
    up_act_fwd(xg, w_fc, None, p["gate_w"], r.row_map, r.mtile_off, act, h, 0)
    hf = h[:total].float().cpu()
    assert hf[valid][:, I:].max() <= -2.9 and hf[valid][:, I:].min() >= -12.1
    gw = torch.zeros(total)
    gw[valid] = p["gate_w"].float().cpu()[rm[valid]]
    exp_act = gw[:, None] * hf[:, :I] * torch.nn.functional.silu(hf[:, I:])  # from the kernel's own saved pre-activations
    torch.testing.assert_close(act[:total].float().cpu()[valid], exp_act[valid], **tol)

    # backward: saved pre-activations with the gate half in [-12, -3]
    re = torch.from_numpy(_row_expert(ref, E)[:total])
    dyg = _padded_rows(ref, H, dtype, 5)
    hb = _padded_rows(ref, 2 * I, dtype, 6)
    gen = torch.Generator().manual_seed(7)
    gates = -(3.0 + 9.0 * torch.rand(r.capacity, I, generator=gen))
    gates[torch.from_numpy(ref["row_map"] < 0)] = 0
    hb[:, I:] = gates.to(dtype).cuda()
    dh = torch.full((r.capacity, 2 * I), float("nan"), dtype=dtype, device="cuda")
    dgates = torch.zeros(T * k, dtype=torch.float32, device="cuda")
    dgrad_down(dyg, p["w_proj"], hb, p["gate_w"], r.row_map, r.mtile_off, dh, dgates, None, 0)
    wp = p["w_proj"].float().cpu()
    g = torch.zeros(total, I)
    for e in range(E):
        rows = re == e
        g[rows] = dyg[:total].float().cpu()[rows] @ wp[e]
    hbf = hb[:total].float().cpu()
    up_, gate_ = hbf[:, :I], hbf[:, I:]
    s = torch.sigmoid(gate_)
    exp_dh = torch.cat([gw[:, None] * g * gate_ * s, gw[:, None] * g * up_ * (s + gate_ * s * (1 - s))], dim=1)
    torch.testing.assert_close(dh[:total].float().cpu(), exp_dh, **tol)
    exp_dg = torch.zeros(T * k)
    exp_dg[rm[valid]] = (up_ * gate_ * s * g).sum(-1)[valid]
    torch.testing.assert_close(dgates.cpu(), exp_dg, rtol=2e-2, atol=4e-3 * I**0.5)


def test_sm_budget_changes_the_grid_not_the_result():
    """A grouped GEMM confined to a few SMs (so that another stream's kernels can run beside it) writes the same bits."""
    from cute_kernels import _lib
    from cute_kernels.moe import grouped_linear

    counts, K, N = [700, 900, 0, 131], 512, 1024
    E = len(counts)
    ids, r, ref = _routing(counts, 1)
    x = _padded_rows(ref, K, torch.bfloat16, 1)
    g = torch.Generator().manual_seed(2)
    w = torch.randn(E, N, K, generator=g).mul(0.1).bfloat16().cuda()
    full = torch.empty(x.size(0), N, dtype=torch.bfloat16, device="cuda")
    grouped_linear(x, w, r.mtile_off, full, False)
    total = int(ref["padded_off"][-1])
    all_sms = _lib.lib.ck_gemm_sm_budget()
    assert all_sms == torch.cuda.get_device_properties(0).multi_processor_count
    for sms in (2, 6, all_sms - 16):
        y = torch.full_like(full, float("nan"))
        with _lib.gemm_sm_budget(sms):
            assert _lib.lib.ck_gemm_sm_budget() == sms
            grouped_linear(x, w, r.mtile_off, y, False)
        assert _lib.lib.ck_gemm_sm_budget() == all_sms
        assert torch.equal(y[:total].view(torch.int16), full[:total].view(torch.int16))


def test_bad_arguments_are_rejected():
    from cute_kernels import _lib

    x = torch.zeros(128, 60, dtype=torch.bfloat16, device="cuda")  # K not a multiple of 8
    w = torch.zeros(1, 64, 60, dtype=torch.bfloat16, device="cuda")
    off = torch.tensor([0, 1], dtype=torch.int32, device="cuda")
    y = torch.zeros(128, 64, dtype=torch.bfloat16, device="cuda")
    st = _lib.lib.ck_moe_grouped_linear(x.data_ptr(), w.data_ptr(), off.data_ptr(), y.data_ptr(), 1, 128, 64, 60, 0, 2,
                                        None, None)
    assert st == -1


@pytest.mark.expects_dev_status
def test_capacity_guard_flags_instead_of_overrunning():
    """Tile tables that describe more rows than were allocated: the kernel refuses and flags CK_DEV_META."""
    import cute_kernels
    from cute_kernels import _lib
    from cute_kernels.moe import grouped_linear

    x = torch.zeros(128, 64, dtype=torch.bfloat16, device="cuda")
    w = torch.zeros(1, 64, 64, dtype=torch.bfloat16, device="cuda")
    off = torch.tensor([0, 5], dtype=torch.int32, device="cuda")  # claims 5 tiles, only 1 allocated
    y = torch.zeros(128, 64, dtype=torch.bfloat16, device="cuda")
    grouped_linear(x, w, off, y, False)
    with pytest.raises(RuntimeError, match="CK_DEV_META"):
        cute_kernels.check_device_status()
