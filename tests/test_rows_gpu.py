"""Row permutation kernels, the scatter-store grouped linear and the expert-shard function (1 GPU)."""

import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist

import ck_oracle as orc

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
@pytest.mark.parametrize("T,k,H", [(1, 1, 8), (33, 2, 64), (257, 8, 136), (1000, 4, 512), (65, 6, 2056), (40, 3, 4096)])
def test_gather_combine_dots(dtype, T, k, H):
    from cute_kernels.moe import combine_rows, gather_rows_scaled, row_dots

    g = torch.Generator().manual_seed(T + k)
    x = torch.randn(T, H, generator=g).to(dtype).cuda()
    w = torch.rand(T * k, generator=g).to(dtype).cuda()
    perm = torch.randperm(T * k, generator=g)
    idx = perm.to(torch.int32).cuda()                      # sorted position j -> flat slot
    pos = torch.empty_like(idx)
    pos[idx.long()] = torch.arange(T * k, dtype=torch.int32, device="cuda")

    rows = torch.full((T * k, H), float("nan"), dtype=dtype, device="cuda")
    gather_rows_scaled(x, rows, idx, None, k)
    assert torch.equal(rows, x[(idx.long() // k)])
    gather_rows_scaled(x, rows, idx, w, k)
    exp = (x.float()[idx.long() // k] * w.float()[idx.long()].unsqueeze(1)).to(dtype)
    torch.testing.assert_close(rows, exp, rtol=1e-2 if dtype != torch.float32 else 1e-6, atol=1e-6)
    idx2 = idx.clone()
    idx2[0] = -1
    gather_rows_scaled(x, rows, idx2, None, k)
    assert (rows[0] == 0).all()

    src = torch.randn(T * k, H, generator=g).to(dtype).cuda()
    out = torch.empty(T, H, dtype=dtype, device="cuda")
    combine_rows(src, pos, w, out, k)
    exp = (src.float()[pos.long()].view(T, k, H) * w.float().view(T, k, 1)).sum(1)
    tol = dict(rtol=2e-2, atol=2e-2) if dtype != torch.float32 else dict(rtol=1e-5, atol=1e-5)
    torch.testing.assert_close(out.float(), exp, **tol)
    combine_rows(src, pos, None, out, k)
    torch.testing.assert_close(out.float(), src.float()[pos.long()].view(T, k, H).sum(1), **tol)
    # no position table: the k rows of token t are rows t*k .. t*k+k-1; a missing row (-1) contributes nothing
    combine_rows(src, None, None, out, k)
    torch.testing.assert_close(out.float(), src.float().view(T, k, H).sum(1), **tol)
    pos2 = pos.clone()
    pos2[::k] = -1
    combine_rows(src, pos2, None, out, k)
    keep = torch.ones(T, k, 1)
    keep[:, 0] = 0
    torch.testing.assert_close(out.float().cpu(), (src.float().cpu()[pos.long().cpu()].view(T, k, H) * keep).sum(1), **tol)

    dots = torch.empty(T * k, dtype=dtype, device="cuda")
    row_dots(src, pos, x, dots, k)
    exp = (src.float()[pos.long()] * x.float().repeat_interleave(k, 0)).sum(1)
    tol = dict(rtol=2e-2, atol=2e-2 * H**0.5 / 4) if dtype != torch.float32 else dict(rtol=1e-4, atol=1e-4)
    torch.testing.assert_close(dots.float(), exp, **tol)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_expert_shard_matches_oracle(dtype):
    from cute_kernels.moe import expert_shard

    E, H, I, n = 4, 128, 192, 700
    g = torch.Generator().manual_seed(3)
    ids = torch.randint(0, E, (n,), generator=g)
    ids[ids == 2] = 1  # leave one expert without rows
    rows = torch.randn(n, H, generator=g)
    w_fc = 0.05 * torch.randn(E, 2 * I, H, generator=g)
    w_proj = 0.05 * torch.randn(E, H, I, generator=g)
    dy = torch.randn(n, H, generator=g)
    rc = rows.clone().requires_grad_()
    wfc_c, wproj_c = w_fc.clone().requires_grad_(), w_proj.clone().requires_grad_()
    yr = orc.moe_experts_ref(rc, torch.ones(n, 1), ids.view(-1, 1), wfc_c, wproj_c, orc.swiglu_packed_ref)
    yr.backward(dy)
    rk = rows.to(dtype).cuda().requires_grad_()
    wfc_k, wproj_k = w_fc.to(dtype).cuda().requires_grad_(), w_proj.to(dtype).cuda().requires_grad_()
    y = expert_shard(rk, ids.cuda(), wfc_k, wproj_k)
    y.backward(dy.to(dtype).cuda())
    tol = dict(rtol=2e-2, atol=2e-2) if dtype == torch.bfloat16 else dict(rtol=6e-3, atol=6e-3)
    torch.testing.assert_close(y.float().cpu(), yr.detach(), **tol)
    torch.testing.assert_close(rk.grad.float().cpu(), rc.grad, **tol)
    wtol = {k_: v * 4 for k_, v in tol.items()}
    torch.testing.assert_close(wfc_k.grad.float().cpu(), wfc_c.grad, **wtol)
    torch.testing.assert_close(wproj_k.grad.float().cpu(), wproj_c.grad, **wtol)
    assert (wfc_k.grad[2] == 0).all() and (wproj_k.grad[2] == 0).all()  # the empty expert gets exact zeros


def test_expert_parallel_single_rank_group():
    """World size 1 over NCCL: the whole dispatch / return / combine path with the exchange being a self copy."""
    import cute_kernels as ck

    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("nccl", rank=0, world_size=1, device_id=torch.device("cuda", 0))
    try:
        cfg = dict(T=300, H=128, I=256, E=8, k=2)
        inp = orc.gen_moe_inputs(0, **cfg)
        ref = orc.moe_fwd_bwd_ref(inp)
        dt = torch.bfloat16
        x = inp["x"].to(dt).cuda().requires_grad_()
        rw = inp["router_weights"].to(dt).cuda().requires_grad_()
        w_fc = inp["w_fc"].to(dt).cuda().requires_grad_()
        w_proj = inp["w_proj"].to(dt).cuda().requires_grad_()
        ep = ck.ExpertParallelMoE(cfg["E"], cfg["k"])
        y = ep(x, rw, inp["selected_experts"].cuda(), w_fc, w_proj)
        y.backward(inp["grad_out"].to(dt).cuda())
        tol = dict(rtol=2e-2, atol=2e-2)
        torch.testing.assert_close(y.float().cpu(), ref["y"], **tol)
        torch.testing.assert_close(x.grad.float().cpu(), ref["dx"], **tol)
        torch.testing.assert_close(rw.grad.float().cpu(), ref["d_router_weights"], **tol)
        wtol = dict(rtol=2e-2, atol=6e-2)
        torch.testing.assert_close(w_fc.grad.float().cpu(), ref["d_w_fc"], **wtol)
        torch.testing.assert_close(w_proj.grad.float().cpu(), ref["d_w_proj"], **wtol)
    finally:
        dist.destroy_process_group()
