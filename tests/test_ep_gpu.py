"""Expert parallelism on real GPUs against the CPU oracle, over both transports: NCCL all-to-all around the fused
grouped-GEMM path, and peer-memory loads / stores issued by the kernels themselves (symmetric memory).
Needs at least 2 GPUs; skipped otherwise."""

import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import ck_oracle as orc

pytestmark = pytest.mark.gpu


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, cfg, out_dir):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        import cute_kernels as ck
        from cute_kernels.expert_parallel import ExpertParallelMoE

        E, k, T = cfg["E"], cfg["k"], cfg["T"]
        full = orc.gen_moe_inputs(cfg["seed"], T * world, cfg["H"], cfg["I"], E, k, cfg["expert_bias"])
        sl = slice(rank * T, (rank + 1) * T)
        epr = E // world
        dt = torch.bfloat16
        x = full["x"][sl].to(dt).cuda().requires_grad_()
        rw = full["router_weights"][sl].to(dt).cuda().requires_grad_()
        w_fc = full["w_fc"][rank * epr : (rank + 1) * epr].to(dt).cuda().requires_grad_()
        w_proj = full["w_proj"][rank * epr : (rank + 1) * epr].to(dt).cuda().requires_grad_()
        if cfg.get("transport") == "peer":
            from cute_kernels.peer_parallel import PeerExpertParallelMoE

            ep = PeerExpertParallelMoE(E, k, T + 7, cfg["H"], dt, None)   # buffers larger than the batch
        else:
            ep = ExpertParallelMoE(E, k, None, chunks=cfg.get("chunks", 1))
        y = ep(x, rw, full["selected_experts"][sl].cuda(), w_fc, w_proj)
        y.backward(full["grad_out"][sl].to(dt).cuda())
        torch.cuda.synchronize()
        ck.check_device_status()
        torch.save({n: v.float().cpu() for n, v in dict(y=y.detach(), dx=x.grad, d_router_weights=rw.grad, d_w_fc=w_fc.grad,
                                                        d_w_proj=w_proj.grad).items()}, os.path.join(out_dir, f"rank{rank}.pt"))
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
@pytest.mark.parametrize("cfg", [dict(E=8, k=2, T=300, H=128, I=256, expert_bias=False, seed=0),
                                 dict(E=16, k=4, T=257, H=64, I=72, expert_bias=True, seed=1),
                                 dict(E=8, k=2, T=300, H=128, I=256, expert_bias=False, seed=0, chunks=2),
                                 dict(E=16, k=4, T=257, H=64, I=72, expert_bias=True, seed=1, chunks=3),
                                 dict(E=8, k=2, T=300, H=128, I=256, expert_bias=False, seed=0, transport="peer"),
                                 dict(E=2, k=1, T=513, H=256, I=128, expert_bias=True, seed=2, transport="peer")])
def test_expert_parallel_two_gpus(tmp_path, cfg):
    world = 2
    mp.spawn(_worker, args=(world, _free_port(), cfg, str(tmp_path)), nprocs=world, join=True)
    full = orc.gen_moe_inputs(cfg["seed"], cfg["T"] * world, cfg["H"], cfg["I"], cfg["E"], cfg["k"], cfg["expert_bias"])
    ref = orc.moe_fwd_bwd_ref(full)
    epr = cfg["E"] // world
    tol = dict(rtol=2e-2, atol=2e-2)
    for rank in range(world):
        got = torch.load(os.path.join(tmp_path, f"rank{rank}.pt"))
        sl = slice(rank * cfg["T"], (rank + 1) * cfg["T"])
        el = slice(rank * epr, (rank + 1) * epr)
        torch.testing.assert_close(got["y"], ref["y"][sl], **tol)
        torch.testing.assert_close(got["dx"], ref["dx"][sl], **tol)
        torch.testing.assert_close(got["d_router_weights"], ref["d_router_weights"][sl], **tol)
        wtol = dict(rtol=2e-2, atol=2e-2 * max(1.0, (cfg["T"] * world / 64) ** 0.5))
        torch.testing.assert_close(got["d_w_fc"], ref["d_w_fc"][el], **wtol)
        torch.testing.assert_close(got["d_w_proj"], ref["d_w_proj"][el], **wtol)
