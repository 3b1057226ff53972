"""Expert-parallel dispatch / return logic on CPU ranks (gloo), with the oracle as the expert math.

Contract: G ranks, each with its own tokens and E/G experts, must reproduce the single-process layer that
holds all E experts on the concatenated batch -- forward, input grads, router-weight grads and the
expert-weight grads of the local shard."""

import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import ck_oracle as orc


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _cpu_route(ids, num_experts):
    srt = torch.sort(ids, stable=True)
    return srt.indices.to(torch.int32), torch.bincount(ids, minlength=num_experts)


def _cpu_experts(rows, local_ids, w_fc, w_proj, act_kind):
    ones = torch.ones(rows.size(0), 1, dtype=rows.dtype)
    return orc.moe_experts_ref(rows, ones, local_ids.view(-1, 1), w_fc, w_proj, orc.swiglu_packed_ref)


def _worker(rank, world, port, cfg, out_dir):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from cute_kernels.expert_parallel import ExpertParallelMoE, gather_expert_state_dict, shard_expert_state_dict

        E, k, T = cfg["E"], cfg["k"], cfg["T"]
        full = orc.gen_moe_inputs(cfg["seed"], T * world, cfg["H"], cfg["I"], E, k, cfg["expert_bias"])
        sl = slice(rank * T, (rank + 1) * T)
        epr = E // world
        x = full["x"][sl].clone().requires_grad_()
        rw = full["router_weights"][sl].clone().requires_grad_()
        w_fc = full["w_fc"][rank * epr : (rank + 1) * epr].clone().requires_grad_()
        w_proj = full["w_proj"][rank * epr : (rank + 1) * epr].clone().requires_grad_()
        ep = ExpertParallelMoE(E, k, None, expert_fn=_cpu_experts, route_fn=_cpu_route)
        y = ep(x, rw, full["selected_experts"][sl], w_fc, w_proj)
        y.backward(full["grad_out"][sl])
        torch.save(dict(y=y.detach(), dx=x.grad, d_router_weights=rw.grad, d_w_fc=w_fc.grad, d_w_proj=w_proj.grad),
                   os.path.join(out_dir, f"rank{rank}.pt"))
        # state-dict helpers round-trip
        sd = {"gate.weight": torch.arange(E * 4.0).view(E, 4), "c_fc.weight": full["w_fc"], "c_proj.weight": full["w_proj"]}
        local = shard_expert_state_dict(sd, rank, world)
        assert local["c_fc.weight"].shape[0] == epr
        back = gather_expert_state_dict(local)
        for key in sd:
            assert torch.equal(back[key], sd[key]), key
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("cfg", [
    dict(E=8, k=2, T=96, H=32, I=48, expert_bias=False, seed=0),
    dict(E=4, k=4, T=50, H=16, I=24, expert_bias=True, seed=1),   # skewed routing: uneven splits, every expert hit by every token
    dict(E=16, k=1, T=7, H=16, I=8, expert_bias=False, seed=2),   # some experts (and maybe a whole rank) get no rows
])
def test_expert_parallel_matches_single_process(tmp_path, cfg):
    world = 2
    mp.spawn(_worker, args=(world, _free_port(), cfg, str(tmp_path)), nprocs=world, join=True)
    full = orc.gen_moe_inputs(cfg["seed"], cfg["T"] * world, cfg["H"], cfg["I"], cfg["E"], cfg["k"], cfg["expert_bias"])
    ref = orc.moe_fwd_bwd_ref(full)
    epr = cfg["E"] // world
    for rank in range(world):
        got = torch.load(os.path.join(tmp_path, f"rank{rank}.pt"))
        sl = slice(rank * cfg["T"], (rank + 1) * cfg["T"])
        el = slice(rank * epr, (rank + 1) * epr)
        torch.testing.assert_close(got["y"], ref["y"][sl], rtol=1e-5, atol=1e-6)
        torch.testing.assert_close(got["dx"], ref["dx"][sl], rtol=1e-5, atol=1e-6)
        torch.testing.assert_close(got["d_router_weights"], ref["d_router_weights"][sl], rtol=1e-5, atol=1e-6)
        torch.testing.assert_close(got["d_w_fc"], ref["d_w_fc"][el], rtol=1e-5, atol=1e-6)
        torch.testing.assert_close(got["d_w_proj"], ref["d_w_proj"][el], rtol=1e-5, atol=1e-6)
