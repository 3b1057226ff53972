"""Expert parallelism over peer memory, emulated on one GPU: every virtual rank owns its buffers, the pointer tables
name all of them, and the phases run in lock step (the place of the collectives) -- the kernels, the slot arithmetic
and the autograd bookkeeping are the ones the multi-GPU run uses.  Checked against the CPU oracle on the
concatenated batch."""

import pytest
import torch

import ck_oracle as orc

pytestmark = pytest.mark.gpu


def _virtual_world(world, max_tokens, H, k, dt):
    from cute_kernels.peer_parallel import PeerBuffers, packed_publication

    S = max_tokens * k
    dev = torch.device("cuda")
    raw = []
    for _ in range(world):
        published, ids, weights = packed_publication(S, dt, dev)
        raw.append(dict(tokens=torch.full((max_tokens, H), float("nan"), dtype=dt, device=dev),
                        rows=torch.full((S, H), float("nan"), dtype=dt, device=dev),
                        weights=weights, dgates=torch.full((S,), float("nan"), dtype=torch.float32, device=dev),
                        ids=ids, published=published))
    ptrs = {name: [r[name].data_ptr() for r in raw] for name in ("tokens", "rows", "dgates")}
    return [PeerBuffers(rank, world, max_tokens, k, raw[rank]["tokens"], raw[rank]["rows"], raw[rank]["weights"],
                        raw[rank]["dgates"], raw[rank]["ids"], ptrs["tokens"], ptrs["rows"], ptrs["dgates"],
                        raw[rank]["published"])
            for rank in range(world)]


CASES = [
    dict(world=2, E=8, k=2, T=[300, 300], H=128, I=256, seed=0),
    dict(world=4, E=8, k=2, T=[130, 97, 5, 256], H=64, I=72, seed=1),     # ragged ranks, discard bin in use
    dict(world=4, E=4, k=1, T=[64, 64, 64, 64], H=128, I=128, seed=2),    # one expert per rank, top-1
    dict(world=2, E=16, k=4, T=[257, 0], H=64, I=136, seed=3),            # a rank without tokens
    dict(world=8, E=8, k=2, T=[40] * 8, H=256, I=128, seed=4),
    dict(world=2, E=8, k=2, T=[300, 300], H=128, I=256, seed=5, min_tiles_to_split=4),   # two-window pull, small
    dict(world=2, E=4, k=2, T=[1500, 1400], H=64, I=64, seed=6, min_tiles_to_split=16),  # two-window pull, larger
    dict(world=4, E=8, k=2, T=[130, 97, 5, 256], H=64, I=72, seed=7, fused_pull=True),   # rows pulled by the GEMM's own producer warp
    dict(world=2, E=16, k=4, T=[257, 0], H=64, I=136, seed=8, fused_pull=True),
    dict(world=4, E=8, k=2, T=[130, 97, 5, 256], H=64, I=72, seed=9, capacity=4.0),      # no read-back of the row count
    dict(world=2, E=8, k=2, T=[300, 300], H=128, I=256, seed=10, capacity=1.5, placement=[1, 0, 0, 1, 1, 0, 1, 0]),
    dict(world=4, E=16, k=4, T=[200, 190, 210, 64], H=64, I=136, seed=11, placement="balanced", expert_bias=True),
]


@pytest.mark.parametrize("dt", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("cfg", CASES)
def test_peer_engine_lockstep(cfg, dt):
    import cute_kernels as ck
    from cute_kernels.peer_parallel import PeerExpertEngine

    world, E, k, H, I = cfg["world"], cfg["E"], cfg["k"], cfg["H"], cfg["I"]
    Ts = cfg["T"]
    full = orc.gen_moe_inputs(cfg["seed"], sum(Ts), H, I, E, k, cfg.get("expert_bias", False))
    ref = orc.moe_fwd_bwd_ref(full)
    epr = E // world
    starts = [sum(Ts[:r]) for r in range(world)]
    sl = [slice(starts[r], starts[r] + Ts[r]) for r in range(world)]
    max_tokens = max(max(Ts), 1)
    bufs = _virtual_world(world, max_tokens, H, k, dt)
    placement = cfg.get("placement")
    if placement == "balanced":  # experts spread over the ranks by the rows they receive
        loads = torch.bincount(full["selected_experts"].reshape(-1), minlength=E).tolist()
        placement = ck.balanced_expert_placement(loads, world)
        per_rank = [sum(loads[e] for e in range(E) if placement[e] == r) for r in range(world)]
        blocks = [sum(loads[r * epr:(r + 1) * epr]) for r in range(world)]
        assert max(per_rank) <= max(blocks)
    cap_rows = None if "capacity" not in cfg else int(cfg["capacity"] * max_tokens * k) + epr * 128
    eng = [PeerExpertEngine(b, E, expert_to_rank=placement, capacity_rows=cap_rows) for b in bufs]
    for e in eng:
        e.MIN_TILES_TO_SPLIT = cfg.get("min_tiles_to_split", e.MIN_TILES_TO_SPLIT)
        e.FUSED_PULL = cfg.get("fused_pull", False)
    owned_ids = [e.local_expert_ids for e in eng]
    w_fc = [full["w_fc"][owned_ids[r]].to(dt).cuda().contiguous() for r in range(world)]
    w_proj = [full["w_proj"][owned_ids[r]].to(dt).cuda().contiguous() for r in range(world)]

    # ---- forward, phase by phase ----
    for r in range(world):
        eng[r].publish(full["x"][sl[r]].to(dt).cuda(), full["router_weights"][sl[r]].to(dt).cuda(),
                       full["selected_experts"][sl[r]].to(torch.int32).cuda())
    # the all-gather of the packed (ids | weights) buffers, done by hand
    ids_all, weights_all = bufs[0].split_published(torch.cat([b.published for b in bufs]))
    assert torch.equal(ids_all, torch.cat([b.ids for b in bufs]))
    plans = [eng[r].plan(ids_all) for r in range(world)]
    owned = sum(int(p.routing.counts[:epr].long().sum()) for p in plans)
    assert owned == sum(Ts) * k                       # every routed row has exactly one owner
    if cfg["seed"] in (5, 6):
        assert all(p.split > 0 for p in plans)        # these cases exercise the overlapped two-window pull
    saved = [eng[r].fwd_compute(plans[r], weights_all, w_fc[r], w_proj[r], True) for r in range(world)]
    ys = [eng[r].fwd_finish(Ts[r]) for r in range(world)]
    # ---- backward ----
    for r in range(world):
        eng[r].bwd_publish(full["grad_out"][sl[r]].to(dt).cuda())
    grads = [eng[r].bwd_compute(plans[r], saved[r], weights_all, w_fc[r], w_proj[r], True, True, True) for r in range(world)]
    backs = [eng[r].bwd_finish(Ts[r], True) for r in range(world)]
    torch.cuda.synchronize()
    ck.check_device_status()

    tol = dict(rtol=2e-2, atol=2e-2) if dt == torch.bfloat16 else dict(rtol=6e-3, atol=6e-3)  # fp32 runs as TF32
    n = sum(Ts)
    wtol = dict(rtol=tol["rtol"], atol=tol["atol"] * max(1.0, (n / 64) ** 0.5))
    for r in range(world):
        el = owned_ids[r]
        torch.testing.assert_close(ys[r].float().cpu(), ref["y"][sl[r]], **tol)
        dx, d_rw = backs[r]
        torch.testing.assert_close(dx.float().cpu(), ref["dx"][sl[r]], **tol)
        torch.testing.assert_close(d_rw.float().cpu(), ref["d_router_weights"][sl[r]],
                                   rtol=tol["rtol"], atol=tol["atol"] * max(1.0, (I / 256) ** 0.5))
        torch.testing.assert_close(grads[r][0].float().cpu(), ref["d_w_fc"][el], **wtol)
        torch.testing.assert_close(grads[r][1].float().cpu(), ref["d_w_proj"][el], **wtol)


def test_peer_plan_rejects_out_of_range_ids():
    from cute_kernels.peer_parallel import PeerExpertEngine

    bufs = _virtual_world(2, 16, 64, 2, torch.bfloat16)
    eng = PeerExpertEngine(bufs[0], 8)
    ids = torch.randint(0, 8, (2 * 32,), dtype=torch.int32, device="cuda")
    ids[5] = 9
    with pytest.raises(RuntimeError, match="outside"):
        eng.plan(ids)
    ids[5] = 8          # the padding value of unused slots is fine
    assert eng.plan(ids).rows % 128 == 0


def test_peer_kernels_reject_bad_tables():
    from cute_kernels import _lib
    import ctypes

    x = torch.zeros(128, 64, dtype=torch.bfloat16, device="cuda")
    i32 = torch.zeros(130, dtype=torch.int32, device="cuda")
    arr = (ctypes.c_void_p * 1)(x.data_ptr() + 2)  # misaligned buffer
    st = _lib.lib.ck_moe_gather_rows_peer(arr, 1, 128, x.data_ptr(), i32.data_ptr(), i32.data_ptr(), i32.data_ptr(), 1, 128, 1,
                                          64, 0, 128, _lib.dtype_code(torch.bfloat16), None, None)
    assert st == -1
    arr = (ctypes.c_void_p * 1)(x.data_ptr())
    st = _lib.lib.ck_peer_gather_scalars(arr, 17, 128, i32.data_ptr(), 1, x.data_ptr(), 2, None, None)   # too many peers
    assert st == -1
    st = _lib.lib.ck_peer_gather_scalars(arr, 1, 1 << 31, i32.data_ptr(), 1, x.data_ptr(), 2, None, None)  # slots overflow int32
    assert st == -2


def test_peer_scalar_kernels():
    from cute_kernels import _lib
    import ctypes

    S, world = 50, 3
    bufs = [torch.arange(S, device="cuda", dtype=torch.float32) + 100 * r for r in range(world)]
    arr = (ctypes.c_void_p * world)(*[b.data_ptr() for b in bufs])
    flat = torch.tensor([0, 49, 50, 149, 77], dtype=torch.int32, device="cuda")
    out = torch.empty(5, dtype=torch.float32, device="cuda")
    assert _lib.lib.ck_peer_gather_scalars(arr, world, S, flat.data_ptr(), 5, out.data_ptr(), 4, None, None) == 0
    assert out.tolist() == [0.0, 49.0, 100.0, 249.0, 127.0]
    vals = torch.arange(world * S, device="cuda", dtype=torch.float32) * -1.0
    flat2 = torch.tensor([3, -1, 60, 149], dtype=torch.int32, device="cuda")
    assert _lib.lib.ck_peer_scatter_scalars(vals.data_ptr(), flat2.data_ptr(), 4, 1, arr, world, S, 4, None, None) == 0
    assert bufs[0][3].item() == -3.0 and bufs[1][10].item() == -60.0 and bufs[2][49].item() == -149.0
    assert _lib.lib.ck_peer_scatter_scalars(vals.data_ptr(), flat2.data_ptr(), 4, 0, arr, world, S, 4, None, None) == 0
    assert bufs[0][3].item() == 0.0 and bufs[1][10].item() == -2.0 and bufs[2][49].item() == -3.0
    assert bufs[0][4].item() == 4.0   # untouched neighbours


def test_combine_rows_identity_positions():
    from cute_kernels.moe import combine_rows

    src = torch.randn(24, 64, device="cuda").bfloat16()
    out = torch.empty(8, 64, device="cuda", dtype=torch.bfloat16)
    combine_rows(src, None, None, out, 3)
    torch.testing.assert_close(out.float(), src.float().view(8, 3, 64).sum(1), rtol=1e-2, atol=1e-2)
