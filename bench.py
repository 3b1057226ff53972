"""Benchmark of the MoE expert path: forward + backward tokens/s on the Mixtral-shaped layer.

  python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference] [--workload c4|c5|c1]

One "step" is one forward + backward of the expert path (route -> gather -> up+SwiGLU -> down+combine ->
backward) over one synthetic batch with the shapes of the named configuration, bf16.  Rank 0 prints one
JSON line.  ``value`` is timed with CUDA events with the inputs resident in HBM; ``e2e`` repeats the
measurement with pinned host buffers, the host<->device copies inside the timed region.  ``roofline`` is the
grouped-GEMM kernel family against the measured dense bf16 peak; ``cpu_baseline`` is the CPU oracle port of
the reference's torch path timed on the host cores on a bounded sample.

With --gpus N > 1 (launched by torch.distributed.run, one rank per GPU) the experts are partitioned across
the ranks and tokens travel by NCCL all-to-all (weak scaling: every rank brings its own T tokens).

``--impl reference`` times the CPU oracle port alone (rank 0 only) and prints the same line with
``"impl": "reference"``.
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
for _p in (os.path.join(ROOT, "cute-kernels_b200"), os.path.join(ROOT, "oracle")):
    if _p not in sys.path:
        sys.path.insert(0, _p)

import torch  # noqa: E402

WORKLOADS = {
    "c4": dict(name="c4_mixtral_moe_fwd_bwd", T=16384, H=4096, I=14336, E=8, k=2, expert_bias=False),
    "c5": dict(name="c5_finegrained_moe_fwd_bwd", T=32768, H=2048, I=1408, E=64, k=8, expert_bias=True),
    # profiling-sized slice of c4: same hidden / intermediate sizes, 4 experts, 2048 tokens (weights > L2, ~4 GB held)
    "c4s": dict(name="c4_slice_moe_fwd_bwd", T=2048, H=4096, I=14336, E=4, k=2, expert_bias=False),
    "c1": dict(name="c1_small_moe_fwd_bwd", T=512, H=256, I=512, E=8, k=2, expert_bias=False),
}
COMBINE_ROWS = {"auto": None, "red": False, "rows": True}  # --combine -> fused_experts(deterministic=...)
METRIC = "moe_fwd_bwd_tokens_per_s"
UNIT = "tokens/s"
GEMM_KERNELS = ("up_act_fwd", "down_combine_fwd", "dgrad_down", "dgrad_up", "wgrad", "grouped_linear",
                "grouped_linear_scatter", "grouped_linear_scatter_peer", "up_act_fwd_peer", "dgrad_down_peer")


def measured_peaks() -> dict:
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            return dict(json.load(f), source="measured")
    except OSError:
        return dict(hbm_gbs=6650.0, bf16_tflops=1590.0, bf16_tflops_sustained=1400.0, source="fallback")


def host_info() -> tuple[int, str]:
    model = "unknown"
    try:
        for line in open("/proc/cpuinfo"):
            if line.startswith("model name"):
                model = line.split(":", 1)[1].strip()
                break
    except OSError:
        pass
    return os.cpu_count() or 1, model


def bind_to_gpu_numa_node(device_index: int) -> int | None:
    """Runs this process on the CPUs of the NUMA node the GPU hangs off, so that the pinned staging buffers it allocates
    afterwards (first touch) and the copies it issues stay on that node's memory and PCIe root.  Reads sysfs only; returns
    the node, or None when the topology is not exposed (single-node hosts, containers without the PCI tree)."""
    try:
        prop = torch.cuda.get_device_properties(device_index)
        bdf = f"{prop.pci_domain_id:04x}:{prop.pci_bus_id:02x}:{prop.pci_device_id:02x}.0"
        with open(f"/sys/bus/pci/devices/{bdf}/numa_node") as f:
            node = int(f.read().strip())
        if node < 0:
            return None
        with open(f"/sys/devices/system/node/node{node}/cpulist") as f:
            cpus: set[int] = set()
            for part in f.read().strip().split(","):
                lo, _, hi = part.partition("-")
                cpus.update(range(int(lo), int(hi or lo) + 1))
        allowed = cpus & os.sched_getaffinity(0)
        if not allowed:
            return None
        os.sched_setaffinity(0, allowed)
        return node
    except (OSError, ValueError, AttributeError):
        return None


# ---------------------------------------------------------------------------------------------------
# synthetic inputs
# ---------------------------------------------------------------------------------------------------
def make_device_inputs(w: dict, device: torch.device, seed: int, experts: slice | None = None) -> dict:
    """x ~ N(0,1), router logits ~ N(0,1) (+ per-expert bias for c5), weights ~ N(0, 0.02), grad ~ N(0,1);
    generated on the device (random init of the named architecture; parity uses the seeded CPU generator)."""
    g = torch.Generator(device=device).manual_seed(seed)
    T, H, I, E, k = w["T"], w["H"], w["I"], w["E"], w["k"]
    dt = torch.bfloat16
    x = torch.randn(T, H, generator=g, device=device, dtype=torch.float32).to(dt)
    logits = torch.randn(T, E, generator=g, device=device)
    if w["expert_bias"]:
        gb = torch.Generator(device=device).manual_seed(12345)  # the same expert bias on every rank
        logits = logits + torch.randn(E, generator=gb, device=device)
    vals, sel = logits.topk(k, dim=-1) if k > 1 else logits.max(dim=-1, keepdim=True)
    rw = torch.softmax(vals.float(), dim=-1).to(dt)
    e0, e1 = (0, E) if experts is None else (experts.start, experts.stop)
    gw = torch.Generator(device=device).manual_seed(777)
    w_fc = torch.empty(e1 - e0, 2 * I, H, device=device, dtype=dt).normal_(0, 0.02, generator=gw)
    w_proj = torch.empty(e1 - e0, H, I, device=device, dtype=dt).normal_(0, 0.02, generator=gw)
    grad_out = torch.randn(T, H, generator=g, device=device, dtype=torch.float32).to(dt)
    return dict(x=x, router_weights=rw, selected_experts=sel, w_fc=w_fc, w_proj=w_proj, grad_out=grad_out)


# ---------------------------------------------------------------------------------------------------
# clocks
# ---------------------------------------------------------------------------------------------------
class ClockSampler:
    FIELDS = ("timestamp,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int) -> None:
        self.path = tempfile.mktemp(prefix="ck_clocks_", suffix=".csv")
        self.proc = None
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "100", "-i", str(gpu_index)],
                stdout=open(self.path, "w"), stderr=subprocess.DEVNULL)
        except OSError:
            self.proc = None

    def mark_begin(self) -> None:
        self.t_begin = time.time()

    def mark_end(self) -> None:
        self.t_end = time.time()

    def stop(self) -> dict:
        """Median SM clock and the throttle reasons seen between mark_begin() and mark_end()."""
        import datetime

        out = dict(sm_mhz=None, sm_max_mhz=None, reasons=[], samples=0)
        if self.proc is None:
            return out
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        rows = []
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        try:
            for line in open(self.path):
                parts = [p.strip() for p in line.split(",")]
                if len(parts) < 8:
                    continue
                try:
                    ts = datetime.datetime.strptime(parts[0], "%Y/%m/%d %H:%M:%S.%f").timestamp()
                    rows.append((ts, float(parts[1]), float(parts[2]), float(parts[3]),
                                 [n for n, v in zip(names, parts[4:8]) if v.lower().startswith("active")]))
                except ValueError:
                    continue
            os.unlink(self.path)
        except OSError:
            pass
        t0, t1 = getattr(self, "t_begin", 0.0), getattr(self, "t_end", float("inf"))
        inside = [r for r in rows if t0 <= r[0] <= t1 + 0.1]
        window = "timed_region"
        if not inside:  # region shorter than the sampling period: use the samples since warm-up began
            inside, window = rows, "warmup_and_timed_region"
        if inside:
            out.update(sm_mhz=statistics.median(r[1] for r in inside), sm_max_mhz=max(r[2] for r in inside),
                       reasons=sorted({n for r in inside for n in r[4]}), samples=len(inside),
                       power_w_max=max(r[3] for r in inside), window=window)
        return out


# ---------------------------------------------------------------------------------------------------
# the CPU arm (oracle port of the reference's torch path)
# ---------------------------------------------------------------------------------------------------
def cpu_arm(w: dict, steps: int, warmup: int, budget_s: float) -> dict:
    """Times the CPU restatement of MoE_Torch's expert path (oracle/ck_oracle.py) with every host thread.

    The sample keeps the layer's hidden / intermediate sizes and top-k but instantiates only E_s experts and
    T_s tokens: FLOPs per token are those of the full workload, while the reference's autograd cost that
    grows with E * weight bytes (index-select backward of ``weight[e]``) stays inside the time budget."""
    import ck_oracle as orc

    cores, model = host_info()
    torch.set_num_threads(cores)
    E_s = max(w["k"], min(w["E"], 2 if w["H"] * w["I"] > 1 << 24 else w["E"]))
    T_s = max(64, min(w["T"] * E_s // w["E"], 512 if w["H"] * w["I"] > 1 << 24 else w["T"]))
    g = torch.Generator().manual_seed(0)
    H, I, k = w["H"], w["I"], w["k"]
    dt = torch.bfloat16
    x = torch.randn(T_s, H, generator=g).to(dt)
    logits = torch.randn(T_s, E_s, generator=g)
    rw, sel = orc.routing_weights_ref(logits, k, dt)
    w_fc = (torch.randn(E_s, 2 * I, H, generator=g) * 0.02).to(dt)
    w_proj = (torch.randn(E_s, H, I, generator=g) * 0.02).to(dt)
    inp = dict(x=x, router_weights=rw, selected_experts=sel, w_fc=w_fc, w_proj=w_proj,
               grad_out=torch.randn(T_s, H, generator=g).to(dt))
    times = []
    t_start = time.time()
    for i in range(warmup + steps):
        t0 = time.time()
        orc.moe_fwd_bwd_ref(inp, dtype=dt)
        dt_s = time.time() - t0
        if i >= warmup:
            times.append(dt_s)
        if time.time() - t_start > budget_s and times:
            break
    per_step = sum(times) / len(times)
    return dict(value=T_s / per_step, unit=UNIT, cores=cores, kind="port", cpu_model=model, ms_per_step=per_step * 1e3,
                steps_timed=len(times),
                sample=f"{T_s} tokens over {E_s} of {w['E']} experts (top-{k}, H={H}, I={I}, bf16): same FLOPs per token "
                       f"as the full workload")


# ---------------------------------------------------------------------------------------------------
# parity of the timed configuration (outside the timed regions)
# ---------------------------------------------------------------------------------------------------
def _within(got: torch.Tensor, ref: torch.Tensor, atol: float, rtol: float = 2e-2) -> tuple[float, float]:
    """(worst |got - ref| / (atol + rtol |ref|), max |got - ref|)."""
    err = (got.float() - ref.float()).abs()
    return float((err / (atol + rtol * ref.float().abs())).max().item()), float(err.max().item())


def parity_check(inp: dict, y: torch.Tensor, dx: torch.Tensor, w: dict, world: int, rank: int, n_tokens: int = 32,
                 placement: list[int] | None = None) -> dict:
    """Recomputes, in fp32 with plain torch on the GPU, what the timed step must have produced, from the same inputs:
    y and dx of ``n_tokens`` sampled tokens of this rank (each needs only its own k experts), and the first 64 rows of
    both weight gradients of this rank's first expert over the rows of ALL ranks routed to it.  Every rank builds its
    expert weights from the same seed and shape, so expert e's weights are entry ``slot[e]`` (its position among its
    owner's experts; ``e % experts_per_rank`` for contiguous blocks) of every rank's local tensors: each rank can restate
    any expert without an exchange.  Tolerance: rtol 2e-2 with atol 2e-2
    taken relative to the reference's RMS (outputs / input grads) or scaled by sqrt(rows / 64) (weight grads)."""
    import torch.distributed as dist
    import torch.nn.functional as F

    T, H, I, E, k = w["T"], w["H"], w["I"], w["E"], w["k"]
    epr = E // world
    if placement is None:
        placement = [e // epr for e in range(E)]
    slot = [sum(1 for f in range(e) if placement[f] == placement[e]) for e in range(E)]  # local index at the owner
    mine = [e for e in range(E) if placement[e] == rank]
    dev = y.device
    prev = torch.backends.cuda.matmul.allow_tf32
    torch.backends.cuda.matmul.allow_tf32 = False
    try:
        x, rw, sel, go = inp["x"], inp["router_weights"], inp["selected_experts"].long(), inp["grad_out"]
        w_fc, w_proj = inp["w_fc"].detach(), inp["w_proj"].detach()
        checks = {}

        # (1) sampled tokens: y, dx
        g = torch.Generator(device="cpu").manual_seed(99 + rank)
        toks = torch.randperm(T, generator=g)[:n_tokens].to(dev)
        xs = x[toks].float().requires_grad_()
        ys = torch.zeros(n_tokens, H, device=dev)
        for j in range(k):
            for e in sel[toks, j].unique().tolist():
                m = (sel[toks, j] == e).nonzero().squeeze(1)
                h = F.linear(xs[m], w_fc[slot[e]].float())
                a = h[:, :I] * F.silu(h[:, I:])
                ys = ys.index_add(0, m, F.linear(a, w_proj[slot[e]].float()) * rw[toks[m], j].float().unsqueeze(1))
        ys.backward(go[toks].float())
        rms = lambda t: max(1.0, float(t.float().pow(2).mean().sqrt().item()))  # noqa: E731
        checks["y"] = _within(y[toks], ys.detach(), 2e-2 * rms(ys.detach()))
        checks["dx"] = _within(dx[toks], xs.grad, 2e-2 * rms(xs.grad))

        # (2) weight-grad rows of this rank's first expert, over every rank's rows routed to it
        def gathered(t):
            if world == 1:
                return t
            out = torch.empty((world * t.size(0),) + tuple(t.shape[1:]), dtype=t.dtype, device=dev)
            dist.all_gather_into_tensor(out, t.contiguous())
            return out

        x_all, rw_all, sel_all, go_all = gathered(x), gathered(rw), gathered(sel), gathered(go)
        e_glob = mine[0]
        tok_e, slot_e = (sel_all == e_glob).nonzero(as_tuple=True)
        n_e = int(tok_e.numel())
        rows = 64
        if n_e > 0:
            X = x_all[tok_e].float()
            h = F.linear(X, w_fc[0].float())
            up, gate = h[:, :I], h[:, I:]
            sg = torch.sigmoid(gate)
            act = up * gate * sg
            wv = rw_all[tok_e, slot_e].float().unsqueeze(1)
            dyw = go_all[tok_e].float() * wv
            ref_dwproj = dyw[:, :rows].t() @ act                                # d_w_proj[0][:rows, :]
            da = dyw @ w_proj[0].float()                                        # [n_e, I]
            d_up = da[:, :rows] * gate[:, :rows] * sg[:, :rows]                # first `rows` "up" features
            ref_dwfc = d_up.t() @ X                                             # d_w_fc[0][:rows, :]
            checks["d_w_proj[first expert, :64]"] = _within(inp["w_proj"].grad[0, :rows], ref_dwproj, 2e-2 * rms(ref_dwproj))
            checks["d_w_fc[first expert, :64]"] = _within(inp["w_fc"].grad[0, :rows], ref_dwfc, 2e-2 * rms(ref_dwfc))
        worst = max(v[0] for v in checks.values())
        ok = worst <= 1.0 and all(v[0] == v[0] for v in checks.values())
    finally:
        torch.backends.cuda.matmul.allow_tf32 = prev
    flag = torch.tensor([1.0 if ok else 0.0, worst, max(v[1] for v in checks.values())], device=dev, dtype=torch.float64)
    if world > 1:
        both = torch.stack([flag[0], -flag[1], -flag[2]])
        dist.all_reduce(both, op=dist.ReduceOp.MIN)
        flag = torch.stack([both[0], -both[1], -both[2]])
    return dict(ok=bool(flag[0].item() == 1.0), worst_err_over_bound=float(flag[1].item()), max_abs=float(flag[2].item()),
                checked=f"y, dx of {n_tokens} sampled tokens per rank; first 64 rows of d_w_proj and d_w_fc of each rank's "
                        f"first expert over all ranks' rows; fp32 torch restatement of the layer on the same inputs",
                tolerance="rtol 2e-2, atol 2e-2 x max(1, rms(ref))",
                rank0={k_: dict(err_over_bound=round(v[0], 4), max_abs=v[1]) for k_, v in checks.items()})


# ---------------------------------------------------------------------------------------------------
# the GPU arm
# ---------------------------------------------------------------------------------------------------
def gpu_arm(args, w: dict) -> dict | None:
    import torch.distributed as dist

    import cute_kernels as ck
    from cute_kernels import _lib

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} needs {args.gpus} ranks (torch.distributed.run), found WORLD_SIZE={world}")
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    numa_node = bind_to_gpu_numa_node(local_rank) if world > 1 else None
    if world > 1:
        if os.environ.get("NCCL_DEBUG", "").upper() == "VERSION":
            os.environ["NCCL_DEBUG"] = "WARN"  # keep stdout to the one JSON line
        dist.init_process_group("nccl", device_id=device)

    T, H, I, E, k = w["T"], w["H"], w["I"], w["E"], w["k"]
    if world > 1:
        from cute_kernels.expert_parallel import ExpertParallelMoE

        assert E % world == 0, "experts must divide evenly across ranks"
        epr = E // world
        inp = make_device_inputs(w, device, seed=1000 + rank, experts=slice(rank * epr, (rank + 1) * epr))
        ep, transport, placement = None, "nccl_all_to_all", None
        if args.ep_transport in ("auto", "peer"):
            # rows move by NVLink loads / stores issued from the permutation kernels and the GEMM epilogues
            ok = torch.ones(1, device=device)
            try:
                from cute_kernels.peer_parallel import PeerExpertParallelMoE

                # rows to allocate per step: read back from the device (default; measured equal or faster at 2 GPUs), or a
                # fixed capacity with no read-back
                # expert placement: contiguous blocks, or balanced by the rows every expert receives (all ranks' routing of
                # this batch; a training loop would use a running histogram)
                use_balanced = args.ep_placement == "balanced" or (args.ep_placement == "auto" and w["expert_bias"])
                if use_balanced:
                    from cute_kernels.expert_parallel import balanced_expert_placement

                    hist = torch.bincount(inp["selected_experts"].reshape(-1).long(), minlength=E).float()
                    dist.all_reduce(hist)
                    placement = balanced_expert_placement(hist.tolist(), world)
                cap_factor = args.ep_capacity_factor if args.ep_capacity_factor > 0 else None
                ep = PeerExpertParallelMoE(E, k, T, H, torch.bfloat16, dist.group.WORLD, capacity_factor=cap_factor,
                                           expert_to_rank=placement)
                if args.ep_overlap == "off":
                    ep.engine.MIN_TILES_TO_SPLIT = None
                ep.engine.PULL_SMS = args.ep_pull_sms
                transport = ("peer_memory" + ("+balanced_placement" if placement is not None else "") +
                             (f"+pull_overlapped_on_{args.ep_pull_sms}_sms" if args.ep_overlap == "on" else ""))
            except Exception as exc:  # symmetric memory not available on this box
                if args.ep_transport == "peer":
                    raise
                print(f"[bench] rank {rank}: peer-memory transport unavailable ({exc}); using NCCL all-to-all", file=sys.stderr)
                ok.zero_()
            dist.all_reduce(ok, op=dist.ReduceOp.MIN)
            if ok.item() == 0:
                ep, transport, placement = None, "nccl_all_to_all", None
        if ep is None:
            ep = ExpertParallelMoE(E, k, dist.group.WORLD, chunks=args.ep_chunks)
            transport = "nccl_all_to_all" + (f"+{args.ep_chunks}_chunks_on_side_streams" if args.ep_chunks > 1 else "")

        def step(x, rw, sel, grad_out):
            x = x.detach().requires_grad_()
            rw = rw.detach().requires_grad_()
            y = ep(x, rw, sel, inp["w_fc"], inp["w_proj"])
            y.backward(grad_out)
            return y, x.grad
    else:
        inp = make_device_inputs(w, device, seed=1000)

        def step(x, rw, sel, grad_out):
            x = x.detach().requires_grad_()
            rw = rw.detach().requires_grad_()
            y = ck.fused_experts(x, rw, sel, inp["w_fc"], inp["w_proj"], k, deterministic=COMBINE_ROWS.get(args.combine))
            y.backward(grad_out)
            return y, x.grad

    inp["w_fc"].requires_grad_()
    inp["w_proj"].requires_grad_()

    def zero_wgrads():
        inp["w_fc"].grad = None
        inp["w_proj"].grad = None

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # ---- device-resident timing ------------------------------------------------------------------------
    sampler = ClockSampler(local_rank) if rank == 0 else None
    for _ in range(args.warmup):
        step(inp["x"], inp["router_weights"], inp["selected_experts"], inp["grad_out"])
        zero_wgrads()
    barrier()
    ck.check_device_status()
    _lib.launch_log.reset()
    _lib.launch_log.record_events = True
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    if sampler:
        sampler.mark_begin()
    e0.record()
    for _ in range(args.steps):
        step(inp["x"], inp["router_weights"], inp["selected_experts"], inp["grad_out"])
        zero_wgrads()
    e1.record()
    barrier()
    if sampler:
        sampler.mark_end()
    _lib.launch_log.record_events = False
    ms_total = e0.elapsed_time(e1)
    clocks = sampler.stop() if sampler else None
    launches = _lib.launch_log.count
    per_kernel: dict[str, list[float]] = {}
    for name, _work, a, b in _lib.launch_log.events:
        per_kernel.setdefault(name, []).append(a.elapsed_time(b))
    ck.check_device_status()

    t = torch.tensor([ms_total], device=device, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_total = float(t.item())
    ms_per_step = ms_total / args.steps
    value = world * T / (ms_per_step * 1e-3)
    # every rank's own GEMM time per step: the ranks meet at four collectives per step, so the slowest GPU under the power
    # cap sets the pace of all of them
    rank_gemm_ms = None
    if world > 1:
        mine = torch.tensor([sum(sum(ts) for n, ts in per_kernel.items() if n in GEMM_KERNELS) / args.steps], device=device,
                            dtype=torch.float64)
        allr = torch.empty(world, device=device, dtype=torch.float64)
        dist.all_gather_into_tensor(allr, mine)
        rank_gemm_ms = [round(v, 3) for v in allr.tolist()]

    # ---- end to end: pinned host buffers in, results out, inside the timed region ------------------------
    host = {n: inp[n].cpu().pin_memory() for n in ("x", "router_weights", "selected_experts", "grad_out")}
    y_host = torch.empty(T, H, dtype=torch.bfloat16).pin_memory()
    dx_host = torch.empty(T, H, dtype=torch.bfloat16).pin_memory()

    # Every step's inputs come from pinned host memory and its results go back to it, all inside the timed region.
    # The copies run on two more streams, one per direction (PCIe is full duplex): inputs of step i+1 and results of
    # step i-1 move while step i computes.
    h2d_stream = torch.cuda.Stream(device=device)
    d2h_stream = torch.cuda.Stream(device=device)
    main_stream = torch.cuda.current_stream()

    def stage_in():
        with torch.cuda.stream(h2d_stream):
            dev = {n: v.to(device, non_blocking=True) for n, v in host.items()}
            ev = torch.cuda.Event()
            ev.record(h2d_stream)
        return dev, ev

    step_marks: list = []  # CK_BENCH_DEBUG: one event per end-to-end step, printed as per-step milliseconds on stderr

    def e2e_loop(n_steps: int) -> None:
        pending = stage_in()
        for i in range(n_steps):
            if os.environ.get("CK_BENCH_DEBUG"):
                ev_dbg = torch.cuda.Event(enable_timing=True)
                ev_dbg.record(main_stream)
                step_marks.append((time.perf_counter(), ev_dbg))
            dev, ev = pending
            if i + 1 < n_steps:
                pending = stage_in()
            main_stream.wait_event(ev)
            for v in dev.values():
                v.record_stream(main_stream)
            y, dx = step(dev["x"], dev["router_weights"], dev["selected_experts"], dev["grad_out"])
            done = torch.cuda.Event()
            done.record(main_stream)
            with torch.cuda.stream(d2h_stream):
                d2h_stream.wait_event(done)
                y_host.copy_(y, non_blocking=True)
                dx_host.copy_(dx, non_blocking=True)
                y.record_stream(d2h_stream)
                dx.record_stream(d2h_stream)
            zero_wgrads()
        main_stream.wait_stream(d2h_stream)  # the last results have reached the host before the clock stops

    e2e_loop(max(1, min(args.warmup, 2)))
    barrier()
    e0.record()
    e2e_loop(args.steps)
    e1.record()
    barrier()
    t = torch.tensor([e0.elapsed_time(e1)], device=device, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    e2e_ms = float(t.item()) / args.steps
    if step_marks and rank == 0:
        marks = step_marks[-args.steps:]
        print("[bench] e2e step starts, device ms: " + " ".join(f"{marks[0][1].elapsed_time(m[1]):.1f}" for m in marks) +
              " | host ms: " + " ".join(f"{(m[0] - marks[0][0]) * 1e3:.1f}" for m in marks), file=sys.stderr)
    h2d = sum(v.numel() * v.element_size() for v in host.values())
    d2h = 2 * T * H * 2
    ck.check_device_status()
    # the same copies with no compute at all, every rank at once: what the host side (PCIe, host memory, IOMMU) allows
    y_dev = torch.empty(T, H, dtype=torch.bfloat16, device=device)
    barrier()
    e0.record()
    for _ in range(4):
        with torch.cuda.stream(h2d_stream):
            keep = [v.to(device, non_blocking=True) for v in host.values()]
        with torch.cuda.stream(d2h_stream):
            y_host.copy_(y_dev, non_blocking=True)
            dx_host.copy_(y_dev, non_blocking=True)
        main_stream.wait_stream(h2d_stream)
        main_stream.wait_stream(d2h_stream)
    e1.record()
    barrier()
    del keep
    t = torch.tensor([e0.elapsed_time(e1)], device=device, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    copies_alone_ms = float(t.item()) / 4

    # ---- parity of this very configuration, untimed: one more step on the resident inputs, checked in fp32 ----------
    parity = None
    if not args.no_parity:
        zero_wgrads()
        y_chk, dx_chk = step(inp["x"], inp["router_weights"], inp["selected_experts"], inp["grad_out"])
        torch.cuda.synchronize()
        parity = parity_check(inp, y_chk.detach(), dx_chk, w, world, rank, placement=placement if world > 1 else None)
        del y_chk, dx_chk
        zero_wgrads()
        ck.check_device_status()

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return None

    # ---- roofline of the grouped-GEMM kernel family ---------------------------------------------------------
    peaks = measured_peaks()
    R = T * k  # routed rows per rank (weak scaling: the same on every rank on average)
    algo = {  # algorithmic FLOPs per launch: 2 * rows * N * K with un-padded rows
        "up_act_fwd": 2.0 * R * (2 * I) * H, "down_combine_fwd": 2.0 * R * H * I, "dgrad_down": 2.0 * R * H * I,
        "dgrad_up": 2.0 * R * (2 * I) * H, "wgrad": 2.0 * R * H * I * 1.5,  # two launches per step: (H x I) and (2I x H)
        "grouped_linear_scatter": 2.0 * R * H * I * 1.5,  # expert-parallel shards: down (H x I) and dgrad-up (2I x H)
        "grouped_linear_scatter_peer": 2.0 * R * H * I * 1.5,  # the same two GEMMs storing into the owners' buffers
        "up_act_fwd_peer": 2.0 * R * (2 * I) * H, "dgrad_down_peer": 2.0 * R * H * I,  # rows pulled over NVLink by the producer warps
    }
    kernels = {}
    for name, ts in per_kernel.items():
        kernels[name] = dict(launches=len(ts), ms_avg=sum(ts) / len(ts), ms_total=sum(ts))
        if name in algo:
            kernels[name]["tflops"] = algo[name] / (kernels[name]["ms_avg"] * 1e-3) / 1e12
    gemm_ms = sum(v["ms_total"] for n, v in kernels.items() if n in GEMM_KERNELS) / args.steps
    gemm_flops = 18.0 * k * H * I * T
    dom = max((n for n in kernels if n in algo), key=lambda n: kernels[n]["ms_total"])
    peak = float(peaks.get("bf16_tflops_sustained") or peaks["bf16_tflops"])
    roofline = dict(
        bound="tensor",
        kernel=f"{'grouped_gemm_pair_kernel' if os.environ.get('CK_GEMM_CTA_PAIR', '1') != '0' else 'grouped_gemm_kernel'}<bf16> ({dom})", achieved=kernels[dom]["tflops"], peak=peak,
        unit="TFLOP/s", frac=kernels[dom]["tflops"] / peak,
        traffic=None,  # DRAM bytes per launch need an ncu capture of this very build; a constant here would go stale
        traffic_unit="bytes per launch (dram__bytes_read.sum + dram__bytes_write.sum)",
        peak_source=f"bf16_tflops_sustained of {peaks['source']}",
        all_gemms=dict(ms_per_step=gemm_ms, tflops=gemm_flops / (gemm_ms * 1e-3) / 1e12,
                       frac_of_measured_sustained=gemm_flops / (gemm_ms * 1e-3) / 1e12 / peak,
                       frac_of_measured_burst=gemm_flops / (gemm_ms * 1e-3) / 1e12 / float(peaks["bf16_tflops"]),
                       frac_of_nominal_2250=gemm_flops / (gemm_ms * 1e-3) / 1e12 / 2250.0),
        kernels={n: {kk: round(vv, 4) if isinstance(vv, float) else vv for kk, vv in v.items()} for n, v in kernels.items()},
    )

    cpu = cpu_arm(w, steps=3, warmup=1, budget_s=45.0) if (world == 1 and not args.no_cpu_baseline) else None

    # ---- the other configurations, measured in the same run outside the timed regions (N = 1 only) --------------------
    aux = None
    if world == 1 and not args.no_aux:
        del host, y_host, dx_host
        inp.clear()
        torch.cuda.empty_cache()
        hbm_peak = float(peaks["hbm_gbs"])
        flush = torch.zeros(128 << 20, dtype=torch.float32, device=device)
        aux = dict(
            peak_hbm_gbs=hbm_peak, peak_source=f"hbm_gbs / bf16_tflops_sustained of {peaks['source']}",
            c2_route_count=measure_c2(10, 3, flush, hbm_peak),
            c3_swiglu=measure_c3(10, 3, flush, hbm_peak),
            rmsnorm=measure_rmsnorm(10, 3, flush, hbm_peak),
        )
        del flush
        torch.cuda.empty_cache()
        if w["name"] != WORKLOADS["c5"]["name"]:
            aux["c5_finegrained_moe"] = measure_moe_brief(WORKLOADS["c5"], 5, 3, device, peak)

    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic",
        "config": {"workload": w["name"], "tokens_per_gpu": T, "hidden": H, "intermediate": I, "experts": E, "top_k": k,
                   "parallelism": f"ep{world}" if world > 1 else "single",
                   **({"ep_transport": transport, "host_numa_node_rank0": numa_node} if world > 1 else {}),
                   "l2_policy": "inputs_exceed_l2",
                   "step": "route+gather+up_swiglu+down_combine+backward(dgrad,wgrad,swiglu_bwd,router_grad)"},
        "clocks": clocks,
        "e2e": {"value": world * T / (e2e_ms * 1e-3), "unit": UNIT, "ms_per_step": e2e_ms, "h2d_bytes_per_step": h2d,
                "d2h_bytes_per_step": d2h, "copies_alone_ms_per_step": round(copies_alone_ms, 3)},
        "gpu_launches": launches,
        "roofline": roofline,
    }
    if rank_gemm_ms is not None:
        line["rank_gemm_ms_per_step"] = rank_gemm_ms
    if parity is not None:
        line["parity"] = parity
    if aux is not None:
        line["aux"] = aux
    if cpu is not None:
        line["cpu_baseline"] = cpu
    if world > 1:
        dist.destroy_process_group()
    return line


# ---------------------------------------------------------------------------------------------------
# HBM-bound pieces: routing (count + scan + stable scatter) and stand-alone SwiGLU
# ---------------------------------------------------------------------------------------------------
def _time_each(fn, steps: int, warmup: int, flush: torch.Tensor | None) -> list[float]:
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    out = []
    for _ in range(steps):
        if flush is not None:
            flush.add_(1)  # 512 MB written: evicts the 126 MB L2 between timed launches
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        out.append(e0.elapsed_time(e1))
    return out


def _time_kernels(fn, steps: int, warmup: int, flush: torch.Tensor | None) -> tuple[float, float]:
    """(median device time of this library's launches inside one call of ``fn``, median time of the whole call).
    The first is bracketed by CUDA events around each C-ABI call on the launching stream; the second also holds whatever
    the caller's framework does around them (autograd dispatch, allocations) while the GPU waits."""
    from cute_kernels import _lib

    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    kern, whole = [], []
    for _ in range(steps):
        if flush is not None:
            flush.add_(1)
        _lib.launch_log.reset()
        _lib.launch_log.record_events = True
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        _lib.launch_log.record_events = False
        whole.append(e0.elapsed_time(e1))
        kern.append(sum(a.elapsed_time(b) for _n, _w, a, b in _lib.launch_log.events))
    _lib.launch_log.reset()
    return statistics.median(kern), statistics.median(whole)


def measure_c2(steps: int, warmup: int, flush: torch.Tensor, peak: float) -> dict:
    """count and count + scan + stable scatter over 2^24 int32 ids, 64 experts, uniform and Zipf(1.2) draws."""
    import numpy as np

    import cute_kernels as ck

    dev = flush.device
    n, E = 1 << 24, 64
    g = torch.Generator(device=dev).manual_seed(0)
    p_zipf = 1.0 / torch.arange(1, E + 1, device=dev, dtype=torch.float64).pow(1.2)
    draws = {"uniform": torch.randint(0, E, (n,), generator=g, device=dev, dtype=torch.int32),
             "zipf": torch.multinomial((p_zipf / p_zipf.sum()).float(), n, replacement=True, generator=g).to(torch.int32)}
    out = {}
    for name, ids in draws.items():
        t_route = statistics.median(_time_each(lambda: ck.route(ids, E, with_tile_metadata=False), steps, warmup, flush))
        t_count = statistics.median(_time_each(lambda: ck.continuous_count_cute(ids, E), steps, warmup, flush))
        out[name] = dict(route_ms=t_route, route_gbs=12.0 * n / (t_route * 1e-3) / 1e9, route_frac=12.0 * n / (t_route * 1e-3) / 1e9 / peak,
                         count_ms=t_count, count_gbs=4.0 * n / (t_count * 1e-3) / 1e9, count_frac=4.0 * n / (t_count * 1e-3) / 1e9 / peak)
    out["algorithmic_bytes"] = dict(route=12 * n, count=4 * n)
    out["n_ids"], out["experts"] = n, E
    return out


def measure_c3(steps: int, warmup: int, flush: torch.Tensor, peak: float) -> dict:
    """Stand-alone SwiGLU forward and backward on [16384, 14336] bf16."""
    import cute_kernels as ck

    dev = flush.device
    rows, cols = 16384, 14336
    g = torch.Generator(device=dev).manual_seed(0)
    gate = torch.randn(rows, cols, generator=g, device=dev, dtype=torch.float32).bfloat16().requires_grad_()
    up = torch.randn(rows, cols, generator=g, device=dev, dtype=torch.float32).bfloat16().requires_grad_()
    dy = torch.randn(rows, cols, generator=g, device=dev, dtype=torch.float32).bfloat16()
    nel = rows * cols
    with torch.no_grad():
        # the 512 MB flush write also lets the host run ahead, so the events bracket device time only
        f_ms = statistics.median(_time_each(lambda: ck.swiglu_cute(gate, up), steps, warmup, flush))
    out = ck.swiglu_cute(gate, up)

    def bwd():
        gate.grad = None
        up.grad = None
        out.backward(dy, retain_graph=True)

    b_ms = statistics.median(_time_each(bwd, steps, warmup, flush))
    return dict(shape=[rows, cols], fwd_ms=f_ms, fwd_gbs=6.0 * nel / (f_ms * 1e-3) / 1e9, fwd_frac=6.0 * nel / (f_ms * 1e-3) / 1e9 / peak,
                bwd_ms=b_ms, bwd_gbs=10.0 * nel / (b_ms * 1e-3) / 1e9, bwd_frac=10.0 * nel / (b_ms * 1e-3) / 1e9 / peak,
                algorithmic_bytes=dict(fwd=6 * nel, bwd=10 * nel))


def measure_rmsnorm(steps: int, warmup: int, flush: torch.Tensor, peak: float) -> dict:
    """RMSNorm and fused residual-add + RMSNorm on the Mixtral-shaped layer's input [16384, 4096] bf16, with weight.
    Algorithmic bytes per element: forward 2 x 2 B (4 x 2 B with the residual), backward 3 x 2 B (5 x 2 B)."""
    import cute_kernels as ck

    dev = flush.device
    rows, cols = 16384, 4096
    g = torch.Generator(device=dev).manual_seed(0)
    mk = lambda *shape: torch.randn(*shape, generator=g, device=dev, dtype=torch.float32).bfloat16()  # noqa: E731
    x, res, w, dy = mk(rows, cols).requires_grad_(), mk(rows, cols).requires_grad_(), mk(cols).requires_grad_(), mk(rows, cols)
    nel = rows * cols
    out = {"shape": [rows, cols]}
    with torch.no_grad():
        f_ms = _time_kernels(lambda: ck.rmsnorm_cute(x, w, 1e-5), steps, warmup, flush)
        ff_ms = _time_kernels(lambda: ck.fused_residual_add_rmsnorm_cute(x, res, w, 1e-5, 0.9), steps, warmup, flush)
    z = ck.rmsnorm_cute(x, w, 1e-5)
    zf, rf = ck.fused_residual_add_rmsnorm_cute(x, res, w, 1e-5, 0.9)

    def bwd():
        x.grad = res.grad = w.grad = None
        z.backward(dy, retain_graph=True)

    def fbwd():
        x.grad = res.grad = w.grad = None
        torch.autograd.backward([zf, rf], [dy, dy], retain_graph=True)

    b_ms = _time_kernels(bwd, steps, warmup, flush)
    fb_ms = _time_kernels(fbwd, steps, warmup, flush)
    # ms / gbs / frac: the kernels' own device time; op_ms: the whole call as a user makes it (the backward goes through
    # the autograd engine, whose dispatch leaves the GPU idle for tens of microseconds on a 100-microsecond kernel)
    for name, (ms, op_ms), elems in (("fwd", f_ms, 2), ("bwd", b_ms, 3), ("fused_fwd", ff_ms, 4), ("fused_bwd", fb_ms, 5)):
        gbs = elems * 2.0 * nel / (ms * 1e-3) / 1e9
        out[name] = dict(ms=ms, op_ms=op_ms, gbs=gbs, frac=gbs / peak, algorithmic_bytes=elems * 2 * nel)
    return out


def measure_moe_brief(w: dict, steps: int, warmup: int, device: torch.device, peak_tflops: float) -> dict:
    """tokens/s and grouped-GEMM TFLOP/s of one more MoE configuration (single GPU, inputs resident)."""
    import cute_kernels as ck
    from cute_kernels import _lib

    inp = make_device_inputs(w, device, seed=2000)
    inp["w_fc"].requires_grad_()
    inp["w_proj"].requires_grad_()
    T, H, I, k = w["T"], w["H"], w["I"], w["k"]

    def step():
        x = inp["x"].detach().requires_grad_()
        rw = inp["router_weights"].detach().requires_grad_()
        y = ck.fused_experts(x, rw, inp["selected_experts"], inp["w_fc"], inp["w_proj"], k)
        y.backward(inp["grad_out"])
        inp["w_fc"].grad = None
        inp["w_proj"].grad = None

    for _ in range(warmup):
        step()
    torch.cuda.synchronize()
    _lib.launch_log.reset()
    _lib.launch_log.record_events = True
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        step()
    e1.record()
    torch.cuda.synchronize()
    _lib.launch_log.record_events = False
    ms = e0.elapsed_time(e1) / steps
    per: dict[str, float] = {}
    for name, _work, a, b in _lib.launch_log.events:
        per[name] = per.get(name, 0.0) + a.elapsed_time(b) / steps
    _lib.launch_log.reset()
    gemm_ms = sum(v for n, v in per.items() if n in GEMM_KERNELS)
    flops = 18.0 * k * H * I * T
    ck.check_device_status()
    return dict(workload=w["name"], tokens=T, hidden=H, intermediate=I, experts=w["E"], top_k=k, steps=steps, ms_per_step=ms,
                tokens_per_s=T / (ms * 1e-3), gemm_ms_per_step=gemm_ms, gemm_tflops=flops / (gemm_ms * 1e-3) / 1e12,
                gemm_frac_of_measured_sustained=flops / (gemm_ms * 1e-3) / 1e12 / peak_tflops,
                kernels_ms_per_step={n: round(v, 4) for n, v in sorted(per.items())})


def gemm_cycle_profile(w: dict, device: torch.device) -> dict:
    """Cycle accounting of the CTA-pair GEMM launches of one layer shape (both combine flavours of the down projection and of
    dgrad-up, and the two weight gradients), one isolated launch each.

    Needs a library built with ``make -C cute-kernels_b200/csrc clean all EXTRA=-DCK_GEMM_PROFILE`` (it exports
    ck_gemm_profile_read; the default build does not).  Per GEMM: cycles of the issuing thread per pair tile against the
    tensor pipe's 4096 MAC/clk/SM, where the issuing and the loading warps spent their time, and how long the epilogue
    warps were busy."""
    import ctypes

    import cute_kernels as ck
    from cute_kernels import _lib
    from cute_kernels.moe import (dgates_parts, dgrad_down, dgrad_up, down_combine_fwd, grouped_linear_scatter, up_act_fwd,
                                  wgrad)

    lib = ctypes.CDLL(_lib.LIB_PATH)
    if not hasattr(lib, "ck_gemm_profile_read"):
        raise SystemExit("the library was not built with -DCK_GEMM_PROFILE")
    T, H, I, E, k = w["T"], w["H"], w["I"], w["E"], w["k"]
    dt = torch.bfloat16
    g = torch.Generator(device=device).manual_seed(0)
    ids = torch.randn(T, E, generator=g, device=device).topk(k, dim=-1).indices.int()
    r = ck.route(ids.reshape(-1), E)
    cap = r.capacity
    rows = int((r.row_map >= 0).sum())
    padded_rows = int(r.padded_off[E].item())
    gate_w = torch.rand(T * k, generator=g, device=device).to(dt)
    xg = torch.randn(cap, H, generator=g, device=device).to(dt)
    w_proj = torch.empty(E, H, I, device=device, dtype=dt).normal_(0, 0.02, generator=g)
    w_fc = torch.empty(E, 2 * I, H, device=device, dtype=dt).normal_(0, 0.02, generator=g)
    h = torch.randn(cap, 2 * I, generator=g, device=device).to(dt)
    dh = torch.empty(cap, 2 * I, device=device, dtype=dt)
    act = torch.randn(cap, I, generator=g, device=device).to(dt)
    dg_part = torch.empty(dgates_parts(I), cap, device=device, dtype=torch.float32)
    out32 = torch.zeros(T, H, device=device, dtype=torch.float32)
    dw_proj = torch.empty(E, H, I, device=device, dtype=dt)
    dw_fc = torch.empty(E, 2 * I, H, device=device, dtype=dt)
    rows_h = torch.empty(T * k, H, device=device, dtype=dt)  # per-(token, slot) result rows of the row-store flavour
    swiglu = _lib.CK_ACT_SWIGLU
    launches = {
        "up_act_fwd": (lambda: up_act_fwd(xg, w_fc, None, gate_w, r.row_map, r.mtile_off, act, dh, swiglu), 2.0 * rows * H * 2 * I, H),
        "down_combine_fwd": (lambda: down_combine_fwd(act, w_proj, None, None, r.row_map, r.mtile_off, out32, k), 2.0 * rows * H * I, I),
        "dgrad_down": (lambda: dgrad_down(xg, w_proj, h, gate_w, r.row_map, r.mtile_off, dh, None, dg_part, swiglu), 2.0 * rows * H * I, H),
        "dgrad_up": (lambda: dgrad_up(dh, w_fc, r.row_map, r.mtile_off, out32, k), 2.0 * rows * H * 2 * I, 2 * I),
        # the deterministic flavour (default for top-k > 2): rows stored by row_map, summed per token by a second kernel
        "down_row_store": (lambda: grouped_linear_scatter(act, w_proj, None, None, r.mtile_off, r.row_map, rows_h, False), 2.0 * rows * H * I, I),
        "dgrad_up_row_store": (lambda: grouped_linear_scatter(dh, w_fc, None, None, r.mtile_off, r.row_map, rows_h, True), 2.0 * rows * H * 2 * I, 2 * I),
        # weight gradients contract over an expert's padded rows: K = padded rows / experts on average
        "wgrad_c_proj": (lambda: wgrad(xg, act, r.padded_off, dw_proj), 2.0 * rows * H * I, padded_rows / E),
        "wgrad_c_fc": (lambda: wgrad(dh, xg, r.padded_off, dw_fc), 2.0 * rows * H * 2 * I, padded_rows / E),
    }
    slots, ctas = 16, 160
    out = {}
    for name, (fn, flops, K) in launches.items():
        for _ in range(2):
            fn()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1)
        buf = (ctypes.c_ulonglong * (ctas * slots))()
        if lib.ck_gemm_profile_read(buf) != 0:
            raise SystemExit("ck_gemm_profile_read failed")
        n_ctas = 2 * (torch.cuda.get_device_properties(device).multi_processor_count // 2)
        rows_ = [[float(buf[c * slots + i]) for i in range(slots)] for c in range(n_ctas)]
        lead, peer = rows_[0::2], rows_[1::2]
        mean = lambda xs: sum(xs) / len(xs)  # noqa: E731
        total = mean([c[2] for c in lead])
        tiles = mean([c[3] for c in lead])
        ideal = tiles * (K / 64.0) * 512.0  # 128 x 256 x 64 MACs per CTA and k-block at 4096 MAC/clk
        out[name] = dict(ms=round(ms, 4), tflops=round(flops / ms / 1e9, 1), pair_tiles_per_cta_pair=round(tiles, 1),
                         issuer_kcycles=round(total / 1e3, 1), tensor_pipe_frac_of_4096_mac_per_clk=round(ideal / total, 4),
                         sm_mhz_during_launch=round(total / ms / 1e3, 0),
                         issuer_wait_accumulator_frac=round(mean([c[0] / c[2] for c in lead]), 4),
                         issuer_wait_stage_frac=round(mean([c[1] / c[2] for c in lead]), 4),
                         issuer_stage_ready_frac=round(mean([c[8] / max(c[9], 1.0) for c in lead]), 4),
                         producer_stage_free_frac=round(mean([c[10] / max(a[9], 1.0) for c, a in zip(peer, lead)]), 4),
                         producer_wait_frac=round(mean([c[11] / max(c[12], 1.0) for c in peer]), 4),
                         epilogue_busy_frac=round(mean([c[5] / c[2] for c in lead]), 4))
    ck.check_device_status()
    return out


def micro_arm(args, which: str) -> dict:
    import cute_kernels as ck

    torch.cuda.set_device(0)
    dev = torch.device("cuda", 0)
    peaks = measured_peaks()
    peak = float(peaks["hbm_gbs"])
    sampler = ClockSampler(0)
    flush = torch.zeros(128 << 20, dtype=torch.float32, device=dev)
    if which == "c2":
        sampler.mark_begin()
        results = measure_c2(args.steps, args.warmup, flush, peak)
        sampler.mark_end()
        head = results["uniform"]
        line = dict(metric="route_hbm_gb_per_s", value=head["route_gbs"], unit="GB/s", ms_per_step=head["route_ms"],
                    config=dict(workload="c2_count_scan_stable_scatter", n_ids=results["n_ids"], experts=results["experts"],
                                ids_dtype="int32", l2_policy="l2_flushed_between_launches", draws=["uniform", "zipf(1.2)"]),
                    roofline=dict(bound="hbm", kernel="route_hist + route_scan + route_scatter (3 launches)",
                                  achieved=head["route_gbs"], peak=peak, unit="GB/s", frac=head["route_gbs"] / peak,
                                  traffic=None, algorithmic_bytes=results["algorithmic_bytes"]["route"],
                                  peak_source=f"hbm_gbs of {peaks['source']}"),
                    detail=results)
    elif which == "rmsnorm":
        sampler.mark_begin()
        results = measure_rmsnorm(args.steps, args.warmup, flush, peak)
        sampler.mark_end()
        head = results["bwd"]
        line = dict(metric="rmsnorm_bwd_hbm_gb_per_s", value=head["gbs"], unit="GB/s", ms_per_step=head["ms"],
                    config=dict(workload="rmsnorm_fwd_bwd", shape=results["shape"], l2_policy="l2_flushed_between_launches"),
                    roofline=dict(bound="hbm", kernel="rmsnorm_bwd_kernel<bf16> + rmsnorm_dw_reduce_kernel", achieved=head["gbs"],
                                  peak=peak, unit="GB/s", frac=head["frac"], traffic=None,
                                  algorithmic_bytes=head["algorithmic_bytes"], peak_source=f"hbm_gbs of {peaks['source']}"),
                    detail=results)
    else:
        sampler.mark_begin()
        results = measure_c3(args.steps, args.warmup, flush, peak)
        sampler.mark_end()
        nel = results["shape"][0] * results["shape"][1]
        both = 16.0 * nel / ((results["fwd_ms"] + results["bwd_ms"]) * 1e-3) / 1e9
        line = dict(metric="swiglu_fwd_bwd_hbm_gb_per_s", value=both, unit="GB/s", ms_per_step=results["fwd_ms"] + results["bwd_ms"],
                    config=dict(workload="c3_swiglu_fwd_bwd", shape=results["shape"], l2_policy="inputs_exceed_l2"),
                    roofline=dict(bound="hbm", kernel="swiglu_bwd_vec_kernel<bf16>", achieved=results["bwd_gbs"], peak=peak,
                                  unit="GB/s", frac=results["bwd_gbs"] / peak, traffic=None, algorithmic_bytes=10 * nel,
                                  peak_source=f"hbm_gbs of {peaks['source']}"),
                    detail=results)
    ck.check_device_status()
    line.update(n_gpus=1, steps=args.steps, warmup=args.warmup, higher_is_better=True, scaling="weak", vs_baseline=None,
                dtype="int32" if which == "c2" else "bf16", data="synthetic", clocks=sampler.stop(), gpu_launches=None)
    return line


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--workload", default="c4", choices=sorted(WORKLOADS) + ["c2", "c3", "rmsnorm"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-parity", action="store_true", help="skip the untimed fp32 parity check of the timed configuration")
    ap.add_argument("--no-aux", action="store_true", help="N = 1: skip the routing / SwiGLU / fine-grained-layer figures")
    ap.add_argument("--ep-transport", default="auto", choices=["auto", "peer", "nccl"],
                    help="N > 1: rows cross GPUs by peer-memory loads/stores from the kernels (default when symmetric "
                         "memory is available) or by NCCL all-to-all")
    ap.add_argument("--ep-placement", default="auto", choices=["auto", "block", "balanced"],
                    help="N > 1, peer transport: experts in contiguous blocks per rank, or placed by load (longest processing "
                         "time first); auto = balanced for the skewed configuration, blocks otherwise")
    ap.add_argument("--combine", default="auto", choices=["auto", "red", "rows"],
                    help="N = 1: how the k expert outputs of a token are summed: fp32 red.add from the GEMM epilogue, or rows "
                         "stored once and summed in slot order by a second kernel; auto = the library's choice")
    ap.add_argument("--ep-overlap", default="on", choices=["on", "off"],
                    help="N > 1, peer transport: pull most of the routed rows over NVLink while the GEMM already runs on the "
                         "first quarter of them (the GEMM leaves --ep-pull-sms SMs to the pull)")
    ap.add_argument("--ep-pull-sms", type=int, default=16)
    ap.add_argument("--ep-chunks", type=int, default=1,
                    help="N > 1, NCCL transport: token chunks pipelined on side streams (all-to-all of one chunk overlaps the "
                         "GEMMs of another); 1 = no overlap.  Measured at 2 GPUs: 2 chunks 30.36 -> 30.02 ms per step on the "
                         "Mixtral-shaped layer, 20.1 -> 22.9 ms on the 64-expert one (twice the launches, half-size GEMMs)")
    ap.add_argument("--ep-capacity-factor", type=float, default=0.0,
                    help="N > 1, peer transport: rows allocated per rank = factor x tokens x top_k with no read-back of the row "
                         "count; 0 (default) = read the exact count back every step")
    ap.add_argument("--gemm-cycles", action="store_true",
                    help="profile builds of the library only: per-role cycle accounting of the grouped GEMMs (no bench line)")
    args = ap.parse_args()
    if args.gemm_cycles:
        torch.cuda.set_device(0)
        w = WORKLOADS[args.workload if args.workload in WORKLOADS else "c4"]
        print(json.dumps(dict(metric="gemm_cycle_profile", config=dict(workload=w["name"]),
                              kernels=gemm_cycle_profile(w, torch.device("cuda", 0)))))
        return
    if args.workload in ("c2", "c3", "rmsnorm"):
        if args.warmup < 3:
            args.warmup = 3
        print(json.dumps(micro_arm(args, args.workload)))
        return
    w = WORKLOADS[args.workload]

    if args.impl == "reference":
        if int(os.environ.get("RANK", "0")) != 0:
            return
        cpu = cpu_arm(w, steps=args.steps, warmup=args.warmup, budget_s=150.0)
        line = {
            "impl": "reference", "metric": METRIC, "value": cpu["value"], "unit": UNIT, "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": cpu["ms_per_step"], "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": w["name"], "hidden": w["H"], "intermediate": w["I"], "experts": w["E"], "top_k": w["k"]},
            "cpu_baseline": cpu,
            "e2e": {"value": cpu["value"], "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        }
        print(json.dumps(line))
        return

    if args.warmup < 3:
        args.warmup = 3
    line = gpu_arm(args, w)
    if line is not None:
        print(json.dumps(line))
        if line.get("parity") is not None and not line["parity"]["ok"]:
            raise SystemExit("parity check of the timed configuration FAILED: " + json.dumps(line["parity"]))


if __name__ == "__main__":
    main()
