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
METRIC = "moe_fwd_bwd_tokens_per_s"
UNIT = "tokens/s"
# DRAM bytes (read + write) per launch of each GEMM family on the full c4 workload, from a one-pass ncu capture of this
# command (dram__bytes_read.sum + dram__bytes_write.sum; wgrad = mean of its two launches); the summary is under profiles/
MEASURED_DRAM_TRAFFIC = {
    "c4_mixtral_moe_fwd_bwd": {"up_act_fwd": 5910e6, "down_combine_fwd": 6276e6, "dgrad_down": 6500e6, "wgrad": 3686e6,
                               "dgrad_up": 13209e6},
}
GEMM_KERNELS = ("up_act_fwd", "down_combine_fwd", "dgrad_down", "dgrad_up", "wgrad", "grouped_linear",
                "grouped_linear_scatter", "grouped_linear_scatter_peer")


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
        ep, transport = None, "nccl_all_to_all"
        if args.ep_transport in ("auto", "peer"):
            # rows move by NVLink loads / stores issued from the permutation kernels and the GEMM epilogues
            ok = torch.ones(1, device=device)
            try:
                from cute_kernels.peer_parallel import PeerExpertParallelMoE

                ep = PeerExpertParallelMoE(E, k, T, H, torch.bfloat16, dist.group.WORLD)
                transport = "peer_memory"
            except Exception as exc:  # symmetric memory not available on this box
                if args.ep_transport == "peer":
                    raise
                print(f"[bench] rank {rank}: peer-memory transport unavailable ({exc}); using NCCL all-to-all", file=sys.stderr)
                ok.zero_()
            dist.all_reduce(ok, op=dist.ReduceOp.MIN)
            if ok.item() == 0:
                ep, transport = None, "nccl_all_to_all"
        if ep is None:
            ep = ExpertParallelMoE(E, k, dist.group.WORLD)

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
            y = ck.fused_experts(x, rw, sel, inp["w_fc"], inp["w_proj"], k)
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

    def e2e_loop(n_steps: int) -> None:
        pending = stage_in()
        for i in range(n_steps):
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
    h2d = sum(v.numel() * v.element_size() for v in host.values())
    d2h = 2 * T * H * 2
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
        traffic=(MEASURED_DRAM_TRAFFIC.get(w["name"], {}).get(dom) if world == 1 else None),
        traffic_unit="bytes per launch (dram__bytes_read.sum + dram__bytes_write.sum, one ncu capture)",
        peak_source=f"bf16_tflops_sustained of {peaks['source']}",
        all_gemms=dict(ms_per_step=gemm_ms, tflops=gemm_flops / (gemm_ms * 1e-3) / 1e12,
                       frac_of_measured_sustained=gemm_flops / (gemm_ms * 1e-3) / 1e12 / peak,
                       frac_of_measured_burst=gemm_flops / (gemm_ms * 1e-3) / 1e12 / float(peaks["bf16_tflops"]),
                       frac_of_nominal_2250=gemm_flops / (gemm_ms * 1e-3) / 1e12 / 2250.0),
        kernels={n: {kk: round(vv, 4) if isinstance(vv, float) else vv for kk, vv in v.items()} for n, v in kernels.items()},
    )

    cpu = cpu_arm(w, steps=1, warmup=0, budget_s=60.0) if (world == 1 and not args.no_cpu_baseline) else None

    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic",
        "config": {"workload": w["name"], "tokens_per_gpu": T, "hidden": H, "intermediate": I, "experts": E, "top_k": k,
                   "parallelism": f"ep{world}" if world > 1 else "single",
                   **({"ep_transport": transport} if world > 1 else {}), "l2_policy": "inputs_exceed_l2",
                   "step": "route+gather+up_swiglu+down_combine+backward(dgrad,wgrad,swiglu_bwd,router_grad)"},
        "clocks": clocks,
        "e2e": {"value": world * T / (e2e_ms * 1e-3), "unit": UNIT, "ms_per_step": e2e_ms, "h2d_bytes_per_step": h2d,
                "d2h_bytes_per_step": d2h},
        "gpu_launches": launches,
        "roofline": roofline,
    }
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


def micro_arm(args, which: str) -> dict:
    import numpy as np

    import ck_oracle as orc
    import cute_kernels as ck

    torch.cuda.set_device(0)
    dev = torch.device("cuda", 0)
    peaks = measured_peaks()
    peak = float(peaks["hbm_gbs"])
    sampler = ClockSampler(0)
    flush = torch.zeros(128 << 20, dtype=torch.float32, device=dev)
    results = {}
    if which == "c2":
        n, E = 1 << 24, 64
        for dist_name in ("uniform", "zipf"):
            ids = torch.from_numpy(orc.gen_ids(0, n, E, dist_name, np.int32)).to(dev)
            t_route = _time_each(lambda: ck.route(ids, E, with_tile_metadata=False), args.steps, args.warmup, flush)
            t_count = _time_each(lambda: ck.continuous_count_cute(ids, E), args.steps, args.warmup, flush)
            results[dist_name] = dict(
                route_ms=statistics.median(t_route), route_gbs=12.0 * n / (statistics.median(t_route) * 1e-3) / 1e9,
                count_ms=statistics.median(t_count), count_gbs=4.0 * n / (statistics.median(t_count) * 1e-3) / 1e9)
        sampler.mark_begin(); sampler.mark_end()
        head = results["uniform"]
        line = dict(metric="route_hbm_gb_per_s", value=head["route_gbs"], unit="GB/s", ms_per_step=head["route_ms"],
                    config=dict(workload="c2_count_scan_stable_scatter", n_ids=n, experts=E, ids_dtype="int32",
                                l2_policy="l2_flushed_between_launches", draws=["uniform", "zipf(1.2)"]),
                    roofline=dict(bound="hbm", kernel="route_hist + route_scan + route_scatter (3 launches)",
                                  achieved=head["route_gbs"], peak=peak, unit="GB/s", frac=head["route_gbs"] / peak,
                                  traffic=None, algorithmic_bytes=12 * n, peak_source=f"hbm_gbs of {peaks['source']}"),
                    detail=results)
    else:
        rows, cols = 16384, 14336
        g = torch.Generator(device=dev).manual_seed(0)
        gate = torch.randn(rows, cols, generator=g, device=dev, dtype=torch.float32).bfloat16().requires_grad_()
        up = torch.randn(rows, cols, generator=g, device=dev, dtype=torch.float32).bfloat16().requires_grad_()
        dy = torch.randn(rows, cols, generator=g, device=dev, dtype=torch.float32).bfloat16()
        nel = rows * cols
        with torch.no_grad():
            # the 512 MB flush write also lets the host run ahead, so the events bracket device time only
            t_fwd = _time_each(lambda: ck.swiglu_cute(gate, up), args.steps, args.warmup, flush)
        out = ck.swiglu_cute(gate, up)

        def bwd():
            gate.grad = None
            up.grad = None
            out.backward(dy, retain_graph=True)

        t_bwd = _time_each(bwd, args.steps, args.warmup, flush)
        sampler.mark_begin(); sampler.mark_end()
        f_ms, b_ms = statistics.median(t_fwd), statistics.median(t_bwd)
        results = dict(fwd_ms=f_ms, fwd_gbs=6.0 * nel / (f_ms * 1e-3) / 1e9, bwd_ms=b_ms, bwd_gbs=10.0 * nel / (b_ms * 1e-3) / 1e9)
        both = 16.0 * nel / ((f_ms + b_ms) * 1e-3) / 1e9
        line = dict(metric="swiglu_fwd_bwd_hbm_gb_per_s", value=both, unit="GB/s", ms_per_step=f_ms + b_ms,
                    config=dict(workload="c3_swiglu_fwd_bwd", shape=[rows, cols], l2_policy="inputs_exceed_l2"),
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
    ap.add_argument("--workload", default="c4", choices=sorted(WORKLOADS) + ["c2", "c3"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--ep-transport", default="auto", choices=["auto", "peer", "nccl"],
                    help="N > 1: rows cross GPUs by peer-memory loads/stores from the kernels (default when symmetric "
                         "memory is available) or by NCCL all-to-all")
    args = ap.parse_args()
    if args.workload in ("c2", "c3"):
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


if __name__ == "__main__":
    main()
