"""Generates the golden vectors under tests/golden/ by running the REFERENCE's own torch path.

Run in a container that has the reference checkout:
    PYTHONDONTWRITEBYTECODE=1 python tests/golden/make_golden.py /path/to/reference [rmsnorm]
(a second argument regenerates that fixture file alone)
It imports MoE_Torch, swiglu_torch, swiglu_packed_torch, continuous_count_torch, rmsnorm_torch and
fused_residual_add_rmsnorm_torch from that checkout,
feeds them seeded inputs (the generators of oracle/ck_oracle.py), and stores inputs' seeds and the
reference outputs as small .npz files.  The fixtures, not the checkout, travel with the repository.
"""

import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, os.path.join(ROOT, "oracle"))
import ck_oracle as orc  # noqa: E402


def main(ref_path: str, only: str | None = None) -> None:
    sys.path.insert(0, ref_path)
    from cute_kernels import (MoE_Torch, continuous_count_torch, fused_residual_add_rmsnorm_torch, rmsnorm_torch,
                              swiglu_packed_torch, swiglu_torch)

    torch.manual_seed(0)

    # ---- continuous_count / routing: reference test recipe (tests/kernels/continuous_count_test.py:33-41)
    out = {}
    for name, n, E, dist, dt in [("u72_i64", 4099, 72, "uniform", np.int64), ("u72_i32", 3001, 72, "uniform", np.int32),
                                 ("zipf64", 20000, 64, "zipf", np.int32), ("tiny", 5, 8, "uniform", np.int64)]:
        ids = orc.gen_ids(7, n, E, dist, dt)
        t = torch.from_numpy(ids)
        out[f"{name}_counts"] = continuous_count_torch(t, E).numpy()
        srt = torch.sort(t.long(), stable=True)
        out[f"{name}_sorted_idx"] = srt.indices.numpy().astype(np.int32)
        out[f"{name}_end_off"] = t.long().bincount(minlength=E).cumsum(-1).numpy().astype(np.int32)
        out[f"{name}_meta"] = np.array([n, E, {"uniform": 0, "zipf": 1}[dist], np.dtype(dt).itemsize])
    if only is None:
        np.savez_compressed(os.path.join(HERE, "routing.npz"), **out)

    # ---- swiglu fwd/bwd, fp32 + bf16 (tests/kernels/swiglu_test.py:33-49)
    out = {}
    g = torch.Generator().manual_seed(11)
    for name, shape, dt in [("f32", (37, 53), torch.float32), ("bf16", (64, 96), torch.bfloat16), ("f16", (9, 40), torch.float16)]:
        gate = torch.randn(shape, generator=g).to(dt).requires_grad_()
        up = torch.randn(shape, generator=g).to(dt).requires_grad_()
        dy = torch.randn(shape, generator=g).to(dt)
        z = swiglu_torch(gate, up)
        z.backward(dy)
        xp = torch.cat([up.detach(), gate.detach()], dim=-1).requires_grad_()
        zp = swiglu_packed_torch(xp)
        zp.backward(dy)
        for k, v in dict(gate=gate, up=up, dy=dy, out=z, dgate=gate.grad, dup=up.grad, packed_out=zp, packed_dx=xp.grad).items():
            out[f"{name}_{k}"] = v.detach().float().numpy()
    if only is None:
        np.savez_compressed(os.path.join(HERE, "swiglu.npz"), **out)

    # ---- rmsnorm / fused residual add + rmsnorm fwd+bwd (tests/kernels/rmsnorm_test.py:51-72,
    #      tests/kernels/fused_residual_add_rmsnorm_test.py:45-86: eps 1e-5, loss = sum, resp. sum(2 z + 3 r))
    out = {}
    g = torch.Generator().manual_seed(21)
    for name, shape, dt, has_w, mult in [("f32_w", (13, 200), torch.float32, True, 0.9), ("f32_now", (5, 33), torch.float32, False, None),
                                         ("bf16_w", (24, 256), torch.bfloat16, True, 0.9), ("f16_w", (3, 1032), torch.float16, True, None)]:
        x = torch.randn(shape, generator=g).to(dt).requires_grad_()
        res = torch.randn(shape, generator=g).to(dt).requires_grad_()
        w = torch.randn(shape[-1], generator=g).to(dt).requires_grad_() if has_w else None
        z = rmsnorm_torch(x, w, 1e-5)
        z.sum().backward()
        rec = dict(x=x, res=res, z=z, dx=x.grad)
        if has_w:
            rec.update(w=w, dw=w.grad)
        x2 = x.detach().clone().requires_grad_()
        w2 = w.detach().clone().requires_grad_() if has_w else None
        z2, r2 = fused_residual_add_rmsnorm_torch(x2, res, w2, 1e-5, mult)
        (z2 * 2 + r2 * 3).sum().backward()
        rec.update(fz=z2, fr=r2, fdx=x2.grad, fdres=res.grad)
        if has_w:
            rec.update(fdw=w2.grad)
        for k, v in rec.items():
            out[f"{name}_{k}"] = v.detach().float().numpy()
        out[f"{name}_meta"] = np.array([0.0 if mult is None else mult, float(has_w)])
    np.savez_compressed(os.path.join(HERE, "rmsnorm.npz"), **out)
    if only == "rmsnorm":
        return

    # ---- MoE fwd+bwd through MoE_Torch itself (reference module, reference routing)
    out = {}
    cases = {
        "small": dict(T=96, H=64, I=128, E=4, k=2, expert_bias=False, seed=3),
        "c1": dict(orc.CONFIGS["c1_cpu"], seed=0),
        "skew": dict(T=200, H=64, I=64, E=8, k=4, expert_bias=True, seed=5),
    }
    for name, c in cases.items():
        seed = c.pop("seed")
        inp = orc.gen_moe_inputs(seed, **c)
        moe = MoE_Torch(num_experts=c["E"], num_experts_per_tok=c["k"], hidden_size=c["H"], intermediate_size=c["I"],
                        activation_function=swiglu_packed_torch, is_glu=True, add_bias=False, std=0.02)
        with torch.no_grad():
            moe.c_fc.weight.copy_(inp["w_fc"])
            moe.c_proj.weight.copy_(inp["w_proj"])
        x = inp["x"].clone().requires_grad_()
        rw = inp["router_weights"].clone().requires_grad_()
        # the expert path with the generator's routing (logits exactly N(0,1)), as in the benchmark configs
        y = moe._compute_experts(x, rw, inp["selected_experts"])
        y.backward(inp["grad_out"])
        full = name != "c1"
        res = dict(y=y.detach(), dx=x.grad, d_router_weights=rw.grad, d_w_fc=moe.c_fc.weight.grad, d_w_proj=moe.c_proj.weight.grad)
        for k, v in res.items():
            v = v.float()
            out[f"{name}_{k}_sum"] = np.array([v.double().sum().item(), v.double().abs().sum().item(), v.double().pow(2).sum().item()])
            if full or k in ("d_router_weights",):
                out[f"{name}_{k}"] = v.numpy()
            else:
                flat = v.reshape(-1)
                stride = max(1, flat.numel() // 4096)
                out[f"{name}_{k}_sample"] = flat[::stride][:4096].numpy()
        out[f"{name}_cfg"] = np.array([seed, c["T"], c["H"], c["I"], c["E"], c["k"], int(c["expert_bias"])])
        # end-to-end module forward (router included) on the small cases
        if full:
            with torch.no_grad():
                moe.gate.weight.copy_(torch.randn(c["E"], c["H"], generator=torch.Generator().manual_seed(seed + 100)) / c["H"] ** 0.5)
                y2, logits = moe(inp["x"])
            out[f"{name}_module_y"] = y2.numpy()
            out[f"{name}_module_logits"] = logits.numpy()
            out[f"{name}_module_gate_w"] = moe.gate.weight.detach().numpy()
    np.savez_compressed(os.path.join(HERE, "moe.npz"), **out)
    for f in ("routing.npz", "swiglu.npz", "rmsnorm.npz", "moe.npz"):
        print(f, os.path.getsize(os.path.join(HERE, f)))


if __name__ == "__main__":
    if len(sys.argv) not in (2, 3):
        raise SystemExit("usage: make_golden.py /path/to/reference [rmsnorm]")
    main(sys.argv[1], sys.argv[2] if len(sys.argv) == 3 else None)
