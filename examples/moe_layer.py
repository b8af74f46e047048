"""Times the expert-parallel MoE layer and checks sampled tokens against the CPU oracle.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node W --master-addr 127.0.0.1 \
        --master-port 29570 examples/moe_layer.py [--tokens 4096] [--hidden 4096] [--ffn 14336] \
        [--experts 8] [--iters 10] [--check-tokens 16]

Default shape: the Mixtral-8x7B-shaped layer of the configuration list -- 4096 tokens per rank,
hidden 4096, 8 experts with ffn 14336, top-2 routing from router logits ~N(0,1) plus a per-expert
bias ~N(0,0.5) (load skew), bf16 with fp32 accumulation.  Prints one JSON line on rank 0: time per
layer call (CUDA events, maximum over ranks), the roofline max(flops at the measured GEMM peak,
dispatch + combine bytes at 900 GB/s per direction) at uniform load, how skewed the routing was,
and the worst rel-L2 of the checked tokens.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from edmir_b200 import linear, moe, symm  # noqa: E402
from oracle import moe as oracle  # noqa: E402
from oracle import tp_linear as tpo  # noqa: E402


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", type=int, default=4096)
    ap.add_argument("--hidden", type=int, default=4096)
    ap.add_argument("--ffn", type=int, default=14336)
    ap.add_argument("--experts", type=int, default=8)
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--check-tokens", type=int, default=16)
    args = ap.parse_args()
    rank, world = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", 0)))
    torch.cuda.set_device(dev)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    T, H, F, E = args.tokens, args.hidden, args.ffn, args.experts
    e_local = E // world
    if world > 1:
        ctx = symm.SymmetricContext.create(moe.window_bytes(T, H, E, world), 1 << 20)
    else:
        ctx = symm.SymmetricContext(0, 1, moe.window_bytes(T, H, E, 1), 1 << 20)
    ws = moe.MoEWorkspace(T, H, F, E, world, device=dev)
    gen = torch.Generator(device="cpu").manual_seed(5000 + rank)
    x = torch.randn(T, H, generator=gen).to(torch.bfloat16).to(dev)
    logits = torch.from_numpy(oracle.router_logits(T, E, 6000 + rank)).to(dev)
    w1 = (torch.randn(e_local * 2 * F, H, device=dev) * 0.02).to(torch.bfloat16)
    w2 = (torch.randn(e_local * H, F, device=dev) * 0.02).to(torch.bfloat16)
    out = torch.empty(T, H, dtype=torch.bfloat16, device=dev)

    def sync():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()

    for _ in range(3):
        moe.moe_forward(ctx, ws, x, logits, w1, w2, out)
    sync()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.iters):
        moe.moe_forward(ctx, ws, x, logits, w1, w2, out)
    e1.record()
    sync()
    us = torch.tensor([e0.elapsed_time(e1) / args.iters * 1e3], device=dev)
    if world > 1:
        dist.all_reduce(us, op=dist.ReduceOp.MAX)
    us = float(us.item())

    # load: rows every expert received in total
    idx = ws.topk_idx.clone()
    per_expert = torch.bincount(idx.reshape(-1).long(), minlength=E).to(torch.float64)
    if world > 1:
        dist.all_reduce(per_expert)
    # parity on a few tokens: the experts' weights come to every rank one expert at a time
    n_check = min(args.check_tokens, T)
    pick = torch.linspace(0, T - 1, n_check).long()
    xs = x[pick.to(dev)].float().cpu().numpy().astype(np.float64)
    sel, wts = oracle.top2(logits[pick.to(dev)].cpu().numpy())
    want = np.zeros((n_check, H))
    for e in range(E):
        owner, el = e // e_local, e % e_local
        w1_e = w1[el * 2 * F:(el + 1) * 2 * F].clone() if owner == rank else torch.empty(2 * F, H, dtype=torch.bfloat16, device=dev)
        w2_e = w2[el * H:(el + 1) * H].clone() if owner == rank else torch.empty(H, F, dtype=torch.bfloat16, device=dev)
        if world > 1:
            dist.broadcast(w1_e, owner)
            dist.broadcast(w2_e, owner)
        hit = (sel == e).any(axis=1)          # an expert is selected at most once per token
        if hit.any():
            weight = np.where(sel[hit] == e, wts[hit], 0.0).sum(axis=1, keepdims=True)
            want[hit] += weight * oracle.expert_ffn(xs[hit], w1_e.float().cpu().numpy(), w2_e.float().cpu().numpy())
    err = torch.tensor([tpo.rel_l2(out[pick.to(dev)].float().cpu().numpy(), want)], device=dev, dtype=torch.float64)
    same_idx = torch.tensor([float(np.array_equal(idx[pick.to(dev)].cpu().numpy(), sel))], device=dev)
    if world > 1:
        dist.all_reduce(err, op=dist.ReduceOp.MAX)
        dist.all_reduce(same_idx, op=dist.ReduceOp.MIN)
    st = linear.status()
    assert st[0] == 0, st[:8]
    if rank == 0:
        flops = moe.layer_flops(T, H, F)
        wire = 2 * moe.dispatch_bytes(T, H, world)
        peak = 1635.9e12
        try:
            with open(os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "MEASURED_PEAKS.json")) as f:
                peak = float(json.load(f)["bf16_tflops"]) * 1e12
        except Exception:
            pass
        roof_us = max(flops / peak, wire / 900e9) * 1e6
        mean = float(per_expert.mean().item())
        print(json.dumps({
            "workload": f"mixtral-8x7b-shaped MoE layer, ep{world}: {T} tokens/rank, hidden {H}, {E} experts x ffn {F}, top-2",
            "us_per_layer": round(us, 1), "tflops_per_gpu_uniform": round(flops / us / 1e6, 1),
            "roofline_us_uniform_load": round(roof_us, 1), "roofline_frac": round(roof_us / us, 4),
            "dispatch_plus_combine_bytes_per_dir": wire,
            "rows_per_expert": [int(v) for v in per_expert.tolist()],
            "most_loaded_over_mean": round(float(per_expert.max().item()) / mean, 3),
            "parity": {"tokens_checked_per_rank": n_check, "max_rel_l2": float(f"{float(err.item()):.3e}"),
                       "routing_matches_oracle": bool(same_idx.item() == 1.0), "ok": bool(err.item() <= 1e-2)},
        }), flush=True)
    sync()
    ctx.close()
    if world > 1:
        dist.destroy_process_group()
    if err.item() > 1e-2 or same_idx.item() != 1.0:
        sys.exit("MoE parity check failed")


if __name__ == "__main__":
    main()
