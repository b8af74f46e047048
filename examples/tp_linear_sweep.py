"""Runs one tensor-parallel linear at several token counts, with every schedule candidate, and
prints what the cost model predicted next to what was measured.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node W --master-addr 127.0.0.1 \
        --master-port 29550 examples/tp_linear_sweep.py --op gemm_ar --k-total 14336 --n 4096 \
        --tokens 1,16,128,1024,8192

Default shape: the Llama-3-8B-shaped row-parallel down_proj (weights [14336/TP, 4096], GEMM +
all-reduce).  ``--op ag_gemm`` / ``gemm_rs`` run the other layer ops; for ``ag_gemm`` ``--k-total``
is K and ``--n`` is divided by TP.  Candidate 0 is the unfused sequence (this library's GEMM,
then the torch.distributed collective); the others are schedules of the fused kernel
(``--max-candidates`` best-scoring ones are run).
"""
from __future__ import annotations

import argparse
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from edmir_b200 import linear, lowering, symm  # noqa: E402
from edmir_b200.calibration import Calibration  # noqa: E402


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--op", default="gemm_ar", choices=lowering.OPS)
    ap.add_argument("--k-total", type=int, default=14336)
    ap.add_argument("--n", type=int, default=4096)
    ap.add_argument("--tokens", default="1,16,128,1024,8192")
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--max-candidates", type=int, default=8)
    args = ap.parse_args()
    rank, world = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", 0)))
    torch.cuda.set_device(dev)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    calib = Calibration.load()
    tokens = [int(t) for t in args.tokens.split(",")]
    max_m = max(tokens)
    ctx = None
    if world > 1:
        ctx = symm.SymmetricContext.create(symm.default_window_bytes(max_m, args.n, args.k_total, world),
                                           2 * max_m * args.n * 2 + (1 << 20))
    for M in tokens:
        if args.op == "ag_gemm":
            K, N = args.k_total, args.n // world
            if M % world:
                continue
            a = torch.randn(M // world, K, device=dev).bfloat16()
        else:
            K, N = args.k_total // world, args.n
            if args.op == "gemm_rs" and M % (128 * world):
                continue
            a = torch.randn(M, K, device=dev).bfloat16()
        b = (torch.randn(N, K, device=dev) * 0.02).bfloat16()
        spec = lowering.TPLinearSpec(args.op, M, N, K, world)
        sel = lowering.select_schedule(spec, calib, tp_rank=rank)
        out = ctx.empty((M, N), torch.bfloat16) if (ctx is not None and args.op == "gemm_ar") else None
        measured = []
        ranked = sorted(range(len(sel.schedules)), key=lambda i: (sel.costs[i].makespan, i))
        run = sorted(set(ranked[:args.max_candidates]) | {0, sel.chosen})
        for sched in [sel.schedules[i] for i in run]:
            fn = lowering.lower(spec, ctx, sched)
            for _ in range(3):
                fn(a, b, out)
            torch.cuda.synchronize()
            if world > 1:
                dist.barrier()
                torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(args.iters):
                fn(a, b, out)
            e1.record()
            torch.cuda.synchronize()
            t = torch.tensor([e0.elapsed_time(e1) / args.iters * 1e3], device=dev)
            if world > 1:
                dist.all_reduce(t, op=dist.ReduceOp.MAX)
            measured.append(float(t.item()))
        if rank == 0:
            best = run[min(range(len(measured)), key=lambda i: measured[i])]
            cells = "  ".join(f"[{i}] {sel.schedules[i].label()} model {sel.costs[i].makespan / 1e3:.1f} measured {m:.1f}"
                              for i, m in zip(run, measured))
            print(f"{args.op} tp{world} M={M} N={N} K={K}: chosen [{sel.chosen}], fastest [{best}] | {cells}", flush=True)
    st = linear.status()
    assert st[0] == 0, st[:8]
    if ctx is not None:
        dist.barrier()
        torch.cuda.synchronize()
        ctx.close()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
