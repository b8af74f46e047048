"""Controlled overlap probe: when does fusing the exchange into the GEMM help, do nothing, or hurt?

    python -m torch.distributed.run --nnodes=1 --nproc-per-node W --master-addr 127.0.0.1 \
        --master-port 29560 examples/overlap_probe.py [--op ag_gemm|gemm_rs|gemm_ar] \
        [--tokens 128,1024,8192] [--k 8192] [--n 1280] [--json out.json]

For every token count (the message size and the compute window move together with it) the probe
measures the unfused sequence -- this library's GEMM, then the ``torch.distributed`` collective
-- as the *before* execution and a set of fused schedules (varying chunk count, transport and
the number of pusher CTAs, i.e. where and when the transfer starts relative to the compute
window) as *after* executions.  Each measurement becomes an EDM graph
(``lowering.run_measured``); each before/after pair is labelled by the reference's overlap
analysis (EDM-IR/ir/analysis.py:126-149: gain > 5 % "material", > 0 "small", 0 "none", < 0
"regression"), which is the experiment the reference plans as its controlled overlap
intervention (paper/mlsys-2027/claims-and-experiments.md:140-162).  The summary counts how many
pairs fell into the helpful / neutral / harmful regimes and prints one example of each.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from edmir_b200 import graph_json, linear, lowering, symm  # noqa: E402
from edmir_b200.calibration import Calibration  # noqa: E402
from edmir_b200.ir.analysis import analyze_exposure, analyze_overlap  # noqa: E402
from edmir_b200.schedule import Schedule  # noqa: E402

REGIME = {"material": "helpful", "small": "neutral", "none": "neutral", "regression": "harmful", "unknown": "neutral"}


def probe_schedules(op: str, world: int, rows_per_rank: int) -> list[Schedule]:
    """The fused schedules the probe varies: for the all-gather the transfer can start early or
    late (chunks), take SMs from the GEMM (pusher CTAs) or none (copy engines); the
    reduce-scatter / all-reduce have their one fused schedule."""
    if op != "ag_gemm":
        return [Schedule()]
    out = []
    for chunks in (1, 4):
        if chunks > rows_per_rank:
            continue
        out += [Schedule(chunks=chunks, transport="sm", pusher_ctas=4), Schedule(chunks=chunks, transport="sm", pusher_ctas=16),
                Schedule(chunks=chunks, transport="sm", pusher_ctas=48), Schedule(chunks=chunks, transport="ce", side_streams=2)]
    if world > 2:
        out.append(Schedule(chunks=2, transport="hybrid", pusher_ctas=8, ce_peers=(world - 1) // 2, side_streams=1))
    return out


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--op", default="ag_gemm", choices=lowering.OPS)
    ap.add_argument("--tokens", default="256,1024,8192")
    ap.add_argument("--k", type=int, default=8192, help="K of the GEMM (row-parallel ops: per rank)")
    ap.add_argument("--n", type=int, default=1280, help="N of the GEMM (per rank)")
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--json", help="write every labelled pair (and its two EDM graphs) to this file")
    args = ap.parse_args()
    rank, world = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
    if world < 2:
        sys.exit("the probe compares fused and unfused exchanges: run it on at least two ranks")
    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", 0)))
    torch.cuda.set_device(dev)
    dist.init_process_group("nccl", device_id=dev)
    tokens = [int(t) for t in args.tokens.split(",")]
    max_m = max(tokens)
    ctx = symm.SymmetricContext.create(symm.default_window_bytes(max_m, args.n, args.k, world),
                                       max_m * args.n * 2 + (1 << 20))
    calib = Calibration.load()
    results = []
    for M in tokens:
        if M % world or (args.op == "gemm_rs" and M % (128 * world)):
            continue
        rows = M // world if args.op == "ag_gemm" else M
        a = torch.randn(rows, args.k, device=dev).bfloat16()
        b = (torch.randn(args.n, args.k, device=dev) * 0.02).bfloat16()
        spec = lowering.TPLinearSpec(args.op, M, args.n, args.k, world)
        ctx.reset_heap()
        out = ctx.empty((M, args.n), torch.bfloat16) if args.op == "gemm_ar" else None
        # the GEMM alone (same extents, no exchange): the compute window
        ga = torch.randn(M, args.k, device=dev).bfloat16()
        gout = torch.empty(M, args.n, dtype=torch.bfloat16, device=dev)
        for _ in range(3):
            linear.gemm(ga, b, gout)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(args.iters):
            linear.gemm(ga, b, gout)
        e1.record()
        torch.cuda.synchronize()
        window_us = e0.elapsed_time(e1) / args.iters * 1e3

        def measure(sched):
            dist.barrier()
            _, graph, us = lowering.run_measured(spec, ctx, sched, a, b, out, iters=args.iters, gemm_only_us=window_us)
            t = torch.tensor([us], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)   # the launch is as slow as its slowest rank
            if float(t.item()) != us:
                graph = lowering.measured_graph(spec, sched, float(t.item()), min(window_us, float(t.item())),
                                                tp_rank=rank, device=str(dev))
            return graph, float(t.item())

        before, before_us = measure(Schedule(fused=False))
        sel = lowering.select_schedule(spec, calib)
        for sched in probe_schedules(args.op, world, M // world) + [sel.schedule]:
            after, after_us = measure(sched)
            gain = analyze_overlap(before, after)
            ex = analyze_exposure(after)
            results.append({"tokens": M, "schedule": sched.label(), "selected": sched == sel.schedule,
                            "message_bytes": next((u.movement.size_bytes for u in after.uops.values()
                                                   if u.op.startswith("comm.") and u.movement), None),
                            "compute_window_us": round(window_us, 1), "before_us": round(before_us, 1),
                            "after_us": round(after_us, 1), "gain_ratio": round(gain.gain_ratio, 4),
                            "label": gain.label, "regime": REGIME[gain.label],
                            "exposed_comm_us": round(ex.exposed_comm_us, 1), "ecr": round(ex.ecr, 4),
                            "graphs": {"before": graph_json.to_dict(before), "after": graph_json.to_dict(after)}})
            if rank == 0:
                r = results[-1]
                print(f"{args.op} tp{world} M={M:<6d} {r['schedule']:18s} window {r['compute_window_us']:8.1f} us  "
                      f"before {r['before_us']:8.1f}  after {r['after_us']:8.1f}  gain {100 * r['gain_ratio']:+6.1f} %  "
                      f"{r['label']:10s} -> {r['regime']}{'  (selected)' if r['selected'] else ''}", flush=True)
    if rank == 0:
        seen = {}
        for r in results:
            seen.setdefault(r["regime"], []).append(r)
        print("regimes: " + ", ".join(f"{k} {len(v)}" for k, v in sorted(seen.items())))
        for regime, rows in sorted(seen.items()):
            best = max(rows, key=lambda r: abs(r["gain_ratio"]))
            print(f"  {regime}: M={best['tokens']} {best['schedule']} gain {100 * best['gain_ratio']:+.1f} % "
                  f"(window {best['compute_window_us']} us, exposed comm {best['exposed_comm_us']} us)")
        if args.json:
            with open(args.json, "w") as f:
                json.dump(results, f, indent=1)
    st = linear.status()
    assert st[0] == 0, st[:8]
    dist.barrier()
    torch.cuda.synchronize()
    ctx.close()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
