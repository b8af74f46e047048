"""Per-role device time of the fused launches (where a launch spends its time).

    python -m torch.distributed.run --nnodes=1 --nproc-per-node W --master-addr 127.0.0.1 \
        --master-port 29530 examples/role_profile.py [--tokens 8192] [--chunks 2] \
        [--transport sm|ce|hybrid] [--pusher-ctas 16] [--ce-peers 2] [--side-streams 2] [--probe]

For each linear of the benchmark layer (qkv, gate_up: all-gather+GEMM; o_proj, down:
GEMM+reduce-scatter; TP=8-local extents) it prints the launch time and, from the library's
device-side accounting (``edm_profile_enable``), the microseconds per CTA and launch that each
warp role spent waiting or working, for the fused launch and for the same GEMM without exchange.
``--probe`` also times the raw link (``edm_comm_p2p_probe``) to the next rank.
"""
from __future__ import annotations

import argparse
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from edmir_b200 import linear, symm  # noqa: E402
from edmir_b200.schedule import Schedule  # noqa: E402

LAYER = (("qkv", "ag_gemm", 8192, 1280), ("gate_up", "ag_gemm", 8192, 7168),
         ("o_proj", "gemm_rs", 1024, 8192), ("down", "gemm_rs", 3584, 8192))


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", type=int, default=8192)
    ap.add_argument("--chunks", type=int, default=2)
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--probe", action="store_true")
    ap.add_argument("--transport", default="sm", choices=("sm", "ce", "hybrid"), help="how all-gather shards travel")
    ap.add_argument("--pusher-ctas", type=int, default=0, help="CTAs that only push the shard (0: push warps in every GEMM CTA)")
    ap.add_argument("--ce-peers", type=int, default=0, help="hybrid: farthest peers served by copy engines")
    ap.add_argument("--side-streams", type=int, default=2, help="copy engines: streams the copies are spread over")
    args = ap.parse_args()
    sched = Schedule(chunks=args.chunks, transport=args.transport, pusher_ctas=args.pusher_ctas,
                     ce_peers=args.ce_peers, side_streams=args.side_streams)
    rank, world = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", 0)))
    torch.cuda.set_device(dev)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    M = args.tokens
    ctx = symm.SymmetricContext.create(symm.default_window_bytes(M, 8192, 8192, world), 1 << 20) if world > 1 else None

    def measure(label, fn):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()
        linear.profile_read(True)
        linear.profile_enable(True)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(args.iters):
            fn()
        e1.record()
        torch.cuda.synchronize()
        prof = linear.profile_read(True)
        linear.profile_enable(False)
        ctas = max(prof["ctas"], 1)
        if rank == 0:
            per = {k: round(v / ctas / 1e3, 1) for k, v in prof.items() if v and k != "ctas" and not k.startswith("reserved") }
            print(f"{label}: {e0.elapsed_time(e1) / args.iters * 1e3:.1f} us/launch  per-CTA us: {per}", flush=True)

    for name, op, K, N in LAYER:
        rows = M // world if op == "ag_gemm" else M
        a = torch.randn(rows, K, device=dev).bfloat16()
        b = (torch.randn(N, K, device=dev) * 0.02).bfloat16()
        full_a = torch.randn(M, K, device=dev).bfloat16()
        out = torch.empty(M // world if op == "gemm_rs" else M, N, dtype=torch.bfloat16, device=dev)
        plain_out = torch.empty(M, N, dtype=torch.bfloat16, device=dev)
        if world > 1:
            if op == "ag_gemm":
                measure(f"{name} {op} tp{world} {sched.label()}", lambda: ctx.ag_gemm(a, b, out, schedule=sched))
            else:
                measure(f"{name} {op} tp{world}", lambda: ctx.gemm_rs(a, b, out))
        measure(f"{name} gemm only", lambda: linear.gemm(full_a, b, plain_out))

    if args.probe and world > 1:
        for mode in (0, 1):
            nbytes = 64 << 20
            peer = (rank + 1) % world
            for _ in range(3):
                ctx.p2p_probe(peer, nbytes, mode)
            torch.cuda.synchronize()
            dist.barrier()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(10):
                ctx.p2p_probe(peer, nbytes, mode)
            e1.record()
            torch.cuda.synchronize()
            us = e0.elapsed_time(e1) / 10 * 1e3
            if rank == 0:
                print(f"link probe mode {mode}: 64 MiB to rank+1 in {us:.1f} us = {nbytes / us / 1e3:.0f} GB/s", flush=True)
    st = linear.status()
    assert st[0] == 0, st[:8]
    if ctx is not None:
        dist.barrier()
        torch.cuda.synchronize()
        ctx.close()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
