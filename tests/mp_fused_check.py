"""Multi-process parity check of the fused operators on real GPUs (one process per GPU).

    python -m torch.distributed.run --nnodes=1 --nproc-per-node W --master-addr 127.0.0.1 \
        --master-port 29511 tests/mp_fused_check.py [--big]

Every rank builds all ranks' seeded inputs on the CPU, evaluates the oracle locally and compares
its own device result.  Exit code 0 means every rank passed.  Launched by
tests/test_multigpu.py when at least two GPUs are visible.
"""
import dataclasses
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

from edmir_b200 import linear, symm  # noqa: E402
from edmir_b200.schedule import Schedule  # noqa: E402
from oracle import tp_linear as oracle  # noqa: E402

BF16_TOL, FP32_TOL = 1e-2, 1e-5


def rand(shape, scale, dtype, seed):
    g = torch.Generator(device="cpu").manual_seed(seed)
    return (torch.randn(*shape, generator=g, dtype=torch.float32) * scale).to(dtype)


def main() -> int:
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ["LOCAL_RANK"]))
    dev = torch.device("cuda", int(os.environ["LOCAL_RANK"]))
    dist.init_process_group("nccl", device_id=dev)
    big = "--big" in sys.argv
    ctx = symm.SymmetricContext.create(512 << 20 if big else 96 << 20, 64 << 20)
    linear.clear_status()
    failures = []
    npf = lambda t: t.float().cpu().numpy()

    cases = [("gemm_rs", 256 * world, 512, 256, torch.bfloat16, 1),
             ("gemm_ar", 200, 1032, 264, torch.bfloat16, 1),
             ("gemm_ar", 1, 4096, 1792, torch.bfloat16, 1),
             ("ag_gemm", 256 * world, 520, 512, torch.bfloat16, 2),
             ("ag_gemm", 64 * world, 256, 128, torch.bfloat16, 1),
             ("ag_gemm_ce", 256 * world, 520, 512, torch.bfloat16, 2),
             ("ag_gemm_cs", 256 * world, 520, 512, torch.bfloat16, 2),
             ("ag_gemm_push", 256 * world, 520, 512, torch.bfloat16, 2),
             ("ag_gemm_push", 64 * world, 256, 136, torch.bfloat16, 1),
             ("ag_gemm_hybrid", 256 * world, 264, 512, torch.bfloat16, 2),
             ("gemm_ar", 256, 1024, 512, torch.float32, 1),
             ("gemm_ar_oneshot", 1, 4096, 1792, torch.bfloat16, 1),
             ("gemm_ar_oneshot", 48, 1032, 264, torch.bfloat16, 1),
             ("gemm_ar_oneshot", 128, 1024, 512, torch.float32, 1)]
    if big:
        cases += [("gemm_rs", 8192, 8192, 1024, torch.bfloat16, 1), ("ag_gemm", 8192, 1280, 8192, torch.bfloat16, 4),
                  ("ag_gemm_ce", 8192, 1280, 8192, torch.bfloat16, 2), ("ag_gemm_cs", 8192, 1280, 8192, torch.bfloat16, 4), ("ag_gemm_push", 8192, 1280, 8192, torch.bfloat16, 4),
                  ("ag_gemm_hybrid", 8192, 2048, 8192, torch.bfloat16, 2), ("gemm_ar", 1024, 4096, 14336 // world, torch.bfloat16, 1)]
    schedules = {"": Schedule(transport="sm"), "_ce": Schedule(transport="ce"), "_cs": Schedule(transport="cs"),
                 "_push": Schedule(transport="sm", pusher_ctas=16),
                 "_hybrid": Schedule(transport="hybrid", pusher_ctas=8, ce_peers=max(1, (world - 1) // 2), side_streams=1),
                 "_oneshot": Schedule(one_shot=True)}
    for idx, (op, M, N, K, dtype, chunks) in enumerate(cases):
        wscale = 1.0 if dtype == torch.float32 else 0.02
        suffix = next((k for k in ("_ce", "_cs", "_push", "_hybrid", "_oneshot") if op.endswith(k)), "")
        op = op[:len(op) - len(suffix)] if suffix else op
        sched = dataclasses.replace(schedules[suffix], chunks=chunks) if op == "ag_gemm" else schedules[suffix]
        rows = M // world if op == "ag_gemm" else M
        a_all = [rand((rows, K), 1.0, dtype, 1000 * idx + r) for r in range(world)]
        b_all = [rand((N, K), wscale, dtype, 1000 * idx + 500 + r) for r in range(world)]
        # this rank's expected result only (the full-size cases are hundreds of GFLOP in float64)
        if op == "ag_gemm":
            want = oracle.gemm(np.concatenate([npf(t) for t in a_all], axis=0), npf(b_all[rank]))
        else:
            lo, hi = (rank * (M // world), (rank + 1) * (M // world)) if op == "gemm_rs" else (0, M)
            want = None
            for s in range(world):  # fixed rank order, like the reduction
                part = oracle.gemm(npf(a_all[s][lo:hi]), npf(b_all[s]))
                want = part if want is None else want + part
        a, b = a_all[rank].to(dev), b_all[rank].to(dev)
        out = None
        for call in range(3):
            torch.cuda.synchronize()
            dist.barrier()
            ctx.poison()           # nobody has copies in flight: a row read before it arrives is a NaN
            torch.cuda.synchronize()
            dist.barrier()
            if op == "gemm_rs":
                out = ctx.gemm_rs(a, b)
            elif op == "gemm_ar":
                out = ctx.gemm_ar(a, b, out, schedule=sched)
            else:
                out = ctx.ag_gemm(a, b, schedule=sched)
            torch.cuda.synchronize()
            err = oracle.rel_l2(npf(out), want)
            tol = FP32_TOL if dtype == torch.float32 else BF16_TOL
            if not err <= tol:
                failures.append((op, M, N, K, str(dtype), call, err))
        if op == "gemm_ar":  # all ranks must hold identical bits
            mine = out.view(torch.uint8).to(torch.int32).sum().reshape(1).to(torch.float64)
            lo, hi = mine.clone(), mine.clone()
            dist.all_reduce(lo, op=dist.ReduceOp.MIN)
            dist.all_reduce(hi, op=dist.ReduceOp.MAX)
            if lo.item() != hi.item():
                failures.append((op, "ranks differ"))
    st = linear.status()
    if st[0] != 0:
        failures.append(("device status", st[:8]))
    flag = torch.tensor([len(failures)], device=dev)
    dist.all_reduce(flag)
    if failures:
        print(f"rank {rank} FAILURES: {failures}", flush=True)
    elif rank == 0:
        print(f"multi-GPU parity ok on {world} ranks ({len(cases)} cases)", flush=True)
    dist.barrier()
    torch.cuda.synchronize()
    ctx.close()
    dist.destroy_process_group()
    return 1 if flag.item() else 0


if __name__ == "__main__":
    sys.exit(main())
