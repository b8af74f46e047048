"""Schedule sweep: every all-gather schedule family, the reduce-scatter and all-reduce launches and
the link probe on the ranks of one box, each next to the cost model's prediction.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node W --master-addr 127.0.0.1 \
        --master-port 29512 examples/schedule_sweep.py

Shapes: the Llama-3-70B layer at TP=8-local extents and 8192 tokens (qkv, gate_up: all-gather +
GEMM; o_proj, down: GEMM + reduce-scatter) and the Llama-3-8B down_proj with all-reduce at
1..8192 tokens (fused kernel, one-shot schedule, this library's GEMM + the library all-reduce).  Prints one JSON line per measurement on rank 0 (CUDA events, maximum over ranks)
and writes them to ``out/sweep_tp<W>.json``.  The figures calibrate
``edmir_b200/calibration_b200.json``.
"""
import json, os, sys, time
sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import torch, torch.distributed as dist
from edmir_b200 import linear, lowering, symm
from edmir_b200.calibration import Calibration
from edmir_b200.schedule import Schedule

rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
dev = torch.device("cuda", int(os.environ["LOCAL_RANK"])); torch.cuda.set_device(dev)
dist.init_process_group("nccl", device_id=dev)
M = 8192
ctx = symm.SymmetricContext.create(symm.default_window_bytes(M, 8192, 8192, world) // 2 + (64 << 20), 8192 * 4096 * 2 + (1 << 20))
calib = Calibration.load()
out_lines = []

def timed(fn, iters=20, warm=3):
    for _ in range(warm): fn()
    torch.cuda.synchronize(); dist.barrier(); torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters): fn()
    e1.record(); torch.cuda.synchronize()
    t = torch.tensor([e0.elapsed_time(e1) / iters * 1e3], device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())

def emit(**kw):
    if rank == 0:
        print(json.dumps(kw), flush=True)
        out_lines.append(kw)

t_start = time.time()
# ---- all-gather + GEMM
for name, K, N in (("qkv", 8192, 1280), ("gate_up", 8192, 7168)):
    x = torch.randn(M // world, K, device=dev).bfloat16()
    w = (torch.randn(N, K, device=dev) * 0.02).bfloat16()
    out = torch.empty(M, N, device=dev, dtype=torch.bfloat16)
    xg = torch.randn(M, K, device=dev).bfloat16()
    emit(op=name, sched="gemm_only", us=timed(lambda: linear.gemm(xg, w, out)))
    spec = lowering.TPLinearSpec("ag_gemm", M, N, K, world)
    sel = lowering.select_schedule(spec, calib)
    cands = []
    for p in (8, 12, 16, 24, 32):
        for c in (1, 2, 4):
            cands.append(Schedule(chunks=c, transport="sm", pusher_ctas=p))
    cands += [Schedule(chunks=2, transport="sm", pusher_ctas=0), Schedule(chunks=1, transport="ce", side_streams=2),
              Schedule(chunks=4, transport="ce", side_streams=2), Schedule(chunks=2, transport="ce", side_streams=2),
              Schedule(chunks=2, transport="cs", side_streams=2), Schedule(chunks=4, transport="cs", side_streams=2),
              Schedule(chunks=4, transport="cs", side_streams=4), Schedule(chunks=8, transport="cs", side_streams=2)]
    if world > 2:
        far = (world - 1) // 2
        cands += [Schedule(chunks=4, transport="hybrid", pusher_ctas=8, ce_peers=far, side_streams=1),
                  Schedule(chunks=4, transport="hybrid", pusher_ctas=16, ce_peers=max(1, far // 2), side_streams=1)]
    for s in cands:
        try:
            us = timed(lambda: ctx.ag_gemm(x, w, out, schedule=s), iters=15)
        except Exception as e:
            emit(op=name, sched=s.label(), error=str(e)); continue
        g = lowering.schedule_graph(spec, s, calib)
        emit(op=name, sched=s.label(), us=round(us, 1), model_us=round(lowering.graph_cost(g).makespan / 1e3, 1),
             chosen=(s.label() == sel.schedule.label()))
# ---- reduce-scatter
for name, K, N in (("o_proj", 1024, 8192), ("down", 3584, 8192)):
    a = torch.randn(M, K, device=dev).bfloat16()
    b = (torch.randn(N, K, device=dev) * 0.02).bfloat16()
    out = torch.empty(M // world, N, device=dev, dtype=torch.bfloat16)
    full = torch.empty(M, N, device=dev, dtype=torch.bfloat16)
    emit(op=name, sched="gemm_only", us=timed(lambda: linear.gemm(a, b, full)))
    spec = lowering.TPLinearSpec("gemm_rs", M, N, K, world)
    sel = lowering.select_schedule(spec, calib)
    emit(op=name, sched="fused", us=round(timed(lambda: ctx.gemm_rs(a, b, out)), 1), model_us=round(sel.predicted_us, 1))
    def unf():
        torch.matmul(a, b.t(), out=full); dist.reduce_scatter_tensor(out, full)
    emit(op=name, sched="unfused_nccl", us=round(timed(unf), 1))
# ---- all-reduce (8B down_proj): fused kernel, one-shot (where it is a candidate), GEMM + library all-reduce
K, N = 14336 // world, 4096
w = (torch.randn(N, K, device=dev) * 0.02).bfloat16()
for m in (1, 16, 128, 512, 1024, 8192):
    a = torch.randn(m, K, device=dev).bfloat16()
    o_sym = ctx.empty((m, N), torch.bfloat16)
    o_any = torch.empty(m, N, device=dev, dtype=torch.bfloat16)
    spec = lowering.TPLinearSpec("gemm_ar", m, N, K, world)
    for s in (c for c in lowering.candidates(spec) if c.fused):
        us = timed(lambda: ctx.gemm_ar(a, w, o_any if s.one_shot else o_sym, schedule=s), iters=30)
        g = lowering.schedule_graph(spec, s, calib)
        emit(op=f"ar_m{m}", sched=s.label(), us=round(us, 1), model_us=round(lowering.graph_cost(g).makespan / 1e3, 1))
    def unf():
        linear.gemm(a, w, o_any); dist.all_reduce(o_any)
    emit(op=f"ar_m{m}", sched="unfused", us=round(timed(unf, iters=30), 1))
    emit(op=f"ar_m{m}", sched="gemm_only", us=round(timed(lambda: linear.gemm(a, w, o_any), iters=30), 1))
    ctx.reset_heap()
# ---- link probe: one peer and all peers
for mode in (0, 1, 2, 3):
    nbytes = 64 << 20
    us = timed(lambda: ctx.p2p_probe((rank + 1) % world, nbytes, mode), iters=10)
    emit(op="probe", sched=f"mode{mode}_next", us=round(us, 1), gbs=round(nbytes / us / 1e3, 1))
st = linear.status()
emit(op="status", sched=str(st[:6]), us=0, elapsed_s=round(time.time() - t_start, 1))
if rank == 0:
    os.makedirs("out", exist_ok=True)
    json.dump(out_lines, open(f"out/sweep_tp{world}.json", "w"), indent=1)
dist.barrier(); torch.cuda.synchronize(); ctx.close(); dist.destroy_process_group()
