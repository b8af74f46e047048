"""Host-side multi-rank logic on CPU: two gloo ranks agree on the layer semantics the fused
operators implement (sharding of operands, which rows each rank ends up with) and on the
schedule the selector picks.  No GPU involved: arithmetic is the CPU oracle's, exchanged with
torch.distributed collectives."""
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

WORKER = r'''
import os, sys
import numpy as np, torch, torch.distributed as dist
sys.path.insert(0, sys.argv[1])
from oracle import tp_linear as oracle
from edmir_b200 import lowering
from edmir_b200.calibration import Calibration, wire_bytes

dist.init_process_group("gloo")
rank, world = dist.get_rank(), dist.get_world_size()
M, N, K = 64, 48, 32
gen = lambda seed, shape: torch.randn(*shape, generator=torch.Generator().manual_seed(seed), dtype=torch.float64)
a_all = [gen(10 + r, (M, K)) for r in range(world)]
b_all = [gen(20 + r, (N, K)) for r in range(world)]

# GEMM + reduce-scatter: local partial, then the collective the fused kernel replaces
part = a_all[rank] @ b_all[rank].T
mine = None
chunks = list(part.chunk(world, dim=0))
gathered = [torch.empty_like(chunks[0]) for _ in range(world)]
for owner in range(world):                      # gloo has no reduce_scatter: reduce each block to its owner
    blk = chunks[owner].clone()
    dist.reduce(blk, dst=owner)
    if owner == rank:
        mine = blk
want_rs = oracle.gemm_reduce_scatter([x.numpy() for x in a_all], [x.numpy() for x in b_all])
assert np.allclose(mine.numpy(), want_rs[rank]), "reduce-scatter rows"

# GEMM + all-reduce
full = part.clone(); dist.all_reduce(full)
assert np.allclose(full.numpy(), oracle.gemm_all_reduce([x.numpy() for x in a_all], [x.numpy() for x in b_all])[rank])

# all-gather + GEMM: token-sharded x, column-sharded w
x_all = [gen(30 + r, (M // world, K)) for r in range(world)]
w_all = [gen(40 + r, (N, K)) for r in range(world)]
xs = [torch.empty_like(x_all[0]) for _ in range(world)]
dist.all_gather(xs, x_all[rank])
got = torch.cat(xs, 0) @ w_all[rank].T
assert np.allclose(got.numpy(), oracle.all_gather_gemm([x.numpy() for x in x_all], [x.numpy() for x in w_all])[rank])

# every rank must pick the same schedule for the same spec (the launches are SPMD)
spec = lowering.TPLinearSpec("gemm_rs", 8192, 8192, 3584, 8)
sel = lowering.select_schedule(spec, Calibration(), tp_rank=rank)
picks = [None] * world
dist.all_gather_object(picks, (sel.chosen, [c.makespan for c in sel.costs]))
assert all(p == picks[0] for p in picks), picks
assert wire_bytes("gemm_rs", 8192, 8192, 3584, 8) == 7 * 1024 * 8192 * 2
dist.barrier()
if rank == 0:
    print("gloo host checks ok")
'''


def test_two_gloo_ranks_agree(tmp_path, native_lib):
    script = tmp_path / "worker.py"
    script.write_text(WORKER)
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", MASTER_PORT="29541")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr",
           "127.0.0.1", "--master-port", "29541", str(script), ROOT]
    proc = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=300)
    assert proc.returncode == 0, proc.stdout[-2000:] + proc.stderr[-2000:]
    assert "gloo host checks ok" in proc.stdout
