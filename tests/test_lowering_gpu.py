"""The lowering's launch and measurement path on a GPU (single rank: the schedule degenerates to
the plain GEMM), and the device-side role accounting."""
import pytest
import torch

from edmir_b200 import linear, lowering, symm
from edmir_b200.ir.analysis import analyze_exposure
from edmir_b200.ir.printing import format_summary
from oracle import tp_linear as oracle

pytestmark = pytest.mark.gpu


def test_run_measured_single_rank(cuda_clean):
    spec = lowering.TPLinearSpec("gemm_rs", 512, 256, 128, 1)
    sel = lowering.select_schedule(spec)
    assert sel.schedule.chunks == 1
    g = torch.Generator(device="cpu").manual_seed(5)
    a = torch.randn(512, 128, generator=g).to(torch.bfloat16).cuda()
    b = (torch.randn(256, 128, generator=g) * 0.02).to(torch.bfloat16).cuda()
    out, graph, us = lowering.run_measured(spec, None, sel.schedule, a, b, iters=3, warmup=1)
    assert oracle.rel_l2(out.float().cpu().numpy(), oracle.gemm(a.float().cpu().numpy(), b.float().cpu().numpy())) <= 1e-2
    ex = analyze_exposure(graph)
    assert us > 0 and ex.phase_time_us == pytest.approx(us) and ex.total_comm_us == 0.0
    assert "critical_path_us=" in format_summary(graph)


def test_role_accounting_counts_ctas(cuda_clean):
    a = torch.zeros(1024, 256, dtype=torch.bfloat16, device="cuda")
    b = torch.zeros(512, 256, dtype=torch.bfloat16, device="cuda")
    linear.profile_read(reset=True)
    linear.profile_enable(True)
    try:
        linear.gemm(a, b)
        prof = linear.profile_read(reset=True)
    finally:
        linear.profile_enable(False)
    assert prof["ctas"] == 16                      # 4 x 2 pair tiles -> 16 CTAs
    assert prof["kernel_total"] > 0 and prof["epilogue_total"] > 0
    linear.gemm(a, b)
    assert linear.profile_read(reset=True)["ctas"] == 0   # accounting is off again


def _rand(shape, scale, seed):
    g = torch.Generator(device="cpu").manual_seed(seed)
    return (torch.randn(*shape, generator=g) * scale).to(torch.bfloat16)


@pytest.mark.parametrize("world", [2, 4])
@pytest.mark.parametrize("op,M,N,K", [("ag_gemm", 1024, 512, 256), ("gemm_rs", 1024, 512, 256), ("gemm_ar", 200, 520, 136)])
def test_every_fused_candidate_lowers_to_a_correct_launch(cuda_clean, world, op, M, N, K):
    # each schedule the selector can return, launched through the lowering on emulated ranks
    spec = lowering.TPLinearSpec(op, M, N, K, world)
    sel = lowering.select_schedule(spec)
    fused = [s for s in sel.schedules if s.fused]
    assert sel.schedule in fused and len(fused) >= 1
    g = symm.EmulatedGroup(world, 64 << 20, 16 << 20)
    try:
        rows = M // world if op == "ag_gemm" else M
        a = [_rand((rows, K), 1.0, 10 + r) for r in range(world)]
        b = [_rand((N, K), 0.02, 20 + r) for r in range(world)]
        fn = {"ag_gemm": oracle.all_gather_gemm, "gemm_rs": oracle.gemm_reduce_scatter, "gemm_ar": oracle.gemm_all_reduce}[op]
        want = fn([t.float().numpy() for t in a], [t.float().numpy() for t in b])
        a_d, b_d = [t.cuda() for t in a], [t.cuda() for t in b]
        if op == "gemm_ar":
            outs = [ctx.empty((M, N), torch.bfloat16) for ctx in g.ranks]
        else:
            outs = [torch.empty(M // world if op == "gemm_rs" else M, N, dtype=torch.bfloat16, device="cuda") for _ in range(world)]
        for sched in fused:
            torch.cuda.synchronize()
            g.poison()
            for o in outs:
                o.fill_(float("nan"))
            lowering.lower_emulated(spec, g, sched)(a_d, b_d, outs)
            torch.cuda.synchronize()
            for r in range(world):
                assert oracle.rel_l2(outs[r].float().cpu().numpy(), want[r]) <= 1e-2, (sched.label(), r)
        with pytest.raises(ValueError):
            lowering.lower_emulated(spec, g, sel.schedules[0])   # the unfused baseline
    finally:
        torch.cuda.synchronize()
        g.close()
