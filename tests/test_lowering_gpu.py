"""The lowering's launch and measurement path on a GPU (single rank: the schedule degenerates to
the plain GEMM), and the device-side role accounting."""
import pytest
import torch

from edmir_b200 import linear, lowering
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
