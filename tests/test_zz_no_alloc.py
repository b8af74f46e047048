"""The allocation-free fp32 GEMM entry point (``edm_gemm_fp32_static``) must agree with the
ordinary one (``edm_gemm_fp32``).

It exists for callers that cannot allocate device memory or pass a workspace where they need the
product; its scratch is a fixed array inside the library that every call shares and that keeps
the previous call's contents.  So the check runs two calls in a row with different shapes and
data: the second one would pick up stale scratch if the entry point relied on anything it did not
rewrite itself.  Both entry points are called through the C ABI.  This file is named to be
collected last, so a run that stops at the first failure has already covered everything else.
"""
import pytest
import torch

from edmir_b200 import _lib, linear
from oracle import tp_linear as oracle

pytestmark = pytest.mark.gpu

FP32_TOL = 1e-5


def _rand(shape, seed):
    g = torch.Generator(device="cpu").manual_seed(seed)
    return torch.randn(*shape, generator=g, dtype=torch.float32)


def test_static_scratch_gemm_matches_workspace_gemm_twice(cuda_clean):
    # (M, N, K): the CPU-runnable reference configuration first, then a ragged shape whose K needs
    # several accumulation segments (running sums in the shared scratch) and whose operands
    # overlay the first call's leftovers differently
    for call, (M, N, K) in enumerate([(256, 1024, 512), (300, 264, 1100)]):
        a = _rand((M, K), 40 + call).cuda()
        b = _rand((N, K), 50 + call).cuda()
        want = linear.gemm_fp32(a, b)
        got = torch.full((M, N), float("nan"), dtype=torch.float32, device="cuda")
        linear.gemm_fp32_static(a, b, got)
        torch.cuda.synchronize()
        assert oracle.rel_l2(got.cpu().numpy(), want.cpu().numpy()) <= FP32_TOL, (call, M, N, K)
        assert oracle.rel_l2(got.cpu().numpy(), oracle.gemm(a.cpu().numpy(), b.cpu().numpy())) <= FP32_TOL


def test_static_scratch_gemm_rejects_oversize(cuda_clean):
    # 8 * (M*K + N*K) = 16 MiB > the 8 MiB the built-in scratch gives to operand copies
    a = torch.zeros(1024, 1024, dtype=torch.float32, device="cuda")
    b = torch.zeros(1024, 1024, dtype=torch.float32, device="cuda")
    out = torch.zeros(1024, 1024, dtype=torch.float32, device="cuda")
    with pytest.raises(_lib.EdmError) as err:
        linear.gemm_fp32_static(a, b, out)
    assert err.value.code == _lib.EDM_ERR_CAPACITY
