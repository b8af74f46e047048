"""Parity of the sm_100a GEMM (called through the C ABI) against the CPU oracle.

Tolerances are the ones the path is specified with: rel-L2 <= 1e-2 for bf16 (fp32
accumulation), <= 1e-5 for fp32.  Exact properties (selection matrices, repeatability) are
checked bit for bit, including at the full benchmark sizes where the oracle would be too slow.
"""
import numpy as np
import pytest
import torch

from edmir_b200 import linear
from oracle import tp_linear as oracle

pytestmark = pytest.mark.gpu

BF16_TOL = 1e-2
FP32_TOL = 1e-5


def _rand(shape, scale, dtype, seed):
    g = torch.Generator(device="cpu").manual_seed(seed)
    return (torch.randn(*shape, generator=g, dtype=torch.float32) * scale).to(dtype)


@pytest.mark.parametrize("M,N,K", [
    (128, 256, 64), (128, 256, 512), (256, 512, 128),      # whole tiles
    (1, 4096, 1792), (16, 4096, 1792), (128, 4096, 1792),  # decode-sized rows
    (1000, 768, 520), (130, 264, 72), (8, 8, 8),           # ragged M, N, K edges
    (5, 1000, 264), (128, 40, 4096),                       # narrow (128x32) tiles with a ragged last tile
    (1024, 4096, 3584),
    (2560, 2048, 8192), (2500, 2000, 4104),                # 80 tiles on 74 CTA pairs: last wave cut in 8 along K
    (200, 20480, 2048),                                    # 160 tiles on 148 CTAs: last wave cut in 8
    (128, 4096, 7168), (16, 4096, 14336), (1, 4096, 7168),  # decode: 16 wide tiles cut in 8 along K
    (100, 520, 4104), (64, 8192, 3584),                    # ragged pieces; 32 tiles cut in 4
])
def test_gemm_bf16_matches_oracle(cuda_clean, M, N, K):
    a = _rand((M, K), 1.0, torch.bfloat16, 1)
    b = _rand((N, K), 0.02, torch.bfloat16, 2)
    out = linear.gemm(a.cuda(), b.cuda())
    want = oracle.gemm(a.float().numpy(), b.float().numpy())
    assert oracle.rel_l2(out.float().cpu().numpy(), want) <= BF16_TOL


@pytest.mark.parametrize("M", [1, 7, 16, 32, 33, 64, 65, 100, 128])
@pytest.mark.parametrize("N,K", [(4096, 1792), (520, 264), (4096, 14336), (128, 64), (17920, 512), (1024, 8192),
                                 (136, 8)])
def test_decode_kernel_matches_oracle(cuda_clean, M, N, K):
    # up to 64 tokens: weights on the MMA's M side, a cluster of CTAs per 128-column tile cutting K;
    # 65 to 128 rows (general kernel: narrow tiles or wide pieces) run the same checks.
    # Strided tokens, ragged N and K, a row stride wider than the output, and guard rows around it.
    a_wide = _rand((M, K + 24), 1.0, torch.bfloat16, 11).cuda()
    a = a_wide[:, :K]
    b = _rand((N, K), 0.02, torch.bfloat16, 12).cuda()
    guard = torch.full((M + 2, N + 8), 5.0, dtype=torch.bfloat16, device="cuda")
    out = guard[1:M + 1, :N]
    first = None
    for _ in range(3):
        linear.gemm(a, b, out)
        torch.cuda.synchronize()
        first = out.clone() if first is None else first
        assert torch.equal(out, first)          # fixed summation order: repeatable bit for bit
    want = oracle.gemm(a.float().cpu().numpy(), b.float().cpu().numpy())
    assert oracle.rel_l2(out.float().cpu().numpy(), want) <= BF16_TOL
    assert torch.all(guard[0] == 5.0) and torch.all(guard[M + 1] == 5.0) and torch.all(guard[:, N:] == 5.0)
    assert linear.status()[0] == 0


@pytest.mark.parametrize("M,N,K", [(256, 1024, 512), (300, 520, 260), (4, 4, 4), (128, 256, 2048)])
def test_gemm_fp32_matches_oracle(cuda_clean, M, N, K):
    a = _rand((M, K), 1.0, torch.float32, 3)
    b = _rand((N, K), 1.0, torch.float32, 4)
    out = linear.gemm_fp32(a.cuda(), b.cuda())
    want = oracle.gemm(a.numpy(), b.numpy())
    assert oracle.rel_l2(out.cpu().numpy(), want) <= FP32_TOL


def test_config1_single_rank_pieces(cuda_clean):
    # the CPU-runnable reference configuration, one rank at a time: A_r[256,512] @ B_r[512,1024]
    a_sh, b_sh = oracle.config1_inputs()
    total = None
    for a, b in zip(a_sh, b_sh):
        part = linear.gemm_fp32(torch.from_numpy(a).cuda(), torch.from_numpy(np.ascontiguousarray(b.T)).cuda())
        total = part if total is None else total + part
    assert oracle.rel_l2(total.cpu().numpy(), oracle.config1_output(a_sh, b_sh)) <= FP32_TOL


def test_strided_operands_and_output(cuda_clean):
    M, N, K = 200, 520, 136
    a_full = _rand((M, K + 24), 1.0, torch.bfloat16, 5).cuda()
    b_full = _rand((N, K + 8), 0.02, torch.bfloat16, 6).cuda()
    out_full = torch.zeros(M, N + 16, dtype=torch.bfloat16, device="cuda")
    a, b, out = a_full[:, :K], b_full[:, :K], out_full[:, :N]
    linear.gemm(a, b, out)
    want = oracle.gemm(a.float().cpu().numpy(), b.float().cpu().numpy())
    assert oracle.rel_l2(out.float().cpu().numpy(), want) <= BF16_TOL
    assert torch.count_nonzero(out_full[:, N:]) == 0  # nothing written past N


@pytest.mark.parametrize("M,N,K", [(8192, 8192, 3584), (8192, 1280, 8192)])
def test_selection_matrix_is_bit_exact_at_full_size(cuda_clean, M, N, K):
    # rows of A are one-hot, so D[m, n] must equal B[n, k(m)] exactly; full down_proj extents, and
    # the qkv extents whose last wave of tiles is cut along K (partial sums of 0 and one value)
    g = torch.Generator(device="cpu").manual_seed(7)
    pick = torch.randint(0, K, (M,), generator=g)
    a = torch.zeros(M, K, dtype=torch.bfloat16)
    a[torch.arange(M), pick] = 1.0
    b = _rand((N, K), 0.02, torch.bfloat16, 8)
    out = linear.gemm(a.cuda(), b.cuda())
    want = b.cuda()[:, pick.cuda()].t().contiguous()
    assert torch.equal(out, want)


def test_captured_launches_replay_with_new_inputs(cuda_clean):
    # A shape that eager launches cut along K.  Captured launches must not rely on per-launch
    # values from the host (a replay repeats them): every replay has to give the product of what
    # is in the operand buffers at that moment.
    a = _rand((64, 7168), 1.0, torch.bfloat16, 21).cuda()
    b = _rand((4096, 7168), 0.02, torch.bfloat16, 22).cuda()
    out = torch.zeros(64, 4096, dtype=torch.bfloat16, device="cuda")
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        linear.gemm(a, b, out)          # first use of the variants outside capture
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=side):
            for _ in range(2):
                linear.gemm(a, b, out)
        for step in range(3):
            a.copy_(_rand((64, 7168), 1.0, torch.bfloat16, 30 + step).cuda())
            out.zero_()
            graph.replay()
            side.synchronize()
            want = oracle.gemm(a.float().cpu().numpy(), b.float().cpu().numpy())
            assert oracle.rel_l2(out.float().cpu().numpy(), want) <= BF16_TOL, step
    torch.cuda.current_stream().wait_stream(side)
    eager = linear.gemm(a, b)           # eager launches (cut along K) still work afterwards
    assert oracle.rel_l2(eager.float().cpu().numpy(), want) <= BF16_TOL


def test_repeatable_bit_for_bit(cuda_clean):
    a = _rand((2048, 1024), 1.0, torch.bfloat16, 9).cuda()
    b = _rand((2048, 1024), 0.02, torch.bfloat16, 10).cuda()
    first = linear.gemm(a, b).clone()
    for _ in range(3):
        assert torch.equal(linear.gemm(a, b), first)


def test_reference_operator_shim(cuda_clean):
    # the reference's only operator: bf16(A[32,16] @ B[32,16]^T (+ C)), EDM-IR/ir/c-extension/mma.cu:267-271
    a = _rand((32, 16), 1.0, torch.bfloat16, 11).cuda()
    b = _rand((32, 16), 1.0, torch.bfloat16, 12).cuda()
    c = _rand((32, 32), 1.0, torch.float32, 13).cuda()
    want = a.float() @ b.float().t()
    got = linear.tiled_mma_bf16_bf16_bf16_fp32(a, b)
    assert got.dtype == torch.bfloat16 and oracle.rel_l2(got.float().cpu().numpy(), want.cpu().numpy()) <= BF16_TOL
    got_c = linear.tiled_mma_bf16_bf16_bf16_fp32(a, b, c)
    assert oracle.rel_l2(got_c.float().cpu().numpy(), (want + c).cpu().numpy()) <= BF16_TOL


def test_bad_arguments_raise(cuda_clean):
    a = torch.zeros(8, 8, dtype=torch.bfloat16, device="cuda")
    with pytest.raises(ValueError):
        linear.gemm(a, torch.zeros(8, 16, dtype=torch.bfloat16, device="cuda"))   # K mismatch
    with pytest.raises(ValueError):
        linear.gemm(a.float(), a.float())                                        # wrong dtype
    with pytest.raises(ValueError):
        linear.gemm(a.cpu(), a.cpu())                                            # no CPU path
    with pytest.raises(ValueError):
        linear.gemm(a[:, :4], a[:, :4])                                          # K not a multiple of 8
