"""Host-resident operands: uploads, kernels and downloads on three streams give the same results
as the one-stream sequence, also when device buffers are reused step after step."""
import pytest
import torch

from edmir_b200 import host_io, linear

pytestmark = pytest.mark.gpu


def _rand(shape, scale, seed):
    g = torch.Generator(device="cpu").manual_seed(seed)
    return (torch.randn(*shape, generator=g, dtype=torch.float32) * scale).to(torch.bfloat16)


def test_staged_steps_match_direct_launches(cuda_clean):
    shapes = [(1024, 512, 2048), (512, 1536, 1024), (2048, 256, 512)]   # M, N, K per linear
    weights = [_rand((n, k), 0.02, 10 + i).cuda() for i, (_, n, k) in enumerate(shapes)]
    a_dev = [torch.empty(m, k, dtype=torch.bfloat16, device="cuda") for m, _, k in shapes]
    out_dev = [torch.empty(m, n, dtype=torch.bfloat16, device="cuda") for m, n, _ in shapes]
    io = host_io.HostStaging()
    steps = 4
    # every step has its own host inputs and outputs, the device buffers are shared by all steps
    a_host = [[_rand((m, k), 1.0, 100 * s + i).pin_memory() for i, (m, _, k) in enumerate(shapes)]
              for s in range(steps)]
    out_host = [[torch.zeros(m, n, dtype=torch.bfloat16).pin_memory() for m, n, _ in shapes] for _ in range(steps)]
    for s in range(steps):
        for i in range(len(shapes)):
            io.run(a_host[s][i], a_dev[i], lambda i=i: linear.gemm(a_dev[i], weights[i], out_dev[i]),
                   out_dev[i], out_host[s][i])
        io.drain()
    torch.cuda.synchronize()
    for s in range(steps):
        for i in range(len(shapes)):
            want = linear.gemm(a_host[s][i].cuda(), weights[i])
            assert torch.equal(out_host[s][i].cuda(), want), (s, i)


def test_unpinned_buffers_are_refused(cuda_clean):
    io = host_io.HostStaging()
    a = torch.zeros(128, 64, dtype=torch.bfloat16)
    d = torch.zeros(128, 64, dtype=torch.bfloat16, device="cuda")
    with pytest.raises(ValueError):
        io.run(a, d, lambda: None, d, a)
