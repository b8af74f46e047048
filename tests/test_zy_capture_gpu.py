"""Fused launches refuse stream capture (their exchange flags carry a per-call counter kept on the
host, which a graph replay would repeat) and leave the context usable."""
import pytest
import torch

from edmir_b200 import symm

pytestmark = pytest.mark.gpu


def test_fused_launch_on_a_capturing_stream_is_refused(cuda_clean):
    g = symm.EmulatedGroup(2, 32 << 20, 1 << 20)
    try:
        a = [torch.ones(256, 64, dtype=torch.bfloat16, device="cuda") for _ in range(2)]
        b = [torch.ones(256, 64, dtype=torch.bfloat16, device="cuda") for _ in range(2)]
        out = [torch.zeros(128, 256, dtype=torch.bfloat16, device="cuda") for _ in range(2)]
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        graph = torch.cuda.CUDAGraph()
        with pytest.raises(ValueError):
            with torch.cuda.stream(side):
                with torch.cuda.graph(graph, stream=side):
                    g.run("gemm_rs", a, b, out)
        torch.cuda.synchronize()
        g.run("gemm_rs", a, b, out)      # outside capture the same call goes through
        torch.cuda.synchronize()
        assert torch.all(out[0] == 128.0) and torch.all(out[1] == 128.0)   # 2 ranks x K=64 ones
    finally:
        g.close()
