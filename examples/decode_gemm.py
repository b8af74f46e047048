"""Times decode-sized GEMMs (a few tokens against a weight matrix) on one GPU.

    python examples/decode_gemm.py [--n 4096] [--k 1792,3584,7168,14336] [--tokens 1,16,32,64,128] [--graph]
    EDM_DECODE=0 python examples/decode_gemm.py      # the same shapes through the general kernel

Default shapes: the Llama-3-8B-shaped down_proj (N = 4096) with K = 14336 / TP for TP = 8, 4, 2, 1.
Prints one JSON line per shape: microseconds per call in a loop of back-to-back launches (CUDA
events) that rotates over enough copies of the weights (>= 256 MB in total) that no launch finds
them in the 126 MB L2, what ``torch.matmul`` takes in the same loop, the launch plan, the fraction
of the HBM roofline (weights read once at the measured copy bandwidth) and the rel-L2 against an
fp32 matmul.  ``--graph`` also replays a CUDA graph of 24 captured launches (same rotation), which
takes the host's issue rate out of the figure (launches of up to 64 rows use no global scratch
and can be captured).
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from edmir_b200 import linear  # noqa: E402


def timed(fn, iters: int = 50, warm: int = 5) -> float:
    for _ in range(warm):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / iters * 1e3


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--n", type=int, default=4096)
    ap.add_argument("--k", default="1792,3584,7168,14336")
    ap.add_argument("--tokens", default="1,16,32,64,128")
    ap.add_argument("--graph", action="store_true")
    args = ap.parse_args()
    dev = torch.device("cuda", 0)
    hbm_gbs = 6546.0
    try:
        with open(os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "MEASURED_PEAKS.json")) as f:
            hbm_gbs = float(json.load(f)["hbm_gbs"])
    except Exception:
        pass
    N = args.n
    for K in (int(v) for v in args.k.split(",")):
        w = (torch.randn(N, K, device=dev) * 0.02).to(torch.bfloat16)
        ws = [w] + [w.clone() for _ in range(min(23, -(-(256 << 20) // (N * K * 2)) - 1))]
        turn = [0]

        def next_w():
            turn[0] = (turn[0] + 1) % len(ws)
            return ws[turn[0]]

        for M in (int(v) for v in args.tokens.split(",")):
            a = torch.randn(M, K, device=dev).to(torch.bfloat16)
            out = torch.empty(M, N, device=dev, dtype=torch.bfloat16)
            us = timed(lambda: linear.gemm(a, next_w(), out))
            lib = timed(lambda: torch.matmul(a, next_w().t(), out=out))
            graph_us = lib_graph_us = None
            if args.graph:
                def replayed(call):
                    side = torch.cuda.Stream()
                    side.wait_stream(torch.cuda.current_stream())
                    g = torch.cuda.CUDAGraph()
                    with torch.cuda.stream(side):
                        call()
                        torch.cuda.synchronize()
                        with torch.cuda.graph(g, stream=side):
                            for _ in range(24):
                                call()
                    torch.cuda.synchronize()
                    return timed(g.replay, iters=10, warm=2) / 24
                graph_us = round(replayed(lambda: linear.gemm(a, next_w(), out)), 1)
                lib_graph_us = round(replayed(lambda: torch.matmul(a, next_w().t(), out=out)), 1)
            linear.gemm(a, w, out)
            ref = torch.matmul(a.float(), w.float().t())
            err = float((out.float() - ref).norm() / ref.norm())
            roof_us = 2.0 * (M * K + N * K + M * N) / (hbm_gbs * 1e3)
            print(json.dumps({"tokens": M, "N": N, "K": K, "us": round(us, 1), "torch_matmul_us": round(lib, 1),
                              "graph_us": graph_us, "torch_matmul_graph_us": lib_graph_us, "weight_copies": len(ws), "plan": linear.gemm_plan(M, N, K), "hbm_roofline_us": round(roof_us, 1),
                              "roofline_frac": round(roof_us / us, 3), "rel_l2": float(f"{err:.2e}")}), flush=True)
    assert linear.status()[0] == 0, linear.status()[:8]


if __name__ == "__main__":
    main()
