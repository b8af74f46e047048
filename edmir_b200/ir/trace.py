"""Overlap probe: a real host-to-device copy, an event wait and a GEMM, reported as EDM UOps.

Same entry point, arguments and output as the reference probe (EDM-IR/ir/trace.py:55-119 driver,
:122-172 one measured iteration, :204-266 graph, :269-297 command line): the activation travels
from pinned host memory on a copy stream, the compute stream waits for the copy's event and
multiplies, three CUDA-event intervals are measured under ``edm.<ns>:<name>.iter<N>`` NVTX
ranges, and each iteration becomes a six-node graph (phase markers, copy, event record, event
wait, GEMM).  What differs is the multiply: it is this package's sm_100a kernel (bf16 with fp32
accumulation, or the split-tf32 fp32 path) instead of ``torch.matmul``, so the probe measures
the operator the rest of the package launches.  ``--dtype float16`` is accepted for command-line
compatibility and runs the bf16 kernel on bf16 data (the kernel has no fp16 variant); the
printed dtype says so.

    python -m edmir_b200.ir.trace --matrix 2048 --iters 3 --dtype bfloat16
"""
from __future__ import annotations

import argparse
from contextlib import contextmanager
from dataclasses import dataclass
from typing import Any, Sequence

from . import ops
from .builder import EDMBuilder
from .device import detect_device, format_device_spec
from .printing import format_critical_path, format_summary, format_uops
from .uop import MovementDesc, buffer_ref, param_ref

DTYPES = ("float16", "bfloat16", "float32")


def _load_torch() -> Any | None:
    try:
        import torch
    except Exception as exc:  # pragma: no cover - torch is a hard dependency of the operators
        print(f"torch unavailable: {exc}")
        return None
    return torch


@contextmanager
def nvtx_range(torch: Any, name: str):
    """Push/pop one NVTX range; names follow ``edm.<ns>:<name>.iter<N>`` so the reference's
    profiler import (EDM-IR/ir/nsys_export.py:74-88) maps them back to op names."""
    torch.cuda.nvtx.range_push(name)
    try:
        yield
    finally:
        try:
            torch.cuda.nvtx.range_pop()
        except Exception:
            pass


@dataclass(frozen=True, slots=True)
class TraceSample:
    iteration: int
    copy_us: float
    wait_us: float
    compute_us: float
    bytes_moved: int


class _Interval:
    """Two timing events recorded on one stream."""

    def __init__(self, torch: Any, stream: Any):
        self.stream = stream
        self.begin = torch.cuda.Event(enable_timing=True)
        self.end = torch.cuda.Event(enable_timing=True)

    def __enter__(self):
        self.begin.record(self.stream)
        return self

    def __exit__(self, *exc):
        self.end.record(self.stream)
        return False

    def us(self) -> float:
        return float(self.begin.elapsed_time(self.end)) * 1e3


def _multiply(torch: Any, a_gpu: Any, b_gpu: Any) -> Any:
    """``a @ b^T`` on the package's kernel (both operands K-major, EDM-IR/ir/c-extension/mma.cu:24-25)."""
    from .. import linear

    if a_gpu.dtype == torch.float32:
        return linear.gemm_fp32(a_gpu, b_gpu)
    return linear.gemm(a_gpu, b_gpu)


def run_iteration(*, torch: Any, iteration: int, a_cpu: Any, a_gpu: Any, b_gpu: Any, copy_stream: Any,
                  compute_stream: Any) -> TraceSample:
    """One measured copy -> wait -> GEMM pass (EDM-IR/ir/trace.py:122-172)."""
    copy_done = torch.cuda.Event()
    copy_t = _Interval(torch, copy_stream)
    wait_t = _Interval(torch, compute_stream)
    gemm_t = _Interval(torch, compute_stream)
    tag = f"iter{iteration}"
    result = None
    with nvtx_range(torch, f"edm.phase:trace.{tag}"):
        with torch.cuda.stream(copy_stream), nvtx_range(torch, f"edm.kv:transfer.h2d.{tag}"), copy_t:
            a_gpu.copy_(a_cpu, non_blocking=True)
            copy_done.record(copy_stream)
        with torch.cuda.stream(compute_stream):
            with nvtx_range(torch, f"edm.event:wait.copy_done.{tag}"), wait_t:
                compute_stream.wait_event(copy_done)
            with nvtx_range(torch, f"edm.compute:qkv.matmul.{tag}"), gemm_t:
                result = _multiply(torch, a_gpu, b_gpu)
    gemm_t.end.synchronize()
    if result is None:
        raise RuntimeError("trace workload did not produce a result")
    return TraceSample(iteration=iteration, copy_us=copy_t.us(), wait_us=wait_t.us(), compute_us=gemm_t.us(),
                       bytes_moved=a_cpu.numel() * a_cpu.element_size())


def build_graph(*, copy_us: float, compute_us: float, bytes_moved: int, device: str, matrix: int, dtype: str,
                wait_us: float, iteration: int):
    """The three measured intervals laid end to end as a six-node EDM graph
    (EDM-IR/ir/trace.py:204-266: same node names, ops, streams and edges)."""
    phase = f"trace.iter{iteration}"
    t_copy = copy_us
    t_wait = t_copy + wait_us
    t_done = t_wait + compute_us
    where = {"device": device}
    tags = {"matrix": matrix, "dtype": dtype, "iteration": iteration}

    b = EDMBuilder(default_phase=phase)
    begin = b.phase_begin(phase, 0.0)
    copy = b.movement("h2d_activation_copy", 0.0, t_copy, op=ops.MOVEMENT_COPY, stream="copy",
                      movement=MovementDesc(kind="h2d_copy", backend="cuda", size_bytes=bytes_moved),
                      reads=(buffer_ref("host_activation"),),
                      writes=(buffer_ref("device_activation", "write", location=device),), attrs=dict(tags), **where)
    record = b.record_event("copy_done", t_copy, stream="copy", **where)
    wait = b.wait_event("wait_copy_done", t_copy, t_wait, stream="compute",
                        attrs={"measured_wait_us": wait_us, "iteration": iteration}, **where)
    gemm = b.compute("qkv_matmul", t_wait, t_done, op=ops.COMPUTE_QKV, stream="compute",
                     reads=(buffer_ref("device_activation", location=device),
                            param_ref("qkv_weight", location=device)),
                     writes=(buffer_ref("qkv_output", "write", location=device),), attrs=dict(tags), **where)
    end = b.phase_end(phase, t_done)

    b.sequence(begin, copy, record, kind=ops.STREAM_ORDER)
    b.edge(record, wait, ops.EVENT_DEPENDENCY, event="copy_done")
    b.edge(copy, gemm, ops.DATA_DEPENDENCY, data_id="device_activation")
    b.sequence(wait, gemm, end, kind=ops.STREAM_ORDER)
    return b.build()


def print_timing_table(samples: Sequence[TraceSample]) -> None:
    print("\n== raw CUDA timing ==")
    print("iter  h2d_copy_us  event_wait_us  matmul_us  copy_bytes")
    for s in samples:
        print(f"{s.iteration:>4}  {s.copy_us:>11.3f}  {s.wait_us:>13.3f}  {s.compute_us:>9.3f}  {s.bytes_moved}")


def print_selected_uops(graphs: Sequence[Any], mode: str) -> None:
    if mode == "none" or not graphs:
        return
    chosen = [len(graphs) - 1] if mode == "last" else range(len(graphs))
    for i in chosen:
        graph = graphs[i]
        path, _ = graph.critical_path()
        print(f"\n== EDM UOps iter={i} ==")
        print(format_uops(graph, highlight=path))
        print(format_critical_path(graph))
        print(format_summary(graph))


def run_trace(matrix: int, warmup: int, iters: int, dtype_name: str, print_uops: str) -> list:
    """Warm up, run ``iters`` measured iterations on ``cuda:0``, print the timing table and the
    selected graphs (EDM-IR/ir/trace.py:55-119).  Returns the graphs (the reference returns
    nothing; callers that only want the printout can ignore it)."""
    torch = _load_torch()
    if torch is None:
        return []
    if not torch.cuda.is_available():
        print("CUDA unavailable; trace.py requires a CUDA device for real ops.")
        print(format_device_spec(detect_device(0)))
        return []
    if dtype_name not in DTYPES:
        raise ValueError(f"dtype must be one of {DTYPES}")
    run_dtype = "bfloat16" if dtype_name == "float16" else dtype_name
    if run_dtype != dtype_name:
        print("note: float16 requested; the sm_100a kernel computes bf16 x bf16 -> fp32, running bfloat16")
    dtype = getattr(torch, run_dtype)

    spec = detect_device(0)
    device_label = "cuda:0" + (f"/{spec.cuda_arch}" if spec is not None and spec.cuda_arch else "")
    print("== device ==")
    print(format_device_spec(spec))

    torch.cuda.set_device(0)
    copy_stream, compute_stream = torch.cuda.Stream(), torch.cuda.Stream()
    a_cpu = torch.randn((matrix, matrix), dtype=torch.float32).to(dtype).pin_memory()
    a_gpu = torch.empty((matrix, matrix), dtype=dtype, device="cuda")
    b_gpu = torch.randn((matrix, matrix), dtype=torch.float32, device="cuda").to(dtype)
    for _ in range(warmup):
        a_gpu.copy_(a_cpu, non_blocking=True)
        _multiply(torch, a_gpu, b_gpu)
    torch.cuda.synchronize()

    samples, graphs = [], []
    for it in range(iters):
        s = run_iteration(torch=torch, iteration=it, a_cpu=a_cpu, a_gpu=a_gpu, b_gpu=b_gpu,
                          copy_stream=copy_stream, compute_stream=compute_stream)
        samples.append(s)
        graphs.append(build_graph(copy_us=s.copy_us, compute_us=s.compute_us, bytes_moved=s.bytes_moved,
                                  device=device_label, matrix=matrix, dtype=run_dtype, wait_us=s.wait_us,
                                  iteration=it))
    print_timing_table(samples)
    print_selected_uops(graphs, print_uops)
    return graphs


def parse_args(argv: Sequence[str] | None = None) -> argparse.Namespace:
    p = argparse.ArgumentParser(description="Run a real CUDA op and print EDM-IR UOps.")
    p.add_argument("--matrix", type=int, default=2048, help="square matrix size for H2D copy and matmul")
    p.add_argument("--warmup", type=int, default=2, help="warmup iterations before measured trace")
    p.add_argument("--iters", type=int, default=1, help="measured iterations to record after warmup")
    p.add_argument("--dtype", choices=DTYPES, default="float16", help="tensor dtype for the trace workload")
    p.add_argument("--print-uops", choices=("last", "all", "none"), default="last",
                   help="which measured iterations should print EDM UOps")
    return p.parse_args(argv)


def main(argv: Sequence[str] | None = None) -> None:
    args = parse_args(argv)
    if args.iters < 1:
        raise SystemExit("--iters must be >= 1")
    run_trace(matrix=args.matrix, warmup=args.warmup, iters=args.iters, dtype_name=args.dtype,
              print_uops=args.print_uops)


if __name__ == "__main__":
    main()
