"""Lowering of a tensor-parallel linear layer: spec -> schedule candidates (EDM graphs) ->
selected schedule -> launch -> measured UOps.

The reference has no lowering ("EDM-IR represents observed execution", paper/mlsys-2027/
edm-ir.md:7); what it does have, and what this module keeps, is the node API the result is
reported in (``UOp``/``MovementDesc``/``EDMBuilder``, EDM-IR/ir/uop.py:44-142, builder.py:22-110),
the analysis that scores candidates (analysis.py:36-65) and the way a measured run is turned
into a graph (CUDA-event timing and ``edm.<ns>:<name>.iter<N>`` NVTX ranges,
EDM-IR/ir/trace.py:26-43, :122-172, :204-266).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, Sequence

from . import selector
from .calibration import Calibration, cost_params, wire_bytes
from .ir import EDMBuilder, EDMGraph, MovementDesc, TensorDesc
from .ir import ops as irops

OPS = ("gemm_rs", "gemm_ar", "ag_gemm")
_COMM_OP = {"gemm_rs": irops.COMM_REDUCE_SCATTER, "gemm_ar": irops.COMM_ALL_REDUCE,
            "ag_gemm": irops.COMM_ALL_GATHER}


@dataclass(frozen=True)
class TPLinearSpec:
    """One tensor-parallel linear call.  ``M, N, K`` are the per-rank GEMM extents
    (``ag_gemm``: M counts gathered rows)."""

    op: str
    M: int
    N: int
    K: int
    world: int
    dtype: str = "bf16"

    def __post_init__(self) -> None:
        if self.op not in OPS:
            raise ValueError(f"unknown tensor-parallel op: {self.op}")
        if min(self.M, self.N, self.K, self.world) < 1:
            raise ValueError("extents and world must be positive")
        if self.op != "gemm_ar" and self.M % self.world:
            raise ValueError("M must be divisible by the number of ranks")


@dataclass(frozen=True)
class Schedule:
    """A candidate: ``chunks == 1`` is the unfused sequence (GEMM kernel, then the collective);
    ``chunks > 1`` is the fused kernel with that exchange granularity."""

    index: int
    chunks: int

    @property
    def fused(self) -> bool:
        return self.chunks > 1


def candidates(spec: TPLinearSpec, chunk_counts: Sequence[int] = selector.DEFAULT_CANDIDATES) -> list[Schedule]:
    if spec.world == 1:
        return [Schedule(0, 1)]
    out = []
    for c in chunk_counts:
        if spec.op == "ag_gemm" and c > spec.M // spec.world:
            continue
        out.append(Schedule(len(out), c))
    return out


@dataclass(frozen=True)
class Selection:
    spec: TPLinearSpec
    schedules: list
    costs: list          # selector.CandidateCost per schedule
    chosen: int
    graphs: list         # candidate EDM graphs, same order

    @property
    def schedule(self) -> Schedule:
        return self.schedules[self.chosen]


def select_schedule(spec: TPLinearSpec, calib: Calibration | None = None,
                    chunk_counts: Sequence[int] = selector.DEFAULT_CANDIDATES, tp_rank: int | None = None) -> Selection:
    """Score every candidate with the native cost model and return the arg-min (ties: lowest
    index).  The unfused candidate is costed with the library collective's bandwidth, the fused
    ones with the in-kernel push bandwidth; each is one ``edm_schedule_cost`` evaluation."""
    calib = calib or Calibration.load()
    scheds = candidates(spec, chunk_counts)
    costs, graphs = [], []
    for s in scheds:
        p = cost_params(spec.op, spec.M, spec.N, spec.K, spec.world, calib, fused=s.fused)
        costs.append(selector.schedule_cost(p, s.chunks))
        graphs.append(selector.candidate_graph(p, s.chunks, spec.op if spec.world > 1 else "gemm_rs",
                                               world=spec.world, tp_rank=tp_rank, schedule_index=s.index))
    chosen = min(range(len(costs)), key=lambda i: (costs[i].makespan, i))
    return Selection(spec, scheds, costs, chosen, graphs)


# ---------------------------------------------------------------- launching
def lower(spec: TPLinearSpec, ctx, schedule: Schedule) -> Callable:
    """Returns ``fn(a, b, out) -> out`` running ``schedule`` for ``spec``.

    ``ctx`` is a ``symm.SymmetricContext`` (``None`` for a single rank).  The unfused schedule
    uses this library's GEMM followed by the ``torch.distributed`` collective; fused schedules
    are one launch of the fused kernel."""
    from . import linear

    if spec.world == 1 or ctx is None:
        return lambda a, b, out=None: linear.gemm(a, b, out)
    if schedule.fused:
        if spec.op == "ag_gemm":
            return lambda x, w, out=None: ctx.ag_gemm(x, w, out, chunks=schedule.chunks)
        if spec.op == "gemm_rs":
            return lambda a, b, out=None: ctx.gemm_rs(a, b, out)
        return lambda a, b, out=None: ctx.gemm_ar(a, b, out)

    import torch
    import torch.distributed as dist

    def unfused(a, b, out=None):
        if spec.op == "ag_gemm":
            full = torch.empty((spec.M, spec.K), dtype=a.dtype, device=a.device)
            dist.all_gather_into_tensor(full, a)
            return linear.gemm(full, b, out)
        part = linear.gemm(a, b)
        if spec.op == "gemm_rs":
            if out is None:
                out = torch.empty((spec.M // spec.world, spec.N), dtype=a.dtype, device=a.device)
            dist.reduce_scatter_tensor(out, part)
            return out
        dist.all_reduce(part)
        if out is not None:
            out.copy_(part)
            return out
        return part

    return unfused


def nvtx_name(namespace: str, name: str, iteration: int | None = None) -> str:
    """``edm.<ns>:<name>[.iter<N>]`` -- the range-name grammar the reference's profiler import
    parses (EDM-IR/ir/nsys_export.py:17, :74-88)."""
    base = f"edm.{namespace}:{name}"
    return base if iteration is None else f"{base}.iter{iteration}"


def measured_graph(spec: TPLinearSpec, schedule: Schedule, total_us: float, gemm_only_us: float,
                   tp_rank: int = 0, device: str | None = None, iteration: int | None = None) -> EDMGraph:
    """The observed execution of one call as an EDM graph: a ``compute.gemm`` node and a
    ``comm.*`` node inside a ``tp_linear`` phase.  For a fused launch both run over the same
    interval and the part of the collective that was not hidden is ``total - gemm_only``; that
    exposed tail is what ends up on the critical path (``analyze_exposure`` reports it as
    ``exposed_comm_us``).  For the unfused schedule the collective simply follows the GEMM."""
    exposed = max(total_us - gemm_only_us, 0.0)
    nbytes = wire_bytes(spec.op, spec.M, spec.N, spec.K, spec.world) if spec.world > 1 else 0
    b = EDMBuilder(default_phase="tp_linear")
    begin = b.phase_begin("tp_linear", 0.0)
    common = dict(tp_rank=tp_rank, device=device,
                  attrs={"schedule_index": schedule.index, "chunks": schedule.chunks, "fused": schedule.fused,
                         "M": spec.M, "N": spec.N, "K": spec.K})
    gemm = b.compute("gemm" if iteration is None else f"gemm.iter{iteration}", 0.0, gemm_only_us,
                     op=irops.COMPUTE_GEMM, stream="compute",
                     tensor=TensorDesc(name="out", shape=(spec.M, spec.N), dtype=spec.dtype), **common)
    nodes = [gemm]
    if spec.world > 1:
        comm = b.comm(spec.op if iteration is None else f"{spec.op}.iter{iteration}",
                      gemm_only_us, gemm_only_us + exposed, op=_COMM_OP[spec.op],
                      stream="nvlink" if schedule.fused else "nccl",
                      movement=MovementDesc(kind=_COMM_OP[spec.op].split(".", 1)[1],
                                            backend="nvlink-p2p" if schedule.fused else "nccl",
                                            size_bytes=nbytes, group="tp",
                                            group_ranks=tuple(range(spec.world))), **common)
        b.data_edge(gemm, comm, "partial" if spec.op != "ag_gemm" else "gathered")
        nodes.append(comm)
    end = b.phase_end("tp_linear", total_us)
    b.bind_phase(begin, end, *nodes)
    return b.build()


def run_measured(spec: TPLinearSpec, ctx, schedule: Schedule, a, b, out=None, iters: int = 10, warmup: int = 3,
                 gemm_only_us: float | None = None):
    """Runs the schedule ``iters`` times under NVTX ranges, times it with CUDA events on the
    current stream, and returns ``(out, graph, total_us)`` with the measured EDM graph."""
    import torch

    from . import linear

    fn = lower(spec, ctx, schedule)
    for _ in range(warmup):
        out = fn(a, b, out)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(iters):
        torch.cuda.nvtx.range_push(nvtx_name("compute" if not schedule.fused else "comm",
                                             f"tp_linear.{spec.op}", i))
        out = fn(a, b, out)
        torch.cuda.nvtx.range_pop()
    e1.record()
    torch.cuda.synchronize()
    total_us = e0.elapsed_time(e1) / iters * 1e3
    if gemm_only_us is None:
        # the same GEMM extents without any exchange, on this rank
        rows = spec.M
        ga = torch.empty((rows, spec.K), dtype=a.dtype, device=a.device).normal_()
        gout = torch.empty((rows, spec.N), dtype=a.dtype, device=a.device)
        for _ in range(warmup):
            linear.gemm(ga, b, gout)
        e0.record()
        for _ in range(iters):
            linear.gemm(ga, b, gout)
        e1.record()
        torch.cuda.synchronize()
        gemm_only_us = e0.elapsed_time(e1) / iters * 1e3
    rank = ctx.rank if ctx is not None else 0
    graph = measured_graph(spec, schedule, total_us, min(gemm_only_us, total_us), tp_rank=rank,
                           device=str(a.device))
    return out, graph, total_us
