"""Schedule selector: which chunking / overlap to run a tensor-parallel linear with.

A *candidate* is "split the layer into c chunks, chunk i of the GEMM feeding (or fed by) chunk i
of the collective".  ``c == 1`` is the unfused schedule (GEMM, then the collective); ``c > 1``
overlaps.  Each candidate is a small EDM graph (built here with ``EDMBuilder`` so it can be
printed and analysed with the ordinary passes) and its cost is the critical path of that graph,
exactly as the reference's evaluator computes it (EDM-IR/ir/analysis.py:36-65).  The native
library evaluates the same graphs in int64 (``edm_select_schedule``); ``select`` calls it.

Durations come from the alpha-beta form of the reference's model (paper/mlsys-2027/model.md:98,
``T_comm = alpha + beta * m``) with the split costs of model.md:161-168, in integer nanoseconds,
from a calibration table measured on the B200 (``calibration.py``).
"""
from __future__ import annotations

import ctypes as C
from dataclasses import asdict, dataclass
from typing import Sequence

from . import _lib
from .ir import EDMBuilder, EDMGraph, MovementDesc
from .ir import ops as irops

DEFAULT_CANDIDATES = (1, 2, 4, 8)

_COMM_OP = {"gemm_rs": irops.COMM_REDUCE_SCATTER, "gemm_ar": irops.COMM_ALL_REDUCE,
            "ag_gemm": irops.COMM_ALL_GATHER}


@dataclass(frozen=True)
class CostParams:
    """Integer inputs of the cost model (any one time unit; nanoseconds by convention)."""

    gemm_total: int          # unchunked GEMM duration
    comm_bytes: int          # bytes per GPU per direction the unchunked collective moves
    alpha: int               # fixed cost per collective chunk
    beta_num: int            # transfer time = ceil(bytes * beta_num / beta_den)
    beta_den: int
    split_overhead: int      # added to every GEMM chunk when c > 1
    comm_first: int = 0      # 1: the collective feeds the GEMM (all-gather + GEMM)

    def to_c(self) -> "_lib.CostParams":
        return _lib.CostParams(self.gemm_total, self.comm_bytes, self.alpha, self.beta_num,
                               self.beta_den, self.split_overhead, self.comm_first, 0)


@dataclass(frozen=True)
class CandidateCost:
    chunks: int
    makespan: int
    exposed_comm: int
    total_comm: int
    gemm_chunk: int
    comm_chunk: int


def schedule_cost(params: CostParams, chunks: int) -> CandidateCost:
    out = _lib.CandidateCost()
    cp = params.to_c()
    _lib.check(_lib.load().edm_schedule_cost(C.byref(cp), chunks, C.byref(out)), "edm_schedule_cost")
    return CandidateCost(chunks, out.makespan, out.exposed_comm, out.total_comm, out.gemm_chunk,
                         out.comm_chunk)


def select(params: CostParams, candidates: Sequence[int] = DEFAULT_CANDIDATES):
    """Returns ``(chosen_index, [CandidateCost, ...])``; ties go to the lowest index."""
    n = len(candidates)
    if n == 0:
        raise ValueError("no candidates")
    cand = (C.c_int32 * n)(*candidates)
    costs = (_lib.CandidateCost * n)()
    chosen = C.c_int32(-1)
    cp = params.to_c()
    _lib.check(_lib.load().edm_select_schedule(C.byref(cp), cand, n, costs, C.byref(chosen)),
               "edm_select_schedule")
    return chosen.value, [CandidateCost(candidates[i], c.makespan, c.exposed_comm, c.total_comm,
                                        c.gemm_chunk, c.comm_chunk) for i, c in enumerate(costs)]


# ---------------------------------------------------------------- candidate graphs
def _share(total: int, c: int, i: int) -> int:
    return total // c + (1 if i < total % c else 0)


def candidate_graph(params: CostParams, chunks: int, op: str = "gemm_rs", *, world: int = 1,
                    tp_rank: int | None = None, schedule_index: int | None = None) -> EDMGraph:
    """The EDM graph of one candidate: ``phase.begin``, c ``compute.gemm`` nodes on stream
    "compute", c ``comm.*`` nodes on stream "comm", ``phase.end``; GEMM chain and collective
    chain in stream order, one data dependency per chunk, everything bound to the phase.
    Node and edge creation order is part of the cost model (it decides ties)."""
    c = chunks
    p = params
    gemm_d = [_share(p.gemm_total, c, i) + (p.split_overhead if c > 1 else 0) for i in range(c)]
    byts = [_share(p.comm_bytes, c, i) for i in range(c)]
    comm_d = [p.alpha + -(-(b * p.beta_num) // p.beta_den) for b in byts]

    g_span, m_span = [], []
    g_end = m_end = 0
    for i in range(c):
        if p.comm_first:
            m0 = m_end; m_end = m0 + comm_d[i]
            g0 = max(g_end, m_end); g_end = g0 + gemm_d[i]
        else:
            g0 = g_end; g_end = g0 + gemm_d[i]
            m0 = max(g_end, m_end); m_end = m0 + comm_d[i]
        g_span.append((g0, g0 + gemm_d[i]))
        m_span.append((m0, m0 + comm_d[i]))

    b = EDMBuilder(default_phase="tp_linear")
    begin = b.phase_begin("tp_linear", 0)
    common = {"tp_rank": tp_rank}
    gemms = [b.compute(f"gemm.{i}", *g_span[i], op=irops.COMPUTE_GEMM, stream="compute",
                       attrs={"chunk": i, "schedule_index": schedule_index}, **common)
             for i in range(c)]
    comms = [b.comm(f"{op}.{i}", *m_span[i], op=_COMM_OP[op], stream="comm",
                    movement=MovementDesc(kind=_COMM_OP[op].split(".", 1)[1], backend="nvlink-p2p",
                                          size_bytes=byts[i], group="tp",
                                          group_ranks=tuple(range(world))),
                    attrs={"chunk": i, "schedule_index": schedule_index}, **common)
             for i in range(c)]
    end = b.phase_end("tp_linear", max(g_end, m_end))
    b.sequence(*gemms, kind=irops.STREAM_ORDER)
    b.sequence(*comms, kind=irops.STREAM_ORDER)
    for i in range(c):
        if p.comm_first:
            b.data_edge(comms[i], gemms[i], f"chunk{i}")
        else:
            b.data_edge(gemms[i], comms[i], f"chunk{i}")
    b.bind_phase(begin, end, *gemms, *comms)
    return b.build()


def describe(params: CostParams) -> dict:
    return asdict(params)
