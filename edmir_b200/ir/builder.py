"""EDMBuilder: a small DSL for trace-shaped graphs.

Mirrors the reference builder (EDM-IR/ir/builder.py:22-110): ids are handed out from 0 in
creation order, ``default_phase`` fills ``phase`` unless given, ``comm``/``movement`` default
their op to ``comm.all_gather`` (so callers should pass ``op=``), ``bind_phase`` adds
``begin -> body`` and ``body -> end`` phase-boundary edges per body node in argument order.
The schedule selector's candidate graphs are built with this class, so edge insertion order
here is part of the cost model's tie-breaking contract.
"""
from __future__ import annotations

from typing import Any

from . import ops
from .graph import EDMGraph
from .uop import DataRef, MovementDesc, TensorDesc, UOp


class EDMBuilder:
    def __init__(self, default_phase: str | None = None) -> None:
        self.graph = EDMGraph()
        self.default_phase = default_phase
        self._next_id = 0

    # ------------------------------------------------------------ nodes
    def uop(self, op: ops.OpKind, name: str, start_us: float, end_us: float, **kwargs: Any) -> UOp:
        if "phase" not in kwargs:
            kwargs["phase"] = self.default_phase
        node = UOp(id=self._next_id, op=op, name=name, start_us=start_us, end_us=end_us, **kwargs)
        self._next_id += 1  # only consumed when construction succeeded
        return self.graph.add_uop(node)

    def phase_begin(self, phase: str, start_us: float = 0.0) -> UOp:
        return self.uop(ops.PHASE_BEGIN, phase, start_us, start_us, phase=phase)

    def phase_end(self, phase: str, end_us: float) -> UOp:
        return self.uop(ops.PHASE_END, phase, end_us, end_us, phase=phase)

    def compute(self, name: str, start_us: float, end_us: float,
                op: ops.OpKind = ops.COMPUTE_OTHER, **kwargs: Any) -> UOp:
        return self.uop(op, name, start_us, end_us, **kwargs)

    def movement(self, name: str, start_us: float, end_us: float,
                 op: ops.OpKind = ops.COMM_ALL_GATHER, movement: MovementDesc | None = None,
                 **kwargs: Any) -> UOp:
        return self.uop(op, name, start_us, end_us, movement=movement, **kwargs)

    def comm(self, name: str, start_us: float, end_us: float,
             op: ops.OpKind = ops.COMM_ALL_GATHER, movement: MovementDesc | None = None,
             **kwargs: Any) -> UOp:
        return self.movement(name, start_us, end_us, op=op, movement=movement, **kwargs)

    def record_event(self, name: str, ts_us: float, **kwargs: Any) -> UOp:
        return self.uop(ops.EVENT_RECORD, name, ts_us, ts_us, **kwargs)

    def wait_event(self, name: str, start_us: float, end_us: float | None = None, **kwargs: Any) -> UOp:
        stop = start_us if end_us is None else end_us
        return self.uop(ops.EVENT_WAIT, name, start_us, stop, **kwargs)

    # ------------------------------------------------------------ edges
    def edge(self, src: UOp, dst: UOp, kind: ops.EdgeKind, **attrs: Any) -> None:
        self.graph.add_edge(src.id, dst.id, kind, **attrs)

    def sequence(self, *uops: UOp, kind: ops.EdgeKind = ops.STREAM_ORDER, **attrs: Any) -> None:
        for i in range(len(uops) - 1):
            self.edge(uops[i], uops[i + 1], kind, **attrs)

    def bind_phase(self, begin: UOp, end: UOp, *body: UOp) -> None:
        for node in body:
            self.edge(begin, node, ops.PHASE_BOUNDARY)
            self.edge(node, end, ops.PHASE_BOUNDARY)

    def data_edge(self, src: UOp, dst: UOp, data_id: str) -> None:
        self.edge(src, dst, ops.DATA_DEPENDENCY, data_id=data_id)

    def build(self) -> EDMGraph:
        return self.graph


__all__ = ["DataRef", "EDMBuilder", "MovementDesc", "TensorDesc"]
