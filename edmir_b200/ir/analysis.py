"""Analysis passes over an EDM graph: critical path, exposure ratios, overlap gain.

Same results and tie-breaking as the reference passes (EDM-IR/ir/analysis.py):
* ``analyze_critical_path`` (:36-65): longest path by summed ``dur_us``; a node's parent is
  the FIRST predecessor (edge-insertion order) with the maximal prefix; the path ends at the
  node maximising ``(prefix, end_us, id)``.
* ``phase_duration_us`` (:68-86): ``phase.begin``/``phase.end`` markers if both exist, else the
  min/max timestamps.
* exposure (:89-123): comm / data-movement time lying on the critical path over phase time.
* ``classify_gain`` (:139-149): > 5 % material, > 0 small, == 0 none, < 0 regression.
The graph argument is duck-typed (``uops``, ``topological_order()``, ``predecessors()``).
This is also the evaluator the native schedule selector is checked against.
"""
from __future__ import annotations

from dataclasses import dataclass

from .ops import is_comm, is_data_movement


@dataclass(frozen=True, slots=True)
class CriticalPathResult:
    path: tuple[int, ...]
    duration_us: float


@dataclass(frozen=True, slots=True)
class ExposureResult:
    phase_time_us: float
    critical_path_us: float
    total_comm_us: float
    exposed_comm_us: float
    total_data_movement_us: float
    exposed_data_movement_us: float
    ecr: float
    edmr: float
    critical_path: tuple[int, ...]


@dataclass(frozen=True, slots=True)
class OverlapGainResult:
    before_us: float
    after_us: float
    gain_us: float
    gain_ratio: float
    label: str


def analyze_critical_path(graph) -> CriticalPathResult:
    preds = graph.predecessors()
    prefix: dict[int, float] = {}
    came_from: dict[int, int | None] = {}
    for uid in graph.topological_order():
        dur = graph.uops[uid].dur_us
        incoming = preds.get(uid)
        if not incoming:
            prefix[uid], came_from[uid] = dur, None
            continue
        chosen = incoming[0]
        for cand in incoming[1:]:
            if prefix[cand] > prefix[chosen]:  # strict: earlier edge wins ties
                chosen = cand
        prefix[uid], came_from[uid] = prefix[chosen] + dur, chosen

    if not prefix:
        return CriticalPathResult(path=(), duration_us=0.0)

    last = max(prefix, key=lambda u: (prefix[u], graph.uops[u].end_us, u))
    chain: list[int] = []
    node: int | None = last
    while node is not None:
        chain.append(node)
        node = came_from[node]
    return CriticalPathResult(path=tuple(reversed(chain)), duration_us=prefix[last])


def phase_duration_us(graph) -> float:
    nodes = list(graph.uops.values())
    if not nodes:
        return 0.0
    begins = [n.start_us for n in nodes if n.op == "phase.begin"]
    ends = [n.end_us for n in nodes if n.op == "phase.end"]
    if begins and ends:
        return max(ends) - min(begins)
    return max(n.end_us for n in nodes) - min(n.start_us for n in nodes)


def _summed(graph, keep, only: set[int] | None = None) -> float:
    return sum(n.dur_us for n in graph.uops.values()
               if keep(n.op) and (only is None or n.id in only))


def _path_set(graph, critical_path) -> set[int]:
    return set(analyze_critical_path(graph).path if critical_path is None else critical_path)


def total_comm_us(graph) -> float:
    return _summed(graph, is_comm)


def exposed_comm_us(graph, critical_path: tuple[int, ...] | None = None) -> float:
    return _summed(graph, is_comm, _path_set(graph, critical_path))


def total_data_movement_us(graph) -> float:
    return _summed(graph, is_data_movement)


def exposed_data_movement_us(graph, critical_path: tuple[int, ...] | None = None) -> float:
    return _summed(graph, is_data_movement, _path_set(graph, critical_path))


def analyze_exposure(graph) -> ExposureResult:
    crit = analyze_critical_path(graph)
    phase = phase_duration_us(graph)
    comm_on_path = exposed_comm_us(graph, crit.path)
    move_on_path = exposed_data_movement_us(graph, crit.path)
    return ExposureResult(
        phase_time_us=phase,
        critical_path_us=crit.duration_us,
        total_comm_us=total_comm_us(graph),
        exposed_comm_us=comm_on_path,
        total_data_movement_us=total_data_movement_us(graph),
        exposed_data_movement_us=move_on_path,
        ecr=comm_on_path / phase if phase != 0 else 0.0,
        edmr=move_on_path / phase if phase != 0 else 0.0,
        critical_path=crit.path,
    )


def classify_gain(gain_us: float, baseline_us: float) -> str:
    if baseline_us <= 0:
        return "unknown"
    ratio = gain_us / baseline_us
    if ratio > 0.05:
        return "material"
    if ratio > 0.0:
        return "small"
    return "none" if ratio == 0.0 else "regression"


def analyze_overlap(before, after) -> OverlapGainResult:
    t0, t1 = phase_duration_us(before), phase_duration_us(after)
    gain = t0 - t1
    return OverlapGainResult(
        before_us=t0,
        after_us=t1,
        gain_us=gain,
        gain_ratio=gain / t0 if t0 != 0 else 0.0,
        label=classify_gain(gain, t0),
    )


__all__ = [
    "CriticalPathResult", "ExposureResult", "OverlapGainResult",
    "analyze_critical_path", "analyze_exposure", "analyze_overlap", "classify_gain",
    "exposed_comm_us", "exposed_data_movement_us", "phase_duration_us",
    "total_comm_us", "total_data_movement_us",
]
