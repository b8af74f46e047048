"""Fixed-width text dumps of UOps and the exposure summary.

Output format is the reference's (EDM-IR/ir/printing.py:11-92) so existing log scrapers keep
working: one line per UOp with ``%id op name start->end dur=..us`` and trailing tags, a
``critical_path=`` chain, and ``key=value`` summary lines with three decimals.
"""
from __future__ import annotations

from collections.abc import Iterable

from .analysis import analyze_exposure
from .graph import EDMGraph
from .ops import is_data_movement
from .uop import DataRef, UOp


def _refs(refs: tuple[DataRef, ...]) -> str:
    return ",".join(f"{r.kind}:{r.data_id}" for r in refs)


def _tags(uop: UOp) -> str:
    out = [f"{key}={uop.attr(key)}" for key in ("phase", "stream", "device") if uop.attr(key) is not None]
    rank = uop.attr("global_rank")
    if rank is not None:
        out.append(f"rank={rank}")
    mv = uop.movement
    if mv is not None:
        if mv.size_bytes is not None:
            out.append(f"bytes={mv.size_bytes}")
        if mv.group is not None:
            out.append(f"group={mv.group}")
    if uop.reads:
        out.append("reads=" + _refs(uop.reads))
    if uop.writes:
        out.append("writes=" + _refs(uop.writes))
    return "  " + " ".join(out) if out else ""


def format_uop(uop: UOp, *, highlight: bool = False) -> str:
    star = "*" if highlight else " "
    return (f"{star}%{uop.id:03d} {uop.op:<20} {uop.name:<24} "
            f"{uop.start_us:9.3f}->{uop.end_us:9.3f} dur={uop.dur_us:9.3f}us{_tags(uop)}")


def format_uops(graph: EDMGraph, *, highlight: Iterable[int] = ()) -> str:
    marked = set(highlight)
    return "\n".join(format_uop(graph.uops[uid], highlight=uid in marked) for uid in sorted(graph.uops))


def format_critical_path(graph: EDMGraph) -> str:
    path, total = graph.critical_path()
    if not path:
        return "critical_path=<empty>\ncritical_path_us=0.000"
    chain = " -> ".join(f"%{uid}:{graph.uops[uid].op}" for uid in path)
    return f"critical_path={chain}\ncritical_path_us={total:.3f}"


def format_summary(graph: EDMGraph) -> str:
    ex = analyze_exposure(graph)
    rows = [
        ("phase_us", ex.phase_time_us), ("critical_path_us", ex.critical_path_us),
        ("total_comm_us", ex.total_comm_us), ("exposed_comm_us", ex.exposed_comm_us),
        ("ecr", ex.ecr), ("total_data_movement_us", ex.total_data_movement_us),
        ("exposed_data_movement_us", ex.exposed_data_movement_us), ("edmr", ex.edmr),
    ]
    lines = [f"{k}={v:.3f}" for k, v in rows]
    movers = [uid for uid in ex.critical_path if is_data_movement(graph.uops[uid].op)]
    shown = ", ".join(f"%{uid}:{graph.uops[uid].op}" for uid in movers) if movers else "<none>"
    lines.append("exposed_data_movement=" + shown)
    return "\n".join(lines)


__all__ = ["format_critical_path", "format_summary", "format_uop", "format_uops"]
