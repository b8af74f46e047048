"""Profiler round trip: an Nsight Systems sqlite export of a run of this package -> EDM graph.

The fused launches and the overlap probe wrap their work in NVTX ranges named
``edm.<namespace>:<name>[.iter<N>]`` (``lowering.nvtx_name``, ``ir/trace.py``).  The reference
reads such profiles back into flat tables: ranges whose text starts with ``edm.``, CUDA runtime
calls, kernels and memcpys joined to the innermost range that encloses the runtime call with the
same correlation id (EDM-IR/ir/nsys_export.py:74-88 grammar, :91-183 readers, :193-208 join).
This module performs the same read and join, and goes one step further than the reference's CSV
export: every range that owns GPU work becomes a ``UOp`` whose interval is the span of that
work on the device, so the analysis passes (``analyze_exposure`` etc.) run on what the profiler
saw.  Only the standard library and the ``ir`` package are used; no GPU is needed to import.
"""
from __future__ import annotations

import re
import sqlite3
from dataclasses import dataclass, field
from pathlib import Path

from .ir import EDMBuilder, EDMGraph, MovementDesc
from .ir import ops as irops

_ITER = re.compile(r"\.iter(\d+)$")


def parse_edm_text(text: str) -> tuple[str, int | None]:
    """``edm.compute:qkv.matmul.iter3`` -> (``compute.qkv.matmul``, 3); a trailing ``.iter<N>`` is
    optional; text that does not start with ``edm.`` is returned unchanged."""
    iteration = None
    m = _ITER.search(text)
    if m:
        iteration = int(m.group(1))
        text = text[:m.start()]
    if not text.startswith("edm."):
        return text, iteration
    body = text[4:]
    ns, sep, name = body.partition(":")
    return (f"{ns}.{name}" if sep else body), iteration


@dataclass(frozen=True)
class GpuEvent:
    kind: str              # "kernel" | "memcpy"
    name: str
    start_ns: int
    end_ns: int
    stream_id: int | None
    correlation_id: int
    bytes: int | None = None
    copy_kind: str | None = None


@dataclass
class ProfiledRange:
    text: str
    op: str
    iteration: int | None
    start_ns: int
    end_ns: int
    global_tid: int | None
    events: list = field(default_factory=list)   # GpuEvent launched from inside this range (innermost)

    @property
    def dur_ns(self) -> int:
        return self.end_ns - self.start_ns


def _tables(conn) -> set:
    return {r[0] for r in conn.execute("select name from sqlite_master where type='table'")}


def _columns(conn, table: str) -> list:
    return [r[1] for r in conn.execute(f'pragma table_info("{table}")')]


def _int(v):
    return None if v is None else int(v)


def read_profile(sqlite_path: str | Path) -> tuple[list[ProfiledRange], list[GpuEvent], int]:
    """Returns ``(ranges, unattached_events, origin_ns)``: the ``edm.*`` NVTX ranges in start
    order, each with the GPU events launched from inside it, the GPU events no range claims, and
    the earliest timestamp in the profile."""
    path = Path(sqlite_path)
    if not path.exists():
        raise FileNotFoundError(path)
    conn = sqlite3.connect(str(path))
    conn.row_factory = sqlite3.Row
    try:
        tables = _tables(conn)
        strings = {}
        if "StringIds" in tables:
            strings = {int(r["id"]): str(r["value"]) for r in conn.execute('select id, value from "StringIds"')}

        def text_of(v) -> str:
            if v is None:
                return ""
            return strings[v] if isinstance(v, int) and v in strings else str(v)

        ranges: list[ProfiledRange] = []
        if "NVTX_EVENTS" in tables and "text" in _columns(conn, "NVTX_EVENTS"):
            for r in conn.execute('select start, end, text, globalTid from "NVTX_EVENTS" '
                                  "where text like 'edm.%' and end is not null order by start"):
                op, it = parse_edm_text(str(r["text"]))
                ranges.append(ProfiledRange(str(r["text"]), op, it, int(r["start"]), int(r["end"]), _int(r["globalTid"])))

        calls = []  # (start, end, correlation id)
        if "CUPTI_ACTIVITY_KIND_RUNTIME" in tables:
            calls = [(int(r["start"]), int(r["end"]), int(r["correlationId"]))
                     for r in conn.execute('select start, end, correlationId from "CUPTI_ACTIVITY_KIND_RUNTIME" order by start')]

        events: list[GpuEvent] = []
        if "CUPTI_ACTIVITY_KIND_KERNEL" in tables:
            cols = {c.lower(): c for c in _columns(conn, "CUPTI_ACTIVITY_KIND_KERNEL")}
            name_col = next((cols[c] for c in ("demangledname", "shortname", "mangledname") if c in cols), None)
            for r in conn.execute('select * from "CUPTI_ACTIVITY_KIND_KERNEL" order by start'):
                events.append(GpuEvent("kernel", text_of(r[name_col]) if name_col else "kernel", int(r["start"]),
                                       int(r["end"]), _int(r["streamId"]), int(r["correlationId"])))
        if "CUPTI_ACTIVITY_KIND_MEMCPY" in tables:
            labels = {}
            if "ENUM_CUDA_MEMCPY_OPER" in tables:
                labels = {int(r["id"]): str(r["label"]) for r in conn.execute('select id, label from "ENUM_CUDA_MEMCPY_OPER"')}
            for r in conn.execute('select * from "CUPTI_ACTIVITY_KIND_MEMCPY" order by start'):
                kind = _int(r["copyKind"])
                events.append(GpuEvent("memcpy", "cuda_memcpy", int(r["start"]), int(r["end"]), _int(r["streamId"]),
                                       int(r["correlationId"]), _int(r["bytes"]),
                                       "" if kind is None else labels.get(kind, str(kind))))
        events.sort(key=lambda e: (e.start_ns, e.end_ns, e.kind))
    finally:
        conn.close()

    # runtime call -> innermost enclosing range (shortest; the first of equals); a later call with
    # the same correlation id replaces an earlier one
    owner: dict[int, ProfiledRange] = {}
    for start, end, corr in calls:
        best = None
        for rg in ranges:
            if rg.start_ns <= start and end <= rg.end_ns and (best is None or rg.dur_ns < best.dur_ns):
                best = rg
        if best is not None:
            owner[corr] = best
    loose = []
    for ev in events:
        rg = owner.get(ev.correlation_id)
        (rg.events if rg is not None else loose).append(ev)
    origin = min([r.start_ns for r in ranges] + [c[0] for c in calls] + [e.start_ns for e in events], default=0)
    return ranges, loose, origin


def _movement_for(op: str, events: list) -> MovementDesc | None:
    nbytes = sum(e.bytes or 0 for e in events if e.kind == "memcpy")
    if irops.is_comm(op):
        return MovementDesc(kind=op.split(".", 1)[1], backend="nvlink-p2p", size_bytes=nbytes or None)
    if nbytes:
        kinds = {e.copy_kind for e in events if e.kind == "memcpy" and e.copy_kind}
        return MovementDesc(kind=(kinds.pop() if len(kinds) == 1 else "copy"), backend="cuda", size_bytes=nbytes)
    return None


def known_op(op: str) -> str:
    """The EDM op a range's op string stands for: itself when it is in the vocabulary, else its
    longest dotted prefix that is (``compute.qkv.matmul`` -> ``compute.qkv``), else ``compute.other``."""
    parts = op.split(".")
    while len(parts) >= 2:
        cand = ".".join(parts)
        if cand in irops.ALL_OPS:
            return cand
        parts.pop()
    return irops.COMPUTE_OTHER


def profile_to_graph(sqlite_path: str | Path, iteration: int | None = None, phase: str = "profile") -> EDMGraph:
    """EDM graph of the ``edm.*`` ranges that own GPU work (optionally of one iteration only).

    A node spans its range's GPU events (microseconds from the profile's first timestamp); its op
    is the range's op, shortened to the longest prefix the EDM vocabulary knows (``known_op``; the
    range's own op string is kept in ``attrs["nvtx_op"]``).  Nodes are chained in ``stream_order`` per
    CUDA stream, and a node on one stream that starts after a node on another stream has ended
    gets no edge: the profile does not record why it waited."""
    ranges, _, origin = read_profile(sqlite_path)
    us = lambda ns: (ns - origin) / 1000.0
    b = EDMBuilder(default_phase=phase)
    picked = [r for r in ranges if r.events and (iteration is None or r.iteration == iteration)]
    if not picked:
        return b.build()
    t0 = min(e.start_ns for r in picked for e in r.events)
    t1 = max(e.end_ns for r in picked for e in r.events)
    begin = b.phase_begin(phase, us(t0))
    nodes, last_on_stream = [], {}
    for r in sorted(picked, key=lambda r: min(e.start_ns for e in r.events)):
        start = min(e.start_ns for e in r.events)
        end = max(e.end_ns for e in r.events)
        stream = r.events[0].stream_id
        op = known_op(r.op)
        attrs = {"nvtx_op": r.op, "nvtx_text": r.text, "iteration": r.iteration, "gpu_events": len(r.events),
                 "kernels": sorted({e.name for e in r.events if e.kind == "kernel"})}
        common = dict(stream=None if stream is None else f"stream{stream}", attrs=attrs)
        if irops.is_compute(op):
            node = b.compute(r.op.split(".", 1)[-1], us(start), us(end), op=op, **common)
        else:
            node = b.movement(r.op.split(".", 1)[-1], us(start), us(end), op=op,
                              movement=_movement_for(op, r.events), **common)
        prev = last_on_stream.get(stream)
        if prev is not None:
            b.edge(prev, node, irops.STREAM_ORDER)
        last_on_stream[stream] = node
        nodes.append(node)
    end = b.phase_end(phase, us(t1))
    b.bind_phase(begin, end, *nodes)
    return b.build()
