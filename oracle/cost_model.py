"""Restatement of the reference's graph cost evaluation, on plain lists, plus the chunked
pipeline candidates the schedule selector scores.  TEST INFRASTRUCTURE (see ``__init__``).

What is restated and where it comes from:
* ``topological_order``  -- EDM-IR/ir/graph.py:54-72 (Kahn; start set = sorted zero-indegree
  ids; successors in edge-insertion order).
* ``critical_path``      -- EDM-IR/ir/analysis.py:36-65 (parent = first predecessor with the
  maximal prefix, ``max(..., key=)`` semantics; end = max by ``(prefix, end_us, id)``).
* ``phase_duration``     -- EDM-IR/ir/analysis.py:68-86.
* ``exposure``           -- EDM-IR/ir/analysis.py:89-123 (comm = ops starting ``comm.``;
  data movement additionally ``kv.transfer`` and ``movement.copy``, EDM-IR/ir/ops.py:119-124).
* ``candidate_graph``    -- no reference counterpart (the reference has no selector); it is the
  graph EDM-IR/ir/builder.py:22-110 would hold for "c GEMM chunks feeding c collective chunks",
  with durations from the alpha-beta form of paper/mlsys-2027/model.md:98 and the split
  overhead of model.md:161-168.

PINNED against the reference itself: ``tests/golden/analysis_golden.json`` and
``tests/golden/selector_golden.json`` hold outputs of the reference's own ``EDMBuilder`` +
``analyze_critical_path`` / ``analyze_exposure`` for the same graphs (see
``tests/golden/make_golden.py``).
"""
from __future__ import annotations

from collections import deque

# A graph here is: nodes = list of dicts {id, op, start, end}; edges = list of (src, dst).


def topological_order(nodes, edges) -> list[int]:
    indeg = {n["id"]: 0 for n in nodes}
    succ: dict[int, list[int]] = {}
    for s, d in edges:
        indeg[d] += 1
        succ.setdefault(s, []).append(d)
    ready = deque(sorted(u for u, k in indeg.items() if k == 0))
    order = []
    while ready:
        u = ready.popleft()
        order.append(u)
        for v in succ.get(u, ()):
            indeg[v] -= 1
            if indeg[v] == 0:
                ready.append(v)
    if len(order) != len(nodes):
        raise ValueError("cycle")
    return order


def critical_path(nodes, edges):
    """Returns ``(path_ids, duration)``."""
    by_id = {n["id"]: n for n in nodes}
    pred: dict[int, list[int]] = {}
    for s, d in edges:
        pred.setdefault(d, []).append(s)
    best, parent = {}, {}
    for u in topological_order(nodes, edges):
        dur = by_id[u]["end"] - by_id[u]["start"]
        if not pred.get(u):
            best[u], parent[u] = dur, None
            continue
        p = max(pred[u], key=lambda q: best[q])  # first maximum
        best[u], parent[u] = best[p] + dur, p
    if not best:
        return [], 0
    end = max(best, key=lambda u: (best[u], by_id[u]["end"], u))
    path, cur = [], end
    while cur is not None:
        path.append(cur)
        cur = parent[cur]
    path.reverse()
    return path, best[end]


def phase_duration(nodes):
    if not nodes:
        return 0
    begins = [n["start"] for n in nodes if n["op"] == "phase.begin"]
    ends = [n["end"] for n in nodes if n["op"] == "phase.end"]
    if begins and ends:
        return max(ends) - min(begins)
    return max(n["end"] for n in nodes) - min(n["start"] for n in nodes)


def _is_comm(op: str) -> bool:
    return op.startswith("comm.")


def _is_movement(op: str) -> bool:
    return _is_comm(op) or op in ("kv.transfer", "movement.copy")


def exposure(nodes, edges) -> dict:
    path, dur = critical_path(nodes, edges)
    on_path = set(path)
    phase = phase_duration(nodes)

    def total(pred, only=None):
        return sum(n["end"] - n["start"] for n in nodes
                   if pred(n["op"]) and (only is None or n["id"] in only))

    ec, em = total(_is_comm, on_path), total(_is_movement, on_path)
    return {
        "phase_time_us": phase, "critical_path_us": dur, "critical_path": path,
        "total_comm_us": total(_is_comm), "exposed_comm_us": ec,
        "total_data_movement_us": total(_is_movement), "exposed_data_movement_us": em,
        "ecr": 0.0 if phase == 0 else ec / phase, "edmr": 0.0 if phase == 0 else em / phase,
    }


# ---------------------------------------------------------------- schedule candidates
def _share(total: int, c: int, i: int) -> int:
    return total // c + (1 if i < total % c else 0)


def chunk_durations(params: dict, c: int):
    """Integer durations of the c GEMM chunks and the c collective chunks."""
    g = [_share(params["gemm_total"], c, i) + (params["split_overhead"] if c > 1 else 0) for i in range(c)]
    m = [params["alpha"] + -(-(_share(params["comm_bytes"], c, i) * params["beta_num"]) // params["beta_den"])
         for i in range(c)]
    return g, m


def candidate_graph(params: dict, c: int, comm_op: str = "comm.reduce_scatter"):
    """Nodes and edges of the c-chunk pipeline, in builder creation / insertion order:
    ids 0 = phase.begin, 1..c = GEMM chunks, c+1..2c = collective chunks, 2c+1 = phase.end;
    edges: GEMM chain, collective chain, per-chunk data dependency, then the phase binding
    (begin->node, node->end for each body node in id order).  Timestamps are the
    as-soon-as-possible schedule."""
    g, m = chunk_durations(params, c)
    comm_first = bool(params.get("comm_first", 0))
    nodes = [{"id": 0, "op": "phase.begin", "start": 0, "end": 0}]
    g_t, m_t = [], []
    g_end = m_end = 0
    for i in range(c):
        if not comm_first:
            gs = g_end; g_end = gs + g[i]
            ms = max(g_end, m_end); m_end = ms + m[i]
        else:
            ms = m_end; m_end = ms + m[i]
            gs = max(g_end, m_end); g_end = gs + g[i]
        g_t.append((gs, gs + g[i])); m_t.append((ms, ms + m[i]))
    for i in range(c):
        nodes.append({"id": 1 + i, "op": "compute.gemm", "start": g_t[i][0], "end": g_t[i][1]})
    for i in range(c):
        nodes.append({"id": 1 + c + i, "op": comm_op, "start": m_t[i][0], "end": m_t[i][1]})
    fin = max(g_end, m_end)
    nodes.append({"id": 2 * c + 1, "op": "phase.end", "start": fin, "end": fin})
    edges = [(1 + i, 2 + i) for i in range(c - 1)]
    edges += [(1 + c + i, 2 + c + i) for i in range(c - 1)]
    edges += [((1 + c + i, 1 + i) if comm_first else (1 + i, 1 + c + i)) for i in range(c)]
    for u in range(1, 2 * c + 1):
        edges.append((0, u))
        edges.append((u, 2 * c + 1))
    return nodes, edges


def schedule_cost(params: dict, c: int) -> dict:
    nodes, edges = candidate_graph(params, c)
    ex = exposure(nodes, edges)
    g, m = chunk_durations(params, c)
    return {"makespan": ex["critical_path_us"], "exposed_comm": ex["exposed_comm_us"],
            "total_comm": ex["total_comm_us"], "gemm_chunk": g[0], "comm_chunk": m[0]}


def select_schedule(params: dict, candidates) -> tuple[int, list[dict]]:
    """Index of the candidate with the smallest makespan (ties: lowest index) and all costs."""
    costs = [schedule_cost(params, c) for c in candidates]
    best = min(range(len(costs)), key=lambda i: costs[i]["makespan"])
    return best, costs
