"""Lowering of a tensor-parallel linear layer: spec -> schedule candidates (EDM graphs) ->
selected schedule -> launch -> measured UOps.

The reference has no lowering ("EDM-IR represents observed execution", paper/mlsys-2027/
edm-ir.md:7); what it does have, and what this module keeps, is the node API the result is
reported in (``UOp``/``MovementDesc``/``EDMBuilder``, EDM-IR/ir/uop.py:44-142, builder.py:22-110),
the analysis that scores candidates (analysis.py:36-65) and the way a measured run is turned
into a graph (CUDA-event timing and ``edm.<ns>:<name>.iter<N>`` NVTX ranges,
EDM-IR/ir/trace.py:26-43, :122-172, :204-266).

A candidate is a ``schedule.Schedule``; its predicted execution is an EDM graph with integer
nanosecond durations (``schedule_graph``): GEMM nodes per shard and chunk, transfer nodes per peer
and chunk on the streams that carry them, flag publications, the launch itself.  The graph's
critical path, evaluated by the native library with the reference's tie rules
(``edm_graph_cost``), is the candidate's cost; the terms follow the reference's overlap model
(paper/mlsys-2027/model.md:98 transfer = alpha + beta*m, :118 exposed = what the compute window
does not cover, :161-168 what splitting and new contention cost).
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass
from functools import lru_cache
from typing import Callable, Sequence

from . import _lib
from .calibration import Calibration, gemm_ns, tile_ns, wire_bytes
from .ir import EDMBuilder, EDMGraph, MovementDesc, TensorDesc
from .ir import ops as irops
from .schedule import Schedule

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


# ---------------------------------------------------------------- candidates
# (4 pusher CTAs were a candidate once: they deliver a shard just in time on paper and 20-30 % late
# in every measurement)
AG_PUSHER_CTAS = (8, 16, 24, 32)
AG_CHUNKS = (1, 2, 4, 8)
ONE_SHOT_MAX_BYTES = 4 << 20   # partial [M, N] above which a one-shot all-reduce is not even scored


def candidates(spec: TPLinearSpec, include_unfused: bool = True) -> list[Schedule]:
    """The schedules a call can run with, indexed in the order returned.

    Index 0 is the unfused sequence (this library's GEMM, then the ``torch.distributed``
    collective): it is scored like the others so the model can say when fusion does not pay, but
    ``select_schedule`` only picks it when asked to (it is a library collective, kept as the
    comparison baseline).  All-gather + GEMM: kernel pushes by dedicated pusher CTAs (how many SMs
    to give up) or by warps inside every GEMM CTA, copy engines on one or two side streams, or
    both, each at several flag granularities.  GEMM + reduce-scatter / all-reduce have one fused
    schedule: every tile is pushed as it is finished, there is no coarser granularity to choose.
    Small all-reduces also have the one-shot schedule (plain GEMM, then every rank reads all
    partials): one flag round trip instead of two, W-1 times the partial as link reads."""
    if spec.world == 1:
        return [Schedule(index=0)]
    out: list[Schedule] = []
    if include_unfused:
        out.append(Schedule(fused=False))
    if spec.op != "ag_gemm":
        out.append(Schedule())
        if spec.op == "gemm_ar" and spec.M * spec.N * 2 <= ONE_SHOT_MAX_BYTES and (spec.N * 2) % 16 == 0:
            out.append(Schedule(one_shot=True))
    else:
        rows = spec.M // spec.world
        chunk_ok = [c for c in AG_CHUNKS if c <= rows and (rows // c) >= 1]
        for c in chunk_ok:
            for p in AG_PUSHER_CTAS:
                out.append(Schedule(chunks=c, transport="sm", pusher_ctas=p))
        for c in chunk_ok[:3]:
            out.append(Schedule(chunks=c, transport="sm", pusher_ctas=0))
            # (one side stream delivers in consumption order but at ~60 % of the rate of two, and
            # measured slower on every shape: not a candidate)
            out.append(Schedule(chunks=c, transport="ce", side_streams=2))
            # (the striped copy-engine transport "cs" -- a stream per chunk, all engines on one peer at
            # a time -- can be asked for but is not a candidate: 314-477 us against 297 us for a stream
            # per peer on the qkv shape at 8 ranks, never ahead at 2 or 4)
        if spec.world > 2:
            for c in chunk_ok[1:3]:
                for p in (8, 16):
                    for far in sorted({max(1, (spec.world - 1) // 3), (spec.world - 1) // 2}):
                        out.append(Schedule(chunks=c, transport="hybrid", pusher_ctas=p, ce_peers=far, side_streams=1))
    return [s.with_index(i) for i, s in enumerate(out)]


# ---------------------------------------------------------------- predicted execution
class _Plan:
    """Tasks with integer durations and dependencies, laid out as soon as possible and emitted
    through ``EDMBuilder`` in creation order (which is part of the tie-breaking contract)."""

    def __init__(self, phase: str):
        self.phase = phase
        self.tasks: list[dict] = []

    def add(self, kind: str, name: str, op: str, dur: int, deps: Sequence[int] = (), stream: str | None = None,
            after: int | None = None, **kw) -> int:
        """``after``: the previous task on the same stream (stream order); ``deps``: data dependencies."""
        start = 0
        for d in list(deps) + ([after] if after is not None else []):
            start = max(start, self.tasks[d]["end"])
        self.tasks.append({"kind": kind, "name": name, "op": op, "start": start, "end": start + max(int(dur), 0),
                           "deps": list(deps), "after": after, "stream": stream, "kw": kw})
        return len(self.tasks) - 1

    def build(self, common: dict) -> EDMGraph:
        b = EDMBuilder(default_phase=self.phase)
        begin = b.phase_begin(self.phase, 0)
        nodes = []
        for t in self.tasks:
            make = {"compute": b.compute, "comm": b.comm}.get(t["kind"])
            if make is not None:
                node = make(t["name"], t["start"], t["end"], op=t["op"], stream=t["stream"], **common, **t["kw"])
            else:
                node = b.uop(t["op"], t["name"], t["start"], t["end"], stream=t["stream"], **common, **t["kw"])
            nodes.append(node)
        end = b.phase_end(self.phase, max([t["end"] for t in self.tasks], default=0))
        for i, t in enumerate(self.tasks):
            if t["after"] is not None:
                b.edge(nodes[t["after"]], nodes[i], irops.STREAM_ORDER)
        for i, t in enumerate(self.tasks):
            for d in t["deps"]:
                b.data_edge(nodes[d], nodes[i], t["name"])
        b.bind_phase(begin, end, *nodes)
        return b.build()


def schedule_graph(spec: TPLinearSpec, sched: Schedule, calib: Calibration, tp_rank: int | None = None) -> EDMGraph:
    """The predicted execution of ``sched`` for ``spec`` as an EDM graph (durations in ns)."""
    W = spec.world
    wire = wire_bytes(spec.op, spec.M, spec.N, spec.K, W)
    comm_op = _COMM_OP[spec.op]
    group = tuple(range(W))
    plan = _Plan("tp_linear")
    attrs = {"schedule_index": sched.index, "schedule": sched.label()}
    common = {"tp_rank": tp_rank}

    def move(nbytes: int, backend: str) -> MovementDesc:
        return MovementDesc(kind=comm_op.split(".", 1)[1], backend=backend, size_bytes=int(nbytes), group="tp",
                            group_ranks=group)

    if W == 1:
        plan.add("compute", "gemm", irops.COMPUTE_GEMM, gemm_ns(spec.M, spec.N, spec.K, calib), stream="compute",
                 attrs=dict(attrs))
        return plan.build(common)

    if not sched.fused:
        # two launches: the library collective at its own rate, before (all-gather) or after the GEMM
        coll = calib.launch_ns + int(wire / calib.nccl_gbs) + W * calib.skew_ns_per_rank
        full = gemm_ns(spec.M, spec.N, spec.K, calib, plain=spec.op != "ag_gemm")
        if spec.op == "ag_gemm":
            m = plan.add("comm", "all_gather", comm_op, coll, stream="nccl", movement=move(wire, "nccl"), attrs=dict(attrs))
            plan.add("compute", "gemm", irops.COMPUTE_GEMM, calib.launch_ns + full, deps=(m,), stream="compute",
                     attrs=dict(attrs))
        else:
            g = plan.add("compute", "gemm", irops.COMPUTE_GEMM, calib.launch_ns + full, stream="compute", attrs=dict(attrs))
            plan.add("comm", spec.op, comm_op, coll, deps=(g,), stream="nccl", movement=move(wire, "nccl"),
                     attrs=dict(attrs))
        return plan.build(common)

    skew = (W - 1) * calib.skew_ns_per_rank
    if spec.op == "ag_gemm":
        c = sched.chunks
        first_d = 1
        ce_lo = {"sm": W, "ce": first_d, "cs": first_d, "hybrid": max(first_d, W - sched.ce_peers)}[sched.transport]
        striped = sched.transport == "cs"
        pushes = ce_lo > first_d
        uses_ce = ce_lo < W
        pushers = sched.pusher_ctas if pushes else 0
        units = calib.gemm_units - pushers // 2
        total = gemm_ns(spec.M, spec.N, spec.K, calib, units=units)
        if pushes and pushers == 0:
            total = int(total * calib.sm_push_slowdown)  # push warps share the GEMM CTAs' memory pipes
        push_rate = min(calib.link_gbs, pushers * calib.pusher_cta_gbs) if pushers else calib.link_gbs
        n_streams = min(max(sched.side_streams, 1), c if striped else max(W - ce_lo, 1)) if uses_ce else 0
        # striped: every stream serves the same peer, the engines together reach the one-peer rate
        ce_rate = (calib.ce_gbs_one_peer if striped else calib.ce_rate(n_streams, W - ce_lo)) if uses_ce else 0.0
        if pushes and uses_ce and push_rate + ce_rate > calib.link_gbs:  # both share the link
            scale = calib.link_gbs / (push_rate + ce_rate)
            push_rate, ce_rate = push_rate * scale, ce_rate * scale
        shard = wire // (W - 1)
        setup = plan.add("other", "launch", irops.RUNTIME_LAUNCH_GAP,
                         calib.launch_ns + skew + (calib.ce_launch_ns if uses_ce else 0), stream="compute")
        # a tile cannot finish sooner than one tile time after its rows have landed (half of it plus
        # the exchange where the last wave is cut along K)
        floor = int(tile_ns(spec.K, calib) * (0.65 if spec.K * 2 // 128 >= 32 else 1.0))
        # transfers: one chain per carrier, shards in the order their consumers need them
        last = {"push": setup}
        for s in range(n_streams):
            last[f"ce{s}"] = setup
        ready: dict = {}
        for d in range(1, W):
            if d < ce_lo:
                stream, rate, backend = "push", push_rate, "nvlink-p2p"
            else:
                stream, rate, backend = f"ce{d % n_streams}", ce_rate / n_streams, "copy-engine"
            pushed = d < ce_lo
            per_chunk = (calib.push_chunk_ns if pushers else calib.sm_chunk_ns) if pushed else calib.ce_op_ns
            publish = (calib.push_publish_ns if pushers else calib.publish_ns) if pushed else 0
            for k in range(c):
                nbytes = shard // c + (1 if k < shard % c else 0)
                if striped:
                    stream = f"ce{k % n_streams}"
                node = plan.add("comm", f"all_gather.s{d}.c{k}", comm_op, int(nbytes / rate) + per_chunk, stream=stream,
                                after=last[stream], movement=move(nbytes, backend),
                                attrs={**attrs, "chunk": k, "shard": d})
                last[stream] = node
                # the chunk's flag becomes visible one publication later (not link time); a copy
                # engine's flag write is part of its stream operation
                ready[(d, k)] = plan.add("other", f"flag.s{d}.c{k}", irops.EVENT_RECORD, publish,
                                         deps=(node,), stream=stream + ".flags")
        prev = setup
        for j in range(W):
            for k in range(c):
                share = total // (W * c) + (1 if (j * c + k) < total % (W * c) else 0)
                deps = (ready[(j, k)],) if j > 0 else ()
                prev = plan.add("compute", f"gemm.s{j}.c{k}", irops.COMPUTE_GEMM, share, deps=deps, stream="compute",
                                after=prev, attrs={**attrs, "chunk": k, "shard": j})
                if j > 0 and share < floor:
                    plan.add("compute", f"tile.s{j}.c{k}", irops.COMPUTE_GEMM, floor, deps=deps, stream=f"tiles.s{j}",
                             attrs={**attrs, "chunk": k, "shard": j})
        return plan.build(common)

    if sched.one_shot:
        # plain GEMM (its fixed cost covers the launch), second launch, one flag round trip, then W-1
        # remote reads of the whole partial; the ranks' launches drift apart by about half the skew
        setup = plan.add("other", "launch", irops.RUNTIME_LAUNCH_GAP, skew // 2, stream="compute")
        g = plan.add("compute", "gemm", irops.COMPUTE_GEMM, gemm_ns(spec.M, spec.N, spec.K, calib, plain=True),
                     stream="compute", after=setup, attrs=dict(attrs))
        flag = plan.add("other", "flags", irops.EVENT_RECORD, calib.one_shot_sync_ns, deps=(g,), stream="push.flags")
        pull = (W - 1) * spec.M * spec.N * 2
        plan.add("comm", "gemm_ar.pull", comm_op, int(pull / calib.all_to_all_rate(W)), deps=(flag,), stream="push",
                 movement=move(pull, "nvlink-p2p"), attrs=dict(attrs))
        return plan.build(common)

    # GEMM + reduce-scatter / all-reduce: tiles are pushed as they finish; modelled as G groups of
    # tile rounds.  The last group's flags and its reduction at the owner cannot overlap anything.
    tiles = -(-spec.M // 256) * -(-spec.N // 256)
    rounds = max(1, -(-tiles // calib.gemm_units))
    G = min(8, rounds)
    total = gemm_ns(spec.M, spec.N, spec.K, calib)
    push_bytes = wire if spec.op == "gemm_rs" else wire // 2
    # (a rank only waits for peers' tiles at the very end: about half the drift of the launches shows)
    setup = plan.add("other", "launch", irops.RUNTIME_LAUNCH_GAP, calib.launch_ns + skew // 2, stream="compute")
    g_prev, m_prev = setup, None
    for i in range(G):
        g_prev = plan.add("compute", f"gemm.{i}", irops.COMPUTE_GEMM, total // G + (1 if i < total % G else 0),
                          stream="compute", after=g_prev, attrs={**attrs, "chunk": i})
        nbytes = push_bytes // G + (1 if i < push_bytes % G else 0)
        m_prev = plan.add("comm", f"{spec.op}.{i}", comm_op, int(nbytes / calib.all_to_all_rate(W)), deps=(g_prev,), stream="push",
                          after=m_prev, movement=move(nbytes, "nvlink-p2p"), attrs={**attrs, "chunk": i})
    flag = plan.add("other", "flags", irops.EVENT_RECORD, calib.publish_ns, deps=(m_prev,), stream="push.flags")
    own_bytes = (spec.M // W if spec.op == "gemm_rs" else -(-spec.M // W)) * spec.N * 2
    red = plan.add("compute", "reduce", irops.COMPUTE_OTHER, int(own_bytes * W / G / calib.reduce_gbs), deps=(flag,),
                   stream="reduce", attrs=dict(attrs))
    if spec.op == "gemm_ar":
        # the owner stores the reduced tiles into every rank's output: the second half of the wire bytes
        tail = wire // 2 // G
        plan.add("comm", "gemm_ar.result", comm_op, int(tail / calib.all_to_all_rate(W)) + calib.publish_ns, deps=(red,),
                 stream="push", movement=move(tail, "nvlink-p2p"), attrs=dict(attrs))
    return plan.build(common)


@dataclass(frozen=True)
class ScheduleCost:
    makespan: int       # critical-path duration, ns
    exposed_comm: int   # duration of comm nodes on the critical path
    total_comm: int


def graph_cost(graph: EDMGraph) -> ScheduleCost:
    """Critical path and exposed communication of a graph with integer durations, evaluated by
    the native library (bit-exact with ``analyze_critical_path`` / ``analyze_exposure``)."""
    ids = sorted(graph.uops)
    pos = {u: i for i, u in enumerate(ids)}
    n, m = len(ids), len(graph.edges)
    dur = (C.c_int64 * max(n, 1))(*[int(graph.uops[u].end_us - graph.uops[u].start_us) for u in ids])
    end = (C.c_int64 * max(n, 1))(*[int(graph.uops[u].end_us) for u in ids])
    comm = (C.c_uint8 * max(n, 1))(*[1 if irops.is_comm(graph.uops[u].op) else 0 for u in ids])
    src = (C.c_int32 * max(m, 1))(*[pos[e.src] for e in graph.edges])
    dst = (C.c_int32 * max(m, 1))(*[pos[e.dst] for e in graph.edges])
    makespan, exposed = C.c_int64(), C.c_int64()
    _lib.check(_lib.load().edm_graph_cost(n, dur, end, comm, m, src, dst, C.byref(makespan), C.byref(exposed),
                                          None, None), "edm_graph_cost")
    total = sum(int(graph.uops[u].end_us - graph.uops[u].start_us) for u in ids if irops.is_comm(graph.uops[u].op))
    return ScheduleCost(makespan.value, exposed.value, total)


@dataclass(frozen=True)
class Selection:
    spec: TPLinearSpec
    schedules: list
    costs: list          # ScheduleCost per schedule
    chosen: int
    graphs: list         # candidate EDM graphs, same order

    @property
    def schedule(self) -> Schedule:
        return self.schedules[self.chosen]

    @property
    def predicted_us(self) -> float:
        return self.costs[self.chosen].makespan / 1e3


@lru_cache(maxsize=256)
def _select(spec: TPLinearSpec, calib: Calibration, allow_unfused: bool, tp_rank: int | None) -> Selection:
    scheds = candidates(spec)
    graphs = [schedule_graph(spec, s, calib, tp_rank) for s in scheds]
    costs = [graph_cost(g) for g in graphs]
    pool = [i for i, s in enumerate(scheds) if s.fused or allow_unfused or spec.world == 1]
    chosen = min(pool, key=lambda i: (costs[i].makespan, i))
    return Selection(spec, scheds, costs, chosen, graphs)


def select_schedule(spec: TPLinearSpec, calib: Calibration | None = None, allow_unfused: bool = False,
                    tp_rank: int | None = None) -> Selection:
    """Score every candidate and return the arg-min of the critical path (ties: lowest index).
    The unfused sequence is scored too but only chosen with ``allow_unfused`` (it needs an
    initialised ``torch.distributed`` group and is a library collective)."""
    return _select(spec, calib or Calibration.load(), allow_unfused, tp_rank)


# ---------------------------------------------------------------- launching
def lower(spec: TPLinearSpec, ctx, schedule: Schedule) -> Callable:
    """Returns ``fn(a, b, out) -> out`` running ``schedule`` for ``spec``.

    ``ctx`` is a ``symm.SymmetricContext`` (``None`` for a single rank).  Fused schedules are one
    launch of the fused kernel with every schedule field passed through ``edm_tp_call_t``; the
    unfused schedule is this library's GEMM followed by the ``torch.distributed`` collective."""
    from . import linear

    if spec.world == 1 or ctx is None:
        return lambda a, b, out=None: linear.gemm(a, b, out)
    if schedule.fused:
        if spec.op == "ag_gemm":
            return lambda x, w, out=None: ctx.ag_gemm(x, w, out, schedule=schedule)
        if spec.op == "gemm_rs":
            return lambda a, b, out=None: ctx.gemm_rs(a, b, out, schedule=schedule)
        return lambda a, b, out=None: ctx.gemm_ar(a, b, out, schedule=schedule)

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


def lower_emulated(spec: TPLinearSpec, group, schedule: Schedule) -> Callable:
    """The same lowering for a ``symm.EmulatedGroup`` (all ranks of the group on one device, one
    cooperative launch): returns ``fn(a_list, b_list, out_list) -> out_list``.  Only fused
    schedules can be emulated (the unfused one needs a process group)."""
    if not schedule.fused:
        raise ValueError("the unfused schedule runs a torch.distributed collective: it cannot be emulated on one device")
    if group.world != spec.world:
        raise ValueError("the group's size differs from the spec's")
    return lambda a_list, b_list, out_list: group.run(spec.op, a_list, b_list, out_list, schedule=schedule)


def nvtx_name(namespace: str, name: str, iteration: int | None = None) -> str:
    """``edm.<ns>:<name>[.iter<N>]`` -- the range-name grammar the reference's profiler import
    parses (EDM-IR/ir/nsys_export.py:17, :74-88)."""
    base = f"edm.{namespace}:{name}"
    return base if iteration is None else f"{base}.iter{iteration}"


def launch_range_name(spec: TPLinearSpec, iteration: int | None = None) -> str:
    """NVTX range of one launch: it parses back to the op the launch's exchange stands for
    (``comm.reduce_scatter`` ...), or ``compute.gemm`` on a single rank."""
    if spec.world == 1:
        return nvtx_name("compute", "gemm", iteration)
    return nvtx_name("comm", _COMM_OP[spec.op].split(".", 1)[1], iteration)


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
                         "schedule": schedule.label(), "M": spec.M, "N": spec.N, "K": spec.K})
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
        torch.cuda.nvtx.range_push(launch_range_name(spec, i))
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
