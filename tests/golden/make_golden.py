"""Generates the golden fixtures in this directory by RUNNING THE REFERENCE.

    python tests/golden/make_golden.py <reference checkout>/EDM-IR

Imports the reference's own ``ir`` package from the directory given on the command line and writes:
* ``analysis_golden.json`` -- the graphs of the reference's tests (tests/analysis_test.py:16-58)
  and demo (examples/synthetic_demo.py:24-128) serialised node by node, with the reference's
  ``analyze_critical_path`` / ``analyze_exposure`` / ``phase_duration_us`` outputs;
* ``selector_golden.json`` -- chunked GEMM->collective pipeline candidates built with the
  reference's ``EDMBuilder`` and scored with its ``analyze_critical_path`` /
  ``analyze_exposure``, for a sweep of integer cost parameters and chunk counts;
* ``gain_golden.json`` -- ``classify_gain`` labels around its thresholds;
* ``trace_golden.json`` -- the six-node graphs the reference's overlap probe builds from three
  measured intervals (ir/trace.py:204-266), with their analysis results and text dumps;
* ``nsys_golden.json`` -- a small hand-made profile (the rows of an Nsight Systems sqlite export:
  NVTX ranges named by the ``edm.<ns>:<name>.iter<N>`` grammar, runtime calls, kernels, memcpys)
  and what the reference's exporter (ir/nsys_export.py:211-314) makes of it.
The reference is only needed to regenerate; tests read the JSON.
"""
from __future__ import annotations

import importlib.util
import itertools
import json
import os
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
if len(sys.argv) < 2:
    sys.exit("usage: make_golden.py <reference checkout>/EDM-IR")
REF = sys.argv[1]
sys.path.insert(0, REF)

import ir  # noqa: E402  (the reference package)
from ir import EDMBuilder  # noqa: E402
from ir.analysis import analyze_critical_path, analyze_exposure, classify_gain, phase_duration_us  # noqa: E402
from ir.ops import COMPUTE_GEMM, DATA_DEPENDENCY, STREAM_ORDER  # noqa: E402

assert os.path.realpath(ir.__file__).startswith(os.path.realpath(REF)), "not the reference package"


def dump_graph(graph) -> dict:
    ex = analyze_exposure(graph)
    cp = analyze_critical_path(graph)
    return {
        "nodes": [{"id": u.id, "op": u.op, "name": u.name, "start": u.start_us, "end": u.end_us,
                   "phase": u.phase} for u in graph.uops.values()],
        "edges": [[e.src, e.dst, e.kind] for e in graph.edges],
        "expect": {
            "critical_path": list(cp.path), "critical_path_us": cp.duration_us,
            "phase_time_us": phase_duration_us(graph),
            "total_comm_us": ex.total_comm_us, "exposed_comm_us": ex.exposed_comm_us,
            "total_data_movement_us": ex.total_data_movement_us,
            "exposed_data_movement_us": ex.exposed_data_movement_us,
            "ecr": ex.ecr, "edmr": ex.edmr,
        },
    }


def reference_test_graphs() -> dict:
    out = {}
    # the two graphs of the reference's tests/analysis_test.py, rebuilt through its builder
    from ir import MovementDesc
    from ir.ops import COMM_ALL_GATHER, MOVEMENT_COPY

    b = EDMBuilder(default_phase="decode")
    begin = b.phase_begin("decode", 10.0)
    comp = b.compute("decode_gemm", 20.0, 40.0, op=COMPUTE_GEMM)
    end = b.phase_end("decode", 60.0)
    b.compute("unrelated_profiler_noise", 1000.0, 2000.0, op=COMPUTE_GEMM)
    b.sequence(begin, comp, end, kind=STREAM_ORDER)
    out["test_phase_boundaries"] = dump_graph(b.build())

    b = EDMBuilder(default_phase="prefill")
    begin = b.phase_begin("prefill", 0.0)
    copy = b.movement("h2d_activation", 0.0, 20.0, op=MOVEMENT_COPY,
                      movement=MovementDesc(kind="h2d_copy", backend="cuda", size_bytes=1024))
    comm = b.comm("tp_all_gather", 20.0, 30.0, op=COMM_ALL_GATHER,
                  movement=MovementDesc(kind="all_gather", backend="nccl", size_bytes=2048))
    comp = b.compute("gemm", 30.0, 100.0, op=COMPUTE_GEMM)
    end = b.phase_end("prefill", 100.0)
    b.sequence(begin, copy, comm, comp, end, kind=STREAM_ORDER)
    out["test_ecr_edmr"] = dump_graph(b.build())

    # the demo graphs, taken from the reference's example module as it stands
    spec = importlib.util.spec_from_file_location("ref_demo", os.path.join(REF, "examples", "synthetic_demo.py"))
    demo = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(demo)
    for name in ("hidden_communication", "exposed_communication", "harmful_overlap"):
        if hasattr(demo, name):
            out["demo_" + name] = dump_graph(getattr(demo, name)())
    return out


def build_candidate(params: dict, c: int, comm_op: str):
    """c GEMM chunks and c collective chunks through the reference's builder."""
    share = lambda total, i: total // c + (1 if i < total % c else 0)
    g = [share(params["gemm_total"], i) + (params["split_overhead"] if c > 1 else 0) for i in range(c)]
    m = [params["alpha"] + -(-(share(params["comm_bytes"], i) * params["beta_num"]) // params["beta_den"])
         for i in range(c)]
    comm_first = bool(params["comm_first"])
    g_t, m_t, g_end, m_end = [], [], 0, 0
    for i in range(c):
        if not comm_first:
            gs = g_end; g_end = gs + g[i]
            ms = max(g_end, m_end); m_end = ms + m[i]
        else:
            ms = m_end; m_end = ms + m[i]
            gs = max(g_end, m_end); g_end = gs + g[i]
        g_t.append((gs, gs + g[i])); m_t.append((ms, ms + m[i]))
    b = EDMBuilder(default_phase="layer")
    begin = b.phase_begin("layer", 0)
    gemms = [b.compute(f"gemm.{i}", g_t[i][0], g_t[i][1], op=COMPUTE_GEMM, stream="compute") for i in range(c)]
    comms = [b.comm(f"comm.{i}", m_t[i][0], m_t[i][1], op=comm_op, stream="comm") for i in range(c)]
    end = b.phase_end("layer", max(g_end, m_end))
    b.sequence(*gemms, kind=STREAM_ORDER)
    b.sequence(*comms, kind=STREAM_ORDER)
    for i in range(c):
        if comm_first:
            b.edge(comms[i], gemms[i], DATA_DEPENDENCY, data_id=f"chunk{i}")
        else:
            b.edge(gemms[i], comms[i], DATA_DEPENDENCY, data_id=f"chunk{i}")
    b.bind_phase(begin, end, *gemms, *comms)
    return b.build()


def selector_cases() -> list:
    cases = []
    grid = itertools.product(
        (0, 997, 8000, 123457),             # gemm_total
        (0, 4000, 1000003),                 # comm_bytes
        (0, 300),                           # alpha
        ((1, 1), (3, 7), (1000, 770)),      # beta
        (0, 100, 999),                      # split overhead
        (0, 1),                             # comm_first
    )
    cand = [1, 2, 3, 4, 8, 16]
    for gt, cb, al, (bn, bd), so, cf in grid:
        params = {"gemm_total": gt, "comm_bytes": cb, "alpha": al, "beta_num": bn, "beta_den": bd,
                  "split_overhead": so, "comm_first": cf}
        costs = []
        for c in cand:
            graph = build_candidate(params, c, "comm.all_gather" if cf else "comm.reduce_scatter")
            ex = analyze_exposure(graph)
            # [makespan, exposed comm, total comm] as the reference returned them
            costs.append([ex.critical_path_us, ex.exposed_comm_us, ex.total_comm_us])
        chosen = min(range(len(cand)), key=lambda i: costs[i][0])
        cases.append({"p": [gt, cb, al, bn, bd, so, cf], "costs": costs, "chosen": chosen})
    return cases


def trace_cases() -> list:
    from ir import trace as ref_trace
    from ir.printing import format_uops

    cases = []
    for kw in (dict(copy_us=100.0, compute_us=250.5, bytes_moved=8 << 20, device="cuda:0/sm_100", matrix=2048,
                    dtype="bfloat16", wait_us=3.25, iteration=0),
               dict(copy_us=700.125, compute_us=90.0, bytes_moved=1 << 25, device="cuda:0", matrix=4096,
                    dtype="float32", wait_us=0.0, iteration=7)):
        g = ref_trace.build_graph(**kw)
        d = dump_graph(g)
        d["args"] = kw
        d["text"] = format_uops(g)
        d["edge_attrs"] = [dict(e.attrs) for e in g.edges]
        cases.append(d)
    return cases


NSYS_PROFILE = {
    # table -> (columns, rows); times in ns
    "StringIds": (("id", "value"), [[1, "cudaLaunchKernelExC_v11060"], [2, "cudaMemcpyAsync_v3020"],
                                    [3, "void edm::tp_gemm_kernel<2, 256, false, __nv_bfloat16>(edm::LaunchParams)"],
                                    [4, "void edm::split_tf32_kernel(float const*, float*, float*, long, long, long)"]]),
    "NVTX_EVENTS": (("start", "end", "text", "globalTid"), [
        [1000, 90000, "edm.phase:trace.iter0", 77],
        [2000, 20000, "edm.kv:transfer.h2d.iter0", 77],
        [21000, 23000, "edm.event:wait.copy_done.iter0", 77],
        [24000, 60000, "edm.compute:qkv.matmul.iter0", 77],
        [100000, 180000, "edm.comm:reduce_scatter.iter1", 77],
        [181000, 260000, "edm.comm:all_gather.iter1", 77],
        [300000, 310000, "edm.compute:gemm", 78],
        [320000, 330000, "not an edm range", 78],
        [340000, None, "edm.compute:gemm.iter9", 78],
    ]),
    "CUPTI_ACTIVITY_KIND_RUNTIME": (("start", "end", "correlationId", "nameId", "globalTid"), [
        [3000, 4000, 11, 2, 77], [25000, 26000, 12, 1, 77], [27000, 28000, 13, 1, 77],
        [101000, 102000, 14, 1, 77], [182000, 183000, 15, 1, 77], [184000, 185000, 16, 2, 77],
        [301000, 302000, 17, 1, 78], [500000, 501000, 18, 1, 78],
    ]),
    "CUPTI_ACTIVITY_KIND_KERNEL": (("start", "end", "streamId", "correlationId", "demangledName"), [
        [30000, 31000, 7, 12, 4], [31500, 58000, 7, 13, 3], [103000, 175000, 7, 14, 3],
        [186000, 255000, 7, 15, 3], [303000, 309000, 7, 17, 3], [502000, 503000, 7, 18, 3],
    ]),
    "CUPTI_ACTIVITY_KIND_MEMCPY": (("start", "end", "streamId", "correlationId", "bytes", "copyKind"), [
        [5000, 19000, 13, 11, 8388608, 1], [186500, 240000, 14, 16, 16777216, 8],
    ]),
    "ENUM_CUDA_MEMCPY_OPER": (("id", "label"), [[1, "CUDA_MEMCPY_KIND_HTOD"], [8, "CUDA_MEMCPY_KIND_DTOD"]]),
}


def nsys_case() -> dict:
    import csv
    import sqlite3
    import tempfile

    from ir.nsys_export import export_nsys, parse_edm_text

    with tempfile.TemporaryDirectory() as tmp:
        db = os.path.join(tmp, "profile.sqlite")
        with sqlite3.connect(db) as conn:
            for table, (cols, rows) in NSYS_PROFILE.items():
                conn.execute(f'create table "{table}" ({", ".join(cols)})')
                conn.executemany(f'insert into "{table}" values ({", ".join("?" for _ in cols)})', rows)
        out = os.path.join(tmp, "out")
        export_nsys(db, out)
        tables = {}
        for name in ("edm_nvtx_ranges", "edm_cuda_events", "edm_iteration_summary"):
            with open(os.path.join(out, name + ".csv"), newline="") as f:
                tables[name] = list(csv.DictReader(f))
    texts = ["edm.compute:qkv.matmul.iter3", "edm.comm:reduce_scatter", "edm.phase:trace.iter12", "edm.odd",
             "plain text.iter4", "edm.kv:transfer.h2d.iter0", "edm.comm:tp_linear.ag_gemm.iter10", "edm.a:b:c.iter1"]
    return {"profile": {t: {"columns": list(c), "rows": r} for t, (c, r) in NSYS_PROFILE.items()},
            "export": tables, "grammar": [[t, list(parse_edm_text(t))] for t in texts]}


def main() -> None:
    with open(os.path.join(HERE, "trace_golden.json"), "w") as f:
        json.dump(trace_cases(), f, indent=1)
    with open(os.path.join(HERE, "nsys_golden.json"), "w") as f:
        json.dump(nsys_case(), f, indent=1)
    with open(os.path.join(HERE, "analysis_golden.json"), "w") as f:
        json.dump(reference_test_graphs(), f, indent=1)
    cases = selector_cases()
    with open(os.path.join(HERE, "selector_golden.json"), "w") as f:
        json.dump({"param_order": ["gemm_total", "comm_bytes", "alpha", "beta_num", "beta_den",
                                   "split_overhead", "comm_first"],
                   "candidates": [1, 2, 3, 4, 8, 16], "cases": cases}, f, separators=(",", ":"))
    gains = [[g, b, classify_gain(g, b)] for g, b in
             [(6.0, 100.0), (5.0, 100.0), (5.0001, 100.0), (0.0, 100.0), (-1.0, 100.0), (1.0, 0.0),
              (1e-9, 1.0), (3.0, -2.0)]]
    with open(os.path.join(HERE, "gain_golden.json"), "w") as f:
        json.dump(gains, f)
    print(f"{len(cases)} selector cases written")


if __name__ == "__main__":
    main()
