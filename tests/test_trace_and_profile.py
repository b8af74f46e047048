"""The overlap probe's graph builder and the profiler import, against fixtures produced by running
the reference (tests/golden/make_golden.py): ``trace_golden.json`` holds the graphs the
reference's ``ir/trace.py:build_graph`` returns, ``nsys_golden.json`` a small profile and what the
reference's ``ir/nsys_export.py:export_nsys`` makes of it."""
import json
import os
import sqlite3

import pytest

from edmir_b200 import lowering, nsys_import
from edmir_b200.ir import trace
from edmir_b200.ir.analysis import analyze_critical_path, analyze_exposure, phase_duration_us
from edmir_b200.ir.printing import format_uops


def _load(golden_dir, name):
    with open(os.path.join(golden_dir, name)) as f:
        return json.load(f)


def test_probe_graph_equals_the_reference_graph(golden_dir):
    for case in _load(golden_dir, "trace_golden.json"):
        g = trace.build_graph(**case["args"])
        nodes = [{"id": u.id, "op": u.op, "name": u.name, "start": u.start_us, "end": u.end_us, "phase": u.phase}
                 for u in g.uops.values()]
        assert nodes == case["nodes"]
        assert [[e.src, e.dst, e.kind] for e in g.edges] == case["edges"]
        assert [dict(e.attrs) for e in g.edges] == case["edge_attrs"]
        assert format_uops(g) == case["text"]
        cp, ex, want = analyze_critical_path(g), analyze_exposure(g), case["expect"]
        assert list(cp.path) == want["critical_path"] and cp.duration_us == want["critical_path_us"]
        assert phase_duration_us(g) == want["phase_time_us"]
        assert (ex.exposed_data_movement_us, ex.edmr) == (want["exposed_data_movement_us"], want["edmr"])


def test_probe_command_line_matches_the_reference_flags():
    args = trace.parse_args(["--matrix", "512", "--warmup", "1", "--iters", "3", "--dtype", "float32",
                             "--print-uops", "all"])
    assert (args.matrix, args.warmup, args.iters, args.dtype, args.print_uops) == (512, 1, 3, "float32", "all")
    d = trace.parse_args([])
    assert (d.matrix, d.warmup, d.iters, d.dtype, d.print_uops) == (2048, 2, 1, "float16", "last")
    with pytest.raises(SystemExit):
        trace.main(["--iters", "0"])


def _make_profile(tmp_path, golden):
    db = tmp_path / "profile.sqlite"
    with sqlite3.connect(db) as conn:
        for table, spec in golden["profile"].items():
            cols = spec["columns"]
            conn.execute(f'create table "{table}" ({", ".join(cols)})')
            conn.executemany(f'insert into "{table}" values ({", ".join("?" for _ in cols)})', spec["rows"])
    return db


def test_nvtx_grammar(golden_dir):
    golden = _load(golden_dir, "nsys_golden.json")
    for text, (op, iteration) in golden["grammar"]:
        assert nsys_import.parse_edm_text(text) == (op, iteration), text
    # what the launches emit parses back to op names
    assert nsys_import.parse_edm_text(lowering.nvtx_name("comm", "reduce_scatter", 4)) == ("comm.reduce_scatter", 4)
    assert nsys_import.parse_edm_text(lowering.nvtx_name("compute", "gemm")) == ("compute.gemm", None)


def test_profile_import_matches_the_reference_export(tmp_path, golden_dir):
    golden = _load(golden_dir, "nsys_golden.json")
    ranges, loose, origin = nsys_import.read_profile(_make_profile(tmp_path, golden))
    us = lambda ns: f"{(ns - origin) / 1000.0:.3f}"
    got_ranges = [{"iteration": "" if r.iteration is None else str(r.iteration), "op": r.op, "text": r.text,
                   "start_us": us(r.start_ns), "end_us": us(r.end_ns), "dur_us": f"{r.dur_ns / 1000.0:.3f}",
                   "global_tid": str(r.global_tid)} for r in ranges]
    assert got_ranges == golden["export"]["edm_nvtx_ranges"]
    # every GPU event with the range the reference attaches it to
    got_events = sorted(
        [(e.start_ns, e.kind, e.correlation_id, r.op, r.text) for r in ranges for e in r.events] +
        [(e.start_ns, e.kind, e.correlation_id, "", "") for e in loose])
    want_events = sorted((int(round(float(row["start_us"]) * 1000)) + origin, row["kind"], int(row["correlation_id"]),
                          row["edm_op"], row["edm_text"]) for row in golden["export"]["edm_cuda_events"])
    assert got_events == want_events
    names = {e.name for r in ranges for e in r.events if e.kind == "kernel"}
    assert any("tp_gemm_kernel" in n for n in names)


def test_profile_becomes_an_edm_graph(tmp_path, golden_dir):
    golden = _load(golden_dir, "nsys_golden.json")
    db = _make_profile(tmp_path, golden)
    g = nsys_import.profile_to_graph(db, iteration=1)
    body = [u for u in g.uops.values() if not u.op.startswith("phase.")]
    assert [u.op for u in body] == ["comm.reduce_scatter", "comm.all_gather"]
    rs, ag = body
    assert (rs.start_us, rs.end_us) == (102.0, 174.0)           # the kernel's span, from the profile's origin
    assert (ag.start_us, ag.end_us) == (185.0, 254.0)           # kernel 186-255 us and copy 186.5-240 us
    assert ag.movement.size_bytes == 16777216 and ag.attrs["gpu_events"] == 2
    ex = analyze_exposure(g)
    assert ex.total_comm_us == pytest.approx(72.0 + 69.0) and ex.phase_time_us == pytest.approx(254.0 - 102.0)
    whole = nsys_import.profile_to_graph(db)
    ops_seen = [u.op for u in whole.uops.values()]
    assert "compute.qkv" in ops_seen and "kv.transfer" in ops_seen and "compute.gemm" in ops_seen
    assert nsys_import.known_op("compute.qkv.matmul") == "compute.qkv" and nsys_import.known_op("x.y") == "compute.other"
    assert nsys_import.profile_to_graph(db, iteration=99).uops == {}
    with pytest.raises(FileNotFoundError):
        nsys_import.read_profile(tmp_path / "absent.sqlite")
