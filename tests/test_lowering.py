"""Host logic of the lowering: candidates, calibration arithmetic, selection, measured graphs."""
import random

import pytest

from edmir_b200 import lowering, selector
from edmir_b200.calibration import Calibration, cost_params, gemm_ns, wire_bytes
from edmir_b200.ir.analysis import analyze_exposure
from edmir_b200.schedule import Schedule
from oracle import cost_model


def test_wire_bytes_match_the_layer_formulas():
    # per GPU per direction, bf16: RS (W-1)/W*M*N*2, AG (W-1)/W*M*K*2, AR twice RS
    assert wire_bytes("gemm_rs", 8192, 8192, 3584, 8) == 117_440_512
    assert wire_bytes("ag_gemm", 8192, 1280, 8192, 8) == 117_440_512
    assert wire_bytes("gemm_ar", 8192, 4096, 1792, 8) == 2 * 7 * 1024 * 4096 * 2
    assert wire_bytes("gemm_rs", 8192, 8192, 3584, 1) == 0
    with pytest.raises(ValueError):
        wire_bytes("nonsense", 1, 1, 1, 2)


def test_cost_params_are_integers_from_the_table():
    calib = Calibration(gemm_tflops=1000.0, link_gbs=500.0, nccl_gbs=250.0, publish_ns=10_000, launch_ns=5_000,
                        split_ns=1_000)
    fused = cost_params("gemm_rs", 1024, 1024, 1024, 2, calib, fused=True)
    unfused = cost_params("gemm_rs", 1024, 1024, 1024, 2, calib, fused=False)
    assert fused.gemm_total == round(2 * 1024**3 / 1e6) and fused.comm_bytes == 512 * 1024 * 2
    assert (fused.alpha, fused.beta_den, unfused.alpha, unfused.beta_den) == (10_000, 500, 5_000, 250)
    assert cost_params("ag_gemm", 1024, 1024, 1024, 2, calib).comm_first == 1
    assert all(isinstance(v, int) for v in selector.describe(fused).values())
    # the GEMM term: whole waves of tiles with a fixed part per tile, never below the flop rate
    assert gemm_ns(8192, 8192, 1024, calib) >= round(2 * 8192 * 8192 * 1024 / 1e6)
    assert gemm_ns(8192, 8192, 1024, calib, units=37) > gemm_ns(8192, 8192, 1024, calib, units=74)
    assert hash(Calibration.load()) == hash(Calibration.load())   # usable as a cache key


def test_candidates():
    spec = lowering.TPLinearSpec("ag_gemm", 8192, 1280, 8192, 8)
    scheds = lowering.candidates(spec)
    assert [s.index for s in scheds] == list(range(len(scheds)))
    assert not scheds[0].fused and all(s.fused for s in scheds[1:])
    # a fused one-chunk schedule exists and is not the unfused one
    assert any(s.fused and s.chunks == 1 for s in scheds)
    assert {s.transport for s in scheds[1:]} == {"sm", "ce", "hybrid"}
    assert {s.pusher_ctas for s in scheds if s.transport == "sm"} == {0, 8, 16, 24, 32}
    # two-row shards cannot be cut into more than two chunks; two ranks have no far peers
    tiny = lowering.candidates(lowering.TPLinearSpec("ag_gemm", 16, 64, 64, 8))
    assert max(s.chunks for s in tiny) == 2
    assert all(s.transport != "hybrid" for s in lowering.candidates(lowering.TPLinearSpec("ag_gemm", 512, 64, 64, 2)))
    # reduce-scatter / all-reduce: unfused and the one fused schedule; one rank: nothing to choose
    assert [s.fused for s in lowering.candidates(lowering.TPLinearSpec("gemm_rs", 8192, 8192, 1024, 8))] == [False, True]
    assert lowering.candidates(lowering.TPLinearSpec("gemm_rs", 128, 64, 64, 1)) == [Schedule(index=0)]
    # decode-sized all-reduces can also run one-shot; large ones and reduce-scatters cannot
    small = lowering.candidates(lowering.TPLinearSpec("gemm_ar", 16, 4096, 1792, 8))
    assert [s.label() for s in small] == ["unfused", "sm-p0-c1", "oneshot"] and small[2].one_shot
    assert not any(s.one_shot for s in lowering.candidates(lowering.TPLinearSpec("gemm_ar", 8192, 4096, 1792, 8)))
    assert not any(s.one_shot for s in lowering.candidates(lowering.TPLinearSpec("gemm_rs", 64, 4096, 1792, 8)))
    assert not any(s.one_shot for s in lowering.candidates(lowering.TPLinearSpec("gemm_ar", 16, 36, 64, 2)))
    with pytest.raises(ValueError):
        lowering.TPLinearSpec("gemm_rs", 100, 64, 64, 8)
    with pytest.raises(ValueError):
        lowering.TPLinearSpec("bogus", 128, 64, 64, 8)
    with pytest.raises(ValueError):
        Schedule(transport="carrier-pigeon")


@pytest.mark.parametrize("op,M,N,K,world", [("ag_gemm", 8192, 1280, 8192, 8), ("ag_gemm", 8192, 7168, 8192, 2),
                                            ("gemm_rs", 8192, 8192, 1024, 8), ("gemm_ar", 128, 4096, 1792, 4),
                                            ("gemm_ar", 1024, 4096, 1792, 8)])
def test_selection_is_the_native_critical_path_of_each_candidate_graph(native_lib, op, M, N, K, world):
    spec = lowering.TPLinearSpec(op, M, N, K, world)
    sel = lowering.select_schedule(spec, Calibration())
    fused = [i for i, s in enumerate(sel.schedules) if s.fused]
    assert sel.chosen in fused
    assert sel.costs[sel.chosen].makespan == min(sel.costs[i].makespan for i in fused)
    assert sel.predicted_us == sel.costs[sel.chosen].makespan / 1e3
    # every candidate's native cost equals what the analysis pass reports for its EDM graph
    for cost, graph in zip(sel.costs, sel.graphs):
        ex = analyze_exposure(graph)
        assert (ex.critical_path_us, ex.exposed_comm_us, ex.total_comm_us) == (cost.makespan, cost.exposed_comm, cost.total_comm)
    # allowing the library collective can only lower the chosen cost
    loose = lowering.select_schedule(spec, Calibration(), allow_unfused=True)
    assert loose.costs[loose.chosen].makespan <= sel.costs[sel.chosen].makespan


def test_model_prefers_pushers_where_the_link_binds_and_few_where_compute_binds(native_lib):
    calib = Calibration()
    qkv = lowering.select_schedule(lowering.TPLinearSpec("ag_gemm", 8192, 1280, 8192, 8), calib).schedule
    gate_up = lowering.select_schedule(lowering.TPLinearSpec("ag_gemm", 8192, 7168, 8192, 8), calib).schedule
    assert qkv.transport in ("sm", "hybrid") and qkv.pusher_ctas >= 8
    assert gate_up.pusher_ctas <= 8


def test_native_graph_cost_matches_the_pinned_oracle_on_random_graphs(native_lib):
    # random DAGs with integer durations: the native evaluator against the restatement that is
    # pinned to the reference's analyze_critical_path / analyze_exposure
    import ctypes as C

    rng = random.Random(7)
    for _ in range(200):
        n = rng.randint(1, 24)
        nodes = []
        for i in range(n):
            start = rng.randint(0, 50)
            nodes.append({"id": i, "op": rng.choice(["compute.gemm", "comm.all_gather", "comm.p2p", "phase.begin"]),
                          "start": start, "end": start + rng.randint(0, 30)})
        order = list(range(n))
        rng.shuffle(order)   # a random topological order, so ids and dependencies are unrelated
        edges = [(order[a], order[b]) for a in range(n) for b in range(a + 1, n) if rng.random() < 0.2]
        rng.shuffle(edges)
        path, dur = cost_model.critical_path(nodes, edges)
        exposed = sum(nd["end"] - nd["start"] for nd in nodes if nd["id"] in path and nd["op"].startswith("comm."))
        d = (C.c_int64 * n)(*[nd["end"] - nd["start"] for nd in nodes])
        e = (C.c_int64 * n)(*[nd["end"] for nd in nodes])
        c = (C.c_uint8 * n)(*[1 if nd["op"].startswith("comm.") else 0 for nd in nodes])
        m = len(edges)
        src = (C.c_int32 * max(m, 1))(*[a for a, _ in edges])
        dst = (C.c_int32 * max(m, 1))(*[b for _, b in edges])
        mk, ex, plen = C.c_int64(), C.c_int64(), C.c_int32(n)
        buf = (C.c_int32 * n)()
        assert native_lib.edm_graph_cost(n, d, e, c, m, src, dst, C.byref(mk), C.byref(ex), buf, C.byref(plen)) == 0
        assert (mk.value, ex.value, list(buf[:plen.value])) == (dur, exposed, path)
    # a cycle is refused
    d = (C.c_int64 * 2)(1, 1); e = (C.c_int64 * 2)(1, 1); c = (C.c_uint8 * 2)(0, 0)
    src = (C.c_int32 * 2)(0, 1); dst = (C.c_int32 * 2)(1, 0)
    mk, ex = C.c_int64(), C.c_int64()
    assert native_lib.edm_graph_cost(2, d, e, c, 2, src, dst, C.byref(mk), C.byref(ex), None, None) == 1


def test_measured_graph_reports_exposed_communication():
    spec = lowering.TPLinearSpec("gemm_rs", 8192, 8192, 1024, 8)
    g = lowering.measured_graph(spec, Schedule(index=1), total_us=240.0, gemm_only_us=110.0, tp_rank=3)
    ex = analyze_exposure(g)
    assert ex.phase_time_us == 240.0 and ex.exposed_comm_us == pytest.approx(130.0)
    assert ex.ecr == pytest.approx(130.0 / 240.0)
    comm = [u for u in g.uops.values() if u.op == "comm.reduce_scatter"][0]
    assert comm.movement.size_bytes == 117_440_512 and comm.tp_rank == 3 and comm.attrs["schedule_index"] == 1
    assert lowering.nvtx_name("comm", "tp_linear.gemm_rs", 3) == "edm.comm:tp_linear.gemm_rs.iter3"
    assert lowering.launch_range_name(spec, 2) == "edm.comm:reduce_scatter.iter2"
    one = lowering.TPLinearSpec("gemm_rs", 128, 64, 64, 1)
    assert lowering.launch_range_name(one) == "edm.compute:gemm"
    single = lowering.measured_graph(one, Schedule(), 5.0, 5.0)
    assert analyze_exposure(single).total_comm_us == 0.0


def test_example_scripts_compile():
    # the examples need GPUs (most of them several) to run; here they only have to parse and import-check
    import glob
    import os
    import py_compile

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    scripts = sorted(glob.glob(os.path.join(root, "examples", "*.py")))
    assert len(scripts) >= 6
    for path in scripts:
        py_compile.compile(path, doraise=True)
