"""Host logic of the lowering: candidates, calibration arithmetic, selection, measured graphs."""
import pytest

from edmir_b200 import lowering, selector
from edmir_b200.calibration import Calibration, cost_params, wire_bytes
from edmir_b200.ir.analysis import analyze_exposure


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


def test_candidates_and_selection(native_lib):
    spec = lowering.TPLinearSpec("ag_gemm", 8192, 1280, 8192, 8)
    scheds = lowering.candidates(spec)
    assert [s.chunks for s in scheds] == [1, 2, 4, 8] and not scheds[0].fused and scheds[1].fused
    assert [s.chunks for s in lowering.candidates(lowering.TPLinearSpec("ag_gemm", 16, 64, 64, 8))] == [1, 2]
    assert lowering.candidates(lowering.TPLinearSpec("gemm_rs", 128, 64, 64, 1)) == [lowering.Schedule(0, 1)]
    sel = lowering.select_schedule(spec, Calibration())
    assert sel.costs[sel.chosen].makespan == min(c.makespan for c in sel.costs)
    # every candidate's native cost equals the critical path of its EDM graph
    for cost, graph in zip(sel.costs, sel.graphs):
        ex = analyze_exposure(graph)
        assert (ex.critical_path_us, ex.exposed_comm_us) == (cost.makespan, cost.exposed_comm)
    with pytest.raises(ValueError):
        lowering.TPLinearSpec("gemm_rs", 100, 64, 64, 8)
    with pytest.raises(ValueError):
        lowering.TPLinearSpec("bogus", 128, 64, 64, 8)


def test_measured_graph_reports_exposed_communication():
    spec = lowering.TPLinearSpec("gemm_rs", 8192, 8192, 1024, 8)
    g = lowering.measured_graph(spec, lowering.Schedule(2, 4), total_us=240.0, gemm_only_us=110.0, tp_rank=3)
    ex = analyze_exposure(g)
    assert ex.phase_time_us == 240.0 and ex.exposed_comm_us == pytest.approx(130.0)
    assert ex.ecr == pytest.approx(130.0 / 240.0)
    comm = [u for u in g.uops.values() if u.op == "comm.reduce_scatter"][0]
    assert comm.movement.size_bytes == 117_440_512 and comm.tp_rank == 3 and comm.attrs["schedule_index"] == 2
    assert lowering.nvtx_name("comm", "tp_linear.gemm_rs", 3) == "edm.comm:tp_linear.gemm_rs.iter3"
    single = lowering.measured_graph(lowering.TPLinearSpec("gemm_rs", 128, 64, 64, 1), lowering.Schedule(0, 1), 5.0, 5.0)
    assert analyze_exposure(single).total_comm_us == 0.0
