"""The re-implemented EDM-IR package behaves like the reference's: same results on the graphs the
reference computed (golden JSON), same exceptions, same device-registry behaviour.  The cases
mirror EDM-IR/tests/analysis_test.py and EDM-IR/tests/device_test.py."""
import json
import os

import pytest

from edmir_b200 import ir
from edmir_b200.ir import ops
from edmir_b200.ir.analysis import analyze_exposure, classify_gain, phase_duration_us
from edmir_b200.ir.device import (DeviceRegistry, DeviceSpec, arch_from_compute_capability, detect_device,
                                  format_device_spec, get_device_spec, install_calibration,
                                  known_device_specs, match_device_spec, register_device_spec,
                                  supported_nvidia_specs)
from edmir_b200.ir.printing import format_critical_path, format_summary, format_uops


def _rebuild(g):
    graph = ir.EDMGraph()
    for n in g["nodes"]:
        graph.add_uop(ir.UOp(id=n["id"], op=n["op"], name=n["name"], start_us=n["start"], end_us=n["end"],
                             phase=n["phase"]))
    for s, d, k in g["edges"]:
        graph.add_edge(s, d, k)
    return graph


def test_exported_names():
    for name in ("EDMBuilder", "EDMGraph", "Edge", "UOp", "MovementDesc", "TensorDesc", "DataRef",
                 "analyze_critical_path", "analyze_exposure", "analyze_overlap", "DeviceSpec",
                 "DeviceRegistry", "register_device_spec", "detect_device", "buffer_ref", "param_ref",
                 "const_ref", "DATA_BUFFER", "DEFAULT_REGISTRY", "CriticalPathResult"):
        assert hasattr(ir, name) and name in ir.__all__, name
    assert len(ops.ALL_OPS) == 29 and len(ops.ALL_EDGE_KINDS) == 8
    assert ops.COMPUTE_GEMM == "compute.gemm" and ops.COMM_REDUCE_SCATTER == "comm.reduce_scatter"


def test_matches_reference_outputs(golden_dir):
    with open(os.path.join(golden_dir, "analysis_golden.json")) as f:
        data = json.load(f)
    for name, g in data.items():
        graph = _rebuild(g)
        ex = analyze_exposure(graph)
        want = g["expect"]
        assert list(ex.critical_path) == want["critical_path"], name
        assert ex.critical_path_us == want["critical_path_us"]
        assert ex.phase_time_us == want["phase_time_us"]
        assert ex.total_comm_us == want["total_comm_us"]
        assert ex.exposed_comm_us == want["exposed_comm_us"]
        assert ex.total_data_movement_us == want["total_data_movement_us"]
        assert ex.exposed_data_movement_us == want["exposed_data_movement_us"]
        assert ex.ecr == want["ecr"] and ex.edmr == want["edmr"]
        assert "critical_path_us=" in format_critical_path(graph)
        assert format_summary(graph).startswith("phase_us=")
        assert len(format_uops(graph, highlight=ex.critical_path).splitlines()) == len(graph.uops)


def test_gain_labels(golden_dir):
    with open(os.path.join(golden_dir, "gain_golden.json")) as f:
        for gain, base, label in json.load(f):
            assert classify_gain(gain, base) == label


def test_phase_duration_prefers_phase_boundaries():
    b = ir.EDMBuilder(default_phase="decode")
    begin = b.phase_begin("decode", 10.0)
    comp = b.compute("decode_gemm", 20.0, 40.0, op=ops.COMPUTE_GEMM)
    end = b.phase_end("decode", 60.0)
    b.compute("unrelated_profiler_noise", 1000.0, 2000.0, op=ops.COMPUTE_GEMM)
    b.sequence(begin, comp, end, kind=ops.STREAM_ORDER)
    assert phase_duration_us(b.build()) == 50.0


def test_ecr_and_edmr_are_split():
    b = ir.EDMBuilder(default_phase="prefill")
    begin = b.phase_begin("prefill", 0.0)
    copy = b.movement("h2d_activation", 0.0, 20.0, op=ops.MOVEMENT_COPY,
                      movement=ir.MovementDesc(kind="h2d_copy", backend="cuda", size_bytes=1024))
    comm = b.comm("tp_all_gather", 20.0, 30.0, op=ops.COMM_ALL_GATHER,
                  movement=ir.MovementDesc(kind="all_gather", backend="nccl", size_bytes=2048))
    comp = b.compute("gemm", 30.0, 100.0, op=ops.COMPUTE_GEMM)
    end = b.phase_end("prefill", 100.0)
    b.sequence(begin, copy, comm, comp, end, kind=ops.STREAM_ORDER)
    ex = analyze_exposure(b.build())
    assert (ex.phase_time_us, ex.total_comm_us, ex.exposed_comm_us) == (100.0, 10.0, 10.0)
    assert (ex.total_data_movement_us, ex.exposed_data_movement_us) == (30.0, 30.0)
    assert ex.ecr == pytest.approx(0.1) and ex.edmr == pytest.approx(0.3)


def test_error_behaviour():
    with pytest.raises(ValueError):
        ops.check_op("compute.nonsense")
    with pytest.raises(ValueError):
        ops.check_edge_kind("nonsense")
    with pytest.raises(ValueError):
        ir.UOp(id=0, op=ops.COMPUTE_GEMM, name="x", start_us=2.0, end_us=1.0)
    with pytest.raises(ValueError):
        ir.DataRef("d", "read", kind="nonsense")
    g = ir.EDMGraph()
    g.add_uop(ir.UOp(id=0, op=ops.COMPUTE_GEMM, name="x", start_us=0.0, end_us=1.0))
    with pytest.raises(ValueError):
        g.add_uop(ir.UOp(id=0, op=ops.COMPUTE_GEMM, name="y", start_us=0.0, end_us=1.0))
    with pytest.raises(KeyError):
        g.add_edge(0, 7, ops.STREAM_ORDER)
    g.add_uop(ir.UOp(id=1, op=ops.COMPUTE_GEMM, name="y", start_us=0.0, end_us=1.0))
    g.add_edge(0, 1, ops.STREAM_ORDER)
    g.add_edge(1, 0, ops.STREAM_ORDER)
    with pytest.raises(ValueError):
        g.topological_order()
    assert ir.analyze_critical_path(ir.EDMGraph()).path == ()


def test_uop_attr_and_builder_defaults():
    b = ir.EDMBuilder(default_phase="p")
    u = b.comm("c", 0.0, 1.0, tp_rank=3, attrs={"chunk": 2, "stream": "ignored"})
    assert u.id == 0 and u.op == ops.COMM_ALL_GATHER and u.phase == "p"
    assert u.attr("tp_rank") == 3 and u.attr("chunk") == 2 and u.attr("missing", 7) == 7
    assert u.attr("stream") == "ignored"  # unset schema field falls back to attrs
    assert u.dur_us == 1.0 and u.op_class == "comm"
    w = b.wait_event("w", 5.0)
    assert (w.start_us, w.end_us) == (5.0, 5.0)
    assert ir.buffer_ref("x").kind == ir.DATA_BUFFER and ir.param_ref("w").kind == ir.DATA_PARAM
    assert ir.const_ref("c", location="smem").location == "smem"


def test_builtin_specs_and_registry():
    h100 = get_device_spec("NVIDIA H100 80GB HBM3")
    assert (h100.name, h100.arch, h100.compute_capability, h100.cuda_arch) == ("H100", "Hopper", (9, 0), "sm90")
    assert h100.supports_tma and h100.supports_wgmma and h100.supports_fp8
    rtx = get_device_spec("GeForce RTX 5090")
    assert (rtx.name, rtx.arch, rtx.cuda_arch, rtx.supports_nvlink) == ("RTX 5090", "Blackwell", "sm120", False)
    b200 = get_device_spec("NVIDIA B200")
    assert b200.compute_capability == (10, 0) and get_device_spec("sm100") is b200
    assert not b200.supports_wgmma and b200.attrs["tensor_core_isa"] == "tcgen05"

    reg = DeviceRegistry()
    spec = DeviceSpec("Test GPU", arch="Hopper", compute_capability=(9, 0))
    reg.register(spec, aliases=("test-gpu", "sm90-test"))
    assert reg.get("NVIDIA Test GPU") is spec and reg.match("sm90-test dev0") is spec
    with pytest.raises(ValueError):
        reg.register(DeviceSpec("Test GPU"))
    newer = DeviceSpec("Test GPU", arch="Blackwell", compute_capability=(10, 0))
    reg.register(newer, replace_existing=True)
    assert reg.get("test gpu") is newer
    with pytest.raises(KeyError):
        reg.get("no such device")

    assert arch_from_compute_capability((9, 0)) == "Hopper"
    assert arch_from_compute_capability((10, 0)) == arch_from_compute_capability((12, 0)) == "Blackwell"
    assert arch_from_compute_capability((8, 0)) is None and arch_from_compute_capability(None) is None
    names = {s.name for s in known_device_specs()}
    assert {"H100", "B200", "RTX 5090"} <= names
    assert all(s.arch in {"Hopper", "Blackwell"} for s in supported_nvidia_specs())
    own = DeviceRegistry()
    got = register_device_spec(DeviceSpec("Unit Test GPU", arch="Hopper"), aliases=("unit-test-gpu",), registry=own)
    assert match_device_spec("unit test gpu", registry=own) is got
    d = detect_device()
    assert d is None or isinstance(d, DeviceSpec)
    assert format_device_spec(None) == "device=<none>" and "name=B200" in format_device_spec(b200)


def test_install_calibration_fills_measured_fields():
    reg = DeviceRegistry()
    reg.register(DeviceSpec("B200", arch="Blackwell", compute_capability=(10, 0), memory_kind="HBM"))
    spec = install_calibration({"hbm_gbs": 6546.2, "nvlink_gbs_per_dir": 770.0, "bf16_tflops": 1635.9}, registry=reg)
    assert spec.hbm_bandwidth_gbps == 6546.2 and spec.nvlink_bandwidth_gbps == 770.0
    assert spec.attrs["bf16_tflops"] == 1635.9 and reg.get("b200") is spec
