"""Host-side arithmetic of bench.py: rooflines, wire bytes, forced schedules (no GPU)."""
import importlib.util
import os

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
spec = importlib.util.spec_from_file_location("bench", os.path.join(ROOT, "bench.py"))
bench = importlib.util.module_from_spec(spec)
spec.loader.exec_module(bench)

PEAKS = {"hbm_gbs": 6546.2, "bf16_tflops": 1635.9, "bf16_tflops_sustained": 1388.5}


def test_wire_bytes_per_direction():
    assert bench.nvlink_bytes("gemm_rs", 8192, 1024, 8192, 8) == 7 / 8 * 8192 * 8192 * 2
    assert bench.nvlink_bytes("ag_gemm", 8192, 8192, 1280, 8) == 7 / 8 * 8192 * 8192 * 2
    assert bench.nvlink_bytes("gemm_ar", 1024, 1792, 4096, 8) == 2 * 7 / 8 * 1024 * 4096 * 2
    assert bench.nvlink_bytes("gemm_rs", 8192, 1024, 8192, 1) == 0


def test_rooflines_of_the_configuration_list():
    # the table of per-shape rooflines: microseconds and the binding term
    us, bind = bench.roofline_of("ag_gemm", 8192, 8192, 1280, 8, PEAKS)
    assert bind == "nvlink" and abs(us - 130.5) < 0.1
    us, bind = bench.roofline_of("ag_gemm", 8192, 8192, 7168, 8, PEAKS)
    assert bind == "tensor" and abs(us - 588.1) < 0.1
    us, bind = bench.roofline_of("gemm_rs", 8192, 3584, 8192, 8, PEAKS)
    assert bind == "tensor" and abs(us - 294.0) < 0.1
    us, bind = bench.roofline_of("gemm_ar", 8192, 1792, 4096, 8, PEAKS)
    assert bind == "nvlink" and abs(us - 130.5) < 0.1
    us, bind = bench.roofline_of("gemm_ar", 16, 1792, 4096, 8, PEAKS)   # decode: streaming the weights binds
    assert bind == "hbm" and 2.2 < us < 2.4
    us, bind = bench.roofline_of("gemm", 8192, 14336, 4096, 1, PEAKS)
    assert bind == "tensor" and abs(us - 588.1) < 0.1


def test_forced_schedules_and_workload():
    assert bench.parse_forced("qkv=3, gate_up=12") == {"qkv": 3, "gate_up": 12}
    assert bench.parse_forced("") == {}
    cfg = bench.workload_config(8192, 8)
    assert cfg["tokens"] == 8192 and cfg["tp"] == 8 and "workload" in cfg and "model" not in cfg
    assert [op for _, op, _, _ in bench.LAYER_OPS] == ["ag_gemm", "ag_gemm", "gemm_rs", "gemm_rs"]
