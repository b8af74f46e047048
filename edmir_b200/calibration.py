"""Calibration tables for the schedule selector.

The reference's model leaves its parameters to measurement ("calibrated from nccl-tests, P2P
tests, and serving traces", paper/mlsys-2027/model.md:111) and ships none.  This module holds
the ones measured on B200 with this library's own kernels (``edm_comm_p2p_probe`` for the link,
the GEMM kernel for the compute rate) and turns a layer shape into the integer
``CostParams`` (nanoseconds) the selector consumes.
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass, field

from .selector import CostParams

_HERE = os.path.dirname(os.path.abspath(__file__))
DEFAULT_TABLE = os.path.join(_HERE, "calibration_b200.json")


@dataclass(frozen=True)
class Calibration:
    """Measured figures of one device class.

    ``gemm_tflops``: sustained bf16 rate of the GEMM kernel at large shapes.
    ``gemm_tile_us``: time of one wave of tiles at K=1024 (sets the floor for small shapes).
    ``link_gbs``: bytes per nanosecond a GPU pushes into peers' windows, per direction.
    ``ag_link_gbs``: what the copy engines (the default all-gather transport) deliver per direction.
    ``publish_ns``: latency from "data landed" to "flag visible" (one system-scope fence batch).
    ``launch_ns``: cost of one more kernel / collective launch on the stream.
    ``nccl_gbs``: what the unfused collective sustains per direction (for the c = 1 candidate).
    """

    name: str = "B200"
    gemm_tflops: float = 1400.0
    link_gbs: float = 660.0
    ag_link_gbs: float = 470.0
    nccl_gbs: float = 380.0
    publish_ns: int = 15_000
    launch_ns: int = 8_000
    split_ns: int = 2_000
    extra: dict = field(default_factory=dict)

    @classmethod
    def load(cls, path: str = DEFAULT_TABLE) -> "Calibration":
        with open(path) as f:
            raw = json.load(f)
        known = {k: raw[k] for k in ("name", "gemm_tflops", "link_gbs", "ag_link_gbs", "nccl_gbs", "publish_ns",
                                     "launch_ns", "split_ns") if k in raw}
        return cls(**known, extra={k: v for k, v in raw.items() if k not in known})

    def as_device_table(self) -> dict:
        """Fields for ``ir.device.install_calibration``."""
        return {"nvlink_gbs_per_dir": self.link_gbs, "bf16_tflops": self.gemm_tflops,
                "flag_publish_ns": self.publish_ns, **self.extra}


def wire_bytes(op: str, M: int, N: int, K: int, world: int, elem_bytes: int = 2) -> int:
    """Bytes per GPU per direction the exchange of one layer call moves."""
    if world <= 1:
        return 0
    if op == "ag_gemm":
        return (world - 1) * (M // world) * K * elem_bytes
    if op == "gemm_rs":
        return (world - 1) * (M // world) * N * elem_bytes
    if op == "gemm_ar":
        return 2 * (world - 1) * (M // world) * N * elem_bytes
    raise ValueError(f"unknown op {op}")


def cost_params(op: str, M: int, N: int, K: int, world: int, calib: Calibration,
                fused: bool = True) -> CostParams:
    """Integer (nanosecond) model inputs for one layer call.

    ``fused=False`` describes the unfused sequence (library GEMM, then an NCCL collective): the
    collective runs at ``nccl_gbs`` and pays a launch; ``fused=True`` describes in-kernel pushes at
    ``link_gbs`` (copy-engine deliveries at ``ag_link_gbs`` for the all-gather) where a chunk costs
    one flag publication."""
    flops = 2 * M * N * K
    gemm_ns = int(round(flops / (calib.gemm_tflops * 1e3)))  # TFLOP/s = 1e3 flop/ns
    gbs = calib.nccl_gbs if not fused else (calib.ag_link_gbs if op == "ag_gemm" else calib.link_gbs)
    # transfer ns = bytes / (GB/s) ; keep it rational: bytes * 1000 / (gbs * 1000) with integer gbs
    beta_den = max(int(round(gbs)), 1)
    return CostParams(
        gemm_total=gemm_ns,
        comm_bytes=wire_bytes(op, M, N, K, world),
        alpha=calib.publish_ns if fused else calib.launch_ns,
        beta_num=1,
        beta_den=beta_den,  # 1 GB/s = 1 byte/ns
        split_overhead=calib.split_ns,
        comm_first=1 if op == "ag_gemm" else 0,
    )
