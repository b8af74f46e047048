"""Calibration tables for the schedule selector.

The reference's model leaves its parameters to measurement ("calibrated from nccl-tests, P2P
tests, and serving traces", paper/mlsys-2027/model.md:111) and ships none.  This module holds
the ones measured on B200 with this library's own kernels (``edm_comm_p2p_probe`` for the link,
the GEMM kernel for the compute rate, the fused launches for the fixed costs) and turns a layer
shape into the integer ``CostParams`` (nanoseconds) the chunk-count selector consumes.
``lowering.schedule_graph`` uses the same table for the per-schedule candidate graphs.
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass, field, fields

from .selector import CostParams

_HERE = os.path.dirname(os.path.abspath(__file__))
DEFAULT_TABLE = os.path.join(_HERE, "calibration_b200.json")


@dataclass(frozen=True)
class Calibration:
    """Measured figures of one device class (rates in GB/s = bytes per nanosecond).

    ``gemm_tflops``: bf16 rate of the GEMM kernel on all ``gemm_units`` CTA pairs at large shapes.
    ``tile_ns_per_kblock`` / ``tile_fixed_ns``: time a CTA pair spends per 64-element K block of a
      256x256 tile and per tile (fill, drain, epilogue hand-over); they set the cost of short-K tiles.
    ``link_gbs``: what one GPU pushes per direction to one peer at a time (the link probe; the
      pusher CTAs of an all-gather, which serve their peers one after the other, reach it).
    ``fabric_gbs``: what it pushes per direction when every rank of an 8-rank group sends to all its
      peers at once (tile pushes of the reduce-scatter; the library collectives land there too).
    ``ce_op_ns``: what every further copy + flag write costs a copy-engine stream;
    ``push_chunk_ns``: what a chunk boundary costs the pusher warps (their pipelines drain);
    ``sm_chunk_ns``: what it costs push warps inside the GEMM CTAs (a fence on a busy SM per flag);
    ``one_shot_sync_ns``: one-shot all-reduce -- second launch, fence, flag flight, first remote load;
    ``decode_fixed_ns`` / ``decode_gbs``: decode kernel (GEMMs of up to 64 rows): launch to first MMA
    plus the cluster reduction, and the rate at which it streams the weights; ``row_block_*``: the
    same two figures for 65 to 128 rows on the general kernel;
    ``push_publish_ns``: latency from "all pusher warps have counted a chunk" to "flag visible".
    ``pusher_cta_gbs``: what one CTA that only pushes delivers (bulk copies through shared memory).
    ``ce_gbs``: what the copy engines deliver per direction with 1, 2, ... side streams when the
      shard goes to several peers (measured at 8 ranks); ``ce_gbs_one_peer``: to a single peer (2 ranks).
    ``sm_push_slowdown``: factor on the GEMM when warps inside every GEMM CTA push the shard.
    ``publish_ns``: latency from "data landed" to "flag visible" (one system-scope fence batch).
    ``launch_ns``: start-up and tear-down of one fused launch; ``ce_launch_ns``: what the stream
      operations of the copy-engine transport add per launch.
    ``skew_ns_per_rank``: what waiting for the slowest of W ranks adds to a launch that needs data
      from every peer, per additional rank.
    ``reduce_gbs``: rate at which an owner adds up partial tiles (reads of all W slots).
    ``nccl_gbs``: what the unfused library collective sustains per direction (comparison baseline).
    """

    name: str = "B200"
    gemm_tflops: float = 1450.0
    gemm_units: int = 74
    tile_ns_per_kblock: int = 100
    tile_fixed_ns: int = 1_200
    link_gbs: float = 650.0
    fabric_gbs: float = 520.0
    pusher_cta_gbs: float = 48.0
    ce_gbs: tuple = (315.0, 515.0, 515.0, 515.0)
    ce_gbs_one_peer: float = 740.0
    ce_op_ns: int = 5_000
    push_chunk_ns: int = 1_500
    sm_chunk_ns: int = 4_500
    one_shot_sync_ns: int = 8_000
    decode_fixed_ns: int = 8_000
    decode_gbs: float = 6000.0
    row_block_fixed_ns: int = 14_500
    row_block_gbs: float = 5100.0
    push_publish_ns: int = 5_000
    ag_link_gbs: float = 470.0
    sm_push_slowdown: float = 1.17
    nccl_gbs: float = 380.0
    reduce_gbs: float = 2500.0
    publish_ns: int = 15_000
    launch_ns: int = 12_000
    ce_launch_ns: int = 35_000
    skew_ns_per_rank: int = 4_000
    split_ns: int = 2_000
    extra: dict = field(default_factory=dict, compare=False, hash=False)

    @classmethod
    def load(cls, path: str = DEFAULT_TABLE) -> "Calibration":
        with open(path) as f:
            raw = json.load(f)
        names = {f.name for f in fields(cls)} - {"extra"}
        known = {k: (tuple(v) if isinstance(v, list) else v) for k, v in raw.items() if k in names}
        return cls(**known, extra={k: v for k, v in raw.items() if k not in names})

    def as_device_table(self) -> dict:
        """Fields for ``ir.device.install_calibration``."""
        return {"nvlink_gbs_per_dir": self.link_gbs, "bf16_tflops": self.gemm_tflops,
                "flag_publish_ns": self.publish_ns, **self.extra}

    def all_to_all_rate(self, world: int) -> float:
        """Per-direction rate when every rank pushes to all peers at once: the pair rate at two ranks,
        the fabric rate from eight on, linear in between."""
        if world <= 2:
            return float(self.link_gbs)
        f = min(world - 2, 6) / 6.0
        return float(self.link_gbs + f * (self.fabric_gbs - self.link_gbs))

    def ce_rate(self, side_streams: int, peers: int = 7) -> float:
        """Copy-engine rate per direction: the single-peer rate at one peer, the table (measured
        with seven peers) from seven on, linear in between (three peers: 229.6 us measured for the
        qkv all-gather at four ranks, 226 us with this interpolation)."""
        if peers <= 1:
            return float(self.ce_gbs_one_peer)
        n = min(max(side_streams, 1), len(self.ce_gbs))
        f = min(peers - 1, 6) / 6.0
        return float(self.ce_gbs_one_peer + f * (self.ce_gbs[n - 1] - self.ce_gbs_one_peer))


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


def tile_ns(K: int, calib: Calibration, elem_bytes: int = 2) -> int:
    """Time a CTA pair needs for one 256x256 tile: its K blocks plus a fixed part."""
    k_blocks = -(-K * elem_bytes // 128)
    return k_blocks * calib.tile_ns_per_kblock + calib.tile_fixed_ns


def last_wave(tiles: int, units: int, k_blocks: int) -> float:
    """What the incomplete last wave of ``tiles`` on ``units`` CTA pairs costs, in tile times: its
    tiles are cut along K into 2, 4 or 8 pieces when that many free pairs exist (the kernel's rule),
    plus the exchange of partial sums; a whole tile time otherwise."""
    rest = tiles % units
    if rest == 0:
        return 0.0
    parts = 1
    if k_blocks >= 32:
        parts = min(units // rest, k_blocks // 4, 8)
        while parts & (parts - 1):
            parts &= parts - 1
    return 1.0 if parts < 2 else 1.0 / parts + 0.15


def gemm_ns(M: int, N: int, K: int, calib: Calibration, units: int | None = None, elem_bytes: int = 2,
            plain: bool = False) -> int:
    """Time of the GEMM alone on ``units`` CTA pairs: whole waves of 256x256 tiles plus the last
    one (see ``last_wave``), but never less than the flops at the calibrated rate.  ``plain``: a
    launch without an exchange, which runs the decode kernel for up to 64 rows (the weights
    streamed once at ``decode_gbs`` plus a fixed cost)."""
    if plain and M <= 64 and -(-N // 128) <= 2 * calib.gemm_units:
        return int(calib.decode_fixed_ns + N * K * elem_bytes / calib.decode_gbs)
    if plain and M <= 128 and -(-N // 256) * 2 <= 2 * calib.gemm_units:
        # one row block on the general kernel: narrow tiles or wide pieces, weights streamed once
        return int(calib.row_block_fixed_ns + N * K * elem_bytes / calib.row_block_gbs)
    units = calib.gemm_units if units is None else max(units, 1)
    tiles = -(-M // 256) * -(-N // 256)
    k_blocks = -(-K * elem_bytes // 128)
    waves = tiles // units + last_wave(tiles, units, k_blocks)
    by_tiles = int(waves * tile_ns(K, calib, elem_bytes))
    by_rate = int(round(2 * M * N * K / (calib.gemm_tflops * 1e3) * calib.gemm_units / units))  # TFLOP/s = 1e3 flop/ns
    return max(by_tiles, by_rate)


def cost_params(op: str, M: int, N: int, K: int, world: int, calib: Calibration,
                fused: bool = True) -> CostParams:
    """Integer (nanosecond) inputs of the chunk-count model for one layer call.

    ``fused=False`` describes the unfused sequence (library GEMM, then an NCCL collective): the
    collective runs at ``nccl_gbs`` and pays a launch; ``fused=True`` describes in-kernel pushes at
    ``link_gbs`` (copy-engine deliveries at ``ag_link_gbs`` for the all-gather) where a chunk costs
    one flag publication."""
    flops = 2 * M * N * K
    total = int(round(flops / (calib.gemm_tflops * 1e3)))
    gbs = calib.nccl_gbs if not fused else (calib.ag_link_gbs if op == "ag_gemm" else calib.link_gbs)
    # transfer ns = bytes / (GB/s); kept rational: 1 GB/s = 1 byte/ns
    beta_den = max(int(round(gbs)), 1)
    return CostParams(
        gemm_total=total,
        comm_bytes=wire_bytes(op, M, N, K, world),
        alpha=calib.publish_ns if fused else calib.launch_ns,
        beta_num=1,
        beta_den=beta_den,
        split_overhead=calib.split_ns,
        comm_first=1 if op == "ag_gemm" else 0,
    )
