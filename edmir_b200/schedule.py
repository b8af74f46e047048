"""The schedule of one fused tensor-parallel launch: everything the selector may choose.

A ``Schedule`` is what ``lowering.select_schedule`` returns and what the operators in ``symm``
pass to the library through ``edm_tp_call_t`` (``include/edm_b200.h``); nothing on that path
reads environment variables.  The reference has no schedules (it only observes executions,
paper/mlsys-2027/edm-ir.md:7); the knobs follow the terms of its overlap model
(paper/mlsys-2027/model.md:161-168): ``chunks`` is the split granularity, ``pusher_ctas`` the
resources taken from compute ("new contention"), ``transport`` who moves the bytes.
"""
from __future__ import annotations

from dataclasses import dataclass, replace

TRANSPORTS = ("sm", "ce", "hybrid", "cs")


@dataclass(frozen=True)
class Schedule:
    index: int = 0
    fused: bool = True       # False: GEMM kernel, then a separate library collective (comparison baseline)
    chunks: int = 1          # all-gather: flag granularity, chunks per shard
    transport: str = "sm"    # all-gather: "sm" kernel pushes, "ce" copy engines (a stream per peer), "hybrid" both,
                             # "cs" copy engines striped (a stream per chunk: all engines on one peer at a time)
    pusher_ctas: int = 0     # all-gather, kernel pushes: CTAs that only push (0: push warps in every GEMM CTA)
    ce_peers: int = 0        # all-gather, hybrid: how many of the farthest peers the copy engines serve
    side_streams: int = 2    # all-gather, copy engines: streams the copies are spread over
    band_rows: int = 0       # tile walk: row blocks per band (0: library default)
    band_cols: int = 0       # tile walk: column blocks per super-tile (0: whole width)
    one_shot: bool = False   # all-reduce: plain GEMM, then every rank adds up all partials itself (decode-sized M)

    def __post_init__(self) -> None:
        if self.transport not in TRANSPORTS:
            raise ValueError(f"transport must be one of {TRANSPORTS}")
        if self.chunks < 1 or self.pusher_ctas < 0 or self.ce_peers < 0 or not 0 <= self.side_streams <= 4:
            raise ValueError("chunks >= 1, pusher_ctas >= 0, ce_peers >= 0, side_streams in 0..4")

    def with_index(self, index: int) -> "Schedule":
        return replace(self, index=index)

    def label(self) -> str:
        if not self.fused:
            return "unfused"
        if self.one_shot:
            return "oneshot"
        bits = [self.transport]
        if self.transport not in ("ce", "cs"):
            bits.append(f"p{self.pusher_ctas}")
        if self.transport == "hybrid":
            bits.append(f"ce{self.ce_peers}")
        if self.transport != "sm":
            bits.append(f"s{self.side_streams}")
        bits.append(f"c{self.chunks}")
        return "-".join(bits)


DEFAULT = Schedule()
