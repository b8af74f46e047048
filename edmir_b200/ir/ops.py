"""EDM-IR vocabulary: op names and dependency-edge kinds.

Same names, constants and validation behaviour as the reference vocabulary
(EDM-IR/ir/ops.py:9-54 names, :57-98 sets, :101-108 checks, :111-140 predicates).  Op names
are ``<namespace>.<name>`` strings so dumps stay readable and passes can group by prefix.
The tables below are the single source; the module-level constants (``COMPUTE_GEMM``,
``STREAM_ORDER``, ...) are generated from them.
"""
from __future__ import annotations

OpKind = str
EdgeKind = str

# namespace -> member names, in the order the reference lists them
_OP_TABLE: dict[str, tuple[str, ...]] = {
    "phase": ("begin", "end"),
    "request": ("enqueue",),
    "batch": ("form",),
    "ubatch": ("split",),
    "metadata": ("attn", "kv", "position"),
    "kv": ("lookup", "transfer", "materialize"),
    "movement": ("copy",),
    "compute": ("qkv", "attn", "mlp", "gemm", "other"),
    "comm": ("all_reduce", "all_gather", "reduce_scatter", "all_to_all", "p2p", "kv_transfer", "other"),
    "event": ("record", "wait"),
    "stream": ("yield",),
    "runtime": ("launch_gap",),
    "contention": ("resource",),
}

_EDGE_TABLE: tuple[str, ...] = (
    "stream_order",
    "data_dependency",
    "event_dependency",
    "collective_dependency",
    "scheduler_dependency",
    "kv_readiness",
    "phase_boundary",
    "resource_contention",
)


def _publish() -> tuple[frozenset, frozenset]:
    ops = []
    for ns, members in _OP_TABLE.items():
        for member in members:
            value = f"{ns}.{member}"
            globals()[f"{ns}_{member}".upper()] = value
            ops.append(value)
    for kind in _EDGE_TABLE:
        globals()[kind.upper()] = kind
    return frozenset(ops), frozenset(_EDGE_TABLE)


ALL_OPS, ALL_EDGE_KINDS = _publish()


def check_op(op: str) -> None:
    if op not in ALL_OPS:
        raise ValueError(f"unknown EDM op: {op}")


def check_edge_kind(kind: str) -> None:
    if kind not in ALL_EDGE_KINDS:
        raise ValueError(f"unknown EDM edge kind: {kind}")


def namespace(op: str) -> str:
    head, _, _ = op.partition(".")
    return head


def is_namespace(op: str, ns: str) -> bool:
    return op.startswith(f"{ns}.")


def is_comm(op: str) -> bool:
    return is_namespace(op, "comm")


def is_compute(op: str) -> bool:
    return is_namespace(op, "compute")


def is_metadata(op: str) -> bool:
    return is_namespace(op, "metadata")


def is_kv(op: str) -> bool:
    return is_namespace(op, "kv")


def is_data_movement(op: str) -> bool:
    # collectives plus the two non-collective movers
    return is_comm(op) or op in ("kv.transfer", "movement.copy")


def is_stream_overhead(op: str) -> bool:
    return is_namespace(op, "event") or op == "stream.yield"
