"""ctypes binding of ``libedm_b200.so`` (declarations mirror ``include/edm_b200.h``).

There is no CPU fallback: if the library is missing or fails to load, importing the
operators raises, loudly.
"""
from __future__ import annotations

import ctypes as C
import os

from . import build as _build

EDM_OK = 0
EDM_ERR_BAD_ARG = 1
EDM_ERR_CUDA = 2
EDM_ERR_DEVICE_TIMEOUT = 3
EDM_ERR_CAPACITY = 4
EDM_ERR_NOT_SYMMETRIC = 5
EDM_ERR_UNSUPPORTED = 6

EDM_DTYPE_BF16 = 0
EDM_DTYPE_FP32 = 1

EDM_OP_GEMM = 0
EDM_OP_GEMM_RS = 1
EDM_OP_GEMM_AR = 2
EDM_OP_AG_GEMM = 3

EDM_TRANSPORT_SM = 0
EDM_TRANSPORT_COPY_ENGINE = 1
EDM_TRANSPORT_HYBRID = 2
EDM_TRANSPORT_COPY_ENGINE_STRIPED = 3

EDM_MAX_RANKS = 8
EDM_IPC_HANDLE_BYTES = 64

_ERR_NAMES = {
    EDM_ERR_BAD_ARG: "bad argument (shape, alignment or null pointer)",
    EDM_ERR_CUDA: "CUDA call failed",
    EDM_ERR_DEVICE_TIMEOUT: "device-side wait timed out",
    EDM_ERR_CAPACITY: "window, flag, workspace or heap capacity exceeded",
    EDM_ERR_NOT_SYMMETRIC: "all-reduce output is not in the symmetric heap",
    EDM_ERR_UNSUPPORTED: "unsupported shape or dtype for this operator",
}


class TpCall(C.Structure):
    """``edm_tp_call_t``."""

    _fields_ = [
        ("op", C.c_int32), ("dtype", C.c_int32),
        ("a", C.c_void_p), ("lda", C.c_int64),
        ("b", C.c_void_p), ("ldb", C.c_int64),
        ("d", C.c_void_p), ("ldd", C.c_int64),
        ("M", C.c_int64), ("N", C.c_int64), ("K", C.c_int64),
        ("chunks", C.c_int32), ("transport", C.c_int32),
        ("workspace", C.c_void_p), ("workspace_bytes", C.c_size_t),
        ("pusher_ctas", C.c_int32), ("ce_peers", C.c_int32), ("side_streams", C.c_int32),
        ("band_rows", C.c_int32), ("band_cols", C.c_int32), ("one_shot", C.c_int32),
    ]


class MoeCall(C.Structure):
    """``edm_moe_call_t``."""

    _fields_ = [
        ("tokens", C.c_int32), ("hidden", C.c_int32), ("ffn", C.c_int32), ("experts", C.c_int32),
        ("x", C.c_void_p), ("ldx", C.c_int64),
        ("logits", C.c_void_p), ("ld_logits", C.c_int64),
        ("w1", C.c_void_p), ("ldw1", C.c_int64),
        ("w2", C.c_void_p), ("ldw2", C.c_int64),
        ("out", C.c_void_p), ("ldo", C.c_int64),
        ("workspace", C.c_void_p), ("workspace_bytes", C.c_size_t),
    ]


class CostParams(C.Structure):
    """``edm_cost_params_t``."""

    _fields_ = [
        ("gemm_total", C.c_int64), ("comm_bytes", C.c_int64), ("alpha", C.c_int64),
        ("beta_num", C.c_int64), ("beta_den", C.c_int64), ("split_overhead", C.c_int64),
        ("comm_first", C.c_int32), ("reserved", C.c_int32),
    ]


class CandidateCost(C.Structure):
    """``edm_candidate_cost_t``."""

    _fields_ = [
        ("makespan", C.c_int64), ("exposed_comm", C.c_int64), ("total_comm", C.c_int64),
        ("gemm_chunk", C.c_int64), ("comm_chunk", C.c_int64),
    ]


_vp, _i64, _i32, _sz = C.c_void_p, C.c_int64, C.c_int32, C.c_size_t

# name -> (restype, argtypes); every symbol the header declares
SIGNATURES = {
    "edm_version": (C.c_int, []),
    "edm_last_cuda_error": (C.c_int, []),
    "edm_status_read": (C.c_int, [C.POINTER(C.c_uint32)]),
    "edm_status_clear": (C.c_int, []),
    "edm_status_check": (C.c_int, []),
    "edm_set_timeout_ms": (C.c_int, [C.c_uint32]),
    "edm_profile_enable": (C.c_int, [C.c_int]),
    "edm_profile_read": (C.c_int, [C.POINTER(C.c_uint64), C.c_int]),
    "edm_gemm_bf16": (C.c_int, [_vp, _i64, _vp, _i64, _vp, _i64, _i64, _i64, _i64, _vp]),
    "edm_gemm_fp32_workspace_bytes": (_sz, [_i64, _i64, _i64]),
    "edm_gemm_fp32": (C.c_int, [_vp, _i64, _vp, _i64, _vp, _i64, _i64, _i64, _i64, _vp, _sz, _vp]),
    "edm_gemm_fp32_static": (C.c_int, [_vp, _i64, _vp, _i64, _vp, _i64, _i64, _i64, _i64, _vp]),
    "edm_comm_create": (C.c_int, [C.c_int, C.c_int, _sz, _sz, C.POINTER(_vp)]),
    "edm_comm_destroy": (C.c_int, [_vp]),
    "edm_comm_export": (C.c_int, [_vp, _vp]),
    "edm_comm_import": (C.c_int, [_vp, C.c_int, _vp]),
    "edm_comm_link_local": (C.c_int, [_vp, C.c_int, _vp]),
    "edm_comm_heap_alloc": (C.c_int, [_vp, _sz, C.POINTER(_vp)]),
    "edm_comm_heap_reset": (C.c_int, [_vp]),
    "edm_comm_poison": (C.c_int, [_vp, C.c_int, _vp]),
    "edm_comm_p2p_probe": (C.c_int, [_vp, C.c_int, _sz, C.c_int, _vp]),
    "edm_tile_walk": (C.c_int, [C.c_int, C.c_int, C.c_int, _i64, _i64, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int,
                                C.POINTER(C.c_int32), _i64, C.POINTER(_i64)]),
    "edm_gemm_plan": (C.c_int, [_i64, _i64, _i64, C.c_int, C.POINTER(C.c_int32)]),
    "edm_tail_split": (C.c_int, [_i64, C.c_int, _i64, C.POINTER(C.c_int32)]),
    "edm_comm_rank": (C.c_int, [_vp]),
    "edm_comm_world": (C.c_int, [_vp]),
    "edm_tp_launch": (C.c_int, [_vp, C.POINTER(TpCall), _vp]),
    "edm_tp_launch_emulated": (C.c_int, [C.POINTER(_vp), C.POINTER(TpCall), C.c_int, _vp]),
    "edm_gemm_rs_bf16": (C.c_int, [_vp, _vp, _i64, _vp, _i64, _vp, _i64, _i64, _i64, _i64, _vp]),
    "edm_gemm_ar_bf16": (C.c_int, [_vp, _vp, _i64, _vp, _i64, _vp, _i64, _i64, _i64, _i64, _vp]),
    "edm_ag_gemm_bf16": (C.c_int, [_vp, _vp, _i64, _vp, _i64, _vp, _i64, _i64, _i64, _i64, _i32, _vp]),
    "edm_moe_window_bytes": (_sz, [_i64, _i64, _i64, C.c_int]),
    "edm_moe_workspace_bytes": (_sz, [_i64, _i64, _i64, _i64, C.c_int]),
    "edm_moe_routing_offsets": (C.c_int, [_i64, _i64, _i64, _i64, C.c_int, C.POINTER(_sz)]),
    "edm_moe_forward": (C.c_int, [_vp, C.POINTER(MoeCall), _vp]),
    "edm_moe_forward_emulated": (C.c_int, [C.POINTER(_vp), C.POINTER(MoeCall), C.c_int, _vp]),
    "edm_schedule_cost": (C.c_int, [C.POINTER(CostParams), _i32, C.POINTER(CandidateCost)]),
    "edm_graph_cost": (C.c_int, [_i32, C.POINTER(_i64), C.POINTER(_i64), C.POINTER(C.c_uint8), _i32,
                                 C.POINTER(_i32), C.POINTER(_i32), C.POINTER(_i64), C.POINTER(_i64),
                                 C.POINTER(_i32), C.POINTER(_i32)]),
    "edm_select_schedule": (C.c_int, [C.POINTER(CostParams), C.POINTER(_i32), _i32,
                                      C.POINTER(CandidateCost), C.POINTER(_i32)]),
}

_lib = None


def lib_path() -> str:
    # EDM_LIB_PATH selects another build of the same library (kernel experiments)
    return os.environ.get("EDM_LIB_PATH") or _build.LIB_PATH


def load() -> C.CDLL:
    """Load the library (once) and attach signatures.  Raises if it is not built."""
    global _lib
    if _lib is not None:
        return _lib
    path = lib_path()
    if not os.path.exists(path):
        raise RuntimeError(
            f"{path} is missing: build it with `python -m edmir_b200.build` "
            "(there is no CPU or PyTorch fallback for these operators)")
    lib = C.CDLL(path)
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)  # AttributeError here means header and library disagree
        fn.restype = res
        fn.argtypes = args
    _lib = lib
    return lib


class EdmError(RuntimeError):
    def __init__(self, code: int, where: str, detail: str = ""):
        self.code = code
        msg = f"{where}: {_ERR_NAMES.get(code, 'error')} (code {code})"
        if detail:
            msg += f" [{detail}]"
        super().__init__(msg)


def check(code: int, where: str) -> None:
    """Translate a status return into the exception the reference's callers expect:
    argument problems raise ValueError, everything else RuntimeError."""
    if code == EDM_OK:
        return
    detail = ""
    if code == EDM_ERR_CUDA:
        detail = f"cudaError={load().edm_last_cuda_error()}"
    if code in (EDM_ERR_BAD_ARG, EDM_ERR_UNSUPPORTED):
        raise ValueError(f"{where}: {_ERR_NAMES[code]} (code {code})")
    raise EdmError(code, where, detail)
