"""Single-GPU GEMM operators on torch tensors, backed by the sm_100a kernel.

Operand convention is the reference's (EDM-IR/ir/c-extension/mma.cu:24-25): ``a`` is
``[M, K]``, ``b`` is ``[N, K]`` (both K-major), the result is ``[M, N]``.  A torch
``nn.Linear`` weight is already ``[N, K]``; a ``[K, N]`` weight is prepared once with
``prepare_weight``.
"""
from __future__ import annotations

import ctypes as C

import torch

from . import _lib


def _require_cuda(*tensors: torch.Tensor) -> None:
    for t in tensors:
        if not t.is_cuda:
            raise ValueError("operands must be CUDA tensors (there is no CPU path)")


def _check_2d(t: torch.Tensor, name: str) -> None:
    if t.dim() != 2:
        raise ValueError(f"{name} must be 2-D, got shape {tuple(t.shape)}")
    if t.stride(1) != 1:
        raise ValueError(f"{name} must have unit stride along its last dimension")


def _stream() -> int:
    """Raw handle of torch's current stream on the current device (as an integer for ctypes)."""
    return torch._C._cuda_getCurrentRawStream(torch.cuda.current_device())


def prepare_weight(w_kn: torch.Tensor) -> torch.Tensor:
    """``[K, N]`` weight -> K-major ``[N, K]`` copy (done once, outside the hot path)."""
    return w_kn.t().contiguous()


_gemm_bf16 = None  # the bound C entry point (attribute lookups on a CDLL cost microseconds per call)


def gemm(a: torch.Tensor, b: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
    """``out[M,N] = a[M,K] @ b[N,K]^T`` in bf16 with fp32 accumulation."""
    global _gemm_bf16
    if not (a.is_cuda and b.is_cuda):
        raise ValueError("operands must be CUDA tensors (there is no CPU path)")
    if a.dim() != 2 or b.dim() != 2 or a.stride(1) != 1 or b.stride(1) != 1:
        _check_2d(a, "a")
        _check_2d(b, "b")
    if a.dtype != torch.bfloat16 or b.dtype != torch.bfloat16:
        raise ValueError("gemm expects bfloat16 operands")
    M, K = a.shape
    N, Kb = b.shape
    if K != Kb:
        raise ValueError(f"inner dimensions differ: a is {tuple(a.shape)}, b is {tuple(b.shape)}")
    if out is None:
        out = torch.empty((M, N), dtype=torch.bfloat16, device=a.device)
    else:
        if out.dim() != 2 or out.stride(1) != 1:
            _check_2d(out, "out")
        if out.shape[0] != M or out.shape[1] != N or out.dtype != torch.bfloat16 or not out.is_cuda:
            raise ValueError("out must be a bfloat16 CUDA tensor of shape [M, N]")
    if _gemm_bf16 is None:
        _gemm_bf16 = _lib.load().edm_gemm_bf16
    rc = _gemm_bf16(a.data_ptr(), a.stride(0), b.data_ptr(), b.stride(0), out.data_ptr(), out.stride(0), M, N, K,
                    _stream())
    if rc:
        _lib.check(rc, "edm_gemm_bf16")
    return out


def gemm_fp32_workspace_bytes(M: int, N: int, K: int) -> int:
    return int(_lib.load().edm_gemm_fp32_workspace_bytes(M, N, K))


def gemm_fp32(a: torch.Tensor, b: torch.Tensor, out: torch.Tensor | None = None,
              workspace: torch.Tensor | None = None) -> torch.Tensor:
    """``out = a @ b^T`` for fp32 tensors at fp32-level accuracy (three tf32 tensor-core
    passes over a high/low split of each operand)."""
    _require_cuda(a, b)
    _check_2d(a, "a")
    _check_2d(b, "b")
    if a.dtype != torch.float32 or b.dtype != torch.float32:
        raise ValueError("gemm_fp32 expects float32 operands")
    M, K = a.shape
    N, Kb = b.shape
    if K != Kb:
        raise ValueError(f"inner dimensions differ: a is {tuple(a.shape)}, b is {tuple(b.shape)}")
    if out is None:
        out = torch.empty((M, N), dtype=torch.float32, device=a.device)
    need = gemm_fp32_workspace_bytes(M, N, K)
    if workspace is None:
        workspace = torch.empty(need, dtype=torch.uint8, device=a.device)
    lib = _lib.load()
    rc = lib.edm_gemm_fp32(a.data_ptr(), a.stride(0), b.data_ptr(), b.stride(0), out.data_ptr(),
                           out.stride(0), M, N, K, workspace.data_ptr(),
                           workspace.numel() * workspace.element_size(), _stream())
    _lib.check(rc, "edm_gemm_fp32")
    return out


def gemm_fp32_static(a: torch.Tensor, b: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """``out = a @ b^T`` in fp32 without any allocation: for callers that can neither allocate
    device memory nor pass a workspace where they need the product.  ``out`` is required (this
    wrapper does not allocate either).  Scratch is a fixed 12 MiB array inside the library, so
    ``8 * (M*K + N*K)`` bytes must fit in 8 MiB (``EdmError`` with the capacity code otherwise),
    calls must not overlap on the GPU, and the first call on a device should precede any
    stream capture."""
    _require_cuda(a, b, out)
    _check_2d(a, "a")
    _check_2d(b, "b")
    _check_2d(out, "out")
    if a.dtype != torch.float32 or b.dtype != torch.float32 or out.dtype != torch.float32:
        raise ValueError("gemm_fp32_static expects float32 tensors")
    M, K = a.shape
    N, Kb = b.shape
    if K != Kb or tuple(out.shape) != (M, N):
        raise ValueError("shapes must be a[M,K], b[N,K], out[M,N]")
    rc = _lib.load().edm_gemm_fp32_static(a.data_ptr(), a.stride(0), b.data_ptr(), b.stride(0),
                                          out.data_ptr(), out.stride(0), M, N, K, _stream())
    _lib.check(rc, "edm_gemm_fp32_static")
    return out


def tiled_mma_bf16_bf16_bf16_fp32(a: torch.Tensor, b: torch.Tensor,
                                  c: torch.Tensor | None = None) -> torch.Tensor:
    """Drop-in for the reference's only native operator (EDM-IR/ir/c-extension/mma.cu:175,
    :267-271): ``bf16(a[M,K] @ b[N,K]^T (+ c))`` with fp32 accumulation, for any M, N, K
    rather than the single 32x32x16 tile.  Shape or dtype mismatches raise ``ValueError``
    instead of terminating the process (mma.cu:119-136)."""
    if c is None:
        return gemm(a, b)
    if c.dtype != torch.float32 or tuple(c.shape) != (a.shape[0], b.shape[0]):
        raise ValueError("c must be float32 of shape [M, N]")
    acc = gemm_fp32(a.float(), b.float())
    return (acc + c).to(torch.bfloat16)


def gemm_plan(M: int, N: int, K: int, sms: int = 148) -> dict:
    """What ``gemm`` would launch for this shape on a GPU with ``sms`` SMs: CTAs per tile, tile
    width, CTAs launched and the number of pieces split tiles are cut into along K (host only)."""
    out = (C.c_int32 * 4)()
    _lib.check(_lib.load().edm_gemm_plan(M, N, K, sms, out), "edm_gemm_plan")
    return {"cta_group": int(out[0]), "block_n": int(out[1]), "ctas": int(out[2]), "pieces": int(out[3])}


def status() -> list[int]:
    """Device status words (all zero unless a bounded device-side wait expired)."""
    buf = (C.c_uint32 * 16)()
    _lib.check(_lib.load().edm_status_read(buf), "edm_status_read")
    return list(buf)


def clear_status() -> None:
    _lib.check(_lib.load().edm_status_clear(), "edm_status_clear")


def set_timeout_ms(ms: int) -> None:
    _lib.check(_lib.load().edm_set_timeout_ms(int(ms)), "edm_set_timeout_ms")


PROFILE_SLOTS = ("producer_gather_wait", "producer_stage_wait", "mma_operand_wait", "mma_accumulator_wait",
                 "epilogue_accumulator_wait", "epilogue_staging_wait", "epilogue_landing_wait", "epilogue_total",
                 "reducer_partial_wait", "reducer_total", "push_load_wait", "push_buffer_wait", "push_publish",
                 "push_total", "kernel_total", "ctas", "epilogue_flag_fence", "epilogue_copy_issue",
                 "epilogue_accumulator_load", "push_flag_fence", "producer_flag_poll", "producer_proxy_fence",
                 "epilogue_tile_loop", "epilogue_final_notes")


def profile_enable(on: bool = True) -> None:
    """Switch the device-side per-role time accounting on or off for later launches."""
    _lib.check(_lib.load().edm_profile_enable(1 if on else 0), "edm_profile_enable")


def profile_read(reset: bool = True) -> dict:
    """Accumulated nanoseconds per role (summed over CTAs) since the last reset, by name."""
    buf = (C.c_uint64 * 24)()
    _lib.check(_lib.load().edm_profile_read(buf, 1 if reset else 0), "edm_profile_read")
    return dict(zip(PROFILE_SLOTS, (int(v) for v in buf)))
