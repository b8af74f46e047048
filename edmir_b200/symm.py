"""Symmetric memory contexts and the fused tensor-parallel linear operators.

One ``SymmetricContext`` per rank owns a device allocation with the same layout on every rank
(flag words, a double-buffered window for tiles / shards in flight, a bump heap for tensors
peers store into).  Peers map each other's allocation through CUDA IPC; the handles travel
over ``torch.distributed`` (any backend), which is used for bootstrap only -- the data path is
in-kernel stores over NVLink.

``EmulatedGroup`` builds W contexts on ONE device and runs the W ranks' kernels as a single
cooperative launch, each rank on 1/W of the SMs.  That is how the multi-rank protocol is
checked on a single GPU (kernels that wait on each other may not be separate launches there).
"""
from __future__ import annotations

import ctypes as C
from typing import Sequence

import torch

from . import _lib
from .linear import _check_2d, _require_cuda, _stream
from .schedule import Schedule

_OPS = {"gemm_rs": _lib.EDM_OP_GEMM_RS, "gemm_ar": _lib.EDM_OP_GEMM_AR, "ag_gemm": _lib.EDM_OP_AG_GEMM}
_TRANSPORTS = {"sm": _lib.EDM_TRANSPORT_SM, "ce": _lib.EDM_TRANSPORT_COPY_ENGINE,
               "hybrid": _lib.EDM_TRANSPORT_HYBRID, "cs": _lib.EDM_TRANSPORT_COPY_ENGINE_STRIPED}
_DTYPES = {torch.bfloat16: _lib.EDM_DTYPE_BF16, torch.float32: _lib.EDM_DTYPE_FP32}


class _DevicePtr:
    """Exposes a raw device range through ``__cuda_array_interface__`` (as bytes)."""

    def __init__(self, ptr: int, nbytes: int, owner):
        self._owner = owner  # keeps the context alive while views exist
        self.__cuda_array_interface__ = {
            "shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 3, "strides": None,
        }


def default_window_bytes(max_m: int, max_n: int, max_k: int, world: int) -> int:
    """Window size (both parities) that fits GEMM+RS/AR of [max_m, max_n] and AG of [max_m, max_k]."""
    tiles = -(-max_m // 128) * -(-max_n // 256)
    slots = (-(-tiles // world) + 1) * world * 128 * 256 * 4
    gather = max_m * max_k * 2
    return 2 * max(slots, gather)


class SymmetricContext:
    def __init__(self, rank: int, world: int, window_bytes: int, heap_bytes: int, device=None):
        if device is None:
            device = torch.cuda.current_device()
        self.device = torch.device("cuda", device) if isinstance(device, int) else torch.device(device)
        self.rank, self.world = rank, world
        self._lib = _lib.load()
        handle = C.c_void_p()
        with torch.cuda.device(self.device):
            _lib.check(self._lib.edm_comm_create(rank, world, window_bytes, heap_bytes, C.byref(handle)),
                       "edm_comm_create")
        self._h = handle
        self._workspace: torch.Tensor | None = None
        self._calls: dict = {}
        self._tp_launch = self._lib.edm_tp_launch  # bound once: attribute lookups on a CDLL are slow

    # ---------------------------------------------------------------- setup
    @classmethod
    def create(cls, window_bytes: int, heap_bytes: int, group=None) -> "SymmetricContext":
        """Collective over ``group``: allocate, exchange IPC handles, map every peer."""
        import torch.distributed as dist

        rank, world = dist.get_rank(group), dist.get_world_size(group)
        ctx = cls(rank, world, window_bytes, heap_bytes)
        if world > 1:
            buf = C.create_string_buffer(_lib.EDM_IPC_HANDLE_BYTES)
            _lib.check(ctx._lib.edm_comm_export(ctx._h, buf), "edm_comm_export")
            handles: list = [None] * world
            dist.all_gather_object(handles, bytes(buf.raw), group=group)
            for peer, raw in enumerate(handles):
                if peer == rank:
                    continue
                _lib.check(ctx._lib.edm_comm_import(ctx._h, peer, C.create_string_buffer(raw, len(raw))),
                           "edm_comm_import")
            dist.barrier(group=group)
        return ctx

    def close(self) -> None:
        if self._h is not None and self._h.value:
            self._lib.edm_comm_destroy(self._h)
            self._h = None

    # ---------------------------------------------------------------- symmetric tensors
    def empty(self, shape: Sequence[int], dtype: torch.dtype) -> torch.Tensor:
        """Tensor in the symmetric heap (peers can store into it).  Every rank must allocate
        the same sequence of shapes."""
        n = 1
        for s in shape:
            n *= int(s)
        nbytes = n * torch.empty((), dtype=dtype).element_size()
        ptr = C.c_void_p()
        _lib.check(self._lib.edm_comm_heap_alloc(self._h, max(nbytes, 1), C.byref(ptr)), "edm_comm_heap_alloc")
        raw = torch.as_tensor(_DevicePtr(ptr.value, max(nbytes, 1), self), device=self.device)
        return raw[:nbytes].view(dtype).view(*shape)

    def reset_heap(self) -> None:
        _lib.check(self._lib.edm_comm_heap_reset(self._h), "edm_comm_heap_reset")

    def poison(self, byte_value: int = 0xFF) -> None:
        """Fill this rank's window (tile slots / gather buffers, both halves) with ``byte_value``
        on the current stream; 0xFF makes every element a NaN, so a read of data that has not
        arrived yet becomes visible in the result.  Call it only between launches."""
        _lib.check(self._lib.edm_comm_poison(self._h, byte_value, _stream()), "edm_comm_poison")

    def p2p_probe(self, peer: int, nbytes: int, mode: int = 0) -> None:
        """Launch one link-probe copy of ``nbytes`` into ``peer``'s window (time it with events)."""
        _lib.check(self._lib.edm_comm_p2p_probe(self._h, peer, nbytes, mode, _stream()), "edm_comm_p2p_probe")

    # ---------------------------------------------------------------- launches
    def _call(self, op: str, a, b, out, schedule: Schedule | None = None) -> "_lib.TpCall":
        """Validated ``edm_tp_call_t`` for one launch.  Built once per distinct (operands, schedule)
        and kept: a steady-state launch is a dictionary lookup plus the library call."""
        sched = schedule or Schedule()
        key = (op, a.data_ptr(), b.data_ptr(), out.data_ptr(), a.shape, b.shape, out.shape, a.stride(0),
               b.stride(0), out.stride(0), a.dtype, sched)
        call = self._calls.get(key)
        if call is not None:
            return call
        _require_cuda(a, b, out)
        for t, n in ((a, "a"), (b, "b"), (out, "out")):
            _check_2d(t, n)
        if a.dtype != b.dtype or a.dtype != out.dtype or a.dtype not in _DTYPES:
            raise ValueError("operands and output must share a dtype of bfloat16 or float32")
        N, K = b.shape
        if a.shape[1] != K:
            raise ValueError("inner dimensions differ")
        M = a.shape[0] * self.world if op == "ag_gemm" else a.shape[0]
        want = (M // self.world, N) if op == "gemm_rs" else (M, N)
        if tuple(out.shape) != want:
            raise ValueError(f"out must have shape {want} for {op}, got {tuple(out.shape)}")
        if not sched.fused:
            raise ValueError("an unfused schedule is not a launch of the fused kernel")
        call = _lib.TpCall()
        call.op, call.dtype = _OPS[op], _DTYPES[a.dtype]
        call.a, call.lda = a.data_ptr(), a.stride(0)
        call.b, call.ldb = b.data_ptr(), b.stride(0)
        call.d, call.ldd = out.data_ptr(), out.stride(0)
        call.M, call.N, call.K = M, N, K
        call.chunks = sched.chunks
        call.transport = _TRANSPORTS[sched.transport]
        call.pusher_ctas, call.ce_peers, call.side_streams = sched.pusher_ctas, sched.ce_peers, sched.side_streams
        call.band_rows, call.band_cols = sched.band_rows, sched.band_cols
        if sched.one_shot and op != "gemm_ar":
            raise ValueError("one_shot is a schedule of gemm_ar")
        call.one_shot = 1 if sched.one_shot else 0
        if a.dtype == torch.float32:
            need = int(self._lib.edm_gemm_fp32_workspace_bytes(a.shape[0], N, K))
            if self._workspace is None or self._workspace.numel() < need:
                self._workspace = torch.empty(need, dtype=torch.uint8, device=a.device)
                self._calls.clear()  # cached calls point at the old workspace
            call.workspace, call.workspace_bytes = self._workspace.data_ptr(), self._workspace.numel()
        if len(self._calls) >= 256:
            self._calls.clear()
        self._calls[key] = call
        return call

    def _launch(self, op: str, a, b, out, schedule: Schedule | None = None):
        call = self._call(op, a, b, out, schedule)
        rc = self._tp_launch(self._h, C.byref(call), _stream())
        if rc:
            _lib.check(rc, f"edm_tp_launch({op})")
        return out

    def gemm_rs(self, a: torch.Tensor, b: torch.Tensor, out: torch.Tensor | None = None,
                schedule: Schedule | None = None) -> torch.Tensor:
        """Row-parallel linear + reduce-scatter: ``out[M/W, N]`` = rows ``rank*M/W ..`` of
        ``sum_r a_r @ b_r^T``."""
        if out is None:
            out = torch.empty((a.shape[0] // self.world, b.shape[0]), dtype=a.dtype, device=a.device)
        return self._launch("gemm_rs", a, b, out, schedule)

    def gemm_ar(self, a: torch.Tensor, b: torch.Tensor, out: torch.Tensor | None = None,
                schedule: Schedule | None = None) -> torch.Tensor:
        """Row-parallel linear + all-reduce: every rank ends with ``sum_r a_r @ b_r^T``.  ``out``
        must come from ``self.empty`` (peers store reduced tiles straight into it), except with a
        ``one_shot`` schedule -- this rank's GEMM into the window, then one kernel in which every
        rank adds up all partials itself -- which writes any device tensor."""
        if out is None:
            if schedule is not None and schedule.one_shot:
                out = torch.empty((a.shape[0], b.shape[0]), dtype=a.dtype, device=a.device)
            else:
                out = self.empty((a.shape[0], b.shape[0]), a.dtype)
        return self._launch("gemm_ar", a, b, out, schedule)

    def ag_gemm(self, x: torch.Tensor, w: torch.Tensor, out: torch.Tensor | None = None,
                chunks: int | None = None, transport: str | None = None,
                schedule: Schedule | None = None) -> torch.Tensor:
        """All-gather of the token-sharded ``x[M/W, K]`` fused with ``out[M, N/W] = X @ w^T``.

        ``schedule`` says how the shards travel (see ``schedule.Schedule``): pushed by the kernel
        -- by warps inside every GEMM CTA, or by ``pusher_ctas`` CTAs that do nothing else --,
        delivered by copy engines on the library's side streams, or both.  ``chunks`` and
        ``transport`` alone are shorthand for ``Schedule(chunks=..., transport=...)``; the default
        is copy engines, one chunk."""
        if schedule is None:
            schedule = Schedule(chunks=chunks or 1, transport=transport or "ce")
        elif chunks is not None or transport is not None:
            raise ValueError("pass either a schedule or chunks/transport, not both")
        if out is None:
            out = torch.empty((x.shape[0] * self.world, w.shape[0]), dtype=x.dtype, device=x.device)
        return self._launch("ag_gemm", x, w, out, schedule)


class EmulatedGroup:
    """W ranks on one device; ``run`` executes all of them in one cooperative launch."""

    def __init__(self, world: int, window_bytes: int, heap_bytes: int, device=None):
        if not 1 <= world <= 4:
            raise ValueError("an emulated group holds 1 to 4 ranks")
        self.world = world
        self.ranks = [SymmetricContext(r, world, window_bytes, heap_bytes, device) for r in range(world)]
        lib = self.ranks[0]._lib
        for a in self.ranks:
            for b in self.ranks:
                if a is not b:
                    _lib.check(lib.edm_comm_link_local(a._h, b.rank, b._h), "edm_comm_link_local")

    def run(self, op: str, a_list, b_list, out_list, chunks: int | None = None, transport: str | None = None,
            schedule: Schedule | None = None):
        if schedule is None:
            schedule = Schedule(chunks=chunks or 1, transport=transport or "sm")
        calls = (_lib.TpCall * self.world)()
        for r, ctx in enumerate(self.ranks):
            calls[r] = ctx._call(op, a_list[r], b_list[r], out_list[r], schedule)
        handles = (C.c_void_p * self.world)(*[ctx._h for ctx in self.ranks])
        lib = self.ranks[0]._lib
        _lib.check(lib.edm_tp_launch_emulated(handles, calls, self.world, _stream()),
                   f"edm_tp_launch_emulated({op})")
        return out_list

    def poison(self, byte_value: int = 0xFF) -> None:
        for ctx in self.ranks:
            ctx.poison(byte_value)

    def close(self) -> None:
        for ctx in self.ranks:
            ctx.close()


def tile_walk(op: str, rank: int, world: int, M: int, N: int, tile_m: int = 256, tile_n: int = 256,
              band_rows: int = 0, units: int = 74, band_cols: int = 0) -> list[tuple[int, int, int, int]]:
    """Order in which rank ``rank`` computes the output tiles of an ``[M, N]`` launch, as
    ``(row_block, col_block, owner, index_among_owner's_tiles)``; holes of the all-reduce walk
    have row and column -1.  Evaluated on the host by the same code the kernel runs."""
    lib = _lib.load()
    code = _lib.EDM_OP_GEMM if op == "gemm" else _OPS[op]
    n = C.c_int64()
    _lib.check(lib.edm_tile_walk(code, rank, world, M, N, tile_m, tile_n, band_rows, band_cols, units, None, 0, C.byref(n)),
               "edm_tile_walk")
    buf = (C.c_int32 * (4 * n.value))()
    _lib.check(lib.edm_tile_walk(code, rank, world, M, N, tile_m, tile_n, band_rows, band_cols, units, buf, n.value,
                                 C.byref(n)), "edm_tile_walk")
    return [tuple(buf[4 * i:4 * i + 4]) for i in range(n.value)]


def tail_split(tiles: int, units: int, k_blocks: int) -> tuple[int, int, int]:
    """``(whole_tiles, split_tiles, pieces)``: how a launch of ``tiles`` tiles on ``units`` CTAs (or
    pairs) cuts the tiles of an incomplete last wave along K (``pieces == 1``: not at all)."""
    out = (C.c_int32 * 3)()
    _lib.check(_lib.load().edm_tail_split(tiles, units, k_blocks, out), "edm_tail_split")
    return int(out[0]), int(out[1]), int(out[2])
