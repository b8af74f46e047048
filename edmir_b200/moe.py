"""Expert-parallel mixture-of-experts layer on the symmetric windows of ``symm``.

``moe_forward`` runs one layer call on this rank (every rank of the context makes the same
call): top-2 routing from the router logits, dispatch of the selected token rows to the ranks
that hold their experts, ``down(silu(gate(x)) * up(x))`` per expert as two grouped GEMMs, return
of the rows and their combination weighted by the softmax of the two selected logits.  The
exchanges are stores into the peers' windows with flag words, as in the fused linears; nothing
goes through ``torch.distributed``.  ``moe_forward_emulated`` runs the ranks of a
``symm.EmulatedGroup`` on one device.

The reference has no MoE code; the op names this layer reports in graphs are its
``comm.all_to_all`` (EDM-IR/ir/ops.py:35) and the ``ep_rank`` tag (EDM-IR/ir/uop.py:106).

Weights: ``w1`` is ``[E_local * 2F, H]`` (per local expert the F gate rows, then the F up rows),
``w2`` is ``[E_local * H, F]``; expert ``e`` lives on rank ``e // E_local``.
"""
from __future__ import annotations

import ctypes as C

import torch

from . import _lib
from .ir import EDMBuilder, EDMGraph, MovementDesc
from .ir import ops as irops
from .linear import _check_2d, _require_cuda, _stream


def window_bytes(tokens: int, hidden: int, experts: int, world: int) -> int:
    """Window size (both halves) a context needs for this layer shape."""
    n = int(_lib.load().edm_moe_window_bytes(tokens, hidden, experts, world))
    if n == 0:
        raise ValueError("unsupported MoE shape (experts <= 64 and divisible by world; hidden % 8 == 0)")
    return n


def workspace_bytes(tokens: int, hidden: int, ffn: int, experts: int, world: int) -> int:
    n = int(_lib.load().edm_moe_workspace_bytes(tokens, hidden, ffn, experts, world))
    if n == 0:
        raise ValueError("unsupported MoE shape")
    return n


class MoEWorkspace:
    """Scratch of one rank for one layer shape: routing results, row-block tables, activations."""

    def __init__(self, tokens: int, hidden: int, ffn: int, experts: int, world: int, device=None):
        self.shape = (tokens, hidden, ffn, experts, world)
        self.buf = torch.empty(workspace_bytes(*self.shape), dtype=torch.uint8,
                               device=device if device is not None else torch.cuda.current_device())
        off = (C.c_size_t * 3)()
        _lib.check(_lib.load().edm_moe_routing_offsets(*self.shape, off), "edm_moe_routing_offsets")
        self._off = [int(o) for o in off]

    def _view(self, i: int, dtype):
        tokens = self.shape[0]
        return self.buf[self._off[i]:self._off[i] + tokens * 2 * 4].view(dtype).view(tokens, 2)

    @property
    def topk_idx(self) -> torch.Tensor:
        """Selected experts of the last call, int32 ``[T, 2]``."""
        return self._view(0, torch.int32)

    @property
    def topk_weight(self) -> torch.Tensor:
        return self._view(1, torch.float32)

    @property
    def slot(self) -> torch.Tensor:
        """Position of every (token, choice) among this rank's rows for the same expert."""
        return self._view(2, torch.int32)


def _call(ctx, ws: MoEWorkspace, x, logits, w1, w2, out) -> "_lib.MoeCall":
    _require_cuda(x, logits, w1, w2, out)
    for t, n in ((x, "x"), (logits, "logits"), (w1, "w1"), (w2, "w2"), (out, "out")):
        _check_2d(t, n)
    T, H = x.shape
    E = logits.shape[1]
    F = w2.shape[1]
    if x.dtype != torch.bfloat16 or w1.dtype != torch.bfloat16 or w2.dtype != torch.bfloat16 or out.dtype != torch.bfloat16:
        raise ValueError("x, w1, w2 and out must be bfloat16")
    if logits.dtype != torch.float32 or logits.shape[0] != T:
        raise ValueError("logits must be float32 [T, E]")
    if E % ctx.world:
        raise ValueError("the number of experts must be divisible by the number of ranks")
    e_local = E // ctx.world
    if tuple(w1.shape) != (e_local * 2 * F, H) or tuple(w2.shape) != (e_local * H, F) or tuple(out.shape) != (T, H):
        raise ValueError("shapes must be w1 [E_local*2F, H], w2 [E_local*H, F], out [T, H]")
    if ws.shape != (T, H, F, E, ctx.world):
        raise ValueError(f"workspace was made for {ws.shape}, the call is {(T, H, F, E, ctx.world)}")
    call = _lib.MoeCall()
    call.tokens, call.hidden, call.ffn, call.experts = T, H, F, E
    call.x, call.ldx = x.data_ptr(), x.stride(0)
    call.logits, call.ld_logits = logits.data_ptr(), logits.stride(0)
    call.w1, call.ldw1 = w1.data_ptr(), w1.stride(0)
    call.w2, call.ldw2 = w2.data_ptr(), w2.stride(0)
    call.out, call.ldo = out.data_ptr(), out.stride(0)
    call.workspace, call.workspace_bytes = ws.buf.data_ptr(), ws.buf.numel()
    return call


def moe_forward(ctx, ws: MoEWorkspace, x, logits, w1, w2, out=None) -> torch.Tensor:
    """One layer call on this rank of ``ctx`` (a ``symm.SymmetricContext``)."""
    if out is None:
        out = torch.empty_like(x)
    call = _call(ctx, ws, x, logits, w1, w2, out)
    _lib.check(ctx._lib.edm_moe_forward(ctx._h, C.byref(call), _stream()), "edm_moe_forward")
    return out


def moe_forward_emulated(group, ws_list, x_list, logits_list, w1_list, w2_list, out_list):
    """All ranks of a ``symm.EmulatedGroup`` on one device; every stage is one launch over all ranks."""
    n = group.world
    calls = (_lib.MoeCall * n)()
    for r, ctx in enumerate(group.ranks):
        calls[r] = _call(ctx, ws_list[r], x_list[r], logits_list[r], w1_list[r], w2_list[r], out_list[r])
    handles = (C.c_void_p * n)(*[ctx._h for ctx in group.ranks])
    lib = group.ranks[0]._lib
    _lib.check(lib.edm_moe_forward_emulated(handles, calls, n, _stream()), "edm_moe_forward_emulated")
    return out_list


def layer_flops(tokens_per_rank: int, hidden: int, ffn: int, top_k: int = 2) -> float:
    """Flops one rank performs when the load is uniform: every rank processes ``tokens * top_k``
    rows through gate, up and down projections."""
    return 2.0 * tokens_per_rank * top_k * hidden * ffn * 3


def dispatch_bytes(tokens_per_rank: int, hidden: int, world: int, top_k: int = 2) -> float:
    """Bytes per GPU and direction of the dispatch (and again of the combine) at uniform load."""
    return tokens_per_rank * top_k * hidden * 2.0 * (world - 1) / world


def measured_graph(tokens: int, hidden: int, ffn: int, experts: int, world: int, total_us: float,
                   ep_rank: int = 0, device: str | None = None) -> EDMGraph:
    """One measured layer call as an EDM graph: ``comm.all_to_all`` (dispatch), ``compute.mlp``
    (the experts), ``comm.all_to_all`` (combine), tagged with ``ep_rank``.  Only the total is
    measured from outside; the split follows the byte and flop counts at the calibrated rates'
    ratio, and is marked as such in the node attributes."""
    nbytes = int(dispatch_bytes(tokens, hidden, world))
    b = EDMBuilder(default_phase="moe_layer")
    begin = b.phase_begin("moe_layer", 0.0)
    wire_us = nbytes / 650e3 if world > 1 else 0.0       # 650 GB/s
    comp_us = layer_flops(tokens, hidden, ffn) / 1.45e9   # 1450 TFLOP/s
    scale = total_us / max(2 * wire_us + comp_us, 1e-9)
    t1, t2 = wire_us * scale, (wire_us + comp_us) * scale
    common = dict(ep_rank=ep_rank, device=device, attrs={"experts": experts, "split": "apportioned, not measured"})
    mv = lambda: MovementDesc(kind="all_to_all", backend="nvlink-p2p", size_bytes=nbytes, group="ep",
                              group_ranks=tuple(range(world)))
    d = b.comm("dispatch", 0.0, t1, op=irops.COMM_ALL_TO_ALL, stream="nvlink", movement=mv(), **common)
    m = b.compute("experts", t1, t2, op=irops.COMPUTE_MLP, stream="compute", **common)
    c = b.comm("combine", t2, total_us, op=irops.COMM_ALL_TO_ALL, stream="nvlink", movement=mv(), **common)
    end = b.phase_end("moe_layer", total_us)
    b.data_edge(d, m, "tokens")
    b.data_edge(m, c, "expert_out")
    b.bind_phase(begin, end, d, m, c)
    return b.build()
