"""float64 definition of the expert-parallel MoE layer, ranks emulated in-process.
TEST INFRASTRUCTURE (see ``oracle/__init__.py``).

PARITY UNPINNED: the reference contains no MoE code; it only names the pieces
(``comm.all_to_all``, EDM-IR/ir/ops.py:35; the ``ep_rank`` tag, EDM-IR/ir/uop.py:106) and plans a
dispatch/combine study (experiments/deepep-vs-nccl-ep-h100/README.md:19-57).  The definition here
follows the layer semantics of the configuration list: top-2 routing from the router logits,
per-expert ``down(silu(gate(x)) * up(x))``, outputs combined with the softmax of the two selected
logits.

Conventions shared with the device code (they make the integer results comparable bit for bit):
* top-2: the largest logit, then the largest of the rest; equal logits go to the lower expert index;
* every (token, choice) pair of a source rank gets a slot in its expert's buffer: pairs are
  ordered by (source rank, token, choice), so the row of a pair is
  ``sum(counts of lower ranks for that expert) + (number of earlier pairs of this rank for it)``;
* expert ``e`` lives on rank ``e // (E / W)``.
"""
from __future__ import annotations

import numpy as np


def top2(logits) -> tuple[np.ndarray, np.ndarray]:
    """``(idx[T,2] int32, weights[T,2] float64)``: the two selected experts per token and the
    softmax over their two logits."""
    lg = np.asarray(logits, dtype=np.float64)
    T, E = lg.shape
    order = np.lexsort((np.arange(E)[None, :].repeat(T, 0), -lg), axis=1)  # by logit desc, index asc
    idx = order[:, :2].astype(np.int32)
    sel = np.take_along_axis(lg, idx.astype(np.int64), axis=1)
    ex = np.exp(sel - sel.max(axis=1, keepdims=True))
    return idx, ex / ex.sum(axis=1, keepdims=True)


def slots(idx_per_rank, experts: int):
    """Row of every (token, choice) pair inside its expert's buffer, and the rows per expert.
    ``idx_per_rank``: list over source ranks of ``idx[T,2]``.  Returns ``(rows_per_rank, counts)``
    with ``rows_per_rank[r][t, k]`` the row and ``counts[r, e]`` the pairs rank r sends to e."""
    W = len(idx_per_rank)
    counts = np.zeros((W, experts), dtype=np.int64)
    local = []
    for r, idx in enumerate(idx_per_rank):
        flat = np.asarray(idx).reshape(-1)  # (token, choice) order
        pos = np.zeros(flat.shape[0], dtype=np.int64)
        for e in range(experts):
            hit = flat == e
            pos[hit] = np.arange(hit.sum())
            counts[r, e] = hit.sum()
        local.append(pos.reshape(np.asarray(idx).shape))
    base = np.cumsum(counts, axis=0) - counts  # pairs of lower ranks
    rows = [local[r] + base[r][np.asarray(idx_per_rank[r])] for r in range(W)]
    return rows, counts


def silu(x):
    return x / (1.0 + np.exp(-x))


def expert_ffn(x, w1, w2):
    """``down(silu(gate(x)) * up(x))`` with ``w1 = [gate; up]`` of shape ``[2F, H]`` and ``w2 [H, F]``
    (both K-major, like every weight of this package)."""
    x = np.asarray(x, dtype=np.float64)
    w1 = np.asarray(w1, dtype=np.float64)
    F = w1.shape[0] // 2
    y = x @ w1.T
    return (silu(y[:, :F]) * y[:, F:]) @ np.asarray(w2, dtype=np.float64).T


def moe_layer(x_per_rank, logits_per_rank, w1_per_expert, w2_per_expert):
    """Every rank's output ``[T, H]``: ``sum_k weight[t,k] * expert_ffn_{idx[t,k]}(x[t])``."""
    outs = []
    for x, lg in zip(x_per_rank, logits_per_rank):
        x = np.asarray(x, dtype=np.float64)
        idx, wts = top2(lg)
        out = np.zeros_like(x)
        for e in range(len(w1_per_expert)):
            for k in range(2):
                hit = idx[:, k] == e
                if hit.any():
                    out[hit] += wts[hit, k:k + 1] * expert_ffn(x[hit], w1_per_expert[e], w2_per_expert[e])
        outs.append(out)
    return outs


def router_logits(tokens: int, experts: int, seed: int, bias_seed: int = 99):
    """Router logits ~N(0,1) plus a per-expert bias ~N(0,0.5) shared by all ranks (load skew)."""
    import torch

    g = torch.Generator(device="cpu").manual_seed(seed)
    gb = torch.Generator(device="cpu").manual_seed(bias_seed)
    bias = torch.randn(experts, generator=gb, dtype=torch.float32) * 0.5
    return (torch.randn(tokens, experts, generator=g, dtype=torch.float32) + bias).numpy()
