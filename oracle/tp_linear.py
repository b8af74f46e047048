"""float64 definitions of the fused tensor-parallel linear ops, ranks emulated in-process.

PARITY UNPINNED (see ``oracle/__init__.py``): there is no reference implementation of this
arithmetic; the nearest reference code is the one-tile ``C = A * B^T`` demo kernel with the
same K-major ("TN") operand convention (EDM-IR/ir/c-extension/mma.cu:24-25, :58).

Operand convention: ``a_r`` is ``[M, K_r]``, ``b_r`` is ``[N, K_r]``; ``x_r`` is ``[M/W, K]``,
``w_r`` is ``[N_r, K]``.  Inputs may be numpy arrays or anything ``np.asarray`` accepts.
"""
from __future__ import annotations

import numpy as np


def _f64(x) -> np.ndarray:
    return np.asarray(x, dtype=np.float64)


def gemm(a, b) -> np.ndarray:
    """``a[M,K] @ b[N,K]^T``."""
    return _f64(a) @ _f64(b).T


def gemm_all_reduce(a_shards, b_shards) -> list[np.ndarray]:
    """Row-parallel linear + all-reduce: every rank holds ``sum_r a_r @ b_r^T``."""
    total = None
    for a, b in zip(a_shards, b_shards):  # fixed rank order 0..W-1
        part = gemm(a, b)
        total = part if total is None else total + part
    return [total for _ in a_shards]


def gemm_reduce_scatter(a_shards, b_shards) -> list[np.ndarray]:
    """Row-parallel linear + reduce-scatter: rank r holds rows ``[r*M/W, (r+1)*M/W)`` of the sum."""
    world = len(a_shards)
    total = gemm_all_reduce(a_shards, b_shards)[0]
    m = total.shape[0]
    if m % world:
        raise ValueError("M must be divisible by the number of ranks")
    rows = m // world
    return [total[r * rows:(r + 1) * rows] for r in range(world)]


def all_gather_gemm(x_shards, w_shards) -> list[np.ndarray]:
    """Sequence-parallel input, column-parallel linear: rank r holds ``concat(x) @ w_r^T``."""
    x = np.concatenate([_f64(s) for s in x_shards], axis=0)
    return [x @ _f64(w).T for w in w_shards]


def rel_l2(got, want) -> float:
    got, want = _f64(got), _f64(want)
    denom = np.linalg.norm(want)
    return float(np.linalg.norm(got - want) / (denom if denom else 1.0))


def config1_inputs(world: int = 2, m: int = 256, k: int = 512, n: int = 1024, seed: int = 0):
    """The CPU-runnable reference configuration: per-rank ``A_r[m,k]`` and ``B_r[k,n]`` ~N(0,1)
    from one torch generator seeded with ``seed`` (drawn rank by rank, A before B).  Returns
    float32 numpy arrays ``(a_shards, b_kn_shards)``; note ``B`` is ``[K, N]`` here, so the
    K-major operand the kernels take is its transpose."""
    import torch

    gen = torch.Generator(device="cpu")
    gen.manual_seed(seed)
    a_shards, b_shards = [], []
    for _ in range(world):
        a_shards.append(torch.randn(m, k, generator=gen, dtype=torch.float32).numpy())
        b_shards.append(torch.randn(k, n, generator=gen, dtype=torch.float32).numpy())
    return a_shards, b_shards


def config1_output(a_shards, b_kn_shards) -> np.ndarray:
    """``sum_r A_r @ B_r`` in float64 (B given as ``[K, N]``)."""
    total = None
    for a, b in zip(a_shards, b_kn_shards):
        part = _f64(a) @ _f64(b)
        total = part if total is None else total + part
    return total
