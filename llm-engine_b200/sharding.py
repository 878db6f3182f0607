"""Multi-GPU sharding of the paged-KV path: by sequence, with no data-path exchange.

Every GPU owns a block pool and a set of sequences; a step on one GPU touches only that
GPU's memory, so the only cross-rank traffic is the benchmark's own bookkeeping (a barrier
and two scalar reductions).  llm-engine itself is single-GPU
(src/model/cuda/cuda_model.cu:239); this is the harness around it.
"""
from __future__ import annotations

import numpy as np


def rank_seed(base_seed: int, rank: int) -> int:
    """Weak scaling: every rank draws its own batch of the same shape."""
    return base_seed + 1000 * rank


def deal_sequences(ctx_lengths, world: int, rank: int, policy: str = "balanced") -> np.ndarray:
    """Strong scaling: indices of the sequences of ONE batch that `rank` owns.

    round_robin: sequence i goes to rank i % world.
    balanced:    longest-first greedy on context length, so every rank reads about the same
                 number of K/V bytes (contexts in one batch can differ by 64x).
    Every sequence is owned by exactly one rank."""
    L = np.asarray(ctx_lengths, dtype=np.int64)
    if world <= 1:
        return np.arange(L.size)
    if policy == "round_robin":
        return np.arange(rank, L.size, world)
    if policy != "balanced":
        raise ValueError(policy)
    load = np.zeros(world, dtype=np.int64)
    owner = np.empty(L.size, dtype=np.int64)
    for i in np.argsort(-L, kind="stable"):
        r = int(np.argmin(load))
        owner[i] = r
        load[r] += L[i] + 1
    return np.nonzero(owner == rank)[0]


def reduce_step(tokens_this_rank: float, ms_this_rank: float, dist=None, device=None):
    """(total tokens over ranks, max time over ranks): whole-job throughput = tokens / time."""
    if dist is None or not dist.is_initialized() or dist.get_world_size() == 1:
        return float(tokens_this_rank), float(ms_this_rank)
    import torch
    t = torch.tensor([tokens_this_rank], dtype=torch.float64, device=device)
    m = torch.tensor([ms_this_rank], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.SUM)
    dist.all_reduce(m, op=dist.ReduceOp.MAX)
    return float(t.item()), float(m.item())
