"""Multi-GPU layout of the verify path: replicas, no data-path collective.

Verifying one sequence touches only that sequence's block table, KV rows,
recurrent state and draft rows, and the weights are read-only, so the path
shards by sequence: every GPU holds a full model replica and a session for its
own sequences. The only exchanges are host-side: a barrier around the timed
region and the reduction of the per-rank results (a few numbers per rank).
"""
from __future__ import annotations

from dataclasses import dataclass


def sequences_of_rank(n_sequences: int, world: int, rank: int) -> list[int]:
    """Sequence ids served by `rank`: sequence s lives on GPU s mod world."""
    if world <= 0 or not 0 <= rank < world:
        raise ValueError(f"rank {rank} is outside a world of {world}")
    return list(range(rank, n_sequences, world))


def rank_of_sequence(seq: int, world: int) -> int:
    return seq % world


@dataclass
class StepTotals:
    device_ms: float      # max over ranks: the job is as slow as its slowest replica
    wall_s: float         # max over ranks
    emitted: float        # sum over ranks
    accepted: float       # sum over ranks
    ranks: int


def reduce_totals(dist, device, device_ms: float, wall_s: float, emitted: float, accepted: float) -> StepTotals:
    """Max of the times and sum of the token counts over all ranks.

    `dist` is torch.distributed (already initialised) or None for a single
    process; `device` is the torch device the backend reduces on ("cuda" for
    nccl, "cpu" for gloo).
    """
    if dist is None:
        return StepTotals(device_ms, wall_s, emitted, accepted, 1)
    import torch

    t = torch.tensor([device_ms, wall_s], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    n = torch.tensor([emitted, accepted], dtype=torch.float64, device=device)
    dist.all_reduce(n, op=dist.ReduceOp.SUM)
    return StepTotals(float(t[0]), float(t[1]), float(n[0]), float(n[1]), dist.get_world_size())


def gather_results(dist, accepted: list[int], tokens: list[list[int]], world: int, n_sequences: int):
    """Collects per-sequence results (accepted counts and emitted ids) on every rank, in sequence order.

    Each rank passes the results of sequences_of_rank(n_sequences, world, rank), in that order.
    """
    if dist is None:
        return accepted, tokens
    parts: list = [None] * world
    dist.all_gather_object(parts, (accepted, tokens))
    acc_all: list = [None] * n_sequences
    tok_all: list = [None] * n_sequences
    for r, (acc_r, tok_r) in enumerate(parts):
        for i, s in enumerate(sequences_of_rank(n_sequences, world, r)):
            acc_all[s], tok_all[s] = acc_r[i], tok_r[i]
    return acc_all, tok_all
