"""Data-parallel sharding of a packed batch over the GPUs of one box.

The reference is single-GPU. Sequences never attend across `cu_seqlens` boundaries
and the weights are read-only, so the batch shards by document: one model replica per
rank, each rank encodes a cost-balanced group of whole sequences, and one gather of
the output embeddings at the end is the only communication. No layer is sharded.

The cost of a sequence follows the FLOP model of the forward: per token
L*(8H^2 + 6HI) multiply-adds for the four projections plus 4H per attended
(query, key) pair, where a global layer attends s^2 pairs and a local layer
s^2 (s <= 65) or 129 s - 4160 pairs
(benchmarks/packed_attention_dispatch_bench.py:63-66).
"""
from __future__ import annotations

from dataclasses import dataclass

import numpy as np
import torch
from torch import Tensor


def local_pairs(s: np.ndarray, half_window: int = 64) -> np.ndarray:
    """Attended (query, key) pairs of one sequence in a sliding-window layer."""
    s = np.asarray(s, dtype=np.float64)
    w = 2 * half_window + 1
    band = w * s - half_window * (half_window + 1)
    return np.where(s <= half_window + 1, s * s, band)


def sequence_costs(lengths, *, hidden: int, intermediate: int, n_layers: int, n_global: int,
                   half_window: int = 64) -> np.ndarray:
    """Model FLOPs (multiply-add = 2) of encoding each sequence."""
    s = np.asarray(lengths, dtype=np.float64)
    gemm = s * n_layers * (8.0 * hidden * hidden + 6.0 * hidden * intermediate)
    attn = 4.0 * hidden * (n_global * s * s + (n_layers - n_global) * local_pairs(s, half_window))
    return gemm + attn


def costs_for_model(lengths, model) -> np.ndarray:
    cfg = model.config
    n_layers = len(model.layers)
    n_global = sum(1 for l in model.layers if getattr(l, "attention_type", "") == "full_attention")
    if n_global == 0:
        n_global = (n_layers + 2) // 3
    return sequence_costs(lengths, hidden=cfg.hidden_size, intermediate=cfg.intermediate_size,
                          n_layers=n_layers, n_global=n_global,
                          half_window=int(cfg.local_attention) // 2)


def balance(costs, world_size: int) -> list[np.ndarray]:
    """Longest-processing-time greedy: heaviest sequence first into the lightest rank.

    Returns, per rank, the indices of its sequences (in descending-cost order, ties by
    index), deterministic on every rank. Makespan is within 4/3 of optimal.
    """
    costs = np.asarray(costs, dtype=np.float64)
    order = np.lexsort((np.arange(costs.size), -costs))
    loads = np.zeros(world_size, dtype=np.float64)
    groups: list[list[int]] = [[] for _ in range(world_size)]
    for i in order:
        r = int(np.argmin(loads))  # first minimum: deterministic
        groups[r].append(int(i))
        loads[r] += costs[i]
    return [np.asarray(g, dtype=np.int64) for g in groups]


@dataclass
class ShardPlan:
    """Who encodes what, and how to put the gathered rows back in global packed order."""

    world_size: int
    lengths: np.ndarray                 # [N] all sequence lengths, original order
    groups: list[np.ndarray]            # per rank: indices into the original order
    tokens_per_rank: np.ndarray         # [world]
    max_tokens: int                     # rows of each padded shard in the gather
    restore_index: np.ndarray           # [T_total] flat row in the [world, max_tokens] gather

    @property
    def total_tokens(self) -> int:
        return int(self.lengths.sum())


def plan_shards(lengths, world_size: int, costs=None) -> ShardPlan:
    lengths = np.asarray(lengths, dtype=np.int64)
    if lengths.size == 0 or (lengths <= 0).any():
        raise ValueError("plan_shards needs at least one sequence and positive lengths")
    costs = lengths.astype(np.float64) if costs is None else np.asarray(costs, dtype=np.float64)
    groups = balance(costs, world_size)
    tokens = np.asarray([int(lengths[g].sum()) for g in groups], dtype=np.int64)
    max_tokens = int(max(1, tokens.max()))
    starts = np.concatenate(([0], np.cumsum(lengths)))  # global packed offsets
    restore = np.empty(int(starts[-1]), dtype=np.int64)
    for r, g in enumerate(groups):
        local = 0
        for i in g:
            n = int(lengths[i])
            restore[starts[i]:starts[i] + n] = r * max_tokens + local + np.arange(n)
            local += n
    return ShardPlan(world_size, lengths, groups, tokens, max_tokens, restore)


def local_batch(plan: ShardPlan, rank: int, sequences):
    """This rank's sequences (a list of 1-D id tensors), in the plan's order."""
    return [sequences[int(i)] for i in plan.groups[rank]]


def gather_embeddings(local_out: Tensor, plan: ShardPlan, group=None) -> Tensor:
    """All ranks receive the `[T_total, H]` embeddings in the original packed order.

    Each rank contributes its `[T_r, H]` rows padded to `plan.max_tokens`; one
    all-gather (NCCL over NVLink on GPUs, gloo on CPU for tests) and one row gather
    with `plan.restore_index` undo the sharding.
    """
    import torch.distributed as dist

    world = plan.world_size
    hidden = local_out.shape[-1]
    padded = local_out.new_zeros(plan.max_tokens, hidden)
    padded[: local_out.shape[0]] = local_out
    if world == 1:
        gathered = padded
    else:
        gathered = local_out.new_empty(world * plan.max_tokens, hidden)
        if dist.get_backend(group) == "nccl":
            dist.all_gather_into_tensor(gathered, padded, group=group)
        else:
            parts = list(gathered.view(world, plan.max_tokens, hidden).unbind(0))
            dist.all_gather(parts, padded, group=group)
    index = torch.from_numpy(plan.restore_index).to(local_out.device)
    return gathered.index_select(0, index)


def gather_pooled(local_pooled: Tensor, plan: ShardPlan, group=None) -> Tensor:
    """All ranks receive the `[N, H]` per-sequence embeddings in the original sequence order.

    The gather that follows a pooling head (`ops.pool_packed`): each rank contributes one row
    per sequence of its group, `[N_r, H]`, padded to the largest group, so a multi-GPU
    encode moves N * H values over NVLink instead of T * H."""
    import torch.distributed as dist

    world = plan.world_size
    width = local_pooled.shape[-1]
    max_rows = max(1, max(len(g) for g in plan.groups))
    padded = local_pooled.new_zeros(max_rows, width)
    padded[: local_pooled.shape[0]] = local_pooled
    if world == 1:
        gathered = padded
    else:
        gathered = local_pooled.new_empty(world * max_rows, width)
        if dist.get_backend(group) == "nccl":
            dist.all_gather_into_tensor(gathered, padded, group=group)
        else:
            parts = list(gathered.view(world, max_rows, width).unbind(0))
            dist.all_gather(parts, padded, group=group)
    index = np.empty(len(plan.lengths), dtype=np.int64)
    for r, g in enumerate(plan.groups):
        index[np.asarray(g, dtype=np.int64)] = r * max_rows + np.arange(len(g))
    return gathered.index_select(0, torch.from_numpy(index).to(local_pooled.device))
