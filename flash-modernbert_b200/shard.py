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
                   half_window: int = 64, attn_global_weight: float = 2.0,
                   attn_local_weight: float = 5.0) -> np.ndarray:
    """Cost of encoding each sequence, in GEMM-equivalent FLOPs (multiply-add = 2).

    Attention FLOPs are weighted by how much slower than the projections the attention kernels
    retire them on a B200: the full-attention kernel runs at about half the GEMMs' rate
    (exp2-bound at head dim 64), the sliding-window kernel at about a fifth (per algorithmic
    pair; it is instruction-issue bound). With both weights 1 this is the plain FLOP model."""
    s = np.asarray(lengths, dtype=np.float64)
    gemm = s * n_layers * (8.0 * hidden * hidden + 6.0 * hidden * intermediate)
    attn_g = 4.0 * hidden * n_global * s * s
    attn_l = 4.0 * hidden * (n_layers - n_global) * local_pairs(s, half_window)
    return gemm + attn_global_weight * attn_g + attn_local_weight * attn_l


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
    """Who encodes what, and where each sequence lands in the gathered output.

    The gathered tensors are in RANK-MAJOR order: rank 0's sequences (in the order it encodes
    them), then rank 1's, and so on. Every rank's rows are then one contiguous range of the
    result, so the gather writes them straight into place: no padding to a common size and no
    row permutation afterwards. `order`, `seq_rows` and `seq_slot` are the host-side tables that
    take a caller from its own sequence numbering to that layout."""

    world_size: int
    lengths: np.ndarray                 # [N] all sequence lengths, original order
    groups: list[np.ndarray]            # per rank: indices into the original order
    tokens_per_rank: np.ndarray         # [world]
    order: np.ndarray                   # [N] original index of the n-th sequence in rank-major order
    seq_slot: np.ndarray                # [N] position of original sequence i in rank-major order
    seq_rows: np.ndarray                # [N] first row of original sequence i in the gathered [T, H]
    row_start: np.ndarray               # [world + 1] first gathered row of each rank
    slot_start: np.ndarray              # [world + 1] first gathered sequence slot of each rank

    @property
    def total_tokens(self) -> int:
        return int(self.lengths.sum())

    @property
    def max_tokens(self) -> int:
        return int(max(1, self.tokens_per_rank.max()))

    def restore_index(self) -> np.ndarray:
        """[T_total] gathered row of every row of the original packed order."""
        starts = np.concatenate(([0], np.cumsum(self.lengths)))
        index = np.empty(int(starts[-1]), dtype=np.int64)
        for i, n in enumerate(self.lengths):
            index[starts[i]:starts[i + 1]] = self.seq_rows[i] + np.arange(int(n))
        return index

    def gathered_cu_seqlens(self) -> np.ndarray:
        """int32 [N + 1] boundaries of the gathered (rank-major) packed rows."""
        return np.concatenate(([0], np.cumsum(self.lengths[self.order]))).astype(np.int32)


def plan_shards(lengths, world_size: int, costs=None) -> ShardPlan:
    lengths = np.asarray(lengths, dtype=np.int64)
    if lengths.size == 0 or (lengths <= 0).any():
        raise ValueError("plan_shards needs at least one sequence and positive lengths")
    costs = lengths.astype(np.float64) if costs is None else np.asarray(costs, dtype=np.float64)
    groups = balance(costs, world_size)
    tokens = np.asarray([int(lengths[g].sum()) for g in groups], dtype=np.int64)
    order = np.concatenate(groups).astype(np.int64)
    seq_slot = np.empty(lengths.size, dtype=np.int64)
    seq_slot[order] = np.arange(lengths.size)
    rows_in_order = np.concatenate(([0], np.cumsum(lengths[order])))[:-1]
    seq_rows = np.empty(lengths.size, dtype=np.int64)
    seq_rows[order] = rows_in_order
    row_start = np.concatenate(([0], np.cumsum(tokens)))
    slot_start = np.concatenate(([0], np.cumsum([len(g) for g in groups])))
    return ShardPlan(world_size, lengths, groups, tokens, order, seq_slot, seq_rows, row_start, slot_start)


def local_batch(plan: ShardPlan, rank: int, sequences):
    """This rank's sequences (a list of 1-D id tensors), in the plan's order."""
    return [sequences[int(i)] for i in plan.groups[rank]]


def _gather_ranges(local: Tensor, starts: np.ndarray, group=None, out: Tensor | None = None) -> Tensor:
    """All ranks receive every rank's rows: rank r's `[starts[r+1] - starts[r], W]` block lands at
    rows `starts[r]:starts[r+1]` of the result. On NCCL this is ONE all-gather with uneven block
    sizes whose receive buffers are views of the result itself (torch issues it as grouped
    broadcasts over NVLink); gloo, used by the CPU tests, needs equal sizes and goes through a
    padded copy."""
    import torch.distributed as dist

    world = len(starts) - 1
    width = local.shape[-1]
    total = int(starts[-1])
    if out is None:
        out = local.new_empty(total, width)
    if local.shape[0] != int(starts[1] - starts[0]) and world == 1:
        raise ValueError("local block does not match the plan")
    if world == 1:
        out.copy_(local)
        return out
    rank = dist.get_rank(group)
    if local.shape[0] != int(starts[rank + 1] - starts[rank]):
        raise ValueError(f"rank {rank}: local block of {local.shape[0]} rows, plan says "
                         f"{int(starts[rank + 1] - starts[rank])}")
    views = [out[int(starts[r]):int(starts[r + 1])] for r in range(world)]
    if dist.get_backend(group) == "nccl":
        dist.all_gather(views, local.contiguous(), group=group)
    else:
        biggest = max(1, int(np.max(np.diff(starts))))
        padded = local.new_zeros(biggest, width)
        padded[: local.shape[0]] = local
        parts = [local.new_empty(biggest, width) for _ in range(world)]
        dist.all_gather(parts, padded, group=group)
        for r in range(world):
            views[r].copy_(parts[r][: views[r].shape[0]])
    return out


def gather_embeddings(local_out: Tensor, plan: ShardPlan, group=None, *, restore: bool = False,
                      out: Tensor | None = None) -> Tensor:
    """All ranks receive the `[T_total, H]` token embeddings in rank-major order (see
    `ShardPlan`): sequence i's rows start at `plan.seq_rows[i]`. Nothing but the NCCL transfer
    touches the rows. `restore=True` additionally permutes them into the original packed order
    (one row gather: 2 * T * H * 2 bytes of extra HBM traffic per rank)."""
    gathered = _gather_ranges(local_out, plan.row_start, group, out)
    if not restore:
        return gathered
    index = torch.from_numpy(plan.restore_index()).to(local_out.device)
    return gathered.index_select(0, index)


def gather_pooled(local_pooled: Tensor, plan: ShardPlan, group=None, *, restore: bool = True) -> Tensor:
    """All ranks receive the `[N, H]` per-sequence embeddings.

    The gather that follows a pooling head (`packed_forward_pooled`): each rank contributes one
    row per sequence of its group, so a multi-GPU encode moves N * H values over NVLink instead
    of T * H. `restore=True` (default; the tensor is small) returns them in the callers' original
    sequence order, else in rank-major order (`plan.order[n]` is the original index of row n)."""
    gathered = _gather_ranges(local_pooled, plan.slot_start, group)
    if not restore:
        return gathered
    return gathered.index_select(0, torch.from_numpy(plan.seq_slot).to(local_pooled.device))
