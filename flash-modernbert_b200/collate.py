"""Building packed batches on the caller's side of `packed_forward`.

`pack_sequences` follows benchmarks/helpers/packed_collator.py:68-96: concatenate the
real tokens, `cu_seqlens` = int32 prefix sums with a leading 0, `position_ids` =
`arange(L_i)` per sequence, empty input and empty sequences refused.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch
from torch import Tensor


@dataclass
class PackedBatch:
    input_ids: Tensor      # int64 [T]
    cu_seqlens: Tensor     # int32 [N+1]
    max_seqlen: int
    position_ids: Tensor   # int64 [T]
    seqlens: Tensor        # int32 [N] (host)

    def to(self, device) -> "PackedBatch":
        return PackedBatch(self.input_ids.to(device), self.cu_seqlens.to(device), self.max_seqlen,
                           self.position_ids.to(device), self.seqlens)

    def forward_args(self) -> tuple[Tensor, Tensor, int, Tensor]:
        """The positional tail of `packed_forward(model, params, *args)`."""
        return self.input_ids, self.cu_seqlens, self.max_seqlen, self.position_ids

    @property
    def total_tokens(self) -> int:
        return int(self.input_ids.shape[0])


def pack_sequences(sequences, *, device=None) -> PackedBatch:
    seqs = [s if isinstance(s, Tensor) else torch.tensor(s, dtype=torch.int64) for s in sequences]
    if not seqs:
        raise ValueError("pack_sequences got no sequences")
    seqlens = torch.tensor([s.numel() for s in seqs], dtype=torch.int32)
    if int(seqlens.min()) == 0:
        raise ValueError("pack_sequences got an empty sequence (length 0)")
    input_ids = torch.cat([s.to(torch.int64).reshape(-1) for s in seqs])
    cu_seqlens = torch.zeros(len(seqs) + 1, dtype=torch.int32)
    cu_seqlens[1:] = seqlens.cumsum(0, dtype=torch.int32)
    position_ids = torch.cat([torch.arange(int(n), dtype=torch.int64) for n in seqlens])
    batch = PackedBatch(input_ids, cu_seqlens, int(seqlens.max()), position_ids, seqlens)
    return batch.to(device) if device is not None else batch


def token_budget_batches(lengths, token_budget: int, *, sort_by_length: bool = True,
                         max_sequences: int | None = None) -> list[list[int]]:
    """Micro-batches of sequence indices holding at most `token_budget` real tokens each.

    The greedy rule of benchmarks/helpers/packed_training.py:175-202: walk the sequences in
    order and start a new batch when the next one would push the running total past the
    budget; a batch always takes at least one sequence, so a single sequence longer than the
    budget forms a batch of its own. `sort_by_length` walks them longest first, as the
    showcases order their batches (benchmarks/showcases/inference.py:179-183): neighbours then
    have similar lengths and a batch's attention cost is even. `max_sequences` also caps the
    number of sequences per batch (the sequence capacity of a CUDA-graph bucket)."""
    if token_budget <= 0:
        raise ValueError("token_budget must be positive")
    if max_sequences is not None and max_sequences <= 0:
        raise ValueError("max_sequences must be positive")
    sizes = [int(n) for n in lengths]
    if any(n <= 0 for n in sizes):
        raise ValueError("token_budget_batches got an empty sequence (length 0)")
    order = sorted(range(len(sizes)), key=lambda i: -sizes[i]) if sort_by_length else list(range(len(sizes)))
    batches: list[list[int]] = []
    current: list[int] = []
    tokens = 0
    for i in order:
        full = current and (tokens + sizes[i] > token_budget or
                            (max_sequences is not None and len(current) >= max_sequences))
        if full:
            batches.append(current)
            current, tokens = [], 0
        current.append(i)
        tokens += sizes[i]
    if current:
        batches.append(current)
    return batches


def encode_in_batches(model, params, sequences, token_budget: int, *, pool: str | None = "mean",
                      normalize: bool = True, device=None, sort_by_length: bool = True,
                      max_sequences: int | None = None):
    """Encodes any number of sequences through `packed_forward` in token-budget micro-batches
    (the loop of benchmarks/showcases/inference.py:186-209) and returns the results in the
    order of `sequences`: `[N, H]` sentence embeddings for `pool="mean"` / `"cls"`, or a list
    of per-sequence `[L_i, H]` hidden states for `pool=None`. Workspace and CUDA-graph buckets
    are bounded by the budget, whatever the corpus size."""
    from . import ops
    from .forward import packed_forward

    seqs = list(sequences)
    if not seqs:
        raise ValueError("encode_in_batches got no sequences")
    lengths = [int(torch.as_tensor(s).numel()) for s in seqs]
    device = device if device is not None else next(model.parameters()).device
    pooled = None
    hidden_list: list = [None] * len(seqs)
    for indices in token_budget_batches(lengths, token_budget, sort_by_length=sort_by_length,
                                        max_sequences=max_sequences):
        batch = pack_sequences([seqs[i] for i in indices], device=device)
        hidden = packed_forward(model, params, *batch.forward_args())
        if pool is None:
            bounds = batch.cu_seqlens.tolist()
            for slot, i in enumerate(indices):
                hidden_list[i] = hidden[bounds[slot]:bounds[slot + 1]]
            continue
        emb = ops.pool_packed(hidden, batch.cu_seqlens, pool, normalize)
        if pooled is None:
            pooled = torch.empty(len(seqs), emb.shape[-1], dtype=emb.dtype, device=emb.device)
        pooled[torch.tensor(indices, device=emb.device)] = emb
    return hidden_list if pool is None else pooled
