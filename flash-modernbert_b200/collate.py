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
