"""Seeded synthetic workloads and random-init ModernBERT weights (TEST INFRASTRUCTURE).

Stands in for the text corpora and hub checkpoints the reference benchmarks use
(benchmarks/helpers/common.py:39-126), which are not available offline: same shapes,
batch sizes and length skew, ids uniform in the vocabulary, weights normal(0, 0.02).
Used by tests/, bench.py and __graft_entry__.smoke() only.

Per configuration one fresh CPU generator seeded with 0 draws the lengths first and
the token ids second, so every machine derives identical batches.
"""
from __future__ import annotations

import math
from dataclasses import dataclass

import torch

VOCAB = 50368

ARCHS = {
    #          hidden layers heads intermediate
    "base":  dict(hidden_size=768, num_hidden_layers=22, num_attention_heads=12, intermediate_size=1152),
    "large": dict(hidden_size=1024, num_hidden_layers=28, num_attention_heads=16, intermediate_size=2624),
    "1b":    dict(hidden_size=1792, num_hidden_layers=28, num_attention_heads=28, intermediate_size=3840),
    # small shapes for fast parity tests; same layer pattern (global on 0, 3, ...)
    "tiny":  dict(hidden_size=256, num_hidden_layers=4, num_attention_heads=4, intermediate_size=384),
}


@dataclass
class Workload:
    name: str
    arch: str
    lengths: list[int]
    ids: torch.Tensor  # int64 [T], all sequences concatenated in order

    @property
    def total_tokens(self) -> int:
        return int(self.ids.shape[0])

    @property
    def max_seqlen(self) -> int:
        return max(self.lengths)

    def sequences(self) -> list[torch.Tensor]:
        return list(torch.split(self.ids, self.lengths))

    def sorted_by_length(self) -> "Workload":
        """Length-descending order, as the reference's showcase batches its inputs
        (benchmarks/showcases/inference.py:179-183)."""
        order = sorted(range(len(self.lengths)), key=lambda i: (-self.lengths[i], i))
        seqs = self.sequences()
        return Workload(self.name, self.arch, [self.lengths[i] for i in order],
                        torch.cat([seqs[i] for i in order]))


def _ids(gen: torch.Generator, total: int, vocab: int = VOCAB) -> torch.Tensor:
    return torch.randint(5, vocab, (total,), generator=gen, dtype=torch.int64)


def _lognormal(gen: torch.Generator, n: int, median: float, sigma: float, lo: int, hi: int):
    z = torch.randn(n, generator=gen)  # float32 draw: part of the workload definition
    raw = torch.exp(sigma * z + math.log(median)).round().clamp_(lo, hi)
    return [int(v) for v in raw.tolist()]


def workload(name: str, vocab: int = VOCAB, seed: int = 0) -> Workload:
    """cfg1..cfg5 of the build's baseline definition (seed 0), plus reduced variants for
    tests. Other seeds give further batches of the same distribution (the multi-GPU
    bench encodes one per GPU)."""
    gen = torch.Generator().manual_seed(seed)
    if name == "cfg1":      # parity batch: 32 sequences, lengths U[16, 512]
        lengths = torch.randint(16, 513, (32,), generator=gen).tolist()
        arch = "base"
    elif name == "cfg2":    # queries: 1024 sequences, lengths U[8, 48]
        lengths = torch.randint(8, 49, (1024,), generator=gen).tolist()
        arch = "base"
    elif name == "cfg3":    # documents (headline): 512, lognormal(median 400, sigma .8) in [64, 8192]
        lengths = _lognormal(gen, 512, 400.0, 0.8, 64, 8192)
        arch = "base"
    elif name == "cfg3q":   # every fourth document of cfg3: a profiling-sized slice of the headline workload
        lengths = _lognormal(gen, 512, 400.0, 0.8, 64, 8192)[::4]
        arch = "base"
    elif name == "cfg4":    # long documents on the large model: 64, U[2048, 8192]
        lengths = torch.randint(2048, 8193, (64,), generator=gen).tolist()
        arch = "large"
    elif name == "cfg5":    # mixed index on the 1B model: 8192 queries + 8192 documents
        lengths = torch.randint(8, 49, (8192,), generator=gen).tolist()
        lengths += _lognormal(gen, 8192, 600.0, 0.8, 64, 4096)
        arch = "1b"
    elif name == "tiny_mixed":  # ragged lengths incl. tile edges, for the tiny model
        lengths = [1, 2, 31, 32, 33, 63, 64, 65, 127, 128, 129, 200, 17, 300]
        arch = "tiny"
    elif name == "tiny_short":
        lengths = torch.randint(8, 49, (64,), generator=gen).tolist()
        arch = "tiny"
    else:
        raise KeyError(name)
    return Workload(name, arch, [int(v) for v in lengths], _ids(gen, int(sum(lengths)), vocab))


def make_config(arch: str, vocab: int = VOCAB, **overrides):
    from transformers import ModernBertConfig

    kw = dict(ARCHS[arch])
    kw.update(vocab_size=vocab, attn_implementation="eager")
    if vocab < VOCAB:  # the default special-token ids lie beyond a reduced vocabulary
        kw.update(pad_token_id=0, bos_token_id=1, eos_token_id=2, cls_token_id=1, sep_token_id=2)
    kw.update(overrides)
    return ModernBertConfig(**kw)


def make_model(arch: str, vocab: int = VOCAB, *, dtype=torch.float32, device="cpu", **overrides):
    """Random-init ModernBertModel: seed 0, every Linear/Embedding weight redrawn
    normal(0, 0.02) in a fixed order, LayerNorm weights 1, then rounded to bf16 so a
    bf16 copy (GPU) and an fp32 copy (CPU oracle) hold identical values."""
    from transformers import ModernBertModel

    torch.manual_seed(0)
    model = ModernBertModel(make_config(arch, vocab, **overrides))
    gen = torch.Generator().manual_seed(0)
    with torch.no_grad():
        for _, p in sorted(model.named_parameters(), key=lambda kv: kv[0]):
            if p.dim() >= 2:
                p.copy_(torch.randn(p.shape, generator=gen) * 0.02)
            else:
                p.fill_(1.0)
            p.copy_(p.to(torch.bfloat16).to(torch.float32))
    model.eval()
    return model.to(device=device, dtype=dtype)
