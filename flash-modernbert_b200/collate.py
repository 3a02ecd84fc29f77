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
    from .forward import packed_forward, packed_forward_pooled

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
        if pool is None:
            hidden = packed_forward(model, params, *batch.forward_args())
            bounds = batch.cu_seqlens.tolist()
            for slot, i in enumerate(indices):
                hidden_list[i] = hidden[bounds[slot]:bounds[slot + 1]]
            continue
        # pooling runs inside the final LayerNorm: the [T, H] hidden state is never materialised
        emb = packed_forward_pooled(model, params, *batch.forward_args(), pool=pool, normalize=normalize)
        if pooled is None:
            pooled = torch.empty(len(seqs), emb.shape[-1], dtype=emb.dtype, device=emb.device)
        pooled[torch.tensor(indices, device=emb.device)] = emb
    return hidden_list if pool is None else pooled


# ---------------------------------------------------------------------------
# Serving windows that mix queries and documents
# ---------------------------------------------------------------------------


@dataclass
class ServingWindow:
    """One window of requests encoded as ONE packed batch, whatever mix of short queries and
    long documents it holds (benchmarks/showcases/mixed_serving.py:151-193, `unified_packed`).

    `requests[n]` is the caller's id of the n-th sequence of `batch`; `kinds[n]` its kind."""

    requests: list[int]
    kinds: list[str]
    batch: PackedBatch


def mixed_windows(kinds, lengths, *, requests_per_window: int, query_fraction: float, windows: int,
                  seed: int = 0) -> list[list[int]]:
    """Request indices of `windows` serving windows, each holding
    `round(requests_per_window * query_fraction)` queries and the rest documents, drawn
    without replacement inside a window and shuffled into arrival order: the sampling of
    benchmarks/showcases/mixed_serving.py:151-172. `kinds[i]` is "query" or "document"."""
    import random

    n_query = round(requests_per_window * query_fraction)
    n_document = requests_per_window - n_query
    if not n_query or not n_document:
        raise ValueError("each window must contain both query and document requests")
    by_kind = {k: [i for i, kind in enumerate(kinds) if kind == k] for k in ("query", "document")}
    if len(by_kind["query"]) < n_query or len(by_kind["document"]) < n_document:
        raise ValueError("not enough requests of each kind to fill a window")
    del lengths  # the draw does not look at lengths; kept in the signature for bucket-aware callers
    rng = random.Random(int(seed))
    out = []
    for _ in range(int(windows)):
        chosen = rng.sample(by_kind["query"], n_query) + rng.sample(by_kind["document"], n_document)
        rng.shuffle(chosen)
        out.append(chosen)
    return out


def plan_windows(lengths, *, token_buckets, max_sequences: int | None = None) -> list[list[int]]:
    """Arrival-order windows sized for CUDA-graph token buckets: requests are taken in order and a
    window is closed when the next request would push it past the LARGEST bucket (or past
    `max_sequences`); each window then replays the smallest captured bucket that holds it.
    Unlike `token_budget_batches` nothing is reordered, so a window holds whatever mix of queries
    and documents arrived together; the attention schedule sends each sequence to the kernel that
    suits its length, so mixing costs nothing."""
    budgets = sorted(int(b) for b in token_buckets)
    if not budgets or budgets[0] <= 0:
        raise ValueError("plan_windows needs positive token_buckets")
    return token_budget_batches(lengths, budgets[-1], sort_by_length=False, max_sequences=max_sequences)


def encode_window(model, params, sequences, requests=None, kinds=None, *, pool: str | None = None,
                  normalize: bool = True, device=None):
    """Encodes one mixed window as a single packed batch in arrival order. Returns
    `(ServingWindow, result)` where result is the packed `[T, H]` hidden state (`pool=None`; slice it
    with `window.batch.cu_seqlens`) or `[N, H]` pooled embeddings, row n belonging to
    `window.requests[n]`."""
    from .forward import packed_forward, packed_forward_pooled

    seqs = list(sequences)
    device = device if device is not None else next(model.parameters()).device
    batch = pack_sequences(seqs, device=device)
    window = ServingWindow(list(requests) if requests is not None else list(range(len(seqs))),
                           list(kinds) if kinds is not None else ["?"] * len(seqs), batch)
    if pool is None:
        return window, packed_forward(model, params, *batch.forward_args())
    return window, packed_forward_pooled(model, params, *batch.forward_args(), pool=pool, normalize=normalize)
