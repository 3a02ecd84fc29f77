"""Bucketed CUDA graphs for `packed_forward` and for the padded `[B, S]` API, keyed on capacities.

Role of packed_encoders/graph.py:44-74 (GraphConfig), 209-396 (packed runner) and
435-472 (toggles). The reference keys a packed graph on `(M_bucket, N, Smax, backend)`,
so ragged traffic captures a graph per distinct sequence count and longest length.
Here every kernel reads the real boundaries (`cu_seqlens`) from device memory and the
attention grid is sized from capacities only, so one graph serves a whole bucket:
the key is `(token capacity, sequence capacity, query-tile height)`.

Tokens between the real total and the bucket capacity run through the GEMMs and
tails (wasted work, as in packed_encoders/graph.py:244-248) but lie outside
`cu_seqlens`, so attention never touches them; their output rows are discarded.
"""
from __future__ import annotations

import warnings

import os
from collections import OrderedDict
from dataclasses import dataclass

import torch
from torch import Tensor, nn

from . import _lib, forward
from .config import ModernBertParams
from .locate import find_encoder
from .state import get_state

GRAPH_ENV_VAR = "PACKED_ENCODERS_GRAPH"


def graphs_globally_disabled() -> bool:
    """True when the `PACKED_ENCODERS_GRAPH=0` kill switch is set."""
    return os.environ.get(GRAPH_ENV_VAR, "1") == "0"


@dataclass(frozen=True)
class GraphConfig:
    """Bucketing policy. Field names and defaults follow packed_encoders/graph.py:44-74.

    - `pad_to`: token totals are rounded up to a multiple of this to form a bucket,
      unless `token_buckets` lists explicit budgets (then the smallest budget that
      fits is used, and totals above the largest budget run eager).
    - `max_batch`: sequence capacity of every graph; calls with more sequences run
      eager. Left None, the capacity is the sequence count rounded up to a power of two.
    - `max_seq`: calls whose longest sequence exceeds it run eager.
    - `max_tokens`: totals above it are never captured.
    - `max_graphs`: LRU bound on live graphs.
    - `warmup`: eager runs on a side stream before capture.
    - `seq_buckets` (with `max_batch`): graphs captured at `pack()` time instead of on first
      sight, as packed_encoders/graph.py:410-427 does for the padded runner: one per listed
      longest-sequence bound s, sized for `max_batch` sequences of s tokens. With
      `token_buckets` (and `max_batch`) every listed budget is pre-captured as well.
    """

    pad_to: int = 64
    max_batch: int | None = None
    seq_buckets: tuple[int, ...] | None = None
    max_graphs: int = 32
    max_tokens: int = 2 ** 20
    max_seq: int | None = None
    warmup: int = 3
    token_buckets: tuple[int, ...] | None = None


def _round_up(value: int, multiple: int) -> int:
    return ((value + multiple - 1) // multiple) * multiple


def _pow2_at_least(value: int) -> int:
    return 1 << max(0, (int(value) - 1).bit_length())


def query_tile_rows(max_seqlen: int) -> int:
    """Rows per attention query tile the library picks for a longest length (16/32/64/128)."""
    if max_seqlen <= 16:
        return 16
    if max_seqlen <= 32:
        return 32
    if max_seqlen <= 64:
        return 64
    return 128


def _tile_class_seqlen(rows: int) -> int:
    """A max_seqlen that selects the `rows`-row query tile."""
    return {16: 16, 32: 32, 64: 64}.get(rows, 1 << 30)


@dataclass
class _PackedStaticInputs:
    """Fixed-address inputs of one captured graph."""

    input_ids: Tensor
    cu_seqlens: Tensor
    position_ids: Tensor

    def stage(self, packed_ids: Tensor, cu_seqlens: Tensor, position_ids: Tensor) -> int:
        m_real = packed_ids.shape[0]
        n_real = cu_seqlens.shape[0] - 1
        self.input_ids[:m_real].copy_(packed_ids)
        self.input_ids[m_real:].zero_()
        self.position_ids[:m_real].copy_(position_ids)
        self.position_ids[m_real:].zero_()
        self.cu_seqlens[: n_real + 1].copy_(cu_seqlens)
        if n_real + 1 < self.cu_seqlens.shape[0]:
            self.cu_seqlens[n_real + 1:].fill_(m_real)
        return m_real


@dataclass
class _PackedCaptured:
    graph: "torch.cuda.CUDAGraph"
    inputs: _PackedStaticInputs
    out: Tensor


class _PackedGraphRunner:
    """Capture-and-replay of `packed_forward` per `(token cap, sequence cap, tile rows)`."""

    def __init__(self, model: nn.Module, params: ModernBertParams, config: GraphConfig):
        self._model = model
        self._params = params
        self._config = config
        self._device = next(model.parameters()).device
        self._cache: OrderedDict[tuple[int, int, int], _PackedCaptured] = OrderedDict()
        self._workspace: Tensor | None = None
        self._generation = -1
        self.captures = 0
        self.replays = 0
        self.eager_calls = 0

    # -- policy -------------------------------------------------------------
    def bucket_for(self, total_tokens: int, n_seqs: int, max_seqlen: int) -> tuple[int, int, int] | None:
        """The cache key for a call, or None when the call must run eager."""
        cfg = self._config
        if cfg.max_seq is not None and max_seqlen > cfg.max_seq:
            return None
        if cfg.max_batch is not None and n_seqs > cfg.max_batch:
            return None
        if total_tokens > cfg.max_tokens or total_tokens <= 0:
            return None
        if cfg.token_buckets:
            fits = [b for b in sorted(cfg.token_buckets) if b >= total_tokens]
            if not fits:
                return None
            token_cap = fits[0]
        else:
            token_cap = _round_up(total_tokens, cfg.pad_to)
        seq_cap = cfg.max_batch if cfg.max_batch is not None else _pow2_at_least(n_seqs)
        return token_cap, seq_cap, query_tile_rows(max_seqlen)

    # -- call ----------------------------------------------------------------
    def __call__(self, packed_ids: Tensor, cu_seqlens: Tensor, max_seqlen: int,
                 position_ids: Tensor | None) -> Tensor:
        total = packed_ids.shape[0]
        n_seqs = cu_seqlens.numel() - 1
        key = self.bucket_for(total, n_seqs, int(max_seqlen))
        if key is None:
            self.eager_calls += 1
            return self._eager(packed_ids, cu_seqlens, max_seqlen, position_ids)
        binding = forward.get_binding(self._model, self._params)
        binding.check()  # a fault recorded by the previous call (eager or replay) is raised here
        if int(max_seqlen) > binding.max_positions:
            self.eager_calls += 1  # the eager call grows the RoPE tables
            return self._eager(packed_ids, cu_seqlens, max_seqlen, position_ids)
        if binding.generation != self._generation:
            self._cache.clear()
            self._generation = binding.generation
        if position_ids is None:
            position_ids = forward.positions_from_cu_seqlens(cu_seqlens, total)
        captured = self._cache.get(key)
        if captured is not None:
            self._cache.move_to_end(key)
        else:
            captured = self._capture(*key)
            while len(self._cache) >= self._config.max_graphs:
                self._cache.popitem(last=False)
            self._cache[key] = captured
        m_real = captured.inputs.stage(packed_ids, cu_seqlens, position_ids)
        captured.graph.replay()
        self.replays += 1
        out = captured.out[:m_real].clone()
        binding.after_call()  # the replayed kernels write the same status word as eager ones
        return out

    def _eager(self, packed_ids, cu_seqlens, max_seqlen, position_ids):
        return forward.packed_forward(
            self._model, self._params, packed_ids, cu_seqlens, max_seqlen, position_ids,
            _allow_graph=False,
        )

    # -- pre-capture ---------------------------------------------------------
    def precapture_keys(self) -> list[tuple[int, int, int]]:
        """Cache keys to capture ahead of the first call, largest token capacity first (the
        workspace then never has to grow, which would drop the graphs captured before)."""
        cfg = self._config
        if cfg.max_batch is None or not (cfg.seq_buckets or cfg.token_buckets):
            return []
        keys = set()
        for s in cfg.seq_buckets or ():
            key = self.bucket_for(cfg.max_batch * int(s), cfg.max_batch, int(s))
            if key is not None:
                keys.add(key)
        if cfg.token_buckets:
            longest = [int(s) for s in cfg.seq_buckets] if cfg.seq_buckets else [cfg.max_seq or (1 << 30)]
            for budget in cfg.token_buckets:
                for s in longest:
                    key = self.bucket_for(int(budget), cfg.max_batch, min(s, int(budget)))
                    if key is not None:
                        keys.add(key)
        return sorted(keys, reverse=True)[: cfg.max_graphs]

    def precapture(self) -> int:
        """Captures `precapture_keys()` now; returns how many graphs that made."""
        binding = forward.get_binding(self._model, self._params)
        self._generation = binding.generation
        made = 0
        for key in self.precapture_keys():
            if key not in self._cache:
                self._cache[key] = self._capture(*key)
                made += 1
        return made

    # -- capture ---------------------------------------------------------------
    def _ensure_workspace(self, binding, token_cap: int, seq_cap: int) -> Tensor:
        need = binding.workspace_bytes(token_cap, seq_cap)
        if self._workspace is None or self._workspace.numel() < need:
            # Captured graphs hold the old arena's address: drop them with it.
            self._cache.clear()
            self._workspace = None
            self._workspace = torch.empty(need, dtype=torch.uint8, device=self._device)
        return self._workspace

    def _capture(self, token_cap: int, seq_cap: int, tile_rows: int) -> _PackedCaptured:
        dev = self._device
        binding = forward.get_binding(self._model, self._params)
        binding.check()
        workspace = self._ensure_workspace(binding, token_cap, seq_cap)
        static = _PackedStaticInputs(
            input_ids=torch.zeros(token_cap, dtype=torch.int64, device=dev),
            cu_seqlens=torch.zeros(seq_cap + 1, dtype=torch.int32, device=dev),
            position_ids=torch.zeros(token_cap, dtype=torch.int64, device=dev),
        )
        # A valid stand-in distribution for warm-up and capture: one sequence of
        # min(token_cap, tile class) tokens, everything else empty.
        first = min(token_cap, tile_rows)
        static.cu_seqlens[1:].fill_(first)
        static.position_ids[:first] = torch.arange(first, device=dev)
        out = torch.empty(token_cap, self._params.hidden_size, dtype=torch.bfloat16, device=dev)
        max_seqlen = min(_tile_class_seqlen(tile_rows), binding.max_positions)
        binding.refresh()

        def run():
            binding.run(static.input_ids, static.cu_seqlens, static.position_ids, max_seqlen, out,
                        workspace=workspace, refresh=False)

        with torch.no_grad():
            side = torch.cuda.Stream(device=dev)
            side.wait_stream(torch.cuda.current_stream(dev))
            with torch.cuda.stream(side):
                for _ in range(max(1, self._config.warmup)):
                    run()
            torch.cuda.current_stream(dev).wait_stream(side)
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                run()
        self.captures += 1
        return _PackedCaptured(graph=graph, inputs=static, out=out)


# ---------------------------------------------------------------------------
# Padded [B, S] runner (packed_encoders/graph.py:112-201)
# ---------------------------------------------------------------------------


@dataclass
class _StaticInputs:
    """Fixed-address `[B_cap, S_bucket]` inputs of one captured padded graph."""

    input_ids: Tensor
    attention_mask: Tensor

    def stage(self, input_ids: Tensor, attention_mask: Tensor | None) -> None:
        """Write a real `(b, s)` batch into the corner of the static buffers; everything
        outside it is padding (mask 0), including the rows beyond `b`."""
        b, s = input_ids.shape
        self.input_ids.zero_()
        self.input_ids[:b, :s] = input_ids
        self.attention_mask.zero_()
        if attention_mask is None:
            self.attention_mask[:b, :s] = 1
        else:
            self.attention_mask[:b, :s] = (attention_mask != 0).to(self.attention_mask.dtype)


@dataclass
class _Captured:
    graph: "torch.cuda.CUDAGraph"
    inputs: _StaticInputs
    out: Tensor
    keep: tuple  # index / scratch tensors the graph's kernels write to


class _GraphRunner:
    """One captured graph per `(batch capacity, sequence bucket)` for `model(input_ids,
    attention_mask)`, the role of packed_encoders/graph.py:112-201: one graph serves every
    batch of at most `max_batch` rows whose width rounds up to the bucket.

    The captured region is the whole padded call: mask -> `cu_seqlens` / indices (`_unpad`),
    the gather of the real token ids, the packed forward at a capacity of `B_cap * S_bucket`
    tokens, and the scatter back to `[B_cap, S_bucket, H]` with zero pad rows. The number of
    real tokens never comes back to the host (the kernels read it and `cu_seqlens` on the
    device), so a replay has no synchronisation in front of it, unlike the eager `_unpad`."""

    def __init__(self, model: nn.Module, params: ModernBertParams, config: GraphConfig):
        self._model = model
        self._params = params
        self._config = config
        self._device = next(model.parameters()).device
        self._cache: OrderedDict[tuple[int, int], _Captured] = OrderedDict()
        self._workspace: Tensor | None = None
        self._generation = -1
        self.captures = 0
        self.replays = 0
        self.eager_calls = 0

    def bucket_for(self, b: int, s: int) -> tuple[int, int] | None:
        cfg = self._config
        if cfg.max_seq is not None and s > cfg.max_seq:
            return None
        if cfg.max_batch is not None and b > cfg.max_batch:
            return None
        bb = b if cfg.max_batch is None else cfg.max_batch
        sb = _round_up(s, cfg.pad_to)
        if bb * sb > cfg.max_tokens or bb * sb <= 0:
            return None
        return bb, sb

    def __call__(self, input_ids: Tensor, attention_mask: Tensor | None) -> Tensor:
        b, s = input_ids.shape
        key = self.bucket_for(b, s)
        binding = forward.get_binding(self._model, self._params)
        if key is None or key[1] > binding.max_positions:
            self.eager_calls += 1
            return self._eager(input_ids, attention_mask)
        binding.check()
        if binding.generation != self._generation:
            self._cache.clear()
            self._generation = binding.generation
        captured = self._cache.get(key)
        if captured is not None:
            self._cache.move_to_end(key)
        else:
            captured = self._capture(*key)
            self._insert(key, captured)
        captured.inputs.stage(input_ids, attention_mask)
        captured.graph.replay()
        self.replays += 1
        out = captured.out[:b, :s].clone()
        binding.after_call()
        return out

    def _eager(self, input_ids: Tensor, attention_mask: Tensor | None) -> Tensor:
        return forward.fused_forward(self._model, self._params, input_ids, attention_mask)

    def _insert(self, key: tuple[int, int], captured: _Captured) -> None:
        self._cache[key] = captured
        while len(self._cache) > self._config.max_graphs:
            self._cache.popitem(last=False)

    def precapture(self, batch: int, seq_buckets) -> int:
        binding = forward.get_binding(self._model, self._params)
        self._generation = binding.generation
        made = 0
        for s in sorted({_round_up(int(v), self._config.pad_to) for v in seq_buckets}, reverse=True):
            key = self.bucket_for(batch, s)
            if key is not None and key[1] <= binding.max_positions and key not in self._cache:
                self._insert(key, self._capture(*key))
                made += 1
        return made

    def _capture(self, bb: int, sb: int) -> _Captured:
        dev = self._device
        lib = _lib.load()
        binding = forward.get_binding(self._model, self._params)
        binding.check()
        cap = bb * sb
        cfg = self._config
        need = binding.workspace_bytes(cap, bb)
        if cfg.max_batch is not None and cfg.max_seq is not None:
            # the largest bucket this runner can ever capture: sized once, the arena never regrows
            largest = min(cfg.max_batch * _round_up(cfg.max_seq, cfg.pad_to), cfg.max_tokens)
            need = max(need, binding.workspace_bytes(largest, cfg.max_batch))
        if self._workspace is None or self._workspace.numel() < need:
            self._cache.clear()  # graphs captured so far hold the old arena's address
            self._workspace = None
            self._workspace = torch.empty(need, dtype=torch.uint8, device=dev)
        workspace = self._workspace
        static = _StaticInputs(
            input_ids=torch.zeros(bb, sb, dtype=torch.int64, device=dev),
            attention_mask=torch.ones(bb, sb, dtype=torch.int64, device=dev),
        )
        hidden = self._params.hidden_size
        seqlens = torch.zeros(bb, dtype=torch.int32, device=dev)
        cu = torch.zeros(bb + 1, dtype=torch.int32, device=dev)
        indices = torch.zeros(cap, dtype=torch.int64, device=dev)
        positions = torch.zeros(cap, dtype=torch.int64, device=dev)
        totals = torch.zeros(2, dtype=torch.int32, device=dev)
        packed_ids = torch.zeros(cap, dtype=torch.int64, device=dev)
        packed_out = torch.empty(cap, hidden, dtype=torch.bfloat16, device=dev)
        out = torch.empty(bb, sb, hidden, dtype=torch.bfloat16, device=dev)
        binding.refresh()

        def run():
            stream = _lib.current_stream_ptr()
            positions.zero_()  # entries beyond the real count must stay inside the RoPE table
            _lib.check(lib.pe_unpad_build(static.attention_mask.data_ptr(), 8, bb, sb, seqlens.data_ptr(),
                                          cu.data_ptr(), indices.data_ptr(), positions.data_ptr(),
                                          totals.data_ptr(), None, stream), "pe_unpad_build")
            _lib.check(lib.pe_gather_rows_counted(static.input_ids.data_ptr(), indices.data_ptr(),
                                                  totals.data_ptr(), cap, 8, packed_ids.data_ptr(), stream),
                       "pe_gather_rows_counted")
            binding.run(packed_ids, cu, positions, sb, packed_out, workspace=workspace, refresh=False)
            _lib.check(lib.pe_repad_scatter_counted(packed_out.data_ptr(), indices.data_ptr(),
                                                    totals.data_ptr(), cap, cap, hidden * 2,
                                                    out.data_ptr(), stream), "pe_repad_scatter_counted")

        with torch.no_grad(), torch.cuda.device(dev):
            side = torch.cuda.Stream(device=dev)
            side.wait_stream(torch.cuda.current_stream(dev))
            with torch.cuda.stream(side):
                for _ in range(max(1, self._config.warmup)):
                    run()
            torch.cuda.current_stream(dev).wait_stream(side)
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                run()
        self.captures += 1
        return _Captured(graph=graph, inputs=static, out=out,
                         keep=(seqlens, cu, indices, positions, totals, packed_ids, packed_out))


def build_runner(model: nn.Module, params: ModernBertParams, config: GraphConfig) -> _GraphRunner:
    """The padded-API runner, with its `seq_buckets` captured now when `max_batch` says at which
    batch capacity (packed_encoders/graph.py:410-427)."""
    runner = _GraphRunner(model, params, config)
    if config.seq_buckets and config.max_batch is not None:
        runner.precapture(config.max_batch, config.seq_buckets)
    return runner


def build_packed_runner(model: nn.Module, params: ModernBertParams, config: GraphConfig,
                        backend: str | None = None) -> _PackedGraphRunner:
    del backend
    runner = _PackedGraphRunner(model, params, config)
    if config.seq_buckets or config.token_buckets:
        if config.max_batch is None:
            if config.seq_buckets:
                warnings.warn(
                    "GraphConfig.seq_buckets needs max_batch to know the sequence capacity to "
                    "pre-capture at; skipping pre-capture (graphs are still captured on first sight).",
                    stacklevel=2,
                )
        else:
            runner.precapture()
    return runner


# ---------------------------------------------------------------------------
# Runtime toggles (packed_encoders/graph.py:435-472)
# ---------------------------------------------------------------------------


def set_cuda_graph(model: object, enabled: bool, *, config: GraphConfig | None = None) -> None:
    """Turn the graph layer on or off after `pack()`; the runner is built on first enable."""
    state = get_state(model)
    if enabled and state.packed_graph_runner is None:
        encoder = find_encoder(model)
        state.packed_graph_runner = build_packed_runner(encoder, state.params, config or GraphConfig())
        state.graph_runner = build_runner(encoder, state.params, config or GraphConfig())
    state.graph_enabled = bool(enabled)


class _NoCudaGraph:
    def __init__(self, model: object):
        self._state = get_state(model)
        self._previous = self._state.graph_enabled

    def __enter__(self):
        self._previous = self._state.graph_enabled
        self._state.graph_enabled = False
        return self

    def __exit__(self, *exc):
        self._state.graph_enabled = self._previous
        return False


def no_cuda_graph(model: object) -> _NoCudaGraph:
    """Context manager: run eager inside the block, restore the previous setting after."""
    return _NoCudaGraph(model)
