"""Host side of the packed forward: the reference's entry points, backed by the C ABI.

Same names and argument meaning as packed_encoders/forward.py: `_unpad` (384-403),
`_repad` (406-412), `packed_forward` (415-516), `_varlen_forward` (617-639) and
`fused_forward` (642-691). Every device operation is a call into libpe_b200.so;
torch is used for device memory, streams and argument checks only. There is no
rectangular/SDPA path and no backend choice: a padded batch is always unpadded,
run packed, and re-padded.
"""
from __future__ import annotations

import ctypes
import os

import torch
from torch import Tensor, nn

from . import _lib
from .config import ModernBertParams
from .errors import PackedEncodersError
from .state import ATTR

_GRAPH_ENV = "PACKED_ENCODERS_GRAPH"
_BINDING_ATTR = "_pe_b200_binding"
_CHECK_ENV = "PE_B200_CHECK_STATUS"


def _require_cuda_tensor(t: Tensor, name: str, dtype: torch.dtype | None = None) -> Tensor:
    if not isinstance(t, Tensor) or not t.is_cuda:
        raise PackedEncodersError(f"{name} must be a CUDA tensor (this package has no CPU path)")
    if dtype is not None and t.dtype != dtype:
        raise ValueError(f"{name} must have dtype {dtype}, got {t.dtype}")
    return t if t.is_contiguous() else t.contiguous()


# ---------------------------------------------------------------------------
# C-ABI view of a live HF model
# ---------------------------------------------------------------------------


def _layer_is_global(layer: nn.Module, layer_idx: int, params: ModernBertParams) -> bool:
    kind = getattr(layer, "attention_type", None)
    if kind == "full_attention":
        return True
    if kind == "sliding_attention":
        return False
    return params.is_global_layer(layer_idx)


def _weight_of(module: nn.Module, what: str) -> Tensor:
    if getattr(module, "bias", None) is not None:
        raise PackedEncodersError(
            f"{what} has a bias; the packed path implements bias-free ModernBERT only and "
            "refuses to drop it"
        )
    w = module.weight
    if not w.is_cuda:
        raise PackedEncodersError(f"{what}.weight is on {w.device}; move the model to a B200 first")
    if w.dtype != torch.bfloat16:
        raise PackedEncodersError(
            f"{what}.weight is {w.dtype}; the CUDA path computes in bf16 - call model.to(torch.bfloat16)"
        )
    if not w.is_contiguous():
        raise PackedEncodersError(f"{what}.weight is not contiguous")
    return w


class ModelBinding:
    """Pointer tables, RoPE tables, status word and scratch arena for one encoder.

    Weights stay the HF parameters in HF layout (packed_encoders/pack.py:3-6); their
    addresses are re-read on every eager call, so `.to()`/in-place updates are seen.
    """

    def __init__(self, model: nn.Module, params: ModernBertParams):
        self.lib = _lib.load()
        self.model = model
        self.params = params
        if params.head_dim != 64:
            raise PackedEncodersError(f"head_dim={params.head_dim}: the kernels support 64 only")
        emb_w = _weight_of(model.embeddings.tok_embeddings, "embeddings.tok_embeddings")
        self.device = emb_w.device
        with torch.cuda.device(self.device):
            _lib.check(self.lib.pe_device_check(), "pe_device_check")
        self.n_layers = len(model.layers)
        self.intermediate = model.layers[0].mlp.Wo.weight.shape[1]
        self._layers_c = (_lib.PeLayerWeights * self.n_layers)()
        self._model_c = _lib.PeModel()
        self._status = torch.zeros(1, dtype=torch.int32, device=self.device)
        self._status_host = torch.zeros(1, dtype=torch.int32).pin_memory()
        self._workspace: Tensor | None = None
        self._rope: tuple[Tensor, Tensor] | None = None
        self._rope_key: tuple | None = None
        self.max_positions = 0
        self.generation = 0
        self._ensure_rope(int(getattr(model.config, "max_position_embeddings", 8192)))
        self.refresh()

    # -- tables ---------------------------------------------------------------
    def _ensure_rope(self, min_positions: int) -> None:
        p = self.params
        key = (p.global_rope_theta, p.local_rope_theta)
        if self._rope is not None and self.max_positions >= min_positions and self._rope_key == key:
            return
        rows = max(int(min_positions), 128)
        tables = []
        with torch.cuda.device(self.device):
            stream = _lib.current_stream_ptr()
            for theta in key:
                t = torch.empty(rows, 64, dtype=torch.bfloat16, device=self.device)
                _lib.check(self.lib.pe_rope_table(float(theta), rows, t.data_ptr(), stream),
                           "pe_rope_table")
                tables.append(t)
        self._rope = (tables[0], tables[1])
        self._rope_key = key
        self.max_positions = rows
        self.generation += 1  # captured graphs that baked the old tables are stale

    def refresh(self) -> None:
        """Re-read every weight address into the C structs."""
        m, p = self.model, self.params
        for i, layer in enumerate(m.layers):
            c = self._layers_c[i]
            attn_norm = layer.attn_norm
            c.attn_norm_w = (
                None if isinstance(attn_norm, nn.Identity)
                else _weight_of(attn_norm, f"layers[{i}].attn_norm").data_ptr()
            )
            c.wqkv = _weight_of(layer.attn.Wqkv, f"layers[{i}].attn.Wqkv").data_ptr()
            c.wo = _weight_of(layer.attn.Wo, f"layers[{i}].attn.Wo").data_ptr()
            c.mlp_norm_w = _weight_of(layer.mlp_norm, f"layers[{i}].mlp_norm").data_ptr()
            c.wi = _weight_of(layer.mlp.Wi, f"layers[{i}].mlp.Wi").data_ptr()
            c.wo_mlp = _weight_of(layer.mlp.Wo, f"layers[{i}].mlp.Wo").data_ptr()
            c.is_global = 1 if _layer_is_global(layer, i, p) else 0
        mc = self._model_c
        mc.hidden = p.hidden_size
        mc.n_heads = p.num_attention_heads
        mc.head_dim = p.head_dim
        mc.intermediate = int(self.intermediate)
        mc.n_layers = self.n_layers
        mc.vocab = int(m.embeddings.tok_embeddings.weight.shape[0])
        mc.half_window = p.sliding_half_window
        mc.max_positions = self.max_positions
        mc.eps = float(p.norm_eps)
        mc.tok_emb = _weight_of(m.embeddings.tok_embeddings, "embeddings.tok_embeddings").data_ptr()
        mc.emb_norm_w = _weight_of(m.embeddings.norm, "embeddings.norm").data_ptr()
        mc.final_norm_w = _weight_of(m.final_norm, "final_norm").data_ptr()
        mc.rope_global = self._rope[0].data_ptr()
        mc.rope_local = self._rope[1].data_ptr()
        mc.layers = ctypes.cast(self._layers_c, ctypes.POINTER(_lib.PeLayerWeights))

    # -- scratch ----------------------------------------------------------------
    def workspace_bytes(self, total_tokens: int, n_seqs: int) -> int:
        return int(self.lib.pe_forward_workspace_bytes(ctypes.byref(self._model_c), total_tokens, n_seqs))

    def workspace(self, total_tokens: int, n_seqs: int) -> Tensor:
        need = self.workspace_bytes(total_tokens, n_seqs)
        if self._workspace is None or self._workspace.numel() < need:
            self._workspace = None  # release before growing
            self._workspace = torch.empty(need, dtype=torch.uint8, device=self.device)
        return self._workspace

    # -- status ---------------------------------------------------------------
    def check(self, sync: bool = False) -> None:
        """Raise if a kernel recorded a fault. `sync=True` waits for the device first."""
        if sync:
            self._status_host.copy_(self._status, non_blocking=False)
        code = int(self._status_host[0])
        if code != 0:
            self._status.zero_()
            self._status_host.zero_()
            raise _lib.NativeLibraryError(
                f"a CUDA kernel reported status {code} (1xx: GEMM pipeline wait gave up, "
                "2xx: attention, 301: token id outside the vocabulary, 302: position outside "
                "the RoPE table, 303: cu_seqlens entry outside [0, T] or decreasing)"
            )

    def after_call(self) -> None:
        """What every forward does once its kernels are enqueued: with PE_B200_CHECK_STATUS=1
        wait and raise on this very call, else start the read-back of the status word that the
        next call's `check()` inspects."""
        if os.environ.get(_CHECK_ENV, "0") == "1":
            self.check(sync=True)
        else:
            self._status_host.copy_(self._status, non_blocking=True)

    # -- the call ---------------------------------------------------------------
    def run(self, ids: Tensor, cu_seqlens: Tensor, position_ids: Tensor, max_seqlen: int,
            out: Tensor | None, *, workspace: Tensor | None = None, refresh: bool = True,
            pooled: Tensor | None = None, pool_mode: int = 1, normalize: bool = True) -> Tensor | None:
        """Enqueue one forward. `out` receives the `[T, H]` hidden state; with `pooled` (an
        `[N, H]` tensor) the pooling head runs inside the final LayerNorm and `out` may be None."""
        total = ids.shape[0]
        n_seqs = cu_seqlens.shape[0] - 1
        if max_seqlen > self.max_positions:
            self._ensure_rope(max_seqlen)
            refresh = True
        if refresh:
            self.refresh()
        ws = workspace if workspace is not None else self.workspace(total, n_seqs)
        with torch.cuda.device(self.device):
            if pooled is None:
                rc = self.lib.pe_forward_packed(
                    ctypes.byref(self._model_c), ids.data_ptr(), cu_seqlens.data_ptr(),
                    position_ids.data_ptr(), total, n_seqs, int(max_seqlen), ws.data_ptr(), ws.numel(),
                    out.data_ptr(), self._status.data_ptr(), _lib.current_stream_ptr())
            else:
                rc = self.lib.pe_forward_packed_pooled(
                    ctypes.byref(self._model_c), ids.data_ptr(), cu_seqlens.data_ptr(),
                    position_ids.data_ptr(), total, n_seqs, int(max_seqlen), ws.data_ptr(), ws.numel(),
                    int(pool_mode), 1 if normalize else 0, _lib.ptr(out), pooled.data_ptr(),
                    self._status.data_ptr(), _lib.current_stream_ptr())
        _lib.check(rc, "pe_forward_packed" if pooled is None else "pe_forward_packed_pooled")
        return out


def get_binding(model: nn.Module, params: ModernBertParams) -> ModelBinding:
    state = getattr(model, ATTR, None)
    holder = state if state is not None else model
    attr = "binding" if state is not None else _BINDING_ATTR
    binding = getattr(holder, attr, None)
    if binding is None or binding.params != params:
        binding = ModelBinding(model, params)
        if state is not None:
            state.binding = binding
        else:
            object.__setattr__(model, _BINDING_ATTR, binding)
    return binding


# ---------------------------------------------------------------------------
# Padding boundary
# ---------------------------------------------------------------------------


def _mask_for_kernel(attention_mask: Tensor) -> tuple[Tensor, int]:
    if attention_mask.dtype == torch.bool:
        return attention_mask.contiguous().view(torch.uint8), 1
    size = attention_mask.element_size()
    if attention_mask.dtype.is_floating_point or size not in (1, 4, 8):
        return (attention_mask != 0).contiguous().view(torch.uint8), 1
    return attention_mask.contiguous(), size


def _unpad(x: Tensor, attention_mask: Tensor) -> tuple[Tensor, Tensor, Tensor, int, Tensor]:
    """Strip padding from `x` [B, S, ...] using `attention_mask` [B, S] (non-zero = real).

    Returns `(x_packed, indices, cu_seqlens, max_seqlen, position_ids)` with the
    dtypes and order of packed_encoders/forward.py:384-403: `indices` int64 flat
    row-major positions, `cu_seqlens` int32 `[B+1]`, `position_ids = indices % S`.
    One host synchronisation (the read-back of T and max_seqlen), as in the reference.
    """
    attention_mask = _require_cuda_tensor(attention_mask, "attention_mask")
    x = _require_cuda_tensor(x, "x")
    b, s = attention_mask.shape
    if x.shape[0] != b or x.shape[1] != s:
        raise ValueError(f"x {tuple(x.shape)} does not match attention_mask {(b, s)}")
    lib = _lib.load()
    dev = attention_mask.device
    mask, width = _mask_for_kernel(attention_mask)
    seqlens = torch.empty(b, dtype=torch.int32, device=dev)
    cu_seqlens = torch.empty(b + 1, dtype=torch.int32, device=dev)
    indices_full = torch.empty(b * s, dtype=torch.int64, device=dev)
    positions_full = torch.empty(b * s, dtype=torch.int64, device=dev)
    totals_dev = torch.empty(2, dtype=torch.int32, device=dev)
    totals_host = (ctypes.c_int32 * 2)()
    with torch.cuda.device(dev):
        stream = _lib.current_stream_ptr()
        _lib.check(lib.pe_unpad_build(mask.data_ptr(), width, b, s, seqlens.data_ptr(),
                                      cu_seqlens.data_ptr(), indices_full.data_ptr(),
                                      positions_full.data_ptr(), totals_dev.data_ptr(),
                                      totals_host, stream), "pe_unpad_build")
        total, max_seqlen = int(totals_host[0]), int(totals_host[1])
        indices = indices_full[:total]
        position_ids = positions_full[:total]
        rest = tuple(x.shape[2:])
        row_bytes = x.element_size()
        for d in rest:
            row_bytes *= d
        x_packed = torch.empty((total, *rest), dtype=x.dtype, device=dev)
        if row_bytes > 0:
            _lib.check(lib.pe_gather_rows(x.data_ptr(), indices.data_ptr(), total, row_bytes,
                                          x_packed.data_ptr(), stream), "pe_gather_rows")
    return x_packed, indices, cu_seqlens, max_seqlen, position_ids


def _repad(x_packed: Tensor, indices: Tensor, b: int, s: int) -> Tensor:
    """Inverse of `_unpad` (packed_encoders/forward.py:406-412): `[T, H]` -> `[B, S, H]`,
    pad rows exactly zero. One kernel writes every output row once."""
    x_packed = _require_cuda_tensor(x_packed, "x_packed")
    indices = _require_cuda_tensor(indices, "indices", torch.int64)
    hidden = x_packed.shape[-1]
    out = torch.empty(b * s, hidden, dtype=x_packed.dtype, device=x_packed.device)
    lib = _lib.load()
    with torch.cuda.device(x_packed.device):
        _lib.check(lib.pe_repad_scatter(x_packed.data_ptr(), indices.data_ptr(), x_packed.shape[0],
                                        b * s, hidden * x_packed.element_size(), out.data_ptr(),
                                        _lib.current_stream_ptr()), "pe_repad_scatter")
    return out.reshape(b, s, hidden)


def _has_padding(attention_mask: Tensor | None) -> bool:
    return attention_mask is not None and not bool((attention_mask == 1).all())


def positions_from_cu_seqlens(cu_seqlens: Tensor, total: int) -> Tensor:
    """`arange(L_i)` per sequence, int64 `[total]` (benchmarks/helpers/packed_collator.py:94)."""
    token = torch.arange(total, device=cu_seqlens.device, dtype=torch.int64)
    seq = torch.searchsorted(cu_seqlens[1:].to(torch.int64), token, right=True)
    seq = seq.clamp_(max=cu_seqlens.shape[0] - 2)
    return token - cu_seqlens.to(torch.int64)[seq]


# ---------------------------------------------------------------------------
# Entry points
# ---------------------------------------------------------------------------


def packed_forward(
    model: nn.Module,
    params: ModernBertParams,
    packed_ids: Tensor,
    cu_seqlens: Tensor,
    max_seqlen: int,
    position_ids: Tensor | None = None,
    *,
    backend: str | None = None,
    _allow_graph: bool = True,
) -> Tensor:
    """Encode an already-packed batch; returns the packed last hidden state `[T, H]` bf16.

    Signature and contract of packed_encoders/forward.py:415-516. `packed_ids` int64
    `[T]`, `cu_seqlens` int32 `[N+1]` (cu[0] = 0, cu[N] = T), `max_seqlen` >= the longest
    sequence, `position_ids` int64 `[T]` (None = `arange` per sequence). `backend` is
    accepted for source compatibility and ignored: there is one attention kernel family.
    With a packed graph runner installed by `pack(cuda_graph=GraphConfig(...))` the call
    replays a bucketed CUDA graph unless `PACKED_ENCODERS_GRAPH=0`.
    """
    del backend
    state = getattr(model, ATTR, None)
    if (
        _allow_graph
        and state is not None
        and state.packed_graph_runner is not None
        and state.graph_enabled
        and os.environ.get(_GRAPH_ENV, "1") != "0"
        and not torch.is_grad_enabled()
        and not torch.is_autocast_enabled("cuda")
    ):
        return state.packed_graph_runner(packed_ids, cu_seqlens, max_seqlen, position_ids)

    packed_ids = _require_cuda_tensor(packed_ids, "packed_ids", torch.int64)
    cu_seqlens = _require_cuda_tensor(cu_seqlens, "cu_seqlens", torch.int32)
    if packed_ids.dim() != 1 or cu_seqlens.dim() != 1 or cu_seqlens.shape[0] < 2:
        raise ValueError("packed_ids must be [T] and cu_seqlens [N+1] with N >= 1")
    total = packed_ids.shape[0]
    if position_ids is None:
        position_ids = positions_from_cu_seqlens(cu_seqlens, total)
    position_ids = _require_cuda_tensor(position_ids, "position_ids", torch.int64)
    if position_ids.shape != packed_ids.shape:
        raise ValueError("position_ids must have the shape of packed_ids")
    if int(max_seqlen) <= 0:
        raise ValueError("max_seqlen must be positive")

    binding = get_binding(model, params)
    binding.check()
    out = torch.empty(total, params.hidden_size, dtype=torch.bfloat16, device=packed_ids.device)
    if total == 0:
        return out
    binding.run(packed_ids, cu_seqlens, position_ids, int(max_seqlen), out)
    binding.after_call()
    return out


def packed_forward_pooled(
    model: nn.Module,
    params: ModernBertParams,
    packed_ids: Tensor,
    cu_seqlens: Tensor,
    max_seqlen: int,
    position_ids: Tensor | None = None,
    *,
    pool: str = "mean",
    normalize: bool = True,
    return_hidden: bool = False,
) -> Tensor | tuple[Tensor, Tensor]:
    """`packed_forward` followed by the pooling every caller of the reference applies to its
    result (benchmarks/showcases/inference.py:193-209: fp32 segment mean, `F.normalize`, cast
    back), as one library call: the pooling runs inside the final LayerNorm, so the `[T, H]`
    hidden state is not read back and, unless `return_hidden`, never written.

    Returns `[N, H]` bf16 sentence embeddings (`pool="mean"` or `"cls"`), or
    `(hidden [T, H], embeddings [N, H])` with `return_hidden=True`. Always eager (no graph replay).
    """
    if pool not in ("mean", "cls"):
        raise ValueError(f"packed_forward_pooled: pool must be 'mean' or 'cls', got {pool!r}")
    packed_ids = _require_cuda_tensor(packed_ids, "packed_ids", torch.int64)
    cu_seqlens = _require_cuda_tensor(cu_seqlens, "cu_seqlens", torch.int32)
    if packed_ids.dim() != 1 or cu_seqlens.dim() != 1 or cu_seqlens.shape[0] < 2:
        raise ValueError("packed_ids must be [T] and cu_seqlens [N+1] with N >= 1")
    total = packed_ids.shape[0]
    if position_ids is None:
        position_ids = positions_from_cu_seqlens(cu_seqlens, total)
    position_ids = _require_cuda_tensor(position_ids, "position_ids", torch.int64)
    if position_ids.shape != packed_ids.shape:
        raise ValueError("position_ids must have the shape of packed_ids")
    if int(max_seqlen) <= 0:
        raise ValueError("max_seqlen must be positive")
    binding = get_binding(model, params)
    binding.check()
    dev = packed_ids.device
    n_seqs = cu_seqlens.shape[0] - 1
    hidden = torch.empty(total, params.hidden_size, dtype=torch.bfloat16, device=dev) if return_hidden else None
    if total == 0:
        pooled = torch.zeros(n_seqs, params.hidden_size, dtype=torch.bfloat16, device=dev)
        return (hidden, pooled) if return_hidden else pooled
    pooled = torch.empty(n_seqs, params.hidden_size, dtype=torch.bfloat16, device=dev)
    binding.run(packed_ids, cu_seqlens, position_ids, int(max_seqlen), hidden, pooled=pooled,
                pool_mode=1 if pool == "mean" else 0, normalize=normalize)
    binding.after_call()
    return (hidden, pooled) if return_hidden else pooled


def _varlen_forward(
    model: nn.Module,
    params: ModernBertParams,
    input_ids: Tensor,
    attention_mask: Tensor,
    *,
    backend: str | None = None,
) -> Tensor:
    """`_unpad` -> `packed_forward` -> `_repad` (packed_encoders/forward.py:617-639)."""
    b, s = input_ids.shape
    packed_ids, indices, cu_seqlens, max_seqlen, position_ids = _unpad(
        input_ids.unsqueeze(-1), attention_mask
    )
    if packed_ids.shape[0] == 0:
        return torch.zeros(b, s, params.hidden_size, dtype=torch.bfloat16, device=input_ids.device)
    out = packed_forward(
        model, params, packed_ids.squeeze(-1), cu_seqlens, max_seqlen, position_ids, backend=backend
    )
    return _repad(out, indices, b, s)


def fused_forward(
    model: nn.Module,
    params: ModernBertParams,
    input_ids: Tensor,
    attention_mask: Tensor | None,
    *,
    backend: str | None = None,
) -> Tensor:
    """Padded-API forward: `[B, S]` ids (+ mask) -> `[B, S, H]` last hidden state, pad rows zero.

    Role of packed_encoders/forward.py:642-691, without its rectangular branch: a batch
    with no mask is its own packing (every row a full sequence), anything else goes
    through `_varlen_forward`.
    """
    input_ids = _require_cuda_tensor(input_ids, "input_ids")
    if input_ids.dtype != torch.int64:
        input_ids = input_ids.to(torch.int64)
    b, s = input_ids.shape
    if attention_mask is None:
        dev = input_ids.device
        cu = torch.arange(0, (b + 1) * s, s, dtype=torch.int32, device=dev)
        pos = torch.arange(s, dtype=torch.int64, device=dev).repeat(b)
        out = packed_forward(model, params, input_ids.reshape(-1), cu, s, pos, backend=backend)
        return out.reshape(b, s, -1)
    return _varlen_forward(model, params, input_ids, attention_mask, backend=backend)
