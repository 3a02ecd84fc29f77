"""pack() / unpack(): install the CUDA forward on a live HF ModernBertModel, in place.

Keeps the reference's surface (packed_encoders/pack.py:28-36, 212-220, 224-297): the
same keyword arguments, idempotence, the `_packed_encoders` state attribute, the
patched `forward(input_ids, attention_mask, *, return_dict=True, **kwargs)` returning
`BaseModelOutput(last_hidden_state=[B, S, H])`, and the same refusals. Weights are
never copied or re-laid out. What differs: `attention_backend` no longer selects
anything (one CUDA kernel family), training graphs are refused, and graphs for the
padded API ride on the packed runner (unpad -> bucketed graph -> re-pad).
"""
from __future__ import annotations

import warnings

import torch
from torch import Tensor, nn
from transformers.modeling_outputs import BaseModelOutput

from . import _lib
from .config import ModernBertParams
from .errors import PackedEncodersError
from .forward import fused_forward, get_binding
from .graph import GraphConfig, build_packed_runner, build_runner, graphs_globally_disabled
from .locate import find_encoder
from .state import ATTR, PatchState
from .validate import validate as _validate

_ACCEPTED_BACKENDS = ("sdpa", "flash", "triton", "auto", "cuda")


def pack(
    target: object,
    *,
    cuda_graph: bool | GraphConfig = False,
    train_cuda_graph: object = False,
    cuda_graph_seq_cutoff: int = 64,
    attention_backend: str | None = None,
    validate: bool = True,
) -> object:
    """Patch the ModernBERT encoder inside `target` and return `target`.

    `cuda_graph=True` enables bucketed graphs for calls whose longest sequence is at
    most `cuda_graph_seq_cutoff`; a `GraphConfig` is used as given. `attention_backend`
    accepts the reference's names for source compatibility; every value resolves to the
    single sm_100a kernel family. `validate=True` runs the architecture / device /
    numerics gate first and raises `ValidationError` on a miss.
    """
    if attention_backend is not None and attention_backend not in _ACCEPTED_BACKENDS:
        raise PackedEncodersError(
            f"attention_backend must be one of {_ACCEPTED_BACKENDS} or None, got {attention_backend!r}"
        )
    if train_cuda_graph:
        raise PackedEncodersError(
            "train_cuda_graph: training-step graphs are not part of this inference-only build"
        )
    encoder = find_encoder(target)

    existing = getattr(encoder, ATTR, None)
    if existing is not None:
        if cuda_graph and existing.packed_graph_runner is None:
            _enable_graphs(encoder, existing, cuda_graph, cuda_graph_seq_cutoff)
        return target

    _lib.load()  # fail here, loudly, if the CUDA library was not built
    if validate:
        _validate(encoder)
    else:
        _require_cuda(encoder)

    params = ModernBertParams.from_hf_config(encoder.config)
    state = PatchState(params=params, original_forward=encoder.forward, attention_backend="cuda")
    setattr(encoder, ATTR, state)
    try:
        get_binding(encoder, params)  # checks dtype / device / bias-freeness of every weight
        if cuda_graph:
            _enable_graphs(encoder, state, cuda_graph, cuda_graph_seq_cutoff)
    except Exception:
        delattr(encoder, ATTR)
        raise
    encoder.forward = _make_forward(encoder, state)
    return target


def _enable_graphs(encoder: nn.Module, state: PatchState, cuda_graph: bool | GraphConfig,
                   seq_cutoff: int | None) -> None:
    config = cuda_graph if isinstance(cuda_graph, GraphConfig) else GraphConfig(max_seq=seq_cutoff)
    state.packed_graph_runner = build_packed_runner(encoder, state.params, config)
    state.graph_runner = build_runner(encoder, state.params, config)
    state.graph_enabled = True


def unpack(target: object) -> object:
    """Restore the stock forward and drop the patch state (and its device buffers)."""
    encoder = find_encoder(target)
    state = getattr(encoder, ATTR, None)
    if state is None:
        return target
    encoder.forward = state.original_forward
    delattr(encoder, ATTR)
    return target


def _make_forward(encoder: nn.Module, state: PatchState):
    def forward(
        input_ids: Tensor | None = None,
        attention_mask: Tensor | None = None,
        *,
        return_dict: bool = True,
        **kwargs,
    ):
        if input_ids is None:
            raise NotImplementedError("input_ids is required (inputs_embeds is unsupported)")
        _reject_unsupported(kwargs)
        wants_graph = (
            state.packed_graph_runner is not None
            and state.graph_enabled
            and not graphs_globally_disabled()
        )
        if (
            wants_graph
            and (torch.is_grad_enabled() or torch.is_autocast_enabled("cuda"))
            and not state.graph_skip_warned
        ):
            state.graph_skip_warned = True
            warnings.warn(
                "CUDA graphs are enabled but skipped because autograd or autocast is active; "
                "they apply to plain bf16 inference under torch.no_grad().",
                stacklevel=2,
            )
        use_graph = (
            wants_graph
            and state.graph_runner is not None
            and not torch.is_grad_enabled()
            and not torch.is_autocast_enabled("cuda")
            and input_ids.is_cuda
            and input_ids.dim() == 2
        )
        if use_graph:
            hidden = state.graph_runner(input_ids.to(torch.int64), attention_mask)
        else:
            hidden = fused_forward(encoder, state.params, input_ids, attention_mask)
        if not return_dict:
            return (hidden,)
        return BaseModelOutput(last_hidden_state=hidden)

    return forward


def _reject_unsupported(kwargs: dict) -> None:
    if kwargs.get("inputs_embeds") is not None:
        raise NotImplementedError("inputs_embeds is not supported")
    if kwargs.get("output_attentions"):
        raise NotImplementedError("output_attentions is not supported")
    if kwargs.get("output_hidden_states"):
        raise NotImplementedError("output_hidden_states is not supported")
    token_type_ids = kwargs.get("token_type_ids")
    if token_type_ids is not None and bool(token_type_ids.any()):
        raise NotImplementedError("non-zero token_type_ids are not supported")


def _require_cuda(encoder: nn.Module) -> None:
    try:
        device = next(encoder.parameters()).device
    except StopIteration as exc:
        raise PackedEncodersError("the model has no parameters") from exc
    if device.type != "cuda":
        raise PackedEncodersError(f"the packed path requires CUDA weights; the model is on {device!r}")
