"""Per-model patch state, stored on the encoder as `encoder._packed_encoders`.

Same attribute name and the same role as packed_encoders/state.py:18-43: it keeps the
original forward (so unpack() can restore it and validate() has stock HF to compare
against) and the graph runners. The `binding` field is new: the C-ABI view of the
model's weights (pointer tables, RoPE tables, workspace arena).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Callable

from .config import ModernBertParams
from .errors import PackedEncodersError
from .locate import find_encoder

ATTR = "_packed_encoders"


@dataclass
class PatchState:
    params: ModernBertParams
    original_forward: Callable[..., Any]
    attention_backend: str = "cuda"
    graph_runner: Any = None          # padded [B, S] API runner (routes through the packed one)
    graph_enabled: bool = False
    graph_skip_warned: bool = False
    packed_graph_runner: Any = None   # graph._PackedGraphRunner | None
    train_graph_runner: Any = None    # always None: training graphs are out of scope
    train_graph_enabled: bool = False
    binding: Any = None               # forward.ModelBinding, built lazily


def get_state(target: object) -> PatchState:
    encoder = find_encoder(target)
    state = getattr(encoder, ATTR, None)
    if not isinstance(state, PatchState):
        raise PackedEncodersError("this model has not been patched with pack()")
    return state
