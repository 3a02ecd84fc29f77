"""find_encoder: reach the ModernBertModel inside whatever the caller holds.

Same search as packed_encoders/locate.py:18-60: the object itself, then element 0
of an indexable container (SentenceTransformer / PyLate pipelines), then the usual
wrapper attributes, at most four levels deep; an unknown container raises instead
of guessing.
"""
from __future__ import annotations

from torch import nn

from .config import SUPPORTED_MODEL_TYPES
from .errors import UnsupportedTargetError

_WRAPPER_ATTRS = ("auto_model", "model", "modernbert", "bert", "encoder")
_MAX_DEPTH = 4


def is_modernbert_encoder(module: object) -> bool:
    if not isinstance(module, nn.Module):
        return False
    model_type = getattr(getattr(module, "config", None), "model_type", None)
    if model_type not in SUPPORTED_MODEL_TYPES:
        return False
    return all(hasattr(module, name) for name in ("embeddings", "layers", "final_norm"))


def find_encoder(target: object, *, _depth: int = 0) -> nn.Module:
    if is_modernbert_encoder(target):
        return target  # type: ignore[return-value]
    if _depth < _MAX_DEPTH:
        for candidate in _children(target):
            try:
                return find_encoder(candidate, _depth=_depth + 1)
            except UnsupportedTargetError:
                continue
    raise UnsupportedTargetError(
        f"no ModernBERT encoder found in {type(target).__name__!r}: pass a Hugging Face "
        "ModernBertModel, a SentenceTransformer / PyLate model wrapping one, or a task model "
        "that exposes it as .auto_model / .model"
    )


def _children(target: object):
    if hasattr(target, "__getitem__"):
        try:
            first = target[0]
        except (KeyError, IndexError, TypeError):
            first = None
        if first is not None and first is not target:
            yield first
    for attr in _WRAPPER_ATTRS:
        sub = getattr(target, attr, None)
        if isinstance(sub, nn.Module) and sub is not target:
            yield sub
