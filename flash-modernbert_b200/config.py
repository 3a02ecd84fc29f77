"""ModernBertParams: the few numbers of a HF ModernBERT config that the forward reads.

Mirrors packed_encoders/config.py:17-81 (field names, derived properties, both RoPE
config schemas). One deliberate difference: `global_attn_every_n_layers` is optional
on the HF config (transformers 5.x replaced it by `layer_types`); when it is absent
it is derived from `layer_types`, and per-layer globalness is always taken from the
layer module first (packed_encoders/forward.py:150-158).
"""
from __future__ import annotations

from dataclasses import dataclass

SUPPORTED_MODEL_TYPES = frozenset({"modernbert", "mmbert"})


@dataclass(frozen=True)
class ModernBertParams:
    hidden_size: int
    num_attention_heads: int
    num_hidden_layers: int
    norm_eps: float
    global_rope_theta: float
    local_rope_theta: float
    local_attention: int
    global_attn_every_n_layers: int

    @property
    def head_dim(self) -> int:
        heads = self.num_attention_heads
        if self.hidden_size % heads != 0:
            raise ValueError(
                f"hidden_size={self.hidden_size} is not divisible by num_attention_heads={heads}"
            )
        return self.hidden_size // heads

    @property
    def scaling(self) -> float:
        return self.head_dim ** -0.5

    @property
    def sliding_half_window(self) -> int:
        return self.local_attention // 2

    def is_global_layer(self, layer_idx: int) -> bool:
        return layer_idx % self.global_attn_every_n_layers == 0

    @classmethod
    def from_hf_config(cls, config) -> "ModernBertParams":
        model_type = getattr(config, "model_type", None)
        if model_type not in SUPPORTED_MODEL_TYPES:
            raise ValueError(
                "only ModernBERT-architecture checkpoints "
                f"{sorted(SUPPORTED_MODEL_TYPES)} are supported; got model_type={model_type!r}"
            )
        theta_g, theta_l = _rope_thetas(config)
        return cls(
            hidden_size=int(config.hidden_size),
            num_attention_heads=int(config.num_attention_heads),
            num_hidden_layers=int(config.num_hidden_layers),
            norm_eps=float(config.norm_eps),
            global_rope_theta=theta_g,
            local_rope_theta=theta_l,
            local_attention=int(config.local_attention),
            global_attn_every_n_layers=_global_every(config),
        )


def _global_every(config) -> int:
    every = getattr(config, "global_attn_every_n_layers", None)
    if every:
        return int(every)
    layer_types = getattr(config, "layer_types", None)
    if layer_types:
        full = [i for i, t in enumerate(layer_types) if t == "full_attention"]
        if len(full) >= 2:
            return full[1] - full[0]
        if len(full) == 1:
            return max(len(layer_types), 1)
    return 3


def _rope_thetas(config) -> tuple[float, float]:
    """(global, local) theta from either the flat attributes (transformers 4.x) or
    `rope_parameters[{full,sliding}_attention]` (transformers 5.x)."""
    theta_g = getattr(config, "global_rope_theta", None)
    theta_l = getattr(config, "local_rope_theta", None)
    if theta_g is None or theta_l is None:
        table = getattr(config, "rope_parameters", None)
        table = table if isinstance(table, dict) else {}
        default = getattr(config, "rope_theta", 160_000.0)
        theta_g = theta_g or table.get("full_attention", {}).get("rope_theta") or default
        theta_l = theta_l or table.get("sliding_attention", {}).get("rope_theta") or default
    return float(theta_g), float(theta_l)
