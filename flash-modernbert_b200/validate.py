"""validate(): the gate that decides whether the CUDA path may be enabled.

Gates 1, 2 and 4 of packed_encoders/validate.py:45-69: architecture
(`ModernBertParams.from_hf_config`), device (here: compute capability 10.x only, the
library carries sm_100a code alone) and numerics (the packed forward against the stock
HF forward at a few sequence lengths, flat cosine >= `cos_threshold`). The
reference's gate 3 checks its CuteDSL JIT toolchain; the equivalent here is that the
prebuilt library loads and resolves its driver entry point.
"""
from __future__ import annotations

from dataclasses import dataclass, field

import torch
import torch.nn.functional as F
from torch import Tensor, nn

from . import _lib, forward
from .config import ModernBertParams
from .errors import ValidationError
from .locate import find_encoder
from .state import ATTR

VALIDATED_CAPABILITIES = frozenset({(10, 0)})
DEFAULT_SEQ_LENS = (128, 512, 2048)
DEFAULT_COS_THRESHOLD = 0.997


@dataclass
class ValidationReport:
    model_type: str
    capability: tuple[int, int]
    library_version: int
    cosine: dict[int, float] = field(default_factory=dict)


def validate(
    target: object,
    *,
    seq_lens: tuple[int, ...] = DEFAULT_SEQ_LENS,
    cos_threshold: float = DEFAULT_COS_THRESHOLD,
) -> ValidationReport:
    """Run every gate; return a report or raise `ValidationError`."""
    encoder = find_encoder(target)
    try:
        params = ModernBertParams.from_hf_config(encoder.config)
    except ValueError as exc:
        raise ValidationError(str(exc)) from exc
    device = _encoder_device(encoder)
    capability = torch.cuda.get_device_capability(device)
    if capability not in VALIDATED_CAPABILITIES:
        raise ValidationError(
            f"compute capability sm_{capability[0]}{capability[1]} is not supported: the library "
            "is built for sm_100a (B200) only"
        )
    try:
        lib = _lib.load()
        with torch.cuda.device(device):
            _lib.check(lib.pe_device_check(), "pe_device_check")
    except _lib.NativeLibraryError as exc:
        raise ValidationError(str(exc)) from exc
    report = ValidationReport(encoder.config.model_type, capability, int(lib.pe_version()))
    _check_numerics(encoder, params, device, seq_lens, cos_threshold, report)
    return report


def _encoder_device(encoder: nn.Module) -> torch.device:
    try:
        device = next(encoder.parameters()).device
    except StopIteration as exc:
        raise ValidationError("the model has no parameters to validate") from exc
    if device.type != "cuda":
        raise ValidationError(
            f"the packed path requires CUDA weights; the model is on {device!r}. Move it to a GPU first."
        )
    return device


def _check_numerics(encoder, params, device, seq_lens, cos_threshold, report) -> None:
    dtype = next(encoder.parameters()).dtype
    if dtype != torch.bfloat16:
        raise ValidationError(f"the packed path requires bf16 weights; got {dtype}")
    vocab = int(encoder.config.vocab_size)
    generator = torch.Generator(device=device).manual_seed(0)
    stock = _stock_forward(encoder)
    max_pos = int(getattr(encoder.config, "max_position_embeddings", 8192))
    with torch.no_grad():
        for seq_len in seq_lens:
            if seq_len > max_pos:
                continue
            ids = torch.randint(5, vocab, (2, seq_len), generator=generator, device=device)
            mask = torch.ones((2, seq_len), dtype=torch.long, device=device)
            expected = stock(ids, mask)
            actual = forward.fused_forward(encoder, params, ids, mask)
            forward.get_binding(encoder, params).check(sync=True)
            cos = F.cosine_similarity(expected.flatten().float(), actual.flatten().float(), dim=0).item()
            report.cosine[seq_len] = cos
            if not cos >= cos_threshold:
                raise ValidationError(
                    f"packed forward diverged from stock HF at S={seq_len}: cosine {cos:.6f} < "
                    f"{cos_threshold}"
                )


def _stock_forward(encoder: nn.Module):
    state = getattr(encoder, ATTR, None)
    hf_forward = state.original_forward if state is not None else encoder.forward

    def run(ids: Tensor, mask: Tensor) -> Tensor:
        out = hf_forward(input_ids=ids, attention_mask=mask)
        return out.last_hidden_state if hasattr(out, "last_hidden_state") else out[0]

    return run
