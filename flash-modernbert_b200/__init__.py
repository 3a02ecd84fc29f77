"""B200-native padding-free ModernBERT inference forward behind the packed-encoders API.

    import flash_modernbert_b200 as pe
    pe.pack(model)                                   # patch a live HF ModernBertModel
    pe.pack(model, cuda_graph=pe.GraphConfig(max_batch=1024, max_seq=64))
    out = pe.packed_forward(encoder, params, ids, cu_seqlens, max_seqlen, position_ids)
    pe.unpack(model)

The directory name carries a hyphen, so load it under the module name
`flash_modernbert_b200` (tests/conftest.py, bench.py and __graft_entry__.py show the
three-line importlib recipe). All device work happens in libpe_b200.so (hand-written
sm_100a CUDA behind a C ABI, include/pe_b200.h); there is no fallback path.
"""
from __future__ import annotations

from .collate import (PackedBatch, ServingWindow, encode_in_batches, encode_window, mixed_windows,
                      pack_sequences, plan_windows, token_budget_batches)
from .config import ModernBertParams
from .errors import PackedEncodersError, UnsupportedTargetError, ValidationError
from .forward import fused_forward, packed_forward, packed_forward_pooled
from .graph import GraphConfig, no_cuda_graph, set_cuda_graph
from .locate import find_encoder
from .pack import pack, unpack
from .state import PatchState, get_state
from .validate import ValidationReport, validate

__all__ = [
    "pack",
    "unpack",
    "validate",
    "ValidationReport",
    "GraphConfig",
    "set_cuda_graph",
    "no_cuda_graph",
    "packed_forward",
    "packed_forward_pooled",
    "fused_forward",
    "ModernBertParams",
    "PatchState",
    "get_state",
    "find_encoder",
    "pack_sequences",
    "PackedBatch",
    "token_budget_batches",
    "encode_in_batches",
    "ServingWindow",
    "mixed_windows",
    "plan_windows",
    "encode_window",
    "PackedEncodersError",
    "UnsupportedTargetError",
    "ValidationError",
]
