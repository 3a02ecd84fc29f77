"""Single-op entry points on torch tensors, one C-ABI call each.

Names and argument meaning follow the inference branches of packed_encoders/ops.py
(`fused_layer_norm` 191-208, `fused_add_layer_norm` 303-314, `_linear` 290-300,
`fused_geglu` 275-280, `geglu_mlp` 317-319, `flash_attention_qkv_bshd` 485-532), so
the parity tests read like the reference's. `packed_forward` does not go through
these wrappers (it is one C call); they exist for callers that compose their own
pipeline and for per-kernel tests. All tensors must be CUDA bf16 and contiguous.
"""
from __future__ import annotations

import torch
from torch import Tensor

from . import _lib
from .errors import PackedEncodersError


def _bf16_cuda(t: Tensor, name: str) -> Tensor:
    if not t.is_cuda or t.dtype != torch.bfloat16:
        raise PackedEncodersError(f"{name} must be a CUDA bf16 tensor, got {t.dtype} on {t.device}")
    return t if t.is_contiguous() else t.contiguous()


def _index_cuda(t: Tensor, name: str, dtype: torch.dtype, like: Tensor) -> Tensor:
    """An index operand (`cu_seqlens`, `position_ids`, token ids): the library reads it as raw
    `dtype` data on the device of `like`, so anything else is refused here instead of being
    misread there (an int64 `cu_seqlens` would give wrong boundaries, a CPU tensor a host
    address inside a kernel)."""
    if not isinstance(t, Tensor) or not t.is_cuda:
        raise PackedEncodersError(f"{name} must be a CUDA tensor (this package has no CPU path)")
    if t.dtype != dtype:
        raise ValueError(f"{name} must have dtype {dtype}, got {t.dtype}")
    if t.device != like.device:
        raise PackedEncodersError(f"{name} is on {t.device}, the data it indexes on {like.device}")
    return t if t.is_contiguous() else t.contiguous()


class _Call:
    """Device guard + stream + status word for one library call."""

    def __init__(self, ref: Tensor):
        self.lib = _lib.load()
        self.device = ref.device
        self.guard = torch.cuda.device(self.device)

    def __enter__(self):
        self.guard.__enter__()
        self.stream = _lib.current_stream_ptr()
        return self

    def __exit__(self, *exc):
        return self.guard.__exit__(*exc)


_status_words: dict[int, Tensor] = {}


def status_word(device: torch.device) -> Tensor:
    idx = device.index if device.index is not None else torch.cuda.current_device()
    if idx not in _status_words:
        _status_words[idx] = torch.zeros(1, dtype=torch.int32, device=torch.device("cuda", idx))
    return _status_words[idx]


def check_status(device: torch.device) -> None:
    """Synchronise and raise if any kernel launched through this module reported a fault."""
    word = status_word(device)
    code = int(word.item())
    if code != 0:
        word.zero_()
        raise _lib.NativeLibraryError(f"a CUDA kernel reported status {code}")


def fused_layer_norm(x: Tensor, weight: Tensor, eps: float) -> Tensor:
    x = _bf16_cuda(x, "x")
    flat = x.reshape(-1, x.shape[-1])
    y = torch.empty_like(flat)
    with _Call(x) as c:
        _lib.check(c.lib.pe_add_ln(flat.data_ptr(), None, _bf16_cuda(weight, "weight").data_ptr(),
                                   float(eps), flat.shape[0], flat.shape[1], None, y.data_ptr(),
                                   c.stream), "pe_add_ln")
    return y.view(x.shape)


def fused_add_layer_norm(x: Tensor, residual: Tensor, weight: Tensor, eps: float) -> tuple[Tensor, Tensor]:
    """`x_new = x + residual` (rounded to bf16), `y = LN(x_new)`; returns `(x_new, y)`."""
    x = _bf16_cuda(x, "x")
    residual = _bf16_cuda(residual, "residual")
    flat = x.reshape(-1, x.shape[-1])
    x_new = torch.empty_like(flat)
    y = torch.empty_like(flat)
    with _Call(x) as c:
        _lib.check(c.lib.pe_add_ln(flat.data_ptr(), residual.reshape(flat.shape).data_ptr(),
                                   _bf16_cuda(weight, "weight").data_ptr(), float(eps),
                                   flat.shape[0], flat.shape[1], x_new.data_ptr(), y.data_ptr(),
                                   c.stream), "pe_add_ln")
    return x_new.view(x.shape), y.view(x.shape)


def embed_layer_norm(ids: Tensor, table: Tensor, weight: Tensor, eps: float) -> Tensor:
    """`LN(table[ids])`: the embedding prologue of packed_encoders/forward.py:472-476."""
    table = _bf16_cuda(table, "table")
    ids = _index_cuda(ids, "ids", torch.int64, table)
    out = torch.empty(ids.numel(), table.shape[1], dtype=torch.bfloat16, device=table.device)
    with _Call(table) as c:
        _lib.check(c.lib.pe_embed_ln(ids.data_ptr(), table.data_ptr(),
                                     _bf16_cuda(weight, "weight").data_ptr(), float(eps),
                                     ids.numel(), table.shape[1], table.shape[0], out.data_ptr(),
                                     status_word(table.device).data_ptr(), c.stream), "pe_embed_ln")
    return out.view(*ids.shape, table.shape[1])


def _linear(x: Tensor, weight: Tensor) -> Tensor:
    """`x @ weight.T`, weight `[out, in]` as `nn.Linear` stores it; no bias."""
    x = _bf16_cuda(x, "x")
    weight = _bf16_cuda(weight, "weight")
    flat = x.reshape(-1, x.shape[-1])
    out = torch.empty(flat.shape[0], weight.shape[0], dtype=torch.bfloat16, device=x.device)
    with _Call(x) as c:
        _lib.check(c.lib.pe_gemm_bf16_tn(flat.data_ptr(), weight.data_ptr(), out.data_ptr(),
                                         flat.shape[0], weight.shape[0], weight.shape[1],
                                         status_word(x.device).data_ptr(), c.stream),
                   "pe_gemm_bf16_tn")
    return out.view(*x.shape[:-1], weight.shape[0])


def fused_geglu(proj: Tensor) -> Tensor:
    proj = _bf16_cuda(proj, "proj")
    flat = proj.reshape(-1, proj.shape[-1])
    inter = flat.shape[1] // 2
    out = torch.empty(flat.shape[0], inter, dtype=torch.bfloat16, device=proj.device)
    with _Call(proj) as c:
        _lib.check(c.lib.pe_geglu(flat.data_ptr(), flat.shape[0], inter, out.data_ptr(), c.stream),
                   "pe_geglu")
    return out.view(*proj.shape[:-1], inter)


def linear_geglu(x: Tensor, wi: Tensor) -> Tensor:
    """`fused_geglu(_linear(x, wi))` as one kernel (the projection never reaches memory)."""
    x = _bf16_cuda(x, "x")
    wi = _bf16_cuda(wi, "wi")
    flat = x.reshape(-1, x.shape[-1])
    inter = wi.shape[0] // 2
    out = torch.empty(flat.shape[0], inter, dtype=torch.bfloat16, device=x.device)
    with _Call(x) as c:
        _lib.check(c.lib.pe_gemm_geglu_bf16(flat.data_ptr(), wi.data_ptr(), out.data_ptr(),
                                            flat.shape[0], inter, wi.shape[1],
                                            status_word(x.device).data_ptr(), c.stream),
                   "pe_gemm_geglu_bf16")
    return out.view(*x.shape[:-1], inter)


def geglu_mlp(x: Tensor, wi: Tensor, wo: Tensor) -> Tensor:
    return _linear(linear_geglu(x, wi), wo)


def rope_table(theta: float, max_positions: int, device) -> Tensor:
    """bf16 `[max_positions, 64]`: cos of the 32 frequencies, then sin."""
    table = torch.empty(max_positions, 64, dtype=torch.bfloat16, device=device)
    with _Call(table) as c:
        _lib.check(c.lib.pe_rope_table(float(theta), max_positions, table.data_ptr(), c.stream),
                   "pe_rope_table")
    return table


def rope_qk_inplace(qkv: Tensor, position_ids: Tensor, table: Tensor, n_heads: int) -> Tensor:
    """Rotate the q and k thirds of the fused `qkv [T, 3*n_heads*64]` in place."""
    if not qkv.is_contiguous():
        raise PackedEncodersError("qkv must be contiguous for the in-place rotation")
    qkv = _bf16_cuda(qkv, "qkv")
    pos = _index_cuda(position_ids, "position_ids", torch.int64, qkv)
    with _Call(qkv) as c:
        _lib.check(c.lib.pe_rope_qk_inplace(qkv.data_ptr(), pos.data_ptr(),
                                            _bf16_cuda(table, "table").data_ptr(), table.shape[0],
                                            qkv.shape[0], n_heads,
                                            status_word(qkv.device).data_ptr(), c.stream),
                   "pe_rope_qk_inplace")
    return qkv


def linear_qkv_rope(x: Tensor, wqkv: Tensor, position_ids: Tensor, table: Tensor, n_heads: int) -> Tensor:
    """`rope_qk_inplace(_linear(x, wqkv), ...)` as one kernel: the rotation runs in the GEMM epilogue."""
    x = _bf16_cuda(x, "x")
    wqkv = _bf16_cuda(wqkv, "wqkv")
    flat = x.reshape(-1, x.shape[-1])
    pos = _index_cuda(position_ids, "position_ids", torch.int64, x)
    out = torch.empty(flat.shape[0], 3 * n_heads * 64, dtype=torch.bfloat16, device=x.device)
    with _Call(x) as c:
        _lib.check(c.lib.pe_gemm_qkv_rope_bf16(flat.data_ptr(), wqkv.data_ptr(), out.data_ptr(),
                                               flat.shape[0], n_heads, wqkv.shape[1],
                                               pos.data_ptr(),
                                               _bf16_cuda(table, "table").data_ptr(), table.shape[0],
                                               status_word(x.device).data_ptr(), c.stream),
                   "pe_gemm_qkv_rope_bf16")
    return out


def linear_residual(x: Tensor, weight: Tensor, residual: Tensor, *, inplace: bool = False) -> Tensor:
    """`residual + _linear(x, weight)` with the projection rounded to bf16 before the add, as one
    kernel. `inplace=True` writes the sum over `residual`."""
    x = _bf16_cuda(x, "x")
    weight = _bf16_cuda(weight, "weight")
    residual = _bf16_cuda(residual, "residual")
    flat = x.reshape(-1, x.shape[-1])
    res = residual.reshape(flat.shape[0], weight.shape[0])
    out = res if inplace else torch.empty_like(res)
    with _Call(x) as c:
        _lib.check(c.lib.pe_gemm_residual_bf16(flat.data_ptr(), weight.data_ptr(), res.data_ptr(),
                                               out.data_ptr(), flat.shape[0], weight.shape[0],
                                               weight.shape[1], status_word(x.device).data_ptr(),
                                               c.stream), "pe_gemm_residual_bf16")
    return out.view(residual.shape)


def attention_varlen_qkv(qkv: Tensor, cu_seqlens: Tensor, max_seqlen: int, n_heads: int,
                         half_window: int | None) -> Tensor:
    """Varlen attention on the fused, already-rotated `qkv [T, 3*n_heads*64]`;
    `half_window=None` is full attention. Returns `[T, n_heads*64]`."""
    qkv = _bf16_cuda(qkv, "qkv")
    cu = _index_cuda(cu_seqlens, "cu_seqlens", torch.int32, qkv)
    total = qkv.shape[0]
    n_seqs = cu.numel() - 1
    out = torch.empty(total, n_heads * 64, dtype=torch.bfloat16, device=qkv.device)
    with _Call(qkv) as c:
        ws_bytes = int(c.lib.pe_attn_workspace_bytes(total, n_seqs))
        ws = torch.empty(ws_bytes, dtype=torch.uint8, device=qkv.device)
        _lib.check(c.lib.pe_attn_varlen(qkv.data_ptr(), cu.data_ptr(), n_seqs,
                                        total, n_heads, -1 if half_window is None else half_window,
                                        int(max_seqlen), out.data_ptr(), ws.data_ptr(), ws_bytes,
                                        status_word(qkv.device).data_ptr(), c.stream),
                   "pe_attn_varlen")
    return out


def attention_varlen_qkv_static(qkv: Tensor, cu_seqlens: Tensor, max_seqlen: int, n_heads: int,
                                half_window: int | None) -> Tensor:
    """`attention_varlen_qkv` through the entry point that brings its own scratch: for callers
    that cannot allocate device memory (a host process whose allocator owns the whole GPU, a
    request path with a frozen memory budget). At most 4096 sequences and 1,048,576 tokens;
    calls share one built-in table, so keep them on one stream. Only the output tensor is
    created here, by the caller's own allocator."""
    qkv = _bf16_cuda(qkv, "qkv")
    cu = _index_cuda(cu_seqlens, "cu_seqlens", torch.int32, qkv)
    total = qkv.shape[0]
    out = torch.empty(total, n_heads * 64, dtype=torch.bfloat16, device=qkv.device)
    with _Call(qkv) as c:
        _lib.check(c.lib.pe_attn_varlen_static(qkv.data_ptr(), cu.data_ptr(),
                                               cu.numel() - 1, total, n_heads,
                                               -1 if half_window is None else half_window,
                                               int(max_seqlen), out.data_ptr(),
                                               status_word(qkv.device).data_ptr(), c.stream),
                   "pe_attn_varlen_static")
    return out


def pool_packed(hidden: Tensor, cu_seqlens: Tensor, mode: str = "mean", normalize: bool = True) -> Tensor:
    """Sentence embeddings from the packed last hidden state, as the reference's callers compute
    them right after `packed_forward` (benchmarks/showcases/inference.py:193-206): per sequence
    the fp32 mean of its token rows (`mode="mean"`) or its first token (`mode="cls"`),
    optionally L2-normalised like `F.normalize`, rounded to bf16 last. `[T, H]` -> `[N, H]`."""
    if mode not in ("mean", "cls"):
        raise ValueError(f"pool_packed: mode must be 'mean' or 'cls', got {mode!r}")
    hidden = _bf16_cuda(hidden, "hidden")
    total, width = hidden.shape
    cu = _index_cuda(cu_seqlens, "cu_seqlens", torch.int32, hidden)
    n_seqs = cu.numel() - 1
    out = torch.empty(n_seqs, width, dtype=torch.bfloat16, device=hidden.device)
    with _Call(hidden) as c:
        ws_bytes = int(c.lib.pe_pool_workspace_bytes(total, n_seqs, width)) if mode == "mean" else 0
        ws = torch.empty(max(ws_bytes, 1), dtype=torch.uint8, device=hidden.device)
        _lib.check(c.lib.pe_pool_packed(hidden.data_ptr(), cu.data_ptr(), n_seqs, total, width,
                                        1 if mode == "mean" else 0, 1 if normalize else 0,
                                        out.data_ptr(), ws.data_ptr(), ws_bytes, c.stream),
                   "pe_pool_packed")
    return out


def project_normalize(hidden: Tensor, weight: Tensor) -> Tensor:
    """Token-level projection head: `F.normalize(F.linear(hidden, weight), p=2, dim=-1)` in one
    kernel, as the reference's ColBERT indexing path computes it after `packed_forward`
    (benchmarks/helpers/packed_index.py:182-186). `weight` is `[out_features <= 256, H]`."""
    hidden = _bf16_cuda(hidden, "hidden")
    weight = _bf16_cuda(weight, "weight")
    flat = hidden.reshape(-1, hidden.shape[-1])
    if weight.shape[0] > 256:
        raise ValueError("project_normalize: at most 256 output features (one tile holds whole rows)")
    out = torch.empty(flat.shape[0], weight.shape[0], dtype=torch.bfloat16, device=hidden.device)
    with _Call(hidden) as c:
        _lib.check(c.lib.pe_gemm_l2norm_bf16(flat.data_ptr(), weight.data_ptr(), out.data_ptr(),
                                             flat.shape[0], weight.shape[0], weight.shape[1],
                                             status_word(hidden.device).data_ptr(), c.stream),
                   "pe_gemm_l2norm_bf16")
    return out.view(*hidden.shape[:-1], weight.shape[0])
