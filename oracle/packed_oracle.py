"""CPU restatement of the reference's packed ModernBERT forward (TEST INFRASTRUCTURE).

This module is the checker for the CUDA library, never the product: only tests/,
bench.py's cpu_baseline / reference arm and __graft_entry__.smoke() import it.

Every function restates one piece of pau-mensa/flash-modernbert (`packed_encoders`)
in plain torch on the CPU, with the reference's rounding points: residual add rounded
to bf16 before the LayerNorm statistics, statistics in fp32 with var = E[x^2] - mean^2,
cos/sin tables stored in bf16, every GEMM / GeGLU / RoPE / attention output
materialised in bf16, softmax in fp32 with P rounded to bf16 before P*V. With
`faithful=False` the same functions run in plain fp32 (no intermediate rounding),
which is the HF-eager-fp32 arithmetic.

Pinned by tests/golden: the integer plumbing against outputs of the reference's own
`_unpad` / `_repad` / `pack_sequences` / `_rope_tables` run on the CPU, the model
against Hugging Face ModernBertModel eager fp32 (tests/golden/make_golden.py).
"""
from __future__ import annotations

import math

import numpy as np
import torch
import torch.nn.functional as F
from torch import Tensor

BF16 = torch.bfloat16


def _r(x: Tensor, faithful: bool) -> Tensor:
    """Round to bf16 and back to fp32 at a materialisation point."""
    return x.to(BF16).to(torch.float32) if faithful else x


# ---------------------------------------------------------------------------
# Integer plumbing (bit-exact)
# ---------------------------------------------------------------------------


def unpad(x: np.ndarray, attention_mask: np.ndarray):
    """packed_encoders/forward.py:384-403. Returns (x_packed, indices int64,
    cu_seqlens int32 [B+1], max_seqlen int, position_ids int64)."""
    mask = np.asarray(attention_mask)
    b, s = mask.shape
    seqlens = (mask != 0).sum(axis=1).astype(np.int32)
    indices = np.flatnonzero(mask.reshape(-1) != 0).astype(np.int64)
    cu_seqlens = np.zeros(b + 1, dtype=np.int32)
    cu_seqlens[1:] = np.cumsum(seqlens, dtype=np.int32)
    max_seqlen = int(seqlens.max()) if b else 0
    x = np.asarray(x)
    x_packed = x.reshape(b * s, *x.shape[2:])[indices]
    position_ids = indices % s
    return x_packed, indices, cu_seqlens, max_seqlen, position_ids


def repad(x_packed: np.ndarray, indices: np.ndarray, b: int, s: int) -> np.ndarray:
    """packed_encoders/forward.py:406-412: zeros, then rows scattered to `indices`."""
    x_packed = np.asarray(x_packed)
    out = np.zeros((b * s, x_packed.shape[-1]), dtype=x_packed.dtype)
    out[np.asarray(indices)] = x_packed
    return out.reshape(b, s, x_packed.shape[-1])


def pack_sequences(sequences):
    """benchmarks/helpers/packed_collator.py:68-96. Returns (ids int64 [T],
    cu_seqlens int32 [N+1], max_seqlen, position_ids int64 [T])."""
    seqs = [np.asarray(s, dtype=np.int64).reshape(-1) for s in sequences]
    if not seqs:
        raise ValueError("pack_sequences got no sequences")
    lens = np.asarray([s.size for s in seqs], dtype=np.int32)
    if lens.min() == 0:
        raise ValueError("pack_sequences got an empty sequence (length 0)")
    cu = np.zeros(len(seqs) + 1, dtype=np.int32)
    cu[1:] = np.cumsum(lens, dtype=np.int32)
    pos = np.concatenate([np.arange(int(n), dtype=np.int64) for n in lens])
    return np.concatenate(seqs), cu, int(lens.max()), pos


# ---------------------------------------------------------------------------
# Floating-point pieces
# ---------------------------------------------------------------------------


def rope_tables(seq_len: int, head_dim: int, theta: float, dtype=BF16):
    """packed_encoders/forward.py:40-51: (cos, sin), each [seq_len, head_dim], fp32 math
    then cast to `dtype`."""
    inv_freq = 1.0 / (theta ** (torch.arange(0, head_dim, 2, dtype=torch.float32) / head_dim))
    pos = torch.arange(seq_len, dtype=torch.float32)
    freqs = torch.outer(pos, inv_freq)
    emb = torch.cat((freqs, freqs), dim=-1)
    return emb.cos().to(dtype), emb.sin().to(dtype)


def layer_norm(x: Tensor, weight: Tensor, eps: float, faithful: bool = True) -> Tensor:
    """packed_encoders/_kernels/triton_layer_norm.py:26-59 without residual."""
    x = x.float()
    h = x.shape[-1]
    mean = x.sum(-1, keepdim=True) / h
    var = (x * x).sum(-1, keepdim=True) / h - mean * mean
    y = (x - mean) * torch.rsqrt(var + eps) * weight.float()
    return _r(y, faithful)


def add_layer_norm(x: Tensor, residual: Tensor, weight: Tensor, eps: float, faithful: bool = True):
    """packed_encoders/_kernels/triton_layer_norm.py:40-47: the sum is rounded to bf16
    before the statistics. Returns (x_new, y)."""
    x_new = _r(x.float() + residual.float(), faithful)
    return x_new, layer_norm(x_new, weight, eps, faithful)


def linear(x: Tensor, weight: Tensor, faithful: bool = True) -> Tensor:
    """packed_encoders/ops.py:290-300: y = x W^T, no bias, fp32 accumulation, bf16 out."""
    return _r(x.float() @ weight.float().t(), faithful)


def geglu(proj: Tensor, faithful: bool = True) -> Tensor:
    """packed_encoders/_kernels/triton_layer_norm.py:62-79: exact-erf GELU of the first half
    times the second half."""
    a, gate = proj.float().chunk(2, dim=-1)
    return _r(a * 0.5 * (1.0 + torch.erf(a * 0.7071067811865476)) * gate, faithful)


def rope_apply(x: Tensor, cos: Tensor, sin: Tensor, faithful: bool = True) -> Tensor:
    """packed_encoders/_kernels/rope.py:184-197 on x [T, heads, D] with per-token cos/sin
    [T, D]: out = x*cos + rotate_half(x)*sin, split-half pairing (j, j + D/2)."""
    x = x.float()
    half = x.shape[-1] // 2
    rotated = torch.cat((-x[..., half:], x[..., :half]), dim=-1)
    out = x * cos.float().unsqueeze(1) + rotated * sin.float().unsqueeze(1)
    return _r(out, faithful)


def attention(q: Tensor, k: Tensor, v: Tensor, cu_seqlens, half_window: int | None,
              scaling: float = 0.125, faithful: bool = True) -> Tensor:
    """Per-sequence softmax(q k^T * scaling + mask) v on [T, heads, D] tensors, the fp32
    reference of tests/test_packed_short_attention.py:33-46; `half_window` None = full,
    else keys with |i - j| <= half_window (packed_encoders/forward.py:65-69). In faithful
    mode P is rounded to bf16 before P*V as the kernels do
    (packed_encoders/_kernels/triton_packed_attention.py:129-132)."""
    bounds = [int(c) for c in np.asarray(cu_seqlens).tolist()]
    rows = []
    for start, end in zip(bounds, bounds[1:]):
        if end == start:
            continue
        qf, kf, vf = q[start:end].float(), k[start:end].float(), v[start:end].float()
        scores = torch.einsum("qhd,khd->hqk", qf, kf) * scaling
        if half_window is not None:
            pos = torch.arange(end - start)
            outside = (pos[:, None] - pos[None, :]).abs() > half_window
            scores = scores.masked_fill(outside.unsqueeze(0), float("-inf"))
        m = scores.amax(-1, keepdim=True)
        p = torch.exp(scores - m)
        denom = p.sum(-1, keepdim=True)
        ctx = torch.einsum("hqk,khd->qhd", _r(p, faithful), vf) / denom.permute(1, 0, 2)
        rows.append(ctx)
    return _r(torch.cat(rows), faithful)


# ---------------------------------------------------------------------------
# The model
# ---------------------------------------------------------------------------


def _is_global(layer, idx: int) -> bool:
    kind = getattr(layer, "attention_type", None)
    if kind == "full_attention":
        return True
    if kind == "sliding_attention":
        return False
    return idx % 3 == 0


def _thetas(config) -> tuple[float, float]:
    g = getattr(config, "global_rope_theta", None)
    l = getattr(config, "local_rope_theta", None)
    if g is None or l is None:
        table = getattr(config, "rope_parameters", None) or {}
        g = g or table.get("full_attention", {}).get("rope_theta", 160000.0)
        l = l or table.get("sliding_attention", {}).get("rope_theta", 10000.0)
    return float(g), float(l)


@torch.no_grad()
def packed_forward(model, packed_ids, cu_seqlens, max_seqlen: int, position_ids,
                   faithful: bool = True) -> Tensor:
    """packed_encoders/forward.py:415-516 (packed_forward) + 229-277 (core) + 161-226
    (_encoder_layer) on the CPU, reading weights off a Hugging Face ModernBertModel.
    Returns fp32 [T, H] holding bf16-representable values when `faithful`."""
    cfg = model.config
    nh = cfg.num_attention_heads
    hd = cfg.hidden_size // nh
    eps = float(cfg.norm_eps)
    half_window = int(cfg.local_attention) // 2
    ids = torch.as_tensor(np.asarray(packed_ids), dtype=torch.int64)
    pos = torch.as_tensor(np.asarray(position_ids), dtype=torch.int64)
    total = ids.shape[0]

    table_dtype = BF16 if faithful else torch.float32
    theta_g, theta_l = _thetas(cfg)
    cos_g, sin_g = rope_tables(max_seqlen, hd, theta_g, table_dtype)
    cos_l, sin_l = rope_tables(max_seqlen, hd, theta_l, table_dtype)
    cos_g, sin_g, cos_l, sin_l = (t.index_select(0, pos) for t in (cos_g, sin_g, cos_l, sin_l))

    emb = model.embeddings.tok_embeddings.weight.float().index_select(0, ids)
    x = layer_norm(_r(emb, faithful), model.embeddings.norm.weight, eps, faithful)

    pending = None
    for idx, layer in enumerate(model.layers):
        is_global = _is_global(layer, idx)
        cos, sin = (cos_g, sin_g) if is_global else (cos_l, sin_l)
        if isinstance(layer.attn_norm, torch.nn.Identity):
            if pending is not None:
                x = _r(x + pending, faithful)
            normed = x
        elif pending is None:
            normed = layer_norm(x, layer.attn_norm.weight, eps, faithful)
        else:
            x, normed = add_layer_norm(x, pending, layer.attn_norm.weight, eps, faithful)
        qkv = linear(normed, layer.attn.Wqkv.weight, faithful).view(total, 3, nh, hd)
        q = rope_apply(qkv[:, 0], cos, sin, faithful)
        k = rope_apply(qkv[:, 1], cos, sin, faithful)
        ctx = attention(q, k, qkv[:, 2], cu_seqlens, None if is_global else half_window,
                        hd ** -0.5, faithful).reshape(total, nh * hd)
        wo_out = linear(ctx, layer.attn.Wo.weight, faithful)
        x, normed = add_layer_norm(x, wo_out, layer.mlp_norm.weight, eps, faithful)
        act = geglu(linear(normed, layer.mlp.Wi.weight, faithful), faithful)
        pending = linear(act, layer.mlp.Wo.weight, faithful)
    if pending is None:
        return layer_norm(x, model.final_norm.weight, eps, faithful)
    return add_layer_norm(x, pending, model.final_norm.weight, eps, faithful)[1]


@torch.no_grad()
def hf_eager_packed(model, sequences) -> Tensor:
    """Hugging Face eager forward, one unpadded sequence at a time, concatenated to the
    packed `[T, H]` layout. `model` must be an fp32 CPU ModernBertModel built with
    attn_implementation="eager". This is the CPU baseline the bench reports."""
    outs = []
    for seq in sequences:
        ids = torch.as_tensor(np.asarray(seq), dtype=torch.int64).view(1, -1)
        outs.append(model(input_ids=ids, attention_mask=torch.ones_like(ids)).last_hidden_state[0])
    return torch.cat(outs)


@torch.no_grad()
def hf_eager_padded(model, input_ids: Tensor, attention_mask: Tensor) -> Tensor:
    """Hugging Face eager forward on a padded [B, S] batch; returns [B, S, H]."""
    return model(input_ids=input_ids, attention_mask=attention_mask).last_hidden_state


def pool(hidden: Tensor, cu_seqlens, mode: str = "mean", normalize: bool = True) -> Tensor:
    """Sentence embeddings from a packed hidden state, following
    benchmarks/showcases/inference.py:193-206 of the reference: segment sums in fp32
    (`index_add_` of `hidden.float()`), divided by the lengths, `F.normalize(p=2, dim=-1)`
    (eps 1e-12), cast to the hidden state's dtype last. `mode="cls"` takes the first token of
    each sequence instead of the mean. Zero-length sequences give zero rows."""
    cu = [int(v) for v in cu_seqlens]
    rows = []
    for b, e in zip(cu[:-1], cu[1:]):
        if e == b:
            rows.append(torch.zeros(hidden.shape[-1], dtype=torch.float32))
        elif mode == "cls":
            rows.append(hidden[b].float())
        else:
            rows.append(hidden[b:e].float().sum(0) / float(e - b))
    pooled = torch.stack(rows) if rows else torch.zeros(0, hidden.shape[-1])
    if normalize:
        pooled = torch.nn.functional.normalize(pooled, p=2, dim=-1)
    return pooled.to(hidden.dtype)


def project_normalize(hidden: Tensor, weight: Tensor) -> Tensor:
    """ColBERT-style token head, following benchmarks/helpers/packed_index.py:182-186 of the
    reference: a bias-free Dense projection of the token embeddings (computed and stored in the
    hidden state's dtype) followed by `F.normalize(p=2, dim=-1)` on that tensor."""
    y = (hidden.float() @ weight.float().t()).to(hidden.dtype)
    return torch.nn.functional.normalize(y, p=2, dim=-1)


def cosine_report(actual: Tensor, expected: Tensor) -> dict:
    """Per-token and flat cosine, and max-abs error, between two [T, H] tensors."""
    a, e = actual.float(), expected.float()
    per_tok = F.cosine_similarity(a, e, dim=-1)
    return {
        "min_token_cos": float(per_tok.min()),
        "mean_token_cos": float(per_tok.mean()),
        "flat_cos": float(F.cosine_similarity(a.flatten(), e.flatten(), dim=0)),
        "max_abs": float((a - e).abs().max()),
    }
