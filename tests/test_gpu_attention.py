"""Varlen attention against the fp32 per-sequence reference (the oracle restates
tests/test_packed_short_attention.py:33-46 of the reference), through the C ABI."""
from __future__ import annotations

import pytest
import torch

from oracle import packed_oracle as O

pytestmark = pytest.mark.gpu

EDGE_LENGTHS = [1, 2, 31, 32, 33, 63, 64, 65, 127, 128, 129, 191, 192, 193, 257, 700]


def _qkv(lengths, n_heads, device, seed=0, scale=1.0):
    gen = torch.Generator().manual_seed(seed)
    total = sum(lengths)
    qkv = torch.randn(total, 3, n_heads, 64, generator=gen)
    qkv[:, 0] *= scale
    qkv = qkv.to(torch.bfloat16)
    cu = torch.zeros(len(lengths) + 1, dtype=torch.int32)
    cu[1:] = torch.tensor(lengths).cumsum(0)
    return qkv, cu


def _run(qkv, cu, n_heads, half_window, device, max_seqlen=None):
    from flash_modernbert_b200 import ops

    lengths = (cu[1:] - cu[:-1]).tolist()
    flat = qkv.reshape(qkv.shape[0], -1).to(device)
    return ops.attention_varlen_qkv(flat, cu.to(device), max_seqlen or max(lengths), n_heads, half_window)


def _check(out, qkv, cu, half_window, what):
    ref = O.attention(qkv[:, 0], qkv[:, 1], qkv[:, 2], cu, half_window, faithful=False)
    got = out.cpu().float().view_as(ref)
    err = (got - ref).abs()
    rep = O.cosine_report(got.reshape(got.shape[0], -1), ref.reshape(ref.shape[0], -1))
    assert float(err.max()) < 0.03 and float(err.mean()) < 2e-3, (what, float(err.max()), float(err.mean()))
    assert rep["min_token_cos"] > 0.9995, (what, rep)


@pytest.mark.parametrize("half_window", [None, 64])
def test_ragged_and_tile_edges(pe, cuda_device, half_window):
    qkv, cu = _qkv(EDGE_LENGTHS, 12, cuda_device)
    out = _run(qkv, cu, 12, half_window, cuda_device)
    _check(out, qkv, cu, half_window, f"edges window={half_window}")


@pytest.mark.parametrize("lengths", [[5], [16, 3, 16, 1], [32, 20, 7, 32], [48, 8, 30, 41, 19], [96, 65, 64, 80, 1]])
@pytest.mark.parametrize("half_window", [None, 64])
def test_short_query_tiles(pe, cuda_device, lengths, half_window):
    """max_seqlen <= 16 / <= 32 / <= 64 select the 16-, 32- and 64-row register-tiled kernels;
    longer batches take the 128-row tensor-memory kernel (the other tests)."""
    qkv, cu = _qkv(lengths, 4, cuda_device, seed=1)
    out = _run(qkv, cu, 4, half_window, cuda_device)
    _check(out, qkv, cu, half_window, f"short {lengths}")


@pytest.mark.parametrize("n_heads", [1, 3, 6, 28])
def test_short_tiles_shared_among_heads(pe, cuda_device, n_heads):
    """A sequence of at most 16 (32) tokens shares its 64-row tile among four (two) heads, four heads
    to a CTA: head counts that leave slots of the last step empty (1, 3, 6) and one that fills
    several CTAs per tile (28), lengths on both sides of 16 / 32 / 48, with and without a band."""
    lengths = [1, 15, 16, 17, 31, 32, 33, 47, 48, 49, 64, 9, 24]
    qkv, cu = _qkv(lengths, n_heads, cuda_device, seed=31)
    for hw in (None, 64, 5):
        _check(_run(qkv, cu, n_heads, hw, cuda_device), qkv, cu, hw, f"shared tiles heads={n_heads} window={hw}")
    short = [l for l in lengths if l <= 32]
    qkv, cu = _qkv(short, n_heads, cuda_device, seed=32)      # 32-row tiles: two heads per step at most
    _check(_run(qkv, cu, n_heads, None, cuda_device), qkv, cu, None, f"shared 32-row tiles heads={n_heads}")


def test_small_window_and_long_sequence(pe, cuda_device):
    qkv, cu = _qkv([2048, 5, 900], 2, cuda_device, seed=2)
    for hw in (None, 64, 8):
        _check(_run(qkv, cu, 2, hw, cuda_device), qkv, cu, hw, f"long window={hw}")


@pytest.mark.parametrize("scale", [0.01, 1.0, 8.0])
def test_deterministic_and_finite(pe, cuda_device, scale):
    # tests/test_packed_short_attention.py:95-107 of the reference
    qkv, cu = _qkv([100, 37, 128], 12, cuda_device, seed=3, scale=scale)
    a = _run(qkv, cu, 12, 64, cuda_device)
    b = _run(qkv, cu, 12, 64, cuda_device)
    assert torch.equal(a, b) and bool(torch.isfinite(a.float()).all())


@pytest.mark.parametrize("q_scale", [8.0, 40.0])
def test_row_maximum_drifts_far_between_key_tiles(pe, cuda_device, q_scale):
    """Scores spread over hundreds of log2 units, so the running row maximum jumps by more
    than 2^8 (the accumulator is rescaled) and by more than 2^60 (a key tile is redone against
    a new reference) from one 128-key tile to the next, upwards, and downwards from the initial
    reference.  Some rows get a strongly negative offset so that every score is far below 0."""
    qkv, cu = _qkv([700, 300, 130], 4, cuda_device, seed=11, scale=q_scale)
    q = qkv[:, 0].float()
    k = qkv[:, 1].float()
    # keys 0..199 of the first sequence anti-aligned with its queries' mean direction: low scores
    # early, high scores late
    d = q[:700].mean(0, keepdim=True)
    k[:200] -= 0.5 * d / d.norm(dim=-1, keepdim=True) * 8
    qkv[:, 1] = k.to(torch.bfloat16)
    # second sequence: every score against its first 128 keys is about -1000 (2^-190 after
    # scaling), against the rest about 0 - the first tile lies far below the initial reference,
    # the second far above the first
    gen = torch.Generator().manual_seed(12)
    qkv[700:1000, 0] = (4.1 + 0.1 * torch.randn(300, 4, 64, generator=gen)).to(torch.bfloat16)
    qkv[700:828, 1] = (-4.1 + 0.1 * torch.randn(128, 4, 64, generator=gen)).to(torch.bfloat16)
    qkv[828:1000, 1] = (0.02 * torch.randn(172, 4, 64, generator=gen)).to(torch.bfloat16)
    for hw in (None, 200, 64):   # 64: the sliding-window kernel's exact-maximum fallback
        out = _run(qkv, cu, 4, hw, cuda_device)
        ref = O.attention(qkv[:, 0], qkv[:, 1], qkv[:, 2], cu, hw, faithful=False)
        got = out.cpu().float().view_as(ref)
        assert bool(torch.isfinite(got).all())
        rep = O.cosine_report(got.reshape(got.shape[0], -1), ref.reshape(ref.shape[0], -1))
        # near-one-hot softmax rows: P's bf16 rounding decides ties, so compare directions
        assert rep["min_token_cos"] > 0.995 and rep["mean_token_cos"] > 0.9995, (q_scale, hw, rep)


def test_window_score_far_above_the_rows_own_keys(pe, cuda_device):
    """Every query of two interior tiles scores about -1000 against the keys near it (2^-180
    after scaling) and about 0 against a few keys further back in its window, so a reference
    exponent taken from nearby keys is off by far more than 2^60.  Sliding-window layers: the
    cheap unmasked reference is refused and the exact masked maximum taken.  Full attention over
    the same data: first key tiles vanish against the initial reference, later ones overflow the
    inherited one - both send the warp through the by-hand path."""
    qkv, cu = _qkv([900, 260], 4, cuda_device, seed=21)
    gen = torch.Generator().manual_seed(22)
    qkv[256:512, 0] = (4.0 + 0.1 * torch.randn(256, 4, 64, generator=gen)).to(torch.bfloat16)
    qkv[230:512, 1] = (-4.0 + 0.1 * torch.randn(282, 4, 64, generator=gen)).to(torch.bfloat16)
    qkv[300:330, 1] = (0.02 * torch.randn(30, 4, 64, generator=gen)).to(torch.bfloat16)   # the keys that win
    qkv[420:424, 1] = (0.02 * torch.randn(4, 4, 64, generator=gen)).to(torch.bfloat16)
    for hw in (64, None):
        out = _run(qkv, cu, 4, hw, cuda_device)
        ref = O.attention(qkv[:, 0], qkv[:, 1], qkv[:, 2], cu, hw, faithful=False)
        got = out.cpu().float().view_as(ref)
        assert bool(torch.isfinite(got).all())
        rep = O.cosine_report(got.reshape(got.shape[0], -1), ref.reshape(ref.shape[0], -1))
        assert rep["min_token_cos"] > 0.995 and rep["mean_token_cos"] > 0.9995, (hw, rep)
        # rows that see none of the winning keys are ordinary rows: tight agreement
        calm = torch.cat([torch.arange(0, 200), torch.arange(600, 1160)])
        assert float((got[calm] - ref[calm]).abs().max()) < 0.03


@pytest.mark.parametrize("half_window", [None, 64])
def test_no_cross_sequence_leakage(pe, cuda_device, half_window):
    # tests/test_packed_short_attention.py:110-124 of the reference
    qkv, cu = _qkv([70, 45, 130], 12, cuda_device, seed=4)
    base = _run(qkv, cu, 12, half_window, cuda_device)
    other = qkv.clone()
    other[70:, 1:] *= 100                                   # K and V of the other sequences
    out = _run(other, cu, 12, half_window, cuda_device)
    assert torch.equal(out[:70], base[:70])


def test_trailing_empty_sequences_and_padding_tokens(pe, cuda_device):
    """Graph buckets: cu_seqlens padded with repeats of T, tokens beyond cu[-1] ignored."""
    qkv, cu = _qkv([40, 25], 4, cuda_device, seed=5)
    base = _run(qkv, cu, 4, None, cuda_device)
    padded_qkv = torch.cat([qkv, torch.randn(63, 3, 4, 64).to(torch.bfloat16)])
    padded_cu = torch.cat([cu, torch.full((5,), 65, dtype=torch.int32)])
    out = _run(padded_qkv, padded_cu, 4, None, cuda_device, max_seqlen=64)
    assert torch.equal(out[:65], base)


def test_full_size_properties(pe, cuda_device):
    """cfg3 lengths (306,851 tokens, longest 8192), 12 heads: spot-check sequences against
    the reference and check that uniform V gives V back (softmax rows sum to one)."""
    from oracle import synthetic as S

    lengths = S.workload("cfg3").sorted_by_length().lengths
    total = sum(lengths)
    gen = torch.Generator(device=cuda_device).manual_seed(0)
    qkv = torch.randn(total, 3, 12, 64, device=cuda_device, generator=gen).to(torch.bfloat16)
    cu = torch.zeros(len(lengths) + 1, dtype=torch.int32)
    cu[1:] = torch.tensor(lengths).cumsum(0)
    from flash_modernbert_b200 import ops

    for hw in (None, 64):
        out = ops.attention_varlen_qkv(qkv.view(total, -1), cu.to(cuda_device), max(lengths), 12, hw)
        for n in (3, 17, 300, len(lengths) - 1):           # long, mid, short, shortest
            s, e = int(cu[n]), int(cu[n + 1])
            sub = qkv[s:e, :, 4:7].cpu()                    # three of the twelve heads
            ref = O.attention(sub[:, 0], sub[:, 1], sub[:, 2], [0, e - s], hw, faithful=False)
            got = out[s:e].view(e - s, 12, 64)[:, 4:7].cpu().float()
            err = (got - ref).abs()
            assert float(err.max()) < 0.03, (hw, n, float(err.max()))
    const_v = qkv.clone()
    const_v[:, 2] = 0.5
    out = ops.attention_varlen_qkv(const_v.view(total, -1), cu.to(cuda_device), max(lengths), 12, 64)
    assert float((out.float() - 0.5).abs().max()) < 4e-3


@pytest.mark.parametrize("half_window", [None, 64])
def test_mixed_window_of_queries_and_documents(pe, cuda_device, half_window):
    """A serving window that mixes ~30-token queries with documents
    (benchmarks/showcases/mixed_serving.py:151-193 of the reference): the schedule sends the
    sequences of at most 64 tokens to the register-tiled kernel and the rest to the tensor-memory
    kernels, inside one call. Checked against the fp32 reference, and the queries' rows are
    bit-equal to the same queries encoded without the documents."""
    lengths = [30, 700, 8, 48, 129, 64, 65, 17, 2048, 41, 1, 300, 33]
    qkv, cu = _qkv(lengths, 4, cuda_device, seed=21)
    out = _run(qkv, cu, 4, half_window, cuda_device)
    _check(out, qkv, cu, half_window, f"mixed window={half_window}")
    short = [i for i, n in enumerate(lengths) if n <= 64]
    bounds = cu.tolist()
    rows = torch.cat([torch.arange(bounds[i], bounds[i + 1]) for i in short])
    q_short = qkv[rows]
    cu_short = torch.zeros(len(short) + 1, dtype=torch.int32)
    cu_short[1:] = torch.tensor([lengths[i] for i in short]).cumsum(0)
    alone = _run(q_short, cu_short, 4, half_window, cuda_device, max_seqlen=64)
    assert torch.equal(out[rows.to(cuda_device)], alone)


def test_bad_cu_seqlens_is_clamped_and_reported(pe, cuda_device):
    """A cu_seqlens whose entries run past the T given to the call (or backwards) must not make
    any kernel leave the caller's buffers: the schedule clamps the boundaries, the call reports
    status 303, and rows at or beyond T stay untouched. qkv and out are allocated for the larger
    claimed count, so that even an unguarded kernel would stay inside its own allocations."""
    from flash_modernbert_b200 import _lib, ops

    lib = _lib.load()
    nh, claimed, given = 2, 1024, 640
    gen = torch.Generator().manual_seed(3)
    qkv = torch.randn(claimed, 3 * nh * 64, generator=gen).to(torch.bfloat16).to(cuda_device)
    for cu_list in ([0, 300, 700, 1024], [0, 500, 400, 640], [-5, 200, 640, 640]):
        cu = torch.tensor(cu_list, dtype=torch.int32, device=cuda_device)
        out = torch.full((claimed, nh * 64), 7.0, dtype=torch.bfloat16, device=cuda_device)
        status = torch.zeros(1, dtype=torch.int32, device=cuda_device)
        ws_bytes = int(lib.pe_attn_workspace_bytes(given, len(cu_list) - 1))
        ws = torch.empty(ws_bytes, dtype=torch.uint8, device=cuda_device)
        rc = lib.pe_attn_varlen(qkv.data_ptr(), cu.data_ptr(), len(cu_list) - 1, given, nh, -1, 512,
                                out.data_ptr(), ws.data_ptr(), ws_bytes, status.data_ptr(),
                                _lib.current_stream_ptr())
        assert rc == 0, _lib.last_error()
        torch.cuda.synchronize()
        assert int(status.item()) == 303, (cu_list, int(status.item()))
        assert bool((out[given:] == 7.0).all()), cu_list           # nothing written past T
        assert bool(torch.isfinite(out[:given].float()).all())
    # a consistent table reports nothing
    cu = torch.tensor([0, 300, 640], dtype=torch.int32, device=cuda_device)
    status.zero_()
    out = ops.attention_varlen_qkv(qkv[:given].contiguous(), cu, 340, nh, None)
    ops.check_status(cuda_device)


def test_index_operands_are_validated(pe, cuda_device):
    """int64 cu_seqlens, CPU position_ids and the like are refused before any kernel sees them."""
    from flash_modernbert_b200 import ops

    qkv = torch.zeros(16, 3 * 64, dtype=torch.bfloat16, device=cuda_device)
    with pytest.raises(ValueError, match="int32"):
        ops.attention_varlen_qkv(qkv, torch.tensor([0, 16], device=cuda_device), 16, 1, None)
    with pytest.raises(pe.PackedEncodersError, match="CUDA"):
        ops.attention_varlen_qkv(qkv, torch.tensor([0, 16], dtype=torch.int32), 16, 1, None)
    table = ops.rope_table(10000.0, 64, cuda_device)
    with pytest.raises(pe.PackedEncodersError, match="CUDA"):
        ops.rope_qk_inplace(qkv, torch.arange(16), table, 1)
    with pytest.raises(ValueError, match="int64"):
        ops.rope_qk_inplace(qkv, torch.arange(16, dtype=torch.int32, device=cuda_device), table, 1)
    emb = torch.zeros(32, 64, dtype=torch.bfloat16, device=cuda_device)
    with pytest.raises(ValueError, match="int64"):
        ops.embed_layer_norm(torch.zeros(4, dtype=torch.int32, device=cuda_device), emb, emb[0], 1e-5)
