"""Parity of the memory-bound kernels with the CPU oracle and the golden fixtures,
through the C ABI, on a B200."""
from __future__ import annotations

import numpy as np
import pytest
import torch

from oracle import packed_oracle as O

pytestmark = pytest.mark.gpu

UNPAD_CASES = [
    "ref_lengths_5_2_4", "ref_roundtrip", "ref_no_padding", "single_token", "left_padded",
    "holes", "one_empty_row", "rand_32x485", "rand_7x1000", "rand_300x33",
]


def _bits(t: torch.Tensor) -> torch.Tensor:
    return t.contiguous().view(torch.int16).to(torch.int32)


def assert_bf16_close(actual, expected_f32, max_ulp=1, max_frac=0.02, what="", atol=0.0):
    """`actual` bf16 CUDA vs an fp32 CPU tensor of bf16-representable values: equal except
    for at most `max_frac` of the elements, each within `max_ulp` bf16 steps (or within
    `atol` in value, for results that sit next to zero after a cancellation)."""
    a = actual.detach().cpu()
    e = expected_f32.to(torch.bfloat16)
    ulp = (_bits(a) - _bits(e)).abs()
    # bit distance is meaningful where the signs agree; tiny values across zero are compared in value
    same_sign = (a.float() * e.float()) >= 0
    bad = (ulp > max_ulp) & same_sign & ((a.float() - e.float()).abs() > atol)
    cross = (~same_sign) & ((a.float() - e.float()).abs() > 1e-2)
    assert not bool(bad.any() or cross.any()), (
        f"{what}: {int(bad.sum())} elements off by more than {max_ulp} ulp; "
        f"max abs {float((a.float() - e.float()).abs().max())}")
    frac = float((ulp > 0).float().mean())
    assert frac <= max(max_frac, 1.5 / ulp.numel()), f"{what}: {frac:.4f} of the elements differ in the last bit"


@pytest.mark.parametrize("case", UNPAD_CASES)
@pytest.mark.parametrize("mask_dtype", [torch.int64, torch.int32, torch.bool])
def test_unpad_repad_bit_exact(pe, cuda_device, golden_dir, case, mask_dtype):
    from flash_modernbert_b200 import forward

    g = np.load(golden_dir / "unpad_cases.npz")
    mask = torch.from_numpy(g[f"{case}.mask"]).to(cuda_device).to(mask_dtype)
    x = torch.from_numpy(g[f"{case}.x"]).to(cuda_device)
    xp, idx, cu, max_s, pos = forward._unpad(x, mask)
    assert idx.dtype == torch.int64 and cu.dtype == torch.int32 and pos.dtype == torch.int64
    assert np.array_equal(idx.cpu().numpy(), g[f"{case}.indices"])
    assert np.array_equal(cu.cpu().numpy(), g[f"{case}.cu_seqlens"])
    assert max_s == int(g[f"{case}.max_seqlen"])
    assert np.array_equal(pos.cpu().numpy(), g[f"{case}.position_ids"])
    assert np.array_equal(xp.cpu().numpy(), g[f"{case}.x_packed"])
    b, s = mask.shape
    rep = forward._repad(xp, idx, b, s)
    assert np.array_equal(rep.cpu().numpy(), g[f"{case}.repad"])


def test_unpad_repad_large_roundtrip(pe, cuda_device):
    """cfg3-sized padded batch: 512 x 8192 mask, bf16 rows of 768 - size-independent properties."""
    from flash_modernbert_b200 import forward
    from oracle import synthetic as S

    lengths = torch.tensor(S.workload("cfg3").lengths, device=cuda_device)
    b, s = lengths.numel(), int(lengths.max())
    mask = (torch.arange(s, device=cuda_device)[None, :] < lengths[:, None]).to(torch.int64)
    ids = torch.randint(5, 50368, (b, s), device=cuda_device)
    packed_ids, idx, cu, max_s, pos = forward._unpad(ids.unsqueeze(-1), mask)
    assert packed_ids.shape[0] == 306851 and max_s == 8192 and int(cu[-1]) == 306851
    assert torch.equal(cu[1:] - cu[:-1], lengths.to(torch.int32))
    assert bool((idx[1:] > idx[:-1]).all())                               # ascending
    assert torch.equal(pos, idx % s)
    assert torch.equal(packed_ids.squeeze(-1), ids.reshape(-1)[idx])
    x = torch.randn(packed_ids.shape[0], 768, device=cuda_device).to(torch.bfloat16)
    rep = forward._repad(x, idx, b, s)
    assert torch.equal(rep.reshape(b * s, 768)[idx], x)                   # real rows recovered
    assert int(rep.reshape(b * s, 768).ne(0).any(dim=1).sum()) <= x.shape[0]
    pad_rows = torch.ones(b * s, dtype=torch.bool, device=cuda_device)
    pad_rows[idx] = False
    assert not bool(rep.reshape(b * s, 768)[pad_rows].ne(0).any())        # pad rows exactly zero


@pytest.mark.parametrize("rows,hidden", [(17, 768), (1, 768), (1000, 1024), (333, 1792), (5, 256), (64, 2048)])
def test_add_layer_norm(pe, cuda_device, rows, hidden):
    # tests/test_residual_layer_norm.py:15-40 of the reference: x_new bit-exact; y against the
    # oracle (same formula) up to the last bf16 bit, and against torch's own bf16 layer_norm
    from flash_modernbert_b200 import ops

    torch.manual_seed(0)
    x = torch.randn(rows, hidden).to(torch.bfloat16)
    res = torch.randn(rows, hidden).to(torch.bfloat16)
    w = torch.randn(hidden).to(torch.bfloat16)
    x_new, y = ops.fused_add_layer_norm(x.to(cuda_device), res.to(cuda_device), w.to(cuda_device), 1e-5)
    ox, oy = O.add_layer_norm(x, res, w, 1e-5)
    assert torch.equal(x_new.cpu(), (x + res))
    assert torch.equal(x_new.cpu().float(), ox)
    assert_bf16_close(y, oy, what="add+LN y")
    expected = torch.nn.functional.layer_norm((x + res).to(cuda_device), (hidden,), w.to(cuda_device), None, 1e-5)
    assert_bf16_close(y, expected.float().cpu(), what="add+LN y vs torch")
    y_plain = ops.fused_layer_norm(x.to(cuda_device), w.to(cuda_device), 1e-5)
    assert_bf16_close(y_plain, O.layer_norm(x, w, 1e-5), what="LN y")


def test_add_layer_norm_in_place_and_large(pe, cuda_device):
    from flash_modernbert_b200 import _lib, ops

    torch.manual_seed(1)
    t, h = 40000, 768
    x = torch.randn(t, h, device=cuda_device).to(torch.bfloat16)
    res = torch.randn(t, h, device=cuda_device).to(torch.bfloat16)
    w = torch.ones(h, device=cuda_device, dtype=torch.bfloat16)
    x_new, y = ops.fused_add_layer_norm(x, res, w, 1e-5)
    x2 = x.clone()
    y2 = torch.empty_like(x)
    lib = _lib.load()
    _lib.check(lib.pe_add_ln(x2.data_ptr(), res.data_ptr(), w.data_ptr(), 1e-5, t, h, x2.data_ptr(),
                             y2.data_ptr(), _lib.current_stream_ptr()), "pe_add_ln")
    assert torch.equal(x2, x_new) and torch.equal(y2, y)      # aliasing x_out = x changes nothing
    assert torch.equal(x_new, x + res)
    # linearity-style property at size: LN output has zero mean, unit variance per row
    yf = y.float()
    assert float(yf.mean(dim=1).abs().max()) < 2e-2 and float((yf.var(dim=1, unbiased=False) - 1).abs().max()) < 5e-2


def test_embed_layer_norm(pe, cuda_device):
    from flash_modernbert_b200 import _lib, ops

    torch.manual_seed(2)
    vocab, h = 1000, 768
    table = (torch.randn(vocab, h) * 0.02).to(torch.bfloat16)
    w = torch.randn(h).to(torch.bfloat16)
    ids = torch.randint(0, vocab, (777,))
    y = ops.embed_layer_norm(ids.to(cuda_device), table.to(cuda_device), w.to(cuda_device), 1e-5)
    assert_bf16_close(y, O.layer_norm(table[ids], w, 1e-5), what="embed+LN")
    ops.check_status(cuda_device)
    bad = ids.clone()
    bad[5] = vocab + 3
    ops.embed_layer_norm(bad.to(cuda_device), table.to(cuda_device), w.to(cuda_device), 1e-5)
    with pytest.raises(_lib.NativeLibraryError, match="301"):
        ops.check_status(cuda_device)                          # out-of-vocabulary id is reported, not read


def test_rope_table_matches_reference_rows(pe, cuda_device, golden_dir):
    from flash_modernbert_b200 import ops

    g = np.load(golden_dir / "rope_tables.npz")
    rows = torch.from_numpy(g["rows"])
    for theta in (160000.0, 10000.0):
        table = ops.rope_table(theta, 8192, cuda_device).cpu().index_select(0, rows)
        cos = torch.from_numpy(g[f"cos_{int(theta)}"]).view(torch.bfloat16)
        sin = torch.from_numpy(g[f"sin_{int(theta)}"]).view(torch.bfloat16)
        # the reference's table repeats the 32 frequencies: [S, 64] = cat(f, f)
        assert torch.equal(cos[:, :32], cos[:, 32:]) and torch.equal(sin[:, :32], sin[:, 32:])
        # device cosf/sinf/powf vs the CPU's: identical after bf16 rounding except rare last-bit flips
        for got, ref in ((table[:, :32], cos[:, :32]), (table[:, 32:], sin[:, :32])):
            ulp = (_bits(got) - _bits(ref)).abs()
            mism = ulp > 0
            assert float(mism.float().mean()) < 0.02
            assert float((got.float() - ref.float()).abs().max()) < 2 ** -7


@pytest.mark.parametrize("n_heads", [12, 4, 28])
def test_rope_qk_inplace(pe, cuda_device, n_heads):
    from flash_modernbert_b200 import ops

    torch.manual_seed(3)
    t, h = 501, n_heads * 64
    qkv = torch.randn(t, 3 * h).to(torch.bfloat16)
    pos = torch.randint(0, 8192, (t,))
    table = ops.rope_table(160000.0, 8192, cuda_device)
    out = ops.rope_qk_inplace(qkv.clone().to(cuda_device), pos.to(cuda_device), table, n_heads).cpu()
    tab = table.cpu()
    cos = torch.cat((tab[:, :32], tab[:, :32]), dim=1).index_select(0, pos)
    sin = torch.cat((tab[:, 32:], tab[:, 32:]), dim=1).index_select(0, pos)
    q = O.rope_apply(qkv[:, :h].view(t, n_heads, 64), cos, sin)
    k = O.rope_apply(qkv[:, h:2 * h].view(t, n_heads, 64), cos, sin)
    assert_bf16_close(out[:, :h], q.reshape(t, h), what="rope q")
    assert_bf16_close(out[:, h:2 * h], k.reshape(t, h), what="rope k")
    assert torch.equal(out[:, 2 * h:], qkv[:, 2 * h:])                    # v untouched
    ops.check_status(cuda_device)


@pytest.mark.parametrize("rows,inter", [(33, 1152), (1, 8), (500, 2624), (129, 3840)])
def test_geglu(pe, cuda_device, rows, inter):
    from flash_modernbert_b200 import ops

    torch.manual_seed(4)
    proj = (torch.randn(rows, 2 * inter) * 2).to(torch.bfloat16)
    out = ops.fused_geglu(proj.to(cuda_device))
    # gelu(a) for a << 0 is a * (1 + erf(..)) with 1 + erf cancelling: device erff and the host's
    # erf differ in the last bits there, which is far below one bf16 step of any O(1) output
    assert_bf16_close(out, O.geglu(proj), what="geglu", atol=5e-4)
