"""Pooling head on the packed output (`pe_pool_packed`) against the oracle's restatement of
benchmarks/showcases/inference.py:193-206 of the reference, through the C ABI."""
from __future__ import annotations

import pytest
import torch

from oracle import packed_oracle as O

pytestmark = pytest.mark.gpu


def _case(lengths, width, seed=0):
    gen = torch.Generator().manual_seed(seed)
    hidden = (torch.randn(sum(lengths), width, generator=gen) * 1.5 + 0.1).to(torch.bfloat16)
    cu = torch.zeros(len(lengths) + 1, dtype=torch.int32)
    cu[1:] = torch.tensor(lengths).cumsum(0)
    return hidden, cu


@pytest.mark.parametrize("width", [768, 1024, 1792])
@pytest.mark.parametrize("mode", ["mean", "cls"])
@pytest.mark.parametrize("normalize", [True, False])
def test_pool_against_oracle(pe, cuda_device, width, mode, normalize):
    from flash_modernbert_b200 import ops

    # lengths around the 128-row tile edge, one long sequence, one single token
    hidden, cu = _case([1, 127, 128, 129, 700, 64, 2500, 33], width)
    got = ops.pool_packed(hidden.to(cuda_device), cu.to(cuda_device), mode, normalize).cpu().float()
    ref = O.pool(hidden, cu, mode, normalize).float()
    assert got.shape == ref.shape == (8, width)
    if mode == "cls" and not normalize:
        assert torch.equal(got, ref)                      # a copy of a bf16 row
    else:
        # fp32 sums in a different order, then one bf16 rounding: at most one bf16 step apart
        assert float((got - ref).abs().max()) <= 2.0 ** -7 * float(ref.abs().max()) + 1e-6
        if normalize:
            assert float((got.norm(dim=-1) - 1).abs().max()) < 5e-3


def test_pool_is_deterministic_and_handles_empty_sequences(pe, cuda_device):
    """Graph buckets pad cu_seqlens with repeats of T: those sequences must give zero rows."""
    from flash_modernbert_b200 import ops

    hidden, cu = _case([300, 17, 129], 768, seed=1)
    padded_cu = torch.cat([cu, torch.full((3,), int(cu[-1]), dtype=torch.int32)])
    a = ops.pool_packed(hidden.to(cuda_device), padded_cu.to(cuda_device), "mean", True)
    b = ops.pool_packed(hidden.to(cuda_device), padded_cu.to(cuda_device), "mean", True)
    assert torch.equal(a, b)
    assert torch.equal(a[3:].cpu(), torch.zeros(3, 768, dtype=torch.bfloat16))
    ref = O.pool(hidden, cu, "mean", True).float()
    assert float((a[:3].cpu().float() - ref).abs().max()) <= 2.0 ** -7 * float(ref.abs().max()) + 1e-6


def test_pool_full_size(pe, cuda_device):
    """cfg3 lengths (306,851 tokens): mean of a constant hidden state is that constant, and
    normalised rows have unit length."""
    from flash_modernbert_b200 import ops
    from oracle import synthetic as S

    lengths = S.workload("cfg3").sorted_by_length().lengths
    total = sum(lengths)
    cu = torch.zeros(len(lengths) + 1, dtype=torch.int32)
    cu[1:] = torch.tensor(lengths).cumsum(0)
    const = torch.full((total, 768), 0.375, dtype=torch.bfloat16, device=cuda_device)
    out = ops.pool_packed(const, cu.to(cuda_device), "mean", False)
    assert float((out.float() - 0.375).abs().max()) < 1e-3
    gen = torch.Generator(device=cuda_device).manual_seed(0)
    rnd = torch.randn(total, 768, device=cuda_device, generator=gen).to(torch.bfloat16)
    out = ops.pool_packed(rnd, cu.to(cuda_device), "mean", True)
    assert float((out.float().norm(dim=-1) - 1).abs().max()) < 5e-3
    for n in (0, 100, len(lengths) - 1):
        s, e = int(cu[n]), int(cu[n + 1])
        ref = torch.nn.functional.normalize(rnd[s:e].float().mean(0), dim=-1)
        assert float((out[n].float() - ref).abs().max()) < 2e-3


@pytest.mark.parametrize("out_features", [128, 96, 256])
@pytest.mark.parametrize("rows", [1, 130, 5000])
def test_project_normalize_against_oracle(pe, cuda_device, out_features, rows):
    """`pe_gemm_l2norm_bf16`: Dense projection + per-token L2 normalisation in one kernel, against
    the oracle's restatement of benchmarks/helpers/packed_index.py:182-186."""
    from flash_modernbert_b200 import ops

    gen = torch.Generator().manual_seed(3)
    hidden = torch.randn(rows, 768, generator=gen).to(torch.bfloat16)
    weight = (torch.randn(out_features, 768, generator=gen) * 0.03).to(torch.bfloat16)
    got = ops.project_normalize(hidden.to(cuda_device), weight.to(cuda_device)).cpu().float()
    ref = O.project_normalize(hidden, weight).float()
    assert got.shape == ref.shape == (rows, out_features)
    # unit rows; elements within two bf16 steps (the fp32 sums run in a different order)
    assert float((got.norm(dim=-1) - 1).abs().max()) < 6e-3
    assert float((got - ref).abs().max()) <= 2.0 ** -7
    rep = O.cosine_report(got, ref)
    assert rep["min_token_cos"] > 0.9999, rep


@pytest.mark.parametrize("pool", ["mean", "cls"])
@pytest.mark.parametrize("normalize", [True, False])
def test_forward_with_the_pooling_head_fused_into_the_final_norm(pe, cuda_device, pool, normalize):
    """`packed_forward_pooled` (one library call; the pooling runs inside the final LayerNorm and
    the hidden state is not written) against `packed_forward` followed by `pool_packed`, i.e. what
    benchmarks/showcases/inference.py:193-209 of the reference does in three torch ops. The
    hidden state it can return as well is bit-equal to `packed_forward`'s; the embeddings agree
    to one bf16 step (the fp32 sums run in a different, fixed order)."""
    from flash_modernbert_b200 import forward, ops
    from oracle import synthetic as S

    vocab = 1024
    gpu = S.make_model("tiny", vocab, dtype=torch.bfloat16, device=cuda_device)
    wl = S.workload("tiny_mixed", vocab)
    params = pe.ModernBertParams.from_hf_config(gpu.config)
    batch = pe.pack_sequences(wl.sequences(), device=cuda_device)
    hidden = pe.packed_forward(gpu, params, *batch.forward_args())
    expected = ops.pool_packed(hidden, batch.cu_seqlens, pool, normalize)
    got = pe.packed_forward_pooled(gpu, params, *batch.forward_args(), pool=pool, normalize=normalize)
    both_hidden, both = pe.packed_forward_pooled(gpu, params, *batch.forward_args(), pool=pool,
                                                 normalize=normalize, return_hidden=True)
    forward.get_binding(gpu, params).check(sync=True)
    assert got.shape == expected.shape == (len(wl.lengths), 256)
    assert torch.equal(both_hidden, hidden)
    scale = float(expected.float().abs().max())
    for emb in (got, both):
        assert float((emb.float() - expected.float()).abs().max()) <= scale * 2.0 ** -7
    if pool == "cls":
        assert torch.equal(got, expected)          # no summation involved: same bits
    again = pe.packed_forward_pooled(gpu, params, *batch.forward_args(), pool=pool, normalize=normalize)
    assert torch.equal(again, got)                 # fixed summation order
    # with the residual adds left to add+LN kernels (the MLP residual then reaches the final norm
    # as a pending add) the hidden state is the same, so the embeddings are too
    from flash_modernbert_b200 import _lib
    lib = _lib.load()
    try:
        assert lib.pe_set_option(_lib.OPT_FUSED_RESIDUAL, 0) == 0
        unfused = pe.packed_forward_pooled(gpu, params, *batch.forward_args(), pool=pool, normalize=normalize)
    finally:
        lib.pe_set_option(_lib.OPT_FUSED_RESIDUAL, 1)
    assert torch.equal(unfused, got)
