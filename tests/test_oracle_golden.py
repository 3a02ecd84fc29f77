"""The CPU oracle against the committed golden fixtures (outputs of the reference's own
CPU-runnable functions and of Hugging Face eager fp32). No GPU."""
from __future__ import annotations

import numpy as np
import pytest
import torch

from oracle import packed_oracle as O
from oracle import synthetic as S

UNPAD_CASES = [
    "ref_lengths_5_2_4", "ref_roundtrip", "ref_no_padding", "single_token", "left_padded",
    "holes", "one_empty_row", "rand_32x485", "rand_7x1000", "rand_300x33",
]


@pytest.fixture(scope="module")
def unpad_golden(golden_dir):
    return np.load(golden_dir / "unpad_cases.npz")


@pytest.mark.parametrize("case", UNPAD_CASES)
def test_unpad_repad_bit_exact(unpad_golden, case):
    g = unpad_golden
    mask, x = g[f"{case}.mask"], g[f"{case}.x"]
    xp, idx, cu, max_s, pos = O.unpad(x, mask)
    assert idx.dtype == np.int64 and cu.dtype == np.int32 and pos.dtype == np.int64
    assert np.array_equal(idx, g[f"{case}.indices"])
    assert np.array_equal(cu, g[f"{case}.cu_seqlens"])
    assert max_s == int(g[f"{case}.max_seqlen"])
    assert np.array_equal(pos, g[f"{case}.position_ids"])
    assert np.array_equal(xp, g[f"{case}.x_packed"])
    b, s = mask.shape
    assert np.array_equal(O.repad(xp, idx, b, s), g[f"{case}.repad"])


def test_reference_known_answers(unpad_golden):
    # tests/test_varlen.py:62-80 of the reference: cu_seqlens [0,5,7,11], positions = column
    g = unpad_golden
    assert g["ref_lengths_5_2_4.cu_seqlens"].tolist() == [0, 5, 7, 11]
    assert g["ref_lengths_5_2_4.position_ids"].tolist() == [0, 1, 2, 3, 4, 0, 1, 0, 1, 2, 3]
    assert g["ref_no_padding.position_ids"].tolist() == [0, 1, 2, 0, 1, 2]


def test_pack_sequences_bit_exact(golden_dir):
    g = np.load(golden_dir / "pack_sequences.npz")
    seqs = np.split(g["ids"], np.cumsum(g["lengths"])[:-1])
    ids, cu, max_s, pos = O.pack_sequences(seqs)
    assert np.array_equal(ids, g["input_ids"])
    assert np.array_equal(cu, g["cu_seqlens"]) and cu.dtype == np.int32
    assert max_s == int(g["max_seqlen"])
    assert np.array_equal(pos, g["position_ids"])
    with pytest.raises(ValueError):
        O.pack_sequences([])
    with pytest.raises(ValueError):
        O.pack_sequences([[1, 2], []])


def test_collator_matches_unpad_positions():
    # benchmarks/helpers/packed_collator.py:175-196: packing right-padded rows gives the
    # same cu_seqlens / position_ids as unpadding the padded batch.
    lens = [5, 1, 9, 3]
    s = max(lens)
    mask = (np.arange(s)[None, :] < np.asarray(lens)[:, None]).astype(np.int64)
    _, _, cu_u, max_u, pos_u = O.unpad(np.zeros((4, s, 1)), mask)
    _, cu_p, max_p, pos_p = O.pack_sequences([np.arange(n) for n in lens])
    assert np.array_equal(cu_u, cu_p) and max_u == max_p and np.array_equal(pos_u, pos_p)


def test_rope_tables_bit_exact(golden_dir):
    g = np.load(golden_dir / "rope_tables.npz")
    rows = torch.from_numpy(g["rows"])
    for theta in (160000.0, 10000.0):
        cos, sin = O.rope_tables(8192, 64, theta)
        assert np.array_equal(cos.index_select(0, rows).view(torch.int16).numpy(), g[f"cos_{int(theta)}"])
        assert np.array_equal(sin.index_select(0, rows).view(torch.int16).numpy(), g[f"sin_{int(theta)}"])


def test_add_layer_norm_matches_torch_bf16():
    # tests/test_residual_layer_norm.py:15-40 of the reference, on the CPU
    torch.manual_seed(0)
    x = torch.randn(17, 768).to(torch.bfloat16)
    res = torch.randn(17, 768).to(torch.bfloat16)
    w = torch.randn(768).to(torch.bfloat16)
    x_new, y = O.add_layer_norm(x, res, w, 1e-5)
    exp_x = x + res
    exp_y = torch.nn.functional.layer_norm(exp_x.float(), (768,), w.float(), None, 1e-5)
    assert torch.equal(x_new.to(torch.bfloat16), exp_x)
    diff = (y - exp_y.to(torch.bfloat16).float()).abs()
    # identical up to the last bf16 bit of a few elements (E[x^2]-mean^2 vs centred variance)
    assert float(diff.max()) <= 2 ** -6 and float((diff > 0).float().mean()) < 0.02


@pytest.fixture(scope="module")
def tiny(golden_dir):
    g = np.load(golden_dir / "hf_tiny.npz")
    model = S.make_model("tiny", int(g["vocab"]))
    return g, model


def test_workload_definitions_are_stable(tiny):
    g, _ = tiny
    wl = S.workload("tiny_mixed", int(g["vocab"]))
    assert wl.lengths == g["lengths"].tolist()
    assert np.array_equal(wl.ids.numpy(), g["ids"])
    totals = {n: S.workload(n).total_tokens for n in ("cfg1", "cfg2", "cfg3", "cfg4")}
    assert totals == {"cfg1": 8552, "cfg2": 28671, "cfg3": 306851, "cfg4": 352243}
    assert S.workload("cfg3").max_seqlen == 8192 and S.workload("cfg1").max_seqlen == 485


def test_oracle_fp32_matches_hf_eager(tiny):
    g, model = tiny
    ids, cu, max_s, pos = O.pack_sequences(np.split(g["ids"], np.cumsum(g["lengths"])[:-1]))
    out = O.packed_forward(model, ids, cu, max_s, pos, faithful=False)
    ref = torch.from_numpy(g["last_hidden_state"].astype(np.float32))
    assert float((out - ref).abs().max()) < 5e-3  # fixture is stored in fp16
    assert O.cosine_report(out, ref)["min_token_cos"] > 0.99999


def test_oracle_bf16_faithful_tracks_hf_eager(tiny):
    g, model = tiny
    ids, cu, max_s, pos = O.pack_sequences(np.split(g["ids"], np.cumsum(g["lengths"])[:-1]))
    out = O.packed_forward(model, ids, cu, max_s, pos, faithful=True)
    ref = torch.from_numpy(g["last_hidden_state"].astype(np.float32))
    rep = O.cosine_report(out, ref)
    assert rep["min_token_cos"] >= 0.999, rep
    assert rep["max_abs"] < 0.25, rep


def test_attention_window_and_isolation():
    # tests/test_packed_short_attention.py:110-124: other sequences' K/V never leak
    torch.manual_seed(0)
    q, k, v = (torch.randn(40, 2, 64) for _ in range(3))
    cu = [0, 13, 40]
    base = O.attention(q, k, v, cu, 64)
    k2, v2 = k.clone(), v.clone()
    k2[13:] *= 100
    v2[13:] *= 100
    assert torch.equal(O.attention(q, k2, v2, cu, 64)[:13], base[:13])
    # a window of >= len-1 equals full attention
    assert torch.equal(O.attention(q, k, v, cu, 64), O.attention(q, k, v, cu, None))
    far = O.attention(q, k, v, cu, 3)
    assert not torch.equal(far, base)


def test_pool_oracle_known_answers():
    """`oracle.pool` restates benchmarks/showcases/inference.py:193-206: segment mean in fp32,
    F.normalize, cast last."""
    import torch

    from oracle import packed_oracle as O

    hidden = torch.tensor([[3.0, 4.0], [1.0, 0.0], [3.0, 0.0], [0.0, 2.0]], dtype=torch.bfloat16)
    cu = [0, 1, 3, 3, 4]
    mean = O.pool(hidden, cu, "mean", False).float()
    assert mean.tolist() == [[3.0, 4.0], [2.0, 0.0], [0.0, 0.0], [0.0, 2.0]]
    unit = O.pool(hidden, cu, "mean", True).float()
    assert torch.allclose(unit, torch.tensor([[0.6, 0.8], [1.0, 0.0], [0.0, 0.0], [0.0, 1.0]]), atol=4e-3)
    cls = O.pool(hidden, cu, "cls", False).float()
    assert cls.tolist() == [[3.0, 4.0], [1.0, 0.0], [0.0, 0.0], [0.0, 2.0]]
    # against the reference's own formulation (index_add_ over repeat_interleave segments)
    gen = torch.Generator().manual_seed(0)
    h = torch.randn(37, 16, generator=gen).to(torch.bfloat16)
    lens = torch.tensor([5, 20, 12])
    seg = torch.repeat_interleave(torch.arange(3), lens)
    sums = torch.zeros(3, 16).index_add_(0, seg, h.float())
    ref = torch.nn.functional.normalize(sums / lens.unsqueeze(1).float(), p=2, dim=-1).to(torch.bfloat16)
    got = O.pool(h, [0, 5, 25, 37], "mean", True)
    assert float((got.float() - ref.float()).abs().max()) <= 2.0 ** -8


def test_project_normalize_oracle_known_answer():
    import torch

    from oracle import packed_oracle as O

    hidden = torch.tensor([[1.0, 2.0], [0.0, 0.0]], dtype=torch.bfloat16)
    weight = torch.tensor([[3.0, 0.0], [0.0, 2.0]], dtype=torch.bfloat16)
    out = O.project_normalize(hidden, weight).float()
    assert torch.allclose(out[0], torch.tensor([0.6, 0.8]), atol=4e-3)
    assert out[1].tolist() == [0.0, 0.0]          # zero row: divided by eps, stays zero
