"""End-to-end parity of the packed forward and of the pack()/unpack() API on a B200:
against the CPU oracle, the Hugging Face eager golden, HF eager fp32 run on the host, and
(when its install is present) the reference's own GPU packed_forward."""
from __future__ import annotations

import os
import sys

import numpy as np
import pytest
import torch

from conftest import ROOT
from oracle import packed_oracle as O
from oracle import synthetic as S

pytestmark = pytest.mark.gpu

COS_GATE = 0.999  # per-token cosine floor stated by the task's north star


def _packed_inputs(wl, device):
    cu = torch.zeros(len(wl.lengths) + 1, dtype=torch.int32)
    cu[1:] = torch.tensor(wl.lengths).cumsum(0)
    pos = torch.cat([torch.arange(n) for n in wl.lengths])
    return wl.ids.to(device), cu.to(device), wl.max_seqlen, pos.to(device)


@pytest.fixture(scope="module")
def tiny_models(cuda_device, golden_dir):
    g = np.load(golden_dir / "hf_tiny.npz")
    vocab = int(g["vocab"])
    cpu = S.make_model("tiny", vocab)
    gpu = S.make_model("tiny", vocab, dtype=torch.bfloat16, device=cuda_device)
    return g, cpu, gpu, vocab


def test_tiny_model_against_golden_and_oracle(pe, cuda_device, tiny_models):
    from flash_modernbert_b200 import forward

    g, cpu, gpu, vocab = tiny_models
    wl = S.workload("tiny_mixed", vocab)
    params = pe.ModernBertParams.from_hf_config(gpu.config)
    ids, cu, max_s, pos = _packed_inputs(wl, cuda_device)
    out = pe.packed_forward(gpu, params, ids, cu, max_s, pos)
    forward.get_binding(gpu, params).check(sync=True)
    assert out.shape == (wl.total_tokens, 256) and out.dtype == torch.bfloat16
    golden = torch.from_numpy(g["last_hidden_state"].astype(np.float32))
    rep = O.cosine_report(out.cpu(), golden)
    assert rep["min_token_cos"] >= COS_GATE and rep["max_abs"] < 0.25, rep
    oracle = O.packed_forward(cpu, wl.ids, cu.cpu(), max_s, pos.cpu(), faithful=True)
    rep_o = O.cosine_report(out.cpu(), oracle)
    assert rep_o["min_token_cos"] >= 0.9995 and rep_o["max_abs"] < 0.13, rep_o
    # position_ids=None means arange per sequence
    assert torch.equal(pe.packed_forward(gpu, params, ids, cu, max_s, None), out)
    # deterministic
    assert torch.equal(pe.packed_forward(gpu, params, ids, cu, max_s, pos), out)


def test_fused_and_unfused_epilogues_agree(pe, cuda_device, tiny_models):
    from flash_modernbert_b200 import _lib

    _, _, gpu, vocab = tiny_models
    wl = S.workload("tiny_short", vocab)
    params = pe.ModernBertParams.from_hf_config(gpu.config)
    args = _packed_inputs(wl, cuda_device)
    lib = _lib.load()
    try:
        fused = pe.packed_forward(gpu, params, *args)
        _lib.check(lib.pe_set_option(_lib.OPT_FUSED_GEGLU, 0), "pe_set_option")
        _lib.check(lib.pe_set_option(_lib.OPT_FUSED_ROPE, 0), "pe_set_option")
        _lib.check(lib.pe_set_option(_lib.OPT_FUSED_RESIDUAL, 0), "pe_set_option")
        unfused = pe.packed_forward(gpu, params, *args)
    finally:
        lib.pe_set_option(_lib.OPT_FUSED_GEGLU, 1)
        lib.pe_set_option(_lib.OPT_FUSED_ROPE, 1)
        lib.pe_set_option(_lib.OPT_FUSED_RESIDUAL, 1)
    assert torch.equal(fused, unfused)


def test_pack_unpack_api(pe, cuda_device, tiny_models):
    from transformers.modeling_outputs import BaseModelOutput

    _, cpu, gpu, vocab = tiny_models
    wl = S.workload("tiny_short", vocab)
    b, s = len(wl.lengths), wl.max_seqlen
    ids = torch.zeros(b, s, dtype=torch.int64)
    mask = torch.zeros(b, s, dtype=torch.int64)
    for i, seq in enumerate(wl.sequences()):
        ids[i, : seq.numel()] = seq
        mask[i, : seq.numel()] = 1
    stock = O.hf_eager_padded(cpu, ids, mask)
    original = gpu.forward
    report = pe.validate(gpu, seq_lens=(128, 512))
    assert report.capability == (10, 0) and min(report.cosine.values()) >= 0.997
    assert pe.pack(gpu, validate=False) is gpu
    assert pe.pack(gpu) is gpu                                         # idempotent
    try:
        with torch.no_grad():
            out = gpu(input_ids=ids.to(cuda_device), attention_mask=mask.to(cuda_device))
        assert isinstance(out, BaseModelOutput)
        hidden = out.last_hidden_state
        assert hidden.shape == (b, s, 256)
        real = mask.bool()
        assert not bool(hidden.cpu()[~real].ne(0).any())               # pad rows exactly zero
        rep = O.cosine_report(hidden.cpu()[real], stock[real])
        assert rep["min_token_cos"] >= COS_GATE, rep
        tup = gpu(input_ids=ids.to(cuda_device), attention_mask=mask.to(cuda_device), return_dict=False)
        assert isinstance(tup, tuple) and torch.equal(tup[0], hidden)
        nomask = gpu(input_ids=ids[:3, :8].to(cuda_device)).last_hidden_state
        assert nomask.shape == (3, 8, 256)
        for kw in ({"inputs_embeds": torch.zeros(1)}, {"output_attentions": True},
                   {"output_hidden_states": True}, {"token_type_ids": torch.ones(1, 1)}):
            with pytest.raises(NotImplementedError):
                gpu(input_ids=ids.to(cuda_device), **kw)
        with pytest.raises(NotImplementedError):
            gpu(attention_mask=mask.to(cuda_device))
        assert pe.get_state(gpu).params.hidden_size == 256
    finally:
        pe.unpack(gpu)
    assert gpu.forward == original and not hasattr(gpu, "_packed_encoders")


def test_bucketed_cuda_graphs(pe, cuda_device, tiny_models):
    from flash_modernbert_b200 import forward

    _, _, gpu, vocab = tiny_models
    params = pe.ModernBertParams.from_hf_config(gpu.config)
    pe.pack(gpu, validate=False, cuda_graph=pe.GraphConfig(pad_to=256, max_batch=64, max_seq=64))
    try:
        runner = pe.get_state(gpu).packed_graph_runner
        gen = torch.Generator().manual_seed(7)
        for trial in range(6):
            n = int(torch.randint(20, 64, (1,), generator=gen))
            lengths = torch.randint(33, 49, (n,), generator=gen).tolist()
            seqs = [torch.randint(5, vocab, (l,), generator=gen) for l in lengths]
            batch = pe.pack_sequences(seqs, device=cuda_device)
            with torch.no_grad():       # graphs engage only with autograd off, as in the reference
                graphed = pe.packed_forward(gpu, params, *batch.forward_args())
                with pe.no_cuda_graph(gpu):
                    eager = pe.packed_forward(gpu, params, *batch.forward_args())
            forward.get_binding(gpu, params).check(sync=True)
            assert graphed.shape == eager.shape
            assert torch.equal(graphed, eager), trial         # same kernels, same data => same bits
        assert runner.replays == 6
        # ragged traffic shares graphs: keys hold capacities only
        assert runner.captures <= 5 and all(k[1] == 64 and k[2] == 64 for k in runner._cache)
        long_batch = pe.pack_sequences([torch.randint(5, vocab, (100,), generator=gen)], device=cuda_device)
        before = runner.eager_calls
        with torch.no_grad():
            pe.packed_forward(gpu, params, *long_batch.forward_args())    # over max_seq: eager
        assert runner.eager_calls == before + 1
        replays = runner.replays
        pe.packed_forward(gpu, params, *batch.forward_args())         # autograd on: eager
        assert runner.replays == replays
        os.environ["PACKED_ENCODERS_GRAPH"] = "0"
        try:
            with torch.no_grad():
                pe.packed_forward(gpu, params, *batch.forward_args())
            assert runner.replays == replays                          # kill switch
        finally:
            del os.environ["PACKED_ENCODERS_GRAPH"]
        pe.set_cuda_graph(gpu, False)
        assert not pe.get_state(gpu).graph_enabled
    finally:
        pe.unpack(gpu)


@pytest.fixture(scope="module")
def base_models(cuda_device):
    cpu = S.make_model("base")
    gpu = S.make_model("base", dtype=torch.bfloat16, device=cuda_device)
    return cpu, gpu


def test_base_cfg1_against_hf_eager(pe, cuda_device, base_models):
    """cfg1 (32 sequences, 8,552 tokens) on ModernBERT-base: whole batch on the GPU, HF eager
    fp32 on the host for a seeded subset of sequences (bounded CPU time)."""
    from flash_modernbert_b200 import forward

    cpu, gpu = base_models
    wl = S.workload("cfg1")
    params = pe.ModernBertParams.from_hf_config(gpu.config)
    ids, cu, max_s, pos = _packed_inputs(wl, cuda_device)
    out = pe.packed_forward(gpu, params, ids, cu, max_s, pos)
    forward.get_binding(gpu, params).check(sync=True)
    assert bool(torch.isfinite(out.float()).all())
    seqs = wl.sequences()
    picks = [0, 7, 19, 31]
    worst = 1.0
    max_abs = 0.0
    for n in picks:
        ref = O.hf_eager_packed(cpu, [seqs[n]])
        s, e = int(cu[n]), int(cu[n + 1])
        rep = O.cosine_report(out[s:e].cpu(), ref)
        worst = min(worst, rep["min_token_cos"])
        max_abs = max(max_abs, rep["max_abs"])
    print(f"cfg1 vs HF eager fp32: min per-token cosine {worst:.6f}, max-abs {max_abs:.4f}")
    assert worst >= COS_GATE, (worst, max_abs)


def test_base_padded_api_matches_packed(pe, cuda_device, base_models):
    _, gpu = base_models
    wl = S.workload("cfg1")
    params = pe.ModernBertParams.from_hf_config(gpu.config)
    b, s = len(wl.lengths), wl.max_seqlen
    ids = torch.zeros(b, s, dtype=torch.int64)
    mask = torch.zeros(b, s, dtype=torch.int64)
    for i, seq in enumerate(wl.sequences()):
        ids[i, : seq.numel()] = seq
        mask[i, : seq.numel()] = 1
    packed = pe.packed_forward(gpu, params, *_packed_inputs(wl, cuda_device))
    padded = pe.fused_forward(gpu, params, ids.to(cuda_device), mask.to(cuda_device))
    assert padded.shape == (b, s, 768)
    assert torch.equal(padded[mask.bool().to(cuda_device)], packed)
    assert not bool(padded[~mask.bool().to(cuda_device)].ne(0).any())


def test_cfg3_full_size_properties(pe, cuda_device, base_models):
    """The headline workload (512 documents, 306,851 tokens): permutation equivariance over
    sequences and agreement of a sequence encoded alone with the same sequence in the batch."""
    from flash_modernbert_b200 import forward

    _, gpu = base_models
    wl = S.workload("cfg3").sorted_by_length()
    params = pe.ModernBertParams.from_hf_config(gpu.config)
    ids, cu, max_s, pos = _packed_inputs(wl, cuda_device)
    out = pe.packed_forward(gpu, params, ids, cu, max_s, pos)
    forward.get_binding(gpu, params).check(sync=True)
    assert out.shape == (306851, 768) and bool(torch.isfinite(out.float()).all())
    seqs = wl.sequences()
    for n in (0, 100, 511):
        alone = pe.pack_sequences([seqs[n]], device=cuda_device)
        solo = pe.packed_forward(gpu, params, *alone.forward_args())
        s, e = int(cu[n]), int(cu[n + 1])
        rep = O.cosine_report(solo.cpu(), out[s:e].cpu())
        assert rep["min_token_cos"] > 0.9999, (n, rep)   # only batch-size-dependent tiling differs


def test_against_reference_gpu_packed_forward(pe, cuda_device, base_models):
    """Same seeded inputs through the reference's own GPU packed_forward, when its install
    (baseline/_ref) and its JIT toolchains work on this machine."""
    ref_dir = ROOT / "baseline" / "_ref"
    if not (ref_dir / "packed_encoders").exists():
        pytest.skip("reference install not present")
    sys.path.insert(0, str(ref_dir))
    try:
        try:
            from packed_encoders import forward as ref_forward
            from packed_encoders.config import ModernBertParams as RefParams
        except Exception as exc:  # noqa: BLE001
            pytest.skip(f"reference does not import here: {exc}")
        _, gpu = base_models
        wl = S.workload("cfg1")
        ids, cu, max_s, pos = _packed_inputs(wl, cuda_device)
        cfg = gpu.config
        if not hasattr(cfg, "global_attn_every_n_layers"):
            cfg.global_attn_every_n_layers = 3
        try:
            with torch.no_grad():
                ref_out = ref_forward.packed_forward(gpu, RefParams.from_hf_config(cfg), ids, cu, max_s, pos)
            torch.cuda.synchronize()
        except Exception as exc:  # noqa: BLE001
            pytest.skip(f"reference packed_forward does not run here: {type(exc).__name__}: {exc}")
        params = pe.ModernBertParams.from_hf_config(cfg)
        out = pe.packed_forward(gpu, params, ids, cu, max_s, pos)
        rep = O.cosine_report(out.cpu(), ref_out.cpu())
        print(f"vs reference GPU packed_forward: {rep}")
        assert rep["min_token_cos"] >= COS_GATE, rep
    finally:
        sys.path.remove(str(ref_dir))


def _token_cosines(a: torch.Tensor, b: torch.Tensor):
    """Per-token cosine and max-abs of two [T, H] tensors, computed on their device in fp32."""
    worst, max_abs = 1.0, 0.0
    for start in range(0, a.shape[0], 65536):
        x = a[start:start + 65536].float()
        y = b[start:start + 65536].float()
        cos = (x * y).sum(-1) / (x.norm(dim=-1) * y.norm(dim=-1)).clamp_min(1e-12)
        worst = min(worst, float(cos.min()))
        max_abs = max(max_abs, float((x - y).abs().max()))
    return worst, max_abs


def test_cfg3_headline_size_against_reference_gpu_and_hf_eager(pe, cuda_device, base_models):
    """The headline workload at full size (512 documents up to 8,192 tokens, 306,851 tokens): all
    tokens against the reference's own GPU packed_forward (the relation of the reference's
    tests/test_varlen.py:328-381, on the seeded random-init weights), and one whole long document
    (4,000 - 8,192 tokens: dozens of key tiles per query tile) taken out of that batch against
    Hugging Face eager fp32 on the host."""
    from flash_modernbert_b200 import forward

    cpu, gpu = base_models
    wl = S.workload("cfg3").sorted_by_length()
    ids, cu, max_s, pos = _packed_inputs(wl, cuda_device)
    cfg = gpu.config
    if not hasattr(cfg, "global_attn_every_n_layers"):
        cfg.global_attn_every_n_layers = 3
    params = pe.ModernBertParams.from_hf_config(cfg)
    out = pe.packed_forward(gpu, params, ids, cu, max_s, pos)
    forward.get_binding(gpu, params).check(sync=True)

    # one whole document between 4,000 and 8,192 tokens, against HF eager fp32
    n = max(i for i, length in enumerate(wl.lengths) if length >= 4000)   # the shortest such (sorted descending)
    s, e = int(cu[n]), int(cu[n + 1])
    ref_doc = O.hf_eager_packed(cpu, [wl.sequences()[n]])
    rep = O.cosine_report(out[s:e].cpu(), ref_doc)
    print(f"cfg3 document of {e - s} tokens vs HF eager fp32: {rep}")
    assert rep["min_token_cos"] >= COS_GATE, rep

    ref_dir = ROOT / "baseline" / "_ref"
    if not (ref_dir / "packed_encoders").exists():
        pytest.skip("reference install not present (HF eager part passed)")
    sys.path.insert(0, str(ref_dir))
    try:
        try:
            from packed_encoders import forward as ref_forward
            from packed_encoders.config import ModernBertParams as RefParams
            with torch.no_grad():
                ref_out = ref_forward.packed_forward(gpu, RefParams.from_hf_config(cfg), ids, cu, max_s, pos)
            torch.cuda.synchronize()
        except Exception as exc:  # noqa: BLE001
            pytest.skip(f"reference packed_forward does not run here: {type(exc).__name__}: {exc}")
        assert ref_out.shape == out.shape == (306851, 768)
        worst, max_abs = _token_cosines(out, ref_out)
        print(f"cfg3 (306,851 tokens) vs reference GPU packed_forward: min per-token cosine {worst:.6f}, "
              f"max-abs {max_abs:.4f}")
        assert worst >= COS_GATE, (worst, max_abs)
    finally:
        sys.path.remove(str(ref_dir))


def _subset(wl, picks):
    seqs = wl.sequences()
    return [seqs[i] for i in picks]


@pytest.mark.parametrize("arch,config,picks", [
    ("large", "cfg4", [5, 40]),          # two long documents (2,048..8,192 tokens) on ModernBERT-large
    ("large", "cfg4", "shortest"),       # one whole document of cfg4 (>= 2,048 tokens), not truncated
    ("1b", "cfg5", [3, 100, 9000]),      # two queries and one document on the 1B-class model
])
def test_other_architectures_against_hf_eager(pe, cuda_device, arch, config, picks):
    """cfg4 / cfg5 architectures (hidden 1024 / 1792, 28 layers, intermediate 2624 / 3840): a
    seeded subset of the config's sequences, packed on the GPU against HF eager fp32 on the host."""
    from flash_modernbert_b200 import forward

    wl = S.workload(config)
    if picks == "shortest":
        seqs = _subset(wl, [min(range(len(wl.lengths)), key=lambda i: wl.lengths[i])])
        assert seqs[0].numel() >= 2048
    else:
        seqs = [s[:2000] for s in _subset(wl, picks)]       # bound the CPU side of the check
    cpu = S.make_model(arch)
    gpu = S.make_model(arch, dtype=torch.bfloat16, device=cuda_device)
    params = pe.ModernBertParams.from_hf_config(gpu.config)
    batch = pe.pack_sequences(seqs, device=cuda_device)
    out = pe.packed_forward(gpu, params, *batch.forward_args())
    forward.get_binding(gpu, params).check(sync=True)
    ref = O.hf_eager_packed(cpu, seqs)
    rep = O.cosine_report(out.cpu(), ref)
    print(f"{config} subset on {arch}: {rep}")
    assert rep["min_token_cos"] >= COS_GATE, rep
    del gpu, cpu
    torch.cuda.empty_cache()


def test_cfg2_queries_through_token_bucket_graphs(pe, cuda_device, base_models):
    """cfg2 (1,024 queries of 8..48 tokens, 28,671 tokens) in batches of 256 sequences: graph
    replays equal the eager forward bit for bit and a handful of graphs serves all batches."""
    from flash_modernbert_b200 import forward

    cpu, gpu = base_models
    wl = S.workload("cfg2")
    seqs = wl.sequences()
    params = pe.ModernBertParams.from_hf_config(gpu.config)
    pe.pack(gpu, validate=False, cuda_graph=pe.GraphConfig(pad_to=4096, max_batch=256, max_seq=64))
    try:
        runner = pe.get_state(gpu).packed_graph_runner
        with torch.no_grad():
            for start in range(0, len(seqs), 256):
                batch = pe.pack_sequences(seqs[start:start + 256], device=cuda_device)
                graphed = pe.packed_forward(gpu, params, *batch.forward_args())
                with pe.no_cuda_graph(gpu):
                    eager = pe.packed_forward(gpu, params, *batch.forward_args())
                assert torch.equal(graphed, eager)
        forward.get_binding(gpu, params).check(sync=True)
        assert runner.replays == 4 and runner.captures == 1    # four ragged batches, one graph
        ref = O.hf_eager_packed(cpu, seqs[768:776])
        got = graphed[: sum(s.numel() for s in seqs[768:776])]
        assert O.cosine_report(got.cpu(), ref)["min_token_cos"] >= COS_GATE
    finally:
        pe.unpack(gpu)


def test_encode_in_token_budget_batches(pe, cuda_device, tiny_models):
    """`encode_in_batches` (the loop of benchmarks/showcases/inference.py:186-209): the same
    embeddings whether the corpus goes through in one batch or in token-budget micro-batches,
    returned in the callers' order."""
    _, _, gpu, vocab = tiny_models
    wl = S.workload("tiny_mixed", vocab)
    params = pe.ModernBertParams.from_hf_config(gpu.config)
    bounds = np.concatenate([[0], np.cumsum(wl.lengths)])
    seqs = [wl.ids[bounds[i]:bounds[i + 1]] for i in range(len(wl.lengths))]
    whole = pe.encode_in_batches(gpu, params, seqs, 10 ** 9, sort_by_length=False)
    budget = max(wl.lengths) + 8                      # forces several micro-batches
    assert len(pe.token_budget_batches(wl.lengths, budget)) > 2
    split = pe.encode_in_batches(gpu, params, seqs, budget)
    assert whole.shape == split.shape == (len(seqs), 256)
    # per-sequence results do not depend on what else is in the batch
    assert float((whole.float() - split.float()).abs().max()) <= 2.0 ** -7
    assert float((split.float().norm(dim=-1) - 1).abs().max()) < 6e-3
    # pool=None: per-sequence hidden states, identical rows to one packed forward
    ids, cu, max_s, pos = _packed_inputs(wl, cuda_device)
    ref = pe.packed_forward(gpu, params, ids, cu, max_s, pos)
    parts = pe.encode_in_batches(gpu, params, seqs, budget, pool=None)
    for i, part in enumerate(parts):
        assert part.shape[0] == wl.lengths[i]
        assert float((part.float() - ref[bounds[i]:bounds[i + 1]].float()).abs().max()) < 0.05


def test_graphs_precaptured_at_pack_time(pe, cuda_device, tiny_models):
    """`GraphConfig(seq_buckets=..., max_batch=...)` captures its graphs inside `pack()`, as
    packed_encoders/graph.py:410-427 does: the first real calls are replays, not captures."""
    _, _, gpu, vocab = tiny_models
    params = pe.ModernBertParams.from_hf_config(gpu.config)
    cfg = pe.GraphConfig(pad_to=256, max_batch=16, max_seq=48, seq_buckets=(16, 48))
    pe.pack(gpu, validate=False, cuda_graph=cfg)
    try:
        runner = pe.get_state(gpu).packed_graph_runner
        assert runner.captures == 2 and sorted(runner._cache) == [(256, 16, 16), (768, 16, 64)]
        gen = torch.Generator().manual_seed(9)
        for lengths in ([16] * 16, [40] * 16, [48] * 9 + [33, 47, 35]):   # 256, 640 and 547 tokens
            seqs = [torch.randint(5, vocab, (l,), generator=gen) for l in lengths]
            batch = pe.pack_sequences(seqs, device=cuda_device)
            with torch.no_grad():
                graphed = pe.packed_forward(gpu, params, *batch.forward_args())
                with pe.no_cuda_graph(gpu):
                    eager = pe.packed_forward(gpu, params, *batch.forward_args())
            assert torch.equal(graphed, eager)
        assert runner.captures == 2 and runner.replays == 3      # nothing captured lazily
    finally:
        pe.unpack(gpu)


def _same_up_to_p_rounding(a: torch.Tensor, b: torch.Tensor) -> bool:
    """Sequences longer than 64 tokens go through the tensor-memory attention kernels, whose
    sliding-window form may take its softmax reference exponent from a whole fetched key chunk,
    rows beyond the end of the sequence included (any reference within 2^60 of the row maximum
    serves). A graph bucket holds padding rows there where the eager batch holds nothing, so P
    can round differently by one bf16 step at the ends of sequences: equal to within that, not
    bit for bit."""
    worst, max_abs = _token_cosines(a.reshape(-1, a.shape[-1]), b.reshape(-1, b.shape[-1]))
    live = (a.float().abs().amax(dim=-1) > 0).reshape(-1)
    x, y = a.reshape(-1, a.shape[-1])[live].float(), b.reshape(-1, b.shape[-1])[live].float()
    cos = (x * y).sum(-1) / (x.norm(dim=-1) * y.norm(dim=-1)).clamp_min(1e-12)
    return float(cos.min()) > 0.9999 and max_abs < 0.05 and torch.equal(a == 0, b == 0)


def _padded(seqs, b_cols=None):
    b, s = len(seqs), b_cols or max(x.numel() for x in seqs)
    ids = torch.zeros(b, s, dtype=torch.int64)
    mask = torch.zeros(b, s, dtype=torch.int64)
    for i, seq in enumerate(seqs):
        ids[i, : seq.numel()] = seq
        mask[i, : seq.numel()] = 1
    return ids, mask


def test_padded_api_through_cuda_graphs(pe, cuda_device, tiny_models):
    """`model(input_ids, attention_mask)` with `cuda_graph=GraphConfig(...)`: what the reference's
    tests/test_graph_bucketing.py:102-234 pins for its rectangular runner - one graph for every
    batch size up to max_batch, the max_seq cut-off, the LRU bound, pre-capture of seq_buckets
    at pack() time, and replay equal to the eager forward."""
    _, _, gpu, vocab = tiny_models
    cfg = pe.GraphConfig(pad_to=64, max_batch=8, max_seq=200, max_graphs=2, seq_buckets=(64,))
    pe.pack(gpu, validate=False, cuda_graph=cfg)
    try:
        state = pe.get_state(gpu)
        runner = state.graph_runner
        assert runner.captures == 1 and list(runner._cache) == [(8, 64)]       # captured inside pack()
        gen = torch.Generator().manual_seed(5)

        def batch(n, lo, hi):
            lengths = torch.randint(lo, hi, (n,), generator=gen).tolist()
            return _padded([torch.randint(5, vocab, (l,), generator=gen) for l in lengths])

        def both(ids, mask):
            with torch.no_grad():
                graphed = gpu(input_ids=ids.to(cuda_device), attention_mask=mask.to(cuda_device)).last_hidden_state
                with pe.no_cuda_graph(gpu):
                    eager = gpu(input_ids=ids.to(cuda_device), attention_mask=mask.to(cuda_device)).last_hidden_state
            return graphed, eager

        for n in (1, 3, 8):                                   # one graph for all b <= max_batch
            ids, mask = batch(n, 20, 60)
            graphed, eager = both(ids, mask)
            assert graphed.shape == eager.shape == (n, ids.shape[1], 256)
            assert torch.equal(graphed, eager)                # same kernels on the same rows
            assert not bool(graphed[~mask.bool().to(cuda_device)].ne(0).any())   # pad rows exactly zero
        assert runner.captures == 1 and runner.replays == 3
        ids, mask = batch(4, 70, 128)                         # the 128 bucket: tensor-memory attention
        graphed, eager = both(ids, mask)
        assert _same_up_to_p_rounding(graphed, eager) and runner.captures == 2
        ids, mask = batch(2, 130, 190)                        # a third bucket evicts the oldest
        graphed, eager = both(ids, mask)
        assert _same_up_to_p_rounding(graphed, eager)
        assert runner.captures == 3 and list(runner._cache) == [(8, 128), (8, 192)]
        before = runner.eager_calls
        ids, mask = batch(2, 201, 260)                        # over max_seq: eager
        both(ids, mask)
        assert runner.eager_calls == before + 1
        ids, mask = batch(9, 20, 60)                          # over max_batch: eager
        both(ids, mask)
        assert runner.eager_calls == before + 2
        with torch.no_grad():                                  # no mask: every row is a full sequence
            nomask = gpu(input_ids=ids[:3, :16].to(cuda_device)).last_hidden_state
            with pe.no_cuda_graph(gpu):
                nomask_eager = gpu(input_ids=ids[:3, :16].to(cuda_device)).last_hidden_state
        assert torch.equal(nomask, nomask_eager)
        replays = runner.replays
        gpu(input_ids=ids[:3, :16].to(cuda_device))           # autograd on: eager
        assert runner.replays == replays
    finally:
        pe.unpack(gpu)


def test_graph_replay_reports_a_bad_token_id(pe, cuda_device, tiny_models):
    """A token id outside the vocabulary fed through a graph replay is reported like in the eager
    path: on the same call with PE_B200_CHECK_STATUS=1, else on the next one."""
    from flash_modernbert_b200 import _lib

    _, _, gpu, vocab = tiny_models
    params = pe.ModernBertParams.from_hf_config(gpu.config)
    pe.pack(gpu, validate=False, cuda_graph=pe.GraphConfig(pad_to=64, max_batch=4, max_seq=64))
    try:
        good = pe.pack_sequences([torch.arange(5, 25), torch.arange(30, 60)], device=cuda_device)
        bad_ids = good.input_ids.clone()
        bad_ids[3] = vocab + 7
        with torch.no_grad():
            pe.packed_forward(gpu, params, *good.forward_args())                  # capture + replay
            pe.packed_forward(gpu, params, bad_ids, good.cu_seqlens, good.max_seqlen, good.position_ids)
            torch.cuda.synchronize()
            with pytest.raises(_lib.NativeLibraryError, match="301"):
                pe.packed_forward(gpu, params, *good.forward_args())              # raised on the next call
            os.environ["PE_B200_CHECK_STATUS"] = "1"
            try:
                with pytest.raises(_lib.NativeLibraryError, match="301"):
                    pe.packed_forward(gpu, params, bad_ids, good.cu_seqlens, good.max_seqlen, good.position_ids)
            finally:
                del os.environ["PE_B200_CHECK_STATUS"]
            assert pe.get_state(gpu).packed_graph_runner.replays >= 3
            pe.packed_forward(gpu, params, *good.forward_args())                  # the word was cleared
    finally:
        pe.unpack(gpu)


def test_non_finite_bucket_padding_never_reaches_real_rows(pe, cuda_device, tiny_models):
    """Graph buckets pad the token dimension; the padding rows of the scratch arena hold whatever
    the previous user of that memory left. With sequences longer than 64 tokens (the tensor-memory
    attention kernels, which fetch whole key/value tiles) a non-finite pattern there must not
    turn the last real sequence into NaN: real rows are bit-equal to the eager run."""
    _, _, gpu, vocab = tiny_models
    params = pe.ModernBertParams.from_hf_config(gpu.config)
    pe.pack(gpu, validate=False, cuda_graph=pe.GraphConfig(pad_to=1024, max_batch=8, max_seq=512))
    try:
        runner = pe.get_state(gpu).packed_graph_runner
        gen = torch.Generator().manual_seed(13)
        seqs = [torch.randint(5, vocab, (l,), generator=gen) for l in (200, 77, 130, 45, 301)]
        batch = pe.pack_sequences(seqs, device=cuda_device)      # 753 tokens in a 1,024 bucket
        with torch.no_grad():
            first = pe.packed_forward(gpu, params, *batch.forward_args())
            runner._workspace.fill_(0xFF)                        # bf16 0xFFFF is a NaN
            poisoned = pe.packed_forward(gpu, params, *batch.forward_args())
            with pe.no_cuda_graph(gpu):
                eager = pe.packed_forward(gpu, params, *batch.forward_args())
        assert runner.replays == 2
        assert bool(torch.isfinite(poisoned.float()).all())
        assert torch.equal(poisoned, first)                      # what the padding held before does not matter
        assert _same_up_to_p_rounding(poisoned, eager)
    finally:
        pe.unpack(gpu)


def test_mixed_serving_window_matches_split_batches(pe, cuda_device, tiny_models):
    """A window holding queries and documents together (benchmarks/showcases/mixed_serving.py:151-193:
    `unified_packed`) gives every request the embedding it gets when queries and documents are
    encoded as two separate batches, as the reference's split baseline does."""
    _, _, gpu, vocab = tiny_models
    params = pe.ModernBertParams.from_hf_config(gpu.config)
    gen = torch.Generator().manual_seed(17)
    kinds = ["query"] * 12 + ["document"] * 12
    lengths = torch.randint(8, 49, (12,), generator=gen).tolist() + torch.randint(65, 400, (12,), generator=gen).tolist()
    seqs = [torch.randint(5, vocab, (l,), generator=gen) for l in lengths]
    windows = pe.mixed_windows(kinds, lengths, requests_per_window=8, query_fraction=0.5, windows=3, seed=1)
    assert all(sum(kinds[i] == "query" for i in w) == 4 and len(set(w)) == 8 for w in windows)
    for chosen in windows:
        window, pooled = pe.encode_window(gpu, params, [seqs[i] for i in chosen], chosen,
                                          [kinds[i] for i in chosen], pool="mean")
        assert window.requests == chosen and pooled.shape == (8, 256)
        for kind in ("query", "document"):
            slots = [n for n, i in enumerate(chosen) if kinds[i] == kind]
            _, split = pe.encode_window(gpu, params, [seqs[chosen[n]] for n in slots], pool="mean")
            assert float((pooled[slots].float() - split.float()).abs().max()) <= 2.0 ** -7
    # arrival-order windows sized for graph buckets: nothing reordered, budgets respected
    plan = pe.plan_windows(lengths, token_buckets=(512, 2048), max_sequences=8)
    assert [i for w in plan for i in w] == list(range(len(lengths)))
    assert all(sum(lengths[i] for i in w) <= 2048 or len(w) == 1 for w in plan) and all(len(w) <= 8 for w in plan)
