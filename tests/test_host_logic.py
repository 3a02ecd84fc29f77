"""Host-side logic that needs no GPU: the C-ABI library loads and exports what the header
declares, config / locate / state / errors semantics, graph bucketing policy, collation,
shard planning, and loud failure without CUDA."""
from __future__ import annotations

import re
from types import SimpleNamespace

import numpy as np
import pytest
import torch
from torch import nn

from conftest import ROOT


def test_library_exports_every_declared_symbol(pe):
    from flash_modernbert_b200 import _lib

    header = (ROOT / "include" / "pe_b200.h").read_text()
    header = re.sub(r"/\*.*?\*/", "", header, flags=re.S)
    declared = set(re.findall(r"\b(pe_[a-z0-9_]+)\s*\(", header))
    assert declared, "no declarations parsed from the header"
    lib = _lib.load()
    for name in sorted(declared):
        assert hasattr(lib, name), f"{name} is declared in include/pe_b200.h but not exported"
    assert declared == set(_lib.PROTOTYPES), declared ^ set(_lib.PROTOTYPES)
    assert lib.pe_version() >= 100


def test_argument_errors_do_not_need_a_gpu(pe):
    from flash_modernbert_b200 import _lib

    lib = _lib.load()
    assert lib.pe_geglu(None, 4, 8, None, None) == _lib.PE_ERR_ARG
    assert "null" in _lib.last_error()
    assert lib.pe_set_option(99, 1) == _lib.PE_ERR_ARG
    assert lib.pe_forward_workspace_bytes(None, 10, 1) == 0
    with pytest.raises(_lib.NativeLibraryError):
        _lib.check(_lib.PE_ERR_ARG, "probe")


def test_missing_library_fails_loudly(pe, tmp_path):
    from flash_modernbert_b200 import _lib

    with pytest.raises(_lib.NativeLibraryError, match="no fallback"):
        _lib.load(tmp_path / "libpe_b200.so")


def test_cpu_tensors_are_refused(pe):
    from flash_modernbert_b200 import forward

    with pytest.raises(pe.PackedEncodersError, match="CUDA"):
        forward._unpad(torch.zeros(2, 3, 1), torch.ones(2, 3, dtype=torch.long))
    with pytest.raises(pe.PackedEncodersError, match="CUDA"):
        forward._repad(torch.zeros(2, 4), torch.tensor([0, 1]), 1, 2)


def _hf_config(**kw):
    from transformers import ModernBertConfig

    return ModernBertConfig(**kw)


def test_params_from_hf_config(pe):
    p = pe.ModernBertParams.from_hf_config(_hf_config())
    assert (p.hidden_size, p.num_attention_heads, p.num_hidden_layers) == (768, 12, 22)
    assert p.head_dim == 64 and p.scaling == 0.125 and p.sliding_half_window == 64
    assert (p.global_rope_theta, p.local_rope_theta) == (160000.0, 10000.0)
    assert p.global_attn_every_n_layers == 3
    assert [p.is_global_layer(i) for i in range(4)] == [True, False, False, True]
    flat = SimpleNamespace(model_type="modernbert", hidden_size=128, num_attention_heads=2,
                           num_hidden_layers=2, norm_eps=1e-5, global_rope_theta=5.0,
                           local_rope_theta=7.0, local_attention=128, global_attn_every_n_layers=2)
    q = pe.ModernBertParams.from_hf_config(flat)
    assert (q.global_rope_theta, q.local_rope_theta, q.global_attn_every_n_layers) == (5.0, 7.0, 2)
    with pytest.raises(ValueError):
        pe.ModernBertParams.from_hf_config(SimpleNamespace(model_type="bert"))


class _FakeEncoder(nn.Module):
    def __init__(self):
        super().__init__()
        self.config = SimpleNamespace(model_type="modernbert")
        self.embeddings = nn.Identity()
        self.layers = nn.ModuleList()
        self.final_norm = nn.Identity()


def test_find_encoder_walks_wrappers(pe):
    enc = _FakeEncoder()
    assert pe.find_encoder(enc) is enc
    head = nn.Module()
    head.model = enc
    assert pe.find_encoder(head) is enc
    st = nn.Module()
    st.auto_model = enc
    pipeline = nn.Sequential(st, nn.Identity())
    assert pe.find_encoder(pipeline) is enc
    with pytest.raises(pe.UnsupportedTargetError):
        pe.find_encoder(nn.Linear(2, 2))
    with pytest.raises(pe.UnsupportedTargetError):
        pe.find_encoder(object())
    with pytest.raises(pe.PackedEncodersError):
        pe.get_state(enc)
    assert pe.unpack(enc) is enc  # unpatched: no-op


def test_pack_refuses_cpu_models_and_bad_arguments(pe):
    from oracle import synthetic as S

    model = S.make_model("tiny", 1024)
    with pytest.raises(pe.PackedEncodersError):
        pe.pack(model, validate=False)            # CPU weights
    with pytest.raises(pe.ValidationError):
        pe.validate(model)
    with pytest.raises(pe.PackedEncodersError):
        pe.pack(model, attention_backend="bogus")
    with pytest.raises(pe.PackedEncodersError):
        pe.pack(model, train_cuda_graph=True)
    assert not hasattr(model, "_packed_encoders")


def test_graph_bucket_policy(pe):
    from flash_modernbert_b200 import graph

    runner = graph._PackedGraphRunner.__new__(graph._PackedGraphRunner)
    runner._config = pe.GraphConfig(pad_to=64, max_batch=1024, max_seq=64, max_tokens=50000)
    # one key for ragged traffic inside a bucket: N and Smax are not part of it
    assert runner.bucket_for(28671, 1024, 48) == (28672, 1024, 64)
    assert runner.bucket_for(28650, 900, 40) == (28672, 1024, 64)
    assert runner.bucket_for(100, 3, 30) == (128, 1024, 32)
    assert runner.bucket_for(100, 3, 16) == (128, 1024, 16)
    assert runner.bucket_for(100, 1025, 16) is None      # too many sequences
    assert runner.bucket_for(100, 3, 65) is None         # too long
    assert runner.bucket_for(50001, 3, 16) is None       # over max_tokens
    runner._config = pe.GraphConfig(token_buckets=(1024, 4096, 16384))
    assert runner.bucket_for(1000, 5, 100) == (1024, 8, 128)
    assert runner.bucket_for(1025, 9, 64) == (4096, 16, 64)
    assert runner.bucket_for(1025, 9, 65) == (4096, 16, 128)
    assert runner.bucket_for(16385, 9, 100) is None
    # graphs captured at pack() time: packed_encoders/graph.py:410-427 pre-captures the listed
    # sequence buckets at max_batch rows; here one key per bucket, largest capacity first
    runner._config = pe.GraphConfig(pad_to=256, max_batch=64, max_seq=64, seq_buckets=(16, 32, 64))
    assert runner.precapture_keys() == [(4096, 64, 64), (2048, 64, 32), (1024, 64, 16)]
    runner._config = pe.GraphConfig(max_batch=8, token_buckets=(1024, 4096), max_seq=48)
    assert runner.precapture_keys() == [(4096, 8, 64), (1024, 8, 64)]
    runner._config = pe.GraphConfig(seq_buckets=(16,))          # no max_batch: nothing to size them by
    assert runner.precapture_keys() == []


def test_graph_runner_lru_with_fakes(pe, monkeypatch):
    """Cache order and eviction with fake capture objects, as the reference tests its packed
    runner on the CPU (tests/test_graph_bucketing.py:237-294)."""
    from flash_modernbert_b200 import forward, graph

    class FakeGraph:
        def replay(self):
            pass

    class FakeInputs:
        def stage(self, ids, cu, pos):
            return ids.shape[0]

    runner = graph._PackedGraphRunner.__new__(graph._PackedGraphRunner)
    runner._config = pe.GraphConfig(pad_to=64, max_batch=8, max_seq=512, max_graphs=2)
    runner._model = runner._params = None
    runner._cache = __import__("collections").OrderedDict()
    runner._generation = 0
    runner.captures = runner.replays = runner.eager_calls = 0
    monkeypatch.setattr(forward, "get_binding",
                        lambda m, p: SimpleNamespace(max_positions=8192, generation=0,
                                                     check=lambda: None, after_call=lambda: None))
    captured_keys = []

    def fake_capture(token_cap, seq_cap, rows):
        captured_keys.append((token_cap, seq_cap, rows))
        return graph._PackedCaptured(graph=FakeGraph(), inputs=FakeInputs(),
                                     out=torch.zeros(token_cap, 4))

    monkeypatch.setattr(runner, "_capture", fake_capture)
    monkeypatch.setattr(runner, "_eager", lambda *a: "eager")

    def call(total, n, smax):
        return runner(torch.zeros(total, dtype=torch.long), torch.zeros(n + 1, dtype=torch.int32),
                      smax, torch.zeros(total, dtype=torch.long))

    assert call(60, 2, 40).shape == (60, 4)
    assert call(64, 5, 64).shape == (64, 4)         # same bucket: no new capture
    assert captured_keys == [(64, 8, 64)]
    call(100, 2, 40)
    call(200, 2, 40)                                # evicts the least recently used (64)
    assert list(runner._cache) == [(128, 8, 64), (256, 8, 64)]
    call(100, 2, 40)                                # promote 128
    call(300, 2, 40)                                # evicts 256
    assert list(runner._cache) == [(128, 8, 64), (320, 8, 64)]
    assert call(100, 9, 40) == "eager" and runner.eager_calls == 1


def test_pack_sequences_collator(pe):
    batch = pe.pack_sequences([[11, 12], [21], [31, 32, 33]])
    assert batch.input_ids.tolist() == [11, 12, 21, 31, 32, 33]
    assert batch.cu_seqlens.tolist() == [0, 2, 3, 6] and batch.cu_seqlens.dtype == torch.int32
    assert batch.position_ids.tolist() == [0, 1, 0, 0, 1, 2] and batch.max_seqlen == 3
    assert batch.forward_args()[2] == 3
    with pytest.raises(ValueError):
        pe.pack_sequences([])
    with pytest.raises(ValueError):
        pe.pack_sequences([[1], []])


def test_positions_from_cu_seqlens(pe):
    from flash_modernbert_b200 import forward

    cu = torch.tensor([0, 2, 3, 6, 6], dtype=torch.int32)
    assert forward.positions_from_cu_seqlens(cu, 6).tolist() == [0, 1, 0, 0, 1, 2]


def test_shard_plan_balances_and_restores(pe):
    from flash_modernbert_b200 import shard
    from oracle import synthetic as S

    lengths = S.workload("cfg3").lengths
    costs = shard.sequence_costs(lengths, hidden=768, intermediate=1152, n_layers=22, n_global=8)
    for world in (1, 2, 4, 8):
        plan = shard.plan_shards(lengths, world, costs)
        seen = np.sort(np.concatenate(plan.groups))
        assert np.array_equal(seen, np.arange(len(lengths)))       # every sequence exactly once
        loads = np.asarray([costs[g].sum() for g in plan.groups])
        assert loads.max() / loads.mean() < 1.02                    # cost-balanced within 2 %
        restore = plan.restore_index()
        assert np.array_equal(np.sort(restore), np.arange(plan.total_tokens))   # a permutation of the rows
        # each rank's rows are one contiguous range of the gathered tensor
        for r, g in enumerate(plan.groups):
            rows = np.sort(np.concatenate([plan.seq_rows[i] + np.arange(lengths[i]) for i in g]))
            assert rows[0] == plan.row_start[r] and rows[-1] == plan.row_start[r + 1] - 1
            assert np.array_equal(rows, np.arange(rows[0], rows[-1] + 1))
        assert np.array_equal(plan.order[plan.seq_slot], np.arange(len(lengths)))
    # the FLOP model's local-layer pair count (129 s - 4160 beyond 65 tokens)
    assert shard.local_pairs(np.array([10, 65, 66, 1000])).tolist() == [100, 4225, 4354, 124840]
    with pytest.raises(ValueError):
        shard.plan_shards([], 2)


def test_token_budget_batches_follow_the_greedy_rule(pe):
    """benchmarks/helpers/packed_training.py:175-202 of the reference: a new batch starts when the
    next unit would exceed the budget; a batch always takes at least one unit."""
    lengths = [5, 3, 9, 2, 2, 7, 1]
    batches = pe.token_budget_batches(lengths, 10, sort_by_length=False)
    assert batches == [[0, 1], [2], [3, 4], [5, 6]]
    assert all(sum(lengths[i] for i in b) <= 10 for b in batches)
    assert pe.token_budget_batches([30, 2], 10, sort_by_length=False) == [[0], [1]]   # oversize unit alone
    longest_first = pe.token_budget_batches(lengths, 10)
    assert sorted(i for b in longest_first for i in b) == list(range(7))
    assert longest_first[0] == [2] and all(sum(lengths[i] for i in b) <= 10 for b in longest_first)
    capped = pe.token_budget_batches([1] * 7, 100, max_sequences=3)
    assert [len(b) for b in capped] == [3, 3, 1]
    import pytest
    with pytest.raises(ValueError):
        pe.token_budget_batches([1, 0], 10)
    with pytest.raises(ValueError):
        pe.token_budget_batches([1], 0)
