"""The N > 1 gather path with world_size 2 on the CPU (gloo): each rank 'encodes' its
shard with a stand-in function of the token id, and every rank must receive the rows
of all sequences in the original packed order."""
from __future__ import annotations

import os
import socket

import numpy as np
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from conftest import load_package


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank: int, world: int, port: int, lengths, result_dir: str):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        load_package()
        from flash_modernbert_b200 import shard

        total = int(sum(lengths))
        ids = torch.arange(total, dtype=torch.int64)
        seqs = list(torch.split(ids, lengths))
        plan = shard.plan_shards(lengths, world)
        mine = shard.local_batch(plan, rank, seqs)
        local_ids = torch.cat(mine) if mine else torch.zeros(0, dtype=torch.int64)
        # stand-in encoder: row t = [id, 2*id, rank]
        local_out = torch.stack([local_ids.float(), 2 * local_ids.float(),
                                 torch.full_like(local_ids, rank).float()], dim=1)
        ranked = shard.gather_embeddings(local_out, plan)          # rank-major: no permutation
        assert ranked.shape == (total, 3)
        for i, n in enumerate(lengths):
            rows = ranked[plan.seq_rows[i]:plan.seq_rows[i] + n]
            assert torch.equal(rows[:, 0], seqs[i].float())
        assert np.array_equal(plan.gathered_cu_seqlens(),
                              np.concatenate(([0], np.cumsum(np.asarray(lengths)[plan.order]))))
        full = shard.gather_embeddings(local_out, plan, restore=True)
        assert full.shape == (total, 3)
        assert torch.equal(full[:, 0], ids.float()) and torch.equal(full[:, 1], 2 * ids.float())
        owners = np.empty(total, dtype=np.int64)
        starts = np.concatenate(([0], np.cumsum(lengths)))
        for r, g in enumerate(plan.groups):
            for i in g:
                owners[starts[i]:starts[i + 1]] = r
        assert np.array_equal(full[:, 2].numpy().astype(np.int64), owners)
        # the pooled gather: one row per sequence, back in the callers' order
        first_ids = torch.stack([m[0].float() for m in mine]) if mine else torch.zeros(0)
        pooled = torch.stack([first_ids, torch.full_like(first_ids, float(rank))], dim=1)
        all_pooled = shard.gather_pooled(pooled, plan)
        assert all_pooled.shape == (len(lengths), 2)
        assert torch.equal(all_pooled[:, 0], torch.tensor(starts[:-1], dtype=torch.float32))
        seq_owner = np.empty(len(lengths), dtype=np.int64)
        for r, g in enumerate(plan.groups):
            seq_owner[np.asarray(g, dtype=np.int64)] = r
        assert np.array_equal(all_pooled[:, 1].numpy().astype(np.int64), seq_owner)
        ranked_pooled = shard.gather_pooled(pooled, plan, restore=False)
        assert torch.equal(ranked_pooled[:, 0], torch.tensor(starts[:-1][plan.order], dtype=torch.float32))
        with open(os.path.join(result_dir, f"ok{rank}"), "w") as f:
            f.write("ok")
    finally:
        dist.destroy_process_group()


def test_gather_embeddings_world2(tmp_path):
    lengths = [5, 3, 8, 2, 7, 1, 9]
    mp.spawn(_worker, args=(2, _free_port(), lengths, str(tmp_path)), nprocs=2, join=True)
    assert (tmp_path / "ok0").exists() and (tmp_path / "ok1").exists()


def test_single_rank_is_identity():
    load_package()
    from flash_modernbert_b200 import shard

    plan = shard.plan_shards([4, 2, 6], 1)
    seqs = list(torch.split(torch.arange(12), [4, 2, 6]))
    local = torch.cat(shard.local_batch(plan, 0, seqs)).float().unsqueeze(1)
    assert torch.equal(shard.gather_embeddings(local, plan, restore=True)[:, 0], torch.arange(12).float())
    pooled = torch.tensor([[0.0], [4.0], [6.0]])                       # one row per sequence, callers' order
    local_rows = pooled[torch.from_numpy(np.asarray(plan.groups[0]))]   # as rank 0 produces them
    assert torch.equal(shard.gather_pooled(local_rows, plan), pooled)
