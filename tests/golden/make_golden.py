"""Generates the golden fixtures in this directory. Run where a checkout of the reference
(pau-mensa/flash-modernbert) is available; it is imported from the directory REFERENCE_ROOT names:

    REFERENCE_ROOT=<checkout of the reference> python tests/golden/make_golden.py

Fixtures (all small .npz files, committed):
  unpad_cases.npz     outputs of the reference's own _unpad / _repad
                      (packed_encoders/forward.py:384-412) on hand-made and random masks,
                      including the vectors of tests/test_varlen.py:62-99
  pack_sequences.npz  outputs of benchmarks/helpers/packed_collator.py:68-96
  rope_tables.npz     rows of the reference's _rope_tables (packed_encoders/forward.py:40-51)
                      for theta 160000 and 10000, stored as raw bf16 bits
  hf_tiny.npz         Hugging Face ModernBertModel eager fp32 last hidden state of the
                      seeded "tiny" model on the "tiny_mixed" workload (fp16 storage)
The tests never import the reference; they read these files.
"""
from __future__ import annotations

import os
import sys
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).resolve().parent
ROOT = HERE.parent.parent
REFERENCE_ROOT = os.environ.get("REFERENCE_ROOT")
if not REFERENCE_ROOT or not Path(REFERENCE_ROOT, "packed_encoders").is_dir():
    raise SystemExit("set REFERENCE_ROOT to a checkout of the reference (the directory that holds packed_encoders/)")
sys.path.insert(0, str(ROOT))
sys.path.insert(0, REFERENCE_ROOT)

from oracle import synthetic  # noqa: E402

TINY_VOCAB = 1024
ROPE_ROWS = np.unique(np.concatenate([np.arange(0, 256), np.arange(256, 8192, 61), [8191]]))


def masks() -> dict[str, np.ndarray]:
    gen = torch.Generator().manual_seed(0)
    cases = {
        # tests/test_varlen.py:62-80
        "ref_lengths_5_2_4": np.array([[1, 1, 1, 1, 1], [1, 1, 0, 0, 0], [1, 1, 1, 1, 0]]),
        # tests/test_varlen.py:83-90
        "ref_roundtrip": np.array([[1, 1, 1, 0], [1, 0, 0, 0], [1, 1, 1, 1]]),
        # tests/test_varlen.py:93-99
        "ref_no_padding": np.ones((2, 3), dtype=np.int64),
        "single_token": np.array([[1]]),
        "left_padded": np.array([[0, 0, 1, 1], [0, 1, 1, 1], [1, 1, 1, 1]]),
        "holes": np.array([[1, 0, 1, 0, 1, 1, 0], [0, 0, 0, 0, 0, 0, 1], [1, 1, 1, 1, 1, 1, 1]]),
        "one_empty_row": np.array([[1, 1, 0], [0, 0, 0], [1, 0, 0]]),
    }
    for name, (b, s) in {"rand_32x485": (32, 485), "rand_7x1000": (7, 1000), "rand_300x33": (300, 33)}.items():
        lens = torch.randint(1, s + 1, (b,), generator=gen)
        lens[0] = s
        cases[name] = (torch.arange(s)[None, :] < lens[:, None]).to(torch.int64).numpy()
    return {k: np.asarray(v, dtype=np.int64) for k, v in cases.items()}


def main() -> None:
    from packed_encoders import forward as ref_forward
    from benchmarks.helpers.packed_collator import pack_sequences as ref_pack

    # ---- unpad / repad -------------------------------------------------------
    out = {}
    gen = torch.Generator().manual_seed(1)
    for name, mask in masks().items():
        b, s = mask.shape
        x = torch.randint(-1000, 1000, (b, s, 3), generator=gen, dtype=torch.int64)
        xp, idx, cu, max_s, pos = ref_forward._unpad(x, torch.from_numpy(mask))
        rep = ref_forward._repad(xp, idx, b, s)
        out[f"{name}.mask"] = mask
        out[f"{name}.x"] = x.numpy()
        out[f"{name}.x_packed"] = xp.numpy()
        out[f"{name}.indices"] = idx.numpy()
        out[f"{name}.cu_seqlens"] = cu.numpy()
        out[f"{name}.max_seqlen"] = np.asarray(max_s, dtype=np.int64)
        out[f"{name}.position_ids"] = pos.numpy()
        out[f"{name}.repad"] = rep.numpy()
        assert cu.dtype == torch.int32 and idx.dtype == torch.int64 and pos.dtype == torch.int64
    np.savez_compressed(HERE / "unpad_cases.npz", **out)

    # ---- pack_sequences --------------------------------------------------------
    gen = torch.Generator().manual_seed(2)
    lens = torch.randint(1, 200, (37,), generator=gen).tolist()
    seqs = [torch.randint(5, 50368, (n,), generator=gen) for n in lens]
    batch = ref_pack(seqs)
    np.savez_compressed(
        HERE / "pack_sequences.npz",
        lengths=np.asarray(lens, dtype=np.int64),
        ids=torch.cat(seqs).numpy(),
        input_ids=batch.input_ids.numpy(),
        cu_seqlens=batch.cu_seqlens.numpy(),
        max_seqlen=np.asarray(batch.max_seqlen, dtype=np.int64),
        position_ids=batch.position_ids.numpy(),
    )

    # ---- rope tables -------------------------------------------------------------
    rope = {"rows": ROPE_ROWS.astype(np.int64)}
    for theta in (160000.0, 10000.0):
        cos, sin = ref_forward._rope_tables(8192, 64, theta, "cpu", torch.bfloat16)
        rows = torch.from_numpy(ROPE_ROWS)
        rope[f"cos_{int(theta)}"] = cos[0].index_select(0, rows).view(torch.int16).numpy()
        rope[f"sin_{int(theta)}"] = sin[0].index_select(0, rows).view(torch.int16).numpy()
    np.savez_compressed(HERE / "rope_tables.npz", **rope)

    # ---- HF eager fp32 on the tiny model -----------------------------------------
    from oracle import packed_oracle

    model = synthetic.make_model("tiny", TINY_VOCAB)
    wl = synthetic.workload("tiny_mixed", TINY_VOCAB)
    hidden = packed_oracle.hf_eager_packed(model, wl.sequences())
    # the same batch through HF's padded path, to pin that per-sequence == padded
    b, s = len(wl.lengths), wl.max_seqlen
    ids = torch.zeros(b, s, dtype=torch.int64)
    mask = torch.zeros(b, s, dtype=torch.int64)
    for i, seq in enumerate(wl.sequences()):
        ids[i, : seq.numel()] = seq
        mask[i, : seq.numel()] = 1
    padded = packed_oracle.hf_eager_padded(model, ids, mask)
    padded_real = padded[mask.bool()]
    assert torch.allclose(padded_real, hidden, atol=2e-5, rtol=1e-4), (padded_real - hidden).abs().max()
    np.savez_compressed(
        HERE / "hf_tiny.npz",
        lengths=np.asarray(wl.lengths, dtype=np.int64),
        ids=wl.ids.numpy(),
        last_hidden_state=hidden.to(torch.float16).numpy(),
        vocab=np.asarray(TINY_VOCAB, dtype=np.int64),
    )
    for f in sorted(HERE.glob("*.npz")):
        print(f.name, f.stat().st_size)


if __name__ == "__main__":
    main()
