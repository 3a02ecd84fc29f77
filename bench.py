"""Benchmark of the packed ModernBERT forward: packed tokens/s, ModernBERT-base document
encoding (512 documents, lognormal lengths, 306,851 tokens per GPU), bf16, on N B200s.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload cfg3]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
        --master-port P bench.py --gpus N --steps K --warmup W

One step = one pass of `packed_forward` over this rank's shard of the batch. For N > 1 the step
also pools the hidden state into one embedding per document (inside the final LayerNorm) and
gathers those embeddings over NCCL, which is what a multi-GPU caller consumes; the gather of the
full `[T, H]` token embeddings is timed as well and reported beside it. Weak scaling: the global
batch is N seeded copies of the workload, split into cost-balanced document groups, one per rank.

Rank 0 prints ONE JSON line. Besides the headline workload it carries, under "workloads", the
other seeded configurations (query batch with and without CUDA graphs, long documents on the large
model, the mixed 1B-class index in token-budget micro-batches). `--impl reference` times the
unmodified reference (`packed_encoders` installed under baseline/_ref) on the same inputs, shard
plan and gathers, falling back to Hugging Face eager fp32 on the host cores if the reference's GPU
path does not run.
"""
from __future__ import annotations

import argparse
import importlib.util
import json
import os
import statistics
import sys
import threading
import time
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

METRIC = "packed tokens/sec, ModernBERT-base doc encode bf16"
# DRAM bytes (read + write) of the four GEMM launches of one ModernBERT-base layer per token,
# measured once with ncu on a 71,567-token slice of the workload. GEMM traffic grows in proportion
# to the rows, so a full launch is this times its tokens; the JSON line says that it is scaled.
NCU_GEMM_DRAM_BYTES_PER_TOKEN = 1259.7e6 / 71567
UNIT = "tokens/s"
DATA = "synthetic (seeded lengths and token ids, random-init weights normal(0, 0.02))"
CFG5_TOKEN_BUDGET = 262144

WORKLOAD_TEXT = {
    "cfg1": "cfg1: ModernBERT-base, 32 sequences, lengths uniform [16, 512]",
    "cfg2": "cfg2: ModernBERT-base, 1,024 queries, lengths uniform [8, 48]",
    "cfg3": "cfg3: ModernBERT-base, 512 documents, lengths lognormal(median 400, sigma 0.8) clipped to [64, 8192]",
    "cfg3q": "cfg3q: every fourth document of cfg3 (profiling slice)",
    "cfg4": "cfg4: ModernBERT-large, 64 documents, lengths uniform [2048, 8192]",
    "cfg5": "cfg5: 1B-class ModernBERT, 8,192 queries uniform [8, 48] + 8,192 documents lognormal(median 600, sigma 0.8) "
            "clipped to [64, 4096], token-budget micro-batches of 262,144 tokens",
}


def workload_text(name: str) -> str:
    """The `config.workload` string; both arms print the same one for the same workload."""
    return WORKLOAD_TEXT.get(name, name) + "; packed by cu_seqlens, length-descending, one seeded copy per GPU"


def load_package():
    name = "flash_modernbert_b200"
    if name in sys.modules:
        return sys.modules[name]
    pkg = ROOT / "flash-modernbert_b200"
    spec = importlib.util.spec_from_file_location(name, pkg / "__init__.py",
                                                  submodule_search_locations=[str(pkg)])
    module = importlib.util.module_from_spec(spec)
    sys.modules[name] = module
    spec.loader.exec_module(module)
    return module


# ---------------------------------------------------------------------------
# clocks
# ---------------------------------------------------------------------------


class ClockSampler:
    """Samples SM clock and throttle reasons of one GPU through NVML while running (read-only)."""

    REASONS = {
        0x8: "hw_slowdown", 0x40: "hw_thermal_slowdown", 0x20: "sw_thermal_slowdown",
        0x4: "sw_power_cap", 0x80: "hw_power_brake_slowdown",
    }

    def __init__(self, index: int, period_s: float = 0.02):
        self.index, self.period = index, period_s
        self.samples: list[int] = []
        self.times: list[float] = []
        self.reasons: set[str] = set()
        self.max_mhz = None
        self._stop = threading.Event()
        self._thread = None
        try:
            import pynvml

            pynvml.nvmlInit()
            self._nvml = pynvml
            self._handle = pynvml.nvmlDeviceGetHandleByIndex(self._physical_index(index))
            self.max_mhz = int(pynvml.nvmlDeviceGetMaxClockInfo(self._handle, pynvml.NVML_CLOCK_SM))
        except Exception:  # noqa: BLE001 - clocks are reported as unavailable
            self._nvml = None

    @staticmethod
    def _physical_index(index: int) -> int:
        visible = os.environ.get("CUDA_VISIBLE_DEVICES")
        if visible:
            parts = [p for p in visible.split(",") if p.strip()]
            if index < len(parts) and parts[index].strip().isdigit():
                return int(parts[index])
        return index

    def _loop(self):
        n = self._nvml
        while not self._stop.is_set():
            try:
                self.samples.append(int(n.nvmlDeviceGetClockInfo(self._handle, n.NVML_CLOCK_SM)))
                self.times.append(time.perf_counter())
                mask = int(n.nvmlDeviceGetCurrentClocksEventReasons(self._handle))
                for bit, name in self.REASONS.items():
                    if mask & bit:
                        self.reasons.add(name)
            except Exception:  # noqa: BLE001
                pass
            self._stop.wait(self.period)

    def __enter__(self):
        if self._nvml is not None:
            self._thread = threading.Thread(target=self._loop, daemon=True)
            self._thread.start()
        return self

    def __exit__(self, *exc):
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=2)
        return False

    def median_between(self, t0: float, t1: float):
        picks = [s for s, t in zip(self.samples, self.times) if t0 <= t <= t1]
        return int(statistics.median(picks)) if picks else None

    def summary(self) -> dict:
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": ["unavailable"]}
        return {"sm_mhz": int(statistics.median(self.samples)), "sm_max_mhz": self.max_mhz,
                "reasons": sorted(self.reasons), "samples": len(self.samples)}


# ---------------------------------------------------------------------------
# workload
# ---------------------------------------------------------------------------


def measured_peaks() -> dict:
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        p = json.loads(path.read_text())
        return {"hbm_gbs": p["hbm_gbs"], "bf16_tflops": p["bf16_tflops"],
                "bf16_tflops_sustained": p.get("bf16_tflops_sustained", p["bf16_tflops"]),
                "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0,
            "source": "fallback"}


def build_global_batch(workload: str, world: int):
    """N seeded copies of the workload (copy r uses seed r), each length-descending."""
    from oracle import synthetic as S

    lengths, seqs, arch = [], [], None
    for r in range(world):
        wl = S.workload(workload, seed=r).sorted_by_length()
        arch = wl.arch
        lengths += wl.lengths
        seqs += wl.sequences()
    return arch, lengths, seqs


def model_flops(model, lengths) -> dict:
    """Algorithmic work of one forward over `lengths` (multiply-add = 2 FLOPs) and the
    minimum tail traffic of the unfused op list and of the op list this library runs, bf16."""
    import numpy as np

    load_package()
    from flash_modernbert_b200 import shard

    cfg = model.config
    H, I, L = cfg.hidden_size, cfg.intermediate_size, len(model.layers)
    G = sum(1 for l in model.layers if getattr(l, "attention_type", "") == "full_attention")
    s = np.asarray(lengths, dtype=np.float64)
    T = float(s.sum())
    gemm = T * L * (8.0 * H * H + 6.0 * H * I)
    attn = 4.0 * H * (G * float((s * s).sum()) + (L - G) * float(shard.local_pairs(s).sum()))
    tail = 4 * T * H + L * (2 * 8 * T * H + 8 * T * H + 256 * T + 6 * T * I) - 8 * T * H + 6 * T * H
    # fused op list: embed+LN (4TH), 2L-1 plain LayerNorms (4TH each), final LN (4TH); the residual
    # reads of the two residual GEMMs (2TH each) are counted with the tails they replace
    tail_fused = 4 * T * H + (2 * L - 1) * 4 * T * H + 4 * T * H + 2 * L * 2 * T * H
    return {"gemm_flops": gemm, "attn_flops": attn, "tail_bytes": tail, "tail_bytes_fused": tail_fused,
            "tokens": T}


def launches_per_forward(model, max_seqlen: int, pooled: bool = False) -> int:
    """Kernels of libpe_b200.so that one forward enqueues."""
    n = 3  # embedding+LN, attention schedule, zeroing of bucket-padding rows
    per_attn = 2 if max_seqlen > 64 else 1  # tensor-memory kernel + the short-sequence kernel
    for layer in model.layers:
        has_norm = not isinstance(layer.attn_norm, torch.nn.Identity)
        n += (1 if has_norm else 0) + 5 + per_attn  # Wqkv+RoPE, attention, Wo, LN, Wi+GeGLU, Wo_mlp
    return n + (3 if pooled else 1)  # final LN, or pool schedule + fused LN/pool + finish


def time_gemm_kernels(model, tokens: int, device, clocks: "ClockSampler | None" = None,
                      bursts: int = 6, burst_len: int = 8, sustained_reps: int = 40) -> dict:
    """Duration of each GEMM launch shape of one layer, timed alone with CUDA events on the
    launching stream (each launch streams > 126 MB, so L2 does not hold it), two ways: the best of
    several short bursts after a pause (how the burst peak it is compared with was measured: best
    of 10), and the average of a long back-to-back run under the power cap (the sustained figure)."""
    load_package()
    from flash_modernbert_b200 import ops

    cfg = model.config
    H, I = cfg.hidden_size, cfg.intermediate_size
    layer = model.layers[1]
    gen = torch.Generator(device=device).manual_seed(0)
    xh = torch.randn(tokens, H, device=device, generator=gen).to(torch.bfloat16)
    xi = torch.randn(tokens, I, device=device, generator=gen).to(torch.bfloat16)
    pos = torch.arange(tokens, device=device, dtype=torch.int64) % 512
    xres = torch.zeros(tokens, H, device=device, dtype=torch.bfloat16)
    table = ops.rope_table(10000.0, 8192, device)
    nh = cfg.num_attention_heads
    shapes = {
        "Wqkv+RoPE": (lambda: ops.linear_qkv_rope(xh, layer.attn.Wqkv.weight, pos, table, nh),
                      2.0 * tokens * 3 * H * H),
        "Wo+residual": (lambda: ops.linear_residual(xh, layer.attn.Wo.weight, xres, inplace=True),
                        2.0 * tokens * H * H),
        "Wi+GeGLU": (lambda: ops.linear_geglu(xh, layer.mlp.Wi.weight), 2.0 * tokens * 2 * I * H),
        "Wo_mlp+residual": (lambda: ops.linear_residual(xi, layer.mlp.Wo.weight, xres, inplace=True),
                            2.0 * tokens * I * H),
    }

    def timed(fn, reps):
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0 = time.perf_counter()
        start.record()
        for _ in range(reps):
            fn()
        end.record()
        torch.cuda.synchronize(device)
        return start.elapsed_time(end) / reps, t0, time.perf_counter()

    out = {}
    for name, (fn, flops) in shapes.items():
        for _ in range(3):
            fn()
        torch.cuda.synchronize(device)
        best = None
        for _ in range(bursts):
            time.sleep(0.03)
            ms, _, _ = timed(fn, burst_len)
            best = ms if best is None else min(best, ms)
        ms_sus, t0, t1 = timed(fn, sustained_reps)
        mhz = clocks.median_between(t0, t1) if clocks is not None else None
        out[name] = {"ms": round(best, 4), "tflops": round(flops / best / 1e9, 1), "flops": flops,
                     "ms_sustained": round(ms_sus, 4), "tflops_sustained": round(flops / ms_sus / 1e9, 1),
                     "sm_mhz_sustained": mhz, "kcycles_sustained": round(ms_sus * mhz, 1) if mhz else None}
    return out


def cpu_baseline_hf_eager(arch: str, seqs, target_tokens: int = 6000) -> dict:
    """Hugging Face eager fp32 on the host cores over a bounded, evenly spaced sample of the
    workload's sequences."""
    from oracle import packed_oracle as O
    from oracle import synthetic as S

    model = S.make_model(arch)
    stride = max(1, len(seqs) // 16)
    sample, tokens = [], 0
    for seq in seqs[stride // 2::stride]:
        if tokens + seq.numel() > target_tokens and sample:
            continue
        sample.append(seq)
        tokens += seq.numel()
    O.hf_eager_packed(model, sample[-1:])  # warm-up on the shortest pick
    t0 = time.perf_counter()
    O.hf_eager_packed(model, sample)
    dt = time.perf_counter() - t0
    return {"value": round(tokens / dt, 1), "unit": UNIT, "cores": torch.get_num_threads(),
            "kind": "port", "impl": "Hugging Face ModernBertModel eager fp32 (oracle.hf_eager_packed)",
            "sample": f"{len(sample)} of {len(seqs)} sequences, {tokens} tokens, {dt:.1f} s"}


# ---------------------------------------------------------------------------
# plumbing shared by the two arms
# ---------------------------------------------------------------------------


def dist_setup(gpus: int):
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world > 1:
        import torch.distributed as dist

        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        torch.cuda.set_device(local_rank)
        from datetime import timedelta

        # a rank that fails outside a collective must not leave the others waiting for long
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank), timeout=timedelta(minutes=6))
    elif gpus > 1:
        raise SystemExit("--gpus N > 1 must be launched with torch.distributed.run (one rank per GPU)")
    return world, rank, local_rank


class OverlappedGather:
    """The end-of-step gather of the `[T, H]` token embeddings, issued on a stream of its own so
    that it overlaps the next step's forward. Every rank's rows land straight in their range of
    one preallocated result (two of them, alternating, so a step never waits for the previous
    gather's buffer). `drain()` makes the current stream wait for every gather issued so far;
    the timed region ends with it, so all K gathers lie inside the measurement."""

    def __init__(self, plan, shard_module, hidden: int, device):
        self.plan, self.shard = plan, shard_module
        self.stream = torch.cuda.Stream()
        self.results = [torch.empty(plan.total_tokens, hidden, dtype=torch.bfloat16, device=device)
                        for _ in range(2)]
        self.turn = 0

    def __call__(self, local_out):
        ready = torch.cuda.Event()
        ready.record()
        dst = self.results[self.turn]
        self.turn ^= 1
        with torch.cuda.stream(self.stream):
            self.stream.wait_event(ready)
            self.shard.gather_embeddings(local_out, self.plan, out=dst)
            local_out.record_stream(self.stream)
        return dst

    def drain(self):
        torch.cuda.current_stream().wait_stream(self.stream)


def timed_steps(step_fn, steps: int, warmup: int, world: int, device, drain_fn=None, per_step: bool = False):
    """Milliseconds per step: K steps between CUDA events, barrier + synchronize on both
    sides, maximum over ranks. `drain_fn` (if any) joins side streams before the end event.
    With `per_step` also returns (wall-clock start, [ms of each step on this rank])."""
    import torch.distributed as dist

    for _ in range(warmup):
        step_fn()
    if drain_fn is not None:
        drain_fn()
    torch.cuda.synchronize(device)
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize(device)
    marks = [torch.cuda.Event(enable_timing=True) for _ in range(steps + 1)]
    t0 = time.perf_counter()
    marks[0].record()
    for i in range(steps):
        step_fn()
        if i + 1 < steps:
            marks[i + 1].record()
    if drain_fn is not None:
        drain_fn()
    marks[steps].record()
    torch.cuda.synchronize(device)
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize(device)
    ms = torch.tensor([marks[0].elapsed_time(marks[steps]) / steps], device=device, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    if per_step:
        return float(ms.item()), t0, [marks[i].elapsed_time(marks[i + 1]) for i in range(steps)]
    return float(ms.item())


def clock_normalised(ms: float, t0: float, step_ms: list, clocks: ClockSampler) -> dict:
    """The step in clock-independent units: ms x median SM MHz = thousands of SM cycles, per step
    and binned by the clock each step ran at (the step is power-capped, so its clock moves)."""
    out = {"step_kcycles": None, "per_step": [], "by_clock": {}}
    mhz_all = clocks.summary().get("sm_mhz")
    if mhz_all:
        out["step_kcycles"] = round(ms * mhz_all, 1)
    t = t0
    bins: dict[int, list] = {}
    for dt in step_ms:
        mhz = clocks.median_between(t, t + dt / 1e3)
        t += dt / 1e3
        out["per_step"].append({"ms": round(dt, 3), "sm_mhz": mhz, "kcycles": round(dt * mhz, 1) if mhz else None})
        if mhz:
            bins.setdefault(int(round(mhz / 50.0)) * 50, []).append(dt)
    out["by_clock"] = {str(k): {"steps": len(v), "mean_ms": round(sum(v) / len(v), 3)} for k, v in sorted(bins.items())}
    return out


def reference_modules():
    """The unmodified reference, imported from its install under baseline/_ref."""
    ref_dir = str(ROOT / "baseline" / "_ref")
    if ref_dir not in sys.path:
        sys.path.insert(0, ref_dir)
    import packed_encoders as ref_pkg
    from packed_encoders import forward as ref_forward
    from packed_encoders import ops as ref_ops
    from packed_encoders.config import ModernBertParams as RefParams

    return ref_pkg, ref_forward, ref_ops, RefParams


def torch_mean_pool(hidden, seqlens_dev):
    """What the reference's showcase does with the output of packed_forward
    (benchmarks/showcases/inference.py:193-206): fp32 segment mean by index_add_, F.normalize."""
    import torch.nn.functional as F

    n = seqlens_dev.shape[0]
    segments = torch.repeat_interleave(torch.arange(n, device=hidden.device), seqlens_dev)
    sums = torch.zeros(n, hidden.shape[-1], device=hidden.device, dtype=torch.float32)
    sums.index_add_(0, segments, hidden.float())
    pooled = sums / seqlens_dev.unsqueeze(1).float()
    return F.normalize(pooled, p=2, dim=-1).to(hidden.dtype)


def make_encoder(impl: str, arch: str, device):
    """(model, forward(batch) -> [T, H], pooled(batch) -> [N, H]) for one arm."""
    from oracle import synthetic as S

    model = S.make_model(arch, dtype=torch.bfloat16, device=device)
    if impl == "ours":
        pe = load_package()
        params = pe.ModernBertParams.from_hf_config(model.config)

        def fwd(batch):
            return pe.packed_forward(model, params, *batch.forward_args())

        def pooled(batch):
            return pe.packed_forward_pooled(model, params, *batch.forward_args(), pool="mean", normalize=True)

        return model, params, fwd, pooled
    _, ref_forward, _, RefParams = reference_modules()
    if not hasattr(model.config, "global_attn_every_n_layers"):
        model.config.global_attn_every_n_layers = 3
    params = RefParams.from_hf_config(model.config)

    def fwd(batch):
        with torch.no_grad():
            return ref_forward.packed_forward(model, params, *batch.forward_args())

    def pooled(batch):
        return torch_mean_pool(fwd(batch), batch.seqlens_dev)

    return model, params, fwd, pooled


def to_device(batch, device):
    batch = batch.to(device)
    batch.seqlens_dev = batch.seqlens.to(device=device, dtype=torch.int64)
    return batch


# ---------------------------------------------------------------------------
# the other seeded workloads (both arms)
# ---------------------------------------------------------------------------


def run_single_batch_workload(impl: str, name: str, device, steps: int, warmup: int, graphs: bool = False) -> dict:
    """One packed batch per step on one GPU (cfg1, cfg2, cfg4). `graphs=True`: through each arm's
    own packed CUDA-graph runner, `pack(model, validate=False, cuda_graph=GraphConfig(...))`."""
    pe = load_package()
    from oracle import synthetic as S

    wl = S.workload(name).sorted_by_length()
    model, params, fwd, _ = make_encoder(impl, wl.arch, device)
    batch = to_device(pe.pack_sequences(wl.sequences()), device)
    note = None
    try:
        if graphs:
            if impl == "ours":
                pe.pack(model, validate=False,
                        cuda_graph=pe.GraphConfig(pad_to=1024, max_batch=len(wl.lengths), max_seq=64))
                runner = pe.get_state(model).packed_graph_runner
            else:
                ref_pkg = reference_modules()[0]
                ref_pkg.pack(model, validate=False,
                             cuda_graph=ref_pkg.GraphConfig(pad_to=64, max_batch=len(wl.lengths), max_seq=64))

        def step():
            with torch.no_grad():
                return fwd(batch)

        ms = timed_steps(step, steps, warmup, 1, device)
        if graphs and impl == "ours":
            note = f"{runner.captures} graph captured, {runner.replays} replays"
    finally:
        if graphs:
            (pe if impl == "ours" else reference_modules()[0]).unpack(model)
    out = {"ms_per_step": round(ms, 3), "value": round(wl.total_tokens / ms * 1e3, 1), "unit": UNIT,
           "tokens": wl.total_tokens, "sequences": len(wl.lengths), "steps": steps,
           "workload": workload_text(name) + ("; through the packed CUDA-graph runner" if graphs else "")}
    if note:
        out["graphs"] = note
    del model
    torch.cuda.empty_cache()
    return out


def run_cfg5(impl: str, world: int, rank: int, device, steps: int, warmup: int) -> dict:
    """The mixed index on the 1B-class model: 16,384 sequences / 6.9 M tokens in total (strong
    scaling: the corpus is fixed), cost-balanced over the ranks, each rank encoding its share in
    token-budget micro-batches (the loop of benchmarks/showcases/inference.py:186-209 with the
    budget rule of benchmarks/helpers/packed_training.py:175-202) down to one mean-pooled,
    normalised embedding per sequence, then one NCCL gather of the `[N, H]` embeddings."""
    pe = load_package()
    from flash_modernbert_b200 import shard
    from oracle import synthetic as S

    wl = S.workload("cfg5")
    model, params, _, pooled = make_encoder(impl, wl.arch, device)
    plan = shard.plan_shards(wl.lengths, world, shard.costs_for_model(wl.lengths, model))
    seqs = wl.sequences()
    mine = shard.local_batch(plan, rank, seqs)
    my_lengths = [int(s.numel()) for s in mine]
    micro = pe.token_budget_batches(my_lengths, CFG5_TOKEN_BUDGET)
    batches = [to_device(pe.pack_sequences([mine[i] for i in idx]), device) for idx in micro]
    slots = [torch.tensor(idx, device=device) for idx in micro]
    local = torch.empty(len(mine), model.config.hidden_size, dtype=torch.bfloat16, device=device)

    def step():
        with torch.no_grad():
            for batch, where in zip(batches, slots):
                local[where] = pooled(batch)
        return shard.gather_pooled(local, plan) if world > 1 else local

    out = step()
    torch.cuda.synchronize(device)
    assert bool(torch.isfinite(out.float()).all())
    ms = timed_steps(step, steps, warmup, world, device)
    del model
    torch.cuda.empty_cache()
    return {"ms_per_step": round(ms, 1), "value": round(plan.total_tokens / ms * 1e3, 1), "unit": UNIT,
            "tokens": plan.total_tokens, "sequences": len(wl.lengths), "steps": steps, "scaling": "strong",
            "micro_batches_rank0": len(batches), "token_budget": CFG5_TOKEN_BUDGET,
            "tokens_per_gpu": [int(t) for t in plan.tokens_per_rank],
            "result": "mean-pooled, L2-normalised [N, H] embeddings, NCCL gather of [N, H]",
            "workload": workload_text("cfg5")}


def run_extras(impl: str, world: int, rank: int, device, which: list[str]) -> dict:
    out = {}
    for name in which:
        try:
            if name == "cfg5":
                res = run_cfg5(impl, world, rank, device, steps=2, warmup=1)
            elif world > 1:
                continue  # single-batch workloads are one-GPU measurements
            elif name == "cfg2_graphs":
                res = run_single_batch_workload(impl, "cfg2", device, steps=20, warmup=3, graphs=True)
            elif name == "cfg4":
                res = run_single_batch_workload(impl, name, device, steps=4, warmup=3)
            else:
                res = run_single_batch_workload(impl, name, device, steps=20, warmup=3)
        except Exception as exc:  # noqa: BLE001 - an extra must not take the headline down
            res = {"unavailable": f"{type(exc).__name__}: {str(exc)[:200]}"}
        out[name] = res
    return out


# ---------------------------------------------------------------------------
# arms
# ---------------------------------------------------------------------------


def run_arm(args, impl: str) -> None:
    world, rank, local_rank = dist_setup(args.gpus)
    device = torch.device("cuda", local_rank)
    torch.cuda.set_device(device)
    pe = load_package()  # the reference arm uses only its host-side helpers (collation, shard plan)
    from flash_modernbert_b200 import shard

    arch, lengths, seqs = build_global_batch(args.workload, world)
    why = None
    kind = None
    line_extra = {}
    try:
        model, params, fwd, pooled = make_encoder(impl, arch, device)
        if impl == "reference":
            kind = reference_modules()[2]._load_flash_attn()[2]
        plan = shard.plan_shards(lengths, world, shard.costs_for_model(lengths, model))
        mine = shard.local_batch(plan, rank, seqs)
        batch_host = pe.pack_sequences(mine)
        batch = to_device(batch_host, device)
        hidden = model.config.hidden_size

        # The step. One GPU: ids -> [T, H] last hidden state (the metric's definition). Several
        # GPUs: the same forward with the pooling head, then the gather of the [N, H] embeddings.
        if world == 1:
            def step():
                with torch.no_grad():
                    return fwd(batch)
        elif impl == "ours":
            def step():
                _, emb = pe.packed_forward_pooled(model, params, *batch.forward_args(), pool="mean",
                                                  normalize=True, return_hidden=True)
                return shard.gather_pooled(emb, plan)
        else:
            def step():
                return shard.gather_pooled(torch_mean_pool(fwd(batch), batch.seqlens_dev), plan)

        out = step()
        torch.cuda.synchronize(device)
        if impl == "ours":
            from flash_modernbert_b200 import forward

            forward.get_binding(model, params).check(sync=True)
        assert bool(torch.isfinite(out[:: max(1, out.shape[0] // 4096)].float()).all())
        del out

        with ClockSampler(local_rank) as clocks:
            ms, t0, step_ms = timed_steps(step, args.steps, args.warmup, world, device, per_step=True)
        line_extra["clock_normalised"] = clock_normalised(ms, t0, step_ms, clocks)

        # The gather of the full [T, H] token embeddings (what a token-level consumer such as a
        # ColBERT index needs), on its own stream, overlapping the next step's forward.
        if world > 1:
            gather = OverlappedGather(plan, shard, hidden, device)

            def step_tokens():
                with torch.no_grad():
                    return gather(fwd(batch))

            k = max(3, args.steps // 2)
            ms_tok = timed_steps(step_tokens, k, 3, world, device, drain_fn=gather.drain)
            line_extra["token_gather"] = {
                "value": round(plan.total_tokens / ms_tok * 1e3, 1), "unit": UNIT, "ms_per_step": round(ms_tok, 3),
                "steps": k, "bytes_received_per_rank": int(plan.total_tokens * hidden * 2),
                "what": "packed_forward, then one uneven NCCL all-gather of [T, H] straight into rank-major row "
                        "ranges (no padding, no row permutation) on a side stream overlapping the next step"}
            del gather

        # End to end through the public API from pinned host buffers: H2D of the step's inputs,
        # the forward, D2H of the result.
        e2e = None
        if impl == "ours":
            pinned = [t.pin_memory() for t in (batch_host.input_ids, batch_host.cu_seqlens, batch_host.position_ids)]
            emb_host = torch.empty(len(mine), hidden, dtype=torch.bfloat16).pin_memory()

            def step_e2e():
                ids, cu, pos = (t.to(device, non_blocking=True) for t in pinned)
                emb = pe.packed_forward_pooled(model, params, ids, cu, batch_host.max_seqlen, pos,
                                               pool="mean", normalize=True)
                if world > 1:
                    shard.gather_pooled(emb, plan)
                emb_host.copy_(emb, non_blocking=True)
                torch.cuda.current_stream().synchronize()

            ms_e2e = timed_steps(step_e2e, args.steps, max(3, args.warmup), world, device)
            e2e = {"value": round(plan.total_tokens / ms_e2e * 1e3, 1), "unit": UNIT,
                   "h2d_bytes_per_step": int(sum(t.numel() * t.element_size() for t in pinned)),
                   "d2h_bytes_per_step": int(emb_host.numel() * emb_host.element_size()),
                   "result": "mean-pooled, L2-normalised embedding of every sequence, [N, H] bf16 "
                             "(pooled inside the final LayerNorm)"}

            # The same with the whole [T, H] hidden state brought to the host, double-buffered on a
            # copy stream so that the transfer of step i overlaps the forward of step i + 1.
            if world == 1:
                full_host = [torch.empty(batch.total_tokens, hidden, dtype=torch.bfloat16).pin_memory() for _ in range(2)]
                copy_stream = torch.cuda.Stream()
                state = {"turn": 0}

                def step_full():
                    ids, cu, pos = (t.to(device, non_blocking=True) for t in pinned)
                    hid = pe.packed_forward(model, params, ids, cu, batch_host.max_seqlen, pos)
                    done = torch.cuda.Event()
                    done.record()
                    with torch.cuda.stream(copy_stream):
                        copy_stream.wait_event(done)
                        full_host[state["turn"]].copy_(hid, non_blocking=True)
                        hid.record_stream(copy_stream)
                    state["turn"] ^= 1

                k = max(3, args.steps // 2)
                ms_full = timed_steps(step_full, k, 3, 1, device,
                                      drain_fn=lambda: torch.cuda.current_stream().wait_stream(copy_stream))
                e2e["full_output"] = {
                    "value": round(plan.total_tokens / ms_full * 1e3, 1), "unit": UNIT, "steps": k,
                    "d2h_bytes_per_step": int(batch.total_tokens * hidden * 2),
                    "what": "[T, H] last hidden state copied to pinned host memory on a copy stream, "
                            "overlapping the next step"}
                del full_host
    except Exception as exc:  # noqa: BLE001
        if impl == "ours":
            raise
        why = f"{type(exc).__name__}: {str(exc)[:200]}"

    if world > 1:
        import torch.distributed as dist

        flag = torch.tensor([0 if why is None else 1], device=device)
        dist.all_reduce(flag)
        if int(flag.item()) and why is None:
            why = "another rank could not run the reference's GPU path"

    base = {"metric": METRIC, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "data": DATA}
    if impl == "reference":
        base = {"impl": "reference", **base}

    if why is not None:  # reference arm only: its GPU path did not run
        if world > 1:
            import torch.distributed as dist

            dist.destroy_process_group()
        if rank != 0:
            return
        cpu = cpu_baseline_hf_eager(arch, seqs)
        base.update({
            "value": cpu["value"], "ms_per_step": None, "dtype": "f32", "cpu_baseline": cpu,
            "config": {"workload": workload_text(args.workload)},
            "reference_path": "Hugging Face eager fp32 on the host cores (the reference's own oracle, "
                              f"packed_encoders/validate.py:150-160); its GPU path did not run: {why}",
            "e2e": {"value": cpu["value"], "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        })
        print(json.dumps(base), flush=True)
        return

    total_tokens = plan.total_tokens
    value = round(total_tokens / ms * 1e3, 1)
    parallelism = (f"dp{world}: one replica per GPU, cost-balanced document groups (one plan for both arms); "
                   + ("no collective" if world == 1 else
                      "NCCL gather of the mean-pooled [N, H] embeddings each step; the [T, H] gather is timed under token_gather"))
    base.update({
        "value": value, "ms_per_step": round(ms, 3), "dtype": "bf16",
        "config": {"workload": workload_text(args.workload), "tokens_per_gpu": [int(t) for t in plan.tokens_per_rank],
                   "global_tokens": total_tokens, "sequences": len(lengths), "parallelism": parallelism,
                   "l2": "every step streams > 5 GB of activations through a 126 MB L2; no explicit flush"},
        "clocks": clocks.summary(),
    })
    base.update(line_extra)

    extras = [] if args.no_extras else (["cfg5"] if world > 1 else ["cfg1", "cfg2", "cfg2_graphs", "cfg4", "cfg5"])
    if args.workload != "cfg3":
        extras = []

    if impl == "reference":
        # beside `config`, not inside it: the two arms' `config` objects are identical
        base["reference_path"] = (
            f"packed_encoders.forward.packed_forward on the GPU (flash kind: {kind}; Triton LN/GeGLU, CuteDSL RoPE, "
            "cuBLAS GEMMs), one replica per GPU")
        base["e2e"] = {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}
        del model
        torch.cuda.empty_cache()
        if extras:
            base["workloads"] = run_extras(impl, world, rank, device, extras)
        if world > 1:
            import torch.distributed as dist

            dist.destroy_process_group()
        if rank == 0:
            print(json.dumps(base), flush=True)
        return

    # ---- our arm: roofline, step model, launches ----
    line = base
    line["e2e"] = e2e
    pooled_step = world > 1
    line["gpu_launches"] = launches_per_forward(model, batch_host.max_seqlen, pooled_step) * args.steps
    if rank == 0:
        peaks = measured_peaks()
        work = model_flops(model, [int(s.numel()) for s in mine])
        with ClockSampler(local_rank, period_s=0.005) as gemm_clocks:
            gemm = time_gemm_kernels(model, batch.total_tokens, device, gemm_clocks)
        gemm_ms_layer = sum(v["ms"] for v in gemm.values())
        gemm_flops_layer = sum(v["flops"] for v in gemm.values())
        achieved = gemm_flops_layer / gemm_ms_layer / 1e9
        achieved_sustained = gemm_flops_layer / sum(v["ms_sustained"] for v in gemm.values()) / 1e9
        flops_ms = (work["gemm_flops"] + work["attn_flops"]) / (peaks["bf16_tflops_sustained"] * 1e9)
        ideal_ms = flops_ms + work["tail_bytes"] / (peaks["hbm_gbs"] * 1e6)
        ideal_fused_ms = flops_ms + work["tail_bytes_fused"] / (peaks["hbm_gbs"] * 1e6)
        line["roofline"] = {
            "bound": "tensor", "kernel": "gemm_bf16_tn_kernel (tcgen05; the four launches of one layer: Wqkv+RoPE, Wo+residual, Wi+GeGLU, Wo_mlp+residual)",
            "achieved": round(achieved, 1), "peak": peaks["bf16_tflops"], "unit": "TFLOP/s",
            "frac": round(achieved / peaks["bf16_tflops"], 4),
            "peak_source": f"{peaks['source']} burst (cuBLAS best of 10); achieved = best of 6 bursts of 8 launches per shape",
            "sustained": {"achieved": round(achieved_sustained, 1), "peak": peaks["bf16_tflops_sustained"],
                          "frac": round(achieved_sustained / peaks["bf16_tflops_sustained"], 4),
                          "how": "40 launches back to back per shape, under the power cap, against the sustained cuBLAS peak"},
            "traffic": (round(NCU_GEMM_DRAM_BYTES_PER_TOKEN * batch.total_tokens / 1e9, 3)
                        if arch == "base" else None),
            "traffic_unit": "GB per layer (four launches)",
            "traffic_source": "not measured in this run: one ncu capture on a 71,567-token slice (activations partly "
                              "L2-resident there, so it reads low), scaled by tokens",
            "algorithmic_gb": round(19968 * batch.total_tokens / 1e9, 3),
            "per_shape": {k: {kk: vv for kk, vv in v.items() if kk != "flops"} for k, v in gemm.items()},
        }
        line["step_model"] = {
            "gemm_tflop": round(work["gemm_flops"] / 1e12, 2), "attn_tflop": round(work["attn_flops"] / 1e12, 2),
            "tail_gb_unfused": round(work["tail_bytes"] / 1e9, 1), "tail_gb_this_library": round(work["tail_bytes_fused"] / 1e9, 1),
            "roofline_ms": round(ideal_ms, 2), "frac_of_roofline": round(ideal_ms / ms, 4),
            "roofline_ms_fused_op_list": round(ideal_fused_ms, 2),
            "frac_of_roofline_fused_op_list": round(ideal_fused_ms / ms, 4),
            "peaks": f"{peaks['bf16_tflops_sustained']} TFLOP/s sustained, {peaks['hbm_gbs']} GB/s ({peaks['source']})",
        }
    del model
    torch.cuda.empty_cache()
    if extras:
        line["workloads"] = run_extras(impl, world, rank, device, extras)
    if world > 1:
        import torch.distributed as dist

        dist.destroy_process_group()
    if rank != 0:
        return
    if world == 1 and not args.no_cpu_baseline:
        line["cpu_baseline"] = cpu_baseline_hf_eager(arch, seqs)
    print(json.dumps(line), flush=True)


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", choices=("ours", "reference"), default="ours")
    ap.add_argument("--workload", default="cfg3")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-extras", action="store_true",
                    help="skip the other seeded workloads (cfg1, cfg2 with and without graphs, cfg4, cfg5)")
    ap.add_argument("--gemm-pair", type=int, choices=(0, 1), default=None,
                    help="A/B switch: 0 runs every GEMM on single-CTA 128 x 256 tiles instead of CTA pairs")
    args = ap.parse_args()
    args.warmup = max(3, args.warmup)
    if args.gemm_pair is not None and args.impl == "ours":
        load_package()
        from flash_modernbert_b200 import _lib

        _lib.check(_lib.load().pe_set_option(_lib.OPT_GEMM_PAIR, args.gemm_pair), "pe_set_option")
    run_arm(args, args.impl)


if __name__ == "__main__":
    main()
