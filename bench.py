"""Benchmark of the packed ModernBERT forward: packed tokens/s, ModernBERT-base document
encoding (512 documents, lognormal lengths, 306,851 tokens per GPU), bf16, on N B200s.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload cfg3]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
        --master-port P bench.py --gpus N --steps K --warmup W

One step = one pass of `packed_forward` over this rank's shard of the batch (plus, for
N > 1, the NCCL gather of the output embeddings). Weak scaling: the global batch is N
seeded copies of the workload, split into cost-balanced document groups, one per rank.
Rank 0 prints one JSON line. `--impl reference` times the unmodified reference
(`packed_encoders` installed under baseline/_ref) on the same inputs, falling back to
Hugging Face eager fp32 on the host cores if the reference's GPU path does not run.
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
# from one ncu capture on a 71,567-token slice of the workload (profiles/gemm_tcgen05_cfg3q.md);
# GEMM traffic grows in proportion to the rows, so a full launch is this times its tokens.
NCU_GEMM_DRAM_BYTES_PER_TOKEN = 1256.2e6 / 71567
UNIT = "tokens/s"


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
    """Samples SM clock and throttle reasons of one GPU through NVML while running."""

    REASONS = {
        0x8: "hw_slowdown", 0x40: "hw_thermal_slowdown", 0x20: "sw_thermal_slowdown",
        0x4: "sw_power_cap", 0x80: "hw_power_brake_slowdown",
    }

    def __init__(self, index: int, period_s: float = 0.05):
        self.index, self.period = index, period_s
        self.samples: list[int] = []
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
    minimum tail traffic of the unfused op list, bf16."""
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
    return {"gemm_flops": gemm, "attn_flops": attn, "tail_bytes": tail, "tokens": T}


def launches_per_forward(model) -> int:
    """Kernels of libpe_b200.so that one pe_forward_packed call enqueues."""
    n = 2  # embedding+LN, attention schedule
    for layer in model.layers:
        has_norm = not isinstance(layer.attn_norm, torch.nn.Identity)
        n += (1 if has_norm else 0) + 6  # Wqkv+RoPE, attention, Wo, add+LN, Wi+GeGLU, Wo_mlp
    return n + 1  # final add+LN


def time_gemm_kernels(model, tokens: int, device, reps: int = 5) -> dict:
    """Average duration of each GEMM launch shape of one layer, timed alone with CUDA
    events on the launching stream (each launch streams > 126 MB, so L2 does not hold it)."""
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
    out = {}
    for name, (fn, flops) in shapes.items():
        for _ in range(2):
            fn()
        torch.cuda.synchronize(device)
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        for _ in range(reps):
            fn()
        end.record()
        torch.cuda.synchronize(device)
        ms = start.elapsed_time(end) / reps
        out[name] = {"ms": round(ms, 4), "tflops": round(flops / ms / 1e9, 1), "flops": flops}
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
# arms
# ---------------------------------------------------------------------------


def dist_setup(gpus: int):
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world > 1:
        import torch.distributed as dist

        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        torch.cuda.set_device(local_rank)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    elif gpus > 1:
        raise SystemExit("--gpus N > 1 must be launched with torch.distributed.run (one rank per GPU)")
    return world, rank, local_rank


class OverlappedGather:
    """The end-of-step gather of a multi-GPU run, issued on a stream of its own so that it
    overlaps the next step's forward (the encoder never waits for NVLink). `drain()` makes the
    current stream wait for every gather issued so far; the timed region ends with it, so all
    K gathers lie inside the measurement."""

    def __init__(self, plan, shard_module):
        self.plan, self.shard = plan, shard_module
        self.stream = torch.cuda.Stream()
        self.last = None

    def __call__(self, local_out):
        ready = torch.cuda.Event()
        ready.record()
        with torch.cuda.stream(self.stream):
            self.stream.wait_event(ready)
            self.last = self.shard.gather_embeddings(local_out, self.plan)
            local_out.record_stream(self.stream)
        return self.last

    def drain(self):
        torch.cuda.current_stream().wait_stream(self.stream)


def timed_steps(step_fn, steps: int, warmup: int, world: int, device, drain_fn=None) -> float:
    """Milliseconds per step: K steps between CUDA events, barrier + synchronize on both
    sides, maximum over ranks. `drain_fn` (if any) joins side streams before the end event."""
    import torch.distributed as dist

    for _ in range(warmup):
        step_fn()
    torch.cuda.synchronize(device)
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize(device)
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(steps):
        step_fn()
    if drain_fn is not None:
        drain_fn()
    end.record()
    torch.cuda.synchronize(device)
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize(device)
    ms = torch.tensor([start.elapsed_time(end) / steps], device=device, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    return float(ms.item())


def run_ours(args) -> None:
    world, rank, local_rank = dist_setup(args.gpus)
    device = torch.device("cuda", local_rank)
    torch.cuda.set_device(device)
    pe = load_package()
    from flash_modernbert_b200 import forward, shard
    from oracle import synthetic as S

    arch, lengths, seqs = build_global_batch(args.workload, world)
    model = S.make_model(arch, dtype=torch.bfloat16, device=device)
    params = pe.ModernBertParams.from_hf_config(model.config)
    plan = shard.plan_shards(lengths, world, shard.costs_for_model(lengths, model))
    mine = shard.local_batch(plan, rank, seqs)
    batch_host = pe.pack_sequences(mine)
    batch = batch_host.to(device)
    binding = forward.get_binding(model, params)

    gather = OverlappedGather(plan, shard) if world > 1 else None

    def step():
        out = pe.packed_forward(model, params, *batch.forward_args())
        if gather is not None:
            out = gather(out)
        return out

    out = step()
    torch.cuda.synchronize(device)
    binding.check(sync=True)
    assert bool(torch.isfinite(out[:: max(1, out.shape[0] // 4096)].float()).all())
    del out

    with ClockSampler(local_rank) as clocks:
        ms = timed_steps(step, args.steps, args.warmup, world, device,
                         drain_fn=gather.drain if gather is not None else None)

    # End to end through the public API from pinned host buffers: H2D of the step's inputs,
    # the forward, D2H of the per-sequence first-token embeddings ([N, H], what a
    # CLS-pooled encoder hands back).
    pinned = [t.pin_memory() for t in (batch_host.input_ids, batch_host.cu_seqlens, batch_host.position_ids)]
    first_rows = batch.cu_seqlens[:-1].to(torch.int64)
    result_host = torch.empty(len(mine), params.hidden_size, dtype=torch.bfloat16).pin_memory()

    def step_e2e():
        ids, cu, pos = (t.to(device, non_blocking=True) for t in pinned)
        out = pe.packed_forward(model, params, ids, cu, batch_host.max_seqlen, pos)
        if world > 1:
            out_all = shard.gather_embeddings(out, plan)  # noqa: F841 - part of the job
        result_host.copy_(out.index_select(0, first_rows), non_blocking=True)
        torch.cuda.current_stream().synchronize()

    ms_e2e = timed_steps(step_e2e, args.steps, max(3, args.warmup), world, device)

    if rank != 0:
        import torch.distributed as dist

        dist.destroy_process_group()
        return

    total_tokens = plan.total_tokens
    peaks = measured_peaks()
    work = model_flops(model, [int(s.numel()) for s in mine])
    gemm = time_gemm_kernels(model, batch.total_tokens, device)
    gemm_ms_layer = sum(v["ms"] for v in gemm.values())
    gemm_flops_layer = sum(v["flops"] for v in gemm.values())
    achieved = gemm_flops_layer / gemm_ms_layer / 1e9
    ideal_ms = (work["gemm_flops"] + work["attn_flops"]) / (peaks["bf16_tflops_sustained"] * 1e9) \
        + work["tail_bytes"] / (peaks["hbm_gbs"] * 1e6)
    line = {
        "metric": METRIC, "value": round(total_tokens / ms * 1e3, 1), "unit": UNIT,
        "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(ms, 3),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic (seeded lengths and token ids, random-init weights normal(0, 0.02))",
        "config": {
            "workload": f"{args.workload}: ModernBERT-{arch}, {len(lengths) // world} sequences per GPU "
                        f"(cfg3 = documents, lengths lognormal(median 400, sigma 0.8) clipped to [64, 8192]), "
                        f"packed by cu_seqlens, length-descending",
            "tokens_per_gpu": [int(t) for t in plan.tokens_per_rank],
            "global_tokens": total_tokens, "sequences": len(lengths),
            "parallelism": f"dp{world}: one replica per GPU, cost-balanced document groups, NCCL gather of [T, H] on its own stream, overlapping the next step",
            "l2": "every step streams > 5 GB of activations through a 126 MB L2; no explicit flush",
        },
        "e2e": {
            "value": round(total_tokens / ms_e2e * 1e3, 1), "unit": UNIT,
            "h2d_bytes_per_step": int(sum(t.numel() * t.element_size() for t in pinned)),
            "d2h_bytes_per_step": int(result_host.numel() * result_host.element_size()),
            "result": "first-token embedding of every sequence, [N, H] bf16",
        },
        "gpu_launches": launches_per_forward(model) * args.steps,
        "clocks": clocks.summary(),
        "roofline": {
            "bound": "tensor", "kernel": "gemm_bf16_tn_kernel (tcgen05; the four launches of one layer: Wqkv+RoPE, Wo+residual, Wi+GeGLU, Wo_mlp+residual)",
            "achieved": round(achieved, 1), "peak": peaks["bf16_tflops"], "unit": "TFLOP/s",
            "frac": round(achieved / peaks["bf16_tflops"], 4), "peak_source": f"{peaks['source']} burst",
            "traffic": (round(NCU_GEMM_DRAM_BYTES_PER_TOKEN * batch.total_tokens / 1e9, 3)
                        if arch == "base" else None),
            "traffic_unit": "GB per layer (four launches), ncu on a 71,567-token slice scaled by tokens",
            "algorithmic_gb": round(19968 * batch.total_tokens / 1e9, 3), "per_shape": {k: {"ms": v["ms"], "tflops": v["tflops"]} for k, v in gemm.items()},
        },
        "step_model": {
            "gemm_tflop": round(work["gemm_flops"] / 1e12, 2), "attn_tflop": round(work["attn_flops"] / 1e12, 2),
            "tail_gb": round(work["tail_bytes"] / 1e9, 1), "roofline_ms": round(ideal_ms, 2),
            "frac_of_roofline": round(ideal_ms / ms, 4),
            "peaks": f"{peaks['bf16_tflops_sustained']} TFLOP/s sustained, {peaks['hbm_gbs']} GB/s ({peaks['source']})",
        },
    }
    if world == 1 and not args.no_cpu_baseline:
        line["cpu_baseline"] = cpu_baseline_hf_eager(arch, seqs)
    print(json.dumps(line), flush=True)
    if world > 1:
        import torch.distributed as dist

        dist.destroy_process_group()


def run_reference(args) -> None:
    """The unmodified reference (baseline/_ref) on the same inputs: every rank encodes its
    shard with the reference's GPU packed_forward; torch.distributed gathers. If that path
    cannot run here, rank 0 times Hugging Face eager fp32 on the host cores instead."""
    world, rank, local_rank = dist_setup(args.gpus)
    device = torch.device("cuda", local_rank)
    torch.cuda.set_device(device)
    pe = load_package()  # host-side helpers only (collation, shard plan); no kernel of ours runs
    from flash_modernbert_b200 import shard
    from oracle import synthetic as S

    arch, lengths, seqs = build_global_batch(args.workload, world)
    plan = shard.plan_shards(lengths, world)
    mine = shard.local_batch(plan, rank, seqs)
    batch = pe.pack_sequences(mine, device=device)
    why = None
    ms = None
    kind = None
    try:
        sys.path.insert(0, str(ROOT / "baseline" / "_ref"))
        from packed_encoders import forward as ref_forward
        from packed_encoders import ops as ref_ops
        from packed_encoders.config import ModernBertParams as RefParams

        model = S.make_model(arch, dtype=torch.bfloat16, device=device)
        if not hasattr(model.config, "global_attn_every_n_layers"):
            model.config.global_attn_every_n_layers = 3
        ref_params = RefParams.from_hf_config(model.config)
        kind = ref_ops._load_flash_attn()[2]

        gather = OverlappedGather(plan, shard) if world > 1 else None

        def step():
            with torch.no_grad():
                out = ref_forward.packed_forward(model, ref_params, *batch.forward_args())
            if gather is not None:
                out = gather(out)
            return out

        step()
        torch.cuda.synchronize(device)
        with ClockSampler(local_rank) as clocks:
            ms = timed_steps(step, args.steps, args.warmup, world, device,
                             drain_fn=gather.drain if gather is not None else None)
    except Exception as exc:  # noqa: BLE001
        why = f"{type(exc).__name__}: {str(exc)[:200]}"
    if world > 1:
        import torch.distributed as dist

        flag = torch.tensor([0 if why is None else 1], device=device)
        dist.all_reduce(flag)
        if int(flag.item()) and why is None:
            why = "another rank could not run the reference's GPU path"
        dist.destroy_process_group()
    if rank != 0:
        return
    base = {"impl": "reference", "metric": METRIC, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "data": "synthetic (seeded lengths and token ids, random-init weights normal(0, 0.02))"}
    if why is None:
        value = round(plan.total_tokens / ms * 1e3, 1)
        base.update({
            "value": value, "ms_per_step": round(ms, 3), "dtype": "bf16",
            "config": {"workload": args.workload, "global_tokens": plan.total_tokens,
                       "reference_path": f"packed_encoders.forward.packed_forward on the GPU (flash kind: {kind}; "
                                         "Triton LN/GeGLU, CuteDSL RoPE, cuBLAS GEMMs), one replica per GPU"},
            "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "clocks": clocks.summary(),
        })
    else:
        cpu = cpu_baseline_hf_eager(arch, seqs)
        base.update({
            "value": cpu["value"], "ms_per_step": None, "dtype": "f32", "cpu_baseline": cpu,
            "config": {"workload": args.workload,
                       "reference_path": "Hugging Face eager fp32 on the host cores (the reference's own oracle, "
                                         f"packed_encoders/validate.py:150-160); its GPU path did not run: {why}"},
            "e2e": {"value": cpu["value"], "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        })
    print(json.dumps(base), flush=True)


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", choices=("ours", "reference"), default="ours")
    ap.add_argument("--workload", default="cfg3")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    args = ap.parse_args()
    args.warmup = max(3, args.warmup)
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
