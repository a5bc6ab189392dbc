#!/usr/bin/env python
"""Benchmark of the decoder hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--impl ours|reference]

One step = one decode call (one cooperative megakernel launch) on one batch of synthetic
input: a seeded random-init model of the named shape whose KV cache already holds the stated
number of keys (filled by a seeded prefill of uniform-random token ids).  Prints ONE JSON line.

* ``value``      decode microseconds per generated token with inputs resident in HBM:
                 max-over-ranks device time of K back-to-back launches / (K * batch * N)
* ``e2e``        the same metric through the public API -- ``torch.compile(StatefulDecoder(model),
                 backend=make_backend(mode="decode"))`` captured with ``megabake_b200.graphed`` --
                 with HOST buffers: per step a pinned host->device copy of token and position ids,
                 the graph replay (the megakernel launch and the greedy pick of every row on the
                 device, ``mb_greedy_advance``) and a device->host read of the picked ids,
                 synchronised every step
* ``parity``     one more step of the benched workload, outside every timed region, by the kernel
                 and by the CPU oracle on copies of the same KV cache: max-abs and cosine of the
                 logits, greedy ids, and both forwards' distance from the fp32 forward
* ``device_loop`` the same compiled step with the next token picked on the device
                 (``mb_greedy_advance``) and 8 steps per CUDA graph replay: no host work per token,
                 the picked ids are read once at the end (host wall clock)
* ``roofline``   HBM roofline of the megakernel: algorithmic bytes per launch (weights once +
                 the valid KV rows) / mean launch time, against the measured copy bandwidth
* ``cpu_baseline`` / ``--impl reference``  the CPU port of the reference forward (``oracle/``),
                 timed on this box's host cores on the same workload

Multi-GPU: one process per GPU under torchrun, independent replicas (seed + rank), no collective
on the data path; the only collective is the max-reduction of the timing scalar.
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

# workload name -> (model preset, batch, cached keys)
WORKLOADS = {
    "qwen2-0.5b-b8-k4096": ("qwen2-0.5b", 8, 4096),
    "qwen2-0.5b-b4-k4096": ("qwen2-0.5b", 4, 4096),
    "qwen2-0.5b-b1-k4096": ("qwen2-0.5b", 1, 4096),
    "smollm-135m-b1-k32": ("smollm-135m", 1, 32),
    "llama-3.2-1b-b1-k512": ("llama-3.2-1b", 1, 512),
    "llama-3.2-1b-b1-k8192": ("llama-3.2-1b", 1, 8192),
    "smollm-1.7b-b1-k8192": ("smollm-1.7b", 1, 8192),
    "smollm-1.7b-b8-k8192": ("smollm-1.7b", 8, 8192),
}
# prefill workloads: name -> (model preset, batch, prompt tokens)
PREFILL_WORKLOADS = {
    "gemma-2b-prefill-t128": ("gemma-2b", 1, 128),
    "gemma-2b-prefill-t512": ("gemma-2b", 1, 512),
    "gemma-2b-prefill-t2048": ("gemma-2b", 1, 2048),
    "smollm-135m-prefill-t128": ("smollm-135m", 1, 128),
}
DEFAULT_WORKLOAD = "qwen2-0.5b-b8-k4096"
METRIC = "decode_us_per_token"
UNIT = "us/token"
LOOP_STEPS = 8  # decode steps per CUDA graph in the device-side greedy loop


def measured_tensor_peak() -> tuple[float, str]:
    """Dense bf16 TFLOP/s a library GEMM sustains on this pool's B200s (a prefill step is a
    long run of GEMMs under the power cap, so the sustained figure is the denominator)."""
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        try:
            return float(json.loads(path.read_text())["bf16_tflops_sustained"]), "measured sustained"
        except Exception:
            pass
    return 1590.0, "fallback"


def measured_peaks() -> tuple[float, str]:
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        try:
            return float(json.loads(path.read_text())["hbm_gbs"]), "measured"
        except Exception:
            pass
    return 6650.0, "fallback"


def ncu_traffic(workload: str):
    """DRAM bytes per launch from the committed ncu summary, if one covers this workload."""
    path = ROOT / "profiles" / "dram_traffic.json"
    if path.exists():
        try:
            return json.loads(path.read_text()).get(workload)
        except Exception:
            return None
    return None


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index = index
        self.samples: list[list[str]] = []
        self._stop = threading.Event()
        self._thread = threading.Thread(target=self._run, daemon=True)

    def _run(self):
        while not self._stop.is_set():
            try:
                out = subprocess.run(
                    ["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.FIELDS}",
                     "--format=csv,noheader,nounits"], capture_output=True, text=True, timeout=5)
                if out.returncode == 0 and out.stdout.strip():
                    self.samples.append([c.strip() for c in out.stdout.strip().split(",")])
            except Exception:
                pass
            self._stop.wait(0.1)

    def __enter__(self):
        self._thread.start()
        return self

    def __exit__(self, *exc):
        self._stop.set()
        self._thread.join(timeout=6)

    def summary(self) -> dict:
        clocks = [float(s[0]) for s in self.samples if s and s[0].replace(".", "").isdigit()]
        reasons = set()
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        for sample in self.samples:
            for name, flag in zip(names, sample[2:6]):
                if flag.lower().startswith("active"):
                    reasons.add(name)
        return {
            "sm_mhz": statistics.median(clocks) if clocks else None,
            "sm_max_mhz": float(self.samples[0][1]) if self.samples else None,
            "reasons": sorted(reasons),
            "samples": len(self.samples),
        }


def build_workload(name: str, rank: int, extra_steps: int, device, cache_fill: str = "prefill"):
    import torch

    from megabake_b200 import models

    preset, batch, keys = WORKLOADS[name]
    spec = models.get_spec(preset)
    capacity = keys + extra_steps + 1
    weights = models.init_weights(spec, seed=rank, device=device, on_device=True)
    inv_freq = models.inv_freq_buffer(spec, device)
    state = models.make_state(spec, batch, capacity, device)
    if keys > 0 and cache_fill == "prefill":
        models.fill_cache_by_prefill(spec, weights, inv_freq, state, keys, seed=100 + rank)
    elif keys > 0:
        # profiling runs: seeded random rows instead of thousands of library launches
        gen = torch.Generator(device=device).manual_seed(100 + rank)
        for index in range(spec.layers):
            for t in state[3 * index: 3 * index + 2]:
                t[:, :keys].normal_(0.0, 1.0, generator=gen)
            state[3 * index + 2].fill_(keys)
    return spec, batch, keys, capacity, weights, inv_freq, state


def max_over_ranks(values, device, distributed: bool) -> list[float]:
    """Element-wise maximum of per-rank scalars (the timing rule for multi-GPU runs: the job is
    as slow as its slowest replica).  Works on any initialised process group: NCCL with a CUDA
    device here, gloo with ``"cpu"`` in the CPU tests."""
    import torch

    tensor = torch.tensor(list(values), dtype=torch.float64, device=device)
    if distributed:
        import torch.distributed as dist
        dist.all_reduce(tensor, op=dist.ReduceOp.MAX)
    return [float(x) for x in tensor.cpu()]


def whole_job_rate(units_per_rank: float, world: int, seconds: float) -> float:
    """Throughput of the whole job: every rank processed ``units_per_rank`` in ``seconds``
    (the max over ranks) -- weak scaling, no unit is shared between replicas."""
    return units_per_rank * world / seconds


def decode_config(workload: str, world: int, cache_fill: str) -> dict:
    """The workload description both arms print (the same keys and values, so that the two lines
    can be compared field by field); what is particular to an arm goes elsewhere in its line."""
    from megabake_b200 import models

    preset, batch, keys = WORKLOADS[workload]
    spec = models.get_spec(preset)
    bytes_per_step = (models.direct_program(spec, batch, keys + 1).weight_bytes()
                      + batch * keys * models.direct_program(spec, batch, keys + 1).kv_bytes_per_key())
    return {
        "workload": workload, "model": spec.name, "batch_per_gpu": batch, "cached_keys": keys,
        "replicas": world, "parallelism": f"dp{world} replicas",
        "weights": "seeded N(0,0.02) random init, tied embeddings", "cache_fill": cache_fill,
        "l2": f"inputs larger than L2: weights + KV read per step {bytes_per_step / 1e6:.0f} MB "
              "vs 126 MB L2",
    }


def prefill_config(workload: str, world: int) -> dict:
    from megabake_b200 import models

    preset, batch, tokens = PREFILL_WORKLOADS[workload]
    spec = models.get_spec(preset)
    gemm_flops, _ = prefill_flops(spec, tokens)
    return {
        "workload": workload, "model": spec.name, "batch_per_gpu": batch, "prompt_tokens": tokens,
        "replicas": world, "parallelism": f"dp{world} replicas",
        "weights": "seeded N(0,0.02) random init, tied embeddings",
        "l2": f"inputs larger than L2: {gemm_flops / (2 * tokens) * 2 / 1e6:.0f} MB of weights read "
              "per step vs 126 MB L2",
    }


def algorithmic_bytes(spec, program, batch: int, mean_keys: float) -> float:
    return program.weight_bytes() + batch * mean_keys * program.kv_bytes_per_key()


def parity_check(spec, weights, inv_freq, state, ids, position, decoder, ids_dev, pos_dev,
                 logits) -> dict:
    """One decode step by the kernel against the CPU oracle on copies of the same state."""
    import torch

    from oracle import decoder_oracle as oracle
    from oracle.adapters import oracle_config, oracle_weights

    torch.set_num_threads(os.cpu_count() or 1)
    cpu_weights = {k: v.cpu() for k, v in weights.items()}
    cfg = oracle_config(spec)
    ref_state = [t.cpu() for t in state]
    wide_state = [t.float() if t.dtype == torch.bfloat16 else t.clone() for t in ref_state]
    pos = torch.full((ids.shape[0], 1), position, dtype=torch.int64)
    with torch.no_grad():
        reference = oracle.decode_step(cfg, oracle_weights(cpu_weights, inv_freq.cpu()), ids, pos,
                                       ref_state)
        wide = oracle.decode_step(cfg, oracle_weights({k: v.float() for k, v in cpu_weights.items()},
                                                      inv_freq.cpu().float()), ids, pos, wide_state)
    decoder.launch_into(ids_dev, pos_dev, logits)
    decoder.check()
    got = logits.float().cpu()
    ref = reference.float()

    def cos(a, b):
        a, b = a.double().flatten(), b.double().flatten()
        return float(a @ b / (a.norm() * b.norm()))

    return {
        "max_abs": float((got - ref).abs().max()), "cosine": cos(got, ref),
        "greedy_ids_equal": bool(torch.equal(got[:, -1].argmax(-1), ref[:, -1].argmax(-1))),
        "kernel_vs_fp32_max_abs": float((got - wide).abs().max()),
        "eager_vs_fp32_max_abs": float((ref - wide).abs().max()),
        "kernel_vs_fp32_cosine": cos(got, wide), "eager_vs_fp32_cosine": cos(ref, wide),
        "against": "CPU oracle (the reference's eager bf16 forward) and the same forward in fp32, "
                   "one step on the benched weights and KV cache",
    }


def cpu_reference_run(name: str, steps: int, warmup: int, time_limit_s: float, rank: int = 0) -> dict:
    """Time the CPU port of the reference forward on this box's host cores."""
    import torch

    from megabake_b200 import models
    from oracle import decoder_oracle as oracle
    from oracle.adapters import oracle_config, oracle_weights

    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    preset, batch, keys = WORKLOADS[name]
    spec = models.get_spec(preset)
    capacity = keys + steps + warmup + 1
    weights = models.init_weights(spec, seed=rank)
    inv_freq = models.inv_freq_buffer(spec)
    state = models.make_state(spec, batch, capacity)
    if keys > 0:
        # same protocol as the GPU arm; on CPU the fill is the slow part, so use seeded random
        # K/V rows of the prefill's magnitude when the context is long (timing is unaffected)
        if keys <= 512:
            models.fill_cache_by_prefill(spec, weights, inv_freq, state, keys, seed=100 + rank)
        else:
            gen = torch.Generator().manual_seed(100 + rank)
            for index in range(spec.layers):
                for t in state[3 * index: 3 * index + 2]:
                    t[:, :keys] = torch.randn(t[:, :keys].shape, generator=gen).to(t.dtype)
                state[3 * index + 2].fill_(keys)
    cfg, ow = oracle_config(spec), oracle_weights(weights, inv_freq)
    ids = torch.randint(0, spec.vocab, (batch, 1), generator=torch.Generator().manual_seed(7))
    times = []
    started = time.perf_counter()
    with torch.no_grad():
        for call in range(warmup + steps):
            pos = torch.full((batch, 1), keys + call, dtype=torch.int64)
            t0 = time.perf_counter()
            oracle.decode_step(cfg, ow, ids, pos, state)
            dt = time.perf_counter() - t0
            if call >= warmup:
                times.append(dt)
            if time.perf_counter() - started > time_limit_s and len(times) >= 2:
                break
    per_step = statistics.median(times)
    return {
        "value": per_step * 1e6 / batch, "unit": UNIT, "cores": cores, "kind": "port",
        "sample": f"{len(times)} decode steps of {name} (median), CPU port of the reference "
                  f"eager forward, {cores} threads",
        "ms_per_step": per_step * 1e3, "steps": len(times),
    }


def prefill_flops(spec, tokens: int) -> tuple[float, float]:
    """(GEMM flops, attention flops) of one causal prefill of ``tokens`` positions, batch 1:
    every projection and the LM head at every position; attention as 4 * T^2 * Hq * D * L."""
    q_dim, kv_dim = spec.heads * spec.head_dim, spec.kv_heads * spec.head_dim
    per_layer = (q_dim * spec.hidden + 2 * kv_dim * spec.hidden + spec.hidden * q_dim
                 + 3 * spec.hidden * spec.intermediate)
    params = spec.layers * per_layer + spec.vocab * spec.hidden
    return 2.0 * params * tokens, 4.0 * tokens * tokens * q_dim * spec.layers


def cpu_prefill_run(name: str, steps: int, time_limit_s: float) -> dict:
    """Time the CPU port of the reference prefill forward on this box's host cores."""
    import torch

    from megabake_b200 import models
    from oracle import decoder_oracle as oracle
    from oracle.adapters import oracle_config, oracle_weights

    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    preset, batch, tokens = PREFILL_WORKLOADS[name]
    spec = models.get_spec(preset)
    weights = models.init_weights(spec, seed=0)
    cfg, ow = oracle_config(spec), oracle_weights(weights, models.inv_freq_buffer(spec))
    ids = torch.randint(0, spec.vocab, (batch, tokens), generator=torch.Generator().manual_seed(7))
    times = []
    started = time.perf_counter()
    with torch.no_grad():
        for _ in range(max(steps, 1)):
            t0 = time.perf_counter()
            oracle.prefill(cfg, ow, ids)
            times.append(time.perf_counter() - t0)
            if time.perf_counter() - started > time_limit_s:
                break
    per_step = statistics.median(times)
    return {
        "value": batch * tokens / per_step, "unit": "tok/s", "cores": cores, "kind": "port",
        "sample": f"{len(times)} prefill(s) of {name} (median), CPU port of the reference eager "
                  f"forward, {cores} threads",
        "ms_per_step": per_step * 1e3, "steps": len(times),
    }


def run_prefill(args) -> None:
    import torch

    from megabake_b200 import models
    from megabake_b200.engine import BoundDecoder
    from megabake_b200.planner import plan_prefill

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: there is no CPU execution path "
                         "(use --impl reference for the CPU baseline)")
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    distributed = world > 1
    if distributed:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=device)
    steps, warmup = args.steps, max(args.warmup, 3)
    preset, batch, tokens = PREFILL_WORKLOADS[args.workload]
    spec = models.get_spec(preset)
    weights = models.init_weights(spec, seed=rank, device=device)
    inv_freq = models.inv_freq_buffer(spec, device)
    layout = plan_prefill(models.direct_prefill_program(spec, batch, tokens))
    host_ids = torch.randint(0, spec.vocab, (batch, tokens),
                             generator=torch.Generator().manual_seed(7 + rank)).pin_memory()
    ids = host_ids.to(device)
    call_args = models.direct_prefill_arguments(spec, weights, inv_freq, ids)
    bound = BoundDecoder(layout, call_args)
    logits = torch.empty(batch, tokens, spec.vocab, dtype=torch.bfloat16, device=device)
    positions = bound._positions

    def barrier():
        if distributed:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(warmup):
        bound.launch_into(ids, positions, logits)
    bound.check()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with ClockSampler(local_rank) as sampler:
        barrier()
        start.record()
        for _ in range(steps):
            bound.launch_into(ids, positions, logits)
        stop.record()
        barrier()
    bound.check()
    device_ms = start.elapsed_time(stop)
    launches = bound.plan.launches   # kernel launches one prefill enqueues, as the library reports it

    # End to end through the public API: torch.compile(PrefillLogits(model),
    # backend=make_backend(mode="prefill")) captured once with megabake_b200.graphed.  Per step:
    # pinned host ids -> device, graph replay (every kernel of the prefill plan), greedy pick of
    # the last position on the device, device -> host read of it, synchronised every step.
    e2e_s = None
    if not args.skip_e2e:
        from megabake_b200 import PrefillLogits, graphed, make_backend

        bound.close()
        del bound, logits
        model = models.build_hf_model(spec, device=device, weights=weights)
        del weights, call_args
        torch.cuda.empty_cache()
        backend = make_backend(mode="prefill")
        step_fn = torch.compile(PrefillLogits(model).eval(), backend=backend, fullgraph=True,
                                dynamic=False)
        with torch.no_grad():
            graph_call = graphed(step_fn, ids)
        compiled = backend.megabake_last_callable
        host_pick = torch.zeros(batch, dtype=torch.int64).pin_memory()

        def e2e_step():
            ids.copy_(host_ids, non_blocking=True)
            out = graph_call(ids)
            host_pick.copy_(out[:, -1].argmax(-1), non_blocking=True)
            torch.cuda.synchronize()

        for _ in range(warmup):
            e2e_step()
        barrier()
        t0 = time.perf_counter()
        for _ in range(steps):
            e2e_step()
        barrier()
        e2e_s = time.perf_counter() - t0
        compiled.check()

    device_ms, e2e_ms = max_over_ranks([device_ms, (e2e_s or 0.0) * 1e3], device, distributed)
    if rank == 0:
        peak, peak_kind = measured_tensor_peak()
        ms_per_step = device_ms / steps
        gemm_flops, attn_flops = prefill_flops(spec, tokens)
        gemm_flops *= batch
        attn_flops *= batch
        achieved = gemm_flops / (ms_per_step * 1e-3) / 1e12
        line = {
            "metric": "prefill_tokens_per_s",
            "value": whole_job_rate(batch * tokens, world, ms_per_step * 1e-3),
            "unit": "tok/s", "n_gpus": world, "steps": steps, "warmup": warmup,
            "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": prefill_config(args.workload, world),
            "plan": {"kernel_launches_per_step": launches,
                     "attention_tflop_per_step": attn_flops / 1e12},
            "roofline": {
                "bound": "tensor", "achieved": achieved, "peak": peak, "unit": "TFLOP/s",
                "frac": achieved / peak, "traffic": None,
                "peak_source": f"{peak_kind} cuBLAS bf16 GEMM",
                "algorithmic_flops_per_step": gemm_flops,
                "note": "GEMM flops of the whole step (projections + LM head at every position) "
                        "over the whole step time, attention and row kernels included in the time",
            },
            "e2e": None if e2e_s is None else {
                "value": batch * tokens * world / (e2e_ms * 1e-3 / steps), "unit": "tok/s",
                "h2d_bytes_per_step": batch * tokens * 8, "d2h_bytes_per_step": batch * 8,
                "ms_per_step": e2e_ms / steps,
                "path": "torch.compile(PrefillLogits, backend=make_backend(mode='prefill')) under "
                        "megabake_b200.graphed + torch argmax of the last position, synchronised "
                        "every step",
            },
            "gpu_launches": steps * launches,
            "clocks": sampler.summary(),
        }
        if world == 1 and not args.no_cpu_baseline:
            base = cpu_prefill_run(args.workload, 3, time_limit_s=25.0)
            line["cpu_baseline"] = {k: base[k] for k in ("value", "unit", "cores", "kind", "sample")}
        emit(line)
    if distributed:
        dist.barrier()
        dist.destroy_process_group()


def run_reference(args) -> None:
    """The reference's own CPU implementation of the path -- its eager forward, restated in
    ``oracle/`` and pinned bit for bit to fixtures the reference produced -- on this box's host
    cores, on the same workload, metric and unit as the GPU arm.  Its compiled sm100 kernels need
    torch 2.14 and CuTe-DSL 4.8, neither of which exists on the box, so no GPU number of the
    reference can be measured here."""
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if rank != 0:
        return
    steps, warmup = args.steps, max(args.warmup, 3)
    if args.workload in PREFILL_WORKLOADS:
        result = cpu_prefill_run(args.workload, steps, time_limit_s=120.0)
        emit({
            "impl": "reference", "metric": "prefill_tokens_per_s", "value": result["value"],
            "unit": "tok/s", "n_gpus": args.gpus, "steps": steps, "warmup": warmup,
            "steps_timed": result["steps"],
            "ms_per_step": result["ms_per_step"], "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": prefill_config(args.workload, world),
            "cpu_baseline": {k: result[k] for k in ("value", "unit", "cores", "kind", "sample")},
            "e2e": {"value": result["value"], "unit": "tok/s", "h2d_bytes_per_step": 0,
                    "d2h_bytes_per_step": 0},
            "gpu_launches": 0, "device": "host cpu",
        })
        return
    result = cpu_reference_run(args.workload, steps, warmup, time_limit_s=120.0)
    line = {
        "impl": "reference", "metric": METRIC, "value": result["value"], "unit": UNIT,
        "n_gpus": args.gpus, "steps": steps, "warmup": warmup, "steps_timed": result["steps"],
        "ms_per_step": result["ms_per_step"], "higher_is_better": False, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": decode_config(args.workload, world, args.cache_fill),
        "cpu_baseline": {k: result[k] for k in ("value", "unit", "cores", "kind", "sample")},
        "e2e": {"value": result["value"], "unit": UNIT, "h2d_bytes_per_step": 0,
                "d2h_bytes_per_step": 0},
        "gpu_launches": 0, "device": "host cpu",
    }
    emit(line)


def run_ours(args) -> None:
    import torch

    from megabake_b200 import models
    from megabake_b200.engine import BoundDecoder
    from megabake_b200.planner import plan_decode

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: there is no CPU execution path "
                         "(use --impl reference for the CPU baseline)")
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    distributed = world > 1
    if distributed:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=device)

    steps, warmup = args.steps, max(args.warmup, 3)
    total_calls = 3 * (steps + warmup) + 97  # three timed loops, graph warm-ups, the parity step
    spec, batch, keys, capacity, weights, inv_freq, state = build_workload(
        args.workload, rank, total_calls, device, args.cache_fill)
    program = models.direct_program(spec, batch, capacity)
    layout = plan_decode(program)
    ids = torch.randint(0, spec.vocab, (batch, 1), generator=torch.Generator().manual_seed(7 + rank))
    ids_dev = ids.to(device)
    pos_all = (torch.arange(total_calls, dtype=torch.int64)[:, None, None] + keys).expand(
        total_calls, batch, 1).contiguous().to(device)
    call_args = models.direct_arguments(spec, weights, inv_freq, ids_dev, pos_all[0], state)
    decoder = BoundDecoder(layout, call_args)
    logits = torch.empty(batch, 1, spec.vocab, dtype=torch.bfloat16, device=device)

    def barrier():
        if distributed:
            dist.barrier()
        torch.cuda.synchronize()

    # ---- resident-input timing -----------------------------------------------------------
    call = 0
    for _ in range(warmup):
        decoder.launch_into(ids_dev, pos_all[call], logits)
        call += 1
    decoder.check()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    first_key = keys + call
    with ClockSampler(local_rank) as sampler:
        barrier()
        start.record()
        for _ in range(steps):
            decoder.launch_into(ids_dev, pos_all[call], logits)
            call += 1
        stop.record()
        barrier()
    decoder.check()
    device_ms = start.elapsed_time(stop)
    mean_keys = first_key + (steps - 1) / 2 + 1

    # ---- parity of the benched workload (outside every timed region) ---------------------------
    # One more step of this very workload -- same weights, same KV cache as it stands now -- by
    # the kernel and by the CPU oracle (and by the oracle in fp32, the yardstick of the
    # reference's own long-context test): rank 0 only, skipped when the host copy would be huge.
    parity = None
    state_bytes = sum(t.numel() * t.element_size() for t in state)
    if rank == 0 and not args.no_parity and state_bytes <= 6 << 30:
        parity = parity_check(spec, weights, inv_freq, state, ids, keys + call, decoder, ids_dev,
                              pos_all[call], logits)
        call += 1
    elif rank == 0:
        parity = {"skipped": "--no-parity" if args.no_parity else
                  f"KV state of {state_bytes / 2**30:.1f} GiB: covered by tests/test_gpu_config_parity.py"}

    # ---- end-to-end timing through the public API -------------------------------------------
    # torch.compile(wrapper, backend=make_backend(mode="decode")) captured once in a CUDA graph
    # with megabake_b200.graphed (the reference's own recipe for steady-state decode).  Per
    # step: pinned host -> device copy of token and position ids, graph replay (one megakernel
    # launch), device argmax, device -> host read of the picked ids, synchronised every step.
    from megabake_b200 import StatefulDecoder, graphed, make_backend

    if args.skip_e2e:
        return _report(args, spec, program, layout, batch, keys, steps, warmup, device_ms, None,
                       mean_keys, {"ctas": decoder.plan.ctas, "ring_stages": decoder.plan.stages},
                       sampler, rank, world, distributed, device, parity=parity)
    plan_info = {"ctas": decoder.plan.ctas, "ring_stages": decoder.plan.stages}
    decoder.close()
    del decoder
    model = models.build_hf_model(spec, device=device, weights=weights)
    del weights, call_args
    torch.cuda.empty_cache()
    wrapper = StatefulDecoder(model, capacity).eval()
    backend = make_backend(mode="decode")
    step_fn = torch.compile(wrapper, backend=backend, fullgraph=True, dynamic=False)
    host_ids = ids.clone().pin_memory()
    host_pos = torch.zeros(batch, 1, dtype=torch.int64).pin_memory()
    host_pick = torch.zeros(batch, dtype=torch.int64).pin_memory()
    dev_ids = torch.empty_like(ids_dev)
    dev_pos = torch.full((batch, 1), keys + call, dtype=torch.int64, device=device)
    dev_ids.copy_(ids_dev)
    from megabake_b200 import runtime as rt

    dev_pick = torch.zeros(batch, 1, dtype=torch.int64, device=device)

    def step_and_pick(token, position, *kv_state):
        # the compiled step, then the greedy pick of every row on the device (mb_greedy_advance):
        # two launches in one CUDA graph
        rt.greedy_advance(step_fn(token, position, *kv_state), dev_pick)
        return dev_pick

    with torch.no_grad():
        graph_call = graphed(step_and_pick, dev_ids, dev_pos, *state)
    compiled_decoder = backend.megabake_last_callable

    def e2e_step(index: int):
        host_pos.fill_(keys + index)
        dev_ids.copy_(host_ids, non_blocking=True)
        dev_pos.copy_(host_pos, non_blocking=True)
        picked = graph_call(dev_ids, dev_pos, *state)
        host_pick.copy_(picked[:, 0], non_blocking=True)
        torch.cuda.synchronize()

    for _ in range(warmup):
        e2e_step(call)
        call += 1
    barrier()
    t0 = time.perf_counter()
    for _ in range(steps):
        e2e_step(call)
        call += 1
    barrier()
    e2e_s = time.perf_counter() - t0
    compiled_decoder.check()

    # ---- multi-step loop with the pick on the device ------------------------------------------
    # The same compiled step, but the next token is picked by mb_greedy_advance on the device and
    # LOOP_STEPS x (decode launch, pick) are captured in one CUDA graph: the host only replays
    # graphs and reads all picked ids once at the end.
    per_graph = LOOP_STEPS
    replays = max(1, steps // per_graph)
    picked = torch.zeros(batch, (replays + 4) * per_graph, dtype=torch.int64, device=device)
    cursor = torch.zeros(batch, dtype=torch.int32, device=device)
    dev_pos.fill_(keys + call)

    def device_loop(token, position, *kv_state):
        for _ in range(per_graph):
            out = step_fn(token, position, *kv_state)
            rt.greedy_advance(out, token, position, picked, cursor)
        return picked

    with torch.no_grad():
        loop_call = graphed(device_loop, dev_ids, dev_pos, *state)
    cursor.zero_()
    loop_call(dev_ids, dev_pos, *state)  # one untimed replay
    barrier()
    t0 = time.perf_counter()
    for _ in range(replays):
        loop_call(dev_ids, dev_pos, *state)
    host_picks = picked.cpu()  # the one device -> host read (synchronises)
    barrier()
    loop_s = time.perf_counter() - t0
    compiled_decoder.check()
    assert int(cursor.min()) == (replays + 1) * per_graph and int(host_picks.max()) < spec.vocab
    loop = {"seconds": loop_s, "steps": replays * per_graph, "per_graph": per_graph,
            "d2h_bytes": host_picks.numel() * 8}

    return _report(args, spec, program, layout, batch, keys, steps, warmup, device_ms, e2e_s,
                   mean_keys, plan_info, sampler, rank, world, distributed, device, loop, parity)


def _report(args, spec, program, layout, batch, keys, steps, warmup, device_ms, e2e_s, mean_keys,
            plan_info, sampler, rank, world, distributed, device, loop=None, parity=None) -> None:
    import torch

    device_ms, e2e_ms, loop_ms = max_over_ranks(
        [device_ms, (e2e_s or 0.0) * 1e3, (loop["seconds"] if loop else 0.0) * 1e3], device,
        distributed)

    if rank == 0:
        peak, peak_kind = measured_peaks()
        ms_per_step = device_ms / steps
        bytes_per_launch = algorithmic_bytes(spec, program, batch, mean_keys)
        achieved = bytes_per_launch / (ms_per_step * 1e-3) / 1e9
        line = {
            "metric": METRIC, "value": ms_per_step * 1e3 / (batch * world), "unit": UNIT,
            "n_gpus": world, "steps": steps, "warmup": warmup, "ms_per_step": ms_per_step,
            "higher_is_better": False, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
            "data": "synthetic",
            "config": decode_config(args.workload, world, args.cache_fill),
            "plan": {"tokens_per_s": whole_job_rate(batch, world, ms_per_step * 1e-3),
                     "phases": len(layout.phases), "grid_barriers": layout.intervals,
                     "ctas": plan_info["ctas"], "ring_stages": plan_info["ring_stages"]},
            "roofline": {
                "bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s",
                "frac": achieved / peak, "traffic": ncu_traffic(args.workload),
                "peak_source": f"{peak_kind} copy bandwidth",
                "algorithmic_bytes_per_launch": bytes_per_launch,
            },
            "e2e": None if e2e_s is None else {
                "value": e2e_ms * 1e3 / steps / (batch * world), "unit": UNIT,
                "h2d_bytes_per_step": 2 * batch * 8, "d2h_bytes_per_step": batch * 8,
                "ms_per_step": e2e_ms / steps,
                "path": "torch.compile(StatefulDecoder, backend=make_backend(mode='decode')) + the "
                        "on-device greedy pick under megabake_b200.graphed; pinned host ids in, "
                        "picked ids out, synchronised every step",
            },
            "gpu_launches": steps,  # one decode_kernel per step in the timed resident loop
            "clocks": sampler.summary(),
        }
        line["parity"] = parity
        if loop is not None:
            line["device_loop"] = {
                "value": loop_ms * 1e3 / loop["steps"] / (batch * world), "unit": UNIT,
                "ms_per_step": loop_ms / loop["steps"], "steps": loop["steps"],
                "steps_per_graph": loop["per_graph"], "launches_per_step": 2,
                "h2d_bytes_per_step": 0, "d2h_bytes_total": loop["d2h_bytes"],
                "path": "the same compiled step + mb_greedy_advance (pick on the device), "
                        f"{loop['per_graph']} steps per CUDA graph replay, host wall clock, picked "
                        "ids read once at the end",
            }
        if world == 1 and not args.no_cpu_baseline:
            base = cpu_reference_run(args.workload, 8, 1, time_limit_s=25.0)
            line["cpu_baseline"] = {k: base[k] for k in ("value", "unit", "cores", "kind", "sample")}
        emit(line)
    if distributed:
        import torch.distributed as dist
        dist.barrier()
        dist.destroy_process_group()


_RESULT_STREAM = None


def emit(line: dict) -> None:
    """The one JSON line of the run, on the process's original stdout."""
    stream = _RESULT_STREAM or sys.stdout
    stream.write(json.dumps(line) + "\n")
    stream.flush()


def main() -> None:
    # Libraries print banners on stdout (NCCL's version line under torchrun): keep the original
    # stdout for the result line alone and send everything else to stderr.
    global _RESULT_STREAM
    sys.stdout.flush()
    _RESULT_STREAM = os.fdopen(os.dup(1), "w")
    os.dup2(2, 1)
    parser = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=200)
    parser.add_argument("--warmup", type=int, default=10)
    parser.add_argument("--workload", default=DEFAULT_WORKLOAD,
                        choices=sorted(WORKLOADS) + sorted(PREFILL_WORKLOADS))
    parser.add_argument("--impl", default="ours", choices=["ours", "reference"])
    parser.add_argument("--no-cpu-baseline", action="store_true")
    parser.add_argument("--no-parity", action="store_true",
                        help="skip the one-step comparison with the CPU oracle")
    parser.add_argument("--skip-e2e", action="store_true",
                        help="profiler runs: only the resident-input loop (e2e is reported null)")
    parser.add_argument("--cache-fill", default="prefill", choices=["prefill", "random"],
                        help="how the KV cache gets its cached keys (random: for profiler runs)")
    args = parser.parse_args()
    if args.impl == "reference":
        run_reference(args)
    elif args.workload in PREFILL_WORKLOADS:
        run_prefill(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
