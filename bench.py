"""Decode and prefill throughput of GPT-2 (random weights, synthetic tokens) on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference] [--points all|small] [--profile]

A step is one decode step of a batch of 8 sequences of GPT-2 small.  The run prints one JSON line: `value` is decoded
tokens per second, timed on the device with CUDA events over exactly K steps; `e2e` is the same through the public
generate entry point with host tokens in and out; `prefill`, `roofline` and `points` explain it.  `points` holds the
other workloads (GPT-2 small at batch 1 and 64, GPT-2 medium with 8 prompts of unequal lengths, GPT-2 XL at batch 64
with its cache for 64 x 1,024 positions resident), each measured as 10 repetitions after 3 unmeasured ones, the cache
state made anew for every repetition, with median, 95th percentile, minimum and maximum and a roofline fraction.
`--profile` prints, instead, where a prefill and a decode step spend their time, kernel by kernel.
"""
from __future__ import annotations

import argparse
import json
import statistics
import subprocess
import sys
import tempfile
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}
CONTEXT = 1024
PREFILL_TOKENS = 2048
REPETITIONS, WARM_REPETITIONS = 10, 3


def peaks():
    path = ROOT / "MEASURED_PEAKS.json"
    if path.is_file():
        try:
            data = json.loads(path.read_text())
            return {"hbm_gbs": float(data["hbm_gbs"]), "bf16_tflops": float(data["bf16_tflops"]),
                    "bf16_tflops_sustained": float(data.get("bf16_tflops_sustained", data["bf16_tflops"])),
                    "source": "measured"}
        except (KeyError, ValueError, json.JSONDecodeError):
            pass
    return dict(FALLBACK_PEAKS, bf16_tflops_sustained=1400.0, source="fallback")


class ClockSampler:
    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.file = tempfile.NamedTemporaryFile("w+", suffix=".csv", delete=False)
        self.proc = None

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", "0", f"--query-gpu={self.FIELDS}",
                                          "--format=csv,noheader,nounits", "-lms", "20"], stdout=self.file,
                                         stderr=subprocess.DEVNULL)
        except OSError:
            self.proc = None
        return self

    def __exit__(self, *exc):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()

    def summary(self):
        self.file.flush()
        rows = [line.split(", ") for line in Path(self.file.name).read_text().splitlines() if line.strip()]
        rows = [r for r in rows if len(r) >= 8]
        if not rows:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi gave no samples"]}
        sm = [float(r[0]) for r in rows if r[0].replace(".", "").isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(r[4 + i].strip().lower() == "active" for r in rows)]
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": float(rows[0][1]), "reasons": reasons,
                "samples": len(rows)}


def gpt2(size: str) -> dict:
    sizes = {"small": (12, 768, 12), "medium": (24, 1024, 16), "xl": (48, 1600, 25)}
    n_layer, n_embd, n_head = sizes[size]
    return dict(model_type="gpt2", n_layer=n_layer, n_embd=n_embd, n_head=n_head, n_inner=4 * n_embd, vocab_size=50257,
                n_positions=1024, layer_norm_epsilon=1e-5, activation_function="gelu_new")


def weight_bytes(cfg, elem=2):
    d, m, L, V, P = cfg["n_embd"], cfg["n_inner"], cfg["n_layer"], cfg["vocab_size"], cfg["n_positions"]
    per_layer = (d * 3 * d + d * d + 2 * d * m) * elem + (3 * d + d + m + d + 4 * d) * 4
    return L * per_layer + V * d * elem + 2 * d * 4          # layers + tied readout table + final norm


def kv_bytes_per_token(cfg, elem=2):
    return 2 * cfg["n_layer"] * cfg["n_embd"] * elem


def prefill_flops(cfg, lengths):
    d, m, L, V = cfg["n_embd"], cfg["n_inner"], cfg["n_layer"], cfg["vocab_size"]
    tokens = sum(lengths)
    gemm = 2 * tokens * L * (d * 3 * d + d * d + 2 * d * m)
    attention = sum(L * 2 * s * s * d for s in lengths)          # QK^T and PV over the causal half
    return gemm + attention + 2 * len(lengths) * d * V


def make_engine(cfg, bt, torch, *, max_tokens, max_slots, fast_weights=False):
    """An engine with random weights of `cfg` (written as a model folder and loaded like any other).  The large
    models draw their weights on the device: the host generator would take minutes."""
    with tempfile.TemporaryDirectory() as folder:
        bt.write_random_model(folder, cfg, seed=0, storage="bfloat16", device="cuda" if fast_weights else None)
        return bt.Engine.from_folder(folder, "bfloat16", max_tokens=max_tokens, max_slots=max_slots)


def start_decode(engine, cfg, prompts, new_tokens, bt, events=None):
    """Prefills `prompts` and composes the decode step of the batch; returns (graph, slots).  `events`: a pair of CUDA
    events recorded before and after the prompts' step."""
    from burn_transformers_b200.engine.graphs import DecodeSession
    from burn_transformers_b200.sampling.sampler import DeviceSampler
    from burn_transformers_b200.sampling.tracker import SequenceTracker

    batch = len(prompts)
    config = bt.GenerationConfig(max_new_tokens=new_tokens + 2)
    sampler = DeviceSampler(config, cfg["vocab_size"], engine.device, batch)
    trackers = [SequenceTracker(i, p, config) for i, p in enumerate(prompts)]
    slots = {i: engine.new_sequence() for i in range(batch)}
    try:
        if events is not None:
            events[0].record()
        logits = engine.step([bt.StepEntry(slots[i], p, [len(p) - 1]) for i, p in enumerate(prompts)])
        if events is not None:
            events[1].record()
        ids, logps = sampler.select(logits, trackers)
        for t, tok, lp in zip(trackers, ids, logps):
            t.push(tok, lp)
        engine.cache.reserve([(slots[i], len(p) + new_tokens + 1) for i, p in enumerate(prompts)])
        session = DecodeSession(engine, config, batch)
        return session._compose(trackers, slots), slots
    except BaseException:
        for s in slots.values():
            engine.release(s)
        raise


def decode_points(engine, cfg, batch, prompt_len, steps, warmup, torch, bt, rng):
    """`warmup` + `steps` decode steps of `batch` sequences after a prefill of `prompt_len` tokens each: every
    step is one replay of the recorded forward + greedy selection + advance, the selected tokens being fed
    forward on the device.  Returns (ms per step on the device, kernels launched in the timed region, mean
    context of the timed steps)."""
    prompts = [rng.integers(0, cfg["vocab_size"], prompt_len).tolist() for _ in range(batch)]
    graph, slots = start_decode(engine, cfg, prompts, steps + warmup, bt)
    try:
        for _ in range(warmup):
            graph.run()
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        start.record()
        for _ in range(steps):
            graph.run()
        stop.record()
        torch.cuda.synchronize()
        ms = start.elapsed_time(stop) / steps
        launches = graph.launches * steps
    finally:
        for s in slots.values():
            engine.release(s)
    mean_ctx = prompt_len + warmup + (steps + 1) / 2
    return ms, launches, mean_ctx


def spread(samples):
    """Median, 95th percentile, minimum and maximum of the repetitions."""
    ordered = sorted(samples)
    p95 = ordered[min(len(ordered) - 1, int(round(0.95 * (len(ordered) - 1))))]
    return {"median": statistics.median(ordered), "p95": p95, "min": ordered[0], "max": ordered[-1], "n": len(ordered)}


def decode_series(engine, cfg, prompt_lengths, steps, torch, bt, rng, pk):
    """A decode workload measured as the reference's protocol asks: 3 unmeasured repetitions, then 10 measured
    ones, each with the cache state made anew (new slots, a new prefill of new random prompts of these lengths) and
    `steps` decode steps timed on the device.  Returns tokens per second at the median with the spread of ms per
    step and the fraction of the copy rate: bytes a step has to read (every weight once, the cache of the live
    requests at the mean context of the timed steps) over its median time."""
    batch = len(prompt_lengths)
    samples, prompt_samples = [], []
    for rep in range(WARM_REPETITIONS + REPETITIONS):
        prompts = [rng.integers(0, cfg["vocab_size"], n).tolist() for n in prompt_lengths]
        around_prompts = (torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True))
        graph, slots = start_decode(engine, cfg, prompts, steps + 1, bt, around_prompts)
        try:
            graph.run()
            start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            start.record()
            for _ in range(steps):
                graph.run()
            stop.record()
            torch.cuda.synchronize()
            if rep >= WARM_REPETITIONS:
                samples.append(start.elapsed_time(stop) / steps)
                prompt_samples.append(around_prompts[0].elapsed_time(around_prompts[1]))
        finally:
            for s in slots.values():
                engine.release(s)
    stats = spread(samples)
    mean_ctx = sum(prompt_lengths) / batch + 1 + (steps + 1) / 2
    step_bytes = weight_bytes(cfg) + batch * mean_ctx * kv_bytes_per_token(cfg)
    achieved = step_bytes / (stats["median"] * 1e-3) / 1e9
    # the prompts' own step (all prompts of the batch in one step; a recorded shape replayed from the third repetition)
    prompt_stats = spread(prompt_samples)
    prompt_flops = prefill_flops(cfg, prompt_lengths)
    prompt_step = {"tokens": int(sum(prompt_lengths)), "ms": prompt_stats,
                   "tokens_per_s": sum(prompt_lengths) / prompt_stats["median"] * 1e3,
                   "frac": prompt_flops / (prompt_stats["median"] * 1e-3) / (pk["bf16_tflops"] * 1e12), "of": "burst"}
    return {"tokens_per_s": batch / stats["median"] * 1e3, "ms_per_step": stats, "batch": batch, "steps": steps,
            "mean_context": mean_ctx, "prompt_step": prompt_step,
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": pk["hbm_gbs"], "unit": "GB/s",
                         "frac": achieved / pk["hbm_gbs"], "of": pk["source"]}}


def e2e_decode(engine, cfg, batch, prompt_len, new_tokens, torch, bt, rng):
    """Decoded tokens per second through generate_causal_streaming: host token lists in, host tokens out;
    timed from the first emitted token to the last, so the prompt step is outside."""
    prompts = [rng.integers(0, cfg["vocab_size"], prompt_len).tolist() for _ in range(batch)]
    stamps = []

    def on_token(token):
        if token.sequence == batch - 1:
            stamps.append(time.perf_counter())

    torch.cuda.synchronize()
    bt.generate_causal_streaming(engine, bt.CausalGenerationRequest(prompts, bt.GenerationConfig(max_new_tokens=new_tokens)),
                                 on_token)
    torch.cuda.synchronize()
    seconds = stamps[-1] - stamps[0]
    return batch * (len(stamps) - 1) / seconds


def timed_prefill(engine, prompts, torch, bt):
    """Median device time (ms) of the prompts' step over 10 repetitions after 3 unmeasured ones (the first two build
    the kernels' state and record the shape; the rest replay it), slots released and taken anew in between."""
    times = []
    for rep in range(WARM_REPETITIONS + REPETITIONS):
        slots = [engine.new_sequence() for _ in prompts]
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        a.record()
        engine.step([bt.StepEntry(s, p, [len(p) - 1]) for s, p in zip(slots, prompts)])
        b.record()
        torch.cuda.synchronize()
        if rep >= WARM_REPETITIONS:
            times.append(a.elapsed_time(b))
        for s in slots:
            engine.release(s)
    return spread(times)


def run_profile(args, torch, bt, kernels, pk):
    """Where a prefill of 2 x 1,024 tokens and decode steps at batch 8 and 64 spend their time (--model): every
    kernel between two CUDA events, launched directly (no recorded graph, so gaps between launches are not in the
    figures), with the rate each kernel class achieved; the fused decode step by its own timeline of block 0."""
    import numpy as np
    cfg = gpt2(args.model)
    rng = np.random.default_rng(0)
    engine = make_engine(cfg, bt, torch, max_tokens=64 * CONTEXT, max_slots=64, fast_weights=args.model != "small")
    d, L = cfg["n_embd"], cfg["n_layer"]
    report = {"profile": True, "model": args.model, "peaks": pk}

    def table(rows, attention_flops=0.0, attention_bytes=0.0, steps=1):
        out = []
        for row in rows:
            if row["kernel"].startswith("attention"):
                row["flops"], row["bytes"] = attention_flops, attention_bytes
                seconds = row["ms"] * 1e-3
                row["tflops"] = attention_flops / seconds / 1e12 if attention_flops else None
                row["gbs"] = attention_bytes / seconds / 1e9 if attention_bytes else None
            out.append({"kernel": row["kernel"], "launches": row["launches"] // steps, "us": round(row["ms"] * 1e3 / steps, 2),
                        "share": round(row["share"], 4),
                        "tflops": None if row["tflops"] is None else round(row["tflops"], 1),
                        "frac_of_bf16_peak": None if row["tflops"] is None else round(row["tflops"] / pk["bf16_tflops"], 4),
                        "gbs": None if row["gbs"] is None else round(row["gbs"], 1),
                        "frac_of_copy_rate": None if row["gbs"] is None else round(row["gbs"] / pk["hbm_gbs"], 4)})
        return out

    # prefill, launched kernel by kernel (a shape is recorded as a graph from its third occurrence: use new shapes)
    lengths = [PREFILL_TOKENS // 2] * 2
    for warm in range(2):
        prompts = [rng.integers(0, cfg["vocab_size"], n - warm).tolist() for n in lengths]
        slots = [engine.new_sequence() for _ in prompts]
        with kernels.KernelProfile() as prof:
            engine.step([bt.StepEntry(s, p, [len(p) - 1]) for s, p in zip(slots, prompts)])
        rows = prof.summary()
        for s in slots:
            engine.release(s)
    report["prefill_2x1024"] = table(rows, attention_flops=sum(L * 2 * s * s * d for s in lengths))
    # decode steps as separate kernels
    engine.use_fused_step = False
    for batch in (8, 64):
        prompts = [rng.integers(0, cfg["vocab_size"], 512).tolist() for _ in range(batch)]
        graph, slots = start_decode(engine, cfg, prompts, 40, bt)
        try:
            for _ in range(3):
                graph._issue()
            steps = 8
            with kernels.KernelProfile() as prof:
                for _ in range(steps):
                    graph._issue()
            rows = prof.summary()
        finally:
            for s in slots.values():
                engine.release(s)
        kv = batch * 520 * kv_bytes_per_token(cfg) * steps
        report[f"decode_b{batch}_separate_kernels"] = table(rows, attention_bytes=kv, steps=steps)
    # the fused decode step: block 0's timeline, by kind of phase
    engine.use_fused_step = True
    engine._graphs.clear()
    prompts = [rng.integers(0, cfg["vocab_size"], 512).tolist() for _ in range(8)]
    graph, slots = start_decode(engine, cfg, prompts, 40, bt)
    try:
        for _ in range(4):
            graph.run()
        program = graph.program
        if program is not None:
            n = len(program.phases)
            trace = torch.zeros(8 * n, dtype=torch.int64, device=engine.device)
            torch.cuda.synchronize()
            program.launch(trace=trace)
            torch.cuda.synchronize()
            t = trace.cpu().numpy().reshape(n, 8)
            kinds = {0: "embed", 1: "product", 2: "attention", 3: "selection"}
            groups: dict[str, list[float]] = {}
            for i, ph in enumerate(program.phases):
                if t[i, 0] == 0:
                    continue
                name = kinds[ph.type] + (f" N={ph.N} K={ph.K}" if ph.type == 1 else "")
                end_of_previous = t[i - 1, 1] if i > 0 and t[i - 1, 1] else t[i, 0]
                groups.setdefault(name, []).append((t[i, 1] - end_of_previous) / 1e3)
            total = (t[n - 2, 1] - t[0, 0]) / 1e3 if n >= 2 else 0.0
            report["decode_b8_fused_step"] = {
                "phases": [{"phase": k, "count": len(v), "us_each": round(statistics.median(v), 2),
                            "us_total": round(sum(v), 1)} for k, v in groups.items()],
                "us_block0": round(float(total), 1)}
    finally:
        for s in slots.values():
            engine.release(s)
    print(json.dumps(report))
    return 0


def run_ours(args):
    import numpy as np
    import torch

    import burn_transformers_b200 as bt
    from burn_transformers_b200 import kernels

    if not torch.cuda.is_available():
        print(json.dumps({"error": "no CUDA device: this benchmark has no CPU path"}))
        return 1
    pk = peaks()
    if args.profile:
        return run_profile(args, torch, bt, kernels, pk)
    cfg = gpt2("small")
    batch, steps, warmup = 8, args.steps, args.warmup
    if steps + warmup > CONTEXT - 4:
        print(json.dumps({"error": f"steps + warmup must stay below the context of {CONTEXT}"}))
        return 1
    prompt_len = min(512, CONTEXT - steps - warmup - 2)
    rng = np.random.default_rng(0)
    # (a run of one workload, for a profiler, holds only the cache that workload needs)
    cache_rows = max(args.batch, 2) if args.only != "all" else 64
    engine = make_engine(cfg, bt, torch, max_tokens=cache_rows * CONTEXT, max_slots=64)
    if args.separate_kernels:
        engine.use_fused_step = False
    before_all = kernels.launch_count()
    if args.only == "decode":
        ms, launches, mean_ctx = decode_points(engine, cfg, args.batch, prompt_len, steps, warmup, torch, bt, rng)
        print(json.dumps({"only": "decode", "batch": args.batch, "ms_per_step": ms, "tokens_per_s": args.batch / ms * 1e3,
                          "gpu_launches": launches, "mean_context": mean_ctx}))
        return 0
    # prefill: 2 sequences x 1,024 tokens
    lengths = [PREFILL_TOKENS // 2] * 2
    prompts = [rng.integers(0, cfg["vocab_size"], n).tolist() for n in lengths]
    prefill_stats = timed_prefill(engine, prompts, torch, bt)
    prefill_ms = prefill_stats["median"]
    if args.only == "prefill":
        print(json.dumps({"only": "prefill", "tokens": PREFILL_TOKENS, "ms": prefill_ms, "spread": prefill_stats}))
        return 0
    flops = prefill_flops(cfg, lengths)
    prefill = {"value": PREFILL_TOKENS / prefill_ms * 1e3, "tokens": PREFILL_TOKENS, "ms": prefill_ms,
               "frac": flops / (prefill_ms * 1e-3) / (pk["bf16_tflops"] * 1e12), "of": "burst",
               "frac_of_sustained": flops / (prefill_ms * 1e-3) / (pk["bf16_tflops_sustained"] * 1e12),
               "spread_ms": prefill_stats}
    # the other workloads: GPT-2 small at batch 1 and 64, then (larger models) medium and XL
    points, detail = {}, {}
    series_steps = min(steps, 64)
    for b in (1, 64):
        detail[f"decode_b{b}"] = decode_series(engine, cfg, [512] * b, series_steps, torch, bt, rng, pk)
        points[f"decode_b{b}"] = detail[f"decode_b{b}"]["tokens_per_s"]
    with ClockSampler() as clocks:
        ms, launches, mean_ctx = decode_points(engine, cfg, batch, prompt_len, steps, warmup, torch, bt, rng)
        e2e = e2e_decode(engine, cfg, batch, prompt_len, steps, torch, bt, rng)
    launches_small = kernels.launch_count() - before_all
    detail["decode_b8"] = decode_series(engine, cfg, [512] * batch, series_steps, torch, bt, rng, pk)
    # the same batch at a short and at a long context (the cache's share of a step's bytes goes from 10 % to 55 %)
    for prompt in (128, 900):
        key = f"decode_b8_ctx{prompt}"
        detail[key] = decode_series(engine, cfg, [prompt] * batch, series_steps, torch, bt, rng, pk)
        points[key] = detail[key]["tokens_per_s"]
    h2d = round(engine.last_session.h2d_bytes / max(1, engine.last_session.steps), 1)
    d2h = round(engine.last_session.d2h_bytes / max(1, engine.last_session.steps), 1)
    if args.points == "all":
        del engine
        torch.cuda.empty_cache()
        # GPT-2 medium: 8 prompts with lengths uniform in [16, 900], 128 decode steps
        medium = gpt2("medium")
        lengths_m = [int(n) for n in np.random.default_rng(7).integers(16, 901, 8)]
        eng = make_engine(medium, bt, torch, max_tokens=8 * CONTEXT + 64 * 8, max_slots=8, fast_weights=True)
        detail["medium_ragged8"] = dict(decode_series(eng, medium, lengths_m, 128, torch, bt, rng, pk), prompt_lengths=lengths_m)
        points["medium_ragged8"] = detail["medium_ragged8"]["tokens_per_s"]
        del eng
        torch.cuda.empty_cache()
        # GPT-2 XL: batch 64, prompts of 256 tokens, 256 decode steps, the cache for 64 x 1,024 positions resident
        xl = gpt2("xl")
        eng = make_engine(xl, bt, torch, max_tokens=64 * CONTEXT, max_slots=64, fast_weights=True)
        detail["xl_b64"] = decode_series(eng, xl, [256] * 64, 256, torch, bt, rng, pk)
        detail["xl_b64"]["cache_resident_gb"] = round(64 * CONTEXT * kv_bytes_per_token(xl) / 1e9, 1)
        points["xl_b64"] = detail["xl_b64"]["tokens_per_s"]
        del eng
        torch.cuda.empty_cache()
    value = batch / ms * 1e3
    step_bytes = weight_bytes(cfg) + batch * mean_ctx * kv_bytes_per_token(cfg)
    achieved = step_bytes / (ms * 1e-3) / 1e9
    line = {
        "metric": "decode tok/s at batch 8 (GPT-2 small, 512-token prompts decoded toward the 1,024 context)",
        "value": value, "unit": "tokens/s", "n_gpus": 1, "steps": steps, "warmup": warmup, "ms_per_step": ms,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic: uniform random token ids, random weights (normal std 0.02)",
        "config": {"model": "gpt2-small", "n_layer": cfg["n_layer"], "n_layer_of_config": 12, "n_embd": cfg["n_embd"],
                   "n_head": cfg["n_head"], "head_dim": 64, "n_inner": cfg["n_inner"], "vocab_size": cfg["vocab_size"],
                   "n_positions": cfg["n_positions"], "global_batch": batch, "seq_len": CONTEXT,
                   "prompt_len": prompt_len, "parallelism": "single-gpu", "kv_cache": "bf16 paged (64 tokens)",
                   "sampling": "greedy on device", "l2": "working set of a step exceeds L2 (weights 249 MB + cache)",
                   "peaks": pk["source"]},
        "clocks": clocks.summary(),
        "e2e": {"value": e2e, "unit": "tokens/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                "note": "generate_causal_streaming: prompts as host lists, every step's ids and log-probabilities "
                        "read back to pinned host memory; tokens are fed forward on the device, so a step's own "
                        "input copy is the integers of a recomposed batch only"},
        "gpu_launches": launches,
        "prefill": prefill,
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": achieved / pk["hbm_gbs"], "bytes_per_step": step_bytes, "of": pk["source"]},
        "points": points,
        "detail": detail,
        "launches_total": launches_small,
    }
    print(json.dumps(line))
    return 0


def main() -> int:
    parser = argparse.ArgumentParser(description=__doc__)
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=256)
    parser.add_argument("--warmup", type=int, default=8)
    parser.add_argument("--impl", choices=["ours", "reference"], default="ours")
    parser.add_argument("--only", choices=["all", "decode", "prefill"], default="all",
                        help="for profiling: run only the decode steps (at --batch) or only the prefill")
    parser.add_argument("--batch", type=int, default=8, help="batch of the decode steps under --only decode")
    parser.add_argument("--separate-kernels", action="store_true",
                        help="decode steps as a CUDA graph of separate kernels instead of the fused decode step")
    parser.add_argument("--points", choices=["all", "small"], default="all",
                        help="small: leave out the GPT-2 medium and XL workloads (they take about a minute more)")
    parser.add_argument("--profile", action="store_true",
                        help="print where a prefill and a decode step spend their time, kernel by kernel, instead")
    parser.add_argument("--model", choices=["small", "medium", "xl"], default="small", help="the model --profile looks at")
    args = parser.parse_args()
    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable": "the reference is a Rust crate (Cargo.toml only): pip "
                          "cannot install it and there is no cargo or rustc in this image; it also publishes no GPT-2 "
                          "generation path"}))
        return 0
    if args.gpus != 1:
        print(f"bench.py measures one GPU only: this library serves one model on one GPU (asked for --gpus {args.gpus})")
        return 2
    if args.warmup < 3:
        args.warmup = 3
    return run_ours(args)


if __name__ == "__main__":
    sys.exit(main())
