"""Decode and prefill throughput of GPT-2 small (random weights, synthetic tokens) on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]

A step is one decode step of a batch of 8 sequences.  The run prints one JSON line: `value` is decoded
tokens per second, timed on the device with CUDA events over exactly K steps; `e2e` is the same through the
public generate entry point with host tokens in and out; `prefill`, `roofline` and `points` explain it.
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
                                          "--format=csv,noheader,nounits", "-lms", "100"], stdout=self.file,
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


def gpt2_small():
    return dict(model_type="gpt2", n_layer=12, n_embd=768, n_head=12, n_inner=3072, vocab_size=50257,
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


def decode_points(engine, cfg, batch, prompt_len, steps, warmup, torch, bt, rng):
    """`warmup` + `steps` decode steps of `batch` sequences after a prefill of `prompt_len` tokens each: every
    step is one replay of the recorded forward + greedy selection + advance, the selected tokens being fed
    forward on the device.  Returns (ms per step on the device, kernels launched in the timed region, mean
    context of the timed steps)."""
    from burn_transformers_b200.engine.graphs import DecodeSession
    from burn_transformers_b200.sampling.sampler import DeviceSampler
    from burn_transformers_b200.sampling.tracker import SequenceTracker

    config = bt.GenerationConfig(max_new_tokens=steps + warmup + 2)
    prompts = [rng.integers(0, cfg["vocab_size"], prompt_len).tolist() for _ in range(batch)]
    sampler = DeviceSampler(config, cfg["vocab_size"], engine.device, batch)
    trackers = [SequenceTracker(i, p, config) for i, p in enumerate(prompts)]
    slots = {i: engine.new_sequence() for i in range(batch)}
    try:
        logits = engine.step([bt.StepEntry(slots[i], p, [len(p) - 1]) for i, p in enumerate(prompts)])
        ids, logps = sampler.select(logits, trackers)
        for t, tok, lp in zip(trackers, ids, logps):
            t.push(tok, lp)
        engine.cache.reserve([(slots[i], prompt_len + steps + warmup + 1) for i in range(batch)])
        session = DecodeSession(engine, config, batch)
        graph = session._compose(trackers, slots)
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


def run_ours(args):
    import numpy as np
    import torch

    import burn_transformers_b200 as bt
    from burn_transformers_b200 import kernels

    if not torch.cuda.is_available():
        print(json.dumps({"error": "no CUDA device: this benchmark has no CPU path"}))
        return 1
    cfg = gpt2_small()
    pk = peaks()
    batch, steps, warmup = 8, args.steps, args.warmup
    if steps + warmup > CONTEXT - 4:
        print(json.dumps({"error": f"steps + warmup must stay below the context of {CONTEXT}"}))
        return 1
    prompt_len = min(512, CONTEXT - steps - warmup - 2)
    rng = np.random.default_rng(0)
    with tempfile.TemporaryDirectory() as folder:
        bt.write_random_model(folder, cfg, seed=0, storage="bfloat16")
        engine = bt.Engine.from_folder(folder, "bfloat16", max_tokens=64 * CONTEXT, max_slots=64)
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
    times = []
    for rep in range(7):
        slots = [engine.new_sequence() for _ in prompts]
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        a.record()
        engine.step([bt.StepEntry(s, p, [len(p) - 1]) for s, p in zip(slots, prompts)])
        b.record()
        torch.cuda.synchronize()
        times.append(a.elapsed_time(b))
        for s in slots:
            engine.release(s)
    prefill_ms = statistics.median(times[3:])      # the first runs build the kernels' state and record the shape
    if args.only == "prefill":
        print(json.dumps({"only": "prefill", "tokens": PREFILL_TOKENS, "ms": prefill_ms}))
        return 0
    prefill = {"value": PREFILL_TOKENS / prefill_ms * 1e3, "tokens": PREFILL_TOKENS, "ms": prefill_ms,
               "frac": prefill_flops(cfg, lengths) / (prefill_ms * 1e-3) / (pk["bf16_tflops"] * 1e12)}
    # decode at batch 1 and 64 (shorter runs), then the headline at batch 8 under the clock sampler
    points = {}
    for b in (1, 64):
        ms, _, _ = decode_points(engine, cfg, b, 512, min(steps, 64), max(3, min(warmup, 8)), torch, bt, rng)
        points[f"decode_b{b}"] = b / ms * 1e3
    with ClockSampler() as clocks:
        ms, launches, mean_ctx = decode_points(engine, cfg, batch, prompt_len, steps, warmup, torch, bt, rng)
        e2e = e2e_decode(engine, cfg, batch, prompt_len, steps, torch, bt, rng)
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
        "e2e": {"value": e2e, "unit": "tokens/s",
                "h2d_bytes_per_step": round(engine.last_session.h2d_bytes / max(1, engine.last_session.steps), 1),
                "d2h_bytes_per_step": round(engine.last_session.d2h_bytes / max(1, engine.last_session.steps), 1),
                "note": "generate_causal_streaming: prompts as host lists, every step's ids and log-probabilities "
                        "read back to pinned host memory; tokens are fed forward on the device, so a step's own "
                        "input copy is the integers of a recomposed batch only"},
        "gpu_launches": launches,
        "prefill": prefill,
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": achieved / pk["hbm_gbs"], "bytes_per_step": step_bytes, "of": pk["source"]},
        "points": points,
        "launches_total": kernels.launch_count() - before_all,
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
