#!/usr/bin/env python3
"""Decode and prefill throughput of the engine on one B200, at the Qwen3-8B layer sizes with
random weights and seeded synthetic token ids.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--layers L] [--impl ours|reference]
                    [--shape 8b|4b|32b] [--serve]

A *step* is one decode step of a batch of 8 requests that each hold 1,024 tokens of context.
``value`` is decoded tokens per second over exactly K steps, timed on the device with CUDA events
after W warm-up steps, through the same captured step and host loop that generation uses.
``e2e`` is the same quantity through ``Engine.generate`` with host token lists in and out.
The line also carries a 2,048-token prefill, the decode step's HBM roofline, and decode at batch
1 and 64.  Weights (15 GB) are far larger than L2, so every step reads them from HBM.
``--shape`` runs the same at the 4B or 32B layer sizes (the 32B at 2,048 tokens of context and
batch 1, 8 and 32), and ``--serve`` times a mixed workload of 16 requests through the scheduler.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}

QWEN3_8B = dict(num_hidden_layers=36, hidden_size=4096, num_attention_heads=32, num_key_value_heads=8,
                head_dim=128, intermediate_size=12288, vocab_size=151936, max_position_embeddings=8192,
                rms_norm_eps=1e-6, rope_theta=1000000.0, tie_word_embeddings=False)
# the other layer shapes the baseline names, for --shape (the default run is the 8B shape)
SHAPES = {
    "8b": ("Qwen3-8B", QWEN3_8B, 1024),
    "4b": ("Qwen3-4B", dict(QWEN3_8B, hidden_size=2560, intermediate_size=9728, max_position_embeddings=32768,
                            tie_word_embeddings=True), 1024),
    "32b": ("Qwen3-32B", dict(QWEN3_8B, num_hidden_layers=64, hidden_size=5120, num_attention_heads=64,
                              intermediate_size=25600), 2048),
}
CONTEXT = 1024
PREFILL_TOKENS = 2048


def load_peaks() -> dict:
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            data = json.load(f)
        peaks = {"hbm_gbs": float(data["hbm_gbs"]), "bf16_tflops": float(data["bf16_tflops"]),
                 "source": "measured"}
        if "bf16_tflops_sustained" in data:
            peaks["bf16_tflops_sustained"] = float(data["bf16_tflops_sustained"])
        return peaks
    except (OSError, KeyError, ValueError, TypeError):
        return dict(FALLBACK_PEAKS)


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while a timed region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.proc = None
        self.lines = []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", "0", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-lms", "200"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.25)
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
            out, _ = self.proc.communicate()
        clocks, max_clock, reasons = [], None, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in out.splitlines():
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 6:
                continue
            try:
                clocks.append(float(parts[0]))
                max_clock = float(parts[1])
            except ValueError:
                continue
            for name, value in zip(names, parts[2:6]):
                if value.lower() == "active":
                    reasons.add(name)
        return {"sm_mhz": statistics.median(clocks) if clocks else None, "sm_max_mhz": max_clock,
                "samples": len(clocks), "reasons": sorted(reasons)}


def seeded_tokens(vocab: int, n: int, seed: int):
    import numpy as np
    return np.random.default_rng(seed).integers(0, vocab, size=n).tolist()


def fill_requests(executor, batch: int, context: int, vocab: int, tag: str):
    """Admits ``batch`` requests and brings each to ``context`` tokens; returns them with the
    last token fed still to come (so the next step is a decode step at that context)."""
    from mrun_b200.engine import StepEntry
    requests = [executor.admit((tag, i)) for i in range(batch)]
    per_step = max(1, PREFILL_TOKENS // context)
    for start in range(0, batch, per_step):
        group = requests[start:start + per_step]
        executor.step([StepEntry(r, seeded_tokens(vocab, context - 1, 1000 + start + i), [])
                       for i, r in enumerate(group)])
    return requests


def time_decode(executor, requests, vocab: int, steps: int, warmup: int, profiler_range: bool = False,
                repeats: int = 1):
    """Device times (ms, one per repeat) of ``steps`` decode steps the way generation runs them: a
    step is launched with the tokens of the step before it taken on the device, then that step's
    tokens are read back into pinned host memory.  Also the kernel launches of one repeat."""
    import torch
    from mrun_b200.engine import StepEntry
    n = len(requests)
    first = seeded_tokens(vocab, n, 7)
    pinned = [torch.empty(n, dtype=torch.int32, pin_memory=True) for _ in range(2)]
    state = {"event": None, "turn": 0}

    def one(first_step: bool):
        tokens = first if first_step else [0] * n
        sources = None if first_step else list(range(n))
        out = executor.decode_step([StepEntry(r, [t], [0]) for r, t in zip(requests, tokens)], None, sources)
        pinned[state["turn"]].copy_(out, non_blocking=True)
        event = torch.cuda.Event()
        event.record()
        if state["event"] is not None:
            state["event"].synchronize()
            pinned[state["turn"] ^ 1].tolist()          # the step before is read here
        state["event"], state["turn"] = event, state["turn"] ^ 1

    one(True)
    for _ in range(warmup - 1):
        one(False)
    times, launches = [], 0
    for repeat in range(repeats):
        torch.cuda.synchronize()
        begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        before = executor.launches.total
        if profiler_range and repeat == 0:   # lets a profiler started with --profile-from-start off see only this
            torch.cuda.profiler.start()
        begin.record()
        for _ in range(steps):
            one(False)
        end.record()
        torch.cuda.synchronize()
        if profiler_range and repeat == 0:
            torch.cuda.profiler.stop()
        times.append(begin.elapsed_time(end))
        launches = executor.launches.total - before
    return times, launches


def serve(args, config, model_name: str, full_layers: int, page_size: int, peaks: dict) -> int:
    """The baseline's mixed workload: 16 requests whose prompts hold 64 to 16,384 seeded tokens,
    prompts cut into portions under a budget of 2,048 tokens a step beside the decoding of the
    others, 256 tokens decoded for each.  Everything goes through ``Engine.generate``; the times
    are the host's clock around that one call (it ends when the last token is on the host)."""
    import numpy as np
    import torch
    from mrun_b200 import Engine
    from mrun_b200.kernels import lib as kernel_lib

    requests, decode_tokens = 16, 256
    lengths = np.random.default_rng(11).integers(64, 16384 + 1, size=requests).tolist()
    prompts = [seeded_tokens(config.vocab_size, n, 200 + i) for i, n in enumerate(lengths)]
    capacity = sum(-(-(n + decode_tokens) // page_size) for n in lengths) + 64
    engine = Engine.from_config(config, seed=0, dtype="bfloat16", page_size=page_size, num_pages=capacity,
                                max_requests=requests, max_batch_tokens=PREFILL_TOKENS)
    engine.generate([p[:300] for p in prompts[:4]], max_tokens=8, ignore_eos=True)       # warm-up: shapes, graphs
    engine.generate(prompts[:2], max_tokens=4, ignore_eos=True)
    sampler = ClockSampler()
    sampler.start()
    steps_before, launches = engine.stats.steps, engine.executor.launches.total
    torch.cuda.synchronize()
    begin = time.perf_counter()
    generations = engine.generate(prompts, max_tokens=decode_tokens, ignore_eos=True)
    torch.cuda.synchronize()
    seconds = time.perf_counter() - begin
    clocks = sampler.stop()
    decoded = sum(len(g.tokens) for g in generations)
    last_first = max(g.first_token_time for g in generations)
    finished = max(g.finished_time for g in generations)
    tail = sum(sum(1 for t in g.token_times if t > last_first) for g in generations)
    steps = engine.stats.steps - steps_before
    line = {
        "metric": f"tokens/s, prompts and decoded, {requests} mixed requests ({model_name} bf16)",
        "value": round((sum(lengths) + decoded) / seconds, 1), "unit": "tok/s", "n_gpus": 1,
        "steps": steps, "warmup": 2, "ms_per_step": round(seconds * 1e3 / max(1, steps), 4),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic (seeded uniform token ids, N(0,0.02) weights)", "impl": "ours",
        "config": {"model": f"{model_name} shape", "layers": config.num_hidden_layers, "layers_of_config": full_layers,
                   "hidden": config.hidden_size, "heads": config.num_attention_heads,
                   "kv_heads": config.num_key_value_heads, "head_dim": config.head_dim,
                   "intermediate": config.intermediate_size, "vocab": config.vocab_size,
                   "tied": config.tie_word_embeddings, "global_batch": requests, "prompt_tokens": sum(lengths),
                   "longest_prompt": max(lengths), "decoded_per_request": decode_tokens,
                   "max_batch_tokens": PREFILL_TOKENS, "page_size": page_size, "parallelism": "single GPU"},
        "seconds": round(seconds, 3), "decoded": decoded,
        "time_to_first_token_s": {"median": round(statistics.median(g.time_to_first_token_s for g in generations), 3),
                                  "max": round(max(g.time_to_first_token_s for g in generations), 3)},
        "decode_tail": {"value": round(tail / max(finished - last_first, 1e-9), 1), "unit": "tok/s",
                        "note": "all 16 decoding side by side, after the last prompt ended"},
        "preemptions": sum(g.preemptions for g in generations),
        "gpu_launches": engine.executor.launches.total - launches, "clocks": clocks, "peaks": peaks,
        "kernel_entry_calls": kernel_lib.call_count(),
    }
    print(json.dumps(line))
    return 0


def main() -> int:
    parser = argparse.ArgumentParser()
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=64)
    parser.add_argument("--warmup", type=int, default=8)
    parser.add_argument("--impl", choices=["ours", "reference"], default="ours")
    parser.add_argument("--layers", type=int, default=None,
                        help="run fewer layers than the configuration has (both numbers are reported)")
    parser.add_argument("--skip-points", action="store_true", help="only the batch-8 decode and the prefill")
    parser.add_argument("--batches", default=None,
                        help="decode batch sizes to run, comma separated (for profiling one point)")
    parser.add_argument("--skip-prefill", action="store_true")
    parser.add_argument("--shape", choices=sorted(SHAPES), default="8b",
                        help="layer sizes: the baseline's 8B shape, or its 4B and 32B shapes")
    parser.add_argument("--serve", action="store_true",
                        help="instead of the decode step: 16 requests with prompts of 64 to 16,384 tokens and "
                             "256 decoded tokens each through Engine.generate, prompts cut at 2,048 tokens")
    parser.add_argument("--context", type=int, default=None,
                        help="tokens each request holds when decoding is timed (the default is the baseline's)")
    parser.add_argument("--prefill-depth", type=int, default=0,
                        help="tokens already in the cache before the timed portion of 2,048 (0: a fresh prompt)")
    parser.add_argument("--skip-e2e", action="store_true")
    parser.add_argument("--page-size", type=int, default=16, help="keys a cache page holds")
    parser.add_argument("--repeats", type=int, default=5,
                        help="how many times the K timed steps are run (the line carries the median, the "
                             "fastest and the slowest)")
    parser.add_argument("--profiler-range", nargs="?", const="decode", default=None, choices=["decode", "prefill"],
                        help="bracket the timed decode steps (or the last timed prefill) with "
                             "cudaProfilerStart/Stop, for a profiler started with --profile-from-start off")
    args = parser.parse_args()

    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable":
                          "hupe1980/mrun is a Rust workspace over an Apple Metal array library (nuvec): "
                          "no cargo/rustc here, no pip-installable package, no Metal device"}))
        return 0
    if args.gpus != 1:
        print(f"bench.py measures one GPU: this engine has no multi-GPU path, --gpus {args.gpus} is not run")
        return 2
    if args.warmup < 3:
        args.warmup = 3

    import torch
    from mrun_b200 import Engine
    from mrun_b200.config import Qwen3Config
    from mrun_b200.kernels import lib as kernel_lib

    peaks = load_peaks()
    model_name, shape_sizes, shape_context = SHAPES[args.shape]
    sizes = dict(shape_sizes)
    if args.context is None:
        args.context = shape_context
    full_layers = sizes["num_hidden_layers"]
    if args.layers is not None:
        sizes["num_hidden_layers"] = args.layers
    if args.serve:
        sizes["max_position_embeddings"] = max(sizes["max_position_embeddings"], 16384 + 256 + 64)
    config = Qwen3Config(**sizes)
    page_size = args.page_size
    if args.serve:
        return serve(args, config, model_name, full_layers, page_size, peaks)
    batches = [8] if args.skip_points else [8, 1, 32 if args.shape == "32b" else 64]
    if args.batches:
        batches = [int(b) for b in args.batches.split(",")]
    args.repeats = max(1, args.repeats)
    slack = args.repeats * args.steps + args.warmup + 64
    context = args.context
    # the requests of every batch size are alive together, so that the clocks can be sampled over all of them
    capacity = max(sum(batches) * (context + slack), 8 * (context + 2 * slack)) + args.prefill_depth + PREFILL_TOKENS + 4 * 64
    sizes["max_position_embeddings"] = max(sizes["max_position_embeddings"], context + slack + 64,
                                           args.prefill_depth + PREFILL_TOKENS + 64)
    config = Qwen3Config(**sizes)
    engine = Engine.from_config(config, seed=0, dtype="bfloat16", page_size=page_size,
                                num_pages=-(-capacity // page_size), max_requests=max(64, sum(batches)),
                                max_batch_tokens=max(PREFILL_TOKENS, args.prefill_depth))
    executor = engine.executor
    vocab = config.vocab_size
    kv_bytes = config.kv_bytes_per_token(2)
    # every weight the step uses, once; of an embedding table that is not also the head only B rows
    weight_bytes = executor.model.weight_bytes()
    if not config.tie_word_embeddings:
        weight_bytes -= vocab * config.hidden_size * 2

    # ---------------------------------------------------------------- prefill, 2,048 tokens
    from mrun_b200.engine import StepEntry
    prompt = seeded_tokens(vocab, PREFILL_TOKENS, 3)
    times = []
    for i in range(0 if args.skip_prefill else 2 + 3):
        request = executor.admit(("prefill", i))
        for start in range(0, args.prefill_depth, 4 * PREFILL_TOKENS):        # the depth, untimed
            executor.step([StepEntry(request, seeded_tokens(vocab, min(4 * PREFILL_TOKENS, args.prefill_depth - start), 5), [])])
        torch.cuda.synchronize()
        begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        ranged = args.profiler_range == "prefill" and i == 4
        if ranged:
            torch.cuda.profiler.start()
        begin.record()
        executor.step([StepEntry(request, prompt, [PREFILL_TOKENS - 1])])
        end.record()
        torch.cuda.synchronize()
        if ranged:
            torch.cuda.profiler.stop()
        executor.release(request)
        if i >= 2:
            times.append(begin.elapsed_time(end))
    prefill_ms = statistics.median(times) if times else float("nan")
    h, d = config.hidden_size, config.head_dim
    linear_params = config.num_hidden_layers * ((config.num_attention_heads + 2 * config.num_key_value_heads) * d * h
                                                + config.num_attention_heads * d * h
                                                + 3 * h * config.intermediate_size)
    prefill_flops = 2.0 * PREFILL_TOKENS * linear_params + 2.0 * vocab * h \
        + config.num_hidden_layers * (2.0 * PREFILL_TOKENS ** 2 + 4.0 * PREFILL_TOKENS * args.prefill_depth) \
        * config.num_attention_heads * d
    prefill = {"value": round(PREFILL_TOKENS / prefill_ms * 1e3, 1), "tokens": PREFILL_TOKENS,
               "ms": round(prefill_ms, 3), **({"depth": args.prefill_depth} if args.prefill_depth else {}),
               "frac": round(prefill_flops / (prefill_ms * 1e-3) / (peaks["bf16_tflops"] * 1e12), 4)}
    if "bf16_tflops_sustained" in peaks:
        prefill["frac_sustained"] = round(prefill_flops / (prefill_ms * 1e-3) / (peaks["bf16_tflops_sustained"] * 1e12), 4)
    if not times:                        # --skip-prefill: nothing was measured, and NaN is no JSON
        prefill = {"skipped": True, "tokens": PREFILL_TOKENS}

    # ---------------------------------------------------------------- decode at batch 8 / 1 / 64
    results = {}
    launches = 0
    all_requests = {batch: fill_requests(executor, batch, context, vocab, f"decode{batch}") for batch in batches}
    sampler = ClockSampler()             # clocks and throttle reasons over every timed decode region
    sampler.start()
    for batch in batches:
        times, n_launch = time_decode(executor, all_requests[batch], vocab, args.steps, args.warmup,
                                      args.profiler_range == "decode", args.repeats)
        if batch == batches[0]:
            launches = n_launch
        results[batch] = times
    clocks = sampler.stop()
    for requests in all_requests.values():
        for r in requests:
            executor.release(r)
    main_batch = batches[0]
    context_mid = context + args.warmup + args.repeats * args.steps / 2.0

    def point(batch):
        """tok/s and the HBM roofline of a batch size: every weight once and the live requests' cache."""
        ms = statistics.median(results[batch]) / args.steps
        step_bytes = weight_bytes + batch * context_mid * kv_bytes + batch * h * 2
        achieved = step_bytes / (ms * 1e-3) / 1e9
        return ms, {"value": round(batch / (ms * 1e-3), 1), "ms_per_step": round(ms, 4),
                    "ms_per_step_min": round(min(results[batch]) / args.steps, 4),
                    "ms_per_step_max": round(max(results[batch]) / args.steps, 4),
                    "bound": "hbm", "achieved": round(achieved, 1), "peak": peaks["hbm_gbs"], "unit": "GB/s",
                    "frac": round(achieved / peaks["hbm_gbs"], 4), "of": peaks["source"]}

    ms_per_step, main_point = point(main_batch)
    value = main_point["value"]
    roofline = {k: main_point[k] for k in ("bound", "achieved", "peak", "unit", "frac", "of")}
    repeats = {"n": args.repeats, "ms_per_step_min": main_point["ms_per_step_min"],
               "ms_per_step_max": main_point["ms_per_step_max"], "value_is": "median over the repeats"}
    others = {f"decode_b{b}": point(b)[1] for b in batches if b != main_batch}
    points = {name: p["value"] for name, p in others.items()}
    points_roofline = {name: {k: p[k] for k in ("ms_per_step", "ms_per_step_min", "ms_per_step_max", "achieved", "frac")}
                       for name, p in others.items()}

    # ---------------------------------------------------------------- end to end, Engine.generate
    if args.skip_e2e:
        line = {"metric": f"decode tok/s at batch {main_batch}", "value": round(value, 1), "ms_per_step": round(ms_per_step, 4),
                "roofline": roofline, "points": points, "points_roofline": points_roofline, "repeats": repeats,
                "gpu_launches": launches, "prefill": prefill}
        print(json.dumps(line))
        return 0
    # Token lists in, token lists out, through Engine.generate.  The token budget of this engine
    # takes the eight prompts in one step, so all eight decode side by side for every step of
    # the window that is timed: from the first token of each (read back on the host) to the last.
    from mrun_b200.engine.engine import Engine as EngineClass
    e2e_engine = EngineClass(executor, max_batch_tokens=main_batch * context)
    out_tokens = args.steps + 1
    prompts = [seeded_tokens(vocab, context, 50 + i) for i in range(main_batch)]
    e2e_engine.generate(prompts, max_tokens=4, ignore_eos=True)         # warm the prompt step's shapes
    uploaded = executor.staging.bytes_uploaded
    steps_before = e2e_engine.stats.steps
    d2h_before = e2e_engine.stats.d2h_bytes
    torch.cuda.synchronize()
    generations = e2e_engine.generate(prompts, max_tokens=out_tokens, ignore_eos=True)
    torch.cuda.synchronize()
    short = [len(g.tokens) for g in generations if len(g.tokens) != out_tokens or g.finish_reason != "length"]
    if short:
        raise RuntimeError(f"end-to-end run: generations ended early ({short} of {out_tokens} tokens)")
    last_first = max(g.first_token_time for g in generations)
    finished = max(g.finished_time for g in generations)
    decoded = sum(sum(1 for t in g.token_times if t > last_first) for g in generations)
    e2e_value = decoded / max(finished - last_first, 1e-9)
    n_steps = max(1, e2e_engine.stats.steps - steps_before)
    engine = e2e_engine
    e2e = {"value": round(e2e_value, 1), "unit": "tok/s",
           "h2d_bytes_per_step": round((executor.staging.bytes_uploaded - uploaded) / n_steps, 1),
           "d2h_bytes_per_step": round((engine.stats.d2h_bytes - d2h_before) / n_steps, 1)}

    line = {
        "metric": f"decode tok/s at batch {main_batch} ({model_name} bf16, {context:,}-token prompts)",
        "value": round(value, 1), "unit": "tok/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": round(ms_per_step, 4), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic (seeded uniform token ids, N(0,0.02) weights)",
        "impl": "ours",
        "config": {
            "model": f"{model_name} shape", "layers": config.num_hidden_layers, "layers_of_config": full_layers,
            "hidden": h, "heads": config.num_attention_heads, "kv_heads": config.num_key_value_heads,
            "head_dim": d, "intermediate": config.intermediate_size, "vocab": vocab,
            "rope_theta": config.rope_theta, "rms_norm_eps": config.rms_norm_eps,
            "tied": config.tie_word_embeddings, "global_batch": main_batch, "seq_len": context,
            "max_context": config.max_position_embeddings, "page_size": page_size,
            "parallelism": "single GPU", "l2": f"inputs larger than L2 ({weight_bytes / 1e9:.0f} GB of weights per step)",
        },
        "e2e": e2e, "gpu_launches": launches, "clocks": clocks,
        "prefill": prefill, "roofline": roofline, "points": points, "points_roofline": points_roofline,
        "repeats": repeats, "peaks": peaks, "kernel_entry_calls": kernel_lib.call_count(),
    }
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
