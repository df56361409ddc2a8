#!/usr/bin/env python3
"""Decode and prefill throughput of the engine on one B200, as one JSON line.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--preset smollm2-135m] [--batch 8]
    python bench.py --impl reference ...

A "step" is one decode step of the whole batch.  The default run has the layer sizes of the
SmolLM2-135M-shaped configuration with random weights N(0, 0.02), bfloat16, a batch of 8
sequences whose prompts have unequal lengths uniform in [128, 2048], and a context limit of
4096.  `value` is decoded tokens per second, timed on the device with CUDA events over exactly
K steps after W warm-up steps; `e2e` is the same through the Python entry point with host
token ids in and out every step.  Also on the line: a 2,048-token prefill, the decode step's
HBM roofline, decode at batch 1 and 64, the clocks seen during the timed steps, and the
number of kernels launched in them.  More than one GPU is not what this library does: N > 1
prints a line that says so and exits with 2.
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}


def read_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(p) as f:
            d = json.load(f)
        return {"hbm_gbs": float(d["hbm_gbs"]), "bf16_tflops": float(d["bf16_tflops"]),
                "bf16_tflops_sustained": float(d.get("bf16_tflops_sustained", d["bf16_tflops"])), "source": "measured"}
    except Exception:
        return dict(FALLBACK_PEAKS, bf16_tflops_sustained=1400.0, source="fallback")


class ClockSampler:
    """nvidia-smi clock and throttle-reason samples every 200 ms while the timed steps run."""
    QUERY = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.lines, self.proc, self.thread = [], None, None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", "0", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                                          "-lms", "200"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            return
        self.thread = threading.Thread(target=lambda: [self.lines.append(l) for l in self.proc.stdout], daemon=True)
        self.thread.start()

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.25)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for l in self.lines:
            f = [x.strip() for x in l.split(",")]
            if len(f) < 7:
                continue
            try:
                sm.append(float(f[0]))
                mx.append(float(f[1]))
            except ValueError:
                continue
            for n, v in zip(names, f[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def prompt_lengths(batch, lo, hi, seed):
    import random
    r = random.Random(seed)
    return [r.randint(lo, hi) for _ in range(batch)]


def random_prompt(n, vocab, seed):
    import random
    r = random.Random(seed)
    return [r.randrange(vocab) for _ in range(n)]


def decode_bytes(model, cache, lengths):
    """Bytes one decode step has to read: every weight once, and the cache of the live requests."""
    return model.weight_bytes() + cache.bytes_per_token() * sum(lengths)


def prefill_flops(cfg, T):
    """Matrix products of all layers over T tokens, causal attention, and the head on the last row."""
    D, I, nh, nkv, hd, L, V = (cfg.hidden_size, cfg.intermediate_size, cfg.num_attention_heads, cfg.num_key_value_heads,
                               cfg.head_dim, cfg.num_hidden_layers, cfg.vocab_size)
    per_layer = (nh + 2 * nkv) * hd * D + nh * hd * D + 3 * D * I
    linear = 2.0 * T * per_layer * L
    attn = 4.0 * nh * hd * (T * (T + 1) / 2.0) * L
    return linear + attn + 2.0 * D * V


def time_decode(engine, params, batch, steps, warmup, ctx_limit, vocab, seed, e2e):
    """Prefill `batch` prompts of unequal lengths (untimed), then W warm-up and K timed decode steps.
    Device-timed (CUDA events around the K steps), or end to end (wall clock, host tokens in and out)."""
    import torch
    lens = prompt_lengths(batch, 128, 2048, seed)
    lens = [min(l, ctx_limit - steps - warmup - 1) for l in lens]
    slots = engine.open(batch)
    engine.seed(slots, params)
    toks = engine.prefill_sampled(slots, [random_prompt(n, vocab, seed + 1 + i) for i, n in enumerate(lens)], params)
    for _ in range(warmup):
        toks = engine.decode_sampled(slots, toks, params)
    torch.cuda.synchronize()
    from edgelm_b200.csrc import ops
    launches0 = ops.LAUNCHES
    h2d = d2h = 0
    ctx_sum = sum(engine.length(s) for s in slots) * steps + batch * steps * (steps - 1) // 2
    if e2e:
        t0 = time.perf_counter()
        for _ in range(steps):
            toks = engine.decode_sampled(slots, toks, params)  # host ids in, host ids out, every step
            h2d += engine.h2d_bytes_last
            d2h += 4 * batch
        torch.cuda.synchronize()
        ms = (time.perf_counter() - t0) * 1e3
    else:
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        start.record()
        for _ in range(steps):
            engine.decode_launch(slots, toks, params)  # the same ids again: what is timed is the device's work
            h2d += engine.h2d_bytes_last
        end.record()
        torch.cuda.synchronize()
        ms = start.elapsed_time(end)
    launches = ops.LAUNCHES - launches0
    mean_ctx = ctx_sum / steps
    engine.close(slots)
    return {"ms": ms, "tok_s": batch * steps / (ms / 1e3), "launches": launches, "h2d": h2d // steps, "d2h": d2h // steps,
            "mean_ctx_tokens": mean_ctx}


def time_prefill(engine, T, vocab, seed, warmup=3, reps=5):
    import torch
    from edgelm_b200.engine.engine import StepEntry
    prompt = random_prompt(T, vocab, seed)
    times = []
    for i in range(warmup + reps):
        slot = engine.open(1)[0]
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        s.record()
        engine.step([StepEntry(slot, prompt, [T - 1])])
        e.record()
        torch.cuda.synchronize()
        engine.close([slot])
        if i >= warmup:
            times.append(s.elapsed_time(e))
    return statistics.median(times)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=128)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--preset", default="smollm2-135m")
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--ctx", type=int, default=4096)
    ap.add_argument("--layers", type=int, default=None, help="fewer layers than the preset (named in config)")
    ap.add_argument("--dtype", default="bfloat16")
    ap.add_argument("--no-points", action="store_true", help="skip decode at batch 1 and 64")
    ap.add_argument("--no-graphs", action="store_true")
    args = ap.parse_args()

    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable": "adarsh-sgh/edgelm is a C++17 CPU program with no setup.py or "
                          "pyproject.toml: 'pip install --no-index --target baseline/_ref' of its checkout ends with 'not installable'; "
                          "it has no GPU path and no batch > 1"}))
        return 0
    if args.gpus != 1:
        print(json.dumps({"error": f"this library runs on one GPU; --gpus {args.gpus} is not supported", "n_gpus": args.gpus}))
        return 2
    steps, warmup = max(1, args.steps), max(3, args.warmup)

    import torch
    from edgelm_b200.engine.engine import Engine
    from edgelm_b200.presets import preset_config, random_model
    from edgelm_b200.sampling import SamplingParams

    peaks = read_peaks()
    cfg = preset_config(args.preset)
    full_layers = cfg.num_hidden_layers
    model = random_model(cfg, seed=0, sigma=0.02, dtype=args.dtype, layers=args.layers)
    cfg = model.config
    params = SamplingParams(0.0, 40, 42)  # greedy, as edgelm's bench command (src/main.cpp:199-217)
    vocab = cfg.vocab_size
    max_b = args.batch if args.no_points else max(args.batch, 64)
    engine = Engine(model, max_tokens=max_b * args.ctx, max_step_tokens=8192, use_graphs=not args.no_graphs)

    clocks = ClockSampler()
    clocks.start()
    dev = time_decode(engine, params, args.batch, steps, warmup, args.ctx, vocab, seed=11, e2e=False)
    clock_rec = clocks.stop()
    e2e = time_decode(engine, params, args.batch, steps, warmup, args.ctx, vocab, seed=11, e2e=True)
    pre_ms = time_prefill(engine, 2048, vocab, seed=5)
    points = {}
    if not args.no_points:
        for b in (1, 64):
            r = time_decode(engine, params, b, min(steps, 64), warmup, args.ctx, vocab, seed=13 + b, e2e=False)
            points[f"decode_b{b}"] = round(r["tok_s"], 1)

    step_s = dev["ms"] / 1e3 / steps
    bytes_step = model.weight_bytes() + engine.cache.bytes_per_token() * dev["mean_ctx_tokens"]
    achieved = bytes_step / step_s / 1e9
    flops = prefill_flops(cfg, 2048)
    out = {
        "metric": "decode tok/s", "value": round(dev["tok_s"], 1), "unit": "tok/s", "n_gpus": 1, "steps": steps,
        "warmup": warmup, "ms_per_step": round(dev["ms"] / steps, 4), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16" if args.dtype in ("bfloat16", "bf16") else "fp32", "data": "synthetic: random weights N(0,0.02), uniform random token ids",
        "impl": "ours",
        "config": {
            "model": args.preset, "layers": cfg.num_hidden_layers, "layers_of_preset": full_layers, "hidden": cfg.hidden_size,
            "heads": cfg.num_attention_heads, "kv_heads": cfg.num_key_value_heads, "head_dim": cfg.head_dim,
            "intermediate": cfg.intermediate_size, "vocab": cfg.vocab_size, "rope_theta": cfg.rope_theta,
            "rms_norm_eps": cfg.rms_norm_eps, "tied": cfg.tie_word_embeddings, "global_batch": args.batch,
            "seq_len": args.ctx, "prompt_lens": "uniform[128,2048]", "mean_ctx": round(dev["mean_ctx_tokens"] / args.batch, 1),
            "parallelism": "single-gpu", "cuda_graphs": not args.no_graphs,
            "l2": "each step reads %.0f MB of weights and cache, more than the 126 MB L2" % (bytes_step / 1e6),
        },
        "e2e": {"value": round(e2e["tok_s"], 1), "unit": "tok/s", "h2d_bytes_per_step": e2e["h2d"], "d2h_bytes_per_step": e2e["d2h"]},
        "gpu_launches": dev["launches"],
        "prefill": {"value": round(2048 / (pre_ms / 1e3), 1), "tokens": 2048, "ms": round(pre_ms, 3),
                    "frac": round(flops / (pre_ms / 1e3) / (peaks["bf16_tflops"] * 1e12), 4)},
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": peaks["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / peaks["hbm_gbs"], 4), "peaks": "of " + peaks["source"]},
        "points": points,
        "clocks": clock_rec,
    }
    print(json.dumps(out))
    return 0


if __name__ == "__main__":
    sys.exit(main())
