#!/usr/bin/env python3
"""Decode and prefill throughput of the engine on one B200, as one JSON line.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--preset smollm2-135m] [--batch 8] [--sizes a,b | none]
    python bench.py --impl reference ...

A "step" is one decode step of the whole batch.  The default run has the layer sizes of the
SmolLM2-135M-shaped configuration with random weights N(0, 0.02), bfloat16, a batch of 8
sequences whose prompts have unequal lengths uniform in [128, 2048], and a context limit of
4096.  `value` is decoded tokens per second, timed on the device with CUDA events over exactly
K steps after W warm-up steps; `e2e` is the same through the Python entry point with host
token ids in and out every step.  Also on the line: a 2,048-token prefill (through the step
function, and the device time of its kernels alone), the decode step's HBM roofline, decode at
batch 1 and 64 and at a context of 8,192, each with its fraction of the roofline, edgelm's own
benchmark workload (one sequence, 128 + 64 tokens) in float32 and bfloat16, the same
measurements at the layer sizes of the larger SmolLM2 shapes (`sizes`; the flat copies of
their headline figures are in `points`), the clocks seen during the timed steps, and the number
of kernels launched in them.  More than one GPU is not what this library does: N > 1 prints a
line that says so and exits with 2.

`--impl reference` times adarsh-sgh/edgelm itself (baseline/reference_arm.py): its stock
`bench` command on the CPU, float32, one sequence; it has nothing else.
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
PUBLISHED_DECODE_TOK_S = 159.3   # edgelm's README.md:83: SmolLM2-135M, float32, one sequence, 128 + 64 tokens, Apple M5, 10 threads


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
    import numpy as np
    return np.random.default_rng(seed).integers(0, vocab, size=n)


def time_decode(engine, params, batch, steps, warmup, ctx_limit, vocab, seed, e2e, prompt_range=(128, 2048)):
    """Prefill `batch` prompts of unequal lengths (untimed), then W warm-up and K timed decode steps.
    Device-timed (CUDA events around the K steps), or end to end (wall clock, host tokens in and out)."""
    import torch
    from edgelm_b200.csrc import ops
    lens = prompt_lengths(batch, prompt_range[0], prompt_range[1], seed)
    lens = [min(l, ctx_limit - steps - warmup - 1) for l in lens]
    slots = engine.open(batch)
    engine.seed(slots, params)
    toks = engine.prefill_sampled(slots, [random_prompt(n, vocab, seed + 1 + i) for i, n in enumerate(lens)], params)
    for _ in range(warmup):
        toks = engine.decode_sampled(slots, toks, params)
    torch.cuda.synchronize()
    launches0 = ops.LAUNCHES
    h2d = d2h = 0
    ctx_sum = sum(engine.length(s) for s in slots) * steps + batch * steps * (steps - 1) // 2
    if e2e:
        t0 = time.perf_counter()
        for _ in range(steps):
            toks = engine.decode_sampled(slots, toks, params)  # host ids in, host ids out (with the error word), every step
            h2d += engine.h2d_bytes_last
            d2h += 4 * batch + 4
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
    engine.check_device_errors()
    return {"ms": ms, "tok_s": batch * steps / (ms / 1e3), "launches": launches, "h2d": h2d // steps, "d2h": d2h // steps,
            "mean_ctx_tokens": mean_ctx, "steps": steps}


def hbm_frac(model, engine, r, peaks):
    """Bytes a decode step has to read (every weight it uses once, the cache of the live requests) / its time / the peak."""
    bytes_step = model.weight_bytes() + engine.cache.bytes_per_token() * r["mean_ctx_tokens"]
    achieved = bytes_step / (r["ms"] / 1e3 / r["steps"]) / 1e9
    return bytes_step, achieved, achieved / peaks["hbm_gbs"]


def time_prefill(engine, T, vocab, seed, warmup=3, reps=5):
    """A prompt of T tokens through the step function (host work included), and the device time of its kernels
    alone (the step's captured graph, replayed)."""
    import torch
    from edgelm_b200.engine.engine import StepEntry
    prompt = random_prompt(T, vocab, seed)
    times, kernels = [], None
    for i in range(warmup + reps):
        slot = engine.open(1)[0]
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        s.record()
        engine.step([StepEntry(slot, prompt, [T - 1])])
        e.record()
        torch.cuda.synchronize()
        if i == warmup + reps - 1:
            g = engine._step_graphs.get(((T,), 1))
            if g is not None:   # the slot is still open: replaying the graph runs the same step on the same pages again
                ks = []
                for _ in range(reps):
                    s2, e2 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                    s2.record()
                    g["graph"].replay()
                    e2.record()
                    torch.cuda.synchronize()
                    ks.append(s2.elapsed_time(e2))
                kernels = statistics.median(ks)
        engine.close([slot])
        if i >= warmup:
            times.append(s.elapsed_time(e))
    engine.check_device_errors()
    return statistics.median(times), kernels


def edgelm_workload(model, prompt_len=128, gen=64, reps=3):
    """edgelm's own benchmark (src/main.cpp:173-233) through the Python entry point: one sequence, its pseudo-random
    prompt of 128 ids, then 64 x (decode, argmax) with host ids in and out; wall clock, medians after a warm-up."""
    import torch
    from edgelm_b200.engine.engine import Engine
    from edgelm_b200.sampling import SamplingParams
    vocab = model.plan.vocab_size
    x, prompt = 12345, []
    lo = 1000 if vocab > 2000 else 0
    for _ in range(prompt_len):
        x = (x * 6364136223846793005 + 1442695040888963407) & ((1 << 64) - 1)
        prompt.append(lo + (x >> 33) % (vocab - lo))
    engine = Engine(model, max_tokens=256, max_step_tokens=prompt_len)
    params = SamplingParams()
    pre, dec = [], []
    for r in range(-1, reps):
        slots = engine.open(1)
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        toks = engine.prefill_sampled(slots, [prompt], params)
        t1 = time.perf_counter()
        for _ in range(gen):
            toks = engine.decode_sampled(slots, toks, params)
        t2 = time.perf_counter()
        engine.close(slots)
        if r >= 0:
            pre.append(prompt_len / (t1 - t0))
            dec.append(gen / (t2 - t1))
    return statistics.median(pre), statistics.median(dec)


def measure(preset, args, peaks, steps, warmup, batches, with_clocks):
    """Everything for one shape: decode at each batch size (device and end to end), the long context, prefill."""
    import torch
    from edgelm_b200.engine.engine import Engine
    from edgelm_b200.presets import preset_config, random_model
    from edgelm_b200.sampling import SamplingParams
    cfg = preset_config(preset)
    model = random_model(cfg, seed=0, sigma=0.02, dtype=args.dtype, layers=args.layers if preset == args.preset else None)
    full_layers = len(cfg.plan().schedule)
    params = SamplingParams(0.0, 40, 42)  # greedy, as edgelm's bench command (src/main.cpp:199-217)
    vocab = model.plan.vocab_size
    long_ctx = min(8192, model.plan.max_positions)
    max_tokens = max(max(batches) * args.ctx, 8 * long_ctx if args.long else 0)
    engine = Engine(model, max_tokens=max_tokens, max_step_tokens=8192, use_graphs=not args.no_graphs)
    out = {"model": model, "engine": engine, "full_layers": full_layers, "decode": {}, "clocks": None}
    for b in batches:
        k = steps if b == args.batch else min(steps, 64)
        clocks = ClockSampler() if (with_clocks and b == args.batch) else None
        if clocks:
            clocks.start()
        dev = time_decode(engine, params, b, k, warmup, args.ctx, vocab, seed=11 if b == args.batch else 13 + b, e2e=False)
        if clocks:
            out["clocks"] = clocks.stop()
        e2e = time_decode(engine, params, b, k, warmup, args.ctx, vocab, seed=11 if b == args.batch else 13 + b, e2e=True)
        bytes_step, achieved, frac = hbm_frac(model, engine, dev, peaks)
        out["decode"][b] = {"dev": dev, "e2e": e2e, "bytes_step": bytes_step, "achieved": achieved, "frac": frac}
    if args.long:
        k = min(steps, 64)
        dev = time_decode(engine, params, 8, k, warmup, long_ctx, vocab, seed=29, e2e=False,
                          prompt_range=(long_ctx - 292, long_ctx - 292))
        bytes_step, achieved, frac = hbm_frac(model, engine, dev, peaks)
        out["long"] = {"dev": dev, "ctx": long_ctx, "bytes_step": bytes_step, "achieved": achieved, "frac": frac}
    step_ms, kernel_ms = time_prefill(engine, 2048, vocab, seed=5)
    flops = model.flops(2048, 2048 * 2049 / 2.0, 1)
    out["prefill"] = {"ms": step_ms, "kernels_ms": kernel_ms, "flops": flops,
                      "frac": flops / (step_ms / 1e3) / (peaks["bf16_tflops"] * 1e12),
                      "kernels_frac": flops / (kernel_ms / 1e3) / (peaks["bf16_tflops"] * 1e12) if kernel_ms else None}
    torch.cuda.synchronize()
    return out


def summary(m):
    """The figures of one shape as a small dict (for `sizes`)."""
    d = {"layers": len(m["model"].schedule), "layers_of_preset": m["full_layers"]}
    for b, r in m["decode"].items():
        d[f"decode_b{b}"] = {"tok_s": round(r["dev"]["tok_s"], 1), "ms_per_step": round(r["dev"]["ms"] / r["dev"]["steps"], 4),
                             "e2e_tok_s": round(r["e2e"]["tok_s"], 1), "gb_s": round(r["achieved"], 1), "frac": round(r["frac"], 4)}
    if "long" in m:
        r = m["long"]
        d[f"decode_b8_ctx{r['ctx']}"] = {"tok_s": round(r["dev"]["tok_s"], 1), "ms_per_step": round(r["dev"]["ms"] / r["dev"]["steps"], 4),
                                         "gb_s": round(r["achieved"], 1), "frac": round(r["frac"], 4)}
    p = m["prefill"]
    d["prefill_2048"] = {"tok_s": round(2048 / (p["ms"] / 1e3), 1), "ms": round(p["ms"], 3), "frac": round(p["frac"], 4),
                         "kernels_ms": round(p["kernels_ms"], 3) if p["kernels_ms"] else None,
                         "kernels_frac": round(p["kernels_frac"], 4) if p["kernels_frac"] else None}
    return d


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
    ap.add_argument("--sizes", default="smollm2-360m,smollm2-1.7b", help="other shapes measured on the same line, or 'none'")
    ap.add_argument("--no-points", action="store_true", help="only the headline batch: no batch 1 and 64, no long context, no other sizes")
    ap.add_argument("--no-graphs", action="store_true")
    args = ap.parse_args()

    if args.impl == "reference":
        sys.path.insert(0, os.path.join(ROOT, "baseline"))
        import reference_arm
        return reference_arm.main()
    if args.gpus != 1:
        print(json.dumps({"error": f"this library runs on one GPU; --gpus {args.gpus} is not supported", "n_gpus": args.gpus}))
        return 2
    steps, warmup = max(1, args.steps), max(3, args.warmup)
    args.long = not args.no_points

    import torch

    peaks = read_peaks()
    batches = [args.batch] if args.no_points else sorted({1, args.batch, 64})
    main_m = measure(args.preset, args, peaks, steps, warmup, batches, with_clocks=True)
    model, engine = main_m["model"], main_m["engine"]
    head = main_m["decode"][args.batch]
    dev, e2e = head["dev"], head["e2e"]
    sizes_of = model.sizes()
    points = {}
    for b, r in main_m["decode"].items():
        if b != args.batch:
            points[f"decode_b{b}"] = round(r["dev"]["tok_s"], 1)
        points[f"decode_b{b}_frac"] = round(r["frac"], 4)
        points[f"decode_b{b}_e2e"] = round(r["e2e"]["tok_s"], 1)
    if "long" in main_m:
        points[f"decode_b8_ctx{main_m['long']['ctx']}"] = round(main_m["long"]["dev"]["tok_s"], 1)
        points[f"decode_b8_ctx{main_m['long']['ctx']}_frac"] = round(main_m["long"]["frac"], 4)
    pre = main_m["prefill"]
    clock_rec = main_m["clocks"]
    if pre["kernels_ms"]:
        points["prefill_kernels_ms"] = round(pre["kernels_ms"], 3)
        points["prefill_kernels_frac"] = round(pre["kernels_frac"], 4)
    sizes = {args.preset: summary(main_m)}
    vs_baseline = None
    if not args.no_points:
        # edgelm's own workload (one sequence, 128 + 64 tokens), the one row its published numbers have
        _, dec16 = edgelm_workload(model)
        points["edgelm_bench_b1_bf16"] = round(dec16, 1)
        del main_m, engine
        torch.cuda.empty_cache()
        if args.preset == "smollm2-135m":
            from edgelm_b200.presets import preset_config, random_model
            m32 = random_model(preset_config(args.preset), seed=0, sigma=0.02, dtype="float32")
            _, dec32 = edgelm_workload(m32)
            points["edgelm_bench_b1_f32"] = round(dec32, 1)
            vs_baseline = round(dec32 / PUBLISHED_DECODE_TOK_S, 2)
            del m32
        torch.cuda.empty_cache()
        for other in [s for s in args.sizes.split(",") if s and s != "none" and s != args.preset]:
            m = measure(other, args, peaks, min(steps, 64), warmup, batches, with_clocks=False)
            sizes[other] = summary(m)
            tag = other.replace("smollm2-", "").replace(".", "p")
            for b, r in m["decode"].items():
                points[f"{tag}_decode_b{b}"] = round(r["dev"]["tok_s"], 1)
                points[f"{tag}_decode_b{b}_frac"] = round(r["frac"], 4)
            if "long" in m:
                points[f"{tag}_decode_b8_ctx{m['long']['ctx']}_frac"] = round(m["long"]["frac"], 4)
            points[f"{tag}_prefill_tok_s"] = round(2048 / (m["prefill"]["ms"] / 1e3), 1)
            points[f"{tag}_prefill_frac"] = round(m["prefill"]["frac"], 4)
            del m
            torch.cuda.empty_cache()

    out = {
        "metric": "decode tok/s", "value": round(dev["tok_s"], 1), "unit": "tok/s", "n_gpus": 1, "steps": steps,
        "warmup": warmup, "ms_per_step": round(dev["ms"] / steps, 4), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": vs_baseline,
        "vs_baseline_of": "points.edgelm_bench_b1_f32 / 159.3 tok/s (edgelm README.md:83: the same shape and workload, float32, one "
                          "sequence, Apple M5 CPU); batch 8, bfloat16 and 2,048-token prompts have no published counterpart",
        "dtype": "bf16" if args.dtype in ("bfloat16", "bf16") else "fp32", "data": "synthetic: random weights N(0,0.02), uniform random token ids",
        "impl": "ours",
        "config": {
            "model": args.preset, "layers": sizes_of["layers"], "layers_of_preset": sizes[args.preset]["layers_of_preset"],
            "hidden": sizes_of["hidden"], "heads": sizes_of.get("heads"), "kv_heads": sizes_of.get("kv_heads"),
            "head_dim": sizes_of.get("head_dim"), "intermediate": sizes_of.get("intermediate"), "vocab": sizes_of.get("vocab"),
            "rope_theta": sizes_of.get("rope_theta"), "rms_norm_eps": sizes_of.get("rms_norm_eps"), "tied": sizes_of.get("tied"),
            "global_batch": args.batch, "seq_len": args.ctx, "prompt_lens": "uniform[128,2048]",
            "mean_ctx": round(dev["mean_ctx_tokens"] / args.batch, 1), "parallelism": "single-gpu", "cuda_graphs": not args.no_graphs,
            "l2": "each step reads %.0f MB of weights and cache, more than the 126 MB L2" % (head["bytes_step"] / 1e6),
        },
        "e2e": {"value": round(e2e["tok_s"], 1), "unit": "tok/s", "h2d_bytes_per_step": e2e["h2d"], "d2h_bytes_per_step": e2e["d2h"]},
        "gpu_launches": dev["launches"],
        "prefill": {"value": round(2048 / (pre["ms"] / 1e3), 1), "tokens": 2048, "ms": round(pre["ms"], 3), "frac": round(pre["frac"], 4)},
        "roofline": {"bound": "hbm", "achieved": round(head["achieved"], 1), "peak": peaks["hbm_gbs"], "unit": "GB/s",
                     "frac": round(head["frac"], 4), "peaks": "of " + peaks["source"]},
        "points": points,
        "sizes": sizes,
        "clocks": clock_rec,
    }
    print(json.dumps(out))
    return 0


if __name__ == "__main__":
    sys.exit(main())
