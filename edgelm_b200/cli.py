"""Command line in the manner of adarsh-sgh/edgelm's (src/main.cpp:366-395): sub-commands
run | bench | info | logits with its option names and meanings where it has them.

  python -m edgelm_b200 run    -m DIR -p "5,17,3;9,9" [-n 64] [--temp 0.8 --top-k 40 --seed 1] [--dtype bf16|f32]
                               [--ctx 1024] [--batch 8192] [--slots 8] [--ignore-eos] [--stop 2,7]
                               [--verbose] [--profile trace.json] [--stats]
  python -m edgelm_b200 bench  -m DIR [--prompt-len 128] [--gen 64] [--reps 3] [--batch-sizes 1,8] [--json]
  python -m edgelm_b200 info   -m DIR [--dtype ..] [--ops]
  python -m edgelm_b200 logits -m DIR --tokens 1,2,3 [--prefill k] --out logits.f32

A model is a folder with config.json and *.safetensors (`-m`), or `--preset NAME` for random
weights of a known shape.  There is no tokenizer here: prompts are token ids, comma-separated,
several prompts separated by `;` (or one per line in `--tokens-file`); output is token ids.
edgelm's options that name what this library does not have (quantized dtypes, --act, --backend,
--threads, --no-simd, --no-fuse, --no-prefault) are not accepted.
"""
import argparse
import json
import statistics
import sys
import time


def _ids(text):
    return [int(t) for t in text.replace(" ", "").split(",") if t != ""]


def _prompts(args):
    if args.tokens_file:
        with open(args.tokens_file) as f:
            return [_ids(line) for line in f if line.strip()]
    return [_ids(p) for p in args.prompt.split(";") if p.strip()]


def _dtype(name):
    table = {"bf16": "bfloat16", "bfloat16": "bfloat16", "f32": "float32", "fp32": "float32", "float32": "float32"}
    if name not in table:
        raise SystemExit("edgelm_b200: --dtype must be bf16|f32")
    return table[name]


def _model(args):
    """A loaded DecoderModel from -m DIR or --preset NAME (random weights, seed --random-seed)."""
    from .engine.engine import load_model
    from .presets import preset_config, random_model
    if args.model:
        return load_model(args.model, _dtype(args.dtype))
    if args.preset:
        return random_model(preset_config(args.preset), seed=args.random_seed, dtype=_dtype(args.dtype))
    raise SystemExit("edgelm_b200: give a model folder with -m or a shape with --preset")


def _engine(args, model, slots=None, profile=False):
    from .engine.engine import Engine
    ctx = min(args.ctx, model.plan.max_positions)
    slots = slots or args.slots
    return Engine(model, max_tokens=(ctx + 63) // 64 * 64 * slots, max_step_tokens=args.batch, profile=profile)


def _describe(model, engine):
    """What `info` and `run --verbose` print: the model as its parts describe themselves (no architecture's
    configuration fields are read here), the cache as it accounts for itself, the step's workspace."""
    desc = model.describe()
    lines = [f"model   : {type(model.config).__name__ if getattr(model, 'config', None) is not None else 'plan'}, {desc[0]}"]
    lines += [f"          {l.strip()}" for l in desc[1:]]
    lines += [f"cache   : {l}" for l in engine.cache.describe()]
    peak = f", {100.0 * engine.ws.peak / engine.ws.capacity:.0f} % used so far" if engine.ws.peak else ""
    lines.append(f"arena   : {engine.ws.capacity / 1e6:.2f} MB for steps of up to {engine.max_step_tokens} tokens and "
                 f"{engine.max_step_seqs} sequences{peak}")
    return "\n".join(lines)


def _finish_profile(args, engine):
    if engine.profiler is None:
        return
    if args.stats:
        print("\n" + engine.profiler.stats(), end="")
    if args.profile:
        n = engine.profiler.write_trace(args.profile)
        print(f"trace: {args.profile} ({n} events; open in ui.perfetto.dev)")


def cmd_run(args):
    from .engine.generate import GenerationLoop
    from .sampling import SamplingParams
    t0 = time.perf_counter()
    model = _model(args)
    load_ms = (time.perf_counter() - t0) * 1e3
    engine = _engine(args, model, profile=bool(args.profile or args.stats))
    if args.verbose:
        print(_describe(model, engine))
    prompts = _prompts(args)
    if args.bos:
        prompts = [[model.plan.bos_token_id] + p for p in prompts]
    stop = _ids(args.stop) if args.stop is not None else list(model.plan.stop_token_ids)
    loop = GenerationLoop(engine, SamplingParams(args.temp, args.top_k, args.seed), max_new_tokens=args.n, stop_ids=stop,
                          ignore_eos=args.ignore_eos, max_batch=args.slots)
    out = loop.run(prompts)
    for p, g in zip(prompts, out):
        print(",".join(str(t) for t in p) + " => " + ",".join(str(t) for t in g.tokens) + f"  [{g.finish_reason}]")
    print(f"\n[{str(model.dtype).replace('torch.', '')}] load {load_ms:.0f} ms, {loop.stats.summary()}")
    _finish_profile(args, engine)
    return 0


def cmd_bench(args):
    """edgelm's bench (src/main.cpp:173-233): a fixed pseudo-random prompt (its LCG, low ids skipped),
    one warm-up then `reps` runs of prefill + argmax + gen x (decode, argmax); medians."""
    from .sampling import SamplingParams
    model = _model(args)
    vocab = model.plan.vocab_size
    P, G = args.prompt_len, args.gen
    x, prompt = 12345, []
    lo = 1000 if vocab > 2000 else 0
    for _ in range(P):
        x = (x * 6364136223846793005 + 1442695040888963407) & ((1 << 64) - 1)
        prompt.append(lo + (x >> 33) % (vocab - lo))
    params = SamplingParams()
    import torch
    if not args.json:
        print(f"{'dtype':<9} {'batch':>5} | {'prefill/s':>10} {'TTFT ms':>9} | {'decode/s':>10} | {'arena MB':>9}")
    for b in [int(v) for v in args.batch_sizes.split(",")]:
        args.ctx = max(args.ctx, P + G + 8)
        engine = _engine(args, model, slots=b)
        pre, ttft, dec = [], [], []
        for r in range(-1, args.reps):
            slots = engine.open(b)
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            toks = engine.prefill_sampled(slots, [prompt] * b, params)
            f_ms = (time.perf_counter() - t0) * 1e3
            t1 = time.perf_counter()
            for _ in range(G):
                toks = engine.decode_sampled(slots, toks, params)
            d_ms = (time.perf_counter() - t1) * 1e3
            engine.close(slots)
            if r < 0:
                continue
            pre.append(b * P / (f_ms / 1e3))
            ttft.append(f_ms)
            dec.append(b * G / (d_ms / 1e3))
        row = {"dtype": str(model.dtype).replace("torch.", ""), "batch": b, "prompt": P, "gen": G,
               "prefill_tok_s": round(statistics.median(pre), 2), "ttft_ms": round(statistics.median(ttft), 2),
               "decode_tok_s": round(statistics.median(dec), 2), "weights_mb": round(model.weight_bytes() / 1e6, 2),
               "arena_mb": round(engine.ws.capacity / 1e6, 3), "cache_mb": round(engine.cache.storage_bytes() / 1e6, 2)}
        if args.json:
            print(json.dumps(row))
        else:
            print(f"{row['dtype']:<9} {b:>5} | {row['prefill_tok_s']:>10.1f} {row['ttft_ms']:>9.1f} | {row['decode_tok_s']:>10.1f} | {row['arena_mb']:>9.2f}")
        sys.stdout.flush()
        del engine
    return 0


def cmd_info(args):
    model = _model(args)
    engine = _engine(args, model)
    print(_describe(model, engine))
    if args.ops:
        print("   0 embedding")
        for i, e in enumerate(model.schedule):
            layer = model.layers[e.layer]
            reads = f" (reads the cache of run {e.reads_cache_of})" if e.reads_cache_of is not None else ""
            print(f"  {i + 1:3d} {getattr(layer, 'prefix', '')} {layer.describe()}{reads}")
        print(f"  {len(model.schedule) + 1:3d} final norm + {model.head.kind}")
    return 0


def cmd_logits(args):
    """edgelm's logits command (src/main.cpp:328-356): one step of the first k ids with logits at every
    position, then one step per remaining id; raw float32 [n_ids, vocab]."""
    import numpy as np

    from .engine.engine import StepEntry
    model = _model(args)
    ids = _ids(args.tokens)
    k = min(args.prefill if args.prefill is not None else len(ids), len(ids))
    args.ctx = max(64, len(ids) + 1)
    engine = _engine(args, model, slots=1)
    slot = engine.open(1)[0]
    parts = []
    if k > 0:
        parts.append(engine.step([StepEntry(slot, ids[:k], list(range(k)))]).cpu().numpy())
    for t in ids[k:]:
        parts.append(engine.step([StepEntry(slot, [t], [0])]).cpu().numpy())
    engine.check_device_errors()
    out = np.concatenate(parts, axis=0).astype("<f4")
    out.tofile(args.out)
    print(f"{len(ids)} tokens x {model.plan.vocab_size} logits -> {args.out}")
    return 0


def build_parser():
    ap = argparse.ArgumentParser(prog="edgelm_b200", description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    sub = ap.add_subparsers(dest="cmd")

    def common(p):
        p.add_argument("-m", "--model", help="model folder (config.json + *.safetensors)")
        p.add_argument("--preset", help="a built-in shape with random weights instead of -m")
        p.add_argument("--random-seed", type=int, default=0)
        p.add_argument("--dtype", default="bf16", help="bf16 | f32 (f32: everything in true 32-bit)")
        p.add_argument("--ctx", type=int, default=1024, help="max context per sequence")
        p.add_argument("--batch", type=int, default=8192, help="tokens per forward (longer steps are cut)")
        p.add_argument("--slots", type=int, default=8, help="sequences alive at once")

    r = sub.add_parser("run")
    common(r)
    r.add_argument("-p", "--prompt", default="1,2,3", help='token ids, e.g. "5,17,3;9,9" for two prompts')
    r.add_argument("--tokens-file", help="one prompt (comma-separated ids) per line")
    r.add_argument("-n", "--n", type=int, default=64, help="max new tokens")
    r.add_argument("--temp", type=float, default=0.0)
    r.add_argument("--top-k", type=int, default=40)
    r.add_argument("--seed", type=int, default=42)
    r.add_argument("--bos", action="store_true", help="prepend the bos token")
    r.add_argument("--ignore-eos", action="store_true")
    r.add_argument("--stop", help="stop token ids (default: the model's eos ids)")
    r.add_argument("--verbose", action="store_true")
    r.add_argument("--profile", help="write a Chrome trace here")
    r.add_argument("--stats", action="store_true")
    r.set_defaults(fn=cmd_run)

    b = sub.add_parser("bench")
    common(b)
    b.add_argument("--prompt-len", type=int, default=128)
    b.add_argument("--gen", type=int, default=64)
    b.add_argument("--reps", type=int, default=3)
    b.add_argument("--batch-sizes", default="1,8", help="sequences per batch (edgelm lists thread counts here)")
    b.add_argument("--json", action="store_true")
    b.set_defaults(fn=cmd_bench)

    i = sub.add_parser("info")
    common(i)
    i.add_argument("--ops", action="store_true", help="list the scheduled layers and their parts")
    i.set_defaults(fn=cmd_info)

    l = sub.add_parser("logits")
    common(l)
    l.add_argument("--tokens", required=True)
    l.add_argument("--prefill", type=int, default=None)
    l.add_argument("--out", default="logits.f32")
    l.set_defaults(fn=cmd_logits)
    return ap


def main(argv=None):
    ap = build_parser()
    args = ap.parse_args(argv)
    if not args.cmd:
        ap.print_help()
        return 0
    try:
        return args.fn(args)
    except (RuntimeError, ValueError, KeyError, OSError) as e:  # as edgelm's main: message, exit code 1
        print(f"edgelm_b200: {e}", file=sys.stderr)
        return 1


if __name__ == "__main__":
    sys.exit(main())
