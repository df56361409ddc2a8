"""The reference arm of bench.py: adarsh-sgh/edgelm itself, unmodified, timed on this machine.

edgelm is a C++17 CPU program (no Python package: `pip install` of its checkout ends with
"Neither 'setup.py' nor 'pyproject.toml' found"), so its own install procedure is used instead:
cmake.  `prepare()` copies its sources into the git-ignored folder `baseline/_ref/edgelm` and builds
`baseline/_ref/build/edgelm` (about 10 s); both travel with the repository's working tree, and a
missing binary is rebuilt from the copied sources where the arm runs.  `run()` then

  1. writes a SmolLM2-135M-shaped model with random float32 weights N(0, 0.02) in edgelm's own
     format with edgelm's own writer (tools/elm.py: build_graph, write_elm) and a placeholder
     tokenizer (the bench command feeds token ids, not text), and
  2. runs edgelm's stock benchmark, `edgelm bench --prompt-len 128 --gen 64 --json`
     (src/main.cpp:173-233: a 128-token prompt, then 64 greedy decode steps, medians).

What it measures is what edgelm can do: float32 on the CPU, one sequence.  It has no GPU path, no
batch above 1 and no bfloat16, so those rows of this library's benchmark have no counterpart.
"""
import json
import os
import shutil
import subprocess
import sys
import tempfile
import time

HERE = os.path.dirname(os.path.abspath(__file__))
REF = os.path.join(HERE, "_ref")
SRC = os.path.join(REF, "edgelm")
BUILD = os.path.join(REF, "build")
BINARY = os.path.join(BUILD, "edgelm")

# config.json keys of the SmolLM2-135M shape -> the names edgelm's exporter uses (tools/export.py:44-54)
SHAPE_135M = dict(vocab=49152, dim=576, hidden=1536, n_layers=30, n_heads=9, n_kv_heads=3, head_dim=64, max_seq=8192,
                  rope_theta=100000.0, norm_eps=1e-5, bos=0, eos=0, tied=True)


class Unavailable(RuntimeError):
    pass


def prepare(checkout="/root/reference", log=None):
    """Sources into baseline/_ref/edgelm (when a checkout is at hand) and the binary built from them."""
    if not os.path.exists(os.path.join(SRC, "CMakeLists.txt")):
        if not os.path.exists(os.path.join(checkout, "CMakeLists.txt")):
            raise Unavailable(f"no copy of edgelm's sources under baseline/_ref and no checkout at {checkout}")
        os.makedirs(REF, exist_ok=True)
        shutil.copytree(checkout, SRC, ignore=shutil.ignore_patterns(".git", "build", "models", "out"))
    if os.path.exists(BINARY):
        return BINARY
    cmake = shutil.which("cmake")
    if cmake is None:
        raise Unavailable("cmake is not installed, and edgelm has no other build")
    for cmd in ([cmake, "-S", SRC, "-B", BUILD, "-DEDGELM_TESTS=OFF", "-DCMAKE_BUILD_TYPE=Release"],
                [cmake, "--build", BUILD, "-j", str(min(16, os.cpu_count() or 2)), "--target", "edgelm_cli"]):
        r = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
        if log:
            log(r.stdout[-2000:])
        if r.returncode != 0:
            raise Unavailable("edgelm's cmake build failed: " + r.stdout.strip().splitlines()[-1][:200])
    if not os.path.exists(BINARY):
        raise Unavailable("edgelm's cmake build produced no binary")
    return BINARY


def write_model(path, shape, seed=0, sigma=0.02):
    """A random model of `shape` as a float32 .elm file, through edgelm's own tools."""
    import numpy as np
    sys.path.insert(0, os.path.join(SRC, "tools"))
    try:
        import elm
    finally:
        sys.path.pop(0)
    rng = np.random.default_rng(seed)
    D, H, V = shape["dim"], shape["hidden"], shape["vocab"]
    qd, kd = shape["n_heads"] * shape["head_dim"], shape["n_kv_heads"] * shape["head_dim"]

    def mat(*s):
        return rng.standard_normal(s, dtype=np.float32) * np.float32(sigma)

    def vec(n):
        return (1 + rng.standard_normal(n, dtype=np.float32) * np.float32(sigma)).astype(np.float32)
    W = {"model.embed_tokens.weight": mat(V, D), "model.norm.weight": vec(D)}
    for l in range(shape["n_layers"]):
        p = f"model.layers.{l}."
        W[p + "input_layernorm.weight"] = vec(D)
        W[p + "post_attention_layernorm.weight"] = vec(D)
        W[p + "self_attn.q_proj.weight"] = mat(qd, D)
        W[p + "self_attn.k_proj.weight"] = mat(kd, D)
        W[p + "self_attn.v_proj.weight"] = mat(kd, D)
        W[p + "self_attn.o_proj.weight"] = mat(D, qd)
        W[p + "mlp.gate_proj.weight"] = mat(H, D)
        W[p + "mlp.up_proj.weight"] = mat(H, D)
        W[p + "mlp.down_proj.weight"] = mat(D, H)
    if not shape["tied"]:
        W["lm_head.weight"] = mat(V, D)
    tok = ([b"<%d>" % i for i in range(V)], [0] * V, [])   # ids in, ids out: the bench command never tokenizes
    return elm.write_elm(path, shape, elm.build_graph(shape, W), tok, "f32")


def run(threads=None, reps=1, prompt_len=128, gen=64):
    """The stock benchmark on a 135M-shaped random model; returns the JSON line's dict."""
    binary = prepare()
    n_cpu = os.cpu_count() or 1
    if threads is None:
        threads = sorted({t for t in (4, 16) if t <= max(4, n_cpu)})
    tmp = tempfile.mkdtemp(prefix="edgelm_ref_")
    try:
        model = os.path.join(tmp, "smollm2-135m-random.f32.elm")
        t0 = time.time()
        size = write_model(model, SHAPE_135M)
        t_write = time.time() - t0
        cmd = [binary, "bench", "-m", model, "--prompt-len", str(prompt_len), "--gen", str(gen), "--reps", str(reps),
               "--threads", ",".join(str(t) for t in threads), "--json"]
        t0 = time.time()
        r = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True, timeout=1500)
        wall = time.time() - t0
        if r.returncode != 0:
            raise Unavailable(f"edgelm bench exited with {r.returncode}: {(r.stderr or r.stdout).strip()[-200:]}")
        rows = [json.loads(l) for l in r.stdout.splitlines() if l.startswith("{")]
        if not rows:
            raise Unavailable("edgelm bench printed no row")
    finally:
        shutil.rmtree(tmp, ignore_errors=True)
    best = max(rows, key=lambda x: x["decode_tok_s"])
    return {
        "metric": "decode tok/s", "value": best["decode_tok_s"], "unit": "tok/s", "n_gpus": 1, "steps": gen, "warmup": 1,
        "ms_per_step": round(1e3 / best["decode_tok_s"], 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": round(best["decode_tok_s"] / 159.3, 4),
        "dtype": "fp32", "data": "synthetic: random weights N(0,0.02), edgelm's own pseudo-random prompt", "impl": "reference",
        "config": {"model": "smollm2-135m", "layers": 30, "device": "cpu (edgelm has no GPU path)", "backend": best["backend"],
                   "simd": best["simd"], "threads": best["threads"], "cpus": n_cpu, "global_batch": 1, "prompt_len": prompt_len,
                   "gen": gen, "seq_len": prompt_len + gen + 8, "parallelism": "single process",
                   "command": "edgelm bench --prompt-len 128 --gen 64 --json (src/main.cpp:173-233)",
                   "no_counterpart": "batch above 1, bfloat16, 2,048-token prompts"},
        "prefill": {"value": best["prefill_tok_s"], "tokens": prompt_len, "ms": best["ttft_ms"]},
        "rows": [{k: row[k] for k in ("threads", "prefill_tok_s", "ttft_ms", "decode_tok_s")} for row in rows],
        "model_file_mb": round(size / 1e6, 1), "write_s": round(t_write, 1), "bench_s": round(wall, 1),
    }


def main():
    try:
        print(json.dumps(run()))
    except Unavailable as e:
        print(json.dumps({"impl": "reference", "unavailable": str(e)}))
    return 0


if __name__ == "__main__":
    if "--prepare" in sys.argv:
        print(prepare(log=print))
    else:
        sys.exit(main())
