#!/usr/bin/env python3
"""Writes the golden files of this folder from adarsh-sgh/edgelm's own code, on the CPU.

    python tests/golden/make_golden.py --reference /path/to/edgelm

Model: edgelm's NumPy forward (tools/reference.py:72-94) is imported and run on the two tiny
models of golden_models.py; its logits at every position go to tiny_a.npz / tiny_b.npz.
Sampler: edgelm's C++ Sampler (src/tokenizer.cpp:191-211) is compiled with g++ together with
sampler_driver.cpp and draws from fixed logit rows; the token ids go to sampler.npz.
The files are small (tens of KB) and are checked by tests/test_plain.py, which needs neither
edgelm nor a compiler.  This script was run once; it is kept so that the files can be remade.
"""
import argparse
import os
import subprocess
import sys
import tempfile

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, HERE)
import golden_models as gm  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, help="checkout of adarsh-sgh/edgelm")
    args = ap.parse_args()
    sys.path.insert(0, os.path.join(args.reference, "tools"))
    import reference as ref  # edgelm's tools/reference.py

    for name, cfg, n in (("tiny_a", gm.TINY_A, 40), ("tiny_b", gm.TINY_B, 70)):
        W = gm.weights(cfg)
        toks = gm.tokens(cfg, n, cfg["seed"])
        rcfg = dict(n_heads=cfg["n_heads"], n_kv_heads=cfg["n_kv_heads"], head_dim=cfg["head_dim"],
                    norm_eps=cfg["eps"], rope_theta=cfg["theta"], n_layers=cfg["n_layers"], tied=cfg["tied"])
        logits = ref.forward(rcfg, W, toks)
        np.savez_compressed(os.path.join(HERE, name + ".npz"), tokens=toks, logits=logits.astype(np.float32))
        print(name, logits.shape, "max |logit|", float(np.abs(logits).max()))

    with tempfile.TemporaryDirectory() as tmp:
        exe = os.path.join(tmp, "sampler_driver")
        subprocess.run(["g++", "-O1", "-std=c++17", "-I", os.path.join(args.reference, "include"),
                        os.path.join(HERE, "sampler_driver.cpp"),
                        os.path.join(args.reference, "src", "tokenizer.cpp"), "-o", exe], check=True)
        cases, out = [], {}
        for i, (temp, k, seed, vocab) in enumerate([(0.8, 20, 7, 397), (1.0, 40, 42, 256), (0.5, 0, 3, 100),
                                                     (1.3, 1000, 9, 64), (0.0, 40, 1, 397), (0.7, 1, 5, 397)]):
            rows = gm.sampler_logits(24, vocab, i)
            r = subprocess.run([exe, repr(temp), str(k), str(seed), "24", str(vocab)], input=rows.tobytes(),
                               stdout=subprocess.PIPE, check=True)
            ids = np.array([int(x) for x in r.stdout.split()], dtype=np.int64)
            cases.append((temp, k, seed, vocab))
            out[f"ids_{i}"] = ids
        out["cases"] = np.array(cases, dtype=np.float64)
        np.savez_compressed(os.path.join(HERE, "sampler.npz"), **out)
        print("sampler cases", len(cases))


if __name__ == "__main__":
    main()
