"""bin/trace_run as a user runs it: a subprocess fed JSON steps, logits read back from files."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest

import helpers as H

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


class Replay:
    def __init__(self, model_dir, dtype, out_dir, max_tokens):
        self.out = str(out_dir)
        self.p = subprocess.Popen([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", model_dir, "--dtype", dtype,
                                   "--out", self.out, "--max-tokens", str(max_tokens)], stdin=subprocess.PIPE,
                                  stdout=subprocess.PIPE, text=True)
        self.n = 0

    def step(self, entries, end=()):
        rec = {"step": self.n, "entries": entries, "end": list(end)}
        self.p.stdin.write(json.dumps(rec) + "\n")
        self.p.stdin.flush()
        line = self.p.stdout.readline().strip()
        assert line == f"done {self.n}", line
        path = os.path.join(self.out, f"{self.n}.f32")
        self.n += 1
        wanted = sum(len(e["want"]) for e in entries)
        if not wanted:
            assert not os.path.exists(path)
            return None
        return np.fromfile(path, dtype="<f4").reshape(wanted, -1)

    def finish(self):
        self.p.stdin.close()
        assert self.p.wait(timeout=120) == 0


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["tiny_a", "tiny_b"])
def test_replay_modes(tmp_path, name, dtype):
    d = H.make_model_dir(tmp_path, name)
    oracle = H.Oracle(d)
    top = H.TINY[name][0]["max_position_embeddings"]
    lens = [l for l in (70, 3, 128, 33, 200) if l <= top]
    reqs = {f"r{i}": H.tokens_for(name, n, 300 + i) for i, n in enumerate(lens)}
    # room for the three largest rounded up to 64: the batches below never hold more
    room = sum(sorted(((n + 63) // 64 * 64 for n in lens), reverse=True)[:3])
    rp = Replay(d, dtype, tmp_path / "out", room)
    tol = H.TOL[dtype]
    # each request alone and whole
    for rid, toks in reqs.items():
        lg = rp.step([{"id": rid + "w", "tokens": toks, "want": list(range(len(toks)))}], end=[rid + "w"])
        assert H.rel_err(lg, oracle.logits(toks)) < tol
    # the last 32 tokens one by one; nothing wanted from the first step
    for rid, toks in reqs.items():
        head = max(1, len(toks) - 32)
        assert rp.step([{"id": rid + "t", "tokens": toks[:head], "want": []}]) is None
        rows = [rp.step([{"id": rid + "t", "tokens": [t], "want": [0]}]) for t in toks[head:]]
        rp.step([], end=[rid + "t"])
        assert H.rel_err(np.concatenate(rows), oracle.logits(toks)[head:]) < tol
    # batches of unequal lengths that start together; shorter requests end earlier; one batch after another
    ids = list(reqs)
    for b0 in range(0, len(ids), 3):
        batch = ids[b0:b0 + 3]
        fed = {r: max(1, len(reqs[r]) - 5) for r in batch}
        got = {r: [] for r in batch}
        lg = rp.step([{"id": r, "tokens": reqs[r][:fed[r]], "want": [fed[r] - 1]} for r in batch],
                     end=[r for r in batch if fed[r] == len(reqs[r])])
        for i, r in enumerate(batch):
            got[r].append(lg[i:i + 1])
        live = [r for r in batch if fed[r] < len(reqs[r])]
        while live:
            ending = [r for r in live if fed[r] + 1 == len(reqs[r])]
            lg = rp.step([{"id": r, "tokens": [reqs[r][fed[r]]], "want": [0]} for r in live], end=ending)
            for i, r in enumerate(live):
                got[r].append(lg[i:i + 1])
                fed[r] += 1
            live = [r for r in live if r not in ending]
        for r in batch:
            first = max(1, len(reqs[r]) - 5) - 1
            assert H.rel_err(np.concatenate(got[r]), oracle.logits(reqs[r])[first:]) < tol, (r,)
    rp.finish()
