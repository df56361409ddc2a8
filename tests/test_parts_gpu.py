"""Each part of a layer alone against the plain implementation, and the framework's openness:
a toy mixer with a state of its own, a toy architecture, a schedule that runs a layer twice;
all defined here, none of them touching the package's files."""
import json
import math

import numpy as np
import pytest
import torch

import helpers as H
import plain_llama as plain

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


class Ctx:
    """The least a part needs from a step: an engine's context filled for given sequences."""

    def __init__(self, engine, seqs):
        from edgelm_b200.engine.engine import StepEntry
        self.engine = engine
        self.slots = engine.open(len(seqs))
        self.entries = [StepEntry(s, t, list(range(len(t)))) for s, t in zip(self.slots, seqs)]


def build_part(role, spec, dtype, tensors, prefix=""):
    from edgelm_b200.parts.registry import BuildEnv
    part = BuildEnv(dtype=dtype).build(role, spec)
    part.load(tensors, prefix, DEV)
    return part


def null_ctx(n_tokens=0):
    from edgelm_b200.engine.arena import Workspace
    from edgelm_b200.engine.batch import StepContext
    ws = Workspace(1 << 24, torch.device(DEV))
    err = torch.zeros(1, dtype=torch.int32, device=DEV)
    return StepContext(ws, err, torch.device(DEV), 148)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_norm_embedding_head_swiglu_alone(dtype):
    from edgelm_b200.config.base import PartSpec
    g = torch.Generator().manual_seed(5)
    D, I, V, T = 88, 136, 301, 37
    tol = 2e-5 if dtype == torch.float32 else 2e-2
    ctx = null_ctx()
    # norm
    w = (1 + 0.1 * torch.randn(D, generator=g))
    x = torch.randn(T, D, generator=g) * 2
    norm = build_part("norm", PartSpec("rmsnorm", {"dim": D, "eps": 1e-4, "name": "n.weight"}), dtype, {"p.n.weight": w}, "p.")
    out = torch.empty(T, D, dtype=dtype, device=DEV)
    norm.forward(ctx, x.to(DEV), out)
    assert H.rel_err(out.float().cpu().numpy(), plain.rmsnorm(x.numpy(), w.numpy(), 1e-4)) < tol
    # embedding
    table = torch.randn(V, D, generator=g).to(dtype)
    emb = build_part("embedding", PartSpec("embedding", {"vocab_size": V, "dim": D, "name": "e"}), dtype, {"e": table})
    ctx.token_ids = torch.tensor([0, V - 1, 7], dtype=torch.int32, device=DEV)
    xe = torch.empty(3, D, device=DEV)
    emb.forward(ctx, xe)
    assert np.array_equal(xe.cpu().numpy(), plain.embed(table.float().numpy(), [0, V - 1, 7]))
    # head, untied and tied
    hw = (torch.randn(V, D, generator=g) * 0.1).to(dtype)
    head = build_part("head", PartSpec("lm_head", {"vocab_size": V, "dim": D, "tied_to": None, "name": "h"}), dtype, {"h": hw})
    xn = torch.randn(T, D, generator=g).to(dtype)
    logits = torch.empty(T, V, device=DEV)
    head.forward(ctx, xn.to(DEV), logits)
    assert H.rel_err(logits.cpu().numpy(), xn.float().numpy() @ hw.float().numpy().T) < 2e-5
    # feed-forward, many rows (tile / tensor-core kernels) and few (decode kernels)
    wg, wu, wd = [(torch.randn(*s, generator=g) * 0.1).to(dtype) for s in ((I, D), (I, D), (D, I))]
    ffn = build_part("ffn", PartSpec("swiglu", {"hidden_size": D, "intermediate_size": I,
                                                 "names": {"gate": "g", "up": "u", "down": "d"}}), dtype,
                     {"p.g": wg, "p.u": wu, "p.d": wd}, "p.")
    for rows in (T, 3):
        h = torch.randn(rows, D, generator=g).to(dtype)
        xr = torch.randn(rows, D, generator=g)
        xd = xr.clone().to(DEV)
        ctx.ws.reset()
        ffn.forward(ctx, h.to(DEV), xd)
        want = xr.numpy() + plain.swiglu_mlp(h.float().numpy(), wg.float().numpy(), wu.float().numpy(), wd.float().numpy())
        assert H.rel_err(xd.cpu().numpy(), want) < tol


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_rope_table_and_attention_alone(dtype, tmp_path):
    """The attention mixer through a one-layer model whose feed-forward weights are zero: what comes
    out of the layer is x + attention(x), prompt in one step and token by token."""
    from edgelm_b200.engine.engine import Engine, StepEntry, load_model
    from edgelm_b200.weights import read_dir, write_file
    cfg = dict(H.TINY_B, num_hidden_layers=1, num_attention_heads=6, num_key_value_heads=2, head_dim=16, hidden_size=48,
               intermediate_size=24, vocab_size=61, rope_theta=500.0)
    from edgelm_b200 import write_model_dir
    from edgelm_b200.config import config_class_for
    d = write_model_dir(str(tmp_path / "m"), config_class_for(cfg).from_dict(cfg), seed=4, sigma=0.2, dtype="float32")
    t = dict(read_dir(d))
    t["model.layers.0.mlp.down_proj.weight"] = torch.zeros_like(t["model.layers.0.mlp.down_proj.weight"])
    write_file(str(tmp_path / "m" / "model.safetensors"), {k: v.clone() for k, v in t.items()})
    model = load_model(d, "float32" if dtype == torch.float32 else "bfloat16")
    rope = model.layers[0].mixer.positions
    c, s = plain.rope_angles(np.arange(cfg["max_position_embeddings"]), 16, 500.0)
    assert np.array_equal(rope.cos.cpu().numpy(), c) and np.array_equal(rope.sin.cpu().numpy(), s)  # float64 angles, then float32
    eng = Engine(model, max_tokens=256)
    pcfg, W = plain.read_model(d)
    toks = [int(v) for v in np.random.default_rng(3).integers(0, 61, size=90)]
    want = plain.forward(pcfg, W, toks)
    tol = 2e-5 if dtype == torch.float32 else 3e-2
    assert H.rel_err(H.run_whole(eng, toks), want) < tol
    assert H.rel_err(H.run_tail_one_by_one(eng, toks, 40), want) < tol


# ----------------------------------------------------------------------------- a toy mixer with a state of its own
def _register_toy():
    """A mixer that keeps one vector per sequence: s <- decay * s + h_t; output s W^T.  Torch ops
    on the device, token by token: a toy to show the interfaces, not a kernel."""
    from edgelm_b200.config import register_architecture
    from edgelm_b200.config.base import LayerSpec, ModelPlan, PartSpec, ScheduleEntry
    from edgelm_b200.parts import Part, StateNeed, register_mixer
    from edgelm_b200.parts.registry import MIXERS

    if "toy_decay_state" in MIXERS:
        return

    @register_mixer("toy_decay_state")
    class ToyStateMixer(Part):
        def __init__(self, spec, env):
            self.dim, self.decay, self.name = spec["dim"], float(spec["decay"]), spec["name"]
            self.w = None

        def weight_shapes(self, prefix):
            return {prefix + self.name: (self.dim, self.dim)}

        def load(self, tensors, prefix, device):
            self.w = tensors[prefix + self.name].to(device=device, dtype=torch.float32)

        def cache_need(self):
            return StateNeed((self.dim,))

        def forward(self, ctx, h, x, cache):
            state = cache.state                      # [slots, dim] float32, zero when a sequence starts
            slots = ctx.seq_slots.long()
            t0 = 0
            for i, n in enumerate(ctx.seq_lengths):
                s = state.index_select(0, slots[i:i + 1])[0]     # (indexing by a device tensor: nothing is read on the host)
                for t in range(t0, t0 + n):
                    s = self.decay * s + h[t].float()
                    x[t] += s @ self.w.T
                state.index_copy_(0, slots[i:i + 1], s[None])
                t0 += n

    @register_mixer("toy_decay_state_replayable")
    class ToyStateMixerReplayable(ToyStateMixer):
        # Nothing in `forward` reads device data on the host (the slots are indexed as device tensors, the loops run
        # over the step's shape, which a captured graph is keyed by): steps through it may be replayed from a graph.
        graph_safe = True

    @register_architecture("ToyStateForCausalLM", model_type="toy_state")
    class ToyConfig:
        def __init__(self, d):
            self.d = d

        @classmethod
        def from_dict(cls, d):
            return cls(d)

        def plan(self):
            d = self.d
            D, V = d["width"], d["vocab_size"]
            norm = lambda name: PartSpec("rmsnorm", {"dim": D, "eps": d["eps"], "name": name})
            toy = PartSpec("toy_decay_state_replayable" if d.get("replayable") else "toy_decay_state",
                           {"dim": D, "decay": d["decay"], "name": "mix.weight"})
            att = PartSpec("attention", {"hidden_size": D, "num_heads": 2, "num_kv_heads": 1, "head_dim": 16,
                                         "positions": PartSpec("rope", {"head_dim": 16, "theta": 1000.0, "max_positions": 128}),
                                         "names": {"q": "q.weight", "k": "k.weight", "v": "v.weight", "o": "o.weight"}})
            ffn = PartSpec("swiglu", {"hidden_size": D, "intermediate_size": d["inner"],
                                      "names": {"gate": "g.weight", "up": "u.weight", "down": "d.weight"}})
            layers = (LayerSpec("l0.", "prenorm", toy, norm("n1.weight"), ffn, norm("n2.weight")),
                      LayerSpec("l1.", "prenorm", att, norm("n1.weight"), ffn, norm("n2.weight")))
            # the state layer runs twice (each run has a state of its own), with the attention layer between
            schedule = (ScheduleEntry(0), ScheduleEntry(1), ScheduleEntry(0))
            return ModelPlan(hidden_size=D, vocab_size=V, max_positions=128,
                             embedding=PartSpec("embedding", {"vocab_size": V, "dim": D, "name": "emb.weight"}),
                             layers=layers, schedule=schedule, final_norm=norm("final.weight"),
                             head=PartSpec("lm_head", {"vocab_size": V, "dim": D, "tied_to": "emb.weight", "name": "head.weight"}))


def _toy_plain(W, d, tokens):
    """The toy model in plain NumPy: whole sequence, no cache."""
    D = d["width"]

    def toy_layer(x):
        h = plain.rmsnorm(x, W["l0.n1.weight"], d["eps"])
        s = np.zeros(D, dtype=np.float32)
        out = x.copy()
        for t in range(len(x)):
            s = np.float32(d["decay"]) * s + h[t]
            out[t] += s @ W["l0.mix.weight"].T
        h2 = plain.rmsnorm(out, W["l0.n2.weight"], d["eps"])
        return out + plain.swiglu_mlp(h2, W["l0.g.weight"], W["l0.u.weight"], W["l0.d.weight"])

    def att_layer(x):
        h = plain.rmsnorm(x, W["l1.n1.weight"], d["eps"])
        pos = np.arange(len(x))
        q = plain.rope(h @ W["l1.q.weight"].T, pos, 2, 16, 1000.0)
        k = plain.rope(h @ W["l1.k.weight"].T, pos, 1, 16, 1000.0)
        a = plain.attention(q, k, h @ W["l1.v.weight"].T, 2, 1, 16)
        x = x + a @ W["l1.o.weight"].T
        h2 = plain.rmsnorm(x, W["l1.n2.weight"], d["eps"])
        return x + plain.swiglu_mlp(h2, W["l1.g.weight"], W["l1.u.weight"], W["l1.d.weight"])

    x = plain.embed(W["emb.weight"], tokens)
    x = toy_layer(att_layer(toy_layer(x)))
    return plain.rmsnorm(x, W["final.weight"], d["eps"]) @ W["emb.weight"].T


def test_toy_mixer_with_state_registers_builds_and_steps(tmp_path):
    _register_toy()
    from edgelm_b200.config import read_config, registered_architectures
    from edgelm_b200.engine.engine import Engine, load_model
    from edgelm_b200.engine.model import expected_weights
    from edgelm_b200.weights import random_tensors, write_file
    assert "ToyStateForCausalLM" in registered_architectures()
    d = {"architectures": ["ToyStateForCausalLM"], "vocab_size": 53, "width": 40, "inner": 56, "eps": 1e-5, "decay": 0.8}
    folder = tmp_path / "toy"
    folder.mkdir()
    (folder / "config.json").write_text(json.dumps(d))
    cfg = read_config(str(folder))
    exp = expected_weights(cfg.plan())
    assert exp["l0.mix.weight"] == (40, 40) and "head.weight" not in exp
    write_file(str(folder / "model.safetensors"), random_tensors(exp, seed=9, sigma=0.15, dtype=torch.float32))
    model = load_model(str(folder), "float32")
    eng = Engine(model, max_tokens=512)
    assert len(eng.cache.state_groups) == 1 and eng.cache.state_groups[0].n_entries == 2  # two runs, two states
    assert len(eng.cache.kv_groups) == 1 and eng.cache.kv_groups[0].n_entries == 1
    W = {k: v.float().numpy() for k, v in __import__("edgelm_b200.weights", fromlist=["read_dir"]).read_dir(str(folder)).items()}
    reqs = [[int(v) for v in np.random.default_rng(i).integers(0, 53, size=n)] for i, n in enumerate([20, 7, 70, 33])]
    for r in reqs:
        want = _toy_plain(W, d, r)
        assert H.rel_err(H.run_whole(eng, r), want) < 5e-5
        assert H.rel_err(H.run_tail_one_by_one(eng, r, 10), want) < 5e-5
    # unequal batches on reused slots: a slot's state starts from zero again
    got = H.run_batches(eng, reqs, batch_size=2, decode_tail=5)
    for r, g in zip(reqs, got):
        assert H.rel_err(g, _toy_plain(W, d, r)) < 5e-5
    eng.cache.check()


def _toy_folder(tmp_path, name="toy", **extra):
    from edgelm_b200.config import read_config
    from edgelm_b200.engine.model import expected_weights
    from edgelm_b200.weights import random_tensors, read_dir, write_file
    d = {"architectures": ["ToyStateForCausalLM"], "vocab_size": 53, "width": 40, "inner": 56, "eps": 1e-5, "decay": 0.8, **extra}
    folder = tmp_path / name
    folder.mkdir()
    (folder / "config.json").write_text(json.dumps(d))
    exp = expected_weights(read_config(str(folder)).plan())
    write_file(str(folder / "model.safetensors"), random_tensors(exp, seed=9, sigma=0.15, dtype=torch.float32))
    W = {k: v.float().numpy() for k, v in read_dir(str(folder)).items()}
    return d, str(folder), W


def _toy_greedy(W, d, prompt, n):
    seq, out = list(prompt), []
    for _ in range(n):
        out.append(int(np.argmax(_toy_plain(W, d, seq)[-1])))
        seq.append(out[-1])
    return out


def test_a_state_mixer_that_allows_graphs_advances_its_state_once(tmp_path):
    """Decode steps of a model whose mixer keeps a fixed-size state are captured like any other (one eager run, then
    the capture, then the replay, all in the step that meets a batch size first): the state must move once in that
    step.  Greedy generation through the entry point against the plain toy model."""
    _register_toy()
    import edgelm_b200
    d, folder, W = _toy_folder(tmp_path, replayable=True)
    eng = edgelm_b200.load_engine(folder, dtype="float32", ctx=128, slots=3)
    assert eng.use_graphs and eng.cache.state_groups
    prompts = [[5, 17, 3, 44], [9], [int(v) for v in np.random.default_rng(1).integers(0, 53, size=40)]]
    got = edgelm_b200.generate(None, prompts, n=10, engine=eng, slots=3, stop=[], ignore_eos=True)
    assert eng._graphs, "the decode steps were not captured"
    assert got == [_toy_greedy(W, d, p, 10) for p in prompts]
    # a prompt step whose shape comes back is captured too (at its second appearance), on the state of fresh slots
    from edgelm_b200.engine.engine import StepEntry
    long = [[int(v) for v in np.random.default_rng(10 + i).integers(0, 53, size=50)] for i in range(3)]
    for r in long:
        slot = eng.open(1)[0]
        lg = eng.step([StepEntry(slot, r, list(range(50)))]).cpu().numpy()
        lg2 = eng.step([StepEntry(slot, [7], [0])]).cpu().numpy()
        eng.close([slot])
        assert H.rel_err(np.concatenate([lg, lg2]), _toy_plain(W, d, r + [7])) < 5e-5
    assert ((50,), 50) in eng._step_graphs


def test_a_toy_architecture_through_every_program(tmp_path, capsys):
    """run, info, bench and logits of the command line, and bin/trace_run as its own process, on the folder of an
    architecture that only this test file knows: none of them reads an architecture's configuration fields."""
    import os
    import subprocess
    import sys
    _register_toy()
    from edgelm_b200.cli import main
    d, folder, W = _toy_folder(tmp_path)
    assert main(["info", "-m", folder, "--ops", "--dtype", "f32"]) == 0
    out = capsys.readouterr().out
    assert "ToyConfig" in out and "toy_decay_state(" in out and "fixed-size state of 2 layer run(s)" in out and "keys/values of 1 layer run(s)" in out
    toks = [int(v) for v in np.random.default_rng(5).integers(0, 53, size=14)]
    path = str(tmp_path / "lg.f32")
    assert main(["logits", "-m", folder, "--dtype", "f32", "--tokens", ",".join(map(str, toks)), "--prefill", "6", "--out", path]) == 0
    assert H.rel_err(np.fromfile(path, dtype="<f4").reshape(14, -1), _toy_plain(W, d, toks)) < 5e-5
    capsys.readouterr()
    assert main(["run", "-m", folder, "--dtype", "f32", "-p", "5,17,3;9", "-n", "5", "--ignore-eos", "--verbose"]) == 0
    out = capsys.readouterr().out
    assert "5,17,3 => " + ",".join(map(str, _toy_greedy(W, d, [5, 17, 3], 5))) in out and "9 => " + ",".join(map(str, _toy_greedy(W, d, [9], 5))) in out
    assert main(["bench", "-m", folder, "--dtype", "f32", "--prompt-len", "12", "--gen", "3", "--reps", "1", "--batch-sizes", "2", "--json"]) == 0
    row = json.loads(capsys.readouterr().out.strip().splitlines()[-1])
    assert row["batch"] == 2 and row["decode_tok_s"] > 0
    # the replay program in a process of its own learns the architecture from a plugin named in the environment
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    env = dict(os.environ, EDGELM_B200_PLUGINS="test_parts_gpu:_register_toy",
               PYTHONPATH=os.pathsep.join([os.path.dirname(os.path.abspath(__file__)), root, os.environ.get("PYTHONPATH", "")]))
    outdir = tmp_path / "replay"
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": toks[:9], "want": list(range(9))}], "end": []}]
    steps += [{"step": i + 1, "entries": [{"id": "a", "tokens": [t], "want": [0]}], "end": ["a"] if i == 4 else []} for i, t in enumerate(toks[9:])]
    r = subprocess.run([sys.executable, os.path.join(root, "bin", "trace_run"), "--model", folder, "--dtype", "float32", "--out", str(outdir),
                        "--max-tokens", "64"], input="\n".join(json.dumps(s) for s in steps) + "\n", text=True, capture_output=True, env=env, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    assert [l for l in r.stdout.splitlines() if l.startswith("done")] == [f"done {i}" for i in range(6)]
    got = np.concatenate([np.fromfile(outdir / f"{i}.f32", dtype="<f4").reshape(-1, 53) for i in range(6)])
    assert H.rel_err(got, _toy_plain(W, d, toks)) < 5e-5


# ----------------------------------------------------------------------------- layers with a window beside layers without
def _register_windowed():
    """A toy architecture whose layers use the package's own attention, some with a window: two cache groups with
    different needs (every key; the last keys), each with storage of its own."""
    from edgelm_b200.config import register_architecture
    from edgelm_b200.config.base import LayerSpec, ModelPlan, PartSpec, ScheduleEntry
    from edgelm_b200.config.registry import registered_architectures

    if "ToyWindowedForCausalLM" in registered_architectures():
        return

    @register_architecture("ToyWindowedForCausalLM", model_type="toy_windowed")
    class ToyWindowedConfig:
        def __init__(self, d):
            self.d = d

        @classmethod
        def from_dict(cls, d):
            return cls(d)

        def plan(self):
            d = self.d
            D, V, hd = d["width"], d["vocab_size"], d["head_dim"]
            norm = lambda name: PartSpec("rmsnorm", {"dim": D, "eps": 1e-5, "name": name})
            rope = PartSpec("rope", {"head_dim": hd, "theta": 2000.0, "max_positions": d["positions"]})
            names = {"q": "q.weight", "k": "k.weight", "v": "v.weight", "o": "o.weight"}
            att = lambda w: PartSpec("attention", {"hidden_size": D, "num_heads": d["heads"], "num_kv_heads": d["kv_heads"], "head_dim": hd,
                                                   "positions": rope, "names": names, **({"window": w} if w else {})})
            ffn = PartSpec("swiglu", {"hidden_size": D, "intermediate_size": d["inner"],
                                      "names": {"gate": "g.weight", "up": "u.weight", "down": "d.weight"}})
            layers = tuple(LayerSpec(f"l{i}.", "prenorm", att(w), norm("n1.weight"), ffn, norm("n2.weight")) for i, w in enumerate(d["windows"]))
            return ModelPlan(hidden_size=D, vocab_size=V, max_positions=d["positions"],
                             embedding=PartSpec("embedding", {"vocab_size": V, "dim": D, "name": "emb.weight"}),
                             layers=layers, schedule=tuple(ScheduleEntry(i) for i in range(len(layers))), final_norm=norm("final.weight"),
                             head=PartSpec("lm_head", {"vocab_size": V, "dim": D, "tied_to": "emb.weight", "name": "head.weight"}))


def _windowed_plain(W, d, tokens):
    """The toy model in plain NumPy: whole sequence, no cache; a windowed layer masks the keys before its window."""
    nh, nkv, hd = d["heads"], d["kv_heads"], d["head_dim"]
    x = plain.embed(W["emb.weight"], tokens)
    T = len(tokens)
    pos = np.arange(T)
    for i, w in enumerate(d["windows"]):
        p = f"l{i}."
        h = plain.rmsnorm(x, W[p + "n1.weight"], 1e-5)
        q = plain.rope(h @ W[p + "q.weight"].T, pos, nh, hd, 2000.0).reshape(T, nh, hd)
        k = plain.rope(h @ W[p + "k.weight"].T, pos, nkv, hd, 2000.0).reshape(T, nkv, hd)
        v = (h @ W[p + "v.weight"].T).reshape(T, nkv, hd)
        a = np.zeros((T, nh, hd), dtype=np.float32)
        hidden = pos[None, :] > pos[:, None]
        if w:
            hidden = hidden | (pos[None, :] < pos[:, None] - w + 1)
        for hh in range(nh):
            sc = (q[:, hh] @ k[:, hh // (nh // nkv)].T).astype(np.float32) * np.float32(1.0 / math.sqrt(hd))
            sc[hidden] = -np.inf
            sc = sc - sc.max(axis=1, keepdims=True)
            pr = np.exp(sc).astype(np.float32)
            a[:, hh] = (pr / pr.sum(axis=1, keepdims=True)) @ v[:, hh // (nh // nkv)]
        x = (x + a.reshape(T, nh * hd) @ W[p + "o.weight"].T).astype(np.float32)
        h2 = plain.rmsnorm(x, W[p + "n2.weight"], 1e-5)
        x = (x + plain.swiglu_mlp(h2, W[p + "g.weight"], W[p + "u.weight"], W[p + "d.weight"])).astype(np.float32)
    return plain.rmsnorm(x, W["final.weight"], 1e-5) @ W["emb.weight"].T


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("shape", [dict(width=48, heads=4, kv_heads=2, head_dim=16, inner=72, windows=[40, 0, 100]),
                                   dict(width=64, heads=2, kv_heads=1, head_dim=64, inner=96, windows=[0, 70])])
def test_windowed_layers_beside_full_ones(tmp_path, dtype, shape):
    """Whole prompts (cut into pieces by the engine so that a windowed group holds its window and one piece), the last
    tokens one by one far beyond the window (pages are given back on the way), unequal batches on reused slots."""
    _register_windowed()
    from edgelm_b200.config import read_config
    from edgelm_b200.engine.engine import Engine, load_model
    from edgelm_b200.engine.model import expected_weights
    from edgelm_b200.weights import random_tensors, read_dir, write_file
    d = {"architectures": ["ToyWindowedForCausalLM"], "vocab_size": 97, "positions": 700, **shape}
    folder = tmp_path / "win"
    folder.mkdir()
    (folder / "config.json").write_text(json.dumps(d))
    exp = expected_weights(read_config(str(folder)).plan())
    write_file(str(folder / "model.safetensors"), random_tensors(exp, seed=21, sigma=0.12, dtype=torch.bfloat16))
    W = {k: v.float().numpy() for k, v in read_dir(str(folder)).items()}
    eng = Engine(load_model(str(folder), dtype), max_tokens=64 * 30, max_seqs=4)
    groups = {g.window: g for g in eng.cache.kv_groups}
    assert len(groups) == len(set(shape["windows"])) and None in groups            # a group per need
    for w, g in groups.items():
        if w:
            assert g.n_pages == 4 * g.pages_per_seq < groups[None].n_pages          # storage of its own, sized by the window
    tol = H.TOL[dtype]
    reqs = [[int(v) for v in np.random.default_rng(40 + i).integers(0, 97, size=n)] for i, n in enumerate([650, 30, 257, 129, 64, 300])]
    want = [_windowed_plain(W, d, r) for r in reqs]
    for r, wnt in list(zip(reqs, want))[:3]:
        assert H.rel_err(H.run_whole(eng, r), wnt) < tol, len(r)
        assert H.rel_err(H.run_tail_one_by_one(eng, r, min(len(r) - 1, 200)), wnt) < tol, len(r)
        eng.cache.check()
    got = H.run_batches(eng, reqs, batch_size=3, decode_tail=20)
    for r, g_, wnt in zip(reqs, got, want):
        assert H.rel_err(g_, wnt) < tol, len(r)
    eng.cache.check()
    assert all(g.pool.available() == g.n_pages for g in eng.cache.kv_groups)
    eng.check_device_errors()
    # generation (captured decode steps) equals the plain model's greedy choice
    import edgelm_b200
    if dtype == "float32":
        out = edgelm_b200.generate(None, [reqs[1], reqs[4]], n=60, engine=eng, slots=2, stop=[], ignore_eos=True)
        for p, o_ in zip([reqs[1], reqs[4]], out):
            lg = _windowed_plain(W, d, p + o_[:-1])
            assert [int(np.argmax(lg[len(p) - 1 + j])) for j in range(60)] == o_


# ----------------------------------------------------------------------------- a toy feed-forward with routing, a toy position encoding
def _register_toy_routed():
    """A feed-forward that sends every token to one of a few small experts (the router's first maximum) and scales
    the expert's output by the router's softmax weight, and a rotary encoding whose positions are divided by a
    factor.  Torch ops and the package's own rotation kernel; toys to show the interfaces."""
    from edgelm_b200.config import register_architecture
    from edgelm_b200.config.base import LayerSpec, ModelPlan, PartSpec, ScheduleEntry
    from edgelm_b200.csrc import ops
    from edgelm_b200.parts import Part, register_ffn, register_positions
    from edgelm_b200.parts.registry import FEED_FORWARDS

    if "toy_top1_experts" in FEED_FORWARDS:
        return

    @register_ffn("toy_top1_experts")
    class ToyRoutedFeedForward(Part):
        def __init__(self, spec, env):
            self.dim, self.inner, self.n_experts = spec["dim"], spec["inner"], spec["experts"]

        def weight_shapes(self, prefix):
            shapes = {prefix + "router.weight": (self.n_experts, self.dim)}
            for e in range(self.n_experts):
                shapes[prefix + f"experts.{e}.in.weight"] = (self.inner, self.dim)
                shapes[prefix + f"experts.{e}.out.weight"] = (self.dim, self.inner)
            return shapes

        def load(self, tensors, prefix, device):
            f = lambda name: tensors[prefix + name].to(device=device, dtype=torch.float32)
            self.router = f("router.weight")
            self.w_in = [f(f"experts.{e}.in.weight") for e in range(self.n_experts)]
            self.w_out = [f(f"experts.{e}.out.weight") for e in range(self.n_experts)]

        def forward(self, ctx, h, x):
            hf = h.float()
            logits = hf @ self.router.T                       # float32 router logits
            chosen = logits.argmax(dim=1)
            weight = torch.softmax(logits, dim=1).gather(1, chosen[:, None])
            for e in range(self.n_experts):
                y = torch.nn.functional.silu(hf @ self.w_in[e].T) @ self.w_out[e].T
                x += torch.where((chosen == e)[:, None], y * weight, torch.zeros_like(y))

    @register_positions("toy_interpolated_rope")
    class InterpolatedRotaryPositions(Part):
        def __init__(self, spec, env):
            self.head_dim, self.theta, self.factor = spec["head_dim"], float(spec["theta"]), float(spec["factor"])
            self.max_positions = spec["max_positions"]
            self.cos = self.sin = None

        def load(self, tensors, prefix, device):
            i = torch.arange(0, self.head_dim, 2, dtype=torch.float64)
            inv = torch.pow(torch.tensor(self.theta, dtype=torch.float64), -(i / self.head_dim))
            ang = (torch.arange(self.max_positions, dtype=torch.float64) / self.factor)[:, None] * inv[None, :]
            self.cos = torch.cos(ang).to(torch.float32).to(device).contiguous()
            self.sin = torch.sin(ang).to(torch.float32).to(device).contiguous()

        def rotation_tables(self):
            return self.cos, self.sin

        def encode_and_append(self, ctx, qkv, cache, n_heads, n_kv_heads):
            ops.rope_kv_append(qkv, ctx.tok_pos, ctx.tok_seq, ctx.seq_index, ctx.page_table(cache.group), self.cos, self.sin,
                               cache.k, cache.v, n_heads, n_kv_heads, self.head_dim, ctx.err)

    @register_architecture("ToyRoutedForCausalLM", model_type="toy_routed")
    class ToyRoutedConfig:
        def __init__(self, d):
            self.d = d

        @classmethod
        def from_dict(cls, d):
            return cls(d)

        def plan(self):
            d = self.d
            D, V = d["width"], d["vocab_size"]
            norm = lambda name: PartSpec("rmsnorm", {"dim": D, "eps": d["eps"], "name": name})

            def att(positions):
                return PartSpec("attention", {"hidden_size": D, "num_heads": 3, "num_kv_heads": 1, "head_dim": 16, "positions": positions,
                                              "names": {"q": "q.weight", "k": "k.weight", "v": "v.weight", "o": "o.weight"}})
            squeezed = PartSpec("toy_interpolated_rope", {"head_dim": 16, "theta": 1000.0, "factor": d["factor"], "max_positions": 128})
            rope = PartSpec("rope", {"head_dim": 16, "theta": 1000.0, "max_positions": 128})
            routed = PartSpec("toy_top1_experts", {"dim": D, "inner": d["inner"], "experts": d["experts"]})
            dense = PartSpec("swiglu", {"hidden_size": D, "intermediate_size": d["inner"],
                                        "names": {"gate": "g.weight", "up": "u.weight", "down": "d.weight"}})
            # two layers with different position encodings and different feed-forwards
            layers = (LayerSpec("l0.", "prenorm", att(squeezed), norm("n1.weight"), routed, norm("n2.weight")),
                      LayerSpec("l1.", "prenorm", att(rope), norm("n1.weight"), dense, norm("n2.weight")))
            return ModelPlan(hidden_size=D, vocab_size=V, max_positions=128,
                             embedding=PartSpec("embedding", {"vocab_size": V, "dim": D, "name": "emb.weight"}),
                             layers=layers, schedule=(ScheduleEntry(0), ScheduleEntry(1)), final_norm=norm("final.weight"),
                             head=PartSpec("lm_head", {"vocab_size": V, "dim": D, "tied_to": "emb.weight", "name": "head.weight"}))


def _toy_routed_plain(W, d, tokens):
    """The toy model in plain NumPy: whole sequence, no cache."""
    n = len(tokens)

    def att(x, p, positions):
        h = plain.rmsnorm(x, W[p + "n1.weight"], d["eps"])
        q = plain.rope(h @ W[p + "q.weight"].T, positions, 3, 16, 1000.0)
        k = plain.rope(h @ W[p + "k.weight"].T, positions, 1, 16, 1000.0)
        return x + plain.attention(q, k, h @ W[p + "v.weight"].T, 3, 1, 16) @ W[p + "o.weight"].T

    x = plain.embed(W["emb.weight"], tokens)
    x = att(x, "l0.", np.arange(n) / d["factor"])
    h = plain.rmsnorm(x, W["l0.n2.weight"], d["eps"])
    logits = h @ W["l0.router.weight"].T
    out = x.copy()
    for t in range(n):
        e = int(np.argmax(logits[t]))
        p = np.exp(logits[t] - logits[t].max())
        y = plain.silu(h[t] @ W[f"l0.experts.{e}.in.weight"].T) @ W[f"l0.experts.{e}.out.weight"].T
        out[t] += y * np.float32(p[e] / p.sum())
    x = att(out, "l1.", np.arange(n))
    h = plain.rmsnorm(x, W["l1.n2.weight"], d["eps"])
    x = x + plain.swiglu_mlp(h, W["l1.g.weight"], W["l1.u.weight"], W["l1.d.weight"])
    return plain.rmsnorm(x, W["final.weight"], d["eps"]) @ W["emb.weight"].T


def test_toy_routed_feed_forward_and_position_encoding_register_build_and_step(tmp_path):
    _register_toy_routed()
    from edgelm_b200.config import read_config
    from edgelm_b200.engine.engine import Engine, load_model
    from edgelm_b200.engine.model import expected_weights
    from edgelm_b200.weights import random_tensors, read_dir, write_file
    d = {"architectures": ["ToyRoutedForCausalLM"], "vocab_size": 47, "width": 24, "inner": 40, "experts": 3, "eps": 1e-6, "factor": 2.5}
    folder = tmp_path / "toy_routed"
    folder.mkdir()
    (folder / "config.json").write_text(json.dumps(d))
    exp = expected_weights(read_config(str(folder)).plan())
    assert exp["l0.router.weight"] == (3, 24) and exp["l0.experts.2.out.weight"] == (24, 40) and "l1.router.weight" not in exp
    tensors = random_tensors(exp, seed=3, sigma=0.2, dtype=torch.float32)
    tensors["l0.router.weight"] = tensors["l0.router.weight"] * 6.0   # clear choices: no token sits on the fence between two experts
    write_file(str(folder / "model.safetensors"), tensors)
    model = load_model(str(folder), "float32")
    assert type(model.layers[0].mixer.positions).__name__ == "InterpolatedRotaryPositions"
    assert type(model.layers[1].mixer.positions).__name__ == "RotaryPositions"
    eng = Engine(model, max_tokens=512)
    W = {k: v.float().numpy() for k, v in read_dir(str(folder)).items()}
    reqs = [[int(v) for v in np.random.default_rng(10 + i).integers(0, 47, size=n)] for i, n in enumerate([26, 5, 90, 41])]
    used = set()
    for r in reqs:
        want = _toy_routed_plain(W, d, r)
        assert H.rel_err(H.run_whole(eng, r), want) < 5e-5
        assert H.rel_err(H.run_tail_one_by_one(eng, r, 12), want) < 5e-5
        h = plain.rmsnorm(plain.embed(W["emb.weight"], r), W["l0.n1.weight"], d["eps"])
        used |= set(np.argmax(h @ W["l0.router.weight"].T, axis=1).tolist())
    assert len(used) > 1   # (a rough check on the first norm's output that the router does not send everything one way)
    got = H.run_batches(eng, reqs, batch_size=3, decode_tail=6)
    for r, g in zip(reqs, got):
        assert H.rel_err(g, _toy_routed_plain(W, d, r)) < 5e-5
    eng.cache.check()


def test_cli_commands(tmp_path, capsys):
    from edgelm_b200.cli import main
    d = H.make_model_dir(tmp_path, "tiny_a")
    o = H.Oracle(d)
    assert main(["info", "-m", d, "--ops", "--dtype", "f32"]) == 0
    out = capsys.readouterr().out
    assert "cache   :" in out and "keys/values of 2 layer run(s)" in out and "attention(heads 4, kv_heads 2, head_dim 16" in out and "swiglu(intermediate 128)" in out
    toks = H.tokens_for("tiny_a", 12, 400)
    path = str(tmp_path / "lg.f32")
    assert main(["logits", "-m", d, "--dtype", "f32", "--tokens", ",".join(map(str, toks)), "--prefill", "5", "--out", path]) == 0
    lg = np.fromfile(path, dtype="<f4").reshape(12, -1)
    assert H.rel_err(lg, o.logits(toks)) < 2e-5
    capsys.readouterr()
    trace = str(tmp_path / "t.json")
    assert main(["run", "-m", d, "--dtype", "f32", "-p", "5,17,3;9", "-n", "6", "--ignore-eos", "--profile", trace, "--stats"]) == 0
    out = capsys.readouterr().out
    want = [plain.generate(o.cfg, o.W, p, 6, stop_ids=[], ignore_eos=True) for p in ([5, 17, 3], [9])]
    assert "5,17,3 => " + ",".join(map(str, want[0])) in out and "9 => " + ",".join(map(str, want[1])) in out
    assert "decode" in out and json.load(open(trace))["traceEvents"]
    assert main(["bench", "--preset", "tiny-b", "--prompt-len", "20", "--gen", "4", "--reps", "1", "--batch-sizes", "1,3", "--json"]) == 0
    rows = [json.loads(l) for l in capsys.readouterr().out.strip().splitlines()]
    assert [r["batch"] for r in rows] == [1, 3] and all(r["decode_tok_s"] > 0 for r in rows)
    assert main(["run", "-m", str(tmp_path / "nowhere")]) == 1


# ----------------------------------------------------------------------------- a layer that reads another layer's cache
def _register_reader():
    """A mixer without a cache of its own: it averages the VALUES that an earlier attention layer left in
    its cache (kv head 0, all positions up to the token's own) and projects the mean.  The schedule names
    the entry whose cache it reads."""
    from edgelm_b200.config import register_architecture
    from edgelm_b200.config.base import LayerSpec, ModelPlan, PartSpec, ScheduleEntry
    from edgelm_b200.parts import Part, register_mixer
    from edgelm_b200.parts.registry import MIXERS

    if "toy_value_reader" in MIXERS:
        return

    @register_mixer("toy_value_reader")
    class ValueReader(Part):
        def __init__(self, spec, env):
            self.dim, self.hd, self.name = spec["dim"], spec["head_dim"], spec["name"]
            self.w = None

        def weight_shapes(self, prefix):
            return {prefix + self.name: (self.dim, self.hd)}

        def load(self, tensors, prefix, device):
            self.w = tensors[prefix + self.name].to(device=device, dtype=torch.float32)

        def forward(self, ctx, h, x, cache):
            table = ctx.page_table(cache.group).long()      # [sequences, pages]: rows of the other entry's group
            v = cache.v                                      # [pages, kv_heads, 64, head_dim] of the entry it reads
            t0 = 0
            for i, (n, p0) in enumerate(zip(ctx.seq_lengths, ctx.seq_first_positions)):
                pos = torch.arange(p0 + n, device=x.device)
                rows = v[table[i, pos // 64], 0, pos % 64].float()          # values of positions 0 .. p0 + n - 1
                means = torch.cumsum(rows, 0)[p0:] / (pos[p0:] + 1).unsqueeze(1)
                x[t0:t0 + n] += means @ self.w.T
                t0 += n

    @register_architecture("ToyReaderForCausalLM", model_type="toy_reader")
    class ReaderConfig:
        def __init__(self, d):
            self.d = d

        @classmethod
        def from_dict(cls, d):
            return cls(d)

        def plan(self):
            d = self.d
            D, V, hd = d["width"], d["vocab_size"], d.get("head_dim", 16)
            norm = lambda name: PartSpec("rmsnorm", {"dim": D, "eps": 1e-5, "name": name})
            rope = PartSpec("rope", {"head_dim": hd, "theta": 1000.0, "max_positions": 256})
            names = {"q": "q.weight", "k": "k.weight", "v": "v.weight", "o": "o.weight"}
            att = PartSpec("attention", {"hidden_size": D, "num_heads": 2, "num_kv_heads": 2, "head_dim": hd, "positions": rope, "names": names})
            reader = PartSpec("toy_value_reader", {"dim": D, "head_dim": hd, "name": "read.weight"})
            ffn = lambda inter: PartSpec("swiglu", {"hidden_size": D, "intermediate_size": inter,
                                                    "names": {"gate": "g.weight", "up": "u.weight", "down": "d.weight"}})
            layers = (LayerSpec("a.", "prenorm", att, norm("n1.weight"), ffn(24), norm("n2.weight")),
                      LayerSpec("r.", "prenorm", reader, norm("n1.weight"), ffn(24), norm("n2.weight")))
            schedule = (ScheduleEntry(0), ScheduleEntry(1, reads_cache_of=0))
            if d.get("third_layer"):   # another attention layer, with other head counts and another width inside
                att3 = PartSpec("attention", {"hidden_size": D, "num_heads": 3, "num_kv_heads": 1, "head_dim": hd, "positions": rope, "names": names})
                layers += (LayerSpec("c.", "prenorm", att3, norm("n1.weight"), ffn(40), norm("n2.weight")),)
                schedule += (ScheduleEntry(2),)
            return ModelPlan(hidden_size=D, vocab_size=V, max_positions=256,
                             embedding=PartSpec("embedding", {"vocab_size": V, "dim": D, "name": "emb.weight"}),
                             layers=layers, schedule=schedule,
                             final_norm=norm("final.weight"),
                             head=PartSpec("lm_head", {"vocab_size": V, "dim": D, "tied_to": None, "name": "head.weight"}))


def _reader_plain(W, tokens, hd, third_layer):
    """The toy reader architecture, whole sequences, in plain NumPy."""
    x = plain.embed(W["emb.weight"], tokens)
    h = plain.rmsnorm(x, W["a.n1.weight"], 1e-5)
    pos = np.arange(len(x))
    q = plain.rope(h @ W["a.q.weight"].T, pos, 2, hd, 1000.0)
    k = plain.rope(h @ W["a.k.weight"].T, pos, 2, hd, 1000.0)
    v = h @ W["a.v.weight"].T
    x = x + plain.attention(q, k, v, 2, 2, hd) @ W["a.o.weight"].T
    x = x + plain.swiglu_mlp(plain.rmsnorm(x, W["a.n2.weight"], 1e-5), W["a.g.weight"], W["a.u.weight"], W["a.d.weight"])
    means = np.cumsum(v[:, :hd], axis=0) / (pos + 1)[:, None]          # kv head 0 of the attention layer's values
    x = x + means.astype(np.float32) @ W["r.read.weight"].T
    x = x + plain.swiglu_mlp(plain.rmsnorm(x, W["r.n2.weight"], 1e-5), W["r.g.weight"], W["r.u.weight"], W["r.d.weight"])
    if third_layer:
        h = plain.rmsnorm(x, W["c.n1.weight"], 1e-5)
        q = plain.rope(h @ W["c.q.weight"].T, pos, 3, hd, 1000.0)
        k = plain.rope(h @ W["c.k.weight"].T, pos, 1, hd, 1000.0)
        x = x + plain.attention(q, k, h @ W["c.v.weight"].T, 3, 1, hd) @ W["c.o.weight"].T
        x = x + plain.swiglu_mlp(plain.rmsnorm(x, W["c.n2.weight"], 1e-5), W["c.g.weight"], W["c.u.weight"], W["c.d.weight"])
    return plain.rmsnorm(x, W["final.weight"], 1e-5) @ W["head.weight"].T


def test_a_layer_reads_another_layers_cache(tmp_path):
    _register_reader()
    from edgelm_b200.config import read_config
    from edgelm_b200.engine.engine import Engine, load_model
    from edgelm_b200.engine.model import expected_weights
    from edgelm_b200.weights import random_tensors, read_dir, write_file
    d = {"architectures": ["ToyReaderForCausalLM"], "vocab_size": 41, "width": 32}
    folder = tmp_path / "reader"
    folder.mkdir()
    (folder / "config.json").write_text(json.dumps(d))
    exp = expected_weights(read_config(str(folder)).plan())
    write_file(str(folder / "model.safetensors"), random_tensors(exp, seed=3, sigma=0.2, dtype=torch.float32))
    eng = Engine(load_model(str(folder), "float32"), max_tokens=512)
    assert len(eng.cache.kv_groups) == 1 and eng.cache.kv_groups[0].n_entries == 1 and eng.cache.entries[1] is None
    W = {k: v.float().numpy() for k, v in read_dir(str(folder)).items()}

    plain_model = lambda tokens: _reader_plain(W, tokens, 16, third_layer=False)
    reqs = [[int(v) for v in np.random.default_rng(10 + i).integers(0, 41, size=n)] for i, n in enumerate([70, 9, 130])]
    for r in reqs:
        want = plain_model(r)
        assert H.rel_err(H.run_whole(eng, r), want) < 5e-5
        assert H.rel_err(H.run_tail_one_by_one(eng, r, 8), want) < 5e-5
    for r, g in zip(reqs, H.run_batches(eng, reqs, batch_size=2, decode_tail=4)):
        assert H.rel_err(g, plain_model(r)) < 5e-5


def test_layers_of_other_kinds_between_attention_layers_in_bfloat16(tmp_path):
    """Attention layer, a toy layer that reads the first one's cache, attention layer with other head counts: the
    float32 engine and the bfloat16 engine (tensor-core kernels for the attention layers, the toy layer's own
    forward between them) against plain NumPy, token by token and in unequal batches."""
    _register_reader()
    from edgelm_b200.config import read_config
    from edgelm_b200.engine.engine import Engine, load_model
    from edgelm_b200.engine.model import expected_weights
    from edgelm_b200.weights import random_tensors, read_dir, write_file
    d = {"architectures": ["ToyReaderForCausalLM"], "vocab_size": 41, "width": 32, "head_dim": 32, "third_layer": True}
    folder = tmp_path / "sandwich"
    folder.mkdir()
    (folder / "config.json").write_text(json.dumps(d))
    exp = expected_weights(read_config(str(folder)).plan())
    write_file(str(folder / "model.safetensors"), random_tensors(exp, seed=4, sigma=0.2, dtype=torch.float32))
    reqs = [[int(v) for v in np.random.default_rng(20 + i).integers(0, 41, size=n)] for i, n in enumerate([70, 9, 130, 64])]
    W = {k: v.float().numpy() for k, v in read_dir(str(folder)).items()}
    want = [_reader_plain(W, r, 32, third_layer=True) for r in reqs]
    for dtype, tol in (("float32", 5e-5), ("bfloat16", H.TOL["bfloat16"])):
        eng = Engine(load_model(str(folder), dtype), max_tokens=1024)
        got = [H.run_tail_one_by_one(eng, r, 12) for r in reqs] + H.run_batches(eng, reqs, batch_size=3, decode_tail=6)
        eng.check_device_errors()
        for a, b in zip(got, want + want):
            assert np.isfinite(a).all() and H.rel_err(a, b) < tol, dtype
