"""Shared by the GPU tests: the two tiny configurations, model folders with random weights in a
temporary place, the plain implementation's logits, and drivers that cut one token stream
through the engine in different ways."""
import numpy as np
import torch

import plain_llama as plain

# Two tiny configurations that differ in every size and option: layers, width, head counts and
# grouping (4/2 grouped vs 3/1 multi-query), head size, feed-forward width (200 is no multiple
# of 16), vocabulary (397 is odd), theta, eps, tied vs separate head, positions, weight scale.
TINY_A = dict(model_type="llama", architectures=["LlamaForCausalLM"], vocab_size=256, hidden_size=64,
              intermediate_size=128, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2, head_dim=16,
              max_position_embeddings=128, rope_theta=10000.0, rms_norm_eps=1e-5, tie_word_embeddings=True,
              bos_token_id=0, eos_token_id=0)
TINY_B = dict(model_type="llama", architectures=["LlamaForCausalLM"], vocab_size=397, hidden_size=96,
              intermediate_size=200, num_hidden_layers=3, num_attention_heads=3, num_key_value_heads=1, head_dim=32,
              max_position_embeddings=256, rope_theta=100000.0, rms_norm_eps=1e-6, tie_word_embeddings=False,
              bos_token_id=1, eos_token_id=2)
# widths that no vector load divides (50 = 2 * 25, 70, 101): every matrix product takes its any-size path
TINY_C = dict(model_type="llama", architectures=["LlamaForCausalLM"], vocab_size=101, hidden_size=50,
              intermediate_size=70, num_hidden_layers=2, num_attention_heads=6, num_key_value_heads=3, head_dim=48,
              max_position_embeddings=160, rope_theta=777.0, rms_norm_eps=3e-4, tie_word_embeddings=True,
              bos_token_id=0, eos_token_id=1)
# a head size that the tensor-core kernels take (64), and room for contexts of many pages
TINY_D = dict(model_type="llama", architectures=["LlamaForCausalLM"], vocab_size=300, hidden_size=72,
              intermediate_size=88, num_hidden_layers=3, num_attention_heads=4, num_key_value_heads=2, head_dim=64,
              max_position_embeddings=1200, rope_theta=50000.0, rms_norm_eps=2e-5, tie_word_embeddings=False,
              bos_token_id=0, eos_token_id=1)
TINY = {"tiny_a": (TINY_A, 0, 0.09), "tiny_b": (TINY_B, 2, 0.07), "tiny_c": (TINY_C, 5, 0.1), "tiny_d": (TINY_D, 8, 0.08)}  # config, seed, sigma (large enough for logits of order 1)

TOL = {"float32": 2e-5, "bfloat16": 3e-2}


def rel_err(a, b):
    """adarsh-sgh/edgelm's metric (tests/common.hpp:69-76): max |a-b| / max(1, max |b|)."""
    a = np.asarray(a, dtype=np.float64)
    b = np.asarray(b, dtype=np.float64)
    assert a.shape == b.shape, (a.shape, b.shape)
    return float(np.abs(a - b).max() / max(1.0, np.abs(b).max()))


def make_model_dir(tmp, name, file_dtype="bfloat16"):
    from edgelm_b200 import write_model_dir
    from edgelm_b200.config import config_class_for
    cfg_dict, seed, sigma = TINY[name]
    cfg = config_class_for(cfg_dict).from_dict(cfg_dict)
    return write_model_dir(str(tmp / f"{name}_{file_dtype}"), cfg, seed, sigma=sigma, dtype=file_dtype)


def tokens_for(name, n, salt):
    vocab = TINY[name][0]["vocab_size"]
    rng = np.random.default_rng(1000 + salt)
    return [int(t) for t in rng.integers(0, vocab, size=n)]


class Oracle:
    """The plain implementation on a model folder, logits cached per token tuple."""

    def __init__(self, model_dir):
        self.cfg, self.W = plain.read_model(model_dir)
        self._memo = {}

    def logits(self, tokens):
        key = tuple(tokens)
        if key not in self._memo:
            self._memo[key] = plain.forward(self.cfg, self.W, list(tokens))
        return self._memo[key]


def run_whole(engine, tokens):
    """One request alone and whole: one step, logits at every position."""
    from edgelm_b200.engine.engine import StepEntry
    slot = engine.open(1)[0]
    out = engine.step([StepEntry(slot, tokens, list(range(len(tokens))))]).cpu().numpy()
    engine.close([slot])
    return out


def run_tail_one_by_one(engine, tokens, tail=32):
    """The first len - tail tokens in one step, then the last `tail` tokens one by one."""
    from edgelm_b200.engine.engine import StepEntry
    slot = engine.open(1)[0]
    head = max(0, len(tokens) - tail)
    parts = []
    if head:
        parts.append(engine.step([StepEntry(slot, tokens[:head], list(range(head)))]).cpu().numpy())
    for t in tokens[head:]:
        parts.append(engine.step([StepEntry(slot, [t], [0])]).cpu().numpy())
    engine.close([slot])
    return np.concatenate(parts, axis=0)


def run_batches(engine, requests, batch_size, decode_tail, prompt_rows=None):
    """Batches of unequal lengths, one after another.  In each batch all requests start together:
    step 0 brings each request's first len - decode_tail tokens (at least 1), then every step
    brings one token per request still running; shorter requests end earlier and give back what
    they hold.  Returns per request its logits at every position (with `prompt_rows`: at the last
    so many positions of its first step, then at every later position)."""
    from edgelm_b200.engine.engine import StepEntry
    out = [None] * len(requests)
    for b0 in range(0, len(requests), batch_size):
        idxs = list(range(b0, min(len(requests), b0 + batch_size)))
        slots = dict(zip(idxs, engine.open(len(idxs))))
        fed = {}
        entries = []
        for i in idxs:
            n0 = max(1, len(requests[i]) - decode_tail)
            want = list(range(n0)) if prompt_rows is None else list(range(max(0, n0 - prompt_rows), n0))
            entries.append(StepEntry(slots[i], requests[i][:n0], want))
            fed[i] = n0
        lg = engine.step(entries).cpu().numpy()
        rows = {i: [] for i in idxs}
        r = 0
        for e, i in zip(entries, idxs):
            rows[i].append(lg[r:r + len(e.want)])
            r += len(e.want)
        live = list(idxs)
        while live:
            for i in [i for i in live if fed[i] == len(requests[i])]:
                engine.close([slots.pop(i)])
                live.remove(i)
            if not live:
                break
            lg = engine.step([StepEntry(slots[i], [requests[i][fed[i]]], [0]) for i in live]).cpu().numpy()
            for r, i in enumerate(live):
                rows[i].append(lg[r:r + 1])
                fed[i] += 1
        for i in idxs:
            out[i] = np.concatenate(rows[i], axis=0)
        engine.cache.check()
    return out


def make_preset_dir(tmp, preset, layers, seed=0, sigma=0.02):
    """A model folder with a built-in shape's layer sizes (width, heads, head size, feed-forward width,
    vocabulary, theta, eps, tied head: all untouched) cut to `layers` layers, random weights N(0, sigma)
    in a bfloat16 file: small enough for the plain implementation to follow on the CPU."""
    import dataclasses

    from edgelm_b200 import write_model_dir
    from edgelm_b200.presets import preset_config
    cfg = dataclasses.replace(preset_config(preset), num_hidden_layers=int(layers))
    return write_model_dir(str(tmp / f"{preset}_{layers}L"), cfg, seed, sigma=sigma, dtype="bfloat16")


def decisive_agreement(got, want, gap=0.15):
    """Share of rows of `got` whose argmax is `want`'s, among the rows where `want` is decisive (its two
    largest logits at least `gap` apart), and the number of such rows."""
    want = np.asarray(want)
    top2 = np.partition(want, -2, axis=-1)[:, -2:]
    decisive = (top2[:, 1] - top2[:, 0]) >= gap
    if not decisive.any():
        return 1.0, 0
    same = np.asarray(got).argmax(-1)[decisive] == want.argmax(-1)[decisive]
    return float(same.mean()), int(decisive.sum())
