"""The engine against the plain implementation at the layer sizes of SmolLM2-135M, 360M and 1.7B
(width 576 / 960 / 2048, 9/3, 15/5 and 32/32 heads of 64, feed-forward 1536 / 2560 / 8192, vocabulary
49,152, tied head), cut to two layers (one for the long contexts) so that the plain NumPy side
stays cheap, in float32 and in bfloat16, in every way of cutting the work.  These are the sizes at
which the dispatch picks the persistent tcgen05 products, split-K, the walking few-rows kernel,
the tcgen05 prefill attention and the wave-filling decode splits; the tiny configurations reach
none of them.  adarsh-sgh/edgelm checks its real model in the same cuts (tools/check_real.py:79-93:
whole prompt, and a prompt's head then single tokens; tests/test_e2e.cpp:12-75)."""
import numpy as np
import pytest
import torch

import helpers as H
import plain_llama as plain

pytestmark = pytest.mark.gpu

DTYPES = ["float32", "bfloat16"]
VOCAB = 49152


@pytest.fixture(scope="module")
def dirs(tmp_path_factory):
    tmp = tmp_path_factory.mktemp("real_sizes")
    made = {}

    def get(preset, layers):
        if (preset, layers) not in made:
            made[(preset, layers)] = H.make_preset_dir(tmp, preset, layers, seed=3 + layers)
        return made[(preset, layers)]
    return get


_oracles = {}


_hidden = {}


def plain_logits(d, toks, rows):
    """The plain implementation's logits at `rows` of one whole sequence; the residual stream after the last
    layer is kept per (model, sequence), so that the second dtype and other rows cost the head only."""
    if d not in _oracles:
        _oracles.clear()            # one at a time: the largest holds 0.8 GB of float32 weights
        _oracles[d] = plain.read_model(d)
    cfg, W = _oracles[d]
    key = (d, len(toks), hash(tuple(toks)))
    if key not in _hidden:
        _hidden[key] = plain.hidden(cfg, W, toks)
    return plain.lm_head(cfg, W, _hidden[key][np.asarray(rows, dtype=np.int64)])


def ids(n, salt):
    return [int(t) for t in np.random.default_rng(9000 + salt).integers(0, VOCAB, size=n)]


def engine(d, dtype, max_tokens, **kw):
    from edgelm_b200.engine.engine import Engine
    return Engine.from_dir(d, dtype=dtype, max_tokens=max_tokens, **kw)


def check(got, want, dtype, what):
    err = H.rel_err(got, want)
    assert err < H.TOL[dtype], (what, err)
    if dtype == "float32":
        rate, n = H.decisive_agreement(got, want, gap=1e-3)
        assert rate == 1.0, (what, rate, n)
    else:
        rate, n = H.decisive_agreement(got, want)
        assert n == 0 or rate >= 0.99, (what, rate, n)


SAMPLED = sorted({0, 1, 2, 62, 63, 64, 65, 127, 128, 129, 255, 256, 1000, 1023, 1024, 1025, 1500, 1983, 1984, 1985,
                  2015, 2016, 2040, 2046, 2047} | set(range(31, 2048, 53)))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("preset", ["smollm2-135m", "smollm2-360m", "smollm2-1.7b"])
def test_whole_prompt_and_tail_one_by_one(dirs, preset, dtype):
    """A 2,048-token prompt whole (logits at 60 odd places: page edges, tile edges, the ends), and the same
    tokens as 2,016 at once then 32 one by one."""
    from edgelm_b200.engine.engine import StepEntry
    d = dirs(preset, 2)
    toks = ids(2048, 1)
    want = plain_logits(d, toks, SAMPLED)
    eng = engine(d, dtype, max_tokens=2048 + 64)
    slot = eng.open(1)[0]
    whole = eng.step([StepEntry(slot, toks, SAMPLED)]).cpu().numpy()
    eng.close([slot])
    check(whole, want, dtype, "whole")
    # the same again: this shape is now replayed from its captured graph, on other pages
    filler = eng.open(1)[0]
    eng.step([StepEntry(filler, toks[:1], [])])
    slot = eng.open(1)[0]
    again = eng.step([StepEntry(slot, toks, SAMPLED)]).cpu().numpy()
    eng.close([slot, filler])
    check(again, want, dtype, "whole, second time")
    slot = eng.open(1)[0]
    head = [p for p in SAMPLED if p < 2016]
    parts = [eng.step([StepEntry(slot, toks[:2016], head)]).cpu().numpy()]
    for t in toks[2016:]:
        parts.append(eng.step([StepEntry(slot, [t], [0])]).cpu().numpy())
    eng.close([slot])
    tail = np.concatenate(parts)
    rows = head + list(range(2016, 2048))
    want_tail = plain_logits(d, toks, rows)
    check(tail, want_tail, dtype, "tail one by one")
    # cutting changes rounding only.  (float32: the products of many rows and of one row sum their K terms in other
    # orders; with K up to 8,192 that is 3e-6 here, where the tiny models' K of 200 gives under 1e-6.)
    both = [i for i, p in enumerate(SAMPLED) if p in rows]
    pick = [rows.index(SAMPLED[i]) for i in both]
    assert H.rel_err(tail[pick], whole[both]) < (8e-6 if dtype == "float32" else 2e-2)
    if dtype == "bfloat16":   # no drift with position: the late rows are as close to the plain logits as the early ones
        e = np.abs(whole - want).max(axis=1)
        early, late = e[:len(e) // 4].mean(), e[-(len(e) // 4):].mean()
        assert late < 2.0 * early + 1e-3, (early, late)
    eng.check_device_errors()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("preset", ["smollm2-135m", "smollm2-1.7b"])
def test_unequal_batches_then_decoding(dirs, preset, dtype):
    """30 requests with prompts of 1 to 700 tokens and 8 more tokens each, in batches of 24 that start together:
    the first batch decodes 24 rows a step (the tensor-core product split over K), the second runs on the slots
    and pages the first gave back."""
    d = dirs(preset, 2)
    rng = np.random.default_rng(77)
    lens = [1, 700, 64, 65] + [int(x) for x in rng.integers(2, 700, size=26)]
    reqs = [ids(n + 8, 100 + i) for i, n in enumerate(lens)]
    eng = engine(d, dtype, max_tokens=sum(-(-len(r) // 64) * 64 for r in reqs[:24]) + 64)
    got = H.run_batches(eng, reqs, batch_size=24, decode_tail=8, prompt_rows=4)
    for i, (r, g) in enumerate(zip(reqs, got)):
        n0 = len(r) - 8
        rows = list(range(max(0, n0 - 4), len(r)))
        assert g.shape[0] == len(rows)
        check(g, plain_logits(d, r, rows), dtype, ("request", i, len(r)))
    assert eng.cache.slots.available() == eng.cache.n_slots
    eng.check_device_errors()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("preset", ["smollm2-135m", "smollm2-1.7b"])
def test_sampled_decoding_from_the_captured_graph(dirs, preset, dtype):
    """Greedy generation of 8 and of 20 sequences through the calls the generation loop makes (prompt step,
    then decode steps replayed from a CUDA graph with the sampler inside): every token the engine chose is
    the plain implementation's choice given the same prefix."""
    from edgelm_b200.sampling import SamplingParams
    d = dirs(preset, 2)
    eng = engine(d, dtype, max_tokens=20 * 512)
    params = SamplingParams()
    for B, salt in ((8, 300), (20, 400)):
        prompts = [ids(int(n), salt + i) for i, n in enumerate(np.random.default_rng(salt).integers(3, 400, size=B))]
        slots = eng.open(B)
        toks = eng.prefill_sampled(slots, prompts, params)
        outs = [[t] for t in toks]
        for _ in range(5):
            toks = eng.decode_sampled(slots, toks, params)
            for o, t in zip(outs, toks):
                o.append(t)
        eng.close(slots)
        assert len(eng._graphs) >= 1
        for p, o in zip(prompts, outs):
            seq = p + o[:-1]
            lg = plain_logits(d, seq, list(range(len(p) - 1, len(seq))))
            for j, t in enumerate(o):
                if dtype == "float32":
                    assert lg[j, t] >= lg[j].max() - 1e-4, (B, len(p), j)
                else:
                    assert lg[j, t] >= lg[j].max() - 0.12, (B, len(p), j)
    eng.check_device_errors()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("preset,prompt,tail", [("smollm2-135m", 8100, 60), ("smollm2-1.7b", 5000, 40)])
def test_long_context(dirs, preset, prompt, tail, dtype):
    """One layer, a prompt of thousands of tokens in one step and then single tokens, up to the last page of the
    position table: page tables of 128 pages, decode attention split 64 ways, the prompt attention's longest rows."""
    from edgelm_b200.engine.engine import StepEntry
    d = dirs(preset, 1)
    toks = ids(prompt + tail, 7)
    head = sorted({0, 63, 64, 4095, 4096, prompt - 1} | set(range(500, prompt, 997)))
    head = [p for p in head if p < prompt]
    rows = head + list(range(prompt, prompt + tail))
    want = plain_logits(d, toks, rows)
    eng = engine(d, dtype, max_tokens=8192 + 64)
    slot = eng.open(1)[0]
    parts = [eng.step([StepEntry(slot, toks[:prompt], head)]).cpu().numpy()]
    for t in toks[prompt:]:
        parts.append(eng.step([StepEntry(slot, [t], [0])]).cpu().numpy())
    eng.close([slot])
    got = np.concatenate(parts)
    check(got, want, dtype, "long context")
    eng.check_device_errors()


@pytest.mark.parametrize("preset", ["smollm2-135m", "smollm2-360m", "smollm2-1.7b"])
def test_workspace_covers_the_largest_steps(dirs, preset):
    """What the parts declare (`workspace_bytes`) against what the largest steps take: a prompt step of
    `max_step_tokens` tokens, a prompt step of 64 sequences, a decode step of 64 sequences.  `Workspace.alloc`
    raises when a part declared too little."""
    from edgelm_b200.engine.engine import StepEntry
    d = dirs(preset, 2)
    eng = engine(d, "bfloat16", max_tokens=8192 + 64 * 128, max_step_tokens=8192)
    slot = eng.open(1)[0]
    eng.step([StepEntry(slot, ids(8192, 1), [8191])])
    eng.close([slot])
    peak_prompt = eng.ws.peak
    slots = eng.open(64)
    eng.step([StepEntry(s, ids(1 + (i * 7) % 100, i), [0]) for i, s in enumerate(slots)])
    eng.step([StepEntry(s, [5], [0]) for s in slots])
    eng.close(slots)
    torch.cuda.synchronize()
    assert 0 < peak_prompt <= eng.ws.peak <= eng.ws.capacity
    assert eng.ws.peak >= 0.5 * eng.ws.capacity, "the declaration is more than twice what any step takes"
    eng.check_device_errors()
