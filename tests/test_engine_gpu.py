"""The engine against the plain implementation, in float32 and in bfloat16, in every way of
cutting the same token streams: whole, tail one by one, unequal batches on reused slots."""
import numpy as np
import pytest
import torch

import helpers as H
import plain_llama as plain

pytestmark = pytest.mark.gpu

NAMES = ["tiny_a", "tiny_b", "tiny_c"]
DTYPES = ["float32", "bfloat16"]


@pytest.fixture(scope="module")
def model_dirs(tmp_path_factory):
    tmp = tmp_path_factory.mktemp("models")
    return {n: H.make_model_dir(tmp, n) for n in NAMES + ["tiny_d"]}


@pytest.fixture(scope="module")
def oracles(model_dirs):
    return {n: H.Oracle(d) for n, d in model_dirs.items()}


_engines = {}


def engine_for(model_dirs, name, dtype, max_tokens=1024, **kw):
    from edgelm_b200.engine.engine import Engine
    key = (name, dtype, max_tokens, tuple(sorted(kw.items())))
    if key not in _engines:
        _engines[key] = Engine.from_dir(model_dirs[name], dtype=dtype, max_tokens=max_tokens, **kw)
    return _engines[key]


def lengths_for(name):
    top = H.TINY[name][0]["max_position_embeddings"]
    return [l for l in (1, 5, 33, 64, 65, 100, 128, 200) if l <= top]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_whole_requests(model_dirs, oracles, name, dtype):
    eng = engine_for(model_dirs, name, dtype)
    for i, n in enumerate(lengths_for(name)):
        toks = H.tokens_for(name, n, i)
        got = H.run_whole(eng, toks)
        want = oracles[name].logits(toks)
        assert H.rel_err(got, want) < H.TOL[dtype], (n,)
        if dtype == "float32":
            assert (got.argmax(-1) == want.argmax(-1)).all()
    eng.cache.check()
    eng.check_device_errors()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_tail_one_by_one(model_dirs, oracles, name, dtype):
    eng = engine_for(model_dirs, name, dtype)
    for i, n in enumerate(lengths_for(name)):
        toks = H.tokens_for(name, n, i)
        got = H.run_tail_one_by_one(eng, toks, 32)
        want = oracles[name].logits(toks)
        assert H.rel_err(got, want) < H.TOL[dtype], (n,)
        whole = H.run_whole(eng, toks)
        # cutting changes only rounding: far tighter than the distance to the oracle
        assert H.rel_err(got, whole) < (2e-6 if dtype == "float32" else 2e-2), (n,)
    eng.check_device_errors()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_unequal_batches_on_reused_slots(model_dirs, oracles, name, dtype):
    # a cache so small that the second and third batch must reuse the first one's pages
    eng = engine_for(model_dirs, name, dtype, max_tokens=448)
    top = H.TINY[name][0]["max_position_embeddings"]
    lens = [l for l in (3, 70, 17, 128, 64, 1, 40, 65, 9, 100) if l <= top]
    reqs = [H.tokens_for(name, n, 50 + i) for i, n in enumerate(lens)]
    got = H.run_batches(eng, reqs, batch_size=3, decode_tail=6)
    for r, g in zip(reqs, got):
        assert H.rel_err(g, oracles[name].logits(r)) < H.TOL[dtype], (len(r),)
    assert eng.cache.slots.available() == eng.cache.n_slots
    assert all(g.pool.available() == g.pool.n for g in eng.cache.kv_groups)
    eng.check_device_errors()


@pytest.mark.parametrize("name", NAMES)
def test_batch_does_not_change_a_request(model_dirs, name):
    """float32: a request's logits in a batch equal its logits alone to rounding of the last bit or two."""
    from edgelm_b200.engine.engine import StepEntry
    eng = engine_for(model_dirs, name, "float32")
    reqs = [H.tokens_for(name, n, 70 + i) for i, n in enumerate([37, 5, 66])]
    alone = [H.run_whole(eng, r) for r in reqs]
    slots = eng.open(3)
    lg = eng.step([StepEntry(s, r, list(range(len(r)))) for s, r in zip(slots, reqs)]).cpu().numpy()
    eng.close(slots)
    r0 = 0
    for a in alone:
        assert H.rel_err(lg[r0:r0 + len(a)], a) < 1e-6
        r0 += len(a)


@pytest.mark.parametrize("dtype", DTYPES)
def test_long_decoding(model_dirs, oracles, dtype):
    """One prompt token, then 200 decoded one by one across three page edges."""
    name = "tiny_b"
    eng = engine_for(model_dirs, name, dtype)
    toks = H.tokens_for(name, 201, 90)
    got = H.run_tail_one_by_one(eng, toks, tail=200)
    assert H.rel_err(got, oracles[name].logits(toks)) < H.TOL[dtype]


def test_decode_steps_of_few_sequences_over_many_pages(model_dirs, oracles):
    """bfloat16 decode steps of a few sequences whose contexts span one, nine and eighteen pages in one batch (the
    decode attention deals a sequence's pages to many blocks and folds them), sequences that end earlier, a slot
    used again."""
    name = "tiny_d"
    eng = engine_for(model_dirs, name, "bfloat16", max_tokens=4096)
    lens = [1100, 40, 530, 7, 449]
    reqs = [H.tokens_for(name, n, 300 + i) for i, n in enumerate(lens)]
    want = [oracles[name].logits(r) for r in reqs]
    got = H.run_batches(eng, reqs, batch_size=3, decode_tail=24)
    for g, w in zip(got, want):
        assert H.rel_err(g, w) < H.TOL["bfloat16"]
    eng.cache.check()
    eng.check_device_errors()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_first_tokens(model_dirs, oracles, name, dtype):
    eng = engine_for(model_dirs, name, dtype)
    for n in (1, 2, 3):
        toks = H.tokens_for(name, n, 95 + n)
        assert H.rel_err(H.run_whole(eng, toks), oracles[name].logits(toks)) < H.TOL[dtype]
        assert H.rel_err(H.run_tail_one_by_one(eng, toks, tail=n), oracles[name].logits(toks)) < H.TOL[dtype]


@pytest.mark.parametrize("name", NAMES)
def test_cut_steps_equal_whole(model_dirs, oracles, name):
    """A step larger than max_step_tokens is cut inside the engine; wants may be unsorted."""
    from edgelm_b200.engine.engine import StepEntry
    eng = engine_for(model_dirs, name, "float32", max_tokens=512, max_step_tokens=64)
    reqs = [H.tokens_for(name, n, 110 + i) for i, n in enumerate([100, 30, 90])]
    slots = eng.open(3)
    wants = [list(reversed(range(len(r)))) for r in reqs]
    lg = eng.step([StepEntry(s, r, w) for s, r, w in zip(slots, reqs, wants)]).cpu().numpy()
    eng.close(slots)
    r0 = 0
    for r in reqs:
        want = oracles[name].logits(r)[::-1]
        assert H.rel_err(lg[r0:r0 + len(r)], want) < H.TOL["float32"]
        r0 += len(r)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_greedy_generation_through_entry_point(model_dirs, oracles, name, dtype):
    import edgelm_b200
    prompts = [H.tokens_for(name, n, 130 + i) for i, n in enumerate([5, 9, 16, 1, 30])]
    o = oracles[name]
    eng = edgelm_b200.load_engine(model_dirs[name], dtype=dtype, ctx=128, slots=2)
    got = edgelm_b200.generate(None, prompts, n=12, engine=eng, slots=2, stop=[], ignore_eos=True)
    for p, g in zip(prompts, got):
        assert len(g) == 12
        if dtype == "float32":
            assert g == plain.generate(o.cfg, o.W, p, 12, stop_ids=[], ignore_eos=True)
        else:  # bfloat16 may pick another of two near-equal logits: every choice must be the oracle's best within rounding
            seq = list(p)
            for t in g:
                lg = o.logits(seq)[-1]
                assert lg[t] >= lg.max() - 0.1
                seq.append(t)
    assert eng.cache.slots.available() == eng.cache.n_slots
    # eager steps give the same tokens as replayed graphs
    eng2 = edgelm_b200.load_engine(model_dirs[name], dtype=dtype, ctx=128, slots=2, use_graphs=False)
    assert edgelm_b200.generate(None, prompts, n=12, engine=eng2, slots=2, stop=[], ignore_eos=True) == got


def test_long_greedy_generation_patches_the_step_in_place(model_dirs, oracles):
    """float32, 150 tokens from prompts of unequal lengths: consecutive decode steps patch the step's metadata in
    place (ids, positions, the page-table rows that gain a page) instead of laying it out again; the tokens are
    the plain implementation's across three page edges."""
    import edgelm_b200
    name = "tiny_b"
    o = oracles[name]
    prompts = [H.tokens_for(name, n, 170 + i) for i, n in enumerate([60, 3, 64])]
    eng = edgelm_b200.load_engine(model_dirs[name], dtype="float32", ctx=256, slots=3)
    calls = {"patched": 0, "laid_out": 0}
    refill, fill = eng.buffers.refill_next_token, eng.buffers.fill

    def count_refill(*a, **k):
        ok = refill(*a, **k)
        calls["patched"] += bool(ok)
        return ok

    def count_fill(*a, **k):
        calls["laid_out"] += 1
        return fill(*a, **k)
    eng.buffers.refill_next_token, eng.buffers.fill = count_refill, count_fill
    got = edgelm_b200.generate(None, prompts, n=150, engine=eng, slots=3, stop=[], ignore_eos=True)
    assert got == [plain.generate(o.cfg, o.W, p, 150, stop_ids=[], ignore_eos=True) for p in prompts]
    assert calls["patched"] > 100 and calls["laid_out"] < 10
    eng.cache.check()


def test_sampled_generation_and_stop(model_dirs, oracles):
    import edgelm_b200
    name = "tiny_b"
    o = oracles[name]
    prompts = [H.tokens_for(name, n, 150 + i) for i, n in enumerate([1, 7, 30, 64])]
    eng = edgelm_b200.load_engine(model_dirs[name], dtype="float32", ctx=128, slots=4)
    got = edgelm_b200.generate(None, prompts, n=12, temp=0.8, top_k=20, seed=7, engine=eng, slots=4, stop=[], ignore_eos=True)
    for i, (p, g) in enumerate(zip(prompts, got)):
        assert g == plain.generate(o.cfg, o.W, p, 12, temperature=0.8, top_k=20, seed=7 + i, stop_ids=[], ignore_eos=True)
    again = edgelm_b200.generate(None, prompts, n=12, temp=0.8, top_k=20, seed=7, engine=eng, slots=4, stop=[], ignore_eos=True)
    assert again == got
    # a stop token ends its sequence early and is not emitted
    stop = got[1][4]
    cut = edgelm_b200.generate(None, prompts, n=12, temp=0.8, top_k=20, seed=7, engine=eng, slots=4, stop=[stop],
                               return_details=True)
    want1 = got[1][:got[1].index(stop)]
    assert cut[1].tokens == want1 and cut[1].finish_reason == "stop"
    for g, c in zip(got, cut):
        if stop not in g:
            assert c.tokens == g and c.finish_reason == "length"


def test_session_and_profiler(model_dirs, oracles, tmp_path):
    import json
    import edgelm_b200
    name = "tiny_a"
    toks = H.tokens_for(name, 20, 170)
    s = edgelm_b200.Session(model_dirs[name], dtype="float32", max_ctx=64, all_logits=True, profile=True)
    a = s.prefill(toks[:8]).cpu().numpy()
    b = np.concatenate([s.decode(t).cpu().numpy() for t in toks[8:]])
    assert s.pos == 20
    assert H.rel_err(np.concatenate([a, b]), oracles[name].logits(toks)) < 2e-5
    s.reset()
    assert s.pos == 0
    n = s.engine.profiler.write_trace(str(tmp_path / "trace.json"))
    tr = json.load(open(tmp_path / "trace.json"))
    names = {e["name"] for e in tr["traceEvents"]}
    assert {"qkv_proj", "attn_prefill", "attn_decode", "lm_head", "prefill", "decode"} <= names
    assert all(e["ph"] in ("X", "M") for e in tr["traceEvents"]) and n > 13
    assert "decode:" in s.engine.profiler.stats()


def test_context_overflow_and_bad_input(model_dirs):
    from edgelm_b200.cache import CacheError
    from edgelm_b200.engine.engine import EngineError, StepEntry
    eng = engine_for(model_dirs, "tiny_a", "float32", max_tokens=256)
    slot = eng.open(1)[0]
    with pytest.raises(CacheError, match="positions"):
        eng.step([StepEntry(slot, [1] * 129, [])])
    with pytest.raises(EngineError, match="vocabulary"):
        eng.step([StepEntry(slot, [256], [0])])
    with pytest.raises(EngineError, match="twice"):
        eng.step([StepEntry(slot, [1], [0]), StepEntry(slot, [2], [0])])
    eng.close([slot])
    with pytest.raises(CacheError):
        eng.step([StepEntry(slot, [1], [0])])
    held = eng.open(4)
    for s in held:
        eng.step([StepEntry(s, [1] * 64, [])])
    with pytest.raises(CacheError, match="full"):
        eng.step([StepEntry(held[0], [1], [0])])
    eng.close(held)
    eng.cache.check()


@pytest.mark.parametrize("dtype", DTYPES)
def test_generation_reads_the_device_error_word(model_dirs, oracles, dtype):
    """What a kernel reports (here: set from the host, no kernel is made to give up) ends generation with an
    error instead of tokens sampled from bad logits: in the prompt step, in a captured decode step, in `step`,
    and through the entry point; afterwards the engine works again."""
    import edgelm_b200
    from edgelm_b200.csrc import ops
    from edgelm_b200.engine.engine import StepEntry
    from edgelm_b200.sampling import SamplingParams
    name = "tiny_d"
    eng = edgelm_b200.load_engine(model_dirs[name], dtype=dtype, ctx=256, slots=4)
    params = SamplingParams()
    prompts = [H.tokens_for(name, n, 400 + i) for i, n in enumerate([9, 40])]
    slots = eng.open(2)
    eng.err.fill_(8)
    with pytest.raises(ops.KernelError, match="wait ran out"):
        eng.prefill_sampled(slots, prompts, params)
    assert int(eng.err.item()) == 0
    eng.close(slots)
    slots = eng.open(2)
    toks = eng.prefill_sampled(slots, prompts, params)
    toks = eng.decode_sampled(slots, toks, params)          # captures the decode graph
    eng.err.fill_(4)
    with pytest.raises(ops.KernelError, match="page"):
        eng.decode_sampled(slots, toks, params)
    eng.close(slots)
    slot = eng.open(1)[0]
    eng.err.fill_(1)
    eng.step([StepEntry(slot, prompts[0], [0])])            # not waited for: the next call reports it
    with pytest.raises(ops.KernelError, match="vocabulary"):
        eng.step([StepEntry(slot, [3], [0])])
    eng.close([slot])
    eng.err.fill_(2)
    with pytest.raises(ops.KernelError, match="position"):
        edgelm_b200.generate(None, prompts, n=4, engine=eng, slots=2, stop=[], ignore_eos=True)
    eng.cache.check()
    assert eng.cache.slots.available() == eng.cache.n_slots   # the loop gave its slots back on the way out
    got = edgelm_b200.generate(None, prompts, n=6, engine=eng, slots=2, stop=[], ignore_eos=True)
    if dtype == "float32":
        o = oracles[name]
        assert got == [plain.generate(o.cfg, o.W, p, 6, stop_ids=[], ignore_eos=True) for p in prompts]


@pytest.mark.parametrize("dtype", DTYPES)
def test_prompt_steps_replayed_from_a_graph(model_dirs, oracles, dtype):
    """A prompt step whose shape comes back is captured at its second appearance and replayed from then on: other
    tokens, other slots and pages, the same shape.  Every run is compared with the plain implementation."""
    name = "tiny_b"
    eng = edgelm_b200_engine(model_dirs[name], dtype)
    from edgelm_b200.engine.engine import StepEntry
    lens = (70, 33)
    for rep in range(4):
        reqs = [H.tokens_for(name, n, 500 + 10 * rep + i) for i, n in enumerate(lens)]
        filler = eng.open(rep)              # other slots, hence other pages, each time
        for f in filler:
            eng.step([StepEntry(f, [1] * (64 * rep + 1), [])])
        slots = eng.open(2)
        lg = eng.step([StepEntry(s, r, list(range(len(r)))) for s, r in zip(slots, reqs)]).cpu().numpy()
        assert (((70, 33), 103) in eng._step_graphs) == (rep >= 1), rep
        r0 = 0
        for r in reqs:
            assert H.rel_err(lg[r0:r0 + len(r)], oracles[name].logits(r)) < H.TOL[dtype], (rep,)
            r0 += len(r)
        eng.close(slots + filler)
    eng.check_device_errors()
    eng.cache.check()


def edgelm_b200_engine(model_dir, dtype):
    from edgelm_b200.engine.engine import Engine
    return Engine.from_dir(model_dir, dtype=dtype, max_tokens=1024)
