"""Host-side bookkeeping: the cache's slots and pages, and the generation loop's decisions."""
import random

import pytest

from edgelm_b200.cache import CacheError, FreeList, SequenceCache, pages_for
from edgelm_b200.engine.generate import GenerationError, GenerationLoop, plan_batches
from edgelm_b200.parts.base import KVNeed, StateNeed
from edgelm_b200.sampling import SamplingParams, xorshift64


def make_cache(max_tokens=512, max_pos=256, layers=3, **kw):
    return SequenceCache([KVNeed(2, 16)] * layers, max_tokens, max_pos, device=None, **kw)


def test_free_list():
    f = FreeList(3, "thing")
    a, b, c = f.take(), f.take(), f.take()
    assert (a, b, c) == (0, 1, 2)
    with pytest.raises(CacheError, match="no free thing"):
        f.take()
    f.give(1)
    with pytest.raises(CacheError, match="not held"):
        f.give(1)
    with pytest.raises(CacheError, match="not held"):
        f.give(7)
    assert f.take() == 1
    f.check()


def test_groups_and_sizes():
    c = SequenceCache([KVNeed(2, 16), None, KVNeed(2, 16), KVNeed(1, 32), StateNeed((4, 8))], 640, 256, device=None)
    assert len(c.kv_groups) == 2 and len(c.state_groups) == 1
    assert c.entries[1] is None and c.entries[0].group is c.entries[2].group and c.entries[0].index == 0 and c.entries[2].index == 1
    assert c.entries[3].group is not c.entries[0].group
    assert c.n_pages == 10 and c.max_pages_per_seq == 4 and c.n_slots == 10
    assert make_cache(100).n_pages == 2 and pages_for(65) == 2 and pages_for(64) == 1 and pages_for(0) == 0
    with pytest.raises(CacheError, match="window"):
        SequenceCache([KVNeed(2, 16, window=0)], 256, 256, device=None)


def test_sequences_grow_and_give_back():
    c = make_cache(max_tokens=320, max_pos=256)  # 5 pages
    a, b = c.open(), c.open()
    c.reserve(a, 65)
    c.advance(a, 65)
    assert c.kv_groups[0].n_held[a] == 2 and c.length[a] == 65
    c.reserve(a, 1)          # position 65 lies in the second page already
    assert c.kv_groups[0].n_held[a] == 2
    c.reserve(b, 128)
    c.advance(b, 128)
    c.check()
    assert c.tokens_held() == 4 * 64
    c.reserve(a, 63)         # up to 128: still two pages
    c.advance(a, 63)
    c.reserve(a, 1)          # the fifth and last page
    with pytest.raises(CacheError, match="full"):
        c.reserve(b, 1)
    c.check()
    pages_a = [int(p) for p in c.kv_groups[0].table[a] if p >= 0]
    c.close(a)
    assert c.length[a] == 0 and c.kv_groups[0].pool.available() == 3
    c.reserve(b, 1)          # room again: a page that a held before is used again
    assert int(c.kv_groups[0].table[b, 2]) in pages_a
    with pytest.raises(CacheError, match="not held"):
        c.reserve(a, 1)
    with pytest.raises(CacheError, match="not held"):
        c.close(a)
    a2 = c.open()
    assert a2 == a and c.length[a2] == 0  # the slot is used again, from length 0
    c.close(a2)
    c.close(b)
    c.check()
    assert c.slots.available() == c.n_slots and c.kv_groups[0].pool.available() == 5


def test_longer_than_the_position_table():
    c = make_cache(max_tokens=1024, max_pos=100)
    s = c.open()
    c.reserve(s, 100)
    c.advance(s, 100)
    with pytest.raises(CacheError, match="positions"):
        c.reserve(s, 1)


def test_random_open_close_never_loses_anything():
    rng = random.Random(3)
    c = make_cache(max_tokens=64 * 20, max_pos=64 * 6, layers=2)
    live = {}
    for _ in range(2000):
        r = rng.random()
        try:
            if r < 0.25 and c.slots.available():
                live[c.open()] = 0
            elif r < 0.8 and live:
                s = rng.choice(list(live))
                n = rng.choice([1, 1, 1, 7, 64, 100])
                c.reserve(s, n)
                c.advance(s, n)
                live[s] += n
            elif live:
                s = rng.choice(list(live))
                c.close(s)
                del live[s]
        except CacheError:
            pass
        c.check()
        for s, n in live.items():
            assert c.length[s] == n
    for s in list(live):
        c.close(s)
    c.check()
    assert c.kv_groups[0].pool.available() == 20


# ----------------------------------------------------------------------------- generation loop
class ScriptedBackend:
    """Stands in for the engine: token t of request r is script[r][t]; records what the loop does."""

    def __init__(self, script, capacity_tokens=64 * 8, max_positions=4096):
        self.script, self.capacity_tokens, self.max_positions = script, capacity_tokens, max_positions
        self.free, self.req_of, self.fed, self.log, self.max_live = list(range(100)), {}, {}, [], 0
        self.seeded = []

    def open(self, n):
        slots = [self.free.pop(0) for _ in range(n)]
        self.log.append(("open", tuple(slots)))
        return slots

    def close(self, slots):
        for s in slots:
            assert s in self.req_of, "closed twice or never used"
            del self.req_of[s]
            self.free.insert(0, s)
        self.log.append(("close", tuple(slots)))

    def seed(self, slots, params, first_request_index=0):
        self.seeded.append((tuple(slots), first_request_index))

    def prefill_sampled(self, slots, prompts, params):
        out = []
        for s, p in zip(slots, prompts):
            r = p[0]  # the test's prompts start with their request number
            self.req_of[s], self.fed[r] = r, 0
            out.append(self.script[r][0])
        self.max_live = max(self.max_live, len(self.req_of))
        self.log.append(("prefill", tuple(slots), tuple(len(p) for p in prompts)))
        return out

    def decode_sampled(self, slots, tokens, params):
        out = []
        for s, t in zip(slots, tokens):
            r = self.req_of[s]
            assert t == self.script[r][self.fed[r]], "the loop fed back another token than it was given"
            self.fed[r] += 1
            out.append(self.script[r][self.fed[r]])
        self.log.append(("decode", tuple(slots)))
        return out


def test_loop_decisions():
    EOS = 99
    script = {0: [5, 6, 7, 8, 9, 10], 1: [EOS, 1, 1, 1, 1, 1], 2: [4, 4, EOS, 4, 4, 4], 3: [1, 2, 3, 4, 5, 6], 4: [7, EOS, 7, 7, 7, 7]}
    prompts = [[r] + [0] * r for r in range(5)]
    be = ScriptedBackend(script)
    loop = GenerationLoop(be, SamplingParams(), max_new_tokens=4, stop_ids=[EOS], max_batch=3)
    out = loop.run(prompts)
    assert [g.tokens for g in out] == [[5, 6, 7, 8], [], [4, 4], [1, 2, 3, 4], [7]]
    assert [g.finish_reason for g in out] == ["length", "stop", "stop", "length", "stop"]
    assert be.max_live == 3 and not be.req_of  # never more than max_batch alive; everything given back
    # batch 1 = requests 0,1,2 start together; request 1 leaves after the prompt step, 2 two steps later; then batch 2
    kinds = [l[0] for l in be.log]
    assert kinds.count("prefill") == 2 and be.log[1] == ("prefill", (0, 1, 2), (1, 2, 3))
    decodes = [l[1] for l in be.log if l[0] == "decode"]
    assert decodes[:3] == [(0, 2), (0, 2), (0,)]  # the n-th token is emitted but never fed back: 3 decode steps for 4 tokens
    assert be.log[-1][0] == "close"
    second = [l for l in be.log if l[0] == "open"][1][1]
    assert set(second) <= {0, 1, 2}  # the second batch runs on slots the first gave back
    assert be.seeded == [((0, 1, 2), 0), (second, 3)]
    assert loop.stats.batches == 2 and loop.stats.prefill_tokens == 1 + 2 + 3 + 4 + 5


def test_loop_ignore_eos_and_zero_tokens():
    script = {0: [99, 99, 3]}
    be = ScriptedBackend(script)
    out = GenerationLoop(be, max_new_tokens=3, stop_ids=[99], ignore_eos=True).run([[0]])
    assert out[0].tokens == [99, 99, 3] and out[0].finish_reason == "length"
    assert GenerationLoop(ScriptedBackend(script), max_new_tokens=0).run([[0]])[0].tokens == []


def test_plan_batches():
    assert plan_batches([10, 10, 10, 10, 10], 8, 2, 10_000, 4096) == [[0, 1], [2, 3], [4]]
    # room: each request holds prompt + max_new - 1 tokens rounded up to 64: 128 here; 300 tokens of cache fit two
    assert plan_batches([100, 100, 100], 20, 8, 300, 4096) == [[0, 1], [2]]
    assert plan_batches([60, 60], 5, 8, 128, 4096) == [[0, 1]]
    with pytest.raises(GenerationError, match="context"):
        plan_batches([100], 30, 8, 10_000, 128)
    with pytest.raises(GenerationError, match="cache holds"):
        plan_batches([200], 10, 8, 128, 4096)
    with pytest.raises(GenerationError, match="empty"):
        plan_batches([0], 10, 8, 128, 4096)


def test_sampling_params_and_stream():
    p = SamplingParams()
    assert (p.temperature, p.top_k, p.seed) == (0.0, 40, 42) and p.greedy
    assert SamplingParams(0.8, 1, 1).greedy and not SamplingParams(0.8, 0, 1).greedy
    import plain_llama as plain
    s = plain.Sampler(0.8, 40, 7)
    assert SamplingParams(0.8, 40, 7).initial_state(0) == s.state
    assert SamplingParams(0.8, 40, 7).initial_state(2) == plain.Sampler(0.8, 40, 9).state
    x = s.state
    s.sample([0.0, 1.0, 2.0])
    assert xorshift64(x) == s.state


def test_decode_splits_rule():
    """Blocks per (sequence, kv head) of the decode attention: about two blocks an SM for few pairs; whole waves of
    resident blocks once there are as many pairs as SMs; never less than one, never more than 16."""
    from edgelm_b200.engine.batch import StepContext
    ctx = StepContext(None, None, "cpu", 148)

    def splits(n_seqs, n_kv, resident=None):
        ctx.n_seqs = n_seqs
        return ctx.decode_splits(n_kv, resident)
    assert splits(1, 1) == 16 and splits(2, 3) == 16 and splits(8, 3) == 13 and splits(8, 3, 3) == 13      # few pairs: the caller's knowledge changes nothing
    assert splits(4, 32, 3) == 3                                                    # 128 pairs, under the SMs: ceil(296 / 128)
    assert splits(8, 32) == 2 and splits(8, 32, 3) == 3                             # 256 pairs: two waves of 444 blocks hold 3 splits
    assert splits(16, 32) == 1 and splits(16, 32, 3) == 2                           # 512 pairs: three waves hold 2
    assert splits(64, 32, 3) == 1 and splits(64, 5, 3) == 2 and splits(64, 3, 3) == 2
    assert splits(8, 32, 1) == 2                                                    # one block an SM: nothing fills a wave twice over
    ctx._fixed_splits = 5
    assert splits(8, 32, 3) == 5


def test_capacity_is_the_caches_own_account():
    """Room is counted by the cache: whole pages for key/value groups, nothing for a model whose mixers keep
    fixed-size states only, which is then bound by its slots alone."""
    kv = make_cache(max_tokens=640)
    assert kv.capacity_tokens == 640 and kv.footprint(1) == 64 and kv.footprint(65) == 128 and kv.footprint(0) == 0
    st = SequenceCache([StateNeed((4, 8)), StateNeed((4, 8))], 640, 4096, device=None, max_seqs=3)
    assert st.capacity_tokens is None and st.footprint(5000) == 0 and st.n_slots == 3
    a = st.open()
    st.reserve(a, 3000)          # no pages to run out of
    st.advance(a, 3000)
    st.check()
    assert plan_batches([900, 900, 900, 900], 100, 3, st.capacity_tokens, 4096, st.footprint) == [[0, 1, 2], [3]]
    assert plan_batches([100, 100, 100], 29, 8, kv.capacity_tokens, 256, kv.footprint) == [[0, 1, 2]]
    assert plan_batches([100] * 6, 29, 8, kv.capacity_tokens, 256, kv.footprint) == [[0, 1, 2, 3, 4], [5]]


def test_the_loop_asks_the_backend_for_its_account():
    class StateOnly(ScriptedBackend):
        max_seqs = 2

        def footprint(self, length):
            return 0
    be = StateOnly({0: [5] * 9, 1: [6] * 9, 2: [7] * 9}, capacity_tokens=None)
    loop = GenerationLoop(be, max_new_tokens=3, max_batch=8)
    out = loop.run([[0] * 500, [1] * 700, [2] * 900])
    assert [g.tokens for g in out] == [[5] * 3, [6] * 3, [7] * 3]
    assert be.max_live == 2      # the backend's slots, not the caller's max_batch, bound a batch


def test_a_windowed_group_keeps_the_window_and_one_piece():
    """Two groups with different needs, each with storage of its own: every key, and the last 100 keys.  The windowed
    one gives pages back as a sequence grows, never holds more than the window and one piece of a step, and its
    pool is sized for that."""
    c = SequenceCache([KVNeed(2, 16), KVNeed(2, 16, window=100), KVNeed(2, 16, window=100), None], 64 * 64, 4096, device=None,
                      max_seqs=4, piece_tokens=128)
    full, win = c.kv_groups
    assert full.window is None and win.window == 100 and win.n_entries == 2 and c.piece_tokens == 128
    assert win.pages_per_seq == pages_for(99 + 128) + 1 == 5 and win.n_pages == 4 * 5 and full.n_pages == 64
    s = c.open()
    length = 0
    for piece in [128, 128, 44, 1, 1, 1, 128, 7] + [1] * 150:
        c.reserve(s, piece)
        lo = win.first_page(length)             # the first page a token of this piece sees
        assert all(win.table[s, i] >= 0 for i in range(lo, pages_for(length + piece)))
        c.advance(s, piece)
        length += piece
        c.check()
        assert int(win.n_held[s]) <= win.pages_per_seq
        assert int(full.n_held[s]) == pages_for(length)
        assert all(win.table[s, i] < 0 for i in range(0, win.first_page(length)))    # given back
    assert win.pool.available() == win.n_pages - int(win.n_held[s])
    c.close(s)
    c.check()
    assert win.pool.available() == win.n_pages and full.pool.available() == 64
    # a long prompt is reserved piece by piece: the first call takes the first piece's pages only
    s = c.open()
    c.reserve(s, 1000)
    assert int(win.n_held[s]) == 2 and int(full.n_held[s]) == pages_for(1000)
    c.close(s)
    # the footprint a planner counts is in units of the largest pool
    assert c.footprint(64) == 64 * 4 and c.footprint(4000) == max(pages_for(4000), -(-5 * 64 // 20)) * 64
    only = SequenceCache([KVNeed(2, 16, window=100)], 64 * 64, 4096, device=None, max_seqs=4, piece_tokens=128)
    assert only.footprint(4000) == 16 * 64 and only.capacity_tokens == 64 * 64   # four sequences of any length fit


def test_random_windowed_sequences_never_lose_a_page():
    rng = random.Random(11)
    c = SequenceCache([KVNeed(1, 16, window=70), KVNeed(1, 16)], 40 * 64, 2000, device=None, max_seqs=6, piece_tokens=64)
    live = {}
    for _ in range(1500):
        try:
            r = rng.random()
            if r < 0.2 and c.slots.available():
                live[c.open()] = 0
            elif r < 0.85 and live:
                s = rng.choice(list(live))
                n = rng.choice([1, 1, 1, 5, 64, 33])
                c.reserve(s, n)
                c.advance(s, n)
                live[s] += n
            elif live:
                s = rng.choice(list(live))
                c.close(s)
                del live[s]
        except CacheError:
            pass
        c.check()
    for s in list(live):
        c.close(s)
    c.check()
    assert all(g.pool.available() == g.n_pages for g in c.kv_groups)


def test_a_step_of_one_token_each_reserves_like_one_sequence_at_a_time():
    """`reserve_next` / `advance_next` (a decode step's bookkeeping for all its sequences at once) leave the cache as
    `reserve(slot, 1)` / `advance(slot, 1)` per sequence do: the same tables, lengths, pools and errors, with a full
    group and a windowed one, across page edges, the window's edge and the end of the position table."""
    needs = [KVNeed(2, 16), KVNeed(2, 16, window=70), None]
    a = SequenceCache(needs, 30 * 64, 400, device=None, max_seqs=5, piece_tokens=64)
    b = SequenceCache(needs, 30 * 64, 400, device=None, max_seqs=5, piece_tokens=64)
    starts = [1, 63, 64, 130, 200]
    slots = []
    for c in (a, b):
        slots = [c.open() for _ in starts]
        for s, n in zip(slots, starts):
            c.reserve(s, n)
            c.advance(s, n)
    for step in range(210):
        failed = [None, None]
        try:
            a.reserve_next(slots)
            a.advance_next(slots)
        except CacheError as e:
            failed[0] = str(e)
        try:
            for s in slots:
                b.reserve(s, 1)
            for s in slots:
                b.advance(s, 1)
        except CacheError as e:
            failed[1] = str(e)
        assert failed[0] == failed[1]
        if failed[0]:
            assert "longer than the 400 positions" in failed[0] and step == 200   # the sequence that began at 200
            break
        a.check()
        assert (a.length == b.length).all()
        for ga, gb in zip(a.kv_groups, b.kv_groups):
            assert (ga.n_held == gb.n_held).all() and (ga.low == gb.low).all() and ga.pool.available() == gb.pool.available()
            assert ((ga.table >= 0) == (gb.table >= 0)).all()
    else:
        raise AssertionError("the position table's end was never reached")
    with pytest.raises(CacheError, match="not held"):
        a.reserve_next([slots[0], 4 if 4 not in slots else 99])


def test_the_quiet_steps_of_a_decode_batch_end_when_anything_else_touches_the_cache():
    """Between page edges `reserve_next` answers from a count of steps that need nothing; whatever else touches the
    cache (a sequence opened, closed, or stepped on its own) ends that count, so the next call looks again."""
    rng = random.Random(5)
    needs = [KVNeed(2, 16)]
    a = SequenceCache(needs, 40 * 64, 1000, device=None, max_seqs=6)
    b = SequenceCache(needs, 40 * 64, 1000, device=None, max_seqs=6)
    live = []
    for c in (a, b):
        live = [c.open() for _ in range(3)]
        for s, n in zip(live, (5, 70, 129)):
            c.reserve(s, n)
            c.advance(s, n)
    extra = None
    for step in range(400):
        r = rng.random()
        if r < 0.05 and extra is None:                       # another sequence comes and goes beside the batch
            extra = a.open()
            assert b.open() == extra
            for c in (a, b):
                c.reserve(extra, 64)
                c.advance(extra, 64)
        elif r < 0.1 and extra is not None:
            a.close(extra)
            b.close(extra)
            extra = None
        elif r < 0.13 and len(live) > 1:                     # a sequence of the batch ends
            s = live.pop(rng.randrange(len(live)))
            a.close(s)
            b.close(s)
            with pytest.raises(CacheError, match="not held"):
                a.reserve_next(live + [s])
        a.reserve_next(live)
        a.advance_next(live)
        for s in live:
            b.reserve(s, 1)
        for s in live:
            b.advance(s, 1)
        a.check()
        assert (a.length == b.length).all()
        ga, gb = a.kv_groups[0], b.kv_groups[0]
        assert (ga.n_held == gb.n_held).all() and ga.pool.available() == gb.pool.available() and ((ga.table >= 0) == (gb.table >= 0)).all()
