"""The generation loop: requests in, tokens out, batch after batch.

One batch at a time.  Its sequences start together with prompts of any lengths (one step), then
decode one token each per step.  After every step the loop decides, per sequence, as
adarsh-sgh/edgelm's run command does (src/main.cpp:149-163): a stop token ends the sequence and
is not emitted (unless stops are ignored); otherwise the token is emitted; a sequence that has
emitted `max_new_tokens` ends without its last token being fed back.  A sequence that ends
leaves the batch at once and gives back what it holds; no other request joins a running
batch.  When the batch is empty the next one starts, on the slots just freed, until every
request is served.

The loop talks to a backend with six methods (open, close, seed, prefill_sampled,
decode_sampled, and the two capacity attributes); the engine is one, and the tests drive the
loop's decisions with a scripted one on the CPU.
"""
import time
from dataclasses import dataclass, field
from typing import List, Optional, Sequence

from ..cache.cache import PAGE
from ..sampling.params import SamplingParams


class GenerationError(ValueError):
    pass


@dataclass
class Generation:
    prompt_len: int
    tokens: List[int] = field(default_factory=list)
    finish_reason: Optional[str] = None  # "stop" or "length"


@dataclass
class GenerationStats:
    batches: int = 0
    prefill_tokens: int = 0
    prefill_s: float = 0.0      # time to the first sampled token of each batch, summed
    decode_tokens: int = 0
    decode_steps: int = 0
    decode_s: float = 0.0

    def summary(self):
        pf = self.prefill_tokens / self.prefill_s if self.prefill_s > 0 else 0.0
        dc = self.decode_tokens / self.decode_s if self.decode_s > 0 else 0.0
        return (f"{self.batches} batch(es), prompt {self.prefill_tokens} tok, TTFT {self.prefill_s * 1e3:.1f} ms "
                f"(prefill {pf:.1f} tok/s), decode {self.decode_tokens} tok in {self.decode_steps} steps {dc:.1f} tok/s")


def round_up_page(n):
    return (int(n) + PAGE - 1) // PAGE * PAGE


def plan_batches(prompt_lens: Sequence[int], max_new_tokens: int, max_batch: int, capacity_tokens: Optional[int],
                 max_positions: int, footprint=round_up_page) -> List[List[int]]:
    """Requests, in order, into batches: at most `max_batch` sequences, and room in the cache for
    every sequence at its longest (prompt + max_new_tokens - 1 tokens are ever written).  How much
    room a sequence of some length takes is the cache's own account (`footprint`; by default whole
    pages of 64 tokens), and so is the room there is (`capacity_tokens`; None: no bound but the
    number of sequences).  A request that cannot fit even alone is refused here, before anything runs."""
    if max_batch < 1:
        raise GenerationError("max_batch must be at least 1")
    if capacity_tokens is None:
        capacity_tokens = float("inf")
    batches, cur, cur_tokens = [], [], 0
    for i, n in enumerate(prompt_lens):
        if n < 1:
            raise GenerationError(f"request {i} has an empty prompt")
        if n + max_new_tokens > max_positions:
            raise GenerationError(f"request {i}: prompt of {n} tokens + {max_new_tokens} new tokens exceeds the context of {max_positions}")
        need = footprint(n + max(max_new_tokens - 1, 0))
        if need > capacity_tokens:
            raise GenerationError(f"request {i} needs room for {need} tokens; the cache holds {capacity_tokens}")
        if cur and (len(cur) == max_batch or cur_tokens + need > capacity_tokens):
            batches.append(cur)
            cur, cur_tokens = [], 0
        cur.append(i)
        cur_tokens += need
    if cur:
        batches.append(cur)
    return batches


class GenerationLoop:
    def __init__(self, backend, params: SamplingParams = SamplingParams(), max_new_tokens=64, stop_ids=(),
                 ignore_eos=False, max_batch=64):
        self.backend, self.params = backend, params
        self.max_new_tokens = int(max_new_tokens)
        self.stop_ids = frozenset(int(s) for s in stop_ids)
        self.ignore_eos = bool(ignore_eos)
        self.max_batch = int(max_batch)
        self.stats = GenerationStats()

    def _decide(self, gen: Generation, token: int):
        """What a freshly sampled token means for its sequence: returns True if it goes on."""
        if token in self.stop_ids and not self.ignore_eos:
            gen.finish_reason = "stop"
            return False
        gen.tokens.append(int(token))
        if len(gen.tokens) >= self.max_new_tokens:
            gen.finish_reason = "length"
            return False
        return True

    def run(self, prompts: Sequence[Sequence[int]]) -> List[Generation]:
        results = [Generation(prompt_len=len(p)) for p in prompts]
        if self.max_new_tokens <= 0:
            for g in results:
                g.finish_reason = "length"
            return results
        be = self.backend
        batches = plan_batches([len(p) for p in prompts], self.max_new_tokens, min(self.max_batch, getattr(be, "max_seqs", self.max_batch)),
                               be.capacity_tokens, be.max_positions, getattr(be, "footprint", round_up_page))
        for batch in batches:
            self._run_batch(batch, prompts, results)
        return results

    def _run_batch(self, batch, prompts, results):
        be = self.backend
        slots = be.open(len(batch))
        live = dict(zip(batch, slots))  # request index -> slot, in batch order
        try:
            be.seed(slots, self.params, first_request_index=batch[0])
            t0 = time.perf_counter()
            tokens = be.prefill_sampled(slots, [list(prompts[i]) for i in batch], self.params)
            self.stats.batches += 1
            self.stats.prefill_tokens += sum(len(prompts[i]) for i in batch)
            self.stats.prefill_s += time.perf_counter() - t0
            t1 = time.perf_counter()
            while True:
                going, feed = [], []
                for i, tok in zip(list(live), tokens):
                    if self._decide(results[i], int(tok)):
                        going.append(i)
                        feed.append(int(tok))
                    else:
                        be.close([live.pop(i)])  # ends earlier: leaves the batch now
                if not going:
                    break
                tokens = be.decode_sampled([live[i] for i in going], feed, self.params)
                self.stats.decode_steps += 1
                self.stats.decode_tokens += len(going)
            self.stats.decode_s += time.perf_counter() - t1
        finally:
            if live:
                be.close(list(live.values()))
