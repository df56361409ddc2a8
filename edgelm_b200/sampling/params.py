"""Sampling options, with adarsh-sgh/edgelm's names, defaults and meanings
(include/edgelm/tokenizer.hpp:33-37, src/tokenizer.cpp:191-211): temperature 0 is greedy,
top_k 40 (<= 0: the whole vocabulary, 1: greedy), seed 42."""
from dataclasses import dataclass

MASK64 = (1 << 64) - 1
GOLDEN = 0x9E3779B97F4A7C15


@dataclass(frozen=True)
class SamplingParams:
    temperature: float = 0.0
    top_k: int = 40
    seed: int = 42

    @property
    def greedy(self):
        return self.temperature <= 0.0 or self.top_k == 1

    def key(self):
        return ("greedy",) if self.greedy else (float(self.temperature), int(self.top_k))

    def initial_state(self, request_index=0):
        """xorshift64 state of a request's stream: edgelm seeds one sampler with
        seed * 0x9E3779B97F4A7C15 + 1 (src/tokenizer.cpp:191); request i of a call uses seed + i,
        so that request 0 draws edgelm's own stream and no two requests share one."""
        return ((int(self.seed) + int(request_index)) * GOLDEN + 1) & MASK64


def xorshift64(state):
    """One step of the generator (src/tokenizer.cpp:201-203); returns the new state."""
    s = state & MASK64
    s ^= (s << 13) & MASK64
    s ^= s >> 7
    s ^= (s << 17) & MASK64
    return s
