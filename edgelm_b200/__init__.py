"""edgelm_b200: a small Llama inference library for one NVIDIA B200 (sm_100a).

Everything between a request's tokens and its next token: a typed configuration read from
config.json, weights from safetensors by tensor name, layers put together from parts, a paged
cache with a slot per sequence, one step function, a generation loop and a sampler, on
hand-written CUDA kernels.  The Python entry points below follow adarsh-sgh/edgelm's own
manner: a `Session` that prefills and decodes one sequence and hands out logits
(include/edgelm/runtime.hpp:28-49), sampling options named as its `run` command names them
(src/main.cpp:74-86), and `generate` for whole batches of requests.
"""
import importlib
import os

from .config import ConfigError, LlamaConfig, read_config, register_architecture, registered_architectures
from .sampling import SamplingParams
from .weights import WeightsError, write_model_dir

__version__ = "0.1.0"


def load_plugins(names=None):
    """Import modules that register parts or architectures of their own, so that every program of the package (the
    command line, bin/trace_run, bench.py) knows them without a change to the package's files.  `names`: a list of
    "module" or "module:function" (the function is called once the module is imported); by default the
    comma-separated list in the environment variable EDGELM_B200_PLUGINS."""
    if names is None:
        names = [n.strip() for n in os.environ.get("EDGELM_B200_PLUGINS", "").split(",") if n.strip()]
    for name in names:
        module, _, fn = name.partition(":")
        m = importlib.import_module(module)
        if fn:
            getattr(m, fn)()


def load_engine(model, dtype="bfloat16", ctx=1024, slots=8, max_tokens=None, batch=8192, profile=False, device="cuda:0",
                use_graphs=True):
    """An Engine for a model folder.  `ctx` is the longest sequence, `slots` how many sequences
    may live at once (together they size the cache, unless `max_tokens` gives its size in
    tokens directly); `batch` is the most tokens one forward runs (longer steps are cut)."""
    from .engine.engine import Engine, load_model
    m = load_model(model, dtype, device) if isinstance(model, str) else model
    ctx = min(int(ctx), m.plan.max_positions)
    if max_tokens is None:
        max_tokens = (ctx + 63) // 64 * 64 * int(slots)
    return Engine(m, max_tokens, max_step_tokens=batch, max_seqs=None, profile=profile, use_graphs=use_graphs)


def generate(model, prompts, n=64, temp=0.0, top_k=40, seed=42, stop=None, ignore_eos=False, dtype="bfloat16",
             ctx=1024, slots=8, engine=None, return_details=False):
    """Generate up to `n` tokens for every prompt (lists of token ids).

    `model` is a model folder; or pass a ready `engine`.  Options as edgelm's run command:
    temp (0 = greedy), top_k (40; <= 0 whole vocabulary), seed (42); `stop` defaults to the
    model's eos ids.  Prompts run in batches of at most `slots` sequences, one batch after
    another.  Returns a list of token lists (or Generation records with return_details)."""
    from .engine.generate import GenerationLoop
    eng = engine or load_engine(model, dtype=dtype, ctx=ctx, slots=slots)
    stop_ids = eng.plan.stop_token_ids if stop is None else stop
    loop = GenerationLoop(eng, SamplingParams(float(temp), int(top_k), int(seed)), max_new_tokens=n, stop_ids=stop_ids,
                          ignore_eos=ignore_eos, max_batch=slots)
    out = loop.run(prompts)
    generate.last_stats = loop.stats
    return out if return_details else [g.tokens for g in out]


class Session:
    """One sequence through the step function, in the manner of edgelm's Session
    (include/edgelm/runtime.hpp:28-49): prefill(tokens) and decode(token) return the logits of
    the last position (all positions with all_logits=True); reset() starts over; pos is the
    number of tokens in the cache."""

    def __init__(self, model, dtype="bfloat16", max_ctx=1024, max_batch=128, all_logits=False, profile=False, engine=None):
        self.engine = engine or load_engine(model, dtype=dtype, ctx=max_ctx, slots=1, batch=max_batch, profile=profile)
        self.all_logits = all_logits
        self.slot = self.engine.open(1)[0]

    @property
    def pos(self):
        return self.engine.length(self.slot)

    def forward(self, tokens):
        from .engine.engine import StepEntry
        tokens = [int(t) for t in tokens]
        want = list(range(len(tokens))) if self.all_logits else [len(tokens) - 1]
        return self.engine.step([StepEntry(self.slot, tokens, want)])

    def prefill(self, tokens):
        return self.forward(tokens)

    def decode(self, token):
        return self.forward([token])

    def reset(self):
        self.engine.close([self.slot])
        self.slot = self.engine.open(1)[0]


load_plugins()

__all__ = ["load_plugins", "ConfigError", "LlamaConfig", "read_config", "register_architecture", "registered_architectures",
           "SamplingParams", "WeightsError", "write_model_dir", "load_engine", "generate", "Session"]
