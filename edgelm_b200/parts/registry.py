"""Registries of parts: mixers, feed-forwards, norms, position encodings, block arrangements,
embeddings and heads, each under the `kind` that a PartSpec names.

A part is built as `cls(spec, env)`: `spec.params` holds its sizes and constants, `env` the
compute dtype and the factory for shared sub-parts.  No part knows which model it is in.
Anything registered here, from this package or from outside it, can be named by a plan.
"""
from dataclasses import dataclass, field

import torch

from ..config.base import ConfigError, PartSpec

MIXERS, FEED_FORWARDS, NORMS, POSITION_ENCODINGS, BLOCKS, EMBEDDINGS, HEADS = {}, {}, {}, {}, {}, {}, {}
_TABLES = {"mixer": MIXERS, "ffn": FEED_FORWARDS, "norm": NORMS, "positions": POSITION_ENCODINGS, "block": BLOCKS,
           "embedding": EMBEDDINGS, "head": HEADS}


def _register(table, what):
    def outer(kind):
        def deco(cls):
            table[kind] = cls
            cls.kind = kind
            return cls
        return deco
    outer.__doc__ = f"Class decorator: register a {what} under a kind name."
    return outer


register_mixer = _register(MIXERS, "mixer")
register_ffn = _register(FEED_FORWARDS, "feed-forward")
register_norm = _register(NORMS, "norm")
register_positions = _register(POSITION_ENCODINGS, "position encoding")
register_block = _register(BLOCKS, "block arrangement")
register_embedding = _register(EMBEDDINGS, "embedding")
register_head = _register(HEADS, "head")


@dataclass
class BuildEnv:
    """What every part is built with: the compute dtype (float32: everything in true 32-bit;
    bfloat16: matrices, activations and cache in bfloat16 with float32 statistics) and a pool
    of shared sub-parts (one position table per distinct spec)."""
    dtype: torch.dtype
    shared: dict = field(default_factory=dict)

    def build(self, role, spec: PartSpec):
        table = _TABLES[role]
        if spec.kind not in table:
            raise ConfigError(f"no {role} of kind '{spec.kind}' is registered; registered: {', '.join(sorted(table)) or 'none'}")
        return table[spec.kind](spec, self)

    def build_shared(self, role, spec: PartSpec):
        key = (role, spec.key())
        if key not in self.shared:
            self.shared[key] = self.build(role, spec)
        return self.shared[key]
