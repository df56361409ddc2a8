from . import attention, block, embedding, head, norm, rope, swiglu  # noqa: F401  (registration)
from .base import KVNeed, Part, StateNeed
from .registry import (BuildEnv, register_block, register_embedding, register_ffn, register_head, register_mixer,
                       register_norm, register_positions)

__all__ = ["KVNeed", "Part", "StateNeed", "BuildEnv", "register_block", "register_embedding", "register_ffn",
           "register_head", "register_mixer", "register_norm", "register_positions"]
