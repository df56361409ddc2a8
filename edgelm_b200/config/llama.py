"""The Llama decoder's configuration, from its own config.json keys.

Keys and defaults follow adarsh-sgh/edgelm's exporter (tools/export.py:44-54):
num_key_value_heads defaults to the head count, head_dim to hidden_size / heads, rope_theta to
10000, tie_word_embeddings to False, eos/bos ids to 0; rope_scaling must be absent; rms_norm_eps
has no default.  The architecture itself is tools/elm.py:105-161: pre-norm blocks of grouped-
query attention with rotary positions and a SwiGLU feed-forward, RMSNorm everywhere, and a
head that is the embedding when tied.
"""
from dataclasses import dataclass
from typing import Optional, Tuple

from .base import ConfigError, LayerSpec, ModelPlan, PartSpec, ScheduleEntry, optional, require
from .registry import register_architecture


@register_architecture("LlamaForCausalLM", model_type="llama")
@dataclass(frozen=True)
class LlamaConfig:
    vocab_size: int
    hidden_size: int
    intermediate_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    max_position_embeddings: int
    rope_theta: float
    rms_norm_eps: float
    tie_word_embeddings: bool
    bos_token_id: int
    eos_token_ids: Tuple[int, ...]

    architecture = "LlamaForCausalLM"

    @classmethod
    def from_dict(cls, d):
        mt = d.get("model_type", "llama")
        if mt != "llama":
            raise ConfigError(f"config.json: model_type is '{mt}', this class reads 'llama'")
        if d.get("rope_scaling"):
            raise ConfigError("config.json: rope_scaling is set; scaled rotary positions are not part of this architecture's code")
        for key in ("attention_bias", "mlp_bias"):
            if d.get(key):
                raise ConfigError(f"config.json: {key} is true; the projections here have no bias")
        act = d.get("hidden_act", "silu")
        if act != "silu":
            raise ConfigError(f"config.json: hidden_act is '{act}'; the feed-forward here is SwiGLU (silu)")
        nh = require(d, "num_attention_heads", int)
        hidden = require(d, "hidden_size", int)
        eos = d.get("eos_token_id", 0)
        if eos is None:
            eos = 0
        eos_ids = tuple(int(e) for e in eos) if isinstance(eos, (list, tuple)) else (int(eos),)
        if nh <= 0:
            raise ConfigError("config.json: num_attention_heads must be positive")
        cfg = cls(
            vocab_size=require(d, "vocab_size", int),
            hidden_size=hidden,
            intermediate_size=require(d, "intermediate_size", int),
            num_hidden_layers=require(d, "num_hidden_layers", int),
            num_attention_heads=nh,
            num_key_value_heads=optional(d, "num_key_value_heads", int, nh),
            head_dim=optional(d, "head_dim", int, hidden // nh),
            max_position_embeddings=require(d, "max_position_embeddings", int),
            rope_theta=optional(d, "rope_theta", float, 10000.0),
            rms_norm_eps=require(d, "rms_norm_eps", float),
            tie_word_embeddings=optional(d, "tie_word_embeddings", bool, False),
            bos_token_id=optional(d, "bos_token_id", int, 0),
            eos_token_ids=eos_ids,
        )
        cfg.check()
        return cfg

    def check(self):
        for name in ("vocab_size", "hidden_size", "intermediate_size", "num_hidden_layers", "num_attention_heads",
                     "num_key_value_heads", "head_dim", "max_position_embeddings"):
            if getattr(self, name) <= 0:
                raise ConfigError(f"config.json: {name} must be positive, found {getattr(self, name)}")
        if self.num_attention_heads % self.num_key_value_heads:
            raise ConfigError(f"config.json: {self.num_attention_heads} attention heads are not a multiple of "
                              f"{self.num_key_value_heads} key/value heads")
        if self.head_dim % 2:
            raise ConfigError(f"config.json: head_dim {self.head_dim} is odd; rotary positions pair the two halves of a head")
        if not self.rms_norm_eps > 0 or not self.rope_theta > 0:
            raise ConfigError("config.json: rms_norm_eps and rope_theta must be positive")

    def to_dict(self):
        """The config.json this configuration reads back to itself."""
        return {
            "architectures": [self.architecture], "model_type": "llama",
            "vocab_size": self.vocab_size, "hidden_size": self.hidden_size,
            "intermediate_size": self.intermediate_size, "num_hidden_layers": self.num_hidden_layers,
            "num_attention_heads": self.num_attention_heads, "num_key_value_heads": self.num_key_value_heads,
            "head_dim": self.head_dim, "max_position_embeddings": self.max_position_embeddings,
            "rope_theta": self.rope_theta, "rms_norm_eps": self.rms_norm_eps,
            "tie_word_embeddings": self.tie_word_embeddings, "bos_token_id": self.bos_token_id,
            "eos_token_id": self.eos_token_ids[0] if len(self.eos_token_ids) == 1 else list(self.eos_token_ids),
            "hidden_act": "silu", "attention_bias": False, "mlp_bias": False, "rope_scaling": None,
        }

    def plan(self) -> ModelPlan:
        norm = PartSpec("rmsnorm", {"dim": self.hidden_size, "eps": self.rms_norm_eps})
        rope = PartSpec("rope", {"head_dim": self.head_dim, "theta": self.rope_theta,
                                 "max_positions": self.max_position_embeddings})
        mixer = PartSpec("attention", {
            "hidden_size": self.hidden_size, "num_heads": self.num_attention_heads,
            "num_kv_heads": self.num_key_value_heads, "head_dim": self.head_dim, "positions": rope,
            "names": {"q": "self_attn.q_proj.weight", "k": "self_attn.k_proj.weight",
                      "v": "self_attn.v_proj.weight", "o": "self_attn.o_proj.weight"},
        })
        ffn = PartSpec("swiglu", {
            "hidden_size": self.hidden_size, "intermediate_size": self.intermediate_size,
            "names": {"gate": "mlp.gate_proj.weight", "up": "mlp.up_proj.weight", "down": "mlp.down_proj.weight"},
        })
        layers = tuple(
            LayerSpec(prefix=f"model.layers.{l}.", block="prenorm", mixer=mixer,
                      mixer_norm=PartSpec("rmsnorm", {**norm.params, "name": "input_layernorm.weight"}),
                      ffn=ffn, ffn_norm=PartSpec("rmsnorm", {**norm.params, "name": "post_attention_layernorm.weight"}))
            for l in range(self.num_hidden_layers))
        return ModelPlan(
            hidden_size=self.hidden_size, vocab_size=self.vocab_size, max_positions=self.max_position_embeddings,
            embedding=PartSpec("embedding", {"vocab_size": self.vocab_size, "dim": self.hidden_size,
                                             "name": "model.embed_tokens.weight"}),
            layers=layers,
            schedule=tuple(ScheduleEntry(l) for l in range(self.num_hidden_layers)),
            final_norm=PartSpec("rmsnorm", {**norm.params, "name": "model.norm.weight"}),
            head=PartSpec("lm_head", {"vocab_size": self.vocab_size, "dim": self.hidden_size,
                                      "tied_to": "model.embed_tokens.weight" if self.tie_word_embeddings else None,
                                      "name": "lm_head.weight"}),
            stop_token_ids=self.eos_token_ids, bos_token_id=self.bos_token_id,
        ).validate()
