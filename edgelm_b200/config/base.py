"""What a configuration turns into: a plan of parts, layer by layer, and the order they run in.

An architecture's typed configuration (read from its own config.json keys) produces a
`ModelPlan`.  The plan is plain data: which mixer, feed-forward, norms and block arrangement
each layer has, with every size and constant as a parameter of that part; and a schedule, the
list of layers in the order they run.  A schedule entry may name a layer a second time (the
same weights run again, with a cache entry of its own) or point at an earlier entry whose
cache it reads instead of keeping one.  The generic model (engine/model.py) builds itself
from a plan through the part registries and knows nothing else about the architecture.
"""
from dataclasses import dataclass, field
from typing import Any, Mapping, Optional, Tuple


class ConfigError(ValueError):
    """A config.json that is missing a key, holds a value of the wrong kind, or asks for
    something this architecture's code does not compute."""


@dataclass(frozen=True)
class PartSpec:
    """One part: the name it is registered under and its sizes and constants."""
    kind: str
    params: Mapping[str, Any] = field(default_factory=dict)

    def __getitem__(self, key):
        return self.params[key]

    def get(self, key, default=None):
        return self.params.get(key, default)

    def key(self):
        """Hashable identity, used to share one instance between layers (position tables)."""
        def freeze(v):
            if isinstance(v, PartSpec):
                return v.key()
            if isinstance(v, Mapping):
                return tuple(sorted((k, freeze(x)) for k, x in v.items()))
            if isinstance(v, (list, tuple)):
                return tuple(freeze(x) for x in v)
            return v
        return (self.kind, freeze(self.params))


@dataclass(frozen=True)
class LayerSpec:
    """One layer: its arrangement and its four parts.  `prefix` starts its tensors' names."""
    prefix: str
    block: str
    mixer: PartSpec
    mixer_norm: PartSpec
    ffn: PartSpec
    ffn_norm: PartSpec


@dataclass(frozen=True)
class ScheduleEntry:
    """One run of a layer.  `reads_cache_of` is the index of an earlier schedule entry whose
    cache this run's mixer reads (it then keeps none of its own)."""
    layer: int
    reads_cache_of: Optional[int] = None


@dataclass(frozen=True)
class ModelPlan:
    hidden_size: int
    vocab_size: int
    max_positions: int
    embedding: PartSpec
    layers: Tuple[LayerSpec, ...]
    schedule: Tuple[ScheduleEntry, ...]
    final_norm: PartSpec
    head: PartSpec
    stop_token_ids: Tuple[int, ...] = ()
    bos_token_id: Optional[int] = None

    def first_runs(self, n):
        """The same plan cut to its first `n` schedule entries (and the layers they name): a shallower model of the
        same layer sizes, for runs where the full depth costs too much memory or time."""
        import dataclasses
        n = int(n)
        if not 1 <= n <= len(self.schedule):
            raise ConfigError(f"a plan of {len(self.schedule)} layer runs cannot be cut to {n}")
        schedule = self.schedule[:n]
        used = sorted({e.layer for e in schedule})
        renumber = {old: new for new, old in enumerate(used)}
        return dataclasses.replace(self, layers=tuple(self.layers[i] for i in used),
                                   schedule=tuple(ScheduleEntry(renumber[e.layer], e.reads_cache_of) for e in schedule)).validate()

    def validate(self):
        if not self.layers or not self.schedule:
            raise ConfigError("a model needs at least one layer and one schedule entry")
        for i, e in enumerate(self.schedule):
            if not 0 <= e.layer < len(self.layers):
                raise ConfigError(f"schedule entry {i} names layer {e.layer}; there are {len(self.layers)}")
            if e.reads_cache_of is not None:
                j = e.reads_cache_of
                if not 0 <= j < i:
                    raise ConfigError(f"schedule entry {i} reads the cache of entry {j}, which does not run before it")
                if self.schedule[j].reads_cache_of is not None:
                    raise ConfigError(f"schedule entry {i} reads the cache of entry {j}, which keeps none itself")
        return self


def require(d, key, kind, where="config.json"):
    """d[key] as `kind` (int, float, bool, str); bool is not accepted for a number."""
    if key not in d or d[key] is None:
        raise ConfigError(f"{where}: key '{key}' is missing")
    return coerce(d[key], key, kind, where)


def optional(d, key, kind, default, where="config.json"):
    if key not in d or d[key] is None:
        return default
    return coerce(d[key], key, kind, where)


def coerce(v, key, kind, where="config.json"):
    if kind is bool:
        if isinstance(v, bool):
            return v
    elif kind is int:
        if isinstance(v, int) and not isinstance(v, bool):
            return v
        if isinstance(v, float) and v == int(v):
            return int(v)
    elif kind is float:
        if isinstance(v, (int, float)) and not isinstance(v, bool):
            return float(v)
    elif kind is str:
        if isinstance(v, str):
            return v
    raise ConfigError(f"{where}: key '{key}' should be {kind.__name__}, found {v!r}")
