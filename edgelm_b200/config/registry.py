"""One registry from an architecture's name to its configuration class.

`architectures[0]` of config.json picks the entry; a config.json without that key falls back
to `model_type`.  An architecture registers a class with two things: `from_dict(dict)` that
reads and checks its own keys, and `plan()` that returns the ModelPlan.
"""
import json
import os

from .base import ConfigError

_ARCHITECTURES = {}
_MODEL_TYPES = {}


def register_architecture(name, model_type=None):
    """Class decorator: `@register_architecture("LlamaForCausalLM", model_type="llama")`."""
    def deco(cls):
        for need in ("from_dict", "plan"):
            if not hasattr(cls, need):
                raise TypeError(f"{cls.__name__} lacks {need}(); an architecture's configuration needs from_dict and plan")
        _ARCHITECTURES[name] = cls
        if model_type:
            _MODEL_TYPES[model_type] = cls
        return cls
    return deco


def registered_architectures():
    return sorted(_ARCHITECTURES)


def config_class_for(config_dict):
    archs = config_dict.get("architectures")
    if archs:
        name = archs[0]
        if name in _ARCHITECTURES:
            return _ARCHITECTURES[name]
        raise ConfigError(f"architecture '{name}' is not registered; registered: {', '.join(registered_architectures()) or 'none'}")
    mt = config_dict.get("model_type")
    if mt in _MODEL_TYPES:
        return _MODEL_TYPES[mt]
    raise ConfigError(f"config.json names no registered architecture (architectures={archs!r}, model_type={mt!r}); "
                      f"registered: {', '.join(registered_architectures()) or 'none'}")


def read_config(model_dir_or_file):
    """Typed configuration of the model folder (or of a config.json path)."""
    path = model_dir_or_file
    if os.path.isdir(path):
        path = os.path.join(path, "config.json")
    try:
        with open(path) as f:
            d = json.load(f)
    except FileNotFoundError:
        raise ConfigError(f"no config.json at {path}") from None
    except json.JSONDecodeError as e:
        raise ConfigError(f"{path} is not valid JSON: {e}") from None
    if not isinstance(d, dict):
        raise ConfigError(f"{path} does not hold a JSON object")
    return config_class_for(d).from_dict(d)
