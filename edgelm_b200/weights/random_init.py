"""Random-weights mode: a model folder (config.json, model.safetensors) from a configuration
and a seed.

Matrices (embedding and head included) are N(0, sigma), vectors (norm weights) 1 + N(0, sigma),
drawn on the CPU from one torch generator in the order of the model's own list of expected
tensors, then rounded to the file's dtype.  The folder is what any other model folder is: the
loader reads it back by tensor name.
"""
import json
import os

import torch

from . import safetensors_io

_FILE_DTYPES = {"bfloat16": torch.bfloat16, "float32": torch.float32, "bf16": torch.bfloat16, "fp32": torch.float32,
                "f32": torch.float32}


def random_tensors(expected, seed, sigma=0.02, dtype=torch.bfloat16, device="cpu"):
    """name -> random tensor for every expected (name -> shape)."""
    if device != "cpu":
        gen = torch.Generator(device=device).manual_seed(int(seed))
    else:
        gen = torch.Generator().manual_seed(int(seed))
    out = {}
    for name, shape in expected.items():
        t = torch.randn(tuple(shape), generator=gen, dtype=torch.float32, device=device) * sigma
        if len(shape) == 1:
            t += 1.0
        out[name] = t.to(dtype)
    return out


def write_model_dir(model_dir, config, seed, sigma=0.02, dtype="bfloat16"):
    """Write config.json and model.safetensors for `config` (a registered architecture's
    configuration object) with random weights; returns the folder."""
    from ..engine.model import expected_weights  # the model's own list of tensor names and shapes
    file_dtype = _FILE_DTYPES[dtype] if isinstance(dtype, str) else dtype
    os.makedirs(model_dir, exist_ok=True)
    expected = expected_weights(config.plan())
    tensors = random_tensors(expected, seed, sigma, file_dtype)
    with open(os.path.join(model_dir, "config.json"), "w") as f:
        json.dump(config.to_dict(), f, indent=1)
    safetensors_io.write_file(os.path.join(model_dir, "model.safetensors"), tensors,
                              metadata={"format": "pt", "seed": seed, "sigma": sigma})
    return model_dir
