"""config.json contents of the model shapes the benchmarks and the command line can build with
random weights (no checkpoint is needed or read).  These are data, handed to the same
configuration reader as any config.json; no size here is known to model code."""

def _llama(vocab, hidden, inter, layers, heads, kv_heads, head_dim, max_pos, theta, eps, tied):
    return {"architectures": ["LlamaForCausalLM"], "model_type": "llama", "vocab_size": vocab, "hidden_size": hidden,
            "intermediate_size": inter, "num_hidden_layers": layers, "num_attention_heads": heads,
            "num_key_value_heads": kv_heads, "head_dim": head_dim, "max_position_embeddings": max_pos,
            "rope_theta": theta, "rms_norm_eps": eps, "tie_word_embeddings": tied, "bos_token_id": 0, "eos_token_id": 0}


PRESETS = {
    "tiny-a": _llama(256, 64, 128, 2, 4, 2, 16, 128, 10000.0, 1e-5, True),
    "tiny-b": _llama(397, 96, 200, 3, 3, 1, 32, 256, 100000.0, 1e-6, False),
    "smollm2-135m": _llama(49152, 576, 1536, 30, 9, 3, 64, 8192, 100000.0, 1e-5, True),
    "smollm2-360m": _llama(49152, 960, 2560, 32, 15, 5, 64, 8192, 100000.0, 1e-5, True),
    "smollm2-1.7b": _llama(49152, 2048, 8192, 24, 32, 32, 64, 8192, 130000.0, 1e-5, True),
}


def preset_config(name):
    from .config import config_class_for
    if name not in PRESETS:
        raise KeyError(f"unknown preset '{name}'; there are: {', '.join(sorted(PRESETS))}")
    d = PRESETS[name]
    return config_class_for(d).from_dict(d)


def random_model(config, seed=0, sigma=0.02, dtype="bfloat16", device="cuda:0", layers=None):
    """A DecoderModel of `config` with random weights made on the device (matrices N(0, sigma),
    norm weights 1 + N(0, sigma)); `layers` keeps only the plan's first so many layer runs (the configuration
    object stays whole: it is the plan that is cut)."""
    import torch

    from .engine.engine import DTYPES
    from .engine.model import DecoderModel
    from .weights import random_tensors
    plan = config.plan()
    if layers is not None and int(layers) != len(plan.schedule):
        plan = plan.first_runs(layers)
    torch_dtype = DTYPES[dtype] if isinstance(dtype, str) else dtype
    model = DecoderModel(plan, torch_dtype)
    tensors = random_tensors(model.expected_weights(), seed, sigma, torch_dtype, device=device)
    model.load(tensors, device)
    model.config = config
    return model
