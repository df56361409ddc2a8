"""The two tiny models and token streams behind the committed golden files.

Weights come from an integer hash, so that they are the same bits on every machine and
NumPy version: make_golden.py (which ran edgelm's own code once) and test_plain.py (which
checks the plain implementation against what that run wrote) both call this file.
"""
import numpy as np

TINY_A = dict(vocab=256, dim=64, inter=128, n_layers=2, n_heads=4, n_kv_heads=2, head_dim=16,
              max_pos=128, theta=10000.0, eps=1e-5, tied=True, eos=0, sigma=0.02, seed=0)
TINY_B = dict(vocab=397, dim=96, inter=200, n_layers=3, n_heads=3, n_kv_heads=1, head_dim=32,
              max_pos=256, theta=100000.0, eps=1e-6, tied=False, eos=0, sigma=0.05, seed=2)


def _hash_u32(idx, salt):
    x = idx.astype(np.uint64) + np.uint64((int(salt) * 0x9E3779B97F4A7C15) & 0xFFFFFFFFFFFFFFFF)
    x ^= x >> np.uint64(30)
    x = x * np.uint64(0xBF58476D1CE4E5B9)
    x ^= x >> np.uint64(27)
    x = x * np.uint64(0x94D049BB133111EB)
    x ^= x >> np.uint64(31)
    return (x >> np.uint64(32)).astype(np.uint32)


def _uniform_pm1(n, salt):
    """n values in (-1, 1), each a multiple of 2^-15 (exact in float32 and in bfloat16 after scaling by 1)."""
    u = _hash_u32(np.arange(n, dtype=np.uint64), salt)
    return ((u >> np.uint32(16)).astype(np.int64) - 32768 + 0.5).astype(np.float64) / 32768.0


def weights(cfg):
    """name -> float32 array; matrices sigma*sqrt(3)*U(-1,1) (variance sigma^2), norm weights 1 + that."""
    D, I, V = cfg["dim"], cfg["inter"], cfg["vocab"]
    qd, kd = cfg["n_heads"] * cfg["head_dim"], cfg["n_kv_heads"] * cfg["head_dim"]
    shapes = {"model.embed_tokens.weight": (V, D), "model.norm.weight": (D,)}
    for l in range(cfg["n_layers"]):
        p = f"model.layers.{l}."
        shapes[p + "input_layernorm.weight"] = (D,)
        shapes[p + "post_attention_layernorm.weight"] = (D,)
        shapes[p + "self_attn.q_proj.weight"] = (qd, D)
        shapes[p + "self_attn.k_proj.weight"] = (kd, D)
        shapes[p + "self_attn.v_proj.weight"] = (kd, D)
        shapes[p + "self_attn.o_proj.weight"] = (D, qd)
        shapes[p + "mlp.gate_proj.weight"] = (I, D)
        shapes[p + "mlp.up_proj.weight"] = (I, D)
        shapes[p + "mlp.down_proj.weight"] = (D, I)
    if not cfg["tied"]:
        shapes["lm_head.weight"] = (V, D)
    amp = cfg["sigma"] * np.sqrt(3.0)
    # larger weights than sigma alone would give: logits of order 1, so that a wrong formula shows
    W = {}
    for i, (name, shp) in enumerate(shapes.items()):
        n = int(np.prod(shp))
        u = _uniform_pm1(n, cfg["seed"] * 1000 + i).reshape(shp)
        if len(shp) == 1:
            W[name] = (1.0 + amp * u).astype(np.float32)
        else:
            W[name] = (amp * 8.0 * u).astype(np.float32)
    return W


def tokens(cfg, n, salt):
    return (_hash_u32(np.arange(n, dtype=np.uint64), 7777 + salt) % np.uint32(cfg["vocab"])).astype(np.int64)


def sampler_logits(n_rows, vocab, salt):
    """Logit rows for the sampler golden, with a few exact ties in each row."""
    x = _uniform_pm1(n_rows * vocab, 4242 + salt).reshape(n_rows, vocab) * 6.0
    x = np.round(x * 8.0) / 8.0  # coarse grid: many equal values
    return x.astype(np.float32)
