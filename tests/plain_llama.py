"""Plain, slow Llama decoder in NumPy: the oracle that every engine test compares with.

Whole sequences, no cache, one function per part, float32 arithmetic throughout.  It shares
no code with the package under test: it has its own config.json reader, its own safetensors
reader and its own sampler.  Every function is a restatement of a formula of
adarsh-sgh/edgelm; the file:line after each name is the place in that project where the
formula stands.  `tests/golden/make_golden.py` ran edgelm's own NumPy model
(tools/reference.py, imported on the CPU) against this file once; the outputs it wrote are
committed under tests/golden/ and checked by tests/test_plain.py.
"""
import json
import os
import struct

import numpy as np

f32 = np.float32


# ----------------------------------------------------------------------------- config
def read_config(model_dir):
    """config.json -> dict of the sizes and constants the formulas need.

    Keys and defaults as tools/export.py:44-54: num_key_value_heads defaults to the head
    count, head_dim to hidden/heads, rope_theta to 10000, tie_word_embeddings to False;
    rope_scaling must be absent.
    """
    with open(os.path.join(model_dir, "config.json")) as f:
        c = json.load(f)
    assert c["model_type"] == "llama"
    assert not c.get("rope_scaling")
    nh = c["num_attention_heads"]
    return dict(
        vocab=c["vocab_size"], dim=c["hidden_size"], inter=c["intermediate_size"],
        n_layers=c["num_hidden_layers"], n_heads=nh,
        n_kv_heads=c.get("num_key_value_heads", nh),
        head_dim=c.get("head_dim", c["hidden_size"] // nh),
        max_pos=c["max_position_embeddings"],
        theta=float(c.get("rope_theta", 10000.0)), eps=float(c["rms_norm_eps"]),
        tied=bool(c.get("tie_word_embeddings", False)),
        eos=c.get("eos_token_id", 0) or 0,
    )


# ----------------------------------------------------------------------------- weights
def read_safetensors(path):
    """name -> float32 ndarray (tools/export.py:18-41): u64 LE header length, JSON header,
    data_offsets relative to the end of the header; BF16 widened by a 16-bit shift."""
    with open(path, "rb") as f:
        raw = f.read()
    (n,) = struct.unpack("<Q", raw[:8])
    header = json.loads(raw[8:8 + n])
    base = 8 + n
    out = {}
    for name, meta in header.items():
        if name == "__metadata__":
            continue
        b, e = meta["data_offsets"]
        buf = np.frombuffer(raw, dtype=np.uint8, count=e - b, offset=base + b)
        dt = meta["dtype"]
        if dt == "BF16":
            a = (buf.view(np.uint16).astype(np.uint32) << 16).view(np.float32)
        elif dt == "F16":
            a = buf.view(np.float16).astype(np.float32)
        elif dt == "F32":
            a = buf.view(np.float32).copy()
        else:
            raise ValueError(f"{name}: unsupported dtype {dt}")
        out[name] = a.reshape(meta["shape"])
    return out


def read_model(model_dir):
    cfg = read_config(model_dir)
    W = {}
    for fn in sorted(os.listdir(model_dir)):  # tools/export.py:57-63
        if fn.endswith(".safetensors"):
            W.update(read_safetensors(os.path.join(model_dir, fn)))
    return cfg, W


def bf16_round(a):
    """float32 -> nearest bfloat16 (ties to even) -> float32.  Not in edgelm (it has no
    reduced-precision floats); used to give the oracle the same weights a bfloat16 file holds."""
    u = np.ascontiguousarray(a, dtype=np.float32).view(np.uint32).astype(np.uint64)
    r = ((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint32) << 16
    return r.astype(np.uint32).view(np.float32).reshape(np.shape(a))


# ----------------------------------------------------------------------------- parts
def embed(table, ids):
    """x[t] = E[id_t], ids range-checked (src/kernels_ref.cpp:41-46, tools/reference.py:76-78)."""
    ids = np.asarray(ids)
    assert ids.min() >= 0 and ids.max() < table.shape[0], "token id out of range"
    return table[ids].astype(f32)


def rmsnorm(x, w, eps):
    """y = x * (1/sqrt(mean(x^2) + eps)) * w (src/kernels_ref.cpp:48-56, tools/reference.py:11-14)."""
    x = x.astype(f32)
    ms = np.mean(x * x, axis=-1, keepdims=True, dtype=f32)
    inv = f32(1.0) / np.sqrt(ms + f32(eps))
    return (x * inv).astype(f32) * w.astype(f32)


def rope_angles(positions, hd, theta):
    """cos/sin [len(positions), hd/2]; inverse frequencies and angles in float64, then
    rounded to float32 (src/kernels_ref.cpp:11-21, tools/reference.py:17-20)."""
    i = np.arange(0, hd, 2, dtype=np.float64)
    inv = np.power(np.float64(theta), -(i / hd))
    ang = np.asarray(positions, dtype=np.float64)[:, None] * inv[None, :]
    return np.cos(ang).astype(f32), np.sin(ang).astype(f32)


def rope(x, positions, n_heads, hd, theta):
    """Half-split pairing (i, i+hd/2): y_i = a c - b s, y_{i+hd/2} = b c + a s
    (src/kernels_ref.cpp:82-98, tools/reference.py:23-31)."""
    t = x.shape[0]
    c, s = rope_angles(positions, hd, theta)
    x = x.reshape(t, n_heads, hd)
    h = hd // 2
    a, b = x[..., :h], x[..., h:]
    c, s = c[:, None, :], s[:, None, :]
    y = np.concatenate([a * c - b * s, b * c + a * s], axis=-1)
    return y.reshape(t, n_heads * hd).astype(f32)


def attention(q, k, v, n_heads, n_kv, hd):
    """Causal softmax(q k^T / sqrt(hd)) v over the whole sequence; query head h reads key
    head h // (n_heads / n_kv); the scale is applied after the dot product
    (src/kernels_ref.cpp:119-140, tools/reference.py:34-53)."""
    t = q.shape[0]
    q = q.reshape(t, n_heads, hd)
    k = k.reshape(t, n_kv, hd)
    v = v.reshape(t, n_kv, hd)
    grp = n_heads // n_kv
    scale = f32(1.0 / np.sqrt(hd))
    out = np.zeros((t, n_heads, hd), dtype=f32)
    future = np.arange(t)[None, :] > np.arange(t)[:, None]
    for h in range(n_heads):
        kh, vh = k[:, h // grp, :], v[:, h // grp, :]
        sc = (q[:, h, :] @ kh.T).astype(f32) * scale
        sc[future] = -np.inf
        sc = sc - sc.max(axis=1, keepdims=True)
        p = np.exp(sc).astype(f32)
        p = p / p.sum(axis=1, keepdims=True)
        out[:, h, :] = p @ vh
    return out.reshape(t, n_heads * hd)


def silu(x):
    """z / (1 + exp(-z)) (src/kernels_ref.cpp:146-148, tools/reference.py:56-57)."""
    return (x / (f32(1.0) + np.exp(-x))).astype(f32)


def swiglu_mlp(h, wg, wu, wd):
    """down(silu(gate(h)) * up(h)), no bias (src/kernels_ref.cpp:153-160, tools/elm.py:140-152)."""
    return ((silu(h @ wg.T) * (h @ wu.T)).astype(f32) @ wd.T).astype(f32)


def decoder_layer(cfg, W, l, x):
    """Pre-norm block: x1 = x + O(attn(...N1 x)); x2 = x1 + MLP(N2 x1)
    (tools/elm.py:122-153, tools/reference.py:79-91)."""
    p = f"model.layers.{l}."
    nh, nkv, hd = cfg["n_heads"], cfg["n_kv_heads"], cfg["head_dim"]
    pos = np.arange(x.shape[0])
    h = rmsnorm(x, W[p + "input_layernorm.weight"], cfg["eps"])
    q = h @ W[p + "self_attn.q_proj.weight"].T
    k = h @ W[p + "self_attn.k_proj.weight"].T
    v = h @ W[p + "self_attn.v_proj.weight"].T
    q = rope(q, pos, nh, hd, cfg["theta"])
    k = rope(k, pos, nkv, hd, cfg["theta"])
    a = attention(q, k, v, nh, nkv, hd)
    x = (x + a @ W[p + "self_attn.o_proj.weight"].T).astype(f32)
    h2 = rmsnorm(x, W[p + "post_attention_layernorm.weight"], cfg["eps"])
    m = swiglu_mlp(h2, W[p + "mlp.gate_proj.weight"], W[p + "mlp.up_proj.weight"],
                   W[p + "mlp.down_proj.weight"])
    return (x + m).astype(f32)


def lm_head(cfg, W, x):
    """Final norm, then logits = xn H^T with H the embedding when tied
    (tools/elm.py:154-160, tools/reference.py:92-94)."""
    xn = rmsnorm(x, W["model.norm.weight"], cfg["eps"])
    head = W["model.embed_tokens.weight"] if cfg["tied"] else W["lm_head.weight"]
    return (xn @ head.T).astype(f32)


def forward(cfg, W, tokens, rows=None):
    """Logits [len(tokens), vocab] for every position of one whole sequence, or [len(rows), vocab] for
    the positions `rows` (edgelm's LAST_ROWS idea, tools/elm.py:154-156: the layers run on every position,
    the head only where logits are wanted; with a large vocabulary the head is most of the work)."""
    x = hidden(cfg, W, tokens)
    return lm_head(cfg, W, x if rows is None else x[np.asarray(rows, dtype=np.int64)])


def hidden(cfg, W, tokens):
    """The residual stream [len(tokens), dim] after the last layer, before the final norm."""
    W = {k: np.asarray(v, dtype=f32) for k, v in W.items()}
    x = embed(W["model.embed_tokens.weight"], tokens)
    for l in range(cfg["n_layers"]):
        x = decoder_layer(cfg, W, l, x)
    return x


# ----------------------------------------------------------------------------- sampling
def argmax(logits):
    """Index of the first maximum (src/tokenizer.cpp:187-189)."""
    return int(np.argmax(np.asarray(logits)))


MASK64 = (1 << 64) - 1


class Sampler:
    """Greedy when temperature <= 0 or top_k == 1; else top-k (k <= 0: whole vocabulary),
    p_i = exp((l_i - l_0) / T), one xorshift64 draw, inverse-CDF walk in descending order
    (src/tokenizer.cpp:191-211).  Equal logits are ordered by lower index first (edgelm's
    partial_sort leaves that order open)."""

    def __init__(self, temperature=0.0, top_k=40, seed=42):
        self.temperature = float(temperature)
        self.top_k = int(top_k)
        self.state = (int(seed) * 0x9E3779B97F4A7C15 + 1) & MASK64

    def sample(self, logits):
        logits = np.asarray(logits, dtype=f32)
        n = logits.shape[0]
        if self.temperature <= 0.0 or self.top_k == 1:
            return argmax(logits)
        k = min(self.top_k, n) if self.top_k > 0 else n
        order = np.argsort(-logits.astype(np.float64), kind="stable")[:k]
        top = logits[order]
        p = np.exp(((top - top[0]) / f32(self.temperature)).astype(f32)).astype(np.float64)
        total = 0.0
        for x in p:
            total += float(x)
        s = self.state
        s ^= (s << 13) & MASK64
        s ^= s >> 7
        s ^= (s << 17) & MASK64
        self.state = s
        r = (s >> 11) * (1.0 / 9007199254740992.0) * total
        for i in range(k):
            r -= float(p[i])
            if r <= 0:
                return int(order[i])
        return int(order[k - 1])


def generate(cfg, W, prompt, max_new_tokens, temperature=0.0, top_k=40, seed=42,
             stop_ids=None, ignore_eos=False):
    """edgelm's run loop (src/main.cpp:149-163) on whole-sequence forwards: sample from the
    last position; a stop token ends the sequence and is not emitted; at most
    max_new_tokens are emitted and the last one is never fed back."""
    stop = set([cfg["eos"]] if stop_ids is None else stop_ids)
    sampler = Sampler(temperature, top_k, seed)
    seq = list(prompt)
    out = []
    for _ in range(max_new_tokens):
        nxt = sampler.sample(forward(cfg, W, seq)[-1])
        if nxt in stop and not ignore_eos:
            break
        out.append(nxt)
        seq.append(nxt)
    return out
