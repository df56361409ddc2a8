"""Configuration, registry and weights: what is read, what is refused, and how errors read."""
import json
import struct

import pytest
import torch

from edgelm_b200.config import ConfigError, LlamaConfig, read_config, register_architecture, registered_architectures
from edgelm_b200.config.base import LayerSpec, ModelPlan, PartSpec, ScheduleEntry
from edgelm_b200.engine.model import DecoderModel, expected_weights
from edgelm_b200.weights import WeightsError, check, keep_dtype, load_checked, read_dir, write_file, write_model_dir

import helpers as H


def write_cfg(tmp_path, d):
    (tmp_path / "config.json").write_text(json.dumps(d))
    return str(tmp_path)


def test_llama_keys_and_defaults(tmp_path):
    d = dict(H.TINY_B)
    for k in ("num_key_value_heads", "head_dim", "rope_theta", "tie_word_embeddings", "bos_token_id", "eos_token_id"):
        d.pop(k)
    c = read_config(write_cfg(tmp_path, d))
    assert isinstance(c, LlamaConfig)
    assert c.num_key_value_heads == 3 and c.head_dim == 32 and c.rope_theta == 10000.0
    assert c.tie_word_embeddings is False and c.eos_token_ids == (0,) and c.bos_token_id == 0
    full = read_config(write_cfg(tmp_path, H.TINY_B))
    assert (full.vocab_size, full.hidden_size, full.intermediate_size, full.num_hidden_layers) == (397, 96, 200, 3)
    assert (full.num_attention_heads, full.num_key_value_heads, full.head_dim) == (3, 1, 32)
    assert full.rope_theta == 100000.0 and full.rms_norm_eps == 1e-6 and full.eos_token_ids == (2,)
    assert read_config(write_cfg(tmp_path, full.to_dict())) == full  # what it writes, it reads back


def test_head_dim_need_not_divide_hidden(tmp_path):
    d = dict(H.TINY_A, head_dim=48, num_attention_heads=3, num_key_value_heads=3)
    c = read_config(write_cfg(tmp_path, d))
    w = expected_weights(c.plan())
    assert w["model.layers.0.self_attn.q_proj.weight"] == (144, 64)
    assert w["model.layers.0.self_attn.o_proj.weight"] == (64, 144)


@pytest.mark.parametrize("change,match", [
    ({"rms_norm_eps": None}, "rms_norm_eps"), ({"vocab_size": None}, "vocab_size"),
    ({"rope_scaling": {"type": "linear", "factor": 2}}, "rope_scaling"), ({"num_key_value_heads": 3}, "multiple"),
    ({"head_dim": 15}, "odd"), ({"hidden_size": "64"}, "hidden_size"), ({"num_hidden_layers": 0}, "positive"),
    ({"attention_bias": True}, "bias"), ({"hidden_act": "gelu"}, "hidden_act"), ({"tie_word_embeddings": 1}, "tie_word"),
    ({"architectures": ["MambaForCausalLM"]}, "not registered"),
])
def test_config_errors(tmp_path, change, match):
    d = dict(H.TINY_A)
    for k, v in change.items():
        if v is None:
            d.pop(k)
        else:
            d[k] = v
    with pytest.raises(ConfigError, match=match):
        read_config(write_cfg(tmp_path, d))


def test_registry_by_name_and_model_type(tmp_path):
    assert "LlamaForCausalLM" in registered_architectures()
    d = dict(H.TINY_A)
    d.pop("architectures")
    assert isinstance(read_config(write_cfg(tmp_path, d)), LlamaConfig)  # falls back to model_type
    with pytest.raises(ConfigError, match="no config.json"):
        read_config(str(tmp_path / "nowhere"))
    with pytest.raises(TypeError):
        register_architecture("Broken")(type("X", (), {}))


def test_plan_is_data_layer_by_layer():
    c = LlamaConfig.from_dict(H.TINY_B)
    p = c.plan()
    assert len(p.layers) == 3 and [e.layer for e in p.schedule] == [0, 1, 2]
    assert p.layers[1].prefix == "model.layers.1." and p.layers[1].mixer.kind == "attention"
    assert p.layers[0].mixer["num_kv_heads"] == 1 and p.layers[0].ffn["intermediate_size"] == 200
    assert p.layers[0].mixer["positions"]["theta"] == 100000.0 and p.final_norm["eps"] == 1e-6
    assert p.head["tied_to"] is None
    # a schedule may run a layer twice or read an earlier entry's cache; what cannot work is refused
    ModelPlan(**{**p.__dict__, "schedule": (ScheduleEntry(0), ScheduleEntry(1), ScheduleEntry(1), ScheduleEntry(2))}).validate()
    with pytest.raises(ConfigError, match="does not run before"):
        ModelPlan(**{**p.__dict__, "schedule": (ScheduleEntry(0, reads_cache_of=0),)}).validate()
    with pytest.raises(ConfigError, match="names layer"):
        ModelPlan(**{**p.__dict__, "schedule": (ScheduleEntry(5),)}).validate()
    bad = LayerSpec("x.", "prenorm", PartSpec("no_such_mixer", {}), p.layers[0].mixer_norm, p.layers[0].ffn, p.layers[0].ffn_norm)
    with pytest.raises(ConfigError, match="no_such_mixer"):
        DecoderModel(ModelPlan(**{**p.__dict__, "layers": (bad,), "schedule": (ScheduleEntry(0),)}), torch.float32)


def test_expected_weights_names():
    a = expected_weights(LlamaConfig.from_dict(H.TINY_A).plan())
    assert "lm_head.weight" not in a and a["model.embed_tokens.weight"] == (256, 64) and len(a) == 2 + 2 * 9
    b = expected_weights(LlamaConfig.from_dict(H.TINY_B).plan())
    assert b["lm_head.weight"] == (397, 96) and b["model.layers.2.mlp.down_proj.weight"] == (96, 200)
    assert b["model.layers.0.self_attn.k_proj.weight"] == (32, 96) and b["model.norm.weight"] == (96,)


def test_random_model_dir_round_trip(tmp_path):
    d = H.make_model_dir(tmp_path, "tiny_b")
    t = read_dir(d)
    exp = expected_weights(read_config(d).plan())
    assert set(t) == set(exp) and all(tuple(t[n].shape) == tuple(s) for n, s in exp.items())
    assert all(v.dtype == torch.bfloat16 for v in t.values())
    assert abs(float(t["model.norm.weight"].float().mean()) - 1) < 0.05 and abs(float(t["lm_head.weight"].float().mean())) < 0.01
    (tmp_path / "again").mkdir()
    d2 = H.make_model_dir(tmp_path / "again", "tiny_b")
    again = read_dir(d2)
    assert all(torch.equal(t[n], again[n]) for n in t)  # same seed, same bits
    d32 = H.make_model_dir(tmp_path, "tiny_b", "float32")
    t32 = load_checked(d32, exp)
    assert all(v.dtype == torch.float32 for v in t32.values())  # stored in 32 bits, kept in 32 bits


def test_one_error_lists_everything(tmp_path):
    d = H.make_model_dir(tmp_path, "tiny_a")
    t = dict(read_dir(d))
    t.pop("model.layers.1.mlp.up_proj.weight")
    t.pop("model.norm.weight")
    t["model.layers.0.self_attn.q_proj.weight"] = torch.zeros(64, 32, dtype=torch.bfloat16)
    t["something.else"] = torch.zeros(3)
    t["lm_head.weight"] = torch.zeros(256, 64, dtype=torch.bfloat16)  # a tied model's stored copy: ignored
    write_file(str(tmp_path / "tiny_a_bfloat16" / "model.safetensors"), t)
    model = DecoderModel(read_config(d).plan(), torch.float32)
    with pytest.raises(WeightsError) as ei:
        load_checked(d, model.expected_weights(), model.ignorable_weights())
    e = ei.value
    assert e.missing == ["model.layers.1.mlp.up_proj.weight", "model.norm.weight"]
    assert e.unexpected == ["something.else"]
    assert e.wrong_shape == [("model.layers.0.self_attn.q_proj.weight", (64, 32), (64, 64))]
    msg = str(e)
    for s in ("missing (2)", "unexpected (1)", "wrong shape (1)", "something.else", "is [64, 32], expected [64, 64]"):
        assert s in msg
    check({"a": (2,)}, {"a": torch.zeros(2)})  # nothing wrong, nothing raised


def test_untied_model_needs_its_head(tmp_path):
    d = H.make_model_dir(tmp_path, "tiny_b")
    t = dict(read_dir(d))
    t.pop("lm_head.weight")
    write_file(str(tmp_path / "tiny_b_bfloat16" / "model.safetensors"), t)
    model = DecoderModel(read_config(d).plan(), torch.float32)
    with pytest.raises(WeightsError, match="lm_head.weight"):
        load_checked(d, model.expected_weights(), model.ignorable_weights())


def test_kept_dtypes():
    half = torch.tensor([1.0009765625, 0.333251953125], dtype=torch.float16)   # 10 mantissa bits: bfloat16 would lose some
    assert keep_dtype(half).dtype == torch.float16 and torch.equal(keep_dtype(half), half)
    assert keep_dtype(torch.zeros(2, dtype=torch.bfloat16)).dtype == torch.bfloat16
    assert keep_dtype(torch.zeros(2, dtype=torch.float32)).dtype == torch.float32
    assert keep_dtype(torch.zeros(2, dtype=torch.float64)).dtype == torch.float32
    assert keep_dtype(torch.zeros(2, dtype=torch.int64)).dtype == torch.int32
    assert keep_dtype(torch.zeros(2, dtype=torch.uint8)).dtype == torch.int32


def test_broken_files(tmp_path):
    p = tmp_path / "m"
    p.mkdir()
    with pytest.raises(WeightsError, match="no .safetensors"):
        read_dir(str(p))
    (p / "a.safetensors").write_bytes(b"abc")
    with pytest.raises(WeightsError, match="too short"):
        read_dir(str(p))
    (p / "a.safetensors").write_bytes(struct.pack("<Q", 1 << 40) + b"{}")
    with pytest.raises(WeightsError, match="header length"):
        read_dir(str(p))
    h = json.dumps({"x": {"dtype": "F32", "shape": [4], "data_offsets": [0, 8]}}).encode()
    (p / "a.safetensors").write_bytes(struct.pack("<Q", len(h)) + h + b"\0" * 8)
    with pytest.raises(WeightsError, match="byte range"):
        read_dir(str(p))
    h = json.dumps({"x": {"dtype": "F8_E4M3", "shape": [4], "data_offsets": [0, 4]}}).encode()
    (p / "a.safetensors").write_bytes(struct.pack("<Q", len(h)) + h + b"\0" * 4)
    with pytest.raises(WeightsError, match="dtype"):
        read_dir(str(p))


def test_plain_reader_agrees_with_ours(tmp_path):
    import plain_llama as plain
    d = H.make_model_dir(tmp_path, "tiny_a")
    ours = read_dir(d)
    cfg, theirs = plain.read_model(d)
    assert cfg["theta"] == 10000.0 and cfg["tied"] is True
    for n, t in ours.items():
        assert (t.float().numpy() == theirs[n]).all()
