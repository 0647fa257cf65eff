"""Configuration, registry, safetensors reading and the weight errors (no GPU)."""
import json
import os

import pytest
import torch

import carbon_engine_b200.models  # noqa: F401
from carbon_engine_b200.config.base import ConfigError, merge_overrides
from carbon_engine_b200.config.qwen3 import Qwen3Config
from carbon_engine_b200.config.registry import (load_config, register_architecture, registered_architectures,
                                                 resolve_architecture, unregister_architecture)
from carbon_engine_b200.weights.loader import WeightError, check_tensors, write_random_model
from carbon_engine_b200.weights.random_init import RandomWeights, random_tensor
from carbon_engine_b200.weights.safetensors_io import SafetensorsError, TensorDirectory, write_safetensors
from carbon_engine_b200.parts.base import TensorSpec
from helpers import TINY, make_model_dir

BASE = dict(architectures=["Qwen3ForCausalLM"], vocab_size=100, hidden_size=48, num_hidden_layers=2,
            num_attention_heads=6)


def test_defaults_follow_the_reference():
    c = Qwen3Config.from_dict(dict(BASE))
    assert c.num_key_value_heads == 6 and c.head_dim == 8 and c.intermediate_size == 192
    assert c.rms_norm_eps == 1e-6 and c.rope_theta == 10000.0 and c.max_position_embeddings == 4096
    assert c.tie_word_embeddings is False and c.hidden_act == "silu"
    assert c.layer_types == ("full_attention", "full_attention") and c.sliding_window is None


def test_every_key_is_read():
    c = Qwen3Config.from_dict(dict(TINY["C"]["config"], eos_token_id=[7, 9], bos_token_id=1))
    assert (c.num_hidden_layers, c.hidden_size, c.num_attention_heads, c.num_key_value_heads, c.head_dim) == (4, 80, 6, 3, 48)
    assert c.q_width == 288 and c.kv_width == 144 and c.intermediate_size == 112 and c.vocab_size == 301
    assert c.rope_theta == 50000.0 and c.rms_norm_eps == 3e-6 and c.sliding_window == 37
    assert c.eos_token_ids == (7, 9) and c.bos_token_id == 1
    assert Qwen3Config.from_dict(c.to_json_dict()) == c


def test_rope_theta_under_rope_parameters():
    c = Qwen3Config.from_dict(dict(BASE, rope_parameters={"rope_theta": 5e5, "rope_type": "default"}))
    assert c.rope_theta == 5e5


def test_rope_scaling_keys_and_defaults():
    """linear, llama3 and yarn with the reference's keys and defaults (src/config.rs:483-519), and the
    frequencies they give (src/model/layers.rs:169-234; the values of its own test, :735-751)."""
    import math
    import plain_qwen3 as plain
    from carbon_engine_b200.parts.rope import rope_inv_freq
    base = dict(BASE, hidden_size=64, num_attention_heads=1, num_key_value_heads=1, head_dim=64, rope_theta=1000000.0,
                max_position_embeddings=131072)
    plain_freq = rope_inv_freq(64, 1e6, None)
    c = Qwen3Config.from_dict(dict(base, rope_scaling={"rope_type": "yarn", "factor": 4.0,
                                                       "original_max_position_embeddings": 32768}))
    rs = c.rope_scaling
    assert (rs.kind, rs.factor, rs.original_max_position, rs.beta_fast, rs.beta_slow) == ("yarn", 4.0, 32768, 32.0, 1.0)
    assert abs(rs.attention_factor - (0.1 * math.log(4.0) + 1.0)) < 1e-12
    yarn = rope_inv_freq(64, 1e6, rs)
    # high-frequency dimensions are left alone, low-frequency ones are divided by the factor
    assert yarn[0] == plain_freq[0] and abs(yarn[31] - plain_freq[31] / 4.0) < 1e-15
    assert all(p / 4.0 - 1e-18 <= y <= p for y, p in zip(yarn, plain_freq))
    assert any(p / 4.0 + 1e-12 < y < p - 1e-12 for y, p in zip(yarn, plain_freq))          # and a ramp between
    # yarn without original_max_position_embeddings takes max_position_embeddings; mscale pairs give the factor
    c2 = Qwen3Config.from_dict(dict(base, rope_parameters={"type": "yarn", "factor": 8.0, "mscale": 1.0, "mscale_all_dim": 0.5}))
    assert c2.rope_scaling.original_max_position == 131072
    assert abs(c2.rope_scaling.attention_factor - (0.1 * math.log(8) + 1) / (0.05 * math.log(8) + 1)) < 1e-12
    lin = Qwen3Config.from_dict(dict(base, rope_scaling={"rope_type": "linear", "factor": 2.0})).rope_scaling
    assert rope_inv_freq(64, 1e6, lin) == [f / 2.0 for f in plain_freq]
    l3 = Qwen3Config.from_dict(dict(base, rope_scaling={"rope_type": "llama3", "factor": 8.0})).rope_scaling
    assert (l3.low_freq_factor, l3.high_freq_factor, l3.original_max_position) == (1.0, 4.0, 8192)
    got = rope_inv_freq(64, 1e6, l3)
    assert got[0] == plain_freq[0] and abs(got[31] - plain_freq[31] / 8.0) < 1e-18
    # the engine's frequencies are those of the plain implementation, for every kind
    for raw in ({"rope_type": "yarn", "factor": 4.0, "original_max_position_embeddings": 32768},
                {"rope_type": "yarn", "factor": 2.5, "beta_fast": 16, "beta_slow": 2, "attention_factor": 1.3},
                {"rope_type": "linear", "factor": 3.0},
                {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                 "original_max_position_embeddings": 8192}):
        cfg = Qwen3Config.from_dict(dict(base, rope_scaling=raw))
        want, att = plain.scaled_inv_freq(64, 1e6, raw, 131072)
        assert torch.allclose(torch.tensor(rope_inv_freq(64, 1e6, cfg.rope_scaling), dtype=torch.float64), want, rtol=1e-14, atol=0)
        assert abs(att - (cfg.rope_scaling.attention_factor if raw["rope_type"] == "yarn" else 1.0)) < 1e-12
        again = Qwen3Config.from_dict(cfg.to_json_dict())                 # and the scaling survives the round trip
        assert again.rope_scaling == cfg.rope_scaling
    assert Qwen3Config.from_dict(dict(base, rope_scaling={"rope_type": "default"})).rope_scaling is None
    # the tables of the part: cos and sin carry YaRN's attention factor
    from carbon_engine_b200.parts.rope import RotaryEmbedding
    raw = {"rope_type": "yarn", "factor": 4.0, "original_max_position_embeddings": 64}
    part = RotaryEmbedding(64, 1e6, 300, scaling=Qwen3Config.from_dict(dict(base, rope_scaling=raw)).rope_scaling)
    part.prepare(torch.device("cpu"))
    c, s_ = plain.rope_tables(torch.arange(300), 64, 1e6, raw)
    assert torch.allclose(part.cos.double(), c, atol=1e-7) and torch.allclose(part.sin.double(), s_, atol=1e-7)
    assert abs(float(part.cos[0, 0]) - (0.1 * math.log(4.0) + 1.0)) < 1e-6


@pytest.mark.parametrize("bad,word", [
    (dict(num_key_value_heads=4), "multiple"), (dict(head_dim=7), "even"), (dict(hidden_act="gelu"), "silu"),
    (dict(rope_scaling={"rope_type": "dynamic", "factor": 4.0}), "dynamic"),
    (dict(rope_scaling={"rope_type": "linear", "factor": 0.0}), "factor"), (dict(quantization_config={"bits": 4}), "quantis"),
    (dict(vocab_size=0), "vocab_size"), (dict(attention_bias=True), "attention_bias"),
    (dict(layer_types=["full_attention"]), "layer_types"),
    (dict(layer_types=["full_attention", "sliding_attention"]), "sliding_window"),
])
def test_bad_configs_are_refused(bad, word):
    with pytest.raises(ConfigError, match=word):
        Qwen3Config.from_dict(dict(BASE, **bad))


def test_missing_required_key():
    d = dict(BASE)
    del d["num_hidden_layers"]
    with pytest.raises(ConfigError, match="num_hidden_layers"):
        Qwen3Config.from_dict(d)


def test_overrides_merge_config_sections_only():
    base = {"a": 1, "text_config": {"x": 1, "y": 2}, "rope_scaling": {"k": 1}}
    out = merge_overrides(base, {"a": 2, "text_config": {"y": 3}, "rope_scaling": {"j": 5}})
    assert out == {"a": 2, "text_config": {"x": 1, "y": 3}, "rope_scaling": {"j": 5}}


def test_registry_by_architecture_then_model_type():
    assert "Qwen3ForCausalLM" in registered_architectures()
    assert resolve_architecture({"architectures": ["Qwen3ForCausalLM"]}).name == "Qwen3ForCausalLM"
    assert resolve_architecture({"model_type": "qwen3"}).name == "Qwen3ForCausalLM"
    with pytest.raises(ConfigError, match="registered: .*Qwen3ForCausalLM"):
        resolve_architecture({"architectures": ["NopeForCausalLM"], "model_type": "nope"})
    register_architecture("ToyLM", lambda raw: None, lambda cfg, n: None, model_types=("toy",))
    try:
        assert resolve_architecture({"model_type": "toy"}).name == "ToyLM"
        with pytest.raises(ValueError):
            register_architecture("ToyLM", lambda raw: None, lambda cfg, n: None)
    finally:
        unregister_architecture("ToyLM")


def test_load_config_reads_generation_eos_and_overrides(tmp_path):
    d = tmp_path / "m"
    d.mkdir()
    (d / "config.json").write_text(json.dumps(dict(BASE, eos_token_id=3)))
    (d / "generation_config.json").write_text(json.dumps({"eos_token_id": [3, 8]}))
    arch, cfg = load_config(str(d), {"rms_norm_eps": 1e-5})
    assert arch.name == "Qwen3ForCausalLM" and cfg.eos_token_ids == (3, 8) and cfg.rms_norm_eps == 1e-5


def test_random_weights_are_seeded_and_distributed():
    spec = TensorSpec("model.layers.0.mlp.up_proj.weight", (64, 96), "linear")
    a = random_tensor(spec, 3, "cpu", torch.float32)
    b = random_tensor(spec, 3, "cpu", torch.float32, chunk=1000)       # chunking does not change the values
    c = random_tensor(spec, 4, "cpu", torch.float32)
    assert torch.equal(a, b) and not torch.equal(a, c)
    assert abs(a.std().item() - 0.02) < 0.002 and abs(a.mean().item()) < 0.002
    n = random_tensor(TensorSpec("model.norm.weight", (4096,), "norm"), 3, "cpu", torch.float32)
    assert abs(n.mean().item() - 1.0) < 0.01 and abs(n.std().item() - 0.1) < 0.01


def test_written_folder_round_trips(tmp_path):
    out = make_model_dir(str(tmp_path), "B", sharpen=1.0)
    arch, cfg = load_config(out)
    model = arch.build_model(cfg, 64)
    td = TensorDirectory(out)
    check_tensors(model.all_tensor_specs(), td)
    gen = RandomWeights(model.all_tensor_specs(), TINY["B"]["seed"], "cpu")
    for s in model.all_tensor_specs():
        assert torch.equal(td.get(s.name), gen(s.name)), s.name
    assert td.dtype("model.norm.weight") == torch.float32                   # stored in 32-bit, stays so
    assert td.dtype("model.layers.0.mlp.up_proj.weight") == torch.bfloat16
    assert "lm_head.weight" in td


def test_one_error_lists_missing_unexpected_and_wrong_shapes(tmp_path):
    out = make_model_dir(str(tmp_path), "A", sharpen=1.0)
    td = TensorDirectory(out)
    tensors = {n: td.get(n).clone() for n in td.names()}
    del tensors["model.layers.1.mlp.down_proj.weight"]
    del tensors["model.norm.weight"]
    tensors["model.layers.0.self_attn.q_proj.weight"] = torch.zeros(8, 64, dtype=torch.bfloat16)
    tensors["lm_head.weight"] = torch.zeros(256, 64, dtype=torch.bfloat16)      # tied model: a redundant copy, ignored
    tensors["model.layers.0.self_attn.rotary_emb.inv_freq"] = torch.zeros(8)    # recomputed, ignored
    tensors["model.layers.0.self_attn.q_bias"] = torch.zeros(64)                # nobody declares this
    tensors["model.layers.0.self_attn.k_norm.weight"] = torch.zeros(16, dtype=torch.int32)
    bad = tmp_path / "bad"
    bad.mkdir()
    (bad / "config.json").write_text(open(os.path.join(out, "config.json")).read())
    write_safetensors(str(bad / "model.safetensors"), tensors.items())
    arch, cfg = load_config(str(bad))
    model = arch.build_model(cfg, 64)
    with pytest.raises(WeightError) as ei:
        check_tensors(model.all_tensor_specs(), TensorDirectory(str(bad)), model.all_ignorable_tensors())
    e = ei.value
    assert set(e.missing) == {"model.layers.1.mlp.down_proj.weight", "model.norm.weight"}
    assert e.unexpected == ["model.layers.0.self_attn.q_bias"]
    with pytest.raises(WeightError) as strict:          # without the parts' list every undeclared tensor is reported
        check_tensors(model.all_tensor_specs(), TensorDirectory(str(bad)))
    assert "lm_head.weight" in strict.value.unexpected
    assert len(e.wrong_shape) == 1 and "q_proj" in e.wrong_shape[0] and "[8, 64]" in e.wrong_shape[0]
    assert len(e.wrong_dtype) == 1 and "k_norm" in e.wrong_dtype[0]
    msg = str(e)
    for word in ("missing", "unexpected", "wrong shapes", "down_proj", "q_bias"):
        assert word in msg


def test_sharded_folder_and_reader_errors(tmp_path):
    d = tmp_path / "s"
    d.mkdir()
    write_safetensors(str(d / "model-00001-of-00002.safetensors"), [("a", torch.arange(6, dtype=torch.float32).view(2, 3))])
    write_safetensors(str(d / "model-00002-of-00002.safetensors"), [("b", torch.ones(4, dtype=torch.bfloat16))])
    (d / "model.safetensors.index.json").write_text(json.dumps(
        {"weight_map": {"a": "model-00001-of-00002.safetensors", "b": "model-00002-of-00002.safetensors"}}))
    td = TensorDirectory(str(d))
    assert sorted(td.names()) == ["a", "b"] and td.get("a")[1, 2] == 5 and td.dtype("b") == torch.bfloat16
    empty = tmp_path / "e"
    empty.mkdir()
    with pytest.raises(SafetensorsError, match="no .safetensors"):
        TensorDirectory(str(empty))
    (empty / "x.safetensors").write_bytes(b"\x05\x00\x00")
    with pytest.raises(SafetensorsError, match="too short"):
        TensorDirectory(str(empty))
    (d / "model.safetensors.index.json").write_text("{}")
    with pytest.raises(SafetensorsError, match="weight_map"):
        TensorDirectory(str(d))
