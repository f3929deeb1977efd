"""Configuration and registry (no GPU)."""

import json

import pytest

from hetero_serve_b200.architectures.gpt2 import GPT2Config
from hetero_serve_b200.config import (Architecture, ConfigError, EngineConfig,
                                      architecture_of, load_model_config, preset,
                                      register_architecture, registered_architectures,
                                      unregister_architecture)
from conftest import TINY_A, TINY_B


def test_reads_gpt2_keys():
    c = GPT2Config.from_dict(TINY_B)
    assert (c.n_layer, c.n_embd, c.n_head, c.head_dim) == (3, 96, 3, 32)
    assert c.inner_dim == 320 and c.vocab_size == 1000 and c.n_positions == 256
    assert c.layer_norm_epsilon == 1e-6 and c.activation_function == "gelu"
    assert c.scale_attn_by_inverse_layer_idx is True and c.eos_token_id == 999


def test_defaults_and_derived():
    c = GPT2Config.from_dict({"n_layer": 2, "n_embd": 64, "n_head": 4, "vocab_size": 50,
                              "n_ctx": 32})              # the reference's key for the table
    assert c.n_positions == 32 and c.inner_dim == 256
    assert c.layer_norm_epsilon == 1e-5 and c.activation_function == "gelu_new"
    assert c.kv_bytes_per_token(2) == 2 * 2 * 64 * 2
    assert abs(c.attention_scale(1) - 0.25) < 1e-12


def test_attention_scale_options():
    c = GPT2Config.from_dict(TINY_B)
    assert abs(c.attention_scale(2) - (1 / 32 ** 0.5) / 3) < 1e-15
    c2 = c.replace(scale_attn_weights=False)
    assert c2.attention_scale(0) == 1.0 and abs(c2.attention_scale(1) - 0.5) < 1e-15


@pytest.mark.parametrize("patch,needle", [
    ({"n_layer": None}, "n_layer"),
    ({"n_embd": 65}, "multiple of n_head"),
    ({"activation_function": "swish"}, "activation_function"),
    ({"n_head": 0}, "n_head"),
    ({"layer_norm_epsilon": 0}, "layer_norm_epsilon"),
    ({"vocab_size": "512"}, "vocab_size"),
    ({"scale_attn_by_inverse_layer_idx": 1}, "true or false"),
    ({"n_ctx": 64}, "disagree"),
])
def test_bad_config_is_refused(patch, needle):
    raw = dict(TINY_A)
    raw.update(patch)
    raw = {k: v for k, v in raw.items() if v is not None}
    with pytest.raises(ConfigError, match=needle):
        GPT2Config.from_dict(raw)


def test_missing_positions():
    raw = {k: v for k, v in TINY_A.items() if k != "n_positions"}
    with pytest.raises(ConfigError, match="n_positions"):
        GPT2Config.from_dict(raw)


def test_registry_selects_by_architecture_name(tmp_path):
    assert "GPT2LMHeadModel" in registered_architectures()
    assert architecture_of({"architectures": ["GPT2LMHeadModel"]}).name == "GPT2LMHeadModel"
    assert architecture_of({"model_type": "gpt2"}).name == "GPT2LMHeadModel"
    with pytest.raises(ConfigError, match="unknown architecture"):
        architecture_of({"architectures": ["LlamaForCausalLM"]})
    with pytest.raises(ConfigError, match="no known architecture"):
        architecture_of({"n_layer": 2})
    (tmp_path / "config.json").write_text(json.dumps(TINY_A))
    arch, cfg = load_model_config(tmp_path)
    assert arch.name == "GPT2LMHeadModel" and cfg.n_embd == 64
    with pytest.raises(ConfigError, match="no config.json"):
        load_model_config(tmp_path / "nowhere")
    (tmp_path / "config.json").write_text("{not json")
    with pytest.raises(ConfigError, match="not valid JSON"):
        load_model_config(tmp_path)


def test_register_and_unregister():
    arch = Architecture("ToyForTest", GPT2Config, lambda c: None, lambda c, s: {}, ("toy-test",))
    register_architecture(arch)
    try:
        with pytest.raises(ConfigError, match="already registered"):
            register_architecture(arch)
        assert architecture_of({"model_type": "toy-test"}).name == "ToyForTest"
    finally:
        unregister_architecture("ToyForTest")
    assert "ToyForTest" not in registered_architectures()


def test_spec_is_built_from_config_alone():
    from hetero_serve_b200.architectures.gpt2 import build_spec
    spec = build_spec(GPT2Config.from_dict(TINY_B))
    assert len(spec.layers) == 3 and spec.vocab_size == 1000 and spec.max_positions == 256
    m = spec.layers[2].mixer.params
    assert m["n_heads"] == 3 and m["head_dim"] == 32
    assert abs(m["scale"] - (1 / 32 ** 0.5) / 3) < 1e-15
    assert spec.layers[0].feed_forward.params["activation"] == "gelu_erf"
    assert spec.layers[0].feed_forward.params["inner"] == 320
    assert spec.layers[1].norm1.params["eps"] == 1e-6
    assert [c.layer for c in spec.schedule] == [0, 1, 2]


def test_presets_and_engine_config():
    assert preset("medium")["n_embd"] == 1024 and preset("tiny-b")["n_inner"] == 320
    with pytest.raises(ConfigError):
        preset("huge")
    assert EngineConfig(dtype="bf16").dtype == "bfloat16"
    assert EngineConfig(block_size=16, num_blocks=4).capacity_tokens == 64
    for bad in (dict(dtype="fp8"), dict(block_size=10), dict(num_blocks=0), dict(policy="x")):
        with pytest.raises(ConfigError):
            EngineConfig(**bad)
