"""Configuration and registry (no GPU)."""
import json

import pytest

import helpers
from atoma_infer_b200.config import (ConfigError, EngineConfig, LlamaConfig, architecture, architecture_of,
                                     known_architectures, register_architecture)


def test_every_key_is_read_from_config_json():
    a, b = LlamaConfig.from_dict(helpers.CONFIG_A), LlamaConfig.from_dict(helpers.CONFIG_B)
    assert (a.hidden_size, a.num_attention_heads, a.num_key_value_heads, a.head_dim) == (64, 4, 2, 16)
    assert (b.hidden_size, b.num_attention_heads, b.num_key_value_heads, b.head_dim) == (192, 3, 1, 64)
    assert a.rms_norm_eps == 1e-5 and b.rms_norm_eps == 1e-6
    assert a.rope_scaling is None and b.rope_scaling.rope_type == "llama3" and b.rope_scaling.factor == 8.0
    assert a.tie_word_embeddings and not b.tie_word_embeddings
    assert a.eos_token_ids == (255,) and b.eos_token_ids == (998, 999)
    assert abs(b.softmax_scale - 1 / 8) < 1e-12


def test_defaults_follow_the_reference():
    d = {k: v for k, v in helpers.CONFIG_A.items()
         if k not in ("num_key_value_heads", "rope_theta", "tie_word_embeddings", "eos_token_id")}
    c = LlamaConfig.from_dict(d)
    assert c.num_key_value_heads == c.num_attention_heads  # models/src/llama.rs:54-57
    assert c.rope_theta == 10000.0                          # :60-62
    assert c.tie_word_embeddings is False                   # :79
    assert c.eos_token_ids == ()


def test_head_dim_key_overrides_the_quotient():
    c = LlamaConfig.from_dict(dict(helpers.CONFIG_A, head_dim=32))
    assert c.head_dim == 32 and c.q_size == 128


@pytest.mark.parametrize("patch, word", [
    ({"hidden_size": None}, "hidden_size"),
    ({"rms_norm_eps": None}, "rms_norm_eps"),
    ({"num_attention_heads": 5}, "multiple"),
    ({"num_key_value_heads": 3}, "multiple"),
    ({"attention_bias": True}, "bias"),
    ({"hidden_act": "gelu"}, "hidden_act"),
    ({"rope_scaling": {"rope_type": "yarn", "factor": 2.0}}, "yarn"),
    ({"rope_scaling": {"rope_type": "llama3", "factor": 2.0}}, "missing"),
    ({"eos_token_id": "x"}, "eos_token_id"),
    ({"vocab_size": 0}, "vocab_size"),
])
def test_bad_configs_are_refused_with_the_key_named(patch, word):
    d = dict(helpers.CONFIG_A)
    d.update(patch)
    with pytest.raises(ConfigError) as e:
        LlamaConfig.from_dict(d)
    assert word in str(e.value)


def test_round_trip_through_json():
    for cfg in (helpers.CONFIG_A, helpers.CONFIG_B):
        c = LlamaConfig.from_dict(cfg)
        assert LlamaConfig.from_dict(json.loads(json.dumps(c.to_dict()))) == c


def test_registry_chooses_by_architecture_name(tmp_path):
    assert "LlamaForCausalLM" in known_architectures()
    (tmp_path / "config.json").write_text(json.dumps(helpers.CONFIG_B))
    arch, cfg = architecture_of(str(tmp_path))
    assert arch.name == "LlamaForCausalLM" and cfg.vocab_size == 1000
    spec = arch.build_spec(cfg)
    assert len(spec.layers) == 3 and spec.head_tensor == "lm_head.weight"
    (tmp_path / "config.json").write_text(json.dumps(dict(helpers.CONFIG_B, architectures=["NopeForCausalLM"])))
    with pytest.raises(ConfigError) as e:
        architecture_of(str(tmp_path))
    assert "NopeForCausalLM" in str(e.value) and "LlamaForCausalLM" in str(e.value)
    with pytest.raises(ConfigError):
        register_architecture("LlamaForCausalLM", dict, dict)
    # a folder without an "architectures" list: its model_type chooses; neither: one clear error
    bare = {k: v for k, v in helpers.CONFIG_B.items() if k != "architectures"}
    (tmp_path / "config.json").write_text(json.dumps(dict(bare, model_type="llama")))
    assert architecture_of(str(tmp_path))[0].name == "LlamaForCausalLM"
    (tmp_path / "config.json").write_text(json.dumps(bare))
    with pytest.raises(ConfigError) as e:
        architecture_of(str(tmp_path))
    assert "architectures" in str(e.value) and "model_type" in str(e.value)


def test_engine_config_checks_and_toml(tmp_path):
    with pytest.raises(ConfigError):
        EngineConfig(max_num_batched_tokens=8, max_num_sequences=16)
    with pytest.raises(ConfigError):
        EngineConfig(enable_chunked_prefill=False, max_model_len=4096, max_num_batched_tokens=1024)
    with pytest.raises(ConfigError):
        EngineConfig(dtype="fp8")
    toml = tmp_path / "c.toml"
    toml.write_text('[inference]\ndtype = "bf16"\ndevice_ids = [0]\nmodel_name = "x"\n[cache]\nblock_size = 16\n'
                    'cache_dtype = "bf16"\ngpu_memory_utilization = 0.5\nswap_space_fraction = 0.1\n[scheduler]\n'
                    'max_num_batched_tokens = 1024\nmax_num_sequences = 32\nmax_model_len = 1024\ndelay_factor = 0.8\n'
                    'enable_chunked_prefill = false\nblock_size = 16\n[validation]\nbest_of = 1\nmax_input_length = 4096\n'
                    'max_total_tokens = 8192\n')
    c = EngineConfig.from_toml(str(toml))
    assert (c.dtype, c.block_size, c.gpu_memory_utilization, c.max_num_sequences) == ("bfloat16", 16, 0.5, 32)
    assert c.enable_chunked_prefill is False and c.max_total_tokens == 8192
