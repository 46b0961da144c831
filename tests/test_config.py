"""Configuration: keys, defaults and checks of config.json, the architecture registry."""
import json

import pytest

from rust_inference_b200.config import (ConfigError, UnsupportedArchitecture, config_from_dict, load_config,
                                        registered_architectures)
from tiny_configs import TINY_A, TINY_B

BASE = {"architectures": ["Qwen3ForCausalLM"], "vocab_size": 10, "hidden_size": 8, "intermediate_size": 16,
        "num_hidden_layers": 4, "num_attention_heads": 2, "num_key_value_heads": 1}


def test_defaults_follow_the_reference():
    c = config_from_dict(BASE)                       # src/models/config.rs:58-77 of the reference
    assert c.head_dim == 4 and c.max_position_embeddings == 40960
    assert c.rms_norm_eps == 1e-6 and c.rope_theta == 1_000_000.0 and c.tie_word_embeddings is False
    assert c.eos_token_ids == ()


def test_every_size_reaches_the_spec():
    for d in (TINY_A, TINY_B):
        c = config_from_dict(d)
        s = c.to_spec()
        assert s.vocab_size == d["vocab_size"] and s.hidden_size == d["hidden_size"]
        assert len(s.layers) == d["num_hidden_layers"] == len(s.schedule)
        a = s.layers[0].mixer
        assert (a.num_heads, a.num_kv_heads, a.head_dim) == (d["num_attention_heads"], d["num_key_value_heads"], d["head_dim"])
        assert a.position.theta == d["rope_theta"] and a.qk_norm.eps == d["rms_norm_eps"]
        assert s.layers[0].ffn.intermediate_size == d["intermediate_size"]
        assert s.final_norm.eps == d["rms_norm_eps"] and s.tie_embeddings == d["tie_word_embeddings"]
        assert s.max_positions == d["max_position_embeddings"]
        assert s.layers[1].prefix("mixer") == "model.layers.1.self_attn."
        assert config_from_dict(c.to_dict()) == c
    assert config_from_dict(TINY_B).to_spec().stop_ids == (7, 300)


def test_architecture_by_model_type_and_unknown():
    d = dict(BASE)
    del d["architectures"]
    d["model_type"] = "qwen3"
    assert config_from_dict(d).hidden_size == 8
    with pytest.raises(UnsupportedArchitecture):
        config_from_dict({**BASE, "architectures": ["LlamaForCausalLM"]})
    with pytest.raises(UnsupportedArchitecture):
        config_from_dict({k: v for k, v in BASE.items() if k != "architectures"})
    assert "Qwen3ForCausalLM" in registered_architectures()


@pytest.mark.parametrize("change", [
    {"num_attention_heads": 0}, {"num_key_value_heads": 0}, {"num_attention_heads": 3, "num_key_value_heads": 2},
    {"head_dim": 5}, {"rope_scaling": {"rope_type": "yarn", "factor": 4.0}}, {"attention_bias": True},
    {"use_sliding_window": True, "sliding_window": 16}, {"num_experts": 8}, {"hidden_act": "gelu"},
    {"quantization_config": {"quant_method": "fp8"}}, {"vocab_size": 0}, {"rms_norm_eps": 0.0},
    {"hidden_size": "64"},
])
def test_refused(change):
    with pytest.raises(ConfigError):
        config_from_dict({**BASE, **change})


def test_accepted_forms():
    assert config_from_dict({**BASE, "rope_scaling": None}).rope_scaling is None
    assert config_from_dict({**BASE, "rope_scaling": {"type": "default"}}).rope_scaling == {"type": "default"}
    assert config_from_dict({**BASE, "eos_token_id": 3}).eos_token_ids == (3,)
    assert config_from_dict({**BASE, "use_sliding_window": False, "sliding_window": None, "torch_dtype": "bfloat16"})


def test_missing_keys_and_files(tmp_path):
    with pytest.raises(ConfigError, match="hidden_size"):
        config_from_dict({k: v for k, v in BASE.items() if k != "hidden_size"})
    with pytest.raises(ConfigError):
        load_config(str(tmp_path))
    (tmp_path / "config.json").write_text("{not json")
    with pytest.raises(ConfigError):
        load_config(str(tmp_path))
    (tmp_path / "config.json").write_text(json.dumps(BASE))
    assert load_config(str(tmp_path)).num_hidden_layers == 4
