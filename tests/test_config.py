"""Configuration and registry: keys, defaults, refusals."""

import json
import os

import pytest

from sllm_b200 import models  # noqa: F401
from sllm_b200.config import (Architecture, ConfigError, get_architecture, known_architectures, load_config,
                              register_architecture, unregister_architecture)
from sllm_b200.models.qwen2 import Qwen2Config, plan
from tests.conftest import TINY_A, TINY_B


def test_reads_keys_and_defaults():
    c = Qwen2Config.from_dict(TINY_A)
    assert (c.hidden_size, c.num_hidden_layers, c.num_attention_heads, c.num_key_value_heads) == (64, 2, 4, 2)
    assert c.head_dim == 16 and c.rotary_dim == 16 and c.tie_word_embeddings and c.rms_norm_eps == 1e-6
    raw = dict(TINY_B)
    del raw["head_dim"], raw["num_key_value_heads"], raw["rms_norm_eps"], raw["tie_word_embeddings"]
    c = Qwen2Config.from_dict(raw)
    assert c.head_dim == 96 // 3 and c.num_key_value_heads == 3
    assert c.rms_norm_eps == 1e-6 and c.tie_word_embeddings is False


@pytest.mark.parametrize("key", ["hidden_size", "num_hidden_layers", "num_attention_heads", "intermediate_size",
                                 "vocab_size", "max_position_embeddings", "rope_theta"])
def test_missing_key_is_named(key):
    raw = dict(TINY_A)
    del raw[key]
    with pytest.raises(ConfigError, match=key):
        Qwen2Config.from_dict(raw)


@pytest.mark.parametrize("over,word", [
    ({"hidden_size": "64"}, "hidden_size"), ({"num_hidden_layers": 0}, "num_hidden_layers"),
    ({"num_key_value_heads": 3}, "multiple"), ({"hidden_act": "gelu"}, "hidden_act"),
    ({"use_sliding_window": True}, "use_sliding_window"), ({"rope_scaling": {"type": "yarn"}}, "rope_scaling"),
    ({"rms_norm_eps": -1.0}, "rms_norm_eps"), ({"tie_word_embeddings": "yes"}, "tie_word_embeddings"),
    ({"partial_rotary_factor": 1.5}, "partial_rotary_factor"),
])
def test_refusals(over, word):
    raw = dict(TINY_A)
    raw.update(over)
    with pytest.raises(ConfigError, match=word):
        Qwen2Config.from_dict(raw)


def test_plan_is_data_from_config():
    for raw in (TINY_A, TINY_B):
        c = Qwen2Config.from_dict(raw)
        p = plan(c)
        assert len(p.layers) == c.num_hidden_layers and [e.layer for e in p.run_list] == list(range(len(p.layers)))
        assert p.layers[0].part("mixer").params["num_heads"] == c.num_attention_heads
        assert p.layers[0].part("mixer").params["scale"] == c.head_dim ** -0.5
        assert p.layers[0].part("mixer_norm").params["eps"] == c.rms_norm_eps
        assert p.position.params["theta"] == c.rope_theta
        assert (p.head_name is None) == c.tie_word_embeddings


def test_registry(tmp_path):
    assert "Qwen2ForCausalLM" in known_architectures()
    assert get_architecture("qwen2").name == "Qwen2ForCausalLM"
    with pytest.raises(ConfigError, match="unknown architecture"):
        get_architecture("NoSuchModel")
    with open(tmp_path / "config.json", "w") as f:
        json.dump(TINY_A, f)
    arch, cfg = load_config(str(tmp_path))
    assert arch.name == "Qwen2ForCausalLM" and cfg.vocab_size == 256
    with open(tmp_path / "config.json", "w") as f:
        json.dump({k: v for k, v in TINY_A.items() if k != "architectures"}, f)
    with pytest.raises(ConfigError, match="architectures"):
        load_config(str(tmp_path))
    with pytest.raises(ConfigError, match="not found"):
        load_config(str(tmp_path / "nowhere"))
    # registering twice is refused unless asked
    a = Architecture("ToyArch", Qwen2Config, plan)
    register_architecture(a)
    with pytest.raises(ConfigError, match="already"):
        register_architecture(a)
    unregister_architecture("ToyArch")
