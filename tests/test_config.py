"""Configuration and registry (no GPU)."""
import json
import os

import pytest

from mini_engine_b200.config import (ConfigError, EngineConfig, Qwen3Config, get_architecture,
                                     load_model_config, registered_architectures)
from tiny_configs import TINY_A, TINY_B, TINY_C


def test_reads_every_size_from_config_json(tmp_path):
    for raw in (TINY_A, TINY_B, TINY_C):
        (tmp_path / "config.json").write_text(json.dumps(raw))
        cfg = load_model_config(str(tmp_path))
        assert isinstance(cfg, Qwen3Config)
        for key in ("hidden_size", "num_hidden_layers", "num_attention_heads", "num_key_value_heads", "head_dim",
                    "intermediate_size", "vocab_size", "rms_norm_eps", "rope_theta", "tie_word_embeddings",
                    "max_position_embeddings"):
            assert getattr(cfg, key) == raw[key], key
    assert cfg.window_of_layer(0) is None and cfg.window_of_layer(1) == 24


def test_head_dim_and_kv_heads_defaults():
    raw = dict(TINY_A)
    del raw["head_dim"], raw["num_key_value_heads"]
    cfg = Qwen3Config.from_dict(raw)
    assert cfg.head_dim == 16 and cfg.num_key_value_heads == 4


def test_rope_theta_in_rope_parameters():
    raw = dict(TINY_A)
    del raw["rope_theta"]
    raw["rope_parameters"] = {"rope_theta": 12345.0, "rope_type": "default"}
    assert Qwen3Config.from_dict(raw).rope_theta == 12345.0


@pytest.mark.parametrize("change, word", [
    ({"hidden_act": "gelu"}, "hidden_act"),
    ({"attention_bias": True}, "attention_bias"),
    ({"rope_scaling": {"rope_type": "yarn", "factor": 4.0}}, "rope scaling"),
    ({"num_key_value_heads": 3}, "multiple"),
    ({"hidden_size": None}, "hidden_size"),
    ({"vocab_size": "many"}, "vocab_size"),
    ({"use_sliding_window": True, "sliding_window": None}, "sliding_window"),
    ({"architectures": ["NoSuchModel"]}, "unknown architecture"),
])
def test_refuses_what_it_cannot_honour(tmp_path, change, word):
    raw = dict(TINY_A)
    raw.update(change)
    (tmp_path / "config.json").write_text(json.dumps(raw))
    with pytest.raises(ConfigError, match=word):
        load_model_config(str(tmp_path))


def test_registry_lists_qwen3():
    assert "Qwen3ForCausalLM" in registered_architectures()
    assert get_architecture("Qwen3ForCausalLM").name == "Qwen3ForCausalLM"


def test_plan_is_data(tmp_path):
    cfg = Qwen3Config.from_dict(TINY_C)
    plan = get_architecture(cfg.architecture).plan(cfg)
    assert len(plan.blocks) == 4 and [c.block for c in plan.schedule] == [0, 1, 2, 3]
    assert [b.mixer.args["window"] for b in plan.blocks] == [None, 24, None, 24]
    assert plan.blocks[0].mixer.args["head_dim"] == 48


def test_engine_config_checks(tmp_path):
    (tmp_path / "config.json").write_text(json.dumps(TINY_A))
    cfg = EngineConfig(str(tmp_path), max_model_len=100000)
    assert cfg.max_model_len == TINY_A["max_position_embeddings"]        # config.py:26
    assert cfg.kvcache_block_size == 16 and cfg.max_num_seqs == 512 and cfg.max_num_batched_tokens == 16384
    assert cfg.enable_chunked_prefill and cfg.scheduling_policy == "fcfs" and cfg.dtype == "bfloat16"
    with pytest.raises(ConfigError):
        EngineConfig(str(tmp_path), max_num_seqs=64, max_num_batched_tokens=32)
    with pytest.raises(ConfigError):
        EngineConfig(str(tmp_path), scheduling_policy="random")
    with pytest.raises(ConfigError):
        EngineConfig(str(tmp_path), enable_chunked_prefill=False, max_num_batched_tokens=128, max_num_seqs=4)
    with pytest.raises(ConfigError):
        EngineConfig(str(tmp_path / "nowhere"))
    with pytest.raises(ConfigError):
        EngineConfig(str(tmp_path), dtype="float16")
