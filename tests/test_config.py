"""Configuration and registry (no GPU)."""
import json
import os
import tempfile

import pytest

from helpers import TINY
from lite_lang_b200.config import (ConfigError, EngineConfig, config_from_dict, known_architectures, load_config,
                                   register_architecture)
from lite_lang_b200.models.qwen2 import Qwen2Config


def test_registry_knows_qwen2():
    assert "Qwen2ForCausalLM" in known_architectures()
    cfg = config_from_dict(TINY["A"]["config"])
    assert isinstance(cfg, Qwen2Config)


def test_every_key_is_read_from_config_json():
    d = dict(TINY["C"]["config"])
    cfg = config_from_dict(d)
    assert cfg.hidden_size == 160 and cfg.num_hidden_layers == 4
    assert cfg.num_attention_heads == 8 and cfg.num_key_value_heads == 2
    assert cfg.head_dim == 64            # given explicitly, not hidden / heads
    assert cfg.intermediate_size == 208 and cfg.vocab_size == 331
    assert cfg.rope_theta == 50000.0 and cfg.rms_norm_eps == 3e-6
    assert cfg.max_position_embeddings == 512 and cfg.tie_word_embeddings is False
    assert cfg.sliding_window == 40 and cfg.max_window_layers == 1
    assert [cfg.window_of_layer(i) for i in range(4)] == [None, 40, 40, 40]


def test_head_dim_defaults_to_hidden_over_heads():
    cfg = config_from_dict(TINY["B"]["config"])
    assert cfg.head_dim == 32


def test_round_trip_through_folder():
    cfg = config_from_dict(TINY["B"]["config"])
    with tempfile.TemporaryDirectory() as d:
        with open(os.path.join(d, "config.json"), "w") as fh:
            json.dump(cfg.to_dict(), fh)
        assert load_config(d) == cfg


def test_model_spec_carries_constants_as_parameters():
    cfg = config_from_dict(TINY["C"]["config"])
    spec = cfg.model_spec()
    assert len(spec.layers) == 4 and [s.layer for s in spec.order] == [0, 1, 2, 3]
    m0, m1 = spec.layers[0].parts["mixer"], spec.layers[1].parts["mixer"]
    assert m0.kind == "gqa_attention" and m0.params["window"] is None and m1.params["window"] == 40
    assert m0.params["head_dim"] == 64 and m0.params["num_kv_heads"] == 2
    assert m0.params["position"].params["theta"] == 50000.0
    assert spec.layers[0].parts["mixer_norm"].params["eps"] == 3e-6
    assert spec.layers[2].parts["feed_forward"].params["intermediate_size"] == 208
    assert spec.head.params["tied_to"] is None
    assert sorted(spec.layers[0].parts) == ["feed_forward", "feed_forward_norm", "mixer", "mixer_norm"]
    specA = config_from_dict(TINY["A"]["config"]).model_spec()
    assert specA.head.params["tied_to"] == "model.embed_tokens.weight"


@pytest.mark.parametrize("key", ["hidden_size", "num_hidden_layers", "num_attention_heads", "num_key_value_heads",
                                 "intermediate_size", "vocab_size"])
def test_missing_required_key(key):
    d = dict(TINY["A"]["config"])
    del d[key]
    with pytest.raises(ConfigError, match=key):
        config_from_dict(d)


def test_validation_errors():
    d = dict(TINY["A"]["config"], num_key_value_heads=3)
    with pytest.raises(ConfigError, match="multiple"):
        config_from_dict(d)
    d = dict(TINY["A"]["config"], hidden_act="gelu")
    with pytest.raises(ConfigError, match="hidden_act"):
        config_from_dict(d)
    d = dict(TINY["A"]["config"], rope_scaling={"type": "yarn", "factor": 2})
    with pytest.raises(ConfigError, match="rope_scaling"):
        config_from_dict(d)
    d = dict(TINY["A"]["config"], head_dim=15)
    with pytest.raises(ConfigError, match="even"):
        config_from_dict(d)


def test_unknown_architecture_lists_known_ones():
    with pytest.raises(ConfigError, match="Qwen2ForCausalLM"):
        config_from_dict({"architectures": ["NopeForCausalLM"]})
    with pytest.raises(ConfigError, match="architectures"):
        config_from_dict({"hidden_size": 8})


def test_engine_config():
    e = EngineConfig(dtype="bf16")
    assert e.dtype == "bfloat16" and e.model_len == 4200
    assert EngineConfig(dtype="fp32").dtype == "float32"
    with pytest.raises(ValueError):
        EngineConfig(dtype="float16")
    with pytest.raises(ValueError):
        EngineConfig(page_size=0)


def test_another_architecture_can_be_registered():
    class Other(Qwen2Config):
        architecture = "OtherForCausalLM"
    register_architecture("OtherForCausalLM", Other)
    d = dict(TINY["A"]["config"], architectures=["OtherForCausalLM"])
    assert isinstance(config_from_dict(d), Other)
