"""Configuration and registry (no GPU)."""

import json
import os

import pytest

from rust_llm_inference_server_b200.config import (ConfigError, LlamaConfig, lookup_architecture,
                                                   read_config_json, register_architecture,
                                                   registered_architectures, unregister_architecture)
from rust_llm_inference_server_b200.models.llama import describe_llama
from tests.tiny_configs import TINY_A, TINY_B


def test_required_keys_are_reported_together():
    d = dict(TINY_A)
    del d["rope_theta"], d["vocab_size"]
    with pytest.raises(ConfigError) as e:
        LlamaConfig.from_dict(d)
    assert "rope_theta" in str(e.value) and "vocab_size" in str(e.value)


def test_defaults_follow_the_reference():
    d = {k: v for k, v in TINY_B.items() if k not in ("head_dim", "tie_word_embeddings", "rope_scaling")}
    cfg = LlamaConfig.from_dict(d)
    assert cfg.head_dim == 96 // 3            # hidden / heads when absent (config.rs:44-47)
    assert cfg.tie_word_embeddings is False   # false when absent (config.rs:19-20)
    assert cfg.rope_scaling is None
    assert cfg.kv_bytes_per_token(2) == 2 * 3 * 1 * 32 * 2


def test_every_size_comes_from_the_file():
    a, b = LlamaConfig.from_dict(TINY_A), LlamaConfig.from_dict(TINY_B)
    sa, sb = describe_llama(a), describe_llama(b)
    assert (len(sa.layers), len(sb.layers)) == (2, 3)
    assert sa.lm_head.weight == sa.embedding.weight and sb.lm_head.weight == "lm_head.weight"
    m = sb.layers[1].mixer
    assert (m.n_heads, m.n_kv_heads, m.head_dim, m.hidden) == (3, 1, 32, 96)
    assert m.position.scaling.factor == 32.0 and m.position.theta == 500000.0
    assert sb.layers[0].norm1.eps == 1e-6 and sa.layers[0].norm1.eps == 1e-5
    assert sb.layers[2].feed_forward.intermediate == 256
    assert [c.layer for c in sb.order] == [0, 1, 2]


def test_bad_values_are_refused():
    for key, val in (("num_key_value_heads", 3), ("head_dim", 15), ("hidden_size", -1), ("rms_norm_eps", 0)):
        with pytest.raises(ConfigError):
            LlamaConfig.from_dict(dict(TINY_A, **{key: val}))
    with pytest.raises(ConfigError):
        LlamaConfig.from_dict(dict(TINY_A, rope_scaling={"rope_type": "llama3", "factor": 8.0}))


def test_rope_scaling_type_alias_and_other_types():
    rs = dict(TINY_B["rope_scaling"])
    rs["type"] = rs.pop("rope_type")
    assert LlamaConfig.from_dict(dict(TINY_B, rope_scaling=rs)).rope_scaling.rope_type == "llama3"
    cfg = LlamaConfig.from_dict(dict(TINY_B, rope_scaling={"rope_type": "linear", "factor": 2.0}))
    assert cfg.rope_scaling.rope_type == "linear"


def test_registry_picks_by_name_and_lists_known_names():
    assert "LlamaForCausalLM" in registered_architectures()
    assert lookup_architecture({}).name == "LlamaForCausalLM"     # the reference reads any config as Llama
    with pytest.raises(ConfigError) as e:
        lookup_architecture({"architectures": ["NoSuchModel"]})
    assert "NoSuchModel" in str(e.value) and "LlamaForCausalLM" in str(e.value)
    register_architecture("ToyOnlyHere", lambda d: d, lambda c: None)
    try:
        assert lookup_architecture({"architectures": ["ToyOnlyHere"]}).name == "ToyOnlyHere"
        with pytest.raises(ValueError):
            register_architecture("ToyOnlyHere", lambda d: d, lambda c: None)
    finally:
        unregister_architecture("ToyOnlyHere")


def test_read_config_json_and_generation_config(tmp_path):
    with pytest.raises(ConfigError):
        read_config_json(str(tmp_path))
    (tmp_path / "config.json").write_text(json.dumps(dict(TINY_A, eos_token_id=2)))
    assert LlamaConfig.from_dict(read_config_json(str(tmp_path))).eos_token_ids == (2,)
    (tmp_path / "generation_config.json").write_text(json.dumps({"eos_token_id": [5, 6]}))
    assert LlamaConfig.from_dict(read_config_json(str(tmp_path))).eos_token_ids == (5, 6)
    rt = LlamaConfig.from_dict(LlamaConfig.from_dict(TINY_B).to_dict())
    assert rt == LlamaConfig.from_dict(TINY_B)
