"""Configuration and registry (CPU)."""
import json
import math

import pytest

from conftest import TINY_A, TINY_B, TINY_C
from infinicore_infer_b200.config import (ConfigError, MiniCPMConfig, ModelSpec, RunEntry,
                                           config_class_for, read_config, register_architecture)
from plain_minicpm import plain_scales


def test_reads_every_key_of_tiny_a():
    c = MiniCPMConfig.from_dict(TINY_A)
    assert (c.num_hidden_layers, c.hidden_size, c.num_attention_heads, c.num_key_value_heads) == (2, 64, 4, 4)
    assert (c.head_dim, c.intermediate_size, c.vocab_size, c.max_position_embeddings) == (16, 160, 256, 320)
    assert c.rms_norm_eps == 1e-5 and c.rope_theta == 10000.0
    assert c.tie_word_embeddings and c.eos_token_id == (2,)


@pytest.mark.parametrize("cfg", [TINY_A, TINY_B, TINY_C])
def test_scales_follow_the_reference(cfg):
    c = MiniCPMConfig.from_dict(cfg)
    emb, res, logit = plain_scales(cfg)
    assert c.scale_emb == emb
    assert math.isclose(c.residual_scale, res, rel_tol=0, abs_tol=0)
    assert c.logit_scale == logit
    spec = c.model_spec()
    assert spec.embed_scale == emb and spec.logit_scale == logit
    assert all(layer.residual_scale == res for layer in spec.layers)


def test_logit_scale_is_floor_division_and_multiplies():
    cfg = dict(TINY_A, hidden_size=72, num_attention_heads=4, dim_model_base=16)   # 72 // 16 = 4
    assert MiniCPMConfig.from_dict(cfg).logit_scale == 4.0
    assert MiniCPMConfig.from_dict(dict(cfg, logit_scale=0.25)).logit_scale == 0.25


def test_llama_has_no_scales_even_if_keys_are_present():
    c = MiniCPMConfig.from_dict(dict(TINY_A, model_type="llama"))
    assert (c.scale_emb, c.residual_scale, c.logit_scale) == (1.0, 1.0, 1.0)


def test_scales_need_all_three_keys():
    cfg = dict(TINY_A)
    del cfg["scale_depth"]
    c = MiniCPMConfig.from_dict(cfg)
    assert (c.scale_emb, c.residual_scale, c.logit_scale) == (1.0, 1.0, 1.0)


def test_defaults_of_the_reference():
    cfg = dict(TINY_A)
    del cfg["rope_theta"], cfg["num_key_value_heads"]
    c = MiniCPMConfig.from_dict(cfg)
    assert c.rope_theta == 100000.0          # scripts/jiuge.py:133
    assert c.num_key_value_heads == c.num_attention_heads


def test_head_dim_key_is_honoured():
    c = MiniCPMConfig.from_dict(TINY_C)
    assert c.head_dim == 48
    attn = c.model_spec().layers[0].mixer
    assert attn.head_dim == 48 and math.isclose(attn.softmax_scale, 48 ** -0.5)


def test_max_tokens_overrides_context():
    assert MiniCPMConfig.from_dict(TINY_A, max_tokens=100).max_position_embeddings == 100


@pytest.mark.parametrize("bad, word", [
    ({"hidden_size": None}, "hidden_size"),
    ({"num_key_value_heads": 3}, "multiple"),
    ({"hidden_size": 66}, "multiple"),
    ({"num_hidden_layers": 0}, "positive"),
    ({"vocab_size": 2.5}, "positive"),
    ({"rope_scaling": {"type": "longrope"}}, "rope_scaling"),
])
def test_bad_values_raise_named_errors(bad, word):
    cfg = dict(TINY_A, **bad)
    with pytest.raises(ConfigError, match=word):
        MiniCPMConfig.from_dict(cfg)


def test_missing_keys_are_listed_together():
    cfg = dict(TINY_A)
    del cfg["vocab_size"], cfg["rms_norm_eps"]
    with pytest.raises(ConfigError) as e:
        MiniCPMConfig.from_dict(cfg)
    assert "vocab_size" in str(e.value) and "rms_norm_eps" in str(e.value)


def test_registry_by_model_type_and_architectures(tmp_path):
    assert config_class_for({"model_type": "minicpm"}) is MiniCPMConfig
    assert config_class_for({"model_type": "fm9g"}) is MiniCPMConfig
    assert config_class_for({"model_type": "llama"}) is MiniCPMConfig
    assert config_class_for({"architectures": ["MiniCPMForCausalLM"]}) is MiniCPMConfig
    with pytest.raises(ConfigError, match="Unsupported model architecture"):
        config_class_for({"model_type": "mamba"})
    (tmp_path / "config.json").write_text(json.dumps(TINY_B))
    assert read_config(str(tmp_path)).hidden_size == 96
    with pytest.raises(ConfigError, match="config.json"):
        read_config(str(tmp_path / "nowhere"))


def test_another_architecture_can_be_registered():
    class Other:
        @classmethod
        def from_dict(cls, cfg, max_tokens=None):
            return cls()
    register_architecture("toy-arch", Other)
    assert config_class_for({"model_type": "toy-arch"}) is Other


def test_round_trip_through_config_json():
    for cfg in (TINY_A, TINY_B, TINY_C):
        c = MiniCPMConfig.from_dict(cfg)
        assert MiniCPMConfig.from_dict(json.loads(json.dumps(c.to_dict()))) == c


def test_run_order_is_checked():
    spec = MiniCPMConfig.from_dict(TINY_A).model_spec()
    kw = {f: getattr(spec, f) for f in spec.__dataclass_fields__}
    ModelSpec(**dict(kw, order=(RunEntry(0, 0), RunEntry(1, 1), RunEntry(0, 2), RunEntry(1, 0, False))))
    with pytest.raises(ConfigError, match="both write"):
        ModelSpec(**dict(kw, order=(RunEntry(0, 0), RunEntry(1, 0))))
    with pytest.raises(ConfigError, match="before any entry has written"):
        ModelSpec(**dict(kw, order=(RunEntry(0, 1, False), RunEntry(1, 1))))
    with pytest.raises(ConfigError, match="names layer"):
        ModelSpec(**dict(kw, order=(RunEntry(5, 0),)))
