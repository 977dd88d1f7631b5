"""Configuration and registry (no GPU)."""
import json

import pytest

from conftest import TINY_A, TINY_B
from zinfer_b200.config import (ConfigError, Family, Qwen3Config, UnknownArchitecture, family_for, load_config,
                                qwen3_model_spec, register_family, registered, unregister_family)


def test_reads_every_key_of_config_json():
    cfg = Qwen3Config.from_dict(TINY_B)
    for k in ("vocab_size", "hidden_size", "intermediate_size", "num_hidden_layers", "num_attention_heads",
              "num_key_value_heads", "head_dim", "max_position_embeddings", "rms_norm_eps", "rope_theta",
              "tie_word_embeddings"):
        assert getattr(cfg, k) == TINY_B[k]
    assert cfg.num_attention_heads * cfg.head_dim != cfg.hidden_size  # head size independent of the width


def test_unknown_keys_are_ignored_and_round_trip():
    cfg = Qwen3Config.from_dict({**TINY_A, "some_future_key": 3, "bos_token_id": 1})
    assert Qwen3Config.from_dict(cfg.to_dict()) == cfg


@pytest.mark.parametrize("key", ["hidden_size", "num_key_value_heads", "rope_theta", "rms_norm_eps", "vocab_size"])
def test_missing_required_key_is_an_error(key):
    raw = dict(TINY_A)
    del raw[key]
    with pytest.raises(ConfigError, match=key):
        Qwen3Config.from_dict(raw)


def test_head_dim_defaults_to_width_over_heads():
    raw = dict(TINY_A)
    del raw["head_dim"]
    assert Qwen3Config.from_dict(raw).head_dim == 16


@pytest.mark.parametrize("patch,match", [
    ({"num_key_value_heads": 3}, "multiple"), ({"head_dim": 15}, "even"), ({"vocab_size": 0}, "positive"),
    ({"rope_scaling": {"type": "yarn"}}, "rope_scaling"), ({"use_sliding_window": True}, "use_sliding_window"),
    ({"attention_bias": True}, "attention_bias"), ({"hidden_act": "gelu"}, "hidden_act")])
def test_what_would_change_the_arithmetic_is_refused(patch, match):
    with pytest.raises(ConfigError, match=match):
        Qwen3Config.from_dict({**TINY_A, **patch})


def test_registry_by_architecture_and_model_type(tmp_path):
    assert "Qwen3ForCausalLM" in registered()
    assert family_for({"architectures": ["Qwen3ForCausalLM"]}).name == "Qwen3ForCausalLM"
    assert family_for({"model_type": "qwen3"}).name == "Qwen3ForCausalLM"
    with pytest.raises(UnknownArchitecture, match="registered: .*Qwen3ForCausalLM"):
        family_for({"architectures": ["LlamaForCausalLM"], "model_type": "llama"})
    with pytest.raises(UnknownArchitecture):
        family_for({})
    (tmp_path / "config.json").write_text(json.dumps(TINY_B))
    fam, cfg = load_config(str(tmp_path))
    assert fam.name == "Qwen3ForCausalLM" and cfg.num_hidden_layers == 3


def test_another_family_can_be_registered():
    fam = Family("ToyForCausalLM", "toy", Qwen3Config, qwen3_model_spec)
    register_family(fam)
    try:
        assert family_for({"model_type": "toy"}) is fam
        with pytest.raises(ValueError):
            register_family(Family("ToyForCausalLM", "toy2", Qwen3Config, qwen3_model_spec))
    finally:
        unregister_family("ToyForCausalLM")
    assert "ToyForCausalLM" not in registered()


def test_model_spec_carries_every_constant():
    for raw in (TINY_A, TINY_B):
        cfg = Qwen3Config.from_dict(raw)
        spec = qwen3_model_spec(cfg)
        assert len(spec.layers) == cfg.num_hidden_layers == len(spec.schedule)
        block = spec.layers[0].block.params
        mixer = block["mixer"].params
        assert (mixer["num_heads"], mixer["num_kv_heads"], mixer["head_dim"]) == (
            cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim)
        assert mixer["qk_norm_eps"] == cfg.rms_norm_eps and mixer["position"].params["theta"] == cfg.rope_theta
        assert block["feed_forward"].params["intermediate_size"] == cfg.intermediate_size
        assert block["mixer_norm"].params["eps"] == cfg.rms_norm_eps
        assert spec.head.params["tied_to"] == ("model.embed_tokens" if cfg.tie_word_embeddings else None)
        assert spec.layers[1].prefix == "model.layers.1."
