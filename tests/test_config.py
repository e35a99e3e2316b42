"""Configuration and registry (no GPU)."""
import json

import pytest

import ghost_infer_b200 as gi
from ghost_infer_b200.config import (ConfigError, LlamaConfig, UnknownArchitectureError, load_config, parse_config,
                                     register_architecture, registered_architectures, unregister_architecture)
from ghost_infer_b200.config.llama_spec import build_llama_spec
from conftest import TINY_A, TINY_B


def test_parse_tiny_a():
    c = LlamaConfig.from_dict(TINY_A)
    assert (c.hidden_size, c.num_hidden_layers, c.num_attention_heads, c.num_key_value_heads) == (64, 2, 4, 2)
    assert c.head_dim == 16 and c.intermediate_size == 176 and c.vocab_size == 256
    assert c.rope_scaling is None and c.rope_theta == 10000.0 and c.rms_norm_eps == 1e-5
    assert not c.tie_word_embeddings and c.eos_token_ids == (7,)
    assert c.q_dim == 64 and c.kv_dim == 32 and c.group_size == 2
    assert abs(c.attention_scale - 0.25) < 1e-12


def test_parse_tiny_b_and_defaults():
    c = LlamaConfig.from_dict(TINY_B)
    assert c.rope_scaling.factor == 8.0 and c.rope_scaling.original_max_position_embeddings == 32
    assert c.tie_word_embeddings and c.eos_token_ids == (3, 5)
    d = {k: v for k, v in TINY_A.items() if k not in ("num_key_value_heads", "head_dim", "rope_theta", "rms_norm_eps")}
    c = LlamaConfig.from_dict(d)
    assert c.num_key_value_heads == 4          # defaults to the head count (src/model.rs:198)
    assert c.head_dim == 16                    # hidden / heads (src/model.rs:167)
    assert c.rope_theta == 10000.0 and c.rms_norm_eps == 1e-5


def test_roundtrip_to_dict():
    for raw in (TINY_A, TINY_B):
        c = LlamaConfig.from_dict(raw)
        assert LlamaConfig.from_dict(c.to_dict()) == c


@pytest.mark.parametrize("change, needle", [
    ({"hidden_size": None}, "hidden_size"),
    ({"num_attention_heads": 3, "num_key_value_heads": 2}, "multiple"),
    ({"head_dim": 15}, "even"),
    ({"vocab_size": 0}, "positive"),
    ({"num_hidden_layers": 1.5}, "integer"),
    ({"rope_scaling": {"rope_type": "yarn", "factor": 2.0}}, "yarn"),
    ({"rope_scaling": {"rope_type": "llama3", "factor": 8.0}}, "low_freq_factor"),
    ({"attention_bias": True}, "bias"),
    ({"hidden_act": "gelu"}, "gelu"),
    ({"eos_token_id": 999}, "vocabulary"),
    ({"rms_norm_eps": 0.0}, "rms_norm_eps"),
])
def test_config_errors(change, needle):
    raw = dict(TINY_A)
    raw.update(change)
    if change.get("hidden_size", 1) is None:
        del raw["hidden_size"]
    with pytest.raises(ConfigError) as e:
        LlamaConfig.from_dict(raw)
    assert needle in str(e.value)


def test_unknown_architecture_lists_registered():
    raw = dict(TINY_A, architectures=["MambaForCausalLM"])
    with pytest.raises(UnknownArchitectureError) as e:
        parse_config(raw)
    assert "MambaForCausalLM" in str(e.value) and "LlamaForCausalLM" in str(e.value)


def test_registry_add_and_remove():
    assert "LlamaForCausalLM" in registered_architectures()
    register_architecture("ToyForCausalLM", LlamaConfig.from_dict, build_llama_spec)
    try:
        assert "ToyForCausalLM" in registered_architectures()
        with pytest.raises(ValueError):
            register_architecture("ToyForCausalLM", LlamaConfig.from_dict, build_llama_spec)
        m = gi.Model.from_config_dict(dict(TINY_A, architectures=["ToyForCausalLM"]))
        assert len(m.layers) == 2
    finally:
        unregister_architecture("ToyForCausalLM")
    assert "ToyForCausalLM" not in registered_architectures()


def test_load_config_from_folder(tmp_path):
    (tmp_path / "config.json").write_text(json.dumps(TINY_B))
    c = load_config(str(tmp_path))
    assert isinstance(c, LlamaConfig) and c.hidden_size == 96
    with pytest.raises(ConfigError):
        load_config(str(tmp_path / "nowhere"))
    (tmp_path / "config.json").write_text("{not json")
    with pytest.raises(ConfigError):
        load_config(str(tmp_path))


def test_spec_is_data():
    spec = build_llama_spec(LlamaConfig.from_dict(TINY_B))
    assert len(spec.layers) == 3 and [e.layer for e in spec.schedule] == [0, 1, 2]
    l0 = spec.layers[0]
    assert l0.mixer.kind == "gqa_attention" and l0.ffn.kind == "swiglu" and l0.mixer_norm.kind == "rmsnorm"
    assert l0.mixer["num_heads"] == 3 and l0.mixer["num_kv_heads"] == 1 and l0.mixer["head_dim"] == 32
    assert l0.mixer["position"].kind == "rotary" and l0.mixer["position"]["scaling"]["factor"] == 8.0
    assert l0.ffn["intermediate_size"] == 256 and l0.mixer_norm["eps"] == 1e-6
    assert spec.head["tied"] is True and spec.stop_token_ids == (3, 5)


def test_manifest_names_and_shapes():
    m = gi.Model.from_config_dict(TINY_A)
    man = {w.name: w for w in m.weight_manifest()}
    assert man["model.embed_tokens.weight"].shape == (256, 64)
    assert man["model.layers.1.self_attn.k_proj.weight"].shape == (32, 64)
    assert man["model.layers.0.mlp.down_proj.weight"].shape == (64, 176)
    assert man["model.norm.weight"].init == "ones" and man["lm_head.weight"].shape == (256, 64)
    mb = gi.Model.from_config_dict(TINY_B)
    assert "lm_head.weight" not in {w.name for w in mb.weight_manifest()}
