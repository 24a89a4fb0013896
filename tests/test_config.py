"""Configuration and registry (no GPU)."""
import copy
import json

import pytest

import tiny_configs
from rust_deeplearning_b200.config.base import (ConfigError, architecture_for, load_config, register_architecture,
                                                registered_architectures, Architecture)
from rust_deeplearning_b200.config.gemma2 import Gemma2Config, build_spec

# the shape the reference's own parsing test uses (rustml/nlp/main/src/api/types.rs:907-919), with the keys it omits
GEMMA2_2B = {
    "architectures": ["Gemma2ForCausalLM"], "model_type": "gemma2", "hidden_size": 2304, "intermediate_size": 9216,
    "num_hidden_layers": 26, "num_attention_heads": 8, "num_key_value_heads": 4, "head_dim": 256, "vocab_size": 256000,
    "rms_norm_eps": 1e-6, "max_position_embeddings": 8192, "rope_theta": 10000.0, "attn_logit_softcapping": 50.0,
    "final_logit_softcapping": 30.0, "sliding_window": 4096, "query_pre_attn_scalar": 256,
    "hidden_activation": "gelu_pytorch_tanh", "bos_token_id": 2, "eos_token_id": 1,
}


def test_registry_names_the_architecture():
    assert "Gemma2ForCausalLM" in registered_architectures()
    assert architecture_for(GEMMA2_2B).name == "Gemma2ForCausalLM"
    assert architecture_for({"model_type": "gemma2"}).name == "Gemma2ForCausalLM"      # by model_type alone
    with pytest.raises(ConfigError) as e:
        architecture_for({"architectures": ["LlamaForCausalLM"], "model_type": "llama"})
    assert "Gemma2ForCausalLM" in str(e.value)                                           # lists what is registered
    with pytest.raises(ConfigError):
        register_architecture(Architecture("Gemma2ForCausalLM", "gemma2", Gemma2Config.from_dict, build_spec))


@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_every_size_comes_from_the_file(name):
    raw, _ = tiny_configs.config(name)
    cfg = load_config(raw)
    assert (cfg.num_hidden_layers, cfg.hidden_size, cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim,
            cfg.intermediate_size, cfg.vocab_size) == tuple(raw[k] for k in (
                "num_hidden_layers", "hidden_size", "num_attention_heads", "num_key_value_heads", "head_dim",
                "intermediate_size", "vocab_size"))
    assert cfg.rms_norm_eps == raw["rms_norm_eps"] and cfg.rope_theta == raw["rope_theta"]
    assert cfg.sliding_window == raw["sliding_window"]
    assert cfg.attn_logit_softcapping == raw["attn_logit_softcapping"]
    assert cfg.final_logit_softcapping == raw["final_logit_softcapping"]
    spec = build_spec(cfg)
    assert len(spec.layers) == raw["num_hidden_layers"] and len(spec.schedule) == raw["num_hidden_layers"]
    for i, layer in enumerate(spec.layers):
        p = layer.mixer.params
        want_window = raw["sliding_window"] if (i % 2 == 0 and raw["sliding_window"]) else None
        assert p["window"] == want_window                                   # even layers local, odd global
        assert p["score_scale"] == pytest.approx(raw["query_pre_attn_scalar"] ** -0.5)
        assert p["softcap"] == raw["attn_logit_softcapping"]
        assert p["position"].params["theta"] == raw["rope_theta"]
        assert all(n.params["eps"] == raw["rms_norm_eps"] and n.params["offset"] == 1.0 for n in layer.norms.values())
        assert set(layer.norms) == {"pre_mixer", "post_mixer", "pre_feed_forward", "post_feed_forward"}
    assert spec.head.params["softcap"] == raw["final_logit_softcapping"]
    assert spec.head.tensors["weight"].name == "model.embed_tokens.weight"    # tied
    assert spec.embedding.params["scale"] == pytest.approx(raw["hidden_size"] ** 0.5)


def test_gemma2_2b_shape_and_tensor_names():
    cfg = load_config(GEMMA2_2B)
    spec = build_spec(cfg)
    names = spec.tensor_specs()
    assert len(names) == 26 * 11 + 2
    assert names["model.layers.25.self_attn.q_proj.weight"].shape == (8 * 256, 2304)
    assert names["model.layers.0.self_attn.k_proj.weight"].shape == (4 * 256, 2304)
    assert names["model.layers.3.mlp.down_proj.weight"].shape == (2304, 9216)
    assert names["model.norm.weight"].kind == "vector"
    assert sum(int(__import__("numpy").prod(t.shape)) for t in names.values()) == 2_614_341_888
    assert spec.stop_token_ids == (1,)


def test_optional_keys_and_their_defaults():
    raw = copy.deepcopy(GEMMA2_2B)
    for k in ("num_key_value_heads", "attn_logit_softcapping", "final_logit_softcapping", "sliding_window"):
        del raw[k]
    raw["hidden_act"] = raw.pop("hidden_activation")
    cfg = load_config(raw)
    assert cfg.num_key_value_heads == 8 and cfg.sliding_window is None
    assert cfg.attn_logit_softcapping is None and cfg.final_logit_softcapping is None
    assert all(t == "full_attention" for t in cfg.layer_types)
    raw["eos_token_id"] = [1, 107]
    assert load_config(raw).eos_token_id == (1, 107)
    raw["layer_types"] = ["full_attention"] * 26
    assert load_config(raw).layer_types == tuple(["full_attention"] * 26)
    raw["tie_word_embeddings"] = False
    assert "lm_head.weight" in build_spec(load_config(raw)).tensor_specs()


def test_all_problems_are_reported_together():
    raw = copy.deepcopy(GEMMA2_2B)
    del raw["head_dim"], raw["rope_theta"]
    raw["num_hidden_layers"] = "26"
    raw["num_key_value_heads"] = 3
    raw["rms_norm_eps"] = -1
    with pytest.raises(ConfigError) as e:
        load_config(raw)
    msg = str(e.value)
    for piece in ("head_dim", "rope_theta", "num_hidden_layers", "multiple of num_key_value_heads", "rms_norm_eps"):
        assert piece in msg, piece
    bad = copy.deepcopy(GEMMA2_2B)
    bad["head_dim"] = 255
    with pytest.raises(ConfigError):
        load_config(bad)
    bad = copy.deepcopy(GEMMA2_2B)
    bad["layer_types"] = ["sliding_attention"] * 25
    with pytest.raises(ConfigError):
        load_config(bad)
    # sizes beyond what 32-bit indices hold, numbers that are not finite, names of the wrong type: refused, not tried
    for key, value in (("num_hidden_layers", 2 ** 40), ("vocab_size", 2 ** 31), ("rms_norm_eps", float("inf")),
                       ("rope_theta", float("nan")), ("architectures", 5), ("architectures", [5, None]), ("model_type", ["gemma2"])):
        bad = copy.deepcopy(GEMMA2_2B)
        bad[key] = value
        if key == "architectures":
            bad.pop("model_type", None)
        if key == "model_type":
            bad.pop("architectures", None)
        with pytest.raises(ConfigError):
            load_config(bad)


def test_config_json_from_a_folder(tmp_path):
    (tmp_path / "config.json").write_text(json.dumps(GEMMA2_2B))
    assert load_config(str(tmp_path)).hidden_size == 2304
    with pytest.raises(ConfigError):
        load_config(str(tmp_path / "nowhere"))
    (tmp_path / "config.json").write_text("{not json")
    with pytest.raises(ConfigError):
        load_config(str(tmp_path))
