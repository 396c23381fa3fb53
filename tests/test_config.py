"""Configuration and registry (no GPU)."""
import json
import os

import pytest

import wick_b200 as wick
from helpers import CONFIG_A, CONFIG_B, CONFIG_C, tmp_root


def test_fields_come_from_config_json_keys():
    a = wick.config_from_json(CONFIG_A)
    assert isinstance(a, wick.Qwen3Config)
    assert (a.hidden_size, a.num_attention_heads, a.num_key_value_heads, a.head_dim) == (64, 4, 2, 16)
    assert (a.intermediate_size, a.num_hidden_layers, a.vocab_size) == (192, 2, 512)
    assert a.rope_theta == 10000.0 and a.rms_norm_eps == 1e-6 and a.tie_word_embeddings
    assert a.q_dim == 64 and a.kv_dim == 32
    b = wick.config_from_json(CONFIG_B)
    assert b.rope_theta == 1e6, "rope_theta inside rope_parameters (config.rs:79-86)"
    assert b.q_dim == 192 != b.hidden_size, "head_dim is decoupled from hidden_size / heads"
    assert b.eos_token_ids == (7, 9) and b.stop_token_ids == (7, 9)


def test_defaults_follow_the_reference():
    j = dict(architectures=["Qwen3ForCausalLM"], hidden_size=64, num_attention_heads=4, intermediate_size=8,
             num_hidden_layers=1, vocab_size=10)
    c = wick.config_from_json(j)
    assert c.num_key_value_heads == 4          # config.rs:72
    assert c.head_dim == 16                    # config.rs:73
    assert c.max_position_embeddings == 4096   # config.rs:116
    assert c.rms_norm_eps == 1e-6              # config.rs:117
    assert c.rope_theta == 10000.0             # config.rs:86
    assert c.tie_word_embeddings is False and c.eos_token_ids == () and c.bos_token_id is None


def test_top_level_rope_theta_wins():
    j = dict(CONFIG_B, rope_theta=777.0)
    assert wick.config_from_json(j).rope_theta == 777.0


def test_model_type_selects_when_architectures_is_absent():
    j = dict(CONFIG_A)
    del j["architectures"]
    assert wick.config_from_json(j).architecture == "qwen3"
    del j["model_type"]
    with pytest.raises(wick.ConfigError, match="no architectures"):
        wick.config_from_json(j)


@pytest.mark.parametrize("patch, message", [
    ({"architectures": ["GPT2LMHeadModel"]}, "unsupported architecture GPT2LMHeadModel"),
    ({"hidden_size": None}, "missing hidden_size"),
    ({"vocab_size": None}, "missing vocab_size"),
    ({"num_hidden_layers": None}, "missing num_hidden_layers"),
    ({"intermediate_size": None}, "missing intermediate_size"),
    ({"hidden_act": "gelu"}, "unsupported activation gelu"),
    ({"num_key_value_heads": 3}, "multiple of num_key_value_heads"),
    ({"head_dim": 15}, "head_dim must be even"),
    ({"rope_scaling": {"rope_type": "yarn", "factor": 4.0}}, "unsupported rope_scaling type"),
    ({"attention_bias": True}, "attention_bias"),
    ({"use_sliding_window": True, "sliding_window": 128}, "sliding_window"),
    ({"layer_types": ["full_attention", "sliding_attention"]}, "layer_types"),
])
def test_bad_configs_are_refused(patch, message):
    j = dict(CONFIG_A)
    for k, v in patch.items():
        if v is None:
            j.pop(k)
        else:
            j[k] = v
    with pytest.raises(wick.ConfigError, match=message):
        wick.config_from_json(j)


def test_ignored_keys_of_a_real_config_do_not_matter():
    j = dict(CONFIG_A, attention_dropout=0.0, initializer_range=0.25, dtype="float32", pad_token_id=None,
             use_cache=True, sliding_window=None, use_sliding_window=False, max_window_layers=28,
             layer_types=["full_attention"] * 2, transformers_version="5.20.2", attention_bias=False)
    assert wick.config_from_json(j) == wick.config_from_json(CONFIG_A)


def test_round_trip_through_to_json():
    for j in (CONFIG_A, CONFIG_B, CONFIG_C):
        c = wick.config_from_json(j)
        c2 = wick.config_from_json(json.loads(json.dumps(c.to_json())))
        assert c2 == wick.Qwen3Config(**{**c.__dict__, "architecture": "Qwen3ForCausalLM"})


def test_load_config_merges_generation_config_stop_tokens():
    d = os.path.join(tmp_root(), "cfg-merge")
    os.makedirs(d, exist_ok=True)
    json.dump(dict(CONFIG_B, eos_token_id=7), open(os.path.join(d, "config.json"), "w"))
    json.dump({"eos_token_id": [7, 11, 12]}, open(os.path.join(d, "generation_config.json"), "w"))
    assert wick.load_config(d).eos_token_ids == (7, 11, 12)    # config.rs:140-149
    with pytest.raises(wick.ConfigError, match="config.json"):
        wick.load_config(os.path.join(d, "nowhere"))


def test_registry_maps_names_to_one_architecture_and_takes_new_ones():
    assert wick.get_architecture("Qwen3ForCausalLM") is wick.get_architecture("qwen3")
    assert "Qwen3ForCausalLM" in wick.architecture_names()
    spec = wick.get_architecture("qwen3").build_spec(wick.config_from_json(CONFIG_B))
    assert len(spec.layers) == 3 and [e.layer for e in spec.schedule] == [0, 1, 2]
    assert spec.layers[1].mixer.kind == "gqa_attention" and spec.layers[1].mixer.params["head_dim"] == 32
    assert spec.layers[0].mixer.params["qk_norm"].params == {"width": 32, "eps": 1e-5}
    assert spec.head.params["tied"] is False and spec.vocab == 1000

    # another architecture is one more entry
    class ToyConfig(wick.Qwen3Config):
        pass

    arch = wick.Architecture(names=("ToyForCausalLM",), config_cls=ToyConfig,
                             build_spec=wick.get_architecture("qwen3").build_spec)
    wick.register_architecture(arch)
    c = wick.config_from_json(dict(CONFIG_A, architectures=["ToyForCausalLM"]))
    assert type(c) is ToyConfig and c.architecture == "ToyForCausalLM"


def test_param_count_of_the_8b_shape():
    c = wick.config_from_json(dict(architectures=["Qwen3ForCausalLM"], hidden_size=4096, num_attention_heads=32,
                                   num_key_value_heads=8, head_dim=128, intermediate_size=12288,
                                   num_hidden_layers=36, vocab_size=151936))
    assert c.param_count() == 8_190_735_360


def test_schedule_validation():
    spec = wick.get_architecture("qwen3").build_spec(wick.config_from_json(CONFIG_A))
    import dataclasses
    bad = dataclasses.replace(spec, schedule=(wick.ScheduleEntry(0), wick.ScheduleEntry(5)))
    with pytest.raises(ValueError, match="names layer 5"):
        bad.validate()
    bad = dataclasses.replace(spec, schedule=(wick.ScheduleEntry(0, read_cache_of=0),))
    with pytest.raises(ValueError, match="does not run before"):
        bad.validate()
    ok = dataclasses.replace(spec, schedule=(wick.ScheduleEntry(0), wick.ScheduleEntry(1), wick.ScheduleEntry(1),
                                             wick.ScheduleEntry(0, read_cache_of=0)))
    ok.validate()
