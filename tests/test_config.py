import json

import pytest

from conftest import TINY
from lumenllm_b200.config import (ConfigError, ParametersFile, Qwen3Config, config_from_dict,
                                  load_config)


def test_fields_come_from_config_json():
    for name, d in TINY.items():
        c = config_from_dict(d)
        assert isinstance(c, Qwen3Config)
        for k in ("hidden_size", "num_hidden_layers", "num_attention_heads", "num_key_value_heads",
                  "head_dim", "intermediate_size", "vocab_size", "rope_theta", "rms_norm_eps",
                  "max_position_embeddings", "tie_word_embeddings"):
            assert getattr(c, k) == d[k], (name, k)
        spec = c.model_spec()
        assert len(spec.layers) == d["num_hidden_layers"]
        m = spec.layers[0].mixer.params
        assert (m["num_heads"], m["num_kv_heads"], m["head_dim"]) == (
            d["num_attention_heads"], d["num_key_value_heads"], d["head_dim"])
        assert m["softmax_scale"] == d["head_dim"] ** -0.5
        assert m["position"].params["theta"] == d["rope_theta"]
        assert spec.layers[0].norms["mixer"].params["eps"] == d["rms_norm_eps"]
        assert [e.layer for e in spec.schedule] == list(range(d["num_hidden_layers"]))


def test_defaults_of_absent_keys():
    d = dict(architectures=["Qwen3ForCausalLM"], hidden_size=64, num_hidden_layers=1,
             num_attention_heads=4, vocab_size=10, intermediate_size=8)
    c = config_from_dict(d)
    assert c.num_key_value_heads == 4 and c.head_dim == 16
    assert c.rope_theta == 10000.0 and c.rms_norm_eps == 1e-5
    assert c.tie_word_embeddings is False


def test_head_dim_is_decoupled_from_width():
    c = config_from_dict(TINY["B"])
    assert c.num_attention_heads * c.head_dim != c.hidden_size
    m = c.model_spec().layers[0].mixer
    from lumenllm_b200.parts import part_tensors
    t = part_tensors("mixer", m)
    assert t["model.layers.0.self_attn.q_proj.weight"][0] == (256, 96)
    assert t["model.layers.0.self_attn.o_proj.weight"][0] == (96, 256)


def test_window_layers():
    c = config_from_dict(TINY["C"])
    assert [c.window_of_layer(i) for i in range(4)] == [0, 24, 24, 24]
    spec = c.model_spec()
    assert [l.mixer.params["window"] for l in spec.layers] == [0, 24, 24, 24]
    d = dict(TINY["C"], layer_types=["sliding_attention", "full_attention"] * 2)
    c2 = config_from_dict(d)
    assert [c2.window_of_layer(i) for i in range(4)] == [24, 0, 24, 0]


def test_registry_by_model_type_and_unknown():
    d = dict(TINY["A"])
    d.pop("architectures")
    assert isinstance(config_from_dict(d), Qwen3Config)
    with pytest.raises(ConfigError, match="unknown architecture"):
        config_from_dict(dict(TINY["A"], architectures=["LlamaForCausalLM"], model_type="llama"))


@pytest.mark.parametrize("patch, msg", [
    ({"attention_bias": True}, "attention_bias"),
    ({"hidden_act": "gelu"}, "hidden_act"),
    ({"rope_scaling": {"rope_type": "yarn", "factor": 4.0}}, "rope_scaling"),
    ({"num_key_value_heads": 3}, "multiple"),
    ({"head_dim": 15}, "even"),
    ({"hidden_size": -1}, "positive"),
    ({"use_sliding_window": True, "sliding_window": None}, "sliding_window"),
])
def test_refused_values(patch, msg):
    with pytest.raises(ConfigError, match=msg):
        config_from_dict(dict(TINY["A"], **patch))


def test_missing_key_and_missing_file(tmp_path):
    d = dict(TINY["A"])
    d.pop("hidden_size")
    with pytest.raises(ConfigError, match="hidden_size"):
        config_from_dict(d)
    with pytest.raises(ConfigError, match="missing file"):
        load_config(tmp_path)
    (tmp_path / "config.json").write_text("{not json")
    with pytest.raises(ConfigError, match="not valid JSON"):
        load_config(tmp_path)


def test_round_trip_and_eos():
    c = config_from_dict(dict(TINY["B"], eos_token_id=[5, 7]))
    assert c.eos_token_ids == (5, 7)
    c2 = config_from_dict(c.to_dict())
    assert c2 == c
    assert config_from_dict(dict(TINY["B"], eos_token_id=9)).model_spec().eos_token_ids == (9,)


def test_schedule_validation():
    from dataclasses import replace
    from lumenllm_b200.config import ScheduleEntry
    spec = config_from_dict(TINY["A"]).model_spec()
    ok = replace(spec, schedule=(ScheduleEntry(0), ScheduleEntry(1), ScheduleEntry(0),
                                 ScheduleEntry(1, cache_from=1)))
    ok.validate()
    with pytest.raises(ConfigError, match="does not run before"):
        replace(spec, schedule=(ScheduleEntry(0, cache_from=1), ScheduleEntry(1))).validate()
    with pytest.raises(ConfigError, match="names layer"):
        replace(spec, schedule=(ScheduleEntry(5),)).validate()


def test_parameters_file(tmp_path):
    p = tmp_path / "parameters.json"
    p.write_text(json.dumps({
        "model": {"path": "m", "compute": "cuda:0", "store": "vram", "dtype": "float32",
                  "hidden-layers": {"kv-cache": {"context-size": 512, "type-k": "f32"}},
                  "other-parameters": {"temperature": 0.7, "top-p": 0.9, "top-k": 40, "min-p": 0.05,
                                       "seed": 3, "batch-size": 4}},
        "cuda": {"device": 0}}))
    pf = ParametersFile.from_path(p)
    assert pf.model_path == str(tmp_path / "m") and pf.dtype == "float32"
    assert pf.context_size == 512 and pf.batch_size == 4
    s = pf.sampling
    assert (s.temperature, s.top_p, s.top_k, s.min_p, s.seed) == (0.7, 0.9, 40, 0.05, 3)
    with pytest.raises(ConfigError, match="unknown key"):
        ParametersFile.from_dict({"model": {"path": "m", "colour": 1}})
    with pytest.raises(ConfigError, match="exactly one"):
        ParametersFile.from_dict({"model": {}})
    with pytest.raises(ConfigError, match="CUDA device"):
        ParametersFile.from_dict({"model": {"path": "m", "compute": "cpu"}})
    with pytest.raises(ConfigError, match="quantized"):
        ParametersFile.from_dict({"model": {"path": "m", "hidden-layers": {
            "kv-cache": {"type-k": "fp8"}}}})
    assert ParametersFile.from_dict({"model": {"path": "m"}}).sampling.temperature == 0.0


def test_eos_ids_are_the_union_of_both_files(tmp_path):
    """config.json names one id, generation_config.json another (a number or a list in either):
    generation stops at both; a folder without the second file keeps config.json's."""
    import json
    from lumenllm_b200.config import load_config
    (tmp_path / "config.json").write_text(json.dumps(dict(TINY["B"], eos_token_id=5)))
    assert load_config(tmp_path).model_spec().eos_token_ids == (5,)
    (tmp_path / "generation_config.json").write_text(json.dumps({"eos_token_id": [9, 5], "top_k": 20}))
    assert load_config(tmp_path).model_spec().eos_token_ids == (5, 9)
    (tmp_path / "config.json").write_text(json.dumps(dict(TINY["B"])))
    (tmp_path / "generation_config.json").write_text(json.dumps({"eos_token_id": 7}))
    assert load_config(tmp_path).model_spec().eos_token_ids == (7,)
    (tmp_path / "generation_config.json").write_text(json.dumps({"temperature": 0.6}))
    assert load_config(tmp_path).model_spec().eos_token_ids == ()
    (tmp_path / "generation_config.json").write_text(json.dumps({"eos_token_id": "x"}))
    with pytest.raises(ConfigError, match="generation_config.json.*eos_token_id"):
        load_config(tmp_path)
    (tmp_path / "generation_config.json").write_text("{not json")
    with pytest.raises(ConfigError, match="not valid JSON"):
        load_config(tmp_path)
