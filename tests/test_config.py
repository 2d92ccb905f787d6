"""Typed configuration and the architecture registry."""
import json

import pytest

from conftest import TINY_A, TINY_B
from math_utils_b200.config import (ConfigError, Gpt2Config, architecture_for, known_architectures,
                                    load_config)


def test_gpt2_keys_are_read():
    c = Gpt2Config.from_json(TINY_B)
    assert (c.n_layer, c.n_embd, c.n_head, c.inner, c.vocab_size, c.n_positions) == (3, 96, 3, 320, 1031, 80)
    assert c.head_dim == 32 and c.layer_norm_epsilon == 1e-6 and c.activation_function == "gelu"
    assert c.scale_attn_by_inverse_layer_idx is True and c.eos_token_ids == (11, 500)
    a = Gpt2Config.from_json(TINY_A)
    assert a.eos_token_ids == (7,) and a.inner == 256 and a.activation_function == "gelu_new"


def test_n_inner_defaults_to_four_times_width():
    raw = dict(TINY_A); raw.pop("n_inner")
    assert Gpt2Config.from_json(raw).inner == 4 * 64
    raw["n_inner"] = None
    assert Gpt2Config.from_json(raw).inner == 4 * 64


@pytest.mark.parametrize("key", ["n_layer", "n_embd", "n_head", "vocab_size", "n_positions"])
def test_sizes_have_no_default(key):
    raw = dict(TINY_A); raw.pop(key)
    with pytest.raises(ConfigError, match=key):
        Gpt2Config.from_json(raw)


@pytest.mark.parametrize("key,value", [("n_layer", 0), ("n_embd", "64"), ("n_head", 2.5),
                                        ("layer_norm_epsilon", -1.0), ("activation_function", "relu"),
                                        ("scale_attn_by_inverse_layer_idx", 1), ("eos_token_id", "x")])
def test_bad_values_name_their_key(key, value):
    with pytest.raises(ConfigError, match=key):
        Gpt2Config.from_json(dict(TINY_A, **{key: value}))


def test_heads_must_divide_width():
    with pytest.raises(ConfigError, match="n_head"):
        Gpt2Config.from_json(dict(TINY_A, n_head=5))


def test_plan_carries_every_size_and_option():
    plan = Gpt2Config.from_json(TINY_B).plan()
    assert plan.vocab_size == 1031 and plan.hidden_size == 96 and plan.max_positions == 80
    assert len(plan.layers) == 3 and [e.layer for e in plan.schedule] == [0, 1, 2]
    m0, m2 = plan.layers[0].mixer.params, plan.layers[2].mixer.params
    assert m0["n_heads"] == 3 and m0["head_dim"] == 32 and m0["window"] == 0
    assert m0["softmax_scale"] == pytest.approx(32 ** -0.5)
    assert m2["softmax_scale"] == pytest.approx(32 ** -0.5 / 3)       # scale_attn_by_inverse_layer_idx
    assert plan.layers[1].feed_forward.params == {"hidden_size": 96, "inner_size": 320, "activation": "gelu",
                                                  "weight_layout": "in_out"}
    assert plan.layers[1].norm1.params["eps"] == 1e-6
    assert plan.layers[1].mixer.tensors["qkv_weight"] == "h.1.attn.c_attn.weight"
    assert plan.stop_ids == (11, 500)


def test_registry_by_model_type_and_by_architecture():
    assert architecture_for({"model_type": "gpt2"}).config_class is Gpt2Config
    assert architecture_for({"architectures": ["GPT2LMHeadModel"]}).config_class is Gpt2Config
    assert "gpt2" in known_architectures() and "GPT2LMHeadModel" in known_architectures()
    with pytest.raises(ConfigError, match="known:.*gpt2"):
        architecture_for({"model_type": "llama"})
    with pytest.raises(ConfigError, match="model_type"):
        architecture_for({})


def test_load_config_from_folder(tmp_path):
    (tmp_path / "config.json").write_text(json.dumps(TINY_A))
    arch, config, plan = load_config(str(tmp_path))
    assert config.n_embd == 64 and plan.architecture == "GPT2LMHeadModel"
    (tmp_path / "config.json").write_text("{not json")
    with pytest.raises(ConfigError, match="not valid JSON"):
        load_config(str(tmp_path))
    with pytest.raises(ConfigError, match="no such file"):
        load_config(str(tmp_path / "missing"))


def test_schedule_validation():
    from dataclasses import replace
    from math_utils_b200.config import ScheduleEntry
    plan = Gpt2Config.from_json(TINY_A).plan()
    replace(plan, schedule=(ScheduleEntry(0, 0), ScheduleEntry(1, 1), ScheduleEntry(0, 0))).validate()
    with pytest.raises(ConfigError, match="runs later"):
        replace(plan, schedule=(ScheduleEntry(0, 1), ScheduleEntry(1, 1))).validate()
    with pytest.raises(ConfigError, match="names layer"):
        replace(plan, schedule=(ScheduleEntry(5, 0),)).validate()
    with pytest.raises(ConfigError, match="owns none"):
        replace(plan, schedule=(ScheduleEntry(0, 0), ScheduleEntry(1, 0), ScheduleEntry(1, 1))).validate()


def test_extra_parts_of_a_layer_are_checked():
    """A layer may carry parts beyond the four; their names are its own and each is (name, role, PartSpec)."""
    from dataclasses import replace
    plan = Gpt2Config.from_json(TINY_A).plan()
    first = plan.layers[0]
    third = ("norm3", "norm", first.norm1)
    replace(plan, layers=(replace(first, extra=(third,)),) + plan.layers[1:]).validate()
    with pytest.raises(ConfigError, match="is taken"):
        replace(plan, layers=(replace(first, extra=(("mixer", "norm", first.norm1),)),) + plan.layers[1:]).validate()
    with pytest.raises(ConfigError, match="is taken"):
        replace(plan, layers=(replace(first, extra=(third, third)),) + plan.layers[1:]).validate()
    with pytest.raises(ConfigError, match="an extra part is"):
        replace(plan, layers=(replace(first, extra=(("norm3", first.norm1),)),) + plan.layers[1:]).validate()


def test_stop_ids_of_generation_config_are_added(tmp_path):
    """eos_token_id of generation_config.json joins config.json's (include/ai/LocalModel.hpp:1788-1792)."""
    import json
    from math_utils_b200.config import load_config
    (tmp_path / "config.json").write_text(json.dumps(TINY_B))
    assert load_config(str(tmp_path))[2].stop_ids == (11, 500)
    (tmp_path / "generation_config.json").write_text(json.dumps({"eos_token_id": [500, 3], "max_length": 20}))
    assert load_config(str(tmp_path))[2].stop_ids == (11, 500, 3)
    (tmp_path / "generation_config.json").write_text(json.dumps({"eos_token_id": 9}))
    assert load_config(str(tmp_path))[2].stop_ids == (11, 500, 9)
    (tmp_path / "generation_config.json").write_text("not json")
    assert load_config(str(tmp_path))[2].stop_ids == (11, 500)
