"""Configuration and registry (CPU)."""

import json

import pytest

from conftest import TINY_A, TINY_B, TINY_C
from tandem_b200.config.engine_config import EngineConfig
from tandem_b200.config.model_config import ConfigError, Qwen3Config, read_config_json
from tandem_b200.models.qwen3 import build_plan
from tandem_b200.registry import resolve_architecture, supported_architectures


def test_reads_every_size_from_config():
    c = Qwen3Config.from_dict(TINY_B)
    assert (c.num_hidden_layers, c.hidden_size, c.num_attention_heads, c.num_key_value_heads, c.head_dim) == (3, 96, 6, 2, 32)
    assert (c.intermediate_size, c.vocab_size, c.rope_theta, c.rms_norm_eps) == (256, 1000, 1e6, 1e-5)
    assert not c.tie_word_embeddings and c.max_position_embeddings == 512
    assert c.q_size == 192 != c.hidden_size  # head_dim is decoupled from hidden_size / heads


def test_defaults_follow_the_reference():
    d = dict(architectures=["Qwen3ForCausalLM"], vocab_size=10, hidden_size=32, num_hidden_layers=1,
             num_attention_heads=4, intermediate_size=8)
    c = Qwen3Config.from_dict(d)
    assert c.num_key_value_heads == 4 and c.head_dim == 8  # model_config.py:100-101,125
    assert c.rms_norm_eps == 1e-6 and c.rope_theta == 10000.0 and c.max_position_embeddings == 4096
    assert c.tie_word_embeddings is False and c.sliding_window is None


def test_rope_parameters_block():
    d = dict(TINY_A, rope_parameters={"rope_theta": 5e5, "rope_type": "default"})
    d.pop("rope_theta")
    assert Qwen3Config.from_dict(d).rope_theta == 5e5


@pytest.mark.parametrize("patch, word", [
    ({"rope_scaling": {"rope_type": "yarn", "factor": 4.0}}, "rope scaling"),
    ({"attention_bias": True}, "attention_bias"),
    ({"quantization_config": {"quant_method": "awq"}}, "quantized"),
    ({"hidden_act": "gelu"}, "hidden_act"),
    ({"num_key_value_heads": 3}, "multiple"),
    ({"head_dim": 15}, "even"),
    ({"vocab_size": None}, "vocab_size"),
    ({"use_sliding_window": True}, "sliding_window"),
])
def test_rejects_what_it_does_not_implement(patch, word):
    with pytest.raises(ConfigError, match=word):
        Qwen3Config.from_dict(dict(TINY_A, **patch))


def test_layer_types_decide_which_layers_have_a_window():
    kinds = ["sliding_attention", "full_attention", "sliding_attention", "full_attention"]
    c = Qwen3Config.from_dict(dict(TINY_C, layer_types=kinds, use_sliding_window=False))
    assert [c.layer_window(i) for i in range(4)] == [20, None, 20, None]
    assert Qwen3Config.from_dict(c.to_dict()) == c
    none = Qwen3Config.from_dict(dict(TINY_C, layer_types=["full_attention"] * 4))
    assert [none.layer_window(i) for i in range(4)] == [None] * 4
    with pytest.raises(ConfigError, match="4 layers"):
        Qwen3Config.from_dict(dict(TINY_C, layer_types=kinds[:3]))
    with pytest.raises(ConfigError, match="chunked_attention"):
        Qwen3Config.from_dict(dict(TINY_C, layer_types=["chunked_attention"] * 4))
    with pytest.raises(ConfigError, match="sliding_window"):
        Qwen3Config.from_dict(dict(TINY_A, layer_types=["sliding_attention"] * 2))


def test_unknown_architecture_lists_supported():
    with pytest.raises(NotImplementedError, match="Qwen3ForCausalLM"):
        resolve_architecture({"architectures": ["GPT2LMHeadModel"]})
    assert resolve_architecture({"model_type": "qwen3"}).name == "Qwen3ForCausalLM"
    assert supported_architectures() == ["Qwen3ForCausalLM"]


def test_round_trip_and_eos(tmp_path):
    c = Qwen3Config.from_dict(dict(TINY_C, eos_token_id=[5, 7]))
    assert Qwen3Config.from_dict(c.to_dict()) == c
    (tmp_path / "config.json").write_text(json.dumps(dict(TINY_A, eos_token_id=3)))
    (tmp_path / "generation_config.json").write_text(json.dumps({"eos_token_id": [3, 9]}))
    assert Qwen3Config.from_dict(read_config_json(str(tmp_path))).eos_token_ids == (3, 9)


def test_plan_is_chosen_layer_by_layer():
    plan = build_plan(Qwen3Config.from_dict(TINY_C))
    assert [l.slot("mixer").window for l in plan.layers] == [None, None, 20, 20]
    assert [r.layer for r in plan.order] == [0, 1, 2, 3] and all(r.cache_of is None for r in plan.order)
    m = plan.layers[0].slot("mixer")
    assert (m.num_heads, m.num_kv_heads, m.head_dim, m.qk_norm, m.qk_norm_eps) == (6, 3, 48, True, 3e-6)
    assert m.scale == 48 ** -0.5 and m.position.theta == 500000.0 and m.position.rotary_dim == 48
    assert plan.head.weight == "lm_head.weight" and build_plan(Qwen3Config.from_dict(TINY_A)).head.weight is None


def test_plan_rejects_bad_order():
    from dataclasses import replace

    from tandem_b200.config.plan import RunStep

    plan = build_plan(Qwen3Config.from_dict(TINY_A))
    replace(plan, order=(RunStep(0), RunStep(1), RunStep(0), RunStep(1, cache_of=1)))  # twice, and shared: fine
    with pytest.raises(ValueError):
        replace(plan, order=(RunStep(0), RunStep(5)))
    with pytest.raises(ValueError):
        replace(plan, order=(RunStep(0, cache_of=0),))


def test_engine_config_checks():
    assert EngineConfig(model="x", dtype="bf16").resolved_dtype == "bfloat16"
    assert EngineConfig(model="x").resolved_dtype == "bfloat16"
    with pytest.raises(ValueError):
        EngineConfig(model="x", dtype="float16")
    with pytest.raises(ValueError):
        EngineConfig(model="x", schedule_policy="random")
