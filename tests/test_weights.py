"""Weight loading by name, its one error, and the random-weights mode (CPU)."""

import json
import os

import pytest
import torch
from safetensors.torch import load_file, save_file

from conftest import TINY_A, TINY_B
from tandem_b200.config.model_config import Qwen3Config
from tandem_b200.config.plan import ParamSpec, WeightSource
from tandem_b200.models.qwen3 import build_plan, tensor_shapes
from tandem_b200.weights.loader import SafetensorsFolder, TensorDict, WeightError, load_parameters
from tandem_b200.weights.random_init import write_random_model


def _params(cfg_dict):
    from tandem_b200.registry import part

    plan = build_plan(Qwen3Config.from_dict(cfg_dict))
    params = {"embedding": ParamSpec((plan.embedding.vocab_size, plan.embedding.hidden_size),
                                     (WeightSource(plan.embedding.weight),))}
    for i, layer in enumerate(plan.layers):
        for slot, family, spec in layer.parts:
            for local, ps in part(family, spec.kind).params(spec).items():
                params[f"layers.{i}.{slot}.{local}"] = ps
    params["final_norm.weight"] = ParamSpec((plan.final_norm.size,), (WeightSource(plan.final_norm.weight),), "vector")
    if plan.head.weight:
        params["head"] = ParamSpec((plan.head.vocab_size, plan.head.hidden_size), (WeightSource(plan.head.weight),))
    return params, plan


def test_random_folder_has_config_and_every_tensor(tmp_path):
    folder = write_random_model(TINY_B, str(tmp_path / "m"), seed=5)
    cfg = json.load(open(os.path.join(folder, "config.json")))
    assert cfg["architectures"] == ["Qwen3ForCausalLM"] and cfg["head_dim"] == 32
    t = load_file(os.path.join(folder, "model.safetensors"))
    assert {n: tuple(v.shape) for n, v in t.items()} == tensor_shapes(Qwen3Config.from_dict(TINY_B))
    assert all(v.dtype == torch.bfloat16 for v in t.values())
    w = t["model.layers.1.mlp.down_proj.weight"].float()
    assert abs(w.std().item() - 0.02) < 0.002 and abs(w.mean().item()) < 0.002
    n = t["model.layers.0.input_layernorm.weight"].float()
    assert 0.9 <= n.min() and n.max() <= 1.1 and n.std() > 0.01


def test_random_weights_depend_on_seed_only(tmp_path):
    a = load_file(os.path.join(write_random_model(TINY_A, str(tmp_path / "a"), seed=1), "model.safetensors"))
    b = load_file(os.path.join(write_random_model(TINY_A, str(tmp_path / "b"), seed=1), "model.safetensors"))
    c = load_file(os.path.join(write_random_model(TINY_A, str(tmp_path / "c"), seed=2), "model.safetensors"))
    assert all(torch.equal(a[n], b[n]) for n in a)
    assert not torch.equal(a["model.embed_tokens.weight"], c["model.embed_tokens.weight"])


def test_fused_rows_and_held_dtypes(tmp_path):
    folder = write_random_model(TINY_B, str(tmp_path / "m"), seed=5)
    raw = load_file(os.path.join(folder, "model.safetensors"))
    params, plan = _params(TINY_B)
    got = load_parameters(params, SafetensorsFolder(folder), torch.bfloat16, "cpu", plan.ignored_weights)
    p = "model.layers.2.self_attn"
    qkv = got["layers.2.mixer.qkv"]
    assert qkv.shape == (192 + 64 + 64, 96) and qkv.dtype == torch.bfloat16
    assert torch.equal(qkv[:192], raw[f"{p}.q_proj.weight"])  # rows [q | k | v], loader.py:50-51 of the reference
    assert torch.equal(qkv[192:256], raw[f"{p}.k_proj.weight"]) and torch.equal(qkv[256:], raw[f"{p}.v_proj.weight"])
    gu = got["layers.0.feed_forward.gate_up"]
    assert torch.equal(gu[:256], raw["model.layers.0.mlp.gate_proj.weight"])
    assert torch.equal(gu[256:], raw["model.layers.0.mlp.up_proj.weight"])
    assert got["layers.1.mixer.q_norm"].dtype == torch.float32  # norm weights are held in 32 bits
    assert got["final_norm.weight"].dtype == torch.float32
    full = load_parameters(params, SafetensorsFolder(folder), torch.float32, "cpu", plan.ignored_weights)
    assert full["head"].dtype == torch.float32 and torch.equal(full["head"], raw["lm_head.weight"].float())


def test_tensors_spread_over_several_files(tmp_path):
    """A folder may hold its tensors in several *.safetensors files (python/tandem/models/loader.py:67-78)."""
    folder = write_random_model(TINY_B, str(tmp_path / "m"), seed=5)
    path = os.path.join(folder, "model.safetensors")
    raw = load_file(path)
    names = sorted(raw)
    params, plan = _params(TINY_B)
    whole = load_parameters(params, SafetensorsFolder(folder), torch.bfloat16, "cpu", plan.ignored_weights)
    os.remove(path)
    for i in range(3):
        save_file({n: raw[n] for n in names[i::3]}, os.path.join(folder, f"model-{i + 1:05d}-of-00003.safetensors"))
    parts = load_parameters(params, SafetensorsFolder(folder), torch.bfloat16, "cpu", plan.ignored_weights)
    assert parts.keys() == whole.keys() and all(torch.equal(parts[k], whole[k]) for k in whole)


def test_a_32_bit_vector_stays_32_bit(tmp_path):
    folder = write_random_model(TINY_A, str(tmp_path / "m"), seed=5)
    path = os.path.join(folder, "model.safetensors")
    raw = load_file(path)
    exact = torch.full((64,), 1.0 + 2.0 ** -20)  # not representable in bfloat16
    raw["model.norm.weight"] = exact
    save_file(raw, path)
    params, plan = _params(TINY_A)
    got = load_parameters(params, SafetensorsFolder(folder), torch.bfloat16, "cpu", plan.ignored_weights)
    assert torch.equal(got["final_norm.weight"], exact)


def test_one_error_lists_missing_unexpected_and_shapes(tmp_path):
    folder = write_random_model(TINY_A, str(tmp_path / "m"), seed=5)
    path = os.path.join(folder, "model.safetensors")
    raw = load_file(path)
    del raw["model.layers.1.mlp.up_proj.weight"]
    del raw["model.norm.weight"]
    raw["model.layers.0.self_attn.k_proj.weight"] = torch.zeros(16, 64, dtype=torch.bfloat16)
    raw["model.layers.0.extra.weight"] = torch.zeros(3)
    raw["model.layers.0.self_attn.rotary_emb.inv_freq"] = torch.zeros(8)  # ignored as in loader.py:16
    raw["lm_head.weight"] = torch.zeros(512, 64)  # tied model: tolerated (loader.py:94-97)
    save_file(raw, path)
    params, plan = _params(TINY_A)
    with pytest.raises(WeightError) as e:
        load_parameters(params, SafetensorsFolder(folder), torch.float32, "cpu", plan.ignored_weights)
    err = e.value
    assert err.missing == ["model.layers.1.mlp.up_proj.weight", "model.norm.weight"]
    assert err.unexpected == ["model.layers.0.extra.weight"]
    assert err.wrong_shape == [("model.layers.0.self_attn.k_proj.weight", (16, 64), (32, 64))]
    text = str(err)
    for word in ("missing", "unexpected", "wrong shape", "up_proj", "extra.weight", "(16, 64)", "(32, 64)"):
        assert word in text


def test_no_safetensors_files(tmp_path):
    with pytest.raises(FileNotFoundError):
        SafetensorsFolder(str(tmp_path))


def test_tensor_dict_source():
    params = {"w": ParamSpec((4, 2), (WeightSource("a", 0, 1), WeightSource("b", 1, 3)))}
    src = TensorDict({"a": torch.ones(1, 2), "b": torch.zeros(3, 2)})
    got = load_parameters(params, src, torch.float32, "cpu")
    assert got["w"].tolist() == [[1, 1], [0, 0], [0, 0], [0, 0]]
    with pytest.raises(WeightError):
        load_parameters(params, TensorDict({"a": torch.ones(2, 2)}), torch.float32, "cpu")
