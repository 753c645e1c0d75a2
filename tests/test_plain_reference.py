"""The plain implementation itself (CPU): against 12vivi/tandem's own model code through the
committed golden files, and its parts against direct formulas."""

import os
import tempfile

import numpy as np
import pytest
import torch

import plain_qwen3 as plain
from conftest import TINY, random_tokens
from tandem_b200.weights.random_init import write_random_model

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


@pytest.mark.parametrize("name", ["A", "B"])
def test_plain_matches_the_reference_model(name, tmp_path, monkeypatch):
    g = np.load(os.path.join(GOLDEN, f"tiny{name}.npz"))
    folder = write_random_model(TINY[name], str(tmp_path / "m"), seed=int(g["seed"]), dtype="float32", std=float(g["std"]))
    cfg, w = plain.read_folder(folder, torch.float64)
    tokens = g["tokens"].tolist()
    assert tokens == random_tokens(int(g["seed"]), len(tokens), cfg["vocab_size"])
    ref = torch.from_numpy(g["logits"])
    # the reference normalises in float32 even in a float64 run (layers/ops.py:31-34): mirror that
    # to compare every other operation at float64 precision
    monkeypatch.setattr(plain, "NORM_DTYPE", torch.float32)
    ours = plain.forward(cfg, w, tokens, torch.float64)
    assert ours.shape == ref.shape
    torch.testing.assert_close(ours, ref, atol=1e-9, rtol=1e-9)
    monkeypatch.setattr(plain, "NORM_DTYPE", None)
    assert (plain.forward(cfg, w, tokens, torch.float64) - ref).abs().max() < 5e-6
    # float32 stays close to float64
    cfg32, w32 = plain.read_folder(folder, torch.float32)
    assert (plain.forward(cfg32, w32, tokens).double() - ref).abs().max() < 2e-5


def test_rms_norm_and_rope_formulas():
    x = torch.tensor([[3.0, 4.0, 0.0, 0.0]])
    y = plain.rms_norm(x, torch.tensor([1.0, 2.0, 1.0, 1.0]), 0.0)
    torch.testing.assert_close(y, torch.tensor([[3 / 2.5, 8 / 2.5, 0.0, 0.0]]))
    cos, sin = plain.rope_tables(4, 100.0, 3, torch.float64)
    assert cos.shape == (3, 4) and torch.allclose(cos[0], torch.ones(4, dtype=torch.float64))
    # position 2, pair (0, 2) rotates by 2 * 100^0 = 2 rad, pair (1, 3) by 2 * 100^-0.5 = 0.2 rad
    v = torch.tensor([[[1.0, 1.0, 0.0, 0.0]]], dtype=torch.float64)
    r = plain.apply_rope(v, cos[2:3], sin[2:3])[0, 0]
    expect = torch.tensor([np.cos(2.0), np.cos(0.2), np.sin(2.0), np.sin(0.2)])
    torch.testing.assert_close(r, expect, atol=1e-6, rtol=1e-6)  # the angles are built in float32


def test_attention_is_causal_grouped_and_windowed():
    torch.manual_seed(0)
    q, k, v = torch.randn(6, 4, 8), torch.randn(6, 2, 8), torch.randn(6, 2, 8)
    o = plain.attention_scores(q, k, v, None)
    torch.testing.assert_close(o[0, 0], v[0, 0])  # the first token sees only itself
    torch.testing.assert_close(o[0, 3], v[0, 1])  # query heads 2, 3 read kv head 1
    k2 = k.clone()
    k2[5] += 10.0  # a later key must not change earlier outputs
    torch.testing.assert_close(plain.attention_scores(q, k2, v, None)[:5], o[:5])
    w1 = plain.attention_scores(q, k, v, 1)
    torch.testing.assert_close(w1[:, 0], v[:, 0])  # window 1: every token sees only itself
    w3 = plain.attention_scores(q, k, v, 3)
    torch.testing.assert_close(w3[:3], o[:3])
    assert not torch.allclose(w3[5], o[5])


def test_window_layers_follow_config():
    cfg = dict(TINY["C"])
    d = plain.derived(cfg)
    assert d["window"] == 20 and d["first_window_layer"] == 2
    folder = write_random_model(cfg, tempfile.mkdtemp(), seed=3, dtype="float32", std=0.1)
    c, w = plain.read_folder(folder)
    tokens = random_tokens(1, 60, 777)
    full = plain.forward(dict(c, use_sliding_window=False), w, tokens)
    win = plain.forward(c, w, tokens)
    torch.testing.assert_close(win[:20], full[:20])  # inside the window nothing changes
    assert (win[40:] - full[40:]).abs().max() > 1e-4


def test_sampling_filters():
    # the reference's own check: each filter maps [.5, .3, .15, .05] to [.625, .375, 0, 0]
    # (tests/test_spec_and_sampling.py:72-79 of 12vivi/tandem)
    logits = torch.log(torch.tensor([0.5, 0.3, 0.15, 0.05]))
    want = torch.tensor([0.625, 0.375, 0.0, 0.0], dtype=torch.float64)
    for kw in (dict(top_k=2), dict(top_p=0.7), dict(min_p=0.5)):
        torch.testing.assert_close(plain.filtered_probs(logits, 1.0, **kw), want, atol=1e-6, rtol=1e-6)
    assert plain.inverse_cdf_draw(want, 0.0) == 0 and plain.inverse_cdf_draw(want, 0.62) == 0
    assert plain.inverse_cdf_draw(want, 0.63) == 1 and plain.inverse_cdf_draw(want, 0.999) == 1
