"""Random tiny configurations (head sizes from 16 to 256, any number of heads and groups, widths
and vocabularies that are no power of two, windows, tied or untied heads), random page sizes and
random ways of cutting and mixing the requests: the engine against the plain implementation, in
float32 and in bfloat16.  The seeds are fixed; each builds its own model folder in a temporary place."""

import random

import numpy as np
import pytest
import torch

import plain_qwen3 as plain
import replay_cases as rc

pytestmark = pytest.mark.gpu

HEAD_SIZES = [16, 32, 48, 64, 80, 96, 112, 128, 160, 192, 256]


def random_config(rng: random.Random) -> dict:
    hd = rng.choice(HEAD_SIZES)
    nkv = rng.choice([1, 2, 3, 4])
    groups = rng.choice([1, 2, 3, 4, 5, 6, 7, 8, 16] if hd <= 128 else [1, 2, 4])
    cfg = dict(architectures=["Qwen3ForCausalLM"], model_type="qwen3", num_hidden_layers=rng.randint(1, 3),
               hidden_size=(8 if rng.random() < 0.6 else 2) * rng.randint(8, 40), num_attention_heads=nkv * groups,
               num_key_value_heads=nkv, head_dim=hd, intermediate_size=(8 if rng.random() < 0.6 else 2) * rng.randint(8, 64),
               vocab_size=rng.randint(100, 3000), rope_theta=rng.choice([1e4, 5e5, 1e6]),
               rms_norm_eps=rng.choice([1e-6, 1e-5, 3e-6]), tie_word_embeddings=rng.random() < 0.5,
               max_position_embeddings=512)
    kind = rng.random()
    if kind < 0.3:
        cfg.update(use_sliding_window=True, sliding_window=rng.randint(4, 70),
                   max_window_layers=rng.randint(0, cfg["num_hidden_layers"]))
    elif kind < 0.5:  # the newer spelling: a kind per layer
        cfg.update(sliding_window=rng.randint(4, 70),
                   layer_types=[rng.choice(["full_attention", "sliding_attention"]) for _ in range(cfg["num_hidden_layers"])])
    return cfg


def random_steps(rng: random.Random, requests: dict) -> list:
    regime = rng.choice(["mixed", "mixed", "portions", "tail", "whole"])
    if regime == "mixed":
        return rc.mixed(requests, live=rng.randint(2, 4), portion=rng.randint(2, 40), decode_after=rng.choice([0.3, 0.6, 0.9]))
    if regime == "portions":
        return rc.changing_portions(requests, sizes=tuple(rng.randint(2, 30) for _ in range(9)))
    if regime == "tail":
        return rc.tail_one_by_one(requests, tail=rng.randint(1, 40))
    return rc.whole(requests)


@pytest.mark.parametrize("seed", range(24))
def test_random_configuration(tmp_path, seed):
    from tandem_b200.engine.core import build_executor, load_model
    from tandem_b200.engine.executor import StepEntry
    from tandem_b200.weights.random_init import write_random_model

    rng = random.Random(seed)
    cfg = random_config(rng)
    page_size = rng.choice([1, 2, 4, 8, 16, 32, 48, 64, 128])
    g = torch.Generator().manual_seed(seed)
    requests = {f"r{i}": torch.randint(0, cfg["vocab_size"], (rng.randint(1, 160),), generator=g).tolist()
                for i in range(rng.randint(2, 6))}
    steps = random_steps(rng, requests)
    need = rc.tokens_needed(steps, round_to=max(64, page_size))
    folder = str(tmp_path)
    write_random_model(cfg, folder, seed=seed, dtype="bfloat16", std=0.05)
    c, w64 = plain.read_folder(folder, torch.float64)
    _, w16 = plain.read_folder(folder, torch.bfloat16)
    full = {rid: plain.forward(c, w64, t, torch.float64) for rid, t in requests.items()}
    low = {rid: plain.forward(c, w16, t, torch.bfloat16).double() for rid, t in requests.items()}
    for dtype in ("float32", "bfloat16"):
        decoder, _ = load_model(folder, dtype, "cuda:0")
        ex = build_executor(decoder, page_size=page_size, num_pages=-(-need // page_size), max_requests=8)
        out = {}
        for st in steps:
            logits = ex.step([StepEntry(e["id"], e["tokens"], e["want"]) for e in st["entries"]], end=st["end"])
            if logits.shape[0]:
                out[st["step"]] = logits.cpu().double().numpy()
            ex.manager.check()
        assert ex.manager.all_free()
        per_request = rc.collect(steps, out)
        for rid, ref in full.items():
            got = torch.from_numpy(np.stack(per_request[rid]))
            err = (got - ref).abs().max().item()
            where = int((got - ref).abs().max(-1).values.argmax())
            if dtype == "float32":
                assert err < 1e-4, (cfg, page_size, rid, err, where)
            else:  # the rule of the reference's GPU test (tests/test_gpu_fastpath.py:107-122)
                base = (low[rid] - ref).abs().max().item()
                assert err <= 1.5 * base + 0.02, (cfg, page_size, rid, err, base, where)
