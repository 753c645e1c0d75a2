"""Writes tests/golden/tiny{A,B}.npz: logits of 12vivi/tandem's own model code on tiny random models.

Run once on the CPU, with $TANDEM_REFERENCE naming a checkout of 12vivi/tandem:

    TANDEM_REFERENCE=<checkout> python tests/golden/make_golden.py

For each tiny configuration it writes a random-weights folder (seeded, so the test can write
the same folder again), loads it with the reference's own config parser, model builder and
weight loader, runs one whole prompt through ``model(...)`` + ``compute_logits`` in float64 the
way the reference's tests/test_model_equivalence.py:17-28 does, and stores the token ids and
the logits.  tests/test_plain_reference.py compares the plain implementation with these files.
"""

import os
import sys
import tempfile

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
sys.path.insert(0, os.path.dirname(HERE))
sys.path.insert(0, os.path.join(os.environ["TANDEM_REFERENCE"], "python"))

from conftest import TINY, random_tokens  # noqa: E402
from tandem_b200.weights.random_init import write_random_model  # noqa: E402

GOLDEN = {"A": dict(seed=101, std=0.1, tokens=33), "B": dict(seed=202, std=0.1, tokens=70)}


def main() -> None:
    from tandem.executor.forward_context import ForwardContext, build_attention_metadata
    from tandem.cache.kv_cache import KVCache
    from tandem.layers.attention import TorchAttentionBackend
    from tandem.model_config import ModelConfig
    from tandem.models import build_model
    from tandem.models.loader import cast_parameters, load_weights

    for name, g in GOLDEN.items():
        folder = write_random_model(TINY[name], tempfile.mkdtemp(), seed=g["seed"], dtype="float32", std=g["std"])
        mc = ModelConfig.from_pretrained(folder)
        model = build_model(mc, mc.max_position_embeddings)
        cast_parameters(model, torch.float64)
        load_weights(model, folder)
        model.eval()
        tokens = random_tokens(g["seed"], g["tokens"], mc.vocab_size)
        bs = 4
        blocks = list(range(-(-len(tokens) // bs)))
        kv = KVCache(mc.num_hidden_layers, len(blocks) + 1, bs, mc.num_key_value_heads, mc.head_dim, torch.float64,
                     torch.device("cpu"))
        positions, meta = build_attention_metadata([(blocks, 0, len(tokens))], bs, torch.device("cpu"))
        ctx = ForwardContext(meta, kv, TorchAttentionBackend(), None)
        with torch.inference_mode():
            logits = model.compute_logits(model(torch.tensor(tokens), positions, ctx))
        np.savez_compressed(os.path.join(HERE, f"tiny{name}.npz"), tokens=np.array(tokens, dtype=np.int64),
                            logits=logits.double().numpy(), seed=g["seed"], std=g["std"])
        print(name, tuple(logits.shape), float(logits.abs().max()))


if __name__ == "__main__":
    main()
