"""Qwen3 dense: configuration -> model plan, and its random-weight recipe.

The plan spells out what python/tandem/models/llama_family.py:35-116 builds for the qwen3
family: every layer a pre-norm block of GQA attention (per-head q/k RMSNorm, rotary positions,
python/tandem/layers/attention.py:59-106) and a SwiGLU feed-forward
(python/tandem/layers/mlp.py:23-44), a final RMSNorm and a tied or untied output head.
Checkpoint tensor names are the Hugging Face ones that python/tandem/models/loader.py:22-26
fuses into ``qkv_proj`` and ``gate_up_proj``.
"""

from __future__ import annotations

from typing import Iterator

import torch

from tandem_b200.config.model_config import Qwen3Config
from tandem_b200.config.plan import (
    AttentionSpec,
    EmbeddingSpec,
    GatedMLPSpec,
    HeadSpec,
    LayerSpec,
    ModelPlan,
    NormSpec,
    PositionSpec,
    RunStep,
)
from tandem_b200.registry import Architecture, register_architecture


def build_plan(cfg: Qwen3Config) -> ModelPlan:
    position = PositionSpec("rope", rotary_dim=cfg.head_dim, theta=cfg.rope_theta,
                            max_position=cfg.max_position_embeddings)
    layers = []
    for i in range(cfg.num_hidden_layers):
        p = f"model.layers.{i}"
        layers.append(LayerSpec.of(
            "prenorm",
            mixer=AttentionSpec(
                "attention", prefix=f"{p}.self_attn", hidden_size=cfg.hidden_size,
                num_heads=cfg.num_attention_heads, num_kv_heads=cfg.num_key_value_heads,
                head_dim=cfg.head_dim, scale=cfg.head_dim ** -0.5,  # attention.py:71
                qk_norm=True, qk_norm_eps=cfg.rms_norm_eps, window=cfg.layer_window(i), position=position,
            ),
            feed_forward=GatedMLPSpec("gated_mlp", prefix=f"{p}.mlp", hidden_size=cfg.hidden_size,
                                      intermediate_size=cfg.intermediate_size, activation="silu"),
            mixer_norm=NormSpec("rmsnorm", cfg.hidden_size, cfg.rms_norm_eps, f"{p}.input_layernorm.weight"),
            feed_forward_norm=NormSpec("rmsnorm", cfg.hidden_size, cfg.rms_norm_eps,
                                       f"{p}.post_attention_layernorm.weight"),
        ))
    return ModelPlan(
        embedding=EmbeddingSpec(cfg.vocab_size, cfg.hidden_size, "model.embed_tokens.weight"),
        layers=tuple(layers),
        order=tuple(RunStep(i) for i in range(cfg.num_hidden_layers)),
        final_norm=NormSpec("rmsnorm", cfg.hidden_size, cfg.rms_norm_eps, "model.norm.weight"),
        head=HeadSpec(cfg.vocab_size, cfg.hidden_size, None if cfg.tie_word_embeddings else "lm_head.weight"),
        max_position=cfg.max_position_embeddings,
        # loader.py:16 ignores these; a tied checkpoint may still carry lm_head (loader.py:94-97)
        ignored_weights=(r"rotary_emb\.inv_freq$", r"\.attn\.bias$", r"\.masked_bias$")
        + ((r"^lm_head\.weight$",) if cfg.tie_word_embeddings else ()),
        eos_token_ids=tuple(cfg.eos_token_ids),
    )


def tensor_shapes(cfg: Qwen3Config) -> dict[str, tuple]:
    """Checkpoint tensor name -> shape, in file order."""
    H, I, q, kv = cfg.hidden_size, cfg.intermediate_size, cfg.q_size, cfg.kv_size
    shapes: dict[str, tuple] = {"model.embed_tokens.weight": (cfg.vocab_size, H)}
    for i in range(cfg.num_hidden_layers):
        p = f"model.layers.{i}"
        shapes[f"{p}.input_layernorm.weight"] = (H,)
        shapes[f"{p}.self_attn.q_proj.weight"] = (q, H)
        shapes[f"{p}.self_attn.k_proj.weight"] = (kv, H)
        shapes[f"{p}.self_attn.v_proj.weight"] = (kv, H)
        shapes[f"{p}.self_attn.q_norm.weight"] = (cfg.head_dim,)
        shapes[f"{p}.self_attn.k_norm.weight"] = (cfg.head_dim,)
        shapes[f"{p}.self_attn.o_proj.weight"] = (H, q)
        shapes[f"{p}.post_attention_layernorm.weight"] = (H,)
        shapes[f"{p}.mlp.gate_proj.weight"] = (I, H)
        shapes[f"{p}.mlp.up_proj.weight"] = (I, H)
        shapes[f"{p}.mlp.down_proj.weight"] = (H, I)
    shapes["model.norm.weight"] = (H,)
    if not cfg.tie_word_embeddings:
        shapes["lm_head.weight"] = (cfg.vocab_size, H)
    return shapes


def random_weights(cfg: Qwen3Config, seed: int, device: str = "cpu", dtype: torch.dtype = torch.bfloat16,
                   std: float = 0.02, norm_spread: float = 0.1) -> Iterator[tuple[str, torch.Tensor]]:
    """Seeded random tensors by checkpoint name: matrices and the embedding N(0, std), norm
    weights 1 + U(-norm_spread, norm_spread).  Each tensor has a generator of its own, seeded by
    (seed, position in the file), so one tensor does not depend on the sizes of the others."""
    for index, (name, shape) in enumerate(tensor_shapes(cfg).items()):
        g = torch.Generator(device=device).manual_seed((seed * 1_000_003 + index) % (2**63 - 1))
        if len(shape) == 1:
            t = 1.0 + norm_spread * (2.0 * torch.rand(shape, generator=g, device=device, dtype=torch.float32) - 1.0)
        else:
            t = torch.empty(shape, device=device, dtype=torch.float32).normal_(0.0, std, generator=g)
        yield name, t.to(dtype)


register_architecture(
    Architecture("Qwen3ForCausalLM", Qwen3Config, build_plan, random_weights),
    model_types=("qwen3",),
)
