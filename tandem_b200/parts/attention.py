"""Grouped-query attention over the paged cache.

One fused projection (rows [q | k | v], python/tandem/layers/attention.py:69-74 of
12vivi/tandem), optional per-head RMSNorm of q and k before the rotary encoding
(attention.py:75-78,101-104), keys and values written to the token's slot before the scores are
taken, so a portion attends to itself through the cache (attention.py:43-48), causal softmax
attention with scale and an optional window, then the output projection (attention.py:106).
Every size is a parameter of the spec; the mixer does not know which model it serves.
"""

from __future__ import annotations

import torch

from tandem_b200.cache.manager import KVNeed
from tandem_b200.config.plan import AttentionSpec, ParamSpec, WeightSource
from tandem_b200.kernels import attention as attention_kernels
from tandem_b200.kernels import ops
from tandem_b200.parts.base import Mixer, StepContext
from tandem_b200.parts.shared import position_encoding


class PagedAttention(Mixer):
    capturable = True  # forward only launches kernels: decode steps may be captured in CUDA graphs
    capturable_portions = True  # and so may steps in which requests bring several tokens (it reads the batch from device arrays only)
    takes_deferred = True  # x may be a norm whose scale is pending; with ``defer`` the output projection may stay pending

    @staticmethod
    def params(spec: AttentionSpec) -> dict:
        q, kv, H, p = spec.num_heads * spec.head_dim, spec.num_kv_heads * spec.head_dim, spec.hidden_size, spec.prefix
        out = {
            "qkv": ParamSpec((q + 2 * kv, H), (WeightSource(f"{p}.q_proj.weight", 0, q),
                                               WeightSource(f"{p}.k_proj.weight", q, kv),
                                               WeightSource(f"{p}.v_proj.weight", q + kv, kv))),
            "o": ParamSpec((H, q), (WeightSource(f"{p}.o_proj.weight"),)),
        }
        if spec.qk_norm:
            out["q_norm"] = ParamSpec((spec.head_dim,), (WeightSource(f"{p}.q_norm.weight"),), role="vector")
            out["k_norm"] = ParamSpec((spec.head_dim,), (WeightSource(f"{p}.k_norm.weight"),), role="vector")
        return out

    @staticmethod
    def kv_need(spec: AttentionSpec) -> KVNeed:
        return KVNeed(spec.num_kv_heads, spec.head_dim, spec.window)

    def __init__(self, spec: AttentionSpec, weights: dict, dtype: torch.dtype, device) -> None:
        if spec.num_heads % spec.num_kv_heads:
            raise ValueError(f"{spec.num_heads} query heads cannot share {spec.num_kv_heads} kv heads")
        self.spec = spec
        self.qkv = weights["qkv"]
        self.o = weights["o"]
        self.q_norm = weights.get("q_norm")
        self.k_norm = weights.get("k_norm")
        self.position = position_encoding(spec.position, device)

    def step_arrays(self, ctx: StepContext, out: dict) -> None:
        """Cut the step's attention work on the host: items for requests that bring one token
        (split-KV decode kernel), tiles for those that bring more (prefill kernel)."""
        s = self.spec
        attention_kernels.plan_step(ctx, s.window, s.num_heads, s.num_kv_heads, s.head_dim, out)

    def step_array_capacity(self, bucket: int, max_model_len: int, page_size: int, out: dict) -> None:
        """The most entries ``step_arrays`` can produce for a step of up to ``bucket`` single tokens
        (CUDA graphs keep the arrays in static memory); also sizes the decode kernel's scratch."""
        s = self.spec
        key = attention_kernels.plan_key(s.window, s.num_heads, s.num_kv_heads, s.head_dim, self.qkv.dtype)
        groups = s.num_heads // s.num_kv_heads
        if key + ("items",) in out or \
                not attention_kernels.tensor_core_path_applies(self.qkv.dtype, s.head_dim, page_size, groups):
            return
        items = attention_kernels.decode_items_capacity(bucket, s.num_kv_heads, max_model_len)
        out[key + ("items",)] = items * attention_kernels.ITEM_INTS
        out[key + ("count",)] = 1
        out[key + ("tiles",)] = 0
        attention_kernels._workspace(self.qkv.device, items, s.num_kv_heads, groups, s.head_dim)

    def mixed_step_array_capacity(self, tokens: int, seqs: int, max_model_len: int, page_size: int, out: dict) -> None:
        """The same for steps of up to ``tokens`` tokens of up to ``seqs`` requests, prompt portions among
        them (``ctx.static_layout``): decode items for the requests that bring one token, and the prefill
        kernel's queues at their full length.  Leaves ``out`` alone where such steps cannot be captured."""
        s = self.spec
        key = attention_kernels.plan_key(s.window, s.num_heads, s.num_kv_heads, s.head_dim, self.qkv.dtype)
        groups = s.num_heads // s.num_kv_heads
        if key + ("items",) in out or \
                not attention_kernels.tensor_core_path_applies(self.qkv.dtype, s.head_dim, page_size, groups) or \
                not attention_kernels.tcgen05_prefill_applies(s.head_dim, page_size):
            return
        from tandem_b200.kernels.gemm_bf16 import sm_count

        blocks = sm_count(self.qkv.device)
        items = attention_kernels.decode_items_capacity(seqs, s.num_kv_heads, max_model_len)
        out[key + ("items",)] = items * attention_kernels.ITEM_INTS
        out[key + ("count",)] = 1
        out[key + ("tiles",)] = (attention_kernels.prefill_queue_capacity(tokens, seqs, groups, s.num_kv_heads, blocks)
                                 * blocks * attention_kernels.WORK_INTS)
        attention_kernels._workspace(self.qkv.device, items, s.num_kv_heads, groups, s.head_dim)

    def forward(self, x, ctx: StepContext, defer: bool = False):
        s = self.spec
        qkv = ops.linear(x, self.qkv)
        kv = ctx.kv(self)
        fresh = None
        if attention_kernels.decodes_only(ctx, s.num_heads, s.num_kv_heads, s.head_dim, s.window, qkv.dtype) and \
                attention_kernels.fresh_applies(s.head_dim, self.position.rotary_dim, kv.writable, qkv.shape[0],
                                                ops.linear_streams(qkv.shape[0], self.qkv)):
            # single tokens only: decode attention normalises, rotates and stores what it needs itself
            fresh = dict(positions=ctx.positions, slots=kv.slots, q_norm=self.q_norm, k_norm=self.k_norm,
                         cos_sin=self.position.cos_sin, eps=s.qk_norm_eps)
        else:
            qkv = ops.qk_norm_rope_kv(qkv, ctx.positions, kv.slots, self.q_norm, self.k_norm, self.position.cos_sin,
                                      kv.k, kv.v, s.num_heads, s.num_kv_heads, s.head_dim, self.position.rotary_dim,
                                      kv.page_size, s.qk_norm_eps, write_kv=kv.writable)
        o = attention_kernels.paged_attention(qkv, kv, ctx, s.num_heads, s.num_kv_heads, s.head_dim, s.window, s.scale, fresh)
        return ops.linear(o, self.o, defer=defer)
