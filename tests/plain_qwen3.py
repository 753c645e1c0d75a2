"""A plain, slow Qwen3-dense forward pass: whole sequences, no cache, one function per part.

Written from the formulas of 12vivi/tandem (each function cites the file and lines it follows)
and compared once with tandem's own model code on the CPU (``tests/golden/make_golden.py``
wrote ``tests/golden/*.npz``; ``tests/test_plain_reference.py`` checks them).  It shares no code
with ``tandem_b200``: it reads ``config.json`` and ``model.safetensors`` itself, through the
checkpoint's own tensor names, and computes in one dtype (float32 or float64) throughout.

The optional sliding window follows the meaning the ``sliding_window`` /
``max_window_layers`` keys have in Qwen config files (layers with index >= max_window_layers
see only the last ``sliding_window`` keys); tandem itself rejects ``use_sliding_window``
(python/tandem/model_config.py:97-98).
"""

from __future__ import annotations

import json
import os

import torch
from safetensors import safe_open


# --------------------------------------------------------------------------- reading
def read_folder(folder: str, dtype: torch.dtype = torch.float32):
    """(config dict, {checkpoint name: tensor cast to ``dtype``})."""
    with open(os.path.join(folder, "config.json"), encoding="utf-8") as f:
        cfg = json.load(f)
    tensors = {}
    for fn in sorted(os.listdir(folder)):
        if fn.endswith(".safetensors"):
            with safe_open(os.path.join(folder, fn), framework="pt", device="cpu") as f:
                for name in f.keys():
                    tensors[name] = f.get_tensor(name).to(dtype)
    return cfg, tensors


def derived(cfg: dict) -> dict:
    """Sizes that config.json may leave out (python/tandem/model_config.py:100-101,125,128-132)."""
    nh = cfg["num_attention_heads"]
    rope = cfg.get("rope_parameters") or {}
    kinds = cfg.get("layer_types")  # newer files name each layer "full_attention" or "sliding_attention"
    if kinds is not None:
        window = cfg.get("sliding_window") if "sliding_attention" in kinds else None
    else:
        window = cfg.get("sliding_window") if cfg.get("use_sliding_window") else None
    return dict(
        L=cfg["num_hidden_layers"],
        H=cfg["hidden_size"],
        nh=nh,
        nkv=cfg.get("num_key_value_heads") or nh,
        hd=cfg.get("head_dim") or cfg["hidden_size"] // nh,
        eps=float(cfg.get("rms_norm_eps", 1e-6)),
        theta=float(rope.get("rope_theta") or cfg.get("rope_theta") or 10000.0),
        tied=bool(cfg.get("tie_word_embeddings", False)),
        window=window,
        first_window_layer=(cfg.get("max_window_layers") or 0) if window else None,
        windowed=[k == "sliding_attention" for k in kinds] if kinds is not None else None,
    )


# --------------------------------------------------------------------------- parts
NORM_DTYPE = None  # set to torch.float32 to normalise in float32 whatever the model dtype, as the reference does


def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """y = weight * x * rsqrt(mean(x^2) + eps) over the last dimension
    (python/tandem/layers/norm.py:15-19; python/tandem/layers/ops.py:29-34).  The reference casts x
    to float32 for the normalisation even when the model runs in float64; with NORM_DTYPE unset
    this function stays in the dtype it is given."""
    xn = x if NORM_DTYPE is None else x.to(NORM_DTYPE)
    xn = xn * torch.rsqrt(xn.pow(2).mean(-1, keepdim=True) + eps)
    return weight * xn.to(x.dtype)


def rope_tables(head_dim: int, theta: float, length: int, dtype: torch.dtype):
    """cos, sin of shape [length, head_dim]: inv_freq[j] = theta^(-2j/hd), angles = pos * inv_freq,
    the half table repeated twice (python/tandem/layers/rotary.py:10-13,41-49).  The angles are
    built in float32 as the reference does, then cast."""
    inv_freq = 1.0 / (theta ** (torch.arange(0, head_dim, 2, dtype=torch.int64).to(torch.float32) / head_dim))
    freqs = torch.outer(torch.arange(length, dtype=torch.float32), inv_freq)
    emb = torch.cat([freqs, freqs], dim=-1)
    return emb.cos().to(dtype), emb.sin().to(dtype)


def apply_rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """x [T, heads, hd] -> x*cos + rotate_half(x)*sin with rotate_half(x) = [-x2, x1]
    (python/tandem/layers/rotary.py:55-64; python/tandem/layers/ops.py:20-22,51-61)."""
    half = x.shape[-1] // 2
    rotated = torch.cat((-x[..., half:], x[..., :half]), dim=-1)
    return x * cos[:, None, :] + rotated * sin[:, None, :]


def attention_scores(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, window) -> torch.Tensor:
    """Causal softmax attention of one whole sequence.  q [T, nh, hd]; k, v [T, nkv, hd].
    Query head h reads kv head h // (nh / nkv); scale hd^-0.5; a query at position p sees keys
    0..p (python/tandem/layers/attention.py:46-56,71; python/tandem/executor/forward_context.py:70-74),
    or only keys p-window+1..p when ``window`` is given."""
    T, nh, hd = q.shape
    groups = nh // k.shape[1]
    k = k.repeat_interleave(groups, dim=1)
    v = v.repeat_interleave(groups, dim=1)
    s = torch.einsum("qhd,khd->hqk", q, k) * hd**-0.5
    pos = torch.arange(T)
    visible = pos[None, :] <= pos[:, None]
    if window is not None:
        visible &= pos[None, :] > pos[:, None] - window
    s = s.masked_fill(~visible[None], float("-inf"))
    p = torch.softmax(s, dim=-1)
    return torch.einsum("hqk,khd->qhd", p, v)


def attention_block(x: torch.Tensor, w: dict, prefix: str, d: dict, cos, sin, window) -> torch.Tensor:
    """q/k/v projections, per-head RMSNorm on q and k before RoPE, attention, output projection
    (python/tandem/layers/attention.py:84,97-106)."""
    T = x.shape[0]
    q = (x @ w[f"{prefix}.q_proj.weight"].T).view(T, d["nh"], d["hd"])
    k = (x @ w[f"{prefix}.k_proj.weight"].T).view(T, d["nkv"], d["hd"])
    v = (x @ w[f"{prefix}.v_proj.weight"].T).view(T, d["nkv"], d["hd"])
    q = rms_norm(q, w[f"{prefix}.q_norm.weight"], d["eps"])
    k = rms_norm(k, w[f"{prefix}.k_norm.weight"], d["eps"])
    q = apply_rope(q, cos, sin)
    k = apply_rope(k, cos, sin)
    o = attention_scores(q, k, v, window)
    return o.reshape(T, d["nh"] * d["hd"]) @ w[f"{prefix}.o_proj.weight"].T


def swiglu(x: torch.Tensor, w: dict, prefix: str) -> torch.Tensor:
    """down(silu(gate(x)) * up(x)), silu(a) = a * sigmoid(a)
    (python/tandem/layers/mlp.py:10-20,41-44; python/tandem/layers/ops.py:45-48)."""
    gate = x @ w[f"{prefix}.gate_proj.weight"].T
    up = x @ w[f"{prefix}.up_proj.weight"].T
    return ((gate * torch.sigmoid(gate)) * up) @ w[f"{prefix}.down_proj.weight"].T


def decoder_layer(h: torch.Tensor, w: dict, i: int, d: dict, cos, sin) -> torch.Tensor:
    """h <- h + attn(norm(h)); h <- h + mlp(norm(h))  (python/tandem/models/llama_family.py:11-16,59-67)."""
    p = f"model.layers.{i}"
    if d["windowed"] is not None:
        window = d["window"] if d["windowed"][i] else None
    else:
        window = d["window"] if d["window"] is not None and i >= d["first_window_layer"] else None
    h = h + attention_block(rms_norm(h, w[f"{p}.input_layernorm.weight"], d["eps"]), w, f"{p}.self_attn", d, cos, sin, window)
    h = h + swiglu(rms_norm(h, w[f"{p}.post_attention_layernorm.weight"], d["eps"]), w, f"{p}.mlp")
    return h


def forward(cfg: dict, w: dict, token_ids, dtype: torch.dtype = torch.float32) -> torch.Tensor:
    """Logits [T, vocab] of one whole sequence (python/tandem/models/llama_family.py:86-116)."""
    d = derived(cfg)
    ids = torch.as_tensor(token_ids, dtype=torch.long)
    cos, sin = rope_tables(d["hd"], d["theta"], len(ids), dtype)
    h = w["model.embed_tokens.weight"][ids]
    for i in range(d["L"]):
        h = decoder_layer(h, w, i, d, cos, sin)
    h = rms_norm(h, w["model.norm.weight"], d["eps"])
    head = w["model.embed_tokens.weight"] if d["tied"] else w["lm_head.weight"]
    return h @ head.T


def greedy(cfg: dict, w: dict, prompt, n: int, dtype: torch.dtype = torch.float32) -> list[int]:
    """n greedy tokens, recomputing the whole sequence each time."""
    ids = list(prompt)
    for _ in range(n):
        ids.append(int(forward(cfg, w, ids, dtype)[-1].argmax()))
    return ids[len(prompt):]


# --------------------------------------------------------------------------- sampling
def filtered_probs(logits: torch.Tensor, temperature: float, top_k: int = -1, top_p: float = 1.0,
                   min_p: float = 0.0) -> torch.Tensor:
    """One row [V] -> probabilities after temperature, top-k, top-p and min-p
    (python/tandem/layers/sampler.py:19-49)."""
    x = logits.double() / max(temperature, 1e-5)
    V = x.shape[-1]
    if 0 < top_k < V:
        kth = x.sort(descending=True).values[top_k - 1]
        x = x.masked_fill(x < kth, float("-inf"))
    p = torch.softmax(x, dim=-1)
    if top_p < 1.0:
        sp, idx = p.sort(descending=True)
        cum = sp.cumsum(-1)
        sp = sp.masked_fill((cum - sp) > top_p, 0.0)
        p = torch.zeros_like(p).scatter_(0, idx, sp)
    if min_p > 0:
        p = p.masked_fill(p < min_p * p.max(), 0.0)
    return p / p.sum()


def inverse_cdf_draw(probs: torch.Tensor, u: float) -> int:
    """The first index whose cumulative probability exceeds u * total, in vocabulary order.
    tandem draws with torch.multinomial (python/tandem/layers/sampler.py:63); the engine draws
    by inverse CDF from one uniform number so that a draw does not depend on the batch."""
    cum = probs.double().cumsum(-1)
    idx = int(torch.searchsorted(cum, torch.tensor(u * float(cum[-1]), dtype=torch.float64), right=True))
    return min(idx, probs.numel() - 1)
