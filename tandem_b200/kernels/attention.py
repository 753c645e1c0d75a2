"""Choice of the paged-attention kernel for a step, and the host-side plans the kernels need.

float32 always runs the CUDA-core kernel (true 32-bit arithmetic, batch-invariant bit for bit).
bfloat16 runs the tensor-core kernels where they take the shape, and the CUDA-core kernel
otherwise; all of them read the same cache layout.

The decode kernel (every request of the step brings one token) works on *items*: a request's
visible keys cut into ranges, so that few long requests still fill the GPU (split-KV, as
12vivi/tandem's python/tandem/layers/triton_decode_attn.py:132-172 does).  ``plan_decode`` cuts
them on the host; the items travel to the device with the batch description.
"""

from __future__ import annotations

import ctypes
from typing import Optional

import torch

from tandem_b200.kernels import ops
from tandem_b200.kernels.build import load_library

ITEM_INTS = 6
STAGE_KEYS = 64  # keys per shared-memory stage of the decode kernel: items are cut at multiples of it
TARGET_BLOCKS = 148 * 2  # one wave at two blocks per SM


def decode_page_size_ok(page_size: int) -> bool:
    return page_size in (1, 2, 4, 8) or page_size % 16 == 0


def fast_decode_applies(dtype: torch.dtype, head_dim: int, page_size: int) -> bool:
    return dtype == torch.bfloat16 and head_dim % 16 == 0 and head_dim <= 256 and decode_page_size_ok(page_size)


def plan_decode(starts, window: Optional[int], num_kv_heads: int, target_blocks: int = TARGET_BLOCKS) -> list:
    """Items [token row, request, key begin, key end, first item of the request, its item count]
    for a step in which request b brings one token at position starts[b]."""
    lo = [max(0, s - window + 1) if window else 0 for s in starts]
    longest = max(s + 1 - l for s, l in zip(starts, lo))
    pieces = max(1, target_blocks // max(1, len(starts) * num_kv_heads))
    split = max(STAGE_KEYS, -(-(-(-longest // pieces)) // STAGE_KEYS) * STAGE_KEYS)
    items = []
    for b, (s, l) in enumerate(zip(starts, lo)):
        first, k = len(items), l
        while k <= s:
            nxt = min(s + 1, (k // split + 1) * split)
            items.append([b, b, k, nxt, first, 0])
            k = nxt
        for it in items[first:]:
            it[5] = len(items) - first
    return items


_workspaces: dict = {}


def _workspace(device, items: int, num_kv_heads: int, groups: int, head_dim: int):
    """Scratch of the decode kernel, kept and grown per device: partial outputs, their (max, sum),
    arrival counters (zero between launches) and the status word."""
    key = str(device)
    rows = items * num_kv_heads * groups
    ws = _workspaces.get(key)
    if ws is None or ws["rows"] < rows or ws["hd"] < head_dim:
        rows = max(rows, ws["rows"] if ws else 0)
        hd = max(head_dim, ws["hd"] if ws else 0)
        ws = dict(rows=rows, hd=hd,
                  part_o=torch.empty(rows * hd, dtype=torch.float32, device=device),
                  part_ml=torch.empty(rows * 2, dtype=torch.float32, device=device),
                  counters=torch.zeros(rows + 64, dtype=torch.int32, device=device))
        _workspaces[key] = ws
    return ws


def paged_attention_decode(qkv: torch.Tensor, kv, items: torch.Tensor, count: torch.Tensor, num_heads: int,
                           num_kv_heads: int, head_dim: int, scale: float) -> torch.Tensor:
    """One token per request: ``items`` int32 [capacity * 6] and ``count`` int32 [1] (how many of
    them are real) as ``plan_decode`` cut them."""
    T = qkv.shape[0]
    capacity = items.numel() // ITEM_INTS
    groups = num_heads // num_kv_heads
    out = torch.empty((T, num_heads * head_dim), dtype=qkv.dtype, device=qkv.device)
    ws = _workspace(qkv.device, capacity, num_kv_heads, groups, head_dim)
    lib = load_library("attention_decode", (f"TB_HD={head_dim}",))
    ops._check(lib.tb_attention_decode(
        ops._stream(), ops._ptr(qkv), qkv.stride(0), ops._ptr(kv.k), ops._ptr(kv.v), ops._ptr(kv.block_table),
        kv.block_table.stride(0), ops._ptr(items), ops._ptr(count), capacity, ops._ptr(out), ops._ptr(ws["part_o"]),
        ops._ptr(ws["part_ml"]), ops._ptr(ws["counters"]), ops._ptr(ops.status_word(qkv.device)), num_heads,
        num_kv_heads, kv.page_size, ctypes.c_float(scale)), "attention_decode")
    return out


def paged_attention(qkv: torch.Tensor, kv, ctx, num_heads: int, num_kv_heads: int, head_dim: int,
                    window: Optional[int], scale: float) -> torch.Tensor:
    """Attention output [T, nh * hd] for the query heads in the first nh*hd columns of qkv."""
    key = ("decode", window, num_kv_heads)
    if key in ctx.extras:
        return paged_attention_decode(qkv, kv, ctx.extras[key], ctx.extras[key + ("count",)], num_heads, num_kv_heads,
                                      head_dim, scale)
    return ops.paged_attention_simt(qkv, kv.k, kv.v, kv.block_table, ctx.seq_of_token, ctx.positions, num_heads,
                                    num_kv_heads, head_dim, kv.page_size, window, scale)
