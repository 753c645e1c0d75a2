"""Choice of the paged-attention kernel for a step.

float32 always runs the CUDA-core kernel (true 32-bit arithmetic, batch-invariant bit for bit).
bfloat16 runs the tensor-core kernels where they take the shape and the CUDA-core kernel
otherwise; both read the same cache layout.
"""

from __future__ import annotations

from typing import Optional

import torch

from tandem_b200.kernels import ops


def paged_attention(qkv: torch.Tensor, kv, ctx, num_heads: int, num_kv_heads: int, head_dim: int,
                    window: Optional[int], scale: float) -> torch.Tensor:
    """Attention output [T, nh * hd] for the query heads in the first nh*hd columns of qkv."""
    return ops.paged_attention_simt(qkv, kv.k, kv.v, kv.block_table, ctx.seq_of_token, ctx.positions, num_heads,
                                    num_kv_heads, head_dim, kv.page_size, window, scale)
