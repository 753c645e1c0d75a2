"""Values that a kernel has still to produce, so that the kernel which needs them can make them itself.

Between two matrix products of a decoder layer stand a residual add and an RMSNorm.  At up to
eight rows each of them is a launch on the critical path that costs about 3 us for a few hundred
nanoseconds of arithmetic.  RMSNorm scales a row by one number, and a product is linear in its
rows, so the streaming product (``csrc/gemv_bf16.cu``) can take both along without any block
reading a row twice: the product in front adds its result into the residual, writes the residual
times the norm's weight beside it and leaves partial sums of squares; the product behind reads
those rows and multiplies row m of its result by rsqrt(mean square + eps).  For that the value
that travels between the parts of a layer must be allowed to be *not computed yet*:

``PendingLinear``  a product x @ W^T that has not been launched: what a mixer or a feed-forward
                   returns when its arrangement asks for it (``forward(..., defer=True)``).
``PendingNorm``    RMSNorm(residual) * weight of which the rows' scale has been left out: what the
                   norm returns, after it has had the pending product added into the residual by the
                   product's own kernel, when the part behind it takes such input.

Only parts that say ``takes_deferred = True`` ever meet one of these; everything else gets tensors
(``tensor`` computes what is pending with the stand-alone kernels).  12vivi/tandem fuses the same
pair into its small-batch product (python/tandem/layers/triton_gemv.py:92-145,356-378).
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Optional

import torch


@dataclass
class PendingLinear:
    x: torch.Tensor  # [M, K]
    weight: torch.Tensor  # [N, K]

    @property
    def shape(self) -> tuple:
        return (self.x.shape[0], self.weight.shape[0])


@dataclass
class PendingNorm:
    residual: torch.Tensor  # [M, H] float32, everything added
    weight: torch.Tensor  # [H] float32
    eps: float
    out_dtype: torch.dtype
    scaled: torch.Tensor  # [M, H] bfloat16(residual * weight): the normalised rows but for their scale
    partials: torch.Tensor  # [parts, 8 or 16] float32 (gemm_bf16.gemv_partial_rows of M): sums of squares of the rows, per block of the kernel that wrote them
    parts: int

    @property
    def shape(self) -> tuple:
        return tuple(self.residual.shape)


def is_pending(v: Any) -> bool:
    return isinstance(v, (PendingLinear, PendingNorm))


def tensor(v: Any) -> Optional[torch.Tensor]:
    """What ``v`` stands for, computed now by the stand-alone kernels; tensors and None pass through."""
    if v is None or isinstance(v, torch.Tensor):
        return v
    from tandem_b200.kernels import ops

    if isinstance(v, PendingLinear):
        return ops.linear(v.x, v.weight)
    if isinstance(v, PendingNorm):
        return ops.add_rmsnorm(None, v.residual, v.weight, v.eps, v.out_dtype)
    raise TypeError(f"{type(v).__name__} stands for no tensor")
