"""bfloat16 matrix products x [M, K] @ w [N, K]^T with float32 accumulation.

12vivi/tandem runs these through cuBLAS (``torch.nn.functional.linear``,
python/tandem/layers/linear.py:14) except at batch <= 8, where its own weight-streaming
kernels take over (python/tandem/layers/triton_gemv.py:285-297).  The same split is made here:
small M goes to this package's weight-streaming kernel, the rest to the library product.
"""

from __future__ import annotations

import torch

_mm_out_dtype = True  # torch.mm(..., out_dtype=) is tried once


def _library(x: torch.Tensor, weight: torch.Tensor, out_dtype: torch.dtype) -> torch.Tensor:
    global _mm_out_dtype
    if out_dtype == torch.float32 and _mm_out_dtype:
        try:
            return torch.mm(x, weight.t(), out_dtype=torch.float32)
        except (TypeError, RuntimeError):
            _mm_out_dtype = False
    y = torch.mm(x, weight.t())
    return y if y.dtype == out_dtype else y.to(out_dtype)


def linear(x: torch.Tensor, weight: torch.Tensor, out_dtype: torch.dtype) -> torch.Tensor:
    return _library(x, weight, out_dtype)
