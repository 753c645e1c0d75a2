"""bfloat16 matrix products x [M, K] @ w [N, K]^T with float32 accumulation.

12vivi/tandem runs these through cuBLAS (``torch.nn.functional.linear``,
python/tandem/layers/linear.py:14) except at batch <= 8, where its own weight-streaming
kernels take over (python/tandem/layers/triton_gemv.py:285-297).  The same split is made here,
further up: up to 64 rows go to this package's tcgen05 weight-streaming kernel
(``csrc/gemm_skinny.cu``), more rows to the library product.
"""

from __future__ import annotations

import torch

from tandem_b200.kernels import ops
from tandem_b200.kernels.build import load_library

SKINNY_MAX_ROWS = 64
_mm_out_dtype = True  # torch.mm(..., out_dtype=) is tried once
_scratch: dict = {}


def _library(x: torch.Tensor, weight: torch.Tensor, out_dtype: torch.dtype) -> torch.Tensor:
    global _mm_out_dtype
    if out_dtype == torch.float32 and _mm_out_dtype:
        try:
            return torch.mm(x, weight.t(), out_dtype=torch.float32)
        except (TypeError, RuntimeError):
            _mm_out_dtype = False
    y = torch.mm(x, weight.t())
    return y if y.dtype == out_dtype else y.to(out_dtype)


def skinny_scratch(device):
    """Scratch of the skinny kernel, once per device: float32 partials of tiles whose K range is
    shared between blocks, the tiles' arrival counters (zero between launches), the block count."""
    key = str(device)
    if key not in _scratch:
        blocks = torch.cuda.get_device_properties(device).multi_processor_count
        _scratch[key] = (torch.empty(blocks * 2 * SKINNY_MAX_ROWS * 128, dtype=torch.float32, device=device),
                         torch.zeros(1 << 16, dtype=torch.int32, device=device), blocks)
    return _scratch[key]


def skinny_applies(M: int, N: int, K: int) -> bool:
    """What the skinny kernel takes at all."""
    return 0 < M <= SKINNY_MAX_ROWS and K % 8 == 0 and N <= (1 << 14) * 128


def skinny_preferred(M: int, N: int, K: int) -> bool:
    """Where the skinny kernel is the faster one on a B200 (measured per shape inside CUDA graphs,
    weights rotated through more than L2): up to 16 rows always; up to 64 rows for very tall
    weights (the output head), where its stream-K split keeps every SM streaming to the end.
    12vivi/tandem keeps such a table per shape as well (python/tandem/layers/triton_gemv.py:221-267)."""
    return skinny_applies(M, N, K) and (M <= 16 or N >= 65536)


def skinny(x: torch.Tensor, weight: torch.Tensor, out_dtype: torch.dtype) -> torch.Tensor:
    M, K = x.shape
    N = weight.shape[0]
    y = torch.empty((M, N), dtype=out_dtype, device=x.device)
    partial, counters, blocks = skinny_scratch(x.device)
    lib = load_library("gemm_skinny")
    ops._check(lib.tb_gemm_skinny(ops._stream(), ops._ptr(x), ops._ptr(weight), ops._ptr(y), ops._ptr(partial),
                                  ops._ptr(counters), ops._ptr(ops.status_word(x.device)), M, N, K,
                                  int(out_dtype == torch.float32), blocks), "gemm_skinny")
    return y


def linear(x: torch.Tensor, weight: torch.Tensor, out_dtype: torch.dtype) -> torch.Tensor:
    if out_dtype not in (torch.bfloat16, torch.float32):
        raise ops.KernelError(f"the bfloat16 product returns bfloat16 or float32, not {out_dtype}")
    if skinny_preferred(x.shape[0], weight.shape[0], x.shape[1]):
        return skinny(x, weight, out_dtype)
    return _library(x, weight, out_dtype)
