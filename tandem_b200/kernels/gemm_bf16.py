"""bfloat16 matrix products x [M, K] @ w [N, K]^T with float32 accumulation.

12vivi/tandem runs these through cuBLAS (``torch.nn.functional.linear``,
python/tandem/layers/linear.py:14) except at small batch, where its own weight-streaming
kernels take over for the shapes on which they beat cuBLAS, by a table measured per shape
(python/tandem/layers/triton_gemv.py:221-297).  The same is done here: up to 64 rows may go to
this package's tcgen05 weight-streaming kernel (``csrc/gemm_skinny.cu``); which of the two is
faster for a shape is measured once, the first time the shape is seen outside a stream capture.
``TANDEM_GEMM=skinny`` or ``=library`` forces one of them.
"""

from __future__ import annotations

import os

import torch

from tandem_b200.kernels import ops
from tandem_b200.kernels.build import load_library

SKINNY_MAX_ROWS = 64
_mm_out_dtype = True  # torch.mm(..., out_dtype=) is tried once
_sm_count: dict = {}
_choice: dict = {}  # (padded rows, N, K, out dtype) -> True: the skinny kernel is the faster one
_flush: dict = {}


def _library(x: torch.Tensor, weight: torch.Tensor, out_dtype: torch.dtype) -> torch.Tensor:
    global _mm_out_dtype
    if out_dtype == torch.float32 and _mm_out_dtype:
        try:
            return torch.mm(x, weight.t(), out_dtype=torch.float32)
        except (TypeError, RuntimeError):
            _mm_out_dtype = False
    y = torch.mm(x, weight.t())
    return y if y.dtype == out_dtype else y.to(out_dtype)


def sm_count(device) -> int:
    key = str(device)
    if key not in _sm_count:
        _sm_count[key] = torch.cuda.get_device_properties(device).multi_processor_count
    return _sm_count[key]


def skinny_scratch(device):
    """Scratch of the skinny kernel, once per device: float32 partials of tiles whose K range is
    shared between blocks, and the tiles' arrival counters (zero between launches)."""
    key = ("scratch", str(device))
    if key not in _sm_count:
        _sm_count[key] = (torch.empty(sm_count(device) * 2 * SKINNY_MAX_ROWS * 128, dtype=torch.float32, device=device),
                          torch.zeros(1 << 16, dtype=torch.int32, device=device))
    return _sm_count[key]


def skinny_applies(M: int, N: int, K: int) -> bool:
    """What the skinny kernel takes at all."""
    return 0 < M <= SKINNY_MAX_ROWS and K % 8 == 0 and N <= (1 << 14) * 128


def skinny(x: torch.Tensor, weight: torch.Tensor, out_dtype: torch.dtype) -> torch.Tensor:
    M, K = x.shape
    N = weight.shape[0]
    y = torch.empty((M, N), dtype=out_dtype, device=x.device)
    partial, counters = skinny_scratch(x.device)
    lib = load_library("gemm_skinny")
    ops._check(lib.tb_gemm_skinny(ops._stream(), ops._ptr(x), ops._ptr(weight), ops._ptr(y), ops._ptr(partial),
                                  ops._ptr(counters), ops._ptr(ops.status_word(x.device)), M, N, K,
                                  int(out_dtype == torch.float32), sm_count(x.device)), "gemm_skinny")
    return y


def _measure(fn, x, weight, out_dtype, flush) -> float:
    """Median device time of fn over a few runs, the weights pushed out of L2 before each."""
    times = []
    for i in range(5):
        flush.zero_()
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        fn(x, weight, out_dtype)
        stop.record()
        stop.synchronize()
        if i:
            times.append(start.elapsed_time(stop))
    return sorted(times)[len(times) // 2]


def skinny_preferred(x: torch.Tensor, weight: torch.Tensor, out_dtype: torch.dtype) -> bool:
    M, K = x.shape
    N = weight.shape[0]
    if not skinny_applies(M, N, K):
        return False
    forced = os.environ.get("TANDEM_GEMM")
    if forced in ("skinny", "library"):
        return forced == "skinny"
    key = (16 if M <= 16 else (32 if M <= 32 else 64), N, K, out_dtype)
    if key not in _choice:
        if torch.cuda.is_current_stream_capturing():
            return M <= 16  # nothing can be timed while a graph is being captured
        dev = str(x.device)
        with torch.inference_mode():
            if dev not in _flush:
                _flush[dev] = torch.empty(192 << 20, dtype=torch.uint8, device=x.device)  # larger than L2
            a = _measure(skinny, x, weight, out_dtype, _flush[dev])
            b = _measure(_library, x, weight, out_dtype, _flush[dev])
        _choice[key] = a <= b
    return _choice[key]


def choices() -> dict:
    """What has been measured so far: (padded rows, N, K, out dtype) -> the skinny kernel won."""
    return dict(_choice)


def linear(x: torch.Tensor, weight: torch.Tensor, out_dtype: torch.dtype) -> torch.Tensor:
    if out_dtype not in (torch.bfloat16, torch.float32):
        raise ops.KernelError(f"the bfloat16 product returns bfloat16 or float32, not {out_dtype}")
    if skinny_preferred(x, weight, out_dtype):
        return skinny(x, weight, out_dtype)
    return _library(x, weight, out_dtype)
