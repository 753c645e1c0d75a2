"""bfloat16 matrix products x [M, K] @ w [N, K]^T with float32 accumulation.

12vivi/tandem runs these through cuBLAS (``torch.nn.functional.linear``,
python/tandem/layers/linear.py:14) except at small batch, where its own weight-streaming
kernels take over for the shapes on which they beat cuBLAS, by a table measured per shape
(python/tandem/layers/triton_gemv.py:221-297).  The same is done here: up to 64 rows may go to
this package's tcgen05 weight-streaming kernel (``csrc/gemm_skinny.cu``); which of the two is
faster for a shape is measured once, the first time the shape is seen outside a stream capture.
Up to eight rows may also go to a kernel that streams the weights through registers into ``mma.sync``
(``csrc/gemv_bf16.cu``, no shared-memory ring, no tensor memory, no merge between blocks),
measured against the other two in the same way.  ``TANDEM_GEMM=skinny``, ``=gemv`` or ``=library``
forces one of them where it applies.

A caller whose output goes to a kernel that takes split input (``ops.add_rmsnorm``,
``ops.qk_norm_rope_kv``, ``ops.silu_mul``) may allow a ``SplitOutput``: the skinny kernel then
leaves the partial sums of the tiles that several blocks share to that kernel, which adds them
on its way in (``csrc/split_output.cuh``), and the product ends three trips to the L2 earlier.
Measured on a B200 at Qwen3-8B sizes and 8 rows: the product alone gets 3 to 5 us shorter (o_proj
14.1 -> 8.9 us, down_proj 23.3 -> 18.6 us), the reading kernel 2 to 5 us longer, product plus norm
0.7 to 1.6 us shorter back to back, but a whole decode step came out 2 % slower (1,860 against
1,896 tok/s).  So it is off unless ``TANDEM_SPLIT_OUTPUT=1``; the values are bit for bit the same
either way.
"""

from __future__ import annotations

import os

import torch

from tandem_b200.kernels import ops
from tandem_b200.kernels.build import load_library

SKINNY_MAX_ROWS = 64
GEMV_MAX_ROWS = 8  # tb_gemv_max_rows() of csrc/gemv_bf16.cu
SPLIT_MAX_ROWS = 32  # beyond this the partials are more than a reader should add up
_mm_out_dtype = True  # torch.mm(..., out_dtype=) is tried once
_sm_count: dict = {}
_choice: dict = {}  # (class of rows, N, K, out dtype, split) -> "skinny" | "gemv" | "library", the fastest when measured
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


class SplitOutput:
    """The output [M, N] of a skinny product whose shared tiles are still partial sums in the
    kernel's scratch memory.  It lives until the next skinny product on the device; kernels that
    take split input read it, anything else goes through ``ops.as_tensor``."""

    __slots__ = ("y", "partial", "tiles", "mpad", "serial")

    def __init__(self, y, partial, tiles, mpad, serial) -> None:
        self.y, self.partial, self.tiles, self.mpad, self.serial = y, partial, tiles, mpad, serial

    @property
    def shape(self):
        return self.y.shape

    @property
    def dtype(self):
        return self.y.dtype

    @property
    def device(self):
        return self.y.device

    def check(self) -> None:
        if _serial.get(str(self.y.device)) != self.serial:
            raise ops.KernelError("a split output was read after another skinny product had reused its scratch memory")


_serial: dict = {}  # device -> number of skinny products launched (their scratch is shared)
_tiles: dict = {}


def split_tiles(device, N: int, K: int):
    """int32 [N tiles, 3] on the device: which blocks contribute to each tile of a skinny product of
    this shape (first block, last block, slot of the first one's partial)."""
    key = (str(device), N, K)
    if key not in _tiles:
        host = torch.zeros(3 * -(-N // 128), dtype=torch.int32)
        load_library("gemm_skinny").tb_gemm_skinny_tiles(N, K, sm_count(device), ops._ptr(host))
        _tiles[key] = host.to(device)
    return _tiles[key]


def split_enabled() -> bool:
    return os.environ.get("TANDEM_SPLIT_OUTPUT", "0") == "1"


def skinny_applies(M: int, N: int, K: int) -> bool:
    """What the skinny kernel takes at all."""
    return 0 < M <= SKINNY_MAX_ROWS and K % 8 == 0 and N <= (1 << 14) * 128


def skinny(x: torch.Tensor, weight: torch.Tensor, out_dtype: torch.dtype, split: bool = False):
    """The tcgen05 weight-streaming kernel.  ``split``: return a ``SplitOutput`` (bfloat16 only)."""
    M, K = x.shape
    N = weight.shape[0]
    y = torch.empty((M, N), dtype=out_dtype, device=x.device)
    partial, counters = skinny_scratch(x.device)
    tiles = split_tiles(x.device, N, K) if split else None
    lib = load_library("gemm_skinny")
    ops._check(lib.tb_gemm_skinny(ops._stream(), ops._ptr(x), ops._ptr(weight), ops._ptr(y), ops._ptr(partial),
                                  ops._ptr(counters), ops._ptr(ops.status_word(x.device)), M, N, K,
                                  int(out_dtype == torch.float32), sm_count(x.device), int(split)), "gemm_skinny")
    dev = str(x.device)
    _serial[dev] = _serial.get(dev, 0) + 1
    if not split:
        return y
    return SplitOutput(y, partial, tiles, 16 if M <= 16 else (32 if M <= 32 else 64), _serial[dev])


def wide(x: torch.Tensor, weight: torch.Tensor, out_dtype: torch.dtype, gated: bool = False) -> torch.Tensor:
    """The tcgen05 kernel for many rows (``csrc/gemm_wide.cu``): 128 x 256 output tiles, one
    persistent block per SM.  ``gated``: the weight's rows are [gate | up]; returns
    silu(x gate^T) * (x up^T), [M, rows / 2]."""
    M, K = x.shape
    N = weight.shape[0]
    y = torch.empty((M, N // 2 if gated else N), dtype=out_dtype, device=x.device)
    lib = load_library("gemm_wide")
    ops._check(lib.tb_gemm_wide(ops._stream(), ops._ptr(x), ops._ptr(weight), ops._ptr(y), ops._ptr(ops.status_word(x.device)),
                                M, N, K, int(out_dtype == torch.float32), int(gated), sm_count(x.device)), "gemm_wide")
    return y


def wide_applies(M: int, N: int, K: int) -> bool:
    return M > 0 and K % 8 == 0 and N % 8 == 0


def _measure(fn, x, weight, out_dtype, flush) -> float:
    """Median device time of fn over a few runs, the weights pushed out of L2 before each."""
    times = []
    for i in range(5):
        flush.zero_()
        flush.zero_()  # twice: the device is still busy when the timed launch has been queued, so host time is not measured
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        fn(x, weight, out_dtype)
        stop.record()
        stop.synchronize()
        if i:
            times.append(start.elapsed_time(stop))
    return sorted(times)[len(times) // 2]


def gemv_applies(M: int, N: int, K: int) -> bool:
    """What the register-streaming kernel takes: up to eight rows."""
    return 0 < M <= GEMV_MAX_ROWS and K > 0 and K % 8 == 0


def gemv(x: torch.Tensor, weight: torch.Tensor, out_dtype: torch.dtype, gated: bool = False) -> torch.Tensor:
    """The weight-streaming kernel for up to eight rows (``csrc/gemv_bf16.cu``): weights from global
    memory straight into registers, ``mma.sync`` against the rows of x in shared memory.  ``gated``:
    the weight's rows are [gate | up]; returns silu(x gate^T) * (x up^T), [M, rows / 2], the values
    the product followed by ``ops.silu_mul`` gives."""
    M, K = x.shape
    N = weight.shape[0]
    y = torch.empty((M, N // 2 if gated else N), dtype=out_dtype, device=x.device)
    ops._check(load_library("gemv_bf16").tb_gemv(ops._stream(), ops._ptr(x), ops._ptr(weight), ops._ptr(y), M, N, K,
                                                 int(out_dtype == torch.float32), int(gated), sm_count(x.device)), "gemv")
    return y


def preferred(x: torch.Tensor, weight: torch.Tensor, out_dtype: torch.dtype, split: bool = False) -> str:
    """"skinny", "gemv" or "library": the fastest of those that take the shape, measured once per
    class of shapes (rows up to 1, 2, 4, 8, 16, 32, 64), the weights pushed out of L2 before each run."""
    M, K = x.shape
    N = weight.shape[0]
    can = [name for name, ok in (("skinny", skinny_applies(M, N, K)),
                                 ("gemv", gemv_applies(M, N, K) and not split and x.is_contiguous()
                                  and x.data_ptr() % 16 == 0 and weight.data_ptr() % 16 == 0)) if ok]
    if not can:
        return "library"
    forced = os.environ.get("TANDEM_GEMM")
    if forced in ("skinny", "gemv", "library"):
        return forced if forced == "library" or forced in can else ("skinny" if "skinny" in can else "library")
    # classes of rows as the CUDA graphs' buckets are (1, 2, 4, 8, 16, ...): a batch of 5 is measured when it
    # first runs and decides for the graph of 8 that is captured right after it
    rows = next(c for c in (1, 2, 4, 8, 16, 32, 64) if M <= c)
    key = (rows, N, K, out_dtype, split)
    if key not in _choice:
        if torch.cuda.is_current_stream_capturing():
            # nothing can be timed while a graph is being captured: what usually wins
            return "gemv" if "gemv" in can else ("skinny" if M <= 16 and "skinny" in can else "library")
        dev = str(x.device)
        with torch.inference_mode():
            if dev not in _flush:
                _flush[dev] = torch.empty(192 << 20, dtype=torch.uint8, device=x.device)  # larger than L2
            runs = {"library": _library}
            if "skinny" in can:
                runs["skinny"] = lambda x_, w_, d_: skinny(x_, w_, d_, split)
            if "gemv" in can:
                runs["gemv"] = gemv
            times = {name: _measure(fn, x, weight, out_dtype, _flush[dev]) for name, fn in runs.items()}
        _choice[key] = min(times, key=times.get)
    best = _choice[key]
    return best if best == "library" or best in can else ("skinny" if "skinny" in can else "library")


def _row_bucket(M: int) -> int:
    """Row counts are measured in classes: up to 128, 256, 512, ... (powers of two)."""
    b = 128
    while b < M:
        b *= 2
    return b


def gated(x: torch.Tensor, weight: torch.Tensor) -> torch.Tensor:
    """silu(x gate^T) * (x up^T) for a weight whose rows are [gate | up]: [M, rows / 2] bfloat16.
    Up to eight rows: inside the streaming kernel where that kernel wins the product.  Otherwise few
    rows: the product, then the activation kernel (which takes a split output).  Many rows: the
    wide tcgen05 kernel with the activation in its epilogue, if that was measured to be faster than
    the library product followed by the activation kernel for this class of shapes
    (``TANDEM_GEMM=wide`` or ``=library`` forces one)."""
    M, K = x.shape
    N = weight.shape[0]
    if M <= GEMV_MAX_ROWS and N % 16 == 0 and preferred(x, weight, torch.bfloat16) == "gemv":
        return gemv(x, weight, torch.bfloat16, gated=True)  # the streaming kernel won the product alone: the activation rides along
    if M <= SKINNY_MAX_ROWS or not wide_applies(M, N, K) or N % 16:
        return ops.silu_mul(linear(x, weight, torch.bfloat16, split_ok=True))
    forced = os.environ.get("TANDEM_GEMM")
    if forced in ("wide", "library", "skinny"):
        use_wide = forced == "wide"
    else:
        key = ("gated", _row_bucket(M), N, K)
        if key not in _choice:
            if torch.cuda.is_current_stream_capturing():
                return ops.silu_mul(_library(x, weight, torch.bfloat16))
            dev = str(x.device)
            with torch.inference_mode():
                if dev not in _flush:
                    _flush[dev] = torch.empty(192 << 20, dtype=torch.uint8, device=x.device)
                a = _measure(lambda x_, w_, d_: wide(x_, w_, d_, gated=True), x, weight, torch.bfloat16, _flush[dev])
                b = _measure(lambda x_, w_, d_: ops.silu_mul(_library(x_, w_, d_)), x, weight, torch.bfloat16, _flush[dev])
            _choice[key] = a <= b
        use_wide = _choice[key]
    if use_wide:
        return wide(x, weight, torch.bfloat16, gated=True)
    return ops.silu_mul(_library(x, weight, torch.bfloat16))


def choices() -> dict:
    """What has been measured so far: (class of rows, N, K, out dtype, split) -> the kernel that won."""
    return dict(_choice)


def linear(x: torch.Tensor, weight: torch.Tensor, out_dtype: torch.dtype, split_ok: bool = False):
    """``split_ok``: the caller hands the result to a kernel that takes split input (or through
    ``ops.as_tensor``), so a ``SplitOutput`` may come back instead of a tensor."""
    if out_dtype not in (torch.bfloat16, torch.float32):
        raise ops.KernelError(f"the bfloat16 product returns bfloat16 or float32, not {out_dtype}")
    split = (split_ok and out_dtype == torch.bfloat16 and x.shape[0] <= SPLIT_MAX_ROWS and weight.shape[0] % 8 == 0
             and split_enabled())
    which = preferred(x, weight, out_dtype, split)
    if which == "skinny":
        return skinny(x, weight, out_dtype, split)
    if which == "gemv":
        return gemv(x, weight, out_dtype)
    return _library(x, weight, out_dtype)
