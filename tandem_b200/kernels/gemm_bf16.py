"""bfloat16 matrix products x [M, K] @ w [N, K]^T with float32 accumulation.

12vivi/tandem runs these through cuBLAS (``torch.nn.functional.linear``,
python/tandem/layers/linear.py:14) except at small batch, where its own weight-streaming
kernels take over for the shapes on which they beat cuBLAS, by a table kept per GPU and shape
(python/tandem/layers/triton_gemv.py:221-297).  The same is done here, with three kernels of
this package beside the library:

* up to 8 rows, and up to 16 where the rows of x fit into shared memory: ``csrc/gemv_bf16.cu``
  streams the weights through registers into ``mma.sync`` (no shared-memory ring, no tensor
  memory, no merge between blocks);
* up to 64 rows: ``csrc/gemm_skinny.cu``, the tcgen05 weight-streaming kernel, where the weight
  matrix is large enough to pay for its fixed cost; the library otherwise;
* more rows: the library, except for the gate/up projection, whose activation runs in the
  epilogue of ``csrc/gemm_wide.cu``.

Which kernel computes a shape is fixed (``choose``, ``choose_gated``): a table of shapes that were
measured on a B200 (``MEASURED``), and a rule for all others.  The same shape always runs the same
kernel, so bfloat16 results are reproducible from run to run and a CUDA graph captures what an
eager step runs.  ``python -m tandem_b200.kernels.microbench dispatch`` times every candidate and
prints the table's lines and what the rule would have picked.
``TANDEM_GEMM=skinny``, ``=gemv``, ``=wide``, ``=pair`` or ``=library`` forces one kernel where it applies.
"""

from __future__ import annotations

import ctypes
from typing import Optional

import torch

from tandem_b200.kernels import ops
from tandem_b200.kernels.build import load_library

SKINNY_MAX_ROWS = 64
GEMV_MAX_ROWS = 16  # tb_gemv_max_rows() of csrc/gemv_bf16.cu
GEMV_ROWS_ANY_K = 8  # up to so many rows x may stay in global memory; more must fit into shared memory
GEMV_SMEM_BYTES_TWO_TILES = 130 * 1024  # tb_gemv_max_smem_bytes_two_tiles()
GEMV_MAX_K = 16384  # beyond this the streaming kernel's rows of x outgrow shared memory and it falls behind (measured at K = 25600)
# The skinny kernel costs about 9 us whatever the shape; the library's small-batch kernels cost less
# to start and stream a little more slowly.  The skinny kernel wins from this many weight bytes on
# (per class of rows; measured: it takes the output head at every class, gate_up of Qwen3-32B up to 16 rows).
SKINNY_MIN_WEIGHT_BYTES = {1: 200 << 20, 2: 200 << 20, 4: 400 << 20, 8: 400 << 20, 16: 400 << 20, 32: 1 << 30, 64: 1 << 30}
# gate/up with the activation in the epilogue of a tcgen05 kernel.  From 192 rows on the kernel of
# block pairs (256-row tiles) is the fastest by 2 to 10 % (measured at the gate_up sizes of
# Qwen3-8B, -14B and -32B, 192 to 8,192 rows) unless its last tile of 256 rows is less than half
# full and the rows are few (384 rows: 75 against 67 us).  Else the single-block kernel where one
# wave of its 128-row tiles is full (64 to 128 rows) or the waves are many (from 1536 rows); in
# between the library's tilings followed by the activation kernel are 5 to 10 % faster.
WIDE_GATED_ROWS = ((64, 128), (1536, None))
# Below that the single-block kernel is a weight stream with the activation thrown in (one tile of 128 rows,
# mostly empty): it beats the library's product followed by the activation kernel where the weights are
# large (Qwen3-14B gate_up, 340 MiB: 60 against 62 to 67 us at 16 to 64 rows; Qwen3-32B, 500 MiB: 86 to 88
# against 93 to 97) and loses where they are small (Qwen3-8B, 192 MiB: 39 against 36 to 38 us up to 56 rows).
WIDE_GATED_FEW_ROWS_MIN_WEIGHT_BYTES = 300 << 20
PAIR_GATED_MIN_ROWS = 192
PAIR_MAX_PADDING = 1.08  # rows the pair kernel computes (whole tiles of 256) over those the single-block kernel does (of 128)
_mm_out_dtype = True  # torch.mm(..., out_dtype=) is tried once
_sm_count: dict = {}


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
    key = ops.device_key(device)
    if key not in _sm_count:
        _sm_count[key] = torch.cuda.get_device_properties(device).multi_processor_count
    return _sm_count[key]


def skinny_scratch(device):
    """Scratch of the skinny kernel, once per device: float32 partials of tiles whose K range is
    shared between blocks, and the tiles' arrival counters (zero between launches)."""
    key = ("scratch", ops.device_key(device))
    if key not in _sm_count:
        _sm_count[key] = (torch.empty(sm_count(device) * 2 * SKINNY_MAX_ROWS * 128, dtype=torch.float32, device=device),
                          torch.zeros(1 << 16, dtype=torch.int32, device=device))
    return _sm_count[key]


def skinny_applies(M: int, N: int, K: int) -> bool:
    """What the skinny kernel takes at all."""
    return 0 < M <= SKINNY_MAX_ROWS and K % 8 == 0 and N <= (1 << 14) * 128


def skinny(x: torch.Tensor, weight: torch.Tensor, out_dtype: torch.dtype) -> torch.Tensor:
    """The tcgen05 weight-streaming kernel (``csrc/gemm_skinny.cu``)."""
    M, K = x.shape
    N = weight.shape[0]
    y = torch.empty((M, N), dtype=out_dtype, device=x.device)
    partial, counters = skinny_scratch(x.device)
    lib = load_library("gemm_skinny")
    ops._check(lib.tb_gemm_skinny(ops._stream(), ops._ptr(x), ops._ptr(weight), ops._ptr(y), ops._ptr(partial),
                                  ops._ptr(counters), ops._ptr(ops.status_word(x.device)), M, N, K,
                                  int(out_dtype == torch.float32), sm_count(x.device)), "gemm_skinny")
    return y


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


def wide_pair(x: torch.Tensor, weight: torch.Tensor, out_dtype: torch.dtype, gated: bool = False) -> torch.Tensor:
    """The tcgen05 kernel for many rows by pairs of blocks (``csrc/gemm_wide_pair.cu``, cta_group::2):
    256 x 256 output tiles per pair, each block bringing its 128 rows of x and its half of the
    tile's weight rows.  ``gated`` as for ``wide``."""
    M, K = x.shape
    N = weight.shape[0]
    y = torch.empty((M, N // 2 if gated else N), dtype=out_dtype, device=x.device)
    lib = load_library("gemm_wide_pair")
    ops._check(lib.tb_gemm_wide_pair(ops._stream(), ops._ptr(x), ops._ptr(weight), ops._ptr(y), ops._ptr(ops.status_word(x.device)),
                                     M, N, K, int(out_dtype == torch.float32), int(gated), sm_count(x.device)), "gemm_wide_pair")
    return y


def wide_applies(M: int, N: int, K: int) -> bool:
    return M > 0 and K % 8 == 0 and N % 8 == 0


def gemv_applies(M: int, N: int, K: int) -> bool:
    """What the register-streaming kernel takes (tb_gemv_takes of csrc/gemv_bf16.cu): up to eight
    rows, or up to sixteen whose padded copy fits into 130 KB of shared memory beside the block's
    partial tiles (14 rows of 4,096, 11 of 5,120)."""
    if not (0 < M <= GEMV_MAX_ROWS and K > 0 and K % 8 == 0):
        return False
    if M <= GEMV_ROWS_ANY_K:
        return True
    pieces = K // 8
    stride = pieces + (4 - pieces % 8 + 8) % 8
    return M * stride * 16 + 16 * 256 * 4 <= GEMV_SMEM_BYTES_TWO_TILES


def gemv_partial_rows(M: int) -> int:
    """Entries in a row of the partial sums of squares that the kernel leaves or reads at M rows."""
    return 8 if M <= GEMV_ROWS_ANY_K else 16


def gemv_preferred(M: int, N: int, K: int) -> bool:
    """Where the streaming kernel is the rule's choice among what takes the shape."""
    return gemv_applies(M, N, K) and K <= GEMV_MAX_K and M <= GEMV_ROWS_ANY_K


def gemv(x: torch.Tensor, weight: torch.Tensor, out_dtype: torch.dtype, gated: bool = False, scale=None) -> torch.Tensor:
    """The weight-streaming kernel for up to sixteen rows (``csrc/gemv_bf16.cu``): weights from global
    memory straight into registers, ``mma.sync`` against the rows of x in shared memory.  ``gated``:
    the weight's rows are [gate | up]; returns silu(x gate^T) * (x up^T), [M, rows / 2], the values
    the product followed by ``ops.silu_mul`` gives.  ``scale`` (a ``deferred.PendingNorm`` whose
    ``scaled`` rows are x): row m of the product is multiplied by the norm's scale of that row first."""
    M, K = x.shape
    N = weight.shape[0]
    y = torch.empty((M, N // 2 if gated else N), dtype=out_dtype, device=x.device)
    lib = load_library("gemv_bf16")
    if scale is None:
        ops._check(lib.tb_gemv(ops._stream(), ops._ptr(x), ops._ptr(weight), ops._ptr(y), M, N, K,
                               int(out_dtype == torch.float32), int(gated), sm_count(x.device)), "gemv")
    else:
        ops._check(lib.tb_gemv_scaled(ops._stream(), ops._ptr(x), ops._ptr(weight), ops._ptr(y), M, N, K, int(out_dtype == torch.float32),
                                      int(gated), sm_count(x.device), ops._ptr(scale.partials), scale.parts, ctypes.c_float(scale.eps)),
                   "gemv (rows scaled)")
    return y


def gemv_add(x: torch.Tensor, weight: torch.Tensor, residual: torch.Tensor, norm_weight: torch.Tensor) -> tuple:
    """residual [M, N] (float32) += bfloat16(x @ weight^T), by the streaming kernel itself.  Returns
    (bfloat16(residual * norm_weight) [M, N], the blocks' partial sums of squares of the new rows
    [parts, 8 or, above eight rows, 16], parts)."""
    lib = load_library("gemv_bf16")
    M, K = x.shape
    N = weight.shape[0]
    parts = lib.tb_gemv_grid(N, 0, sm_count(x.device))
    partials = torch.empty((parts, gemv_partial_rows(M)), dtype=torch.float32, device=x.device)
    scaled = torch.empty((M, N), dtype=torch.bfloat16, device=x.device)
    ops._check(lib.tb_gemv_add(ops._stream(), ops._ptr(x), ops._ptr(weight), ops._ptr(residual), ops._ptr(norm_weight), ops._ptr(scaled),
                               ops._ptr(partials), M, N, K, sm_count(x.device)), "gemv (added into the residual)")
    return scaled, partials, parts


def add_fusable(x: torch.Tensor, weight: torch.Tensor) -> bool:
    """A product that the streaming kernel runs, and so may add into the residual itself."""
    if ops.env("TANDEM_FUSE_NORM", "1") == "0":
        return False
    return (x.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16
            and choose(x.shape[0], weight.shape[0], x.shape[1], _aligned(x, weight)) == "gemv")


def scale_fusable(norm, weight: torch.Tensor) -> bool:
    """A norm with its rows' scale pending whose reader is a product that the streaming kernel runs."""
    M, K = norm.scaled.shape
    return (weight.dtype == torch.bfloat16 and weight.shape[1] == K
            and choose(M, weight.shape[0], K, _aligned(norm.scaled, weight)) == "gemv")


ROW_CLASSES = (1, 2, 4, 8, 16, 32, 64)

# Measured on a B200: (rows of W, K) -> class of rows -> the fastest kernel (this package's kept where
# within 2 % of it), for the projections of Qwen3-8B, -14B and -32B and the output head; what
# ``python -m tandem_b200.kernels.microbench dispatch --shapes 8b|14b|32b`` prints.  Shapes that are
# not listed follow the rule in ``choose``.  12vivi/tandem keeps such a table per GPU
# (python/tandem/layers/triton_gemv.py:221-267).
# The class of 9 to 16 rows names the streaming kernel for the first three products of a Qwen3-8B layer:
# it takes them up to 14 rows (``gemv_applies``; 15 and 16 fall through to the rule), alone it is level
# with the library there (qkv 11.7 against 12.1 us, o 9.2 against 9.9, gate_up 34.3 against 34.4 at 12
# rows), and in a decode step it takes the add and the norm between the products along and lets decode
# attention move in early: 3.78 against 3.99 ms at batch 9, 3.94 against 4.12 at 12, 4.15 against 4.23 at 14.
# With K = 5120 it takes up to 11 rows, and a step gains from it for gate_up alone (Qwen3-14B at batch 10:
# 6.34 against 6.48 ms, 6.38 with o and qkv as well; Qwen3-32B: 13.31 against 13.49 ms, 13.49 with qkv as well).
_G, _S, _L = "gemv", "skinny", "library"
MEASURED = {
    (6144, 4096): {1: _G, 2: _G, 4: _G, 8: _G, 16: _G, 32: _L, 64: _L},
    (4096, 4096): {1: _G, 2: _G, 4: _G, 8: _G, 16: _G, 32: _L, 64: _L},
    (24576, 4096): {1: _G, 2: _G, 4: _G, 8: _G, 16: _G, 32: _L, 64: _L},
    (4096, 12288): {1: _G, 2: _G, 4: _G, 8: _G, 16: _L, 32: _L, 64: _L},
    (151936, 4096): {1: _G, 2: _G, 4: _G, 8: _G, 16: _S, 32: _S, 64: _S},
    (7168, 5120): {1: _L, 2: _L, 4: _L, 8: _L, 16: _L, 32: _L, 64: _L},
    (5120, 5120): {1: _L, 2: _L, 4: _L, 8: _L, 16: _L, 32: _L, 64: _L},
    (34816, 5120): {1: _G, 2: _G, 4: _G, 8: _G, 16: _G, 32: _L, 64: _L},
    (5120, 17408): {1: _L, 2: _L, 4: _L, 8: _L, 16: _L, 32: _L, 64: _L},
    (151936, 5120): {1: _S, 2: _S, 4: _S, 8: _G, 16: _S, 32: _S, 64: _S},
    (10240, 5120): {1: _G, 2: _L, 4: _G, 8: _G, 16: _L, 32: _L, 64: _L},
    (5120, 8192): {1: _G, 2: _L, 4: _L, 8: _L, 16: _L, 32: _L, 64: _L},
    (51200, 5120): {1: _G, 2: _G, 4: _G, 8: _G, 16: _G, 32: _S, 64: _L},
    (5120, 25600): {1: _S, 2: _S, 4: _S, 8: _S, 16: _S, 32: _L, 64: _L},
}


def row_class(M: int) -> int:
    """Row counts fall into classes: up to 1, 2, 4, 8, 16, 32, 64 rows."""
    return next(c for c in ROW_CLASSES if M <= c) if M <= SKINNY_MAX_ROWS else 0


_library_only = False


def keep_library_products(on: bool = True) -> None:
    """Process-wide: every bfloat16 product goes to the library, as ``TANDEM_GEMM=library`` does (12vivi/tandem's
    ``--no-small-batch-gemv``, python/tandem/entrypoints/cli.py:35-36: keep cuBLAS for the decoder projections)."""
    global _library_only
    _library_only = bool(on)


def _forced() -> Optional[str]:
    return "library" if _library_only else ops.env("TANDEM_GEMM")


def choose(M: int, N: int, K: int, aligned: bool = True) -> str:
    """"gemv", "skinny" or "library" for a product of these sizes: a fixed rule, the same on every
    run.  ``aligned``: x and the weight are contiguous and start on 16-byte boundaries."""
    can_gemv = gemv_applies(M, N, K) and aligned
    can_skinny = skinny_applies(M, N, K) and aligned
    forced = _forced()
    if forced == "library" or (forced == "gemv" and can_gemv) or (forced == "skinny" and can_skinny):
        return forced
    measured = MEASURED.get((N, K), {}).get(row_class(M))
    if measured == "library" or (measured == "gemv" and can_gemv) or (measured == "skinny" and can_skinny):
        return measured
    if can_gemv and gemv_preferred(M, N, K):
        return "gemv"
    if can_skinny and N * K * 2 >= SKINNY_MIN_WEIGHT_BYTES[row_class(M)]:
        return "skinny"
    return "library"


def choose_gated(M: int, N: int, K: int, aligned: bool = True) -> str:
    """Who computes silu(x gate^T) * (x up^T): "gemv" (activation inside the streaming kernel),
    "pair" or "wide" (activation in the epilogue of a tcgen05 kernel for many rows: pairs of blocks,
    or single blocks), or "product" (the product as ``choose`` says, then the activation kernel)."""
    if N % 16:
        return "product"
    forced = _forced()
    if M <= GEMV_MAX_ROWS and choose(M, N, K, aligned) == "gemv":
        return "gemv"
    if M <= GEMV_ROWS_ANY_K:
        return "product"
    if forced in ("wide", "pair"):
        return forced if wide_applies(M, N, K) and aligned else "product"
    if forced in ("library", "skinny", "gemv"):
        return "product"
    if not (wide_applies(M, N, K) and aligned):
        return "product"
    if M >= PAIR_GATED_MIN_ROWS and -(-M // 256) * 256 <= PAIR_MAX_PADDING * (-(-M // 128) * 128):
        return "pair"
    in_range = any(lo <= M and (hi is None or M <= hi) for lo, hi in WIDE_GATED_ROWS)
    if M < WIDE_GATED_ROWS[0][0] and N * K * 2 >= WIDE_GATED_FEW_ROWS_MIN_WEIGHT_BYTES:
        in_range = True
    return "wide" if in_range else "product"


def _aligned(x: torch.Tensor, weight: torch.Tensor) -> bool:
    return x.is_contiguous() and weight.is_contiguous() and x.data_ptr() % 16 == 0 and weight.data_ptr() % 16 == 0


def gated(x: torch.Tensor, weight: torch.Tensor) -> torch.Tensor:
    """silu(x gate^T) * (x up^T) for a weight whose rows are [gate | up]: [M, rows / 2] bfloat16."""
    M, K = x.shape
    N = weight.shape[0]
    which = choose_gated(M, N, K, _aligned(x, weight))
    if which == "gemv":
        return gemv(x, weight, torch.bfloat16, gated=True)
    if which == "wide":
        return wide(x, weight, torch.bfloat16, gated=True)
    if which == "pair":
        return wide_pair(x, weight, torch.bfloat16, gated=True)
    return ops.silu_mul(linear(x, weight, torch.bfloat16))


def linear(x: torch.Tensor, weight: torch.Tensor, out_dtype: torch.dtype) -> torch.Tensor:
    if out_dtype not in (torch.bfloat16, torch.float32):
        raise ops.KernelError(f"the bfloat16 product returns bfloat16 or float32, not {out_dtype}")
    which = choose(x.shape[0], weight.shape[0], x.shape[1], _aligned(x, weight))
    if which == "skinny":
        return skinny(x, weight, out_dtype)
    if which == "gemv":
        return gemv(x, weight, out_dtype)
    return _library(x, weight, out_dtype)
