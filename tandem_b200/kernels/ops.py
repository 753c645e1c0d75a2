"""Tensor-level entry points of the CUDA kernels.

Each function checks what it is given (device, dtype, layout, sizes), refuses what the kernel
does not take with a clear error, and launches on the current CUDA stream.  There is no CPU
path and no library stand-in for these operations: a tensor that is not on a CUDA device, or a
library that cannot be built, raises.
"""

from __future__ import annotations

import ctypes
import os
from typing import Optional

import torch

from tandem_b200.kernels.build import load_library

_DTYPE_CODE = {torch.float32: 0, torch.bfloat16: 1}


class KernelError(RuntimeError):
    pass


def _code(dtype: torch.dtype) -> int:
    try:
        return _DTYPE_CODE[dtype]
    except KeyError:
        raise KernelError(f"kernels take float32 or bfloat16 tensors, not {dtype}") from None


def _ptr(t: Optional[torch.Tensor]) -> ctypes.c_void_p:
    return ctypes.c_void_p(0 if t is None else t.data_ptr())


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)
_raw_device = getattr(torch._C, "_cuda_getDevice", None)


def _stream() -> ctypes.c_void_p:
    """The current CUDA stream's handle.  Through torch's C entry points where it has them: the Python
    wrappers around the same question took a fifth of the host's time in a step that is not replayed
    from a CUDA graph (15 us a launch)."""
    if _raw_stream is not None and _raw_device is not None:
        return ctypes.c_void_p(_raw_stream(_raw_device()))
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


_environ_bytes = getattr(os.environ, "_data", None)  # the mapping behind os.environ, keyed by encoded names (POSIX)
_encoded_names: dict = {}


def env(name: str, default: Optional[str] = None) -> Optional[str]:
    """``os.environ.get(name, default)``, read afresh at every call (tests and users change these
    switches while a process runs) but without encoding the name each time: the switches are asked
    for some fifteen times a layer."""
    if type(_environ_bytes) is not dict:
        return os.environ.get(name, default)
    key = _encoded_names.get(name)
    if key is None:
        key = _encoded_names[name] = os.fsencode(name)
    value = _environ_bytes.get(key)
    return default if value is None else os.fsdecode(value)


def device_key(device) -> str:
    """A dictionary key for per-device caches; ``str(torch.device)`` costs 2 us, so it is taken once per device object."""
    key = _device_keys.get(device)
    if key is None:
        key = _device_keys[device] = str(device)
    return key


_device_keys: dict = {}


def _need(t: torch.Tensor, name: str, dtype=None, contiguous: bool = True) -> None:
    if not t.is_cuda:
        raise KernelError(f"{name} must be on a CUDA device (there is no CPU path), got {t.device}")
    if dtype is not None and t.dtype != dtype:
        raise KernelError(f"{name} must be {dtype}, got {t.dtype}")
    if contiguous and not t.is_contiguous():
        raise KernelError(f"{name} must be contiguous")


launches = 0  # kernels of this package launched so far (CUDA-graph replays count what they captured)


def _check(status: int, what: str) -> None:
    global launches
    launches += 1
    if status != 0:
        detail = {10001: "unsupported dtype", 10002: "unsupported size"}.get(status, f"CUDA error {status}")
        raise KernelError(f"{what}: {detail}")


_status: dict = {}


def status_word(device) -> torch.Tensor:
    """int32 [1] on the device where kernels record a fault they survived (0: none): a bounded
    wait that gave up (1), a block table entry that should have held a page (2)."""
    key = device_key(device)
    if key not in _status:
        with torch.inference_mode(False):  # an ordinary tensor: it is written in and outside inference mode
            _status[key] = torch.zeros(1, dtype=torch.int32, device=device)
    return _status[key]


def raise_status(device, code: int) -> None:
    """Clear the status word and raise for the fault ``code`` that was read from it."""
    status_word(device).zero_()
    what = {1: "a bounded wait inside a kernel gave up", 2: "a kernel met a missing page in a block table"}
    raise KernelError(f"kernel status {code}: {what.get(code, 'unknown fault')}; results of this step are invalid")


def check_status(device) -> None:
    """Read the status word (this waits for the device) and raise if a kernel recorded a fault."""
    code = int(status_word(device).item())
    if code:
        raise_status(device, code)


# ----------------------------------------------------------------------------- token-wise
def embedding(ids: torch.Tensor, table: torch.Tensor, scale: float = 1.0, positions: Optional[torch.Tensor] = None,
              position_table: Optional[torch.Tensor] = None) -> torch.Tensor:
    """ids [T] int32, table [V, H] -> float32 [T, H] (the start of the residual stream):
    ``scale * table[ids]``, plus ``position_table[positions]`` where a learned table [P, H] of
    absolute positions is given."""
    _need(ids, "ids", torch.int32)
    _need(table, "embedding table")
    T, (V, H) = ids.numel(), table.shape
    max_pos = 0
    if position_table is not None:
        _need(position_table, "position table", table.dtype)
        _need(positions, "positions", torch.int32)
        if position_table.shape[1] != H or positions.numel() != T:
            raise KernelError(f"position table {tuple(position_table.shape)} / {positions.numel()} positions do not fit "
                              f"{T} tokens of width {H}")
        max_pos = position_table.shape[0]
    out = torch.empty((T, H), dtype=torch.float32, device=table.device)
    lib = load_library("tokenwise")
    _check(lib.tb_embedding(_stream(), _ptr(ids), _ptr(table), _ptr(out), T, H, V, _code(table.dtype), ctypes.c_float(scale),
                            _ptr(positions if position_table is not None else None), _ptr(position_table), max_pos), "embedding")
    return out


def scale_softcap(logits: torch.Tensor, scale: float = 1.0, softcap: Optional[float] = None) -> torch.Tensor:
    """In place on float32 logits: ``scale * x``, then ``softcap * tanh(x / softcap)`` where a cap is given."""
    _need(logits, "logits", torch.float32)
    if softcap is not None and softcap <= 0:
        raise KernelError(f"a logit cap must be positive, got {softcap}")
    lib = load_library("tokenwise")
    _check(lib.tb_scale_softcap(_stream(), _ptr(logits), ctypes.c_longlong(logits.numel()), ctypes.c_float(scale),
                                ctypes.c_float(softcap or 0.0)), "scale_softcap")
    return logits


def take_tokens(ids: torch.Tensor, source: torch.Tensor, tokens: torch.Tensor) -> None:
    """ids[i] = tokens[source[i]] wherever source[i] >= 0 (all int32, in place): tokens that the
    step before sampled enter this step's batch without a trip to the host."""
    _need(ids, "ids", torch.int32)
    _need(source, "source", torch.int32)
    _need(tokens, "tokens", torch.int32)
    if source.numel() != ids.numel():
        raise KernelError(f"source has {source.numel()} entries, ids {ids.numel()}")
    lib = load_library("tokenwise")
    _check(lib.tb_take_tokens(_stream(), _ptr(ids), _ptr(source), _ptr(tokens), ids.numel(), tokens.numel()), "take_tokens")


def add_rmsnorm(x, residual: torch.Tensor, weight: torch.Tensor, eps: float,
                out_dtype: torch.dtype, rows: Optional[torch.Tensor] = None, defer: bool = False):
    """residual += x (in place, float32; skipped when x is None); returns RMSNorm(residual) * weight
    in ``out_dtype``.  With ``rows`` [R] int32 only those rows are updated and returned, in that order.

    ``x`` may be a product that has not been launched (``deferred.PendingLinear``).  With ``defer``
    (the reader takes a ``deferred.PendingNorm``) such a product is then added into the residual by
    its own kernel and the norm comes back with its rows' scale left to the product behind it."""
    from tandem_b200.kernels import deferred, gemm_bf16

    if isinstance(x, deferred.PendingLinear):
        if defer and rows is None and out_dtype == torch.bfloat16 and x.shape == tuple(residual.shape) \
                and gemm_bf16.add_fusable(x.x, x.weight):
            _need(residual, "residual", torch.float32)
            _need(weight, "norm weight", torch.float32)
            scaled, partials, parts = gemm_bf16.gemv_add(x.x, x.weight, residual, weight)
            return deferred.PendingNorm(residual, weight, eps, out_dtype, scaled, partials, parts)
        x = deferred.tensor(x)
    _need(residual, "residual", torch.float32)
    _need(weight, "norm weight", torch.float32)
    T, H = residual.shape
    if weight.numel() != H:
        raise KernelError(f"norm weight has {weight.numel()} elements, rows have {H}")
    if x is not None:
        _need(x, "x", out_dtype)
        if x.shape != residual.shape:
            raise KernelError(f"x {tuple(x.shape)} and residual {tuple(residual.shape)} differ")
    n = T
    if rows is not None:
        _need(rows, "rows", torch.int32)
        n = rows.numel()
    y = torch.empty((n, H), dtype=out_dtype, device=residual.device)
    lib = load_library("tokenwise")
    _check(lib.tb_add_rmsnorm(_stream(), _ptr(x), _ptr(residual), _ptr(weight), _ptr(y), _ptr(rows), n, H,
                              ctypes.c_float(eps), _code(out_dtype)), "add_rmsnorm")
    return y


def qk_norm_rope_kv(qkv: torch.Tensor, positions: torch.Tensor, slots: Optional[torch.Tensor],
                    q_weight: Optional[torch.Tensor], k_weight: Optional[torch.Tensor], cos_sin: Optional[torch.Tensor],
                    k_cache: Optional[torch.Tensor], v_cache: Optional[torch.Tensor], num_heads: int,
                    num_kv_heads: int, head_dim: int, rotary_dim: int, page_size: int, eps: float,
                    write_kv: bool = True) -> torch.Tensor:
    """In place on qkv [T, (nh + 2 nkv) hd]: per-head RMSNorm (if weights) and rotary encoding of q
    and k; k and v of every token are stored at ``slots[t]`` of the caches
    [pages, nkv, page_size, hd] (unless ``write_kv`` is false or the slot is negative)."""
    _need(qkv, "qkv")
    T = qkv.shape[0]
    if qkv.shape[1] != (num_heads + 2 * num_kv_heads) * head_dim:
        raise KernelError(f"qkv has {qkv.shape[1]} columns, expected {(num_heads + 2 * num_kv_heads) * head_dim}")
    _need(positions, "positions", torch.int32)
    if rotary_dim % 2 or rotary_dim > head_dim:
        raise KernelError(f"rotary_dim {rotary_dim} must be even and at most head_dim {head_dim}")
    max_pos = 1
    if rotary_dim:
        _need(cos_sin, "cos_sin", torch.float32)
        if cos_sin.shape[1] != rotary_dim:
            raise KernelError(f"cos_sin has {cos_sin.shape[1]} columns, rotary_dim is {rotary_dim}")
        max_pos = cos_sin.shape[0]
    for w, n in ((q_weight, "q_norm weight"), (k_weight, "k_norm weight")):
        if w is not None:
            _need(w, n, torch.float32)
            if w.numel() != head_dim:
                raise KernelError(f"{n} has {w.numel()} elements, head_dim is {head_dim}")
    if write_kv:
        _need(slots, "slots", torch.int32)
        for c, n in ((k_cache, "k_cache"), (v_cache, "v_cache")):
            _need(c, n, qkv.dtype)
            if tuple(c.shape[1:]) != (num_kv_heads, page_size, head_dim):
                raise KernelError(f"{n} has shape {tuple(c.shape)}, expected [pages, {num_kv_heads}, {page_size}, {head_dim}]")
    lib = load_library("tokenwise")
    _check(lib.tb_qk_norm_rope_kv(_stream(), _ptr(qkv), _ptr(positions), _ptr(slots), _ptr(q_weight), _ptr(k_weight),
                                  _ptr(cos_sin), _ptr(k_cache), _ptr(v_cache), T, num_heads, num_kv_heads, head_dim,
                                  rotary_dim, page_size, ctypes.c_float(eps), int(bool(write_kv)), max_pos,
                                  _code(qkv.dtype)), "qk_norm_rope_kv")
    return qkv


def silu_mul(gate_up: torch.Tensor) -> torch.Tensor:
    """[T, 2I] = [gate | up] -> silu(gate) * up, [T, I]."""
    _need(gate_up, "gate_up")
    T, two_i = gate_up.shape
    if two_i % 2:
        raise KernelError("gate_up must have an even number of columns")
    out = torch.empty((T, two_i // 2), dtype=gate_up.dtype, device=gate_up.device)
    lib = load_library("tokenwise")
    _check(lib.tb_silu_mul(_stream(), _ptr(gate_up), _ptr(out), T, two_i // 2, _code(gate_up.dtype)), "silu_mul")
    return out


# ----------------------------------------------------------------------------- matrix products
def streaming_row_limit(width: int) -> int:
    """The most rows of ``width`` elements that the streaming kernel takes (bfloat16): a batch of so many
    decoding requests still has its products of that width run by it, one more goes to the library."""
    from tandem_b200.kernels import gemm_bf16

    return max((m for m in range(1, gemm_bf16.GEMV_MAX_ROWS + 1) if gemm_bf16.gemv_applies(m, 1, width)), default=0)


def linear_streams(rows: int, weight: torch.Tensor) -> bool:
    """Whether ``linear`` of so many rows with this weight runs this package's streaming kernel (all of
    whose blocks are resident at once, so that a kernel behind it may move in early)."""
    from tandem_b200.kernels import gemm_bf16

    return weight.dtype == torch.bfloat16 and gemm_bf16.choose(rows, weight.shape[0], weight.shape[1], weight.is_contiguous()) == "gemv"


def linear(x, weight: torch.Tensor, out_dtype: Optional[torch.dtype] = None, defer: bool = False):
    """x [M, K] @ weight [N, K]^T -> [M, N].  float32 operands run the CUDA-core kernel (true
    32-bit arithmetic); bfloat16 operands run on the tensor cores with float32 accumulation.

    ``x`` may be a norm whose rows' scale is still pending (``deferred.PendingNorm``).  With
    ``defer`` the product itself may stay pending (``deferred.PendingLinear``) for a norm that has it
    added into the residual by its own kernel; that happens only where the streaming kernel runs it."""
    from tandem_b200.kernels import deferred, gemm_bf16

    if isinstance(x, deferred.PendingNorm):
        if gemm_bf16.scale_fusable(x, weight):
            return gemm_bf16.gemv(x.scaled, weight, out_dtype or x.out_dtype, scale=x)
        x = deferred.tensor(x)
    if defer and x.dtype == torch.bfloat16 and out_dtype in (None, torch.bfloat16) and gemm_bf16.add_fusable(x, weight):
        return deferred.PendingLinear(x, weight)
    _need(x, "x")
    _need(weight, "weight")
    if x.dtype != weight.dtype:
        raise KernelError(f"x is {x.dtype} but the weight is {weight.dtype}")
    M, K = x.shape
    N, K2 = weight.shape
    if K != K2:
        raise KernelError(f"x has {K} columns, the weight has {K2}")
    out_dtype = out_dtype or x.dtype
    if x.dtype == torch.float32:
        if out_dtype != torch.float32:
            raise KernelError("the 32-bit product returns float32")
        out = torch.empty((M, N), dtype=torch.float32, device=x.device)
        lib = load_library("gemm_f32")
        _check(lib.tb_gemm_f32(_stream(), _ptr(x), _ptr(weight), _ptr(out), M, N, K, K, N), "gemm_f32")
        return out
    return gemm_bf16.linear(x, weight, out_dtype)


def gated_linear(x, weight: torch.Tensor) -> torch.Tensor:
    """silu(x gate^T) * (x up^T) for a weight [2I, K] whose rows are [gate | up]: [M, I].  In
    bfloat16 with many rows the activation may run in the epilogue of the product.  ``x`` may be a
    norm whose rows' scale is still pending (``deferred.PendingNorm``)."""
    from tandem_b200.kernels import deferred, gemm_bf16

    if isinstance(x, deferred.PendingNorm):
        if weight.shape[0] % 16 == 0 and gemm_bf16.scale_fusable(x, weight):
            return gemm_bf16.gemv(x.scaled, weight, torch.bfloat16, gated=True, scale=x)
        x = deferred.tensor(x)
    if x.dtype == torch.float32:
        return silu_mul(linear(x, weight))
    _need(x, "x")
    _need(weight, "weight", x.dtype)
    if x.shape[1] != weight.shape[1] or weight.shape[0] % 2:
        raise KernelError(f"x {tuple(x.shape)} and the gate/up weight {tuple(weight.shape)} do not fit")
    return gemm_bf16.gated(x, weight)


# ----------------------------------------------------------------------------- attention
def paged_attention_simt(qkv: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, block_table: torch.Tensor,
                         seq_of_token: torch.Tensor, positions: torch.Tensor, num_heads: int, num_kv_heads: int,
                         head_dim: int, page_size: int, window: Optional[int], scale: float) -> torch.Tensor:
    """Causal attention of every token of the step over its request's pages, on the CUDA cores.
    ``qkv`` [T, >= nh*hd]: the query heads are the first nh*hd columns of each row."""
    _need(qkv, "qkv")
    for c, n in ((k_cache, "k_cache"), (v_cache, "v_cache")):
        _need(c, n, qkv.dtype)
    _need(block_table, "block_table", torch.int32)
    _need(seq_of_token, "seq_of_token", torch.int32)
    _need(positions, "positions", torch.int32)
    T = qkv.shape[0]
    if num_heads % num_kv_heads:
        raise KernelError(f"{num_heads} query heads cannot share {num_kv_heads} kv heads")
    if head_dim > 512:
        raise KernelError(f"head_dim {head_dim} is larger than the 512 this kernel takes")
    out = torch.empty((T, num_heads * head_dim), dtype=qkv.dtype, device=qkv.device)
    lib = load_library("attention_simt")
    _check(lib.tb_attention_simt(_stream(), _ptr(qkv), qkv.stride(0), _ptr(k_cache), _ptr(v_cache), _ptr(block_table),
                                 block_table.stride(0), _ptr(seq_of_token), _ptr(positions), _ptr(out), T, num_heads,
                                 num_kv_heads, head_dim, page_size, int(window or 0), ctypes.c_float(scale),
                                 _code(qkv.dtype)), "attention_simt")
    return out


# ----------------------------------------------------------------------------- sampling
_ARGMAX_ROWS = 4096
_argmax_scratch: dict = {}


def argmax(logits: torch.Tensor) -> torch.Tensor:
    """[R, V] float32 -> int32 [R], the lowest index among equal maxima."""
    _need(logits, "logits", torch.float32)
    R, V = logits.shape
    out = torch.empty((R,), dtype=torch.int32, device=logits.device)
    lib = load_library("sampling")
    chunks = min(64, max(592 // max(1, R), V // 8192), V // 2048)
    if chunks < 2 or R > _ARGMAX_ROWS:
        _check(lib.tb_argmax(_stream(), _ptr(logits), _ptr(out), R, V), "argmax")
        return out
    key = device_key(logits.device)
    if key not in _argmax_scratch:  # zero before and after every call: the kernel cleans up after itself
        _argmax_scratch[key] = (torch.zeros(_ARGMAX_ROWS, dtype=torch.int64, device=logits.device),
                                torch.zeros(_ARGMAX_ROWS, dtype=torch.int32, device=logits.device))
    best, arrivals = _argmax_scratch[key]
    _check(lib.tb_argmax_split(_stream(), _ptr(logits), _ptr(out), _ptr(best), _ptr(arrivals), R, V, chunks), "argmax")
    return out


_sample_scratch: dict = {}


def sample(logits: torch.Tensor, temperature: torch.Tensor, top_k: torch.Tensor, top_p: torch.Tensor,
           min_p: torch.Tensor, uniform: torch.Tensor, any_top_k: bool = True, any_top_p: bool = True) -> torch.Tensor:
    """One token per row of logits [R, V] float32.  Per-row options as tensors [R]: temperature
    (< 1e-5: argmax), top_k (<= 0: off), top_p (>= 1: off), min_p (<= 0: off) and the uniform
    number in [0, 1) that decides the draw.  ``any_top_k`` / ``any_top_p``: whether any row uses that
    filter at all (its passes over the logits are skipped otherwise)."""
    _need(logits, "logits", torch.float32)
    R, V = logits.shape
    for t, n, dt in ((temperature, "temperature", torch.float32), (top_k, "top_k", torch.int32),
                     (top_p, "top_p", torch.float32), (min_p, "min_p", torch.float32),
                     (uniform, "uniform", torch.float32)):
        _need(t, n, dt)
        if t.numel() != R:
            raise KernelError(f"{n} has {t.numel()} entries for {R} rows")
    out = torch.empty((R,), dtype=torch.int32, device=logits.device)
    lib = load_library("sampling")
    per_row = lib.tb_sample_scratch_bytes()
    key = device_key(logits.device)
    scratch = _sample_scratch.get(key)
    if scratch is None or scratch.numel() < R * per_row:  # histograms and partial sums of the rows, kept per device
        scratch = _sample_scratch[key] = torch.empty(max(R, 64) * per_row, dtype=torch.uint8, device=logits.device)
    scratch[: R * per_row].zero_()
    _check(lib.tb_sample(_stream(), _ptr(logits), _ptr(temperature), _ptr(top_k), _ptr(top_p), _ptr(min_p),
                         _ptr(uniform), _ptr(scratch), _ptr(out), R, V, int(any_top_k), int(any_top_p)), "sample")
    return out
