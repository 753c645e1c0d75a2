"""Choice of the paged-attention kernel for a step, and the host-side plans the kernels need.

float32 always runs the CUDA-core kernel (true 32-bit arithmetic, batch-invariant bit for bit).
bfloat16 runs the tensor-core kernels where they take the shape, and the CUDA-core kernel
otherwise; all of them read the same cache layout.

The tensor-core path splits a step in two.  Requests that bring one token go to the decode kernel,
which works on *items*: a request's visible keys cut into ranges, so that few long requests still
fill the GPU (split-KV, as 12vivi/tandem's python/tandem/layers/triton_decode_attn.py:132-172
does).  Requests that bring more go to the prefill kernel, which works on *tiles* of query tokens.
Both plans are cut on the host and travel to the device with the batch description.
"""

from __future__ import annotations

import ctypes
from typing import Optional

import torch

from tandem_b200.kernels import ops
from tandem_b200.parts.base import PlanTooLarge
from tandem_b200.kernels.build import load_library

ITEM_INTS = 6  # token row, request, key begin, key end, first item of the request, its item count
TILE_INTS = 4  # first token row, request, first position, number of tokens
STAGE_KEYS = 64  # keys per shared-memory stage: items are cut at multiples of it
TILE_ROWS = 128  # rows (token x query head of the group) of a prefill tile
WORK_INTS = 5  # the tcgen05 prefill kernel's item: first token row, request, first position, number of tokens, kv head
STEP_KEYS = 128  # keys per step of the tcgen05 prefill kernel
ITEM_FIXED_STEPS = 1.5  # what an item costs beside its steps (query tiles in, output rows out), in steps
TARGET_BLOCKS = 148 * 2  # one wave at two blocks per SM
MAX_SPLITS = 64  # items per request the kernel's fast merge takes
MIN_ITEM_KEYS = 320  # a request is not cut into items shorter than this (measured: decode attention, batch 1 to 16)


def page_size_ok(page_size: int) -> bool:
    return page_size in (1, 2, 4, 8) or page_size % 16 == 0


def tensor_core_path_applies(dtype: torch.dtype, head_dim: int, page_size: int, groups: int) -> bool:
    return (dtype == torch.bfloat16 and head_dim % 16 == 0 and head_dim <= 256 and page_size_ok(page_size)
            and 1 <= groups <= TILE_ROWS)


def decode_pieces(num_rows: int, num_kv_heads: int, longest: int, target_blocks: int = TARGET_BLOCKS) -> int:
    """Into how many items the keys of every request of a decode step are cut.  As many as fill the
    GPU once, but none shorter than a few stages: every further item of a request costs the merging
    block a little.  Where the requests alone are more blocks than the GPU holds at once they run in
    rounds, and more, shorter items fill the last round better: 40 requests x 8 kv heads are two
    rounds of whole requests but 4/3 rounds' worth of thirds (measured at 2,048 and 8,192 tokens of
    context: 76 -> 70 and 276 -> 218 us; at 48 requests 78 -> 79 and 282 -> 249 us; each further item
    of a request is reckoned at 10 %, which leaves 56 and 64 requests whole, as measured)."""
    blocks = max(1, num_rows * num_kv_heads)
    most = max(1, min(MAX_SPLITS - 1, -(-longest // MIN_ITEM_KEYS)))
    if blocks <= target_blocks:
        return min(most, max(1, target_blocks // blocks))
    best, best_cost = 1, float(-(-blocks // target_blocks))
    for pieces in (2, 3, 4, 6):
        if pieces > most:
            break
        cost = -(-blocks * pieces // target_blocks) / pieces * (1.0 + 0.10 * (pieces - 1))
        if cost < 0.97 * best_cost:
            best, best_cost = pieces, cost
    return best


def decode_items_capacity(bucket: int, num_kv_heads: int, longest: int) -> int:
    """The most items ``plan_decode`` makes for up to ``bucket`` requests of up to ``longest`` keys
    (a request whose range straddles one more multiple of the items' length has one item more)."""
    return max(r * (decode_pieces(r, num_kv_heads, longest) + 1) for r in range(1, bucket + 1)) + 8


def plan_decode(rows, window: Optional[int], num_kv_heads: int, target_blocks: int = TARGET_BLOCKS) -> list:
    """``rows``: (token row, request, position) of every request that brings one token.  Returns
    the items [token row, request, key begin, key end, first item of the request, its item count]."""
    if not rows:
        return []
    lo = [max(0, p - window + 1) if window else 0 for _, _, p in rows]
    longest = max(p + 1 - l for (_, _, p), l in zip(rows, lo))
    pieces = decode_pieces(len(rows), num_kv_heads, longest, target_blocks)
    split = max(STAGE_KEYS, -(-(-(-longest // pieces)) // STAGE_KEYS) * STAGE_KEYS)
    items = []
    for (t, b, p), l in zip(rows, lo):
        first, k = len(items), l
        while k <= p:
            nxt = min(p + 1, (k // split + 1) * split)
            items.append([t, b, k, nxt, first, 0])
            k = nxt
        for it in items[first:]:
            it[5] = len(items) - first
    return items


def prefill_library(head_dim: int):
    extra = tuple(d for d in ops.env("TANDEM_PREFILL_DEFS", "").split(",") if d)
    return load_library("attention_prefill", (f"TB_HD={head_dim}",) + extra)


def tcgen05_prefill_applies(head_dim: int, page_size: int) -> bool:
    """The tcgen05 prefill kernel takes head sizes 64 and 128 and pages of 8 keys or a multiple of 16
    (``TANDEM_PREFILL=mma`` keeps the mma.sync kernel)."""
    return (head_dim in (64, 128) and (page_size == 8 or page_size % 16 == 0)
            and ops.env("TANDEM_PREFILL", "tcgen05") != "mma")


def plan_prefill(seqs, groups: int, tile_rows: int = TILE_ROWS) -> list:
    """``seqs``: (first token row, request, first position, number of tokens) of every request that
    brings several tokens.  Returns tiles of at most tile_rows // groups tokens, those with the most keys first
    (the mma.sync kernel's plan: one block per tile and kv head)."""
    per_tile = tile_rows // groups
    tiles = [[t0 + off, b, p0 + off, min(per_tile, n - off)] for t0, b, p0, n in seqs for off in range(0, n, per_tile)]
    tiles.sort(key=lambda x: -(x[2] + x[3]))
    return tiles


def _item_steps(p0: int, ntok: int, per_tile: int, window: Optional[int]) -> int:
    """Steps of 128 keys that the two query tiles of an item take together (as the kernel counts them)."""
    kb = max(0, p0 - window + 1) if window else 0
    s0 = kb // STEP_KEYS * STEP_KEYS
    steps = 0
    for first in (0, per_tile):
        last = min(ntok, first + per_tile)
        if last > first:
            kb_t = max(0, p0 + first - window + 1) if window else 0
            steps += -(-(p0 + last - s0) // STEP_KEYS) - (kb_t - s0) // STEP_KEYS
    return steps


def plan_prefill_queues(seqs, groups: int, num_kv_heads: int, window: Optional[int], blocks: int,
                        tile_rows: int = TILE_ROWS, fixed_blocks: bool = False) -> list:
    """The tcgen05 kernel's plan.  ``seqs`` as for ``plan_prefill``; an item is up to two tiles' worth
    of consecutive tokens of a request for one kv head, [first token row, request, first position,
    number of tokens, kv head].  One persistent block per SM walks a queue of items; the queues are
    balanced here (heaviest item first, each to the block with the least work so far), so that the
    kernel neither counts nor fetches anything at run time.  Returns [queue position][block][5];
    an item without tokens ends a block's queue.  ``fixed_blocks``: queues for all ``blocks`` blocks
    even where the items are fewer (a CUDA graph launches the same grid whatever the step brings)."""
    import heapq

    per_tile = tile_rows // groups
    items = []
    for t0, b, p0, n in seqs:
        for off in range(0, n, 2 * per_tile):
            ntok = min(2 * per_tile, n - off)
            cost = _item_steps(p0 + off, ntok, per_tile, window) + ITEM_FIXED_STEPS
            items.extend((cost, [t0 + off, b, p0 + off, ntok, h]) for h in range(num_kv_heads))
    if not items:
        return []
    items.sort(key=lambda x: -x[0])
    blocks = max(1, blocks if fixed_blocks else min(blocks, len(items)))
    queues = [[] for _ in range(blocks)]
    heap = [(0.0, c) for c in range(blocks)]
    for cost, item in items:
        load, c = heapq.heappop(heap)
        queues[c].append(item)
        heapq.heappush(heap, (load + cost, c))
    longest = max(len(q) for q in queues)
    return [[q[k] if k < len(q) else [0] * WORK_INTS for q in queues] for k in range(longest)]


def prefill_queue_capacity(tokens: int, seqs: int, groups: int, num_kv_heads: int, blocks: int, tile_rows: int = TILE_ROWS) -> int:
    """Queue positions that ``plan_prefill_queues`` is given room for in a CUDA graph for steps of up to
    ``tokens`` tokens of up to ``seqs`` requests: the items at their most (every request's last item may be
    short) shared out evenly, and two more; a step whose balance by cost needs more runs without a graph."""
    per_item = 2 * (tile_rows // groups)
    items = (tokens // per_item + min(seqs, tokens)) * num_kv_heads
    return -(-items // max(1, blocks)) + 2


def prefill_plan(seqs, num_heads: int, num_kv_heads: int, head_dim: int, page_size: int, window: Optional[int],
                 device) -> torch.Tensor:
    """The plan for whichever prefill kernel takes this shape, on the device: [queue position, block, 5]
    for the tcgen05 kernel, [tiles * 4] for the mma.sync kernel."""
    groups = num_heads // num_kv_heads
    if tcgen05_prefill_applies(head_dim, page_size):
        from tandem_b200.kernels.gemm_bf16 import sm_count

        queues = plan_prefill_queues(seqs, groups, num_kv_heads, window, sm_count(device))
        return torch.tensor(queues, dtype=torch.int32).view(len(queues), -1, WORK_INTS).to(device)
    return torch.tensor([x for t in plan_prefill(seqs, groups) for x in t], dtype=torch.int32).to(device)


_workspaces: dict = {}


def _workspace(device, items: int, num_kv_heads: int, groups: int, head_dim: int):
    """Scratch of the decode kernel, kept and grown per device: partial outputs, their (max, sum)
    and arrival counters (zero between launches).  A scratch that was outgrown is kept, not freed:
    CUDA graphs captured while it was current still write to it when they are replayed."""
    key = ops.device_key(device)
    rows = items * num_kv_heads * groups
    ws = _workspaces.get(key)
    if ws is None or ws["rows"] < rows or ws["hd"] < head_dim:
        rows = max(rows, ws["rows"] if ws else 0)
        hd = max(head_dim, ws["hd"] if ws else 0)
        retired = (ws["retired"] + [ws]) if ws else []
        ws = dict(rows=rows, hd=hd, retired=retired,
                  part_o=torch.empty(rows * hd, dtype=torch.float32, device=device),
                  part_ml=torch.empty(rows * 2, dtype=torch.float32, device=device),
                  counters=torch.zeros(rows + 64, dtype=torch.int32, device=device))
        if retired:
            retired[-1]["retired"] = []
        _workspaces[key] = ws
    return ws


FRESH_MAX_TOKENS = 8  # rows up to which the projection in front is always taken to be this package's streaming kernel


def fresh_applies(head_dim: int, rotary_dim: int, writable: bool, num_tokens: int = 1, streamed: bool = False) -> bool:
    """Whether decode attention should make its query rows and the newest key itself from the raw
    projection (per-head norm, rotary encoding, cache write folded in): the whole head rotates and
    the head size is a power of two, as the stand-alone kernel's fast path wants it too, and the
    step has at most eight tokens, or the projection in front is the streaming kernel (``streamed``).
    Measured on a decode step at Qwen3-8B sizes: 3.54 against 3.61 ms at batch 8, 313.5 against 311 tok/s
    at batch 1, 3.95 against 3.99 ms at batch 12 behind the streaming kernel; nothing to speak of at 16,
    48 and 64 tokens, and 5.99 against 5.06 ms at 32, where the kernel in front is then a library
    product whose blocks do not all fit at once and the attention blocks that move in early take their room."""
    return (writable and rotary_dim == head_dim and head_dim & (head_dim - 1) == 0 and 16 <= head_dim <= 256
            and (num_tokens <= FRESH_MAX_TOKENS or streamed) and ops.env("TANDEM_FRESH_ATTENTION", "1") != "0")


def paged_attention_decode(qkv: torch.Tensor, kv, items: torch.Tensor, count: torch.Tensor, num_heads: int,
                           num_kv_heads: int, head_dim: int, scale: float,
                           out: Optional[torch.Tensor] = None, fresh: Optional[dict] = None) -> torch.Tensor:
    """One token per request: ``items`` int32 [capacity * 6] and ``count`` int32 [1] (how many of
    them are real) as ``plan_decode`` cut them.  Writes the rows of ``out`` that the items name.

    ``fresh`` (positions, slots, q_norm, k_norm, cos_sin, eps): ``qkv`` is the raw projection; the
    kernel normalises and rotates its query rows and each request's new key itself and writes
    the new key and value to the cache (what ``ops.qk_norm_rope_kv`` would have done in front of it)."""
    T = qkv.shape[0]
    capacity = items.numel() // ITEM_INTS
    groups = num_heads // num_kv_heads
    if out is None:
        out = torch.empty((T, num_heads * head_dim), dtype=qkv.dtype, device=qkv.device)
    ws = _workspace(qkv.device, capacity, num_kv_heads, groups, head_dim)
    lib = load_library("attention_decode", (f"TB_HD={head_dim}",))
    ops._check(lib.tb_attention_decode(
        ops._stream(), ops._ptr(qkv), qkv.stride(0), ops._ptr(kv.k), ops._ptr(kv.v), ops._ptr(kv.block_table),
        kv.block_table.stride(0), ops._ptr(items), ops._ptr(count), capacity, ops._ptr(out), ops._ptr(ws["part_o"]),
        ops._ptr(ws["part_ml"]), ops._ptr(ws["counters"]), ops._ptr(ops.status_word(qkv.device)), num_heads,
        num_kv_heads, kv.page_size, ctypes.c_float(scale), *_fresh_args(fresh, qkv, num_heads, num_kv_heads, head_dim)),
        "attention_decode")
    return out


def _fresh_args(fresh: Optional[dict], qkv: torch.Tensor, num_heads: int, num_kv_heads: int, head_dim: int) -> tuple:
    if fresh is None:
        return (0, None, None, None, None, None, ctypes.c_float(0.0), 0)
    cos_sin, positions, slots = fresh["cos_sin"], fresh["positions"], fresh["slots"]
    ops._need(cos_sin, "cos_sin", torch.float32)
    ops._need(positions, "positions", torch.int32)
    ops._need(slots, "slots", torch.int32)
    if qkv.shape[1] != (num_heads + 2 * num_kv_heads) * head_dim or not qkv.is_contiguous():
        raise ops.KernelError("decode attention from the raw projection wants qkv [T, (nh + 2 nkv) * hd], contiguous")
    if cos_sin.shape[1] != head_dim or positions.numel() != qkv.shape[0] or slots.numel() != qkv.shape[0]:
        raise ops.KernelError("cos_sin, positions or slots do not fit the rows of qkv")
    for w in (fresh.get("q_norm"), fresh.get("k_norm")):
        if w is not None:
            ops._need(w, "norm weight", torch.float32)
            if w.numel() != head_dim:
                raise ops.KernelError(f"a head norm weight has {w.numel()} elements, head_dim is {head_dim}")
    return (1, ops._ptr(fresh.get("q_norm")), ops._ptr(fresh.get("k_norm")), ops._ptr(cos_sin), ops._ptr(positions), ops._ptr(slots),
            ctypes.c_float(fresh["eps"]), cos_sin.shape[0])


def paged_attention_prefill(qkv: torch.Tensor, kv, tiles: torch.Tensor, num_heads: int, num_kv_heads: int,
                            head_dim: int, window: Optional[int], scale: float,
                            out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Several tokens per request: ``tiles`` is the plan that ``prefill_plan`` makes for the kernel
    that takes this shape (int32 [queue positions, blocks, 5] as ``plan_prefill_queues`` balanced them
    for the tcgen05 kernel, [n * 4] as ``plan_prefill`` cut them for the mma.sync kernel)."""
    T = qkv.shape[0]
    if out is None:
        out = torch.empty((T, num_heads * head_dim), dtype=qkv.dtype, device=qkv.device)
    if tcgen05_prefill_applies(head_dim, kv.page_size):
        if tiles.dim() != 3 or tiles.shape[2] != WORK_INTS:
            raise ops.KernelError("the tcgen05 prefill kernel wants its plan as [queue positions, blocks, 5]")
        lib = load_library("attention_prefill_tc", (f"TB_HD={head_dim}",))
        ops._check(lib.tb_attention_prefill_tc(
            ops._stream(), ops._ptr(qkv), T, qkv.stride(0), ops._ptr(kv.k), ops._ptr(kv.v), ops._ptr(kv.block_table),
            kv.block_table.stride(0), ops._ptr(tiles), tiles.shape[0], tiles.shape[1], ops._ptr(out),
            ops._ptr(ops.status_word(qkv.device)), num_heads, num_kv_heads, kv.page_size, int(window or 0),
            ctypes.c_float(scale)), "attention_prefill_tc")
        return out
    ops._check(prefill_library(head_dim).tb_attention_prefill(
        ops._stream(), ops._ptr(qkv), qkv.stride(0), ops._ptr(kv.k), ops._ptr(kv.v), ops._ptr(kv.block_table),
        kv.block_table.stride(0), ops._ptr(tiles), tiles.numel() // TILE_INTS, ops._ptr(out),
        ops._ptr(ops.status_word(qkv.device)), num_heads, num_kv_heads, kv.page_size, int(window or 0),
        ctypes.c_float(scale)), "attention_prefill")
    return out


def plan_key(window: Optional[int], num_heads: int, num_kv_heads: int, head_dim: int, dtype: torch.dtype) -> tuple:
    """What a step's attention plan depends on, and with it which kernel runs: layers that agree in
    all of this share one plan; two layers with equal head counts and different head sizes do not."""
    return ("attention", window, num_heads, num_kv_heads, head_dim, str(dtype))


def plan_step(ctx, window: Optional[int], num_heads: int, num_kv_heads: int, head_dim: int, out: dict) -> None:
    """Cut this step's attention work for the tensor-core kernels (if they apply) and put the
    arrays into ``out``; what was planned is remembered in ``ctx.scratch`` for ``paged_attention``."""
    key = plan_key(window, num_heads, num_kv_heads, head_dim, ctx.dtype)
    groups = num_heads // num_kv_heads
    if key in ctx.scratch or not tensor_core_path_applies(ctx.dtype, head_dim, ctx.page_size, groups):
        return
    single, several, row = [], [], 0
    for b, (start, n) in enumerate(zip(ctx.host_starts, ctx.host_lens)):
        (single if n == 1 else several).append((row, b, start) if n == 1 else (row, b, start, n))
        row += n
    items = plan_decode(single, window, num_kv_heads)
    out[key + ("items",)] = [x for it in items for x in it]
    out[key + ("count",)] = [len(items)]
    if tcgen05_prefill_applies(head_dim, ctx.page_size):
        from tandem_b200.kernels.gemm_bf16 import sm_count

        blocks = sm_count(ctx.device)
        queues = plan_prefill_queues(several, groups, num_kv_heads, window, blocks, fixed_blocks=ctx.static_layout)
        if ctx.static_layout:  # every queue position of the graph's capacity, empty ones included; both kernels always run
            import numpy as np

            capacity = prefill_queue_capacity(ctx.num_tokens, ctx.num_seqs, groups, num_kv_heads, blocks)
            if len(queues) > capacity:
                raise PlanTooLarge(f"{len(queues)} queue positions, the graph has room for {capacity}")
            laid_out = np.zeros((capacity, blocks, WORK_INTS), dtype=np.int32)
            if queues:
                laid_out[: len(queues)] = np.asarray(queues, dtype=np.int32)
            out[key + ("tiles",)] = laid_out.reshape(-1)
            ctx.scratch[key] = (1, capacity)
            return
        ctx.scratch[key] = (len(items), len(queues))
        out[key + ("tiles",)] = [x for row in queues for item in row for x in item]
    else:
        if ctx.static_layout:
            raise PlanTooLarge("steps with prompt portions are captured only where the tcgen05 prefill kernel applies")
        tiles = plan_prefill(several, groups)
        out[key + ("tiles",)] = [x for t in tiles for x in t]
        ctx.scratch[key] = (len(items), len(tiles))


def decodes_only(ctx, num_heads: int, num_kv_heads: int, head_dim: int, window: Optional[int], dtype: torch.dtype) -> bool:
    """The step was planned for the tensor-core kernels and brings single tokens only: all of its
    attention is the decode kernel's."""
    planned = ctx.scratch.get(plan_key(window, num_heads, num_kv_heads, head_dim, dtype))
    return planned is not None and planned[1] == 0 and planned[0] > 0


def paged_attention(qkv: torch.Tensor, kv, ctx, num_heads: int, num_kv_heads: int, head_dim: int,
                    window: Optional[int], scale: float, fresh: Optional[dict] = None) -> torch.Tensor:
    """Attention output [T, nh * hd] for the query heads in the first nh*hd columns of qkv.
    ``fresh``: see ``paged_attention_decode`` (only for steps for which ``decodes_only`` holds)."""
    key = plan_key(window, num_heads, num_kv_heads, head_dim, qkv.dtype)
    planned = ctx.scratch.get(key)
    if planned is None:
        return ops.paged_attention_simt(qkv, kv.k, kv.v, kv.block_table, ctx.seq_of_token, ctx.positions, num_heads,
                                        num_kv_heads, head_dim, kv.page_size, window, scale)
    num_items, num_tiles = planned
    out = torch.empty((qkv.shape[0], num_heads * head_dim), dtype=qkv.dtype, device=qkv.device)
    if num_tiles:
        tiles = ctx.extras[key + ("tiles",)]
        if tcgen05_prefill_applies(head_dim, kv.page_size):
            tiles = tiles.view(num_tiles, -1, WORK_INTS)  # num_tiles: queue positions
        paged_attention_prefill(qkv, kv, tiles, num_heads, num_kv_heads, head_dim, window, scale, out)
    if num_items:
        paged_attention_decode(qkv, kv, ctx.extras[key + ("items",)], ctx.extras[key + ("count",)], num_heads,
                               num_kv_heads, head_dim, scale, out, fresh)
    return out
