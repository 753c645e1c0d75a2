"""The physical layout of a cache tile, in Python (``tandem_b200/csrc/cache_layout.cuh`` is the
same map for the kernels).

A cache tensor has the logical shape [pages, kv heads, page_size, head_dim].  float32 caches and
head sizes that are no multiple of 64 store exactly that.  bfloat16 caches with head_dim a
multiple of 64 (page sizes below 8 or multiples of 8) store each [page_size, head_dim] tile as
[row groups of 8][head_dim/64 column blocks][8 rows][64], the eight 16-byte chunks of every
128-byte row XOR-ed with (row mod 8); a page of fewer than eight rows is one short group.
"""

from __future__ import annotations

import torch


def swizzled(dtype: torch.dtype, head_dim: int, page_size: int) -> bool:
    return (torch.empty((), dtype=dtype).element_size() == 2 and head_dim % 64 == 0
            and (page_size < 8 or page_size % 8 == 0))


def tile_offsets(page_size: int, head_dim: int, dtype: torch.dtype) -> torch.Tensor:
    """int64 [page_size, head_dim]: where element (row, dim) sits inside the flattened tile."""
    r = torch.arange(page_size)[:, None]
    d = torch.arange(head_dim)[None, :]
    if not swizzled(dtype, head_dim, page_size):
        return r * head_dim + d
    block, dd = d // 64, d % 64
    rows = min(page_size, 8)
    group, rr = (r // 8, r % 8) if page_size >= 8 else (0 * r, r)
    return ((group * (head_dim // 64) + block) * rows + rr) * 64 + ((((dd // 8) ^ (r % 8)) * 8) | (dd % 8))


def to_physical(logical: torch.Tensor) -> torch.Tensor:
    """A cache filled in logical order [pages, kv heads, page_size, head_dim] -> as the kernels store it."""
    pages, nkv, ps, hd = logical.shape
    off = tile_offsets(ps, hd, logical.dtype).reshape(-1).to(logical.device)
    out = torch.empty_like(logical).view(pages, nkv, ps * hd)
    out[:, :, off] = logical.reshape(pages, nkv, ps * hd)
    return out.view(pages, nkv, ps, hd)


def to_logical(physical: torch.Tensor) -> torch.Tensor:
    pages, nkv, ps, hd = physical.shape
    off = tile_offsets(ps, hd, physical.dtype).reshape(-1).to(physical.device)
    return physical.reshape(pages, nkv, ps * hd)[:, :, off].view(pages, nkv, ps, hd)
