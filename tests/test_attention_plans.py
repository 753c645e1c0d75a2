"""The host-side plans of the tensor-core attention kernels (no GPU needed): every token is
planned once, items respect the kernels' limits, and the prefill queues are balanced."""
import random

import pytest

from tandem_b200.kernels import attention as A


def _steps(item, per_tile, window):
    return A._item_steps(item[2], item[3], per_tile, window)


@pytest.mark.parametrize("groups,nkv,window,blocks", [(4, 8, None, 148), (1, 2, None, 5), (3, 2, 70, 7), (7, 1, 9, 148), (128, 1, None, 3)])
def test_prefill_queues_cover_every_token_once_and_are_balanced(groups, nkv, window, blocks):
    rng = random.Random(groups * 1000 + nkv)
    seqs, row = [], 0
    for b in range(9):
        n, start = rng.choice([2, 3, 17, 64, 65, 200, 700]), rng.choice([0, 5, 63, 64, 1000])
        seqs.append((row, b, start, n))
        row += n
    queues = A.plan_prefill_queues(seqs, groups, nkv, window, blocks)
    per_tile = A.TILE_ROWS // groups
    width = len(queues[0])
    assert 1 <= width <= blocks and all(len(q) == width for q in queues)
    seen, loads = {}, [0.0] * width
    for c in range(width):
        ended = False
        for k in range(len(queues)):
            item = queues[k][c]
            assert len(item) == A.WORK_INTS
            if item[3] == 0:
                ended = True  # nothing behind the end of a block's queue
                continue
            assert not ended
            t0, b, p0, ntok, h = item
            assert 1 <= ntok <= 2 * per_tile and 0 <= h < nkv
            for i in range(ntok):
                assert seen.setdefault((t0 + i, h), (b, p0 + i)) == (b, p0 + i)
                seen[(t0 + i, h)] = None  # a second item with this token and head fails the line above
            loads[c] += _steps(item, per_tile, window) + A.ITEM_FIXED_STEPS
    assert len(seen) == row * nkv
    for t0, b, p0, n in seqs:  # positions follow the rows
        assert all((t0 + i, h) in seen for i in range(n) for h in range(nkv))
    heaviest = max(_steps(it, per_tile, window) + A.ITEM_FIXED_STEPS for q in queues for it in q if it[3])
    assert max(loads) <= sum(loads) / width + heaviest  # longest-processing-time-first keeps within one item of the mean


def test_item_steps_counts_what_the_kernel_walks():
    # 64 tokens from position 1984 on, 32 to a tile: both tiles walk the 16 steps of 128 keys
    assert A._item_steps(1984, 64, 32, None) == 32
    # one tile only
    assert A._item_steps(0, 20, 32, None) == 1
    # the second tile ends in a step that the first never reaches
    assert A._item_steps(96, 64, 32, None) == 1 + 2
    # a window: steps that lie before every query's window are not walked
    assert A._item_steps(1000, 64, 32, 100) == A._item_steps(1000 - 896, 64, 32, 100)


def test_prefill_tiles_for_the_mma_kernel():
    tiles = A.plan_prefill([(0, 0, 10, 70), (70, 1, 0, 5)], 4)
    assert sorted(t[3] for t in tiles) == [5, 6, 32, 32]
    assert [t[2] + t[3] for t in tiles] == sorted((t[2] + t[3] for t in tiles), reverse=True)


def test_decode_items_cover_the_visible_keys():
    rows = [(0, 0, 4999), (1, 1, 10), (2, 2, 700)]
    for window in (None, 300):
        items = A.plan_decode(rows, window, 8)
        for t, b, p in rows:
            mine = [it for it in items if it[0] == t]
            lo = max(0, p - window + 1) if window else 0
            assert mine[0][2] == lo and mine[-1][3] == p + 1
            assert all(x[3] == y[2] for x, y in zip(mine, mine[1:]))
            assert all(it[5] == len(mine) and it[4] == items.index(mine[0]) for it in mine)


def test_decode_pieces_fill_the_rounds():
    # few requests: as many items as fill the GPU once, none shorter than 320 keys
    assert A.decode_pieces(1, 8, 2048) == 7 and A.decode_pieces(8, 8, 2048) == 4 and A.decode_pieces(8, 8, 300) == 1
    # whole requests that fit at once stay whole
    assert A.decode_pieces(32, 8, 8192) == 1 and A.decode_pieces(36, 8, 8192) == 1
    # a round and a bit: shorter items fill the last round
    assert A.decode_pieces(40, 8, 8192) == 3 and A.decode_pieces(48, 8, 8192) == 3 and A.decode_pieces(40, 8, 600) == 2
    # nearly two full rounds: nothing to gain
    assert A.decode_pieces(64, 8, 8192) == 1
    # the capacity a CUDA graph reserves covers every plan of its bucket
    for bucket in (1, 8, 64):
        cap = A.decode_items_capacity(bucket, 8, 4096)
        for n in range(1, bucket + 1):
            for length in (1, 319, 4096):
                assert len(A.plan_decode([(i, i, length - 1) for i in range(n)], None, 8)) <= cap
