"""Which kernel computes a bfloat16 product is a fixed function of its sizes (no GPU needed to ask)."""

import pytest

from tandem_b200.kernels import gemm_bf16 as G

QKV, O, GATE_UP, DOWN, HEAD = (6144, 4096), (4096, 4096), (24576, 4096), (4096, 12288), (151936, 4096)


def test_the_streaming_kernel_takes_what_fits_into_shared_memory():
    for N, K in (QKV, O, GATE_UP):
        assert [G.choose(M, N, K) for M in (1, 8, 9, 14)] == ["gemv"] * 4
        assert [G.choose(M, N, K) for M in (15, 16, 32, 64, 65, 2048)] == ["library"] * 6
    assert [G.choose(M, *DOWN) for M in (1, 8, 9, 16)] == ["gemv", "gemv", "library", "library"]  # nine rows of 12,288 do not fit
    assert [G.choose(M, *HEAD) for M in (8, 9, 16, 64, 65)] == ["gemv", "skinny", "skinny", "skinny", "library"]
    assert G.gemv_applies(14, 1, 4096) and not G.gemv_applies(15, 1, 4096)
    assert G.gemv_applies(11, 1, 5120) and not G.gemv_applies(12, 1, 5120)
    assert G.gemv_applies(8, 1, 25600) and not G.gemv_applies(8, 1, 25604) and not G.gemv_applies(17, 1, 64)
    assert G.gemv_partial_rows(8) == 8 and G.gemv_partial_rows(9) == 16
    # a shape that was never measured follows the rule: the streaming kernel up to eight rows only
    assert [G.choose(M, 1000, 1024) for M in (8, 9, 64)] == ["gemv", "library", "library"]
    assert G.choose(8, 1000, 1024, aligned=False) == "library"


def test_gated_products():
    assert [G.choose_gated(M, *GATE_UP) for M in (1, 14, 15, 63, 64, 128, 129, 192, 384, 2048)] == \
        ["gemv", "gemv", "product", "product", "wide", "wide", "product", "pair", "product", "pair"]
    # large weights: the single-block kernel as soon as the streaming kernel no longer takes the rows
    assert [G.choose_gated(M, 34816, 5120) for M in (8, 11, 12, 64, 128, 129, 256)] == ["gemv", "gemv", "wide", "wide", "wide", "product", "pair"]
    assert G.choose_gated(32, 24576 + 8, 4096) == "product"  # halves that are no multiple of 8 rows
    assert G.choose_gated(32, 34816, 5120, aligned=False) == "product"


@pytest.mark.parametrize("forced", ["library", "gemv", "skinny", "wide", "pair"])
def test_a_kernel_can_be_forced_where_it_applies(monkeypatch, forced):
    monkeypatch.setenv("TANDEM_GEMM", forced)
    assert G.choose(16, *DOWN) == ("skinny" if forced == "skinny" else "library")  # the streaming kernel does not take it
    assert G.choose(4, *QKV) == (forced if forced in ("library", "skinny") else "gemv")
    assert G.choose_gated(256, *GATE_UP) == (forced if forced in ("wide", "pair") else "product")
    assert G.choose_gated(4, *GATE_UP) == ("gemv" if forced not in ("library", "skinny") else "product")


def test_the_library_can_be_kept_for_every_product():
    G.keep_library_products()
    try:
        assert G.choose(1, *QKV) == "library" and G.choose(8, *HEAD) == "library"
        assert G.choose_gated(4, *GATE_UP) == "product" and G.choose_gated(2048, *GATE_UP) == "product"
    finally:
        G.keep_library_products(False)
    assert G.choose(1, *QKV) == "gemv"
