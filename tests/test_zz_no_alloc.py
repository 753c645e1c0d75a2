"""tb_argmax_static, the argmax entry point that allocates nothing, called the way a program
without this package's Python layer would call it: through its exported C symbol, with raw device
pointers.  Its result must equal that of the regular entry points on two calls in a row (the
scratch inside the library is shared by all calls), and sizes beyond its limit must be refused.
This file sorts last so that a run stopping at the first failure has run every other test before."""

import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu

MAX_ROWS = 4096
TOO_LARGE = 10003


def entry_point():
    from tandem_b200.kernels.build import compile_library

    lib = ctypes.CDLL(compile_library("sampling"))
    fn = lib.tb_argmax_static
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_int]
    return fn


def test_argmax_static_matches_the_regular_entry_points_twice_in_a_row():
    from tandem_b200.kernels import ops

    fn = entry_point()
    stream = torch.cuda.current_stream().cuda_stream
    g = torch.Generator().manual_seed(0)
    for call, (R, V, chunks) in enumerate([(8, 151936, 37), (8, 151936, 37), (64, 50000, 4), (3, 777, 1), (MAX_ROWS, 4100, 2)]):
        logits = torch.randn(R, V, generator=g).cuda()
        logits[0, V // 3] = logits[0, V - 1] = 50.0  # equal maxima: the lowest index wins
        out = torch.full((R,), -7, dtype=torch.int32, device="cuda")
        assert fn(stream, logits.data_ptr(), out.data_ptr(), R, V, chunks) == 0
        want = ops.argmax(logits)  # the existing entry points (tb_argmax / tb_argmax_split)
        torch.cuda.synchronize()
        assert torch.equal(out, want), call
        assert out.tolist() == logits.argmax(-1).tolist() and int(out[0]) == V // 3


def test_argmax_static_refuses_what_it_cannot_hold():
    fn = entry_point()
    stream = torch.cuda.current_stream().cuda_stream
    logits = torch.zeros(MAX_ROWS + 1, 8, device="cuda")
    out = torch.full((MAX_ROWS + 1,), -7, dtype=torch.int32, device="cuda")
    assert fn(stream, logits.data_ptr(), out.data_ptr(), MAX_ROWS + 1, 8, 1) == TOO_LARGE
    assert fn(stream, logits.data_ptr(), out.data_ptr(), 4, 0, 1) == 10002
    torch.cuda.synchronize()
    assert bool((out == -7).all())  # nothing ran
