"""The allocation-free argmax entry point, called through its exported C symbol.

Some users of the kernel library cannot allocate device memory when they call it (a host program
without a tensor library and with a fixed memory plan; code running while a stream is being captured),
so ``pb_argmax_noalloc`` keeps its scratch in an array built into the library.  The test calls the symbol
with raw pointers, the way such a caller would, twice in a row on different inputs - the second call finds
the first call's leftovers in the shared array - and compares with the ordinary entry point.

The file sorts last so that a run that stops at the first failure has run every other test before it.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _symbol():
    from prelude_b200.csrc import build
    lib = ctypes.CDLL(build.build())
    fn = lib.pb_argmax_noalloc
    fn.argtypes = [ctypes.c_void_p, ctypes.c_longlong, ctypes.c_int, ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p]
    fn.restype = ctypes.c_int
    lib.pb_last_error.restype = ctypes.c_char_p
    return lib, fn


@pytest.mark.parametrize("rows,vocab", [(1, 7), (8, 151936), (64, 5000), (256, 331)])
def test_noalloc_argmax_matches_the_ordinary_entry_point_twice_in_a_row(rows, vocab):
    from prelude_b200.ops import kernels as K
    lib, fn = _symbol()
    torch.cuda.init()
    stream = torch.cuda.current_stream().cuda_stream
    for call in range(2):                                   # the second call meets the first call's scratch contents
        g = torch.Generator(device="cpu").manual_seed(100 * call + rows)
        logits = torch.randn(rows, vocab + 5, generator=g).cuda()[:, :vocab]     # rows of a wider tensor
        logits[0, vocab // 2] = 60.0
        logits[0, vocab - 1] = 60.0                          # a tie: the smaller index wins
        want = K.argmax(logits)                              # the existing entry point (allocates its scratch with torch)
        out = torch.full((rows,), -1, dtype=torch.int32, device="cuda")
        # nothing is taken from torch's allocator either: its count of allocations ever made does not move
        # (the bytes in use may, whenever Python frees another test's tensors)
        before = torch.cuda.memory_stats()["allocation.all.allocated"]
        rc = fn(logits.data_ptr(), logits.stride(0), rows, vocab, out.data_ptr(), stream)
        assert rc == 0, lib.pb_last_error()
        assert torch.cuda.memory_stats()["allocation.all.allocated"] == before
        torch.cuda.synchronize()
        assert torch.equal(out, want) and int(out[0]) == vocab // 2
        assert out.tolist() == torch.argmax(logits, -1).tolist()


def test_noalloc_argmax_refuses_more_rows_than_its_scratch_holds():
    lib, fn = _symbol()
    logits = torch.zeros(257, 16, device="cuda")
    out = torch.zeros(257, dtype=torch.int32, device="cuda")
    rc = fn(logits.data_ptr(), 16, 257, 16, out.data_ptr(), torch.cuda.current_stream().cuda_stream)
    assert rc != 0 and b"256 rows" in lib.pb_last_error()
