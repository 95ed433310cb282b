"""The allocation-free arg max, called through its exported C symbol.

``mls_argmax_static`` serves callers that cannot allocate device memory when they
need a token (a memory budget fixed at start-up, a loop that must not touch the
allocator, a host without PyTorch's allocator to borrow scratch memory from).  Its
scratch memory is an array inside the library image.  The test calls it twice in
a row on different logits, with nothing in between that would reset the shared
array, and compares each result with the existing entry point (``mls_sample`` with
no temperatures), which gets its scratch memory from the caller.  It also checks
that a request beyond the array's size is refused.  The file sorts last so that a
run that stops at the first failure has run every other test before.
"""

import ctypes

import pytest
import torch

from mini_llm_stack_b200.ops import library
from mini_llm_stack_b200.ops.kernels import Runtime

pytestmark = pytest.mark.gpu
TOO_LARGE = 100003


def _entry():
    lib = library.load("argmax_static")
    fn = lib.mls_argmax_static
    fn.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_void_p]
    fn.restype = ctypes.c_int
    return fn


def test_static_argmax_matches_the_allocating_entry_point_twice_in_a_row():
    dev = torch.device("cuda:0")
    torch.cuda.set_device(dev)
    fn = _entry()
    ops = Runtime(dev, torch.float32).ops
    stream = torch.cuda.current_stream(dev).cuda_stream
    gen = torch.Generator().manual_seed(123)
    for call, (rows, vocab) in enumerate([(7, 128256), (64, 50257)]):
        logits = (torch.randn((rows, vocab), generator=gen) * 3).to(dev)
        logits[1, 5] = logits[1, vocab - 3] = logits[1].max() + 2        # a tie: index 5 wins
        logits[2, vocab - 1] = logits[2].max() + 1                       # the very last logit
        want = torch.empty(rows, dtype=torch.int32, device=dev)
        ops.sample(logits, None, None, want)
        got = torch.full((rows,), -1, dtype=torch.int32, device=dev)
        rc = fn(logits.data_ptr(), got.data_ptr(), rows, vocab, stream)
        assert rc == 0, f"call {call}: mls_argmax_static returned {rc}"
        torch.cuda.synchronize()
        assert torch.equal(got, want), f"call {call}"
        assert got.tolist() == [int(torch.argmax(r)) for r in logits.cpu()]
        assert got[1].item() == 5 and got[2].item() == vocab - 1


def test_static_argmax_refuses_more_than_its_array_holds():
    dev = torch.device("cuda:0")
    torch.cuda.set_device(dev)
    fn = _entry()
    stream = torch.cuda.current_stream(dev).cuda_stream
    rows, vocab = 1025, 65536                      # 1025 * 16 pairs > 16384
    logits = torch.zeros((rows, vocab), device=dev)
    out = torch.full((rows,), -7, dtype=torch.int32, device=dev)
    assert fn(logits.data_ptr(), out.data_ptr(), rows, vocab, stream) == TOO_LARGE
    torch.cuda.synchronize()
    assert bool((out == -7).all())                 # nothing was launched
    assert fn(logits.data_ptr(), out.data_ptr(), 1024, vocab, stream) == 0
    torch.cuda.synchronize()
    assert bool((out[:1024] == 0).all())           # all equal: the lowest index
