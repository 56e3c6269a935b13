"""The allocation-free greedy choice, called through its exported C symbol.

Some users of the kernel library cannot allocate device memory at the moment they need a
result: their process gave all of it to its own allocator at start-up, or they are inside a loop
where cudaMalloc would stall the device.  ``mg_argmax_wide_noalloc`` serves them: inputs and
outputs are the caller's, the scratch lives inside the library.  This test owns the tensors it
passes (the test may allocate; the entry point must not need to), calls the symbol twice in a
row on different data, and holds each result to the existing entry point ``mg_argmax_wide``
(exact equality: both pick the lowest index among the largest values).  It also checks that a
request beyond the built-in scratch is refused with a clear message.  The file name makes pytest
collect it last, so a run that stops at the first failure has already run everything else.
"""

from __future__ import annotations

import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu

MAX_PARTS = 8192          # MG_NOALLOC_MAX_PARTS in csrc/no_alloc.h


def _library():
    from mini_gpt_inference_b200.kernels import library

    lib = library.load(verbose=False)
    fn = lib.mg_argmax_wide_noalloc
    fn.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_int,
                   ctypes.c_void_p]
    fn.restype = ctypes.c_int
    return lib, fn


def _existing(lib, logits, limit):
    rows, vocab = logits.shape
    parts = lib.mg_argmax_parts(vocab)
    out = torch.empty(rows, dtype=torch.int32, device=logits.device)
    scratch_v = torch.empty(rows * parts, dtype=torch.float32, device=logits.device)
    scratch_i = torch.empty(rows * parts, dtype=torch.int32, device=logits.device)
    stream = torch.cuda.current_stream().cuda_stream
    assert lib.mg_argmax_wide(logits.data_ptr(), out.data_ptr(), scratch_v.data_ptr(),
                              scratch_i.data_ptr(), rows, vocab, limit, stream) == 0
    return out


def test_no_alloc_argmax_matches_the_existing_entry_point_twice_in_a_row():
    torch.cuda.init()
    torch.empty(1, device="cuda:0")                       # the device's context exists
    lib, fn = _library()
    gen = torch.Generator().manual_seed(0)
    cases = [(8, 50304, 0), (64, 50257, 50000), (3, 509, 0), (1, 2049, 2048)]
    for rows, vocab, limit in cases:
        first = (torch.randn(rows, vocab, generator=gen) * 3).cuda()
        second = (torch.randn(rows, vocab, generator=gen) * 3).cuda()
        second[0, vocab - 1] = 100.0                      # a winner in the last slice
        if rows > 1:
            second[1, 7] = second[1, vocab // 2] = 50.0   # a tie: the lower index wins
        out = torch.full((rows,), -1, dtype=torch.int32, device="cuda:0")
        stream = torch.cuda.current_stream().cuda_stream
        for logits in (first, second):                    # two calls in a row, same scratch
            rc = fn(logits.data_ptr(), out.data_ptr(), rows, vocab, limit, stream)
            assert rc == 0, lib.mg_last_error().decode()
            want = _existing(lib, logits, limit)
            torch.cuda.synchronize()
            assert torch.equal(out, want), (rows, vocab, limit)
            # and to a reference that is no kernel of this library: the largest value among the
            # ids below the limit, the lowest index on ties
            upto = limit if limit > 0 else vocab
            host = logits[:, :upto].cpu()
            top = host.max(dim=1, keepdim=True).values
            lowest = (host == top).int().argmax(dim=1).to(torch.int32)
            assert torch.equal(out.cpu(), lowest), (rows, vocab, limit)
        upto = limit if limit > 0 else vocab
        if upto == vocab:
            assert out[0] == vocab - 1                    # the planted winner of the second call
        if rows > 1:
            assert out[1] == 7                            # the lower index of the planted tie


def test_no_alloc_argmax_refuses_more_than_its_scratch_holds():
    lib, fn = _library()
    rows, vocab = 400, 50304                              # 400 * 25 slices > 8192
    assert rows * ((vocab + 2047) // 2048) > MAX_PARTS
    logits = torch.zeros(rows, vocab, device="cuda:0")
    out = torch.full((rows,), -7, dtype=torch.int32, device="cuda:0")
    rc = fn(logits.data_ptr(), out.data_ptr(), rows, vocab, 0, torch.cuda.current_stream().cuda_stream)
    assert rc != 0
    message = lib.mg_last_error().decode()
    assert "exceeds the built-in scratch" in message and str(MAX_PARTS) in message
    torch.cuda.synchronize()
    assert (out == -7).all()                              # nothing ran
