"""The allocation-free greedy selection (csrc/no_alloc.h), called through its exported C
symbol the way a C host would call it, against the ordinary entry point.

Some hosts of the kernel library cannot allocate device memory when they need a token: a
server that gave the whole GPU to its cache pool, a loop that cannot afford cudaMalloc's
device synchronisation, a C caller without a caching allocator.  For them the library
keeps the reduction's piece buffers in a fixed 512 KiB array of its own.  This test checks
that the variant returns exactly what the ordinary one returns, twice in a row (the second
call finds the first call's leftovers in the shared array), that it refuses requests beyond
its stated limit, and that it asks the CUDA runtime for no memory.

Collected last on purpose (file name): a run that stops at the first failure has then
already run every other test.
"""
import ctypes

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def library():
    from coheryn_ai_studio_b200.csrc import build
    lib = build.core_library()
    lib.coheryn_last_error.restype = ctypes.c_char_p
    lib.coheryn_argmax_static.restype = ctypes.c_int
    lib.coheryn_argmax_static.argtypes = [ctypes.c_void_p, ctypes.c_long, ctypes.c_int, ctypes.c_int,
                                          ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p]
    return lib


def test_static_argmax_matches_the_ordinary_entry_point_twice():
    from coheryn_ai_studio_b200 import ops
    lib = library()
    dev = torch.device("cuda:0")
    rng = np.random.default_rng(7)
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    # two calls in a row of different shapes: the second starts from the first one's leftovers
    for rows, vocab in [(9, 151936), (64, 1000), (3, 151936)]:
        x = rng.standard_normal((rows, vocab)).astype(np.float32)
        x[0, 5] = x[0, vocab - 1] = 50.0                  # a tie across pieces: the lowest id wins
        logits = torch.from_numpy(x).to(dev)
        want = torch.empty(rows, dtype=torch.int32, device=dev)
        ops.argmax(logits, want, status)                  # the ordinary entry point (allocates its pieces)
        got = torch.full((rows,), -1, dtype=torch.int32, device=dev)
        torch.cuda.synchronize()
        before = torch.cuda.memory_allocated(dev)
        rc = lib.coheryn_argmax_static(logits.data_ptr(), logits.stride(0), rows, vocab, got.data_ptr(),
                                       status.data_ptr(), stream)
        assert rc == 0, lib.coheryn_last_error().decode()
        torch.cuda.synchronize()
        assert torch.cuda.memory_allocated(dev) == before
        assert torch.equal(got, want)                      # bit-identical choice (tolerance zero)
        assert got[0].item() == 5 and status.item() == 0


def test_static_argmax_refuses_what_does_not_fit():
    lib = library()
    dev = torch.device("cuda:0")
    logits = torch.zeros(2, 8, device=dev)
    out = torch.zeros(2, dtype=torch.int32, device=dev)
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    # 2,000 rows of 151,936 logits would need 76,000 slots; the array has 65,536
    rc = lib.coheryn_argmax_static(logits.data_ptr(), 151936, 2000, 151936, out.data_ptr(), status.data_ptr(), stream)
    assert rc != 0 and b"static scratch holds 65536" in lib.coheryn_last_error()
    torch.cuda.synchronize()
    # 65,536 rows of a small vocabulary fit the slots but not the launch grid: refused as well
    rc = lib.coheryn_argmax_static(logits.data_ptr(), 8, 65536, 8, out.data_ptr(), status.data_ptr(), stream)
    assert rc != 0 and b"at most 65535 rows" in lib.coheryn_last_error()
    torch.cuda.synchronize()
