"""The allocation-free sampling entry point, called through its exported C symbol.

Some callers of this library cannot allocate device memory when they ask for a
token (they run where cudaMalloc is forbidden, or under a memory budget fixed at
start-up, or must stay out of torch's allocator).  ``pllm_sample_static`` serves
them: the scratch memory that sampling needs between its two launches lives in
a fixed array inside the library.  This test calls it twice in a row on
different logits and expects exactly the tokens of the ordinary entry point
(``pllm_sample``, scratch from the caller), which the other tests check against
the plain implementation; the same kernels run, so the tolerance is equality.
It also checks that requests beyond the stated limits are refused.

Collected last (the file name sorts after every other test file).
"""

import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def test_static_sampling_matches_the_ordinary_entry_point_twice_in_a_row():
    from paged_llm_rs_b200.csrc.build import load_library

    L = load_library()
    P, I = ctypes.c_void_p, ctypes.c_int
    static = L.pllm_sample_static
    static.argtypes = [P, I, I, ctypes.c_longlong, P, P, P, P]
    static.restype = I
    ordinary = L.pllm_sample
    ordinary.argtypes = [P, I, I, ctypes.c_longlong, P, P, P, P, P]
    ordinary.restype = I
    scratch_floats = L.pllm_sample_scratch_floats
    scratch_floats.argtypes = [I, I]
    scratch_floats.restype = ctypes.c_longlong

    dev = "cuda:0"
    torch.cuda.set_device(0)
    stream = torch.cuda.current_stream().cuda_stream
    g = torch.Generator(device=dev).manual_seed(11)
    for call, (rows, vocab) in enumerate([(7, 151936), (64, 50001)]):     # two calls in a row, other shapes
        logits = torch.randn(rows, vocab, device=dev, generator=g) * 3
        temp = torch.rand(rows, device=dev, generator=g) + 0.2
        temp[::3] = 0.0                                                   # some rows greedy
        uni = torch.rand(rows, device=dev, generator=g)
        got = torch.full((rows,), -1, dtype=torch.int32, device=dev)
        want = torch.full((rows,), -2, dtype=torch.int32, device=dev)
        scratch = torch.empty(scratch_floats(rows, vocab), dtype=torch.float32, device=dev)
        assert ordinary(logits.data_ptr(), rows, vocab, logits.stride(0), temp.data_ptr(), uni.data_ptr(),
                        want.data_ptr(), scratch.data_ptr(), stream) == 0
        assert static(logits.data_ptr(), rows, vocab, logits.stride(0), temp.data_ptr(), uni.data_ptr(),
                      got.data_ptr(), stream) == 0
        torch.cuda.synchronize()
        assert torch.equal(got, want), call
        assert (got[::3].cpu() == logits[::3].argmax(-1).cpu().int()).all()

    # beyond the limits: refused, nothing launched, the output untouched
    tokens = torch.full((65,), -7, dtype=torch.int32, device=dev)
    small = torch.zeros(65, 8, device=dev)
    z = torch.zeros(65, device=dev)
    assert static(small.data_ptr(), 65, 8, 8, z.data_ptr(), z.data_ptr(), tokens.data_ptr(), stream) == -4
    assert static(small.data_ptr(), 1, (1 << 20) + 1, 8, z.data_ptr(), z.data_ptr(), tokens.data_ptr(), stream) == -4
    torch.cuda.synchronize()
    assert (tokens == -7).all()
