"""The sampling entry point that allocates nothing (csrc/kernels/sample_no_alloc.h), called through its
exported C symbol, against the ordinary sampling entry point (GPU).

It serves callers that cannot ask CUDA for memory while they pick tokens: a serving loop that gave all
free device memory to the cache, a thread that must not trigger the device-wide synchronisation of an
allocation, a host program that links the library without an allocator of its own.  Its scratch is a
fixed array inside the library, shared by all calls, so the test makes two calls in a row and expects
both to be right although the second one finds what the first one left."""
import ctypes
from ctypes import c_int, c_void_p

import pytest
import torch

pytestmark = pytest.mark.gpu


def test_no_alloc_sampling_matches_the_ordinary_entry_point_twice():
    from cbis_b200.kernels import library, ops
    from cbis_b200.sampling import request_key
    lib = ctypes.CDLL(library.build_kernels())
    fn = lib.cbis_sample_no_alloc
    fn.restype = c_int
    stream = c_void_p(torch.cuda.current_stream().cuda_stream)
    g = torch.Generator().manual_seed(123)
    for call, (R, V) in enumerate([(7, 50257), (64, 50257), (3, 317), (256, 9000)]):
        logits = torch.randn(R, V, generator=g).cuda()
        logits[0, V // 3] = logits[0, V - 1] = 40.0                       # a tie: the first maximum wins
        temps = torch.tensor([0.0 if r % 3 == 0 else 0.5 + 0.1 * (r % 7) for r in range(R)], device="cuda")
        keys = torch.tensor([request_key(5, r, call) for r in range(R)], dtype=torch.int64, device="cuda")
        want = torch.empty(R, dtype=torch.int32, device="cuda")
        ops.sample(logits, temps, keys, want)                             # the existing entry point
        for again in range(2):                                            # two calls in a row share the scratch
            got = torch.full((R,), -1, dtype=torch.int32, device="cuda")
            st = fn(c_void_p(logits.data_ptr()), c_int(logits.stride(0)), c_void_p(temps.data_ptr()),
                    c_void_p(keys.data_ptr()), c_void_p(got.data_ptr()), c_int(R), c_int(V), stream)
            assert st == 0
            assert torch.equal(got.cpu(), want.cpu()), (R, V, again)
        greedy = torch.empty(R, dtype=torch.int32, device="cuda")
        st = fn(c_void_p(logits.data_ptr()), c_int(logits.stride(0)), None, None, c_void_p(greedy.data_ptr()),
                c_int(R), c_int(V), stream)
        ops.sample(logits, None, None, want)
        assert st == 0 and greedy[0].item() == V // 3 and torch.equal(greedy.cpu(), want.cpu())


def test_no_alloc_sampling_refuses_more_rows_than_its_scratch_holds():
    from cbis_b200.kernels import library
    lib = ctypes.CDLL(library.build_kernels())
    logits = torch.zeros(257, 8, device="cuda")
    out = torch.full((257,), -7, dtype=torch.int32, device="cuda")
    st = lib.cbis_sample_no_alloc(c_void_p(logits.data_ptr()), c_int(8), None, None, c_void_p(out.data_ptr()),
                                  c_int(257), c_int(8), c_void_p(torch.cuda.current_stream().cuda_stream))
    assert st == -4                                                        # CBIS_ERR_TOO_LARGE, nothing launched
    torch.cuda.synchronize()
    assert (out == -7).all()
