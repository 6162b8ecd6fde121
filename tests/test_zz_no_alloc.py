"""The entry point that allocates nothing (csrc/no_alloc.h), called through its
exported C symbol, against the ordinary entry point, twice in a row.

It is for callers that cannot get device memory when they need a token chosen:
a host thread with a latency bound (an allocation may lock and synchronise), a
process whose device memory all belongs to another allocator, code inside a
callback whose contract forbids allocating.  This file is named to be
collected last: if it fails, a run that stops at the first failure has already
run every other test.
"""

import ctypes

import pytest
import torch

from flashdecode_cuda_b200 import kernels as K

pytestmark = pytest.mark.gpu


def symbol():
    fn = K.lib().fd_sample_no_alloc
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p,
                   ctypes.c_ulonglong, ctypes.c_void_p, ctypes.c_void_p]
    return fn


def call(fn, logits, out, temp=None, req=None, step=None, seed=0):
    ptr = lambda t: None if t is None else t.data_ptr()
    n, V = logits.shape
    return fn(ptr(logits), n, V, ptr(temp), ptr(req), ptr(step), seed, ptr(out),
              torch.cuda.current_stream().cuda_stream)


@pytest.mark.parametrize("V", [333, 151936])
def test_same_tokens_as_the_ordinary_entry_point_twice_in_a_row(V):
    fn = symbol()
    g = torch.Generator().manual_seed(V)
    for round_ in range(2):                       # the second call finds the first call's leftovers in the array
        n = 9 if round_ == 0 else 4               # ... laid out for another row count
        logits = torch.randn(n, V, generator=g).cuda()
        logits[1] = 0.5                           # all tied: the lowest index
        temp = torch.tensor([0.0, 0.0, 0.7, 1.5, 0.0, 0.9, 0.0, 2.0, 0.3][:n]).cuda()
        req = torch.arange(100, 100 + n, dtype=torch.int64).cuda()
        step = torch.arange(n, dtype=torch.int32).cuda() + round_
        want_g = torch.empty(n, dtype=torch.int32, device="cuda")
        want_t = torch.empty_like(want_g)
        K.sample(logits, want_g)
        K.sample(logits, want_t, temp, req, step, seed=2 ** 40 + 3)
        got_g = torch.full_like(want_g, -1)
        got_t = torch.full_like(want_g, -1)
        assert call(fn, logits, got_g) == 0
        assert call(fn, logits, got_t, temp, req, step, seed=2 ** 40 + 3) == 0
        torch.cuda.synchronize()
        assert got_g.tolist() == want_g.tolist()            # token ids: equal, no tolerance needed
        assert got_t.tolist() == want_t.tolist()
        assert got_g[1].item() == 0


def test_sizes_beyond_the_static_array_are_refused():
    fn = symbol()
    out = torch.zeros(300, dtype=torch.int32, device="cuda")
    assert call(fn, torch.zeros(257, 8, device="cuda"), out) != 0
    assert b"at most 256" in K.lib().fd_last_error()
    wide = torch.zeros(1, 64 * 4096 + 1, device="cuda")
    assert call(fn, wide, out) != 0
    assert b"262144" in K.lib().fd_last_error()
    assert call(fn, torch.zeros(1, 64 * 4096, device="cuda"), out) == 0
    torch.cuda.synchronize()
