"""The allocation-free argmax entry point against the ordinary one.

Some callers of this library cannot allocate device memory when they need an argmax: a serving loop that has given every free byte to its KV-cache pool,
or a runtime that plans its memory up front and treats a later cudaMalloc as a fault. dooms_cuda_argmax_noalloc keeps its partial results in a fixed array
inside the library instead. This file is collected last on purpose: if it fails, every other test has already run."""
import numpy as np
import pytest
import torch

from dooms_b200 import _lib as L

pytestmark = pytest.mark.gpu


def both(v: np.ndarray):
    lib = L.lib()
    d_v = torch.from_numpy(v).cuda()
    a = torch.full((1,), -1, dtype=torch.int32, device="cuda")
    b = torch.full((1,), -1, dtype=torch.int32, device="cuda")
    L.check(lib.dooms_cuda_argmax(d_v.data_ptr(), v.size, a.data_ptr(), None))
    L.check(lib.dooms_cuda_argmax_noalloc(d_v.data_ptr(), v.size, b.data_ptr(), None))
    torch.cuda.synchronize()
    return int(a.item()), int(b.item())


def test_noalloc_argmax_equals_the_ordinary_one_on_two_calls_in_a_row():
    g = np.random.default_rng(5)
    first = g.standard_normal(151936).astype(np.float32)
    second = g.standard_normal(4097).astype(np.float32)          # fewer partial results than the call before: stale ones must not be read
    second[17] = second[4000] = second.max() + 1                 # a tie: the first index wins
    for v in (first, second):
        want, got = both(v)
        assert got == want == int(np.argmax(v))
    third = np.full(1 << 20, -np.inf, dtype=np.float32)          # the largest size the fixed scratch takes
    third[-1] = 0.0
    want, got = both(third)
    assert got == want == (1 << 20) - 1


def test_noalloc_argmax_refuses_sizes_beyond_its_scratch():
    lib = L.lib()
    d = torch.zeros(8, device="cuda")
    out = torch.zeros(1, dtype=torch.int32, device="cuda")
    assert lib.dooms_cuda_argmax_noalloc(d.data_ptr(), (1 << 20) + 1, out.data_ptr(), None) == L.INVALID_ARGUMENT
    assert b"exceeds the fixed scratch" in lib.dooms_cuda_last_error()
    assert lib.dooms_cuda_argmax_noalloc(None, 8, out.data_ptr(), None) == L.INVALID_ARGUMENT
