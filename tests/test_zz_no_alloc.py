"""The allocation-free rescale entry point must give exactly what the regular one gives.

It exists for callers that cannot allocate device memory while they run (for example while a
CUDA graph is being captured, or under a fixed memory budget): its scratch is a fixed array
inside the library.  Collected last on purpose, so an early-exit run has already seen every
other test."""
import ctypes as C

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def test_rescale_no_alloc_matches_rescale_twice_in_a_row():
    import torch

    if not torch.cuda.is_available():
        pytest.fail("GPU tests need a CUDA device; there is no CPU fallback")
    from lancelot_b200 import cabi
    from lancelot_b200._lib import InvalidArgument, check, lib

    lib.lb_rescale_no_alloc_max_words.restype = C.c_size_t
    logn, n, L = 13, 1 << 13, 3
    mods = cabi.coeff_modulus_create(n, [60, 40, 40, 60])
    ctx = cabi.Context(logn, mods, 1)
    from oracle import binding
    oracle = binding.Oracle(logn, mods, 1)
    rng = np.random.default_rng(99)
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    for call in range(2):  # the second call reuses the array the first one left dirty
        ct = np.stack([rng.integers(0, mods[r % L], n, dtype=np.uint64) for r in range(3 * L)]).reshape(3, L, n)
        d = cabi.to_device(ct)
        want = cabi.to_host(ctx.rescale(L, d))
        out = ctx.empty(3, L - 1, n)
        check(lib.lb_rescale_no_alloc(ctx.h, L, 3, C.c_void_p(d.data_ptr()), C.c_void_p(out.data_ptr()), stream))
        torch.cuda.synchronize()
        assert np.array_equal(cabi.to_host(out), want), "call %d differs from lb_rescale" % call
        assert np.array_equal(want, oracle.rescale(L, ct)), "call %d differs from the CPU checker" % call
    # beyond the fixed scratch: refused with a clear message, nothing launched
    too_many = int(lib.lb_rescale_no_alloc_max_words()) // n + 1
    big = ctx.empty(too_many, L, n)
    with pytest.raises(InvalidArgument, match="static scratch"):
        check(lib.lb_rescale_no_alloc(ctx.h, L, too_many, C.c_void_p(big.data_ptr()), C.c_void_p(big.data_ptr()), stream))
