"""GPU: the allocation-free sort entry point against the ordinary one and against numpy's stable sort.

``ks_sort_pairs_u32_noalloc`` exists for callers that cannot let this library allocate on the device (a plugin inside a
serving process whose allocator owns the whole GPU, a thread that must not block on the allocator).  Its scratch is a
fixed array inside the library that every call reuses, so the test sorts twice in a row with different sizes and data:
the second result must not depend on what the first call left behind.  Runs last (file name) so that a failure here
cannot hide the other tests in a stop-at-first-failure run.
"""
import ctypes

import numpy as np
import pytest

from kernel_scheduling_b200 import _lib

pytestmark = pytest.mark.gpu


def _sorted_by_noalloc(lib, torch, keys, vals, begin_bit, end_bit):
    dk = torch.from_numpy(keys.view(np.int32)).cuda()
    dv = torch.from_numpy(vals.view(np.int32)).cuda() if vals is not None else None
    torch.cuda.synchronize()
    stream = torch.cuda.current_stream().cuda_stream
    r = lib.ks_sort_pairs_u32_noalloc(ctypes.c_void_p(stream), ctypes.c_void_p(dk.data_ptr()), ctypes.c_void_p(dv.data_ptr()) if dv is not None else None,
                                      len(keys), begin_bit, end_bit)
    assert r == len(keys), lib.ks_last_error(None)
    return dk.cpu().numpy().view(np.uint32), (dv.cpu().numpy().view(np.uint32) if dv is not None else None)


def test_noalloc_sort_matches_the_handle_based_sort(builder):
    import torch

    lib = _lib.load()
    rng = np.random.default_rng(21)
    cases = [(700_001, 0, 32, True), (123_457, 3, 19, True), (4096, 0, 8, False), (1 << 20, 0, 24, True), (1, 0, 32, True)]
    for n, b0, b1, with_vals in cases:  # back to back: each call finds the previous call's leftovers in the scratch
        keys = rng.integers(0, 1 << 32, n, dtype=np.uint64).astype(np.uint32)
        vals = np.arange(n, dtype=np.uint32) if with_vals else None
        want_k, want_v = builder.sort_pairs(keys, vals, b0, b1)
        got_k, got_v = _sorted_by_noalloc(lib, torch, keys, vals, b0, b1)
        assert np.array_equal(got_k, want_k), (n, b0, b1)
        if with_vals:
            assert np.array_equal(got_v, want_v), (n, b0, b1)
        # ... and against numpy directly (both entry points run the same kernels): a stable sort on the chosen key bits
        digit = (keys >> np.uint32(b0)) & np.uint32((1 << (b1 - b0)) - 1) if b1 - b0 < 32 else keys
        order = np.argsort(digit, kind="stable")
        assert np.array_equal(got_k, keys[order]), (n, b0, b1)
        if with_vals:
            assert np.array_equal(got_v, vals[order]), (n, b0, b1)


def test_noalloc_sort_refuses_what_does_not_fit():
    import torch

    lib = _lib.load()
    d = torch.zeros(8, dtype=torch.int32, device="cuda")
    r = lib.ks_sort_pairs_u32_noalloc(None, ctypes.c_void_p(d.data_ptr()), None, (1 << 20) + 1, 0, 32)
    assert r == -_lib.ERR_TOO_LARGE
    assert b"at most" in lib.ks_last_error(None)
    assert lib.ks_sort_pairs_u32_noalloc(None, ctypes.c_void_p(d.data_ptr()), None, 8, 5, 40) == -_lib.ERR_ARG
