"""The allocation-free column sum (akgb_reduce_sum_axis0_f32_noalloc), called through the C ABI.

It serves callers that cannot allocate device memory at the call site (memory-planned regions, an
exhausted or closing allocator, latency-critical loops): its partial sums live in an array built into
the library.  Checked here against the regular entry point (akgb_launch with a workspace) on two calls
in a row with different data and shapes — the second call finds the first call's partials in the shared
array and must not be affected by them — and for its size limit.

This file sorts last on purpose: a run that stops at the first failure has then already run every
other test.
"""
import ctypes

import numpy as np
import pytest

from akg_b200 import FusedKernel, _capi, descs

pytestmark = pytest.mark.gpu


def _reference(x):
    import torch
    k = FusedKernel(descs.reduce_sum_axis0(x.shape[0], x.shape[1]))
    out = torch.empty(x.shape[1], dtype=torch.float32, device="cuda")
    k.launch([x, out])
    torch.cuda.synchronize()
    return out


def _noalloc(lib, x):
    import torch
    out = torch.full((x.shape[1],), float("nan"), dtype=torch.float32, device="cuda")
    st = lib.akgb_reduce_sum_axis0_f32_noalloc(ctypes.c_void_p(x.data_ptr()), ctypes.c_void_p(out.data_ptr()),
                                               x.shape[0], x.shape[1],
                                               ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
    assert st == _capi.AKGB_OK, lib.akgb_last_error()
    torch.cuda.synchronize()
    return out


def test_two_calls_in_a_row_match_the_workspace_entry_point(lib):
    import torch
    g = torch.Generator(device="cuda")
    g.manual_seed(1234)
    # first call: large values, many splits, so the shared array is left full of big partials
    x1 = torch.randn((8192, 4096), generator=g, device="cuda", dtype=torch.float32) * 1000.0
    # second call: a different shape with small values; stale partials would show at once
    x2 = torch.randn((3000, 1000), generator=g, device="cuda", dtype=torch.float32) * 1e-3
    for x in (x1, x2):
        got = _noalloc(lib, x)
        want = _reference(x)
        assert torch.equal(got, want)  # same kernels, same split: bit-identical
        truth = x.double().sum(dim=0)
        bound = 1e-5 * x.abs().double().sum(dim=0)
        assert bool(((got.double() - truth).abs() <= bound).all())
    # and once more on the first input, after the small one
    assert torch.equal(_noalloc(lib, x1), _reference(x1))


def test_sizes_beyond_the_built_in_scratch_are_rejected(lib):
    import torch
    cols = 65536 + 8  # one vector beyond the documented maximum width
    x = torch.zeros((64, cols), dtype=torch.float32, device="cuda")
    out = torch.empty(cols, dtype=torch.float32, device="cuda")
    st = lib.akgb_reduce_sum_axis0_f32_noalloc(ctypes.c_void_p(x.data_ptr()), ctypes.c_void_p(out.data_ptr()), 64, cols,
                                               None)
    assert st == _capi.AKGB_TOO_LARGE
    assert b"scratch" in lib.akgb_last_error()
    st = lib.akgb_reduce_sum_axis0_f32_noalloc(None, ctypes.c_void_p(out.data_ptr()), 64, cols, None)
    assert st == _capi.AKGB_INVALID_ARG
    # the widest accepted input still works
    xw = torch.ones((40, 65536), dtype=torch.float32, device="cuda")
    assert torch.equal(_noalloc(lib, xw), torch.full((65536,), 40.0, device="cuda"))
