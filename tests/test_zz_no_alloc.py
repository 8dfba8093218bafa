"""The allocation-free GroupNorm statistics entry point, called through the C ABI.

It exists for hosts that cannot give the library scratch memory at call time
(all device memory reserved up front, or operator callbacks in which cudaMalloc
is forbidden); its scratch is an array built into the shared library.  The test
checks it against the regular entry point (caller-owned scratch) on two calls in
a row, because the built-in array keeps whatever the previous call left in it.
Collected last on purpose: a failure here cannot hide any other test's result.
"""
import ctypes as C

import pytest
import torch

from tests._util import assert_close, cuda_or_skip

pytestmark = pytest.mark.gpu


def _stats_noalloc(l, _lib, x, groups):
    B, H, W, Ci = x.shape
    out = torch.empty((2, B, groups), device=x.device, dtype=torch.float32)
    rc = l.bxl_groupnorm_stats_noalloc_f16(x.data_ptr(), x.stride(0), B, H * W, Ci, groups, out.data_ptr(),
                                            torch.cuda.current_stream().cuda_stream)
    _lib.check(rc, l)
    return out


def test_noalloc_stats_match_regular_entry_point_twice():
    dev = cuda_or_skip()
    from basedxl_b200 import _lib, ops

    l = _lib.lib()
    g = torch.Generator().manual_seed(0)
    xs = [
        (torch.randn(2, 32, 32, 1280, generator=g) * 2 + 0.5).half().to(dev),   # the benchmark GroupNorm shape
        (torch.randn(1, 16, 128, 320, generator=g) - 1.0).half().to(dev),        # a different shape reusing the same array
    ]
    for x in xs:  # two calls in a row on the shared built-in array
        expected = ops.groupnorm_stats(x, 32)
        got = _stats_noalloc(l, _lib, x, 32)
        torch.cuda.synchronize()
        assert_close(got, expected.float().cpu(), tol=1e-3, what="no-alloc groupnorm moments")
    # and once more on the first input: the previous call's leftovers must not matter
    assert_close(_stats_noalloc(l, _lib, xs[0], 32), ops.groupnorm_stats(xs[0], 32).float().cpu(), tol=1e-3)
    _lib.device_status()


def test_noalloc_rejects_sizes_beyond_the_builtin_scratch():
    dev = cuda_or_skip()
    from basedxl_b200 import _lib

    l = _lib.lib()
    limit = l.bxl_groupnorm_stats_noalloc_max_bg()
    groups = 32
    B = limit // groups + 1
    x = torch.zeros(B, 2, 2, 64, device=dev, dtype=torch.float16)
    out = torch.empty((2, B, groups), device=dev, dtype=torch.float32)
    rc = l.bxl_groupnorm_stats_noalloc_f16(x.data_ptr(), x.stride(0), B, 4, 64, groups, out.data_ptr(),
                                            torch.cuda.current_stream().cuda_stream)
    assert rc != 0
    assert b"exceeds the built-in scratch" in l.bxl_last_error()
