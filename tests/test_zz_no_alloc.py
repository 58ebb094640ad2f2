"""The allocation-free reduce (`mimk_reduce_static`) against the ordinary `mimk_reduce`, through the C ABI.

Some users of the library may not let it allocate: an embedder that has planned all device memory up front (a
fixed budget, or its own allocator that a hidden cudaMalloc would go around), or a latency-critical loop that cannot
afford the device-wide stall an allocation can cause.  For them the split-axis reduction keeps its partial results
in a 1 MiB array that is part of the library image.  This file is collected last on purpose, so a failure here never
hides another test's result, and it must pass both on its own in a fresh process and after every other test.
"""
import ctypes as C

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _reduce(fn, x, outer, ln, inner, monoid):
    out = torch.full((outer, inner), float("nan"), device="cuda")
    st = fn(x.data_ptr(), out.data_ptr(), 0, outer, ln, inner, monoid, torch.cuda.current_stream().cuda_stream)
    assert st == 0, st
    torch.cuda.synchronize()
    return out


def test_static_reduce_matches_reduce_twice_in_a_row():
    from mimir_b200 import _lib
    L = _lib.lib()
    g = torch.Generator(device="cpu").manual_seed(77)
    # two calls in a row whose plans both split the reduced axis (partials in the static array), with different
    # shapes and monoids so that the second call meets the first call's leftovers in the array
    cases = [(1, 20000, 96, _lib.SUM), (3, 4096, 40, _lib.MAX), (2, 9000, 7, _lib.SUM), (1, 300, 513, _lib.MIN)]
    for outer, ln, inner, monoid in cases:
        x = torch.randn((outer, ln, inner), generator=g).cuda()
        want = _reduce(L.mimk_reduce, x, outer, ln, inner, monoid)
        got = _reduce(L.mimk_reduce_static, x, outer, ln, inner, monoid)
        assert torch.equal(got, want)        # one plan, the same kernels: the same bits
        if monoid == _lib.SUM:
            # and the tolerance of the reduce tests against f64: 1e-6 of the largest absolute partial sum
            scale = float(x.double().abs().sum(dim=1).max())
            ref = x.double().sum(dim=1)
            assert float((got.double() - ref).abs().max()) <= 1e-6 * scale + 1e-6
    # the property the entry point exists for: once the first call on this device has resolved the array's address,
    # further calls -- split plans included -- leave the device's free memory exactly where it was (outputs are
    # allocated beforehand; torch's caching allocator is not involved in the calls themselves)
    x = torch.randn((1, 20000, 96), generator=g).cuda()
    out = torch.empty((1, 96), device="cuda")
    n = C.c_int64(0)
    assert L.mimk_reduce_plan(1, 20000, 96, torch.cuda.get_device_properties(0).multi_processor_count, C.byref(n)) == 0
    assert n.value > 0                                   # this shape does use the static partials
    stream = torch.cuda.current_stream().cuda_stream
    torch.cuda.synchronize()
    free0 = torch.cuda.mem_get_info()[0]
    for monoid in (_lib.SUM, _lib.MAX, _lib.SUM):
        assert L.mimk_reduce_static(x.data_ptr(), out.data_ptr(), 0, 1, 20000, 96, monoid, stream) == 0
    torch.cuda.synchronize()
    assert torch.cuda.mem_get_info()[0] == free0
    # inner == 1 (row reduce) and a degenerate axis go through the same entry point without touching the array
    x = torch.randn((50, 1000), generator=g).cuda()
    assert torch.equal(_reduce(L.mimk_reduce_static, x, 50, 1000, 1, _lib.SUM), _reduce(L.mimk_reduce, x, 50, 1000, 1, _lib.SUM))
    out = torch.full((4,), 7.0, device="cuda")
    assert L.mimk_reduce_static(None, out.data_ptr(), 0, 4, 0, 1, _lib.SUM, None) == 0
    torch.cuda.synchronize()
    assert torch.equal(out, torch.zeros(4, device="cuda"))


def test_static_reduce_validates_like_reduce():
    from mimir_b200 import _lib
    L = _lib.lib()
    assert L.mimk_reduce_static(None, None, 0, -1, 4, 1, _lib.SUM, None) == 1
    assert L.mimk_reduce_static(None, None, _lib.BF16, 1, 4, 1, _lib.SUM, None) == 4
    assert L.mimk_reduce_static(None, None, 0, 1, 4, 1, 9, None) == 1
