"""CPU-only checks of the drop-in boundary: the library loads, exports every symbol include/mimk.h declares,
and validates arguments before touching a device."""
import ctypes as C
import os
import re

import pytest

import __graft_entry__ as entry

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def lib():
    entry.build()
    from mimir_b200 import _lib
    return _lib


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "mimk.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(mimk_[a-z0-9_]+)\s*\(", text)))


def test_header_symbols_are_exported(lib):
    names = declared_symbols()
    assert len(names) >= 13
    L = lib.lib()
    for n in names:
        assert hasattr(L, n), n
    assert sorted(lib.SYMBOLS) == names


def test_abi_version_and_status_strings(lib):
    L = lib.lib()
    assert L.mimk_abi_version() == 2
    assert L.mimk_status_str(0) == b"ok"
    for code in range(1, 10):
        s = L.mimk_status_str(code)
        assert s and s != b"unknown status"
    assert L.mimk_status_str(1234) == b"unknown status"


def test_argument_validation_needs_no_device(lib):
    L = lib.lib()
    assert L.mimk_gemm(None, None) == 1
    d = lib.GemmDesc()
    d.batch, d.m, d.n, d.k = 1, -4, 4, 4
    assert L.mimk_gemm(C.byref(d), None) == 1          # negative extent
    d.m = 4
    d.in_dtype = 7
    assert L.mimk_gemm(C.byref(d), None) == 4          # dtype
    d.in_dtype, d.out_dtype, d.post = lib.F32, lib.F32, lib.POST_BIAS
    assert L.mimk_gemm(C.byref(d), None) == 1          # bias epilogue without its operand
    assert L.mimk_attn_fwd(None, None) == 1
    assert L.mimk_mlp_gated(None, None) == 1
    assert L.mimk_reduce(None, None, lib.F32, -1, 4, 1, lib.SUM, None) == 1
    assert L.mimk_reduce(None, None, lib.I32, 1, 4, 1, lib.SUM, None) == 4
    assert L.mimk_map(99, None, None, None, lib.F32, 1, 1, 1, 0, None) == 1
    assert L.mimk_map_reduce_post(None, None) == 1
    assert L.mimk_host_map_reduce_post(None) == 1
    m = lib.MrpDesc()
    m.ro, m.rn = 3, 2                                   # more output loops than loops
    assert L.mimk_map_reduce_post(C.byref(m), None) == 1
    assert L.mimk_host_map_reduce_post(C.byref(m)) == 1
    assert L.mimk_mrp_classify(None) == 0
    assert L.mimk_chain_order(0, None, None, 0, 8, None, None) == 1
    # the fused reduce-scatter: row blocks must tile the result exactly, in whole 32-row boxes
    d = lib.GemmDesc()
    d.batch, d.m, d.n, d.k = 1, 512, 256, 256
    d.in_dtype, d.out_dtype, d.post = lib.BF16, lib.F32, lib.POST_ID
    g = lib.GatherDst()
    g.n_dst, g.ldc, g.col_off = 2, 256, 0
    assert L.mimk_gemm_reduce_scatter(C.byref(d), None, 256, None) == 1
    assert L.mimk_gemm_reduce_scatter(C.byref(d), C.byref(g), 128, None) == 2      # E_SHAPE: 2 x 128 rows != m
    d.m = 80
    assert L.mimk_gemm_reduce_scatter(C.byref(d), C.byref(g), 40, None) == 3       # E_ALIGN: not whole 32-row boxes


def test_no_cpu_fallback_without_device(lib):
    import torch
    if torch.cuda.is_available():
        pytest.skip("a device is present")
    L = lib.lib()
    assert L.mimk_device_check() == 6                   # MIMK_E_NO_DEVICE
    d = lib.GemmDesc()
    d.batch, d.m, d.n, d.k = 1, 4, 4, 4
    d.in_dtype, d.out_dtype = lib.F32, lib.F32
    assert L.mimk_gemm(C.byref(d), None) == 6
    m = lib.MrpDesc()                                   # a valid empty-loop instance still needs the device
    m.ro = m.rn = 1
    m.sr[0] = m.so[0] = 4
    m.nis, m.comb, m.acc_dtype, m.out_dtype = 1, lib.F_FIRST, lib.F32, lib.F32
    m.in_dtype[0] = lib.F32
    m.in_map[0].rows, m.map_out.rows = 1, 1
    m.in_map[0].coef[0][0] = m.map_out.coef[0][0] = 1
    m.in_shape[0][0] = 4
    assert L.mimk_map_reduce_post(C.byref(m), None) == 6
    buf = (C.c_float * 4)()
    m.in_[0] = C.addressof(buf)
    m.out = C.addressof(buf)
    assert L.mimk_host_map_reduce_post(C.byref(m)) == 6
    with pytest.raises(ValueError):
        from mimir_b200 import tensor as T
        T.product_2d(torch.zeros(2, 2), torch.zeros(2, 2))


def test_host_shape_errors_mirror_the_reference(lib):
    # the reference's refly.check message for mismatching contractions (tensor.mim:1393)
    import torch
    from mimir_b200 import tensor as T
    if not torch.cuda.is_available():
        pytest.skip("shape checks run after the device check")
    with pytest.raises(ValueError, match="contracting dims don't match"):
        T.product_2d(torch.zeros(2, 3, device="cuda"), torch.zeros(4, 2, device="cuda"))


def test_reduce_plan_fits_the_static_array_on_148_sms(lib):
    """mimk_reduce_static keeps its partial results in MIMK_REDUCE_STATIC_BYTES of the library image. The plan (shared
    with mimk_reduce) must fit there for every shape on a 148-SM device; with more SMs it can grow past it, which is
    when the entry point answers MIMK_E_WORKSPACE."""
    L = lib.lib()
    cap = (1 << 20) // 4
    n = C.c_int64(0)
    worst = 0
    for total in [1, 2, 7, 255, 256, 257, 1000, 4096, 20000, 50000, 75000, 75775, 75776, 75777, 100000, 10 ** 6]:
        for ln in [1, 63, 255, 256, 300, 4096, 9000, 65536, 10 ** 6]:
            for outer in (1, 3):
                if total % outer:
                    continue
                assert L.mimk_reduce_plan(outer, ln, total // outer, 148, C.byref(n)) == 0
                assert 0 <= n.value <= cap, (total, ln, n.value)
                worst = max(worst, n.value)
                if n.value:
                    assert n.value % total == 0 and ln >= 256       # whole slices, only long axes are split
    assert worst > cap // 2                                          # the sweep reaches the large plans
    assert L.mimk_reduce_plan(1, 4096, 1, 148, C.byref(n)) == 0 and n.value == 0          # row reduce: no partials
    assert L.mimk_reduce_plan(1, 10 ** 6, 100000, 264, C.byref(n)) == 0 and n.value > cap   # a larger machine can exceed
    assert L.mimk_reduce_plan(-1, 4, 4, 148, C.byref(n)) == 1
    assert L.mimk_reduce_plan(1, 4, 4, 148, None) == 1
