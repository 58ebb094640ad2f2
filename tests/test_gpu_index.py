"""GPU parity of the constructors and the data-dependent indexing operators (splat, generate, gather, scatter, concat,
repeat, reshape) against the oracle's restatement of the reference's loops: the reference's known answers and seeded
cases; integer and copy work is bit exact."""
import numpy as np
import pytest
import torch

import oracle as mo

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def T():
    from mimir_b200 import tensor
    return tensor


def cu(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def test_generate_exec_30(T):
    # lit/tensor/generate_exec.mim:12-20
    g = T.generate((2, 3), lambda i, _j: T.splat((2, 3), 20, torch.int32).masked_fill(i == 0, 10))
    assert g.dtype == torch.int32 and int(g[0, 2]) + int(g[1, 1]) == 30
    want = mo.generate((2, 3), lambda i, _j: np.int32(10 if i == 0 else 20))
    assert np.array_equal(g.cpu().numpy(), want)


def test_gather_scatter_exec_93(T):
    # lit/tensor/gather_scatter_exec.mim:15-21
    x = cu(np.array([[10, 11, 12], [20, 21, 22]], dtype=np.int32))
    index = cu(np.array([[2, 0], [1, 1]], dtype=np.int32))
    updates = cu(np.array([[10, 20], [30, 40]], dtype=np.int32))
    g = T.gather(1, x, index)
    s = T.scatter(1, x, index, updates)
    T.device_status()
    assert int(g[0, 0]) + int(g[1, 0]) + int(s[0, 0]) + int(s[1, 1]) == 93
    assert s.cpu().tolist() == [[20, 11, 10], [20, 40, 22]]


@pytest.mark.parametrize("dtype", [np.float32, np.int32, np.int64])
@pytest.mark.parametrize("idx_dtype", [np.int32, np.int64])
def test_gather_scatter_match_the_loops(T, dtype, idx_dtype):
    rng = np.random.default_rng(17)
    for dim in range(3):
        s_src = (7, 9, 11)
        s_idx = tuple(5 if d == dim else s_src[d] - (d % 2) for d in range(3))     # <= the source off the indexed axis
        s_upd = tuple(v + 1 for v in s_idx)                                          # updates may be larger than the index
        x = rng.integers(-100, 100, s_src).astype(dtype)
        index = rng.integers(0, s_src[dim], s_idx).astype(idx_dtype)                # duplicates along the line are likely
        upd = rng.integers(-100, 100, s_upd).astype(dtype)
        g = T.gather(dim, cu(x), cu(index))
        s = T.scatter(dim, cu(x), cu(index), cu(upd))
        T.device_status()
        assert np.array_equal(g.cpu().numpy(), mo.gather(dim, x, index)), dim
        assert np.array_equal(s.cpu().numpy(), mo.scatter(dim, x, index, upd)), dim


def test_gather_bf16_and_large(T):
    g = torch.Generator().manual_seed(2)
    x = torch.randn(64, 1000, 33, generator=g).to(torch.bfloat16).cuda()
    index = torch.randint(0, 1000, (64, 300, 33), generator=g).cuda()
    got = T.gather(1, x, index)
    assert torch.equal(got, torch.gather(x, 1, index))          # the same element picks, bit for bit
    upd = torch.randn(64, 300, 33, generator=g).to(torch.bfloat16).cuda()
    sc = T.scatter(1, x, index, upd)
    want = mo.scatter(1, x[:2].float().cpu().numpy(), index[:2].cpu().numpy(), upd[:2].float().cpu().numpy())
    assert np.array_equal(sc[:2].float().cpu().numpy(), want)


def test_out_of_range_index_is_reported_not_followed(T):
    from mimir_b200 import _lib as L
    x = cu(np.arange(12, dtype=np.int32).reshape(3, 4))
    index = cu(np.array([[0, 9, 1]], dtype=np.int64))            # 9 is outside axis 1 (extent 4)
    out = T.gather(1, x, index)
    with pytest.raises(L.MimkError) as e:
        T.device_status()
    assert e.value.status == 2                                   # MIMK_E_SHAPE
    assert out[0, 0].item() == 0 and out[0, 2].item() == 1       # the in-range picks were made
    T.device_status()                                            # the flag is cleared, the context usable


def test_splat_iota_reshape_repeat_concat(T):
    assert torch.equal(T.splat((3, 5), 2.5), torch.full((3, 5), 2.5, device="cuda"))
    assert torch.equal(T.splat((4,), -3, torch.int64), torch.full((4,), -3, dtype=torch.int64, device="cuda"))
    assert torch.equal(T.splat((2, 2), 1.5, torch.bfloat16), torch.full((2, 2), 1.5, dtype=torch.bfloat16, device="cuda"))
    co = T.iota((3, 4, 5), 1)
    assert np.array_equal(co.cpu().numpy(), np.indices((3, 4, 5))[1])
    lin = T.generate_affine((3, 4), (4, 1, 7), torch.int32)          # 4 i + j + 7
    assert np.array_equal(lin.cpu().numpy(), (np.arange(12).reshape(3, 4) + 7).astype(np.int32))
    rng = np.random.default_rng(4)
    x = rng.standard_normal((3, 4, 5)).astype(np.float32)
    assert np.array_equal(T.reshape(cu(x), (5, 12)).cpu().numpy(), x.reshape(5, 12))
    assert np.array_equal(T.repeat(cu(x), (6, 4, 15)).cpu().numpy(), mo.repeat(x, (6, 4, 15)))
    xi = rng.integers(0, 9, (2, 3)).astype(np.int64)
    assert np.array_equal(T.repeat(cu(xi), (4, 9)).cpu().numpy(), np.tile(xi, (2, 3)))
    parts = [rng.standard_normal((3, n, 5)).astype(np.float32) for n in (2, 0, 4, 1)]
    assert np.array_equal(T.concat(1, [cu(p) for p in parts]).cpu().numpy(), mo.concat(1, parts))
    assert np.array_equal(T.concat(0, [cu(x), cu(x)]).cpu().numpy(), np.concatenate([x, x], 0))
    assert np.array_equal(T.concat(2, [cu(x), cu(x[:, :, :2])]).cpu().numpy(), np.concatenate([x, x[:, :, :2]], 2))


def test_select_and_grouped_convolution(T):
    rng = np.random.default_rng(8)
    a, b = rng.standard_normal((5, 7)).astype(np.float32), rng.standard_normal((5, 7)).astype(np.float32)
    cond = rng.integers(0, 2, (5, 7)).astype(bool)
    assert np.array_equal(T.select(cu(cond), cu(a), cu(b)).cpu().numpy(), np.where(cond, a, b))
    # the generate_exec body with the library's own operators: i == 0 ? 10 : 20
    i = T.iota((2, 3), 0)
    g = T.select(i == 0, T.splat((2, 3), 10, torch.int32), T.splat((2, 3), 20, torch.int32))
    assert int(g[0, 2]) + int(g[1, 1]) == 30
    # conv_grouped (lit/tensor/conv_grouped.mim shapes, scaled down): groups 2 and 3, with stride / padding / dilation
    for (n, cin, cout, groups, k, stride, dil, pad) in [(2, 8, 6, 2, 3, 1, 1, 1), (1, 6, 9, 3, 1, 1, 1, 0), (2, 4, 4, 2, 3, 2, 2, 2)]:
        x = rng.standard_normal((n, cin, 9, 10)).astype(np.float32)
        w = rng.standard_normal((cout, cin // groups, k, k)).astype(np.float32)
        got = T.conv_grouped(cu(x), cu(w), groups, (stride, stride), (dil, dil), (pad, pad))
        want = torch.nn.functional.conv2d(torch.from_numpy(x).double(), torch.from_numpy(w).double(), stride=stride, padding=pad,
                                          dilation=dil, groups=groups).numpy()
        assert got.shape == want.shape and mo.normalised_error(got.cpu().numpy(), want) < 1e-5
    # groups = 1 is the dense convolution
    x = rng.standard_normal((1, 3, 6, 6)).astype(np.float32)
    w = rng.standard_normal((4, 3, 3, 3)).astype(np.float32)
    assert torch.equal(T.conv_grouped(cu(x), cu(w), 1), T.conv(cu(x), cu(w)))
    assert T.get(T.set_(T.from_array([[1, 2], [3, 4]], torch.int32), (1, 0), 9), (1, 0)) == 9


def test_broadcast_expands_unit_axes(T):
    x = np.arange(12, dtype=np.float32).reshape(3, 1, 4)
    assert np.array_equal(T.broadcast(cu(x), (3, 5, 4)).cpu().numpy(), np.broadcast_to(x, (3, 5, 4)))


@pytest.mark.parametrize("dim", [0, 1, 2])
def test_scatter_with_one_thread_per_update_keeps_the_last_visit(T, dim):
    """Index tensors large enough for the one-thread-per-update form (a winner per destination): a narrow source axis
    makes almost every destination a duplicate; the loops' row-major rule decides, bit for bit."""
    rng = np.random.default_rng(23 + dim)
    s_src = [30, 40, 50]
    s_src[dim] = 6                                               # few destinations per line: heavy duplication
    s_idx = [30, 40, 50]
    s_idx[dim] = 45
    x = rng.integers(-1000, 1000, s_src).astype(np.int32)
    index = rng.integers(0, 6, s_idx).astype(np.int64)
    upd = rng.integers(-1000, 1000, s_idx).astype(np.int32)
    got = T.scatter(dim, cu(x), cu(index), cu(upd))
    T.device_status()
    assert np.array_equal(got.cpu().numpy(), mo.scatter(dim, x, index, upd))


def test_scatter_few_updates_into_a_large_table(T):
    """An index tensor past the one-thread-per-update threshold scattered into an input far larger than itself: the
    library must not clear a winner table of the input's size for it (the per-line kernel runs), and the loops' rule
    still decides the duplicates."""
    rng = np.random.default_rng(31)
    x = rng.integers(-1000, 1000, (64, 40000)).astype(np.int32)        # 2.56 M cells
    index = rng.integers(0, 40000, (64, 80)).astype(np.int64)          # 5120 updates, some duplicates per line
    index[:, 40:] = index[:, :40]
    upd = rng.integers(-1000, 1000, (64, 80)).astype(np.int32)
    got = T.scatter(1, cu(x), cu(index), cu(upd))
    T.device_status()
    assert np.array_equal(got.cpu().numpy(), mo.scatter(1, x, index, upd))
