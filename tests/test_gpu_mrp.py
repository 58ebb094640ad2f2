"""GPU parity of the generic `map_reduce_post` kernel: the reference's integer known answers (bit exact) and
seeded comparisons with the oracle's interpreter on the same descriptors."""
import numpy as np
import pytest
import torch

import oracle as mo

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def T():
    from mimir_b200 import tensor
    return tensor


@pytest.fixture(scope="module")
def L():
    from mimir_b200 import _lib
    return _lib


def cu(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def test_exec_map_reduce_42_and_epilogue_46(T, L):
    t = cu((np.arange(12, dtype=np.int32) + 1).reshape(3, 4))
    out = T.map_reduce_post((3,), (3, 4), L.F_ADD, 0, L.P_ID, T.proj_map(2, (0,)), [T.id_map(2)], [t])
    assert out.tolist() == [10, 26, 42]                      # lit/buffer/exec_map_reduce.mim
    tt = cu(np.array([[1, 5, 9], [2, 6, 10], [3, 7, 11], [4, 8, 12]], dtype=np.int32))
    bias = cu(np.array([1, 2, 3], dtype=np.int32))
    out = T.map_reduce_post((3,), (3, 4), L.F_ADD, 0, L.P_ADD_PLUS1, T.proj_map(2, (0,)), [T.proj_map(2, (1, 0))], [tt],
                            [T.id_map(1)], [bias])
    assert out.tolist() == [12, 29, 46]                      # lit/buffer/exec_epilogue.mim


def test_exec_interchange_ktile_tile(T, L):
    a = cu((np.arange(6, dtype=np.int32) + 1).reshape(2, 3))
    b = cu(np.add.outer(np.arange(3), np.arange(4)).astype(np.int32))
    mm = lambda a, b, m, l, k: T.map_reduce_post((m, l), (m, l, k), L.F_MULADD, 0, L.P_ID, T.proj_map(3, (0, 1)),
                                                 [T.proj_map(3, (0, 2)), T.proj_map(3, (2, 1))], [a, b])
    assert int(mm(a, b, 2, 4, 3)[1, 2]) == 47                # lit/buffer/exec_interchange.mim
    ones, twos = cu(np.ones((2, 4), np.int32)), cu(np.full((4, 2), 2, np.int32))
    assert int(mm(ones, twos, 2, 2, 4)[1, 1]) == 8           # lit/buffer/exec_ktile.mim
    # lit/buffer/exec_tile.mim: loops (io, jo, ii, ji, ko, ki), packed output (io, ii, jo, ji); C_packed[0,1,1,0] = 80
    a = cu(np.repeat(np.arange(1, 5, dtype=np.int32)[:, None], 8, axis=1))
    b = cu(np.repeat(np.array([[1, 3, 5, 7]], dtype=np.int32), 8, axis=0))
    ma = [[2, 0, 1, 0, 0, 0, 0], [0, 0, 0, 0, 4, 1, 0]]
    mb = [[0, 0, 0, 0, 4, 1, 0], [0, 2, 0, 1, 0, 0, 0]]
    out = T.map_reduce_post((2, 2, 2, 2), (2, 2, 2, 2, 2, 4), L.F_MULADD, 0, L.P_ID, T.proj_map(6, (0, 2, 1, 3)), [ma, mb],
                            [a, b])
    assert int(out[0, 1, 1, 0]) == 80
    assert np.array_equal(out.reshape(4, 4).cpu().numpy(), a.cpu().numpy() @ b.cpu().numpy())


def test_exec_conv_63(T, L):
    def conv(cin):
        x, w = cu(np.ones((2, cin, 4, 4), np.int32)), cu(np.ones((2, cin, 3, 3), np.int32))
        mi = [[0] * 8 for _ in range(4)]
        mi[0][0] = 1; mi[1][4] = 1; mi[2][2] = 1; mi[2][5] = 1; mi[3][3] = 1; mi[3][6] = 1
        return T.map_reduce_post((2, 2, 2, 2), (2, 2, 2, 2, cin, 3, 3), L.F_MULADD, 0, L.P_ID, T.proj_map(7, (0, 1, 2, 3)),
                                 [mi, T.proj_map(7, (1, 4, 5, 6))], [x, w])
    assert int(conv(3)[1, 1, 1, 1]) + int(conv(4)[0, 1, 0, 1]) == 63   # lit/buffer/exec_conv.mim


def test_heterogeneous_166_365(T, L):
    # lit/btensor/map_reduce_post.mim:22-36 -- I32 and I64 inputs, I32 accumulator, I64 epilogue input and result
    a = cu(np.array([[[1, 2, 3]], [[4, 5, 6]]], dtype=np.int32))
    b = cu(np.array([[[10, 20, 30]], [[40, 50, 60]]], dtype=np.int64))
    p = cu(np.array([[100], [200]], dtype=np.int64))
    out = T.map_reduce_post((2, 1), (2, 1, 3), L.F_MIX, 0, L.P_ADD, T.proj_map(3, (0, 1)), [T.id_map(3), T.id_map(3)],
                            [a, b], [T.id_map(2)], [p], acc_dtype=torch.int32, out_dtype=torch.int64)
    assert out.reshape(-1).tolist() == [166, 365]


def test_int32_wraps_like_the_oracle(T, L):
    rng = np.random.default_rng(0)
    a = rng.integers(-2**31, 2**31 - 1, (5, 9), dtype=np.int64).astype(np.int32)
    b = rng.integers(-2**31, 2**31 - 1, (9, 4), dtype=np.int64).astype(np.int32)
    got = T.map_reduce_post((5, 4), (5, 4, 9), L.F_MULADD, 0, L.P_ID, T.proj_map(3, (0, 1)),
                            [T.proj_map(3, (0, 2)), T.proj_map(3, (2, 1))], [cu(a), cu(b)])
    assert np.array_equal(got.cpu().numpy(), mo.product_2d(a, b))


def test_float_instances_match_the_interpreter(T, L):
    rng = np.random.default_rng(1)
    x = rng.standard_normal((6, 7, 5)).astype(np.float32)
    # reduce over the middle axis: output loops (0, 2), reduction loop 1
    got = T.map_reduce_post((6, 5), (6, 5, 7), L.F_ADD, 0.0, L.P_ID, T.proj_map(3, (0, 1)), [T.proj_map(3, (0, 2, 1))],
                            [cu(x)])
    assert np.array_equal(got.cpu().numpy(), mo.reduce(x, 1))        # same ascending fold order: same bits
    mx = T.map_reduce_post((6, 5), (6, 5, 7), L.F_MAX, float("-inf"), L.P_ID, T.proj_map(3, (0, 1)),
                           [T.proj_map(3, (0, 2, 1))], [cu(x)])
    assert np.array_equal(mx.cpu().numpy(), mo.reduce(x, 1, "max"))
    # binary_ax exp(x - max) with y broadcast along axis 1
    e = T.map_reduce_post((6, 7, 5), (6, 7, 5), L.F_SUBEXP, 0.0, L.P_ID, T.id_map(3), [T.id_map(3), T.proj_map(3, (0, 2))],
                          [cu(x), mx])
    want = mo.binary_ax(mo.F_SUBEXP_F32, 1, x, mo.reduce(x, 1, "max"))
    assert np.allclose(e.cpu().numpy(), want, rtol=2e-6, atol=0)
    # transposed copy, flipped copy (negative coefficient + constant), strided slice, broadcast
    t2 = rng.standard_normal((4, 9)).astype(np.float32)
    tr = T.map_reduce_post((9, 4), (9, 4), L.F_FIRST, 0.0, L.P_ID, T.id_map(2), [T.proj_map(2, (1, 0))], [cu(t2)])
    assert np.array_equal(tr.cpu().numpy(), t2.T)
    fl = T.map_reduce_post((4, 9), (4, 9), L.F_FIRST, 0.0, L.P_ID, T.id_map(2), [[[-1, 0, 3], [0, -1, 8]]], [cu(t2)])
    assert np.array_equal(fl.cpu().numpy(), t2[::-1, ::-1])
    sl = T.map_reduce_post((2, 4), (2, 4), L.F_FIRST, 0.0, L.P_ID, T.id_map(2), [[[2, 0, 1], [0, 2, 0]]], [cu(t2)])
    assert np.array_equal(sl.cpu().numpy(), t2[1::2, 0:8:2])
    bc = T.map_reduce_post((3, 9), (3, 9), L.F_FIRST, 0.0, L.P_ID, T.id_map(2), [[[0, 1, 0]]], [cu(t2[0])])
    assert np.array_equal(bc.cpu().numpy(), np.broadcast_to(t2[0], (3, 9)))


def test_fc_fixture_through_the_generic_kernel(T, L):
    # lit/tensor/fc_aux.cpp with the bias+relu epilogue in the `post` slot and W read through its transpose
    M, K, N = 5, 33, 7
    x = ((np.arange(M * K) % 13).astype(np.float32) / np.float32(13.0) - np.float32(0.4)).reshape(M, K)
    w = (((7 * np.arange(N * K)) % 11).astype(np.float32) / np.float32(11.0) - np.float32(0.5)).reshape(N, K)
    bias = ((np.arange(N) % 5).astype(np.float32) / np.float32(5.0) - np.float32(0.4))
    got = T.map_reduce_post((M, N), (M, N, K), L.F_MULADD, 0.0, L.P_ADD_RELU, T.proj_map(3, (0, 1)),
                            [T.proj_map(3, (0, 2)), T.proj_map(3, (1, 2))], [cu(x), cu(w)], [T.proj_map(2, (1,))], [cu(bias)])
    ref = np.maximum((x.astype(np.float64) @ w.astype(np.float64).T + bias).astype(np.float32), 0)
    assert (np.abs(ref - got.cpu().numpy()) <= 1e-4 + 1e-4 * np.abs(ref)).all()
    # and it agrees with the specialised contraction kernel
    spec = T.product_2d(cu(x), T.transpose_2d(cu(w)), post="bias_relu", bias=cu(bias))
    assert np.allclose(spec.cpu().numpy(), got.cpu().numpy(), rtol=1e-6, atol=1e-6)


def test_out_of_range_maps_are_refused(T, L):
    from mimir_b200 import MimkError
    t = cu(np.zeros((3, 4), np.float32))
    with pytest.raises(MimkError) as e:   # reads column 4 of a 4-column tensor
        T.map_reduce_post((3, 4), (3, 4), L.F_FIRST, 0.0, L.P_ID, T.id_map(2), [[[1, 0, 0], [0, 1, 1]]], [t])
    assert e.value.status == 2
    with pytest.raises(MimkError) as e:   # writes outside the result
        T.map_reduce_post((3, 3), (3, 4), L.F_FIRST, 0.0, L.P_ID, T.id_map(2), [T.id_map(2)], [t])
    assert e.value.status == 2
    # zero-sized output, dynamic-bound style empty reduction
    out = T.map_reduce_post((0, 4), (0, 4), L.F_FIRST, 0.0, L.P_ID, T.id_map(2), [T.id_map(2)], [cu(np.zeros((0, 4), np.float32))])
    assert out.shape == (0, 4)
    out = T.map_reduce_post((3,), (3, 0), L.F_ADD, 0.0, L.P_ID, T.proj_map(2, (0,)), [T.id_map(2)], [cu(np.zeros((3, 0), np.float32))])
    assert out.tolist() == [0.0, 0.0, 0.0]


def test_shape_ops_conv_pool_dot_general(T, L):
    rng = np.random.default_rng(5)
    x = rng.standard_normal((3, 4, 5)).astype(np.float32)
    assert np.array_equal(T.transpose(cu(x), (2, 0, 1)).cpu().numpy(), x.transpose(2, 0, 1))
    assert np.array_equal(T.flip(cu(x)).cpu().numpy(), x[::-1, ::-1, ::-1])
    assert np.array_equal(T.slice_(cu(x), (1, 0, 1), (1, 2, 2), (2, 2, 2)).cpu().numpy(), x[1:3, 0:4:2, 1:5:2])
    b = rng.standard_normal((1, 5)).astype(np.float32)
    assert np.array_equal(T.broadcast_in_dim(cu(b), (4, 5), (0, 1)).cpu().numpy(), np.broadcast_to(b, (4, 5)))
    assert np.array_equal(T.pad(cu(x), (1, 0, 2), (0, 1, 1), 7.0).cpu().numpy(),
                          np.pad(x, ((1, 0), (0, 1), (2, 1)), constant_values=7.0))
    # conv: the reference's all-ones fixture (lit/buffer/exec_conv.mim) and a seeded one against torch's own
    ones = lambda *s: cu(np.ones(s, np.int32))
    assert int(T.conv(ones(2, 3, 4, 4), ones(2, 3, 3, 3))[1, 1, 1, 1]) + int(T.conv(ones(2, 4, 4, 4), ones(2, 4, 3, 3))[0, 1, 0, 1]) == 63
    xi = rng.standard_normal((2, 3, 9, 8)).astype(np.float32)
    w = rng.standard_normal((4, 3, 3, 2)).astype(np.float32)
    got = T.conv(cu(xi), cu(w), stride=(2, 1), dilation=(1, 2), padding=(1, 1))
    want = torch.nn.functional.conv2d(torch.from_numpy(xi).double(), torch.from_numpy(w).double(), stride=(2, 1),
                                      dilation=(1, 2), padding=(1, 1)).numpy()
    assert got.shape == want.shape and mo.normalised_error(got.cpu().numpy(), want) < 1e-5
    pm = T.pool("max", cu(xi), (2, 2), padding=(1, 0))
    wantp = torch.nn.functional.max_pool2d(torch.from_numpy(xi), (2, 2), padding=(1, 0)).numpy()
    assert np.array_equal(pm.cpu().numpy(), wantp)
    # dot_general: batch axis 1 of a with axis 0 of b, contraction over two axes
    a = rng.standard_normal((4, 3, 5, 6)).astype(np.float32)
    bb = rng.standard_normal((3, 6, 7, 5)).astype(np.float32)
    got = T.dot_product(cu(a), cu(bb), ((2, 3), (3, 1)), ((1,), (0,)))
    want = np.einsum("abcd,bdec->bae", a.astype(np.float64), bb.astype(np.float64))
    assert got.shape == want.shape and mo.normalised_error(got.cpu().numpy(), want) < 1e-5
    with pytest.raises(ValueError, match="contracting dims don't match"):
        T.dot_product(cu(a), cu(bb), ((2,), (0,)))


def test_large_float_instances_run_on_the_specialised_kernels(T, L):
    """Descriptors the recognisers take (contraction, axis fold, elementwise) give what the specialised entry points
    give -- same kernels, same bits -- and stay within the float tolerance of the f64 truth."""
    g = torch.Generator().manual_seed(5)
    M, N, K = 384, 512, 256
    a = torch.randn(M, K, generator=g).cuda()
    b = torch.randn(K, N, generator=g).cuda()
    maps = [T.proj_map(3, (0, 2)), T.proj_map(3, (2, 1))]
    assert T.mrp_route((M, N), (M, N, K), L.F_MULADD, 0.0, L.P_ID, T.proj_map(3, (0, 1)), maps, [a.shape, b.shape],
                       [a.dtype, b.dtype]) == "gemm"
    got = T.map_reduce_post((M, N), (M, N, K), L.F_MULADD, 0.0, L.P_ID, T.proj_map(3, (0, 1)), maps, [a, b])
    assert torch.equal(got, T.product_2d(a, b))
    truth = a.double().cpu().numpy() @ b.double().cpu().numpy()
    assert mo.normalised_error(got.cpu().numpy(), truth) <= 1e-5

    # bf16, right operand stored [N, K] and read through its transpose, bias + relu in the epilogue, bf16 result
    ah = a.to(torch.bfloat16)
    wh = torch.randn(N, K, generator=g).to(torch.bfloat16).cuda()
    bias = torch.randn(N, generator=g).cuda()
    got = T.map_reduce_post((M, N), (M, N, K), L.F_MULADD, 0.0, L.P_ADD_RELU, T.proj_map(3, (0, 1)),
                            [T.proj_map(3, (0, 2)), T.proj_map(3, (1, 2))], [ah, wh], [T.proj_map(2, (1,))], [bias],
                            out_dtype=torch.bfloat16)
    assert torch.equal(got, T.product_2d(ah, T.transpose_2d(wh), post="bias_relu", bias=bias))
    truth = np.maximum(ah.double().cpu().numpy() @ wh.double().cpu().numpy().T + bias.double().cpu().numpy(), 0)
    assert mo.normalised_error(got.float().cpu().numpy(), truth) <= 2e-2

    # batched, batch loop first (bmm, tensor.mim:1416-1417)
    B = 6
    ab = torch.randn(B, 128, 192, generator=g).cuda()
    bb = torch.randn(B, 192, 128, generator=g).cuda()
    got = T.map_reduce_post((B, 128, 128), (B, 128, 128, 192), L.F_MULADD, 0.0, L.P_ID, T.proj_map(4, (0, 1, 2)),
                            [T.proj_map(4, (0, 1, 3)), T.proj_map(4, (0, 3, 2))], [ab, bb])
    assert torch.equal(got, T.bmm(ab, bb))
    assert mo.normalised_error(got.cpu().numpy(), ab.double().cpu().numpy() @ bb.double().cpu().numpy()) <= 1e-5

    # axis folds of a [96, 160, 128] tensor
    x = torch.randn(96, 160, 128, generator=g).cuda()
    xs = list(x.shape)
    for ax in range(3):
        out = [s for i, s in enumerate(xs) if i != ax]
        subs = [0, 1]
        subs.insert(ax, 2)
        s = T.map_reduce_post(out, out + [xs[ax]], L.F_ADD, 0.0, L.P_ID, T.proj_map(3, (0, 1)), [T.proj_map(3, subs)], [x])
        assert torch.equal(s, T.reduce("sum", ax, x))
        assert mo.normalised_error(s.cpu().numpy(), x.double().cpu().numpy().sum(axis=ax)) <= 1e-5
        m = T.map_reduce_post(out, out + [xs[ax]], L.F_MAX, float("-inf"), L.P_ID, T.proj_map(3, (0, 1)), [T.proj_map(3, subs)], [x])
        assert np.array_equal(m.cpu().numpy(), x.cpu().numpy().max(axis=ax))

    # elementwise: silu; product; exp(x - max) with the maximum broadcast along the middle axis; bias over the leading axes
    y = torch.randn(96, 160, 128, generator=g).cuda()
    got = T.map_reduce_post(xs, xs, L.F_FIRST, 0.0, L.P_SILU, T.id_map(3), [T.id_map(3)], [x])
    assert torch.equal(got, T.unary("silu", x))
    assert mo.normalised_error(got.cpu().numpy(), (x.double() * torch.sigmoid(x.double())).cpu().numpy()) <= 1e-5
    got = T.map_reduce_post(xs, xs, L.F_MUL2, 0.0, L.P_ID, T.id_map(3), [T.id_map(3), T.id_map(3)], [x, y])
    assert np.array_equal(got.cpu().numpy(), x.cpu().numpy() * y.cpu().numpy())
    mx = T.reduce("max", 1, x)
    got = T.map_reduce_post(xs, xs, L.F_SUBEXP, 0.0, L.P_ID, T.id_map(3), [T.id_map(3), T.proj_map(3, (0, 2))], [x, mx])
    want = np.exp(x.double().cpu().numpy() - mx.double().cpu().numpy()[:, None, :])
    assert mo.normalised_error(got.cpu().numpy(), want) <= 1e-5
    row = torch.randn(160, 128, generator=g).cuda()
    got = T.map_reduce_post(xs, xs, L.F_ADD2, 0.0, L.P_ID, T.id_map(3), [T.id_map(3), T.proj_map(3, (1, 2))], [x, row])
    assert np.array_equal(got.cpu().numpy(), x.cpu().numpy() + row.cpu().numpy()[None])


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.int64, torch.int32])
def test_large_axis_permutations_are_tiled_copies(T, L, dtype):
    """tensor.transpose of tensors large enough to leave the per-cell kernel: every permutation that moves the fastest
    axis, with extents that end inside a 32 x 32 tile. A copy: bit exact for every element type."""
    g = torch.Generator().manual_seed(9)
    shape = (70, 161, 130)
    x = torch.randint(-1000, 1000, shape, generator=g).to(dtype).cuda()
    for perm in ((2, 1, 0), (1, 2, 0), (2, 0, 1), (0, 2, 1)):
        out_shape = [shape[p] for p in perm]
        inv = [perm.index(j) for j in range(3)]                  # input axis j is indexed by output loop inv[j]
        assert T.mrp_route(out_shape, out_shape, L.F_FIRST, 0, L.P_ID, T.id_map(3), [T.proj_map(3, inv)], [shape], [dtype],
                           acc_dtype=torch.float32 if dtype.is_floating_point else dtype, out_dtype=dtype) == "permute"
        got = T.transpose(x, perm)
        assert torch.equal(got, x.permute(perm).contiguous()), perm
    m = torch.randint(-1000, 1000, (3000, 1111), generator=g).to(dtype).cuda()
    assert torch.equal(T.transpose(m, (1, 0)), m.t().contiguous())


def test_two_byte_permutations_with_even_extents_move_pairs(T, L):
    """bf16 tensors whose transposed extents are even take the pair-moving kernel; extents that end inside its 128 x 128
    tile, every permutation that moves the fastest axis. Bit exact."""
    g = torch.Generator().manual_seed(10)
    shape = (6, 258, 130)
    x = torch.randn(shape, generator=g).to(torch.bfloat16).cuda()
    for perm in ((2, 1, 0), (1, 2, 0), (2, 0, 1), (0, 2, 1)):
        assert torch.equal(T.transpose(x, perm), x.permute(perm).contiguous()), perm
    m = torch.randn(2050, 1026, generator=g).to(torch.bfloat16).cuda()
    assert torch.equal(T.transpose(m, (1, 0)), m.t().contiguous())


def test_bf16_descriptors_reach_the_fold_and_map_kernels(T, L):
    g = torch.Generator().manual_seed(14)
    x = torch.randn(1024, 2048, generator=g).to(torch.bfloat16).cuda()
    y = torch.randn(1024, 2048, generator=g).to(torch.bfloat16).cuda()
    s = T.map_reduce_post((1024,), (1024, 2048), L.F_MAX, float("-inf"), L.P_ID, T.proj_map(2, (0,)), [T.id_map(2)], [x],
                          out_dtype=torch.bfloat16)
    assert torch.equal(s, x.amax(1))
    m = T.map_reduce_post((1024, 2048), (1024, 2048), L.F_MUL2, 0.0, L.P_ID, T.id_map(2), [T.id_map(2), T.id_map(2)], [x, y],
                          out_dtype=torch.bfloat16)
    assert torch.equal(m, (x.float() * y.float()).to(torch.bfloat16))


def test_remaining_buffer_known_answers(T, L):
    """lit/buffer/exec_strip (24), exec_unroll (111), exec_size1 (42), exec_pad_concat (42), exec_get_set (50),
    exec_local_tensors (42), two_same_shape_binary / _set (42) and lit/btensor/read_transpose (5), through the C ABI."""
    ones = cu(np.ones((2, 8, 3), np.int32))
    mi = [[1, 0, 0, 0, 0], [0, 4, 1, 0, 0], [0, 0, 0, 1, 0]]       # the 8-loop strip-mined by 4: (i, 4 jo + ji, k)
    out = T.map_reduce_post((2,), (2, 2, 4, 3), L.F_ADD, 0, L.P_ID, T.proj_map(4, (0,)), [mi], [ones])
    assert out.tolist() == [24, 24]
    out = T.map_reduce_post((2,), (2, 37, 3), L.F_ADD, 0, L.P_ID, T.proj_map(3, (0,)), [T.id_map(3)], [cu(np.ones((2, 37, 3), np.int32))])
    assert int(out[1]) == 111
    a, b = cu(np.array([[7, 8, 9]], np.int32)), cu(np.array([[10, 20, 30], [4, 5, 6]], np.int32))
    p, c = T.pad(a, (0, 1), (0, 1), 5), T.concat(0, [a, b])
    assert p.tolist() == [[5, 7, 8, 9, 5]] and int(c[1, 2]) + int(p[0, 1]) + int(p[0, 0]) == 42
    t, u = cu(np.array([10, 20, 30], np.int32)), cu(np.array([1, 2], np.int32))
    p, c = T.pad(t, (1,), (2,), 5), T.concat(0, [t, u])
    assert p.tolist() == [5, 10, 20, 30, 5, 5] and int(p[3]) + int(c[4]) + int(c[0]) == 42
    t = cu((np.arange(12, dtype=np.int32) + 1).reshape(3, 4))
    s = T.set_(t, (0, 0), 42)
    assert T.get(s, (0, 0)) + T.get(s, (1, 2)) + T.get(t, (0, 0)) == 50
    m = cu(np.array([[10, 20], [30, 40]], np.int32))
    s, bc = T.set_(m, (1, 1), 2), T.broadcast(cu(np.array([[5, 7]], np.int32)), (2, 2))
    assert T.get(s, (1, 1)) + T.get(s, (1, 0)) + T.get(bc, (1, 0)) + T.get(bc, (0, 0)) == 42
    x = np.array([[10, 1, 2, 3], [4, 5, 30, 7], [8, 9, 10, 11]], np.int32)
    y = np.array([[5, 1, 1, 1], [1, 1, 3, 1], [1, 1, 1, 1]], np.int32)
    add = T.map_reduce_post((3, 4), (3, 4), L.F_ADD2, 0, L.P_ID, T.id_map(2), [T.id_map(2), T.id_map(2)], [cu(x), cu(y)])
    sub = T.map_reduce_post((3, 4), (3, 4), L.F_ADD2, 0, L.P_ID, T.id_map(2), [T.id_map(2), T.id_map(2)], [cu(x), cu(-y)])
    c = T.concat(0, [add, sub])
    assert int(c[0, 0]) + int(c[4, 2]) == 42
    t = cu(np.array([[12, 2, 3, 4], [5, 6, 30, 8], [9, 10, 11, 12]], np.int32))
    assert T.get(T.set_(t, (0, 0), 2), (1, 2)) + T.get(T.set_(t, (1, 2), 40), (0, 0)) == 42
    d = T.map_reduce_post((4, 2), (4, 2), L.F_FIRST, 0, L.P_ID, T.id_map(2), [T.proj_map(2, (1, 0))], [cu(np.full((2, 4), 5, np.int32))])
    assert int(d[3, 1]) == 5


@pytest.mark.parametrize("dtype", [np.int32, np.int64, np.float32])
def test_maps_with_floordiv_and_rem(T, L, dtype):
    """reshape_map (tensor.mim:1224-1233) as an input map, bit for bit against the oracle's interpreter: the plain
    reshape (which the library recognises and runs as one copy), the unpack of a packed shape (tensor.mim:1405-1411),
    and a fold that reads a reshape through a composed map (what fuse_read_through leaves, fuse.cpp:542-589)."""
    rng = np.random.default_rng(3)
    x = rng.integers(-1000, 1000, (3, 4, 5)).astype(dtype)
    f_first, f_add = (L.F_FIRST, L.F_ADD)
    o_first = mo.F_FIRST_F32 if dtype == np.float32 else mo.F_FIRST_I32
    init = 0.0 if dtype == np.float32 else 0
    for s_out in [(10, 6), (60,), (2, 2, 15), (5, 4, 3)]:
        r = len(s_out)
        got = T.map_reduce_post(s_out, s_out, f_first, init, L.P_ID, T.id_map(r), [T.reshape_map((3, 4, 5), s_out)], [cu(x)])
        assert np.array_equal(got.cpu().numpy(), x.reshape(s_out))
        assert T.mrp_route(s_out, s_out, f_first, init, L.P_ID, T.id_map(r), [T.reshape_map((3, 4, 5), s_out)], [(3, 4, 5)],
                           [torch.from_numpy(x).dtype], acc_dtype=torch.from_numpy(x).dtype if dtype != np.float32 else torch.float32,
                           out_dtype=torch.from_numpy(x).dtype) == "copy"
    # a strided slice of the reshaped view is not a whole-tensor reshape: the per-cell kernel evaluates the map
    view = T.compose_reshape([[2, 0, 1], [0, 1, 0]], 2, (10, 6), (3, 4, 5))           # view[2 o0 + 1, o1]
    got = T.map_reduce_post((4, 6), (4, 6), f_first, init, L.P_ID, T.id_map(2), [view], [cu(x)])
    assert np.array_equal(got.cpu().numpy(), x.reshape(10, 6)[1:9:2])
    if dtype != np.float32:
        # row sums of a (6, 10) view of the stored (3, 4, 5): the consumer's (o, r) composed behind the reshape
        comp = T.compose_reshape(T.id_map(2), 2, (6, 10), (3, 4, 5))
        got = T.map_reduce_post((6,), (6, 10), f_add, 0, L.P_ID, T.proj_map(2, (0,)), [comp], [cu(x)])
        assert np.array_equal(got.cpu().numpy(), x.reshape(6, 10).sum(1))
        if dtype == np.int32:      # and the oracle's interpreter on the same descriptor, bit for bit
            lin = [10, 1, 0]
            want = mo.map_reduce_post((6,), (6, 10), mo.F_ADD_I32, np.int32(0), mo.P_ID, mo.proj_map(2, (0,)),
                                      [mo.DivModMap([lin, lin, lin], [20, 5, 1], [3, 4, 5])], [x])
            assert np.array_equal(got.cpu().numpy(), want)
    # a map whose floordiv / rem could leave the operand is refused before any launch
    bad = T.AccessMap([[1, 0]], div=[1], mod=[0])
    with pytest.raises(Exception):
        T.map_reduce_post((70,), (70,), f_first, init, L.P_ID, T.id_map(1), [bad], [cu(x.reshape(60))])
    neg = T.AccessMap([[1, -3]], div=[2], mod=[0])                                     # linear part can go negative
    with pytest.raises(Exception):
        T.map_reduce_post((10,), (10,), f_first, init, L.P_ID, T.id_map(1), [neg], [cu(x.reshape(60))])


def test_large_reshape_read_through_at_scale(T, L):
    """A fold reading a reshape through a composed floordiv / rem map at a size where every thread's index arithmetic
    matters: column sums of a (4096, 600) view of a tensor stored (600, 64, 64), against numpy (f32 sums of small
    integers are exact)."""
    rng = np.random.default_rng(4)
    x = rng.integers(-3, 4, (600, 64, 64)).astype(np.float32)
    comp = T.compose_reshape(T.proj_map(2, (1, 0)), 2, (4096, 600), (600, 64, 64))       # view[r, o]: fold over the rows
    got = T.map_reduce_post((600,), (600, 4096), L.F_ADD, 0.0, L.P_ID, T.proj_map(2, (0,)), [comp], [cu(x)])
    T.device_status()
    assert np.array_equal(got.cpu().numpy(), x.reshape(4096, 600).sum(0))


def test_composed_combiners_small_and_large(T, L):
    """fold(acc, outer(inner(a, b))) through the descriptor: the per-cell kernel on small instances (bit-equal to the
    interpreter for exactly rounded operations), the fold kernels with the producer inlined on large ones."""
    rng = np.random.default_rng(9)
    x = rng.standard_normal((6, 7, 5)).astype(np.float32)
    y = rng.standard_normal((6, 5)).astype(np.float32)
    sub_sq = L.f_composed(L.F_ADD, L.OP_SUB, L.OP_SQUARE)
    got = T.map_reduce_post((6, 5), (6, 5, 7), sub_sq, 0.0, L.P_ID, T.proj_map(3, (0, 1)),
                            [T.proj_map(3, (0, 2, 1)), T.proj_map(3, (0, 1))], [cu(x), cu(y)])
    want = mo.map_reduce_post((6, 5), (6, 5, 7), mo.f_composed(0, 1, 22), np.float32(0), mo.P_ID, T.proj_map(3, (0, 1)),
                              [T.proj_map(3, (0, 2, 1)), T.proj_map(3, (0, 1))], [x, y])
    assert np.allclose(got.cpu().numpy(), want, rtol=1e-6, atol=1e-6)
    mabs = T.map_reduce_post((6, 5), (6, 5, 7), L.f_composed(L.F_MAX, L.OP_ABS), float("-inf"), L.P_ID, T.proj_map(3, (0, 1)),
                             [T.proj_map(3, (0, 2, 1))], [cu(x)])
    assert np.array_equal(mabs.cpu().numpy(), np.abs(x).max(axis=1))
    # a map (no fold) with a producer chain: FIRST(relu(a * b))
    e = T.map_reduce_post((6, 7, 5), (6, 7, 5), L.f_composed(L.F_FIRST, L.OP_MUL, L.OP_RELU), 0.0, L.P_ID, T.id_map(3),
                          [T.id_map(3), T.proj_map(3, (0, 2))], [cu(x), cu(y)])
    assert np.array_equal(e.cpu().numpy(), np.maximum(x * y[:, None, :], 0))
    # integer accumulators take no composed combiner
    xi = cu(np.arange(12, dtype=np.int32).reshape(3, 4))
    with pytest.raises(RuntimeError):
        T.map_reduce_post((3,), (3, 4), L.f_composed(L.F_ADD, L.OP_SQUARE), 0, L.P_ID, T.proj_map(2, (0,)), [T.id_map(2)], [xi],
                          acc_dtype=torch.int32)
    # large: routed to the fold kernel
    X = rng.standard_normal((512, 4096)).astype(np.float32)
    m = X.max(axis=1)
    desc = dict(So=(512,), Sr=(512, 4096), init=0.0, post=L.P_ID, map_out=T.proj_map(2, (0,)))
    assert T.mrp_route([512], [512, 4096], L.f_composed(L.F_ADD, L.OP_SUBEXP), 0.0, L.P_ID, T.proj_map(2, (0,)),
                       [T.id_map(2), T.proj_map(2, (0,))], [[512, 4096], [512]], [torch.float32, torch.float32]) == "reduce"
    den = T.map_reduce_post(desc["So"], desc["Sr"], L.f_composed(L.F_ADD, L.OP_SUBEXP), 0.0, L.P_ID, desc["map_out"],
                            [T.id_map(2), T.proj_map(2, (0,))], [cu(X), cu(m)])
    want = np.exp(X.astype(np.float64) - m[:, None]).sum(axis=1)
    assert np.abs(den.cpu().numpy() - want).max() / np.abs(want).max() < 1e-5


def test_large_convolutions_run_as_contractions(T, L):
    """From 2^27 multiply-adds on, conv gathers its patches with one copy operation and contracts them with the weights on the
    tensor cores (f32 as 3xTF32, bf16 directly); the result is held to the same tolerance as the per-cell kernel's."""
    rng = np.random.default_rng(21)
    x = rng.standard_normal((4, 64, 32, 32)).astype(np.float32)
    w = (rng.standard_normal((128, 64, 3, 3)) * 0.05).astype(np.float32)
    assert T._conv_on_tensor_cores(torch.float32, 4, 64, 128, 3, 3, 32, 32)
    got = T.conv(cu(x), cu(w), padding=(1, 1))
    want = torch.nn.functional.conv2d(torch.from_numpy(x).double(), torch.from_numpy(w).double(), padding=(1, 1)).numpy()
    assert got.shape == want.shape and mo.normalised_error(got.cpu().numpy(), want) < 1e-5
    # fewer filters than one tensor-core tile (and not a multiple of 4): zero filters fill the tile and are dropped again
    w3 = (rng.standard_normal((30, 64, 3, 3)) * 0.05).astype(np.float32)
    x3 = rng.standard_normal((16, 64, 64, 64)).astype(np.float32)
    assert T._conv_on_tensor_cores(torch.float32, 16, 64, 30, 3, 3, 32, 32)
    got3 = T.conv(cu(x3), cu(w3), stride=(2, 2), padding=(1, 1))
    want3 = torch.nn.functional.conv2d(torch.from_numpy(x3).double(), torch.from_numpy(w3).double(), stride=2, padding=1).numpy()
    assert got3.shape == want3.shape and mo.normalised_error(got3.cpu().numpy(), want3) < 1e-5
    # strided and dilated, bf16
    xb = torch.from_numpy(rng.standard_normal((8, 64, 30, 29)).astype(np.float32)).to(torch.bfloat16)
    wb = torch.from_numpy((rng.standard_normal((64, 64, 3, 3)) * 0.05).astype(np.float32)).to(torch.bfloat16)
    gotb = T.conv(xb.cuda(), wb.cuda(), stride=(1, 1), dilation=(2, 1), padding=(2, 1))
    wantb = torch.nn.functional.conv2d(xb.double(), wb.double(), dilation=(2, 1), padding=(2, 1)).numpy()
    assert gotb.shape == wantb.shape and mo.normalised_error(gotb.float().cpu().numpy(), wantb) < 2e-2
    # the per-cell kernel on the same f32 problem (threshold lifted) agrees
    keep = T.CONV_CONTRACTION_MIN_WORK
    try:
        T.CONV_CONTRACTION_MIN_WORK = 1 << 62
        ref = T.conv(cu(x[:1]), cu(w), padding=(1, 1))
    finally:
        T.CONV_CONTRACTION_MIN_WORK = keep
    assert mo.normalised_error(got[:1].cpu().numpy(), ref.cpu().numpy().astype(np.float64)) < 1e-5


def test_windows_at_scale_against_torch(T):
    """pool / pad / depthwise conv / flip at sizes where the compiled per-cell walk takes four cells per thread and pass
    (millions of cells), against torch's own operators on the same tensors."""
    F = torch.nn.functional
    g = torch.Generator(device="cuda").manual_seed(77)
    x = torch.randn((8, 64, 224, 224), generator=g, device="cuda")
    assert torch.equal(T.pool("max", x, (2, 2)), F.max_pool2d(x, 2))
    assert torch.equal(T.pool("max", x, (3, 3), (2, 2), (1, 1), (1, 1)), F.max_pool2d(x, 3, 2, 1))
    assert torch.equal(T.pool("min", x, (2, 3), (2, 3)), -F.max_pool2d(-x, (2, 3)))
    got, want = T.pool("sum", x, (3, 3), (1, 1)), F.avg_pool2d(x, 3, 1) * 9
    assert float((got - want).abs().max()) <= 1e-5 * float(want.abs().max())
    assert torch.equal(T.pad(x, (0, 0, 1, 2), (0, 0, 3, 0), -1.5), F.pad(x, (2, 0, 1, 3), value=-1.5))
    assert torch.equal(T.flip(x), torch.flip(x, (0, 1, 2, 3)))
    xb = x.to(torch.bfloat16)
    assert torch.equal(T.pool("max", xb, (2, 2)), F.max_pool2d(xb.float(), 2).to(torch.bfloat16))
    xd = torch.randn((16, 128, 56, 56), generator=g, device="cuda")
    wd = torch.randn((128, 1, 3, 3), generator=g, device="cuda")
    got, want = T.conv_grouped(xd, wd, 128, padding=(1, 1)), F.conv2d(xd, wd, padding=1, groups=128)
    assert float((got - want).abs().max()) <= 1e-5 * float(want.abs().max())
    T.device_status()


def test_strided_slice_of_a_tensor_beyond_2_to_31_elements(T):
    """An operand of more than 2^31 elements makes the compiled walk keep 64-bit offsets; fewer than 2^31 cells are written."""
    rows, cols = (1 << 20) + 2, 2048
    # distinct-looking finite values built in 16-bit arithmetic (no 64-bit temporaries of 2^31 elements): a pattern of row and
    # column with the top exponent bit cleared -- no inf / NaN, whose payload a copy through f32 need not keep
    r16 = torch.arange(rows, device="cuda", dtype=torch.int32).to(torch.int16)[:, None]
    c16 = torch.arange(cols, device="cuda", dtype=torch.int32).to(torch.int16)[None, :]
    x = ((r16 * 251 + c16 * 7) & -16385).view(torch.bfloat16)
    assert x.shape == (rows, cols) and x.numel() > (1 << 31)
    y = T.slice_(x, (1, 0), (2, 1), ((rows - 1) // 2, cols))
    T.device_status()
    assert torch.equal(y.view(torch.int16), x[1::2][: (rows - 1) // 2].view(torch.int16))
