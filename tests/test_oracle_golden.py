"""Pins the CPU oracle against the reference's own known-answer tests (CPU only, no GPU).

Every case re-creates the inputs of a reference test from the formulas in that test and must reproduce the
answer the reference asserts (an exit code for the integer tests, a tolerance against a double-precision
scalar loop for the floating-point ones).  File names are paths inside the MimIR project.
"""
import numpy as np
import pytest

import oracle as mo


def arange_i32(*shape, start=1):
    return (np.arange(int(np.prod(shape)), dtype=np.int32) + start).reshape(shape)


# ------------------------------------------------------------------ integer known answers
def test_exec_map_reduce_row_sum_42():
    # lit/buffer/exec_map_reduce.mim:25-32 -- row sums of ((1..4),(5..8),(9..12)); out[2] = 42
    t = arange_i32(3, 4)
    out = mo.map_reduce_post((3,), (3, 4), mo.F_ADD_I32, np.int32(0), mo.P_ID, mo.proj_map(2, (0,)),
                             [mo.id_map(2)], [t])
    assert out.tolist() == [10, 26, 42]
    assert mo.reduce(t, 1).tolist() == [10, 26, 42]


def test_exec_epilogue_46():
    # lit/buffer/exec_epilogue.mim:27-38 -- transposed read absorbed into the access map, bias (1,2,3) and +1
    # fused into `post`; out[2] = 42 + 3 + 1 = 46
    t = np.array([[1, 5, 9], [2, 6, 10], [3, 7, 11], [4, 8, 12]], dtype=np.int32)
    bias = np.array([1, 2, 3], dtype=np.int32)
    out = mo.map_reduce_post((3,), (3, 4), mo.F_ADD_I32, np.int32(0), mo.P_ADD_PLUS1_I32, mo.proj_map(2, (0,)),
                             [mo.proj_map(2, (1, 0))], [t], [mo.id_map(1)], [bias])
    assert out.tolist() == [12, 29, 46]
    # the unfused chain gives the same cells
    sums = mo.reduce(mo.transpose_2d(t), 1)
    assert (sums + bias + 1).tolist() == out.tolist()


def test_exec_interchange_47():
    # lit/buffer/exec_interchange.mim:20-27 -- ((1,2,3),(4,5,6)) . b, b[k][j] = k + j; out[1][2] = 47
    a = arange_i32(2, 3)
    b = np.add.outer(np.arange(3), np.arange(4)).astype(np.int32)
    out = mo.product_2d(a, b)
    assert out[1, 2] == 47
    assert (out == a @ b).all()


def test_exec_ktile_8():
    # lit/buffer/exec_ktile.mim:21-26 -- 2x4 ones . 4x2 twos; C[1,1] = 8, also with the K loop split (1, 4)
    a = np.ones((2, 4), np.int32)
    b = np.full((4, 2), 2, np.int32)
    assert mo.product_2d(a, b)[1, 1] == 8
    # dot_schedule's K strip-mine by 4 (tensor.mim:993-995): loops (m, l, ko, ki), k = 4*ko + ki
    ma = np.zeros((2, 5), np.int64); ma[0, 0] = 1; ma[1, 2] = 4; ma[1, 3] = 1
    mb = np.zeros((2, 5), np.int64); mb[0, 2] = 4; mb[0, 3] = 1; mb[1, 1] = 1
    out = mo.map_reduce_post((2, 2), (2, 2, 1, 4), mo.F_MULADD_I32, np.int32(0), mo.P_ID, mo.proj_map(4, (0, 1)),
                             [ma, mb], [a, b])
    assert out[1, 1] == 8


def test_exec_tile_80_packed_output():
    # lit/buffer/exec_tile.mim:23-45 -- A[i][k] = i+1 (4x8), B[k][j] = 2j+1 (8x4); i, j strip-mined by 2, k by 4,
    # loops interchanged to (io, jo, ii, ji, ko, ki); the output is packed (io, ii, jo, ji):
    # C_packed[0,1,1,0] = C[1,2] = 80.
    a = np.repeat(np.arange(1, 5, dtype=np.int32)[:, None], 8, axis=1)
    b = np.repeat(np.array([[1, 3, 5, 7]], dtype=np.int32), 8, axis=0)
    n = 6  # loop vector (io, jo, ii, ji, ko, ki)
    ma = np.zeros((2, n + 1), np.int64); ma[0, 0] = 2; ma[0, 2] = 1; ma[1, 4] = 4; ma[1, 5] = 1   # (2io+ii, 4ko+ki)
    mb = np.zeros((2, n + 1), np.int64); mb[0, 4] = 4; mb[0, 5] = 1; mb[1, 1] = 2; mb[1, 3] = 1   # (4ko+ki, 2jo+ji)
    mout = mo.proj_map(n, (0, 2, 1, 3))                                                           # (io, ii, jo, ji)
    out = mo.map_reduce_post((2, 2, 2, 2), (2, 2, 2, 2, 2, 4), mo.F_MULADD_I32, np.int32(0), mo.P_ID, mout,
                             [ma, mb], [a, b])
    assert out[0, 1, 1, 0] == 80
    c = a @ b
    assert (out.transpose(0, 1, 2, 3).reshape(2, 2, 2, 2) == c.reshape(2, 2, 2, 2)).all()  # (io,ii,jo,ji) is row-major C
    assert c[1, 2] == 80


def _conv_ones(cin):
    # lit/buffer/exec_conv.mim:21-31 -- all-ones conv, stride 1, pad 0: every cell = cin*3*3
    x = np.ones((2, cin, 4, 4), np.int32)
    w = np.ones((2, cin, 3, 3), np.int32)
    n = 7  # (n, co, oh, ow, ci, kh, kw)   tensor.mim:1274-1280
    mi = np.zeros((4, n + 1), np.int64)
    mi[0, 0] = 1; mi[1, 4] = 1; mi[2, 2] = 1; mi[2, 5] = 1; mi[3, 3] = 1; mi[3, 6] = 1
    return mo.map_reduce_post((2, 2, 2, 2), (2, 2, 2, 2, cin, 3, 3), mo.F_MULADD_I32, np.int32(0), mo.P_ID,
                              mo.proj_map(n, (0, 1, 2, 3)), [mi, mo.proj_map(n, (1, 4, 5, 6))], [x, w])


def test_exec_conv_63():
    assert int(_conv_ones(3)[1, 1, 1, 1]) + int(_conv_ones(4)[0, 1, 0, 1]) == 63


def test_btensor_heterogeneous_166_365():
    # lit/btensor/map_reduce_post.mim:22-36 -- I32 and I64 inputs over (2,1,3), I64 epilogue input (100,200),
    # size-1 axes, accumulator I32, result I64: (166, 365)
    a = np.array([[[1, 2, 3]], [[4, 5, 6]]], dtype=np.int32)
    b = np.array([[[10, 20, 30]], [[40, 50, 60]]], dtype=np.int64)
    p = np.array([[100], [200]], dtype=np.int64)
    out = mo.map_reduce_post((2, 1), (2, 1, 3), mo.F_MIX_I32_I64, np.int32(0), mo.P_CONV_ADD_I64,
                             mo.proj_map(3, (0, 1)), [mo.id_map(3), mo.id_map(3)], [a, b], [mo.id_map(2)], [p],
                             out_dtype=mo.I64)
    assert out.reshape(-1).tolist() == [166, 365]


def test_dynamic_bound_counts():
    # lit/btensor/map_reduce_post.mim:41-58 -- scalar output, reduction bound n, every read at index 0 of a
    # buffer of ones: value == n
    src = np.ones(3, np.int32)
    first = np.zeros((1, 2), np.int64)
    for n in (0, 1, 7):
        out = mo.map_reduce_post((), (n,), mo.F_ADD_I32, np.int32(0), mo.P_ID, np.zeros((0, 2), np.int64), [first],
                                 [src])
        assert int(out) == n


# ------------------------------------------------------------------ floating point, reference drivers' formulas
def _attn_inputs(N, D=8):
    # lit/tensor/attn_aux.cpp:28-34
    i = np.arange(N * D)
    x = ((i % 13).astype(np.float32) / np.float32(13.0) - np.float32(0.4)).reshape(N, D)
    j = np.arange(D * D)
    wq = (((7 * j) % 11).astype(np.float32) / np.float32(11.0) - np.float32(0.5)).reshape(D, D)
    wk = (((5 * j) % 9).astype(np.float32) / np.float32(9.0) - np.float32(0.5)).reshape(D, D)
    wv = (((3 * j) % 7).astype(np.float32) / np.float32(7.0) - np.float32(0.5)).reshape(D, D)
    return x, wq, wk, wv


def _attn_double_reference(x, wq, wk, wv):
    # lit/tensor/attn_aux.cpp:36-56, in numpy float64
    xd = x.astype(np.float64)
    q, k, v = xd @ wq.astype(np.float64), xd @ wk.astype(np.float64), xd @ wv.astype(np.float64)
    s = q @ k.T
    p = np.exp(s - s.max(axis=1, keepdims=True))
    p /= p.sum(axis=1, keepdims=True)
    return p @ v


@pytest.mark.parametrize("N", [4, 64])
def test_attn_exec(N):
    x, wq, wk, wv = _attn_inputs(N)
    ref = _attn_double_reference(x, wq, wk, wv)
    out = mo.attention_composed(x, wq, wk, wv)  # f32, the seven map_reduce_post ops
    assert (np.abs(ref - out) <= 1e-4 + 1e-4 * np.abs(ref)).all()  # attn_aux.cpp:62
    # the direct truth routine is the driver's double loop
    q, k, v = (mo.product_2d(x, w) for w in (wq, wk, wv))
    o2 = mo.attention(q[None], k[None], v[None], scale=1.0, causal=False)[0]
    assert (np.abs(ref - o2) <= 1e-4 + 1e-4 * np.abs(ref)).all()
    o3 = mo.attention(q[None], k[None], v[None], scale=1.0, causal=False, truth=False)[0]
    assert (np.abs(ref - o3) <= 1e-4 + 1e-4 * np.abs(ref)).all()


@pytest.mark.parametrize("M,K,N", [(6, 40, 8), (5, 33, 7)])
def test_fc_exec(M, K, N):
    # lit/tensor/fc_aux.cpp:16-42 -- relu(x W^T + b), W stored [N,K]
    i = np.arange(M * K)
    x = ((i % 13).astype(np.float32) / np.float32(13.0) - np.float32(0.4)).reshape(M, K)
    j = np.arange(N * K)
    w = (((7 * j) % 11).astype(np.float32) / np.float32(11.0) - np.float32(0.5)).reshape(N, K)
    bias = ((np.arange(N) % 5).astype(np.float32) / np.float32(5.0) - np.float32(0.4))
    s = x.astype(np.float64) @ w.astype(np.float64).T
    ref = np.maximum((s + bias).astype(np.float32), np.float32(0))
    out = mo.product_2d(x, w, b_transposed=True, post=mo.P_BIAS_RELU_F32, post_in=bias)
    assert (np.abs(ref - out) <= 1e-4 + 1e-4 * np.abs(ref)).all()
    # direct loop == interpreter bit for bit (same fold order)
    assert np.array_equal(mo.gemm(x, w, b_nk=True), mo.product_2d(x, w, b_transposed=True))


def test_hlo_exec_mlp_forward():
    # lit/tensor/hlo_aux.cpp:41-84 -- every array a[i] = (i % 100)/100; rel <= 1e-3 on the 128 outputs
    B, IN, H, OUT = 128, 784, 1024, 10

    def init(n):
        return ((np.arange(n) % 100).astype(np.float32) / np.float32(100.0))

    arg0, arg1, arg2, arg3 = init(IN * H).reshape(IN, H), init(H), init(H * H).reshape(H, H), init(H)
    arg4, arg5, arg6 = init(H * OUT).reshape(H, OUT), init(OUT), init(B * IN).reshape(B, IN)
    h0 = np.tanh(mo.gemm(arg6, arg0) + arg1)
    h1 = np.tanh(mo.gemm(h0, arg2) + arg3)
    out = (mo.gemm(h1, arg4) + arg5).max(axis=1)
    d0 = np.tanh(arg6.astype(np.float64) @ arg0 + arg1)
    d1 = np.tanh(d0 @ arg2 + arg3)
    ref = (d1 @ arg4 + arg5).max(axis=1)
    rel = np.abs(ref - out) / (np.abs(ref) + 1e-6)
    assert rel.max() <= 1e-3
    # the interpreter with the fused bias+tanh epilogue agrees with the direct loop on a slice of layer 0
    sl = mo.product_2d(arg6[:4], np.ascontiguousarray(arg0[:, :16]), post=mo.P_BIAS_TANH_F32,
                       post_in=np.ascontiguousarray(arg1[:16]))
    assert np.allclose(sl, h0[:4, :16], rtol=0, atol=1e-6)


def test_reduce_exec():
    # lit/tensor/reduce_exec.mim:19-43 -- x[a,b,c] = 12a + 4b + c over (2,3,4)
    x = np.arange(24, dtype=np.float32).reshape(2, 3, 4)
    a, b = np.meshgrid(np.arange(3), np.arange(4), indexing="ij")
    assert np.abs(mo.reduce(x, 0) - (12 + 2 * (4 * a + b))).max() < 1e-5
    a, b = np.meshgrid(np.arange(2), np.arange(4), indexing="ij")
    assert np.abs(mo.reduce(x, 1) - (36 * a + 12 + 3 * b)).max() < 1e-5
    a, b = np.meshgrid(np.arange(2), np.arange(3), indexing="ij")
    assert np.abs(mo.reduce(x, 2) - (48 * a + 16 * b + 6)).max() < 1e-5
    p = mo.softmax(x, 1)
    assert np.abs(mo.reduce(p, 1) - 1.0).max() < 1e-5
    peak = 1.0 / (1.0 + np.exp(-4.0) + np.exp(-8.0))
    assert abs(p[1, 2, 3] - peak) < 1e-5
    total = mo.reduce(mo.reduce(mo.reduce(x, 0), 0), 0)
    assert abs(float(total) - 276.0) < 1e-5
    # direct loops agree with the interpreter
    for ax in range(3):
        assert np.array_equal(mo.reduce_axis(x, ax), mo.reduce(x, ax))
    assert np.allclose(mo.softmax_rows(x.reshape(6, 4)), mo.softmax(x.reshape(6, 4), 1), rtol=0, atol=0)


# ------------------------------------------------------------------ oracle self-consistency on seeded inputs
def test_direct_loops_match_interpreter_seeded():
    rng = np.random.default_rng(7)
    a = rng.uniform(-1, 1, (9, 17)).astype(np.float32)
    b = rng.uniform(-1, 1, (17, 5)).astype(np.float32)
    assert np.array_equal(mo.gemm(a, b), mo.product_2d(a, b))
    t = mo.gemm_truth(a, b)
    assert np.allclose(t, mo.product_2d(a, b, mode="f64"), rtol=1e-14, atol=0)
    assert mo.normalised_error(mo.gemm(a, b), t) < 1e-6
    assert np.array_equal(mo.gemm_truth(a, b, rows=[3, 8]), t[[3, 8]])


def test_bf16_round_to_nearest_even():
    x = np.array([1.0, 1.00390625, 1.01171875, -2.5, 3.4028234663852886e38, np.inf, 0.0], dtype=np.float32)
    y = mo.from_bf16(mo.to_bf16(x))
    # 1 + 2^-8 is a tie -> even mantissa (1.0); 1 + 3*2^-8 is a tie -> rounds up to even 1.015625
    assert y[0] == 1.0 and y[1] == 1.0 and y[2] == np.float32(1.015625) and y[3] == -2.5
    assert np.isinf(y[4]) and np.isinf(y[5]) and y[6] == 0.0
    try:
        import torch
    except ImportError:
        return
    r = np.random.default_rng(0).standard_normal(4096).astype(np.float32)
    t = torch.from_numpy(r).to(torch.bfloat16).view(torch.int16).numpy().view(np.uint16)
    assert np.array_equal(t, mo.to_bf16(r))


def test_causal_attention_matches_masked_dense():
    rng = np.random.default_rng(3)
    q, k, v = (rng.standard_normal((2, 16, 8)).astype(np.float32) for _ in range(3))
    o = mo.attention(q, k, v, scale=0.25, causal=True)
    s = np.einsum("hid,hjd->hij", q.astype(np.float64), k.astype(np.float64)) * 0.25
    s = np.where(np.tril(np.ones((16, 16), bool)), s, -np.inf)
    p = np.exp(s - s.max(-1, keepdims=True))
    p /= p.sum(-1, keepdims=True)
    assert np.allclose(o, p @ v.astype(np.float64), rtol=1e-12, atol=1e-12)
    o32 = mo.attention(q, k, v, scale=0.25, causal=True, truth=False)
    assert mo.normalised_error(o32, o) < 1e-5
    assert np.array_equal(mo.attention(q, k, v, scale=0.25, causal=True, heads=[1])[0], o[1])


# ------------------------------------------------------------------ constructors and data-dependent indexing
def test_generate_exec_30():
    # lit/tensor/generate_exec.mim:12-20 -- generate (2, 3) with body (i, _) -> i == 0 ? 10 : 20; g[0,2] + g[1,1] = 30
    g = mo.generate((2, 3), lambda i, _j: np.int32(10 if i == 0 else 20))
    assert int(g[0, 2]) + int(g[1, 1]) == 30


def test_gather_scatter_exec_93():
    # lit/tensor/gather_scatter_exec.mim:15-21 -- gather / scatter along axis 1; 12 + 21 + 20 + 40 = 93, the duplicate
    # destination (1, 1) keeps the later update
    x = np.array([[10, 11, 12], [20, 21, 22]], dtype=np.int32)
    index = np.array([[2, 0], [1, 1]], dtype=np.int32)
    updates = np.array([[10, 20], [30, 40]], dtype=np.int32)
    g = mo.gather(1, x, index)
    s = mo.scatter(1, x, index, updates)
    assert g.tolist() == [[12, 10], [21, 21]]
    assert s.tolist() == [[20, 11, 10], [20, 40, 22]]
    assert int(g[0, 0]) + int(g[1, 0]) + int(s[0, 0]) + int(s[1, 1]) == 93


# ------------------------------------------------------------------ the remaining integer known answers of lit/buffer and lit/btensor
def _pad(x, lo, hi, value):
    """tensor.pad, constant mode (tensor.mim:275-290): the result filled with `value`, the input copied in at offset lo."""
    r = x.ndim
    shape = [lo[d] + x.shape[d] + hi[d] for d in range(r)]
    mo_ = np.zeros((r, r + 1), np.int64)
    for d in range(r):
        mo_[d, d], mo_[d, r] = 1, lo[d]
    return mo.map_reduce_post(shape, x.shape, mo.F_FIRST_I32, np.int32(0), mo.P_ID, mo_, [mo.id_map(r)], [x],
                              dst=np.full(shape, value, x.dtype))


def _set(t, index, value):
    s = t.copy()
    s[index] = value                # tensor.set: a copy with one cell replaced (tensor.mim, `set`)
    return s


def test_exec_strip_24():
    # lit/buffer/exec_strip.mim:16-29 -- ones (2, 8, 3) summed over the last two axes with the 8-loop strip-mined by 4:
    # loops (i, jo, ji, k), input read at (i, 4 jo + ji, k); out[1] = 24
    t = np.ones((2, 8, 3), np.int32)
    mi = np.zeros((3, 5), np.int64); mi[0, 0] = 1; mi[1, 1] = 4; mi[1, 2] = 1; mi[2, 3] = 1
    out = mo.map_reduce_post((2,), (2, 2, 4, 3), mo.F_ADD_I32, np.int32(0), mo.P_ID, mo.proj_map(4, (0,)), [mi], [t])
    assert out.tolist() == [24, 24]


def test_exec_unroll_111():
    # lit/buffer/exec_unroll.mim:18-28 -- ones (2, 37, 3), an unroll schedule that changes no value; out[1] = 111
    t = np.ones((2, 37, 3), np.int32)
    out = mo.map_reduce_post((2,), (2, 37, 3), mo.F_ADD_I32, np.int32(0), mo.P_ID, mo.proj_map(3, (0,)), [mo.id_map(3)], [t])
    assert int(out[1]) == 111


def test_exec_size1_42_and_pad_concat_42():
    # lit/buffer/exec_size1.mim:14-28 -- size-1 axes: pad (1,3) by one cell of 5 on either side of axis 1, concat along 0
    a = np.array([[7, 8, 9]], np.int32)
    b = np.array([[10, 20, 30], [4, 5, 6]], np.int32)
    p = _pad(a, (0, 1), (0, 1), 5)
    c = mo.concat(0, [a, b])
    assert p.tolist() == [[5, 7, 8, 9, 5]]
    assert int(c[1, 2]) + int(p[0, 1]) + int(p[0, 0]) == 42
    # lit/buffer/exec_pad_concat.mim:13-27 -- rank 1: pad by (1, 2), concat of lengths 3 and 2
    t, u = np.array([10, 20, 30], np.int32), np.array([1, 2], np.int32)
    p = _pad(t, (1,), (2,), 5)
    c = mo.concat(0, [t, u])
    assert p.tolist() == [5, 10, 20, 30, 5, 5]
    assert int(p[3]) + int(c[4]) + int(c[0]) == 42


def test_exec_get_set_50_local_tensors_42_and_same_shape_42():
    # lit/buffer/exec_get_set.mim:9-16
    t = (np.arange(12, dtype=np.int32) + 1).reshape(3, 4)
    s = _set(t, (0, 0), 42)
    assert int(s[0, 0]) + int(s[1, 2]) + int(t[0, 0]) == 50
    # lit/buffer/exec_local_tensors.mim:12-16 -- broadcast (1, 2) -> (2, 2) as a copy whose read map drops the unit axis
    m = np.array([[10, 20], [30, 40]], np.int32)
    s = _set(m, (1, 1), 2)
    row = np.array([[5, 7]], np.int32)
    bmap = np.zeros((2, 3), np.int64); bmap[1, 1] = 1
    b = mo.map_reduce_post((2, 2), (2, 2), mo.F_FIRST_I32, np.int32(0), mo.P_ID, mo.id_map(2), [bmap], [row])
    assert b.tolist() == [[5, 7], [5, 7]]
    assert int(s[1, 1]) + int(s[1, 0]) + int(b[1, 0]) + int(b[0, 0]) == 42
    # lit/buffer/two_same_shape_binary.mim:11-24 -- two maps of one shape, concatenated
    x = np.array([[10, 1, 2, 3], [4, 5, 30, 7], [8, 9, 10, 11]], np.int32)
    y = np.array([[5, 1, 1, 1], [1, 1, 3, 1], [1, 1, 1, 1]], np.int32)
    c = mo.concat(0, [x + y, x - y])
    assert int(c[0, 0]) + int(c[4, 2]) == 42
    # lit/buffer/two_same_shape_set.mim:8-18 -- two sets of one tensor do not see each other
    t = np.array([[12, 2, 3, 4], [5, 6, 30, 8], [9, 10, 11, 12]], np.int32)
    a, b = _set(t, (0, 0), 2), _set(t, (1, 2), 40)
    assert int(a[1, 2]) + int(b[0, 0]) == 42


def test_btensor_read_transpose_5():
    # lit/btensor/read_transpose.mim:12-24 -- a (2, 4) buffer of fives copied through proj_map (1, 0) into (4, 2); cell [3, 1]
    m = np.full((2, 4), 5, np.int32)
    d = mo.map_reduce_post((4, 2), (4, 2), mo.F_FIRST_I32, np.int32(0), mo.P_ID, mo.id_map(2), [mo.proj_map(2, (1, 0))], [m])
    assert int(d[3, 1]) == 5 and d.shape == (4, 2)


def test_reshape_map_and_packed_unpack():
    """Access maps with floordiv / rem: `reshape_map` (tensor.mim:1224-1233) alone, the unpack copy behind a packed
    dot_product (tensor.mim:1405-1411: the packed result of exec_tile reshaped... here through reshape_map of its packed
    shape), and a consumer that reads a reshape through a composed map (fuse_read_through, fuse.cpp:542-589)."""
    x = (np.arange(60, dtype=np.int32) * 7 - 100).reshape(3, 4, 5)
    y = mo.map_reduce_post((10, 6), (10, 6), mo.F_FIRST_I32, np.int32(0), mo.P_ID, mo.id_map(2), [mo.reshape_map((3, 4, 5), (10, 6))], [x])
    assert np.array_equal(y, x.reshape(10, 6))
    # exec_tile's packed product C_packed[io, ii, jo, ji] (lit/buffer/exec_tile.mim:23-45): a reshape of the packed shape
    # (2,2,2,2) to (4,4) is NOT the matrix (the packing interleaves jo and ii); reading it through the packing's own map is
    a = np.repeat(np.arange(1, 5, dtype=np.int32)[:, None], 8, axis=1)
    b = np.repeat(np.array([[1, 3, 5, 7]], dtype=np.int32), 8, axis=0)
    ma = np.zeros((2, 7), np.int64); ma[0, 0] = 2; ma[0, 2] = 1; ma[1, 4] = 4; ma[1, 5] = 1
    mb = np.zeros((2, 7), np.int64); mb[0, 4] = 4; mb[0, 5] = 1; mb[1, 1] = 2; mb[1, 3] = 1
    packed = mo.map_reduce_post((2, 2, 2, 2), (2, 2, 2, 2, 2, 4), mo.F_MULADD_I32, np.int32(0), mo.P_ID,
                                mo.proj_map(6, (0, 2, 1, 3)), [ma, mb], [a, b])
    flat = mo.map_reduce_post((16,), (16,), mo.F_FIRST_I32, np.int32(0), mo.P_ID, mo.id_map(1), [mo.reshape_map((2, 2, 2, 2), (16,))], [packed])
    assert np.array_equal(flat, packed.reshape(16))
    # row sums of a (6, 10) VIEW of a tensor stored (3, 4, 5): the consumer's map (o, r) composed behind the reshape
    lin = [10, 1, 0]
    comp = mo.DivModMap([lin, lin, lin], [20, 5, 1], [3, 4, 5])
    sums = mo.map_reduce_post((6,), (6, 10), mo.F_ADD_I32, np.int32(0), mo.P_ID, mo.proj_map(2, (0,)), [comp], [x])
    assert np.array_equal(sums, x.reshape(6, 10).sum(1))


# ------------------------------------------------------------------ the reference's training-step fixtures, through the oracle
def test_hlo_train_fixture_through_the_interpreter():
    """lit/tensor/hlo_train_aux.cpp:24-76 -- one training step of a one-layer tanh MLP (N=4, I=8, O=3) for the fixture's three
    input patterns, every contraction and fold through the map_reduce_post interpreter (as lowered, f32), held to the
    fixture's 1e-4 against its own scalar recipe in f64."""
    N, I, O, lr, c = 4, 8, 3, 0.001, 0.5
    for mode in range(3):
        def make(n):
            i = np.arange(n)
            v = (i % 100) / np.float32(100.0) if mode == 0 else (np.full(n, 0.5) if mode == 1 else 0.01 * ((i % 7) + 1))
            return v.astype(np.float32)
        w, b, x, t = make(I * O).reshape(I, O), make(O), make(N * I).reshape(N, I), make(N * O).reshape(N, O)
        z64 = x.astype(np.float64) @ w.astype(np.float64)
        d64 = c * (np.tanh(z64 + b) - t)
        ref = (w[0, 0] - lr * (x.T.astype(np.float64) @ d64)[0, 0]) + (b[0] - lr * d64.sum(0)[0]) + (d64 @ w.T.astype(np.float64))[0, 0] + z64[0].max()
        z = mo.product_2d(x, w)
        a = mo.product_2d(x, w, post=mo.P_BIAS_TANH_F32, post_in=b)
        d = (np.float32(c) * (a - t)).astype(np.float32)
        dW = mo.product_2d(mo.transpose_2d(x), d)                       # x^T d
        dx = mo.product_2d(d, w, b_transposed=True)                     # d w^T: w read through transpose_2d
        db = mo.reduce(d, 0)
        got = (w[0, 0] - lr * dW[0, 0]) + (b[0] - lr * db[0]) + dx[0, 0] + mo.reduce(z, 1, "max")[0]
        assert abs(float(got) - float(ref)) <= 1e-4, (mode, got, ref)


def test_hlo_step_fixture_through_the_direct_loops():
    """lit/tensor/hlo_step_aux.cpp:33-158 -- one SGD step of the tanh MLP 128/784/1024/10 (softmax-loss gradient, backward
    contractions over transposed reads, column sums, the digest of six update deltas): the contractions and folds on the
    oracle's as-lowered f32 loops, against the same program in f64; the fixture's bound (1e-2 of the digest's scale + 1e-6)."""
    B, I, H, O, lr, c = 128, 784, 1024, 10, np.float32(0.001), np.float32(-0.0078125)

    def pat(n, mod, mul, sub):
        return (mul * ((np.arange(n) % mod).astype(np.float32) / np.float32(mod) - np.float32(sub))).astype(np.float32)
    W1, W2, W3 = pat(I * H, 89, 0.05, 0.5).reshape(I, H), pat(H * H, 83, 0.05, 0.5).reshape(H, H), pat(H * O, 79, 0.1, 0.5).reshape(H, O)
    b1 = (0.01 * ((np.arange(H) % 7).astype(np.float32) - 3.0)).astype(np.float32)
    b2 = (0.01 * ((np.arange(H) % 5).astype(np.float32) - 2.0)).astype(np.float32)
    b3 = (0.01 * ((np.arange(O) % 3).astype(np.float32) - 1.0)).astype(np.float32)
    X = pat(B * I, 97, 0.05, 0.0).reshape(B, I)
    Y = np.zeros((B, O), np.float32)
    Y[np.arange(B), np.arange(B) % O] = 1.0

    def step(mm, colsum, rowsum, rowmax, dt):
        X_, Y_, W1_, W2_, W3_ = (a.astype(dt) for a in (X, Y, W1, W2, W3))
        h1 = np.tanh(mm(X_, W1_) + b1.astype(dt))
        h2 = np.tanh(mm(h1, W2_) + b2.astype(dt))
        logits = mm(h2, W3_) + b3.astype(dt)
        e = np.exp(logits - rowmax(logits)[:, None])
        q = rowsum(Y_ * dt(-c)) / rowsum(e)
        dlog = Y_ * dt(c) + e * q[:, None]
        v59 = mm(dlog, W3_.T.copy())
        v66 = mm(v59, W2_.T.copy()) * (1 - h1)
        v68 = v66 + v66 * h1
        return [mm(X_.T.copy(), v68)[3, 5], colsum(v68)[7], mm(h1.T.copy(), v59)[11, 13], colsum(v59)[17],
                mm(h2.T.copy(), dlog)[19, 2], colsum(dlog)[3]]

    ref = step(lambda a, b: a @ b, lambda m: m.sum(0), lambda m: m.sum(1), lambda m: m.max(1), np.float64)
    got = step(lambda a, b: mo.gemm(a, b), lambda m: mo.reduce_axis(m, 0), lambda m: mo.reduce_axis(m, 1),
               lambda m: mo.reduce_axis(m, 1, "max"), np.float32)
    olds = [W1[3, 5], b1[7], W2[11, 13], b2[17], W3[19, 2], b3[3]]
    delta = lambda old, g: float(np.float32(old) - (np.float32(old) - lr * np.float32(g)))
    g_ref, g_got = [delta(o, g) for o, g in zip(olds, ref)], [delta(o, g) for o, g in zip(olds, got)]
    scale = sum(abs(v) for v in g_ref)
    assert abs(sum(g_got) - sum(g_ref)) <= 1e-2 * scale + 1e-6
