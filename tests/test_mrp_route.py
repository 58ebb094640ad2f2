"""Host-side recognition of `map_reduce_post` instances (mimk_mrp_classify): which descriptors are a contraction,
an axis fold or an elementwise map -- the shapes the derived ops expand to (tensor.mim:1381-1396, 1151-1167) -- and
which must stay on the per-cell kernel. Needs no GPU."""
import pytest
import torch

import __graft_entry__ as entry


@pytest.fixture(scope="module")
def TL():
    entry.build()
    from mimir_b200 import _lib as L
    from mimir_b200 import tensor as T
    return T, L


F32, BF16, I32 = torch.float32, torch.bfloat16, torch.int32
NEG_INF = float("-inf")


def gemm_route(T, L, M, N, K, *, nk=False, dt=F32, post=None, batch=None, a_batched=True, b_batched=True, **kw):
    nb = 0 if batch is None else 1
    n = 3 + nb
    lead = [batch] if nb else []
    lm, ln, lk = nb, nb + 1, nb + 2
    a_map = T.proj_map(n, ([0] if nb and a_batched else []) + [lm, lk])
    b_map = T.proj_map(n, ([0] if nb and b_batched else []) + ([ln, lk] if nk else [lk, ln]))
    a_shape = (lead if a_batched else []) + [M, K]
    b_shape = (lead if b_batched else []) + ([N, K] if nk else [K, N])
    post = L.P_ID if post is None else post
    return T.mrp_route(lead + [M, N], lead + [M, N, K], kw.pop("f", L.F_MULADD), kw.pop("init", 0.0), post,
                       T.proj_map(n, list(range(2 + nb))), [a_map, b_map], [a_shape, b_shape], [dt, dt], **kw)


def test_contractions_are_recognised(TL):
    T, L = TL
    assert gemm_route(T, L, 256, 256, 256) == "gemm"
    assert gemm_route(T, L, 512, 384, 128, nk=True, dt=BF16, out_dtype=BF16) == "gemm"
    assert gemm_route(T, L, 256, 256, 256, post=L.P_RELU) == "gemm"
    assert gemm_route(T, L, 128, 128, 64, batch=8) == "gemm"
    assert gemm_route(T, L, 128, 128, 64, batch=8, b_batched=False) == "gemm"     # one right operand for every batch
    # bias row read at the last write coordinate; full-shape addend at identity
    assert gemm_route(T, L, 256, 256, 256, post=L.P_ADD_RELU, post_maps=[T.proj_map(2, [1])], post_shapes=[[256]],
                      post_dtypes=[F32]) == "gemm"
    assert gemm_route(T, L, 256, 256, 256, post=L.P_ADD, post_maps=[T.id_map(2)], post_shapes=[[256, 256]],
                      post_dtypes=[F32]) == "gemm"


def test_what_is_not_a_dense_contraction_stays_generic(TL):
    T, L = TL
    assert gemm_route(T, L, 64, 64, 64) == "generic"                              # small: keeps the ascending fold
    assert gemm_route(T, L, 256, 256, 256, init=1.0) == "generic"                 # not the ring's zero
    assert gemm_route(T, L, 256, 256, 256, post=L.P_ADD, post_maps=[T.proj_map(2, [0])], post_shapes=[[256]],
                      post_dtypes=[F32]) == "generic"                             # bias along rows: no such epilogue
    # integer contraction: bit-exact wrap-around arithmetic, never re-associated
    assert gemm_route(T, L, 256, 256, 256, dt=I32, init=0, acc_dtype=I32) == "generic"
    # left operand read transposed
    n = 3
    r = T.mrp_route([256, 256], [256, 256, 256], L.F_MULADD, 0.0, L.P_ID, T.proj_map(n, [0, 1]),
                    [T.proj_map(n, [2, 0]), T.proj_map(n, [2, 1])], [[256, 256], [256, 256]], [F32, F32])
    assert r == "generic"
    # a slice of a larger operand: the buffer is not exactly the loop box
    r = T.mrp_route([256, 256], [256, 256, 256], L.F_MULADD, 0.0, L.P_ID, T.proj_map(n, [0, 1]),
                    [T.proj_map(n, [0, 2]), T.proj_map(n, [2, 1])], [[256, 512], [256, 256]], [F32, F32])
    assert r == "generic"
    # packed (transposed) output
    r = T.mrp_route([256, 256], [256, 256, 256], L.F_MULADD, 0.0, L.P_ID, T.proj_map(n, [1, 0]),
                    [T.proj_map(n, [0, 2]), T.proj_map(n, [2, 1])], [[256, 256], [256, 256]], [F32, F32])
    assert r == "generic"


def test_axis_folds_and_maps(TL):
    T, L = TL
    # reduce over each axis of a [64, 128, 256] tensor: loops (o0, o1, r), the folded loop placed at axis `ax`
    shape = [64, 128, 256]
    for ax in range(3):
        out = [s for i, s in enumerate(shape) if i != ax]
        subs = [0, 1]
        subs.insert(ax, 2)
        for f, init in ((L.F_ADD, 0.0), (L.F_MAX, NEG_INF), (L.F_MIN, float("inf"))):
            r = T.mrp_route(out, out + [shape[ax]], f, init, L.P_ID, T.proj_map(3, [0, 1]), [T.proj_map(3, subs)], [shape], [F32])
            assert r == "reduce", (ax, f)
    assert T.mrp_route([2048], [2048, 2048], L.F_MAX, 0.0, L.P_ID, T.proj_map(2, [0]), [T.id_map(2)], [[2048, 2048]], [F32]) == "generic"
    assert T.mrp_route([2048], [2048, 2048], L.F_ADD, 0, L.P_ID, T.proj_map(2, [0]), [T.id_map(2)], [[2048, 2048]], [I32],
                       acc_dtype=I32) == "generic"
    # elementwise: unary, binary, binary_ax (second operand lacks one axis), bias over leading axes
    big = [1024, 2048]
    assert T.mrp_route(big, big, L.F_FIRST, 0.0, L.P_SILU, T.id_map(2), [T.id_map(2)], [big], [F32]) == "map"
    assert T.mrp_route(big, big, L.F_MUL2, 0.0, L.P_ID, T.id_map(2), [T.id_map(2), T.id_map(2)], [big, big], [F32, F32]) == "map"
    assert T.mrp_route(big, big, L.F_SUBEXP, 0.0, L.P_ID, T.id_map(2), [T.id_map(2), T.proj_map(2, [0])], [big, [1024]],
                       [F32, F32]) == "map"
    assert T.mrp_route(big, big, L.F_ADD2, 0.0, L.P_ID, T.id_map(2), [T.id_map(2), T.proj_map(2, [1])], [big, [2048]],
                       [F32, F32]) == "map"
    # a transposing copy is not an elementwise map over identical layouts: it is a tiled copy, for any element type
    assert T.mrp_route([2048, 1024], [2048, 1024], L.F_FIRST, 0.0, L.P_ID, T.id_map(2), [T.proj_map(2, [1, 0])], [big], [F32]) == "permute"
    assert T.mrp_route([2048, 1024], [2048, 1024], L.F_FIRST, 0, L.P_ID, T.id_map(2), [T.proj_map(2, [1, 0])], [big], [I32],
                       acc_dtype=I32) == "permute"
    # ... unless both sides share their fastest axis (coalesced as it is), the shapes do not match, or it is small
    assert T.mrp_route([128, 64, 256], [128, 64, 256], L.F_FIRST, 0.0, L.P_ID, T.id_map(3), [T.proj_map(3, [1, 0, 2])],
                       [[64, 128, 256]], [F32]) == "generic"
    assert T.mrp_route([2048, 1024], [2048, 1024], L.F_FIRST, 0.0, L.P_ID, T.id_map(2), [T.proj_map(2, [1, 0])], [[1024, 4096]],
                       [F32]) == "generic"
    assert T.mrp_route([64, 32], [64, 32], L.F_FIRST, 0.0, L.P_ID, T.id_map(2), [T.proj_map(2, [1, 0])], [[32, 64]], [F32]) == "generic"


def test_bf16_folds_and_maps_are_recognised_too(TL):
    T, L = TL
    big = [1024, 2048]
    assert T.mrp_route([1024], big, L.F_ADD, 0.0, L.P_ID, T.proj_map(2, [0]), [T.id_map(2)], [big], [BF16], out_dtype=BF16) == "reduce"
    assert T.mrp_route([1024], big, L.F_ADD, 0.0, L.P_ID, T.proj_map(2, [0]), [T.id_map(2)], [big], [BF16], out_dtype=F32) == "generic"
    assert T.mrp_route(big, big, L.F_ADD2, 0.0, L.P_ID, T.id_map(2), [T.id_map(2), T.id_map(2)], [big, big], [BF16, BF16],
                       out_dtype=BF16) == "map"
    assert T.mrp_route(big, big, L.F_ADD2, 0.0, L.P_ID, T.id_map(2), [T.id_map(2), T.id_map(2)], [big, big], [BF16, F32]) == "generic"


def test_reshape_maps_are_recognised_and_floordiv_maps_disqualify_the_rest(TL):
    T, L = TL
    # reshape_map of the whole operand (tensor.mim:1224-1233): one copy, at any size and for any element type
    for s_in, s_out in [((3, 4, 5), (10, 6)), ((3, 4, 5), (60,)), ((60,), (3, 4, 5)), ((2048, 512), (1024, 1024))]:
        r = len(s_out)
        for dt in (F32, I32):
            assert T.mrp_route(s_out, s_out, L.F_FIRST, 0.0 if dt == F32 else 0, L.P_ID, T.id_map(r), [T.reshape_map(s_in, s_out)],
                               [s_in], [dt], acc_dtype=dt, out_dtype=dt) == "copy"
    # the division by the innermost stride (1) and the outermost rem may be left out: still a reshape
    m = T.reshape_map((3, 4, 5), (10, 6))
    m.div[2], m.mod[0] = 0, 0
    assert T.mrp_route((10, 6), (10, 6), L.F_FIRST, 0.0, L.P_ID, T.id_map(2), [m], [(3, 4, 5)], [F32]) == "copy"
    # anything else with a floordiv / rem stays on the per-cell kernel: another rem, a fold through a reshape, a contraction
    m = T.reshape_map((3, 4, 5), (10, 6))
    m.mod[1] = 2
    assert T.mrp_route((10, 6), (10, 6), L.F_FIRST, 0.0, L.P_ID, T.id_map(2), [m], [(3, 4, 5)], [F32]) == "generic"
    big = (2048, 4096)
    comp = T.compose_reshape(T.id_map(2), 2, big, (4096, 2048))
    assert T.mrp_route((2048,), big, L.F_ADD, 0.0, L.P_ID, T.proj_map(2, [0]), [comp], [(4096, 2048)], [F32]) == "generic"
    a_map = T.AccessMap(T.proj_map(3, (0, 2)), div=[0, 0], mod=[0, 1024])
    assert T.mrp_route((1024, 1024), (1024, 1024, 1024), L.F_MULADD, 0.0, L.P_ID, T.proj_map(3, (0, 1)),
                       [a_map, T.proj_map(3, (2, 1))], [(1024, 1024), (1024, 1024)], [F32, F32]) == "generic"


def test_folds_with_an_inlined_producer(TL):
    """fold(acc, outer(inner(a, b))): what fuse_map_reduce leaves of a map feeding a reduce (phase/fuse.cpp:183-358)."""
    T, L = TL
    shape = [64, 128, 256]
    sq = L.f_composed(L.F_ADD, L.OP_SQUARE)                       # sum of squares: one input
    sub_sq = L.f_composed(L.F_ADD, L.OP_SUB, L.OP_SQUARE)         # sum of (x - y)^2
    max_abs = L.f_composed(L.F_MAX, L.OP_ABS)
    for ax in range(3):
        out = [s for i, s in enumerate(shape) if i != ax]
        subs = [0, 1]
        subs.insert(ax, 2)
        xm = T.proj_map(3, subs)
        assert T.mrp_route(out, out + [shape[ax]], sq, 0.0, L.P_ID, T.proj_map(3, [0, 1]), [xm], [shape], [F32]) == "reduce"
        assert T.mrp_route(out, out + [shape[ax]], max_abs, NEG_INF, L.P_ID, T.proj_map(3, [0, 1]), [xm], [shape], [F32]) == "reduce"
        # second operand of the producer: x's shape; x's shape without the folded axis; x's axes from the folded one on
        assert T.mrp_route(out, out + [shape[ax]], sub_sq, 0.0, L.P_ID, T.proj_map(3, [0, 1]), [xm, xm], [shape, shape],
                           [F32, F32]) == "reduce"
        assert T.mrp_route(out, out + [shape[ax]], sub_sq, 0.0, L.P_ID, T.proj_map(3, [0, 1]), [xm, T.proj_map(3, [0, 1])],
                           [shape, out], [F32, F32]) == "reduce"
        assert T.mrp_route(out, out + [shape[ax]], sub_sq, 0.0, L.P_ID, T.proj_map(3, [0, 1]), [xm, T.proj_map(3, subs[ax:])],
                           [shape, shape[ax:]], [F32, F32]) == "reduce"
    # the softmax denominator, in its fixed and its general spelling
    big = [1024, 2048]
    for f in (L.F_ADD_SUBEXP, L.f_composed(L.F_ADD, L.OP_SUBEXP)):
        assert T.mrp_route([1024], big, f, 0.0, L.P_ID, T.proj_map(2, [0]), [T.id_map(2), T.proj_map(2, [0])], [big, [1024]],
                           [F32, F32]) == "reduce"
    # not expressible on the fold kernels: a second operand over part of the leading axes only, mixed element types,
    # a fold that does not start from its identity
    assert T.mrp_route([64, 128], [64, 128, 256], sub_sq, 0.0, L.P_ID, T.proj_map(3, [0, 1]),
                       [T.id_map(3), T.proj_map(3, [0])], [shape, [64]], [F32, F32]) == "generic"
    assert T.mrp_route([1024], big, sub_sq, 0.0, L.P_ID, T.proj_map(2, [0]), [T.id_map(2), T.id_map(2)], [big, big],
                       [F32, BF16]) == "generic"
    assert T.mrp_route([1024], big, sq, 1.0, L.P_ID, T.proj_map(2, [0]), [T.id_map(2)], [big], [F32]) == "generic"


def test_composed_combiners_in_the_oracle():
    import numpy as np
    import oracle as mo
    rng = np.random.default_rng(3)
    x = rng.standard_normal((5, 7, 3)).astype(np.float32)
    m = x.max(axis=1)
    proj = lambda n, subs: [[1 if l == s else 0 for l in range(n)] + [0] for s in subs]
    got = mo.map_reduce_post((5, 3), (5, 3, 7), mo.f_composed(0, 22), np.float32(0), mo.P_ID, proj(3, (0, 1)), [proj(3, (0, 2, 1))], [x])
    want = np.zeros((5, 3), np.float32)
    for a in range(7):
        want = want + x[:, a, :] * x[:, a, :]
    assert np.array_equal(got, want)                              # ascending fold, one rounding per operation
    den = mo.map_reduce_post((5, 3), (5, 3, 7), mo.f_composed(0, 6), np.float32(0), mo.P_ID, proj(3, (0, 1)),
                             [proj(3, (0, 2, 1)), proj(3, (0, 1))], [x, m])
    fixed = mo.map_reduce_post((5, 3), (5, 3, 7), mo.F_ADD_SUBEXP_F32, np.float32(0), mo.P_ID, proj(3, (0, 1)),
                               [proj(3, (0, 2, 1)), proj(3, (0, 1))], [x, m])
    assert np.array_equal(den, fixed)
    mabs = mo.map_reduce_post((5, 3), (5, 3, 7), mo.f_composed(2, 23), np.float32(-np.inf), mo.P_ID, proj(3, (0, 1)), [proj(3, (0, 2, 1))], [x])
    assert np.array_equal(mabs, np.abs(x).max(axis=1))
    # the rest of math.mim's unary operators (sqrt, 1 / sqrt, log, exp2, log2, logistic), each behind |x| + 1 or alone
    p = (np.abs(x) + np.float32(1)).astype(np.float32)
    for code, fn in ((24, np.sqrt), (25, lambda v: np.float32(1) / np.sqrt(v)), (26, np.log), (28, np.log2)):
        got = mo.map_reduce_post((5, 7, 3), (5, 7, 3), mo.f_composed(4, code), np.float32(0), mo.P_ID, proj(3, (0, 1, 2)), [proj(3, (0, 1, 2))], [p])
        assert np.allclose(got, fn(p).astype(np.float32), rtol=2e-7, atol=0)
    for code, fn in ((27, np.exp2), (29, lambda v: np.float32(1) / (np.float32(1) + np.exp(-v)))):
        got = mo.map_reduce_post((5, 7, 3), (5, 7, 3), mo.f_composed(4, code), np.float32(0), mo.P_ID, proj(3, (0, 1, 2)), [proj(3, (0, 1, 2))], [x])
        assert np.allclose(got, fn(x).astype(np.float32), rtol=2e-7, atol=0)


def test_elementwise_operators_with_a_unary_one_behind_them(TL):
    T, L = TL
    big = [1024, 2048]
    relu_add = L.f_composed(L.F_FIRST, L.OP_ADD, L.OP_RELU)
    assert T.mrp_route(big, big, relu_add, 0.0, L.P_ID, T.id_map(2), [T.id_map(2), T.proj_map(2, [1])], [big, [2048]], [F32, F32]) == "map"
    assert T.mrp_route(big, big, relu_add, 0.0, L.P_ID, T.id_map(2), [T.id_map(2), T.id_map(2)], [big, big], [F32, F32]) == "map"
    assert T.mrp_route(big, big, L.f_composed(L.F_FIRST, L.OP_SQUARE, L.OP_NEG), 0.0, L.P_ID, T.id_map(2), [T.id_map(2)], [big], [F32]) == "map"
    # a transposed first operand is not an elementwise map
    assert T.mrp_route([2048, 1024], [2048, 1024], relu_add, 0.0, L.P_ID, T.id_map(2), [T.proj_map(2, [1, 0]), T.id_map(2)],
                       [big, [2048, 1024]], [F32, F32]) == "generic"


def _pool_maps(T, stride, dilation):
    mi = [[0] * 7 for _ in range(4)]
    mi[0][0] = mi[1][1] = 1
    mi[2][2], mi[2][4] = stride[0], dilation[0]
    mi[3][3], mi[3][5] = stride[1], dilation[1]
    return mi


def test_which_per_cell_kernel_runs_a_generic_instance(TL):
    """The compiled walk takes floating-point windows / gathers / pads after dropping extent-1 loops and merging the
    neighbours every operand's linear form agrees on; integers and floordiv / rem maps stay on the interpreting kernels."""
    T, L = TL
    # NCHW max pool 2x2 / 2 whose windows tile the rows exactly (32 = 2 * 16): n, c and oh merge -- every operand's form steps
    # extent(inner) * step(inner) per outer index -- and ow stays apart (two columns per step, rows 32 apart)
    shape_in, so = [8, 16, 32, 32], [8, 16, 16, 16]
    pool = lambda dt, **kw: T.mrp_cell_kernel(so, so + [2, 2], L.F_MAX, NEG_INF, L.P_ID, T.proj_map(6, (0, 1, 2, 3)),
                                             [_pool_maps(T, (2, 2), (1, 1))], [shape_in], [dt], **kw)
    assert pool(F32) == ("compiled", 2, 2)
    assert pool(BF16, out_dtype=BF16) == ("compiled", 2, 2)
    assert pool(BF16) == ("linear", 0, 0)                                   # bf16 in, f32 out: not one element type
    # 3x3 / 2 over 33 rows: 16 windows do not tile 33 rows, so oh no longer merges with c; n and c still do
    so3 = [8, 16, 16, 16]
    assert T.mrp_cell_kernel(so3, so3 + [3, 3], L.F_MAX, NEG_INF, L.P_ID, T.proj_map(6, (0, 1, 2, 3)),
                             [_pool_maps(T, (2, 2), (1, 1))], [[8, 16, 33, 33]], [F32]) == ("compiled", 3, 2)
    # a 1x1 "window": the reduction loops have extent 1 and vanish; stride 1 then lets oh and ow merge with everything
    one = T.mrp_cell_kernel(shape_in, shape_in + [1, 1], L.F_MAX, NEG_INF, L.P_ID, T.proj_map(6, (0, 1, 2, 3)),
                            [_pool_maps(T, (1, 1), (1, 1))], [shape_in], [F32])
    assert one == ("compiled", 1, 0)
    # conv, loops (n, co, oh, ow | ci, kh, kw): nothing merges on the output side (x ignores co, w ignores n, oh, ow);
    # kh and kw walk w contiguously but x with a row pitch, so only the weights would merge them
    n, cin, cout, h, kh = 2, 8, 16, 12, 3
    mi = [[0] * 8 for _ in range(4)]
    mi[0][0], mi[1][4] = 1, 1
    mi[2][2], mi[2][5] = 1, 1
    mi[3][3], mi[3][6] = 1, 1
    oh = h - kh + 1
    conv = T.mrp_cell_kernel([n, cout, oh, oh], [n, cout, oh, oh, cin, kh, kh], L.F_MULADD, 0.0, L.P_ID, T.proj_map(7, (0, 1, 2, 3)),
                             [mi, T.proj_map(7, (1, 4, 5, 6))], [[n, cin, h, h], [cout, cin, kh, kh]], [F32, F32])
    assert conv == ("compiled", 4, 3)
    # the same convolution on integers keeps the interpreting walk (linear form: no floordiv / rem)
    convi = T.mrp_cell_kernel([n, cout, oh, oh], [n, cout, oh, oh, cin, kh, kh], L.F_MULADD, 0, L.P_ID, T.proj_map(7, (0, 1, 2, 3)),
                              [mi, T.proj_map(7, (1, 4, 5, 6))], [[n, cin, h, h], [cout, cin, kh, kh]], [I32, I32], acc_dtype=I32)
    assert convi == ("linear", 0, 0)
    # pad: the result is written through o + lo; rows of the padded result are longer than x's, so h and w stay apart
    mo = [[0] * 5 for _ in range(4)]
    for d_ in range(4):
        mo[d_][d_] = 1
    mo[2][4], mo[3][4] = 1, 2
    pad = T.mrp_cell_kernel([8, 16, 35, 34], shape_in, L.F_FIRST, 0.0, L.P_ID, mo, [T.id_map(4)], [shape_in], [F32])
    assert pad == ("compiled", 3, 0)
    # a read through reshape_map (floordiv / rem) is interpreted
    rm = T.reshape_map([6, 4], [24])
    resh = T.mrp_cell_kernel([24], [24], L.F_FIRST, 0.0, L.P_ID, T.id_map(1), [rm], [[6, 4]], [F32])
    assert resh[0] == "interpreted"


def test_loop_merging_of_the_compiled_walk_on_copies_and_grouped_windows(TL):
    T, L = TL
    # flip: every axis reversed -- x's steps are the negated row-major strides, so all four loops still merge into one
    s = [4, 6, 10, 12]
    fm = [[0] * 5 for _ in range(4)]
    for d_ in range(4):
        fm[d_][d_], fm[d_][4] = -1, s[d_] - 1
    assert T.mrp_cell_kernel(s, s, L.F_FIRST, 0.0, L.P_ID, T.id_map(4), [fm], [s], [F32]) == ("compiled", 1, 0)
    # rows 1, 3, 5, ... of a matrix: rows and columns stay apart (x steps two rows where the result steps one)
    sm = [[2, 0, 1], [0, 1, 0]]
    assert T.mrp_cell_kernel([8, 32], [8, 32], L.F_FIRST, 0.0, L.P_ID, T.id_map(2), [sm], [[17, 32]], [F32]) == ("compiled", 2, 0)
    # the patch gather of a convolution run as a contraction: (n, oh, ow, ci, kh, kw) -> six loops, none of them mergeable
    # (3x3 windows over 12 columns: neither the rows of windows nor the windows of a row tile x)
    n, cin, h, kh = 2, 8, 12, 3
    oh = h - kh + 1
    mi = [[0] * 7 for _ in range(4)]
    mi[0][0], mi[1][3] = 1, 1
    mi[2][1], mi[2][4] = 1, 1
    mi[3][2], mi[3][5] = 1, 1
    shape = [n, oh, oh, cin, kh, kh]
    assert T.mrp_cell_kernel(shape, shape, L.F_FIRST, 0.0, L.P_ID, T.id_map(6), [mi], [[n, cin, h, h]], [F32]) == ("compiled", 6, 0)
    # grouped convolution, loops (n, g, co, oh, ow | ci, kh, kw) over x viewed [n, g, ci, H, W] and w viewed [g, co, ci, kh, kw]
    g, co, ci = 4, 2, 3
    mx = [[0] * 9 for _ in range(5)]
    mx[0][0], mx[1][1], mx[2][5] = 1, 1, 1
    mx[3][3], mx[3][6] = 1, 1
    mx[4][4], mx[4][7] = 1, 1
    so = [n, g, co, oh, oh]
    got = T.mrp_cell_kernel(so, so + [ci, kh, kh], L.F_MULADD, 0.0, L.P_ID, T.proj_map(8, (0, 1, 2, 3, 4)),
                            [mx, T.proj_map(8, (1, 2, 5, 6, 7))], [[n, g, ci, h, h], [g, co, ci, kh, kh]], [F32, F32])
    assert got == ("compiled", 5, 3)
    # four reduction loops that do not merge: beyond the compiled walk's three, the interpreting linear walk takes it
    m4 = [[0, 2, 0, 0, 0, 0], [0, 0, 2, 0, 0, 0], [0, 0, 0, 2, 0, 0], [0, 0, 0, 0, 2, 0]]
    got = T.mrp_cell_kernel([5], [5, 2, 2, 2, 2], L.F_ADD, 0.0, L.P_ID, T.proj_map(5, (0,)), [m4], [[3, 3, 3, 3]], [F32])
    assert got == ("linear", 0, 0)
