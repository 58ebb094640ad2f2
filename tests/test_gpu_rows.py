"""GPU parity: reduce / softmax / RMSNorm / elementwise against the CPU oracle, through the C ABI."""
import numpy as np
import pytest
import torch

import oracle as mo
from tests.util import TOL_BF16, TOL_F32, f64, nerr, randn, uniform

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def T():
    from mimir_b200 import tensor
    return tensor


def test_reduce_exec_fixture(T):
    # lit/tensor/reduce_exec.mim:19-43 on the device
    x = torch.arange(24, dtype=torch.float32).reshape(2, 3, 4).cuda()
    xn = x.cpu().numpy()
    for ax in range(3):
        assert np.abs(T.reduce("sum", ax, x).cpu().numpy() - mo.reduce(xn, ax)).max() < 1e-5
    p = T.softmax(1, x)
    assert np.abs(T.reduce("sum", 1, p).cpu().numpy() - 1.0).max() < 1e-5
    peak = 1.0 / (1.0 + np.exp(-4.0) + np.exp(-8.0))
    assert abs(float(p[1, 2, 3]) - peak) < 1e-5
    total = T.reduce("sum", 0, T.reduce("sum", 0, T.reduce("sum", 0, x)))
    assert abs(float(total) - 276.0) < 1e-5
    assert nerr(p.cpu().numpy(), mo.softmax(xn, 1)) < TOL_F32


@pytest.mark.parametrize("rows,cols", [(3, 4), (7, 33), (64, 128), (33, 1000), (16, 4096), (8, 8192), (4, 16384),
                                       (2, 32768), (2, 40000), (5, 8190)])
def test_softmax_rows_f32(T, rows, cols):
    x = randn((rows, cols), 11 + cols)
    y = T.softmax(1, x)
    want = mo.softmax_rows(x.cpu().numpy(), truth=True)
    assert nerr(f64(y), want) < TOL_F32
    # as-lowered f32 oracle: same ops, different summation order
    assert nerr(f64(y), mo.softmax_rows(x.cpu().numpy())) < TOL_F32


@pytest.mark.parametrize("rows,cols", [(16, 8192), (9, 1024), (5, 100)])
def test_softmax_and_rmsnorm_to_bf16(T, rows, cols):
    x = randn((rows, cols), 5)
    gamma = uniform((cols,), 6, 0.5, 1.5)
    y = T.softmax(1, x, out_dtype=torch.bfloat16)
    assert y.dtype == torch.bfloat16
    want = mo.softmax_rows(x.cpu().numpy(), truth=True)
    assert nerr(f64(y), want) < TOL_BF16
    # the stored value is the f32 result rounded to nearest even: compare bit patterns with the f32 kernel
    y32 = T.softmax(1, x)
    assert torch.equal(y, y32.to(torch.bfloat16))
    z = T.rmsnorm(x, gamma, 1e-6, out_dtype=torch.bfloat16)
    wz = mo.rmsnorm_rows(x.cpu().numpy(), gamma.cpu().numpy(), 1e-6, truth=True)
    assert nerr(f64(z), wz) < TOL_BF16
    z32 = T.rmsnorm(x, gamma, 1e-6)
    assert nerr(f64(z32), wz) < TOL_F32
    assert torch.equal(z, z32.to(torch.bfloat16))


def test_softmax_rmsnorm_chain(T):
    x = randn((12, 2048), 21)
    gamma = uniform((2048,), 22, 0.5, 1.5)
    fused = T.softmax_rmsnorm(x, gamma, 1e-6)
    p = mo.softmax_rows(x.cpu().numpy(), truth=True)
    want = p / np.sqrt((p * p).mean(axis=1, keepdims=True) + 1e-6) * gamma.cpu().numpy().astype(np.float64)
    assert nerr(f64(fused), want) < TOL_F32
    x2 = randn((3, 1001), 23)      # generic (unaligned) kernel
    g2 = uniform((1001,), 24, 0.5, 1.5)
    p2 = mo.softmax_rows(x2.cpu().numpy(), truth=True)
    w2 = p2 / np.sqrt((p2 * p2).mean(axis=1, keepdims=True) + 1e-6) * g2.cpu().numpy().astype(np.float64)
    assert nerr(f64(T.softmax_rmsnorm(x2, g2, 1e-6)), w2) < TOL_F32


def test_softmax_bf16_input(T):
    x = randn((6, 512), 31, dtype=torch.bfloat16)
    y = T.softmax(1, x)
    want = mo.softmax_rows(x.float().cpu().numpy(), truth=True)
    assert nerr(f64(y), want) < TOL_BF16


@pytest.mark.parametrize("shape,ax", [((5, 7, 9), 0), ((5, 7, 9), 1), ((5, 7, 9), 2), ((1, 5000, 64), 1),
                                      ((300, 4096), 1), ((2048, 130), 0), ((3, 1), 1)])
@pytest.mark.parametrize("monoid", ["sum", "max", "min"])
def test_reduce_axes(T, shape, ax, monoid):
    x = randn(shape, 41 + ax)
    got = T.reduce(monoid, ax, x)
    want = mo.reduce_axis(x.cpu().numpy(), ax, monoid, truth=True)
    assert got.shape == want.shape
    if monoid == "sum":
        # error of an f32 sum, relative to the largest partial magnitude
        scale = np.abs(x.cpu().numpy().astype(np.float64)).sum(axis=ax).max()
        assert np.abs(f64(got) - want).max() <= 1e-6 * scale + 1e-6
    else:
        assert np.array_equal(got.cpu().numpy().astype(np.float64), want)


def test_softmax_middle_axis(T):
    x = randn((4, 37, 6), 51)
    got = T.softmax(1, x)
    assert nerr(f64(got), mo.softmax(x.cpu().numpy(), 1)) < TOL_F32


def test_softmax_middle_axis_bf16(T):
    # bf16 operands along an axis that is not the last one (statistics in f32, result rounded to bf16)
    x = randn((4, 37, 6), 52, dtype=torch.bfloat16)
    want = mo.softmax(x.float().cpu().numpy(), 1)
    assert nerr(f64(T.softmax(1, x)), want) < TOL_BF16
    assert nerr(f64(T.softmax(1, x, out_dtype=torch.float32)), want) < TOL_F32


def test_bmm_rejects_mixed_element_types(T):
    a = randn((2, 8, 8), 53)
    with pytest.raises(TypeError):
        T.bmm(a, a.to(torch.bfloat16))


def test_elementwise_and_binary_ax(T):
    x = randn((6, 10, 4), 61)
    y = randn((6, 10, 4), 62)
    xn, yn = x.cpu().numpy(), y.cpu().numpy()
    assert np.allclose(T.binary("add", x, y).cpu().numpy(), xn + yn, rtol=0, atol=0)
    assert np.allclose(T.binary("mul", x, y).cpu().numpy(), xn * yn, rtol=0, atol=0)
    assert np.allclose(T.unary("relu", x).cpu().numpy(), np.maximum(xn, 0), rtol=0, atol=0)
    assert np.allclose(T.unary("tanh", x).cpu().numpy(), np.tanh(xn), rtol=1e-6, atol=1e-6)
    mx = T.reduce("max", 1, x)
    e = T.binary_ax("subexp", 1, x, mx)
    want = mo.binary_ax(mo.F_SUBEXP_F32, 1, xn, mx.cpu().numpy())
    assert nerr(e.cpu().numpy(), want) < TOL_F32
    # the reference's own four-op softmax, run op by op on the device, equals the fused kernel
    s = T.binary_ax("div", 1, e, T.reduce("sum", 1, e))
    assert nerr(f64(s), f64(T.softmax(1, x))) < TOL_F32


def test_empty_and_degenerate(T):
    e = torch.empty((0, 16), device="cuda")
    assert T.softmax(1, e).shape == (0, 16)
    assert T.reduce("sum", 1, e).shape == (0,)
    one = randn((4, 1), 71)
    assert torch.equal(T.softmax(1, one), torch.ones_like(one))
    z = T.reduce("sum", 1, torch.empty((3, 0), device="cuda"))
    assert torch.equal(z, torch.zeros(3, device="cuda"))
    m = T.reduce("max", 1, torch.empty((3, 0), device="cuda"))
    assert torch.isinf(m).all() and (m < 0).all()


def test_full_size_softmax_properties(T):
    # the bench workload's shape: rows sum to one, argmax preserved, idempotent statistics
    x = randn((16384, 8192), 81)
    y = T.softmax(1, x, out_dtype=torch.bfloat16)
    sums = y.float().sum(dim=1)
    assert (sums - 1).abs().max() < 2e-2
    assert torch.equal(y.float().argmax(dim=1), x.argmax(dim=1)) or \
        (y.float().max(dim=1).values == y.float().gather(1, x.argmax(dim=1, keepdim=True)).squeeze(1)).all()
    rows = [0, 1, 8191, 16383]
    want = mo.softmax_rows(x[rows].cpu().numpy(), truth=True)
    assert nerr(f64(y[rows]), want) < TOL_BF16


def test_elementwise_operators_on_bf16_operands():
    """unary / binary / binary_ax with BF16 operands: arithmetic in f32 on the exact operand values, one rounding at the
    store -- bit-identical to f32 arithmetic on the widened operands followed by round-to-nearest-even."""
    from mimir_b200 import tensor as T
    g = torch.Generator().manual_seed(6)
    for shape in ((64, 1024), (7, 33, 5)):                       # the 128-bit path and the scalar path
        x = torch.randn(shape, generator=g).to(torch.bfloat16).cuda()
        y = torch.randn(shape, generator=g).to(torch.bfloat16).cuda()
        assert torch.equal(T.binary("add", x, y), (x.float() + y.float()).to(torch.bfloat16))
        assert torch.equal(T.binary("mul", x, y, out_dtype=torch.float32), x.float() * y.float())
        assert torch.equal(T.unary("relu", x), torch.relu(x))
        got = T.unary("silu", x, out_dtype=torch.float32)
        want = x.double() / (1 + torch.exp(-x.double()))
        assert ((got.double() - want).abs().max() / want.abs().max()).item() <= 1e-5
        for ax in range(len(shape)):
            yb = torch.randn([s for i, s in enumerate(shape) if i != ax], generator=g).to(torch.bfloat16).cuda()
            assert torch.equal(T.binary_ax("sub", ax, x, yb), (x.float() - yb.float().unsqueeze(ax)).to(torch.bfloat16))
    with pytest.raises(TypeError):
        T.binary("add", torch.zeros(4, device="cuda"), torch.zeros(4, device="cuda", dtype=torch.bfloat16))


def test_reduce_on_bf16_operands():
    """reduce with BF16 operands: f32 accumulation of the exact operand values, one rounding at the store; every axis of a
    rank-3 tensor (row kernel, middle-axis kernel with and without a split of the folded axis)."""
    from mimir_b200 import tensor as T
    g = torch.Generator().manual_seed(12)
    for shape in ((48, 1024, 8), (6, 4096, 3), (33, 70, 129)):
        x = torch.randn(shape, generator=g).to(torch.bfloat16).cuda()
        for ax in range(3):
            assert torch.equal(T.reduce("max", ax, x), x.amax(ax))
            s = T.reduce("sum", ax, x)
            want = x.double().sum(ax)
            assert s.dtype == torch.bfloat16
            assert ((s.double() - want).abs().max() / want.abs().max()).item() <= TOL_BF16


@pytest.mark.parametrize("shape,ax", [((37, 1000), 1), ((64, 4096), 1), ((6, 300, 40), 1), ((2048, 96), 0), ((3, 5, 7), 2),
                                      ((8, 4100, 24), 1)])
def test_reduce_with_an_inlined_producer(T, shape, ax):
    """Folds over produced values (phase/fuse.cpp:183-358): the produced tensor is never written."""
    x = randn(shape, 5 + ax + shape[-1])
    xn = x.cpu().numpy().astype(np.float64)
    red_shape = tuple(s for i, s in enumerate(shape) if i != ax)
    # sum of squares (RMSNorm's statistic), largest magnitude
    assert nerr(f64(T.reduce_fused("sum", ax, x, "square")), (xn * xn).sum(axis=ax)) < TOL_F32
    assert np.array_equal(T.reduce_fused("max", ax, x, "abs").cpu().numpy(), np.abs(x.cpu().numpy()).max(axis=ax))
    # the softmax denominator: sum of exp(x - max), y broadcast along the folded axis
    mx = T.reduce("max", ax, x)
    den = T.reduce_fused("sum", ax, x, "subexp", mx)
    want = np.exp(xn - np.expand_dims(xn.max(axis=ax), ax)).sum(axis=ax)
    assert den.shape == red_shape and nerr(f64(den), want) < TOL_F32
    # variance numerator: sum of (x - mean)^2
    mean = randn(red_shape, 17)
    got = T.reduce_fused("sum", ax, x, "sub", mean, outer="square")
    want = ((xn - np.expand_dims(mean.cpu().numpy().astype(np.float64), ax)) ** 2).sum(axis=ax)
    assert nerr(f64(got), want) < TOL_F32
    # y of x's shape (a dot product along the axis), and y over the axes from the folded one on (weights)
    y0 = randn(shape, 23)
    assert nerr(f64(T.reduce_fused("sum", ax, x, "mul", y0)), (xn * y0.cpu().numpy().astype(np.float64)).sum(axis=ax)) < TOL_F32
    w = randn(shape[ax:], 29)
    assert nerr(f64(T.reduce_fused("sum", ax, x, "mul", w, outer="relu")),
                np.maximum(xn * w.cpu().numpy().astype(np.float64), 0).sum(axis=ax)) < TOL_F32
    # operators without a compile-time instance go through the run-time form: unary (no operand at all), binary in each placement
    assert nerr(f64(T.reduce_fused("sum", ax, x, "tanh")), np.tanh(xn).sum(axis=ax)) < TOL_F32
    assert nerr(f64(T.reduce_fused("max", ax, x, "neg", outer="silu")), ((-xn) / (1 + np.exp(xn))).max(axis=ax)) < TOL_F32
    assert nerr(f64(T.reduce_fused("sum", ax, x, "max", y0)), np.maximum(xn, y0.cpu().numpy().astype(np.float64)).sum(axis=ax)) < TOL_F32
    pos = uniform(red_shape, 31, 0.5, 2.0)
    assert nerr(f64(T.reduce_fused("sum", ax, x, "div", pos)),
                (xn / np.expand_dims(pos.cpu().numpy().astype(np.float64), ax)).sum(axis=ax)) < TOL_F32
    assert nerr(f64(T.reduce_fused("min", ax, x, "min", w)), np.minimum(xn, w.cpu().numpy().astype(np.float64)).min(axis=ax)) < TOL_F32


def test_reduce_with_an_inlined_producer_bf16_and_arguments(T):
    from mimir_b200 import _lib as L
    x = randn((300, 2048), 3).to(torch.bfloat16)
    xn = x.float().cpu().numpy().astype(np.float64)
    got = T.reduce_fused("sum", 1, x, "square")
    assert got.dtype == torch.bfloat16 and nerr(f64(got.float()), (xn * xn).sum(axis=1)) < TOL_BF16
    # the same fold as the composition that writes the produced tensor
    two_pass = T.reduce("sum", 1, T.binary("mul", x.float(), x.float()))
    assert nerr(f64(got.float()), f64(two_pass)) < TOL_BF16
    # a binary producer needs its operand and a placement; a unary one takes none
    pre = L.Producer()
    pre.inner_op, pre.outer_op, pre.y_mode, pre.y = L.OP_SUB, L.OP_COPY, 3, None
    xf = x.float()
    out = torch.empty(300, device="cuda")
    import ctypes as C
    assert L.lib().mimk_reduce_fused(xf.data_ptr(), C.byref(pre), out.data_ptr(), L.F32, 300, 2048, 1, L.SUM, None) == 1  # MIMK_E_ARG
    pre.inner_op, pre.y_mode = 99, 3
    assert L.lib().mimk_reduce_fused(xf.data_ptr(), C.byref(pre), out.data_ptr(), L.F32, 300, 2048, 1, L.SUM, None) == 1


def test_scratch_using_calls_on_two_streams_do_not_share_a_buffer(T):
    """Split-axis folds keep partial results in a cached buffer; that buffer belongs to the stream of the call, so the same
    entry point may run on two streams at once."""
    x1, x2 = randn((4, 60000, 24), 71), randn((4, 60000, 24), 72)        # few columns, long axis: the plan splits the axis
    want1, want2 = T.reduce("sum", 1, x1).clone(), T.reduce("sum", 1, x2).clone()
    torch.cuda.synchronize()
    sa, sb = torch.cuda.Stream(), torch.cuda.Stream()
    outs = []
    for _ in range(20):
        with torch.cuda.stream(sa):
            a = T.reduce("sum", 1, x1)
        with torch.cuda.stream(sb):
            b = T.reduce("sum", 1, x2)
        outs.append((a, b))
    torch.cuda.synchronize()
    for a, b in outs:
        assert torch.equal(a, want1) and torch.equal(b, want2)


def test_elementwise_operators_with_a_unary_one_behind_them(T):
    """outer(inner(x, y)) in one pass: relu(x + bias), |x - y|, tanh(x * v) -- in every placement of the second operand."""
    x, y = randn((37, 300, 8), 51), randn((37, 300, 8), 52)
    xn, yn = x.cpu().numpy().astype(np.float64), y.cpu().numpy().astype(np.float64)
    assert nerr(f64(T.binary("sub", x, y, then="abs")), np.abs(xn - yn)) < TOL_F32
    v = randn((37, 8), 53)
    vn = v.cpu().numpy().astype(np.float64)
    assert nerr(f64(T.binary_ax("mul", 1, x, v, then="tanh")), np.tanh(xn * vn[:, None, :])) < TOL_F32
    assert nerr(f64(T.unary("square", x, then="neg")), -(xn * xn)) < TOL_F32
    # the rest of math.mim's unary operators, alone, behind a binary one, and inlined into a fold
    pos = np.abs(xn) + 0.5
    xp = T.unary("abs", x, then=None)
    xp = T.binary("add", xp, torch.full_like(xp, 0.5))
    for name, fn in (("sqrt", np.sqrt), ("rsqrt", lambda v: 1 / np.sqrt(v)), ("log", np.log), ("log2", np.log2)):
        assert nerr(f64(T.unary(name, xp)), fn(pos)) < TOL_F32
    assert nerr(f64(T.unary("exp2", x)), np.exp2(xn)) < TOL_F32
    assert nerr(f64(T.unary("sigmoid", x)), 1 / (1 + np.exp(-xn))) < TOL_F32
    assert nerr(f64(T.binary("mul", x, x, then="sqrt")), np.abs(xn)) < TOL_F32                       # sqrt(x * x)
    assert nerr(f64(T.reduce_fused("sum", 1, xp, "log")), np.log(pos).sum(axis=1)) < TOL_F32          # a sum of logarithms
    big, bias = randn((512, 4096), 54), randn((512,), 55)
    got = T.binary_ax("add", 1, big, bias, then="relu", out_dtype=torch.bfloat16)          # the 128-bit path, bf16 out
    want = np.maximum(big.cpu().numpy().astype(np.float64) + bias.cpu().numpy().astype(np.float64)[:, None], 0)
    assert got.dtype == torch.bfloat16 and nerr(f64(got.float()), want) < TOL_BF16
    # the same through a descriptor: FIRST(relu(a + b)) with b broadcast along the last axis, routed to the map kernel
    from mimir_b200 import _lib as L
    d = T.map_reduce_post((512, 4096), (512, 4096), L.f_composed(L.F_FIRST, L.OP_ADD, L.OP_RELU), 0.0, L.P_ID, T.id_map(2),
                          [T.id_map(2), T.proj_map(2, (0,))], [big, bias])
    assert nerr(f64(d), want) < TOL_F32
