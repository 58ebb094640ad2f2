"""GPU parity of mimk_program_run: the reference's attention and softmax fixtures handed over as lists of map_reduce_post
descriptors (what a per-operation lowering emits), run fused, against the fixtures' own references and against the same list
run op by op."""
import numpy as np
import pytest
import torch

import oracle as mo
from tests.util import TOL_BF16, TOL_F32, bits, f64, nerr, randn

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def TL():
    from mimir_b200 import _lib, tensor
    return tensor, _lib


def new(shape, dtype=torch.float32):
    return torch.full(tuple(shape), float("nan"), dtype=dtype, device="cuda")


def softmax_ops(T, L, P, x, ax, fused=False):
    shape, r = list(x.shape), x.dim()
    red = shape[:ax] + shape[ax + 1:]
    fold_sr = red + [shape[ax]]
    fold_map = [j if j < ax else (r - 1 if j == ax else j - 1) for j in range(r)]
    drop = [i if i < ax else i + 1 for i in range(r - 1)]
    mx = P.op(new(red, x.dtype), fold_sr, L.F_MAX, float("-inf"), L.P_ID, T.proj_map(r, range(r - 1)), [T.proj_map(r, fold_map)], [x])
    if fused:
        sm = P.op(new(red, x.dtype), fold_sr, L.F_ADD_SUBEXP, 0.0, L.P_ID, T.proj_map(r, range(r - 1)),
                  [T.proj_map(r, fold_map), T.proj_map(r, range(r - 1))], [x, mx])
        return P.op(new(shape, x.dtype), shape, L.F_SUBEXP_DIV, 0.0, L.P_ID, T.id_map(r),
                    [T.id_map(r), T.proj_map(r, drop), T.proj_map(r, drop)], [x, mx, sm]), (mx, sm)
    e = P.op(new(shape, x.dtype), shape, L.F_SUBEXP, 0.0, L.P_ID, T.id_map(r), [T.id_map(r), T.proj_map(r, drop)], [x, mx])
    sm = P.op(new(red, x.dtype), fold_sr, L.F_ADD, 0.0, L.P_ID, T.proj_map(r, range(r - 1)), [T.proj_map(r, fold_map)], [e])
    return P.op(new(shape, x.dtype), shape, L.F_DIV, 0.0, L.P_ID, T.id_map(r), [T.id_map(r), T.proj_map(r, drop)], [e, sm]), (mx, e, sm)


def matmul(T, L, P, a, b, b_nk=False):
    m, k = a.shape
    n = b.shape[0] if b_nk else b.shape[1]
    return P.op(new((m, n), a.dtype), (m, n, k), L.F_MULADD, 0.0, L.P_ID, T.proj_map(3, (0, 1)),
                [T.proj_map(3, (0, 2)), T.proj_map(3, (1, 2) if b_nk else (2, 1))], [a, b])


@pytest.mark.parametrize("fused", [False, True])
def test_reduce_exec_softmax_as_a_program(TL, fused):
    """lit/tensor/reduce_exec.mim:19-43 -- x[a,b,c] = 12a + 4b + c, softmax along axis 1: rows sum to 1, peak
    1 / (1 + e^-4 + e^-8); and seeded shapes along every axis against the oracle's four-operation chain."""
    T, L = TL
    x = torch.arange(24, dtype=torch.float32).reshape(2, 3, 4).cuda()
    P = T.Program()
    y, temps = softmax_ops(T, L, P, x, 1, fused)
    assert P.classify()[0] == "softmax"
    P.run()
    T.device_status()
    assert np.abs(f64(y).sum(1) - 1).max() <= 1e-5
    assert abs(float(y[0, 2, 0]) - 1 / (1 + np.exp(-4) + np.exp(-8))) <= 1e-5
    assert all(torch.isnan(t).all() for t in temps)                # the chain's temporaries were never written
    for shape, ax in [((64, 1000), 1), ((7, 129, 5), 1), ((33, 17), 0), ((3, 4, 257), 2)]:
        x = randn(shape, 5 + ax)
        P = T.Program()
        y, _ = softmax_ops(T, L, P, x, ax, fused)
        P.run()
        T.device_status()
        assert nerr(f64(y), mo.softmax(x.cpu().numpy(), ax)) <= TOL_F32


@pytest.mark.parametrize("fused", [False, True])
@pytest.mark.parametrize("n", [4, 64])
def test_attn_aux_fixture_as_a_program(TL, n, fused):
    """lit/tensor/attn_aux.cpp:25-67 with attn_exec.mim:20-28 as the list of operations the program lowers to: three
    projections, S = q k^T through transpose_2d, the softmax operations, O = P v. The list runs as three contractions and
    ONE attention call; held to the fixture's bound against its double-precision loops, and compared with the same list
    run op by op."""
    T, L = TL
    D = 8
    i, j = np.arange(n * D), np.arange(D * D)
    x = ((i % 13) / np.float32(13.0) - np.float32(0.4)).astype(np.float32).reshape(n, D)
    wq = (((7 * j) % 11) / np.float32(11.0) - np.float32(0.5)).astype(np.float32).reshape(D, D)
    wk = (((5 * j) % 9) / np.float32(9.0) - np.float32(0.5)).astype(np.float32).reshape(D, D)
    wv = (((3 * j) % 7) / np.float32(7.0) - np.float32(0.5)).astype(np.float32).reshape(D, D)
    q64, k64, v64 = (x.astype(np.float64) @ w.astype(np.float64) for w in (wq, wk, wv))
    s64 = q64 @ k64.T
    p64 = np.exp(s64 - s64.max(1, keepdims=True))
    ref = (p64 / p64.sum(1, keepdims=True)) @ v64
    cx, cq, ck, cv = (torch.from_numpy(a).cuda() for a in (x, wq, wk, wv))

    def build():
        P = T.Program()
        q, k, v = matmul(T, L, P, cx, cq), matmul(T, L, P, cx, ck), matmul(T, L, P, cx, cv)
        s = matmul(T, L, P, q, k, b_nk=True)
        p, _ = softmax_ops(T, L, P, s, 1, fused)
        return P, matmul(T, L, P, p, v), s
    P, out, s = build()
    steps = P.classify()
    assert steps[:4] == ["op", "op", "op", "attention"] and set(steps[4:]) == {"absorbed"}
    P.run()
    T.device_status()
    assert (np.abs(ref - f64(out)) <= 1e-4 + 1e-4 * np.abs(ref)).all()
    assert torch.isnan(s).all()                                    # the score matrix was never materialised
    # the same operations one at a time through mimk_map_reduce_post
    P2, out2, s2 = build()
    for d in P2.descs:
        import ctypes as C
        L.check(L.lib().mimk_map_reduce_post(C.byref(d), None), "map_reduce_post")
    T.device_status()
    assert (np.abs(ref - f64(out2)) <= 1e-4 + 1e-4 * np.abs(ref)).all() and not torch.isnan(s2).any()
    assert nerr(f64(out), f64(out2)) <= TOL_F32


def test_attention_program_at_scale_runs_the_tensor_core_kernel(TL):
    """The same list at batch x heads = 8, 1024 x 1024 x 128 in bf16, with a leading batch loop on every operation: fused
    into one mimk_attn_fwd call (no score matrix), against the oracle on sampled heads."""
    T, L = TL
    BH, S, D = 8, 1024, 128
    q, k, v = (randn((BH, S, D), 90 + i, 0.3, torch.bfloat16) for i in range(3))
    P = T.Program()
    bmm = lambda a, b, n, kk, b_nk: P.op(new((BH, S, n), torch.bfloat16), (BH, S, n, kk), L.F_MULADD, 0.0, L.P_ID, T.proj_map(4, (0, 1, 2)),
                                         [T.proj_map(4, (0, 1, 3)), T.proj_map(4, (0, 2, 3) if b_nk else (0, 3, 2))], [a, b])
    s = bmm(q, k, S, D, True)
    p, _ = softmax_ops(T, L, P, s, 2, fused=False)
    o = bmm(p, v, D, S, False)
    assert P.classify()[0] == "attention"
    P.run()
    T.device_status()
    heads = [0, 5]
    want = mo.attention(bits(q), bits(k), bits(v), scale=1.0, causal=False, bf16=True, heads=heads)
    assert nerr(f64(o[heads]), want) <= TOL_BF16 and torch.isnan(s.float()).all()


def test_centred_sum_as_a_program_of_a_map_and_folds(TL):
    """A plain fold, then the map x + (-mean) (binary_ax) and the fold of its result: the map -> fold pair runs fused (the
    tensor x - mean is never written: it stays NaN) and gives what the op-by-op run and numpy give."""
    T, L = TL
    x = randn((96, 700, 12), 41)
    xn = x.cpu().numpy().astype(np.float64)
    shape, red = list(x.shape), [96, 12]

    def build(P, keep):
        s = P.op(new(red), red + [700], L.F_ADD, 0.0, L.P_ID, T.proj_map(3, (0, 1)), [T.proj_map(3, (0, 2, 1))], [x])
        d = P.op(new(shape), shape, L.F_ADD2, 0.0, L.P_ID, T.id_map(3), [T.id_map(3), T.proj_map(3, (0, 2))], [x, keep["neg_mean"]])
        keep["d"] = d
        a = P.op(new(red), red + [700], L.F_ADD, 0.0, L.P_ID, T.proj_map(3, (0, 1)), [T.proj_map(3, (0, 2, 1))], [d])
        return s, a

    neg_mean = torch.from_numpy((-xn.mean(axis=1)).astype(np.float32)).cuda()
    keep = {"neg_mean": neg_mean}
    P = T.Program()
    s, a = build(P, keep)
    assert P.classify() == ["op", "fold_of_map", "absorbed"]
    P.run()
    T.device_status()
    assert torch.isnan(keep["d"]).all()                       # the produced tensor was never written
    want = (xn - xn.mean(axis=1, keepdims=True)).sum(axis=1)
    assert np.abs(f64(a) - want).max() < 1e-3                  # sums of ~700 centred values: absolute tolerance
    assert nerr(f64(s), xn.sum(axis=1)) < TOL_F32
    # op by op gives the same numbers (other summation order inside the fold kernels: tolerance, not bits)
    keep2 = {"neg_mean": neg_mean}
    ops = T.Program()
    s2, a2 = build(ops, keep2)
    for dsc in ops.descs:
        L.check(L.lib().mimk_map_reduce_post(dsc, None), "op by op")
    torch.cuda.synchronize()
    assert not torch.isnan(keep2["d"]).any()
    assert np.abs(f64(a) - f64(a2)).max() < 1e-3
