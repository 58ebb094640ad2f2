"""GPU parity: attention forward against the oracle's f64 routine (the reference driver's check)."""
import numpy as np
import pytest
import torch

import oracle as mo
from tests.util import TOL_BF16, TOL_F32, bits, f64, nerr, randn

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def T():
    from mimir_b200 import tensor
    return tensor


@pytest.mark.parametrize("bh,sq,sk,d", [(1, 4, 4, 8), (2, 64, 64, 8), (3, 33, 70, 40), (2, 128, 128, 64)])
@pytest.mark.parametrize("causal", [False, True])
def test_attention_f32(T, bh, sq, sk, d, causal):
    if causal and sq != sk:
        pytest.skip("the oracle's mask is defined for square scores")
    q, k, v = randn((bh, sq, d), 1), randn((bh, sk, d), 2), randn((bh, sk, d), 3)
    scale = 1.0 / d ** 0.5
    o, lse = T.attention(q, k, v, scale=scale, causal=causal, return_lse=True)
    if sq == sk:
        want = mo.attention(q.cpu().numpy(), k.cpu().numpy(), v.cpu().numpy(), scale=scale, causal=causal)
    else:
        s = np.einsum("hid,hjd->hij", f64(q), f64(k)) * scale
        p = np.exp(s - s.max(-1, keepdims=True))
        want = (p / p.sum(-1, keepdims=True)) @ f64(v)
    assert nerr(f64(o), want) <= TOL_F32
    s = np.einsum("hid,hjd->hij", f64(q), f64(k)) * scale
    if causal:
        s = np.where(np.tril(np.ones((sq, sk), bool)), s, -np.inf)
    want_lse = np.log(np.exp(s - s.max(-1, keepdims=True)).sum(-1)) + s.max(-1)
    assert np.abs(lse.cpu().numpy() - want_lse).max() < 1e-4


@pytest.mark.parametrize("bh,s,d", [(2, 128, 128), (2, 256, 128), (3, 384, 128), (1, 1024, 128), (2, 200, 128),
                                    (2, 512, 64), (3, 300, 64), (2, 1024, 64), (5, 129, 64), (9, 4096 + 64, 64)])
@pytest.mark.parametrize("causal", [True, False])
def test_attention_bf16(T, bh, s, d, causal):
    q, k, v = (randn((bh, s, d), 10 + i, 1.0, torch.bfloat16) for i in range(3))
    scale = 1.0 / d ** 0.5
    o = T.attention(q, k, v, scale=scale, causal=causal)
    T.device_status()
    want = mo.attention(bits(q), bits(k), bits(v), scale=scale, causal=causal, bf16=True)
    assert nerr(f64(o), want) <= TOL_BF16


def test_attention_config_c4_heads(T):
    # batch=4, heads=32, seqlen=4096, head_dim=128, causal: every head computed, three checked against the oracle
    q, k, v = (randn((4, 32, 4096, 128), 1240 + i, 1.0, torch.bfloat16) for i in range(3))
    scale = 1.0 / 128 ** 0.5
    o = T.attention(q, k, v, scale=scale, causal=True)
    T.device_status()
    heads = [0, 77, 127]
    qf, kf, vf = (t.reshape(128, 4096, 128) for t in (q, k, v))
    want = mo.attention(bits(qf[heads]), bits(kf[heads]), bits(vf[heads]), scale=scale, causal=True, bf16=True)
    assert nerr(f64(o.reshape(128, 4096, 128)[heads]), want) <= TOL_BF16
    # first query row attends to one key only: O[0] = V[0] exactly
    assert torch.equal(o[..., 0, :], v[..., 0, :])


def test_attention_bf16_rectangular_and_lse(T):
    # tensor-core kernel: more keys than queries (no mask), and the log-sum-exp output
    q = randn((2, 200, 128), 31, 1.0, torch.bfloat16)
    k = randn((2, 520, 128), 32, 1.0, torch.bfloat16)
    v = randn((2, 520, 128), 33, 1.0, torch.bfloat16)
    scale = 0.07
    o, lse = T.attention(q, k, v, scale=scale, causal=False, return_lse=True)
    T.device_status()
    s = np.einsum("hid,hjd->hij", f64(q), f64(k)) * scale
    p = np.exp(s - s.max(-1, keepdims=True))
    want = (p / p.sum(-1, keepdims=True)) @ f64(v)
    assert nerr(f64(o), want) <= TOL_BF16
    want_lse = np.log(p.sum(-1)) + s.max(-1)
    assert np.abs(lse.cpu().numpy() - want_lse).max() < 2e-3
    # causal, square, lse
    q2, k2, v2 = (randn((1, 384, 128), 40 + i, 1.0, torch.bfloat16) for i in range(3))
    o2, lse2 = T.attention(q2, k2, v2, scale=scale, causal=True, return_lse=True)
    s2 = np.einsum("hid,hjd->hij", f64(q2), f64(k2)) * scale
    s2 = np.where(np.tril(np.ones((384, 384), bool)), s2, -np.inf)
    want2 = np.log(np.exp(s2 - s2.max(-1, keepdims=True)).sum(-1)) + s2.max(-1)
    assert np.abs(lse2.cpu().numpy() - want2).max() < 2e-3


def test_attention_large_score_range(T):
    # scores spanning hundreds of log2 units exercise the lazy rescale of O (the running max jumps by far more than 2^8)
    g = torch.Generator().manual_seed(5)
    q = (torch.randn(1, 512, 128, generator=g) * 4).to(torch.bfloat16).cuda()
    k = (torch.randn(1, 512, 128, generator=g) * 4).to(torch.bfloat16).cuda()
    k[:, 300:, :] *= 3          # later keys score much higher: the maximum grows tile after tile
    v = torch.randn(1, 512, 128, generator=g).to(torch.bfloat16).cuda()
    for causal in (False, True):
        o = T.attention(q, k, v, scale=0.25, causal=causal)
        T.device_status()
        want = mo.attention(bits(q), bits(k), bits(v), scale=0.25, causal=causal, bf16=True)
        assert torch.isfinite(o.float()).all()
        assert nerr(f64(o), want) <= TOL_BF16


@pytest.mark.parametrize("d", [128, 64])
@pytest.mark.parametrize("s", [1, 2, 127, 129, 255, 257, 383])
@pytest.mark.parametrize("causal", [True, False])
def test_attention_bf16_ragged_lengths(T, s, causal, d):
    # query / key counts around the 128-row tile and 256-row pair boundaries: out-of-range rows are zero-filled by TMA
    # on the way in and never stored on the way out
    q, k, v = (randn((3, s, d), 50 + i + s, 1.0, torch.bfloat16) for i in range(3))
    guard = torch.full((3, s + 8, d), 7.0, dtype=torch.bfloat16, device="cuda")   # rows past s must stay untouched
    o = T.attention(q, k, v, scale=0.09, causal=causal)
    T.device_status()
    want = mo.attention(bits(q), bits(k), bits(v), scale=0.09, causal=causal, bf16=True)
    assert nerr(f64(o), want) <= TOL_BF16
    assert torch.equal(guard, torch.full_like(guard, 7.0))


def test_attention_no_keys(T):
    q = randn((2, 5, 16), 1)
    k = torch.empty((2, 0, 16), device="cuda")
    o, lse = T.attention(q, k, k.clone(), scale=1.0, return_lse=True)
    assert torch.equal(o, torch.zeros_like(o)) and torch.isinf(lse).all() and (lse < 0).all()


@pytest.mark.parametrize("bh,s,d,causal", [(3, 1024, 64, True), (2, 1024, 128, False), (20, 512, 64, True), (2, 640, 72, False),
                                                (1, 8320, 16, True)])   # the last: rows longer than the fused softmax takes
def test_attention_f32_at_scale_runs_the_composition(T, bh, s, d, causal):
    """f32 problems of 2^24 score-products or more run as S = Q K^T, softmax, O = P V on the contraction and row kernels
    (three-TF32 products, f32-grade): held to the f32 tolerance against the f64 truth on sampled heads."""
    q, k, v = (randn((bh, s, d), 70 + i, 1.0) for i in range(3))
    scale = 1.0 / d ** 0.5
    o = T.attention(q, k, v, scale=scale, causal=causal)
    T.device_status()
    heads = sorted({0, bh - 1, bh // 2})
    want = mo.attention(q.cpu().numpy(), k.cpu().numpy(), v.cpu().numpy(), scale=scale, causal=causal, heads=heads)
    assert nerr(f64(o[heads]), want) <= TOL_F32


@pytest.mark.parametrize("n", [4, 64])
def test_attn_aux_fixture(T, n):
    """lit/tensor/attn_aux.cpp:25-67 with attn_exec.mim:20-28 -- out = softmax_rows((x wq)(x wk)^T) (x wv), D = 8, no
    scale, no mask, inputs from the fixture's formulas; composed from the operators as the program composes it and through
    the fused entry point; the fixture's bound |ref - out| <= 1e-4 + 1e-4 |ref| against its double-precision loops."""
    D = 8
    i = np.arange(n * D)
    x = ((i % 13) / np.float32(13.0) - np.float32(0.4)).astype(np.float32).reshape(n, D)
    j = np.arange(D * D)
    wq = (((7 * j) % 11) / np.float32(11.0) - np.float32(0.5)).astype(np.float32).reshape(D, D)
    wk = (((5 * j) % 9) / np.float32(9.0) - np.float32(0.5)).astype(np.float32).reshape(D, D)
    wv = (((3 * j) % 7) / np.float32(7.0) - np.float32(0.5)).astype(np.float32).reshape(D, D)
    q64, k64, v64 = (x.astype(np.float64) @ w.astype(np.float64) for w in (wq, wk, wv))
    s = q64 @ k64.T
    p = np.exp(s - s.max(1, keepdims=True))
    ref = (p / p.sum(1, keepdims=True)) @ v64
    cx, cq, ck, cv = (torch.from_numpy(a).cuda() for a in (x, wq, wk, wv))
    q, k, v = T.product_2d(cx, cq), T.product_2d(cx, ck), T.product_2d(cx, cv)
    composed = T.product_2d(T.softmax(1, T.product_2d(q, T.transpose_2d(k))), v)
    fused = T.attention(q[None], k[None], v[None], scale=1.0, causal=False)[0]
    for out in (composed, fused):
        assert (np.abs(ref - f64(out)) <= 1e-4 + 1e-4 * np.abs(ref)).all()


@pytest.mark.parametrize("bh,s,d,causal", [(3, 1024, 96, True), (2, 512, 256, False), (5, 1024, 32, True), (2, 648, 40, False)])
def test_attention_bf16_other_head_dims_run_the_composition(T, bh, s, d, causal):
    """bf16 with a head_dim the fused kernels do not take: S = Q K^T (f32 scores), softmax to bf16 P, O = P V."""
    q, k, v = (randn((bh, s, d), 80 + i, 1.0, torch.bfloat16) for i in range(3))
    scale = 1.0 / d ** 0.5
    o = T.attention(q, k, v, scale=scale, causal=causal)
    T.device_status()
    heads = sorted({0, bh - 1})
    want = mo.attention(bits(q), bits(k), bits(v), scale=scale, causal=causal, bf16=True, heads=heads)
    assert nerr(f64(o[heads]), want) <= TOL_BF16
