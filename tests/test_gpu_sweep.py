"""Seeded sweeps over shapes that end inside tiles, switch kernels, or sit at alignment limits: every case goes through
the C ABI and is checked against the oracle's f64 truth on sampled rows / heads (normalised error, the tolerances of the
parity tests)."""
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


def _dims(rng, choices, n):
    return [int(rng.choice(choices)) for _ in range(n)]


M_CHOICES = [1, 7, 64, 127, 128, 129, 200, 256, 384, 511, 512, 640, 1000, 1536, 2048]
NK8 = [8, 16, 24, 64, 72, 120, 128, 136, 192, 256, 264, 320, 512, 520, 1024, 1288]


@pytest.mark.parametrize("seed", range(24))
def test_bf16_contractions(T, seed):
    rng = np.random.default_rng(1000 + seed)
    m = int(rng.choice(M_CHOICES))
    n, k = _dims(rng, NK8, 2)
    if seed % 6 == 0:                       # enough 256 x 256 tiles for the paired-SM kernel, ragged at both edges
        m, n = 2048 + 8 * int(rng.integers(0, 40)), 2560 + 8 * int(rng.integers(0, 40))
    nk = bool(rng.integers(0, 2))
    post = [None, "relu", "silu", "bias", "bias_relu", "add"][int(rng.integers(0, 6))]
    out_dtype = [torch.bfloat16, torch.float32][int(rng.integers(0, 2))]
    a = randn((m, k), seed, 0.5, torch.bfloat16)
    b = randn((n, k) if nk else (k, n), seed + 1, 0.5, torch.bfloat16)
    bv = b.t() if nk else b
    bias = randn((n,), seed + 2) if post in ("bias", "bias_relu") else None
    full = randn((m, n), seed + 3).to(out_dtype) if post == "add" else None
    c = T.product_2d(a, bv, post=post, bias=bias, full=full, out_dtype=out_dtype)
    T.device_status()
    rows = sorted(set(int(r) for r in rng.integers(0, m, 6)) | {0, m - 1})
    want = mo.gemm_truth(bits(a), bits(b), b_nk=nk, bf16=True, rows=rows)
    if bias is not None:
        want = want + f64(bias)[None]
    if full is not None:
        want = want + f64(full)[rows]
    if post in ("relu", "bias_relu"):
        want = np.maximum(want, 0)
    if post == "silu":
        want = want / (1 + np.exp(-want))
    tol = TOL_BF16 if out_dtype == torch.bfloat16 else 1e-4
    assert nerr(f64(c[rows]), want) <= tol, (m, n, k, nk, post, out_dtype)


@pytest.mark.parametrize("seed", range(12))
def test_f32_contractions(T, seed):
    rng = np.random.default_rng(2000 + seed)
    m, n, k = (int(rng.choice([1, 5, 33, 127, 128, 129, 256, 300, 512, 777, 1024])) for _ in range(3))
    if seed % 4 == 0:
        k = 4 * int(rng.integers(32, 300))  # the tensor-core route needs K % 4 == 0 and a large enough problem
        m, n = max(m, 256), max(n, 256)
    nk = bool(rng.integers(0, 2))
    a = randn((m, k), seed, 1.0)
    b = randn((n, k) if nk else (k, n), seed + 1, 1.0)
    c = T.product_2d(a, b.t() if nk else b)
    T.device_status()
    rows = sorted(set(int(r) for r in rng.integers(0, m, 6)) | {0, m - 1})
    want = mo.gemm_truth(a.cpu().numpy(), b.cpu().numpy(), b_nk=nk, rows=rows)
    assert nerr(f64(c[rows]), want) <= TOL_F32, (m, n, k, nk)


@pytest.mark.parametrize("seed", range(12))
def test_attention_shapes(T, seed):
    rng = np.random.default_rng(3000 + seed)
    bh = int(rng.choice([1, 3, 8, 17]))
    s = int(rng.choice([1, 64, 127, 128, 129, 255, 256, 300, 512, 1000, 1025]))
    causal = bool(rng.integers(0, 2))
    if seed % 3 == 0:
        dtype, d, tol = torch.float32, int(rng.choice([8, 32, 64, 80])), 1e-4
    else:
        dtype, d, tol = torch.bfloat16, int(rng.choice([64, 128])), TOL_BF16
    q, k, v = (randn((bh, s, d), seed * 3 + i, 1.0, dtype) for i in range(3))
    scale = float(d) ** -0.5
    o = T.attention(q, k, v, scale=scale, causal=causal)
    T.device_status()
    heads = sorted({0, bh - 1, int(rng.integers(0, bh))})
    if dtype == torch.bfloat16:
        want = mo.attention(bits(q), bits(k), bits(v), scale=scale, causal=causal, bf16=True, heads=heads)
    else:
        want = mo.attention(q.cpu().numpy(), k.cpu().numpy(), v.cpu().numpy(), scale=scale, causal=causal, heads=heads)
    assert nerr(f64(o[heads]), want) <= tol, (bh, s, d, causal, dtype)


@pytest.mark.parametrize("seed", range(12))
def test_row_operators(T, seed):
    rng = np.random.default_rng(4000 + seed)
    rows = int(rng.choice([1, 3, 64, 257, 1000]))
    cols = int(rng.choice([1, 4, 7, 100, 1024, 1027, 4096, 8192, 8200, 20000, 70001]))
    out_dtype = [torch.float32, torch.bfloat16][int(rng.integers(0, 2))]
    tol = TOL_F32 if out_dtype == torch.float32 else TOL_BF16
    x = randn((rows, cols), seed, 2.0)
    gamma = randn((cols,), seed + 1, 0.25) + 1.0
    sm = T.softmax(1, x, out_dtype=out_dtype)
    rn = T.rmsnorm(x, gamma, 1e-6, out_dtype=out_dtype)
    T.device_status()
    xs, gs = x.cpu().numpy(), gamma.cpu().numpy()
    assert nerr(f64(sm), mo.softmax_rows(xs, truth=True)) <= tol, (rows, cols)
    assert nerr(f64(rn), mo.rmsnorm_rows(xs, gs, 1e-6, truth=True)) <= tol, (rows, cols)
    for monoid in ("sum", "max"):
        for ax in (0, 1):
            got = T.reduce(monoid, ax, x)
            want = mo.reduce_axis(xs, ax, monoid, truth=True)
            if monoid == "max":
                assert np.array_equal(f64(got), want)
            else:
                assert np.max(np.abs(f64(got) - want)) <= 1e-5 * max(1.0, float(np.max(np.abs(xs)))) * np.sqrt(xs.shape[ax]), (rows, cols, ax)
