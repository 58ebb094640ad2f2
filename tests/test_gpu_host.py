"""GPU parity of the host-buffer entry points (upload, run, download) -- the reference-facing call."""
import numpy as np
import pytest
import torch

import oracle as mo
from tests.util import TOL_BF16, TOL_F32, nerr

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def H():
    from mimir_b200 import host
    return host


def _randn(shape, seed, std=1.0):
    g = torch.Generator().manual_seed(seed)
    return torch.randn(shape, generator=g) * std


@pytest.mark.parametrize("rows,cols,pinned", [(10, 256, False), (5000, 8192, True), (4099, 1000, True)])
def test_host_rows(H, rows, cols, pinned):
    x = _randn((rows, cols), 1)
    gamma = torch.rand(cols, generator=torch.Generator().manual_seed(2)) + 0.5
    if pinned:
        x = x.pin_memory()
    y = H.softmax_rows(x, out_dtype=torch.bfloat16)
    sel = [0, rows // 2, rows - 1]
    assert nerr(y[sel].double().numpy(), mo.softmax_rows(x[sel].numpy(), truth=True)) < TOL_BF16
    assert (y.float().sum(1) - 1).abs().max() < 2e-2
    z = H.rmsnorm(x, gamma, 1e-6)
    assert nerr(z[sel].double().numpy(), mo.rmsnorm_rows(x[sel].numpy(), gamma.numpy(), 1e-6, truth=True)) < TOL_F32
    ys, yr = H.softmax_and_rmsnorm(x, gamma, 1e-6, out_dtype=torch.bfloat16)
    assert torch.equal(ys, y) and torch.equal(yr, H.rmsnorm(x, gamma, 1e-6, out_dtype=torch.bfloat16))
    # the device-resident path gives the same bits
    from mimir_b200 import tensor as T
    assert torch.equal(T.softmax(1, x.cuda(), out_dtype=torch.bfloat16).cpu(), y)


def test_host_gemm_and_attention(H):
    a, b = _randn((100, 64), 3), _randn((64, 72), 4)
    c = H.product_2d(a, b)
    assert nerr(c.double().numpy(), mo.gemm_truth(a.numpy(), b.numpy())) <= TOL_F32
    q, k, v = (_randn((2, 48, 16), 5 + i) for i in range(3))
    o = H.attention(q, k, v, scale=0.25, causal=True)
    assert nerr(o.double().numpy(), mo.attention(q.numpy(), k.numpy(), v.numpy(), scale=0.25, causal=True)) <= TOL_F32
