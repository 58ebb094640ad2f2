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


def test_host_map_reduce_post_known_answers_and_routed_contraction():
    """The generic operation with host operands: the reference's integer known answers (bit exact) and a contraction
    large enough to be handed to the tensor-core kernel, both through mimk_host_map_reduce_post."""
    from mimir_b200 import _lib as L
    from mimir_b200 import host as H
    from mimir_b200 import tensor as T
    # lit/buffer/exec_map_reduce.mim:25-32 (row sums, out[2] = 42) and exec_epilogue.mim:27-38 (transposed read, bias, +1: 46)
    t = (torch.arange(12, dtype=torch.int32) + 1).reshape(3, 4)
    out = H.map_reduce_post((3,), (3, 4), L.F_ADD, 0, L.P_ID, T.proj_map(2, (0,)), [T.id_map(2)], [t])
    assert out.tolist() == [10, 26, 42]
    tt = t.t().contiguous()
    bias = torch.tensor([1, 2, 3], dtype=torch.int32)
    out = H.map_reduce_post((3,), (3, 4), L.F_ADD, 0, L.P_ADD_PLUS1, T.proj_map(2, (0,)), [T.proj_map(2, (1, 0))], [tt],
                            [T.id_map(1)], [bias])
    assert out.tolist() == [12, 29, 46]
    # a write map that covers every other cell leaves the rest of the caller's buffer alone
    buf = torch.full((8,), -7, dtype=torch.int32)
    H.map_reduce_post((8,), (4,), L.F_FIRST, 0, L.P_ID, [[2, 0]], [T.id_map(1)], [torch.arange(4, dtype=torch.int32)], out=buf)
    assert buf.tolist() == [0, -7, 1, -7, 2, -7, 3, -7]
    # f32 contraction given as a descriptor (routed to the contraction kernels), against the f64 truth
    g = torch.Generator().manual_seed(3)
    a, b = torch.randn(256, 192, generator=g), torch.randn(192, 320, generator=g)
    c = H.map_reduce_post((256, 320), (256, 320, 192), L.F_MULADD, 0.0, L.P_ID, T.proj_map(3, (0, 1)),
                          [T.proj_map(3, (0, 2)), T.proj_map(3, (2, 1))], [a, b])
    assert mo.normalised_error(c.numpy(), a.double().numpy() @ b.double().numpy()) <= 1e-5
