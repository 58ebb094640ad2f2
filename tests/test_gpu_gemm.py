"""GPU parity: the dot family (f32 CUDA-core path, bf16 tcgen05 path, epilogues, gated MLP) against the oracle."""
import numpy as np
import pytest
import torch

import oracle as mo
from tests.util import TOL_BF16, TOL_F32, bits, f64, nerr, randn, uniform

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def T():
    from mimir_b200 import tensor
    return tensor


def test_config_c1_f32_256(T):
    a, b = uniform((256, 256), 1234), uniform((256, 256), 1235)
    c = T.product_2d(a, b)
    an, bn = a.cpu().numpy(), b.cpu().numpy()
    assert nerr(f64(c), mo.gemm_truth(an, bn)) <= TOL_F32
    assert nerr(f64(c), mo.gemm(an, bn)) <= TOL_F32


@pytest.mark.parametrize("M,K,N", [(6, 40, 8), (5, 33, 7)])
def test_fc_exec_fixture(T, M, K, N):
    # lit/tensor/fc_aux.cpp:16-42 -- relu(x W^T + b), W stored [N,K], bias/relu fused into `post`
    x = ((torch.arange(M * K) % 13).float() / 13.0 - 0.4).reshape(M, K).cuda()
    w = (((7 * torch.arange(N * K)) % 11).float() / 11.0 - 0.5).reshape(N, K).cuda()
    bias = ((torch.arange(N) % 5).float() / 5.0 - 0.4).cuda()
    out = T.product_2d(x, T.transpose_2d(w), post="bias_relu", bias=bias)
    s = x.double().cpu().numpy() @ w.double().cpu().numpy().T
    ref = np.maximum((s + bias.cpu().numpy()).astype(np.float32), 0)
    assert (np.abs(ref - out.cpu().numpy()) <= 1e-4 + 1e-4 * np.abs(ref)).all()


def test_attn_exec_fixture_composed_on_device(T):
    # lit/tensor/attn_exec.mim:20-22 op by op: three product_2d, scores through transpose_2d, softmax, product_2d
    for N in (4, 64):
        D = 8
        x = ((torch.arange(N * D) % 13).float() / 13.0 - 0.4).reshape(N, D).cuda()
        j = torch.arange(D * D)
        wq = (((7 * j) % 11).float() / 11.0 - 0.5).reshape(D, D).cuda()
        wk = (((5 * j) % 9).float() / 9.0 - 0.5).reshape(D, D).cuda()
        wv = (((3 * j) % 7).float() / 7.0 - 0.5).reshape(D, D).cuda()
        q, k, v = T.product_2d(x, wq), T.product_2d(x, wk), T.product_2d(x, wv)
        out = T.product_2d(T.softmax(1, T.product_2d(q, T.transpose_2d(k))), v)
        xd = x.double().cpu().numpy()
        qd, kd, vd = (xd @ w.double().cpu().numpy() for w in (wq, wk, wv))
        s = qd @ kd.T
        p = np.exp(s - s.max(1, keepdims=True))
        ref = (p / p.sum(1, keepdims=True)) @ vd
        assert (np.abs(ref - out.cpu().numpy()) <= 1e-4 + 1e-4 * np.abs(ref)).all()
        fused = T.attention(q, k, v)
        assert (np.abs(ref - fused.cpu().numpy()) <= 1e-4 + 1e-4 * np.abs(ref)).all()


def test_hlo_mlp_fixture(T):
    # lit/tensor/hlo_aux.cpp:41-84 -- tanh MLP 128/784/1024/10 with bias+tanh epilogues, rel <= 1e-3
    B, IN, H, OUT = 128, 784, 1024, 10

    def init(n):
        return ((torch.arange(n) % 100).float() / 100.0).cuda()

    w0, b0, w1, b1 = init(IN * H).reshape(IN, H), init(H), init(H * H).reshape(H, H), init(H)
    w2, b2, x = init(H * OUT).reshape(H, OUT), init(OUT), init(B * IN).reshape(B, IN)
    h0 = T.product_2d(x, w0, post="bias_tanh", bias=b0)
    h1 = T.product_2d(h0, w1, post="bias_tanh", bias=b1)
    out = T.reduce("max", 1, T.product_2d(h1, w2, post="bias", bias=b2))
    d0 = np.tanh(x.double().cpu().numpy() @ w0.double().cpu().numpy() + b0.cpu().numpy())
    d1 = np.tanh(d0 @ w1.double().cpu().numpy() + b1.cpu().numpy())
    ref = (d1 @ w2.double().cpu().numpy() + b2.cpu().numpy()).max(axis=1)
    rel = np.abs(ref - out.cpu().numpy()) / (np.abs(ref) + 1e-6)
    assert rel.max() <= 1e-3


@pytest.mark.parametrize("M,N,K", [(1, 1, 1), (17, 19, 23), (64, 64, 64), (130, 70, 257), (256, 512, 100)])
@pytest.mark.parametrize("nk", [False, True])
def test_f32_shapes(T, M, N, K, nk):
    a = uniform((M, K), M * 7 + K)
    b = uniform((N, K) if nk else (K, N), N * 3 + K)
    c = T.product_2d(a, T.transpose_2d(b) if nk else b)
    want = mo.gemm_truth(a.cpu().numpy(), b.cpu().numpy(), b_nk=nk)
    assert nerr(f64(c), want) <= TOL_F32


def test_bmm_f32(T):
    a, b = uniform((5, 33, 20), 1), uniform((5, 20, 17), 2)
    c = T.bmm(a, b)
    for i in range(5):
        assert nerr(f64(c[i]), mo.gemm_truth(a[i].cpu().numpy(), b[i].cpu().numpy())) <= TOL_F32


# ------------------------------------------------------------------ tensor-core path
@pytest.mark.parametrize("M,N,K", [(128, 256, 64), (128, 256, 256), (256, 512, 512), (384, 264, 200), (100, 72, 136),
                                   (1000, 1000, 1000), (2048, 2048, 2048)])
@pytest.mark.parametrize("nk", [True, False])
@pytest.mark.parametrize("out_dtype", [torch.bfloat16, torch.float32])
def test_bf16_tensor_core(T, M, N, K, nk, out_dtype):
    a = randn((M, K), 100 + M, 0.5, torch.bfloat16)
    b = randn((N, K) if nk else (K, N), 200 + N, 0.5, torch.bfloat16)
    c = T.product_2d(a, T.transpose_2d(b) if nk else b, out_dtype=out_dtype)
    T.device_status()
    rows = None if M * N * K <= 300 * 300 * 300 else sorted(set(np.random.default_rng(M).integers(0, M, 48).tolist() + [0, M - 1]))
    want = mo.gemm_truth(bits(a), bits(b), b_nk=nk, bf16=True, rows=rows)
    got = f64(c) if rows is None else f64(c[rows])
    tol = TOL_BF16 if out_dtype == torch.bfloat16 else 1e-4   # f32 store: only the accumulation order differs
    assert nerr(got, want) <= tol


def test_bf16_structured_identity(T):
    # B = identity picks columns of A exactly: any layout/descriptor mistake shows up as a permutation
    M, K = 256, 256
    a = randn((M, K), 3, 1.0, torch.bfloat16)
    eye = torch.eye(K, dtype=torch.bfloat16, device="cuda")
    for b in (eye, T.transpose_2d(eye.clone())):
        c = T.product_2d(a, b)
        T.device_status()
        assert torch.equal(c, a)
    # a single one in B at (k0, n0) moves column k0 of A to column n0 of C
    for nk in (False, True):
        b = torch.zeros((K, K), dtype=torch.bfloat16, device="cuda")
        b[37, 201] = 1
        bb = T.transpose_2d(b.t().contiguous()) if nk else b
        c = T.product_2d(a, bb)
        want = torch.zeros_like(a)
        want[:, 201] = a[:, 37]
        assert torch.equal(c, want)


def test_bf16_epilogues(T):
    M, N, K = 256, 320, 192
    a = randn((M, K), 1, 0.3, torch.bfloat16)
    w = randn((N, K), 2, 0.3, torch.bfloat16)
    bias = uniform((N,), 3)
    res = randn((M, N), 4, 1.0, torch.bfloat16)
    acc = mo.gemm_truth(bits(a), bits(w), b_nk=True, bf16=True)
    bn = bias.cpu().numpy().astype(np.float64)
    cases = {
        "bias": acc + bn, "bias_relu": np.maximum(acc + bn, 0), "bias_tanh": np.tanh(acc + bn),
        "relu": np.maximum(acc, 0), "silu": acc / (1 + np.exp(-acc)),
    }
    for post, want in cases.items():
        c = T.product_2d(a, T.transpose_2d(w), post=post, bias=bias if "bias" in post else None, out_dtype=torch.float32)
        assert nerr(f64(c), want) <= 1e-4, post
    c = T.product_2d(a, T.transpose_2d(w), post="add", full=res)
    assert nerr(f64(c), acc + f64(res)) <= TOL_BF16


def test_bf16_linearity_and_checksum_full_size(T):
    # config C3's shape: C.1 = A.(B.1) and row samples against the oracle
    n = 8192
    a = randn((n, n), 1236, 0.02, torch.bfloat16)
    b = randn((n, n), 1237, 0.02, torch.bfloat16)   # stored [N,K]
    c = T.product_2d(a, T.transpose_2d(b), out_dtype=torch.float32)
    T.device_status()
    ones = torch.ones(n, dtype=torch.float64, device="cuda")
    lhs = c.double() @ ones
    rhs = a.double() @ (b.double() @ ones)          # B^T 1 for B stored [N,K] is the row sums of... (b^T)1 = b.sum(0)
    rhs = a.double() @ b.double().sum(dim=0)
    assert (lhs - rhs).abs().max() / rhs.abs().max() < 1e-3
    rows = [0, 127, 128, 4095, 8191]
    want = mo.gemm_truth(bits(a), bits(b), b_nk=True, bf16=True, rows=rows)
    assert nerr(f64(c[rows]), want) <= 1e-4
    cb = T.product_2d(a, T.transpose_2d(b))
    assert nerr(f64(cb[rows]), want) <= TOL_BF16


def test_bmm_bf16(T):
    a = randn((3, 128, 64), 5, 0.5, torch.bfloat16)
    b = randn((3, 64, 256), 6, 0.5, torch.bfloat16)
    c = T.bmm(a, b, out_dtype=torch.float32)
    T.device_status()
    for i in range(3):
        assert nerr(f64(c[i]), mo.gemm_truth(bits(a[i]), bits(b[i]), bf16=True)) <= 1e-4


@pytest.mark.parametrize("nk", [False, True])
def test_mlp_gated(T, nk):
    M, K, F, N = 256, 192, 384, 128
    x = randn((M, K), 1, 1.0, torch.bfloat16)
    w1 = randn((K, F), 2, 0.05, torch.bfloat16)
    w3 = randn((K, F), 3, 0.05, torch.bfloat16)
    w2 = randn((F, N), 4, 0.05, torch.bfloat16)
    if nk:
        y = T.mlp_gated(x, T.transpose_2d(w1.t().contiguous()), T.transpose_2d(w3.t().contiguous()),
                        T.transpose_2d(w2.t().contiguous()))
    else:
        y = T.mlp_gated(x, w1, w3, w2)
    T.device_status()
    want = mo.mlp_gated_truth(bits(x), bits(w1), bits(w3), bits(w2))
    assert nerr(f64(y), want) <= TOL_BF16


def test_zero_extents(T):
    a = torch.empty((0, 8), device="cuda")
    b = torch.empty((8, 4), device="cuda")
    assert T.product_2d(a, b).shape == (0, 4)
    # K = 0: the fold never runs, every cell is the ring's zero (tensor.mim:1332 with init = R#_0)
    c = T.product_2d(torch.empty((3, 0), device="cuda"), torch.empty((0, 5), device="cuda"))
    assert torch.equal(c, torch.zeros(3, 5, device="cuda"))
    cb = T.product_2d(torch.empty((8, 0), device="cuda", dtype=torch.bfloat16),
                      torch.empty((0, 8), device="cuda", dtype=torch.bfloat16))
    assert torch.equal(cb, torch.zeros(8, 8, device="cuda", dtype=torch.bfloat16))


def test_mlp_config_c5_full_size_rows(T):
    # X[8192,4096], W1/W3[4096,14336], W2[14336,4096]: the whole block on the device, two rows against the oracle,
    # plus linearity in X (the block is positively homogeneous of degree 1 only through the gate, so use additivity
    # of the second contraction instead: Y is linear in W2)
    M, K, F, N = 8192, 4096, 14336, 4096
    x = randn((M, K), 1238, 1.0, torch.bfloat16)
    w1 = randn((K, F), 1239, 0.02, torch.bfloat16)
    w3 = randn((K, F), 1240, 0.02, torch.bfloat16)
    w2 = randn((F, N), 1241, 0.02, torch.bfloat16)
    y = T.mlp_gated(x, w1, w3, w2)
    T.device_status()
    rows = [0, 8191]
    want = mo.mlp_gated_truth(bits(x[rows]), bits(w1), bits(w3), bits(w2))
    assert nerr(f64(y[rows]), want) <= TOL_BF16
    y2 = T.mlp_gated(x, w1, w3, (w2.float() * 2).to(torch.bfloat16))      # doubling W2 is exact in bf16
    assert torch.equal(y2[rows].float(), (y[rows].float() * 2).to(torch.bfloat16).float())


def test_gemm_flat_entry_point(T):
    # the scalar-argument form emitted code would call: same result as the descriptor form
    from mimir_b200 import _lib
    a, b = uniform((40, 24), 1), uniform((24, 56), 2)
    c = torch.empty((40, 56), device="cuda")
    st = _lib.lib().mimk_gemm_flat(40, 56, 24, a.data_ptr(), b.data_ptr(), c.data_ptr(), _lib.F32, _lib.F32, _lib.B_KN,
                                   _lib.POST_ID, None, torch.cuda.current_stream().cuda_stream)
    assert st == 0
    assert torch.equal(c, T.product_2d(a, b))


@pytest.mark.parametrize("nk", [True, False])
def test_paired_sm_kernel_shapes(T, nk):
    # enough 256-row tiles (>= 74) for the cta_group::2 kernel: ragged M / N / K, both B layouts, f32 store, epilogue
    M, N, K = 4000, 4104, 520
    a = randn((M, K), 7, 0.5, torch.bfloat16)
    b = randn((N, K) if nk else (K, N), 8, 0.5, torch.bfloat16)
    bias = uniform((N,), 9)
    c = T.product_2d(a, T.transpose_2d(b) if nk else b, post="bias_relu", bias=bias, out_dtype=torch.float32)
    T.device_status()
    rows = [0, 127, 128, 255, 256, 2049, 3999]
    acc = mo.gemm_truth(bits(a), bits(b), b_nk=nk, bf16=True, rows=rows)
    want = np.maximum(acc + bias.cpu().numpy().astype(np.float64), 0)
    assert nerr(f64(c[rows]), want) <= 1e-4
    # column sums of the un-fused product agree with a . (B 1) -- every tile contributes
    c0 = T.product_2d(a, T.transpose_2d(b) if nk else b, out_dtype=torch.float32)
    ones = torch.ones(N, dtype=torch.float64, device="cuda")
    bsum = (b.double().sum(dim=0) if nk else b.double().sum(dim=1))
    lhs, rhs = c0.double() @ ones, a.double() @ bsum
    assert (lhs - rhs).abs().max() / rhs.abs().max() < 1e-3


def test_paired_sm_gated_mlp(T):
    M, K, F, N = 2048, 256, 4096, 512
    x = randn((M, K), 1, 1.0, torch.bfloat16)
    w1, w3 = randn((K, F), 2, 0.05, torch.bfloat16), randn((K, F), 3, 0.05, torch.bfloat16)
    w2 = randn((F, N), 4, 0.05, torch.bfloat16)
    y = T.mlp_gated(x, w1, w3, w2)
    T.device_status()
    rows = [0, 129, 2047]
    want = mo.mlp_gated_truth(bits(x[rows]), bits(w1), bits(w3), bits(w2))
    assert nerr(f64(y[rows]), want) <= TOL_BF16


@pytest.mark.parametrize("nk", [False, True])
@pytest.mark.parametrize("m,n,K", [(96, 80, 520), (32, 32, 4), (33, 100, 128), (256, 256, 256), (7, 260, 1028)])
def test_small_f32_products_same_bits_on_either_cuda_core_kernel(T, m, n, K, nk):
    # a small product runs on 32 x 32 tiles with K staged in chunks; a product with several hundred 64 x 64 tiles (and an
    # N the tensor-core path does not take) runs on the 64 x 64 kernel. Both fold every cell in ascending k with one fma
    # per step, so a corner of the large product equals the small product of the same rows and columns bit for bit.
    M, N = 1280, 961
    a = uniform((M, K), 500 + K)
    b = uniform((N, K) if nk else (K, N), 501 + K)
    big = T.product_2d(a, T.transpose_2d(b) if nk else b)
    bs = b[:n].contiguous() if nk else b[:, :n].contiguous()
    small = T.product_2d(a[:m].contiguous(), T.transpose_2d(bs) if nk else bs)
    T.device_status()
    assert torch.equal(small, big[:m, :n])
    want = mo.gemm_truth(a[:m].cpu().numpy(), bs.cpu().numpy(), b_nk=nk)
    assert nerr(f64(small), want) <= TOL_F32


@pytest.mark.parametrize("M,N,K,nk", [(512, 512, 8192, True), (384, 640, 4100, False), (1024, 1024, 1024, False)])
def test_f32_on_tensor_cores_keeps_f32_accuracy(T, M, N, K, nk):
    # large f32 contractions run as three TF32 products per term with K cut into chunks summed in f32: the error must
    # stay at the f32 path's tolerance for any K (an unchunked accumulation drifts past 1e-5 around K = 1024)
    a = uniform((M, K), 70 + K)
    b = uniform((N, K) if nk else (K, N), 71 + K)
    c = T.product_2d(a, T.transpose_2d(b) if nk else b, post="bias", bias=uniform((N,), 3))
    T.device_status()
    rows = [0, 127, 128, M - 1]
    want = mo.gemm_truth(a.cpu().numpy(), b.cpu().numpy(), b_nk=nk, rows=rows) + uniform((N,), 3).cpu().numpy().astype(np.float64)
    assert nerr(f64(c[rows]), want) <= TOL_F32


@pytest.mark.parametrize("nk", [False, True])
def test_f32_on_tensor_cores_non_finite_operands(T, nk):
    # inf / NaN operands (and a finite value whose TF32 head rounds up to inf) must give what the scalar ascending fold
    # gives -- +-inf where every product has one sign, NaN where inf meets 0 or -inf -- not the NaN a head/tail split of
    # inf would spread over the row
    M, N, K = 512, 512, 640                                 # 2^27 products and more go to the tensor cores
    a, b = uniform((M, K), 90), uniform((N, K) if nk else (K, N), 91)
    a[3, 5], a[10, 0], a[200, 17] = float("inf"), float("nan"), 3.4028e38
    a[77, 8] = float("-inf")
    if nk:
        b[9, 7], b[300, 8] = float("-inf"), 0.0
    else:
        b[7, 9], b[8, 300] = float("-inf"), 0.0
    c = T.product_2d(a, T.transpose_2d(b) if nk else b).cpu().numpy()
    T.device_status()
    want = mo.gemm(a.cpu().numpy(), b.cpu().numpy(), b_nk=nk)
    assert (np.isnan(c) == np.isnan(want)).all()
    inf = np.isinf(want)
    assert (np.isinf(c) == inf).all() and (c[inf] == want[inf]).all()
    assert np.isnan(want[77, 300]) and np.isinf(want[3, 0]) and np.isnan(want[10]).all()   # the case is what it claims
    fin = np.isfinite(want)
    truth = mo.gemm_truth(np.where(np.isfinite(a.cpu().numpy()), a.cpu().numpy(), 0), np.where(np.isfinite(b.cpu().numpy()), b.cpu().numpy(), 0), b_nk=nk)
    rows = [r for r in range(M) if r not in (3, 10, 77, 200)]
    cols = [j for j in range(N) if j != 9]
    sub = np.ix_(rows, cols)
    assert fin[sub].all() and nerr(c[sub].astype(np.float64), truth[sub]) <= TOL_F32


@pytest.mark.parametrize("nk", [False, True])
def test_reduce_scatter_epilogue_on_one_gpu(T, nk):
    """The contraction whose epilogue ADDS its f32 tiles into the owners' row blocks (bulk reductions), with every
    "owner" a buffer of this GPU: four row blocks, two calls into accumulators that start from a known value."""
    from mimir_b200 import shard

    class Blocks:                       # the parts of a GatheredMatrix the call looks at, all on this GPU
        def __init__(self, world, rows, cols):
            self.all = [torch.full((rows, cols), 0.5, dtype=torch.float32, device="cuda") for _ in range(world)]
            self.world, self.rank, self.rows, self.cols = world, 1, rows, cols
            self.local, self.ptrs = self.all[1], [t.data_ptr() for t in self.all]

    M, N, K, W = 1280, 520, 384, 4
    a = randn((M, K), 410, dtype=torch.bfloat16)
    b = randn((N, K) if nk else (K, N), 411, 0.05, dtype=torch.bfloat16)
    bv = T.transpose_2d(b) if nk else b
    acc = Blocks(W, M // W, N)
    shard.gemm_reduce_scatter(a, bv, acc)
    shard.gemm_reduce_scatter(a, bv, acc)
    T.device_status()
    got = torch.cat(acc.all)
    whole = T.product_2d(a, bv, out_dtype=torch.float32)
    # one contribution per call and cell, so the order of the additions is fixed here: (0.5 + c) + c up to the last bit of
    # the product itself (the reference product may come from the one-CTA kernel)
    assert float((got - ((whole + 0.5) + whole)).abs().max()) <= 1e-5
    want = mo.gemm_truth(bits(a), bits(b), b_nk=nk, bf16=True, rows=[0, M - 1])
    assert nerr(f64(got[[0, M - 1]] - 0.5) / 2, want) <= TOL_BF16
    # malformed requests are refused before anything is launched
    with pytest.raises(ValueError):
        shard.gemm_reduce_scatter(a[:100], bv, acc)


@pytest.mark.parametrize("M,G,kp,N", [(300, 4, 128, 264), (2560, 8, 256, 2048), (512, 2, 64, 8)])
@pytest.mark.parametrize("nk", [False, True])
def test_left_operand_as_k_panels(T, M, G, kp, N, nk):
    """A handed over as G column panels [G, M, kp] (an all-gather's receive buffer) gives the bits of the product with
    the panels laid side by side, on the one-CTA and on the paired-SM kernel."""
    a = randn((M, G * kp), 300 + M, dtype=torch.bfloat16)
    b = randn((N, G * kp) if nk else (G * kp, N), 301 + M, 0.05, dtype=torch.bfloat16)
    bv = T.transpose_2d(b) if nk else b
    panels = a.reshape(M, G, kp).permute(1, 0, 2).contiguous()
    got = T.product_2d_panels(panels, bv)
    T.device_status()
    assert torch.equal(got, T.product_2d(a, bv))
    rows = [0, M - 1]
    want = mo.gemm_truth(bits(a), bits(b), b_nk=nk, bf16=True, rows=rows)
    assert nerr(f64(got[rows]), want) <= TOL_BF16


def test_chain_product_matches_the_chain_as_written():
    """Whatever association the price list picks (lit/tensor/reassoc.mim's chains, scaled up), the product is the one
    the chain as written gives, within the float tolerance of the f64 truth."""
    from mimir_b200 import reassoc as R
    from mimir_b200 import tensor as T
    g = torch.Generator().manual_seed(21)

    def rnd(r, c, scale=1.0):
        return (torch.randn(r, c, generator=g) * scale).cuda()
    # attention scores (x wq) (x wk)^T as the chain x . wq . wk^T . x^T (reassoc.mim:113-124)
    x, wq, wk = rnd(640, 96), rnd(96, 96, 0.1), rnd(96, 96, 0.1)
    mats = [x, wq, T.transpose_2d(wk), T.transpose_2d(x)]
    truth = (x.double() @ wq.double() @ wk.double().t() @ x.double().t()).cpu().numpy()
    for model in ("lanes", "b200"):
        got = R.chain_product(mats, model=model)
        assert got.shape == (640, 640) and got.is_contiguous()
        assert mo.normalised_error(got.cpu().numpy(), truth) <= 1e-5
    written = [(0, 0, 1, False), (2, 2, 3, True), (0, 1, 3, False)]      # the right factor built as x . wk, read transposed
    got = R.chain_product(mats, written=written, model="lanes")
    assert mo.normalised_error(got.cpu().numpy(), truth) <= 1e-5
    # low-rank bottleneck x (U V), bf16: re-associated to (x U) V
    xb, u, v = rnd(65536, 768).bfloat16(), rnd(768, 8, 0.05).bfloat16(), rnd(8, 768, 0.05).bfloat16()
    splits, _, moved = R.choose((65536, 768, 8, 768), None, R.right_deep(3), model="b200")
    assert moved and [s[:3] for s in splits] == [(0, 0, 1), (0, 1, 2)]
    got = R.chain_product([xb, u, v], written=R.right_deep(3))
    truth = (xb[:4096].double() @ u.double() @ v.double()).cpu().numpy()
    assert mo.normalised_error(got[:4096].float().cpu().numpy(), truth) <= 2e-2
    # a node built transposed: X . (A^T . B^T)
    X, A, B = rnd(512, 384, 0.1), rnd(256, 384, 0.1), rnd(128, 256, 0.1)
    got = R.chain_product([X, T.transpose_2d(A), T.transpose_2d(B)])
    truth = (X.double() @ A.double().t() @ B.double().t()).cpu().numpy()
    assert mo.normalised_error(got.cpu().numpy(), truth) <= 1e-5


@pytest.mark.parametrize("nk", [False, True])
def test_long_batches_run_as_one_launch(T, nk):
    """96 batch entries with ragged extents (rows and columns that end inside a tile): the batched kernel walks
    (batch, tile) pairs; every entry must equal the unbatched product of its operands, bit for bit."""
    B, M, N, K = 96, 200, 264, 72
    a = randn((B, M, K), 31, 0.5, torch.bfloat16)
    b = randn((B, N, K) if nk else (B, K, N), 32, 0.5, torch.bfloat16)
    bv = b.transpose(1, 2) if nk else b
    c = T.bmm(a, bv)
    T.device_status()
    for i in (0, 1, 47, 95):
        assert torch.equal(c[i], T.product_2d(a[i], bv[i]))
    want = mo.gemm_truth(bits(a[95]), bits(bv[95].contiguous()), bf16=True)
    assert nerr(f64(c[95]), want) <= TOL_BF16
    # one right operand for every entry (batch stride 0), a full-shape addend per entry in the epilogue
    full = randn((B, M, N), 33, 1.0, torch.bfloat16)
    out = torch.empty((B, M, N), dtype=torch.bfloat16, device="cuda")
    b0 = b[0].contiguous()
    T._gemm(a, b0, 1 if nk else 0, B, M, N, K, M * K, 0, out, "add", None, full)
    T.device_status()
    for i in (0, 50, 95):
        assert torch.equal(out[i], T.product_2d(a[i], bv[0], post="add", full=full[i]))


def test_hlo_train_step_fixture(T):
    """lit/tensor/hlo_train_aux.cpp:24-76 -- one training step of a one-layer tanh MLP (N=4, I=8, O=3): forward, the
    backward products through transposed reads, the bias gradient as an axis fold, for the fixture's three input
    patterns. The returned scalar is rebuilt from this library's operators and held to the fixture's 1e-4."""
    N, I, O, lr, c = 4, 8, 3, 0.001, 0.5

    def make(n, mode):
        i = np.arange(n)
        v = (i % 100) / np.float32(100.0) if mode == 0 else (np.full(n, 0.5) if mode == 1 else 0.01 * ((i % 7) + 1))
        return v.astype(np.float32)
    for mode in range(3):
        w, b, x, t = make(I * O, mode).reshape(I, O), make(O, mode), make(N * I, mode).reshape(N, I), make(N * O, mode).reshape(N, O)
        # the fixture's scalar reference
        z = x @ w
        a = np.tanh(z + b)
        d = np.float32(c) * (a - t)
        dW, db, dx = x.T @ d, d.sum(0), d @ w.T
        ref = (w[0, 0] - lr * dW[0, 0]) + (b[0] - lr * db[0]) + dx[0, 0] + z[0].max()
        # the same step from the operators
        cw, cb, cx, ct = (torch.from_numpy(v).cuda() for v in (w, b, x, t))
        gz = T.product_2d(cx, cw)
        ga = T.product_2d(cx, cw, post="bias_tanh", bias=cb)
        half = torch.full_like(ga, c)
        gd = T.binary("mul", half, T.binary("sub", ga, ct))
        gdW = T.transpose(T.product_2d(T.transpose_2d(gd).contiguous(), cx), (1, 0))      # dW = (d^T x)^T
        gdx = T.product_2d(gd, T.transpose_2d(cw))                                       # dx = d w^T
        gdb = T.reduce("sum", 0, gd)
        rmax = T.reduce("max", 1, gz)
        got = (w[0, 0] - lr * gdW[0, 0].item()) + (b[0] - lr * gdb[0].item()) + gdx[0, 0].item() + rmax[0].item()
        assert abs(got - ref) <= 1e-4, (mode, got, ref)


def test_hlo_training_step_fixture(T):
    """lit/tensor/hlo_step_aux.cpp:33-158 -- one SGD step of the tanh MLP 128/784/1024/10: forward, the softmax-loss
    gradient, the backward contractions over transposed reads, column sums, and the digest of six update deltas, held to
    the fixture's bound (1e-2 of the digest's scale + 1e-6)."""
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

    def digest(mm, tanh, colsum, rowmax, rowsum, exp_shift, mul, add, scal, div):
        """The fixture's computation over abstract operators, so that numpy (f64) and the library run the same program."""
        h1 = tanh(mm(X_, W1_), b1_)
        h2 = tanh(mm(h1, W2_), b2_)
        logits = add(mm(h2, W3_), b3_, row=True)
        e = exp_shift(logits, rowmax(logits))
        ssum = rowsum(e)
        gs = rowsum(scal(Y_, -c))
        q = div(gs, ssum)                                         # the row sums are positive: the fixture's selects pick gs / |ssum|
        dlog = add(scal(Y_, c), mul(e, q, col=True))
        d2 = mm(dlog, W3_, bt=True)                              # dlog . W3^T
        v59 = d2                                                  # s (1 - h2) + s h2 = s
        s1 = mm(v59, W2_, bt=True)
        v66 = mul(s1, add(scal(h1, -1.0), 1.0))
        v68 = add(v66, mul(v66, h1))
        dW1 = mm(X_, v68, at=True)
        dW2 = mm(h1, v59, at=True)
        dW3 = mm(h2, dlog, at=True)
        return [dW1[3, 5], colsum(v68)[7], dW2[11, 13], colsum(v59)[17], dW3[19, 2], colsum(dlog)[3]]

    # f64 reference
    X_, Y_, W1_, W2_, W3_, b1_, b2_, b3_ = (a.astype(np.float64) for a in (X, Y, W1, W2, W3, b1, b2, b3))
    ref = digest(lambda a, b, at=False, bt=False: (a.T if at else a) @ (b.T if bt else b), lambda z, b: np.tanh(z + b),
                 lambda m: m.sum(0), lambda m: m.max(1), lambda m: m.sum(1), lambda m, r: np.exp(m - r[:, None]),
                 lambda a, b, col=False: a * (b[:, None] if col else b), lambda a, b, row=False: a + b, lambda a, k: a * float(k),
                 lambda a, b: a / b)
    ref = [float(v) for v in ref]

    # the same program on the library's operators
    cu = lambda a: torch.from_numpy(np.ascontiguousarray(a, dtype=np.float32)).cuda()
    X_, Y_, W1_, W2_, W3_, b1_, b2_, b3_ = (cu(a) for a in (X, Y, W1, W2, W3, b1, b2, b3))

    def mm(a, b, at=False, bt=False):
        if at:
            a = T.transpose(a, (1, 0))
        return T.product_2d(a, T.transpose_2d(b) if bt else b)

    def add(a, b, row=False):
        if isinstance(b, float):
            return T.binary("add", a, torch.full_like(a, b))
        return T.binary_ax("add", 0, a, b) if row else T.binary("add", a, b)

    def mul(a, b, col=False):
        return T.binary_ax("mul", 1, a, b) if col else T.binary("mul", a, b)
    got = digest(mm, lambda z, b: T.unary("tanh", T.binary_ax("add", 0, z, b)), lambda m: T.reduce("sum", 0, m),
                 lambda m: T.reduce("max", 1, m), lambda m: T.reduce("sum", 1, m), lambda m, r: T.binary_ax("subexp", 1, m, r),
                 mul, add, lambda a, k: T.binary("mul", a, torch.full_like(a, float(k))), lambda a, b: T.binary("div", a, b))
    got = [float(v.item()) for v in got]
    olds = [W1[3, 5], b1[7], W2[11, 13], b2[17], W3[19, 2], b3[3]]
    delta = lambda old, g: float(np.float32(old) - (np.float32(old) - lr * np.float32(g)))
    g_ref, g_got = [delta(o, g) for o, g in zip(olds, ref)], [delta(o, g) for o, g in zip(olds, got)]
    scale = sum(abs(v) for v in g_ref)
    assert abs(sum(g_got) - sum(g_ref)) <= 1e-2 * scale + 1e-6
    for a, b in zip(got, ref):                                   # and every gradient element on its own
        assert abs(a - b) <= 1e-4 * max(1.0, abs(b)) + 1e-6, (got, ref)
