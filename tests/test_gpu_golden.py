"""The CUDA path against the committed fixtures (tests/golden/cases.npz): the same seeded inputs through the C ABI,
compared with the frozen f64 answers. Tolerances: 1e-5 normalised for f32 results, 2e-2 for bf16 results, 1e-4 for
f32 stores of bf16 contractions."""
import numpy as np
import pytest
import torch

from tests.test_golden_fixtures import FIX, MG
from tests.util import TOL_BF16, TOL_F32, f64, nerr

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def T():
    from mimir_b200 import tensor
    return tensor


def dev(x, bf16=False):
    t = torch.from_numpy(np.ascontiguousarray(x))
    if bf16:
        t = t.view(torch.int16).view(torch.bfloat16)
    return t.cuda()


@pytest.mark.parametrize("name", sorted(n for n, (k, _) in MG.CASES.items() if k == "gemm"))
def test_contractions(T, name):
    _, p = MG.CASES[name]
    a, b = (dev(x, p["bf16"]) for x in MG.inputs("gemm", p))
    rows = p.get("rows", list(range(p["m"])))
    bv = b.t() if p["nk"] else b
    c = T.product_2d(a, bv, out_dtype=torch.float32)
    assert nerr(f64(c[rows]), FIX[name]) <= (1e-4 if p["bf16"] else TOL_F32)
    if p["bf16"]:
        assert nerr(f64(T.product_2d(a, bv)[rows]), FIX[name]) <= TOL_BF16


def test_rows_and_reductions(T):
    _, p = MG.CASES["softmax_rows"]
    (x,) = MG.inputs("softmax", p)
    assert nerr(f64(T.softmax(1, dev(x))), FIX["softmax_rows"]) <= TOL_F32
    assert nerr(f64(T.softmax(1, dev(x), out_dtype=torch.bfloat16)), FIX["softmax_rows"]) <= TOL_BF16
    _, p = MG.CASES["rmsnorm_rows"]
    x, g = MG.inputs("rmsnorm", p)
    assert nerr(f64(T.rmsnorm(dev(x), dev(g), p["eps"])), FIX["rmsnorm_rows"]) <= TOL_F32
    assert nerr(f64(T.rmsnorm(dev(x), dev(g), p["eps"], out_dtype=torch.bfloat16)), FIX["rmsnorm_rows"]) <= TOL_BF16
    for name in ("reduce_sum_ax0", "reduce_max_ax1", "reduce_sum_ax2"):
        _, p = MG.CASES[name]
        (x,) = MG.inputs("reduce", p)
        got = f64(T.reduce(p["monoid"], p["ax"], dev(x)))
        if p["monoid"] == "max":
            assert np.array_equal(got, FIX[name])
        else:
            assert nerr(got, FIX[name]) <= TOL_F32


@pytest.mark.parametrize("name", sorted(n for n, (k, _) in MG.CASES.items() if k == "attn"))
def test_attention(T, name):
    _, p = MG.CASES[name]
    q, k, v = (dev(x, p["bf16"]) for x in MG.inputs("attn", p))
    o = T.attention(q, k, v, scale=float(p["d"]) ** -0.5, causal=p["causal"])
    T.device_status()
    got = f64(o[p["heads"]])
    if "qrows" in p:
        got = got[:, p["qrows"]]
    assert nerr(got, FIX[name]) <= (TOL_BF16 if p["bf16"] else 1e-4)


def test_mlp_gated(T):
    _, p = MG.CASES["mlp_gated"]
    x, w1, w3, w2 = (dev(t, True) for t in MG.inputs("mlp", p))
    y = T.mlp_gated(x, w1, w3, w2)
    assert nerr(f64(y[p["rows"]]), FIX["mlp_gated"]) <= TOL_BF16
