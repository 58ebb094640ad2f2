"""Matrix-chain association for chains of `product_2d`: what the reference's `tensor.reassoc` phase decides at
compile time (MimIR src/mim/plug/tensor/phase/reassoc.cpp), decided here when the chain is about to run.

    chain_product([x, wq, transpose_2d(wk), transpose_2d(x)])      # attention scores, lit/tensor/reassoc.mim:114-124

`model="lanes"` is the reference's price list (vector-lane slots of its CPU schedules) and reproduces its documented
decisions; `model="b200"` prices a product in estimated seconds on this GPU (tile- and wave-quantised tensor-core time
against HBM time) and is the default for running chains. The decision itself is C (mimk_chain_order / mimk_chain_cost).
"""
from __future__ import annotations

import ctypes as C

import torch

from . import _lib as L

_MODEL = {"lanes": 0, "b200": 1}


def _args(dims, transposed, model, dtype, vec):
    dims = [int(d) for d in dims]
    n = len(dims) - 1
    if n < 1:
        raise ValueError("a chain needs at least one matrix")
    if transposed is not None and len(transposed) != n:
        raise ValueError("one `transposed` flag per matrix")
    if model not in _MODEL:
        raise ValueError("model must be 'lanes' or 'b200'")
    c_dims = (C.c_int64 * (n + 1))(*dims)
    c_t = (C.c_int32 * n)(*[int(bool(t)) for t in transposed]) if transposed is not None else None
    param = int(vec) if model == "lanes" else {torch.float32: L.F32, torch.bfloat16: L.BF16}[dtype]
    return n, c_dims, c_t, _MODEL[model], param


def chain_order(dims, transposed=None, *, model="b200", dtype=torch.bfloat16, vec=8):
    """The cheapest bracketing of a chain whose matrix i is dims[i] x dims[i+1].  Returns (splits, cost): splits is a
    list of (i, s, j, t) -- multiply sub-chain i..s by sub-chain s+1..j, storing the product transposed when t -- in an
    order in which they can be executed."""
    n, c_dims, c_t, m, param = _args(dims, transposed, model, dtype, vec)
    out = (L.ChainSplit * max(n - 1, 1))()
    cost = C.c_double()
    L.check(L.lib().mimk_chain_order(n, c_dims, c_t, m, param, out, C.byref(cost)), "chain_order")
    return [(out[q].i, out[q].s, out[q].j, bool(out[q].t)) for q in range(n - 1)], cost.value


def chain_cost(dims, splits, transposed=None, *, model="b200", dtype=torch.bfloat16, vec=8) -> float:
    """The price of the given products (e.g. of a chain as written) under the same model."""
    n, c_dims, c_t, m, param = _args(dims, transposed, model, dtype, vec)
    arr = (L.ChainSplit * max(len(splits), 1))()
    for q, sp in enumerate(splits):
        arr[q].i, arr[q].s, arr[q].j = sp[0], sp[1], sp[2]
        arr[q].t = int(bool(sp[3])) if len(sp) > 3 else 0
    cost = C.c_double()
    L.check(L.lib().mimk_chain_cost(n, c_dims, c_t, m, param, arr, len(splits), C.byref(cost)), "chain_cost")
    return cost.value


def left_deep(n: int):
    """((A0 A1) A2) ... : the bracketing of `a * b * c * d` as the reference's infix product parses it."""
    return [(0, j - 1, j, False) for j in range(1, n)]


def right_deep(n: int):
    """A0 (A1 (A2 ...))"""
    return [(i, i, n - 1, False) for i in range(n - 2, -1, -1)]


def choose(dims, transposed=None, written=None, **kw):
    """The bracketing to run: the optimum, unless the chain as `written` costs no more (reassoc.cpp:349-351 keeps the
    program as it is on a tie).  Returns (splits, cost, reassociated?)."""
    best, cost = chain_order(dims, transposed, **kw)
    if written is not None:
        wcost = chain_cost(dims, written, transposed, **kw)
        if wcost <= cost:
            return list(written), wcost, False
    return best, cost, written is not None


def chain_product(mats, *, written=None, model="b200", out_dtype=None) -> torch.Tensor:
    """mats[0] . mats[1] . ... multiplied in the cheapest association.  Each matrix is a rank-2 device tensor or a
    `transpose_2d` view of one (read through, not copied, when it is a right operand)."""
    from . import tensor as T

    mats = list(mats)
    if not mats:
        raise ValueError("empty chain")
    for a, b in zip(mats, mats[1:]):
        if a.dim() != 2 or b.dim() != 2 or a.shape[1] != b.shape[0]:
            raise ValueError("chain_product: shapes do not chain")
    if len(mats) == 1:
        return mats[0]
    dims = [mats[0].shape[0]] + [m.shape[1] for m in mats]
    transposed = [(not m.is_contiguous()) and m.t().is_contiguous() for m in mats]
    splits, _, _ = choose(dims, transposed, written, model=model, dtype=mats[0].dtype)
    part = {(i, i): m for i, m in enumerate(mats)}
    last = len(mats) - 1
    for sp in splits:
        i, s, j = sp[0], sp[1], sp[2]
        t = len(sp) > 3 and sp[3]
        final = (i, j) == (0, last)
        lhs, rhs = part.pop((i, s)), part.pop((s + 1, j))
        od = out_dtype if final else None
        # a node stored transposed is the product of the transposed parts in reverse order, seen through a transpose
        part[(i, j)] = T.product_2d(rhs.t(), lhs.t(), out_dtype=od).t() if t else T.product_2d(lhs, rhs, out_dtype=od)
    out = part[(0, last)]
    return out if out.is_contiguous() else out.contiguous()
