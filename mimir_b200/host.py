"""Host-buffer form of the operators: CPU tensors in, CPU tensors out, the device in between.

This is the call a program lowered by the reference's GPU path makes today -- every operation uploads its inputs,
launches, and downloads its result (MimIR src/mim/plug/gpu/phase/lower_map_reduce.cpp:317-395) -- served by the
`mimk_host_*` entry points of include/mimk.h.  Pass pinned tensors (`tensor.pin_memory()`) for full copy speed.
"""
from __future__ import annotations

import ctypes as C

import torch

from . import _lib as L
from .tensor import _DT, _POST, _b_layout


def _cpu(*ts):
    for t in ts:
        if t is not None and t.is_cuda:
            raise ValueError("mimir_b200.host takes host tensors; use mimir_b200.tensor for device tensors")


def _rows(kind, x, gamma, eps, out, out_dtype):
    _cpu(x, gamma, out)
    x = x.contiguous()
    cols = x.shape[-1]
    rows = x.numel() // max(cols, 1)
    if out is None:
        out = torch.empty(x.shape, dtype=out_dtype or x.dtype)
    if gamma is not None:
        gamma = gamma.to(torch.float32).contiguous()
        if gamma.numel() != cols:
            raise ValueError("gamma extent must equal the last extent of x")
    L.check(L.lib().mimk_host_rows(kind, x.data_ptr(), gamma.data_ptr() if gamma is not None else None, out.data_ptr(),
                                   _DT[x.dtype], _DT[out.dtype], rows, cols, float(eps)), "host_rows")
    return out


def softmax_rows(x, *, out=None, out_dtype=None):
    return _rows(L.ROWS_SOFTMAX, x, None, 0.0, out, out_dtype)


def rmsnorm(x, gamma, eps, *, out=None, out_dtype=None):
    return _rows(L.ROWS_RMSNORM, x, gamma, eps, out, out_dtype)


def softmax_rmsnorm(x, gamma, eps, *, out=None, out_dtype=None):
    return _rows(L.ROWS_SOFTMAX_RMSNORM, x, gamma, eps, out, out_dtype)


def softmax_and_rmsnorm(x, gamma, eps, *, out_softmax=None, out_rmsnorm=None, out_dtype=None):
    """softmax(x) and rmsnorm(x) along the last axis from one upload of x; returns (softmax, rmsnorm)."""
    _cpu(x, gamma, out_softmax, out_rmsnorm)
    x = x.contiguous()
    cols = x.shape[-1]
    rows = x.numel() // max(cols, 1)
    gamma = gamma.to(torch.float32).contiguous()
    if gamma.numel() != cols:
        raise ValueError("gamma extent must equal the last extent of x")
    if out_softmax is None:
        out_softmax = torch.empty(x.shape, dtype=out_dtype or x.dtype)
    if out_rmsnorm is None:
        out_rmsnorm = torch.empty(x.shape, dtype=out_softmax.dtype)
    if out_softmax.dtype != out_rmsnorm.dtype:
        raise TypeError("both results share one element type")
    L.check(L.lib().mimk_host_rows_pair(x.data_ptr(), gamma.data_ptr(), out_softmax.data_ptr(), out_rmsnorm.data_ptr(),
                                        _DT[x.dtype], _DT[out_softmax.dtype], rows, cols, float(eps)), "host_rows_pair")
    return out_softmax, out_rmsnorm


def product_2d(a, b, *, post=None, bias=None, out=None, out_dtype=None):
    _cpu(a, b, bias, out)
    if a.dim() != 2 or b.dim() != 2 or a.shape[1] != b.shape[0]:
        raise ValueError("contracting dims don't match")
    a = a.contiguous()
    b_store, layout = _b_layout(b)
    m, k = a.shape
    n = b.shape[1]
    if out is None:
        out = torch.empty((m, n), dtype=out_dtype or a.dtype)
    if bias is not None:
        bias = bias.to(torch.float32).contiguous()
    d = L.GemmDesc()
    d.batch, d.m, d.n, d.k = 1, m, n, k
    d.a, d.b, d.c = a.data_ptr(), b_store.data_ptr(), out.data_ptr()
    d.stride_c = m * n
    d.in_dtype, d.out_dtype, d.b_layout, d.post = _DT[a.dtype], _DT[out.dtype], layout, _POST[post]
    d.post_row = bias.data_ptr() if bias is not None else None
    L.check(L.lib().mimk_host_gemm(C.byref(d)), "host product_2d")
    return out


def attention(q, k, v, *, scale=1.0, causal=False, out=None):
    _cpu(q, k, v, out)
    q, k, v = q.contiguous(), k.contiguous(), v.contiguous()
    if out is None:
        out = torch.empty_like(q)
    d = L.AttnDesc()
    bh = q.numel() // (q.shape[-1] * q.shape[-2])
    d.batch_heads, d.seq_q, d.seq_k, d.head_dim = bh, q.shape[-2], k.shape[-2], q.shape[-1]
    d.q, d.k, d.v, d.o = q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr()
    d.scale, d.causal, d.dtype = float(scale), int(causal), _DT[q.dtype]
    L.check(L.lib().mimk_host_attn_fwd(C.byref(d)), "host attention")
    return out


def mlp_gated(x, w1, w3, w2, *, out=None):
    _cpu(x, w1, w3, w2, out)
    x = x.contiguous()
    w1s, lay = _b_layout(w1)
    w3s, _ = _b_layout(w3)
    w2s, _ = _b_layout(w2)
    m, k = x.shape
    f, n = w1.shape[1], w2.shape[1]
    if out is None:
        out = torch.empty((m, n), dtype=x.dtype)
    d = L.MlpDesc()
    d.m, d.k, d.f, d.n = m, k, f, n
    d.x, d.w1, d.w3, d.w2, d.y = x.data_ptr(), w1s.data_ptr(), w3s.data_ptr(), w2s.data_ptr(), out.data_ptr()
    d.dtype, d.b_layout = _DT[x.dtype], lay
    L.check(L.lib().mimk_host_mlp_gated(C.byref(d)), "host mlp_gated")
    return out


def map_reduce_post(So, Sr, f: int, init, post: int, map_out, maps, ins, post_maps=(), post_ins=(), *,
                    acc_dtype=None, out_dtype=None, out=None) -> torch.Tensor:
    """`map_reduce_post` on host tensors: the call the reference's GPU path wraps around EVERY operation (upload the
    inputs and epilogue inputs, run, download the result). Arguments as mimir_b200.tensor.map_reduce_post; `out`
    (optional) supplies the result buffer, whose cells a non-covering write map leaves as they are."""
    from .tensor import _mrp_desc
    _cpu(*ins, *post_ins, out)
    So, Sr = [int(v) for v in So], [int(v) for v in Sr]
    ins = [t.contiguous() for t in ins]
    post_ins = [t.contiguous() for t in post_ins]
    if acc_dtype is None:
        acc_dtype = torch.float32 if ins and ins[0].dtype in (torch.float32, torch.bfloat16) else (ins[0].dtype if ins else torch.int32)
    if out_dtype is None:
        out_dtype = out.dtype if out is not None else acc_dtype
    if out is None:
        out = torch.zeros(So, dtype=out_dtype)
    elif tuple(out.shape) != tuple(So) or out.dtype != out_dtype or not out.is_contiguous():
        raise ValueError("out must be a contiguous tensor of the result's shape and element type")
    d = _mrp_desc(So, Sr, f, init, post, map_out, maps, [(t.data_ptr(), t.dtype, tuple(t.shape)) for t in ins], post_maps,
                  [(t.data_ptr(), t.dtype, tuple(t.shape)) for t in post_ins], acc_dtype, out_dtype, out.data_ptr())
    L.check(L.lib().mimk_host_map_reduce_post(C.byref(d)), "host map_reduce_post")
    return out
