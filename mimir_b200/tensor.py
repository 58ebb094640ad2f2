"""Host-side mirror of the reference's `tensor` plugin operators, on CUDA torch tensors.

Names and argument meaning follow MimIR's src/mim/plug/tensor/tensor.mim (product_2d 510-513, bmm 404-407,
transpose_2d, reduce 1151-1157, binary_ax 1162-1167, softmax 1172-1176, unary/binary 361-394); a dense row-major
tensor is what `tensor.Tensor r s T` bufferises to (tensor.mim:48-50, buffer/phase/lower_ptr.cpp:16-20).
torch is used for device memory and streams only; every operator is one call into the C ABI (include/mimk.h).
Shape errors the reference reports at compile time ("contracting dims don't match", tensor.mim:1393) are raised
as ValueError before anything is launched; kernel-side failures raise MimkError.
"""
from __future__ import annotations

import ctypes as C
import math

import torch

from . import _lib as L

_DT = {torch.float32: L.F32, torch.bfloat16: L.BF16, torch.int32: L.I32, torch.int64: L.I64}
_TORCH = {v: k for k, v in _DT.items()}
_MONOID = {"sum": L.SUM, "add": L.SUM, "max": L.MAX, "fmax": L.MAX, "min": L.MIN, "fmin": L.MIN}
_POST = {None: L.POST_ID, "id": L.POST_ID, "bias": L.POST_BIAS, "bias_relu": L.POST_BIAS_RELU,
         "bias_tanh": L.POST_BIAS_TANH, "relu": L.POST_RELU, "silu": L.POST_SILU, "add": L.POST_ADD_FULL}
_BINOP = {"add": L.OP_ADD, "sub": L.OP_SUB, "mul": L.OP_MUL, "div": L.OP_DIV, "max": L.OP_MAX, "min": L.OP_MIN,
          "subexp": L.OP_SUBEXP}
_UNOP = {"relu": L.OP_RELU, "tanh": L.OP_TANH, "exp": L.OP_EXP, "silu": L.OP_SILU, "neg": L.OP_NEG, "copy": L.OP_COPY,
         "square": L.OP_SQUARE, "abs": L.OP_ABS, "sqrt": L.OP_SQRT, "rsqrt": L.OP_RSQRT, "log": L.OP_LOG, "exp2": L.OP_EXP2,
         "log2": L.OP_LOG2, "sigmoid": L.OP_SIGMOID}


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _dt(t: torch.Tensor) -> int:
    try:
        return _DT[t.dtype]
    except KeyError:
        raise TypeError(f"unsupported element type {t.dtype}") from None


def _dev(*ts):
    for t in ts:
        if t is not None and not t.is_cuda:
            raise ValueError("mimir_b200.tensor operates on CUDA tensors only (there is no CPU path)")


def device_status() -> None:
    """Synchronise the current stream and raise if a kernel gave up on a bounded wait."""
    L.check(L.lib().mimk_device_status(_stream()), "device_status")


def transpose_2d(t: torch.Tensor) -> torch.Tensor:
    """A read-through view: consumers absorb it into their access maps (fuse.cpp:542-589), nothing is copied."""
    if t.dim() != 2:
        raise ValueError("transpose_2d expects a rank-2 tensor")
    return t.t()


def _b_layout(b: torch.Tensor):
    """Row-major [K,N] -> KN; a transpose_2d view of a row-major [N,K] tensor -> NK (no copy either way)."""
    if b.is_contiguous():
        return b, L.B_KN
    if b.transpose(-1, -2).is_contiguous():
        return b.transpose(-1, -2), L.B_NK
    return b.contiguous(), L.B_KN


def _gemm(a, b_store, layout, batch, m, n, k, sa, sb, out, post, bias, full):
    d = L.GemmDesc()
    d.batch, d.m, d.n, d.k = batch, m, n, k
    d.a, d.b, d.c = a.data_ptr(), b_store.data_ptr(), out.data_ptr()
    d.stride_a, d.stride_b, d.stride_c = sa, sb, m * n
    d.in_dtype, d.out_dtype, d.b_layout, d.post = _dt(a), _dt(out), layout, _POST[post]
    d.post_row = bias.data_ptr() if bias is not None else None
    d.post_full = full.data_ptr() if full is not None else None
    L.check(L.lib().mimk_gemm(C.byref(d), _stream()), "product_2d")


def product_2d(a: torch.Tensor, b: torch.Tensor, *, post=None, bias=None, full=None, out_dtype=None) -> torch.Tensor:
    """C[m,l] = post(sum_k a[m,k] * b[k,l]).  `b` may be a transpose_2d view of a [l,k] tensor."""
    _dev(a, b, bias, full)
    if a.dim() != 2 or b.dim() != 2:
        raise ValueError("product_2d expects rank-2 tensors")
    if a.shape[1] != b.shape[0]:
        raise ValueError("contracting dims don't match")
    if a.dtype != b.dtype:
        raise TypeError("product_2d: both operands share the ring's element type")
    a = a.contiguous()
    b_store, layout = _b_layout(b)
    m, k = a.shape
    n = b.shape[1]
    out = torch.empty((m, n), dtype=out_dtype or a.dtype, device=a.device)
    if bias is not None:
        bias = bias.to(torch.float32).contiguous()
        if bias.numel() != n:
            raise ValueError("bias extent must equal the output's last extent")
    if full is not None:
        full = full.to(out.dtype).contiguous()
        if tuple(full.shape) != (m, n):
            raise ValueError("epilogue operand must have the output's shape")
    _gemm(a, b_store, layout, 1, m, n, k, 0, 0, out, post, bias, full)
    return out


def product_2d_panels(a_panels: torch.Tensor, b: torch.Tensor, *, out_dtype=None) -> torch.Tensor:
    """C = A . b where A [m, G * kp] is given as its G column panels `a_panels` [G, m, kp] -- what an all-gather of
    column slabs delivers -- so that the consumer of a gathered matrix reads it in place (mimk_gemm_kpanels)."""
    _dev(a_panels, b)
    if a_panels.dim() != 3 or b.dim() != 2:
        raise ValueError("product_2d_panels expects [G, m, kp] panels and a rank-2 right operand")
    G, m, kp = a_panels.shape
    if G * kp != b.shape[0]:
        raise ValueError("contracting dims don't match")
    if a_panels.dtype != b.dtype:
        raise TypeError("product_2d_panels: both operands share the ring's element type")
    a_panels = a_panels.contiguous()
    b_store, layout = _b_layout(b)
    n = b.shape[1]
    out = torch.empty((m, n), dtype=out_dtype or a_panels.dtype, device=a_panels.device)
    d = L.GemmDesc()
    d.batch, d.m, d.n, d.k = 1, m, n, G * kp
    d.a, d.b, d.c = a_panels.data_ptr(), b_store.data_ptr(), out.data_ptr()
    d.stride_c = m * n
    d.in_dtype, d.out_dtype, d.b_layout, d.post = _dt(a_panels), _dt(out), layout, L.POST_ID
    L.check(L.lib().mimk_gemm_kpanels(C.byref(d), G, _stream()), "product_2d_panels")
    return out


def bmm(a: torch.Tensor, b: torch.Tensor, *, out_dtype=None) -> torch.Tensor:
    """C[B,m,n] = sum_k a[B,m,k] * b[B,k,n] (tensor.mim:404-407, batching axis 0)."""
    _dev(a, b)
    if a.dim() != 3 or b.dim() != 3:
        raise ValueError("bmm expects rank-3 tensors")
    if a.shape[0] != b.shape[0] or a.shape[2] != b.shape[1]:
        raise ValueError("contracting dims don't match")
    if a.dtype != b.dtype:
        raise TypeError("bmm: both operands share the ring's element type")
    a = a.contiguous()
    b_store, layout = _b_layout(b)
    bt, m, k = a.shape
    n = b.shape[2]
    out = torch.empty((bt, m, n), dtype=out_dtype or a.dtype, device=a.device)
    _gemm(a, b_store, layout, bt, m, n, k, m * k, k * n, out, None, None, None)
    return out


def _view3(x: torch.Tensor, ax: int):
    ax = ax % x.dim()
    outer = math.prod(x.shape[:ax])
    inner = math.prod(x.shape[ax + 1:])
    return ax, outer, x.shape[ax], inner


def reduce(monoid: str, ax: int, x: torch.Tensor) -> torch.Tensor:
    """`reduce (g, init) ax x`: folds axis `ax` away; monoid names the (g, init) pair (sum/max/min)."""
    _dev(x)
    x = x.contiguous()
    ax, outer, ln, inner = _view3(x, ax)
    out = torch.empty(x.shape[:ax] + x.shape[ax + 1:], dtype=x.dtype, device=x.device)
    L.check(L.lib().mimk_reduce(x.data_ptr(), out.data_ptr(), _dt(x), outer, ln, inner, _MONOID[monoid], _stream()),
            "reduce")
    return out


def reduce_fused(monoid: str, ax: int, x: torch.Tensor, inner: str, y: torch.Tensor | None = None, outer: str = "copy") -> torch.Tensor:
    """`reduce (g, init) ax` of an elementwise producer of x that is never written: every element v becomes
    outer(inner(v, y)) as the fold reads it -- what `fuse_tensor` makes of a map feeding a reduce (phase/fuse.cpp:183-358).
    `inner` is a binary operator name with `y` of x's shape, of x's shape without axis `ax` (binary_ax), or of x's trailing
    axes from `ax` on; or a unary name with y = None. `outer` is a unary name."""
    _dev(x)
    _same_float(x)
    x = x.contiguous()
    ax, outer_n, ln, inner_n = _view3(x, ax)
    pre = L.Producer()
    pre.outer_op = _UNOP[outer]
    if y is None:
        pre.inner_op, pre.y_mode, pre.y = _UNOP[inner], 3, None
    else:
        _dev(y)
        _same_float(x, y)
        y = y.contiguous()
        if tuple(y.shape) == tuple(x.shape):
            pre.y_mode = 0
        elif tuple(y.shape) == tuple(x.shape[:ax] + x.shape[ax + 1:]):
            pre.y_mode = 1
        elif tuple(y.shape) == tuple(x.shape[ax:]):
            pre.y_mode = 2
        else:
            raise ValueError("reduce_fused: y must have x's shape, x's shape without axis ax, or x's axes from ax on")
        pre.inner_op, pre.y = _BINOP[inner], y.data_ptr()
    out = torch.empty(x.shape[:ax] + x.shape[ax + 1:], dtype=x.dtype, device=x.device)
    L.check(L.lib().mimk_reduce_fused(x.data_ptr(), C.byref(pre), out.data_ptr(), _dt(x), outer_n, ln, inner_n, _MONOID[monoid],
                                      _stream()), "reduce_fused")
    return out


def softmax(ax: int, x: torch.Tensor, *, out_dtype=None) -> torch.Tensor:
    """`softmax m ax x`: exp(x - max) / sum exp(x - max) along `ax`, one pass over memory."""
    _dev(x)
    x = x.contiguous()
    ax, outer, ln, inner = _view3(x, ax)
    out = torch.empty(x.shape, dtype=out_dtype or x.dtype, device=x.device)
    L.check(L.lib().mimk_softmax(x.data_ptr(), out.data_ptr(), _dt(x), _dt(out), outer, ln, inner, _stream()), "softmax")
    return out


def rmsnorm(x: torch.Tensor, gamma: torch.Tensor, eps: float, *, out_dtype=None) -> torch.Tensor:
    """y = x * rrt(mean(x^2, last axis) + eps) * gamma."""
    _dev(x, gamma)
    x = x.contiguous()
    cols = x.shape[-1]
    if gamma.numel() != cols:
        raise ValueError("gamma extent must equal the last extent of x")
    gamma = gamma.to(torch.float32).contiguous()
    out = torch.empty(x.shape, dtype=out_dtype or x.dtype, device=x.device)
    L.check(L.lib().mimk_rmsnorm(x.data_ptr(), gamma.data_ptr(), out.data_ptr(), _dt(x), _dt(out), x.numel() // max(cols, 1),
                                 cols, eps, _stream()), "rmsnorm")
    return out


def softmax_rmsnorm(x: torch.Tensor, gamma: torch.Tensor, eps: float, *, out_dtype=None) -> torch.Tensor:
    """rmsnorm(softmax(x, last axis)) in one kernel."""
    _dev(x, gamma)
    x = x.contiguous()
    cols = x.shape[-1]
    if gamma.numel() != cols:
        raise ValueError("gamma extent must equal the last extent of x")
    gamma = gamma.to(torch.float32).contiguous()
    out = torch.empty(x.shape, dtype=out_dtype or x.dtype, device=x.device)
    L.check(L.lib().mimk_softmax_rmsnorm(x.data_ptr(), gamma.data_ptr(), out.data_ptr(), _dt(x), _dt(out),
                                         x.numel() // max(cols, 1), cols, eps, _stream()), "softmax_rmsnorm")
    return out


def _same_float(*ts):
    dt = ts[0].dtype
    if dt not in (torch.float32, torch.bfloat16) or any(t.dtype != dt for t in ts):
        raise TypeError("elementwise operators take F32 or BF16 tensors of one element type")
    return dt


def _op(table, op: str, then) -> int:
    """An operator name, optionally with a unary one applied to its result (`then`): MIMK_OP_COMPOSED."""
    return table[op] if then is None else L.op_composed(table[op], _UNOP[then])


def unary(op: str, x: torch.Tensor, *, out_dtype=None, then: str | None = None) -> torch.Tensor:
    _dev(x)
    _same_float(x)
    x = x.contiguous()
    out = torch.empty(x.shape, dtype=out_dtype or x.dtype, device=x.device)
    L.check(L.lib().mimk_map_t(_op(_UNOP, op, then), x.data_ptr(), None, out.data_ptr(), _dt(x), _dt(out), 1, x.numel(), 1, 3, _stream()),
            "unary")
    return out


def binary(op: str, x: torch.Tensor, y: torch.Tensor, *, out_dtype=None, then: str | None = None) -> torch.Tensor:
    _dev(x, y)
    _same_float(x, y)
    if x.shape != y.shape:
        raise ValueError("binary expects operands of one shape")
    x, y = x.contiguous(), y.contiguous()
    out = torch.empty(x.shape, dtype=out_dtype or x.dtype, device=x.device)
    L.check(L.lib().mimk_map_t(_op(_BINOP, op, then), x.data_ptr(), y.data_ptr(), out.data_ptr(), _dt(x), _dt(out), 1, x.numel(), 1, 0,
                               _stream()), "binary")
    return out


def binary_ax(op: str, ax: int, x: torch.Tensor, y: torch.Tensor, *, out_dtype=None, then: str | None = None) -> torch.Tensor:
    """`binary_ax app ax (x, y)`: y lacks axis `ax` of x and is broadcast along it. `then`: a unary operator applied to the
    result in the same pass (a producer inlined into an elementwise consumer)."""
    _dev(x, y)
    _same_float(x, y)
    x, y = x.contiguous(), y.contiguous()
    ax, outer, ln, inner = _view3(x, ax)
    if tuple(y.shape) != tuple(x.shape[:ax] + x.shape[ax + 1:]):
        raise ValueError("binary_ax: y must have x's shape without axis ax")
    out = torch.empty(x.shape, dtype=out_dtype or x.dtype, device=x.device)
    L.check(L.lib().mimk_map_t(_op(_BINOP, op, then), x.data_ptr(), y.data_ptr(), out.data_ptr(), _dt(x), _dt(out), outer, ln, inner, 1,
                               _stream()), "binary_ax")
    return out


def attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, *, scale: float = 1.0, causal: bool = False,
              return_lse: bool = False):
    """softmax(scale * q k^T [+ causal mask]) v over the trailing [seq, head_dim] axes; leading axes are batch x head.
    With scale = 1 and causal = False on rank-2 tensors this is lit/tensor/attn_exec.mim:22."""
    _dev(q, k, v)
    if q.shape[:-2] != k.shape[:-2] or k.shape != v.shape or q.shape[-1] != k.shape[-1]:
        raise ValueError("contracting dims don't match")
    q, k, v = q.contiguous(), k.contiguous(), v.contiguous()
    bh = math.prod(q.shape[:-2])
    o = torch.empty_like(q)
    lse = torch.empty(q.shape[:-1], dtype=torch.float32, device=q.device) if return_lse else None
    d = L.AttnDesc()
    d.batch_heads, d.seq_q, d.seq_k, d.head_dim = bh, q.shape[-2], k.shape[-2], q.shape[-1]
    d.q, d.k, d.v, d.o = q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr()
    d.lse = lse.data_ptr() if lse is not None else None
    d.scale, d.causal, d.dtype = float(scale), int(causal), _dt(q)
    L.check(L.lib().mimk_attn_fwd(C.byref(d), _stream()), "attention")
    return (o, lse) if return_lse else o


def mlp_gated(x: torch.Tensor, w1: torch.Tensor, w3: torch.Tensor, w2: torch.Tensor, *, h: torch.Tensor | None = None):
    """(silu(x w1) * (x w3)) w2, bf16; weights row-major [in, out] or transpose_2d views of [out, in]."""
    _dev(x, w1, w3, w2, h)
    if x.shape[1] != w1.shape[0] or w1.shape != w3.shape or w1.shape[1] != w2.shape[0]:
        raise ValueError("contracting dims don't match")
    x = x.contiguous()
    w1s, lay1 = _b_layout(w1)
    w3s, lay3 = _b_layout(w3)
    w2s, lay2 = _b_layout(w2)
    if not (lay1 == lay3 == lay2):
        raise ValueError("mlp_gated: the three weights must share one storage layout")
    m, k = x.shape
    f, n = w1.shape[1], w2.shape[1]
    y = torch.empty((m, n), dtype=x.dtype, device=x.device)
    d = L.MlpDesc()
    d.m, d.k, d.f, d.n = m, k, f, n
    d.x, d.w1, d.w3, d.w2, d.y = x.data_ptr(), w1s.data_ptr(), w3s.data_ptr(), w2s.data_ptr(), y.data_ptr()
    d.h = h.data_ptr() if h is not None else None
    d.dtype, d.b_layout = _dt(x), lay1
    L.check(L.lib().mimk_mlp_gated(C.byref(d), _stream()), "mlp_gated")
    return y


# ------------------------------------------------------------------------------------------------ the generic op
def proj_map(n_loops: int, subs):
    """`proj_map subs`: result j reads loop variable subs[j] (tensor.mim:196-203), as a coefficient matrix."""
    subs = list(subs)
    m = [[0] * (n_loops + 1) for _ in subs]
    for j, s in enumerate(subs):
        m[j][s] = 1
    return m


def id_map(n: int):
    return proj_map(n, range(n))


class AccessMap(list):
    """An access map with, per result, an optional floordiv and rem behind the linear form: result j =
    (row_j . (loops, 1)) floordiv div[j] rem mod[j] (each applied when > 0) -- the shape affine.delinearize has
    (affine.mim:103-108). A plain list of coefficient rows is a map without either."""

    def __init__(self, rows, div=None, mod=None):
        super().__init__([list(r) for r in rows])
        self.div = [int(v) for v in (div if div is not None else [0] * len(self))]
        self.mod = [int(v) for v in (mod if mod is not None else [0] * len(self))]
        if len(self.div) != len(self) or len(self.mod) != len(self):
            raise ValueError("div / mod need one entry per result")


def reshape_map(s_in, s_out) -> AccessMap:
    """`reshape_map (s_in, s_out)`: o -> delinearize(linearize(o, s_out), s_in), the row-major output-to-input index
    map (tensor.mim:1224-1233)."""
    s_in, s_out = [int(v) for v in s_in], [int(v) for v in s_out]
    if math.prod(s_in) != math.prod(s_out):
        raise ValueError("reshape_map: element counts differ")
    lin = [math.prod(s_out[l + 1:]) for l in range(len(s_out))] + [0]
    return AccessMap([lin for _ in s_in], div=[math.prod(s_in[j + 1:]) for j in range(len(s_in))], mod=s_in)


def compose_reshape(consumer_map, n_loops: int, s_view, s_in) -> AccessMap:
    """What fuse_read_through leaves when a consumer reads a reshape of `s_in` to `s_view` through `consumer_map` (over
    n_loops loop variables, one result per axis of the view): the consumer's coordinates are linearised over the view's
    shape and delinearised over the stored shape (fuse.cpp:542-589 with reshape_map, tensor.mim:1224-1233)."""
    s_view, s_in = [int(v) for v in s_view], [int(v) for v in s_in]
    if getattr(consumer_map, "div", None) and (any(consumer_map.div) or any(consumer_map.mod)):
        raise ValueError("compose_reshape: the consumer's map must be affine")
    lin = [0] * (n_loops + 1)
    for j, row in enumerate(consumer_map):
        stride = math.prod(s_view[j + 1:])
        for l in range(n_loops + 1):
            lin[l] += stride * int(row[l])
    return AccessMap([lin for _ in s_in], div=[math.prod(s_in[j + 1:]) for j in range(len(s_in))], mod=s_in)


def _fill_map(dst, m, n_loops):
    rows = len(m)
    if rows > L.MRP_MAX_RANK:
        raise ValueError("access map has too many results")
    dst.rows = rows
    for j, row in enumerate(m):
        row = [int(v) for v in row]
        if len(row) != n_loops + 1:
            raise ValueError("access map row must have n_loops + 1 coefficients (the last one is the constant)")
        for l in range(n_loops):
            dst.coef[j][l] = row[l]
        dst.coef[j][n_loops] = row[n_loops]
        dst.div[j] = getattr(m, "div", None)[j] if getattr(m, "div", None) else 0
        dst.mod[j] = getattr(m, "mod", None)[j] if getattr(m, "mod", None) else 0


def _mrp_desc(So, Sr, f, init, post, map_out, maps, in_meta, post_maps, post_meta, acc_dtype, out_dtype, out_ptr):
    """The C descriptor of one `map_reduce_post`; operands as (pointer, torch dtype, shape) triples."""
    ro, rn = len(So), len(Sr)
    if rn > L.MRP_MAX_LOOPS or ro > L.MRP_MAX_RANK or len(in_meta) > L.MRP_MAX_INPUTS or len(post_meta) > 1:
        raise ValueError("map_reduce_post: too many loops, axes or inputs for the generic kernel")
    d = L.MrpDesc()
    d.ro, d.rn, d.nis, d.nps = ro, rn, len(in_meta), len(post_meta)
    for i, v in enumerate(Sr):
        d.sr[i] = v
    for i, v in enumerate(So):
        d.so[i] = v
    for i, ((ptr, dt, shape), m) in enumerate(zip(in_meta, maps)):
        if len(shape) > L.MRP_MAX_RANK:
            raise ValueError("input rank too large for the generic kernel")
        d.in_[i] = ptr
        d.in_dtype[i] = _DT[dt]
        for j, v in enumerate(shape):
            d.in_shape[i][j] = v
        if len(m) != len(shape):
            raise ValueError("access map must have one result per input axis")
        _fill_map(d.in_map[i], m, rn)
    for i, ((ptr, dt, shape), m) in enumerate(zip(post_meta, post_maps)):
        d.post_in[i] = ptr
        d.post_dtype[i] = _DT[dt]
        for j, v in enumerate(shape):
            d.post_shape[i][j] = v
        if len(m) != len(shape):
            raise ValueError("epilogue access map must have one result per epilogue-input axis")
        _fill_map(d.post_map[i], m, ro)
    if len(map_out) != ro:
        raise ValueError("map_out must have one result per output axis")
    _fill_map(d.map_out, map_out, rn)
    d.comb, d.post = f, post
    d.acc_dtype, d.out_dtype = _DT[acc_dtype], _DT[out_dtype]
    if acc_dtype == torch.float32:
        import struct
        d.init_bits = struct.unpack("<i", struct.pack("<f", float(init)))[0]
    else:
        d.init_bits = int(init)
    d.out = out_ptr
    return d


ROUTES = {0: "generic", 1: "gemm", 2: "reduce", 3: "map", 4: "permute", 5: "copy"}


def mrp_route(So, Sr, f: int, init, post: int, map_out, maps, in_shapes, in_dtypes, post_maps=(), post_shapes=(),
              post_dtypes=(), *, acc_dtype=torch.float32, out_dtype=None) -> str:
    """Which kernel family `map_reduce_post` would run this instance on ("generic", "gemm", "reduce" or "map"), from
    shapes and dtypes alone -- host logic, no device needed (mimk_mrp_classify)."""
    So, Sr = [int(v) for v in So], [int(v) for v in Sr]
    d = _mrp_desc(So, Sr, f, init, post, map_out, maps, [(0, dt, tuple(sh)) for sh, dt in zip(in_shapes, in_dtypes)], post_maps,
                  [(0, dt, tuple(sh)) for sh, dt in zip(post_shapes, post_dtypes)], acc_dtype, out_dtype or acc_dtype, 0)
    return ROUTES[L.lib().mimk_mrp_classify(C.byref(d))]


CELL_KERNELS = {0: "interpreted", 1: "linear", 2: "compiled"}


def mrp_cell_kernel(So, Sr, f: int, init, post: int, map_out, maps, in_shapes, in_dtypes, *, acc_dtype=torch.float32,
                    out_dtype=None):
    """Which per-cell kernel an instance that stays on the "generic" route runs on, and for "compiled" how many output and
    reduction loops are left after merging: ("compiled", 3, 2) for an NCHW pool. Host logic (mimk_mrp_cell_kernel)."""
    So, Sr = [int(v) for v in So], [int(v) for v in Sr]
    d = _mrp_desc(So, Sr, f, init, post, map_out, maps, [(0, dt, tuple(sh)) for sh, dt in zip(in_shapes, in_dtypes)], (), [],
                  acc_dtype, out_dtype or acc_dtype, 0)
    loops = (C.c_int32 * 2)()
    kind = L.lib().mimk_mrp_cell_kernel(C.byref(d), loops)
    return CELL_KERNELS[kind], int(loops[0]), int(loops[1])


def map_reduce_post(So, Sr, f: int, init, post: int, map_out, maps, ins, post_maps=(), post_ins=(), *,
                    acc_dtype=None, out_dtype=None) -> torch.Tensor:
    """`map_reduce_post` itself (tensor.mim:159-169): combiner / epilogue by id (mimir_b200._lib.F_*, P_*), access
    maps as coefficient matrices [results][n_loops + 1].  `init` is a Python number of the accumulator type.
    Large float instances that are a contraction, an axis fold or an elementwise map run on those kernels
    (see `mrp_route`); everything else on the one-thread-per-cell kernel."""
    _dev(*ins, *post_ins)
    So, Sr = [int(v) for v in So], [int(v) for v in Sr]
    ins = [t.contiguous() for t in ins]
    post_ins = [t.contiguous() for t in post_ins]
    if acc_dtype is None:
        acc_dtype = torch.float32 if (ins and ins[0].dtype in (torch.float32, torch.bfloat16)) or not ins and isinstance(init, float) else (ins[0].dtype if ins else torch.int32)
    if out_dtype is None:
        out_dtype = acc_dtype
    dev = ins[0].device if ins else (post_ins[0].device if post_ins else torch.device("cuda"))
    # a write map that stores loop vector o at o covers the whole result; anything else may leave cells untouched
    covers = So == Sr[:len(So)] and [list(r) for r in map_out] == [list(r) for r in proj_map(len(Sr), range(len(So)))]
    out = (torch.empty if covers else torch.zeros)(So, dtype=out_dtype, device=dev)
    d = _mrp_desc(So, Sr, f, init, post, map_out, maps, [(t.data_ptr(), t.dtype, tuple(t.shape)) for t in ins], post_maps,
                  [(t.data_ptr(), t.dtype, tuple(t.shape)) for t in post_ins], acc_dtype, out_dtype, out.data_ptr())
    L.check(L.lib().mimk_map_reduce_post(C.byref(d), _stream()), "map_reduce_post")
    return out


# ------------------------------------------------------------------------------------------------ programs
STEPS = {0: "op", 1: "softmax", 2: "attention", 3: "absorbed", 4: "fold_of_map"}


class Operand:
    """An operand known by address, element type and shape only (for classifying a program without a device)."""

    def __init__(self, ptr: int, dtype, shape):
        self.ptr, self.dtype, self.shape = int(ptr), dtype, tuple(int(v) for v in shape)


def _meta(t):
    return (t.ptr, t.dtype, t.shape) if isinstance(t, Operand) else (t.data_ptr(), t.dtype, tuple(t.shape))


class Program:
    """An ordered list of `map_reduce_post` operations whose results feed later operations (by address), as a lowering
    that emits one launcher call per operation produces it. `run` executes it through mimk_program_run: chains that spell
    softmax (tensor.mim:1172-1176, also in fuse_tensor's three-operation form) or attention (lit/tensor/attn_exec.mim:20-22)
    run as one fused kernel, everything else op by op."""

    def __init__(self):
        self.descs, self.keep = [], []

    def op(self, out, Sr, f: int, init, post: int, map_out, maps, ins, post_maps=(), post_ins=(), *, acc_dtype=None):
        """Append one operation writing into `out` (a tensor or an Operand); returns `out` for use as a later input."""
        So = list(_meta(out)[2])
        if acc_dtype is None:
            dt = _meta(ins[0])[1] if ins else _meta(out)[1]
            acc_dtype = torch.float32 if dt in (torch.float32, torch.bfloat16) else dt
        d = _mrp_desc(So, [int(v) for v in Sr], f, init, post, map_out, maps, [_meta(t) for t in ins], post_maps,
                      [_meta(t) for t in post_ins], acc_dtype, _meta(out)[1], _meta(out)[0])
        self.descs.append(d)
        self.keep.append((out, ins, post_ins))
        return out

    def _array(self):
        arr = (L.MrpDesc * max(len(self.descs), 1))()
        for i, d in enumerate(self.descs):
            C.memmove(C.byref(arr[i]), C.byref(d), C.sizeof(L.MrpDesc))
        return arr

    def classify(self):
        """How each operation would run: "op", "softmax" / "attention" / "fold_of_map" (first operation of a fused
        chain), "absorbed"."""
        steps = (C.c_int32 * max(len(self.descs), 1))()
        L.check(L.lib().mimk_program_classify(self._array(), len(self.descs), steps), "program_classify")
        return [STEPS[steps[i]] for i in range(len(self.descs))]

    def run(self):
        L.check(L.lib().mimk_program_run(self._array(), len(self.descs), _stream()), "program_run")


# ------------------------------------------------------------------------------------------------ the rest of the op surface
# Every operator below is ONE `map_reduce_post` with the access maps the reference's `_impl` lams build
# (tensor.mim:1086-1134, 1182-1327, 1367-1411, 1443-1468), run by the generic kernel.
def _copy_fn(t):
    return L.F_FIRST, (0.0 if t.dtype in (torch.float32, torch.bfloat16) else 0)


def transpose(x: torch.Tensor, perm) -> torch.Tensor:
    """`transpose perm x`: out[o] = x[o[inv perm]] -- output axis i is input axis perm[i] (tensor.mim:1459)."""
    perm = [int(p) for p in perm]
    r = x.dim()
    if sorted(perm) != list(range(r)):
        raise ValueError("transpose: perm must be a permutation of the axes")
    so = [x.shape[p] for p in perm]
    inv = [perm.index(i) for i in range(r)]
    f, init = _copy_fn(x)
    return map_reduce_post(so, so, f, init, L.P_ID, id_map(r), [proj_map(r, inv)], [x], acc_dtype=_acc(x), out_dtype=x.dtype)


def _acc(t):
    return torch.float32 if t.dtype in (torch.float32, torch.bfloat16) else t.dtype


def flip(x: torch.Tensor) -> torch.Tensor:
    """`flip x`: every axis reversed, read map (s - 1) - o (tensor.mim:1094-1101)."""
    r = x.dim()
    m = [[0] * (r + 1) for _ in range(r)]
    for d in range(r):
        m[d][d] = -1
        m[d][r] = x.shape[d] - 1
    f, init = _copy_fn(x)
    return map_reduce_post(x.shape, x.shape, f, init, L.P_ID, id_map(r), [m], [x], acc_dtype=_acc(x), out_dtype=x.dtype)


def slice_(x: torch.Tensor, start, stride, shape) -> torch.Tensor:
    """`slice`: out[o] = x[start + o * stride] with the given result shape."""
    r = x.dim()
    m = [[0] * (r + 1) for _ in range(r)]
    for d in range(r):
        m[d][d] = int(stride[d])
        m[d][r] = int(start[d])
    f, init = _copy_fn(x)
    return map_reduce_post(list(shape), list(shape), f, init, L.P_ID, id_map(r), [m], [x], acc_dtype=_acc(x), out_dtype=x.dtype)


def broadcast_in_dim(x: torch.Tensor, shape, index) -> torch.Tensor:
    """`broadcast_in_dim`: input axis i reads output loop index[i], or 0 where its extent is 1 (bid_map, tensor.mim:1080-1089)."""
    shape = [int(s) for s in shape]
    ro = len(shape)
    m = [[0] * (ro + 1) for _ in range(x.dim())]
    for i, o in enumerate(index):
        if x.shape[i] != 1:
            if x.shape[i] != shape[o]:
                raise ValueError("broadcast_in_dim: extents must match or be 1")
            m[i][int(o)] = 1
    f, init = _copy_fn(x)
    return map_reduce_post(shape, shape, f, init, L.P_ID, id_map(ro), [m], [x], acc_dtype=_acc(x), out_dtype=x.dtype)


def broadcast(x: torch.Tensor, shape) -> torch.Tensor:
    """`broadcast (s_in, s_out, input)`: same rank, every extent equal to the output's or 1; size-1 axes are expanded
    (tensor.mim:209-218) -- broadcast_in_dim with the identity axis assignment."""
    if x.dim() != len(shape):
        raise ValueError("broadcast keeps the rank; use broadcast_in_dim to add axes")
    return broadcast_in_dim(x, shape, range(x.dim()))


def pad(x: torch.Tensor, lo, hi, value=0) -> torch.Tensor:
    """`pad`: x placed at offset `lo` inside a tensor filled with `value` (edge padding only)."""
    r = x.dim()
    shape = [x.shape[d] + int(lo[d]) + int(hi[d]) for d in range(r)]
    out = torch.full(shape, value, dtype=x.dtype, device=x.device)
    if x.numel() == 0:
        return out
    mo = [[0] * (r + 1) for _ in range(r)]
    for d in range(r):
        mo[d][d] = 1
        mo[d][r] = int(lo[d])
    f, init = _copy_fn(x)
    # the copy writes through map_out = o + lo into the pre-filled result
    d = _mrp_into(out, list(x.shape), f, init, L.P_ID, mo, [id_map(r)], [x])
    return d


def _mrp_into(out, Sr, f, init, post, map_out, maps, ins):
    """map_reduce_post writing into an existing tensor `out` (destination passing, as btensor does)."""
    So = list(out.shape)
    ro, rn = len(So), len(Sr)
    d = L.MrpDesc()
    d.ro, d.rn, d.nis, d.nps = ro, rn, len(ins), 0
    for i, v in enumerate(Sr):
        d.sr[i] = int(v)
    for i, v in enumerate(So):
        d.so[i] = int(v)
    for i, (t, m) in enumerate(zip(ins, maps)):
        t = t.contiguous()
        d.in_[i] = t.data_ptr()
        d.in_dtype[i] = _dt(t)
        for j, v in enumerate(t.shape):
            d.in_shape[i][j] = v
        _fill_map(d.in_map[i], m, rn)
    _fill_map(d.map_out, map_out, rn)
    d.comb, d.post = f, post
    acc = _acc(out)
    d.acc_dtype, d.out_dtype = _DT[acc], _dt(out)
    if acc == torch.float32:
        import struct
        d.init_bits = struct.unpack("<i", struct.pack("<f", float(init)))[0]
    else:
        d.init_bits = int(init)
    d.out = out.data_ptr()
    L.check(L.lib().mimk_map_reduce_post(C.byref(d), _stream()), "map_reduce_post")
    return out


# From this many multiply-adds on a floating-point convolution runs as a contraction on the tensor cores (patches gathered by
# one copy operation, then product_2d); below it, and for integers, as ONE map_reduce_post on the per-cell kernel, which keeps
# the reference's ascending fold per output cell bit for bit.
CONV_CONTRACTION_MIN_WORK = 1 << 27
_CONV_PATCH_BYTES = 1 << 30   # patches of at most this many bytes at a time (whole images per piece)


def _conv_on_tensor_cores(dtype, n, cin, cout, kh, kw, oh, ow) -> bool:
    k = cin * kh * kw
    if dtype == torch.bfloat16:   # the bf16 contraction's alignment rules
        ok = k % 8 == 0 and cout % 8 == 0
    elif dtype == torch.float32:  # the 3xTF32 contraction wants at least one 128 x 128 tile: fewer filters are padded with zeros
        ok = cout >= 16 and n * oh * ow >= 128
    else:
        return False
    return ok and n * cout * oh * ow * k >= CONV_CONTRACTION_MIN_WORK


def _conv_as_contraction(xp, w, n, cin, cout, kh, kw, oh, ow, stride, dilation) -> torch.Tensor:
    """conv as patches x weights: P[(n, oh, ow), (ci, kh, kw)] = xp[n, ci, oh*s + kh*d, ow*s + kw*d] gathered by one copy
    operation (the read map conv_impl builds, tensor.mim:1254-1282, with the reduction loops turned into axes), then
    P . W^T on the contraction kernels with W read through transpose_2d, then the channel axis moved forward by the tiled
    permutation copy."""
    k = cin * kh * kw
    esize = xp.element_size()
    per_image = oh * ow * k * esize
    step = max(1, min(n, _CONV_PATCH_BYTES // max(per_image, 1)))
    w2 = w.contiguous().view(cout, k)
    cpad = cout
    if xp.dtype == torch.float32 and (cout < 128 or cout % 4):
        # rows of zeros up to one tile of filters (a multiple of 4 beyond it): at most twice the tensor-core work, still
        # far ahead of the per-cell kernel; the zero filters' columns of the product are dropped below
        cpad = max(128, (cout + 3) // 4 * 4)
        w2 = torch.cat([w2, torch.zeros((cpad - cout, k), dtype=w2.dtype, device=w2.device)])
    out = torch.empty((n, cout, oh, ow), dtype=xp.dtype, device=xp.device)
    # loops: 0 n, 1 oh, 2 ow, 3 ci, 4 kh, 5 kw
    mi = [[0] * 7 for _ in range(4)]
    mi[0][0] = 1
    mi[1][3] = 1
    mi[2][1], mi[2][4] = stride[0], dilation[0]
    mi[3][2], mi[3][5] = stride[1], dilation[1]
    for n0 in range(0, n, step):
        nb = min(step, n - n0)
        shape = (nb, oh, ow, cin, kh, kw)
        patches = map_reduce_post(shape, shape, L.F_FIRST, 0.0, L.P_ID, id_map(6), [mi], [xp[n0:n0 + nb].contiguous()],
                                  acc_dtype=torch.float32, out_dtype=xp.dtype)
        y = product_2d(patches.view(nb * oh * ow, k), transpose_2d(w2))          # [(n, oh, ow), cout (+ zero filters)]
        if cpad != cout:
            y = y[:, :cout].contiguous()
        out[n0:n0 + nb] = transpose(y.view(nb, oh, ow, cout), (0, 3, 1, 2))
    return out


def conv(x: torch.Tensor, w: torch.Tensor, stride=(1, 1), dilation=(1, 1), padding=(0, 0)) -> torch.Tensor:
    """`conv R (stride, dilation, padding) (input, weight)`: NCHW input, [Cout, Cin, KH, KW] weight (tensor.mim:434-438).
    Loop vector (n, co, oh, ow, ci, kh, kw); the input is read at (n, ci, oh*s + kh*d, ow*s + kw*d) of the padded tensor
    (conv_impl, tensor.mim:1254-1282)."""
    _dev(x, w)
    n, cin, h, wd = x.shape
    cout, cin2, kh, kw = w.shape
    if cin != cin2:
        raise ValueError("contracting dims don't match")
    xp = pad(x, (0, 0, padding[0], padding[1]), (0, 0, padding[0], padding[1])) if any(padding) else x
    oh = (h + 2 * padding[0] - dilation[0] * (kh - 1) - 1) // stride[0] + 1
    ow = (wd + 2 * padding[1] - dilation[1] * (kw - 1) - 1) // stride[1] + 1
    if _conv_on_tensor_cores(x.dtype, n, cin, cout, kh, kw, oh, ow):
        return _conv_as_contraction(xp, w, n, cin, cout, kh, kw, oh, ow, stride, dilation)
    mi = [[0] * 8 for _ in range(4)]
    mi[0][0] = 1
    mi[1][4] = 1
    mi[2][2], mi[2][5] = stride[0], dilation[0]
    mi[3][3], mi[3][6] = stride[1], dilation[1]
    init = 0.0 if x.dtype in (torch.float32, torch.bfloat16) else 0
    return map_reduce_post((n, cout, oh, ow), (n, cout, oh, ow, cin, kh, kw), L.F_MULADD, init, L.P_ID,
                           proj_map(7, (0, 1, 2, 3)), [mi, proj_map(7, (1, 4, 5, 6))], [xp, w], acc_dtype=_acc(x),
                           out_dtype=x.dtype)


def conv_grouped(x: torch.Tensor, w: torch.Tensor, groups: int, stride=(1, 1), dilation=(1, 1), padding=(0, 0)) -> torch.Tensor:
    """`conv_grouped R (groups, stride, dilation, padding) (input, weight)` (tensor.mim:440-451): NCHW input with
    cin = groups * ci channels, weight [cout, ci, KH, KW] with group g owning output channels [g*co, (g+1)*co).
    Loop vector (n, g, co, oh, ow, ci, kh, kw); input channel g*ci + ci and output channel g*co + co are affine because
    input, weight and result are read through their row-major views with the group as an axis of its own
    (conv_grouped_in_map / conv_grouped_w_map, tensor.mim:1284-1297)."""
    _dev(x, w)
    n, cin, h, wd = x.shape
    cout, ci, kh, kw = w.shape
    groups = int(groups)
    if groups < 1 or ci * groups != cin:
        raise ValueError("conv_grouped: weight must hold cin / groups input channels")
    if cout % groups:
        raise ValueError("conv_grouped: cout must be a multiple of groups")
    co = cout // groups
    xp = pad(x, (0, 0, padding[0], padding[1]), (0, 0, padding[0], padding[1])) if any(padding) else x.contiguous()
    hp, wp = xp.shape[2], xp.shape[3]
    oh = (h + 2 * padding[0] - dilation[0] * (kh - 1) - 1) // stride[0] + 1
    ow = (wd + 2 * padding[1] - dilation[1] * (kw - 1) - 1) // stride[1] + 1
    # loops: 0 n, 1 g, 2 co, 3 oh, 4 ow | 5 ci, 6 kh, 7 kw
    mi = [[0] * 9 for _ in range(5)]                    # input viewed [n, g, ci, H, W]
    mi[0][0], mi[1][1], mi[2][5] = 1, 1, 1
    mi[3][3], mi[3][6] = stride[0], dilation[0]
    mi[4][4], mi[4][7] = stride[1], dilation[1]
    init = 0.0 if x.dtype in (torch.float32, torch.bfloat16) else 0
    out = map_reduce_post((n, groups, co, oh, ow), (n, groups, co, oh, ow, ci, kh, kw), L.F_MULADD, init, L.P_ID,
                          proj_map(8, (0, 1, 2, 3, 4)), [mi, proj_map(8, (1, 2, 5, 6, 7))],
                          [xp.view(n, groups, ci, hp, wp), w.contiguous().view(groups, co, ci, kh, kw)], acc_dtype=_acc(x), out_dtype=x.dtype)
    return out.view(n, cout, oh, ow)


def pool(monoid: str, x: torch.Tensor, kernel, stride=None, dilation=(1, 1), padding=(0, 0)) -> torch.Tensor:
    """`pool (g, init) (kernel, stride, dilation, padding, s_out) input` on NCHW (tensor.mim:499-504); padded cells hold
    the monoid's identity."""
    _dev(x)
    stride = stride or kernel
    n, c, h, wd = x.shape
    ident = {"sum": 0.0, "max": float("-inf"), "min": float("inf")}[monoid]
    comb = {"sum": L.F_ADD, "max": L.F_MAX, "min": L.F_MIN}[monoid]
    xp = pad(x, (0, 0, padding[0], padding[1]), (0, 0, padding[0], padding[1]), ident) if any(padding) else x
    oh = (h + 2 * padding[0] - dilation[0] * (kernel[0] - 1) - 1) // stride[0] + 1
    ow = (wd + 2 * padding[1] - dilation[1] * (kernel[1] - 1) - 1) // stride[1] + 1
    mi = [[0] * 7 for _ in range(4)]
    mi[0][0] = 1
    mi[1][1] = 1
    mi[2][2], mi[2][4] = stride[0], dilation[0]
    mi[3][3], mi[3][5] = stride[1], dilation[1]
    return map_reduce_post((n, c, oh, ow), (n, c, oh, ow, kernel[0], kernel[1]), comb, ident, L.P_ID, proj_map(6, (0, 1, 2, 3)),
                           [mi], [xp], acc_dtype=torch.float32, out_dtype=x.dtype)


def dot_product(a: torch.Tensor, b: torch.Tensor, contract, batch=((), ())) -> torch.Tensor:
    """`dot_product R (c1, c2, b1, b2) (a, b)` (tensor.mim:480-486): result axes are the batching axes, then a's free
    axes, then b's (dot_general_shape). Rank-2 products and bmm go to the contraction kernels; any other pattern is one
    generic map_reduce_post with the subscripts dot_product_impl builds (tensor.mim:1381-1396)."""
    _dev(a, b)
    c1, c2 = [int(i) for i in contract[0]], [int(i) for i in contract[1]]
    b1, b2 = [int(i) for i in batch[0]], [int(i) for i in batch[1]]
    for i, j in zip(b1, b2):
        if a.shape[i] != b.shape[j]:
            raise ValueError("batching dims don't match")
    for i, j in zip(c1, c2):
        if a.shape[i] != b.shape[j]:
            raise ValueError("contracting dims don't match")
    if a.dim() == 2 and b.dim() == 2 and not b1 and c1 == [1] and c2 == [0]:
        return product_2d(a, b)
    if a.dim() == 2 and b.dim() == 2 and not b1 and c1 == [1] and c2 == [1]:
        return product_2d(a, transpose_2d(b))
    if a.dim() == 3 and b.dim() == 3 and b1 == [0] and b2 == [0] and c1 == [2] and c2 == [1]:
        return bmm(a, b)
    free1 = [i for i in range(a.dim()) if i not in b1 and i not in c1]
    free2 = [i for i in range(b.dim()) if i not in b2 and i not in c2]
    so = [a.shape[i] for i in b1] + [a.shape[i] for i in free1] + [b.shape[i] for i in free2]
    sr = so + [a.shape[i] for i in c1]
    nb, r_out, n = len(b1), len(so), len(sr)

    def subs(rank, bd, cd, free, off_free):
        s = []
        for i in range(rank):
            if i in bd:
                s.append(bd.index(i))
            elif i in cd:
                s.append(r_out + cd.index(i))
            else:
                s.append(off_free + free.index(i))
        return s

    s1 = subs(a.dim(), b1, c1, free1, nb)
    s2 = subs(b.dim(), b2, c2, free2, nb + len(free1))
    init = 0.0 if a.dtype in (torch.float32, torch.bfloat16) else 0
    return map_reduce_post(so, sr, L.F_MULADD, init, L.P_ID, proj_map(n, range(r_out)), [proj_map(n, s1), proj_map(n, s2)],
                           [a, b], acc_dtype=_acc(a), out_dtype=a.dtype)


# ------------------------------------------------------------------------------------------------ constructors, indexing
def _i64s(vals):
    vals = [int(v) for v in vals]
    return (C.c_int64 * max(len(vals), 1))(*vals)


def _bits(value, dtype) -> int:
    """`value` as the raw bit pattern of one element of `dtype`."""
    t = torch.tensor([value], dtype=dtype)
    width = {1: torch.int8, 2: torch.int16, 4: torch.int32, 8: torch.int64}[t.element_size()]
    return int(t.view(width).item())


def splat(shape, value, dtype=torch.float32, device="cuda") -> torch.Tensor:
    """`splat (s_out, value)`: every element is `value` (tensor.mim:94-109)."""
    out = torch.empty([int(v) for v in shape], dtype=dtype, device=device)
    L.check(L.lib().mimk_splat(out.data_ptr(), _DT[dtype], out.numel(), _bits(value, dtype), _stream()), "splat")
    return out


def generate_affine(shape, coef, dtype=torch.int64, device="cuda") -> torch.Tensor:
    """out[o] = sum_d coef[d] * o[d] + coef[rank]: `generate` (tensor.mim:77-92) for a body affine in the coordinates."""
    shape = [int(v) for v in shape]
    if len(coef) != len(shape) + 1:
        raise ValueError("one coefficient per axis plus a constant")
    out = torch.empty(shape, dtype=dtype, device=device)
    L.check(L.lib().mimk_generate_affine(out.data_ptr(), _DT[dtype], len(shape), _i64s(shape), _i64s(coef), _stream()), "generate")
    return out


def iota(shape, axis: int, dtype=torch.int64, device="cuda") -> torch.Tensor:
    """The coordinate along `axis` at every position of `shape` (an I64 coordinate of `generate`'s body)."""
    coef = [0] * (len(shape) + 1)
    coef[axis] = 1
    return generate_affine(shape, coef, dtype, device)


def generate(shape, body) -> torch.Tensor:
    """`generate s_out body` (tensor.mim:77-92): `body` is called ONCE with one I64 coordinate tensor per axis (each of
    shape s_out, on the device) and returns the tensor of values -- the per-coordinate evaluation of the reference,
    vectorised over the whole index space."""
    shape = [int(v) for v in shape]
    out = body(*[iota(shape, ax) for ax in range(len(shape))])
    if tuple(out.shape) != tuple(shape):
        raise ValueError("generate: body must return one value per coordinate")
    return out


def gather(dim: int, x: torch.Tensor, index: torch.Tensor) -> torch.Tensor:
    """`gather`: out[o] = x[o with o[dim] := index[o]], out has index's shape (tensor.mim:519-541)."""
    _dev(x, index)
    if x.dim() != index.dim() or index.dtype not in (torch.int32, torch.int64):
        raise ValueError("gather: index must have the input's rank and an integer element type")
    x, index = x.contiguous(), index.contiguous()
    out = torch.empty(index.shape, dtype=x.dtype, device=x.device)
    L.check(L.lib().mimk_gather(x.data_ptr(), index.data_ptr(), out.data_ptr(), _dt(x), _DT[index.dtype], x.dim(), _i64s(x.shape),
                                _i64s(index.shape), int(dim), _stream()), "gather")
    return out


def scatter(dim: int, x: torch.Tensor, index: torch.Tensor, updates: torch.Tensor) -> torch.Tensor:
    """`scatter`: a copy of x with x[u with u[dim] := index[u]] = updates[u] for every u of index's shape, visited in
    row-major order -- a destination named twice keeps the later update (tensor.mim:543-563)."""
    _dev(x, index, updates)
    if x.dim() != index.dim() or x.dim() != updates.dim() or index.dtype not in (torch.int32, torch.int64):
        raise ValueError("scatter: index and updates must have the input's rank; index an integer element type")
    if updates.dtype != x.dtype:
        raise TypeError("scatter: updates share the input's element type")
    x, index, updates = x.contiguous(), index.contiguous(), updates.contiguous()
    out = torch.empty_like(x)
    L.check(L.lib().mimk_scatter(x.data_ptr(), index.data_ptr(), updates.data_ptr(), out.data_ptr(), _dt(x), _DT[index.dtype], x.dim(),
                                 _i64s(x.shape), _i64s(index.shape), _i64s(updates.shape), int(dim), _stream()), "scatter")
    return out


def reshape(x: torch.Tensor, shape) -> torch.Tensor:
    """Row-major `reshape` (tensor.mim:302-313): a dense row-major buffer read with another shape -- no copy."""
    shape = [int(v) for v in shape]
    n = 1
    for v in shape:
        n *= v
    if n != x.numel():
        raise ValueError("reshape: element counts differ")
    return x.contiguous().view(shape)


def repeat(x: torch.Tensor, shape) -> torch.Tensor:
    """`repeat`: out[d] = x[d mod s_in] for s_out a multiple of s_in on every axis (tensor.mim:292-300, repeat_map 1209-1213).
    The modulus becomes affine by splitting every output axis into (copy, position), o_d = copy_d * s_in_d + pos_d: the
    result is written through its row-major view of shape (copies_0, s_in_0, copies_1, s_in_1, ...)."""
    shape = [int(v) for v in shape]
    r = x.dim()
    if len(shape) != r or any(si == 0 or so % si for so, si in zip(shape, x.shape)):
        raise ValueError("repeat: every output extent must be a multiple of the input's")
    if 2 * r > L.MRP_MAX_RANK:
        raise ValueError("repeat: rank too large for the generic kernel")
    split = []
    for d in range(r):
        split += [shape[d] // x.shape[d], x.shape[d]]
    out = torch.empty(shape, dtype=x.dtype, device=x.device)
    f, init = _copy_fn(x)
    _mrp_into(out.view(split), split, f, init, L.P_ID, id_map(2 * r), [proj_map(2 * r, [2 * d + 1 for d in range(r)])], [x])
    return out


def concat(ax: int, xs) -> torch.Tensor:
    """`concat ax`: the inputs joined along `ax` (tensor.mim:245-259): input k is copied to the output at offset
    off_k = sum of the earlier inputs' extents along `ax` -- one copy-style map_reduce_post per input."""
    xs = list(xs)
    if not xs:
        raise ValueError("concat of nothing")
    r = xs[0].dim()
    for t in xs:
        if t.dim() != r or t.dtype != xs[0].dtype or any(t.shape[d] != xs[0].shape[d] for d in range(r) if d != ax):
            raise ValueError("concat: inputs agree on rank, element type and every extent except along ax")
    shape = list(xs[0].shape)
    shape[ax] = sum(t.shape[ax] for t in xs)
    out = torch.empty(shape, dtype=xs[0].dtype, device=xs[0].device)
    off = 0
    for t in xs:
        if t.numel():
            m_out = id_map(r)
            m_out[ax][r] = off
            f, init = _copy_fn(t)
            _mrp_into(out, list(t.shape), f, init, L.P_ID, m_out, [id_map(r)], [t])
        off += t.shape[ax]
    return out


def select(cond: torch.Tensor, a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    """`select (cond, a, b)`: `core.select` mapped over tensors of one shape (tensor.mim:378-384) -- a where cond holds,
    b elsewhere. cond is a Bool tensor."""
    _dev(cond, a, b)
    if cond.dtype != torch.bool or a.dtype != b.dtype or not (tuple(cond.shape) == tuple(a.shape) == tuple(b.shape)):
        raise ValueError("select: a Bool tensor and two tensors of one element type, all of one shape")
    cond, a, b = cond.contiguous(), a.contiguous(), b.contiguous()
    out = torch.empty_like(a)
    L.check(L.lib().mimk_select(cond.data_ptr(), a.data_ptr(), b.data_ptr(), out.data_ptr(), _dt(a), a.numel(), _stream()), "select")
    return out


def from_array(values, dtype=torch.float32, device="cuda") -> torch.Tensor:
    """`from_array`: a nested array literal as a tensor (tensor.mim:52-58)."""
    return torch.tensor(values, dtype=dtype).to(device)


def get(t: torch.Tensor, index):
    """`get (t, index)`: one element as a host scalar (tensor.mim:60-63)."""
    return t[tuple(int(i) for i in index)].item()


def set_(t: torch.Tensor, index, value) -> torch.Tensor:
    """`set (t, index, value)`: a copy of t with one element replaced (value semantics, tensor.mim:64-67)."""
    out = t.clone()
    out[tuple(int(i) for i in index)] = value
    return out
