"""Sharding of the hot-path operators over the GPUs of one node (one process per GPU, torch.distributed).

Each sharded configuration is independent on its output, so the data path needs no collective:
  * contraction C = A B: rank g owns a contiguous slab of B's columns (rows of the stored [N,K] tensor) and
    computes C[:, slab]; A is replicated;
  * attention: rank g owns a contiguous range of batch x head;
  * row-wise operators: rank g owns a contiguous block of rows.
A collective appears only when every rank needs the whole result: `gather_columns` / `gather_rows` all-gather the
shards (NCCL over NVLink on GPUs; the same code runs on gloo for CPU tests).  The reference has no multi-device
support at all (device 0 is hard-coded, MimIR src/mim/plug/nvptx/phase/nvptx.cpp:186-204).
"""
from __future__ import annotations

from typing import Callable, Tuple

import torch
import torch.distributed as dist


def split_range(n: int, rank: int, world: int) -> Tuple[int, int]:
    """[lo, hi) of `n` units for `rank`: contiguous, sizes differ by at most one, earlier ranks take the extra."""
    if world <= 0 or not (0 <= rank < world) or n < 0:
        raise ValueError("split_range: need 0 <= rank < world and n >= 0")
    base, extra = divmod(n, world)
    lo = rank * base + min(rank, extra)
    return lo, lo + base + (1 if rank < extra else 0)


def _world():
    if dist.is_available() and dist.is_initialized():
        return dist.get_rank(), dist.get_world_size()
    return 0, 1


def gather_rows(local: torch.Tensor, total_rows: int) -> torch.Tensor:
    """All-gather row blocks (split_range order) into the full [total_rows, ...] tensor on every rank.
    Uneven blocks are padded to the largest one for the collective and trimmed afterwards."""
    rank, world = _world()
    if world == 1:
        return local
    spans = [split_range(total_rows, r, world) for r in range(world)]
    biggest = max(hi - lo for lo, hi in spans)
    tail = tuple(local.shape[1:])
    send = local.contiguous()
    if send.shape[0] != biggest:
        pad = torch.zeros((biggest,) + tail, dtype=local.dtype, device=local.device)
        pad[: send.shape[0]] = send
        send = pad
    recv = torch.empty((world * biggest,) + tail, dtype=local.dtype, device=local.device)
    dist.all_gather_into_tensor(recv, send)
    if biggest * world == total_rows:
        return recv
    return torch.cat([recv[r * biggest: r * biggest + (hi - lo)] for r, (lo, hi) in enumerate(spans)], dim=0)


def gather_columns(local: torch.Tensor, total_cols: int) -> torch.Tensor:
    """All-gather column slabs C[:, lo:hi] into the full [M, total_cols] tensor on every rank."""
    rank, world = _world()
    if world == 1:
        return local
    if local.dim() == 2 and local.shape[1] * world == total_cols:
        # equal slabs: gather them as [world, m, n] panels (the collective's own layout), then ONE copy interleaves them
        m, n = local.shape
        return gather_panels(local).permute(1, 0, 2).reshape(m, world * n)
    return gather_rows(local.t().contiguous(), total_cols).t().contiguous()


def sharded_product_2d(a: torch.Tensor, b_nk: torch.Tensor, compute: Callable, gather: bool = False):
    """C = a . b_nk^T with b_nk stored [N, K]: this rank's slab of B rows -> its columns of C.
    `compute(a, b_slab)` returns a . b_slab^T (mimir_b200.tensor.product_2d with a transpose_2d view on the GPU)."""
    rank, world = _world()
    n = b_nk.shape[0]
    lo, hi = split_range(n, rank, world)
    c_local = compute(a, b_nk[lo:hi])
    return gather_columns(c_local, n) if gather else (c_local, (lo, hi))


def sharded_heads(q, k, v, compute: Callable, gather: bool = False):
    """Attention over this rank's range of the leading (batch x head) axis."""
    rank, world = _world()
    bh = q.shape[0]
    lo, hi = split_range(bh, rank, world)
    o_local = compute(q[lo:hi], k[lo:hi], v[lo:hi])
    return gather_rows(o_local, bh) if gather else (o_local, (lo, hi))


def sharded_rows(x, compute: Callable, gather: bool = False):
    """A row-wise operator over this rank's block of rows."""
    rank, world = _world()
    rows = x.shape[0]
    lo, hi = split_range(rows, rank, world)
    y_local = compute(x[lo:hi])
    return gather_rows(y_local, rows) if gather else (y_local, (lo, hi))


# ---------------------------------------------------------------------------------------------------------------------
# All-gather fused into the contraction's epilogue (GPUs of one node, peer memory over NVLink)
# ---------------------------------------------------------------------------------------------------------------------
class GatheredMatrix:
    """A [rows, cols] matrix that every rank holds a full copy of, allocated so that each rank can store into every
    other rank's copy (torch symmetric memory: peer-mapped device pointers). `local` is this rank's copy."""

    def __init__(self, rows: int, cols: int, dtype=torch.bfloat16, group=None):
        import torch.distributed._symmetric_memory as symm_mem
        self.group = group or dist.group.WORLD
        self.rank, self.world = dist.get_rank(self.group), dist.get_world_size(self.group)
        if self.world > 8:
            raise ValueError("at most 8 destinations (one node)")
        self.local = symm_mem.empty((rows, cols), dtype=dtype, device=torch.device("cuda", torch.cuda.current_device()))
        self.handle = symm_mem.rendezvous(self.local, self.group)
        self.ptrs = [int(p) for p in self.handle.buffer_ptrs]
        self.rows, self.cols = rows, cols

    def barrier(self, channel: int = 0):
        """Every rank's stores (issued before this call on the current stream) are complete on every rank afterwards.
        Barriers that may be in flight at the same time (on different streams) take different channels."""
        self.handle.barrier(channel=channel, timeout_ms=20000)


def gemm_gather(a: torch.Tensor, b: torch.Tensor, out: GatheredMatrix, col_off: int, *, gated_b2: torch.Tensor | None = None,
                row_off: int = 0):
    """This rank's column slab of `a . b` (or silu(a . b) * (a . gated_b2)) stored straight into every rank's copy of
    `out` at rows [row_off, row_off + m), columns [col_off, col_off + n): the all-gather happens in the contraction's
    epilogue.  `b` (and `gated_b2`) may be transpose_2d views of [n, k] tensors.  Call `out.barrier()` before reading
    `out.local`."""
    import ctypes as C

    from . import _lib as L
    from .tensor import _b_layout, _dt, _stream
    a = a.contiguous()
    b_store, layout = _b_layout(b)
    b2_store = None
    if gated_b2 is not None:
        b2_store, layout2 = _b_layout(gated_b2)
        if layout2 != layout:
            raise ValueError("both right operands must share one storage layout")
    m, k = a.shape
    n = b.shape[1]
    if a.shape[1] != b.shape[0] or row_off < 0 or row_off + m > out.rows or col_off + n > out.cols:
        raise ValueError("contracting dims don't match")
    at = row_off * out.cols * out.local.element_size()
    d = L.GemmDesc()
    d.batch, d.m, d.n, d.k = 1, m, n, k
    d.a, d.b, d.c = a.data_ptr(), b_store.data_ptr(), out.local.data_ptr() + at
    d.stride_c = m * n
    d.in_dtype, d.out_dtype, d.b_layout, d.post = _dt(a), _dt(out.local), layout, L.POST_ID
    g = L.GatherDst()
    g.n_dst = out.world
    for i, ptr in enumerate(out.ptrs):
        g.dst[i] = ptr + at
    g.ldc, g.col_off = out.cols, col_off
    L.check(L.lib().mimk_gemm_gather(C.byref(d), b2_store.data_ptr() if b2_store is not None else None, C.byref(g),
                                     _stream()), "gemm_gather")


def tp_mlp_gated(x, w1_shard, w3_shard, w2_shard, h: "GatheredMatrix | None" = None, gather: str = "auto",
                 y: "GatheredMatrix | None" = None):
    """Tensor-parallel gated MLP: rank g holds columns [g F/G, (g+1) F/G) of W1 and W3 and a column slab of W2.
    Stage 1 computes this rank's H slab, H is all-gathered, stage 2 multiplies the full H with this rank's W2 columns.
    Returns this rank's column slab of Y -- or, when a GatheredMatrix `y` ([M, N], N = all ranks' W2 columns) is given,
    the whole Y on every rank: the output all-gather is then fused into the second contraction's epilogue as well
    (NCCL all-gather of the slabs on the "nccl" path).
    gather = "fused": the H slab is stored straight into every rank's H from the contraction's epilogue (needs `h`);
             "nccl":  a local slab and an NCCL all-gather;
             "auto":  fused when a GatheredMatrix is supplied, NCCL otherwise. Measured for the 8192 x 4096 x 14336 block
                      (bulk stores from shared memory to every rank's H against a separate NCCL all-gather):
                      2 GPUs 1.02 / 1.97 ms, 4 GPUs 0.57 / 1.43 ms, 8 GPUs 0.49 / 1.17 ms."""
    from . import tensor as T
    rank, world = _world()
    if gather == "auto":
        gather = "fused" if h is not None else "nccl"
    f_local = w1_shard.shape[1]
    if world == 1:
        return T.mlp_gated(x, w1_shard, w3_shard, w2_shard)
    if gather == "fused":
        if h is None:
            raise ValueError("the fused all-gather needs a GatheredMatrix for H")
        gemm_gather(x, w1_shard, h, rank * f_local, gated_b2=w3_shard)
        h.barrier()
        if y is None:
            out = T.product_2d(h.local, w2_shard)
        else:
            gemm_gather(h.local, w2_shard, y, rank * w2_shard.shape[1])
            out = y.local
        # One barrier after stage 2 on every rank: nobody overwrites H (the next call) while a peer still reads it,
        # and with a gathered Y every rank's slab has landed everywhere.
        (h if y is None else y).barrier()
        return out
    h_local = torch.empty((x.shape[0], f_local), dtype=x.dtype, device=x.device)
    slab = tp_mlp_gated_nccl(x, w1_shard, w3_shard, w2_shard, h_local, gather_y=y is not None)
    if y is None:
        return slab
    y.local.copy_(slab)
    return y.local


_panel_buffers = {}


def gather_panels(local: torch.Tensor) -> torch.Tensor:
    """NCCL all-gather of every rank's [m, n] column slab into one [world, m, n] tensor (panel g = rank g's slab): the
    collective's natural layout, no transposing copy on either side. The receive buffer is cached per shape."""
    rank, world = _world()
    key = (tuple(local.shape), local.dtype, local.device)
    buf = _panel_buffers.get(key)
    if buf is None:
        buf = _panel_buffers[key] = torch.empty((world,) + tuple(local.shape), dtype=local.dtype, device=local.device)
    dist.all_gather_into_tensor(buf, local.contiguous())
    return buf


def tp_mlp_gated_nccl(x, w1_shard, w3_shard, w2_shard, h_local, gather_y: bool = False):
    """The tensor-parallel gated MLP with a separate NCCL all-gather of H: stage 1 into the local slab, all-gather into
    [world, m, F/world] panels, stage 2 reads the panels in place as the K-panels of its left operand
    (mimir_b200.tensor.product_2d_panels). gather_y: all-gather the Y column slabs too and return the whole Y."""
    from . import tensor as T
    rank, world = _world()
    gemm_gather_local(x, w1_shard, w3_shard, h_local)
    if world == 1:
        return T.product_2d(h_local, w2_shard)
    slab = T.product_2d_panels(gather_panels(h_local), w2_shard)
    if not gather_y:
        return slab
    return gather_columns(slab, slab.shape[1] * world)


def tp_mlp_gated_rows(x, w1_shard, w3_shard, w2_rows, h_local, y_partial: "torch.Tensor | None" = None,
                      out_dtype=None) -> torch.Tensor:
    """The tensor-parallel gated MLP with W2 split by ROWS instead of columns: rank g owns columns [g F/G, (g+1) F/G) of
    W1 / W3 and the matching rows of W2, so its slab of H never leaves the GPU; the second contraction gives an f32
    partial of the WHOLE Y, and a reduce-scatter (NCCL) sums the partials and leaves rows [g M/G, (g+1) M/G) of Y on
    rank g. Per rank it moves (G - 1) / G of M x N f32 instead of (G - 1) / G of M x F bf16 for the gather of H."""
    from . import tensor as T
    rank, world = _world()
    gemm_gather_local(x, w1_shard, w3_shard, h_local)
    m, n = x.shape[0], w2_rows.shape[1]
    out_dtype = out_dtype or x.dtype
    if world == 1:
        return T.product_2d(h_local, w2_rows, out_dtype=out_dtype)
    if m % world:
        raise ValueError("tp_mlp_gated_rows: the row count must divide by the number of ranks")
    if y_partial is None:
        y_partial = torch.empty((m, n), dtype=torch.float32, device=x.device)
    _gemm_into(h_local, w2_rows, y_partial)
    mine = torch.empty((m // world, n), dtype=torch.float32, device=x.device)
    dist.reduce_scatter_tensor(mine, y_partial)
    return mine if out_dtype == torch.float32 else T.unary("copy", mine, out_dtype=out_dtype)


def gemm_reduce_scatter(a: torch.Tensor, b: torch.Tensor, acc: GatheredMatrix):
    """This rank's PARTIAL of `a . b` (its K-slab of a, the matching rows of b) added into the owners' accumulators from
    the contraction's epilogue: row block t of the [m, n] product goes to rank t's `acc` (an f32 GatheredMatrix of
    [m / world, n] per rank) by bulk reductions over NVLink.  Every rank zeroes `acc.local` and calls `acc.barrier()`
    before any rank makes this call, and `acc.barrier()` again before reading `acc.local`."""
    import ctypes as C

    from . import _lib as L
    from .tensor import _b_layout, _dt, _stream
    a = a.contiguous()
    b_store, layout = _b_layout(b)
    m, k = a.shape
    n = b.shape[1]
    if a.shape[1] != b.shape[0] or acc.local.dtype != torch.float32 or acc.rows * acc.world != m or acc.cols != n:
        raise ValueError("gemm_reduce_scatter: acc must be an f32 [m / world, n] GatheredMatrix")
    d = L.GemmDesc()
    d.batch, d.m, d.n, d.k = 1, m, n, k
    d.a, d.b, d.c = a.data_ptr(), b_store.data_ptr(), acc.local.data_ptr()
    d.stride_c = m * n
    d.in_dtype, d.out_dtype, d.b_layout, d.post = _dt(a), L.F32, layout, L.POST_ID
    g = L.GatherDst()
    g.n_dst = acc.world
    for i, ptr in enumerate(acc.ptrs):
        g.dst[i] = ptr
    g.ldc, g.col_off = acc.cols, 0
    g.first = (acc.rank + 1) % acc.world      # every rank starts at another owner's rows; its own come last
    L.check(L.lib().mimk_gemm_reduce_scatter(C.byref(d), C.byref(g), acc.rows, _stream()), "gemm_reduce_scatter")


def tp_mlp_gated_rows_fused(x, w1_shard, w3_shard, w2_rows, h_local, acc: GatheredMatrix, out_dtype=None) -> torch.Tensor:
    """tp_mlp_gated_rows with the reduce-scatter fused into the second contraction's epilogue: no partial Y in this
    GPU's memory and no separate collective; every 32 x 32 piece of the f32 partial is added into the owning rank's
    accumulator `acc` (an f32 GatheredMatrix of [M / world, N]) straight from shared memory while the tensor cores work on
    the next tile. Returns rows [g M/G, (g+1) M/G) of Y: a converted copy, or `acc.local` itself for f32 (valid until the
    next call).  The sum's order is not fixed: results agree with the NCCL form up to f32 rounding."""
    from . import tensor as T
    rank, world = _world()
    out_dtype = out_dtype or x.dtype
    if world == 1:
        gemm_gather_local(x, w1_shard, w3_shard, h_local)
        return T.product_2d(h_local, w2_rows, out_dtype=out_dtype)
    acc.local.zero_()
    gemm_gather_local(x, w1_shard, w3_shard, h_local)
    acc.barrier()                      # every accumulator is zero before anybody adds into it
    gemm_reduce_scatter(h_local, w2_rows, acc)
    acc.barrier()                      # every rank's pieces have landed
    return acc.local if out_dtype == torch.float32 else T.unary("copy", acc.local, out_dtype=out_dtype)


def _gemm_into(a, b, out):
    """out = a b into a caller's buffer (f32 or bf16 result of bf16 operands)."""
    import ctypes as C

    from . import _lib as L
    from .tensor import _b_layout, _dt, _stream
    b_store, layout = _b_layout(b)
    m, k = a.shape
    n = b.shape[1]
    d = L.GemmDesc()
    d.batch, d.m, d.n, d.k = 1, m, n, k
    d.a, d.b, d.c = a.data_ptr(), b_store.data_ptr(), out.data_ptr()
    d.in_dtype, d.out_dtype, d.b_layout, d.post = _dt(a), _dt(out), layout, L.POST_ID
    L.check(L.lib().mimk_gemm(C.byref(d), _stream()), "gemm_into")


def gemm_gather_local(x, w1_shard, w3_shard, h_local):
    """Stage 1 of the tensor-parallel MLP into a LOCAL slab (for the variant that all-gathers with NCCL afterwards)."""
    import ctypes as C

    from . import _lib as L
    from .tensor import _b_layout, _dt, _stream
    b_store, layout = _b_layout(w1_shard)
    b2_store, _ = _b_layout(w3_shard)
    m, k = x.shape
    n = w1_shard.shape[1]
    d = L.GemmDesc()
    d.batch, d.m, d.n, d.k = 1, m, n, k
    d.a, d.b, d.c = x.data_ptr(), b_store.data_ptr(), h_local.data_ptr()
    d.stride_c = m * n
    d.in_dtype, d.out_dtype, d.b_layout, d.post = _dt(x), _dt(h_local), layout, L.POST_ID
    g = L.GatherDst()
    g.n_dst = 1
    g.dst[0] = h_local.data_ptr()
    g.ldc, g.col_off = n, 0
    L.check(L.lib().mimk_gemm_gather(C.byref(d), b2_store.data_ptr(), C.byref(g), _stream()), "gemm_gather_local")
