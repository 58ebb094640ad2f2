"""TEST INFRASTRUCTURE ONLY -- numpy/ctypes front end of the CPU oracle (`mimir_oracle.cpp`).

Only the test-suite, the smoke check and the benchmark's CPU-baseline leg may import this package; the
product (`mimir_b200`) never does.  The derived operators below are built on the generic
`map_reduce_post` interpreter exactly the way the reference derives them (MimIR
`src/mim/plug/tensor/tensor.mim`: `product_2d` 1422, `dot_product_impl` 1367-1411, `reduce` 1151-1157,
`binary_ax` 1162-1167, `softmax` 1172-1176, `transpose` via access maps 1459) so that a mistake in a
derivation shows up against the reference's own known answers.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(_HERE, "_ref", "libmimir_oracle.so")

I32, I64, F32, F64, BF16 = 0, 1, 2, 3, 4
_NP2DT = {np.dtype(np.int32): I32, np.dtype(np.int64): I64, np.dtype(np.float32): F32, np.dtype(np.float64): F64}
_DT2NP = {I32: np.int32, I64: np.int64, F32: np.float32, F64: np.float64, BF16: np.uint16}

# combiner / epilogue ids (keep in step with mimir_oracle.cpp)
F_ADD_I32, F_MULADD_I32, F_MIX_I32_I64, F_ADD_F32, F_MULADD_F32, F_FMAX_F32, F_SUBEXP_F32, F_DIV_F32 = range(8)
F_ADD2_F32, F_FIRST_F32, F_MULADD_F64, F_ADD_F64, F_FMIN_F32, F_MUL2_F32, F_FIRST_I32 = range(8, 15)
F_ADD_SUBEXP_F32, F_SUBEXP_DIV_F32 = 15, 16
# fold(acc, outer(inner(u, v))) in f32 -- a combiner with an elementwise producer inlined (fuse.cpp:183-358).
# fold: 0 add, 2 fmax, 3 fmin, 4 first; inner / outer: the elementwise op numbers of the interpreter (0 add .. 6 exp(u - v),
# 16 relu .. 21 identity, 22 square, 23 abs)
F_COMPOSED = 0x01000000


def f_composed(fold: int, inner: int, outer: int = 21) -> int:
    return F_COMPOSED | fold | (inner << 8) | (outer << 16)
P_ID, P_CONV_ADD_I64, P_ADD_PLUS1_I32, P_BIAS_RELU_F32, P_BIAS_TANH_F32, P_BIAS_F32, P_F64_TO_F32 = range(7)


def build(force: bool = False) -> str:
    """Compile the oracle with the committed Makefile (g++, a second or two)."""
    src = os.path.join(_HERE, "mimir_oracle.cpp")
    if force or not os.path.exists(_SO) or os.path.getmtime(_SO) < os.path.getmtime(src):
        subprocess.run(["make", "-C", _HERE], check=True, capture_output=True)
    return _SO


_lib = None


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        _lib = C.CDLL(build())
        _lib.mo_map_reduce_post.restype = C.c_int
    return _lib


# ---------------------------------------------------------------------------------------------
# timed builds (the benchmark's CPU-baseline legs only; parity always runs on the strict build above)
# ---------------------------------------------------------------------------------------------
TIMED_FLAGS = {
    "fast": "g++ -O3 -march=native -ffp-contract=fast",
    "fastmath": "g++ -O3 -march=native -ffp-contract=fast -ffast-math",
}


def _host_tag() -> str:
    """Names the host CPU (model + ISA flags): -march=native code is built per machine and never carried to another."""
    import hashlib
    text = ""
    try:
        with open("/proc/cpuinfo") as f:
            for line in f:
                if line.startswith(("model name", "flags")):
                    text += line
                if line.strip() == "" and text:
                    break
    except OSError:
        pass
    import platform
    return hashlib.sha1((text or platform.processor() or "unknown").encode()).hexdigest()[:10]


def build_timed() -> dict:
    """Compile the two timed variants for THIS host (a few seconds) and return {variant: path}."""
    tag = _host_tag()
    paths = {v: os.path.join(_HERE, "_ref", f"libmimir_oracle_{v}_{tag}.so") for v in TIMED_FLAGS}
    src = os.path.join(_HERE, "mimir_oracle.cpp")
    if any(not os.path.exists(p) or os.path.getmtime(p) < os.path.getmtime(src) for p in paths.values()):
        subprocess.run(["make", "-C", _HERE, "timed", f"TAG={tag}"], check=True, capture_output=True)
    return paths


class timed_build:
    """`with oracle.timed_build("fast"): ...` runs the direct loops of this module on a timed variant of the library
    (same source, the flags in TIMED_FLAGS) instead of the strict parity build. For timing only."""

    def __init__(self, variant: str):
        self.path = build_timed()[variant]

    def __enter__(self):
        global _lib
        lib()
        self.saved = _lib
        _lib = C.CDLL(self.path)
        _lib.mo_map_reduce_post.restype = C.c_int
        return self

    def __exit__(self, *exc):
        global _lib
        _lib = self.saved
        return False


def _p(a: np.ndarray):
    return a.ctypes.data_as(C.c_void_p)


def _i64(xs) -> np.ndarray:
    return np.ascontiguousarray(np.asarray(list(xs), dtype=np.int64).reshape(-1))


def to_bf16(x: np.ndarray) -> np.ndarray:
    """f32 -> bf16 bit pattern (uint16), round to nearest even."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    y = np.empty(x.shape, dtype=np.uint16)
    lib().mo_f32_to_bf16(_p(x), _p(y), C.c_int64(x.size))
    return y


def from_bf16(x: np.ndarray) -> np.ndarray:
    x = np.ascontiguousarray(x, dtype=np.uint16)
    y = np.empty(x.shape, dtype=np.float32)
    lib().mo_bf16_to_f32(_p(x), _p(y), C.c_int64(x.size))
    return y


# ---------------------------------------------------------------------------------------------
# access maps: dense matrices of shape [results, n_loops + 1]; last column is the constant
# ---------------------------------------------------------------------------------------------
def proj_map(n_loops: int, subs) -> np.ndarray:
    """`proj_map subs` (tensor.mim:196-203): result j reads loop variable subs[j]."""
    subs = list(subs)
    m = np.zeros((len(subs), n_loops + 1), dtype=np.int64)
    for j, s in enumerate(subs):
        m[j, s] = 1
    return m


def id_map(n: int) -> np.ndarray:
    return proj_map(n, range(n))


class DivModMap:
    """An access map with a floordiv and a rem per result behind the linear form: result j =
    (matrix[j] . (loops, 1)) floordiv div[j] rem mod[j], each applied when > 0 (affine.semiop.floordiv / rem; the form
    affine.delinearize has, affine.mim:103-108). Accepted wherever a plain coefficient matrix is."""

    def __init__(self, matrix, div, mod):
        self.matrix = np.asarray(matrix, dtype=np.int64)
        self.div, self.mod = [int(v) for v in div], [int(v) for v in mod]
        assert len(self.div) == len(self.mod) == self.matrix.shape[0]


def reshape_map(s_in, s_out) -> DivModMap:
    """`reshape_map (s_in, s_out)`: o -> delinearize(linearize(o, s_out), s_in) (tensor.mim:1224-1233)."""
    s_in, s_out = [int(v) for v in s_in], [int(v) for v in s_out]
    lin = [int(np.prod(s_out[l + 1:], dtype=np.int64)) for l in range(len(s_out))] + [0]
    return DivModMap([lin for _ in s_in], [int(np.prod(s_in[j + 1:], dtype=np.int64)) for j in range(len(s_in))], s_in)


def _split_maps(maps):
    """(plain matrices, flattened (div, mod) pairs or None)"""
    mats = [m.matrix if isinstance(m, DivModMap) else np.asarray(m, dtype=np.int64) for m in maps]
    if not any(isinstance(m, DivModMap) for m in maps):
        return mats, None
    dm = []
    for m, mat in zip(maps, mats):
        for j in range(mat.shape[0]):
            dm += [m.div[j], m.mod[j]] if isinstance(m, DivModMap) else [0, 0]
    return mats, _i64(dm)


def map_reduce_post(So, Sr, f, init, post, map_out, maps, ins, post_maps=(), post_ins=(), out_dtype=None,
                    in_dtypes=None, post_dtypes=None, dst=None) -> np.ndarray:
    """The one real op (tensor.mim:159-169).  `init` is a numpy scalar of the accumulator type. Maps are coefficient
    matrices or DivModMap objects."""
    maps, in_dm = _split_maps(list(maps))
    post_maps, p_dm = _split_maps(list(post_maps))
    (map_out,), out_dm = _split_maps([map_out])
    So, Sr = [int(s) for s in So], [int(s) for s in Sr]
    Ro, Rn = len(So), len(Sr)
    ins = [np.ascontiguousarray(a) for a in ins]
    post_ins = [np.ascontiguousarray(a) for a in post_ins]
    in_dt = list(in_dtypes) if in_dtypes else [_NP2DT[a.dtype] for a in ins]
    p_dt = list(post_dtypes) if post_dtypes else [_NP2DT[a.dtype] for a in post_ins]
    init = np.asarray(init)
    acc_dt = _NP2DT[init.dtype]
    if out_dtype is None:
        out_dtype = acc_dt
    init_bits = int(np.frombuffer(init.tobytes().ljust(8, b"\0"), dtype=np.int64)[0])
    # destination passing, as btensor.map_reduce does (btensor.mim:102-115): cells the write map never stores keep
    # what `dst` held (zeros without one)
    out = np.zeros(So if So else (), dtype=_DT2NP[out_dtype]) if dst is None else np.array(dst, dtype=_DT2NP[out_dtype], copy=True).reshape(So)

    def pack(arrs, mps, n):
        ranks = np.asarray([a.ndim for a in arrs], dtype=np.int32)
        shapes = _i64(s for a in arrs for s in a.shape)
        for a, m in zip(arrs, mps):
            assert np.asarray(m).shape == (a.ndim, n + 1), (np.asarray(m).shape, a.ndim, n)
        flat = _i64(v for m in mps for v in np.asarray(m, dtype=np.int64).reshape(-1))
        ptrs = (C.c_void_p * max(1, len(arrs)))(*[a.ctypes.data for a in arrs])
        return ranks, shapes, flat, ptrs

    ir, ish, imp, iptr = pack(ins, maps, Rn)
    pr, psh, pmp, pptr = pack(post_ins, post_maps, Ro)
    idt = np.asarray(in_dt + [0], dtype=np.int32)
    pdt = np.asarray(p_dt + [0], dtype=np.int32)
    mo = _i64(np.asarray(map_out, dtype=np.int64).reshape(-1))
    assert np.asarray(map_out).shape == (Ro, Rn + 1)
    rc = lib().mo_map_reduce_post(
        C.c_int(Ro), C.c_int(Rn), _p(_i64(Sr + [0])), _p(_i64(So + [0])),
        C.c_int(len(ins)), iptr, _p(idt), _p(ir), _p(ish), _p(imp),
        C.c_int(len(post_ins)), pptr, _p(pdt), _p(pr), _p(psh), _p(pmp),
        _p(mo), C.c_int(f), C.c_int64(init_bits), C.c_int(post), C.c_int(out_dtype), _p(out),
        _p(in_dm) if in_dm is not None else None, _p(p_dm) if p_dm is not None else None,
        _p(out_dm) if out_dm is not None else None)
    if rc != 0:
        raise ValueError(f"map_reduce_post: access outside a buffer or bad ranks (code {rc})")
    return out


# ---------------------------------------------------------------------------------------------
# derived ops, as the reference derives them
# ---------------------------------------------------------------------------------------------
def product_2d(a: np.ndarray, b: np.ndarray, *, b_transposed: bool = False, mode: str = "f32",
               post=P_ID, post_in=None) -> np.ndarray:
    """`product_2d R (a, b)` = dot_product_impl with loops (m, l, k): maps (0,2) and (2,1) (tensor.mim:1422).
    `b_transposed`: `b` is stored [l, k] and read through `transpose_2d` -- the map (1,2) of the stored tensor.
    An epilogue input (bias [l]) is read at output coordinate 1 (fuse_epilogue, fuse.cpp:408-534)."""
    m, k = a.shape
    l = b.shape[0] if b_transposed else b.shape[1]
    maps = [proj_map(3, (0, 2)), proj_map(3, (1, 2) if b_transposed else (2, 1))]
    if a.dtype == np.int32:
        f, init = F_MULADD_I32, np.int32(0)
    elif mode == "f64":
        f, init = F_MULADD_F64, np.float64(0)
    else:
        f, init = F_MULADD_F32, np.float32(0)
    pm, pi = ([proj_map(2, (1,))], [post_in]) if post_in is not None else ([], [])
    return map_reduce_post((m, l), (m, l, k), f, init, post, proj_map(3, (0, 1)), maps, [a, b], pm, pi)


def reduce(x: np.ndarray, ax: int, monoid: str = "sum", mode: str = "f32") -> np.ndarray:
    """`reduce (g, init) ax x` (tensor.mim:1151-1157): output axes lead, `ax` is the trailing loop."""
    r = x.ndim
    so = [s for i, s in enumerate(x.shape) if i != ax]
    sr = so + [x.shape[ax]]
    subs = [j if j < ax else (r - 1 if j == ax else j - 1) for j in range(r)]
    if x.dtype == np.int32:
        f, init = F_ADD_I32, np.int32(0)
    elif monoid == "sum":
        f, init = (F_ADD_F64, np.float64(0)) if mode == "f64" else (F_ADD_F32, np.float32(0))
    elif monoid == "max":
        f, init = F_FMAX_F32, np.float32(-np.inf)
    else:
        f, init = F_FMIN_F32, np.float32(np.inf)
    return map_reduce_post(so, sr, f, init, P_ID, proj_map(r, range(r - 1)), [proj_map(r, subs)], [x])


def binary_ax(app: int, ax: int, x: np.ndarray, y: np.ndarray) -> np.ndarray:
    """`binary_ax app ax (x, y)` (tensor.mim:1162-1167): y lacks axis ax and is broadcast along it."""
    r = x.ndim
    subs = [i if i < ax else i + 1 for i in range(r - 1)]
    return map_reduce_post(x.shape, x.shape, app, np.float32(0), P_ID, id_map(r), [id_map(r), proj_map(r, subs)],
                           [x, y])


def softmax(x: np.ndarray, ax: int) -> np.ndarray:
    """The four map_reduce ops of the `softmax` lam (tensor.mim:1172-1176)."""
    mx = reduce(x, ax, "max")
    e = binary_ax(F_SUBEXP_F32, ax, x, mx)
    return binary_ax(F_DIV_F32, ax, e, reduce(e, ax, "sum"))


def transpose_2d(x: np.ndarray) -> np.ndarray:
    f, init = (F_FIRST_I32, np.int32(0)) if x.dtype == np.int32 else (F_FIRST_F32, np.float32(0))
    return map_reduce_post(x.shape[::-1], x.shape[::-1], f, init, P_ID, id_map(2), [proj_map(2, (1, 0))], [x])


def attention_composed(x, wq, wk, wv) -> np.ndarray:
    """lit/tensor/attn_exec.mim:20-22: softmax(q k^T) v with q,k,v = x wq, x wk, x wv (f32, as lowered)."""
    q, k, v = product_2d(x, wq), product_2d(x, wk), product_2d(x, wv)
    return product_2d(softmax(product_2d(q, k, b_transposed=True), 1), v)


# ---------------------------------------------------------------------------------------------
# direct loops (larger sizes; same per-cell fold order)
# ---------------------------------------------------------------------------------------------
def _rows(rows):
    if rows is None:
        return None, 0
    r = _i64(rows)
    return r, r.size


def gemm(a, b, *, b_nk=False, bf16=False) -> np.ndarray:
    """As lowered: f32 accumulator, ascending k.  bf16=True: inputs are uint16 bf16 bit patterns."""
    a, b = np.ascontiguousarray(a), np.ascontiguousarray(b)
    m, k = a.shape
    n = b.shape[0] if b_nk else b.shape[1]
    c = np.empty((m, n), dtype=np.float32)
    fn = lib().mo_gemm_bf16 if bf16 else lib().mo_gemm_f32
    fn(_p(a), _p(b), _p(c), C.c_int64(m), C.c_int64(n), C.c_int64(k), C.c_int(int(b_nk)))
    return c


def gemm_truth(a, b, *, b_nk=False, bf16=False, rows=None) -> np.ndarray:
    a, b = np.ascontiguousarray(a), np.ascontiguousarray(b)
    m, k = a.shape
    n = b.shape[0] if b_nk else b.shape[1]
    r, nr = _rows(rows)
    c = np.empty((nr or m, n), dtype=np.float64)
    fn = lib().mo_gemm_truth_bf16 if bf16 else lib().mo_gemm_truth_f32
    fn(_p(a), _p(b), _p(c), C.c_int64(m), C.c_int64(n), C.c_int64(k), C.c_int(int(b_nk)),
       _p(r) if nr else None, C.c_int64(nr))
    return c


_MONOID = {"sum": 0, "max": 1, "min": 2}


def reduce_axis(x, ax: int, monoid="sum", truth=False) -> np.ndarray:
    x = np.ascontiguousarray(x, dtype=np.float32)
    outer = int(np.prod(x.shape[:ax], dtype=np.int64))
    inner = int(np.prod(x.shape[ax + 1:], dtype=np.int64))
    shape = x.shape[:ax] + x.shape[ax + 1:]
    out = np.empty(shape, dtype=np.float64 if truth else np.float32)
    fn = lib().mo_reduce_truth if truth else lib().mo_reduce_f32
    fn(_p(x), _p(out), C.c_int64(outer), C.c_int64(x.shape[ax]), C.c_int64(inner), C.c_int(_MONOID[monoid]))
    return out


def softmax_rows(x, truth=False) -> np.ndarray:
    x = np.ascontiguousarray(x, dtype=np.float32)
    y = np.empty(x.shape, dtype=np.float64 if truth else np.float32)
    fn = lib().mo_softmax_rows_truth if truth else lib().mo_softmax_rows_f32
    fn(_p(x), _p(y), C.c_int64(x.shape[0]), C.c_int64(x.shape[1]))
    return y


def rmsnorm_rows(x, gamma, eps, truth=False) -> np.ndarray:
    x = np.ascontiguousarray(x, dtype=np.float32)
    gamma = np.ascontiguousarray(gamma, dtype=np.float32)
    y = np.empty(x.shape, dtype=np.float64 if truth else np.float32)
    if truth:
        lib().mo_rmsnorm_rows_truth(_p(x), _p(gamma), _p(y), C.c_int64(x.shape[0]), C.c_int64(x.shape[1]),
                                    C.c_double(eps))
    else:
        lib().mo_rmsnorm_rows_f32(_p(x), _p(gamma), _p(y), C.c_int64(x.shape[0]), C.c_int64(x.shape[1]),
                                  C.c_float(eps))
    return y


def attention(q, k, v, *, scale=1.0, causal=False, bf16=False, truth=True, heads=None) -> np.ndarray:
    """q,k,v: [BH, S, D].  truth: f64 (the reference driver's check); else f32 as lowered (all heads)."""
    q, k, v = (np.ascontiguousarray(t) for t in (q, k, v))
    bh, s, d = q.shape
    if truth:
        h, nh = _rows(heads)
        o = np.empty((nh or bh, s, d), dtype=np.float64)
        fn = lib().mo_attn_truth_bf16 if bf16 else lib().mo_attn_truth_f32
        fn(_p(q), _p(k), _p(v), _p(o), C.c_int64(bh), C.c_int64(s), C.c_int64(d), C.c_double(scale),
           C.c_int(int(causal)), _p(h) if nh else None, C.c_int64(nh))
    else:
        o = np.empty((bh, s, d), dtype=np.float32)
        fn = lib().mo_attn_bf16 if bf16 else lib().mo_attn_f32
        fn(_p(q), _p(k), _p(v), _p(o), C.c_int64(bh), C.c_int64(s), C.c_int64(d), C.c_float(scale),
           C.c_int(int(causal)))
    return o


def mlp_gated_truth(x, w1, w3, w2, rows=None) -> np.ndarray:
    """bf16 bit-pattern inputs; x [M,K], w1/w3 [K,F], w2 [F,N]; returns f64 [rows or M, N]."""
    x, w1, w3, w2 = (np.ascontiguousarray(t, dtype=np.uint16) for t in (x, w1, w3, w2))
    m, k = x.shape
    f = w1.shape[1]
    n = w2.shape[1]
    r, nr = _rows(rows)
    y = np.empty((nr or m, n), dtype=np.float64)
    lib().mo_mlp_truth_bf16(_p(x), _p(w1), _p(w3), _p(w2), _p(y), C.c_int64(m), C.c_int64(k), C.c_int64(f),
                            C.c_int64(n), _p(r) if nr else None, C.c_int64(nr))
    return y


def normalised_error(got, want) -> float:
    """max|got - want| / max|want| per tensor -- the parity metric every report states."""
    got = np.asarray(got, dtype=np.float64)
    want = np.asarray(want, dtype=np.float64)
    denom = float(np.max(np.abs(want))) or 1.0
    return float(np.max(np.abs(got - want))) / denom


# ---- constructors and data-dependent indexing (tensor.mim:77-109, 245-313, 519-563): the docstrings' loops, verbatim ----
def generate(shape, body) -> np.ndarray:
    """output[index] = body(index) for every index of `shape` (tensor.mim:81-87); body takes the coordinates as ints."""
    first = body(*([0] * len(shape))) if all(shape) else 0
    out = np.empty(shape, dtype=np.asarray(first).dtype)
    for index in np.ndindex(*shape):
        out[index] = body(*index)
    return out


def gather(dim: int, x: np.ndarray, index: np.ndarray) -> np.ndarray:
    """tensor.mim:527-535."""
    out = np.empty(index.shape, dtype=x.dtype)
    for o in np.ndindex(*index.shape):
        src = tuple(int(index[o]) if d == dim else o[d] for d in range(x.ndim))
        out[o] = x[src]
    return out


def scatter(dim: int, x: np.ndarray, index: np.ndarray, updates: np.ndarray) -> np.ndarray:
    """tensor.mim:549-557: row-major visiting order, so the last update of a destination wins."""
    out = x.copy()
    for u in np.ndindex(*index.shape):
        dst = tuple(int(index[u]) if d == dim else u[d] for d in range(x.ndim))
        out[dst] = updates[u]
    return out


def repeat(x: np.ndarray, shape) -> np.ndarray:
    """out[d] = x[d mod s_in] (tensor.mim:292-300)."""
    out = np.empty(shape, dtype=x.dtype)
    for o in np.ndindex(*shape):
        out[o] = x[tuple(o[d] % x.shape[d] for d in range(x.ndim))]
    return out


def concat(ax: int, xs) -> np.ndarray:
    """out[o] = xs[k][o with o[ax] - off_k], k the input whose range o[ax] falls in (tensor.mim:245-259)."""
    shape = list(xs[0].shape)
    shape[ax] = sum(t.shape[ax] for t in xs)
    out = np.empty(shape, dtype=xs[0].dtype)
    for o in np.ndindex(*shape):
        off = 0
        for t in xs:
            if o[ax] < off + t.shape[ax]:
                out[o] = t[tuple(o[d] - off if d == ax else o[d] for d in range(len(shape)))]
                break
            off += t.shape[ax]
    return out
