"""ctypes binding of libmimk.so -- the C ABI declared in include/mimk.h.

The library is loaded from this directory (built in-tree by `mimir_b200.build`).  There is no fallback: if it is
missing, importing fails, and if no sm_100 device is present every compute call raises MimkError.
"""
from __future__ import annotations

import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libmimk.so")

F32, BF16, I32, I64 = 0, 1, 2, 3
SUM, MAX, MIN = 0, 1, 2
POST_ID, POST_BIAS, POST_BIAS_RELU, POST_BIAS_TANH, POST_RELU, POST_SILU, POST_ADD_FULL = range(7)
B_KN, B_NK = 0, 1
OP_ADD, OP_SUB, OP_MUL, OP_DIV, OP_MAX, OP_MIN, OP_SUBEXP = range(7)
OP_RELU, OP_TANH, OP_EXP, OP_SILU, OP_NEG, OP_COPY, OP_SQUARE, OP_ABS = range(16, 24)
OP_SQRT, OP_RSQRT, OP_LOG, OP_EXP2, OP_LOG2, OP_SIGMOID = range(24, 30)
E_DEVICE_WAIT = 7
ROWS_SOFTMAX, ROWS_RMSNORM, ROWS_SOFTMAX_RMSNORM = 0, 1, 2

# every symbol include/mimk.h declares
SYMBOLS = (
    "mimk_status_str", "mimk_abi_version", "mimk_last_cuda_error", "mimk_device_check", "mimk_device_status", "mimk_selftest_wait_expiry",
    "mimk_gemm", "mimk_gemm_flat", "mimk_gemm_gather", "mimk_gemm_reduce_scatter", "mimk_gemm_kpanels", "mimk_reduce", "mimk_reduce_fused", "mimk_reduce_plan", "mimk_reduce_static", "mimk_softmax", "mimk_rmsnorm", "mimk_softmax_rmsnorm", "mimk_map", "mimk_map_t",
    "mimk_splat", "mimk_select", "mimk_generate_affine", "mimk_gather", "mimk_scatter", "mimk_attn_fwd", "mimk_mlp_gated", "mimk_map_reduce_post", "mimk_mrp_classify", "mimk_mrp_cell_kernel", "mimk_program_classify", "mimk_program_run", "mimk_chain_order", "mimk_chain_cost",
    "mimk_host_rows", "mimk_host_rows_pair", "mimk_host_gemm", "mimk_host_attn_fwd", "mimk_host_mlp_gated", "mimk_host_map_reduce_post", "mimk_host_register",
    "mimk_host_unregister", "mimk_host_release",
)


class MimkError(RuntimeError):
    def __init__(self, status: int, where: str):
        self.status = status
        msg = lib().mimk_status_str(status).decode()
        if status == 5:
            msg += f" (cudaError {lib().mimk_last_cuda_error()})"
        super().__init__(f"{where}: {msg} [status {status}]")


class GemmDesc(C.Structure):
    _fields_ = [
        ("batch", C.c_int64), ("m", C.c_int64), ("n", C.c_int64), ("k", C.c_int64),
        ("a", C.c_void_p), ("b", C.c_void_p), ("c", C.c_void_p),
        ("stride_a", C.c_int64), ("stride_b", C.c_int64), ("stride_c", C.c_int64),
        ("in_dtype", C.c_int32), ("out_dtype", C.c_int32), ("b_layout", C.c_int32), ("post", C.c_int32),
        ("post_row", C.c_void_p), ("post_full", C.c_void_p),
    ]


class ChainSplit(C.Structure):
    _fields_ = [("i", C.c_int32), ("s", C.c_int32), ("j", C.c_int32), ("t", C.c_int32)]


class GatherDst(C.Structure):
    _fields_ = [("n_dst", C.c_int32), ("first", C.c_int32), ("dst", C.c_void_p * 8), ("ldc", C.c_int64), ("col_off", C.c_int64)]


class AttnDesc(C.Structure):
    _fields_ = [
        ("batch_heads", C.c_int64), ("seq_q", C.c_int64), ("seq_k", C.c_int64), ("head_dim", C.c_int64),
        ("q", C.c_void_p), ("k", C.c_void_p), ("v", C.c_void_p), ("o", C.c_void_p), ("lse", C.c_void_p),
        ("scale", C.c_float), ("causal", C.c_int32), ("dtype", C.c_int32),
    ]


class MlpDesc(C.Structure):
    _fields_ = [
        ("m", C.c_int64), ("k", C.c_int64), ("f", C.c_int64), ("n", C.c_int64),
        ("x", C.c_void_p), ("w1", C.c_void_p), ("w3", C.c_void_p), ("w2", C.c_void_p), ("y", C.c_void_p),
        ("h", C.c_void_p), ("dtype", C.c_int32), ("b_layout", C.c_int32),
    ]


class Producer(C.Structure):
    """mimk_producer: outer_op(inner_op(v, y[...])) applied to every element a fold reads."""
    _fields_ = [("inner_op", C.c_int32), ("outer_op", C.c_int32), ("y_mode", C.c_int32), ("pad_", C.c_int32), ("y", C.c_void_p)]


F_COMPOSED_BASE = 0x01000000
OP_COMPOSED_BASE = 0x10000


def op_composed(inner: int, outer: int) -> int:
    """MIMK_OP_COMPOSED: the elementwise operator outer(inner(x, y))."""
    return OP_COMPOSED_BASE | inner | (outer << 8)



def f_composed(fold: int, inner: int, outer: int = OP_COPY) -> int:
    """MIMK_F_COMPOSED: the combiner fold(acc, outer(inner(a, b)))."""
    return F_COMPOSED_BASE | fold | (inner << 8) | (outer << 16)


MRP_MAX_LOOPS, MRP_MAX_RANK, MRP_MAX_INPUTS = 8, 6, 4
F_ADD, F_MULADD, F_MAX, F_MIN, F_FIRST, F_SUBEXP, F_DIV, F_ADD2, F_MUL2, F_MIX, F_ADD_SUBEXP, F_SUBEXP_DIV = range(12)
STEP_OP, STEP_SOFTMAX, STEP_ATTENTION, STEP_ABSORBED, STEP_FOLD_OF_MAP = range(5)
P_ID, P_ADD, P_ADD_PLUS1, P_ADD_RELU, P_ADD_TANH, P_RELU, P_SILU = range(7)


class AffineMap(C.Structure):
    _fields_ = [("rows", C.c_int32), ("pad_", C.c_int32), ("coef", (C.c_int64 * (MRP_MAX_LOOPS + 1)) * MRP_MAX_RANK),
                ("div", C.c_int64 * MRP_MAX_RANK), ("mod", C.c_int64 * MRP_MAX_RANK)]


class MrpDesc(C.Structure):
    _fields_ = [
        ("ro", C.c_int32), ("rn", C.c_int32),
        ("sr", C.c_int64 * MRP_MAX_LOOPS), ("so", C.c_int64 * MRP_MAX_RANK),
        ("nis", C.c_int32), ("nps", C.c_int32),
        ("in_", C.c_void_p * MRP_MAX_INPUTS), ("in_dtype", C.c_int32 * MRP_MAX_INPUTS),
        ("in_shape", (C.c_int64 * MRP_MAX_RANK) * MRP_MAX_INPUTS), ("in_map", AffineMap * MRP_MAX_INPUTS),
        ("post_in", C.c_void_p * MRP_MAX_INPUTS), ("post_dtype", C.c_int32 * MRP_MAX_INPUTS),
        ("post_shape", (C.c_int64 * MRP_MAX_RANK) * MRP_MAX_INPUTS), ("post_map", AffineMap * MRP_MAX_INPUTS),
        ("map_out", AffineMap),
        ("comb", C.c_int32), ("post", C.c_int32), ("acc_dtype", C.c_int32), ("out_dtype", C.c_int32),
        ("init_bits", C.c_int64), ("out", C.c_void_p),
    ]


_lib = None


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise ImportError(f"{LIB_PATH} is missing: run `python -m mimir_b200.build` (there is no fallback path)")
        L = C.CDLL(LIB_PATH)
        L.mimk_status_str.restype = C.c_char_p
        L.mimk_status_str.argtypes = [C.c_int]
        i64, vp, ci, cf = C.c_int64, C.c_void_p, C.c_int, C.c_float
        L.mimk_device_status.argtypes = [vp]
        L.mimk_selftest_wait_expiry.argtypes = [i64, vp]
        L.mimk_gemm.argtypes = [C.POINTER(GemmDesc), vp]
        L.mimk_gemm_gather.argtypes = [C.POINTER(GemmDesc), vp, C.POINTER(GatherDst), vp]
        L.mimk_gemm_reduce_scatter.argtypes = [C.POINTER(GemmDesc), C.POINTER(GatherDst), i64, vp]
        L.mimk_gemm_kpanels.argtypes = [C.POINTER(GemmDesc), i64, vp]
        L.mimk_gemm_flat.argtypes = [i64, i64, i64, vp, vp, vp, C.c_int32, C.c_int32, C.c_int32, C.c_int32, vp, vp]
        L.mimk_reduce.argtypes = [vp, vp, ci, i64, i64, i64, ci, vp]
        L.mimk_reduce_static.argtypes = [vp, vp, ci, i64, i64, i64, ci, vp]
        L.mimk_reduce_fused.argtypes = [vp, C.POINTER(Producer), vp, ci, i64, i64, i64, ci, vp]
        L.mimk_reduce_plan.argtypes = [i64, i64, i64, ci, C.POINTER(i64)]
        L.mimk_softmax.argtypes = [vp, vp, ci, ci, i64, i64, i64, vp]
        L.mimk_rmsnorm.argtypes = [vp, vp, vp, ci, ci, i64, i64, cf, vp]
        L.mimk_softmax_rmsnorm.argtypes = [vp, vp, vp, ci, ci, i64, i64, cf, vp]
        L.mimk_map.argtypes = [ci, vp, vp, vp, ci, i64, i64, i64, ci, vp]
        L.mimk_map_t.argtypes = [ci, vp, vp, vp, ci, ci, i64, i64, i64, ci, vp]
        L.mimk_attn_fwd.argtypes = [C.POINTER(AttnDesc), vp]
        L.mimk_splat.argtypes = [vp, ci, i64, i64, vp]
        L.mimk_select.argtypes = [vp, vp, vp, vp, ci, i64, vp]
        L.mimk_generate_affine.argtypes = [vp, ci, ci, C.POINTER(i64), C.POINTER(i64), vp]
        L.mimk_program_classify.argtypes = [C.POINTER(MrpDesc), C.c_int32, C.POINTER(C.c_int32)]
        L.mimk_program_run.argtypes = [C.POINTER(MrpDesc), C.c_int32, vp]
        L.mimk_gather.argtypes = [vp, vp, vp, ci, ci, ci, C.POINTER(i64), C.POINTER(i64), ci, vp]
        L.mimk_scatter.argtypes = [vp, vp, vp, vp, ci, ci, ci, C.POINTER(i64), C.POINTER(i64), C.POINTER(i64), ci, vp]
        L.mimk_mlp_gated.argtypes = [C.POINTER(MlpDesc), vp]
        L.mimk_map_reduce_post.argtypes = [C.POINTER(MrpDesc), vp]
        L.mimk_mrp_classify.argtypes = [C.POINTER(MrpDesc)]
        L.mimk_mrp_cell_kernel.argtypes = [C.POINTER(MrpDesc), C.POINTER(C.c_int32)]
        L.mimk_chain_order.argtypes = [C.c_int32, C.POINTER(i64), C.POINTER(C.c_int32), C.c_int32, C.c_int32, C.POINTER(ChainSplit), C.POINTER(C.c_double)]
        L.mimk_chain_cost.argtypes = [C.c_int32, C.POINTER(i64), C.POINTER(C.c_int32), C.c_int32, C.c_int32, C.POINTER(ChainSplit), C.c_int32, C.POINTER(C.c_double)]
        L.mimk_host_rows.argtypes = [ci, vp, vp, vp, ci, ci, i64, i64, cf]
        L.mimk_host_rows_pair.argtypes = [vp, vp, vp, vp, ci, ci, i64, i64, cf]
        L.mimk_host_gemm.argtypes = [C.POINTER(GemmDesc)]
        L.mimk_host_map_reduce_post.argtypes = [C.POINTER(MrpDesc)]
        L.mimk_host_attn_fwd.argtypes = [C.POINTER(AttnDesc)]
        L.mimk_host_mlp_gated.argtypes = [C.POINTER(MlpDesc)]
        L.mimk_host_register.argtypes = [vp, C.c_uint64]
        L.mimk_host_unregister.argtypes = [vp]
        for name in SYMBOLS:
            fn = getattr(L, name)
            if name != "mimk_status_str":
                fn.restype = C.c_int
        _lib = L
    return _lib


def check(status: int, where: str) -> None:
    if status != 0:
        raise MimkError(status, where)
