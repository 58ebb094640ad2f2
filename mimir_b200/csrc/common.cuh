// Shared host/device helpers of the mimk kernel library (sm_100a only).
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "mimk.h"

namespace mimk {

// ---- host side ------------------------------------------------------------------------------------
// Records a failed CUDA call for mimk_last_cuda_error() and maps it to MIMK_E_CUDA.
int note_cuda_error(cudaError_t e);
#define MIMK_CUDA_TRY(expr)                                        \
    do {                                                           \
        cudaError_t mimk_e_ = (expr);                              \
        if (mimk_e_ != cudaSuccess) return note_cuda_error(mimk_e_); \
    } while (0)
#define MIMK_TRY(expr)                    \
    do {                                  \
        int mimk_s_ = (expr);             \
        if (mimk_s_ != MIMK_OK) return mimk_s_; \
    } while (0)

inline int launch_status() { return note_cuda_error(cudaGetLastError()); }

struct DeviceInfo {
    int device = -1;
    int sm_count = 0;
    int cc_major = 0;
    int* status_dev = nullptr;   // device-visible alias of the pinned status word
    volatile int* status_host = nullptr;
    // Cached scratch buffers (grown on demand), one per stream that has asked for one: calls on different streams never
    // share a buffer, calls on one stream are ordered by it. `kind` 0 is the general buffer, 1 the second one for callers
    // that run scratch-using entry points themselves.
    struct Scratch {
        cudaStream_t stream = nullptr;
        void* ptr           = nullptr;
        size_t bytes        = 0;
        unsigned long long last_use = 0;
        bool used           = false;
    };
    static constexpr int SCRATCH_SLOTS = 8;
    Scratch scratch[2][SCRATCH_SLOTS];
    unsigned long long scratch_clock = 0;
};
// Per-device lazily created state; returns nullptr (and sets *status) when the device is unusable.
DeviceInfo* device_info(int* status);
// A scratch buffer of at least `bytes` on the current device for work queued on `stream`, cached across calls (grows,
// never shrinks). Up to DeviceInfo::SCRATCH_SLOTS streams keep a buffer of their own; one more evicts the least recently used
// (after waiting for the device).
int get_scratch(size_t bytes, void** out, cudaStream_t stream);
// The second cached buffer (same rules); used by the composed f32 attention for its score matrix.
int get_aux_scratch(size_t bytes, void** out, cudaStream_t stream);

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }
inline size_t dtype_size(int dt) { return dt == MIMK_BF16 ? 2 : (dt == MIMK_I64 ? 8 : 4); }

// kernels implemented in the other translation units
int gemm_simt(const mimk_gemm_desc& d, cudaStream_t s);
int gemm_simt_preferred(const mimk_gemm_desc& d);  // small f32 product: the 32 x 32-tile CUDA-core kernel beats 3xTF32
int gemm_tc_supported(const mimk_gemm_desc& d);
// a_panels > 1: A is given as that many row-major [m, k / a_panels] matrices one after another (the layout an all-gather
// of column slabs delivers); k / a_panels must then be a multiple of 64
int gemm_tc(const mimk_gemm_desc& d, cudaStream_t s, int gated, const void* b2, const mimk_gather_dst* gather = nullptr,
            int64_t a_panels = 1);
int gemm_tc2_supported(const mimk_gemm_desc& d, int gated);  // the paired-SM (cta_group::2) form
// scatter_rows > 0 (gemm_tc2 only): rows [t scatter_rows, (t + 1) scatter_rows) of the f32 result are added into gather->dst[t]
int gemm_tc2(const mimk_gemm_desc& d, cudaStream_t s, int gated, const void* b2, const mimk_gather_dst* gather = nullptr,
             int64_t a_panels = 1, int64_t scatter_rows = 0);
int gemm_tc_any(const mimk_gemm_desc& d, cudaStream_t s, int gated, const void* b2,
                const mimk_gather_dst* gather = nullptr, int64_t a_panels = 1);  // picks between the two
int gemm_f32_tc_supported(const mimk_gemm_desc& d);  // f32 operands on the tensor cores (3xTF32)
int gemm_f32_tc(const mimk_gemm_desc& d, cudaStream_t s);
// map_reduce_post instances that are a contraction, an axis fold or an elementwise map go to those kernels (mrp_route.cu)
bool mrp_try_route(const mimk_mrp_desc& d, void* stream, int* status);
// What a descriptor's access maps spell, whatever its size (the router itself leaves small instances on the per-cell
// kernel): route MIMK_ROUTE_*, and the arguments of the specialised entry point that would take it.
inline bool op_is_binary(int op) { return op >= MIMK_OP_ADD && op <= MIMK_OP_SUBEXP; }
inline bool op_is_unary(int op) { return op >= MIMK_OP_RELU && op <= MIMK_OP_SIGMOID; }  // COPY included
// A (possibly composed) elementwise operator taken apart; false when it names an unknown part.
inline bool decode_op(int op, int* inner, int* outer) {
    *inner = op, *outer = MIMK_OP_COPY;
    if (op & MIMK_OP_COMPOSED_BASE) {
        if (op & ~0x1ffff) return false;
        *inner = op & 0xff, *outer = (op >> 8) & 0xff;
    }
    return (op_is_binary(*inner) || op_is_unary(*inner)) && op_is_unary(*outer);
}
// A composed combiner taken apart; false when `comb` is not one or names an unknown part.
inline bool decode_composed(int comb, int* fold, int* inner, int* outer) {
    if ((comb & ~0x00ffffff) != MIMK_F_COMPOSED_BASE) return false;
    *fold = comb & 0xff, *inner = (comb >> 8) & 0xff, *outer = (comb >> 16) & 0xff;
    if (*fold != MIMK_F_ADD && *fold != MIMK_F_MAX && *fold != MIMK_F_MIN && *fold != MIMK_F_FIRST) return false;
    return (op_is_binary(*inner) || op_is_unary(*inner)) && op_is_unary(*outer);
}
struct MrpPlan {
    int route = MIMK_ROUTE_GENERIC;
    mimk_gemm_desc gemm{};
    int64_t outer = 0, len = 0, inner = 0;  // reduce / map: the [outer, len, inner] view
    int monoid = 0, op = 0, y_mode = 3;
    int pre_inner = -1, pre_outer = -1, pre_y_mode = 3;  // reduce with an inlined producer (pre_inner >= 0); its y is input 1
    int perm[MIMK_MRP_MAX_RANK] = {};
};
MrpPlan mrp_plan(const mimk_mrp_desc& d);
// axis permutation as a tiled copy (permute.cu); perm[j] = the output loop that indexes input axis j
int permute_copy(const void* in, void* out, int esize, int rank, const int64_t* out_shape, const int* perm, cudaStream_t s);
int attn_simt(const mimk_attn_desc& d, cudaStream_t s);
// f32, and bf16 with other head dims, at scale: the composition S = Q K^T, softmax, O = P V on the contraction and row
// kernels (attn_composed.cu)
int attn_composed_supported(const mimk_attn_desc& d);
int attn_composed(const mimk_attn_desc& d, cudaStream_t s);
// bf16, head_dim 64 or 128: one CTA per SM pulls (head, query-tile pair) items, hand-over between items pipelined
int attn_tc_persistent_supported(const mimk_attn_desc& d);
int attn_tc_persistent(const mimk_attn_desc& d, cudaStream_t s);
// bf16, head_dim 128, on paired SMs (cta_group::2): one query tile per CTA, double-buffered scores (attn_tc2.cu)
int attn_tc_pair_supported(const mimk_attn_desc& d);
int attn_tc_pair(const mimk_attn_desc& d, cudaStream_t s);

// ---- device side ----------------------------------------------------------------------------------
#ifdef __CUDACC__
// the scalar meaning of MIMK_OP_* (unary ones ignore b)
__device__ __forceinline__ float apply_op_plain(int op, float a, float b) {
    switch (op) {
        case MIMK_OP_ADD: return a + b;
        case MIMK_OP_SUB: return a - b;
        case MIMK_OP_MUL: return a * b;
        case MIMK_OP_DIV: return a / b;
        case MIMK_OP_MAX: return fmaxf(a, b);
        case MIMK_OP_MIN: return fminf(a, b);
        case MIMK_OP_SUBEXP: return expf(a - b);
        case MIMK_OP_RELU: return fmaxf(0.f, a);
        case MIMK_OP_TANH: return tanhf(a);
        case MIMK_OP_EXP: return expf(a);
        case MIMK_OP_SILU: return a / (1.f + expf(-a));
        case MIMK_OP_NEG: return -a;
        case MIMK_OP_SQUARE: return a * a;
        case MIMK_OP_ABS: return fabsf(a);
        case MIMK_OP_SQRT: return sqrtf(a);
        case MIMK_OP_RSQRT: return 1.f / sqrtf(a);  // math.rrt is a division by rt.sq, not an approximation
        case MIMK_OP_LOG: return logf(a);
        case MIMK_OP_EXP2: return exp2f(a);
        case MIMK_OP_LOG2: return log2f(a);
        case MIMK_OP_SIGMOID: return 1.f / (1.f + expf(-a));
        default: return a;
    }
}
// ... and of a MIMK_OP_COMPOSED pair: outer(inner(a, b))
__device__ __forceinline__ float apply_op(int op, float a, float b) {
    if (op & MIMK_OP_COMPOSED_BASE) return apply_op_plain((op >> 8) & 0xff, apply_op_plain(op & 0xff, a, b), 0.f);
    return apply_op_plain(op, a, b);
}
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}
__device__ __forceinline__ float warp_min(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fminf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// Epilogue `post(acc, row, full)`.
__device__ __forceinline__ float apply_post(int post, float acc, float row, float full) {
    switch (post) {
        case MIMK_POST_BIAS: return acc + row;
        case MIMK_POST_BIAS_RELU: return fmaxf(0.f, acc + row);
        case MIMK_POST_BIAS_TANH: return tanhf(acc + row);
        case MIMK_POST_RELU: return fmaxf(0.f, acc);
        case MIMK_POST_SILU: return acc / (1.f + __expf(-acc));
        case MIMK_POST_ADD_FULL: return acc + full;
        default: return acc;
    }
}

__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}
#endif

}  // namespace mimk
