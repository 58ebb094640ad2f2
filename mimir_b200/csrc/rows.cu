// Bandwidth-bound kernels: reduce, softmax, RMSNorm, elementwise maps.
//
// These are the `map_reduce_post` instances with a short reduction per output cell (MimIR
// src/mim/plug/tensor/tensor.mim:1151-1176). The reference's GPU lowering gives each output cell one thread
// that walks its reduction sequentially (src/mim/plug/gpu/phase/lower_map_reduce.cpp:198-260) and runs softmax
// as four kernels; here a row lives in the registers of one CTA, is read from HBM once with 128-bit loads,
// reduced with warp shuffles, and written once.
#include <math_constants.h>

#include <mutex>

#include "common.cuh"

// Home of the partial results of mimk_reduce_static's split-axis reduction (instead of the library's cached
// cudaMalloc'd scratch). Every GPU that loads the library holds these bytes until the process exits.
constexpr size_t STATIC_PARTIALS = MIMK_REDUCE_STATIC_BYTES / sizeof(float);  // 262144 floats = 1 MiB
static __device__ __align__(256) float g_static_partials[STATIC_PARTIALS];

namespace mimk {
namespace {

enum { ROWS_SOFTMAX = 0, ROWS_RMSNORM = 1, ROWS_SOFTMAX_RMSNORM = 2 };

struct SumOp {
    __device__ float operator()(float a, float b) const { return a + b; }
    __device__ static float ident() { return 0.f; }
};
struct MaxOp {
    __device__ float operator()(float a, float b) const { return fmaxf(a, b); }
    __device__ static float ident() { return -CUDART_INF_F; }
};
struct MinOp {
    __device__ float operator()(float a, float b) const { return fminf(a, b); }
    __device__ static float ident() { return CUDART_INF_F; }
};

template <class Op>
__device__ __forceinline__ float warp_reduce(float v, Op op) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = op(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// Every warp ends up with the block-wide result; `red` (32 floats of shared memory) is free again on return.
template <int THREADS, class Op>
__device__ __forceinline__ float block_reduce(float v, float* red, Op op) {
    v = warp_reduce(v, op);
    if (THREADS == 32) return v;
    const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
    if (l == 0) red[w] = v;
    __syncthreads();
    float r = (l < THREADS / 32) ? red[l] : Op::ident();
    r       = warp_reduce(r, op);
    __syncthreads();
    return r;
}

__device__ __forceinline__ float4 load4(const float* p) { return __ldcs(reinterpret_cast<const float4*>(p)); }
__device__ __forceinline__ float4 load4(const __nv_bfloat16* p) {
    uint2 u = __ldcs(reinterpret_cast<const uint2*>(p));
    float2 a = __bfloat1622float2(*reinterpret_cast<__nv_bfloat162*>(&u.x));
    float2 b = __bfloat1622float2(*reinterpret_cast<__nv_bfloat162*>(&u.y));
    return make_float4(a.x, a.y, b.x, b.y);
}
// the same through the read-only cache path, for operands that many threads re-read (a broadcast row)
__device__ __forceinline__ float4 load4_cached(const float* p) { return __ldg(reinterpret_cast<const float4*>(p)); }
__device__ __forceinline__ float4 load4_cached(const __nv_bfloat16* p) {
    uint2 u = __ldg(reinterpret_cast<const uint2*>(p));
    float2 a = __bfloat1622float2(*reinterpret_cast<__nv_bfloat162*>(&u.x));
    float2 b = __bfloat1622float2(*reinterpret_cast<__nv_bfloat162*>(&u.y));
    return make_float4(a.x, a.y, b.x, b.y);
}
__device__ __forceinline__ void store4(float* p, float4 v) { __stcs(reinterpret_cast<float4*>(p), v); }
__device__ __forceinline__ void store4(__nv_bfloat16* p, float4 v) {
    uint2 u;
    u.x = pack_bf16x2(v.x, v.y);
    u.y = pack_bf16x2(v.z, v.w);
    __stcs(reinterpret_cast<uint2*>(p), u);
}

// One CTA per row (grid-stride over rows); a thread keeps NV float4 of the row in registers.
// Requires cols % 4 == 0, cols <= THREADS * NV * 4 and 16-byte (f32) / 8-byte (bf16) aligned rows.
template <int MODE, int THREADS, int NV, class TIn, class TOut>
__global__ void __launch_bounds__(THREADS, 1024 / THREADS) rows_in_regs_kernel(const TIn* __restrict__ x, const float* __restrict__ gamma,
                                                              TOut* __restrict__ y, int64_t rows, int cols, float eps) {
    __shared__ float red[32];
    const int nvec = cols >> 2;
    for (int64_t row = blockIdx.x; row < rows; row += gridDim.x) {
        const TIn* xr = x + row * cols;
        float4 v[NV];
#pragma unroll
        for (int i = 0; i < NV; ++i) {
            const int idx = i * THREADS + threadIdx.x;
            if (idx < nvec) v[i] = load4(xr + 4 * idx);
        }
        if (MODE == ROWS_SOFTMAX || MODE == ROWS_SOFTMAX_RMSNORM) {
            float mx = -CUDART_INF_F;
#pragma unroll
            for (int i = 0; i < NV; ++i)
                if (i * THREADS + threadIdx.x < nvec)
                    mx = fmaxf(mx, fmaxf(fmaxf(v[i].x, v[i].y), fmaxf(v[i].z, v[i].w)));
            mx        = block_reduce<THREADS>(mx, red, MaxOp());
            float sum = 0.f;
#pragma unroll
            for (int i = 0; i < NV; ++i)
                if (i * THREADS + threadIdx.x < nvec) {
                    v[i].x = expf(v[i].x - mx);
                    v[i].y = expf(v[i].y - mx);
                    v[i].z = expf(v[i].z - mx);
                    v[i].w = expf(v[i].w - mx);
                    sum += (v[i].x + v[i].y) + (v[i].z + v[i].w);
                }
            sum             = block_reduce<THREADS>(sum, red, SumOp());
            const float inv = 1.f / sum;
#pragma unroll
            for (int i = 0; i < NV; ++i) {
                v[i].x *= inv;
                v[i].y *= inv;
                v[i].z *= inv;
                v[i].w *= inv;
            }
        }
        if (MODE == ROWS_RMSNORM || MODE == ROWS_SOFTMAX_RMSNORM) {
            float ss = 0.f;
#pragma unroll
            for (int i = 0; i < NV; ++i)
                if (i * THREADS + threadIdx.x < nvec)
                    ss += (v[i].x * v[i].x + v[i].y * v[i].y) + (v[i].z * v[i].z + v[i].w * v[i].w);
            ss              = block_reduce<THREADS>(ss, red, SumOp());
            const float inv = rsqrtf(ss / float(cols) + eps);
#pragma unroll
            for (int i = 0; i < NV; ++i) {
                const int idx = i * THREADS + threadIdx.x;
                if (idx < nvec) {
                    const float4 g = __ldg(reinterpret_cast<const float4*>(gamma) + idx);
                    v[i].x *= inv * g.x;
                    v[i].y *= inv * g.y;
                    v[i].z *= inv * g.z;
                    v[i].w *= inv * g.w;
                }
            }
        }
        TOut* yr = y + row * cols;
#pragma unroll
        for (int i = 0; i < NV; ++i) {
            const int idx = i * THREADS + threadIdx.x;
            if (idx < nvec) store4(yr + 4 * idx, v[i]);
        }
    }
}

__device__ __forceinline__ float ldf(const float* p, int64_t i) { return p[i]; }
__device__ __forceinline__ float ldf(const __nv_bfloat16* p, int64_t i) { return __bfloat162float(p[i]); }
__device__ __forceinline__ void stf(float* p, int64_t i, float v) { p[i] = v; }
__device__ __forceinline__ void stf(__nv_bfloat16* p, int64_t i, float v) { p[i] = __float2bfloat16_rn(v); }

// Any length / alignment, inner == 1: one CTA per row, the row is re-read from L2 for each pass.
template <int MODE, class TIn, class TOut>
__global__ void __launch_bounds__(256) rows_generic_kernel(const TIn* __restrict__ x, const float* __restrict__ gamma,
                                                          TOut* __restrict__ y, int64_t rows, int64_t cols, float eps) {
    __shared__ float red[32];
    for (int64_t row = blockIdx.x; row < rows; row += gridDim.x) {
        const TIn* xr = x + row * cols;
        TOut* yr      = y + row * cols;
        float mx = 0.f, inv_sum = 1.f;
        if (MODE != ROWS_RMSNORM) {
            mx = -CUDART_INF_F;
            for (int64_t c = threadIdx.x; c < cols; c += 256) mx = fmaxf(mx, ldf(xr, c));
            mx      = block_reduce<256>(mx, red, MaxOp());
            float s = 0.f;
            for (int64_t c = threadIdx.x; c < cols; c += 256) s += expf(ldf(xr, c) - mx);
            inv_sum = 1.f / block_reduce<256>(s, red, SumOp());
        }
        float inv_rms = 1.f;
        if (MODE != ROWS_SOFTMAX) {
            float ss = 0.f;
            for (int64_t c = threadIdx.x; c < cols; c += 256) {
                float v = ldf(xr, c);
                if (MODE == ROWS_SOFTMAX_RMSNORM) v = expf(v - mx) * inv_sum;
                ss += v * v;
            }
            inv_rms = rsqrtf(block_reduce<256>(ss, red, SumOp()) / float(cols) + eps);
        }
        for (int64_t c = threadIdx.x; c < cols; c += 256) {
            float v = ldf(xr, c);
            if (MODE != ROWS_RMSNORM) v = expf(v - mx) * inv_sum;
            if (MODE != ROWS_SOFTMAX) v = v * inv_rms * gamma[c];
            stf(yr, c, v);
        }
    }
}

// softmax along the middle axis of [outer, len, inner] with inner > 1: one thread per (o, i) column, so that
// neighbouring threads read neighbouring addresses.
template <class TIn, class TOut>
__global__ void softmax_strided_kernel(const TIn* __restrict__ x, TOut* __restrict__ y, int64_t outer, int64_t len,
                                       int64_t inner) {
    const int64_t total = outer * inner;
    for (int64_t t = blockIdx.x * int64_t(blockDim.x) + threadIdx.x; t < total; t += int64_t(gridDim.x) * blockDim.x) {
        const int64_t o = t / inner, i = t % inner;
        const int64_t base = o * len * inner + i;
        float mx           = -CUDART_INF_F;
        for (int64_t a = 0; a < len; ++a) mx = fmaxf(mx, ldf(x, base + a * inner));
        float s = 0.f;
        for (int64_t a = 0; a < len; ++a) s += expf(ldf(x, base + a * inner) - mx);
        const float inv = 1.f / s;
        for (int64_t a = 0; a < len; ++a) stf(y, base + a * inner, expf(ldf(x, base + a * inner) - mx) * inv);
    }
}

// ---- reduce ------------------------------------------------------------------------------------
// What a fold does to an element before combining it: nothing, or an inlined elementwise producer (mimk_producer).
// `cell(o, i)` prepares what is constant along the folded axis of output cell (o, i): the second operand itself (y_mode 1),
// or the address its elements start from (y_mode 0 and 2), from where they lie at the same stride as x's (a * inner).
struct NoPre {
    struct Cell {};
    __device__ Cell cell(int64_t, int64_t) const { return Cell{}; }
    __device__ float operator()(float v, const Cell&, int64_t) const { return v; }
    __device__ float4 four(float4 v, const Cell&, int64_t) const { return v; }
};
// INNER / YMODE: the producer's first operator and the placement of its second operand fixed at compile time (the element
// loop then holds no dispatch and no dead addressing), or -1 for the run-time form that takes any of them at a few times
// the cost per element.
template <class TIn, int INNER, int YMODE>
struct MapPre {
    int inner_op, outer_op, y_mode;
    const TIn* y;
    int64_t len, inner;
    struct Cell {
        const TIn* yp;
        float yb;
    };
    static constexpr bool binary  = INNER < 0 || (INNER >= MIMK_OP_ADD && INNER <= MIMK_OP_SUBEXP);
    __device__ int mode() const { return YMODE >= 0 ? YMODE : y_mode; }
    __device__ bool per_element() const { return binary && (mode() == 0 || mode() == 2); }  // y read with every element
    __device__ Cell cell(int64_t o, int64_t i) const {
        Cell c{nullptr, 0.f};
        if (!binary) return c;
        if (mode() == 0) c.yp = y + o * len * inner + i;
        else if (mode() == 2) c.yp = y + i;
        else if (mode() == 1) c.yb = ldf(y, o * inner + i);
        return c;
    }
    __device__ float apply(float v, float b) const {
        float r;
        switch (INNER) {
            case MIMK_OP_ADD: r = v + b; break;
            case MIMK_OP_SUB: r = v - b; break;
            case MIMK_OP_MUL: r = v * b; break;
            case MIMK_OP_SUBEXP: r = expf(v - b); break;
            case MIMK_OP_RELU: r = fmaxf(0.f, v); break;
            case MIMK_OP_EXP: r = expf(v); break;
            case MIMK_OP_COPY: r = v; break;
            case MIMK_OP_SQUARE: r = v * v; break;
            case MIMK_OP_ABS: r = fabsf(v); break;
            default: r = apply_op(inner_op, v, b); break;
        }
        return outer_op == MIMK_OP_COPY ? r : apply_op(outer_op, r, 0.f);
    }
    // element at offset `off` (= a * inner) from the cell's start
    __device__ float operator()(float v, const Cell& c, int64_t off) const {
        const float b = per_element() ? ldf(c.yp, off) : c.yb;
        return apply(v, b);
    }
    // four consecutive elements of a row (inner == 1); the second operand's four come in one 128-bit load
    __device__ float4 four(float4 v, const Cell& c, int64_t off) const {
        float4 b = make_float4(c.yb, c.yb, c.yb, c.yb);
        if (per_element()) b = load4(c.yp + off);
        return make_float4(apply(v.x, b.x), apply(v.y, b.y), apply(v.z, b.z), apply(v.w, b.w));
    }
};
template <class Op, class TIn, class TOut, class Pre>
__global__ void __launch_bounds__(256) reduce_rows_kernel(const TIn* __restrict__ x, TOut* __restrict__ out, int64_t rows,
                                                         int64_t cols, int vec_ok, const Pre pre) {
    __shared__ float red[32];
    Op op;
    for (int64_t row = blockIdx.x; row < rows; row += gridDim.x) {
        const TIn* xr = x + row * cols;
        float acc     = Op::ident();
        const typename Pre::Cell cell = pre.cell(row, 0);
        if (vec_ok) {
            const int64_t nvec = cols >> 2;
            for (int64_t i = threadIdx.x; i < nvec; i += 256) {
                const float4 v = pre.four(load4(xr + 4 * i), cell, 4 * i);
                acc            = op(acc, op(op(v.x, v.y), op(v.z, v.w)));
            }
        } else {
            for (int64_t c = threadIdx.x; c < cols; c += 256) acc = op(acc, pre(ldf(xr, c), cell, c));
        }
        acc = block_reduce<256>(acc, red, op);
        if (threadIdx.x == 0) stf(out, row, acc);
    }
}

// inner > 1: thread per (o, i) column; blockIdx.y splits the reduced axis into `gridDim.y` slices whose partial
// results go to `partial` [slice, outer*inner] (or straight to `out` when there is a single slice).
template <class Op, class TIn, class TDst, class Pre>
__global__ void reduce_mid_kernel(const TIn* __restrict__ x, TDst* __restrict__ dst, int64_t outer, int64_t len,
                                  int64_t inner, int64_t slice_len, const Pre pre) {
    Op op;
    const int64_t total = outer * inner;
    const int64_t a0    = int64_t(blockIdx.y) * slice_len;
    const int64_t a1    = a0 + slice_len < len ? a0 + slice_len : len;
    for (int64_t t = blockIdx.x * int64_t(blockDim.x) + threadIdx.x; t < total; t += int64_t(gridDim.x) * blockDim.x) {
        const int64_t o = t / inner, i = t % inner;
        const TIn* p = x + o * len * inner + i;
        float acc    = Op::ident();
        const typename Pre::Cell cell = pre.cell(o, i);
        for (int64_t a = a0; a < a1; ++a) acc = op(acc, pre(ldf(p, a * inner), cell, a * inner));
        stf(dst, int64_t(blockIdx.y) * total + t, acc);
    }
}
template <class Op, class TOut>
__global__ void reduce_partials_kernel(const float* __restrict__ partial, TOut* __restrict__ out, int64_t total,
                                       int slices) {
    Op op;
    for (int64_t t = blockIdx.x * int64_t(blockDim.x) + threadIdx.x; t < total; t += int64_t(gridDim.x) * blockDim.x) {
        float acc = Op::ident();
        for (int s = 0; s < slices; ++s) acc = op(acc, partial[int64_t(s) * total + t]);
        stf(out, t, acc);
    }
}

// ---- elementwise -------------------------------------------------------------------------------
template <class TIn, class TOut>
__global__ void map_kernel(int op, const TIn* __restrict__ x, const TIn* __restrict__ y, TOut* __restrict__ out,
                           int64_t outer, int64_t len, int64_t inner, int y_mode) {
    const int64_t total = outer * len * inner;
    for (int64_t t = blockIdx.x * int64_t(blockDim.x) + threadIdx.x; t < total; t += int64_t(gridDim.x) * blockDim.x) {
        float b = 0.f;
        if (y_mode == 0) {
            b = ldf(y, t);
        } else if (y_mode == 1) {
            const int64_t o = t / (len * inner), i = t % inner;
            b = ldf(y, o * inner + i);
        } else if (y_mode == 2) {
            b = ldf(y, t % (len * inner));
        }
        stf(out, t, apply_op(op, ldf(x, t), b));
    }
}

// 128-bit form of map_kernel: four consecutive elements per thread. Requires 16-byte aligned x / y / out, a total
// divisible by 4, and a broadcast operand whose index is constant over the four elements (y_mode 1 with inner == 1 and
// len % 4 == 0) or runs with them (y_mode 0; y_mode 2 with (len * inner) % 4 == 0).
template <class TIn, class TOut>
__global__ void __launch_bounds__(256) map_vec4_kernel(int op, const TIn* __restrict__ x, const TIn* __restrict__ y,
                                                      TOut* __restrict__ out, int64_t total4, int64_t len, int64_t period4,
                                                      int y_mode) {
    for (int64_t t = blockIdx.x * int64_t(blockDim.x) + threadIdx.x; t < total4; t += int64_t(gridDim.x) * blockDim.x) {
        const float4 a = load4(x + 4 * t);
        float4 b       = make_float4(0.f, 0.f, 0.f, 0.f);
        if (y_mode == 0) {
            b = load4(y + 4 * t);
        } else if (y_mode == 1) {
            const float v = ldf(y, (4 * t) / len);
            b             = make_float4(v, v, v, v);
        } else if (y_mode == 2) {
            b = load4_cached(y + 4 * (t % period4));
        }
        float4 r;
        r.x = apply_op(op, a.x, b.x);
        r.y = apply_op(op, a.y, b.y);
        r.z = apply_op(op, a.z, b.z);
        r.w = apply_op(op, a.w, b.w);
        store4(out + 4 * t, r);
    }
}

int grid_for(int64_t work_items, int threads, int sm_count, int ctas_per_sm) {
    int64_t blocks = (work_items + threads - 1) / threads;
    int64_t cap    = int64_t(sm_count) * ctas_per_sm;
    if (blocks > cap) blocks = cap;
    if (blocks < 1) blocks = 1;
    return int(blocks);
}

template <int MODE, class TIn, class TOut>
int launch_rows(const TIn* x, const float* gamma, TOut* y, int64_t rows, int64_t cols, float eps, cudaStream_t s,
                const DeviceInfo& dev) {
    const bool in_align  = (reinterpret_cast<uintptr_t>(x) % (4 * sizeof(TIn))) == 0;
    const bool out_align = (reinterpret_cast<uintptr_t>(y) % (4 * sizeof(TOut))) == 0;
    const bool g_align   = MODE == ROWS_SOFTMAX || aligned16(gamma);
    const bool vec       = cols % 4 == 0 && in_align && out_align && g_align && cols <= 32768;
#define MIMK_ROWS_CASE(THREADS, NV, PER_SM)                                                                   \
    if (vec && cols <= THREADS * NV * 4) {                                                                    \
        int grid = int(rows < int64_t(dev.sm_count) * PER_SM ? rows : int64_t(dev.sm_count) * PER_SM);        \
        rows_in_regs_kernel<MODE, THREADS, NV, TIn, TOut><<<grid, THREADS, 0, s>>>(x, gamma, y, rows, int(cols), eps); \
        return launch_status();                                                                               \
    }
    MIMK_ROWS_CASE(32, 1, 32)
    MIMK_ROWS_CASE(32, 4, 32)
    MIMK_ROWS_CASE(128, 4, 16)
    MIMK_ROWS_CASE(256, 4, 8)
    MIMK_ROWS_CASE(256, 8, 4)
    MIMK_ROWS_CASE(512, 8, 2)
    MIMK_ROWS_CASE(1024, 8, 1)
#undef MIMK_ROWS_CASE
    int grid = int(rows < int64_t(dev.sm_count) * 8 ? rows : int64_t(dev.sm_count) * 8);
    rows_generic_kernel<MODE, TIn, TOut><<<grid, 256, 0, s>>>(x, gamma, y, rows, cols, eps);
    return launch_status();
}

template <int MODE>
int dispatch_rows(const void* x, const float* gamma, void* y, int in_dtype, int out_dtype, int64_t rows, int64_t cols,
                  float eps, cudaStream_t s, const DeviceInfo& dev) {
    if (in_dtype == MIMK_F32 && out_dtype == MIMK_F32)
        return launch_rows<MODE>(static_cast<const float*>(x), gamma, static_cast<float*>(y), rows, cols, eps, s, dev);
    if (in_dtype == MIMK_F32 && out_dtype == MIMK_BF16)
        return launch_rows<MODE>(static_cast<const float*>(x), gamma, static_cast<__nv_bfloat16*>(y), rows, cols, eps, s,
                                 dev);
    if (in_dtype == MIMK_BF16 && out_dtype == MIMK_BF16)
        return launch_rows<MODE>(static_cast<const __nv_bfloat16*>(x), gamma, static_cast<__nv_bfloat16*>(y), rows, cols,
                                 eps, s, dev);
    if (in_dtype == MIMK_BF16 && out_dtype == MIMK_F32)
        return launch_rows<MODE>(static_cast<const __nv_bfloat16*>(x), gamma, static_cast<float*>(y), rows, cols, eps, s,
                                 dev);
    return MIMK_E_DTYPE;
}

// How a fold of the middle axis of [outer, len, inner] is laid over the machine: `gx` CTAs over the outer * inner
// columns and, when those alone cannot fill it, `slices` pieces of `slice_len` along the reduced axis whose partial
// results a second kernel combines. The one plan behind mimk_reduce and mimk_reduce_static.
struct ReducePlan {
    int gx, slices;
    int64_t slice_len;
};
ReducePlan reduce_plan(int64_t outer, int64_t len, int64_t inner, int sm_count) {
    ReducePlan p;
    const int64_t total = outer * inner;
    p.gx                = grid_for(total, 256, sm_count, 8);
    p.slices            = 1;
    p.slice_len         = len;
    if (inner > 1 && int64_t(p.gx) < 2 * sm_count && len >= 256) {
        int64_t want = (4LL * sm_count + p.gx - 1) / p.gx;
        int64_t maxs = len / 64;
        int slices   = int(want < maxs ? want : maxs);
        if (slices < 1) slices = 1;
        if (slices > 1024) slices = 1024;
        if (slices > 1) {
            p.slice_len = (len + slices - 1) / slices;
            p.slices    = int((len + p.slice_len - 1) / p.slice_len);
        }
    }
    return p;
}

// `partials(n, &ptr)` supplies room for n floats when the plan splits the axis: the cached allocation for mimk_reduce,
// the array in the library image for mimk_reduce_static. Nothing there needs clearing: every partial the second kernel
// reads is written by the first kernel of the same call.
inline bool pre_vec_ok(const NoPre&) { return true; }
template <class TIn, int INNER, int YMODE>
bool pre_vec_ok(const MapPre<TIn, INNER, YMODE>& p) {  // the second operand's 128-bit loads need its rows aligned too
    return !MapPre<TIn, INNER, YMODE>::binary || (p.y_mode != 0 && p.y_mode != 2) || reinterpret_cast<uintptr_t>(p.y) % (4 * sizeof(TIn)) == 0;
}
template <class Op, class TIn, class TOut, class Partials, class Pre = NoPre>
int reduce_impl(const TIn* x, TOut* out, int64_t outer, int64_t len, int64_t inner, cudaStream_t s, int sm_count,
                Partials partials, Pre pre = Pre()) {
    if (inner == 1) {
        const int vec_ok = (len % 4 == 0) && (reinterpret_cast<uintptr_t>(x) % (4 * sizeof(TIn))) == 0 && pre_vec_ok(pre);
        int grid         = int(outer < int64_t(sm_count) * 8 ? outer : int64_t(sm_count) * 8);
        reduce_rows_kernel<Op><<<grid, 256, 0, s>>>(x, out, outer, len, vec_ok, pre);
        return launch_status();
    }
    const int64_t total = outer * inner;
    const int threads   = 256;
    const ReducePlan p  = reduce_plan(outer, len, inner, sm_count);
    if (p.slices == 1) {
        reduce_mid_kernel<Op><<<dim3(p.gx, 1), threads, 0, s>>>(x, out, outer, len, inner, len, pre);
        return launch_status();
    }
    float* scratch = nullptr;
    MIMK_TRY(partials(size_t(p.slices) * size_t(total), &scratch));
    reduce_mid_kernel<Op><<<dim3(p.gx, p.slices), threads, 0, s>>>(x, scratch, outer, len, inner, p.slice_len, pre);
    MIMK_TRY(launch_status());
    reduce_partials_kernel<Op><<<p.gx, threads, 0, s>>>(static_cast<const float*>(scratch), out, total, p.slices);
    return launch_status();
}

struct CachedPartials {
    cudaStream_t stream;
    int operator()(size_t n, float** out) const {
        void* p = nullptr;
        MIMK_TRY(get_scratch(n * sizeof(float), &p, stream));
        *out = static_cast<float*>(p);
        return MIMK_OK;
    }
};

// ---- reduce without any allocation ------------------------------------------------------------------

struct StaticSetup {
    bool ready = false;
    float* partials = nullptr;  // device address of g_static_partials on this device
    int sm_count = 0;
};
StaticSetup g_static_setup[64];
std::mutex g_static_mutex;

// Once per device, with that device current: resolve the array's device address. In host code the name
// `g_static_partials` is only a stand-in handle for the symbol, never a pointer a kernel may be given.
int static_setup(StaticSetup** out) {
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) {
        cudaGetLastError();
        return MIMK_E_NO_DEVICE;
    }
    std::lock_guard<std::mutex> lock(g_static_mutex);
    StaticSetup& st = g_static_setup[dev];
    if (!st.ready) {
        int major = 0, sms = 0;
        MIMK_CUDA_TRY(cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev));
        if (major != 10) return MIMK_E_NO_DEVICE;
        MIMK_CUDA_TRY(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
        float* ptr = nullptr;
        MIMK_CUDA_TRY(cudaGetSymbolAddress(reinterpret_cast<void**>(&ptr), g_static_partials));
        if (!ptr) return MIMK_E_CUDA;
        st.partials = ptr;
        st.sm_count = sms;
        st.ready    = true;
    }
    *out = &st;
    return MIMK_OK;
}

// The partials of a split plan live in the array of the library image; a plan that needs more is refused before any
// launch.
struct StaticPartials {
    float* base;
    int operator()(size_t n, float** out) const {
        if (n > STATIC_PARTIALS) return MIMK_E_WORKSPACE;
        *out = base;
        return MIMK_OK;
    }
};

}  // namespace
}  // namespace mimk

using namespace mimk;

extern "C" int mimk_reduce(const void* x, void* out, int dtype, int64_t outer, int64_t len, int64_t inner, int monoid,
                           void* stream) {
    if (outer < 0 || len < 0 || inner < 0) return MIMK_E_ARG;
    if (dtype != MIMK_F32 && dtype != MIMK_BF16) return MIMK_E_DTYPE;
    if (monoid < MIMK_SUM || monoid > MIMK_MIN) return MIMK_E_ARG;
    int st          = MIMK_OK;
    DeviceInfo* dev = device_info(&st);
    if (!dev) return st;
    if (outer * inner == 0) return MIMK_OK;
    if (!out || (len > 0 && !x)) return MIMK_E_ARG;  // len == 0: every cell is the monoid's identity, x is not read
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (dtype == MIMK_BF16) {  // bf16 in, f32 accumulation, bf16 out
        const __nv_bfloat16* xh = static_cast<const __nv_bfloat16*>(x);
        __nv_bfloat16* oh       = static_cast<__nv_bfloat16*>(out);
        switch (monoid) {
            case MIMK_SUM: return reduce_impl<SumOp>(xh, oh, outer, len, inner, s, dev->sm_count, CachedPartials{s});
            case MIMK_MAX: return reduce_impl<MaxOp>(xh, oh, outer, len, inner, s, dev->sm_count, CachedPartials{s});
            default: return reduce_impl<MinOp>(xh, oh, outer, len, inner, s, dev->sm_count, CachedPartials{s});
        }
    }
    const float* xf = static_cast<const float*>(x);
    float* of       = static_cast<float*>(out);
    switch (monoid) {
        case MIMK_SUM: return reduce_impl<SumOp>(xf, of, outer, len, inner, s, dev->sm_count, CachedPartials{s});
        case MIMK_MAX: return reduce_impl<MaxOp>(xf, of, outer, len, inner, s, dev->sm_count, CachedPartials{s});
        default: return reduce_impl<MinOp>(xf, of, outer, len, inner, s, dev->sm_count, CachedPartials{s});
    }
}

namespace mimk {
namespace {
template <class T, int INNER, int YMODE>
int reduce_fused_inner(const T* x, const mimk_producer& pr, T* out, int64_t outer, int64_t len, int64_t inner, int monoid,
                       cudaStream_t s, int sm_count) {
    const MapPre<T, INNER, YMODE> pre{pr.inner_op, pr.outer_op, pr.y_mode, static_cast<const T*>(pr.y), len, inner};
    switch (monoid) {
        case MIMK_SUM: return reduce_impl<SumOp>(x, out, outer, len, inner, s, sm_count, CachedPartials{s}, pre);
        case MIMK_MAX: return reduce_impl<MaxOp>(x, out, outer, len, inner, s, sm_count, CachedPartials{s}, pre);
        default: return reduce_impl<MinOp>(x, out, outer, len, inner, s, sm_count, CachedPartials{s}, pre);
    }
}
template <class T, int INNER>
int reduce_fused_binary(const T* x, const mimk_producer& pr, T* out, int64_t outer, int64_t len, int64_t inner, int monoid,
                        cudaStream_t s, int sm_count) {
    switch (pr.y_mode) {
        case 0: return reduce_fused_inner<T, INNER, 0>(x, pr, out, outer, len, inner, monoid, s, sm_count);
        case 1: return reduce_fused_inner<T, INNER, 1>(x, pr, out, outer, len, inner, monoid, s, sm_count);
        default: return reduce_fused_inner<T, INNER, 2>(x, pr, out, outer, len, inner, monoid, s, sm_count);
    }
}
template <class T>
int reduce_fused_typed(const T* x, const mimk_producer& pr, T* out, int64_t outer, int64_t len, int64_t inner, int monoid,
                       cudaStream_t s, int sm_count) {
#define MIMK_FUSED_BINARY(OP) case OP: return reduce_fused_binary<T, OP>(x, pr, out, outer, len, inner, monoid, s, sm_count);
#define MIMK_FUSED_UNARY(OP) case OP: return reduce_fused_inner<T, OP, 3>(x, pr, out, outer, len, inner, monoid, s, sm_count);
    switch (pr.inner_op) {
        MIMK_FUSED_BINARY(MIMK_OP_ADD)
        MIMK_FUSED_BINARY(MIMK_OP_SUB)
        MIMK_FUSED_BINARY(MIMK_OP_MUL)
        MIMK_FUSED_BINARY(MIMK_OP_SUBEXP)
        MIMK_FUSED_UNARY(MIMK_OP_RELU)
        MIMK_FUSED_UNARY(MIMK_OP_EXP)
        MIMK_FUSED_UNARY(MIMK_OP_COPY)
        MIMK_FUSED_UNARY(MIMK_OP_SQUARE)
        MIMK_FUSED_UNARY(MIMK_OP_ABS)
        default: return reduce_fused_inner<T, -1, -1>(x, pr, out, outer, len, inner, monoid, s, sm_count);
    }
#undef MIMK_FUSED_BINARY
#undef MIMK_FUSED_UNARY
}
}  // namespace
}  // namespace mimk

extern "C" int mimk_reduce_fused(const void* x, const mimk_producer* pre, void* out, int dtype, int64_t outer, int64_t len,
                                 int64_t inner, int monoid, void* stream) {
    using namespace mimk;
    if (!pre) return mimk_reduce(x, out, dtype, outer, len, inner, monoid, stream);
    if (outer < 0 || len < 0 || inner < 0) return MIMK_E_ARG;
    if (dtype != MIMK_F32 && dtype != MIMK_BF16) return MIMK_E_DTYPE;
    if (monoid < MIMK_SUM || monoid > MIMK_MIN) return MIMK_E_ARG;
    const bool binary = op_is_binary(pre->inner_op);
    if ((!binary && !op_is_unary(pre->inner_op)) || !op_is_unary(pre->outer_op)) return MIMK_E_ARG;
    if (binary ? (pre->y_mode < 0 || pre->y_mode > 2) : pre->y_mode != 3) return MIMK_E_ARG;
    int st          = MIMK_OK;
    DeviceInfo* dev = device_info(&st);
    if (!dev) return st;
    if (outer * inner == 0) return MIMK_OK;
    if (!out || (len > 0 && (!x || (binary && !pre->y)))) return MIMK_E_ARG;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (dtype == MIMK_BF16)
        return reduce_fused_typed(static_cast<const __nv_bfloat16*>(x), *pre, static_cast<__nv_bfloat16*>(out), outer, len, inner, monoid, s,
                                  dev->sm_count);
    return reduce_fused_typed(static_cast<const float*>(x), *pre, static_cast<float*>(out), outer, len, inner, monoid, s, dev->sm_count);
}

extern "C" int mimk_reduce_plan(int64_t outer, int64_t len, int64_t inner, int sm_count, int64_t* partial_floats) {
    if (outer < 0 || len < 0 || inner < 0 || sm_count < 1 || !partial_floats) return MIMK_E_ARG;
    *partial_floats = 0;
    if (outer * inner == 0 || inner == 1) return MIMK_OK;
    const ReducePlan p = reduce_plan(outer, len, inner, sm_count);
    if (p.slices > 1) *partial_floats = int64_t(p.slices) * outer * inner;
    return MIMK_OK;
}

extern "C" int mimk_reduce_static(const void* x, void* out, int dtype, int64_t outer, int64_t len, int64_t inner,
                                  int monoid, void* stream) {
    if (outer < 0 || len < 0 || inner < 0) return MIMK_E_ARG;
    if (dtype != MIMK_F32) return MIMK_E_DTYPE;
    if (monoid < MIMK_SUM || monoid > MIMK_MIN) return MIMK_E_ARG;
    StaticSetup* st = nullptr;
    MIMK_TRY(static_setup(&st));
    if (outer * inner == 0) return MIMK_OK;
    if (!out || (len > 0 && !x)) return MIMK_E_ARG;
    cudaStream_t s  = static_cast<cudaStream_t>(stream);
    const float* xf = static_cast<const float*>(x);
    float* of       = static_cast<float*>(out);
    switch (monoid) {
        case MIMK_SUM: return reduce_impl<SumOp>(xf, of, outer, len, inner, s, st->sm_count, StaticPartials{st->partials});
        case MIMK_MAX: return reduce_impl<MaxOp>(xf, of, outer, len, inner, s, st->sm_count, StaticPartials{st->partials});
        default: return reduce_impl<MinOp>(xf, of, outer, len, inner, s, st->sm_count, StaticPartials{st->partials});
    }
}

extern "C" int mimk_softmax(const void* x, void* y, int in_dtype, int out_dtype, int64_t outer, int64_t len,
                            int64_t inner, void* stream) {
    if (outer < 0 || len < 0 || inner < 0) return MIMK_E_ARG;
    if ((in_dtype != MIMK_F32 && in_dtype != MIMK_BF16) || (out_dtype != MIMK_F32 && out_dtype != MIMK_BF16))
        return MIMK_E_DTYPE;
    int st          = MIMK_OK;
    DeviceInfo* dev = device_info(&st);
    if (!dev) return st;
    if (outer * len * inner == 0) return MIMK_OK;
    if (!x || !y) return MIMK_E_ARG;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (inner == 1) return dispatch_rows<ROWS_SOFTMAX>(x, nullptr, y, in_dtype, out_dtype, outer, len, 0.f, s, *dev);
    int grid = grid_for(outer * inner, 128, dev->sm_count, 16);
    const bool in16 = in_dtype == MIMK_BF16, out16 = out_dtype == MIMK_BF16;
    const float* xf          = static_cast<const float*>(x);
    const __nv_bfloat16* xh  = static_cast<const __nv_bfloat16*>(x);
    if (!in16 && !out16) softmax_strided_kernel<<<grid, 128, 0, s>>>(xf, static_cast<float*>(y), outer, len, inner);
    else if (!in16) softmax_strided_kernel<<<grid, 128, 0, s>>>(xf, static_cast<__nv_bfloat16*>(y), outer, len, inner);
    else if (!out16) softmax_strided_kernel<<<grid, 128, 0, s>>>(xh, static_cast<float*>(y), outer, len, inner);
    else softmax_strided_kernel<<<grid, 128, 0, s>>>(xh, static_cast<__nv_bfloat16*>(y), outer, len, inner);
    return launch_status();
}

extern "C" int mimk_rmsnorm(const void* x, const void* gamma, void* y, int in_dtype, int out_dtype, int64_t rows,
                            int64_t cols, float eps, void* stream) {
    if (rows < 0 || cols < 0) return MIMK_E_ARG;
    int st          = MIMK_OK;
    DeviceInfo* dev = device_info(&st);
    if (!dev) return st;
    if (rows * cols == 0) return MIMK_OK;
    if (!x || !y || !gamma) return MIMK_E_ARG;
    return dispatch_rows<ROWS_RMSNORM>(x, static_cast<const float*>(gamma), y, in_dtype, out_dtype, rows, cols, eps,
                                       static_cast<cudaStream_t>(stream), *dev);
}

extern "C" int mimk_softmax_rmsnorm(const void* x, const void* gamma, void* y, int in_dtype, int out_dtype, int64_t rows,
                                    int64_t cols, float eps, void* stream) {
    if (rows < 0 || cols < 0) return MIMK_E_ARG;
    int st          = MIMK_OK;
    DeviceInfo* dev = device_info(&st);
    if (!dev) return st;
    if (rows * cols == 0) return MIMK_OK;
    if (!x || !y || !gamma) return MIMK_E_ARG;
    return dispatch_rows<ROWS_SOFTMAX_RMSNORM>(x, static_cast<const float*>(gamma), y, in_dtype, out_dtype, rows, cols, eps,
                                               static_cast<cudaStream_t>(stream), *dev);
}

namespace {
template <class TIn>
int map_impl(int op, const TIn* x, const TIn* y, void* out, int out_dtype, int64_t outer, int64_t len, int64_t inner, int y_mode,
             cudaStream_t s, const DeviceInfo& dev) {
    const int64_t total = outer * len * inner;
    const size_t in_al  = 4 * sizeof(TIn);  // four elements per access
    auto al             = [&](const void* p) { return (reinterpret_cast<uintptr_t>(p) % in_al) == 0; };
    const bool out_al   = (reinterpret_cast<uintptr_t>(out) % (out_dtype == MIMK_F32 ? 16 : 8)) == 0;
    const bool y_ok     = y_mode == 3 || (y_mode == 0 && al(y)) || (y_mode == 1 && inner == 1 && len % 4 == 0) ||
                      (y_mode == 2 && (len * inner) % 4 == 0 && al(y));
    if (total % 4 == 0 && al(x) && out_al && y_ok) {
        const int64_t total4 = total / 4, period4 = y_mode == 2 ? (len * inner) / 4 : 1;
        const int vgrid      = grid_for(total4, 256, dev.sm_count, 8);
        if (out_dtype == MIMK_F32)
            map_vec4_kernel<<<vgrid, 256, 0, s>>>(op, x, y, static_cast<float*>(out), total4, len, period4, y_mode);
        else
            map_vec4_kernel<<<vgrid, 256, 0, s>>>(op, x, y, static_cast<__nv_bfloat16*>(out), total4, len, period4, y_mode);
        return launch_status();
    }
    const int grid = grid_for(total, 256, dev.sm_count, 8);
    if (out_dtype == MIMK_F32) map_kernel<<<grid, 256, 0, s>>>(op, x, y, static_cast<float*>(out), outer, len, inner, y_mode);
    else map_kernel<<<grid, 256, 0, s>>>(op, x, y, static_cast<__nv_bfloat16*>(out), outer, len, inner, y_mode);
    return launch_status();
}
}  // namespace

extern "C" int mimk_map_t(int op, const void* x, const void* y, void* out, int in_dtype, int out_dtype, int64_t outer, int64_t len,
                          int64_t inner, int y_mode, void* stream) {
    if (outer < 0 || len < 0 || inner < 0 || y_mode < 0 || y_mode > 3) return MIMK_E_ARG;
    int op_inner = 0, op_outer = 0;
    if (!decode_op(op, &op_inner, &op_outer)) return MIMK_E_ARG;
    const bool unary = op_is_unary(op_inner), binary = op_is_binary(op_inner);
    if (binary && y_mode == 3) return MIMK_E_ARG;
    if ((in_dtype != MIMK_F32 && in_dtype != MIMK_BF16) || (out_dtype != MIMK_F32 && out_dtype != MIMK_BF16)) return MIMK_E_DTYPE;
    int st          = MIMK_OK;
    DeviceInfo* dev = device_info(&st);
    if (!dev) return st;
    if (outer * len * inner == 0) return MIMK_OK;
    if (!x || !out || (binary && !y)) return MIMK_E_ARG;
    if (unary) y_mode = 3;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (in_dtype == MIMK_F32)
        return map_impl(op, static_cast<const float*>(x), static_cast<const float*>(y), out, out_dtype, outer, len, inner, y_mode, s, *dev);
    return map_impl(op, static_cast<const __nv_bfloat16*>(x), static_cast<const __nv_bfloat16*>(y), out, out_dtype, outer, len, inner,
                    y_mode, s, *dev);
}

extern "C" int mimk_map(int op, const void* x, const void* y, void* out, int out_dtype, int64_t outer, int64_t len,
                        int64_t inner, int y_mode, void* stream) {
    return mimk_map_t(op, x, y, out, MIMK_F32, out_dtype, outer, len, inner, y_mode, stream);
}
