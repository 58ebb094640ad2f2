// CUDA-core contraction: the f32 path of the dot family and the landing place for bf16 shapes the tensor-core
// kernel does not take (extents that break TMA's 16-byte rules).
//
// Each output cell is folded in ascending k with one fused multiply-add per step -- the per-cell order every
// CPU nest of the reference keeps (MimIR src/mim/plug/btensor/btensor.mim:348) under its `fast` math mode,
// which permits contraction (src/mim/plug/ll/ll.cpp:55-68). Shapes are arbitrary (the reference tests
// 5x33 . (7x33)^T, lit/tensor/fc_exec.mim:36); out-of-range tile cells are predicated off.
#include "common.cuh"

namespace mimk {
namespace {

constexpr int TM = 64, TN = 64, TK = 16;

__device__ __forceinline__ float ld(const float* p, int64_t i) { return __ldg(p + i); }
__device__ __forceinline__ float ld(const __nv_bfloat16* p, int64_t i) { return __bfloat162float(p[i]); }
__device__ __forceinline__ void st(float* p, int64_t i, float v) { p[i] = v; }
__device__ __forceinline__ void st(__nv_bfloat16* p, int64_t i, float v) { p[i] = __float2bfloat16_rn(v); }

template <class TIn, class TOut>
__global__ void __launch_bounds__(256) gemm_simt_kernel(const TIn* __restrict__ A, const TIn* __restrict__ B,
                                                       TOut* __restrict__ C, int64_t M, int64_t N, int64_t K,
                                                       int64_t sa, int64_t sb, int64_t sc, int b_nk, int post,
                                                       const float* __restrict__ post_row,
                                                       const TOut* __restrict__ post_full) {
    __shared__ float As[TK][TM + 4];
    __shared__ float Bs[TK][TN + 4];
    const int64_t batch = blockIdx.z;
    A += batch * sa;
    B += batch * sb;
    C += batch * sc;
    if (post_full) post_full += batch * sc;
    const int64_t m0 = int64_t(blockIdx.y) * TM, n0 = int64_t(blockIdx.x) * TN;
    const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
    float acc[4][4] = {};
    // Each thread moves four A and four B elements per k-tile. The next tile's elements are fetched into registers before
    // the current tile is multiplied, so their global-memory latency overlaps the arithmetic (small problems have too few
    // CTAs to hide it by occupancy). The per-cell order of the fold is untouched: ascending k, one fma per step.
    float ra[4], rb[4];
    auto fetch = [&](int64_t k0) {
#pragma unroll
        for (int r = 0; r < 4; ++r) {
            const int i  = threadIdx.x + r * 256;
            const int kk = i % TK, mm = i / TK;
            const int64_t m = m0 + mm, k = k0 + kk;
            ra[r] = (m < M && k < K) ? ld(A, m * K + k) : 0.f;
            if (b_nk) {
                const int64_t n = n0 + mm;
                rb[r] = (n < N && k < K) ? ld(B, n * K + k) : 0.f;
            } else {
                const int nn = i % TN, kb = i / TN;
                const int64_t n = n0 + nn, kr = k0 + kb;
                rb[r] = (n < N && kr < K) ? ld(B, kr * N + n) : 0.f;
            }
        }
    };
    if (K > 0) fetch(0);
    for (int64_t k0 = 0; k0 < K; k0 += TK) {
#pragma unroll
        for (int r = 0; r < 4; ++r) {
            const int i = threadIdx.x + r * 256;
            As[i % TK][i / TK] = ra[r];  // A tile: TM x TK, read with k fastest (unit stride in memory)
            if (b_nk) Bs[i % TK][i / TK] = rb[r];
            else Bs[i / TN][i % TN] = rb[r];
        }
        __syncthreads();
        if (k0 + TK < K) fetch(k0 + TK);
#pragma unroll
        for (int kk = 0; kk < TK; ++kk) {
            float a[4], b[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) a[i] = As[kk][ty * 4 + i];
#pragma unroll
            for (int j = 0; j < 4; ++j) b[j] = Bs[kk][tx * 4 + j];
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int64_t m = m0 + ty * 4 + i;
        if (m >= M) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int64_t n = n0 + tx * 4 + j;
            if (n >= N) continue;
            const float row  = post_row ? post_row[n] : 0.f;
            const float full = post_full ? float(post_full[m * N + n]) : 0.f;
            st(C, m * N + n, apply_post(post, acc[i][j], row, full));
        }
    }
}

template <class TIn, class TOut>
int launch(const mimk_gemm_desc& d, cudaStream_t s) {
    dim3 grid((unsigned)((d.n + TN - 1) / TN), (unsigned)((d.m + TM - 1) / TM), (unsigned)d.batch);
    if (grid.y > 65535 || grid.z > 65535) return MIMK_E_UNSUPPORTED;
    gemm_simt_kernel<TIn, TOut><<<grid, 256, 0, s>>>(
        static_cast<const TIn*>(d.a), static_cast<const TIn*>(d.b), static_cast<TOut*>(d.c), d.m, d.n, d.k, d.stride_a,
        d.stride_b, d.stride_c, d.b_layout == MIMK_B_NK, d.post, static_cast<const float*>(d.post_row),
        static_cast<const TOut*>(d.post_full));
    return launch_status();
}

}  // namespace

int gemm_simt(const mimk_gemm_desc& d, cudaStream_t s) {
    if (d.in_dtype == MIMK_F32 && d.out_dtype == MIMK_F32) return launch<float, float>(d, s);
    if (d.in_dtype == MIMK_F32 && d.out_dtype == MIMK_BF16) return launch<float, __nv_bfloat16>(d, s);
    if (d.in_dtype == MIMK_BF16 && d.out_dtype == MIMK_F32) return launch<__nv_bfloat16, float>(d, s);
    if (d.in_dtype == MIMK_BF16 && d.out_dtype == MIMK_BF16) return launch<__nv_bfloat16, __nv_bfloat16>(d, s);
    return MIMK_E_DTYPE;
}

}  // namespace mimk
