// CUDA-core attention forward: f32 tensors and every shape the tensor-core kernel does not take.
//
// The reference runs `softmax (q * transpose_2d k) * v` (MimIR lit/tensor/attn_exec.mim:20-22) as seven
// map_reduce_post ops with the full score matrix in memory. Here one warp owns one query row and streams the
// keys in chunks of 32 with a running maximum and sum, so no score matrix exists.
#include <math_constants.h>

#include "common.cuh"

namespace mimk {
namespace {

__device__ __forceinline__ float ld(const float* p, int64_t i) { return p[i]; }
__device__ __forceinline__ float ld(const __nv_bfloat16* p, int64_t i) { return __bfloat162float(p[i]); }
__device__ __forceinline__ void st(float* p, int64_t i, float v) { p[i] = v; }
__device__ __forceinline__ void st(__nv_bfloat16* p, int64_t i, float v) { p[i] = __float2bfloat16_rn(v); }

constexpr int WARPS = 4, MAX_D = 256;

template <class T>
__global__ void __launch_bounds__(WARPS * 32) attn_simt_kernel(const T* __restrict__ Q, const T* __restrict__ K,
                                                              const T* __restrict__ V, T* __restrict__ O,
                                                              float* __restrict__ lse, int64_t Sq, int64_t Sk, int D,
                                                              float scale, int causal) {
    __shared__ float qs[WARPS][MAX_D];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int64_t h = blockIdx.y;
    const int64_t i = int64_t(blockIdx.x) * WARPS + warp;
    if (i >= Sq) return;  // whole warp leaves together; no block-wide barrier below
    const T* q = Q + (h * Sq + i) * D;
    const T* k = K + h * Sk * D;
    const T* v = V + h * Sk * D;
    for (int d = lane; d < D; d += 32) qs[warp][d] = ld(q, d);
    __syncwarp();
    int64_t limit = causal ? i + 1 + (Sk - Sq) : Sk;
    if (limit > Sk) limit = Sk;
    float o_acc[MAX_D / 32];
#pragma unroll
    for (int t = 0; t < MAX_D / 32; ++t) o_acc[t] = 0.f;
    float m = -CUDART_INF_F, l = 0.f;
    for (int64_t j0 = 0; j0 < limit; j0 += 32) {
        const int64_t j = j0 + lane;
        float s         = -CUDART_INF_F;
        if (j < limit) {
            float acc      = 0.f;
            const T* kj    = k + j * D;
            for (int d = 0; d < D; ++d) acc = fmaf(qs[warp][d], ld(kj, d), acc);
            s = acc * scale;
        }
        const float m_new = fmaxf(m, warp_max(s));
        const float alpha = (m == -CUDART_INF_F) ? 0.f : expf(m - m_new);
        const float p     = (j < limit) ? expf(s - m_new) : 0.f;
        l                 = l * alpha + warp_sum(p);
#pragma unroll
        for (int t = 0; t < MAX_D / 32; ++t) o_acc[t] *= alpha;
        const int n = int(limit - j0 < 32 ? limit - j0 : 32);
        for (int jj = 0; jj < n; ++jj) {
            const float pj = __shfl_sync(0xffffffffu, p, jj);
            const T* vj    = v + (j0 + jj) * D;
#pragma unroll
            for (int t = 0; t < MAX_D / 32; ++t) {
                const int d = lane + 32 * t;
                if (d < D) o_acc[t] = fmaf(pj, ld(vj, d), o_acc[t]);
            }
        }
        m = m_new;
    }
    T* o            = O + (h * Sq + i) * D;
    const float inv = l > 0.f ? 1.f / l : 0.f;
#pragma unroll
    for (int t = 0; t < MAX_D / 32; ++t) {
        const int d = lane + 32 * t;
        if (d < D) st(o, d, o_acc[t] * inv);
    }
    if (lse && lane == 0) lse[h * Sq + i] = l > 0.f ? m + logf(l) : -CUDART_INF_F;
}

}  // namespace

int attn_simt(const mimk_attn_desc& d, cudaStream_t s) {
    if (d.head_dim > MAX_D) return MIMK_E_UNSUPPORTED;
    if (d.batch_heads > 65535) return MIMK_E_UNSUPPORTED;
    dim3 grid((unsigned)((d.seq_q + WARPS - 1) / WARPS), (unsigned)d.batch_heads);
    if (d.dtype == MIMK_F32)
        attn_simt_kernel<float><<<grid, WARPS * 32, 0, s>>>(static_cast<const float*>(d.q), static_cast<const float*>(d.k),
                                                           static_cast<const float*>(d.v), static_cast<float*>(d.o), d.lse,
                                                           d.seq_q, d.seq_k, int(d.head_dim), d.scale, d.causal);
    else if (d.dtype == MIMK_BF16)
        attn_simt_kernel<__nv_bfloat16><<<grid, WARPS * 32, 0, s>>>(
            static_cast<const __nv_bfloat16*>(d.q), static_cast<const __nv_bfloat16*>(d.k),
            static_cast<const __nv_bfloat16*>(d.v), static_cast<__nv_bfloat16*>(d.o), d.lse, d.seq_q, d.seq_k,
            int(d.head_dim), d.scale, d.causal);
    else
        return MIMK_E_DTYPE;
    return launch_status();
}

}  // namespace mimk
