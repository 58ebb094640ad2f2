// Attention at sizes where one warp per query row is far too slow and the fused tensor-core kernels do not apply (f32;
// bf16 with a head_dim other than 64 / 128): the reference's own composition `softmax (q * transpose_2d k) * v`
// (MimIR lit/tensor/attn_exec.mim:20-22), stage by stage, on this library's kernels.
//   S = Q K^T      batched contraction on the tensor cores, f32 result (f32 operands: three TF32 products per term)
//   S = mask(scale * S), in place
//   P = softmax rows of S (f32 in place; bf16 operands: P stored as bf16 beside S), one pass over HBM
//   O = P V        batched contraction
// The score matrix is materialised, as in the reference (per group of up to 16 heads, in a cached buffer), so this path
// trades HBM traffic for tensor-core throughput; the fused bf16 kernels never materialise it.
#include <cstdlib>

#include "common.cuh"

namespace mimk {
namespace {

// x = scale * x, and -inf above the diagonal of each [rows_per_head x cols] score matrix when `causal`
__global__ void scale_mask_kernel(float* __restrict__ s, long long total4, int cols4, int rows_per_head, float scale, int causal) {
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total4; i += (long long)gridDim.x * blockDim.x) {
        float4 v        = reinterpret_cast<float4*>(s)[i];
        const int c0    = int(i % cols4) * 4;
        const int row   = int((i / cols4) % rows_per_head);
        const float inf = __int_as_float(0xff800000);
        v.x = (causal && c0 + 0 > row) ? inf : v.x * scale;
        v.y = (causal && c0 + 1 > row) ? inf : v.y * scale;
        v.z = (causal && c0 + 2 > row) ? inf : v.z * scale;
        v.w = (causal && c0 + 3 > row) ? inf : v.w * scale;
        reinterpret_cast<float4*>(s)[i] = v;
    }
}

// P = softmax rows of mask(scale * S) in one pass for rows of up to 8192 scores: a CTA per row, the row in registers.
// TOut = float: P over S in place; __nv_bfloat16: P beside S.
constexpr int SM_THREADS = 256, SM_NV = 8;
__device__ __forceinline__ float block_max(float v, float* red) {
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
    __syncthreads();
    float r = red[0];
    for (int w = 1; w < SM_THREADS / 32; ++w) r = fmaxf(r, red[w]);
    __syncthreads();
    return r;
}
__device__ __forceinline__ float block_sum(float v, float* red) {
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
    __syncthreads();
    float r = 0.f;
    for (int w = 0; w < SM_THREADS / 32; ++w) r += red[w];
    __syncthreads();
    return r;
}
template <class TOut>
__global__ void __launch_bounds__(SM_THREADS) scaled_masked_softmax_kernel(const float* __restrict__ s, TOut* __restrict__ p,
                                                                           long long rows, int cols, int rows_per_head, float scale,
                                                                           int causal) {
    __shared__ float red[SM_THREADS / 32];
    const int nvec  = cols >> 2;
    const float inf = __int_as_float(0xff800000);
    for (long long row = blockIdx.x; row < rows; row += gridDim.x) {
        const int qi        = int(row % rows_per_head);
        const int visible   = causal ? (qi + 1 < cols ? qi + 1 : cols) : cols;  // keys [0, visible) take part
        const float4* sr    = reinterpret_cast<const float4*>(s + row * (long long)cols);
        float4 v[SM_NV];
        float mx = inf;
#pragma unroll
        for (int i = 0; i < SM_NV; ++i) {
            const int idx = i * SM_THREADS + threadIdx.x;
            if (idx < nvec) {
                float4 t    = sr[idx];
                const int c = idx * 4;
                t.x = c + 0 < visible ? t.x * scale : inf;
                t.y = c + 1 < visible ? t.y * scale : inf;
                t.z = c + 2 < visible ? t.z * scale : inf;
                t.w = c + 3 < visible ? t.w * scale : inf;
                v[i] = t;
                mx   = fmaxf(mx, fmaxf(fmaxf(t.x, t.y), fmaxf(t.z, t.w)));
            }
        }
        mx        = block_max(mx, red);
        float sum = 0.f;
#pragma unroll
        for (int i = 0; i < SM_NV; ++i)
            if (i * SM_THREADS + threadIdx.x < nvec) {
                v[i].x = expf(v[i].x - mx), v[i].y = expf(v[i].y - mx), v[i].z = expf(v[i].z - mx), v[i].w = expf(v[i].w - mx);
                sum += (v[i].x + v[i].y) + (v[i].z + v[i].w);
            }
        const float inv = 1.f / block_sum(sum, red);
        TOut* pr = p + row * (long long)cols;
#pragma unroll
        for (int i = 0; i < SM_NV; ++i) {
            const int idx = i * SM_THREADS + threadIdx.x;
            if (idx < nvec) {
                if (sizeof(TOut) == 4) {
                    reinterpret_cast<float4*>(pr)[idx] = make_float4(v[i].x * inv, v[i].y * inv, v[i].z * inv, v[i].w * inv);
                } else {
                    uint2 u;
                    u.x = pack_bf16x2(v[i].x * inv, v[i].y * inv);
                    u.y = pack_bf16x2(v[i].z * inv, v[i].w * inv);
                    reinterpret_cast<uint2*>(pr)[idx] = u;
                }
            }
        }
    }
}

constexpr int64_t MAX_SCORE_BYTES = int64_t(2) << 30;  // score buffer per group of heads

}  // namespace

int attn_composed_supported(const mimk_attn_desc& d) {
    if ((d.dtype != MIMK_F32 && d.dtype != MIMK_BF16) || d.lse) return 0;
    const int64_t al = d.dtype == MIMK_F32 ? 4 : 8;  // 16-byte rows for the contraction kernels
    if (d.seq_q < 128 || d.seq_k < 128 || d.seq_k % al != 0 || d.head_dim < 8 || d.head_dim % al != 0) return 0;
    if (d.seq_q >= (int64_t(1) << 31) || d.seq_k >= (int64_t(1) << 31)) return 0;
    if (d.seq_q * d.seq_k * d.head_dim < (int64_t(1) << 24)) return 0;  // small problems: the one-launch kernel
    if (d.seq_q * d.seq_k * 6 > MAX_SCORE_BYTES) return 0;              // one head's scores (and bf16 P) must fit the buffer
    if (d.causal && d.seq_q != d.seq_k) return 0;
    if (!aligned16(d.q) || !aligned16(d.k) || !aligned16(d.v) || !aligned16(d.o)) return 0;
    return 1;
}

int attn_composed(const mimk_attn_desc& d, cudaStream_t s) {
    int st          = MIMK_OK;
    DeviceInfo* dev = device_info(&st);
    if (!dev) return st;
    const bool half        = d.dtype == MIMK_BF16;
    const int64_t es       = half ? 2 : 4;
    const int64_t per_head = d.seq_q * d.seq_k;
    int64_t group = MAX_SCORE_BYTES / (per_head * (half ? 6 : 4));
    if (group > 16) group = 16;  // the f32 tensor-core contraction takes batches of up to 16
    if (group > d.batch_heads) group = d.batch_heads;
    void* scratch = nullptr;
    MIMK_TRY(get_aux_scratch(size_t(group * per_head) * (half ? 6 : 4), &scratch, s));
    float* S = static_cast<float*>(scratch);
    void* P  = half ? static_cast<void*>(S + group * per_head) : static_cast<void*>(S);  // bf16 P beside S, f32 P over S
    const uint8_t* q = static_cast<const uint8_t*>(d.q);
    const uint8_t* k = static_cast<const uint8_t*>(d.k);
    const uint8_t* v = static_cast<const uint8_t*>(d.v);
    uint8_t* o       = static_cast<uint8_t*>(d.o);
    for (int64_t h0 = 0; h0 < d.batch_heads; h0 += group) {
        const int64_t nb = d.batch_heads - h0 < group ? d.batch_heads - h0 : group;
        mimk_gemm_desc g = {};
        g.batch = nb, g.m = d.seq_q, g.n = d.seq_k, g.k = d.head_dim;
        g.a = q + h0 * d.seq_q * d.head_dim * es, g.b = k + h0 * d.seq_k * d.head_dim * es, g.c = S;
        g.stride_a = d.seq_q * d.head_dim, g.stride_b = d.seq_k * d.head_dim, g.stride_c = per_head;
        g.in_dtype = d.dtype, g.out_dtype = MIMK_F32, g.b_layout = MIMK_B_NK, g.post = MIMK_POST_ID;
        MIMK_TRY(mimk_gemm(&g, s));
        if (d.seq_k <= SM_THREADS * SM_NV * 4) {
            const long long rows = nb * d.seq_q, cap = (long long)dev->sm_count * 8;
            const unsigned grid  = unsigned(rows < cap ? rows : cap);
            if (half)
                scaled_masked_softmax_kernel<__nv_bfloat16><<<grid, SM_THREADS, 0, s>>>(S, static_cast<__nv_bfloat16*>(P), rows,
                                                                                        int(d.seq_k), int(d.seq_q), d.scale, d.causal);
            else
                scaled_masked_softmax_kernel<float><<<grid, SM_THREADS, 0, s>>>(S, static_cast<float*>(P), rows, int(d.seq_k),
                                                                                 int(d.seq_q), d.scale, d.causal);
            MIMK_TRY(launch_status());
        } else {  // longer rows: scale and mask in place, then the library's row softmax
            const long long total4 = (long long)(nb * per_head / 4);
            long long blocks = (total4 + 255) / 256;
            const long long cap = (long long)dev->sm_count * 16;
            if (blocks > cap) blocks = cap;
            scale_mask_kernel<<<unsigned(blocks), 256, 0, s>>>(S, total4, int(d.seq_k / 4), int(d.seq_q), d.scale, d.causal);
            MIMK_TRY(launch_status());
            MIMK_TRY(mimk_softmax(S, P, MIMK_F32, d.dtype, nb * d.seq_q, d.seq_k, 1, s));
        }
        mimk_gemm_desc pv = {};
        pv.batch = nb, pv.m = d.seq_q, pv.n = d.head_dim, pv.k = d.seq_k;
        pv.a = P, pv.b = v + h0 * d.seq_k * d.head_dim * es, pv.c = o + h0 * d.seq_q * d.head_dim * es;
        pv.stride_a = per_head, pv.stride_b = d.seq_k * d.head_dim, pv.stride_c = d.seq_q * d.head_dim;
        pv.in_dtype = d.dtype, pv.out_dtype = d.dtype, pv.b_layout = MIMK_B_KN, pv.post = MIMK_POST_ID;
        MIMK_TRY(mimk_gemm(&pv, s));
    }
    return MIMK_OK;
}

}  // namespace mimk
