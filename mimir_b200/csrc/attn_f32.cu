// f32 attention at sizes where one warp per query row is far too slow: the reference's own composition
// `softmax (q * transpose_2d k) * v` (MimIR lit/tensor/attn_exec.mim:20-22), stage by stage, on this library's kernels.
//   S = Q K^T      batched f32 contraction on the tensor cores (three TF32 products per term, f32-grade error)
//   S = mask(scale * S), in place
//   P = softmax rows of S, in place (one pass over HBM)
//   O = P V        batched f32 contraction
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

constexpr int64_t MAX_SCORE_BYTES = int64_t(2) << 30;  // score buffer per group of heads

}  // namespace

int attn_f32_composed_supported(const mimk_attn_desc& d) {
    if (d.dtype != MIMK_F32 || d.lse) return 0;
    if (d.seq_q < 128 || d.seq_k < 128 || d.seq_k % 4 != 0 || d.head_dim < 8 || d.head_dim % 4 != 0) return 0;
    if (d.seq_q >= (int64_t(1) << 31) || d.seq_k >= (int64_t(1) << 31)) return 0;
    if (d.seq_q * d.seq_k * d.head_dim < (int64_t(1) << 24)) return 0;  // small problems: the one-launch kernel
    if (d.seq_q * d.seq_k * 4 > MAX_SCORE_BYTES) return 0;              // one head's scores must fit the buffer
    if (d.causal && d.seq_q != d.seq_k) return 0;
    if (!aligned16(d.q) || !aligned16(d.k) || !aligned16(d.v) || !aligned16(d.o)) return 0;
    return 1;
}

int attn_f32_composed(const mimk_attn_desc& d, cudaStream_t s) {
    int st          = MIMK_OK;
    DeviceInfo* dev = device_info(&st);
    if (!dev) return st;
    const int64_t per_head = d.seq_q * d.seq_k;
    int64_t group = MAX_SCORE_BYTES / (per_head * 4);
    if (group > 16) group = 16;  // the f32 tensor-core contraction takes batches of up to 16
    if (group > d.batch_heads) group = d.batch_heads;
    void* scratch = nullptr;
    MIMK_TRY(get_aux_scratch(size_t(group * per_head) * 4, &scratch));
    float* S = static_cast<float*>(scratch);
    const float* q = static_cast<const float*>(d.q);
    const float* k = static_cast<const float*>(d.k);
    const float* v = static_cast<const float*>(d.v);
    float* o       = static_cast<float*>(d.o);
    for (int64_t h0 = 0; h0 < d.batch_heads; h0 += group) {
        const int64_t nb = d.batch_heads - h0 < group ? d.batch_heads - h0 : group;
        mimk_gemm_desc g = {};
        g.batch = nb, g.m = d.seq_q, g.n = d.seq_k, g.k = d.head_dim;
        g.a = q + h0 * d.seq_q * d.head_dim, g.b = k + h0 * d.seq_k * d.head_dim, g.c = S;
        g.stride_a = d.seq_q * d.head_dim, g.stride_b = d.seq_k * d.head_dim, g.stride_c = per_head;
        g.in_dtype = MIMK_F32, g.out_dtype = MIMK_F32, g.b_layout = MIMK_B_NK, g.post = MIMK_POST_ID;
        MIMK_TRY(mimk_gemm(&g, s));
        const long long total4 = (long long)(nb * per_head / 4);
        long long blocks = (total4 + 255) / 256;
        const long long cap = (long long)dev->sm_count * 16;
        if (blocks > cap) blocks = cap;
        scale_mask_kernel<<<unsigned(blocks), 256, 0, s>>>(S, total4, int(d.seq_k / 4), int(d.seq_q), d.scale, d.causal);
        MIMK_TRY(launch_status());
        MIMK_TRY(mimk_softmax(S, S, MIMK_F32, MIMK_F32, nb * d.seq_q, d.seq_k, 1, s));
        mimk_gemm_desc pv = {};
        pv.batch = nb, pv.m = d.seq_q, pv.n = d.head_dim, pv.k = d.seq_k;
        pv.a = S, pv.b = v + h0 * d.seq_k * d.head_dim, pv.c = o + h0 * d.seq_q * d.head_dim;
        pv.stride_a = per_head, pv.stride_b = d.seq_k * d.head_dim, pv.stride_c = d.seq_q * d.head_dim;
        pv.in_dtype = MIMK_F32, pv.out_dtype = MIMK_F32, pv.b_layout = MIMK_B_KN, pv.post = MIMK_POST_ID;
        MIMK_TRY(mimk_gemm(&pv, s));
    }
    return MIMK_OK;
}

}  // namespace mimk
