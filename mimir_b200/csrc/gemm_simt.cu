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

// ---------------------------------------------------------------------------------------------------------------------
// Small f32 products: 32 x 32 tiles, the K extent staged in 128-wide chunks by asynchronous 16-byte copies.
//
// A product like 256^3 has 16 tiles of 64 x 64: sixteen CTAs on 148 SMs, each walking K in sixteen steps that every one
// pay a global-memory latency. Here the same product is 64 CTAs, and both chunks of a K <= 256 are in flight from the
// first instruction (two stages; longer K streams through them), so a CTA waits for memory once. The fold per cell is
// the one above -- ascending k, one fma per step -- so the two kernels agree bit for bit.
// Thread (tx, ty) of the 16 x 16 block owns rows ty, ty + 16 and, for B stored [N, K], columns tx, tx + 16 (both operands
// K-major in shared memory, read four k at a time: a quarter-warp reads one A address and eight B rows whose pitch of
// KC + 4 floats spreads them over all banks); for B stored [K, N], columns 2 tx, 2 tx + 1 (one 8-byte read per k).
// ---------------------------------------------------------------------------------------------------------------------
constexpr int ST = 32, KC = 128, KP = KC + 4, NP = ST + 4;

__device__ __forceinline__ void cp_async16(void* dst, const void* src, bool valid) {
    const uint32_t d = uint32_t(__cvta_generic_to_shared(dst));
    const int sz     = valid ? 16 : 0;  // 0: nothing is read, the 16 bytes are filled with zeros
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(d), "l"(src), "r"(sz) : "memory");
}

template <bool B_NK>
__global__ void __launch_bounds__(256) gemm_simt_small_kernel(const float* __restrict__ A, const float* __restrict__ B,
                                                             float* __restrict__ C, int64_t M, int64_t N, int64_t K,
                                                             int64_t sa, int64_t sb, int64_t sc, int post,
                                                             const float* __restrict__ post_row,
                                                             const float* __restrict__ post_full) {
    extern __shared__ __align__(16) float smem[];
    constexpr int A_FLOATS = ST * KP, B_FLOATS = B_NK ? ST * KP : KC * NP;
    const int64_t batch = blockIdx.z;
    A += batch * sa;
    B += batch * sb;
    C += batch * sc;
    if (post_full) post_full += batch * sc;
    const int64_t m0 = int64_t(blockIdx.y) * ST, n0 = int64_t(blockIdx.x) * ST;
    const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;

    auto stage = [&](int buf, int64_t k0) {
        float* As = smem + buf * (A_FLOATS + B_FLOATS);
        float* Bs = As + A_FLOATS;
#pragma unroll
        for (int r = 0; r < 4; ++r) {
            const int g = tid + r * 256, row = g >> 5, kq = (g & 31) * 4;  // 32 rows x 32 pieces of four k
            const bool ok = m0 + row < M && k0 + kq < K;
            cp_async16(As + row * KP + kq, ok ? A + (m0 + row) * K + k0 + kq : A, ok);
        }
        if (B_NK) {
#pragma unroll
            for (int r = 0; r < 4; ++r) {
                const int g = tid + r * 256, row = g >> 5, kq = (g & 31) * 4;
                const bool ok = n0 + row < N && k0 + kq < K;
                cp_async16(Bs + row * KP + kq, ok ? B + (n0 + row) * K + k0 + kq : B, ok);
            }
        } else {
#pragma unroll
            for (int r = 0; r < 4; ++r) {
                const int g = tid + r * 256, row = g >> 3, nq = (g & 7) * 4;  // 128 k-rows x 8 pieces of four columns
                const bool ok = k0 + row < K && n0 + nq < N;
                cp_async16(Bs + row * NP + nq, ok ? B + (k0 + row) * N + n0 + nq : B, ok);
            }
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };

    float acc[2][2] = {};
    const int64_t chunks = (K + KC - 1) / KC;
    if (chunks > 0) stage(0, 0);
    if (chunks > 1) stage(1, KC);
    for (int64_t c = 0; c < chunks; ++c) {
        if (c + 1 < chunks) asm volatile("cp.async.wait_group 1;" ::: "memory");
        else asm volatile("cp.async.wait_group 0;" ::: "memory");
        __syncthreads();
        const float* As = smem + int(c & 1) * (A_FLOATS + B_FLOATS);
        const float* Bs = As + A_FLOATS;
        const int kn    = int(K - c * KC < KC ? K - c * KC : KC);  // a multiple of 4
#pragma unroll 4
        for (int k = 0; k < kn; k += 4) {
            const float4 a0 = *reinterpret_cast<const float4*>(As + ty * KP + k);
            const float4 a1 = *reinterpret_cast<const float4*>(As + (ty + 16) * KP + k);
            const float av0[4] = {a0.x, a0.y, a0.z, a0.w}, av1[4] = {a1.x, a1.y, a1.z, a1.w};
            if (B_NK) {
                const float4 b0 = *reinterpret_cast<const float4*>(Bs + tx * KP + k);
                const float4 b1 = *reinterpret_cast<const float4*>(Bs + (tx + 16) * KP + k);
                const float bv0[4] = {b0.x, b0.y, b0.z, b0.w}, bv1[4] = {b1.x, b1.y, b1.z, b1.w};
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    acc[0][0] = fmaf(av0[q], bv0[q], acc[0][0]);
                    acc[0][1] = fmaf(av0[q], bv1[q], acc[0][1]);
                    acc[1][0] = fmaf(av1[q], bv0[q], acc[1][0]);
                    acc[1][1] = fmaf(av1[q], bv1[q], acc[1][1]);
                }
            } else {
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    const float2 b = *reinterpret_cast<const float2*>(Bs + (k + q) * NP + tx * 2);
                    acc[0][0]      = fmaf(av0[q], b.x, acc[0][0]);
                    acc[0][1]      = fmaf(av0[q], b.y, acc[0][1]);
                    acc[1][0]      = fmaf(av1[q], b.x, acc[1][0]);
                    acc[1][1]      = fmaf(av1[q], b.y, acc[1][1]);
                }
            }
        }
        __syncthreads();
        if (c + 2 < chunks) stage(int(c & 1), (c + 2) * KC);
    }
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const int64_t m = m0 + ty + 16 * i;
        if (m >= M) continue;
#pragma unroll
        for (int j = 0; j < 2; ++j) {
            const int64_t n = n0 + (B_NK ? tx + 16 * j : tx * 2 + j);
            if (n >= N) continue;
            const float row  = post_row ? post_row[n] : 0.f;
            const float full = post_full ? post_full[m * N + n] : 0.f;
            C[m * N + n]     = apply_post(post, acc[i][j], row, full);
        }
    }
}

// Worth it while the 64 x 64 tiling leaves most SMs without a tile; needs 16-byte pieces along the operands' rows.
bool small_tiles_apply(const mimk_gemm_desc& d) {
    if (d.in_dtype != MIMK_F32 || d.out_dtype != MIMK_F32 || d.k < 4 || d.k % 4 != 0) return false;
    const bool b_nk = d.b_layout == MIMK_B_NK;
    if (!b_nk && d.n % 4 != 0) return false;
    if (!aligned16(d.a) || !aligned16(d.b) || d.stride_a % 4 != 0 || d.stride_b % 4 != 0) return false;
    const int64_t big = ((d.m + TM - 1) / TM) * ((d.n + TN - 1) / TN) * d.batch;
    return big < 2 * 148 && (d.m + ST - 1) / ST <= 65535 && d.batch <= 65535;
}

int launch_small(const mimk_gemm_desc& d, cudaStream_t s) {
    const bool b_nk = d.b_layout == MIMK_B_NK;
    const int smem  = 2 * (ST * KP + (b_nk ? ST * KP : KC * NP)) * int(sizeof(float));
    auto kern       = b_nk ? gemm_simt_small_kernel<true> : gemm_simt_small_kernel<false>;
    static bool configured[2][64] = {};  // per instance and device: the attribute is a per-device setting
    int dev = 0;
    MIMK_CUDA_TRY(cudaGetDevice(&dev));
    if (!configured[b_nk][dev & 63]) {
        MIMK_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
        configured[b_nk][dev & 63] = true;
    }
    dim3 grid((unsigned)((d.n + ST - 1) / ST), (unsigned)((d.m + ST - 1) / ST), (unsigned)d.batch);
    kern<<<grid, 256, smem, s>>>(static_cast<const float*>(d.a), static_cast<const float*>(d.b), static_cast<float*>(d.c),
                                 d.m, d.n, d.k, d.stride_a, d.stride_b, d.stride_c, d.post,
                                 static_cast<const float*>(d.post_row), static_cast<const float*>(d.post_full));
    return launch_status();
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

// Below 2^27 multiply-adds the small-tile kernel is also faster than three TF32 passes over re-written operands (three
// launches): 256^3 6.3 against 14.0 us, 384^3 8.6 against 18.1, 512^3 17.2 against 18.5 (CUDA-graph replays, warm).
int gemm_simt_preferred(const mimk_gemm_desc& d) {
    return small_tiles_apply(d) && d.m * d.n * d.k < (int64_t(1) << 27) / (d.batch > 0 ? d.batch : 1);
}

int gemm_simt(const mimk_gemm_desc& d, cudaStream_t s) {
    if (small_tiles_apply(d)) return launch_small(d, s);
    if (d.in_dtype == MIMK_F32 && d.out_dtype == MIMK_F32) return launch<float, float>(d, s);
    if (d.in_dtype == MIMK_F32 && d.out_dtype == MIMK_BF16) return launch<float, __nv_bfloat16>(d, s);
    if (d.in_dtype == MIMK_BF16 && d.out_dtype == MIMK_F32) return launch<__nv_bfloat16, float>(d, s);
    if (d.in_dtype == MIMK_BF16 && d.out_dtype == MIMK_BF16) return launch<__nv_bfloat16, __nv_bfloat16>(d, s);
    return MIMK_E_DTYPE;
}

}  // namespace mimk
