// f32 contraction on the tensor cores with f32-grade accuracy: three TF32 products per term ("3xTF32").
//
// Every tensor program the reference can lower today is f32 (its Ring has one element type and the LLVM emitter knows
// half / float / double only, MimIR src/mim/plug/ll/ll.cpp:139-145), so the f32 `product_2d` is the path existing
// programs take. A TF32 multiply keeps 10 mantissa bits, far from the 1e-5 the f32 path is held to; splitting each
// operand into a TF32-representable head and tail, a = a_hi + a_lo, and accumulating
//     a_hi * b_hi + a_lo * b_hi + a_hi * b_lo          (the a_lo * b_lo term is below 2^-22 relative)
// in the f32 accumulators of tensor memory restores about 21 mantissa bits per product.
//
//   split kernel   one pass over A and B: hi = tf32(x), lo = tf32(x - hi), both written K-major (B stored [K,N] is
//                  transposed on the way) into scratch
//   gemm kernel    the structure of gemm_tc.cu with 4-byte elements: 128 x 128 tile, 32-wide k-blocks (one 128-byte
//                  swizzle row), three stages of {A_hi, A_lo, B_hi, B_lo}, tcgen05.mma kind::tf32 (M128 N128 K8), three
//                  instructions per k-step, the same epilogue (`post` slot) as gemm_tc.cu.
// The tensor core does not round its accumulator updates to nearest, so a long K leaves a bias that grows with the number
// of updates (measured: 2e-6 of max|C| at K = 256, 9e-6 at K = 1024). K is therefore cut into chunks of 256: each chunk
// is accumulated in tensor memory from zero (two buffers, ping-pong) and the epilogue warps add the finished chunks in
// registers with ordinary round-to-nearest f32 adds, which keeps the error near 2e-6 for any K.
#include "common.cuh"
#include "sm100.cuh"

namespace mimk {

using namespace sm100;

namespace {

constexpr int BM = 128, BN = 128, BK = 32, STAGES = 3;
constexpr int CHUNK_KB = 8;  // k-blocks per tensor-memory accumulation chunk (256 k)
constexpr int A_BYTES = BM * BK * 4;  // 16 KiB
constexpr int B_BYTES = BN * BK * 4;  // 16 KiB
constexpr int STAGE_BYTES = 2 * A_BYTES + 2 * B_BYTES;
constexpr int NUM_THREADS = 192;
constexpr int GROUP_M = 16;

struct Bars {
    uint64_t full[STAGES];
    uint64_t empty[STAGES];
    uint64_t acc_full[2];
    uint64_t acc_empty[2];
    uint32_t tmem_base;
    int abort_flag;
};
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 + 256;

struct Params {
    int64_t M, N, K;
    void* C;
    const float* post_row;
    const void* post_full;
    int post;
    int* status;
    const float* A0;  // the operands as the caller gave them, for the scalar fold of non-finite cells
    const float* B0;
    int b_nk;
};

__device__ __forceinline__ float to_tf32(float x) {
    uint32_t y;
    asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(y) : "f"(x));
    return __uint_as_float(y);
}

// The tail of the split. A head that is not finite (v is inf or NaN, or a finite v that rounds up past the largest TF32
// value) has no tail: inf - inf would put a NaN where the scalar fold has an inf. Cells whose products involve such an
// operand come out of the tensor cores non-finite either way (inf * 0 from a zero tail is NaN); the epilogue recomputes
// exactly those cells with the scalar fold.
__device__ __forceinline__ float tail_of(float v, float h) { return isfinite(h) ? to_tf32(v - h) : 0.f; }

// hi / lo split of a row-major [rows, cols] matrix, same layout out.
__global__ void split_kernel(const float* __restrict__ x, float* __restrict__ hi, float* __restrict__ lo, int64_t n) {
    for (int64_t i = blockIdx.x * int64_t(blockDim.x) + threadIdx.x; i < n; i += int64_t(gridDim.x) * blockDim.x) {
        const float v = x[i];
        const float h = to_tf32(v);
        hi[i]         = h;
        lo[i]         = tail_of(v, h);
    }
}
// The same with the copies' rows padded to `kp` >= cols elements (zeros in the pad): a K that is not a multiple of 4 gets
// the 16-byte row pitch the bulk loads need, and the zero columns add nothing to the products.
__global__ void split_pad_kernel(const float* __restrict__ x, float* __restrict__ hi, float* __restrict__ lo, int64_t rows,
                                 int64_t cols, int64_t kp) {
    const int64_t n = rows * kp;
    for (int64_t i = blockIdx.x * int64_t(blockDim.x) + threadIdx.x; i < n; i += int64_t(gridDim.x) * blockDim.x) {
        const int64_t r = i / kp, c = i % kp;
        const float v = c < cols ? x[r * cols + c] : 0.f;
        const float h = to_tf32(v);
        hi[i]         = h;
        lo[i]         = tail_of(v, h);
    }
}
// The same for B stored [K, N]: written transposed as [N, K] (K contiguous) through a 32 x 32 shared-memory tile.
__global__ void split_transpose_kernel(const float* __restrict__ x, float* __restrict__ hi, float* __restrict__ lo, int64_t K,
                                       int64_t N, int64_t kp) {
    __shared__ float tile[32][33];
    const int64_t k0 = int64_t(blockIdx.y) * 32, n0 = int64_t(blockIdx.x) * 32;
    for (int r = threadIdx.y; r < 32; r += 8) {
        const int64_t k = k0 + r, n = n0 + threadIdx.x;
        tile[r][threadIdx.x] = (k < K && n < N) ? x[k * N + n] : 0.f;
    }
    __syncthreads();
    for (int r = threadIdx.y; r < 32; r += 8) {
        const int64_t n = n0 + r, k = k0 + threadIdx.x;
        if (n < N && k < kp) {  // columns K..kp of the copy are zeros (the tile holds 0 there)
            const float v  = tile[threadIdx.x][r];
            const float h  = to_tf32(v);
            hi[n * kp + k] = h;
            lo[n * kp + k] = tail_of(v, h);
        }
    }
}

__device__ __forceinline__ void mma_tf32_ss(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                            uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// kind::tf32 instruction descriptor: D format f32 (1 at bit 4), A and B format TF32 (2 at bits 7 and 10), both K-major.
__device__ __forceinline__ uint32_t idesc_tf32(int m, int n) {
    return (1u << 4) | (2u << 7) | (2u << 10) | (uint32_t(n >> 3) << 17) | (uint32_t(m >> 4) << 24);
}

__device__ __forceinline__ void tile_coords(int64_t tile, int64_t tiles_m, int64_t tiles_n, int64_t& tm, int64_t& tn) {
    const int64_t per_group = GROUP_M * tiles_n;
    const int64_t group     = tile / per_group;
    const int64_t first_m   = group * GROUP_M;
    const int64_t gsize     = (tiles_m - first_m) < GROUP_M ? (tiles_m - first_m) : GROUP_M;
    const int64_t in_group  = tile % per_group;
    tm                      = first_m + in_group % gsize;
    tn                      = in_group / gsize;
}

template <class TOut>
__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm_f32_tc_kernel(const __grid_constant__ CUtensorMap tmAh, const __grid_constant__ CUtensorMap tmAl,
                   const __grid_constant__ CUtensorMap tmBh, const __grid_constant__ CUtensorMap tmBl, const Params p) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw_addr  = smem_u32(smem_raw);
    const uint32_t tile_base = (raw_addr + 1023u) & ~1023u;
    Bars* bars               = reinterpret_cast<Bars*>(smem_raw + (tile_base - raw_addr) + STAGES * STAGE_BYTES);
    volatile int* abort_flag = &bars->abort_flag;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int64_t tiles_m = (p.M + BM - 1) / BM, tiles_n = (p.N + BN - 1) / BN;
    const int64_t num_tiles = tiles_m * tiles_n;
    const int num_kb        = int((p.K + BK - 1) / BK);

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(smem_u32(&bars->full[s]), 1);
            mbar_init(smem_u32(&bars->empty[s]), 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(smem_u32(&bars->acc_full[b]), 1);
            mbar_init(smem_u32(&bars->acc_empty[b]), 128);
        }
        bars->abort_flag = 0;
        fence_barrier_init();
        tma_prefetch_desc(&tmAh);
        tma_prefetch_desc(&tmAl);
        tma_prefetch_desc(&tmBh);
        tma_prefetch_desc(&tmBl);
    }
    if (warp == 1) {
        tmem_alloc(smem_u32(&bars->tmem_base), 256);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(&bars->tmem_base);

    if (warp == 0) {
        if (lane == 0) {
            uint32_t stage = 0, phase = 0;
            bool ok = true;
            for (int64_t tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
                int64_t tm, tn;
                tile_coords(tile, tiles_m, tiles_n, tm, tn);
                const int m0 = int(tm * BM), n0 = int(tn * BN);
                for (int kb = 0; kb < num_kb; ++kb) {
                    if (!(ok = mbar_wait(smem_u32(&bars->empty[stage]), phase ^ 1u, abort_flag))) break;
                    const uint32_t full = smem_u32(&bars->full[stage]);
                    const uint32_t s0   = tile_base + stage * STAGE_BYTES;
                    mbar_expect_tx(full, STAGE_BYTES);
                    tma_load_2d(s0, &tmAh, kb * BK, m0, full);
                    tma_load_2d(s0 + A_BYTES, &tmAl, kb * BK, m0, full);
                    tma_load_2d(s0 + 2 * A_BYTES, &tmBh, kb * BK, n0, full);
                    tma_load_2d(s0 + 2 * A_BYTES + B_BYTES, &tmBl, kb * BK, n0, full);
                    if (++stage == STAGES) {
                        stage = 0;
                        phase ^= 1u;
                    }
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            const uint32_t idesc = idesc_tf32(BM, BN);
            uint32_t stage = 0, phase = 0, acc = 0, acc_phase = 0;
            bool ok = true;
            for (int64_t tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
                for (int kb0 = 0; kb0 < num_kb && ok; kb0 += CHUNK_KB) {
                    // one chunk: a fresh accumulator buffer, handed to the epilogue warps when the chunk is complete
                    if (!(ok = mbar_wait(smem_u32(&bars->acc_empty[acc]), acc_phase ^ 1u, abort_flag))) break;
                    tc_fence_after();
                    const uint32_t d0 = tmem_base + acc * BN;
                    const int kb1     = kb0 + CHUNK_KB < num_kb ? kb0 + CHUNK_KB : num_kb;
                    for (int kb = kb0; kb < kb1; ++kb) {
                        if (!(ok = mbar_wait(smem_u32(&bars->full[stage]), phase, abort_flag))) break;
                        tc_fence_after();
                        const uint32_t s0 = tile_base + stage * STAGE_BYTES;
#pragma unroll
                        for (int k = 0; k < BK / 8; ++k) {  // 8 f32 = 32 bytes per k-step inside the 128-byte swizzle row
                            const uint64_t ah = smem_desc_sw128(s0 + k * 32, 16, 1024);
                            const uint64_t al = smem_desc_sw128(s0 + A_BYTES + k * 32, 16, 1024);
                            const uint64_t bh = smem_desc_sw128(s0 + 2 * A_BYTES + k * 32, 16, 1024);
                            const uint64_t bl = smem_desc_sw128(s0 + 2 * A_BYTES + B_BYTES + k * 32, 16, 1024);
                            mma_tf32_ss(d0, al, bh, idesc, (kb > kb0 || k > 0) ? 1u : 0u);  // the small terms first
                            mma_tf32_ss(d0, ah, bl, idesc, 1u);
                            mma_tf32_ss(d0, ah, bh, idesc, 1u);
                        }
                        mma_commit(smem_u32(&bars->empty[stage]));
                        if (++stage == STAGES) {
                            stage = 0;
                            phase ^= 1u;
                        }
                    }
                    if (!ok) break;
                    mma_commit(smem_u32(&bars->acc_full[acc]));
                    if (++acc == 2) {
                        acc = 0;
                        acc_phase ^= 1u;
                    }
                }
            }
        }
    } else {
        const int quarter = warp & 3;
        uint32_t acc = 0, acc_phase = 0;
        bool ok = true;
        TOut* C = static_cast<TOut*>(p.C);
        const TOut* post_full = static_cast<const TOut*>(p.post_full);
        for (int64_t tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
            int64_t tm, tn;
            tile_coords(tile, tiles_m, tiles_n, tm, tn);
            const int64_t row = tm * BM + quarter * 32 + lane;
            const int64_t n0  = tn * BN;
            // sum the K chunks of this tile in registers (round-to-nearest f32 adds): one row, BN columns per thread
            float sum[BN];
#pragma unroll
            for (int i = 0; i < BN; ++i) sum[i] = 0.f;
            for (int kb0 = 0; kb0 < num_kb && ok; kb0 += CHUNK_KB) {
                if (!(ok = mbar_wait(smem_u32(&bars->acc_full[acc]), acc_phase, abort_flag))) break;
                tc_fence_after();
                const uint32_t t0 = tmem_base + acc * BN + (uint32_t(quarter * 32) << 16);
#pragma unroll
                for (int c = 0; c < BN; c += 32) {
                    uint32_t r[32];
                    tmem_ld_32x32(t0 + c, r);
                    tmem_ld_wait();
#pragma unroll
                    for (int i = 0; i < 32; ++i) sum[c + i] += __uint_as_float(r[i]);
                }
                tc_fence_before();
                mbar_arrive(smem_u32(&bars->acc_empty[acc]));
                if (++acc == 2) {
                    acc = 0;
                    acc_phase ^= 1u;
                }
            }
            if (!ok) break;
            if (row < p.M) {
                // columns of this row whose tensor-core result is not finite: recomputed below
                uint32_t bad[BN / 32];
#pragma unroll
                for (int c = 0; c < BN; c += 32) {
                    uint32_t m = 0;
#pragma unroll
                    for (int i = 0; i < 32; ++i) m |= isfinite(sum[c + i]) ? 0u : (1u << i);
                    bad[c / 32] = m;
                }
                // A non-finite cell means an operand of its fold was inf / NaN (or a head overflowed, or the sum did): the
                // split products are then not the f32 products (inf * 0 from a zero tail is NaN). Such cells take the
                // scalar fold of the CUDA-core kernel -- ascending k, one fma per step -- from the caller's operands.
#pragma unroll 1
                for (int w = 0; w < BN / 32; ++w) {
                    uint32_t m = w == 0 ? bad[0] : w == 1 ? bad[1] : w == 2 ? bad[2] : bad[3];
                    while (m) {
                        const int i = __ffs(m) - 1;
                        m &= m - 1;
                        const int64_t col = n0 + w * 32 + i;
                        if (col >= p.N) continue;
                        const float* a = p.A0 + row * p.K;
                        float acc      = 0.f;
                        if (p.b_nk) {
                            const float* b = p.B0 + col * p.K;
                            for (int64_t k = 0; k < p.K; ++k) acc = fmaf(a[k], b[k], acc);
                        } else {
                            const float* b = p.B0 + col;
                            for (int64_t k = 0; k < p.K; ++k) acc = fmaf(a[k], b[k * p.N], acc);
                        }
                        const int idx = w * 32 + i;
#pragma unroll
                        for (int j = 0; j < BN; ++j)
                            if (j == idx) sum[j] = acc;
                    }
                }
#pragma unroll
                for (int c = 0; c < BN; c += 32) {
                    float* v           = sum + c;
                    const int64_t col0 = n0 + c;
                    if (p.post != MIMK_POST_ID) {
#pragma unroll
                        for (int i = 0; i < 32; ++i) {
                            const int64_t col = col0 + i;
                            if (col < p.N) {
                                const float rowv = p.post_row ? __ldg(p.post_row + col) : 0.f;
                                const float full = post_full ? float(post_full[row * p.N + col]) : 0.f;
                                v[i]             = apply_post(p.post, v[i], rowv, full);
                            }
                        }
                    }
                    TOut* dst = C + row * p.N + col0;
                    if (sizeof(TOut) == 2) {
#pragma unroll
                        for (int i = 0; i < 32; i += 8) {
                            if (col0 + i < p.N) {  // N % 8 == 0 for bf16 output
                                uint4 q;
                                q.x = pack_bf16x2(v[i], v[i + 1]);
                                q.y = pack_bf16x2(v[i + 2], v[i + 3]);
                                q.z = pack_bf16x2(v[i + 4], v[i + 5]);
                                q.w = pack_bf16x2(v[i + 6], v[i + 7]);
                                *reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(dst) + i) = q;
                            }
                        }
                    } else {
#pragma unroll
                        for (int i = 0; i < 32; i += 4) {
                            if (col0 + i < p.N)  // N % 4 == 0 for f32 output
                                *reinterpret_cast<float4*>(reinterpret_cast<float*>(dst) + i) =
                                    make_float4(v[i], v[i + 1], v[i + 2], v[i + 3]);
                        }
                    }
                }
            }
        }
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        __syncwarp();
        tc_fence_after();
        tmem_dealloc(tmem_base, 256);
    }
    if (threadIdx.x == 0 && *abort_flag) *p.status = MIMK_E_DEVICE_WAIT;
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

int make_tmap_f32_2d(CUtensorMap* out, const void* base, uint64_t inner, uint64_t outer, uint32_t box_outer) {
    static EncodeTiledFn fn = nullptr;
    if (!fn) {
        void* ptr = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &q) != cudaSuccess ||
            q != cudaDriverEntryPointSuccess) {
            cudaGetLastError();
            return MIMK_E_CUDA;
        }
        fn = reinterpret_cast<EncodeTiledFn>(ptr);
    }
    cuuint64_t dims[2]    = {inner, outer};
    cuuint64_t strides[1] = {inner * 4};
    cuuint32_t box[2]     = {BK, box_outer};
    cuuint32_t estr[2]    = {1, 1};
    CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<void*>(base), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? MIMK_OK : MIMK_E_CUDA;
}

template <class TOut>
int launch(const CUtensorMap& ah, const CUtensorMap& al, const CUtensorMap& bh, const CUtensorMap& bl, const Params& p,
           int sm_count, cudaStream_t s) {
    auto kern = gemm_f32_tc_kernel<TOut>;
    static bool configured[64] = {};
    int dev = 0;
    MIMK_CUDA_TRY(cudaGetDevice(&dev));
    if (!configured[dev & 63]) {
        MIMK_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES));
        configured[dev & 63] = true;
    }
    const int64_t tiles = ((p.M + BM - 1) / BM) * ((p.N + BN - 1) / BN);
    const int grid      = int(tiles < sm_count ? tiles : sm_count);
    kern<<<grid, NUM_THREADS, SMEM_BYTES, s>>>(ah, al, bh, bl, p);
    return launch_status();
}

}  // namespace

// f32 operands, sizes from 128^3-ish upwards, TMA-friendly strides; everything else stays on the CUDA-core kernel.
int gemm_f32_tc_supported(const mimk_gemm_desc& d) {
    if (d.in_dtype != MIMK_F32) return 0;
    if (d.k <= 0) return 0;
    if (d.out_dtype == MIMK_BF16 ? d.n % 8 != 0 : d.n % 4 != 0) return 0;  // 16-byte epilogue stores
    if (d.m < 128 || d.n < 128 || d.m * d.n * d.k < (int64_t(1) << 23)) return 0;
    if (d.m >= (int64_t(1) << 31) || d.n >= (int64_t(1) << 31) || d.k >= (int64_t(1) << 31)) return 0;
    if (!aligned16(d.c)) return 0;  // the operands are re-written as padded hi / lo copies; only the result is stored as is
    if (d.post_full && !aligned16(d.post_full)) return 0;
    if (d.batch > 16) return 0;
    return 1;
}

int gemm_f32_tc(const mimk_gemm_desc& d, cudaStream_t s) {
    int st          = MIMK_OK;
    DeviceInfo* dev = device_info(&st);
    if (!dev) return st;
    const int64_t kp = (d.k + 3) & ~int64_t(3);  // row pitch of the hi / lo copies: 16-byte multiples
    const size_t a_elems = size_t(d.m) * kp, b_elems = size_t(d.n) * kp;
    const size_t a_bytes = (a_elems * 4 + 255) & ~size_t(255), b_bytes = (b_elems * 4 + 255) & ~size_t(255);
    void* scratch = nullptr;
    MIMK_TRY(get_scratch(2 * a_bytes + 2 * b_bytes, &scratch, s));
    uint8_t* base = static_cast<uint8_t*>(scratch);
    float *a_hi = reinterpret_cast<float*>(base), *a_lo = reinterpret_cast<float*>(base + a_bytes);
    float *b_hi = reinterpret_cast<float*>(base + 2 * a_bytes), *b_lo = reinterpret_cast<float*>(base + 2 * a_bytes + b_bytes);
    const size_t out_size = d.out_dtype == MIMK_BF16 ? 2 : 4;
    for (int64_t b = 0; b < d.batch; ++b) {
        const float* A = static_cast<const float*>(d.a) + b * d.stride_a;
        const float* B = static_cast<const float*>(d.b) + b * d.stride_b;
        if (b == 0 || d.stride_a != 0) {
            int grid = int((a_elems + 1023) / 1024 < size_t(dev->sm_count) * 8 ? (a_elems + 1023) / 1024 : size_t(dev->sm_count) * 8);
            if (kp == d.k) split_kernel<<<grid, 256, 0, s>>>(A, a_hi, a_lo, int64_t(a_elems));
            else split_pad_kernel<<<grid, 256, 0, s>>>(A, a_hi, a_lo, d.m, d.k, kp);
            MIMK_TRY(launch_status());
        }
        if (b == 0 || d.stride_b != 0) {
            if (d.b_layout == MIMK_B_NK) {
                int grid = int((b_elems + 1023) / 1024 < size_t(dev->sm_count) * 8 ? (b_elems + 1023) / 1024 : size_t(dev->sm_count) * 8);
                if (kp == d.k) split_kernel<<<grid, 256, 0, s>>>(B, b_hi, b_lo, int64_t(b_elems));
                else split_pad_kernel<<<grid, 256, 0, s>>>(B, b_hi, b_lo, d.n, d.k, kp);
            } else {
                dim3 grid((unsigned)((d.n + 31) / 32), (unsigned)((d.k + 31) / 32));
                if (grid.y > 65535) return MIMK_E_UNSUPPORTED;
                split_transpose_kernel<<<grid, dim3(32, 8), 0, s>>>(B, b_hi, b_lo, d.k, d.n, kp);
            }
            MIMK_TRY(launch_status());
        }
        CUtensorMap tAh, tAl, tBh, tBl;
        MIMK_TRY(make_tmap_f32_2d(&tAh, a_hi, uint64_t(kp), uint64_t(d.m), BM));
        MIMK_TRY(make_tmap_f32_2d(&tAl, a_lo, uint64_t(kp), uint64_t(d.m), BM));
        MIMK_TRY(make_tmap_f32_2d(&tBh, b_hi, uint64_t(kp), uint64_t(d.n), BN));
        MIMK_TRY(make_tmap_f32_2d(&tBl, b_lo, uint64_t(kp), uint64_t(d.n), BN));
        Params p;
        p.M = d.m, p.N = d.n, p.K = d.k;
        p.C         = static_cast<uint8_t*>(d.c) + size_t(b * d.stride_c) * out_size;
        p.post_row  = static_cast<const float*>(d.post_row);
        p.post_full = d.post_full ? static_cast<const uint8_t*>(d.post_full) + size_t(b * d.stride_c) * out_size : nullptr;
        p.post      = d.post;
        p.status    = dev->status_dev;
        p.A0 = A, p.B0 = B, p.b_nk = d.b_layout == MIMK_B_NK;
        MIMK_TRY(d.out_dtype == MIMK_BF16 ? launch<__nv_bfloat16>(tAh, tAl, tBh, tBl, p, dev->sm_count, s)
                                          : launch<float>(tAh, tAl, tBh, tBl, p, dev->sm_count, s));
    }
    return MIMK_OK;
}

}  // namespace mimk
