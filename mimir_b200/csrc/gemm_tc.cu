// bf16 contraction on the 5th-generation tensor cores (tcgen05), f32 accumulators in tensor memory.
//
// This is `dot_product_impl` (MimIR src/mim/plug/tensor/tensor.mim:1367-1411) for bf16 operands: the fold
// `acc = add(acc, mul(a, b))` of `dot_general_fun` (tensor.mim:1332) with To = F32 and Tis = (BF16, BF16),
// followed by the `post` epilogue slot that `fuse_tensor` fills (src/mim/plug/tensor/phase/fuse.cpp:408-534).
// Both right-operand layouts of the reference exist: B stored [K,N] (`dot_schedule`, tensor.mim:989) is an
// MN-major operand, B stored [N,K] read through transpose_2d (`dot_schedule_kvec`, tensor.mim:1015) is K-major.
//
// Structure: one persistent CTA per SM walks output tiles of 128 x 256 (or 128 x 128 twice for the gated form).
//   warp 0       TMA producer: A and B tiles of 64 k-columns into a ring of 128-byte-swizzled shared memory stages
//   warp 1       MMA issuer: one thread issues tcgen05.mma (M=128, N=BN, K=16) and commits stage/accumulator barriers
//   warps 2..5   epilogue: tcgen05.ld the f32 accumulator (one row per thread), apply `post`, stage 32 rows x 128 bytes in
//                128-byte-swizzled shared memory, one bulk (TMA) store per destination
// A batched product (tensor.bmm, tensor.mim:404-407) is ONE launch: the tensor maps are three-dimensional with the
// batch as the outermost coordinate, and the tile walk runs over (batch, tile) pairs, batch-major.
// Two accumulator buffers in TMEM let the epilogue of tile i overlap the main loop of tile i+1.
// Every mbarrier wait is bounded; on expiry the CTA records MIMK_E_DEVICE_WAIT and unwinds (frees TMEM, exits).
#include "common.cuh"
#include "sm100.cuh"

namespace mimk {

using namespace sm100;

namespace {

constexpr int BM = 128, BK = 64, STAGES = 4;
constexpr int ACC_COLS = 256;                  // TMEM columns per accumulator buffer
constexpr int A_BYTES  = BM * BK * 2;          // 16 KiB
constexpr int B_BYTES  = ACC_COLS * BK * 2;    // 32 KiB: one 256-row tile or two 128-row tiles
constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
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
constexpr int OUT_STAGE_BYTES = 4 * 2 * 4096;  // per epilogue warp: two buffers of 32 rows x 128 bytes for the bulk stores
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + OUT_STAGE_BYTES + 1024 /*alignment slack*/ + 256;
static_assert(sizeof(Bars) <= 256, "barrier block too large");
static_assert(SMEM_BYTES <= 232448, "more shared memory than a CTA can have");

// One tensor map per destination matrix (this GPU's C, or every rank's copy of a gathered matrix): [batch, M, N] windows.
struct OutMaps {
    CUtensorMap m[MIMK_MAX_GATHER];
};

struct Params {
    int64_t M, N, K;
    int64_t batch, stride_c;  // batch entries; elements between consecutive results (and full-shape epilogue operands)
    int a_batched, b_batched; // 0: every batch entry reads the same operand (batch coordinate 0)
    int a_panel_k, a_panel_rows;  // A as K-panels: columns per panel (K when A is one matrix) and rows between panels
    // The result tile goes to `n_dst` matrices of leading dimension `ldc`, at column offset `col_off`: one destination
    // (C itself, ldc = N) for an ordinary call; this GPU's and its peers' copies of a gathered matrix when the all-gather
    // of a column-sharded contraction is fused into the epilogue (plain stores to peer-mapped addresses over NVLink).
    void* dst[MIMK_MAX_GATHER];
    int n_dst;
    int64_t ldc, col_off;
    const float* post_row;
    const void* post_full;
    int post;
    int* status;
};

__device__ __forceinline__ void tile_coords(int64_t tile, int64_t tiles_m, int64_t tiles_n, int64_t& tm, int64_t& tn) {
    const int64_t per_group = GROUP_M * tiles_n;
    const int64_t group     = tile / per_group;
    const int64_t first_m   = group * GROUP_M;
    const int64_t gsize     = (tiles_m - first_m) < GROUP_M ? (tiles_m - first_m) : GROUP_M;
    const int64_t in_group  = tile % per_group;
    tm                      = first_m + in_group % gsize;
    tn                      = in_group / gsize;
}

// BN: output-tile width per B operand (256 plain, 128 gated). B_MN: B stored [K,N] (N contiguous).
template <int BN, bool B_MN, bool GATED, class TOut>
__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
               const __grid_constant__ CUtensorMap tmB2, const __grid_constant__ OutMaps om, const Params p) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw_addr  = smem_u32(smem_raw);
    const uint32_t tile_base = (raw_addr + 1023u) & ~1023u;
    Bars* bars = reinterpret_cast<Bars*>(smem_raw + (tile_base - raw_addr) + STAGES * STAGE_BYTES + OUT_STAGE_BYTES);
    volatile int* abort_flag = &bars->abort_flag;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int64_t tiles_m = (p.M + BM - 1) / BM, tiles_n = (p.N + BN - 1) / BN;
    const int64_t per_batch = tiles_m * tiles_n;
    const int64_t num_tiles = per_batch * p.batch;
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
        tma_prefetch_desc(&tmA);
        tma_prefetch_desc(&tmB);
        if (GATED) tma_prefetch_desc(&tmB2);
    }
    if (warp == 1) {
        tmem_alloc(smem_u32(&bars->tmem_base), 512);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(&bars->tmem_base);

    if (warp == 0) {
        // ---------------- TMA producer ----------------
        if (lane == 0) {
            uint32_t stage = 0, phase = 0;
            bool ok = true;
            for (int64_t tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
                int64_t tm, tn;
                const int64_t bz = tile / per_batch;
                tile_coords(tile - bz * per_batch, tiles_m, tiles_n, tm, tn);
                const int m0 = int(tm * BM), n0 = int(tn * BN);
                const int za = p.a_batched ? int(bz) : 0, zb = p.b_batched ? int(bz) : 0;
                for (int kb = 0; kb < num_kb; ++kb) {
                    if (!(ok = mbar_wait(smem_u32(&bars->empty[stage]), phase ^ 1u, abort_flag))) break;
                    const uint32_t full = smem_u32(&bars->full[stage]);
                    const uint32_t sa   = tile_base + stage * STAGE_BYTES;
                    const uint32_t sb   = sa + A_BYTES;
                    mbar_expect_tx(full, A_BYTES + (GATED ? 2 : 1) * BN * BK * 2);
                    const int ka = kb * BK, pa = ka / p.a_panel_k;  // the K-panel of A this k-block lies in
                    tma_load_3d(sa, &tmA, ka - pa * p.a_panel_k, m0 + pa * p.a_panel_rows, za, full);
                    if (!B_MN) {
                        tma_load_3d(sb, &tmB, kb * BK, n0, zb, full);
                        if (GATED) tma_load_3d(sb + BN * BK * 2, &tmB2, kb * BK, n0, zb, full);
                    } else {
#pragma unroll
                        for (int j = 0; j < BN / 64; ++j) {
                            tma_load_3d(sb + j * (BK * 128), &tmB, n0 + j * 64, kb * BK, zb, full);
                            if (GATED) tma_load_3d(sb + BN * BK * 2 + j * (BK * 128), &tmB2, n0 + j * 64, kb * BK, zb, full);
                        }
                    }
                    if (++stage == STAGES) {
                        stage = 0;
                        phase ^= 1u;
                    }
                }
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer ----------------
        if (lane == 0) {
            const uint32_t idesc = idesc_bf16_f32(BM, GATED ? 2 * BN : BN, 0, B_MN ? 1 : 0);
            uint32_t stage = 0, phase = 0, acc = 0, acc_phase = 0;
            bool ok = true;
            for (int64_t tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
                if (!(ok = mbar_wait(smem_u32(&bars->acc_empty[acc]), acc_phase ^ 1u, abort_flag))) break;
                tc_fence_after();
                const uint32_t d0 = tmem_base + acc * ACC_COLS;
                for (int kb = 0; kb < num_kb; ++kb) {
                    if (!(ok = mbar_wait(smem_u32(&bars->full[stage]), phase, abort_flag))) break;
                    tc_fence_after();
                    const uint32_t sa = tile_base + stage * STAGE_BYTES;
                    const uint32_t sb = sa + A_BYTES;
#pragma unroll
                    for (int k = 0; k < BK / 16; ++k) {
                        const uint64_t ad = smem_desc_sw128(sa + k * 32, 16, 1024);
                        const uint32_t boff = B_MN ? k * 2048 : k * 32;
                        const uint32_t lead = B_MN ? BK * 128 : 16;
                        const uint64_t bd   = smem_desc_sw128(sb + boff, lead, 1024);
                        const uint32_t accum = (kb > 0 || k > 0) ? 1u : 0u;
                        // gated: the two 128-row B tiles lie back to back in shared memory and are issued as one 256-row
                        // operand, so one instruction feeds both accumulators (columns [0,128) gate, [128,256) up)
                        mma_f16_ss(d0, ad, bd, idesc, accum);
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
    } else {
        // ---------------- epilogue (warps 2..5) ----------------
        // Each warp owns 32 rows of the tile: accumulator -> registers (tcgen05.ld, one row per thread) -> `post` -> a
        // 128-byte-swizzled [32 x 128 B] piece in shared memory -> one bulk store per destination. Two pieces per warp
        // alternate, so the stores of one drain while the next is converted. Rows and columns past the matrix edge are
        // clipped by the store itself.
        const int quarter = warp & 3;  // TMEM lanes [32*quarter, 32*quarter + 32) are this warp's
        constexpr int CW = 128 / int(sizeof(TOut));  // output columns per 128-byte store row: 64 bf16 or 32 f32
        const uint32_t out_base = tile_base + STAGES * STAGE_BYTES + quarter * 2 * 4096;
        uint32_t acc = 0, acc_phase = 0, chunk_no = 0;
        bool ok = true;
        const TOut* post_full = static_cast<const TOut*>(p.post_full);
        for (int64_t tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
            int64_t tm, tn;
            const int64_t bz = tile / per_batch;
            tile_coords(tile - bz * per_batch, tiles_m, tiles_n, tm, tn);
            const int64_t zoff = bz * p.stride_c;  // this batch entry's full-shape epilogue operand
            const int64_t row0 = tm * BM + quarter * 32;
            const int64_t row  = row0 + lane;
            const int64_t n0   = tn * BN;
            if (!(ok = mbar_wait(smem_u32(&bars->acc_full[acc]), acc_phase, abort_flag))) break;
            tc_fence_after();
            const uint32_t t0 = tmem_base + acc * ACC_COLS + (uint32_t(quarter * 32) << 16);
#pragma unroll 1
            for (int c0 = 0; c0 < BN; c0 += CW, ++chunk_no) {
                const uint32_t buf = out_base + (chunk_no & 1u) * 4096;
                if (lane == 0) bulk_wait_read_1();  // the store that last used this buffer has read it
                __syncwarp();
#pragma unroll
                for (int c = c0; c < c0 + CW; c += 32) {
                    uint32_t r[32];
                    float v[32];
                    tmem_ld_32x32(t0 + c, r);
                    if (GATED) {
                        uint32_t u[32];
                        tmem_ld_32x32(t0 + BN + c, u);
                        tmem_ld_wait();
#pragma unroll
                        for (int i = 0; i < 32; ++i) {
                            const float g = __uint_as_float(r[i]);
                            v[i]          = (g / (1.f + __expf(-g))) * __uint_as_float(u[i]);
                        }
                    } else {
                        tmem_ld_wait();
#pragma unroll
                        for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
                    }
                    if (c + 32 >= BN) {
                        // last read of this accumulator buffer: hand it back before the stores
                        tc_fence_before();
                        mbar_arrive(smem_u32(&bars->acc_empty[acc]));
                    }
                    if (p.post != MIMK_POST_ID && row < p.M) {
#pragma unroll
                        for (int i = 0; i < 32; ++i) {
                            const int64_t col = n0 + c + i;
                            if (col < p.N) {
                                const float rowv = p.post_row ? __ldg(p.post_row + col) : 0.f;
                                const float full = post_full ? float(post_full[zoff + row * p.N + col]) : 0.f;
                                v[i]             = apply_post(p.post, v[i], rowv, full);
                            }
                        }
                    }
                    // this thread's row of the piece: 16-byte units at (unit ^ (row & 7)), the 128-byte swizzle
                    const uint32_t row_addr = buf + lane * 128;
                    if (sizeof(TOut) == 2) {
                        const int unit0 = ((c - c0) * 2) >> 4;  // 32 bf16 = 4 units
#pragma unroll
                        for (int i = 0; i < 32; i += 8) {
                            const uint32_t a = row_addr + ((uint32_t(unit0 + (i >> 3)) ^ uint32_t(lane & 7)) << 4);
                            asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(a), "r"(pack_bf16x2(v[i], v[i + 1])),
                                         "r"(pack_bf16x2(v[i + 2], v[i + 3])), "r"(pack_bf16x2(v[i + 4], v[i + 5])),
                                         "r"(pack_bf16x2(v[i + 6], v[i + 7]))
                                         : "memory");
                        }
                    } else {
#pragma unroll
                        for (int i = 0; i < 32; i += 4) {
                            const uint32_t a = row_addr + ((uint32_t(i >> 2) ^ uint32_t(lane & 7)) << 4);
                            asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(a), "r"(__float_as_uint(v[i])),
                                         "r"(__float_as_uint(v[i + 1])), "r"(__float_as_uint(v[i + 2])),
                                         "r"(__float_as_uint(v[i + 3]))
                                         : "memory");
                        }
                    }
                }
                fence_proxy_async_smem();  // the bulk store reads shared memory through the async proxy
                __syncwarp();
                if (lane == 0) {
                    if (row0 < p.M && n0 + c0 < p.N)
                        for (int t = 0; t < p.n_dst; ++t) tma_store_3d(&om.m[t], buf, int(n0 + c0), int(row0), int(bz));
                    bulk_commit();
                }
            }
            if (++acc == 2) {
                acc = 0;
                acc_phase ^= 1u;
            }
        }
        if (lane == 0) bulk_wait_all();  // every store has landed before the CTA may exit
    }

    // ---------------- teardown ----------------
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, 512);
    }
    if (threadIdx.x == 0 && *abort_flag) *p.status = MIMK_E_DEVICE_WAIT;
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = nullptr;
    if (!fn) {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(p);
        else
            cudaGetLastError();
    }
    return fn;
}

template <int BN, bool B_MN, bool GATED, class TOut>
int launch(const CUtensorMap& tA, const CUtensorMap& tB, const CUtensorMap& tB2, const OutMaps& om, const Params& p,
           int sm_count, cudaStream_t s) {
    auto kern = gemm_tc_kernel<BN, B_MN, GATED, TOut>;
    static bool configured[64] = {};  // per template instance and device: the attribute is a per-device setting
    int dev = 0;
    MIMK_CUDA_TRY(cudaGetDevice(&dev));
    if (!configured[dev & 63]) {
        MIMK_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES));
        configured[dev & 63] = true;
    }
    const int64_t tiles = ((p.M + BM - 1) / BM) * ((p.N + BN - 1) / BN) * p.batch;
    const int grid      = int(tiles < sm_count ? tiles : sm_count);
    kern<<<grid, NUM_THREADS, SMEM_BYTES, s>>>(tA, tB, tB2, om, p);
    return launch_status();
}

}  // namespace

int make_tmap_bf16_2d(CUtensorMap* out, const void* base, uint64_t inner, uint64_t outer, uint64_t row_stride_bytes,
                      uint32_t box_inner, uint32_t box_outer) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) return MIMK_E_CUDA;
    cuuint64_t dims[2]    = {inner, outer};
    cuuint64_t strides[1] = {row_stride_bytes};
    cuuint32_t box[2]     = {box_inner, box_outer};
    cuuint32_t estr[2]    = {1, 1};
    CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? MIMK_OK : MIMK_E_CUDA;
}

int make_tmap_2d(CUtensorMap* out, bool f32, const void* base, uint64_t inner, uint64_t outer, uint64_t row_stride_bytes,
                 uint32_t box_inner, uint32_t box_outer) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) return MIMK_E_CUDA;
    cuuint64_t dims[2]    = {inner, outer};
    cuuint64_t strides[1] = {row_stride_bytes};
    cuuint32_t box[2]     = {box_inner, box_outer};
    cuuint32_t estr[2]    = {1, 1};
    CUresult r = fn(out, f32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base),
                    dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                    CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? MIMK_OK : MIMK_E_CUDA;
}

int make_tmap_bf16_3d(CUtensorMap* out, const void* base, uint64_t inner, uint64_t mid, uint64_t outer,
                      uint64_t mid_stride_bytes, uint64_t outer_stride_bytes, uint32_t box_inner, uint32_t box_mid) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) return MIMK_E_CUDA;
    cuuint64_t dims[3]    = {inner, mid, outer};
    cuuint64_t strides[2] = {mid_stride_bytes, outer_stride_bytes};
    cuuint32_t box[3]     = {box_inner, box_mid, 1};
    cuuint32_t estr[3]    = {1, 1, 1};
    CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(base), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? MIMK_OK : MIMK_E_CUDA;
}

int make_tmap_3d(CUtensorMap* out, bool f32, const void* base, uint64_t inner, uint64_t mid, uint64_t outer,
                 uint64_t mid_stride_bytes, uint64_t outer_stride_bytes, uint32_t box_inner, uint32_t box_mid) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) return MIMK_E_CUDA;
    cuuint64_t dims[3]    = {inner, mid, outer};
    cuuint64_t strides[2] = {mid_stride_bytes, outer_stride_bytes};
    cuuint32_t box[3]     = {box_inner, box_mid, 1};
    cuuint32_t estr[3]    = {1, 1, 1};
    CUresult r = fn(out, f32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(base),
                    dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                    CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? MIMK_OK : MIMK_E_CUDA;
}

int gemm_tc_supported(const mimk_gemm_desc& d) {
    if (d.in_dtype != MIMK_BF16) return 0;
    if (d.k <= 0 || d.k % 8 != 0 || d.n % 8 != 0) return 0;  // TMA: 16-byte strides; epilogue: 16-byte stores
    if (d.m >= (int64_t(1) << 31) || d.n >= (int64_t(1) << 31) || d.k >= (int64_t(1) << 31)) return 0;
    if (!aligned16(d.a) || !aligned16(d.b) || !aligned16(d.c)) return 0;
    if (d.post_full && !aligned16(d.post_full)) return 0;
    if (d.batch >= (int64_t(1) << 31)) return 0;
    if (d.batch > 1) {
        if (d.stride_a % 8 || d.stride_b % 8 || d.stride_c % 8) return 0;  // TMA strides, 16-byte stores
        // batch strides that are whole rows of the operand (dense batches are), below the TMA stride limit
        const int64_t row_b = d.b_layout == MIMK_B_KN ? d.n : d.k;
        if (d.stride_a % d.k || d.stride_b % row_b || d.stride_c % d.n) return 0;
        if (d.stride_a >= (int64_t(1) << 38) || d.stride_b >= (int64_t(1) << 38) || d.stride_c >= (int64_t(1) << 38)) return 0;
    }
    return 1;
}

int gemm_tc(const mimk_gemm_desc& d, cudaStream_t s, int gated, const void* b2, const mimk_gather_dst* gather,
            int64_t a_panels) {
    int st          = MIMK_OK;
    DeviceInfo* dev = device_info(&st);
    if (!dev) return st;
    const bool b_mn = d.b_layout == MIMK_B_KN;
    const int bn    = gated ? 128 : 256;
    // Operands as [batch, rows, cols] tensor maps; an operand shared by all batch entries (stride 0) has one entry.
    const bool a_b = d.batch > 1 && d.stride_a != 0, b_b = d.batch > 1 && d.stride_b != 0;
    const uint64_t na = a_b ? uint64_t(d.batch) : 1, nb = b_b ? uint64_t(d.batch) : 1;
    // (the outermost stride of a one-entry operand is never used; it only has to be a legal value)
    const uint64_t row_b = (b_mn ? uint64_t(d.n) : uint64_t(d.k)) * 2;
    const uint64_t whole_a = uint64_t(d.m) * uint64_t(d.k) * 2, whole_b = uint64_t(d.n) * uint64_t(d.k) * 2;
    const uint64_t sa = a_b ? uint64_t(d.stride_a) * 2 : (whole_a < (uint64_t(1) << 40) ? whole_a : uint64_t(d.k) * 2);
    const uint64_t sb = b_b ? uint64_t(d.stride_b) * 2 : (whole_b < (uint64_t(1) << 40) ? whole_b : row_b);
    const void* B2 = b2 ? b2 : d.b;
    CUtensorMap tA, tB, tB2;
    if (a_panels < 1 || (a_panels > 1 && (d.batch != 1 || d.k % a_panels != 0 || (d.k / a_panels) % BK != 0))) return MIMK_E_UNSUPPORTED;
    const uint64_t kp = uint64_t(d.k / a_panels);  // A as a [panels * m, k / panels] matrix: panel g starts at row g * m
    MIMK_TRY(make_tmap_bf16_3d(&tA, d.a, kp, uint64_t(d.m) * uint64_t(a_panels), na, kp * 2, sa, BK, BM));
    if (b_mn) {
        MIMK_TRY(make_tmap_bf16_3d(&tB, d.b, uint64_t(d.n), uint64_t(d.k), nb, uint64_t(d.n) * 2, sb, 64, BK));
        MIMK_TRY(make_tmap_bf16_3d(&tB2, B2, uint64_t(d.n), uint64_t(d.k), nb, uint64_t(d.n) * 2, sb, 64, BK));
    } else {
        MIMK_TRY(make_tmap_bf16_3d(&tB, d.b, uint64_t(d.k), uint64_t(d.n), nb, uint64_t(d.k) * 2, sb, BK, uint32_t(bn)));
        MIMK_TRY(make_tmap_bf16_3d(&tB2, B2, uint64_t(d.k), uint64_t(d.n), nb, uint64_t(d.k) * 2, sb, BK, uint32_t(bn)));
    }
    Params p;
    p.M = d.m, p.N = d.n, p.K = d.k;
    p.batch = d.batch, p.stride_c = d.batch > 1 ? d.stride_c : 0;
    p.a_batched = a_b, p.b_batched = b_b;
    p.a_panel_k = a_panels > 1 ? int(kp) : int((d.k + BK - 1) / BK * BK), p.a_panel_rows = a_panels > 1 ? int(d.m) : 0;
    if (gather) {
        if (d.batch != 1) return MIMK_E_UNSUPPORTED;
        p.n_dst = gather->n_dst;
        for (int t = 0; t < gather->n_dst; ++t) p.dst[t] = gather->dst[t];
        p.ldc = gather->ldc, p.col_off = gather->col_off;
    } else {
        p.n_dst  = 1;
        p.dst[0] = d.c;
        p.ldc = d.n, p.col_off = 0;
    }
    p.post_row  = static_cast<const float*>(d.post_row);
    p.post_full = d.post_full;
    p.post      = d.post;
    p.status    = dev->status_dev;
    // destination maps: [batch, M, N] windows (row pitch ldc) starting at column col_off, boxes of 32 rows x 128 bytes
    const uint64_t out_size = d.out_dtype == MIMK_BF16 ? 2 : 4;
    const uint64_t pitch    = uint64_t(p.ldc) * out_size;
    const uint64_t whole_c  = uint64_t(d.m) * pitch;
    const uint64_t sc = d.batch > 1 ? uint64_t(d.stride_c) * out_size : (whole_c < (uint64_t(1) << 40) ? whole_c : pitch);
    OutMaps om;
    for (int t = 0; t < p.n_dst; ++t) {
        const uint8_t* base = static_cast<const uint8_t*>(p.dst[t]) + size_t(p.col_off) * out_size;
        MIMK_TRY(make_tmap_3d(&om.m[t], d.out_dtype == MIMK_F32, base, uint64_t(d.n), uint64_t(d.m), uint64_t(d.batch), pitch, sc,
                              uint32_t(128 / out_size), 32));
    }
    for (int t = p.n_dst; t < MIMK_MAX_GATHER; ++t) om.m[t] = om.m[0];
    if (gated) {
        if (d.out_dtype != MIMK_BF16) return MIMK_E_DTYPE;
        return b_mn ? launch<128, true, true, __nv_bfloat16>(tA, tB, tB2, om, p, dev->sm_count, s)
                    : launch<128, false, true, __nv_bfloat16>(tA, tB, tB2, om, p, dev->sm_count, s);
    }
    if (d.out_dtype == MIMK_BF16)
        return b_mn ? launch<256, true, false, __nv_bfloat16>(tA, tB, tB2, om, p, dev->sm_count, s)
                    : launch<256, false, false, __nv_bfloat16>(tA, tB, tB2, om, p, dev->sm_count, s);
    return b_mn ? launch<256, true, false, float>(tA, tB, tB2, om, p, dev->sm_count, s)
                : launch<256, false, false, float>(tA, tB, tB2, om, p, dev->sm_count, s);
}

}  // namespace mimk
