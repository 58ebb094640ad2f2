// bf16 contraction on paired SMs: tcgen05.mma with cta_group::2.
//
// Same operator as gemm_tc.cu (`dot_product_impl`, MimIR src/mim/plug/tensor/tensor.mim:1367-1411, with the `post`
// slot of src/mim/plug/tensor/phase/fuse.cpp:408-534), but two CTAs of a cluster share one 256 x BN output tile: CTA r
// owns rows [128 r, 128 r + 128) of the tile (its A tile and its accumulator, 128 TMEM lanes) and loads only HALF of
// the B tile (BN/2 of its rows); one MMA instruction issued by the even CTA multiplies both A tiles with both B halves.
// Per flop this reads a third less from L2 and shared memory than the one-CTA kernel -- the feed that limits it.
//
//   warp 0 (both CTAs)   TMA producer: own A tile and own B half into own shared memory; completion bytes are
//                        signalled on the EVEN CTA's `full` barrier (cp.async.bulk.tensor ... cta_group::2, no multicast)
//   warp 1 (even CTA)    MMA issuer: tcgen05.mma.cta_group::2 (M 256, N BN, K 16); tcgen05.commit ... multicast::cluster
//                        releases a stage / publishes an accumulator in BOTH CTAs
//   warps 2..5 (both)    epilogue of the CTA's own 128 rows; hands the accumulator back by arriving on the even CTA's
//                        `acc_empty` barrier (remote arrive from the odd CTA)
// Every wait is bounded; a CTA that gives up records MIMK_E_DEVICE_WAIT, and both CTAs meet at a final cluster barrier
// before either releases shared or tensor memory.
#include "common.cuh"
#include "sm100.cuh"

namespace mimk {

using namespace sm100;

namespace {

constexpr int BM = 128;          // rows per CTA (256 per pair)
constexpr int BK = 64, STAGES = 6;
constexpr int ACC_COLS = 256;    // TMEM columns per accumulator buffer (two buffers)
constexpr int A_BYTES  = BM * BK * 2;
constexpr int B_BYTES  = 128 * BK * 2;   // this CTA's half of the B tile(s)
constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
constexpr int NUM_THREADS = 192;
constexpr int GROUP_M = 8;       // pair-tiles (256 rows) per raster group: A of a group (32 MiB at K = 8192) stays in L2

struct Bars {
    uint64_t full[STAGES];
    uint64_t empty[STAGES];
    uint64_t acc_full[2];
    uint64_t acc_empty[2];
    uint32_t tmem_base;
    int abort_flag;
};
constexpr int OUT_STAGE_BYTES = 4 * 2 * 4096;  // per epilogue warp: two buffers of 32 rows x 128 bytes for the bulk stores
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + OUT_STAGE_BYTES + 1024 + 256;

// One tensor map per destination matrix (this GPU's C, or every rank's copy of a gathered matrix).
struct OutMaps {
    CUtensorMap m[MIMK_MAX_GATHER];
};
static_assert(sizeof(Bars) <= 256, "barrier block too large");

struct Params {
    int64_t M, N, K;
    int a_panel_k, a_panel_rows;  // A as K-panels: columns per panel (K when A is one matrix) and rows between panels
    // The result tile goes to `n_dst` matrices of leading dimension `ldc`, at column offset `col_off`: one destination
    // (C itself, ldc = N) for an ordinary call; this GPU's and its peers' copies of a gathered matrix when the all-gather
    // of a column-sharded contraction is fused into the epilogue (plain stores to peer-mapped addresses over NVLink).
    void* dst[MIMK_MAX_GATHER];
    int n_dst;
    int64_t ldc, col_off;
    // > 0: a reduce-scatter fused into the epilogue instead. Rows [t scatter_rows, (t + 1) scatter_rows) of the f32 result
    // are ADDED into destination t (an [scatter_rows, N] matrix: this GPU's or a peer's accumulator) by bulk reductions.
    int64_t scatter_rows;
    int64_t tile_rot;  // row tile (of 256 rows) this GPU starts with
    const float* post_row;
    const void* post_full;
    int post;
    int* status;
};

__device__ __forceinline__ uint32_t cluster_ctarank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
// shared::cluster address of the same location in CTA `rank` of this cluster
__device__ __forceinline__ uint32_t map_to_cta(uint32_t saddr, uint32_t rank) {
    uint32_t d;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(d) : "r"(saddr), "r"(rank));
    return d;
}
__device__ __forceinline__ void cluster_sync() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// TMA tile load into this CTA's shared memory whose completion bytes go to a barrier given by its shared::cluster
// address (here: the even CTA's barrier). No multicast: every CTA fetches its own tile.
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap* m, int x, int y, uint32_t bar_cluster) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(dst), "l"(reinterpret_cast<uint64_t>(m)), "r"(bar_cluster), "r"(x), "r"(y)
        : "memory");
}
__device__ __forceinline__ void tmem_alloc_pair(uint32_t smem_result, uint32_t ncols) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_result), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish_pair() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t ncols) {
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void mma_f16_ss_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                                uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// One arrival on the barrier at this shared-memory offset in BOTH CTAs once every MMA issued so far has completed.
__device__ __forceinline__ void mma_commit_pair(uint32_t bar) {
    asm volatile(
        "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
        ::"r"(bar), "h"((unsigned short)3)
        : "memory");
}

// Bulk (TMA) store of a [32 rows x 128 bytes] shared-memory tile to a destination matrix; rows / columns beyond the
// matrix are clipped by the tensor map. x (in elements) times the element size is a multiple of 128 bytes here.
// `rot` rotates the order of the row tiles (0 for an ordinary call): with a fused reduce-scatter every GPU starts at a
// different owner's rows, so that the GPUs do not all send to the same destination at the same time.
__device__ __forceinline__ void tile_coords(int64_t tile, int64_t tiles_m, int64_t tiles_n, int64_t rot, int64_t& tm,
                                            int64_t& tn) {
    const int64_t per_group = GROUP_M * tiles_n;
    const int64_t group     = tile / per_group;
    const int64_t first_m   = group * GROUP_M;
    const int64_t gsize     = (tiles_m - first_m) < GROUP_M ? (tiles_m - first_m) : GROUP_M;
    const int64_t in_group  = tile % per_group;
    tm                      = first_m + in_group % gsize + rot;
    tm                      = tm >= tiles_m ? tm - tiles_m : tm;
    tn                      = in_group / gsize;
}

// BN: output-tile width per B operand (256 plain, 128 gated); this CTA stages BN/2 rows of each B operand.
template <int BN, bool B_MN, bool GATED, class TOut>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(NUM_THREADS, 1)
gemm_tc2_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                const __grid_constant__ CUtensorMap tmB2, const __grid_constant__ OutMaps om, const Params p) {
    constexpr int BH = BN / 2;                 // B rows staged by this CTA, per operand
    constexpr int BH_BYTES = BH * BK * 2;
    static_assert((GATED ? 2 : 1) * BH_BYTES == B_BYTES, "stage layout assumes 16 KiB of B per CTA");
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw_addr  = smem_u32(smem_raw);
    const uint32_t tile_base = (raw_addr + 1023u) & ~1023u;
    Bars* bars = reinterpret_cast<Bars*>(smem_raw + (tile_base - raw_addr) + STAGES * STAGE_BYTES + OUT_STAGE_BYTES);
    volatile int* abort_flag = &bars->abort_flag;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_ctarank();
    const int64_t pair = blockIdx.x >> 1, num_pairs = gridDim.x >> 1;
    const int64_t tiles_m = (p.M + 2 * BM - 1) / (2 * BM), tiles_n = (p.N + BN - 1) / BN;
    const int64_t num_tiles = tiles_m * tiles_n;
    const int num_kb        = int((p.K + BK - 1) / BK);

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(smem_u32(&bars->full[s]), 1);    // used in the even CTA: its producer's expect_tx arrival
            mbar_init(smem_u32(&bars->empty[s]), 1);   // one multicast commit
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(smem_u32(&bars->acc_full[b]), 1);     // one multicast commit
            mbar_init(smem_u32(&bars->acc_empty[b]), 256);  // used in the even CTA: 128 epilogue threads of each CTA
        }
        bars->abort_flag = 0;
        fence_barrier_init();
        tma_prefetch_desc(&tmA);
        tma_prefetch_desc(&tmB);
        if (GATED) tma_prefetch_desc(&tmB2);
    }
    if (warp == 1) {
        tmem_alloc_pair(smem_u32(&bars->tmem_base), 512);
        tmem_relinquish_pair();
    }
    tc_fence_before();
    __syncthreads();
    cluster_sync();  // the peer's barriers are initialised before anything signals them
    tc_fence_after();
    const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(&bars->tmem_base);

    if (warp == 0) {
        // ---------------- TMA producer (both CTAs) ----------------
        if (lane == 0) {
            uint32_t stage = 0, phase = 0;
            bool ok = true;
            for (int64_t tile = pair; tile < num_tiles && ok; tile += num_pairs) {
                int64_t tm, tn;
                tile_coords(tile, tiles_m, tiles_n, p.tile_rot, tm, tn);
                const int m0 = int(tm * 2 * BM) + int(rank) * BM;
                const int n0 = int(tn * BN) + int(rank) * BH;
                for (int kb = 0; kb < num_kb; ++kb) {
                    if (!(ok = mbar_wait(smem_u32(&bars->empty[stage]), phase ^ 1u, abort_flag))) break;
                    const uint32_t full_even = map_to_cta(smem_u32(&bars->full[stage]), 0);
                    const uint32_t sa = tile_base + stage * STAGE_BYTES;
                    const uint32_t sb = sa + A_BYTES;
                    if (rank == 0) mbar_expect_tx(smem_u32(&bars->full[stage]), 2 * STAGE_BYTES);  // both CTAs' bytes
                    const int ka = kb * BK, pa = ka / p.a_panel_k;  // the K-panel of A this k-block lies in
                    tma_load_2d_pair(sa, &tmA, ka - pa * p.a_panel_k, m0 + pa * p.a_panel_rows, full_even);
                    if (!B_MN) {
                        tma_load_2d_pair(sb, &tmB, kb * BK, n0, full_even);
                        if (GATED) tma_load_2d_pair(sb + BH_BYTES, &tmB2, kb * BK, n0, full_even);
                    } else {
#pragma unroll
                        for (int j = 0; j < BH / 64; ++j) {
                            tma_load_2d_pair(sb + j * (BK * 128), &tmB, n0 + j * 64, kb * BK, full_even);
                            if (GATED) tma_load_2d_pair(sb + BH_BYTES + j * (BK * 128), &tmB2, n0 + j * 64, kb * BK, full_even);
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
        // ---------------- MMA issuer (even CTA only) ----------------
        if (lane == 0 && rank == 0) {
            const uint32_t idesc = idesc_bf16_f32(2 * BM, GATED ? 2 * BN : BN, 0, B_MN ? 1 : 0);
            uint32_t stage = 0, phase = 0, acc = 0, acc_phase = 0;
            bool ok = true;
            for (int64_t tile = pair; tile < num_tiles && ok; tile += num_pairs) {
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
                        const uint64_t ad   = smem_desc_sw128(sa + k * 32, 16, 1024);
                        const uint32_t boff = B_MN ? k * 2048 : k * 32;
                        const uint32_t lead = B_MN ? BK * 128 : 16;
                        const uint64_t bd   = smem_desc_sw128(sb + boff, lead, 1024);
                        const uint32_t accum = (kb > 0 || k > 0) ? 1u : 0u;
                        // gated: this CTA's halves of the two B tiles lie back to back in shared memory, so they form one
                        // 128-row half of a 256-wide operand and one instruction feeds both accumulators
                        mma_f16_ss_pair(d0, ad, bd, idesc, accum);
                    }
                    mma_commit_pair(smem_u32(&bars->empty[stage]));
                    if (++stage == STAGES) {
                        stage = 0;
                        phase ^= 1u;
                    }
                }
                if (!ok) break;
                mma_commit_pair(smem_u32(&bars->acc_full[acc]));
                if (++acc == 2) {
                    acc = 0;
                    acc_phase ^= 1u;
                }
            }
        }
    } else {
        // ---------------- epilogue (warps 2..5, both CTAs) ----------------
        // Each warp owns 32 rows of the CTA's 128: accumulator -> registers (tcgen05.ld, one row per thread) -> `post`
        // -> a 128-byte-swizzled [32 x 128 B] tile in shared memory -> one bulk store per destination. Two tiles per warp
        // alternate, so the stores of one chunk drain while the next chunk is converted. No CTA-wide barrier is involved.
        const int quarter = warp & 3;
        constexpr int CW = 128 / int(sizeof(TOut));  // output columns per 128-byte store row: 64 bf16 or 32 f32
        const uint32_t out_base = tile_base + STAGES * STAGE_BYTES + quarter * 2 * 4096;
        uint32_t acc = 0, acc_phase = 0, chunk_no = 0;
        bool ok = true;
        const TOut* post_full = static_cast<const TOut*>(p.post_full);
        for (int64_t tile = pair; tile < num_tiles && ok; tile += num_pairs) {
            int64_t tm, tn;
            tile_coords(tile, tiles_m, tiles_n, p.tile_rot, tm, tn);
            const int64_t row0 = tm * 2 * BM + int64_t(rank) * BM + quarter * 32;
            const int64_t row  = row0 + lane;
            const int64_t n0   = tn * BN;
            if (!(ok = mbar_wait(smem_u32(&bars->acc_full[acc]), acc_phase, abort_flag))) break;
            tc_fence_after();
            const uint32_t t0 = tmem_base + acc * ACC_COLS + (uint32_t(quarter * 32) << 16);
            const uint32_t acc_empty_even = map_to_cta(smem_u32(&bars->acc_empty[acc]), 0);
#pragma unroll 1
            for (int c0 = 0; c0 < BN; c0 += CW, ++chunk_no) {
                const uint32_t buf = out_base + (chunk_no & 1u) * 4096;
                if (lane == 0) bulk_wait_read_1();  // the store that last used this buffer has read it
                __syncwarp();
#pragma unroll
                for (int c = c0; c < c0 + CW; c += 32) {
                    uint32_t r[32];
                    float v[32];
                    // gated accumulator columns: [gate | up] of the even CTA's B rows, then [gate | up] of the odd CTA's
                    const int gc = GATED ? (c / BH) * 2 * BH + (c % BH) : c;
                    tmem_ld_32x32(t0 + gc, r);
                    if (GATED) {
                        uint32_t u[32];
                        tmem_ld_32x32(t0 + gc + BH, u);
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
                        // last read of this accumulator buffer: hand it back to the issuer in the even CTA
                        tc_fence_before();
                        mbar_arrive_cluster(acc_empty_even);
                    }
                    if (p.post != MIMK_POST_ID && row < p.M) {
#pragma unroll
                        for (int i = 0; i < 32; ++i) {
                            const int64_t col = n0 + c + i;
                            if (col < p.N) {
                                const float rowv = p.post_row ? __ldg(p.post_row + col) : 0.f;
                                const float full = post_full ? float(post_full[row * p.N + col]) : 0.f;
                                v[i]             = apply_post(p.post, v[i], rowv, full);
                            }
                        }
                    }
                    // this thread's row of the tile: 16-byte pieces at (piece ^ (row & 7)), the 128-byte swizzle
                    const uint32_t row_addr = buf + lane * 128;
                    if (sizeof(TOut) == 2) {
                        const int piece0 = ((c - c0) * 2) >> 4;  // 32 bf16 = 4 pieces
#pragma unroll
                        for (int i = 0; i < 32; i += 8) {
                            const uint32_t a = row_addr + ((uint32_t(piece0 + (i >> 3)) ^ uint32_t(lane & 7)) << 4);
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
                    if (row0 < p.M && n0 + c0 < p.N) {
                        if (sizeof(TOut) == 4 && p.scatter_rows > 0) {
                            const int64_t owner = row0 / p.scatter_rows;
                            tma_reduce_add_2d(&om.m[owner], buf, int(n0 + c0), int(row0 - owner * p.scatter_rows));
                        } else {
                            for (int t = 0; t < p.n_dst; ++t) tma_store_2d(&om.m[t], buf, int(n0 + c0), int(row0));
                        }
                    }
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
    // Neither CTA may release shared or tensor memory while the other can still touch it: meet first.
    tc_fence_before();
    __syncthreads();
    cluster_sync();
    if (warp == 1) {
        __syncwarp();
        tc_fence_after();
        tmem_dealloc_pair(tmem_base, 512);
    }
    if (threadIdx.x == 0 && *abort_flag) *p.status = MIMK_E_DEVICE_WAIT;
}

template <int BN, bool B_MN, bool GATED, class TOut>
int launch(const CUtensorMap& tA, const CUtensorMap& tB, const CUtensorMap& tB2, const OutMaps& om, const Params& p,
           int sm_count, cudaStream_t s) {
    auto kern = gemm_tc2_kernel<BN, B_MN, GATED, TOut>;
    static bool configured[64] = {};  // per template instance and device: the attribute is a per-device setting
    int dev = 0;
    MIMK_CUDA_TRY(cudaGetDevice(&dev));
    if (!configured[dev & 63]) {
        MIMK_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES));
        configured[dev & 63] = true;
    }
    const int64_t tiles = ((p.M + 2 * BM - 1) / (2 * BM)) * ((p.N + BN - 1) / BN);
    const int64_t pairs = sm_count / 2;
    const int grid      = int(2 * (tiles < pairs ? tiles : pairs));
    kern<<<grid, NUM_THREADS, SMEM_BYTES, s>>>(tA, tB, tB2, om, p);
    return launch_status();
}

}  // namespace

// Worth it only when there are enough 256-row tiles to go round; smaller problems stay on the one-CTA kernel.
int gemm_tc2_supported(const mimk_gemm_desc& d, int gated) {
    if (!gemm_tc_supported(d)) return 0;
    const int bn = gated ? 128 : 256;
    const int64_t tiles = ((d.m + 255) / 256) * ((d.n + bn - 1) / bn);
    return d.m >= 512 && tiles >= 74;
}

int gemm_tc2(const mimk_gemm_desc& d, cudaStream_t s, int gated, const void* b2, const mimk_gather_dst* gather,
             int64_t a_panels, int64_t scatter_rows) {
    int st          = MIMK_OK;
    DeviceInfo* dev = device_info(&st);
    if (!dev) return st;
    const bool b_mn = d.b_layout == MIMK_B_KN;
    const int bh    = gated ? 64 : 128;  // B rows (or columns, MN-major) staged per CTA and operand
    const size_t out_size = d.out_dtype == MIMK_BF16 ? 2 : 4;
    for (int64_t b = 0; b < d.batch; ++b) {
        const uint8_t* A  = static_cast<const uint8_t*>(d.a) + size_t(b * d.stride_a) * 2;
        const uint8_t* B  = static_cast<const uint8_t*>(d.b) + size_t(b * d.stride_b) * 2;
        const uint8_t* B2 = b2 ? static_cast<const uint8_t*>(b2) + size_t(b * d.stride_b) * 2 : B;
        CUtensorMap tA, tB, tB2;
        if (a_panels < 1 || (a_panels > 1 && (d.batch != 1 || d.k % a_panels != 0 || (d.k / a_panels) % BK != 0))) return MIMK_E_UNSUPPORTED;
        const uint64_t kp = uint64_t(d.k / a_panels);  // A as a [panels * m, k / panels] matrix: panel g starts at row g * m
        MIMK_TRY(make_tmap_bf16_2d(&tA, A, kp, uint64_t(d.m) * uint64_t(a_panels), kp * 2, BK, BM));
        if (b_mn) {
            MIMK_TRY(make_tmap_bf16_2d(&tB, B, uint64_t(d.n), uint64_t(d.k), uint64_t(d.n) * 2, 64, BK));
            MIMK_TRY(make_tmap_bf16_2d(&tB2, B2, uint64_t(d.n), uint64_t(d.k), uint64_t(d.n) * 2, 64, BK));
        } else {
            MIMK_TRY(make_tmap_bf16_2d(&tB, B, uint64_t(d.k), uint64_t(d.n), uint64_t(d.k) * 2, BK, uint32_t(bh)));
            MIMK_TRY(make_tmap_bf16_2d(&tB2, B2, uint64_t(d.k), uint64_t(d.n), uint64_t(d.k) * 2, BK, uint32_t(bh)));
        }
        Params p;
        p.M = d.m, p.N = d.n, p.K = d.k;
        p.a_panel_k = a_panels > 1 ? int(kp) : int((d.k + BK - 1) / BK * BK), p.a_panel_rows = a_panels > 1 ? int(d.m) : 0;
        if (gather) {
            if (d.batch != 1) return MIMK_E_UNSUPPORTED;
            p.n_dst = gather->n_dst;
            for (int t = 0; t < gather->n_dst; ++t) p.dst[t] = gather->dst[t];
            p.ldc = gather->ldc, p.col_off = gather->col_off;
            if (scatter_rows > 0 && (gated || d.out_dtype != MIMK_F32 || scatter_rows % 32 != 0 ||
                                     scatter_rows * gather->n_dst != d.m))
                return MIMK_E_UNSUPPORTED;
        } else {
            if (scatter_rows > 0) return MIMK_E_UNSUPPORTED;
            p.n_dst  = 1;
            p.dst[0] = static_cast<uint8_t*>(d.c) + size_t(b * d.stride_c) * out_size;
            p.ldc = d.n, p.col_off = 0;
        }
        p.post_row  = static_cast<const float*>(d.post_row);
        p.post_full = d.post_full ? static_cast<const uint8_t*>(d.post_full) + size_t(b * d.stride_c) * out_size : nullptr;
        p.post      = d.post;
        p.status    = dev->status_dev;
        p.scatter_rows = scatter_rows;
        p.tile_rot     = 0;
        if (scatter_rows > 0) {
            const int64_t tiles_m = (d.m + 2 * BM - 1) / (2 * BM);
            p.tile_rot = ((int64_t(gather->first) % gather->n_dst) * scatter_rows / (2 * BM)) % tiles_m;
        }
        // destination maps: [M, N] windows (row pitch ldc) starting at column col_off, boxes of 32 rows x 128 bytes;
        // [scatter_rows, N] windows when the row blocks are scattered
        OutMaps om;
        for (int t = 0; t < p.n_dst; ++t) {
            const uint8_t* base = static_cast<const uint8_t*>(p.dst[t]) + size_t(p.col_off) * out_size;
            MIMK_TRY(make_tmap_2d(&om.m[t], d.out_dtype == MIMK_F32, base, uint64_t(d.n),
                                  uint64_t(scatter_rows > 0 ? scatter_rows : d.m),
                                  uint64_t(p.ldc) * out_size, uint32_t(128 / out_size), 32));
        }
        for (int t = p.n_dst; t < MIMK_MAX_GATHER; ++t) om.m[t] = om.m[0];
        int rc;
        if (gated) {
            if (d.out_dtype != MIMK_BF16) return MIMK_E_DTYPE;
            rc = b_mn ? launch<128, true, true, __nv_bfloat16>(tA, tB, tB2, om, p, dev->sm_count, s)
                      : launch<128, false, true, __nv_bfloat16>(tA, tB, tB2, om, p, dev->sm_count, s);
        } else if (d.out_dtype == MIMK_BF16) {
            rc = b_mn ? launch<256, true, false, __nv_bfloat16>(tA, tB, tB2, om, p, dev->sm_count, s)
                      : launch<256, false, false, __nv_bfloat16>(tA, tB, tB2, om, p, dev->sm_count, s);
        } else {
            rc = b_mn ? launch<256, true, false, float>(tA, tB, tB2, om, p, dev->sm_count, s)
                      : launch<256, false, false, float>(tA, tB, tB2, om, p, dev->sm_count, s);
        }
        MIMK_TRY(rc);
    }
    return MIMK_OK;
}

}  // namespace mimk
