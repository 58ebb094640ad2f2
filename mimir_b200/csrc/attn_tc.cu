// Attention forward on the 5th-generation tensor cores: O = softmax(scale * Q K^T [+ causal mask]) V, bf16 in/out,
// f32 scores, statistics and accumulation, head_dim 128.
//
// The reference computes this as the composed program `softmax (q * transpose_2d k) * v` (MimIR
// lit/tensor/attn_exec.mim:20-22): two contractions around the four-op softmax (tensor.mim:1172-1176) with the whole
// score matrix in memory. Here the score tile never leaves the SM:
//
//   one CTA owns two query tiles of 128 rows of one (batch, head) and walks the key/value tiles of 128 keys
//   warps 0..3    softmax of query tile 0, one thread per row: tcgen05.ld the 128 f32 scores of the row into
//   warps 4..7    softmax of query tile 1   registers, running max / sum, exp2 with the scale folded in, P written
//                 back over S in tensor memory as bf16 (tcgen05.st); O is rescaled in tensor memory only when the
//                 running max has grown by more than 2^8 since the last rescale
//   (registers are moved from the third warpgroup to the two softmax warpgroups with setmaxnreg: 208 vs 88 per thread)
//   warp 8        TMA producer: Q once, then K and V tiles into two-stage rings (128-byte-swizzled shared memory)
//   warp 9        MMA issuer (one thread): S_t = Q_t K^T  (tcgen05.mma, M128 N128 K16 x 8, both operands in shared
//                 memory) and O_t += P_t V (A operand = P_t in tensor memory, B operand = V as an MN-major tile)
//   TMEM (512 columns): S_0 | S_1 | O_0 | O_1, 128 f32 columns each; P_t aliases the first 64 columns of S_t.
// While one tile's warps do their exponentials the tensor core works on the other tile.
// Every mbarrier wait is bounded; on expiry the CTA records MIMK_E_DEVICE_WAIT and unwinds.
#include <math_constants.h>

#include <cstdlib>

#include "common.cuh"
#include "sm100.cuh"
#include "attn_common.cuh"

namespace mimk {

using namespace sm100;
using namespace attn;

namespace {

constexpr int BQ = 128, BKV = 128, HD = 128;
constexpr int TILE_BYTES = 128 * 128 * 2;  // a [128 x 128] bf16 tile = two swizzle atoms of [128 x 64]
constexpr int ATOM_BYTES = TILE_BYTES / 2;
constexpr int KV_STAGES = 2;
constexpr int NUM_THREADS = 384;  // three warpgroups: softmax tile 0, softmax tile 1, {producer, MMA, two idle warps}
constexpr int PRODUCER_WARP = 8, MMA_WARP = 9;
// setmaxnreg moves registers between warpgroups inside what the CTA got at launch (168 per thread under
// __launch_bounds__(384, 1)). An increase that the pool cannot satisfy would block for ever, so the budget is checked
// here: two softmax warpgroups and the producer/MMA warpgroup must fit in 168 * 384 registers.
constexpr int LAUNCH_REGS = 168, SOFTMAX_REGS = 208, OTHER_REGS = 88;
static_assert(2 * 128 * SOFTMAX_REGS + 128 * OTHER_REGS <= LAUNCH_REGS * NUM_THREADS, "setmaxnreg budget exceeds the CTA's registers");
static_assert(SOFTMAX_REGS % 8 == 0 && OTHER_REGS % 8 == 0, "setmaxnreg takes multiples of 8");
constexpr float RESCALE_THRESHOLD = 8.f;  // log2 units
constexpr int HEAD_GROUP = 8;             // heads whose CTAs are interleaved longest-first under a causal mask

struct Bars {
    uint64_t q_full;
    uint64_t k_full[KV_STAGES], k_empty[KV_STAGES];
    uint64_t v_full[KV_STAGES], v_empty[KV_STAGES];
    uint64_t s_full[2], p_half[2], p_full[2], o_full[2];
    uint32_t tmem_base;
    int abort_flag;
};
constexpr int SMEM_BYTES = (2 + 2 * KV_STAGES) * TILE_BYTES + 1024 + 256;
static_assert(sizeof(Bars) <= 256, "barrier block too large");

struct Params {
    int64_t Sq, Sk, BH, num_pairs, head_group;
    __nv_bfloat16* O;
    float* lse;
    float scale_log2;  // scale * log2(e)
    int causal;
    int* status;
};

#ifdef MIMK_TRACE
// Bring-up aid (not built into the library): SM-clock timestamps of one CTA's hand-offs.
__device__ long long g_trace[3][64][8];
#define MIMK_TR(role, iter, ev)                                                            \
    do {                                                                                   \
        if (blockIdx.x == 0 && (iter) < 64) g_trace[role][iter][ev] = clock64(); \
    } while (0)
#else
#define MIMK_TR(role, iter, ev) \
    do {                        \
    } while (0)
#endif

// EMU: how many of every eight PAIRS of exponentials go to the polynomial instead of the special-function unit.
template <int EMU>
__global__ void __launch_bounds__(NUM_THREADS, 1)
attn_tc_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
               const __grid_constant__ CUtensorMap tmV, const Params p) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw_addr = smem_u32(smem_raw);
    const uint32_t base     = (raw_addr + 1023u) & ~1023u;
    const uint32_t sQ = base, sK = base + 2 * TILE_BYTES, sV = sK + KV_STAGES * TILE_BYTES;
    Bars* bars = reinterpret_cast<Bars*>(smem_raw + (base - raw_addr) + (2 + 2 * KV_STAGES) * TILE_BYTES);
    volatile int* abort_flag = &bars->abort_flag;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    // CTAs are handed out in blockIdx order. Heads are taken in groups; inside a group all heads' longest query-tile
    // pair (the last one under a causal mask) comes first, then all second-longest, and so on. Longest-first keeps
    // the tail of a causal launch short, while the CTAs of one head still run close together in time and share its
    // K/V tiles through L2. Measured at batch*heads 128, seq 4096: causal 1027 / 1072 / 1050 / 951 TFLOP/s for groups
    // of 1 / 8 / 32 / 128 heads; without a mask all CTAs are equally long and a group of 1 is best (1244 vs 1230 at 8).
    int head, pair;
    {
        const int64_t HG = p.head_group;
        const int64_t per_group = HG * p.num_pairs;
        const int64_t g = blockIdx.x / per_group, r = blockIdx.x % per_group;
        const int64_t gsz = (p.BH - g * HG) < HG ? (p.BH - g * HG) : HG;
        // the last group may be smaller: its CTAs are numbered with its own size
        const int64_t rr = blockIdx.x - g * per_group;
        pair = int(p.num_pairs - 1 - rr / gsz);
        head = int(g * HG + rr % gsz);
        (void)r;
    }
    int64_t q0[2];
    int n_kv[2];
    const int kv_tiles = int((p.Sk + BKV - 1) / BKV);
    for (int t = 0; t < 2; ++t) {
        q0[t] = int64_t(pair) * 2 * BQ + t * BQ;
        if (q0[t] >= p.Sq) {
            n_kv[t] = 0;
        } else if (p.causal) {
            const int diag = int(q0[t] / BKV) + 1;
            n_kv[t]        = diag < kv_tiles ? diag : kv_tiles;
        } else {
            n_kv[t] = kv_tiles;
        }
    }
    const int n_max = n_kv[0] > n_kv[1] ? n_kv[0] : n_kv[1];

    if (threadIdx.x == 0) {
        mbar_init(smem_u32(&bars->q_full), 1);
        for (int s = 0; s < KV_STAGES; ++s) {
            mbar_init(smem_u32(&bars->k_full[s]), 1);
            mbar_init(smem_u32(&bars->k_empty[s]), 1);
            mbar_init(smem_u32(&bars->v_full[s]), 1);
            mbar_init(smem_u32(&bars->v_empty[s]), 1);
        }
        for (int t = 0; t < 2; ++t) {
            mbar_init(smem_u32(&bars->s_full[t]), 1);
            mbar_init(smem_u32(&bars->p_half[t]), 128);
            mbar_init(smem_u32(&bars->p_full[t]), 128);
            mbar_init(smem_u32(&bars->o_full[t]), 1);
        }
        bars->abort_flag = 0;
        fence_barrier_init();
        tma_prefetch_desc(&tmQ);
        tma_prefetch_desc(&tmK);
        tma_prefetch_desc(&tmV);
    }
    if (warp == MMA_WARP) {
        tmem_alloc(smem_u32(&bars->tmem_base), 512);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(&bars->tmem_base);

    if (warp >= 8) {
      asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(OTHER_REGS));
      if (warp == PRODUCER_WARP) {
        // ---------------- TMA producer ----------------
        if (lane == 0 && n_max > 0) {
            const uint32_t qf = smem_u32(&bars->q_full);
            mbar_expect_tx(qf, (n_kv[1] > 0 ? 2 : 1) * TILE_BYTES);
            for (int t = 0; t < 2; ++t)
                if (n_kv[t] > 0) {
                    tma_load_3d(sQ + t * TILE_BYTES, &tmQ, 0, int(q0[t]), head, qf);
                    tma_load_3d(sQ + t * TILE_BYTES + ATOM_BYTES, &tmQ, 64, int(q0[t]), head, qf);
                }
            bool ok = true;
            for (int j = 0; j < n_max && ok; ++j) {
                const int s = j % KV_STAGES;
                const uint32_t ph = (j / KV_STAGES) & 1;
                if (!(ok = mbar_wait(smem_u32(&bars->k_empty[s]), ph ^ 1u, abort_flag))) break;
                const uint32_t kf = smem_u32(&bars->k_full[s]);
                mbar_expect_tx(kf, TILE_BYTES);
                tma_load_3d(sK + s * TILE_BYTES, &tmK, 0, j * BKV, head, kf);
                tma_load_3d(sK + s * TILE_BYTES + ATOM_BYTES, &tmK, 64, j * BKV, head, kf);
                if (!(ok = mbar_wait(smem_u32(&bars->v_empty[s]), ph ^ 1u, abort_flag))) break;
                const uint32_t vf = smem_u32(&bars->v_full[s]);
                mbar_expect_tx(vf, TILE_BYTES);
                tma_load_3d(sV + s * TILE_BYTES, &tmV, 0, j * BKV, head, vf);
                tma_load_3d(sV + s * TILE_BYTES + ATOM_BYTES, &tmV, 64, j * BKV, head, vf);
            }
        }
    } else if (warp == MMA_WARP) {
        // ---------------- MMA issuer ----------------
        if (lane == 0 && n_max > 0) {
            const uint32_t idesc_qk = idesc_bf16_f32(BQ, BKV, 0, 0);
            const uint32_t idesc_pv = idesc_bf16_f32(BQ, HD, 0, 1);
            bool ok = true;
            // Descriptors are built once; a k-step only adds a byte offset (>> 4) to the start-address field.
            // (consecutive tiles / stages are TILE_BYTES apart, i.e. TILE_BYTES >> 4 in the start-address field)
            static_assert(KV_STAGES == 2, "stage selection below assumes two stages");
            const uint64_t dQ0 = smem_desc_sw128(sQ, 16, 1024), dK0 = smem_desc_sw128(sK, 16, 1024);
            const uint64_t dV0 = smem_desc_sw128(sV, ATOM_BYTES, 1024);
            constexpr uint64_t TILE_STEP = uint64_t(TILE_BYTES >> 4);
            // S_t = Q_t K_j^T: 8 k-steps of 16 over head_dim; atom = k-step / 4, 32 bytes per step inside an atom
            auto issue_qk = [&](int t, int j) {
                const uint64_t qa = dQ0 + (t ? TILE_STEP : 0), kb = dK0 + ((j & 1) ? TILE_STEP : 0);
#pragma unroll
                for (int k = 0; k < HD / 16; ++k) {
                    const uint64_t off = uint64_t(((k >> 2) * ATOM_BYTES + (k & 3) * 32) >> 4);
                    mma_f16_ss(tmem_base + t * 128, qa + off, kb + off, idesc_qk, k > 0 ? 1u : 0u);
                }
                mma_commit(smem_u32(&bars->s_full[t]));
            };
            // O_t (+)= P_t V_j, k-steps [k0, k1) of 16 keys each; P from tensor memory (8 columns of packed bf16 pairs
            // per step), V as an MN-major operand: 16 key rows = 2048 bytes per step, the two 64-wide halves of
            // head_dim are ATOM_BYTES apart
            auto issue_pv = [&](int t, int j, int k0, int k1) {
                const uint64_t vb = dV0 + ((j & 1) ? TILE_STEP : 0);
#pragma unroll
                for (int k = k0; k < k1; ++k)
                    mma_f16_ts(tmem_base + 256 + t * 128, tmem_base + t * 128 + k * 8, vb + uint64_t((k * 2048) >> 4), idesc_pv,
                               (j > 0 || k > 0) ? 1u : 0u);
            };
            ok = mbar_wait(smem_u32(&bars->q_full), 0, abort_flag);
            if (ok) ok = mbar_wait(smem_u32(&bars->k_full[0]), 0, abort_flag);
            if (ok) {
                tc_fence_after();
                for (int t = 0; t < 2; ++t)
                    if (n_kv[t] > 0) issue_qk(t, 0);
                mma_commit(smem_u32(&bars->k_empty[0]));
            }
            for (int j = 0; j < n_max && ok; ++j) {
                const int s = j % KV_STAGES, s1 = (j + 1) % KV_STAGES;
                const uint32_t ph = (j / KV_STAGES) & 1, ph1 = ((j + 1) / KV_STAGES) & 1;
                bool v_ready = false, k_ready = false;
                for (int t = 0; t < 2 && ok; ++t) {
                    if (j >= n_kv[t]) continue;
                    // the first 64 keys of P_t are ready before the rest: start O_t += P_t V on them
                    if (!(ok = mbar_wait(smem_u32(&bars->p_half[t]), j & 1, abort_flag))) break;
                    if (!v_ready) {
                        if (!(ok = mbar_wait(smem_u32(&bars->v_full[s]), ph, abort_flag))) break;
                        v_ready = true;
                    }
                    tc_fence_after();
                    MIMK_TR(2, j, t * 4 + 0);
                    issue_pv(t, j, 0, 4);
                    if (!(ok = mbar_wait(smem_u32(&bars->p_full[t]), j & 1, abort_flag))) break;
                    tc_fence_after();
                    issue_pv(t, j, 4, 8);
                    MIMK_TR(2, j, t * 4 + 1);
                    if (j + 1 == n_kv[t]) mma_commit(smem_u32(&bars->o_full[t]));
                    if (j + 1 < n_kv[t]) {
                        if (!k_ready) {
                            if (!(ok = mbar_wait(smem_u32(&bars->k_full[s1]), ph1, abort_flag))) break;
                            k_ready = true;
                            tc_fence_after();
                        }
                        issue_qk(t, j + 1);
                        MIMK_TR(2, j, t * 4 + 2);
                    }
                }
                if (!ok) break;
                mma_commit(smem_u32(&bars->v_empty[s]));
                if (k_ready) mma_commit(smem_u32(&bars->k_empty[s1]));
            }
        }
      }
    } else {
        asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(SOFTMAX_REGS));
        // ---------------- softmax + output, one thread per query row ----------------
        const int t = warp >> 2;
        const int quarter = warp & 3;
        const int row_in_tile = quarter * 32 + lane;
        const int64_t qi = q0[t] + row_in_tile;
        const uint32_t lane_sel = uint32_t(quarter * 32) << 16;
        const uint32_t tS = tmem_base + t * 128 + lane_sel, tO = tmem_base + 256 + t * 128 + lane_sel;
        float m_used = -CUDART_INF_F, l = 0.f;
        bool ok = true;
        for (int j = 0; j < n_kv[t] && ok; ++j) {
            if (row_in_tile == 0) MIMK_TR(t, j, 0);
            if (!(ok = mbar_wait(smem_u32(&bars->s_full[t]), j & 1, abort_flag))) break;
            tc_fence_after();
            if (row_in_tile == 0) MIMK_TR(t, j, 1);
            const int64_t k0 = int64_t(j) * BKV;
            const bool need_mask = (p.causal && k0 + BKV - 1 > q0[t]) || (k0 + BKV > p.Sk);
            int64_t limit = p.Sk;  // keys >= limit are masked for this row
            if (p.causal && qi + 1 < limit) limit = qi + 1;
            // the whole score row (128 f32) in registers: one round trip to tensor memory
            uint32_t r[BKV];
            tmem_ld_slice(tS, r);
            tmem_ld_slice(tS + 32, r + 32);
            tmem_ld_slice(tS + 64, r + 64);
            tmem_ld_slice(tS + 96, r + 96);
            tmem_ld_wait();
            if (row_in_tile == 0) MIMK_TR(t, j, 2);
            if (need_mask) {
#pragma unroll
                for (int i = 0; i < BKV; ++i)
                    if (k0 + i >= limit) r[i] = 0xff800000u;  // -inf: exp2 gives 0
            }
            // eight independent chains of three-input maxima, then one join
            float mx8[8];
#pragma unroll
            for (int c = 0; c < 8; ++c) {
                mx8[c] = max3(__uint_as_float(r[16 * c]), __uint_as_float(r[16 * c + 1]), __uint_as_float(r[16 * c + 2]));
#pragma unroll
                for (int i = 3; i + 1 < 16; i += 2)
                    mx8[c] = max3(mx8[c], __uint_as_float(r[16 * c + i]), __uint_as_float(r[16 * c + i + 1]));
                mx8[c] = fmaxf(mx8[c], __uint_as_float(r[16 * c + 15]));
            }
            float mx = max3(max3(mx8[0], mx8[1], mx8[2]), max3(mx8[3], mx8[4], mx8[5]), fmaxf(mx8[6], mx8[7])) *
                       p.scale_log2;  // scale > 0: max commutes with it
            if (j == 0) {
                m_used = mx;
            } else if (__any_sync(0xffffffffu, mx > m_used + RESCALE_THRESHOLD)) {
                // tcgen05.ld / tcgen05.st are warp-wide instructions: when ANY row of the warp needs its O rescaled the
                // whole warp takes this path, rows that do not need it with alpha = 1.
                // The previous O_t += P_t V has completed: its commit precedes the one that released S_t.
                const float m_new = (mx > m_used + RESCALE_THRESHOLD) ? mx : m_used;
                const float alpha = fast_exp2(m_used - m_new);
#pragma unroll 1
                for (int c = 0; c < HD; c += 32) {
                    uint32_t o[32];
                    tmem_ld_slice(tO + c, o);
                    tmem_ld_wait();
#pragma unroll
                    for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
                    tmem_st_32x32_x32(tO + c, o);
                }
                l *= alpha;
                m_used = m_new;
            }
            // p = exp2(s * scale - m), row sum, P as bf16 over the first 64 columns of S_t
            if (row_in_tile == 0) MIMK_TR(t, j, 3);
            const uint64_t sl2 = pack2(p.scale_log2, p.scale_log2), neg_m = pack2(-m_used, -m_used);
            uint64_t sum2[2] = {pack2(0.f, 0.f), pack2(0.f, 0.f)};
#pragma unroll
            for (int c = 0; c < BKV; c += 32) {
                uint32_t pk[16];
#pragma unroll
                for (int i = 0; i < 32; i += 2) {
                    float xa, xb, a, b;
                    unpack2(fma2(pack2(__uint_as_float(r[c + i]), __uint_as_float(r[c + i + 1])), sl2, neg_m), xa, xb);
                    if (((i >> 1) & 7) < EMU) {
                        poly_exp2_x2(xa, xb, a, b);
                    } else {
                        a = fast_exp2(xa);
                        b = fast_exp2(xb);
                    }
                    sum2[(i >> 1) & 1] = add2(sum2[(i >> 1) & 1], pack2(a, b));
                    pk[i >> 1]         = pack_bf16x2(a, b);
                }
                if (c == 64) {
                    // keys 0..63 of P_t were stored a whole chunk of exponentials ago, so this wait does not stall:
                    // let the tensor core start on them
                    tmem_st_wait();
                    tc_fence_before();
                    mbar_arrive(smem_u32(&bars->p_half[t]));
                }
                tmem_st_32x32_x16(tS + (c >> 1), pk);
            }
            {
                float s0, s1;
                unpack2(add2(sum2[0], sum2[1]), s0, s1);
                l += s0 + s1;
            }
            if (row_in_tile == 0) MIMK_TR(t, j, 4);
            tmem_st_wait();
            tc_fence_before();
            mbar_arrive(smem_u32(&bars->p_full[t]));
            if (row_in_tile == 0) MIMK_TR(t, j, 5);
        }
        if (ok && n_kv[t] > 0) ok = mbar_wait(smem_u32(&bars->o_full[t]), 0, abort_flag);
        if (ok && n_kv[t] > 0) {
            tc_fence_after();
            const float inv = l > 0.f ? 1.f / l : 0.f;
            __nv_bfloat16* dst = p.O + (int64_t(head) * p.Sq + qi) * HD;
#pragma unroll 1
            for (int c = 0; c < HD; c += 32) {
                uint32_t r[32];
                tmem_ld_slice(tO + c, r);
                tmem_ld_wait();
                if (qi < p.Sq) {
#pragma unroll
                    for (int i = 0; i < 32; i += 8) {
                        uint4 q;
                        q.x = pack_bf16x2(__uint_as_float(r[i]) * inv, __uint_as_float(r[i + 1]) * inv);
                        q.y = pack_bf16x2(__uint_as_float(r[i + 2]) * inv, __uint_as_float(r[i + 3]) * inv);
                        q.z = pack_bf16x2(__uint_as_float(r[i + 4]) * inv, __uint_as_float(r[i + 5]) * inv);
                        q.w = pack_bf16x2(__uint_as_float(r[i + 6]) * inv, __uint_as_float(r[i + 7]) * inv);
                        *reinterpret_cast<uint4*>(dst + c + i) = q;
                    }
                }
            }
            if (p.lse && qi < p.Sq)
                p.lse[int64_t(head) * p.Sq + qi] = l > 0.f ? (m_used + log2f(l)) * 0.6931471805599453f : -CUDART_INF_F;
        }
    }

    // ---------------- teardown ----------------
    tc_fence_before();
    __syncthreads();
    if (warp == MMA_WARP) {
        __syncwarp();
        tc_fence_after();
        tmem_dealloc(tmem_base, 512);
    }
    if (threadIdx.x == 0 && *abort_flag) *p.status = MIMK_E_DEVICE_WAIT;
}

}  // namespace

#ifdef MIMK_TRACE
extern "C" int mimk_debug_attn_trace(long long* host_out) {
    return cudaMemcpyFromSymbol(host_out, g_trace, sizeof(g_trace)) == cudaSuccess ? 0 : 5;
}
#endif

int attn_tc_supported(const mimk_attn_desc& d) {
    if (d.dtype != MIMK_BF16 || d.head_dim != HD) return 0;
    if (d.seq_k <= 0 || d.seq_q <= 0) return 0;
    if (d.causal && d.seq_q != d.seq_k) return 0;
    if (d.batch_heads > 65535 || d.seq_q >= (int64_t(1) << 31) || d.seq_k >= (int64_t(1) << 31)) return 0;
    if (!aligned16(d.q) || !aligned16(d.k) || !aligned16(d.v) || !aligned16(d.o)) return 0;
    if (!(d.scale > 0.f)) return 0;
    return 1;
}

int attn_tc(const mimk_attn_desc& d, cudaStream_t s) {
    int st          = MIMK_OK;
    DeviceInfo* dev = device_info(&st);
    if (!dev) return st;
    CUtensorMap tQ, tK, tV;
    const uint64_t row = HD * 2;
    MIMK_TRY(make_tmap_bf16_3d(&tQ, d.q, HD, uint64_t(d.seq_q), uint64_t(d.batch_heads), row, uint64_t(d.seq_q) * row, 64, BQ));
    MIMK_TRY(make_tmap_bf16_3d(&tK, d.k, HD, uint64_t(d.seq_k), uint64_t(d.batch_heads), row, uint64_t(d.seq_k) * row, 64, BKV));
    MIMK_TRY(make_tmap_bf16_3d(&tV, d.v, HD, uint64_t(d.seq_k), uint64_t(d.batch_heads), row, uint64_t(d.seq_k) * row, 64, BKV));
    // pairs of exponentials sent to the FMA-pipe polynomial, out of every eight (MIMK_ATTN_EMU=0..2 overrides for experiments)
    static int emu = -1;
    if (emu < 0) {
        const char* e = getenv("MIMK_ATTN_EMU");
        emu           = e ? atoi(e) : 0;
        if (emu < 0 || emu > 2) emu = 0;
    }
    static bool configured[64] = {};  // the shared-memory opt-in is a per-device setting
    if (!configured[dev->device & 63]) {
        MIMK_CUDA_TRY(cudaFuncSetAttribute(attn_tc_kernel<0>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES));
        MIMK_CUDA_TRY(cudaFuncSetAttribute(attn_tc_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES));
        MIMK_CUDA_TRY(cudaFuncSetAttribute(attn_tc_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES));
        configured[dev->device & 63] = true;
    }
    Params p;
    p.Sq = d.seq_q, p.Sk = d.seq_k, p.BH = d.batch_heads;
    p.O          = static_cast<__nv_bfloat16*>(d.o);
    p.lse        = d.lse;
    p.scale_log2 = d.scale * 1.4426950408889634f;
    p.causal     = d.causal;
    p.status     = dev->status_dev;
    p.num_pairs = (d.seq_q + 2 * BQ - 1) / (2 * BQ);
    {
        static int hg = -1;
        if (hg < 0) {
            const char* e = getenv("MIMK_ATTN_HEAD_GROUP");
            hg            = e ? atoi(e) : 0;
            if (hg < 1) hg = 0;
        }
        p.head_group = hg ? hg : (d.causal ? HEAD_GROUP : 1);
    }
    if (p.num_pairs * d.batch_heads >= (int64_t(1) << 31)) return MIMK_E_UNSUPPORTED;
    dim3 grid((unsigned)(p.num_pairs * d.batch_heads));
    if (emu == 0)
        attn_tc_kernel<0><<<grid, NUM_THREADS, SMEM_BYTES, s>>>(tQ, tK, tV, p);
    else if (emu == 1)
        attn_tc_kernel<1><<<grid, NUM_THREADS, SMEM_BYTES, s>>>(tQ, tK, tV, p);
    else
        attn_tc_kernel<2><<<grid, NUM_THREADS, SMEM_BYTES, s>>>(tQ, tK, tV, p);
    return launch_status();
}

}  // namespace mimk
