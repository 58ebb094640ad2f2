// Attention forward on the 5th-generation tensor cores: O = softmax(scale * Q K^T [+ causal mask]) V, bf16 in/out,
// f32 scores, statistics and accumulation, head_dim 64 or 128. Persistent: one CTA per SM takes (head, query-tile pair)
// work items from a global counter until none is left, and the hand-over between items is pipelined.
//
// The reference computes this as the composed program `softmax (q * transpose_2d k) * v` (MimIR
// lit/tensor/attn_exec.mim:20-22): two contractions around the four-op softmax (tensor.mim:1172-1176) with the whole
// score matrix in memory. Here the score tile never leaves the SM:
//
//   a work item is two query tiles of 128 rows of one (batch, head); the CTA walks their key/value tiles of 128 keys
//   warps 0..3    softmax of query tile 0, one thread per row: tcgen05.ld the 128 f32 scores of the row into
//   warps 4..7    softmax of query tile 1   registers, running max / sum, exp2 with the scale folded in, P written
//                 back over S in tensor memory as bf16 (tcgen05.st); O is rescaled in tensor memory only when the
//                 running max has grown by more than 2^8 since the last rescale
//   (registers are moved from the third warpgroup to the two softmax warpgroups with setmaxnreg: 208 vs 88 per thread)
//   warp 8        work fetch + TMA producer: Q, then K and V tiles into two-stage rings (128-byte-swizzled shared memory)
//   warp 9        MMA issuer: S_t = Q_t K^T  (tcgen05.mma, M128 N128 K16 x 8, both operands in shared memory) and
//                 O_t += P_t V (A operand = P_t in tensor memory, B operand = V as an MN-major tile). The whole warp
//                 runs the role's control flow and one elected lane issues: descriptor arithmetic then stays in uniform
//                 registers, which matters because the tensor core queues only about two MMAs, so the issuing thread
//                 must deliver one every 64 clocks while sharing its scheduler with two softmax warps (measured: 8
//                 MMAs per 612 clk issued from a one-lane branch, 552 clk this way, 520 clk on an otherwise idle SM).
//                 K / V stages are released by the softmax warps (they observe the completion of every contraction
//                 anyway): each tcgen05.commit less shortens this warp's path from one tile to the next
//   TMEM (512 columns): S_0 | S_1 | O_0 | O_1; P_t aliases the first 64 columns of S_t.
// While one tile's warps do their exponentials the tensor core works on the other tile.
//
// What a one-item CTA would pay per item and this kernel hides: the CTA launch, barrier and tensor-memory set-up, the load
// latency of Q and of the first K/V tiles, the pipeline fill and drain (measured at head_dim 128: 5.8 us per item beside
// 1.84 us per step of 128 keys, i.e. 3.2 steps' worth on items that are 4 to 64 steps long).
//   producer   fetches the next item as soon as the K/V ring has room: its Q tiles are loaded when the last S = Q K^T
//              of the previous item has been issued, its first K/V tiles while the previous item's last steps compute
//   MMA        issues S = Q K^T of the next item's first key tile right behind the previous item's last O += P V; the
//              first O += P V of an item (which overwrites O_t) waits until the previous item's O_t has been read
//   softmax    reads the finished O_t into registers, releases it, then normalises and stores from registers
// Barriers live across items, so every role keeps running counts (K/V tiles, S tiles, P tiles, items per tile) and
// derives stage and parity from them. Every mbarrier wait is bounded; on expiry the CTA records MIMK_E_DEVICE_WAIT and
// unwinds.
#include <math_constants.h>

#include <cstdlib>
#include <mutex>

#include "common.cuh"
#include "sm100.cuh"
#include "attn_common.cuh"

namespace mimk {

using namespace sm100;
using namespace attn;

namespace {

constexpr int BQ = 128, BKV = 128;
constexpr int ATOM_BYTES = 128 * 64 * 2;  // one 128-byte-swizzle atom: 128 rows x 64 bf16
// a [128 rows x head_dim] bf16 tile = head_dim / 64 atoms side by side
__host__ __device__ constexpr int tile_bytes(int hd) { return (hd / 64) * ATOM_BYTES; }
constexpr int KV_STAGES = 2;
constexpr int NUM_THREADS = 384;  // softmax tile 0, softmax tile 1, {producer, MMA, two idle warps}
constexpr int PRODUCER_WARP = 8, MMA_WARP = 9;
// setmaxnreg moves registers between warpgroups inside what the CTA got at launch (168 per thread under
// __launch_bounds__(384, 1)). An increase that the pool cannot satisfy would block for ever, so the budget is checked.
constexpr int LAUNCH_REGS = 168;
template <int SOFTMAX_REGS, int OTHER_REGS>
struct RegSplit {
    static_assert(2 * 128 * SOFTMAX_REGS + 128 * OTHER_REGS <= LAUNCH_REGS * NUM_THREADS, "setmaxnreg budget exceeds the CTA's registers");
    static_assert(SOFTMAX_REGS % 8 == 0 && OTHER_REGS % 8 == 0, "setmaxnreg takes multiples of 8");
};
constexpr float RESCALE_THRESHOLD = 8.f;  // log2 units
constexpr int WORK_SLOTS = 2;
// O_t += P_t V starts when this many keys of P_t are stored; the rest follows behind it. With 96 of 128 the tensor core is
// still busy with the first part when the last 32 keys arrive, and little of the contraction is left behind them.
constexpr int P_FIRST_KEYS = 96;
static_assert(P_FIRST_KEYS % 32 == 0 && P_FIRST_KEYS > 0 && P_FIRST_KEYS < 128, "P is handed over at a 32-key chunk boundary");

struct Bars {
    uint64_t q_full[2], q_empty[2];
    uint64_t k_full[KV_STAGES], k_empty[KV_STAGES];
    uint64_t v_full[KV_STAGES], v_empty[KV_STAGES];
    uint64_t s_full[2], p_half[2], p_full[2], o_full[2], o_empty[2];
    uint64_t work_full[WORK_SLOTS], work_empty[WORK_SLOTS];
    int work_item[WORK_SLOTS];
    uint32_t tmem_base;
    int abort_flag;
};
constexpr int OUT_STAGE_BYTES = 8 * 4096;  // per softmax warp: 32 rows x 128 bytes of O on their way to a bulk store
__host__ __device__ constexpr int smem_bytes(int hd) { return (2 + 2 * KV_STAGES) * tile_bytes(hd) + OUT_STAGE_BYTES + 1024 + 256; }
static_assert(sizeof(Bars) <= 256, "barrier block too large");
static_assert(smem_bytes(128) <= 232448, "more shared memory than a CTA can have");

struct Params {
    int64_t Sq, Sk;
    int BH, num_pairs, head_group, num_items;
    __nv_bfloat16* O;
    float* lse;
    float scale_log2;  // scale * log2(e)
    int causal;
    int* counter;  // [0] next work item, [1] CTAs that have finished: both zero at launch, set back to zero by the last CTA
    int* status;
};

// Work counters of launches in flight: a launch takes the next slot, so launches on different streams do not share one (up
// to COUNTER_SLOTS of them at a time). A slot is two ints, the next item and the number of CTAs that have finished; the
// last CTA to finish sets both back to zero, so no launch has to clear its slot first (a memset node in front of every
// launch costs 2-3 us, which shows on a 70 us launch).
constexpr int COUNTER_SLOTS = 64;
__device__ int g_work_counters[COUNTER_SLOTS][2];

struct Item {
    int head;
    int q0[2];
    int n_kv[2], n_max;
};

// Items are numbered so that taking them in order is longest-first inside groups of heads (the heads of a group share
// the L2 with their K / V streams; all heads at once thrash it): inside a
// group all heads' longest query-tile pair comes first, then all second-longest, and so on.
__device__ __forceinline__ Item decode_item(const Params& p, int item) {
    Item it;
    const int HG = p.head_group;
    const int per_group = HG * p.num_pairs;
    const int g   = item / per_group;
    const int gsz = (p.BH - g * HG) < HG ? (p.BH - g * HG) : HG;  // the last group may be smaller
    const int rr  = item - g * per_group;
    const int pair = p.num_pairs - 1 - rr / gsz;
    it.head        = g * HG + rr % gsz;
    const int kv_tiles = int((p.Sk + BKV - 1) / BKV);
    for (int t = 0; t < 2; ++t) {
        it.q0[t] = pair * 2 * BQ + t * BQ;
        if (it.q0[t] >= p.Sq) {
            it.n_kv[t] = 0;
        } else if (p.causal) {
            const int diag = it.q0[t] / BKV + 1;
            it.n_kv[t]     = diag < kv_tiles ? diag : kv_tiles;
        } else {
            it.n_kv[t] = kv_tiles;
        }
    }
    it.n_max = it.n_kv[0] > it.n_kv[1] ? it.n_kv[0] : it.n_kv[1];
    return it;
}

// HD: head_dim, 64 or 128 (one or two swizzle atoms per tile row; O_t takes HD tensor-memory columns).
template <int HD, int SOFTMAX_REGS, int OTHER_REGS>
__global__ void __launch_bounds__(NUM_THREADS, 1)
attn_tc_persistent_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                          const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmO, const Params p) {
    (void)sizeof(RegSplit<SOFTMAX_REGS, OTHER_REGS>);
    static_assert(HD == 64 || HD == 128, "head_dim 64 or 128");
    constexpr int TILE_BYTES = tile_bytes(HD);
    constexpr int ATOMS = HD / 64;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw_addr = smem_u32(smem_raw);
    const uint32_t base     = (raw_addr + 1023u) & ~1023u;
    const uint32_t sQ = base, sK = base + 2 * TILE_BYTES, sV = sK + KV_STAGES * TILE_BYTES;
    const uint32_t sOut = sV + KV_STAGES * TILE_BYTES;
    Bars* bars = reinterpret_cast<Bars*>(smem_raw + (base - raw_addr) + (2 + 2 * KV_STAGES) * TILE_BYTES + OUT_STAGE_BYTES);
    volatile int* abort_flag = &bars->abort_flag;
    volatile int* work_item  = bars->work_item;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        for (int t = 0; t < 2; ++t) {
            mbar_init(smem_u32(&bars->q_full[t]), 1);
            mbar_init(smem_u32(&bars->q_empty[t]), 1);
            mbar_init(smem_u32(&bars->s_full[t]), 1);
            mbar_init(smem_u32(&bars->p_half[t]), 128);
            mbar_init(smem_u32(&bars->p_full[t]), 128);
            mbar_init(smem_u32(&bars->o_full[t]), 1);
            mbar_init(smem_u32(&bars->o_empty[t]), 128);
        }
        for (int s = 0; s < KV_STAGES; ++s) {
            mbar_init(smem_u32(&bars->k_full[s]), 1);
            mbar_init(smem_u32(&bars->k_empty[s]), 2);  // one release per query tile
            mbar_init(smem_u32(&bars->v_full[s]), 1);
            mbar_init(smem_u32(&bars->v_empty[s]), 2);
        }
        for (int w = 0; w < WORK_SLOTS; ++w) {
            mbar_init(smem_u32(&bars->work_full[w]), 1);
            mbar_init(smem_u32(&bars->work_empty[w]), 9);  // the MMA thread and one lane of each softmax warp
        }
        bars->abort_flag = 0;
        fence_barrier_init();
        tma_prefetch_desc(&tmQ);
        tma_prefetch_desc(&tmK);
        tma_prefetch_desc(&tmV);
        tma_prefetch_desc(&tmO);
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
        // ---------------- work fetch + TMA producer ----------------
        if (lane == 0) {
            uint32_t g = 0;              // K/V tiles loaded so far (stage = g % KV_STAGES)
            uint32_t qc[2] = {0, 0};     // Q tiles loaded so far, per tile slot
            bool ok = true;
            for (uint32_t w = 0; ok; ++w) {
                const uint32_t slot = w % WORK_SLOTS, wph = (w / WORK_SLOTS) & 1u;
                if (!(ok = mbar_wait(smem_u32(&bars->work_empty[slot]), wph ^ 1u, abort_flag))) break;
                const int item  = atomicAdd(p.counter, 1);
                const bool last = item >= p.num_items;
                work_item[slot] = last ? -1 : item;
                mbar_arrive(smem_u32(&bars->work_full[slot]));  // release: the slot's content is visible to the waiters
                if (last) break;
                const Item it = decode_item(p, item);
                for (int t = 0; t < 2 && ok; ++t) {
                    if (it.n_kv[t] == 0) continue;
                    // the previous occupant's last S = Q K^T has been issued and completed
                    if (!(ok = mbar_wait(smem_u32(&bars->q_empty[t]), (qc[t] & 1u) ^ 1u, abort_flag))) break;
                    const uint32_t qf = smem_u32(&bars->q_full[t]);
                    mbar_expect_tx(qf, TILE_BYTES);
#pragma unroll
                    for (int a = 0; a < ATOMS; ++a)
                        tma_load_3d(sQ + t * TILE_BYTES + a * ATOM_BYTES, &tmQ, a * 64, it.q0[t], it.head, qf);
                    ++qc[t];
                }
                for (int j = 0; j < it.n_max && ok; ++j, ++g) {
                    const uint32_t s = g % KV_STAGES, ph = (g / KV_STAGES) & 1u;
                    if (!(ok = mbar_wait(smem_u32(&bars->k_empty[s]), ph ^ 1u, abort_flag))) break;
                    const uint32_t kf = smem_u32(&bars->k_full[s]);
                    mbar_expect_tx(kf, TILE_BYTES);
#pragma unroll
                    for (int a = 0; a < ATOMS; ++a)
                        tma_load_3d(sK + s * TILE_BYTES + a * ATOM_BYTES, &tmK, a * 64, j * BKV, it.head, kf);
                    if (!(ok = mbar_wait(smem_u32(&bars->v_empty[s]), ph ^ 1u, abort_flag))) break;
                    const uint32_t vf = smem_u32(&bars->v_full[s]);
                    mbar_expect_tx(vf, TILE_BYTES);
#pragma unroll
                    for (int a = 0; a < ATOMS; ++a)
                        tma_load_3d(sV + s * TILE_BYTES + a * ATOM_BYTES, &tmV, a * 64, j * BKV, it.head, vf);
                }
            }
        }
      } else if (warp == MMA_WARP) {
        // ---------------- MMA issuer ----------------
        // One thread issues both tiles' contractions in the fixed order tile 0, tile 1, tile 0, ...: that order is what
        // keeps the two softmax warpgroups half a period apart (two independent issuing threads fall into step, and
        // then the exponentials of both tiles and the contractions of both tiles take turns instead of overlapping).
        // The K / V stages are released by the softmax warps, which see the completion of these contractions anyway:
        // every tcgen05.commit less shortens this thread's path from one tile to the next.
        {
            const bool leader = elect_one();  // the lane that issues; everything else below is warp-uniform
            const uint32_t idesc_qk = idesc_bf16_f32(BQ, BKV, 0, 0);
            const uint32_t idesc_pv = idesc_bf16_f32(BQ, HD, 0, 1);
            static_assert(KV_STAGES == 2, "stage selection below assumes two stages");
            const uint64_t dQ0 = smem_desc_sw128(sQ, 16, 1024), dK0 = smem_desc_sw128(sK, 16, 1024);
            const uint64_t dV0 = smem_desc_sw128(sV, ATOM_BYTES, 1024);
            constexpr uint64_t TILE_STEP = uint64_t(TILE_BYTES >> 4);
            // S_t = Q_t K^T with K in ring stage `stage`: 8 k-steps of 16 over head_dim
            auto issue_qk = [&](int t, uint32_t stage) {
                const uint64_t qa = dQ0 + (t ? TILE_STEP : 0), kb = dK0 + (stage ? TILE_STEP : 0);
                if (leader) {
#pragma unroll
                    for (int k = 0; k < HD / 16; ++k) {
                        const uint64_t off = uint64_t(((k >> 2) * ATOM_BYTES + (k & 3) * 32) >> 4);
                        mma_f16_ss(tmem_base + t * 128, qa + off, kb + off, idesc_qk, k > 0 ? 1u : 0u);
                    }
                    mma_commit(smem_u32(&bars->s_full[t]));
                }
                __syncwarp();
            };
            // O_t (+)= P_t V with V in ring stage `stage`, k-steps [k0, k1) of 16 keys; `first` = first key tile of the item
            auto issue_pv = [&](int t, uint32_t stage, bool first, int k0, int k1) {
                const uint64_t vb = dV0 + (stage ? TILE_STEP : 0);
                if (leader) {
#pragma unroll
                    for (int k = k0; k < k1; ++k)
                        mma_f16_ts(tmem_base + 256 + t * 128, tmem_base + t * 128 + k * 8, vb + uint64_t((k * 2048) >> 4), idesc_pv,
                                   (!first || k > 0) ? 1u : 0u);
                }
                __syncwarp();
            };
            auto commit  = [&](uint64_t* bar) { if (leader) mma_commit(smem_u32(bar)); };
            auto release = [&](uint64_t* bar) { if (leader) mbar_arrive(smem_u32(bar)); };
            uint32_t g = 0;                // K/V tiles consumed so far
            uint32_t qc0 = 0, qc1 = 0;     // items in which tile slot t took part (parity of q_full / o_empty)
            uint32_t pc0 = 0, pc1 = 0;     // P tiles consumed per tile slot (parity of p_half / p_full)
            bool ok = true;
            for (uint32_t w = 0; ok; ++w) {
                const uint32_t slot = w % WORK_SLOTS, wph = (w / WORK_SLOTS) & 1u;
                if (!(ok = mbar_wait(smem_u32(&bars->work_full[slot]), wph, abort_flag))) break;
                const int item = work_item[slot];
                __syncwarp();  // every lane has read the slot
                release(&bars->work_empty[slot]);
                if (item < 0) break;
                const Item it = decode_item(p, item);
                const int n0 = it.n_kv[0], n1 = it.n_kv[1], n_max = it.n_max;  // scalars: nothing below indexes an array by tile
                if (n_max == 0) continue;
                // first key tile: S_t = Q_t K_0^T for both tiles
                if (n0 > 0) ok = mbar_wait(smem_u32(&bars->q_full[0]), qc0 & 1u, abort_flag);
                if (ok && n1 > 0) ok = mbar_wait(smem_u32(&bars->q_full[1]), qc1 & 1u, abort_flag);
                if (ok) ok = mbar_wait(smem_u32(&bars->k_full[g % KV_STAGES]), (g / KV_STAGES) & 1u, abort_flag);
                if (!ok) break;
                tc_fence_after();
                if (n0 > 0) {
                    issue_qk(0, g % KV_STAGES);
                    if (n0 == 1) commit(&bars->q_empty[0]);  // the item's only S for this tile
                } else {
                    release(&bars->k_empty[g % KV_STAGES]);  // in place of the warpgroup that has no tile
                }
                if (n1 > 0) {
                    issue_qk(1, g % KV_STAGES);
                    if (n1 == 1) commit(&bars->q_empty[1]);
                } else {
                    release(&bars->k_empty[g % KV_STAGES]);
                }
                for (int j = 0; j < n_max && ok; ++j) {
                    const uint32_t gj = g + uint32_t(j);
                    const uint32_t s = gj % KV_STAGES, s1 = (gj + 1) % KV_STAGES;
                    const uint32_t ph = (gj / KV_STAGES) & 1u, ph1 = ((gj + 1) / KV_STAGES) & 1u;
                    bool v_ready = false, k_ready = false;
                    // one key tile of one query tile: O_t += P_t V_j, then S_t = Q_t K_{j+1}^T
                    auto tile_step = [&](const int t, const int n_kv, const uint32_t qc, uint32_t& pc) -> bool {
                        if (j >= n_kv) {
                            // this tile has no key tile j (and none after it): pass the V stage of tile j and the K stage
                            // of tile j + 1 on in its warpgroup's place, once they are filled (a release before that
                            // could complete the PREVIOUS phase of the barrier)
                            if (!v_ready) {
                                if (!mbar_wait(smem_u32(&bars->v_full[s]), ph, abort_flag)) return false;
                                v_ready = true;
                            }
                            release(&bars->v_empty[s]);
                            if (j + 1 < n_max) {
                                if (!k_ready) {
                                    if (!mbar_wait(smem_u32(&bars->k_full[s1]), ph1, abort_flag)) return false;
                                    k_ready = true;
                                    tc_fence_after();
                                }
                                release(&bars->k_empty[s1]);
                            }
                            return true;
                        }
                        // the item's first O_t = P V overwrites O_t: the previous item's result must have been read
                        if (j == 0 && !mbar_wait(smem_u32(&bars->o_empty[t]), (qc & 1u) ^ 1u, abort_flag)) return false;
                        // the first keys of P_t are ready before the rest: start O_t += P_t V on them
                        if (!mbar_wait(smem_u32(&bars->p_half[t]), pc & 1u, abort_flag)) return false;
                        if (!v_ready) {
                            if (!mbar_wait(smem_u32(&bars->v_full[s]), ph, abort_flag)) return false;
                            v_ready = true;
                        }
                        tc_fence_after();
                        issue_pv(t, s, j == 0, 0, P_FIRST_KEYS / 16);
                        if (!mbar_wait(smem_u32(&bars->p_full[t]), pc & 1u, abort_flag)) return false;
                        tc_fence_after();
                        issue_pv(t, s, j == 0, P_FIRST_KEYS / 16, BKV / 16);
                        ++pc;
                        if (j + 1 == n_kv) {
                            commit(&bars->o_full[t]);
                            // the other tile goes on: K of tile j + 1 is passed on in this warpgroup's place
                            if (j + 1 < n_max) {
                                if (!k_ready) {
                                    if (!mbar_wait(smem_u32(&bars->k_full[s1]), ph1, abort_flag)) return false;
                                    k_ready = true;
                                    tc_fence_after();
                                }
                                release(&bars->k_empty[s1]);
                            }
                        } else {
                            if (!k_ready) {
                                if (!mbar_wait(smem_u32(&bars->k_full[s1]), ph1, abort_flag)) return false;
                                k_ready = true;
                                tc_fence_after();
                            }
                            issue_qk(t, s1);
                            // the item's last S for this tile: its Q buffer may be refilled once this has completed
                            if (j + 2 == n_kv) commit(&bars->q_empty[t]);
                        }
                        return true;
                    };
                    ok = tile_step(0, n0, qc0, pc0);
                    if (ok) ok = tile_step(1, n1, qc1, pc1);
                }
                g += uint32_t(n_max);
                qc0 += n0 > 0 ? 1u : 0u;
                qc1 += n1 > 0 ? 1u : 0u;
            }
        }
      }
    } else {
        asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(SOFTMAX_REGS));
        // ---------------- softmax + output, one thread per query row ----------------
        const int t = warp >> 2;
        const int quarter = warp & 3;
        const int row_in_tile = quarter * 32 + lane;
        const uint32_t lane_sel = uint32_t(quarter * 32) << 16;
        const uint32_t tS = tmem_base + t * 128 + lane_sel, tO = tmem_base + 256 + t * 128 + lane_sel;
        uint32_t sc = 0;  // S tiles consumed so far by this tile slot (parity of s_full)
        uint32_t oc = 0;  // items in which this tile slot took part (parity of o_full)
        uint32_t g  = 0;  // K/V tiles of all items so far (stage of the K / V barriers this warpgroup releases)
        const bool releaser = quarter == 0 && lane == 0;
        bool ok = true;
        for (uint32_t w = 0; ok; ++w) {
            const uint32_t slot = w % WORK_SLOTS, wph = (w / WORK_SLOTS) & 1u;
            if (!(ok = mbar_wait(smem_u32(&bars->work_full[slot]), wph, abort_flag))) break;
            const int item = work_item[slot];
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&bars->work_empty[slot]));
            if (item < 0) break;
            const Item it = decode_item(p, item);
            const int n_kv = t ? it.n_kv[1] : it.n_kv[0];
            const int q0   = t ? it.q0[1] : it.q0[0];
            if (n_kv == 0) {
                g += uint32_t(it.n_max);
                continue;
            }
            const int64_t qi = int64_t(q0) + row_in_tile;
            float m_used = -CUDART_INF_F, l = 0.f;
            for (int j = 0; j < n_kv && ok; ++j, ++sc) {
                if (!(ok = mbar_wait(smem_u32(&bars->s_full[t]), sc & 1u, abort_flag))) break;
                tc_fence_after();
                // S_t of key tile j is complete, and with it everything this tile's MMA thread issued before it: the K
                // stage of tile j and the V stage of tile j - 1 have been read for this query tile
                if (releaser) {
                    mbar_arrive(smem_u32(&bars->k_empty[(g + uint32_t(j)) % KV_STAGES]));
                    if (j > 0) mbar_arrive(smem_u32(&bars->v_empty[(g + uint32_t(j) - 1u) % KV_STAGES]));
                }
                const int64_t k0 = int64_t(j) * BKV;
                const bool need_mask = (p.causal && k0 + BKV - 1 > q0) || (k0 + BKV > p.Sk);
                int64_t limit = p.Sk;  // keys >= limit are masked for this row
                if (p.causal && qi + 1 < limit) limit = qi + 1;
                // the whole score row (128 f32) in registers: one round trip to tensor memory
                uint32_t r[BKV];
                uint32_t pk[16];
                const uint64_t sl2 = pack2(p.scale_log2, p.scale_log2);
                uint64_t sum2[2]   = {pack2(0.f, 0.f), pack2(0.f, 0.f)};
                auto mask_chunk = [&](const int c) {
#pragma unroll
                    for (int i = 0; i < 32; ++i)
                        if (k0 + c + i >= limit) r[c + i] = 0xff800000u;  // -inf: exp2 gives 0
                };
                // p = exp2(s * scale - m) for keys [c, c + 32) of the row, added to the row sum, packed as bf16 into pk
                auto exp_chunk = [&](const int c, const float m_ref) {
                    const uint64_t neg_m = pack2(-m_ref, -m_ref);
#pragma unroll
                    for (int i = 0; i < 32; i += 2) {
                        float xa, xb;
                        unpack2(fma2(pack2(__uint_as_float(r[c + i]), __uint_as_float(r[c + i + 1])), sl2, neg_m), xa, xb);
                        const float a = fast_exp2(xa), b = fast_exp2(xb);
                        sum2[(i >> 1) & 1] = add2(sum2[(i >> 1) & 1], pack2(a, b));
                        pk[i >> 1]         = pack_bf16x2(a, b);
                    }
                };
                // two independent chains of three-input maxima per 32 keys, eight in all, then one join
                float mx8[8];
                auto max_chunk = [&](const int c) {
#pragma unroll
                    for (int h = 0; h < 2; ++h) {
                        const int b = c + 16 * h;
                        float m = max3(__uint_as_float(r[b]), __uint_as_float(r[b + 1]), __uint_as_float(r[b + 2]));
#pragma unroll
                        for (int i = 3; i + 1 < 16; i += 2) m = max3(m, __uint_as_float(r[b + i]), __uint_as_float(r[b + i + 1]));
                        mx8[(c >> 4) + h] = fmaxf(m, __uint_as_float(r[b + 15]));
                    }
                };
                tmem_ld_slice(tS, r);
                tmem_ld_slice(tS + 32, r + 32);
                tmem_ld_slice(tS + 64, r + 64);
                tmem_ld_slice(tS + 96, r + 96);
                tmem_ld_wait();
                if (need_mask) {
                    mask_chunk(0);
                    mask_chunk(32);
                    mask_chunk(64);
                    mask_chunk(96);
                }
                max_chunk(0);
                max_chunk(32);
                max_chunk(64);
                max_chunk(96);
                float mx = max3(max3(mx8[0], mx8[1], mx8[2]), max3(mx8[3], mx8[4], mx8[5]), fmaxf(mx8[6], mx8[7])) *
                           p.scale_log2;  // scale > 0: max commutes with it
                if (j == 0) {
                    m_used = mx;
                } else if (__any_sync(0xffffffffu, mx > m_used + RESCALE_THRESHOLD)) {
                    // tcgen05.ld / tcgen05.st are warp-wide: when ANY row of the warp needs its O rescaled the whole warp
                    // takes this path, rows that do not need it with alpha = 1. The previous O_t += P_t V has completed:
                    // its commit precedes the one that released S_t.
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
                // P as bf16 over the first 64 columns of S_t
#pragma unroll
                for (int c = 0; c < BKV; c += 32) {
                    exp_chunk(c, m_used);
                    if (c == P_FIRST_KEYS) {
                        // the first keys of P_t were stored a whole chunk of exponentials ago, so this wait does not stall:
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
                tmem_st_wait();
                tc_fence_before();
                mbar_arrive(smem_u32(&bars->p_full[t]));
            }
            if (!ok) break;
            if (!(ok = mbar_wait(smem_u32(&bars->o_full[t]), oc & 1u, abort_flag))) break;
            ++oc;
            tc_fence_after();
            if (releaser) mbar_arrive(smem_u32(&bars->v_empty[(g + uint32_t(n_kv) - 1u) % KV_STAGES]));  // the last O_t += P_t V has read its V stage
            g += uint32_t(it.n_max);
            // the finished row of O_t into registers, then hand O_t back: the next item's first O_t = P V may overwrite it
            uint32_t o[HD];
#pragma unroll
            for (int c = 0; c < HD; c += 32) tmem_ld_slice(tO + c, o + c);
            tmem_ld_wait();
            tc_fence_before();
            mbar_arrive(smem_u32(&bars->o_empty[t]));
            // Normalised rows go out as [32 rows x 64 columns] pieces (one per 64 of head_dim) per warp: registers -> 128-byte-swizzled shared
            // memory -> one bulk store each (rows past seq_q are clipped by the store). A row-per-thread store straight
            // to global memory would touch 32 different lines per instruction.
            const float inv = l > 0.f ? 1.f / l : 0.f;
            const uint32_t buf = sOut + uint32_t(warp) * 4096u, row_addr = buf + uint32_t(lane) * 128u;
#pragma unroll
            for (int half = 0; half < ATOMS; ++half) {
                if (half > 0) {
                    if (lane == 0) bulk_wait_read_0();  // the first piece has left shared memory
                    __syncwarp();
                }
#pragma unroll
                for (int i = 0; i < 64; i += 8) {
                    const uint32_t* v = o + half * 64 + i;
                    const uint32_t a  = row_addr + ((uint32_t(i >> 3) ^ uint32_t(lane & 7)) << 4);
                    asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(a),
                                 "r"(pack_bf16x2(__uint_as_float(v[0]) * inv, __uint_as_float(v[1]) * inv)),
                                 "r"(pack_bf16x2(__uint_as_float(v[2]) * inv, __uint_as_float(v[3]) * inv)),
                                 "r"(pack_bf16x2(__uint_as_float(v[4]) * inv, __uint_as_float(v[5]) * inv)),
                                 "r"(pack_bf16x2(__uint_as_float(v[6]) * inv, __uint_as_float(v[7]) * inv))
                                 : "memory");
                }
                fence_proxy_async_smem();  // the bulk store reads shared memory through the async proxy
                __syncwarp();
                if (lane == 0) {
                    tma_store_3d(&tmO, buf, half * 64, q0 + quarter * 32, it.head);
                    bulk_commit();
                }
            }
            if (p.lse && qi < p.Sq)
                p.lse[int64_t(it.head) * p.Sq + qi] = l > 0.f ? (m_used + log2f(l)) * 0.6931471805599453f : -CUDART_INF_F;
            // the staging piece is rewritten by this warp's next item: its last store must have read it by then
            if (lane == 0) bulk_wait_read_0();
            __syncwarp();
        }
        if (lane == 0) bulk_wait_all();  // every store has landed before the CTA may exit
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
    // every role of this CTA is past its last use of the work counter
    if (threadIdx.x == 0 && atomicAdd(p.counter + 1, 1) == int(gridDim.x) - 1) {
        p.counter[0] = 0;
        p.counter[1] = 0;
    }
}

template <int HD>
int launch_persistent(const CUtensorMap& tQ, const CUtensorMap& tK, const CUtensorMap& tV, const CUtensorMap& tO, const Params& p,
                      int grid, cudaStream_t s) {
    static bool configured[64] = {};  // per template instance and device: the shared-memory opt-in is a per-device setting
    int dev = 0;
    MIMK_CUDA_TRY(cudaGetDevice(&dev));
    if (!configured[dev & 63]) {
        MIMK_CUDA_TRY(cudaFuncSetAttribute(attn_tc_persistent_kernel<HD, 208, 88>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes(HD)));
        configured[dev & 63] = true;
    }
    attn_tc_persistent_kernel<HD, 208, 88><<<grid, NUM_THREADS, smem_bytes(HD), s>>>(tQ, tK, tV, tO, p);
    return launch_status();
}

}  // namespace

int attn_tc_persistent_supported(const mimk_attn_desc& d) {
    if (d.dtype != MIMK_BF16 || (d.head_dim != 64 && d.head_dim != 128)) return 0;
    if (d.seq_k <= 0 || d.seq_q <= 0) return 0;
    if (d.causal && d.seq_q != d.seq_k) return 0;
    if (d.batch_heads > 65535 || d.seq_q >= (int64_t(1) << 31) || d.seq_k >= (int64_t(1) << 31)) return 0;
    if (!aligned16(d.q) || !aligned16(d.k) || !aligned16(d.v) || !aligned16(d.o)) return 0;
    if (!(d.scale > 0.f)) return 0;
    return 1;
}

int attn_tc_persistent(const mimk_attn_desc& d, cudaStream_t s) {
    int st          = MIMK_OK;
    DeviceInfo* dev = device_info(&st);
    if (!dev) return st;
    // per device: the counters' address and the shared-memory opt-in
    static int* counters[64]  = {};
    static unsigned next_slot[64] = {};
    static std::mutex mutex;
    const int di = dev->device & 63;
    int* counter = nullptr;
    {
        std::lock_guard<std::mutex> lock(mutex);
        if (!counters[di]) {
            void* sym = nullptr;
            MIMK_CUDA_TRY(cudaGetSymbolAddress(&sym, g_work_counters));
            counters[di] = static_cast<int*>(sym);
        }
        counter = counters[di] + 2 * (next_slot[di]++ % COUNTER_SLOTS);
    }
    CUtensorMap tQ, tK, tV, tO;
    const uint64_t HD  = uint64_t(d.head_dim);
    const uint64_t row = HD * 2;
    MIMK_TRY(make_tmap_bf16_3d(&tO, d.o, HD, uint64_t(d.seq_q), uint64_t(d.batch_heads), row, uint64_t(d.seq_q) * row, 64, 32));
    MIMK_TRY(make_tmap_bf16_3d(&tQ, d.q, HD, uint64_t(d.seq_q), uint64_t(d.batch_heads), row, uint64_t(d.seq_q) * row, 64, BQ));
    MIMK_TRY(make_tmap_bf16_3d(&tK, d.k, HD, uint64_t(d.seq_k), uint64_t(d.batch_heads), row, uint64_t(d.seq_k) * row, 64, BKV));
    MIMK_TRY(make_tmap_bf16_3d(&tV, d.v, HD, uint64_t(d.seq_k), uint64_t(d.batch_heads), row, uint64_t(d.seq_k) * row, 64, BKV));
    Params p;
    p.Sq = d.seq_q, p.Sk = d.seq_k, p.BH = int(d.batch_heads);
    p.O          = static_cast<__nv_bfloat16*>(d.o);
    p.lse        = d.lse;
    p.scale_log2 = d.scale * 1.4426950408889634f;
    p.causal     = d.causal;
    p.status     = dev->status_dev;
    const int64_t pairs = (d.seq_q + 2 * BQ - 1) / (2 * BQ);
    if (pairs * d.batch_heads >= (int64_t(1) << 30)) return MIMK_E_UNSUPPORTED;
    p.num_pairs  = int(pairs);
    p.head_group = d.causal ? 8 : 1;
    p.num_items  = int(pairs * d.batch_heads);
    p.counter = counter;
    const int grid = int(p.num_items < dev->sm_count ? p.num_items : dev->sm_count);
    return d.head_dim == 64 ? launch_persistent<64>(tQ, tK, tV, tO, p, grid, s) : launch_persistent<128>(tQ, tK, tV, tO, p, grid, s);
}

}  // namespace mimk
