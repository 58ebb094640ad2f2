// Attention forward on paired SMs: tcgen05.mma with cta_group::2, one query tile per CTA, scores double-buffered.
//
// Same program as attn_tc_p.cu -- `softmax (q * transpose_2d k) * v` (MimIR lit/tensor/attn_exec.mim:20-22) with scale, an
// optional causal mask and batch x heads -- for head_dim 128, bf16. What changes is the shape of the pipeline.
//
// attn_tc_p.cu keeps two query tiles per CTA, each with one score buffer that P overwrites in place: per key tile a
// query tile's chain is softmax -> O += P V -> S = Q K^T -> softmax, so the tensor pipe and the exp2 unit alternate (each
// about 57 % busy). Here a cluster of two CTAs works on 256 consecutive query rows of one head, 128 per CTA:
//   * both contractions are ONE instruction stream issued by the even CTA (M = 256 across the pair). Each CTA stages its
//     own Q tile and only HALF of every K tile (64 keys) and V tile (64 of head_dim): half the shared-memory operand
//     traffic per flop, and room for deeper K / V rings;
//   * tensor memory per CTA: S_a S_b (f32 scores of two consecutive key tiles), O, and P_a P_b (bf16) in columns of their
//     own. S = Q K^T of key tile g+2 is issued as soon as the softmax has READ S of tile g, three to four tiles ahead of
//     the O += P V it feeds, so neither unit waits for the other's round trip;
//   * the two softmax warpgroups of a CTA share its 128 rows: warpgroup b takes key tiles of parity b (one thread per row,
//     the 128 scores of the row in registers). The running maximum travels between them through shared memory (it is
//     known right after the tile's maximum, long before the exponentials are done); each keeps its own partial row sum;
//     O is rescaled -- rarely: only when the maximum grew by more than 2^8 -- by the warpgroup that saw the growth,
//     between two O += P V that the barriers keep apart. The warpgroup of an item's last key tile normalises and stores.
//
//   warp 8 (both CTAs)   TMA producer: Q, then K running four key tiles ahead of V
//   warps 9, 10 (even)   MMA issuers: S = Q K^T and O += P V, one thread each
//   warps 0-3, 4-7       softmax warpgroups 0 and 1
// Work items (head, 256-row block) come from a global counter read by the even CTA's producer, which hands each item to
// both CTAs through shared memory (a store into the peer's slot, then an arrive on the peer's barrier). Barriers live across items;
// every role derives stage and parity from running counts. Every wait is bounded; a CTA that gives up records
// MIMK_E_DEVICE_WAIT, all roles unwind, and both CTAs meet at a cluster barrier before tensor memory is released.
// No TMA multicast: every CTA loads its own tiles from this GPU's memory.
#include <math_constants.h>

#include <cstdio>
#include <cstdlib>
#include <mutex>

#include "common.cuh"
#include "sm100.cuh"
#include "attn_common.cuh"

namespace mimk {

using namespace sm100;
using namespace attn;

namespace {

constexpr int BQ = 128, BKV = 128, HD = 128;
constexpr int ATOM_BYTES = 128 * 64 * 2;   // 128 rows x 64 bf16, one 128-byte-swizzle atom column
constexpr int Q_BYTES  = 2 * ATOM_BYTES;   // this CTA's [128 x 128] query tile
constexpr int KH_BYTES = 2 * 64 * 64 * 2;  // this CTA's 64 keys of a K tile: two atoms of 64 rows x 64 of head_dim
constexpr int KH_ATOM  = 64 * 64 * 2;
constexpr int VH_BYTES = 128 * 64 * 2;     // this CTA's 64 head_dim columns of a V tile: 128 keys x 128 bytes
constexpr int Q_STAGES = 2, K_STAGES = 3, V_STAGES = 4;
constexpr int K_LEAD = 4;                  // key tiles the K loads run ahead of the V loads
constexpr int WORK_SLOTS = 8;
constexpr int NUM_THREADS = 384;
constexpr int PRODUCER_WARP = 8, MMA_WARP = 9;
constexpr int SOFTMAX_REGS = 208, OTHER_REGS = 88, LAUNCH_REGS = 168;
static_assert(2 * 128 * SOFTMAX_REGS + 128 * OTHER_REGS <= LAUNCH_REGS * NUM_THREADS, "setmaxnreg budget exceeds the CTA's registers");
constexpr float RESCALE_THRESHOLD = 8.f;   // log2 units
// tensor-memory columns
constexpr uint32_t COL_S = 0, COL_O = 256, COL_P = 384;

struct Bars {
    // waited on in the even CTA only (transaction bytes or arrivals come from both CTAs)
    uint64_t q_full[Q_STAGES], k_full[K_STAGES], v_full[V_STAGES];
    uint64_t s_free[2], p_full[2], o_empty;
    uint64_t work_empty[WORK_SLOTS];
    // one copy per CTA: s_full / pv_done complete by the MMA thread's multicast commits, the others by this CTA's own threads
    uint64_t q_empty[Q_STAGES], k_empty[K_STAGES], v_empty[V_STAGES];
    uint64_t s_full[2], pv_done[2];
    uint64_t work_full[WORK_SLOTS];
    int work_item[WORK_SLOTS];
    uint32_t tmem_base;
    int abort_flag;
};
static_assert(sizeof(Bars) <= 512, "barrier block too large");
constexpr int OUT_STAGE_BYTES = 8 * 4096;  // per softmax warp: 32 rows x 128 bytes of O on their way to a bulk store
constexpr int TILES_BYTES = Q_STAGES * Q_BYTES + K_STAGES * KH_BYTES + V_STAGES * VH_BYTES + OUT_STAGE_BYTES;
constexpr int EXCH_BYTES  = 2 * 4 * 128 * 4 + 2 * 4 * 128 * 8 + 64;  // running maxima [2][4][128], final (m, l) [2][4][128], flag words
constexpr int SMEM_BYTES  = TILES_BYTES + 512 + EXCH_BYTES + 1024;
static_assert(SMEM_BYTES <= 232448, "more shared memory than a CTA can have");

struct Params {
    int64_t Sq, Sk;
    int BH, num_blocks, head_group, num_items;
    float* lse;
    float scale_log2;  // scale * log2(e)
    int causal;
    int* counter;      // next work item; zeroed before the launch
    int* status;
    long long* trace;  // NULL, or (MIMK_ATTN_TRACE=1) room for time stamps of the first cluster's roles
};

constexpr int COUNTER_SLOTS = 64;
__device__ int g_pair_counters[COUNTER_SLOTS];

// Where bounded waits gave up: [0] = number of records, then up to 40 records of (site, CTA, the role's key-tile counters). Written
// only on the failure path; MIMK_ATTN_DEBUG=1 makes the launcher wait for the kernel and print them to stderr.
__device__ int g_pair_waits[128];
__device__ __noinline__ void note_wait(int site, int extra) {
    if ((threadIdx.x & 31) != 0) return;
    const int i = atomicAdd(&g_pair_waits[0], 1);
    if (i < 40) {
        g_pair_waits[1 + 3 * i] = site;
        g_pair_waits[2 + 3 * i] = int(blockIdx.x);
        g_pair_waits[3 + 3 * i] = extra;
    }
}

struct Item {
    int head, q0, n;  // q0: first query row of the 256-row block; n: key tiles to visit
};
// Items are numbered so that taking them in order is longest-first inside groups of heads: inside a group all heads'
// last (longest, under a causal mask) block comes first, then all second-last, and so on.
__device__ __forceinline__ Item decode_item(const Params& p, int item) {
    Item it;
    const int HG = p.head_group;
    const int per_group = HG * p.num_blocks;
    const int g   = item / per_group;
    const int gsz = (p.BH - g * HG) < HG ? (p.BH - g * HG) : HG;
    const int rr  = item - g * per_group;
    const int blk = p.num_blocks - 1 - rr / gsz;
    it.head       = g * HG + rr % gsz;
    it.q0         = blk * 2 * BQ;
    const int kv_tiles = int((p.Sk + BKV - 1) / BKV);
    const int diag     = 2 * blk + 2;  // key tiles up to the diagonal of the block's second query tile
    it.n               = (p.causal && diag < kv_tiles) ? diag : kv_tiles;
    return it;
}

constexpr int TRACE_ROLES = 6, TRACE_CAP = 1024;  // roles: producer, issuer of S, softmax warpgroup 0 / 1, issuer of O
// A time stamp of one step of one role of the first cluster's CTAs: (code, key tile) and the global timer (ns), stored at the role's own
// running index (plain stores, no atomics: the traced warp is barely disturbed). For reading the pipeline.
__device__ __forceinline__ void trace(const Params& p, int role, uint32_t& idx, int code, uint32_t g) {
#ifndef MIMK_ATTN_PAIR_TRACE
    // compiled out unless asked for: even the untaken branch per step cost the hot loops 8 % (0.562 -> 0.518 ms at 128 heads x 4096)
    (void)p, (void)role, (void)idx, (void)code, (void)g;
#else
    if (p.trace && blockIdx.x < 2 && idx < TRACE_CAP) {
        long long* at = p.trace + ((size_t(blockIdx.x) * TRACE_ROLES + role) * TRACE_CAP + idx) * 2;
        unsigned long long ns;
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(ns));
        at[0] = (static_cast<long long>(code + 100 * int(blockIdx.x)) << 32) | g;
        at[1] = static_cast<long long>(ns);
        ++idx;
    }
#endif
}

// ---- cluster-scope helpers -------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t cluster_ctarank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
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
// Hand-over between warp w of one softmax warpgroup and warp w of the other (they own the same 32 query rows): the
// publisher writes its values, then a running count into a flag word; the consumer spins on the count (bounded) and reads.
// Counts only grow, so a consumer that is late cannot mistake a later publication for an earlier one, and a shared-memory
// flag answers within tens of cycles where a suspended mbarrier wait takes hundreds to wake.
__device__ __forceinline__ void flag_publish(volatile uint32_t* flag, uint32_t count, int lane) {
    __threadfence_block();
    __syncwarp();
    if (lane == 0) *flag = count;
}
__device__ __forceinline__ bool flag_wait(volatile uint32_t* flag, uint32_t count, volatile int* abort_flag) {
    if (*flag >= count) {
        __threadfence_block();
        return true;
    }
    const long long t0 = clock64();
    unsigned spins     = 0;
    while (*flag < count) {
        if ((++spins & 255u) == 0) {
            if (*abort_flag) return false;
            if (clock64() - t0 > WAIT_LIMIT_CYCLES) {
                *abort_flag = 1;
                return false;
            }
        }
    }
    __threadfence_block();
    return true;
}
// Arrive on a barrier of the even CTA without a cluster-scope release: what the hot barriers order is tensor-memory traffic,
// which tcgen05.wait / tcgen05.fence already order; a cluster-scope release costs a memory-barrier stall per arrival.
__device__ __forceinline__ void mbar_arrive_peer(uint32_t cluster_addr) {
    asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
__device__ __forceinline__ void st_cluster_u32(uint32_t cluster_addr, int v) {
    asm volatile("st.shared::cluster.u32 [%0], %1;" ::"r"(cluster_addr), "r"(v) : "memory");
}
// try_wait that also acquires what the other CTA of the cluster released before its arrive
__device__ __forceinline__ bool mbar_try_wait_cl(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}
__device__ __forceinline__ bool mbar_wait_cl(uint32_t bar, uint32_t parity, volatile int* abort_flag) {
    if (mbar_try_wait_cl(bar, parity)) return true;
    const long long t0 = clock64();
    unsigned spins     = 0;
    while (!mbar_try_wait_cl(bar, parity)) {
        if ((++spins & 63u) == 0) {
            if (*abort_flag) return false;
            if (clock64() - t0 > WAIT_LIMIT_CYCLES) {
                *abort_flag = 1;
                return false;
            }
        }
    }
    return true;
}
// TMA tile load into this CTA's shared memory; the completion bytes go to the barrier at `bar_cluster` (a shared::cluster
// address: the even CTA's barrier). No multicast.
__device__ __forceinline__ void tma_load_3d_pair(uint32_t dst, const CUtensorMap* m, int x, int y, int z, uint32_t bar_cluster) {
    asm volatile(
        "cp.async.bulk.tensor.3d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
        ::"r"(dst), "l"(reinterpret_cast<uint64_t>(m)), "r"(bar_cluster), "r"(x), "r"(y), "r"(z)
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
__device__ __forceinline__ void mma_ss_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ void mma_ts_pair(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
        ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// One arrival on the barrier at this shared-memory offset in BOTH CTAs once every MMA issued so far has completed.
__device__ __forceinline__ void commit_pair(uint32_t bar) {
    asm volatile(
        "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
        ::"r"(bar), "h"((unsigned short)3)
        : "memory");
}

// PUBLISH_AT: after how many of a key tile's 128 exponentials the running maximum is handed to the other warpgroup, whose
// own exponentials wait for it. 0 lets both warpgroups' exponentials overlap freely; 128 runs them strictly one after the other
// (the other warpgroup's tensor-memory load and maximum then overlap this one's exponentials: the exp2 unit always has one
// warpgroup at full rate instead of two in lockstep and then none).
template <int PUBLISH_AT>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(NUM_THREADS, 1)
attn_tc_pair_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                    const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmO, const Params p) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw_addr = smem_u32(smem_raw);
    const uint32_t base     = (raw_addr + 1023u) & ~1023u;
    const uint32_t sQ = base, sK = sQ + Q_STAGES * Q_BYTES, sV = sK + K_STAGES * KH_BYTES, sOut = sV + V_STAGES * VH_BYTES;
    uint8_t* gen   = smem_raw + (base - raw_addr) + TILES_BYTES;
    Bars* bars     = reinterpret_cast<Bars*>(gen);
    // Four turns per slot array: a slot is rewritten four publications later, by which time the tensor-core barriers
    // this warp passed in between prove that the partner warp has moved past the tile that read it.
    float* m_sh    = reinterpret_cast<float*>(gen + 512);                     // [2 warpgroups][4 turns][128]
    float2* ml_sh  = reinterpret_cast<float2*>(gen + 512 + 2 * 4 * 128 * 4);  // [2 warpgroups][4 turns][128]
    volatile uint32_t* flags = reinterpret_cast<volatile uint32_t*>(gen + 512 + 2 * 4 * 128 * 4 + 2 * 4 * 128 * 8);  // [2 kinds][2 warpgroups][4 warps]
    volatile int* abort_flag = &bars->abort_flag;
    volatile int* work_item  = bars->work_item;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_ctarank();

    if (threadIdx.x == 0) {
        for (int i = 0; i < Q_STAGES; ++i) {
            mbar_init(smem_u32(&bars->q_full[i]), 1);
            mbar_init(smem_u32(&bars->q_empty[i]), 1);
        }
        for (int i = 0; i < K_STAGES; ++i) {
            mbar_init(smem_u32(&bars->k_full[i]), 1);
            mbar_init(smem_u32(&bars->k_empty[i]), 1);
        }
        for (int i = 0; i < V_STAGES; ++i) {
            mbar_init(smem_u32(&bars->v_full[i]), 1);
            mbar_init(smem_u32(&bars->v_empty[i]), 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(smem_u32(&bars->s_free[b]), 8);   // the four warps of one warpgroup of each CTA
            mbar_init(smem_u32(&bars->p_full[b]), 8);
            mbar_init(smem_u32(&bars->s_full[b]), 1);
            mbar_init(smem_u32(&bars->pv_done[b]), 1);
        }
        mbar_init(smem_u32(&bars->o_empty), 8);
        for (int w = 0; w < WORK_SLOTS; ++w) {
            mbar_init(smem_u32(&bars->work_full[w]), 1);
            // consumers of a slot: even CTA -- the two MMA threads and 8 softmax warps; odd CTA -- its producer and 8 softmax warps
            mbar_init(smem_u32(&bars->work_empty[w]), 19);
        }
        bars->abort_flag = 0;
        for (int i = 0; i < 16; ++i) flags[i] = 0;
        fence_barrier_init();
        tma_prefetch_desc(&tmQ);
        tma_prefetch_desc(&tmK);
        tma_prefetch_desc(&tmV);
        tma_prefetch_desc(&tmO);
    }
    if (warp == MMA_WARP) {
        tmem_alloc_pair(smem_u32(&bars->tmem_base), 512);
        tmem_relinquish_pair();
    }
    tc_fence_before();
    __syncthreads();
    cluster_sync();  // the peer's barriers are initialised before anything signals them
    tc_fence_after();
    const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(&bars->tmem_base);

    if (warp >= 8) {
      asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(OTHER_REGS));
      if (warp == PRODUCER_WARP) {
        // ---------------- work fetch (even CTA) + TMA producer (both CTAs) ----------------
#define DBG_G (k_g * 1000u + v_g)
        if (lane == 0) {
            uint32_t tri = 0;
            uint32_t fetched = 0;          // items taken from the work ring by the K cursor
            bool no_more = false, ok = true;
            uint32_t k_g = 0, v_g = 0;     // key tiles whose K / V load has been issued
            uint32_t k_item = 0, v_item = 0;
            int k_j = 0, v_j = 0;
            Item ki = {0, 0, 0}, vi = {0, 0, 0};
            while (ok) {
                // K cursor: up to K_LEAD key tiles ahead of the V cursor
                while (ok && !no_more && k_g < v_g + K_LEAD) {
                    if (k_j == ki.n) {  // next item
                        const uint32_t slot = fetched % WORK_SLOTS, wph = (fetched / WORK_SLOTS) & 1u;
                        int val;
                        if (rank == 0) {
                            if (!(ok = mbar_wait_cl(smem_u32(&bars->work_empty[slot]), wph ^ 1u, abort_flag))) { note_wait(1, int(DBG_G)); break; }
                            const int item = atomicAdd(p.counter, 1);
                            val            = item >= p.num_items ? -1 : item;
                            work_item[slot] = val;
                            st_cluster_u32(map_to_cta(smem_u32(&bars->work_item[slot]), 1), val);
                            mbar_arrive(smem_u32(&bars->work_full[slot]));
                            mbar_arrive_cluster(map_to_cta(smem_u32(&bars->work_full[slot]), 1));
                        } else {
                            if (!(ok = mbar_wait_cl(smem_u32(&bars->work_full[slot]), wph, abort_flag))) { note_wait(2, int(DBG_G)); break; }
                            val = work_item[slot];
                        }
                        if (val < 0) {
                            no_more = true;
                            break;
                        }
                        ki  = decode_item(p, val);
                        k_j = 0;
                        k_item = fetched++;
                        // this CTA's query tile of the item
                        const uint32_t qs = k_item % Q_STAGES, qph = (k_item / Q_STAGES) & 1u;
                        if (!(ok = mbar_wait(smem_u32(&bars->q_empty[qs]), qph ^ 1u, abort_flag))) { note_wait(3, int(DBG_G)); break; }
                        const uint32_t qf = map_to_cta(smem_u32(&bars->q_full[qs]), 0);
                        if (rank == 0) mbar_expect_tx(smem_u32(&bars->q_full[qs]), 2 * Q_BYTES);
                        tma_load_3d_pair(sQ + qs * Q_BYTES, &tmQ, 0, ki.q0 + int(rank) * BQ, ki.head, qf);
                        tma_load_3d_pair(sQ + qs * Q_BYTES + ATOM_BYTES, &tmQ, 64, ki.q0 + int(rank) * BQ, ki.head, qf);
                    }
                    const uint32_t s = k_g % K_STAGES, ph = (k_g / K_STAGES) & 1u;
                    if (!(ok = mbar_wait(smem_u32(&bars->k_empty[s]), ph ^ 1u, abort_flag))) { note_wait(4, int(DBG_G)); break; }
                    const uint32_t kf = map_to_cta(smem_u32(&bars->k_full[s]), 0);
                    if (rank == 0) mbar_expect_tx(smem_u32(&bars->k_full[s]), 2 * KH_BYTES);
                    const int key0 = k_j * BKV + int(rank) * 64;   // this CTA's half of the tile's keys
                    tma_load_3d_pair(sK + s * KH_BYTES, &tmK, 0, key0, ki.head, kf);
                    tma_load_3d_pair(sK + s * KH_BYTES + KH_ATOM, &tmK, 64, key0, ki.head, kf);
                    trace(p, 0, tri, 30, k_g);
                    ++k_j, ++k_g;
                }
                if (!ok) break;
                if (v_g == k_g) break;  // nothing left: every item's K and V are on their way
                // V cursor
                if (v_j == vi.n) {
                    if (v_g > 0 && rank == 1)  // the odd CTA's producer is a consumer of the work ring: done with the item
                        mbar_arrive_cluster(map_to_cta(smem_u32(&bars->work_empty[(v_item) % WORK_SLOTS]), 0));
                    if (v_g > 0) ++v_item;
                    vi  = decode_item(p, work_item[v_item % WORK_SLOTS]);
                    v_j = 0;
                }
                const uint32_t s = v_g % V_STAGES, ph = (v_g / V_STAGES) & 1u;
                if (!(ok = mbar_wait(smem_u32(&bars->v_empty[s]), ph ^ 1u, abort_flag))) { note_wait(5, int(DBG_G)); break; }
                const uint32_t vf = map_to_cta(smem_u32(&bars->v_full[s]), 0);
                if (rank == 0) mbar_expect_tx(smem_u32(&bars->v_full[s]), 2 * VH_BYTES);
                tma_load_3d_pair(sV + s * VH_BYTES, &tmV, int(rank) * 64, v_j * BKV, vi.head, vf);  // this CTA's half of head_dim
                trace(p, 0, tri, 31, v_g);
                ++v_j, ++v_g;
            }
            // the odd CTA's producer hands back its last item and the slot that said "no more"
            if (rank == 1 && ok) {
                if (v_g > 0) mbar_arrive_cluster(map_to_cta(smem_u32(&bars->work_empty[v_item % WORK_SLOTS]), 0));
                mbar_arrive_cluster(map_to_cta(smem_u32(&bars->work_empty[fetched % WORK_SLOTS]), 0));
            }
        }
      } else if (warp == MMA_WARP) {
#undef DBG_G
        // ---------------- issuer of S = Q K^T (even CTA) ----------------
        // The two contractions have an issuing thread each (this warp and the next): issuing a group of eight instructions
        // and its commit costs a thread about as long as the group runs, so one thread for both was the bottleneck. The
        // streams need no order between them beyond what the barriers give.
#define DBG_G (qk_g)
        if (rank == 0) {
            // the whole warp runs the control flow and one elected lane issues: descriptor arithmetic stays in uniform
            // registers, and the issuing thread must deliver an instruction every 64 clocks on a scheduler it shares
            const bool leader = elect_one();
            const uint32_t idesc_qk = idesc_bf16_f32(2 * BQ, BKV, 0, 0);
            const uint64_t dQ0 = smem_desc_sw128(sQ, 16, 1024), dK0 = smem_desc_sw128(sK, 16, 1024);
            uint32_t tri = 0;
            bool ok = true;
            uint32_t qk_g = 0;
            for (uint32_t item = 0; ok; ++item) {
                const uint32_t slot = item % WORK_SLOTS, wph = (item / WORK_SLOTS) & 1u;
                if (!(ok = mbar_wait(smem_u32(&bars->work_full[slot]), wph, abort_flag))) { note_wait(6, int(DBG_G)); break; }
                const int val = work_item[slot];
                __syncwarp();
                if (leader) mbar_arrive(smem_u32(&bars->work_empty[slot]));  // the item's length is all this warp needs of it
                if (val < 0) break;
                const int n = decode_item(p, val).n;
                if (!(ok = mbar_wait(smem_u32(&bars->q_full[item % Q_STAGES]), (item / Q_STAGES) & 1u, abort_flag))) { note_wait(7, int(DBG_G)); break; }
                const uint64_t qa = dQ0 + uint64_t(((item % Q_STAGES) * Q_BYTES) >> 4);
                for (int j = 0; j < n; ++j, ++qk_g) {
                    const uint32_t b = qk_g & 1u, s = qk_g % K_STAGES;
                    if (!(ok = mbar_wait(smem_u32(&bars->k_full[s]), (qk_g / K_STAGES) & 1u, abort_flag))) { note_wait(8, int(DBG_G)); break; }
                    // the score buffer is free once both CTAs' softmax has read key tile g-2 out of it
                    if (qk_g >= 2 && !(ok = mbar_wait(smem_u32(&bars->s_free[b]), ((qk_g >> 1) - 1u) & 1u, abort_flag))) { note_wait(17, int(DBG_G)); break; }
                    tc_fence_after();
                    const uint64_t kb = dK0 + uint64_t((s * KH_BYTES) >> 4);
                    if (leader) {
#pragma unroll
                        for (int k = 0; k < HD / 16; ++k) {
                            const uint64_t qoff = uint64_t(((k >> 2) * ATOM_BYTES + (k & 3) * 32) >> 4);
                            const uint64_t koff = uint64_t(((k >> 2) * KH_ATOM + (k & 3) * 32) >> 4);
                            mma_ss_pair(tmem_base + COL_S + b * 128, qa + qoff, kb + koff, idesc_qk, k > 0 ? 1u : 0u);
                        }
                        // ONE completion signal per group: the K and Q stages are handed back to the producers by the
                        // softmax threads that see it (a commit costs the issuing thread a few hundred cycles)
                        commit_pair(smem_u32(&bars->s_full[b]));
                    }
                    __syncwarp();
                    trace(p, 1, tri, 1, qk_g);
                }
            }
        }
      } else if (warp == MMA_WARP + 1) {
#undef DBG_G
        // ---------------- issuer of O (+)= P V (even CTA) ----------------
#define DBG_G (pv_g)
        if (rank == 0) {
            const bool leader = elect_one();
            const uint32_t idesc_pv = idesc_bf16_f32(2 * BQ, HD, 0, 1);
            const uint64_t dV0 = smem_desc_sw128(sV, ATOM_BYTES, 1024);
            uint32_t tri = 0;
            bool ok = true;
            uint32_t pv_g = 0;
            for (uint32_t item = 0; ok; ++item) {
                const uint32_t slot = item % WORK_SLOTS, wph = (item / WORK_SLOTS) & 1u;
                if (!(ok = mbar_wait(smem_u32(&bars->work_full[slot]), wph, abort_flag))) { note_wait(9, int(DBG_G)); break; }
                const int val = work_item[slot];
                __syncwarp();
                if (leader) mbar_arrive(smem_u32(&bars->work_empty[slot]));
                if (val < 0) break;
                const int n = decode_item(p, val).n;
                // the item's first O = P V overwrites O: both CTAs have read the previous item's result
                if (item > 0 && !(ok = mbar_wait(smem_u32(&bars->o_empty), (item - 1u) & 1u, abort_flag))) { note_wait(18, int(DBG_G)); break; }
                for (int j = 0; j < n; ++j, ++pv_g) {
                    const uint32_t b = pv_g & 1u, s = pv_g % V_STAGES;
                    if (!(ok = mbar_wait(smem_u32(&bars->v_full[s]), (pv_g / V_STAGES) & 1u, abort_flag))) { note_wait(10, int(DBG_G)); break; }
                    if (!(ok = mbar_wait(smem_u32(&bars->p_full[b]), (pv_g >> 1) & 1u, abort_flag))) { note_wait(16, int(DBG_G)); break; }
                    tc_fence_after();
                    const uint64_t vb = dV0 + uint64_t((s * VH_BYTES) >> 4);
                    if (leader) {
#pragma unroll
                        for (int k = 0; k < BKV / 16; ++k)
                            mma_ts_pair(tmem_base + COL_O, tmem_base + COL_P + b * 64 + k * 8, vb + uint64_t((k * 2048) >> 4), idesc_pv,
                                        (j > 0 || k > 0) ? 1u : 0u);
                        commit_pair(smem_u32(&bars->pv_done[b]));  // the V stage goes back through the softmax thread that sees this
                    }
                    __syncwarp();
                    trace(p, 4, tri, 2, pv_g);
                }
            }
        }
      }
#undef DBG_G
    } else {
        asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(SOFTMAX_REGS));
        // ---------------- softmax + output: warpgroup b takes key tiles of parity b, one thread per query row ----------------
        // (control flow is warp-uniform; every wait's outcome is made warp-uniform too, so that a warp gives up as one)
#define DBG_G (G * 1000u + items)
        const uint32_t b = uint32_t(warp >> 2), ob = b ^ 1u;
        const int quarter = warp & 3;
        const int row = quarter * 32 + lane;
        const uint32_t lane_sel = uint32_t(quarter * 32) << 16;
        const uint32_t tS = tmem_base + COL_S + b * 128 + lane_sel, tO = tmem_base + COL_O + lane_sel;
        const uint32_t tP = tmem_base + COL_P + b * 64 + lane_sel;
        // barriers this thread arrives on in the even CTA
        const uint32_t s_free_bar = map_to_cta(smem_u32(&bars->s_free[b]), 0), p_full_bar = map_to_cta(smem_u32(&bars->p_full[b]), 0);
        const uint32_t o_empty_bar = map_to_cta(smem_u32(&bars->o_empty), 0);
        uint32_t tri = 0;
        uint32_t v_rel = b;      // first key tile of this parity whose V stage has not been handed back yet
        uint32_t pubs_b = 0, pubs_ob = 0;  // end-of-item (m, l) hand-overs so far by this warpgroup / by the other
        volatile uint32_t* m_flag_b  = flags + b * 4 + quarter;       // running maxima published by this warp
        volatile uint32_t* m_flag_ob = flags + ob * 4 + quarter;
        volatile uint32_t* e_flag_b  = flags + 8 + b * 4 + quarter;   // end-of-item hand-overs
        volatile uint32_t* e_flag_ob = flags + 8 + ob * 4 + quarter;
        uint32_t G = 0;          // key tiles of all items so far
        uint32_t items = 0;      // items so far
        bool ok = true;
        for (uint32_t w = 0; ok; ++w) {
            const uint32_t slot = w % WORK_SLOTS, wph = (w / WORK_SLOTS) & 1u;
            if (!(ok = __all_sync(0xffffffffu, mbar_wait_cl(smem_u32(&bars->work_full[slot]), wph, abort_flag)))) { note_wait(11, int(DBG_G)); break; }
            const int val = work_item[slot];
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(map_to_cta(smem_u32(&bars->work_empty[slot]), 0));
            if (val < 0) break;
            const Item it = decode_item(p, val);
            const int n   = it.n;
            const int q0  = it.q0 + int(rank) * BQ;
            const int64_t qi = int64_t(q0) + row;
            float m_mine = -CUDART_INF_F, l_mine = 0.f;  // this warpgroup's own row sum, relative to the maximum it last used
            for (int j = int((G ^ b) & 1u); j < n && ok; j += 2) {
                const uint32_t g = G + uint32_t(j), kseq = g >> 1;
                if (!(ok = __all_sync(0xffffffffu, mbar_wait(smem_u32(&bars->s_full[b]), kseq & 1u, abort_flag)))) { note_wait(12, int(DBG_G)); break; }
                const bool tr = quarter == 0 && lane == 0;
                if (tr) {  // S = Q K^T of this key tile has completed: its K stage (and after the item's last tile its Q stage) is free
                    mbar_arrive(smem_u32(&bars->k_empty[g % K_STAGES]));
                    if (j + 1 == n) mbar_arrive(smem_u32(&bars->q_empty[items % Q_STAGES]));
                }
                if (tr) trace(p, 2 + int(b), tri, 10, g);
                tc_fence_after();
                // the whole score row (128 f32) in registers; the buffer goes back to the tensor core at once
                uint32_t r[BKV];
                tmem_ld_slice(tS, r);
                tmem_ld_slice(tS + 32, r + 32);
                tmem_ld_slice(tS + 64, r + 64);
                tmem_ld_slice(tS + 96, r + 96);
                tmem_ld_wait();
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive_peer(s_free_bar);
                if (tr) trace(p, 2 + int(b), tri, 11, g);
                const int64_t k0 = int64_t(j) * BKV;
                const bool need_mask = (p.causal && k0 + BKV - 1 > q0) || (k0 + BKV > p.Sk);
                if (need_mask) {
                    int64_t limit = p.Sk;  // keys >= limit are masked for this row
                    if (p.causal && qi + 1 < limit) limit = qi + 1;
#pragma unroll
                    for (int i = 0; i < BKV; ++i)
                        if (k0 + i >= limit) r[i] = 0xff800000u;  // -inf: exp2 gives 0
                }
                float mx8[8];
#pragma unroll
                for (int c = 0; c < 8; ++c) {
                    mx8[c] = max3(__uint_as_float(r[16 * c]), __uint_as_float(r[16 * c + 1]), __uint_as_float(r[16 * c + 2]));
#pragma unroll
                    for (int i = 3; i + 1 < 16; i += 2)
                        mx8[c] = max3(mx8[c], __uint_as_float(r[16 * c + i]), __uint_as_float(r[16 * c + i + 1]));
                    mx8[c] = fmaxf(mx8[c], __uint_as_float(r[16 * c + 15]));
                }
                const float mx = max3(max3(mx8[0], mx8[1], mx8[2]), max3(mx8[3], mx8[4], mx8[5]), fmaxf(mx8[6], mx8[7])) *
                                 p.scale_log2;  // scale > 0: max commutes with it
                // the running maximum: from the other warpgroup's previous key tile, grown only past the threshold
                // (the slot a warp writes for key tile g held tile g-4's value, which the partner warp read before it published
                // tile g-3's, which this warp read before tile g-2's ...: the data dependence keeps the two in step)
                float m_prev = -CUDART_INF_F, m_new = mx;
                if (j > 0) {
                    if (!(ok = __all_sync(0xffffffffu, flag_wait(m_flag_ob, ((g - 1u) >> 1) + 1u, abort_flag)))) { note_wait(13, int(DBG_G)); break; }
                    m_prev = m_sh[(ob * 4 + (((g - 1u) >> 1) & 3u)) * 128 + row];
                    m_new  = (mx > m_prev + RESCALE_THRESHOLD) ? mx : m_prev;
                }
                if (tr) trace(p, 2 + int(b), tri, 12, g);
                m_sh[(b * 4 + (kseq & 3u)) * 128 + row] = m_new;
                if (PUBLISH_AT == 0) flag_publish(m_flag_b, kseq + 1u, lane);
                if (j > 0 && __any_sync(0xffffffffu, m_new != m_prev)) {
                    // O still refers to m_prev: once O += P V of the previous key tile has completed (this tile's own is not
                    // issued before this warpgroup hands over P), scale the rows of this warp. tcgen05.ld / st are warp-wide:
                    // rows that need no rescale take part with alpha = 1.
                    if (!(ok = __all_sync(0xffffffffu, mbar_wait(smem_u32(&bars->pv_done[ob]), ((g - 1u) >> 1) & 1u, abort_flag)))) { note_wait(14, int(DBG_G)); break; }
                    tc_fence_after();
                    const float alpha = fast_exp2(m_prev - m_new);
#pragma unroll 1
                    for (int c = 0; c < HD; c += 32) {
                        uint32_t o[32];
                        tmem_ld_slice(tO + c, o);
                        tmem_ld_wait();
#pragma unroll
                        for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
                        tmem_st_32x32_x32(tO + c, o);
                    }
                    tmem_st_wait();
                }
                // p = exp2(s * scale - m) as bf16 pairs, kept in the registers the scores came in (P_b may still be read by the
                // tensor core: O += P V of this warpgroup's previous key tile was issued only when that tile ended)
                const uint64_t sl2 = pack2(p.scale_log2, p.scale_log2), neg_m = pack2(-m_new, -m_new);
                uint64_t sum2[2] = {pack2(0.f, 0.f), pack2(0.f, 0.f)};
#pragma unroll
                for (int i = 0; i < BKV; i += 2) {
                    if (PUBLISH_AT > 0 && PUBLISH_AT < BKV && i == PUBLISH_AT) flag_publish(m_flag_b, kseq + 1u, lane);
                    float xa, xb;
                    unpack2(fma2(pack2(__uint_as_float(r[i]), __uint_as_float(r[i + 1])), sl2, neg_m), xa, xb);
                    const float ea = fast_exp2(xa), eb = fast_exp2(xb);
                    sum2[(i >> 1) & 1] = add2(sum2[(i >> 1) & 1], pack2(ea, eb));
                    r[i >> 1]          = pack_bf16x2(ea, eb);  // slot i/2 <= i: already consumed
                }
                if (tr) trace(p, 2 + int(b), tri, 13, g);
                if (PUBLISH_AT >= BKV) flag_publish(m_flag_b, kseq + 1u, lane);
                // P_b is free once that O += P V has completed -- by now it has had a whole tile's exponentials to do so
                if (g >= 2 && !(ok = __all_sync(0xffffffffu, mbar_wait(smem_u32(&bars->pv_done[b]), (kseq - 1u) & 1u, abort_flag)))) { note_wait(19, int(DBG_G)); break; }
                if (tr && g >= 2 && v_rel <= g - 2u) {  // O += P V of key tile g-2 has completed: its V stage is free
                    mbar_arrive(smem_u32(&bars->v_empty[(g - 2u) % V_STAGES]));
                    v_rel = g;
                }
                if (tr) trace(p, 2 + int(b), tri, 14, g);
                tc_fence_after();
#pragma unroll
                for (int c = 0; c < BKV / 2; c += 16) {
                    uint32_t pk[16];
#pragma unroll
                    for (int i = 0; i < 16; ++i) pk[i] = r[c + i];
                    tmem_st_32x32_x16(tP + c, pk);
                }
                tmem_st_wait();
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive_peer(p_full_bar);
                if (tr) trace(p, 2 + int(b), tri, 15, g);
                {
                    float s0, s1;
                    unpack2(add2(sum2[0], sum2[1]), s0, s1);
                    l_mine = l_mine * fast_exp2(m_mine - m_new) + (s0 + s1);  // first tile of this warpgroup: 0 * 2^-inf = 0
                    m_mine = m_new;
                }
                if (tr) trace(p, 2 + int(b), tri, 16, g);
            }
            if (!ok) break;
            // ---- end of the item: the warpgroup of the last key tile owns the result ----
            const uint32_t last_b = (G + uint32_t(n) - 1u) & 1u;
            if (n >= 2 && b != last_b) {  // hand this warpgroup's partial row sum to the one that owns the result
                ml_sh[(b * 4 + (pubs_b & 3u)) * 128 + row] = make_float2(m_mine, l_mine);
                flag_publish(e_flag_b, ++pubs_b, lane);
            }
            if (b == last_b) {
                float l = l_mine;
                if (n >= 2) {
                    if (!(ok = __all_sync(0xffffffffu, flag_wait(e_flag_ob, pubs_ob + 1u, abort_flag)))) { note_wait(15, int(DBG_G)); break; }
                    const float2 o2 = ml_sh[(ob * 4 + (pubs_ob & 3u)) * 128 + row];
                    ++pubs_ob;
                    l += o2.y * fast_exp2(o2.x - m_mine);  // the last tile's maximum is the largest
                }
                const uint32_t g_last = G + uint32_t(n) - 1u;  // O += P V of the item's last key tile: this warpgroup's own tile
                if (!(ok = __all_sync(0xffffffffu, mbar_wait(smem_u32(&bars->pv_done[b]), (g_last >> 1) & 1u, abort_flag)))) { note_wait(16, int(DBG_G)); break; }
                if (quarter == 0 && lane == 0 && v_rel <= g_last) {
                    mbar_arrive(smem_u32(&bars->v_empty[g_last % V_STAGES]));
                    v_rel = g_last + 2u;
                }
                tc_fence_after();
                uint32_t o[HD];
#pragma unroll
                for (int c = 0; c < HD; c += 32) tmem_ld_slice(tO + c, o + c);
                tmem_ld_wait();
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive_peer(o_empty_bar);  // the next item's first O = P V may overwrite O
                // Normalised rows go out as [32 rows x 64 columns] pieces per warp: registers -> 128-byte-swizzled shared
                // memory -> one bulk store each (rows past seq_q are clipped by the store).
                const float inv = l > 0.f ? 1.f / l : 0.f;
                const uint32_t buf = sOut + uint32_t(warp) * 4096u, row_addr = buf + uint32_t(lane) * 128u;
#pragma unroll
                for (int half = 0; half < 2; ++half) {
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
                    p.lse[int64_t(it.head) * p.Sq + qi] = l > 0.f ? (m_mine + log2f(l)) * 0.6931471805599453f : -CUDART_INF_F;
                if (lane == 0) bulk_wait_read_0();  // the staging piece is rewritten by this warp's next result
                __syncwarp();
            }
            G += uint32_t(n);
            ++items;
        }
        if (lane == 0) bulk_wait_all();  // every store has landed before the CTA may exit
    }

#undef DBG_G
    // ---------------- teardown ----------------
    // Neither CTA may release shared or tensor memory while the other can still touch it: meet first.
    tc_fence_before();
    __syncthreads();
    cluster_sync();
    if (warp == MMA_WARP) {
        __syncwarp();
        tc_fence_after();
        tmem_dealloc_pair(tmem_base, 512);
    }
    if (threadIdx.x == 0 && *abort_flag) *p.status = MIMK_E_DEVICE_WAIT;
}

}  // namespace

int attn_tc_pair_supported(const mimk_attn_desc& d) {
    if (d.dtype != MIMK_BF16 || d.head_dim != 128) return 0;
    if (d.seq_k <= 0 || d.seq_q <= 0) return 0;
    if (d.causal && d.seq_q != d.seq_k) return 0;
    if (d.batch_heads > 65535 || d.seq_q >= (int64_t(1) << 31) || d.seq_k >= (int64_t(1) << 31)) return 0;
    if (!aligned16(d.q) || !aligned16(d.k) || !aligned16(d.v) || !aligned16(d.o)) return 0;
    if (!(d.scale > 0.f)) return 0;
    return 1;
}

static int* wait_records() {
    void* sym = nullptr;
    return cudaGetSymbolAddress(&sym, g_pair_waits) == cudaSuccess ? static_cast<int*>(sym) : nullptr;
}

int attn_tc_pair(const mimk_attn_desc& d, cudaStream_t s) {
    int st          = MIMK_OK;
    DeviceInfo* dev = device_info(&st);
    if (!dev) return st;
    static int* counters[64]      = {};
    static unsigned next_slot[64] = {};
    static bool configured[64]    = {};
    static std::mutex mutex;
    const int di = dev->device & 63;
    int* counter = nullptr;
    {
        std::lock_guard<std::mutex> lock(mutex);
        if (!counters[di]) {
            void* sym = nullptr;
            MIMK_CUDA_TRY(cudaGetSymbolAddress(&sym, g_pair_counters));
            counters[di] = static_cast<int*>(sym);
        }
        if (!configured[di]) {
            MIMK_CUDA_TRY(cudaFuncSetAttribute(attn_tc_pair_kernel<0>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES));
            MIMK_CUDA_TRY(cudaFuncSetAttribute(attn_tc_pair_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES));
            MIMK_CUDA_TRY(cudaFuncSetAttribute(attn_tc_pair_kernel<96>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES));
            MIMK_CUDA_TRY(cudaFuncSetAttribute(attn_tc_pair_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES));
            configured[di] = true;
        }
        counter = counters[di] + (next_slot[di]++ % COUNTER_SLOTS);
    }
    CUtensorMap tQ, tK, tV, tO;
    const uint64_t row = uint64_t(HD) * 2;
    MIMK_TRY(make_tmap_bf16_3d(&tO, d.o, HD, uint64_t(d.seq_q), uint64_t(d.batch_heads), row, uint64_t(d.seq_q) * row, 64, 32));
    MIMK_TRY(make_tmap_bf16_3d(&tQ, d.q, HD, uint64_t(d.seq_q), uint64_t(d.batch_heads), row, uint64_t(d.seq_q) * row, 64, BQ));
    MIMK_TRY(make_tmap_bf16_3d(&tK, d.k, HD, uint64_t(d.seq_k), uint64_t(d.batch_heads), row, uint64_t(d.seq_k) * row, 64, 64));
    MIMK_TRY(make_tmap_bf16_3d(&tV, d.v, HD, uint64_t(d.seq_k), uint64_t(d.batch_heads), row, uint64_t(d.seq_k) * row, 64, BKV));
    Params p;
    p.Sq = d.seq_q, p.Sk = d.seq_k, p.BH = int(d.batch_heads);
    p.lse        = d.lse;
    p.scale_log2 = d.scale * 1.4426950408889634f;
    p.causal     = d.causal;
    p.status     = dev->status_dev;
    const int64_t blocks = (d.seq_q + 2 * BQ - 1) / (2 * BQ);
    if (blocks * d.batch_heads >= (int64_t(1) << 30)) return MIMK_E_UNSUPPORTED;
    p.num_blocks = int(blocks);
    p.head_group = d.causal ? 8 : 1;
    p.num_items  = int(blocks * d.batch_heads);
    p.counter    = counter;
    MIMK_CUDA_TRY(cudaMemsetAsync(p.counter, 0, sizeof(int), s));
    const int pairs = dev->sm_count / 2;
    const int grid  = 2 * (p.num_items < pairs ? p.num_items : pairs);
    static int debug = -1;
    if (debug < 0) {
        const char* e = getenv("MIMK_ATTN_DEBUG");
        debug         = (e && e[0] == '1') ? 1 : 0;
    }
    if (debug) MIMK_CUDA_TRY(cudaMemsetAsync(wait_records(), 0, 128 * sizeof(int), s));
    // Time stamps of the roles: only in a build with -DMIMK_ATTN_PAIR_TRACE, and then only with MIMK_ATTN_TRACE=1
    static int tracing = -1;
    static long long* trace_buf[64] = {};
#ifdef MIMK_ATTN_PAIR_TRACE
    if (tracing < 0) {
        const char* e = getenv("MIMK_ATTN_TRACE");
        tracing       = (e && e[0] == '1') ? 1 : 0;
    }
#else
    tracing = 0;
#endif
    p.trace = nullptr;
    if (tracing) {  // measurement aid only: allocates, and waits for the kernel
        if (!trace_buf[di]) MIMK_CUDA_TRY(cudaMalloc(&trace_buf[di], 2 * TRACE_ROLES * TRACE_CAP * 2 * sizeof(long long)));
        MIMK_CUDA_TRY(cudaMemsetAsync(trace_buf[di], 0, 2 * TRACE_ROLES * TRACE_CAP * 2 * sizeof(long long), s));
        p.trace = trace_buf[di];
    }
    static int publish_at = -1;  // MIMK_ATTN_PUBLISH=0|64|96|128 (for A/B measurements)
    if (publish_at < 0) {
        const char* e = getenv("MIMK_ATTN_PUBLISH");
        publish_at    = e ? atoi(e) : 64;
    }
    switch (publish_at) {
        case 0: attn_tc_pair_kernel<0><<<grid, NUM_THREADS, SMEM_BYTES, s>>>(tQ, tK, tV, tO, p); break;
        case 64: attn_tc_pair_kernel<64><<<grid, NUM_THREADS, SMEM_BYTES, s>>>(tQ, tK, tV, tO, p); break;
        case 96: attn_tc_pair_kernel<96><<<grid, NUM_THREADS, SMEM_BYTES, s>>>(tQ, tK, tV, tO, p); break;
        case 128: attn_tc_pair_kernel<128><<<grid, NUM_THREADS, SMEM_BYTES, s>>>(tQ, tK, tV, tO, p); break;
        default: attn_tc_pair_kernel<64><<<grid, NUM_THREADS, SMEM_BYTES, s>>>(tQ, tK, tV, tO, p); break;
    }
    MIMK_TRY(launch_status());
    if (tracing) {
        static long long host[2 * TRACE_ROLES * TRACE_CAP * 2];
        MIMK_CUDA_TRY(cudaStreamSynchronize(s));
        MIMK_CUDA_TRY(cudaMemcpy(host, trace_buf[di], sizeof(host), cudaMemcpyDeviceToHost));
        for (int r = 0; r < 2 * TRACE_ROLES; ++r)
            for (int i = 0; i < TRACE_CAP; ++i) {
                const long long* at = host + (size_t(r) * TRACE_CAP + i) * 2;
                if (at[1] == 0) break;
                fprintf(stderr, "T %d %d %lld\n", int(at[0] >> 32), int(at[0] & 0xffffffff), at[1]);
            }
    }
    if (debug) {
        int rec[128];
        MIMK_CUDA_TRY(cudaStreamSynchronize(s));
        MIMK_CUDA_TRY(cudaMemcpy(rec, wait_records(), sizeof(rec), cudaMemcpyDeviceToHost));
        for (int i = 0; i < rec[0] && i < 40; ++i)
            fprintf(stderr, "attn_tc_pair: wait site %d gave up in CTA %d (counters %d)\n", rec[1 + 3 * i], rec[2 + 3 * i], rec[3 + 3 * i]);
    }
    return MIMK_OK;
}

}  // namespace mimk
