// C-ABI entry points that only validate and dispatch, plus the per-device state of the library.
#include <cstdlib>
#include <mutex>

#include "common.cuh"
#include "sm100.cuh"

namespace mimk {

static thread_local int g_last_cuda_error = 0;

int note_cuda_error(cudaError_t e) {
    if (e == cudaSuccess) return MIMK_OK;
    g_last_cuda_error = int(e);
    return MIMK_E_CUDA;
}

namespace {
constexpr int MAX_DEVICES = 64;
DeviceInfo g_devices[MAX_DEVICES];
bool g_device_ready[MAX_DEVICES];
std::mutex g_mutex;
}  // namespace

DeviceInfo* device_info(int* status) {
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess || dev < 0 || dev >= MAX_DEVICES) {
        cudaGetLastError();
        *status = MIMK_E_NO_DEVICE;
        return nullptr;
    }
    std::lock_guard<std::mutex> lock(g_mutex);
    DeviceInfo& d = g_devices[dev];
    if (!g_device_ready[dev]) {
        cudaDeviceProp prop;
        if (cudaGetDeviceProperties(&prop, dev) != cudaSuccess) {
            cudaGetLastError();
            *status = MIMK_E_NO_DEVICE;
            return nullptr;
        }
        if (prop.major != 10) {  // the kernels are built for sm_100a only
            *status = MIMK_E_NO_DEVICE;
            return nullptr;
        }
        d.device   = dev;
        d.sm_count = prop.multiProcessorCount;
        d.cc_major = prop.major;
        int* host  = nullptr;
        if (cudaHostAlloc(reinterpret_cast<void**>(&host), 64, cudaHostAllocMapped) != cudaSuccess ||
            cudaHostGetDevicePointer(reinterpret_cast<void**>(&d.status_dev), host, 0) != cudaSuccess) {
            *status = note_cuda_error(cudaGetLastError());
            return nullptr;
        }
        *host              = 0;
        d.status_host      = host;
        g_device_ready[dev] = true;
    }
    return &d;
}

namespace {
int scratch_for(int kind, size_t bytes, void** out, cudaStream_t stream) {
    int st        = MIMK_OK;
    DeviceInfo* d = device_info(&st);
    if (!d) return st;
    std::lock_guard<std::mutex> lock(g_mutex);
    DeviceInfo::Scratch* slots = d->scratch[kind];
    DeviceInfo::Scratch* e     = nullptr;
    for (int i = 0; i < DeviceInfo::SCRATCH_SLOTS && !e; ++i)
        if (slots[i].used && slots[i].stream == stream) e = &slots[i];
    for (int i = 0; i < DeviceInfo::SCRATCH_SLOTS && !e; ++i)
        if (!slots[i].used) e = &slots[i];
    if (!e) {  // every slot belongs to another stream: take over the one used longest ago
        e = &slots[0];
        for (int i = 1; i < DeviceInfo::SCRATCH_SLOTS; ++i)
            if (slots[i].last_use < e->last_use) e = &slots[i];
        MIMK_CUDA_TRY(cudaDeviceSynchronize());  // its stream may still have work queued on the buffer
        if (e->ptr) MIMK_CUDA_TRY(cudaFree(e->ptr));
        *e = DeviceInfo::Scratch{};
    }
    e->used = true, e->stream = stream, e->last_use = ++d->scratch_clock;
    if (e->bytes < bytes) {
        if (e->ptr) {
            MIMK_CUDA_TRY(cudaDeviceSynchronize());  // queued work may still use the old buffer
            MIMK_CUDA_TRY(cudaFree(e->ptr));
            e->ptr = nullptr, e->bytes = 0;
        }
        const size_t want = (bytes + (size_t(1) << 20) - 1) & ~((size_t(1) << 20) - 1);
        MIMK_CUDA_TRY(cudaMalloc(&e->ptr, want));
        e->bytes = want;
    }
    *out = e->ptr;
    return MIMK_OK;
}
}  // namespace

int get_scratch(size_t bytes, void** out, cudaStream_t stream) { return scratch_for(0, bytes, out, stream); }
int get_aux_scratch(size_t bytes, void** out, cudaStream_t stream) { return scratch_for(1, bytes, out, stream); }

}  // namespace mimk

using namespace mimk;

namespace mimk {
// The paired-SM kernel when the problem has enough 256-row tiles, else the one-CTA kernel.
// MIMK_GEMM_2CTA=0 forces the one-CTA kernel, =2 the paired one whenever it can run (for A/B measurements).
int gemm_tc_any(const mimk_gemm_desc& d, cudaStream_t s, int gated, const void* b2, const mimk_gather_dst* gather,
                int64_t a_panels) {
    static int allow_pair = -1;
    if (allow_pair < 0) {
        const char* e = getenv("MIMK_GEMM_2CTA");
        allow_pair    = (e && e[0] == '0') ? 0 : ((e && e[0] == '2') ? 2 : 1);
    }
    // the paired kernel takes one launch per batch entry; long batches go to the one-CTA kernel, which walks
    // (batch, tile) pairs in a single launch
    if (allow_pair == 2 && d.batch <= 64 && gemm_tc_supported(d)) return gemm_tc2(d, s, gated, b2, gather, a_panels);
    if (allow_pair && d.batch <= 64 && gemm_tc2_supported(d, gated)) return gemm_tc2(d, s, gated, b2, gather, a_panels);
    return gemm_tc(d, s, gated, b2, gather, a_panels);
}
}  // namespace mimk

extern "C" const char* mimk_status_str(int status) {
    switch (status) {
        case MIMK_OK: return "ok";
        case MIMK_E_ARG: return "invalid argument";
        case MIMK_E_SHAPE: return "inconsistent shape";
        case MIMK_E_ALIGN: return "misaligned pointer or extent";
        case MIMK_E_DTYPE: return "unsupported element type combination";
        case MIMK_E_CUDA: return "CUDA call failed";
        case MIMK_E_NO_DEVICE: return "no usable sm_100 device";
        case MIMK_E_DEVICE_WAIT: return "bounded device-side wait expired";
        case MIMK_E_UNSUPPORTED: return "unsupported configuration";
        case MIMK_E_WORKSPACE: return "scratch buffer missing or too small";
        default: return "unknown status";
    }
}

extern "C" int mimk_abi_version(void) { return MIMK_ABI_VERSION; }
extern "C" int mimk_last_cuda_error(void) { return g_last_cuda_error; }

extern "C" int mimk_device_check(void) {
    int st = MIMK_OK;
    return device_info(&st) ? MIMK_OK : st;
}

extern "C" int mimk_device_status(void* stream) {
    int st        = MIMK_OK;
    DeviceInfo* d = device_info(&st);
    if (!d) return st;
    MIMK_CUDA_TRY(cudaStreamSynchronize(static_cast<cudaStream_t>(stream)));
    const int flag = *d->status_host;
    *d->status_host = 0;
    // kernels store a status code there: a bounded wait that expired, or an index outside its axis in gather / scatter
    return flag == MIMK_E_SHAPE ? MIMK_E_SHAPE : (flag ? MIMK_E_DEVICE_WAIT : MIMK_OK);
}

static int check_gemm(const mimk_gemm_desc* d) {
    if (!d) return MIMK_E_ARG;
    if (d->batch < 0 || d->m < 0 || d->n < 0 || d->k < 0) return MIMK_E_ARG;
    if (d->in_dtype != MIMK_F32 && d->in_dtype != MIMK_BF16) return MIMK_E_DTYPE;
    if (d->out_dtype != MIMK_F32 && d->out_dtype != MIMK_BF16) return MIMK_E_DTYPE;
    if (d->b_layout != MIMK_B_KN && d->b_layout != MIMK_B_NK) return MIMK_E_ARG;
    if (d->post < MIMK_POST_ID || d->post > MIMK_POST_ADD_FULL) return MIMK_E_ARG;
    if (d->stride_a < 0 || d->stride_b < 0 || d->stride_c < 0) return MIMK_E_ARG;
    const bool needs_row  = d->post == MIMK_POST_BIAS || d->post == MIMK_POST_BIAS_RELU || d->post == MIMK_POST_BIAS_TANH;
    const bool needs_full = d->post == MIMK_POST_ADD_FULL;
    if (needs_row && !d->post_row) return MIMK_E_ARG;
    if (needs_full && !d->post_full) return MIMK_E_ARG;
    if (d->batch > 1 && d->stride_c < d->m * d->n) return MIMK_E_SHAPE;  // output batches must not overlap
    return MIMK_OK;
}

extern "C" int mimk_gemm(const mimk_gemm_desc* d, void* stream) {
    MIMK_TRY(check_gemm(d));
    int st = MIMK_OK;
    if (!device_info(&st)) return st;
    if (d->batch == 0 || d->m == 0 || d->n == 0) return MIMK_OK;
    if (!d->c || (d->k > 0 && (!d->a || !d->b))) return MIMK_E_ARG;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (gemm_tc_supported(*d)) return gemm_tc_any(*d, s, 0, nullptr);
    static int f32_tc = -1;  // MIMK_F32_TC=0 keeps f32 contractions on the CUDA cores (for A/B measurements)
    if (f32_tc < 0) {
        const char* e = getenv("MIMK_F32_TC");
        f32_tc        = (e && e[0] == '0') ? 0 : 1;
    }
    if (f32_tc && gemm_f32_tc_supported(*d) && !gemm_simt_preferred(*d)) return gemm_f32_tc(*d, s);
    return gemm_simt(*d, s);
}

extern "C" int mimk_gemm_gather(const mimk_gemm_desc* d, const void* b2, const mimk_gather_dst* g, void* stream) {
    MIMK_TRY(check_gemm(d));
    if (!g || g->n_dst < 1 || g->n_dst > MIMK_MAX_GATHER || g->ldc < 0 || g->col_off < 0) return MIMK_E_ARG;
    if (g->col_off + d->n > g->ldc) return MIMK_E_SHAPE;
    if (g->ldc % 8 != 0 || g->col_off % 8 != 0) return MIMK_E_ALIGN;  // 16-byte stores into every destination
    for (int t = 0; t < g->n_dst; ++t)
        if (!g->dst[t] || !aligned16(g->dst[t])) return MIMK_E_ARG;
    int st = MIMK_OK;
    if (!device_info(&st)) return st;
    if (d->batch != 1 || d->post_full) return MIMK_E_UNSUPPORTED;
    if (d->m == 0 || d->n == 0) return MIMK_OK;
    if (!d->a || !d->b) return MIMK_E_ARG;
    if (b2 && d->out_dtype != MIMK_BF16) return MIMK_E_DTYPE;
    mimk_gemm_desc dd = *d;
    dd.c              = g->dst[0];  // only its alignment is looked at; the tiles go to g->dst[*]
    if (!gemm_tc_supported(dd)) return MIMK_E_UNSUPPORTED;
    return gemm_tc_any(dd, static_cast<cudaStream_t>(stream), b2 ? 1 : 0, b2, g);
}

extern "C" int mimk_gemm_reduce_scatter(const mimk_gemm_desc* d, const mimk_gather_dst* g, int64_t rows_per_dst,
                                       void* stream) {
    MIMK_TRY(check_gemm(d));
    if (!g || g->n_dst < 1 || g->n_dst > MIMK_MAX_GATHER || g->ldc < 0 || g->col_off < 0 || rows_per_dst < 1) return MIMK_E_ARG;
    if (g->col_off + d->n > g->ldc || rows_per_dst * g->n_dst != d->m) return MIMK_E_SHAPE;
    if (g->ldc % 4 != 0 || g->col_off % 4 != 0 || rows_per_dst % 32 != 0) return MIMK_E_ALIGN;  // 16-byte pieces, 32-row boxes
    for (int t = 0; t < g->n_dst; ++t)
        if (!g->dst[t] || !aligned16(g->dst[t])) return MIMK_E_ARG;
    int st = MIMK_OK;
    if (!device_info(&st)) return st;
    if (d->batch != 1 || d->post_full || d->post_row || d->post != MIMK_POST_ID) return MIMK_E_UNSUPPORTED;
    if (d->out_dtype != MIMK_F32 || d->in_dtype != MIMK_BF16) return MIMK_E_DTYPE;
    if (d->n == 0) return MIMK_OK;
    if (!d->a || !d->b) return MIMK_E_ARG;
    mimk_gemm_desc dd = *d;
    dd.c              = g->dst[0];  // only its alignment is looked at; the tiles go to g->dst[*]
    if (!gemm_tc_supported(dd)) return MIMK_E_UNSUPPORTED;
    return gemm_tc2(dd, static_cast<cudaStream_t>(stream), 0, nullptr, g, 1, rows_per_dst);
}

extern "C" int mimk_gemm_kpanels(const mimk_gemm_desc* d, int64_t panels, void* stream) {
    MIMK_TRY(check_gemm(d));
    if (panels < 1) return MIMK_E_ARG;
    if (panels == 1) return mimk_gemm(d, stream);
    int st = MIMK_OK;
    if (!device_info(&st)) return st;
    if (d->batch != 1 || d->k % panels != 0 || (d->k / panels) % 64 != 0) return MIMK_E_UNSUPPORTED;
    if (d->m == 0 || d->n == 0) return MIMK_OK;
    if (!d->a || !d->b || !d->c) return MIMK_E_ARG;
    if (!gemm_tc_supported(*d)) return MIMK_E_UNSUPPORTED;
    return gemm_tc_any(*d, static_cast<cudaStream_t>(stream), 0, nullptr, nullptr, panels);
}

extern "C" int mimk_gemm_flat(int64_t m, int64_t n, int64_t k, const void* a, const void* b, void* c, int32_t in_dtype,
                              int32_t out_dtype, int32_t b_layout, int32_t post, const void* post_row, void* stream) {
    mimk_gemm_desc d = {};
    d.batch = 1, d.m = m, d.n = n, d.k = k;
    d.a = a, d.b = b, d.c = c;
    d.in_dtype = in_dtype, d.out_dtype = out_dtype, d.b_layout = b_layout, d.post = post;
    d.post_row = post_row;
    return mimk_gemm(&d, stream);
}

extern "C" int mimk_attn_fwd(const mimk_attn_desc* d, void* stream) {
    if (!d) return MIMK_E_ARG;
    if (d->batch_heads < 0 || d->seq_q < 0 || d->seq_k < 0 || d->head_dim < 0) return MIMK_E_ARG;
    if (d->dtype != MIMK_F32 && d->dtype != MIMK_BF16) return MIMK_E_DTYPE;
    int st = MIMK_OK;
    if (!device_info(&st)) return st;
    if (d->batch_heads == 0 || d->seq_q == 0 || d->head_dim == 0) return MIMK_OK;
    if (!d->q || !d->o || (d->seq_k > 0 && (!d->k || !d->v))) return MIMK_E_ARG;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    // bf16 with head_dim 64 or 128 runs on the persistent tensor-core kernel (attn_tc_p.cu). MIMK_ATTN_PAIRED=1 sends head_dim
    // 128 to the paired-SM kernel instead (attn_tc2.cu: cta_group::2, double-buffered scores) -- held to the same tolerance; measured at
    // 128 heads x 4096: 0.56 / 0.92 ms (causal / full) against 0.49 / 0.87 ms here, so it is not the default.
    static int paired = -1;
    if (paired < 0) {
        const char* e = getenv("MIMK_ATTN_PAIRED");
        paired        = (e && e[0] == '1') ? 1 : 0;
    }
    if (paired && attn_tc_pair_supported(*d)) return attn_tc_pair(*d, s);
    if (attn_tc_persistent_supported(*d)) return attn_tc_persistent(*d, s);
    static int composed = -1;  // MIMK_ATTN_COMPOSED=0 keeps every such problem on the one-launch CUDA-core kernel
    if (composed < 0) {
        const char* e = getenv("MIMK_ATTN_COMPOSED");
        composed      = (e && e[0] == '0') ? 0 : 1;
    }
    if (composed && attn_composed_supported(*d)) return attn_composed(*d, s);
    return attn_simt(*d, s);
}

extern "C" int mimk_mlp_gated(const mimk_mlp_desc* d, void* stream) {
    if (!d) return MIMK_E_ARG;
    if (d->m < 0 || d->k < 0 || d->f < 0 || d->n < 0) return MIMK_E_ARG;
    if (d->dtype != MIMK_BF16) return MIMK_E_DTYPE;
    if (d->b_layout != MIMK_B_KN && d->b_layout != MIMK_B_NK) return MIMK_E_ARG;
    int st = MIMK_OK;
    if (!device_info(&st)) return st;
    if (d->m == 0 || d->n == 0) return MIMK_OK;
    if (!d->x || !d->w1 || !d->w3 || !d->w2 || !d->y) return MIMK_E_ARG;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    void* h        = d->h;
    if (!h) MIMK_TRY(get_scratch(size_t(d->m) * size_t(d->f) * 2, &h, static_cast<cudaStream_t>(stream)));
    // stage 1: H = silu(X W1) * (X W3), both contractions in one kernel with two accumulators
    mimk_gemm_desc g1 = {};
    g1.batch = 1, g1.m = d->m, g1.n = d->f, g1.k = d->k;
    g1.a = d->x, g1.b = d->w1, g1.c = h;
    g1.in_dtype = MIMK_BF16, g1.out_dtype = MIMK_BF16, g1.b_layout = d->b_layout, g1.post = MIMK_POST_ID;
    if (!gemm_tc_supported(g1)) return MIMK_E_UNSUPPORTED;
    MIMK_TRY(gemm_tc_any(g1, s, 1, d->w3));
    // stage 2: Y = H W2
    mimk_gemm_desc g2 = {};
    g2.batch = 1, g2.m = d->m, g2.n = d->n, g2.k = d->f;
    g2.a = h, g2.b = d->w2, g2.c = d->y;
    g2.in_dtype = MIMK_BF16, g2.out_dtype = MIMK_BF16, g2.b_layout = d->b_layout, g2.post = MIMK_POST_ID;
    if (gemm_tc_supported(g2)) return gemm_tc_any(g2, s, 0, nullptr);
    return gemm_simt(g2, s);
}

// ---- self-test of the bounded-wait path --------------------------------------------------------------------------
namespace mimk {
namespace {
// Waits on a barrier that nothing will ever arrive on, with a limit of `limit_cycles`, then reports like the real
// kernels do: sets the status word and returns normally. No trap, no fault, no endless loop.
__global__ void wait_expiry_kernel(long long limit_cycles, int* status) {
    __shared__ uint64_t bar;
    __shared__ int abort_flag;
    if (threadIdx.x == 0) {
        sm100::mbar_init(sm100::smem_u32(&bar), 1);
        abort_flag = 0;
        sm100::fence_barrier_init();
    }
    __syncthreads();
    volatile int* af = &abort_flag;
    const bool ok = sm100::mbar_wait_limit(sm100::smem_u32(&bar), 0, af, limit_cycles);
    __syncthreads();
    if (threadIdx.x == 0 && (!ok || *af)) *status = MIMK_E_DEVICE_WAIT;
}
}  // namespace
}  // namespace mimk

extern "C" int mimk_selftest_wait_expiry(int64_t limit_cycles, void* stream) {
    if (limit_cycles < 0 || limit_cycles > 2000000000LL) return MIMK_E_ARG;
    int st        = MIMK_OK;
    DeviceInfo* d = device_info(&st);
    if (!d) return st;
    wait_expiry_kernel<<<1, 64, 0, static_cast<cudaStream_t>(stream)>>>(limit_cycles, d->status_dev);
    return launch_status();
}
