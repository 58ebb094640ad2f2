// Host-buffer entry points: upload, run, download.
//
// They stand in for the wrapper the reference emits around every GPU-lowered operation (MimIR
// src/mim/plug/gpu/phase/lower_map_reduce.cpp:317-395: gpu.buf_alloc_copy per input, gpu.alloc.block for the
// output, gpu.launch, gpu.buf_copy_to_host, gpu.free -- all blocking on the null stream). Here the device buffers
// come from a cached arena, copies are asynchronous, and every operator is cut into pieces that travel through three
// streams -- `up` (host to device copies), `work` (kernels) and `down` (device to host copies), ordered by events -- so
// that the upload of piece i+1, the kernel on piece i and the download of piece i-1 overlap: row blocks for the
// row-wise operators, row panels of A and C for a contraction (B resident), groups of heads for attention, row panels
// of the result for the gated MLP. A call that fails part-way drains all three streams before it returns, so no copy
// to or from the caller's buffers is left in flight.
#include <mutex>

#include "common.cuh"

namespace mimk {
namespace {

struct HostCtx {
    bool ready = false;
    void* arena = nullptr;
    size_t arena_bytes = 0;
    cudaStream_t up = nullptr, work = nullptr, down = nullptr;
    static constexpr int MAX_EVENTS = 64;
    cudaEvent_t uploaded[MAX_EVENTS], computed[MAX_EVENTS], drained[MAX_EVENTS];
};
HostCtx g_ctx[64];
std::mutex g_host_mutex;

int get_ctx(HostCtx** out) {
    int st          = MIMK_OK;
    DeviceInfo* dev = device_info(&st);
    if (!dev) return st;
    HostCtx& c = g_ctx[dev->device];
    if (!c.ready) {
        MIMK_CUDA_TRY(cudaStreamCreateWithFlags(&c.up, cudaStreamNonBlocking));
        MIMK_CUDA_TRY(cudaStreamCreateWithFlags(&c.work, cudaStreamNonBlocking));
        MIMK_CUDA_TRY(cudaStreamCreateWithFlags(&c.down, cudaStreamNonBlocking));
        for (int i = 0; i < HostCtx::MAX_EVENTS; ++i) {
            MIMK_CUDA_TRY(cudaEventCreateWithFlags(&c.uploaded[i], cudaEventDisableTiming));
            MIMK_CUDA_TRY(cudaEventCreateWithFlags(&c.computed[i], cudaEventDisableTiming));
            MIMK_CUDA_TRY(cudaEventCreateWithFlags(&c.drained[i], cudaEventDisableTiming));
        }
        c.ready = true;
    }
    *out = &c;
    return MIMK_OK;
}

int arena(HostCtx& c, size_t bytes, uint8_t** out) {
    if (c.arena_bytes < bytes) {
        if (c.arena) {
            MIMK_CUDA_TRY(cudaDeviceSynchronize());
            MIMK_CUDA_TRY(cudaFree(c.arena));
            c.arena = nullptr, c.arena_bytes = 0;
        }
        size_t want = (bytes + (size_t(1) << 21) - 1) & ~((size_t(1) << 21) - 1);
        MIMK_CUDA_TRY(cudaMalloc(&c.arena, want));
        c.arena_bytes = want;
    }
    *out = static_cast<uint8_t*>(c.arena);
    return MIMK_OK;
}

inline size_t round256(size_t b) { return (b + 255) & ~size_t(255); }

// Ends a host call: waits for everything queued on the three streams (also after a failure in the middle, so that no
// asynchronous copy still touches the caller's buffers) and folds in the device status word.
int finish(HostCtx& c, int st) {
    const cudaError_t e0 = cudaStreamSynchronize(c.up), e1 = cudaStreamSynchronize(c.work), e2 = cudaStreamSynchronize(c.down);
    if (st != MIMK_OK) {
        mimk_device_status(c.work);  // clear the word; the first failure is what the caller hears
        return st;
    }
    if (e0 != cudaSuccess) return note_cuda_error(e0);
    if (e1 != cudaSuccess) return note_cuda_error(e1);
    if (e2 != cudaSuccess) return note_cuda_error(e2);
    return mimk_device_status(c.work);
}

// The event ring: piece b uses slot b % MAX_EVENTS of each event array. Before a slot is recorded again, the host waits
// for the download that last used it, so an event is never re-recorded while a stream still waits on it.
int ring_guard(HostCtx& c, int64_t b) {
    if (b >= HostCtx::MAX_EVENTS) MIMK_CUDA_TRY(cudaEventSynchronize(c.drained[int(b % HostCtx::MAX_EVENTS)]));
    return MIMK_OK;
}

}  // namespace
}  // namespace mimk

using namespace mimk;

extern "C" int mimk_host_register(void* ptr, uint64_t bytes) {
    if (!ptr) return MIMK_E_ARG;
    MIMK_CUDA_TRY(cudaHostRegister(ptr, bytes, cudaHostRegisterDefault));
    return MIMK_OK;
}
extern "C" int mimk_host_unregister(void* ptr) {
    if (!ptr) return MIMK_E_ARG;
    MIMK_CUDA_TRY(cudaHostUnregister(ptr));
    return MIMK_OK;
}
extern "C" int mimk_host_release(void) {
    std::lock_guard<std::mutex> lock(g_host_mutex);
    HostCtx* c = nullptr;
    MIMK_TRY(get_ctx(&c));
    if (c->arena) {
        MIMK_CUDA_TRY(cudaDeviceSynchronize());
        MIMK_CUDA_TRY(cudaFree(c->arena));
        c->arena = nullptr, c->arena_bytes = 0;
    }
    return MIMK_OK;
}

namespace {
int host_rows_body(HostCtx* c, int kind, const void* x, const void* gamma, void* y, void* y2, int in_dtype, int out_dtype,
                   int64_t rows, int64_t cols, float eps) {
    const bool both = kind == 3;
    const size_t in_row = size_t(cols) * dtype_size(in_dtype), out_row = size_t(cols) * dtype_size(out_dtype);
    // Row blocks of about 32 MiB of input: small enough to overlap, large enough to fill the machine.
    int64_t block_rows = int64_t((size_t(32) << 20) / in_row);
    if (block_rows < 1) block_rows = 1;
    block_rows = (block_rows + 3) & ~int64_t(3);
    if (block_rows > rows) block_rows = rows;
    const int64_t nblocks = (rows + block_rows - 1) / block_rows;
    const int slots       = nblocks < 3 ? int(nblocks) : 3;  // ring of device buffers
    const size_t in_slot  = round256(size_t(block_rows) * in_row);
    const size_t out_one  = round256(size_t(block_rows) * out_row);
    const size_t out_slot = (both ? 2 : 1) * out_one;
    const size_t g_bytes  = round256(size_t(cols) * 4);
    uint8_t* base         = nullptr;
    MIMK_TRY(arena(*c, g_bytes + size_t(slots) * (in_slot + out_slot), &base));
    float* d_gamma = reinterpret_cast<float*>(base);
    if (kind != MIMK_ROWS_SOFTMAX) MIMK_CUDA_TRY(cudaMemcpyAsync(d_gamma, gamma, size_t(cols) * 4, cudaMemcpyHostToDevice, c->up));
    for (int64_t b = 0; b < nblocks; ++b) {
        const int slot   = int(b % slots);
        const int ev     = int(b % HostCtx::MAX_EVENTS);
        const int64_t r0 = b * block_rows;
        const int64_t nr = rows - r0 < block_rows ? rows - r0 : block_rows;
        uint8_t* d_in    = base + g_bytes + size_t(slot) * in_slot;
        uint8_t* d_out   = base + g_bytes + size_t(slots) * in_slot + size_t(slot) * out_slot;
        MIMK_TRY(ring_guard(*c, b));
        // the input slot is free once the kernels that last read it are done, the output slot once its download drained
        if (b >= slots) {
            const int prev = int((b - slots) % HostCtx::MAX_EVENTS);
            MIMK_CUDA_TRY(cudaStreamWaitEvent(c->up, c->computed[prev], 0));
            MIMK_CUDA_TRY(cudaStreamWaitEvent(c->work, c->drained[prev], 0));
        }
        MIMK_CUDA_TRY(cudaMemcpyAsync(d_in, static_cast<const uint8_t*>(x) + size_t(r0) * in_row, size_t(nr) * in_row,
                                      cudaMemcpyHostToDevice, c->up));
        MIMK_CUDA_TRY(cudaEventRecord(c->uploaded[ev], c->up));
        MIMK_CUDA_TRY(cudaStreamWaitEvent(c->work, c->uploaded[ev], 0));
        if (kind == MIMK_ROWS_SOFTMAX || both) MIMK_TRY(mimk_softmax(d_in, d_out, in_dtype, out_dtype, nr, cols, 1, c->work));
        if (kind == MIMK_ROWS_RMSNORM) MIMK_TRY(mimk_rmsnorm(d_in, d_gamma, d_out, in_dtype, out_dtype, nr, cols, eps, c->work));
        if (both) MIMK_TRY(mimk_rmsnorm(d_in, d_gamma, d_out + out_one, in_dtype, out_dtype, nr, cols, eps, c->work));
        if (kind == MIMK_ROWS_SOFTMAX_RMSNORM)
            MIMK_TRY(mimk_softmax_rmsnorm(d_in, d_gamma, d_out, in_dtype, out_dtype, nr, cols, eps, c->work));
        MIMK_CUDA_TRY(cudaEventRecord(c->computed[ev], c->work));
        MIMK_CUDA_TRY(cudaStreamWaitEvent(c->down, c->computed[ev], 0));
        MIMK_CUDA_TRY(cudaMemcpyAsync(static_cast<uint8_t*>(y) + size_t(r0) * out_row, d_out, size_t(nr) * out_row,
                                      cudaMemcpyDeviceToHost, c->down));
        if (both)
            MIMK_CUDA_TRY(cudaMemcpyAsync(static_cast<uint8_t*>(y2) + size_t(r0) * out_row, d_out + out_one, size_t(nr) * out_row,
                                          cudaMemcpyDeviceToHost, c->down));
        MIMK_CUDA_TRY(cudaEventRecord(c->drained[ev], c->down));
    }
    return MIMK_OK;
}

// kind 0..2: one result `y`; kind 3: softmax into `y` and RMSNorm into `y2` from ONE upload of x.
int host_rows_impl(int kind, const void* x, const void* gamma, void* y, void* y2, int in_dtype, int out_dtype,
                   int64_t rows, int64_t cols, float eps) {
    const bool both = kind == 3;
    if ((!both && (kind < MIMK_ROWS_SOFTMAX || kind > MIMK_ROWS_SOFTMAX_RMSNORM)) || rows < 0 || cols < 0) return MIMK_E_ARG;
    if ((in_dtype != MIMK_F32 && in_dtype != MIMK_BF16) || (out_dtype != MIMK_F32 && out_dtype != MIMK_BF16))
        return MIMK_E_DTYPE;
    std::lock_guard<std::mutex> lock(g_host_mutex);
    HostCtx* c = nullptr;
    MIMK_TRY(get_ctx(&c));
    if (rows * cols == 0) return MIMK_OK;
    if (!x || !y || (both && !y2) || (kind != MIMK_ROWS_SOFTMAX && !gamma)) return MIMK_E_ARG;
    return finish(*c, host_rows_body(c, kind, x, gamma, y, y2, in_dtype, out_dtype, rows, cols, eps));
}
}  // namespace

extern "C" int mimk_host_rows(int kind, const void* x, const void* gamma, void* y, int in_dtype, int out_dtype,
                              int64_t rows, int64_t cols, float eps) {
    if (kind == 3) return MIMK_E_ARG;
    return host_rows_impl(kind, x, gamma, y, nullptr, in_dtype, out_dtype, rows, cols, eps);
}

extern "C" int mimk_host_rows_pair(const void* x, const void* gamma, void* y_softmax, void* y_rmsnorm, int in_dtype,
                                   int out_dtype, int64_t rows, int64_t cols, float eps) {
    return host_rows_impl(3, x, gamma, y_softmax, y_rmsnorm, in_dtype, out_dtype, rows, cols, eps);
}

namespace {
// C = post(A B) with host operands. One batch entry whose A has at least two panels of rows is pipelined: B (and the
// bias row) first, then per panel of rows the upload of the A panel (and of the full-shape epilogue operand's panel),
// the contraction of that panel on `work`, and the download of its rows of C. Everything else goes up, runs, comes down.
int host_gemm_body(HostCtx* c, const mimk_gemm_desc* h) {
    const size_t es = dtype_size(h->in_dtype), os = dtype_size(h->out_dtype);
    // batch strides: a dense batch is uploaded as one block; stride 0 (shared operand) as a single matrix
    const size_t a_elems = size_t(h->m) * h->k * (h->stride_a ? h->batch : 1);
    const size_t b_elems = size_t(h->k) * h->n * (h->stride_b ? h->batch : 1);
    const size_t c_elems = size_t(h->m) * h->n * h->batch;
    if (h->batch > 1 && ((h->stride_a && h->stride_a != h->m * h->k) || (h->stride_b && h->stride_b != h->k * h->n) ||
                         h->stride_c != h->m * h->n))
        return MIMK_E_UNSUPPORTED;
    const size_t a_b = round256(a_elems * es), b_b = round256(b_elems * es), c_b = round256(c_elems * os);
    const size_t row_b = h->post_row ? round256(size_t(h->n) * 4) : 0, full_b = h->post_full ? c_b : 0;
    uint8_t* base = nullptr;
    MIMK_TRY(arena(*c, a_b + b_b + c_b + row_b + full_b, &base));
    mimk_gemm_desc d = *h;
    d.a = base, d.b = base + a_b, d.c = base + a_b + b_b;
    if (h->post_row) d.post_row = base + a_b + b_b + c_b;
    if (h->post_full) d.post_full = base + a_b + b_b + c_b + row_b;
    uint8_t *d_a = base, *d_c = base + a_b + b_b, *d_full = base + a_b + b_b + c_b + row_b;

    // panels of about 16 MiB of A (or of C, whichever row is longer), whole 256-row tiles
    int64_t panel = h->m;
    if (h->batch == 1 && h->k > 0 && h->in_dtype == MIMK_BF16) {  // f32 operands are re-split per call: one call
        const size_t row_bytes = size_t(h->k) * es > size_t(h->n) * os ? size_t(h->k) * es : size_t(h->n) * os;
        int64_t rows           = int64_t((size_t(16) << 20) / row_bytes) & ~int64_t(255);
        if (rows >= 256 && rows * 2 <= h->m) panel = rows;
    }
    if (b_elems) MIMK_CUDA_TRY(cudaMemcpyAsync(const_cast<void*>(d.b), h->b, b_elems * es, cudaMemcpyHostToDevice, c->up));
    if (h->post_row)
        MIMK_CUDA_TRY(cudaMemcpyAsync(const_cast<void*>(d.post_row), h->post_row, size_t(h->n) * 4, cudaMemcpyHostToDevice, c->up));
    if (panel == h->m) {
        if (a_elems) MIMK_CUDA_TRY(cudaMemcpyAsync(d_a, h->a, a_elems * es, cudaMemcpyHostToDevice, c->up));
        if (h->post_full) MIMK_CUDA_TRY(cudaMemcpyAsync(d_full, h->post_full, c_elems * os, cudaMemcpyHostToDevice, c->up));
        MIMK_CUDA_TRY(cudaEventRecord(c->uploaded[0], c->up));
        MIMK_CUDA_TRY(cudaStreamWaitEvent(c->work, c->uploaded[0], 0));
        MIMK_TRY(mimk_gemm(&d, c->work));
        MIMK_CUDA_TRY(cudaEventRecord(c->computed[0], c->work));
        MIMK_CUDA_TRY(cudaStreamWaitEvent(c->down, c->computed[0], 0));
        MIMK_CUDA_TRY(cudaMemcpyAsync(h->c, d.c, c_elems * os, cudaMemcpyDeviceToHost, c->down));
        return MIMK_OK;
    }
    const int64_t npanels = (h->m + panel - 1) / panel;
    for (int64_t b = 0; b < npanels; ++b) {
        const int ev     = int(b % HostCtx::MAX_EVENTS);
        const int64_t r0 = b * panel, nr = h->m - r0 < panel ? h->m - r0 : panel;
        MIMK_TRY(ring_guard(*c, b));
        MIMK_CUDA_TRY(cudaMemcpyAsync(d_a + size_t(r0) * h->k * es, static_cast<const uint8_t*>(h->a) + size_t(r0) * h->k * es,
                                      size_t(nr) * h->k * es, cudaMemcpyHostToDevice, c->up));
        if (h->post_full)
            MIMK_CUDA_TRY(cudaMemcpyAsync(d_full + size_t(r0) * h->n * os, static_cast<const uint8_t*>(h->post_full) + size_t(r0) * h->n * os,
                                          size_t(nr) * h->n * os, cudaMemcpyHostToDevice, c->up));
        MIMK_CUDA_TRY(cudaEventRecord(c->uploaded[ev], c->up));
        MIMK_CUDA_TRY(cudaStreamWaitEvent(c->work, c->uploaded[ev], 0));
        mimk_gemm_desc dp = d;
        dp.m = nr;
        dp.a = d_a + size_t(r0) * h->k * es;
        dp.c = d_c + size_t(r0) * h->n * os;
        if (h->post_full) dp.post_full = d_full + size_t(r0) * h->n * os;
        MIMK_TRY(mimk_gemm(&dp, c->work));
        MIMK_CUDA_TRY(cudaEventRecord(c->computed[ev], c->work));
        MIMK_CUDA_TRY(cudaStreamWaitEvent(c->down, c->computed[ev], 0));
        MIMK_CUDA_TRY(cudaMemcpyAsync(static_cast<uint8_t*>(h->c) + size_t(r0) * h->n * os, dp.c, size_t(nr) * h->n * os,
                                      cudaMemcpyDeviceToHost, c->down));
        MIMK_CUDA_TRY(cudaEventRecord(c->drained[ev], c->down));
    }
    return MIMK_OK;
}

// Attention with host operands, in groups of heads: the upload of group g+1's q, k, v overlaps the kernel on group g and
// the download of group g-1's rows of o. A group holds about 32 MiB of q + k + v (at least 8 heads when there are that
// many), so that a launch still fills the machine.
int host_attn_body(HostCtx* c, const mimk_attn_desc* h) {
    const size_t es   = dtype_size(h->dtype);
    const size_t q_h  = size_t(h->seq_q) * h->head_dim * es, k_h = size_t(h->seq_k) * h->head_dim * es;
    const size_t q_b  = size_t(h->batch_heads) * q_h, k_b = size_t(h->batch_heads) * k_h;
    const size_t l_b  = h->lse ? size_t(h->batch_heads) * h->seq_q * 4 : 0;
    uint8_t* base     = nullptr;
    MIMK_TRY(arena(*c, 2 * round256(q_b) + 2 * round256(k_b) + round256(l_b), &base));
    uint8_t* p   = base;
    uint8_t* d_q = p; p += round256(q_b);
    uint8_t* d_k = p; p += round256(k_b);
    uint8_t* d_v = p; p += round256(k_b);
    uint8_t* d_o = p; p += round256(q_b);
    float* d_l   = h->lse ? reinterpret_cast<float*>(p) : nullptr;
    int64_t group = int64_t((size_t(32) << 20) / (q_h + 2 * k_h + 1));
    if (group < 8) group = 8;
    if (group * 2 > h->batch_heads) group = h->batch_heads;
    const int64_t ngroups = (h->batch_heads + group - 1) / group;
    for (int64_t b = 0; b < ngroups; ++b) {
        const int ev     = int(b % HostCtx::MAX_EVENTS);
        const int64_t h0 = b * group, nh = h->batch_heads - h0 < group ? h->batch_heads - h0 : group;
        MIMK_TRY(ring_guard(*c, b));
        MIMK_CUDA_TRY(cudaMemcpyAsync(d_q + h0 * q_h, static_cast<const uint8_t*>(h->q) + h0 * q_h, nh * q_h, cudaMemcpyHostToDevice, c->up));
        if (k_h) {
            MIMK_CUDA_TRY(cudaMemcpyAsync(d_k + h0 * k_h, static_cast<const uint8_t*>(h->k) + h0 * k_h, nh * k_h, cudaMemcpyHostToDevice, c->up));
            MIMK_CUDA_TRY(cudaMemcpyAsync(d_v + h0 * k_h, static_cast<const uint8_t*>(h->v) + h0 * k_h, nh * k_h, cudaMemcpyHostToDevice, c->up));
        }
        MIMK_CUDA_TRY(cudaEventRecord(c->uploaded[ev], c->up));
        MIMK_CUDA_TRY(cudaStreamWaitEvent(c->work, c->uploaded[ev], 0));
        mimk_attn_desc d = *h;
        d.batch_heads    = nh;
        d.q = d_q + h0 * q_h, d.k = d_k + h0 * k_h, d.v = d_v + h0 * k_h, d.o = d_o + h0 * q_h;
        d.lse = h->lse ? d_l + h0 * h->seq_q : nullptr;
        MIMK_TRY(mimk_attn_fwd(&d, c->work));
        MIMK_CUDA_TRY(cudaEventRecord(c->computed[ev], c->work));
        MIMK_CUDA_TRY(cudaStreamWaitEvent(c->down, c->computed[ev], 0));
        MIMK_CUDA_TRY(cudaMemcpyAsync(static_cast<uint8_t*>(h->o) + h0 * q_h, d.o, nh * q_h, cudaMemcpyDeviceToHost, c->down));
        if (h->lse) MIMK_CUDA_TRY(cudaMemcpyAsync(h->lse + h0 * h->seq_q, d.lse, size_t(nh) * h->seq_q * 4, cudaMemcpyDeviceToHost, c->down));
        MIMK_CUDA_TRY(cudaEventRecord(c->drained[ev], c->down));
    }
    return MIMK_OK;
}
}  // namespace

extern "C" int mimk_host_gemm(const mimk_gemm_desc* h) {
    if (!h) return MIMK_E_ARG;
    if (h->batch < 0 || h->m < 0 || h->n < 0 || h->k < 0) return MIMK_E_ARG;
    if ((h->in_dtype != MIMK_F32 && h->in_dtype != MIMK_BF16) || (h->out_dtype != MIMK_F32 && h->out_dtype != MIMK_BF16))
        return MIMK_E_DTYPE;
    std::lock_guard<std::mutex> lock(g_host_mutex);
    HostCtx* c = nullptr;
    MIMK_TRY(get_ctx(&c));
    if (h->batch == 0 || h->m == 0 || h->n == 0) return MIMK_OK;
    if (!h->c || (h->k > 0 && (!h->a || !h->b))) return MIMK_E_ARG;
    return finish(*c, host_gemm_body(c, h));
}

extern "C" int mimk_host_attn_fwd(const mimk_attn_desc* h) {
    if (!h) return MIMK_E_ARG;
    if (h->batch_heads < 0 || h->seq_q < 0 || h->seq_k < 0 || h->head_dim < 0) return MIMK_E_ARG;
    if (h->dtype != MIMK_F32 && h->dtype != MIMK_BF16) return MIMK_E_DTYPE;
    std::lock_guard<std::mutex> lock(g_host_mutex);
    HostCtx* c = nullptr;
    MIMK_TRY(get_ctx(&c));
    if (h->batch_heads == 0 || h->seq_q == 0 || h->head_dim == 0) return MIMK_OK;
    if (!h->q || !h->o || (h->seq_k > 0 && (!h->k || !h->v))) return MIMK_E_ARG;
    return finish(*c, host_attn_body(c, h));
}

// The generic operation with host operands: what the reference's wrapper does around every map_reduce_post --
// upload each input and epilogue input, run, download the result (lower_map_reduce.cpp:111-126, 267-297).
extern "C" int mimk_host_map_reduce_post(const mimk_mrp_desc* h) {
    if (!h) return MIMK_E_ARG;
    if (h->ro < 0 || h->rn < h->ro || h->rn > MIMK_MRP_MAX_LOOPS || h->ro > MIMK_MRP_MAX_RANK) return MIMK_E_ARG;
    if (h->nis < 0 || h->nis > MIMK_MRP_MAX_INPUTS || h->nps < 0 || h->nps > 1) return MIMK_E_ARG;
    auto elems = [](const int64_t* shape, int rank, size_t* out) {
        size_t n = 1;
        for (int j = 0; j < rank; ++j) {
            if (shape[j] < 0) return false;
            n *= size_t(shape[j]);
        }
        *out = n;
        return true;
    };
    auto known = [](int dt) { return dt == MIMK_F32 || dt == MIMK_BF16 || dt == MIMK_I32 || dt == MIMK_I64; };
    size_t in_bytes[MIMK_MRP_MAX_INPUTS] = {}, post_bytes = 0, out_elems = 0, total = 0;
    for (int i = 0; i < h->nis; ++i) {
        size_t n = 0;
        if (!known(h->in_dtype[i]) || h->in_map[i].rows < 0 || h->in_map[i].rows > MIMK_MRP_MAX_RANK) return MIMK_E_ARG;
        if (!elems(h->in_shape[i], h->in_map[i].rows, &n)) return MIMK_E_ARG;
        in_bytes[i] = n * dtype_size(h->in_dtype[i]);
        if (in_bytes[i] && !h->in[i]) return MIMK_E_ARG;
        total += round256(in_bytes[i]);
    }
    if (h->nps == 1) {
        size_t n = 0;
        if (!known(h->post_dtype[0]) || h->post_map[0].rows < 0 || h->post_map[0].rows > MIMK_MRP_MAX_RANK) return MIMK_E_ARG;
        if (!elems(h->post_shape[0], h->post_map[0].rows, &n)) return MIMK_E_ARG;
        post_bytes = n * dtype_size(h->post_dtype[0]);
        if (post_bytes && !h->post_in[0]) return MIMK_E_ARG;
        total += round256(post_bytes);
    }
    if (!known(h->out_dtype) || !elems(h->so, h->ro, &out_elems)) return MIMK_E_ARG;
    const size_t out_bytes = out_elems * dtype_size(h->out_dtype);
    if (out_bytes && !h->out) return MIMK_E_ARG;
    total += round256(out_bytes);
    std::lock_guard<std::mutex> lock(g_host_mutex);
    HostCtx* c = nullptr;
    MIMK_TRY(get_ctx(&c));
    if (out_bytes == 0) return MIMK_OK;
    auto body = [&]() -> int {
    uint8_t* base = nullptr;
    MIMK_TRY(arena(*c, total, &base));
    mimk_mrp_desc d = *h;
    uint8_t* p      = base;
    for (int i = 0; i < h->nis; ++i) {
        d.in[i] = p;
        if (in_bytes[i]) MIMK_CUDA_TRY(cudaMemcpyAsync(p, h->in[i], in_bytes[i], cudaMemcpyHostToDevice, c->up));
        p += round256(in_bytes[i]);
    }
    if (h->nps == 1) {
        d.post_in[0] = p;
        if (post_bytes) MIMK_CUDA_TRY(cudaMemcpyAsync(p, h->post_in[0], post_bytes, cudaMemcpyHostToDevice, c->up));
        p += round256(post_bytes);
    }
    d.out = p;
    // a write map need not cover the result (packed or partial outputs): cells it never stores keep the caller's bytes
    MIMK_CUDA_TRY(cudaMemcpyAsync(p, h->out, out_bytes, cudaMemcpyHostToDevice, c->up));
    MIMK_CUDA_TRY(cudaEventRecord(c->uploaded[0], c->up));
    MIMK_CUDA_TRY(cudaStreamWaitEvent(c->work, c->uploaded[0], 0));
    MIMK_TRY(mimk_map_reduce_post(&d, c->work));
    MIMK_CUDA_TRY(cudaMemcpyAsync(h->out, d.out, out_bytes, cudaMemcpyDeviceToHost, c->work));
    return MIMK_OK;
    };
    return finish(*c, body());
}

namespace {
// The gated MLP block with host operands. Uploads in the order the stages need them: X, W1, W3, then W2 while stage 1
// (H = silu(X W1) * (X W3)) runs; stage 2 (Y = H W2) runs in panels of rows whose downloads overlap the next panel.
int host_mlp_body(HostCtx* c, const mimk_mlp_desc* h) {
    const size_t x_b = round256(size_t(h->m) * h->k * 2), w1_b = round256(size_t(h->k) * h->f * 2);
    const size_t w2_b = round256(size_t(h->f) * h->n * 2), y_b = round256(size_t(h->m) * h->n * 2);
    const size_t h_b  = round256(size_t(h->m) * h->f * 2);
    uint8_t* base     = nullptr;
    MIMK_TRY(arena(*c, x_b + 2 * w1_b + w2_b + y_b + h_b, &base));
    uint8_t* p   = base;
    uint8_t* d_x = p; p += x_b;
    uint8_t* d_w1 = p; p += w1_b;
    uint8_t* d_w3 = p; p += w1_b;
    uint8_t* d_w2 = p; p += w2_b;
    uint8_t* d_y = p; p += y_b;
    uint8_t* d_h = p;
    MIMK_CUDA_TRY(cudaMemcpyAsync(d_x, h->x, size_t(h->m) * h->k * 2, cudaMemcpyHostToDevice, c->up));
    MIMK_CUDA_TRY(cudaMemcpyAsync(d_w1, h->w1, size_t(h->k) * h->f * 2, cudaMemcpyHostToDevice, c->up));
    MIMK_CUDA_TRY(cudaMemcpyAsync(d_w3, h->w3, size_t(h->k) * h->f * 2, cudaMemcpyHostToDevice, c->up));
    MIMK_CUDA_TRY(cudaEventRecord(c->uploaded[0], c->up));
    MIMK_CUDA_TRY(cudaMemcpyAsync(d_w2, h->w2, size_t(h->f) * h->n * 2, cudaMemcpyHostToDevice, c->up));
    MIMK_CUDA_TRY(cudaEventRecord(c->uploaded[1], c->up));
    MIMK_CUDA_TRY(cudaStreamWaitEvent(c->work, c->uploaded[0], 0));
    mimk_gemm_desc g1 = {};
    g1.batch = 1, g1.m = h->m, g1.n = h->f, g1.k = h->k;
    g1.a = d_x, g1.b = d_w1, g1.c = d_h;
    g1.in_dtype = MIMK_BF16, g1.out_dtype = MIMK_BF16, g1.b_layout = h->b_layout, g1.post = MIMK_POST_ID;
    if (!gemm_tc_supported(g1)) return MIMK_E_UNSUPPORTED;
    MIMK_TRY(gemm_tc_any(g1, c->work, 1, d_w3));
    MIMK_CUDA_TRY(cudaStreamWaitEvent(c->work, c->uploaded[1], 0));
    int64_t panel = int64_t((size_t(16) << 20) / (size_t(h->n) * 2 + 1)) & ~int64_t(255);
    if (panel < 256 || panel * 2 > h->m) panel = h->m;
    const int64_t npanels = (h->m + panel - 1) / panel;
    for (int64_t b = 0; b < npanels; ++b) {
        const int ev     = int(b % HostCtx::MAX_EVENTS);
        const int64_t r0 = b * panel, nr = h->m - r0 < panel ? h->m - r0 : panel;
        MIMK_TRY(ring_guard(*c, b));
        mimk_gemm_desc g2 = {};
        g2.batch = 1, g2.m = nr, g2.n = h->n, g2.k = h->f;
        g2.a = d_h + size_t(r0) * h->f * 2, g2.b = d_w2, g2.c = d_y + size_t(r0) * h->n * 2;
        g2.in_dtype = MIMK_BF16, g2.out_dtype = MIMK_BF16, g2.b_layout = h->b_layout, g2.post = MIMK_POST_ID;
        MIMK_TRY(mimk_gemm(&g2, c->work));
        MIMK_CUDA_TRY(cudaEventRecord(c->computed[ev], c->work));
        MIMK_CUDA_TRY(cudaStreamWaitEvent(c->down, c->computed[ev], 0));
        MIMK_CUDA_TRY(cudaMemcpyAsync(static_cast<uint8_t*>(h->y) + size_t(r0) * h->n * 2, g2.c, size_t(nr) * h->n * 2,
                                      cudaMemcpyDeviceToHost, c->down));
        MIMK_CUDA_TRY(cudaEventRecord(c->drained[ev], c->down));
    }
    return MIMK_OK;
}
}  // namespace

extern "C" int mimk_host_mlp_gated(const mimk_mlp_desc* h) {
    if (!h) return MIMK_E_ARG;
    if (h->m < 0 || h->k < 0 || h->f < 0 || h->n < 0) return MIMK_E_ARG;
    if (h->dtype != MIMK_BF16) return MIMK_E_DTYPE;
    if (h->b_layout != MIMK_B_KN && h->b_layout != MIMK_B_NK) return MIMK_E_ARG;
    std::lock_guard<std::mutex> lock(g_host_mutex);
    HostCtx* c = nullptr;
    MIMK_TRY(get_ctx(&c));
    if (h->m == 0 || h->n == 0) return MIMK_OK;
    if (!h->x || !h->w1 || !h->w3 || !h->w2 || !h->y) return MIMK_E_ARG;
    return finish(*c, host_mlp_body(c, h));
}
