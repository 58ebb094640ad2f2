// Host-buffer entry points: upload, run, download.
//
// They stand in for the wrapper the reference emits around every GPU-lowered operation (MimIR
// src/mim/plug/gpu/phase/lower_map_reduce.cpp:317-395: gpu.buf_alloc_copy per input, gpu.alloc.block for the
// output, gpu.launch, gpu.buf_copy_to_host, gpu.free -- all blocking on the null stream). Here the device buffers
// come from a cached arena, copies are asynchronous, and row-wise operators are streamed through the device in
// row blocks on two streams so that the upload of block i+1, the kernel on block i and the download of block i-1
// overlap.
#include <mutex>

#include "common.cuh"

namespace mimk {
namespace {

struct HostCtx {
    bool ready = false;
    void* arena = nullptr;
    size_t arena_bytes = 0;
    cudaStream_t up = nullptr, down = nullptr;
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
        // the slot is free again once the download that last used it has drained
        if (b >= slots) MIMK_CUDA_TRY(cudaStreamWaitEvent(c->up, c->drained[int((b - slots) % HostCtx::MAX_EVENTS)], 0));
        MIMK_CUDA_TRY(cudaMemcpyAsync(d_in, static_cast<const uint8_t*>(x) + size_t(r0) * in_row, size_t(nr) * in_row,
                                      cudaMemcpyHostToDevice, c->up));
        if (kind == MIMK_ROWS_SOFTMAX || both) MIMK_TRY(mimk_softmax(d_in, d_out, in_dtype, out_dtype, nr, cols, 1, c->up));
        if (kind == MIMK_ROWS_RMSNORM) MIMK_TRY(mimk_rmsnorm(d_in, d_gamma, d_out, in_dtype, out_dtype, nr, cols, eps, c->up));
        if (both) MIMK_TRY(mimk_rmsnorm(d_in, d_gamma, d_out + out_one, in_dtype, out_dtype, nr, cols, eps, c->up));
        if (kind == MIMK_ROWS_SOFTMAX_RMSNORM)
            MIMK_TRY(mimk_softmax_rmsnorm(d_in, d_gamma, d_out, in_dtype, out_dtype, nr, cols, eps, c->up));
        MIMK_CUDA_TRY(cudaEventRecord(c->computed[ev], c->up));
        MIMK_CUDA_TRY(cudaStreamWaitEvent(c->down, c->computed[ev], 0));
        MIMK_CUDA_TRY(cudaMemcpyAsync(static_cast<uint8_t*>(y) + size_t(r0) * out_row, d_out, size_t(nr) * out_row,
                                      cudaMemcpyDeviceToHost, c->down));
        if (both)
            MIMK_CUDA_TRY(cudaMemcpyAsync(static_cast<uint8_t*>(y2) + size_t(r0) * out_row, d_out + out_one, size_t(nr) * out_row,
                                          cudaMemcpyDeviceToHost, c->down));
        MIMK_CUDA_TRY(cudaEventRecord(c->drained[ev], c->down));
        // keep at most MAX_EVENTS blocks in flight so that an event is never re-recorded while still awaited
        if (b + 1 >= HostCtx::MAX_EVENTS) MIMK_CUDA_TRY(cudaEventSynchronize(c->drained[int((b + 1) % HostCtx::MAX_EVENTS)]));
    }
    MIMK_CUDA_TRY(cudaStreamSynchronize(c->down));
    MIMK_CUDA_TRY(cudaStreamSynchronize(c->up));
    return MIMK_OK;
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
    if (a_elems) MIMK_CUDA_TRY(cudaMemcpyAsync(const_cast<void*>(d.a), h->a, a_elems * es, cudaMemcpyHostToDevice, c->up));
    if (b_elems) MIMK_CUDA_TRY(cudaMemcpyAsync(const_cast<void*>(d.b), h->b, b_elems * es, cudaMemcpyHostToDevice, c->up));
    if (h->post_row) {
        d.post_row = base + a_b + b_b + c_b;
        MIMK_CUDA_TRY(cudaMemcpyAsync(const_cast<void*>(d.post_row), h->post_row, size_t(h->n) * 4, cudaMemcpyHostToDevice, c->up));
    }
    if (h->post_full) {
        d.post_full = base + a_b + b_b + c_b + row_b;
        MIMK_CUDA_TRY(cudaMemcpyAsync(const_cast<void*>(d.post_full), h->post_full, c_elems * os, cudaMemcpyHostToDevice, c->up));
    }
    MIMK_TRY(mimk_gemm(&d, c->up));
    MIMK_CUDA_TRY(cudaMemcpyAsync(h->c, d.c, c_elems * os, cudaMemcpyDeviceToHost, c->up));
    return mimk_device_status(c->up);
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
    const size_t es  = dtype_size(h->dtype);
    const size_t q_b = size_t(h->batch_heads) * h->seq_q * h->head_dim * es;
    const size_t k_b = size_t(h->batch_heads) * h->seq_k * h->head_dim * es;
    const size_t l_b = h->lse ? size_t(h->batch_heads) * h->seq_q * 4 : 0;
    uint8_t* base    = nullptr;
    MIMK_TRY(arena(*c, 2 * round256(q_b) + 2 * round256(k_b) + round256(l_b), &base));
    mimk_attn_desc d = *h;
    uint8_t* p       = base;
    d.q = p, p += round256(q_b);
    d.k = p, p += round256(k_b);
    d.v = p, p += round256(k_b);
    d.o = p, p += round256(q_b);
    d.lse = h->lse ? reinterpret_cast<float*>(p) : nullptr;
    MIMK_CUDA_TRY(cudaMemcpyAsync(const_cast<void*>(d.q), h->q, q_b, cudaMemcpyHostToDevice, c->up));
    if (k_b) {
        MIMK_CUDA_TRY(cudaMemcpyAsync(const_cast<void*>(d.k), h->k, k_b, cudaMemcpyHostToDevice, c->up));
        MIMK_CUDA_TRY(cudaMemcpyAsync(const_cast<void*>(d.v), h->v, k_b, cudaMemcpyHostToDevice, c->up));
    }
    MIMK_TRY(mimk_attn_fwd(&d, c->up));
    MIMK_CUDA_TRY(cudaMemcpyAsync(h->o, d.o, q_b, cudaMemcpyDeviceToHost, c->up));
    if (h->lse) MIMK_CUDA_TRY(cudaMemcpyAsync(h->lse, d.lse, l_b, cudaMemcpyDeviceToHost, c->up));
    return mimk_device_status(c->up);
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
    MIMK_TRY(mimk_map_reduce_post(&d, c->up));
    MIMK_CUDA_TRY(cudaMemcpyAsync(h->out, d.out, out_bytes, cudaMemcpyDeviceToHost, c->up));
    return mimk_device_status(c->up);
}

extern "C" int mimk_host_mlp_gated(const mimk_mlp_desc* h) {
    if (!h) return MIMK_E_ARG;
    if (h->m < 0 || h->k < 0 || h->f < 0 || h->n < 0) return MIMK_E_ARG;
    if (h->dtype != MIMK_BF16) return MIMK_E_DTYPE;
    std::lock_guard<std::mutex> lock(g_host_mutex);
    HostCtx* c = nullptr;
    MIMK_TRY(get_ctx(&c));
    if (h->m == 0 || h->n == 0) return MIMK_OK;
    if (!h->x || !h->w1 || !h->w3 || !h->w2 || !h->y) return MIMK_E_ARG;
    const size_t x_b = round256(size_t(h->m) * h->k * 2), w1_b = round256(size_t(h->k) * h->f * 2);
    const size_t w2_b = round256(size_t(h->f) * h->n * 2), y_b = round256(size_t(h->m) * h->n * 2);
    const size_t h_b  = round256(size_t(h->m) * h->f * 2);
    uint8_t* base     = nullptr;
    MIMK_TRY(arena(*c, x_b + 2 * w1_b + w2_b + y_b + h_b, &base));
    mimk_mlp_desc d = *h;
    uint8_t* p      = base;
    d.x = p, p += x_b;
    d.w1 = p, p += w1_b;
    d.w3 = p, p += w1_b;
    d.w2 = p, p += w2_b;
    d.y = p, p += y_b;
    d.h = p;
    MIMK_CUDA_TRY(cudaMemcpyAsync(const_cast<void*>(d.x), h->x, size_t(h->m) * h->k * 2, cudaMemcpyHostToDevice, c->up));
    MIMK_CUDA_TRY(cudaMemcpyAsync(const_cast<void*>(d.w1), h->w1, size_t(h->k) * h->f * 2, cudaMemcpyHostToDevice, c->up));
    MIMK_CUDA_TRY(cudaMemcpyAsync(const_cast<void*>(d.w3), h->w3, size_t(h->k) * h->f * 2, cudaMemcpyHostToDevice, c->up));
    MIMK_CUDA_TRY(cudaMemcpyAsync(const_cast<void*>(d.w2), h->w2, size_t(h->f) * h->n * 2, cudaMemcpyHostToDevice, c->up));
    MIMK_TRY(mimk_mlp_gated(&d, c->up));
    MIMK_CUDA_TRY(cudaMemcpyAsync(h->y, d.y, size_t(h->m) * h->n * 2, cudaMemcpyDeviceToHost, c->up));
    return mimk_device_status(c->up);
}
