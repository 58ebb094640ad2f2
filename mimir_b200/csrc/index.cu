// Constructors and data-dependent indexing of the tensor plugin: splat, generate (affine bodies), gather, scatter
// (MimIR src/mim/plug/tensor/tensor.mim:77-109, 519-563). None of them is a map_reduce_post: generate / splat read no
// input, gather / scatter pick a coordinate from an index tensor. All are bandwidth-bound element-wise kernels.
#include "common.cuh"

namespace mimk {
namespace {

constexpr int MAX_RANK = MIMK_MRP_MAX_RANK;

struct Shape {
    int rank;
    int64_t ext[MAX_RANK];
};

template <class T>
__global__ void splat_kernel(T* out, long long n, T value) {
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) out[i] = value;
}

// out[o] = sum_d coef[d] * o[d] + coef[rank], in wrap-around int64, then converted to the element type
struct Coef {
    long long c[MAX_RANK + 1];
};
template <class T>
__global__ void generate_affine_kernel(T* out, long long n, Shape s, Coef coef_in) {
    unsigned long long coef[MAX_RANK + 1];
    for (int d = 0; d <= s.rank; ++d) coef[d] = (unsigned long long)coef_in.c[d];
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
        long long rest = i;
        unsigned long long v = coef[s.rank];
        for (int d = s.rank - 1; d >= 0; --d) {
            v += coef[d] * (unsigned long long)(rest % s.ext[d]);
            rest /= s.ext[d];
        }
        out[i] = static_cast<T>((long long)v);
    }
}

// One thread per index element: out[o] = input[o with o[dim] := index[o]]   (tensor.mim:527-541)
template <class T, class I>
__global__ void gather_kernel(const T* __restrict__ in, const I* __restrict__ index, T* __restrict__ out, long long n, Shape src,
                              Shape idx, int dim, int* status) {
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
        const long long sel = (long long)index[i];
        if (sel < 0 || sel >= src.ext[dim]) {  // the reference's index type `Idx (s_src#dim)` rules this out
            *status = MIMK_E_SHAPE;
            continue;
        }
        long long rest = i, off = 0, stride = 1;
        for (int d = idx.rank - 1; d >= 0; --d) {
            const long long c = rest % idx.ext[d];
            rest /= idx.ext[d];
            off += (d == dim ? sel : c) * stride;
            stride *= src.ext[d];
        }
        out[i] = in[off];
    }
}

// One thread per line of the index tensor along `dim`, walking the line in ascending order: every destination that two
// updates share lies on one such line, so the last update visited in row-major order wins, as the reference defines
// (tensor.mim:545-557). `out` already holds a copy of `input`.
template <class T, class I>
__global__ void scatter_kernel(const I* __restrict__ index, const T* __restrict__ upd, T* __restrict__ out, long long lines,
                               Shape src, Shape idx, Shape ups, int dim, int* status) {
    for (long long line = blockIdx.x * (long long)blockDim.x + threadIdx.x; line < lines; line += (long long)gridDim.x * blockDim.x) {
        // coordinates of the line (all axes but dim), and the strides of `dim` in the three tensors
        long long rest = line, i_off = 0, u_off = 0, o_off = 0, i_str = 1, u_str = 1, o_str = 1;
        long long i_dim = 0, u_dim = 0, o_dim = 0;
        for (int d = idx.rank - 1; d >= 0; --d) {
            if (d == dim) {
                i_dim = i_str, u_dim = u_str, o_dim = o_str;
            } else {
                const long long c = rest % idx.ext[d];
                rest /= idx.ext[d];
                i_off += c * i_str, u_off += c * u_str, o_off += c * o_str;
            }
            i_str *= idx.ext[d], u_str *= ups.ext[d], o_str *= src.ext[d];
        }
        for (long long k = 0; k < idx.ext[dim]; ++k) {
            const long long sel = (long long)index[i_off + k * i_dim];
            if (sel < 0 || sel >= src.ext[dim]) {
                *status = MIMK_E_SHAPE;
                continue;
            }
            out[o_off + sel * o_dim] = upd[u_off + k * u_dim];
        }
    }
}

// The same rule with one thread per update, for index tensors whose lines are long or few: first every update proposes
// its position along `dim` for its destination (atomicMax -- two updates can only meet on one line, where a later
// position means a later visit in row-major order), then the update that holds the destination's maximum stores.
template <class I>
__device__ __forceinline__ bool scatter_target(const I* __restrict__ index, long long i, const Shape& src, const Shape& idx,
                                               const Shape& ups, int dim, int* status, long long* dst, long long* u_off, int* k) {
    const long long sel = (long long)index[i];
    if (sel < 0 || sel >= src.ext[dim]) {
        *status = MIMK_E_SHAPE;
        return false;
    }
    long long rest = i, o = 0, u = 0, o_str = 1, u_str = 1;
    for (int d = idx.rank - 1; d >= 0; --d) {
        const long long c = rest % idx.ext[d];
        rest /= idx.ext[d];
        if (d == dim) *k = int(c);
        o += (d == dim ? sel : c) * o_str;
        u += c * u_str;
        o_str *= src.ext[d], u_str *= ups.ext[d];
    }
    *dst = o, *u_off = u;
    return true;
}
template <class I>
__global__ void scatter_propose_kernel(const I* __restrict__ index, int* __restrict__ winner, long long n, Shape src, Shape idx,
                                       Shape ups, int dim, int* status) {
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
        long long dst, u;
        int k;
        if (scatter_target(index, i, src, idx, ups, dim, status, &dst, &u, &k)) atomicMax(winner + dst, k);
    }
}
template <class T, class I>
__global__ void scatter_commit_kernel(const I* __restrict__ index, const T* __restrict__ upd, const int* __restrict__ winner,
                                      T* __restrict__ out, long long n, Shape src, Shape idx, Shape ups, int dim, int* status) {
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
        long long dst, u;
        int k;
        if (scatter_target(index, i, src, idx, ups, dim, status, &dst, &u, &k) && winner[dst] == k) out[dst] = upd[u];
    }
}

// out[i] = cond[i] ? a[i] : b[i]   (tensor.select, tensor.mim:378-384; cond one byte per element, non-zero = true)
template <class T>
__global__ void select_kernel(const uint8_t* __restrict__ cond, const T* __restrict__ a, const T* __restrict__ b, T* __restrict__ out,
                              long long n) {
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x)
        out[i] = cond[i] ? a[i] : b[i];
}

bool load_shape(Shape& s, int rank, const int64_t* ext, long long* total) {
    if (rank < 0 || rank > MAX_RANK || (rank > 0 && !ext)) return false;
    s.rank = rank;
    long long n = 1;
    for (int d = 0; d < rank; ++d) {
        if (ext[d] < 0) return false;
        s.ext[d] = ext[d];
        n *= ext[d];
    }
    *total = n;
    return true;
}

unsigned grid_for(DeviceInfo* dev, long long n, int block = 256) {
    long long g = (n + block - 1) / block;
    const long long cap = (long long)dev->sm_count * 16;
    return unsigned(g < cap ? (g < 1 ? 1 : g) : cap);
}

}  // namespace
}  // namespace mimk

using namespace mimk;

extern "C" int mimk_splat(void* out, int dtype, int64_t n, int64_t value_bits, void* stream) {
    if (n < 0) return MIMK_E_ARG;
    if (dtype != MIMK_F32 && dtype != MIMK_BF16 && dtype != MIMK_I32 && dtype != MIMK_I64) return MIMK_E_DTYPE;
    int st          = MIMK_OK;
    DeviceInfo* dev = device_info(&st);
    if (!dev) return st;
    if (n == 0) return MIMK_OK;
    if (!out) return MIMK_E_ARG;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const unsigned g = grid_for(dev, n);
    switch (dtype_size(dtype)) {
        case 2: splat_kernel<uint16_t><<<g, 256, 0, s>>>(static_cast<uint16_t*>(out), n, uint16_t(value_bits)); break;
        case 4: splat_kernel<uint32_t><<<g, 256, 0, s>>>(static_cast<uint32_t*>(out), n, uint32_t(value_bits)); break;
        default: splat_kernel<uint64_t><<<g, 256, 0, s>>>(static_cast<uint64_t*>(out), n, uint64_t(value_bits)); break;
    }
    return launch_status();
}

extern "C" int mimk_generate_affine(void* out, int dtype, int rank, const int64_t* shape, const int64_t* coef, void* stream) {
    Shape sh;
    long long n = 0;
    if (!load_shape(sh, rank, shape, &n) || !coef) return MIMK_E_ARG;
    if (dtype != MIMK_F32 && dtype != MIMK_I32 && dtype != MIMK_I64) return MIMK_E_DTYPE;
    int st          = MIMK_OK;
    DeviceInfo* dev = device_info(&st);
    if (!dev) return st;
    if (n == 0) return MIMK_OK;
    if (!out) return MIMK_E_ARG;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    Coef dc{};
    for (int d = 0; d <= rank; ++d) dc.c[d] = coef[d];
    const unsigned g = grid_for(dev, n);
    if (dtype == MIMK_F32) generate_affine_kernel<float><<<g, 256, 0, s>>>(static_cast<float*>(out), n, sh, dc);
    else if (dtype == MIMK_I32) generate_affine_kernel<int><<<g, 256, 0, s>>>(static_cast<int*>(out), n, sh, dc);
    else generate_affine_kernel<long long><<<g, 256, 0, s>>>(static_cast<long long*>(out), n, sh, dc);
    return launch_status();
}

namespace {

template <class T>
int gather_typed(const void* in, const void* index, void* out, int index_dtype, long long n, const Shape& src, const Shape& idx,
                 int dim, DeviceInfo* dev, cudaStream_t s) {
    const unsigned g = grid_for(dev, n);
    if (index_dtype == MIMK_I32)
        gather_kernel<T, int><<<g, 256, 0, s>>>(static_cast<const T*>(in), static_cast<const int*>(index), static_cast<T*>(out), n, src,
                                                 idx, dim, dev->status_dev);
    else
        gather_kernel<T, long long><<<g, 256, 0, s>>>(static_cast<const T*>(in), static_cast<const long long*>(index),
                                                       static_cast<T*>(out), n, src, idx, dim, dev->status_dev);
    return launch_status();
}

template <class T, class I>
int scatter_any(const I* index, const T* upd, T* out, long long n_idx, long long n_src, const Shape& src, const Shape& idx,
                const Shape& ups, int dim, DeviceInfo* dev, cudaStream_t s) {
    const long long lines = n_idx / idx.ext[dim];
    // few or long lines leave one-thread-per-line without parallelism: one thread per update and a winner per destination.
    // The winner table has one int per element of the input and is cleared on every call, so this pays only while the
    // input is not much larger than the index tensor: a handful of updates into a huge table keeps the per-line kernel,
    // which touches the updated cells alone.
    if (n_idx >= 4096 && idx.ext[dim] > 4 && idx.ext[dim] < (int64_t(1) << 31) && n_src <= 8 * n_idx) {
        void* scratch = nullptr;
        MIMK_TRY(get_scratch(size_t(n_src) * sizeof(int), &scratch, s));
        int* winner = static_cast<int*>(scratch);
        MIMK_CUDA_TRY(cudaMemsetAsync(winner, 0xff, size_t(n_src) * sizeof(int), s));  // -1: no update names this cell
        const unsigned g = grid_for(dev, n_idx);
        scatter_propose_kernel<I><<<g, 256, 0, s>>>(index, winner, n_idx, src, idx, ups, dim, dev->status_dev);
        MIMK_TRY(launch_status());
        scatter_commit_kernel<T, I><<<g, 256, 0, s>>>(index, upd, winner, out, n_idx, src, idx, ups, dim, dev->status_dev);
        return launch_status();
    }
    const unsigned g = grid_for(dev, lines, 128);
    scatter_kernel<T, I><<<g, 128, 0, s>>>(index, upd, out, lines, src, idx, ups, dim, dev->status_dev);
    return launch_status();
}

template <class T>
int scatter_typed(const void* index, const void* upd, void* out, int index_dtype, long long n_idx, long long n_src, const Shape& src,
                  const Shape& idx, const Shape& ups, int dim, DeviceInfo* dev, cudaStream_t s) {
    if (index_dtype == MIMK_I32)
        return scatter_any(static_cast<const int*>(index), static_cast<const T*>(upd), static_cast<T*>(out), n_idx, n_src, src, idx, ups,
                           dim, dev, s);
    return scatter_any(static_cast<const long long*>(index), static_cast<const T*>(upd), static_cast<T*>(out), n_idx, n_src, src, idx,
                       ups, dim, dev, s);
}

bool value_dtype_ok(int dt) { return dt == MIMK_F32 || dt == MIMK_BF16 || dt == MIMK_I32 || dt == MIMK_I64; }

}  // namespace

extern "C" int mimk_gather(const void* input, const void* index, void* out, int dtype, int index_dtype, int rank,
                           const int64_t* s_src, const int64_t* s_idx, int dim, void* stream) {
    Shape src, idx;
    long long n_src = 0, n = 0;
    if (!load_shape(src, rank, s_src, &n_src) || !load_shape(idx, rank, s_idx, &n)) return MIMK_E_ARG;
    if (rank < 1 || dim < 0 || dim >= rank) return MIMK_E_ARG;
    if (!value_dtype_ok(dtype) || (index_dtype != MIMK_I32 && index_dtype != MIMK_I64)) return MIMK_E_DTYPE;
    for (int d = 0; d < rank; ++d)
        if (d != dim && idx.ext[d] > src.ext[d]) return MIMK_E_SHAPE;  // s_idx#d <= s_src#d off the indexed axis
    int st          = MIMK_OK;
    DeviceInfo* dev = device_info(&st);
    if (!dev) return st;
    if (n == 0) return MIMK_OK;
    if (!input || !index || !out) return MIMK_E_ARG;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    switch (dtype_size(dtype)) {
        case 2: return gather_typed<uint16_t>(input, index, out, index_dtype, n, src, idx, dim, dev, s);
        case 4: return gather_typed<uint32_t>(input, index, out, index_dtype, n, src, idx, dim, dev, s);
        default: return gather_typed<uint64_t>(input, index, out, index_dtype, n, src, idx, dim, dev, s);
    }
}

extern "C" int mimk_scatter(const void* input, const void* index, const void* updates, void* out, int dtype, int index_dtype,
                            int rank, const int64_t* s_src, const int64_t* s_idx, const int64_t* s_updates, int dim, void* stream) {
    Shape src, idx, ups;
    long long n_src = 0, n_idx = 0, n_ups = 0;
    if (!load_shape(src, rank, s_src, &n_src) || !load_shape(idx, rank, s_idx, &n_idx) || !load_shape(ups, rank, s_updates, &n_ups))
        return MIMK_E_ARG;
    if (rank < 1 || dim < 0 || dim >= rank) return MIMK_E_ARG;
    if (!value_dtype_ok(dtype) || (index_dtype != MIMK_I32 && index_dtype != MIMK_I64)) return MIMK_E_DTYPE;
    for (int d = 0; d < rank; ++d) {
        if (d != dim && idx.ext[d] > src.ext[d]) return MIMK_E_SHAPE;
        if (idx.ext[d] > ups.ext[d]) return MIMK_E_SHAPE;
    }
    int st          = MIMK_OK;
    DeviceInfo* dev = device_info(&st);
    if (!dev) return st;
    if (n_src == 0) return MIMK_OK;
    if (!input || !out) return MIMK_E_ARG;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (out != input)
        MIMK_CUDA_TRY(cudaMemcpyAsync(out, input, size_t(n_src) * dtype_size(dtype), cudaMemcpyDeviceToDevice, s));
    if (n_idx == 0) return MIMK_OK;
    if (!index || !updates) return MIMK_E_ARG;
    switch (dtype_size(dtype)) {
        case 2: return scatter_typed<uint16_t>(index, updates, out, index_dtype, n_idx, n_src, src, idx, ups, dim, dev, s);
        case 4: return scatter_typed<uint32_t>(index, updates, out, index_dtype, n_idx, n_src, src, idx, ups, dim, dev, s);
        default: return scatter_typed<uint64_t>(index, updates, out, index_dtype, n_idx, n_src, src, idx, ups, dim, dev, s);
    }
}

extern "C" int mimk_select(const void* cond, const void* a, const void* b, void* out, int dtype, int64_t n, void* stream) {
    if (n < 0) return MIMK_E_ARG;
    if (!value_dtype_ok(dtype)) return MIMK_E_DTYPE;
    int st          = MIMK_OK;
    DeviceInfo* dev = device_info(&st);
    if (!dev) return st;
    if (n == 0) return MIMK_OK;
    if (!cond || !a || !b || !out) return MIMK_E_ARG;
    cudaStream_t s   = static_cast<cudaStream_t>(stream);
    const unsigned g = grid_for(dev, n);
    const uint8_t* c = static_cast<const uint8_t*>(cond);
    switch (dtype_size(dtype)) {
        case 2: select_kernel<uint16_t><<<g, 256, 0, s>>>(c, static_cast<const uint16_t*>(a), static_cast<const uint16_t*>(b), static_cast<uint16_t*>(out), n); break;
        case 4: select_kernel<uint32_t><<<g, 256, 0, s>>>(c, static_cast<const uint32_t*>(a), static_cast<const uint32_t*>(b), static_cast<uint32_t*>(out), n); break;
        default: select_kernel<uint64_t><<<g, 256, 0, s>>>(c, static_cast<const uint64_t*>(a), static_cast<const uint64_t*>(b), static_cast<uint64_t*>(out), n); break;
    }
    return launch_status();
}
