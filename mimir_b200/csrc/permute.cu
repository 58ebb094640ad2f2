// Axis permutation of a dense tensor (tensor.transpose, MimIR src/mim/plug/tensor/tensor.mim:1443-1468: a copy-style
// map_reduce_post whose input map is `transpose_map`) as a tiled copy: a 64 x 64 tile over the output's fastest axis
// and the input's fastest axis goes through shared memory, so both the reads and the writes are coalesced. The
// per-cell kernel reads such an instance with a stride between neighbouring threads.
#include "common.cuh"

namespace mimk {
namespace {

constexpr int TILE = 64, ROWS = 4;  // 64 x 64 elements per step, 16 loads in flight per thread

struct PermuteParams {
    int rank;                          // output loops (<= MIMK_MRP_MAX_RANK)
    int qy;                            // the output loop along which the INPUT is contiguous (!= rank - 1)
    int64_t shape[MIMK_MRP_MAX_RANK];  // output extents
    int64_t istr[MIMK_MRP_MAX_RANK];   // input stride (elements) of each output loop
    int64_t ostr[MIMK_MRP_MAX_RANK];   // output stride (elements) of each output loop
    int64_t tiles_x, tiles_y, n_blocks;
};

template <class T>
__global__ void __launch_bounds__(TILE * ROWS) permute_kernel(const T* __restrict__ in, T* __restrict__ out, const PermuteParams p) {
    __shared__ T tile[TILE][TILE + 1];
    const int xl = p.rank - 1, yl = p.qy;
    for (int64_t blk = blockIdx.x; blk < p.n_blocks; blk += gridDim.x) {
        int64_t rest    = blk;
        const int64_t x0 = (rest % p.tiles_x) * TILE;
        rest /= p.tiles_x;
        const int64_t y0 = (rest % p.tiles_y) * TILE;
        rest /= p.tiles_y;
        int64_t ibase = 0, obase = 0;
        for (int l = p.rank - 2; l >= 0; --l) {  // the remaining loops, fastest first
            if (l == yl) continue;
            const int64_t c = rest % p.shape[l];
            rest /= p.shape[l];
            ibase += c * p.istr[l];
            obase += c * p.ostr[l];
        }
        // read: threadIdx.x runs along the input's contiguous axis
        const int64_t y = y0 + threadIdx.x;
#pragma unroll
        for (int k = 0; k < TILE; k += ROWS) {
            const int64_t x = x0 + threadIdx.y + k;
            if (x < p.shape[xl] && y < p.shape[yl]) tile[threadIdx.y + k][threadIdx.x] = in[ibase + y * p.istr[yl] + x * p.istr[xl]];
        }
        __syncthreads();
        // write: threadIdx.x runs along the output's contiguous axis
        const int64_t xo = x0 + threadIdx.x;
#pragma unroll
        for (int k = 0; k < TILE; k += ROWS) {
            const int64_t yo = y0 + threadIdx.y + k;
            if (xo < p.shape[xl] && yo < p.shape[yl]) out[obase + xo * p.ostr[xl] + yo * p.ostr[yl]] = tile[threadIdx.x][threadIdx.y + k];
        }
        __syncthreads();
    }
}

// Two-byte elements, both transposed extents even: the same tiled copy moving PAIRS -- 32-bit global loads along the
// input's contiguous axis, 32-bit global stores along the output's -- over a tile of 128 x 128 elements.
constexpr int PT = 128, PROWS = 4, PPITCH = PT + 2;
__global__ void __launch_bounds__(64 * PROWS) permute_pairs_kernel(const uint16_t* __restrict__ in, uint16_t* __restrict__ out,
                                                                   const PermuteParams p) {
    __shared__ __align__(4) uint16_t tile[PT][PPITCH];
    const int xl = p.rank - 1, yl = p.qy;
    for (int64_t blk = blockIdx.x; blk < p.n_blocks; blk += gridDim.x) {
        int64_t rest    = blk;
        const int64_t x0 = (rest % p.tiles_x) * PT;
        rest /= p.tiles_x;
        const int64_t y0 = (rest % p.tiles_y) * PT;
        rest /= p.tiles_y;
        int64_t ibase = 0, obase = 0;
        for (int l = p.rank - 2; l >= 0; --l) {
            if (l == yl) continue;
            const int64_t c = rest % p.shape[l];
            rest /= p.shape[l];
            ibase += c * p.istr[l];
            obase += c * p.ostr[l];
        }
        const int64_t y = y0 + 2 * threadIdx.x;  // this thread's pair along the input's contiguous axis
#pragma unroll 8
        for (int k = 0; k < PT; k += PROWS) {
            const int64_t x = x0 + threadIdx.y + k;
            if (x < p.shape[xl] && y < p.shape[yl])
                *reinterpret_cast<uint32_t*>(&tile[threadIdx.y + k][2 * threadIdx.x]) =
                    *reinterpret_cast<const uint32_t*>(in + ibase + y + x * p.istr[xl]);
        }
        __syncthreads();
        const int64_t xo = x0 + 2 * threadIdx.x;  // this thread's pair along the output's contiguous axis
#pragma unroll 8
        for (int k = 0; k < PT; k += PROWS) {
            const int yo_l    = threadIdx.y + k;
            const int64_t yo  = y0 + yo_l;
            if (xo < p.shape[xl] && yo < p.shape[yl]) {
                const uint32_t v = uint32_t(tile[2 * threadIdx.x][yo_l]) | (uint32_t(tile[2 * threadIdx.x + 1][yo_l]) << 16);
                *reinterpret_cast<uint32_t*>(out + obase + xo + yo * p.ostr[yl]) = v;
            }
        }
        __syncthreads();
    }
}

}  // namespace

// out[o] = in[o permuted]: `perm[j]` is the output loop that indexes input axis j. `esize` = bytes per element (2, 4, 8).
// Returns MIMK_E_UNSUPPORTED when the fastest axes of input and output coincide (a strided copy, no transposition).
int permute_copy(const void* in, void* out, int esize, int rank, const int64_t* out_shape, const int* perm, cudaStream_t s) {
    if (rank < 2 || rank > MIMK_MRP_MAX_RANK) return MIMK_E_UNSUPPORTED;
    if (perm[rank - 1] == rank - 1) return MIMK_E_UNSUPPORTED;
    int st          = MIMK_OK;
    DeviceInfo* dev = device_info(&st);
    if (!dev) return st;
    PermuteParams p;
    p.rank = rank;
    p.qy   = perm[rank - 1];
    int64_t total = 1;
    for (int l = 0; l < rank; ++l) p.shape[l] = out_shape[l], total *= out_shape[l];
    if (total == 0) return MIMK_OK;
    int64_t stride = 1;
    for (int l = rank - 1; l >= 0; --l) p.ostr[l] = stride, stride *= out_shape[l];
    stride = 1;
    for (int j = rank - 1; j >= 0; --j) p.istr[perm[j]] = stride, stride *= out_shape[perm[j]];
    const bool pairs = esize == 2 && p.shape[rank - 1] % 2 == 0 && p.shape[p.qy] % 2 == 0 &&
                       (reinterpret_cast<uintptr_t>(in) & 3u) == 0 && (reinterpret_cast<uintptr_t>(out) & 3u) == 0;
    const int tile = pairs ? PT : TILE;
    p.tiles_x  = (p.shape[rank - 1] + tile - 1) / tile;
    p.tiles_y  = (p.shape[p.qy] + tile - 1) / tile;
    p.n_blocks = p.tiles_x * p.tiles_y;
    for (int l = 0; l < rank - 1; ++l)
        if (l != p.qy) p.n_blocks *= p.shape[l];
    const int64_t cap = int64_t(dev->sm_count) * 32;
    const unsigned grid = unsigned(p.n_blocks < cap ? p.n_blocks : cap);
    if (pairs) {
        permute_pairs_kernel<<<grid, dim3(64, PROWS), 0, s>>>(static_cast<const uint16_t*>(in), static_cast<uint16_t*>(out), p);
        return launch_status();
    }
    const dim3 block(TILE, ROWS);
    switch (esize) {
        case 2: permute_kernel<uint16_t><<<grid, block, 0, s>>>(static_cast<const uint16_t*>(in), static_cast<uint16_t*>(out), p); break;
        case 4: permute_kernel<uint32_t><<<grid, block, 0, s>>>(static_cast<const uint32_t*>(in), static_cast<uint32_t*>(out), p); break;
        case 8: permute_kernel<uint64_t><<<grid, block, 0, s>>>(static_cast<const uint64_t*>(in), static_cast<uint64_t*>(out), p); break;
        default: return MIMK_E_DTYPE;
    }
    return launch_status();
}

}  // namespace mimk
