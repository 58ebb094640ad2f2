// The generic `map_reduce_post`: every instance the specialised kernels do not take.
//
// Semantics follow the reference's value-world lowering (MimIR src/mim/plug/tensor/phase/lower_map_reduce.cpp:93-206):
// output loops over the leading Ro bounds of Sr, the accumulator seeded with `init`, the trailing loops folded in
// ascending order with the combiner, `post` applied once per cell with the epilogue inputs read at the write
// coordinates, the result stored at `map_out` of the output loop vector (reduction slots 0). The launch shape is the
// reference GPU lowering's (one thread per output cell, lower_map_reduce.cpp:132-139, 198-206); what differs is that
// maps, combiner and epilogue are data, not generated code, and that the host proves every access in range first.
#include "common.cuh"

namespace mimk {
namespace {

struct Val {
    long long i;
    float f;
};

__device__ __forceinline__ Val load_val(const void* p, int dt, long long off) {
    Val v;
    v.i = 0;
    v.f = 0.f;
    switch (dt) {
        case MIMK_F32: v.f = static_cast<const float*>(p)[off]; break;
        case MIMK_BF16: v.f = __bfloat162float(static_cast<const __nv_bfloat16*>(p)[off]); break;
        case MIMK_I32: v.i = static_cast<const int*>(p)[off]; break;
        default: v.i = static_cast<const long long*>(p)[off]; break;
    }
    return v;
}

__device__ __forceinline__ long long wrap(long long x, int dt) { return dt == MIMK_I32 ? (long long)(int)x : x; }

__device__ __forceinline__ Val combine(int id, int acc_dt, Val acc, const Val* in) {
    Val r = acc;
    if (acc_dt == MIMK_F32) {
        switch (id) {
            case MIMK_F_ADD: r.f = acc.f + in[0].f; break;
            case MIMK_F_MULADD: r.f = fmaf(in[0].f, in[1].f, acc.f); break;
            case MIMK_F_MAX: r.f = fmaxf(acc.f, in[0].f); break;
            case MIMK_F_MIN: r.f = fminf(acc.f, in[0].f); break;
            case MIMK_F_FIRST: r.f = in[0].f; break;
            case MIMK_F_SUBEXP: r.f = expf(in[0].f - in[1].f); break;
            case MIMK_F_DIV: r.f = in[0].f / in[1].f; break;
            case MIMK_F_ADD2: r.f = in[0].f + in[1].f; break;
            case MIMK_F_MUL2: r.f = in[0].f * in[1].f; break;
            case MIMK_F_ADD_SUBEXP: r.f = acc.f + expf(in[0].f - in[1].f); break;
            case MIMK_F_SUBEXP_DIV: r.f = expf(in[0].f - in[1].f) / in[2].f; break;
            default:
                if (id & MIMK_F_COMPOSED_BASE) {  // fold(acc, outer(inner(a, b))): a producer inlined into the operand read
                    const float v = apply_op((id >> 16) & 0xff, apply_op((id >> 8) & 0xff, in[0].f, in[1].f), 0.f);
                    switch (id & 0xff) {
                        case MIMK_F_ADD: r.f = acc.f + v; break;
                        case MIMK_F_MAX: r.f = fmaxf(acc.f, v); break;
                        case MIMK_F_MIN: r.f = fminf(acc.f, v); break;
                        default: r.f = v; break;
                    }
                }
                break;
        }
    } else {
        unsigned long long a = (unsigned long long)acc.i, x = (unsigned long long)in[0].i, y = (unsigned long long)in[1].i;
        switch (id) {
            case MIMK_F_ADD: a = a + x; break;
            case MIMK_F_MULADD: a = a + x * y; break;
            case MIMK_F_MAX: a = (unsigned long long)(acc.i > in[0].i ? acc.i : in[0].i); break;
            case MIMK_F_MIN: a = (unsigned long long)(acc.i < in[0].i ? acc.i : in[0].i); break;
            case MIMK_F_FIRST: a = x; break;
            case MIMK_F_ADD2: a = x + y; break;
            case MIMK_F_MUL2: a = x * y; break;
            case MIMK_F_MIX: a = a + x + y; break;
            default: break;
        }
        r.i = wrap((long long)a, acc_dt);
    }
    return r;
}

__device__ __forceinline__ void store_post(int post, int acc_dt, int out_dt, Val acc, Val p0, void* out, long long off) {
    if (acc_dt == MIMK_F32) {
        float v = acc.f;
        switch (post) {
            case MIMK_P_ADD: v = acc.f + p0.f; break;
            case MIMK_P_ADD_PLUS1: v = acc.f + p0.f + 1.f; break;
            case MIMK_P_ADD_RELU: v = fmaxf(0.f, acc.f + p0.f); break;
            case MIMK_P_ADD_TANH: v = tanhf(acc.f + p0.f); break;
            case MIMK_P_RELU: v = fmaxf(0.f, acc.f); break;
            case MIMK_P_SILU: v = acc.f / (1.f + expf(-acc.f)); break;
            default: break;
        }
        if (out_dt == MIMK_BF16)
            static_cast<__nv_bfloat16*>(out)[off] = __float2bfloat16_rn(v);
        else
            static_cast<float*>(out)[off] = v;
    } else {
        // unsigned widening of a 32-bit accumulator into a 64-bit result (core.conv.u), then the epilogue
        unsigned long long a = acc_dt == MIMK_I32 && out_dt == MIMK_I64 ? (unsigned long long)(unsigned int)acc.i
                                                                       : (unsigned long long)acc.i;
        switch (post) {
            case MIMK_P_ADD: a = a + (unsigned long long)p0.i; break;
            case MIMK_P_ADD_PLUS1: a = a + (unsigned long long)p0.i + 1ull; break;
            case MIMK_P_RELU: a = (long long)a > 0 ? a : 0ull; break;
            default: break;
        }
        if (out_dt == MIMK_I32)
            static_cast<int*>(out)[off] = (int)a;
        else
            static_cast<long long*>(out)[off] = (long long)a;
    }
}

__device__ __forceinline__ long long map_offset(const mimk_affine_map& m, int n, const long long* loop, const int64_t* shape) {
    unsigned long long off = 0;
    for (int j = 0; j < m.rows; ++j) {
        unsigned long long v = (unsigned long long)m.coef[j][n];
        for (int l = 0; l < n; ++l) v += (unsigned long long)m.coef[j][l] * (unsigned long long)loop[l];
        if (m.div[j] > 0) v /= (unsigned long long)m.div[j];  // affine.semiop.floordiv, then rem: the shape of delinearize
        if (m.mod[j] > 0) v %= (unsigned long long)m.mod[j];
        off = off * (unsigned long long)shape[j] + v;
    }
    return (long long)off;
}

__global__ void __launch_bounds__(256) mrp_generic_kernel(const __grid_constant__ mimk_mrp_desc d, long long n_out,
                                                         long long n_red) {
    for (long long o = blockIdx.x * (long long)blockDim.x + threadIdx.x; o < n_out; o += (long long)gridDim.x * blockDim.x) {
        long long loop[MIMK_MRP_MAX_LOOPS];
        long long rem = o;
        for (int l = d.ro - 1; l >= 0; --l) {
            loop[l] = rem % d.sr[l];
            rem /= d.sr[l];
        }
        Val acc;
        acc.i = d.acc_dtype == MIMK_I32 ? (long long)(int)d.init_bits : d.init_bits;
        acc.f = __int_as_float((int)d.init_bits);
        for (long long r = 0; r < n_red; ++r) {
            long long rr = r;
            for (int l = d.rn - 1; l >= d.ro; --l) {
                loop[l] = rr % d.sr[l];
                rr /= d.sr[l];
            }
            Val in[MIMK_MRP_MAX_INPUTS];
            for (int i = 0; i < d.nis; ++i)
                in[i] = load_val(d.in[i], d.in_dtype[i], map_offset(d.in_map[i], d.rn, loop, d.in_shape[i]));
            for (int i = d.nis; i < 3; ++i) in[i].i = 0, in[i].f = 0.f;
            acc = combine(d.comb, d.acc_dtype, acc, in);
        }
        for (int l = d.ro; l < d.rn; ++l) loop[l] = 0;
        long long wc[MIMK_MRP_MAX_RANK];
        for (int j = 0; j < d.ro; ++j) {
            unsigned long long v = (unsigned long long)d.map_out.coef[j][d.rn];
            for (int l = 0; l < d.rn; ++l) v += (unsigned long long)d.map_out.coef[j][l] * (unsigned long long)loop[l];
            if (d.map_out.div[j] > 0) v /= (unsigned long long)d.map_out.div[j];
            if (d.map_out.mod[j] > 0) v %= (unsigned long long)d.map_out.mod[j];
            wc[j] = (long long)v;
        }
        Val p0;
        p0.i = 0, p0.f = 0.f;
        if (d.nps > 0) p0 = load_val(d.post_in[0], d.post_dtype[0], map_offset(d.post_map[0], d.ro, wc, d.post_shape[0]));
        unsigned long long woff = 0;
        for (int j = 0; j < d.ro; ++j) woff = woff * (unsigned long long)d.so[j] + (unsigned long long)wc[j];
        store_post(d.post, d.acc_dtype, d.out_dtype, acc, p0, d.out, (long long)woff);
    }
}

// The same walk for instances whose input maps carry no floordiv / rem -- all but the reshape family: every input's offset
// is then ONE linear form of the loop vector (the host folds the row-major strides into the coefficients; in range was
// proven there, so the wrap-around arithmetic of the coordinates never wraps), and the reduction loops are walked like an
// odometer: an add per input and step instead of divisions and a matrix product. The fold order is unchanged (last loop
// fastest), so the results are the same bits.
struct LinearMaps {
    long long base[MIMK_MRP_MAX_INPUTS];
    long long lin[MIMK_MRP_MAX_INPUTS][MIMK_MRP_MAX_LOOPS];
};
__global__ void __launch_bounds__(256) mrp_linear_kernel(const __grid_constant__ mimk_mrp_desc d, const __grid_constant__ LinearMaps lm,
                                                        long long n_out, long long n_red) {
    for (long long o = blockIdx.x * (long long)blockDim.x + threadIdx.x; o < n_out; o += (long long)gridDim.x * blockDim.x) {
        long long loop[MIMK_MRP_MAX_LOOPS];
        if (n_out < (1ll << 31)) {  // every extent then fits 32 bits too: a 32-bit division costs a fifth of a 64-bit one
            unsigned rem = (unsigned)o;
            for (int l = d.ro - 1; l >= 0; --l) {
                const unsigned e = (unsigned)d.sr[l], q = rem / e;
                loop[l] = rem - q * e;
                rem     = q;
            }
        } else {
            long long rem = o;
            for (int l = d.ro - 1; l >= 0; --l) {
                loop[l] = rem % d.sr[l];
                rem /= d.sr[l];
            }
        }
        long long off[MIMK_MRP_MAX_INPUTS];
        for (int i = 0; i < d.nis; ++i) {
            off[i] = lm.base[i];
            for (int l = 0; l < d.ro; ++l) off[i] += lm.lin[i][l] * loop[l];
        }
        long long cnt[MIMK_MRP_MAX_LOOPS];
        for (int l = d.ro; l < d.rn; ++l) cnt[l] = 0;
        Val acc;
        acc.i = d.acc_dtype == MIMK_I32 ? (long long)(int)d.init_bits : d.init_bits;
        acc.f = __int_as_float((int)d.init_bits);
        for (long long r = 0; r < n_red; ++r) {
            Val in[MIMK_MRP_MAX_INPUTS];
            for (int i = 0; i < d.nis; ++i) in[i] = load_val(d.in[i], d.in_dtype[i], off[i]);
            for (int i = d.nis; i < 3; ++i) in[i].i = 0, in[i].f = 0.f;
            acc = combine(d.comb, d.acc_dtype, acc, in);
            for (int l = d.rn - 1; l >= d.ro; --l) {  // next point of the reduction box
                for (int i = 0; i < d.nis; ++i) off[i] += lm.lin[i][l];
                if (++cnt[l] < d.sr[l]) break;
                for (int i = 0; i < d.nis; ++i) off[i] -= lm.lin[i][l] * d.sr[l];
                cnt[l] = 0;
            }
        }
        for (int l = d.ro; l < d.rn; ++l) loop[l] = 0;
        long long wc[MIMK_MRP_MAX_RANK];
        for (int j = 0; j < d.ro; ++j) {
            unsigned long long v = (unsigned long long)d.map_out.coef[j][d.rn];
            for (int l = 0; l < d.rn; ++l) v += (unsigned long long)d.map_out.coef[j][l] * (unsigned long long)loop[l];
            if (d.map_out.div[j] > 0) v /= (unsigned long long)d.map_out.div[j];
            if (d.map_out.mod[j] > 0) v %= (unsigned long long)d.map_out.mod[j];
            wc[j] = (long long)v;
        }
        Val p0;
        p0.i = 0, p0.f = 0.f;
        if (d.nps > 0) p0 = load_val(d.post_in[0], d.post_dtype[0], map_offset(d.post_map[0], d.ro, wc, d.post_shape[0]));
        unsigned long long woff = 0;
        for (int j = 0; j < d.ro; ++j) woff = woff * (unsigned long long)d.so[j] + (unsigned long long)wc[j];
        store_post(d.post, d.acc_dtype, d.out_dtype, acc, p0, d.out, (long long)woff);
    }
}

// Folds the row-major strides of every input into its map's coefficients; false when a map has a floordiv / rem.
bool linear_maps(const mimk_mrp_desc& d, LinearMaps& lm) {
    for (int i = 0; i < d.nis; ++i) {
        const mimk_affine_map& m = d.in_map[i];
        lm.base[i] = 0;
        for (int l = 0; l < MIMK_MRP_MAX_LOOPS; ++l) lm.lin[i][l] = 0;
        long long stride = 1;
        for (int j = m.rows - 1; j >= 0; --j) {
            if (m.div[j] > 0 || m.mod[j] > 0) return false;
            lm.base[i] += m.coef[j][d.rn] * stride;
            for (int l = 0; l < d.rn; ++l) lm.lin[i][l] += m.coef[j][l] * stride;
            stride *= d.in_shape[i][j];
        }
    }
    return true;
}

// ---------------------------------------------------------------------------------------------------------------------
// The compiled form of the same walk, for the instances that matter in volume: floating-point windows (conv, conv_grouped,
// pool), patch gathers, pads and strided copies -- same element type everywhere, f32 accumulator, no epilogue operand, no
// floordiv / rem in any map, fewer than 2^31 cells. The host turns the descriptor into a plan: every operand's offset (the
// result's too) as one linear form of the loop vector, output loops of extent 1 dropped and neighbours merged where every
// form allows it (n and c of an NCHW pool become one loop), each remaining extent with the multiplier and shift that
// replace its division (Granlund-Montgomery, exact below 2^31), at most three reduction loops. The kernel is then
// straight-line: no local arrays, the combiner a template argument. Fold order per cell is unchanged (reduction loops in
// order, last fastest), so the results are the same bits as the interpreting kernels'.
// ---------------------------------------------------------------------------------------------------------------------
constexpr int WIN_OUT = 6, WIN_RED = 3;
struct WindowPlan {
    unsigned ext[WIN_OUT], mul[WIN_OUT], shift[WIN_OUT];  // output loops, unused ones in front with extent 1
    long long lin[4][WIN_OUT];                            // offset step per loop: inputs 0..2, result
    long long base[4];
    int rext[WIN_RED];                                    // reduction loops, unused ones in front with extent 1
    long long rlin[3][WIN_RED];
    int nis, comb, post;
    int first;  // first output loop in use
    int n_red_loops;  // reduction loops in use (for mimk_mrp_cell_kernel; the kernel walks all three slots)
    // The outermost loop in use cut into four equal parts (when its extent allows): a thread's four cells then share every
    // loop index but that one, their offsets differ by `quarter_step`, and one decomposition serves all four.
    int split;
    long long quarter_step[4];
    float init;
};

__device__ __forceinline__ size_t win_at(unsigned off) { return size_t(off); }
__device__ __forceinline__ size_t win_at(long long off) { return size_t(off); }
template <class T, class Off> __device__ __forceinline__ float win_ld(const T* p, Off off);
template <> __device__ __forceinline__ float win_ld<float, unsigned>(const float* p, unsigned off) { return __ldg(p + win_at(off)); }
template <> __device__ __forceinline__ float win_ld<float, long long>(const float* p, long long off) { return __ldg(p + win_at(off)); }
template <> __device__ __forceinline__ float win_ld<__nv_bfloat16, unsigned>(const __nv_bfloat16* p, unsigned off) {
    return __bfloat162float(__ldg(p + win_at(off)));
}
template <> __device__ __forceinline__ float win_ld<__nv_bfloat16, long long>(const __nv_bfloat16* p, long long off) {
    return __bfloat162float(__ldg(p + win_at(off)));
}

// COMB: one of MIMK_F_ADD / MULADD / MAX / MIN / FIRST, or -1 for "whatever the plan says" (any floating-point combiner).
// Off: unsigned when every operand has fewer than 2^31 elements -- offsets are then computed modulo 2^32, which is exact for
// the in-range values the host has proven them to be, at a third of the instructions of 64-bit arithmetic.
template <class T, int COMB, class Off, int CELLS>
__global__ void __launch_bounds__(256) mrp_window_kernel(const T* __restrict__ in0, const T* __restrict__ in1,
                                                        const T* __restrict__ in2, T* __restrict__ out,
                                                        const __grid_constant__ WindowPlan p, unsigned n_out) {
    const int comb = COMB >= 0 ? COMB : p.comb;
    const int nis  = COMB == MIMK_F_MULADD ? 2 : (COMB >= 0 ? 1 : p.nis);
    // CELLS = 4 cells per thread and pass when there are enough cells to go round: a copy-like instance has one load per
    // cell, and a thread with a single load in flight leaves the memory system idle -- 2048 threads x 4 bytes per SM is a
    // quarter of what the bandwidth-latency product needs.
    const unsigned long long step = gridDim.x * 256ull;
    const bool split               = CELLS == 4 && p.split;  // the same for every thread
    const unsigned long long limit = split ? n_out / 4 : n_out;
    for (unsigned long long o64 = blockIdx.x * 256ull + threadIdx.x; o64 < limit; o64 += split ? step : step * CELLS) {
        Off o0[CELLS], o1[CELLS], o2[CELLS], oo[CELLS];
        bool live[CELLS];
#pragma unroll
        for (int c = 0; c < CELLS; ++c) {
            if (split && c > 0) {  // cell c = cell 0 with the outermost index moved on by c quarters of its extent
                live[c] = true;
                o0[c] = o0[0] + Off(c) * Off(p.quarter_step[0]), o1[c] = o1[0] + Off(c) * Off(p.quarter_step[1]);
                o2[c] = o2[0] + Off(c) * Off(p.quarter_step[2]), oo[c] = oo[0] + Off(c) * Off(p.quarter_step[3]);
                continue;
            }
            const unsigned long long cell = o64 + c * step;
            live[c]      = cell < limit;
            unsigned rem = unsigned(live[c] ? cell : o64);  // a cell past the end repeats the first one and is not stored
            o0[c] = Off(p.base[0]), o1[c] = Off(p.base[1]), o2[c] = Off(p.base[2]), oo[c] = Off(p.base[3]);
#pragma unroll
            for (int l = WIN_OUT - 1; l >= 0; --l) {
                if (l < p.first) break;  // the same for every thread
                const unsigned q = __umulhi(rem, p.mul[l]) >> p.shift[l];
                const Off ix     = Off(rem - q * p.ext[l]);
                rem              = q;
                o0[c] += Off(p.lin[0][l]) * ix, oo[c] += Off(p.lin[3][l]) * ix;
                if (nis > 1) o1[c] += Off(p.lin[1][l]) * ix;
                if (nis > 2) o2[c] += Off(p.lin[2][l]) * ix;
            }
        }
        Val acc[CELLS];
#pragma unroll
        for (int c = 0; c < CELLS; ++c) acc[c].i = 0, acc[c].f = p.init;
        for (int r0 = 0; r0 < p.rext[0]; ++r0) {
            for (int r1 = 0; r1 < p.rext[1]; ++r1) {
                Off r01[3];  // this row of the window, relative to the cell
#pragma unroll
                for (int i = 0; i < 3; ++i) r01[i] = Off(r0) * Off(p.rlin[i][0]) + Off(r1) * Off(p.rlin[i][1]);
#pragma unroll 2
                for (int r2 = 0; r2 < p.rext[2]; ++r2) {
#pragma unroll
                    for (int c = 0; c < CELLS; ++c) {
                        Val in[3];
                        in[0].i = in[1].i = in[2].i = 0;
                        in[0].f = win_ld(in0, Off(o0[c] + r01[0]));
                        in[1].f = nis > 1 ? win_ld(in1, Off(o1[c] + r01[1])) : 0.f;
                        in[2].f = nis > 2 ? win_ld(in2, Off(o2[c] + r01[2])) : 0.f;
                        acc[c]  = combine(comb, MIMK_F32, acc[c], in);
                    }
#pragma unroll
                    for (int i = 0; i < 3; ++i) r01[i] += Off(p.rlin[i][2]);
                }
            }
        }
#pragma unroll
        for (int c = 0; c < CELLS; ++c) {
            float v = acc[c].f;
            if (p.post == MIMK_P_RELU) v = fmaxf(0.f, v);
            else if (p.post == MIMK_P_SILU) v = v / (1.f + expf(-v));
            if (!live[c]) continue;
            if (sizeof(T) == 2) reinterpret_cast<__nv_bfloat16*>(out)[win_at(oo[c])] = __float2bfloat16_rn(v);
            else reinterpret_cast<float*>(out)[win_at(oo[c])] = v;
        }
    }
}

// Builds the plan; false when the instance is outside what the compiled walk covers.
bool window_plan(const mimk_mrp_desc& d, const LinearMaps& lm, long long n_out, WindowPlan& p) {
    if (d.acc_dtype != MIMK_F32 || (d.out_dtype != MIMK_F32 && d.out_dtype != MIMK_BF16) || d.nps != 0) return false;
    if (d.post != MIMK_P_ID && d.post != MIMK_P_RELU && d.post != MIMK_P_SILU) return false;
    if (d.nis < 1 || d.nis > 3 || n_out >= (1ll << 31)) return false;
    for (int i = 0; i < d.nis; ++i)
        if (d.in_dtype[i] != d.out_dtype) return false;
    // the result's offset as a linear form of the output loops
    long long olin[MIMK_MRP_MAX_LOOPS] = {}, obase = 0, stride = 1;
    for (int j = d.map_out.rows - 1; j >= 0; --j) {
        if (d.map_out.div[j] > 0 || d.map_out.mod[j] > 0) return false;
        obase += d.map_out.coef[j][d.rn] * stride;
        for (int l = 0; l < d.ro; ++l) olin[l] += d.map_out.coef[j][l] * stride;
        stride *= d.so[j];
    }
    // loops as (extent, step of every form), innermost last; drop extent 1, merge neighbours every form agrees on
    struct Loop {
        long long ext, lin[4];
    };
    auto compact = [&](int first, int last, bool with_out, Loop* out_loops, int cap) -> int {
        int n = 0;
        for (int l = first; l < last; ++l) {
            if (d.sr[l] == 1) continue;
            Loop cur;
            cur.ext = d.sr[l];
            for (int i = 0; i < 3; ++i) cur.lin[i] = i < d.nis ? lm.lin[i][l] : 0;
            cur.lin[3] = with_out ? olin[l] : 0;
            bool merged = false;
            if (n > 0) {
                Loop& prev = out_loops[n - 1];  // prev is the outer neighbour: prev.lin == cur.lin * cur.ext on every form
                merged     = prev.ext * cur.ext < (1ll << 31);
                for (int f = 0; f < 4 && merged; ++f) merged = prev.lin[f] == cur.lin[f] * cur.ext;
                if (merged) {
                    prev.ext *= cur.ext;
                    for (int f = 0; f < 4; ++f) prev.lin[f] = cur.lin[f];
                }
            }
            if (!merged) {
                if (n == cap) return -1;
                out_loops[n++] = cur;
            }
        }
        return n;
    };
    Loop ol[WIN_OUT], rl[WIN_RED];
    const int no = compact(0, d.ro, true, ol, WIN_OUT);
    const int nr = compact(d.ro, d.rn, false, rl, WIN_RED);
    if (no < 0 || nr < 0) return false;
    for (int l = 0; l < WIN_OUT; ++l) {
        const int src = l - (WIN_OUT - no);
        const long long e = src >= 0 ? ol[src].ext : 1;
        p.ext[l] = unsigned(e);
        if (e == 1) {
            p.mul[l] = 0, p.shift[l] = 0;  // never looked at: loops before `first` are skipped
        } else {
            int sft = 0;
            while ((1ll << sft) < e) ++sft;  // ceil(log2 e)
            const unsigned __int128 one = 1;
            p.mul[l]   = unsigned(((one << (31 + sft)) + e - 1) / e);  // below 2^32 for e >= 2; exact quotients for n < 2^31
            p.shift[l] = unsigned(sft - 1);
        }
        for (int f = 0; f < 4; ++f) p.lin[f][l] = src >= 0 ? ol[src].lin[f] : 0;
    }
    for (int l = 0; l < WIN_RED; ++l) {
        const int src = l - (WIN_RED - nr);
        if (src >= 0 && rl[src].ext >= (1ll << 31)) return false;
        p.rext[l] = src >= 0 ? int(rl[src].ext) : 1;
        for (int i = 0; i < 3; ++i) p.rlin[i][l] = src >= 0 ? rl[src].lin[i] : 0;
    }
    for (int i = 0; i < 3; ++i) p.base[i] = i < d.nis ? lm.base[i] : 0;
    p.base[3] = obase;
    p.nis = d.nis, p.comb = d.comb, p.post = d.post, p.first = WIN_OUT - no;
    p.n_red_loops = nr;
    p.split = no > 0 && ol[0].ext % 4 == 0;
    for (int f = 0; f < 4; ++f) p.quarter_step[f] = p.split ? ol[0].lin[f] * (ol[0].ext / 4) : 0;
    const int bits = int(d.init_bits);
    memcpy(&p.init, &bits, sizeof(float));
    return true;
}

template <class T, class Off, int CELLS>
void launch_window(const mimk_mrp_desc& d, const WindowPlan& p, unsigned blocks, unsigned n_out, cudaStream_t s) {
    const T* a = static_cast<const T*>(d.in[0]);
    const T* b = static_cast<const T*>(d.nis > 1 ? d.in[1] : d.in[0]);
    const T* c = static_cast<const T*>(d.nis > 2 ? d.in[2] : d.in[0]);
    T* o       = static_cast<T*>(d.out);
    switch (d.comb) {
        case MIMK_F_ADD: mrp_window_kernel<T, MIMK_F_ADD, Off, CELLS><<<blocks, 256, 0, s>>>(a, b, c, o, p, n_out); break;
        case MIMK_F_MAX: mrp_window_kernel<T, MIMK_F_MAX, Off, CELLS><<<blocks, 256, 0, s>>>(a, b, c, o, p, n_out); break;
        case MIMK_F_MIN: mrp_window_kernel<T, MIMK_F_MIN, Off, CELLS><<<blocks, 256, 0, s>>>(a, b, c, o, p, n_out); break;
        case MIMK_F_FIRST: mrp_window_kernel<T, MIMK_F_FIRST, Off, CELLS><<<blocks, 256, 0, s>>>(a, b, c, o, p, n_out); break;
        case MIMK_F_MULADD:
            if (d.nis == 2) {
                mrp_window_kernel<T, MIMK_F_MULADD, Off, CELLS><<<blocks, 256, 0, s>>>(a, b, c, o, p, n_out);
                break;
            }
            [[fallthrough]];
        default: mrp_window_kernel<T, -1, Off, 1><<<blocks, 256, 0, s>>>(a, b, c, o, p, n_out); break;
    }
}

// Range of an access map over the box 0 <= loop[l] < bound[l]: every result coordinate must stay in [0, extent). The
// linear form is bounded first, then the floordiv / rem are applied to the bounds.
bool map_in_range(const mimk_affine_map& m, int n, const int64_t* bounds, const int64_t* shape) {
    for (int j = 0; j < m.rows; ++j) {
        __int128 lo = m.coef[j][n], hi = m.coef[j][n];
        for (int l = 0; l < n; ++l) {
            const __int128 c = m.coef[j][l];
            const __int128 span = c * (__int128)(bounds[l] - 1);
            if (span < 0) lo += span; else hi += span;
        }
        if (m.div[j] < 0 || m.mod[j] < 0) return false;
        if (m.div[j] > 0 || m.mod[j] > 0) {
            // the division is unsigned: a linear part that can go negative would wrap to a huge index
            if (lo < 0) return false;
            if (m.div[j] > 0) lo /= m.div[j], hi /= m.div[j];
            if (m.mod[j] > 0) {
                // inside one period the remainder keeps the interval; across a period boundary it covers [0, mod)
                if (lo / m.mod[j] == hi / m.mod[j]) lo %= m.mod[j], hi %= m.mod[j];
                else lo = 0, hi = m.mod[j] - 1;
            }
        }
        if (lo < 0 || hi >= (__int128)shape[j]) return false;
    }
    return true;
}

bool dtype_ok(int dt) { return dt == MIMK_F32 || dt == MIMK_BF16 || dt == MIMK_I32 || dt == MIMK_I64; }

}  // namespace
}  // namespace mimk

using namespace mimk;

extern "C" int mimk_mrp_cell_kernel(const mimk_mrp_desc* d, int32_t* loops) {
    if (loops) loops[0] = loops[1] = 0;
    if (!d || d->ro < 0 || d->rn < d->ro || d->rn > MIMK_MRP_MAX_LOOPS || d->ro > MIMK_MRP_MAX_RANK) return MIMK_CELL_INTERPRETED;
    if (d->nis < 0 || d->nis > MIMK_MRP_MAX_INPUTS || d->map_out.rows != d->ro) return MIMK_CELL_INTERPRETED;
    long long n_out = 1, n_red = 1;
    for (int l = 0; l < d->rn; ++l) {
        if (d->sr[l] < 0) return MIMK_CELL_INTERPRETED;
        (l < d->ro ? n_out : n_red) *= d->sr[l];
    }
    LinearMaps lm;
    WindowPlan wp;
    if (n_red <= 0 || !linear_maps(*d, lm)) return MIMK_CELL_INTERPRETED;
    if (!window_plan(*d, lm, n_out, wp)) return MIMK_CELL_LINEAR;
    if (loops) loops[0] = WIN_OUT - wp.first, loops[1] = wp.n_red_loops;
    return MIMK_CELL_COMPILED;
}

extern "C" int mimk_map_reduce_post(const mimk_mrp_desc* d, void* stream) {
    if (!d) return MIMK_E_ARG;
    if (d->ro < 0 || d->rn < d->ro || d->rn > MIMK_MRP_MAX_LOOPS || d->ro > MIMK_MRP_MAX_RANK) return MIMK_E_ARG;
    if (d->nis < 0 || d->nis > MIMK_MRP_MAX_INPUTS || d->nps < 0 || d->nps > 1) return MIMK_E_ARG;
    int c_fold = 0, c_inner = 0, c_outer = 0;
    const bool composed = decode_composed(d->comb, &c_fold, &c_inner, &c_outer);
    if (!composed && (d->comb < MIMK_F_ADD || d->comb > MIMK_F_SUBEXP_DIV)) return MIMK_E_ARG;
    if (d->post < MIMK_P_ID || d->post > MIMK_P_SILU) return MIMK_E_ARG;
    if (d->acc_dtype != MIMK_F32 && d->acc_dtype != MIMK_I32 && d->acc_dtype != MIMK_I64) return MIMK_E_DTYPE;
    const bool facc = d->acc_dtype == MIMK_F32;
    if (facc ? (d->out_dtype != MIMK_F32 && d->out_dtype != MIMK_BF16) : (d->out_dtype != MIMK_I32 && d->out_dtype != MIMK_I64))
        return MIMK_E_DTYPE;
    const int need = composed ? (op_is_binary(c_inner) ? 2 : 1) : d->comb == MIMK_F_SUBEXP_DIV ? 3
                     : (d->comb == MIMK_F_MULADD || d->comb == MIMK_F_SUBEXP || d->comb == MIMK_F_DIV || d->comb == MIMK_F_ADD2 ||
                        d->comb == MIMK_F_MUL2 || d->comb == MIMK_F_MIX || d->comb == MIMK_F_ADD_SUBEXP) ? 2 : 1;
    if (d->nis != need) return MIMK_E_ARG;
    if (!facc && (d->comb == MIMK_F_SUBEXP || d->comb == MIMK_F_DIV || d->comb == MIMK_F_ADD_SUBEXP || d->comb == MIMK_F_SUBEXP_DIV)) return MIMK_E_DTYPE;
    if (facc && d->comb == MIMK_F_MIX) return MIMK_E_DTYPE;
    if (composed && !facc) return MIMK_E_DTYPE;
    const bool post_needs = d->post >= MIMK_P_ADD && d->post <= MIMK_P_ADD_TANH;
    if (post_needs != (d->nps == 1)) return MIMK_E_ARG;
    if (!facc && (d->post == MIMK_P_ADD_RELU || d->post == MIMK_P_ADD_TANH || d->post == MIMK_P_SILU)) return MIMK_E_DTYPE;
    long long n_out = 1, n_red = 1;
    for (int l = 0; l < d->rn; ++l) {
        if (d->sr[l] < 0) return MIMK_E_ARG;
        if (l < d->ro) n_out *= d->sr[l]; else n_red *= d->sr[l];
    }
    for (int j = 0; j < d->ro; ++j)
        if (d->so[j] < 0) return MIMK_E_ARG;
    for (int i = 0; i < d->nis; ++i) {
        if (!dtype_ok(d->in_dtype[i]) || d->in_map[i].rows < 0 || d->in_map[i].rows > MIMK_MRP_MAX_RANK) return MIMK_E_ARG;
        if ((d->in_dtype[i] == MIMK_F32 || d->in_dtype[i] == MIMK_BF16) != facc) return MIMK_E_DTYPE;
    }
    if (d->nps == 1) {
        if (!dtype_ok(d->post_dtype[0]) || d->post_map[0].rows < 0 || d->post_map[0].rows > MIMK_MRP_MAX_RANK) return MIMK_E_ARG;
        if ((d->post_dtype[0] == MIMK_F32 || d->post_dtype[0] == MIMK_BF16) != facc) return MIMK_E_DTYPE;
    }
    if (d->map_out.rows != d->ro) return MIMK_E_SHAPE;
    int st          = MIMK_OK;
    DeviceInfo* dev = device_info(&st);
    if (!dev) return st;
    if (n_out == 0) return MIMK_OK;
    if (!d->out) return MIMK_E_ARG;
    // Prove every access in range over the whole iteration box before anything is launched.
    int64_t out_bounds[MIMK_MRP_MAX_LOOPS];
    for (int l = 0; l < d->rn; ++l) out_bounds[l] = l < d->ro ? d->sr[l] : 1;  // reduction slots are 0 at write-back
    if (!map_in_range(d->map_out, d->rn, out_bounds, d->so)) return MIMK_E_SHAPE;
    if (n_red > 0)
        for (int i = 0; i < d->nis; ++i) {
            if (!d->in[i]) return MIMK_E_ARG;
            if (!map_in_range(d->in_map[i], d->rn, d->sr, d->in_shape[i])) return MIMK_E_SHAPE;
        }
    if (d->nps == 1) {
        if (!d->post_in[0]) return MIMK_E_ARG;
        // the epilogue input is read at the write coordinates, which range over the result's shape
        if (!map_in_range(d->post_map[0], d->ro, d->so, d->post_shape[0])) return MIMK_E_SHAPE;
    }
    int routed = MIMK_OK;
    if (n_red > 0 && mrp_try_route(*d, stream, &routed)) return routed;
    long long blocks = (n_out + 255) / 256;
    const long long cap = (long long)dev->sm_count * 8;
    if (blocks > cap) blocks = cap;
    LinearMaps lm;
    WindowPlan wp;
    const bool linear = n_red > 0 && linear_maps(*d, lm);
    if (linear && window_plan(*d, lm, n_out, wp)) {
        bool narrow = true;  // every operand below 2^31 elements: 32-bit offsets
        long long cells = 1;
        for (int j = 0; j < d->ro; ++j) cells *= d->so[j];
        narrow = cells < (1ll << 31);
        for (int i = 0; i < d->nis; ++i) {
            cells = 1;
            for (int j = 0; j < d->in_map[i].rows; ++j) cells *= d->in_shape[i][j];
            narrow = narrow && cells < (1ll << 31);
        }
        const auto st = static_cast<cudaStream_t>(stream);
        const unsigned nb = (unsigned)blocks, no = (unsigned)n_out;
        const bool many = n_out >= cap * 256 * 8;  // every thread of a full grid gets at least two passes of four cells
        const bool f32  = d->out_dtype == MIMK_F32;
        if (many) {
            if (f32) narrow ? launch_window<float, unsigned, 4>(*d, wp, nb, no, st) : launch_window<float, long long, 4>(*d, wp, nb, no, st);
            else narrow ? launch_window<__nv_bfloat16, unsigned, 4>(*d, wp, nb, no, st) : launch_window<__nv_bfloat16, long long, 4>(*d, wp, nb, no, st);
        } else {
            if (f32) narrow ? launch_window<float, unsigned, 1>(*d, wp, nb, no, st) : launch_window<float, long long, 1>(*d, wp, nb, no, st);
            else narrow ? launch_window<__nv_bfloat16, unsigned, 1>(*d, wp, nb, no, st) : launch_window<__nv_bfloat16, long long, 1>(*d, wp, nb, no, st);
        }
    } else if (linear)
        mrp_linear_kernel<<<(unsigned)blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(*d, lm, n_out, n_red);
    else
        mrp_generic_kernel<<<(unsigned)blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(*d, n_out, n_red);
    return launch_status();
}
