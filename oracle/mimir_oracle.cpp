// TEST INFRASTRUCTURE ONLY -- CPU oracle for the MimIR `tensor` hot path.
//
// This file restates, in plain single-threaded C++17, what the reference's LLVM-CPU lowering of a
// `tensor.*` program computes. It is the checker the CUDA kernels are compared against and the timed
// CPU baseline; nothing in the product path may call it.
//
// Parity status: the generic `map_reduce_post` interpreter and the derived f32 ops are PINNED by the
// reference's own known-answer tests (lit/buffer/exec_*.mim exit codes, lit/btensor/map_reduce_post.mim,
// lit/tensor/{attn,fc,hlo}_aux.cpp, lit/tensor/reduce_exec.mim) -- see tests/test_oracle_golden.py.
// The extensions the reference has no test for (bf16 round-to-nearest-even storage, causal masking,
// softmax scale, RMSNorm, SiLU gating) are "parity unpinned": this file defines them.
//
// What it follows in the reference (paths inside the MimIR project):
//   * semantics of the one real op:      src/mim/plug/tensor/tensor.mim:114-169
//   * executable spec of the loop nest:  src/mim/plug/tensor/phase/lower_map_reduce.cpp:93-206
//   * canonical (classic) nest order:    src/mim/plug/btensor/btensor.mim:349-377, 529-559
//   * affine index arithmetic (i64 wrap): include/mim/plug/affine/phase/lower_index.h:11-27
//   * row-major buffers:                  src/mim/plug/buffer/phase/lower_ptr.cpp:13-85
//   * dot family:                         src/mim/plug/tensor/tensor.mim:1332, 1367-1423
//   * reduce / binary_ax / softmax:       src/mim/plug/tensor/tensor.mim:1139-1176
//   * attention composition:              lit/tensor/attn_exec.mim:20-22
//
// Two arithmetic modes exist for the floating-point ops:
//   "as lowered": f32 accumulators, ascending reduction index per output cell (the order every CPU nest
//                 keeps, btensor.mim:348), one rounding per add and per mul;
//   "truth":      f64 accumulation of the exact (f32 or bf16) inputs -- what the reference's own
//                 *_aux.cpp drivers compare against.
#include <cmath>
#include <cstdint>
#include <cstdlib>
#include <cstring>
#include <limits>
#include <vector>

#define MO_API extern "C"

// ----------------------------------------------------------------------------------------------
// dtypes and scalar helpers
// ----------------------------------------------------------------------------------------------
enum { MO_I32 = 0, MO_I64 = 1, MO_F32 = 2, MO_F64 = 3, MO_BF16 = 4 };

static inline float bf16_to_f32(uint16_t h) {
    uint32_t u = uint32_t(h) << 16;
    float f;
    std::memcpy(&f, &u, 4);
    return f;
}
// round-to-nearest-even, NaN kept quiet (what __float2bfloat16_rn does)
static inline uint16_t f32_to_bf16(float f) {
    uint32_t u;
    std::memcpy(&u, &f, 4);
    if ((u & 0x7fffffffu) > 0x7f800000u) return uint16_t((u >> 16) | 0x40);
    u += 0x7fffu + ((u >> 16) & 1u);
    return uint16_t(u >> 16);
}

MO_API void mo_f32_to_bf16(const float* x, uint16_t* y, int64_t n) {
    for (int64_t i = 0; i < n; ++i) y[i] = f32_to_bf16(x[i]);
}
MO_API void mo_bf16_to_f32(const uint16_t* x, float* y, int64_t n) {
    for (int64_t i = 0; i < n; ++i) y[i] = bf16_to_f32(x[i]);
}

union Val {
    int32_t i32;
    int64_t i64;
    float f32;
    double f64;
};

static inline Val load_val(const void* p, int dt, int64_t off) {
    Val v;
    v.i64 = 0;
    switch (dt) {
        case MO_I32: v.i32 = static_cast<const int32_t*>(p)[off]; break;
        case MO_I64: v.i64 = static_cast<const int64_t*>(p)[off]; break;
        case MO_F32: v.f32 = static_cast<const float*>(p)[off]; break;
        case MO_F64: v.f64 = static_cast<const double*>(p)[off]; break;
        case MO_BF16: v.f32 = bf16_to_f32(static_cast<const uint16_t*>(p)[off]); break;
    }
    return v;
}
static inline void store_val(void* p, int dt, int64_t off, Val v) {
    switch (dt) {
        case MO_I32: static_cast<int32_t*>(p)[off] = v.i32; break;
        case MO_I64: static_cast<int64_t*>(p)[off] = v.i64; break;
        case MO_F32: static_cast<float*>(p)[off] = v.f32; break;
        case MO_F64: static_cast<double*>(p)[off] = v.f64; break;
        case MO_BF16: static_cast<uint16_t*>(p)[off] = f32_to_bf16(v.f32); break;
    }
}

// ----------------------------------------------------------------------------------------------
// generic map_reduce_post interpreter
// ----------------------------------------------------------------------------------------------
// Combiners `f(acc, ins)` and epilogues `post(acc, post_ins)` the fixtures need. A bf16 input is widened
// to f32 on load, so the f32 combiners serve it too. The *_F64 combiners are the "truth" mode.
enum {
    MO_F_ADD_I32 = 0,      // acc + a                       (exec_map_reduce.mim:22)
    MO_F_MULADD_I32 = 1,   // acc + a*b                     (exec_tile.mim:21, ring (I32,0,+,*))
    MO_F_MIX_I32_I64 = 2,  // acc + a + (i32)b              (lit/btensor/map_reduce_post.mim:17-18)
    MO_F_ADD_F32 = 3,      // pool_fun add
    MO_F_MULADD_F32 = 4,   // dot_general_fun ring (F32,0,add,mul)      (tensor.mim:1332)
    MO_F_FMAX_F32 = 5,     // pool_fun fmax
    MO_F_SUBEXP_F32 = 6,   // binary_ax app = exp(u - v), acc ignored   (tensor.mim:1175)
    MO_F_DIV_F32 = 7,      // binary_ax app = u / v                     (tensor.mim:1176)
    MO_F_ADD2_F32 = 8,     // binary app = u + v
    MO_F_FIRST_F32 = 9,    // copy-style ops: acc ignored, returns the element (transpose, broadcast, reshape)
    MO_F_MULADD_F64 = 10,
    MO_F_ADD_F64 = 11,
    MO_F_FMIN_F32 = 12,
    MO_F_MUL2_F32 = 13,    // binary app = u * v
    MO_F_FIRST_I32 = 14,
    MO_F_ADD_SUBEXP_F32 = 15,  // acc + exp(u - v): the sum fold of softmax with its producer inlined (fuse.cpp:225-245)
    MO_F_SUBEXP_DIV_F32 = 16,  // exp(u - v) / w: the divide with the exponential recomputed
    // The general form of a combiner after fuse_map_reduce inlined an injective elementwise producer into the operand read
    // (src/mim/plug/tensor/phase/fuse.cpp:183-358): id = MO_F_COMPOSED | fold | inner << 8 | outer << 16 computes
    // fold(acc, outer(inner(u, v))) in f32, one rounding per operation. fold: 0 add, 2 fmax, 3 fmin, 4 first; inner / outer:
    // 0 add, 1 sub, 2 mul, 3 div, 4 fmax, 5 fmin, 6 exp(u - v); 16 relu, 17 tanh, 18 exp, 19 x / (1 + exp(-x)), 20 neg,
    // 21 identity, 22 square, 23 abs, 24 sqrt, 25 1 / sqrt, 26 log, 27 exp2, 28 log2, 29 1 / (1 + exp(-x))
    // (math.mim:147, 297-298, 167-169, 283-284).
    MO_F_COMPOSED = 0x01000000,
};
enum {
    MO_P_ID = 0,
    MO_P_CONV_ADD_I64 = 1,    // (i64)(u32)acc + b            (lit/btensor/map_reduce_post.mim:19-20)
    MO_P_ADD_PLUS1_I32 = 2,   // acc + b + 1                  (exec_epilogue.mim:33)
    MO_P_BIAS_RELU_F32 = 3,   // fmax(0, acc + b)             (fc_exec.mim:27-31)
    MO_P_BIAS_TANH_F32 = 4,   // tanh(acc + b)                (hlo_exec.mim)
    MO_P_BIAS_F32 = 5,        // acc + b
    MO_P_F64_TO_F32 = 6,      // truth mode: narrow once at the end
};

static inline float elementwise(int op, float a, float b) {
    switch (op) {
        case 0: return a + b;
        case 1: return a - b;
        case 2: return a * b;
        case 3: return a / b;
        case 4: return std::fmax(a, b);
        case 5: return std::fmin(a, b);
        case 6: return std::exp(a - b);
        case 16: return std::fmax(0.0f, a);
        case 17: return std::tanh(a);
        case 18: return std::exp(a);
        case 19: return a / (1.0f + std::exp(-a));
        case 20: return -a;
        case 22: return a * a;
        case 23: return std::fabs(a);
        case 24: return std::sqrt(a);
        case 25: return 1.0f / std::sqrt(a);
        case 26: return std::log(a);
        case 27: return std::exp2(a);
        case 28: return std::log2(a);
        case 29: return 1.0f / (1.0f + std::exp(-a));
        default: return a;
    }
}
static inline Val comb(int id, Val acc, const Val* in) {
    Val r = acc;
    if (id & MO_F_COMPOSED) {
        volatile float inner = elementwise((id >> 8) & 0xff, in[0].f32, in[1].f32);  // one rounding per op: no contraction
        volatile float v     = elementwise((id >> 16) & 0xff, inner, 0.0f);
        switch (id & 0xff) {
            case 0: r.f32 = acc.f32 + v; break;
            case 2: r.f32 = std::fmax(acc.f32, v); break;
            case 3: r.f32 = std::fmin(acc.f32, v); break;
            default: r.f32 = v; break;
        }
        return r;
    }
    switch (id) {
        case MO_F_ADD_I32: r.i32 = int32_t(uint32_t(acc.i32) + uint32_t(in[0].i32)); break;
        case MO_F_MULADD_I32: r.i32 = int32_t(uint32_t(acc.i32) + uint32_t(in[0].i32) * uint32_t(in[1].i32)); break;
        case MO_F_MIX_I32_I64:
            r.i32 = int32_t(uint32_t(acc.i32) + uint32_t(in[0].i32) + uint32_t(uint64_t(in[1].i64)));
            break;
        case MO_F_ADD_F32: r.f32 = acc.f32 + in[0].f32; break;
        case MO_F_MULADD_F32: {
            volatile float p = in[0].f32 * in[1].f32;  // one rounding per op: no contraction
            r.f32            = acc.f32 + p;
            break;
        }
        case MO_F_FMAX_F32: r.f32 = std::fmax(acc.f32, in[0].f32); break;
        case MO_F_FMIN_F32: r.f32 = std::fmin(acc.f32, in[0].f32); break;
        case MO_F_SUBEXP_F32: r.f32 = std::exp(in[0].f32 - in[1].f32); break;
        case MO_F_DIV_F32: r.f32 = in[0].f32 / in[1].f32; break;
        case MO_F_ADD2_F32: r.f32 = in[0].f32 + in[1].f32; break;
        case MO_F_MUL2_F32: r.f32 = in[0].f32 * in[1].f32; break;
        case MO_F_FIRST_F32: r.f32 = in[0].f32; break;
        case MO_F_FIRST_I32: r.i32 = in[0].i32; break;
        case MO_F_MULADD_F64: r.f64 = acc.f64 + in[0].f64 * in[1].f64; break;
        case MO_F_ADD_F64: r.f64 = acc.f64 + in[0].f64; break;
        case MO_F_ADD_SUBEXP_F32: r.f32 = acc.f32 + std::exp(in[0].f32 - in[1].f32); break;
        case MO_F_SUBEXP_DIV_F32: r.f32 = std::exp(in[0].f32 - in[1].f32) / in[2].f32; break;
    }
    return r;
}
static inline Val post(int id, Val acc, const Val* p) {
    Val r = acc;
    switch (id) {
        case MO_P_ID: break;
        case MO_P_CONV_ADD_I64: r.i64 = int64_t(uint64_t(uint32_t(acc.i32)) + uint64_t(p[0].i64)); break;
        case MO_P_ADD_PLUS1_I32: r.i32 = int32_t(uint32_t(acc.i32) + uint32_t(p[0].i32) + 1u); break;
        case MO_P_BIAS_RELU_F32: r.f32 = std::fmax(0.0f, acc.f32 + p[0].f32); break;
        case MO_P_BIAS_TANH_F32: r.f32 = std::tanh(acc.f32 + p[0].f32); break;
        case MO_P_BIAS_F32: r.f32 = acc.f32 + p[0].f32; break;
        case MO_P_F64_TO_F32: r.f32 = float(acc.f64); break;
    }
    return r;
}

// An affine access map with `rows` results over `n` loop variables, as a dense matrix: result j =
// sum_l coef[j*(n+1)+l]*loop[l] + coef[j*(n+1)+n], in wrap-around i64 (lower_index.h:14-20). This covers
// affine.lit / op.add / op.sub / op.neg / semiop.mul, i.e. every map the dot family, reduce, binary_ax and
// the strip-mined schedules build; floordiv/rem maps (reshape) are handled by passing `div`/`mod` columns:
// when divs != nullptr, result j is first computed linearly, then floordiv'ed by divs[j] (if > 0) and
// reduced modulo mods[j] (if > 0) -- the shape `delinearize` produces (affine.mim:103-108).
struct Map {
    int rows;
    const int64_t* coef;
    const int64_t* divs;
    const int64_t* mods;
};

static inline int64_t linear_offset(const Map& m, int n, const int64_t* loop, const int64_t* shape) {
    uint64_t off = 0;
    for (int j = 0; j < m.rows; ++j) {
        const int64_t* c = m.coef + int64_t(j) * (n + 1);
        uint64_t v       = uint64_t(c[n]);
        for (int l = 0; l < n; ++l) v += uint64_t(c[l]) * uint64_t(loop[l]);
        if (m.divs && m.divs[j] > 0) v = v / uint64_t(m.divs[j]);
        if (m.mods && m.mods[j] > 0) v = v % uint64_t(m.mods[j]);
        off = off * uint64_t(shape[j]) + v;  // row-major lea chain (mem.h:36-42)
    }
    return int64_t(off);
}

// out[map_out(o)] = post(fold_r f(acc, (in_i[maps_i(o,r)])_i), (post_in_j[post_maps_j(map_out(o))])_j)
// Shapes and maps are passed flattened, one after another. Returns 0, or a negative code for bad arguments
// (any access outside a buffer is reported, never performed).
MO_API int mo_map_reduce_post(int Ro, int Rn, const int64_t* Sr, const int64_t* So,                        //
                       int nis, const void* const* ins, const int* in_dt, const int* in_rank,       //
                       const int64_t* in_shapes, const int64_t* in_maps,                            //
                       int nps, const void* const* pins, const int* p_dt, const int* p_rank,        //
                       const int64_t* p_shapes, const int64_t* p_maps,                              //
                       const int64_t* map_out, int comb_id, int64_t init_bits, int post_id, int out_dt, void* out,
                       // optional floordiv / rem per map result, (div, mod) pairs in the order of the maps' results; NULL = none
                       const int64_t* in_divmod, const int64_t* p_divmod, const int64_t* out_divmod) {
    if (Ro < 0 || Rn < Ro || Rn > 16 || nis > 8 || nps > 8) return -1;
    std::vector<Map> maps(nis), pmaps(nps);
    std::vector<int64_t> divs, mods, pdivs, pmods;
    std::vector<const int64_t*> ishape(nis), pshape(nps);
    std::vector<int64_t> isize(nis), psize(nps);
    {
        // (div, mod) pairs are unzipped into one array of divs and one of mods per map
        const int64_t *s = in_shapes, *m = in_maps, *dm = in_divmod;
        for (int i = 0; i < nis; ++i) {
            ishape[i] = s;
            maps[i]   = Map{in_rank[i], m, nullptr, nullptr};
            if (dm) {
                for (int j = 0; j < in_rank[i]; ++j) divs.push_back(dm[2 * j]), mods.push_back(dm[2 * j + 1]);
                dm += 2 * in_rank[i];
            }
            isize[i]  = 1;
            for (int j = 0; j < in_rank[i]; ++j) isize[i] *= s[j];
            s += in_rank[i];
            m += int64_t(in_rank[i]) * (Rn + 1);
        }
        s = p_shapes, m = p_maps, dm = p_divmod;
        for (int j = 0; j < nps; ++j) {
            pshape[j] = s;
            pmaps[j]  = Map{p_rank[j], m, nullptr, nullptr};
            if (dm) {
                for (int k = 0; k < p_rank[j]; ++k) pdivs.push_back(dm[2 * k]), pmods.push_back(dm[2 * k + 1]);
                dm += 2 * p_rank[j];
            }
            psize[j]  = 1;
            for (int k = 0; k < p_rank[j]; ++k) psize[j] *= s[k];
            s += p_rank[j];
            m += int64_t(p_rank[j]) * (Ro + 1);
        }
    }
    // the vectors are complete now: hand each map its slice
    {
        size_t at = 0;
        for (int i = 0; i < nis && in_divmod; ++i) maps[i].divs = divs.data() + at, maps[i].mods = mods.data() + at, at += size_t(in_rank[i]);
        at = 0;
        for (int j = 0; j < nps && p_divmod; ++j) pmaps[j].divs = pdivs.data() + at, pmaps[j].mods = pmods.data() + at, at += size_t(p_rank[j]);
    }
    std::vector<int64_t> odivs, omods;
    for (int j = 0; j < Ro && out_divmod; ++j) odivs.push_back(out_divmod[2 * j]), omods.push_back(out_divmod[2 * j + 1]);
    Map mout{Ro, map_out, nullptr, nullptr};
    int64_t osize = 1;
    for (int j = 0; j < Ro; ++j) osize *= So[j];

    int64_t n_out = 1, n_red = 1;
    for (int l = 0; l < Ro; ++l) n_out *= Sr[l];
    for (int l = Ro; l < Rn; ++l) n_red *= Sr[l];
    if (n_out == 0) return 0;

    Val init;
    init.i64 = init_bits;
    const bool f64_mode = comb_id == MO_F_MULADD_F64 || comb_id == MO_F_ADD_F64;  // truth: widen on load
    int64_t loop[16] = {0};
    Val in[8], pin[8];
    for (int64_t o = 0; o < n_out; ++o) {
        // delinearise o into the leading Ro loop variables (classic nest: last output loop fastest)
        int64_t rem = o;
        for (int l = Ro - 1; l >= 0; --l) {
            loop[l] = rem % Sr[l];
            rem /= Sr[l];
        }
        Val acc = init;
        for (int64_t r = 0; r < n_red; ++r) {
            int64_t rr = r;
            for (int l = Rn - 1; l >= Ro; --l) {
                loop[l] = rr % Sr[l];
                rr /= Sr[l];
            }
            for (int i = 0; i < nis; ++i) {
                int64_t off = linear_offset(maps[i], Rn, loop, ishape[i]);
                if (off < 0 || off >= isize[i]) return -2;
                in[i] = load_val(ins[i], in_dt[i], off);
                if (f64_mode && (in_dt[i] == MO_F32 || in_dt[i] == MO_BF16)) in[i].f64 = double(in[i].f32);
            }
            acc = comb(comb_id, acc, in);
        }
        // write-back: reduction slots are 0 (lower_map_reduce.cpp:158-160)
        for (int l = Ro; l < Rn; ++l) loop[l] = 0;
        int64_t wc[16];
        {
            for (int j = 0; j < Ro; ++j) {
                const int64_t* c = map_out + int64_t(j) * (Rn + 1);
                uint64_t v       = uint64_t(c[Rn]);
                for (int l = 0; l < Rn; ++l) v += uint64_t(c[l]) * uint64_t(loop[l]);
                if (!odivs.empty() && odivs[j] > 0) v /= uint64_t(odivs[j]);
                if (!omods.empty() && omods[j] > 0) v %= uint64_t(omods[j]);
                wc[j] = int64_t(v);
            }
        }
        for (int j = 0; j < nps; ++j) {
            int64_t off = linear_offset(pmaps[j], Ro, wc, pshape[j]);
            if (off < 0 || off >= psize[j]) return -3;
            pin[j] = load_val(pins[j], p_dt[j], off);
        }
        Val res      = post(post_id, acc, pin);
        (void)mout;
        int64_t woff = 0;  // row-major offset of the write coordinates (mem.h:36-42)
        for (int j = 0; j < Ro; ++j) woff = int64_t(uint64_t(woff) * uint64_t(So[j]) + uint64_t(wc[j]));
        if (woff < 0 || woff >= osize) return -4;
        store_val(out, out_dt, woff, res);
    }
    return 0;
}

// ----------------------------------------------------------------------------------------------
// direct loops for sizes the interpreter is too slow for (same fold order; checked against it in tests)
// ----------------------------------------------------------------------------------------------
template <class T>
static inline float ldf(const T* p, int64_t i);
template <>
inline float ldf<float>(const float* p, int64_t i) {
    return p[i];
}
template <>
inline float ldf<uint16_t>(const uint16_t* p, int64_t i) {
    return bf16_to_f32(p[i]);
}

// product_2d (tensor.mim:1422-1423): C[m,n] = sum_k A[m,k] * B(k,n); b_nk != 0 reads B through
// transpose_2d of a row-major [N,K] tensor (fuse_read_through, fuse.cpp:542-589).
// "As lowered": f32 accumulator, ascending k.
template <class T>
static void gemm_as_lowered(const T* A, const T* B, float* C, int64_t M, int64_t N, int64_t K, int b_nk) {
    if (b_nk) {
        for (int64_t m = 0; m < M; ++m)
            for (int64_t n = 0; n < N; ++n) {
                float acc = 0.f;
                for (int64_t k = 0; k < K; ++k) acc += ldf(A, m * K + k) * ldf(B, n * K + k);
                C[m * N + n] = acc;
            }
    } else {
        // same per-cell order (ascending k), loop order chosen so the inner loop is unit stride
        std::vector<float> row(N);
        for (int64_t m = 0; m < M; ++m) {
            for (int64_t n = 0; n < N; ++n) row[n] = 0.f;
            for (int64_t k = 0; k < K; ++k) {
                float a = ldf(A, m * K + k);
                for (int64_t n = 0; n < N; ++n) row[n] += a * ldf(B, k * N + n);
            }
            for (int64_t n = 0; n < N; ++n) C[m * N + n] = row[n];
        }
    }
}
MO_API void mo_gemm_f32(const float* A, const float* B, float* C, int64_t M, int64_t N, int64_t K, int b_nk) {
    gemm_as_lowered(A, B, C, M, N, K, b_nk);
}
MO_API void mo_gemm_bf16(const uint16_t* A, const uint16_t* B, float* C, int64_t M, int64_t N, int64_t K, int b_nk) {
    gemm_as_lowered(A, B, C, M, N, K, b_nk);
}

// Truth: f64 accumulation of the exact inputs, for the listed output rows only (nrows == 0: all rows).
// C is [nrows or M, N] doubles.
template <class T>
static void gemm_truth(const T* A, const T* B, double* C, int64_t M, int64_t N, int64_t K, int b_nk,
                       const int64_t* rows, int64_t nrows) {
    int64_t R = nrows ? nrows : M;
    std::vector<double> acc(N);
    for (int64_t r = 0; r < R; ++r) {
        int64_t m = nrows ? rows[r] : r;
        if (b_nk) {
            for (int64_t n = 0; n < N; ++n) {
                double a0 = 0, a1 = 0, a2 = 0, a3 = 0;  // f64: order immaterial at the tolerances used
                int64_t k = 0;
                for (; k + 4 <= K; k += 4) {
                    a0 += double(ldf(A, m * K + k)) * double(ldf(B, n * K + k));
                    a1 += double(ldf(A, m * K + k + 1)) * double(ldf(B, n * K + k + 1));
                    a2 += double(ldf(A, m * K + k + 2)) * double(ldf(B, n * K + k + 2));
                    a3 += double(ldf(A, m * K + k + 3)) * double(ldf(B, n * K + k + 3));
                }
                for (; k < K; ++k) a0 += double(ldf(A, m * K + k)) * double(ldf(B, n * K + k));
                C[r * N + n] = (a0 + a1) + (a2 + a3);
            }
        } else {
            for (int64_t n = 0; n < N; ++n) acc[n] = 0;
            for (int64_t k = 0; k < K; ++k) {
                double a = ldf(A, m * K + k);
                for (int64_t n = 0; n < N; ++n) acc[n] += a * double(ldf(B, k * N + n));
            }
            for (int64_t n = 0; n < N; ++n) C[r * N + n] = acc[n];
        }
    }
}
MO_API void mo_gemm_truth_f32(const float* A, const float* B, double* C, int64_t M, int64_t N, int64_t K, int b_nk,
                       const int64_t* rows, int64_t nrows) {
    gemm_truth(A, B, C, M, N, K, b_nk, rows, nrows);
}
MO_API void mo_gemm_truth_bf16(const uint16_t* A, const uint16_t* B, double* C, int64_t M, int64_t N, int64_t K, int b_nk,
                        const int64_t* rows, int64_t nrows) {
    gemm_truth(A, B, C, M, N, K, b_nk, rows, nrows);
}

// reduce (tensor.mim:1151-1157) over the middle axis of a [outer, len, inner] view, monoid 0=sum 1=max 2=min.
// As lowered: ascending index along the axis, f32.
MO_API void mo_reduce_f32(const float* x, float* out, int64_t outer, int64_t len, int64_t inner, int monoid) {
    for (int64_t o = 0; o < outer; ++o)
        for (int64_t i = 0; i < inner; ++i) {
            float acc = monoid == 0 ? 0.f : (monoid == 1 ? -INFINITY : INFINITY);
            for (int64_t a = 0; a < len; ++a) {
                float v = x[(o * len + a) * inner + i];
                acc     = monoid == 0 ? acc + v : (monoid == 1 ? std::fmax(acc, v) : std::fmin(acc, v));
            }
            out[o * inner + i] = acc;
        }
}
MO_API void mo_reduce_truth(const float* x, double* out, int64_t outer, int64_t len, int64_t inner, int monoid) {
    for (int64_t o = 0; o < outer; ++o)
        for (int64_t i = 0; i < inner; ++i) {
            double acc = monoid == 0 ? 0. : (monoid == 1 ? -INFINITY : INFINITY);
            for (int64_t a = 0; a < len; ++a) {
                double v = x[(o * len + a) * inner + i];
                acc      = monoid == 0 ? acc + v : (monoid == 1 ? std::fmax(acc, v) : std::fmin(acc, v));
            }
            out[o * inner + i] = acc;
        }
}

// softmax along the last axis (tensor.mim:1172-1176), exactly the four ops the lam expands to:
// mx = reduce fmax -inf; e = exp(x - mx); s = reduce add 0 e; e / s. f32, three passes over the row.
MO_API void mo_softmax_rows_f32(const float* x, float* y, int64_t rows, int64_t cols) {
    std::vector<float> e(cols);
    for (int64_t r = 0; r < rows; ++r) {
        const float* xr = x + r * cols;
        float mx        = -INFINITY;
        for (int64_t c = 0; c < cols; ++c) mx = std::fmax(mx, xr[c]);
        for (int64_t c = 0; c < cols; ++c) e[c] = std::exp(xr[c] - mx);
        float s = 0.f;
        for (int64_t c = 0; c < cols; ++c) s += e[c];
        for (int64_t c = 0; c < cols; ++c) y[r * cols + c] = e[c] / s;
    }
}
MO_API void mo_softmax_rows_truth(const float* x, double* y, int64_t rows, int64_t cols) {
    for (int64_t r = 0; r < rows; ++r) {
        const float* xr = x + r * cols;
        double mx       = -INFINITY;
        for (int64_t c = 0; c < cols; ++c) mx = std::fmax(mx, double(xr[c]));
        double s = 0.;
        for (int64_t c = 0; c < cols; ++c) s += (y[r * cols + c] = std::exp(double(xr[c]) - mx));
        for (int64_t c = 0; c < cols; ++c) y[r * cols + c] /= s;
    }
}

// RMSNorm rows (not a reference op; composed from reduce + binary_ax + math.rrt, math.mim:297-298):
// y = x * rrt(mean(x^2) + eps) * gamma.    parity unpinned.
MO_API void mo_rmsnorm_rows_f32(const float* x, const float* gamma, float* y, int64_t rows, int64_t cols, float eps) {
    for (int64_t r = 0; r < rows; ++r) {
        const float* xr = x + r * cols;
        float ss        = 0.f;
        for (int64_t c = 0; c < cols; ++c) ss += xr[c] * xr[c];
        float inv = 1.0f / std::sqrt(ss / float(cols) + eps);
        for (int64_t c = 0; c < cols; ++c) y[r * cols + c] = xr[c] * inv * gamma[c];
    }
}
MO_API void mo_rmsnorm_rows_truth(const float* x, const float* gamma, double* y, int64_t rows, int64_t cols, double eps) {
    for (int64_t r = 0; r < rows; ++r) {
        const float* xr = x + r * cols;
        double ss       = 0.;
        for (int64_t c = 0; c < cols; ++c) ss += double(xr[c]) * double(xr[c]);
        double inv = 1.0 / std::sqrt(ss / double(cols) + eps);
        for (int64_t c = 0; c < cols; ++c) y[r * cols + c] = double(xr[c]) * inv * double(gamma[c]);
    }
}

// Attention forward per (batch*head): O = softmax(scale * Q K^T [+ causal mask]) V.
// With scale = 1, causal = 0, one head this is the reference's test program (attn_exec.mim:20-22), and the
// reference driver's check (attn_aux.cpp:36-56) is exactly this f64 routine. Scale, mask and bf16 inputs
// are extensions (parity unpinned): mask = -inf before the max; key j visible to query i iff j <= i.
// Q,K,V: [BH, S, D] contiguous; `heads` lists which BH indices to compute (nheads == 0: all); O is
// [nheads or BH, S, D] doubles.
template <class T>
static void attn_truth(const T* Q, const T* K, const T* V, double* O, int64_t BH, int64_t S, int64_t D, double scale,
                       int causal, const int64_t* heads, int64_t nheads) {
    int64_t H = nheads ? nheads : BH;
    std::vector<double> p(S), q(D), kd(size_t(S) * D), vd(size_t(S) * D);
    for (int64_t hh = 0; hh < H; ++hh) {
        int64_t h   = nheads ? heads[hh] : hh;
        const T* Qh = Q + h * S * D;
        const T* Kh = K + h * S * D;
        const T* Vh = V + h * S * D;
        for (int64_t i = 0; i < S * D; ++i) {
            kd[i] = ldf(Kh, i);
            vd[i] = ldf(Vh, i);
        }
        for (int64_t i = 0; i < S; ++i) {
            for (int64_t d = 0; d < D; ++d) q[d] = ldf(Qh, i * D + d);
            int64_t lim = causal ? i + 1 : S;
            double mx   = -INFINITY;
            for (int64_t j = 0; j < lim; ++j) {
                double s         = 0;
                const double* kj = &kd[j * D];
                for (int64_t d = 0; d < D; ++d) s += q[d] * kj[d];
                p[j] = s * scale;
                mx   = std::fmax(mx, p[j]);
            }
            double sum = 0;
            for (int64_t j = 0; j < lim; ++j) sum += (p[j] = std::exp(p[j] - mx));
            double* o = O + (hh * S + i) * D;
            for (int64_t d = 0; d < D; ++d) o[d] = 0;
            for (int64_t j = 0; j < lim; ++j) {
                double w         = p[j] / sum;
                const double* vj = &vd[j * D];
                for (int64_t d = 0; d < D; ++d) o[d] += w * vj[d];
            }
        }
    }
}
MO_API void mo_attn_truth_f32(const float* Q, const float* K, const float* V, double* O, int64_t BH, int64_t S, int64_t D,
                       double scale, int causal, const int64_t* heads, int64_t nheads) {
    attn_truth(Q, K, V, O, BH, S, D, scale, causal, heads, nheads);
}
MO_API void mo_attn_truth_bf16(const uint16_t* Q, const uint16_t* K, const uint16_t* V, double* O, int64_t BH, int64_t S,
                        int64_t D, double scale, int causal, const int64_t* heads, int64_t nheads) {
    attn_truth(Q, K, V, O, BH, S, D, scale, causal, heads, nheads);
}

// As lowered (f32): the unfused chain the reference materialises -- scores [S,S], softmax rows, P V.
template <class T>
static void attn_as_lowered(const T* Q, const T* K, const T* V, float* O, int64_t BH, int64_t S, int64_t D,
                            float scale, int causal) {
    std::vector<float> sc(size_t(S) * S), pr(size_t(S) * S);
    for (int64_t h = 0; h < BH; ++h) {
        const T* Qh = Q + h * S * D;
        const T* Kh = K + h * S * D;
        const T* Vh = V + h * S * D;
        for (int64_t i = 0; i < S; ++i)
            for (int64_t j = 0; j < S; ++j) {
                float acc = 0.f;
                for (int64_t d = 0; d < D; ++d) acc += ldf(Qh, i * D + d) * ldf(Kh, j * D + d);
                sc[i * S + j] = (causal && j > i) ? -INFINITY : acc * scale;
            }
        mo_softmax_rows_f32(sc.data(), pr.data(), S, S);
        for (int64_t i = 0; i < S; ++i) {
            float* o = O + (h * S + i) * D;
            for (int64_t d = 0; d < D; ++d) o[d] = 0.f;
            for (int64_t j = 0; j < S; ++j) {
                float w = pr[i * S + j];
                for (int64_t d = 0; d < D; ++d) o[d] += w * ldf(Vh, j * D + d);
            }
        }
    }
}
MO_API void mo_attn_f32(const float* Q, const float* K, const float* V, float* O, int64_t BH, int64_t S, int64_t D,
                 float scale, int causal) {
    attn_as_lowered(Q, K, V, O, BH, S, D, scale, causal);
}
MO_API void mo_attn_bf16(const uint16_t* Q, const uint16_t* K, const uint16_t* V, float* O, int64_t BH, int64_t S, int64_t D,
                  float scale, int causal) {
    attn_as_lowered(Q, K, V, O, BH, S, D, scale, causal);
}

// Gated MLP rows (composition of product_2d, math.slf (math.mim:283-284), binary mul, product_2d):
// H = bf16(silu(X W1) * (X W3)); Y = H W2. W1,W3: [K,F] row-major, W2: [F,N] row-major. Truth for the listed
// rows: f64 accumulation, H rounded to bf16 (the stored intermediate), Y in f64.       parity unpinned.
MO_API void mo_mlp_truth_bf16(const uint16_t* X, const uint16_t* W1, const uint16_t* W3, const uint16_t* W2, double* Y,
                       int64_t M, int64_t K, int64_t F, int64_t N, const int64_t* rows, int64_t nrows) {
    int64_t R = nrows ? nrows : M;
    std::vector<double> g(F), u(F), y(N);
    std::vector<float> h(F);
    for (int64_t r = 0; r < R; ++r) {
        int64_t m = nrows ? rows[r] : r;
        for (int64_t f = 0; f < F; ++f) g[f] = u[f] = 0;
        for (int64_t k = 0; k < K; ++k) {
            double x = bf16_to_f32(X[m * K + k]);
            for (int64_t f = 0; f < F; ++f) {
                g[f] += x * double(bf16_to_f32(W1[k * F + f]));
                u[f] += x * double(bf16_to_f32(W3[k * F + f]));
            }
        }
        for (int64_t f = 0; f < F; ++f) {
            double s = g[f] / (1.0 + std::exp(-g[f]));
            h[f]     = bf16_to_f32(f32_to_bf16(float(s * u[f])));
        }
        for (int64_t n = 0; n < N; ++n) y[n] = 0;
        for (int64_t f = 0; f < F; ++f) {
            double hv = h[f];
            for (int64_t n = 0; n < N; ++n) y[n] += hv * double(bf16_to_f32(W2[f * N + n]));
        }
        for (int64_t n = 0; n < N; ++n) Y[r * N + n] = y[n];
    }
}

