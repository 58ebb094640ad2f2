// Recognisers for `map_reduce_post`: which descriptors are really a contraction, an axis reduction or an elementwise
// map over dense row-major operands, and can therefore run on the specialised kernels instead of the one-thread-per-
// cell kernel.
//
// The reference has the same split on the compiler side: the derived ops of the tensor plugin (dot family
// src/mim/plug/tensor/tensor.mim:1367-1423, reduce 1151-1157, binary_ax 1162-1167, unary/binary 361-394) all expand to
// one `map_reduce_post`, and a lowering that wants a fast kernel has to recognise them again from the access maps
// (the shapes are listed with dot_product_impl's subscript construction, tensor.mim:1381-1396). Here the recognition
// runs on the descriptor at call time, so code emitted for the generic operation gets the tensor-core contraction and
// the bandwidth-bound row kernels without knowing about them.
//
// Only floating-point instances above a size threshold are re-routed: the specialised kernels fold in a different
// order than the ascending per-cell fold of the classic nest (btensor.mim:349-377), which integer instances and small
// float instances keep bit for bit. Re-association of a float fold is what the reference's `fast` math mode grants its
// own CPU back end (src/mim/plug/ll/ll.cpp:949-1108).
#include <cstdlib>

#include "common.cuh"

namespace mimk {
namespace {

// Is result `j` of `m` exactly loop variable `l` (over `n` loop variables)?
bool row_is_loop(const mimk_affine_map& m, int j, int n, int l) {
    for (int c = 0; c < n; ++c)
        if (m.coef[j][c] != (c == l ? 1 : 0)) return false;
    return m.coef[j][n] == 0 && m.div[j] <= 0 && m.mod[j] <= 0;
}

// The write map stores output loop vector o at o, and the result has exactly the loop bounds as its shape.
bool out_is_identity(const mimk_mrp_desc& d) {
    if (d.map_out.rows != d.ro) return false;
    for (int j = 0; j < d.ro; ++j)
        if (!row_is_loop(d.map_out, j, d.rn, j) || d.so[j] != d.sr[j]) return false;
    return true;
}

uint32_t init32(const mimk_mrp_desc& d) { return (uint32_t)((uint64_t)d.init_bits & 0xffffffffu); }

int64_t prod(const int64_t* v, int lo, int hi) {
    int64_t p = 1;
    for (int i = lo; i < hi; ++i) p *= v[i];
    return p;
}

using Plan = MrpPlan;

// Operand `i` as a matrix [..batch, r, c]: its last two results are loops (lr, lc); with a leading batch result (loop 0)
// when the operand has one. Returns 0 = no match, 1 = matrix without batch axis, 2 = matrix with batch axis.
int matrix_operand(const mimk_mrp_desc& d, int i, int lr, int lc, bool batched) {
    const mimk_affine_map& m = d.in_map[i];
    const int r              = m.rows;
    if (r == 2 || (r == 3 && batched)) {
        const int o = r - 2;
        if (!row_is_loop(m, o, d.rn, lr) || !row_is_loop(m, o + 1, d.rn, lc)) return 0;
        if (d.in_shape[i][o] != d.sr[lr] || d.in_shape[i][o + 1] != d.sr[lc]) return 0;
        if (r == 3 && (!row_is_loop(m, 0, d.rn, 0) || d.in_shape[i][0] != d.sr[0])) return 0;
        return r == 3 ? 2 : 1;
    }
    return 0;
}

bool plan_gemm(const mimk_mrp_desc& d, Plan& p) {
    if (d.comb != MIMK_F_MULADD || d.nis != 2 || d.acc_dtype != MIMK_F32 || init32(d) != 0u) return false;
    if ((d.ro != 2 && d.ro != 3) || d.rn != d.ro + 1 || !out_is_identity(d)) return false;
    if (d.in_dtype[0] != d.in_dtype[1] || (d.in_dtype[0] != MIMK_F32 && d.in_dtype[0] != MIMK_BF16)) return false;
    const bool batched = d.ro == 3;
    const int lm = d.ro - 2, ln = d.ro - 1, lk = d.ro;
    const int a = matrix_operand(d, 0, lm, lk, batched);
    if (!a) return false;
    int layout  = MIMK_B_KN;
    int b       = matrix_operand(d, 1, lk, ln, batched);
    if (!b) {
        b      = matrix_operand(d, 1, ln, lk, batched);
        layout = MIMK_B_NK;
    }
    if (!b) return false;
    mimk_gemm_desc& g = p.gemm;
    g.batch = batched ? d.sr[0] : 1;
    g.m = d.sr[lm], g.n = d.sr[ln], g.k = d.sr[lk];
    g.a = d.in[0], g.b = d.in[1], g.c = d.out;
    g.stride_a = a == 2 ? g.m * g.k : 0;
    g.stride_b = b == 2 ? g.k * g.n : 0;
    g.stride_c = g.m * g.n;
    g.in_dtype = d.in_dtype[0], g.out_dtype = d.out_dtype, g.b_layout = layout;
    g.post_row = nullptr, g.post_full = nullptr;
    switch (d.post) {
        case MIMK_P_ID: g.post = MIMK_POST_ID; return true;
        case MIMK_P_RELU: g.post = MIMK_POST_RELU; return true;
        case MIMK_P_SILU: g.post = MIMK_POST_SILU; return true;
        case MIMK_P_ADD:
        case MIMK_P_ADD_RELU:
        case MIMK_P_ADD_TANH: {
            if (d.nps != 1) return false;
            const mimk_affine_map& pm = d.post_map[0];
            // a bias row: one result, the last write coordinate
            if (pm.rows == 1 && row_is_loop(pm, 0, d.ro, d.ro - 1) && d.post_dtype[0] == MIMK_F32 && d.post_shape[0][0] == g.n) {
                g.post = d.post == MIMK_P_ADD ? MIMK_POST_BIAS : d.post == MIMK_P_ADD_RELU ? MIMK_POST_BIAS_RELU : MIMK_POST_BIAS_TANH;
                g.post_row = d.post_in[0];
                return true;
            }
            // a full-shape addend read at the write coordinates
            if (d.post == MIMK_P_ADD && pm.rows == d.ro && d.post_dtype[0] == d.out_dtype) {
                for (int j = 0; j < d.ro; ++j)
                    if (!row_is_loop(pm, j, d.ro, j) || d.post_shape[0][j] != d.so[j]) return false;
                g.post = MIMK_POST_ADD_FULL;
                g.post_full = d.post_in[0];
                return true;
            }
            return false;
        }
        default: return false;
    }
}

bool plan_reduce(const mimk_mrp_desc& d, Plan& p) {
    // a plain fold, or one whose combiner has an elementwise producer inlined: fold(acc, outer(inner(a [, b])))
    int fold = d.comb, inner_op = -1, outer_op = MIMK_OP_COPY;
    const bool composed = decode_composed(d.comb, &fold, &inner_op, &outer_op);
    if (d.comb == MIMK_F_ADD_SUBEXP) fold = MIMK_F_ADD, inner_op = MIMK_OP_SUBEXP;
    const int nis = inner_op >= 0 && op_is_binary(inner_op) ? 2 : 1;
    if (d.nis != nis || d.nps != 0 || d.post != MIMK_P_ID || d.rn != d.ro + 1 || d.ro < 1) return false;
    if (d.acc_dtype != MIMK_F32 || !out_is_identity(d)) return false;
    if ((d.in_dtype[0] != MIMK_F32 && d.in_dtype[0] != MIMK_BF16) || d.out_dtype != d.in_dtype[0]) return false;
    if (nis == 2 && d.in_dtype[1] != d.in_dtype[0]) return false;
    (void)composed;
    const uint32_t init = init32(d);
    if (fold == MIMK_F_ADD && init == 0u) p.monoid = MIMK_SUM;
    else if (fold == MIMK_F_MAX && init == 0xff800000u) p.monoid = MIMK_MAX;
    else if (fold == MIMK_F_MIN && init == 0x7f800000u) p.monoid = MIMK_MIN;
    else return false;
    const mimk_affine_map& m = d.in_map[0];
    if (m.rows != d.rn) return false;
    // the folded loop sits at one axis `ax` of the operand; the output loops fill the other axes in order
    int ax = -1;
    for (int j = 0; j < m.rows; ++j)
        if (row_is_loop(m, j, d.rn, d.ro)) { ax = j; break; }
    if (ax < 0) return false;
    for (int j = 0; j < m.rows; ++j) {
        const int l = j < ax ? j : j == ax ? d.ro : j - 1;
        if (!row_is_loop(m, j, d.rn, l) || d.in_shape[0][j] != d.sr[l]) return false;
    }
    p.outer = prod(d.sr, 0, ax), p.len = d.sr[d.ro], p.inner = prod(d.sr, ax, d.ro);
    if (inner_op < 0) return true;
    p.pre_inner = inner_op, p.pre_outer = outer_op, p.pre_y_mode = 3;
    if (nis == 1) return true;
    // where the producer's second operand sits relative to the folded operand's axes (axis j of x is loop
    // j below `ax`, the folded loop at `ax`, loop j - 1 above): all of them (0), all but the folded one (1), or the
    // folded one and everything after it (2)
    const mimk_affine_map& y = d.in_map[1];
    auto loop_of = [&](int j) { return j < ax ? j : j == ax ? d.ro : j - 1; };
    auto rows_from = [&](int first_axis, int skip) {
        int j = first_axis;
        for (int r = 0; r < y.rows; ++r, ++j) {
            if (j == skip) ++j;
            if (j >= m.rows || !row_is_loop(y, r, d.rn, loop_of(j)) || d.in_shape[1][r] != d.sr[loop_of(j)]) return false;
        }
        return true;
    };
    if (y.rows == m.rows && rows_from(0, -1)) p.pre_y_mode = 0;
    else if (y.rows == m.rows - 1 && rows_from(0, ax)) p.pre_y_mode = 1;
    else if (y.rows == m.rows - ax && rows_from(ax, -1)) p.pre_y_mode = 2;
    else return false;
    return true;
}

// How operand `i` of an elementwise instance relates to the output loops: 0 = same shape, read at identity;
// 1 = one axis `ax` dropped (broadcast along it); 2 = only the trailing axes from `ax` on (broadcast over the leading
// ones); -1 = none of these.
int broadcast_kind(const mimk_mrp_desc& d, int i, int* ax) {
    const mimk_affine_map& m = d.in_map[i];
    const int n              = d.ro;
    auto rows_are = [&](int first_loop, int skip) {
        int l = first_loop;
        for (int j = 0; j < m.rows; ++j, ++l) {
            if (l == skip) ++l;
            if (l >= n || !row_is_loop(m, j, d.rn, l) || d.in_shape[i][j] != d.sr[l]) return false;
        }
        return true;
    };
    if (m.rows == n && rows_are(0, -1)) return 0;
    if (m.rows >= 1 && m.rows < n && rows_are(n - m.rows, -1)) {
        *ax = n - m.rows;
        return 2;
    }
    if (m.rows == n - 1)
        for (int a = 0; a < n; ++a)
            if (rows_are(0, a)) {
                *ax = a;
                return 1;
            }
    return -1;
}

bool plan_map(const mimk_mrp_desc& d, Plan& p) {
    if (d.rn != d.ro || d.ro < 1 || d.nps != 0 || d.acc_dtype != MIMK_F32 || !out_is_identity(d)) return false;
    for (int i = 0; i < d.nis; ++i)  // operands of one floating-point element type
        if ((d.in_dtype[i] != MIMK_F32 && d.in_dtype[i] != MIMK_BF16) || d.in_dtype[i] != d.in_dtype[0]) return false;
    int ax = 0;
    // FIRST(outer(inner(a [, b]))): an elementwise operator with a unary one behind it
    int c_fold = 0, c_inner = 0, c_outer = 0;
    if (decode_composed(d.comb, &c_fold, &c_inner, &c_outer)) {
        if (c_fold != MIMK_F_FIRST || d.post != MIMK_P_ID || d.nis != (op_is_binary(c_inner) ? 2 : 1)) return false;
        if (broadcast_kind(d, 0, &ax) != 0) return false;
        p.op = MIMK_OP_COMPOSED(c_inner, c_outer);
        if (d.nis == 1) {
            p.outer = 1, p.len = prod(d.sr, 0, d.ro), p.inner = 1, p.y_mode = 3;
            return true;
        }
        switch (broadcast_kind(d, 1, &ax)) {
            case 0: p.outer = 1, p.len = prod(d.sr, 0, d.ro), p.inner = 1, p.y_mode = 0; return true;
            case 1: p.outer = prod(d.sr, 0, ax), p.len = d.sr[ax], p.inner = prod(d.sr, ax + 1, d.ro), p.y_mode = 1; return true;
            case 2: p.outer = prod(d.sr, 0, ax), p.len = prod(d.sr, ax, d.ro), p.inner = 1, p.y_mode = 2; return true;
            default: return false;
        }
    }
    if (d.nis == 1 && d.comb == MIMK_F_FIRST) {
        if (broadcast_kind(d, 0, &ax) != 0) return false;
        p.op = d.post == MIMK_P_ID ? MIMK_OP_COPY : d.post == MIMK_P_RELU ? MIMK_OP_RELU : d.post == MIMK_P_SILU ? MIMK_OP_SILU : -1;
        if (p.op < 0) return false;
        p.outer = 1, p.len = prod(d.sr, 0, d.ro), p.inner = 1, p.y_mode = 3;
        return true;
    }
    if (d.nis != 2 || d.post != MIMK_P_ID) return false;
    switch (d.comb) {
        case MIMK_F_ADD2: p.op = MIMK_OP_ADD; break;
        case MIMK_F_MUL2: p.op = MIMK_OP_MUL; break;
        case MIMK_F_DIV: p.op = MIMK_OP_DIV; break;
        case MIMK_F_SUBEXP: p.op = MIMK_OP_SUBEXP; break;
        default: return false;
    }
    if (broadcast_kind(d, 0, &ax) != 0) return false;
    switch (broadcast_kind(d, 1, &ax)) {
        case 0: p.outer = 1, p.len = prod(d.sr, 0, d.ro), p.inner = 1, p.y_mode = 0; return true;
        case 1: p.outer = prod(d.sr, 0, ax), p.len = d.sr[ax], p.inner = prod(d.sr, ax + 1, d.ro), p.y_mode = 1; return true;
        case 2: p.outer = prod(d.sr, 0, ax), p.len = prod(d.sr, ax, d.ro), p.inner = 1, p.y_mode = 2; return true;
        default: return false;
    }
}

// A copy whose input map permutes the output loops (tensor.transpose): any element type, it moves bits only.
bool plan_permute(const mimk_mrp_desc& d, Plan& p) {
    if (d.comb != MIMK_F_FIRST || d.post != MIMK_P_ID || d.nis != 1 || d.nps != 0 || d.rn != d.ro || d.ro < 2) return false;
    if (d.in_dtype[0] != d.out_dtype || !out_is_identity(d)) return false;
    const mimk_affine_map& m = d.in_map[0];
    if (m.rows != d.ro) return false;
    bool seen[MIMK_MRP_MAX_RANK] = {};
    for (int j = 0; j < m.rows; ++j) {
        int l = -1;
        for (int c = 0; c < d.ro; ++c)
            if (row_is_loop(m, j, d.rn, c)) { l = c; break; }
        if (l < 0 || seen[l] || d.in_shape[0][j] != d.sr[l]) return false;
        seen[l]   = true;
        p.perm[j] = l;
    }
    return p.perm[d.ro - 1] != d.ro - 1;  // the same fastest axis on both sides: the per-cell kernel is coalesced already
}

// A copy whose input map is `reshape_map` of the whole operand -- delinearize(linearize(o, s_out), s_in), tensor.mim:1224-1233
// -- reads element i of the flat input into element i of the flat output: no element moves.
bool plan_reshape(const mimk_mrp_desc& d) {
    if (d.comb != MIMK_F_FIRST || d.post != MIMK_P_ID || d.nis != 1 || d.nps != 0 || d.rn != d.ro || d.ro < 1) return false;
    if (d.in_dtype[0] != d.out_dtype || !out_is_identity(d)) return false;
    const mimk_affine_map& m = d.in_map[0];
    if (m.rows < 1 || prod(d.in_shape[0], 0, m.rows) != prod(d.so, 0, d.ro)) return false;
    for (int j = 0; j < m.rows; ++j) {
        // linearize(o, s_out): the row-major strides of the result's shape, no constant
        for (int l = 0; l < d.ro; ++l)
            if (m.coef[j][l] != prod(d.so, l + 1, d.ro)) return false;
        if (m.coef[j][d.rn] != 0) return false;
        // delinearize(., s_in)#j = (lin floordiv stride_j) rem s_in#j; a division by 1 and the outermost rem may be left out
        const int64_t stride = prod(d.in_shape[0], j + 1, m.rows);
        if (!(m.div[j] == stride || (stride == 1 && m.div[j] <= 0))) return false;
        if (!(m.mod[j] == d.in_shape[0][j] || (j == 0 && m.mod[j] <= 0))) return false;
    }
    return true;
}

// Below this many combiner applications the per-cell kernel is kept: it is launch-bound there anyway, and it keeps
// the ascending fold of the classic nest bit for bit.
constexpr long long ROUTE_MIN_WORK = 1ll << 20;

Plan make_plan(const mimk_mrp_desc& d, bool any_size = false) {
    Plan p;
    if (d.ro < 0 || d.rn < d.ro || d.rn > MIMK_MRP_MAX_LOOPS || d.ro > MIMK_MRP_MAX_RANK) return p;
    if (d.nis < 1 || d.nis > 2) return p;
    for (int i = 0; i < d.nis; ++i)
        if (d.in_map[i].rows < 0 || d.in_map[i].rows > MIMK_MRP_MAX_RANK) return p;
    long double work = 1;
    for (int l = 0; l < d.rn; ++l) {
        if (d.sr[l] <= 0) return p;
        work *= (long double)d.sr[l];
    }
    if (plan_reshape(d)) {  // bits only, the same at any size
        p.route = MIMK_ROUTE_COPY;
        return p;
    }
    if (!any_size && work < (long double)ROUTE_MIN_WORK) return p;
    if (plan_gemm(d, p)) p.route = MIMK_ROUTE_GEMM;
    else if (plan_reduce(d, p)) p.route = MIMK_ROUTE_REDUCE;
    else if (plan_map(d, p)) p.route = MIMK_ROUTE_MAP;
    else if (plan_permute(d, p)) p.route = MIMK_ROUTE_PERMUTE;
    return p;
}

}  // namespace

MrpPlan mrp_plan(const mimk_mrp_desc& d) { return make_plan(d, true); }

// Runs `d` on a specialised kernel when one applies. Returns false when the generic kernel should take it; otherwise
// *status holds the specialised entry point's status. MIMK_MRP_ROUTE=0 in the environment keeps everything generic.
bool mrp_try_route(const mimk_mrp_desc& d, void* stream, int* status) {
    static const bool enabled = [] {
        const char* e = std::getenv("MIMK_MRP_ROUTE");
        return !(e && e[0] == '0');
    }();
    if (!enabled) return false;
    const Plan p = make_plan(d);
    switch (p.route) {
        case MIMK_ROUTE_GEMM: *status = mimk_gemm(&p.gemm, stream); return true;
        case MIMK_ROUTE_REDUCE:
            if (p.pre_inner >= 0) {
                const mimk_producer pre{p.pre_inner, p.pre_outer, p.pre_y_mode, 0, d.nis == 2 ? d.in[1] : nullptr};
                *status = mimk_reduce_fused(d.in[0], &pre, d.out, d.in_dtype[0], p.outer, p.len, p.inner, p.monoid, stream);
            } else {
                *status = mimk_reduce(d.in[0], d.out, d.in_dtype[0], p.outer, p.len, p.inner, p.monoid, stream);
            }
            return true;
        case MIMK_ROUTE_MAP:
            *status = mimk_map_t(p.op, d.in[0], d.nis == 2 ? d.in[1] : nullptr, d.out, d.in_dtype[0], d.out_dtype, p.outer, p.len, p.inner,
                                 p.y_mode, stream);
            return true;
        case MIMK_ROUTE_PERMUTE: {
            const int esize = d.out_dtype == MIMK_BF16 ? 2 : d.out_dtype == MIMK_I64 ? 8 : 4;
            *status = permute_copy(d.in[0], d.out, esize, d.ro, d.sr, p.perm, static_cast<cudaStream_t>(stream));
            return true;
        }
        case MIMK_ROUTE_COPY: {
            const size_t esize = d.out_dtype == MIMK_BF16 ? 2 : d.out_dtype == MIMK_I64 ? 8 : 4;
            *status = note_cuda_error(cudaMemcpyAsync(d.out, d.in[0], size_t(prod(d.so, 0, d.ro)) * esize, cudaMemcpyDeviceToDevice,
                                                      static_cast<cudaStream_t>(stream)));
            return true;
        }
        default: return false;
    }
}

}  // namespace mimk

extern "C" int mimk_mrp_classify(const mimk_mrp_desc* d) {
    if (!d) return MIMK_ROUTE_GENERIC;
    return mimk::make_plan(*d).route;
}
