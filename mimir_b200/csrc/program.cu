// Program-level recognisers: chains of `map_reduce_post` operations that spell softmax or attention run as one fused
// kernel.
//
// By the time any phase of the reference runs, `softmax` is already four map_reduce operations -- max-fold, exp(x - max),
// sum-fold, divide (MimIR src/mim/plug/tensor/tensor.mim:1172-1176) -- or three after fuse_tensor has inlined the
// exponential into its two consumers (src/mim/plug/tensor/phase/fuse.cpp:225-245), and attention is seven: two
// contractions around that softmax (lit/tensor/attn_exec.mim:20-22). A lowering that emits one launcher call per
// operation therefore hands this library a list; run op by op it costs three passes over the matrix for softmax and a
// materialised score matrix for attention. Here the list is matched against those shapes (on the single-operation
// recognisers of mrp_route.cu plus the dataflow between operations: an input pointer equal to an earlier `out`), and a
// chain whose temporaries feed nothing else runs on mimk_softmax / mimk_attn_fwd.
#include "common.cuh"

namespace mimk {
namespace {

bool is_float(int dt) { return dt == MIMK_F32 || dt == MIMK_BF16; }

// Does any operation outside [lo, hi) read `ptr`?
bool read_outside(const mimk_mrp_desc* ops, int n, int lo, int hi, const void* ptr) {
    for (int i = 0; i < n; ++i) {
        if (i >= lo && i < hi) continue;
        for (int k = 0; k < ops[i].nis; ++k)
            if (ops[i].in[k] == ptr) return true;
        for (int k = 0; k < ops[i].nps; ++k)
            if (ops[i].post_in[k] == ptr) return true;
    }
    return false;
}

struct Softmax {
    int len_ops = 0;  // operations the chain spans (4 unfused, 3 fused)
    const void* x = nullptr;
    void* y = nullptr;
    int in_dtype = 0, out_dtype = 0;
    int64_t outer = 0, len = 0, inner = 0;
};

// A fold of x along one axis with (fmax, -inf): the view [outer, len, inner] it is taken over.
bool match_max_fold(const mimk_mrp_desc& d, Softmax& s) {
    const MrpPlan p = mrp_plan(d);
    if (p.route != MIMK_ROUTE_REDUCE || p.monoid != MIMK_MAX) return false;
    s.x = d.in[0], s.in_dtype = d.in_dtype[0];
    s.outer = p.outer, s.len = p.len, s.inner = p.inner;
    return true;
}
bool same_view(const MrpPlan& p, const Softmax& s) { return p.outer == s.outer && p.len == s.len && p.inner == s.inner; }
// An elementwise plan whose second operand lacks the softmax axis. Along the leading axis that is the same thing as an
// operand broadcast over the leading extent, which is how the single-operation recogniser reports it.
bool along_axis(const MrpPlan& p, const Softmax& s) {
    if (p.y_mode == 1) return same_view(p, s);
    return p.y_mode == 2 && s.outer == 1 && p.outer == s.len && p.len * p.inner == s.inner;
}

// The fused forms fuse_map_reduce leaves are not among the single-operation routes: match their maps here.
//   sum fold:  comb ADD_SUBEXP, init 0, inputs (x read like a fold along the axis, max read at the output loops)
//   divide:    comb SUBEXP_DIV, inputs (x at identity, max and sum with the axis dropped)
bool match_fused_sum(const mimk_mrp_desc& d, const Softmax& s, const void* mx) {
    if (d.comb != MIMK_F_ADD_SUBEXP || d.nis != 2 || d.nps != 0 || d.post != MIMK_P_ID || d.acc_dtype != MIMK_F32) return false;
    if ((uint32_t)((uint64_t)d.init_bits & 0xffffffffu) != 0u || d.in[0] != s.x || d.in[1] != mx) return false;
    // the same operation with a plain add over x alone is the fold the router knows; the max operand must be read at the
    // output loops in order
    mimk_mrp_desc fold = d;
    fold.comb = MIMK_F_ADD, fold.nis = 1;
    fold.out_dtype = d.in_dtype[0];
    const MrpPlan p = mrp_plan(fold);
    if (p.route != MIMK_ROUTE_REDUCE || p.monoid != MIMK_SUM || !same_view(p, s)) return false;
    const mimk_affine_map& m = d.in_map[1];
    if (m.rows != d.ro) return false;
    for (int j = 0; j < m.rows; ++j) {
        for (int c = 0; c <= d.rn; ++c)
            if (m.coef[j][c] != (c == j ? 1 : 0)) return false;
        if (m.div[j] > 0 || m.mod[j] > 0 || d.in_shape[1][j] != d.sr[j]) return false;
    }
    return true;
}
bool match_fused_div(const mimk_mrp_desc& d, const Softmax& s, const void* mx, const void* sum) {
    if (d.comb != MIMK_F_SUBEXP_DIV || d.nis != 3 || d.nps != 0 || d.post != MIMK_P_ID || d.acc_dtype != MIMK_F32) return false;
    if (d.in[0] != s.x || d.in[1] != mx || d.in[2] != sum) return false;
    // exp(x - max) alone is the binary_ax map the router knows; the sum operand must be read through the max operand's map
    mimk_mrp_desc m2 = d;
    m2.comb = MIMK_F_SUBEXP, m2.nis = 2;
    const MrpPlan p = mrp_plan(m2);
    if (p.route != MIMK_ROUTE_MAP || p.op != MIMK_OP_SUBEXP || !along_axis(p, s)) return false;
    const mimk_affine_map &a = d.in_map[1], &b = d.in_map[2];
    if (a.rows != b.rows) return false;
    for (int j = 0; j < a.rows; ++j) {
        for (int c = 0; c <= d.rn; ++c)
            if (a.coef[j][c] != b.coef[j][c]) return false;
        if (a.div[j] != b.div[j] || a.mod[j] != b.mod[j] || d.in_shape[1][j] != d.in_shape[2][j]) return false;
    }
    return true;
}

bool match_softmax(const mimk_mrp_desc* ops, int n, int at, Softmax& s) {
    if (at + 3 > n) return false;
    if (!match_max_fold(ops[at], s)) return false;
    const void* mx = ops[at].out;
    if (!is_float(s.in_dtype) || ops[at].out_dtype != s.in_dtype) return false;
    // fused form: three operations
    if (match_fused_sum(ops[at + 1], s, mx) && match_fused_div(ops[at + 2], s, mx, ops[at + 1].out)) {
        s.len_ops = 3, s.y = ops[at + 2].out, s.out_dtype = ops[at + 2].out_dtype;
        if (read_outside(ops, n, at, at + 3, mx) || read_outside(ops, n, at, at + 3, ops[at + 1].out)) return false;
        return true;
    }
    if (at + 4 > n) return false;
    // e = exp(x - max) along the axis
    const MrpPlan pe = mrp_plan(ops[at + 1]);
    if (pe.route != MIMK_ROUTE_MAP || pe.op != MIMK_OP_SUBEXP || !along_axis(pe, s)) return false;
    if (ops[at + 1].in[0] != s.x || ops[at + 1].in[1] != mx) return false;
    const void* e = ops[at + 1].out;
    // sum = fold of e along the axis
    const MrpPlan ps = mrp_plan(ops[at + 2]);
    if (ps.route != MIMK_ROUTE_REDUCE || ps.monoid != MIMK_SUM || !same_view(ps, s) || ops[at + 2].in[0] != e) return false;
    const void* sum = ops[at + 2].out;
    // y = e / sum along the axis
    const MrpPlan pd = mrp_plan(ops[at + 3]);
    if (pd.route != MIMK_ROUTE_MAP || pd.op != MIMK_OP_DIV || !along_axis(pd, s)) return false;
    if (ops[at + 3].in[0] != e || ops[at + 3].in[1] != sum) return false;
    s.len_ops = 4, s.y = ops[at + 3].out, s.out_dtype = ops[at + 3].out_dtype;
    if (read_outside(ops, n, at, at + 4, mx) || read_outside(ops, n, at, at + 4, e) || read_outside(ops, n, at, at + 4, sum)) return false;
    return true;
}

struct Attention {
    int len_ops = 0;
    mimk_attn_desc desc{};
};

// S = q k^T (k stored [keys, head_dim], read through transpose_2d), softmax of S along its last axis, O = P v.
bool match_attention(const mimk_mrp_desc* ops, int n, int at, Attention& a) {
    if (at + 5 > n) return false;
    const MrpPlan p1 = mrp_plan(ops[at]);
    if (p1.route != MIMK_ROUTE_GEMM || p1.gemm.b_layout != MIMK_B_NK || p1.gemm.post != MIMK_POST_ID) return false;
    const mimk_gemm_desc& g1 = p1.gemm;
    if (!is_float(g1.in_dtype) || g1.out_dtype != g1.in_dtype) return false;
    if (g1.batch > 1 && (g1.stride_a == 0 || g1.stride_b == 0)) return false;  // every batch entry has its own q and k
    Softmax s;
    if (!match_softmax(ops, n, at + 1, s)) return false;
    // the softmax runs over the key axis of exactly these scores
    if (s.x != g1.c || s.inner != 1 || s.len != g1.n || s.outer != g1.batch * g1.m || s.in_dtype != g1.out_dtype ||
        s.out_dtype != s.in_dtype)
        return false;
    const int last = at + 1 + s.len_ops;
    if (last >= n) return false;
    const MrpPlan p2 = mrp_plan(ops[last]);
    if (p2.route != MIMK_ROUTE_GEMM || p2.gemm.b_layout != MIMK_B_KN || p2.gemm.post != MIMK_POST_ID) return false;
    const mimk_gemm_desc& g2 = p2.gemm;
    if (g2.a != s.y || g2.in_dtype != s.out_dtype || g2.out_dtype != g1.in_dtype) return false;
    if (g2.batch != g1.batch || g2.m != g1.m || g2.k != g1.n) return false;
    if (g2.batch > 1 && (g2.stride_a == 0 || g2.stride_b == 0)) return false;
    if (g2.n != g1.k) return false;  // v has q's head_dim (the fused kernels keep one head_dim)
    if (read_outside(ops, n, at, last + 1, g1.c) || read_outside(ops, n, at, last + 1, s.y)) return false;
    a.len_ops = last + 1 - at;
    mimk_attn_desc& d = a.desc;
    d.batch_heads = g1.batch, d.seq_q = g1.m, d.seq_k = g1.n, d.head_dim = g1.k;
    d.q = g1.a, d.k = g1.b, d.v = g2.b, d.o = g2.c, d.lse = nullptr;
    d.scale = 1.f, d.causal = 0, d.dtype = g1.in_dtype;
    return true;
}

// An elementwise map (unary, binary, binary_ax, bias-style broadcast) followed by a fold of its result along one axis,
// the result read by nothing else: the fold runs over the produced values without the tensor being written.
struct FoldOfMap {
    const void* x = nullptr;
    void* out = nullptr;
    mimk_producer pre{};
    int dtype = 0, monoid = 0;
    int64_t outer = 0, len = 0, inner = 0;
};
bool match_fold_of_map(const mimk_mrp_desc* ops, int n, int at, FoldOfMap& f) {
    if (at + 2 > n) return false;
    const mimk_mrp_desc &m = ops[at], &r = ops[at + 1];
    const MrpPlan pm = mrp_plan(m), pf = mrp_plan(r);
    if (pm.route != MIMK_ROUTE_MAP || pf.route != MIMK_ROUTE_REDUCE || pf.pre_inner >= 0) return false;
    if (r.in[0] != m.out || !is_float(m.in_dtype[0]) || m.out_dtype != m.in_dtype[0] || r.in_dtype[0] != m.out_dtype) return false;
    if (pm.outer * pm.len * pm.inner != pf.outer * pf.len * pf.inner) return false;
    if (read_outside(ops, n, at, at + 2, m.out)) return false;
    // where the map's second operand sits in the fold's [outer, len, inner] view
    int mode = -1;
    if (pm.y_mode == 3 || pm.y_mode == 0) mode = pm.y_mode;
    else if (pm.y_mode == 1 && pm.outer == pf.outer && pm.len == pf.len && pm.inner == pf.inner) mode = 1;
    else if (pm.y_mode == 2 && pm.outer == pf.outer && pm.len == pf.len * pf.inner) mode = 2;
    else if (pm.y_mode == 2 && pf.outer == 1 && pm.outer == pf.len && pm.len == pf.inner) mode = 1;  // y lacks the leading, folded axis
    if (mode < 0) return false;
    const bool unary = pm.y_mode == 3;
    f.x = m.in[0], f.out = r.out, f.dtype = m.in_dtype[0], f.monoid = pf.monoid;
    f.outer = pf.outer, f.len = pf.len, f.inner = pf.inner;
    int op_inner = 0, op_outer = 0;
    if (!decode_op(pm.op, &op_inner, &op_outer)) return false;  // the map's operator may itself be a composed pair
    f.pre.inner_op = op_inner, f.pre.outer_op = op_outer, f.pre.y_mode = mode, f.pre.pad_ = 0;
    f.pre.y = unary ? nullptr : m.in[1];
    return true;
}

// steps[i] for every operation; returns the number of fused chains.
int classify(const mimk_mrp_desc* ops, int n, int32_t* steps, Softmax* sm, Attention* at_out, FoldOfMap* fm_out) {
    int chains = 0;
    for (int i = 0; i < n;) {
        Attention a;
        Softmax s;
        FoldOfMap fm;
        if (match_attention(ops, n, i, a)) {
            steps[i] = MIMK_STEP_ATTENTION;
            for (int k = 1; k < a.len_ops; ++k) steps[i + k] = MIMK_STEP_ABSORBED;
            if (at_out) at_out[i] = a;
            i += a.len_ops, ++chains;
        } else if (match_softmax(ops, n, i, s)) {
            steps[i] = MIMK_STEP_SOFTMAX;
            for (int k = 1; k < s.len_ops; ++k) steps[i + k] = MIMK_STEP_ABSORBED;
            if (sm) sm[i] = s;
            i += s.len_ops, ++chains;
        } else if (match_fold_of_map(ops, n, i, fm)) {
            steps[i] = MIMK_STEP_FOLD_OF_MAP, steps[i + 1] = MIMK_STEP_ABSORBED;
            if (fm_out) fm_out[i] = fm;
            i += 2, ++chains;
        } else {
            steps[i++] = MIMK_STEP_OP;
        }
    }
    return chains;
}

bool sane(const mimk_mrp_desc& d) {
    return d.ro >= 0 && d.rn >= d.ro && d.rn <= MIMK_MRP_MAX_LOOPS && d.ro <= MIMK_MRP_MAX_RANK && d.nis >= 0 &&
           d.nis <= MIMK_MRP_MAX_INPUTS && d.nps >= 0 && d.nps <= 1;
}

}  // namespace
}  // namespace mimk

using namespace mimk;

extern "C" int mimk_program_classify(const mimk_mrp_desc* ops, int32_t n_ops, int32_t* steps) {
    if (n_ops < 0 || (n_ops > 0 && (!ops || !steps))) return MIMK_E_ARG;
    for (int i = 0; i < n_ops; ++i)
        if (!sane(ops[i])) return MIMK_E_ARG;
    classify(ops, n_ops, steps, nullptr, nullptr, nullptr);
    return MIMK_OK;
}

extern "C" int mimk_program_run(const mimk_mrp_desc* ops, int32_t n_ops, void* stream) {
    if (n_ops < 0 || (n_ops > 0 && !ops)) return MIMK_E_ARG;
    if (n_ops > 4096) return MIMK_E_UNSUPPORTED;
    for (int i = 0; i < n_ops; ++i)
        if (!sane(ops[i])) return MIMK_E_ARG;
    if (n_ops == 0) return MIMK_OK;
    int32_t* steps = new int32_t[n_ops];
    Softmax* sm    = new Softmax[n_ops];
    Attention* at  = new Attention[n_ops];
    FoldOfMap* fm  = new FoldOfMap[n_ops];
    classify(ops, n_ops, steps, sm, at, fm);
    int st = MIMK_OK;
    for (int i = 0; i < n_ops && st == MIMK_OK; ++i) {
        switch (steps[i]) {
            case MIMK_STEP_ATTENTION: st = mimk_attn_fwd(&at[i].desc, stream); break;
            case MIMK_STEP_SOFTMAX:
                st = mimk_softmax(sm[i].x, sm[i].y, sm[i].in_dtype, sm[i].out_dtype, sm[i].outer, sm[i].len, sm[i].inner, stream);
                break;
            case MIMK_STEP_FOLD_OF_MAP:
                st = mimk_reduce_fused(fm[i].x, &fm[i].pre, fm[i].out, fm[i].dtype, fm[i].outer, fm[i].len, fm[i].inner, fm[i].monoid, stream);
                break;
            case MIMK_STEP_OP: st = mimk_map_reduce_post(&ops[i], stream); break;
            default: break;  // absorbed into the chain before it
        }
    }
    delete[] steps;
    delete[] sm;
    delete[] at;
    delete[] fm;
    return st;
}
