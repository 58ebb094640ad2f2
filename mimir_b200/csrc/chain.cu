// Matrix-chain association: in which order to multiply A0 · A1 · … · A(n-1).
//
// The reference decides this at compile time (tensor.reassoc, MimIR src/mim/plug/tensor/phase/reassoc.cpp): it
// flattens nested product_2d / transpose_2d applications into a chain, prices every product
// «x,y»·«y,z» in vector-lane slots of its CPU schedules (reassoc.cpp:89-128: the trailing extent z is the vector
// loop and is charged rounded up to whole vectors; when the right operand is a leaf read through a transpose the
// contraction y is the vector loop instead) and rebuilds the cheapest bracketing (reassoc.cpp:172-206). With
// symbolic extents it emits a run-time tournament over the surviving bracketings (reassoc.cpp:287-313).
//
// Here every extent is known when the chain is about to run, so the tournament collapses into one dynamic program
// evaluated at call time. Two price lists:
//   MIMK_COST_LANES  the reference's, unchanged, so that its documented decisions can be reproduced;
//   MIMK_COST_B200   seconds on this GPU: a product is the slower of its tensor-core time -- whole output tiles in whole
//                    waves over the SMs, K in whole K-steps -- and its HBM time, plus a launch; a transposed leaf
//                    used as a LEFT operand pays for the copy that makes it row-major (the contraction kernels read
//                    only the right operand through a transpose).
// Host logic only: no device is touched.
#include <cmath>
#include <vector>

#include "common.cuh"

namespace mimk {
namespace {

struct Chain {
    int n;
    const int64_t* dims;
    const int32_t* transposed;  // may be null
    int model, param;
    bool leaf_t(int i) const { return transposed && transposed[i] != 0; }
};

double lanes(double v, double vec) { return std::ceil(v / vec) * vec; }

// Figures of this library's own kernels on one B200: bf16 contraction 1.45 PFLOP/s sustained (128 x 256 tiles, K-step
// 64), f32 contraction as three TF32 products 0.21 PFLOP/s (128 x 128 tiles, K-step 32), 6.4 TB/s of HBM, 148 SMs.
constexpr double SMS = 148.0, HBM_BPS = 6.4e12, LAUNCH_S = 4e-6;

double b200_product(double m, double k, double n, int dtype) {
    const bool half   = dtype == MIMK_BF16;
    const double tm   = 128.0, tn = half ? 256.0 : 128.0, tk = half ? 64.0 : 32.0;
    const double peak = half ? 1.45e15 : 0.21e15;
    const double es   = half ? 2.0 : 4.0;
    const double tiles = std::ceil(m / tm) * std::ceil(n / tn);
    const double waves = std::ceil(tiles / SMS);
    const double t_tc  = waves * (2.0 * tm * tn * lanes(k, tk)) / (peak / SMS);
    const double t_mem = (m * k + k * n + m * n) * es / HBM_BPS;
    return std::fmax(t_tc, t_mem) + LAUNCH_S;
}

// One product of sub-chains i..s and s+1..j. `t` asks for the product stored transposed, i.e. the kernel computes
// (s+1..j)^T . (i..s)^T (reassoc.cpp:224-231: (A . B)^T = B^T . A^T); `ol` / `orr` say whether the left / right part is
// itself stored transposed (a transposed leaf, or a node built with t). The operand the kernel sees on its right is read
// through a transpose whenever its storage and the consumer disagree.
double product_cost(const Chain& c, int i, int s, int j, bool t, bool ol, bool orr) {
    const double x = (double)c.dims[i], y = (double)c.dims[s + 1], z = (double)c.dims[j + 1];
    const double m = t ? z : x, n = t ? x : z;              // the kernel's output is m x n
    const bool right_through_transpose = t ? (ol != t) : (orr != t);
    const bool left_needs_copy         = t ? (orr != t) : (ol != t);
    if (c.model == MIMK_COST_LANES) {
        const double vec = c.param > 0 ? (double)c.param : 8.0;
        return right_through_transpose ? m * lanes(y, vec) * n : m * y * lanes(n, vec);
    }
    double cost = b200_product(m, y, n, c.param);
    if (left_needs_copy) {  // the contraction kernels read only their right operand through a transpose
        const double es = c.param == MIMK_BF16 ? 2.0 : 4.0;
        cost += 2.0 * m * y * es / HBM_BPS + LAUNCH_S;
    }
    return cost;
}

bool chain_ok(const Chain& c) {
    if (c.n < 1 || c.n > MIMK_CHAIN_MAX || !c.dims) return false;
    if (c.model != MIMK_COST_LANES && c.model != MIMK_COST_B200) return false;
    if (c.model == MIMK_COST_B200 && c.param != MIMK_F32 && c.param != MIMK_BF16) return false;
    for (int i = 0; i <= c.n; ++i)
        if (c.dims[i] < 0) return false;
    return true;
}

struct Choice {
    int s = 0;
    bool ol = false, orr = false;
};

void emit(const std::vector<Choice>& pick, int n, int i, int j, bool t, mimk_chain_split* out, int* count) {
    if (i == j) return;
    const Choice& p = pick[(i * n + j) * 2 + t];
    emit(pick, n, i, p.s, p.ol, out, count);
    emit(pick, n, p.s + 1, j, p.orr, out, count);
    out[*count].i = i, out[*count].s = p.s, out[*count].j = j, out[*count].t = t;
    ++*count;
}

}  // namespace
}  // namespace mimk

using namespace mimk;

extern "C" int mimk_chain_order(int32_t n, const int64_t* dims, const int32_t* transposed, int32_t model, int32_t param,
                                mimk_chain_split* splits, double* cost) {
    const Chain c{n, dims, transposed, model, param};
    if (!chain_ok(c) || (n > 1 && !splits)) return MIMK_E_ARG;
    // best[(i, j, t)]: cheapest way to have sub-chain i..j stored plainly (t = 0) or transposed (t = 1). A leaf is stored
    // the way it is given; the reference's price list only ever builds plain nodes (reassoc.cpp:131-144).
    std::vector<double> best(n * n * 2, INFINITY);
    std::vector<Choice> pick(n * n * 2);
    for (int i = 0; i < n; ++i) best[(i * n + i) * 2 + (c.leaf_t(i) ? 1 : 0)] = 0.0;
    const int n_orient = model == MIMK_COST_B200 ? 2 : 1;
    for (int len = 2; len <= n; ++len)
        for (int i = 0; i + len <= n; ++i) {
            const int j = i + len - 1;
            for (int t = 0; t < n_orient; ++t) {
                double b = INFINITY;
                Choice ch;
                for (int s = i; s < j; ++s)  // equal costs keep the first (lowest) split, like reassoc.cpp:188-196
                    for (int ol = 0; ol < 2; ++ol)
                        for (int orr = 0; orr < 2; ++orr) {
                            const double l = best[(i * n + s) * 2 + ol], r = best[((s + 1) * n + j) * 2 + orr];
                            if (!(l < INFINITY) || !(r < INFINITY)) continue;
                            const double v = product_cost(c, i, s, j, t != 0, ol != 0, orr != 0) + l + r;
                            if (v < b) b = v, ch.s = s, ch.ol = ol != 0, ch.orr = orr != 0;
                        }
                best[(i * n + j) * 2 + t] = b;
                pick[(i * n + j) * 2 + t] = ch;
            }
        }
    int count = 0;
    emit(pick, n, 0, n - 1, false, splits, &count);  // the chain's own result is stored plainly
    if (cost) *cost = n > 1 ? best[(n - 1) * 2] : 0.0;
    return MIMK_OK;
}

extern "C" int mimk_chain_cost(int32_t n, const int64_t* dims, const int32_t* transposed, int32_t model, int32_t param,
                               const mimk_chain_split* splits, int32_t n_splits, double* cost) {
    const Chain c{n, dims, transposed, model, param};
    if (!chain_ok(c) || !cost || n_splits < 0 || (n_splits > 0 && !splits)) return MIMK_E_ARG;
    // how a part i..j is stored: a leaf as given, a node as the product that builds it says
    auto stored_t = [&](int i, int j, bool* t) {
        if (i == j) {
            *t = c.leaf_t(i);
            return true;
        }
        for (int q = 0; q < n_splits; ++q)
            if (splits[q].i == i && splits[q].j == j) {
                *t = splits[q].t != 0;
                return true;
            }
        return false;
    };
    double total = 0.0;
    for (int q = 0; q < n_splits; ++q) {
        const mimk_chain_split& sp = splits[q];
        if (sp.i < 0 || sp.i > sp.s || sp.s >= sp.j || sp.j >= n) return MIMK_E_ARG;
        bool ol = false, orr = false;
        if (!stored_t(sp.i, sp.s, &ol) || !stored_t(sp.s + 1, sp.j, &orr)) return MIMK_E_ARG;
        total += product_cost(c, sp.i, sp.s, sp.j, sp.t != 0, ol, orr);
    }
    *cost = total;
    return MIMK_OK;
}
