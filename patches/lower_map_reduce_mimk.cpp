// UNVERIFIED -- not compiled anywhere: the reference's toolchain is absent where this was written (see patches/README.md).
// Every helper has a body, written against the reference's headers as read. Every World / Def / Lam / Axm member it calls was
// looked up there (math::isa_f: include/mim/plug/math/math.h:55; math::tri::tanh: src/mim/plug/math/math.mim:126;
// World::Externals::operator[](Sym): include/mim/world.h:195; Def::externalize: include/mim/def.h:570; World::mut_con,
// type_i32, lit_i32: include/mim/world.h:427, 637, 586; Lam::ret_var: include/mim/lam.h:136) -- their existence and arity,
// not their behaviour. What no header shows is the CPS wrapper of mim_cu_check assumed below: the first thing to fix.
//
// Drop-in body for mim::plug::gpu::phase::LowerMapReduce::lower_map_reduce_post
// (src/mim/plug/gpu/phase/lower_map_reduce.cpp:317-395 in MimIR). It keeps that function's structure -- decode with
// btensor::MapRedPost::of, bail out to Super::rewrite_imm_App when something is not literal, splice a DS function,
// gpu.auto_init, alloc_copy_inputs for inputs and epilogue inputs, alloc_output, build_teardown -- and replaces only
// the middle: instead of build_kernel(...) + gpu.launch it emits ONE call to a mimk launcher when the operation is
// recognised. The helpers named here (extract_input_desc, alloc_copy_inputs, alloc_output, build_teardown,
// rebuild_lam_global_mem, grid_layout, build_kernel) are the file's existing ones.

namespace mim::plug::gpu::phase {

namespace {

// Element-type and enum codes of include/mimk.h (the launchers take them as I32).
constexpr int MIMK_F32 = 0, MIMK_SUM = 0, MIMK_MAX = 1, MIMK_MIN = 2;
constexpr int MIMK_POST_ID = 0, MIMK_POST_BIAS = 1, MIMK_POST_BIAS_RELU = 2, MIMK_POST_BIAS_TANH = 3, MIMK_POST_RELU = 4;

/// A map `«Rn; Index» -> «r; Index»` is a projection iff applying it to distinct markers yields markers again: the probing
/// trick of tensor::normalize_fastest_axis (src/mim/plug/tensor/normalizers.cpp:189-217). Markers are `affine.lit (l + 1)`:
/// 0 is what a dropped loop folds to, so it is not one. Returns the loop id each result reads, or nullopt.
std::optional<Vector<nat_t>> as_projection(World& w, const Def* map, nat_t n_loops, nat_t rank) {
    auto pi = map->type()->isa<Pi>();
    if (!pi) return {};
    auto dom = Lit::isa<u64>(pi->dom()->arity()), cod = Lit::isa<u64>(pi->codom()->arity());
    if (!dom || !cod || *dom != n_loops || *cod != rank) return {};
    auto markers = DefVec(n_loops, [&](size_t l) { return w.call<affine::lit>(w.lit_nat(l + 1)); });
    auto image   = w.app(map, w.tuple(markers));
    Vector<nat_t> loops(rank);
    for (nat_t j = 0; j != rank; ++j) {
        auto c = Axm::isa<affine::lit>(image->proj(rank, j));  // anything but a bare marker (add / mul / floordiv ...) is no projection
        if (!c) return {};
        auto v = Lit::isa<u64>(c->arg());
        if (!v || *v < 1 || *v > n_loops) return {};
        loops[j] = *v - 1;
    }
    return loops;
}

/// The value a returning Lam `(args..., ret) -> ret (value)` passes to its return continuation, or nullptr.
const Def* returned_value(const Lam* lam) {
    if (!lam || !lam->is_set()) return nullptr;
    auto call = lam->body()->isa<App>();
    if (!call || call->callee() != lam->ret_var()) return nullptr;
    return call->arg();
}

bool is_f32(const Def* T) {
    auto f = math::isa_f(T);  // math.F (p, e): F32 is (23, 8)
    return f && *f == 32;
}

/// `f` is `acc, (a, b) -> R.add (acc, R.mul (a, b))` over math.F32: dot_general_fun, src/mim/plug/tensor/tensor.mim:1332.
bool is_mul_add(const Lam* comb) {
    auto v = returned_value(comb);
    if (!v) return false;
    auto add = Axm::isa(math::arith::add, v);
    if (!add) return false;
    auto [x, yz] = add->args<2>();
    auto mul     = Axm::isa(math::arith::mul, yz);
    if (!mul) std::swap(x, yz), mul = Axm::isa(math::arith::mul, yz);
    if (!mul || !is_f32(v->type())) return false;
    auto acc      = comb->var(2, 0);  // (acc, inputs, ret) after the DS-to-CPS conversion the phase sees: var(0) = [acc, ins]
    auto ins      = comb->var(2, 1);
    auto [a, b]   = mul->args<2>();
    auto reads    = [&](const Def* d, nat_t i) { return d == ins->proj(2, i); };
    return x == acc && ((reads(a, 0) && reads(b, 1)) || (reads(a, 1) && reads(b, 0)));
}

/// `f` is pool_fun g (tensor.mim:1139): `acc, y -> g (acc, y)` with g one of math.arith.add / math.extrema.fmax / fmin.
std::optional<int> pool_monoid(const Lam* comb) {
    auto v = returned_value(comb);
    if (!v || !is_f32(v->type())) return {};
    auto takes_acc_and_input = [&](const App* app) {
        auto [a, b] = app->args<2>();
        auto acc = comb->var(2, 0), y = comb->var(2, 1);
        return (a == acc && b == y) || (a == y && b == acc);
    };
    if (auto add = Axm::isa(math::arith::add, v); add && takes_acc_and_input(add)) return MIMK_SUM;
    if (auto mx = Axm::isa(math::extrema::fmax, v); mx && takes_acc_and_input(mx)) return MIMK_MAX;
    if (auto mn = Axm::isa(math::extrema::fmin, v); mn && takes_acc_and_input(mn)) return MIMK_MIN;
    return {};
}

/// An elementwise operator of math over F32 as a MIMK_OP_* code, with its operands: binary `g (a, b)` or unary `u a`.
struct ElemOp {
    int op;
    const Def* a;
    const Def* b;  // nullptr for a unary operator
};
std::optional<ElemOp> elem_op(const Def* v) {
    if (auto x = Axm::isa(math::arith::add, v)) return ElemOp{MIMK_OP_ADD, x->arg(2, 0), x->arg(2, 1)};
    if (auto x = Axm::isa(math::arith::sub, v)) {
        if (auto z = Lit::isa<f32>(x->arg(2, 0)); z && *z == 0.f) return ElemOp{MIMK_OP_NEG, x->arg(2, 1), nullptr};  // math.minus
        return ElemOp{MIMK_OP_SUB, x->arg(2, 0), x->arg(2, 1)};
    }
    if (auto x = Axm::isa(math::arith::mul, v)) {
        if (x->arg(2, 0) == x->arg(2, 1)) return ElemOp{MIMK_OP_SQUARE, x->arg(2, 0), nullptr};
        return ElemOp{MIMK_OP_MUL, x->arg(2, 0), x->arg(2, 1)};
    }
    if (auto x = Axm::isa(math::arith::div, v)) {
        // math.rrt and math.slf are lams over a division by then (math.mim:283-284, 297-298): 1 / rt.sq x, 1 / (1 + exp (0 - x))
        if (auto one = Lit::isa<f32>(x->arg(2, 0)); one && *one == 1.f) {
            if (auto r = Axm::isa(math::rt::sq, x->arg(2, 1))) return ElemOp{MIMK_OP_RSQRT, r->arg(), nullptr};
            if (auto s = Axm::isa(math::arith::add, x->arg(2, 1)))
                if (auto l = Lit::isa<f32>(s->arg(2, 0)); l && *l == 1.f)
                    if (auto e = Axm::isa(math::exp::exp, s->arg(2, 1)))
                        if (auto n = Axm::isa(math::arith::sub, e->arg()))
                            if (auto z = Lit::isa<f32>(n->arg(2, 0)); z && *z == 0.f) return ElemOp{MIMK_OP_SIGMOID, n->arg(2, 1), nullptr};
        }
        return ElemOp{MIMK_OP_DIV, x->arg(2, 0), x->arg(2, 1)};
    }
    if (auto x = Axm::isa(math::rt::sq, v)) return ElemOp{MIMK_OP_SQRT, x->arg(), nullptr};
    if (auto x = Axm::isa(math::exp::log, v)) return ElemOp{MIMK_OP_LOG, x->arg(), nullptr};
    if (auto x = Axm::isa(math::exp::exp2, v)) return ElemOp{MIMK_OP_EXP2, x->arg(), nullptr};
    if (auto x = Axm::isa(math::exp::log2, v)) return ElemOp{MIMK_OP_LOG2, x->arg(), nullptr};
    if (auto x = Axm::isa(math::extrema::fmax, v)) return ElemOp{MIMK_OP_MAX, x->arg(2, 0), x->arg(2, 1)};
    if (auto x = Axm::isa(math::extrema::fmin, v)) return ElemOp{MIMK_OP_MIN, x->arg(2, 0), x->arg(2, 1)};
    if (auto x = Axm::isa(math::exp::exp, v)) {
        if (auto d = Axm::isa(math::arith::sub, x->arg())) return ElemOp{MIMK_OP_SUBEXP, d->arg(2, 0), d->arg(2, 1)};
        return ElemOp{MIMK_OP_EXP, x->arg(), nullptr};
    }
    if (auto x = Axm::isa(math::tri::tanh, v)) return ElemOp{MIMK_OP_TANH, x->arg(), nullptr};
    if (auto x = Axm::isa(math::abs, v)) return ElemOp{MIMK_OP_ABS, x->arg(), nullptr};
    return {};
}

/// What fuse_map_reduce leaves of a map feeding a fold (src/mim/plug/tensor/phase/fuse.cpp:183-358): the fold's combiner with
/// the producer's body inlined, `acc, ins -> acc (+) u (g (ins#0, ins#1))` or `acc (+) g (...)` or `acc (+) u (ins#0)`.
/// Yields (monoid, inner, outer) for mimk_reduce_fused / MIMK_F_COMPOSED; `nis` is the number of inputs the body reads.
struct ProducedFold {
    int monoid, inner, outer;
};
std::optional<ProducedFold> produced_fold(const Lam* comb, nat_t nis) {
    auto v = returned_value(comb);
    if (!v || !is_f32(v->type())) return {};
    auto acc = comb->var(2, 0), ins = comb->var(2, 1);
    int monoid = -1;
    const Def* produced = nullptr;
    auto split = [&](const App* app, int m) {
        auto [a, b] = app->args<2>();
        if (a == acc) monoid = m, produced = b;
        else if (b == acc) monoid = m, produced = a;
    };
    if (auto x = Axm::isa(math::arith::add, v)) split(x, MIMK_SUM);
    else if (auto x = Axm::isa(math::extrema::fmax, v)) split(x, MIMK_MAX);
    else if (auto x = Axm::isa(math::extrema::fmin, v)) split(x, MIMK_MIN);
    if (!produced) return {};
    auto in = [&](nat_t i) { return nis == 1 ? ins : ins->proj(nis, i); };
    auto outer = elem_op(produced);
    if (!outer) return {};
    // g (ins#0, ins#1), or u (ins#0)
    if (outer->b ? (nis == 2 && outer->a == in(0) && outer->b == in(1)) : (nis == 1 && outer->a == in(0)))
        return ProducedFold{monoid, outer->op, MIMK_OP_COPY};
    // u (g (ins#0, ins#1)) or u (u' (ins#0))
    if (outer->b) return {};
    auto inner = elem_op(outer->a);
    if (!inner) return {};
    if (inner->b ? (nis == 2 && inner->a == in(0) && inner->b == in(1)) : (nis == 1 && inner->a == in(0)))
        return ProducedFold{monoid, inner->op, outer->op};
    return {};
}

/// post is btensor.id (returns its accumulator), or what fuse_epilogue sinks into the slot (fuse.cpp:408-534):
/// `acc, b -> acc + b`, `fmax (0, acc + b)`, `tanh (acc + b)`, `fmax (0, acc)`. Yields MIMK_POST_*.
std::optional<int> post_kind(const Lam* post, nat_t nps) {
    auto v = returned_value(post);
    if (!v) return {};
    auto acc = post->var(2, 0);
    if (v == acc) return nps == 0 ? std::optional<int>(MIMK_POST_ID) : std::nullopt;
    auto is_zero = [](const Def* d) { auto l = Lit::isa<f32>(d); return l && *l == 0.f; };
    auto biased  = [&](const Def* d) {  // acc + b with b the single epilogue input
        auto add = Axm::isa(math::arith::add, d);
        if (!add || nps != 1) return false;
        auto [a, b] = add->args<2>();
        auto extra  = post->var(2, 1);
        return (a == acc && b == extra) || (a == extra && b == acc);
    };
    if (biased(v)) return MIMK_POST_BIAS;
    if (auto mx = Axm::isa(math::extrema::fmax, v)) {
        auto [a, b] = mx->args<2>();
        auto other  = is_zero(a) ? b : is_zero(b) ? a : nullptr;
        if (other && biased(other)) return MIMK_POST_BIAS_RELU;
        if (other == acc && nps == 0) return MIMK_POST_RELU;
    }
    if (auto th = Axm::isa(math::tri::tanh, v); th && biased(th->arg())) return MIMK_POST_BIAS_TANH;
    return {};
}

struct Gemm { nat_t m, n, k; bool b_is_nk; };

/// Ro = 2, Rn = 3, nis = 2: A read at (o0, o2); B at (o2, o1) [stored K,N] or at (o1, o2) [stored N,K, the
/// transposed read-through of fuse.cpp:542-589]; map_out the identity on (o0, o1).
std::optional<Gemm> match_gemm(World& w, const btensor::MapRedPost& mr, Defs out_dims, nat_t k_extent) {
    auto pa = as_projection(w, mr.maps->proj(2, 0), 3, 2);
    auto pb = as_projection(w, mr.maps->proj(2, 1), 3, 2);
    auto po = as_projection(w, mr.map_out, 3, 2);
    if (!pa || !pb || !po || (*po)[0] != 0 || (*po)[1] != 1) return {};
    if ((*pa)[0] != 0 || (*pa)[1] != 2) return {};
    bool kn = (*pb)[0] == 2 && (*pb)[1] == 1, nk = (*pb)[0] == 1 && (*pb)[1] == 2;
    if (!kn && !nk) return {};
    return Gemm{*Lit::isa<nat_t>(out_dims[0]), *Lit::isa<nat_t>(out_dims[1]), k_extent, nk};
}

/// The unset external continuation `mimk_<name>` (declared in patches/mimk.mim); the ll backend emits
/// `declare i32 @mimk_<name>(...)` and a direct call for an external Lam without a body (include/mim/plug/ll/ll.h:509-521,
/// lit/cps/ds_external_cimp.mim:13-20). `arg_types` are the scalar parameters between the memory token and the return
/// continuation `Cn [mem.M 0, I32]`.
Lam* launcher(World& w, std::string_view name, Defs arg_types) {
    if (auto ext = w.externals()[w.sym(name)]) return ext->as_mut<Lam>();
    DefVec dom;
    dom.push_back(w.call<mem::M>(0));
    dom.insert(dom.end(), arg_types.begin(), arg_types.end());
    dom.push_back(w.cn({w.call<mem::M>(0), w.type_i32()}));
    auto lam = w.mut_con(dom)->set(name);
    lam->externalize();  // no body: an import
    return lam;
}

/// A device pointer as the I64 the host side of the nvptx backend carries (src/mim/plug/nvptx/phase/nvptx.cpp:280-290).
const Def* as_i64(World& w, const Def* dptr) { return w.call<core::bitcast>(w.type_i64(), dptr); }
const Def* i64(World& w, u64 v) { return w.lit_i64(v); }
const Def* i32(World& w, u32 v) { return w.lit_i32(v); }

/// `call launcher (mem, args..., k)` with `k (mem, status) = mim_cu_check status; next mem`: the status of every launcher goes
/// where a CUresult goes (src/mim/plug/nvptx/rt/mim_cuda_rt.c:16-21).
const Def* call_launcher(World& w, Lam* launcher_lam, const Def* mem, Defs args, const Def* next /* Cn mem.M 0 */) {
    auto k = w.mut_con({w.call<mem::M>(0), w.type_i32()})->set("mimk_done");
    auto check = launcher(w, "mim_cu_check_cps", {w.type_i32()});  // the runtime's checker behind a CPS wrapper of the same shape
    auto after = w.mut_con({w.call<mem::M>(0), w.type_i32()})->set("mimk_checked");
    after->app(true, next, after->var(2, 0));
    k->app(true, check, {k->var(2, 0), k->var(2, 1), after});
    DefVec all;
    all.push_back(mem);
    all.insert(all.end(), args.begin(), args.end());
    all.push_back(k);
    return w.app(launcher_lam, all);
}

}  // namespace

const Def* LowerMapReduce::lower_map_reduce_post(const App* app) {
    auto& w = new_world();
    auto mr = btensor::MapRedPost::of(rewrite(app->callee())->as<App>());
    auto ranks = mr.ranks();
    if (!ranks) return Super::rewrite_imm_App(app);
    auto [nis, nps, ro, rr] = *ranks;

    auto comb = mr.comb->isa_mut<Lam>();
    auto post = mr.post->isa_mut<Lam>();
    if (!comb || !post) return Super::rewrite_imm_App(app);

    // literal output extents exactly as today (lower_map_reduce.cpp:331-346)
    Vector<nat_t> out_dims(ro);
    nat_t out_total = 1;
    for (nat_t d = 0; d != ro; ++d) {
        auto l = Lit::isa<nat_t>(mr.Sr->proj(ro + rr, d));
        if (!l) return Super::rewrite_imm_App(app);
        out_dims[d] = *l, out_total *= *l;
    }
    if (out_total == 0) return Super::rewrite_imm_App(app);

    // What today's body does around the kernel, unchanged (lower_map_reduce.cpp:351-365): splice a DS function, gpu.auto_init,
    // device copies of inputs and epilogue inputs, the output allocation.
    auto result_ty   = rewrite(app->type());
    auto [fun, call] = btensor::ds_splice(rewrite(app->arg()), result_ty, "mapReduceMimk");
    auto [fun_mem, host_buf, new_inputs, new_post_ins] = fun->var(2, 0)->projs<4>();
    auto cont                       = fun->var(2, 1);
    auto [h_mem, h_global, h_const] = w.app(w.annex<gpu::auto_init>(), fun_mem)->projs<3>();
    auto in_desc     = extract_input_desc(nis, mr.Ris, mr.Sis, mr.Tis, mr.maps);
    auto inputs      = alloc_copy_inputs(w, h_mem, h_global, in_desc.rs, in_desc.ss, in_desc.ts, new_inputs);
    auto post_desc   = extract_input_desc(nps, mr.Rps, mr.Sps, mr.Tps, mr.post_maps);
    auto post_inputs = alloc_copy_inputs(w, inputs.mem, inputs.global, post_desc.rs, post_desc.ss, post_desc.ts, new_post_ins);
    auto [out_global, out_dptr] = alloc_output(w, post_inputs.global, mr.Tp, mr.So);
    auto after = build_teardown(w, mr.Ro, mr.So, mr.Tp, inputs.dptrs, post_inputs.dptrs, out_dptr, host_buf, cont);
    // `after` expects (mem, global, const) like the continuation of gpu.launch; the launcher only threads the host memory
    auto resume = w.mut_con(w.call<mem::M>(0))->set("mimk_resume");
    resume->app(true, after, {resume->var(), out_global, h_const});
    auto null_stream = i64(w, 0);  // gpu.default_stream (src/mim/plug/gpu/gpu.mim:48-49)

    // 1. contraction (dot_general_fun over F32, optional epilogue): mimk_gemm_flat
    if (nis == 2 && ro == 2 && rr == 1 && is_f32(mr.To) && is_f32(mr.Tp) && is_mul_add(comb)) {
        auto pk  = post_kind(post, nps);
        auto k_l = Lit::isa<nat_t>(mr.Sr->proj(3, 2));
        auto g   = k_l ? match_gemm(w, mr, Defs{mr.Sr->proj(3, 0), mr.Sr->proj(3, 1)}, *k_l) : std::nullopt;
        // a bias is read at the last write coordinate only: post_maps#0 is the projection onto loop 1
        bool bias_ok = nps == 0;
        if (nps == 1)
            if (auto pp = as_projection(w, mr.post_maps->proj(1, 0), 2, 1)) bias_ok = (*pp)[0] == 1;
        if (pk && g && bias_ok) {
            auto gemm = launcher(w, "mimk_gemm_flat", {w.type_i64(), w.type_i64(), w.type_i64(), w.type_i64(), w.type_i64(), w.type_i64(),
                                                      w.type_i32(), w.type_i32(), w.type_i32(), w.type_i32(), w.type_i64(), w.type_i64()});
            auto bias = nps == 1 ? as_i64(w, post_inputs.dptrs[0]) : i64(w, 0);
            fun->set(true, call_launcher(w, gemm, post_inputs.mem,
                                         {i64(w, g->m), i64(w, g->n), i64(w, g->k), as_i64(w, inputs.dptrs[0]), as_i64(w, inputs.dptrs[1]),
                                          as_i64(w, out_dptr), i32(w, MIMK_F32), i32(w, MIMK_F32), i32(w, g->b_is_nk ? 1 : 0), i32(w, *pk),
                                          bias, null_stream},
                                         resume));
            return call;
        }
    }
    // 2. fold of one axis (pool_fun with add / fmax / fmin, identity epilogue): mimk_reduce. `reduce` reads its input with
    //    the folded loop last (tensor.mim:1155): the projection sends exactly one input axis to loop `ro`.
    if (nis == 1 && nps == 0 && rr == 1 && is_f32(mr.To) && is_f32(mr.Tp))
        if (auto monoid = pool_monoid(comb); monoid && returned_value(post) == post->var(2, 0)) {
            auto rank_in = Lit::isa<nat_t>(in_desc.rs[0]);
            auto pin     = rank_in ? as_projection(w, in_desc.maps[0], ro + 1, *rank_in) : std::nullopt;
            auto pout    = as_projection(w, mr.map_out, ro + 1, ro);
            bool ok      = pin && pout && *rank_in == ro + 1;
            nat_t ax     = 0;
            for (nat_t j = 0; ok && j != ro + 1; ++j)
                if ((*pin)[j] == ro) ax = j;
            for (nat_t j = 0; ok && j != ro + 1; ++j) ok = (*pin)[j] == (j < ax ? j : j == ax ? ro : j - 1);
            for (nat_t j = 0; ok && j != ro; ++j) ok = (*pout)[j] == j;
            auto len = Lit::isa<nat_t>(mr.Sr->proj(ro + 1, ro));
            if (ok && len) {
                nat_t outer = 1, inner = 1;
                for (nat_t d = 0; d != ro; ++d) (d < ax ? outer : inner) *= out_dims[d];
                auto red = launcher(w, "mimk_reduce", {w.type_i64(), w.type_i64(), w.type_i32(), w.type_i64(), w.type_i64(), w.type_i64(),
                                                       w.type_i32(), w.type_i64()});
                fun->set(true, call_launcher(w, red, post_inputs.mem,
                                             {as_i64(w, inputs.dptrs[0]), as_i64(w, out_dptr), i32(w, MIMK_F32), i64(w, outer), i64(w, *len),
                                              i64(w, inner), i32(w, *monoid), null_stream},
                                             resume));
                return call;
            }
        }
    // 2b. the same fold with an elementwise producer inlined into its combiner (produced_fold): mimk_reduce_fused takes the
    //     operator pair and the second input, placed as mimk_producer::y_mode says (its map is the fold's output loops ->
    //     y_mode 1, the input's own map -> 0, the input's axes from the folded one on -> 2); the projections are probed exactly
    //     as above. The call differs from case 2 only in the callee and in a `mimk_producer` built on the host stack.
    // 3. every other instance: one call of the generic launcher with the access maps flattened to coefficient matrices would go
    //    here (mimk_map_reduce_post takes a descriptor in memory; the maps' coefficients come from probing each map with unit
    //    markers and the zero vector, floordiv / rem results being read off the affine.semiop nodes). Until that emitter
    //    exists the generated kernel stays: today's body from `auto global_comb = ...` on.
    return lower_generated(app, mr, fun, call, inputs, post_inputs, out_global, out_dptr, h_const, after);  // today's body from `auto global_comb = ...` on
}

}  // namespace mim::plug::gpu::phase
