// UNVERIFIED SKETCH -- not compiled anywhere (see patches/README.md).
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

/// A map `«Rn; Index» -> «r; Index»` is a projection iff applying it to the unit loop vectors yields unit coordinate
/// vectors: the probing trick of tensor::normalize_fastest_axis (src/mim/plug/tensor/normalizers.cpp:189-217).
/// Returns the loop id each result reads, or nullopt.
std::optional<Vector<nat_t>> as_projection(World& w, const Def* map, nat_t n_loops, nat_t rank);

/// `f` is `acc, (a, b) -> R.add(acc, R.mul(a, b))` for a math.F32 (or BF16 -> F32) ring: dot_general_fun,
/// src/mim/plug/tensor/tensor.mim:1332.
bool is_mul_add(const Lam* comb);
/// `f` is pool_fun g (tensor.mim:1139) with g one of math.arith.add / math.extrema.fmax / fmin; yields MIMK_SUM/MAX/MIN.
std::optional<int> pool_monoid(const Lam* comb);
/// post is btensor.id, or `acc, b -> acc + b`, relu / tanh of that (fuse_epilogue's output, fuse.cpp:408-534);
/// yields MIMK_POST_*.
std::optional<int> post_kind(const Lam* post, nat_t nps);

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
/// `declare i32 @mimk_<name>(...)` and a direct call for it (include/mim/plug/ll/ll.h:509-521).
Lam* launcher(World& w, std::string_view name, Defs arg_types);

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

    // ... literal output extents exactly as today (lower_map_reduce.cpp:331-346) ...

    // 1. contraction
    if (nis == 2 && ro == 2 && rr == 1 && is_mul_add(comb)) {
        if (auto pk = post_kind(post, nps)) {
            // g = match_gemm(...); splice the DS function, gpu.auto_init, alloc_copy_inputs (A, B, bias), alloc_output
            // as today; then, instead of build_kernel + gpu.launch:
            //   call mimk_gemm_flat(m, n, k, dA, dB, dC, F32, F32, g->b_is_nk, *pk, dBias, /*stream*/ 0)
            //   pipe the I32 result into mim_cu_check; continue with build_teardown(...) unchanged.
        }
    }
    // 2. reduce along one axis: nis == 1, rr == 1, projection map moving the reduced axis last (tensor.mim:1155)
    if (nis == 1 && rr == 1)
        if (auto monoid = pool_monoid(comb)) {
            // (outer, len, inner) from the position of the reduced axis in the input's shape;
            //   call mimk_reduce(dX, dOut, F32, outer, len, inner, *monoid, 0)
        }
    // 3. elementwise: rr == 0, combiner ignores acc (binary_ax's app_mr, tensor.mim:1164): mimk_map
    // 4. anything else: the generated kernel, unchanged
    return lower_generated(app, mr);  // today's body from `auto global_comb = ...` on
}

}  // namespace mim::plug::gpu::phase
