/* mimk.h -- C ABI of the B200 (sm_100a) kernel library behind MimIR's `tensor` plugin.
 *
 * Every entry point is what a lowered `tensor.*` / `btensor.map_reduce_post` call binds to once the
 * `gpu.lower_btensor_map_reduce` phase emits launcher calls instead of one-thread-per-cell NVPTX kernels.
 * The "replaces" notes give the reference interface (paths inside the MimIR project) each one stands in for.
 *
 * Conventions (from the reference's run-time ABI, lit/tensor/hlo_aux.cpp:19-23, lit/tensor/fc_aux.cpp:10-14):
 *   - a tensor is a bare pointer to a dense row-major buffer; shapes travel as int64_t;
 *   - unless a name contains `_host_`, every pointer is a DEVICE pointer valid on the current CUDA device and
 *     the call is asynchronous on `stream` (a cudaStream_t passed as void*; NULL = the default stream);
 *   - every call returns an int status (0 = ok) instead of aborting, so emitted code can pipe it to
 *     `mim_cu_check(int)` (src/mim/plug/nvptx/rt/mim_cuda_rt.c:16-21) exactly like a CUresult;
 *   - entry points that need scratch beyond their arguments (f32 contractions on the tensor cores, split-axis
 *     reductions, mimk_mlp_gated without `h`, composed attention, large scatters) take it from a cached buffer that belongs
 *     to the stream of the call: calls on different streams never share one (up to 8 streams per device keep a buffer;
 *     a ninth takes over the least recently used after a device-wide wait), calls on one stream are ordered by it;
 *   - nothing here falls back to the CPU: without a usable sm_100 device every compute call fails with
 *     MIMK_E_NO_DEVICE.
 */
#ifndef MIMK_H_
#define MIMK_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define MIMK_ABI_VERSION 2 /* 2: mimk_affine_map carries per-result floordiv / rem (div, mod) */

/* ---- element types (math.F32 / math.BF16, src/mim/plug/math/math.mim:26,34; I32/I64 of the core plugin) ---- */
enum { MIMK_F32 = 0, MIMK_BF16 = 1, MIMK_I32 = 2, MIMK_I64 = 3 };

/* ---- status codes ---- */
enum {
    MIMK_OK = 0,
    MIMK_E_ARG = 1,         /* null pointer, negative extent, unknown enum value */
    MIMK_E_SHAPE = 2,       /* extents inconsistent with each other */
    MIMK_E_ALIGN = 3,       /* a pointer or leading dimension misses the alignment the kernel needs */
    MIMK_E_DTYPE = 4,       /* this dtype combination has no kernel */
    MIMK_E_CUDA = 5,        /* a CUDA runtime/driver call failed; see mimk_last_cuda_error() */
    MIMK_E_NO_DEVICE = 6,   /* no CUDA device, or not compute capability 10.x */
    MIMK_E_DEVICE_WAIT = 7, /* a bounded wait inside a kernel expired (reported by mimk_device_status) */
    MIMK_E_UNSUPPORTED = 8, /* well-formed request outside what the kernels cover */
    MIMK_E_WORKSPACE = 9,   /* scratch buffer missing or too small */
};

/* Human-readable name of a status code. Never NULL. */
const char* mimk_status_str(int status);
/* MIMK_ABI_VERSION the library was built with (cf. Plugin::version, include/mim/plugin.h:159). */
int mimk_abi_version(void);
/* cudaError_t of the most recent failed CUDA call on this host thread (0 if none). */
int mimk_last_cuda_error(void);
/* MIMK_OK iff the current device can run the kernels (compute capability 10.x). */
int mimk_device_check(void);
/* Synchronises `stream` and returns MIMK_E_DEVICE_WAIT if any kernel since the last call gave up on a bounded
 * wait (its results are then undefined), MIMK_E_SHAPE if a gather / scatter met an index outside its axis (that
 * access was skipped), MIMK_OK otherwise. Clears the flag. */
int mimk_device_status(void* stream);

/* Launches a one-CTA kernel that waits, with a limit of `limit_cycles` SM clocks, on a barrier nothing arrives on, and
 * then reports exactly like the compute kernels: the status word is set and the kernel returns normally. After it,
 * mimk_device_status() must answer MIMK_E_DEVICE_WAIT and the context must still be usable. This is how the
 * failure path (cf. mim_cu_check, src/mim/plug/nvptx/rt/mim_cuda_rt.c:16-21) is tested without faulting a GPU. */
int mimk_selftest_wait_expiry(int64_t limit_cycles, void* stream);

/* ---- reduction monoids: the (g, init) pairs handed to `reduce` / `pool_fun`
 *      (src/mim/plug/tensor/tensor.mim:1139-1157): sum = (arith.add, 0), max = (extrema.fmax, -inf), ... ---- */
enum { MIMK_SUM = 0, MIMK_MAX = 1, MIMK_MIN = 2 };

/* ---- epilogues: what `fuse_tensor` sinks into the `post` slot of a reducing map_reduce_post
 *      (src/mim/plug/tensor/phase/fuse.cpp:408-534); `row` operands are epilogue inputs read at output
 *      coordinate 1 (a bias broadcast over rows), `full` operands at identity coordinates. ---- */
enum {
    MIMK_POST_ID = 0,
    MIMK_POST_BIAS = 1,      /* acc + row[n] */
    MIMK_POST_BIAS_RELU = 2, /* fmax(0, acc + row[n])            lit/tensor/fc_exec.mim:27-31 */
    MIMK_POST_BIAS_TANH = 3, /* tanh(acc + row[n])               lit/tensor/hlo_exec.mim */
    MIMK_POST_RELU = 4,      /* fmax(0, acc) */
    MIMK_POST_SILU = 5,      /* acc * slf(acc)                    math.slf, src/mim/plug/math/math.mim:283-284 */
    MIMK_POST_ADD_FULL = 6,  /* acc + full[m,n] */
};

/* ---- right-operand layouts of the dot family ---- */
enum {
    MIMK_B_KN = 0, /* B stored row-major [K,N]:  product_2d (a, b)                    tensor.mim:510-513 */
    MIMK_B_NK = 1, /* B stored row-major [N,K]:  product_2d (a, transpose_2d w), the read-through of
                      fuse.cpp:542-589 -- "column-major B" */
};

/* C[b,m,n] = post(sum_k A[b,m,k] * B[b,k,n]).
 * Replaces: tensor.product_2d / tensor.bmm / 2-D tensor.dot_product lowered through dot_product_impl
 * (src/mim/plug/tensor/tensor.mim:404-407, 480-486, 510-513, 1367-1423) and the kernel that
 * gpu::phase::LowerMapReduce::build_kernel generates for them (src/mim/plug/gpu/phase/lower_map_reduce.cpp:148-265).
 * in_dtype F32: f32-grade results -- small or oddly shaped problems fold each cell in ascending k on the CUDA cores,
 * larger ones run on the tensor cores as three TF32 products per term (head/tail split, about 21 mantissa bits per
 * product, f32 accumulation). in_dtype BF16: f32 accumulation on the tensor cores.
 * out_dtype F32 or BF16 (round to nearest even). batch strides are in elements; 0 re-uses the operand. */
typedef struct mimk_gemm_desc {
    int64_t batch, m, n, k;
    const void* a;
    const void* b;
    void* c;
    int64_t stride_a, stride_b, stride_c;
    int32_t in_dtype, out_dtype, b_layout, post;
    const void* post_row;  /* f32 [n], or NULL */
    const void* post_full; /* out_dtype [m,n] per batch, or NULL */
} mimk_gemm_desc;
int mimk_gemm(const mimk_gemm_desc* desc, void* stream);
/* The all-gather of a column-sharded contraction fused into its epilogue. Each GPU computes its column slab
 * C[:, col_off : col_off + n] and stores every tile directly into `n_dst` copies of the full [m, ldc] matrix -- its own
 * and its peers' (peer-mapped device pointers, e.g. from CUDA IPC or torch symmetric memory): stores over NVLink
 * (bulk stores from a shared-memory staging tile in the paired-SM kernel, 16-byte stores otherwise) while the tensor
 * cores work on the next tile, instead of a separate NCCL all-gather afterwards.
 * `b2` non-NULL selects the gated form, silu(A b) * (A b2) (bf16 out), as in mimk_mlp_gated's first stage.
 * The caller orders this call before the consumers of the gathered matrix on every GPU (a barrier across ranks after
 * the kernel has completed). No counterpart in the reference, which has no multi-device support
 * (src/mim/plug/nvptx/phase/nvptx.cpp:186-204). bf16 inputs only; batch must be 1; no full-shape epilogue operand. */
#define MIMK_MAX_GATHER 8
typedef struct mimk_gather_dst {
    int32_t n_dst;
    int32_t first; /* mimk_gemm_reduce_scatter: the destination whose rows this GPU computes first; 0 otherwise */
    void* dst[MIMK_MAX_GATHER];
    int64_t ldc, col_off; /* in elements */
} mimk_gather_dst;
int mimk_gemm_gather(const mimk_gemm_desc* desc, const void* b2, const mimk_gather_dst* dsts, void* stream);
/* A reduce-scatter fused into a contraction's epilogue: the counterpart of mimk_gemm_gather for a contraction whose K
 * dimension is sharded (every GPU holds a K-slab of A and the matching rows of B, so its product is a PARTIAL of the whole
 * [m, n] result). Row block t of the f32 result, rows [t rows_per_dst, (t + 1) rows_per_dst), is ADDED into dsts->dst[t],
 * an f32 [rows_per_dst, ldc] accumulator on the GPU that owns those rows (this GPU's or a peer-mapped pointer), at column
 * offset col_off: bulk reductions (cp.reduce.async.bulk.tensor, f32 add performed by the memory system at the
 * destination) from the shared-memory staging tile, over NVLink for a peer, while the tensor cores work on the next
 * tile -- no partial matrix is written to this GPU's memory and no separate collective follows.
 * The caller zeroes every accumulator and orders that before any GPU's call (a barrier across ranks), and orders every
 * GPU's call before the accumulators are read (another barrier). The order of the additions is not fixed, so the sum is
 * reproducible only up to f32 rounding. Every GPU should start at a different destination (dsts->first, e.g. the rank after
 * its own, so that its own rows come last): GPUs that walk the row blocks in the same order all send to one destination
 * at a time and share that GPU's inbound link. bf16 operands, f32 result, batch = 1, no epilogue, m = n_dst * rows_per_dst,
 * rows_per_dst a multiple of 32, ldc and col_off multiples of 4. No counterpart in the reference
 * (src/mim/plug/nvptx/phase/nvptx.cpp:186-204: one device). */
int mimk_gemm_reduce_scatter(const mimk_gemm_desc* desc, const mimk_gather_dst* dsts, int64_t rows_per_dst, void* stream);
/* mimk_gemm whose left operand arrives as `panels` row-major [m, k / panels] matrices stored one after another -- panel g
 * holds columns [g k/panels, (g+1) k/panels) of A. That is the layout an all-gather of column slabs delivers (every
 * rank's [m, k/panels] slab, in rank order), so the contraction that consumes a gathered matrix reads it where the
 * collective put it, with no transposing copy in between. bf16 operands, batch = 1, k / panels a multiple of 64.
 * No counterpart in the reference, which has no multi-device support (src/mim/plug/nvptx/phase/nvptx.cpp:186-204). */
int mimk_gemm_kpanels(const mimk_gemm_desc* desc, int64_t panels, void* stream);
/* The same call with scalar arguments only (batch = 1, no full-shape epilogue operand): emitted code can call it
 * without building a struct in memory -- an `extern con` with scalar parameters is all the binding needs
 * (lit/cps/ds_external_cimp.mim:13-20). */
int mimk_gemm_flat(int64_t m, int64_t n, int64_t k, const void* a, const void* b, void* c, int32_t in_dtype,
                   int32_t out_dtype, int32_t b_layout, int32_t post, const void* post_row, void* stream);

/* out[o,i] = fold_a g(x[o,a,i]) over the middle axis of a [outer, len, inner] view; inner == 1 is a row reduce.
 * Replaces: tensor.reduce (tensor.mim:1151-1157) lowered by gpu.lower_btensor_map_reduce. dtype F32 or BF16 (x and out;
 * accumulation in f32 either way). */
int mimk_reduce(const void* x, void* out, int dtype, int64_t outer, int64_t len, int64_t inner, int monoid,
                void* stream);

/* How many f32 partial results mimk_reduce / mimk_reduce_static keep for this problem on a device with `sm_count` SMs:
 * 0 when the reduced axis is not split (row reductions, or enough columns to fill the machine), else slices * outer *
 * inner. Pure host logic (needs no device): lets a caller of mimk_reduce_static see beforehand whether a plan fits
 * MIMK_REDUCE_STATIC_BYTES. No counterpart in the reference. */
int mimk_reduce_plan(int64_t outer, int64_t len, int64_t inner, int sm_count, int64_t* partial_floats);

/* mimk_reduce for callers that must not have the library allocate: the same arguments and, for F32 operands, the same
 * results bit for bit (one plan, the same kernels) -- F32 ONLY, a BF16 request returns MIMK_E_DTYPE -- but no
 * cudaMalloc / cudaFree / cudaHostAlloc is ever issued, on any call. (No counterpart in the reference, whose
 * generated wrappers allocate per operation.) Two kinds of caller need this: an embedder that plans all device
 * memory itself -- a fixed memory budget, or an allocator of its own that a hidden cudaMalloc would bypass -- and
 * a latency-critical loop that cannot take the device-wide synchronisation an allocation may imply.
 * Where mimk_reduce keeps the partial results of a split reduction in a cached allocation, this entry point keeps
 * them in a fixed 1 MiB array inside the library image (MIMK_REDUCE_STATIC_BYTES; every GPU that loads the library
 * holds it until the process exits). A call whose plan needs more partials than fit (mimk_reduce_plan tells) returns
 * MIMK_E_WORKSPACE and launches nothing; the plan grows with the SM count, and with the 148 SMs of a B200 no plan
 * exceeds 227 072 floats (0.87 MiB), so there the refusal cannot occur.
 * The first call on each device resolves the array's device address (with that device current) and reads two
 * device attributes; make that first call before any stream capture begins. All calls on a device share the one
 * array, so two calls whose kernels may overlap on the GPU (different streams, no dependency between them) race
 * on it: order them. Nothing needs zeroing between calls -- each call overwrites every partial it later reads. */
#define MIMK_REDUCE_STATIC_BYTES (1u << 20)
int mimk_reduce_static(const void* x, void* out, int dtype, int64_t outer, int64_t len, int64_t inner, int monoid,
                       void* stream);

/* An injective elementwise producer inlined into a consumer's operand read -- what tensor::phase::Fuse::fuse_map_reduce
 * does (src/mim/plug/tensor/phase/fuse.cpp:183-358, legality at :225-233): every element v the consumer reads becomes
 *   outer_op(inner_op(v, y[...]))
 * inner_op: a binary MIMK_OP_* with the second operand y placed by y_mode exactly as in mimk_map (0 same shape, 1
 * [outer, inner] broadcast along the consumer's folded axis, 2 [len*inner] broadcast over `outer`), or a unary one /
 * MIMK_OP_COPY (y unused, y_mode 3); outer_op: a unary MIMK_OP_* or MIMK_OP_COPY. y has the element type of x. */
typedef struct mimk_producer {
    int32_t inner_op, outer_op, y_mode, pad_;
    const void* y;
} mimk_producer;
/* mimk_reduce over produced values: out[o,i] = fold_a pre(x[o,a,i]) in one pass over x -- sum of squares, sum of
 * exp(x - max) (the softmax denominator), max |x|, sum of (x - mean)^2, a weighted row sum ... -- without the produced
 * tensor ever being written. The folds run on the same kernels as mimk_reduce (128-bit loads, split axis). dtype F32 or
 * BF16 (x, y, out); arithmetic in f32. */
int mimk_reduce_fused(const void* x, const mimk_producer* pre, void* out, int dtype, int64_t outer, int64_t len,
                      int64_t inner, int monoid, void* stream);

/* y = softmax(x) along the middle axis of a [outer, len, inner] view, in one pass over HBM.
 * Replaces: the four map_reduce_post ops the `softmax` lam expands to (tensor.mim:1172-1176).
 * x F32 (or BF16), y F32 or BF16; statistics in f32. */
int mimk_softmax(const void* x, void* y, int in_dtype, int out_dtype, int64_t outer, int64_t len, int64_t inner,
                 void* stream);

/* y[r,c] = x[r,c] * rrt(mean_c(x[r,:]^2) + eps) * gamma[c].
 * Replaces: the reduce + binary_ax + math.rrt chain (tensor.mim:1151-1167, math.mim:297-298). gamma F32. */
int mimk_rmsnorm(const void* x, const void* gamma, void* y, int in_dtype, int out_dtype, int64_t rows, int64_t cols,
                 float eps, void* stream);

/* y = rmsnorm(softmax_rows(x)) fused into one pass (the chained reading of "row softmax + RMSNorm"). */
int mimk_softmax_rmsnorm(const void* x, const void* gamma, void* y, int in_dtype, int out_dtype, int64_t rows,
                         int64_t cols, float eps, void* stream);

/* ---- elementwise: tensor.unary / tensor.binary / binary_ax (tensor.mim:361-394, 1162-1167) ---- */
enum {
    MIMK_OP_ADD = 0, MIMK_OP_SUB = 1, MIMK_OP_MUL = 2, MIMK_OP_DIV = 3, MIMK_OP_MAX = 4, MIMK_OP_MIN = 5,
    MIMK_OP_SUBEXP = 6, /* exp(x - y): the softmax producer, tensor.mim:1175 */
    /* unary (y operand ignored) */
    MIMK_OP_RELU = 16, MIMK_OP_TANH = 17, MIMK_OP_EXP = 18, MIMK_OP_SILU = 19, MIMK_OP_NEG = 20, MIMK_OP_COPY = 21,
    MIMK_OP_SQUARE = 22, MIMK_OP_ABS = 23,
    /* the rest of math.mim's unary operators over F that tensor programs apply elementwise: rt.sq (math.mim:147), rrt =
     * 1 / rt.sq (:297-298), exp.log / exp.exp2 / exp.log2 (:167-169), slf = 1 / (1 + exp(-x)) (:283-284) */
    MIMK_OP_SQRT = 24, MIMK_OP_RSQRT = 25, MIMK_OP_LOG = 26, MIMK_OP_EXP2 = 27, MIMK_OP_LOG2 = 28, MIMK_OP_SIGMOID = 29,
};
/* An elementwise operator with a unary one applied to its result -- outer(inner(x, y)): one more level of producer
 * inlining for elementwise consumers (relu(x + bias), tanh(x * y), |x - y| ...). inner: any MIMK_OP_*; outer: a unary one. */
#define MIMK_OP_COMPOSED_BASE 0x10000
#define MIMK_OP_COMPOSED(inner, outer) (MIMK_OP_COMPOSED_BASE | (inner) | ((outer) << 8))
/* out[o,a,i] = op(x[o,a,i], y[...]) over a [outer, len, inner] view of x (F32); op may be a MIMK_OP_COMPOSED pair.
 * y_mode 0: y has x's shape (tensor.binary); 1: y is [outer, inner], broadcast along the middle axis
 * (binary_ax); 2: y is [len*inner], broadcast over `outer` (a bias row); 3: unary, y unused. */
int mimk_map(int op, const void* x, const void* y, void* out, int out_dtype, int64_t outer, int64_t len,
             int64_t inner, int y_mode, void* stream);
/* The same with the operands' element type given: x and y F32 or BF16 (both of in_dtype), arithmetic in f32. */
int mimk_map_t(int op, const void* x, const void* y, void* out, int in_dtype, int out_dtype, int64_t outer, int64_t len,
               int64_t inner, int y_mode, void* stream);

/* ---- constructors and data-dependent indexing (tensor.mim:77-109, 519-563): not map_reduce_post instances ----
 * Shapes are `rank` extents (rank <= MIMK_MRP_MAX_RANK), tensors dense row-major.
 * mimk_splat: every element = the low bytes of value_bits (tensor.splat, tensor.mim:94-109); any element type.
 * mimk_generate_affine: out[o] = sum_d coef[d] * o[d] + coef[rank] in wrap-around int64, converted to I32 / I64 / F32:
 *   tensor.generate (tensor.mim:77-92) for bodies that are affine in the coordinates -- the coordinate tensors themselves
 *   (coef = unit vector) from which any other body can be computed with the elementwise operators.
 * mimk_gather: out[o] = input[o with o[dim] := index[o]], out has the index's shape (tensor.mim:519-541).
 * mimk_scatter: out = input, then out[u with u[dim] := index[u]] = updates[u] for every u of the index's shape in
 *   row-major order -- where two updates name one destination the later one wins (tensor.mim:543-563). out may alias
 *   input. Large index tensors use the library's cached scratch buffer (one int per element of input).
 * dtype: element type of input / updates / out (F32, BF16, I32, I64); index_dtype I32 or I64. The reference's index type
 * `Idx (s_src#dim)` cannot hold an out-of-range value; here such a value skips its access and mimk_device_status reports
 * MIMK_E_SHAPE. */
int mimk_splat(void* out, int dtype, int64_t n, int64_t value_bits, void* stream);
/* out[i] = cond[i] ? a[i] : b[i]: tensor.select (tensor.mim:378-384); cond holds one byte per element (non-zero = true). */
int mimk_select(const void* cond, const void* a, const void* b, void* out, int dtype, int64_t n, void* stream);
int mimk_generate_affine(void* out, int dtype, int rank, const int64_t* shape, const int64_t* coef, void* stream);
int mimk_gather(const void* input, const void* index, void* out, int dtype, int index_dtype, int rank, const int64_t* s_src,
                const int64_t* s_idx, int dim, void* stream);
int mimk_scatter(const void* input, const void* index, const void* updates, void* out, int dtype, int index_dtype, int rank,
                 const int64_t* s_src, const int64_t* s_idx, const int64_t* s_updates, int dim, void* stream);

/* O[h,i,:] = softmax_j(scale * Q[h,i,:].K[h,j,:] (+ causal mask j <= i + seq_k - seq_q)) V[h,j,:].
 * Replaces: the composed program `softmax (q * transpose_2d k) * v` (lit/tensor/attn_exec.mim:20-22), seven
 * map_reduce_post ops with a materialised score matrix; scale, mask and batching are extensions.
 * q,o: [batch_heads, seq_q, head_dim]; k,v: [batch_heads, seq_k, head_dim]; dtype F32 or BF16 (o same dtype);
 * bf16 with head_dim 64 or 128 runs fused on the tensor cores; f32, and bf16 with other head dims, from 2^24
 * score-products on run as the composition S = Q K^T, softmax, O = P V on the contraction and row kernels (the score
 * matrix lives in a cached library buffer; not when lse is requested); everything else on a warp-per-query CUDA-core kernel;
 * lse (optional, f32 [batch_heads, seq_q]) receives log-sum-exp of the scaled scores. */
typedef struct mimk_attn_desc {
    int64_t batch_heads, seq_q, seq_k, head_dim;
    const void* q;
    const void* k;
    const void* v;
    void* o;
    float* lse;
    float scale;
    int32_t causal, dtype;
} mimk_attn_desc;
int mimk_attn_fwd(const mimk_attn_desc* desc, void* stream);

/* Y = (silu(X W1) * (X W3)) W2 with the gated product H kept in `dtype`.
 * Replaces: two product_2d + math.slf + binary mul (epilogue-fused into one contraction) + product_2d.
 * x [m,k]; w1,w3 [k,f] (b_layout KN) or [f,k] (NK); w2 [f,n] (KN) or [n,f] (NK); y [m,n].
 * h is scratch for the [m,f] intermediate (dtype elements); NULL lets the library use its own cached buffer. */
typedef struct mimk_mlp_desc {
    int64_t m, k, f, n;
    const void* x;
    const void* w1;
    const void* w3;
    const void* w2;
    void* y;
    void* h;
    int32_t dtype, b_layout;
} mimk_mlp_desc;
int mimk_mlp_gated(const mimk_mlp_desc* desc, void* stream);

/* ---- the generic operation ------------------------------------------------------------------------------
 * out[map_out(o)] = post(fold_r f(acc, (in_i[maps_i(o, r)])_i), (post_in_j[post_maps_j(map_out(o))])_j)
 * over the loop vector (o..., r...) with bounds `sr`: the leading `ro` loops are the output loops, the trailing
 * `rn - ro` loops are folded, ascending, per output cell (classic nest order).
 * Replaces: btensor.map_reduce_post itself (src/mim/plug/btensor/btensor.mim:102-115; decoder struct MapRedPost,
 * include/mim/plug/btensor/btensor.h:20-52) for every instance the specialised entry points above do not take --
 * strip-mined / interchanged domains, packed outputs, transposes, slices, broadcasts, convolutions, mixed element
 * types. One thread per output cell walks its reduction, like the kernel gpu::phase::LowerMapReduce::build_kernel
 * generates (src/mim/plug/gpu/phase/lower_map_reduce.cpp:148-265), but with the access maps as data.
 * An access map is a matrix: result j = sum_l coef[j][l] * loop[l] + coef[j][n_loops], in wrap-around int64
 * (include/mim/plug/affine/phase/lower_index.h:14-20), optionally followed per result by a floor division and a
 * remainder -- result j = (linear_j floordiv div[j]) rem mod[j], each applied when > 0, unsigned like the reference's
 * lowering of affine.semiop.floordiv / rem to core.div (lower_index.h:22-27). That is the form affine.delinearize takes
 * (src/mim/plug/affine/affine.mim:103-108), hence `reshape_map` (src/mim/plug/tensor/tensor.mim:1224-1233), the unpack
 * copy behind a packed dot_product (tensor.mim:1405-1411), and what fuse_read_through composes behind a consumer's map
 * when it absorbs a reshape (src/mim/plug/tensor/phase/fuse.cpp:542-589). Buffers are row-major. Every access is
 * bounds-checked on the host against the loop bounds before launch (MIMK_E_SHAPE), so a wrong map never reads outside a
 * buffer; a map with div / mod must have a linear part that cannot go negative. */
#define MIMK_MRP_MAX_LOOPS 8
#define MIMK_MRP_MAX_RANK 6
#define MIMK_MRP_MAX_INPUTS 4
enum { /* combiners f(acc, ins) */
    MIMK_F_ADD = 0,     /* acc + a                      pool_fun add          */
    MIMK_F_MULADD = 1,  /* acc + a * b                  dot_general_fun, tensor.mim:1332 */
    MIMK_F_MAX = 2, MIMK_F_MIN = 3,
    MIMK_F_FIRST = 4,   /* a (acc ignored): copy-style ops, tensor_copy, tensor.mim:1074 */
    MIMK_F_SUBEXP = 5,  /* exp(a - b)  */
    MIMK_F_DIV = 6, MIMK_F_ADD2 = 7, MIMK_F_MUL2 = 8, /* a / b, a + b, a * b (acc ignored): binary / binary_ax */
    MIMK_F_MIX = 9,     /* acc + a + (acc type)b         lit/btensor/map_reduce_post.mim:17-18 */
    /* combiners with an injective producer inlined, as fuse_map_reduce leaves them (src/mim/plug/tensor/phase/fuse.cpp:183-358;
       softmax after fusion, fuse.cpp:225-245): */
    MIMK_F_ADD_SUBEXP = 10, /* acc + exp(a - b)              the sum fold of softmax with exp(x - max) inlined */
    MIMK_F_SUBEXP_DIV = 11, /* exp(a - b) / c (acc ignored)  the divide with the exponential recomputed; three inputs */
};
/* The general form of a combiner with an inlined producer: f(acc, a [, b]) = fold(acc, outer(inner(a, b))) with
 * fold one of MIMK_F_ADD / MAX / MIN / FIRST, inner a binary MIMK_OP_* over the two inputs (a, b) or a unary one /
 * MIMK_OP_COPY over the single input, outer a unary MIMK_OP_* or MIMK_OP_COPY. Floating-point accumulators only.
 * MIMK_F_ADD_SUBEXP is MIMK_F_COMPOSED(MIMK_F_ADD, MIMK_OP_SUBEXP, MIMK_OP_COPY). When the maps spell a fold along one
 * axis with the second input broadcast as mimk_producer allows, the instance runs on mimk_reduce_fused. */
#define MIMK_F_COMPOSED_BASE 0x01000000
#define MIMK_F_COMPOSED(fold, inner, outer) (MIMK_F_COMPOSED_BASE | (fold) | ((inner) << 8) | ((outer) << 16))
enum { /* epilogues post(acc, post_ins) */
    MIMK_P_ID = 0,
    MIMK_P_ADD = 1,       /* widen(acc) + p0 (unsigned widening when the output type is wider)  map_reduce_post.mim:19-20 */
    MIMK_P_ADD_PLUS1 = 2, /* acc + p0 + 1                                                 lit/buffer/exec_epilogue.mim:33 */
    MIMK_P_ADD_RELU = 3,  /* fmax(0, acc + p0) */
    MIMK_P_ADD_TANH = 4,  /* tanh(acc + p0) */
    MIMK_P_RELU = 5, MIMK_P_SILU = 6,
};
typedef struct mimk_affine_map {
    int32_t rows; /* number of results (the rank of the tensor it indexes) */
    int32_t pad_;
    int64_t coef[MIMK_MRP_MAX_RANK][MIMK_MRP_MAX_LOOPS + 1];
    int64_t div[MIMK_MRP_MAX_RANK]; /* > 0: the linear form of result j is floor-divided by it; 0: not */
    int64_t mod[MIMK_MRP_MAX_RANK]; /* > 0: then reduced modulo it; 0: not */
} mimk_affine_map;
typedef struct mimk_mrp_desc {
    int32_t ro, rn;                   /* output loops, all loops (rn >= ro) */
    int64_t sr[MIMK_MRP_MAX_LOOPS];   /* loop bounds */
    int64_t so[MIMK_MRP_MAX_RANK];    /* shape of the result (rank ro) */
    int32_t nis, nps;                 /* inputs, epilogue inputs */
    const void* in[MIMK_MRP_MAX_INPUTS];
    int32_t in_dtype[MIMK_MRP_MAX_INPUTS];
    int64_t in_shape[MIMK_MRP_MAX_INPUTS][MIMK_MRP_MAX_RANK];
    mimk_affine_map in_map[MIMK_MRP_MAX_INPUTS];   /* over the rn loop variables */
    const void* post_in[MIMK_MRP_MAX_INPUTS];
    int32_t post_dtype[MIMK_MRP_MAX_INPUTS];
    int64_t post_shape[MIMK_MRP_MAX_INPUTS][MIMK_MRP_MAX_RANK];
    mimk_affine_map post_map[MIMK_MRP_MAX_INPUTS]; /* over the ro write coordinates */
    mimk_affine_map map_out;                       /* over the rn loop variables (reduction slots read 0) */
    int32_t comb, post;
    int32_t acc_dtype, out_dtype;     /* F32, I32 or I64 accumulators; out additionally BF16 */
    int64_t init_bits;                /* the accumulator's initial value, as raw bits (low bytes) */
    void* out;
} mimk_mrp_desc;
int mimk_map_reduce_post(const mimk_mrp_desc* desc, void* stream);

/* Which kernel family mimk_map_reduce_post runs a descriptor on. Large floating-point instances whose access maps
 * spell a contraction over dense matrices (tensor.mim:1381-1396; right operand [K,N] or its transposed read-through
 * [N,K]; optional batch loop; id / relu / silu / bias / full-addend epilogue), a fold of one axis with (add, 0),
 * (fmax, -inf) or (fmin, +inf) (tensor.mim:1151-1157), or an elementwise unary / binary / binary_ax instance
 * (tensor.mim:361-394, 1162-1167) are handed to mimk_gemm, mimk_reduce and mimk_map. These fold in another order than
 * the ascending per-cell fold, which is why integer instances and instances with fewer than 2^20 combiner
 * applications always stay on the per-cell kernel. A copy that permutes axes (tensor.transpose, tensor.mim:1443-1468;
 * any element type, 2^20 elements or more) runs as a tiled copy through shared memory; a copy through `reshape_map`
 * of a whole tensor (tensor.reshape, tensor.mim:1224-1241) moves no element and is one device-to-device copy, at any size.
 * MIMK_MRP_ROUTE=0 in the environment keeps every instance on the per-cell kernel.
 * Pure host logic: needs no device. No counterpart in the reference, whose GPU lowering has the one kernel shape. */
enum { MIMK_ROUTE_GENERIC = 0, MIMK_ROUTE_GEMM = 1, MIMK_ROUTE_REDUCE = 2, MIMK_ROUTE_MAP = 3, MIMK_ROUTE_PERMUTE = 4, MIMK_ROUTE_COPY = 5 };
int mimk_mrp_classify(const mimk_mrp_desc* desc);
/* Which per-cell kernel an instance that stays on MIMK_ROUTE_GENERIC runs on -- all three keep the reference's kernel shape
 * (one thread per output cell, the reduction loops folded in order: lower_map_reduce.cpp:198-260) and give the same bits:
 *   INTERPRETED  maps, combiner and epilogue read as data; the only one that takes floordiv / rem in an input map
 *   LINEAR       every input's offset one linear form of the loop vector, the reduction box walked like an odometer
 *   COMPILED     the linear forms in straight-line code with the combiner fixed at compile time: floating-point instances
 *                with one element type throughout, no epilogue operand, fewer than 2^31 cells, and -- after loops of extent
 *                1 are dropped and neighbours merged where every operand's form allows it (n and c of an NCHW pool become
 *                one loop) -- at most 6 output and 3 reduction loops. `loops`, if not NULL, receives those two counts.
 * conv / conv_grouped / pool / pad / strided copies of tensor.mim:434-451, 499-504 land on COMPILED. Pure host logic. */
enum { MIMK_CELL_INTERPRETED = 0, MIMK_CELL_LINEAR = 1, MIMK_CELL_COMPILED = 2 };
int mimk_mrp_cell_kernel(const mimk_mrp_desc* desc, int32_t* loops);

/* ---- programs: a list of map_reduce_post operations -----------------------------------------------------------
 * `ops` are executed in order; an input (or epilogue input) whose pointer equals the `out` of an earlier operation reads
 * that operation's result. Chains that spell a known composition run as ONE fused kernel instead of op by op:
 *   softmax     max-fold, exp(x - max), sum-fold, divide along one axis (the `softmax` lam, tensor.mim:1172-1176), also in
 *               the three-operation form fuse_tensor leaves (the exponential inlined into the sum fold and recomputed in
 *               the divide, fuse.cpp:225-245)                                            -> mimk_softmax, one pass over x
 *   attention   S = q k^T (k read through transpose_2d), softmax of S along its last axis, O = P v
 *               (lit/tensor/attn_exec.mim:20-22), with or without a leading batch loop   -> mimk_attn_fwd, scale 1, no mask
 * A chain is fused only when its temporaries (every result inside it but the last) feed nothing outside it in `ops`; they are
 * then never written. Everything else runs through mimk_map_reduce_post. These are the recognisers the compiler-side lowering
 * needs once it emits launcher calls per operation; no counterpart in the reference, whose GPU lowering handles one operation
 * at a time (src/mim/plug/gpu/phase/lower_map_reduce.cpp:317-395).
 * mimk_program_classify is pure host logic (needs no device): steps[i] says how operation i runs. */
enum {
    MIMK_STEP_OP = 0,        /* by itself, through mimk_map_reduce_post */
    MIMK_STEP_SOFTMAX = 1,   /* first operation of a softmax chain: the chain runs as mimk_softmax */
    MIMK_STEP_ATTENTION = 2, /* first operation of an attention chain: the chain runs as mimk_attn_fwd */
    MIMK_STEP_ABSORBED = 3,  /* a later operation of a fused chain */
    MIMK_STEP_FOLD_OF_MAP = 4, /* an elementwise map whose only reader is the fold after it: the pair runs as
                                  mimk_reduce_fused and the produced tensor is never written (fuse.cpp:183-358) */
};
int mimk_program_classify(const mimk_mrp_desc* ops, int32_t n_ops, int32_t* steps);
int mimk_program_run(const mimk_mrp_desc* ops, int32_t n_ops, void* stream);

/* ---- matrix-chain association ------------------------------------------------------------------------------
 * In which order to multiply the chain A0 . A1 . ... . A(n-1), matrix i being dims[i] x dims[i+1]; transposed[i] != 0
 * marks a leaf that is stored [dims[i+1], dims[i]] and read through transpose_2d (NULL: none is).
 * Replaces: the decision of the tensor.reassoc phase (src/mim/plug/tensor/phase/reassoc.cpp:89-128 cost of one
 * product, 172-206 the dynamic program, 287-313 the run-time tournament for extents unknown at compile time) -- taken
 * here when the chain is about to run, with every extent known.
 * model MIMK_COST_LANES: the reference's price list, vector-lane slots of its CPU schedules; param = vector width
 * (its `-X tensor:vec-width`, default 8). model MIMK_COST_B200: estimated seconds on one B200 (whole output tiles in
 * whole waves over 148 SMs against HBM time, plus a launch; a transposed leaf on the left pays a copy); param = the
 * element type, MIMK_F32 or MIMK_BF16.
 * mimk_chain_order writes the n-1 products of the cheapest bracketing in an order in which they can be executed (each
 * one multiplies the results of sub-chains i..s and s+1..j); equal costs keep the lowest split. Under MIMK_COST_B200 a
 * sub-chain may also be built transposed when that saves a copy; under MIMK_COST_LANES every node is plain, as in the
 * phase. mimk_chain_cost prices the products it is given (every sub-chain they use must be among them), e.g. the
 * chain as written, so that a caller can keep that on a tie as the phase does (reassoc.cpp:349-351).
 * Pure host logic: needs no device. */
#define MIMK_CHAIN_MAX 64
enum { MIMK_COST_LANES = 0, MIMK_COST_B200 = 1 };
typedef struct mimk_chain_split {
    int32_t i, s, j; /* multiply sub-chain i..s by sub-chain s+1..j */
    int32_t t;       /* != 0: store the product transposed, i.e. compute (s+1..j)^T . (i..s)^T (reassoc.cpp:224-231) */
} mimk_chain_split;
int mimk_chain_order(int32_t n, const int64_t* dims, const int32_t* transposed, int32_t model, int32_t param,
                     mimk_chain_split* splits, double* cost);
int mimk_chain_cost(int32_t n, const int64_t* dims, const int32_t* transposed, int32_t model, int32_t param,
                    const mimk_chain_split* splits, int32_t n_splits, double* cost);

/* ---- host-buffer forms -------------------------------------------------------------------------------
 * Same operators with HOST pointers: inputs are copied to the device, the kernel runs, the result is copied
 * back and the call returns when the result is in host memory.
 * Replaces: the per-operation wrapper gpu.lower_btensor_map_reduce emits around its kernel -- gpu.buf_alloc_copy
 * for every input and epilogue input, gpu.alloc.block for the output, gpu.launch, gpu.buf_copy_to_host, gpu.free
 * (src/mim/plug/gpu/phase/lower_map_reduce.cpp:111-126, 267-297, 317-395), i.e. the run-time ABI
 * `extern "C" T* f(T* in0, ...)` of an emitted tensor function (lit/tensor/hlo_aux.cpp:19-23).
 * Differences in mechanism only: device buffers come from a cached per-device arena instead of cuMemAlloc/cuMemFree
 * per call, copies are asynchronous on private streams, and row-wise operators stream the matrix through the device
 * in row blocks so that upload, kernel and download overlap. Copies run at full speed only from page-locked host
 * memory (mimk_host_register or any cudaHostAlloc/cudaHostRegister'd buffer); pageable memory works but is slower. */
enum { MIMK_ROWS_SOFTMAX = 0, MIMK_ROWS_RMSNORM = 1, MIMK_ROWS_SOFTMAX_RMSNORM = 2 };
int mimk_host_rows(int kind, const void* x, const void* gamma, void* y, int in_dtype, int out_dtype, int64_t rows,
                   int64_t cols, float eps);
/* softmax(x) and rmsnorm(x) of the same matrix from ONE upload of x: two consumers of one tensor, which the reference's
 * per-operation wrappers would upload twice (lower_map_reduce.cpp:111-122 runs once per operation). */
int mimk_host_rows_pair(const void* x, const void* gamma, void* y_softmax, void* y_rmsnorm, int in_dtype, int out_dtype,
                        int64_t rows, int64_t cols, float eps);
/* desc holds host pointers (a, b, c, post_row, post_full). */
int mimk_host_gemm(const mimk_gemm_desc* desc);
/* desc holds host pointers (q, k, v, o, lse). */
int mimk_host_attn_fwd(const mimk_attn_desc* desc);
/* desc holds host pointers (x, w1, w3, w2, y); h is ignored. */
int mimk_host_mlp_gated(const mimk_mlp_desc* desc);
/* mimk_map_reduce_post with HOST operands: every input and epilogue input is uploaded, the result comes back in
 * desc->out -- the per-operation wrapper of the reference for ANY map_reduce_post instance
 * (src/mim/plug/gpu/phase/lower_map_reduce.cpp:111-126, 267-297, 317-395). Cells the write map never stores keep the
 * bytes the caller's buffer held. */
int mimk_host_map_reduce_post(const mimk_mrp_desc* desc);
/* Page-lock / unlock a host range so that the copies above are asynchronous DMA. */
int mimk_host_register(void* ptr, uint64_t bytes);
int mimk_host_unregister(void* ptr);
/* Release the cached device arena of the current device (it is otherwise kept until process exit). */
int mimk_host_release(void);

#ifdef __cplusplus
}
#endif
#endif /* MIMK_H_ */
