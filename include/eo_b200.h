/*
 * C ABI of libeo_b200.so: hand-written sm_100a kernels for the Newton-Schulz orthogonalization
 * path of the Muon / OrthogonalizedOptimizer step.
 *
 * Conventions shared by every entry point:
 *   - plain pointers and sizes only; device pointers unless a name says `host_`;
 *   - `stream` is a cudaStream_t passed as void* (NULL = the legacy default stream); work is only
 *     enqueued, nothing synchronises the stream;
 *   - the return value is an eo_status; on failure eo_last_error() describes it (thread-local);
 *   - matrices are row-major with a leading dimension `ld*` counted in elements and a batch
 *     stride counted in elements; bf16 operands must have 16-byte-aligned base pointers and
 *     ld / stride multiples of 8 elements (fp32: 4), which is what a TMA descriptor needs;
 *   - no entry point allocates or frees device memory: callers own inputs, outputs and scratch.
 *
 * Citations name the file:line of the reference (NVIDIA-NeMo/Emerging-Optimizers) call site that
 * an entry point stands in for.
 */
#ifndef EO_B200_H_
#define EO_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum eo_status {
  EO_OK = 0,
  EO_ERR_BAD_ARG = 1,       /* shape / alignment / flag rejected before any launch */
  EO_ERR_CUDA = 2,          /* a CUDA runtime or driver call failed */
  EO_ERR_UNSUPPORTED = 3,   /* device is not compute capability 10.x */
  EO_ERR_WORKSPACE = 4,     /* scratch buffer too small */
  EO_ERR_DEVICE_WAIT = 5    /* a bounded wait inside a kernel ran out (see eo_read_device_status) */
} eo_status;

/* Library / build identification: "eo_b200 <version> sm_100a". */
const char* eo_version(void);

/* Message of the last failure on the calling thread ("" if none). */
const char* eo_last_error(void);

/*
 * Tuning knobs (process-wide).  "gemm_tile_m": 0 (default) lets each launch choose between 128-row tiles and
 * 256-row tiles (two MMAs per k-step sharing one B tile: fewer operand bytes per FLOP, used for large problems
 * with long K); 128 or 256 forces one.  Results do not depend on the choice.  "gemm_pair" (default 1): plain bf16
 * products with 256 x 256 tiles run on CTA pairs (tcgen05 cta_group::2); same bits as with 0.  "gemm_split_k"
 * (default 1): the pair kernel may cut the K range of the tiles of a launch's last, nearly empty round into pieces
 * whose fp32 partial sums are added in a fixed order; which tiles are cut depends on M, N, K and the triangular
 * flag only (never on the batch size), results are deterministic and differ from "gemm_split_k" 0 by the rounding
 * of those partial sums.  The partial sums live in a per-stream workspace that the library allocates on first use
 * and keeps; a call that would have to grow it during stream capture fails with EO_ERR_UNSUPPORTED.
 * "gemm_pair_group_m" (default 8), "gemm_pair_band" (default 8), "gemm_pair_hint_a", "gemm_pair_hint_b" (default
 * 0): tile order and L2 eviction policies of the pair kernel; results do not depend on them.  "peer_wait_ms"
 * (default 10000): how long a kernel waits for a flag that another rank has to raise before it gives up;
 * "tp_lower_only" (default 1): see eo_tp_gram_allreduce.
 */
int eo_set_option(const char* name, int value);

/*
 * Host-only: the work-item schedule the CTA-pair kernel would follow for a plain bf16 product of `batch` matrices
 * M x N x K (`tri`: lower-triangular SYRK, M == N) on a GPU with `sm_count` SMs, under the current options.  Uses
 * the launcher's own planning code and the kernel's own index decoding, compiled for the host; no device is
 * touched.  Writes the number of work items to *n_items and, if `out` is not NULL (room for `capacity` items of
 * six ints), per item: matrix, tile row, tile column (256 x 256 tiles), first k-block, one past the last k-block
 * (64-element blocks), and the index of the split tile the item is a K piece of (-1: a whole tile).  For tests of
 * the index arithmetic; nothing in the product calls it.
 */
int eo_debug_pair_schedule(int M, int N, int K, int tri, int batch, int sm_count, int* out, int64_t capacity,
                           int64_t* n_items);

/*
 * Reads and clears the status word that kernels of this library write when one of their bounded
 * waits (mbarrier, accumulator hand-off, peer flag) runs out.  Synchronises `stream` first.
 * *host_code receives 0 when every kernel completed normally.
 */
int eo_read_device_status(uint32_t* host_code, void* stream);

/*
 * General tensor-core product with a fused affine epilogue, fp32 accumulation:
 *
 *     D[b] = alpha * op(A[b]) * op(B[b])^T + beta * C[b],     b = 0 .. batch-1
 *
 * op(A) is M x K and op(B) is N x K.  `a_mn_major == 0`: A is stored M x K row-major (K
 * contiguous, leading dimension lda); `a_mn_major == 1`: A is stored K x M row-major (M
 * contiguous).  Same for B with N.  C and D are M x N row-major.
 *
 * `precision`: 0 = bf16 operands (A, B, C bf16; planeA / planeB ignored);
 *              1 = fp32-accurate product of split operands: A and B each point to three bf16 planes
 *                  (see eo_split_f32) `planeA` / `planeB` elements apart, all with the layout given by
 *                  lda / strideA (ldb / strideB); the six plane products p_i * q_j with i + j <= 2 are
 *                  accumulated in fp32.  C and D are fp32.
 * `d_fp32`   : D is fp32 (1) or bf16 (0; only with precision 0).
 * `round_bf16`: with d_fp32, round alpha*acc + beta*C to bf16 first, then widen and multiply by
 *               post_scale (keeps the rounding point of a bf16 kernel followed by `.to(float32) * s`).
 * C may be NULL when beta == 0.
 *
 * Stands in for torch.addmm / torch.baddbmm at
 * emerging_optimizers/orthogonalized_optimizers/muon_utils.py:374-377, 407-410, 439-441, 473-475,
 * and for the trailing `.to(torch.float32)` (:269) and scale multiply
 * (emerging_optimizers/orthogonalized_optimizers/muon.py:132) when d_fp32 is set.
 */
int eo_gemm(const void* A, int a_mn_major, int64_t lda, int64_t strideA, int64_t planeA,
            const void* B, int b_mn_major, int64_t ldb, int64_t strideB, int64_t planeB,
            const void* C, int64_t ldc, int64_t strideC,
            void* D, int64_t ldd, int64_t strideD,
            int batch, int M, int N, int K,
            float alpha, float beta, float post_scale,
            int precision, int d_fp32, int round_bf16, void* stream);

/*
 * Symmetric rank-k update, lower triangle computed and mirrored:
 *
 *     D[b] = alpha * A[b] * A[b]^T + beta * C[b],     A[b] is N x K,  C[b], D[b] are N x N
 *
 * `a_trans == 0`: A stored N x K row-major; `a_trans == 1`: A stored K x N row-major (i.e. the
 * caller's A is a transposed view of a contiguous K x N array).  C must be symmetric; only its
 * lower triangle is read.  `skip_upper != 0` leaves the strict upper triangle of D untouched.
 * `precision` as in eo_gemm (0: bf16 in/out; 1: A given as three bf16 planes `planeA` elements apart,
 * C and D fp32).
 *
 * Stands in for tsyrk_ex / tsyrk_ex_small_matrix (emerging_optimizers/triton_kernels/syrk.py:335-500)
 * and batched_tsyrk_ex (emerging_optimizers/triton_kernels/batched_syrk.py:266-363).
 */
int eo_syrk(const void* A, int a_trans, int64_t lda, int64_t strideA, int64_t planeA,
            const void* C, int64_t ldc, int64_t strideC,
            void* D, int64_t ldd, int64_t strideD,
            int batch, int N, int K, float alpha, float beta, int skip_upper,
            int precision, void* stream);

/*
 * Split an fp32 matrix batch into three bf16 planes with x = p0 + p1 + p2 (to 2^-24 relative):
 * p0 = bf16(x), p1 = bf16(x - p0), p2 = bf16(x - p0 - p1).  Plane i is written at
 * planes + i * plane_stride (elements), each with leading dimension ldo and batch stride strideo.
 * Feeds the precision-1 mode of eo_gemm / eo_syrk, which stands in for the fp32 ("highest" / "high")
 * matmuls of muon_utils.py:370-377 when torch.get_float32_matmul_precision() is not "medium" (:245).
 */
int eo_split_f32(const float* x, int batch, int64_t rows, int64_t cols, int64_t ld, int64_t stride,
                 void* planes, int64_t ldo, int64_t strideo, int64_t plane_stride, void* stream);

/*
 * Bytes of scratch eo_sumsq_f32 needs for `batch` matrices of rows x cols.
 */
size_t eo_sumsq_scratch_bytes(int batch, int64_t rows, int64_t cols);

/*
 * sumsq[b] = sum over the rows x cols fp32 matrix b of x^2, accumulated in float64 in a fixed
 * order (run-to-run deterministic).  `sumsq` is double[batch] on the device; `scratch` must hold
 * eo_sumsq_scratch_bytes(...) bytes.
 *
 * First half of torch.nn.functional.normalize / torch.linalg.vector_norm at
 * emerging_optimizers/orthogonalized_optimizers/muon_utils.py:216, 221 and of
 * distributed_normalize_p2 (:140-141); a tensor-parallel caller all-reduces `sumsq` between this
 * call and eo_normalize_f32.
 */
int eo_sumsq_f32(const float* x, int batch, int64_t rows, int64_t cols, int64_t ld, int64_t stride,
                 double* sumsq, void* scratch, size_t scratch_bytes, void* stream);

/*
 * Same result as eo_sumsq_f32, bit for bit, for callers that cannot hand over device scratch.
 * (No counterpart in the reference; added for this library's embedders.)
 *
 * Who needs it: code that runs where device allocation is off the table - inside a framework's
 * allocator callback or memory-pool trim hook, in a hot loop that has promised its owner a fixed
 * memory footprint, or in a host that only receives raw device pointers from another runtime and has
 * no allocator of its own to ask for a scratch buffer.  For them the per-block partial sums live in an
 * array compiled into the library image (65536 doubles = 512 KiB, held by every GPU that loads the
 * library until the process exits).  The call itself makes no cudaMalloc / cudaFree and calls no
 * allocating routine.
 *
 * Limits and rules:
 *   - batch * blocks_per_matrix must not exceed eo_sumsq_noalloc_max_partials() (a matrix uses
 *     ceil(rows * cols / 32768) blocks, at most 1024); larger requests fail with EO_ERR_WORKSPACE and
 *     launch nothing - use eo_sumsq_f32 for those;
 *   - the array is shared by every call on a device and keeps whatever the last call left; nothing
 *     needs clearing because each call overwrites every slot it later reads, but two calls whose
 *     kernels may overlap on one GPU (different streams, different threads) race on it: serialise them;
 *   - the first call of any entry point of this library on a device resolves the array's device
 *     address (and does the other one-time set-up); make that first call outside stream capture.
 */
int eo_sumsq_f32_noalloc(const float* x, int batch, int64_t rows, int64_t cols, int64_t ld, int64_t stride,
                         double* sumsq, void* stream);

/* Capacity of the built-in scratch of eo_sumsq_f32_noalloc, in partial sums (doubles). */
size_t eo_sumsq_noalloc_max_partials(void);

/*
 * out[b] = x[b] / denom[b],  denom[b] = (float)sqrt(sumsq[b]), clamped from below by eps when
 * `clamp_eps` is set.  Output is bf16 (out_fp32 == 0) or fp32; with out_fp32 and round_bf16 the
 * quotient is rounded to bf16 and widened again.
 *
 * Second half of the normalisation at muon_utils.py:143-146, 216, 222 fused with the bf16
 * down-cast at :262.
 */
int eo_normalize_f32(const float* x, int batch, int64_t rows, int64_t cols, int64_t ld, int64_t stride,
                     const double* sumsq, float eps, int clamp_eps,
                     void* out, int64_t ldo, int64_t strideo, int out_fp32, int round_bf16, void* stream);

/*
 * First half of a deferred Frobenius normalisation: ONE pass over the fp32 batch writes it rounded to bf16,
 * un-normalised (out_bf16, leading dimension ldo, batch stride strideo), and accumulates the sum of squares of the
 * fp32 values as eo_sumsq_f32 does; scales[2 b] = 1 / max(norm_b, eps)^2 and scales[2 b + 1] = 1 / max(norm_b, eps)
 * (fp32, on the device) are what eo_newton_schulz_bf16 takes as `dev_scales`.  sumsq may be NULL.  Scratch as for
 * eo_sumsq_f32.  Saves one of the two reads of the input that "sum of squares, then divide and narrow" needs.
 *
 * Stands in for the norm and the division of
 * emerging_optimizers/orthogonalized_optimizers/muon_utils.py:216 together with the bf16 cast of :262.
 */
int eo_cast_sumsq_f32(const float* x, int batch, int64_t rows, int64_t cols, int64_t ld, int64_t stride,
                      void* out_bf16, int64_t ldo, int64_t strideo, float eps, double* sumsq, float* scales,
                      void* scratch, size_t scratch_bytes, void* stream);

/*
 * Elementwise parts of one Muon step on a flat, contiguous, 16-byte-aligned fp32 parameter of `numel`
 * elements.  With g' = g + l2_weight_decay * p, lerp(a, b, w) as torch.lerp computes it:
 *
 *   eo_muon_momentum_f32 : m <- lerp(m, g', 1 - momentum) in place;
 *                          sumsq[0] = sum u^2 (float64, fixed order), u = nesterov ? lerp(g', m, momentum) : m
 *   eo_muon_normalize_bf16: out = bf16(u / max((float)sqrt(sumsq[0]), eps)), u recomputed from g, p and the
 *                          updated m (so u itself never goes to memory)
 *   eo_muon_apply_f32    : p <- (p + shrink * p) - lr * ((update * scale) * extra_scale)
 *
 * `momentum` is a double so that 1 - momentum is rounded to fp32 once, as the weight of torch.lerp_ is.
 * `scratch` of eo_muon_momentum_f32 must hold eo_muon_scratch_bytes(numel) bytes.  `p` may be NULL when
 * l2_weight_decay == 0.  `update` is bf16 (update_is_bf16 != 0) or fp32.
 *
 * Stand in for emerging_optimizers/orthogonalized_optimizers/orthogonalized_optimizer.py:185-199 (weight
 * decay on the gradient, `lerp_`, Nesterov `lerp`), muon_utils.py:216, 262 (normalise, bf16 cast), and
 * mixin.py:44-52 + muon.py:131-132 + orthogonalized_optimizer.py:208 (parameter shrink, scale, `p.add_`).
 */
size_t eo_muon_scratch_bytes(int64_t numel);
int eo_muon_momentum_f32(const float* g, float* m, const float* p, int64_t numel, double momentum, int nesterov,
                         float l2_weight_decay, double* sumsq, void* scratch, size_t scratch_bytes, void* stream);
int eo_muon_normalize_bf16(const float* g, const float* m, const float* p, int64_t numel, double momentum,
                           int nesterov, float l2_weight_decay, const double* sumsq, float eps, void* out,
                           void* stream);
int eo_muon_apply_f32(float* p, const void* update, int update_is_bf16, int64_t numel, float shrink, float scale,
                      float extra_scale, float lr, void* stream);

/*
 * Multi-tensor forms of the three calls above for a group of parameters (host arrays of device
 * pointers; the tables travel in kernel parameters, nothing is copied to the device).
 *
 *   eo_muon_prepare_batch: for n tensors of the same `numel`: momentum update, sum of squares
 *       (sumsq[i], device double[n]) and the normalised bf16 tensor written to
 *       out_stack + i * slot_stride - the stacked (n, rows, cols) input of a batched Newton-Schulz run.
 *       `p` may be NULL when l2_weight_decay == 0.  scratch: eo_muon_prepare_scratch_bytes(n, numel).
 *       With `dev_scales` (device float[2 n]) the normalisation is deferred: out_stack receives bf16(u), not
 *       divided, in the same single pass that updates the momentum (g and m are read once instead of twice), and
 *       dev_scales[2 i], dev_scales[2 i + 1] = 1 / max(norm_i, eps)^2, 1 / max(norm_i, eps) are handed to
 *       eo_newton_schulz_bf16, which applies them in its first two epilogues.  NULL keeps the two-pass form.
 *   eo_muon_apply_batch  : weight update of n tensors of any sizes; update[i] is bf16 or fp32 for all i.
 *       max_blocks_per_tensor > 0 caps the grid (blocks of 256 threads per tensor) so that an update running
 *       beside tensor-core kernels on another stream takes only a slice of the SMs and of HBM bandwidth;
 *       0 sizes the grid for full bandwidth.
 *
 * Results are bit-identical to the single-tensor calls.
 */
size_t eo_muon_prepare_scratch_bytes(int n, int64_t numel);
int eo_muon_prepare_batch(int n, const float* const* g, float* const* m, const float* const* p, int64_t numel,
                          double momentum, int nesterov, float l2_weight_decay, float eps, void* out_stack,
                          int64_t slot_stride, double* sumsq, float* dev_scales, void* scratch, size_t scratch_bytes,
                          void* stream);
int eo_muon_apply_batch(int n, float* const* p, const void* const* update, int update_is_bf16, const int64_t* numel,
                        const float* scale, float shrink, float extra_scale, float lr, int max_blocks_per_tensor,
                        void* stream);

/*
 * The whole iteration loop of newton_schulz on the bf16 path in one call:
 *
 *     for (a, b, c) in host_abc[0 .. steps):  A = X X^T;  S = b A + c A A  (skipped if c == 0);
 *                                             X <- a X + S X   (a X + b A X if c == 0)
 *
 * X is the normalised bf16 iterate, (batch, rows, cols) row-major with leading dimension `ld` and batch
 * stride `stride` (multiples of 8, 16-byte-aligned base); the iteration runs on the wide orientation
 * (on X^T, without copying, when rows > cols).  The last step writes `out` (bf16, or fp32 = bf16-rounded
 * values widened, with ldo / strideo); X is used as a ping-pong buffer and is clobbered when steps > 1.
 * `flags`: bit 0 selects the lower-triangular kernel for A and S (falls back to the general kernel when rows
 * or cols is not a multiple of 8); bit 1 disables the fused small-matrix kernel.  That kernel is used for
 * batches of wide matrices with rows <= 128 (per-head / split-QKV blocks, cols >= 256, steps <= 16): one
 * persistent kernel runs every iteration of a matrix with A, A^2 and S kept in shared memory; the first
 * iteration reads the iterate twice, every iteration reads it once (its new value feeds the next Gram matrix
 * while still in shared memory) and writes it once.  `host_abc` is a host array of 3 * steps floats.
 * `workspace`: eo_newton_schulz_workspace_bytes(batch, rows, cols) bytes, 256-byte aligned.
 * `dev_scales`: NULL when X is already normalised.  Otherwise X is the un-normalised bf16 image written by
 * eo_cast_sumsq_f32 and dev_scales its per-matrix factors: the first Gram epilogue multiplies by 1 / norm^2, the
 * first update epilogue by 1 / norm (in the small-matrix kernel too), so the Frobenius normalisation costs no
 * pass of its own.  The first iterate is then rounded to bf16 before instead of after the division.
 *
 * Stands in for the step loop of emerging_optimizers/orthogonalized_optimizers/muon_utils.py:265-269 with
 * the step functions of :348-476; launches 3 * steps (2 * steps when c == 0) kernels, or one.
 */
size_t eo_newton_schulz_workspace_bytes(int batch, int rows, int cols);
int eo_newton_schulz_bf16(void* X, int batch, int rows, int cols, int64_t ld, int64_t stride, const float* host_abc,
                          int steps, int flags, void* out, int out_fp32, int64_t ldo, int64_t strideo, void* workspace,
                          size_t workspace_bytes, const float* dev_scales, void* stream);

/*
 * The same loop for the fp32 ("highest" / "high") path: `steps` iterations on a normalised fp32 iterate X (batch x
 * rows x cols, row-major, ld / stride in elements; the Gram matrix is taken over the shorter side), every product
 * computed on three bf16 planes per operand (see eo_split_f32) with fp32 accumulation, A, S and the iterate kept
 * in fp32.  X is not modified; the result goes to `out` (ldo / strideo in elements), which also serves as a
 * ping-pong buffer.  Per iteration: split X, A (lower-triangular kernel), split A, S (likewise; skipped when
 * c == 0), split S, X' -- the same kernels in the same order as the per-step entry points, driven from one call
 * so that the host cost of about thirty launches is paid in C rather than in the caller's interpreter.
 * A single matrix (batch == 1) whose Gram matrix has too few tiles for the SMs gets its A product sliced along
 * the contraction dimension (2, 4 or 8 slices as batches of one launch, fp32 partial matrices in the workspace,
 * summed in a fixed order by the pass that splits A); results then differ from the per-step entry points by fp32
 * summation order only.
 * `workspace`: eo_newton_schulz_f32_workspace_bytes(batch, rows, cols) bytes, 256-byte aligned.
 *
 * Stands in for the step loop of emerging_optimizers/orthogonalized_optimizers/muon_utils.py:265-269 when
 * torch.get_float32_matmul_precision() is not "medium" (:245-262 select the fp32 step functions).
 */
size_t eo_newton_schulz_f32_workspace_bytes(int batch, int rows, int cols);
int eo_newton_schulz_f32(const float* X, int batch, int rows, int cols, int64_t ld, int64_t stride,
                         const float* host_abc, int steps, float* out, int64_t ldo, int64_t strideo, void* workspace,
                         size_t workspace_bytes, void* stream);

/*
 * Tensor-parallel Gram matrix: SYRK and all-reduce in ONE kernel (one NVSwitch box, 2..8 ranks).
 *
 * Every rank holds a shard X_r (N x K_r, bf16; `x_trans` as `a_trans` of eo_syrk) of a matrix sharded along
 * the contraction dimension, and all ranks make this call.  The kernel computes the partial Gram X_r X_r^T tile by
 * tile (lower-triangle tiles only).  The epilogue of tile t writes the bf16 partial into the rank's own partial
 * buffer and publishes `seq` in a flag word of the tile's owner (rank t mod world).  Reducer warps of the same
 * CTAs serve the tiles this rank owns: they wait for the `world` flags of a tile (bounded by the option
 * "peer_wait_ms", default 10 s; on expiry the device status word is set and the tile is filled with NaN on every
 * rank, so that a failed exchange cannot pass for a result), sum the partials in fp32 with one rounding - one
 * NVSwitch load-reduce per 16 bytes when the multicast aliases are given, plain loads from every peer otherwise -
 * and store the tile and its mirror image into the Gram matrix of every rank (multicast stores, or one store per
 * peer).  The exchange of a tile overlaps the main loop of the following tiles.
 *
 * partial_ptrs / flag_ptrs / gram_ptrs: host arrays of `world` device pointers, entry r addressing rank r's
 * buffer (peer-mapped, e.g. symmetric memory): partial tiles of eo_tp_gram_inbox_bytes(N, world) bytes, flags of
 * eo_tp_gram_flag_count(N, world) uint32 (zeroed once at creation), Gram matrix N x ld_gram bf16.
 * partials_multicast / gram_multicast: multicast (NVLS) addresses mapping all ranks' partial buffers / Gram
 * matrices, or both NULL.  `seq` must increase by one with every call on the same buffers (first call: 1).
 * After the call and a barrier across the ranks (which orders the owners' stores before the readers, and every
 * rank's reads of the partial buffers before the next call overwrites them) every rank's Gram matrix holds the
 * full symmetric sum - or, with the option "tp_lower_only" (default 1), its lower triangle, which every rank
 * completes on its own copy with eo_tp_gram_mirror: the reducers then read and store whole tile rows (512
 * contiguous bytes per warp) and half as many bytes cross NVLink.
 *
 * Stands in for tsyrk_ex + torch.distributed.all_reduce at
 * emerging_optimizers/orthogonalized_optimizers/muon_utils.py:434-436 (and :370-372).
 */
size_t eo_tp_gram_inbox_bytes(int N, int world);
size_t eo_tp_gram_flag_count(int N, int world);
int eo_tp_gram_allreduce(const void* X, int x_trans, int64_t ldx, int N, int K, int world, int rank,
                         void* const* partial_ptrs, void* const* flag_ptrs, void* const* gram_ptrs,
                         const void* partials_multicast, void* gram_multicast, int64_t ld_gram, uint32_t seq,
                         void* stream);

/* Copies the strict lower triangle of the N x N bf16 matrix `gram` (leading dimension ld_gram) onto its upper one. */
int eo_tp_gram_mirror(void* gram, int N, int64_t ld_gram, void* stream);

/*
 * Copies `bytes` bytes (a multiple of 16, both pointers 16-byte aligned) from local memory through a multicast
 * (NVLS) address: the data lands at the same offset in the buffer of every rank the address maps.  The
 * tensor-parallel iteration uses it to all-gather the row blocks of S = b A + c A^2 (each rank copies its block;
 * 512 contiguous bytes per warp).  The caller orders readers behind a barrier across the ranks.
 * Stands in for the all-gather a sharded torch.addmm (muon_utils.py:374) needs; no call site in the reference.
 */
int eo_multicast_copy(const void* src, void* dst_multicast, size_t bytes, void* stream);

/*
 * General bf16 product D = alpha * op(A) op(B)^T + beta * C (single matrix, conventions of eo_gemm) whose result
 * is stored through a multicast (NVLS) address: every element lands in the buffer of every rank mapped by
 * `D_multicast`.  With each rank computing a block of rows of one matrix this is "product + all-gather" in one
 * kernel; the tensor-parallel iteration uses it for S = b A + c A^2 (a rank's row block costs 2 N^3 / world FLOP
 * instead of N^3 for the redundant symmetric product).  N must be a multiple of 32, rows 16-byte aligned; C is
 * read from local memory.  The caller orders readers behind a barrier across the ranks.
 *
 * Stands in for torch.addmm at emerging_optimizers/orthogonalized_optimizers/muon_utils.py:374 under
 * tensor parallelism (:277-345), where the reference computes S redundantly on every rank.
 */
int eo_gemm_multicast(const void* A, int a_mn_major, int64_t lda, const void* B, int b_mn_major, int64_t ldb,
                      const void* C, int64_t ldc, void* D_multicast, int64_t ldd, int M, int N, int K, float alpha,
                      float beta, void* stream);

/*
 * Enqueues a copy of the device status word (see eo_read_device_status) into `pinned_host_code` on `stream`
 * without synchronising and without clearing it: a caller polls the host word later, e.g. at its next call.
 */
int eo_peek_device_status_async(uint32_t* pinned_host_code, void* stream);

#ifdef __cplusplus
}
#endif

#endif /* EO_B200_H_ */
