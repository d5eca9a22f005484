/*
 * flagblas_b200 -- C ABI of the B200 (sm_100a) GEMM back end.
 *
 * Plain pointers and sizes only: every entry point can be bound from C, ctypes,
 * pybind11 or cgo without any tensor library.  All matrices are ROW-MAJOR with
 * `ld*` = row stride in elements, exactly as in the reference's Python
 * operators.  Every function returns 0 (FB_OK) or a negative FB_ERR_* code; none
 * throws, aborts or synchronises the device.  Work is enqueued on `stream`
 * (a cudaStream_t passed as void*; NULL = the legacy default stream) of the
 * CUDA device that is current on the calling thread.
 *
 * Each declaration cites the reference interface it stands in for, by the
 * reference project's own paths.
 */
#ifndef FLAGBLAS_B200_H_
#define FLAGBLAS_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ---- status codes ------------------------------------------------------- */
enum {
  FB_OK = 0,
  FB_ERR_INVALID_ARG = -1,   /* bad enum, negative size, ld too small, NULL pointer */
  FB_ERR_WORKSPACE = -2,     /* workspace missing or smaller than fb_*_workspace_bytes() */
  FB_ERR_LAUNCH = -3,        /* CUDA reported an error at launch (see fb_last_cuda_error) */
  FB_ERR_UNSUPPORTED = -4,   /* device is not sm_100, or size beyond 2^31-1 */
  FB_ERR_DRIVER = -5,        /* tensor-map encoder unavailable / rejected the arguments */
  FB_ERR_TOO_LARGE = -6      /* request exceeds a fixed capacity (see the entry point) */
};

/* ---- element / arithmetic types ----------------------------------------- */
enum {
  FB_F32 = 0,   /* fp32 storage, IEEE FFMA on the CUDA cores          (sgemm)     */
  FB_TF32 = 1,  /* fp32 storage, TF32 tensor-core multiply, fp32 acc  (tf32gemm)  */
  FB_F16 = 2,   /* fp16 storage, fp32 accumulate, one rounding        (hgemm)     */
  FB_BF16 = 3   /* bf16 storage, fp32 accumulate, one rounding        (bfgemm)    */
};

/* transposition flags: same numeric values as the reference's
 * CUBLAS_OP_N / CUBLAS_OP_T (src/flag_blas/ops/level3/sgemm.py:30-32). */
enum { FB_OP_N = 0, FB_OP_T = 1 };

/*
 * Dense GEMM:  C[m,n] <- alpha * op(A) * op(B) + beta * C      (in place on C)
 *
 *   transa = N: A stored [m, lda>=k];   transa = T: A stored [k, lda>=m]
 *   transb = N: B stored [k, ldb>=n];   transb = T: B stored [n, ldb>=k]
 *   C stored [m, ldc>=n].  C is never read when beta == 0.
 *   m == 0 or n == 0: nothing is done.  k == 0 or alpha == 0: the m x n block
 *   of C is scaled by beta.
 *
 * Replaces the bodies of
 *   sgemm   src/flag_blas/ops/level3/sgemm.py:421-477
 *           (+ src/flag_blas/runtime/backend/_nvidia/hopper/ops/sgemm.py:1512-1662)
 *   hgemm   src/flag_blas/ops/level3/hgemm.py:473-529
 *           (+ .../hopper/ops/hgemm.py:2279-2422)
 *   bfgemm  src/flag_blas/ops/level3/bfgemm.py:473-529
 *           (+ .../hopper/ops/bfgemm.py:1048-1268)
 * and provides the dense TF32 flavour the reference only has in grouped form
 * (src/flag_blas/ops/level3/group_gemm.py:427-581).
 *
 * Tensor-core types need A and B with 16-byte aligned base and row pitch to be
 * fetched in place; otherwise the operand is first packed into `workspace`
 * (size from fb_gemm_workspace_bytes, 256-byte aligned device memory).  FB_F32
 * never needs a workspace.
 */
int fb_gemm(int dtype, int transa, int transb, int64_t m, int64_t n, int64_t k, float alpha, const void* A,
            int64_t lda, const void* B, int64_t ldb, float beta, void* C, int64_t ldc, void* workspace,
            size_t workspace_bytes, void* stream);

/* Bytes of workspace fb_gemm asks for with these arguments (0 when none): packed copies of operands that cannot be
 * fetched in place (required), plus optional scratch for fp32 partial sums (a split of a long k range, the
 * stream-K tail of a half-empty last wave of tiles); without the optional part the call runs unsplit.
 * A call that uses the stream-K part has CTAs that wait (bounded, about a second) for other CTAs of the same
 * launch; it never launches more CTAs than the device can hold, and whatever precedes it on its stream finishes
 * without it.  Two such calls must not share the SMs (each could hold a part and wait for CTAs that cannot start;
 * the waits would run out and both end with device status 107), so a stream-K call that follows one made through
 * this library on another stream of the device first waits for everything submitted to that stream so far.
 * Streams under graph capture are not ordered this way: a caller that captures large GEMMs on several streams of
 * one graph passes only the required part of the workspace (or sets FLAGBLAS_B200_STREAMK=0) and gets whole tiles. */
size_t fb_gemm_workspace_bytes(int dtype, int transa, int transb, int64_t m, int64_t n, int64_t k, const void* A,
                               int64_t lda, const void* B, int64_t ldb);

/* Element types of fb_gemm_ex (the GEMMs outside the tensor-core path). */
enum { FB_F64 = 4, FB_C64 = 5, FB_C128 = 6 };
/* Conjugate transpose, accepted by fb_gemm_ex for the complex types
 * (CUBLAS_OP_C, src/flag_blas/ops/level3/cgemm.py:59-60). */
enum { FB_OP_C = 2 };

/*
 * Dense GEMM in double, complex<float> or complex<double>, on the CUDA cores (IEEE FMAs in the
 * operand's own precision):   C[m,n] <- alpha * op(A) * op(B) + beta * C,   op = N, T (or C, complex only).
 * Same layout rules and early-outs as fb_gemm.  alpha and beta point to HOST memory: {re, im}
 * (im ignored for FB_F64).  Complex matrices are interleaved (re, im) pairs; ld* count complex elements.
 * Replaces the bodies of
 *   dgemm  src/flag_blas/ops/level3/dgemm.py:160-208
 *   cgemm  src/flag_blas/ops/level3/cgemm.py:192-254
 *   zgemm  src/flag_blas/ops/level3/zgemm.py:192-254
 * Never needs a workspace.
 */
int fb_gemm_ex(int dtype, int transa, int transb, int64_t m, int64_t n, int64_t k, const double* alpha, const void* A,
               int64_t lda, const void* B, int64_t ldb, const double* beta, void* C, int64_t ldc, void* stream);

/*
 * Triangular matrix product, out of place (the reference's row-major strmm / dtrmm / ctrmm / ztrmm):
 *     side = 0 (left):   C[m,n] <- alpha * op(tri(A))[m,m] * B[m,n]
 *     side = 1 (right):  C[m,n] <- alpha * B[m,n] * op(tri(A))[n,n]
 *   A row-major [k, lda >= k] (k = m or n); only its lower (uplo = 0: col <= row) or upper (uplo = 1)
 *   triangle is read; diag = 1 reads the diagonal as 1; trans = N, T (or C for the complex types).
 *   dtype FB_F32 / FB_F64 / FB_C64 / FB_C128; alpha = host {re, im}.  alpha == 0 zero-fills the m x n block of C.
 *   B and C must not overlap (the Python wrappers copy B first when they do).
 * Replaces the bodies of strmm / dtrmm / ctrmm / ztrmm, src/flag_blas/ops/level3/trmm.py:2095-2231,
 * 2234-2329, 3161-3292, 4743-4939 (generic kernel :39-196).
 */
int fb_trmm(int dtype, int side, int uplo, int trans, int diag, int64_t m, int64_t n, const double* alpha, const void* A,
            int64_t lda, const void* B, int64_t ldb, void* C, int64_t ldc, void* stream);

/*
 * Matrix-vector product (the one-column limit of the GEMM path):
 *     trans = N:  y[m] <- alpha * A * x[n]   + beta * y
 *     trans = T:  y[n] <- alpha * A^T * x[m] + beta * y
 *   A stored [m, lda>=n] row-major; x and y strided by incx, incy > 0 (elements).
 *   dtype FB_F32 / FB_F16 / FB_BF16: storage type of A, x and y; products and sums in fp32,
 *   alpha * acc + beta * y formed in fp32 and rounded once.  y is not read when beta == 0.
 *   m == 0 or n == 0: nothing is done.  alpha == 0: the len_y strided elements of y are
 *   scaled by beta (zero-filled when beta == 0) and A, x are not touched.
 * Replaces the bodies of
 *   sgemv   src/flag_blas/ops/level2/gemv.py:2285-2375
 *   hgemv   src/flag_blas/ops/level2/gemv.py:2814-2926
 *   bfgemv  src/flag_blas/ops/level2/gemv.py:2929-3041
 * Shapes with few output elements per SM split the reduced dimension; they need
 * fb_gemv_workspace_bytes(...) bytes of 16-byte aligned device scratch (0 otherwise).  The
 * additions happen in a fixed order: results are reproducible from run to run.
 */
int fb_gemv(int dtype, int trans, int64_t m, int64_t n, float alpha, const void* A, int64_t lda, const void* x,
            int64_t incx, float beta, void* y, int64_t incy, void* workspace, size_t workspace_bytes, void* stream);

size_t fb_gemv_workspace_bytes(int dtype, int trans, int64_t m, int64_t n);

/* 8-bit floating-point storage formats of fb_gemv_fp8 (OCP FP8; e4m3 = torch.float8_e4m3fn). */
enum { FB_FP8_E4M3 = 0, FB_FP8_E5M2 = 1 };

/*
 * Matrix-vector product with an FP8 matrix and an FP8 vector, transposed form only:
 *     y[n] <- alpha * A^T * x[m] + beta * y
 *   A stored [m, lda>=n] row-major in `a_format`, x in `x_format` (strided by incx), y of type
 *   y_dtype = FB_F32 / FB_F16 / FB_BF16 (strided by incy); every product and sum in fp32, one rounding.
 *   Early-outs as fb_gemv.  16-byte aligned A and lda use 16-byte loads, anything else works too.
 * Replaces the body of fp8_gemv, src/flag_blas/ops/level2/gemv.py:3044-3124 (kernels :2158-2282).
 * Scratch: fb_gemv_fp8_workspace_bytes(m, n) bytes, 16-byte aligned, when the rows are split.
 */
int fb_gemv_fp8(int a_format, int x_format, int y_dtype, int64_t m, int64_t n, float alpha, const void* A, int64_t lda,
                const void* x, int64_t incx, float beta, void* y, int64_t incy, void* workspace,
                size_t workspace_bytes, void* stream);

size_t fb_gemv_fp8_workspace_bytes(int64_t m, int64_t n);

/*
 * Grouped GEMM:  for g in [0, group_count):
 *     out_g[m_g,n_g] <- alpha * A_g[m_g,k_g] * B_g + beta * C_g
 *
 * Every array argument is DEVICE memory and is only read on the device:
 *   d_a/d_b/d_c/d_out : int64 addresses of A_g, B_g, C_g, out_g
 *   d_m/d_n/d_k       : int32 sizes;   d_lda/d_ldb/d_ldc : int32 row strides
 *   (out_g and C_g share d_ldc, as in the reference).
 *   b_k_contiguous = 0: B_g stored [k_g, ldb>=n_g]  (group_bfgemm / group_hgemm)
 *   b_k_contiguous = 1: B_g stored [n_g, ldb>=k_g]  (group_tf32gemm)
 * Any base address and any row pitch work, as in the reference (block pointers with
 * boundary checks, src/flag_blas/ops/level3/group_gemm.py:162-185): an A_g / B_g whose base
 * and pitch are 16-byte aligned is fetched by TMA, any other by the kernel's producer warps
 * with ordinary loads (slower, same results).  Only an address or pitch that is not even a
 * multiple of the element size is refused: that group is skipped and fb_device_status()
 * reports 201 (the arrays live on the device, so the host cannot check them at the call).
 * Groups with m_g == 0 or n_g == 0 produce no work.
 *
 * Replaces group_bfgemm / group_hgemm / group_tf32gemm,
 *   src/flag_blas/ops/level3/group_gemm.py:221-262, 380-421, 540-581
 *   (+ src/flag_blas/runtime/backend/_nvidia/hopper/ops/group_gemm.py:699-891).
 * dtype is FB_BF16, FB_F16 or FB_TF32.  m_hint / n_hint / k_hint are the
 * reference's M, N, K arguments (total rows of all groups, columns, depth):
 * host-side hints that only steer the tile plan, 0 = unknown.  A call whose
 * m_hint says the groups average at most 64 rows (m_hint <= 64 * group_count:
 * the reference's use_small_m case) takes a plan built for groups of a few
 * rows; results do not depend on the hints.  `workspace` holds the device-built
 * tile table and tensor maps: fb_group_workspace_bytes(group_count) bytes,
 * 256-byte aligned; it may be reused by the next call on the same stream.
 */
int fb_group_gemm(int dtype, int b_k_contiguous, const int64_t* d_a, const int64_t* d_b, const int64_t* d_c,
                  const int64_t* d_out, const int32_t* d_m, const int32_t* d_n, const int32_t* d_k,
                  const int32_t* d_lda, const int32_t* d_ldb, const int32_t* d_ldc, int group_count, int64_t m_hint,
                  int64_t n_hint, int64_t k_hint, float alpha, float beta, void* workspace, size_t workspace_bytes,
                  void* stream);

/*
 * The grouped GEMM in two steps, for callers that run one grouping more than once (the layers of a model that
 * share a routing; a benchmark loop).  (No counterpart in the reference, whose kernels rebuild their per-group
 * descriptors on every call.)
 *   fb_group_gemm_prepare  builds the tile table and the tensor maps of the groups in `workspace`
 *                          (fb_group_workspace_bytes(group_count) bytes; fb_group_min_workspace_bytes for whole tiles only);
 *   fb_group_gemm_run      runs the GEMM over a prepared workspace: out_g <- alpha * A_g * B_g + beta * C_g with the
 *                          addresses, sizes and pitches the arrays held when prepare ran.
 * dtype, b_k_contiguous, group_count and the three hints must be the same in both calls (they select the tile plan);
 * the workspace must stay untouched between them; the environment switches must not change in between.
 * fb_group_gemm(...) = prepare + run.  A beta != 0 run needs d_c to have been given to prepare.
 */
int fb_group_gemm_prepare(int dtype, int b_k_contiguous, const int64_t* d_a, const int64_t* d_b, const int64_t* d_c,
                          const int64_t* d_out, const int32_t* d_m, const int32_t* d_n, const int32_t* d_k,
                          const int32_t* d_lda, const int32_t* d_ldb, const int32_t* d_ldc, int group_count,
                          int64_t m_hint, int64_t n_hint, int64_t k_hint, void* workspace, size_t workspace_bytes,
                          void* stream);
int fb_group_gemm_run(int dtype, int b_k_contiguous, int group_count, int64_t m_hint, int64_t n_hint, int64_t k_hint,
                      float alpha, float beta, void* workspace, size_t workspace_bytes, void* stream);

/*
 * Grouped matmul over row segments of one matrix:
 *     C[o_{g-1}:o_g, :] <- A[o_{g-1}:o_g, :] @ B[g]        (o_{-1} = 0)
 *   A [M, lda>=k]; B[g] at b + g*b_group_stride with rows `ldb` apart, stored
 *   [k, n] (b_k_contiguous = 0) or [n, k] (b_k_contiguous = 1); C [M, ldc>=n];
 *   d_offs = int32 DEVICE array of cumulative end rows.  dtype FB_BF16 / FB_F16.
 * Replaces group_mm, src/flag_blas/ops/level3/group_gemm.py:689-717
 *   (+ .../hopper/ops/group_gemm.py:894-943).
 */
int fb_group_mm(int dtype, int b_k_contiguous, const void* A, int64_t lda, const void* B, int64_t ldb,
                int64_t b_group_stride, void* C, int64_t ldc, const int32_t* d_offs, int group_count, int64_t n,
                int64_t k, void* workspace, size_t workspace_bytes, void* stream);

/* Bytes the grouped entry points ask for: the two tile tables with their tensor maps (required) plus the
 * partial-sum slots of the stream-K tail (optional: with only the tables' bytes the call runs whole tiles). */
size_t fb_group_workspace_bytes(int group_count);

/* The required part alone: tile tables and tensor maps.  A grouped call given exactly this much runs every tile whole. */
size_t fb_group_min_workspace_bytes(int group_count);

/*
 * fb_group_gemm without a workspace argument, for callers that are not allowed to allocate
 * device memory at all.  (This entry point has no counterpart in the reference.)
 *
 * Who needs it: code that runs inside another runtime's enqueue/execute hook, where the host
 * forbids cudaMalloc on the hot path, and services that reserved all of HBM for their own pool
 * up front, so that a later cudaMalloc would fail or stall.  Such callers still own and pass every
 * input and output; only the call's internal scratch (tile table + per-group tensor maps) is
 * taken from a fixed array inside the library instead of from `workspace`.
 *
 * Limits and rules:
 *   - at most fb_no_alloc_max_groups() (= 256) groups per call; more returns FB_ERR_TOO_LARGE;
 *   - the array costs about 245 KB of device memory on every GPU that loads the library, for
 *     the life of the process;
 *   - the first call on each device looks the array's address up (cudaGetSymbolAddress); make
 *     that first call before starting any stream capture on that device.  If it is also the
 *     process's first use of this library on that device, the CUDA runtime loads the library's
 *     module at that moment, which is when the array and the kernels are placed in device
 *     memory: a service that hands all of HBM to its own pool must make this first call (a
 *     group_count of 1 with m = 0 is enough) BEFORE it does so;
 *   - all calls share the one array per device: two calls whose GPU work can overlap (different
 *     streams, different threads) race on it -- order them on one stream or with events;
 *   - the library itself calls no cudaMalloc / cudaFree / allocating library routine, on any call.
 * Results: bit for bit those of fb_group_gemm called with a workspace of exactly the tables' size
 * (the required part of fb_group_workspace_bytes; this entry point's array holds nothing else).
 * A call of fb_group_gemm that also received the optional partial-sum scratch may split the k
 * range of the tiles of a half-empty last wave between CTAs when k is long; it then adds the
 * same products in another order, and the two results agree within fp32 summation rounding
 * (well inside the operator's tolerance), not bit for bit.
 */
int fb_group_gemm_no_alloc(int dtype, int b_k_contiguous, const int64_t* d_a, const int64_t* d_b, const int64_t* d_c,
                           const int64_t* d_out, const int32_t* d_m, const int32_t* d_n, const int32_t* d_k,
                           const int32_t* d_lda, const int32_t* d_ldb, const int32_t* d_ldc, int group_count,
                           int64_t m_hint, int64_t n_hint, int64_t k_hint, float alpha, float beta, void* stream);

/* Largest group_count fb_group_gemm_no_alloc accepts. */
int fb_no_alloc_max_groups(void);

/* ---- diagnostics -------------------------------------------------------- */

/* Human-readable text for an FB_* code or a device status. */
const char* fb_status_string(int status);

/*
 * Device-side status word of the current device: 0, or the code left by a
 * kernel that gave up on a bounded wait (1xx) or skipped a group whose operand
 * addresses are not element-aligned (2xx).  Synchronises the device.  `reset` != 0 clears the word.
 */
int fb_device_status(int reset);

/* cudaError_t (as int) of the last failed CUDA call made by this library on this thread. */
int fb_last_cuda_error(void);

/*
 * The library's FLAGBLAS_B200_* environment switches (plan overrides for tests and profiling
 * sweeps; INTEGRATION.md lists them) are read once per process.  A program that changes one
 * with setenv() while running calls this to have every switch read again on its next use.
 */
void fb_reload_env(void);

/*
 * Profiling aid: when set to a device buffer of 16 int64, CTA 0 of every tensor-core GEMM launched
 * afterwards adds up SM cycles spent per role and phase (producer: [0] waiting for a free stage,
 * [1] issuing copies; MMA issuer: [2] waiting for data, [3] issuing MMAs, [4] committing,
 * [5] waiting for a free accumulator, [6] total; epilogue: [7] waiting, [8] draining) and stores
 * them there.  NULL (the default) switches the accounting off.  Not thread safe.
 */
void fb_debug_set_profile_buffer(void* device_buffer_16_int64);

/* Hash of the sources this binary was compiled from (set by the build recipe); the Python loader refuses a
 * binary whose id differs from the sources next to it. */
const char* fb_build_id(void);

/* Number of SMs the persistent kernels size their grids with on the current device. */
int fb_sm_count(void);

/*
 * Self-test of the bounded-wait path: one CTA waits on an mbarrier that nothing
 * ever completes, with a limit of `limit_cycles` SM clocks, and must come back
 * with the time-out status.  Returns that device status (105 when the path works).
 * Synchronises the device; leaves the status word cleared.
 */
int fb_selftest_bounded_wait(int64_t limit_cycles, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* FLAGBLAS_B200_H_ */
