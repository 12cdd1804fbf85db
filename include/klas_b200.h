/*
 * klas_b200.h -- C ABI of the B200-native Klas matrix-multiply library.
 *
 * Every function here has C linkage, takes plain pointers and sizes, and
 * returns a klas_status (0 = success).  Unless the name ends in `_host`, all
 * data pointers are DEVICE pointers on the current CUDA device, the call is
 * asynchronous on `stream` (a cudaStream_t passed as void*, NULL = the legacy
 * default stream) and allocates nothing.
 *
 * Each entry point names the reference interface (FStarLang/kuiper, paths
 * relative to that project) whose work it takes over.  The reference's own
 * C++-linkage names (dist/Klas_*.h) are thin wrappers over these functions:
 * see include/klas/Klas_*.h.
 */
#ifndef KLAS_B200_H
#define KLAS_B200_H 1

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum klas_status_e {
    KLAS_OK = 0,
    KLAS_ERR_INVALID = 1,      /* bad argument (null pointer, bad enum, misaligned) */
    KLAS_ERR_UNSUPPORTED = 2,  /* legal request this kernel cannot serve (e.g. K % 8 != 0 on the tensor-core path) */
    KLAS_ERR_CUDA = 3,         /* a CUDA runtime/driver call failed; see klas_b200_last_error() */
    KLAS_ERR_TIMEOUT = 4,      /* a bounded device-side wait gave up; output is undefined, context still usable */
    KLAS_ERR_TOO_LARGE = 5     /* size beyond a documented fixed limit */
} klas_status;

typedef enum klas_dtype_e {
    KLAS_F32 = 0,
    KLAS_F64 = 1,
    KLAS_U32 = 2,
    KLAS_U64 = 3,
    KLAS_BF16 = 4,
    KLAS_F16 = 5
} klas_dtype;

/* Storage order of the three matrices of a CUDA-core GEMM. */
typedef enum klas_layout_e {
    KLAS_RRR = 0,  /* A, B, C row-major */
    KLAS_CCC = 1   /* A, B, C column-major */
} klas_layout;

/* Storage order of the B operand of a tensor-core GEMM (A and C/D are row-major). */
typedef enum klas_b_major_e {
    KLAS_B_ROW_MAJOR = 0,  /* B is shared x cols, cols contiguous (the reference's layout) */
    KLAS_B_COL_MAJOR = 1   /* B is stored as cols x shared, shared contiguous ("TN" GEMM) */
} klas_b_major;

/*
 * Element-wise hooks of klas_b200_gemm_tc_fused.  The reference threads arbitrary functions
 * through its tensor-core kernels when they are extracted (mapA / mapB / comb:
 * include/kuiper/tensorcores.h:30-59); a compiled library offers a fixed menu.
 * A map is evaluated in f32 on each 16-bit element and rounded back once to the element type.
 * Every map sends 0 to 0.
 */
typedef enum klas_map_e {
    KLAS_MAP_ID = 0,      /* x */
    KLAS_MAP_SQRT = 1,    /* sqrt(x); NaN for x < 0.  Tensor-core path: hardware approximation, at most 1 ulp of f32
                             before the rounding, bf16 inputs below 1.2e-38 give 0 */
    KLAS_MAP_ABS = 2,     /* |x| */
    KLAS_MAP_SQUARE = 3,  /* x * x */
    KLAS_MAP_RELU = 4,    /* max(x, 0) */
    KLAS_MAP_NEG = 5      /* -x */
} klas_map;

/* How the accumulator acc = map_a(A).map_b(B) meets the old value c of C. */
typedef enum klas_comb_e {
    KLAS_COMB_NEW = 0,    /* acc (C not read) */
    KLAS_COMB_AXPBY = 1,  /* alpha * acc + beta * c */
    KLAS_COMB_MAX = 2,    /* max(c, acc) */
    KLAS_COMB_MIN = 3,    /* min(c, acc) */
    KLAS_COMB_MUL = 4,    /* c * acc */
    KLAS_COMB_RELU = 5,   /* max(acc, 0) (C not read) */
    KLAS_COMB_SCALED = 6  /* alpha * acc (C not read) */
} klas_comb;

/* Last error message of the calling thread ("" if none). Never NULL. */
const char *klas_b200_last_error(void);

/* Library ABI version (major * 1000 + minor). */
int klas_b200_version(void);

/* Number of streaming multiprocessors of the current device (grid sizing aid). */
int klas_b200_sm_count(void);

/*
 * CUDA-core GEMM on f32 / f64 / u32 / u64 (bf16 accepted: f32 accumulate, one
 * rounding at the end).  Integers wrap mod 2^32 / 2^64.
 *
 *   alpha == NULL && beta == NULL :  C = A.B            (C is never read)
 *   otherwise (both non-NULL)     :  C = beta*C + alpha*(A.B)   (C read even if beta == 0)
 *
 * alpha/beta point to HOST scalars of type `dtype`.  A is m x k, B is k x n,
 * C is m x n in `layout`; with batch > 1 the matrices are contiguous pages
 * [batch][m][k], [batch][k][n], [batch][m][n].  Any m, n, k >= 0 is legal.
 *
 * Replaces: Klas_GEMM_SHMem_g_{matmul,gemm}_* (dist/Klas_GEMM_SHMem.h:8-187),
 * Klas_GEMM_Tiled_* (dist/Klas_GEMM_Tiled.h), Klas_GEMM_BlockTiling1D_*
 * (dist/Klas_GEMM_BlockTiling1D.h:8-131), Klas_GEMM_BlockTiling2D_g_gemm_*
 * (dist/Klas_GEMM_BlockTiling2D.h:8-1376) and Klas_GEMM_Naive{1,2}_* (dist/Klas_GEMM_Naive1.h:8-65).
 */
int klas_b200_gemm(int dtype, int layout, uint32_t batch,
                   uint64_t m, uint64_t n, uint64_t k,
                   const void *alpha, const void *beta,
                   const void *A, const void *B, void *C, void *stream);

/*
 * C = A.B (one matrix, no alpha / beta) for callers that asked the reference for its compensated
 * sums: Klas_GEMM_Naive3_* add each row-by-column sum with Kahan's correction in the element type
 * (dist/Klas_GEMM_Naive3.cu:17-30).  KLAS_F32 is accumulated here in f64 -- the products of f32
 * numbers are exact in f64 and the sum carries 29 more bits than a compensated f32 sum recovers --
 * and rounded to f32 once; KLAS_BF16 is accumulated in f32 as in klas_b200_gemm (again more than
 * bf16 compensation keeps).  KLAS_F64 takes the plain kernel: its sums are ordinary f64 sums in
 * ascending k, WITHOUT compensation -- within the drivers' tolerance, but a cancellation-heavy
 * sum loses the digits the reference's correction term would have kept.
 * Replaces: Klas_GEMM_Naive3_g_matmul_{bf16,f32,f64}_{rrr,ccc} (dist/Klas_GEMM_Naive3.h:8-41).
 */
int klas_b200_gemm_compensated(int dtype, int layout, uint64_t m, uint64_t n, uint64_t k,
                               const void *A, const void *B, void *C, void *stream);

/*
 * General batched CUDA-core GEMM: `batch` row-major products
 *
 *   C_p = comb( C_p, map_a(A_p) . map_b(B_p) ),     p = 0 .. batch-1
 *
 * where X_p starts `stride_x` elements after X_(p-1) and consecutive rows of X are `ldx`
 * elements apart (lda >= k, ldb >= n, ldc >= n).  stride_a or stride_b may be 0: every page
 * then multiplies the same matrix.  Pages of C must not overlap.  dtype as klas_b200_gemm;
 * map_a / map_b: klas_map (KLAS_MAP_SQRT needs a floating type; on the unsigned types abs and
 * relu are the identity and neg, square wrap); comb: klas_comb, with alpha / beta (host
 * scalars of the matrix dtype) required for KLAS_COMB_AXPBY and ignored otherwise.  Maps are
 * evaluated in the arithmetic type (f32 for bf16 storage) on the way into shared memory.
 *
 * Replaces: the rank-3 strided entries with mapA / mapB / comb that the reference's sources
 * define for its shared-memory and 2-D block-tiling kernels and derive the rank-2 ones from
 * (src/lib/kernel/gemm/Kuiper.Kernel.GEMM.SHMem.fsti:40-97, ...BlockTiling2D.fsti:34-60), of
 * which it exports the contiguous f32 case as Klas_GEMM_Naive1_g_batched_* (dist/Klas_GEMM_Naive1.h:54-66).
 */
int klas_b200_gemm_strided(int dtype, uint32_t batch, uint64_t m, uint64_t n, uint64_t k,
                           const void *alpha, const void *beta,
                           const void *A, uint64_t lda, uint64_t stride_a,
                           const void *B, uint64_t ldb, uint64_t stride_b,
                           void *C, uint64_t ldc, uint64_t stride_c,
                           int map_a, int map_b, int comb, void *stream);

/*
 * Tensor-core GEMM (tcgen05 UMMA, fp32 accumulation in tensor memory):
 *
 *   D = out_dtype( alpha * (A.B) + beta * C )      if C != NULL
 *   D = out_dtype( A.B )                           if C == NULL (alpha, beta ignored)
 *
 * A: rows x shared row-major, in_dtype (KLAS_BF16 or KLAS_F16).
 * B: shared x cols, in_dtype, storage order `b_major`.
 * C: rows x cols row-major, out_dtype, may alias D (in-place accumulate).
 * D: rows x cols row-major, out_dtype (KLAS_F32, KLAS_F16 or KLAS_BF16).
 * batch > 1: contiguous pages of A, B, C, D.
 * Requires shared % 8 == 0, cols % 8 == 0 and 16-byte aligned A, B, C, D.
 * `status_word`: optional device int (may be NULL) that receives a non-zero
 * code when a bounded device-side wait gives up.
 * A small output with a long shared dimension (128 x 256 tiles filling less than half of the SMs,
 * e.g. 1024 x 1024 x 4096) is computed as up to 8 partial products over parts of the shared
 * dimension, which a second kernel on the same stream adds in a fixed order: the result is the
 * same from run to run and within fp32 re-association of the one-pass product.  The same is done
 * for the tiles of a part-filled last round when the shared dimension is long (2560 x 2048 x 8192:
 * one launch for the 74 tile pairs of the full round, one for the last 6 cut into 8 parts; KLAS_KNOB_TC_TAIL).  The parts live
 * in a device buffer the library keeps per (device, stream), allocated at the first such call on
 * the stream (a call that would have to allocate while the stream is recording a CUDA graph
 * runs in one pass instead) and freed by klas_b200_release_workspace(); at most 8 streams per
 * device get one, further streams run in one pass.  A CUDA graph that recorded such a call holds
 * the buffer's address: do not release the workspace while the graph may still be launched.
 * KLAS_KNOB_TC_KSPLIT = 1 turns the split off.
 *
 * Replaces: Klas_GEMM_TensorCore2D_g_gemm_{bf16_f32,f16_f16}_* (dist/Klas_GEMM_TensorCore2D.h:8-1220),
 * Klas_GEMM_TensorCore2D_To_g_gemm_bf16_f32_bf16_* (dist/Klas_GEMM_TensorCore2D_To.h),
 * Klas_GEMM_TensorCore_g_gemm_f16_{f16,f32}_* (dist/Klas_GEMM_TensorCore.h:8-85).
 */
int klas_b200_gemm_tc(int in_dtype, int out_dtype, int b_major, uint32_t batch,
                      uint64_t rows, uint64_t shared, uint64_t cols,
                      const void *A, const void *B, const void *C, void *D,
                      float alpha, float beta, int *status_word, void *stream);

/*
 * Tensor-core GEMM with element-wise hooks fused into the kernel:
 *
 *   D = out_dtype( comb( C, map_a(A) . map_b(B) ) )
 *
 * map_a / map_b (klas_map) are applied to the operand tiles in shared memory, between the
 * copy from global memory and the tensor-core instruction, by dedicated warps: no mapped copy
 * of A or B is ever written to global memory.  comb (klas_comb) runs in the epilogue on the
 * fp32 accumulator.  C is required for AXPBY / MAX / MIN / MUL and ignored otherwise; alpha and
 * beta matter for AXPBY (alpha also for SCALED) only.  Everything else as klas_b200_gemm_tc (which is the case
 * map_a = map_b = KLAS_MAP_ID, comb = C ? AXPBY : NEW).
 *
 * Replaces: the fused tensor-core kernels the reference generates from
 * Kuiper.Kernel.GEMM.TensorCore2D (mapA / mapB / comb hooks, include/kuiper/tensorcores.h:30-59)
 * and the demonstration Kuiper_Example_Fused_GEMM_gemm_sqrt_fused, C = sqrt(A).B in f16
 * (dist/Kuiper_Example_Fused_GEMM.h:9-15), which runs one thread per output element.
 */
int klas_b200_gemm_tc_fused(int in_dtype, int out_dtype, int b_major, uint32_t batch,
                            uint64_t rows, uint64_t shared, uint64_t cols,
                            const void *A, const void *B, const void *C, void *D,
                            float alpha, float beta, int map_a, int map_b, int comb,
                            int *status_word, void *stream);

/*
 * klas_b200_gemm_tc_fused on operands that are windows of larger arrays: rows of A, B and C / D
 * are lda, ldb, ldd elements apart and consecutive pages stride_a, stride_b, stride_d elements
 * apart (0 = packed: the row length, resp. rows x the row stride).  C, where the combine rule
 * reads it, has D's strides.  The last dimension of every operand stays contiguous.  With
 * KLAS_B_COL_MAJOR the "rows" of B are its `cols` stored rows of `shared` elements.  The strides
 * go into the tensor maps of the TMA copies, so a window costs nothing over a packed operand.
 * Requires every stride to be a multiple of 8 elements (16-byte steps for the 16-bit operands)
 * and not shorter than the row it steps over, besides what klas_b200_gemm_tc requires.
 * A page stride of 0 cannot share one matrix between pages on this path (a tensor map has no
 * zero stride); use klas_b200_gemm_strided, or one call per page, for that.
 *
 * Replaces: the strided row-major A and B that the reference's tensor-core kernel accepts in
 * its sources (`strided_row_major lA / lB`, row stride a multiple of the copy vector:
 * src/lib/kernel/gemm/Kuiper.Kernel.GEMM.TensorCore2D.fsti:29-36), which its exported entries
 * instantiate with packed rows only (dist/Klas_GEMM_TensorCore2D.h:8-1220).
 */
int klas_b200_gemm_tc_strided(int in_dtype, int out_dtype, int b_major, uint32_t batch,
                              uint64_t rows, uint64_t shared, uint64_t cols,
                              const void *A, uint64_t lda, uint64_t stride_a,
                              const void *B, uint64_t ldb, uint64_t stride_b,
                              const void *C, void *D, uint64_t ldd, uint64_t stride_d,
                              float alpha, float beta, int map_a, int map_b, int comb,
                              int *status_word, void *stream);

/*
 * Reads (and then clears) the current device's tensor-core status word.
 * Returns KLAS_OK and *site = 0 when no bounded wait has given up since the
 * last call; otherwise KLAS_ERR_TIMEOUT and *site = the code of the first wait
 * that gave up.  Synchronises with the default stream; `site` may be NULL.
 * While the word is non-zero every later klas_b200_gemm_tc launch on that
 * device drains immediately, so call this after a suspicious result.
 * No counterpart in the reference (its kernels have no waits that can fail).
 */
int klas_b200_gemm_tc_status(int *site);

/*
 * The same word without touching the device: the kernels also write the site code to a
 * host-visible mirror (a 4-byte pinned, mapped allocation made once per device by the first
 * tensor-core launch there -- make that launch outside any stream capture).  Returns 0 or the site
 * code; it is exact once the launches of interest have been synchronised with, and costs a load.
 * A blocking caller checks this after its synchronise and calls klas_b200_gemm_tc_status() only
 * when it is non-zero (the reference-named wrappers do).  Asynchronous callers of
 * klas_b200_gemm_tc / _fused / _strided / _sdpa_fused MUST look at one of the two after they
 * synchronise: a wait that gave up leaves D undefined, and while the word is set later launches
 * on the device drain at once.  No counterpart in the reference.
 */
int klas_b200_gemm_tc_status_peek(void);

/*
 * Diagnostic: launches one warp that waits, with the same bounded wait the tensor-core
 * pipeline uses, on a barrier nothing will ever signal.  After `limit_ms` (1..1000) the wait
 * gives up, the device status word receives site 0x7F, `*gave_up` (optional device int) is set
 * to 1, and the kernel returns normally: the context stays usable and the next
 * klas_b200_gemm_tc_status() call reports KLAS_ERR_TIMEOUT once.  Lets a host program (or a
 * test) exercise its handling of a stalled pipeline without stalling one.
 * No counterpart in the reference.
 */
int klas_b200_debug_wait_probe(uint32_t limit_ms, int *gave_up, void *stream);

/*
 * CSR x dense:  C[rows x cols] = CSR(A)[rows x shared] . B[shared x cols],
 * B and C row-major, dtype KLAS_F32 or KLAS_U32 (wrapping).  Each row's
 * products are summed in CSR order starting from 0.  Every row of C is
 * overwritten (all-zero rows included).  `row_indices` (in the reference a permutation of
 * 0..rows-1 giving the order in which rows are scheduled) may be NULL and is not read: work is
 * cut into ranges of equal size (rows + nonzeros) instead.
 * CSR: row_off[0] == 0, monotone, row_off[rows] == nnz, columns < shared.
 * A row with more than max(1024, (rows + nnz) / (4 * resident warps)) nonzeros is summed in
 * pieces that are added to C atomically: for such rows the f32 result is within the tolerance
 * but the order of the pieces, hence the last bits, may change from call to call.  All other
 * rows are summed in CSR order and repeat bit for bit.
 *
 * Replaces: Klas_SPMM_spmm_{f32,u32}, Klas_SPMM_g_spmm_f32_* (dist/Klas_SPMM.h:15-673).
 */
int klas_b200_spmm(int dtype, uint32_t rows, uint32_t shared, uint32_t cols, uint32_t nnz,
                   const void *elems, const uint32_t *col_ind, const uint32_t *row_off,
                   const uint32_t *row_indices, const void *B, void *C, void *stream);

/*
 * Measurement aid for klas_b200_spmm (f32, cols % 4 == 0): issues exactly the reads of B that the
 * SpMM kernel issues for a matrix with these column indices -- for every nonzero and every slab
 * of 128 columns one 512-byte piece of row col_ind[i] of B (shared x cols, row-major) -- and
 * nothing else: no values, no products, no C.  Its duration is the time the memory system needs
 * to deliver the gathers, the ceiling a bench reports the SpMM kernel against (with random
 * columns the gathers, nnz * 4 * cols bytes from L2 to the SMs, outweigh the bytes DRAM moves by
 * more than an order of magnitude).  Writes nothing.
 * No counterpart in the reference.
 */
int klas_b200_spmm_gather_probe(uint32_t shared, uint32_t cols, uint32_t nnz, const uint32_t *col_ind,
                                const void *B, void *stream);

/*
 * Building the CSR operand of klas_b200_spmm on the device, from a dense row-major rows x cols
 * matrix (dtype KLAS_F32 or KLAS_U32).  An entry is kept when it compares != 0 (so -0.0 is
 * dropped and NaN kept), in ascending column order within a row.
 *
 *   klas_b200_csr_count      writes row_off[0 .. rows]; row_off[rows] is nnz (read it back to
 *                            size elems / col_ind).  nnz must stay below 2^32.
 *   klas_b200_csr_fill       writes elems[nnz], col_ind[nnz] for the row_off of the count step.
 *   klas_b200_csr_row_order  row_indices[rows] = the rows by decreasing length, equal lengths by
 *                            increasing row: the schedule klas_b200_spmm takes as `row_indices`.
 *                            Needs klas_b200_csr_row_order_scratch_bytes(rows) bytes of 8-byte
 *                            aligned device scratch (sort keys), caller-owned.
 *
 * Replaces: the host-side preparation every reference SpMM caller runs first, sparsify_f32 /
 * sparsify_u32 (test/spmm_common.c.inc:73-137) and mk_row_indices (test/spmm_common.c.inc:139-157;
 * its std::sort leaves the order of equal-length rows open, here it is fixed).
 */
int klas_b200_csr_count(int dtype, uint32_t rows, uint32_t cols, const void *dense, uint32_t *row_off, void *stream);
int klas_b200_csr_fill(int dtype, uint32_t rows, uint32_t cols, const void *dense, const uint32_t *row_off,
                       void *elems, uint32_t *col_ind, void *stream);
size_t klas_b200_csr_row_order_scratch_bytes(uint32_t rows);
int klas_b200_csr_row_order(uint32_t rows, const uint32_t *row_off, uint32_t *row_indices, void *scratch,
                            size_t scratch_bytes, void *stream);

/*
 * (min, +) product on 16-bit path lengths with 0 = "no path":
 *   C[i][j] = add(C[i][j], add over k of mult(A[i][k], B[k][j])),
 *   mult(x, y) = 0 if x == 0 or y == 0 else (x + y) mod 2^16,  add = the smaller non-zero one.
 * A m x k, B k x n, C m x n, row-major device arrays; C must not overlap A or B.  Squaring a
 * distance matrix is A == B.  Bit-exact with the reference on every input, wrap-around included.
 * Replaces: Kuiper_GraphDist_matmul_dist_gpu (dist/Kuiper_GraphDist.h:11-12, kernel
 * dist/Kuiper_GraphDist.cu:9-45), which is the square case m = n = k, A = B.
 */
int klas_b200_minplus_u16(uint32_t m, uint32_t n, uint32_t k, const uint16_t *A, const uint16_t *B, uint16_t *C,
                          void *stream);

/*
 * Host-buffer variants: same semantics, but every data pointer is a HOST
 * pointer (pinned memory makes the copies asynchronous and faster).  The call
 * stages inputs into a per-device workspace that grows on demand and is kept
 * until klas_b200_release_workspace(), runs the kernel, copies the result
 * back and returns after the result is in host memory.  The workspace, streams and events are
 * one set per device: calls from several host threads on the same device are serialised by the
 * library (a per-device lock held for the whole call); calls on different devices run in parallel.
 */
int klas_b200_gemm_host(int dtype, int layout, uint32_t batch,
                        uint64_t m, uint64_t n, uint64_t k,
                        const void *alpha, const void *beta,
                        const void *A, const void *B, void *C);

int klas_b200_gemm_tc_host(int in_dtype, int out_dtype, int b_major, uint32_t batch,
                           uint64_t rows, uint64_t shared, uint64_t cols,
                           const void *A, const void *B, const void *C, void *D,
                           float alpha, float beta);

int klas_b200_spmm_host(int dtype, uint32_t rows, uint32_t shared, uint32_t cols, uint32_t nnz,
                        const void *elems, const uint32_t *col_ind, const uint32_t *row_off,
                        const uint32_t *row_indices, const void *B, void *C);

/*
 * Host placement for the host-buffer variants.  On a two-socket node a GPU reads and writes host
 * memory at full PCIe rate only when the buffers live on the socket it hangs off; with eight
 * ranks whose pinned buffers all sit on one socket the copies of half the GPUs cross the
 * socket link and the node's aggregate rate collapses.
 *   klas_b200_host_numa_node         NUMA node of the current device (from sysfs), -1 if unknown.
 *   klas_b200_host_bind_near_device  restricts the CALLING THREAD to that node's CPUs and makes the
 *                                    node the preferred one for memory it allocates from now on;
 *                                    call it before allocating the pinned buffers.  Changes only
 *                                    the calling thread's affinity and memory policy, nothing of the
 *                                    GPU.  KLAS_ERR_UNSUPPORTED when the node is unknown or its CPUs
 *                                    are not available to the process (nothing is changed then).
 * No counterpart in the reference.
 */
int klas_b200_host_numa_node(void);
int klas_b200_host_bind_near_device(void);

/*
 * Row-wise neighbours of the products (what sits either side of Q.K^T and P.V in an
 * attention block).  dtype KLAS_F16 / KLAS_F32 / KLAS_F64 unless said otherwise (softmax also
 * KLAS_BF16); 16-bit data is processed in fp32 and rounded once.
 *
 * klas_b200_softmax: in place, a[r][c] = exp(a[r][c] - max_r) / sum_c exp(a[r][c] - max_r) for
 * every row of the row-major rows x cols matrix `a` (log_softmax != 0: a[r][c] - max_r - log(sum)).
 * rows == 1 is the vector case: the vector is cut into chunks (16384 elements or more, at most
 * 2048 chunks) folded by separate CTAs, which needs `scratch`: klas_b200_softmax_scratch_bytes(rows, cols) bytes of 16-byte
 * aligned device memory (0 for rows > 1), caller-owned, overwritten.
 * Replaces: Klas_Softmax_softmax_gpu{,_n}_* (dist/Klas_Softmax.h), Klas_LogSoftmax_log_softmax_gpu{,_n}_*
 * (dist/Klas_LogSoftmax.h), Klas_RowSoftmax_row_softmax_rm_* (dist/Klas_RowSoftmax.h:7-11).
 * klas_b200_softmax_host: the same on a HOST buffer (copy in, compute, copy out); replaces the
 * host-pointer variants Klas_Softmax_softmax{,_n}_* and Klas_LogSoftmax_log_softmax{,_n}_*.
 */
size_t klas_b200_softmax_scratch_bytes(uint64_t rows, uint64_t cols);
int klas_b200_softmax(int dtype, int log_softmax, uint64_t rows, uint64_t cols, void *a,
                      void *scratch, size_t scratch_bytes, void *stream);
int klas_b200_softmax_host(int dtype, int log_softmax, uint64_t rows, uint64_t cols, void *a);

/*
 * klas_b200_softmax_static: the vector case (rows == 1) of klas_b200_softmax without a scratch
 * argument and without any allocation.  No counterpart in the reference.
 *
 * For callers that cannot supply scratch and must not allocate: a process that gave all device
 * memory to its own arena at start-up, or a latency-critical loop where cudaMalloc / cudaFree
 * are off limits because they synchronise the device.  The per-chunk statistics go to a fixed
 * 16 KiB array inside the library's device image instead, which limits the vector to
 * KLAS_B200_SOFTMAX_STATIC_MAX_COLS elements; a longer vector is refused with KLAS_ERR_TOO_LARGE
 * (use klas_b200_softmax).  Same kernels, same results as klas_b200_softmax.
 *
 * The function calls no allocator (CUDA's or the host library's workspace).  The first call on
 * each device looks up the array's device address (cudaGetSymbolAddress, with that device
 * current); make that first call outside any stream capture.  All calls on one device share the
 * array: calls that may overlap in time (several streams or threads) race on it and must be
 * serialised by the caller.  The array keeps the previous call's statistics; none of it needs
 * clearing, every entry read is written first by the same call.  The address looked up by the
 * first call is kept per device ordinal for the life of the process: after cudaDeviceReset() (or
 * anything else that destroys the device's primary context) it is stale and this entry point must
 * not be called again in that process.
 */
#define KLAS_B200_SOFTMAX_STATIC_MAX_COLS 16777216ull   /* 1024 chunks of 16384 elements */
int klas_b200_softmax_static(int dtype, int log_softmax, uint64_t cols, void *a, void *stream);

/*
 * Scaled dot-product attention in the three steps of the reference's naive kernel
 * (src/lib/kernel/Kuiper.Kernel.SDPA.Naive.fst:390-470: batched GEMM, row softmax, batched GEMM),
 * for `pages` = batch x heads independent heads:
 *
 *   S = scale * Q.K^T + bias      written over `bias_scores`
 *   P = softmax of every row of S (in place)
 *   O = P.V
 *
 * Q [pages][l][e], K [pages][s][e], V [pages][s][ev], bias_scores [pages][l][s], out [pages][l][ev],
 * all row-major, contiguous, of one dtype (KLAS_F16 or KLAS_BF16) and 16-byte aligned; e, s and ev
 * multiples of 8.  Products accumulate in fp32 on the tensor cores; S, P and O are rounded to
 * `dtype` once each.  has_bias == 0: `bias_scores` is only the scratch for S (its contents on
 * entry are ignored).  On return it holds P.  Three launches on `stream`.
 */
int klas_b200_sdpa(int dtype, uint32_t pages, uint64_t l, uint64_t s, uint64_t e, uint64_t ev,
                   const void *Q, const void *K, const void *V, void *bias_scores, int has_bias,
                   void *out, float scale, void *stream);

/*
 * The same attention in ONE kernel that never writes the scores to global memory (running row
 * maximum and sum, as in the reference's Kuiper.Kernel.FlashAttention,
 * src/lib/kernel/Kuiper.Kernel.FlashAttention.fst): O = softmax(scale * Q.K^T).V per head, no
 * bias.  Q [pages][l][e], K [pages][s][e], V [pages][s][e], out [pages][l][e], row-major,
 * contiguous, 16-byte aligned, dtype KLAS_F16 or KLAS_BF16; e = 64 or 128 (other head
 * dimensions: KLAS_ERR_UNSUPPORTED, use klas_b200_sdpa).  Any l and s >= 1; scale > 0.  fp32 accumulation and
 * fp32 softmax statistics; probabilities are rounded to `dtype` before they multiply V.  A
 * bounded device-side wait that gives up is reported by klas_b200_gemm_tc_status().
 */
int klas_b200_sdpa_fused(int dtype, uint32_t pages, uint64_t l, uint64_t s, uint64_t e,
                         const void *Q, const void *K, const void *V, void *out, float scale, void *stream);

/*
 * b[r][c] = scale[r] * b[r][c] for the m x n matrix b, row-major (col_major == 0) or
 * column-major.  Replaces: Klas_RowScale_rowscale_*_{rowmajor,colmajor} (dist/Klas_RowScale.h:7-23).
 */
int klas_b200_rowscale(int dtype, int col_major, uint64_t m, uint64_t n, const void *scale, void *b,
                       void *stream);

/*
 * *result = sum of a[0..n) (dtype F16, F32, F64, U32 or U64; integers wrap; floating-point sums
 * are folded in a fixed order, so repeated calls agree bit for bit).  `result` is a device
 * scalar; `scratch` = klas_b200_reduce_scratch_bytes(n) bytes of 8-byte aligned device memory.
 * klas_b200_reduce_sum_host: `a` on the device, `result` on the host, blocking.
 * Replaces: Klas_HReduce_reduce_*_plus (dist/Klas_HReduce.h:7-20) and
 * Klas_AtomicReduce_reduce_* (dist/Klas_AtomicReduce.h:7-13).
 */
size_t klas_b200_reduce_scratch_bytes(uint64_t n);
int klas_b200_reduce_sum(int dtype, uint64_t n, const void *a, void *result, void *scratch,
                         size_t scratch_bytes, void *stream);
int klas_b200_reduce_sum_host(int dtype, uint64_t n, const void *a, void *result);

/*
 * ---- Several GPUs of one node, one host thread --------------------------------------------------
 *
 * The products shard without any exchange of data: dense GEMM by row blocks of A and C with B
 * replicated on every device, batched GEMM by pages, CSR x dense by CSR row ranges with B
 * replicated.  A context holds one stream per device; a sharded call launches the single-GPU kernel
 * on every device's stream with that device's shard pointers and returns (asynchronous, like the
 * single-GPU entries); klas_b200_mg_synchronize waits for all devices and reports a tensor-core
 * wait that gave up.  Pointer arrays have one entry per device of the context, in its order;
 * every pointer is a device pointer on ITS device.  `bounds` arrays have count + 1 entries:
 * device i owns rows (or pages) [bounds[i], bounds[i+1]) and its shard pointer addresses its
 * first row; a device may own nothing.
 *
 * `gather` asks for the result assembled, by NCCL over NVLink on the same streams (loaded with
 * dlopen when first needed; without an NCCL library a gather returns KLAS_ERR_UNSUPPORTED and
 * everything else still works): KLAS_MG_NO_GATHER leaves the shards where they are (`full`
 * ignored); KLAS_MG_GATHER_ALL fills full[i] on every device with all rows; KLAS_MG_GATHER_FIRST
 * fills full[0] only.  Shards of unequal size are fine.
 *
 * No counterpart in the reference, which is single-GPU (dist/Klas_*.h run on the current device).
 */
typedef struct klas_mg_context_s klas_mg_context;
typedef enum klas_mg_gather_e { KLAS_MG_NO_GATHER = 0, KLAS_MG_GATHER_ALL = 1, KLAS_MG_GATHER_FIRST = 2 } klas_mg_gather;

int klas_b200_mg_create(const int *devices, int count, klas_mg_context **ctx);
int klas_b200_mg_destroy(klas_mg_context *ctx);
int klas_b200_mg_count(const klas_mg_context *ctx);
void *klas_b200_mg_stream(const klas_mg_context *ctx, int index);   /* cudaStream_t of device `index`, for the caller's own copies */
int klas_b200_mg_synchronize(klas_mg_context *ctx);

/* Host-only partitioners.  Row blocks: `parts` contiguous blocks of [0, rows) whose boundaries are
 * multiples of `align` (256 = the tensor-core tile height), as even as that allows.  CSR ranges:
 * equal row counts, or (balance_nnz != 0, row_off a HOST array of rows + 1 offsets) boundaries by
 * binary search on row_off so that every range holds about nnz / parts nonzeros. */
int klas_b200_mg_row_blocks(uint64_t rows, int parts, uint64_t align, uint64_t *bounds);
int klas_b200_mg_csr_row_ranges(const uint32_t *row_off, uint32_t rows, int parts, int balance_nnz, uint32_t *bounds);

/* Copies `bytes` bytes from buffers[root] into every other device's buffer: the one-off replication of B. */
int klas_b200_mg_broadcast(klas_mg_context *ctx, void *const *buffers, size_t bytes, int root);

/* D_i = A_i . B on every device (klas_b200_gemm_tc with C = NULL); A_i = rows row_bounds[i] .. of A. */
int klas_b200_mg_gemm_tc(klas_mg_context *ctx, int in_dtype, int out_dtype, int b_major, const uint64_t *row_bounds,
                         uint64_t shared, uint64_t cols, const void *const *A_shards, const void *const *B_replicas,
                         void *const *D_shards, int gather, void *const *D_full);
/* Batched: device i multiplies its pages of A by its pages of B (nothing is replicated). */
int klas_b200_mg_gemm_tc_batched(klas_mg_context *ctx, int in_dtype, int out_dtype, int b_major, const uint64_t *page_bounds,
                                 uint64_t rows, uint64_t shared, uint64_t cols, const void *const *A_pages,
                                 const void *const *B_pages, void *const *D_pages, int gather, void *const *D_full);
/* CUDA-core GEMM C_i = A_i . B (klas_b200_gemm, row-major, alpha = beta = NULL). */
int klas_b200_mg_gemm(klas_mg_context *ctx, int dtype, const uint64_t *row_bounds, uint64_t n, uint64_t k,
                      const void *const *A_shards, const void *const *B_replicas, void *const *C_shards, int gather,
                      void *const *C_full);
/* CSR x dense on CSR row ranges: device i holds its rows' nonzeros (nnz[i], elems[i], col_ind[i]) and
 * their row offsets REBASED to start at 0 (row_off[i], rows_i + 1 entries), and a replica of B. */
int klas_b200_mg_spmm(klas_mg_context *ctx, int dtype, const uint32_t *row_bounds, uint32_t shared, uint32_t cols,
                      const uint32_t *nnz, const void *const *elems, const uint32_t *const *col_ind,
                      const uint32_t *const *row_off, const void *const *B_replicas, void *const *C_shards, int gather,
                      void *const *C_full);

/*
 * Tuning / testing knobs.  The library picks tile shapes and schedules from the problem size;
 * these process-wide overrides exist so that a test or a tuning run can force each variant and
 * compare (every variant gives bit-identical results, which is what the tests check).  They are
 * plain atomics read at launch time: set them while no other thread is launching.  The library
 * never reads the environment.
 *
 *   KLAS_KNOB_TC_MODE    tensor-core tile: 0 library's choice (default), 1 single-CTA 128x256,
 *                        2 single-CTA 128x128, 3 CTA pair 256x256, 4 wide pair 512x256,
 *                        5 single-CTA 128x64
 *   KLAS_KNOB_TC_RASTER  tile columns swept together: 0 default (8), else 1..1024
 *   KLAS_KNOB_SIMT_SPLIT_K  CTAs per output tile along K in the CUDA-core kernel: 0 library's choice
 *                        (two when one part-filled wave of tiles would leave each SM with one CTA), 1 never, 2 whenever legal
 *   KLAS_KNOB_F64_MODE   0 library's choice, 1 keep fp64 products on the CUDA-core kernel
 *   KLAS_KNOB_SIMT_TILE  CUDA-core tile of 4-byte types: -1 library's choice, 0 64x64, 1 128x64, 2 128x128
 *   KLAS_KNOB_SPMM_SLAB  columns per slab of the SpMM kernel: 0 library's choice, 32, 64 or 128
 *   KLAS_KNOB_TC_KSPLIT  parts a tile's K range is cut into (single-CTA and pair tiles): 0 library's choice,
 *                        1 never, 2..8 that many where the shape allows it
 *   KLAS_KNOB_TC_TAIL    a part-filled last round of single-CTA or pair tiles cut along K in a second launch:
 *                        0 library's choice, 1 never, 2 whenever there is one
 *   KLAS_KNOB_HOST_GRID  blocks per side of the 2-D schedule of klas_b200_gemm_tc_host: -1 default (4),
 *                        0 row blocks only, 1..16
 * Returns KLAS_ERR_INVALID for an unknown knob or a value outside its range.  klas_b200_debug_get
 * returns the current value (INT32_MIN for an unknown knob).  No counterpart in the reference.
 */
typedef enum klas_knob_e {
    KLAS_KNOB_TC_MODE = 0,
    KLAS_KNOB_TC_RASTER = 1,
    KLAS_KNOB_SIMT_SPLIT_K = 2,
    KLAS_KNOB_F64_MODE = 3,
    KLAS_KNOB_SIMT_TILE = 4,
    KLAS_KNOB_HOST_GRID = 5,
    KLAS_KNOB_SPMM_SLAB = 6,
    KLAS_KNOB_TC_KSPLIT = 7,
    KLAS_KNOB_TC_TAIL = 8,
    KLAS_KNOB_COUNT = 9
} klas_knob;
int klas_b200_debug_set(int knob, int value);
int klas_b200_debug_get(int knob);

/*
 * What klas_b200_gemm_tc would run for a shape on a device with `sm_count` SMs: no device is touched.
 *   *kind       0 single-CTA tiles (128 rows), 1 CTA-pair tiles (256 x 256), 2 wide pair tiles (512 x 256)
 *   *tile_cols  columns of a tile (256, or 128 / 64 for narrow single-CTA tiles)
 *   *k_parts    parts every tile's shared dimension is cut into (1: one pass)
 *   *tail_cut   1: only the tiles of a part-filled last round are cut, in a second launch
 * The plan follows the tuning knobs.  It is what the tile-choice tests and the tuning run look at;
 * a launch that finds no buffer for the parts (see klas_b200_gemm_tc) still runs in one pass.
 * Any output pointer may be NULL.
 */
int klas_b200_gemm_tc_plan(uint64_t rows, uint64_t shared, uint64_t cols, uint32_t batch, int sm_count,
                           int *kind, int *tile_cols, int *k_parts, int *tail_cut);

/* Frees the calling device's workspaces: the host-variant staging buffers and the partial-product
 * buffers of the tensor-core GEMM's K split.  Synchronises the device. */
int klas_b200_release_workspace(void);

#ifdef __cplusplus
}
#endif
#endif /* KLAS_B200_H */
