/*
 * blb200.h — C ABI of the B200 (sm_100a) batched-GEMM library `libbatchlas_b200.so`.
 *
 * This is the seam a BatchLAS maintainer binds to replace
 *     template Event batchlas::gemm<Backend::CUDA, T>(Queue&, const MatrixView<T>&,
 *         const MatrixView<T>&, const MatrixView<T>&, T, T, Transpose, Transpose,
 *         ComputePrecision)
 * (BatchLAS src/backends/cublas.cc:1574-1585 -> gemm_vendor, :152-179 -> gemm_vendor_impl,
 * :106-150, which ends in one cublasGemmStridedBatchedEx call).  The reference has no C ABI
 * of its own for gemm; the closest precedent is its POD launch descriptor
 * `GemmLaunchDescriptor` + `cudaError_t launch_float(variant, desc, cudaStream_t)`
 * (BatchLAS src/backends/gemm_cublasdx_kernels.hh:21-48).  The descriptor below keeps that
 * shape and widens it to four dtypes, three transposes and 64-bit strides.
 *
 * Plain pointers and sizes only: no C++ types, no torch types.
 */
#ifndef BLB200_API_H_INCLUDED
#define BLB200_API_H_INCLUDED

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Element type.  Complex values are interleaved (re, im) pairs, as std::complex<T>. */
typedef enum { BLB200_S = 0, BLB200_D = 1, BLB200_C = 2, BLB200_Z = 3 } blb200_dtype;

/* Operand transform.  Same ordinals as batchlas::Transpose {NoTrans, Trans, ConjTrans}
 * (BatchLAS include/blas/enums.hh:78-82).  For real dtypes H behaves as T. */
typedef enum { BLB200_N = 0, BLB200_T = 1, BLB200_H = 2 } blb200_op;

/* Status codes.  0 = success, > 0 = a cudaError_t from the runtime, < 0 = one of these. */
enum {
  BLB200_OK = 0,
  BLB200_E_NULL = -1,        /* null descriptor, or null A/B/C with work to do          */
  BLB200_E_SHAPE = -2,       /* negative dim, ld smaller than the stored row count      */
  BLB200_E_DTYPE = -3,       /* dtype / op out of range                                 */
  BLB200_E_UNSUPPORTED = -4, /* forced kernel cannot run this problem                   */
  BLB200_E_NO_DEVICE = -5,   /* no sm_100 device current                                */
  BLB200_E_TOO_LARGE = -6,   /* problem exceeds a fixed capacity of the entry point     */
  BLB200_E_INTERNAL = -7
};

/* Kernel ids for `kernel_hint` (0 = let the dispatcher choose). */
enum {
  BLB200_K_AUTO = 0,
  BLB200_K_GENERIC = 1, /* any dtype/op/ld/alignment; predicated scalar loads              */
  BLB200_K_SMALL32 = 2, /* whole 32x32x32 float matrices per warp, TMA bulk-copy ring           */
  BLB200_K_SMALL64 = 3, /* whole 64x64x64 float matrices per warp pair, TMA ring (tiled+bulk)   */
  BLB200_K_TILED = 4,   /* register-blocked FFMA/DFMA smem tiles fed by 16-byte async copies    */
  BLB200_K_DMMA = 5,    /* FP64 tensor-core (mma.sync m8n8k4) tiles, double and complex<double> */
  BLB200_K_SGEMM128 = 6, /* float, A not transposed: 128x128x32 tiles, 8x8 blocks, packed FP32 FMA */
  BLB200_K_SMALL_RING = 7, /* any dtype, packed items up to 32x32 (k <= 64): whole items per warp, TMA ring */
  BLB200_K_DMMA_TMA = 8, /* double: the DMMA tiles fed by tensor-map TMA copies (128-byte swizzle) instead of cp.async */
  BLB200_K_SGEMM_TMA = 9 /* float, A not transposed, long k: 128x128x32 tiles fed by tensor-map TMA copies, 16x8 blocks, no CTA barrier */
};
/* Split-K has no kernel id: it needs scratch, which only its own entry points below receive. */

/*
 * One strided-batched GEMM:  C_b <- alpha * op_a(A_b) * op_b(B_b) + beta * C_b,  b in [0,batch).
 * All matrices are column-major; element (i,j) of item b is at  base[b*stride + j*ld + i].
 * m,n,k are the op-effective dims: op_a(A) is m x k, op_b(B) is k x n, C is m x n.
 * Stored shapes: A is (op_a==N ? m x k : k x m), B is (op_b==N ? k x n : n x k).
 *
 * Semantics follow BLAS, as the reference's host path does (BatchLAS
 * src/backends/netlib_lapack.cc:141-168): m==0||n==0 is a no-op; k==0 scales C by beta;
 * beta==0 never reads C (C may hold NaN/garbage); padding rows (>= m within ldc) and the
 * gap between ldc*n and stride_c are never written.
 */
typedef struct blb200_gemm_desc {
  const void* a;
  const void* b;
  void* c;
  int32_t m, n, k, batch;
  int64_t lda, ldb, ldc;                /* elements */
  int64_t stride_a, stride_b, stride_c; /* elements between consecutive batch items */
  double alpha[2], beta[2];             /* re, im; im ignored for real dtypes; rounded to T */
  int32_t dtype, op_a, op_b;            /* blb200_dtype, blb200_op, blb200_op */
  int32_t kernel_hint;                  /* BLB200_K_* ; 0 = auto */
} blb200_gemm_desc;

/* Validate the descriptor (shape rules of BatchLAS src/backends/gemm_variant.hh:19-44 in their
 * strided form: non-negative dims, ld >= stored rows).  Touches no device. */
int blb200_gemm_validate(const blb200_gemm_desc* desc);

/* Launch on `cuda_stream` (a cudaStream_t; NULL = the legacy default stream) of the current
 * device, with a/b/c DEVICE pointers.  Asynchronous; allocates nothing.  Replaces
 * gemm_vendor_impl's cublasGemmStridedBatchedEx (BatchLAS src/backends/cublas.cc:126-147). */
int blb200_gemm_strided_batched(const blb200_gemm_desc* desc, void* cuda_stream);

/* Heterogeneous batch: item b computes an m_items[b] x n_items[b] x k_items[b] product inside the
 * capacity (desc->m, n, k) that ld/stride were laid out for; one launch for the whole batch.
 * The arrays are DEVICE-readable int32[batch] (device or managed memory); a NULL array means every
 * item uses the capacity; values above the capacity are clamped to it.  Per item the BLAS rules
 * hold: m or n == 0 -> untouched, k == 0 -> C scaled by beta.  This is gemm on views with per-item
 * active dimensions (BatchLAS include/blas/matrix.hh:62-63,117-124; gemm_heterogeneous,
 * include/blas/functions/gemm.hh:48-78), which the reference's CUDA route runs as one launch per
 * item (src/backends/cublas.cc:59-104).  The caller checks that the per-item shapes of A, B and C
 * agree (the reference does so on the host, src/backends/gemm_variant.hh:29-41). */
int blb200_gemm_heterogeneous(const blb200_gemm_desc* desc, const int32_t* m_items, const int32_t* n_items,
                              const int32_t* k_items, void* cuda_stream);

/* ---- split-K ---------------------------------------------------------------------------------
 * For problems with fewer output tiles than SMs and a long k (small m x n, small batch): k is cut
 * into `splits` chunks computed side by side into scratch partials, then summed with alpha/beta.
 * Counterpart of the reference's experimental split-K + reduce (BatchLAS
 * src/sycl/gemm/split_k.hh:52-162), for every dtype / op pair / shape.
 *
 * blb200_gemm_splitk_plan: returns the number of splits that would be used (`splits` = 0 lets the
 * library choose; 1 = splitting does not help) and writes the scratch bytes needed.
 * blb200_gemm_splitk: runs with caller-provided DEVICE scratch (16-byte aligned, at least the
 * planned bytes; typically a lease from the queue's workspace arena).  Allocates nothing; falls
 * back to the ordinary launch when the plan says 1. */
int32_t blb200_gemm_splitk_plan(const blb200_gemm_desc* desc, int32_t splits, size_t* workspace_bytes);
int blb200_gemm_splitk(const blb200_gemm_desc* desc, int32_t splits, void* workspace, size_t workspace_bytes,
                       void* cuda_stream);

/* Split-K for callers that are not allowed to allocate device memory.  (No counterpart in the
 * reference: it always takes its split-K partials from a freshly allocated Matrix.)
 *
 * Who needs it: a host program that has handed the whole of HBM to its own pool, a plug-in whose
 * embedding runtime owns the allocator, or a latency-critical loop in which a call into the CUDA
 * allocator (which may synchronise the device or fail late) is forbidden.  Such callers cannot
 * produce the scratch that blb200_gemm_splitk asks for, and cannot let the library call
 * cudaMalloc for them either.
 *
 * This variant therefore keeps the partials in one fixed array inside the library image,
 * blb200_gemm_splitk_static_capacity() bytes (8 MiB) on every GPU that loads the library, held
 * until the process exits.  It calls no cudaMalloc, cudaFree or other allocating routine.  A/B/C
 * are passed exactly as for blb200_gemm_splitk.
 *   - A plan that needs more scratch than the capacity is refused with BLB200_E_TOO_LARGE
 *     ("problem exceeds the fixed capacity of this entry point"); ask blb200_gemm_splitk_plan for
 *     the bytes beforehand, or pass a smaller `splits`.
 *   - The first call on each device looks up the array's device address (with that device
 *     current).  Make that first call during start-up, before any stream capture begins.
 *   - All calls share the one array, and it keeps whatever the previous call left in it.  The
 *     kernels overwrite every partial element they later read, so no clearing is needed; but two
 *     calls that can overlap on the GPU (different streams, different host threads) race on the
 *     array.  Keep calls to this entry point ordered on one stream per device.
 *   - When the plan says that splitting does not help (fewer than 2 splits), the call runs the
 *     ordinary launch, which needs no scratch at all.
 *   - The looked-up address is remembered per device ordinal for the life of the process; it does
 *     not survive a cudaDeviceReset (do not reset a device between calls to this entry point). */
size_t blb200_gemm_splitk_static_capacity(void);
int blb200_gemm_splitk_static(const blb200_gemm_desc* desc, int32_t splits, void* cuda_stream);

/* Same operation with a/b/c HOST pointers (pinned for full speed; pageable works, slower).
 * The batch is cut into chunks; chunk i+1's host->device copies and chunk i-1's device->host
 * copy overlap chunk i's kernel on three streams of `device`.  The streams and a memory pool of
 * the library's own (cudaMemPoolCreate; the application's default pool is not touched) are made
 * on the first call for a device and kept; device staging is taken from that pool and returned to
 * it before the call returns, so later calls reuse it.  One call at a time per device (calls for
 * the same device serialise; different devices run side by side).
 * Synchronous: C is complete in host memory on return.  This is the path that stands in for
 * the reference's host-visible (USM shared) Matrix storage (BatchLAS src/matrix.cc:150-166),
 * where operands live on the host side and move to the GPU on use.
 * `chunk_items` = batch items per chunk, 0 = choose automatically. */
int blb200_gemm_strided_batched_host(const blb200_gemm_desc* desc, int device, int32_t chunk_items);

/* One call over several GPUs of the box: batch items are independent, so GPU g of G takes the
 * contiguous item range [floor(g*B/G), floor((g+1)*B/G)) (blb200_shard_range), runs the pipeline
 * above on its slice of the caller's host A, B, C from a host thread of its own, and writes its
 * disjoint slice of C.  No data crosses between GPUs; the only gather is each GPU's device->host
 * copy into the caller's C.  `devices` lists n_devices distinct CUDA device ordinals.  Synchronous;
 * returns the first non-zero status of any shard.  This is the multi-GPU form of the call for
 * which the reference would open one Queue per GPU (BatchLAS include/util/sycl-device-queue.hh:75)
 * and split the batch by hand. */
int blb200_gemm_strided_batched_host_multi(const blb200_gemm_desc* desc, const int32_t* devices, int32_t n_devices,
                                           int32_t chunk_items);
/* The shard rule, usable without a GPU: first item and item count of shard `shard` of `shards`. */
void blb200_shard_range(int64_t batch, int32_t shard, int32_t shards, int64_t* first, int64_t* count);
/* Returns the staging memory cached for `device` by the host entry points to the driver. */
int blb200_host_staging_trim(int device);

/* Name of the kernel the calling thread's most recent launch used ("" before any). */
const char* blb200_last_kernel_name(void);
/* Number of kernels this library has launched from the calling thread so far. */
uint64_t blb200_launch_count(void);
/* Text for a status code (library codes and cudaError_t values). */
const char* blb200_status_string(int status);
/* Library version, "major.minor". */
const char* blb200_version(void);
/* With BATCHLAS_KERNEL_TRACE=1 in the environment every launch is bracketed by CUDA events and a
 * Chrome trace (BATCHLAS_KERNEL_TRACE_PATH, default batchlas_b200_trace.json) is written at process
 * exit; this writes it now (waits for the recorded launches) and clears the record.  Tracing
 * mirrors BatchLAS src/util/kernel-trace.hh:46-215.  No-op when tracing is off. */
int blb200_trace_flush(void);
/* Synchronises the current device and reports whether any kernel of this library ever gave up
 * on one of its bounded waits: *out = 0 when none did, else a small code naming the wait
 * (1xx: 32^3 / 64^3 float rings, 2xx: gemv ring, 3xx: small-matrix ring, 4xx: TMA-fed DMMA tiles,
 * BLB200_WAIT_SELFTEST: the
 * self-test below).  Failure detection in the sense of BatchLAS's queue error handling
 * (src/util/queue-impl.cc wait_and_throw): the host learns of a lost copy instead of hanging. */
int blb200_device_status(int* out);
/* Synchronises the current device and clears the status words, so that a later
 * blb200_device_status reports only what happened after this call. */
int blb200_device_status_reset(void);
/* Self-test of the failure path: launches one warp that waits, with the library's own bounded
 * wait and a limit of `max_polls` polls (1 .. 65536, i.e. at most a few milliseconds), on a barrier
 * that nothing ever completes.  The wait gives up, the kernel returns normally, and
 * blb200_device_status then reports BLB200_WAIT_SELFTEST.  Nothing faults and no copy is in flight;
 * the device stays usable.  Asynchronous. */
enum { BLB200_WAIT_SELFTEST = 901 };
int blb200_selftest_wait_expiry(uint32_t max_polls, void* cuda_stream);

/* Diagnostic: measured FMA issue rate of the current device in TFLOP/s (2 flops per FMA) for
 * dtype BLB200_S (FFMA) or BLB200_D (DFMA) — the pipe peak that compute-bound shapes are judged
 * against, next to the nominal SMs x lanes x 2 x clock figure.  dtype BLB200_Z selects the FP64
 * tensor-core (mma.sync m8n8k4) rate instead.  Synchronous. */
int blb200_measure_pipe_peak(int32_t dtype, double* tflops);

/* ---- per-queue workspace arena -------------------------------------------------------
 * Bump/LIFO arena with the lease semantics of BatchLAS's WorkspaceArena (src/queue.hh:41-226,
 * include/util/workspace.hh:70-162), re-backed by cudaMallocAsync on the queue's stream:
 * blocks grow geometrically (max(request, 2*last, 64 KiB)), an innermost release rewinds the
 * cursor, an out-of-order release is only marked and reclaimed once it becomes innermost,
 * trim refuses while anything is leased.  One arena belongs to one stream and, like the
 * reference's Queue, is not thread-safe. */
typedef struct blb200_arena blb200_arena;
typedef struct blb200_lease {
  void* ptr;
  size_t bytes;
  size_t block, offset;
  uint64_t seq; /* 0 = empty lease */
} blb200_lease;

/* `device` < 0 builds a host-memory arena (malloc-backed) with identical bookkeeping: it exists
 * so the lease logic can be exercised where no GPU is present. */
int blb200_arena_create(int device, void* cuda_stream, blb200_arena** out);
int blb200_arena_destroy(blb200_arena* arena);
int blb200_arena_acquire(blb200_arena* arena, size_t bytes, blb200_lease* out);
int blb200_arena_release(blb200_arena* arena, const blb200_lease* lease);
/* 1 = memory returned to the pool, 0 = refused because a lease is outstanding, <0 error. */
int blb200_arena_trim(blb200_arena* arena);
size_t blb200_arena_capacity(const blb200_arena* arena);
size_t blb200_arena_block_count(const blb200_arena* arena);
size_t blb200_arena_alignment(const blb200_arena* arena);

/* ---- level-3 operations that BatchLAS builds on gemm -----------------------------------
 * The reference's CUDA backend turns symm/hemm and trmm into "expand the stored triangle to a
 * full matrix, then gemm" and syrk/herk into "gemm into scratch, then accumulate one triangle"
 * (src/backends/cublas.cc:181-352 symm/hemm, :441-606 accumulate_hermitian + herk, :697-796 syrk,
 * :905-997 trmm; src/backends/triangular_expand.hh).  These entry points do the same on the
 * B200 gemm kernels.  `workspace` is device memory of at least
 * blb200_level3_workspace_bytes(dtype, order, batch) bytes, 16-byte aligned — in BatchLAS a lease
 * from the queue's arena; order = the side length of the square operand (m for side left,
 * n for side right; n for syrk/herk).  Nothing is allocated.
 * side: 0 = Left, 1 = Right; uplo: 0 = Upper, 1 = Lower (the reference's Side / Uplo). */
size_t blb200_level3_workspace_bytes(int32_t dtype, int32_t order, int32_t batch);

/* symm (hermitian 0) / hemm (hermitian 1, complex only): C <- alpha*A*B + beta*C (Left) or
 * alpha*B*A + beta*C (Right); only the `uplo` triangle of A is read, for hemm the imaginary part
 * of its diagonal is taken as zero.  desc: a = A, b = B (m x n), c = C (m x n); k, op_a, op_b are
 * ignored.  Replaces symm_vendor / hemm_vendor, cublas.cc:181-352. */
int blb200_symm(const blb200_gemm_desc* desc, int32_t side, int32_t uplo, int32_t hermitian, void* workspace,
                size_t workspace_bytes, void* cuda_stream);

/* trmm, out of place as the reference's: C <- alpha*op_a(tri(A))*B (Left) or alpha*B*op_a(tri(A))
 * (Right); unit_diag != 0 takes the diagonal as ones.  beta, k, op_b are ignored.
 * Replaces trmm_vendor_impl, cublas.cc:905-997. */
int blb200_trmm(const blb200_gemm_desc* desc, int32_t side, int32_t uplo, int32_t unit_diag, void* workspace,
                size_t workspace_bytes, void* cuda_stream);

/* syrk (hermitian 0: op_a N -> A*A^T, T -> A^T*A) / herk (hermitian 1: op_a N -> A*A^H,
 * H -> A^H*A; only the real parts of alpha and beta are used and the diagonal comes out real):
 * the `uplo` triangle of C (n x n) <- alpha*product + beta*C; the other triangle is not touched.
 * desc: a = A (n x k for op N, else k x n), c = C; b, m, op_b are ignored.
 * Replaces herk_vendor (cublas.cc:504-606) and syrk_vendor (cublas.cc:697-796). */
int blb200_syrk(const blb200_gemm_desc* desc, int32_t uplo, int32_t hermitian, void* workspace, size_t workspace_bytes,
                void* cuda_stream);

/* syr2k (hermitian 0: op_a N or T) / her2k (hermitian 1: op_a N or H, complex only, only the real
 * part of beta is used, the diagonal comes out real): the `uplo` triangle of C (n x n) <-
 * alpha*op(A)*op(B)^T + alpha*op(B)*op(A)^T + beta*C, resp. alpha*op(A)*op(B)^H +
 * conj(alpha)*op(B)*op(A)^H + beta*C.  desc: a = A, b = B (same shape: n x k for op N, else k x n),
 * c = C; m, op_b are ignored.  Replaces her2k_vendor's gemm route (cublas.cc:609-666) and
 * syr2k_vendor (cublas.cc:799-902). */
int blb200_syr2k(const blb200_gemm_desc* desc, int32_t uplo, int32_t hermitian, void* workspace, size_t workspace_bytes,
                 void* cuda_stream);

/* ---- the steps either side of gemm: gemv and elementwise helpers ---------------------------
 * Strided-batched gemv:  y_b <- alpha * op_a(A_b) * x_b + beta * y_b.  A_b is the stored m x n
 * column-major matrix; op N reads x of length n and writes y of length m, op T / H the other way
 * round (H conjugates A; for real dtypes H = T).  Vector element i of item b is at
 * base[b*stride + i*inc], inc >= 1 (BatchLAS VectorView, include/blas/matrix.hh:1320-1380).
 * BLAS rules: an empty y is a no-op, an empty x scales y by beta, beta == 0 never reads y.
 * Replaces gemv_vendor (cublasXgemv / cublasXgemvStridedBatched), src/backends/cublas.cc:1092-1113;
 * public call include/blas/functions/gemv.hh:22-43. */
typedef struct blb200_gemv_desc {
  const void* a;
  const void* x;
  void* y;
  int32_t m, n, batch;       /* stored shape of A, number of items */
  int64_t lda, stride_a;     /* elements */
  int64_t incx, stride_x;
  int64_t incy, stride_y;
  double alpha[2], beta[2];
  int32_t dtype, op_a;       /* blb200_dtype, blb200_op */
} blb200_gemv_desc;
int blb200_gemv_strided_batched(const blb200_gemv_desc* desc, void* cuda_stream);

/* Elementwise helpers on batched column-major views of one shape (rows x cols x batch), each with
 * its own ld / stride; C may alias A or B (every element is read and written by one thread).
 * blb200_elementwise: C <- A (op) B, op 0 add, 1 subtract, 2 multiply (Hadamard), 3 divide.
 * blb200_axpby:       C <- alpha*A + beta*B (both products are always formed, as the reference does).
 * Scaling in place is axpby with B = C = A and beta = 0.
 * Replaces linalg::elementwise_into / axpby_into / scale, BatchLAS src/extra/elementwise.cc:42-112
 * (declared include/blas/linalg-ops.hh:59-83). */
typedef struct blb200_ewise_desc {
  const void* a;
  const void* b;
  void* c;
  int32_t rows, cols, batch;
  int64_t lda, ldb, ldc;
  int64_t stride_a, stride_b, stride_c;
  int32_t dtype;
} blb200_ewise_desc;
int blb200_elementwise(const blb200_ewise_desc* desc, int32_t op, void* cuda_stream);
int blb200_axpby(const blb200_ewise_desc* desc, const double alpha[2], const double beta[2], void* cuda_stream);

/* ---- synthetic inputs ------------------------------------------------------------------
 * Counter-based generator: element `i` of tensor `tensor_id` under `seed` depends only on
 * (seed, tensor_id, first_index + i), so any shard on any GPU count reproduces the same data.
 * dist 0: uniform[-1,1]; dist 1: normal(0,1)*scale.  Complex dtypes fill re and im
 * independently (count = number of complex elements).  Device pointer, asynchronous. */
int blb200_fill(void* dst, int32_t dtype, uint64_t count, uint64_t first_index, uint64_t seed,
                uint32_t tensor_id, int32_t dist, double scale, void* cuda_stream);

#ifdef __cplusplus
}
#endif
#endif /* BLB200_API_H_INCLUDED */
