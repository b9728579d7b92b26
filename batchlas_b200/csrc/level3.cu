// The level-3 operations that BatchLAS's CUDA backend builds on top of gemm, behind the same C ABI:
//   symm / hemm   C <- alpha*A*B + beta*C (or B*A), A symmetric / Hermitian, one triangle stored:
//                 A is expanded to a full matrix in scratch, then one gemm
//                 (BatchLAS src/backends/cublas.cc:181-352, expand_mirrored in triangular_expand.hh).
//   trmm          C <- alpha*op(tri(A))*B (or B*op(tri(A))), out of place: the triangle is expanded
//                 with zeros (and a unit diagonal on request), then one gemm with beta = 0
//                 (cublas.cc:905-997, expand_triangular).
//   syrk / herk   C_tri <- alpha*op(A)*op(A)^T|H + beta*C_tri: one gemm into scratch, then the
//                 requested triangle is accumulated into C; for herk alpha/beta are real and the
//                 diagonal comes out exactly real (cublas.cc:441-606, accumulate_hermitian).
// The scratch (k x k or n x n per item, ld rounded to 16 bytes as the reference's expanded_ld does,
// triangular_expand.hh:33-36) is passed in by the caller — in BatchLAS terms a lease from the
// queue's workspace arena.  Nothing here allocates.
#include "common.cuh"

namespace blb200 {
namespace {

size_t elem_bytes(int dtype) { return dtype == BLB200_S ? 4 : (dtype == BLB200_Z ? 16 : 8); }
long long expanded_ld(int dtype, int n) {
  const long long vec = (long long)(16 / elem_bytes(dtype));
  return ((long long)(n > 0 ? n : 1) + vec - 1) / vec * vec;
}

enum ExpandMode { kMirror = 0, kMirrorConj = 1, kTriangular = 2 };

// dst (k x k, ld ldd) <- full form of the `lower`/upper triangle of src.
template <typename T>
__global__ void __launch_bounds__(256) expand_kernel(const T* __restrict__ src, T* __restrict__ dst, int k, int batch,
                                                     long long lds, long long ss, long long ldd, long long sd, int lower,
                                                     int mode, int unit_diag) {
  const long long per = (long long)k * k, total = per * batch;
  const long long step = (long long)gridDim.x * blockDim.x;
  for (long long flat = (long long)blockIdx.x * blockDim.x + threadIdx.x; flat < total; flat += step) {
    const long long b = flat / per, rem = flat - b * per;
    const int j = (int)(rem / k), i = (int)(rem - (long long)j * k);
    const bool stored = lower ? (i >= j) : (i <= j);
    const T* s = src + b * ss;
    T v;
    if (i == j) {
      v = s[(long long)j * lds + i];
      if (mode == kTriangular && unit_diag) v = Scalar<T>::make(1.0, 0.0);
      if constexpr (Scalar<T>::is_complex) {
        if (mode == kMirrorConj) v.y = 0;  // a Hermitian diagonal is real whatever the storage holds
      }
    } else if (stored) {
      v = s[(long long)j * lds + i];
    } else if (mode == kTriangular) {
      v = Scalar<T>::zero();
    } else {
      v = s[(long long)i * lds + j];
      if (mode == kMirrorConj) v = Scalar<T>::conj(v);
    }
    dst[b * sd + (long long)j * ldd + i] = v;
  }
}

// C_tri <- product_tri + beta * C_tri   (alpha is already in the product); hermitian: beta real,
// diagonal forced real.
template <typename T>
__global__ void __launch_bounds__(256) accumulate_triangle_kernel(const T* __restrict__ prod, T* __restrict__ C, int n,
                                                                  int batch, long long ldp, long long sp, long long ldc,
                                                                  long long sc, int lower, T beta, bool beta_zero,
                                                                  int hermitian) {
  const long long per = (long long)n * n, total = per * batch;
  const long long step = (long long)gridDim.x * blockDim.x;
  for (long long flat = (long long)blockIdx.x * blockDim.x + threadIdx.x; flat < total; flat += step) {
    const long long b = flat / per, rem = flat - b * per;
    const int j = (int)(rem / n), i = (int)(rem - (long long)j * n);
    if (lower ? (i < j) : (i > j)) continue;
    T v = prod[b * sp + (long long)j * ldp + i];
    T* c = C + b * sc + (long long)j * ldc + i;
    if (!beta_zero) {
      T prior = *c;
      if constexpr (Scalar<T>::is_complex) {
        if (hermitian && i == j) prior.y = 0;  // not referenced: must not leak into the real part
      }
      Scalar<T>::fma(v, beta, prior);
    }
    if constexpr (Scalar<T>::is_complex) {
      if (hermitian && i == j) v.y = 0;
    }
    *c = v;
  }
}

// ---- tiled versions for order >= 32 ------------------------------------------------------------------
// One block per (item, pair of 32 x 32 tiles).  The stored tile is read once, coalesced, into shared
// memory and written twice: as it is, and transposed (conjugated / zeroed as the mode asks) into the
// mirror tile, so the unreferenced triangle is never read and every global access runs along rows.
constexpr int kTile = 32;

__device__ __forceinline__ void decode_pair(int idx, int nt, int& p, int& q) {  // idx -> (p >= q), column by column
  q = 0;
  while (idx >= nt - q) {
    idx -= nt - q;
    ++q;
  }
  p = q + idx;
}

template <typename T>
__global__ void __launch_bounds__(256) expand_tiled_kernel(const T* __restrict__ src, T* __restrict__ dst, int k,
                                                           long long lds, long long ss, long long ldd, long long sd,
                                                           int lower, int mode, int unit_diag) {
  __shared__ T tile[kTile][kTile + 1];
  const int nt = (k + kTile - 1) / kTile, pairs = nt * (nt + 1) / 2;
  const T* s = src + (long long)blockIdx.x * ss;
  T* d = dst + (long long)blockIdx.x * sd;
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
  for (int pair = blockIdx.y; pair < pairs; pair += gridDim.y) {
    int p, q;
    decode_pair(pair, nt, p, q);
    const int r0 = (lower ? p : q) * kTile, c0 = (lower ? q : p) * kTile;  // the stored tile: rows r0.., columns c0..
    __syncthreads();
    for (int jj = ty; jj < kTile; jj += 8) {
      const int i = r0 + tx, j = c0 + jj;
      const bool stored = lower ? (i >= j) : (i <= j);
      if (i < k && j < k && stored) tile[jj][tx] = s[(long long)j * lds + i];
    }
    __syncthreads();
    // the stored tile itself
    for (int jj = ty; jj < kTile; jj += 8) {
      const int i = r0 + tx, j = c0 + jj;
      if (i >= k || j >= k) continue;
      const bool stored = lower ? (i >= j) : (i <= j);
      T v;
      if (i == j) {
        v = tile[jj][tx];
        if (mode == kTriangular && unit_diag) v = Scalar<T>::make(1.0, 0.0);
        if constexpr (Scalar<T>::is_complex) {
          if (mode == kMirrorConj) v.y = 0;
        }
      } else if (stored) {
        v = tile[jj][tx];
      } else if (mode == kTriangular) {  // only in a diagonal tile
        v = Scalar<T>::zero();
      } else {
        v = tile[tx][jj];
        if (mode == kMirrorConj) v = Scalar<T>::conj(v);
      }
      d[(long long)j * ldd + i] = v;
    }
    if (p == q) continue;
    // the mirror tile: rows c0.., columns r0..
    for (int jj = ty; jj < kTile; jj += 8) {
      const int i = c0 + tx, j = r0 + jj;
      if (i >= k || j >= k) continue;
      T v;
      if (mode == kTriangular) {
        v = Scalar<T>::zero();
      } else {
        v = tile[tx][jj];
        if (mode == kMirrorConj) v = Scalar<T>::conj(v);
      }
      d[(long long)j * ldd + i] = v;
    }
  }
}

template <typename T>
__global__ void __launch_bounds__(256) accumulate_tiled_kernel(const T* __restrict__ prod, T* __restrict__ C, int n,
                                                               long long ldp, long long sp, long long ldc, long long sc,
                                                               int lower, T beta, bool beta_zero, int hermitian) {
  const int nt = (n + kTile - 1) / kTile, pairs = nt * (nt + 1) / 2;
  const T* pr = prod + (long long)blockIdx.x * sp;
  T* c = C + (long long)blockIdx.x * sc;
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
  for (int pair = blockIdx.y; pair < pairs; pair += gridDim.y) {
    int p, q;
    decode_pair(pair, nt, p, q);
    const int r0 = (lower ? p : q) * kTile, c0 = (lower ? q : p) * kTile;
#pragma unroll 4
    for (int jj = ty; jj < kTile; jj += 8) {
      const int i = r0 + tx, j = c0 + jj;
      if (i >= n || j >= n || (lower ? (i < j) : (i > j))) continue;
      T v = pr[(long long)j * ldp + i];
      T* dst = c + (long long)j * ldc + i;
      if (!beta_zero) {
        T prior = *dst;
        if constexpr (Scalar<T>::is_complex) {
          if (hermitian && i == j) prior.y = 0;
        }
        Scalar<T>::fma(v, beta, prior);
      }
      if constexpr (Scalar<T>::is_complex) {
        if (hermitian && i == j) v.y = 0;
      }
      *dst = v;
    }
  }
}

// Two-sided accumulate of syr2k / her2k: the `lower`/upper triangle of C <- P + P^T|H + beta * C,
// P = alpha * op(A) * op(B)^T|H already in scratch (BatchLAS accumulate_hermitian<T, TwoSided>,
// src/backends/cublas.cc:441-502).  Both tiles of P that meet in an output tile go through shared
// memory, so P is read along its rows only.
template <typename T>
__global__ void __launch_bounds__(256) accumulate2_tiled_kernel(const T* __restrict__ prod, T* __restrict__ C, int n,
                                                                long long ldp, long long sp, long long ldc, long long sc,
                                                                int lower, T beta, bool beta_zero, int hermitian) {
  __shared__ T mirror[kTile][kTile + 1];
  const int nt = (n + kTile - 1) / kTile, pairs = nt * (nt + 1) / 2;
  const T* pr = prod + (long long)blockIdx.x * sp;
  T* c = C + (long long)blockIdx.x * sc;
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
  for (int pair = blockIdx.y; pair < pairs; pair += gridDim.y) {
    int p, q;
    decode_pair(pair, nt, p, q);
    const int r0 = (lower ? p : q) * kTile, c0 = (lower ? q : p) * kTile;  // output tile: rows r0.., columns c0..
    __syncthreads();
    for (int jj = ty; jj < kTile; jj += 8) {  // the tile of P across the diagonal: rows c0.., columns r0..
      const int i = c0 + tx, j = r0 + jj;
      if (i < n && j < n) mirror[jj][tx] = pr[(long long)j * ldp + i];
    }
    __syncthreads();
    for (int jj = ty; jj < kTile; jj += 8) {
      const int i = r0 + tx, j = c0 + jj;
      if (i >= n || j >= n || (lower ? (i < j) : (i > j))) continue;
      T v = pr[(long long)j * ldp + i];
      T w = mirror[tx][jj];  // P(j, i)
      if (hermitian) w = Scalar<T>::conj(w);
      if constexpr (Scalar<T>::is_complex) {
        v.x += w.x;
        v.y += w.y;
      } else {
        v += w;
      }
      T* dst = c + (long long)j * ldc + i;
      if (!beta_zero) {
        T prior = *dst;
        if constexpr (Scalar<T>::is_complex) {
          if (hermitian && i == j) prior.y = 0;
        }
        Scalar<T>::fma(v, beta, prior);
      }
      if constexpr (Scalar<T>::is_complex) {
        if (hermitian && i == j) v.y = 0;
      }
      *dst = v;
    }
  }
}

dim3 pair_grid(int order, int batch) {
  const int nt = (order + kTile - 1) / kTile;
  const long long pairs = (long long)nt * (nt + 1) / 2;
  return dim3((unsigned)batch, (unsigned)(pairs < 65535 ? pairs : 65535), 1);
}

template <typename F>
int for_dtype(int dtype, F&& f) {
  switch (dtype) {
    case BLB200_S: return f((float*)nullptr);
    case BLB200_D: return f((double*)nullptr);
    case BLB200_C: return f((float2*)nullptr);
    case BLB200_Z: return f((double2*)nullptr);
    default: return BLB200_E_DTYPE;
  }
}

unsigned grid_for(long long total) {
  const long long want = (total + 255) / 256, cap = (long long)device_info().sm_count * 16;
  return (unsigned)(want < 1 ? 1 : (want < cap ? want : cap));
}

int expand(int dtype, const void* src, void* dst, int k, int batch, long long lds, long long ss, long long ldd,
           long long sd, int lower, int mode, int unit_diag, cudaStream_t stream) {
  if (k == 0 || batch == 0) return BLB200_OK;
  return for_dtype(dtype, [&](auto* tag) {
    using T = std::remove_pointer_t<decltype(tag)>;
    if (k >= kTile)
      expand_tiled_kernel<T><<<pair_grid(k, batch), 256, 0, stream>>>((const T*)src, (T*)dst, k, lds, ss, ldd, sd, lower,
                                                                      mode, unit_diag);
    else
      expand_kernel<T><<<grid_for((long long)k * k * batch), 256, 0, stream>>>((const T*)src, (T*)dst, k, batch, lds, ss,
                                                                              ldd, sd, lower, mode, unit_diag);
    return (int)cudaGetLastError();
  });
}

int check_common(const blb200_gemm_desc* d, int side, int uplo) {
  if (!d) return BLB200_E_NULL;
  if (d->dtype < BLB200_S || d->dtype > BLB200_Z) return BLB200_E_DTYPE;
  if (side < 0 || side > 1 || uplo < 0 || uplo > 1) return BLB200_E_DTYPE;
  if (d->m < 0 || d->n < 0 || d->batch < 0) return BLB200_E_SHAPE;
  if (d->stride_a < 0 || d->stride_b < 0 || d->stride_c < 0) return BLB200_E_SHAPE;
  return BLB200_OK;
}

}  // namespace
}  // namespace blb200

extern "C" {

size_t blb200_level3_workspace_bytes(int32_t dtype, int32_t order, int32_t batch) {
  if (dtype < BLB200_S || dtype > BLB200_Z || order <= 0 || batch <= 0) return 0;
  return (size_t)blb200::expanded_ld(dtype, order) * (size_t)order * (size_t)batch * blb200::elem_bytes(dtype);
}

// symm (hermitian = 0) / hemm (hermitian = 1).  desc: a = A (k x k, k = m for side left, n for
// right; only the `uplo` triangle is read), b = B (m x n), c = C (m x n); m, n, lda/ldb/ldc,
// strides, alpha, beta, dtype are used; k, op_a, op_b are ignored.
int blb200_symm(const blb200_gemm_desc* desc, int32_t side, int32_t uplo, int32_t hermitian, void* workspace,
                size_t workspace_bytes, void* cuda_stream) {
  using namespace blb200;
  int rc = check_common(desc, side, uplo);
  if (rc != BLB200_OK) return rc;
  if (hermitian && desc->dtype < BLB200_C) return BLB200_E_DTYPE;  // BLAS has no real ?hemm
  if (desc->m == 0 || desc->n == 0 || desc->batch == 0) return BLB200_OK;
  const int k = side == 0 ? desc->m : desc->n;
  if (desc->lda < k || desc->ldb < desc->m || desc->ldc < desc->m) return BLB200_E_SHAPE;
  if (!desc->a || !desc->b || !desc->c) return BLB200_E_NULL;
  const size_t need = blb200_level3_workspace_bytes(desc->dtype, k, desc->batch);
  if (!workspace) return BLB200_E_NULL;
  if (workspace_bytes < need) return BLB200_E_TOO_LARGE;
  cudaStream_t stream = (cudaStream_t)cuda_stream;
  const long long ld = expanded_ld(desc->dtype, k);
  rc = expand(desc->dtype, desc->a, workspace, k, desc->batch, desc->lda, desc->stride_a, ld, ld * k, uplo == 1,
              hermitian ? kMirrorConj : kMirror, 0, stream);
  if (rc != BLB200_OK) return rc;
  blb200_gemm_desc g = *desc;
  g.op_a = g.op_b = BLB200_N;
  g.k = k;
  g.kernel_hint = 0;
  if (side == 0) {  // C = alpha * Afull * B + beta * C
    g.a = workspace; g.lda = ld; g.stride_a = ld * k;
  } else {          // C = alpha * B * Afull + beta * C
    g.a = desc->b; g.lda = desc->ldb; g.stride_a = desc->stride_b;
    g.b = workspace; g.ldb = ld; g.stride_b = ld * k;
  }
  return dispatch(&g, stream);
}

// trmm, out of place: C <- alpha * op(tri(A)) * B (side left) or alpha * B * op(tri(A)) (right).
// desc fields as for blb200_symm; op_a is the transpose applied to the triangle; beta is ignored.
int blb200_trmm(const blb200_gemm_desc* desc, int32_t side, int32_t uplo, int32_t unit_diag, void* workspace,
                size_t workspace_bytes, void* cuda_stream) {
  using namespace blb200;
  int rc = check_common(desc, side, uplo);
  if (rc != BLB200_OK) return rc;
  if (desc->op_a < BLB200_N || desc->op_a > BLB200_H) return BLB200_E_DTYPE;
  if (desc->m == 0 || desc->n == 0 || desc->batch == 0) return BLB200_OK;
  const int k = side == 0 ? desc->m : desc->n;
  if (desc->lda < k || desc->ldb < desc->m || desc->ldc < desc->m) return BLB200_E_SHAPE;
  if (!desc->a || !desc->b || !desc->c) return BLB200_E_NULL;
  const size_t need = blb200_level3_workspace_bytes(desc->dtype, k, desc->batch);
  if (!workspace) return BLB200_E_NULL;
  if (workspace_bytes < need) return BLB200_E_TOO_LARGE;
  cudaStream_t stream = (cudaStream_t)cuda_stream;
  const long long ld = expanded_ld(desc->dtype, k);
  rc = expand(desc->dtype, desc->a, workspace, k, desc->batch, desc->lda, desc->stride_a, ld, ld * k, uplo == 1,
              kTriangular, unit_diag != 0, stream);
  if (rc != BLB200_OK) return rc;
  blb200_gemm_desc g = *desc;
  g.k = k;
  g.beta[0] = g.beta[1] = 0.0;
  g.kernel_hint = 0;
  // The expanded operand keeps its zeros, and the tile kernels are told where they are so that each
  // output tile stops (or starts) its k loop at the diagonal: about half the work for a square B.
  const bool lower_after_op = (uplo == 1) == (desc->op_a == BLB200_N);
  StructureHints hints{0, 0, 0, 0};
  if (side == 0) {
    g.a = workspace; g.lda = ld; g.stride_a = ld * k;
    g.op_a = desc->op_a; g.op_b = BLB200_N;
    hints.tri_a = lower_after_op ? 1 : 2;
  } else {
    g.a = desc->b; g.lda = desc->ldb; g.stride_a = desc->stride_b;
    g.b = workspace; g.ldb = ld; g.stride_b = ld * k;
    g.op_a = BLB200_N; g.op_b = desc->op_a;
    hints.tri_b = lower_after_op ? 1 : 2;
  }
  return dispatch_structured(&g, &hints, stream);
}

// syrk (hermitian = 0: op_a N or T) / herk (hermitian = 1: op_a N or H, alpha/beta real).
// desc: a = A (n x k for op N, k x n otherwise), c = C (n x n, only the `uplo` triangle is read and
// written); n, k, lda, ldc, stride_a, stride_c, alpha, beta, dtype, op_a are used.
int blb200_syrk(const blb200_gemm_desc* desc, int32_t uplo, int32_t hermitian, void* workspace, size_t workspace_bytes,
                void* cuda_stream) {
  using namespace blb200;
  if (!desc) return BLB200_E_NULL;
  blb200_gemm_desc seen = *desc;  // b, m and stride_b are documented as ignored: they are not validated
  seen.m = seen.n;
  seen.stride_b = 0;
  int rc = check_common(&seen, 0, uplo);
  if (rc != BLB200_OK) return rc;
  if (hermitian && desc->dtype < BLB200_C) return BLB200_E_DTYPE;
  const int n = desc->n, k = desc->k;
  if (k < 0) return BLB200_E_SHAPE;
  int opa = desc->op_a;
  if (!hermitian && opa == BLB200_H && desc->dtype < BLB200_C) opa = BLB200_T;  // the same thing for real data
  if (hermitian ? (opa != BLB200_N && opa != BLB200_H) : (opa != BLB200_N && opa != BLB200_T)) return BLB200_E_DTYPE;
  if (n == 0 || desc->batch == 0) return BLB200_OK;
  if (desc->lda < (opa == BLB200_N ? n : (k > 1 ? k : 1)) || desc->ldc < n) return BLB200_E_SHAPE;
  if (!desc->c || (k > 0 && !desc->a)) return BLB200_E_NULL;
  cudaStream_t stream = (cudaStream_t)cuda_stream;
  blb200_gemm_desc g = *desc;
  g.m = n; g.n = n; g.k = k;
  g.b = desc->a; g.ldb = desc->lda; g.stride_b = desc->stride_a;
  g.op_a = opa;
  g.op_b = (opa == BLB200_N) ? (hermitian ? BLB200_H : BLB200_T) : BLB200_N;
  if (hermitian) g.alpha[1] = g.beta[1] = 0.0;
  g.kernel_hint = 0;
  // First choice: a tile kernel writes the wanted triangle of C itself — tiles wholly in the other
  // triangle do nothing, tiles on the diagonal mask their stores — so there is no scratch, no second
  // pass and about half the arithmetic.
  if (k > 0) {
    const StructureHints hints{0, 0, uplo == 1 ? 1 : 2, hermitian ? 1 : 0};
    rc = dispatch_structured(&g, &hints, stream);
    if (rc != BLB200_E_UNSUPPORTED) return rc;
  }
  // Otherwise (operands the tile kernels do not take): full product into scratch, then accumulate.
  const size_t need = blb200_level3_workspace_bytes(desc->dtype, n, desc->batch);
  if (!workspace) return BLB200_E_NULL;
  if (workspace_bytes < need) return BLB200_E_TOO_LARGE;
  const long long ld = expanded_ld(desc->dtype, n);
  g.c = workspace; g.ldc = ld; g.stride_c = ld * n;
  g.beta[0] = g.beta[1] = 0.0;
  rc = dispatch(&g, stream);
  if (rc != BLB200_OK) return rc;
  return for_dtype(desc->dtype, [&](auto* tag) {
    using T = std::remove_pointer_t<decltype(tag)>;
    const T beta = Scalar<T>::make(desc->beta[0], hermitian ? 0.0 : desc->beta[1]);
    const bool beta_zero = desc->beta[0] == 0.0 && (hermitian || desc->dtype < BLB200_C || desc->beta[1] == 0.0);
    if (n >= kTile)
      accumulate_tiled_kernel<T><<<pair_grid(n, desc->batch), 256, 0, stream>>>(
          (const T*)workspace, (T*)desc->c, n, ld, ld * n, desc->ldc, desc->stride_c, uplo == 1, beta, beta_zero,
          hermitian);
    else
      accumulate_triangle_kernel<T><<<grid_for((long long)n * n * desc->batch), 256, 0, stream>>>(
          (const T*)workspace, (T*)desc->c, n, desc->batch, ld, ld * n, desc->ldc, desc->stride_c, uplo == 1, beta,
          beta_zero, hermitian);
    return (int)cudaGetLastError();
  });
}

// syr2k (hermitian = 0: C_tri <- alpha*op(A)*op(B)^T + alpha*op(B)*op(A)^T + beta*C_tri, op_a N or T)
// her2k (hermitian = 1: C_tri <- alpha*op(A)*op(B)^H + conj(alpha)*op(B)*op(A)^H + beta*C_tri, op_a N or
// H, beta real, diagonal real).  One gemm P = alpha*op(A)*op(B)^T|H into scratch, then P + P^T|H is
// accumulated into the wanted triangle.  desc: a = A, b = B (same shape as A), c = C (n x n).
int blb200_syr2k(const blb200_gemm_desc* desc, int32_t uplo, int32_t hermitian, void* workspace, size_t workspace_bytes,
                 void* cuda_stream) {
  using namespace blb200;
  int rc = check_common(desc, 0, uplo);
  if (rc != BLB200_OK) return rc;
  if (hermitian && desc->dtype < BLB200_C) return BLB200_E_DTYPE;
  const int n = desc->n, k = desc->k;
  if (k < 0) return BLB200_E_SHAPE;
  int opa = desc->op_a;
  if (!hermitian && opa == BLB200_H && desc->dtype < BLB200_C) opa = BLB200_T;
  if (hermitian ? (opa != BLB200_N && opa != BLB200_H) : (opa != BLB200_N && opa != BLB200_T)) return BLB200_E_DTYPE;
  if (n == 0 || desc->batch == 0) return BLB200_OK;
  const long long min_ld = opa == BLB200_N ? n : (k > 1 ? k : 1);
  if (desc->lda < min_ld || desc->ldb < min_ld || desc->ldc < n) return BLB200_E_SHAPE;
  if (!desc->c || (k > 0 && (!desc->a || !desc->b))) return BLB200_E_NULL;
  const size_t need = blb200_level3_workspace_bytes(desc->dtype, n, desc->batch);
  if (!workspace) return BLB200_E_NULL;
  if (workspace_bytes < need) return BLB200_E_TOO_LARGE;
  cudaStream_t stream = (cudaStream_t)cuda_stream;
  const long long ld = expanded_ld(desc->dtype, n);
  blb200_gemm_desc g = *desc;
  g.m = n; g.n = n; g.k = k;
  g.op_a = opa;
  g.op_b = (opa == BLB200_N) ? (hermitian ? BLB200_H : BLB200_T) : BLB200_N;
  g.c = workspace; g.ldc = ld; g.stride_c = ld * n;
  g.beta[0] = g.beta[1] = 0.0;
  g.kernel_hint = 0;
  rc = dispatch(&g, stream);
  if (rc != BLB200_OK) return rc;
  return for_dtype(desc->dtype, [&](auto* tag) {
    using T = std::remove_pointer_t<decltype(tag)>;
    const T beta = Scalar<T>::make(desc->beta[0], hermitian ? 0.0 : desc->beta[1]);
    const bool beta_zero = desc->beta[0] == 0.0 && (hermitian || desc->dtype < BLB200_C || desc->beta[1] == 0.0);
    accumulate2_tiled_kernel<T><<<pair_grid(n, desc->batch), 256, 0, stream>>>(
        (const T*)workspace, (T*)desc->c, n, ld, ld * n, desc->ldc, desc->stride_c, uplo == 1, beta, beta_zero, hermitian);
    return (int)cudaGetLastError();
  });
}

}  // extern "C"
