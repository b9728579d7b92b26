// Generic batched GEMM: every dtype, every op pair, any ld / stride / base alignment, any
// (m, n, k) including k == 0.  One CTA computes one BM x BN tile of one batch item from
// shared-memory tiles filled by predicated scalar loads.  It is the total fallback of the
// dispatcher and the in-GPU cross-check for the specialised kernels.
//
// Behaviour it pins (same rules as BatchLAS src/backends/netlib_lapack.cc:141-168 and BLAS):
// beta == 0 never reads C; rows >= m inside ldc and the gap between ldc*n and stride_c are never
// written; k == 0 scales C by beta.
#include "common.cuh"

namespace blb200 {
namespace {

// 16 x 16 threads; each owns a TM x TN block of C whose rows/cols are strided by 16 so that a
// half-warp touches 16 consecutive rows of one column (coalesced C traffic, conflict-free A reads).
// `het` carries optional per-item dims (device-readable int arrays of length batch, or null): the
// heterogeneous batch of BatchLAS (MatrixView active_rows_/active_cols_, include/blas/matrix.hh:62-63;
// the reference's CUDA route launches once per item, src/backends/cublas.cc:59-104).  p.m/p.n/p.k
// are then the capacities the tile grid is laid over; tiles outside an item's dims do nothing.
template <typename T, int TM, int TN, int BK>
__global__ void __launch_bounds__(256) gemm_generic_kernel(GemmParams p, HeteroDims het, long long tiles_m,
                                                           long long tiles_n) {
  constexpr int BM = 16 * TM, BN = 16 * TN;
  __shared__ T As[BK][BM + 1];
  __shared__ T Bs[BK][BN + 1];

  const int tid = threadIdx.x;
  const int tx = tid & 15, ty = tid >> 4;
  const long long tiles_per_item = tiles_m * tiles_n;
  const long long total = tiles_per_item * p.batch;
  const T alpha = Scalar<T>::make(p.alpha[0], p.alpha[1]);
  const T beta = Scalar<T>::make(p.beta[0], p.beta[1]);
  const bool beta_zero = Scalar<T>::is_zero(beta);
  const bool conj_a = Scalar<T>::is_complex && p.op_a == BLB200_H;
  const bool conj_b = Scalar<T>::is_complex && p.op_b == BLB200_H;

  const int k_full = p.k;
  for (long long tile = blockIdx.x; tile < total; tile += gridDim.x) {
    p.k = k_full;
    const long long vitem = tile / tiles_per_item;
    const long long rem = tile - vitem * tiles_per_item;
    const SplitView sv = resolve_split(p, vitem);
    const long long item = sv.item;
    if (p.splits > 1) p.k = sv.k;
    const int m0 = (int)(rem % tiles_m) * BM;
    const int n0 = (int)(rem / tiles_m) * BN;
    p.m = item_dim(het.m, item, het.m ? het.cap_m : p.m);  // clamped to [0, capacity], as in the tile kernels
    p.n = item_dim(het.n, item, het.n ? het.cap_n : p.n);
    p.k = item_dim(het.k, item, het.k ? het.cap_k : p.k);
    if (m0 >= p.m || n0 >= p.n) continue;  // uniform across the CTA
    const T* A = (const T*)p.a + item * p.sa + sv.a_off;
    const T* B = (const T*)p.b + item * p.sb + sv.b_off;
    T* C = (T*)p.c + vitem * p.sc;

    T acc[TM][TN];
#pragma unroll
    for (int i = 0; i < TM; ++i)
#pragma unroll
      for (int j = 0; j < TN; ++j) acc[i][j] = Scalar<T>::zero();

    for (int k0 = 0; k0 < p.k; k0 += BK) {
      // op(A) tile -> As[kk][mm]
      if (p.op_a == BLB200_N) {
        for (int idx = tid; idx < BM * BK; idx += 256) {
          const int mm = idx % BM, kk = idx / BM;
          const int gm = m0 + mm, gk = k0 + kk;
          As[kk][mm] = (gm < p.m && gk < p.k) ? A[(long long)gk * p.lda + gm] : Scalar<T>::zero();
        }
      } else {
        for (int idx = tid; idx < BM * BK; idx += 256) {
          const int kk = idx % BK, mm = idx / BK;
          const int gm = m0 + mm, gk = k0 + kk;
          T v = (gm < p.m && gk < p.k) ? A[(long long)gm * p.lda + gk] : Scalar<T>::zero();
          As[kk][mm] = conj_a ? Scalar<T>::conj(v) : v;
        }
      }
      // op(B) tile -> Bs[kk][nn]
      if (p.op_b == BLB200_N) {
        for (int idx = tid; idx < BN * BK; idx += 256) {
          const int kk = idx % BK, nn = idx / BK;
          const int gn = n0 + nn, gk = k0 + kk;
          Bs[kk][nn] = (gn < p.n && gk < p.k) ? B[(long long)gn * p.ldb + gk] : Scalar<T>::zero();
        }
      } else {
        for (int idx = tid; idx < BN * BK; idx += 256) {
          const int nn = idx % BN, kk = idx / BN;
          const int gn = n0 + nn, gk = k0 + kk;
          T v = (gn < p.n && gk < p.k) ? B[(long long)gk * p.ldb + gn] : Scalar<T>::zero();
          Bs[kk][nn] = conj_b ? Scalar<T>::conj(v) : v;
        }
      }
      __syncthreads();
#pragma unroll
      for (int kk = 0; kk < BK; ++kk) {
        T af[TM], bf[TN];
#pragma unroll
        for (int i = 0; i < TM; ++i) af[i] = As[kk][tx + 16 * i];
#pragma unroll
        for (int j = 0; j < TN; ++j) bf[j] = Bs[kk][ty + 16 * j];
#pragma unroll
        for (int i = 0; i < TM; ++i)
#pragma unroll
          for (int j = 0; j < TN; ++j) Scalar<T>::fma(acc[i][j], af[i], bf[j]);
      }
      __syncthreads();
    }

#pragma unroll
    for (int j = 0; j < TN; ++j) {
      const int gn = n0 + ty + 16 * j;
      if (gn >= p.n) continue;
#pragma unroll
      for (int i = 0; i < TM; ++i) {
        const int gm = m0 + tx + 16 * i;
        if (gm >= p.m) continue;
        T* dst = C + (long long)gn * p.ldc + gm;
        *dst = epilogue<T>(alpha, acc[i][j], beta, beta_zero, dst);
      }
    }
  }
}

template <typename T, int TM, int TN, int BK>
int launch_one(const GemmParams& p, const HeteroDims& het, cudaStream_t stream) {
  constexpr int BM = 16 * TM, BN = 16 * TN;
  const long long tiles_m = (p.m + BM - 1) / BM, tiles_n = (p.n + BN - 1) / BN;
  const long long total = tiles_m * tiles_n * (long long)p.batch;
  if (total == 0) return BLB200_OK;
  const long long cap = (long long)device_info().sm_count * 64;  // grid-stride beyond this
  const unsigned grid = (unsigned)(total < cap ? total : cap);
  gemm_generic_kernel<T, TM, TN, BK><<<grid, 256, 0, stream>>>(p, het, tiles_m, tiles_n);
  return (int)cudaGetLastError();
}

template <typename T>
int launch_typed(const GemmParams& p, const HeteroDims& het, cudaStream_t stream) {
  // Small outputs take 16x16 tiles (one element per thread) so that CTAs are not mostly idle;
  // larger ones take 4x4 (real) or 2x2 (complex) register blocks.
  const bool tiny = p.m <= 16 || p.n <= 16;
  if (tiny) return launch_one<T, 1, 1, 16>(p, het, stream);
  if (sizeof(T) <= 8 && !Scalar<T>::is_complex && p.m > 32 && p.n > 32)
    return launch_one<T, 4, 4, 16>(p, het, stream);
  return launch_one<T, 2, 2, 16>(p, het, stream);
}

}  // namespace

int launch_generic_hetero(const GemmParams& p, const HeteroDims& het, int dtype, cudaStream_t stream) {
  int rc;
  switch (dtype) {
    case BLB200_S: rc = launch_typed<float>(p, het, stream); break;
    case BLB200_D: rc = launch_typed<double>(p, het, stream); break;
    case BLB200_C: rc = launch_typed<float2>(p, het, stream); break;
    case BLB200_Z: rc = launch_typed<double2>(p, het, stream); break;
    default: return BLB200_E_DTYPE;
  }
  if (rc == BLB200_OK) note_launch((het.m || het.n || het.k) ? "generic_hetero" : "generic");
  return rc;
}

int launch_generic(const GemmParams& p, int dtype, cudaStream_t stream) {
  HeteroDims none{};
  return launch_generic_hetero(p, none, dtype, stream);
}

}  // namespace blb200
