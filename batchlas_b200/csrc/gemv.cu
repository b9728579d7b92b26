// Strided-batched gemv for the four dtypes: y <- alpha * op(A) * x + beta * y.
//
// The operation reads every element of A once and does one multiply-add with it, so the only bound
// that matters is HBM bandwidth: m*n*sizeof(T) bytes per item (x and y are noise).  Design:
//   * A warp always reads A along its columns (consecutive rows = consecutive addresses), 32 lanes
//     = one 128..512-byte run per request, several independent requests in flight per lane.
//   * op N  (y = A x):   a lane owns RV rows (i = lane + 32 r) of a row tile and walks the columns,
//     128 bytes of A per lane in flight at a time; x comes in 32 values per coalesced request and is
//     handed round the warp by shuffle.
//   * op T/H (y = A^T x): a warp owns a group of columns (8, or up to 32 for short columns) and
//     walks the rows in chunks of 32; each lane keeps one partial sum per column, folded across the
//     warp once at the end with a halving butterfly.  Units start at staggered rows.
//   * A unit of work is (item, row tile) or (item, column group).  When units are plentiful (large
//     batch of small matrices) every warp takes whole units, eight independent warps per CTA and a
//     grid-stride loop, so tiny matrices do not pay a CTA launch each.  When they are few (one big
//     matrix) the eight warps of a CTA split the reduction dimension of one unit and combine their
//     partial sums through shared memory, which keeps enough bytes in flight to fill HBM.
// Everything is predicated: any m, n, lda, inc, alignment.  Large batches of small packed matrices
// take the TMA-ring kernel of gemv_ring.cu instead.
#include "common.cuh"

namespace blb200 {
// The TMA-ring kernel for large batches of small packed matrices (gemv_ring.cu).
bool gemv_ring_supported(int dtype, const void* a, const void* x, const void* y, int m, int n, int batch, long long lda,
                         long long sa, long long incx, long long sx, long long incy, long long sy, bool trans,
                         bool beta_zero);
int launch_gemv_ring(int dtype, const void* a, const void* x, void* y, int m, int n, int batch, long long sa, long long sx,
                     long long sy, const double* alpha, const double* beta, bool trans, bool conj, cudaStream_t stream);

namespace {

constexpr int kWarps = 8, kThreads = kWarps * 32;

struct GemvParams {
  const void* a;
  const void* x;
  void* y;
  int m, n, batch;
  long long lda, sa, incx, sx, incy, sy;
  double alpha[2], beta[2];
  int conj_a;
  int ksplit;           // warps cooperating on one unit: 1 or kWarps
  long long tiles;      // units per item
  long long units;      // tiles * batch
};

template <typename T>
__device__ __forceinline__ T ld_conj(const T* p, bool conj) {
  T v = *p;
  if constexpr (Scalar<T>::is_complex) {
    if (conj) v.y = -v.y;
  }
  return v;
}

template <typename T>
__device__ __forceinline__ T add(T a, T b) {
  if constexpr (Scalar<T>::is_complex) return T{a.x + b.x, a.y + b.y};
  else return a + b;
}

template <typename T>
__device__ __forceinline__ T shfl_xor(T v, int d) {
  if constexpr (Scalar<T>::is_complex) return T{__shfl_xor_sync(0xffffffffu, v.x, d), __shfl_xor_sync(0xffffffffu, v.y, d)};
  else return __shfl_xor_sync(0xffffffffu, v, d);
}

template <typename T>
__device__ __forceinline__ T shfl_idx(T v, int src) {
  if constexpr (Scalar<T>::is_complex) return T{__shfl_sync(0xffffffffu, v.x, src), __shfl_sync(0xffffffffu, v.y, src)};
  else return __shfl_sync(0xffffffffu, v, src);
}

template <typename T>
__device__ __forceinline__ void store_y(T* y, T alpha, T sum, T beta, bool beta_zero) {
  *y = epilogue<T>(alpha, sum, beta, beta_zero, y);
}

// ---- op N ------------------------------------------------------------------------------------------
template <typename T, int RV>
__global__ void __launch_bounds__(kThreads) gemv_n_kernel(GemvParams p) {
  // columns per unrolled step: RV * CS independent loads per lane = 128 bytes of registers
  constexpr int CS = 128 / (RV * (int)sizeof(T));
  __shared__ T part[kWarps][32 * RV];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int per_cta = kWarps / p.ksplit;  // units a CTA works on at a time
  const int slot = warp / p.ksplit, kpart = warp % p.ksplit;
  const long long groups = (p.units + per_cta - 1) / per_cta;
  const T alpha = Scalar<T>::make(p.alpha[0], p.alpha[1]), beta = Scalar<T>::make(p.beta[0], p.beta[1]);
  const bool beta_zero = p.beta[0] == 0.0 && p.beta[1] == 0.0;

  for (long long grp = blockIdx.x; grp < groups; grp += gridDim.x) {
    const long long unit = grp * per_cta + slot;
    const bool live = unit < p.units;
    T acc[RV], prior[RV];
#pragma unroll
    for (int r = 0; r < RV; ++r) acc[r] = prior[r] = Scalar<T>::zero();
    long long item = 0;
    int row0 = 0;
    if (live) {
      item = unit / p.tiles;
      row0 = (int)(unit - item * p.tiles) * (32 * RV);
      const T* A = (const T*)p.a + item * p.sa;
      const T* x = (const T*)p.x + item * p.sx;
      // this warp's share of the columns: [j_begin, j_end)
      const int chunk = (p.n + p.ksplit - 1) / p.ksplit;
      const int j_begin = kpart * chunk, j_end = min(p.n, j_begin + chunk);
      bool in[RV];
#pragma unroll
      for (int r = 0; r < RV; ++r) in[r] = row0 + lane + 32 * r < p.m;
      if (p.ksplit == 1 && !beta_zero) {  // ask for y now, so that its latency hides behind the walk over A
#pragma unroll
        for (int r = 0; r < RV; ++r)
          if (in[r]) prior[r] = ((const T*)p.y)[item * p.sy + (long long)(row0 + lane + 32 * r) * p.incy];
      }
      // Columns in blocks of 32: lane l fetches x[jb + l] once (one coalesced request) and the block's
      // values are handed round by shuffle, CS columns of A in flight at a time.
      for (int jb = j_begin; jb < j_end; jb += 32) {
        const T xl = jb + lane < j_end ? x[(long long)(jb + lane) * p.incx] : Scalar<T>::zero();
        const T* col = A + (long long)jb * p.lda + row0 + lane;
        const int nb = min(32, j_end - jb);
#pragma unroll
        for (int c0 = 0; c0 < 32; c0 += CS) {
          if (c0 < nb) {  // warp-uniform
            T av[CS][RV];
#pragma unroll
            for (int c = 0; c < CS; ++c)
#pragma unroll
              for (int r = 0; r < RV; ++r)
                av[c][r] = (in[r] && c0 + c < nb) ? col[(long long)(c0 + c) * p.lda + 32 * r] : Scalar<T>::zero();
#pragma unroll
            for (int c = 0; c < CS; ++c) {
              const T xv = shfl_idx(xl, c0 + c);
#pragma unroll
              for (int r = 0; r < RV; ++r) Scalar<T>::fma(acc[r], av[c][r], xv);
            }
          }
        }
      }
    }
    if (p.ksplit > 1) {  // the CTA works on one unit: fold the eight column shares
#pragma unroll
      for (int r = 0; r < RV; ++r) part[warp][lane + 32 * r] = acc[r];
      __syncthreads();
      if (live) {
        for (int e = threadIdx.x; e < 32 * RV; e += kThreads) {
          T s = part[0][e];
#pragma unroll
          for (int w = 1; w < kWarps; ++w) s = add(s, part[w][e]);
          const int row = row0 + e;
          if (row < p.m) store_y<T>((T*)p.y + item * p.sy + (long long)row * p.incy, alpha, s, beta, beta_zero);
        }
      }
      __syncthreads();
    } else if (live) {
#pragma unroll
      for (int r = 0; r < RV; ++r) {
        const int row = row0 + lane + 32 * r;
        if (row < p.m) ((T*)p.y)[item * p.sy + (long long)row * p.incy] = epilogue<T>(alpha, acc[r], beta, beta_zero, &prior[r]);
      }
    }
  }
}

// ---- op T / H --------------------------------------------------------------------------------------
// Folds N per-lane partial sums (one per column) across the 32 lanes with N-1 + (5 - log2 N) shuffles
// instead of 5 N: while more than one column is left, a lane keeps one half of the columns and hands
// the other half to its partner.  Afterwards v[0] of lane L is the total of column (L >> (5 - log2 N)).
template <typename T, int N>
__device__ __forceinline__ void fold_columns(T (&v)[N], int lane) {
#pragma unroll
  for (int step = 0; step < 5; ++step) {
    const int off = 16 >> step;
    const int h = N >> (step + 1);  // columns kept per lane after this step
    if (h >= 1) {
      const bool upper = (lane & off) != 0;
#pragma unroll
      for (int k = 0; k < h; ++k) {
        const T send = upper ? v[k] : v[k + h];
        const T keep = upper ? v[k + h] : v[k];
        v[k] = add(keep, shfl_xor(send, off));
      }
    } else {
      v[0] = add(v[0], shfl_xor(v[0], off));
    }
  }
}

// CT columns per unit, RC row chunks of 32 per unrolled step (CT * RC loads in flight per lane).
template <typename T, int CT, int RC>
__global__ void __launch_bounds__(kThreads) gemv_t_kernel(GemvParams p) {
  constexpr int LOG_CT = CT == 32 ? 5 : (CT == 16 ? 4 : (CT == 8 ? 3 : (CT == 4 ? 2 : 1)));
  __shared__ T part[kWarps][CT];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int per_cta = kWarps / p.ksplit;
  const int slot = warp / p.ksplit, kpart = warp % p.ksplit;
  const long long groups = (p.units + per_cta - 1) / per_cta;
  const T alpha = Scalar<T>::make(p.alpha[0], p.alpha[1]), beta = Scalar<T>::make(p.beta[0], p.beta[1]);
  const bool beta_zero = p.beta[0] == 0.0 && p.beta[1] == 0.0;
  const bool conj = p.conj_a != 0;
  const int my_col = lane >> (5 - LOG_CT);                       // column this lane ends up holding
  const bool writer = (lane & ((1 << (5 - LOG_CT)) - 1)) == 0;

  for (long long grp = blockIdx.x; grp < groups; grp += gridDim.x) {
    const long long unit = grp * per_cta + slot;
    const bool live = unit < p.units;
    T acc[CT];
#pragma unroll
    for (int c = 0; c < CT; ++c) acc[c] = Scalar<T>::zero();
    T prior = Scalar<T>::zero();
    long long item = 0;
    int col0 = 0;
    if (live) {
      item = unit / p.tiles;
      col0 = (int)(unit - item * p.tiles) * CT;
      if (p.ksplit == 1 && !beta_zero && writer && col0 + my_col < p.n)  // asked for now, needed after the walk
        prior = ((const T*)p.y)[item * p.sy + (long long)(col0 + my_col) * p.incy];
      const T* A = (const T*)p.a + item * p.sa + (long long)col0 * p.lda;
      const T* x = (const T*)p.x + item * p.sx;
      const int ncol = min(CT, p.n - col0);
      // this warp's share of the rows, in whole chunks of 32
      const int chunks = (p.m + 31) / 32, share = (chunks + p.ksplit - 1) / p.ksplit;
      const int i_begin = kpart * share * 32, i_end = min(p.m, i_begin + share * 32);
      if (ncol == CT) {
        // Units start at different rows and wrap round, so that warps walking columns whose starts
        // are a power of two apart do not all ask the same memory channels at the same time.
        const int steps = (i_end - i_begin + 32 * RC - 1) / (32 * RC);
        const int first = steps > 1 ? (int)((((unsigned long long)unit * 2654435761ull) >> 12) % (unsigned)steps) : 0;
        for (int sidx = 0; sidx < steps; ++sidx) {
          int st = first + sidx;
          if (st >= steps) st -= steps;
          const int i0 = i_begin + st * (32 * RC) + lane;
          T av[RC][CT], xv[RC];
#pragma unroll
          for (int r = 0; r < RC; ++r) {
            const int i = i0 + 32 * r;
            const bool in = i < i_end;
            xv[r] = in ? x[(long long)i * p.incx] : Scalar<T>::zero();
#pragma unroll
            for (int c = 0; c < CT; ++c) av[r][c] = in ? ld_conj(A + (long long)c * p.lda + i, conj) : Scalar<T>::zero();
          }
#pragma unroll
          for (int r = 0; r < RC; ++r)
#pragma unroll
            for (int c = 0; c < CT; ++c) Scalar<T>::fma(acc[c], av[r][c], xv[r]);
        }
      } else {
        for (int i = i_begin + lane; i < i_end; i += 32) {
          const T xv = x[(long long)i * p.incx];
#pragma unroll
          for (int c = 0; c < CT; ++c)
            if (c < ncol) Scalar<T>::fma(acc[c], ld_conj(A + (long long)c * p.lda + i, conj), xv);
        }
      }
    }
    fold_columns<T, CT>(acc, lane);  // lane L now holds the sum of column L >> (5 - log2 CT) in acc[0]
    if (p.ksplit > 1) {
      if (writer) part[warp][my_col] = acc[0];
      __syncthreads();
      if (live && threadIdx.x < CT && col0 + (int)threadIdx.x < p.n) {
        T s = part[0][threadIdx.x];
#pragma unroll
        for (int w = 1; w < kWarps; ++w) s = add(s, part[w][threadIdx.x]);
        store_y<T>((T*)p.y + item * p.sy + (long long)(col0 + threadIdx.x) * p.incy, alpha, s, beta, beta_zero);
      }
      __syncthreads();
    } else if (live && writer && col0 + my_col < p.n) {
      ((T*)p.y)[item * p.sy + (long long)(col0 + my_col) * p.incy] = epilogue<T>(alpha, acc[0], beta, beta_zero, &prior);
    }
  }
}

// y <- beta * y for an empty reduction (the BLAS rule for a zero-length x).
template <typename T>
__global__ void __launch_bounds__(256) scale_y_kernel(T* y, long long len, int batch, long long inc, long long stride,
                                                      T beta, bool beta_zero) {
  const long long total = len * batch, step = (long long)gridDim.x * blockDim.x;
  for (long long f = (long long)blockIdx.x * blockDim.x + threadIdx.x; f < total; f += step) {
    const long long b = f / len, i = f - b * len;
    T* dst = y + b * stride + i * inc;
    *dst = beta_zero ? Scalar<T>::zero() : Scalar<T>::mul(beta, *dst);
  }
}

// CTAs of `kern` that fit on the whole device at once: the size of a persistent grid.
template <typename Kern>
long long resident_ctas(Kern kern) {
  int per_sm = 0;
  if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kern, kThreads, 0) != cudaSuccess || per_sm < 1) per_sm = 1;
  return (long long)per_sm * device_info().sm_count;
}

template <typename T>
int launch_typed(GemvParams p, bool trans, cudaStream_t stream) {
  const int out_len = trans ? p.n : p.m, red_len = trans ? p.m : p.n;
  const long long cap = (long long)device_info().sm_count * 8;
  if (red_len == 0) {
    const long long total = (long long)out_len * p.batch;
    const long long want = (total + 255) / 256;
    const T beta = Scalar<T>::make(p.beta[0], p.beta[1]);
    scale_y_kernel<T><<<(unsigned)(want < cap ? want : cap), 256, 0, stream>>>(
        (T*)p.y, out_len, p.batch, p.incy, p.sy, beta, p.beta[0] == 0.0 && p.beta[1] == 0.0);
    return (int)cudaGetLastError();
  }
  const long long enough = (long long)device_info().sm_count * 32;  // warps that can fill the memory system
  auto plan = [&](long long tiles) {  // fills tiles / units / ksplit, returns the CTA-level group count
    p.tiles = tiles;
    p.units = tiles * p.batch;
    // Few units: let the eight warps of a CTA share each one.  Tiny reductions are not worth splitting.
    p.ksplit = (p.units < enough && red_len >= 8 * 32) ? kWarps : 1;
    return (p.units + (kWarps / p.ksplit) - 1) / (kWarps / p.ksplit);
  };
  auto go = [&](auto kern, long long groups) {
    const long long fit = resident_ctas(kern);
    kern<<<(unsigned)(groups < fit ? groups : fit), kThreads, 0, stream>>>(p);
  };
  if (trans) {
    // Short columns: as many columns per warp as 128 bytes of registers hold, one row chunk per step.
    // Long columns: 8 (4 for 16-byte elements) columns, several row chunks per step.
    constexpr int WIDE = 128 / (int)sizeof(T) > 32 ? 32 : 128 / (int)sizeof(T);   // 32, 16, 16, 8
    constexpr int NARROW = sizeof(T) >= 16 ? 4 : 8;
    constexpr int RC = 128 / (NARROW * (int)sizeof(T)) > 4 ? 4 : 128 / (NARROW * (int)sizeof(T));  // 4, 2, 2, 2
    const bool wide = p.m <= 64 && p.n >= WIDE && (long long)((p.n + WIDE - 1) / WIDE) * p.batch * kWarps >= enough;
    if (wide) go(gemv_t_kernel<T, WIDE, 1>, plan((p.n + WIDE - 1) / WIDE));
    else go(gemv_t_kernel<T, NARROW, RC>, plan((p.n + NARROW - 1) / NARROW));
  } else {
    // rows per lane: as many as the matrix offers, fewer when that leaves too few units in flight
    int rv = p.m > 64 ? 4 : (p.m > 32 ? 2 : 1);
    while (rv > 1 && ((p.m + 32 * rv - 1) / (32 * rv)) * (long long)p.batch * kWarps < enough) rv >>= 1;
    const long long groups = plan((p.m + 32 * rv - 1) / (32 * rv));
    if (rv == 4) go(gemv_n_kernel<T, 4>, groups);
    else if (rv == 2) go(gemv_n_kernel<T, 2>, groups);
    else go(gemv_n_kernel<T, 1>, groups);
  }
  return (int)cudaGetLastError();
}

}  // namespace
}  // namespace blb200

extern "C" int blb200_gemv_strided_batched(const blb200_gemv_desc* d, void* cuda_stream) {
  using namespace blb200;
  if (!d) return BLB200_E_NULL;
  if (d->dtype < BLB200_S || d->dtype > BLB200_Z || d->op_a < BLB200_N || d->op_a > BLB200_H) return BLB200_E_DTYPE;
  if (d->m < 0 || d->n < 0 || d->batch < 0) return BLB200_E_SHAPE;
  if (d->lda < (d->m > 1 ? d->m : 1) || d->incx < 1 || d->incy < 1) return BLB200_E_SHAPE;
  if (d->stride_a < 0 || d->stride_x < 0 || d->stride_y < 0) return BLB200_E_SHAPE;
  const bool trans = d->op_a != BLB200_N;
  const int out_len = trans ? d->n : d->m, red_len = trans ? d->m : d->n;
  if (out_len == 0 || d->batch == 0) return BLB200_OK;
  if (!d->y || (red_len > 0 && (!d->a || !d->x))) return BLB200_E_NULL;
  GemvParams p{};
  p.a = d->a; p.x = d->x; p.y = d->y;
  p.m = d->m; p.n = d->n; p.batch = d->batch;
  p.lda = d->lda; p.sa = d->stride_a;
  p.incx = d->incx; p.sx = d->stride_x; p.incy = d->incy; p.sy = d->stride_y;
  const bool cplx = d->dtype >= BLB200_C;
  p.alpha[0] = d->alpha[0]; p.alpha[1] = cplx ? d->alpha[1] : 0.0;
  p.beta[0] = d->beta[0]; p.beta[1] = cplx ? d->beta[1] : 0.0;
  p.conj_a = cplx && d->op_a == BLB200_H;
  cudaStream_t stream = (cudaStream_t)cuda_stream;
  int rc;
  if (red_len > 0 && gemv_ring_supported(d->dtype, d->a, d->x, d->y, d->m, d->n, d->batch, d->lda, d->stride_a, d->incx,
                                         d->stride_x, d->incy, d->stride_y, trans, p.beta[0] == 0.0 && p.beta[1] == 0.0)) {
    rc = launch_gemv_ring(d->dtype, d->a, d->x, d->y, d->m, d->n, d->batch, d->stride_a, d->stride_x, d->stride_y, p.alpha,
                          p.beta, trans, p.conj_a != 0, stream);
    if (rc == BLB200_OK) note_launch("gemv_ring");
    if (rc != BLB200_E_UNSUPPORTED) return rc;
  }
  switch (d->dtype) {
    case BLB200_S: rc = launch_typed<float>(p, trans, stream); break;
    case BLB200_D: rc = launch_typed<double>(p, trans, stream); break;
    case BLB200_C: rc = launch_typed<float2>(p, trans, stream); break;
    default: rc = launch_typed<double2>(p, trans, stream); break;
  }
  if (rc == BLB200_OK) note_launch("gemv");
  return rc;
}
