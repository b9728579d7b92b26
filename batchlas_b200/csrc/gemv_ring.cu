// gemv for large batches of small packed matrices, fed by the same loader as the small-matrix gemm
// kernels: whole matrices stream into a shared-memory ring by untiled TMA bulk copies that complete
// on one "full" mbarrier per slot; a slot belongs to one warp for the whole launch, which forms
// y = A x or y = A^T x out of it and then itself issues the copies of the item that uses the slot
// next (no producer warp, no "empty" barriers: see gemm_small.cu).  HBM sees nothing but long sequential
// reads of A, so the kernel runs at copy speed where the load/compute loop of the general kernel is
// latency-bound (a 32 x 32 float matrix is only 4 KiB).
//
// x and (when beta != 0) the old y travel through the ring with their matrix: requesting them from
// the consumer warps, even one item ahead, left their latency exposed and cost a third of the
// bandwidth.  The consumers therefore touch global memory only to store y.
//
// Preconditions (checked by gemv_ring_supported): packed columns (lda == m), unit increments, m and n
// at most 128, item size at most 16 KiB; A, x and y items each a multiple of 16 bytes long and
// starting on 16-byte boundaries (what a bulk copy needs).
//
// Ring discipline: the slot count is a multiple of the warp count and slot s always belongs to
// warp s % CW, so a warp never waits on a round of a slot before finishing the previous one.
// Every wait is bounded; on expiry the waiter records a code in the device status word and returns.
#include "common.cuh"
#include "ptx.cuh"

namespace blb200 {
namespace {

enum WaitCode { kRingWaitFull = 201 };
constexpr int kMaxItemBytes = 16384;
constexpr int kMaxDim = 128;

template <typename T>
__device__ __forceinline__ T conj_if(T v, bool conj) {
  if constexpr (Scalar<T>::is_complex) {
    if (conj) v.y = -v.y;
  }
  return v;
}

template <typename T>
__device__ __forceinline__ T add2(T a, T b) {
  if constexpr (Scalar<T>::is_complex) return T{a.x + b.x, a.y + b.y};
  else return a + b;
}

// What one lane needs to issue the copies of an item into a slot.  Kept out of line: inlined into
// the item loop it pushed the transposed variants past their register budget (720 bytes of spills).
template <typename T>
struct RingCopy {
  const T* A;
  const T* X;
  const T* Y;
  long long sa, sx, sy;
  unsigned char* smem;
  uint64_t* full_bar;
  int slot_bytes;
  uint32_t a_bytes, x_bytes, y_bytes;
  bool beta_zero;
};
template <typename T, bool XY_RING>
__device__ __noinline__ void ring_issue(RingCopy<T> c, int slot, int jj) {
  unsigned char* st = c.smem + (size_t)slot * c.slot_bytes;
  const long long item = (long long)blockIdx.x + (long long)jj * gridDim.x;
  if (XY_RING) {
    mbar_arrive_expect_tx(&c.full_bar[slot], c.a_bytes + c.x_bytes + (c.beta_zero ? 0u : c.y_bytes));
    bulk_g2s(st, c.A + item * c.sa, c.a_bytes, &c.full_bar[slot]);
    bulk_g2s(st + c.a_bytes, c.X + item * c.sx, c.x_bytes, &c.full_bar[slot]);
    if (!c.beta_zero) bulk_g2s(st + c.a_bytes + c.x_bytes, c.Y + item * c.sy, c.y_bytes, &c.full_bar[slot]);
  } else {
    mbar_arrive_expect_tx(&c.full_bar[slot], c.a_bytes);
    bulk_g2s(st, c.A + item * c.sa, c.a_bytes, &c.full_bar[slot]);
  }
}

// CW warps; blockDim = 32 * CW; dynamic smem: stages * slot_bytes, then the barriers,
// then (XY_RING = false) CW * kMaxDim elements of per-warp scratch for x.
// XY_RING = true:  a slot holds [A item | x item | old y item (only when beta != 0)].
// XY_RING = false: a slot holds the A item; each consumer warp fetches x and the old y itself, one
//                  item ahead.  For matrices of a few KiB the two extra 128-byte bulk copies per item
//                  cost more than they save (32 x 32 float: 0.55 of the copy bandwidth against 0.85).
template <typename T, int CW, bool TRANS, bool XY_RING>
__global__ void __launch_bounds__(32 * CW, 1)
    gemv_ring_kernel(const T* __restrict__ A, const T* __restrict__ X, T* __restrict__ Y, int m, int n, long long sa,
                     long long sx, long long sy, int batch, T alpha, T beta, bool beta_zero, bool conj, int stages,
                     int slot_bytes) {
  extern __shared__ __align__(128) unsigned char smem[];
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + (size_t)stages * slot_bytes);
  const int xlen = TRANS ? m : n, ylen = TRANS ? n : m;
  const uint32_t a_bytes = (uint32_t)(m * n * (int)sizeof(T)), x_bytes = (uint32_t)(xlen * (int)sizeof(T)),
                 y_bytes = (uint32_t)(ylen * (int)sizeof(T));

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    for (int s = 0; s < stages; ++s) mbar_init(&full_bar[s], 1);
    mbar_fence_init();
  }
  __syncthreads();

  // Items of this CTA: blockIdx.x, blockIdx.x + gridDim.x, ...; the j-th one uses slot j % stages.
  const int my_items = (batch > (int)blockIdx.x) ? (batch - 1 - (int)blockIdx.x) / (int)gridDim.x + 1 : 0;

  const RingCopy<T> copy{A, X, Y, sa, sx, sy, smem, full_bar, slot_bytes, a_bytes, x_bytes, y_bytes, beta_zero};
  auto issue = [&](int slot, int jj) { ring_issue<T, XY_RING>(copy, slot, jj); };

  const int cw = warp;
  constexpr int RV = kMaxDim / 32;
  T* x_scratch = reinterpret_cast<T*>(full_bar + stages) + (size_t)cw * kMaxDim;  // XY_RING = false only
  if (lane == 0)
    for (int slot = cw; slot < stages && slot < my_items; slot += CW) issue(slot, slot);

  // XY_RING = false: x and the old y of the next item are requested while this one is worked on
  T xr[RV], prior[RV];
  auto fetch_xy = [&](int j) {
    const long long item = (long long)blockIdx.x + (long long)j * gridDim.x;
    const T* xg = X + item * sx;
    const T* yg = Y + item * sy;
#pragma unroll
    for (int r = 0; r < RV; ++r) {
      const int i = lane + 32 * r;
      xr[r] = i < xlen ? xg[i] : Scalar<T>::zero();
      prior[r] = (!beta_zero && i < ylen) ? yg[i] : Scalar<T>::zero();
    }
  };
  if (!XY_RING && cw < my_items) fetch_xy(cw);

  int s = cw;
  uint32_t round = 0;
  for (int j = cw; j < my_items; j += CW) {
    const long long item = (long long)blockIdx.x + (long long)j * gridDim.x;
    T* yg = Y + item * sy;
    T prior_now[RV];
    const T* xs;
    if (!XY_RING) {
      __syncwarp();  // the previous item's readers of the scratch are done
#pragma unroll
      for (int r = 0; r < RV; ++r)
        if (lane + 32 * r < xlen) x_scratch[lane + 32 * r] = xr[r];
      __syncwarp();
#pragma unroll
      for (int r = 0; r < RV; ++r) prior_now[r] = prior[r];
      if (j + CW < my_items) fetch_xy(j + CW);
      xs = x_scratch;
    }
    if (!mbar_wait(&full_bar[s], round & 1u, kRingWaitFull)) return;
    const T* As = reinterpret_cast<const T*>(smem + (size_t)s * slot_bytes);
    if (XY_RING) {
      xs = reinterpret_cast<const T*>(smem + (size_t)s * slot_bytes + a_bytes);
      const T* ys = reinterpret_cast<const T*>(smem + (size_t)s * slot_bytes + a_bytes + x_bytes);
#pragma unroll
      for (int r = 0; r < RV; ++r)
        prior_now[r] = (!beta_zero && lane + 32 * r < ylen) ? ys[lane + 32 * r] : Scalar<T>::zero();
    }

    // Eight independent shared-memory reads of A per lane are issued before the multiply-adds that
    // use them, and each output has two accumulation chains: a CTA has few warps, so the latency has
    // to be covered inside each one.  Lanes past the end of y work on a clamped index and are dropped
    // at the store, which keeps the inner loops free of predicates.
    T acc[RV];
#pragma unroll
    for (int r = 0; r < RV; ++r) acc[r] = Scalar<T>::zero();
    if (!TRANS) {
      // lane owns rows lane + 32 r; a column is read by consecutive lanes at consecutive addresses,
      // x[j] is a broadcast read
      const int rv = (m + 31) >> 5;
#pragma unroll
      for (int r = 0; r < RV; ++r) {
        if (r < rv) {  // warp-uniform
          const T* colp = As + min(lane + 32 * r, m - 1);
          T a0 = Scalar<T>::zero(), a1 = Scalar<T>::zero();
          int jc = 0;
          for (; jc + 8 <= n; jc += 8) {
            T av[8], xv[8];
#pragma unroll
            for (int u = 0; u < 8; ++u) {
              av[u] = colp[(size_t)(jc + u) * m];
              xv[u] = xs[jc + u];
            }
#pragma unroll
            for (int u = 0; u < 8; u += 2) {
              Scalar<T>::fma(a0, av[u], xv[u]);
              Scalar<T>::fma(a1, av[u + 1], xv[u + 1]);
            }
          }
          for (; jc < n; ++jc) Scalar<T>::fma(a0, colp[(size_t)jc * m], xs[jc]);
          acc[r] = add2(a0, a1);
        }
      }
    } else {
      // lane owns columns lane + 32 c and walks their rows starting at its own offset, so that the 32
      // lanes of a request sit in 32 different banks although the columns are m elements apart
      const int cv = (n + 31) >> 5;
      const int i0 = lane % m;
#pragma unroll
      for (int c = 0; c < RV; ++c) {
        if (c < cv) {  // warp-uniform
          const T* colp = As + (size_t)min(lane + 32 * c, n - 1) * m;
          T a0 = Scalar<T>::zero(), a1 = Scalar<T>::zero();
          int t = 0;
          for (; t + 8 <= m; t += 8) {
            T av[8], xv[8];
#pragma unroll
            for (int u = 0; u < 8; ++u) {
              int i = i0 + t + u;
              i -= i >= m ? m : 0;
              av[u] = conj_if(colp[i], conj);
              xv[u] = xs[i];
            }
#pragma unroll
            for (int u = 0; u < 8; u += 2) {
              Scalar<T>::fma(a0, av[u], xv[u]);
              Scalar<T>::fma(a1, av[u + 1], xv[u + 1]);
            }
          }
          for (; t < m; ++t) {
            int i = i0 + t;
            i -= i >= m ? m : 0;
            Scalar<T>::fma(a0, conj_if(colp[i], conj), xs[i]);
          }
          acc[c] = add2(a0, a1);
        }
      }
    }
#pragma unroll
    for (int r = 0; r < RV; ++r) {
      const int i = lane + 32 * r;
      if (i < ylen) yg[i] = epilogue<T>(alpha, acc[r], beta, beta_zero, &prior_now[r]);
    }
    // every lane is past its reads of the slot; the refill goes out right behind the (asynchronous)
    // stores, where nothing of the item is live in registers any more
    __syncwarp();
    if (lane == 0 && j + stages < my_items) {
      fence_async_smem();
      issue(s, j + stages);
    }
    s += CW;
    if (s >= stages) {
      s -= stages;
      ++round;
    }
  }
}

inline bool aligned16(const void* ptr) { return (reinterpret_cast<uintptr_t>(ptr) & 15u) == 0; }

template <typename T, int CW, bool TRANS, bool XY_RING>
int launch_cw(const void* a, const void* x, void* y, int m, int n, int batch, long long sa, long long sx, long long sy,
              const double* alpha, const double* beta, bool conj, int stages, int slot_bytes, cudaStream_t stream) {
  const DeviceInfo& dev = device_info();
  const size_t smem = (size_t)stages * slot_bytes + (size_t)stages * sizeof(uint64_t) +
                      (XY_RING ? 0 : (size_t)CW * kMaxDim * sizeof(T));
  auto kern = gemv_ring_kernel<T, CW, TRANS, XY_RING>;
  static thread_local int configured_for = -1;
  int cur = 0;
  cudaGetDevice(&cur);
  if (configured_for != cur) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)dev.smem_optin);
    if (e != cudaSuccess) return (int)e;
    configured_for = cur;
  }
  const int grid = batch < dev.sm_count ? batch : dev.sm_count;
  kern<<<grid, 32 * CW, smem, stream>>>((const T*)a, (const T*)x, (T*)y, m, n, sa, sx, sy, batch,
                                            Scalar<T>::make(alpha[0], alpha[1]), Scalar<T>::make(beta[0], beta[1]),
                                            beta[0] == 0.0 && beta[1] == 0.0, conj, stages, slot_bytes);
  return (int)cudaGetLastError();
}

// Matrices of 8 KiB and more take x and y through the ring (the CTA then has few consumer warps and
// cannot hide a global load); smaller ones let the consumers fetch them.
constexpr int kXyRingFromBytes = 8192;

template <typename T>
int launch_typed(const void* a, const void* x, void* y, int m, int n, int batch, long long sa, long long sx, long long sy,
                 const double* alpha, const double* beta, bool trans, bool conj, cudaStream_t stream) {
  const bool beta_zero = beta[0] == 0.0 && beta[1] == 0.0;
  const int a_bytes = m * n * (int)sizeof(T);
  const bool xy_ring = a_bytes >= kXyRingFromBytes;
  const int slot_bytes = a_bytes + (xy_ring ? ((trans ? m : n) + (beta_zero ? 0 : (trans ? n : m))) * (int)sizeof(T) : 0);
  // barriers and, without XY_RING, 16 warps' worth of x scratch come out of the same budget
  const size_t reserve = 4096 + (xy_ring ? 0 : (size_t)16 * kMaxDim * sizeof(T));
  const size_t budget = device_info().smem_optin > reserve + 8192 ? device_info().smem_optin - reserve : 0;
  const int fit = (int)(budget / (size_t)slot_bytes);
  // Consumers first (a CTA is alone on its SM and each warp has to cover its own latencies), then
  // slots: 16 warps with two slots each when that fits, else one slot per warp.
  int cw, stages;
  if (fit >= 32) { cw = 16; stages = 32; }
  else if (fit >= 16) { cw = 16; stages = 16; }
  else if (fit >= 8) { cw = 8; stages = 8; }
  else return BLB200_E_UNSUPPORTED;
#define BLB_ARGS a, x, y, m, n, batch, sa, sx, sy, alpha, beta, conj, stages, slot_bytes, stream
#define BLB_GO(CW_)                                                                                         \
  if (xy_ring) return trans ? launch_cw<T, CW_, true, true>(BLB_ARGS) : launch_cw<T, CW_, false, true>(BLB_ARGS); \
  return trans ? launch_cw<T, CW_, true, false>(BLB_ARGS) : launch_cw<T, CW_, false, false>(BLB_ARGS)
  if (cw == 16) { BLB_GO(16); }
  BLB_GO(8);
#undef BLB_GO
#undef BLB_ARGS
}

}  // namespace

int gemv_ring_device_status(int* out) { return read_device_status_word(out); }
int gemv_ring_device_status_clear() { return clear_device_status_word(); }

bool gemv_ring_supported(int dtype, const void* a, const void* x, const void* y, int m, int n, int batch, long long lda,
                         long long sa, long long incx, long long sx, long long incy, long long sy, bool trans,
                         bool beta_zero) {
  const long long es = dtype == BLB200_S ? 4 : (dtype == BLB200_Z ? 16 : 8);
  if (m < 1 || n < 1 || m > kMaxDim || n > kMaxDim || lda != m || incx != 1 || incy != 1) return false;
  const long long a_bytes = (long long)m * n * es, x_bytes = (trans ? m : n) * es, y_bytes = (trans ? n : m) * es;
  if (a_bytes % 16 || a_bytes > kMaxItemBytes || a_bytes < 256) return false;
  if (!aligned16(a) || (sa * es) % 16) return false;
  if (a_bytes >= kXyRingFromBytes) {  // x and y go through the ring as bulk copies of their own
    if (x_bytes % 16 || !aligned16(x) || (sx * es) % 16) return false;
    if (!beta_zero && (y_bytes % 16 || !aligned16(y) || (sy * es) % 16)) return false;
  }
  if (batch > 1 && (sa < (long long)m * n || sx < (trans ? m : n) || sy < (trans ? n : m))) return false;  // overlapping items
  return batch >= 8 * device_info().sm_count;  // a ring per SM needs a queue of items to pay off
}

int launch_gemv_ring(int dtype, const void* a, const void* x, void* y, int m, int n, int batch, long long sa, long long sx,
                     long long sy, const double* alpha, const double* beta, bool trans, bool conj, cudaStream_t stream) {
  switch (dtype) {
    case BLB200_S: return launch_typed<float>(a, x, y, m, n, batch, sa, sx, sy, alpha, beta, trans, conj, stream);
    case BLB200_D: return launch_typed<double>(a, x, y, m, n, batch, sa, sx, sy, alpha, beta, trans, conj, stream);
    case BLB200_C: return launch_typed<float2>(a, x, y, m, n, batch, sa, sx, sy, alpha, beta, trans, conj, stream);
    case BLB200_Z: return launch_typed<double2>(a, x, y, m, n, batch, sa, sx, sy, alpha, beta, trans, conj, stream);
    default: return BLB200_E_DTYPE;
  }
}

}  // namespace blb200
